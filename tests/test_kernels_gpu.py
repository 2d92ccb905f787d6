"""Each kernel alone against a plain float64 statement of the same operation,
at sizes other than the engine's (ragged, not powers of two)."""
import math

import numpy as np
import pytest
import torch

import plain_gpt2

pytestmark = pytest.mark.gpu

DT = {"float32": torch.float32, "bfloat16": torch.bfloat16}


def dev(a, dtype=torch.float32):
    return torch.as_tensor(np.asarray(a)).to("cuda", dtype)


def assert_close(got, want, dtype, what="", k=1, extra_abs=0.0):
    """float32 results: max |diff| <= 1e-5 x rms of the expected values (the
    reference's measure for kernels, src/gpu-testing.cpp:79-95); for a sum of
    k float32 terms the rounding of the running sum grows like sqrt(k), so the
    bound is scaled by sqrt(k / 512) beyond 512 terms; the tensor cores cut the
    running sum off instead of rounding it, which grows like k and overtakes the
    root beyond some 3,300 terms (k / 1280).  bfloat16
    results are rounded to 8 bits of mantissa on output, so each element may
    be off by 2^-9 of its own size; allow 2^-7 of it plus 0.6 % of the rms for
    the rounding of intermediate results."""
    want = np.asarray(want, dtype=np.float64)
    got = np.asarray(got, dtype=np.float64)
    assert got.shape == want.shape, (what, got.shape, want.shape)
    rms = max(np.sqrt((want ** 2).mean()), 1e-30)
    diff = np.abs(got - want)
    bound = (1e-5 * max(1.0, math.sqrt(k / 512.0), k / 1280.0) * rms if dtype == "float32"
             else 2.0 ** -7 * np.abs(want) + 6e-3 * rms + extra_abs)
    worst = float((diff / bound).max()) if dtype != "float32" else float(diff.max() / bound)
    assert worst <= 1.0, f"{what}: error is {worst:.2f} x the bound (rms {rms:.3g}, max |diff| {diff.max():.3g})"


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_embed(dtype):
    from math_utils_b200.csrc import ops
    rng = np.random.default_rng(0)
    table = dev(rng.standard_normal((37, 72)), DT[dtype])
    pos = dev(rng.standard_normal((19, 72)), DT[dtype])
    ids = torch.tensor([0, 36, 5, 5, 17], dtype=torch.int32, device="cuda")
    p = torch.tensor([0, 18, 3, 4, 9], dtype=torch.int32, device="cuda")
    got = ops.embed(ids, p, table, pos).cpu().numpy()
    want = table.double().cpu().numpy()[ids.cpu()] + pos.double().cpu().numpy()[p.cpu()]
    assert np.abs(got - want).max() < 1e-6
    got = ops.embed(ids, None, table, None).cpu().numpy()
    assert np.array_equal(got, table.float().cpu().numpy()[ids.cpu()])


@pytest.mark.parametrize("out_dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("hidden,eps", [(48, 1e-5), (1000, 1e-6), (1600, 1e-3), (2048, 1e-5), (2052, 1e-5), (50, 1e-5)])
def test_layernorm(hidden, eps, out_dtype):
    """Widths on both sides of what the warp-per-row kernel takes (a multiple of 4 up to 2,048)."""
    from math_utils_b200.csrc import ops
    rng = np.random.default_rng(1)
    x = (rng.standard_normal((11, hidden)) * 3 + 5).astype(np.float32)     # a mean far from zero
    g = rng.standard_normal(hidden).astype(np.float32)
    b = rng.standard_normal(hidden).astype(np.float32)
    want = plain_gpt2.layer_norm(x.astype(np.float64), g.astype(np.float64), b.astype(np.float64), eps)
    got = ops.layernorm(dev(x), dev(g), dev(b), eps, DT[out_dtype]).float().cpu().numpy()
    assert_close(got, want, out_dtype, "layernorm")
    rows = torch.tensor([10, 0, 3], dtype=torch.int32, device="cuda")
    got = ops.layernorm(dev(x), dev(g), dev(b), eps, DT[out_dtype], rows=rows).float().cpu().numpy()
    assert_close(got, want[[10, 0, 3]], out_dtype, "layernorm of picked rows")


@pytest.mark.parametrize("n_rows", [1, 5, 64, 301])
def test_layernorm_row_counts_and_no_bias(n_rows):
    """Row counts that leave the last block of four rows partly empty, the many-rows variant (more than 64),
    and a norm without a bias; twice in a row, so that a second launch finds the first one's parameters
    gone from shared memory and stages its own."""
    from math_utils_b200.csrc import ops
    rng = np.random.default_rng(n_rows)
    hidden = 200
    x = (rng.standard_normal((n_rows, hidden)) * 2 - 1).astype(np.float32)
    for trial in range(2):
        g = rng.standard_normal(hidden).astype(np.float32)
        b = rng.standard_normal(hidden).astype(np.float32)
        want = plain_gpt2.layer_norm(x.astype(np.float64), g.astype(np.float64), b.astype(np.float64), 1e-5)
        got = ops.layernorm(dev(x), dev(g), dev(b), 1e-5, torch.float32).cpu().numpy()
        assert_close(got, want, "float32", f"layernorm of {n_rows} rows")
        want = plain_gpt2.layer_norm(x.astype(np.float64), g.astype(np.float64), np.zeros(hidden), 1e-5)
        got = ops.layernorm(dev(x), dev(g), None, 1e-5, torch.bfloat16).float().cpu().numpy()
        assert_close(got, want, "bfloat16", f"layernorm of {n_rows} rows without a bias")


GEMM_SHAPES = [(1, 50, 24), (13, 77, 40), (64, 96, 320), (130, 257, 136), (5, 1031, 96), (200, 64, 8)]


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("m,n,k", GEMM_SHAPES)
@pytest.mark.parametrize("act", [None, "gelu_new", "gelu"])
def test_linear(m, n, k, act, dtype):
    """Every product kernel behind ops.linear, with bias, activation and residual."""
    from math_utils_b200.csrc import ops
    rng = np.random.default_rng(m * 1000 + n)
    a = dev(rng.standard_normal((m, k)), DT[dtype])
    w = dev(rng.standard_normal((n, k)) / math.sqrt(k), DT[dtype])
    bias = dev(rng.standard_normal(n))
    res = dev(rng.standard_normal((m, n)))
    z = a.double().cpu().numpy() @ w.double().cpu().numpy().T + bias.double().cpu().numpy()
    if act:
        z = plain_gpt2.ACTIVATIONS[act](z)
    got = ops.linear(a, w, bias, act=act).float().cpu().numpy()
    assert_close(got, z, dtype, "output in the compute dtype")
    # float32 output of bfloat16 operands: only the accumulation differs from float64
    got = ops.linear(a, w, bias, act=act, residual=res, out_dtype=torch.float32).cpu().numpy()
    assert_close(got, z + res.double().cpu().numpy(), "float32", "with residual, float32 out")
    x = res.clone()                                       # adding into the residual in place
    ops.linear(a, w, bias, act=act, residual=x, out=x)
    assert_close(x.cpu().numpy(), z + res.double().cpu().numpy(), "float32", "in place")
    got = ops.linear(a, w, None, out_dtype=torch.float32).cpu().numpy()
    assert_close(got, a.double().cpu().numpy() @ w.double().cpu().numpy().T, "float32", "no bias")


def test_linear_rows_do_not_depend_on_the_batch():
    """float32: a row's product is the same bits whatever else is in the batch."""
    from math_utils_b200.csrc import ops
    rng = np.random.default_rng(3)
    a = dev(rng.standard_normal((70, 200)))
    w = dev(rng.standard_normal((90, 200)))
    full = ops.linear(a, w)
    for rows in ([0], [69], list(range(5, 22))):
        part = ops.linear(a[rows].contiguous(), w)
        assert torch.equal(part, full[rows])


def paged_setup(rng, seq_lens, n_kv_heads, head_dim, dtype, page=64, shuffle=True):
    """Random keys/values laid into shuffled pages; returns them flat too."""
    n_pages_seq = [-(-n // page) for n in seq_lens]
    total = sum(n_pages_seq) + 3
    order = rng.permutation(total) if shuffle else np.arange(total)
    max_pages = max(n_pages_seq)
    table = np.zeros((len(seq_lens), max_pages), dtype=np.int32)
    kv = torch.zeros((total, 2, n_kv_heads, page, head_dim), dtype=DT[dtype], device="cuda")
    ks, vs, nxt = [], [], 0
    for s, n in enumerate(seq_lens):
        k = dev(rng.standard_normal((n, n_kv_heads * head_dim)), DT[dtype])
        v = dev(rng.standard_normal((n, n_kv_heads * head_dim)), DT[dtype])
        ks.append(k); vs.append(v)
        for i in range(n_pages_seq[s]):
            table[s, i] = order[nxt]; nxt += 1
    return kv, torch.as_tensor(table).cuda(), ks, vs


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("n_heads,n_kv_heads,head_dim,window", [
    (4, 4, 16, 0), (6, 2, 48, 0), (3, 3, 80, 0), (8, 2, 128, 37), (5, 1, 256, 0), (2, 2, 64, 1), (4, 2, 32, 200),
    (5, 5, 20, 0), (6, 3, 8, 50), (3, 1, 7, 0), (2, 2, 100, 0)])
def test_attention_over_pages(n_heads, n_kv_heads, head_dim, window, dtype):
    """Whole prompts appended and attended in one call, then a single-token step
    with the keys split over warps; any head count, grouping, size (head sizes that
    are no multiple of 16, or odd, included) and window.  The split leaves the keys
    past n_splits x split_keys to the last part."""
    from math_utils_b200.csrc import ops
    rng = np.random.default_rng(head_dim + n_heads)
    seq_lens = [1, 70, 129, 64]
    kv, table, ks, vs = paged_setup(rng, seq_lens, n_kv_heads, head_dim, dtype)
    tok_pos = torch.tensor([p for n in seq_lens for p in range(n)], dtype=torch.int32, device="cuda")
    tok_seq = torch.tensor([s for s, n in enumerate(seq_lens) for _ in range(n)], dtype=torch.int32, device="cuda")
    k_all, v_all = torch.cat(ks), torch.cat(vs)
    ops.kv_append(k_all, v_all, tok_pos, tok_seq, table, 64, n_kv_heads, head_dim, kv)
    q_all = dev(rng.standard_normal((sum(seq_lens), n_heads * head_dim)), DT[dtype])
    out = torch.empty_like(q_all)
    scale = 0.37 / math.sqrt(head_dim)
    ops.attention(q_all, out, kv, table, 64, tok_pos, tok_seq, n_heads, n_kv_heads, head_dim, scale, window)
    o = 0
    want_rows = []
    for s, n in enumerate(seq_lens):
        want = plain_gpt2.causal_attention(q_all[o:o + n].double().cpu().numpy(), ks[s].double().cpu().numpy(),
                                           vs[s].double().cpu().numpy(), n_heads, n_kv_heads, scale, window)
        assert_close(out[o:o + n].float().cpu().numpy(), want, dtype, f"sequence {s}")
        want_rows.append(want[-1])
        o += n
    # single-token step for the last position of each sequence, keys split 5 ways
    last = torch.tensor(np.cumsum(seq_lens) - 1, dtype=torch.int64, device="cuda")
    q1 = q_all[last].contiguous()
    pos1 = tok_pos[last].contiguous()
    seq1 = torch.arange(len(seq_lens), dtype=torch.int32, device="cuda")
    out1 = torch.empty_like(q1)
    n_splits, split_keys = 3, 32               # 96 < 129 keys: the last part takes the rest
    part_o = torch.full((len(seq_lens) * n_heads * n_splits * head_dim,), float("nan"), device="cuda")
    part_ml = torch.full((len(seq_lens) * n_heads * n_splits * 2,), float("nan"), device="cuda")
    ops.attention(q1, out1, kv, table, 64, pos1, seq1, n_heads, n_kv_heads, head_dim, scale, window,
                  n_splits, split_keys, part_o, part_ml)
    assert_close(out1.float().cpu().numpy(), np.stack(want_rows), dtype, "split keys")


def test_attention_finds_a_far_key():
    """One key among hundreds is made to dominate: the output must be its value.
    Random scores would hide a wrong page or a dropped key."""
    from math_utils_b200.csrc import ops
    rng = np.random.default_rng(9)
    n, heads, dh = 700, 2, 32
    kv, table, ks, vs = paged_setup(rng, [n], heads, dh, "float32")
    pos = torch.arange(n, dtype=torch.int32, device="cuda")
    seq = torch.zeros(n, dtype=torch.int32, device="cuda")
    for target in (0, 63, 64, 383, 640, 699):
        k = ks[0].clone()
        q = dev(rng.standard_normal((1, heads * dh)))
        k[target] = q[0] * 40.0                                # its score towers over the rest
        ops.kv_append(k, vs[0], pos, seq, table, 64, heads, dh, kv)
        out = torch.empty_like(q)
        p1 = torch.tensor([n - 1], dtype=torch.int32, device="cuda")
        s1 = torch.zeros(1, dtype=torch.int32, device="cuda")
        for n_splits in (1, 7):
            part_o = torch.zeros(heads * n_splits * dh, device="cuda")
            part_ml = torch.zeros(heads * n_splits * 2, device="cuda")
            ops.attention(q, out, kv, table, 64, p1, s1, heads, heads, dh, 1.0, 0, n_splits, 128, part_o, part_ml)
            assert torch.allclose(out[0], vs[0][target], atol=1e-4), (target, n_splits)


def test_window_edge():
    """The key just outside the window must not be seen, the one just inside must."""
    from math_utils_b200.csrc import ops
    rng = np.random.default_rng(4)
    n, dh, window = 200, 16, 70
    kv, table, ks, vs = paged_setup(rng, [n], 1, dh, "float32")
    q = dev(rng.standard_normal((1, dh)))
    pos = torch.arange(n, dtype=torch.int32, device="cuda")
    seq = torch.zeros(n, dtype=torch.int32, device="cuda")
    p1 = torch.tensor([n - 1], dtype=torch.int32, device="cuda")
    s1 = torch.zeros(1, dtype=torch.int32, device="cuda")
    first_inside = n - window                      # position 130 is the oldest key the query sees
    for target, seen in ((first_inside, True), (first_inside - 1, False)):
        k = ks[0].clone()
        k[target] = q[0] * 40.0
        ops.kv_append(k, vs[0], pos, seq, table, 64, 1, dh, kv)
        out = torch.empty_like(q)
        ops.attention(q, out, kv, table, 64, p1, s1, 1, 1, dh, 1.0, window)
        assert torch.allclose(out[0], vs[0][target], atol=1e-4) == seen


def test_argmax_first_maximum_wins():
    from math_utils_b200.csrc import ops
    rng = np.random.default_rng(5)
    x = rng.standard_normal((6, 50257)).astype(np.float32)
    x[1, 777] = x[1, 40000] = 9.0
    x[2, :] = -3.0                                  # all equal: index 0
    x[3, 50256] = 11.0
    got = ops.argmax(dev(x)).cpu().tolist()
    assert got == [plain_gpt2.argmax(r) for r in x] and got[1] == 777 and got[2] == 0 and got[3] == 50256
    # the kernels' status word handed on behind the tokens; fed tokens without fed positions
    out = torch.full((7,), -1, dtype=torch.int32, device="cuda")
    fed = torch.full((6,), -1, dtype=torch.int32, device="cuda")
    ops.argmax(dev(x), out=out[:6], feed=(fed, None, 0), status_to=out[6:])
    assert out.cpu().tolist() == got + [0] and fed.cpu().tolist() == got


@pytest.mark.parametrize("vocab,top_k,temperature", [(1031, 0, 0.8), (1031, 20, 0.7), (50257, 40, 1.0),
                                                      (513, 5, 1.5), (50257, 0, 1.0),
                                                      (140001, 0, 0.9), (140001, 300, 1.1)])   # (past the limit of
                                                      # the per-warp histograms: the block's one histogram)
def test_sample_follows_the_plain_rule(vocab, top_k, temperature):
    from math_utils_b200.csrc import ops
    rng = np.random.default_rng(vocab + top_k)
    rows = 24
    x = (rng.standard_normal((rows, vocab)) * 2.5).astype(np.float32)
    x[3, 5] = x[3, 9] = x[3].max() + 1.0           # tied leaders
    x[4, :] = 0.25                                  # everything tied
    req = torch.arange(100, 100 + rows, dtype=torch.int64, device="cuda")
    draws = torch.zeros(rows, dtype=torch.int32, device="cuda")
    logits = dev(x)
    for n in range(3):
        got = ops.sample(logits, temperature, top_k, 42, req, draws).cpu().tolist()
        for r in range(rows):
            u = plain_gpt2.uniform_draw(42, 100 + r, n)
            want, margin = plain_gpt2.sample_top_k(x[r], temperature, top_k or -1, u)    # the kernel's 0 keeps all
            # a disagreement is allowed only where u falls within rounding of a boundary
            assert got[r] == want or margin < 1e-5, (r, n, got[r], want, margin)
    assert draws.cpu().tolist() == [3] * rows
    out = torch.full((rows + 1,), -1, dtype=torch.int32, device="cuda")
    fed = torch.full((rows,), -1, dtype=torch.int32, device="cuda")
    draws.zero_()
    first = ops.sample(logits, temperature, top_k, 42, req, draws).cpu().tolist()
    draws.zero_()
    ops.sample(logits, temperature, top_k, 42, req, draws, out=out[:rows], feed=(fed, None, 0), status_to=out[rows:])
    assert out.cpu().tolist() == first + [0] and fed.cpu().tolist() == first


@pytest.mark.parametrize("top_k", [40, 0, 2000])
@pytest.mark.parametrize("rows", [3, 40, 70, 150])
def test_sample_with_blocks_sharing_a_row(rows, top_k):
    """8, 4, 2 or 1 blocks share a row's passes, by how many rows there are: the token must not depend on it
    (ties at the threshold and among the kept tokens included).  A top_k of 40 is gathered into a list, 2,000 is
    not, 0 keeps the whole vocabulary."""
    from math_utils_b200.csrc import ops
    rng = np.random.default_rng(rows)
    vocab, temperature = 50257, 0.7
    x = (rng.standard_normal((rows, vocab)) * 2.5).astype(np.float32)
    x[0, 11] = x[0, 30011] = x[0].max() + 1.0      # tied leaders in different blocks' shares
    x[1, :] = 0.25                                  # everything tied: the threshold cuts by index
    x[2, 5000:5100] = x[2].max()                    # a hundred tied at the top, forty kept
    req = torch.arange(7, 7 + rows, dtype=torch.int64, device="cuda")
    draws = torch.zeros(rows, dtype=torch.int32, device="cuda")
    logits = dev(x)
    for n in range(2):
        got = ops.sample(logits, temperature, top_k, 3, req, draws).cpu().tolist()
        for r in range(rows if rows <= 40 else 12):
            u = plain_gpt2.uniform_draw(3, 7 + r, n)
            want, margin = plain_gpt2.sample_top_k(x[r], temperature, top_k or -1, u)
            assert got[r] == want or margin < 1e-5, (r, n, got[r], want, margin)
    alone = [ops.sample(logits[r:r + 1].contiguous(), temperature, top_k, 3, req[r:r + 1],
                        torch.ones(1, dtype=torch.int32, device="cuda")).item() for r in range(min(rows, 6))]
    assert alone == got[:len(alone)]                # the same token from eight blocks a row as from fewer


def test_sample_distribution():
    """Frequencies over many requests follow softmax(l / T) of the kept tokens."""
    from math_utils_b200.csrc import ops
    l = np.array([2.0, 1.0, 0.0, -1.0, 3.0, -5.0, 0.5], dtype=np.float32)
    rows = 20000
    logits = dev(np.tile(l, (rows, 1)))
    req = torch.arange(rows, dtype=torch.int64, device="cuda")
    draws = torch.zeros(rows, dtype=torch.int32, device="cuda")
    got = ops.sample(logits, 0.9, 4, 7, req, draws).cpu().numpy()
    keep = np.argsort(-l)[:4]
    p = np.exp(l[keep] / 0.9); p /= p.sum()
    freq = np.array([(got == k).mean() for k in keep])
    assert set(np.unique(got)) <= set(keep.tolist())
    assert np.abs(freq - p).max() < 0.015


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("n_heads,n_kv_heads,head_dim,window", [
    (4, 4, 16, 0), (6, 2, 48, 0), (3, 3, 80, 0), (8, 2, 128, 70), (5, 1, 256, 0), (12, 12, 64, 0), (4, 2, 32, 1)])
def test_single_token_attention_kernel(n_heads, n_kv_heads, head_dim, window, dtype):
    """The one-launch kernel of single-token steps: the new key and value come
    from the step's projections and are appended by the kernel itself."""
    from math_utils_b200.csrc import ops
    rng = np.random.default_rng(7 * head_dim + n_heads)
    seq_lens = [1, 64, 65, 200, 129, 448]
    kv, table, ks, vs = paged_setup(rng, seq_lens, n_kv_heads, head_dim, dtype)
    # the cache holds all but the last token of every sequence
    tok_pos = torch.tensor([p for n in seq_lens for p in range(n - 1)], dtype=torch.int32, device="cuda")
    tok_seq = torch.tensor([s for s, n in enumerate(seq_lens) for _ in range(n - 1)], dtype=torch.int32, device="cuda")
    ops.kv_append(torch.cat([k[:-1] for k in ks]), torch.cat([v[:-1] for v in vs]), tok_pos, tok_seq, table, 64,
                  n_kv_heads, head_dim, kv)
    scale = 0.41 / math.sqrt(head_dim)
    q = dev(rng.standard_normal((len(seq_lens), n_heads * head_dim)), DT[dtype])
    k_new = torch.stack([k[-1] for k in ks]).contiguous()
    v_new = torch.stack([v[-1] for v in vs]).contiguous()
    pos1 = torch.tensor([n - 1 for n in seq_lens], dtype=torch.int32, device="cuda")
    seq1 = torch.arange(len(seq_lens), dtype=torch.int32, device="cuda")
    n_pages = table.shape[1]
    want = np.stack([plain_gpt2.causal_attention(
        np.repeat(q[s:s + 1].double().cpu().numpy(), n, axis=0), ks[s].double().cpu().numpy(),
        vs[s].double().cpu().numpy(), n_heads, n_kv_heads, scale, window)[-1] for s, n in enumerate(seq_lens)])
    for round_ in range(2):                   # with the append, then over the appended cache
        out = torch.full_like(q, float("nan"))
        ops.attention_decode(q, k_new if round_ == 0 else None, v_new if round_ == 0 else None, out, kv, table, 64,
                             pos1, seq1, n_heads, n_kv_heads, head_dim, scale, window, n_pages)
        assert_close(out.float().cpu().numpy(), want, dtype, f"launch {round_}")
    # the appended keys are where the general kernel looks for them
    out2 = torch.empty_like(q)
    ops.attention(q, out2, kv, table, 64, pos1, seq1, n_heads, n_kv_heads, head_dim, scale, window)
    assert_close(out2.float().cpu().numpy(), want, dtype, "after the append")


@pytest.mark.parametrize("warps", [2, 3, 6, 12, 24])
@pytest.mark.parametrize("n_heads,n_kv_heads,head_dim,window", [
    (5, 5, 64, 0), (16, 1, 64, 0), (12, 4, 32, 0), (9, 3, 64, 100), (6, 3, 32, 64), (22, 2, 64, 0), (34, 2, 32, 0),
    (4, 2, 128, 0), (6, 1, 96, 70), (3, 3, 128, 200)])
def test_single_token_attention_on_tensor_cores(n_heads, n_kv_heads, head_dim, window, warps):
    """The tensor-core kernel of single-token steps (pages staged in shared
    memory by bulk copies) at its shapes of block, with and without blocks that share a
    sequence as a cluster (several pages per warp, more pages than the ring holds), with grouped heads up to 16 per kv head and windows
    that start inside a page; one key far back is made to carry most of the weight
    of its head, so a misplaced column shows."""
    from math_utils_b200.csrc import ops
    rng = np.random.default_rng(1000 * warps + head_dim + n_heads)
    seq_lens = [1, 2, 63, 64, 65, 128, 700, 1000]     # 16 pages: 8 per warp of 2, a ring holds 2
    kv, table, ks, vs = paged_setup(rng, seq_lens, n_kv_heads, head_dim, "bfloat16")
    scale = 1.0 / math.sqrt(head_dim)
    q = dev(rng.standard_normal((len(seq_lens), n_heads * head_dim)), torch.bfloat16)
    # the last sequences: the key at `far` answers head 1's query
    for s, far in ((6, 37), (7, 901)):
        if window and seq_lens[s] - far > window:
            far = seq_lens[s] - window            # the first position the window still holds
        h, g = 1, 1 // (n_heads // n_kv_heads)
        ks[s][far, g * head_dim:(g + 1) * head_dim] = (6.0 * q[s, h * head_dim:(h + 1) * head_dim].float()).to(torch.bfloat16)
    tok_pos = torch.tensor([p for n in seq_lens for p in range(n - 1)], dtype=torch.int32, device="cuda")
    tok_seq = torch.tensor([s for s, n in enumerate(seq_lens) for _ in range(n - 1)], dtype=torch.int32, device="cuda")
    ops.kv_append(torch.cat([k[:-1] for k in ks]), torch.cat([v[:-1] for v in vs]), tok_pos, tok_seq, table, 64,
                  n_kv_heads, head_dim, kv)
    k_new = torch.stack([k[-1] for k in ks]).contiguous()
    v_new = torch.stack([v[-1] for v in vs]).contiguous()
    pos1 = torch.tensor([n - 1 for n in seq_lens], dtype=torch.int32, device="cuda")
    assert ops.decode_tc_ok(q, k_new, v_new, kv, 64, n_heads, n_kv_heads, head_dim) == (n_heads // n_kv_heads <= 16)
    want = np.stack([plain_gpt2.causal_attention(
        np.repeat(q[s:s + 1].double().cpu().numpy(), n, axis=0), ks[s].double().cpu().numpy(),
        vs[s].double().cpu().numpy(), n_heads, n_kv_heads, scale, window)[-1] for s, n in enumerate(seq_lens)])
    vmax = max(float(v.abs().max()) for v in vs)
    for round_ in range(2):                       # with the append, then over the appended cache
        out = torch.full_like(q, float("nan"))
        ops.attention_decode(q, k_new if round_ == 0 else None, v_new if round_ == 0 else None, out, kv, table, 64,
                             pos1, None, n_heads, n_kv_heads, head_dim, scale, window, table.shape[1], warps=warps)
        # probabilities are rounded to bfloat16 before they meet the values: 2^-9 of a value's size each
        assert_close(out.float().cpu().numpy(), want, "bfloat16", f"launch {round_}", extra_abs=2.0 ** -8 * vmax)
    out2 = torch.empty_like(q)
    seq1 = torch.arange(len(seq_lens), dtype=torch.int32, device="cuda")
    ops.attention(q, out2, kv, table, 64, pos1, seq1, n_heads, n_kv_heads, head_dim, scale, window)
    assert_close(out2.float().cpu().numpy(), want, "bfloat16", "the general kernel over the appended cache")
    ops.check_status()


@pytest.mark.parametrize("m,n,k", [(1, 50, 24), (8, 2304, 768), (13, 77, 40), (16, 1031, 96), (3, 130, 1600),
                                   (12, 130, 8192), (5, 72, 4096), (24, 2304, 768), (32, 3072, 768), (17, 130, 1600),
                                   (29, 77, 40), (20, 768, 1024)])
@pytest.mark.parametrize("act", [None, "gelu_new"])
def test_product_with_the_norm_inside(m, n, k, act):
    """LayerNorm folded into the few-rows product against norm-then-product; rows too wide for the
    kernel's shared memory (12 x 8,192) are normed first instead of refused."""
    from math_utils_b200.csrc import ops
    rng = np.random.default_rng(m + n + k)
    x = (rng.standard_normal((m + 3, k)) * 2 + 0.5).astype(np.float32)
    g, b = rng.standard_normal(k).astype(np.float32), rng.standard_normal(k).astype(np.float32)
    w = dev(rng.standard_normal((n, k)) / math.sqrt(k), torch.bfloat16)
    bias = dev(rng.standard_normal(n))
    rows = torch.tensor(rng.permutation(m + 3)[:m].astype(np.int32), device="cuda")
    for r in (None, rows):
        lazy = ops.NormedInput(dev(x if r is not None else x[:m]), dev(g), dev(b), 1e-5, torch.bfloat16, rows=r)
        got = ops.linear(lazy, w, bias, act=act, out_dtype=torch.float32).cpu().numpy()
        src = x[:m] if r is None else x[r.cpu().numpy()]
        h = plain_gpt2.layer_norm(src.astype(np.float64), g.astype(np.float64), b.astype(np.float64), 1e-5)
        h = dev(h, torch.bfloat16).double().cpu().numpy()           # the kernel rounds the norm to bfloat16
        z = h[:m] @ w.double().cpu().numpy().T + bias.double().cpu().numpy()
        if act:
            z = plain_gpt2.ACTIVATIONS[act](z)
        # a normed value that lands on a rounding boundary may round the other way: allow for one such
        # flip per row on top of the float32 bound (2^-9 of one term among k)
        rms = np.sqrt((z ** 2).mean())
        assert np.abs(got - z).max() < 1e-5 * rms + 2.0 ** -8 * 4.0 / math.sqrt(k) * 3, (m, n, k)


@pytest.mark.parametrize("m,n,k", [(65, 64, 64), (128, 128, 64), (129, 130, 72), (257, 200, 328), (1000, 520, 768),
                                   (2048, 2304, 768), (2048, 768, 3072), (300, 1031, 96), (70, 50257, 64)])
@pytest.mark.parametrize("tile", [0, 64, 128, 256])
def test_tensor_core_product(m, n, k, tile):
    """The tcgen05 / TMA kernel at ragged sizes: more than one k-block ring turn,
    edges in m, n and k, every tile width (0: the kernel's own choice), every
    epilogue."""
    from math_utils_b200.csrc import ops
    rng = np.random.default_rng(m + n + k)
    a = dev(rng.standard_normal((m, k)), torch.bfloat16)
    w = dev(rng.standard_normal((n, k)) / math.sqrt(k), torch.bfloat16)
    bias = dev(rng.standard_normal(n))
    res = dev(rng.standard_normal((m, n)))
    assert ops.tc_ok(a, w)
    z = a.double().cpu().numpy() @ w.double().cpu().numpy().T
    got = ops.gemm_tc(a, w, None, out_dtype=torch.float32, tile=tile).cpu().numpy()
    ops.check_status()
    assert_close(got, z, "float32", "plain product", k=k)
    zb = z + bias.double().cpu().numpy()
    got = ops.gemm_tc(a, w, bias, act="gelu_new", tile=tile).float().cpu().numpy()
    assert_close(got, plain_gpt2.gelu_new(zb), "bfloat16", "bias, gelu, bfloat16 out")
    x = res.clone()
    ops.gemm_tc(a, w, bias, residual=x, out=x, tile=tile)
    assert_close(x.cpu().numpy(), zb + res.double().cpu().numpy(), "float32", "residual in place", k=k)
    ops.check_status()


@pytest.mark.parametrize("m,n,k", [(64, 2304, 768), (64, 768, 3072), (40, 770, 1600), (17, 50, 256), (33, 1031, 96),
                                   (64, 3072, 768), (5, 100, 72), (64, 1600, 6400), (1, 16, 64), (64, 768, 768)])
@pytest.mark.parametrize("splits", [0, 1, 2, 8, 16])
def test_rows_product(m, n, k, splits):
    """The tcgen05 kernel for up to 64 rows (the weights as the 128-row operand, k cut over a thread-block
    cluster whose blocks each finish a share of the tile's columns from parts pushed into their shared
    memory): its own choice of the cut and forced ones (16 falls back to 8 where the device has no
    clusters of 16), ragged edges in every direction, a k longer than the ring of stages holds, every
    epilogue; twice, bit for bit the same, since the parts are added in rank order."""
    from math_utils_b200.csrc import ops
    rng = np.random.default_rng(m + n + k)
    a = dev(rng.standard_normal((m, k)), torch.bfloat16)
    w = dev(rng.standard_normal((n, k)) / math.sqrt(k), torch.bfloat16)
    bias = dev(rng.standard_normal(n))
    res = dev(rng.standard_normal((m, n)))
    z = a.double().cpu().numpy() @ w.double().cpu().numpy().T
    zb = z + bias.double().cpu().numpy()
    runs = []
    for _ in range(2):
        got = ops.gemm_rows(a, w, None, out_dtype=torch.float32, splits=splits)
        assert_close(got.cpu().numpy(), z, "float32", "plain product", k=k)
        act = ops.gemm_rows(a, w, bias, act="gelu_new", splits=splits)
        assert_close(act.float().cpu().numpy(), plain_gpt2.gelu_new(zb), "bfloat16", "bias, gelu, bfloat16 out")
        x = res.clone()
        ops.gemm_rows(a, w, bias, residual=x, out=x, splits=splits)
        assert_close(x.cpu().numpy(), zb + res.double().cpu().numpy(), "float32", "residual in place", k=k)
        ops.check_status()
        runs.append((got, act, x))
    for first, second in zip(*runs):
        assert torch.equal(first, second)
    # a view with a row stride of its own, as the engine's q | k | v buffer has
    wide = torch.zeros((m, n + 24), dtype=torch.bfloat16, device="cuda")
    ops.gemm_rows(a, w, bias, out=wide[:, 8:8 + n], splits=splits)
    assert_close(wide[:, 8:8 + n].float().cpu().numpy(), zb, "bfloat16", "into a strided view")
    assert float(wide[:, :8].abs().sum()) == 0.0 and float(wide[:, 8 + n:].abs().sum()) == 0.0


@pytest.mark.parametrize("m,n,k", [(8, 50257, 768), (1, 50257, 768), (5, 40003, 776), (16, 38000, 384), (3, 70, 64),
                                   (11, 9001, 520)])
def test_streamed_product(m, n, k):
    """The product for an output head (few rows, very many columns): weights through shared memory by bulk
    copies, tile after tile per block.  With given activations and with the norm made inside; a last tile
    with fewer rows than a strip, or none in a strip; a k that is no multiple of 32; bias and gelu; a
    strided output; twice, bit for bit the same."""
    from math_utils_b200.csrc import ops
    rng = np.random.default_rng(m + n + k)
    a = dev(rng.standard_normal((m, k)), torch.bfloat16)
    w = dev(rng.standard_normal((n, k)) / math.sqrt(k), torch.bfloat16)
    bias = dev(rng.standard_normal(n))
    assert ops.library().mu_gemm_stream_fits(m, k, k, 1) == 1
    z = a.double().cpu().numpy() @ w.double().cpu().numpy().T
    zb = z + bias.double().cpu().numpy()
    runs = []
    for _ in range(2):
        got = ops.gemm_stream(a, w, None, out_dtype=torch.float32)
        assert_close(got.cpu().numpy(), z, "float32", "plain product", k=k)
        act = ops.gemm_stream(a, w, bias, act="gelu_new")
        assert_close(act.float().cpu().numpy(), plain_gpt2.gelu_new(zb), "bfloat16", "bias, gelu, bfloat16 out")
        runs.append((got, act))
    assert torch.equal(runs[0][0], runs[1][0]) and torch.equal(runs[0][1], runs[1][1])
    # the norm made inside: rows picked out of a larger float32 matrix, a mean far from zero
    x = (rng.standard_normal((m + 3, k)) * 2 + 4).astype(np.float32)
    rows = rng.permutation(m + 3)[:m].astype(np.int32)
    gamma, beta = rng.standard_normal(k).astype(np.float32), rng.standard_normal(k).astype(np.float32)
    normed = plain_gpt2.layer_norm(x[rows].astype(np.float64), gamma.astype(np.float64), beta.astype(np.float64), 1e-5)
    as_bf16 = dev(normed, torch.bfloat16).double().cpu().numpy()          # the kernel rounds the normed rows
    lazy = ops.NormedInput(dev(x), dev(gamma), dev(beta), 1e-5, torch.bfloat16, rows=torch.from_numpy(rows).cuda())
    wide = torch.zeros((m, n + 9), dtype=torch.float32, device="cuda")
    ops.gemm_stream(lazy, w, None, out=wide[:, 4:4 + n])
    # the norm made inside is the norm kernel's arithmetic: the same bfloat16 rows, hence the same product to the bit
    separate = ops.gemm_stream(lazy.materialize_copy(), w, None, out_dtype=torch.float32)
    assert torch.equal(wide[:, 4:4 + n], separate)
    # and against the plain norm: a normed value that lands on a rounding boundary may round the other way
    # (2^-9 of its size, times a weight): allow for a handful of such flips per row on top of the float32 bound
    z_normed = as_bf16 @ w.double().cpu().numpy().T
    rms = np.sqrt((z_normed ** 2).mean())
    flip = 2.0 ** -9 * np.abs(as_bf16).max() * float(w.abs().max())
    assert np.abs(wide[:, 4:4 + n].cpu().numpy() - z_normed).max() < 1e-5 * rms + 6 * flip
    assert float(wide[:, :4].abs().sum()) == 0.0 and float(wide[:, 4 + n:].abs().sum()) == 0.0
    ops.check_status()
    # sizes it does not take are refused, not mangled
    assert ops.library().mu_gemm_stream_fits(17, k, k, 0) == 0 and ops.library().mu_gemm_stream_fits(m, 4096, 4096, 0) == 0
    assert ops.library().mu_gemm_stream_fits(m, k, k + 8, 0) == 0


@pytest.mark.parametrize("m,n,k", [(64, 2304, 768), (64, 768, 3072), (40, 770, 1600), (128, 264, 2048), (200, 72, 520),
                                   (33, 50, 256)])
@pytest.mark.parametrize("parts", [-1, 2, 5, 64])
def test_tensor_core_product_cut_along_k(m, n, k, parts):
    """Few output tiles and a long k: the kernel cuts k over several blocks, which leave their parts in a
    workspace; the block with a tile's last ticket adds them in the order of k.  The kernel's own choice of
    parts and forced ones (64: as many as k has 64-deep stages), ragged edges, every epilogue; run twice,
    since a launch must leave the tickets as it found them, and bit for bit the same, since the order of
    the sum is fixed."""
    from math_utils_b200.csrc import ops
    rng = np.random.default_rng(m + n + k)
    a = dev(rng.standard_normal((m, k)), torch.bfloat16)
    w = dev(rng.standard_normal((n, k)) / math.sqrt(k), torch.bfloat16)
    bias = dev(rng.standard_normal(n))
    res = dev(rng.standard_normal((m, n)))
    z = a.double().cpu().numpy() @ w.double().cpu().numpy().T
    zb = z + bias.double().cpu().numpy()
    runs = []
    for _ in range(2):
        got = ops.gemm_tc(a, w, None, out_dtype=torch.float32, splits=parts)
        assert_close(got.cpu().numpy(), z, "float32", "plain product", k=k)
        act = ops.gemm_tc(a, w, bias, act="gelu", splits=parts)
        assert_close(act.float().cpu().numpy(), plain_gpt2.gelu_erf(zb), "bfloat16", "bias, gelu, bfloat16 out")
        x = res.clone()
        ops.gemm_tc(a, w, bias, residual=x, out=x, splits=parts)
        assert_close(x.cpu().numpy(), zb + res.double().cpu().numpy(), "float32", "residual in place", k=k)
        ops.check_status()
        runs.append((got, act, x))
    for first, second in zip(*runs):
        assert torch.equal(first, second)


@pytest.mark.parametrize("n_heads,n_kv_heads,head_dim,window", [
    (4, 4, 16, 0), (6, 2, 48, 0), (3, 3, 80, 0), (8, 2, 128, 70), (12, 12, 64, 0), (4, 2, 32, 1), (2, 1, 112, 130)])
def test_prompt_attention_on_tensor_cores(n_heads, n_kv_heads, head_dim, window):
    """Whole prompts and a prompt continued from a filled cache, tiles that end
    inside a page, several sequences in one launch."""
    from math_utils_b200.csrc import ops
    rng = np.random.default_rng(11 * head_dim + n_heads)
    totals = [1, 64, 65, 200, 333]
    starts = [0, 0, 0, 70, 128]                    # tokens the cache already holds
    kv, table, ks, vs = paged_setup(rng, totals, n_kv_heads, head_dim, "bfloat16")
    all_pos = torch.tensor([p for n in totals for p in range(n)], dtype=torch.int32, device="cuda")
    all_seq = torch.tensor([s for s, n in enumerate(totals) for _ in range(n)], dtype=torch.int32, device="cuda")
    ops.kv_append(torch.cat(ks), torch.cat(vs), all_pos, all_seq, table, 64, n_kv_heads, head_dim, kv)
    tok_pos = torch.tensor([p for n, s in zip(totals, starts) for p in range(s, n)], dtype=torch.int32, device="cuda")
    tok_seq = torch.tensor([i for i, (n, s) in enumerate(zip(totals, starts)) for _ in range(s, n)],
                           dtype=torch.int32, device="cuda")
    tiles, flat = [], 0
    for n, s in zip(totals, starts):
        for o in range(0, n - s, 64):
            tiles.append((flat + o, min(64, n - s - o)))
        flat += n - s
    tiles_t = torch.tensor(tiles, dtype=torch.int32, device="cuda")
    q_all = dev(rng.standard_normal((flat, n_heads * head_dim + 8)), torch.bfloat16)[:, :n_heads * head_dim]
    out = torch.full((flat, n_heads * head_dim), float("nan"), dtype=torch.bfloat16, device="cuda")
    scale = 0.6 / math.sqrt(head_dim)
    assert ops.prefill_ok(q_all, head_dim, 64)
    ops.attention_prefill(q_all, out, kv, table, 64, tok_pos, tok_seq, tiles_t, n_heads, n_kv_heads, head_dim,
                          scale, window)
    o = 0
    for i, (n, s) in enumerate(zip(totals, starts)):
        want = plain_gpt2.causal_attention(q_all[o:o + n - s].double().cpu().numpy(), ks[i].double().cpu().numpy(),
                                           vs[i].double().cpu().numpy(), n_heads, n_kv_heads, scale, window, start=s)
        # probabilities are rounded to bfloat16 before they meet the values: where one key carries
        # most of the weight that is up to 2^-9 of the largest value, whatever the size of the output
        vmax = float(vs[i].abs().max())
        assert_close(out[o:o + n - s].float().cpu().numpy(), want, "bfloat16", f"sequence {i}",
                     extra_abs=2.0 ** -8 * vmax)
        o += n - s


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("n_kv_heads,head_dim", [(3, 16), (2, 64), (1, 80), (5, 256)])
def test_append_by_tiles_writes_the_same_cache(n_kv_heads, head_dim, dtype):
    """Keys and values appended a tile at a time (16-byte runs of positions
    where the tile's first position allows it) leave the cache as the
    token-by-token append does: whole tiles, tails, tiles that start inside a
    page at positions that are and are not multiples of 8."""
    from math_utils_b200.csrc import ops
    rng = np.random.default_rng(head_dim + n_kv_heads)
    totals = [1, 64, 65, 200, 333, 100]
    starts = [0, 0, 0, 70, 128, 8]
    kv_a, table, ks, vs = paged_setup(rng, totals, n_kv_heads, head_dim, dtype)
    kv_b = torch.zeros_like(kv_a)
    tok_pos = torch.tensor([p for n, s in zip(totals, starts) for p in range(s, n)], dtype=torch.int32, device="cuda")
    tok_seq = torch.tensor([i for i, (n, s) in enumerate(zip(totals, starts)) for _ in range(s, n)],
                           dtype=torch.int32, device="cuda")
    k_all = torch.cat([k[s:] for k, s in zip(ks, starts)])
    v_all = torch.cat([v[s:] for v, s in zip(vs, starts)])
    tiles, flat = [], 0
    for n, s in zip(totals, starts):
        for o in range(0, n - s, 64):
            tiles.append((flat + o, min(64, n - s - o)))
        flat += n - s
    tiles_t = torch.tensor(tiles, dtype=torch.int32, device="cuda")
    ops.kv_append(k_all, v_all, tok_pos, tok_seq, table, 64, n_kv_heads, head_dim, kv_a)
    ops.kv_append(k_all, v_all, tok_pos, tok_seq, table, 64, n_kv_heads, head_dim, kv_b, tiles=tiles_t)
    assert torch.equal(kv_a, kv_b)
    # and the layout itself: a key row per position, a value row per dimension
    page = int(table[4, 2])                                   # sequence 4, positions 128..191
    flat_k = kv_a[page, 0].reshape(n_kv_heads, 64, head_dim)
    flat_v = kv_a[page, 1].reshape(n_kv_heads, head_dim, 64)
    want_k = ks[4][128:192].reshape(64, n_kv_heads, head_dim).permute(1, 0, 2)
    want_v = vs[4][128:192].reshape(64, n_kv_heads, head_dim).permute(1, 2, 0)
    assert torch.equal(flat_k, want_k) and torch.equal(flat_v, want_v)


@pytest.mark.parametrize("n_heads,n_kv_heads,window", [(12, 12, 0), (4, 2, 0), (6, 2, 100), (3, 1, 64), (2, 2, 1)])
def test_prompt_attention_on_tcgen05(n_heads, n_kv_heads, window):
    """The tcgen05 prompt kernel (head size 64): whole prompts and prompts
    continued from a filled cache, tiles of up to 128 queries that start and end
    inside pages, several sequences in one launch, grouped heads and windows;
    in the longest sequence one key far back answers one head's last queries, so
    a misplaced page or column shows."""
    from math_utils_b200.csrc import ops
    head_dim = 64
    rng = np.random.default_rng(17 * n_heads + window)
    totals = [1, 64, 65, 200, 333, 1000]
    starts = [0, 0, 0, 70, 128, 0]                 # tokens the cache already holds
    kv, table, ks, vs = paged_setup(rng, totals, n_kv_heads, head_dim, "bfloat16")
    flat_total = sum(n - s for n, s in zip(totals, starts))
    q_all = dev(rng.standard_normal((flat_total, n_heads * head_dim + 16)), torch.bfloat16)[:, :n_heads * head_dim]
    # sequence 5, head 1: the key at `far` is six times the last query of the head
    far = 1000 - window if window and window < 900 else 37
    off5 = flat_total - 1000
    g = 1 // (n_heads // n_kv_heads) if n_heads > 1 else 0
    hq = 1 if n_heads > 1 else 0
    ks[5][far, g * head_dim:(g + 1) * head_dim] = (6.0 * q_all[off5 + 999, hq * head_dim:(hq + 1) * head_dim].float()).to(torch.bfloat16)
    all_pos = torch.tensor([p for n in totals for p in range(n)], dtype=torch.int32, device="cuda")
    all_seq = torch.tensor([s for s, n in enumerate(totals) for _ in range(n)], dtype=torch.int32, device="cuda")
    ops.kv_append(torch.cat(ks), torch.cat(vs), all_pos, all_seq, table, 64, n_kv_heads, head_dim, kv)
    tok_pos = torch.tensor([p for n, s in zip(totals, starts) for p in range(s, n)], dtype=torch.int32, device="cuda")
    tok_seq = torch.tensor([i for i, (n, s) in enumerate(zip(totals, starts)) for _ in range(s, n)],
                           dtype=torch.int32, device="cuda")
    tiles, flat = [], 0
    for n, s in zip(totals, starts):
        for o in range(0, n - s, 128):
            tiles.append((flat + o, min(128, n - s - o)))
        flat += n - s
    tiles.sort(key=lambda t: -t[1])
    tiles_t = torch.tensor(tiles, dtype=torch.int32, device="cuda")
    out = torch.full((flat, n_heads * head_dim), float("nan"), dtype=torch.bfloat16, device="cuda")
    scale = 1.0 / math.sqrt(head_dim)
    assert ops.prefill_tc_ok(q_all, out, head_dim, 64)
    ops.attention_prefill_tc(q_all, out, kv, table, 64, tok_pos, tok_seq, tiles_t, n_heads, n_kv_heads, head_dim,
                             scale, window)
    ops.check_status()
    o = 0
    for i, (n, s) in enumerate(zip(totals, starts)):
        want = plain_gpt2.causal_attention(q_all[o:o + n - s].double().cpu().numpy(), ks[i].double().cpu().numpy(),
                                           vs[i].double().cpu().numpy(), n_heads, n_kv_heads, scale, window, start=s)
        vmax = float(vs[i].abs().max())
        assert_close(out[o:o + n - s].float().cpu().numpy(), want, "bfloat16", f"sequence {i}",
                     extra_abs=2.0 ** -8 * vmax)
        o += n - s
