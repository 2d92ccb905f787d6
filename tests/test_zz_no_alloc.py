"""mu_attention_static_scratch, the attention entry point for callers that cannot
allocate device memory (a plug-in inside someone else's memory pool, a loop
that must stay out of the allocator): its scratch is a fixed array inside the
library.  Called here through its exported C symbol, twice in a row with
different inputs, and compared with the ordinary entry point, which takes its
scratch from the caller, and with the plain attention of tests/plain_gpt2.py.
This file is collected last on purpose."""
import ctypes
import math

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu

STATIC_SCRATCH_FLOATS = 1 << 20
ERR_STATIC_SCRATCH = 6


def c_entry():
    from math_utils_b200.csrc import ops
    lib = ops.library()
    fn = lib.mu_attention_static_scratch
    p, ll, i, f = ctypes.c_void_p, ctypes.c_longlong, ctypes.c_int, ctypes.c_float
    fn.argtypes = [p, ll, p, ll, p, p, i, i, p, p, i, i, i, i, f, i, i, i, i, p]
    fn.restype = i
    return fn


def make_case(seed, dtype, lens, n_heads, n_kv_heads, head_dim):
    from math_utils_b200.csrc import ops
    g = torch.Generator(device="cuda").manual_seed(seed)
    page = 64
    pages_of = [-(-n // page) for n in lens]
    n_pages = sum(pages_of) + 2
    kv = torch.zeros((n_pages, 2, n_kv_heads, page, head_dim), dtype=dtype, device="cuda")
    table = torch.zeros((len(lens), max(pages_of)), dtype=torch.int32)
    order = torch.randperm(n_pages, generator=torch.Generator().manual_seed(seed)).tolist()
    nxt = 0
    for s, k in enumerate(pages_of):
        for j in range(k):
            table[s, j] = order[nxt]; nxt += 1
    table = table.cuda()
    pos = torch.tensor([p for n in lens for p in range(n)], dtype=torch.int32, device="cuda")
    seq = torch.tensor([s for s, n in enumerate(lens) for _ in range(n)], dtype=torch.int32, device="cuda")
    k = torch.randn((sum(lens), n_kv_heads * head_dim), generator=g, device="cuda").to(dtype)
    v = torch.randn((sum(lens), n_kv_heads * head_dim), generator=g, device="cuda").to(dtype)
    ops.kv_append(k, v, pos, seq, table, page, n_kv_heads, head_dim, kv)
    q = torch.randn((len(lens), n_heads * head_dim), generator=g, device="cuda").to(dtype)
    qpos = torch.tensor([n - 1 for n in lens], dtype=torch.int32, device="cuda")
    qseq = torch.arange(len(lens), dtype=torch.int32, device="cuda")
    make_case.keys_values = (k.double().cpu().numpy(), v.double().cpu().numpy())      # for the plain attention
    return q, kv, table, qpos, qseq


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_static_scratch_matches_caller_scratch_twice(dtype):
    from math_utils_b200.csrc import ops
    fn = c_entry()
    n_heads, n_kv_heads, head_dim, n_splits, split_keys = 6, 2, 48, 4, 64
    stream = torch.cuda.current_stream().cuda_stream
    for call, lens in enumerate(([200, 37, 129], [64, 250, 5])):          # the second call meets the first one's leftovers
        q, kv, table, qpos, qseq = make_case(10 + call, dtype, lens, n_heads, n_kv_heads, head_dim)
        scale = 1.0 / math.sqrt(head_dim)
        units = len(lens) * n_heads * n_splits
        want = torch.empty_like(q)
        ops.attention(q, want, kv, table, 64, qpos, qseq, n_heads, n_kv_heads, head_dim, scale, 0, n_splits,
                      split_keys, torch.empty(units * head_dim, device="cuda"), torch.empty(units * 2, device="cuda"))
        got = torch.full_like(q, float("nan"))
        torch.cuda.synchronize()
        rc = fn(q.data_ptr(), q.stride(0), got.data_ptr(), got.stride(0), kv.data_ptr(), table.data_ptr(),
                table.shape[1], 64, qpos.data_ptr(), qseq.data_ptr(), len(lens), n_heads, n_kv_heads, head_dim,
                scale, 0, n_splits, split_keys, int(dtype == torch.bfloat16), stream)
        torch.cuda.synchronize()
        assert rc == 0
        # same kernels, same order of operations: the two entry points agree to the last bit,
        # which is well inside the 1e-5 x rms that the kernel tests allow
        diff = (got.float() - want.float()).abs().max().item()
        rms = want.float().pow(2).mean().sqrt().item()
        assert torch.isfinite(got.float()).all() and diff <= 1e-5 * rms, (call, diff, rms)
        # and both are the attention the plain implementation computes: each sequence's last query over all
        # of its keys, with the bounds of the kernel tests
        import plain_gpt2
        from test_kernels_gpu import assert_close
        keys, values = make_case.keys_values
        start = 0
        for s, n in enumerate(lens):
            qs = np.repeat(q[s:s + 1].double().cpu().numpy(), n, axis=0)
            plain = plain_gpt2.causal_attention(qs, keys[start:start + n], values[start:start + n], n_heads, n_kv_heads,
                                                scale)[-1]
            assert_close(got[s].float().cpu().numpy(), plain, "float32" if dtype == torch.float32 else "bfloat16",
                         f"call {call} sequence {s}")
            start += n


def test_static_scratch_refuses_what_does_not_fit():
    fn = c_entry()
    q, kv, table, qpos, qseq = make_case(3, torch.float32, [70, 70], 4, 4, 64)
    out = torch.zeros_like(q)
    n_tokens, n_heads, head_dim = 2, 4, 64
    n_splits = STATIC_SCRATCH_FLOATS // (n_tokens * n_heads * (head_dim + 2)) + 1
    rc = fn(q.data_ptr(), q.stride(0), out.data_ptr(), out.stride(0), kv.data_ptr(), table.data_ptr(),
            table.shape[1], 64, qpos.data_ptr(), qseq.data_ptr(), n_tokens, n_heads, 4, head_dim, 0.125, 0,
            n_splits, 32, 0, torch.cuda.current_stream().cuda_stream)
    torch.cuda.synchronize()
    assert rc == ERR_STATIC_SCRATCH and float(out.abs().sum()) == 0.0      # refused, nothing launched
