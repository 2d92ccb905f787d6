"""Python face of the CUDA kernels: torch tensors in, launches on the current stream.

The kernels live in one shared object built from the ``.cu`` files beside this
module (``build.py``) and are called through their ``extern "C"`` launchers.
There is no other implementation behind these functions: if the library cannot
be built or loaded, or a tensor is not on a CUDA device, they raise.
"""
from __future__ import annotations

import ctypes
import os
import threading
from typing import Optional

import torch

from . import build

ACT_CODES = {None: 0, "none": 0, "gelu_new": 1, "gelu": 2}

_ERRORS = {
    1: "bad argument (a size, stride or pointer the kernel cannot take)",
    2: "unsupported size for this kernel",
    3: "the CUDA runtime refused the launch",
    4: "a pointer or stride breaks an alignment rule of this kernel",
    5: "the kernel library could not set itself up on this device",
}


class KernelError(RuntimeError):
    pass


_lib = None
_lock = threading.Lock()


def _switch(name: str) -> bool:
    return os.environ.get(name, "1") != "0"


# Switches for measurements, read once when this module is imported:
#   MU_B200_PDL=0         plain stream order between kernels (no programmatic dependent launch)
#   MU_B200_ATT_TC=0      single-token attention on CUDA cores instead of mma.sync
#   MU_B200_PREFILL_TC=0  prompt attention on mma.sync instead of tcgen05
PDL, ATT_TC, PREFILL_TC = _switch("MU_B200_PDL"), _switch("MU_B200_ATT_TC"), _switch("MU_B200_PREFILL_TC")

_c_int, _c_ll, _c_f, _c_p, _c_ull = ctypes.c_int, ctypes.c_longlong, ctypes.c_float, ctypes.c_void_p, ctypes.c_ulonglong

_SIGNATURES = {
    "mu_copy_async": [_c_p, _c_p, _c_ll, _c_p],
    "mu_embed": [_c_p, _c_p, _c_p, _c_p, _c_p, _c_int, _c_int, _c_int, _c_p],
    "mu_layernorm": [_c_p, _c_p, _c_p, _c_p, _c_p, _c_int, _c_int, _c_f, _c_int, _c_p],
    "mu_gemm_simt": [_c_p, _c_p, _c_p, _c_p, _c_p, _c_int, _c_int, _c_int, _c_ll, _c_ll, _c_ll, _c_ll,
                     _c_int, _c_int, _c_int, _c_p],
    "mu_gemm_skinny": [_c_p, _c_p, _c_p, _c_p, _c_p, _c_int, _c_int, _c_int, _c_ll, _c_ll, _c_ll, _c_ll,
                       _c_int, _c_int, _c_p],
    "mu_gemm_tc_split_workspace": [_c_p, _c_ll, _c_p, _c_int],
    "mu_gemm_tc": [_c_p, _c_p, _c_p, _c_p, _c_p, _c_int, _c_int, _c_int, _c_ll, _c_ll, _c_ll, _c_ll,
                   _c_int, _c_int, _c_int, _c_int, _c_p, _c_p],
    "mu_gemm_rows": [_c_p, _c_p, _c_p, _c_p, _c_p, _c_int, _c_int, _c_int, _c_ll, _c_ll, _c_ll, _c_ll,
                     _c_int, _c_int, _c_int, _c_p, _c_p],
    "mu_kv_append": [_c_p, _c_ll, _c_p, _c_ll, _c_p, _c_p, _c_p, _c_int, _c_int, _c_int, _c_int,
                     _c_int, _c_p, _c_int, _c_p, _c_int, _c_p],
    "mu_attention": [_c_p, _c_ll, _c_p, _c_ll, _c_p, _c_p, _c_int, _c_int, _c_p, _c_p, _c_int,
                     _c_int, _c_int, _c_int, _c_f, _c_int, _c_int, _c_int, _c_p, _c_p, _c_int, _c_p],
    "mu_attention_prefill": [_c_p, _c_ll, _c_p, _c_ll, _c_p, _c_p, _c_int, _c_int, _c_p, _c_p, _c_p, _c_int,
                             _c_int, _c_int, _c_int, _c_f, _c_int, _c_p, _c_p],
    "mu_attention_prefill_tc": [_c_p, _c_ll, _c_int, _c_p, _c_ll, _c_p, _c_ll, _c_p, _c_int, _c_int, _c_p, _c_p,
                                _c_p, _c_int, _c_int, _c_int, _c_int, _c_f, _c_int, _c_p, _c_ll, _c_p, _c_ll,
                                _c_p, _c_int, _c_p, _c_p],
    "mu_layernorm_gemm_tc": [_c_p, _c_p, _c_p, _c_p, _c_f, _c_p, _c_p, _c_p, _c_p, _c_p, _c_int, _c_int, _c_int,
                             _c_ll, _c_ll, _c_ll, _c_int, _c_int, _c_p, _c_p],
    "mu_argmax": [_c_p, _c_ll, _c_int, _c_int, _c_p, _c_p, _c_p, _c_p, _c_int, _c_p, _c_p, _c_p],
    "mu_gemm_stream_fits": [_c_int, _c_int, _c_ll, _c_int],
    "mu_gemm_stream": [_c_p, _c_ll, _c_p, _c_ll, _c_p, _c_p, _c_p, _c_f, _c_p, _c_p, _c_p, _c_int, _c_int, _c_int,
                       _c_ll, _c_ll, _c_int, _c_int, _c_p, _c_p],
    "mu_gemm_skinny_ln": [_c_p, _c_ll, _c_p, _c_p, _c_p, _c_f, _c_p, _c_p, _c_p, _c_p, _c_int, _c_int, _c_int,
                          _c_ll, _c_ll, _c_ll, _c_int, _c_int, _c_p],
    "mu_attention_decode": [_c_p, _c_ll, _c_p, _c_ll, _c_p, _c_ll, _c_p, _c_ll, _c_p, _c_p, _c_int, _c_int,
                            _c_p, _c_p, _c_int, _c_int, _c_int, _c_int, _c_f, _c_int, _c_int, _c_int, _c_int, _c_p],
    "mu_attention_decode_tc": [_c_p, _c_ll, _c_p, _c_ll, _c_p, _c_ll, _c_p, _c_ll, _c_p, _c_p, _c_int, _c_int,
                               _c_p, _c_p, _c_int, _c_int, _c_int, _c_int, _c_f, _c_int, _c_int, _c_p, _c_p],
    "mu_sample": [_c_p, _c_ll, _c_int, _c_int, _c_f, _c_int, _c_ull, _c_p, _c_p, _c_p, _c_p, _c_p, _c_int,
                  _c_p, _c_p, _c_p],
}


def library() -> ctypes.CDLL:
    """The loaded kernel library; builds it at the first call if needed."""
    global _lib
    if _lib is None:
        with _lock:
            if _lib is None:
                path = build.library_path()
                try:
                    lib = ctypes.CDLL(path)
                except OSError as e:
                    raise KernelError(f"cannot load the CUDA kernels of math_utils_b200 from {path}: {e}") from None
                for name, argtypes in _SIGNATURES.items():
                    try:
                        fn = getattr(lib, name)
                    except AttributeError:
                        continue          # optional kernels are looked up where they are used
                    fn.argtypes = argtypes
                    fn.restype = _c_int
                if not PDL:
                    lib.mu_set_pdl(0)         # plain stream order between kernels
                _lib = lib
    return _lib


launch_count = 0      # kernels of this library launched so far (a merge after a split counts too)


def _check(code: int, what, launches: int = 1) -> None:
    """``what`` names the call for the error message: a string, or a tuple of a
    format and its arguments, put together only when there is an error."""
    global launch_count
    if code != 0:
        if isinstance(what, tuple):
            what = what[0].format(*what[1:])
        raise KernelError(f"{what}: {_ERRORS.get(code, f'error {code}')}")
    launch_count += launches


try:
    _raw_stream = torch._C._cuda_getCurrentRawStream        # the current stream's handle without a Stream object
except AttributeError:                                       # pragma: no cover
    _raw_stream = None


_current_device = getattr(torch._C, "_cuda_getDevice", None)


def _stream() -> int:
    if _raw_stream is not None and _current_device is not None:
        return _raw_stream(_current_device())
    return torch.cuda.current_stream().cuda_stream


def _ptr(t: Optional[torch.Tensor]) -> Optional[int]:
    return None if t is None else t.data_ptr()


def _need_cuda(*tensors) -> None:
    for t in tensors:
        if t is not None and not t.is_cuda:
            raise KernelError("math_utils_b200 kernels run on CUDA tensors only; got a tensor on " + str(t.device))


def _is_bf16(t: torch.Tensor) -> int:
    if t.dtype == torch.bfloat16:
        return 1
    if t.dtype == torch.float32:
        return 0
    raise KernelError(f"kernels take bfloat16 or float32, got {t.dtype}")


def _i32(t: Optional[torch.Tensor], name: str) -> None:
    if t is not None and (t.dtype != torch.int32 or not t.is_contiguous()):
        raise KernelError(f"{name} must be a contiguous int32 tensor")


def set_pdl(enabled: bool) -> None:
    """Switches programmatic stream serialization of the launches on or off
    (on unless MU_B200_PDL=0 when the module was imported): with it a kernel may start, and fetch what no
    kernel of the step writes, while the kernel before it ends.  Launches
    already recorded in a CUDA graph keep the mode they were recorded with."""
    library().mu_set_pdl(1 if enabled else 0)


def copy_async(dst: torch.Tensor, src: torch.Tensor, stream: Optional[torch.cuda.Stream] = None) -> None:
    """dst <- src (same size and dtype, contiguous; host tensors pinned) as a
    plain asynchronous copy on the current stream, or on ``stream``.  The
    caller keeps both tensors alive until the copy is over (a copy recorded in
    a CUDA graph: as long as the graph)."""
    if dst.dtype != src.dtype or dst.numel() != src.numel() or not dst.is_contiguous() or not src.is_contiguous():
        raise KernelError("copy_async needs contiguous tensors of one dtype and size")
    for t in (dst, src):
        if not t.is_cuda and not t.is_pinned():
            raise KernelError("copy_async needs pinned host memory")
    _check(library().mu_copy_async(dst.data_ptr(), src.data_ptr(), dst.numel() * dst.element_size(),
                                   _stream() if stream is None else stream.cuda_stream), "copy_async", launches=0)


_workspaces = {}
_retired = []


def zeroed_workspace(name: str, device, n_bytes: int) -> torch.Tensor:
    """A device buffer that kernels with tickets use and leave zero again.  It
    is kept per purpose and device and only ever grows, so its address stays put
    for launches recorded in a CUDA graph as long as no larger size is asked for
    later."""
    key = (name, str(device))
    buf = _workspaces.get(key)
    if buf is None or buf.numel() < n_bytes:
        if buf is not None:
            _retired.append(buf)        # a recorded graph may still point at it
        buf = torch.zeros(max(n_bytes, 65536), dtype=torch.uint8, device=device)
        _workspaces[key] = buf
    return buf


# ------------------------------------------------------------------ elementwise
def embed(ids: torch.Tensor, positions: Optional[torch.Tensor], table: torch.Tensor,
          pos_table: Optional[torch.Tensor], out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """out[t] = table[ids[t]] + pos_table[positions[t]] as float32 [T, hidden]."""
    _need_cuda(ids, positions, table, pos_table)
    _i32(ids, "ids"); _i32(positions, "positions")
    n, hidden = ids.numel(), table.shape[1]
    if pos_table is not None and (pos_table.dtype != table.dtype or pos_table.shape[1] != hidden):
        raise KernelError("the position table must match the token table in dtype and width")
    if not table.is_contiguous() or (pos_table is not None and not pos_table.is_contiguous()):
        raise KernelError("embedding tables must be contiguous")
    if out is None:
        out = torch.empty((n, hidden), dtype=torch.float32, device=table.device)
    _check(library().mu_embed(_ptr(ids), _ptr(positions),
                              _ptr(table), _ptr(pos_table), _ptr(out), n, hidden, _is_bf16(table), _stream()),
           "embed")
    return out


def layernorm(x: torch.Tensor, gamma: torch.Tensor, beta: Optional[torch.Tensor], eps: float,
              out_dtype: torch.dtype, rows: Optional[torch.Tensor] = None,
              out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """LayerNorm of float32 rows (optionally the rows that ``rows`` picks)."""
    _need_cuda(x, gamma, beta, rows)
    _i32(rows, "rows")
    if x.dtype != torch.float32 or not x.is_contiguous():
        raise KernelError("layernorm input must be contiguous float32")
    if gamma.dtype != torch.float32 or (beta is not None and beta.dtype != torch.float32):
        raise KernelError("layernorm parameters must be float32")
    hidden = x.shape[-1]
    n = rows.numel() if rows is not None else x.numel() // hidden
    if out is None:
        out = torch.empty((n, hidden), dtype=out_dtype, device=x.device)
    _check(library().mu_layernorm(_ptr(x), _ptr(rows), _ptr(gamma), _ptr(beta), _ptr(out), n, hidden,
                                  float(eps), _is_bf16(out), _stream()), ("layernorm(hidden={})", hidden))
    return out


# ------------------------------------------------------------------------ GEMM
def _gemm_args(a, w, bias, residual, out, out_dtype):
    _need_cuda(a, w, bias, residual, out)
    if a.dim() != 2 or w.dim() != 2 or a.shape[1] != w.shape[1]:
        raise KernelError(f"gemm shapes do not agree: a {tuple(a.shape)}, w {tuple(w.shape)}")
    if a.dtype != w.dtype:
        raise KernelError(f"gemm operands differ in dtype: {a.dtype} and {w.dtype}")
    if a.stride(1) != 1 or w.stride(1) != 1:
        raise KernelError("gemm operands must have unit stride along k")
    m, k = a.shape
    n = w.shape[0]
    if out is None:
        out = torch.empty((m, n), dtype=out_dtype, device=a.device)
    if out.shape != (m, n) or out.stride(1) != 1:
        raise KernelError("gemm output has the wrong shape or stride")
    if bias is not None and (bias.dtype != torch.float32 or bias.numel() != n):
        raise KernelError("gemm bias must be float32 of length n")
    if residual is not None and (residual.dtype != torch.float32 or residual.shape != (m, n)
                                 or residual.stride(1) != 1):
        raise KernelError("gemm residual must be float32 [m, n]")
    return m, n, k, out


def gemm_simt(a: torch.Tensor, w: torch.Tensor, bias: Optional[torch.Tensor] = None,
              act: Optional[str] = None, residual: Optional[torch.Tensor] = None,
              out: Optional[torch.Tensor] = None, out_dtype: Optional[torch.dtype] = None) -> torch.Tensor:
    """out = act(a @ w^T + bias) + residual on CUDA cores, any shape, any of the
    two dtypes; with float32 operands this is the true 32-bit product."""
    m, n, k, out = _gemm_args(a, w, bias, residual, out, out_dtype or a.dtype)
    _check(library().mu_gemm_simt(
        _ptr(a), _ptr(w), _ptr(bias), _ptr(residual), _ptr(out), m, n, k, a.stride(0), w.stride(0),
        out.stride(0), residual.stride(0) if residual is not None else 0, ACT_CODES[act],
        _is_bf16(a), _is_bf16(out), _stream()), ("gemm_simt({}x{}x{})", m, n, k))
    return out


_status = {}


def status_word(device) -> torch.Tensor:
    """A device word that kernels with bounded waits write to when a wait runs
    out (it stays 0 otherwise); ``check_status`` reads it."""
    word = _status.get(device)
    if word is None:
        word = _status[device] = _status[str(device)] = torch.zeros(1, dtype=torch.int32, device=device)
        _split_workspace(device)
    return word


def _rows_kernel(m: int, n: int, k: int) -> bool:
    """Whether a product of m rows goes to ``mu_gemm_rows``: 33 to 64 rows always; 17 to 32 rows where the
    weights are 16 million or more (the output head, which that kernel streams faster than the few-rows
    kernel does at that many rows).  Up to 16 rows the few-rows kernel with the norm folded in stays ahead
    inside a step, where its weights are on their way while the kernels before it end."""
    return 33 <= m <= 64 or (17 <= m <= 32 and n * k >= (1 << 24))


def _split_workspace(device) -> None:
    """Room for tensor-core products that are cut along k (few output tiles,
    long k: a batch of 33 to 128 single tokens): partial tiles for one tile per
    SM at the widest tile, and a ticket per tile.  Set once per device, at the
    first use of a kernel with a status word, hence never inside a capture."""
    parts = scratch("gemm_tc_parts", device, sm_count(device) * 128 * 256, torch.float32)
    tickets = zeroed_workspace("gemm_tc_tickets", device, 4 * 1024)
    _check(library().mu_gemm_tc_split_workspace(parts.data_ptr(), parts.numel() * 4, tickets.data_ptr(),
                                                tickets.numel() // 4), "gemm_tc_split_workspace", launches=0)


_WAITS = {1: "tensor-core product: loads", 2: "tensor-core product: tensor cores",
          3: "tensor-core product: epilogue", 4: "single-token attention: a page copy",
          5: "prompt attention: loads", 6: "prompt attention: tensor cores", 7: "prompt attention: softmax",
          8: "streamed product: a weight copy"}


def raise_status(device, code: int) -> None:
    """Clears the status word and raises for the wait that ran out."""
    word = _status.get(str(torch.device(device)))
    if word is not None:
        word.zero_()
    raise KernelError(f"a kernel gave up a bounded wait ({_WAITS.get(code, f'code {code}')}); the results of "
                      "the steps since the last check are not valid")


def check_status(device="cuda:0") -> None:
    """Raises if a kernel gave up a bounded wait since the last check (this
    synchronises with the device)."""
    word = _status.get(str(torch.device(device)))
    if word is not None:
        code = int(word.item())
        if code != 0:
            raise_status(device, code)


def tc_ok(a: torch.Tensor, w: torch.Tensor) -> bool:
    """Whether gemm_tc takes this product (alignment rules of its TMA loads)."""
    return (a.dtype == torch.bfloat16 and a.shape[1] % 8 == 0 and a.stride(0) % 8 == 0
            and w.stride(0) % 8 == 0 and a.data_ptr() % 16 == 0 and w.data_ptr() % 16 == 0)


def gemm_tc(a: torch.Tensor, w: torch.Tensor, bias: Optional[torch.Tensor] = None,
            act: Optional[str] = None, residual: Optional[torch.Tensor] = None,
            out: Optional[torch.Tensor] = None, out_dtype: Optional[torch.dtype] = None,
            tile: int = 0, splits: int = -1) -> torch.Tensor:
    """The product on the tcgen05 tensor cores (TMA loads, accumulator in tensor memory).
    ``tile``: width of the output tiles (64, 128, 256; 0: the library chooses); ``splits``: parts that k
    is cut into (-1: the library chooses; 0 or 1: none)."""
    m, n, k, out = _gemm_args(a, w, bias, residual, out, out_dtype or a.dtype)
    _check(library().mu_gemm_tc(
        _ptr(a), _ptr(w), _ptr(bias), _ptr(residual), _ptr(out), m, n, k, a.stride(0), w.stride(0),
        out.stride(0), residual.stride(0) if residual is not None else 0, ACT_CODES[act],
        _is_bf16(out), int(tile), int(splits), _ptr(status_word(a.device)), _stream()),
        ("gemm_tc({}x{}x{})", m, n, k))
    return out


def gemm_rows(a: torch.Tensor, w: torch.Tensor, bias: Optional[torch.Tensor] = None,
              act: Optional[str] = None, residual: Optional[torch.Tensor] = None,
              out: Optional[torch.Tensor] = None, out_dtype: Optional[torch.dtype] = None,
              splits: int = 0) -> torch.Tensor:
    """The product for up to 64 rows on the tcgen05 tensor cores: tiles of 16 output columns, a block per
    tile, k cut over a thread-block cluster where the tiles are few (``splits`` blocks per tile, 0: chosen
    by the library), the parts added in rank order in the first block's shared memory."""
    m, n, k, out = _gemm_args(a, w, bias, residual, out, out_dtype or a.dtype)
    _check(library().mu_gemm_rows(
        _ptr(a), _ptr(w), _ptr(bias), _ptr(residual), _ptr(out), m, n, k, a.stride(0), w.stride(0),
        out.stride(0), residual.stride(0) if residual is not None else 0, ACT_CODES[act],
        _is_bf16(out), int(splits), _ptr(status_word(a.device)), _stream()), ("gemm_rows({}x{}x{})", m, n, k))
    return out


def gemm_skinny(a: torch.Tensor, w: torch.Tensor, bias: Optional[torch.Tensor] = None,
                act: Optional[str] = None, residual: Optional[torch.Tensor] = None,
                out: Optional[torch.Tensor] = None, out_dtype: Optional[torch.dtype] = None) -> torch.Tensor:
    """The product for a few rows (single-token steps): streams the weights once
    through mma.sync with the weight rows as the wide operand."""
    m, n, k, out = _gemm_args(a, w, bias, residual, out, out_dtype or a.dtype)
    _check(library().mu_gemm_skinny(
        _ptr(a), _ptr(w), _ptr(bias), _ptr(residual), _ptr(out), m, n, k, a.stride(0), w.stride(0),
        out.stride(0), residual.stride(0) if residual is not None else 0, ACT_CODES[act],
        _is_bf16(out), _stream()), ("gemm_skinny({}x{}x{})", m, n, k))
    return out


# ------------------------------------------------------------------- attention
def kv_append(k: torch.Tensor, v: torch.Tensor, tok_pos, tok_seq, block_table: torch.Tensor,
              page_tokens: int, n_kv_heads: int, head_dim: int, kv_pages: torch.Tensor,
              tiles: Optional[torch.Tensor] = None) -> None:
    """Copies keys and values of this step's tokens ([T, n_kv_heads * head_dim]
    views, unit inner stride) into their pages (values transposed: dimension-major
    within a page).  ``tiles`` (int32 [n, 2]: first flat token and count <= 64 of
    runs of tokens of one sequence) lets prompt values be written a tile at a time."""
    _need_cuda(k, v, tok_pos, tok_seq, block_table, kv_pages)
    for t, name in ((tok_pos, "tok_pos"), (tok_seq, "tok_seq"), (block_table, "block_table")):
        _i32(t, name)
    if k.dtype != kv_pages.dtype or v.dtype != kv_pages.dtype:
        raise KernelError("keys, values and the cache must share a dtype")
    if k.stride(1) != 1 or v.stride(1) != 1:
        raise KernelError("keys and values must have unit inner stride")
    _check(library().mu_kv_append(
        _ptr(k), k.stride(0), _ptr(v), v.stride(0), _ptr(tok_pos), _ptr(tok_seq),
        _ptr(block_table), block_table.shape[1], page_tokens, k.shape[0], n_kv_heads, head_dim,
        _ptr(kv_pages), _is_bf16(kv_pages), _ptr(tiles), tiles.shape[0] if tiles is not None else 0, _stream()),
        ("kv_append(head_dim={})", head_dim))


def attention(q: torch.Tensor, out: torch.Tensor, kv_pages: torch.Tensor, block_table: torch.Tensor,
              page_tokens: int, tok_pos, tok_seq, n_heads: int, n_kv_heads: int, head_dim: int,
              scale: float, window: int = 0, n_splits: int = 1, split_keys: int = 0,
              part_o: Optional[torch.Tensor] = None, part_ml: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Attention of each query token ([T, n_heads * head_dim] view) over the
    cached keys first..its position; writes ``out`` [T, n_heads * head_dim]."""
    _need_cuda(q, out, kv_pages, block_table, tok_pos, tok_seq, part_o, part_ml)
    for t, name in ((tok_pos, "tok_pos"), (tok_seq, "tok_seq"), (block_table, "block_table")):
        _i32(t, name)
    if q.dtype != kv_pages.dtype or out.dtype != kv_pages.dtype:
        raise KernelError("queries, output and the cache must share a dtype")
    if q.stride(1) != 1 or out.stride(1) != 1:
        raise KernelError("queries and output must have unit inner stride")
    n_tokens = q.shape[0]
    if n_splits > 1:
        need_o, need_ml = n_tokens * n_heads * n_splits * head_dim, n_tokens * n_heads * n_splits * 2
        if (part_o is None or part_ml is None or part_o.numel() < need_o or part_ml.numel() < need_ml
                or part_o.dtype != torch.float32 or part_ml.dtype != torch.float32):
            raise KernelError("split attention needs float32 scratch for its partial results")
    _check(library().mu_attention(
        _ptr(q), q.stride(0), _ptr(out), out.stride(0), _ptr(kv_pages), _ptr(block_table),
        block_table.shape[1], page_tokens, _ptr(tok_pos), _ptr(tok_seq), n_tokens,
        n_heads, n_kv_heads, head_dim, float(scale), int(window), int(n_splits), int(split_keys),
        _ptr(part_o), _ptr(part_ml), _is_bf16(kv_pages), _stream()),
        ("attention(heads={}/{}, head_dim={})", n_heads, n_kv_heads, head_dim), launches=2 if n_splits > 1 else 1)
    return out


# -------------------------------------------------------------------- sampling
def _status_args(status_to: Optional[torch.Tensor], device):
    if status_to is None:
        return None, None
    _i32(status_to, "status_to")
    if not status_to.is_cuda or status_to.numel() != 1:
        raise KernelError("status_to must be one int32 word on the device")
    return _ptr(status_word(device)), _ptr(status_to)


def argmax(logits: torch.Tensor, out: Optional[torch.Tensor] = None, feed=None,
           status_to: Optional[torch.Tensor] = None) -> torch.Tensor:
    """First maximum of each row.  ``feed`` = (token_ids, tok_pos, last_pos): the
    tokens also become the next single-token step's inputs and the positions
    (if not None) move on by one (what ``advance`` does, without its launch).
    ``status_to``: a device word that receives the kernels' status word, so
    that one copy brings tokens and status to the host."""
    _need_cuda(logits, out)
    if logits.dtype != torch.float32 or logits.dim() != 2 or logits.stride(1) != 1:
        raise KernelError("logits must be float32 [rows, vocab] with unit inner stride")
    n, vocab = logits.shape
    if out is None:
        out = torch.empty((n,), dtype=torch.int32, device=logits.device)
    ws = zeroed_workspace("argmax", logits.device, 2 * n * 8)
    ids, pos, last = feed if feed is not None else (None, None, 0)
    _check(library().mu_argmax(_ptr(logits), logits.stride(0), n, vocab, _ptr(out), _ptr(ws), _ptr(ids), _ptr(pos),
                               int(last), *_status_args(status_to, logits.device), _stream()), "argmax")
    return out


def sample(logits: torch.Tensor, temperature: float, top_k: int, seed: int,
           request_ids: Optional[torch.Tensor], draw_index: torch.Tensor,
           out: Optional[torch.Tensor] = None, feed=None, status_to: Optional[torch.Tensor] = None) -> torch.Tensor:
    """One token per row by temperature / top-k; ``draw_index`` (int32 per row)
    counts the draws of each request and is advanced by one.  ``feed`` and
    ``status_to`` as for ``argmax``."""
    _need_cuda(logits, request_ids, draw_index, out)
    if logits.dtype != torch.float32 or logits.dim() != 2 or logits.stride(1) != 1:
        raise KernelError("logits must be float32 [rows, vocab] with unit inner stride")
    if request_ids is not None and request_ids.dtype != torch.int64:
        raise KernelError("request_ids must be int64")
    _i32(draw_index, "draw_index")
    n, vocab = logits.shape
    if out is None:
        out = torch.empty((n,), dtype=torch.int32, device=logits.device)
    _check(library().mu_sample(_ptr(logits), logits.stride(0), n, vocab, float(temperature), int(top_k),
                               int(seed) & ((1 << 64) - 1), _ptr(request_ids), _ptr(draw_index), _ptr(out),
                               _ptr(feed[0]) if feed else None, _ptr(feed[1]) if feed else None,
                               int(feed[2]) if feed else 0, *_status_args(status_to, logits.device), _stream()),
           "sample")
    return out


class NormedInput:
    """The LayerNorm of (rows of) a float32 matrix that has not been computed
    yet: a product kernel that can make it on the fly takes this instead of a
    tensor; anything else calls ``materialize``."""

    def __init__(self, x: torch.Tensor, gamma: torch.Tensor, beta: Optional[torch.Tensor], eps: float,
                 out_dtype: torch.dtype, rows: Optional[torch.Tensor] = None):
        self.x, self.gamma, self.beta, self.eps, self.out_dtype, self.rows = x, gamma, beta, eps, out_dtype, rows
        self._value = None

    @property
    def n_rows(self) -> int:
        return self.rows.numel() if self.rows is not None else self.x.shape[0]

    def materialize(self) -> torch.Tensor:
        if self._value is None:
            self._value = layernorm(self.x, self.gamma, self.beta, self.eps, self.out_dtype, rows=self.rows)
        return self._value

    def materialize_copy(self) -> torch.Tensor:
        """The norm computed for an onlooker; what a product does with this input stays as it was."""
        return layernorm(self.x, self.gamma, self.beta, self.eps, self.out_dtype, rows=self.rows)


def gemm_skinny_ln(x: NormedInput, w: torch.Tensor, bias, act, residual, out, out_dtype) -> torch.Tensor:
    """act(LayerNorm(x) @ w^T + bias) + residual with the norm made inside the product kernel."""
    _need_cuda(x.x, w, bias, residual, out, x.rows)
    m, k, n = x.n_rows, x.x.shape[1], w.shape[0]
    if out is None:
        out = torch.empty((m, n), dtype=out_dtype or w.dtype, device=w.device)
    if bias is not None and (bias.dtype != torch.float32 or bias.numel() != n):
        raise KernelError("gemm bias must be float32 of length n")
    if residual is not None and (residual.dtype != torch.float32 or residual.shape != (m, n)):
        raise KernelError("gemm residual must be float32 [m, n]")
    _check(library().mu_gemm_skinny_ln(
        _ptr(x.x), x.x.stride(0), _ptr(x.rows), _ptr(x.gamma), _ptr(x.beta), float(x.eps), _ptr(w), _ptr(bias),
        _ptr(residual), _ptr(out), m, n, k, w.stride(0), out.stride(0),
        residual.stride(0) if residual is not None else 0, ACT_CODES[act], _is_bf16(out), _stream()),
        ("gemm_skinny_ln({}x{}x{})", m, n, k))
    return out


def _stream_kernel(m: int, n: int, k: int, ldw: int, with_norm: bool, device) -> bool:
    """Whether a product of up to 16 rows goes to ``mu_gemm_stream``: very many output columns (an output head:
    what the few-rows kernel would run as blocks of 128 columns each), weight rows one after another, and a k
    short enough for two tiles of 64 weight rows to share an SM's shared memory."""
    return (m <= 16 and n >= 256 * sm_count(device)
            and bool(library().mu_gemm_stream_fits(int(m), int(k), int(ldw), 1 if with_norm else 0)))


def gemm_stream(x, w: torch.Tensor, bias=None, act=None, out=None, out_dtype=None) -> torch.Tensor:
    """act(x @ w^T + bias) for up to 16 rows and very many output columns, the weights streamed through shared
    memory by bulk copies.  ``x``: bfloat16 [m, k], or a ``NormedInput`` (the norm is made inside the kernel)."""
    normed = isinstance(x, NormedInput)
    if normed:
        _need_cuda(x.x, w, bias, out, x.rows)
        m, k = x.n_rows, x.x.shape[1]
    else:
        _need_cuda(x, w, bias, out)
        m, k = x.shape
    n = w.shape[0]
    if w.dtype != torch.bfloat16 or w.shape[1] != k or w.stride(1) != 1:
        raise KernelError("gemm_stream needs bfloat16 weights [n, k] with unit stride along k")
    if out is None:
        out = torch.empty((m, n), dtype=out_dtype or w.dtype, device=w.device)
    if bias is not None and (bias.dtype != torch.float32 or bias.numel() != n):
        raise KernelError("gemm bias must be float32 of length n")
    _check(library().mu_gemm_stream(
        None if normed else _ptr(x), 0 if normed else x.stride(0),
        _ptr(x.x) if normed else None, x.x.stride(0) if normed else 0, _ptr(x.rows) if normed else None,
        _ptr(x.gamma) if normed else None, _ptr(x.beta) if normed else None, float(x.eps) if normed else 0.0,
        _ptr(w), _ptr(bias), _ptr(out), m, n, k, w.stride(0), out.stride(0), ACT_CODES[act], _is_bf16(out),
        _ptr(status_word(w.device)), _stream()), ("gemm_stream({}x{}x{})", m, n, k))
    return out


SKINNY_LN_SMEM = 160 * 1024          # the limit of mu_gemm_skinny_ln (gemm_skinny.cuh)

_sm_counts = {}


def sm_count(device) -> int:
    n = _sm_counts.get(device)
    if n is None:
        n = _sm_counts[device] = torch.cuda.get_device_properties(device).multi_processor_count
    return n


def decode_ok(head_dim: int) -> bool:
    """Whether the one-launch single-token attention kernels take this head size
    (multiples of 16 up to 256: their key rows are read in 16-byte pieces); other
    sizes append first and then run the general kernel."""
    return head_dim % 16 == 0 and 16 <= head_dim <= 256


def decode_tc_ok(q, k_new, v_new, kv_pages, page_tokens: int, n_heads: int, n_kv_heads: int,
                 head_dim: int) -> bool:
    """Whether the tensor-core single-token attention takes this case (else the
    CUDA-core kernel does): bfloat16, head sizes 32, 64, 96 and 128, at most 16 query
    heads per kv head, 16-byte aligned rows.  MU_B200_ATT_TC=0 switches it off."""
    if not ATT_TC:
        return False
    if kv_pages.dtype != torch.bfloat16 or page_tokens != 64 or head_dim not in (32, 64, 96, 128):
        return False
    if n_heads % n_kv_heads != 0 or n_heads // n_kv_heads > 16:
        return False
    for t in (q, k_new, v_new):
        if t is not None and (t.stride(0) % 8 != 0 or t.data_ptr() % 16 != 0):
            return False
    return True


def decode_block_shape(blocks: int, sms: int) -> int:
    """The shape of the tensor-core single-token attention kernel's blocks for this many (sequence, kv head)
    pairs, as the code ``mu_attention_decode_tc`` takes.  No more blocks than SMs: large ones (6), all pages of
    a sequence in flight at once; up to twice as many: three groups of two warps, two blocks an SM (3); more:
    small ones, three an SM (2; the large ones would run in waves).  Very few: four (24) or two (12) large
    blocks share a sequence's pages as a cluster, while the clusters fill two thirds or half of the SMs at
    most (a cluster is placed within one part of the chip, so a fuller grid of clusters runs in waves)."""
    if 6 * blocks <= sms:
        return 24
    if 4 * blocks <= sms:
        return 12
    if blocks <= sms:
        return 6
    return 3 if blocks <= 2 * sms else 2


def attention_decode(q: torch.Tensor, k_new: Optional[torch.Tensor], v_new: Optional[torch.Tensor],
                     out: torch.Tensor, kv_pages: torch.Tensor, block_table: torch.Tensor, page_tokens: int,
                     tok_pos, tok_seq, n_heads: int, n_kv_heads: int, head_dim: int, scale: float,
                     window: int, n_splits: int, warps: int = 0) -> torch.Tensor:
    """Single-token attention, one launch: appends ``k_new`` / ``v_new`` (if
    given), attends page by page, merges in shared memory.  ``n_splits``: how
    many warps share a sequence's pages (its page count is a good choice; at most
    16 are used).  ``tok_seq`` None: token t is sequence t.  ``warps``: the shape of a
    block (tensor-core kernel: 2, 3 or 6 groups of warps, 12 or 24 for six groups in
    each of two or four blocks that share a sequence; CUDA-core kernel: an upper bound
    on its warps); 0: chosen here."""
    _need_cuda(q, k_new, v_new, out, kv_pages, block_table, tok_pos, tok_seq)
    for t, name in ((tok_pos, "tok_pos"), (tok_seq, "tok_seq"), (block_table, "block_table")):
        _i32(t, name)
    n_tokens = q.shape[0]
    if decode_tc_ok(q, k_new, v_new, kv_pages, page_tokens, n_heads, n_kv_heads, head_dim):
        if not warps:
            warps = decode_block_shape(n_tokens * n_kv_heads, sm_count(q.device))
        _check(library().mu_attention_decode_tc(
            _ptr(q), q.stride(0), _ptr(k_new), k_new.stride(0) if k_new is not None else 0, _ptr(v_new),
            v_new.stride(0) if v_new is not None else 0, _ptr(out), out.stride(0), _ptr(kv_pages),
            _ptr(block_table), block_table.shape[1], page_tokens, _ptr(tok_pos), _ptr(tok_seq), n_tokens,
            n_heads, n_kv_heads, head_dim, float(scale), int(window), int(warps),
            _ptr(status_word(q.device)), _stream()),
            ("attention_decode_tc(heads={}/{}, head_dim={})", n_heads, n_kv_heads, head_dim))
        return out
    _check(library().mu_attention_decode(
        _ptr(q), q.stride(0), _ptr(k_new), k_new.stride(0) if k_new is not None else 0, _ptr(v_new),
        v_new.stride(0) if v_new is not None else 0, _ptr(out), out.stride(0), _ptr(kv_pages),
        _ptr(block_table), block_table.shape[1], page_tokens, _ptr(tok_pos), _ptr(tok_seq), n_tokens,
        n_heads, n_kv_heads, head_dim, float(scale), int(window), int(n_splits), int(warps), _is_bf16(kv_pages),
        _stream()),
        ("attention_decode(heads={}/{}, head_dim={})", n_heads, n_kv_heads, head_dim))
    return out


def prefill_ok(q: torch.Tensor, head_dim: int, page_tokens: int) -> bool:
    """Whether the tensor-core prompt attention takes this case."""
    return (q.dtype == torch.bfloat16 and page_tokens == 64 and head_dim % 16 == 0 and 16 <= head_dim <= 128
            and q.stride(0) % 8 == 0 and q.data_ptr() % 16 == 0)


def attention_prefill(q: torch.Tensor, out: torch.Tensor, kv_pages: torch.Tensor, block_table: torch.Tensor,
                      page_tokens: int, tok_pos, tok_seq, tiles: torch.Tensor, n_heads: int, n_kv_heads: int,
                      head_dim: int, scale: float, window: int = 0) -> torch.Tensor:
    """Flash-style causal attention of prompt tokens on tensor cores.  ``tiles``
    int32 [n, 2]: first flat query index and query count (<= 64) of each tile;
    the kernel's blocks take them in this order, so the tiles with the most keys
    should come first."""
    _need_cuda(q, out, kv_pages, block_table, tok_pos, tok_seq, tiles)
    for t, name in ((tok_pos, "tok_pos"), (tok_seq, "tok_seq"), (block_table, "block_table"), (tiles, "tiles")):
        _i32(t, name)
    counter = zeroed_workspace("attention_prefill_items", q.device, 8)
    _check(library().mu_attention_prefill(
        _ptr(q), q.stride(0), _ptr(out), out.stride(0), _ptr(kv_pages), _ptr(block_table), block_table.shape[1],
        page_tokens, _ptr(tok_pos), _ptr(tok_seq), _ptr(tiles), tiles.shape[0], n_heads, n_kv_heads, head_dim,
        float(scale), int(window), _ptr(counter), _stream()), ("attention_prefill(heads={}/{}, head_dim={})", n_heads, n_kv_heads, head_dim))
    return out


def prefill_tc_ok(q: torch.Tensor, out: torch.Tensor, head_dim: int, page_tokens: int) -> bool:
    """Whether the tcgen05 prompt attention takes this case: bfloat16, head size
    64, pages of 64, query and output rows 16-byte aligned.  MU_B200_PREFILL_TC=0
    switches it off (the mma.sync kernel then runs)."""
    if not PREFILL_TC:
        return False
    return (q.dtype == torch.bfloat16 and head_dim == 64 and page_tokens == 64 and q.stride(0) % 8 == 0
            and q.data_ptr() % 16 == 0 and out.stride(0) % 8 == 0 and out.data_ptr() % 16 == 0)


def attention_prefill_tc(q: torch.Tensor, out: torch.Tensor, kv_pages: torch.Tensor, block_table: torch.Tensor,
                         page_tokens: int, tok_pos, tok_seq, tiles: torch.Tensor, n_heads: int, n_kv_heads: int,
                         head_dim: int, scale: float, window: int = 0, k_new: Optional[torch.Tensor] = None,
                         v_new: Optional[torch.Tensor] = None, append_tiles: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Causal attention of prompt tokens on the tcgen05 tensor cores (TMA loads,
    scores and outputs in tensor memory).  ``tiles`` int32 [n, 2]: first flat
    query index and query count (<= 128) of each tile, longest tiles first.
    With ``k_new`` / ``v_new`` the step's keys and values are appended to the
    cache first, in the same call (``append_tiles``: tiles of <= 64 tokens)."""
    _need_cuda(q, out, kv_pages, block_table, tok_pos, tok_seq, tiles, k_new, v_new, append_tiles)
    for t, name in ((tok_pos, "tok_pos"), (tok_seq, "tok_seq"), (block_table, "block_table"), (tiles, "tiles"),
                    (append_tiles, "append_tiles")):
        _i32(t, name)
    if k_new is not None and (k_new.dtype != kv_pages.dtype or v_new is None or v_new.dtype != kv_pages.dtype
                              or k_new.stride(1) != 1 or v_new.stride(1) != 1):
        raise KernelError("keys, values and the cache must share a dtype; unit stride within a row")
    _check(library().mu_attention_prefill_tc(
        _ptr(q), q.stride(0), q.shape[0], _ptr(out), out.stride(0), _ptr(kv_pages), kv_pages.shape[0],
        _ptr(block_table), block_table.shape[1], page_tokens, _ptr(tok_pos), _ptr(tok_seq), _ptr(tiles),
        tiles.shape[0], n_heads, n_kv_heads, head_dim, float(scale), int(window),
        _ptr(k_new), k_new.stride(0) if k_new is not None else 0, _ptr(v_new),
        v_new.stride(0) if v_new is not None else 0, _ptr(append_tiles),
        append_tiles.shape[0] if append_tiles is not None else 0,
        _ptr(status_word(q.device)), _stream()),
        ("attention_prefill_tc(heads={}/{}, head_dim={})", n_heads, n_kv_heads, head_dim),
        launches=2 if k_new is not None else 1)
    return out


_scratch = {}


def scratch(name: str, device, numel: int, dtype) -> torch.Tensor:
    """A device buffer kept per purpose, device and dtype that only ever grows
    (a buffer it outgrows is kept alive: a recorded graph may still point at it)."""
    key = (name, device, dtype)
    buf = _scratch.get(key)
    if buf is None or buf.numel() < numel:
        if buf is not None:
            _retired.append(buf)
        buf = _scratch[key] = torch.empty(max(numel, 1), dtype=dtype, device=device)
    return buf


def _layernorm_gemm_tc(x: "NormedInput", weight, bias, act, residual, out, out_dtype):
    """The norm and the tensor-core product of it from one call into the library
    (two launches), for more than 64 rows of bfloat16; None if the case is not its."""
    m, k = x.n_rows, x.x.shape[1]
    n = weight.shape[0]
    if (m <= 64 or x._value is not None or weight.dtype != torch.bfloat16 or x.out_dtype != torch.bfloat16
            or x.x.dtype != torch.float32 or not x.x.is_contiguous() or weight.dim() != 2 or weight.shape[1] != k
            or weight.stride(1) != 1 or k % 8 != 0 or weight.stride(0) % 8 != 0 or weight.data_ptr() % 16 != 0):
        return None
    if not (x.x.is_cuda and weight.is_cuda and x.gamma.dtype == torch.float32
            and (x.beta is None or x.beta.dtype == torch.float32)):
        return None
    if out is None:
        out = torch.empty((m, n), dtype=out_dtype or torch.bfloat16, device=weight.device)
    elif out.shape != (m, n) or out.stride(1) != 1 or not out.is_cuda:
        raise KernelError("gemm output has the wrong shape, stride or device")
    if bias is not None and (bias.dtype != torch.float32 or bias.numel() != n or not bias.is_cuda):
        raise KernelError("gemm bias must be float32 of length n on the device")
    ldr = 0
    if residual is not None:
        if residual.dtype != torch.float32 or residual.shape != (m, n) or residual.stride(1) != 1 or not residual.is_cuda:
            raise KernelError("gemm residual must be float32 [m, n] on the device")
        ldr = residual.stride(0)
    _i32(x.rows, "rows")
    normed = scratch("layernorm_out", weight.device, m * k, torch.bfloat16)
    _check(library().mu_layernorm_gemm_tc(
        x.x.data_ptr(), _ptr(x.rows), x.gamma.data_ptr(), _ptr(x.beta), float(x.eps), normed.data_ptr(),
        weight.data_ptr(), _ptr(bias), _ptr(residual), out.data_ptr(), m, n, k, weight.stride(0), out.stride(0),
        ldr, ACT_CODES[act], _is_bf16(out), status_word(weight.device).data_ptr(), _stream()),
        ("layernorm_gemm_tc({}x{}x{})", m, n, k), launches=2)
    return out


# ------------------------------------------------------ a whole layer of a prompt step in one call
class PromptLayerArgs(ctypes.Structure):
    """Everything ``mu_prompt_layer`` needs; the layout is ``MuPromptLayerArgs`` of prompt_layer.cu."""
    _fields_ = (
        [(n, _c_p) for n in ("x", "normed", "qkv", "attn", "inner_buf", "tok_pos", "tok_seq", "block_table",
                             "tiles_wide", "tiles", "status", "stream", "kv_pages", "ln1_gamma", "ln1_beta",
                             "qkv_weight", "qkv_bias", "out_weight", "out_bias", "ln2_gamma", "ln2_beta",
                             "up_weight", "up_bias", "down_weight", "down_bias")]
        + [(n, _c_ll) for n in ("n_cache_pages", "ld_qkv_weight", "ld_out_weight", "ld_up_weight", "ld_down_weight")]
        + [(n, _c_f) for n in ("eps1", "eps2", "scale")]
        + [(n, _c_int) for n in ("n_tokens", "hidden", "inner", "n_heads", "n_kv_heads", "head_dim", "window", "act",
                                 "max_pages", "page_tokens", "n_tiles_wide", "n_tiles", "owns_cache")])


_PROMPT_LAUNCHES = ("", "the norm and the q | k | v product", "the cache append and the attention", "the output projection",
                    "the norm and the feed-forward's first product", "the feed-forward's second product")


def prompt_layer(args: PromptLayerArgs) -> None:
    """Issues the launches of one pre-norm layer of a prompt step (eight kernels) from one call."""
    lib = library()
    fn = lib.mu_prompt_layer
    if fn.argtypes is None:
        if lib.mu_prompt_layer_args_size() != ctypes.sizeof(PromptLayerArgs):
            raise KernelError("the layer-call layout of the Python side and of the kernel library differ")
        fn.argtypes, fn.restype = [ctypes.POINTER(PromptLayerArgs)], _c_int
    args.stream = _stream()
    code = fn(ctypes.byref(args))
    if code != 0:
        raise KernelError(f"prompt layer, {_PROMPT_LAUNCHES[min(code // 100, 5)]}: "
                          f"{_ERRORS.get(code % 100, f'error {code % 100}')}")
    global launch_count
    launch_count += 7 + int(bool(args.owns_cache))


# -------------------------------------------------------------------- dispatch
def linear(x: torch.Tensor, weight: torch.Tensor, bias: Optional[torch.Tensor] = None,
           act: Optional[str] = None, residual: Optional[torch.Tensor] = None,
           out: Optional[torch.Tensor] = None, out_dtype: Optional[torch.dtype] = None) -> torch.Tensor:
    """act(x @ weight^T + bias) + residual through the kernel that fits the
    dtype and the shape.  float32 operands always take the CUDA-core kernel.
    ``x`` may be a ``NormedInput``: with few rows and bfloat16 weights the norm is
    made inside the product kernel, otherwise it is computed first."""
    if isinstance(x, NormedInput) and weight.dtype == torch.bfloat16 and _rows_kernel(x.n_rows, *weight.shape):
        x = x.materialize()          # a very wide product: the norm as a launch of its own costs less than it saves
    if isinstance(x, NormedInput):
        k_in = x.x.shape[1]
        # the few-rows kernel keeps the normed rows (8, 16 or 32 of them), gamma and beta in shared memory
        fits = 8 * (1 if x.n_rows <= 8 else 2 if x.n_rows <= 16 else 4) * (k_in + 8) * 2 + 8 * k_in <= SKINNY_LN_SMEM
        if (weight.dtype == torch.bfloat16 and x.out_dtype == torch.bfloat16 and x.n_rows <= 32 and fits
                and k_in % 8 == 0 and weight.stride(0) % 8 == 0 and weight.data_ptr() % 16 == 0
                and x.x.dtype == torch.float32 and x.x.stride(1) == 1):
            if (residual is None and x.x.stride(0) % 4 == 0 and x.x.data_ptr() % 16 == 0
                    and _stream_kernel(x.n_rows, weight.shape[0], k_in, weight.stride(0), True, weight.device)):
                return gemm_stream(x, weight, bias, act, out, out_dtype)      # an output head
            return gemm_skinny_ln(x, weight, bias, act, residual, out, out_dtype)
        fused = _layernorm_gemm_tc(x, weight, bias, act, residual, out, out_dtype)
        if fused is not None:
            return fused
        x = x.materialize()
    # One pass over what the kernels need, then straight to the library (this is the call a prompt
    # step makes a hundred times): the shapes must agree here; alignment, strides and sizes that a
    # kernel cannot take come back from the library as an error code.
    if x.dim() != 2 or weight.dim() != 2:
        raise KernelError(f"gemm shapes do not agree: a {tuple(x.shape)}, w {tuple(weight.shape)}")
    m, k = x.shape
    n, kw = weight.shape
    dtype = x.dtype
    if k != kw or dtype != weight.dtype or x.stride(1) != 1 or weight.stride(1) != 1:
        raise KernelError(f"gemm operands do not agree: a {tuple(x.shape)} {dtype}, w {tuple(weight.shape)} "
                          f"{weight.dtype}, unit stride along k needed")
    if not (x.is_cuda and weight.is_cuda):
        raise KernelError("math_utils_b200 kernels run on CUDA tensors only")
    if out is None:
        out = torch.empty((m, n), dtype=out_dtype or dtype, device=x.device)
    elif out.shape != (m, n) or out.stride(1) != 1 or not out.is_cuda:
        raise KernelError("gemm output has the wrong shape, stride or device")
    if bias is not None and (bias.dtype != torch.float32 or bias.numel() != n or not bias.is_cuda):
        raise KernelError("gemm bias must be float32 of length n on the device")
    ldr = 0
    if residual is not None:
        if residual.dtype != torch.float32 or residual.shape != (m, n) or residual.stride(1) != 1 or not residual.is_cuda:
            raise KernelError("gemm residual must be float32 [m, n] on the device")
        ldr = residual.stride(0)
    lda, ldw = x.stride(0), weight.stride(0)
    pa, pw = x.data_ptr(), weight.data_ptr()
    pb = None if bias is None else bias.data_ptr()
    pr = None if residual is None else residual.data_ptr()
    lib = library()
    code = ACT_CODES[act]
    tensor_cores = (dtype == torch.bfloat16 and k % 8 == 0 and lda % 8 == 0 and ldw % 8 == 0
                    and pa % 16 == 0 and pw % 16 == 0)
    # 33 to 64 rows, and fewer where the weights are very many (the output head): the tcgen05 kernel for few
    # rows (weights as the wide operand, k cut over a cluster); up to 32 rows otherwise the mma.sync kernel
    # that streams weights straight into fragments; more than 64 rows the large tcgen05 kernel
    if tensor_cores and _rows_kernel(m, n, k):
        _check(lib.mu_gemm_rows(pa, pw, pb, pr, out.data_ptr(), m, n, k, lda, ldw, out.stride(0), ldr, code,
                                _is_bf16(out), 0, status_word(x.device).data_ptr(), _stream()),
               ("gemm_rows({}x{}x{})", m, n, k))
    elif tensor_cores and m <= 32:
        _check(lib.mu_gemm_skinny(pa, pw, pb, pr, out.data_ptr(), m, n, k, lda, ldw, out.stride(0), ldr, code,
                                  _is_bf16(out), _stream()), ("gemm_skinny({}x{}x{})", m, n, k))
    elif tensor_cores:
        _check(lib.mu_gemm_tc(pa, pw, pb, pr, out.data_ptr(), m, n, k, lda, ldw, out.stride(0), ldr, code,
                              _is_bf16(out), 0, -1, status_word(x.device).data_ptr(), _stream()),
               ("gemm_tc({}x{}x{})", m, n, k))
    else:
        _check(lib.mu_gemm_simt(pa, pw, pb, pr, out.data_ptr(), m, n, k, lda, ldw, out.stride(0), ldr, code,
                                _is_bf16(x), _is_bf16(out), _stream()), ("gemm_simt({}x{}x{})", m, n, k))
    return out
