"""Tensor-level wrappers of the CUDA launchers.

Each function checks devices, dtypes, shapes and contiguity on the host, then
calls the C entry point on the current CUDA stream.  Outputs are allocated by the
caller or here with ``torch.empty`` (the caching allocator, so that a step can be
captured in a CUDA graph).  Matrix products run on this library's own kernels:
float32 on FFMA kernels, bfloat16 on the mma.sync small-M kernel (up to 64 rows), the
cluster split-K tcgen05 kernel (9 to 128 rows) and the tcgen05/TMA GEMMs (whole
prompts; sizes they refuse go through the small-M kernel 64 rows at a time).  A library
product (cuBLAS through ``torch.matmul``) is used only when ``QNN_GEMM=cublas`` asks
for it, for comparisons.
"""
from __future__ import annotations

import ctypes
import os
from typing import Optional, Tuple

import torch

from . import lib as _lib

F32, BF16 = 0, 1
EPI_NONE, EPI_SOFTCAP, EPI_GATED = 0, 1, 2
EPI_ACT = 5                  # act(x w^T) without a gate; the launchers get it as epilogue "none" with the code below
ACT_ALONE = 16               # added to an activation's code: the product's epilogue applies it to the plain product
ACT_CODES = {"gelu_tanh": 0, "silu": 1, "relu2": 2}
ACT_XIELU = 3                # an activation with two constants of its own (``act_consts``); never a gate
SKINNY_MAX_ROWS = 64


def dt_code(t: torch.Tensor) -> int:
    if t.dtype == torch.float32:
        return F32
    if t.dtype == torch.bfloat16:
        return BF16
    raise TypeError(f"unsupported dtype {t.dtype} (float32 or bfloat16 expected)")


def _p(t: Optional[torch.Tensor]):
    return None if t is None else ctypes.c_void_p(t.data_ptr())


_raw_stream = getattr(torch._C, "_cuda_getCurrentRawStream", None)
_raw_device = getattr(torch._C, "_cuda_getDevice", None)


def _stream():
    """The current device's current stream as a handle for the launchers.  Asked for at every launch, so by the
    two plain C calls where this torch has them (``torch.cuda.current_stream()`` walks a dozen Python frames, a
    third of the host time of a short step)."""
    if _raw_stream is not None and _raw_device is not None:
        return ctypes.c_void_p(_raw_stream(_raw_device()))
    return ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)


def _req(t: torch.Tensor, name: str, dtype=None, dim=None) -> None:
    if not t.is_cuda:
        raise _lib.KernelError(f"{name} must be a CUDA tensor: quicknn_b200 has no CPU path")
    if not t.is_contiguous():
        raise ValueError(f"{name} must be contiguous")
    if dtype is not None and t.dtype != dtype:
        raise TypeError(f"{name} must be {dtype}, got {t.dtype}")
    if dim is not None and t.dim() != dim:
        raise ValueError(f"{name} must have {dim} dimensions, got {tuple(t.shape)}")


def embed(tokens: torch.Tensor, table: torch.Tensor, scale: float, out: Optional[torch.Tensor] = None):
    _req(tokens, "tokens", torch.int32, 1)
    _req(table, "table", None, 2)
    T, (V, H) = tokens.numel(), table.shape
    if out is None:
        out = torch.empty((T, H), dtype=torch.float32, device=tokens.device)
    _req(out, "out", torch.float32, 2)
    L = _lib.load()
    _lib.check(L.qnn_embed(_p(tokens), _p(table), dt_code(table), float(scale), _p(out), T, H, V, _stream()),
               "embed")
    return out


def embed_rmsnorm(tokens: torch.Tensor, table: torch.Tensor, scale: float, weight: torch.Tensor, eps: float,
                  unit_offset: bool, out_dtype: torch.dtype):
    """``embed`` and the first norm of what it gives in one kernel: (rows [T, H] float32, rmsnorm(rows))."""
    _req(tokens, "tokens", torch.int32, 1)
    _req(table, "table", None, 2)
    _req(weight, "weight", None, 1)
    T, (V, H) = tokens.numel(), table.shape
    if weight.numel() != H:
        raise ValueError(f"norm weight has {weight.numel()} elements for width {H}")
    out = torch.empty((T, H), dtype=torch.float32, device=tokens.device)
    normed = torch.empty((T, H), dtype=out_dtype, device=tokens.device)
    _lib.check(_lib.load().qnn_embed_rmsnorm(_p(tokens), _p(table), dt_code(table), float(scale), _p(out), _p(weight),
                                             dt_code(weight), float(eps), int(unit_offset), _p(normed), dt_code(normed),
                                             T, H, V, _stream()), "embed_rmsnorm")
    return out, normed


def rmsnorm(x: torch.Tensor, weight: torch.Tensor, eps: float, unit_offset: bool, out_dtype: torch.dtype,
            out: Optional[torch.Tensor] = None):
    _req(x, "x", None, 2)
    _req(weight, "weight", None, 1)
    T, H = x.shape
    if weight.numel() != H:
        raise ValueError(f"norm weight has {weight.numel()} elements for width {H}")
    if out is None:
        out = torch.empty((T, H), dtype=out_dtype, device=x.device)
    _req(out, "out", out_dtype, 2)
    L = _lib.load()
    _lib.check(L.qnn_rmsnorm(_p(x), dt_code(x), _p(weight), dt_code(weight), float(eps), int(unit_offset),
                             _p(out), dt_code(out), T, H, _stream()), "rmsnorm")
    return out


def add_rmsnorm(resid: torch.Tensor, y: torch.Tensor, w_post: torch.Tensor, eps_post: float, unit_post: bool,
                w_next: Optional[torch.Tensor] = None, eps_next: float = 0.0, unit_next: bool = False,
                out_dtype: Optional[torch.dtype] = None):
    """resid += rmsnorm(y, w_post); returns rmsnorm(resid, w_next) when w_next is given."""
    _req(resid, "resid", torch.float32, 2)
    _req(y, "y", None, 2)
    T, H = resid.shape
    if tuple(y.shape) != (T, H) or w_post.numel() != H or (w_next is not None and w_next.numel() != H):
        raise ValueError("add_rmsnorm: shapes do not agree")
    out = None
    if w_next is not None:
        out = torch.empty((T, H), dtype=out_dtype, device=resid.device)
    L = _lib.load()
    _lib.check(L.qnn_add_rmsnorm(_p(resid), _p(y), dt_code(y), _p(w_post), dt_code(w_post), float(eps_post),
                                 int(unit_post), _p(w_next), dt_code(w_next) if w_next is not None else 0,
                                 float(eps_next), int(unit_next), _p(out), dt_code(out) if out is not None else 0,
                                 T, H, _stream()), "add_rmsnorm")
    return out


def add_(resid: torch.Tensor, y: torch.Tensor):
    _req(resid, "resid", torch.float32)
    _req(y, "y")
    if resid.numel() != y.numel():
        raise ValueError("add_: sizes differ")
    L = _lib.load()
    _lib.check(L.qnn_add(_p(resid), _p(y), dt_code(y), resid.numel(), _stream()), "add")
    return resid


def gated_act(gu: torch.Tensor, activation: str):
    _req(gu, "gate_up", None, 2)
    T, I2 = gu.shape
    out = torch.empty((T, I2 // 2), dtype=gu.dtype, device=gu.device)
    L = _lib.load()
    _lib.check(L.qnn_gated_act(_p(gu), _p(out), dt_code(gu), T, I2 // 2, ACT_CODES[activation], _stream()),
               "gated_act")
    return out


def softcap(x: torch.Tensor, cap: Optional[float]):
    _req(x, "x")
    out = torch.empty(x.shape, dtype=torch.float32, device=x.device)
    L = _lib.load()
    _lib.check(L.qnn_softcap(_p(x), dt_code(x), _p(out), float(cap or 0.0), x.numel(), _stream()), "softcap")
    return out


def gather_rows(src: torch.Tensor, rows: torch.Tensor, out_dtype: torch.dtype):
    _req(src, "src", None, 2)
    _req(rows, "rows", torch.int32, 1)
    out = torch.empty((rows.numel(), src.shape[1]), dtype=out_dtype, device=src.device)
    L = _lib.load()
    _lib.check(L.qnn_gather_rows(_p(src), dt_code(src), _p(rows), _p(out), dt_code(out), rows.numel(),
                                 src.shape[1], _stream()), "gather_rows")
    return out


def cast(x: torch.Tensor, dtype: torch.dtype):
    if x.dtype == dtype:
        return x
    _req(x, "x")
    out = torch.empty(x.shape, dtype=dtype, device=x.device)
    L = _lib.load()
    _lib.check(L.qnn_cast(_p(x), dt_code(x), _p(out), dt_code(out), x.numel(), _stream()), "cast")
    return out


def check_finite(x: torch.Tensor, flag: Optional[torch.Tensor] = None):
    """Set ``flag`` (default: this device's non-finite word, read by ``raise_on_status``) if
    ``x`` holds NaN or Inf."""
    _req(x, "x", torch.float32)
    if flag is None:
        flag = finite_flag(x.device)
    _req(flag, "flag", torch.int32)
    L = _lib.load()
    _lib.check(L.qnn_check_finite(_p(x), x.numel(), _p(flag), _stream()), "check_finite")


def rope_cache_write(qkv: torch.Tensor, n_heads: int, n_kv: int, head_dim: int, rot_dim: int,
                     inv_freq: torch.Tensor, tok_pos: torch.Tensor, tok_slot: torch.Tensor,
                     k_pool: Optional[torch.Tensor], v_pool: Optional[torch.Tensor],
                     page_table: Optional[torch.Tensor], page_size: int, ring: int,
                     slot_len: Optional[torch.Tensor], write_cache: bool):
    _req(qkv, "qkv", None, 2)
    T = qkv.shape[0]
    if qkv.shape[1] != (n_heads + 2 * n_kv) * head_dim:
        raise ValueError("rope_cache_write: qkv width does not match the head counts")
    _req(inv_freq, "inv_freq", torch.float32, 1)
    if inv_freq.numel() != rot_dim // 2:
        raise ValueError("rope_cache_write: inv_freq has the wrong length")
    _req(tok_pos, "tok_pos", torch.int32, 1)
    _req(tok_slot, "tok_slot", torch.int32, 1)
    if write_cache:
        for n, t in (("k_pool", k_pool), ("v_pool", v_pool)):
            if t is None and n == "v_pool":            # a line that keeps keys only
                continue
            _req(t, n, qkv.dtype, 4)
            if tuple(t.shape[1:]) != (n_kv, page_size, head_dim):
                raise ValueError(f"{n} has shape {tuple(t.shape)}, expected [pages, {n_kv}, {page_size}, {head_dim}]")
        _req(page_table, "page_table", torch.int32, 2)
        _req(slot_len, "slot_len", torch.int32, 1)
    L = _lib.load()
    _lib.check(L.qnn_rope_cache_write(
        _p(qkv), dt_code(qkv), T, n_heads, n_kv, head_dim, rot_dim, _p(inv_freq), _p(tok_pos), _p(tok_slot),
        _p(k_pool), _p(v_pool), _p(page_table), page_table.shape[1] if page_table is not None else 0,
        page_size, ring, _p(slot_len), int(write_cache), _stream()), "rope_cache_write")


_no_freq = {}


def cache_append(qkv: torch.Tensor, n_heads: int, n_kv: int, head_dim: int, tok_pos: torch.Tensor,
                 tok_slot: torch.Tensor, line) -> None:
    """Append the keys and values of the packed q|k|v rows to a cache line as they are (no rotation).
    ``line`` is a cache line view (k, v, page_table, page_size, ring, slot_len)."""
    f = _no_freq.get(qkv.device)
    if f is None:
        f = _no_freq[qkv.device] = torch.zeros(0, dtype=torch.float32, device=qkv.device)
    rope_cache_write(qkv, n_heads, n_kv, head_dim, 0, f, tok_pos, tok_slot, line.k, line.v if line.has_values else None,
                     line.page_table, line.page_size, line.ring, line.slot_len, True)


FUSE_ROPE = os.environ.get("QNN_FUSE_ROPE", "1") != "0"


def qkv_rope_cache_fusable(x: torch.Tensor, w: torch.Tensor, head_dim: int, rot_dim: int) -> bool:
    """Whether qkv_rope_cache takes this product: bfloat16 on both sides, few rows, a matrix
    that the small-M kernel would multiply anyway, a rotation over the whole head."""
    M, K = x.shape
    if x.dtype != torch.bfloat16 or w.dtype != torch.bfloat16 or not FUSE_ROPE:
        return False
    if M > SKINNY_MAX_ROWS or K % 8 or head_dim % 16 or rot_dim != head_dim:
        return False
    return not _takes_skinny_tcgen05(M, w.shape[0], K)


def qkv_rope_cache(x: torch.Tensor, w: torch.Tensor, n_heads: int, n_kv: int, head_dim: int,
                   inv_freq: torch.Tensor, tok_pos: torch.Tensor, tok_slot: torch.Tensor,
                   k_pool: Optional[torch.Tensor], v_pool: Optional[torch.Tensor],
                   page_table: Optional[torch.Tensor], page_size: int, ring: int,
                   slot_len: Optional[torch.Tensor], write_cache: bool) -> torch.Tensor:
    """linear(x, w) followed by rope_cache_write(...) as one kernel: the stacked q|k|v product
    with Q and K rotated and K, V appended to the cache in its epilogue.  Returns qkv."""
    _req(x, "x", torch.bfloat16, 2)
    _req(w, "w", torch.bfloat16, 2)
    M, K = x.shape
    N = (n_heads + 2 * n_kv) * head_dim
    if tuple(w.shape) != (N, K):
        raise ValueError(f"qkv_rope_cache: w is {tuple(w.shape)}, expected {(N, K)}")
    _req(inv_freq, "inv_freq", torch.float32, 1)
    if inv_freq.numel() != head_dim // 2:
        raise ValueError("qkv_rope_cache: inv_freq has the wrong length")
    _req(tok_pos, "tok_pos", torch.int32, 1)
    _req(tok_slot, "tok_slot", torch.int32, 1)
    if tok_pos.numel() < M or tok_slot.numel() < M:
        raise ValueError("qkv_rope_cache: fewer positions than rows")
    if write_cache:
        for n, t in (("k_pool", k_pool), ("v_pool", v_pool)):
            _req(t, n, torch.bfloat16, 4)
            if tuple(t.shape[1:]) != (n_kv, page_size, head_dim):
                raise ValueError(f"{n} has shape {tuple(t.shape)}, expected [pages, {n_kv}, {page_size}, {head_dim}]")
        _req(page_table, "page_table", torch.int32, 2)
        _req(slot_len, "slot_len", torch.int32, 1)
    qkv = torch.empty((M, N), dtype=torch.bfloat16, device=x.device)
    L = _lib.load()
    _lib.check(L.qnn_skinny_qkv_rope(
        _p(x), _p(w), _p(qkv), M, K, n_heads, n_kv, head_dim, _p(inv_freq), _p(tok_pos), _p(tok_slot),
        _p(k_pool), _p(v_pool), _p(page_table), page_table.shape[1] if page_table is not None else 0,
        page_size, ring, _p(slot_len), int(write_cache), _stream()), "skinny_qkv_rope")
    return qkv


_status = {}


def status_words(device) -> torch.Tensor:
    """Two int32 words per device that kernels set and the host reads together: [0] the status of
    the tcgen05 kernels' bounded waits (1 loads, 2 tensor-core issue, 4 epilogue), [1] the
    non-finite flag of ``check_finite``."""
    device = torch.device(device)
    t = _status.get(device)
    if t is None:
        t = torch.zeros(2, dtype=torch.int32, device=device)
        _status[device] = t
    return t


def _status_word(device) -> torch.Tensor:
    return status_words(device)[0:1]


def finite_flag(device) -> torch.Tensor:
    return status_words(device)[1:2]


def wait_status_message(v: int) -> str:
    return (f"a tcgen05 kernel gave up waiting (status {v}: 1 loads, 2 tensor-core issue, 4 epilogue); "
            f"its result is not valid")


def raise_on_status(device) -> None:
    """Read both words (one 8-byte copy; it synchronises, so call it where the host waits anyway)
    and raise if a bounded wait ran out or a checked tensor held NaN or Inf since the last call."""
    t = _status.get(torch.device(device))
    if t is None:
        return
    wait, bad = t.tolist()
    if wait or bad:
        t.zero_()
    if wait:
        raise _lib.KernelError(wait_status_message(wait))
    if bad:
        raise _lib.NonFiniteLogits("the model produced non-finite logits")


check_gemm_status = raise_on_status


GEMM_2CTA = os.environ.get("QNN_GEMM_2CTA", "1") != "0"


def gemm_tcgen05(x: torch.Tensor, w: torch.Tensor, *, epilogue: int = EPI_NONE, activation: str = "gelu_tanh",
                 pair: Optional[bool] = None, out: Optional[torch.Tensor] = None, act_consts=(0.0, 0.0)):
    """x w^T for whole prompts on the 5th-generation tensor cores (bfloat16, any M; K a multiple of 8).
    Epilogues: none, gated (w = [gate; up] stacked), or an activation alone (``"xielu"`` with its two
    constants in ``act_consts``).  With more than 128 rows pairs of CTAs
    compute 256 x 256 tiles (``pair``; QNN_GEMM_2CTA=0 keeps one CTA per tile).  Returns None when
    the sizes are refused."""
    _req(x, "x", torch.bfloat16, 2)
    _req(w, "w", torch.bfloat16, 2)
    M, K = x.shape
    N = w.shape[0]
    if epilogue not in (EPI_NONE, EPI_GATED, EPI_ACT) or K % 8 or w.shape[1] != K:
        return None
    if activation == "xielu" and epilogue != EPI_ACT:
        raise ValueError("gemm_tcgen05: xielu is an activation without a gate")
    act_code = (ACT_XIELU if activation == "xielu" else ACT_CODES[activation]) + (ACT_ALONE if epilogue == EPI_ACT else 0)
    ka, kb = float(act_consts[0]), float(act_consts[1])
    if epilogue == EPI_ACT:
        epilogue = EPI_NONE
    n_out = N // 2 if epilogue == EPI_GATED else N
    if out is None:
        out = torch.empty((M, n_out), dtype=torch.bfloat16, device=x.device)
    else:
        _req(out, "out", torch.bfloat16, 2)
        if tuple(out.shape) != (M, n_out):
            raise ValueError(f"gemm_tcgen05: out is {tuple(out.shape)}, the product [{M}, {n_out}]")
    L = _lib.load()
    if pair is None:
        pair = GEMM_2CTA and M > 128
    if pair:
        code = L.qnn_gemm_tcgen05_2cta(_p(x), _p(w), _p(out), M, N, K, epilogue, act_code, ka, kb,
                                       _p(_status_word(x.device)), _stream())
        if code != _lib.ERR_UNSUPPORTED:
            _lib.check(code, "gemm_tcgen05_2cta")
            return out
    code = L.qnn_gemm_tcgen05(_p(x), _p(w), _p(out), M, N, K, epilogue, act_code, ka, kb,
                              _p(_status_word(x.device)), _stream())
    if code == _lib.ERR_UNSUPPORTED:
        return None
    _lib.check(code, "gemm_tcgen05")
    return out


def gemm_skinny_tcgen05(x: torch.Tensor, w: torch.Tensor, *, epilogue: int = EPI_NONE, cap: Optional[float] = None,
                        activation: str = "gelu_tanh", out: Optional[torch.Tensor] = None):
    """x w^T for up to 128 rows: TMA + tcgen05 with K split over a thread-block cluster and summed
    through distributed shared memory.  Epilogues: none (bfloat16), softcap (float32), gated.
    Returns None when the sizes are refused."""
    _req(x, "x", torch.bfloat16, 2)
    _req(w, "w", torch.bfloat16, 2)
    M, K = x.shape
    N = w.shape[0]
    if M > 128 or K % 8 or w.shape[1] != K:
        return None
    act_code = ACT_CODES[activation] + (ACT_ALONE if epilogue == EPI_ACT else 0)
    if epilogue == EPI_ACT:
        epilogue = EPI_NONE
    n_out = N // 2 if epilogue == EPI_GATED else N
    out_dtype = torch.float32 if epilogue == EPI_SOFTCAP else torch.bfloat16
    if out is None:
        out = torch.empty((M, n_out), dtype=out_dtype, device=x.device)
    else:
        _req(out, "out", out_dtype, 2)
        if tuple(out.shape) != (M, n_out):
            raise ValueError(f"gemm_skinny_tcgen05: out is {tuple(out.shape)}, the product [{M}, {n_out}]")
    L = _lib.load()
    code = L.qnn_gemm_skinny_tcgen05(_p(x), _p(w), _p(out), M, N, K, epilogue, float(cap or 0.0),
                                     act_code, _p(_status_word(x.device)), _stream())
    if code == _lib.ERR_UNSUPPORTED:
        return None
    _lib.check(code, "gemm_skinny_tcgen05")
    return out


USE_TCGEN05 = os.environ.get("QNN_GEMM", "tcgen05") != "cublas"
# From this many rows on, products against big matrices (>= 2^24 weights) take the cluster split-K
# tcgen05 kernel instead of the mma.sync small-M kernel (measured on B200: up to 8 rows, one 8-row
# tile of mma.sync, and for the small q/k/v and o matrices up to about 30 rows, the mma.sync kernel is
# the faster one; at 12 and 16 rows the step gains 8-9 % with the tcgen05 kernel for the big matrices).
SKINNY_TCGEN05_FROM = int(os.environ.get("QNN_SKINNY_TCGEN05_FROM", "9"))
SKINNY_TCGEN05_MIN_WEIGHTS = 1 << 24
SKINNY_TCGEN05_ANY_FROM = 32          # from this many rows on, the small matrices too (q|k|v at 32 rows: 10.7 against 13.0 us)


def _takes_skinny_tcgen05(M: int, N: int, K: int) -> bool:
    return USE_TCGEN05 and SKINNY_TCGEN05_FROM <= M <= 128 and (M >= SKINNY_TCGEN05_ANY_FROM or
                                                                N * K >= SKINNY_TCGEN05_MIN_WEIGHTS)


_SM_COUNT: dict = {}


def _rows_for_the_small_kernel(M: int, n_out: int, K: int, epilogue: int, device) -> int:
    """How many of the last rows of a whole-prompt product go to the kernel for few rows instead (0: none).

    The prompt kernel works in 256 x 256 tiles (256 x 128 outputs when gated), a pair of SMs per tile, so its time
    goes up by a round of tiles when the tile count passes a multiple of the pairs.  Measured for the down product
    (2304 x 9216): 2048 rows (72 tiles on 74 pairs) 58 us, 2049 rows 92 us, 4096 / 4097 rows 114 / 140 us, 6144 /
    6145 rows 175 / 212 us: a round that only a few tiles open costs about 0.6 of a tile's time.  The kernel for few
    rows takes the weights' bytes once more plus 5 us up to 32 rows and 9 us up to 64 (2049 rows: 66 us together, 4097:
    123, 6145: 179); with more rows it costs what the round does (2200 rows in two launches: 90 against 92 us), and
    for the matrices with a short inner size the round is cheap, so only up to 64 rows are cut off, and only where
    the round costs well more than they do."""
    if not GEMM_2CTA or M <= 256:
        return 0
    tail = M % 256
    if tail == 0 or tail > 64:
        return 0
    key = str(device)
    if key not in _SM_COUNT:
        _SM_COUNT[key] = torch.cuda.get_device_properties(device).multi_processor_count if device.type == "cuda" else 148
    pairs = max(1, _SM_COUNT[key] // 2)
    per_row_tile = -(-n_out // (128 if epilogue == EPI_GATED else 256))
    rounds = lambda m_tiles: -(-m_tiles * per_row_tile // pairs)          # noqa: E731
    if rounds(-(-M // 256)) == rounds(M // 256):
        return 0
    weights = n_out * (2 if epilogue == EPI_GATED else 1) * K
    round_us = 0.6 * 2.0 * 256 * 256 * K / 22.0e6                # a tile at a pair's share of 1.6 PFLOP/s
    small_us = 2.0 * weights / 6.5e6 + (5.0 if tail <= 32 else 9.0)
    return tail if round_us > 1.5 * small_us else 0


def linear(x: torch.Tensor, w: torch.Tensor, *, epilogue: int = EPI_NONE, cap: Optional[float] = None,
           activation: str = "gelu_tanh", out_dtype: Optional[torch.dtype] = None, act_consts=None):
    """y = x w^T with an optional epilogue.  x: [M, K]; w: [N, K] (gated: [2*N_out, K]).

    float32: FFMA kernels only.  bfloat16: the tensor-core small-M kernel up to 64 rows (the cluster
    split-K tcgen05 kernel from 9 rows on against big matrices), the tcgen05/TMA kernel above that; an inner
    size that is no multiple of 8 (rows that do not start on 16 bytes) goes to a plain kernel; a library
    product (cuBLAS) only when QNN_GEMM=cublas is set."""
    _req(x, "x", None, 2)
    _req(w, "w", None, 2)
    M, K = x.shape
    N = w.shape[0]
    if w.shape[1] != K:
        raise ValueError(f"linear: x is [*, {K}] but w is [*, {w.shape[1]}]")
    if x.dtype != w.dtype:
        raise TypeError(f"linear: x is {x.dtype} but w is {w.dtype}")
    n_out = N // 2 if epilogue == EPI_GATED else N
    if out_dtype is None:
        out_dtype = torch.float32 if epilogue == EPI_SOFTCAP else x.dtype
    if activation == "xielu":
        # the tcgen05 kernels for whole prompts apply it in their epilogue; the kernels for few rows and float32 take
        # the product and then the activation's own kernel
        if epilogue != EPI_ACT or act_consts is None:
            raise ValueError("linear: xielu is an activation without a gate and comes with its two constants")
        if x.dtype == torch.bfloat16 and M > SKINNY_MAX_ROWS and K % 8 == 0 and USE_TCGEN05 and out_dtype == torch.bfloat16:
            y = gemm_tcgen05(x, w, epilogue=EPI_ACT, activation="xielu", act_consts=act_consts)
            if y is not None:
                return y
        if (x.dtype == torch.bfloat16 and M <= SKINNY_MAX_ROWS and K % 8 == 0 and out_dtype == torch.bfloat16
                and not _takes_skinny_tcgen05(M, N, K)):
            out = torch.empty((M, N), dtype=torch.bfloat16, device=x.device)      # the kernel for few rows has it too
            _lib.check(_lib.load().qnn_skinny_bf16(_p(x), _p(w), _p(out), dt_code(out), M, N, K, EPI_NONE, 0.0,
                                                   ACT_XIELU + ACT_ALONE, float(act_consts[0]), float(act_consts[1]),
                                                   _stream()), "skinny_bf16")
            return out
        return xielu_(linear(x, w, out_dtype=out_dtype), act_consts[0], act_consts[1])
    if epilogue == EPI_ACT and (x.dtype == torch.float32 or K % 8 or not USE_TCGEN05 or out_dtype != torch.bfloat16):
        # act(x w^T) where the product's kernels have no such epilogue: the product, then the activation
        return activation_(linear(x, w, out_dtype=out_dtype), activation)
    L = _lib.load()
    capv = float(cap or 0.0)
    act = ACT_CODES[activation] + (ACT_ALONE if epilogue == EPI_ACT else 0)
    fused_act = epilogue == EPI_ACT
    if fused_act:
        epilogue = EPI_NONE               # the bfloat16 kernels below read the activation from `act`
    if x.dtype == torch.float32:
        if out_dtype != torch.float32:
            raise TypeError("float32 products give float32")
        out = torch.empty((M, n_out), dtype=torch.float32, device=x.device)
        if M <= 8:
            _lib.check(L.qnn_gemv_f32(_p(x), _p(w), _p(out), M, N, K, epilogue, capv, act, _stream()), "gemv_f32")
        elif epilogue == EPI_GATED:
            gu = torch.empty((M, N), dtype=torch.float32, device=x.device)
            _lib.check(L.qnn_sgemm_f32(_p(x), _p(w), _p(gu), M, N, K, EPI_NONE, 0.0, _stream()), "sgemm_f32")
            out = gated_act(gu, activation)
        else:
            _lib.check(L.qnn_sgemm_f32(_p(x), _p(w), _p(out), M, N, K, epilogue, capv, _stream()), "sgemm_f32")
        return out
    # bfloat16
    if K % 8:                                  # rows that do not start on 16 bytes: the plain kernel for any inner size
        out = torch.empty((M, n_out), dtype=out_dtype, device=x.device)
        _lib.check(L.qnn_linear_bf16_any(_p(x), _p(w), _p(out), dt_code(out), M, N, K, epilogue, capv, act, _stream()),
                   "linear_bf16_any")
        return out
    kind = EPI_ACT if fused_act else epilogue          # what the tcgen05 wrappers are asked for
    if _takes_skinny_tcgen05(M, N, K) and out_dtype == (torch.float32 if epilogue == EPI_SOFTCAP else torch.bfloat16):
        y = gemm_skinny_tcgen05(x, w, epilogue=kind, cap=cap, activation=activation)
        if y is not None:
            return y
    def small(xr: torch.Tensor, out: torch.Tensor) -> None:
        _lib.check(L.qnn_skinny_bf16(_p(xr), _p(w), _p(out), dt_code(out), xr.shape[0], N, K, epilogue, capv, act, 0.0, 0.0,
                                     _stream()), "skinny_bf16")

    if M <= SKINNY_MAX_ROWS:
        out = torch.empty((M, n_out), dtype=out_dtype, device=x.device)
        small(x, out)
        return out
    if USE_TCGEN05:
        if epilogue in (EPI_NONE, EPI_GATED) and out_dtype == torch.bfloat16:
            tail = _rows_for_the_small_kernel(M, n_out, K, epilogue, x.device)
            if tail:
                # the last rows would open one more round of 256 x 256 tiles: they go to the kernel for few rows
                head = M - tail
                out = torch.empty((M, n_out), dtype=out_dtype, device=x.device)
                ok = (gemm_tcgen05(x[:head], w, epilogue=kind, activation=activation, out=out[:head]) is not None
                      and gemm_skinny_tcgen05(x[head:], w, epilogue=kind, activation=activation,
                                              out=out[head:]) is not None)
                if ok:
                    return out
            y = gemm_tcgen05(x, w, epilogue=kind, activation=activation)
            if y is not None:
                return y
        elif epilogue == EPI_SOFTCAP:          # logits wanted at many places: the product, then the cap in float32
            y = gemm_tcgen05(x, w)
            if y is not None:
                return softcap(y, cap)
        # sizes that the tcgen05 kernels refuse: the small-M kernel, 64 rows at a time
        out = torch.empty((M, n_out), dtype=out_dtype, device=x.device)
        for r0 in range(0, M, SKINNY_MAX_ROWS):
            small(x[r0:r0 + SKINNY_MAX_ROWS], out[r0:r0 + SKINNY_MAX_ROWS])
        return out
    y = torch.matmul(x, w.t())                 # QNN_GEMM=cublas: the library product, for comparisons
    if epilogue == EPI_GATED:
        return gated_act(y, activation)
    if epilogue == EPI_SOFTCAP:
        return softcap(y, cap)
    return y if out_dtype == y.dtype else cast(y, out_dtype)


ATTN_TCGEN05 = os.environ.get("QNN_ATTN", "tcgen05") != "mma"
# A step that continues sequences takes the tensor-core prompt kernel from this many rows of a sequence on.  Measured
# at 8 heads of 256, one sequence, launched eagerly: 8 new rows on 4000 cached tokens 108 us against 3776 us of the
# generic kernel (a warp per row and kv head that walks the keys one after the other), 512 rows on 7000: 152 us against
# 8477; so always, where the sizes allow.
EXTEND_TENSOR_CORE_FROM = int(os.environ.get("QNN_EXTEND_TC_FROM", "1"))


def attention_refusal(dtype: torch.dtype, n_heads: int, n_kv: int, head_dim: int) -> Optional[str]:
    """None if the attention kernels take these head counts and this head size in ``dtype``, else the
    reason in words.  Asked when a model is loaded."""
    code = _lib.load().qnn_attn_supports(BF16 if dtype == torch.bfloat16 else F32, n_heads, n_kv, head_dim)
    if code == 0:
        return None
    vec = 8 if dtype == torch.bfloat16 else 4
    if code == _lib.ERR_ARGUMENT:
        return f"{n_kv} key/value heads do not divide {n_heads} query heads"
    return (f"head size {head_dim} in {dtype}: the attention kernels take multiples of {vec} up to {128 * vec} "
            f"(less when four or more query heads share a key/value head)")


def linear_refusal(dtype: torch.dtype, inner: int) -> Optional[str]:
    """None if the matrix products take this inner size in ``dtype``, else the reason.  Every size is taken:
    bfloat16 rows of whole 16-byte pieces (a multiple of 8) by the tensor-core kernels, others by a plain one."""
    if inner <= 0:
        return f"an inner size of {inner}"
    return None


def _check_slopes(slopes: Optional[torch.Tensor], n_heads: int) -> None:
    if slopes is not None:
        _req(slopes, "slopes", torch.float32, 1)
        if slopes.numel() != n_heads:
            raise ValueError(f"attention: {slopes.numel()} distance slopes for {n_heads} query heads")


def attn_prefill(qkv: torch.Tensor, n_heads: int, n_kv: int, head_dim: int, tok_pos: torch.Tensor,
                 tok_row0: torch.Tensor, scale: float, cap: Optional[float], window: Optional[int],
                 seq_row0: Optional[torch.Tensor] = None, seq_len: Optional[torch.Tensor] = None,
                 max_len: int = 0, slopes: Optional[torch.Tensor] = None):
    """Causal (optionally windowed) attention of this step's own rows.  qkv: [T, (nq+2nkv)*hd]
    after rotation; returns [T, nq*hd].  bfloat16 with head sizes 64/128/256 runs on the tensor
    cores when the per-sequence arrays (first row, length) are given; everything else takes the
    generic kernel.  ``slopes`` (float32, one per query head, optional): ``slope * (i - j)`` is subtracted from the
    score of query position i and key position j."""
    _req(qkv, "qkv", None, 2)
    _check_slopes(slopes, n_heads)
    T = qkv.shape[0]
    out = torch.empty((T, n_heads * head_dim), dtype=qkv.dtype, device=qkv.device)
    es = qkv.element_size()
    q_ptr = qkv.data_ptr()
    k_ptr = q_ptr + n_heads * head_dim * es
    v_ptr = k_ptr + n_kv * head_dim * es
    L = _lib.load()
    if (qkv.dtype == torch.bfloat16 and seq_row0 is not None and seq_len is not None and max_len > 0
            and head_dim in (64, 128, 256)):
        _req(seq_row0, "seq_row0", torch.int32, 1)
        _req(seq_len, "seq_len", torch.int32, 1)
        if ATTN_TCGEN05:
            code = L.qnn_attn_prefill_tcgen05(
                _p(qkv), T, _p(out), out.shape[1], _p(seq_row0), _p(seq_len), None, seq_row0.numel(), int(max_len),
                n_heads, n_kv, head_dim, float(scale), float(cap or 0.0), int(window or 0),
                _p(_status_word(qkv.device)), _p(slopes), _stream())
            if code != _lib.ERR_UNSUPPORTED:
                _lib.check(code, "attn_prefill_tcgen05")
                return out
        code = L.qnn_attn_prefill_mma(
            ctypes.c_void_p(q_ptr), ctypes.c_void_p(k_ptr), ctypes.c_void_p(v_ptr), qkv.shape[1], _p(out),
            out.shape[1], _p(seq_row0), _p(seq_len), seq_row0.numel(), int(max_len), n_heads, n_kv, head_dim,
            float(scale), float(cap or 0.0), int(window or 0), _p(slopes), _stream())
        if code != _lib.ERR_UNSUPPORTED:
            _lib.check(code, "attn_prefill_mma")
            return out
    _lib.check(L.qnn_attn_prefill_generic(
        ctypes.c_void_p(q_ptr), ctypes.c_void_p(k_ptr), ctypes.c_void_p(v_ptr), qkv.shape[1], dt_code(qkv),
        _p(out), out.shape[1], _p(tok_pos), _p(tok_row0), T, n_heads, n_kv, head_dim, float(scale),
        float(cap or 0.0), int(window or 0), _p(slopes), _stream()), "attn_prefill")
    return out


def attn_prefill_paged(qkv: torch.Tensor, n_heads: int, n_kv: int, head_dim: int, k_pool: torch.Tensor,
                       v_pool: torch.Tensor, page_table: torch.Tensor, page_size: int, ring: int,
                       tok_pos: torch.Tensor, tok_slot: torch.Tensor, scale: float, cap: Optional[float],
                       window: Optional[int], slopes: Optional[torch.Tensor] = None):
    """Several query rows per sequence against the paged cache (keys written earlier in the
    same step by the layer that owns the line).  q = the first nq*hd columns of qkv."""
    _req(qkv, "qkv", None, 2)
    _check_slopes(slopes, n_heads)
    _req(k_pool, "k_pool", qkv.dtype, 4)
    _req(v_pool, "v_pool", qkv.dtype, 4)
    T = qkv.shape[0]
    out = torch.empty((T, n_heads * head_dim), dtype=qkv.dtype, device=qkv.device)
    L = _lib.load()
    _lib.check(L.qnn_attn_prefill_paged(
        _p(qkv), qkv.shape[1], dt_code(qkv), _p(k_pool), _p(v_pool), _p(page_table), page_table.shape[1],
        page_size, ring, _p(out), out.shape[1], _p(tok_pos), _p(tok_slot), T, n_heads, n_kv, head_dim,
        float(scale), float(cap or 0.0), int(window or 0), _p(slopes), _stream()), "attn_prefill_paged")
    return out


def attn_shared_tensor_core(q: torch.Tensor, n_heads: int, n_kv: int, head_dim: int, k_pool: torch.Tensor,
                            v_pool: torch.Tensor, page_table: torch.Tensor, page_size: int, ring: int, slots: torch.Tensor,
                            seq_row0: torch.Tensor, seq_len: torch.Tensor, scale: float, cap: Optional[float],
                            window: Optional[int], longest: int, whole=None,
                            slopes: Optional[torch.Tensor] = None) -> Optional[torch.Tensor]:
    """Attention of query rows ``q`` ([rows, n_heads * head_dim]) whose keys and values, this step's positions included,
    are in the paged cache already (a layer that reads the line another layer wrote earlier in the step), on the
    tensor-core prompt kernel: keys and values are copied out of the pages beside the queries into whole sequences,
    as ``attn_extend`` does.  ``whole``: the sequences with their cached tokens in front when the step continues
    sequences; None for whole prompts.  Returns None where that kernel does not serve (the caller takes the generic one)."""
    if not (ATTN_TCGEN05 and q.dtype == torch.bfloat16 and head_dim in (64, 128, 256)):
        return None
    _req(q, "q", torch.bfloat16, 2)
    _check_slopes(slopes, n_heads)
    L = _lib.load()
    width = (n_heads + 2 * n_kv) * head_dim
    if whole is None:
        B, total, most = seq_row0.numel(), q.shape[0], int(longest)
        start, row0, length, new_row0, new_len = None, seq_row0, seq_len, seq_row0, seq_len
    else:
        B, total, most = whole.row0.numel(), whole.total, whole.longest
        start, row0, length, new_row0, new_len = whole.start, whole.row0, whole.length, whole.new_row0, whole.new_len
    rows = torch.empty((total, width), dtype=q.dtype, device=q.device)
    _lib.check(L.qnn_attn_extend_gather(
        _p(q), _p(k_pool), _p(v_pool), _p(page_table), page_table.shape[1], page_size, ring, _p(slots), _p(start),
        _p(new_row0), _p(new_len), _p(row0), _p(rows), B, most, n_heads, n_kv, head_dim, 1, _stream()), "attn_extend_gather")
    out_rows = torch.empty((total, n_heads * head_dim), dtype=q.dtype, device=q.device)
    code = L.qnn_attn_prefill_tcgen05(
        _p(rows), total, _p(out_rows), out_rows.shape[1], _p(row0), _p(length), _p(start), B, most, n_heads, n_kv,
        head_dim, float(scale), float(cap or 0.0), int(window or 0), _p(_status_word(q.device)), _p(slopes), _stream())
    if code == _lib.ERR_UNSUPPORTED:
        return None
    _lib.check(code, "attn_prefill_tcgen05")
    return out_rows if whole is None else gather_rows(out_rows, whole.tok_row, q.dtype)


def attn_extend(qkv: torch.Tensor, n_heads: int, n_kv: int, head_dim: int, k_pool: torch.Tensor, v_pool: torch.Tensor,
                page_table: torch.Tensor, page_size: int, ring: int, tok_pos: torch.Tensor, tok_row0: torch.Tensor,
                tok_slot: torch.Tensor, scale: float, cap: Optional[float], window: Optional[int], whole=None,
                slopes: Optional[torch.Tensor] = None):
    """Attention of a step that continues sequences by several tokens: each row sees the cached
    positions before its sequence's first row of this step (from the cache, as earlier steps left it)
    and this step's own rows from there to itself (from ``qkv``, already rotated).  The caller appends
    this step's keys and values to the cache afterwards.

    ``whole`` (a ``WholeSequences``, optional) describes the step's sequences laid out with their cached
    tokens in front; with it, bfloat16 rows of head size 64, 128 or 256 go through the tensor-core prompt
    kernel: the cached keys and values are copied out of the pages into that layout, the kernel leaves out
    the query tiles that lie before each sequence's new rows, and the new rows' outputs are picked out.
    The generic kernel walks the keys once per row and kv head: it serves float32 and the other head sizes."""
    _req(qkv, "qkv", None, 2)
    _check_slopes(slopes, n_heads)
    _req(k_pool, "k_pool", qkv.dtype, 4)
    _req(v_pool, "v_pool", qkv.dtype, 4)
    for n, t in (("tok_pos", tok_pos), ("tok_row0", tok_row0), ("tok_slot", tok_slot)):
        _req(t, n, torch.int32, 1)
    T = qkv.shape[0]
    if (whole is not None and ATTN_TCGEN05 and qkv.dtype == torch.bfloat16 and head_dim in (64, 128, 256)
            and whole.most_new >= EXTEND_TENSOR_CORE_FROM):
        L = _lib.load()
        B = whole.row0.numel()
        rows = torch.empty((whole.total, qkv.shape[1]), dtype=qkv.dtype, device=qkv.device)
        _lib.check(L.qnn_attn_extend_gather(
            _p(qkv), _p(k_pool), _p(v_pool), _p(page_table), page_table.shape[1], page_size, ring, _p(whole.slots),
            _p(whole.start), _p(whole.new_row0), _p(whole.new_len), _p(whole.row0), _p(rows), B, whole.longest,
            n_heads, n_kv, head_dim, 0, _stream()), "attn_extend_gather")
        out_rows = torch.empty((whole.total, n_heads * head_dim), dtype=qkv.dtype, device=qkv.device)
        code = L.qnn_attn_prefill_tcgen05(
            _p(rows), whole.total, _p(out_rows), out_rows.shape[1], _p(whole.row0), _p(whole.length), _p(whole.start), B,
            whole.longest, n_heads, n_kv, head_dim, float(scale), float(cap or 0.0), int(window or 0),
            _p(_status_word(qkv.device)), _p(slopes), _stream())
        if code != _lib.ERR_UNSUPPORTED:
            _lib.check(code, "attn_prefill_tcgen05")
            return gather_rows(out_rows, whole.tok_row, qkv.dtype)
    out = torch.empty((T, n_heads * head_dim), dtype=qkv.dtype, device=qkv.device)
    es = qkv.element_size()
    q_ptr = qkv.data_ptr()
    k_ptr = q_ptr + n_heads * head_dim * es
    v_ptr = k_ptr + n_kv * head_dim * es
    L = _lib.load()
    _lib.check(L.qnn_attn_extend(
        ctypes.c_void_p(q_ptr), ctypes.c_void_p(k_ptr), ctypes.c_void_p(v_ptr), qkv.shape[1], dt_code(qkv),
        _p(k_pool), _p(v_pool), _p(page_table), page_table.shape[1], page_size, ring, _p(out), out.shape[1],
        _p(tok_pos), _p(tok_row0), _p(tok_slot), T, n_heads, n_kv, head_dim, float(scale), float(cap or 0.0),
        int(window or 0), _p(slopes), _stream()), "attn_extend")
    return out


def attn_decode(qkv: torch.Tensor, n_heads: int, n_kv: int, head_dim: int, k_pool: torch.Tensor,
                v_pool: torch.Tensor, page_table: torch.Tensor, page_size: int, ring: int,
                slots: torch.Tensor, slot_len: torch.Tensor, scale: float, cap: Optional[float],
                window: Optional[int], n_splits: int, part_o: torch.Tensor, part_ml: torch.Tensor,
                slopes: Optional[torch.Tensor] = None):
    """One query row per sequence against the paged cache.  q = the first nq*hd columns of qkv.
    ``slots``, ``slot_len`` and ``page_table`` must be complete before the kernel that runs just before
    this one on the stream starts (host copies and earlier kernels are): the tensor-core kernel reads
    them while that kernel may still run."""
    _req(qkv, "qkv", None, 2)
    _check_slopes(slopes, n_heads)
    B = qkv.shape[0]
    _req(k_pool, "k_pool", qkv.dtype, 4)
    _req(v_pool, "v_pool", qkv.dtype, 4)
    _req(page_table, "page_table", torch.int32, 2)
    _req(slots, "slots", torch.int32, 1)
    _req(slot_len, "slot_len", torch.int32, 1)
    need = B * n_heads * n_splits
    if part_o.numel() < need * head_dim or part_ml.numel() < need * 2:
        raise ValueError("attn_decode: scratch is too small")
    out = torch.empty((B, n_heads * head_dim), dtype=qkv.dtype, device=qkv.device)
    L = _lib.load()
    _lib.check(L.qnn_attn_decode(
        _p(qkv), qkv.shape[1], dt_code(qkv), _p(k_pool), _p(v_pool), _p(page_table), page_table.shape[1],
        page_size, ring, _p(slots), _p(slot_len), B, n_heads, n_kv, head_dim, float(scale), float(cap or 0.0),
        int(window or 0), _p(part_o), _p(part_ml), n_splits, _p(out), out.shape[1], _p(slopes), _stream()), "attn_decode", 2)
    return out


def sample_scratch_bytes(rows: int, vocab: int, top_k: int) -> int:
    L = _lib.load()
    return int(L.qnn_sample_scratch_bytes(rows, vocab, top_k))


def sample(logits: torch.Tensor, top_k: int, temperature: float, top_p: float, penalty: float,
           rng_state: torch.Tensor, seen: Optional[torch.Tensor], seen_rows: Optional[torch.Tensor],
           scratch: torch.Tensor, out_tokens: torch.Tensor, error_flag: Optional[torch.Tensor],
           status: Optional[torch.Tensor] = None):
    """``status`` (one int32 on the device) is OR-ed into ``error_flag`` as bit 1 plus its value
    from bit 8 up: what the step's kernels reported reaches the host with the ids."""
    _req(logits, "logits", torch.float32, 2)
    R, V = logits.shape
    _req(out_tokens, "out_tokens", torch.int32, 1)
    _req(rng_state, "rng_state", torch.int32, 1)
    if out_tokens.numel() < R or rng_state.numel() < R:
        raise ValueError("sample: out_tokens / rng_state are shorter than the batch")
    if scratch.numel() * scratch.element_size() < sample_scratch_bytes(R, V, top_k):
        raise ValueError("sample: scratch is too small")
    L = _lib.load()
    _lib.check(L.qnn_sample(_p(logits), R, V, int(top_k), float(temperature), float(top_p), float(penalty),
                            _p(rng_state), _p(seen), _p(seen_rows), _p(scratch), _p(out_tokens), _p(error_flag),
                            _p(status), _stream()), "sample", 4 if (temperature > 0 and top_k > 1 and V > 1) else 2)
    return out_tokens


def head_argmax_fusable(x: torch.Tensor, w: torch.Tensor) -> bool:
    """Whether ``head_argmax`` takes this product: bfloat16 on both sides, an inner size in whole 16-byte
    vectors, and at most 128 rows."""
    M, K = x.shape
    return x.dtype == torch.bfloat16 and w.dtype == torch.bfloat16 and K % 8 == 0 and 1 <= M <= 128


def head_candidates(vocab: int) -> int:
    """The most candidates per row that ``head_argmax`` writes (one per 16 output columns)."""
    return (vocab + 15) // 16


def head_argmax(x: torch.Tensor, w: torch.Tensor, cap: Optional[float], cand: torch.Tensor,
                error_flag: Optional[torch.Tensor]) -> Optional[int]:
    """softcap(x w^T) reduced in the product's epilogue to the best (value, id) of every group of output
    columns: ``cand`` (float32, at least rows * head_candidates(vocab) * 2) is filled, the logits are not
    written.  The product is the one that ``linear`` would run for these sizes: the mma.sync small-M kernel
    (a candidate per 16 columns) or, from 9 rows on against a big matrix, the tcgen05 kernel (a candidate
    per 128 columns).  Returns the number of candidates per row, or None when the sizes are refused (the
    caller then forms the logits).  NaN or Inf sets bit 0 of ``error_flag``."""
    _req(x, "x", torch.bfloat16, 2)
    _req(w, "w", torch.bfloat16, 2)
    _req(cand, "cand", torch.float32)
    M, K = x.shape
    N = w.shape[0]
    if w.shape[1] != K:
        raise ValueError(f"head_argmax: x is [*, {K}] but w is [*, {w.shape[1]}]")
    if cand.numel() < M * head_candidates(N) * 2:
        raise ValueError("head_argmax: the candidate buffer is too small")
    L = _lib.load()
    if _takes_skinny_tcgen05(M, N, K):
        code = L.qnn_gemm_skinny_tcgen05_argmax(_p(x), _p(w), _p(cand), M, N, K, float(cap or 0.0), _p(error_flag),
                                                _p(_status_word(x.device)), _stream())
        if code != _lib.ERR_UNSUPPORTED:
            _lib.check(code, "gemm_skinny_tcgen05_argmax")
            return (N + 127) // 128
    if M > SKINNY_MAX_ROWS:
        return None
    _lib.check(L.qnn_skinny_argmax(_p(x), _p(w), _p(cand), M, N, K, float(cap or 0.0), _p(error_flag), _stream()),
               "skinny_argmax")
    return (N + 15) // 16


def sample_candidates(cand: torch.Tensor, rows: int, ncand: int, vocab: int, top_k: int, temperature: float,
                      top_p: float, rng_state: torch.Tensor, seen: Optional[torch.Tensor],
                      seen_rows: Optional[torch.Tensor], out_tokens: torch.Tensor,
                      error_flag: Optional[torch.Tensor], status: Optional[torch.Tensor] = None) -> torch.Tensor:
    """The merge-and-draw half of ``sample`` on candidates [rows, ncand] of (value, id) pairs."""
    _req(cand, "cand", torch.float32)
    _req(out_tokens, "out_tokens", torch.int32, 1)
    _req(rng_state, "rng_state", torch.int32, 1)
    if cand.numel() < rows * ncand * 2 or out_tokens.numel() < rows or rng_state.numel() < rows:
        raise ValueError("sample_candidates: a buffer is shorter than the batch")
    L = _lib.load()
    _lib.check(L.qnn_sample_candidates(_p(cand), rows, ncand, vocab, int(top_k), float(temperature), float(top_p),
                                       _p(rng_state), _p(seen), _p(seen_rows), _p(out_tokens), _p(error_flag),
                                       _p(status), _stream()), "sample_candidates")
    return out_tokens


def mark_seen(tokens: torch.Tensor, rows: torch.Tensor, seen: torch.Tensor):
    _req(tokens, "tokens", torch.int32, 1)
    _req(rows, "rows", torch.int32, 1)
    _req(seen, "seen", torch.uint8, 2)
    L = _lib.load()
    _lib.check(L.qnn_mark_seen(_p(tokens), _p(rows), _p(seen), seen.shape[1], tokens.numel(), _stream()),
               "mark_seen")


# ---- the residual stream with a multiplier, norms over pieces of rows -----------------------------------

def add_scaled_rmsnorm(resid: torch.Tensor, y: torch.Tensor, scale: float, w_next: Optional[torch.Tensor] = None,
                       eps_next: float = 0.0, unit_next: bool = False, out_dtype: Optional[torch.dtype] = None):
    """resid += scale * y (float32 stream, in place); returns rmsnorm(resid, w_next) when ``w_next`` is given."""
    _req(resid, "resid", torch.float32, 2)
    _req(y, "y", None, 2)
    T, H = resid.shape
    if tuple(y.shape) != (T, H) or (w_next is not None and w_next.numel() != H):
        raise ValueError("add_scaled_rmsnorm: shapes do not agree")
    out = None
    if w_next is not None:
        _req(w_next, "w_next", None, 1)
        out = torch.empty((T, H), dtype=out_dtype, device=resid.device)
    _lib.check(_lib.load().qnn_add_scaled_rmsnorm(
        _p(resid), _p(y), dt_code(y), float(scale), _p(w_next), dt_code(w_next) if w_next is not None else 0,
        float(eps_next), int(unit_next), _p(out), dt_code(out) if out is not None else 0, T, H, _stream()),
        "add_scaled_rmsnorm")
    return out


def _col_ptr(t: torch.Tensor, col: int):
    return ctypes.c_void_p(t.data_ptr() + col * t.element_size())


def rmsnorm_cols(x: torch.Tensor, col0: int, n: int, weight: torch.Tensor, eps: float, out: torch.Tensor,
                 out_col0: int = 0, out2_col0: Optional[int] = None) -> torch.Tensor:
    """RMS norm (plain weight) of the columns ``col0 .. col0 + n`` of every row of ``x``, written to the columns
    ``out_col0 ..`` of ``out`` and, if given, once more to ``out2_col0 ..``: a piece of a stacked product's
    rows normed into a packed buffer, float32 math."""
    _req(x, "x", None, 2)
    _req(out, "out", None, 2)
    _req(weight, "weight", None, 1)
    T = x.shape[0]
    ends = [out_col0 + n] + ([out2_col0 + n] if out2_col0 is not None else [])
    if out.shape[0] != T or weight.numel() != n or col0 + n > x.shape[1] or max(ends) > out.shape[1]:
        raise ValueError("rmsnorm_cols: shapes do not agree")
    _lib.check(_lib.load().qnn_rmsnorm_strided(
        _col_ptr(x, col0), dt_code(x), x.shape[1], _p(weight), dt_code(weight), float(eps), _col_ptr(out, out_col0),
        dt_code(out), out.shape[1], _col_ptr(out, out2_col0) if out2_col0 is not None else None, out.shape[1], T, n,
        _stream()), "rmsnorm_strided")
    return out


def copy_cols(src: torch.Tensor, dst: torch.Tensor, dst_col0: int) -> torch.Tensor:
    """dst[:, dst_col0 : dst_col0 + src.shape[1]] = src, rows of the same element type."""
    _req(src, "src", None, 2)
    _req(dst, "dst", src.dtype, 2)
    T, n = src.shape
    if dst.shape[0] != T or dst_col0 + n > dst.shape[1]:
        raise ValueError("copy_cols: shapes do not agree")
    _lib.check(_lib.load().qnn_copy_rows(_p(src), dt_code(src), n, _col_ptr(dst, dst_col0), dst.shape[1], T, n, _stream()),
               "copy_rows")
    return dst


def copy_col_range(src: torch.Tensor, src_col0: int, n: int, dst: torch.Tensor, dst_col0: int) -> torch.Tensor:
    """dst[:, dst_col0 : dst_col0 + n] = src[:, src_col0 : src_col0 + n], rows of the same element type."""
    _req(src, "src", None, 2)
    _req(dst, "dst", src.dtype, 2)
    T = src.shape[0]
    if dst.shape[0] != T or src_col0 + n > src.shape[1] or dst_col0 + n > dst.shape[1]:
        raise ValueError("copy_col_range: shapes do not agree")
    _lib.check(_lib.load().qnn_copy_rows(_col_ptr(src, src_col0), dt_code(src), src.shape[1], _col_ptr(dst, dst_col0),
                                         dst.shape[1], T, n, _stream()), "copy_rows")
    return dst


def scale_heads(x: torch.Tensor, gate_logits: torch.Tensor, n_heads: int) -> torch.Tensor:
    """x[t, h, :] *= sigmoid(gate_logits[t, h]) in place; the gate is float32."""
    _req(x, "x", None, 2)
    _req(gate_logits, "gate_logits", torch.float32, 2)
    T, HD = x.shape
    if HD % n_heads or tuple(gate_logits.shape) != (T, n_heads):
        raise ValueError("scale_heads: shapes do not agree")
    _lib.check(_lib.load().qnn_scale_heads(_p(x), dt_code(x), _p(gate_logits), T, n_heads, HD // n_heads, _stream()),
               "scale_heads")
    return x


def gate_heads(o: torch.Tensor, x: torch.Tensor, w_gate: torch.Tensor, n_heads: int) -> torch.Tensor:
    """o[t, h, :] *= sigmoid(x[t, :] . w_gate[h, :]) in place: ``small_linear_f32`` and ``scale_heads`` in one kernel
    (the logits and the sigmoid in float32)."""
    _req(o, "o", None, 2)
    _req(x, "x", None, 2)
    _req(w_gate, "w_gate", None, 2)
    T, HD = o.shape
    if HD % n_heads or x.shape[0] != T or tuple(w_gate.shape) != (n_heads, x.shape[1]):
        raise ValueError("gate_heads: shapes do not agree")
    _lib.check(_lib.load().qnn_gate_heads(_p(x), dt_code(x), _p(w_gate), dt_code(w_gate), x.shape[1], _p(o), dt_code(o), T,
                                          n_heads, HD // n_heads, _stream()), "gate_heads")
    return o


def small_linear_f32(x: torch.Tensor, w: torch.Tensor, decay_bias: Optional[torch.Tensor] = None,
                     tau: Optional[float] = None) -> torch.Tensor:
    """x w^T with float32 sums and a float32 result, whatever the element types: for the few outputs that feed
    float32 math (a gate per head, decay logits).  With ``decay_bias`` and ``tau`` the result is the decay
    sigmoid(x w^T + bias)^(1/tau) itself.  A plain kernel; the order of a sum depends on the inner size only."""
    _req(x, "x", None, 2)
    _req(w, "w", None, 2)
    T, K = x.shape
    N = w.shape[0]
    if w.shape[1] != K:
        raise ValueError(f"small_linear_f32: x is [*, {K}] but w is [*, {w.shape[1]}]")
    if decay_bias is not None:
        _req(decay_bias, "decay_bias", None, 1)
        if decay_bias.numel() != N or tau is None or not tau > 0:
            raise ValueError("small_linear_f32: a decay needs one bias per output and a positive tau")
    out = torch.empty((T, N), dtype=torch.float32, device=x.device)
    _lib.check(_lib.load().qnn_small_linear_f32(_p(x), dt_code(x), _p(w), dt_code(w), _p(out), T, N, K, _p(decay_bias),
                                                dt_code(decay_bias) if decay_bias is not None else 0,
                                                float(tau or 0.0), _stream()), "small_linear_f32")
    return out


# ---- gated linear attention -------------------------------------------------------------------------------

GLA_SEGMENT = 256            # rows of a segment when long sequences are walked in segments side by side
GLA_SEGMENTS_FROM = 512      # the longest sequence of a step from which that is done


def gla_scan(proj: torch.Tensor, q_col: int, k_col: int, v_col: int, decay: torch.Tensor, q_scale: float,
             seq_row0: Optional[torch.Tensor], seq_len: Optional[torch.Tensor], slots: torch.Tensor,
             state: torch.Tensor, n_seqs: int, n_heads: int, dim: int, vdim: int, longest: int = 0,
             key_from_decay: bool = False) -> torch.Tensor:
    """The recurrence S = diag(a) S + k v^T, o = S^T (q q_scale) over the rows of every sequence in order, from the
    state of the sequence's slot and back into it.  ``proj`` holds q and k ([*, heads*dim]) and v ([*, heads*vdim])
    from the given columns on; ``decay`` the decays a, float32 [rows, heads*dim]; returns o, float32 [rows, heads*vdim].

    ``longest``: the most rows that one sequence brings (0: unknown).  From 512 rows on the sequences are cut into
    segments of 256 rows that run side by side (the recurrence is linear in the state: each segment's own state and
    decay product first, a short pass over the segments in order, then the outputs); results differ from the walk
    in one piece by rounding only.  ``key_from_decay``: the keys are 1 - a, formed in float32 inside the scan (what the
    forget gate lets go is what is written); ``k_col`` is then not read."""
    _req(proj, "proj", None, 2)
    _req(decay, "decay", torch.float32, 2)
    _req(slots, "slots", torch.int32, 1)
    _req(state, "state", torch.float32)
    T = proj.shape[0]
    if tuple(decay.shape) != (T, n_heads * dim) or slots.numel() < n_seqs:
        raise ValueError("gla_scan: shapes do not agree")
    if tuple(state.shape[1:]) != (n_heads, dim, vdim):
        raise ValueError(f"gla_scan: the state is {tuple(state.shape)}, expected [slots, {n_heads}, {dim}, {vdim}]")
    if (seq_row0 is None) != (seq_len is None):
        raise ValueError("gla_scan: first rows and row counts come together")
    if seq_row0 is None and T < n_seqs:
        raise ValueError("gla_scan: fewer rows than sequences")
    out = torch.empty((T, n_heads * vdim), dtype=torch.float32, device=proj.device)
    if seq_row0 is not None and longest >= GLA_SEGMENTS_FROM and n_seqs * -(-longest // GLA_SEGMENT) <= 65535:
        nseg = -(-longest // GLA_SEGMENT)
        scratch = torch.zeros((n_seqs * nseg, n_heads, dim, vdim), dtype=torch.float32, device=proj.device)
        seg_decay = torch.empty((n_seqs * nseg, n_heads * dim), dtype=torch.float32, device=proj.device)
        _lib.check(_lib.load().qnn_gla_scan_segments(
            _col_ptr(proj, q_col), _col_ptr(proj, k_col), _col_ptr(proj, v_col), proj.shape[1], dt_code(proj), _p(decay),
            decay.shape[1], float(q_scale), _p(seq_row0), _p(seq_len), _p(slots), _p(state), _p(out), out.shape[1],
            n_seqs, n_heads, dim, vdim, GLA_SEGMENT, nseg, _p(scratch), _p(seg_decay), int(key_from_decay), _stream()),
            "gla_scan_segments", 4)
        return out
    _lib.check(_lib.load().qnn_gla_scan(
        _col_ptr(proj, q_col), _col_ptr(proj, k_col), _col_ptr(proj, v_col), proj.shape[1], dt_code(proj), _p(decay),
        decay.shape[1], float(q_scale), _p(seq_row0), _p(seq_len), _p(slots), _p(state),
        _p(out), out.shape[1], n_seqs, n_heads, dim, vdim, int(key_from_decay), _stream()), "gla_scan")
    return out


def gla_norm_gate(o: torch.Tensor, weight: torch.Tensor, eps: float, proj: torch.Tensor, g_col: int, n_heads: int,
                  vdim: int) -> torch.Tensor:
    """Per head: RMS norm of ``o`` over vdim (weight shared by the heads), times silu of the gate columns of
    ``proj``; returns [rows, heads*vdim] of proj's element type."""
    _req(o, "o", torch.float32, 2)
    _req(proj, "proj", None, 2)
    _req(weight, "weight", None, 1)
    T = o.shape[0]
    if o.shape[1] != n_heads * vdim or weight.numel() != vdim or proj.shape[0] != T or g_col + n_heads * vdim > proj.shape[1]:
        raise ValueError("gla_norm_gate: shapes do not agree")
    out = torch.empty((T, n_heads * vdim), dtype=proj.dtype, device=o.device)
    _lib.check(_lib.load().qnn_gla_norm_gate(_p(o), o.shape[1], _p(weight), dt_code(weight), float(eps),
                                             _col_ptr(proj, g_col), proj.shape[1], _p(out), out.shape[1], dt_code(proj),
                                             T, n_heads, vdim, _stream()), "gla_norm_gate")
    return out


# ---- routed experts -----------------------------------------------------------------------------------------

MOE_SCORES = {"sigmoid": 0, "softmax": 1}
GATED_CLAMPED = 2            # the gated activation g' * sigmoid(alpha g') * (u' + 1) of clamped g', u'


def moe_route(x: torch.Tensor, w_router: torch.Tensor, top: int, score: str = "sigmoid", renormalize: bool = False,
              correction: Optional[torch.Tensor] = None, scale: float = 1.0, extra: int = 0,
              groups: Optional[Tuple[int, int]] = None):
    """(expert ids int32 [rows*top], scores float32 [rows*top]): the ``top`` best experts of every row by
    score(x w_router^T), logits and scores in float32, ties to the lower index.  With ``correction`` (float32, one per
    expert) the experts are ranked by score + correction and weighted by the score alone.  ``scale`` multiplies the
    weights (after the renormalisation, if any).  With ``extra`` = n the matrix has n more rows behind the experts';
    their products with the rows come back as a third result, float32 [rows, n], and take no part in the choice.
    ``groups`` = (count, keep): the experts form ``count`` equal groups of neighbours; a group's score is the sum of
    its two largest ranking values, and only experts of the ``keep`` best groups can be chosen."""
    _req(x, "x", None, 2)
    _req(w_router, "w_router", None, 2)
    T, W = x.shape
    E = w_router.shape[0] - int(extra)
    if extra < 0 or E < 1:
        raise ValueError("moe_route: the extra rows leave no expert")
    if w_router.shape[1] != W:
        raise ValueError("moe_route: the router's inner size differs from the rows'")
    if correction is not None:
        _req(correction, "correction", torch.float32, 1)
        if correction.numel() != E:
            raise ValueError("moe_route: a correction per expert")
    sel_e = torch.empty(T * top, dtype=torch.int32, device=x.device)
    sel_w = torch.empty(T * top, dtype=torch.float32, device=x.device)
    more = torch.empty((T, int(extra)), dtype=torch.float32, device=x.device) if extra else None
    count, keep = (int(groups[0]), int(groups[1])) if groups else (1, 1)
    if E % count or not (1 <= keep <= count) or keep * (E // count) < top:
        raise ValueError(f"moe_route: {count} groups of which {keep} are kept do not fit {E} experts and top {top}")
    _lib.check(_lib.load().qnn_moe_route(_p(x), dt_code(x), _p(w_router), dt_code(w_router), T, W, E, int(top),
                                         MOE_SCORES[score], int(renormalize), _p(correction), float(scale), _p(sel_e),
                                         _p(sel_w), int(extra), _p(more), count, keep, _stream()), "moe_route")
    return (sel_e, sel_w, more) if extra else (sel_e, sel_w)


MOE_GROUPED_FROM = 64        # rows per expert (on average) from which prompts take the grouped tcgen05 product


def moe_experts(x: torch.Tensor, sel_e: torch.Tensor, sel_w: torch.Tensor, top: int, w_gate_up: torch.Tensor,
                w_down: torch.Tensor, activation: int, limit: float, alpha: float, weight_on_input: bool,
                shared: Optional[torch.Tensor] = None, grouped: Optional[bool] = None,
                shared_gate: Optional[torch.Tensor] = None, identity: bool = False, gated: bool = True) -> torch.Tensor:
    """sum over a row's chosen experts of down_e(act(gate_e(x'), up_e(x'))) (+ ``shared``), float32 [rows, width].
    ``activation``: ``GATED_CLAMPED`` or the code of a plain gate (act(g) * u, e.g. ``ACT_CODES["silu"]``).
    ``identity``: expert ids from the number of experts on are identity experts (their output is the row itself
    times the score); they take no part in the products.  ``shared_gate`` (float32 [rows]): the shared expert's
    output is multiplied by its sigmoid.
    The score multiplies the expert's input (x' = score * x) or its output.  w_gate_up: [experts, 2*ff, width]
    (gate rows, then up rows); w_down: [experts, width, ff].  Everything stays on the device.
    ``gated`` False: the experts are down_e(act(up_e(x'))); w_gate_up is then [experts, ff, width] (up rows alone) and
    ``activation`` one of ``ACT_CODES``.

    Three kinds of tile: with many rows per expert (prompts; bfloat16, the clamped activation, widths in whole 16-byte
    pieces) the rows are gathered expert after expert and both products are grouped tcgen05 GEMMs over tiles of 128
    rows (``grouped``: None = by size); else tensor-core tiles of 16 or 64 rows (mma.sync) where the widths are whole
    blocks of 32; else plain tiles."""
    _req(x, "x", None, 2)
    _req(w_gate_up, "w_gate_up", x.dtype, 3)
    _req(w_down, "w_down", x.dtype, 3)
    T, W = x.shape
    E, ff2, _ = w_gate_up.shape
    nm = 2 if gated else 1
    ff = ff2 // nm
    if tuple(w_gate_up.shape) != (E, nm * ff, W) or tuple(w_down.shape) != (E, W, ff) or sel_e.numel() != T * top:
        raise ValueError("moe_experts: shapes do not agree")
    if not gated and activation not in ACT_CODES.values():
        raise ValueError("moe_experts: experts without a gate take a plain activation")
    L = _lib.load()
    n = T * top
    if grouped is None:
        grouped = n >= MOE_GROUPED_FROM * E
    grouped = bool(grouped and USE_TCGEN05 and x.dtype == torch.bfloat16
                   and (activation in (GATED_CLAMPED, ACT_CODES["silu"]) or not gated) and W % 8 == 0 and ff % 8 == 0)
    if activation != GATED_CLAMPED:
        limit = 0.0                                 # the grouped product's epilogue reads "no limit" as silu(g) * u
    extra = (shared_gate, (sel_e, sel_w, E, x) if identity else None)
    tile_rows = 128 if grouped else int(L.qnn_moe_tile_rows(n, E, dt_code(x), W, ff))   # else 16, or 64 with many rows each
    max_tiles = int(L.qnn_moe_max_tiles(n, E, tile_rows))
    meta = torch.empty(E + 1 + n + 2 * max_tiles + 1, dtype=torch.int32, device=x.device)
    offsets, perm = meta[:E + 1], meta[E + 1:E + 1 + n]
    tiles, n_tiles = meta[E + 1 + n:E + 1 + n + 2 * max_tiles], meta[E + 1 + n + 2 * max_tiles:]
    _lib.check(L.qnn_moe_plan(_p(sel_e), n, E, tile_rows, _p(offsets), _p(perm), _p(tiles), _p(n_tiles), _stream()),
               "moe_plan")
    hidden = torch.empty((n, ff), dtype=x.dtype, device=x.device)
    ys = torch.empty((n, W), dtype=torch.float32, device=x.device)
    if grouped:
        gathered = torch.empty((n, W), dtype=x.dtype, device=x.device)
        status = _p(_status_word(x.device))
        _lib.check(L.qnn_moe_gather(_p(x), W, _p(perm), _p(sel_w), top, int(weight_on_input), _p(gathered), n, _stream()),
                   "moe_gather")
        # without a gate the epilogue is the activation alone, its code in the place of `scale_output`
        code = L.qnn_moe_tcgen05(_p(gathered), _p(w_gate_up), _p(hidden), n, E, nm * ff, W, EPI_GATED if gated else EPI_ACT,
                                 _p(offsets), _p(perm), _p(sel_w), _p(tiles), _p(n_tiles), max_tiles,
                                 0 if gated else int(activation), float(limit), float(alpha), status, _stream())
        if code == _lib.ERR_UNSUPPORTED:           # sizes the grouped product refuses: the other tiles
            return moe_experts(x, sel_e, sel_w, top, w_gate_up, w_down, activation, limit, alpha, weight_on_input, shared,
                               grouped=False, shared_gate=shared_gate, identity=identity, gated=gated)
        _lib.check(code, "moe_tcgen05")
        _lib.check(L.qnn_moe_tcgen05(_p(hidden), _p(w_down), _p(ys), n, E, W, ff, EPI_NONE, _p(offsets), _p(perm), _p(sel_w),
                                     _p(tiles), _p(n_tiles), max_tiles, int(not weight_on_input), 0.0, 0.0, status,
                                     _stream()), "moe_tcgen05")
        return _moe_sum(L, ys, top, shared, T, W, *extra)
    _lib.check(L.qnn_moe_gate_up(_p(x), dt_code(x), W, _p(w_gate_up), ff, _p(offsets), _p(perm), _p(sel_w), _p(tiles),
                                 _p(n_tiles), max_tiles, tile_rows, top, int(weight_on_input),
                                 int(activation) + (0 if gated else ACT_ALONE), float(limit),
                                 float(alpha), _p(hidden), _stream()), "moe_gate_up")
    _lib.check(L.qnn_moe_down(_p(hidden), dt_code(x), ff, _p(w_down), W, _p(offsets), _p(perm), _p(sel_w), _p(tiles),
                              _p(n_tiles), max_tiles, tile_rows, int(not weight_on_input), _p(ys), _stream()), "moe_down")
    return _moe_sum(L, ys, top, shared, T, W, *extra)


def _moe_sum(L, ys: torch.Tensor, top: int, shared: Optional[torch.Tensor], T: int, W: int,
             shared_gate: Optional[torch.Tensor] = None, identity=None) -> torch.Tensor:
    """out[t] = sum over the row's experts (+ the shared expert's output, gated or not), float32.  ``identity``:
    (expert ids, scores, number of experts, rows) when ids from that number on stand for the row itself."""
    if top == 1 and shared is None and identity is None:
        return ys
    if shared_gate is not None:
        _req(shared_gate, "shared_gate", torch.float32)
        if shared is None or shared_gate.numel() != T:
            raise ValueError("moe_experts: a gate per row, for a shared expert")
    sel_e, sel_w, E, x = identity if identity is not None else (None, None, 0, None)
    if shared is not None:
        _req(shared, "shared", None, 2)
        if tuple(shared.shape) != (T, W):
            raise ValueError("moe_experts: the shared expert's output has another shape")
    out = torch.empty((T, W), dtype=torch.float32, device=ys.device)
    _lib.check(L.qnn_moe_combine(_p(ys), top, _p(shared), dt_code(shared) if shared is not None else 0, _p(shared_gate),
                                 _p(sel_e), _p(sel_w), int(E), _p(x), dt_code(x) if x is not None else 0, _p(out), T, W,
                                 _stream()), "moe_combine")
    return out


def gated_act_clamped(gu: torch.Tensor, limit: float, alpha: float) -> torch.Tensor:
    """[rows, 2*I] (gate | up) -> [rows, I]: g = min(gate, limit), u = clamp(up, -limit, limit),
    g * sigmoid(alpha * g) * (u + 1)."""
    _req(gu, "gate_up", None, 2)
    T, I2 = gu.shape
    out = torch.empty((T, I2 // 2), dtype=gu.dtype, device=gu.device)
    _lib.check(_lib.load().qnn_gated_act_clamped(_p(gu), _p(out), dt_code(gu), T, I2 // 2, float(limit), float(alpha),
                                                 _stream()), "gated_act_clamped")
    return out


# ---- layer norm, post-norm residual stream, branches side by side -------------------------------------------------------

def layernorm(x: torch.Tensor, weight: torch.Tensor, eps: float, out_dtype: torch.dtype) -> torch.Tensor:
    """(x - mean) / sqrt(var + eps) * weight over every row, float32 sums (var: the mean of the squared deviations)."""
    _req(x, "x", None, 2)
    _req(weight, "weight", None, 1)
    T, H = x.shape
    if weight.numel() != H:
        raise ValueError(f"norm weight has {weight.numel()} elements for width {H}")
    out = torch.empty((T, H), dtype=out_dtype, device=x.device)
    _lib.check(_lib.load().qnn_layernorm(_p(x), dt_code(x), _p(weight), dt_code(weight), float(eps), _p(out), dt_code(out),
                                         T, H, _stream()), "layernorm")
    return out


def add_layernorm(resid: torch.Tensor, y: torch.Tensor, weight: torch.Tensor, eps: float,
                  bias: Optional[torch.Tensor] = None, copy_dtype: Optional[torch.dtype] = None) -> Optional[torch.Tensor]:
    """resid += layernorm(y + bias) * weight (float32 stream, in place).  With ``copy_dtype`` the new stream is
    also returned in that element type (the stream itself when that is float32): what the next sublayer reads."""
    _req(resid, "resid", torch.float32, 2)
    _req(y, "y", None, 2)
    _req(weight, "weight", None, 1)
    T, H = resid.shape
    if tuple(y.shape) != (T, H) or weight.numel() != H or (bias is not None and bias.numel() != H):
        raise ValueError("add_layernorm: shapes do not agree")
    copy = None
    if copy_dtype is not None and copy_dtype != torch.float32:
        copy = torch.empty((T, H), dtype=copy_dtype, device=resid.device)
    _lib.check(_lib.load().qnn_add_layernorm(
        _p(resid), _p(y), dt_code(y), _p(bias), dt_code(bias) if bias is not None else 0, _p(weight), dt_code(weight),
        float(eps), _p(copy), dt_code(copy) if copy is not None else 0, T, H, _stream()), "add_layernorm")
    return resid if (copy_dtype == torch.float32) else copy


def _pointer_array(ts):
    return (ctypes.c_void_p * len(ts))(*[t.data_ptr() for t in ts])


def _check_branches(ys, ws, what: str):
    if not (1 <= len(ys) <= 4) or len(ws) != len(ys):
        raise ValueError(f"{what}: one to four branches, a weight each")
    T, H = ys[0].shape
    for y, w in zip(ys, ws):
        _req(y, "branch", ys[0].dtype, 2)
        _req(w, "branch weight", ws[0].dtype, 1)
        if tuple(y.shape) != (T, H) or w.numel() != H:
            raise ValueError(f"{what}: shapes do not agree")
    return T, H


def mean_rmsnorm(ys, ws, eps: float, out_dtype: torch.dtype) -> torch.Tensor:
    """(1/n) sum_b ys[b] / sqrt(mean(ys[b]^2) + eps) * ws[b] over every row: branches that ran side by side, each
    RMS-normed with a plain weight, averaged.  float32 math."""
    T, H = _check_branches(ys, ws, "mean_rmsnorm")
    out = torch.empty((T, H), dtype=out_dtype, device=ys[0].device)
    _lib.check(_lib.load().qnn_mean_rmsnorm(_pointer_array(ys), _pointer_array(ws), len(ys), dt_code(ys[0]), dt_code(ws[0]),
                                            float(eps), _p(out), dt_code(out), T, H, _stream()), "mean_rmsnorm")
    return out


def add_mean_layernorm(resid: torch.Tensor, ys, ws, eps_branch: float, weight: torch.Tensor, eps: float,
                       copy_dtype: Optional[torch.dtype] = None) -> Optional[torch.Tensor]:
    """``add_layernorm(resid, mean_rmsnorm(ys, ws), weight)`` in one kernel; the mean is never rounded."""
    _req(resid, "resid", torch.float32, 2)
    T, H = _check_branches(ys, ws, "add_mean_layernorm")
    if tuple(resid.shape) != (T, H) or weight.numel() != H:
        raise ValueError("add_mean_layernorm: shapes do not agree")
    copy = None
    if copy_dtype is not None and copy_dtype != torch.float32:
        copy = torch.empty((T, H), dtype=copy_dtype, device=resid.device)
    _lib.check(_lib.load().qnn_add_mean_layernorm(
        _p(resid), _pointer_array(ys), _pointer_array(ws), len(ys), dt_code(ys[0]), dt_code(ws[0]), float(eps_branch),
        _p(weight), dt_code(weight), float(eps), _p(copy), dt_code(copy) if copy is not None else 0, T, H, _stream()),
        "add_mean_layernorm")
    return resid if (copy_dtype == torch.float32) else copy


def add_bias_(y: torch.Tensor, bias: torch.Tensor) -> torch.Tensor:
    """y[t, :] += bias, in place."""
    _req(y, "y", None, 2)
    _req(bias, "bias", None, 1)
    if bias.numel() != y.shape[1]:
        raise ValueError("add_bias_: one bias per column")
    _lib.check(_lib.load().qnn_add_bias(_p(y), dt_code(y), _p(bias), dt_code(bias), y.shape[0], y.shape[1], _stream()),
               "add_bias")
    return y


def activation_(x: torch.Tensor, kind: str) -> torch.Tensor:
    """x = act(x) elementwise, in place."""
    _req(x, "x")
    _lib.check(_lib.load().qnn_activation(_p(x), dt_code(x), _p(x), ACT_CODES[kind], x.numel(), _stream()), "activation")
    return x


def activation(x: torch.Tensor, kind: str) -> torch.Tensor:
    """act(x) elementwise, one of ``ACT_CODES`` (float32 math)."""
    _req(x, "x")
    out = torch.empty_like(x)
    _lib.check(_lib.load().qnn_activation(_p(x), dt_code(x), _p(out), ACT_CODES[kind], x.numel(), _stream()), "activation")
    return out


# ---- the rows of a stacked q | k | v product on their way to attention or to a recurrence ----------------------------

def head_prep(src: torch.Tensor, col0: int, n_q: int, n_k: int, n_v_cols: int, head_dim: int, *,
              dst: Optional[torch.Tensor] = None, dst_col0: int = 0, bias: Optional[torch.Tensor] = None,
              q_norm: Optional[torch.Tensor] = None, k_norm: Optional[torch.Tensor] = None, norm_dim: int = 0,
              eps: float = 0.0, rot_dim: int = 0, inv_freq: Optional[torch.Tensor] = None, interleaved: bool = False,
              tok_pos: Optional[torch.Tensor] = None, tok_slot: Optional[torch.Tensor] = None, line=None,
              append: bool = False, norm_whole: bool = False, norm_last: bool = False, plain_norm: bool = False,
              values_are_keys: bool = False) -> torch.Tensor:
    """Bias, an RMS norm per head of queries and keys, rotation and the append to a cache line, in one kernel.

    ``src``: rows that hold, from column ``col0`` on, ``n_q`` query heads and ``n_k`` key heads of ``head_dim`` columns
    and then ``n_v_cols`` value columns.  ``dst`` (default: in place) gets the same layout from ``dst_col0`` on in its
    own element type.  ``bias``: over those columns.  ``q_norm`` / ``k_norm``: weights [norm_dim] of a norm over the
    first ``norm_dim`` columns of each head.  ``rot_dim``: rotated columns per head, by ``tok_pos * inv_freq``, pairs
    (j, j + rot_dim/2) or, ``interleaved``, (2j, 2j + 1).  ``append``: keys and values go to ``line``.
    ``norm_whole``: one norm over all query heads together and one over all key heads together instead of one per
    head (the first ``norm_dim`` columns of every head count); the weights are then [n_q * norm_dim] and
    [n_k * norm_dim].  ``norm_last``: the heads are rotated first and normed then.  ``plain_norm``: the norm has no
    weights (``q_norm`` and ``k_norm`` stay None, ``norm_dim`` says how many columns).  ``values_are_keys``: ``src`` holds
    queries and keys only; the ``n_v_cols`` = ``n_k * head_dim`` value columns of ``dst`` (another buffer) and the
    line's values are the keys as they are after the bias, before norm and rotation."""
    _req(src, "src", None, 2)
    T = src.shape[0]
    width = (n_q + n_k) * head_dim + n_v_cols
    if values_are_keys:
        if dst is None or dst is src or n_v_cols != n_k * head_dim:
            raise ValueError("head_prep: values that are the keys go to another buffer, as many columns as the keys")
        if col0 + (n_q + n_k) * head_dim > src.shape[1]:
            raise ValueError("head_prep: the heads do not fit the rows")
    elif col0 + width > src.shape[1]:
        raise ValueError("head_prep: the heads do not fit the rows")
    if plain_norm and (q_norm is not None or k_norm is not None or norm_dim <= 0):
        raise ValueError("head_prep: a norm without weights takes none, and a number of columns")
    if dst is None:
        dst, dst_col0 = src, col0
    _req(dst, "dst", None, 2)
    if dst.shape[0] != T or dst_col0 + width > dst.shape[1]:
        raise ValueError("head_prep: the destination does not fit")
    if bias is not None:
        _req(bias, "bias", None, 1)
        if bias.numel() != (width - n_v_cols if values_are_keys else width):
            raise ValueError(f"head_prep: the bias has {bias.numel()} elements for {width} columns")
    wdt = 0
    for w, heads in ((q_norm, n_q), (k_norm, n_k)):
        if w is not None:
            _req(w, "norm weight", None, 1)
            if w.numel() != (norm_dim * heads if norm_whole else norm_dim):
                raise ValueError("head_prep: a norm weight per normed column")
            wdt = dt_code(w)
    if norm_whole and ((n_q > 0 and q_norm is None) or (n_k > 0 and k_norm is None)):
        raise ValueError("head_prep: a norm over all heads needs weights for the queries and for the keys")
    if q_norm is not None and k_norm is not None and q_norm.dtype != k_norm.dtype:
        raise TypeError("head_prep: the two norm weights have one element type")
    if rot_dim:
        _req(inv_freq, "inv_freq", torch.float32, 1)
        _req(tok_pos, "tok_pos", torch.int32, 1)
        if inv_freq.numel() != rot_dim // 2 or tok_pos.numel() < T:
            raise ValueError("head_prep: a frequency per rotated pair and a position per row")
    k_pool = v_pool = table = slot_len = None
    max_pages = page_size = ring = 0
    if append:
        if dst.dtype != line.k.dtype:
            raise TypeError("head_prep: rows that go to the cache have the cache's element type")
        _req(tok_slot, "tok_slot", torch.int32, 1)
        k_pool, v_pool = line.k, (line.v if line.has_values else None)
        if tuple(k_pool.shape[1:]) != (n_k, line.page_size, head_dim):
            raise ValueError(f"head_prep: the cache line is {tuple(k_pool.shape)}, the keys [*, {n_k}, {line.page_size}, {head_dim}]")
        table, slot_len, max_pages = line.page_table, line.slot_len, line.page_table.shape[1]
        page_size, ring = line.page_size, line.ring
    _lib.check(_lib.load().qnn_head_prep(
        _col_ptr(src, col0), dt_code(src), src.shape[1], _col_ptr(dst, dst_col0), dt_code(dst), dst.shape[1], T, n_q, n_k,
        n_v_cols, head_dim, int(norm_dim), int(rot_dim), int(interleaved), _p(bias), dt_code(bias) if bias is not None else 0,
        _p(q_norm), _p(k_norm), wdt, float(eps), _p(inv_freq) if rot_dim else None, _p(tok_pos), _p(tok_slot), _p(k_pool),
        _p(v_pool), _p(table), max_pages, page_size, ring, _p(slot_len), int(append),
        int(norm_whole) | (2 if norm_last else 0) | (4 if plain_norm else 0) | (8 if values_are_keys else 0), _stream()),
        "head_prep")
    return dst


# ---- matrix memories with one decay per head ------------------------------------------------------------------------------

def _segment_rows(longest: int, blocks_per_segment: int, device) -> int:
    """Rows of a segment when long sequences are walked in segments side by side: ``blocks_per_segment`` blocks run for
    every segment index (sequences x heads x blocks of value columns), two of them fit an SM, and the walk takes as
    long as a segment has rows times the rounds of blocks.  So: as many segments as fit the device in one round (of at
    least 128 rows each, whole chunks of 16 rows); where not even two fit, the standing 256 rows.  Measured at 9 heads
    of 128 x 257, one prompt of 2048 rows: 8 segments of 256 are 360 blocks, a second round for 64 of them, 0.41 ms;
    6 segments of 352 are 270 blocks in one round."""
    key = str(device)
    if key not in _SM_COUNT:
        dev = torch.device(device)
        _SM_COUNT[key] = torch.cuda.get_device_properties(dev).multi_processor_count if dev.type == "cuda" else 148
    fit = (2 * _SM_COUNT[key]) // max(1, blocks_per_segment)
    if fit < 2:
        return GLA_SEGMENT
    nseg = max(1, min(fit, longest // 128))
    return max(128, (-(-longest // nseg) + 15) // 16 * 16)


def memory_scan(proj: torch.Tensor, q_col: int, k_col: int, v_col: int, decay: torch.Tensor, decay_ld: int,
                key_weight: Optional[torch.Tensor], kw_col: int, q_scale: float, normaliser: bool,
                seq_row0: Optional[torch.Tensor],
                seq_len: Optional[torch.Tensor], slots: torch.Tensor, state: torch.Tensor, n_seqs: int, n_heads: int,
                dim: int, vdim: int, longest: int = 0) -> torch.Tensor:
    """S_t = d_t S_{t-1} + w_t k_t v_t^T, o_t = S_t^T (q_t q_scale) over the rows of every sequence in order, from
    the state of the sequence's slot and back into it; d and w are one float32 number per (row, head).

    ``decay``: float32 with the decay of (row, head) at ``decay[row * decay_ld + head]`` (``decay_ld`` 0: a constant
    per head); ``key_weight``: float32 rows with the weights of a row's heads from column ``kw_col`` on, or None for 1.  ``normaliser``: the state has a column more
    than v, fed 1 in every row (n_t = d_t n_{t-1} + w_t k_t); the result then has vdim + 1 columns per head, the last
    being n_t . q_t.  ``state``: float32 [slots, floats per slot], a slot's [heads, dim, vdim (+1)] first.  Returns
    float32 [rows, heads * (vdim (+1))].  Long sequences run in segments side by side like ``gla_scan``."""
    _req(proj, "proj", None, 2)
    _req(decay, "decay", torch.float32)
    _req(slots, "slots", torch.int32, 1)
    _req(state, "state", torch.float32, 2)
    T = proj.shape[0]
    vs = vdim + (1 if normaliser else 0)
    if state.shape[1] < n_heads * dim * vs or slots.numel() < n_seqs:
        raise ValueError("memory_scan: the state is too small or there are fewer slots than sequences")
    if (seq_row0 is None) != (seq_len is None):
        raise ValueError("memory_scan: first rows and row counts come together")
    if key_weight is not None:
        _req(key_weight, "key_weight", torch.float32, 2)
        if kw_col + n_heads > key_weight.shape[1] or key_weight.shape[0] != T:
            raise ValueError("memory_scan: a key weight per (row, head)")
    ldw = 0 if key_weight is None else key_weight.shape[1]
    out = torch.empty((T, n_heads * vs), dtype=torch.float32, device=proj.device)
    seg_len = nseg = 0
    scratch = seg_decay = None
    if seq_row0 is not None and longest >= GLA_SEGMENTS_FROM and n_seqs * -(-longest // GLA_SEGMENT) <= 65535:
        seg_len = _segment_rows(longest, n_seqs * n_heads * -(-vs // (64 if dim <= 128 else 32)), proj.device)
        if n_seqs * -(-longest // seg_len) > 65535:
            seg_len = GLA_SEGMENT
        nseg = -(-longest // seg_len)
        scratch = torch.zeros((n_seqs * nseg, n_heads * dim * vs), dtype=torch.float32, device=proj.device)
        seg_decay = torch.empty((n_seqs * nseg, n_heads), dtype=torch.float32, device=proj.device)
    _lib.check(_lib.load().qnn_memory_scan(
        _col_ptr(proj, q_col), _col_ptr(proj, k_col), _col_ptr(proj, v_col), proj.shape[1], dt_code(proj), _p(decay),
        int(decay_ld), _col_ptr(key_weight, kw_col) if key_weight is not None else None, ldw, float(q_scale), int(normaliser), _p(seq_row0), _p(seq_len), _p(slots), _p(state),
        state.shape[1], _p(out), out.shape[1], n_seqs, n_heads, dim, vdim, seg_len, nseg, _p(scratch), _p(seg_decay),
        _stream()), "memory_scan", 4 if seg_len else 1)
    return out


def mlstm_gates(pre: torch.Tensor, bias: torch.Tensor, cap: float, seq_row0: Optional[torch.Tensor],
                seq_len: Optional[torch.Tensor], slots: torch.Tensor, state: torch.Tensor, m_offset: int, n_seqs: int,
                n_heads: int) -> torch.Tensor:
    """From the pre-activations ``pre`` (float32 [rows, 2 heads]: input gates, then forget gates) and ``bias`` [2 heads]:
    i = cap tanh(. / cap), f = log sigmoid(cap tanh(. / cap)), the running maximum m_t = max(f_t + m_{t-1}, i_t) from
    the slot's m (``state[slot, m_offset + head]``) and back into it, and per (row, head) the decay
    exp(f_t + m_{t-1} - m_t), the key weight exp(i_t - m_t) and exp(-m_t): float32 [rows, 3 heads]."""
    _req(pre, "pre", torch.float32, 2)
    _req(bias, "bias", None, 1)
    _req(slots, "slots", torch.int32, 1)
    _req(state, "state", torch.float32, 2)
    T = pre.shape[0]
    if pre.shape[1] != 2 * n_heads or bias.numel() != 2 * n_heads or m_offset + n_heads > state.shape[1]:
        raise ValueError("mlstm_gates: shapes do not agree")
    gates = torch.empty((T, 3 * n_heads), dtype=torch.float32, device=pre.device)
    _lib.check(_lib.load().qnn_mlstm_gates(
        _p(pre), pre.shape[1], _p(bias), dt_code(bias), float(cap), _p(seq_row0), _p(seq_len), _p(slots),
        ctypes.c_void_p(state.data_ptr() + 4 * m_offset), state.shape[1], _p(gates), n_heads, n_seqs, _stream()),
        "mlstm_gates")
    return gates


def head_norm_gate(o: torch.Tensor, head_stride: int, n_heads: int, vdim: int, eps: float, gate: Optional[torch.Tensor],
                   g_col: int, gate_act: str, weight: Optional[torch.Tensor] = None, den: Optional[torch.Tensor] = None,
                   den_col: int = 0, out_dtype: Optional[torch.dtype] = None) -> torch.Tensor:
    """Per head of ``o`` (float32 [rows, heads * head_stride]): divided by max(|o[vdim]|, den) + 1e-6 when ``den``
    (float32 rows, one number per head from column ``den_col`` on) is given; an RMS norm over the first ``vdim``
    columns; times ``weight`` ([vdim]: shared by the heads, [heads * vdim]: per column of the row, None: none); times
    silu or sigmoid of the gate columns of ``gate`` (from ``g_col`` on).  Returns [rows, heads * vdim] of gate's type.
    ``gate_act`` "none" (``gate`` None): no gate, the result has ``out_dtype``."""
    _req(o, "o", torch.float32, 2)
    T = o.shape[0]
    if gate_act == "none":
        if gate is not None or out_dtype is None:
            raise ValueError("head_norm_gate: without a gate, no gate rows and an element type for the result")
        if o.shape[1] != n_heads * head_stride:
            raise ValueError("head_norm_gate: shapes do not agree")
    else:
        _req(gate, "gate", None, 2)
        if o.shape[1] != n_heads * head_stride or gate.shape[0] != T or g_col + n_heads * vdim > gate.shape[1]:
            raise ValueError("head_norm_gate: shapes do not agree")
    mode = 0
    if weight is not None:
        _req(weight, "weight", None, 1)
        mode = 1 if weight.numel() == vdim and n_heads > 1 else (2 if weight.numel() == n_heads * vdim else -1)
        if mode < 0:
            raise ValueError("head_norm_gate: the weight has vdim or heads * vdim elements")
    if den is not None:
        _req(den, "den", torch.float32, 2)
    out = torch.empty((T, n_heads * vdim), dtype=gate.dtype if gate is not None else out_dtype, device=o.device)
    _lib.check(_lib.load().qnn_head_norm_gate(
        _p(o), o.shape[1], head_stride, _col_ptr(den, den_col) if den is not None else None,
        den.shape[1] if den is not None else 0, _p(weight), dt_code(weight) if weight is not None else 0, mode, float(eps),
        _col_ptr(gate, g_col) if gate is not None else None, gate.shape[1] if gate is not None else 0,
        {"silu": 0, "sigmoid": 1, "none": 2}[gate_act], _p(out), out.shape[1], dt_code(out), T,
        n_heads, vdim, _stream()), "head_norm_gate")
    return out


# ---- norms in groups, sublayers side by side, learned positions, gates per element -----------------------------------------

def group_rmsnorm(x: torch.Tensor, weight: torch.Tensor, eps: float, groups: int, out_dtype: torch.dtype) -> torch.Tensor:
    """RMS norm in ``groups`` equal consecutive pieces of every row, each divided by its own
    sqrt(mean(piece^2) + eps), the whole times ``weight``; float32 sums."""
    _req(x, "x", None, 2)
    _req(weight, "weight", None, 1)
    T, H = x.shape
    if weight.numel() != H or groups < 1 or H % groups:
        raise ValueError(f"group_rmsnorm: {weight.numel()} weights, {groups} groups for width {H}")
    out = torch.empty((T, H), dtype=out_dtype, device=x.device)
    _lib.check(_lib.load().qnn_group_rmsnorm(_p(x), dt_code(x), _p(weight), dt_code(weight), float(eps), int(groups), _p(out),
                                             dt_code(out), T, H, _stream()), "group_rmsnorm")
    return out


def add2_group_rmsnorm(resid: torch.Tensor, a: Optional[torch.Tensor], b: Optional[torch.Tensor] = None,
                       w_next: Optional[torch.Tensor] = None, eps: float = 0.0, groups: int = 1,
                       out_dtype: Optional[torch.dtype] = None) -> Optional[torch.Tensor]:
    """resid += a + b (float32 stream, in place; either may be None); returns the grouped norm of the new stream
    with ``w_next`` when that is given, in one kernel."""
    _req(resid, "resid", torch.float32, 2)
    T, H = resid.shape
    for name, t in (("a", a), ("b", b)):
        if t is not None:
            _req(t, name, None, 2)
            if tuple(t.shape) != (T, H):
                raise ValueError("add2_group_rmsnorm: shapes do not agree")
    out = None
    if w_next is not None:
        _req(w_next, "w_next", None, 1)
        if w_next.numel() != H or groups < 1 or H % groups:
            raise ValueError(f"add2_group_rmsnorm: {w_next.numel()} weights, {groups} groups for width {H}")
        out = torch.empty((T, H), dtype=out_dtype, device=resid.device)
    _lib.check(_lib.load().qnn_add2_group_rmsnorm(
        _p(resid), _p(a), dt_code(a) if a is not None else 0, _p(b), dt_code(b) if b is not None else 0, _p(w_next),
        dt_code(w_next) if w_next is not None else 0, float(eps), int(groups), _p(out),
        dt_code(out) if out is not None else 0, T, H, _stream()), "add2_group_rmsnorm")
    return out


def embed_pos(tokens: torch.Tensor, table: torch.Tensor, scale: float, pos_table: torch.Tensor, tok_pos: torch.Tensor,
              w_norm: Optional[torch.Tensor] = None, eps: float = 0.0, groups: int = 1,
              out_dtype: Optional[torch.dtype] = None):
    """table[token] * scale + pos_table[position] as float32 rows; with ``w_norm`` also their grouped norm, in the
    same kernel: (rows, normed rows or None)."""
    _req(tokens, "tokens", torch.int32, 1)
    _req(tok_pos, "tok_pos", torch.int32, 1)
    _req(table, "table", None, 2)
    _req(pos_table, "pos_table", None, 2)
    T, (V, H) = tokens.numel(), table.shape
    if pos_table.shape[1] != H or tok_pos.numel() < T:
        raise ValueError("embed_pos: the position table has another width, or positions are missing")
    out = torch.empty((T, H), dtype=torch.float32, device=tokens.device)
    normed = None
    if w_norm is not None:
        _req(w_norm, "w_norm", None, 1)
        if w_norm.numel() != H or groups < 1 or H % groups:
            raise ValueError(f"embed_pos: {w_norm.numel()} weights, {groups} groups for width {H}")
        normed = torch.empty((T, H), dtype=out_dtype, device=tokens.device)
    _lib.check(_lib.load().qnn_embed_pos(
        _p(tokens), _p(table), dt_code(table), float(scale), _p(pos_table), dt_code(pos_table), _p(tok_pos),
        pos_table.shape[0], _p(out), _p(w_norm), dt_code(w_norm) if w_norm is not None else 0, float(eps), int(groups),
        _p(normed), dt_code(normed) if normed is not None else 0, T, H, V, _stream()), "embed_pos")
    return out, normed


def sigmoid_gate_(o: torch.Tensor, g: torch.Tensor, g_col0: int = 0) -> torch.Tensor:
    """o[t, c] *= sigmoid(g[t, g_col0 + c]) in place: a gate per element, its logits in columns of rows that may be
    wider (a piece of a stacked product)."""
    _req(o, "o", None, 2)
    _req(g, "g", None, 2)
    T, N = o.shape
    if g.shape[0] != T or g_col0 + N > g.shape[1]:
        raise ValueError("sigmoid_gate_: shapes do not agree")
    _lib.check(_lib.load().qnn_sigmoid_gate(_p(o), dt_code(o), N, _col_ptr(g, g_col0), dt_code(g), g.shape[1], T, N,
                                            _stream()), "sigmoid_gate")
    return o


def xielu_(x: torch.Tensor, ap: float, an: float) -> torch.Tensor:
    """In place: x > 0: ap x^2 + x / 2; x <= 0: an (exp(x) - 1 - x) + x / 2."""
    _req(x, "x")
    _lib.check(_lib.load().qnn_xielu(_p(x), dt_code(x), float(ap), float(an), _p(x), x.numel(), _stream()), "xielu")
    return x


# ---- dynamic tanh ------------------------------------------------------------------------------------------------------

def dyt(x: torch.Tensor, alpha: float, weight: torch.Tensor, bias: torch.Tensor, out_dtype: torch.dtype) -> torch.Tensor:
    """tanh(alpha x) * weight + bias over every row, float32 math."""
    _req(x, "x", None, 2)
    _req(weight, "weight", None, 1)
    _req(bias, "bias", None, 1)
    T, H = x.shape
    if weight.numel() != H or bias.numel() != H:
        raise ValueError("dyt: a weight and a bias per column")
    out = torch.empty((T, H), dtype=out_dtype, device=x.device)
    _lib.check(_lib.load().qnn_dyt(_p(x), dt_code(x), float(alpha), _p(weight), dt_code(weight), _p(bias), dt_code(bias),
                                   _p(out), dt_code(out), T, H, _stream()), "dyt")
    return out


def add_dyt(resid: torch.Tensor, a: Optional[torch.Tensor], c: Optional[torch.Tensor] = None, alpha: float = 0.0,
            weight: Optional[torch.Tensor] = None, bias: Optional[torch.Tensor] = None,
            out_dtype: Optional[torch.dtype] = None) -> Optional[torch.Tensor]:
    """resid += a (+ c) in place (float32 stream; ``a`` a sublayer's output, ``c`` float32 rows; either may be None), and,
    with ``weight``, tanh(alpha resid) * weight + bias of the new stream in the same kernel."""
    _req(resid, "resid", torch.float32, 2)
    T, H = resid.shape
    for t, what in ((a, "a"), (c, "c")):
        if t is not None:
            _req(t, what, torch.float32 if what == "c" else None, 2)
            if tuple(t.shape) != (T, H):
                raise ValueError("add_dyt: shapes do not agree")
    out = None
    if weight is not None:
        _req(weight, "weight", None, 1)
        _req(bias, "bias", None, 1)
        if weight.numel() != H or bias.numel() != H or out_dtype is None:
            raise ValueError("add_dyt: a weight and a bias per column, and an element type for the result")
        out = torch.empty((T, H), dtype=out_dtype, device=resid.device)
    _lib.check(_lib.load().qnn_add_dyt(_p(resid), _p(a), dt_code(a) if a is not None else 0, _p(c), float(alpha), _p(weight),
                                       dt_code(weight) if weight is not None else 0, _p(bias),
                                       dt_code(bias) if bias is not None else 0, _p(out),
                                       dt_code(out) if out is not None else 0, T, H, _stream()), "add_dyt")
    return out


def embed_dyt(tokens: torch.Tensor, table: torch.Tensor, scale: float, alpha: float, weight: torch.Tensor,
              bias: torch.Tensor, out_dtype: torch.dtype):
    """(x, dyt(x)) with x = table[tokens] * scale (float32), in one kernel."""
    _req(tokens, "tokens", torch.int32, 1)
    _req(table, "table", None, 2)
    T, (V, H) = tokens.numel(), table.shape
    x = torch.empty((T, H), dtype=torch.float32, device=table.device)
    out = torch.empty((T, H), dtype=out_dtype, device=table.device)
    _lib.check(_lib.load().qnn_embed_dyt(_p(tokens), _p(table), dt_code(table), float(scale), float(alpha), _p(weight),
                                         dt_code(weight), _p(bias), dt_code(bias), _p(x), _p(out), dt_code(out), T, H, V,
                                         _stream()), "embed_dyt")
    return x, out


# ---- gates of a matrix memory whose forget gate also writes ---------------------------------------------------------------

def bounded_gates(rows: torch.Tensor, q_col: int, n_q: int, f_col: int, n_f: int, bias: Optional[torch.Tensor],
                  lower: Optional[torch.Tensor]) -> torch.Tensor:
    """In place: silu over the ``n_q`` query columns of ``rows`` (from ``q_col``).  Returns the forget gates
    f = lower + (1 - lower) * sigmoid(z + bias), float32 [rows, n_f], of the pre-activations z in the ``n_f`` columns from
    ``f_col`` (``bias`` and ``lower`` one per channel; None: 0)."""
    _req(rows, "rows", None, 2)
    T = rows.shape[0]
    if q_col + n_q > rows.shape[1] or f_col + n_f > rows.shape[1]:
        raise ValueError("bounded_gates: the columns do not fit the rows")
    for t in (bias, lower):
        if t is not None:
            _req(t, "bias / lower", None, 1)
            if t.numel() != n_f:
                raise ValueError("bounded_gates: one bias and one lower bound per channel")
    f = torch.empty((T, n_f), dtype=torch.float32, device=rows.device)
    _lib.check(_lib.load().qnn_bounded_gates(_p(rows), dt_code(rows), rows.shape[1], T, q_col, n_q, f_col, n_f, _p(bias),
                                             dt_code(bias) if bias is not None else 0, _p(lower),
                                             dt_code(lower) if lower is not None else 0, _p(f), _stream()), "bounded_gates")
    return f


# ---- attention with sigmoid weights and mixed heads ----------------------------------------------------------------------

MASKS = {"causal": 0, "window": 1, "chunk": 2}
SIGATTN_TENSOR_CORES = os.environ.get("QNN_SIGATTN", "") != "generic"


def sigmoid_attention_refusal(dtype: torch.dtype, n_heads: int, n_kv: int, head_dim: int) -> Optional[str]:
    """Why the sigmoid attention kernel does not take these sizes, or None."""
    if n_kv < 1 or n_heads % n_kv:
        return f"{n_kv} kv heads do not divide {n_heads} heads"
    if not _lib.load().qnn_sigattn_supports(1 if dtype == torch.bfloat16 else 0, n_heads, n_kv, head_dim):
        return (f"{n_heads} heads of {head_dim} columns with {n_kv} kv heads are beyond the sigmoid attention kernel "
                f"(heads x head size up to 4096, a tile of keys within shared memory)")
    return None


def sigmoid_attention(qkv: torch.Tensor, n_heads: int, n_kv: int, head_dim: int, tok_pos: torch.Tensor,
                      tok_row0: Optional[torch.Tensor], tok_slot: Optional[torch.Tensor], line, own_rows: bool,
                      mask: str, mask_size: int, scale: float, pb: Optional[torch.Tensor], talk: Optional[torch.Tensor],
                      gate: Optional[torch.Tensor], gate_col: int = 0, splits: int = 1,
                      seq_row0: Optional[torch.Tensor] = None, seq_len: Optional[torch.Tensor] = None,
                      longest: int = 0) -> torch.Tensor:
    """o_h(i) = sigmoid(gate[i, h]) * sum_j (sum_g talk[h, g] sigmoid(scale q_g(i) . k(j) + pb[g])) v(j) over the keys j
    that position i sees (``mask``: "causal", "window" or "chunk" of ``mask_size``).  ``qkv``: the step's packed q | k | v
    rows.  ``own_rows``: keys at or after the position of a sequence's first row of this step are read from ``qkv``,
    earlier ones from the cache ``line``; False: every key from the line (a decode step after its append).  ``gate``:
    rows whose columns ``gate_col`` .. hold one logit per head (None: no gate).  ``splits``: key ranges per token that
    run as separate blocks and are summed in order.  ``seq_row0`` / ``seq_len`` / ``longest``: given for whole prompts
    (every sequence starts at position 0): bfloat16 rows with head sizes 32 to 256 then run on the tensor cores
    (``QNN_SIGATTN=generic`` keeps the plain kernel).  Returns [rows, heads * head_dim] of qkv's type."""
    _req(qkv, "qkv", None, 2)
    _req(tok_pos, "tok_pos", torch.int32, 1)
    T = qkv.shape[0]
    H, G, D = n_heads, n_kv, head_dim
    if qkv.shape[1] < (H + 2 * G) * D or tok_pos.numel() < T:
        raise ValueError("sigmoid_attention: the rows are narrower than q | k | v, or positions are missing")
    if pb is not None:
        _req(pb, "pb", torch.float32, 1)
    if talk is not None:
        _req(talk, "talk", torch.float32, 2)
    if (pb is not None and pb.numel() != H) or (talk is not None and tuple(talk.shape) != (H, H)):
        raise ValueError("sigmoid_attention: a bias per head and a mixing matrix [heads, heads]")
    k_pool = v_pool = table = None
    max_pages = page_size = ring = 0
    if line is not None:
        k_pool, v_pool, table = line.k, line.v, line.page_table
        if k_pool.dtype != qkv.dtype or tuple(k_pool.shape[1:]) != (G, line.page_size, D):
            raise ValueError("sigmoid_attention: the cache line does not fit the keys")
        max_pages, page_size, ring = table.shape[1], line.page_size, line.ring
    elif not own_rows:
        raise ValueError("sigmoid_attention: keys come from the step's rows or from a cache line")
    if gate is not None:
        _req(gate, "gate", None, 2)
        if gate.shape[0] != T or gate_col + H > gate.shape[1]:
            raise ValueError("sigmoid_attention: a gate logit per row and head")
    out = torch.empty((T, H * D), dtype=qkv.dtype, device=qkv.device)
    if own_rows and seq_row0 is not None and longest > 0 and qkv.dtype == torch.bfloat16 and SIGATTN_TENSOR_CORES:
        _req(seq_row0, "seq_row0", torch.int32, 1)
        _req(seq_len, "seq_len", torch.int32, 1)
        # a query tile that sees many key tiles has them walked in ranges, by blocks of their own
        per_range = ctypes.c_int(0)
        ranges = _lib.load().qnn_sigattn_prefill_ranges(int(longest), MASKS[mask], int(mask_size or 0), H, G, D,
                                                        ctypes.byref(per_range))
        part = torch.empty((ranges, T, H * D), dtype=torch.float32, device=qkv.device) if ranges > 1 else None
        code = _lib.load().qnn_sigattn_prefill_mma(
            _p(qkv), qkv.shape[1], _p(seq_row0), _p(seq_len), seq_row0.numel(), int(longest), MASKS[mask], int(mask_size or 0),
            float(scale), _p(pb), _p(talk), _col_ptr(gate, gate_col) if gate is not None else None,
            dt_code(gate) if gate is not None else 0, gate.shape[1] if gate is not None else 0, _p(out), out.shape[1],
            H, G, D, _p(part), T, _stream())
        if code != _lib.ERR_UNSUPPORTED:           # sizes it refuses: the plain kernel below
            _lib.check(code, "sigmoid_attention (tensor cores)")
            return out
    splits = max(1, int(splits))
    partial = torch.empty((splits, T, H * D), dtype=torch.float32, device=qkv.device) if splits > 1 else None
    _lib.check(_lib.load().qnn_sigattn(
        _p(qkv), dt_code(qkv), qkv.shape[1], _p(k_pool), _p(v_pool), _p(table), max_pages, page_size, ring, _p(tok_pos),
        _p(tok_row0), _p(tok_slot), int(own_rows), MASKS[mask], int(mask_size or 0), float(scale), _p(pb), _p(talk),
        _col_ptr(gate, gate_col) if gate is not None else None, dt_code(gate) if gate is not None else 0,
        gate.shape[1] if gate is not None else 0, _p(out), out.shape[1], _p(partial), splits, T, H, G, D, _stream()),
        "sigmoid_attention", 2 if splits > 1 else 1)
    return out
