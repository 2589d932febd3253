"""Python face of the engine's CUDA kernels.

Every function here launches hand-written sm_100a kernels from `csrc/` on the current CUDA
stream of torch and returns torch tensors.  There is no other implementation behind them: a
tensor that is not on a CUDA device, a missing compiler or an unsupported size raises.
Matrix products with more than a few rows are the one exception to "hand-written": `linear` then calls
the library GEMM that torch binds (cuBLAS), in bfloat16 with float32 accumulation or in true float32
(TF32 off), as the reference does for every projection (F.linear in mini_sglang/layers/linear.py).  Up to
SMALL_M_MAX rows go to this engine's weight-streaming kernel.  The reference's own kernels for the
other operations come from sgl_kernel / flash-attn (mini_sglang/layers/layernorm.py:39-50,
mini_sglang/layers/rotary_embedding.py, mini_sglang/layers/attn/fa3_attn_backend.py).
"""

from __future__ import annotations

import ctypes
import os
from typing import Optional, Sequence, Tuple

import torch

from .csrc import build as _build

_DT = {torch.float32: 0, torch.bfloat16: 1}
_ERR = {1: "element type not handled", 2: "size not supported by the kernel", 3: "kernel launch failed",
        4: "pointer not aligned"}

c_void_p, c_int, c_float, c_ll, c_ull = ctypes.c_void_p, ctypes.c_int, ctypes.c_float, ctypes.c_longlong, ctypes.c_ulonglong


class KernelError(RuntimeError):
    pass


LAUNCHES = 0      # kernels of this engine launched (or recorded into a graph) so far


def _check(code: int, what: str) -> None:
    global LAUNCHES
    LAUNCHES += 1
    if code != 0:
        detail = ""
        if code == 3:
            detail = f" ({torch.cuda.get_device_name()}: the kernels are built for sm_100a only)"
        raise KernelError(f"{what}: {_ERR.get(code, f'error {code}')}{detail}")


def _ptr(t: Optional[torch.Tensor]) -> Optional[int]:
    if t is None:
        return None
    return t.data_ptr()


def _need_cuda(*tensors: Optional[torch.Tensor]) -> None:
    for t in tensors:
        if t is not None and not t.is_cuda:
            raise KernelError("the engine's kernels run on a CUDA device only; got a tensor on " + str(t.device))


def _stream() -> int:
    return torch.cuda.current_stream().cuda_stream


def _dt(t: torch.Tensor) -> int:
    try:
        return _DT[t.dtype]
    except KeyError:
        raise KernelError(f"dtype {t.dtype} is not handled; the engine computes in bfloat16 or float32") from None


_common = None
_attn = {}


def _lib():
    global _common
    if _common is None:
        lib = _build.common_library()
        lib.msgl_embedding.argtypes = [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_void_p]
        lib.msgl_resolve_ids.argtypes = [c_void_p, c_void_p, c_int, c_int, c_void_p]
        lib.msgl_table_delta.argtypes = [c_void_p, c_int, c_void_p, c_int, c_void_p]
        lib.msgl_decode_meta.argtypes = [c_void_p] * 4 + [c_int, c_int, c_void_p, c_int, c_int, c_int, c_int] + [c_void_p] * 9 + [c_int, c_void_p, c_void_p, c_void_p, c_int,
                                         c_void_p]
        lib.msgl_rmsnorm.argtypes = [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_float, c_void_p,
                                     c_int, c_int, c_int, c_void_p]
        lib.msgl_qknorm_rope_kvwrite.argtypes = [c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_int,
                                                 c_float, c_void_p, c_int, c_int, c_void_p, c_void_p, c_void_p,
                                                 c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_void_p]
        lib.msgl_swiglu.argtypes = [c_void_p, c_void_p, c_int, c_int, c_int, c_void_p]
        lib.msgl_cast_from_f32.argtypes = [c_void_p, c_void_p, c_ll, c_int, c_void_p]
        lib.msgl_gemm_small_m.argtypes = [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_ll, c_ll, c_int,
                                          c_int, c_void_p]
        lib.msgl_gemm_tc.argtypes = [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_ll, c_ll, c_int, c_void_p,
                                     c_void_p]
        lib.msgl_gemm_tc2.argtypes = lib.msgl_gemm_tc.argtypes
        lib.msgl_gemm_tc2_splitk.argtypes = [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_ll, c_ll, c_int, c_int,
                                             c_void_p, c_void_p, c_void_p]
        lib.msgl_gemm_tc2_splits.argtypes = [c_int, c_int, c_int, c_int]
        lib.msgl_gemm_tc2_splits.restype = c_int
        lib.msgl_sample.argtypes = [c_void_p, c_int, c_int, c_ll, c_void_p, c_void_p, c_void_p, c_ull, c_void_p,
                                    c_void_p, c_void_p, c_void_p, c_int, c_void_p]
        _common = lib
    return _common


def _attn_lib(head_dim: int):
    hd = head_dim if head_dim in _build.MMA_HEAD_DIMS else 128
    lib = _attn.get(hd)
    if lib is None:
        lib = _build.attention_library(hd)
        lib.msgl_attention.argtypes = [c_void_p] * 10 + [c_int] * 9 + [c_float] + [c_int] * 6 + [c_void_p, c_void_p, c_int, c_void_p]
        lib.msgl_attention_combine.argtypes = [c_void_p] * 5 + [c_int] * 5 + [c_void_p]
        lib.msgl_attention_tc.argtypes = [c_void_p] * 7 + [c_int] * 8 + [c_float] + [c_int] * 5 + [c_void_p, c_void_p]
        lib.msgl_attention_head_dim.restype = c_int
        _attn[hd] = lib
    return lib


def warm_up(head_dims=()) -> None:
    """Build and load the libraries a model needs (compiles at the first call)."""
    _lib()
    for hd in head_dims:
        _attn_lib(hd)


# ---------------------------------------------------------------------------------------

def embedding(ids: torch.Tensor, table: torch.Tensor, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """ids int32 [T], table [V, H] -> float32 [T, H] (the residual stream starts in float32)."""
    _need_cuda(ids, table)
    T, (V, H) = ids.numel(), table.shape
    assert ids.dtype == torch.int32 and table.is_contiguous()
    if out is None:
        out = torch.empty((T, H), dtype=torch.float32, device=table.device)
    _check(_lib().msgl_embedding(_ptr(ids), _ptr(table), _ptr(out), T, H, V, _dt(table), _stream()), "embedding")
    return out


def resolve_ids(ids: torch.Tensor, prev: torch.Tensor) -> None:
    """In place: ids[t] = prev[-1 - ids[t]] where ids[t] < 0 (int32, on the device)."""
    _need_cuda(ids, prev)
    assert ids.dtype == torch.int32 and prev.dtype == torch.int32 and ids.is_contiguous() and prev.is_contiguous()
    _check(_lib().msgl_resolve_ids(_ptr(ids), _ptr(prev), ids.numel(), prev.numel(), _stream()), "resolve_ids")


def table_delta(deltas: torch.Tensor, n_records: int, table: torch.Tensor) -> None:
    """Rows of the device copy of a cache group's block tables, brought up to date: deltas = [n, (slot, count, offset) x n,
    page ids ...] int32 on the device; table int32 [slots, pages per request]."""
    _need_cuda(deltas, table)
    assert deltas.dtype == torch.int32 and table.dtype == torch.int32 and table.is_contiguous()
    _check(_lib().msgl_table_delta(_ptr(deltas), n_records, _ptr(table), table.shape[1], _stream()), "table_delta")


def decode_meta(ids: torch.Tensor, slots_in: torch.Tensor, pos: torch.Tensor, nsplit_in: torch.Tensor, B: int, b: int,
                table: torch.Tensor, page_size: int, mp: int, common: bool, *, input_ids, positions, token_req, q_start, kv_len,
                slots, out_loc, nsplit, block_table, order, window: int = 0, even_in: Optional[torch.Tensor] = None,
                even_out: Optional[torch.Tensor] = None) -> None:
    """The step fields of a decode batch of B requests (captured size b) written on the device from (token id, slot,
    position) per request and the device copy of the block tables; see csrc/elementwise.cu.  `order` receives the rows
    by falling number of keys per kv split (what the attention launch walks first); `even_in` (the even cut of the step's
    keys, made by the host) is copied to `even_out` as it is."""
    _need_cuda(ids, slots_in, pos, nsplit_in, table, input_ids, block_table)
    code = _lib().msgl_decode_meta(_ptr(ids), _ptr(slots_in), _ptr(pos), _ptr(nsplit_in), B, b, _ptr(table), table.shape[1], page_size,
                                   mp, int(common), _ptr(input_ids), _ptr(positions), _ptr(token_req), _ptr(q_start), _ptr(kv_len),
                                   _ptr(slots), _ptr(out_loc), _ptr(nsplit), _ptr(block_table), int(window), _ptr(order),
                                   _ptr(even_in), _ptr(even_out), even_in.numel() if even_in is not None else 0, _stream())
    _check(code, "decode_meta")


def rmsnorm(weight: torch.Tensor, eps: float, *, x: Optional[torch.Tensor] = None,
            residual: Optional[torch.Tensor] = None, residual_out: Optional[torch.Tensor] = None,
            rows: Optional[torch.Tensor] = None, out_dtype: Optional[torch.dtype] = None,
            out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """y = rmsnorm(residual + x) * weight, the sum and the norm in float32.

    x: activation dtype [N, H] or None; residual: float32 [N, H] or None; residual_out: float32
    buffer that receives the sum (may be `residual` itself when `rows` is None);
    rows: int32 [R] picks input rows (outputs are then [R, H]).  Returns y in `out_dtype`
    (default: x's dtype)."""
    _need_cuda(weight, x, residual, residual_out, rows)
    src = x if x is not None else residual
    assert src is not None and src.dim() == 2 and src.is_contiguous()
    H = src.shape[1]
    n_out = rows.numel() if rows is not None else src.shape[0]
    if out_dtype is None:
        out_dtype = x.dtype if x is not None else torch.float32
    if x is not None:
        assert x.dtype == out_dtype
    if residual is not None:
        assert residual.dtype == torch.float32 and residual.shape[1] == H
    assert weight.numel() == H and weight.dtype in (torch.float32, torch.bfloat16)
    if out is None:
        out = torch.empty((n_out, H), dtype=out_dtype, device=src.device)
    code = _lib().msgl_rmsnorm(_ptr(x), _ptr(residual), _ptr(residual_out), _ptr(rows), _ptr(weight),
                               int(weight.dtype == torch.float32), float(eps), _ptr(out), n_out, H, _DT[out_dtype],
                               _stream())
    _check(code, "rmsnorm")
    return out


def qknorm_rope_kvwrite(qkv: torch.Tensor, positions: torch.Tensor, n_q: int, n_kv: int, d: int, *,
                        q_weight: Optional[torch.Tensor], k_weight: Optional[torch.Tensor], eps: float,
                        rope_table: Optional[torch.Tensor], out_loc: Optional[torch.Tensor],
                        k_cache: Optional[torch.Tensor], v_cache: Optional[torch.Tensor], page_size: int,
                        q_out: Optional[torch.Tensor] = None, interleaved: bool = False) -> torch.Tensor:
    """Per-head RMSNorm of q and k (if weights are given), rotary encoding from `rope_table`
    [max_pos, rot] float32 = cos | sin (if given; the first `rot` elements of a head are rotated in halves, element i
    against i + rot/2, or with `interleaved` in neighbouring pairs 2p, 2p+1), k and v written to the paged cache at token
    slots `out_loc` (if a cache is given), q returned as [T, n_q, d]."""
    _need_cuda(qkv, positions, q_weight, k_weight, rope_table, out_loc, k_cache, v_cache)
    T = qkv.shape[0]
    assert qkv.dim() == 2 and qkv.stride(1) == 1 and qkv.shape[1] == (n_q + 2 * n_kv) * d
    assert positions.numel() == T and positions.dtype == torch.int32
    if out_loc is not None:
        assert out_loc.numel() == T and out_loc.dtype == torch.int32, "one cache slot per token"
    if q_out is None:
        q_out = torch.empty((T, n_q, d), dtype=qkv.dtype, device=qkv.device)
    w_f32 = 0
    if q_weight is not None:
        assert k_weight is not None and q_weight.dtype == k_weight.dtype
        w_f32 = int(q_weight.dtype == torch.float32)
    rot, max_pos = (rope_table.shape[1], rope_table.shape[0]) if rope_table is not None else (0, 0)
    if rope_table is not None:
        assert rope_table.dtype == torch.float32 and rope_table.is_contiguous()
    if k_cache is not None:
        assert k_cache.dtype == qkv.dtype and v_cache.dtype == qkv.dtype
    code = _lib().msgl_qknorm_rope_kvwrite(_ptr(qkv), qkv.stride(0), _ptr(positions), _ptr(out_loc), _ptr(q_weight),
                                           _ptr(k_weight), w_f32, float(eps), _ptr(rope_table), rot, max_pos,
                                           _ptr(q_out), _ptr(k_cache), _ptr(v_cache), page_size, n_q, n_kv, d, T,
                                           _dt(qkv), int(bool(interleaved)), _stream())
    _check(code, f"qknorm_rope_kvwrite (head size {d})")
    return q_out


def swiglu(gate_up: torch.Tensor, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """[T, 2I] (gate first) -> [T, I] = silu(gate) * up."""
    _need_cuda(gate_up)
    assert gate_up.dim() == 2 and gate_up.is_contiguous() and gate_up.shape[1] % 2 == 0
    T, I = gate_up.shape[0], gate_up.shape[1] // 2
    if out is None:
        out = torch.empty((T, I), dtype=gate_up.dtype, device=gate_up.device)
    _check(_lib().msgl_swiglu(_ptr(gate_up), _ptr(out), T, I, _dt(gate_up), _stream()), "swiglu")
    return out


def cast_from_f32(x: torch.Tensor, dtype: torch.dtype) -> torch.Tensor:
    _need_cuda(x)
    assert x.dtype == torch.float32 and x.is_contiguous()
    out = torch.empty(x.shape, dtype=dtype, device=x.device)
    _check(_lib().msgl_cast_from_f32(_ptr(x), _ptr(out), x.numel(), _DT[dtype], _stream()), "cast")
    return out


_sample_scratch = {}          # per device: (part, row_max, tickets)
_sm_counts = {}


def sm_count(device) -> int:
    """Number of SMs of a CUDA device (asked once)."""
    dev = torch.device(device)
    idx = dev.index if dev.index is not None else torch.cuda.current_device()
    if idx not in _sm_counts:
        _sm_counts[idx] = int(torch.cuda.get_device_properties(idx).multi_processor_count)
    return _sm_counts[idx]



def _sample_buffers(device, rows: int, slices: int):
    """Scratch of the sampling kernels, kept per device and grown on demand.  The tickets are zero between calls:
    the block that takes a row's last ticket puts it back to zero."""
    key = (device.type, device.index if device.index is not None else torch.cuda.current_device())
    part, row_max, tickets = _sample_scratch.get(key, (None, None, None))
    if part is None or part.numel() < rows * slices * 2 or tickets.numel() < rows:
        n_rows = max(rows, 256, tickets.numel() if tickets is not None else 0)
        part = torch.empty(max(rows * slices * 2, 256 * 64 * 2), dtype=torch.float32, device=device)
        row_max = torch.empty(n_rows, dtype=torch.float32, device=device)
        tickets = torch.zeros(n_rows, dtype=torch.int32, device=device)
        _sample_scratch[key] = (part, row_max, tickets)
    return part, row_max, tickets


def sample(logits: torch.Tensor, temperatures: Optional[torch.Tensor], row_keys: Optional[torch.Tensor],
           steps: Optional[torch.Tensor], seed: int, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """float32 logits [N, V] -> int32 token ids [N]; greedy where temperature is 0."""
    _need_cuda(logits, temperatures, row_keys, steps)
    assert logits.dim() == 2 and logits.dtype == torch.float32 and logits.stride(1) == 1
    N, V = logits.shape
    if out is None:
        out = torch.empty((N,), dtype=torch.int32, device=logits.device)
    if N == 0:
        return out
    if temperatures is not None:
        assert temperatures.dtype == torch.float32 and row_keys.dtype == torch.int32 and steps.dtype == torch.int32
    # blocks per row: about four blocks an SM over all rows, but no slice below 2,048 entries
    sms = sm_count(logits.device)
    slices = max(1, min(-(-4 * sms // N), V // 2048, 64))
    part, row_max, tickets = _sample_buffers(logits.device, N, slices)
    code = _lib().msgl_sample(_ptr(logits), N, V, logits.stride(0), _ptr(temperatures), _ptr(row_keys), _ptr(steps),
                              seed & 0xFFFFFFFFFFFFFFFF, _ptr(out), _ptr(part), _ptr(row_max), _ptr(tickets), slices, _stream())
    _check(code, "sample")
    if temperatures is not None:
        global LAUNCHES
        LAUNCHES += 1            # the race is a kernel of its own
    return out


# ---------------------------------------------------------------------------------------
# attention
# ---------------------------------------------------------------------------------------
VARIANT_SIMT, VARIANT_MMA_ROWS, VARIANT_MMA_DECODE, VARIANT_TC = 0, 1, 2, 3
TC_ROWS = 128                     # query rows per block of the tcgen05 prefill kernel
USE_TC_ATTENTION = os.environ.get("MSGL_NO_TC_ATTENTION", "") == ""
_status = None                    # device int32[64]: word 0 tcgen05 attention, word 2 tcgen05 GEMM, word 3 decode-step kernel; words 4..: debug counters
_status_host = None               # its pinned mirror, refreshed by poll_status()
_status_event = None


def _status_tensor(device) -> torch.Tensor:
    global _status, _status_host
    if _status is None:
        _status = torch.zeros(64, dtype=torch.int32, device=device)
        _status_host = torch.zeros(64, dtype=torch.int32).pin_memory()
    return _status


def poll_status() -> None:
    """Queue a copy of the kernels' status words to the host (no synchronisation).  Not inside a stream capture."""
    global _status_event
    if _status is None:
        return
    _status_host.copy_(_status, non_blocking=True)
    _status_event = torch.cuda.Event()
    _status_event.record()


def raise_if_failed(wait: bool = False) -> None:
    """Raise if a kernel with bounded waits gave up in a launch that the last finished poll_status() saw."""
    if _status_event is None:
        return
    if wait:
        _status_event.synchronize()
    elif not _status_event.query():
        return
    if int(_status_host[0]) != 0:
        raise KernelError("tcgen05 attention: a block timed out waiting for the tensor core; results are invalid")
    if int(_status_host[2]) != 0:
        raise KernelError("tcgen05 GEMM: a block timed out waiting for its pipeline; results are invalid")
    if int(_status_host[3]) != 0:
        raise KernelError("decode step: a block timed out at a grid barrier; results are invalid")


def tc_supported(head_dim: int, dtype: torch.dtype, group: int) -> bool:
    """The tcgen05 prefill attention kernels take bfloat16, head size 128, up to 128 query heads per kv head."""
    return USE_TC_ATTENTION and dtype == torch.bfloat16 and head_dim == 128 and 1 <= group <= TC_ROWS


def check_kernel_status() -> None:
    """Raise if a block of a kernel with bounded waits ever gave up waiting (synchronises)."""
    poll_status()
    raise_if_failed(wait=True)


TC_VERSION = int(os.environ.get("MSGL_TC_VERSION", "2"))      # 2: two query tiles per block in ping-pong (needs TMA page sizes); 1: one tile
_tc2_usable = True


def attention_tc(q: torch.Tensor, out: torch.Tensor, k_cache: torch.Tensor, v_cache: torch.Tensor, *,
                 q_start: torch.Tensor, kv_len: torch.Tensor, block_table: torch.Tensor, n_kv: int, page_size: int,
                 window: int, scale: float, qlen_min: int, qlen_max: int, q_lens: Sequence[int]) -> None:
    """Prefill attention on tcgen05 tensor cores for the requests with q_len in [qlen_min, qlen_max];
    q_lens: the host's copy of every request's number of query tokens (to size the grid)."""
    global _tc2_usable
    _need_cuda(q, out, k_cache, v_cache, q_start, kv_len, block_table)
    T, n_q, d = q.shape
    B = kv_len.numel()
    assert q.is_contiguous() and out.is_contiguous() and block_table.stride(1) == 1 and q.dtype == torch.bfloat16
    status = _status_tensor(q.device)
    group = n_q // n_kv
    whole = k_cache.is_contiguous() and v_cache.is_contiguous() and k_cache.shape == v_cache.shape
    pages = k_cache.shape[0] if whole else 0
    tma_pages = whole and page_size >= 8 and (page_size & (page_size - 1)) == 0
    versions = [2, 1] if (TC_VERSION == 2 and _tc2_usable and tma_pages) else [1]
    for version in versions:
        rows = TC_ROWS * version
        qt = rows // group if group <= TC_ROWS else version
        grid_x = sum(-(-n // qt) for n in q_lens if qlen_min <= n <= qlen_max)
        code = _attn_lib(d).msgl_attention_tc(
            _ptr(q), _ptr(out), _ptr(k_cache), _ptr(v_cache), _ptr(q_start), _ptr(kv_len), _ptr(block_table), B, T, n_q,
            n_kv, d, page_size, block_table.stride(0), window, float(scale), qlen_min, qlen_max, grid_x, pages, version,
            _ptr(status), _stream())
        if code == 2 and version == 2:        # no tensor maps here (driver without the encoder, unaligned cache): one-tile kernel
            _tc2_usable = False
            continue
        _check(code, "attention_tc")
        return


def attention_tile_tokens(variant: int, group: int, head_dim: int = 128) -> int:
    """Tokens per query tile of a kernel variant for a given group size (q heads per kv head)."""
    if variant == VARIANT_MMA_DECODE:
        lib = _attn_lib(head_dim)
        lib.msgl_attention_decode_tile_tokens.restype = c_int
        return int(lib.msgl_attention_decode_tile_tokens(int(group)))
    rows = {VARIANT_MMA_ROWS: 64, VARIANT_TC: TC_ROWS}.get(variant, 16)
    return rows // group if group <= rows else 1


def decode_blocks_per_sm(head_dim: int, dtype: torch.dtype, group: int = 1) -> int:
    """Blocks of the decode attention kernel that fit one SM (used to choose the kv splits)."""
    if not mma_supported(head_dim, dtype):
        return 4
    lib = _attn_lib(head_dim)
    lib.msgl_attention_decode_blocks_per_sm.restype = c_int
    return int(lib.msgl_attention_decode_blocks_per_sm(int(group)))


def even_cut_size(B: int, n_blocks: int) -> int:
    """int32 words of the even cut of a decode step of B requests over n_blocks blocks per kv head: blocks in use, start
    unit of every block [n_blocks + 1], first request of every block [n_blocks], first unit of every request [B + 1], first
    block of every request [B]."""
    return 1 + (n_blocks + 1) + n_blocks + (B + 1) + B


def decode_even_ok(head_dim: int, dtype: torch.dtype, group: int = 1) -> bool:
    """Whether the decode attention launch for this head size takes an even cut of the keys (`attention(even=...)`)."""
    if not mma_supported(head_dim, dtype):
        return False
    lib = _attn_lib(head_dim)
    lib.msgl_attention_decode_even_ok.restype = c_int
    return bool(lib.msgl_attention_decode_even_ok(int(group)))


def mma_supported(head_dim: int, dtype: torch.dtype) -> bool:
    return dtype == torch.bfloat16 and head_dim in _build.MMA_HEAD_DIMS


def attention(q: torch.Tensor, out: torch.Tensor, k_cache: torch.Tensor, v_cache: torch.Tensor, *,
              q_start: torch.Tensor, kv_len: torch.Tensor, block_table: torch.Tensor,
              nsplit: Optional[torch.Tensor], part_o: Optional[torch.Tensor], part_ml: Optional[torch.Tensor],
              n_kv: int, page_size: int, window: int, max_split: int, scale: float, qlen_min: int, qlen_max: int,
              uniform_decode: bool, variant: int, grid_x: int, order: Optional[torch.Tensor] = None,
              even: Optional[torch.Tensor] = None, even_nb: int = 0) -> None:
    """One launch of the paged attention kernel over the requests whose q_len lies in
    [qlen_min, qlen_max]; see csrc/attention.cu for the meaning of every argument.  `order` (uniform decode only):
    int32 [B], a permutation of the requests; the launch's i-th block along x takes request order[i].  `even`: the even cut
    of a decode step's keys over `even_nb` blocks per kv head (engine/step.py: plan_even_cut) in place of `grid_x` blocks."""
    _need_cuda(q, out, k_cache, v_cache, q_start, kv_len, block_table, nsplit, part_o, part_ml, order, even)
    T, n_q, d = q.shape
    B = kv_len.numel()
    assert q.is_contiguous() and out.is_contiguous() and block_table.dim() == 2 and block_table.stride(1) == 1
    assert q_start.numel() == B + 1 and block_table.shape[0] == B and out.shape == q.shape
    assert nsplit is None or nsplit.numel() == B
    assert order is None or (uniform_decode and order.numel() == B and order.dtype == torch.int32)
    assert even is None or (uniform_decode and variant == VARIANT_MMA_DECODE and even.dtype == torch.int32 and
                            even.numel() >= even_cut_size(B, even_nb) and even_nb >= 1)
    if max_split > 1:
        assert part_o.numel() >= max_split * T * n_q * d and part_ml.numel() >= max_split * T * n_q * 2
    code = _attn_lib(d).msgl_attention(
        _ptr(q), _ptr(out), _ptr(k_cache), _ptr(v_cache), _ptr(q_start), _ptr(kv_len), _ptr(block_table),
        _ptr(nsplit), _ptr(part_o), _ptr(part_ml), B, T, n_q, n_kv, d, page_size, block_table.stride(0), window,
        max_split, float(scale), qlen_min, qlen_max, int(uniform_decode), variant, grid_x, _dt(q), _ptr(order), _ptr(even), int(even_nb), _stream())
    _check(code, f"attention (head size {d}, variant {variant})")


def attention_combine(part_o: torch.Tensor, part_ml: torch.Tensor, token_req: Optional[torch.Tensor],
                      nsplit: torch.Tensor, out: torch.Tensor, max_split: int) -> None:
    _need_cuda(part_o, part_ml, token_req, nsplit, out)
    T, n_q, d = out.shape
    code = _attn_lib(d).msgl_attention_combine(_ptr(part_o), _ptr(part_ml), _ptr(token_req), _ptr(nsplit), _ptr(out),
                                               T, n_q, d, max_split, _dt(out), _stream())
    _check(code, "attention_combine")


# ---------------------------------------------------------------------------------------
# matrix products: the library GEMM (cuBLAS through torch)
# ---------------------------------------------------------------------------------------

def set_true_fp32() -> None:
    """float32 products are real float32: no TF32, no reduced-precision reduction."""
    torch.backends.cuda.matmul.allow_tf32 = False
    torch.backends.cudnn.allow_tf32 = False
    torch.backends.cuda.matmul.allow_bf16_reduced_precision_reduction = False
    torch.set_float32_matmul_precision("highest")


SMALL_M_MAX = int(os.environ.get("MSGL_SMALL_M_MAX", "8"))      # tokens up to which the weight-streaming kernel replaces the library GEMM (measured: faster up to 8)
USE_SMALL_M = os.environ.get("MSGL_NO_SMALL_M", "") == ""


def _small_m(weight, x, bias, out, M, N, K, ldo, mode, out_f32) -> int:
    return _lib().msgl_gemm_small_m(_ptr(weight), _ptr(x), _ptr(bias), _ptr(out), M, N, K, x.stride(0), ldo, mode, out_f32, _stream())


def _small_m_ok(x: torch.Tensor, weight: torch.Tensor, bias: Optional[torch.Tensor]) -> bool:
    return (USE_SMALL_M and x.dtype == torch.bfloat16 and weight.dtype == torch.bfloat16 and x.dim() == 2
            and 0 < x.shape[0] <= SMALL_M_MAX and x.stride(1) == 1 and x.stride(0) % 8 == 0 and weight.is_contiguous()
            and weight.shape[1] % 32 == 0 and weight.shape[0] % 16 == 0
            and (bias is None or bias.dtype == torch.bfloat16))


# This engine's tcgen05 GEMM (csrc/gemm_tc.cu) against the library's, measured on B200 at Qwen3-8B's sizes.  With SwiGLU in
# its epilogue the kernel on pairs of SMs (cta_group::2) beats library GEMM + activation kernel from about 256 rows on
# (512 rows: 83 against 86 us, 2,048 rows: 285 against 310 us, 4,096 rows: 0.52 against 0.72 ms; 2,048-token prefill step
# 27.4 -> 26.4 ms).  Its plain products reach 92-95 % of the library's speed at 2,048 rows (the one-block kernel: 88 %), so
# those stay with the library unless MSGL_TC_GEMM=all (prefill step + 1.3 ms).  MSGL_TC_GEMM=0 switches the kernel off,
# MSGL_TC_GEMM_CTAS=1 takes the one-block kernel.
TC_GEMM = os.environ.get("MSGL_TC_GEMM", "swiglu")            # "swiglu" | "all" | "0"
TC_GEMM_MIN_M = int(os.environ.get("MSGL_TC_GEMM_MIN_M", "256"))
TC_GEMM_CTAS = int(os.environ.get("MSGL_TC_GEMM_CTAS", "2"))   # 2: the kernel on pairs of SMs (tcgen05 cta_group::2)
_tc_gemm_usable = True


def _tc_gemm(x: torch.Tensor, weight: torch.Tensor, bias: Optional[torch.Tensor], mode: int) -> Optional[torch.Tensor]:
    """x @ weight^T (mode 0) or SwiGLU of it (mode 1) by the tcgen05 kernel; None where it does not apply."""
    global _tc_gemm_usable
    if not ((TC_GEMM == "all" or (TC_GEMM == "swiglu" and mode == 1)) and _tc_gemm_usable and x.dtype == torch.bfloat16 and weight.dtype == torch.bfloat16 and x.dim() == 2
            and x.shape[0] >= TC_GEMM_MIN_M and x.stride(1) == 1 and x.stride(0) % 8 == 0 and weight.is_contiguous()
            and weight.shape[1] % 8 == 0 and (bias is None or bias.dtype == torch.bfloat16)):
        return None
    M, (N, K) = x.shape[0], weight.shape
    n_out = N // 2 if mode == 1 else N
    if n_out % 8 or (mode == 1 and N % 2):
        return None
    out = torch.empty((M, n_out), dtype=torch.bfloat16, device=x.device)
    fn = _lib().msgl_gemm_tc2 if TC_GEMM_CTAS == 2 else _lib().msgl_gemm_tc
    code = fn(_ptr(weight), _ptr(x), _ptr(bias), _ptr(out), M, N, K, x.stride(0), n_out, mode, _ptr(_status_tensor(x.device)), _stream())
    if code == 2:             # no tensor maps on this driver
        _tc_gemm_usable = False
        return None
    _check(code, "gemm_tc")
    return out


# Between the weight-streaming kernel (up to SMALL_M_MAX rows) and the tiled tcgen05 kernel (from TC_GEMM_MIN_M rows) a product has
# too few output tiles to fill the GPU: there the pair kernel cuts K into ranges as well (split-K) and a second kernel adds
# the ranges' float32 partial sums in order.  Off unless MSGL_TC_MID=1: measured on B200 at Qwen3-8B's sizes it is behind the
# library GEMM at 16 to 128 rows (qkv 18-26 against 12.5 us, o 15-21 against 10, gate/up + SwiGLU 44-66 against 42-45, down 26-33
# against 21-22 us), so these sizes stay with the library.
MID_GEMM = os.environ.get("MSGL_TC_MID", "0") == "1"
MID_GEMM_SPLITS = int(os.environ.get("MSGL_TC_MID_SPLITS", "0"))        # 0: chosen per size
_mid_partials = {}
_mid_splits = {}


def _tc_gemm_mid(x: torch.Tensor, weight: torch.Tensor, bias: Optional[torch.Tensor], mode: int) -> Optional[torch.Tensor]:
    """x @ weight^T (mode 0) or SwiGLU of it (mode 1) for a middling number of rows by the split-K tcgen05 kernel; None where
    it does not apply."""
    global _tc_gemm_usable
    if not (MID_GEMM and TC_GEMM != "0" and TC_GEMM_CTAS == 2 and _tc_gemm_usable and x.dtype == torch.bfloat16
            and weight.dtype == torch.bfloat16 and x.dim() == 2 and SMALL_M_MAX < x.shape[0] < TC_GEMM_MIN_M and x.stride(1) == 1
            and x.stride(0) % 8 == 0 and weight.is_contiguous() and weight.shape[1] % 8 == 0 and weight.shape[0] % 8 == 0
            and weight.shape[1] >= 512 and (bias is None or bias.dtype == torch.bfloat16)):
        return None
    M, (N, K) = x.shape[0], weight.shape
    n_out = N // 2 if mode == 1 else N
    if n_out % 8 or (mode == 1 and N % 16):
        return None
    key = (M, N, K, mode)
    splits = MID_GEMM_SPLITS or _mid_splits.get(key)
    if not splits:
        splits = _mid_splits[key] = int(_lib().msgl_gemm_tc2_splits(M, N, K, mode))
    splits = max(1, min(splits, K // 64))
    part = None
    if splits > 1:
        dev = x.device.index if x.device.index is not None else torch.cuda.current_device()
        part = _mid_partials.get(dev)
        if part is None or part.numel() < splits * M * N:
            part = _mid_partials[dev] = torch.empty(max(splits * M * N, 1 << 22), dtype=torch.float32, device=x.device)
    out = torch.empty((M, n_out), dtype=torch.bfloat16, device=x.device)
    code = _lib().msgl_gemm_tc2_splitk(_ptr(weight), _ptr(x), _ptr(bias), _ptr(out), M, N, K, x.stride(0), n_out, mode, splits,
                                       _ptr(part), _ptr(_status_tensor(x.device)), _stream())
    if code == 2:             # no tensor maps on this driver
        _tc_gemm_usable = False
        return None
    _check(code, "gemm_tc (split-K)")
    if splits > 1:
        global LAUNCHES
        LAUNCHES += 1
    return out


def linear(x: torch.Tensor, weight: torch.Tensor, bias: Optional[torch.Tensor] = None,
           out_dtype: Optional[torch.dtype] = None) -> torch.Tensor:
    """y = x @ weight^T (+ bias); weight is [out, in] as stored in the checkpoint.

    Up to SMALL_M_MAX bfloat16 rows go through this engine's weight-streaming kernel
    (csrc/gemm_small_m.cu); everything else is the library GEMM."""
    _need_cuda(x, weight, bias)
    if _small_m_ok(x, weight, bias) and out_dtype in (None, torch.bfloat16, torch.float32):
        M, (N, K) = x.shape[0], weight.shape
        od = out_dtype or torch.bfloat16
        out = torch.empty((M, N), dtype=od, device=x.device)
        code = _small_m(weight, x, bias, out, M, N, K, N, 0, int(od == torch.float32))
        _check(code, "gemm_small_m")
        return out
    if out_dtype in (None, torch.bfloat16):
        y = _tc_gemm(x, weight, bias, 0) if x.shape[0] >= TC_GEMM_MIN_M else _tc_gemm_mid(x, weight, bias, 0)
        if y is not None:
            return y
    if out_dtype is not None and out_dtype != x.dtype:
        y = torch.mm(x, weight.t(), out_dtype=out_dtype)
        if bias is not None:
            y += bias.to(out_dtype)
        return y
    return torch.nn.functional.linear(x, weight, bias)


def linear_swiglu(x: torch.Tensor, gate_up: torch.Tensor) -> torch.Tensor:
    """silu(x @ gate^T) * (x @ up^T) with gate_up = [gate; up] packed row-wise ([2I, H]).  For a few
    rows the product and the activation are one kernel and the [T, 2I] intermediate never exists."""
    _need_cuda(x, gate_up)
    if _small_m_ok(x, gate_up, None) and (gate_up.shape[0] // 2) % 8 == 0:
        M, (N, K) = x.shape[0], gate_up.shape
        out = torch.empty((M, N // 2), dtype=torch.bfloat16, device=x.device)
        code = _small_m(gate_up, x, None, out, M, N, K, N // 2, 1, 0)
        _check(code, "gemm_small_m (swiglu)")
        return out
    y = _tc_gemm(x, gate_up, None, 1) if x.shape[0] >= TC_GEMM_MIN_M else _tc_gemm_mid(x, gate_up, None, 1)
    if y is not None:
        return y
    return swiglu(torch.nn.functional.linear(x, gate_up))


# ---------------------------------------------------------------------------------------
# the whole decode step in one persistent kernel (csrc/decode_step.cu)
# ---------------------------------------------------------------------------------------
# Off unless MSGL_FUSED_DECODE=1: measured on B200 at Qwen3-8B's sizes the one-kernel step takes 4.2 / 5.4 ms at batch 1 / 8
# (context 4,096) against 3.4 / 4.2 ms kernel by kernel (see profiles/decode_step_kernel_b1_b8.md for where the time goes).
USE_FUSED_DECODE = os.environ.get("MSGL_FUSED_DECODE", "0") == "1"
FUSED_DECODE_MAX_TOKENS = 8
STATUS_WORD_DECODE_STEP = 3


class DsLayer(ctypes.Structure):
    """One run of a layer for the decode-step kernel; mirrors `struct DsLayer`."""
    _fields_ = [("w_qkv", c_void_p), ("b_qkv", c_void_p), ("w_o", c_void_p), ("w_gu", c_void_p), ("w_down", c_void_p),
                ("norm_in", c_void_p), ("norm_post", c_void_p), ("q_norm", c_void_p), ("k_norm", c_void_p),
                ("k_cache", c_void_p), ("v_cache", c_void_p),
                ("eps_in", c_float), ("eps_post", c_float), ("eps_qk", c_float),
                ("norm_f32", c_int), ("qk_norm_f32", c_int), ("pad_", c_int)]


class DsStep(ctypes.Structure):
    """Arguments of one decode step; mirrors `struct DsStep`."""
    _fields_ = [("layers", c_void_p), ("n_layers", c_int), ("M", c_int),
                ("H", c_int), ("n_q", c_int), ("n_kv", c_int), ("I", c_int), ("V", c_int),
                ("page_size", c_int), ("page_shift", c_int), ("bt_stride", c_int), ("max_split", c_int),
                ("scale", c_float),
                ("rope", c_void_p), ("rot", c_int), ("max_pos", c_int),
                ("ids", c_void_p), ("positions", c_void_p), ("kv_len", c_void_p), ("block_table", c_void_p),
                ("out_loc", c_void_p), ("nsplit", c_void_p),
                ("embed", c_void_p), ("final_norm", c_void_p), ("final_f32", c_int), ("eps_final", c_float),
                ("lm_head", c_void_p),
                ("res", c_void_p), ("xn", c_void_p), ("ssq", c_void_p), ("qkv", c_void_p), ("attn", c_void_p), ("act", c_void_p),
                ("part_o", c_void_p), ("part_ml", c_void_p), ("tickets", c_void_p), ("logits", c_void_p),
                ("bar", c_void_p), ("status", c_void_p)]


_decode_libs = {}


def _decode_lib(head_dim: int):
    lib = _decode_libs.get(head_dim)
    if lib is None:
        lib = _build.decode_step_library(head_dim)
        lib.msgl_decode_step_blocks.argtypes = [c_int] * 6
        lib.msgl_decode_step_blocks.restype = c_int
        lib.msgl_decode_step.argtypes = [ctypes.POINTER(DsStep), c_void_p]
        if lib.msgl_decode_step_layer_bytes() != ctypes.sizeof(DsLayer) or lib.msgl_decode_step_struct_bytes() != ctypes.sizeof(DsStep):
            raise KernelError("decode_step: the argument structures of the library and of ops.py differ")
        _decode_libs[head_dim] = lib
    return lib


def decode_step_blocks(tokens: int, hidden: int, n_q: int, n_kv: int, head_dim: int, intermediate: int, vocab: int) -> int:
    """Blocks the decode-step kernel runs with for these sizes on the current device; 0: it does not take them
    (the caller then runs the step kernel by kernel).  Not inside a stream capture the first time."""
    if not USE_FUSED_DECODE or head_dim % 32 or head_dim < 32 or head_dim > 128:      # beyond 128 the accumulators spill
        return 0
    return int(_decode_lib(head_dim).msgl_decode_step_blocks(tokens, hidden, n_q, n_kv, intermediate, vocab))


def decode_step(step: DsStep, head_dim: int) -> None:
    """Launch the decode-step kernel on the current stream."""
    code = _decode_lib(head_dim).msgl_decode_step(ctypes.byref(step), _stream())
    _check(code, f"decode_step (head size {head_dim})")
