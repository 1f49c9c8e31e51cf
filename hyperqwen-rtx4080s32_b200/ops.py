"""Operator layer over the C ABI: the functions the GGUF LinearMethod calls, with the reference's names
and argument meaning (gguf-plugin/gluon/interface.py, gguf-plugin/gluon/tiles.py,
gguf-plugin/gluon/tiles_grouped.py), and the torch custom op that wraps the per-call one so a compiled
graph sees a single traceable call (gguf-plugin/patches/gguf-tiles-grouped.patch:28-74).

All compute happens in libgq_b200.so on the current CUDA device and stream; tensors only carry device
memory.  There is no fallback: a missing library or a CPU tensor raises.
"""
from __future__ import annotations

import contextlib

import ctypes
from typing import Sequence

import numpy as np
import torch

from . import formats as F
from ._lib import DESC_WORDS, MAX_GEMV_ROWS, GqError, check, lib

TILE_TYPES = F.SUPPORTED_TYPES   # every supported type is held tile-major (the reference: GLUON_TILE_TYPES)
GEMV_MAX_ROWS = MAX_GEMV_ROWS    # the grouped kernel's own limit (the C ABI accepts up to 64 rows)
DECODE_MAX_ROWS = 32             # row-count dispatch threshold: above it the tcgen05 kernel takes over

def _stream_ptr(t: torch.Tensor) -> int:
    return torch.cuda.current_stream(t.device).cuda_stream


def _need_cuda(t: torch.Tensor, what: str) -> None:
    if not t.is_cuda:
        raise GqError(f"{what} must be a CUDA tensor (there is no CPU path)")


def _i32_array(vals: Sequence[int]):
    return (ctypes.c_int32 * len(vals))(*[int(v) for v in vals])


def _i64_array(vals: Sequence[int]):
    return (ctypes.c_int64 * len(vals))(*[int(v) for v in vals])


def sm_count(device=None) -> int:
    if torch.cuda.is_available():
        return torch.cuda.get_device_properties(device if device is not None else torch.cuda.current_device()).multi_processor_count
    return 148


# ---- host-only helpers (usable without a GPU) -----------------------------------------------------

def slab_map(wtype: int) -> np.ndarray:
    """map[p] = row * bytes_per_256 + byte: the raw source of packed byte p of a 16-row slab."""
    bb = lib().gq_bytes_per_256(int(wtype))
    if bb == 0:
        raise GqError(f"unsupported GGML type {wtype}")
    m = np.empty(16 * bb, dtype=np.int32)
    check(lib().gq_slab_map(int(wtype), m.ctypes.data_as(ctypes.c_void_p)), "gq_slab_map")
    return m


def packed_bytes(wtype: int, n_out: int, k: int) -> int:
    return check(lib().gq_packed_bytes(int(wtype), int(n_out), int(k)), "gq_packed_bytes")


def build_descs(wtypes: Sequence[int], n_outs: Sequence[int], k: int, split: int) -> np.ndarray:
    """The descriptor table int32 [n_tiles * split, 8] of a run of shards (host array)."""
    n = len(wtypes)
    no = _i64_array(n_outs)
    rows = check(lib().gq_desc_rows(n, no, int(split)), "gq_desc_rows")
    out = np.zeros((rows, DESC_WORDS), dtype=np.int32)
    got = check(lib().gq_build_descs(n, _i32_array(wtypes), no, int(k), int(split), out.ctypes.data_as(ctypes.c_void_p)),
                "gq_build_descs")
    assert got == rows
    return out


def grouped_split_for(n_tiles: int, nb: int, m: int | None = None, block_bytes: int | None = None, sms: int | None = None) -> int:
    """Split-K of a grouped launch (reference: grouped_split_for, gguf-plugin/gluon/tiles_grouped.py:237-250)."""
    return int(lib().gq_split_for(int(n_tiles), int(nb), int(m or 0), int(block_bytes or 0), int(sms or sm_count())))


def run_info(wtypes: Sequence[int]) -> int:
    return check(lib().gq_run_info(len(wtypes), _i32_array(wtypes)), "gq_run_info")


def device_status(device=None, clear: bool = True) -> int:
    """The largest status code a kernel of the library reported on the device since it was last cleared (0: none;
    1: a bounded wait ran out and that call's output is incomplete; 2: bad shape).  Synchronises the stream."""
    dev = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
    with torch.cuda.device(dev):
        return check(lib().gq_device_status(1 if clear else 0, torch.cuda.current_stream(dev).cuda_stream), "gq_device_status")


def set_peer_wait_limit(seconds: float) -> None:
    """Time limit of the waits for another GPU's data in the all-reduce kernels (default 4 s)."""
    check(lib().gq_set_peer_wait_limit_ns(int(seconds * 1e9)), "gq_set_peer_wait_limit_ns")


# ---- load time -----------------------------------------------------------------------------------

def repack_tiles(raw: torch.Tensor, n_out: int, wtype: int) -> torch.Tensor:
    """raw uint8 [n_out, nb * bytes_per_256] (any row stride) -> tiles uint8 [ceil(n_out/64), nb, 64 * bytes_per_256]."""
    _need_cuda(raw, "raw")
    if raw.dtype != torch.uint8 or raw.dim() != 2 or raw.shape[0] != n_out:
        raise GqError(f"raw must be uint8 [n_out, row_bytes], got {raw.dtype} {tuple(raw.shape)}")
    bb = F.BYTES_PER_256[int(wtype)]
    if raw.shape[1] % bb or raw.stride(1) != 1:
        raise GqError(f"row bytes {raw.shape[1]} are not whole {bb}-byte k-blocks of type {wtype}")
    nb = raw.shape[1] // bb
    n_tiles = -(-n_out // 64)
    out = torch.empty((n_tiles, nb, 64 * bb), dtype=torch.uint8, device=raw.device)
    with torch.cuda.device(raw.device):
        check(lib().gq_repack(int(wtype), raw.data_ptr(), n_out, nb * 256, raw.stride(0), out.data_ptr(), _stream_ptr(raw)), "gq_repack")
    return out


def unrepack_tiles(tiles: torch.Tensor, n_out: int, wtype: int) -> torch.Tensor:
    """tiles -> the raw rows uint8 [n_out, nb * bytes_per_256], bit for bit."""
    _need_cuda(tiles, "tiles")
    bb = F.BYTES_PER_256[int(wtype)]
    if tiles.dtype != torch.uint8 or tiles.dim() != 3 or tiles.shape[2] != 64 * bb or not tiles.is_contiguous():
        raise GqError(f"tiles must be contiguous uint8 [n_tiles, nb, {64 * bb}], got {tuple(tiles.shape)}")
    nb = tiles.shape[1]
    raw = torch.empty((n_out, nb * bb), dtype=torch.uint8, device=tiles.device)
    with torch.cuda.device(tiles.device):
        check(lib().gq_unrepack(int(wtype), tiles.data_ptr(), n_out, nb * 256, raw.data_ptr(), raw.stride(0), _stream_ptr(tiles)), "gq_unrepack")
    return raw


def dequantize_tiles(tiles: torch.Tensor, n_out: int, k: int, wtype: int, dtype=torch.float32) -> torch.Tensor:
    """tiles -> weights [n_out, k]: fp32 bit-identical to gguf.quants.dequantize, or bf16 (that value rounded)."""
    _need_cuda(tiles, "tiles")
    if dtype not in (torch.float32, torch.bfloat16):
        raise GqError("dequantize_tiles produces float32 or bfloat16")
    out = torch.empty((n_out, k), dtype=dtype, device=tiles.device)
    with torch.cuda.device(tiles.device):
        check(lib().gq_dequant(int(wtype), tiles.data_ptr(), n_out, k, out.data_ptr(), 0 if dtype == torch.float32 else 1, k,
                               _stream_ptr(tiles)), "gq_dequant")
    return out


def pack_tiles(shards: Sequence[tuple[torch.Tensor, int, int]]):
    """[(tiles, n_out, type)] -> (packed uint8 buffer, meta): the shards' tiles back to back in one buffer."""
    nb = None
    for t, n_out, wt in shards:
        if t.shape[0] != -(-n_out // 64) or (nb is not None and t.shape[1] != nb):
            raise GqError("shards of a run must share K and hold ceil(n_out/64) tiles")
        nb = int(t.shape[1])
    packed = shards[0][0].reshape(-1) if len(shards) == 1 else torch.cat([t.reshape(-1) for t, _, _ in shards])
    meta = {"nb": nb, "n_outs": [int(n) for _, n, _ in shards], "types": [int(w) for _, _, w in shards],
            "n_total": sum(int(n) for _, n, _ in shards)}
    return packed, meta


def prepare_grouped_layer(tiles_list: Sequence[torch.Tensor], n_outs: Sequence[int], wtypes: Sequence[int], ms=range(1, GEMV_MAX_ROWS + 1)):
    """The loader's step for a run of shards (reference: prepare_grouped_layer,
    gguf-plugin/gluon/tiles_grouped.py:253-267): (packed buffer, the shards' tiles as views into it, the
    descriptor tables of every split a batch of 1..64 rows can choose plus split 1, those splits, nb, the
    run's average bytes per 256 weights)."""
    packed, meta = pack_tiles(list(zip(tiles_list, n_outs, wtypes)))
    views, off = [], 0
    for t in tiles_list:
        views.append(packed[off:off + t.numel()].view(t.shape))
        off += t.numel()
    nb, n_total = meta["nb"], meta["n_total"]
    n_tiles = sum(-(-int(n) // 64) for n in n_outs)
    block_bytes = int(round(sum(int(n) * F.BYTES_PER_256[int(w)] for n, w in zip(n_outs, wtypes)) / max(1, n_total)))
    sms = sm_count(packed.device)
    splits = sorted({grouped_split_for(n_tiles, nb, m=m, block_bytes=block_bytes, sms=sms) for m in ms} | {1})
    descs = [torch.from_numpy(build_descs(wtypes, n_outs, nb * 256, s)).to(packed.device) for s in splits]
    return packed, views, descs, splits, nb, block_bytes


# ---- per call ------------------------------------------------------------------------------------

# packed buffer (data_ptr) -> (data_ptr, bytes) of the packed buffer the model multiplies next; filled by
# register_prefetch_chain at load time.  A launch on the key prefetches the value into L2 while it computes.
_NEXT_WEIGHTS: dict[int, tuple[int, int]] = {}


def register_prefetch_chain(packed_in_call_order: Sequence[torch.Tensor], cyclic: bool = True) -> None:
    """Tell the op in which order a model's packed runs are multiplied (qkv, o, gate_up, down, next block ...),
    so each small-batch launch can warm the L2 with its successor's weights."""
    bufs = list(packed_in_call_order)
    for i, b in enumerate(bufs):
        if i + 1 < len(bufs) or cyclic:
            nxt = bufs[(i + 1) % len(bufs)]
            _NEXT_WEIGHTS[b.data_ptr()] = (nxt.data_ptr(), nxt.numel())


def clear_prefetch_chain() -> None:
    _NEXT_WEIGHTS.clear()


_FUSED_AR = None      # the tp.FusedAllReduce in force for the calls inside `with fused_allreduce(ctx)`


@contextlib.contextmanager
def fused_allreduce(ctx):
    """Inside this block the small-batch path of mul_mat_tiles_grouped leaves the SUM over the tensor-parallel
    ranks in its output (gq_gemv_grouped_allreduce) and sets ctx.used; calls it cannot serve (more than 64 rows,
    sizes beyond the context's buffers) run as usual and leave ctx.used alone, so the caller can fall back to a
    separate all-reduce."""
    global _FUSED_AR
    prev, _FUSED_AR = _FUSED_AR, ctx
    try:
        yield ctx
    finally:
        _FUSED_AR = prev


class PreSiluMul:
    """The layer's input is silu(t[:, :K]) * t[:, K:] of the [M, 2K] tensor handed in (vLLM's silu_and_mul in front of
    down_proj), computed inside the activation preparation."""
    kind = 1

    def unfused(self, t: torch.Tensor) -> torch.Tensor:
        k = t.shape[-1] // 2
        return torch.nn.functional.silu(t[..., :k]) * t[..., k:]


class PreAddRMSNorm:
    """The layer's input is RMSNorm(t + residual) * weight (vLLM's fused_add_rms_norm in front of qkv_proj and
    gate_up_proj), computed inside the activation preparation; `residual_out` receives t + residual.  Without a residual,
    plain RMSNorm."""
    kind = 2

    def __init__(self, weight: torch.Tensor, eps: float = 1e-6, residual: torch.Tensor | None = None):
        self.weight, self.eps, self.residual = weight, float(eps), residual
        self.residual_out = torch.empty_like(residual) if residual is not None else None

    def unfused(self, t: torch.Tensor) -> torch.Tensor:
        if self.residual is not None:
            t = t + self.residual
            self.residual_out.copy_(t)
        v = t.float()
        v = v * torch.rsqrt(v.pow(2).mean(-1, keepdim=True) + self.eps)
        return v.to(t.dtype) * self.weight


PRE_MAX_ROWS = 16     # the folded ops live in the integer form's preparation


def grouped_gemm(x: torch.Tensor, packed: torch.Tensor, desc: torch.Tensor, split: int, wtypes: Sequence[int], n_total: int,
                 out: torch.Tensor | None = None, workspace: torch.Tensor | None = None, phases: int = 7, allreduce=None, pre=None) -> torch.Tensor:
    """One grouped launch for 1..64 rows: x bf16 [M, K] -> out bf16 [M, n_total] (out may be a column view).
    `workspace` (uint8, 256-byte aligned, at least gq_workspace_bytes) is allocated per call unless given;
    `phases` selects the launches (1 prepare activations, 2 grouped kernel, 4 partial sum); `allreduce` (a
    tp.FusedAllReduce) makes the output the sum over the tensor-parallel ranks; `pre` (PreSiluMul / PreAddRMSNorm,
    up to 16 rows) folds the op in front of the layer into the activation preparation — x is then that op's input."""
    _need_cuda(x, "x")
    if x.dtype != torch.bfloat16 or x.dim() != 2:
        raise GqError(f"x must be bf16 [M, K], got {x.dtype} {tuple(x.shape)}")
    m, k = int(x.shape[0]), int(x.shape[1])
    if pre is not None:
        if phases != 7 or m > PRE_MAX_ROWS or (allreduce is not None and pre.kind != 1):
            raise GqError(f"a folded op needs the whole call and at most {PRE_MAX_ROWS} rows (with the fused all-reduce: silu_and_mul only)")
        if pre.kind == 1:
            if k % 2:
                raise GqError("silu_and_mul needs an even input width")
            k //= 2
    if m > GEMV_MAX_ROWS:
        raise GqError(f"grouped_gemm takes at most {GEMV_MAX_ROWS} rows, got {m}")
    if x.stride(1) != 1:
        x = x.contiguous()
    if out is None:
        out = torch.empty((m, n_total), dtype=torch.bfloat16, device=x.device)
    elif out.dtype != torch.bfloat16 or out.shape != (m, n_total) or (m > 0 and out.stride(1) != 1):
        raise GqError("out must be bf16 [M, n_total] with unit column stride")
    if m == 0 or n_total == 0:
        return out
    L = lib()
    ws_bytes = check(L.gq_workspace_bytes(m, k, n_total, int(split)), "gq_workspace_bytes")
    ws = workspace if workspace is not None else torch.empty(ws_bytes, dtype=torch.uint8, device=x.device)
    if pre is not None and allreduce is not None:
        with torch.cuda.device(x.device):
            check(L.gq_gemv_grouped_allreduce_silu_mul(x.data_ptr(), m, k, x.stride(0), packed.data_ptr(), desc.data_ptr(), int(desc.shape[0]),
                                                       int(split), run_info(wtypes), out.data_ptr(), out.stride(0), n_total, ws.data_ptr(),
                                                       ws.numel(), allreduce.rank, allreduce.world, allreduce.ptrs, allreduce.max_m,
                                                       allreduce.max_n_total, _stream_ptr(x)), "gq_gemv_grouped_allreduce_silu_mul")
        allreduce.used = True
        return out
    if pre is not None:
        w = res = res_out = None
        if pre.kind == 2:
            w, res, res_out = pre.weight, pre.residual, pre.residual_out
            if w.dtype != torch.bfloat16 or w.numel() != k or not w.is_contiguous() or w.device != x.device:
                raise GqError("the norm weight must be contiguous bf16 [K] on x's device")
            if res is not None and (res.dtype != torch.bfloat16 or res.shape != x.shape or res.stride(1) != 1 or res_out.stride() != res.stride()):
                raise GqError("the residual must be bf16 [M, K] with unit column stride")
        with torch.cuda.device(x.device):
            check(L.gq_gemv_grouped_pre(x.data_ptr(), m, k, x.stride(0), pre.kind, w.data_ptr() if w is not None else None,
                                        res.data_ptr() if res is not None else None, res_out.data_ptr() if res_out is not None else None,
                                        res.stride(0) if res is not None else 0, getattr(pre, "eps", 0.0), packed.data_ptr(), desc.data_ptr(),
                                        int(desc.shape[0]), int(split), run_info(wtypes), out.data_ptr(), out.stride(0), n_total, ws.data_ptr(),
                                        ws.numel(), _stream_ptr(x)), "gq_gemv_grouped_pre")
        return out
    if allreduce is not None:
        with torch.cuda.device(x.device):
            check(L.gq_gemv_grouped_allreduce(x.data_ptr(), m, k, x.stride(0), packed.data_ptr(), desc.data_ptr(), int(desc.shape[0]), int(split),
                                              run_info(wtypes), out.data_ptr(), out.stride(0), n_total, ws.data_ptr(), ws.numel(),
                                              allreduce.rank, allreduce.world, allreduce.ptrs, allreduce.max_m, allreduce.max_n_total,
                                              _stream_ptr(x)), "gq_gemv_grouped_allreduce")
        allreduce.used = True
        return out
    nxt = _NEXT_WEIGHTS.get(packed.data_ptr()) if phases == 7 else None
    if nxt is not None:
        with torch.cuda.device(x.device):
            check(L.gq_gemv_grouped_prefetch(x.data_ptr(), m, k, x.stride(0), packed.data_ptr(), desc.data_ptr(), int(desc.shape[0]), int(split),
                                             run_info(wtypes), out.data_ptr(), out.stride(0), n_total, ws.data_ptr(), ws.numel(), _stream_ptr(x),
                                             nxt[0], min(nxt[1], 96 << 20)), "gq_gemv_grouped_prefetch")
        return out
    with torch.cuda.device(x.device):
        check(L.gq_gemv_grouped_phases(x.data_ptr(), m, k, x.stride(0), packed.data_ptr(), desc.data_ptr(), int(desc.shape[0]), int(split),
                                       run_info(wtypes), out.data_ptr(), out.stride(0), n_total, ws.data_ptr(), ws.numel(), _stream_ptr(x),
                                       int(phases)), "gq_gemv_grouped")
    return out


def prefill_gemm(x: torch.Tensor, packed: torch.Tensor, desc1: torch.Tensor, n_total: int, out: torch.Tensor | None = None, *,
                 wtypes: Sequence[int]) -> torch.Tensor:
    """The large-batch path (tcgen05 dequant-GEMM): x bf16 [M, K] -> out bf16 [M, n_total]; desc1 is the run's
    split-1 descriptor table; wtypes the run's GGML types (they size the shared-memory tables)."""
    _need_cuda(x, "x")
    if x.dtype != torch.bfloat16 or x.dim() != 2:
        raise GqError(f"x must be bf16 [M, K], got {x.dtype} {tuple(x.shape)}")
    m, k = int(x.shape[0]), int(x.shape[1])
    if x.stride(1) != 1 or x.stride(0) % 8 or x.data_ptr() % 16:
        x = x.contiguous()
    if out is None:
        out = torch.empty((m, n_total), dtype=torch.bfloat16, device=x.device)
    elif out.dtype != torch.bfloat16 or out.shape != (m, n_total) or (m > 0 and out.stride(1) != 1):
        raise GqError("out must be bf16 [M, n_total] with unit column stride")
    if m == 0 or n_total == 0:
        return out
    L = lib()
    with torch.cuda.device(x.device):
        ws_bytes = check(L.gq_prefill_workspace_bytes(m, k, n_total, int(desc1.shape[0])), "gq_prefill_workspace_bytes")
    ws = torch.empty(ws_bytes + 1024, dtype=torch.uint8, device=x.device)
    base = (ws.data_ptr() + 1023) // 1024 * 1024
    info = run_info(wtypes)
    with torch.cuda.device(x.device):
        check(L.gq_gemm_prefill(x.data_ptr(), m, k, x.stride(0), packed.data_ptr(), desc1.data_ptr(), int(desc1.shape[0]), info, out.data_ptr(),
                                out.stride(0), n_total, base, ws_bytes, _stream_ptr(x)), "gq_gemm_prefill")
    return out


def mul_mat_tiles_grouped_pre(x: torch.Tensor, pre, packed: torch.Tensor, descs: list[torch.Tensor], desc_splits: list[int],
                              tiles: list[torch.Tensor], n_outs: list[int], weight_types: list[int], nb: int, block_bytes: int) -> torch.Tensor:
    """mul_mat_tiles_grouped of pre(x): up to 16 rows the op is folded into the grouped launch's activation
    preparation; above, it runs as torch operations on the device in front of the usual call."""
    m = int(x.shape[0])
    if m == 0 or m > PRE_MAX_ROWS:
        return mul_mat_tiles_grouped(pre.unfused(x), packed, descs, desc_splits, tiles, n_outs, weight_types, nb, block_bytes)
    n_total = sum(int(n) for n in n_outs)
    n_tiles = sum(-(-int(n) // 64) for n in n_outs)
    s = grouped_split_for(n_tiles, nb, m=m, block_bytes=block_bytes, sms=sm_count(x.device))
    if s not in desc_splits:
        s = 1
    ar = _FUSED_AR
    if ar is not None:
        if pre.kind != 1 or not (m <= ar.max_m and n_total <= ar.max_n_total and s <= 8 and all(int(n) % 2 == 0 for n in n_outs)):
            return mul_mat_tiles_grouped(pre.unfused(x), packed, descs, desc_splits, tiles, n_outs, weight_types, nb, block_bytes)
    return grouped_gemm(x, packed, descs[desc_splits.index(s)], s, weight_types, n_total, pre=pre, allreduce=ar)


def mul_mat_tiles_grouped(x: torch.Tensor, packed: torch.Tensor, descs: list[torch.Tensor], desc_splits: list[int],
                          tiles: list[torch.Tensor], n_outs: list[int], weight_types: list[int], nb: int, block_bytes: int) -> torch.Tensor:
    """A layer's run of shards in one call: x bf16 [M, K] -> [M, sum(n_outs)] (reference:
    gluon_mul_mat_tiles_grouped, gguf-plugin/gluon/interface.py:141-188).  The row-count dispatch lives
    here, inside the op: up to 32 rows one grouped launch at the split of the table for that row count; above, the
    tcgen05 dequant-GEMM (weights dequantised into shared memory once per 64, 128 or 256 batch rows)."""
    m = int(x.shape[0])
    n_total = sum(int(n) for n in n_outs)
    out = torch.empty((m, n_total), dtype=x.dtype, device=x.device)
    if m == 0:
        return out
    n_tiles = sum(-(-int(n) // 64) for n in n_outs)
    # up to 32 rows the grouped kernel streams the weights once per 8 (integer form, to 16 rows) or 32 (fp16 form) rows;
    # from 33 rows the tcgen05 kernel (64-row variant, two CTAs per SM, split-K on narrow layers) dequantises each weight
    # once for all rows and is faster on every layer of the stack (gate_up at 64 rows: 79 us against 116 us for two
    # 32-row launches of the grouped kernel; down: 58 against 84)
    if m <= DECODE_MAX_ROWS:
        s = grouped_split_for(n_tiles, nb, m=m, block_bytes=block_bytes, sms=sm_count(x.device))
        if s not in desc_splits:
            s = 1
        ar = _FUSED_AR
        if ar is not None and not (m <= ar.max_m and n_total <= ar.max_n_total and s <= 8 and all(int(n) % 2 == 0 for n in n_outs)):
            ar = None
        grouped_gemm(x, packed, descs[desc_splits.index(s)], s, weight_types, n_total, out=out, allreduce=ar)
        return out
    prefill_gemm(x, packed, descs[desc_splits.index(1)], n_total, out=out, wtypes=weight_types)
    return out


# ---- torch custom op (traceable boundary) ----------------------------------------------------------

def _fake(x, packed, descs, desc_splits, tiles, n_outs, weight_types, nb, block_bytes):
    return torch.empty(x.shape[0], sum(n_outs), dtype=x.dtype, device=x.device)


_OP_LIB = torch.library.Library("gq_b200", "FRAGMENT")
_OP_LIB.define("fused_mul_mat_gguf_tiles_grouped(Tensor x, Tensor packed, Tensor[] descs, int[] desc_splits, Tensor[] tiles, "
               "int[] n_outs, int[] weight_types, int nb, int block_bytes) -> Tensor")
_OP_LIB.impl("fused_mul_mat_gguf_tiles_grouped", mul_mat_tiles_grouped, "CUDA")
torch.library.register_fake("gq_b200::fused_mul_mat_gguf_tiles_grouped")(_fake)
fused_mul_mat_gguf_tiles_grouped = torch.ops.gq_b200.fused_mul_mat_gguf_tiles_grouped
