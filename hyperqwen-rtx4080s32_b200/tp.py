"""Tensor-parallel sharding of GGUF tensors for the quantized-linear path.

Column-parallel layers (QKV, gate_up) split output rows; row-parallel layers (o, down) split K and sum
the ranks' partial outputs with one all-reduce per layer.  Shards are cut from the RAW block bytes before
the repack, so every rank repacks only what it owns.  vLLM's loader narrows the byte dimension evenly
(vllm/model_executor/layers/linear.py RowParallelLinear.weight_loader), which cuts a 256-weight superblock
in half when K / tp is not a multiple of 256 (hidden 5120 or 17408 over 8 ranks: 640 and 2176 weights).
Here a rank instead keeps every k-block its K range touches, whole, and its activations are zero outside
the range it owns: the shared block contributes x * w only where x is non-zero, so the sum over ranks is
unchanged and no block is re-encoded.  The price is reading one shared block twice across two ranks.
The reference has no tensor-parallel code of its own for this path (docs/multi-gpu.md:8-13 passes
--tensor-parallel-size through to vLLM).
"""
from __future__ import annotations

from dataclasses import dataclass

import torch

from . import formats as F


@dataclass
class KPad:
    """Where a row-parallel rank's own K range [k0, k1) sits inside the k-blocks it stores."""
    left: int       # zero columns before the rank's activations
    own: int        # the rank's K / tp columns
    total: int      # stored K (a multiple of 256)


def row_range(k: int, rank: int, size: int) -> tuple[int, int, int, int]:
    """(k0, k1, first block, one-past-last block) of a rank's K range."""
    if k % size:
        raise ValueError(f"K={k} does not divide over {size} ranks")
    own = k // size
    if own % 32:
        raise ValueError(f"K/tp={own} must be a multiple of 32")
    k0, k1 = rank * own, (rank + 1) * own
    return k0, k1, k0 // F.QK, -(-k1 // F.QK)


def shard_raw(raw: torch.Tensor, wtype: int, parallel: str, rank: int, size: int):
    """raw uint8 [n_out, nb * B] of the full tensor -> (this rank's raw rows, KPad or None)."""
    bb = F.BYTES_PER_256[wtype]
    n_out, nb = raw.shape[0], raw.shape[1] // bb
    if parallel == "column":
        if n_out % size:
            raise ValueError(f"n_out={n_out} does not divide over {size} ranks")
        per = n_out // size
        return raw[rank * per:(rank + 1) * per].contiguous(), None
    if parallel == "row":
        k0, k1, b0, b1 = row_range(nb * F.QK, rank, size)
        shard = raw[:, b0 * bb:b1 * bb].contiguous()
        return shard, KPad(left=k0 - b0 * F.QK, own=k1 - k0, total=(b1 - b0) * F.QK)
    raise ValueError(parallel)


def pad_input(x: torch.Tensor, pad: KPad | None) -> torch.Tensor:
    """x [M, K/tp] -> [M, stored K] with zeros outside the rank's own range."""
    if pad is None or (pad.left == 0 and pad.own == pad.total):
        return x
    out = x.new_zeros((x.shape[0], pad.total))
    out[:, pad.left:pad.left + pad.own] = x
    return out


class PushAllReduce:
    """The library's one-shot all-reduce for small bf16 messages (gq_allreduce_push): each rank stores its vector
    into its slot of every peer's buffer over NVLink, publishes per-CTA flags, waits with a limit for the peers'
    flags and sums from its own memory in rank order.  Buffers come from torch's symmetric memory (peer-mapped
    allocations); messages above `max_bytes` go to NCCL."""

    def __init__(self, max_bytes: int = 64 * 5120 * 2, group=None):
        import ctypes

        import torch.distributed as dist
        import torch.distributed._symmetric_memory as symm_mem

        from ._lib import check, lib

        self.group = group if group is not None else dist.group.WORLD
        self.rank, self.world = dist.get_rank(self.group), dist.get_world_size(self.group)
        self.max_bytes = int(max_bytes)
        L = lib()
        nbytes = check(L.gq_allreduce_buffer_bytes(self.world, self.max_bytes), "gq_allreduce_buffer_bytes")
        self.buf = symm_mem.empty(nbytes, dtype=torch.uint8, device=torch.device("cuda", torch.cuda.current_device()))
        self.handle = symm_mem.rendezvous(self.buf, self.group)
        self.buf.zero_()
        torch.cuda.synchronize()
        dist.barrier(self.group)
        ptrs = [int(p) for p in self.handle.buffer_ptrs]
        assert len(ptrs) == self.world and ptrs[self.rank] == self.buf.data_ptr()
        self._ptrs = (ctypes.c_uint64 * self.world)(*ptrs)
        self._lib = L

    def status(self) -> int:
        off = 2 * 8 * 32 * 4 + 32 * 4      # behind the flags [2 sets][8 ranks][32 CTAs] and the 32 call counters (GQ_AR_CTAS in csrc/gq_b200.cu)
        return int(self.buf[off:off + 4].view(torch.int32).item())

    def __call__(self, t: torch.Tensor) -> torch.Tensor:
        from ._lib import check

        n = t.numel() * t.element_size()
        if t.dtype != torch.bfloat16 or not t.is_contiguous() or n > self.max_bytes or n % 16 or t.data_ptr() % 16:
            import torch.distributed as dist

            dist.all_reduce(t, op=dist.ReduceOp.SUM, group=self.group)
            return t
        check(self._lib.gq_allreduce_push(t.data_ptr(), t.data_ptr(), n, self.rank, self.world, self._ptrs, self.max_bytes,
                                          torch.cuda.current_stream(t.device).cuda_stream), "gq_allreduce_push")
        return t


class FusedAllReduce:
    """Peer buffers for the fused multiply + all-reduce of the row-parallel layers (gq_gemv_grouped_allreduce): the
    grouped kernel's epilogue exchanges the ranks' bf16 partial outputs and leaves their sum in the output, so a
    decode step needs no all-reduce launch at all.  One instance serves the row-parallel layers of ONE output width
    (the first call fixes n_total; the library rejects another width on the same buffers, because the exchanged words'
    positions depend on it) and up to `max_m` rows — in a decoder every row-parallel layer writes the hidden size, so
    one instance serves the whole model; use it through `ops.fused_allreduce(ctx)`."""

    def __init__(self, max_m: int = 64, max_n_total: int = 5120, group=None):
        import ctypes

        import torch.distributed as dist
        import torch.distributed._symmetric_memory as symm_mem

        from ._lib import check, lib

        self.group = group if group is not None else dist.group.WORLD
        self.rank, self.world = dist.get_rank(self.group), dist.get_world_size(self.group)
        self.max_m, self.max_n_total = int(max_m), int(max_n_total)
        nbytes = check(lib().gq_fused_allreduce_buffer_bytes(self.world, self.max_m, self.max_n_total), "gq_fused_allreduce_buffer_bytes")
        self.buf = symm_mem.empty(nbytes, dtype=torch.uint8, device=torch.device("cuda", torch.cuda.current_device()))
        self.handle = symm_mem.rendezvous(self.buf, self.group)
        self.buf.zero_()
        torch.cuda.synchronize()
        dist.barrier(self.group)
        ptrs = [int(p) for p in self.handle.buffer_ptrs]
        assert len(ptrs) == self.world and ptrs[self.rank] == self.buf.data_ptr()
        self.ptrs = (ctypes.c_uint64 * self.world)(*ptrs)
        self.used = False


class LocalFusedAllReduce:
    """The same context for a single process (world size 1, ordinary device memory): the exchange degenerates to a
    round trip through the rank's own buffer.  For tests on one GPU."""

    def __init__(self, max_m: int = 64, max_n_total: int = 5120, device=None):
        import ctypes

        from ._lib import check, lib

        self.rank, self.world = 0, 1
        self.max_m, self.max_n_total = int(max_m), int(max_n_total)
        nbytes = check(lib().gq_fused_allreduce_buffer_bytes(1, self.max_m, self.max_n_total), "gq_fused_allreduce_buffer_bytes")
        self.buf = torch.zeros(nbytes, dtype=torch.uint8, device=device or torch.device("cuda", torch.cuda.current_device()))
        self.ptrs = (ctypes.c_uint64 * 1)(self.buf.data_ptr())
        self.used = False


_FAST = None


def enable_push_all_reduce(max_bytes: int = 64 * 5120 * 2, group=None) -> PushAllReduce:
    """Route all_reduce_ of small bf16 tensors through the library's kernel (call on every rank, after
    init_process_group, outside stream capture)."""
    global _FAST
    _FAST = PushAllReduce(max_bytes, group)
    return _FAST


def disable_push_all_reduce() -> None:
    global _FAST
    _FAST = None


def all_reduce_(t: torch.Tensor, group=None) -> torch.Tensor:
    """Sum of the ranks' partial outputs: the library's push all-reduce for small bf16 messages when enabled,
    else NCCL over NVLink on GPUs (gloo on CPU)."""
    import torch.distributed as dist

    if dist.is_available() and dist.is_initialized() and dist.get_world_size(group) > 1:
        if _FAST is not None and t.is_cuda:
            return _FAST(t)
        dist.all_reduce(t, op=dist.ReduceOp.SUM, group=group)
    return t
