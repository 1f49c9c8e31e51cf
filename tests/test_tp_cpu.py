"""Tensor-parallel sharding logic on CPU: world_size-2 gloo ranks shard the raw GGUF bytes, multiply their
shard with the oracle, and all-reduce the row-parallel partial sums; the result must equal the unsharded
oracle product.  Also the tp = 8 case where K / tp is not a multiple of 256 (whole k-blocks kept, zero
activations outside the rank's own range)."""
import os

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from hyperqwen_rtx4080s32_b200 import formats as F
from hyperqwen_rtx4080s32_b200 import synth, tp
from oracle import oracle


def _rank_main(rank, world, port, results):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        k, n = 1024, 96
        for wtype in (F.Q4_K, F.IQ3_S, F.Q8_0):
            raw = synth.random_blocks(n, k, wtype, seed=3)
            x = synth.activations(4, k).float()
            full = oracle.matmul_f64(x.numpy(), raw.numpy(), wtype)
            # row-parallel: K split, partial sums all-reduced
            shard, pad = tp.shard_raw(raw, wtype, "row", rank, world)
            own = k // world
            xp = tp.pad_input(x[:, rank * own:(rank + 1) * own].contiguous(), pad)
            part = torch.from_numpy(oracle.matmul_f64(xp.numpy(), shard.numpy(), wtype))
            tp.all_reduce_(part)
            assert np.abs(part.numpy() - full).max() <= 1e-9 * np.abs(full).max()
            # column-parallel: rows split, outputs gathered
            cshard, cpad = tp.shard_raw(raw, wtype, "column", rank, world)
            assert cpad is None
            mine = torch.from_numpy(oracle.matmul_f64(x.numpy(), cshard.numpy(), wtype))
            parts = [torch.empty_like(mine) for _ in range(world)]
            dist.all_gather(parts, mine)
            assert np.array_equal(torch.cat(parts, dim=1).numpy(), full)
        results[rank] = "ok"
    finally:
        dist.destroy_process_group()


def test_tp2_gloo_row_and_column_parallel():
    ctx = mp.get_context("spawn")
    with ctx.Manager() as mgr:
        results = mgr.dict()
        port = 29500 + os.getpid() % 2000
        procs = [ctx.Process(target=_rank_main, args=(r, 2, port, results)) for r in range(2)]
        for p in procs:
            p.start()
        for p in procs:
            p.join(120)
            assert p.exitcode == 0
        assert dict(results) == {0: "ok", 1: "ok"}


@pytest.mark.parametrize("k,size", [(5120, 8), (17408, 8), (5120, 4), (1024, 8)])
def test_row_sharding_keeps_whole_blocks(k, size):
    wtype, n = F.Q4_K, 8
    raw = synth.random_blocks(n, k, wtype, seed=1)
    x = synth.activations(2, k).float()
    full = oracle.matmul_f64(x.numpy(), raw.numpy(), wtype)
    total = np.zeros_like(full)
    stored = 0
    for rank in range(size):
        shard, pad = tp.shard_raw(raw, wtype, "row", rank, size)
        assert shard.shape[1] % F.BYTES_PER_256[wtype] == 0 and pad.total == shard.shape[1] // F.BYTES_PER_256[wtype] * 256
        assert pad.left in (0, 128) or (k // size) % 256 == 0 or pad.left % 32 == 0
        own = k // size
        xp = tp.pad_input(x[:, rank * own:(rank + 1) * own].contiguous(), pad)
        assert xp.shape[1] == pad.total
        total += oracle.matmul_f64(xp.numpy(), shard.numpy(), wtype)
        stored += shard.shape[1]
    assert np.abs(total - full).max() <= 1e-9 * np.abs(full).max()
    if (k // size) % 256 == 0:
        assert stored == raw.shape[1]            # nothing duplicated when the cut falls on block boundaries


def test_row_sharding_rejects_bad_splits():
    raw = synth.random_blocks(4, 1024, F.Q4_K, seed=1)
    with pytest.raises(ValueError):
        tp.shard_raw(raw, F.Q4_K, "row", 0, 3)
    with pytest.raises(ValueError):
        tp.shard_raw(raw, F.Q4_K, "column", 0, 3)
