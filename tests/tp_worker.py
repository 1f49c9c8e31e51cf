"""Worker of tests/test_multi_gpu.py: the multi-GPU checks, one process per GPU:

    python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 --master-port P tests/tp_worker.py

Every rank all-reduces seeded bf16 vectors of several sizes with both paths (the push kernel sums in fp32 in
rank order and rounds once; NCCL's result may differ in the last bf16 bit), repeatedly, eagerly and from a
replayed CUDA graph, and times both; then a two-block tensor-parallel stack runs with the all-reduce fused into
the grouped kernel and with the separate push kernel, which must agree bit for bit and must match the fp64 oracle of
the unsharded layer; a fused-exchange buffer refuses a second output width.  Exits non-zero on a mismatch or a device
status other than 0.
"""
from __future__ import annotations

import datetime
import os
import sys

import numpy as np
import torch
import torch.distributed as dist

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

from hyperqwen_rtx4080s32_b200 import _lib, ops, synth, tp  # noqa: E402
from oracle import oracle  # noqa: E402


def main() -> int:
    rank, world, local = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"]), int(os.environ["LOCAL_RANK"])
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    os.environ.setdefault("TORCH_NCCL_ASYNC_ERROR_HANDLING", "0")
    dist.init_process_group("nccl", device_id=dev, timeout=datetime.timedelta(seconds=120))
    fast = tp.PushAllReduce(max_bytes=64 * 5120 * 2)
    ok = True
    for m in (1, 8, 64):
        for rep in range(5):
            g = torch.Generator(device=dev).manual_seed(1000 * rank + 10 * m + rep)
            x = torch.randn((m, 5120), generator=g, device=dev).to(torch.bfloat16)
            ref = x.clone()
            dist.all_reduce(ref)
            parts = [torch.empty_like(x) for _ in range(world)]
            dist.all_gather(parts, x)
            exact = torch.stack([p.float() for p in parts]).sum(0).to(torch.bfloat16)
            y = fast(x.clone())
            torch.cuda.synchronize()
            if not torch.equal(y, exact) or (y.float() - ref.float()).abs().max() > 0.02 * ref.float().abs().max():
                ok = False
                print(f"[rank {rank}] mismatch at M={m} rep={rep}: max diff {(y.float() - exact.float()).abs().max().item()}", flush=True)
    # graph replay + timing
    x = torch.randn((8, 5120), device=dev).to(torch.bfloat16)
    bufs = [x.clone() for _ in range(64)]
    for name, fn in (("push", fast), ("nccl", lambda t: dist.all_reduce(t))):
        for b in bufs[:4]:
            fn(b)
        torch.cuda.synchronize()
        g = torch.cuda.CUDAGraph()
        s = torch.cuda.Stream()
        s.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(s):
            with torch.cuda.graph(g, stream=s, capture_error_mode="thread_local"):
                for b in bufs:
                    fn(b)
        torch.cuda.current_stream().wait_stream(s)
        for _ in range(3):
            g.replay()
        torch.cuda.synchronize()
        dist.barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(5):
            g.replay()
        e1.record()
        torch.cuda.synchronize()
        if rank == 0:
            print(f"{name}: {1e3 * e0.elapsed_time(e1) / (5 * len(bufs)):.2f} us per all-reduce of {x.numel() * 2} bytes over {world} GPUs (graph replay)", flush=True)
    # fused multiply + all-reduce against the unfused path (grouped kernel, then the push all-reduce): the same
    # bf16 partial outputs summed in the same order, so the results must be bit-identical
    from hyperqwen_rtx4080s32_b200 import formats as F, stack as S

    types = [{"q": F.Q4_K, "k": F.Q4_K, "v": F.Q4_K, "o": F.IQ4_XS, "gate": F.Q2_K, "up": F.Q2_K, "down": F.Q6_K},
             {"q": F.IQ3_S, "k": F.Q8_0, "v": F.Q3_K, "o": F.Q5_K, "gate": F.IQ3_S, "up": F.Q3_K, "down": F.Q4_K}]
    stk = S.LinearStack(n_layers=2, device=dev, tp_rank=rank, tp_size=world, types=types)
    tp._FAST = fast
    for m in (1, 8, 33, 64):
        xin = stk.make_inputs(m)
        outs = {}
        for mode in ("unfused", "fused"):
            stk.fused_ar = None
            if mode == "fused":
                if not hasattr(stk, "_far"):
                    stk._far = tp.FusedAllReduce(max_m=64, max_n_total=stk.hidden)
                stk.fused_ar = stk._far
            res = []
            for rep in range(3):
                res.append(stk.step(xin).clone())
            torch.cuda.synchronize()
            outs[mode] = res
        for a, b in zip(outs["unfused"], outs["fused"]):
            if not torch.equal(a, b) or torch.isnan(b).any():
                ok = False
                print(f"[rank {rank}] fused all-reduce differs from the unfused path at M={m}: max diff {(a.float() - b.float()).abs().max().item()}", flush=True)
        # against the oracle of the unsharded layer: the step returns the last block's down projection, summed over ranks
        # (each rank's partial output is rounded to bf16 before the sum: `world` roundings instead of one)
        n_out, k = stk.full_shapes["down"]
        t_down = types[-1]["down"]
        raw = synth.random_blocks(n_out, k, t_down, seed=20261125 % 100000 + 1000 * (len(types) - 1) + 10 * S.TENSORS.index("down"),
                                  device=dev).cpu()      # drawn on the device, as the stack draws it
        x_full = synth.activations(m, k, seed=100 + m + 7)
        rows = np.unique(np.concatenate([np.linspace(0, n_out - 1, 48).astype(np.int64), [0, 63, 64, n_out - 1]]))
        ref = oracle.matmul_f64(x_full.float().numpy(), raw[torch.from_numpy(rows)].numpy(), t_down)
        got = outs["fused"][0][:, torch.from_numpy(rows).to(dev)].float().cpu().numpy()
        err = oracle.rel_err(got, ref)
        if not err < 6e-3 * (1 + 0.5 * (world - 1)):
            ok = False
            print(f"[rank {rank}] tensor-parallel down projection against the oracle at M={m}: rel err {err:.3e}", flush=True)
    # ... and replayed from a CUDA graph
    xin = stk.make_inputs(8)
    stk.fused_ar = stk._far
    want = stk.step(xin).clone()
    torch.cuda.synchronize()
    g = torch.cuda.CUDAGraph()
    s = torch.cuda.Stream()
    s.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(s):
        with torch.cuda.graph(g, stream=s, capture_error_mode="thread_local"):
            got = stk.step(xin)
    torch.cuda.current_stream().wait_stream(s)
    for _ in range(3):
        g.replay()
    torch.cuda.synchronize()
    if not torch.equal(got, want):
        ok = False
        print(f"[rank {rank}] fused all-reduce: graph replay differs", flush=True)
    # the row-parallel down projection with silu_and_mul folded into its preparation, summed over the ranks in the same call
    lin_down = stk.layers[-1]["down"]
    for m in (1, 8, 16):
        up = stk.make_inputs(m)["down"]                                  # this rank's K columns (zero outside its own range)
        gate = synth.activations(m, up.shape[1], seed=900 + m + rank, device=dev)
        gu = torch.cat([gate, up], dim=1)
        with ops.fused_allreduce(stk._far):
            stk._far.used = False
            want_y = lin_down(ops.PreSiluMul().unfused(gu)).clone()
            stk._far.used = False
            got_y = lin_down(gu, pre=ops.PreSiluMul()).clone()
            folded_used = stk._far.used
        torch.cuda.synchronize()
        differ = (got_y != want_y).float().mean().item()
        err = oracle.rel_err(got_y.float().cpu().numpy(), want_y.float().cpu().numpy())
        if not folded_used or torch.isnan(got_y).any() or differ > 0.05 or err > 4e-3:
            ok = False
            print(f"[rank {rank}] folded silu_and_mul + fused all-reduce at M={m}: used {folded_used}, {differ:.4f} of the outputs differ, rel err {err:.3e}", flush=True)
    # a fused-exchange buffer is bound to the output width it was first used with
    lin_small = S.GGUFLinear(1024, [256])
    lin_small.load_shard(synth.random_blocks(256, 1024, F.Q4_K, seed=5).to(dev), F.Q4_K)
    lin_small.finalize()
    try:
        with ops.fused_allreduce(stk._far):
            stk._far.used = False
            lin_small(synth.activations(8, 1024, device=dev))
        refused = False
    except _lib.GqError:
        refused = True
    if not refused:
        ok = False
        print(f"[rank {rank}] a second output width on one fused all-reduce buffer was not refused", flush=True)
    st = max(fast.status(), ops.device_status(dev))
    if st != 0:
        ok = False
        print(f"[rank {rank}] device status {st}", flush=True)
    flag = torch.tensor([1 if ok else 0], device=dev)
    dist.all_reduce(flag, op=dist.ReduceOp.MIN)
    if rank == 0:
        print("tp_worker", "ok" if int(flag.item()) else "FAILED", flush=True)
    dist.barrier()
    torch.cuda.synchronize()
    sys.stdout.flush()
    os._exit(0 if int(flag.item()) else 1)


if __name__ == "__main__":
    main()
