"""Multi-GPU check of the push all-reduce against NCCL, one process per GPU:

    python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 --master-port P \\
        -m hyperqwen_rtx4080s32_b200.tp_check

Every rank all-reduces seeded bf16 vectors of several sizes with both paths (the push kernel sums in fp32 in
rank order and rounds once; NCCL's result may differ in the last bf16 bit), repeatedly, eagerly and from a
replayed CUDA graph, and times both; then a two-block tensor-parallel stack runs with the all-reduce fused into
the grouped kernel and with the separate push kernel, which must agree bit for bit.  Exits non-zero on a mismatch
or a device timeout status.
"""
from __future__ import annotations

import datetime
import os
import sys

import torch
import torch.distributed as dist

from . import tp


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
    from . import formats as F, stack as S

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
    st = fast.status()
    if st != 0:
        ok = False
        print(f"[rank {rank}] device status {st}", flush=True)
    flag = torch.tensor([1 if ok else 0], device=dev)
    dist.all_reduce(flag, op=dist.ReduceOp.MIN)
    if rank == 0:
        print("tp_check", "ok" if int(flag.item()) else "FAILED", flush=True)
    dist.barrier()
    torch.cuda.synchronize()
    sys.stdout.flush()
    os._exit(0 if int(flag.item()) else 1)


if __name__ == "__main__":
    main()
