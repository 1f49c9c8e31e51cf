"""Per-type decode micro-benchmark (the per-type sweep of the dense-decoder projection shapes):

    python -m hyperqwen_rtx4080s32_b200.microbench --types Q4_K Q6_K --shapes gate kv --m 1 8 [--split 1 2] [--eager --iters 3]

For each type x shape x batch it times the grouped kernel alone (activations prepared beforehand) and the
whole call (prepare + kernel + partial sum) as CUDA-graph replays over distinct weight copies totalling
more than the L2, median of 7 — the reference's timing method (gguf-plugin/test_gluon_kq_gpu.py:198-245) —
and prints microseconds and GB/s of raw GGUF block bytes.  --eager launches the kernel a few times without
a graph (the form a profiler capture wants).
"""
from __future__ import annotations

import argparse

import numpy as np
import torch

from . import _lib, formats as F, ops, synth

SHAPES = {"q": (5120, 5120), "kv": (1024, 5120), "o": (5120, 5120), "gate": (17408, 5120), "down": (5120, 17408)}


def _graph_time(fn, n: int, reps: int = 7) -> float:
    g = torch.cuda.CUDAGraph()
    s = torch.cuda.Stream()
    s.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(s):
        fn()
        s.synchronize()
        with torch.cuda.graph(g, stream=s):
            fn()
    torch.cuda.current_stream().wait_stream(s)
    for _ in range(3):
        g.replay()
    ts = []
    for _ in range(reps):
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        g.replay()
        e1.record()
        torch.cuda.synchronize()
        ts.append(e0.elapsed_time(e1))
    return float(np.median(ts)) / n


def prefill_main(a, dev) -> None:
    """Grouped gate_up (K 5120, N 2 x 17408) and down (K 17408, N 5120) at prefill batch sizes: milliseconds and
    TFLOP/s (2 M K N; dequantisation not counted), the whole call (activation layout + the tcgen05 kernel)."""
    shapes = {"gate_up": ([17408, 17408], 5120), "down": ([5120], 17408), "q": ([5120], 5120)}
    for tn in a.types:
        t = F.TYPE_IDS[tn]
        for sn in [s for s in a.shapes if s in shapes] or ["gate_up", "down"]:
            n_outs, k = shapes[sn]
            tiles = [ops.repack_tiles(synth.random_blocks(n, k, t, seed=i, device=dev), n, t) for i, n in enumerate(n_outs)]
            packed, views, descs, splits, nb, bb = ops.prepare_grouped_layer(tiles, n_outs, [t] * len(n_outs))
            del tiles
            d1 = descs[splits.index(1)]
            n_total = sum(n_outs)
            for m in a.m:
                x = synth.activations(m, k, device=dev)
                y = torch.empty((m, n_total), dtype=torch.bfloat16, device=dev)
                for _ in range(2):
                    ops.prefill_gemm(x, packed, d1, n_total, out=y)
                torch.cuda.synchronize()
                if a.eager:
                    print(f"{tn:7} {sn:8} M={m}: eager", flush=True)
                    continue
                ts = []
                for _ in range(5):
                    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                    e0.record()
                    ops.prefill_gemm(x, packed, d1, n_total, out=y)
                    e1.record()
                    torch.cuda.synchronize()
                    ts.append(e0.elapsed_time(e1))
                ms = float(np.median(ts))
                print(f"{tn:7} {sn:8} K={k} N={n_total} M={m:5}: {ms:8.3f} ms  {2.0 * m * k * n_total / ms / 1e9:7.1f} TFLOP/s", flush=True)
            del packed, views, descs
            torch.cuda.empty_cache()


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--types", nargs="*", default=list(F.TYPE_IDS))
    ap.add_argument("--shapes", nargs="*", default=["q", "kv", "gate", "down"])
    ap.add_argument("--m", nargs="*", type=int, default=[1, 8])
    ap.add_argument("--split", nargs="*", type=int, default=[])
    ap.add_argument("--copies-mb", type=float, default=600.0)
    ap.add_argument("--prefill", action="store_true", help="time the large-batch tcgen05 path on gate_up / down (TFLOP/s)")
    ap.add_argument("--eager", action="store_true")
    ap.add_argument("--iters", type=int, default=3)
    a = ap.parse_args()
    dev = torch.device("cuda", 0)
    L = _lib.lib()
    if a.prefill:
        return prefill_main(a, dev)
    for tn in a.types:
        t = F.TYPE_IDS[tn]
        for sn in a.shapes:
            n_out, k = SHAPES[sn] if sn in SHAPES else tuple(int(v) for v in sn.split("x"))   # a name or "NxK"
            nbytes = F.raw_bytes(t, n_out, k)
            ncopy = max(2, int(a.copies_mb * 1e6 // nbytes)) if a.copies_mb > 0 else 1
            packs = []
            for c in range(ncopy):
                raw = synth.random_blocks(n_out, k, t, seed=c, device=dev)
                packs.append(ops.repack_tiles(raw, n_out, t).reshape(-1))
                del raw
            nb, n_tiles = k // 256, -(-n_out // 64)
            if a.copies_mb <= 0:
                packs = packs * 8        # --copies-mb 0: one copy, replayed eight times per graph (weights stay in L2)
                ncopy = 8
            for m in a.m:
                x = synth.activations(m, k, device=dev)
                auto = ops.grouped_split_for(n_tiles, nb, m=m, block_bytes=F.BYTES_PER_256[t])
                cells = []
                for s in (a.split or [auto]):
                    if s > nb:
                        continue
                    d = torch.from_numpy(ops.build_descs([t], [n_out], k, s)).to(dev)
                    ws = torch.empty(L.gq_workspace_bytes(m, k, n_out, s), dtype=torch.uint8, device=dev)
                    y = torch.empty((m, n_out), dtype=torch.bfloat16, device=dev)
                    ops.grouped_gemm(x, packs[0], d, s, [t], n_out, out=y, workspace=ws, phases=1)

                    def kernel_only():
                        for p in packs:
                            ops.grouped_gemm(x, p, d, s, [t], n_out, out=y, workspace=ws, phases=2)

                    def whole_call():
                        for p in packs:
                            ops.grouped_gemm(x, p, d, s, [t], n_out, out=y, workspace=ws, phases=7)

                    if a.eager:
                        for _ in range(a.iters):
                            kernel_only()
                        torch.cuda.synchronize()
                        cells.append(f"S{s}: eager x{a.iters * ncopy}")
                        continue
                    us = 1e3 * _graph_time(kernel_only, ncopy)
                    us_all = 1e3 * _graph_time(whole_call, ncopy)
                    cells.append(f"S{s}: {us:7.1f} us {nbytes / us / 1e3:6.0f} GB/s (call {us_all:6.1f} us)")
                print(f"{tn:7} {sn:5} {n_out}x{k} M={m:2} auto-split={auto} copies={ncopy} | " + " | ".join(cells), flush=True)
            del packs
            torch.cuda.empty_cache()


if __name__ == "__main__":
    main()
