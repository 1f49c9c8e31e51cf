#!/usr/bin/env python
"""Benchmark of the GGUF quantized-linear path on B200.

    python bench.py --gpus N --steps K --warmup W [--impl reference] [--m 8] [--layers 64]

Workload (config.workload): the mixed-type 64-layer decoder linear stack (hidden 5120, 40 q / 8 kv heads
of 128, intermediate 17408; eleven GGML types, about 3.88 bits per weight, 10.25 GB of raw block bytes)
at decode batch M = 8.  A step is one pass of all 256 linears over one batch of synthetic bf16
activations.  `value` is GB/s of raw GGUF block bytes (the reference's convention for its decode kernel)
with inputs resident in HBM, the step replayed as one CUDA graph; `e2e` is the same metric through
GGUFLinearMethod.apply with pinned host inputs copied in and the result copied out inside the timed
region.  With N > 1 the stack is tensor-parallel (column-split qkv / gate_up, row-split o / down, one
NCCL all-reduce per row-parallel layer) and the whole job's bytes are divided by the slowest rank's time
(strong scaling).  `--impl reference` times the CPU restatement of the reference's dequantise-and-multiply
path on the host cores instead.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

METRIC = "decode GEMV HBM GB/s of raw GGUF block bytes (mixed-type 64-layer linear stack)"


def measured_peaks():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        try:
            return json.load(open(p)), "measured"
        except Exception:
            pass
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0}, "fallback"


class ClockSampler:
    """Samples nvidia-smi clocks and throttle reasons every 200 ms while the timed region runs."""
    Q = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
         "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int):
        self.index, self.rows, self.proc = index, [], None

    def __enter__(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--id={self.index}", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits", "-lms", "200"],
                                         stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except Exception:
            self.proc = None
        return self

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append([c.strip() for c in line.split(",")])

    def __exit__(self, *a):
        if self.proc is not None:
            time.sleep(0.25)
            self.proc.terminate()
            try:
                self.proc.wait(timeout=2)
            except Exception:
                self.proc.kill()

    def summary(self):
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for r in self.rows:
            try:
                sm.append(float(r[0])); mx.append(float(r[1]))
                for n, v in zip(names, r[3:7]):
                    if v.lower().startswith("active"):
                        reasons.add(n)
            except Exception:
                continue
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": sorted(reasons), "samples": len(sm)}


def cpu_sample(m: int, n_layers: int, target_s: float = 0.0):
    """The CPU path on a bounded sample: the first n_layers blocks of the stack (same type draw, seeded
    random valid blocks), x . dequantize(W)^T fused in C with all host threads; with target_s the sample is
    passed over repeatedly until about that many seconds of CPU work are done.  Returns (GB/s, seconds, dict)."""
    import numpy as np

    from hyperqwen_rtx4080s32_b200 import formats as F
    from hyperqwen_rtx4080s32_b200 import stack as S
    from hyperqwen_rtx4080s32_b200 import synth
    from oracle import oracle

    oracle.use_all_cores()
    types = S.draw_types(64)[:n_layers]
    shapes = {"q": (5120, 5120), "k": (1024, 5120), "v": (1024, 5120), "o": (5120, 5120), "gate": (17408, 5120),
              "up": (17408, 5120), "down": (5120, 17408)}
    tensors, nbytes = [], 0
    for li, t in enumerate(types):
        for name in S.TENSORS:
            n_out, k = shapes[name]
            raw = synth.random_blocks(n_out, k, t[name], seed=1000 * li + 10 * S.TENSORS.index(name)).numpy()
            tensors.append((raw, t[name], k))
            nbytes += raw.size
    xs = {k: synth.activations(m, k).float().numpy() for k in (5120, 17408)}
    oracle.lib()
    passes, dt = 0, 0.0
    while True:
        t0 = time.perf_counter()
        for raw, wt, k in tensors:
            oracle.matmul_c(xs[k], raw, wt)
        dt += time.perf_counter() - t0
        passes += 1
        if dt >= target_s or passes >= 200:
            break
    info = {"cores": oracle.num_threads(), "kind": "port",
            "sample": f"{n_layers} of 64 blocks ({nbytes / 1e6:.0f} MB of raw blocks) at M={m}, {passes} passes, fused dequantise-and-dot in C (OpenMP), {dt:.1f} s of CPU work"}
    return passes * nbytes / dt / 1e9, dt / passes, info


_emit = print      # replaced in main() by a writer to the process's original stdout


def run_reference(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    from oracle import oracle

    oracle.use_all_cores()
    vals = []
    for _ in range(min(args.warmup, 1)):
        cpu_sample(args.m, 1)
    times = []
    for _ in range(args.steps):
        v, dt, info = cpu_sample(args.m, 1, target_s=min(10.0, 120.0 / max(1, args.steps)))
        vals.append(v); times.append(dt)
    value = statistics.mean(vals)
    line = {"impl": "reference", "metric": METRIC, "value": value, "unit": "GB/s", "n_gpus": args.gpus, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": 1e3 * statistics.mean(times), "higher_is_better": True, "scaling": "strong",
            "vs_baseline": None, "dtype": "f32", "data": "synthetic",
            "config": {"workload": f"mixed-type 64-layer GGUF decoder linear stack (BASELINE configs[3]), decode M={args.m}",
                       "sample": "each step a bounded sample of that workload on the host cores: 1 of its 64 blocks, passed over for about 10 s"},
            "cpu_baseline": dict(info, value=value, unit="GB/s"),
            "e2e": {"value": value, "unit": "GB/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}, "gpu_launches": 0}
    _emit(json.dumps(line))


def gguf_py_sample(m: int):
    """BASELINE's reference-equivalent CPU path on one tensor: gguf.quants.dequantize to fp32 (numpy), then torch fp32
    x @ W.T on all host threads; dequantise and multiply timed separately.  One q projection (5120 x 5120, Q4_K)."""
    import numpy as np
    import torch
    from gguf.quants import dequantize
    from gguf.constants import GGMLQuantizationType

    from hyperqwen_rtx4080s32_b200 import formats as F
    from hyperqwen_rtx4080s32_b200 import synth

    n_out, k = 5120, 5120
    raw = synth.random_blocks(n_out, k, F.Q4_K, seed=1).numpy()
    x = synth.activations(m, k).float()
    t0 = time.perf_counter()
    w = torch.from_numpy(np.ascontiguousarray(dequantize(raw, GGMLQuantizationType.Q4_K).reshape(n_out, k)))
    t1 = time.perf_counter()
    for _ in range(3):
        y = x @ w.T
    t2 = time.perf_counter()
    mm = (t2 - t1) / 3
    return {"tensor": "q 5120 x 5120 Q4_K", "raw_bytes": int(raw.size), "dequantize_s": t1 - t0, "matmul_s": mm, "threads": torch.get_num_threads(),
            "gbs_per_call_dequantise_every_call": raw.size / (t1 - t0 + mm) / 1e9, "gbs_matmul_only_weights_kept_fp32": raw.size / mm / 1e9,
            "what": "gguf.quants.dequantize (numpy) then torch fp32 x @ W.T, M=%d" % m}


def parity_before_timing(st, m, rank, world, dev):
    """One column-parallel (qkv) and one row-parallel (down, summed over ranks) layer of block 0 against the fp64 oracle
    on a subset of output columns, through the same calls the timed step makes.  Outside the timed region."""
    import numpy as np
    import torch

    from hyperqwen_rtx4080s32_b200 import stack as S
    from hyperqwen_rtx4080s32_b200 import synth
    from hyperqwen_rtx4080s32_b200 import tp as _tp
    from oracle import oracle

    x = st.make_inputs(m)
    seed = 20261125 % 100000
    t = st.types[0]
    errs = {}
    # column-parallel: this rank's rows of q
    y = st.layers[0]["qkv"](x["qkv"])
    n_out, k = st.full_shapes["q"]
    raw = synth.random_blocks(n_out, k, t["q"], seed=seed + 10 * S.TENSORS.index("q"), device=dev).cpu()    # as the stack draws it
    if world > 1:
        raw, _ = _tp.shard_raw(raw, t["q"], "column", rank, world)
    rows = np.unique(np.concatenate([np.linspace(0, raw.shape[0] - 1, 40).astype(np.int64), [0, 63, raw.shape[0] - 1]]))
    ref = oracle.matmul_f64(x["qkv"].float().cpu().numpy(), raw[torch.from_numpy(rows)].numpy(), t["q"])
    errs["qkv"] = float(oracle.rel_err(y[:, torch.from_numpy(rows).to(dev)].float().cpu().numpy(), ref))
    # row-parallel: down, the sum over ranks against the unsharded layer
    one = S.LinearStack.__new__(S.LinearStack)
    one.__dict__.update(st.__dict__)
    one.layers = st.layers[:1]
    y = one.step(x)
    n_out, k = st.full_shapes["down"]
    raw = synth.random_blocks(n_out, k, t["down"], seed=seed + 10 * S.TENSORS.index("down"), device=dev).cpu()
    x_full = synth.activations(m, k, seed=100 + m + 7)
    rows = np.unique(np.concatenate([np.linspace(0, n_out - 1, 40).astype(np.int64), [0, 63, n_out - 1]]))
    ref = oracle.matmul_f64(x_full.float().numpy(), raw[torch.from_numpy(rows)].numpy(), t["down"])
    errs["down"] = float(oracle.rel_err(y[:, torch.from_numpy(rows).to(dev)].float().cpu().numpy(), ref))
    torch.cuda.synchronize()
    return errs


# gguf-plugin/README.md:139-145: the reference's per-launch figures at 8 rows on its RTX 4080 SUPER, (microseconds, GB/s)
REFERENCE_TABLE_M8 = {
    (1024, 5120): {"Q3_K": (6.7, 335), "Q5_K": (8.9, 403), "Q6_K": (9.4, 458), "Q8_0": (11.2, 498), "Q4_K": (7.9, 373)},
    (6144, 5120): {"Q3_K": (24.7, 546), "Q5_K": (36.7, 589), "Q6_K": (42.2, 612), "Q8_0": (52.1, 642), "Q4_K": (30.7, 577)},
    (17408, 5120): {"Q3_K": (61.6, 622), "Q5_K": (94.8, 646), "Q6_K": (116.3, 629), "Q8_0": (148.3, 639), "Q4_K": (78.1, 642)},
    (5120, 6144): {"Q3_K": (25.3, 534), "Q5_K": (35.8, 603), "Q6_K": (41.5, 623), "Q8_0": (52.0, 643), "Q4_K": (30.1, 587)},
    (248320, 5120): {"Q3_K": (830.7, 658), "Q5_K": (1288.0, 679), "Q6_K": (1570.7, 664), "Q8_0": (1961.6, 689), "Q4_K": (1057.7, 676)},
}


def run_ours(args):
    import torch
    import torch.distributed as dist

    from hyperqwen_rtx4080s32_b200 import _lib, ops
    from hyperqwen_rtx4080s32_b200 import stack as S

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: the quantized-linear path has no CPU fallback (use --impl reference for the CPU arm)")
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        import datetime

        # graph capture of NCCL collectives: the watchdog thread must not touch CUDA while a capture is open
        os.environ.setdefault("TORCH_NCCL_ASYNC_ERROR_HANDLING", "0")
        dist.init_process_group("nccl", device_id=dev, timeout=datetime.timedelta(seconds=180))
        if not args.nccl_allreduce:
            from hyperqwen_rtx4080s32_b200 import tp as _tp

            # the one-shot push all-reduce serves up to 64 rows; larger messages (M = 4096) go to NCCL
            _tp.enable_push_all_reduce(max_bytes=64 * 5120 * 2)
    L = _lib.lib()
    st = S.LinearStack(n_layers=args.layers, device=dev, tp_rank=rank, tp_size=world)
    fused = world > 1 and not args.nccl_allreduce and not args.unfused_allreduce
    if fused:
        try:
            st.enable_fused_all_reduce(max_m=64)
        except Exception as e:      # no peer-mapped memory on this box: the separate all-reduce still works
            print(f"[rank {rank}] fused all-reduce unavailable ({e}): using the separate all-reduce", file=sys.stderr, flush=True)
            st.fused_ar = None
        ready = torch.tensor([1 if getattr(st, "fused_ar", None) is not None else 0], device=dev)
        dist.all_reduce(ready, op=dist.ReduceOp.MIN)
        if int(ready.item()) == 0:
            st.fused_ar = None
            fused = False
    if fused:
        # the fused exchange must reproduce the separate all-reduce bit for bit on this process group before it is
        # timed; if any rank sees a difference the run falls back to the separate push kernel and says so
        from hyperqwen_rtx4080s32_b200 import tp as _tp

        xin = st.make_inputs(args.m)
        lin = st.layers[0]["o"]
        want = lin(xin["o"]).clone()
        _tp.all_reduce_(want)
        st.fused_ar.used = False
        with ops.fused_allreduce(st.fused_ar):
            got = lin(xin["o"])
        torch.cuda.synchronize()
        same = torch.tensor([1 if (st.fused_ar.used and torch.equal(got, want)) else 0], device=dev)
        dist.all_reduce(same, op=dist.ReduceOp.MIN)
        if int(same.item()) == 0:
            print(f"[rank {rank}] fused all-reduce self-check failed: using the separate push kernel", file=sys.stderr, flush=True)
            st.fused_ar = None
            fused = False
    st.enable_prefetch(args.l2_prefetch and not args.no_l2_prefetch)

    def barrier():
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def timed(fn, steps):
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        barrier()
        e0.record()
        for _ in range(steps):
            fn()
        e1.record()
        barrier()
        ms = e0.elapsed_time(e1)
        if world > 1:
            t = torch.tensor([ms], device=dev)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            ms = float(t.item())
        return ms / steps

    # ---- parity before timing (oracle outside the timed region) ----
    parity = parity_before_timing(st, args.m, rank, world, dev)
    if max(parity.values()) >= 1e-2:
        raise SystemExit(f"[rank {rank}] parity check failed before timing: {parity}")

    side = torch.cuda.Stream()

    def capture_step(m, skip_all_reduce=False):
        """Warm up, then capture one pass of the stack at M rows as a CUDA graph; returns (replay fn, output, captured, inputs)."""
        x_dev = st.make_inputs(m)
        st.skip_all_reduce = skip_all_reduce
        out = None
        for _ in range(max(3, args.warmup) if m <= 64 else 1):
            out = st.step(x_dev)
        torch.cuda.synchronize()
        graph = torch.cuda.CUDAGraph()
        side.wait_stream(torch.cuda.current_stream())
        captured = 1
        try:
            with torch.cuda.stream(side):
                with torch.cuda.graph(graph, stream=side, capture_error_mode="thread_local"):
                    out = st.step(x_dev)
        except Exception as e:   # noqa: BLE001 - a failed capture falls back to eager stepping on every rank
            captured = 0
            print(f"[rank {rank}] CUDA graph capture failed at M={m}, stepping eagerly: {e}", file=sys.stderr, flush=True)
        torch.cuda.current_stream().wait_stream(side)
        torch.cuda.synchronize()
        if world > 1:
            flag = torch.tensor([captured], device=dev)
            dist.all_reduce(flag, op=dist.ReduceOp.MIN)
            captured = int(flag.item())
        st.skip_all_reduce = False
        if captured:
            return graph.replay, out, captured, x_dev, graph

        def eager():
            st.skip_all_reduce = skip_all_reduce
            st.step(x_dev)
            st.skip_all_reduce = False
        return eager, out, captured, x_dev, None

    # ---- the headline: M = args.m ----
    m = args.m
    launches0 = L.gq_launch_count()
    st.step(st.make_inputs(m))
    torch.cuda.synchronize()
    launches_per_step = L.gq_launch_count() - launches0
    run_step, out, captured, x_dev, _g = capture_step(m)
    x_host = {k: v.cpu().pin_memory() for k, v in x_dev.items()}
    out_host = torch.empty((m, st.hidden), dtype=torch.bfloat16).pin_memory()
    for _ in range(max(3, args.warmup)):
        run_step()
    barrier()
    with ClockSampler(local) as clk:
        ms_step = timed(run_step, args.steps)

    def e2e_step():
        for k in x_dev:
            x_dev[k].copy_(x_host[k], non_blocking=True)
        run_step()
        out_host.copy_(out, non_blocking=True)

    for _ in range(3):
        e2e_step()
    ms_e2e = timed(e2e_step, args.steps)
    h2d = sum(v.numel() * 2 for v in x_host.values())
    d2h = out_host.numel() * 2

    # where a step's time goes: the grouped kernel alone (activations prepared beforehand) — the roofline's launch
    # time —, the activation preparation alone, and (tensor parallel) the step without its all-reduces
    runs = []
    for blk in st.layers:
        for name in ("qkv", "o", "gate_up", "down"):
            lin = blk[name]
            for first, (packed, descs, splits, run, nb, block_bytes) in lin.gguf_groups.items():
                n_outs = [lin.gguf_tiles_rows[i] for i in run]
                wts = [lin.gguf_tiles_types[i] for i in run]
                n_tiles = sum(-(-n // 64) for n in n_outs)
                s = ops.grouped_split_for(n_tiles, nb, m=m, block_bytes=block_bytes, sms=ops.sm_count(dev))
                s = s if s in splits else 1
                nt = sum(n_outs)
                ws = torch.empty(L.gq_workspace_bytes(m, nb * 256, nt, s), dtype=torch.uint8, device=dev)
                y = torch.empty((m, nt), dtype=torch.bfloat16, device=dev)
                runs.append((x_dev[name], packed, descs[splits.index(s)], s, wts, nt, y, ws))

    def phase_graph(phases):
        for r in runs:
            ops.grouped_gemm(r[0], r[1], r[2], r[3], r[4], r[5], out=r[6], workspace=r[7], phases=1)
        g = torch.cuda.CUDAGraph()
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):
            for r in runs:
                ops.grouped_gemm(r[0], r[1], r[2], r[3], r[4], r[5], out=r[6], workspace=r[7], phases=phases)
            side.synchronize()
            with torch.cuda.graph(g, stream=side):
                for r in runs:
                    ops.grouped_gemm(r[0], r[1], r[2], r[3], r[4], r[5], out=r[6], workspace=r[7], phases=phases)
        torch.cuda.current_stream().wait_stream(side)
        for _ in range(3):
            g.replay()
        return g

    kgraph = phase_graph(2)
    ms_kernel = timed(kgraph.replay, args.steps)
    pgraph = phase_graph(1)
    ms_prep = timed(pgraph.replay, args.steps)
    del runs, kgraph, pgraph
    breakdown = {"step_ms": ms_step, "grouped_kernel_only_ms": ms_kernel, "activation_preparation_only_ms": ms_prep}
    if world > 1:
        f_noar, *_ = capture_step(m, skip_all_reduce=True)
        for _ in range(3):
            f_noar()
        ms_noar = timed(f_noar, args.steps)
        breakdown.update({"step_without_all_reduce_ms": ms_noar, "exchange_ms": max(0.0, ms_step - ms_noar),
                          "all_reduce_share": max(0.0, ms_step - ms_noar) / ms_step})

    # ---- the other batch sizes of the config: BASELINE configs[3] (one GPU) / configs[4] (tensor parallel) ----
    sweep = {}
    if not args.no_m_sweep:
        for mm in ([1, 4, 64] if world == 1 else [1, 64, 4096]):
            if mm == m:
                continue
            f, _o, cap, _x, _gr = capture_step(mm)
            for _ in range(2):
                f()
            ms_mm = timed(f, max(3, args.steps // 2) if mm <= 64 else 3)
            cell = {"ms_per_step": ms_mm, "gbs": st.raw_bytes_full / (ms_mm * 1e-3) / 1e9, "tokens_per_s": mm / (ms_mm * 1e-3), "cuda_graph": bool(cap)}
            if world > 1:
                f2, *_ = capture_step(mm, skip_all_reduce=True)
                for _ in range(2):
                    f2()
                ms2 = timed(f2, max(3, args.steps // 2) if mm <= 64 else 3)
                cell.update({"step_without_all_reduce_ms": ms2, "all_reduce_share": max(0.0, ms_mm - ms2) / ms_mm,
                             "all_reduce": "fused into the grouped kernel" if (fused and mm <= 64) else "push kernel" if (mm <= 64 and not args.nccl_allreduce) else "nccl"})
            sweep[f"M={mm}"] = cell
            del f, _o, _x, _gr
            torch.cuda.empty_cache()

    # ---- the large-batch leg of the metric: prefill TFLOP/s, BASELINE configs[2] (grouped gate_up and down, Q4_K and
    # Q6_K, M = 512 / 2048 / 8192), through the op ----
    prefill = None
    if world == 1 and not args.no_prefill:
        from hyperqwen_rtx4080s32_b200 import formats as F
        from hyperqwen_rtx4080s32_b200 import synth

        cells = {}
        for tname in ("Q4_K", "Q6_K"):
            wt = F.TYPE_IDS[tname]
            for sname, pn, pk in (("gate_up", [17408, 17408], 5120), ("down", [5120], 17408)):
                ptiles = [ops.repack_tiles(synth.random_blocks(n, pk, wt, seed=900 + i, device=dev), n, wt) for i, n in enumerate(pn)]
                ppacked, pviews, pdescs, psplits, pnb, pbb = ops.prepare_grouped_layer(ptiles, pn, [wt] * len(pn))
                del ptiles
                for pm in (512, 2048, 8192):
                    px = synth.activations(pm, pk, device=dev)
                    pfn = lambda: ops.fused_mul_mat_gguf_tiles_grouped(px, ppacked, pdescs, psplits, pviews, pn, [wt] * len(pn), pnb, pbb)  # noqa: E731
                    for _ in range(3):
                        pfn()
                    ms_pf = timed(pfn, 5)
                    cells[f"{tname} {sname} M={pm}"] = {"ms": ms_pf, "tflops": 2.0 * pm * pk * sum(pn) / (ms_pf * 1e-3) / 1e12}
                    del px
                del ppacked, pviews, pdescs
                torch.cuda.empty_cache()
        head = cells["Q4_K gate_up M=2048"]
        prefill = {"workload": "grouped gate_up (K 5120, N 2 x 17408) and down (K 17408, N 5120), Q4_K and Q6_K, M = 512 / 2048 / 8192 (BASELINE configs[2]); "
                               "dequantisation not counted in the flops; headline cell: Q4_K gate_up M = 2048",
                   "tflops": head["tflops"], "ms": head["ms"], "kernel": "gemm_prefill_kernel (tcgen05, TMEM accumulator)", "cells": cells}

    # ---- the reference's own per-launch table (gguf-plugin/README.md:134-145: its shapes and types at 8 rows, CUDA-graph
    # replays over copies of the layer exceeding the L2, GB/s of the raw block bytes), with its published RTX 4080 SUPER
    # figures beside ours ----
    type_table = None
    if world == 1 and not args.no_type_table:
        from hyperqwen_rtx4080s32_b200 import formats as F
        from hyperqwen_rtx4080s32_b200 import synth

        import numpy as _np

        globals().update(np=_np, torch=torch)
        type_table = {"what": "grouped kernel alone at M = 8, microseconds and GB/s of raw block bytes; ref = the reference's published figures on its "
                              "RTX 4080 SUPER (736 GB/s) for the same shape and type", "cells": {}}
        for (tn_out, tk), ref_row in REFERENCE_TABLE_M8.items():
            for tname, (ref_us, ref_gbs) in ref_row.items():
                wt = F.TYPE_IDS[tname]
                nbytes = F.raw_bytes(wt, tn_out, tk)
                ncopy = max(2, int(400e6 // nbytes))
                packs = [ops.repack_tiles(synth.random_blocks(tn_out, tk, wt, seed=c, device=dev), tn_out, wt).reshape(-1) for c in range(ncopy)]
                tx = synth.activations(m, tk, device=dev)
                ts = ops.grouped_split_for(-(-tn_out // 64), tk // 256, m=m, block_bytes=F.BYTES_PER_256[wt])
                td = torch.from_numpy(ops.build_descs([wt], [tn_out], tk, ts)).to(dev)
                tws = torch.empty(_lib.lib().gq_workspace_bytes(m, tk, tn_out, ts), dtype=torch.uint8, device=dev)
                ty = torch.empty((m, tn_out), dtype=torch.bfloat16, device=dev)
                ops.grouped_gemm(tx, packs[0], td, ts, [wt], tn_out, out=ty, workspace=tws, phases=1)

                def tfn():
                    for pk_ in packs:
                        ops.grouped_gemm(tx, pk_, td, ts, [wt], tn_out, out=ty, workspace=tws, phases=2)

                us = 1e3 * _graph_time(tfn, ncopy)
                type_table["cells"][f"{tname} {tn_out}x{tk}"] = {"us": round(us, 2), "gbs": round(nbytes / us / 1e3, 1), "split": ts,
                                                                 "ref_us": ref_us, "ref_gbs": ref_gbs}
                del packs, tx, td, tws, ty
                torch.cuda.empty_cache()

    status = ops.device_status(dev)
    if world > 1:
        sflag = torch.tensor([status], device=dev)
        dist.all_reduce(sflag, op=dist.ReduceOp.MAX)
        status = int(sflag.item())
    if status != 0:
        raise SystemExit(f"[rank {rank}] a kernel reported device status {status} during the benchmark: the numbers are void")

    if rank == 0:
        peaks, which = measured_peaks()
        if prefill is not None:
            prefill["peak_tflops"] = peaks["bf16_tflops"]
            prefill["frac"] = prefill["tflops"] / peaks["bf16_tflops"]
            prefill["frac_of_sustained"] = prefill["tflops"] / peaks.get("bf16_tflops_sustained", peaks["bf16_tflops"])
            for c in prefill["cells"].values():
                c["frac"] = c["tflops"] / peaks["bf16_tflops"]
        total_bytes = st.raw_bytes_full
        value = total_bytes / (ms_step * 1e-3) / 1e9
        e2e = total_bytes / (ms_e2e * 1e-3) / 1e9
        achieved = st.raw_bytes_local / (ms_kernel * 1e-3) / 1e9
        n_launch = 4 * args.layers
        line = {"metric": METRIC, "value": value, "unit": "GB/s", "n_gpus": world, "steps": args.steps, "warmup": max(3, args.warmup),
                "ms_per_step": ms_step, "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
                "dtype": "u8/s8 weights x 16-bit fixed-point activations -> s32, f32 across 256-blocks (M <= 16); f16 x f16 -> f32 above",
                "data": "synthetic",
                "config": {"workload": f"mixed-type {args.layers}-layer GGUF decoder linear stack (BASELINE configs[3]{'/[4] tensor-parallel' if world > 1 else ''}), decode M={m}",
                           "bits_per_weight": round(8 * total_bytes / st.weights_full, 3), "raw_block_bytes": total_bytes,
                           "l2": "weights (10 GB) far exceed L2; no flush needed", "parallelism": f"tp{world}", "all_reduce": ("none" if world == 1 else "nccl" if args.nccl_allreduce else "fused into the grouped kernel's epilogue, pushed over NVLink peer memory (gq_gemv_grouped_allreduce)" if fused else "push kernel over NVLink peer memory (gq_allreduce_push)"),
                           "cuda_graph": bool(captured), "l2_prefetch_next_layer": bool(st.prefetch),
                           "weights": "random valid blocks (the reference's test method), seeded"},
                "tokens_per_s": m / (ms_step * 1e-3),
                "e2e": {"value": e2e, "unit": "GB/s", "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h, "ms_per_step": ms_e2e,
                        "tokens_per_s": m / (ms_e2e * 1e-3)},
                "gpu_launches": int(launches_per_step * args.steps),
                "roofline": {"bound": "hbm", "kernel": "gemv_grouped_kernel", "achieved": achieved, "peak": peaks["hbm_gbs"], "unit": "GB/s",
                             "frac": achieved / peaks["hbm_gbs"], "peak_source": which, "frac_of_nominal_8TBs": achieved / 8000.0,
                             "launches_per_step": n_launch, "avg_launch_us": 1e3 * ms_kernel / n_launch,
                             # DRAM bytes per launch: ncu captures of single launches of this kernel (profiles/) read
                             # 1.00-1.01 x the raw block bytes (plus the activation tile from L2); scaled to this
                             # workload's average launch
                             "traffic": 1.007 * st.raw_bytes_local / n_launch, "algorithmic_bytes_per_launch": st.raw_bytes_local / n_launch},
                "breakdown": breakdown,
                "parity_before_timing": {"max_rel_err_vs_fp64_oracle": parity, "tolerance": 1e-2},
                "device_status_after_run": status,
                "clocks": clk.summary()}
        if sweep:
            line["other_batch_sizes"] = sweep
        if prefill is not None:
            line["prefill"] = prefill
        if type_table is not None:
            line["per_type_m8"] = type_table
        if world == 1 and not args.no_cpu:
            v, dt, info = cpu_sample(m, 2, target_s=12.0)
            line["cpu_baseline"] = dict(info, value=v, unit="GB/s")
            try:
                line["cpu_baseline_gguf_py"] = gguf_py_sample(m)
            except Exception as e:   # noqa: BLE001 - the gguf package is test infrastructure; its absence only drops this leg
                line["cpu_baseline_gguf_py"] = {"unavailable": str(e)}
        _emit(json.dumps(line))
    if world > 1:
        # leave without tearing NCCL down: destroying a process group whose collectives live inside captured
        # CUDA graphs can block forever, and nothing is left to do
        dist.barrier()
        torch.cuda.synchronize()
        sys.stdout.flush()
        sys.stderr.flush()
        os._exit(0)



# ---- per-type sweeps (the per-type decode sweep of BASELINE configs[1] and the prefill sweep of configs[2]) ----------
#   python bench.py --sweep decode --types Q4_K Q6_K --shapes gate kv --m 1 8 [--split 1 2] [--eager --iters 3]
#   python bench.py --sweep prefill --types Q4_K --shapes gate_up down --m 512 2048 8192
#   python bench.py --sweep neighbours --sweep-m 1 8      (silu_and_mul / add + RMSNorm folded into the layer behind them)
#   python bench.py --sweep served --sweep-m 1 8          (the linear layers of the served checkpoint's own tensor list)
# Decode: for each type x shape x batch the grouped kernel alone (activations prepared beforehand) and the whole call
# (prepare + kernel + partial sum) as CUDA-graph replays over distinct weight copies totalling more than the L2, median of
# 7 — the reference's timing method (gguf-plugin/test_gluon_kq_gpu.py:198-245) —, microseconds and GB/s of raw GGUF block
# bytes.  --eager launches the kernel a few times without a graph (the form a profiler capture wants).
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


def sweep_prefill(a, dev) -> None:
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
                    ops.prefill_gemm(x, packed, d1, n_total, out=y, wtypes=[t] * len(n_outs))
                torch.cuda.synchronize()
                if a.eager:
                    _say(f"{tn:7} {sn:8} M={m}: eager", flush=True)
                    continue
                ts = []
                for _ in range(5):
                    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                    e0.record()
                    ops.prefill_gemm(x, packed, d1, n_total, out=y, wtypes=[t] * len(n_outs))
                    e1.record()
                    torch.cuda.synchronize()
                    ts.append(e0.elapsed_time(e1))
                ms = float(np.median(ts))
                _say(f"{tn:7} {sn:8} K={k} N={n_total} M={m:5}: {ms:8.3f} ms  {2.0 * m * k * n_total / ms / 1e9:7.1f} TFLOP/s", flush=True)
            del packed, views, descs
            torch.cuda.empty_cache()




def sweep_neighbours(a, dev) -> None:
    """The ops either side of a linear at decode batch sizes: down_proj with silu_and_mul in front and gate_up_proj with
    add + RMSNorm in front, as separate torch operations and folded into the layer's activation preparation; microseconds
    per layer, CUDA-graph replay over 24 layers of distinct Q4_K weights (more than the L2)."""
    from hyperqwen_rtx4080s32_b200 import linear

    k, n, layers = 17408, 5120, 24
    downs, gate_ups = [], []
    for i in range(layers):
        lin = linear.GGUFLinear(k, [n])
        lin.load_shard(synth.random_blocks(n, k, F.Q4_K, seed=i, device=dev), F.Q4_K)
        downs.append(lin.finalize())
        lin = linear.GGUFLinear(n, [k, k])
        for j in range(2):
            lin.load_shard(synth.random_blocks(k, n, F.Q4_K, seed=100 + 2 * i + j, device=dev), F.Q4_K, j)
        gate_ups.append(lin.finalize())
    w = torch.ones(n, dtype=torch.bfloat16, device=dev)
    for m in a.m:
        gu = synth.activations(m, 2 * k, device=dev)
        x, res = synth.activations(m, n, device=dev), synth.activations(m, n, seed=5, device=dev)
        pre = ops.PreAddRMSNorm(w, 1e-6, residual=res)
        cases = (("down alone", lambda: [l(gu[:, :k]) for l in downs]),
                 ("silu_and_mul (torch) + down", lambda: [l(torch.nn.functional.silu(gu[:, :k]) * gu[:, k:]) for l in downs]),
                 ("down, silu_and_mul folded", lambda: [l(gu, pre=ops.PreSiluMul()) for l in downs]),
                 ("gate_up alone", lambda: [l(x) for l in gate_ups]),
                 ("add + RMSNorm (torch) + gate_up", lambda: [l(pre.unfused(x)) for l in gate_ups]),
                 ("gate_up, add + RMSNorm folded", lambda: [l(x, pre=pre) for l in gate_ups]))
        for name, fn in cases:
            _say(f"M={m:2} {name:32}: {1e3 * _graph_time(fn, layers):7.2f} us per layer", flush=True)


def sweep_served(a, dev) -> None:
    """The linear layers of the checkpoint the reference serves (names, shapes and GGML types from the tensor list
    tests/golden/qwen35_tensor_names.json; values synthetic): every quantized 2-D weight of the 64 blocks through the
    loader's name map — q / k / v and gate / up fused as vLLM fuses them — plus the LM head, one pass over all of them per
    step as a CUDA graph; milliseconds and GB/s of raw GGUF block bytes.  The type mix is the file's own (IQ3_S, IQ4_XS,
    IQ3_XXS, Q4_K, IQ2_S, ...), not the benchmark's eleven-type draw."""
    import collections
    import json

    from hyperqwen_rtx4080s32_b200 import linear, loader

    fx = json.load(open(os.path.join(os.path.dirname(os.path.abspath(__file__)), "tests", "golden", "qwen35_tensor_names.json")))
    order = {"q": 0, "k": 1, "v": 2, 0: 0, 1: 1, None: 0}
    layers, skipped, by_type, seed = [], [], collections.Counter(), 0
    groups = [(f"blk.{b}.", t) for b, t in sorted(fx["blocks"].items(), key=lambda kv: int(kv[0]))] + [("", fx["top"])]
    for prefix, tensors in groups:
        pending = collections.OrderedDict()
        for name, tname, shape in tensors:
            mapped = loader.map_tensor_name(prefix + name)
            if len(shape) != 2 or mapped is None or tname in ("F32", "F16", "BF16") or name == "token_embd.weight":
                continue
            if mapped.module is None and name != "output.weight":
                continue
            if tname not in F.TYPE_IDS:
                skipped.append(f"{prefix}{name} ({tname})")
                continue
            k, n = shape
            pending.setdefault(mapped.merged or mapped.module or "lm_head", []).append((order[mapped.shard_id], mapped.shard_id, F.TYPE_IDS[tname], n, k))
        for key, shards in pending.items():
            shards.sort(key=lambda sh: sh[0])
            k = shards[0][4]
            lin = linear.GGUFLinear(k, [sh[3] for sh in shards])
            for _, sid, t, n, _ in shards:
                seed += 1
                lin.load_shard(synth.random_blocks(n, k, t, seed=seed, device=dev), t, sid if len(shards) > 1 else None)
                by_type[F.TYPE_NAMES[t]] += F.raw_bytes(t, n, k)
            layers.append((lin.finalize(), k))
        torch.cuda.empty_cache()
    total = sum(by_type.values())
    _say(f"{len(layers)} linear layers, {total / 1e9:.2f} GB of raw blocks: " + ", ".join(f"{t} {100.0 * b / total:.1f} %" for t, b in by_type.most_common())
         + (f"; not built: {', '.join(skipped)}" if skipped else ""))
    for m in a.m:
        xs = {k: synth.activations(m, k, device=dev) for k in {k for _, k in layers}}

        def step():
            for lin, k in layers:
                lin(xs[k])

        ms = _graph_time(step, 1)
        _say(f"M={m:2}: {ms:7.3f} ms per pass over the {len(layers)} layers = {total / ms / 1e6:6.0f} GB/s ({total / ms / 1e6 / 6555.5:.2f} of the measured copy bandwidth)", flush=True)


def run_sweep(a) -> None:
    import numpy as np  # noqa: F401
    import torch

    from hyperqwen_rtx4080s32_b200 import _lib, formats as F, ops, synth

    globals().update(np=np, torch=torch, _lib=_lib, F=F, ops=ops, synth=synth)
    a.types = a.types or list(F.TYPE_IDS)
    a.m = a.sweep_m or ([512, 2048, 8192] if a.sweep == "prefill" else [1, 8])
    a.shapes = a.shapes or (["q", "kv", "gate", "down"] if a.sweep == "decode" else ["gate_up", "down"])
    dev = torch.device("cuda", 0)
    L = _lib.lib()
    if a.sweep == "prefill":
        return sweep_prefill(a, dev)
    if a.sweep == "neighbours":
        return sweep_neighbours(a, dev)
    if a.sweep == "served":
        return sweep_served(a, dev)
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
                _say(f"{tn:7} {sn:5} {n_out}x{k} M={m:2} auto-split={auto} copies={ncopy} | " + " | ".join(cells), flush=True)
            del packs
            torch.cuda.empty_cache()




def _say(*parts, flush=True):
    _emit(" ".join(str(p) for p in parts))


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--m", type=int, default=8)
    ap.add_argument("--layers", type=int, default=64)
    ap.add_argument("--no-cpu", action="store_true", help="skip the CPU baseline leg")
    ap.add_argument("--no-prefill", action="store_true", help="skip the prefill TFLOP/s leg")
    ap.add_argument("--no-type-table", action="store_true", help="skip the reference's per-type table at its own shapes (M = 8)")
    ap.add_argument("--no-m-sweep", action="store_true", help="skip the other batch sizes of the config (M = 1, 4, 64; tensor parallel: 1, 64, 4096)")
    ap.add_argument("--unfused-allreduce", action="store_true", help="tensor parallel: all-reduce with the library's separate push kernel instead of inside the grouped kernel")
    ap.add_argument("--nccl-allreduce", action="store_true", help="tensor parallel: use NCCL for the row-parallel all-reduce instead of the library's push kernel")
    ap.add_argument("--sweep", choices=["decode", "prefill", "neighbours", "served"], help="per-type sweep instead of the benchmark line (prints a table)")
    ap.add_argument("--types", nargs="*", default=[], help="--sweep: GGML type names (default all)")
    ap.add_argument("--shapes", nargs="*", default=[], help="--sweep: q kv o gate down (decode; or NxK), gate_up down q (prefill)")
    ap.add_argument("--sweep-m", nargs="*", type=int, default=[], help="--sweep: batch sizes")
    ap.add_argument("--split", nargs="*", type=int, default=[], help="--sweep decode: split-K factors (default: the library's choice)")
    ap.add_argument("--copies-mb", type=float, default=600.0, help="--sweep decode: megabytes of distinct weight copies per graph (0: one copy, weights stay in L2)")
    ap.add_argument("--eager", action="store_true", help="--sweep: launch without a CUDA graph (for profiler captures)")
    ap.add_argument("--iters", type=int, default=3)
    ap.add_argument("--l2-prefetch", action="store_true", help="warm the L2 with the next layer's weights from the idle producer lanes (measured neutral)")
    ap.add_argument("--no-l2-prefetch", action="store_true", help="accepted for older command lines; the prefetch is off unless --l2-prefetch is given")
    args = ap.parse_args()
    # stdout carries the one JSON line and nothing else: whatever libraries print there (NCCL's version banner, for
    # one) goes to stderr instead, for the whole run and at the file-descriptor level
    sys.stdout.flush()
    json_fd = os.dup(1)
    os.dup2(2, 1)
    global _emit
    _emit = lambda text: os.write(json_fd, (text + "\n").encode())
    if args.sweep:
        run_sweep(args)
    elif args.impl == "reference":
        run_reference(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
