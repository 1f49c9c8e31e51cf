"""The mixed-type decoder linear stack used by the benchmark and the multi-GPU tests: 64 blocks of
(fused QKV, o, fused gate_up, down) linears at hidden 5120, 40 query / 8 KV heads of 128, intermediate
17408, every tensor's GGML type drawn from a seeded distribution over the eleven types (about 3.88 bits
per weight, 10.25 GB).  Weights are random valid blocks (synth.random_blocks) generated on the device.

Only the linears are modelled: attention, normalisation and the activation function between gate_up and
down belong to the engine around this path.  Each linear reads a fixed synthetic input of its shape, so a
"step" is one pass of the quantized-linear path over one batch: 256 LinearMethod.apply calls.
"""
from __future__ import annotations

import numpy as np
import torch

from . import formats as F
from . import synth
from .linear import GGUFLinear

REST = [(F.IQ3_S, .30), (F.Q3_K, .25), (F.Q2_K, .30), (F.IQ4_XS, .06), (F.Q4_K, .05), (F.IQ4_NL, .01), (F.Q4_0, .01), (F.Q5_0, .01), (F.Q8_0, .01)]
SENSITIVE = [(F.Q6_K, .10), (F.Q5_K, .15), (F.Q4_K, .35), (F.IQ4_XS, .40)]
TENSORS = ["q", "k", "v", "o", "gate", "up", "down"]


def draw_types(n_layers: int = 64, seed: int = 20261125) -> list[dict[str, int]]:
    rng = np.random.default_rng(seed)
    out = []
    for _ in range(n_layers):
        d = {}
        for name in TENSORS:
            dist = SENSITIVE if name in ("o", "down") else REST
            d[name] = int(rng.choice([a for a, _ in dist], p=[b for _, b in dist]))
        out.append(d)
    return out


class LinearStack:
    def __init__(self, n_layers: int = 64, hidden: int = 5120, heads: int = 40, kv_heads: int = 8, head_dim: int = 128,
                 inter: int = 17408, seed: int = 20261125, device="cuda", tp_rank: int = 0, tp_size: int = 1, types=None):
        from . import tp as _tp

        self.hidden, self.inter, self.device = hidden, inter, device
        self.tp_rank, self.tp_size = tp_rank, tp_size
        self.types = types if types is not None else draw_types(n_layers, seed)
        shapes = {"q": (heads * head_dim, hidden), "k": (kv_heads * head_dim, hidden), "v": (kv_heads * head_dim, hidden),
                  "o": (hidden, heads * head_dim), "gate": (inter, hidden), "up": (inter, hidden), "down": (hidden, inter)}
        self.full_shapes = shapes
        self.raw_bytes_full = sum(F.raw_bytes(t[n], *shapes[n]) for t in self.types for n in TENSORS)
        self.weights_full = sum(shapes[n][0] * shapes[n][1] for _ in self.types for n in TENSORS)
        self.layers = []
        self.raw_bytes_local = 0
        for li, t in enumerate(self.types):
            blk = {}
            for lname, shards, parallel in (("qkv", ["q", "k", "v"], "column"), ("o", ["o"], "row"),
                                            ("gate_up", ["gate", "up"], "column"), ("down", ["down"], "row")):
                raws, wts, k_pad = [], [], None
                for j, sname in enumerate(shards):
                    n_out, k = shapes[sname]
                    raw = synth.random_blocks(n_out, k, t[sname], seed=seed % 100000 + 1000 * li + 10 * TENSORS.index(sname), device=device)
                    if tp_size > 1:
                        raw, k_pad = _tp.shard_raw(raw, t[sname], parallel, tp_rank, tp_size)
                    raws.append(raw)
                    wts.append(t[sname])
                k_local = raws[0].shape[1] // F.BYTES_PER_256[wts[0]] * 256
                lin = GGUFLinear(k_local, [r.shape[0] for r in raws])
                ids = ["q", "k", "v"] if lname == "qkv" else [0, 1] if lname == "gate_up" else [None]
                for raw, wt, sid in zip(raws, wts, ids):
                    lin.load_shard(raw, wt, sid)
                    self.raw_bytes_local += raw.numel()
                lin.finalize()
                lin.k_pad = k_pad
                blk[lname] = lin
                del raws
            self.layers.append(blk)
        if device != "cpu":
            torch.cuda.empty_cache()
        self.prefetch = False

    def enable_prefetch(self, on: bool = True) -> None:
        """Register the call order of the stack's packed runs so each launch warms the L2 for the next one."""
        from . import ops

        ops.clear_prefetch_chain()
        if on:
            order = [blk[name].gguf_groups[next(iter(blk[name].gguf_groups))][0] for blk in self.layers for name in ("qkv", "o", "gate_up", "down")]
            ops.register_prefetch_chain(order)
        self.prefetch = on

    def input_sizes(self) -> dict[str, int]:
        blk = self.layers[0]
        return {name: blk[name].input_size for name in ("qkv", "o", "gate_up", "down")}

    def step(self, x: dict[str, torch.Tensor]) -> torch.Tensor:
        """One pass: every linear of every block applied to the input of its name; returns the last
        block's `down` output (under tensor parallelism: summed over the ranks)."""
        from . import tp as _tp

        from . import ops

        out = None
        far = getattr(self, "fused_ar", None)
        exchange = not getattr(self, "skip_all_reduce", False)     # False only to time a step without its all-reduces
        for blk in self.layers:
            for name in ("qkv", "o", "gate_up", "down"):
                if self.tp_size > 1 and name in ("o", "down") and exchange:
                    if far is not None:
                        # the all-reduce happens in the grouped kernel's epilogue; a call it cannot serve falls back
                        far.used = False
                        with ops.fused_allreduce(far):
                            out = blk[name](x[name])
                        if not far.used:
                            _tp.all_reduce_(out)
                    else:
                        out = blk[name](x[name])
                        _tp.all_reduce_(out)
                else:
                    out = blk[name](x[name])
        return out

    def enable_fused_all_reduce(self, max_m: int = 64) -> None:
        """Row-parallel layers sum over the ranks inside the grouped kernel (call on every rank, outside capture)."""
        from . import tp as _tp

        self.fused_ar = _tp.FusedAllReduce(max_m=max_m, max_n_total=self.hidden) if self.tp_size > 1 else None

    def make_inputs(self, m: int, seed: int = 0, device=None) -> dict[str, torch.Tensor]:
        """Seeded bf16 N(0, 1) inputs of every linear's (local, padded) K; row-parallel inputs are zero
        outside the rank's own K range."""
        from . import tp as _tp

        dev = device or self.device
        full = {"qkv": self.hidden, "o": self.full_shapes["o"][1], "gate_up": self.hidden, "down": self.inter}
        x = {}
        for name, k in full.items():
            t = synth.activations(m, k, seed=seed + 100 + m + (7 if name in ("o", "down") else 0), device=dev)
            pad = self.layers[0][name].k_pad
            if pad is not None:
                k0 = self.tp_rank * pad.own
                t = _tp.pad_input(t[:, k0:k0 + pad.own].contiguous(), pad)
            x[name] = t
        return x
