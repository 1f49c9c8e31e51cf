"""GGUF file -> the layers of the quantized-linear path.

What the plugin's loader and tensor-name adapter do for `MODEL=*.gguf` (vllm_gguf_plugin/loader.py and
vllm_gguf_plugin/weights_adapter/qwen3_5.py, un-vendored; the reference checks them in
gguf-plugin/test_gguf_rco_cpu.py:84-128 against the tensor list gguf-plugin/iq3s-tensor-names.json of the checkpoint
it serves), narrowed to this path: read the file's tensor table, give every tensor its Hugging Face module name, and
hand the quantized 2-D weights to GGUFLinearMethod's weight loaders — q / k / v and gate / up as the shards of the
merged layers vLLM builds (shard ids "q", "k", "v" and 0, 1) —, which repack them tile-major on the device.  Norms,
convolution and state-space tensors, the vision tower and the projector are not linear-method weights: they are
reported with their names and left to the engine.

The file is read with the `gguf` package (the reference pins gguf==0.17.1, gguf-plugin/requirements.txt:1); tensor data
stay memory-mapped until they are copied to the device, one tensor at a time.
"""
from __future__ import annotations

import re
from dataclasses import dataclass, field
from typing import Iterator

import numpy as np
import torch

from . import formats as F
from .linear import GGUFLinear

# GGUF tensor suffix inside "blk.N." -> (HF module, merged vLLM layer or None, shard id in it)
_BLOCK_LINEAR = {
    "attn_q": ("self_attn.q_proj", "self_attn.qkv_proj", "q"),
    "attn_k": ("self_attn.k_proj", "self_attn.qkv_proj", "k"),
    "attn_v": ("self_attn.v_proj", "self_attn.qkv_proj", "v"),
    "attn_output": ("self_attn.o_proj", None, None),
    "attn_qkv": ("linear_attn.in_proj_qkv", None, None),
    "attn_gate": ("linear_attn.in_proj_z", None, None),
    "ssm_out": ("linear_attn.out_proj", None, None),
    "ffn_gate": ("mlp.gate_proj", "mlp.gate_up_proj", 0),
    "ffn_up": ("mlp.up_proj", "mlp.gate_up_proj", 1),
    "ffn_down": ("mlp.down_proj", None, None),
}
# tensors of a block that are not weights of a linear method
_BLOCK_OTHER = {
    "attn_norm.weight": "input_layernorm.weight", "post_attention_norm.weight": "post_attention_layernorm.weight",
    "attn_q_norm.weight": "self_attn.q_norm.weight", "attn_k_norm.weight": "self_attn.k_norm.weight",
    "ssm_alpha.weight": "linear_attn.in_proj_a.weight", "ssm_beta.weight": "linear_attn.in_proj_b.weight",
    "ssm_conv1d.weight": "linear_attn.conv1d.weight", "ssm_norm.weight": "linear_attn.norm.weight",
    "ssm_dt.bias": "linear_attn.dt_bias", "ssm_a": "linear_attn.A_log",
}
_TOP = {"token_embd.weight": "model.language_model.embed_tokens.weight", "output_norm.weight": "model.language_model.norm.weight",
        "output.weight": "lm_head.weight"}
_GGML_NAMES = {2: "Q4_0", 6: "Q5_0", 8: "Q8_0", 10: "Q2_K", 11: "Q3_K", 12: "Q4_K", 13: "Q5_K", 14: "Q6_K", 16: "IQ2_XXS", 17: "IQ2_XS",
               18: "IQ3_XXS", 19: "IQ1_S", 20: "IQ4_NL", 21: "IQ3_S", 22: "IQ2_S", 23: "IQ4_XS", 29: "IQ1_M", 0: "F32", 1: "F16", 30: "BF16"}


@dataclass(frozen=True)
class MappedName:
    hf_name: str                 # e.g. model.language_model.layers.3.self_attn.q_proj.weight
    layer: int | None            # decoder block, None for top-level tensors
    module: str | None           # HF module inside the block (no ".weight"), None if not a linear weight of a block
    merged: str | None           # the merged vLLM layer this weight is a shard of (qkv_proj, gate_up_proj), if any
    shard_id: object = None      # "q" / "k" / "v" or 0 / 1 inside the merged layer


def map_tensor_name(name: str) -> MappedName | None:
    """GGUF tensor name of the text model -> its Hugging Face name and where it goes; None for names this adapter does not
    know (the vision tower `v.*` and the projector `mm.*` belong to another adapter)."""
    if name in _TOP:
        return MappedName(_TOP[name], None, None, None)
    m = re.fullmatch(r"blk\.(\d+)\.(.+)", name)
    if not m:
        return None
    layer, rest = int(m.group(1)), m.group(2)
    prefix = f"model.language_model.layers.{layer}."
    if rest in _BLOCK_OTHER:
        return MappedName(prefix + _BLOCK_OTHER[rest], layer, None, None)
    if rest.endswith(".weight") and rest[:-7] in _BLOCK_LINEAR:
        module, merged, sid = _BLOCK_LINEAR[rest[:-7]]
        return MappedName(prefix + module + ".weight", layer, module, merged, sid)
    return None


@dataclass
class GGUFTensor:
    name: str
    ggml_type: int
    shape: tuple[int, ...]       # logical shape, outermost first: (n_out, K) for a 2-D weight
    data: np.ndarray             # quantized: uint8 [n_out, row_bytes]; otherwise the values

    @property
    def type_name(self) -> str:
        return _GGML_NAMES.get(self.ggml_type, str(self.ggml_type))


def read_gguf(path: str) -> Iterator[GGUFTensor]:
    """The file's tensors in file order (data memory-mapped by the gguf package)."""
    from gguf import GGUFReader

    for t in GGUFReader(path).tensors:
        shape = tuple(int(d) for d in reversed(t.shape))          # GGUF lists the innermost dimension first
        yield GGUFTensor(str(t.name), int(t.tensor_type), shape, t.data)


@dataclass
class LoadedModel:
    linears: dict[str, GGUFLinear] = field(default_factory=dict)   # "layers.3.self_attn.qkv_proj" / "lm_head" -> layer, finalized
    embedding: GGUFTensor | None = None                            # token_embd.weight, left raw (its rows are gathered)
    other: dict[str, GGUFTensor] = field(default_factory=dict)     # HF name -> norms etc., for the engine
    unmapped: list[str] = field(default_factory=list)              # names this adapter does not know
    unsupported: dict[str, str] = field(default_factory=dict)      # linear weights in a GGML type the kernels do not decode


def load_gguf(path: str, device="cuda", strict: bool = True) -> LoadedModel:
    """Read a GGUF file and build the path's layers: one GGUFLinear per linear module of the text model, with q / k / v
    and gate / up fused as vLLM fuses them; every weight goes through GGUFLinearMethod's weight loaders and is repacked
    tile-major on `device`.  With strict, a linear weight in a type the kernels do not decode raises; otherwise it is listed
    in `unsupported` and its module is left out."""
    out = LoadedModel()
    pending: dict[str, list[tuple[object, GGUFTensor]]] = {}
    order = {"q": 0, "k": 1, "v": 2, 0: 0, 1: 1, None: 0}
    for t in read_gguf(path):
        mapped = map_tensor_name(t.name)
        if mapped is None:
            out.unmapped.append(t.name)
            continue
        if t.name == "token_embd.weight":
            out.embedding = t
            continue
        is_linear = mapped.module is not None or t.name == "output.weight"
        if not is_linear or len(t.shape) != 2 or t.ggml_type in (0, 1, 30):
            out.other[mapped.hf_name] = t
            continue
        if t.ggml_type not in F.SUPPORTED_TYPES:
            if strict:
                raise ValueError(f"{t.name}: GGML type {t.type_name} is not a type the kernels decode")
            out.unsupported[t.name] = t.type_name
            continue
        key = "lm_head" if mapped.layer is None else f"layers.{mapped.layer}.{mapped.merged or mapped.module}"
        pending.setdefault(key, []).append((mapped.shard_id, t))
    for key, shards in pending.items():
        shards.sort(key=lambda s: order[s[0]])
        k = shards[0][1].shape[1]
        if any(t.shape[1] != k for _, t in shards):
            raise ValueError(f"{key}: shards disagree on K")
        lin = GGUFLinear(k, [t.shape[0] for _, t in shards])
        for sid, t in shards:
            want = F.raw_row_bytes(t.ggml_type, k)
            raw = torch.from_numpy(np.array(t.data, copy=True)).reshape(t.shape[0], -1)
            if raw.shape[1] != want:
                raise ValueError(f"{t.name}: {raw.shape[1]} bytes per row, {want} expected for {t.type_name} at K={k}")
            lin.load_shard(raw.to(device), t.ggml_type, sid)
        out.linears[key] = lin.finalize()
    return out


def embedding_lookup(raw: torch.Tensor, wtype: int, ids: torch.Tensor, dtype=torch.bfloat16) -> torch.Tensor:
    """Rows `ids` of a quantized embedding table raw uint8 [vocab, row_bytes] (kept raw, as the plugin keeps it:
    gguf-tiles-all-types.patch:80-89) dequantised to [len(ids), K]: the rows are gathered as bytes, repacked and
    dequantised by the same kernels that serve the weights — bit-identical to gguf.quants.dequantize of those rows."""
    from . import ops

    if int(wtype) not in F.SUPPORTED_TYPES:
        raise ValueError(f"GGML type {wtype} is not a type the kernels decode")
    k = raw.shape[1] // F.BYTES_PER_256[int(wtype)] * F.QK
    flat = ids.reshape(-1).to(raw.device)
    rows = raw.index_select(0, flat)
    n = int(rows.shape[0])
    if n == 0:
        return torch.empty((*ids.shape, k), dtype=dtype, device=raw.device)
    w = ops.dequantize_tiles(ops.repack_tiles(rows, n, int(wtype)), n, k, int(wtype), dtype=dtype)
    return w.reshape(*ids.shape, k)
