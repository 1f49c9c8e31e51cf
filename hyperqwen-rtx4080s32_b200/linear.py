"""Host-side mirror of the plugin's GGUF quantization-method surface for linear layers.

Same three methods, argument meaning, layer attributes and shard conventions as the reference's
`GGUFLinearMethod` after its patches (vllm_gguf_plugin/quantization/linear.py, un-vendored; the
reference carries its diffs: gguf-plugin/patches/gguf-shard-tensors.patch:19-51,
gguf-tiles-all-types.patch:73-131, gguf-tiles-grouped.patch:84-168):

    create_weights(layer, input_size_per_partition, output_partition_sizes, input_size, output_size,
                   params_dtype, **extra_weight_attrs)
    process_weights_after_loading(layer)      # padded/sharded param -> tiles -> groups
    apply(layer, x, bias=None)                # one op call per run of shards, bias added

Layer state left behind (read by apply and by callers of the reference): layer.weight (.shard_id,
.shard_id_map, .data_container, .shard_offset_map), layer.weight_type (.weight_type,
.shard_weight_type), layer.gguf_shards, layer.gguf_tiles, layer.gguf_tiles_rows,
layer.gguf_tiles_types, layer.gguf_groups.  Shard ids are "q","k","v" for a fused QKV layer (that
order is forced) and 0, 1 for gate_up.

It does not import vLLM: `layer` is any torch.nn.Module.  Inside vLLM the class is used as the
`LinearMethodBase` returned by the `gguf` QuantizationConfig.
"""
from __future__ import annotations

from typing import Any

import torch
from torch.nn import Parameter

from . import formats as F
from . import ops


def set_weight_attrs(weight: torch.Tensor, attrs: dict[str, Any] | None) -> None:
    if attrs:
        for k, v in attrs.items():
            setattr(weight, k, v)


def _gguf_ordered_shard_ids(shard_id: list) -> list:
    return ["q", "k", "v"] if "q" in shard_id else list(shard_id)


def gguf_weight_loader(param: Parameter, loaded_weight: torch.Tensor, loaded_shard_id=None) -> None:
    """Collects raw GGUF rows (uint8 [n_out, row_bytes]) of one shard, or of the whole tensor when
    loaded_shard_id is None, into the parameter's data_container; materialised by
    process_weights_after_loading."""
    if loaded_weight.dtype != torch.uint8 or loaded_weight.dim() != 2:
        raise ValueError(f"GGUF weights are uint8 [n_out, row_bytes]; got {loaded_weight.dtype} {tuple(loaded_weight.shape)}")
    if loaded_shard_id is None:
        param.data_container.clear()
        param.shard_id.clear()
        param.shard_id_map.clear()
        param.data_container.append(loaded_weight)
        return
    if loaded_shard_id in param.shard_id_map:
        param.data_container[param.shard_id_map[loaded_shard_id]] = loaded_weight
    else:
        param.shard_id_map[loaded_shard_id] = len(param.data_container)
        param.shard_id.append(loaded_shard_id)
        param.data_container.append(loaded_weight)


def gguf_weight_type_loader(param: Parameter, weight_type: int, loaded_shard_id=None) -> None:
    if int(weight_type) not in F.SUPPORTED_TYPES:
        raise ValueError(f"Unsupported GGUF quantization type {weight_type}")
    if loaded_shard_id is None:
        param.weight_type = int(weight_type)
    else:
        param.shard_weight_type[loaded_shard_id] = int(weight_type)
        if not param.weight_type:
            param.weight_type = int(weight_type)


class GGUFConfig:
    """Config for GGUF (name `gguf`, as `--quantization gguf` selects it; fp8/env.sh:56-65)."""

    def __init__(self, unquantized_modules: list[str] | None = None) -> None:
        self.unquantized_modules = unquantized_modules or []

    def __repr__(self) -> str:
        return "GGUFConfig()"

    @staticmethod
    def get_name() -> str:
        return "gguf"

    @staticmethod
    def get_supported_act_dtypes() -> list[torch.dtype]:
        return [torch.bfloat16]

    @staticmethod
    def get_min_capability() -> int:
        return 100

    def get_quant_method(self, layer: torch.nn.Module, prefix: str = ""):
        return GGUFLinearMethod(self)


class GGUFLinearMethod:
    """Linear method for GGUF on B200."""

    def __init__(self, quant_config: GGUFConfig | None = None):
        self.quant_config = quant_config or GGUFConfig()

    # ---- a1 ----
    def create_weights(self, layer: torch.nn.Module, input_size_per_partition: int, output_partition_sizes: list[int],
                       input_size: int, output_size: int, params_dtype: torch.dtype, **extra_weight_attrs) -> None:
        self.params_dtype = params_dtype
        tensor_shape = (sum(output_partition_sizes), input_size_per_partition)
        weight = Parameter(torch.empty(0, dtype=torch.uint8), requires_grad=False)
        set_weight_attrs(weight, {"input_dim": 1, "output_dim": 0, "tensor_shape": tensor_shape, "is_gguf_weight": True,
                                  "data_container": [], "shard_id": [], "shard_id_map": {}, "weight_loader": gguf_weight_loader})
        set_weight_attrs(weight, extra_weight_attrs)
        layer.register_parameter("weight", weight)
        weight_type = Parameter(torch.empty(len(output_partition_sizes), dtype=torch.uint8), requires_grad=False)
        set_weight_attrs(weight_type, {"is_gguf_weight_type": True, "weight_type": 0, "shard_weight_type": {},
                                       "ignore_warning": True, "weight_loader": gguf_weight_type_loader})
        set_weight_attrs(weight_type, {k: v for k, v in extra_weight_attrs.items() if k != "weight_loader"})
        layer.register_parameter("weight_type", weight_type)
        layer.gguf_input_size_per_partition = input_size_per_partition
        layer.gguf_output_partition_sizes = list(output_partition_sizes)

    # ---- a2, a3, a5 ----
    def process_weights_after_loading(self, layer: torch.nn.Module) -> None:
        fallback = layer.weight_type.weight_type
        types = set(layer.weight_type.shard_weight_type.values()) | ({fallback} if fallback else set())
        for t in types:
            if t not in F.SUPPORTED_TYPES:
                raise ValueError(f"Unsupported GGUF quantization type {t} in layer {layer}.")
        self._create_padded_weight_param(layer)
        self._create_tiles(layer)

    def _create_padded_weight_param(self, layer: torch.nn.Module) -> None:
        """A merged layer whose shards differ in type keeps every shard as its own contiguous tensor in
        layer.gguf_shards (gguf-shard-tensors.patch:19-51); shards of one type are concatenated into one
        tensor; a plain layer's single tensor becomes layer.weight.data."""
        weight = layer.weight
        data_container = weight.data_container
        if not data_container:
            return
        if len(data_container) == 1 and not weight.shard_id:
            weight.data = data_container[0].contiguous()
            data_container.clear()
            return
        fallback = layer.weight_type.weight_type
        ordered = _gguf_ordered_shard_ids(weight.shard_id)
        shard_types = {layer.weight_type.shard_weight_type.get(idx, fallback) for idx in ordered}
        mixed = len(shard_types) > 1
        shard_offset_map: dict[Any, tuple[int, int, int]] = {}
        gguf_shards = {}
        parts = []
        current = 0
        for idx in ordered:
            t = data_container[weight.shard_id_map[idx]]
            start, end, size = current, current + t.size(0), t.size(1)
            if mixed:
                gguf_shards[idx] = t.contiguous()
            else:
                parts.append(t)
            shard_offset_map[idx] = (start, end, size)
            current = end
        if mixed:
            layer.gguf_shards = gguf_shards
            weight.data = torch.empty(0, dtype=torch.uint8, device=data_container[0].device)
        else:
            weight.data = torch.cat(parts, dim=0)
        weight.shard_offset_map = shard_offset_map
        data_container.clear()

    def _create_tiles(self, layer: torch.nn.Module) -> None:
        """Every shard (or the whole weight of a layer whose shards share one type) is repacked tile-major
        once and the raw rows are freed (gguf-tiles-all-types.patch:73-131).  A layer flagged
        `gguf_is_embedding` (the token embedding, whose rows are gathered, never multiplied) stays raw."""
        if getattr(layer, "gguf_is_embedding", False):
            return
        tiles, rows, types = {}, {}, {}
        fallback = layer.weight_type.weight_type
        gguf_shards = getattr(layer, "gguf_shards", None)
        if gguf_shards is not None:
            for idx, shard in gguf_shards.items():
                wtype = layer.weight_type.shard_weight_type.get(idx, fallback)
                if wtype in ops.TILE_TYPES and shard.numel() > 0:
                    tiles[idx] = ops.repack_tiles(shard, shard.shape[0], wtype)
                    rows[idx] = shard.shape[0]
                    types[idx] = wtype
            for idx in tiles:
                gguf_shards[idx] = torch.empty(0, dtype=torch.uint8, device=tiles[idx].device)
        elif layer.weight.data.numel() > 0:
            shard_id = getattr(layer.weight, "shard_id", None)
            wtypes = ({layer.weight_type.shard_weight_type.get(idx, fallback) for idx in shard_id} if shard_id else {fallback})
            wtype = next(iter(wtypes))
            if len(wtypes) == 1 and wtype in ops.TILE_TYPES:
                w = layer.weight.data
                tiles["__all__"] = ops.repack_tiles(w, w.shape[0], wtype)
                rows["__all__"] = w.shape[0]
                types["__all__"] = wtype
                layer.weight.data = torch.empty(0, dtype=torch.uint8, device=w.device)
        if tiles:
            layer.gguf_tiles = tiles
            layer.gguf_tiles_rows = rows
            layer.gguf_tiles_types = types
            self._create_groups(layer)

    def _create_groups(self, layer: torch.nn.Module) -> None:
        """Runs of consecutive tiled shards are packed into one buffer with the descriptor tables of the
        splits a launch can choose; the shards' tiles become views into it
        (gguf-tiles-grouped.patch:84-115).  groups[first_idx] = (packed, descs, splits, run, nb, block_bytes)."""
        tiles, rows, types = layer.gguf_tiles, layer.gguf_tiles_rows, layer.gguf_tiles_types
        if "__all__" in tiles:
            runs = [["__all__"]]
        else:
            runs, run = [], []
            for idx in _gguf_ordered_shard_ids(list(layer.weight.shard_id)):
                if idx in tiles:
                    run.append(idx)
                elif run:
                    runs.append(run)
                    run = []
            if run:
                runs.append(run)
        groups = {}
        for run in runs:
            packed, views, descs, splits, nb, block_bytes = ops.prepare_grouped_layer(
                [tiles[i] for i in run], [rows[i] for i in run], [types[i] for i in run])
            for i, v in zip(run, views):
                tiles[i] = v
            groups[run[0]] = (packed, descs, splits, list(run), nb, block_bytes)
        layer.gguf_groups = groups

    # ---- a6 ----
    def apply(self, layer: torch.nn.Module, x: torch.Tensor, bias: torch.Tensor | None = None) -> torch.Tensor:
        lead = x.shape[:-1]
        x2 = x.reshape(-1, x.shape[-1])
        tiles = getattr(layer, "gguf_tiles", None)
        groups = getattr(layer, "gguf_groups", None)
        if not tiles or not groups:
            raise RuntimeError("GGUF layer has no packed tiles: process_weights_after_loading was not run (there is no raw-row path)")
        result, grouped = [], set()
        order = ["__all__"] if "__all__" in tiles else _gguf_ordered_shard_ids(list(layer.weight.shard_id))
        for idx in order:
            if idx in grouped:
                continue
            if idx not in groups:
                raise RuntimeError(f"shard {idx!r} of a GGUF layer is not tiled")
            packed, descs, splits, run, nb, block_bytes = groups[idx]
            result.append(ops.fused_mul_mat_gguf_tiles_grouped(
                x2, packed, descs, splits, [tiles[i] for i in run], [layer.gguf_tiles_rows[i] for i in run],
                [layer.gguf_tiles_types[i] for i in run], nb, block_bytes))
            grouped.update(run)
        out = result[0] if len(result) == 1 else torch.cat(result, dim=1)
        if bias is not None:
            out.add_(bias)
        return out.reshape(*lead, out.shape[-1])


# ---- standalone loading helpers (what vLLM's weight loaders do for a GGUF checkpoint) -----------------

class GGUFLinear(torch.nn.Module):
    """A bare linear layer driven by GGUFLinearMethod, for use outside vLLM (tests, benchmarks)."""

    def __init__(self, input_size: int, output_partition_sizes: list[int], params_dtype=torch.bfloat16, bias: bool = False):
        super().__init__()
        self.input_size = input_size
        self.output_partition_sizes = list(output_partition_sizes)
        self.quant_method = GGUFLinearMethod(GGUFConfig())
        self.quant_method.create_weights(self, input_size, self.output_partition_sizes, input_size, sum(output_partition_sizes), params_dtype)
        self.bias = Parameter(torch.zeros(sum(output_partition_sizes), dtype=params_dtype), requires_grad=False) if bias else None

    def load_shard(self, raw: torch.Tensor, wtype: int, shard_id=None) -> None:
        self.weight.weight_loader(self.weight, raw, shard_id)
        self.weight_type.weight_loader(self.weight_type, wtype, shard_id)

    def finalize(self) -> "GGUFLinear":
        self.quant_method.process_weights_after_loading(self)
        return self

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        return self.quant_method.apply(self, x, self.bias)
