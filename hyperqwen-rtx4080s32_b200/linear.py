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

import itertools

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

    @staticmethod
    def _is_token_embedding(layer: torch.nn.Module) -> bool:
        """The token embedding's rows are gathered, never multiplied through apply, so it is the one GGUF weight
        that stays raw; the LM head, which vLLM derives from the same class, is multiplied and is tiled
        (gguf-tiles-all-types.patch:80-89 tests isinstance(VocabParallelEmbedding) and not isinstance(ParallelLMHead);
        the same test by class name here, so that the module imports without vLLM)."""
        if getattr(layer, "gguf_is_embedding", False):
            return True
        names = {c.__name__ for c in type(layer).__mro__}
        return "VocabParallelEmbedding" in names and "ParallelLMHead" not in names

    @staticmethod
    def _weight_tensors(layer: torch.nn.Module):
        """The layer's raw weight tensors in output order as (key, rows, type, drop): one entry per shard of a
        mixed-type merged layer (key = shard id), otherwise a single entry "__all__" for the whole weight when it has
        one type.  drop() replaces the raw rows by an empty tensor once they have been repacked."""
        fallback = layer.weight_type.weight_type
        type_of = lambda sid: layer.weight_type.shard_weight_type.get(sid, fallback)  # noqa: E731
        shards = getattr(layer, "gguf_shards", None)
        if shards is not None:
            def dropper(sid):
                def drop():
                    shards[sid] = torch.empty(0, dtype=torch.uint8, device=shards[sid].device)
                return drop
            return [(sid, raw, type_of(sid), dropper(sid)) for sid, raw in shards.items()]
        whole = layer.weight.data
        sids = getattr(layer.weight, "shard_id", None)
        kinds = {type_of(sid) for sid in sids} if sids else {fallback}
        if len(kinds) != 1:
            return []

        def drop_whole():
            layer.weight.data = torch.empty(0, dtype=torch.uint8, device=whole.device)
        return [("__all__", whole, next(iter(kinds)), drop_whole)]

    def _create_tiles(self, layer: torch.nn.Module) -> None:
        """Load-time repack: every weight tensor of the layer that apply multiplies is turned tile-major once and its
        raw rows are freed (the reference's step: gguf-tiles-all-types.patch:73-131).  Leaves on the layer
        gguf_tiles / gguf_tiles_rows / gguf_tiles_types keyed by shard id (or "__all__"), the names the plugin reads."""
        if self._is_token_embedding(layer):
            return
        packed = [(key, ops.repack_tiles(raw, raw.shape[0], wtype), raw.shape[0], wtype, drop)
                  for key, raw, wtype, drop in self._weight_tensors(layer)
                  if wtype in ops.TILE_TYPES and raw.numel() > 0]
        if not packed:
            return
        for _, _, _, _, drop in packed:
            drop()
        layer.gguf_tiles = {key: tiles for key, tiles, _, _, _ in packed}
        layer.gguf_tiles_rows = {key: n for key, _, n, _, _ in packed}
        layer.gguf_tiles_types = {key: wtype for key, _, _, wtype, _ in packed}
        self._create_groups(layer)

    def _create_groups(self, layer: torch.nn.Module) -> None:
        """Shards that follow one another in output order and are all tiled form a run: one packed buffer, one launch
        per call.  groups[first shard of the run] = (packed, descriptor tables, their splits, the run's shard ids, nb,
        average bytes per 256 weights), the tuple the plugin's apply unpacks (gguf-tiles-grouped.patch:84-115); the
        shards' tiles become views into the packed buffer."""
        tiles = layer.gguf_tiles
        if "__all__" in tiles:
            order = ["__all__"]
        else:
            order = _gguf_ordered_shard_ids(list(layer.weight.shard_id))
        # cut the output order wherever a shard is not tiled
        runs = [list(g) for tiled, g in itertools.groupby(order, key=lambda sid: sid in tiles) if tiled]
        layer.gguf_groups = {}
        for run in runs:
            packed, views, descs, splits, nb, block_bytes = ops.prepare_grouped_layer(
                [tiles[sid] for sid in run], [layer.gguf_tiles_rows[sid] for sid in run], [layer.gguf_tiles_types[sid] for sid in run])
            tiles.update(zip(run, views))
            layer.gguf_groups[run[0]] = (packed, descs, splits, run, nb, block_bytes)

    def check_status(self, device=None) -> None:
        """Raise if any kernel of the path has reported a bounded wait that ran out on the device since the last
        check (the result of that call was incomplete).  Synchronises; meant for the engine to call between steps."""
        code = ops.device_status(device, clear=True)
        if code:
            raise RuntimeError(f"gq_b200: a kernel reported device status {code} (1: a bounded wait ran out, 2: bad shape) since the last check")

    # ---- a6 ----
    def apply(self, layer: torch.nn.Module, x: torch.Tensor, bias: torch.Tensor | None = None) -> torch.Tensor:
        return self.apply_with_pre(layer, x, None, bias)

    def apply_with_pre(self, layer: torch.nn.Module, x: torch.Tensor, pre, bias: torch.Tensor | None = None) -> torch.Tensor:
        """apply of pre(x), pre being ops.PreSiluMul / ops.PreAddRMSNorm (or None): the op in front of the layer is folded
        into the launch for up to 16 rows.  An addition to the reference's method, whose apply takes the finished
        activation (gguf-tiles-all-types.patch:203-262)."""
        lead = x.shape[:-1]
        x2 = x.reshape(-1, x.shape[-1])
        if pre is not None and getattr(pre, "residual", None) is not None:
            pre.residual = pre.residual.reshape(-1, pre.residual.shape[-1])
            pre.residual_out = pre.residual_out.reshape(-1, pre.residual_out.shape[-1])
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
            args = (packed, descs, splits, [tiles[i] for i in run], [layer.gguf_tiles_rows[i] for i in run],
                    [layer.gguf_tiles_types[i] for i in run], nb, block_bytes)
            result.append(ops.fused_mul_mat_gguf_tiles_grouped(x2, *args) if pre is None else ops.mul_mat_tiles_grouped_pre(x2, pre, *args))
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

    def forward(self, x: torch.Tensor, pre=None) -> torch.Tensor:
        return self.quant_method.apply_with_pre(self, x, pre, self.bias)
