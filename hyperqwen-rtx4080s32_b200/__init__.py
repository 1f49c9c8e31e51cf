"""B200-native GGUF quantized-linear path: load-time tile repack, small-M grouped GEMV/GEMM,
large-M tcgen05 dequant-GEMM and tensor-parallel sharding, behind the vLLM GGUF LinearMethod
surface (create_weights / process_weights_after_loading / apply)."""
from . import formats  # noqa: F401

__all__ = ["formats"]
