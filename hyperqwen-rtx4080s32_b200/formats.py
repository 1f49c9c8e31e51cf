"""The GGML block types of the quantized-linear path: ids, sizes, names.

The eleven types the benchmark's stack mixes (NORTH_STAR_TYPES) and the four codebook types the served checkpoint
also holds (IQ3_XXS, IQ2_XXS, IQ2_XS, IQ2_S: gguf-plugin/gluon/iq3xxs.py:1-20, gguf-plugin/gluon/iq2.py:1-39; and IQ1_M,
which the reference leaves to the plugin's row path).
Block sizes agree with gguf.constants.GGML_QUANT_SIZES and with the constants the reference keeps
(gguf-plugin/gluon/tiles.py:24-36, gguf-plugin/gluon/kq_tiles.py:22, gguf-plugin/gluon/q2k.py:34).
Every type is handled in segments of 256 weights (one "k-block"): a K-quant superblock, or eight
consecutive 32-weight blocks of a legacy / IQ4_NL type.
"""
from __future__ import annotations

QK = 256          # weights per k-block
TILE_ROWS = 64    # output rows per packed tile
SLAB_ROWS = 16    # output rows per lane-ordered slab inside a tile

Q4_0, Q5_0, Q8_0 = 2, 6, 8
Q2_K, Q3_K, Q4_K, Q5_K, Q6_K = 10, 11, 12, 13, 14
IQ4_NL, IQ3_S, IQ4_XS = 20, 21, 23
IQ2_XXS, IQ2_XS, IQ3_XXS, IQ2_S, IQ1_M = 16, 17, 18, 22, 29

TYPE_NAMES = {Q4_0: "Q4_0", Q5_0: "Q5_0", Q8_0: "Q8_0", Q2_K: "Q2_K", Q3_K: "Q3_K", Q4_K: "Q4_K", Q5_K: "Q5_K",
              Q6_K: "Q6_K", IQ4_NL: "IQ4_NL", IQ3_S: "IQ3_S", IQ4_XS: "IQ4_XS", IQ3_XXS: "IQ3_XXS", IQ2_XXS: "IQ2_XXS",
              IQ2_XS: "IQ2_XS", IQ2_S: "IQ2_S", IQ1_M: "IQ1_M"}
TYPE_IDS = {v: k for k, v in TYPE_NAMES.items()}
SUPPORTED_TYPES = frozenset(TYPE_NAMES)
NORTH_STAR_TYPES = frozenset({Q4_0, Q5_0, Q8_0, Q2_K, Q3_K, Q4_K, Q5_K, Q6_K, IQ4_NL, IQ3_S, IQ4_XS})

# (weights per GGML block, bytes per GGML block)
GGML_BLOCK = {Q4_0: (32, 18), Q5_0: (32, 22), Q8_0: (32, 34), IQ4_NL: (32, 18),
              Q2_K: (256, 84), Q3_K: (256, 110), Q4_K: (256, 144), Q5_K: (256, 176), Q6_K: (256, 210),
              IQ3_S: (256, 110), IQ4_XS: (256, 136), IQ3_XXS: (256, 98), IQ2_XXS: (256, 66), IQ2_XS: (256, 74), IQ2_S: (256, 82), IQ1_M: (256, 56)}
# bytes of one row's 256-weight segment
BYTES_PER_256 = {t: (QK // w) * b for t, (w, b) in GGML_BLOCK.items()}
# types whose value has a per-group minimum term (w = d*sc*q - dmin*m)
MIN_TYPES = frozenset({Q2_K, Q4_K, Q5_K})


def bits_per_weight(wtype: int) -> float:
    return BYTES_PER_256[wtype] * 8.0 / QK


def raw_row_bytes(wtype: int, k: int) -> int:
    if k % QK:
        raise ValueError(f"K={k} is not a multiple of {QK}")
    return k // QK * BYTES_PER_256[wtype]


def raw_bytes(wtype: int, n_out: int, k: int) -> int:
    """Bytes of the raw GGUF blocks of an [n_out, k] tensor: the algorithmic byte count of one GEMV."""
    return n_out * raw_row_bytes(wtype, k)
