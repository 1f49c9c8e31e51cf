"""Host logic of the packed layout and the descriptor tables, and the C-ABI's exported symbols (no GPU)."""
import ctypes
import os
import re

import numpy as np
import pytest

from hyperqwen_rtx4080s32_b200 import formats as F

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_library_exports_every_declared_symbol(gq_lib):
    from hyperqwen_rtx4080s32_b200 import _lib

    header = open(os.path.join(ROOT, "include", "gq_b200.h")).read()
    declared = set(re.findall(r"\b(gq_[a-z0-9_]+)\s*\(", header))
    assert declared, "no declarations found"
    for name in declared:
        assert hasattr(gq_lib, name), f"{name} is declared in include/gq_b200.h but not exported"
    assert declared == set(_lib.SIGNATURES), declared ^ set(_lib.SIGNATURES)


@pytest.mark.parametrize("t", sorted(F.SUPPORTED_TYPES))
def test_slab_map_is_a_permutation(gq_lib, t):
    from hyperqwen_rtx4080s32_b200 import ops

    m = ops.slab_map(t)
    bb = F.BYTES_PER_256[t]
    assert gq_lib.gq_bytes_per_256(t) == bb
    assert m.shape == (16 * bb,) and sorted(m.tolist()) == list(range(16 * bb))
    # lane-ordered chunks: the 16 bytes of lane l in any chunk come from rows g and g+8 only (g = l // 4)
    chunks = {2: 4, 6: 4, 8: 8, 10: 2, 11: 3, 12: 4, 13: 5, 14: 6, 16: 0, 17: 0, 18: 2, 20: 4, 21: 2, 22: 0, 23: 4, 29: 0}[t]
    rows = (m[:512 * chunks] // bb).reshape(chunks, 32, 16)
    for l in range(32):
        assert set(np.unique(rows[:, l])) <= {l // 4, l // 4 + 8}


def test_packed_bytes_and_errors(gq_lib):
    assert gq_lib.gq_packed_bytes(F.Q4_K, 70, 768) == 2 * 3 * 64 * 144
    assert gq_lib.gq_packed_bytes(F.Q4_K, 0, 768) == 0
    assert gq_lib.gq_packed_bytes(99, 70, 768) == -1
    assert gq_lib.gq_packed_bytes(F.Q4_K, 70, 700) == -2
    assert gq_lib.gq_bytes_per_256(99) == 0
    assert gq_lib.gq_run_info(2, (ctypes.c_int32 * 2)(F.Q4_K, F.IQ3_S)) == 144 | (1 << 16) | (1 << 22)      # a codebook type: flag, and its kind bit
    assert gq_lib.gq_run_info(1, (ctypes.c_int32 * 1)(F.IQ2_S)) == 82 | (1 << 16) | (F.IQ2_S << 17) | (1 << 26)  # one type: its id in bits 17..21
    assert gq_lib.gq_run_info(1, (ctypes.c_int32 * 1)(5)) == -1


def test_descriptor_rows_two_shards():
    # the reference's fixture: IQ3_S 70 rows + Q4_K 64 rows over three k-blocks (test_gguf_rco_cpu.py:291-301)
    from hyperqwen_rtx4080s32_b200 import ops

    d = ops.build_descs([F.IQ3_S, F.Q4_K], [70, 64], 768, 1)
    assert d.shape == (3, 8)
    assert d[:, 1].tolist() == [21, 21, 12] and d[:, 2].tolist() == [0, 64, 70] and d[:, 3].tolist() == [64, 6, 64]
    assert d[:, 4].tolist() == [0, 0, 0] and d[:, 5].tolist() == [3, 3, 3]
    t21 = 2 * 3 * 64 * 110
    assert d[1, 0] * 16 == 3 * 64 * 110 and d[2, 0] * 16 == t21


@pytest.mark.parametrize("split", [1, 2, 3, 5, 6, 7, 8, 20])
def test_split_partition_is_balanced_and_complete(split):
    # every split index owns a non-empty k-range and the ranges tile nb (test_gguf_rco_cpu.py:310-323)
    from hyperqwen_rtx4080s32_b200 import ops

    nb = 20
    d = ops.build_descs([F.IQ3_S], [6144], nb * 256, split)
    assert d.shape == (96 * split, 8)
    first = d[d[:, 2] == 0]
    assert first[:, 4].tolist() == [(s * nb) // split for s in range(split)]
    assert first[:, 5].tolist() == [((s + 1) * nb) // split for s in range(split)]
    assert first[:, 6].tolist() == list(range(split)) and (first[:, 5] > first[:, 4]).all()
    # every (tile, k-block) covered exactly once
    cover = np.zeros((96, nb), int)
    for r in d:
        cover[r[2] // 64, r[4]:r[5]] += 1
    assert (cover == 1).all()


def test_split_policy_bounds(gq_lib):
    for n_tiles, nb, m in [(16, 20, 1), (112, 20, 8), (544, 20, 8), (80, 68, 64), (3880, 20, 1), (1, 1, 1), (2, 3, 64)]:
        s = gq_lib.gq_split_for(n_tiles, nb, m, 144, 148)
        assert 1 <= s <= nb


def test_split_policy_on_the_decoder_shapes(gq_lib):
    """148 SMs, four CTAs per SM: the largest split that leaves three k-blocks per CTA, fits a cluster of 8 and keeps
    the launch in one wave with headroom for cluster placement."""
    got = {name: gq_lib.gq_split_for(tiles, nb, 8, 144, 148)
           for name, tiles, nb in [("q", 80, 20), ("qkv", 112, 20), ("gate", 272, 20), ("gate_up", 544, 20), ("down", 80, 68), ("kv", 16, 20)]}
    assert got == {"q": 6, "qkv": 4, "gate": 2, "gate_up": 1, "down": 6, "kv": 6}


def test_fused_allreduce_buffer_size_and_argument_checks(gq_lib):
    b2 = gq_lib.gq_fused_allreduce_buffer_bytes(2, 64, 5120)
    b8 = gq_lib.gq_fused_allreduce_buffer_bytes(8, 64, 5120)
    # a header of per-(tile, warp) call counters, then two slot sets of `world` images of 8-byte words per bf16 pair
    assert b2 % 256 == 0 and b8 - b2 == 2 * 6 * 64 * 5120 * 4
    assert gq_lib.gq_fused_allreduce_buffer_bytes(0, 64, 5120) < 0 and gq_lib.gq_fused_allreduce_buffer_bytes(9, 64, 5120) < 0
    assert gq_lib.gq_fused_allreduce_buffer_bytes(2, 65, 5120) < 0 and gq_lib.gq_fused_allreduce_buffer_bytes(2, 8, 0) < 0
    # rejected on the host before anything touches a device: no peers, rank out of range, batch above the buffers'
    peers = (ctypes.c_uint64 * 2)(0, 0)
    args = [None, 8, 256, 256, None, None, 1, 1, 144, None, 64, 64, None, 0]
    assert gq_lib.gq_gemv_grouped_allreduce(*args, 0, 2, None, 64, 64, None) == -3
    assert gq_lib.gq_gemv_grouped_allreduce(*args, 2, 2, peers, 64, 64, None) == -3
    args[1] = 65
    assert gq_lib.gq_gemv_grouped_allreduce(*args, 0, 2, peers, 64, 64, None) == -2


def test_build_descs_rejects_bad_arguments(gq_lib):
    n = (ctypes.c_int64 * 1)(64)
    buf = (ctypes.c_int32 * 64)()
    assert gq_lib.gq_build_descs(1, (ctypes.c_int32 * 1)(99), n, 768, 1, buf) == -1
    assert gq_lib.gq_build_descs(1, (ctypes.c_int32 * 1)(12), n, 700, 1, buf) == -2
    assert gq_lib.gq_build_descs(1, (ctypes.c_int32 * 1)(12), n, 768, 4, buf) == -3     # split > nb
    assert gq_lib.gq_workspace_bytes(8, 700, 64, 1) == -2
    assert gq_lib.gq_workspace_bytes(8, 768, 64, 2) > gq_lib.gq_workspace_bytes(8, 768, 64, 1) > 0


def test_repack_reference_in_numpy_round_trips():
    """The slab map applied in numpy: repack is a permutation plus zero rows, and inverts exactly, for
    n_out not a multiple of the tile (48, 70, 130) and nb in {1, 3, 4} (the reference's shapes)."""
    from hyperqwen_rtx4080s32_b200 import ops
    from hyperqwen_rtx4080s32_b200.hostref import repack_numpy, unrepack_numpy

    for t in sorted(F.SUPPORTED_TYPES):
        bb = F.BYTES_PER_256[t]
        for n_out, nb in [(48, 1), (70, 3), (130, 4)]:
            raw = (np.arange(n_out * nb * bb, dtype=np.int64) % 251).astype(np.uint8).reshape(n_out, nb * bb)
            tiles = repack_numpy(raw, t, ops.slab_map(t))
            assert tiles.shape == (-(-n_out // 64), nb, 64 * bb)
            assert np.array_equal(unrepack_numpy(tiles, n_out, t, ops.slab_map(t)), raw)
            assert int(tiles.astype(np.int64).sum()) == int(raw.astype(np.int64).sum())     # padding rows are zero
