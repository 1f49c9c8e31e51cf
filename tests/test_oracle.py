"""The CPU oracle pinned against golden vectors: gguf.quants.dequantize outputs and the reference's
own CPU-model fixture (tests/golden/make_golden.py made them)."""
import numpy as np
import pytest

from hyperqwen_rtx4080s32_b200 import formats as F
from oracle import oracle


@pytest.mark.parametrize("name", list(F.TYPE_IDS))
def test_oracle_matches_gguf_py_on_random_blocks(golden, name):
    t = F.TYPE_IDS[name]
    w = oracle.dequantize(golden[f"gguf_{name}_raw"], t)
    assert np.array_equal(w.view(np.uint32), golden[f"gguf_{name}_w"].view(np.uint32))


@pytest.mark.parametrize("name", list(F.TYPE_IDS))
def test_oracle_matches_gguf_py_on_encoded_gaussian(golden, name):
    t = F.TYPE_IDS[name]
    w = oracle.dequantize(golden[f"enc_{name}_raw"], t)
    assert np.array_equal(w.view(np.uint32), golden[f"enc_{name}_w"].view(np.uint32))


@pytest.mark.parametrize("wt", [8, 11, 13, 14])
def test_oracle_matches_reference_cpu_model_fixture(golden, wt):
    # the reference's own check: kq_ref vs gguf-py, default_rng(3), 6 x 512 (test_gguf_rco_cpu.py:345-356)
    w = oracle.dequantize(golden[f"kqref_{wt}_raw"], wt)
    assert np.array_equal(w.view(np.uint32), golden[f"kqref_{wt}_w"].view(np.uint32))


def test_oracle_matches_live_gguf_py_when_installed():
    gguf = pytest.importorskip("gguf")
    from gguf.constants import GGMLQuantizationType as GT
    from gguf.quants import dequantize

    rng = np.random.default_rng(5)
    for name, t in F.TYPE_IDS.items():
        raw = rng.integers(0, 256, size=(3, 2 * F.BYTES_PER_256[t]), dtype=np.uint8)   # every bit pattern, NaN scales included
        with np.errstate(all="ignore"):
            ref = dequantize(raw, GT(t)).reshape(3, 512)
        assert np.array_equal(oracle.dequantize(raw, t).view(np.uint32), ref.view(np.uint32)), name


def test_block_constants_match_reference():
    # gguf-plugin/test_gguf_rco_cpu.py:358-368 pins these block sizes and the IQ4 codebook
    assert (F.BYTES_PER_256[F.IQ3_S], F.BYTES_PER_256[F.IQ4_XS], F.BYTES_PER_256[F.Q4_K]) == (110, 136, 144)
    assert F.BYTES_PER_256[F.Q2_K] == 84 and F.BYTES_PER_256[F.Q8_0] == 8 * 34
    assert tuple(int(v) for v in oracle.iq4_kvalues()) == (-127, -104, -83, -65, -49, -35, -22, -10, 1, 13, 25, 38, 53, 69, 89, 113)
    g = oracle.iq3s_grid_bytes()
    assert g.shape == (512, 4) and int(g[0, 0]) == 1 and g.max() == 15   # top magnitude 15 (gguf-iq3s-grid-top-magnitude.patch)
    for t in F.SUPPORTED_TYPES:
        assert oracle.lib().oracle_bytes_per_256(t) == F.BYTES_PER_256[t]


def test_matmul_c_agrees_with_f64():
    from hyperqwen_rtx4080s32_b200 import synth

    for t in (F.Q4_K, F.IQ3_S, F.Q6_K):
        raw = synth.random_blocks(37, 768, t, seed=9).numpy()
        x = synth.activations(5, 768).float().numpy()
        assert oracle.rel_err(oracle.matmul_c(x, raw, t), oracle.matmul_f64(x, raw, t)) < 1e-5


def test_encoders_are_reasonable():
    from hyperqwen_rtx4080s32_b200 import synth

    w = synth.gaussian_weights(16, 512, seed=1)
    bound = {F.Q2_K: 0.45, F.Q3_K: 0.25, F.IQ3_S: 0.2, F.IQ3_XXS: 0.25, F.IQ2_XXS: 0.45, F.IQ2_XS: 0.4, F.IQ2_S: 0.36, F.IQ1_M: 0.55}
    for t in F.SUPPORTED_TYPES:
        wd = oracle.dequantize(synth.encode(w, t), t)
        assert np.sqrt(((wd - w) ** 2).mean()) / w.std() < bound.get(t, 0.12), F.TYPE_NAMES[t]
