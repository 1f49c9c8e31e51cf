"""Generates tests/golden/dequant_golden.npz — run in a container that has the reference checkout and
the gguf package:  python tests/golden/make_golden.py <path to the reference checkout>

Two families of golden vectors for the oracle (oracle/gguf_oracle.c):
  * gguf_<TYPE>_raw / gguf_<TYPE>_w : random valid blocks of each of the eleven types (seeded, our own
    generator) and gguf.quants.dequantize of them — the format reference the reference's tests use
    (gguf-plugin/test_gguf_rco_cpu.py:345-356, gguf-plugin/test_gluon_kq_gpu.py:123-125).
  * kqref_<id>_raw / kqref_<id>_w : the reference's own fixture, reproduced by importing its CPU model
    (gguf-plugin/gluon/kq_ref.py): random_rows(default_rng(3), 6, 512, wt) for wt in 8, 11, 13, 14 in that
    order, and kq_ref.dequantize(kq_ref.parse(raw, wt)) — what test_gguf_rco_cpu.py:345-356 asserts equal to
    gguf-py.
The .npz travels with the repository; the reference checkout does not.
"""
import importlib.util
import os
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
sys.path.insert(0, ROOT)


def main() -> None:
    if len(sys.argv) < 2:
        raise SystemExit("usage: make_golden.py <path to a checkout of the reference repository>")
    ref_root = sys.argv[1]
    from gguf.constants import GGMLQuantizationType as GT
    from gguf.quants import dequantize

    from hyperqwen_rtx4080s32_b200 import formats as F
    from hyperqwen_rtx4080s32_b200 import synth

    out = {}
    for t, name in F.TYPE_NAMES.items():
        raw = synth.random_blocks(6, 512, t, seed=4242 + t).numpy()
        out[f"gguf_{name}_raw"] = raw
        out[f"gguf_{name}_w"] = dequantize(raw, GT(t)).reshape(6, 512).astype(np.float32)
        enc = synth.encoded_weights(4, 512, t, seed=1000 * t)
        out[f"enc_{name}_raw"] = enc
        out[f"enc_{name}_w"] = dequantize(enc, GT(t)).reshape(4, 512).astype(np.float32)
    spec = importlib.util.spec_from_file_location("kq_ref", os.path.join(ref_root, "gguf-plugin", "gluon", "kq_ref.py"))
    kq_ref = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(kq_ref)
    rng = np.random.default_rng(3)
    for wt in (8, 11, 13, 14):
        raw = kq_ref.random_rows(rng, 6, 512, wt)
        w = kq_ref.dequantize(kq_ref.parse(raw, wt))
        assert np.array_equal(w, dequantize(raw, GT(wt)).reshape(6, 512))
        out[f"kqref_{wt}_raw"] = raw
        out[f"kqref_{wt}_w"] = w.astype(np.float32)
    path = os.path.join(HERE, "dequant_golden.npz")
    np.savez_compressed(path, **out)
    print(path, os.path.getsize(path), "bytes,", len(out), "arrays")


if __name__ == "__main__":
    main()
