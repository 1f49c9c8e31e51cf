"""GGUF file -> layers: the tensor-name adapter against the tensor list of the checkpoint the reference serves
(tests/golden/qwen35_tensor_names.json, made from the reference's own fixture), the file reader on a GGUF file written
here with the gguf package, and — on a GPU — the loaded layers against the oracle."""
import json
import os

import numpy as np
import pytest
import torch

from hyperqwen_rtx4080s32_b200 import formats as F
from hyperqwen_rtx4080s32_b200 import loader, synth
from oracle import oracle

HERE = os.path.dirname(os.path.abspath(__file__))

# the Hugging Face module sets of the two kinds of block and the top-level names the reference's adapter test expects
# (gguf-plugin/test_gguf_rco_cpu.py:63-81)
GDN = {"input_layernorm.weight", "post_attention_layernorm.weight", "linear_attn.in_proj_qkv.weight", "linear_attn.in_proj_z.weight",
       "linear_attn.in_proj_a.weight", "linear_attn.in_proj_b.weight", "linear_attn.conv1d.weight", "linear_attn.norm.weight",
       "linear_attn.out_proj.weight", "linear_attn.dt_bias", "linear_attn.A_log", "mlp.gate_proj.weight", "mlp.up_proj.weight",
       "mlp.down_proj.weight"}
ATTN = {"input_layernorm.weight", "post_attention_layernorm.weight", "self_attn.q_proj.weight", "self_attn.k_proj.weight",
        "self_attn.v_proj.weight", "self_attn.o_proj.weight", "self_attn.q_norm.weight", "self_attn.k_norm.weight",
        "mlp.gate_proj.weight", "mlp.up_proj.weight", "mlp.down_proj.weight"}
TOP = {"model.language_model.embed_tokens.weight", "model.language_model.norm.weight", "lm_head.weight"}


def test_every_text_tensor_of_the_served_checkpoint_maps():
    doc = json.load(open(os.path.join(HERE, "golden", "qwen35_tensor_names.json"), encoding="utf-8"))
    assert {loader.map_tensor_name(n).hf_name for n, _, _ in doc["top"]} == TOP
    assert sorted(int(i) for i in doc["blocks"]) == list(range(64))
    merged = {}
    for i, tensors in doc["blocks"].items():
        mods = set()
        for suffix, typ, dims in tensors:
            m = loader.map_tensor_name(f"blk.{i}.{suffix}")
            assert m is not None and m.layer == int(i), suffix
            assert m.hf_name.startswith(f"model.language_model.layers.{i}.")
            mods.add(m.hf_name.split(f"layers.{i}.", 1)[1])
            if m.merged:
                merged.setdefault((int(i), m.merged), []).append(m.shard_id)
        assert mods == (ATTN if int(i) % 4 == 3 else GDN), i
    # q / k / v and gate / up arrive as the shards vLLM's merged layers expect
    assert all(sorted(map(str, v)) in (["k", "q", "v"], ["0", "1"]) for v in merged.values())
    assert sum(1 for k in merged if k[1].endswith("qkv_proj")) == 16 and sum(1 for k in merged if k[1].endswith("gate_up_proj")) == 64
    for n in doc["vision_examples"]:
        assert loader.map_tensor_name(n) is None


def _write_gguf(path, tensors):
    from gguf import GGMLQuantizationType, GGUFWriter

    w = GGUFWriter(path, "qwen35")
    w.add_uint32("qwen35.block_count", 1)
    for name, arr, t in tensors:
        if t is None:
            w.add_tensor(name, arr)
        else:
            w.add_tensor(name, arr, raw_dtype=GGMLQuantizationType(t))
    w.write_header_to_file()
    w.write_kv_data_to_file()
    w.write_tensors_to_file()
    w.close()


def _tiny_model():
    k, inter = 512, 768
    spec = [("blk.3.attn_q.weight", 256, k, F.Q4_K), ("blk.3.attn_k.weight", 64, k, F.IQ3_S), ("blk.3.attn_v.weight", 64, k, F.Q6_K),
            ("blk.3.attn_output.weight", k, 256, F.IQ4_XS), ("blk.3.ffn_gate.weight", inter, k, F.IQ3_XXS), ("blk.3.ffn_up.weight", inter, k, F.IQ2_XS),
            ("blk.3.ffn_down.weight", k, inter, F.IQ2_S), ("output.weight", 1000, k, F.Q4_K), ("token_embd.weight", 1000, k, F.IQ2_S)]      # the served file's kinds of type
    tensors = [(n, synth.random_blocks(no, kk, t, seed=300 + i).numpy(), t) for i, (n, no, kk, t) in enumerate(spec)]
    tensors.append(("blk.3.attn_norm.weight", np.ones(k, dtype=np.float32), None))
    tensors.append(("v.blk.0.ln1.weight", np.ones(8, dtype=np.float32), None))
    return spec, tensors


def test_reader_returns_the_bytes_that_were_written(tmp_path):
    spec, tensors = _tiny_model()
    path = str(tmp_path / "tiny.gguf")
    _write_gguf(path, tensors)
    got = {t.name: t for t in loader.read_gguf(path)}
    assert set(got) == {n for n, _, _ in tensors}
    for name, arr, t in tensors:
        g = got[name]
        if t is not None:
            no, kk = next((a, b) for n, a, b, _ in spec if n == name)
            assert g.ggml_type == t and g.shape == (no, kk) and np.array_equal(np.asarray(g.data).reshape(no, -1), arr)
    with pytest.raises(ValueError):
        bad = str(tmp_path / "bad.gguf")
        _write_gguf(bad, [("blk.0.ffn_down.weight", np.zeros((64, 2 * 50), dtype=np.uint8), 19)])      # IQ1_S: a type the kernels do not decode
        loader.load_gguf(bad, device="cpu")


@pytest.mark.gpu
def test_layers_loaded_from_a_gguf_file_match_the_oracle(tmp_path):
    dev = torch.device("cuda", 0)
    spec, tensors = _tiny_model()
    path = str(tmp_path / "tiny.gguf")
    _write_gguf(path, tensors)
    model = loader.load_gguf(path, device=dev)
    assert set(model.linears) == {"layers.3.self_attn.qkv_proj", "layers.3.self_attn.o_proj", "layers.3.mlp.gate_up_proj", "layers.3.mlp.down_proj", "lm_head"}
    assert model.unmapped == ["v.blk.0.ln1.weight"] and "model.language_model.layers.3.input_layernorm.weight" in model.other
    raw = {n: a for n, a, _ in tensors}
    typ = {n: t for n, _, _, t in spec}
    groups = {"layers.3.self_attn.qkv_proj": ["blk.3.attn_q.weight", "blk.3.attn_k.weight", "blk.3.attn_v.weight"],
              "layers.3.self_attn.o_proj": ["blk.3.attn_output.weight"], "layers.3.mlp.gate_up_proj": ["blk.3.ffn_gate.weight", "blk.3.ffn_up.weight"],
              "layers.3.mlp.down_proj": ["blk.3.ffn_down.weight"], "lm_head": ["output.weight"]}
    for key, names in groups.items():
        lin = model.linears[key]
        for m in (1, 8, 40):
            x = synth.activations(m, lin.input_size, device=dev)
            y = lin(x).float().cpu().numpy()
            ref = np.concatenate([oracle.matmul_f64(x.float().cpu().numpy(), raw[n], typ[n]) for n in names], axis=1)
            assert oracle.rel_err(y, ref) < 6e-3, (key, m)
    # the embedding stays raw; looking rows up is a gather + the bit-exact dequantiser
    emb = model.embedding
    table = torch.from_numpy(np.array(emb.data, copy=True)).reshape(emb.shape[0], -1).to(dev)
    ids = torch.tensor([[0, 999, 17], [17, 5, 640]], device=dev)
    got = loader.embedding_lookup(table, emb.ggml_type, ids, dtype=torch.float32).cpu().numpy()
    want = oracle.dequantize(raw["token_embd.weight"], F.IQ2_S)[ids.cpu().numpy().reshape(-1)].reshape(2, 3, -1)
    assert np.array_equal(got.view(np.uint32), want.view(np.uint32))
