"""Drop-in fidelity of the host-side surface, checked without a GPU: the three methods of GGUFLinearMethod against
vLLM's LinearMethodBase (the installed vLLM, when it imports), the way the token embedding is told from the LM head,
and a fullgraph Dynamo trace of a module that calls the custom op (fake tensors: no kernel runs)."""
import inspect

import pytest
import torch

from hyperqwen_rtx4080s32_b200 import formats as F
from hyperqwen_rtx4080s32_b200 import ops
from hyperqwen_rtx4080s32_b200.linear import GGUFConfig, GGUFLinearMethod


def test_linear_method_matches_vllm_linear_method_base():
    """The plugin's class derives from vLLM's LinearMethodBase; this mirror must take the same arguments in the same
    order for the three calls vLLM makes (create_weights, process_weights_after_loading, apply)."""
    try:
        from vllm.model_executor.layers.linear import LinearMethodBase
    except Exception as e:   # noqa: BLE001 - vLLM is not a dependency of the path
        pytest.skip(f"vLLM does not import here: {e}")
    for name in ("create_weights", "process_weights_after_loading", "apply"):
        want = list(inspect.signature(getattr(LinearMethodBase, name)).parameters.values())
        got = list(inspect.signature(getattr(GGUFLinearMethod, name)).parameters.values())
        assert [p.name for p in got] == [p.name for p in want], name
        assert [p.kind for p in got] == [p.kind for p in want], name
        for g, w in zip(got, want):
            assert (g.default is inspect.Parameter.empty) == (w.default is inspect.Parameter.empty), f"{name}.{g.name}"
    cfg = GGUFConfig()
    assert cfg.get_name() == "gguf" and torch.bfloat16 in cfg.get_supported_act_dtypes()
    assert isinstance(cfg.get_quant_method(torch.nn.Linear(4, 4)), GGUFLinearMethod)


def test_token_embedding_stays_raw_and_lm_head_is_tiled_by_class_name():
    """gguf-tiles-all-types.patch:80-89: isinstance(VocabParallelEmbedding) and not isinstance(ParallelLMHead)."""
    class VocabParallelEmbedding(torch.nn.Module):
        pass

    class ParallelLMHead(VocabParallelEmbedding):
        pass

    class Plain(torch.nn.Module):
        pass

    is_emb = GGUFLinearMethod._is_token_embedding
    assert is_emb(VocabParallelEmbedding()) and not is_emb(ParallelLMHead()) and not is_emb(Plain())
    flagged = Plain()
    flagged.gguf_is_embedding = True
    assert is_emb(flagged)
    try:
        from vllm.model_executor.layers.vocab_parallel_embedding import ParallelLMHead as VHead, VocabParallelEmbedding as VEmb
    except Exception:   # noqa: BLE001
        return
    assert "VocabParallelEmbedding" in {c.__name__ for c in VEmb.__mro__}
    assert {"VocabParallelEmbedding", "ParallelLMHead"} <= {c.__name__ for c in VHead.__mro__}


def test_custom_op_traces_fullgraph_with_fake_tensors():
    """The reference registers its op so that torch.compile sees one traceable call
    (gguf-plugin/patches/gguf-tiles-grouped.patch:28-74); here Dynamo must capture a module around the op in one graph
    (fullgraph) from fake tensors, with the output shape the fake implementation states."""
    from torch._subclasses.fake_tensor import FakeTensorMode

    nb, n_outs, types = 3, [130, 64], [F.Q4_K, F.Q6_K]

    def fn(x, packed, d1, d2, t0, t1):
        y = ops.fused_mul_mat_gguf_tiles_grouped(x, packed, [d1, d2], [1, 2], [t0, t1], n_outs, types, nb, 177)
        return torch.nn.functional.silu(y[:, :64]) * y[:, 64:128]

    with FakeTensorMode() as mode:
        dev = "meta"
        x = torch.empty((5, 768), dtype=torch.bfloat16, device=dev)
        packed = torch.empty((1 << 16,), dtype=torch.uint8, device=dev)
        d1 = torch.empty((4, 8), dtype=torch.int32, device=dev)
        d2 = torch.empty((8, 8), dtype=torch.int32, device=dev)
        t0 = torch.empty((3, nb, 64 * 144), dtype=torch.uint8, device=dev)
        t1 = torch.empty((1, nb, 64 * 210), dtype=torch.uint8, device=dev)
        y = ops.fused_mul_mat_gguf_tiles_grouped(x, packed, [d1, d2], [1, 2], [t0, t1], n_outs, types, nb, 177)
        assert tuple(y.shape) == (5, 194) and y.dtype == torch.bfloat16
        gm, guards = torch._dynamo.export(fn)(x, packed, d1, d2, t0, t1)
    targets = [n.target for n in gm.graph.nodes if n.op == "call_function"]
    assert any("fused_mul_mat_gguf_tiles_grouped" in str(t) for t in targets), targets
