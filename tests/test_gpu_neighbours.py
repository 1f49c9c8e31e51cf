"""The callers either side of the path: the ops folded into the activation preparation (silu_and_mul in front of
down_proj, fused_add_rms_norm in front of qkv_proj / gate_up_proj) against the unfused sequence and the fp64 oracle,
and the LM head (248,320 x 5,120: 3,880 tiles, split 1) with the quantized embedding lookup next to it."""
import numpy as np
import pytest
import torch

from hyperqwen_rtx4080s32_b200 import formats as F
from hyperqwen_rtx4080s32_b200 import linear, loader, ops, synth
from oracle import oracle

pytestmark = pytest.mark.gpu
TOL = 6e-3


def dev():
    return torch.device("cuda", 0)


def make_layer(n_outs, k, t, seed):
    lin = linear.GGUFLinear(k, n_outs)
    raws = [synth.random_blocks(n, k, t, seed=seed + i, device=dev()) for i, n in enumerate(n_outs)]
    if len(n_outs) == 1:
        lin.load_shard(raws[0], t)
    else:
        for i, r in enumerate(raws):
            lin.load_shard(r, t, i)
    return lin.finalize(), raws


def vllm_silu_and_mul(t: torch.Tensor) -> torch.Tensor:
    """vLLM's silu_and_mul kernel in torch: silu in fp32 rounded to bf16, then a bf16 product."""
    k = t.shape[-1] // 2
    g = t[..., :k].float()
    return (g / (1.0 + torch.exp(-g))).to(torch.bfloat16) * t[..., k:]


def vllm_fused_add_rms_norm(x, residual, weight, eps):
    """vLLM's fused_add_rms_norm kernel in torch: z = x + residual in bf16, variance of z in fp32, the normalised value
    rounded to bf16 and multiplied by the weight in bf16."""
    z = x + residual if residual is not None else x
    v = z.float()
    var = v.pow(2).mean(-1, keepdim=True)
    return (v * torch.rsqrt(var + eps)).to(torch.bfloat16) * weight, z


@pytest.mark.parametrize("t", [F.Q4_K, F.Q2_K, F.IQ3_S, F.Q8_0])
@pytest.mark.parametrize("m", [1, 8, 16])
def test_silu_and_mul_folded_into_down_proj(t, m):
    k, n = 17408, 5120
    lin, raws = make_layer([n], k, t, 8100 + t)
    gu = synth.activations(m, 2 * k, device=dev()) * 2.0
    want_x = vllm_silu_and_mul(gu)
    y_unfused = lin(want_x)
    y = lin(gu, pre=ops.PreSiluMul())
    # the folded op feeds the same bf16 activations into the same kernel: the outputs are the same bits, except where
    # expf on the device and torch.exp differ in the last bit of a silu value (rare); allow a few
    diff = (y.float() - y_unfused.float()).abs()
    assert (diff > 0).float().mean().item() < 0.02, f"{(diff > 0).float().mean().item():.4f} of the outputs differ from the unfused sequence"
    rows = torch.from_numpy(np.linspace(0, n - 1, 64).astype(np.int64)).to(dev())
    ref = oracle.matmul_f64(want_x.float().cpu().numpy(), raws[0][rows].cpu().numpy(), t)
    assert oracle.rel_err(y[:, rows].float().cpu().numpy(), ref) < TOL
    assert ops.device_status() == 0


@pytest.mark.parametrize("t", [F.Q4_K, F.Q3_K, F.IQ4_XS])
@pytest.mark.parametrize("m", [1, 8, 16])
@pytest.mark.parametrize("with_residual", [True, False])
def test_add_rms_norm_folded_into_gate_up_proj(t, m, with_residual):
    k, n_outs, eps = 5120, [17408, 17408], 1e-6
    lin, raws = make_layer(n_outs, k, t, 8200 + t)
    g = torch.Generator(device=dev()).manual_seed(5)
    x = synth.activations(m, k, device=dev())
    res = (torch.randn((m, k), device=dev(), generator=g) * 3.0).to(torch.bfloat16) if with_residual else None
    w = (1.0 + 0.1 * torch.randn(k, device=dev(), generator=g)).to(torch.bfloat16)
    want_x, want_z = vllm_fused_add_rms_norm(x, res, w, eps)
    pre = ops.PreAddRMSNorm(w, eps, residual=res)
    y = lin(x, pre=pre)
    if with_residual:
        assert torch.equal(pre.residual_out, want_z)
    y_unfused = lin(want_x)
    # a different summation order of the mean square can move a normalised value by one bf16 step: the outputs agree
    # to the output rounding, not to the bit
    err_vs_unfused = oracle.rel_err(y.float().cpu().numpy(), y_unfused.float().cpu().numpy())
    assert err_vs_unfused < 4e-3, f"{err_vs_unfused:.3e}"
    rows = torch.from_numpy(np.linspace(0, n_outs[0] - 1, 48).astype(np.int64)).to(dev())
    ref = oracle.matmul_f64(want_x.float().cpu().numpy(), raws[1][rows].cpu().numpy(), t)
    assert oracle.rel_err(y[:, n_outs[0] + rows].float().cpu().numpy(), ref) < TOL
    assert ops.device_status() == 0


def test_folded_ops_above_sixteen_rows_run_unfused_and_bad_arguments_are_refused():
    k, n = 1024, 512
    lin, raws = make_layer([n], k, F.Q4_K, 8300)
    gu = synth.activations(24, 2 * k, device=dev())
    y = lin(gu, pre=ops.PreSiluMul())
    assert torch.equal(y, lin(ops.PreSiluMul().unfused(gu)))
    x = synth.activations(4, k, device=dev())
    w = torch.ones(k, dtype=torch.bfloat16, device=dev())
    pre = ops.PreAddRMSNorm(w, 1e-6, residual=x.clone())
    pre.residual_out = pre.residual                      # in place: refused, every warp of a row reads the old residual
    with pytest.raises(ops.GqError):
        lin(x, pre=pre)
    packed, descs, splits = lin.gguf_groups[next(iter(lin.gguf_groups))][:3]
    with pytest.raises(ops.GqError):
        ops.grouped_gemm(synth.activations(17, k, device=dev()), packed, descs[0], splits[0], [F.Q4_K], n, pre=ops.PreAddRMSNorm(w))


@pytest.mark.parametrize("t", [F.Q6_K, F.Q4_K])
def test_lm_head_shape_and_embedding_lookup(t):
    """The LM head of the served model: 248,320 x 5,120 (3,880 tiles; the split table gives 1) at 1, 8 and 64 rows on
    a subset of the vocabulary, and rows of the same table gathered the way a quantized embedding is."""
    vocab, k = 248320, 5120
    raw = synth.random_blocks(vocab, k, t, seed=8400 + t, device=dev())
    lin = linear.GGUFLinear(k, [vocab])
    lin.load_shard(raw, t)
    lin.finalize()
    assert ops.grouped_split_for(vocab // 64, k // 256, m=8, block_bytes=F.BYTES_PER_256[t], sms=ops.sm_count(dev())) == 1
    rows = torch.from_numpy(np.unique(np.concatenate([np.linspace(0, vocab - 1, 96).astype(np.int64), [0, 63, 64, vocab - 64, vocab - 1]]))).to(dev())
    for m in (1, 8, 64):
        x = synth.activations(m, k, device=dev())
        y = lin(x)
        assert tuple(y.shape) == (m, vocab) and not torch.isnan(y).any()
        ref = oracle.matmul_f64(x.float().cpu().numpy(), raw[rows].cpu().numpy(), t)
        assert oracle.rel_err(y[:, rows].float().cpu().numpy(), ref) < TOL, f"M={m}"
    ids = torch.tensor([[0, 5, vocab - 1], [77777, 5, 123456]], device=dev())
    emb = loader.embedding_lookup(raw, t, ids, dtype=torch.float32)
    want = oracle.dequantize(raw[ids.reshape(-1)].cpu().numpy(), t).reshape(2, 3, k)
    assert np.array_equal(emb.cpu().numpy(), want)
    assert ops.device_status() == 0


def test_silu_and_mul_folded_into_the_fused_all_reduce_call_single_rank():
    """The row-parallel down_proj of a tensor-parallel block in one call (gq_gemv_grouped_allreduce_silu_mul), world size 1: bit-identical
    to the folded call without the exchange; above 16 rows the op falls back to the unfused sequence."""
    from hyperqwen_rtx4080s32_b200 import tp

    k, n = 2048, 512
    lin, raws = make_layer([n], k, F.Q4_K, 8500)
    ctx = tp.LocalFusedAllReduce(max_m=64, max_n_total=n, device=dev())
    for m in (1, 8, 16, 24):
        gu = synth.activations(m, 2 * k, device=dev())
        want = lin(gu, pre=ops.PreSiluMul())
        with ops.fused_allreduce(ctx):
            ctx.used = False
            got = lin(gu, pre=ops.PreSiluMul())
        assert torch.equal(got, want), m
        assert ctx.used == (m <= 16) or m > 16
    assert ops.device_status() == 0
