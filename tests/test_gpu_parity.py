"""GPU parity tests proper: the CUDA path through the C ABI against the CPU oracle on the same seeded
inputs.  Dequantisation and repack are bit-exact; GEMM outputs are within the contract's max relative
error 1e-2 of the fp64 dequantise-then-multiply oracle (bf16 activations, fp32 accumulate, bf16 output)
and within one bf16 rounding of it."""
import numpy as np
import pytest
import torch

from hyperqwen_rtx4080s32_b200 import formats as F
from hyperqwen_rtx4080s32_b200 import ops, synth
from hyperqwen_rtx4080s32_b200.linear import GGUFLinear
from oracle import oracle

pytestmark = pytest.mark.gpu
TOL = 1e-2            # the contract: max |y - y_ref| / max_row |y_ref|
TOL_TIGHT = 6e-3      # bf16 output rounding (2^-8 of the value) plus fp32 accumulation


def dev():
    return torch.device("cuda", 0)


def ref_gemm(x, raw, t):
    return oracle.matmul_f64(x.float().cpu().numpy(), raw.numpy() if isinstance(raw, torch.Tensor) else raw, t)


@pytest.mark.parametrize("t", sorted(F.SUPPORTED_TYPES))
def test_repack_roundtrip_and_golden_positions(t):
    bb = F.BYTES_PER_256[t]
    from hyperqwen_rtx4080s32_b200.hostref import repack_numpy

    for n_out, nb in [(48, 1), (70, 3), (130, 4)]:
        raw = (torch.arange(n_out * nb * bb, dtype=torch.int64) % 251).to(torch.uint8).reshape(n_out, nb * bb)
        tiles = ops.repack_tiles(raw.to(dev()), n_out, t)
        assert tuple(tiles.shape) == (-(-n_out // 64), nb, 64 * bb)
        assert np.array_equal(tiles.cpu().numpy(), repack_numpy(raw.numpy(), t, ops.slab_map(t)))
        assert torch.equal(ops.unrepack_tiles(tiles, n_out, t).cpu(), raw)
    # a strided (row-padded) source
    wide = torch.zeros((70, 3 * bb + 6), dtype=torch.uint8)
    wide[:, :3 * bb] = raw[:70, :3 * bb] if raw.shape[0] >= 70 else 0
    src = wide.to(dev())[:, :3 * bb]
    assert torch.equal(ops.unrepack_tiles(ops.repack_tiles(src, 70, t), 70, t).cpu(), wide[:, :3 * bb])


@pytest.mark.parametrize("t", sorted(F.SUPPORTED_TYPES))
def test_dequant_bit_exact(t, golden):
    name = F.TYPE_NAMES[t]
    for key in (f"gguf_{name}", f"enc_{name}"):
        raw = torch.from_numpy(golden[key + "_raw"])
        tiles = ops.repack_tiles(raw.to(dev()), raw.shape[0], t)
        w = ops.dequantize_tiles(tiles, raw.shape[0], 512, t).cpu().numpy()
        assert np.array_equal(w.view(np.uint32), golden[key + "_w"].view(np.uint32))
        wb = ops.dequantize_tiles(tiles, raw.shape[0], 512, t, torch.bfloat16).cpu()
        assert torch.equal(wb, torch.from_numpy(golden[key + "_w"]).to(torch.bfloat16))
    raw = synth.random_blocks(130, 1024, t, seed=3)
    w = ops.dequantize_tiles(ops.repack_tiles(raw.to(dev()), 130, t), 130, 1024, t).cpu().numpy()
    assert np.array_equal(w.view(np.uint32), oracle.dequantize(raw.numpy(), t).view(np.uint32))


@pytest.mark.parametrize("t", sorted(F.SUPPORTED_TYPES))
@pytest.mark.parametrize("shape", [(130, 768), (48, 5120), (1024, 5120)])
def test_gemv_all_types_all_batches(t, shape):
    n_out, k = shape
    raw = synth.random_blocks(n_out, k, t, seed=11 + t)
    tiles = ops.repack_tiles(raw.to(dev()), n_out, t)
    packed, views, descs, splits, nb, bb = ops.prepare_grouped_layer([tiles], [n_out], [t])
    worst = 0.0
    for m in (1, 2, 4, 8, 16, 17, 32, 33, 64):
        x = synth.activations(m, k, device=dev())
        ref = ref_gemm(x, raw, t)
        for s in sorted(set(splits) | {1, min(2, nb), min(3, nb)}):
            d = descs[splits.index(s)] if s in splits else torch.from_numpy(ops.build_descs([t], [n_out], k, s)).to(dev())
            y = ops.grouped_gemm(x, packed, d, s, [t], n_out)
            y2 = ops.grouped_gemm(x, packed, d, s, [t], n_out)
            assert torch.equal(y, y2) and not torch.isnan(y).any(), "not deterministic or NaN"
            err = oracle.rel_err(y.float().cpu().numpy(), ref)
            worst = max(worst, err)
            assert err < TOL_TIGHT, f"{F.TYPE_NAMES[t]} {shape} M={m} split={s}: {err:.3e}"
    assert worst < TOL


@pytest.mark.parametrize("t", sorted(F.SUPPORTED_TYPES))
def test_gemv_encoded_gaussian_weights(t):
    n_out, k = 256, 1024
    raw = torch.from_numpy(synth.encoded_weights(n_out, k, t, seed=1000 * t + 4))
    tiles = ops.repack_tiles(raw.to(dev()), n_out, t)
    packed, views, descs, splits, nb, bb = ops.prepare_grouped_layer([tiles], [n_out], [t])
    for m in (1, 8, 64):
        x = synth.activations(m, k, device=dev())
        y = ops.mul_mat_tiles_grouped(x, packed, descs, splits, views, [n_out], [t], nb, bb)
        assert oracle.rel_err(y.float().cpu().numpy(), ref_gemm(x, raw, t)) < TOL_TIGHT


def test_activation_range_is_irrelevant():
    """Activations are rescaled by an exact power of two per row before the fp16 MMA, so tiny, huge and
    mixed-magnitude bf16 rows all give the same relative accuracy."""
    t, n_out, k = F.Q4_K, 128, 1024
    raw = synth.random_blocks(n_out, k, t, seed=5)
    tiles = ops.repack_tiles(raw.to(dev()), n_out, t)
    packed, views, descs, splits, nb, bb = ops.prepare_grouped_layer([tiles], [n_out], [t])
    base = synth.activations(4, k).float()
    scales = torch.tensor([1e-30, 1.0, 3e4, 1e30]).reshape(4, 1)
    x = (base * scales).to(torch.bfloat16).to(dev())
    y = ops.mul_mat_tiles_grouped(x, packed, descs, splits, views, [n_out], [t], nb, bb)
    assert oracle.rel_err(y.float().cpu().numpy(), ref_gemm(x, raw, t)) < TOL_TIGHT
    z = torch.zeros((2, k), dtype=torch.bfloat16, device=dev())
    assert float(ops.mul_mat_tiles_grouped(z, packed, descs, splits, views, [n_out], [t], nb, bb).abs().max()) == 0.0


def test_mixed_run_matches_single_shards_bitwise():
    """A mixed-type run in one launch gives every shard's columns bit-identical to the shard alone at the
    same split (the reference's check_mixed, test_gluon_kq_gpu.py:172-195)."""
    k = 1024
    parts = [(70, F.IQ3_S), (130, F.Q6_K), (48, F.Q2_K), (64, F.IQ4_XS)]
    raws = [synth.random_blocks(n, k, t, seed=21 + i) for i, (n, t) in enumerate(parts)]
    tiles = [ops.repack_tiles(r.to(dev()), n, t) for r, (n, t) in zip(raws, parts)]
    n_outs, wts = [n for n, _ in parts], [t for _, t in parts]
    packed, views, descs, splits, nb, bb = ops.prepare_grouped_layer(tiles, n_outs, wts)
    for i, v in enumerate(views):
        assert torch.equal(v, tiles[i])
    for m in (1, 8, 32):
        x = synth.activations(m, k, seed=7 + m, device=dev())
        for s in (1, 2):
            d = torch.from_numpy(ops.build_descs(wts, n_outs, k, s)).to(dev())
            y = ops.grouped_gemm(x, packed, d, s, wts, sum(n_outs))
            col = 0
            for (n, t), tl in zip(parts, tiles):
                d1 = torch.from_numpy(ops.build_descs([t], [n], k, s)).to(dev())
                y1 = ops.grouped_gemm(x, tl.reshape(-1), d1, s, [t], n)
                assert torch.equal(y[:, col:col + n], y1), f"shard {F.TYPE_NAMES[t]} differs at M={m} split={s}"
                col += n


def test_output_into_column_view_and_padding_canaries():
    t, n_out, k = F.Q5_K, 70, 768
    raw = synth.random_blocks(n_out, k, t, seed=2)
    tiles = ops.repack_tiles(raw.to(dev()), n_out, t)
    d = torch.from_numpy(ops.build_descs([t], [n_out], k, 1)).to(dev())
    x = synth.activations(8, k, device=dev())
    wide = torch.full((8, n_out + 64), float("nan"), dtype=torch.bfloat16, device=dev())
    ops.grouped_gemm(x, tiles.reshape(-1), d, 1, [t], n_out, out=wide[:, 32:32 + n_out])
    assert torch.isnan(wide[:, :32]).all() and torch.isnan(wide[:, 32 + n_out:]).all()      # nothing written outside
    assert torch.equal(wide[:, 32:32 + n_out], ops.grouped_gemm(x, tiles.reshape(-1), d, 1, [t], n_out))


def _layer(shards, k, bias=False):
    lin = GGUFLinear(k, [n for _, n, _ in shards], bias=bias)
    raws = {}
    for sid, n, t in shards:
        raws[sid] = synth.random_blocks(n, k, t, seed=31 + (hash(str(sid)) % 7) + t)
        lin.load_shard(raws[sid].to(dev()), t, sid)
    return lin.to(dev()).finalize(), raws


def test_linear_method_single_qkv_gate_up_bias_and_empty_batch():
    k = 1024
    cases = [
        [(None, 130, F.Q4_K)],
        [("q", 256, F.IQ3_S), ("k", 64, F.Q6_K), ("v", 64, F.Q3_K)],     # mixed types, q k v order
        [("v", 64, F.Q4_K), ("q", 256, F.Q4_K), ("k", 64, F.Q4_K)],      # same type, loaded out of order
        [(0, 192, F.IQ4_XS), (1, 192, F.Q2_K)],
    ]
    for shards in cases:
        lin, raws = _layer(shards, k, bias=True)
        lin.bias.data = torch.randn_like(lin.bias.data.float()).to(torch.bfloat16)
        order = ["q", "k", "v"] if "q" in raws else [s for s, _, _ in shards]
        types = {s: t for s, _, t in shards}
        for m in (0, 1, 8, 64, 150):
            x = synth.activations(m, k, device=dev()) if m else torch.empty((0, k), dtype=torch.bfloat16, device=dev())
            y = lin(x)
            assert tuple(y.shape) == (m, sum(n for _, n, _ in shards)) and y.dtype == torch.bfloat16
            if m == 0:
                continue
            ref = np.concatenate([ref_gemm(x, raws[s], types[s]) for s in order], axis=1) + lin.bias.float().cpu().numpy()
            assert oracle.rel_err(y.float().cpu().numpy(), ref) < TOL
        assert lin.weight.data.numel() == 0 or getattr(lin, "gguf_shards", None) is None       # raw rows are freed
        x3 = synth.activations(6, k, device=dev()).reshape(2, 3, k)
        assert tuple(lin(x3).shape) == (2, 3, sum(n for _, n, _ in shards))


def test_cuda_graph_capture_and_replay():
    k = 1024
    lin, raws = _layer([("q", 256, F.Q4_K), ("k", 64, F.IQ3_S), ("v", 64, F.Q8_0)], k)
    x = synth.activations(8, k, device=dev())
    eager = lin(x).clone()
    g = torch.cuda.CUDAGraph()
    s = torch.cuda.Stream()
    s.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(s):
        lin(x)
        s.synchronize()
        with torch.cuda.graph(g, stream=s):
            y = lin(x)
    torch.cuda.current_stream().wait_stream(s)
    x.copy_(synth.activations(8, k, seed=99, device=dev()))
    g.replay()
    torch.cuda.synchronize()
    assert torch.equal(y, lin(x)) and not torch.equal(y, eager)


def test_fake_impl_shape_and_dtype():
    from torch._subclasses.fake_tensor import FakeTensorMode

    lin, _ = _layer([(None, 130, F.Q4_K)], 768)
    packed, descs, splits, run, nb, bb = lin.gguf_groups["__all__"]
    with FakeTensorMode(allow_non_fake_inputs=True):
        x = torch.empty((5, 768), dtype=torch.bfloat16, device=dev())
        y = ops.fused_mul_mat_gguf_tiles_grouped(x, packed, descs, splits, [lin.gguf_tiles["__all__"]], [130], [F.Q4_K], nb, bb)
    assert tuple(y.shape) == (5, 130) and y.dtype == torch.bfloat16


def test_full_size_config0_q4k_properties():
    """BASELINE configs[0] at full size (K=5120, N=17408, M=1): a row subset against the oracle, plus
    linearity in x as the size-independent property."""
    t, n_out, k = F.Q4_K, 17408, 5120
    raw = synth.random_blocks(n_out, k, t, seed=12000 + 4, device=dev())
    tiles = ops.repack_tiles(raw, n_out, t)
    assert torch.equal(ops.unrepack_tiles(tiles, n_out, t), raw)
    packed, views, descs, splits, nb, bb = ops.prepare_grouped_layer([tiles], [n_out], [t])
    x = synth.activations(1, k, device=dev())
    y = ops.mul_mat_tiles_grouped(x, packed, descs, splits, views, [n_out], [t], nb, bb).float().cpu().numpy()
    rows = np.arange(0, n_out, 97)
    ref = ref_gemm(x, raw[rows].cpu(), t)
    assert np.abs(y[:, rows] - ref).max() / np.abs(ref).max() < TOL_TIGHT
    y2 = ops.mul_mat_tiles_grouped((2 * x.float()).to(torch.bfloat16), packed, descs, splits, views, [n_out], [t], nb, bb).float().cpu().numpy()
    assert np.abs(y2 - 2 * y).max() <= 2 ** -7 * np.abs(y).max()


def test_rejects_bad_arguments_on_the_host(gq_lib):
    t, n_out, k = F.Q4_K, 64, 768
    raw = synth.random_blocks(n_out, k, t, seed=1).to(dev())
    tiles = ops.repack_tiles(raw, n_out, t)
    d = torch.from_numpy(ops.build_descs([t], [n_out], k, 1)).to(dev())
    from hyperqwen_rtx4080s32_b200._lib import GqError

    with pytest.raises(GqError):
        ops.grouped_gemm(torch.zeros((65, k), dtype=torch.bfloat16, device=dev()), tiles.reshape(-1), d, 1, [t], n_out)
    with pytest.raises(GqError):
        ops.grouped_gemm(torch.zeros((1, k), dtype=torch.float16, device=dev()), tiles.reshape(-1), d, 1, [t], n_out)
    with pytest.raises(GqError):
        ops.repack_tiles(raw.cpu(), n_out, t)
    x = torch.zeros((1, k), dtype=torch.bfloat16, device=dev())
    ws = torch.empty(256, dtype=torch.uint8, device=dev())
    with pytest.raises(GqError, match="workspace"):
        ops.grouped_gemm(x, tiles.reshape(-1), d, 1, [t], n_out, workspace=ws)
    assert gq_lib.gq_read_status(ws.data_ptr(), 256, 0) >= 0


def test_tensor_parallel_shards_sum_to_the_full_result_on_one_gpu():
    """The tensor-parallel layout emulated on one GPU: each rank's shard (column-split rows, row-split K with
    whole k-blocks and zero-padded activations) runs through the kernel; gathered / summed results equal the
    unsharded oracle product.  tp = 8 makes K / tp = 128-granular (not a multiple of 256)."""
    from hyperqwen_rtx4080s32_b200 import tp

    k, n = 2048, 256
    for size in (2, 8):
        for wtype in (F.Q4_K, F.IQ3_S):
            raw = synth.random_blocks(n, k, wtype, seed=17)
            x = synth.activations(8, k)
            full = ref_gemm(x, raw, wtype)
            cols, total = [], np.zeros_like(full)
            for rank in range(size):
                cs, _ = tp.shard_raw(raw, wtype, "column", rank, size)
                lin = GGUFLinear(k, [cs.shape[0]])
                lin.load_shard(cs.to(dev()), wtype)
                cols.append(lin.finalize()(x.to(dev())).float().cpu().numpy())
                rs, pad = tp.shard_raw(raw, wtype, "row", rank, size)
                own = k // size
                xp = tp.pad_input(x[:, rank * own:(rank + 1) * own].contiguous(), pad).to(dev())
                lin = GGUFLinear(pad.total, [n])
                lin.load_shard(rs.to(dev()), wtype)
                total += lin.finalize()(xp).float().cpu().numpy()
            assert oracle.rel_err(np.concatenate(cols, axis=1), full) < TOL_TIGHT
            assert oracle.rel_err(total, full) < TOL          # eight bf16-rounded partial sums


@pytest.mark.parametrize("t", sorted(F.SUPPORTED_TYPES))
def test_prefill_tcgen05_all_types(t):
    """The large-batch path (dequantise to shared memory, tcgen05 MMA, accumulator in tensor memory) against the
    fp64 oracle: odd tile counts (70 rows: the second tile has 6 valid rows; 320 rows: five tiles, the last pair
    is half empty), batch sizes either side of the 128- and 256-row tiles."""
    for n_out, k in [(70, 768), (320, 1024)]:
        raw = synth.random_blocks(n_out, k, t, seed=11 + t)
        tiles = ops.repack_tiles(raw.to(dev()), n_out, t)
        d1 = torch.from_numpy(ops.build_descs([t], [n_out], k, 1)).to(dev())
        for m in (65, 128, 129, 257, 600):
            x = synth.activations(m, k, device=dev())
            wide = torch.full((m, n_out + 16), float("nan"), dtype=torch.bfloat16, device=dev())
            ops.prefill_gemm(x, tiles.reshape(-1), d1, n_out, out=wide[:, 8:8 + n_out], wtypes=[t])
            assert torch.isnan(wide[:, :8]).all() and torch.isnan(wide[:, 8 + n_out:]).all()
            y = wide[:, 8:8 + n_out]
            assert not torch.isnan(y).any()
            assert torch.equal(y, ops.prefill_gemm(x, tiles.reshape(-1), d1, n_out, wtypes=[t])), "not deterministic"
            err = oracle.rel_err(y.float().cpu().numpy(), ref_gemm(x, raw, t))
            assert err < TOL_TIGHT, f"{F.TYPE_NAMES[t]} [{n_out}x{k}] M={m}: {err:.3e}"


def test_prefill_mixed_run_and_dispatch_boundary():
    """A mixed-type fused layer through the op at M = 64 (grouped kernel) and M = 65 (tcgen05 path): both within
    tolerance of the oracle, and per shard bit-identical to the shard alone on the same path."""
    k = 1024
    parts = [(192, F.Q4_K), (70, F.IQ3_S), (64, F.Q6_K), (130, F.Q2_K)]
    raws = [synth.random_blocks(n, k, t, seed=41 + i) for i, (n, t) in enumerate(parts)]
    tiles = [ops.repack_tiles(r.to(dev()), n, t) for r, (n, t) in zip(raws, parts)]
    n_outs, wts = [n for n, _ in parts], [t for _, t in parts]
    packed, views, descs, splits, nb, bb = ops.prepare_grouped_layer(tiles, n_outs, wts)
    for m in (64, 65, 300):
        x = synth.activations(m, k, device=dev())
        y = ops.fused_mul_mat_gguf_tiles_grouped(x, packed, descs, splits, views, n_outs, wts, nb, bb)
        ref = np.concatenate([ref_gemm(x, r, t) for r, (_, t) in zip(raws, parts)], axis=1)
        assert oracle.rel_err(y.float().cpu().numpy(), ref) < TOL_TIGHT
        if m > 64:
            col = 0
            for (n, t), tl in zip(parts, tiles):
                d1 = torch.from_numpy(ops.build_descs([t], [n], k, 1)).to(dev())
                assert torch.equal(y[:, col:col + n], ops.prefill_gemm(x, tl.reshape(-1), d1, n, wtypes=[t]))
                col += n


def test_row_count_dispatch_takes_the_tcgen05_path_from_33_rows():
    """Up to 32 rows the op runs the grouped kernel, from 33 rows the tcgen05 kernel: same tolerance on both sides of the
    boundary, and bit-identical to calling the kernel of that side directly — for a run wide enough to fill the GPU and
    for a narrow one (where the tcgen05 kernel splits K)."""
    for n_out, k in ((64 * 2 * ops.sm_count(dev()), 512), (320, 5120)):
        t = F.Q4_K
        raw = synth.random_blocks(n_out, k, t, seed=77)
        tl = ops.repack_tiles(raw.to(dev()), n_out, t)
        packed, views, descs, splits, nb, bb = ops.prepare_grouped_layer([tl], [n_out], [t])
        d1 = descs[splits.index(1)]
        for m in (32, 33, 64, 65):
            x = synth.activations(m, k, device=dev())
            y = ops.fused_mul_mat_gguf_tiles_grouped(x, packed, descs, splits, views, [n_out], [t], nb, bb)
            assert oracle.rel_err(y.float().cpu().numpy(), ref_gemm(x, raw, t)) < TOL_TIGHT
            if m > ops.DECODE_MAX_ROWS:
                assert torch.equal(y, ops.prefill_gemm(x, packed, d1, n_out, wtypes=[t]))
            else:
                s = ops.grouped_split_for(n_out // 64, nb, m=m, block_bytes=bb, sms=ops.sm_count(dev()))
                s = s if s in splits else 1
                assert torch.equal(y, ops.grouped_gemm(x, packed, descs[splits.index(s)], s, [t], n_out))


def test_prefill_full_size_down_projection_properties():
    """BASELINE configs[2] shape (down: K 17408, N 5120, Q6_K) at M = 2048: a row/column subset against the
    oracle and linearity in x at full size."""
    t, n_out, k, m = F.Q6_K, 5120, 17408, 2048
    raw = synth.random_blocks(n_out, k, t, seed=14006, device=dev())
    tiles = ops.repack_tiles(raw, n_out, t)
    d1 = torch.from_numpy(ops.build_descs([t], [n_out], k, 1)).to(dev())
    x = synth.activations(m, k, device=dev())
    y = ops.prefill_gemm(x, tiles.reshape(-1), d1, n_out, wtypes=[t]).float()
    rows = torch.arange(0, n_out, 41, device=dev())
    cols_m = np.arange(0, m, 97)
    ref = ref_gemm(x[cols_m].cpu(), raw[rows].cpu(), t)
    assert oracle.rel_err(y[cols_m][:, rows].cpu().numpy(), ref) < TOL_TIGHT
    y2 = ops.prefill_gemm((2 * x.float()).to(torch.bfloat16), tiles.reshape(-1), d1, n_out, wtypes=[t]).float()
    assert float((y2 - 2 * y).abs().max()) <= 2 ** -7 * float(y.abs().max())


def test_fused_all_reduce_single_rank_degenerate():
    """gq_gemv_grouped_allreduce with one rank: the exchange is a round trip through the rank's own buffer, so the
    output is bit-identical to the plain grouped call — for a cluster split, no split, a ragged last tile (scalar
    path), a column-view output, several calls in a row (both slot sets) and a replayed CUDA graph."""
    from hyperqwen_rtx4080s32_b200 import tp

    ctx = tp.LocalFusedAllReduce(max_m=64, max_n_total=512, device=dev())
    for (n_out, k, t) in [(256, 1024, F.Q4_K), (198, 768, F.IQ3_S), (512, 512, F.Q6_K)]:
        raw = synth.random_blocks(n_out, k, t, seed=5)
        tl = ops.repack_tiles(raw.to(dev()), n_out, t)
        for s in (1, 2):
            d = torch.from_numpy(ops.build_descs([t], [n_out], k, s)).to(dev())
            for m in (1, 8, 17, 64):
                x = synth.activations(m, k, device=dev())
                want = ops.grouped_gemm(x, tl.reshape(-1), d, s, [t], n_out)
                for rep in range(3):
                    wide = torch.full((m, n_out + 24), float("nan"), dtype=torch.bfloat16, device=dev())
                    got = ops.grouped_gemm(x, tl.reshape(-1), d, s, [t], n_out, out=wide[:, 8:8 + n_out], allreduce=ctx)
                    assert torch.equal(got, want), f"{F.TYPE_NAMES[t]} n_out={n_out} split={s} M={m} rep={rep}"
                    assert torch.isnan(wide[:, :8]).all() and torch.isnan(wide[:, 8 + n_out:]).all()
    # through the op and a graph
    n_out, k, t = 512, 1024, F.Q4_K
    raw = synth.random_blocks(n_out, k, t, seed=6)
    lin = GGUFLinear(k, [n_out])
    lin.load_shard(raw.to(dev()), t)
    lin.finalize()
    x = synth.activations(8, k, device=dev())
    want = lin(x)
    with ops.fused_allreduce(ctx):
        ctx.used = False
        assert torch.equal(lin(x), want) and ctx.used
        g = torch.cuda.CUDAGraph()
        stream = torch.cuda.Stream()
        stream.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(stream):
            with torch.cuda.graph(g, stream=stream):
                y = lin(x)
        torch.cuda.current_stream().wait_stream(stream)
    for _ in range(3):
        g.replay()
    torch.cuda.synchronize()
    assert torch.equal(y, want)


def test_push_all_reduce_single_rank_degenerate(gq_lib):
    """The push all-reduce kernel with a world of one (its own buffer is the only peer): the result is the input,
    the per-CTA call counters advance, the slot sets alternate, and a replayed CUDA graph keeps working.  The
    multi-rank exchange itself is checked on several GPUs by tests/test_multi_gpu.py."""
    import ctypes

    max_bytes = 64 * 5120 * 2
    nbytes = gq_lib.gq_allreduce_buffer_bytes(1, max_bytes)
    assert nbytes == 4096 + 2 * max_bytes
    buf = torch.zeros(nbytes, dtype=torch.uint8, device=dev())
    ptrs = (ctypes.c_uint64 * 1)(buf.data_ptr())
    stream = torch.cuda.current_stream().cuda_stream
    for m in (1, 8, 64):
        x = synth.activations(m, 5120, seed=m, device=dev())
        y = torch.empty_like(x)
        assert gq_lib.gq_allreduce_push(x.data_ptr(), y.data_ptr(), x.numel() * 2, 0, 1, ptrs, max_bytes, stream) == 0
        torch.cuda.synchronize()
        assert torch.equal(x, y)
    # header: flags [2 sets][8 ranks][32 CTAs] u32, then the 32 per-CTA call counters, then the status word
    counters = buf[2048:2048 + 128].view(torch.int32)
    assert counters.tolist() == [3] * 32 and int(buf[2176:2180].view(torch.int32).item()) == 0
    x = synth.activations(8, 5120, device=dev())
    g = torch.cuda.CUDAGraph()
    s = torch.cuda.Stream()
    s.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(s):
        with torch.cuda.graph(g, stream=s):
            assert gq_lib.gq_allreduce_push(x.data_ptr(), x.data_ptr(), x.numel() * 2, 0, 1, ptrs, max_bytes, s.cuda_stream) == 0
    torch.cuda.current_stream().wait_stream(s)
    before = x.clone()
    for _ in range(3):
        g.replay()
    torch.cuda.synchronize()
    assert torch.equal(x, before) and counters.tolist() == [6] * 32
    assert gq_lib.gq_allreduce_push(x.data_ptr(), x.data_ptr(), max_bytes + 16, 0, 1, ptrs, max_bytes, stream) == -2
    assert gq_lib.gq_allreduce_push(x.data_ptr(), x.data_ptr(), 32, 1, 1, ptrs, max_bytes, stream) == -3
