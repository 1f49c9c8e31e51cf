"""The workspace-free entry point, collected last so a run that stops at the first failure has already been
through every other test.

gq_gemv_grouped_static is for callers that cannot allocate device memory where they make the call (an op
invoked where the framework's allocator must not be touched, or a process whose device memory all belongs to
someone else's pool): its scratch is a fixed 8 MiB buffer inside the library.  Here it is called straight
through the C ABI, twice in a row on different inputs, and each result must equal — bit for bit, since both
entry points run the same kernels in the same order — what gq_gemv_grouped gives with a caller-owned
workspace.  Sizes beyond the built-in buffer must be refused on the host."""
import pytest
import torch

from hyperqwen_rtx4080s32_b200 import formats as F
from hyperqwen_rtx4080s32_b200 import ops, synth
from hyperqwen_rtx4080s32_b200._lib import lib

pytestmark = pytest.mark.gpu


def _call_both(x, packed, desc, split, wts, n_total):
    L = lib()
    dev = x.device
    stream = torch.cuda.current_stream(dev).cuda_stream
    m, k = x.shape
    info = ops.run_info(wts)
    y_ref = torch.empty((m, n_total), dtype=torch.bfloat16, device=dev)
    ws = torch.empty(L.gq_workspace_bytes(m, k, n_total, split), dtype=torch.uint8, device=dev)
    assert L.gq_gemv_grouped(x.data_ptr(), m, k, x.stride(0), packed.data_ptr(), desc.data_ptr(), desc.shape[0], split, info,
                             y_ref.data_ptr(), y_ref.stride(0), n_total, ws.data_ptr(), ws.numel(), stream) == 0
    y = torch.full((m, n_total), float("nan"), dtype=torch.bfloat16, device=dev)
    rc = L.gq_gemv_grouped_static(x.data_ptr(), m, k, x.stride(0), packed.data_ptr(), desc.data_ptr(), desc.shape[0], split, info,
                                  y.data_ptr(), y.stride(0), n_total, stream)
    assert rc == 0, L.gq_last_cuda_error()
    torch.cuda.synchronize()
    return y, y_ref


def test_static_workspace_entry_point_matches_twice_in_a_row():
    dev = torch.device("cuda", 0)
    k = 1024
    parts = [(192, F.Q4_K), (70, F.IQ3_S), (64, F.Q2_K)]
    tiles = [ops.repack_tiles(synth.random_blocks(n, k, t, seed=51 + i).to(dev), n, t) for i, (n, t) in enumerate(parts)]
    n_outs, wts = [n for n, _ in parts], [t for _, t in parts]
    packed, views, descs, splits, nb, bb = ops.prepare_grouped_layer(tiles, n_outs, wts)
    n_total = sum(n_outs)
    # first call: split 2 (uses the partial-sum area), 8 rows; second call: another batch size and split, so the
    # buffer still holds the first call's activations and partials when the second starts
    for m, split, seed in ((8, 2, 1), (33, 1, 2)):
        desc = torch.from_numpy(ops.build_descs(wts, n_outs, k, split)).to(dev)
        x = synth.activations(m, k, seed=seed, device=dev)
        y, y_ref = _call_both(x, packed, desc, split, wts, n_total)
        assert not torch.isnan(y).any()
        assert torch.equal(y, y_ref)
        assert ops.device_status() == 0      # the entry point has no workspace to read a status word from: the device's word


def test_static_workspace_entry_point_rejects_oversized_calls():
    L = lib()
    limit = L.gq_static_workspace_limit()
    assert limit == 8 << 20
    # 64 rows x K = 65536 needs far more than 8 MiB of prepared activations: refused before any launch
    assert L.gq_workspace_bytes(64, 65536, 64, 1) > limit
    rc = L.gq_gemv_grouped_static(1, 64, 65536, 65536, 1, 1, 1, 1, 144, 1, 64, 64, 0)
    assert rc == -6 and b"scratch" in L.gq_last_cuda_error()
