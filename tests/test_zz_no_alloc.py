"""The allocation-free LM-head entry point against the workspace-taking one.

Some hosts may not call cudaMalloc once they are serving (all memory already belongs to a pool,
or the embedding runtime forbids it); for them the library carries its own fixed scratch array,
out of which it takes every byte of global scratch the two stages use - not only the per-tile
partials but also the prepared hidden rows, their row scales and the exchange slots of shared
tiles.  This file is named to be collected last, so a failure here cannot hide any other test when
the run stops at the first failure.  It works alone in a fresh process and after the other tests."""
import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu

_TORCH_DT = {"bf16": torch.bfloat16, "f32": torch.float32}


def _dt(name):
    from quixicore_metal_b200 import _lib
    return {"bf16": _lib.DTYPE_BF16, "f32": _lib.DTYPE_F32}[name]


def _call(entry, h, wq, dtype, mode, k, seed, ws=None, stream=None):
    from quixicore_metal_b200 import _lib
    L = _lib.lib()
    T, K = h.shape
    V = wq.shape[0]
    ids = torch.full((T,), -7, dtype=torch.int32, device="cuda")
    st = stream if stream is not None else torch.cuda.current_stream().cuda_stream
    if stream is not None:
        torch.cuda.current_stream().synchronize()      # ids is filled on torch's stream
    if entry == "noalloc":
        res = L.qx_cuda_lm_head_sample_q_noalloc(st, h.data_ptr(), wq.data_ptr(), None, ids.data_ptr(), T, V, K,
                                                 b"q8_0", _dt(dtype), mode, k, 0.8, seed, 0.9)
    else:
        res = L.qx_cuda_lm_head_sample_q(st, h.data_ptr(), wq.data_ptr(), None, ids.data_ptr(), ws.data_ptr(),
                                         ws.numel(), T, V, K, b"q8_0", _dt(dtype), mode, k, 0.8, seed, 0.9)
    return res, ids


def _free_bytes():
    return torch.cuda.mem_get_info()[0]        # cudaMemGetInfo: free bytes of the device


@pytest.mark.parametrize("dtype,T", [("bf16", 6), ("f32", 6), ("bf16", 40)])
def test_noalloc_entry_matches_workspace_entry_twice(dtype, T):
    """Same ids as the workspace entry on two calls in a row (they share the built-in array and find
    the previous call's contents in it), for 16-bit hidden rows (streaming kernels, whose prepared
    activations come out of the array too), fp32 hidden rows, and more than 16 rows (tensor-core
    stage 1, whose shared tiles use the array's exchange slots)."""
    from oracle import qx_oracle as O
    from quixicore_metal_b200 import _lib
    from tests._util import check_ids
    rng = np.random.default_rng(3)
    V, K = 5000, 512
    wq_np = O.synth_pack("q8_0", (0.02 * rng.standard_normal((V, K))).astype(np.float32))
    wq = torch.from_numpy(wq_np).cuda()
    L = _lib.lib()
    for rep in range(2):
        h = torch.from_numpy(rng.standard_normal((T, K)).astype(np.float32)).cuda().to(_TORCH_DT[dtype])
        logits = O.lm_head_logits(h.float().cpu().numpy(), wq_np, "q8_0")
        for mode, k in ((0, 0), (1, 0), (2, 50), (3, 32)):
            ws = torch.empty(max(1, L.qx_cuda_lm_head_workspace_bytes(T, V, K, mode, k)), dtype=torch.uint8, device="cuda")
            r0, want = _call("workspace", h, wq, dtype, mode, k, 11 + rep, ws)
            r1, got = _call("noalloc", h, wq, dtype, mode, k, 11 + rep)
            assert r0.code == 0 and r1.code == 0, (r0.detail, r1.detail)
            torch.cuda.synchronize()
            # Token ids: the tolerance of every id comparison in this suite - identical wherever the
            # decision margin exceeds fp32 accumulation noise.  (The two entries may share a tile
            # between a different number of thread blocks, which changes the order of the K sum.)
            _, margin = O.lm_head_sample_from_logits(logits, mode, k=k, temperature=0.8, seed=11 + rep, top_p=0.9,
                                                     return_detail=True)
            check_ids(got.cpu().numpy(), want.cpu().numpy(), margin, 2e-5, f"noalloc/{dtype}/T{T}/mode{mode}")
            assert int(got.min()) >= 0
    assert L.qx_cuda_device_error() == 0


@pytest.mark.parametrize("dtype,T", [("bf16", 6), ("f32", 6), ("bf16", 40)])
def test_noalloc_entry_allocates_nothing(dtype, T):
    """Neither the library's own scratch counter nor the device's free memory moves across calls of
    the entry point on a stream the library has never seen."""
    from oracle import qx_oracle as O
    from quixicore_metal_b200 import _lib
    rng = np.random.default_rng(5)
    V, K = 5000, 512
    wq = torch.from_numpy(O.synth_pack("q8_0", (0.02 * rng.standard_normal((V, K))).astype(np.float32))).cuda()
    h = torch.from_numpy(rng.standard_normal((T, K)).astype(np.float32)).cuda().to(_TORCH_DT[dtype])
    L = _lib.lib()
    # first the kernels are loaded and the array's address is looked up (on the default stream)
    for mode, k in ((0, 0), (3, 32)):
        r, _ = _call("noalloc", h, wq, dtype, mode, k, 1)
        assert r.code == 0, r.detail
    torch.cuda.synchronize()
    fresh = torch.cuda.Stream()
    allocs, free0 = L.qx_cuda_scratch_alloc_count(), _free_bytes()
    for mode, k in ((0, 0), (1, 0), (2, 50), (3, 32)):
        r, ids = _call("noalloc", h, wq, dtype, mode, k, 2, stream=fresh.cuda_stream)
        assert r.code == 0, r.detail
    fresh.synchronize()
    assert L.qx_cuda_scratch_alloc_count() == allocs
    assert _free_bytes() == free0
    assert int(ids.min()) >= 0


def test_noalloc_entry_rejects_oversized_requests():
    from quixicore_metal_b200 import _lib
    L = _lib.lib()
    T, V, K = 64, 128256, 64          # 64 rows x 501 tiles x 32 candidates needs ~8 MB of partials
    assert L.qx_cuda_lm_head_workspace_bytes(T, V, K, 3, 32) > (4 << 20)
    h = torch.zeros((T, K), dtype=torch.bfloat16, device="cuda")
    wq = torch.zeros((8, K // 32, 34), dtype=torch.uint8, device="cuda")   # never dereferenced
    ids = torch.zeros(T, dtype=torch.int32, device="cuda")
    st = L.qx_cuda_lm_head_sample_q_noalloc(torch.cuda.current_stream().cuda_stream, h.data_ptr(), wq.data_ptr(),
                                            None, ids.data_ptr(), T, V, K, b"q8_0", _lib.DTYPE_BF16, 3, 32, 0.8, 1, 0.9)
    assert _lib.STATUS_NAMES[st.code] == "insufficient_workspace"
    assert b"scratch" in st.detail
