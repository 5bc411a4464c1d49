"""The allocation-free LM-head entry point against the workspace-taking one.

Some hosts may not call cudaMalloc once they are serving (all memory already belongs to a pool,
or the embedding runtime forbids it); for them the library carries its own fixed scratch array.
This file is named to be collected last, so a failure here cannot hide any other test when the
run stops at the first failure.  It works alone in a fresh process and after the other tests."""
import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


def _call(entry, h, wq, mode, k, seed, ws=None):
    from quixicore_metal_b200 import _lib
    L = _lib.lib()
    T, K = h.shape
    V = wq.shape[0]
    ids = torch.full((T,), -7, dtype=torch.int32, device="cuda")
    st = torch.cuda.current_stream().cuda_stream
    if entry == "noalloc":
        res = L.qx_cuda_lm_head_sample_q_noalloc(st, h.data_ptr(), wq.data_ptr(), None, ids.data_ptr(), T, V, K,
                                                 b"q8_0", _lib.DTYPE_BF16, mode, k, 0.8, seed, 0.9)
    else:
        res = L.qx_cuda_lm_head_sample_q(st, h.data_ptr(), wq.data_ptr(), None, ids.data_ptr(), ws.data_ptr(),
                                         ws.numel(), T, V, K, b"q8_0", _lib.DTYPE_BF16, mode, k, 0.8, seed, 0.9)
    return res, ids


def test_noalloc_entry_matches_workspace_entry_twice():
    from oracle import qx_oracle as O
    from quixicore_metal_b200 import _lib
    rng = np.random.default_rng(3)
    T, V, K = 6, 5000, 512
    wq = torch.from_numpy(O.synth_pack("q8_0", (0.02 * rng.standard_normal((V, K))).astype(np.float32))).cuda()
    L = _lib.lib()
    for rep in range(2):                       # two calls in a row share the built-in scratch
        h = torch.from_numpy(rng.standard_normal((T, K)).astype(np.float32)).cuda().bfloat16()
        for mode, k in ((0, 0), (1, 0), (2, 50), (3, 32)):
            ws = torch.empty(max(1, L.qx_cuda_lm_head_workspace_bytes(T, V, mode, k)), dtype=torch.uint8, device="cuda")
            r0, want = _call("workspace", h, wq, mode, k, 11 + rep, ws)
            r1, got = _call("noalloc", h, wq, mode, k, 11 + rep)
            assert r0.code == 0 and r1.code == 0, (r0.detail, r1.detail)
            torch.cuda.synchronize()
            # integer token ids from the same kernels: identical, not merely close
            np.testing.assert_array_equal(got.cpu().numpy(), want.cpu().numpy())
            assert int(got.min()) >= 0


def test_noalloc_entry_rejects_oversized_requests():
    from quixicore_metal_b200 import _lib
    L = _lib.lib()
    T, V, K = 64, 128256, 64          # 64 rows x 501 tiles x 32 candidates needs ~8 MB of partials
    assert L.qx_cuda_lm_head_workspace_bytes(T, V, 3, 32) > (4 << 20)
    h = torch.zeros((T, K), dtype=torch.bfloat16, device="cuda")
    wq = torch.zeros((8, K // 32, 34), dtype=torch.uint8, device="cuda")   # never dereferenced
    ids = torch.zeros(T, dtype=torch.int32, device="cuda")
    st = L.qx_cuda_lm_head_sample_q_noalloc(torch.cuda.current_stream().cuda_stream, h.data_ptr(), wq.data_ptr(),
                                            None, ids.data_ptr(), T, V, K, b"q8_0", _lib.DTYPE_BF16, 3, 32, 0.8, 1, 0.9)
    assert _lib.STATUS_NAMES[st.code] == "insufficient_workspace"
    assert b"scratch" in st.detail
