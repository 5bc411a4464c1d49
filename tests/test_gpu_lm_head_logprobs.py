"""GPU parity of the LM-head forms that return log-probabilities - lm_head_masked,
lm_head_candidates, lm_head_beam_advance - against the CPU oracle, which restates the reference's own
test oracles (tests/correctness/quantization/lm_head/test_lm_head.py:370-514).  Token ids and parent
beams must be identical; log-probabilities within the reference tests' tolerances."""
import numpy as np
import pytest
import torch

from oracle import qx_oracle as O
from tests._util import FMTS, dev, host, rounded

pytestmark = pytest.mark.gpu

tk = pytest.importorskip("quixicore_metal_b200.tk")


def _mask(rows, V):
    return torch.from_numpy(O.packed_allow_mask(rows, V).view(np.int32)).cuda()


@pytest.mark.parametrize("normalize", ["allowed", "full"])
def test_masked_dense_topk_logprobs_and_empty_row(normalize):
    # test_lm_head.py:392-418
    rng = np.random.default_rng(401 + (normalize == "full"))
    T, V, K, topk = 3, 333, 71, 4
    h = (0.12 * rng.standard_normal((T, K))).astype(np.float32)
    W = (0.11 * rng.standard_normal((V, K))).astype(np.float32)
    bias = (0.03 * rng.standard_normal(V)).astype(np.float32)
    allowed = [[1, 5, 17, 241, 260, 332], [0, 7, 22, 128, 299], []]
    ids, lp = tk.lm_head_masked(dev(h), dev(W), _mask(allowed, V), bias=dev(bias), topk=topk, normalize=normalize)
    logits = (h.astype(np.float64) @ W.astype(np.float64).T + bias).astype(np.float32)
    ref_ids, ref_lp = O.lm_head_masked_from_logits(logits, allowed, topk, normalize)
    np.testing.assert_array_equal(host(ids), ref_ids)
    np.testing.assert_allclose(host(lp)[:2], ref_lp[:2], rtol=5e-5, atol=5e-5)
    assert np.isneginf(host(lp)[2]).all()


def test_masked_ties_choose_lower_token_id():
    # test_lm_head.py:420-427: all logits equal -> ids ascending, logprob = -log(4)
    h = torch.ones((1, 32), device="cuda")
    W = torch.zeros((40, 32), device="cuda")
    ids, lp = tk.lm_head_masked(h, W, _mask([[31, 7, 19, 3]], 40), topk=4)
    np.testing.assert_array_equal(host(ids), np.array([[3, 7, 19, 31]], np.int32))
    np.testing.assert_allclose(host(lp), -np.log(4.0), atol=1e-6)


@pytest.mark.parametrize("fmt", FMTS)
def test_masked_and_candidates_packed(fmt):
    # test_lm_head.py:430-461
    rng = np.random.default_rng(433 + len(fmt))
    T, V, K, topk = 2, 291, 256, 3
    h = (0.08 * rng.standard_normal((T, K))).astype(np.float32)
    packed = O.synth_pack(fmt, (0.1 * rng.standard_normal((V, K))).astype(np.float32))
    bias = (0.02 * rng.standard_normal(V)).astype(np.float32)
    rows = [[2, 9, 36, 117, 257, 290], [0, 5, 32, 88, 180, 233]]
    flat = np.array(rows[0] + rows[1], dtype=np.int32)
    offsets = np.array([0, len(rows[0]), flat.size], dtype=np.int32)
    m_ids, m_lp = tk.lm_head_masked(dev(h), dev(packed), _mask(rows, V), bias=dev(bias), format=fmt, topk=topk)
    c_ids, c_lp = tk.lm_head_candidates(dev(h), dev(packed), dev(flat), dev(offsets), bias=dev(bias), format=fmt, topk=topk)
    logits = (O.lm_head_logits(h, packed, fmt) + bias).astype(np.float32)
    e_ids, e_lp = O.lm_head_masked_from_logits(logits, rows, topk)
    np.testing.assert_array_equal(host(m_ids), e_ids)
    np.testing.assert_array_equal(host(c_ids), e_ids)
    np.testing.assert_allclose(host(m_lp), e_lp, rtol=8e-5, atol=8e-5)
    np.testing.assert_allclose(host(c_lp), e_lp, rtol=8e-5, atol=8e-5)


def test_candidates_skip_invalid_and_pad_short_rows():
    # test_lm_head.py:464-482
    rng = np.random.default_rng(457)
    T, V, K, topk = 2, 43, 37, 4
    h = (0.1 * rng.standard_normal((T, K))).astype(np.float32)
    W = (0.1 * rng.standard_normal((V, K))).astype(np.float32)
    cand = np.array([4, -1, V, 2, 17], dtype=np.int32)
    offsets = np.array([0, 3, 5], dtype=np.int32)
    ids, lp = tk.lm_head_candidates(dev(h), dev(W), dev(cand), dev(offsets), topk=topk)
    logits = (h.astype(np.float64) @ W.astype(np.float64).T).astype(np.float32)
    e_ids, e_lp = O.lm_head_candidates_from_logits(logits, cand, offsets, topk)
    np.testing.assert_array_equal(host(ids), e_ids)
    np.testing.assert_allclose(host(lp)[:, :1], e_lp[:, :1], rtol=5e-5, atol=5e-5)
    np.testing.assert_allclose(host(lp)[1, :2], e_lp[1, :2], rtol=5e-5, atol=5e-5)
    assert np.isneginf(host(lp)[1, 2:]).all() and np.isneginf(host(lp)[0, 1:]).all()


@pytest.mark.parametrize("fmt", ["q4_0", "q8_0", "mxfp8", "nvfp4", "mxfp4"])
@pytest.mark.parametrize("dtype", ["f32", "bf16"])
@pytest.mark.parametrize("V", [1024, 1027])
def test_quantized_beam_advance(fmt, dtype, V):
    # test_lm_head.py:485-514
    rng = np.random.default_rng(503 + len(fmt) + len(dtype) + V)
    B, BM, K = 2, 4, 256
    h = rounded(0.18 * rng.standard_normal((B * BM, K)), dtype)
    packed = O.synth_pack(fmt, (0.14 * rng.standard_normal((V, K))).astype(np.float32))
    bias = (0.025 * rng.standard_normal(V)).astype(np.float32)
    cum = (0.1 * rng.standard_normal((B, BM))).astype(np.float32)
    tok, par, score = tk.lm_head_beam_advance(dev(h, dtype), dev(packed), dev(cum), BM, bias=dev(bias), format=fmt)
    logits = (O.lm_head_logits(h, packed, fmt) + bias).astype(np.float32)
    e_tok, e_par, e_score = O.lm_head_beam_advance_from_logits(logits, cum, BM)
    np.testing.assert_array_equal(host(tok), e_tok)
    np.testing.assert_array_equal(host(par), e_par)
    np.testing.assert_allclose(host(score), e_score, rtol=8e-4, atol=2e-3)


def test_beam_advance_first_step_convention_and_wide_beams():
    """Step 0 sets cum[:, 1:] = -inf: every survivor descends from beam 0.  16 beams, 40 rows in one
    call (the tensor-core stage 1), a vocabulary with a ragged last tile."""
    rng = np.random.default_rng(77)
    B, BM, K, V = 3, 16, 512, 2100
    h = rounded(0.2 * rng.standard_normal((B * BM, K)), "bf16")
    packed = O.synth_pack("q8_0", (0.1 * rng.standard_normal((V, K))).astype(np.float32))
    cum = np.full((B, BM), -np.inf, np.float32)
    cum[:, 0] = 0.0
    tok, par, score = tk.lm_head_beam_advance(dev(h, "bf16"), dev(packed), dev(cum), BM, format="q8_0")
    logits = O.lm_head_logits(h, packed, "q8_0")
    e_tok, e_par, e_score = O.lm_head_beam_advance_from_logits(logits, cum, BM)
    assert (host(par) == 0).all()
    np.testing.assert_array_equal(host(tok), e_tok)
    np.testing.assert_allclose(host(score), e_score, rtol=8e-4, atol=2e-3)


@pytest.mark.parametrize("T", [5, 40])
@pytest.mark.parametrize("fmt", ["q8_0", "nvfp4"])
def test_masked_packed_large_vocabulary_bf16(fmt, T):
    """bf16 hidden rows take the streaming (<= 16 rows) and tensor-core (> 16 rows) stage-1 kernels;
    masks that admit a few thousand scattered tokens, one row that admits everything, one nothing."""
    rng = np.random.default_rng(900 + T)
    V, K, topk = 9000 + 37, 512, 8
    h = rounded(0.3 * rng.standard_normal((T, K)), "bf16")
    packed = O.synth_pack(fmt, (0.1 * rng.standard_normal((V, K))).astype(np.float32))
    rows = [sorted(rng.choice(V, size=int(rng.integers(1, 3000)), replace=False).tolist()) for _ in range(T)]
    rows[0] = list(range(V))
    rows[1] = []
    logits = O.lm_head_logits(h, packed, fmt)
    for normalize in ("allowed", "full"):
        ids, lp = tk.lm_head_masked(dev(h, "bf16"), dev(packed), _mask(rows, V), format=fmt, topk=topk, normalize=normalize)
        e_ids, e_lp = O.lm_head_masked_from_logits(logits, rows, topk, normalize)
        # ids identical except where two admitted logits are closer than fp32 accumulation noise
        got, want = host(ids), e_ids
        for t in range(T):
            if not np.array_equal(got[t], want[t]):
                srt = np.sort(logits[t][rows[t]].astype(np.float64))[::-1][:topk + 1]
                assert np.min(-np.diff(srt)) < 2e-5, (t, got[t], want[t])
        ok = np.isfinite(e_lp)
        np.testing.assert_allclose(host(lp)[ok], e_lp[ok], rtol=2e-4, atol=2e-4)
        assert np.isneginf(host(lp)[1]).all() and (host(ids)[1] == -1).all()


def test_error_messages():
    h = torch.zeros(2, 64, device="cuda")
    w = torch.zeros(300, 2, 34, dtype=torch.uint8, device="cuda")
    m = torch.zeros(2, 10, dtype=torch.int32, device="cuda")
    with pytest.raises(ValueError, match="normalize must be"):
        tk.lm_head_masked(h, w, m, format="q8_0", normalize="some")
    with pytest.raises(RuntimeError, match=r"topk must be in \[1,min\(8,V\)\]"):
        tk.lm_head_masked(h, w, m, format="q8_0", topk=9)
    with pytest.raises(RuntimeError, match="allow_mask must be"):
        tk.lm_head_masked(h, w, m[:, :9], format="q8_0")
    with pytest.raises(RuntimeError, match="T\\+1 offsets"):
        tk.lm_head_candidates(h, w, torch.zeros(3, dtype=torch.int32, device="cuda"),
                              torch.zeros(2, dtype=torch.int32, device="cuda"), format="q8_0")
    with pytest.raises(ValueError, match="format must be"):
        tk.lm_head_beam_advance(h, w, torch.zeros(1, 2, device="cuda"), 2, format="q6_K")
    with pytest.raises(RuntimeError, match=r"beam_width must be in \[1,16\]"):
        tk.lm_head_beam_advance(h, w, torch.zeros(1, 2, device="cuda"), 17, format="q8_0")
    with pytest.raises(RuntimeError, match="cum_log_probs must be"):
        tk.lm_head_beam_advance(h, w, torch.zeros(3, 2, device="cuda"), 2, format="q8_0")
