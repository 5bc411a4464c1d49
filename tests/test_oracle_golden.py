"""The CPU oracle against fixtures generated from the reference (tests/golden/make_golden.py) and
against known-answer vectors quoted from the reference's own tests."""
import os

import numpy as np
import pytest

from oracle import qx_oracle as O

FMTS = ["q4_0", "q8_0", "q6_K", "mxfp8", "nvfp4", "mxfp4"]


@pytest.fixture(scope="module")
def G(golden_dir):
    return {n: np.load(os.path.join(golden_dir, n + ".npz")) for n in
            ("formats", "codecs", "rng", "compose")}


def test_codec_tables_match_reference(G):
    np.testing.assert_array_equal(O.e4m3_decode(np.arange(256)), G["codecs"]["e4m3"])
    np.testing.assert_array_equal(O.e2m1_decode(np.arange(16)), G["codecs"]["e2m1"])
    assert O.e4m3_decode(np.array([0x7F]))[0] == 480.0          # no NaN code in this contract
    assert O.e8m0_decode(np.array([127]))[0] == 1.0
    assert O.e8m0_decode(np.array([0]))[0] == np.float32(2.0 ** -127)
    assert np.isinf(O.e8m0_decode(np.array([255]))[0])


@pytest.mark.parametrize("fmt", FMTS)
def test_dequantize_matches_reference_bit_for_bit(G, fmt):
    packed = G["formats"][f"{fmt}_packed"]
    bk, bb = O.FORMATS[fmt]
    assert packed.shape == (6, 512 // bk, bb)
    got = O.dequantize(fmt, packed)
    np.testing.assert_array_equal(got.view(np.uint32), G["formats"][f"{fmt}_dequant"].view(np.uint32))


def test_q6k_known_answer_bytes():
    # bindings/pytorch_mps/tests/test_kernel_extensions.py:191-207 : code -22 at column 169,
    # sub-scale -51, d = 0x8C27; times sqrt(1536) rounds to fp16 0xC993.
    p = np.zeros((1, 1, 210), np.uint8)
    p[0, 0, 105] = 10
    p[0, 0, 192 + 10] = 205
    p[0, 0, 208:210] = (0x27, 0x8C)
    w = O.dequantize("q6_K", p)
    assert np.count_nonzero(w) == 16        # zero codes decode to -32: only the scaled sub-block is non-zero
    v = (w[0, 169] * np.float32(np.sqrt(1536.0))).astype(np.float16)
    assert v.view(np.uint16) == np.uint16(0xC993)


def test_rng_matches_reference_twin(G):
    keys = G["rng"]["keys"]
    u = np.array([O.rng_uniform(int(s), int(a), int(b)) for s, a, b in keys], np.float32)
    np.testing.assert_array_equal(u, G["rng"]["u"])
    g = np.array([O.rng_gumbel(int(s), int(a), int(b)) for s, a, b in keys], np.float64)
    np.testing.assert_allclose(g, G["rng"]["g"], rtol=2e-6, atol=2e-6)   # fp32 log vs float64 log


@pytest.mark.parametrize("fmt", FMTS)
def test_composition_matches_reference_torch_cpu(G, fmt):
    C = G["compose"]
    x, bias, bias2, res = C[f"{fmt}_x"], C[f"{fmt}_bias"], C[f"{fmt}_bias2"], C[f"{fmt}_res"]
    for act in ("none", "silu"):
        got = O.decode_linear_epilogue(x, C[f"{fmt}_gate"], fmt, bias, res, act, "bf16")
        ref = C[f"{fmt}_lin_{act}"]
        # fp64 vs torch fp32 accumulation: at most one bf16 ulp, and only on a few entries
        ulp = np.abs(ref) * 2.0 ** -7 + 1e-30
        assert np.all(np.abs(got - ref) <= ulp)
        assert np.mean(got == ref) > 0.97
    got = O.decode_swiglu(x, C[f"{fmt}_gate"], C[f"{fmt}_up"], fmt, bias, bias2, "bf16")
    ref = C[f"{fmt}_swiglu"]
    assert np.all(np.abs(got - ref) <= np.abs(ref) * 2.0 ** -7 + 1e-30)
    assert np.mean(got == ref) > 0.97


def test_gelu_matches_reference_test_formula():
    # tests/correctness/matmul/decode_linear/test_decode_linear.py:16-25
    v = np.linspace(-6, 6, 4001).astype(np.float32)
    z = v * np.float32(0.7071067811865475)
    az = np.abs(z)
    t = 1.0 / (1.0 + np.float32(0.3275911) * az)
    poly = (((((np.float32(1.061405429) * t - np.float32(1.453152027)) * t
               + np.float32(1.421413741)) * t - np.float32(0.284496736)) * t
             + np.float32(0.254829592)) * t)
    ref = 0.5 * v * (1.0 + np.copysign(1.0 - poly * np.exp(-az * az), z))
    np.testing.assert_allclose(O.gelu_erf_as(v), ref, rtol=0, atol=2e-6)


def test_e4m3_encoder_device_rule():
    dec = O.e4m3_decode(np.arange(256))
    # every finite code below the e=15,m=7 slot round-trips (0x7F is never emitted)
    codes = np.array([c for c in range(256) if (c & 0x7F) != 0x7F and (c & 0x7F) <= 0x7E], np.uint8)
    rt = O.e4m3_encode_device(dec[codes])
    keep = codes != 0x80                                  # -0.0 encodes as +0 (x < 0 is false)
    np.testing.assert_array_equal(rt[keep], codes[keep])
    # exact midpoints between neighbours round to the larger magnitude (half away from zero)
    pos = np.arange(0, 0x7E, dtype=np.uint8)
    mid = ((dec[pos].astype(np.float64) + dec[pos + 1].astype(np.float64)) / 2).astype(np.float32)
    np.testing.assert_array_equal(O.e4m3_encode_device(mid), pos + 1)
    np.testing.assert_array_equal(O.e4m3_encode_device(-mid), (pos + 1) | 0x80)
    # saturation and tiny inputs
    assert O.e4m3_encode_device(np.array([1e9, 448.0, 464.0, -1e9], np.float32)).tolist() == [0x7E, 0x7E, 0x7E, 0xFE]
    assert O.e4m3_encode_device(np.array([2.0 ** -11, -(2.0 ** -11)], np.float32)).tolist() == [0x00, 0x80]
    assert O.e4m3_encode_device(np.array([2.0 ** -10], np.float32)).tolist() == [0x01]
    assert O.e4m3_encode_device(np.array([np.nan], np.float32)).tolist() == [0x7E]


def test_per_token_quantizers_reconstruct():
    # tests/correctness/matmul/decode_linear/test_decode_linear.py:204-215 (<= 0.51 * scale)
    rng = np.random.default_rng(177)
    y = O.round_bf16((0.3 * rng.standard_normal((4, 96))).astype(np.float32))
    y[3] = 0.0
    codes, s = O.quantize_per_token(y, "int8")
    assert codes.dtype == np.int8 and s.dtype == np.float32 and s[3] == 0
    assert np.max(np.abs(codes.astype(np.float32) * s[:, None] - y)) <= s.max() * 0.51 + 1e-6
    codes, s = O.quantize_per_token(y, "fp8")
    rec = O.e4m3_decode(codes) * s[:, None]
    assert np.all(np.abs(rec - y) <= 0.0625 * np.abs(y) + s[:, None] * 2.0 ** -9 + 1e-12)
    assert np.all(codes[3] == 0)


def test_mxfp8_rows_scale_is_ceil_pow2():
    rng = np.random.default_rng(5)
    y = O.round_bf16(rng.standard_normal((3, 128)).astype(np.float32) * 3)
    y[0, :32] = 0
    y[1, 32:64] = 448.0            # amax/448 exactly a power of two -> no bump
    blk = O.quantize_mxfp8_rows(y)
    assert blk.shape == (3, 4, 33)
    s = O.e8m0_decode(blk[..., 0])
    amax = np.abs(y.reshape(3, 4, 32)).max(-1)
    nz = amax > 0
    assert np.all(s[nz] * 448 >= amax[nz]) and np.all(s[nz] * 224 < amax[nz])
    assert blk[0, 0, 0] == 127 and np.all(blk[0, 0, 1:] == 0)
    assert blk[1, 1, 0] == 127
    rec = (s[..., None] * O.e4m3_decode(blk[..., 1:])).reshape(3, 128)
    assert np.max(np.abs(rec - y)) <= np.max(s) * 16 + 1e-6


@pytest.mark.parametrize("fmt", FMTS)
def test_synth_pack_roundtrip(fmt):
    rng = np.random.default_rng(9)
    W = (0.02 * rng.standard_normal((4, 512))).astype(np.float32)
    p = O.synth_pack(fmt, W)
    assert p.shape == (4, 512 // O.FORMATS[fmt][0], O.FORMATS[fmt][1]) and p.dtype == np.uint8
    err = np.abs(O.dequantize(fmt, p) - W).max()
    assert err < {"q8_0": 4e-4, "q6_K": 3e-3, "mxfp8": 5e-3}.get(fmt, 2.5e-2)
    r = O.random_packed(fmt, 3, 512, 1)
    assert np.all(np.isfinite(O.dequantize(fmt, r)))


def test_sampler_modes_small():
    rng = np.random.default_rng(0)
    L = rng.standard_normal((3, 700)).astype(np.float32)
    # argmax with an exact tie picks the lower id
    L[0, 10] = L[0, 400] = 9.0
    assert O.lm_head_sample_from_logits(L, 0)[0] == 10
    assert O.lm_head_sample_from_logits(L, 0, vocab_offset=1000)[0] == 1010
    # k = 1 top-k is argmax whatever the seed
    np.testing.assert_array_equal(O.lm_head_sample_from_logits(L, 2, k=1, seed=5, temperature=0.7),
                                  O.lm_head_sample_from_logits(L, 0))
    # categorical == brute-force Gumbel-max
    tok = O.lm_head_sample_from_logits(L, 1, temperature=0.8, seed=123)
    for t in range(3):
        s = (L[t] * (np.float32(1) / np.float32(0.8))).astype(np.float32) + O.rng_gumbel(123, t, np.arange(700))
        assert tok[t] == int(np.argmax(s))
    # top-p draws stay inside the full-vocab nucleus (test_lm_head.py:278-308)
    for p in (0.5, 0.9):
        ls = L.astype(np.float64) / 0.8
        for seed in range(10):
            tok = O.lm_head_sample_from_logits(L, 3, k=32, temperature=0.8, seed=seed, top_p=p)
            for t in range(3):
                pe = np.exp(ls[t] - ls[t].max()); pe /= pe.sum()
                order = np.argsort(-ls[t], kind="stable")
                n = int(np.searchsorted(np.cumsum(pe[order]), p)) + 1
                assert tok[t] in set(order[:n].tolist())
    # all-equal logits: ties resolve to the lowest id (topk.metal:34-53 tie rule)
    Z = np.zeros((1, 40), np.float32)
    assert O.lm_head_sample_from_logits(Z, 0)[0] == 0


# ---- log-probability forms: the restated reference test oracles behave as the reference tests pin ----
def test_topk_logprobs_ties_padding_and_normalisers():
    from oracle import qx_oracle as O
    # all-equal logits: ids ascending, logprob -log(n) (tests/.../test_lm_head.py:420-427)
    ids, lp = O.topk_logprobs(np.zeros(40, np.float32), [31, 7, 19, 3], 4)
    np.testing.assert_array_equal(ids, [3, 7, 19, 31])
    np.testing.assert_allclose(lp, -np.log(4.0), atol=1e-7)
    # invalid ids skipped, short rows padded (:464-482)
    logits = np.arange(10, dtype=np.float32)
    ids, lp = O.topk_logprobs(logits, [4, -1, 10], 3)
    np.testing.assert_array_equal(ids, [4, -1, -1])
    assert lp[0] == 0.0 and np.isneginf(lp[1:]).all()
    # full-vocabulary normaliser makes the admitted mass less than one
    ids, lp = O.topk_logprobs(logits, [9, 8], 2, normalizer_ids=np.arange(10))
    assert np.exp(lp.astype(np.float64)).sum() < 1.0 and ids.tolist() == [9, 8]
    mask = O.packed_allow_mask([[0, 31, 32, 63], []], 64)
    assert mask.tolist() == [[0x80000001, 0x80000001], [0, 0]]


def test_beam_advance_oracle_first_step():
    from oracle import qx_oracle as O
    rng = np.random.default_rng(1)
    logits = rng.standard_normal((4, 50)).astype(np.float32)           # B = 2, BM = 2
    cum = np.array([[0.0, -np.inf], [0.0, -np.inf]], np.float32)
    tok, par, score = O.lm_head_beam_advance_from_logits(logits, cum, 2)
    assert (par == 0).all()
    for b in range(2):
        row = logits[2 * b].astype(np.float64)
        lsm = row - (row.max() + np.log(np.exp(row - row.max()).sum()))
        np.testing.assert_array_equal(tok[b], np.argsort(-lsm, kind="stable")[:2])
        np.testing.assert_allclose(score[b], np.sort(lsm)[::-1][:2], rtol=1e-6)


# ---- BaseQN separate planes ------------------------------------------------------------------------
@pytest.fixture(scope="module")
def BQ(golden_dir):
    return np.load(os.path.join(golden_dir, "base_q.npz"))


def test_base_q_known_answer_bytes():
    # tests/correctness/quantization/base_q/test_base_q_layout.py:22-44
    for bits, lanes, want in [(2, [0, 1, 2, 3] * 4, [0xE4] * 4), (3, list(range(8)), [0x88, 0xC6, 0xFA]),
                              (4, list(range(8)), [0x10, 0x32, 0x54, 0x76]),
                              (5, list(range(8)), [0x20, 0x88, 0x41, 0x8A, 0x39]),
                              (6, list(range(4)), [0x40, 0x20, 0x0C]), (8, list(range(8)), list(range(8)))]:
        np.testing.assert_array_equal(O.base_q_pack(np.array([lanes], np.uint8), bits), np.array([want], np.uint8))
    np.testing.assert_array_equal(O.base_q_pack(np.array([[0xA, 0xB, 0xC, 0xD, 0xE, 0xF, 0x1, 0x2]]), 4),
                                  [[0xBA, 0xDC, 0xFE, 0x21]])
    # scale codecs at their edges (:58-64)
    e8 = O.base_q_scale_values(np.array([0, 1, 127, 128, 254, 255], np.uint8), "e8m0")
    assert e8[0] == np.float32(2.0 ** -127) and e8[2] == 1.0 and e8[3] == 2.0 and np.isinf(e8[-1])
    np.testing.assert_array_equal(O.base_q_scale_values(np.array([0x00, 0x01, 0x38, 0x40, 0xB8], np.uint8), "e4m3"),
                                  np.array([0.0, 2.0 ** -9, 1.0, 2.0, -1.0], np.float32))


def test_base_q_pack_and_dequantize_match_reference_bit_for_bit(BQ):
    keys = sorted(k[:-6] for k in BQ.files if k.endswith("_lanes"))
    assert len(keys) == 16
    for key in keys:
        bits = int(key[1]); _, sd, g, mode = key.split("_")
        group, sym = int(g[1:]), mode == "sym"
        np.testing.assert_array_equal(O.base_q_pack(BQ[key + "_lanes"], bits), BQ[key + "_codes"])
        np.testing.assert_array_equal(O.base_q_unpack(BQ[key + "_codes"], bits), BQ[key + "_lanes"])
        with np.errstate(over="ignore", invalid="ignore"):
            got = O.base_q_dequantize(BQ[key + "_codes"], BQ[key + "_scales"], None if sym else BQ[key + "_biases"],
                                      bits, group, sd, sym)
        np.testing.assert_array_equal(got.view(np.uint32), BQ[key + "_dequant"].view(np.uint32))
    np.testing.assert_array_equal(O.e8m0_decode(np.arange(256)).view(np.uint32), BQ["e8m0_table"].view(np.uint32))
    np.testing.assert_array_equal(O.e4m3_decode(np.arange(256)).view(np.uint32), BQ["e4m3_table"].view(np.uint32))


def test_base_q_consumers_on_the_reference_test_planes():
    # the hand-made planes of tests/correctness/quantization/base_q/test_base_q.py:20-56 (bf16 scales)
    bits, group = 5, 32
    lane = ((np.arange(3 * 64, dtype=np.uint16).reshape(3, 64) * 5 + 3) % (1 << bits)).astype(np.uint8)
    scales = np.array([[0.125, 0.25], [0.5, 0.0625], [0.03125, 1.0]], np.float32)
    biases = np.array([[0.5, 1.0], [0.25, 0.125], [2.0, 0.0625]], np.float32)
    W = O.base_q_dequantize(O.base_q_pack(lane, bits), scales, biases, bits, group, "bf16")
    np.testing.assert_array_equal(W[1, :3], lane[1, :3] * np.float32(0.5) + np.float32(0.25))
    # embedding: invalid ids give zero rows (:318-329)
    got = O.base_q_embedding(W, np.array([[2, -1], [99, 0]]), "f32")
    np.testing.assert_array_equal(got, np.stack([W[2], 0 * W[0], 0 * W[0], W[0]]).reshape(2, 2, -1))
    # all-equal logits: the lowest id wins (:213-225)
    ids, _, _ = O.base_q_lm_head_argmax(np.zeros((17, 32), np.float32), np.ones((32, 2), np.float32), "f16")
    np.testing.assert_array_equal(ids, [0, 0])
    with pytest.raises(ValueError):
        O.base_q_dequantize(O.base_q_pack(lane, bits), np.zeros((3, 2), np.uint8), np.zeros((3, 2), np.uint8), bits, 32, "e4m3")
