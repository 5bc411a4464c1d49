"""GPU parity of the fused lm_head_sample against the CPU oracle (dequantise, project in fp64,
sample with the restated fused semantics).  Token ids must be identical wherever the oracle's
decision margin is above fp32 accumulation noise."""
import ctypes as C

import numpy as np
import pytest
import torch

from oracle import qx_oracle as O
from tests._util import FMTS, check_ids, dev, host, rounded

pytestmark = pytest.mark.gpu

tk = pytest.importorskip("quixicore_metal_b200.tk")
MODES = {"argmax": 0, "categorical": 1, "topk": 2, "topp": 3}
EPS = 2e-5   # |fp32 - fp64| logit noise is ~3e-6 at K=4096; margins below this are near-ties


def _case(fmt, T, V, K, dtype, seed, hs=0.5, ws=0.3):
    rng = np.random.default_rng(seed)
    W = (ws * rng.standard_normal((V, K))).astype(np.float32)
    Wq = O.synth_pack(fmt, W)
    h = rounded(hs * rng.standard_normal((T, K)), dtype)
    return h, Wq


def _run(h, Wq, fmt, dtype, mode, **kw):
    return host(tk.lm_head_sample(dev(h, dtype), dev(Wq), mode=mode, format=fmt, **kw))


@pytest.mark.parametrize("dtype", ["f32", "bf16"])
@pytest.mark.parametrize("mode", ["argmax", "categorical"])
@pytest.mark.parametrize("fmt", FMTS)
def test_quant_argmax_categorical(fmt, dtype, mode):
    # tests/correctness/quantization/lm_head/test_lm_head.py:132-154 (T,V,K = 4,4000,512)
    h, Wq = _case(fmt, 4, 4000, 512, dtype, 11)
    tok = _run(h, Wq, fmt, dtype, mode, temperature=0.8, seed=3)
    want, margin = O.lm_head_sample(h, Wq, fmt, MODES[mode], temperature=0.8, seed=3, return_detail=True)
    assert tok.dtype == np.int32 and tok.shape == (4,)
    check_ids(tok, want, margin, EPS, f"{fmt}/{mode}")


@pytest.mark.parametrize("k", [1, 8, 32, 50, 64])
@pytest.mark.parametrize("fmt", ["q8_0", "q4_0", "mxfp8", "nvfp4", "mxfp4", "q6_K"])
def test_quant_topk(fmt, k):
    # test_lm_head.py:256-275
    h, Wq = _case(fmt, 4, 4000, 512, "f32", 21 + k)
    for seed in (3, 4):
        tok = _run(h, Wq, fmt, "f32", "topk", k=k, temperature=0.8, seed=seed)
        want, margin = O.lm_head_sample(h, Wq, fmt, 2, k=k, temperature=0.8, seed=seed, return_detail=True)
        check_ids(tok, want, margin, EPS, f"{fmt}/topk{k}")
    if k == 1:
        L = O.lm_head_logits(h, Wq, fmt)
        np.testing.assert_array_equal(tok, L.argmax(-1))


@pytest.mark.parametrize("p", [0.5, 0.9, 1.0])
@pytest.mark.parametrize("fmt", ["q8_0", "q4_0", "mxfp8", "nvfp4", "mxfp4"])
def test_quant_topp(fmt, p):
    # test_lm_head.py:278-308: 40 seeds, every draw inside the full-vocab nucleus; here also
    # equal to the restated fused rule.
    h, Wq = _case(fmt, 2, 4000, 512, "f32", 41 + int(p * 10), hs=0.6)
    L = O.lm_head_logits(h, Wq, fmt)
    exact = total = 0
    for seed in range(40):
        tok = _run(h, Wq, fmt, "f32", "topp", k=32, temperature=0.8, seed=seed, top_p=p)
        want, margin = O.lm_head_sample_from_logits(L, 3, k=32, temperature=0.8, seed=seed, top_p=p,
                                                    return_detail=True)
        exact += check_ids(tok, want, margin, 1e-4, f"{fmt}/topp{p}/seed{seed}")
        total += 2
        ls = L.astype(np.float64) / 0.8
        for t in range(2):
            pe = np.exp(ls[t] - ls[t].max()); pe /= pe.sum()
            order = np.argsort(-ls[t], kind="stable")
            n = min(int(np.searchsorted(np.cumsum(pe[order]), p - 1e-9)) + 1, 4000)
            assert int(tok[t]) in set(order[:n].tolist())
    assert exact >= total - 2


def test_topp_true_normalizer_tail():
    # test_lm_head.py:311-357: V=1024 K=256 p=0.7: many identical rows, noise varies with the row
    V, K, temp, k, p, scale = 1024, 256, 1.0, 32, 0.7, 0.35
    rng = np.random.default_rng(0)
    Wq = O.synth_pack("q8_0", (scale * rng.standard_normal((V, K))).astype(np.float32))
    h1 = (scale * rng.standard_normal((1, K))).astype(np.float32)
    h = np.repeat(h1, 800, axis=0)
    tok = _run(h, Wq, "q8_0", "f32", "topp", k=k, temperature=temp, seed=0, top_p=p)
    want, margin = O.lm_head_sample(h, Wq, "q8_0", 3, k=k, temperature=temp, seed=0, top_p=p, return_detail=True)
    assert check_ids(tok, want, margin, 1e-4, "true-normalizer") >= 790
    L = O.lm_head_logits(h1, Wq, "q8_0")[0].astype(np.float64)
    pool = np.concatenate([np.argsort(-L[a:a + 256])[:k] + a for a in range(0, V, 256)])
    mx = L.max(); Zf = np.exp(L - mx).sum(); Zp = np.exp(L[pool] - mx).sum()
    order = pool[np.argsort(-L[pool])]

    def nucleus(Z):
        cum, s = 0.0, []
        for v in order:
            cum += np.exp(L[v] - mx) / Z; s.append(int(v))
            if cum >= p:
                break
        return set(s)
    true_n, pool_n = nucleus(Zf), nucleus(Zp)
    assert set(tok.tolist()) <= true_n
    assert sum(int(x) in (true_n - pool_n) for x in tok) > 0


@pytest.mark.parametrize("mode", ["argmax", "categorical", "topk", "topp"])
def test_q6k_ragged_vocab_with_bias(mode):
    # test_lm_head.py:157-176 (V=1025: a one-row last tile) plus an fp32 bias
    T, V, K = 3, 1025, 512
    rng = np.random.default_rng(57)
    Wq = O.synth_pack("q6_K", (0.2 * rng.standard_normal((V, K))).astype(np.float32))
    h = (0.25 * rng.standard_normal((T, K))).astype(np.float32)
    bias = rng.standard_normal(V).astype(np.float32)
    tok = _run(h, Wq, "q6_K", "f32", mode, k=8, temperature=0.8, seed=19, bias=dev(bias), top_p=0.9)
    want, margin = O.lm_head_sample(h, Wq, "q6_K", MODES[mode], k=8, temperature=0.8, seed=19,
                                    top_p=0.9, bias=bias, return_detail=True)
    check_ids(tok, want, margin, EPS, mode)


def test_ties_resolve_to_lowest_id():
    """All-equal logits: every mode's tie rule is 'smaller id wins' (topk.metal:34-53)."""
    V, K = 600, 64
    Wq = np.zeros((V, K // 32, 34), np.uint8)           # q8_0 zeros -> all logits 0
    h = np.ones((2, K), np.float32)
    assert _run(h, Wq, "q8_0", "f32", "argmax").tolist() == [0, 0]
    tok = _run(h, Wq, "q8_0", "f32", "topk", k=4, temperature=1.0, seed=1)
    want = O.lm_head_sample(h, Wq, "q8_0", 2, k=4, temperature=1.0, seed=1)
    np.testing.assert_array_equal(tok, want)             # picks among ids {0,1,2,3}
    assert set(tok.tolist()) <= {0, 1, 2, 3}
    tok = _run(h, Wq, "q8_0", "f32", "topp", k=2, temperature=1.0, seed=1, top_p=0.5)
    want = O.lm_head_sample(h, Wq, "q8_0", 3, k=2, temperature=1.0, seed=1, top_p=0.5)
    np.testing.assert_array_equal(tok, want)


@pytest.mark.parametrize("V,k", [(40000, 50), (3000, 50), (40000, 8), (300, 8)])
def test_topk_merge_with_massive_ties_and_few_groups(V, k):
    """All-equal logits over many vocabulary tiles: every candidate of every tile ties at the stage-2
    threshold (more than the merge stage keeps in shared memory after its group-maxima prefilter, so
    it searches the candidates where they lie), and a vocabulary with fewer tiles than k (no
    prefilter).  The top-k set is the k lowest ids, the draw is the oracle's."""
    K = 64
    Wq = np.zeros((V, K // 32, 34), np.uint8)
    h = np.ones((3, K), np.float32)
    for dtype in ("f32", "bf16"):
        tok = _run(h, Wq, "q8_0", dtype, "topk", k=k, temperature=1.0, seed=5)
        want = O.lm_head_sample(h, Wq, "q8_0", 2, k=k, temperature=1.0, seed=5)
        np.testing.assert_array_equal(tok, want)
        assert int(tok.max()) < k


def test_topk_merge_prefilter_matches_the_oracle_on_clustered_logits():
    """Logits in a few tight clusters (many near-equal tile maxima): the prefilter's lower bound keeps
    every member of the true top-k."""
    rng = np.random.default_rng(21)
    V, K, T = 20000, 256, 5
    W = (0.02 * rng.standard_normal((V, K))).astype(np.float32)
    W[rng.integers(0, V, 400)] *= 3.0                  # a few hundred rows stand out
    Wq = O.synth_pack("q8_0", W)
    h = rounded(rng.standard_normal((T, K)), "bf16")
    for k in (8, 50, 64):
        tok = _run(h, Wq, "q8_0", "bf16", "topk", k=k, temperature=0.7, seed=9)
        want, margin = O.lm_head_sample(h, Wq, "q8_0", 2, k=k, temperature=0.7, seed=9, return_detail=True)
        check_ids(tok, want, margin, EPS, f"topk{k}/clustered")


@pytest.mark.parametrize("T", [1, 8, 9, 64])
def test_batch_sizes_q8_0_bf16(T):
    """Hidden-row counts of the benchmark configuration on a reduced vocabulary."""
    h, Wq = _case("q8_0", T, 8192 + 77, 1024, "bf16", 5 + T, hs=1.0, ws=0.02)
    L = O.lm_head_logits(h, Wq, "q8_0")
    for mode, kw in (("argmax", {}), ("topk", dict(k=50)), ("topp", dict(k=32, top_p=0.9)), ("categorical", {})):
        tok = _run(h, Wq, "q8_0", "bf16", mode, temperature=0.8, seed=1234, **kw)
        want, margin = O.lm_head_sample_from_logits(L, MODES[mode], k=kw.get("k", 0), temperature=0.8,
                                                    seed=1234, top_p=kw.get("top_p", 0.9), return_detail=True)
        n = check_ids(tok, want, margin, EPS, f"T{T}/{mode}")
        assert n >= T - 1


@pytest.mark.parametrize("T", [17, 32, 33, 64, 100])
@pytest.mark.parametrize("fmt", ["q8_0", "q4_0", "mxfp8", "nvfp4", "mxfp4"])
def test_many_hidden_rows_all_formats(fmt, T):
    """More than 16 hidden rows per call (the tensor-memory form of stage 1): every packed format,
    row counts on both sides of the 32- and 64-row pass sizes, a ragged last vocabulary tile."""
    dtype = "f16" if T == 33 else "bf16"
    h, Wq = _case(fmt, T, 2048 + 77, 1024, dtype, 300 + T, hs=1.0, ws=0.05)
    L = O.lm_head_logits(h, Wq, fmt)
    for mode, kw in (("argmax", {}), ("topk", dict(k=50)), ("topp", dict(k=32, top_p=0.9)), ("categorical", {})):
        tok = _run(h, Wq, fmt, dtype, mode, temperature=0.8, seed=77, **kw)
        want, margin = O.lm_head_sample_from_logits(L, MODES[mode], k=kw.get("k", 0), temperature=0.8,
                                                    seed=77, top_p=kw.get("top_p", 0.9), return_detail=True)
        n = check_ids(tok, want, margin, EPS, f"{fmt}/T{T}/{mode}")
        assert n >= T - 1


@pytest.mark.parametrize("mode", ["argmax", "categorical", "topk", "topp"])
@pytest.mark.parametrize("shards", [2, 3, 8])
def test_vocab_sharded_merge_equals_single_call(mode, shards):
    """The shard entry points (stage 1 per shard, gather, stage 2) on one device: shards are
    256-aligned slices of the vocabulary, ids stay global.  Must equal the unsharded call."""
    from quixicore_metal_b200 import parallel
    fmt, T, V, K = "q8_0", 5, 4000 + 13, 512
    h, Wq = _case(fmt, T, V, K, "bf16", 77)
    kw = dict(k=16, temperature=0.8, seed=42, top_p=0.9)
    single = _run(h, Wq, fmt, "bf16", mode, **kw)
    hd, wd = dev(h, "bf16"), dev(Wq)
    bounds = parallel.vocab_shard_bounds(V, shards)
    assert all(b[0] % 256 == 0 for b in bounds) and bounds[-1][1] == V
    parts = [parallel.lm_head_shard_partials(hd, wd[a:b].contiguous(), None, a, parallel.max_shard_tiles(V, shards),
                                             fmt, mode, **{k_: v for k_, v in kw.items() if k_ != "top_p"})
             for a, b in bounds]
    merged = parallel.lm_head_merge(parts, mode, max_tiles=parallel.max_shard_tiles(V, shards), **kw)
    np.testing.assert_array_equal(host(merged), single)


@pytest.mark.parametrize("fmt,K", [("q8_0", 256), ("q8_0", 512), ("nvfp4", 512), ("mxfp4", 1024)])
def test_last_round_items_shared_between_ctas(fmt, K):
    """More 256-row tiles than SMs with a small remainder (160 tiles): the tiles of the last, partial
    round are each computed by 2 or 4 CTAs that take a slice of K and exchange partial logits."""
    T, V = 20, 160 * 256 - 40
    h, Wq = _case(fmt, T, V, K, "bf16", 500 + K, hs=1.0, ws=0.05)
    L = O.lm_head_logits(h, Wq, fmt)
    for mode, kw in (("argmax", {}), ("topp", dict(k=32, top_p=0.9)), ("topk", dict(k=8))):
        tok = _run(h, Wq, fmt, "bf16", mode, temperature=0.8, seed=5, **kw)
        want, margin = O.lm_head_sample_from_logits(L, MODES[mode], k=kw.get("k", 0), temperature=0.8,
                                                    seed=5, top_p=kw.get("top_p", 0.9), return_detail=True)
        n = check_ids(tok, want, margin, EPS, f"{fmt}/K{K}/{mode}")
        assert n >= T - 1


@pytest.mark.parametrize("mode", ["argmax", "topk", "topp"])
def test_vocab_sharded_merge_many_hidden_rows(mode):
    """The shard entry points with more than 16 hidden rows (tensor-memory stage 1 per shard, padding
    tiles of the short last shard, global ids through vocab_offset) equal the unsharded call."""
    from quixicore_metal_b200 import parallel
    fmt, T, V, K, shards = "q8_0", 40, 3000 + 13, 512, 3
    h, Wq = _case(fmt, T, V, K, "bf16", 91)
    kw = dict(k=16, temperature=0.8, seed=42, top_p=0.9)
    single = _run(h, Wq, fmt, "bf16", mode, **kw)
    hd, wd = dev(h, "bf16"), dev(Wq)
    bounds = parallel.vocab_shard_bounds(V, shards)
    parts = [parallel.lm_head_shard_partials(hd, wd[a:b].contiguous(), None, a, parallel.max_shard_tiles(V, shards),
                                             fmt, mode, **{k_: v for k_, v in kw.items() if k_ != "top_p"})
             for a, b in bounds]
    merged = parallel.lm_head_merge(parts, mode, max_tiles=parallel.max_shard_tiles(V, shards), **kw)
    np.testing.assert_array_equal(host(merged), single)


def test_generic_dispatch_entry_point():
    """qx_cuda_dispatch with the contract's call structs (kernel_abi.hpp mirror)."""
    from quixicore_metal_b200 import _lib, capi
    h, Wq = _case("q4_0", 3, 1000, 256, "f32", 8)
    hd, wd = dev(h), dev(Wq)
    out = torch.empty(3, dtype=torch.int32, device="cuda")
    call = capi.KernelCall(inputs=[hd, wd], outputs=[out],
                           attrs=dict(format="q4_0", mode=2, topk=8, temperature=0.7, seed=9))
    nbytes = _lib.lib().qx_cuda_workspace_bytes(b"quantized_lm_head_sample", call.ref())
    assert nbytes == _lib.lib().qx_cuda_lm_head_workspace_bytes(3, 1000, 256, 2, 8) > 0
    ws = torch.empty(nbytes, dtype=torch.uint8, device="cuda")
    call.set_workspace(ws)
    _lib.check(_lib.lib().qx_cuda_dispatch(b"quantized_lm_head_sample", call.ref()))
    torch.cuda.synchronize()
    want = O.lm_head_sample(h, Wq, "q4_0", 2, k=8, temperature=0.7, seed=9)
    np.testing.assert_array_equal(host(out), want)
    # projection through the same door
    x = rounded(np.random.default_rng(1).standard_normal((2, 256)), "bf16")
    y = torch.empty(2, 1000, dtype=torch.bfloat16, device="cuda")
    call = capi.KernelCall(inputs=[dev(x, "bf16"), wd], outputs=[y], attrs=dict(format="q4_0", activation=2))
    _lib.check(_lib.lib().qx_cuda_dispatch(b"decode_linear_epilogue", call.ref()))
    torch.cuda.synchronize()
    from tests._util import assert_close_dtype
    assert_close_dtype(host(y), O.decode_linear_epilogue(x, Wq, "q4_0", None, None, 2, "bf16"), "bf16")
    st = _lib.lib().qx_cuda_dispatch(b"attention", call.ref())
    assert _lib.STATUS_NAMES[st.code] == "not_implemented"


def test_lm_head_error_messages():
    h = torch.zeros(2, 64, device="cuda")
    w = torch.zeros(300, 2, 34, dtype=torch.uint8, device="cuda")
    with pytest.raises(ValueError, match="mode must be"):
        tk.lm_head_sample(h, w, mode="beam", format="q8_0")
    with pytest.raises(ValueError, match="quant format"):
        tk.lm_head_sample(h, w, format="q5_0")
    with pytest.raises(RuntimeError, match=r"k must be in \[1, 64\]"):
        tk.lm_head_sample(h, w, mode="topk", k=65, format="q8_0")
    with pytest.raises(RuntimeError, match="temperature must be positive"):
        tk.lm_head_sample(h, w, mode="categorical", temperature=0.0, format="q8_0")
    with pytest.raises(RuntimeError, match="top_p in"):
        tk.lm_head_sample(h, w, mode="topp", top_p=1.5, format="q8_0")
    with pytest.raises(RuntimeError, match="does not match"):
        tk.lm_head_sample(h, w[:, :, :33], format="q8_0")
    with pytest.raises(RuntimeError, match=r"h must be \(T, K\)"):
        tk.lm_head_sample(h, w[:, :1], format="q8_0")
