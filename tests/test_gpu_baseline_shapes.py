"""Parity at the full sizes the benchmark configurations name (not reduced stand-ins):

  1. decode_linear_epilogue q4_0, 4096 x 4096, one row, bias, bf16
  2. decode_swiglu + down projection, q6_K, hidden 4096 / intermediate 14336, 1 / 4 / 8 rows
  3. decode_linear_epilogue nvfp4 and mxfp4, K 8192 -> N 28672, 1 / 16 / 64 / 256 rows, output
     requantised to MXFP8 rows inside the call
  4. lm_head_sample q8_0, 128256-token vocabulary, hidden 4096, 1 / 8 / 64 rows, argmax / top-k 50 /
     top-p 0.9 (pool 32) at temperature 0.8

Weights are seeded N(0, 0.02) packed by the oracle's round-to-nearest packers, activations seeded
N(0, 1) rounded to bf16.  Outputs are compared with the CPU oracle (float64 dot of the exactly
dequantised weights); for the large batches the oracle is evaluated on a sample of the rows, the
requantised codes are checked on every row.  Token ids must be identical wherever the oracle's
decision margin exceeds fp32 accumulation noise."""
import numpy as np
import pytest
import torch

from oracle import qx_oracle as O
from tests._util import assert_close_dtype, check_ids, dev, host, rounded

pytestmark = pytest.mark.gpu

tk = pytest.importorskip("quixicore_metal_b200.tk")
EPS = 2e-5


def _gauss_pack(fmt, N, K, seed, rows_per_chunk=4096):
    rng = np.random.default_rng(seed)
    parts = []
    for r0 in range(0, N, rows_per_chunk):
        n = min(rows_per_chunk, N - r0)
        parts.append(O.synth_pack(fmt, (0.02 * rng.standard_normal((n, K))).astype(np.float32)))
    return np.concatenate(parts)


# ---- configuration 1 ----------------------------------------------------------------------------
def test_config1_q4_0_4096_square_with_bias():
    rng = np.random.default_rng(101)
    K = N = 4096
    Wq = _gauss_pack("q4_0", N, K, 1)
    x = rounded(rng.standard_normal((1, K)), "bf16")
    bias = rounded(0.01 * rng.standard_normal(N), "bf16")
    got = tk.decode_linear_epilogue(dev(x, "bf16"), dev(Wq), dev(bias, "bf16"), format="q4_0")
    assert_close_dtype(host(got), O.decode_linear_epilogue(x, Wq, "q4_0", bias, None, 0, "bf16"), "bf16")


# ---- configuration 2 ----------------------------------------------------------------------------
@pytest.fixture(scope="module")
def mlp_q6k():
    H, I = 4096, 14336
    return (_gauss_pack("q6_K", I, H, 2), _gauss_pack("q6_K", I, H, 3), _gauss_pack("q6_K", H, I, 4))


@pytest.mark.parametrize("M", [1, 4, 8])
def test_config2_q6k_swiglu_mlp(mlp_q6k, M):
    gate, up, down = mlp_q6k
    rng = np.random.default_rng(200 + M)
    x = rounded(rng.standard_normal((M, 4096)), "bf16")
    res = rounded(rng.standard_normal((M, 4096)), "bf16")
    gd, ud, dd = dev(gate), dev(up), dev(down)
    mid = tk.decode_swiglu(dev(x, "bf16"), gd, ud, format="q6_K")
    ref_mid = O.decode_swiglu(x, gate, up, "q6_K", None, None, "bf16")
    assert_close_dtype(host(mid), ref_mid, "bf16")
    # the down projection is checked on the GPU's own intermediate (one rounding apart from the
    # oracle's is a different input, not an error of the projection)
    mid_np = host(mid)
    out = tk.decode_linear_epilogue(mid, dd, None, dev(res, "bf16"), format="q6_K")
    assert_close_dtype(host(out), O.decode_linear_epilogue(mid_np, down, "q6_K", None, res, 0, "bf16"), "bf16")


# ---- configuration 3 ----------------------------------------------------------------------------
@pytest.fixture(scope="module", params=["nvfp4", "mxfp4"])
def wide_projection(request):
    fmt = request.param
    K, N = 8192, 28672
    Wq = _gauss_pack(fmt, N, K, 30 + len(fmt))
    return fmt, Wq, dev(Wq), O.dequantize(fmt, Wq).astype(np.float64)


@pytest.mark.parametrize("M", [1, 16, 64, 256])
def test_config3_fp4_sweep_with_mxfp8_output(wide_projection, M):
    fmt, Wq, wd, W64 = wide_projection
    K, N = 8192, 28672
    rng = np.random.default_rng(300 + M)
    x = rounded(rng.standard_normal((M, K)), "bf16")
    xd = dev(x, "bf16")
    from quixicore_metal_b200 import tk_torch
    # the bf16 output and the MXFP8 rows made from it, from ONE call (a second call may split the
    # work differently and round a few outputs the other way)
    y, blocks = tk_torch.decode_linear_epilogue(xd, wd, xd, xd, fmt, 0, False, False, output_quant="mxfp8",
                                                with_output=True)
    assert blocks.shape == (M, N // 32, 33) and blocks.dtype == torch.uint8
    y_np = host(y)
    # bf16 output against the oracle on a sample of the rows (every row when there are few)
    rows = np.unique(np.concatenate([np.arange(min(M, 8)), np.arange(max(M - 8, 0), M)]))
    ref = O.round_to((x[rows].astype(np.float64) @ W64.T).astype(np.float32), "bf16")
    assert_close_dtype(y_np[rows], ref, "bf16")
    # requantised codes: bit-exact given the GPU's own rounded output, on every row
    np.testing.assert_array_equal(host(blocks), O.quantize_mxfp8_rows(y_np))


# ---- configuration 4 ----------------------------------------------------------------------------
@pytest.fixture(scope="module")
def llama_head():
    V, K = 128256, 4096
    Wq = _gauss_pack("q8_0", V, K, 40, rows_per_chunk=16384)
    rng = np.random.default_rng(41)
    h = rounded(rng.standard_normal((64, K)), "bf16")
    return Wq, dev(Wq), h, O.lm_head_logits(h, Wq, "q8_0")


@pytest.mark.parametrize("mode,k", [("argmax", 0), ("topk", 50), ("topp", 32)])
@pytest.mark.parametrize("T", [1, 8, 64])
def test_config4_lm_head_128k_vocabulary(llama_head, T, mode, k):
    Wq, wd, h, logits = llama_head
    m = {"argmax": 0, "topk": 2, "topp": 3}[mode]
    tok = host(tk.lm_head_sample(dev(h[:T], "bf16"), wd, mode=mode, k=k, temperature=0.8, seed=1234,
                                 format="q8_0", top_p=0.9))
    want, margin = O.lm_head_sample_from_logits(logits[:T], m, k=k, temperature=0.8, seed=1234, top_p=0.9,
                                                return_detail=True)
    exact = check_ids(tok, want, margin, EPS, f"q8_0/{mode}/T{T}")
    assert exact >= T - 1, (exact, T)          # near-ties are rare: at most one row may be one
    assert int(tok.min()) >= 0 and int(tok.max()) < 128256


def test_config4_vocabulary_shards_give_the_single_device_ids(llama_head):
    """The 8-way split of the 128256-row head (63 / 62 tiles per shard), shards run one after the
    other on this GPU and merged by stage 2: the ids of the unsharded call."""
    from quixicore_metal_b200 import parallel
    Wq, wd, h, logits = llama_head
    V, shards, T = 128256, 8, 64
    hd = dev(h[:T], "bf16")
    bounds = parallel.vocab_shard_bounds(V, shards)
    mt = parallel.max_shard_tiles(V, shards)
    for mode, k in (("argmax", 0), ("topk", 50), ("topp", 32)):
        kw = dict(k=k, temperature=0.8, seed=77)
        single = host(tk.lm_head_sample(hd, wd, mode=mode, format="q8_0", top_p=0.9, **kw))
        parts = [parallel.lm_head_shard_partials(hd, wd[a:b], None, a, mt, "q8_0", mode, **kw) for a, b in bounds]
        merged = host(parallel.lm_head_merge(parts, mode, top_p=0.9, max_tiles=mt, **kw))
        # identical except where the decision itself is an fp32 near-tie (a shard and the whole
        # head may add the K slices of a tile in a different order)
        m = {"argmax": 0, "topk": 2, "topp": 3}[mode]
        _, margin = O.lm_head_sample_from_logits(logits[:T], m, k=k, temperature=0.8, seed=77, top_p=0.9,
                                                 return_detail=True)
        check_ids(merged, single, margin, EPS, f"sharded/{mode}")
