"""GPU parity of decode_linear_epilogue / decode_swiglu / output quantizers against the CPU oracle.
Every call goes through the C ABI (via the tk_torch-compatible binding)."""
import os

import numpy as np
import pytest
import torch

from oracle import qx_oracle as O
from tests._util import FMTS, assert_close_dtype, dev, host, rounded

pytestmark = pytest.mark.gpu

tk = pytest.importorskip("quixicore_metal_b200.tk")
ACT = {"none": 0, "gelu": 1, "silu": 2}


def _inputs(fmt, M, K, N, dtype, seed, xs=1.0, ws=0.02, random_bytes=False):
    rng = np.random.default_rng(seed)
    x = rounded(xs * rng.standard_normal((M, K)), dtype)
    if random_bytes:
        Wq = O.random_packed(fmt, N, K, seed + 1)
    else:
        Wq = O.synth_pack(fmt, (ws * rng.standard_normal((N, K))).astype(np.float32))
    bias = rounded(0.01 * rng.standard_normal(N), dtype)
    res = rounded(rng.standard_normal((M, N)), dtype)
    return x, Wq, bias, res


@pytest.mark.parametrize("dtype", ["f32", "bf16", "f16"])
@pytest.mark.parametrize("activation", ["none", "gelu", "silu"])
@pytest.mark.parametrize("fmt", FMTS)
def test_epilogue_reference_test_shape(fmt, activation, dtype):
    # shape and scales of tests/correctness/matmul/decode_linear/test_decode_linear.py:155-171
    rng = np.random.default_rng(131 + len(fmt) + len(activation))
    B, K, N = 2, 512, 35
    x = rounded(0.08 * rng.standard_normal((B, K)), dtype)
    Wq = O.synth_pack(fmt, (0.1 * rng.standard_normal((N, K))).astype(np.float32))
    bias = rounded(0.02 * rng.standard_normal(N), dtype)
    res = rounded(0.03 * rng.standard_normal((B, N)), dtype)
    got = tk.decode_linear_epilogue(dev(x, dtype), dev(Wq), dev(bias, dtype), dev(res, dtype),
                                    activation=activation, format=fmt)
    ref = O.decode_linear_epilogue(x, Wq, fmt, bias, res, ACT[activation], dtype)
    assert got.shape == (B, N) and got.dtype == dev(x, dtype).dtype
    assert_close_dtype(host(got), ref, dtype, scale=0.1)
    # the reference's own tolerance
    np.testing.assert_allclose(host(got), ref, rtol=7e-4 if dtype == "f32" else 4e-2,
                               atol=7e-4 if dtype == "f32" else 4e-2)


@pytest.mark.parametrize("fmt", FMTS)
def test_epilogue_golden_fixture_from_reference(fmt, golden_dir):
    """Inputs packed by the reference's quantizers, outputs of the reference's torch-CPU path."""
    C = np.load(os.path.join(golden_dir, "compose.npz"))
    x, bias, bias2, res = C[f"{fmt}_x"], C[f"{fmt}_bias"], C[f"{fmt}_bias2"], C[f"{fmt}_res"]
    for act in ("none", "silu"):
        got = tk.decode_linear_epilogue(dev(x, "bf16"), dev(C[f"{fmt}_gate"]), dev(bias, "bf16"),
                                        dev(res, "bf16"), activation=act, format=fmt)
        assert_close_dtype(host(got), C[f"{fmt}_lin_{act}"], "bf16")
    got = tk.decode_swiglu(dev(x, "bf16"), dev(C[f"{fmt}_gate"]), dev(C[f"{fmt}_up"]),
                           dev(bias, "bf16"), dev(bias2, "bf16"), format=fmt)
    assert_close_dtype(host(got), C[f"{fmt}_swiglu"], "bf16")


@pytest.mark.parametrize("fmt", FMTS)
def test_epilogue_every_code_value(fmt):
    """Random bytes: all 256 code values of every field, including e4m3 exponent-15 codes."""
    x, Wq, bias, res = _inputs(fmt, 3, 512, 48, "f32", 7, random_bytes=True)
    got = tk.decode_linear_epilogue(dev(x), dev(Wq), dev(bias), dev(res), format=fmt)
    ref = O.decode_linear_epilogue(x, Wq, fmt, bias, res, 0, "f32")
    scale = float(np.abs(O.dequantize(fmt, Wq)).max()) * 30
    assert_close_dtype(host(got), ref, "f32", scale=scale)


@pytest.mark.parametrize("M", [1, 2, 3, 4, 5, 8, 9, 16, 17])
@pytest.mark.parametrize("fmt", FMTS)
def test_epilogue_batch_sweep_bf16(fmt, M):
    K = 1024 if fmt != "q6_K" else 2048
    x, Wq, bias, res = _inputs(fmt, M, K, 130, "bf16", 11 + M)
    got = tk.decode_linear_epilogue(dev(x, "bf16"), dev(Wq), dev(bias, "bf16"), dev(res, "bf16"),
                                    activation="silu", format=fmt)
    ref = O.decode_linear_epilogue(x, Wq, fmt, bias, res, 2, "bf16")
    assert_close_dtype(host(got), ref, "bf16")


@pytest.mark.parametrize("M", [1, 6, 16])
@pytest.mark.parametrize("K,N", [(768, 16), (768, 2400), (1280, 2373), (2048, 4750)])
@pytest.mark.parametrize("fmt", ["nvfp4", "q8_0", "mxfp4", "q6_K"])
def test_streaming_work_split_shapes(fmt, K, N, M):
    """Shapes that stress the streaming kernel's work split: a single 16-row tile, 150 tiles on 148
    CTAs (shares of one and two tiles, every tile cut between warps), a ragged last tile, a K whose
    last stage is partial (the loop that is not unrolled), for one matrix and for a SwiGLU pair."""
    if fmt == "q6_K" and K != 2048:
        pytest.skip("q6_K rows are 16-byte aligned only for K % 2048 == 0")
    x, Wq, bias, res = _inputs(fmt, M, K, N, "bf16", 5 + M + N)
    got = tk.decode_linear_epilogue(dev(x, "bf16"), dev(Wq), dev(bias, "bf16"), dev(res, "bf16"), format=fmt)
    assert_close_dtype(host(got), O.decode_linear_epilogue(x, Wq, fmt, bias, res, 0, "bf16"), "bf16")
    _, Uq, ub, _ = _inputs(fmt, M, K, N, "bf16", 6 + M + N)
    got = tk.decode_swiglu(dev(x, "bf16"), dev(Wq), dev(Uq), dev(bias, "bf16"), dev(ub, "bf16"), format=fmt)
    assert_close_dtype(host(got), O.decode_swiglu(x, Wq, Uq, fmt, bias, ub, "bf16"), "bf16")


@pytest.mark.parametrize("fmt,K", [("q4_0", 32), ("q4_0", 96), ("q8_0", 160), ("q6_K", 256),
                                   ("mxfp8", 32), ("nvfp4", 16), ("nvfp4", 48), ("nvfp4", 272),
                                   ("mxfp4", 224)])
@pytest.mark.parametrize("N", [1, 7, 33])
def test_epilogue_ragged_shapes(fmt, K, N):
    """Smallest legal K, K that is not a multiple of any load width, N = 1."""
    x, Wq, bias, res = _inputs(fmt, 2, K, N, "bf16", 3 + K + N)
    got = tk.decode_linear_epilogue(dev(x, "bf16"), dev(Wq), None, dev(res, "bf16"), format=fmt)
    ref = O.decode_linear_epilogue(x, Wq, fmt, None, res, 0, "bf16")
    assert_close_dtype(host(got), ref, "bf16")
    got = tk.decode_linear_epilogue(dev(x, "bf16"), dev(Wq), dev(bias, "bf16"), None, format=fmt)
    assert_close_dtype(host(got), O.decode_linear_epilogue(x, Wq, fmt, bias, None, 0, "bf16"), "bf16")


@pytest.mark.parametrize("dtype", ["f32", "bf16"])
@pytest.mark.parametrize("fmt", FMTS)
def test_swiglu_reference_test_shape(fmt, dtype):
    # tests/correctness/matmul/decode_linear/test_decode_linear.py:174-201
    rng = np.random.default_rng(151 + len(fmt))
    B, K, N = 2, 512, 33
    x = rounded(0.07 * rng.standard_normal((B, K)), dtype)
    g = O.synth_pack(fmt, (0.09 * rng.standard_normal((N, K))).astype(np.float32))
    u = O.synth_pack(fmt, (0.08 * rng.standard_normal((N, K))).astype(np.float32))
    gb = rounded(0.02 * rng.standard_normal(N), dtype)
    ub = rounded(0.02 * rng.standard_normal(N), dtype)
    got = tk.decode_swiglu(dev(x, dtype), dev(g), dev(u), dev(gb, dtype), dev(ub, dtype), format=fmt)
    ref = O.decode_swiglu(x, g, u, fmt, gb, ub, dtype)
    assert_close_dtype(host(got), ref, dtype, scale=0.01)
    got = tk.decode_swiglu(dev(x, dtype), dev(g), dev(u), format=fmt)
    assert_close_dtype(host(got), O.decode_swiglu(x, g, u, fmt, None, None, dtype), dtype, scale=0.01)


@pytest.mark.parametrize("M", [1, 4, 8])
def test_swiglu_mlp_config_shapes_q6k(M):
    """Llama-3-8B MLP row shapes (hidden 4096) on a slice of the intermediate dimension, then
    the down projection with residual: the two-launch composition of the reference."""
    rng = np.random.default_rng(40 + M)
    K, I = 4096, 512
    x = rounded(rng.standard_normal((M, K)), "bf16")
    g = O.synth_pack("q6_K", (0.02 * rng.standard_normal((I, K))).astype(np.float32))
    u = O.synth_pack("q6_K", (0.02 * rng.standard_normal((I, K))).astype(np.float32))
    d = O.synth_pack("q6_K", (0.02 * rng.standard_normal((256, I))).astype(np.float32))
    res = rounded(rng.standard_normal((M, 256)), "bf16")
    mid = tk.decode_swiglu(dev(x, "bf16"), dev(g), dev(u), format="q6_K")
    mid_ref = O.decode_swiglu(x, g, u, "q6_K", None, None, "bf16")
    assert_close_dtype(host(mid), mid_ref, "bf16")
    out = tk.decode_linear_epilogue(mid, dev(d), None, dev(res, "bf16"), format="q6_K")
    ref = O.decode_linear_epilogue(host(mid), d, "q6_K", None, res, 0, "bf16")
    assert_close_dtype(host(out), ref, "bf16")


# ---- output quantizers: codes are bit-exact given the identical pre-quant values --------------
@pytest.mark.parametrize("kind", ["fp8", "int8"])
@pytest.mark.parametrize("dtype", ["f32", "bf16"])
def test_per_token_quantizer_bit_exact(kind, dtype):
    rng = np.random.default_rng(5)
    y = rounded(rng.standard_normal((7, 333)) * np.array([[1e-3], [1], [50], [0], [3], [1e4], [2e-6]]), dtype)
    fn = tk.quantize_per_token_fp8 if kind == "fp8" else tk.quantize_per_token_int8
    codes, scale = fn(dev(y, dtype))
    rc, rs = O.quantize_per_token(y, kind)
    np.testing.assert_array_equal(host(scale).view(np.uint32), rs.view(np.uint32))
    np.testing.assert_array_equal(host(codes).view(np.uint8), rc.view(np.uint8))


def test_e4m3_midpoints_round_away_from_zero():
    """Exact half-way inputs (common for bf16 values under a power-of-two scale)."""
    dec = O.e4m3_decode(np.arange(256))
    pos = np.arange(0, 0x7E)
    mid = ((dec[pos].astype(np.float64) + dec[pos + 1]) / 2).astype(np.float32)
    row = np.concatenate([mid, -mid, [448.0, -448.0]]).astype(np.float32)[None, :]   # amax 448 -> scale 1
    codes, scale = tk.quantize_per_token_fp8(dev(row))
    assert float(scale[0]) == 1.0
    want = np.concatenate([pos + 1, (pos + 1) | 0x80, [0x7E, 0xFE]]).astype(np.uint8)
    np.testing.assert_array_equal(host(codes)[0], want)


@pytest.mark.parametrize("dtype", ["f32", "bf16"])
def test_mxfp8_rows_bit_exact(dtype):
    rng = np.random.default_rng(9)
    y = rounded(rng.standard_normal((5, 256)) * np.array([[1e-4], [1], [300], [0], [7]]), dtype)
    y[1, 32:64] = 0
    y[2, :32] = rounded(np.full(32, 448.0), dtype)
    from quixicore_metal_b200 import tk_torch
    blocks = tk_torch.quantize_mxfp8_rows(dev(y, dtype))
    np.testing.assert_array_equal(host(blocks), O.quantize_mxfp8_rows(y))


def test_epilogue_output_quant_composition():
    """decode_linear_epilogue(..., output_quant=...) = quantizer applied to the rounded output."""
    x, Wq, bias, res = _inputs("nvfp4", 4, 1024, 256, "bf16", 21)
    y = tk.decode_linear_epilogue(dev(x, "bf16"), dev(Wq), dev(bias, "bf16"), None, format="nvfp4")
    for oq in ("fp8", "int8"):
        codes, scale = tk.decode_linear_epilogue(dev(x, "bf16"), dev(Wq), dev(bias, "bf16"), None,
                                                 format="nvfp4", output_quant=oq)
        rc, rs = O.quantize_per_token(host(y), oq)          # same kernel, same split: same rounded output
        np.testing.assert_array_equal(host(codes).view(np.uint8), rc.view(np.uint8))
        np.testing.assert_array_equal(host(scale), rs)
    from quixicore_metal_b200 import tk_torch
    blocks = tk.decode_linear_epilogue(dev(x, "bf16"), dev(Wq), dev(bias, "bf16"), None,
                                       format="nvfp4", output_quant="mxfp8")
    assert blocks.shape == (4, 256 // 32, 33)
    # fused MXFP8 rows against the output of the same call, for the streaming kernel (4 and 16 rows),
    # 16-row passes / the tcgen05 pipeline (40 rows), SwiGLU, and the second-launch fallback (fp32)
    for M, dtype in ((4, "bf16"), (16, "bf16"), (40, "bf16"), (40, "f16"), (3, "f32")):
        xm, Wm, bm, rm = _inputs("nvfp4", M, 1024, 256, dtype, 300 + M)
        ym, bl = tk_torch.decode_linear_epilogue(dev(xm, dtype), dev(Wm), dev(bm, dtype), dev(rm, dtype), "nvfp4",
                                                 2, True, True, output_quant="mxfp8", with_output=True)
        assert_close_dtype(host(ym), O.decode_linear_epilogue(xm, Wm, "nvfp4", bm, rm, 2, dtype), dtype)
        np.testing.assert_array_equal(host(bl), O.quantize_mxfp8_rows(host(ym)))
        _, Um, ubm, _ = _inputs("nvfp4", M, 1024, 256, dtype, 400 + M)
        gm, bl = tk_torch.decode_swiglu(dev(xm, dtype), dev(Wm), dev(Um), dev(bm, dtype), dev(ubm, dtype), "nvfp4",
                                        True, output_quant="mxfp8", with_output=True)
        np.testing.assert_array_equal(host(bl), O.quantize_mxfp8_rows(host(gm)))
        for oq in ("fp8", "int8"):
            ym, (cq, sq) = tk_torch.decode_linear_epilogue(dev(xm, dtype), dev(Wm), dev(bm, dtype), dev(rm, dtype),
                                                           "nvfp4", 0, True, False, output_quant=oq, with_output=True)
            rc, rs = O.quantize_per_token(host(ym), oq)
            np.testing.assert_array_equal(host(cq).view(np.uint8), rc.view(np.uint8))
            np.testing.assert_array_equal(host(sq), rs)
    # int8 reconstruction bound of test_decode_linear.py:204-215
    codes, scale = tk.decode_linear_epilogue(dev(x, "bf16"), dev(Wq), None, None, format="nvfp4",
                                             activation="silu", output_quant="int8")
    dense = tk.decode_linear_epilogue(dev(x, "bf16"), dev(Wq), None, None, format="nvfp4", activation="silu")
    err = np.max(np.abs(host(codes).astype(np.float32) * host(scale)[:, None] - host(dense)))
    assert err <= float(host(scale).max()) * 0.51 + 1e-6


def test_error_behaviour_matches_reference_messages():
    x = torch.zeros(2, 64, device="cuda")
    w = torch.zeros(3, 2, 18, dtype=torch.uint8, device="cuda")
    with pytest.raises(RuntimeError, match="packed weight must be uint8"):
        tk.decode_linear_epilogue(x, w[:, :1], format="q4_0")
    with pytest.raises(RuntimeError, match="format must be"):
        tk.decode_linear_epilogue(x, w, format="q5_1")
    with pytest.raises(ValueError, match="activation must be"):
        tk.decode_linear_epilogue(x, w, format="q4_0", activation="relu")
    with pytest.raises(RuntimeError, match="bias must be"):
        tk.decode_linear_epilogue(x, w, bias=torch.zeros(4, device="cuda"), format="q4_0")
    with pytest.raises(ValueError, match="both be present"):
        tk.decode_swiglu(x, w, w, gate_bias=torch.zeros(3, device="cuda"), format="q4_0")
    with pytest.raises(ValueError, match="output_quant"):
        tk.decode_linear_epilogue(x, w, format="q4_0", output_quant="fp4")
    # placeholders are ignored when the flag is off (the router passes x itself)
    from quixicore_metal_b200 import tk_torch
    y = tk_torch.decode_linear_epilogue(x, w, x, x, "q4_0", 0, False, False)
    assert y.shape == (2, 3) and float(y.abs().max()) == 0.0


@pytest.fixture(params=["tcgen05", "passes"])
def large_batch_path(request):
    """Batches of 17 - 64 rows have two device paths: the tcgen05 kernels, and the streaming kernel
    run in passes of 16 rows (chosen by default when the projection has few 256-row items).  The
    library option "stream_passes" picks one: 0 = never, 2 = whenever the shape allows."""
    from quixicore_metal_b200 import _lib
    _lib.set_option("stream_passes", 0 if request.param == "tcgen05" else 2)
    yield request.param
    _lib.set_option("stream_passes", 1)


@pytest.mark.parametrize("M", [17, 32, 64, 100, 128, 129, 256])
@pytest.mark.parametrize("fmt", FMTS)
def test_epilogue_large_batch(fmt, M, large_batch_path):
    """Batch > 16 (the tcgen05 path for bf16): several 128-row weight tiles incl. a ragged last one,
    batches that need a second pass (M > 128), every epilogue piece."""
    if large_batch_path == "passes" and M > 64 and fmt != "q6_K":
        pytest.skip("passes serve at most 64 rows (256 for q6_K)")
    K, N = 1024, 300
    x, Wq, bias, res = _inputs(fmt, M, K, N, "bf16", 90 + M)
    got = tk.decode_linear_epilogue(dev(x, "bf16"), dev(Wq), dev(bias, "bf16"), dev(res, "bf16"),
                                    activation="gelu", format=fmt)
    ref = O.decode_linear_epilogue(x, Wq, fmt, bias, res, 1, "bf16")
    assert_close_dtype(host(got), ref, "bf16")


@pytest.mark.parametrize("fmt", ["q8_0", "q4_0", "mxfp8", "nvfp4", "mxfp4"])
def test_large_batch_f16(fmt, large_batch_path):
    """f16 activations at batch > 16: linear with every epilogue piece, and SwiGLU."""
    M, K, N = 40, 512, 384
    x, Wq, bias, res = _inputs(fmt, M, K, N, "f16", 70)
    got = tk.decode_linear_epilogue(dev(x, "f16"), dev(Wq), dev(bias, "f16"), dev(res, "f16"),
                                    activation="silu", format=fmt)
    assert_close_dtype(host(got), O.decode_linear_epilogue(x, Wq, fmt, bias, res, 2, "f16"), "f16")
    _, Uq, ub, _ = _inputs(fmt, M, K, N, "f16", 71)
    got = tk.decode_swiglu(dev(x, "f16"), dev(Wq), dev(Uq), dev(bias, "f16"), dev(ub, "f16"), format=fmt)
    assert_close_dtype(host(got), O.decode_swiglu(x, Wq, Uq, fmt, bias, ub, "f16"), "f16")


@pytest.mark.parametrize("fmt", ["nvfp4", "q8_0"])
def test_epilogue_large_batch_every_code_value(fmt, large_batch_path):
    x, Wq, bias, res = _inputs(fmt, 48, 512, 256, "bf16", 17, random_bytes=True)
    got = tk.decode_linear_epilogue(dev(x, "bf16"), dev(Wq), None, None, format=fmt)
    ref = O.decode_linear_epilogue(x, Wq, fmt, None, None, 0, "bf16")
    assert_close_dtype(host(got), ref, "bf16", scale=float(np.abs(ref).max()))


@pytest.mark.parametrize("M", [24, 130])
@pytest.mark.parametrize("fmt", ["nvfp4", "q6_K", "q8_0"])
def test_swiglu_large_batch(fmt, M, large_batch_path):
    if large_batch_path == "passes" and M > 64 and fmt != "q6_K":
        pytest.skip("passes serve at most 64 rows (256 for q6_K)")
    rng = np.random.default_rng(7 + M)
    K, N = 1024, 200
    x = rounded(rng.standard_normal((M, K)), "bf16")
    g = O.synth_pack(fmt, (0.02 * rng.standard_normal((N, K))).astype(np.float32))
    u = O.synth_pack(fmt, (0.02 * rng.standard_normal((N, K))).astype(np.float32))
    gb = rounded(0.02 * rng.standard_normal(N), "bf16")
    ub = rounded(0.02 * rng.standard_normal(N), "bf16")
    got = tk.decode_swiglu(dev(x, "bf16"), dev(g), dev(u), dev(gb, "bf16"), dev(ub, "bf16"), format=fmt)
    assert_close_dtype(host(got), O.decode_swiglu(x, g, u, fmt, gb, ub, "bf16"), "bf16")


@pytest.mark.parametrize("M", [1, 8, 32])
@pytest.mark.parametrize("fmt", ["nvfp4", "q4_0"])
def test_row_parallel_partials_sum_to_full_projection(fmt, M, large_batch_path):
    """K split over 4 'ranks' at block boundaries: fp32 partials summed = the unsplit projection."""
    from quixicore_metal_b200 import tk_torch
    rng = np.random.default_rng(3 + M)
    K, N, R = 4096, 160, 4
    x = rounded(rng.standard_normal((M, K)), "bf16")
    Wq = O.synth_pack(fmt, (0.02 * rng.standard_normal((N, K))).astype(np.float32))
    bk = O.FORMATS[fmt][0]
    nb = K // bk // R
    total = None
    for r in range(R):
        part = tk_torch.decode_linear_partial(dev(x[:, r * K // R:(r + 1) * K // R], "bf16").contiguous(),
                                              dev(np.ascontiguousarray(Wq[:, r * nb:(r + 1) * nb])), fmt)
        assert part.dtype == torch.float32
        total = part if total is None else total + part
    ref = O.matmul_f64(x, O.dequantize(fmt, Wq))
    np.testing.assert_allclose(host(total), ref, rtol=2e-5, atol=2e-5)


def test_large_batch_weight_ending_at_an_allocation_boundary(large_batch_path):
    """A packed tensor of exactly 9 x 2 MiB fills its allocator segment to the last byte: no load
    of the batch > 16 path may touch anything beyond the tensor."""
    fmt, M, K, N = "nvfp4", 32, 8192, 4096
    Wq = O.random_packed(fmt, N, K, 3)
    assert Wq.nbytes % (2 << 20) == 0
    rng = np.random.default_rng(1)
    x = rounded(rng.standard_normal((M, K)), "bf16")
    torch.cuda.empty_cache()
    wd = dev(Wq)
    got = host(tk.decode_linear_epilogue(dev(x, "bf16"), wd, None, None, format=fmt))
    rows = np.r_[0:8, N - 136:N]                      # first rows and the whole last tile
    ref = O.decode_linear_epilogue(x, Wq[rows], fmt, None, None, 0, "bf16")
    assert_close_dtype(got[:, rows], ref, "bf16", scale=float(np.abs(ref).max()))


def test_wide_dynamic_range_activations():
    """The batch <= 16 path converts activations to row-scaled f16 (row maximum near 2^14).
    Elements more than 2^28 below the row maximum lose bits there, so the guarantee has two terms:
    fp32 accumulation noise relative to sum |x||w|, plus 2^-26 * max|x_row| * sum |w| for the
    elements that fall below f16 resolution."""
    fmt, M, K, N = "q8_0", 4, 1024, 64
    rng = np.random.default_rng(2)
    x = rng.standard_normal((M, K)).astype(np.float32)
    x[0, ::7] *= 1e-12           # far below the row maximum
    x[1, 5] = 3.0e30             # one huge element
    x[2, :] *= 1e-30             # a uniformly tiny row
    x[3, ::3] = 0.0
    x = rounded(x, "bf16")
    Wq = O.synth_pack(fmt, (0.02 * rng.standard_normal((N, K))).astype(np.float32))
    got = host(tk_torch_partial(x, Wq, fmt))
    ref = (x.astype(np.float64) @ O.dequantize(fmt, Wq).astype(np.float64).T)
    Wabs = np.abs(O.dequantize(fmt, Wq)).astype(np.float64)
    scale = np.abs(x).astype(np.float64) @ Wabs.T
    floor = np.abs(x).max(axis=1, keepdims=True).astype(np.float64) * Wabs.sum(axis=1)[None, :] * 2.0 ** -26
    assert np.all(np.abs(got - ref) <= 4e-6 * scale + floor + 1e-37)


def tk_torch_partial(x, Wq, fmt):
    from quixicore_metal_b200 import tk_torch
    return tk_torch.decode_linear_partial(dev(x, "bf16"), dev(Wq), fmt)
