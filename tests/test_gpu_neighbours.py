"""GPU parity of the operators either side of the decode-projection path that share its packed
formats: qgemv / qgemm and the packed embedding lookup (dequant_gather, quantized_embedding).
The cases follow the reference's tests (tests/correctness/quantization/qgemv/test_qgemv.py:20-67,
qgemm/test_qgemm.py, dequant_gather/test_dequant_gather.py:31-77)."""
import numpy as np
import pytest
import torch

from oracle import qx_oracle as O
from tests._util import FMTS, assert_close_dtype, dev, host, rounded

pytestmark = pytest.mark.gpu

tk = pytest.importorskip("quixicore_metal_b200.tk")


@pytest.mark.parametrize("shape", [(128, 128), (67, 512), (300, 2048)])
@pytest.mark.parametrize("fmt", FMTS)
def test_qgemv(shape, fmt):
    N, K = shape
    if K % O.FORMATS[fmt][0] != 0:
        pytest.skip("K must be a multiple of the format's block width")
    rng = np.random.default_rng(0)
    Wq = O.synth_pack(fmt, (rng.standard_normal((N, K)) * 0.3).astype(np.float32))
    x = rounded(rng.standard_normal((K, 1)), "f16")
    got = tk.qgemv(dev(Wq), dev(x, "f16"), format=fmt)
    assert got.shape == (N, 1) and got.dtype == torch.float16
    ref = O.matmul_f64(x.T, O.dequantize(fmt, Wq)).T          # (N, 1), exact fp32 dequantisation
    g = host(got)
    assert np.abs(g - ref).max() / (np.abs(ref).max() + 1e-9) < 2e-2       # the reference's bar
    assert_close_dtype(g, O.round_to(ref, "f16"), "f16", scale=float(np.abs(ref).max()))   # this backend's


@pytest.mark.parametrize("fmt", ["q4_0", "q6_K", "nvfp4"])
def test_qgemv_float32_paths(fmt):
    N, K = 67, 512
    rng = np.random.default_rng(91)
    packed = O.synth_pack(fmt, (0.2 * rng.standard_normal((N, K))).astype(np.float32))
    x = (0.3 * rng.standard_normal((K, 1))).astype(np.float32)
    got = tk.qgemv(dev(packed), dev(x), format=fmt)
    assert got.dtype == torch.float32 and got.shape == (N, 1)
    np.testing.assert_allclose(host(got), O.matmul_f64(x.T, O.dequantize(fmt, packed)).T, rtol=3e-4, atol=3e-4)


@pytest.mark.parametrize("M", [1, 8, 32, 33, 96])
@pytest.mark.parametrize("fmt", ["q8_0", "q4_0", "q6_K", "mxfp4"])
def test_qgemm(fmt, M):
    N, K = 96, 512
    rng = np.random.default_rng(3 + M)
    Wq = O.synth_pack(fmt, (rng.standard_normal((N, K)) * 0.3).astype(np.float32))
    x = rounded(rng.standard_normal((K, M)), "f16")
    got = tk.qgemm(dev(Wq), dev(x, "f16"), format=fmt)
    assert got.shape == (N, M) and got.dtype == torch.float16
    ref = O.matmul_f64(x.T, O.dequantize(fmt, Wq)).T
    g = host(got)
    assert np.abs(g - ref).max() / (np.abs(ref).max() + 1e-9) < 2e-2
    assert_close_dtype(g, O.round_to(ref, "f16"), "f16", scale=float(np.abs(ref).max()))


@pytest.mark.parametrize("fmt,columns", [("q4_0", 96), ("q8_0", 96), ("q6_K", 512)])
def test_dequant_gather_valid_and_invalid_ids_bit_exact(fmt, columns):
    # test_dequant_gather.py:31-53: fp32 decode * scale, one rounding to fp16, zero rows for bad ids
    rng = np.random.default_rng(columns)
    rows = 7
    packed = O.synth_pack(fmt, (0.3 * rng.standard_normal((rows, columns))).astype(np.float32))
    ids = np.array([[3, -1], [6, rows]], dtype=np.int64)
    scale = np.float32(np.sqrt(1536.0))
    got = tk.dequant_gather(dev(packed), dev(ids), fmt, scale=float(scale))
    table = O.dequantize(fmt, packed)
    ref = np.zeros((*ids.shape, columns), dtype=np.float16)
    for index in np.ndindex(ids.shape):
        row = ids[index]
        if 0 <= row < rows:
            ref[index] = (table[row] * scale).astype(np.float16)
    assert got.shape == ref.shape and got.dtype == torch.float16
    np.testing.assert_array_equal(got.cpu().numpy(), ref)


@pytest.mark.parametrize("out_dtype", ["float32", "bfloat16", "float16"])
@pytest.mark.parametrize("fmt", FMTS)
def test_quantized_embedding_formats_add_and_invalid_ids(fmt, out_dtype):
    # test_dequant_gather.py:56-77
    bk = O.FORMATS[fmt][0]
    rng = np.random.default_rng(100 + bk + len(fmt))
    rows, columns = 5, 2 * bk if bk >= 32 else 48          # nvfp4: a width of 16 mod 32
    packed = O.synth_pack(fmt, (0.25 * rng.standard_normal((rows, columns))).astype(np.float32))
    ids = np.array([[3, -1], [1, rows]], dtype=np.int32)
    short = {"float32": "f32", "bfloat16": "bf16", "float16": "f16"}[out_dtype]
    add = rounded(0.03 * rng.standard_normal((*ids.shape, columns)), short)
    scale = np.float32(1.375)
    got = tk.quantized_embedding_lookup(dev(packed), dev(ids), fmt, scale=float(scale), add=dev(add, short),
                                        output_dtype=out_dtype)
    table = O.dequantize(fmt, packed).astype(np.float32)
    ref = np.zeros((*ids.shape, columns), dtype=np.float32)
    for index in np.ndindex(ids.shape):
        row = ids[index]
        if 0 <= row < rows:
            ref[index] = (table[row] * scale).astype(np.float32) + add[index]
    assert tuple(got.shape) == ref.shape
    np.testing.assert_array_equal(host(got), O.round_to(ref, short))       # one rounding, bit-exact


def test_error_messages():
    w = torch.zeros(64, 2, 34, dtype=torch.uint8, device="cuda")
    with pytest.raises(RuntimeError, match=r"x \(K,1\)"):
        tk.qgemv(w, torch.zeros(64, 2, dtype=torch.float16, device="cuda"))
    with pytest.raises(RuntimeError, match="x rows == K"):
        tk.qgemm(w, torch.zeros(32, 4, dtype=torch.float16, device="cuda"))
    with pytest.raises(RuntimeError, match="format must be q4_0, q8_0, or q6_K"):
        tk.dequant_gather(w, torch.zeros(2, dtype=torch.int32, device="cuda"), "mxfp8")
    with pytest.raises(ValueError, match="output_dtype"):
        tk.quantized_embedding_lookup(w, torch.zeros(2, dtype=torch.int32, device="cuda"), "q8_0", output_dtype="int8")
