"""GPU parity of the norm / activation -> quantiser seams against the CPU oracle.  A transcendental
(rsqrt, exp) sits between the inputs and the codes, so - as in the reference's own tests
(tests/correctness/norms/add_norm/test_add_norm.py:120-158, :286-310,
tests/correctness/quantization/act_quant/test_act_quant.py:29-78) - codes are checked by
reconstruction bounds, and against the oracle's codes with a small allowance for borderline
values; scales and the unquantised outputs are checked tightly."""
import numpy as np
import pytest
import torch

from oracle import qx_oracle as O
from tests._util import dev, host, rounded

pytestmark = pytest.mark.gpu

tk = pytest.importorskip("quixicore_metal_b200.tk")
DEC = O.e4m3_decode(np.arange(256))


def _norm_inputs(shape, dtype, seed):
    rng = np.random.default_rng(seed)
    D = shape[-1]
    return (rounded(rng.standard_normal(shape), dtype), rounded(rng.standard_normal(shape), dtype),
            rounded(rng.standard_normal(D), dtype))


def _codes_agree(got, want, frac=0.995):
    got = np.asarray(got).astype(np.int32) & 0xFF
    want = np.asarray(want).astype(np.int32) & 0xFF
    assert (got == want).mean() >= frac, float((got == want).mean())


@pytest.mark.parametrize("dtype", ["bf16", "f16", "f32"])
@pytest.mark.parametrize("shape", [(2, 128, 1024), (4, 64, 512), (8, 256), (3, 4096), (2, 8192), (5, 1000)])
def test_rms_norm_add(shape, dtype):
    x, r, w = _norm_inputs(shape, dtype, 0)
    out, added = tk.rms_norm_add(dev(x, dtype), dev(r, dtype), dev(w, dtype), eps=1e-5)
    n, added_ref = O.rms_norm_add(x, r, w, 1e-5, dtype)
    assert out.shape == x.shape and added.shape == x.shape
    np.testing.assert_array_equal(host(added), added_ref)                 # one exact fp32 add, one rounding
    ulp = {"bf16": 2.0 ** -7, "f16": 2.0 ** -10, "f32": 2.0 ** -20}[dtype]
    assert np.all(np.abs(host(out) - n) <= np.abs(n) * ulp * 1.1 + 1e-6)


@pytest.mark.parametrize("shape", [(4, 64, 512), (8, 256), (3, 4096)])
def test_rms_norm_add_fp8_dynamic_static_and_int8(shape):
    x, r, w = _norm_inputs(shape, "bf16", 1)
    n, added_ref = O.rms_norm_add(x, r, w, 1e-5, "bf16")
    D = shape[-1]
    codes, added, scale = tk.rms_norm_add_fp8(dev(x, "bf16"), dev(r, "bf16"), dev(w, "bf16"))
    rc, rs = O.quantize_groups(n, D, "fp8")
    np.testing.assert_allclose(host(scale).reshape(-1), rs.reshape(-1), rtol=1e-5)
    _codes_agree(host(codes), rc)
    deq = DEC[host(codes)] * host(scale)[..., None]
    assert np.all(np.abs(deq - n) <= 0.0625 * np.abs(n) + 2.0 * host(scale)[..., None])
    np.testing.assert_array_equal(host(added), added_ref)
    # static per-tensor scale
    st = float(np.abs(n).max() / 448.0)
    codes, added = tk.rms_norm_add_fp8(dev(x, "bf16"), dev(r, "bf16"), dev(w, "bf16"), scale=st)
    want = O.e4m3_encode_device((n * np.float32(1.0 / st)).astype(np.float32))
    _codes_agree(host(codes), want)
    # int8 per row
    from quixicore_metal_b200 import tk_torch
    codes, added, scale = tk_torch.rms_norm_add_int8_dyn(dev(x, "bf16"), dev(r, "bf16"), dev(w, "bf16"))
    rc, rs = O.quantize_groups(n, D, "int8")
    np.testing.assert_allclose(host(scale).reshape(-1), rs.reshape(-1), rtol=1e-5)
    assert np.abs(host(codes).astype(np.int32) - rc.astype(np.int32)).max() <= 1
    _codes_agree(host(codes), rc, 0.99)


@pytest.mark.parametrize("ue8m0", [False, True])
@pytest.mark.parametrize("int8", [False, True])
@pytest.mark.parametrize("shape", [(4, 512), (2, 3, 1024), (3, 4096)])
def test_rms_norm_add_per_block(shape, int8, ue8m0):
    x, r, w = _norm_inputs(shape, "bf16", 5)
    n, _ = O.rms_norm_add(x, r, w, 1e-5, "bf16")
    codes, added, scale = tk.rms_norm_add_per_block(dev(x, "bf16"), dev(r, "bf16"), dev(w, "bf16"), int8=int8, ue8m0=ue8m0)
    D, G = shape[-1], 128
    rc, rs = O.quantize_groups(n, G, "int8" if int8 else "fp8", ue8m0)
    sn = host(scale)
    assert sn.shape == tuple(shape[:-1]) + (D // G,)
    np.testing.assert_allclose(sn, rs, rtol=1e-5)
    if ue8m0 and not int8:
        e = np.log2(np.where(sn > 0, sn, 1.0))
        np.testing.assert_array_equal(e, np.round(e))
    _codes_agree(host(codes), rc, 0.99)
    nb = n.reshape(sn.shape + (G,))
    qmax = 127.0 if int8 else 448.0
    assert (sn * qmax >= np.abs(nb).max(-1) - 1e-2).all()


@pytest.mark.parametrize("dtype", ["f32", "bf16"])
@pytest.mark.parametrize("act", ["swiglu", "swiglu_oai"])
def test_silu_mul_quant_per_token(act, dtype):
    rng = np.random.default_rng(0)
    T, D = 33, 768
    x, g = rounded(rng.standard_normal((T, D)), dtype), rounded(rng.standard_normal((T, D)), dtype)
    ref = O.gated_act(act, x, g)
    codes, scale = tk.silu_mul_quant_fp8(dev(x, dtype), dev(g, dtype), act=act)
    sn = host(scale)[:, None]
    recon = sn * DEC[host(codes)]
    assert (np.abs(recon - ref) <= np.abs(ref) * 2.0 ** -4 + sn * 2.0 ** -6 + 1e-5).all()
    assert (sn[:, 0] * 448.0 >= np.abs(ref).max(1) - 1e-3).all()
    rc, rs = O.quantize_groups(ref, D, "fp8")
    np.testing.assert_allclose(sn[:, 0], rs[:, 0], rtol=1e-5)
    _codes_agree(host(codes), rc)
    codes, scale = tk.silu_mul_quant_int8(dev(x, dtype), dev(g, dtype), act=act)
    sn = host(scale)[:, None]
    assert (np.abs(sn * host(codes).astype(np.float64) - ref) <= 0.51 * sn + 1e-6).all()


@pytest.mark.parametrize("ue8m0", [False, True])
@pytest.mark.parametrize("act", ["swiglu", "swiglu_oai"])
def test_silu_mul_quant_fp8_group(act, ue8m0):
    rng = np.random.default_rng(2)
    T, D, G = 8, 512, 128
    x, g = rng.standard_normal((T, D)).astype(np.float32), rng.standard_normal((T, D)).astype(np.float32)
    codes, scale = tk.silu_mul_quant_fp8_group(dev(x), dev(g), group_size=G, ue8m0=ue8m0, act=act)
    sn = host(scale)
    assert sn.shape == (T, D // G)
    ref = O.gated_act(act, x, g).reshape(T, D // G, G)
    if ue8m0:
        e = np.log2(np.where(sn > 0, sn, 1.0))
        np.testing.assert_array_equal(e, np.round(e))
    assert (sn * 448.0 >= np.abs(ref).max(-1) - 1e-3).all()
    recon = sn[..., None] * DEC[host(codes)].reshape(T, D // G, G)
    assert (np.abs(recon - ref) <= np.abs(ref) * 2.0 ** -4 + sn[..., None] * 2.0 ** -6 + 1e-5).all()
    rc, rs = O.quantize_groups(ref.reshape(T, D), G, "fp8", ue8m0)
    np.testing.assert_allclose(sn, rs, rtol=1e-5)


def test_all_zero_rows_and_errors():
    z = torch.zeros((2, 256), dtype=torch.bfloat16, device="cuda")
    codes, scale = tk.silu_mul_quant_fp8(z, z)
    assert float(scale.abs().max()) == 0.0 and int(codes.max()) == 0
    with pytest.raises(RuntimeError, match="D % 128"):
        tk.rms_norm_add_per_block(z[:, :200], z[:, :200], z[0, :200])
    with pytest.raises(RuntimeError, match="group_size"):
        tk.silu_mul_quant_fp8_group(z, z, group_size=96)
    with pytest.raises(RuntimeError, match="act must be"):
        tk.silu_mul_quant_fp8(z, z, act="geglu")
