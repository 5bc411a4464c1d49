"""BaseQN separate-plane consumers against the CPU oracle, through the tk routers.

Follows the reference's tests/correctness/quantization/base_q/test_base_q.py: every code width and
affine mode, the four scale storage types, the three group sizes, output dtypes, gemv / gemm, the
fused q/k/v and SwiGLU forms, batched greedy LM head with the lowest-id tie rule, embedding with
invalid ids, expert stacks, and the validation messages.  Each multiplying op is run at a small
shape (K = 64: the shape-generic kernel) and at shapes that take the streaming tensor-core kernel
(K a multiple of 128, >= 512, 16-bit activations), including ragged row counts, a K that is not a
multiple of the 512-column stage, and more than eight activation columns.

Tolerances: dequantise / embedding fp32 output bit-exact (the decode is two fp32 roundings);
products accumulate in fp32 on the GPU and in float64 in the oracle, so 16-bit outputs may differ
by one ulp of the output format, fp32 outputs by 2e-5 relative to the output scale."""
import numpy as np
import pytest
import torch

from oracle import qx_oracle as O
from tests._util import TORCH_DT, assert_close_dtype, dev, host, rounded

pytestmark = pytest.mark.gpu

tk = pytest.importorskip("quixicore_metal_b200.tk")

BITS = [2, 3, 4, 5, 6, 8]
_PLANE_DT = {"bf16": torch.bfloat16, "f16": torch.float16}


def planes(rows, K, bits, group=32, sd="f16", sym=False, seed=0, lead=()):
    """(device codes, scales, biases, fp32 oracle weights)."""
    codes, scales, biases = O.base_q_random_planes(rows, K, bits, group, sd, sym, seed, lead=lead)
    W = O.base_q_dequantize(codes, scales, biases, bits, group, sd, sym)

    def up(p):
        if p is None:
            return None
        t = torch.from_numpy(p.view(np.int16) if p.dtype == np.uint16 else p).cuda()
        return t.view(_PLANE_DT[sd]) if sd in _PLANE_DT else t
    return dev(codes), up(scales), up(biases), W


def out_scale(W, x):
    return float(np.sqrt((W.astype(np.float64) ** 2).sum(-1).mean()) * np.abs(x).max() + 1e-6)


# ---- dequantise / embedding --------------------------------------------------------------------------
@pytest.mark.parametrize("bits", BITS)
@pytest.mark.parametrize("sym", [False, True])
def test_dequant_all_widths_and_affine_modes(bits, sym):
    c, s, b, W = planes(37, 256, bits, sym=sym, seed=bits)
    got = tk.base_qdequant(c, s, b, bits, 32, "f16", symmetric=sym, output_dtype="float32")
    np.testing.assert_array_equal(host(got).view(np.uint32), W.view(np.uint32))


@pytest.mark.parametrize("bits,sd", [(4, "bf16"), (4, "f16"), (4, "e8m0"), (8, "e4m3"), (3, "e8m0")])
@pytest.mark.parametrize("group", [32, 64, 128])
def test_scale_storage_types_and_group_sizes(bits, sd, group):
    c, s, b, W = planes(9, 512, bits, group, sd, False, seed=group + bits)
    got = tk.base_qdequant(c, s, b, bits, group, sd, output_dtype="float32", layout=f"metal_lane_strided_q{bits}")
    np.testing.assert_array_equal(host(got).view(np.uint32), W.view(np.uint32))


@pytest.mark.parametrize("output_dtype,name", [("float16", "f16"), ("bfloat16", "bf16"), ("float32", "f32")])
def test_dequant_output_dtypes(output_dtype, name):
    c, s, b, W = planes(5, 128, 6, seed=3)
    got = tk.base_qdequant(c, s, b, 6, 32, "f16", output_dtype=output_dtype)
    assert got.dtype == TORCH_DT[name]
    np.testing.assert_array_equal(host(got), O.round_to(W, name))


def test_embedding_shape_invalid_ids_and_values():
    c, s, b, W = planes(11, 192, 5, 64, "bf16", seed=8)
    ids = np.array([[2, -1, 10], [99, 0, 11]], np.int32)
    for od, name in (("float32", "f32"), ("float16", "f16")):
        got = tk.base_qembedding(c, s, b, dev(ids), 5, 64, "bf16", output_dtype=od)
        assert tuple(got.shape) == (2, 3, 192)
        np.testing.assert_array_equal(host(got), O.base_q_embedding(W, ids, name))
    got = tk.base_qembedding(c, s, b, dev(ids.astype(np.int64)), 5, 64, "bf16", output_dtype="float32")
    np.testing.assert_array_equal(host(got), O.base_q_embedding(W, ids, "f32"))


# ---- gemv / gemm ---------------------------------------------------------------------------------------
@pytest.mark.parametrize("bits", BITS)
@pytest.mark.parametrize("dtype", ["f16", "bf16", "f32"])
def test_gemv_and_gemm_small(bits, dtype):
    c, s, b, W = planes(3, 64, bits, seed=20 + bits)
    rng = np.random.default_rng(bits)
    vec = rounded(rng.standard_normal((64, 1)), dtype)
    mat = rounded(rng.standard_normal((64, 7)), dtype)
    got_v = tk.base_qgemv(c, s, b, dev(vec, dtype), bits, 32, "f16")
    got_m = tk.base_qgemm(c, s, b, dev(mat, dtype), bits, 32, "f16")
    routed = tk.base_qgemm(c, s, b, dev(vec, dtype), bits, 32, "f16")
    assert got_v.dtype == TORCH_DT[dtype] and tuple(got_m.shape) == (3, 7)
    assert_close_dtype(host(got_v), O.base_q_matmul(W, vec, dtype), dtype, out_scale(W, vec))
    assert_close_dtype(host(got_m), O.base_q_matmul(W, mat, dtype), dtype, out_scale(W, mat))
    np.testing.assert_array_equal(host(got_v), host(routed))


@pytest.mark.parametrize("bits", BITS)
@pytest.mark.parametrize("sym", [False, True])
def test_gemv_streaming_kernel_every_width(bits, sym):
    rows, K = 301, 1536
    c, s, b, W = planes(rows, K, bits, 32, "f16", sym, seed=40 + bits)
    rng = np.random.default_rng(50 + bits)
    for dtype in ("bf16", "f16"):
        x = rounded(rng.standard_normal((K, 1)), dtype)
        got = tk.base_qgemv(c, s, b, dev(x, dtype), bits, 32, "f16", symmetric=sym)
        assert_close_dtype(host(got), O.base_q_matmul(W, x, dtype), dtype, out_scale(W, x))


@pytest.mark.parametrize("bits,sd,group", [(4, "bf16", 64), (4, "e8m0", 128), (8, "e4m3", 32), (3, "e8m0", 64),
                                           (2, "f16", 128), (6, "bf16", 32), (5, "f16", 64)])
@pytest.mark.parametrize("K", [640, 2048])
def test_gemv_streaming_kernel_scale_types_groups_and_ragged_k(bits, sd, group, K):
    rows = 130
    c, s, b, W = planes(rows, K, bits, group, sd, False, seed=60 + bits + group)
    rng = np.random.default_rng(70 + bits)
    x = rounded(rng.standard_normal((K, 1)), "bf16")
    got = tk.base_qgemv(c, s, b, dev(x, "bf16"), bits, group, sd)
    assert_close_dtype(host(got), O.base_q_matmul(W, x, "bf16"), "bf16", out_scale(W, x))


@pytest.mark.parametrize("bits,M", [(4, 2), (4, 8), (4, 11), (8, 5), (3, 19)])
def test_gemm_streaming_kernel_column_blocks(bits, M):
    rows, K = 200, 1024
    c, s, b, W = planes(rows, K, bits, 64, "bf16", False, seed=80 + bits + M)
    rng = np.random.default_rng(90 + M)
    x = rounded(rng.standard_normal((K, M)), "bf16")
    got = tk.base_qgemm(c, s, b, dev(x, "bf16"), bits, 64, "bf16")
    assert tuple(got.shape) == (rows, M)
    assert_close_dtype(host(got), O.base_q_matmul(W, x, "bf16"), "bf16", out_scale(W, x))


def test_streaming_and_generic_kernels_agree():
    from quixicore_metal_b200 import _lib
    rows, K = 96, 1024
    c, s, b, W = planes(rows, K, 4, 32, "f16", False, seed=5)
    x = dev(rounded(np.random.default_rng(6).standard_normal((K, 3)), "f16"), "f16")
    fast = host(tk.base_qgemm(c, s, b, x, 4, 32, "f16"))
    _lib.set_option("force_generic", 1)
    try:
        slow = host(tk.base_qgemm(c, s, b, x, 4, 32, "f16"))
    finally:
        _lib.set_option("force_generic", 0)
    ref = O.base_q_matmul(W, host(x), "f16")
    assert_close_dtype(fast, ref, "f16", out_scale(W, host(x)))
    assert_close_dtype(slow, ref, "f16", out_scale(W, host(x)))
    assert _lib.lib().qx_cuda_device_error() == 0


# ---- fused q/k/v and SwiGLU ------------------------------------------------------------------------------
@pytest.mark.parametrize("bits", [3, 4, 6, 8])
@pytest.mark.parametrize("sym", [False, True])
@pytest.mark.parametrize("K,dtype", [(64, "f16"), (64, "f32"), (1024, "bf16")])
def test_fused_qkv_and_swiglu(bits, sym, K, dtype):
    q = planes(5 if K == 64 else 160, K, bits, sym=sym, seed=bits + 10)
    k = planes(3 if K == 64 else 40, K, bits, sym=sym, seed=bits + 20)
    v = planes(4 if K == 64 else 47, K, bits, sym=sym, seed=bits + 30)
    gate = planes(7 if K == 64 else 210, K, bits, sym=sym, seed=bits + 40)
    up = planes(7 if K == 64 else 210, K, bits, sym=sym, seed=bits + 50)
    x = rounded(np.random.default_rng(bits + 60).standard_normal((K, 1)), dtype)
    xd = dev(x, dtype)
    outs = tk.base_qgemv_qkv(*q[:3], *k[:3], *v[:3], xd, bits, 32, "f16", symmetric=sym)
    for got, w in zip(outs, (q, k, v)):
        assert_close_dtype(host(got), O.base_q_matmul(w[3], x, dtype), dtype, out_scale(w[3], x))
    got = tk.base_qgemv_swiglu(*gate[:3], *up[:3], xd, bits, 32, "f16", symmetric=sym)
    ref = O.base_q_swiglu(gate[3], up[3], x, dtype)
    sc = out_scale(gate[3], x) * max(1.0, out_scale(up[3], x))
    assert_close_dtype(host(got), ref, dtype, sc)


# ---- greedy LM head ---------------------------------------------------------------------------------------
@pytest.mark.parametrize("bits", [3, 4, 6, 8])
@pytest.mark.parametrize("sym", [False, True])
@pytest.mark.parametrize("batch", [1, 3])
@pytest.mark.parametrize("V,K", [(19, 64), (5003, 1024)])
def test_lm_head_argmax_batched(bits, sym, batch, V, K):
    c, s, b, W = planes(V, K, bits, sym=sym, seed=700 + bits)
    dtype = "f16"
    x = rounded(0.2 * np.random.default_rng(800 + bits).standard_normal((K, batch)), dtype)
    got = host(tk.base_qlm_head_argmax(c, s, b, dev(x, dtype), bits, 32, "f16", symmetric=sym))
    want, gap, r = O.base_q_lm_head_argmax(W, x, dtype)
    assert got.dtype == np.int32 and got.shape == (batch,)
    for j in range(batch):
        # the winner is decided on logits rounded to f16: equal ids unless the two best float64
        # logits are closer than two ulps of that rounding (then either may round on top)
        if got[j] != want[j]:
            assert gap[j] <= 2.0 ** -9 * abs(r[want[j], j]) + 1e-6, (j, got[j], want[j], gap[j])
            assert r[got[j], j] >= r[want[j], j] - 2.0 ** -10 * abs(r[want[j], j])


def test_lm_head_argmax_ties_choose_lower_token():
    for V, K in ((17, 32), (700, 512)):
        codes = dev(O.base_q_pack(np.zeros((V, K), np.uint8), 4))
        scales = torch.zeros((V, K // 32), dtype=torch.float16, device="cuda")
        x = torch.ones((K, 2), dtype=torch.float16, device="cuda")
        got = tk.base_qlm_head_argmax(codes, scales, scales.clone(), x, 4, 32, "f16")
        np.testing.assert_array_equal(host(got), [0, 0])


# ---- expert stacks ------------------------------------------------------------------------------------------
@pytest.mark.parametrize("bits", BITS)
@pytest.mark.parametrize("sym", [False, True])
def test_grouped_expert_gemm_and_swiglu(bits, sym):
    E, N, K = 3, 72, 512
    c, s, b, W = planes(N, K, bits, sym=sym, seed=1100 + bits, lead=(E,))
    rng = np.random.default_rng(1200 + bits)
    x = rounded(0.2 * rng.standard_normal((128, K)), "f16")
    eot = np.array([0, 2, -1, 1], np.int32)
    got_rect = host(tk.base_qmoe_gemm(c, s, b, dev(x, "f16"), dev(eot), bits, 32, "f16", symmetric=sym))
    got_sw = host(tk.base_qmoe_swiglu(c, s, b, dev(x, "f16"), dev(eot), bits, 32, "f16", symmetric=sym))
    assert got_rect.shape == (128, N) and got_sw.shape == (128, N // 2)
    for tile, e in enumerate(eot):
        sl = slice(tile * 32, (tile + 1) * 32)
        if e < 0:
            assert not got_rect[sl].any() and not got_sw[sl].any()
            continue
        logits = x[sl].astype(np.float64) @ W[e].astype(np.float64).T
        sc = out_scale(W[e], x[sl])
        assert_close_dtype(got_rect[sl], O.round_to(logits.astype(np.float32), "f16"), "f16", sc)
        g, u = np.split(logits, 2, axis=1)
        assert_close_dtype(got_sw[sl], O.round_to(((g / (1.0 + np.exp(-g))) * u).astype(np.float32), "f16"), "f16", sc * sc)


@pytest.mark.parametrize("bits,sd", [(4, "bf16"), (4, "e8m0"), (8, "e4m3")])
def test_grouped_expert_scale_storage_types(bits, sd):
    c, s, b, W = planes(40, 640, bits, 32, sd, False, seed=1500 + bits, lead=(2,))
    x = rounded(0.1 * np.random.default_rng(1700).standard_normal((64, 640)), "bf16")
    eot = np.array([1, 0], np.int32)
    got = host(tk.base_qmoe_gemm(c, s, b, dev(x, "bf16"), dev(eot), bits, 32, sd))
    for tile, e in enumerate(eot):
        sl = slice(tile * 32, (tile + 1) * 32)
        ref = O.round_to((x[sl].astype(np.float64) @ W[e].astype(np.float64).T).astype(np.float32), "bf16")
        assert_close_dtype(got[sl], ref, "bf16", out_scale(W[e], x[sl]))


# ---- validation ------------------------------------------------------------------------------------------------
def test_validation_rejects_mismatched_planes():
    c, s, b, _ = planes(3, 64, 4, seed=1)
    with pytest.raises(RuntimeError, match="codes.shape"):
        tk.base_qdequant(c[:, :-1], s, b, 4, 32, "f16")
    with pytest.raises(ValueError, match="biases are required"):
        tk.base_qdequant(c, s, None, 4, 32, "f16")
    z = torch.zeros(tuple(s.shape), dtype=torch.uint8, device="cuda")
    with pytest.raises(RuntimeError, match="only for q8"):
        tk.base_qdequant(c, z, z, 4, 32, scale_dtype="e4m3")
    with pytest.raises(RuntimeError, match="group_size"):
        tk.base_qdequant(c, s, b, 4, 48, "f16")
    with pytest.raises(RuntimeError, match="layout"):
        tk.base_qdequant(c, s, b, 4, 32, "f16", layout="metal_lane_strided_q8")
    with pytest.raises(RuntimeError, match="declared scale_dtype"):
        tk.base_qdequant(c, s, b, 4, 32, "bf16")
    x = torch.zeros((64, 2), dtype=torch.float16, device="cuda")
    with pytest.raises(RuntimeError, match=r"\(K, 1\)"):
        tk.base_qgemv(c, s, b, x, 4, 32, "f16")
    with pytest.raises(ValueError, match="non-empty"):
        tk.base_qlm_head_argmax(c, s, b, x[:, :0], 4, 32, "f16")


def test_library_repeats_the_descriptor_checks():
    """The C entry points validate on their own (a host that binds them directly gets the same
    status codes as the Python layer's messages)."""
    from quixicore_metal_b200 import _lib
    L = _lib.lib()
    c, s, b, _ = planes(3, 64, 4, seed=1)
    out = torch.empty((3, 64), dtype=torch.float32, device="cuda")
    pl = _lib.BaseQPlanes(c.data_ptr(), s.data_ptr(), b.data_ptr())
    st = torch.cuda.current_stream().cuda_stream
    for desc, frag in ((_lib.BaseQDescriptor(7, 32, b"f16", 0, b"metal"), b"bits"),
                       (_lib.BaseQDescriptor(4, 32, b"e4m3", 0, b"metal"), b"only for q8"),
                       (_lib.BaseQDescriptor(4, 32, b"f16", 0, b"rowmajor"), b"layout"),
                       (_lib.BaseQDescriptor(4, 32, b"int8", 0, b"metal"), b"scale_dtype")):
        r = L.qx_cuda_base_qdequant(st, pl, desc, out.data_ptr(), 3, 64, _lib.DTYPE_F32)
        assert _lib.STATUS_NAMES[r.code] == "invalid_argument" and frag in r.detail, r.detail
    nob = _lib.BaseQPlanes(c.data_ptr(), s.data_ptr(), None)
    r = L.qx_cuda_base_qdequant(st, nob, _lib.BaseQDescriptor(4, 32, b"f16", 0, b"metal"), out.data_ptr(), 3, 64, _lib.DTYPE_F32)
    assert b"biases are required" in r.detail
    r = L.qx_cuda_base_qdequant(st, nob, _lib.BaseQDescriptor(4, 32, b"f16", 1, b"metal"), out.data_ptr(), 3, 64, _lib.DTYPE_F32)
    assert r.code == 0
