"""CPU oracle for the quantized decode-projection path (TEST INFRASTRUCTURE, not product code).

A numpy restatement of the reference's arithmetic for `decode_linear_epilogue`, `decode_swiglu`,
fused `lm_head_sample`, the runtime output quantizers and the six packed weight formats.  Only the
tests, the smoke check and the benchmark's CPU-baseline leg may import this module; the CUDA
product path never does.

Parity pin: the decoders, the e4m3 encoder's tie rule, the RNG hash and the q6_K known-answer
bytes are checked against fixtures produced by importing the reference's own `tk.quant`
(`tests/golden/make_golden.py`) and against the constants quoted from its tests.  The MXFP8
*output* requantisation has no reference test that pins its codes: parity unpinned for that rule
(it restates `quantize_per_group_fp8(G=32, ue8m0=1)`).

Every function cites the reference file:line (paths relative to the reference project root)
whose behaviour it restates.
"""
from __future__ import annotations

import numpy as np

# ----------------------------------------------------------------------------------------------
# Block formats.  (block_k weights, block_bytes) per format; packed tensor is uint8
# (N, K/block_k, block_bytes).  kernels/matmul/decode_linear/decode_linear.cpp:25-34
# ----------------------------------------------------------------------------------------------
FORMATS = {
    "q4_0": (32, 18),
    "q8_0": (32, 34),
    "q6_K": (256, 210),
    "mxfp8": (32, 33),
    "nvfp4": (16, 9),
    "mxfp4": (32, 17),
}

NEG_INF = np.float32(-3.4028234663852886e38)  # LMH_NEG_INF, kernels/quantization/lm_head/lm_head.metal
TILE_V = 256                                   # bindings/pytorch_mps/tk_torch/torch_kernels.mm:5048


# ----------------------------------------------------------------------------------------------
# Scalar codecs.  include/metal/ops/warp/register/tile/dequant.metal:271-291,
# bindings/python/tk/quant.py:216-225
# ----------------------------------------------------------------------------------------------
def e4m3_decode(codes: np.ndarray) -> np.ndarray:
    """1-4-3 float, bias 7, no NaN/inf: exponent 15 decodes all eight mantissas (max 480)."""
    c = np.asarray(codes).astype(np.int64)
    man = (c & 7).astype(np.float64)
    exp = (c >> 3) & 15
    mag = np.where(exp == 0, man * 2.0 ** -9, (8.0 + man) * np.exp2(exp.astype(np.float64) - 10.0))
    return np.where((c & 0x80) != 0, -mag, mag).astype(np.float32)


_E2M1_MAG = np.array([0.0, 0.5, 1.0, 1.5, 2.0, 3.0, 4.0, 6.0], np.float32)


def e2m1_decode(nibbles: np.ndarray) -> np.ndarray:
    """1-2-1 float: magnitudes {0,.5,1,1.5,2,3,4,6}, bit 3 is the sign."""
    n = np.asarray(nibbles).astype(np.int64)
    mag = _E2M1_MAG[n & 7]
    return np.where((n & 8) != 0, -mag, mag).astype(np.float32)


def e8m0_decode(codes: np.ndarray) -> np.ndarray:
    """Power-of-two scale 2^(code-127); the byte is the fp32 exponent field, code 0 is the one
    subnormal (2^-127) and code 255 is +inf.  dequant.metal:288-291"""
    c = np.asarray(codes).astype(np.uint32)
    bits = np.where(c == 0, np.uint32(0x00400000), c << np.uint32(23)).astype(np.uint32)
    return bits.view(np.float32)


def _f16_at(packed: np.ndarray, lo: int) -> np.ndarray:
    """Little-endian fp16 stored at byte offset `lo` of every block -> float32 (N, nb)."""
    raw = packed[..., lo].astype(np.uint16) | (packed[..., lo + 1].astype(np.uint16) << 8)
    return raw.view(np.float16).astype(np.float32)


# ----------------------------------------------------------------------------------------------
# Unpackers: packed uint8 (N, nb, block_bytes) -> float32 (N, K).  All products are exact in fp32.
# ----------------------------------------------------------------------------------------------
def dequantize_q4_0(p):
    """{f16 d; u8 qs[16]}: w[i]=d*((qs[i]&15)-8), w[i+16]=d*((qs[i]>>4)-8).  quant.py:67-78"""
    p = np.asarray(p, np.uint8); N, nb, _ = p.shape
    d = _f16_at(p, 0)[..., None]
    qs = p[..., 2:18].astype(np.int32)
    q = np.concatenate([qs & 15, qs >> 4], axis=-1) - 8
    return (d * q.astype(np.float32)).reshape(N, nb * 32)


def dequantize_q8_0(p):
    """{f16 d; i8 qs[32]}: w=d*q.  quant.py:34-43"""
    p = np.asarray(p, np.uint8); N, nb, _ = p.shape
    d = _f16_at(p, 0)[..., None]
    q = p[..., 2:34].view(np.int8).astype(np.float32)
    return (d * q).reshape(N, nb * 32)


def _q6k_column_maps():
    c = np.arange(256)
    chunk, pos = c >> 7, c & 127
    group, l = pos >> 5, pos & 31
    ql_idx = chunk * 64 + l + 32 * (group & 1)
    hi_nib = (group & 2) != 0
    qh_idx = chunk * 32 + l
    qh_shift = 2 * group
    sc_idx = chunk * 8 + (l >> 4) + 2 * group
    return ql_idx, hi_nib, qh_idx, qh_shift, sc_idx


def dequantize_q6_K(p):
    """{u8 ql[128]; u8 qh[64]; i8 sc[16]; f16 d}, 256 weights: 6-bit code = 4 low bits from ql,
    2 high bits from qh, minus 32; w = d*sc[sub]*q with the fp32 product taken as (d*sc)*q.
    quant.py:1168-1184, dequant.metal:640-654"""
    p = np.asarray(p, np.uint8); N, nb, _ = p.shape
    ql_idx, hi_nib, qh_idx, qh_shift, sc_idx = _q6k_column_maps()
    ql = p[..., 0:128].astype(np.int32)[..., ql_idx]
    nib = np.where(hi_nib, ql >> 4, ql & 15)
    hb = (p[..., 128:192].astype(np.int32)[..., qh_idx] >> qh_shift) & 3
    q = (nib | (hb << 4)) - 32
    sc = p[..., 192:208].view(np.int8).astype(np.float32)[..., sc_idx]
    d = _f16_at(p, 208)[..., None]
    return ((d * sc) * q.astype(np.float32)).reshape(N, nb * 256)


def dequantize_mxfp8(p):
    """{e8m0; e4m3[32]}: w = 2^(e-127)*e4m3.  quant.py:325-329"""
    p = np.asarray(p, np.uint8); N, nb, _ = p.shape
    s = e8m0_decode(p[..., 0])[..., None]
    return (s * e4m3_decode(p[..., 1:33])).reshape(N, nb * 32)


def dequantize_nvfp4(p):
    """{e4m3 s; u8 qs[8]}, 16 weights: w[i]=s*e2m1(qs[i]&15), w[i+8]=s*e2m1(qs[i]>>4).
    quant.py:346-352"""
    p = np.asarray(p, np.uint8); N, nb, _ = p.shape
    s = e4m3_decode(p[..., 0])[..., None]
    qs = p[..., 1:9].astype(np.int32)
    nib = np.concatenate([qs & 15, qs >> 4], axis=-1)
    return (s * e2m1_decode(nib)).reshape(N, nb * 16)


def dequantize_mxfp4(p):
    """{e8m0; u8 qs[16]}, 32 weights: low nibble = w[i], high nibble = w[i+16].  quant.py:365-371"""
    p = np.asarray(p, np.uint8); N, nb, _ = p.shape
    s = e8m0_decode(p[..., 0])[..., None]
    qs = p[..., 1:17].astype(np.int32)
    nib = np.concatenate([qs & 15, qs >> 4], axis=-1)
    return (s * e2m1_decode(nib)).reshape(N, nb * 32)


_DEQUANT = {
    "q4_0": dequantize_q4_0, "q8_0": dequantize_q8_0, "q6_K": dequantize_q6_K,
    "mxfp8": dequantize_mxfp8, "nvfp4": dequantize_nvfp4, "mxfp4": dequantize_mxfp4,
}


def dequantize(fmt: str, packed: np.ndarray) -> np.ndarray:
    bk, bb = FORMATS[fmt]
    packed = np.asarray(packed, np.uint8)
    assert packed.ndim == 3 and packed.shape[2] == bb, (fmt, packed.shape)
    return _DEQUANT[fmt](packed)


# ----------------------------------------------------------------------------------------------
# Synthetic packers.  These are NOT the reference's quantizers (its q4_0/q6_K packers run a ggml
# scale search, quant.py:832-856): they are plain round-to-nearest packers that emit valid blocks
# of the same layout, so that a machine without the reference can build packed test inputs.
# Kernel parity is defined on dequantize(packed), so any valid packed tensor is a fair input.
# ----------------------------------------------------------------------------------------------
def _nearest_code(x, values):
    """Index of the nearest table value; ties go to the lower index (the order np.argmin over the
    distances would give).  Both code tables are sign-symmetric - the first half holds the
    magnitudes in ascending order, the second half their negatives - so the search runs on the
    magnitude midpoints: O(n log half) instead of an (n, len(values)) distance matrix."""
    x = np.asarray(x, np.float32)
    half = values.size // 2
    mags = np.asarray(values[:half], np.float64)
    mid = 0.5 * (mags[1:] + mags[:-1])
    m = np.searchsorted(mid, np.abs(x.astype(np.float64)), side="left")      # |x| == midpoint -> smaller magnitude
    neg = (x < 0) & (m > 0)                                                    # nearest-to-zero negatives take +0
    return (m + half * neg).astype(np.uint8)


_E2M1_TABLE = e2m1_decode(np.arange(16))
_E4M3_CODES = np.array([c for c in range(256) if (c & 0x7F) != 0x7F], np.uint8)
_E4M3_TABLE = e4m3_decode(_E4M3_CODES)


def _pack_halves(codes):
    h = codes.shape[-1] // 2
    return (codes[..., :h] | (codes[..., h:] << 4)).astype(np.uint8)


def _f16_bytes(d):
    return np.ascontiguousarray(d.astype(np.float16)).view(np.uint8).reshape(d.shape + (2,))


def synth_pack(fmt: str, W: np.ndarray) -> np.ndarray:
    W = np.ascontiguousarray(W, np.float32); N, K = W.shape
    bk, bb = FORMATS[fmt]
    assert K % bk == 0
    nb = K // bk
    B = W.reshape(N, nb, bk)
    amax = np.abs(B).max(-1)
    out = np.zeros((N, nb, bb), np.uint8)
    if fmt == "q8_0":
        d = (amax / 127.0).astype(np.float16).astype(np.float32)
        ds = np.where(d == 0, 1.0, d)
        out[..., 0:2] = _f16_bytes(d)
        out[..., 2:] = np.clip(np.rint(B / ds[..., None]), -127, 127).astype(np.int8).view(np.uint8)
    elif fmt == "q4_0":
        i = np.abs(B).argmax(-1)[..., None]
        d = (np.take_along_axis(B, i, -1)[..., 0] / -8.0).astype(np.float16).astype(np.float32)
        ds = np.where(d == 0, 1.0, d)
        q = np.clip(np.rint(B / ds[..., None]) + 8, 0, 15).astype(np.uint8)
        out[..., 0:2] = _f16_bytes(d)
        out[..., 2:] = _pack_halves(q)
    elif fmt == "q6_K":
        sub = B.reshape(N, nb, 16, 16)
        smax = np.abs(sub).max(-1) / 31.0                       # per-16 scale
        d = (smax.max(-1) / 127.0).astype(np.float16).astype(np.float32)
        ds = np.where(d == 0, 1.0, d)
        sc = np.clip(np.rint(smax / ds[..., None]), -128, 127).astype(np.int32)
        eff = d[..., None] * sc
        eff = np.where(eff == 0, 1.0, eff)
        code = (np.clip(np.rint(sub / eff[..., None]), -32, 31) + 32).astype(np.int32).reshape(N, nb, 256)
        ql_idx, hi_nib, qh_idx, qh_shift, _ = _q6k_column_maps()
        for c in range(256):
            lo4, hi2 = code[..., c] & 15, (code[..., c] >> 4) & 3
            out[..., ql_idx[c]] |= ((lo4 << 4) if hi_nib[c] else lo4).astype(np.uint8)
            out[..., 128 + qh_idx[c]] |= (hi2 << qh_shift[c]).astype(np.uint8)
        out[..., 192:208] = sc.astype(np.int8).view(np.uint8)
        out[..., 208:210] = _f16_bytes(d)
    elif fmt in ("mxfp8", "mxfp4"):
        top = 448.0 if fmt == "mxfp8" else 6.0
        e = np.where(amax > 0, np.ceil(np.log2(np.maximum(amax, 1e-30) / top)), 0.0)
        code = np.clip(e + 127, 0, 254).astype(np.int32)
        s = e8m0_decode(code)
        scaled = B / s[..., None]
        out[..., 0] = code.astype(np.uint8)
        if fmt == "mxfp8":
            out[..., 1:] = _E4M3_CODES[_nearest_code(scaled, _E4M3_TABLE)]
        else:
            out[..., 1:] = _pack_halves(_nearest_code(scaled, _E2M1_TABLE))
    elif fmt == "nvfp4":
        sb = _E4M3_CODES[_nearest_code(amax / 6.0, _E4M3_TABLE)]
        s = e4m3_decode(sb)
        ss = np.where(s == 0, 1.0, s)
        out[..., 0] = sb
        out[..., 1:] = _pack_halves(_nearest_code(B / ss[..., None], _E2M1_TABLE))
    else:
        raise ValueError(fmt)
    return out


def random_packed(fmt: str, N: int, K: int, seed: int, scale: float = 0.02) -> np.ndarray:
    """Random *bytes* that form valid blocks: every code value appears, scales stay in a sane range.
    Exercises decoder paths a Gaussian packer never reaches (e.g. e4m3 exponent-15 codes)."""
    rng = np.random.default_rng(seed)
    bk, bb = FORMATS[fmt]; nb = K // bk
    out = rng.integers(0, 256, size=(N, nb, bb), dtype=np.uint8)
    if fmt in ("q4_0", "q8_0"):
        out[..., 0:2] = _f16_bytes((scale * rng.standard_normal((N, nb))).astype(np.float32))
    elif fmt == "q6_K":
        out[..., 208:210] = _f16_bytes((scale * 0.02 * rng.standard_normal((N, nb))).astype(np.float32))
    elif fmt in ("mxfp8", "mxfp4"):
        out[..., 0] = rng.integers(110, 126, size=(N, nb), dtype=np.uint8)
    elif fmt == "nvfp4":
        out[..., 0] = rng.integers(0, 0x48, size=(N, nb), dtype=np.uint8) | (
            rng.integers(0, 2, size=(N, nb), dtype=np.uint8) << 7)
    return out


# ----------------------------------------------------------------------------------------------
# dtype rounding helpers (the kernels round exactly once, at the store).
# ----------------------------------------------------------------------------------------------
def round_bf16(v: np.ndarray) -> np.ndarray:
    """fp32 -> bf16 (round to nearest even) -> fp32."""
    b = np.ascontiguousarray(v, np.float32).view(np.uint32).astype(np.uint64)
    r = ((b + 0x7FFF + ((b >> 16) & 1)) >> 16) << 16
    out = (r & 0xFFFFFFFF).astype(np.uint32).view(np.float32)
    return np.where(np.isnan(v), v, out).astype(np.float32)


def round_to(v: np.ndarray, dtype: str) -> np.ndarray:
    v = np.asarray(v, np.float32)
    if dtype in ("bf16", "bfloat16"):
        return round_bf16(v)
    if dtype in ("f16", "float16"):
        return v.astype(np.float16).astype(np.float32)
    return v


# ----------------------------------------------------------------------------------------------
# Epilogue math.  kernels/matmul/decode_linear/decode_linear.metal:154-158,
# include/metal/common/glu_eval.metal:20-47
# ----------------------------------------------------------------------------------------------
def gelu_erf_as(v: np.ndarray) -> np.ndarray:
    """0.5*v*(1+erf(v/sqrt2)) with the 5-term Abramowitz-Stegun erf, all in fp32."""
    f = np.float32
    v = np.asarray(v, f)
    z = v * f(0.70710678118654752440)
    a = np.abs(z)
    t = f(1.0) / (f(1.0) + f(0.3275911) * a)
    poly = (((((f(1.061405429) * t + f(-1.453152027)) * t) + f(1.421413741)) * t
             + f(-0.284496736)) * t + f(0.254829592)) * t
    y = f(1.0) - poly * np.exp(-a * a).astype(f)
    erf = np.where(z < 0, -y, y).astype(f)
    return (f(0.5) * v * (f(1.0) + erf)).astype(f)


def silu(v: np.ndarray) -> np.ndarray:
    v = np.asarray(v, np.float32)
    return (v / (np.float32(1.0) + np.exp(-v).astype(np.float32))).astype(np.float32)


def _act(v, activation):
    if activation in (1, "gelu"):
        return gelu_erf_as(v)
    if activation in (2, "silu"):
        return silu(v)
    return np.asarray(v, np.float32)


def matmul_f64(x: np.ndarray, W: np.ndarray) -> np.ndarray:
    """x (M,K) @ W(N,K).T accumulated in float64, returned as fp32 (the dequantise-then-matmul
    oracle of tests/correctness/matmul/decode_linear/test_decode_linear.py:155-171)."""
    return (np.asarray(x, np.float64) @ np.asarray(W, np.float64).T).astype(np.float32)


def decode_linear_epilogue(x, packed, fmt, bias=None, residual=None, activation=0, dtype="f32"):
    """y = T(act(x.W^T + bias) + residual), fp32 throughout, one rounding to the I/O dtype.
    decode_linear.metal:349-377.  x/bias/residual hold values already rounded to `dtype`."""
    v = matmul_f64(x, dequantize(fmt, packed))
    if bias is not None:
        v = v + np.asarray(bias, np.float32)[None, :]
    v = _act(v.astype(np.float32), activation)
    if residual is not None:
        v = v + np.asarray(residual, np.float32)
    return round_to(v.astype(np.float32), dtype)


def decode_swiglu(x, gate_packed, up_packed, fmt, gate_bias=None, up_bias=None, dtype="f32"):
    """y = T(silu(gate.x+gb) * (up.x+ub)).  decode_linear.metal:417-446"""
    g = matmul_f64(x, dequantize(fmt, gate_packed))
    u = matmul_f64(x, dequantize(fmt, up_packed))
    if gate_bias is not None:
        g = g + np.asarray(gate_bias, np.float32)[None, :]
        u = u + np.asarray(up_bias, np.float32)[None, :]
    return round_to((silu(g) * u).astype(np.float32), dtype)


# ----------------------------------------------------------------------------------------------
# Runtime output quantizers.  kernels/quantization/quant_rt/quant_rt.metal:21-87, :266-306;
# encoders dequant.metal:321-353 (e4m3), :381-385 (int8)
# ----------------------------------------------------------------------------------------------
def e4m3_encode_device(x: np.ndarray) -> np.ndarray:
    """float -> e4m3 code with the DEVICE rule: halves round away from zero, saturate to 0x7E
    (448), magnitudes below 2^-10 give a signed zero code, NaN gives 0x7E."""
    x = np.ascontiguousarray(x, np.float32)
    sign = np.where(x < 0, 0x80, 0).astype(np.uint32)
    a = np.abs(x)
    bits = a.view(np.uint32)
    E = ((bits >> 23) & 0xFF).astype(np.int64) - 127
    frac = (bits & 0x7FFFFF).astype(np.int64)
    # normal branch
    mant = (frac + 0x80000) >> 20
    exp = E + 7
    carry = mant >= 8
    mant = np.where(carry, 0, mant)
    exp = np.where(carry, exp + 1, exp)
    normal = np.where((exp > 15) | ((exp >= 15) & (mant >= 7)), 0x7E, (exp << 3) | mant)
    # subnormal branch: round-half-away of a*512
    with np.errstate(invalid="ignore"):
        sm = np.floor(a.astype(np.float64) * 512.0 + 0.5)
    sm = np.where(np.isnan(sm), 0, sm).astype(np.int64)
    sub = np.where(sm <= 0, 0, np.where(sm >= 8, 8, sm))
    code = np.where(E < -6, sub, normal)
    code = np.where(a >= np.float32(448.0), 0x7E, code)
    code = np.where(np.isnan(x), 0x7E, code)
    return (sign | code.astype(np.uint32)).astype(np.uint8)


def _round_half_away(v):
    v = np.asarray(v, np.float64)
    return np.sign(v) * np.floor(np.abs(v) + 0.5)


def int8_encode(x: np.ndarray) -> np.ndarray:
    return np.clip(_round_half_away(np.asarray(x, np.float32)), -127, 127).astype(np.int8)


def quantize_per_token(y: np.ndarray, kind: str):
    """Per-row dynamic quantization of the (already dtype-rounded) output.  s = amax/448 or /127;
    inv = 1/s in fp32 (0 when s == 0); code = encode(y*inv).  Returns (codes, scale[rows])."""
    y = np.asarray(y, np.float32)
    amax = np.abs(y).max(-1).astype(np.float32)
    s = (amax / np.float32(448.0 if kind == "fp8" else 127.0)).astype(np.float32)
    with np.errstate(divide="ignore"):
        inv = np.where(s > 0, np.float32(1.0) / s, np.float32(0.0)).astype(np.float32)
    scaled = (y * inv[:, None]).astype(np.float32)
    codes = e4m3_encode_device(scaled) if kind == "fp8" else int8_encode(scaled)
    return codes, s


def quantize_mxfp8_rows(y: np.ndarray) -> np.ndarray:
    """(rows, D) -> MXFP8 blocks (rows, D/32, 33) = {e8m0; 32 e4m3 codes}.  Extension rule:
    s = 2^ceil(log2(amax/448)) when amax > 0 (quant_rt.metal:285-288 with G=32, ue8m0=1), stored
    as its biased exponent; an all-zero group stores exponent 127 (s = 1) and zero codes.
    Parity unpinned: no reference test fixes these bytes."""
    y = np.asarray(y, np.float32); R, D = y.shape
    assert D % 32 == 0
    g = y.reshape(R, D // 32, 32)
    amax = np.abs(g).max(-1).astype(np.float32)
    # exact ceil(log2(amax/448)) from the float's bits: amax/448 = m*2^e with m in [1,2)
    q = (np.maximum(amax, np.float32(1e-10)) / np.float32(448.0)).astype(np.float32)
    bits = q.view(np.uint32)
    e = ((bits >> 23) & 0xFF).astype(np.int32) - 127
    e = np.where((bits & 0x7FFFFF) != 0, e + 1, e)
    e = np.where(amax > 0, e, 0)
    code = np.clip(e + 127, 1, 254).astype(np.int32)
    s = e8m0_decode(code)
    inv = (np.float32(1.0) / s).astype(np.float32)
    out = np.zeros((R, D // 32, 33), np.uint8)
    out[..., 0] = code.astype(np.uint8)
    out[..., 1:] = e4m3_encode_device((g * inv[..., None]).astype(np.float32))
    return out


# ----------------------------------------------------------------------------------------------
# RNG.  include/metal/common/rng.metal:18-30; numpy twin
# tests/correctness/quantization/lm_head/test_lm_head.py:23-34
# ----------------------------------------------------------------------------------------------
def rng_uniform(seed, a, b) -> np.ndarray:
    M = np.uint64(0xFFFFFFFF)
    x = (np.uint64(int(seed) & 0xFFFFFFFF) * np.uint64(0x9E3779B9)
         + np.asarray(a, np.uint64) * np.uint64(0x85EBCA77)
         + np.asarray(b, np.uint64) * np.uint64(0xC2B2AE3D)) & M
    x ^= x >> np.uint64(16); x = (x * np.uint64(0x7FEB352D)) & M
    x ^= x >> np.uint64(15); x = (x * np.uint64(0x846CA68B)) & M
    x ^= x >> np.uint64(16)
    return (x >> np.uint64(8)).astype(np.float32) * np.float32(1.0 / 16777216.0)


def rng_gumbel(seed, a, b) -> np.ndarray:
    u = np.maximum(rng_uniform(seed, a, b), np.float32(1e-20))
    return (-np.log(-np.log(u))).astype(np.float32)


# ----------------------------------------------------------------------------------------------
# Fused LM-head sampling.  kernels/quantization/lm_head/lm_head.metal:219-278 (argmax /
# categorical), :444-470 + :579-616 (top-k), :478-529 + :649-702 (top-p); ordering helpers
# include/metal/ops/group/topk.metal:34-85 (value descending, id ascending).
# ----------------------------------------------------------------------------------------------
def lm_head_logits(h: np.ndarray, packed: np.ndarray, fmt: str, chunk_rows: int = 16384) -> np.ndarray:
    """Raw logits (T, V): float64 accumulation of the fp32-exact dequantised weights, rounded to
    fp32 (the tests' oracle, test_lm_head.py:132-154).  The vocabulary is walked in chunks so that
    a 128K-row head needs a few hundred MB of host memory, not the whole fp64 matrix."""
    V = packed.shape[0]
    if V <= chunk_rows:
        return matmul_f64(h, dequantize(fmt, packed))
    h64 = np.asarray(h, np.float64)
    out = np.empty((h64.shape[0], V), np.float32)
    for v0 in range(0, V, chunk_rows):
        W = dequantize(fmt, packed[v0:v0 + chunk_rows]).astype(np.float64)
        out[:, v0:v0 + chunk_rows] = (h64 @ W.T).astype(np.float32)
    return out


def _argmax_low_id(score: np.ndarray, ids: np.ndarray) -> int:
    """Largest score, ties -> smallest id.  Returns the id, or -1 if nothing is valid."""
    if score.size == 0:
        return -1
    best = score.max()
    return int(ids[score == best].min())


def _topk_desc(vals: np.ndarray, ids: np.ndarray, k: int):
    """First k of (value descending, id ascending)."""
    order = np.lexsort((ids, -vals.astype(np.float64)))[:k]
    return vals[order], ids[order]


def lm_head_sample_from_logits(logits, mode, k=0, temperature=1.0, seed=0, top_p=0.9, bias=None,
                               vocab_offset=0, return_detail=False):
    """Token id per row from fp32 raw logits (T, V) holding dot(W[v], h[t]).

    mode 0 argmax / 1 categorical: score = dot*invtemp (+bias) (+gumbel); the bias is added AFTER
    the temperature scale (lm_head.metal:268-270).  mode 2 top-k: raw = dot(+bias); the k largest,
    then Gumbel-max of raw*invtemp + g.  mode 3 top-p: per 256-row vocab tile the top-k pool and the
    tile log-sum-exp of raw*invtemp; bisection of a threshold against the full-vocab normalizer;
    Gumbel-max over the surviving pool entries; -1 when nothing survives.  All fp32.
    `vocab_offset` shifts local row numbers to global ids (RNG key and tie-break use global ids).
    With return_detail, also returns the winning margin per row (gap between the best and the
    second-best perturbed score), which tests use to tell real mismatches from fp32 near-ties."""
    f = np.float32
    L = np.asarray(logits, f)
    T, V = L.shape
    ids = np.arange(V, dtype=np.int64) + int(vocab_offset)
    invtemp = f(1.0) / f(temperature)
    out = np.zeros(T, np.int32)
    margin = np.full(T, np.inf)
    b = None if bias is None else np.asarray(bias, f)

    def pick(score, cand_ids, t):
        if score.size == 0:
            out[t] = -1
            return
        out[t] = _argmax_low_id(score, cand_ids)
        if score.size > 1:
            top2 = np.partition(score.astype(np.float64), -2)[-2:]
            margin[t] = float(top2[1] - top2[0])

    for t in range(T):
        row = L[t]
        if mode in (0, 1):
            s = (row * invtemp).astype(f)
            if b is not None:
                s = (s + b).astype(f)
            if mode == 1:
                s = (s + rng_gumbel(seed, t, ids)).astype(f)
            pick(s, ids, t)
            continue
        raw = row if b is None else (row + b).astype(f)
        if mode == 2:
            tv, ti = _topk_desc(raw, ids, k)
            s = ((tv * invtemp).astype(f) + rng_gumbel(seed, t, ti)).astype(f)
            pick(s, ti, t)
            if V > k:  # membership margin: gap between rank k and rank k+1
                srt = np.sort(raw.astype(np.float64))[::-1]
                margin[t] = min(margin[t], float(srt[k - 1] - srt[k]))
            continue
        # mode 3
        pv, pi, lses = [], [], []
        for v0 in range(0, V, TILE_V):
            seg = raw[v0:v0 + TILE_V]
            tv, ti = _topk_desc(seg, ids[v0:v0 + TILE_V], k)
            pv.append(tv); pi.append(ti)
            tl = (seg * invtemp).astype(f)
            m = tl.max()
            lses.append(f(m + np.log(np.exp((tl - m).astype(f)).astype(f).sum(dtype=f))))
        pv = np.concatenate(pv); pi = np.concatenate(pi); lses = np.array(lses, f)
        ls = (pv * invtemp).astype(f)
        mx = ls.max()
        Z = np.exp((lses - mx).astype(f)).astype(f).sum(dtype=f)
        lo, hi = f(mx - f(40.0)), f(mx)
        for _ in range(32):
            mid = f(f(0.5) * f(lo + hi))
            sm = np.exp((ls[ls >= mid] - mx).astype(f)).astype(f).sum(dtype=f) / Z
            if sm >= f(top_p):
                lo = mid
            else:
                hi = mid
        keep = ls >= lo
        s = (ls[keep] + rng_gumbel(seed, t, pi[keep])).astype(f)
        pick(s, pi[keep], t)
        # threshold margin: distance of the nearest pool entry to the cut
        if keep.any() and (~keep).any():
            margin[t] = min(margin[t], float(ls[keep].min() - ls[~keep].max()))
    if return_detail:
        return out, margin
    return out


def lm_head_sample(h, packed, fmt, mode, k=0, temperature=1.0, seed=0, top_p=0.9, bias=None,
                   return_detail=False):
    """The reference composition: dequantise, project, sample (tk/__init__.py:2357-2412)."""
    return lm_head_sample_from_logits(lm_head_logits(h, packed, fmt), mode, k, temperature, seed,
                                      top_p, bias, 0, return_detail)


# ----------------------------------------------------------------------------------------------
# Vocabulary-sharded form of the fused sampler (no reference counterpart: the reference is single
# device).  A shard emits, per hidden row, the candidates its 256-row tiles would hand to the
# reference's reduce kernels; the merge over shards applies the same reduce rules to the union.
# Because max-with-lowest-id, top-k-of-top-k and sum-of-exp are associative, merge(shards) must
# equal lm_head_sample_from_logits on the concatenated logits - which is what the tests check.
# ----------------------------------------------------------------------------------------------
def lm_head_shard_candidates(logits_local, mode, k=0, temperature=1.0, seed=0, bias_local=None,
                             vocab_offset=0, max_tiles=None):
    """(val (T,C), id (T,C), lse (T,L)) for rows [vocab_offset, vocab_offset+V_local).  Absent
    slots: id -1 / value NEG_INF; absent tiles: lse NEG_INF.  C = 1 (modes 0/1), k (mode 2),
    max_tiles*k (mode 3)."""
    f = np.float32
    L = np.asarray(logits_local, f)
    T, V = L.shape
    ids = np.arange(V, dtype=np.int64) + int(vocab_offset)
    invtemp = f(1.0) / f(temperature)
    tiles = (V + TILE_V - 1) // TILE_V
    max_tiles = tiles if max_tiles is None else max_tiles
    b = None if bias_local is None else np.asarray(bias_local, f)
    C = 1 if mode <= 1 else (k if mode == 2 else max_tiles * k)
    val = np.full((T, C), NEG_INF, f)
    idx = np.full((T, C), -1, np.int32)
    lse = np.full((T, max_tiles if mode == 3 else 0), NEG_INF, f)
    for t in range(T):
        row = L[t]
        if mode <= 1:
            s = (row * invtemp).astype(f)
            if b is not None:
                s = (s + b).astype(f)
            if mode == 1:
                s = (s + rng_gumbel(seed, t, ids)).astype(f)
            w = _argmax_low_id(s, ids)
            val[t, 0], idx[t, 0] = s[w - int(vocab_offset)], w
            continue
        raw = row if b is None else (row + b).astype(f)
        if mode == 2:
            tv, ti = _topk_desc(raw, ids, k)
            val[t, :tv.size], idx[t, :ti.size] = tv, ti
            continue
        for j, v0 in enumerate(range(0, V, TILE_V)):
            seg = raw[v0:v0 + TILE_V]
            tv, ti = _topk_desc(seg, ids[v0:v0 + TILE_V], k)
            val[t, j * k:j * k + tv.size], idx[t, j * k:j * k + ti.size] = tv, ti
            tl = (seg * invtemp).astype(f)
            m = tl.max()
            lse[t, j] = f(m + np.log(np.exp((tl - m).astype(f)).astype(f).sum(dtype=f)))
    return val, idx, lse


def lm_head_merge_candidates(vals, idxs, lses, mode, k=0, temperature=1.0, seed=0, top_p=0.9):
    """Stage 2 over the shards' candidates (lists of the arrays above, one entry per shard)."""
    f = np.float32
    val = np.concatenate(vals, axis=1); idx = np.concatenate(idxs, axis=1).astype(np.int64)
    lse = np.concatenate(lses, axis=1) if mode == 3 else None
    T = val.shape[0]
    invtemp = f(1.0) / f(temperature)
    out = np.zeros(T, np.int32)
    for t in range(T):
        ok = idx[t] >= 0
        v, i = val[t][ok], idx[t][ok]
        if mode <= 1:
            out[t] = _argmax_low_id(v, i)
        elif mode == 2:
            tv, ti = _topk_desc(v, i, k)
            s = ((tv * invtemp).astype(f) + rng_gumbel(seed, t, ti)).astype(f)
            out[t] = _argmax_low_id(s, ti)
        else:
            ls = (v * invtemp).astype(f)
            mx = ls.max()
            tl = lse[t][lse[t] > NEG_INF]
            Z = np.exp((tl - mx).astype(f)).astype(f).sum(dtype=f)
            lo, hi = f(mx - f(40.0)), f(mx)
            for _ in range(32):
                mid = f(f(0.5) * f(lo + hi))
                sm = np.exp((ls[ls >= mid] - mx).astype(f)).astype(f).sum(dtype=f) / Z
                if sm >= f(top_p):
                    lo = mid
                else:
                    hi = mid
            keep = ls >= lo
            s = (ls[keep] + rng_gumbel(seed, t, i[keep])).astype(f)
            out[t] = _argmax_low_id(s, i[keep]) if keep.any() else -1
    return out


# ----------------------------------------------------------------------------------------------
# LM-head forms that return log-probabilities: masked top-k, CSR candidates, beam advance.
# Restated from the reference's own test oracles (tests/correctness/quantization/lm_head/
# test_lm_head.py:370-388 `_packed_allow_mask` / `_topk_logprobs`, :496-510 beam search) and kernels
# (kernels/quantization/lm_head/lm_head.metal:1152-1425, :534-573; sampling.metal:432-458).
# ----------------------------------------------------------------------------------------------
def packed_allow_mask(rows, vocab: int) -> np.ndarray:
    """(T, ceil(V/32)) uint32: bit (v & 31) of word v >> 5 admits token v (test_lm_head.py:370-375)."""
    mask = np.zeros((len(rows), (vocab + 31) // 32), dtype=np.uint32)
    for t, allowed in enumerate(rows):
        for v in allowed:
            mask[t, v // 32] |= np.uint32(1 << (v % 32))
    return mask


def topk_logprobs(logits_row: np.ndarray, candidates, topk: int, normalizer_ids=None):
    """Top-k of the listed tokens by (logit desc, id asc) with logprob = logit - log-sum-exp over the
    listed tokens (or over normalizer_ids); ids outside [0, V) are skipped; short rows are padded
    with id -1 / -inf (test_lm_head.py:378-388)."""
    V = logits_row.shape[0]
    valid = np.array([v for v in candidates if 0 <= v < V], dtype=np.int64)
    out_ids = np.full(topk, -1, np.int32)
    out_lp = np.full(topk, -np.inf, np.float32)
    if valid.size == 0:
        return out_ids, out_lp
    order = np.lexsort((valid, -logits_row[valid].astype(np.float64)))[:topk]
    sel = valid[order]
    norm = valid if normalizer_ids is None else np.asarray(normalizer_ids, np.int64)
    vals = logits_row[norm].astype(np.float64)
    m = vals.max()
    lse = m + np.log(np.exp(vals - m).sum())
    out_ids[:sel.size] = sel
    out_lp[:sel.size] = (logits_row[sel].astype(np.float64) - lse).astype(np.float32)
    return out_ids, out_lp


def lm_head_masked_from_logits(logits: np.ndarray, allowed_rows, topk: int, normalize: str = "allowed"):
    """(ids (T,k), logprobs (T,k)) of tk.lm_head_masked on raw logits (bias already added)."""
    T, V = logits.shape
    full = np.arange(V) if normalize == "full" else None
    out = [topk_logprobs(logits[t], allowed_rows[t], topk, full) for t in range(T)]
    return np.stack([o[0] for o in out]), np.stack([o[1] for o in out])


def lm_head_candidates_from_logits(logits: np.ndarray, candidate_ids, offsets, topk: int):
    """(ids, logprobs) of tk.lm_head_candidates: row t lists candidate_ids[offsets[t]:offsets[t+1]]."""
    T = logits.shape[0]
    out = [topk_logprobs(logits[t], list(candidate_ids[offsets[t]:offsets[t + 1]]), topk) for t in range(T)]
    return np.stack([o[0] for o in out]), np.stack([o[1] for o in out])


def lm_head_beam_advance_from_logits(logits: np.ndarray, cum: np.ndarray, beam_width: int):
    """One exact beam-search step (test_lm_head.py:496-510): log-softmax per beam row, add the beam's
    cumulative score, take the beam_width best of beam_width * V per batch (stable: ties to the lower
    flat index).  Returns (token (B,BM), parent (B,BM), score (B,BM))."""
    B, BM = cum.shape
    V = logits.shape[1]
    L = logits.astype(np.float64)
    m = L.max(axis=1, keepdims=True)
    log_z = m + np.log(np.exp(L - m).sum(axis=1, keepdims=True))
    flat = (L - log_z).reshape(B, BM, V) + cum.astype(np.float64)[:, :, None]
    flat = flat.reshape(B, BM * V)
    sel = np.argsort(-flat, axis=1, kind="stable")[:, :BM]
    return (sel % V).astype(np.int32), (sel // V).astype(np.int32), np.take_along_axis(flat, sel, axis=1).astype(np.float32)


# ----------------------------------------------------------------------------------------------
# Norm / activation -> quantiser seams.  kernels/norms/add_norm/add_norm.metal:26-65, :181-392;
# kernels/quantization/act_quant/act_quant.metal:26-160; include/metal/common/glu_eval.metal:49-66.
# ----------------------------------------------------------------------------------------------
def rms_norm_add(x, residual, weight, eps=1e-5, dtype="bf16"):
    """(normalised fp32 row values BEFORE any rounding, x + residual rounded to dtype).  The norm runs
    on the unrounded fp32 sum: n = ((x + r) * rsqrt(mean((x + r)^2) + eps)) * w."""
    h = (np.asarray(x, np.float32) + np.asarray(residual, np.float32)).astype(np.float32)
    ms = (h.astype(np.float64) ** 2).mean(axis=-1, keepdims=True)
    inv = (1.0 / np.sqrt(ms + eps)).astype(np.float32)
    n = ((h * inv).astype(np.float32) * np.asarray(weight, np.float32)).astype(np.float32)
    return n, round_to(h, dtype)


def gated_act(act: str, x, gate, alpha=1.702, limit=7.0):
    """swiglu: silu(x) * gate; swiglu_oai: x' = min(x, limit), g' = clip(gate, +-limit),
    x' * sigmoid(alpha x') * (1 + g')  (tests/correctness/quantization/act_quant/test_act_quant.py:19-26)."""
    x = np.asarray(x, np.float64); g = np.asarray(gate, np.float64)
    if act == "swiglu_oai":
        x = np.minimum(x, limit); g = np.clip(g, -limit, limit)
        return ((x / (1.0 + np.exp(-x * alpha))) * (1.0 + g)).astype(np.float32)
    return ((x / (1.0 + np.exp(-x))) * g).astype(np.float32)


def quantize_groups(v: np.ndarray, group: int, kind: str = "fp8", ue8m0: bool = False):
    """Per group of `group` columns: s = amax / qmax (fp8, ue8m0: 2^ceil(log2(max(amax, 1e-10) / 448))
    when amax > 0); inv = 1/s (0 when s == 0); codes = encode(v * inv).  Returns (codes, scale (.., D/G)).
    group == D gives the per-row quantisers."""
    f = np.float32
    v = np.asarray(v, f)
    D = v.shape[-1]
    b = v.reshape(v.shape[:-1] + (D // group, group))
    amax = np.abs(b).max(-1)
    qmax = f(448.0) if kind == "fp8" else f(127.0)
    s = (amax / qmax).astype(f)
    if ue8m0 and kind == "fp8":
        q = (np.maximum(amax, f(1e-10)) / qmax).astype(f)
        e = np.ceil(np.log2(q.astype(np.float64)))
        s = np.where(amax > 0, np.exp2(e), s).astype(f)
    with np.errstate(divide="ignore"):
        inv = np.where(s > 0, (f(1.0) / s).astype(f), f(0.0)).astype(f)
    scaled = (b * inv[..., None]).astype(f)
    codes = e4m3_encode_device(scaled) if kind == "fp8" else int8_encode(scaled)
    return codes.reshape(v.shape), s


# ----------------------------------------------------------------------------------------------
# BaseQN: codes, scales and biases in separate planes.  kernels/quantization/base_q/README.md:8-27,
# bindings/python/tk/base_q.py:25-154, kernels/quantization/base_q/base_q.metal:8-41
# ----------------------------------------------------------------------------------------------
BASE_Q_BITS = (2, 3, 4, 5, 6, 8)
BASE_Q_GROUPS = (32, 64, 128)


def base_q_pack(codes: np.ndarray, bits: int) -> np.ndarray:
    """Lane c of a row occupies bits [c*bits, (c+1)*bits) of the row's little-endian bit string
    (bit i of the string is bit i%8 of byte i//8).  base_q.py:25-47"""
    v = np.asarray(codes).astype(np.uint32)
    if bits not in BASE_Q_BITS or (v.shape[-1] * bits) % 8:
        raise ValueError("BaseQN: bits in {2,3,4,5,6,8} and a byte-aligned row")
    if v.size and int(v.max()) >= (1 << bits):
        raise ValueError("BaseQN: code out of range")
    bit = ((v[..., None] >> np.arange(bits, dtype=np.uint32)) & 1).astype(np.uint8)
    return np.packbits(bit.reshape(v.shape[:-1] + (-1,)), axis=-1, bitorder="little")


def base_q_unpack(packed: np.ndarray, bits: int, columns: int | None = None) -> np.ndarray:
    """Inverse of base_q_pack.  base_q.py:50-76, base_q.metal:8-18"""
    p = np.asarray(packed, np.uint8)
    if columns is None:
        columns = p.shape[-1] * 8 // bits
    if columns * bits != p.shape[-1] * 8:
        raise ValueError("BaseQN: columns * bits must equal packed bytes * 8")
    bit = np.unpackbits(p, axis=-1, bitorder="little").reshape(p.shape[:-1] + (columns, bits))
    return (bit.astype(np.uint32) << np.arange(bits, dtype=np.uint32)).sum(-1).astype(np.uint8)


def base_q_scale_values(plane: np.ndarray, scale_dtype: str) -> np.ndarray:
    """Scale / bias plane -> fp32.  uint16 input = raw bf16 / f16 bits.  base_q.py:104-116,
    base_q.metal:20-26"""
    a = np.asarray(plane)
    name = {"bfloat16": "bf16", "float16": "f16"}.get(str(scale_dtype).lower(), str(scale_dtype).lower())
    if name == "bf16":
        return (a.astype(np.uint32) << np.uint32(16)).view(np.float32) if a.dtype == np.uint16 else a.astype(np.float32)
    if name == "f16":
        return (a.view(np.float16) if a.dtype == np.uint16 else a.astype(np.float16)).astype(np.float32)
    if name == "e8m0":
        return e8m0_decode(a)
    if name == "e4m3":
        return e4m3_decode(a)
    raise ValueError("BaseQN: scale_dtype must be bf16, f16, e8m0 or e4m3")


def base_q_dequantize(packed, scales, biases, bits, group, scale_dtype="bf16", symmetric=False) -> np.ndarray:
    """fp32 weights (.., K): asymmetric fl(fl(code * scale) + bias), symmetric
    (code - 2^(bits-1)) * scale, one scale (and bias) per `group` columns.  base_q.py:119-154,
    base_q.metal:28-41"""
    if group not in BASE_Q_GROUPS:
        raise ValueError("BaseQN: group_size must be 32, 64 or 128")
    if str(scale_dtype).lower() == "e4m3" and bits != 8:
        raise ValueError("BaseQN: e4m3 scale storage is valid only for q8")       # base_q_descriptor.h:64-66
    s = base_q_scale_values(scales, scale_dtype)
    K = s.shape[-1] * group
    c = base_q_unpack(packed, bits, K)
    se = np.repeat(s, group, axis=-1)
    if symmetric:
        return ((c.astype(np.int32) - (1 << (bits - 1))).astype(np.float32) * se).astype(np.float32)
    if biases is None:
        raise ValueError("BaseQN: biases are required for asymmetric tensors")
    b = np.repeat(base_q_scale_values(biases, scale_dtype), group, axis=-1)
    return ((c.astype(np.float32) * se).astype(np.float32) + b).astype(np.float32)


def base_q_random_planes(rows, K, bits, group, scale_dtype, symmetric, seed, lead=()):
    """Seeded planes in storage form: (codes uint8, scales, biases or None).  bf16 / f16 planes are
    returned as raw uint16 bits, e8m0 / e4m3 as uint8."""
    rng = np.random.default_rng(seed)
    shape = tuple(lead) + (rows,)
    codes = base_q_pack(rng.integers(0, 1 << bits, size=shape + (K,), dtype=np.uint8), bits)
    G = K // group

    def plane(lo, hi):
        v = (lo + (hi - lo) * rng.random(shape + (G,))).astype(np.float32)
        if scale_dtype == "bf16":
            return (round_bf16(v).view(np.uint32) >> np.uint32(16)).astype(np.uint16)
        if scale_dtype == "f16":
            return v.astype(np.float16).view(np.uint16)
        if scale_dtype == "e8m0":
            return rng.integers(118, 124, size=v.shape, dtype=np.uint8)          # 2^-9 .. 2^-4
        sign = (rng.random(v.shape) < (0.5 if lo < 0 else 0.0)).astype(np.uint8) << 7
        return (rng.integers(0x08, 0x30, size=v.shape, dtype=np.uint8) | sign).astype(np.uint8)
    scales = plane(0.002, 0.02)
    biases = None if symmetric else plane(-0.05, 0.05)
    return codes, scales, biases


def base_q_matmul(W: np.ndarray, x: np.ndarray, dtype: str) -> np.ndarray:
    """dequant(W) (N, K) @ x (K, M), float64 accumulation, rounded to the activation dtype.
    base_q.metal:93-115,222-249"""
    return round_to((W.astype(np.float64) @ np.asarray(x, np.float64)).astype(np.float32), dtype)


def base_q_swiglu(Wg: np.ndarray, Wu: np.ndarray, x: np.ndarray, dtype: str) -> np.ndarray:
    """silu(Wg @ x) * (Wu @ x) with one final rounding.  base_q.metal:165-220"""
    g = Wg.astype(np.float64) @ np.asarray(x, np.float64)
    u = Wu.astype(np.float64) @ np.asarray(x, np.float64)
    return round_to(((g / (1.0 + np.exp(-g))) * u).astype(np.float32), dtype)


def base_q_embedding(W: np.ndarray, ids: np.ndarray, dtype: str) -> np.ndarray:
    """Rows of W by id; a negative or out-of-range id gives a zero row.  README.md:24-27"""
    ids = np.asarray(ids, np.int64)
    ok = (ids >= 0) & (ids < W.shape[0])
    out = np.where(ok[..., None], W[np.where(ok, ids, 0)], np.float32(0.0))
    return round_to(out.astype(np.float32), dtype)


def base_q_lm_head_argmax(W: np.ndarray, x: np.ndarray, dtype: str):
    """Greedy ids over logits rounded to the activation dtype, lowest id on exact ties; also
    returns per column the gap between the two largest float64 logits.  README.md:43-47"""
    logits = W.astype(np.float64) @ np.asarray(x, np.float64)                     # (V, batch)
    r = round_to(logits.astype(np.float32), dtype)
    top2 = np.sort(logits, axis=0)[-2:]
    return np.argmax(r, axis=0).astype(np.int32), (top2[1] - top2[0]), r
