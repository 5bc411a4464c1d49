"""`tk_torch`-compatible binding for CUDA tensors on B200.

Same function names, positional arguments and error behaviour (RuntimeError with the reference's
message text) as the reference's PyTorch-MPS module for the decode-projection path
(bindings/pytorch_mps/tk_torch/__init__.py:932-958, :1738-1745), so the reference's Python router
`tk` can call it unchanged when handed CUDA tensors.  Every function enqueues on torch's current
CUDA stream through the C ABI of libquixicore_cuda.so; torch only provides device memory and the
stream.  There is no eager / CPU fallback: a missing library or a non-CUDA tensor raises.
"""
from __future__ import annotations

import contextlib

import torch

from . import _lib

_DT = {torch.float32: _lib.DTYPE_F32, torch.float16: _lib.DTYPE_F16, torch.bfloat16: _lib.DTYPE_BF16}
_BLOCK = {"q4_0": (32, 18), "q8_0": (32, 34), "q6_K": (256, 210), "mxfp8": (32, 33),
          "nvfp4": (16, 9), "mxfp4": (32, 17)}


_raw_stream = getattr(torch._C, "_cuda_getCurrentRawStream", None)
_NULL_GUARD = contextlib.nullcontext()


def _stream() -> int:
    """Handle of torch's current stream on the current device (without building a Stream object: the
    call is on the path of every eager operator, where a few microseconds of host time are visible)."""
    if _raw_stream is not None:
        return _raw_stream(torch.cuda.current_device())
    return torch.cuda.current_stream().cuda_stream


def _guard(device):
    """Context that makes `device` current; free when it already is."""
    if torch.cuda.current_device() == device.index:
        return _NULL_GUARD
    return torch.cuda.device(device)


def _ptr(t) -> int:
    return 0 if t is None else t.data_ptr()


def _check(cond: bool, msg: str) -> None:
    if not cond:
        raise RuntimeError(msg)


def _same_device(name: str, first, *others) -> None:
    """Every tensor of a call must live on the device of its first operand: the kernels run on that
    device and build TMA descriptors over the raw pointers, so a tensor from another GPU would be
    an illegal address (or a silent peer read).  Placeholders passed for absent operands count too."""
    for t in others:
        if t is not None and t.device != first.device:
            raise RuntimeError(f"{name}: all tensors must be on the same device "
                               f"(got {first.device} and {t.device})")


_WS = {}


def _workspace(device, nbytes: int):
    """Scratch tensor for calls on the current stream of `device`, reused by later calls on the same
    stream (they are ordered, so sharing it is safe) and grown geometrically."""
    key = (device.index, _raw_stream(device.index) if _raw_stream is not None
           else torch.cuda.current_stream(device).cuda_stream)
    ws = _WS.get(key)
    if ws is None or ws.numel() < nbytes:
        size = max(int(nbytes), 1 << 20, 0 if ws is None else 2 * ws.numel())
        ws = torch.empty((size,), dtype=torch.uint8, device=device)
        _WS[key] = ws       # a smaller predecessor stays alive while enqueued work may read it:
        #                     the caching allocator only reuses its block for this same stream
    return ws


def _check_weight(x, weight, fmt: str, name: str) -> int:
    """The reference's check_decode_epilogue_weight (torch_kernels.mm:6376-6405) for CUDA."""
    _check(x.is_cuda and weight.is_cuda and x.dtype in _DT and x.dim() == 2 and x.size(0) > 0
           and x.size(1) > 0, f"{name}: x must be non-empty (B,K) fp32/fp16/bf16")
    _check(fmt in _BLOCK, f"{name}: format must be q4_0, q8_0, q6_K, mxfp8, nvfp4, or mxfp4 "
           "(dense weights are routed to the framework matmul, not to this backend)")
    bk, bb = _BLOCK[fmt]
    K = x.size(1)
    _check(weight.dtype == torch.uint8 and weight.dim() == 3 and weight.size(0) > 0 and K % bk == 0
           and weight.size(1) == K // bk and weight.size(2) == bb,
           f"{name}: packed weight must be uint8 (N,K/block_k,block_bytes)")
    return weight.size(0)


def _quant_outputs(x, B, N, output_quant):
    """Buffers for a fused output quantisation: (kind, codes, scale)."""
    kind = _lib.OUT_QUANT.get(output_quant, -1)
    _check(kind >= 0, "output_quant must be None, 'fp8', 'int8', or 'mxfp8'")
    if kind == 0:
        return 0, None, None
    if kind == 3:
        _check(N % 32 == 0, "output_quant='mxfp8' needs N to be a multiple of 32")
        return 3, torch.empty((B, N // 32, 33), dtype=torch.uint8, device=x.device), None
    codes = torch.empty((B, N), dtype=torch.uint8 if kind == 1 else torch.int8, device=x.device)
    return kind, codes, torch.empty((B,), dtype=torch.float32, device=x.device)


def _quant_result(out, kind, codes, scale, with_output=False):
    if kind == 0:
        return out
    q = codes if kind == 3 else (codes, scale)
    return (out, q) if with_output else q


def decode_linear_epilogue(x, weight, bias, residual, format="", activation=0,
                           use_bias=False, use_residual=False, *, output_quant=None,
                           with_output=False):
    """Packed decode linear with fused bias, activation and residual; returns (B,N) in x.dtype.
    Absent bias / residual are passed as placeholders and ignored when their flag is false.
    output_quant (keyword only, not in the reference's positional signature): 'fp8' / 'int8' return
    (codes, scale) of the per-token quantizer applied to the rounded output, 'mxfp8' the packed
    MXFP8 rows, all inside the same call; with_output=True returns (output, quantised) instead, the
    x.dtype output being the one the codes were made from."""
    fmt, activation = str(format), int(activation)
    _check(0 <= activation <= 2, "decode_linear_epilogue: activation must be 0, 1, or 2")
    N = _check_weight(x, weight, fmt, "decode_linear_epilogue")
    _same_device("decode_linear_epilogue", x, weight, bias if use_bias else None,
                 residual if use_residual else None)
    B, K = x.shape
    _check(not use_bias or (bias.is_cuda and bias.dim() == 1 and bias.size(0) == N
                            and bias.dtype == x.dtype),
           "decode_linear_epilogue: bias must be (N,) with x dtype")
    _check(not use_residual or (residual.is_cuda and residual.dim() == 2 and residual.size(0) == B
                                and residual.size(1) == N and residual.dtype == x.dtype),
           "decode_linear_epilogue: residual must be (B,N) with x dtype")
    with _guard(x.device):
        xc, wc = x.contiguous(), weight.contiguous()
        bc = bias.contiguous() if use_bias else None
        rc = residual.contiguous() if use_residual else None
        out = torch.empty((B, N), dtype=x.dtype, device=x.device)
        kind, codes, scale = _quant_outputs(x, B, N, output_quant)
        _lib.check(_lib.lib().qx_cuda_decode_linear_epilogue(
            _stream(), _ptr(xc), _ptr(wc), _ptr(bc), _ptr(rc), _ptr(out), B, K, N, fmt.encode(),
            _DT[x.dtype], activation, int(bool(use_bias)), int(bool(use_residual)),
            kind, _ptr(codes), _ptr(scale), None, 0))
    return _quant_result(out, kind, codes, scale, with_output)


def decode_linear_partial(x, weight, format):
    """fp32 (B,N) raw projection x @ dequant(weight).T with no epilogue: one rank's share of a
    row-parallel (K-split) linear, summed over ranks by the caller."""
    fmt = str(format)
    N = _check_weight(x, weight, fmt, "decode_linear_partial")
    _same_device("decode_linear_partial", x, weight)
    B, K = x.shape
    with _guard(x.device):
        xc, wc = x.contiguous(), weight.contiguous()
        out = torch.empty((B, N), dtype=torch.float32, device=x.device)
        _lib.check(_lib.lib().qx_cuda_decode_linear_partial(
            _stream(), _ptr(xc), _ptr(wc), _ptr(out), B, K, N, fmt.encode(), _DT[x.dtype], None, 0))
    return out


def decode_swiglu(x, gate_weight, up_weight, gate_bias, up_bias, format="", use_bias=False, *,
                  output_quant=None, with_output=False):
    """Packed gate/up decode projections with fused SwiGLU: silu(gate.x+gb) * (up.x+ub).
    output_quant: as in decode_linear_epilogue."""
    fmt = str(format)
    N = _check_weight(x, gate_weight, fmt, "decode_swiglu")
    up_N = _check_weight(x, up_weight, fmt, "decode_swiglu")
    _check(up_N == N and up_weight.shape == gate_weight.shape,
           "decode_swiglu: gate and up weights must have identical shapes")
    _same_device("decode_swiglu", x, gate_weight, up_weight, gate_bias if use_bias else None,
                 up_bias if use_bias else None)
    _check(not use_bias or (gate_bias.is_cuda and up_bias.is_cuda and gate_bias.dtype == x.dtype
                            and up_bias.dtype == x.dtype and gate_bias.dim() == 1
                            and up_bias.dim() == 1 and gate_bias.size(0) == N
                            and up_bias.size(0) == N),
           "decode_swiglu: both biases must be (N,) with x dtype")
    B, K = x.shape
    with _guard(x.device):
        xc, gc, uc = x.contiguous(), gate_weight.contiguous(), up_weight.contiguous()
        gb = gate_bias.contiguous() if use_bias else None
        ub = up_bias.contiguous() if use_bias else None
        out = torch.empty((B, N), dtype=x.dtype, device=x.device)
        kind, codes, scale = _quant_outputs(x, B, N, output_quant)
        _lib.check(_lib.lib().qx_cuda_decode_swiglu(
            _stream(), _ptr(xc), _ptr(gc), _ptr(uc), _ptr(gb), _ptr(ub), _ptr(out), B, K, N,
            fmt.encode(), _DT[x.dtype], int(bool(use_bias)), kind, _ptr(codes), _ptr(scale), None, 0))
    return _quant_result(out, kind, codes, scale, with_output)


def _quantize_per_token(x, kind: int, name: str):
    _check(x.is_cuda and x.dtype in _DT and x.dim() >= 1 and x.numel() > 0,
           f"{name}: x must be a non-empty CUDA fp32/fp16/bf16 tensor")
    D = x.size(-1)
    rows = x.numel() // D
    with _guard(x.device):
        xc = x.contiguous()
        codes = torch.empty(x.shape, dtype=torch.uint8 if kind == 0 else torch.int8, device=x.device)
        scale = torch.empty(x.shape[:-1], dtype=torch.float32, device=x.device)
        _lib.check(_lib.lib().qx_cuda_quantize_per_token(
            _stream(), _ptr(xc), _ptr(codes), _ptr(scale), rows, D, _DT[x.dtype], kind))
    return codes, scale


def quantize_per_token_fp8(x):
    """Per-row fp8 e4m3 quant. Returns (codes uint8, scale f32), scale = absmax/448."""
    return _quantize_per_token(x, 0, "quantize_per_token_fp8")


def quantize_per_token_int8(x):
    """Per-row symmetric int8 quant. Returns (codes int8, scale f32), scale = absmax/127."""
    return _quantize_per_token(x, 1, "quantize_per_token_int8")


def quantize_mxfp8_rows(x):
    """(rows, D) -> packed MXFP8 blocks (rows, D/32, 33): e8m0 exponent + 32 e4m3 codes, the
    block layout the mxfp8 weight format uses.  Extension over the reference's per-token
    output_quant: the per-group rule with G = 32 and power-of-two scales."""
    _check(x.is_cuda and x.dtype in _DT and x.dim() == 2 and x.size(1) % 32 == 0 and x.numel() > 0,
           "quantize_mxfp8_rows: x must be CUDA (rows, D) fp32/fp16/bf16 with D % 32 == 0")
    rows, D = x.shape
    with _guard(x.device):
        xc = x.contiguous()
        blocks = torch.empty((rows, D // 32, 33), dtype=torch.uint8, device=x.device)
        _lib.check(_lib.lib().qx_cuda_quantize_mxfp8_rows(
            _stream(), _ptr(xc), _ptr(blocks), rows, D, _DT[x.dtype]))
    return blocks


def _check_lm_head(h, Wq, bias, V, K, fmt, mode, topk, temperature, top_p):
    _check(h.is_cuda and Wq.is_cuda and (bias is None or bias.is_cuda) and h.dtype in _DT,
           "lm_head_sample_q: inputs must be CUDA and h must be floating point")
    _same_device("lm_head_sample_q", h, Wq, bias if (bias is not None and bias.numel() > 1) else None)
    _check(h.dim() == 2 and h.size(1) == K, "lm_head_sample_q: h must be (T, K)")
    _check(0 <= mode <= 3, "lm_head_sample_q: mode 0=argmax, 1=categorical, 2=topk, 3=topp")
    _check(temperature > 0.0, "lm_head_sample_q: temperature must be positive")
    _check(fmt in _BLOCK, "lm_head_sample_q: format must be q8_0, q4_0, q6_K, mxfp8, nvfp4, or mxfp4")
    bk, bb = _BLOCK[fmt]
    _check(K % bk == 0 and Wq.dtype == torch.uint8 and Wq.dim() == 3 and Wq.size(0) == V
           and Wq.size(1) == K // bk and Wq.size(2) == bb,
           "lm_head_sample_q: packed weight shape does not match V/K/format")
    _check(h.size(0) > 0 and V > 0 and K > 0, "lm_head_sample_q: T, V, and K must be positive")
    if mode in (2, 3):
        _check(1 <= topk <= 64, "lm_head_sample_q: k must be in [1, 64]")
        _check(mode != 3 or 0.0 < top_p <= 1.0, "lm_head_sample_q: topp requires top_p in (0, 1]")


def lm_head_sample_q(h, Wq, bias, V, K, fmt, mode, topk, temperature, seed, top_p=0.0):
    """Fused LM head + sampling over packed weights; logits are never written to memory.
    mode 0 argmax, 1 categorical, 2 top-k, 3 top-p (nucleus over the per-256-row top-k pool with
    the exact full-vocabulary normalizer).  bias: fp32 (V,) or a 1-element placeholder.
    Returns int32 (T,).  Unlike the Metal original, q6_K takes every mode and every h dtype."""
    V, K, fmt, mode, topk = int(V), int(K), str(fmt), int(mode), int(topk)
    temperature, seed, top_p = float(temperature), int(seed), float(top_p)
    _check_lm_head(h, Wq, bias, V, K, fmt, mode, topk, temperature, top_p)
    if mode in (2, 3):
        _check(topk <= V, "lm_head_sample_q: k must be <= vocab size V")
    T = h.size(0)
    use_bias = bias is not None and bias.numel() > 1
    if use_bias:
        _check(bias.numel() == V, "lm_head_sample_q: bias must be (V,)")
    with _guard(h.device):
        hc, wc = h.contiguous(), Wq.contiguous()
        bc = bias.to(torch.float32).contiguous() if use_bias else None
        out = torch.empty((T,), dtype=torch.int32, device=h.device)
        L = _lib.lib()
        nbytes = L.qx_cuda_lm_head_workspace_bytes(T, V, K, mode, topk)
        ws = _workspace(h.device, nbytes)
        _lib.check(L.qx_cuda_lm_head_sample_q(
            _stream(), _ptr(hc), _ptr(wc), _ptr(bc), _ptr(out), _ptr(ws), nbytes, T, V, K,
            fmt.encode(), _DT[h.dtype], mode, topk, temperature, seed & 0xFFFFFFFF, top_p))
    return out


def lm_head_sample(h, W, bias, mode, k, temperature, seed):
    """Fused LM head + sampling over a dense head W (V,K) in h's dtype: one token id per row of h
    without materialising the (T,V) logits.  mode 0 argmax, 1 categorical, 2 top-k.  bias (V,) or
    a 1-element placeholder.  Returns int32 (T,)."""
    mode, k, temperature, seed = int(mode), int(k), float(temperature), int(seed)
    _check(h.is_cuda, "lm_head_sample: h must be a CUDA tensor")
    _check(h.dim() == 2 and W.dim() == 2 and h.size(1) == W.size(1),
           "lm_head_sample: h (T,K) and W (V,K) must share K")
    _check(h.dtype in _DT and h.dtype == W.dtype,
           "lm_head_sample: h/W must be the same float dtype (f32/f16/bf16)")
    _check(0 <= mode <= 2, "lm_head_sample: mode must be 0/1/2")
    use_bias = bias is not None and bias.numel() > 1
    _same_device("lm_head_sample", h, W, bias if use_bias else None)
    T, K = h.shape
    V = W.size(0)
    if mode == 2:
        _check(1 <= k <= 64, "lm_head_sample: topk k must be in [1, 64]")
        _check(k <= V, "lm_head_sample: topk k must be <= vocab size V")
    with _guard(h.device):
        hc, wc = h.contiguous(), W.contiguous()
        bc = bias.to(torch.float32).contiguous() if use_bias else None
        out = torch.empty((T,), dtype=torch.int32, device=h.device)
        L = _lib.lib()
        nbytes = L.qx_cuda_lm_head_dense_workspace_bytes(T, V, mode, max(k, 1))
        ws = _workspace(h.device, nbytes)
        _lib.check(L.qx_cuda_lm_head_sample_dense(
            _stream(), _ptr(hc), _ptr(wc), _ptr(bc), _ptr(out), _ptr(ws), nbytes, T, V, K,
            _DT[h.dtype], mode, max(k, 1), temperature, seed & 0xFFFFFFFF))
    return out


def _sample_logits(logits, kind: int, name: str, k=0, p=1.0, temperature=1.0, seed=0):
    _check(logits.is_cuda and logits.dtype in _DT and logits.dim() >= 1 and logits.numel() > 0,
           f"{name}: logits must be a non-empty CUDA fp32/fp16/bf16 tensor")
    V = logits.size(-1)
    rows = logits.numel() // V
    with _guard(logits.device):
        lc = logits.contiguous()
        out = torch.empty(logits.shape[:-1], dtype=torch.int32, device=logits.device)
        _lib.check(_lib.lib().qx_cuda_sample_logits(
            _stream(), _ptr(lc), _ptr(out), rows, V, _DT[logits.dtype], kind, int(k), float(p),
            float(temperature), int(seed) & 0xFFFFFFFF))
    return out


def argmax_sample(logits):
    """Greedy sampling: argmax token index over the last (vocab) axis, ties to the smaller index."""
    return _sample_logits(logits, 0, "argmax_sample")


def sample_categorical(logits, temperature=1.0, seed=0):
    """Gumbel-max categorical sampling from softmax(logits / temperature)."""
    return _sample_logits(logits, 1, "sample_categorical", temperature=temperature, seed=seed)


def top_k_sample(logits, k, temperature=1.0, seed=0):
    """Top-k sampling: Gumbel-max from softmax over the k highest logits (k <= 64)."""
    return _sample_logits(logits, 2, "top_k_sample", k=k, temperature=temperature, seed=seed)


def top_p_sample(logits, p, temperature=1.0, seed=0):
    """Top-p (nucleus) sampling: Gumbel-max from the smallest top-probability set with mass >= p."""
    return _sample_logits(logits, 3, "top_p_sample", p=p, temperature=temperature, seed=seed)


def _check_head_weight(h, W, format, name: str):
    """The reference's check_masked_lm_weight (torch_kernels.mm:6625-6653): returns (V, K)."""
    _check(h.is_cuda and W.is_cuda and h.dtype in _DT and h.dim() == 2 and h.size(0) > 0 and h.size(1) > 0,
           f"{name}: h must be non-empty (T,K) fp32/fp16/bf16")
    K = h.size(1)
    if format == "":
        _check(W.dtype == h.dtype and W.dim() == 2 and W.size(0) > 0 and W.size(1) == K,
               f"{name}: dense weight must be (V,K) with h dtype")
        return W.size(0), K
    _check(format in _BLOCK, f"{name}: format must be empty/dense, q4_0, q8_0, q6_K, mxfp8, nvfp4, or mxfp4")
    bk, bb = _BLOCK[format]
    _check(W.dtype == torch.uint8 and W.dim() == 3 and W.size(0) > 0 and K % bk == 0
           and W.size(1) == K // bk and W.size(2) == bb, f"{name}: invalid packed weight shape")
    return W.size(0), K


def lm_head_masked(h, W, bias, allow_mask, format="", topk=1, normalize_allowed=True):
    """Masked dense / packed LM head: (ids int32 (T,topk), logprobs fp32 (T,topk)) of the topk best
    tokens admitted by allow_mask (T, ceil(V/32)) packed 32-bit words; logprobs are normalised over
    the admitted tokens, or over the whole vocabulary when normalize_allowed is false."""
    fmt, topk = str(format), int(topk)
    V, K = _check_head_weight(h, W, fmt, "lm_head_masked")
    T = h.size(0)
    _check(1 <= topk <= 8 and topk <= V, "lm_head_masked: topk must be in [1,min(8,V)]")
    words = (V + 31) // 32
    _check(allow_mask.is_cuda and allow_mask.dim() == 2 and allow_mask.size(0) == T and allow_mask.size(1) == words,
           "lm_head_masked: allow_mask must be (T,ceil(V/32))")
    use_bias = bias is not None and bias.numel() > 1
    _check(not use_bias or (bias.dim() == 1 and bias.size(0) == V),
           "lm_head_masked: bias must be (V,) or scalar placeholder")
    _same_device("lm_head_masked", h, W, allow_mask, bias if use_bias else None)
    with _guard(h.device):
        hc, wc = h.contiguous(), W.contiguous()
        bc = bias.to(torch.float32).contiguous() if use_bias else None
        mc = allow_mask.to(torch.int32).contiguous()
        ids = torch.empty((T, topk), dtype=torch.int32, device=h.device)
        lp = torch.empty((T, topk), dtype=torch.float32, device=h.device)
        L = _lib.lib()
        nbytes = L.qx_cuda_lm_head_masked_workspace_bytes(T, V, K, topk)
        ws = _workspace(h.device, nbytes)
        _lib.check(L.qx_cuda_lm_head_masked(
            _stream(), _ptr(hc), _ptr(wc), _ptr(bc), _ptr(mc), _ptr(ids), _ptr(lp), _ptr(ws), nbytes, T, V, K,
            fmt.encode(), _DT[h.dtype], topk, int(bool(normalize_allowed))))
    return ids, lp


def lm_head_candidates(h, W, bias, candidate_ids, offsets, format="", topk=1):
    """CSR candidate dense / packed LM head: only the listed tokens are projected; returns their topk
    (ids, logprobs) per row, log-probabilities normalised over the valid listed tokens."""
    fmt, topk = str(format), int(topk)
    V, K = _check_head_weight(h, W, fmt, "lm_head_candidates")
    T = h.size(0)
    _check(1 <= topk <= 8 and topk <= V, "lm_head_candidates: topk must be in [1,min(8,V)]")
    _check(candidate_ids.is_cuda and offsets.is_cuda and candidate_ids.dim() == 1 and offsets.dim() == 1
           and offsets.size(0) == T + 1, "lm_head_candidates: flat candidate_ids and T+1 offsets required")
    use_bias = bias is not None and bias.numel() > 1
    _check(not use_bias or (bias.dim() == 1 and bias.size(0) == V),
           "lm_head_candidates: bias must be (V,) or scalar placeholder")
    _same_device("lm_head_candidates", h, W, candidate_ids, offsets, bias if use_bias else None)
    with _guard(h.device):
        hc, wc = h.contiguous(), W.contiguous()
        bc = bias.to(torch.float32).contiguous() if use_bias else None
        cc, oc = candidate_ids.to(torch.int32).contiguous(), offsets.to(torch.int32).contiguous()
        entries = cc.numel()
        ids = torch.empty((T, topk), dtype=torch.int32, device=h.device)
        lp = torch.empty((T, topk), dtype=torch.float32, device=h.device)
        nbytes = max(entries, 1) * 4 + 256
        ws = _workspace(h.device, nbytes)
        _lib.check(_lib.lib().qx_cuda_lm_head_candidates(
            _stream(), _ptr(hc), _ptr(wc), _ptr(bc), _ptr(cc), _ptr(oc), entries, _ptr(ids), _ptr(lp), _ptr(ws),
            nbytes, T, V, K, fmt.encode(), _DT[h.dtype], topk))
    return ids, lp


def lm_head_beam_advance(h, Wq, bias, cum_log_probs, beam_width, fmt="q4_0"):
    """Quantized LM head + exact beam-search advance without full logits: h (B*BM, K), cum_log_probs
    (B, BM) -> (next_token, parent_beam, new cumulative log-probability), each (B, BM)."""
    fmt, BM = str(fmt), int(beam_width)
    _check(h.is_cuda and Wq.is_cuda and cum_log_probs.is_cuda and h.dtype in _DT,
           "lm_head_beam_advance: inputs must be CUDA and h floating point")
    _check(h.dim() == 2 and h.size(0) > 0 and h.size(1) > 0, "lm_head_beam_advance: h must be non-empty (B*BM,K)")
    _check(fmt in ("q4_0", "q8_0", "mxfp8", "nvfp4", "mxfp4"),
           "lm_head_beam_advance: format must be q4_0, q8_0, mxfp8, nvfp4, or mxfp4")
    _check(1 <= BM <= 16, "lm_head_beam_advance: beam_width must be in [1,16]")
    rows, K = h.shape
    bk, bb = _BLOCK[fmt]
    _check(K % bk == 0 and Wq.dtype == torch.uint8 and Wq.dim() == 3 and Wq.size(0) > 0
           and Wq.size(1) == K // bk and Wq.size(2) == bb,
           "lm_head_beam_advance: packed W has invalid shape for its format")
    _check(cum_log_probs.dim() == 2 and cum_log_probs.size(1) == BM and rows == cum_log_probs.size(0) * BM,
           "lm_head_beam_advance: cum_log_probs must be (B,BM), h rows B*BM")
    B, V = cum_log_probs.size(0), Wq.size(0)
    _check(V >= 2 * BM, "lm_head_beam_advance: vocab must be >= 2*beam_width")
    use_bias = bias is not None and bias.numel() > 1
    _check(not use_bias or (bias.dim() == 1 and bias.size(0) == V),
           "lm_head_beam_advance: bias must be (V,) or a scalar placeholder")
    _same_device("lm_head_beam_advance", h, Wq, cum_log_probs, bias if use_bias else None)
    with _guard(h.device):
        hc, wc = h.contiguous(), Wq.contiguous()
        bc = bias.to(torch.float32).contiguous() if use_bias else None
        cc = cum_log_probs.to(torch.float32).contiguous()
        tok = torch.empty((B, BM), dtype=torch.int32, device=h.device)
        par = torch.empty((B, BM), dtype=torch.int32, device=h.device)
        new = torch.empty((B, BM), dtype=torch.float32, device=h.device)
        L = _lib.lib()
        nbytes = L.qx_cuda_lm_head_beam_workspace_bytes(rows, V, K, BM)
        ws = _workspace(h.device, nbytes)
        _lib.check(L.qx_cuda_lm_head_beam_advance(
            _stream(), _ptr(hc), _ptr(wc), _ptr(bc), _ptr(cc), _ptr(tok), _ptr(par), _ptr(new), _ptr(ws), nbytes,
            B, BM, V, K, fmt.encode(), _DT[h.dtype]))
    return tok, par, new


def _qgemm(wq, x, format, name):
    fmt = str(format)
    _check(wq.is_cuda and x.is_cuda, f"{name}: wq and x must be CUDA tensors")
    _check(wq.dtype == torch.uint8, f"{name}: wq must be uint8 packed blocks")
    _check(x.dtype in _DT, f"{name}: x must be float16 (float32 / bfloat16 are accepted too)")
    _check(fmt in _BLOCK, f"{name}: format must be q4_0, q8_0, q6_K, mxfp8, nvfp4, or mxfp4")
    _check(wq.dim() == 3 and x.dim() == 2, f"{name}: wq (N,K/bk,bytes), x (K,M)")
    bk, bb = _BLOCK[fmt]
    N, K = wq.size(0), wq.size(1) * bk
    _check(wq.size(2) == bb and x.size(0) == K and N > 0 and K > 0 and x.size(1) > 0,
           f"{name}: wq (N,K/bk,bytes), x (K,M) with x rows == K")
    _same_device(name, wq, x)
    M = x.size(1)
    with _guard(x.device):
        wc, xc = wq.contiguous(), x.contiguous()
        out = torch.empty((N, M), dtype=x.dtype, device=x.device)
        L = _lib.lib()
        nbytes = L.qx_cuda_qgemm_workspace_bytes(N, K, M, fmt.encode(), _DT[x.dtype])
        ws = _workspace(x.device, nbytes)
        _lib.check(L.qx_cuda_qgemm(_stream(), _ptr(wc), _ptr(xc), _ptr(out), N, K, M, fmt.encode(), _DT[x.dtype],
                                   _ptr(ws), nbytes))
    return out


def qgemm(wq, x, format="q8_0"):
    """Quantized GEMM: out = dequantize(wq) @ x.  wq packed weight blocks (N, K//block_k, block_bytes)
    uint8; x (K, M) float16 -> (N, M) float16."""
    return _qgemm(wq, x, format, "qgemm")


def qgemv(wq, x, format="q8_0"):
    """Quantized GEMV.  x is (K, 1) float16, or fp32 for q4_0 / q6_K (any format here)."""
    _check(x.dim() == 2 and x.size(1) == 1, "qgemv: wq (N,K/bk,bytes), x (K,1)")
    return _qgemm(wq, x, format, "qgemv")


def quantized_embedding(table, ids, add, format, scale=1.0, use_add=False, output_dtype="float16"):
    """Packed embedding lookup with optional additive epilogue: rows of the packed table gathered by
    ids, dequantised in fp32, times scale (+ add), rounded once to output_dtype.  Invalid ids give
    all-zero rows and ignore add."""
    fmt = str(format)
    names = {"float16": torch.float16, "bfloat16": torch.bfloat16, "float32": torch.float32}
    _check(output_dtype in names, "quantized_embedding: output_dtype must be 'float16', 'bfloat16', or 'float32'")
    _check(fmt in _BLOCK, "quantized_embedding: format must be q4_0, q8_0, q6_K, mxfp8, nvfp4, or mxfp4")
    bk, bb = _BLOCK[fmt]
    _check(table.is_cuda and ids.is_cuda and table.dtype == torch.uint8 and table.dim() == 3 and table.size(0) > 0
           and table.size(1) > 0 and table.size(2) == bb and ids.numel() > 0,
           "quantized_embedding: table must be packed uint8 (rows,blocks,block_bytes)")
    dtype = names[output_dtype]
    rows, columns = table.size(0), table.size(1) * bk
    shape = tuple(ids.shape) + (columns,)
    _check(not use_add or (add.dtype == dtype and tuple(add.shape) == shape),
           "quantized_embedding: add must match output shape and output_dtype")
    _same_device("quantized_embedding", table, ids, add if use_add else None)
    with _guard(table.device):
        tc, ic = table.contiguous(), ids.to(torch.int32).contiguous()
        ac = add.contiguous() if use_add else None
        out = torch.empty(shape, dtype=dtype, device=table.device)
        _lib.check(_lib.lib().qx_cuda_quantized_embedding(
            _stream(), _ptr(tc), _ptr(ic), _ptr(ac), _ptr(out), rows, columns, ic.numel(), fmt.encode(),
            float(scale), int(bool(use_add)), _DT[dtype]))
    return out


def dequant_gather(table, ids, format, scale=1.0):
    """Gather packed q4_0 / q8_0 / q6_K rows directly to fp16; invalid ids yield zero rows."""
    _check(str(format) in ("q4_0", "q8_0", "q6_K"), "dequant_gather: format must be q4_0, q8_0, or q6_K")
    return quantized_embedding(table, ids, None, format, scale, False, "float16")


def _rms_norm_add(x, residual, weight, eps, quant, static_scale=0.0, group=0, ue8m0=False, name="rms_norm_add"):
    _check(x.is_cuda and x.dtype in _DT and x.dim() >= 1 and x.numel() > 0,
           f"{name}: x must be a non-empty CUDA fp32/fp16/bf16 tensor")
    D = x.size(-1)
    _check(residual.shape == x.shape and residual.dtype == x.dtype and weight.dim() == 1 and weight.size(0) == D
           and weight.dtype == x.dtype, f"{name}: residual must match x, weight must be (D,) with x dtype")
    _same_device(name, x, residual, weight)
    rows = x.numel() // D
    with _guard(x.device):
        xc, rc, wc = x.contiguous(), residual.contiguous(), weight.contiguous()
        added = torch.empty_like(xc)
        y = torch.empty_like(xc) if quant == 0 else None
        codes = scale = None
        if quant:
            codes = torch.empty(x.shape, dtype=torch.int8 if quant in (3, 5) else torch.uint8, device=x.device)
        if quant in (2, 3):
            scale = torch.empty(x.shape[:-1], dtype=torch.float32, device=x.device)
        elif quant in (4, 5):
            scale = torch.empty(tuple(x.shape[:-1]) + (D // group,), dtype=torch.float32, device=x.device)
        _lib.check(_lib.lib().qx_cuda_rms_norm_add(
            _stream(), _ptr(xc), _ptr(rc), _ptr(wc), _ptr(y), _ptr(codes), _ptr(added), _ptr(scale), rows, D,
            _DT[x.dtype], float(eps), quant, float(static_scale), int(group), int(bool(ue8m0))))
    return y, codes, added, scale


def rms_norm_add(x, residual, weight, eps=1e-5):
    """Fused residual add + RMSNorm.  Returns (out, x + residual)."""
    y, _, added, _ = _rms_norm_add(x, residual, weight, eps, 0)
    return y, added


def rms_norm_add_fp8(x, residual, weight, eps=1e-5, scale=None):
    """Fused add + rms_norm + fp8.  scale=None: dynamic per row (codes, added, scale); else static
    per tensor (codes, added).  codes are e4m3 uint8."""
    if scale is None:
        _, codes, added, s = _rms_norm_add(x, residual, weight, eps, 2, name="rms_norm_add_fp8")
        return codes, added, s
    _check(float(scale) > 0.0, "rms_norm_add_fp8: scale must be positive")
    _, codes, added, _ = _rms_norm_add(x, residual, weight, eps, 1, static_scale=float(scale), name="rms_norm_add_fp8")
    return codes, added


def rms_norm_add_int8_dyn(x, residual, weight, eps=1e-5):
    """Fused add + rms_norm + dynamic per-row symmetric int8: (codes, added, scale)."""
    _, codes, added, s = _rms_norm_add(x, residual, weight, eps, 3, name="rms_norm_add_int8_dyn")
    return codes, added, s


def rms_norm_add_per_block(x, residual, weight, eps=1e-5, int8=False, ue8m0=False):
    """Fused add + rms_norm + per-128-block quant.  Returns (codes, x + residual, scale (rows, D/128))."""
    _check(x.size(-1) % 128 == 0, "rms_norm_add_per_block: per-block quant requires D % 128 == 0")
    _, codes, added, s = _rms_norm_add(x, residual, weight, eps, 5 if int8 else 4, group=128, ue8m0=ue8m0,
                                       name="rms_norm_add_per_block")
    return codes, added, s


_ACTQ_MODES = {"swiglu": 0, "swiglu_oai": 1}


def _silu_mul_quant(x, gate, act, alpha, limit, quant, group=0, ue8m0=False, name="silu_mul_quant_fp8"):
    _check(act in _ACTQ_MODES, f"{name}: act must be 'swiglu' or 'swiglu_oai'")
    _check(x.is_cuda and x.dtype in _DT and x.dim() >= 1 and x.numel() > 0 and gate.shape == x.shape
           and gate.dtype == x.dtype, f"{name}: x and gate must be matching non-empty CUDA float tensors")
    _same_device(name, x, gate)
    D = x.size(-1)
    rows = x.numel() // D
    if quant == 4:
        _check(group > 0 and group % 4 == 0 and D % group == 0,
               f"{name}: group_size must be a multiple of 4 that divides D")
    with _guard(x.device):
        xc, gc = x.contiguous(), gate.contiguous()
        codes = torch.empty(x.shape, dtype=torch.int8 if quant == 3 else torch.uint8, device=x.device)
        sshape = tuple(x.shape[:-1]) + ((D // group,) if quant == 4 else ())
        scale = torch.empty(sshape, dtype=torch.float32, device=x.device)
        _lib.check(_lib.lib().qx_cuda_silu_mul_quant(
            _stream(), _ptr(xc), _ptr(gc), _ptr(codes), _ptr(scale), rows, D, _DT[x.dtype], _ACTQ_MODES[act],
            float(alpha), float(limit), quant, int(group), int(bool(ue8m0))))
    return codes, scale


def silu_mul_quant_fp8(x, gate, act="swiglu", alpha=1.702, limit=7.0):
    """Fused gated activation -> dynamic per-token fp8.  Returns (codes u8, scale)."""
    return _silu_mul_quant(x, gate, act, alpha, limit, 2)


def silu_mul_quant_int8(x, gate, act="swiglu", alpha=1.702, limit=7.0):
    """Fused gated activation -> dynamic per-token int8.  Returns (codes i8, scale)."""
    return _silu_mul_quant(x, gate, act, alpha, limit, 3, name="silu_mul_quant_int8")


def silu_mul_quant_fp8_group(x, gate, group_size=128, ue8m0=False, act="swiglu", alpha=1.702, limit=7.0):
    """Fused gated activation -> per-group fp8 (scale (rows, D/G); ue8m0 = 2^k scales)."""
    return _silu_mul_quant(x, gate, act, alpha, limit, 4, int(group_size), ue8m0, name="silu_mul_quant_fp8_group")


# ---- BaseQN: separate code / scale / bias planes ------------------------------------------------------
_BQ_SCALE = {"bf16": torch.bfloat16, "bfloat16": torch.bfloat16, "f16": torch.float16, "float16": torch.float16,
             "e8m0": torch.uint8, "e4m3": torch.uint8}
_BQ_OUT = {"float16": torch.float16, "f16": torch.float16, "bfloat16": torch.bfloat16, "bf16": torch.bfloat16,
           "float32": torch.float32, "f32": torch.float32}


def _bq_desc(bits, group_size, scale_dtype, symmetric, layout):
    """The descriptor checks of kernels/common/base_q_descriptor.h:34-68 (the library repeats them)."""
    bits, group_size = int(bits), int(group_size)
    _check(bits in (2, 3, 4, 5, 6, 8), "BaseQN: bits must be one of 2, 3, 4, 5, 6, or 8")
    _check(group_size in (32, 64, 128), "BaseQN: group_size must be 32, 64, or 128")
    _check(str(scale_dtype) in _BQ_SCALE, "BaseQN: scale_dtype must be bf16, f16, e8m0, or e4m3")
    _check(str(scale_dtype) != "e4m3" or bits == 8, "BaseQN: e4m3 scale storage is valid only for q8")
    _check(str(layout) in ("metal", "metal_lane_strided", f"metal_lane_strided_q{bits}"),
           f"BaseQN: layout must be metal or metal_lane_strided_q{bits}")
    return _lib.BaseQDescriptor(bits, group_size, str(scale_dtype).encode(), int(bool(symmetric)), str(layout).encode())


def _bq_planes(name, codes, scales, biases, desc, rank=2):
    """The storage checks of kernels/quantization/base_q/base_q.cpp:57-131.  Returns
    (planes struct, kept-alive tensors, leading dims, K)."""
    lead = "experts, output_rows" if rank == 3 else "rows"
    _check(codes.is_cuda and codes.dtype == torch.uint8 and codes.dim() == rank,
           f"{name}: codes must be uint8 ({lead}, packed_bytes)")
    sd = _BQ_SCALE[desc.scale_dtype.decode()]
    _check(scales.is_cuda and scales.dtype == sd and scales.dim() == rank,
           f"{name}: scales must be a rank-{rank} tensor with the declared scale_dtype")
    _check(all(int(n) > 0 for n in scales.shape) and tuple(scales.shape[:-1]) == tuple(codes.shape[:-1]),
           f"{name}: codes/scales rows and group count must be positive and match")
    K = scales.size(-1) * desc.group_size
    _check(K * desc.bits % 8 == 0 and codes.size(-1) == K * desc.bits // 8,
           f"{name}: codes.shape[{rank - 1}] must equal columns * bits / 8")
    _check(desc.symmetric or biases is not None, f"{name}: biases are required for asymmetric BaseQN")
    _check(biases is None or (biases.dtype == scales.dtype and tuple(biases.shape) == tuple(scales.shape)),
           f"{name}: biases must match scales shape and dtype")
    _same_device(name, codes, scales, biases)
    keep = (codes.contiguous(), scales.contiguous(), None if biases is None else biases.contiguous())
    return _lib.BaseQPlanes(_ptr(keep[0]), _ptr(keep[1]), _ptr(keep[2])), keep, tuple(codes.shape[:-1]), K


def _bq_ws(L, device, K, M, V, dtype):
    n = L.qx_cuda_base_q_workspace_bytes(K, M, V, _DT[dtype])
    return (_workspace(device, n), n) if n else (None, 0)


def base_qdequant(codes, scales, biases, bits, group_size, scale_dtype="bf16", symmetric=False, layout="metal",
                  output_dtype="float16"):
    """Decode canonical BaseQN separate code / scale / bias planes to (rows, K)."""
    desc = _bq_desc(bits, group_size, scale_dtype, symmetric, layout)
    _check(str(output_dtype) in _BQ_OUT, "BaseQN: output_dtype must be float16, bfloat16, or float32")
    planes, keep, (rows,), K = _bq_planes("base_qdequant", codes, scales, biases, desc)
    with _guard(codes.device):
        out = torch.empty((rows, K), dtype=_BQ_OUT[str(output_dtype)], device=codes.device)
        _lib.check(_lib.lib().qx_cuda_base_qdequant(_stream(), planes, desc, _ptr(out), rows, K, _DT[out.dtype]))
    return out


def base_qembedding(codes, scales, biases, ids, bits, group_size, scale_dtype="bf16", symmetric=False,
                    layout="metal", output_dtype="float16"):
    """Gather and decode BaseQN weight rows to ids.shape + (K,); ids outside the table give zero rows."""
    desc = _bq_desc(bits, group_size, scale_dtype, symmetric, layout)
    _check(str(output_dtype) in _BQ_OUT, "BaseQN: output_dtype must be float16, bfloat16, or float32")
    planes, keep, (rows,), K = _bq_planes("base_qembedding", codes, scales, biases, desc)
    _check(ids.is_cuda and ids.numel() > 0 and not ids.dtype.is_floating_point,
           "base_qembedding: ids must be a non-empty integer tensor")
    _same_device("base_qembedding", codes, ids)
    with _guard(codes.device):
        ic = ids.to(torch.int32).contiguous()
        out = torch.empty(tuple(ids.shape) + (K,), dtype=_BQ_OUT[str(output_dtype)], device=codes.device)
        _lib.check(_lib.lib().qx_cuda_base_qembedding(_stream(), planes, desc, _ptr(ic), _ptr(out), rows, K,
                                                      ic.numel(), _DT[out.dtype]))
    return out


def _bq_matmul(name, codes, scales, biases, x, desc, gemv_only):
    planes, keep, (rows,), K = _bq_planes(name, codes, scales, biases, desc)
    _check(x.is_cuda and x.dim() == 2 and x.size(0) == K, f"{name}: x must be (K, M) with K matching the packed weights")
    _check(not gemv_only or x.size(1) == 1, "base_qgemv: x must be (K, 1)")
    _check(x.dtype in _DT, "BaseQN matmul: x must be float16, bfloat16, or float32")
    _check(x.size(1) > 0, "BaseQN matmul: M must be positive")
    _same_device(name, codes, x)
    M = x.size(1)
    with _guard(x.device):
        xc = x.contiguous()
        out = torch.empty((rows, M), dtype=x.dtype, device=x.device)
        L = _lib.lib()
        ws, n = _bq_ws(L, x.device, K, M, 0, x.dtype)
        _lib.check(L.qx_cuda_base_qgemm(_stream(), planes, desc, _ptr(xc), _ptr(out), rows, K, M, _DT[x.dtype],
                                        _ptr(ws), n))
    return out


def base_qgemv(codes, scales, biases, x, bits, group_size, scale_dtype="bf16", symmetric=False, layout="metal"):
    """dequant(BaseQN weights) @ x for x (K, 1)."""
    return _bq_matmul("base_qgemv", codes, scales, biases, x, _bq_desc(bits, group_size, scale_dtype, symmetric, layout), True)


def base_qgemm(codes, scales, biases, x, bits, group_size, scale_dtype="bf16", symmetric=False, layout="metal"):
    """dequant(BaseQN weights) @ x for x (K, M)."""
    return _bq_matmul("base_qgemm", codes, scales, biases, x, _bq_desc(bits, group_size, scale_dtype, symmetric, layout), False)


def base_qgemv_qkv(q_codes, q_scales, q_biases, k_codes, k_scales, k_biases, v_codes, v_scales, v_biases, x, bits,
                   group_size, scale_dtype="bf16", symmetric=False, layout="metal"):
    """Q / K / V decode projections of one (K, 1) activation in one launch; row counts may differ."""
    name = "base_qgemv_qkv"
    desc = _bq_desc(bits, group_size, scale_dtype, symmetric, layout)
    q, kq, (qr,), K = _bq_planes(name, q_codes, q_scales, q_biases, desc)
    k, kk, (kr,), K2 = _bq_planes(name, k_codes, k_scales, k_biases, desc)
    v, kv, (vr,), K3 = _bq_planes(name, v_codes, v_scales, v_biases, desc)
    _check(K == K2 == K3, f"{name}: q/k/v must share the inner dimension")
    _check(x.is_cuda and x.dim() == 2 and x.size(0) == K and x.size(1) == 1 and x.dtype in _DT,
           f"{name}: x must be (K, 1) float16, bfloat16, or float32")
    _same_device(name, q_codes, k_codes, v_codes, x)
    with _guard(x.device):
        xc = x.contiguous()
        outs = [torch.empty((r, 1), dtype=x.dtype, device=x.device) for r in (qr, kr, vr)]
        L = _lib.lib()
        ws, n = _bq_ws(L, x.device, K, 1, 0, x.dtype)
        _lib.check(L.qx_cuda_base_qgemv_qkv(_stream(), q, k, v, desc, _ptr(xc), _ptr(outs[0]), _ptr(outs[1]),
                                            _ptr(outs[2]), qr, kr, vr, K, _DT[x.dtype], _ptr(ws), n))
    return tuple(outs)


def base_qgemv_swiglu(gate_codes, gate_scales, gate_biases, up_codes, up_scales, up_biases, x, bits, group_size,
                      scale_dtype="bf16", symmetric=False, layout="metal"):
    """silu(W_gate @ x) * (W_up @ x) straight from BaseQN planes, rounded once."""
    name = "base_qgemv_swiglu"
    desc = _bq_desc(bits, group_size, scale_dtype, symmetric, layout)
    g, kg, (rows,), K = _bq_planes(name, gate_codes, gate_scales, gate_biases, desc)
    u, ku, (rows2,), K2 = _bq_planes(name, up_codes, up_scales, up_biases, desc)
    _check(rows == rows2 and K == K2, f"{name}: gate and up must have the same shape")
    _check(x.is_cuda and x.dim() == 2 and x.size(0) == K and x.size(1) == 1 and x.dtype in _DT,
           f"{name}: x must be (K, 1) float16, bfloat16, or float32")
    _same_device(name, gate_codes, up_codes, x)
    with _guard(x.device):
        xc = x.contiguous()
        out = torch.empty((rows, 1), dtype=x.dtype, device=x.device)
        L = _lib.lib()
        ws, n = _bq_ws(L, x.device, K, 1, 0, x.dtype)
        _lib.check(L.qx_cuda_base_qgemv_swiglu(_stream(), g, u, desc, _ptr(xc), _ptr(out), rows, K, _DT[x.dtype],
                                               _ptr(ws), n))
    return out


def base_qlm_head_argmax(codes, scales, biases, x, bits, group_size, scale_dtype="bf16", symmetric=False,
                         layout="metal"):
    """Greedy token ids (batch,) int32 from a BaseQN LM head (V, K) and activations x (K, batch); logits
    are rounded to the dtype of x, the lower id wins exact ties."""
    name = "base_qlm_head_argmax"
    desc = _bq_desc(bits, group_size, scale_dtype, symmetric, layout)
    _check(x.dim() == 2 and x.size(1) > 0, "base_qlm_head_argmax: x must be non-empty (K, batch)")
    planes, keep, (V,), K = _bq_planes(name, codes, scales, biases, desc)
    _check(x.is_cuda and x.size(0) == K and x.dtype in _DT, f"{name}: x must be (K, batch) with K matching the packed weights")
    _same_device(name, codes, x)
    batch = x.size(1)
    with _guard(x.device):
        xc = x.contiguous()
        ids = torch.empty((batch,), dtype=torch.int32, device=x.device)
        L = _lib.lib()
        ws, n = _bq_ws(L, x.device, K, batch, V, x.dtype)
        _lib.check(L.qx_cuda_base_qlm_head_argmax(_stream(), planes, desc, _ptr(xc), _ptr(ids), V, K, batch,
                                                  _DT[x.dtype], _ptr(ws), n))
    return ids


def _bq_moe(name, codes, scales, biases, input, expert_of_tile, desc, swiglu):
    planes, keep, (experts, expert_rows), K = _bq_planes(name, codes, scales, biases, desc, rank=3)
    _check(input.is_cuda and input.dim() == 2 and input.size(1) == K and input.dtype in (torch.float16, torch.bfloat16),
           f"{name}: input must be (total_rows, K) float16 or bfloat16")
    total = input.size(0)
    _check(total > 0 and total % 32 == 0, f"{name}: input rows must be a positive multiple of 32")
    _check(expert_of_tile.is_cuda and expert_of_tile.dtype == torch.int32 and expert_of_tile.numel() == total // 32,
           f"{name}: expert_of_tile must be int32 (total_rows / 32,)")
    _check(not swiglu or expert_rows % 2 == 0, f"{name}: the gate/up row axis must be even")
    _same_device(name, codes, input, expert_of_tile)
    cols = expert_rows // 2 if swiglu else expert_rows
    with _guard(input.device):
        xc, ec = input.contiguous(), expert_of_tile.contiguous()
        out = torch.zeros((total, cols), dtype=input.dtype, device=input.device)
        L = _lib.lib()
        ws, n = _bq_ws(L, input.device, K, total, 0, input.dtype)
        _lib.check(L.qx_cuda_base_qmoe(_stream(), planes, desc, _ptr(xc), _ptr(ec), _ptr(out), experts, expert_rows,
                                       K, total, int(swiglu), _DT[input.dtype], _ptr(ws), n))
    return out


def base_qmoe_gemm(codes, scales, biases, input, expert_of_tile, bits, group_size, scale_dtype="bf16",
                   symmetric=False, layout="metal"):
    """Padded MoE rows through a BaseQN expert stack: (total_rows, K) -> (total_rows, output_rows)."""
    return _bq_moe("base_qmoe_gemm", codes, scales, biases, input, expert_of_tile,
                   _bq_desc(bits, group_size, scale_dtype, symmetric, layout), False)


def base_qmoe_swiglu(codes, scales, biases, input, expert_of_tile, bits, group_size, scale_dtype="bf16",
                     symmetric=False, layout="metal"):
    """Grouped expert gate / up projection with SwiGLU; the row axis is [gate(I), up(I)]."""
    return _bq_moe("base_qmoe_swiglu", codes, scales, biases, input, expert_of_tile,
                   _bq_desc(bits, group_size, scale_dtype, symmetric, layout), True)
