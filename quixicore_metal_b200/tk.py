"""The reference's public operator API (`tk`) for the decode-projection path, on CUDA tensors.

Mirrors the routers of bindings/python/tk/__init__.py: `decode_linear_epilogue` (:3694-3748),
`decode_swiglu` (:3751-3793), `lm_head_sample` with `format=` (:2357-2412) and the output-quant
helper (:3684-3691): same keyword names, defaults and ValueError texts.  The projections serve
packed formats only (the reference routes dense weights to the framework matmul); lm_head_sample
also has the reference's dense routes.
"""
from __future__ import annotations

from . import tk_torch as _tt

_ACTIVATIONS = {"none": 0, None: 0, "gelu": 1, "silu": 2}
_LM_HEAD_MODES = {"argmax": 0, "categorical": 1, "topk": 2, "topp": 3}
_LM_QUANT_BLOCK_K = {"q8_0": 32, "q4_0": 32, "q6_K": 256, "mxfp8": 32, "nvfp4": 16, "mxfp4": 32}


def quantize_per_token_fp8(x):
    return _tt.quantize_per_token_fp8(x)


def quantize_per_token_int8(x):
    return _tt.quantize_per_token_int8(x)


_OUTPUT_QUANTS = (None, "fp8", "int8", "mxfp8")   # 'mxfp8' (packed rows, e8m0 per 32) is an extension


def decode_linear_epilogue(x, weight, bias=None, residual=None, activation="none", format=None,
                           output_quant=None, use_kernel=None):
    """residual + activation(x @ dequant(weight).T + bias), fp32 accumulation, one rounding to
    x.dtype.  activation: none / gelu (erf) / silu.  output_quant applies the per-token fp8 /
    int8 quantizer to the rounded output (returns (codes, scale)) or, as an extension, packs it as
    'mxfp8' rows - inside the same native call (the reference composes a second operator,
    bindings/python/tk/__init__.py:3684-3691)."""
    if activation not in _ACTIVATIONS:
        raise ValueError("activation must be 'none', 'gelu', or 'silu'")
    if output_quant not in _OUTPUT_QUANTS:
        raise ValueError("output_quant must be None, 'fp8', 'int8', or 'mxfp8'")
    if format is None:
        raise ValueError("decode_linear_epilogue: this backend serves packed weights only; "
                         "pass format=q4_0/q8_0/q6_K/mxfp8/nvfp4/mxfp4")
    if use_kernel is not None and not use_kernel:
        raise ValueError("decode_linear_epilogue: use_kernel=False requires a dense weight")
    use_bias, use_residual = bias is not None, residual is not None
    return _tt.decode_linear_epilogue(x, weight, bias if use_bias else x,
                                      residual if use_residual else x, str(format),
                                      _ACTIVATIONS[activation], use_bias, use_residual,
                                      output_quant=output_quant)


def decode_swiglu(x, gate_weight, up_weight, gate_bias=None, up_bias=None, format=None,
                  output_quant=None, use_kernel=None):
    """silu(gate) * up over two packed projections sharing the activation reads."""
    if (gate_bias is None) != (up_bias is None):
        raise ValueError("decode_swiglu: gate_bias and up_bias must both be present or omitted")
    if output_quant not in _OUTPUT_QUANTS:
        raise ValueError("output_quant must be None, 'fp8', 'int8', or 'mxfp8'")
    if format is None:
        raise ValueError("decode_swiglu: this backend serves packed weights only; "
                         "pass format=q4_0/q8_0/q6_K/mxfp8/nvfp4/mxfp4")
    if use_kernel is not None and not use_kernel:
        raise ValueError("decode_swiglu: use_kernel=False requires dense weights")
    use_bias = gate_bias is not None
    return _tt.decode_swiglu(x, gate_weight, up_weight, gate_bias if use_bias else x,
                             up_bias if use_bias else x, str(format), use_bias,
                             output_quant=output_quant)


def argmax_sample(logits):
    return _tt.argmax_sample(logits)


def sample_categorical(logits, temperature=1.0, seed=0):
    return _tt.sample_categorical(logits, temperature, seed)


def top_k_sample(logits, k, temperature=1.0, seed=0):
    return _tt.top_k_sample(logits, k, temperature, seed)


def top_p_sample(logits, p, temperature=1.0, seed=0):
    return _tt.top_p_sample(logits, p, temperature, seed)


def _lm_head_sample_dense(h, W, mode, k, temperature, seed, bias, fused, top_p):
    """The dense routes of the reference router (bindings/python/tk/__init__.py:2413-2451): the
    fused no-materialisation kernel when asked for (argmax / categorical / topk), otherwise the
    framework matmul followed by the samplers of this backend."""
    import torch
    if fused and mode != "topp":
        b = bias if bias is not None else torch.zeros(1, dtype=torch.float32, device=h.device)
        return _tt.lm_head_sample(h, W, b, _LM_HEAD_MODES[mode], int(k), float(temperature), int(seed))
    logits = torch.matmul(h, W.transpose(-1, -2))
    if bias is not None:
        logits = logits + bias.to(logits.dtype)
    if mode == "argmax":
        return argmax_sample(logits)
    if mode == "categorical":
        return sample_categorical(logits, temperature=temperature, seed=seed)
    if mode == "topk":
        return top_k_sample(logits, k, temperature=temperature, seed=seed)
    return top_p_sample(logits, top_p, temperature=temperature, seed=seed)


def lm_head_sample(h, W, mode="argmax", k=0, temperature=1.0, seed=0, bias=None, fused=False,
                   format=None, top_p=0.9):
    """One token id per row of h.  With format=: over a packed (V, K/block_k, block_bytes) head,
    without ever writing the (T, V) logits.  Without: W is dense (V, K) and the reference's dense
    routes apply (matmul + sampler by default, the fused kernel with fused=True).  mode: argmax / categorical / topk / topp; k defaults to 32 for
    topk / topp; the noise is keyed by the global vocab id, so the draw equals the unfused
    sampler on the same logits and seed."""
    if mode not in _LM_HEAD_MODES:
        raise ValueError(f"lm_head_sample: mode must be one of {list(_LM_HEAD_MODES)}")
    if format is None:
        return _lm_head_sample_dense(h, W, mode, k, temperature, seed, bias, fused, top_p)
    if format not in _LM_QUANT_BLOCK_K:
        raise ValueError(f"lm_head_sample: quant format must be one of {list(_LM_QUANT_BLOCK_K)}")
    kk = int(k) if int(k) > 0 else (32 if mode in ("topk", "topp") else 0)
    V = W.shape[0]
    K = W.shape[1] * _LM_QUANT_BLOCK_K[format]
    return _tt.lm_head_sample_q(h, W, bias, V, K, format, _LM_HEAD_MODES[mode], kk,
                                float(temperature), int(seed), float(top_p))


def lm_head_masked(h, W, allow_mask, bias=None, format=None, topk=1, normalize="allowed"):
    """Project directly into a packed per-row allow mask without materialising logits: (ids, logprobs),
    each (T, topk), of the best admitted tokens.  W dense (V,K) or packed with format=; allow_mask
    (T, ceil(V/32)) packed 32-bit words; normalize 'allowed' (over the admitted tokens) or 'full'
    (the pre-mask full-vocabulary normaliser).  Ties choose the lower token id.
    (bindings/python/tk/__init__.py:2469-2491)"""
    if normalize not in ("allowed", "full"):
        raise ValueError("lm_head_masked: normalize must be 'allowed' or 'full'")
    import torch
    b = bias if bias is not None else torch.zeros(1, dtype=torch.float32, device=h.device)
    return _tt.lm_head_masked(h, W, b, allow_mask, "" if format is None else str(format), int(topk),
                              normalize == "allowed")


def lm_head_candidates(h, W, candidate_ids, offsets, bias=None, format=None, topk=1):
    """Project only CSR-listed token candidates and return their top-k log-probabilities, normalised
    over the valid listed candidates.  (bindings/python/tk/__init__.py:2494-2511)"""
    import torch
    b = bias if bias is not None else torch.zeros(1, dtype=torch.float32, device=h.device)
    return _tt.lm_head_candidates(h, W, b, candidate_ids, offsets, "" if format is None else str(format), int(topk))


def lm_head_beam_advance(h, W, cum_log_probs, beam_width, bias=None, format="q4_0"):
    """Quantized LM head plus exact beam-search advance: next token, parent beam and updated cumulative
    log-probability, each (B, beam_width).  Every format and row count takes the fused no-logits
    kernels here (the reference routes q8_0 / mxfp8 and larger batches through a logits matrix,
    bindings/python/tk/__init__.py:2530-2578)."""
    if format not in ("q4_0", "q8_0", "mxfp8", "nvfp4", "mxfp4"):
        raise ValueError("lm_head_beam_advance: format must be q4_0, q8_0, mxfp8, nvfp4, or mxfp4")
    import torch
    b = bias if bias is not None else torch.zeros(1, dtype=torch.float32, device=h.device)
    return _tt.lm_head_beam_advance(h, W, b, cum_log_probs, int(beam_width), str(format))


def qgemv(wq, x, format="q8_0"):
    """Quantized GEMV (batch-1 decode): out = dequantize(wq) @ x.  wq packed weight blocks
    (N, K//block_k, block_bytes) uint8; x (K, 1) float16 (or fp32).  (tk/__init__.py:3887-3893)"""
    return _tt.qgemv(wq, x, format)


def qgemm(wq, x, format="q8_0"):
    """Quantized GEMM: out = dequantize(wq) @ x; x (K, M) float16 -> (N, M) float16.  Batch 1 goes to
    the GEMV path.  (tk/__init__.py:3179-3187)"""
    if x.shape[-1] == 1:
        return qgemv(wq, x, format)
    return _tt.qgemm(wq, x, format)


def dequant_gather(table, ids, format, scale=1.0):
    """Gather packed q4_0/q8_0/q6_K rows directly to fp16; invalid ids yield zero rows.
    (tk/__init__.py:4132-4136)"""
    return _tt.dequant_gather(table, ids, format, float(scale))


def quantized_embedding_lookup(table, ids, format, scale=1.0, add=None, output_dtype="float16"):
    """Gather packed embedding rows into fp16, bf16 or fp32 output; `add` is an optional output-shaped
    positional / residual term.  Invalid ids produce all-zero rows and ignore `add`.
    (tk/__init__.py:4139-4160)"""
    if output_dtype not in ("float16", "bfloat16", "float32"):
        raise ValueError("output_dtype must be 'float16', 'bfloat16', or 'float32'")
    import torch
    use_add = add is not None
    dtype = {"float16": torch.float16, "bfloat16": torch.bfloat16, "float32": torch.float32}[output_dtype]
    additive = add.to(dtype) if use_add else torch.zeros(1, dtype=dtype, device=table.device)
    return _tt.quantized_embedding(table, ids, additive, format, float(scale), use_add, output_dtype)


# ---- norm / activation -> quantiser seams (bindings/python/tk/__init__.py:606-652, :1489-1522) -------
def rms_norm_add(x, residual, weight, eps=1e-5):
    """Fused residual-add + RMSNorm.  Returns (out, x + residual)."""
    return _tt.rms_norm_add(x, residual, weight, eps)


def rms_norm_add_fp8(x, residual, weight, eps=1e-5, scale=None):
    """Fused add + rms_norm + fp8.  scale=None: dynamic per row (codes, x + residual, scale); else
    static per tensor (codes, x + residual)."""
    return _tt.rms_norm_add_fp8(x, residual, weight, eps, scale)


def rms_norm_add_per_block(x, residual, weight, eps=1e-5, int8=False, ue8m0=False):
    """Fused add + rms_norm + per-128-block quant: (codes, x + residual, scale (rows, D/128))."""
    return _tt.rms_norm_add_per_block(x, residual, weight, eps, int8, ue8m0)


def silu_mul_quant_fp8(x, gate, act="swiglu", alpha=1.702, limit=7.0):
    """Fused gated activation -> dynamic per-token fp8 e4m3: (codes u8, scale (rows,))."""
    return _tt.silu_mul_quant_fp8(x, gate, act=act, alpha=alpha, limit=limit)


def silu_mul_quant_int8(x, gate, act="swiglu", alpha=1.702, limit=7.0):
    """Fused gated activation -> dynamic per-token symmetric int8: (codes i8, scale (rows,))."""
    return _tt.silu_mul_quant_int8(x, gate, act=act, alpha=alpha, limit=limit)


def silu_mul_quant_fp8_group(x, gate, group_size=128, ue8m0=False, act="swiglu", alpha=1.702, limit=7.0):
    """Fused gated activation -> per-group fp8: (codes u8, scale (rows, D/G))."""
    return _tt.silu_mul_quant_fp8_group(x, gate, group_size=group_size, ue8m0=ue8m0, act=act, alpha=alpha, limit=limit)


# ---- BaseQN separate-plane consumers (bindings/python/tk/__init__.py:3896-4105) -----------------------
def _bq_bias(name, biases, scales, symmetric):
    """A symmetric tensor has no bias plane; the reference passes the scales as a placeholder the
    kernels never read (tk/__init__.py:3904-3907).  Here the placeholder is simply absent."""
    if biases is None and not symmetric:
        raise ValueError(f"{name}: biases are required for asymmetric BaseQN")
    return None if symmetric else biases


def base_qdequant(codes, scales, biases, bits, group_size, scale_dtype="bf16", symmetric=False, layout="metal",
                  output_dtype="float16"):
    """Decode canonical BaseQN separate planes to (rows, K).  codes uint8 (rows, K*bits/8); scales and
    asymmetric biases (rows, K/group_size) in the declared storage dtype; symmetric tensors pass
    biases=None."""
    biases = _bq_bias("base_qdequant", biases, scales, symmetric)
    return _tt.base_qdequant(codes, scales, biases, bits, group_size, scale_dtype, symmetric, layout, output_dtype)


def base_qgemv(codes, scales, biases, x, bits, group_size, scale_dtype="bf16", symmetric=False, layout="metal"):
    """dequant(BaseQN weights) @ x for x shaped (K, 1)."""
    biases = _bq_bias("base_qgemv", biases, scales, symmetric)
    return _tt.base_qgemv(codes, scales, biases, x, bits, group_size, scale_dtype, symmetric, layout)


def base_qgemm(codes, scales, biases, x, bits, group_size, scale_dtype="bf16", symmetric=False, layout="metal"):
    """dequant(BaseQN weights) @ x for x shaped (K, M); every M runs on the direct decode kernels."""
    biases = _bq_bias("base_qgemm", biases, scales, symmetric)
    return _tt.base_qgemm(codes, scales, biases, x, bits, group_size, scale_dtype, symmetric, layout)


def base_qgemv_qkv(q_codes, q_scales, q_biases, k_codes, k_scales, k_biases, v_codes, v_scales, v_biases, x, bits,
                   group_size, scale_dtype="bf16", symmetric=False, layout="metal"):
    """Fused BaseQN Q/K/V decode GEMVs over one (K, 1) input; the three matrices share one descriptor
    but may have different row counts.  Returns (q, k, v)."""
    if not symmetric and any(b is None for b in (q_biases, k_biases, v_biases)):
        raise ValueError("base_qgemv_qkv: biases are required for asymmetric BaseQN")
    if symmetric:
        q_biases = k_biases = v_biases = None
    return _tt.base_qgemv_qkv(q_codes, q_scales, q_biases, k_codes, k_scales, k_biases, v_codes, v_scales, v_biases,
                              x, bits, group_size, scale_dtype, symmetric, layout)


def base_qgemv_swiglu(gate_codes, gate_scales, gate_biases, up_codes, up_scales, up_biases, x, bits, group_size,
                      scale_dtype="bf16", symmetric=False, layout="metal"):
    """silu(W_gate @ x) * (W_up @ x) directly from BaseQN planes."""
    if not symmetric and (gate_biases is None or up_biases is None):
        raise ValueError("base_qgemv_swiglu: biases are required for asymmetric BaseQN")
    if symmetric:
        gate_biases = up_biases = None
    return _tt.base_qgemv_swiglu(gate_codes, gate_scales, gate_biases, up_codes, up_scales, up_biases, x, bits,
                                 group_size, scale_dtype, symmetric, layout)


def base_qembedding(codes, scales, biases, ids, bits, group_size, scale_dtype="bf16", symmetric=False,
                    layout="metal", output_dtype="float16"):
    """Gather BaseQN rows and decode directly to ids.shape + (K,); out-of-range ids produce zero rows."""
    biases = _bq_bias("base_qembedding", biases, scales, symmetric)
    return _tt.base_qembedding(codes, scales, biases, ids, bits, group_size, scale_dtype, symmetric, layout,
                               output_dtype)


def base_qlm_head_argmax(codes, scales, biases, x, bits, group_size, scale_dtype="bf16", symmetric=False,
                         layout="metal"):
    """Greedy token ids (batch,) int32 from a packed BaseQN LM head (V, K) and x (K, batch); lower
    token ids win exact ties."""
    biases = _bq_bias("base_qlm_head_argmax", biases, scales, symmetric)
    if x.ndim != 2 or int(x.shape[1]) <= 0:
        raise ValueError("base_qlm_head_argmax: x must be non-empty (K, batch)")
    return _tt.base_qlm_head_argmax(codes, scales, biases, x, bits, group_size, scale_dtype, symmetric, layout)


def base_qmoe_gemm(codes, scales, biases, input, expert_of_tile, bits, group_size, scale_dtype="bf16",
                   symmetric=False, layout="metal"):
    """Padded MoE rows through a BaseQN expert stack.  codes (experts, output_rows, K*bits/8), input
    (total_rows, K), expert_of_tile maps each 32-row tile to its expert -> (total_rows, output_rows)."""
    biases = _bq_bias("base_qmoe_gemm", biases, scales, symmetric)
    return _tt.base_qmoe_gemm(codes, scales, biases, input, expert_of_tile, bits, group_size, scale_dtype, symmetric,
                              layout)


def base_qmoe_swiglu(codes, scales, biases, input, expert_of_tile, bits, group_size, scale_dtype="bf16",
                     symmetric=False, layout="metal"):
    """Fused BaseQN grouped expert gate/up projection and SwiGLU; the packed output-row axis is
    [gate(intermediate), up(intermediate)]."""
    biases = _bq_bias("base_qmoe_swiglu", biases, scales, symmetric)
    return _tt.base_qmoe_swiglu(codes, scales, biases, input, expert_of_tile, bits, group_size, scale_dtype,
                                symmetric, layout)
