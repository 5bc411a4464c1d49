"""Generate the golden fixtures in this directory from the reference itself.

Run where the reference checkout is available (it cannot travel to a GPU machine):

    python tests/golden/make_golden.py /path/to/reference

It imports the reference's numpy packers (`bindings/python/tk/quant.py`) and its torch-CPU
composition (`tk.decode_linear_epilogue(..., use_kernel=False)`), and lifts the numpy RNG twin
out of the reference's LM-head test file.  Outputs (all small, committed):

    formats.npz     per format: reference-packed bytes + reference-dequantised fp32 rows
    codecs.npz      e4m3 / e2m1 decode tables from the reference's codebooks
    rng.npz         rng_uniform / gumbel samples from the reference's numpy twin
    compose.npz     reference torch-CPU outputs of decode_linear_epilogue / decode_swiglu
    base_q.npz      BaseQN planes packed and dequantised by the reference's numpy helpers
                    (`bindings/python/tk/base_q.py`) for every code width, scale storage and group size
"""
import ast
import os
import sys

import numpy as np


def main(ref_root: str) -> None:
    here = os.path.dirname(os.path.abspath(__file__))
    sys.path.insert(0, os.path.join(ref_root, "bindings", "python"))
    import tk  # noqa: E402  (lazy backends: importing needs neither MLX nor MPS)
    import tk.quant as q  # noqa: E402
    import torch  # noqa: E402

    fmts = ["q4_0", "q8_0", "q6_K", "mxfp8", "nvfp4", "mxfp4"]

    # ---- formats: reference quantize + dequantize on seeded Gaussians ----
    out = {}
    for i, fmt in enumerate(fmts):
        rng = np.random.default_rng(100 + i)
        W = (0.02 * rng.standard_normal((6, 512))).astype(np.float32)
        W[1, :32] = 0.0                      # an all-zero block
        W[2, 5] = 3.0                        # an outlier
        quant, dequant = q.QUANT_FORMATS[fmt]
        packed = quant(W)
        out[f"{fmt}_packed"] = packed
        out[f"{fmt}_dequant"] = dequant(packed).astype(np.float32)
    np.savez_compressed(os.path.join(here, "formats.npz"), **out)

    # ---- codec tables ----
    np.savez_compressed(
        os.path.join(here, "codecs.npz"),
        e4m3=q._e4m3_decode_arr(np.arange(256, dtype=np.uint8)),
        e2m1=q._e2m1_decode_arr(np.arange(16, dtype=np.uint8)),
    )

    # ---- RNG twin, lifted from the reference test file without importing it (it needs MLX) ----
    test_path = os.path.join(ref_root, "tests", "correctness", "quantization", "lm_head",
                             "test_lm_head.py")
    tree = ast.parse(open(test_path).read())
    ns = {"np": np}
    for node in tree.body:
        if isinstance(node, ast.FunctionDef) and node.name in ("_rng_uniform", "_gumbel"):
            exec(compile(ast.Module([node], []), test_path, "exec"), ns)
    keys = [(s, a, b) for s in (0, 3, 123, 0xFFFFFFFF) for a in (0, 1, 63) for b in
            (0, 1, 255, 256, 4000, 128255)]
    with np.errstate(over="ignore"):
        u = np.array([float(ns["_rng_uniform"](*k)) for k in keys], np.float32)
        g = np.array([float(ns["_gumbel"](*k)) for k in keys], np.float64)
    np.savez_compressed(os.path.join(here, "rng.npz"), keys=np.array(keys, np.uint64), u=u, g=g)

    # ---- reference torch-CPU composition (tk/__init__.py:3723-3735, :3776-3783) ----
    comp = {}
    for i, fmt in enumerate(fmts):
        rng = np.random.default_rng(200 + i)
        quant, dequant = q.QUANT_FORMATS[fmt]
        M, K, N = 3, 512, 40
        x = torch.from_numpy(rng.standard_normal((M, K)).astype(np.float32)).bfloat16()
        Wg = quant((0.02 * rng.standard_normal((N, K))).astype(np.float32))
        Wu = quant((0.02 * rng.standard_normal((N, K))).astype(np.float32))
        bias = torch.from_numpy((0.01 * rng.standard_normal(N)).astype(np.float32)).bfloat16()
        bias2 = torch.from_numpy((0.01 * rng.standard_normal(N)).astype(np.float32)).bfloat16()
        res = torch.from_numpy(rng.standard_normal((M, N)).astype(np.float32)).bfloat16()
        Wg_f = torch.from_numpy(dequant(Wg).astype(np.float32))
        Wu_f = torch.from_numpy(dequant(Wu).astype(np.float32))
        for act in ("none", "silu"):
            y = tk.decode_linear_epilogue(x, Wg_f, bias, res, activation=act, use_kernel=False)
            comp[f"{fmt}_lin_{act}"] = y.float().numpy()
        y = tk.decode_swiglu(x, Wg_f, Wu_f, bias, bias2, use_kernel=False)
        comp[f"{fmt}_swiglu"] = y.float().numpy()
        comp[f"{fmt}_x"] = x.float().numpy()
        comp[f"{fmt}_gate"] = Wg
        comp[f"{fmt}_up"] = Wu
        comp[f"{fmt}_bias"] = bias.float().numpy()
        comp[f"{fmt}_bias2"] = bias2.float().numpy()
        comp[f"{fmt}_res"] = res.float().numpy()
    np.savez_compressed(os.path.join(here, "compose.npz"), **comp)

    # ---- BaseQN separate planes: the reference's numpy pack + dequantise ----
    import tk.base_q as bq  # noqa: E402
    base = {}
    cases = [(bits, "f16", 32, sym) for bits in bq.BASE_Q_BITS for sym in (False, True)]
    cases += [(4, "bf16", 64, False), (4, "e8m0", 128, False), (8, "e4m3", 32, False), (3, "e8m0", 64, True)]
    for i, (bits, sd, group, sym) in enumerate(cases):
        rng = np.random.default_rng(300 + i)
        rows, K = 5, 256
        lanes = rng.integers(0, 1 << bits, size=(rows, K), dtype=np.uint8)
        G = K // group
        if sd in ("bf16", "f16"):
            sv = (0.002 + 0.02 * rng.random((rows, G))).astype(np.float32)
            bv = (-0.05 + 0.1 * rng.random((rows, G))).astype(np.float32)
            if sd == "f16":
                scales, biases = sv.astype(np.float16).view(np.uint16), bv.astype(np.float16).view(np.uint16)
            else:
                scales = torch.from_numpy(sv).bfloat16().view(torch.int16).numpy().view(np.uint16)
                biases = torch.from_numpy(bv).bfloat16().view(torch.int16).numpy().view(np.uint16)
        else:
            scales = rng.integers(1, 255, size=(rows, G), dtype=np.uint8) if sd == "e8m0" else \
                rng.integers(0, 256, size=(rows, G), dtype=np.uint8)
            biases = rng.integers(100, 140, size=(rows, G), dtype=np.uint8) if sd == "e8m0" else \
                rng.integers(0, 256, size=(rows, G), dtype=np.uint8)
        packed = bq.pack_base_q_codes(lanes, bits)
        key = f"b{bits}_{sd}_g{group}_{'sym' if sym else 'asym'}"
        base[key + "_lanes"] = lanes
        base[key + "_codes"] = packed
        base[key + "_scales"] = scales
        base[key + "_biases"] = biases
        with np.errstate(over="ignore", invalid="ignore"):
            base[key + "_dequant"] = bq.dequantize_base_q(packed, scales, None if sym else biases, bits, group, sd, sym)
    base["e8m0_table"] = bq.decode_e8m0(np.arange(256, dtype=np.uint8))
    base["e4m3_table"] = bq.decode_e4m3(np.arange(256, dtype=np.uint8))
    np.savez_compressed(os.path.join(here, "base_q.npz"), **base)
    print("golden fixtures written to", here)


if __name__ == "__main__":
    if len(sys.argv) != 2:
        sys.exit("usage: make_golden.py <reference checkout>")
    main(sys.argv[1])
