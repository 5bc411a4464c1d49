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
    print("golden fixtures written to", here)


if __name__ == "__main__":
    if len(sys.argv) != 2:
        sys.exit("usage: make_golden.py <reference checkout>")
    main(sys.argv[1])
