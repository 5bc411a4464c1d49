"""Shared helpers for the parity tests: seeded inputs, dtype plumbing, tie-aware id comparison."""
import numpy as np
import torch

from oracle import qx_oracle as O

FMTS = ["q4_0", "q8_0", "q6_K", "mxfp8", "nvfp4", "mxfp4"]
TORCH_DT = {"f32": torch.float32, "f16": torch.float16, "bf16": torch.bfloat16}


def rounded(a: np.ndarray, dtype: str) -> np.ndarray:
    """fp32 array holding values already rounded to the I/O dtype (what both sides consume)."""
    return O.round_to(np.asarray(a, np.float32), dtype)


def dev(a: np.ndarray, dtype: str = None):
    t = torch.from_numpy(np.ascontiguousarray(a)).cuda()
    return t.to(TORCH_DT[dtype]) if dtype else t


def host(t: torch.Tensor) -> np.ndarray:
    return t.detach().float().cpu().numpy() if t.is_floating_point() else t.detach().cpu().numpy()


def assert_close_dtype(got: np.ndarray, ref: np.ndarray, dtype: str, scale: float = 1.0):
    """f32: 2e-5 relative to the row scale; f16/bf16: at most one ulp of the output format (the
    GPU accumulates in fp32, the oracle in fp64, so a value next to a rounding boundary may land
    on either side), with the large majority exact."""
    got = np.asarray(got, np.float64); ref = np.asarray(ref, np.float64)
    if dtype == "f32":
        tol = 2e-5 * (np.abs(ref) + scale)
        assert np.all(np.abs(got - ref) <= tol), float(np.max(np.abs(got - ref) - tol))
        return
    ulp = 2.0 ** (-7 if dtype == "bf16" else -10)
    # absolute term: fp32 accumulation noise (~1e-6 of the pre-activation scale) decides the
    # rounding of outputs that cancel to nearly zero
    tol = np.abs(ref) * ulp * 1.01 + 2e-5 * scale
    bad = np.abs(got - ref) > tol
    assert not bad.any(), (int(bad.sum()), float(np.max(np.abs(got - ref))))
    assert np.mean(got == ref) > 0.9, float(np.mean(got == ref))


def check_ids(got: np.ndarray, want: np.ndarray, margin: np.ndarray, eps: float, what: str = ""):
    """Token ids must be identical wherever the oracle's decision margin exceeds eps; rows whose
    margin is below eps are fp32-order near-ties (the reference's own tests accept those,
    tests/correctness/quantization/lm_head/test_lm_head.py:1-11).  Returns the exact-match count."""
    got = np.asarray(got); want = np.asarray(want)
    exact = got == want
    decided = margin > eps
    assert np.all(exact | ~decided), (what, np.nonzero(~exact & decided)[0][:8], got[~exact][:8], want[~exact][:8])
    return int(exact.sum())
