"""Shared helpers for the parity tests."""
import numpy as np

from oracle import ref

TOL = 1e-5   # maximum relative error on f32 outputs and gradients


def gemm_errors(got: np.ndarray, a: np.ndarray, b: np.ndarray, ref32: np.ndarray | None = None) -> dict:
    """Error of a GEMM result against the f32-faithful oracle and the f64 yardstick.

    A dot product of k terms carries rounding error proportional to S = sum_k |a_ik||b_kj| (not to
    the possibly cancelled result), so the componentwise figure divides by S; the normwise figure
    divides by max|C|.  Both must stay <= TOL.  `f32_vs_f64` is the same componentwise figure for
    the reference's own sequential f32 loop, for comparison.
    """
    if ref32 is None:
        ref32 = ref.matmul(a, b)
    c64 = ref.matmul_f64(a, b)
    s = ref.matmul_absdot(a, b)
    s = np.maximum(s, np.finfo(np.float32).tiny)
    cmax = max(float(np.max(np.abs(c64))), np.finfo(np.float32).tiny)
    return dict(
        comp_vs_ref32=float(np.max(np.abs(got.astype(np.float64) - ref32) / s)),
        norm_vs_ref32=float(np.max(np.abs(got.astype(np.float64) - ref32)) / cmax),
        comp_vs_f64=float(np.max(np.abs(got - c64) / s)),
        norm_vs_f64=float(np.max(np.abs(got - c64)) / cmax),
        f32_vs_f64=float(np.max(np.abs(ref32 - c64) / s)),
        f32_norm_vs_f64=float(np.max(np.abs(ref32 - c64)) / cmax),
    )


def assert_gemm_close(got, a, b, ref32=None, what=""):
    e = gemm_errors(got, a, b, ref32)
    assert e["comp_vs_ref32"] <= TOL and e["norm_vs_ref32"] <= TOL, (what, e)
    # not worse than a few times the reference loop's own distance from the exact product; the floor is the
    # representation error of the split itself when the operands are split inside the kernel (the dropped
    # a_lo*b_lo term, up to 2^-20 |a b|, plus the rounding of the two lo parts, 2^-21 each: ~2e-6)
    assert e["comp_vs_f64"] <= max(4 * e["f32_vs_f64"], 2e-6), (what, e)
    return e


def rel_err(got, want) -> float:
    """max |got - want| / max(|want|, tiny): plain elementwise relative error."""
    got = np.asarray(got, np.float64)
    want = np.asarray(want, np.float64)
    denom = np.maximum(np.abs(want), 1e-30)
    return float(np.max(np.abs(got - want) / denom))


def scaled_err(got, want, scale) -> float:
    """max |got - want| / scale for reductions, where `scale` is the sum of |terms|."""
    return float(np.max(np.abs(np.asarray(got, np.float64) - np.asarray(want, np.float64)) / scale))
