"""Shared helpers of the GPU parity tests."""
import numpy as np


def error_metrics(y, ref, floor=1e-2):
    """max relative error, |y - ref| / max(|ref|, floor * rms(ref)), and mean absolute error."""
    y = np.asarray(y, dtype=np.float64)
    ref = np.asarray(ref, dtype=np.float64)
    rms = float(np.sqrt((ref ** 2).mean())) if ref.size else 0.0
    den = np.maximum(np.abs(ref), floor * rms + 1e-30)
    return float((np.abs(y - ref) / den).max()), float(np.abs(y - ref).mean())


# Tolerance of the matvec against the reference's fp32 host dequant-and-matmul
# (oracle.bcq_matmul_fp32): fp16 output, fp32 reference.
MAX_REL = 1e-2
MAE = 1e-3          # on the fp16 output for k <= 12288, on the fp32 output for every k: for larger k the
                    # fp16 rounding of an exact result alone exceeds 1e-3 (|y| grows as sqrt(k))
# Against the host path that goes through lutGEMM::dequantize_cpu (oracle.bcq_matmul_ref) the dense
# weight is itself rounded to fp16, a +-2^-12 relative perturbation of every weight; the relative error
# is then taken with a floor of 0.1 * rms(ref) in the denominator.
REF16_FLOOR = 0.1


def assert_parity(y, ref, K, what=""):
    """The matvec tolerance: max relative error on the fp16 output, MAE where fp16 rounding allows it."""
    rel, mae = error_metrics(y, ref)
    assert rel <= MAX_REL, f"{what}: max rel err {rel:.3e}"
    if K <= 12288:
        assert mae <= MAE, f"{what}: MAE {mae:.3e}"
