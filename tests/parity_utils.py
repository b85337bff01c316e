"""Shared helpers of the GPU parity tests."""
import numpy as np


def error_metrics(y, ref):
    """max relative error with floor 1e-2 * rms(ref) in the denominator, and mean absolute error."""
    y = np.asarray(y, dtype=np.float64)
    ref = np.asarray(ref, dtype=np.float64)
    rms = float(np.sqrt((ref ** 2).mean())) if ref.size else 0.0
    den = np.maximum(np.abs(ref), 1e-2 * rms + 1e-30)
    return float((np.abs(y - ref) / den).max()), float(np.abs(y - ref).mean())


MAX_REL = 1e-2      # tolerance of the matvec against the host dequant-and-matmul result
MAE = 1e-3          # on the fp16 output for k <= 12288 and on the fp32 output for every k
