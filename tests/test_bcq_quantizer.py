"""BCQ quantiser (the step before the matmul path): oracle pinned on vectors made by the reference's own code;
the device quantiser against the oracle and the same vectors."""
import os

import numpy as np
import pytest

from oracle import bcq_quantizer as bq

GOLD = np.load(os.path.join(os.path.dirname(__file__), "golden", "bcq_quantizer_reference.npz"))
CASES = sorted({k.rsplit("_", 1)[0] for k in GOLD.files})


def _cfg(name):
    N, K, g, q, rounds, _ = (int(v) for v in GOLD[name + "_cfg"])
    return N, K, g, q, rounds


def _compare(alpha, B, alpha_ref, B_ref, w):
    """alpha to fp32 summation-order rounding; codes equal except for weights on a decision boundary, and the
    reconstruction error no worse."""
    assert np.allclose(alpha, alpha_ref, rtol=2e-5, atol=1e-9), np.abs(alpha - alpha_ref).max()
    mismatch = (B != B_ref).any(-1).mean()
    assert mismatch <= 2e-3, mismatch
    N = w.shape[0]
    rec = np.einsum("ngkq,ngq->ngk", B.astype(np.float32), alpha).reshape(N, -1)
    rec_ref = np.einsum("ngkq,ngq->ngk", B_ref.astype(np.float32), alpha_ref).reshape(N, -1)
    e, e_ref = ((rec - w) ** 2).mean(), ((rec_ref - w) ** 2).mean()
    assert e <= e_ref * (1 + 1e-4) + 1e-12, (e, e_ref)


@pytest.mark.parametrize("name", CASES)
def test_oracle_matches_reference_vectors(name):
    N, K, g, q, rounds = _cfg(name)
    w = GOLD[name + "_w"]
    w_hat, B, alpha = bq.quantize(w, q, rounds, g)
    _compare(alpha, B.astype(np.int8), GOLD[name + "_alpha"], GOLD[name + "_B"], w)
    assert np.abs(w_hat - GOLD[name + "_ret"]).max() <= 1e-6


def test_refinement_does_not_increase_the_error():
    rng = np.random.default_rng(0)
    w = rng.normal(0, 0.02, (16, 512)).astype(np.float32)
    errs = [((bq.quantize(w, 3, r, 128)[0] - w) ** 2).mean() for r in (0, 1, 5)]
    assert errs[1] <= errs[0] and errs[2] <= errs[1] * 1.001, errs


@pytest.mark.gpu
@pytest.mark.parametrize("name", CASES)
def test_device_quantiser_matches_reference_vectors(name):
    import lutgemm_b200 as L
    N, K, g, q, rounds = _cfg(name)
    w = GOLD[name + "_w"]
    w_hat, B, alpha = L.bcq_quantize(w, q, rounds, g)
    _compare(alpha, B, GOLD[name + "_alpha"], GOLD[name + "_B"], w)


@pytest.mark.gpu
@pytest.mark.parametrize("N,K,g,q,rounds", [(64, 1024, 128, 3, 15), (48, 768, 32, 4, 6), (8, 2048, 1024, 2, 3),
                                             (33, 640, 64, 8, 2), (16, 4096, 256, 5, 4),
                                             # groups wider than 1024: the CTA-per-group kernel (-1 = one group per row)
                                             (6, 4096, -1, 3, 5), (5, 6144, 2048, 4, 3), (3, 12288, -1, 2, 2), (4, 2080, -1, 1, 0)])
def test_device_quantiser_matches_oracle(N, K, g, q, rounds):
    import lutgemm_b200 as L
    rng = np.random.default_rng(N + K + q)
    w = (rng.standard_t(5, (N, K)) * 0.02).astype(np.float32)
    _, B_ref, alpha_ref = bq.quantize(w, q, rounds, g)
    _, B, alpha = L.bcq_quantize(w, q, rounds, g)
    _compare(alpha, B, alpha_ref, B_ref.astype(np.int8), w)


@pytest.mark.gpu
def test_device_quantiser_feeds_the_matmul():
    """Quantise on the device straight into the container layout, multiply, compare with x W_hat^T from the oracle."""
    import torch
    import lutgemm_b200 as L
    from lutgemm_b200 import synth
    from parity_utils import MAE, MAX_REL, error_metrics
    N, K, g, q = 512, 1024, 128, 3
    rng = np.random.default_rng(3)
    w = rng.normal(0, 0.02, (N, K)).astype(np.float32)
    bW, alpha = L.bcq_quantize_device(torch.from_numpy(w).cuda(), q, rounds=5, group_size=g)
    nq = L.nQWeight_fp16.from_device(bW, alpha, None, K, N, q, False, K // g, copy=False)
    x = synth.activations(1, K, seed=1)
    y = torch.empty((1, N), dtype=torch.float16, device="cuda")
    L.matmul(y, torch.from_numpy(x.view(np.int16)).cuda().view(torch.float16), nq, 1)
    _, B_ref, alpha_ref = bq.quantize(w, q, 5, g)
    a16 = alpha_ref.astype(np.float16).astype(np.float32)
    w_hat16 = np.einsum("ngkq,ngq->ngk", B_ref, a16).reshape(N, K)
    ref = x.astype(np.float32) @ w_hat16.T
    rel, mae = error_metrics(y.float().cpu().numpy(), ref)
    assert rel <= 2 * MAX_REL and mae <= 2 * MAE, (rel, mae)       # a few boundary codes may differ from the oracle's
