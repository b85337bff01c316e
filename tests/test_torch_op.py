"""torch operator / module over the C ABI (the caller's side of the path).  CPU: registration, shape propagation,
no CPU fallback.  GPU: results against the oracle."""
import numpy as np
import pytest
import torch

from lutgemm_b200 import synth, torch_op
from oracle import oracle
from parity_utils import MAE, MAX_REL, error_metrics


def test_fake_implementation_propagates_shapes():
    x = torch.empty((2, 3, 256), dtype=torch.float16, device="meta")
    bW = torch.empty((8, 3, 512), dtype=torch.int32, device="meta")
    alpha = torch.empty((2, 3, 512), dtype=torch.float16, device="meta")
    y = torch.ops.lutgemm_b200.bcq_linear(x, bW, alpha, None)
    assert tuple(y.shape) == (2, 3, 512) and y.dtype == torch.float16


def test_no_cpu_kernel_behind_the_operator():
    x = torch.zeros((1, 64), dtype=torch.float16)
    bW = torch.zeros((2, 1, 8), dtype=torch.int32)
    alpha = torch.zeros((1, 1, 8), dtype=torch.float16)
    with pytest.raises((NotImplementedError, RuntimeError)):
        torch.ops.lutgemm_b200.bcq_linear(x, bW, alpha, None)


def _python_layout(N, K, g, q, seed):
    """Tensors as convert_bcq_format / BCQParameter.compress hand them over (in_ch_wise False)."""
    rng = np.random.default_rng(seed)
    G = K // g
    alpha = np.abs(rng.normal(0, 0.02, (N, G, q))).astype(np.float32)
    binary = (rng.integers(0, 2, (N, G, g, q)) * 2 - 1).astype(np.int8)
    offset = rng.normal(0, 0.01, (N, G)).astype(np.float32)
    return alpha, binary, offset


@pytest.mark.gpu
@pytest.mark.parametrize("lead", [(1,), (7,), (2, 4)])
def test_module_from_python_layout_matches_oracle(lead):
    N, K, g, q = 512, 1024, 128, 3
    alpha, binary, offset = _python_layout(N, K, g, q, seed=5)
    lin = torch_op.BCQLinear.from_python_layout(torch.from_numpy(alpha), torch.from_numpy(binary), torch.from_numpy(offset)[..., None])
    m = int(np.prod(lead))
    x = synth.activations(m, K, seed=m)
    y = lin(torch.from_numpy(x.view(np.int16)).cuda().view(torch.float16).reshape(*lead, K))
    assert tuple(y.shape) == (*lead, N)
    # dense reference from the quantiser's own identity: W[n][k] = sum_i alpha[n][G][i] binary[n][G][k%g][i] + offset[n][G]
    a16 = alpha.astype(np.float16).astype(np.float32)
    o16 = offset.astype(np.float16).astype(np.float32)
    W = (a16[:, :, None, :] * binary).sum(-1) + o16[:, :, None]          # [N, G, g]
    ref = x.astype(np.float32) @ W.reshape(N, K).T
    rel, mae = error_metrics(y.float().cpu().numpy().reshape(m, N), ref)
    assert rel <= MAX_REL and mae <= MAE, (rel, mae)
    torch_op.release_containers()


@pytest.mark.gpu
def test_module_from_uniform_matches_rtn_dequantisation():
    N, K, g, q = 256, 512, 128, 4
    rng = np.random.default_rng(9)
    G = K // g
    scale = np.abs(rng.normal(0, 0.01, (N, G))).astype(np.float32)
    zero = rng.integers(0, 16, (N, G)).astype(np.float32)
    code = rng.integers(0, 16, (N, G, g)).astype(np.int32)
    lin = torch_op.BCQLinear.from_uniform(scale, zero, code, q)
    x = synth.activations(3, K, seed=2)
    y = lin(torch.from_numpy(x.view(np.int16)).cuda().view(torch.float16))
    alpha_k, bW, qb = oracle.python_to_kernel_layout(*oracle.uniform_to_bcq(scale, zero, code, q))
    ref = oracle.bcq_matmul_fp32(x, bW, alpha_k.astype(np.float16), qb.astype(np.float16), g)
    rel, mae = error_metrics(y.float().cpu().numpy(), ref)
    assert rel <= MAX_REL and mae <= MAE, (rel, mae)
    torch_op.release_containers()
