"""TEST INFRASTRUCTURE ONLY: numpy restatement of the reference's BCQ quantiser (greedy + alternating refinement).

Follows examples/bcq.py of the reference for the unweighted case it defaults to (exponent = 0, clipping = 1,
pruning = 0, i.e. wf = 1 everywhere):
  quantize            examples/bcq.py:23-98    (view as [rows, group_size]; greedy, then `rounds` refinements if q > 1)
  greedy              examples/bcq.py:100-128  (b = sign(r), alpha = mean |r|, r -= alpha b, per bit)
  refine              examples/bcq.py:130-157  (normal equations B^T B alpha = B^T w by q steps of CG from the current
                                                alpha, |alpha| sorted descending, then the nearest of the 2^q levels)
  find_B              examples/bcq.py:165-188  (levels sorted; q steps of bisection on midpoints; `w < mid` goes left)
  batch_cg            examples/bcq.py:190-206  (1e-6 added to both denominators)
  list_binary_vecs    examples/bcq.py:159-163  (row c, column i: -1 if bit q-1-i of c is set, else +1)
Pinned by tests/golden/bcq_quantizer_reference.npz, which tests/golden/make_bcq_golden.py made by calling the
reference's own greedy_mean_torch / refine_mean_torch on CPU tensors (its quantize() itself insists on .cuda()).
All arithmetic in float32; sums run in a different order than torch's, so alpha agrees to rounding and the
binary codes agree except for weights that sit on a decision boundary.
"""
import numpy as np

F = np.float32


def binary_matrix(q):
    c = np.arange(1 << q)[:, None]
    i = np.arange(q)[None, :]
    return np.where((c >> (q - 1 - i)) & 1, -1.0, 1.0).astype(F)          # [2^q, q]


def greedy(w, q):
    w = np.ascontiguousarray(w, dtype=F)
    R, g = w.shape
    B = np.zeros((R, g, q), F)
    alpha = np.zeros((R, q), F)
    r = w.copy()
    for i in range(q):
        b = np.sign(r).astype(F)
        a = (np.abs(r).sum(axis=1, dtype=F) / F(g)).astype(F)
        a[np.isnan(a)] = 0
        r -= b * a[:, None]
        B[:, :, i] = b
        alpha[:, i] = a
    return B, alpha


def batch_cg(A, b, x0):
    q = A.shape[1]
    x = x0.astype(F).copy()
    r = (b - np.einsum("rij,rj->ri", A, x)).astype(F)
    rtr_new = (r * r).sum(axis=1, dtype=F)
    p = r.copy()
    for _ in range(q):
        rtr = rtr_new
        Ap = np.einsum("rij,rj->ri", A, p).astype(F)
        a = (rtr / ((p * Ap).sum(axis=1, dtype=F) + F(1e-6))).astype(F)
        x += a[:, None] * p
        r -= a[:, None] * Ap
        rtr_new = (r * r).sum(axis=1, dtype=F)
        beta = (rtr_new / (rtr + F(1e-6))).astype(F)
        p = (r + beta[:, None] * p).astype(F)
    return x


def find_B(w, alpha):
    R, g = w.shape
    q = alpha.shape[1]
    bm = binary_matrix(q)
    v = (alpha @ bm.T).astype(F)                                           # [R, 2^q]
    inds = np.argsort(v, axis=1, kind="stable")
    vs = np.take_along_axis(v, inds, axis=1)
    left = np.zeros((R, g), np.int64)
    right = np.full((R, g), (1 << q) - 1, np.int64)
    rows = np.arange(R)[:, None]
    for _ in range(q):
        ml = (left + right - 1) // 2
        mr = ml + 1
        mid = ((vs[rows, ml] + vs[rows, mr]) / F(2)).astype(F)
        go_left = w < mid
        right = np.where(go_left, ml, right)
        left = np.where(go_left, left, mr)
    return bm[inds[rows, left]]                                            # [R, g, q]


def refine(w, B, alpha):
    Bt = np.transpose(B, (0, 2, 1))
    cov = (Bt @ B).astype(F)
    btw = np.einsum("rqg,rg->rq", Bt, w).astype(F)
    a = batch_cg(cov, btw, alpha)
    a = -np.sort(-np.abs(a), axis=1)
    return find_B(w, a), a.astype(F)


def quantize(w, q, rounds=15, group_size=-1):
    """w float32 [N, K] -> (w_hat [N, K], binary [N, G, g, q] in {-1, 0, +1}, alpha [N, G, q])."""
    w = np.ascontiguousarray(w, dtype=F)
    N, K = w.shape
    g = group_size if group_size > 0 else K
    wr = w.reshape(-1, g)
    B, alpha = greedy(wr, q)
    if rounds > 0 and q > 1:
        for _ in range(rounds):
            B, alpha = refine(wr, B, alpha)
    w_hat = np.einsum("rgq,rq->rg", B, alpha).astype(F).reshape(N, K)
    return w_hat, B.reshape(N, K // g, g, q), alpha.reshape(N, K // g, q)
