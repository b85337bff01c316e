"""Makes tests/golden/bcq_quantizer_reference.npz from the reference's own code (run where the reference tree is mounted).

Imports examples/bcq.py of the reference and calls greedy_mean_torch and refine_mean_torch on CPU tensors in the
order quantize() does (examples/bcq.py:74-80, with wf = 1: the defaults exponent = 0, clipping = 1, pruning = 0);
quantize() itself cannot run without a GPU because it moves the weight with .cuda() (examples/bcq.py:45).

usage: python tests/golden/make_bcq_golden.py <reference root>
"""
import os
import sys

import numpy as np
import torch

CASES = [  # (name, N, K, group_size, q, rounds, seed)
    ("q3_g64_r0", 8, 256, 64, 3, 0, 1),
    ("q3_g128_r3", 8, 256, 128, 3, 3, 2),
    ("q4_g128_r15", 6, 384, 128, 4, 15, 3),
    ("q2_row_r5", 5, 320, -1, 2, 5, 4),
    ("q1_g32_r5", 4, 128, 32, 1, 5, 5),
    ("q6_g256_r4", 3, 512, 256, 6, 4, 6),
]


def main(ref_root):
    sys.path.insert(0, os.path.join(ref_root, "examples"))
    import bcq
    out = {}
    for name, N, K, g, q, rounds, seed in CASES:
        gen = torch.Generator().manual_seed(seed)
        w = (torch.randn(N, K, generator=gen) * 0.02).float()
        gs = g if g > 0 else K
        w_ = w.view(-1, gs).clone()
        wf = torch.ones(w_.shape, dtype=torch.float32)
        ret, B, alpha = bcq.greedy_mean_torch(w_, n_bits=q, wf=wf)
        if rounds > 0 and q > 1:
            for _ in range(rounds):
                ret, B, alpha = bcq.refine_mean_torch(w_, ret, B, alpha, wf=wf, use_bst=True)
        out[name + "_w"] = w.numpy()
        out[name + "_ret"] = ret.reshape(N, K).numpy().astype(np.float32)
        out[name + "_B"] = B.reshape(N, K // gs, gs, q).numpy().astype(np.int8)
        out[name + "_alpha"] = alpha.reshape(N, K // gs, q).numpy().astype(np.float32)
        out[name + "_cfg"] = np.array([N, K, g, q, rounds, seed], np.int64)
    np.savez_compressed(os.path.join(os.path.dirname(os.path.abspath(__file__)), "bcq_quantizer_reference.npz"), **out)
    print("wrote", len(CASES), "cases")


if __name__ == "__main__":
    main(sys.argv[1] if len(sys.argv) > 1 else "/root/reference")
