"""Generates the committed fixtures under tests/golden/ from the REFERENCE itself.

Run once in a container that has the reference tree (default /root/reference):
    python tests/golden/make_golden.py
It (1) imports the reference's Python converter and packer
(examples/rtn_parameter.py, examples/bcq_parameter.py, examples/utils.py) on CPU
torch and records their outputs on seeded inputs, and (2) calls the reference's
own lutGEMM::dequantize_cpu (compiled unmodified into oracle/_ref/) on seeded
containers.  The tests then check the C oracle, and through it the CUDA
library, against these files; the reference tree is not needed to run them.
"""
import os
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
REF = os.environ.get("LUTGEMM_REFERENCE", "/root/reference")
sys.path.insert(0, ROOT)
sys.path.insert(0, os.path.join(REF, "examples"))


def converter_fixture():
    import torch
    from rtn_parameter import RTNParameter
    from bcq_parameter import BCQParameter
    from utils import Packer

    out = {}
    for tag, (N, K, g, q, seed) in {"a": (16, 256, 128, 4, 1), "b": (8, 128, 32, 3, 2), "c": (6, 192, 64, 2, 3)}.items():
        rng = np.random.default_rng(seed)
        G = K // g
        scale = np.abs(rng.standard_normal((N, G, 1)).astype(np.float32) * 0.01).astype(np.float16).astype(np.float32)
        zero = rng.integers(0, 2**q, size=(N, G, 1)).astype(np.float32)
        code = rng.integers(0, 2**q, size=(N, G, g), dtype=np.int32)
        p = RTNParameter(torch.zeros(N, K))
        alpha, binary, bshape, offset = p.convert_bcq_format(
            torch.from_numpy(scale), torch.from_numpy(zero), torch.from_numpy(code), qbits=q,
            do_packing=False, in_ch_wise=False)
        # dense reconstruction through the reference's own BCQ decompress
        w = BCQParameter(torch.zeros(N, K))
        w.decompress(alpha, binary, bshape, offset=offset, do_packing=False, in_ch_wise=False)
        packed, pshape = Packer().pack(binary)
        unpacked = Packer().unpack(packed.clone(), pshape, dtype=torch.float32)
        assert torch.equal(unpacked, binary)
        out.update({
            f"{tag}_scale": scale, f"{tag}_zero": zero, f"{tag}_code": code, f"{tag}_q": np.int32(q),
            f"{tag}_alpha": alpha.numpy().astype(np.float32),
            f"{tag}_binary": binary.numpy().astype(np.int8),
            f"{tag}_offset": offset.numpy().astype(np.float32),
            f"{tag}_dense": w.data.detach().numpy().astype(np.float32),
            f"{tag}_packed_u8": packed.numpy().astype(np.uint8),
        })
    np.savez_compressed(os.path.join(HERE, "converter_reference.npz"), **out)
    print("converter_reference.npz:", len(out), "arrays")


def dequant_fixture():
    from oracle import oracle
    from lutgemm_b200 import synth

    assert oracle.ref_cpu() is not None, "oracle/_ref not built (run make -C oracle)"
    out = {}
    cases = {"s0": (64, 128, 3, 32, False), "s1": (48, 256, 4, 128, False), "s2": (10, 64, 1, 64, False),
             "s3": (34, 96, 8, 32, False), "s4": (32, 128, 2, 128, True)}
    for tag, (N, K, q, g, row_wise) in cases.items():
        bW, alpha, _ = synth.bcq_layer(N, K, q, g, seed=synth.seed_for("golden", N, K, q), signed_alpha=True)
        W = oracle.dequantize_cpu(bW, alpha.astype(np.float16), g, row_wise=row_wise, use_reference=True)
        out.update({f"{tag}_bW": bW, f"{tag}_alpha": alpha.astype(np.float16), f"{tag}_g": np.int32(g),
                    f"{tag}_row_wise": np.int32(row_wise), f"{tag}_W": W})
    np.savez_compressed(os.path.join(HERE, "dequantize_cpu_reference.npz"), **out)
    print("dequantize_cpu_reference.npz:", len(out), "arrays")


if __name__ == "__main__":
    converter_fixture()
    dequant_fixture()
