"""Tensor-parallel decoder linear stack whose whole decode step is ONE kernel launch per GPU.

Same sharding and mathematics as tp_stack.TPLinearStack (column-parallel QKV / FC1 + all-gather, row-parallel
out-proj / FC2 + all-reduce), but the 4 x layers matvecs of a step are handed to lutgemm_sequence_run as one list:
a persistent kernel walks them, its weight stream never stops at a matvec boundary, and results travel between
matvecs and between GPUs in exchange lines that carry the step number (see csrc/gemv_seq.cuh).  No collective
library and no flag words on the data path; torch.distributed is used once, at set-up, to swap the 64-byte handles
of the ranks' exchange memory.
"""
from .tp_stack import TPLinearStack


class SeqTPStack(TPLinearStack):
    def __init__(self, *args, **kwargs):
        super().__init__(*args, **kwargs)
        import torch
        from .api import MatvecSequence
        P, r, h, f, L = self.world, self.rank, self.hidden, self.ffn, self.layers
        self.x_in = torch.zeros(h, dtype=torch.float16, device=self.device)     # the step's input: fill, then step()
        self._y16 = torch.zeros(h, dtype=torch.float16, device=self.device)
        buffers, ops = [], []
        for l in range(L):
            b_qkv, b_out, b_fc1, b_fc2 = 4 * l, 4 * l + 1, 4 * l + 2, 4 * l + 3
            buffers += [(1, 3 * h), (2, h), (1, f), (2, h)]
            wq, wo, w1, w2 = self.weights[l]
            if l == 0:
                ops.append(dict(w=wq, in_kind=0, x_ext=self.x_in, out_kind=1, out_buf=b_qkv, out_off=r * (3 * h // P)))
            else:
                ops.append(dict(w=wq, in_kind=2, in_buf=4 * (l - 1) + 3, out_kind=1, out_buf=b_qkv, out_off=r * (3 * h // P)))
            # the first `hidden` entries of the gathered QKV vector stand in for the attention result
            ops.append(dict(w=wo, in_kind=1, in_buf=b_qkv, in_off=r * (h // P), out_kind=2, out_buf=b_out))
            ops.append(dict(w=w1, in_kind=2, in_buf=b_out, out_kind=1, out_buf=b_fc1, out_off=r * (f // P)))
            ops.append(dict(w=w2, in_kind=1, in_buf=b_fc1, in_off=r * (f // P), out_kind=2, out_buf=b_fc2))
        ops.append(dict(w=None, in_kind=2, in_buf=4 * (L - 1) + 3, n=h, out_kind=0, y_ext=self._y16))
        self.seq = MatvecSequence(ops, buffers, rank=r, world=P)

    def step(self, x=None):
        """One decode step.  x: fp16 [hidden] (copied into self.x_in) or None when the caller has filled self.x_in."""
        if x is not None and x.data_ptr() != self.x_in.data_ptr():
            self.x_in.copy_(x)
        self.seq.run()
        return self._y16

    def device_status(self):
        return self.seq.status()

    def close(self):
        self.seq.close()
