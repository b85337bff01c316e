"""Tensor-parallel decoder linear stack whose whole decode step is ONE kernel launch per GPU.

Same sharding and mathematics as tp_stack.TPLinearStack (column-parallel QKV / FC1 + all-gather, row-parallel
out-proj / FC2 + all-reduce), but the 4 x layers matvecs of a step are handed to lutgemm_sequence_run as one list:
a persistent kernel walks them, its weight stream never stops at a matvec boundary, and results travel between
matvecs and between GPUs in exchange lines that carry the step number (see csrc/gemv_seq.cuh).  No collective
library and no flag words on the data path; torch.distributed is used once, at set-up, to swap the 64-byte handles
of the ranks' exchange memory.
"""
from .tp_stack import TPLinearStack


def stack_program(hidden, ffn, layers, rank, world):
    """The decode step of the stack as a list for lutgemm_sequence_create: (buffers, ops).

    buffers: (kind, n) per layer: gathered QKV vector, out-proj rows, gathered FC1 vector, FC2 rows.
    ops: dicts with the matvec's place in the stack ("layer", "idx" 0..3 = QKV, out-proj, FC1, FC2; idx None = the
    closing step that adds the last rows) and its in_* / out_* fields; the caller adds "w", "x_ext", "y_ext"."""
    P, r, h, f = world, rank, hidden, ffn
    buffers, ops = [], []
    for l in range(layers):
        b_qkv, b_out, b_fc1, b_fc2 = 4 * l, 4 * l + 1, 4 * l + 2, 4 * l + 3
        buffers += [(1, 3 * h), (2, h), (1, f), (2, h)]
        if l == 0:
            ops.append(dict(layer=l, idx=0, in_kind=0, out_kind=1, out_buf=b_qkv, out_off=r * (3 * h // P)))
        else:
            ops.append(dict(layer=l, idx=0, in_kind=2, in_buf=4 * (l - 1) + 3, out_kind=1, out_buf=b_qkv, out_off=r * (3 * h // P)))
        # the first `hidden` entries of the gathered QKV vector stand in for the attention result
        ops.append(dict(layer=l, idx=1, in_kind=1, in_buf=b_qkv, in_off=r * (h // P), out_kind=2, out_buf=b_out))
        ops.append(dict(layer=l, idx=2, in_kind=2, in_buf=b_out, out_kind=1, out_buf=b_fc1, out_off=r * (f // P)))
        ops.append(dict(layer=l, idx=3, in_kind=1, in_buf=b_fc1, in_off=r * (f // P), out_kind=2, out_buf=b_fc2))
    ops.append(dict(layer=layers - 1, idx=None, in_kind=2, in_buf=4 * (layers - 1) + 3, n=h, out_kind=0))
    return buffers, ops


class SeqTPStack(TPLinearStack):
    def __init__(self, *args, **kwargs):
        super().__init__(*args, **kwargs)
        import torch
        from .api import MatvecSequence
        h = self.hidden
        self.x_in = torch.zeros(h, dtype=torch.float16, device=self.device)     # the step's input: fill, then step()
        self._y16 = torch.zeros(h, dtype=torch.float16, device=self.device)
        buffers, ops = stack_program(self.hidden, self.ffn, self.layers, self.rank, self.world)
        for o in ops:
            o["w"] = None if o["idx"] is None else self.weights[o["layer"]][o["idx"]]
            if o["in_kind"] == 0:
                o["x_ext"] = self.x_in
            if o["out_kind"] == 0:
                o["y_ext"] = self._y16
        self.seq = MatvecSequence(ops, buffers, rank=self.rank, world=self.world)

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
