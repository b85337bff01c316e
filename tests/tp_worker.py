"""Worker of the multi-GPU tensor-parallel test (one process per GPU, launched by torch.distributed.run):
runs the same small stack through NCCL collectives and through the fused peer-push kernels and compares."""
import os
import sys

import numpy as np
import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
from lutgemm_b200 import synth, tp_fused, tp_seq, tp_stack  # noqa: E402


def main():
    rank, world, local = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"]), int(os.environ["LOCAL_RANK"])
    torch.cuda.set_device(local)
    dist.init_process_group("nccl", device_id=torch.device(f"cuda:{local}"))
    H, F, Q, G, LAYERS = 1024, 2048, 3, 128, 3
    dev = f"cuda:{local}"
    plain = tp_stack.TPLinearStack(H, F, Q, G, LAYERS, rank=rank, world=world, device=dev, seed=1, generate="host")
    cls = tp_seq.SeqTPStack if "--seq" in sys.argv else tp_fused.FusedTPStack      # one launch per step / one per matvec
    fused = cls(H, F, Q, G, LAYERS, rank=rank, world=world, device=dev, seed=1, generate="host")
    x = torch.from_numpy(synth.activations(1, H, seed=4).view(np.int16)).cuda().view(torch.float16).reshape(-1)
    want = plain.step(x).float().cpu().numpy()
    ok = True
    worst = 0.0
    for rep in range(4):
        got = fused.step(x).float().cpu().numpy()
        err = float(np.abs(got - want).max() / (np.abs(want).max() + 1e-9))
        worst = max(worst, err)
        ok = ok and fused.device_status() == 0 and err <= 2e-3
    torch.cuda.synchronize()
    dist.barrier()
    print(f"TPRESULT rank={rank} ok={ok} worst={worst:.3e}", flush=True)
    fused.close()
    sys.stdout.flush()
    os._exit(0 if ok else 1)


if __name__ == "__main__":
    main()
