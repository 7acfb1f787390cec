"""Two tensor-parallel ranks on two GPUs; rank 1 leaves between steps.  Launched by tests/test_gpu_tp.py as
    python -m torch.distributed.run --nnodes=1 --nproc-per-node 2 --master-addr 127.0.0.1 --master-port P tests/tp_leave_worker.py
Every step is preceded by the host-side gate (bunker_b200.dist.StepGate).  After five steps rank 1 synchronises its
device (nothing of it in flight), announces that it leaves and exits.  Rank 0 must get PeerLost at the gate of step
5 -- on the host, before it launches anything -- with exactly five steps done, and its context must still work."""
import os
import sys
import time

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)

from bunker_b200 import dist  # noqa: E402
from bunker_b200 import model as M  # noqa: E402
from bunker_b200 import ops  # noqa: E402
from bunker_b200 import runtime as R  # noqa: E402


def main():
    rank, world = dist.init("nccl")
    assert world == 2
    local = int(os.environ.get("LOCAL_RANK", rank))
    R.cu(local)
    cfg = M.CONFIG_TINY.with_(max_len=64)
    w = M.synth_weights(cfg)
    gm = M.DecodeModel(cfg, w, batch=1, device=local, tp_rank=rank, tp_size=world)
    gate = dist.StepGate()
    tok = np.array([7], np.int32)
    done = 0
    try:
        for step in range(20):
            if rank == 1 and step == 5:
                assert R.cuSync() == 0, R.last_error()   # between steps: none of this rank's kernels in flight
                gate.leave()
                sys.stdout.flush()
                time.sleep(1.0)                           # let the peer read the note before the store's host goes quiet
                os._exit(0)
            gate.arrive(step, timeout_s=10.0)
            ids, _ = gm.step(tok)
            tok = ids
            done += 1
        print(f"rank {rank}: no peer loss seen", flush=True)
        os._exit(3)
    except dist.PeerLost as e:
        assert rank == 0 and done == 5 and "left before step 5" in str(e), (rank, done, str(e))
        # the context is still usable: the library's status word is clean and a single-GPU op runs
        assert R.cuSync() == 0, R.last_error()
        logits = R.DeviceBuffer.from_numpy(np.arange(4096, dtype=np.float32)[::-1].copy())
        idx, val = R.DeviceBuffer(4), R.DeviceBuffer(4)
        ops.argmax_static(logits.ptr, 4096, 1, idx.ptr, val.ptr)
        assert R.cuSync() == 0, R.last_error()
        assert int(idx.download(np.int32, (1,))[0]) == 0
        print("LEAVE OK: rank 0 learnt on the host, before its sixth launch, that rank 1 had left; context usable", flush=True)
        os._exit(0)   # no collective teardown with a peer that is gone


if __name__ == "__main__":
    main()
