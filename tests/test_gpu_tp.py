"""Tensor-parallel decoding on the GPUs of this box (skipped with fewer than two)."""
import os
import subprocess
import sys

import pytest

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def gpus() -> int:
    import torch

    return torch.cuda.device_count()


@pytest.mark.parametrize("comm", ["peer", "nccl", "peer-folded", "peer-persistent", "peer-whole", "nccl-whole"])
@pytest.mark.parametrize("world", [2, 4, 8])
def test_a_split_model_decodes_the_oracles_tokens(world, comm):
    if gpus() < world:
        pytest.skip(f"{world} GPUs are not here")
    # peer-folded: the exchanges ride in the epilogues of the row-parallel products; peer-persistent: the whole step
    # is one cooperative kernel a rank, exchanges and the choice among the ranks' winners inside it; -whole: every rank
    # keeps the whole attention block, only the MLP and the head are split
    env = dict(os.environ, TP_CHECK_LIMIT="150", NCCL_NVLS_ENABLE="0", TP_COMM=comm.split("-")[0],
               TP_FOLD="1" if comm.endswith("folded") else "0", TP_STEP="persistent" if comm.endswith("persistent") else "graph", TP_ATTENTION="whole" if comm.endswith("whole") else "split",
               TP_CHECK_LOG=os.path.join(ROOT, "gpurun_out", "tp_decode_check.log"))
    run = subprocess.run(
        [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={world}", "--master-addr",
         "127.0.0.1", "--master-port", str(29540 + world), os.path.join(ROOT, "tests", "tp_decode_check.py")],
        capture_output=True, text=True, timeout=300, env=env, cwd=ROOT)
    assert run.returncode == 0 and f"tp{world}: 64 greedy tokens" in run.stdout, run.stdout[-2000:] + run.stderr[-2000:]
