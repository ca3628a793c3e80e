"""Tensor-parallel and data-parallel parity on 2 GPUs (skipped on a single-GPU box)."""
import os
import subprocess
import sys

import pytest
import torch

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("symmetric", ["1", "0"])
def test_tensor_and_data_parallel_match_the_oracle(symmetric):
    """symmetric = 1: exchange memory from the symmetric-memory allocator (multicast where the machine has it: the
    exchange then sums inside the NVLink switch); 0: the library's own CUDA-IPC buffers and plain peer loads."""
    if torch.cuda.device_count() < 2:
        pytest.skip("needs 2 GPUs")
    here = os.path.dirname(os.path.abspath(__file__))
    env = dict(os.environ, NCCL_NVLS_ENABLE="0", B200_TEST_SYMM=symmetric)
    r = subprocess.run([sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2",
                        "--master-addr", "127.0.0.1", "--master-port", "29533", os.path.join(here, "multi_gpu_worker.py")],
                       capture_output=True, text=True, timeout=600, env=env)
    assert r.returncode == 0 and "MULTI_GPU_OK 2" in r.stdout, r.stdout[-2000:] + r.stderr[-4000:]
    assert ("PEER_MEMORY 1" in r.stdout) if symmetric == "0" else ("PEER_MEMORY" in r.stdout), r.stdout[-500:]
