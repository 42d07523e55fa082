"""Tensor-parallel path on real GPUs: spawns one worker per GPU (2, and 4/8 when present)."""
import os
import subprocess
import sys

import pytest
import torch

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _run(world: int, port: int):
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={world}",
           "--master-addr", "127.0.0.1", "--master-port", str(port), os.path.join(ROOT, "tests", "workers", "tp_worker.py")]
    env = dict(os.environ, NCCL_NVLS_ENABLE="0")
    r = subprocess.run(cmd, capture_output=True, text=True, timeout=900, env=env)
    assert r.returncode == 0, r.stdout[-3000:] + "\n" + r.stderr[-6000:]
    staged = os.path.exists(os.path.join(ROOT, "oracle", "_ref", "nanovllm", "__init__.py"))
    for rank in range(world):
        assert f"TP_WORKER_OK rank={rank}" in r.stdout
        if staged:  # the section that runs inside the reference's own sparse MoE block must not have been skipped
            assert f"TP_WORKER_REFERENCE_CALLER_OK rank={rank}" in r.stdout, r.stdout[-2000:]


@pytest.mark.parametrize("world", [2, 4, 8])
def test_tensor_parallel_block_and_all_reduce(world):
    if torch.cuda.device_count() < world:
        pytest.skip(f"needs {world} GPUs")
    _run(world, 29510 + world)


def test_bounded_wait_reports_instead_of_hanging():
    """A flag that nobody advances: the wait gives up after its limit and leaves a status word."""
    import ctypes
    from layered_prefill_b200 import ops
    from layered_prefill_b200._lib import check, lib
    dev = torch.device("cuda", 0)
    meta = torch.zeros(ops.meta_size(), dtype=torch.uint8, device=dev)
    status = torch.zeros(1, dtype=torch.int32, device=dev)
    check(lib.moe_b200_ar_wait_probe(meta.data_ptr(), 200_000, status.data_ptr(),
                                     torch.cuda.current_stream().cuda_stream))
    v = ctypes.c_int32(0)
    check(lib.moe_b200_read_status(status.data_ptr(), ctypes.byref(v), torch.cuda.current_stream().cuda_stream))
    assert v.value == 6
    # the context is still usable
    assert float(torch.ones(4, device=dev).sum()) == 4.0
