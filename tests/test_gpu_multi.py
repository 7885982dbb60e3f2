"""Multi-GPU fused paths (peer-memory lookup, owner-pull gradient update, in-kernel all-reduce).
Runs ``tests/multi_gpu_worker.py`` as child processes, one per GPU; skipped with fewer than 2 GPUs."""
import os
import subprocess
import sys

import pytest
import torch

pytestmark = pytest.mark.gpu
HERE = os.path.dirname(os.path.abspath(__file__))


def _run(nproc, extra, wire="fp32", **more_env):
    env = dict(os.environ)
    env.update(more_env)
    env["RECSDK_B200_ALLREDUCE_WIRE"] = wire     # equality tests keep fp32 on the wire; bf16 has its own case
    env.setdefault("NCCL_NVLS_ENABLE", "0")
    env.setdefault("TORCH_SYMM_MEM_DISABLE_MULTICAST", "1")
    env.setdefault("RECSDK_B200_MULTIMEM", "0")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", str(nproc),
           "--master-addr", "127.0.0.1", "--master-port", "29611", os.path.join(HERE, "multi_gpu_worker.py")] + extra
    p = subprocess.run(cmd, env=env, capture_output=True, text=True, timeout=600)
    sys.stdout.write(p.stdout[-4000:])
    sys.stderr.write(p.stderr[-4000:])
    return p


@pytest.mark.parametrize("graph", [False, True])
def test_sharded_dlrm_matches_single_gpu(graph):
    n = torch.cuda.device_count()
    if n < 2:
        pytest.skip("needs at least 2 GPUs")
    p = _run(min(n, 4) if min(n, 4) % 2 == 0 else 2, ["--graph"] if graph else [])
    assert p.returncode == 0 and "MULTI_GPU_RESULT PASS" in p.stdout


def test_push_allreduce_matches_nccl():
    n = torch.cuda.device_count()
    if n < 2:
        pytest.skip("needs at least 2 GPUs")
    p = _run(min(n, 8), ["--allreduce"])
    assert p.returncode == 0 and "MULTI_GPU_RESULT PASS" in p.stdout


def test_push_exchange_variable_length_bags():
    n = torch.cuda.device_count()
    if n < 2:
        pytest.skip("needs at least 2 GPUs")
    p = _run(min(n, 4) if min(n, 4) % 2 == 0 else 2, ["--varlen"])
    assert p.returncode == 0 and "MULTI_GPU_RESULT PASS" in p.stdout


def test_fused_dynamic_exchange_matches_collective_backend():
    n = torch.cuda.device_count()
    if n < 2:
        pytest.skip("needs at least 2 GPUs")
    p = _run(min(n, 4) if min(n, 4) % 2 == 0 else 2, ["--dynamic"])
    assert p.returncode == 0 and "MULTI_GPU_RESULT PASS" in p.stdout


def test_sharded_dlrm_deterministic_gradient_order():
    """``LCCL_DETERMINISTIC=1``: the owner orders its received entries by (source, feature, position) before the stable sort
    by row, so the sums do not depend on the arrival order; results still match the single-GPU run."""
    n = torch.cuda.device_count()
    if n < 2:
        pytest.skip("needs at least 2 GPUs")
    p = _run(2, [], LCCL_DETERMINISTIC="1")
    assert p.returncode == 0 and "MULTI_GPU_RESULT PASS" in p.stdout


def test_own_ipc_peer_backend():
    """``RECSDK_B200_PEER_BACKEND=ipc``: the peer buffers come from this package's own CUDA-IPC bootstrap instead of PyTorch
    symmetric memory; the push all-reduce and the sharded DLRM step give the same results on them."""
    n = torch.cuda.device_count()
    if n < 2:
        pytest.skip("needs at least 2 GPUs")
    p = _run(min(n, 4), ["--allreduce"], RECSDK_B200_PEER_BACKEND="ipc")
    assert p.returncode == 0 and "MULTI_GPU_RESULT PASS" in p.stdout
    p = _run(2, [], RECSDK_B200_PEER_BACKEND="ipc")
    assert p.returncode == 0 and "MULTI_GPU_RESULT PASS" in p.stdout
