"""Two or more GPUs, one process each: the peer-to-peer compositing path against the single-GPU render."""
import os
import subprocess
import sys

import pytest
import torch

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.mark.skipif(not torch.cuda.is_available() or torch.cuda.device_count() < 2, reason="needs >= 2 GPUs")
@pytest.mark.parametrize("transport", ["peer", "nccl", "peer+occlusion", "nccl+occlusion"])
def test_multi_gpu_matches_single(tmp_path, transport):
    n = min(torch.cuda.device_count(), 4)
    n = 2 if n < 4 else 4
    env = dict(os.environ, NCCL_NVLS_ENABLE="0", PYTHONPATH=ROOT)
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={n}", "--master-addr",
           "127.0.0.1", "--master-port", str(29600 + os.getpid() % 300), os.path.join(ROOT, "tests", "multi_gpu_worker.py"),
           "--transport", transport.split("+")[0], "--out", str(tmp_path), "--occlusion", "1" if "+" in transport else "0"]
    proc = subprocess.run(cmd, env=env, capture_output=True, text=True, timeout=900)
    assert proc.returncode == 0, proc.stdout[-3000:] + proc.stderr[-3000:]
    assert "MULTI_GPU_OK" in proc.stdout


def _spawn_ranks(n, script, args, env_extra, timeout=600):
    port = 29300 + os.getpid() % 300
    procs = []
    for r in range(n):
        env = dict(os.environ, RANK=str(r), LOCAL_RANK=str(r), WORLD_SIZE=str(n), MASTER_ADDR="127.0.0.1",
                   MASTER_PORT=str(port), PYTHONPATH=ROOT, **env_extra)
        procs.append(subprocess.Popen([sys.executable, os.path.join(ROOT, "tests", script)] + args, env=env,
                                      stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True))
    outs = []
    for p in procs:
        try:
            out, _ = p.communicate(timeout=timeout)
        except subprocess.TimeoutExpired:
            p.kill()
            out, _ = p.communicate()
        outs.append(out)
    return [p.returncode for p in procs], outs


@pytest.mark.skipif(not torch.cuda.is_available() or torch.cuda.device_count() < 2, reason="needs >= 2 GPUs")
@pytest.mark.parametrize("mode", ["report", "silent"])
def test_rank_loss_is_detected_between_steps(mode):
    """A rank that leaves between steps (announced, or silently) is noticed by the survivor on the host before its
    next launch; the survivor's context stays usable."""
    codes, outs = _spawn_ranks(2, "rank_loss_worker.py", ["--mode", mode], dict(NCCL_NVLS_ENABLE="0"))
    assert codes == [0, 0], "\n".join(o[-2000:] for o in outs)
    assert "RANK_LOSS_DETECTED rank 0" in outs[0]
    assert "reported a failure" in outs[0] if mode == "report" else "no heartbeat" in outs[0]
