"""main.py command line on CPU: synthetic scene, train an epoch, evaluate only from the saved model."""
import os
import subprocess
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _run(args, cwd):
    env = dict(os.environ, PYTHONPATH=ROOT)
    for k in ("RANK", "WORLD_SIZE", "LOCAL_RANK"):
        env.pop(k, None)
    return subprocess.run([sys.executable, os.path.join(ROOT, "main.py")] + args, cwd=cwd, env=env, capture_output=True,
                          text=True, timeout=600)


def test_train_then_eval_only(tmp_path):
    model = str(tmp_path / "model")
    common = ["--synthetic", "uniform:n=3000:w=64:h=48:views=6:test=2:init=800:deg=1", "-m", model, "--bvh_depth", "1",
              "--MAX_BATCH_SIZE", "2", "--MAX_LOAD", "4", "--device", "cpu", "--eval", "--EVAL_PSNR_INTERVAL", "2"]
    r = _run(common + ["--epochs", "2", "--densify_from_iter", "100000"], str(tmp_path))
    assert r.returncode == 0, r.stdout[-2000:] + r.stderr[-2000:]
    assert "Evaluating test" in r.stdout and "Training complete." in r.stdout
    it = 12
    assert os.path.exists(os.path.join(model, "point_cloud", f"iteration_{it}", "point_cloud.ply"))
    assert os.path.exists(os.path.join(model, "rank_0", "cameras.json"))
    r2 = _run(common + ["--EVAL_ONLY", "--SAVE_EVAL_IMAGE", "--SAVE_EVAL_SUB_IMAGE"], str(tmp_path))
    assert r2.returncode == 0, r2.stdout[-2000:] + r2.stderr[-2000:]
    assert f"[ITER {it}] Evaluating test" in r2.stdout
    imgs = os.listdir(os.path.join(model, "img"))
    assert any(n.startswith("test_") and "_sub_" not in n for n in imgs) and any("_sub_1" in n for n in imgs)
    assert os.listdir(os.path.join(model, "gt"))


def test_failure_exits_non_zero(tmp_path):
    r = _run(["-s", str(tmp_path / "missing"), "-m", str(tmp_path / "m"), "--device", "cpu"], str(tmp_path))
    assert r.returncode != 0
    assert os.path.isdir(os.path.join(tmp_path, "debugger"))


def test_two_ranks_with_cost_assignment(tmp_path):
    """Four sub-models on two gloo ranks, placed by camera count instead of i % world; every sub-model is saved
    by exactly one rank and the merged model holds them all."""
    model = str(tmp_path / "model")
    env = dict(os.environ, PYTHONPATH=ROOT)
    for k in ("RANK", "WORLD_SIZE", "LOCAL_RANK"):
        env.pop(k, None)
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", "2", "--master-addr", "127.0.0.1",
           "--master-port", "29613", os.path.join(ROOT, "main.py"), "--synthetic",
           "uniform:n=3000:w=64:h=48:views=6:test=2:init=800:deg=1", "-m", model, "--bvh_depth", "2", "--MAX_BATCH_SIZE", "2",
           "--MAX_LOAD", "4", "--device", "cpu", "--eval", "--epochs", "1", "--densify_from_iter", "100000",
           "--MODEL_ASSIGNMENT", "cost"]
    r = subprocess.run(cmd, cwd=str(tmp_path), env=env, capture_output=True, text=True, timeout=900)
    assert r.returncode == 0, r.stdout[-2000:] + r.stderr[-2000:]
    assert "Training complete." in r.stdout
    owners = {}
    for rank in (0, 1):
        d = os.path.join(model, f"rank_{rank}", "point_cloud", "iteration_6")
        for n in os.listdir(d):
            if n.startswith("point_cloud_") and n.endswith(".ply"):
                owners.setdefault(int(n[len("point_cloud_"):-4]), []).append(rank)
    assert sorted(owners) == [0, 1, 2, 3] and all(len(v) == 1 for v in owners.values())
    assert {v[0] for v in owners.values()} == {0, 1}
    assert os.path.exists(os.path.join(model, "point_cloud", "iteration_6", "point_cloud.ply"))
