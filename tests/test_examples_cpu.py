"""The example scripts build their experiments and write prototext + launch script."""
import os
import subprocess
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _run(script, *args, cwd=None):
    env = dict(os.environ, PYTHONPATH=ROOT + os.pathsep + os.environ.get("PYTHONPATH", ""))
    return subprocess.run([sys.executable, os.path.join(ROOT, "examples", script)] + list(args), cwd=cwd, env=env,
                          capture_output=True, text=True, timeout=600)


def test_lenet_example_trains_on_synthetic_digits(tmp_path):
    r = _run("lenet.py", "--synthetic", "--num-epochs", "2", "--mini-batch-size", "64", "--work-dir", str(tmp_path),
             cwd=str(tmp_path))
    assert r.returncode == 0, r.stdout[-2000:] + r.stderr[-3000:]
    assert "training epoch 1 objective function" in r.stdout and "accuracy" in r.stdout


def test_distributed_examples_write_their_experiments(tmp_path):
    for script, extra, want in (
            ("cosmoflow.py", ["--procs-per-node", "4", "--depth-groups", "4", "--width", "32"], "depth_groups: 4"),
            ("unet3d.py", ["--procs-per-node", "4", "--depth-groups", "2", "--height-groups", "2", "--volume", "32",
                           "--levels", "2", "--base-channels", "4"], "height_groups: 2"),
            ("gpt.py", ["--procs-per-node", "2", "--layers", "2", "--d-model", "32", "--heads", "2", "--seq", "16",
                        "--vocab", "64", "--layer-parallel", "--lp-count", "2"], "grid_tag")):
        work = tmp_path / script
        r = _run(script, "--setup-only", "--work-dir", str(work), *extra, cwd=str(tmp_path))
        assert r.returncode == 0, script + r.stdout[-2000:] + r.stderr[-3000:]
        found = [os.path.join(d, f) for d, _, fs in os.walk(work) for f in fs if f.endswith(".prototext")]
        assert found, script
        assert want in open(found[0]).read(), script
