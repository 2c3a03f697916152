"""The CPU-runnable examples still run."""
import os
import subprocess
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_weight_sync_example_on_host_memory():
    res = subprocess.run([sys.executable, os.path.join(ROOT, "examples", "weight_sync.py")], capture_output=True, text=True,
                         timeout=180)
    assert res.returncode == 0, res.stdout[-2000:] + res.stderr[-2000:]
    assert "replica: pulled 8 tensors" in res.stdout and "8 tensors verified" in res.stdout


def test_fsdp_device_mesh_example_on_gloo():
    from tests.mp_util import free_port

    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", "2", "--master-addr", "127.0.0.1",
           "--master-port", str(free_port()), os.path.join(ROOT, "examples", "fsdp_device_mesh.py"), "--steps", "2"]
    res = subprocess.run(cmd, capture_output=True, text=True, timeout=240)
    assert res.returncode == 0, res.stdout[-2000:] + res.stderr[-2000:]
    assert "step 1: loss" in res.stdout


def test_package_report_runs_without_a_gpu():
    res = subprocess.run([sys.executable, "-m", "torchcomms_b200"], capture_output=True, text=True, timeout=120, cwd=ROOT)
    assert res.returncode == 0, res.stderr[-2000:]
    assert "backends" in res.stdout and "gloo" in res.stdout and "extension" in res.stdout
