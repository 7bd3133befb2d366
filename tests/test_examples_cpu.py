"""The runnable examples keep running (CPU paths)."""
import os
import runpy
import subprocess
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_single_device_example(capsys):
    runpy.run_path(os.path.join(ROOT, "examples", "single_gpu.py"), run_name="__main__")
    out = capsys.readouterr().out
    assert "max error against dense attention" in out and "checks: ok" in out


def test_context_parallel_example_on_two_cpu_ranks():
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", "2", "--master-addr",
           "127.0.0.1", "--master-port", str(29850 + os.getpid() % 40), os.path.join(ROOT, "examples", "context_parallel.py"),
           "--seq", "1024", "--pattern", "global_local"]
    env = dict(os.environ, CUDA_VISIBLE_DEVICES="")
    r = subprocess.run(cmd, capture_output=True, text=True, cwd=ROOT, env=env, timeout=300)
    assert r.returncode == 0, r.stderr[-2000:]
    lines = [ln for ln in r.stdout.splitlines() if "max error against dense attention" in ln]
    assert len(lines) == 2 and all(float(ln.rsplit(" ", 1)[1]) < 1e-4 for ln in lines), r.stdout


def test_reference_style_campaign_example_on_two_cpu_ranks(tmp_path):
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", "2", "--master-addr",
           "127.0.0.1", "--master-port", str(29890 + os.getpid() % 40),
           os.path.join(ROOT, "examples", "reference_style_campaign.py")]
    env = dict(os.environ, CUDA_VISIBLE_DEVICES="", UA_DATABASE_ROOT=str(tmp_path))
    r = subprocess.run(cmd, capture_output=True, text=True, cwd=ROOT, env=env, timeout=600)
    assert r.returncode == 0, r.stderr[-2000:]
    lines = [ln for ln in r.stdout.splitlines() if ln.startswith("fob=")]
    assert len(lines) == 2 and all("plan checks: ok" in ln for ln in lines), r.stdout
    assert "database: 5 ablation plans measured" in r.stdout, r.stdout[-2000:]
