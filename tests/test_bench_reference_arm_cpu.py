"""The reference arm of bench.py (the CPU oracle timed on the host cores) without a GPU: alone and
launched as two ranks by torch.distributed.run, where rank 0 alone works and prints the line and the
oracle still uses all host threads (the launcher sets OMP_NUM_THREADS=1 for its children)."""
import json
import os
import subprocess
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
SMALL = ["--impl", "reference", "--steps", "1", "--warmup", "0", "--cpu-sample", "1x32+2", "--layers", "2", "--vocab", "1024"]


def _lines(out: str):
    return [json.loads(ln) for ln in out.splitlines() if ln.startswith("{")]


def _check(line, n_gpus):
    assert line["impl"] == "reference" and line["n_gpus"] == n_gpus and line["gpu_launches"] == 0
    assert line["metric"] == "qwen3_0.6b_bf16_prefill_decode_tokens_per_s" and line["unit"] == "tokens/s"
    assert line["higher_is_better"] is True and line["vs_baseline"] is None and line["dtype"] == "f32"
    assert line["value"] > 0 and line["ms_per_step"] > 0 and line["config"]["workload"].startswith("qwen3-0.6b-bf16-b32-p2048-d256")
    cb = line["cpu_baseline"]
    assert cb["kind"] == "port" and cb["value"] == line["value"] and "1 sequence(s) x 32 prompt tokens" in cb["sample"]
    assert cb["cores"] == (os.cpu_count() or 1)
    assert line["e2e"] == {"value": line["value"], "unit": "tokens/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}


def test_reference_arm_single_process():
    r = subprocess.run([sys.executable, os.path.join(ROOT, "bench.py"), *SMALL], capture_output=True, text=True, timeout=600, cwd=ROOT)
    assert r.returncode == 0, r.stderr[-2000:]
    lines = _lines(r.stdout)
    assert len(lines) == 1
    _check(lines[0], 1)


def test_reference_arm_under_the_two_rank_launcher():
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", "2", "--master-addr", "127.0.0.1",
           "--master-port", "29671", os.path.join(ROOT, "bench.py"), "--gpus", "2", *SMALL]
    r = subprocess.run(cmd, capture_output=True, text=True, timeout=600, cwd=ROOT)
    assert r.returncode == 0, r.stderr[-2000:]
    lines = _lines(r.stdout)
    assert len(lines) == 1, r.stdout          # rank 1 prints nothing
    _check(lines[0], 2)
