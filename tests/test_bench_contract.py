"""The measurement script's contract that can be checked without a GPU: the CPU arm prints one JSON line with the
agreed keys, and the algorithmic byte count is the documented formula."""

import json
import subprocess
import sys
from pathlib import Path

ROOT = Path(__file__).resolve().parent.parent


def test_reference_arm_prints_the_agreed_line():
    out = subprocess.run([sys.executable, str(ROOT / "bench.py"), "--impl", "reference", "--steps", "2", "--warmup", "1",
                          "--cpu-seconds", "1"], capture_output=True, text=True, timeout=600, check=True).stdout
    lines = [ln for ln in out.splitlines() if ln.startswith("{")]
    assert len(lines) == 1
    line = json.loads(lines[0])
    assert line["impl"] == "reference" and line["n_gpus"] == 1 and line["steps"] == 2 and line["warmup"] == 1
    assert line["higher_is_better"] is True and line["value"] > 0 and line["ms_per_step"] > 0
    assert line["metric"].startswith("Llama-3.1-8B decode tok/s") and line["unit"].startswith("tok/s")
    assert line["e2e"] == {"value": line["value"], "unit": line["unit"], "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}
    base = line["cpu_baseline"]
    assert base["kind"] == "port" and base["cores"] >= 1 and base["value"] == line["value"] and base["sample"]
    cfg = line["config"]
    assert cfg["workload"] == "llama31-8b-layer attn decode ctx8192 b32 s0.75 fp16 unstructured"
    assert (cfg["batch_per_gpu"], cfg["context"], cfg["q_heads"], cfg["kv_heads"], cfg["head_dim"]) == (32, 8192, 32, 8, 128)


def test_algorithmic_bytes_is_the_documented_formula():
    sys.path.insert(0, str(ROOT))
    import bench

    # per KV head: compressed tokens (K and V payload + 16-byte bitmap + 1-byte id), both centroid tables, the dense
    # window (K and V); plus query and output of every query head
    batch, t_comp, t_dense, nnz, ck, cv = 32, 8128, 64, 32, 32, 32
    want = batch * 8 * (t_comp * 2 * (2 * nnz + 16 + 1) + (ck + cv) * 256 + t_dense * 512) + batch * 32 * 128 * 2 * 2
    assert bench.algorithmic_bytes(batch, t_comp, t_dense, nnz, ck, cv) == want
