"""Host-side pieces of bench.py that need no GPU: the workload is the one the baseline names, the
roofline's traffic figure comes from the committed capture summary, the argument surface the
driver uses exists."""

import json
import subprocess
import sys
from pathlib import Path

ROOT = Path(__file__).resolve().parent.parent


def _bench():
    sys.path.insert(0, str(ROOT))
    import bench

    return bench


def test_workload_is_the_qwen3_8b_shape_of_the_baseline():
    bench = _bench()
    q = bench.QWEN3_8B
    assert (q["num_hidden_layers"], q["hidden_size"], q["num_attention_heads"], q["num_key_value_heads"], q["head_dim"],
            q["intermediate_size"], q["vocab_size"], q["tie_word_embeddings"]) == (36, 4096, 32, 8, 128, 12288, 151936,
                                                                                    False)
    assert bench.SEQ_LEN == 8192 and bench.METRIC.startswith("Qwen3-8B train tokens/s")
    base = json.loads((ROOT / "BASELINE.json").read_text())
    assert base["metric"].startswith(bench.METRIC)


def test_roofline_traffic_comes_from_the_committed_capture():
    bench = _bench()
    traffic, src = bench._traffic_from_profile()
    assert src["from_profile"] is True and (ROOT / src["file"]).exists()
    d = json.loads((ROOT / src["file"]).read_text())
    per_launch = [r + w for r, w in zip(d["dram_read_bytes_per_launch"], d["dram_write_bytes_per_launch"])]
    assert len(per_launch) == 6 and abs(sum(per_launch) / 6 - traffic) < 1e6
    assert (ROOT / d["summary"]).exists()


def test_peaks_fall_back_when_the_measured_file_is_absent(tmp_path, monkeypatch):
    bench = _bench()
    monkeypatch.setattr(bench, "ROOT", tmp_path)
    peaks, kind = bench.load_peaks()
    assert kind == "fallback" and peaks == bench.FALLBACK_PEAKS
    (tmp_path / "MEASURED_PEAKS.json").write_text(json.dumps({"hbm_gbs": 1.0, "bf16_tflops": 2.0, "bf16_tflops_sustained": 3.0}))
    peaks, kind = bench.load_peaks()
    assert kind == "measured" and peaks["bf16_tflops_sustained"] == 3.0


def test_driver_flags_parse():
    out = subprocess.run([sys.executable, str(ROOT / "bench.py"), "--help"], capture_output=True, text=True, timeout=120)
    assert out.returncode == 0
    for flag in ("--gpus", "--steps", "--warmup", "--impl", "--parallel"):
        assert flag in out.stdout
