"""What bench.py promises without a GPU: more than one GPU is refused with one line and exit code 2, the reference
arm says why it is unavailable, the roofline's bytes and flops are the model's, and the peaks come from the
measured file when there is one."""
import importlib.util
import json
import os
import subprocess
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def load_bench():
    spec = importlib.util.spec_from_file_location("bench_under_test", os.path.join(ROOT, "bench.py"))
    module = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(module)
    return module


def run(*arguments):
    return subprocess.run([sys.executable, os.path.join(ROOT, "bench.py"), *arguments], capture_output=True, text=True, timeout=300)


def test_more_than_one_gpu_is_refused_with_one_line():
    result = run("--gpus", "2", "--steps", "3", "--warmup", "3")
    assert result.returncode == 2
    assert len(result.stdout.strip().splitlines()) == 1 and "one GPU" in result.stdout


def test_reference_arm_says_why_it_is_unavailable():
    result = run("--impl", "reference", "--gpus", "1", "--steps", "3", "--warmup", "3")
    assert result.returncode == 0
    line = json.loads(result.stdout.strip().splitlines()[-1])
    assert line["impl"] == "reference" and isinstance(line["unavailable"], str) and "\n" not in line["unavailable"]


def test_roofline_numbers_are_the_models():
    bench = load_bench()
    cfg = bench.QWEN3_8B
    numbers = bench.model_numbers(cfg, cfg["num_hidden_layers"])
    h, i, v = cfg["hidden_size"], cfg["intermediate_size"], cfg["vocab_size"]
    q = cfg["num_attention_heads"] * cfg["head_dim"]
    kv = cfg["num_key_value_heads"] * cfg["head_dim"]
    per_layer = q * h + 2 * kv * h + h * q + 3 * i * h  # q, k, v, o, gate, up, down
    assert numbers["layer_weight_elems"] == per_layer
    assert numbers["weight_bytes"] == 2 * (36 * per_layer + v * h)  # the output head once, the embedding rows are negligible
    assert numbers["kv_bytes_per_token"] == 36 * 2 * kv * 2
    assert numbers["linear_flops_per_token"] == 2 * 36 * per_layer
    assert numbers["attention_flops"](2048) == 36 * 2 * q * 2048 * 2048


def test_peaks_come_from_the_measured_file_when_it_exists(tmp_path, monkeypatch):
    bench = load_bench()
    monkeypatch.setattr(bench, "ROOT", str(tmp_path))
    peaks, source = bench.load_peaks()
    assert source == "fallback" and peaks == bench.FALLBACK_PEAKS
    (tmp_path / "MEASURED_PEAKS.json").write_text(json.dumps({"hbm_gbs": 7000.0, "bf16_tflops": 1500, "clocks": {"sm": 1900}}))
    peaks, source = bench.load_peaks()
    assert source == "measured" and peaks["hbm_gbs"] == 7000.0 and peaks["bf16_tflops"] == 1500.0
    assert peaks["bf16_tflops_sustained"] == bench.FALLBACK_PEAKS["bf16_tflops_sustained"]  # a key the file lacks keeps its fallback
    (tmp_path / "MEASURED_PEAKS.json").write_text("{broken")
    assert bench.load_peaks()[1] == "fallback"
