"""bench.py's CPU arm (`--impl reference`) needs no GPU: its sample and its JSON line are checked here on a small
batch and context (the full-size sample holds 17 GB of K/V on the host and takes minutes)."""
import argparse
import importlib.util
import json
import os

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _bench():
    spec = importlib.util.spec_from_file_location("bench_under_test", os.path.join(ROOT, "bench.py"))
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


def test_cpu_sample_extrapolates_one_layer_and_a_head_slice():
    b = _bench()
    s = b.cpu_decode_sample(2, 1, batch=2, ctx=32)
    assert s["unit"] == "tokens/s" and s["kind"] == "port" and s["cores"] >= 1 and "timed 2x" in s["sample"]
    step_ms = 28 * s["layer_ms"] + (256000 / 32000.0) * s["head_slice_ms"]
    assert abs(step_ms - s["ms_per_step"]) <= 1e-6 * step_ms
    assert abs(s["value"] - 2 / (s["ms_per_step"] / 1e3)) <= 1e-6 * s["value"]


def test_reference_arm_line_honours_the_requested_counts(capsys, monkeypatch):
    b = _bench()
    real = b.cpu_decode_sample
    seen = {}

    def small(steps, warmup, **kw):
        seen["counts"] = (steps, warmup)
        return real(steps, warmup, batch=2, ctx=32)
    monkeypatch.setattr(b, "cpu_decode_sample", small)
    monkeypatch.setenv("RANK", "0")
    b.run_reference(argparse.Namespace(gpus=1, steps=3, warmup=2))
    line = json.loads(capsys.readouterr().out.strip().splitlines()[-1])
    assert seen["counts"] == (3, 2) and line["steps"] == 3 and line["warmup"] == 2
    assert line["impl"] == "reference" and line["metric"] == "decode_tokens_per_s" and line["unit"] == "tokens/s"
    assert line["higher_is_better"] is True and line["n_gpus"] == 1 and line["vs_baseline"] is None
    assert line["e2e"] == {"value": line["value"], "unit": "tokens/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}
    assert set(line["cpu_baseline"]) == {"value", "unit", "cores", "kind", "sample"} and line["cpu_baseline"]["value"] == line["value"]
    assert "workload" in line["config"] and "model" not in line["config"]
    # the other ranks of a torchrun launch print nothing
    monkeypatch.setenv("RANK", "3")
    b.run_reference(argparse.Namespace(gpus=8, steps=3, warmup=2))
    assert capsys.readouterr().out == ""
