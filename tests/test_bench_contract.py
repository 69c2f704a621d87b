"""The benchmark entry points keep their command-line contract (checked without a GPU)."""
import importlib
import os
import subprocess
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_bench_defaults_and_flags(monkeypatch):
    monkeypatch.setattr(sys, "argv", ["bench.py"])
    bench = importlib.import_module("bench")
    args = bench.parse()
    assert args.gpus == 1 and args.warmup >= 3 and args.steps >= 1 and args.impl == "apexw_b200"
    assert (bench.MODEL, bench.SEQ, bench.GLOBAL_BATCH, bench.MICRO_BATCH) == ("llama3-8b", 4096, 64, 1)
    monkeypatch.setattr(sys, "argv", ["bench.py", "--impl", "reference", "--gpus", "8", "--steps", "5", "--warmup", "3"])
    args = bench.parse()
    assert args.impl == "reference" and args.gpus == 8 and args.steps == 5


def test_reference_arm_reports_unavailable_when_the_install_is_missing(tmp_path, monkeypatch):
    bench = importlib.import_module("bench")
    monkeypatch.setattr(bench, "ROOT", str(tmp_path))
    monkeypatch.setattr(sys, "argv", ["bench.py", "--impl", "reference"])
    res = bench.run_reference(bench.parse(), 0, 0, 1)
    assert "unavailable" in res and "baseline/_ref" in res["unavailable"]


def test_entry_points_parse():
    for script in ("bench.py", "bench_fsdp.py"):
        out = subprocess.run([sys.executable, os.path.join(ROOT, script), "--help"], capture_output=True, text=True, timeout=120)
        assert out.returncode == 0 and "--impl" in out.stdout
    out = subprocess.run([sys.executable, "-m", "apexw_b200.microbench", "zero", "--help"], capture_output=True, text=True,
                         timeout=120, cwd=ROOT)
    assert out.returncode == 0 and "--precision" in out.stdout


def test_microbench_optimizer_variants_are_valid_optimizer_arguments():
    """Every ``--variant`` of ``python -m apexw_b200.microbench optimizer`` constructs and steps (here on CPU)."""
    import torch
    import torch.nn as nn
    from apexw_b200 import ApexW, microbench
    for name, kw in microbench.VARIANTS.items():
        if name == "capturable":
            continue                                  # device-resident counters need an accelerator
        for prec in ("compact", "8bit", "ultra"):
            ps = [nn.Parameter(torch.randn(64, 32)), nn.Parameter(torch.randn(48))]
            opt = ApexW(ps, lr=1e-3, precision=prec, **kw)
            for p in ps:
                p.grad = torch.randn_like(p)
            opt.step()
            assert all(torch.isfinite(p).all() for p in ps), (name, prec)
    assert {"default", "lion", "factored", "cautious", "amsgrad", "ademamix"} <= set(microbench.VARIANTS)
