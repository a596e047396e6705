"""GPU: measured plans survive the handle.  o64_plan_tune's results are written to a JSON file and
merged into another handle, which then uses them (the checkpoint of this engine: what was decided,
for which shape, at what measured time, on which device)."""
import json
import os
import subprocess
import sys

import pytest
import torch

import open64_b200 as o

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_save_and_load(eng, tmp_path):
    path = tmp_path / "plans.json"
    best = eng.plan_tune(o.KIND_BF16, 256, 1024, 512)
    eng.plan_tune(o.KIND_S8, 200, 512, 256)
    eng.plan_save(path)
    doc = json.loads(path.read_text())
    assert doc["version"] == 1 and doc["num_sms"] >= 100 and "B200" in doc["device"]
    entries = {(p["kind"], p["M"], p["N"], p["K"]): p for p in doc["plans"]}
    assert (o.KIND_BF16, 256, 1024, 512) in entries and (o.KIND_S8, 200, 512, 256) in entries
    assert entries[(o.KIND_BF16, 256, 1024, 512)]["ms"] == pytest.approx(best["predicted_ms"], rel=1e-3)
    eng.plan_tune_clear()

    other = o.Engine(eng.device)
    try:
        assert other.plan_load(path) == 2
        got = other.plan_get(o.KIND_BF16, 256, 1024, 512)
        for k in ("tile_m", "tile_n", "cta_group"):
            assert got[k] == best[k], k
        # and the loaded plan is what a product of that shape runs with
        A, B = o.workloads.c2_gemm_bf16(256, 1024, 512)
        dev = torch.device("cuda", eng.device)
        c = other.gemm_bf16(A.to(dev), B.to(dev), transB=True)
        ref = (A.float() @ B.float().t())
        assert (c.float().cpu() - ref).abs().max() / ref.abs().max() < 4e-3
    finally:
        other.close()


def test_files_that_do_not_apply(eng, tmp_path):
    with pytest.raises(o.O64Error) as e:
        eng.plan_load(tmp_path / "missing.json")
    assert e.value.status == o.ERR_RANK
    elsewhere = tmp_path / "elsewhere.json"
    elsewhere.write_text('{"version": 1, "device": "Some Other GPU", "num_sms": 148, "plans": ['
                         '{"kind": 1, "swiglu": 0, "M": 64, "N": 64, "K": 64, "gpus": 1, "cta_group": 1, "tile_m": 128, '
                         '"tile_n": 256, "split_k": 1, "ms": 0.01}]}')
    with pytest.raises(o.O64Error) as e:
        eng.plan_load(elsewhere)
    assert e.value.status == o.ERR_CONFORM
    # an entry that names no existing kernel is skipped, the good one beside it is kept
    name = torch.cuda.get_device_name(eng.device)
    sms = torch.cuda.get_device_properties(eng.device).multi_processor_count
    mixed = tmp_path / "mixed.json"
    mixed.write_text(json.dumps({"version": 1, "device": name, "num_sms": sms, "plans": [
        {"kind": 1, "swiglu": 0, "M": 64, "N": 64, "K": 64, "gpus": 1, "cta_group": 2, "tile_m": 999, "tile_n": 256, "split_k": 0, "ms": 1.0},
        {"kind": 3, "swiglu": 0, "M": 640, "N": 640, "K": 640, "gpus": 1, "cta_group": 1, "tile_m": 128, "tile_n": 128, "split_k": 1, "ms": 0.02}]}))
    eng.plan_tune_clear()
    assert eng.plan_load(mixed) == 1
    assert eng.plan_get(o.KIND_S8, 640, 640, 640)["tile_n"] == 128
    eng.plan_tune_clear()


def test_cache_file_named_in_the_environment(built, tmp_path):
    path = tmp_path / "cache.json"
    prog = ("import open64_b200 as o\n"
            "e = o.Engine(0)\n"
            "n0 = e.lib.o64_plan_count(e._h)\n"
            "p = e.plan_tune(o.KIND_BF16, 128, 512, 256) if n0 == 0 else e.plan_get(o.KIND_BF16, 128, 512, 256)\n"
            "print(n0, p['tile_m'], p['tile_n'], p['split_k'])\n")
    env = dict(os.environ, O64_PLAN_CACHE=str(path), PYTHONPATH=ROOT)
    first = subprocess.run([sys.executable, "-c", prog], capture_output=True, text=True, env=env, cwd=ROOT)
    assert first.returncode == 0, first.stderr
    assert path.exists()
    second = subprocess.run([sys.executable, "-c", prog], capture_output=True, text=True, env=env, cwd=ROOT)
    assert second.returncode == 0, second.stderr
    a, b = first.stdout.split(), second.stdout.split()
    assert a[0] == "0" and b[0] == "1" and a[1:] == b[1:]      # the second process found the plan on disk
