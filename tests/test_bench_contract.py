"""CPU: the reference arm of bench.py (the reference's CPU path, timed) prints the contracted line."""
import json
import os
import subprocess
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _run(extra_env=None, *flags):
    env = dict(os.environ)
    env.pop("RANK", None)
    env.pop("WORLD_SIZE", None)
    env.update(extra_env or {})
    return subprocess.run([sys.executable, os.path.join(ROOT, "bench.py"), "--impl", "reference", "--workload", "c1",
                           "--steps", "2", "--warmup", "1", *flags], cwd=ROOT, env=env, capture_output=True,
                          text=True, timeout=600)


def test_reference_arm_prints_one_contract_line():
    r = _run()
    assert r.returncode == 0, r.stderr[-2000:]
    lines = [ln for ln in r.stdout.splitlines() if ln.startswith("{")]
    assert len(lines) == 1
    d = json.loads(lines[0])
    assert d["impl"] == "reference" and d["metric"] == "paged-attn decode tokens/s" and d["unit"] == "tokens/s"
    assert d["higher_is_better"] is True and d["steps"] == 2 and d["warmup"] == 1 and d["n_gpus"] == 1
    assert d["value"] > 0 and abs(d["value"] - 4 / (d["ms_per_step"] / 1e3)) < 1e-6 * d["value"]
    assert d["config"]["workload"].startswith("C1")
    cb = d["cpu_baseline"]
    assert cb["kind"] == "port" and cb["cores"] >= 1 and cb["value"] == d["value"] and "sequences" in cb["sample"]
    assert d["e2e"] == {"value": d["value"], "unit": "tokens/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}


def test_reference_arm_runs_on_rank_zero_only():
    r = _run({"RANK": "1", "WORLD_SIZE": "2"}, "--gpus", "2")
    assert r.returncode == 0 and r.stdout.strip() == ""


def test_cpu_legs_of_the_adjacent_operators():
    # the CPU side of `bench.py --adjacent` (C restatements timed on the host cores, outputs checked),
    # fed with host tensors that already hold the right answers
    import importlib.util

    import numpy as np
    import torch

    from oracle import paged_kv_numpy as oracle
    spec = importlib.util.spec_from_file_location("bench_module", os.path.join(ROOT, "bench.py"))
    bench = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(bench)
    rng = np.random.default_rng(0)
    kc = torch.from_numpy(rng.standard_normal((20, 16, 2, 8)).astype(np.float32)).to(torch.bfloat16)
    vc = torch.from_numpy(rng.integers(-100, 100, (20, 16, 2, 8)).astype(np.int8))
    bt = torch.from_numpy(rng.integers(0, 20, (3, 5)).astype(np.int32))
    lens = np.array([70, 1, 33], np.int32)
    gk, gv = oracle.paged_cache_load_golden(kc.view(torch.int16).numpy(), vc.numpy(), bt.numpy(), lens)
    leg = bench.cpu_leg_cache_load(kc, vc, bt, lens, torch.from_numpy(gk).view(torch.bfloat16), torch.from_numpy(gv))
    assert leg["bit_exact"] is True and leg["cpu_baseline"]["value"] > 0 and leg["cpu_baseline"]["cores"] >= 1
    wrong = torch.from_numpy(gv.copy())
    wrong[5] += 1
    assert bench.cpu_leg_cache_load(kc, vc, bt, lens, torch.from_numpy(gk).view(torch.bfloat16), wrong)["bit_exact"] is False
    lse = torch.from_numpy(rng.standard_normal((3, 50)).astype(np.float32))
    lo = torch.from_numpy(rng.standard_normal((3, 50, 16)).astype(np.float32))
    merged = torch.from_numpy(oracle.fa_update_golden(lse.numpy(), lo.numpy()))
    leg = bench.cpu_leg_fa_update(lse, lo, merged)
    assert leg["max_abs_err"] < 1e-5 and leg["cpu_baseline"]["unit"] == "rows/s"
