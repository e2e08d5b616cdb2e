"""GPU: the standalone C++ benchmark harness (no Python, no PyTorch at run time) runs the decode loop
through the thin C ABI; its dumped step is recomputed by the oracle and its JSON line is checked."""
import json
import os
import struct
import subprocess

import numpy as np
import pytest

from oracle import paged_kv_numpy as oracle
from tests.helpers import BF16, assert_close

pytestmark = pytest.mark.gpu

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
EXE = os.path.join(ROOT, "ms_custom_ops_b200", "bench", "msco_bench")


def _read_dump(path):
    out = {}
    with open(path, "rb") as f:
        while True:
            tag = f.read(32)
            if len(tag) < 32:
                break
            (n,) = struct.unpack("<Q", f.read(8))
            out[tag.rstrip(b"\0").decode()] = f.read(n)
    return out


@pytest.mark.parametrize("flags,kv", [([], "bf16"), (["--int8"], "int8"), (["--fp16", "--head-dim", "64", "--block-size", "32"], "fp16")])
def test_cxx_harness_step_matches_the_oracle(tmp_path, flags, kv):
    assert os.path.exists(EXE), "build the harness with `python -m ms_custom_ops_b200.build`"
    dump = str(tmp_path / "step.bin")
    cmd = [EXE, "--batch", "6", "--q-heads", "16", "--kv-heads", "4", "--len-lo", "90", "--len-hi", "2500", "--steps", "4",
           "--warmup", "3", "--repeats", "2", "--seed", "11", "--dump", dump] + flags
    r = subprocess.run(cmd, capture_output=True, text=True, timeout=300)
    assert r.returncode == 0, r.stderr[-2000:]
    line = json.loads([ln for ln in r.stdout.splitlines() if ln.startswith("{")][-1])
    assert line["harness"] == "msco_bench" and line["kv"] == kv and line["value"] > 0 and line["e2e_value"] > 0
    assert line["e2e_ms_per_step"] >= 0.5 * line["ms_per_step"] and line["pinned_slabs_added_in_e2e_loop"] == 0
    assert line["kernel"] == 2 and line["h2d_bytes_per_step"] > 0 and line["d2h_bytes_per_step"] > 0
    d = _read_dump(dump)
    batch, hq, hkv, hd, bs, nb, width, int8, fp16, step = struct.unpack("<12i", d["header"])[:10]
    qdt = np.float16 if fp16 else BF16
    cdt = np.int8 if int8 else qdt
    lens = np.frombuffer(d["context_lens"], np.int32)
    tables = np.frombuffer(d["block_tables"], np.int32).reshape(batch, width)
    slots = np.frombuffer(d["slot_mapping"], np.int32)
    q = np.frombuffer(d["query"], qdt).reshape(batch, hq, hd)
    key = np.frombuffer(d["key"], qdt).reshape(batch, hkv * hd)
    val = np.frombuffer(d["value"], qdt).reshape(batch, hkv * hd)
    kc = np.frombuffer(d["key_cache"], cdt).reshape(nb, bs, hkv, hd)
    vc = np.frombuffer(d["value_cache"], cdt).reshape(nb, bs, hkv, hd)
    out = np.frombuffer(d["out"], qdt).reshape(batch, hq, hd)
    kd = np.frombuffer(d["k_descale"], np.float32) if int8 else None
    vd = np.frombuffer(d["v_descale"], np.float32) if int8 else None
    # the dumped caches already hold the step's rows; scattering them again must change nothing (bit-exact)
    if int8:
        gk, gv = oracle.reshape_and_cache_quant_golden(key, val, kc, vc, slots, kd, vd)
    else:
        gk, gv = oracle.reshape_and_cache_golden(key, val, kc, vc, slots)
    assert np.array_equal(gk.view(np.uint8), kc.view(np.uint8)) and np.array_equal(gv.view(np.uint8), vc.view(np.uint8))
    assert (slots == tables[np.arange(batch), (lens - 1) // bs] * bs + (lens - 1) % bs).all()
    g = oracle.paged_attention_golden(q, gk, gv, tables, lens, 1.0 / np.sqrt(hd), kd, vd)
    tol = 2e-2 if int8 else (5e-3 if fp16 else 1e-2)
    assert_close(out, g, tol, "msco_bench step")
