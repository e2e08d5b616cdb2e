"""Time the reference's own numpy golden (imported unchanged through the `mindspore` stub) on benchmark
configuration 1, next to this repository's restatements of it.

    python tests/golden/time_reference_golden.py /path/to/reference

Needs a checkout of the reference, which does not travel to the GPU machines: the benchmark there times the
restatements only (bench.py: `cpu_baseline`, `cpu_baseline_numpy`); this script ties them to the original.
"""
import math
import os
import sys
import time

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
sys.path.insert(0, ROOT)

from ms_custom_ops_b200 import workloads  # noqa: E402
from oracle import c_oracle, ms_stub  # noqa: E402
from oracle import paged_kv_numpy as restated  # noqa: E402


def best_of(fn, n=3):
    best = float("inf")
    for _ in range(n):
        t0 = time.perf_counter()
        out = fn()
        best = min(best, time.perf_counter() - t0)
    return best, out


def main(ref_root):
    ms_stub.install()
    sys.path.insert(0, os.path.join(ref_root, "tests", "st"))
    import test_custom_paged_attention as tpa
    import test_custom_reshape_and_cache as trc
    spec = workloads.config_spec(1)
    c = workloads.decode_case(spec)
    gen = tpa.PagedAttentionDataGenerator(0)

    def reference():
        gk, gv = trc.InferenceEngine.nd_inference(c["key"], c["value"], c["key_cache"], c["value_cache"], c["slot_mapping"])
        return gen.compute_golden_reference(c["query"], gk, gv, c["block_tables"], np.ones(spec.batch, np.int32),
                                            c["context_lens"], 1.0 / math.sqrt(spec.head_size), None, 0)

    def numpy_port():
        gk, gv = restated.reshape_and_cache_golden(c["key"], c["value"], c["key_cache"], c["value_cache"], c["slot_mapping"])
        return restated.paged_attention_golden(c["query"], gk, gv, c["block_tables"], c["context_lens"], c["qk_scale"])

    def c_port():
        gk, gv = c_oracle.reshape_and_cache(c["key"], c["value"], c["key_cache"], c["value_cache"], c["slot_mapping"])
        return c_oracle.paged_attention(c["query"], gk, gv, c["block_tables"], c["context_lens"], c["qk_scale"])

    tokens = int(c["context_lens"].sum())
    ref_out = None
    for name, fn in (("reference numpy golden (stub import)", reference), ("numpy restatement", numpy_port),
                     ("C / OpenMP restatement", c_port)):
        t, out = best_of(fn)
        out = np.asarray(out, dtype=np.float32)
        if ref_out is None:
            ref_out = out
        print(f"{name}: {t * 1e3:.2f} ms per step, {spec.batch / t:.1f} decode tokens/s "
              f"({tokens} context tokens, {os.cpu_count()} host cores); max |diff| to the reference golden "
              f"{np.abs(out - ref_out).max():.2e}")


if __name__ == "__main__":
    if len(sys.argv) != 2:
        sys.exit("usage: python tests/golden/time_reference_golden.py /path/to/reference")
    main(sys.argv[1])
