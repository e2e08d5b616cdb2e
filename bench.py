"""Benchmark of the paged-KV decode hot path: reshape_and_cache -> paged_attention.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--workload c2] [--impl reference]

One step = one decode step over one batch of synthetic sequences: the newest
token's K/V rows are scattered into the paged cache (reshape_and_cache), then
paged attention runs over every sequence's context.  Steps follow one another
as in a serving loop: every step every sequence is one token longer.  The
metric is decode tokens per second (= sequences per step / step time), whole job.

Printed JSON line (rank 0):
  value      device-timed throughput with every input resident in HBM
  e2e        the same step through the operator API with the step's inputs in pinned host memory:
             host->device copies of query / new rows / slots / block tables and the device->host
             read of the attention output are inside the timed region; `value` is the serial loop
             (the host waits for every step's result), the pipelined figure is printed beside it
  configs    the other benchmark configurations (c3 int8 KV, c4 long skewed, c5 mixed decode, the
             prefill-heavy scatter of c5, and configuration 2 at head_dim 64 / 256): throughput,
             attention-kernel time, roofline, parity
  roofline   the attention kernel alone: algorithmic bytes / its CUDA-event duration, against the
             measured HBM copy bandwidth (MEASURED_PEAKS.json, else the stated fallback)
  cpu_baseline  the CPU restatement of the reference golden (oracle/, all host cores), timed on
             the same workload; its output doubles as a full-size parity check of the GPU result

With N > 1 (torchrun) the KV cache is partitioned by kv head: each rank owns
num_kv_heads / N heads of every block and the matching q heads, and the
per-head outputs are all-gathered over NCCL.  Total work is fixed: "strong".

`--impl reference` times the CPU implementation of the same path (the oracle
port of the reference's numpy golden, all host threads) on a bounded sample
of the workload and prints the same line with "impl": "reference".
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import sys
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

from ms_custom_ops_b200 import workloads  # noqa: E402

METRIC = "paged-attn decode tokens/s"
UNIT = "tokens/s"
FALLBACK_HBM_GBS = 6650.0
# (dram__bytes_read.sum + dram__bytes_write.sum) / (context tokens * kv heads) from the ncu captures
# in profiles/: config 2 (16-bit KV, 512 algorithmic bytes) and config 3 (int8 KV, 256 algorithmic)
NCU_DRAM_BYTES_PER_TOKEN_HEAD = {"16bit": 525.6, "int8": 266.0}
L2_BYTES = 126 << 20


def workload_spec(name):
    """c1..c5: the benchmark configurations; c2h64 / c2h256: configuration 2 with head_dim 64 / 256 (block_size
    64 for 256: the operator requires block_size * head_dim <= 128 * 128)."""
    name = name.lower()
    if "h" in name:
        base, hd = name.split("h")
        spec = workloads.config_spec(int(base.lstrip("c")))
        spec.head_size = int(hd)
        spec.block_size = min(spec.block_size, 128 * 128 // spec.head_size)
        spec.name += f"-head{hd}"
        return spec
    return workloads.config_spec(int(name.lstrip("c")))


def workload_config(spec, lens, extra=None):
    cfg = {"workload": f"{spec.name}: batch {spec.batch}, {spec.num_heads} q heads / {spec.kv_heads} kv heads, "
                       f"head_dim {spec.head_size}, block_size {spec.block_size}, "
                       f"{'int8 KV + ' if spec.kv_int8 else ''}{spec.dtype}, context_lens {spec.len_dist} "
                       f"[{spec.len_lo},{spec.len_hi}], one new token per sequence via reshape_and_cache",
           "batch": spec.batch, "kv_tokens": int(np.asarray(lens, dtype=np.int64).sum()),
           "seed": spec.seed}
    if extra:
        cfg.update(extra)
    return cfg


# ----------------------------------------------------------------------------------------------
# clocks
# ----------------------------------------------------------------------------------------------
class ClockSampler:
    """SM clock and throttle reasons sampled every few milliseconds between start() and stop().

    Reads NVML (the source nvidia-smi prints: clocks.sm, clocks.max.sm and the
    clocks_event_reasons bits) from a background thread, because the timed regions last only
    milliseconds and nvidia-smi's own loop cannot sample that fast.  Read-only: no setting of the
    GPU is touched.
    """
    REASONS = {0x4: "sw_power_cap", 0x8: "hw_slowdown", 0x20: "sw_thermal_slowdown",
               0x40: "hw_thermal_slowdown", 0x80: "hw_power_brake_slowdown"}

    def __init__(self, gpu_uuid, interval_s=0.004):
        import threading
        self.samples, self.bits, self.max_mhz = [], 0, None
        self._stop = threading.Event()
        self._thread = None
        try:
            import pynvml
            pynvml.nvmlInit()
            try:
                h = pynvml.nvmlDeviceGetHandleByUUID(gpu_uuid)
            except Exception:
                h = pynvml.nvmlDeviceGetHandleByUUID(gpu_uuid.encode())
            self.max_mhz = float(pynvml.nvmlDeviceGetMaxClockInfo(h, pynvml.NVML_CLOCK_SM))
        except Exception:
            return

        def loop():
            while not self._stop.is_set():
                try:
                    self.samples.append(float(pynvml.nvmlDeviceGetClockInfo(h, pynvml.NVML_CLOCK_SM)))
                    self.bits |= int(pynvml.nvmlDeviceGetCurrentClocksEventReasons(h))
                except Exception:
                    pass
                self._stop.wait(interval_s)
        self._thread = threading.Thread(target=loop, daemon=True)

    def start(self):
        if self._thread is not None:
            self._thread.start()
        return self

    def stop(self):
        if self._thread is not None:
            self._stop.set()
            self._thread.join(timeout=2)
        reasons = sorted(name for bit, name in self.REASONS.items() if self.bits & bit)
        return {"sm_mhz": statistics.median(self.samples) if self.samples else None, "sm_max_mhz": self.max_mhz,
                "reasons": reasons, "samples": len(self.samples), "source": "nvml, 4 ms interval, under load"}


def measured_hbm_peak():
    try:
        with open(os.path.join(ROOT, "MEASURED_PEAKS.json")) as f:
            return float(json.load(f)["hbm_gbs"]), "measured"
    except Exception:
        return FALLBACK_HBM_GBS, "fallback"


# ----------------------------------------------------------------------------------------------
# reference arm: CPU implementation of the path on the host cores
# ----------------------------------------------------------------------------------------------
def host_threads():
    """Host cores this process may use (torchrun exports OMP_NUM_THREADS=1; the CPU legs ignore it)."""
    try:
        return len(os.sched_getaffinity(0))
    except AttributeError:
        return os.cpu_count() or 1


def cpu_step(c_oracle, case, threads=0):
    """One decode step on the CPU: scatter the new rows into the caches in place, then attention.
    Returns the output."""
    if case["k_descale"] is not None:
        gk, gv = c_oracle.reshape_and_cache_quant(case["key"], case["value"], case["key_cache"], case["value_cache"],
                                                  case["slot_mapping"], case["k_descale"], case["v_descale"],
                                                  threads=threads, inplace=True)
    else:
        gk, gv = c_oracle.reshape_and_cache(case["key"], case["value"], case["key_cache"], case["value_cache"],
                                            case["slot_mapping"], threads=threads, inplace=True)
    return c_oracle.paged_attention(case["query"], gk, gv, case["block_tables"], case["context_lens"],
                                    case["qk_scale"], case["k_descale"], case["v_descale"], threads=threads)


def run_reference(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return  # one CPU run per job; the other ranks have nothing to do
    from oracle import c_oracle
    spec = workload_spec(args.workload)
    full_batch = spec.batch
    # bounded sample: the first `sample` sequences' worth of the same length distribution
    sample = min(full_batch, args.cpu_sample)
    sspec = workloads.DecodeSpec(**{**spec.__dict__, "batch": sample})
    case = workloads.decode_case(sspec)
    cores = host_threads()
    for _ in range(args.warmup):
        cpu_step(c_oracle, case, cores)
    t0 = time.perf_counter()
    for _ in range(args.steps):
        cpu_step(c_oracle, case, cores)
    dt = (time.perf_counter() - t0) / max(args.steps, 1)
    value = sample / dt
    what = (f"{sample} of {full_batch} sequences per step ({int(case['context_lens'].sum())} context tokens), "
            f"C restatement of the reference numpy golden, OpenMP over (sequence, kv head)")
    line = {
        "impl": "reference", "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": dt * 1e3, "higher_is_better": True,
        "scaling": "strong", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": workload_config(spec, case["context_lens"], {"sample": what}),
        "cpu_baseline": {"value": value, "unit": UNIT, "cores": cores, "kind": "port", "sample": what},
        "e2e": {"value": value, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }
    print(json.dumps(line), flush=True)


# ----------------------------------------------------------------------------------------------
# GPU arm
# ----------------------------------------------------------------------------------------------
def cpu_numpy_config1():
    """The numpy restatement of the reference golden (per-sequence gather + BLAS, one core for the
    gather loop) on configuration 1 exactly: the second CPU figure beside the C / OpenMP one."""
    from oracle import paged_kv_numpy as onp
    spec = workloads.config_spec(1)
    c = workloads.decode_case(spec)
    best = float("inf")
    for _ in range(3):
        t0 = time.perf_counter()
        gk, gv = onp.reshape_and_cache_golden(c["key"], c["value"], c["key_cache"], c["value_cache"], c["slot_mapping"])
        onp.paged_attention_golden(c["query"], gk, gv, c["block_tables"], c["context_lens"], c["qk_scale"])
        best = min(best, time.perf_counter() - t0)
    return {"value": spec.batch / best, "unit": UNIT, "cores": 1, "kind": "port",
            "sample": f"configuration 1 exactly ({spec.batch} sequences, {int(c['context_lens'].sum())} context tokens), "
                      "best of 3; numpy restatement of the reference numpy golden"}


class DecodeLoop:
    """One workload on this rank's GPU, stepped the way a serving loop steps it: every step appends one
    token to every sequence (context_lens grow by one, slot_mapping moves to the new position, a fresh
    cache block is used when a sequence crosses a block boundary), so every step needs a new launch
    plan -- the plan object is re-planned in place (msco_paged_attention_replan) -- and the step is one
    msco_decode_step call: cache scatter + attention, two kernel launches."""

    def __init__(self, ctx, spec, total_steps):
        import torch
        from ms_custom_ops_b200 import _abi, kernels, sharding
        self.torch, self.kernels, self.ctx, self.spec = torch, kernels, ctx, spec
        world, rank, dev = ctx["world"], ctx["rank"], ctx["dev"]
        if spec.kv_heads % world != 0:
            raise SystemExit(f"{spec.kv_heads} kv heads cannot be split over {world} GPUs")
        self.hpr = spec.kv_heads // world
        self.h0, self.h1 = sharding.kv_head_range(rank, world, spec.kv_heads)
        self.hq_local = self.hpr * (spec.num_heads // spec.kv_heads)
        self.total_steps = total_steps
        case = self.case = workloads.decode_case_device(spec, dev, (self.h0, self.h1), growth_steps=total_steps + 2)
        self.lens0 = np.asarray(case["context_lens"], dtype=np.int32)
        self.tables_host = case["block_tables_host"]
        # slot_mapping of every step, resident on the device and in host memory
        bs = spec.block_size
        last = self.lens0.astype(np.int64)[None, :] + np.arange(total_steps + 2, dtype=np.int64)[:, None] - 1
        rows = np.arange(spec.batch)[None, :]
        slots = np.where(last >= 0, self.tables_host[rows, np.maximum(last, 0) // bs].astype(np.int64) * bs
                         + np.maximum(last, 0) % bs, -1).astype(np.int32)
        # sequences that start empty stay out of the scatter until they have a token
        self.slots_host = torch.from_numpy(slots)
        self.slots_dev = self.slots_host.to(dev)
        self.cur_lens = self.lens0.copy()          # lengths of the step being issued (updated in place)
        self.h_lens = torch.from_numpy(self.cur_lens)  # the same memory as a CPU tensor (operator API)
        self.i = 0                                 # index of the next step
        self.quant = 1 if spec.kv_int8 else 0
        q, kc, bt = case["query"], case["key_cache"], case["block_tables"]
        self.desc = kernels.make_pa_desc(q, kc, bt, case["qk_scale"], self.quant)
        self.plan = _abi.PaPlan(self.desc, [int(x) for x in self.lens0 + total_steps + 1])
        ws_bytes = self.plan.workspace_bytes       # partial count grows with the lengths: the last step's is the largest
        self.plan.replan(self.lens0)
        self.info0 = self.plan.info()
        self.ws = torch.empty(max(ws_bytes, self.plan.workspace_bytes, 256), dtype=torch.uint8, device=dev)
        self.out_local = torch.empty_like(q)

    def lens_at(self, i):
        return self.lens0 + np.int32(i)

    def step(self, gather=None):
        """One device-resident decode step (everything it reads is in HBM already).  `gather` (a
        sharding.PeerGather): the step's finishing kernel also pushes the output rows to the peers and
        waits for theirs (msco_decode_step_gather); returns this rank's gathered buffer then."""
        c, i = self.case, self.i
        np.add(self.lens0, np.int32(i), out=self.cur_lens)
        self.plan.replan(self.cur_lens)
        got = self.kernels.decode_step(self.plan, c["key"], c["value"], c["key_cache"], c["value_cache"],
                                       self.slots_dev[i], c["query"], c["block_tables"], self.out_local, self.ws,
                                       c["k_descale"], None, c["v_descale"], None, gather=gather)
        self.i = i + 1
        return got

    def algorithmic_bytes(self, first_step, nsteps):
        """Mean algorithmic bytes per launch over steps [first_step, first_step + nsteps)."""
        spec = self.spec
        kvb = 1 if spec.kv_int8 else 2
        lens_mid = self.lens0.astype(np.float64) + first_step + (nsteps - 1) / 2.0
        fixed = workloads.algorithmic_bytes_attention(np.zeros(spec.batch), self.hq_local, self.hpr, spec.head_size,
                                                      kvb, quant=spec.kv_int8)
        return float(lens_mid.sum()) * 2 * self.hpr * spec.head_size * kvb + fixed

    def cpu_check(self, args, out_gpu, step_index):
        """CPU baseline (C / OpenMP restatement of the reference golden, all host cores) on the state of
        step `step_index`, and the comparison of the GPU output of that step with it."""
        from oracle import c_oracle
        c, spec = self.case, self.spec
        nseq = min(spec.batch, args.cpu_sample)
        lens = self.lens_at(step_index)[:nseq]
        kd, vd = c["k_descale"], c["v_descale"]
        # the step's rows are in the cache already; the scatter is idempotent, so the CPU step that
        # scatters them again reproduces the state the GPU step read
        host = {"query": _to_np(c["query"][:nseq]), "key": _to_np(c["key"][:nseq]), "value": _to_np(c["value"][:nseq]),
                "key_cache": _to_np(c["key_cache"]), "value_cache": _to_np(c["value_cache"]),
                "block_tables": self.tables_host[:nseq], "slot_mapping": self.slots_host[step_index][:nseq].numpy(),
                "context_lens": lens, "qk_scale": c["qk_scale"],
                "k_descale": None if kd is None else kd.cpu().numpy(),
                "v_descale": None if vd is None else vd.cpu().numpy()}
        cores = host_threads()
        ref = cpu_step(c_oracle, host, cores)  # warm-up + reference output
        reps, t_best = 0, float("inf")
        t_begin = time.perf_counter()
        while reps < 3 and time.perf_counter() - t_begin < args.cpu_seconds:
            t0 = time.perf_counter()
            cpu_step(c_oracle, host, cores)
            t_best = min(t_best, time.perf_counter() - t0)
            reps += 1
        if reps == 0:
            t0 = time.perf_counter()
            cpu_step(c_oracle, host, cores)
            t_best, reps = time.perf_counter() - t0, 1
        sample = (f"{nseq} of {spec.batch} sequences ({int(lens.sum())} context tokens), kv heads {self.h0}..{self.h1 - 1}, "
                  f"best of {reps}; C restatement of the reference numpy golden, OpenMP")
        cpu = {"value": nseq / t_best, "unit": UNIT, "cores": cores, "kind": "port", "sample": sample}
        got = out_gpu[:nseq].float().cpu().numpy()
        err = np.abs(got - ref)
        tol = 2e-2 if spec.kv_int8 else (1e-2 if spec.dtype == "bfloat16" else 5e-3)
        checked = {"sequences": nseq, "max_abs_err": float(err.max()), "max_abs_golden": float(np.abs(ref).max()),
                   "rel_l2": float(np.linalg.norm(got - ref) / max(np.linalg.norm(ref), 1e-30)),
                   "within_tolerance": bool(np.all(err <= tol + tol * np.abs(ref))), "tolerance": tol}
        return cpu, checked

    def release(self):
        self.plan.close()
        self.case = self.ws = self.out_local = self.slots_dev = None
        self.torch.cuda.empty_cache()


def measure_decode(ctx, spec, args, full):
    """Times one workload.  Device-resident loop: `repeats` loops of exactly `steps` steps each, CUDA
    events, max over ranks, the median loop is reported.  Then the attention kernel alone (event pairs
    around it), and -- for the headline workload (`full`) -- the end-to-end loops through the operator
    API with the step's inputs in pinned host memory.  Ends with the CPU leg / parity check."""
    import torch
    import torch.distributed as dist

    import ms_custom_ops_b200 as ops
    from ms_custom_ops_b200 import sharding

    world, rank, dev = ctx["world"], ctx["rank"], ctx["dev"]
    K, W, R = args.steps, max(args.warmup, 3), max(args.repeats, 1)
    nprof = min(K, 64)
    total_steps = W + R * K + nprof + (2 * (3 + K) + 8 if full else 0) + 8
    loop = DecodeLoop(ctx, spec, total_steps)
    case = loop.case
    q, key, val = case["query"], case["key"], case["value"]
    kc, vc, bt = case["key_cache"], case["value_cache"], case["block_tables"]
    kd, vd = case["k_descale"], case["v_descale"]
    gathered = torch.empty((world,) + tuple(q.shape), dtype=q.dtype, device=dev) if world > 1 else None
    # the exchange: this library's peer-store all-gather kernel (default) or NCCL (--nccl-gather)
    peer = None
    if world > 1 and not args.nccl_gather:
        try:
            peer = sharding.PeerGather(q.shape, q.dtype, dev, packets=not args.flag_exchange)
        except Exception as e:  # mapping a peer's memory may be refused: say so and fall back to NCCL
            print(f"peer all-gather unavailable ({e}); using NCCL", file=sys.stderr)
        ok = torch.tensor([1 if peer is not None else 0], device=dev)
        dist.all_reduce(ok, op=dist.ReduceOp.MIN)
        if int(ok.item()) == 0:
            peer = None

    def exchange(o):
        if peer is not None:
            return peer.gather(o)
        return sharding.all_gather_outputs(o, gathered)

    fused = peer is not None and not args.separate_gather

    def step():
        # the exchange rides in the step's own finishing kernel (default) or is a launch of its own
        if fused:
            return loop.step(gather=peer)
        loop.step()
        return exchange(loop.out_local) if world > 1 else None

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def max_over_ranks(ms):
        t = torch.tensor([ms], dtype=torch.float64, device=dev)
        if world > 1:
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    # ---- device-resident timed region ------------------------------------------------------
    for _ in range(W):
        step()
    loop.kernels.pa_status(loop.plan, loop.ws)
    packet_form = fused and not args.flag_exchange
    if packet_form:
        # the packet form of the exchange is checked against NCCL before anything is timed; should it
        # disagree or time out on some rank, every rank goes over to the flag form together
        # (every rank runs the same collectives whatever its own outcome: nothing here raises in between)
        mine = step()
        torch.cuda.synchronize()
        timed_out = int(peer.words[1].item()) != 0      # a bounded wait for a peer's packets ran out
        sharding.all_gather_outputs(loop.out_local, gathered)
        torch.cuda.synchronize()
        ok = int((not timed_out) and torch.equal(mine.view(torch.int16), gathered.view(torch.int16)))
        if not ok:
            print(f"packet exchange failed its check on rank {rank} (timed out: {timed_out})", file=sys.stderr)
        t_ok = torch.tensor([ok], device=dev)
        dist.all_reduce(t_ok, op=dist.ReduceOp.MIN)
        if int(t_ok.item()) == 0:
            if rank == 0:
                print("packet exchange did not pass its check: using fences + flags", file=sys.stderr)
            peer.release()
            peer = sharding.PeerGather(q.shape, q.dtype, dev, packets=False)
            packet_form = False
            step()
    # clocks are sampled from the start of the device-timed region to the end of the end-to-end region
    sampler = None
    if rank == 0 and full:
        sampler = ClockSampler("GPU-" + str(torch.cuda.get_device_properties(dev).uuid)).start()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    loops_ms = []
    first_timed = loop.i
    for _ in range(R):
        barrier()
        e0.record()
        for _ in range(K):
            step()
        e1.record()
        barrier()
        loops_ms.append(max_over_ranks(e0.elapsed_time(e1)) / K)
    ms_step = statistics.median(loops_ms)
    # duration of the attention kernel alone: the same steps once more with the library's event pairs
    # recorded directly around that kernel (the pairs would sit between the kernels of the timed
    # region and break their programmatic overlap, so they are taken in a pass of their own)
    loop.plan.profile_enable(True)
    first_prof = loop.i
    for _ in range(nprof):
        step()
    torch.cuda.synchronize()
    kernel_ms = loop.plan.profile_read()
    loop.plan.profile_enable(False)
    info = loop.plan.info()

    spec_b = spec.batch
    result = {"value": spec_b / ms_step * 1e3, "ms_per_step": ms_step, "loops_ms_per_step": loops_ms,
              "first_timed_step": first_timed}
    e2e = None
    if full:
        e2e = measure_e2e(ctx, loop, args, exchange, barrier, max_over_ranks)
    clocks = sampler.stop() if sampler else None
    ops.paged_attention_check_status(dev)
    gather_check = None
    if peer is not None:
        peer.check()
        # the peer-store gather must equal NCCL's all-gather of the same slices, bit for bit
        mine = step()
        torch.cuda.synchronize()
        peer.check()
        sharding.all_gather_outputs(loop.out_local, gathered)
        gather_check = bool(torch.equal(mine.view(torch.int16), gathered.view(torch.int16)))

    # ---- roofline of the attention kernel (rank 0's shard) ----------------------------------
    alg_bytes = loop.algorithmic_bytes(first_prof, nprof)
    peak, peak_src = measured_hbm_peak()
    roofline = {"bound": "hbm", "achieved": None, "peak": peak, "unit": "GB/s", "frac": None, "traffic": None,
                "kernel": "pa_tma_kernel" if info.kernel == 2 else "pa_generic_kernel",
                "peak_source": peak_src, "algorithmic_bytes": alg_bytes}
    if kernel_ms:
        kms = statistics.mean(kernel_ms)
        roofline.update(achieved=alg_bytes / kms / 1e6, frac=alg_bytes / kms / 1e6 / peak, kernel_ms=kms,
                        frac_of_8tbs=alg_bytes / kms / 1e6 / 8000.0, launches_timed=len(kernel_ms))
    # DRAM traffic of one launch: dram__bytes_read.sum + dram__bytes_write.sum of the ncu captures
    # summarised in profiles/pa_tma_kernel_*.md, per context token per kv head, scaled to this
    # launch (traffic grows in proportion to the tokens read; measured on one GPU holding all heads)
    if info.kernel == 2:
        per = NCU_DRAM_BYTES_PER_TOKEN_HEAD["int8" if spec.kv_int8 else "16bit"] * spec.head_size / 128.0
        roofline["traffic"] = per * float(loop.lens_at(first_prof + nprof // 2).sum()) * loop.hpr
        roofline["traffic_source"] = ("ncu capture of config " + ("3" if spec.kv_int8 else "2") +
                                      " on one GPU, scaled by tokens x kv heads of this rank")

    # ---- CPU baseline on the same workload (also the full-size parity check) ---------------
    cpu = checked = None
    if rank == 0 and not args.no_cpu:
        last = loop.i
        loop.step()                 # one more step whose output is compared (its index: `last`)
        torch.cuda.synchronize()
        cpu, checked = loop.cpu_check(args, loop.out_local, last)

    # scatter + attention + the finishing kernel (split merge; also the exchange of a sharded step) [+ a gather
    # launch of its own with --separate-gather]
    finishing = 1 if (info.partials > 0 or min(loop.lens0) == 0 or fused) else 0
    launches_per_step = 2 + finishing + (1 if peer is not None and not fused else 0)
    result.update({
        "roofline": roofline, "cpu_baseline": cpu, "parity_check": checked, "gather_check": gather_check,
        "clocks": clocks, "e2e": e2e, "kernels_per_step": launches_per_step,
        "achieved_gbs_step": alg_bytes / ms_step / 1e6, "alg_bytes": alg_bytes,
        "config": workload_config(spec, loop.lens_at(first_timed), {
            "parallelism": f"kv-head sharding x{world}" + (
                "" if world == 1 else (
                    (" + peer-store all-gather of outputs over NVLink"
                     + ((" from the kernel that finishes the output rows, as 8-byte packets that carry their step number"
                        if packet_form else " from the kernel that finishes the output rows, fences + flags")
                       if fused else " (a launch of its own)"))
                    if peer is not None else " + NCCL all-gather of outputs")),
            "l2": f"inputs larger than L2: {alg_bytes / 1e6:.0f} MB of KV per GPU per step vs {L2_BYTES >> 20} MB",
            "launch": "real decode loop: every step appends one token per sequence (context_lens + 1, slot_mapping "
                      "moves, block tables hold the blocks reserved for the growth), the plan is re-planned in place "
                      "every step, eager launches on one stream (cache scatter, attention, merge of the split "
                      "partials; programmatic launch overlap between them)",
            "timing": f"median of {R} loops of {K} steps each",
            "work_items": info.work_items, "split_partials": info.partials, "grid": info.grid}),
    })
    if peer is not None:
        peer.release()
    loop.release()
    return result


def measure_e2e(ctx, loop, args, exchange, barrier, max_over_ranks):
    """End to end through the operator API (`reshape_and_cache` + `paged_attention`, the calls a user of
    the reference makes), inputs in pinned host memory: every step uploads query / new rows / slots /
    block tables in ONE packed host->device copy and downloads the output into pinned memory.
    Every step is a plan-cache miss (the lengths grew), served by re-planning in place.
    serial    upload -> operators -> download -> the host waits for the result: what one batch of
              autoregressive decode can do, since step i + 1 needs step i's result
    pipelined two independent batches in flight: the upload of step i + 1 and the download of step
              i - 1 run on copy streams while step i computes"""
    import torch

    import ms_custom_ops_b200 as ops

    world, dev = ctx["world"], ctx["dev"]
    spec, case, K = loop.spec, loop.case, args.steps
    q, key, val = case["query"], case["key"], case["value"]
    kc, vc, bt = case["key_cache"], case["value_cache"], case["block_tables"]
    kd, vd = case["k_descale"], case["v_descale"]
    slot0 = loop.slots_dev[0]
    parts = [q, key, val, slot0, bt]
    offs, total = [], 0
    for x in parts:
        offs.append(total)
        total += (x.numel() * x.element_size() + 255) // 256 * 256
    # two staging sets: step i + 1 is uploaded while step i computes
    h_stage = [torch.empty(total, dtype=torch.uint8).pin_memory() for _ in range(2)]
    d_stage = [torch.empty(total, dtype=torch.uint8, device=dev) for _ in range(2)]

    def view(buf, x, off):
        return buf[off:off + x.numel() * x.element_size()].view(x.dtype).view(x.shape)
    for hs in h_stage:
        for x, off in zip(parts, offs):
            view(hs, x, off).copy_(x.cpu())
    h_slot = [view(hs, slot0, offs[3]) for hs in h_stage]
    d_views = [tuple(view(ds, x, off) for x, off in zip(parts, offs)) for ds in d_stage]
    out_shape = (world,) + tuple(q.shape) if world > 1 else tuple(q.shape)
    h_out = [torch.empty(out_shape, dtype=q.dtype).pin_memory() for _ in range(2)]
    pa_kw = dict(q_head_num=loop.hq_local, kv_head_num=loop.hpr, qk_scale=case["qk_scale"])
    if spec.kv_int8:
        pa_kw.update(quant_type=1, k_descale=kd, v_descale=vd)
    h_lens = loop.h_lens

    def set_step(j, slot_i):
        """Host state of step j: lengths (read by the operator on the host) and the slots in staging set slot_i."""
        np.add(loop.lens0, np.int32(j), out=loop.cur_lens)
        h_slot[slot_i].copy_(loop.slots_host[j])

    def operators(slot_i):
        d_q, d_key, d_val, d_slot, d_bt = d_views[slot_i]
        if spec.kv_int8:
            ops.reshape_and_cache_quant(d_key, d_val, kc, vc, d_slot, kd, vd)
        else:
            ops.reshape_and_cache(d_key, d_val, kc, vc, d_slot, 0, 0)
        o = ops.paged_attention(d_q, kc, vc, d_bt, h_lens, **pa_kw)
        return exchange(o) if world > 1 else o

    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)

    def time_loop(fn, finish=None):
        for _ in range(3):
            fn()
        if finish is not None:
            finish()
        barrier()
        c0, a0 = ops.plan_cache_stats(), ops.plan_arena_stats()
        e0.record()
        for _ in range(K):
            fn()
        if finish is not None:
            finish()
        e1.record()
        barrier()
        c1, a1 = ops.plan_cache_stats(), ops.plan_arena_stats()
        stats = {"steps": K, "misses": c1["misses"] - c0["misses"], "hits": c1["hits"] - c0["hits"],
                 "replanned_in_place": c1["recycled"] - c0["recycled"], "plans_created": c1["created"] - c0["created"],
                 "pinned_slabs_added": a1["slabs"] - a0["slabs"], "arena_blocks_taken": a1["block_allocs"] - a0["block_allocs"]}
        return max_over_ranks(e0.elapsed_time(e1)) / K, stats

    # (1) serial.  What step i + 1 needs from step i's result is the CONTENT of its inputs; its lengths
    # (one more token per sequence) and slots are known beforehand, so -- as a serving loop would --
    # the host prepares them, and has the next step's launch plan made (a planning-only operator call
    # that leaves the plan in the cache), while the GPU runs step i.  The staging sets alternate so
    # that the pinned buffer being filled is never the one an upload may still be reading.
    def plan_ahead(slot_i):
        d_q, _, _, _, d_bt = d_views[slot_i]
        ops.paged_attention_workspace_size(d_q, kc, vc, d_bt, h_lens, **pa_kw)

    set_step(loop.i, loop.i & 1)

    def serial_step():
        si = loop.i & 1
        d_stage[si].copy_(h_stage[si], non_blocking=True)
        o = operators(si)
        h_out[0].copy_(o, non_blocking=True)
        set_step(loop.i + 1, si ^ 1)               # host work of the next step, under this step's GPU time
        plan_ahead(si ^ 1)
        torch.cuda.current_stream().synchronize()  # the step's result is read on the host
        loop.i += 1
    serial_ms, serial_stats = time_loop(serial_step)
    set_step(loop.i, 0)                            # the loops below start from the lengths of step loop.i

    # (2) pipelined
    comp = torch.cuda.current_stream()
    s_in, s_out = torch.cuda.Stream(), torch.cuda.Stream()
    ev_in = [torch.cuda.Event() for _ in range(2)]      # staging set uploaded
    ev_done = [torch.cuda.Event() for _ in range(2)]    # operators that read the set have finished
    ev_out = [torch.cuda.Event() for _ in range(2)]     # result is in pinned host memory
    state = {"n": 0, "primed": False}
    d_out = [torch.empty(out_shape, dtype=q.dtype, device=dev) for _ in range(2)] if world > 1 else None

    def upload(slot_i, j):
        ev_in[slot_i].synchronize()                      # the set's previous upload has left the pinned buffer
        h_slot[slot_i].copy_(loop.slots_host[j])
        s_in.wait_event(ev_done[slot_i])                 # the set's previous readers are done
        with torch.cuda.stream(s_in):
            d_stage[slot_i].copy_(h_stage[slot_i], non_blocking=True)
            ev_in[slot_i].record(s_in)

    def pipelined_step():
        n, j = state["n"], loop.i
        cur = n & 1
        if not state["primed"]:
            for e in ev_done + ev_out + ev_in:
                e.record(comp)
            upload(cur, j)
            state["primed"] = True
        upload(cur ^ 1, j + 1)                           # next step's inputs, behind this step's kernels
        np.add(loop.lens0, np.int32(j), out=loop.cur_lens)
        comp.wait_event(ev_in[cur])
        o = operators(cur)
        if world > 1:
            # the gathered buffer is written by the peers again two steps on: download a private copy
            comp.wait_event(ev_out[cur])
            d_out[cur].copy_(o)
            o = d_out[cur]
        ev_done[cur].record(comp)
        ev_out[cur].synchronize()                        # the result of step i - 2 is read on the host
        s_out.wait_event(ev_done[cur])
        with torch.cuda.stream(s_out):
            h_out[cur].copy_(o, non_blocking=True)
            ev_out[cur].record(s_out)
        if world == 1:
            o.record_stream(s_out)
        state["n"] = n + 1
        loop.i = j + 1

    def drain():
        for e in ev_out:
            e.synchronize()
        comp.wait_stream(s_out)
        comp.wait_stream(s_in)
    pipe_ms, pipe_stats = time_loop(pipelined_step, drain)
    h2d = sum(x.numel() * x.element_size() for x in parts)
    d2h = h_out[0].numel() * h_out[0].element_size()
    b = spec.batch
    return {"value": b / serial_ms * 1e3, "unit": UNIT, "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h,
            "ms_per_step": serial_ms,
            "mode": "serial: upload -> reshape_and_cache + paged_attention (operator API) -> download -> host waits; "
                    "lengths grow every step, every step needs a new launch plan (a plan-cache miss, re-planned in "
                    "place), which the host has made by a planning-only operator call while the GPU ran the step "
                    "before -- the lengths of a decode step are known ahead, its inputs are not",
            "plan_cache": serial_stats,
            "pipelined_value": b / pipe_ms * 1e3, "pipelined_ms_per_step": pipe_ms,
            "pipelined_mode": "two independent batches in flight: copy streams move step i+1's inputs and step i-1's "
                              "result while step i computes; results read on the host two steps after launch",
            "pipelined_plan_cache": pipe_stats}


def run_gpu(args):
    import torch
    import torch.distributed as dist

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if world != args.gpus and world > 1:
        raise SystemExit(f"--gpus {args.gpus} but WORLD_SIZE={world}")
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl", device_id=dev)
    ctx = {"world": world, "rank": rank, "dev": dev}

    spec = workload_spec(args.workload)
    head = measure_decode(ctx, spec, args, full=True)

    # ---- the other benchmark configurations, same loop, device-timed + kernel roofline + parity ----
    extras = {}
    if not args.no_extra:
        names = ["c3", "c4", "c5", "c2h64", "c2h256"] if world == 1 else ["c4"]
        if args.configs:
            names = [n for n in names if n in args.configs.split(",")]
        for name in names:
            if name == args.workload.lower():
                continue
            r = measure_decode(ctx, workload_spec(name), args, full=False)
            if rank == 0:
                rf = r["roofline"]
                extras[name] = {
                    "workload": r["config"]["workload"], "kv_tokens": r["config"]["kv_tokens"],
                    "parallelism": r["config"]["parallelism"], "value": r["value"], "unit": UNIT,
                    "ms_per_step": r["ms_per_step"], "attention_kernel_ms": rf.get("kernel_ms"),
                    "roofline": {k: rf.get(k) for k in ("achieved", "peak", "frac", "frac_of_8tbs", "algorithmic_bytes",
                                                        "kernel", "peak_source")},
                    "parity_check": r["parity_check"], "gather_check": r["gather_check"],
                    "cpu_baseline": r["cpu_baseline"], "work_items": r["config"]["work_items"],
                    "split_partials": r["config"]["split_partials"]}
    peak, _ = measured_hbm_peak()
    scatter = adjacent = None
    if world == 1 and not args.no_extra and (not args.configs or "rac_prefill" in args.configs.split(",")):
        scatter = measure_scatter(workload_spec("c5"), dev, peak)
        if rank == 0:
            extras["rac_prefill"] = scatter
    if world == 1 and not args.no_extra and (not args.configs or "mtp4" in args.configs.split(",")):
        extras["mtp4"] = measure_mtp(spec, dev)
    if world == 1 and args.adjacent:
        case = workloads.decode_case_device(spec, dev, (0, spec.kv_heads))
        adjacent = measure_adjacent(case, spec, dev, peak, not args.no_cpu)

    if rank == 0:
        cpu_np = None if args.no_cpu else cpu_numpy_config1()
        line = {
            "metric": METRIC, "value": head["value"], "unit": UNIT, "n_gpus": world, "steps": args.steps,
            "warmup": max(args.warmup, 3), "ms_per_step": head["ms_per_step"], "higher_is_better": True,
            "scaling": "strong", "vs_baseline": None, "dtype": "bf16" if spec.dtype == "bfloat16" else "f16",
            "data": "synthetic", "config": head["config"], "e2e": head["e2e"],
            "gpu_launches": head["kernels_per_step"] * args.steps,
            "roofline": head["roofline"], "cpu_baseline": head["cpu_baseline"], "cpu_baseline_numpy": cpu_np,
            "parity_check": head["parity_check"], "gather_check": head["gather_check"], "clocks": head["clocks"],
            "loops_ms_per_step": head["loops_ms_per_step"], "achieved_gbs_step": head["achieved_gbs_step"],
            "configs": extras, "adjacent_ops": adjacent,
        }
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


def run_gpu_seq_parallel(args):
    """--seq-parallel: the second sharding axis.  Every rank holds ALL heads and a contiguous range of
    whole cache blocks of every sequence; one step = scatter of the new rows (they land on the rank that
    owns each sequence's last block), attention over the local part with the log-sum-exp as second
    output, an all-gather of the per-rank (output, lse) records and their merge (fa_update arithmetic).
    Same metric and timing rules as the default mode; `scaling` is "strong"."""
    import torch
    import torch.distributed as dist

    from ms_custom_ops_b200 import _abi, kernels, sharding

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if world < 2 or world != args.gpus:
        raise SystemExit("--seq-parallel needs torchrun with --gpus N >= 2 ranks")
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
    dist.init_process_group("nccl", device_id=dev)

    spec = workload_spec(args.workload)
    # the same seeded caches on every rank (each rank only reads its own blocks of them)
    case = workloads.decode_case_device(spec, dev, (0, spec.kv_heads))
    lens = np.asarray([int(x) for x in case["context_lens"]], dtype=np.int32)
    quant = 1 if spec.kv_int8 else 0
    q, key, val = case["query"], case["key"], case["value"]
    kc, vc, slot = case["key_cache"], case["value_cache"], case["slot_mapping"]
    kd, vd = case["k_descale"], case["v_descale"]
    tables_host = case["block_tables"].cpu().numpy()
    lt, ll = sharding.seq_shard_tables(tables_host, lens, spec.block_size, rank, world)
    bt_local = torch.from_numpy(lt).to(dev)
    # the last rank's block range always ends with a sequence's last block: the new rows land there
    slot_local = slot if rank == world - 1 else torch.full_like(slot, -1)

    desc = kernels.make_pa_desc(q, kc, bt_local, case["qk_scale"], quant)
    plan = _abi.PaPlan(desc, [int(x) for x in ll])
    info = plan.info()
    ws = torch.empty(max(plan.workspace_bytes, 256), dtype=torch.uint8, device=dev)
    xch = sharding.SeqParallelExchange(spec.batch, spec.num_heads, spec.head_size, q.dtype, dev,
                                       use_peer_stores=not args.nccl_gather)

    def step():
        if quant:
            kernels.rac_scatter_quant(key, val, kc, vc, slot_local, kd, vd)
        else:
            kernels.rac_scatter(key, val, kc, vc, slot_local)
        kernels.pa_launch(plan, q, kc, vc, bt_local, xch.out_local, ws, kd, None, vd, None, None, xch.lse_local)
        return xch.exchange_and_merge()

    def barrier():
        dist.barrier()
        torch.cuda.synchronize()

    for _ in range(max(args.warmup, 3)):
        step()
    kernels.pa_status(plan, ws)
    sampler = ClockSampler("GPU-" + str(torch.cuda.get_device_properties(dev).uuid)).start() if rank == 0 else None
    barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(args.steps):
        step()
    e1.record()
    barrier()
    t = torch.tensor([e0.elapsed_time(e1)], dtype=torch.float64, device=dev)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    ms_step = float(t.item()) / args.steps
    plan.profile_enable(True)
    for _ in range(min(args.steps, 64)):
        step()
    torch.cuda.synchronize()
    kernel_ms = plan.profile_read()
    plan.profile_enable(False)
    clocks = sampler.stop() if sampler else None
    xch.check()
    merged = step().clone()
    torch.cuda.synchronize()

    # end to end, serial: upload query / new rows, step, download the merged output, host waits
    parts = [q, key, val]
    h_parts = [x.cpu().pin_memory() for x in parts]
    h_out = torch.empty(merged.shape, dtype=merged.dtype).pin_memory()

    def e2e_step():
        for d_x, h_x in zip(parts, h_parts):
            d_x.copy_(h_x, non_blocking=True)
        h_out.copy_(step(), non_blocking=True)
        torch.cuda.current_stream().synchronize()
    for _ in range(3):
        e2e_step()
    barrier()
    e0.record()
    for _ in range(args.steps):
        e2e_step()
    e1.record()
    barrier()
    t = torch.tensor([e0.elapsed_time(e1)], dtype=torch.float64, device=dev)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    e2e_ms = float(t.item()) / args.steps

    if rank == 0:
        kvb = 1 if spec.kv_int8 else 2
        alg_bytes = workloads.algorithmic_bytes_attention([int(x) for x in ll], spec.num_heads, spec.kv_heads,
                                                          spec.head_size, kvb, quant=spec.kv_int8)
        peak, peak_src = measured_hbm_peak()
        roofline = {"bound": "hbm", "achieved": None, "peak": peak, "unit": "GB/s", "frac": None, "traffic": None,
                    "kernel": "pa_tma_kernel" if info.kernel == 2 else "pa_generic_kernel", "peak_source": peak_src,
                    "algorithmic_bytes": alg_bytes, "note": "rank 0's part of every context"}
        if kernel_ms:
            kms = statistics.mean(kernel_ms)
            roofline.update(achieved=alg_bytes / kms / 1e6, frac=alg_bytes / kms / 1e6 / peak, kernel_ms=kms,
                            frac_of_8tbs=alg_bytes / kms / 1e6 / 8000.0, launches_timed=len(kernel_ms))
        checked = None
        if not args.no_cpu:
            from oracle import c_oracle
            nseq = min(spec.batch, 8)
            host = {"query": _to_np(q[:nseq]), "key": _to_np(key[:nseq]), "value": _to_np(val[:nseq]),
                    "key_cache": _to_np(kc), "value_cache": _to_np(vc), "block_tables": tables_host[:nseq],
                    "slot_mapping": slot[:nseq].cpu().numpy(), "context_lens": lens[:nseq],
                    "qk_scale": case["qk_scale"], "k_descale": None if kd is None else kd.cpu().numpy(),
                    "v_descale": None if vd is None else vd.cpu().numpy()}
            # rank 0 only wrote the rows it owns into its copy of the caches: let the oracle scatter all
            ref = cpu_step(c_oracle, host, host_threads())
            got = merged[:nseq].float().cpu().numpy()
            err = np.abs(got - ref)
            tol = 2e-2 if spec.kv_int8 else 1e-2
            checked = {"sequences": nseq, "max_abs_err": float(err.max()), "max_abs_golden": float(np.abs(ref).max()),
                       "within_tolerance": bool(np.all(err <= tol + tol * np.abs(ref))), "tolerance": tol}
        launches = 3 + (1 if info.partials > 0 or int(ll.min()) == 0 else 0) + (0 if args.nccl_gather else 1)
        line = {
            "metric": METRIC, "value": spec.batch / ms_step * 1e3, "unit": UNIT, "n_gpus": world, "steps": args.steps,
            "warmup": max(args.warmup, 3), "ms_per_step": ms_step, "higher_is_better": True, "scaling": "strong",
            "vs_baseline": None, "dtype": "bf16" if spec.dtype == "bfloat16" else "f16", "data": "synthetic",
            "config": workload_config(spec, [int(x) for x in lens], {
                "parallelism": f"sequence sharding x{world}: block ranges of every context per rank, all heads; "
                               + ("NCCL" if args.nccl_gather else "peer-store") + " all-gather of (output, lse) records, "
                               "fa_update merge on every rank",
                "l2": f"inputs larger than L2: {alg_bytes / 1e6:.0f} MB of KV on rank 0 per step vs {L2_BYTES >> 20} MB",
                "launch": "eager launches on one stream", "work_items": info.work_items,
                "split_partials": info.partials, "grid": info.grid}),
            "e2e": {"value": spec.batch / e2e_ms * 1e3, "unit": UNIT,
                    "h2d_bytes_per_step": sum(x.numel() * x.element_size() for x in parts),
                    "d2h_bytes_per_step": h_out.numel() * h_out.element_size(), "ms_per_step": e2e_ms,
                    "mode": "serial: upload, step, download, host waits"},
            "gpu_launches": launches * args.steps, "roofline": roofline, "cpu_baseline": None,
            "parity_check": checked, "clocks": clocks,
        }
        print(json.dumps(line), flush=True)
    dist.barrier()
    xch.release()
    dist.destroy_process_group()


def measure_mtp(spec, dev, q_len=4):
    """Multi-token (speculative) decode on the headline workload's shapes: `q_len` query tokens per
    sequence (calc_type = 1, q_seq_lens) against one, same caches and lengths, operator API, device
    resident.  The tokens of a sequence are rows of ONE work item, so the context is read from HBM once:
    the ratio of the two step times is the figure.  Without a mask every token of a sequence sees the
    same context, so row t of the stacked result must equal a one-token decode of query t."""
    import torch
    import ms_custom_ops_b200 as ops
    case = workloads.decode_case_device(spec, dev, (0, spec.kv_heads))
    kc, vc, bt = case["key_cache"], case["value_cache"], case["block_tables"]
    lens = torch.from_numpy(np.asarray(case["context_lens"], dtype=np.int32))
    gen = torch.Generator(device=dev)
    gen.manual_seed(spec.seed + 17)
    q = torch.randn((spec.batch * q_len, spec.num_heads, spec.head_size), generator=gen, device=dev).to(kc.dtype)
    ql = torch.full((spec.batch,), q_len, dtype=torch.int32)
    kw = dict(q_head_num=spec.num_heads, kv_head_num=spec.kv_heads, qk_scale=case["qk_scale"])
    q1 = q.view(spec.batch, q_len, spec.num_heads, spec.head_size)[:, 0].contiguous()

    def timed(fn, reps=20):
        for _ in range(4):
            fn()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(reps):
            fn()
        e1.record()
        torch.cuda.synchronize()
        return e0.elapsed_time(e1) / reps

    one = timed(lambda: ops.paged_attention(q1, kc, vc, bt, lens, **kw))
    many = timed(lambda: ops.paged_attention(q, kc, vc, bt, lens, calc_type=1, q_seq_lens=ql, **kw))
    stacked = ops.paged_attention(q, kc, vc, bt, lens, calc_type=1, q_seq_lens=ql, **kw)
    stacked = stacked.view(spec.batch, q_len, spec.num_heads, spec.head_size)
    worst = 0.0
    for t in range(q_len):
        qt = q.view(spec.batch, q_len, spec.num_heads, spec.head_size)[:, t].contiguous()
        single = ops.paged_attention(qt, kc, vc, bt, lens, **kw)
        worst = max(worst, float((single.float() - stacked[:, t].float()).abs().max()))
    ops.paged_attention_check_status(dev)
    return {"workload": f"{spec.name} shapes, {q_len} query tokens per sequence (calc_type 1), no mask",
            "q_tokens_per_sequence": q_len, "ms_one_token": one, "ms_multi_token": many, "ratio": many / one,
            "tokens_per_s": spec.batch * q_len / many * 1e3,
            "max_abs_diff_vs_one_token_decodes": worst}


def measure_scatter(spec, dev, peak):
    """Prefill-heavy reshape_and_cache of configuration 5: 16384 tokens (8 kv heads x 128) through an
    injective random slot map into 4096 blocks of 128 with 5 % of the slots set to -1, bf16 copy and
    bf16 -> int8 quantising variants.  Four distinct input / cache sets rotate (each > L2), the
    four launches are captured in a CUDA graph and replayed, CUDA events around the replays."""
    import torch
    from ms_custom_ops_b200 import kernels
    tokens, blocks, pad = spec.extra["rac_tokens"], spec.extra["rac_blocks"], spec.extra["pad_frac"]
    c = spec.kv_heads * spec.head_size
    tdt = torch.bfloat16 if spec.dtype == "bfloat16" else torch.float16
    rng = np.random.default_rng(spec.seed)
    gen = torch.Generator(device=dev)
    gen.manual_seed(spec.seed)
    out = {"tokens": tokens, "blocks": blocks, "padding_fraction": pad, "sets": 4,
           "l2": "4 rotating input/cache sets, each larger than L2"}
    kd = torch.rand(c, generator=gen, device=dev) * 0.04 + 0.01
    vd = torch.rand(c, generator=gen, device=dev) * 0.04 + 0.01
    for name, quant in (("copy", False), ("quant_int8", True)):
        sets = []
        for _ in range(4):
            slots = rng.permutation(blocks * spec.block_size)[:tokens].astype(np.int32)
            slots[rng.random(tokens) < pad] = -1
            key = torch.randn((tokens, c), generator=gen, device=dev).to(tdt)
            val = torch.randn((tokens, c), generator=gen, device=dev).to(tdt)
            kc = torch.zeros((blocks, spec.block_size, spec.kv_heads, spec.head_size),
                             dtype=torch.int8 if quant else tdt, device=dev)
            sets.append((key, val, kc, torch.zeros_like(kc), torch.from_numpy(slots).to(dev), slots))

        def go(i):
            key, val, kc, vc, sl, _ = sets[i]
            if quant:
                kernels.rac_scatter_quant(key, val, kc, vc, sl, kd, vd)
            else:
                kernels.rac_scatter(key, val, kc, vc, sl)
        side = torch.cuda.Stream()
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):
            for i in range(4):
                go(i)
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph, stream=side):
                for i in range(4):
                    go(i)
        torch.cuda.current_stream().wait_stream(side)
        for _ in range(3):
            graph.replay()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        reps = 10
        e0.record()
        for _ in range(reps):
            graph.replay()
        e1.record()
        torch.cuda.synchronize()
        ms = e0.elapsed_time(e1) / (reps * 4)
        nbytes = workloads.algorithmic_bytes_scatter(sets[0][5], c, 2, 1 if quant else 2, quant)
        out[name] = {"ms": ms, "algorithmic_bytes": nbytes, "achieved_gbs": nbytes / ms / 1e6,
                     "frac": nbytes / ms / 1e6 / peak, "frac_of_8tbs": nbytes / ms / 1e6 / 8000.0,
                     "tokens_per_s": tokens / ms * 1e3}
        del sets, graph
        torch.cuda.empty_cache()
    return out


def cpu_leg_cache_load(kc, vc, bt, lens, ko, vo):
    """CPU baseline and bit-exactness check of one paged_cache_load: the C restatement of the reference
    golden on all host cores over the same caches (torch tensors in, device or host)."""
    from oracle import c_oracle
    hk, hv, hbt = _to_np(kc), _to_np(vc), bt.cpu().numpy()
    cores = host_threads()
    total = int(np.asarray(lens).sum())
    c_oracle.paged_cache_load(hk[:2], hv[:2], np.zeros((1, 1), np.int32), np.array([1], np.int32), threads=cores)
    t_best = float("inf")
    for _ in range(3):
        t0 = time.perf_counter()
        gk, gv = c_oracle.paged_cache_load(hk, hv, hbt, lens, threads=cores)
        t_best = min(t_best, time.perf_counter() - t0)
    return {
        "cpu_baseline": {"value": total / t_best, "unit": "tokens/s", "cores": cores, "kind": "port",
                         "sample": "the whole batch, best of 3; C restatement of the reference golden, "
                                   "OpenMP over sequences"},
        "bit_exact": bool(np.array_equal(_to_np(ko).view(np.uint8), gk.view(np.uint8)) and
                          np.array_equal(_to_np(vo).view(np.uint8), gv.view(np.uint8)))}


def cpu_leg_fa_update(lse, lo, merged):
    """CPU baseline and error of one fa_update: the C restatement of the reference golden, all cores."""
    from oracle import c_oracle
    cores = host_threads()
    hl, ho = lse.cpu().numpy(), lo.cpu().numpy()
    t_best = float("inf")
    for _ in range(3):
        t0 = time.perf_counter()
        g = c_oracle.fa_update(hl, ho, threads=cores)
        t_best = min(t_best, time.perf_counter() - t0)
    return {
        "cpu_baseline": {"value": hl.shape[1] / t_best, "unit": "rows/s", "cores": cores, "kind": "port",
                         "sample": "all rows, best of 3; C restatement of the reference golden, OpenMP over rows"},
        "max_abs_err": float(np.abs(merged.cpu().numpy() - g).max())}


def measure_adjacent(case, spec, dev, peak, with_cpu):
    """The two operators either side of the decode path, on the same workload, one GPU:
    paged_cache_load gathers every sequence of the batch out of the paged caches (reads and writes the
    whole KV working set, far larger than L2), fa_update merges 3 partial outputs of 256000 rows x 128
    (the reference test's largest shape; 524 MB per launch).  CUDA events around `reps` eager launches."""
    import torch
    from ms_custom_ops_b200 import kernels
    out = {}
    kc, vc, bt = case["key_cache"], case["value_cache"], case["block_tables"]
    lens = np.asarray([int(x) for x in case["context_lens"]], dtype=np.int32)
    total = int(lens.sum())
    krow = kc[0, 0].numel() * kc.element_size()
    vrow = vc[0, 0].numel() * vc.element_size()
    lens_dev = torch.from_numpy(lens).to(dev)
    ko = torch.empty((total,) + tuple(kc.shape[2:]), dtype=kc.dtype, device=dev)
    vo = torch.empty((total,) + tuple(vc.shape[2:]), dtype=vc.dtype, device=dev)
    ws = torch.empty(kernels.cache_load_workspace_bytes(bt.shape[0], bt.shape[1]), dtype=torch.uint8, device=dev)
    oob = torch.zeros(1, dtype=torch.int32, device=dev)

    def timed(fn, reps):
        for _ in range(3):
            fn()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(reps):
            fn()
        e1.record()
        torch.cuda.synchronize()
        return e0.elapsed_time(e1) / reps
    ms = timed(lambda: kernels.cache_load(kc, vc, bt, lens_dev, None, ko, vo, ws, False, oob), 10)
    nbytes = 2 * total * (krow + vrow)
    out["paged_cache_load"] = {
        "tokens": total, "ms": ms, "algorithmic_bytes": nbytes, "achieved_gbs": nbytes / ms / 1e6,
        "frac": nbytes / ms / 1e6 / peak, "frac_of_8tbs": nbytes / ms / 1e6 / 8000.0, "tokens_per_s": total / ms * 1e3,
        "kernels_per_call": 2, "out_of_range_ids": int(oob.item()),
        "l2": f"{nbytes / 2e6:.0f} MB read and as much written per launch vs {L2_BYTES >> 20} MB of L2"}
    if with_cpu:
        out["paged_cache_load"].update(cpu_leg_cache_load(kc, vc, bt, lens, ko, vo))
    del ko, vo
    torch.cuda.empty_cache()

    sp, rows, hd = 3, 2 * 4000 * 32, 128
    gen = torch.Generator(device=dev)
    gen.manual_seed(spec.seed)
    lse = torch.rand((sp, rows), generator=gen, device=dev) * 8 - 4
    lo = torch.rand((sp, rows, hd), generator=gen, device=dev)
    merged = torch.empty((rows, hd), dtype=torch.float32, device=dev)
    ms = timed(lambda: kernels.merge_partials(lse, lo, merged), 20)
    nbytes = (sp * rows * (hd + 1) + rows * hd) * 4
    out["fa_update"] = {
        "sp": sp, "rows": rows, "head_size": hd, "ms": ms, "algorithmic_bytes": nbytes,
        "achieved_gbs": nbytes / ms / 1e6, "frac": nbytes / ms / 1e6 / peak, "frac_of_8tbs": nbytes / ms / 1e6 / 8000.0,
        "rows_per_s": rows / ms * 1e3, "l2": f"{nbytes / 1e6:.0f} MB per launch vs {L2_BYTES >> 20} MB of L2"}
    if with_cpu:
        out["fa_update"].update(cpu_leg_fa_update(lse, lo, merged))
    return out


def _to_np(t):
    import torch
    t = t.detach().cpu().contiguous()
    if t.dtype == torch.bfloat16:
        return t.view(torch.uint16).numpy().view(workloads.bfloat16)
    return t.numpy()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=50)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--workload", default="c2", help="c1..c5: benchmark configuration (default c2)")
    ap.add_argument("--impl", default="b200", choices=["b200", "reference"])
    ap.add_argument("--repeats", type=int, default=5, help="timed loops of --steps steps each; the median is reported")
    ap.add_argument("--no-extra", action="store_true",
                    help="only the headline workload (skip the `configs` entries: c3, c4, c5, prefill scatter)")
    ap.add_argument("--cpu-seconds", type=float, default=12.0, help="time budget of one CPU baseline leg")
    ap.add_argument("--configs", default="", help="comma-separated subset of the `configs` entries to run "
                    "(c3,c4,c5,c2h64,c2h256,rac_prefill,mtp4); default: all")
    ap.add_argument("--nccl-gather", action="store_true", help="exchange outputs with NCCL instead of peer stores")
    ap.add_argument("--flag-exchange", action="store_true",
                    help="N > 1: the step's own exchange uses fences and one flag per rank instead of 8-byte "
                         "packets that carry their step number")
    ap.add_argument("--separate-gather", action="store_true",
                    help="N > 1: launch the peer-store all-gather as a kernel of its own behind the step instead "
                         "of from the step's finishing kernel")
    ap.add_argument("--no-cpu", action="store_true", help="skip the CPU baseline / parity check")
    ap.add_argument("--seq-parallel", action="store_true",
                    help="shard every context over the ranks (all heads per rank) instead of the kv heads")
    ap.add_argument("--adjacent", action="store_true",
                    help="also time paged_cache_load and fa_update on this workload (1 GPU)")
    ap.add_argument("--cpu-sample", type=int, default=64, help="sequences in the CPU sample")
    args = ap.parse_args()
    if args.impl == "reference":
        run_reference(args)
    elif args.seq_parallel:
        run_gpu_seq_parallel(args)
    else:
        run_gpu(args)


if __name__ == "__main__":
    main()
