#!/usr/bin/env python3
"""Benchmark of the PTX front end (lex + parse to records) on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--modules M] [--bytes B]

A step is one pass of the whole front end over one batch of synthetic PTX modules: the fatbin-scale configuration
(4,096 independent modules, ~1 GiB of text, log-normal sizes, mixed sm_80/86/90 targets, 10 % tensor-core tile
statements; every statement drawn independently with fresh registers, int32 immediates and normal(0,1) hex floats).
With N > 1 (torchrun, one rank per GPU) the global module list of N x 4,096 modules is split by byte-balanced greedy
partitioning; ranks exchange nothing on the data path (weak scaling).

Printed JSON line (rank 0):
  value      front-end GB/s of input text with the text already resident in HBM (all kernels, CUDA-event timed on the
             library's stream, max over ranks)
  e2e        the same through ptxfe_parse_batch with pinned host text: H2D of the text and D2H of all result
             records inside the timed region
  roofline   the dominant kernel: algorithmic bytes / its CUDA-event time, against the measured HBM copy peak
  cpu_baseline  the CPU restatement of ptx_parser (the oracle) on all host cores, on a bounded sample of the workload
  parity_checked / parity_ok   outside the timed region: the canonical-dump hash of every 16th module of the timed
             batch, as produced by the timed call, against the oracle's; the run fails if one differs
--impl reference times that CPU implementation as the main line (the Rust crate itself cannot be built here).
"""
import argparse
import ctypes
import json
import os
import subprocess
import sys
import threading
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

METRIC = "ptx_front_end_throughput"
UNIT = "GB/s"


# (dram__bytes_read.sum + dram__bytes_write.sum) / text bytes, from the ncu captures summarised under profiles/
NCU_DRAM_BYTES_PER_TEXT_BYTE = {      # from the ncu captures summarised under profiles/ (512 MiB instance of the workload)
    "lex_emit": 4.20, "lex_mark": 1.32, "structure": 0.74, "lex_context_vectors": 1.03, "emit_records": 4.48,
}


def measured_hbm_peak():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        return float(json.load(open(p))["hbm_gbs"]), "measured"
    return 6650.0, "fallback"


class ClockSampler:
    """SM clock and throttle reasons during the timed region: ONE nvidia-smi process in loop mode (a new process per
    sample would re-initialise NVML every time and disturb the host thread that drives the GPU)."""

    NAMES = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]

    def __init__(self, index):
        self.index, self.samples, self.reasons, self.max_mhz, self.proc, self.stop_flag = index, [], set(), None, None, False

    def start(self):
        q = "clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown," \
            "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap"
        try:
            self.proc = subprocess.Popen(["nvidia-smi", "-i", str(self.index), "--query-gpu=" + q, "--format=csv,noheader,nounits", "-lms", "200"],
                                         stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
        except Exception:
            self.proc = None

    def join(self):
        if not self.proc:
            return
        self.proc.terminate()        # the exact process started above
        try:
            out, _ = self.proc.communicate(timeout=5)
        except Exception:
            self.proc.kill()
            out = ""
        for line in out.strip().split("\n"):
            f = [x.strip() for x in line.split(",")]
            if len(f) < 6:
                continue
            try:
                self.samples.append(float(f[0]))
                self.max_mhz = float(f[1])
            except ValueError:
                continue
            for n, v in zip(self.NAMES, f[2:]):
                if v.lower().startswith("active"):
                    self.reasons.add(n)

    def summary(self):
        return {"sm_mhz": float(np.median(self.samples)) if self.samples else None, "sm_max_mhz": self.max_mhz,
                "reasons": sorted(self.reasons), "samples": len(self.samples)}


def workload_selection(rank, world, n_modules, total_bytes, seed=1001):
    """(module indices of this rank or None for all, modules in the global list, bytes of the global list): the global
    list has world x n_modules modules and is split by byte-balanced greedy partitioning."""
    from zluda_b200 import corpus
    if world == 1:
        return None, n_modules, total_bytes
    sizes = corpus.config1_sizes(seed, n_modules * world, total_bytes * world)
    return corpus.greedy_partition(sizes, world)[rank], n_modules * world, total_bytes * world


def make_workload(rank, world, n_modules, total_bytes, seed=1001):
    """The rank's share of the global module list as a list of bytes objects (small instances: tests)."""
    from zluda_b200 import corpus
    mine, n_all, bytes_all = workload_selection(rank, world, n_modules, total_bytes, seed)
    return corpus.config1(seed=seed, n_modules=n_all, total_bytes=bytes_all, indices=mine)


def make_workload_into(alloc, rank, world, n_modules, total_bytes, seed=1001):
    """The same, generated back to back straight into one host buffer: `alloc(nbytes)` returns a writable uint8 numpy
    array (pinned memory for the GPU arm).  Returns (array, [(address, length)] per module)."""
    from zluda_b200 import corpus
    mine, n_all, bytes_all = workload_selection(rank, world, n_modules, total_bytes, seed)
    blob = alloc(corpus.config1_total_bound(seed, n_all, bytes_all, mine))
    spans = corpus.config1_into(blob, seed, n_all, bytes_all, mine)
    base = blob.ctypes.data
    return blob, [(base + o, l) for o, l in spans]


def cpu_parse_all_cores(mods, seconds_budget=20.0):
    """Oracle (CPU restatement of ptx_parser) over `mods` ((address, length) pairs) with one thread per core; returns
    (GB/s, cores, bytes, modules)."""
    sys.path.insert(0, os.path.join(ROOT, "tests"))
    import oracle_lib
    o = oracle_lib.load()
    cores = os.cpu_count() or 1
    # calibrate on a few modules, then size the sample to the time budget
    t0 = time.perf_counter()
    nb = 0
    for m in mods[:4]:
        o.lib.oracle_parse_only(m[0], m[1], None, None)
        nb += m[1]
    rate1 = nb / max(1e-6, time.perf_counter() - t0)
    budget_bytes = rate1 * cores * seconds_budget * 0.6
    sample, total = [], 0
    for m in mods:
        if total > budget_bytes and len(sample) >= cores:
            break
        sample.append(m)
        total += m[1]
    idx = [0]
    lock = threading.Lock()
    bad = [0]

    def worker():
        while True:
            with lock:
                i = idx[0]
                idx[0] += 1
            if i >= len(sample):
                return
            if o.lib.oracle_parse_only(sample[i][0], sample[i][1], None, None) != 0:
                bad[0] += 1

    t0 = time.perf_counter()
    threads = [threading.Thread(target=worker) for _ in range(cores)]
    for t in threads:
        t.start()
    for t in threads:
        t.join()
    dt = time.perf_counter() - t0
    assert bad[0] == 0, "the oracle rejected a generated module"
    return total / dt / 1e9, cores, total, len(sample)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=5)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--modules", type=int, default=4096)
    ap.add_argument("--bytes", type=int, default=1 << 30)
    ap.add_argument("--kernels-only", action="store_true",
                    help="small profiling runs: skip the end-to-end and CPU legs and print only the per-step kernel times")
    a = ap.parse_args()
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    workload = "fatbin-scale batch: %d modules/GPU, ~%.2f GiB/GPU, config-0 grammar + 10%% mma/ld.shared.v4 tiles" % (
        a.modules, a.bytes / 2**30)
    config = {"workload": workload, "modules_per_gpu": a.modules, "parallelism": "modules sharded by byte-balanced greedy partition, no collective",
              "l2": ("inputs (%.0f MiB/GPU) larger than the 126 MB L2" if a.bytes > 126e6 else
                     "inputs (%.0f MiB/GPU) fit the 126 MB L2: a profiling or smoke size, not a timing configuration") % (a.bytes / 2**20)}

    if a.impl == "reference":
        if rank != 0:
            return
        blob, mods = make_workload_into(lambda n: np.empty(n, dtype=np.uint8), 0, 1, a.modules, a.bytes)
        vals = []
        for _ in range(a.warmup + a.steps):
            gbs, cores, nbytes, nmods = cpu_parse_all_cores(mods, seconds_budget=max(4.0, 60.0 / (a.warmup + a.steps)))
            vals.append(gbs)
        v = float(np.mean(vals[a.warmup:]))
        sample = "%d modules (%.1f MB) of the workload per step" % (nmods, nbytes / 1e6)
        print(json.dumps({
            "metric": METRIC, "value": v, "unit": UNIT, "n_gpus": a.gpus, "steps": a.steps, "warmup": a.warmup,
            "ms_per_step": nbytes / 1e9 / v * 1e3, "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "u8",
            "data": "synthetic", "impl": "reference", "config": config,
            "cpu_baseline": {"value": v, "unit": UNIT, "cores": cores, "kind": "port", "sample": sample},
            "e2e": {"value": v, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
            "note": "CPU restatement of ptx_parser (oracle/), one module per task over all host cores; the Rust crate cannot be built here"}))
        return

    import torch
    import torch.distributed as dist
    import zluda_b200
    torch.cuda.set_device(local_rank)
    if world > 1:
        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))
    os.environ.setdefault("PTXFE_PROFILE", "1")
    # the text is generated straight into pinned host memory: the e2e leg reads it from there
    pinned = []

    def alloc_pinned(n):
        pinned.append(torch.empty(n, dtype=torch.uint8).pin_memory())
        return pinned[-1].numpy()

    blob, mods = make_workload_into(alloc_pinned, rank, world, a.modules, a.bytes)
    nbytes = sum(l for _, l in mods)
    ctx = zluda_b200.Context(local_rank)
    spans = zluda_b200.Texts(mods)       # the (char**, uint64*) arrays of the C call, built once

    def barrier():
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    # ---- kernels only, text resident in HBM
    ctx.stage(spans)
    for _ in range(a.warmup):
        ctx.run()
    sampler = ClockSampler(local_rank)
    sampler.start()
    barrier()
    kernel_ms, prof = 0.0, {}
    t_wall = time.perf_counter()
    for _ in range(a.steps):
        ctx.run()
        st = ctx.stats()
        kernel_ms += st["kernel_ms"]
        for k, v in ctx.profile().items():
            prof[k] = prof.get(k, 0.0) + v
    barrier()
    wall_ms = (time.perf_counter() - t_wall) * 1e3
    stats = ctx.stats()
    if a.kernels_only:
        sampler.stop_flag = True
        sampler.join()
        print(json.dumps({"kernels_only": True, "text_bytes": nbytes, "steps": a.steps, "ms_per_step": kernel_ms / a.steps,
                          "kernels_ms": {k: v / a.steps for k, v in sorted(prof.items(), key=lambda kv: -kv[1])},
                          "gpu_launches": int(stats["n_kernel_launches"]) * a.steps,
                          "step_order": [n for n, _ in ctx.profile_steps()]}))
        return
    # ---- end to end through the public call: pinned host text in, records out.  A second context without the
    # per-step event pairs of the profiling mode (two extra API calls per launch on the host thread that drives the GPU)
    ctx.close()
    os.environ["PTXFE_PROFILE"] = "0"
    ctx = zluda_b200.Context(local_rank)
    for _ in range(max(2, a.warmup)):
        ctx.parse_batch(spans).free()
    barrier()
    t0 = time.perf_counter()
    for step in range(a.steps):
        b = ctx.parse_batch(spans)
        nerr = b.error_count(0)
        if step + 1 < a.steps:
            b.free()
    barrier()
    e2e_ms = (time.perf_counter() - t0) * 1e3
    e2e_stats = ctx.stats()
    sampler.stop_flag = True
    sampler.join()
    # ---- outside the timed region: what the last timed call returned, against the oracle, on every 16th module
    sys.path.insert(0, os.path.join(ROOT, "tests"))
    import oracle_lib
    from concurrent.futures import ThreadPoolExecutor
    # the materialiser: every module's records -> tree (module, functions, statements, operands; names as slices of the
    # text) on all host cores, built and dropped as the CPU arm builds and drops its tree
    t_mat = time.perf_counter()
    n_nodes = b.materialize()
    materialize_ms = (time.perf_counter() - t_mat) * 1e3
    check = list(range(0, len(mods), 16))
    t_par = time.perf_counter()
    with ThreadPoolExecutor(min(32, os.cpu_count() or 1)) as ex:
        ours = list(ex.map(b.dump_hash, check))
    theirs = oracle_lib.load().dump_hashes([mods[i] for i in check])
    n_errors = sum(b.error_count(i) for i in range(len(mods)))
    b.free()
    parity_bad = [i for i, x, y in zip(check, ours, theirs) if x != y]
    parity_s = time.perf_counter() - t_par
    if parity_bad:
        raise SystemExit("bench: parity FAILED: the dumps of modules %s of the timed batch differ from the oracle's" % parity_bad[:8])

    times = torch.tensor([kernel_ms, e2e_ms, float(nbytes), float(e2e_stats["h2d_bytes"]), float(e2e_stats["d2h_bytes"]), float(len(check)),
                          materialize_ms],
                         dtype=torch.float64, device="cuda")
    if world > 1:
        tmax = times.clone()
        dist.all_reduce(tmax, op=dist.ReduceOp.MAX)
        tsum = times.clone()
        dist.all_reduce(tsum, op=dist.ReduceOp.SUM)
        kernel_ms, e2e_ms, total_bytes = float(tmax[0]), float(tmax[1]), float(tsum[2])
        h2d_bytes, d2h_bytes = int(tsum[3]), int(tsum[4])      # whole job: all ranks
        n_checked = int(tsum[5])                               # a rank whose check failed has left with an error
        materialize_ms = float(tmax[6])
    else:
        n_checked = len(check)
        total_bytes = float(nbytes)
        h2d_bytes, d2h_bytes = int(e2e_stats["h2d_bytes"]), int(e2e_stats["d2h_bytes"])
    if rank != 0:
        if world > 1:
            dist.destroy_process_group()
        return
    value = total_bytes * a.steps / (kernel_ms / 1e3) / 1e9
    e2e = total_bytes * a.steps / (e2e_ms / 1e3) / 1e9
    # ---- roofline of the dominant kernel
    peak, peak_kind = measured_hbm_peak()
    T, W, N = stats["n_tokens"], stats["n_result_words"], nbytes
    U = stats["n_units"]
    algo = {   # algorithmic bytes per launch: text read once, tokens / records read or written once
        "lex_context_vectors": N, "lex_mark": N + N // 4, "lex_emit": N + N // 4 + 10 * T,
        "structure": 2 * T + 8 * U,
        "unit_shape_key": 2 * T + 10 * U, "apply_templates": 2 * T + 16 * U, "class_insert": 12 * U,
        "emit_records": 4 * W + 9 * U, "decode_units": N + 8 * T + 4 * W, "decode_emit_flagged": 5 * U,
    }
    top = max(prof, key=prof.get) if prof else None
    roof = None
    if top:
        ms = prof[top] / a.steps
        ab = algo.get(top)
        ach = ab / (ms / 1e3) / 1e9 if ab else None
        # DRAM traffic per launch: dram__bytes_read.sum + dram__bytes_write.sum of one ncu capture of the same kernel on a
        # 512 MiB instance of this workload (profiles/), scaled by text bytes (traffic grows in proportion to the text)
        tpb = NCU_DRAM_BYTES_PER_TEXT_BYTE.get(top)
        roof = {"kernel": top, "bound": "hbm", "achieved": ach, "peak": peak, "peak_kind": peak_kind, "unit": "GB/s",
                "frac": ach / peak if ach else None, "traffic": tpb * N if tpb else None, "ms_per_launch": ms, "algorithmic_bytes": ab,
                "lexer_segmenter": None}
        lex_ms = sum(prof.get(k, 0.0) for k in ("lex_context_vectors", "scan_context", "lex_tile_modules", "lex_mark", "lex_serial_modules",
                                                  "scan_token_counts", "set_token_total", "lex_emit", "module_token_ranges",
                                                  "module_results_init", "mark_module_skip", "structure", "reset_unit_total",
                                                  "module_unit_ranges", "module_unit_ranges_fill")) / a.steps
        # whole front end: text read once, records written once (N + O) over the kernel time of a step
        a_fe = N + 4 * W
        fe_ms = kernel_ms / a.steps
        roof["front_end"] = {"ms": fe_ms, "algorithmic_bytes": a_fe, "achieved": a_fe / (fe_ms / 1e3) / 1e9,
                             "frac": a_fe / (fe_ms / 1e3) / 1e9 / peak}
        roof["frac_of_nominal_8000"] = ach / 8000.0 if ach else None
        if lex_ms > 0:
            a_lex = N + 8 * T
            roof["lexer_segmenter"] = {"ms": lex_ms, "algorithmic_bytes": a_lex, "achieved": a_lex / (lex_ms / 1e3) / 1e9,
                                       "frac": a_lex / (lex_ms / 1e3) / 1e9 / peak}
    cpu_gbs, cores, cpu_bytes, cpu_mods = cpu_parse_all_cores(mods, seconds_budget=15.0)
    line = {
        "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": a.gpus, "steps": a.steps, "warmup": a.warmup,
        "ms_per_step": kernel_ms / a.steps, "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "u8",
        "data": "synthetic", "config": config,
        "e2e": {"value": e2e, "unit": UNIT, "ms_per_step": e2e_ms / a.steps, "h2d_bytes_per_step": h2d_bytes,
                "d2h_bytes_per_step": d2h_bytes, "h2d_ms": e2e_stats["h2d_ms"], "kernel_ms": e2e_stats["kernel_ms"],
                "d2h_ms": e2e_stats["d2h_ms"],
                # the same with every module materialised into a tree on the host cores afterwards (one batch, not overlapped)
                "materialize_ms": materialize_ms, "materialize_nodes": int(n_nodes), "materialize_threads": os.cpu_count(),
                "value_with_materialize": total_bytes / ((e2e_ms / a.steps + materialize_ms) / 1e3) / 1e9},
        "gpu_launches": int(stats["n_kernel_launches"]) * a.steps,
        "roofline": roof,
        "cpu_baseline": {"value": cpu_gbs, "unit": UNIT, "cores": cores, "kind": "port",
                         "sample": "%d modules (%.1f MB) of the same workload" % (cpu_mods, cpu_bytes / 1e6)},
        "clocks": sampler.summary(),
        "stages_ms": {"lex": stats["lex_ms"], "structure": stats["structure_ms"], "decode": stats["decode_ms"]},
        "kernels_ms": {k: v / a.steps for k, v in sorted(prof.items(), key=lambda kv: -kv[1])},
        "parity_checked": n_checked, "parity_ok": True, "parity_seconds": parity_s,
        "counts": {"text_bytes": nbytes, "tokens": int(T), "units": int(stats["n_units"]), "result_words": int(W),
                   "sequential_modules": int(e2e_stats["n_sequential"]), "errors_all_modules": int(n_errors),
                   "classes": int(e2e_stats["n_classes"]), "class_capacity": int(e2e_stats["n_class_capacity"]),
                   "units_templated": int(e2e_stats["n_units"] - e2e_stats["n_untemplated"]),
                   "units_decoded_one_by_one": int(e2e_stats["n_untemplated"]),
                   "signature_words": int(e2e_stats["n_signature_words"]), "signature_capacity": int(e2e_stats["n_signature_capacity"]),
                   "classes_resident_run": int(stats["n_classes"]), "units_decoded_one_by_one_resident_run": int(stats["n_untemplated"])},
        "wall_ms_kernel_loop": wall_ms,
    }
    print(json.dumps(line))
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
