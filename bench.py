"""Benchmark of the paged decode-attention hot path.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--workload NAME]

Workload (default `dense_fp16_b16_16k`): Qwen2.5-1.5B attention shape — 12 query
/ 2 KV heads, head_dim 128, page 16 — batch 16, every sequence at 16 384 tokens
of context, 28 layers each with its own K/V pools of ceil(1.2 x needed) blocks
and one shuffled block table; synthetic N(0,1) fp16 values. A STEP is one decode
step's attention: the 28 layer calls (one launch each: split-KV + merge), i.e. one
pass over 7.5 GB of KV, far more than the 126 MB L2, so nothing is flushed
between steps.

One JSON line comes out:
  value      KV bytes the step must read / step time, GB/s, steps replayed from
             one CUDA graph with everything resident in HBM (all ranks summed).
  e2e        the same metric through the public Python API with HOST buffers:
             each step copies the queries and the new K/V rows of all layers
             from pinned host memory, runs cache.write() and
             paged_decode_attention() per layer, eagerly, reads the outputs
             back to the host, and runs cache.advance() for the next step
             (block tables, lengths and slots shipped to the device) while the
             GPU is still working on this one.
  roofline   the decode kernel alone: CUDA events around replays of a graph of its launches.
  cpu_baseline  the numpy oracle on the host cores, one layer call.
`--impl reference` times that CPU oracle instead (rank 0 only).

With N > 1 (launched by torchrun, one rank per GPU) every rank runs the same
workload on its own GPU — sequences shard across GPUs with no exchange step —
and the time is the max over ranks; `torch.distributed` is used for that
barrier and max only.
"""

from __future__ import annotations

import argparse
import json
import os
import pathlib
import statistics
import subprocess
import sys
import threading
import time

ROOT = pathlib.Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))

WORKLOADS = {
    # name: (batch, context, layers); the first is the benchmark, the rest exist for
    # profiler captures and for the other kernels of the path.
    "dense_fp16_b16_16k": (16, 16384, 28),
    "dense_fp16_b16_4k": (16, 4096, 8),        # small cases for profiler captures
    "dense_fp16_b16_8k": (16, 8192, 8),
    "int8_b32_8k": (32, 8192, 8),
    "dense_fp16_b64_ragged": (64, "loguniform_1k_32k", 8),
    "int8_b32_8k_32k": (32, "uniform_8k_32k", 8),
    "int8_b16_4k": (16, 4096, 8),              # small case for profiler captures
    "sparse50_b8_32k": (8, 32768, 8),
    "sparse50_b8_8k": (8, 8192, 8),            # small case for profiler captures
    "sparse25_b8_32k": (8, 32768, 8),          # the same batch at a 25 % / 12.5 % page budget
    "sparse12_b8_32k": (8, 32768, 8),
}
# Whole decode steps of a random-init Qwen2.5-1.5B-shaped model (28 layers) over the
# paged caches: name -> (batch, context, kv cache kind, sparse ratio, shared prefix)
STEP_WORKLOADS = {
    "qwen_step_b16_16k": (16, 16384, "fp16", None, 0),
    "qwen_step_b16_16k_int8": (16, 16384, "int8", None, 0),
    "qwen_step_b16_16k_sparse50": (16, 16384, "fp16", 0.5, 0),
    "qwen_step_b16_16k_int8_sparse50": (16, 16384, "int8", 0.5, 0),
    "qwen_step_b64_ragged": (64, "loguniform_1k_32k", "fp16", None, 4096),
    "qwen_step_b64_ragged_int8": (64, "loguniform_1k_32k", "int8", None, 4096),
}
METRIC = "paged decode-attn HBM GB/s"
FALLBACK_HBM_GBS = 6650.0
# DRAM bytes per launch of the split-KV kernel on the default workload, from the
# Nsight Compute capture summarised under profiles/ (null until captured).
NCU_TRAFFIC_BYTES = 273_000_000     # 134 MB capture: 134.42 MB read + 3.66 MB written, scaled by pages


def measured_peak():
    path = ROOT / "MEASURED_PEAKS.json"
    if path.exists():
        try:
            return float(json.loads(path.read_text())["hbm_gbs"]), "measured"
        except Exception:
            pass
    return FALLBACK_HBM_GBS, "fallback"


class ClockSampler:
    """nvidia-smi clocks and throttle reasons, every 100 ms, while it runs."""

    FIELDS = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,"
              "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
              "clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int):
        self.rows, self.proc, self.thread = [], None, None
        self.index = index

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--id={self.index}", f"--query-gpu={self.FIELDS}",
                 "--format=csv,noheader,nounits", "-lms", "100"],
                stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
        except OSError:
            return
        self.thread = threading.Thread(target=self._read, daemon=True)
        self.thread.start()

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append((time.time(), [x.strip() for x in line.split(",")]))

    def stop(self):
        if self.proc is not None:
            self.proc.terminate()
            try:
                self.proc.wait(timeout=2)
            except subprocess.TimeoutExpired:
                self.proc.kill()

    def summary(self, t0: float, t1: float) -> dict:
        rows = [r for t, r in self.rows if t0 <= t <= t1 and len(r) >= 6] or \
               [r for _, r in self.rows if len(r) >= 6]
        if not rows:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": [], "samples": 0}
        names = ("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap")
        reasons = [n for i, n in enumerate(names) if any(r[2 + i].lower() == "active" for r in rows)]
        mhz = [float(r[0]) for r in rows if r[0].replace(".", "").isdigit()]
        mx = [float(r[1]) for r in rows if r[1].replace(".", "").isdigit()]
        return {"sm_mhz": statistics.median(mhz) if mhz else None,
                "sm_max_mhz": max(mx) if mx else None, "reasons": reasons, "samples": len(rows)}


def cpu_oracle_layer(q, k_pool, v_pool, tables, lens, repeats=1):
    """One layer call on the host cores (torch CPU ops, every thread) with the
    oracle's gather-then-softmax restatement; numpy arrays in, seconds out."""
    import torch

    from oracle import paged_attention_oracle as orc

    args = [torch.from_numpy(x) for x in (q, k_pool, v_pool, tables, lens)]
    best = float("inf")
    for _ in range(repeats):
        t0 = time.perf_counter()
        orc.paged_decode_torch_cpu(*args)
        best = min(best, time.perf_counter() - t0)
    return best


def host_threads() -> int:
    """Threads of the CPU legs: every CPU this process may run on. Set explicitly,
    because torchrun exports OMP_NUM_THREADS=1 to its workers and only rank 0 runs
    the CPU leg (LS_CPU_THREADS overrides)."""
    import torch

    want = int(os.environ.get("LS_CPU_THREADS", "0"))
    if want <= 0:
        try:
            want = len(os.sched_getaffinity(0))
        except AttributeError:
            want = os.cpu_count() or 1
    if torch.get_num_threads() != want:
        torch.set_num_threads(want)
    return torch.get_num_threads()


def run_reference(args, workload):
    """The CPU restatement of the reference's torch path, on the host cores.
    Each step is a bounded sample of the workload: one layer call over
    `sample_seqs` sequences at the workload's context."""
    import numpy as np

    from latentserve_b200 import synthetic

    batch, context, layers = workload
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    sample_seqs = 4
    cores = host_threads()
    case = synthetic.dense_case([context] * sample_seqs, seed=0, spare=0)
    nbytes = synthetic.kv_bytes_fp16([context] * sample_seqs)
    for _ in range(max(1, min(args.warmup, 2))):
        cpu_oracle_layer(case["q"], case["k_pool"], case["v_pool"], case["block_tables"], case["seq_lens"])
    t0 = time.perf_counter()
    for _ in range(args.steps):
        cpu_oracle_layer(case["q"], case["k_pool"], case["v_pool"], case["block_tables"], case["seq_lens"])
    dt = (time.perf_counter() - t0) / args.steps
    value = nbytes / dt / 1e9
    sample = (f"one layer call over {sample_seqs} of the workload's {batch} sequences at context "
              f"{context} ({nbytes / 1e6:.0f} MB of KV) per step, torch CPU fp32 gather-then-softmax")
    print(json.dumps({
        "impl": "reference", "metric": METRIC, "value": round(value, 3), "unit": "GB/s",
        "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": round(dt * 1e3, 3), "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": args.workload, "batch": batch, "context": context, "layers": layers,
                   "note": "CPU path, bounded sample per step"},
        "cpu_baseline": {"value": round(value, 3), "unit": "GB/s", "cores": cores, "kind": "port",
                         "sample": sample},
        "e2e": {"value": round(value, 3), "unit": "GB/s", "h2d_bytes_per_step": 0,
                "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }))


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=200)
    ap.add_argument("--warmup", type=int, default=10)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="dense_fp16_b16_16k",
                    choices=sorted(WORKLOADS) + sorted(STEP_WORKLOADS))
    ap.add_argument("--kernel", default="mma", choices=["mma", "simt"],
                    help="split-KV kernel variant (simt = CUDA-core kernel, for profiling)")
    ap.add_argument("--no-e2e", action="store_true", help="skip the host-buffer leg")
    ap.add_argument("--no-cpu", action="store_true", help="skip the CPU baseline leg")
    ap.add_argument("--no-pdl", action="store_true",
                    help="ordinary launches instead of programmatic dependent launch")
    ap.add_argument("--loader", default=None, choices=["auto", "tma", "cp_async"],
                    help="page loader of the decode kernels (default: auto = TMA for INT8 and cp.async for "
                         "fp16 in the attention workloads; tma in the whole-step workloads, where it "
                         "measured 1.7 %% faster)")
    ap.add_argument("--no-early", action="store_true",
                    help="with programmatic launch: do not request old pages ahead of the dependency wait")
    ap.add_argument("--projections", default="auto", choices=["auto", "ls", "cublas"],
                    help="decode-step workloads: this library's weight-streaming projections, torch GEMMs, "
                         "or (auto) the former up to 16 rows")
    ap.add_argument("--quick", action="store_true",
                    help="profiler runs: no e2e / CPU legs, no extension of the load for clock sampling")
    args = ap.parse_args()
    if args.workload in STEP_WORKLOADS:
        run_model_step(args)
        return
    workload = WORKLOADS[args.workload]
    if args.quick:
        args.no_e2e = args.no_cpu = True
    if args.impl == "reference":
        run_reference(args, workload)
        return

    import numpy as np
    import torch

    from latentserve_b200 import _lib, cache as lc, paged_decode as pd, paged_decode_cuda as pdc
    from latentserve_b200 import synthetic

    if not torch.cuda.is_available():
        raise SystemExit("bench.py measures the CUDA path and there is no CUDA device")
    _lib.lib()                                    # fail here, loudly, if the library is missing
    pdc.set_programmatic_launch(not args.no_pdl, early_pages=not args.no_early)
    pdc.set_loader(args.loader or "auto")
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    dev = torch.device("cuda", local)
    torch.cuda.set_device(dev)
    dist = None
    if world > 1:
        import torch.distributed as dist
        dist.init_process_group("nccl", device_id=dev)

    batch, context, layers = workload
    impl = pdc.IMPL_SIMT if args.kernel == "simt" else pdc.IMPL_MMA
    rng = np.random.default_rng(1234 + rank)
    if context == "loguniform_1k_32k":
        seq_lens = np.exp(rng.uniform(np.log(1024), np.log(32768), size=batch)).astype(int).tolist()
    elif context == "uniform_8k_32k":
        seq_lens = rng.integers(8192, 32769, size=batch).tolist()
    else:
        seq_lens = [context] * batch
    kind = args.workload.split("_")[0]
    if kind == "int8":
        w = synthetic.int8_pools_on_device(seq_lens, layers, dev, seed=rank)
        tables, lens = w["block_tables"], w["seq_lens"]
        step_bytes = synthetic.kv_bytes_int8(seq_lens) * layers

        def layer_call(i, merge=True):
            L = w["layers"][i]
            return pdc.paged_decode_cuda(w["q"][i], L["k_pool"], L["v_pool"], tables, lens, max(seq_lens),
                                         k_scale=L["k_scale"], v_scale=L["v_scale"],
                                         k_residual=L["k_residual"], res_rows=w["res_rows"], merge=merge)
        launches_per_layer, kernel_name = 1, "decode_kernel<int8>"
    elif kind.startswith("sparse"):
        from latentserve_b200 import paged_sparse as ps

        w = synthetic.sparse_pools_on_device(batch, context, layers, dev, seed=rank)
        tables, lens = w["block_tables"], w["seq_lens"]
        pages = -(-context // 16)
        sparse_ratio = {"50": 0.5, "25": 0.25, "12": 0.125}[kind[len("sparse"):len("sparse") + 2]]
        keep = ps.budget(sparse_ratio, pages)
        # indexer reads kmin+kmax of every page-head, writes and re-reads the scores,
        # attention reads the selected pages
        layer_bytes = batch * 2 * (pages * 512 + pages * 8 + keep * 16 * 512)
        step_bytes = layer_bytes * layers

        def layer_call(i, merge=True):
            k, v = w["pools"][i]
            kmin, kmax = w["bounds"][i]
            return ps.sparse_attention(w["q"][i], k, v, tables, lens, kmin, kmax, ratio=sparse_ratio,
                                       max_seq_len=context)
        launches_per_layer, kernel_name = 3, "page_index + select_pages + decode_kernel<sparse>"
    else:
        w = synthetic.dense_pools_on_device(batch, seq_lens, layers, dev, seed=rank)
        tables, lens = w["block_tables"], w["seq_lens"]
        step_bytes = synthetic.kv_bytes_fp16(seq_lens) * layers

        def layer_call(i, merge=True):
            k, v = w["pools"][i]
            return pdc.paged_decode_cuda(w["q"][i], k, v, tables, lens, max(seq_lens), impl=impl,
                                         merge=merge)
        launches_per_layer = 1
        kernel_name = f"decode_kernel<{args.kernel}> (split-KV + in-kernel merge)"
    default_workload = args.workload == "dense_fp16_b16_16k"

    # One step = the 28 layer calls, captured once.
    side = torch.cuda.Stream()
    with torch.cuda.stream(side):
        for _ in range(3):
            for i in range(layers):
                layer_call(i)
    torch.cuda.synchronize()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        for i in range(layers):
            layer_call(i)

    def barrier():
        if dist is not None:
            dist.barrier()
        torch.cuda.synchronize()

    sampler = ClockSampler(torch.cuda.current_device() if "CUDA_VISIBLE_DEVICES" not in os.environ
                           else int(os.environ["CUDA_VISIBLE_DEVICES"].split(",")[local]))
    sampler.start()
    for _ in range(max(3, args.warmup)):
        graph.replay()
    barrier()
    t_wall0 = time.time()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(args.steps):
        graph.replay()
    e1.record()
    barrier()
    ms_total = e0.elapsed_time(e1)
    # Keep the same load running briefly if the timed region was too short for
    # the 100 ms clock sampler to see it.
    extra_until = t_wall0 + (0.0 if args.quick else 1.2)
    while time.time() < extra_until:
        for _ in range(20):
            graph.replay()
        torch.cuda.synchronize()
    t_wall1 = time.time()
    if dist is not None:
        t = torch.tensor([ms_total], device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms_total = float(t.item())
    ms_step = ms_total / args.steps
    value = world * step_bytes / (ms_step * 1e-3) / 1e9

    # Roofline: the dominant kernel's average launch duration, timed with CUDA
    # events on the launching stream around replays of a graph that holds one
    # launch per layer (so neither Python nor launch latency is in it).
    def graph_us(fn, reps):
        for i in range(layers):
            fn(i)
        torch.cuda.synchronize()
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g):
            for i in range(layers):
                fn(i)
        for _ in range(3):
            g.replay()
        torch.cuda.synchronize()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        for _ in range(reps):
            g.replay()
        b.record()
        torch.cuda.synchronize()
        return a.elapsed_time(b) * 1e3 / (reps * layers)

    reps = max(3, min(50, args.steps))
    breakdown = None
    if kind.startswith("sparse"):
        pages_ = -(-context // 16)
        keep_ = ps.budget(sparse_ratio, pages_)
        sel_fixed = ps.select(ps.page_scores(w["q"][0], *w["bounds"][0], tables, lens), keep_).clone()
        scores_fixed = ps.page_scores(w["q"][0], *w["bounds"][0], tables, lens).clone()
        breakdown = {
            "page_index_us": round(graph_us(lambda i: ps.page_scores(w["q"][i], *w["bounds"][i], tables, lens), reps), 2),
            "select_pages_us": round(graph_us(lambda i: ps.select_for_attention(
                scores_fixed, lens, keep_, sparse_ratio), reps), 2),
            "topk_pages_us_not_on_the_path": round(graph_us(lambda i: ps.select(scores_fixed, keep_), reps), 2),
            "sparse_decode_us": round(graph_us(lambda i: ps.sparse_decode(
                w["q"][i], w["pools"][i][0], w["pools"][i][1], tables, lens, sel_fixed, ratio=sparse_ratio), reps), 2),
        }
        kernel_ms = breakdown["sparse_decode_us"] * 1e-3
        roof_bytes = batch * 2 * keep_ * 16 * 512
        kernel_name = "decode_kernel<sparse> (attention over the selected pages)"
    else:
        kernel_ms = graph_us(lambda i: layer_call(i), reps) * 1e-3
        roof_bytes = step_bytes // layers
    clocks = sampler.summary(t_wall0, t_wall1)
    peak, peak_kind = measured_peak()
    layer_bytes = roof_bytes
    achieved = layer_bytes / (kernel_ms * 1e-3) / 1e9
    roofline = {"bound": "hbm", "achieved": round(achieved, 1), "peak": peak, "unit": "GB/s",
                "frac": round(achieved / peak, 4),
                "traffic": NCU_TRAFFIC_BYTES if default_workload and args.kernel == "mma" else None,
                "peak_kind": f"of {peak_kind}", "kernel": kernel_name,
                "kernel_us": round(kernel_ms * 1e3, 2), "algorithmic_bytes_per_launch": layer_bytes,
                "frac_of_8TBs": round(achieved / 8000.0, 4), "breakdown": breakdown}

    # End to end through the public API with host buffers.
    e2e = None
    if not args.no_e2e and default_workload:
        e2e = run_e2e(args, workload, dev, dist, world)

    cpu = None
    if rank == 0 and world == 1 and not args.no_cpu and default_workload:
        k, v = w["pools"][0]
        blocks = tables.long()
        seqs = min(batch, 4)
        # The sample's blocks, renumbered into a compact pool on the host.
        kb = k[blocks[:seqs].reshape(-1)].cpu().numpy()
        vb = v[blocks[:seqs].reshape(-1)].cpu().numpy()
        tb = np.arange(kb.shape[0], dtype=np.int32).reshape(seqs, -1)
        cpu_cores = host_threads()
        secs = cpu_oracle_layer(w["q"][0][:seqs].cpu().numpy(), kb, vb, tb,
                                lens[:seqs].cpu().numpy(), repeats=3)
        nbytes = synthetic.kv_bytes_fp16([context] * seqs)
        cpu = {"value": round(nbytes / secs / 1e9, 3), "unit": "GB/s", "cores": cpu_cores,
               "kind": "port",
               "sample": f"one layer call over {seqs} of the {batch} sequences "
                         f"({nbytes / 1e6:.0f} MB of KV), torch CPU fp32 gather-then-softmax, best of 3"}
    # The reference's own CUDA kernel (its .cu compiled as it is for sm_100a into oracle/_ref,
    # driven as its host code drives it) on this GPU and this workload, beside ours. Part of
    # the baseline leg; absent when the cubin was not built.
    ref_kernel = None
    if rank == 0 and world == 1 and not args.no_cpu and kind in ("dense", "int8"):
        ref_kernel = time_reference_kernel(kind, w, tables, lens, seq_lens, layers, step_bytes, graph_us)
    sampler.stop()

    if rank == 0:
        line = {
            "metric": METRIC, "value": round(value, 1), "unit": "GB/s", "n_gpus": world,
            "steps": args.steps, "warmup": max(3, args.warmup), "ms_per_step": round(ms_step, 4),
            "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
            "dtype": "i8" if kind == "int8" else "f16", "data": "synthetic",
            "config": {"workload": args.workload, "batch_per_gpu": batch,
                       "context": context if isinstance(context, int) else
                       f"{context}: min {min(seq_lens)}, mean {int(np.mean(seq_lens))}, max {max(seq_lens)}",
                       "layers_per_step": layers, "q_heads": 12, "kv_heads": 2, "head_dim": 128,
                       "page": 16, "pool_blocks": w["num_blocks"], "kernel": args.kernel,
                       "programmatic_launch": not args.no_pdl,
                       "early_pages": not (args.no_pdl or args.no_early), "loader": args.loader or "auto",
                       "parallelism": f"replicas x{world} (sequence-sharded, no collective)",
                       "l2": f"no flush: each step reads {step_bytes / 1e9:.2f} GB, L2 is 126 MB",
                       "step": f"{layers} layer calls ({launches_per_layer} launch(es) each) replayed from one "
                               "CUDA graph"},
            "pct_of_8TBs": round(100.0 * value / world / 8000.0, 2),
            "us_per_layer_call": round(1e3 * ms_step / layers, 2),
            "roofline": roofline, "cpu_baseline": cpu, "reference_kernel": ref_kernel, "e2e": e2e,
            "gpu_launches": launches_per_layer * layers * args.steps, "clocks": clocks,
        }
        print(json.dumps(line))
    if dist is not None:
        dist.barrier()
        dist.destroy_process_group()


def run_model_step(args):
    """Whole decode steps (all 28 layers: GEMMs, norms, RoPE, append, attention,
    output head, greedy argmax) replayed from one CUDA graph. Reports ms per step
    (graph replay only, and the full loop with cache.advance() on the host) and
    tokens per second; with N ranks every rank serves its own sequences."""
    import random

    import numpy as np
    import torch

    from latentserve_b200 import _lib, cache as lc, decode_step as ds, paged_decode_cuda as pdc

    _lib.lib()
    pdc.set_programmatic_launch(not args.no_pdl, early_pages=not args.no_early)
    pdc.set_loader(args.loader or "tma")
    batch, context, kind, ratio, prefix = STEP_WORKLOADS[args.workload]
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    dev = torch.device("cuda", local)
    torch.cuda.set_device(dev)
    dist = None
    if world > 1:
        import torch.distributed as dist
        dist.init_process_group("nccl", device_id=dev)
    rng = np.random.default_rng(1234 + rank)
    if context == "loguniform_1k_32k":
        lens = np.exp(rng.uniform(np.log(1024), np.log(32768), size=batch)).astype(int).tolist()
    else:
        lens = [context] * batch
    steps, warm = args.steps, max(3, args.warmup)
    shape = ds.QwenShape()
    room = steps + warm + 8
    spec = lc.KVCacheSpec(num_layers=shape.num_layers, num_kv_heads=shape.kv_heads,
                          head_dim=shape.head_dim, max_seq_len=max(lens) + room + 16,
                          max_batch_size=batch, device=str(dev))
    blocks = int(1.2 * sum(-(-(n + room) // 16) for n in lens)) + 64
    cache = (lc.Int8PagedKVCache if kind == "int8" else lc.PagedKVCache)(spec, num_blocks=blocks)
    g = torch.Generator(device=dev).manual_seed(rank)
    if kind == "int8" and ratio is not None:       # the INT8 cache keeps bounds from its first write on
        cache.enable_page_bounds()
        for layer in range(shape.num_layers):      # synthetic history: plausible bounds everywhere
            cache.kmin[layer].normal_(generator=g).sub_(1.5)
            cache.kmax[layer].normal_(generator=g).abs_().add_(cache.kmin[layer])
    for layer in range(shape.num_layers):          # synthetic history: random K/V everywhere
        if kind == "int8":
            cache.k_pool[layer].random_(-127, 128, generator=g)
            cache.v_pool[layer].random_(-127, 128, generator=g)
            cache.k_scale_pool[layer].uniform_(0.01, 0.03, generator=g)
            cache.v_scale_pool[layer].uniform_(0.01, 0.03, generator=g)
        else:
            cache.k_pool[layer].normal_(generator=g)
            cache.v_pool[layer].normal_(generator=g)
    random.Random(rank).shuffle(cache.allocator._free)
    shared, owners = [], []
    if prefix:                                     # a quarter of the batch shares one ref-counted prefix
        owners = [i for i in range(batch) if lens[i] > prefix][: max(1, batch // 4)]
        if owners:
            cache.tables[owners[0]].append(prefix)
            shared = cache.tables[owners[0]].blocks[: prefix // 16]
            for i in owners[1:]:
                cache.attach_prefix(i, shared, prefix)
            if kind == "int8":
                cache._fin[owners[0]] = prefix // 16
    for i, n in enumerate(lens):
        have = cache.tables[i].length
        cache.tables[i].append(n - 1 - have)
        if kind == "int8":
            cache._fin[i] = (n - 1) // 16
    if ratio is not None and kind != "int8":
        cache.enable_page_bounds()
    model = ds.DecodeModel(shape, dev, max_pos=max(lens) + room + 16, seed=rank,
                           projections=args.projections)
    model.set_sparse(ratio)
    hint = max(lens) + room
    runner = ds.GraphedStep(model, cache, batch, hint)
    runner.tokens.random_(0, shape.vocab, generator=g)
    cache.advance(1, batch_size=batch)
    runner.positions.copy_(torch.tensor([n - 1 for n in cache.seq_lens], dtype=torch.long))
    runner.capture()
    for _ in range(warm):
        cache.advance(1, batch_size=batch)
        runner.step()
    if dist is not None:
        dist.barrier()
    torch.cuda.synchronize()
    sampler = ClockSampler(local)
    sampler.start()
    t_wall0 = time.time()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(steps):
        cache.advance(1, batch_size=batch)
        runner.step()
    e1.record()
    torch.cuda.synchronize()
    loop_ms = e0.elapsed_time(e1) / steps
    # Graph replay alone (lengths frozen), as the reference quotes its "graph-only" step.
    r0, r1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    reps = max(10, min(steps, 100))
    r0.record()
    for _ in range(reps):
        runner.graph.replay()
    r1.record()
    torch.cuda.synchronize()
    graph_ms = r0.elapsed_time(r1) / reps
    while time.time() < t_wall0 + 1.2:
        runner.graph.replay()
        torch.cuda.synchronize()
    clocks = sampler.summary(t_wall0, time.time())
    sampler.stop()
    if dist is not None:
        t = torch.tensor([loop_ms, graph_ms], device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        loop_ms, graph_ms = float(t[0]), float(t[1])
    mean_len = float(np.mean(lens)) + warm + steps / 2
    kv_per_tok = shape.num_layers * shape.kv_heads * (292 if kind == "int8" else 512)
    kv_bytes = mean_len * batch * kv_per_tok * (ratio if ratio else 1.0)
    floor_ms = (kv_bytes + model.weight_bytes()) / (measured_peak()[0] * 1e9) * 1e3
    if rank == 0:
        print(json.dumps({
            "metric": "Qwen2.5-1.5B decode step ms", "value": round(loop_ms, 4), "unit": "ms",
            "n_gpus": world, "steps": steps, "warmup": warm, "ms_per_step": round(loop_ms, 4),
            "higher_is_better": False, "scaling": "weak", "vs_baseline": None,
            "dtype": "i8" if kind == "int8" else "f16", "data": "synthetic",
            "config": {"workload": args.workload, "batch_per_gpu": batch,
                       "context": f"min {min(lens)}, mean {int(np.mean(lens))}, max {max(lens)}",
                       "kv_cache": kind, "sparse_ratio": ratio, "shared_prefix_tokens": prefix,
                       "sequences_sharing_prefix": len(owners),
                       "layers": shape.num_layers, "programmatic_launch": not args.no_pdl,
                       "projections": "ls" if model.streams_projections(batch) else "cublas",
                       "early_pages": not (args.no_pdl or args.no_early), "loader": args.loader or "tma",
                       "parallelism": f"replicas x{world} (sequence-sharded, no collective)"},
            "graph_replay_ms": round(graph_ms, 4),
            "tokens_per_s": round(world * batch / (loop_ms * 1e-3), 1),
            "hbm_floor_ms": round(floor_ms, 4),
            "frac_of_floor": round(floor_ms / graph_ms, 4), "clocks": clocks,
        }))
    if dist is not None:
        dist.barrier()
        dist.destroy_process_group()


def time_reference_kernel(kind, w, tables, lens, seq_lens, layers, step_bytes, graph_us):
    """us per layer call and GB/s of the reference's split-KV kernel (fills of its m / l
    scratch included, as on every call of its host code; its Triton merge not included)."""
    try:
        from oracle import ref_kernels
    except Exception:                                      # the oracle folder did not travel
        return None
    name = "paged_decode_int8" if kind == "int8" else "paged_decode_fp16"
    if not ref_kernels.available(name):
        return None
    runs = []
    for i in range(layers):
        if kind == "int8":
            L = w["layers"][i]
            runs.append(ref_kernels.RefDecode(w["q"][i], L["k_pool"], L["v_pool"], tables, lens,
                                              max(seq_lens), k_scale=L["k_scale"], v_scale=L["v_scale"],
                                              k_residual=L["k_residual"], res_rows=w["res_rows"]))
        else:
            k, v = w["pools"][i]
            runs.append(ref_kernels.RefDecode(w["q"][i], k, v, tables, lens, max(seq_lens)))
    us = graph_us(lambda i: runs[i].launch(), 3)
    layer_bytes = step_bytes / layers
    return {"value": round(layer_bytes / (us * 1e-6) / 1e9, 1), "unit": "GB/s", "us_per_layer_call": round(us, 2),
            "splits": runs[0].splits,
            "what": f"LatentServe kernels/cuda/{name}.cu compiled for sm_100a, grid (B, splits, H) x 1 warp, "
                    "m / l fills included, split merge not included"}


def run_e2e(args, workload, dev, dist, world):
    """Steps through PagedKVCache + paged_decode_attention with host buffers."""
    import torch

    from latentserve_b200 import cache as lc, paged_decode as pd, synthetic

    batch, context, layers = workload
    h, r, d = 2, 6, 128
    steps = max(3, min(args.steps, 30))
    warm = 3
    need = -(-(context + 2 * (steps + warm) + 6) // 16)      # eager pass, then the graph pass
    spec = lc.KVCacheSpec(num_layers=layers, num_kv_heads=h, head_dim=d,
                          max_seq_len=need * 16, max_batch_size=batch, device=str(dev))
    cache = lc.PagedKVCache(spec, num_blocks=int(1.2 * batch * need) + 1)
    g = torch.Generator(device=dev).manual_seed(1)
    for layer in range(layers):
        cache.k_pool[layer].normal_(generator=g)
        cache.v_pool[layer].normal_(generator=g)
    # Context already in the cache: grow the tables without writing (the pools
    # hold synthetic values everywhere).
    import random
    random.Random(0).shuffle(cache.allocator._free)      # shuffled block tables, as in `value`
    for i in range(batch):
        cache.tables[i].append(context - 1)
    host_q = torch.randn(layers, batch, h, r, d).half().pin_memory()
    host_k = torch.randn(layers, batch, h, 1, d).half().pin_memory()
    host_v = torch.randn(layers, batch, h, 1, d).half().pin_memory()
    host_out = torch.empty(layers, batch, h, r, d, dtype=torch.float16).pin_memory()
    dq, dk, dv = (torch.empty_like(x, device=dev) for x in (host_q, host_k, host_v))
    dout = torch.empty(layers, batch, h, r, d, dtype=torch.float16, device=dev)

    # Per-layer views made once, as a model's layers hold them.
    q_l, k_l, v_l, out_l = ([t[i] for i in range(layers)] for t in (dq, dk, dv, dout))
    host_s = [0.0]

    def layer_calls():
        tables, lens = cache.block_tables_tensor(batch), cache.seq_lens_tensor(batch)
        hint = cache.max_len
        for layer in range(layers):
            cache.write(layer, k_l[layer], v_l[layer])
            pd.paged_decode_attention(q_l[layer], cache.k_pool[layer], cache.v_pool[layer],
                                      tables, lens, max_seq_len=hint, out=out_l[layer])

    graph = [None]

    def step():
        # The cache has been advanced for this step already (by the previous step, below):
        # the host's bookkeeping for step t + 1 runs while the GPU works on step t, and its
        # one small copy is ordered behind step t's kernels on the stream.
        t0 = time.perf_counter()
        dq.copy_(host_q, non_blocking=True)
        dk.copy_(host_k, non_blocking=True)
        dv.copy_(host_v, non_blocking=True)
        if graph[0] is None:
            layer_calls()
        else:
            graph[0].replay()
        host_out.copy_(dout, non_blocking=True)
        cache.advance(1, batch_size=batch)               # next step's slots, lengths and tables
        host_s[0] += time.perf_counter() - t0            # host time to enqueue the step
        torch.cuda.current_stream().synchronize()        # the step's result is on the host

    def timed():
        for _ in range(warm):
            step()
        if dist is not None:
            dist.barrier()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        host_s[0] = 0.0
        e0.record()
        for _ in range(steps):
            step()
        e1.record()
        torch.cuda.synchronize()
        t_ms = e0.elapsed_time(e1)
        if dist is not None:
            t = torch.tensor([t_ms], device=dev)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            t_ms = float(t.item())
        return t_ms / steps, 1e3 * host_s[0] / steps

    cache.advance(1, batch_size=batch)                   # for the first step
    ms, host_ms = timed()
    mean_len = context + warm + (steps + 1) / 2
    # The same step with the 28 layer calls captured once and replayed, the way the
    # reference's serving loop drives this path (runtime/cuda_graph.py: static inputs,
    # advance() on the host, one replay per step). The cache is already advanced.
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        layer_calls()
    torch.cuda.current_stream().wait_stream(side)
    torch.cuda.synchronize()
    cg = torch.cuda.CUDAGraph()
    with torch.cuda.graph(cg):
        layer_calls()
    graph[0] = cg
    g_ms, g_host_ms = timed()
    g_mean_len = context + 2 * warm + steps + (steps + 1) / 2
    step_bytes = synthetic.kv_bytes_fp16([mean_len] * batch) * layers
    g_bytes = synthetic.kv_bytes_fp16([g_mean_len] * batch) * layers
    h2d = (host_q.numel() + host_k.numel() + host_v.numel()) * 2 + batch * (8 + 4)
    d2h = host_out.numel() * 2
    return {"value": round(world * step_bytes / (ms * 1e-3) / 1e9, 1), "unit": "GB/s",
            "h2d_bytes_per_step": int(h2d), "d2h_bytes_per_step": int(d2h),
            "ms_per_step": round(ms, 4), "host_enqueue_ms_per_step": round(host_ms, 4),
            "steps": steps, "gpu_launches_per_step": 2 * layers,
            "path": "PagedKVCache.write + paged_decode_attention per layer, eager; PagedKVCache.advance for "
                    "the next step issued while the GPU works on this one",
            "graph_replay": {"value": round(world * g_bytes / (g_ms * 1e-3) / 1e9, 1), "unit": "GB/s",
                             "ms_per_step": round(g_ms, 4),
                             "host_enqueue_ms_per_step": round(g_host_ms, 4),
                             "path": "same host buffers and copies; the 28 write + attention calls "
                                     "captured in one CUDA graph and replayed"}}


if __name__ == "__main__":
    main()
