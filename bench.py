"""Benchmark of the paged decode-attention hot path.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]
                    [--workload NAME [--only]]

Headline workload (`dense_fp16_b16_16k`): Qwen2.5-1.5B attention shape — 12 query
/ 2 KV heads, head_dim 128, page 16 — batch 16, every sequence at 16 384 tokens
of context, 28 layers each with its own K/V pools of ceil(1.2 x needed) blocks
and one shuffled block table; synthetic N(0,1) fp16 values. A STEP is one decode
step's attention: the 28 layer calls (one launch each: split-KV + merge), i.e. one
pass over 7.5 GB of KV, far more than the 126 MB L2, so nothing is flushed
between steps.

One JSON line comes out:
  value      KV bytes the step must read / step time, GB/s, steps replayed from
             one CUDA graph with everything resident in HBM (all ranks summed).
             Five blocks of exactly K steps are timed, each between a barrier and
             a synchronise, with a second of the same load between the first
             block and the others: `ms_per_step` is the median block, `blocks`
             lists them all with the SM clock sampled during each (the first is
             a burst figure, the later ones run under the power cap).
  e2e        the same metric through the public Python API with HOST buffers:
             each step copies the queries and the new K/V rows of all layers
             from pinned host memory (one copy), runs cache.write() and
             paged_decode_attention() per layer, eagerly (one launch per layer:
             the append rides on the attention kernel), reads the outputs
             back to the host, and runs cache.advance() for the next step
             (block tables, lengths and slots shipped to the device) while the
             GPU is still working on this one.
  roofline   the decode kernel: its launches are all the step's graph holds, so
             its average duration is the timed region / launches (gaps between
             launches count against the kernel).
  cpu_baseline  the oracle's torch-CPU restatement on the host cores, one layer call
             over a bounded sample.
  other_workloads  the other configurations of the path, each measured the same
             way with its own clock sample: the INT8 kernel on 32 ragged
             sequences of 8K-32K, the sparse pipeline at 8 x 32 768 and a 50 %
             budget (with this library's own dense kernel on the same batch),
             the whole decode step of a random-init Qwen2.5-1.5B shape at
             16 x 16 384 (the metric's "decode step ms"), and — at every N — the
             whole step on 64 ragged sequences per GPU with a shared prefix.
`--impl reference` times the CPU restatement instead (rank 0 only).
`--workload NAME` makes NAME the headline; with `--only` nothing but its
device-timed leg runs (for profiler captures on the small cases).

With N > 1 (launched by torchrun, one rank per GPU) every rank runs the same
workload on its own GPU — sequences shard across GPUs with no exchange step —
and the time is the max over ranks; `torch.distributed` is used for that
barrier and max only.
"""

from __future__ import annotations

import argparse
import gc
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
    # name: (batch, context, layers)
    "dense_fp16_b16_16k": (16, 16384, 28),
    "int8_b32_8k_32k": (32, "uniform_8k_32k", 8),
    "sparse50_b8_32k": (8, 32768, 8),
    "sparse25_b8_32k": (8, 32768, 8),          # the same batch at a 25 % / 12.5 % page budget
    "sparse12_b8_32k": (8, 32768, 8),
    "dense_fp16_b64_ragged": (64, "loguniform_1k_32k", 8),
    # small cases, for profiler captures (a few GB on the device, still past L2)
    "dense_fp16_b16_4k": (16, 4096, 8),
    "dense_fp16_b16_8k": (16, 8192, 8),
    "int8_b32_8k": (32, 8192, 8),
    "int8_b16_4k": (16, 4096, 8),
    "sparse50_b8_8k": (8, 8192, 8),
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
HEADLINE = "dense_fp16_b16_16k"
# What the default line carries besides the headline: (name, run at N > 1 too)
OTHER_WORKLOADS = (("int8_b32_8k_32k", False), ("sparse50_b8_32k", False), ("qwen_step_b16_16k", False),
                   ("qwen_step_b64_ragged", True))
BLOCKS = 5                                  # timed blocks of K steps per workload
SUSTAIN_S = 1.0                             # the same load, untimed, between block 1 and the others
METRIC = "paged decode-attn HBM GB/s"
FALLBACK_HBM_GBS = 6650.0
# DRAM bytes a launch of the decode kernel moves, as a multiple of its algorithmic bytes: Nsight
# Compute counted dram__bytes_read + dram__bytes_write on the small cases (16 x 8 192 fp16:
# 134.42 MB read + 0.36 MB written for 134.22 MB; 32 x 8 192 INT8: 153.48 + 0.3 MB for 153.09 MB;
# the selected pages of 8 x 8 192 at 50 %: 33.72 MB for 33.55 MB), and the traffic grows with the
# pages read, so a full-size launch moves the same multiple.
NCU_TRAFFIC_RATIO = {"dense": 1.0042, "int8": 1.0045, "sparse": 1.0051}


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
            return self
        self.thread = threading.Thread(target=self._read, daemon=True)
        self.thread.start()
        return self

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
            self.proc = None

    def mhz(self, t0: float, t1: float):
        """Median SM clock of the samples inside [t0, t1], else of the two nearest."""
        rows = [(t, r) for t, r in self.rows if len(r) >= 6 and r[0].replace(".", "").isdigit()]
        if not rows:
            return None
        inside = [float(r[0]) for t, r in rows if t0 <= t <= t1]
        if inside:
            return statistics.median(inside)
        mid = 0.5 * (t0 + t1)
        near = sorted(rows, key=lambda tr: abs(tr[0] - mid))[:2]
        return statistics.median(float(r[0]) for _, r in near)

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


class Ranks:
    """This process's place among the replicas: one rank per GPU, `torch.distributed`
    for the barrier and the max over ranks only."""

    def __init__(self):
        import torch

        self.world = int(os.environ.get("WORLD_SIZE", "1"))
        self.rank = int(os.environ.get("RANK", "0"))
        self.local = int(os.environ.get("LOCAL_RANK", "0"))
        self.dev = torch.device("cuda", self.local)
        torch.cuda.set_device(self.dev)
        self.dist = None
        if self.world > 1:
            import torch.distributed as dist

            dist.init_process_group("nccl", device_id=self.dev)
            self.dist = dist
        visible = os.environ.get("CUDA_VISIBLE_DEVICES")
        self.smi_index = int(visible.split(",")[self.local]) if visible else self.local

    def barrier(self):
        import torch

        if self.dist is not None:
            self.dist.barrier()
        torch.cuda.synchronize()

    def max_ms(self, values):
        """Element-wise max over ranks of a list of per-rank times."""
        from latentserve_b200 import replicas

        return replicas.max_over_ranks(values, self.dist, self.dev)

    def close(self):
        if self.dist is not None:
            self.dist.barrier()
            self.dist.destroy_process_group()


def timed_blocks(ranks: Ranks, run_step, steps: int, warmup: int, sampler: ClockSampler,
                 blocks: int = BLOCKS, sustain_s: float = SUSTAIN_S):
    """`blocks` timed regions of exactly `steps` calls of `run_step`, each between a
    barrier + synchronise on both sides and timed with CUDA events on the launching
    stream; max over ranks. The same load runs untimed for `sustain_s` seconds between
    the first block and the rest, so the first is a burst figure and the others are
    taken at the clock the GPU settles to. -> per-block [ms per step], [median SM MHz],
    and the wall-clock span of it all."""
    import torch

    for _ in range(max(3, warmup)):
        run_step()
    ms, spans = [], []
    t_begin = time.time()
    for blk in range(blocks):
        ranks.barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        w0 = time.time()
        e0.record()
        for _ in range(steps):
            run_step()
        e1.record()
        ranks.barrier()
        spans.append((w0, time.time()))
        ms.append(e0.elapsed_time(e1) / steps)
        if blk == 0 and blocks > 1:
            until = time.time() + sustain_s
            while time.time() < until:
                for _ in range(10):
                    run_step()
                torch.cuda.synchronize()
    ms = ranks.max_ms(ms)
    time.sleep(0.12)                                     # let the sampler see the last block
    mhz = [sampler.mhz(a, b) for a, b in spans]
    return ms, mhz, (t_begin, time.time())


def block_report(ms, mhz, to_value=None):
    """The blocks of `timed_blocks` as a JSON object; `to_value` maps ms per step to
    the workload's metric."""
    med = statistics.median(ms)
    later = ms[1:] or ms
    rep = {"ms_per_step": [round(x, 4) for x in ms], "sm_mhz": mhz,
           "median_ms": round(med, 4), "min_ms": round(min(ms), 4), "max_ms": round(max(ms), 4),
           "first_block_ms": round(ms[0], 4), "sustained_ms": round(statistics.median(later), 4),
           # time x clock: equal across blocks when the kernel follows the SM clock
           "ms_x_ghz": [None if c is None else round(t * c / 1e3, 4) for t, c in zip(ms, mhz)]}
    if to_value is not None:
        rep["value_first_block"] = round(to_value(ms[0]), 1)
        rep["value_sustained"] = round(to_value(statistics.median(later)), 1)
    return rep


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


def seq_lens_of(context, batch, rng):
    import numpy as np

    if context == "loguniform_1k_32k":
        return np.exp(rng.uniform(np.log(1024), np.log(32768), size=batch)).astype(int).tolist()
    if context == "uniform_8k_32k":
        return rng.integers(8192, 32769, size=batch).tolist()
    return [context] * batch


def graph_us(layers, fn, reps):
    """us per call of `fn(i)`, i over the layers, from replays of one CUDA graph of
    those calls (CUDA events on the launching stream; no Python, no launch latency)."""
    import torch

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


def run_attention(name, args, ranks: Ranks, headline: bool):
    """One attention workload: the step graph timed in blocks, the kernel's roofline
    figures, and (headline only) the host-buffer leg and the CPU baseline."""
    import numpy as np
    import torch

    from latentserve_b200 import paged_decode_cuda as pdc
    from latentserve_b200 import synthetic

    batch, context, layers = WORKLOADS[name]
    dev, rank, world = ranks.dev, ranks.rank, ranks.world
    pdc.set_programmatic_launch(True, early_pages=True)
    pdc.set_loader("auto")
    rng = np.random.default_rng(1234 + rank)
    seq_lens = seq_lens_of(context, batch, rng)
    kind = name.split("_")[0]
    breakdown = ref_kernel = None
    if kind == "int8":
        w = synthetic.int8_pools_on_device(seq_lens, layers, dev, seed=rank)
        tables, lens = w["block_tables"], w["seq_lens"]
        layer_bytes = synthetic.kv_bytes_int8(seq_lens)

        def layer_call(i):
            L = w["layers"][i]
            return pdc.paged_decode_cuda(w["q"][i], L["k_pool"], L["v_pool"], tables, lens, max(seq_lens),
                                         k_scale=L["k_scale"], v_scale=L["v_scale"],
                                         k_residual=L["k_residual"], res_rows=w["res_rows"])
        launches_per_layer, kernel_name = 1, "decode_kernel<int8> (split-KV + in-kernel merge)"
        roof_bytes = layer_bytes
    elif kind.startswith("sparse"):
        from latentserve_b200 import paged_sparse as ps

        w = synthetic.sparse_pools_on_device(batch, context, layers, dev, seed=rank)
        tables, lens = w["block_tables"], w["seq_lens"]
        pages = -(-context // 16)
        ratio = {"50": 0.5, "25": 0.25, "12": 0.125}[kind[len("sparse"):len("sparse") + 2]]
        keep = ps.budget(ratio, pages)
        # indexer reads kmin + kmax of every page-head, the scores are written and read back,
        # attention reads the selected pages
        layer_bytes = batch * 2 * (pages * 512 + pages * 8 + keep * 16 * 512)
        roof_bytes = batch * 2 * keep * 16 * 512

        def layer_call(i):
            k, v = w["pools"][i]
            kmin, kmax = w["bounds"][i]
            return ps.sparse_attention(w["q"][i], k, v, tables, lens, kmin, kmax, ratio=ratio,
                                       max_seq_len=context)
        launches_per_layer = 3
        kernel_name = "decode_kernel<sparse> (attention over the selected pages)"
    else:
        w = synthetic.dense_pools_on_device(batch, seq_lens, layers, dev, seed=rank)
        tables, lens = w["block_tables"], w["seq_lens"]
        layer_bytes = synthetic.kv_bytes_fp16(seq_lens)

        def layer_call(i):
            k, v = w["pools"][i]
            return pdc.paged_decode_cuda(w["q"][i], k, v, tables, lens, max(seq_lens))
        launches_per_layer, kernel_name = 1, "decode_kernel<fp16> (split-KV + in-kernel merge)"
        roof_bytes = layer_bytes
    step_bytes = layer_bytes * layers

    # One step = the layer calls, captured once.
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

    sampler = ClockSampler(ranks.smi_index).start()
    only = args.only
    ms, mhz, span = timed_blocks(ranks, graph.replay, args.steps, args.warmup, sampler,
                                 blocks=1 if only else BLOCKS, sustain_s=0.0 if only else SUSTAIN_S)
    ms_step = statistics.median(ms)

    def to_value(t_ms):
        from latentserve_b200 import replicas

        return replicas.aggregate_throughput(step_bytes, t_ms * 1e-3, world) / 1e9

    reps = max(3, min(50, args.steps))
    own_dense_us = None
    if kind.startswith("sparse"):
        sel_fixed = ps.select(ps.page_scores(w["q"][0], *w["bounds"][0], tables, lens), keep).clone()
        scores_fixed = ps.page_scores(w["q"][0], *w["bounds"][0], tables, lens).clone()
        breakdown = {
            "page_index_us": round(graph_us(layers, lambda i: ps.page_scores(
                w["q"][i], *w["bounds"][i], tables, lens), reps), 2),
            "select_pages_us": round(graph_us(layers, lambda i: ps.select_for_attention(
                scores_fixed, lens, keep, ratio), reps), 2),
            "topk_pages_us_not_on_the_path": round(graph_us(layers, lambda i: ps.select(
                scores_fixed, keep), reps), 2),
            "sparse_decode_us": round(graph_us(layers, lambda i: ps.sparse_decode(
                w["q"][i], w["pools"][i][0], w["pools"][i][1], tables, lens, sel_fixed, ratio=ratio), reps), 2),
        }
        kernel_us = breakdown["sparse_decode_us"]
        own_dense_us = round(graph_us(layers, lambda i: pdc.paged_decode_cuda(
            w["q"][i], w["pools"][i][0], w["pools"][i][1], tables, lens, context), reps), 2)
    else:
        # The step graph holds this kernel's launches and nothing else.
        kernel_us = 1e3 * ms_step / layers
    clocks = sampler.summary(*span)
    peak, peak_kind = measured_peak()
    achieved = roof_bytes / (kernel_us * 1e-6) / 1e9
    roofline = {"bound": "hbm", "achieved": round(achieved, 1), "peak": peak, "unit": "GB/s",
                "frac": round(achieved / peak, 4),
                "traffic": int(round(roof_bytes * NCU_TRAFFIC_RATIO["sparse" if kind.startswith("sparse") else kind])),
                "peak_kind": f"of {peak_kind}", "kernel": kernel_name,
                "kernel_us": round(kernel_us, 2), "algorithmic_bytes_per_launch": roof_bytes,
                "frac_of_8TBs": round(achieved / 8000.0, 4),
                "how": ("CUDA events around replays of a graph of this kernel's launches"
                        if kind.startswith("sparse") else
                        "timed region / launches: the step graph holds this kernel's launches only, "
                        "gaps between them included"),
                "breakdown": breakdown}

    e2e = cpu = None
    if headline and not only:
        e2e = run_e2e(args, WORKLOADS[name], ranks)
        if rank == 0 and world == 1 and kind == "dense":
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
            nbytes = synthetic.kv_bytes_fp16(seq_lens[:seqs])
            cpu = {"value": round(nbytes / secs / 1e9, 3), "unit": "GB/s", "cores": cpu_cores,
                   "kind": "port",
                   "sample": f"one layer call over {seqs} of the {batch} sequences "
                             f"({nbytes / 1e6:.0f} MB of KV), torch CPU fp32 gather-then-softmax, best of 3"}
    # The reference's own CUDA kernels (its .cu files compiled as they are for sm_100a into
    # oracle/_ref, driven as its host code drives them) on this GPU and this workload, beside
    # ours. Part of the baseline leg; absent when the cubins were not built.
    if rank == 0 and world == 1 and not only:
        ref_kernel = time_reference_kernel(kind, w, tables, lens, seq_lens, layers, layer_bytes, context,
                                           ratio if kind.startswith("sparse") else None)
    sampler.stop()

    out = {
        "metric": METRIC, "value": round(to_value(ms_step), 1), "unit": "GB/s", "n_gpus": world,
        "steps": args.steps, "warmup": max(3, args.warmup), "ms_per_step": round(ms_step, 4),
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "i8" if kind == "int8" else "f16", "data": "synthetic",
        "config": {"workload": name, "batch_per_gpu": batch,
                   "context": context if isinstance(context, int) else
                   f"{context}: min {min(seq_lens)}, mean {int(np.mean(seq_lens))}, max {max(seq_lens)}",
                   "layers_per_step": layers, "q_heads": 12, "kv_heads": 2, "head_dim": 128,
                   "page": 16, "pool_blocks": w["num_blocks"], "programmatic_launch": True,
                   "early_pages": True, "loader": "tma (INT8 pools) / cp.async (fp16 pools)",
                   "parallelism": f"replicas x{world} (sequence-sharded, no collective)",
                   "l2": f"no flush: each step reads {step_bytes / 1e9:.2f} GB, L2 is 126 MB",
                   "step": f"{layers} layer calls ({launches_per_layer} launch(es) each) replayed from one "
                           "CUDA graph",
                   "timing": f"{len(ms)} blocks of {args.steps} steps, median block reported"},
        "pct_of_8TBs": round(100.0 * to_value(ms_step) / world / 8000.0, 2),
        "us_per_layer_call": round(1e3 * ms_step / layers, 2),
        "blocks": block_report(ms, mhz, to_value),
        "roofline": roofline, "cpu_baseline": cpu, "reference_kernel": ref_kernel, "e2e": e2e,
        "gpu_launches": launches_per_layer * layers * args.steps * len(ms), "clocks": clocks,
    }
    if own_dense_us is not None:
        out["own_dense_kernel_us_same_batch"] = own_dense_us
        out["pipeline_over_own_dense"] = round(1e3 * ms_step / layers / own_dense_us, 3)
    del graph, w
    release_device_memory()
    return out


def release_device_memory():
    import torch

    gc.collect()
    torch.cuda.synchronize()
    torch.cuda.empty_cache()


def run_model_step(name, args, ranks: Ranks):
    """Whole decode steps (all 28 layers: projections, norms, RoPE, append, attention,
    output head, greedy argmax) replayed from one CUDA graph. Reports ms per step
    (graph replay only, and the full loop with cache.advance() on the host) and
    tokens per second; with N ranks every rank serves its own sequences."""
    import random

    import numpy as np
    import torch

    from latentserve_b200 import cache as lc, decode_step as ds, paged_decode_cuda as pdc

    pdc.set_programmatic_launch(True, early_pages=True)
    pdc.set_loader("tma")
    batch, context, kind, ratio, prefix = STEP_WORKLOADS[name]
    world, rank, dev = ranks.world, ranks.rank, ranks.dev
    total_seqs = batch * world
    if isinstance(context, str) and world > 1:
        # A ragged batch for the whole job, spread over the replicas by outstanding tokens
        # (what a router does); every rank serves its own share.
        from latentserve_b200 import replicas

        all_lens = seq_lens_of(context, total_seqs, np.random.default_rng(1234))
        lens = [all_lens[i] for i in replicas.partition_by_tokens(all_lens, world)[rank]]
        batch = len(lens)
    else:
        lens = seq_lens_of(context, batch, np.random.default_rng(1234 + rank))
    steps, warm = args.steps, max(3, args.warmup)
    blocks = 1 if args.only else 3
    shape = ds.QwenShape()
    room = (steps + 2) * blocks + warm + 24
    spec = lc.KVCacheSpec(num_layers=shape.num_layers, num_kv_heads=shape.kv_heads,
                          head_dim=shape.head_dim, max_seq_len=max(lens) + room + 16,
                          max_batch_size=batch, device=str(dev))
    nblocks = int(1.2 * sum(-(-(n + room) // 16) for n in lens)) + 64
    cache = (lc.Int8PagedKVCache if kind == "int8" else lc.PagedKVCache)(spec, num_blocks=nblocks)
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
    owners = []
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
    model = ds.DecodeModel(shape, dev, max_pos=max(lens) + room + 16, seed=rank)
    model.set_sparse(ratio)
    hint = max(lens) + room
    runner = ds.GraphedStep(model, cache, batch, hint)
    runner.tokens.random_(0, shape.vocab, generator=g)
    cache.advance(1, batch_size=batch)
    runner.positions.copy_(torch.tensor([n - 1 for n in cache.seq_lens], dtype=torch.long))
    runner.capture()

    def loop_step():
        cache.advance(1, batch_size=batch)
        runner.step()

    sampler = ClockSampler(ranks.smi_index).start()
    loop_ms, loop_mhz, span = timed_blocks(ranks, loop_step, steps, warm, sampler, blocks=blocks,
                                           sustain_s=0.0)
    # Graph replay alone (lengths frozen), as the reference quotes its "graph-only" step.
    graph_ms, graph_mhz, span2 = timed_blocks(ranks, runner.graph.replay, steps, 3, sampler,
                                              blocks=blocks, sustain_s=0.0)
    clocks = sampler.summary(span[0], span2[1])
    sampler.stop()
    loop_med, graph_med = statistics.median(loop_ms), statistics.median(graph_ms)
    mean_len = float(np.mean(lens)) + warm + steps * blocks / 2
    kv_per_tok = shape.num_layers * shape.kv_heads * (292 if kind == "int8" else 512)
    kv_bytes = mean_len * batch * kv_per_tok * (ratio if ratio else 1.0)
    floor_ms = (kv_bytes + model.weight_bytes()) / (measured_peak()[0] * 1e9) * 1e3
    out = {
        "metric": "Qwen2.5-1.5B decode step ms", "value": round(loop_med, 4), "unit": "ms",
        "n_gpus": world, "steps": steps, "warmup": warm, "ms_per_step": round(loop_med, 4),
        "higher_is_better": False, "scaling": "weak", "vs_baseline": None,
        "dtype": "i8" if kind == "int8" else "f16", "data": "synthetic",
        "config": {"workload": name, "batch_per_gpu": batch,
                   "context": f"min {min(lens)}, mean {int(np.mean(lens))}, max {max(lens)}",
                   "kv_cache": kind, "sparse_ratio": ratio, "shared_prefix_tokens": prefix,
                   "sequences_sharing_prefix": len(owners),
                   "layers": shape.num_layers, "programmatic_launch": True,
                   "projections": "ls" if model.streams_projections(batch) else "cublas",
                   "early_pages": True, "loader": "tma",
                   "int8_finalize": "inside the captured step" if kind == "int8" else None,
                   "parallelism": f"replicas x{world} (sequence-sharded, no collective)"
                                  + (", sequences assigned by outstanding tokens" if isinstance(context, str)
                                     and world > 1 else ""),
                   "sequences_whole_job": total_seqs,
                   "timing": f"{blocks} blocks of {steps} steps, median block reported"},
        "graph_replay_ms": round(graph_med, 4),
        "tokens_per_s": round(total_seqs / (loop_med * 1e-3), 1),
        "hbm_floor_ms": round(floor_ms, 4),
        "frac_of_floor": round(floor_ms / graph_med, 4),
        "blocks": {"loop": block_report(loop_ms, loop_mhz), "graph_replay": block_report(graph_ms, graph_mhz)},
        "clocks": clocks,
    }
    del runner, model, cache
    release_device_memory()
    return out


def time_reference_kernel(kind, w, tables, lens, seq_lens, layers, layer_bytes, context, ratio):
    """us per layer call and GB/s of the reference's kernels on this workload (fills of its
    m / l scratch included, as on every call of its host code; its Triton merge not included)."""
    try:
        from oracle import ref_kernels
    except Exception:                                      # the oracle folder did not travel
        return None
    name = {"int8": "paged_decode_int8", "dense": "paged_decode_fp16"}.get(kind, "paged_sparse_fp16")
    if not ref_kernels.available(name):
        return None
    runs = []
    for i in range(layers):
        if kind == "int8":
            L = w["layers"][i]
            runs.append(ref_kernels.RefDecode(w["q"][i], L["k_pool"], L["v_pool"], tables, lens,
                                              max(seq_lens), k_scale=L["k_scale"], v_scale=L["v_scale"],
                                              k_residual=L["k_residual"], res_rows=w["res_rows"]))
        elif kind == "dense":
            k, v = w["pools"][i]
            runs.append(ref_kernels.RefDecode(w["q"][i], k, v, tables, lens, max(seq_lens)))
        else:
            k, v = w["pools"][i]
            runs.append(ref_kernels.RefSparse(w["q"][i], k, v, tables, lens, *w["bounds"][i], ratio=ratio,
                                              max_seq_len=context))
    us = graph_us(layers, lambda i: runs[i].launch(), 3)
    what = (f"LatentServe kernels/cuda/{name}.cu compiled for sm_100a, grid (B, splits, H) x 1 warp, "
            "m / l fills included, split merge not included")
    if kind.startswith("sparse"):
        what = ("LatentServe's sparse trio: page_index + torch.topk(sorted) + paged_sparse_fp16 "
                "(kernels/cuda/paged_sparse_fp16.cu compiled for sm_100a, its launch geometry), "
                "m / l fills included, split merge not included")
    return {"value": round(layer_bytes / (us * 1e-6) / 1e9, 1), "unit": "GB/s", "us_per_layer_call": round(us, 2),
            "splits": runs[0].splits, "what": what}


def run_e2e(args, workload, ranks: Ranks):
    """Steps through PagedKVCache + paged_decode_attention with host buffers."""
    import random

    import torch

    from latentserve_b200 import cache as lc, paged_decode as pd, synthetic

    batch, context, layers = workload
    dev, dist, world = ranks.dev, ranks.dist, ranks.world
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
    random.Random(0).shuffle(cache.allocator._free)      # shuffled block tables, as in `value`
    for i in range(batch):
        cache.tables[i].append(context - 1)
    # One pinned host image per step: for every layer and (sequence, KV head) the six query
    # rows, then the new K row, then the new V row; one copy to the device, of which the
    # layers' q / k / v are strided views.
    host_in = torch.randn(layers, batch, h, r + 2, d).half().pin_memory()
    host_out = torch.empty(layers, batch, h, r, d, dtype=torch.float16).pin_memory()
    dev_in = torch.empty_like(host_in, device=dev)
    dout = torch.empty(layers, batch, h, r, d, dtype=torch.float16, device=dev)
    cache.enable_fused_append()                          # the append rides on the attention launch

    # Per-layer views made once, as a model's layers hold them.
    q_l = [dev_in[i, :, :, :r] for i in range(layers)]
    k_l = [dev_in[i, :, :, r:r + 1] for i in range(layers)]
    v_l = [dev_in[i, :, :, r + 1:r + 2] for i in range(layers)]
    out_l = [dout[i] for i in range(layers)]
    host_s = [0.0]
    # Replayed from a graph, the step's copies run beside its kernels: the first layers' inputs
    # go ahead and the rest follow on a copy stream while those layers compute; the results of
    # the leading layers leave for the host while the trailing ones compute. (Eager, the extra
    # stream operations cost the host more at the start of the step than the overlap returns:
    # measured 1.55 ms against 1.51 ms, so the eager step makes one copy each way.) Every byte of
    # host_in and host_out moves inside the step, and the step ends when host_out is complete.
    in_cut = min(2, layers)                              # layers whose inputs are copied first
    out_cut = layers - max(1, layers // 4)               # layers whose results leave early
    s_in, s_out = torch.cuda.Stream(), torch.cuda.Stream()
    ev_in0, ev_in1, ev_out0 = torch.cuda.Event(), torch.cuda.Event(), torch.cuda.Event()

    def layer_range(lo, hi, tables, lens, hint):
        for layer in range(lo, hi):
            cache.write(layer, k_l[layer], v_l[layer])
            pd.paged_decode_attention(q_l[layer], cache.k_pool[layer], cache.v_pool[layer],
                                      tables, lens, max_seq_len=hint, out=out_l[layer])

    def step_body(overlap_copies):
        """One step's copies and layer calls on the current stream (and, overlapped, on two
        copy streams that fork from and rejoin it)."""
        main = torch.cuda.current_stream()
        tables, lens = cache.block_tables_tensor(batch), cache.seq_lens_tensor(batch)
        hint = cache.max_len
        if not overlap_copies:
            dev_in.copy_(host_in, non_blocking=True)
            layer_range(0, layers, tables, lens, hint)
            host_out.copy_(dout, non_blocking=True)
            return
        s_in.wait_stream(main)
        with torch.cuda.stream(s_in):
            dev_in[:in_cut].copy_(host_in[:in_cut], non_blocking=True)
            ev_in0.record()
            if in_cut < layers:
                dev_in[in_cut:].copy_(host_in[in_cut:], non_blocking=True)
            ev_in1.record()
        main.wait_event(ev_in0)
        layer_range(0, in_cut, tables, lens, hint)
        main.wait_event(ev_in1)
        layer_range(in_cut, out_cut, tables, lens, hint)
        ev_out0.record()
        with torch.cuda.stream(s_out):
            s_out.wait_event(ev_out0)
            host_out[:out_cut].copy_(dout[:out_cut], non_blocking=True)
        layer_range(out_cut, layers, tables, lens, hint)
        host_out[out_cut:].copy_(dout[out_cut:], non_blocking=True)
        main.wait_stream(s_out)

    graph = [None]

    def step():
        # The cache has been advanced for this step already (by the previous step, below):
        # the host's bookkeeping for step t + 1 runs while the GPU works on step t, and its
        # one small copy is ordered behind step t's kernels on the stream.
        t0 = time.perf_counter()
        if graph[0] is None:
            step_body(False)
        else:
            graph[0].replay()
        cache.advance(1, batch_size=batch)               # next step's slots, lengths and tables
        host_s[0] += time.perf_counter() - t0            # host time to enqueue the step
        torch.cuda.current_stream().synchronize()        # the step's result is on the host

    def timed():
        for _ in range(warm):
            step()
        ranks.barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        host_s[0] = 0.0
        e0.record()
        for _ in range(steps):
            step()
        e1.record()
        torch.cuda.synchronize()
        t_ms = ranks.max_ms([e0.elapsed_time(e1)])[0]
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
        step_body(True)
    torch.cuda.current_stream().wait_stream(side)
    torch.cuda.synchronize()
    cg = torch.cuda.CUDAGraph()
    with torch.cuda.graph(cg):
        step_body(True)
    graph[0] = cg
    g_ms, g_host_ms = timed()
    g_mean_len = context + 2 * warm + steps + (steps + 1) / 2
    step_bytes = synthetic.kv_bytes_fp16([mean_len] * batch) * layers
    g_bytes = synthetic.kv_bytes_fp16([g_mean_len] * batch) * layers
    h2d = host_in.numel() * 2 + cache._step_bytes
    d2h = host_out.numel() * 2
    out = {"value": round(world * step_bytes / (ms * 1e-3) / 1e9, 1), "unit": "GB/s",
           "h2d_bytes_per_step": int(h2d), "d2h_bytes_per_step": int(d2h),
           "ms_per_step": round(ms, 4), "host_enqueue_ms_per_step": round(host_ms, 4),
           "steps": steps, "gpu_launches_per_step": layers,
           "path": "PagedKVCache.write + paged_decode_attention per layer, eager (the cache in fused-append "
                   "mode: the write rides on the attention launch); PagedKVCache.advance for the next step "
                   "issued while the GPU works on this one",
           "graph_replay": {"value": round(world * g_bytes / (g_ms * 1e-3) / 1e9, 1), "unit": "GB/s",
                            "ms_per_step": round(g_ms, 4),
                            "host_enqueue_ms_per_step": round(g_host_ms, 4),
                            "path": "same host buffers; the copies (split in two each way, on copy streams "
                                    "beside the kernels) and the 28 write + attention calls captured in one "
                                    "CUDA graph and replayed"}}
    del cg, cache
    graph[0] = None
    release_device_memory()
    return out


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=50)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default=HEADLINE, choices=sorted(WORKLOADS) + sorted(STEP_WORKLOADS))
    ap.add_argument("--only", action="store_true",
                    help="the named workload's device-timed leg and nothing else: one block, no host-buffer "
                         "leg, no CPU baseline, no other workloads (profiler captures)")
    args = ap.parse_args()
    if args.impl == "reference":
        run_reference(args, WORKLOADS.get(args.workload, WORKLOADS[HEADLINE]))
        return

    import torch

    from latentserve_b200 import _lib

    if not torch.cuda.is_available():
        raise SystemExit("bench.py measures the CUDA path and there is no CUDA device")
    _lib.lib()                                    # fail here, loudly, if the library is missing
    ranks = Ranks()
    if args.workload in STEP_WORKLOADS:
        line = run_model_step(args.workload, args, ranks)
    else:
        line = run_attention(args.workload, args, ranks, headline=True)
    if args.workload == HEADLINE and not args.only:
        others = {}
        for name, every_n in OTHER_WORKLOADS:
            if ranks.world > 1 and not every_n:
                continue
            if name in STEP_WORKLOADS:
                others[name] = run_model_step(name, args, ranks)
            else:
                others[name] = run_attention(name, args, ranks, headline=False)
        line["other_workloads"] = others
    if ranks.rank == 0:
        print(json.dumps(line))
    ranks.close()


if __name__ == "__main__":
    main()
