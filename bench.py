"""Benchmark of the INT8 shared-KV decode path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl b200|reference] [--workload box|c128|c4mtp|writer]

Default workload ("box"): the box-scale decode step.  2048 concurrent requests with context
lengths log-uniform over 4k..1M tokens are batch-sharded over the N GPUs (longest-first
greedy by KV rows); every GPU holds the INT8 paged KV of its requests for alternating
C4 (top-k 1024 + window 128) and C128 (all compressed rows + window 128) layers, as many
layer pairs as fill about --kv-gb of its HBM.  A *pass* is one decode pass of the hot path
over all resident layers: one attention launch per layer, T = 1 query token per request.  A
*step* is --passes consecutive passes (default: as many as make the K timed steps last about
2.5 s, so that the figure is taken at the clocks the part sustains, not in a 30 ms burst).
There is no collective on the path; ranks only meet at the timing barriers.

Printed JSON line (rank 0):
  value      (request, layer) attention evaluations per second over all GPUs with everything
             resident in HBM, over the K timed steps (replays of a captured pass);
  burst      the same over K single passes (what a 30 ms region at boost clocks gives);
  roofline   for the layer kind with the larger share of a pass (`roofline_other` for the other):
             algorithmic KV bytes per launch over the mean launch duration, CUDA events around
             replays of a graph that holds that kind's launches back to back, taken right after
             the sustained region;
  writer     the paged cache writer at its own configuration (65 536 rows into an original cache
             and 16 384 into a ratio-4 compressed cache per step): rows/s, GB/s, fraction of peak;
  e2e        the decode step through the prepared operators with host buffers: per pass and layer
             one pinned staging buffer (the new KV row of every request, Q and the C4 top-k
             selections) is copied in, the cache writer and the attention run, the BF16 output is
             copied back (three streams, so copies overlap compute); `copy_only` is the same step
             with the kernels left out, the ceiling the copies alone set;
  cpu_baseline  the reference's CPU implementation timed on this host on a bounded sample.
`--workload writer` times the paged cache writer alone and prints rows/s.
`--impl reference` times the reference's own CPU path (`tiled_quantized_reference` of its
reference.py, installed under baseline/_ref/; the CPU restatement under oracle/ when that
file is absent) on a bounded seeded sample.
"""
import argparse
import json
import math
import os
from pathlib import Path
import statistics
import subprocess
import sys
import time

ROOT = Path(__file__).resolve().parent
for entry in (ROOT / "ascend-int8-attention_b200", ROOT):
    if str(entry) not in sys.path:
        sys.path.insert(0, str(entry))

import torch  # noqa: E402

METRIC = "decode attn queries/s/GPU & achieved HBM GB/s (INT8 KV) at 1/2/4/8 B200"
ROW_BYTES = 512
# DRAM traffic (read + written) per algorithmic KV byte, from profiler captures of smaller launches
# of the same kernels (dram__bytes_read.sum + dram__bytes_write.sum over the algorithmic bytes of
# the captured launch); traffic grows in proportion to the queries processed.
TRAFFIC_PER_ALGORITHMIC_BYTE = {4: 1.075, 128: 1.040}


def measured_peaks():
    path = ROOT / "MEASURED_PEAKS.json"
    if path.is_file():
        data = json.loads(path.read_text())
        return float(data["hbm_gbs"]), "measured"
    return 6650.0, "fallback"


# --------------------------------------------------------------------------- workloads
def box_lengths(requests, seed=0):
    from npu_sparse_attn_sharedkv_int8.synthetic import log_uniform_lengths
    return log_uniform_lengths(requests, 4096, 1 << 20, seed)


def shard(lengths, ranks):
    """Longest-first greedy assignment of requests to ranks by KV rows per layer pair."""
    cost = lengths // 4 + lengths // 128 + 256
    order = torch.argsort(cost, descending=True).tolist()
    load, owner = [0] * ranks, [[] for _ in range(ranks)]
    for index in order:
        r = min(range(ranks), key=load.__getitem__)
        owner[r].append(index)
        load[r] += int(cost[index])
    return [sorted(o) for o in owner]


def combine_ranks(elapsed_ms, counts, device, world):
    """Whole-job figures from per-rank ones: the slowest rank's time, the sum of the work counts.
    The only communication of the benchmark (the decode path itself has no exchange step)."""
    if world <= 1:
        return float(elapsed_ms), [float(c) for c in counts]
    import torch.distributed as dist
    times = torch.tensor([elapsed_ms], dtype=torch.float64, device=device)
    totals = torch.tensor(list(counts), dtype=torch.float64, device=device)
    dist.all_reduce(times, op=dist.ReduceOp.MAX)
    dist.all_reduce(totals, op=dist.ReduceOp.SUM)
    return float(times[0]), totals.tolist()


def pair_bytes(lengths):
    """Resident bytes of one C4 + C128 layer pair (compressed pools dominate)."""
    c4 = ((lengths // 4 + 31) // 32).clamp_min(1).sum() * 16384
    c128 = ((lengths // 128 + 31) // 32).clamp_min(1).sum() * 16384
    ori = 2 * 6 * lengths.numel() * 16384
    return int(c4 + c128 + ori)


def workload_label(args):
    return {"box": f"box-scale decode step: {args.requests} requests, ctx log-uniform 4k-1M, alternating C4/C128",
            "c128": f"C128 decode, B=64, T={args.queries}, ctx U[8k,128k], compact pages (stride 38 x 16384 B, offset 16384 B)"
                    + (f", query groups of {args.query_group}" if args.query_group > 1 else ""),
            "c4mtp": "C4 decode with MTP, B=256, T=2, ctx U[32k,128k], top-k 1024 + window 128",
            "writer": "paged INT8 cache writer: 65536 BF16 rows -> original cache + 16384 rows -> ratio-4 compressed cache, random slots"
            }[args.workload]


def build_workload(args, rank, world):
    from npu_sparse_attn_sharedkv_int8 import synthetic
    device = torch.device("cuda", torch.cuda.current_device())
    if args.workload == "box":
        lengths = box_lengths(args.requests, seed=0)
        mine = lengths[torch.tensor(shard(lengths, world)[rank])]
        per_pair = pair_bytes(mine)
        pairs = max(1, round(args.kv_gb * 1e9 / per_pair))
        while pairs > 1 and pairs * per_pair > 165e9:      # leave room for tables, queries and the context
            pairs -= 1
        if args.max_pairs:
            pairs = min(pairs, args.max_pairs)
        ratios = {"pair": [4, 128], "c4": [4], "c128": [128]}[args.layers] * pairs
        work = synthetic.build("box", device, mine, ratios=ratios, queries=1, seed=100 + rank, max_context=1 << 20)
    elif args.workload == "c128":
        lengths = synthetic.uniform_lengths(64, 8192, 131072, seed=1)
        ratios = [128] * args.rotate
        work = synthetic.build("c128", device, lengths, ratios=ratios, queries=args.queries, seed=200 + rank, stride_slots=38,
                               slot_offset=1, max_context=135000)
    else:
        lengths = synthetic.uniform_lengths(256, 32768, 131072, seed=2)
        ratios = [4] * args.rotate
        work = synthetic.build("c4mtp", device, lengths, ratios=ratios, queries=2, seed=300 + rank, max_context=135000)
    return work, workload_label(args)


# --------------------------------------------------------------------------- host memory placement
class HostMemoryNear:
    """While active, this process runs on the CPU cores next to CUDA device `index` (as NVML reports
    them), so that pinned host buffers allocated inside land in that GPU's NUMA node; with several
    ranks on one host, copies through the other socket cost bandwidth.  Does nothing when NVML or
    the affinity calls are unavailable.  The process's CPU affinity is restored on exit; no GPU
    setting is touched."""

    def __init__(self, index):
        self.index, self.saved = index, None

    def __enter__(self):
        try:
            if self.index < 0:
                return self
            import pynvml
            props = torch.cuda.get_device_properties(self.index)
            bus = f"{props.pci_domain_id:08x}:{props.pci_bus_id:02x}:{props.pci_device_id:02x}.0"
            pynvml.nvmlInit()
            handle = pynvml.nvmlDeviceGetHandleByPciBusId(bus.encode())
            words = pynvml.nvmlDeviceGetCpuAffinity(handle, (os.cpu_count() + 63) // 64)
            cpus = {64 * w + b for w, word in enumerate(words) for b in range(64) if (int(word) >> b) & 1}
            allowed = os.sched_getaffinity(0)
            if cpus & allowed:
                self.saved = allowed
                os.sched_setaffinity(0, cpus & allowed)
        except Exception:
            self.saved = None
        return self

    def __exit__(self, *exc):
        if self.saved is not None:
            try:
                os.sched_setaffinity(0, self.saved)
            except Exception:
                pass
        return False


# --------------------------------------------------------------------------- clocks
class ClockSampler:
    FIELDS = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
              "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index):
        self.proc = None
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--id={index}", f"--query-gpu={self.FIELDS}",
                                          "--format=csv,noheader,nounits", "-lms", "50"],
                                         stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
        except OSError:
            pass

    def stop(self):
        if self.proc is None:
            return None
        self.proc.terminate()
        try:
            text, _ = self.proc.communicate(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
            text, _ = self.proc.communicate()
        sm, top, reasons = [], 0, set()
        for line in text.splitlines():
            parts = [p.strip() for p in line.split(",")]
            if len(parts) != 6 or not parts[0].isdigit():
                continue
            sm.append(int(parts[0]))
            top = max(top, int(parts[1]))
            for name, value in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), parts[2:]):
                if value == "Active":
                    reasons.add(name)
        if not sm:
            return None
        busy = [v for v in sm if v >= 0.5 * max(sm)] or sm
        return {"sm_mhz": statistics.median(busy), "sm_max_mhz": top, "reasons": sorted(reasons), "samples": len(sm)}


# --------------------------------------------------------------------------- CPU path
REFERENCE_FILE = ROOT / "baseline" / "_ref" / "npu_sparse_attn_sharedkv_int8" / "reference.py"


def cpu_implementation():
    """(kind, attention(case, scale) -> output): the reference's own `tiled_quantized_reference`
    (tile 128, one running state: its default configuration) when the reference has been installed
    under baseline/_ref/, else the restatement under oracle/.  The reference file is loaded by path
    under another module name because its package has the name of this build's package."""
    if REFERENCE_FILE.is_file():
        import importlib.util
        spec = importlib.util.spec_from_file_location("sharedkv_reference_cpu", REFERENCE_FILE)
        module = importlib.util.module_from_spec(spec)
        sys.modules[spec.name] = module          # dataclasses look their module up while the file is executed
        spec.loader.exec_module(module)

        def attend(case, scale):
            quant = module.CacheQuantization(scale)
            return module.tiled_quantized_reference(case, quant, quant, tile_size=128, splits=1)
        return "reference", attend
    from oracle import sharedkv_oracle as oracle
    return "port", lambda case, scale: oracle.attention_tiled(case, scale, scale)


def cpu_sample_case(ratio, lengths, seed):
    """Small CPU case with the shapes of the workload's requests: every request carries the
    rows it attends to (C4: 1024 selected rows + window; C128: all compressed rows + window)."""
    from npu_sparse_attn_sharedkv_int8.reference import SharedKVCase
    g = torch.Generator().manual_seed(seed)
    batch = len(lengths)
    new_lengths, cmp_pages = [], []
    for length in lengths:
        new_lengths.append(4097 if ratio == 4 else int(length))
        cmp_pages.append(32 if ratio == 4 else max(1, math.ceil(int(length) // 128 / 32)))
    ori_width = math.ceil(max(new_lengths) / 32)
    ori_table = torch.zeros((batch, ori_width), dtype=torch.int32)
    cmp_table = torch.zeros((batch, max(cmp_pages)), dtype=torch.int32)
    used_ori = used_cmp = 0
    for b, length in enumerate(new_lengths):
        for page in range(max(0, length - 128) // 32, (length - 1) // 32 + 1):
            ori_table[b, page] = used_ori
            used_ori += 1
        cmp_table[b, :cmp_pages[b]] = torch.arange(used_cmp, used_cmp + cmp_pages[b], dtype=torch.int32)
        used_cmp += cmp_pages[b]
    indices = None
    if ratio == 4:
        indices = torch.stack([torch.randperm(1024, generator=g).to(torch.int32) for _ in range(batch)]).view(batch, 1, 1024)
    return SharedKVCase(
        q=torch.randn(batch, 8, 512, generator=g).bfloat16(),
        ori=torch.randint(-127, 128, (used_ori, 32, 1, 512), generator=g, dtype=torch.int8), ori_block_table=ori_table,
        cu_q=torch.arange(batch + 1, dtype=torch.int32), seq_lens=torch.tensor(new_lengths, dtype=torch.int32),
        sink=torch.linspace(-2, 2, 8), cmp=torch.randint(-127, 128, (used_cmp, 32, 1, 512), generator=g, dtype=torch.int8),
        cmp_block_table=cmp_table, cmp_indices=indices, ratio=ratio)


def rows_attended(case):
    """KV rows the case's queries read (T = 1 per request in these samples)."""
    s = case.seq_lens.long()
    window = torch.clamp(s, max=128)
    compressed = s // 128 if case.ratio == 128 else torch.clamp(s // 4, max=case.cmp_indices.shape[-1])
    return int((window + compressed).sum())


def time_cpu_path(lengths, ratios, budget_s, threads):
    """Runs the CPU implementation on batches of 8 requests per layer kind until about `budget_s`
    seconds are spent.  Returns (queries/s, rows/s, queries timed, kind)."""
    kind, attend = cpu_implementation()
    if budget_s <= 0:
        return None, None, 0, kind
    torch.set_num_threads(threads)
    scale = torch.full((512,), 0.02)
    g = torch.Generator().manual_seed(7)
    kinds = sorted(set(ratios))
    done, rows, spent = 0, 0, 0.0
    attend(cpu_sample_case(kinds[0], [4096] * 2, 1), scale)     # warm the thread pool
    while spent < budget_s:
        for ratio in kinds:
            pick = lengths[torch.randint(len(lengths), (8,), generator=g)].tolist()
            case = cpu_sample_case(ratio, pick, seed=done)
            start = time.perf_counter()
            attend(case, scale)
            spent += time.perf_counter() - start
            done += len(pick)
            rows += rows_attended(case)
    return done / spent, rows / spent, done, kind


# --------------------------------------------------------------------------- small helpers
def capture(device, body):
    """One CUDA graph of `body()` captured on a side stream."""
    side = torch.cuda.Stream(device)
    side.wait_stream(torch.cuda.current_stream(device))
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.stream(side):
        with torch.cuda.graph(graph, stream=side):
            body()
    torch.cuda.current_stream(device).wait_stream(side)
    return graph


def timed(run, count):
    """Milliseconds (CUDA events on the current stream) of `count` calls of run(i)."""
    begin, finish = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    begin.record()
    for i in range(count):
        run(i)
    finish.record()
    return begin, finish


def clock_note(clocks, ms):
    """Median SM MHz of a region and its time x MHz (compare regions at different clocks by the product)."""
    if not clocks:
        return None
    return dict(clocks, ms_x_mhz=ms * clocks["sm_mhz"])


# --------------------------------------------------------------------------- cache writer
WRITER_METRIC = "paged INT8 KV cache writer rows/s & achieved HBM GB/s (BF16 -> INT8 quantize + slot scatter)"
WRITER_ROWS = ((65536, 1), (16384, 4))          # (rows per step, cache ratio): original cache, ratio-4 compressed cache


def writer_inputs(rows, seed, device):
    """Rows ~ N(0, sigma_c^2) with lognormal per-channel sigma, frozen scale 1.1 absmax / 127,
    a cache of rows/32 + 25 % pages and distinct random slots."""
    g = torch.Generator().manual_seed(seed)
    sigma = torch.exp(0.5 * torch.randn(512, generator=g))
    updates = (torch.randn(rows, 512, generator=g) * sigma).bfloat16()
    scale = (1.1 * updates.float().abs().amax(0) / 127).clamp_min(1e-6)
    pages = rows // 32 + rows // 128
    slots = torch.randperm(pages * 32, generator=g)[:rows].to(torch.int32)
    inverse = scale.double().reciprocal().float()
    return updates.to(device), slots.to(device), inverse.to(device), pages, scale


class WriterBench:
    """The writer at its own configuration: `copies` rotating sets of rows and caches (more than L2
    in all), one graph per launch size that holds one launch per set, and one graph per set that
    holds a whole step (both launches back to back)."""

    def __init__(self, device, rank, copies):
        from npu_sparse_attn_sharedkv_int8 import PreparedCacheWrite
        self.device, self.copies = device, copies
        self.ops, self.host_sets = [], []
        for c in range(copies):
            for rows, ratio in WRITER_ROWS:
                updates, slots, inverse, pages, scale = writer_inputs(rows, 1000 * rank + 10 * c + ratio, device)
                cache = torch.zeros(pages, 32, 1, 512, dtype=torch.int8, device=device)
                self.ops.append(PreparedCacheWrite(cache, updates, slots, inverse))
                if c == 0:
                    self.host_sets.append((updates.cpu().pin_memory(), slots.cpu().pin_memory(), updates, slots, scale))
        self.per_step = len(WRITER_ROWS)
        self.rows_per_step = sum(r for r, _ in WRITER_ROWS)
        for op in self.ops:
            op.run()
        torch.cuda.synchronize(device)
        self.step_graphs = [capture(device, lambda c=c: self.step(c)) for c in range(copies)]
        # one step per rotating set in ONE graph, as a serving step holds the writes of all its layers
        self.round_graph = capture(device, lambda: [self.step(c) for c in range(copies)])
        self.size_graphs = [capture(device, lambda k=k: [self.ops[c * self.per_step + k].run() for c in range(copies)])
                            for k in range(self.per_step)]
        for g in self.step_graphs + self.size_graphs + [self.round_graph]:
            g.replay()
        torch.cuda.synchronize(device)

    def step(self, i):
        for k in range(self.per_step):
            self.ops[(i % self.copies) * self.per_step + k].run()

    def measure(self, seconds):
        """Step time from replays of the step graphs for about `seconds`; per launch size from replays
        of the per-size graphs.  Returns a dict of figures (device time, one rank)."""
        peak, peak_kind = measured_peaks()
        probe_a, probe_b = timed(lambda i: self.round_graph.replay(), 2)
        torch.cuda.synchronize(self.device)
        rounds = max(2, int(seconds * 1000 / max(probe_a.elapsed_time(probe_b) / 2, 1e-3)))
        a, b = timed(lambda i: self.round_graph.replay(), rounds)
        torch.cuda.synchronize(self.device)
        steps = rounds * self.copies
        step_ms = a.elapsed_time(b) / steps
        sizes = {}
        for k, (rows, _) in enumerate(WRITER_ROWS):
            reps = max(4, rounds // 4)
            a, b = timed(lambda i, k=k: self.size_graphs[k].replay(), reps)
            torch.cuda.synchronize(self.device)
            ms = a.elapsed_time(b) / (reps * self.copies)
            sizes[f"{rows}_rows"] = {"ms_per_launch": ms, "gbs": rows * 1536 / 1e6 / ms, "frac": rows * 1536 / 1e6 / ms / peak}
        gbs = self.rows_per_step * 1536 / 1e6 / step_ms
        return {"rows_per_s": self.rows_per_step / (step_ms / 1000), "unit": "rows/s", "ms_per_step": step_ms, "steps_timed": steps,
                "gbs": gbs, "peak": peak, "peak_source": peak_kind, "frac": gbs / peak, "bound": "hbm",
                "algorithmic_bytes_per_step": self.rows_per_step * 1536, "launches_per_step": self.per_step,
                "per_launch": sizes, "kernel": "cache_write_vec",
                "workload": "65536 BF16 rows -> original cache + 16384 rows -> ratio-4 compressed cache, random slots",
                "l2": f"{self.copies} rotating sets of rows and caches ({self.copies * self.rows_per_step * 1536 / 1e6:.0f} MB)"}


def run_writer(args, rank, world, local):
    torch.cuda.set_device(local)
    device = torch.device("cuda", local)
    if world > 1:
        import torch.distributed as dist
        dist.init_process_group("nccl", device_id=device)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    bench = WriterBench(device, rank, max(2, args.rotate))
    for i in range(args.warmup):
        bench.step_graphs[i % bench.copies].replay()
    barrier()
    sampler = ClockSampler(local) if rank == 0 else None
    begin, finish = timed((lambda i: bench.step(i)) if args.no_graph else (lambda i: bench.step_graphs[i % bench.copies].replay()),
                          args.steps)
    barrier()
    detail = bench.measure(1.0)
    clocks = sampler.stop() if sampler else None
    total_ms, counts = combine_ranks(begin.elapsed_time(finish), [bench.rows_per_step * args.steps], device, world)
    value = counts[0] / (total_ms / 1000)

    # end to end: rows and slots come from pinned host memory every step; a 64-byte probe of the cache goes back
    probe = torch.empty(64, dtype=torch.int8).pin_memory()

    def e2e_step(_):
        for k, (host_rows, host_slots, dev_rows, dev_slots, _) in enumerate(bench.host_sets):
            dev_rows.copy_(host_rows, non_blocking=True)
            dev_slots.copy_(host_slots, non_blocking=True)
            bench.ops[k].run()
        probe.copy_(bench.ops[0].cache.view(-1)[:64], non_blocking=True)
    for i in range(3):
        e2e_step(i)
    barrier()
    t0, t1 = timed(e2e_step, args.steps)
    barrier()
    e2e_ms, _ = combine_ranks(t0.elapsed_time(t1), [0], device, world)
    if rank != 0:
        if world > 1:
            dist.destroy_process_group()
        return
    from oracle import sharedkv_oracle as oracle
    torch.set_num_threads(os.cpu_count() or 1)
    host_rows, host_slots, _, _, scale = bench.host_sets[0]
    cpu_cache = torch.zeros(bench.ops[0].cache.shape, dtype=torch.int8)
    cpu_rows, spent = 0, 0.0
    while spent < max(args.cpu_seconds, 0.5):
        start = time.perf_counter()
        oracle.write_cache(cpu_cache, host_rows[:8192], host_slots[:8192].long(), scale.double().reciprocal().float())
        spent += time.perf_counter() - start
        cpu_rows += 8192
    peak, peak_kind = measured_peaks()
    achieved = value / world * 1536 / 1e9
    print(json.dumps({
        "metric": WRITER_METRIC, "value": value, "unit": "rows/s", "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": total_ms / args.steps, "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "int8",
        "data": "synthetic",
        "config": {"workload": workload_label(args), "rows_per_step_per_gpu": bench.rows_per_step,
                   "launch": "host launches" if args.no_graph else "CUDA graph replay of one step", "l2": detail["l2"]},
        "roofline": {"bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s", "frac": achieved / peak, "traffic": None,
                     "peak_source": peak_kind, "ms_per_launch": total_ms / args.steps / bench.per_step,
                     "algorithmic_bytes_per_launch": bench.rows_per_step * 1536 // bench.per_step, "kernel": "cache_write_vec"},
        "sustained": detail,
        "cpu_baseline": {"value": cpu_rows / spent, "unit": "rows/s", "cores": os.cpu_count() or 1, "kind": "port",
                         "sample": f"{cpu_rows} rows in calls of 8192"},
        "e2e": {"value": counts[0] / (e2e_ms / 1000), "unit": "rows/s",
                "h2d_bytes_per_step": sum(h.numel() * 2 + sl.numel() * 4 for h, sl, _, _, _ in bench.host_sets), "d2h_bytes_per_step": 64},
        "gpu_launches": bench.per_step * args.steps, "clocks": clocks}))
    if world > 1:
        dist.destroy_process_group()


# --------------------------------------------------------------------------- reference arm
def run_reference(args, rank, world):
    if rank != 0:
        return
    threads = os.cpu_count() or 1
    lengths = box_lengths(args.requests) if args.workload == "box" else None
    if args.workload == "c128":
        from npu_sparse_attn_sharedkv_int8.synthetic import uniform_lengths
        lengths, ratios = uniform_lengths(64, 8192, 131072, seed=1), [128]
    elif args.workload == "c4mtp":
        from npu_sparse_attn_sharedkv_int8.synthetic import uniform_lengths
        lengths, ratios = uniform_lengths(256, 32768, 131072, seed=2), [4]
    else:
        ratios = [4, 128]
    per_step = max(0.25, min(20.0, 120.0 / max(1, args.steps + args.warmup)))      # about two minutes in all
    for _ in range(args.warmup):
        time_cpu_path(lengths, ratios, per_step / 4, threads)
    rates, row_rates, counted, kind = [], [], 0, "port"
    start = time.perf_counter()
    for _ in range(args.steps):
        qps, rps, n, kind = time_cpu_path(lengths, ratios, per_step, threads)
        rates.append(qps); row_rates.append(rps); counted += n
    elapsed = time.perf_counter() - start
    value = statistics.mean(rates)
    what = ("the reference's tiled_quantized_reference (tile 128, one running state)" if kind == "reference"
            else "the CPU restatement of the reference path (reference file not installed)")
    sample = (f"{counted} queries in {args.steps} steps through {what}, batches of 8 requests per layer kind drawn from the "
              "workload's length distribution")
    print(json.dumps({
        "impl": "reference", "metric": METRIC, "value": value, "unit": "queries/s", "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": 1000 * elapsed / max(1, args.steps),
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "int8", "data": "synthetic",
        "config": {"workload": workload_label(args), "requests": args.requests},
        "kv_gbs": statistics.mean(row_rates) * ROW_BYTES / 1e9,
        "cpu_baseline": {"value": value, "unit": "queries/s", "cores": threads, "kind": kind, "sample": sample},
        "e2e": {"value": value, "unit": "queries/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0}))


# --------------------------------------------------------------------------- host-buffer path
class HostBufferStep:
    """One decode pass through the prepared operators with inputs in pinned host memory.

    Per layer one staging buffer holds everything the layer's launches read that changes from step
    to step: Q [tokens, 8, 512] BF16, the new KV row of every request [tokens, 512] BF16 and, for a
    C4 layer, the top-k selections [tokens, 1024] INT32.  It crosses PCIe as ONE copy; the device
    side of it is what the operators are bound to.  Three streams: the inputs of layer i + 1 go in
    while layer i computes and layer i - 1's output goes back.  `kernels=False` leaves the writer
    and attention launches out (same copies, same events): the ceiling the copies alone set."""

    def __init__(self, work, device, affinity_index):
        from dataclasses import replace
        from npu_sparse_attn_sharedkv_int8 import PreparedAttention, PreparedCacheWrite
        self.work, self.device = work, device
        tokens, layers = work.tokens, len(work.layers)
        self.layers = layers
        q_bytes, row_bytes, idx_bytes = tokens * 8 * 512 * 2, tokens * 512 * 2, tokens * 1024 * 4
        # the new token of request b lands in the last row of its window: logical row seq_len - 1
        last = work.seq_lens_host - 1
        slot_pages = work.ori_table[torch.arange(work.requests, device=device), (last // 32).to(device)].long()
        slots = (slot_pages * 32 + (last % 32).to(device)).to(torch.int32).repeat_interleave(work.queries)
        self.stage, self.ops, self.writers, self.bytes_in = [], [], [], []
        for i, layer in enumerate(work.layers):
            size = q_bytes + row_bytes + (idx_bytes if layer.cmp_indices is not None else 0)
            stage = torch.empty(size, dtype=torch.uint8, device=device)
            q = stage[:q_bytes].view(torch.bfloat16).view(tokens, 8, 512)
            rows = stage[q_bytes:q_bytes + row_bytes].view(torch.bfloat16).view(tokens, 512)
            picks = stage[q_bytes + row_bytes:].view(torch.int32).view(tokens, 1, 1024) if layer.cmp_indices is not None else None
            self.stage.append(stage)
            self.bytes_in.append(size)
            self.ops.append(PreparedAttention(replace(work.case(i), q=q, cmp_indices=picks), layer.ori_scale, layer.cmp_scale))
            self.writers.append(PreparedCacheWrite(layer.ori, rows, slots, layer.ori_scale.double().reciprocal().float()))
        with HostMemoryNear(affinity_index):
            self.host_in = {}
            for i, layer in enumerate(work.layers):
                key = (self.bytes_in[i], i % 4)                        # a few distinct host buffers per size
                if key not in self.host_in:
                    host = torch.empty(self.bytes_in[i], dtype=torch.uint8).pin_memory()
                    host[:q_bytes].view(torch.bfloat16).copy_(torch.randn(tokens * 8 * 512).bfloat16())
                    host[q_bytes:q_bytes + row_bytes].view(torch.bfloat16).copy_(torch.randn(tokens * 512).bfloat16())
                    if layer.cmp_indices is not None:
                        host[q_bytes + row_bytes:].view(torch.int32).copy_(layer.cmp_indices.view(-1).cpu())
                    self.host_in[key] = host
            self.host_out = [torch.empty(tokens, 8, 512, dtype=torch.bfloat16).pin_memory() for _ in range(2)]
        self.copy_in, self.copy_out = torch.cuda.Stream(device), torch.cuda.Stream(device)
        self.staged = [torch.cuda.Event() for _ in range(layers)]
        self.computed = [torch.cuda.Event() for _ in range(layers)]
        self.returned = [torch.cuda.Event() for _ in range(layers)]
        self.used = [False] * layers
        self.h2d_per_pass = sum(self.bytes_in)
        self.d2h_per_pass = layers * tokens * 8 * 512 * 2

    def layer(self, i, slot, kernels):
        main = torch.cuda.current_stream(self.device)
        with torch.cuda.stream(self.copy_in):
            if self.used[i]:
                self.copy_in.wait_event(self.computed[i])           # the previous use of this layer's inputs is over
            self.stage[i].copy_(self.host_in[(self.bytes_in[i], i % 4)], non_blocking=True)
            self.staged[i].record(self.copy_in)
        main.wait_event(self.staged[i])
        if self.used[i]:
            main.wait_event(self.returned[i])                       # the previous output of this layer has been read
        if kernels:
            self.writers[i].run()
            self.ops[i].run()
        self.computed[i].record(main)
        with torch.cuda.stream(self.copy_out):
            self.copy_out.wait_event(self.computed[i])
            self.host_out[slot].copy_(self.ops[i].out, non_blocking=True)
            self.returned[i].record(self.copy_out)
        self.used[i] = True

    def run_pass(self, which, kernels=True):
        main = torch.cuda.current_stream(self.device)
        if torch.cuda.is_current_stream_capturing():      # a captured pass forks its copy streams from the capture stream
            self.copy_in.wait_stream(main)
            self.copy_out.wait_stream(main)
        for n, i in enumerate(which):
            self.layer(i, n & 1, kernels)
        main.wait_stream(self.copy_in)
        main.wait_stream(self.copy_out)                   # the pass ends when its last result is on the host


# --------------------------------------------------------------------------- main
def main():
    parser = argparse.ArgumentParser()
    parser.add_argument("--gpus", type=int, default=1)
    parser.add_argument("--steps", type=int, default=20)
    parser.add_argument("--warmup", type=int, default=3)
    parser.add_argument("--impl", default="b200", choices=("b200", "reference"))
    parser.add_argument("--workload", default="box", choices=("box", "c128", "c4mtp", "writer"))
    parser.add_argument("--requests", type=int, default=2048)
    parser.add_argument("--kv-gb", type=float, default=150.0)
    parser.add_argument("--max-pairs", type=int, default=0)
    parser.add_argument("--layers", default="pair", choices=("pair", "c4", "c128"),
                        help="box workload: layer kinds per pair (one kind keeps a profiler capture small)")
    parser.add_argument("--rotate", type=int, default=8, help="cache copies rotated through by the small workloads")
    parser.add_argument("--queries", type=int, default=1, help="query tokens per request of the c128 workload (chunked-prefill shapes)")
    parser.add_argument("--query-group", type=int, default=1, choices=(1, 2, 4),
                        help="2 or 4: the c128 workload runs the paired-query kernel (two adjacent tokens of a request per work "
                             "item; 4: two such items on the tiling of four tokens)")
    parser.add_argument("--passes", type=int, default=0,
                        help="decode passes per step; 0 = as many as make the timed steps last --seconds")
    parser.add_argument("--seconds", type=float, default=2.5, help="length aimed at for the timed region when --passes is 0")
    parser.add_argument("--cpu-seconds", type=float, default=12.0)
    parser.add_argument("--no-e2e", action="store_true")
    parser.add_argument("--no-writer", action="store_true", help="leave the cache-writer block out of the decode line")
    parser.add_argument("--e2e-graph", action="store_true", help="replay a captured pass in the host-buffer measurement too")
    parser.add_argument("--no-host-affinity", action="store_true", help="allocate host buffers without moving next to the GPU")
    parser.add_argument("--no-graph", action="store_true", help="launch every layer from the host instead of replaying a captured pass")
    args = parser.parse_args()
    rank, world = int(os.environ.get("RANK", 0)), int(os.environ.get("WORLD_SIZE", 1))
    local = int(os.environ.get("LOCAL_RANK", 0))
    if args.impl == "reference":
        run_reference(args, rank, world)
        return
    if args.warmup < 3:
        args.warmup = 3
    if args.workload == "writer":
        run_writer(args, rank, world, local)
        return

    import torch.distributed as dist
    from npu_sparse_attn_sharedkv_int8 import PreparedAttention
    torch.cuda.set_device(local)
    device = torch.device("cuda", local)
    if world > 1:
        dist.init_process_group("nccl", device_id=device)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    work, label = build_workload(args, rank, world)
    layers = len(work.layers)
    grouping = {"query_group": args.query_group} if args.query_group > 1 and args.workload == "c128" else {}
    ops = [PreparedAttention(work.case(i), work.layers[i].ori_scale, work.layers[i].cmp_scale, **grouping) for i in range(layers)]
    rows_per_layer = [work.kv_rows(i) for i in range(layers)]
    # a pass: every resident layer once (box), or one launch on the next of the rotating copies (single-layer workloads)
    pass_layers = [list(range(layers))] if args.workload == "box" else [[i] for i in range(layers)]
    queries_per_pass = work.tokens * len(pass_layers[0])
    launches_per_pass = len(pass_layers[0])

    def run_pass(index):
        for i in pass_layers[index % len(pass_layers)]:
            ops[i].run()

    # ---- resident-in-HBM timing.  The serving stack of the reference replays captured decode steps,
    # so a pass is captured once and replayed.
    for i in range(args.warmup):
        run_pass(i)
    torch.cuda.synchronize()
    if args.no_graph:
        replay = run_pass
    else:
        pass_graphs = [capture(device, lambda k=k: run_pass(k)) for k in range(len(pass_layers))]
        replay = lambda index: pass_graphs[index % len(pass_graphs)].replay()
    for i in range(args.warmup):
        replay(i)
    barrier()
    # burst: K single passes from idle clocks
    sampler = ClockSampler(local) if rank == 0 else None
    begin, finish = timed(replay, args.steps)
    barrier()
    burst_clocks = sampler.stop() if sampler else None
    burst_ms = begin.elapsed_time(finish)
    # sustained: K steps of `passes` passes each
    passes = args.passes
    if passes <= 0:
        local_pass_ms = torch.tensor([burst_ms / args.steps], dtype=torch.float64, device=device)
        if world > 1:
            dist.all_reduce(local_pass_ms, op=dist.ReduceOp.MAX)      # every rank must time the same number of passes
        passes = max(1, math.ceil(args.seconds * 1000 / (args.steps * float(local_pass_ms[0]))))
    sampler = ClockSampler(local) if rank == 0 else None
    begin, finish = timed(replay, args.steps * passes)
    barrier()
    elapsed_ms = begin.elapsed_time(finish)
    # per layer kind, at the clocks the sustained region left: replays of a graph that holds the
    # launches of one kind back to back, CUDA events around every replay
    kinds = sorted({work.layers[i].ratio for i in range(layers)})
    by_kind = {r: [i for i in range(layers) if work.layers[i].ratio == r] for r in kinds}
    kind_graphs = {r: (None if args.no_graph else capture(device, lambda r=r: [ops[i].run() for i in by_kind[r]])) for r in kinds}
    rounds = max(4, min(200, int(500 / max(elapsed_ms / (args.steps * passes), 1e-3))))      # about half a second
    marks = []
    for _ in range(rounds):
        for r in kinds:
            a, b = timed((lambda _i, r=r: kind_graphs[r].replay()) if kind_graphs[r] is not None
                         else (lambda _i, r=r: [ops[i].run() for i in by_kind[r]]), 1)
            marks.append((r, a, b))
    barrier()
    clocks = sampler.stop() if sampler else None
    per_kind = {}
    for r, a, b in marks:
        entry = per_kind.setdefault(r, [0.0, 0, 0])
        entry[0] += a.elapsed_time(b); entry[1] += len(by_kind[r]); entry[2] += sum(rows_per_layer[i] for i in by_kind[r])
    rows_per_pass = sum(rows_per_layer[i] for i in pass_layers[0])
    total_ms, counts = combine_ranks(elapsed_ms, [queries_per_pass * passes * args.steps, rows_per_pass * passes * args.steps],
                                     device, world)
    burst_total_ms, burst_counts = combine_ranks(burst_ms, [queries_per_pass * args.steps], device, world)
    value = counts[0] / (total_ms / 1000)
    kv_gbs = counts[1] * ROW_BYTES / 1e9 / (total_ms / 1000)

    # ---- the cache writer at its own configuration (rank 0's device time; every rank runs it)
    writer = None
    if not args.no_writer:
        writer_bench = WriterBench(device, rank, 4)
        barrier()
        writer = writer_bench.measure(0.5)
        del writer_bench
        barrier()

    # ---- end to end through the prepared operators with host buffers
    e2e = None
    if not args.no_e2e:
        host = HostBufferStep(work, device, -1 if args.no_host_affinity else local)

        def measure(kernels, use_graph):
            host.used[:] = [False] * layers
            for k in range(min(3, len(pass_layers)) if len(pass_layers) > 1 else 3):
                host.run_pass(pass_layers[k % len(pass_layers)], kernels)
            torch.cuda.synchronize()
            run = lambda index: host.run_pass(pass_layers[index % len(pass_layers)], kernels)
            if use_graph:
                graphs = []
                for k in range(len(pass_layers)):
                    host.used[:] = [False] * layers           # replays are ordered by the stream; no cross-pass events
                    graphs.append(capture(device, lambda k=k: host.run_pass(pass_layers[k], kernels)))
                host.used[:] = [False] * layers
                run = lambda index: graphs[index % len(graphs)].replay()
                run(0)
            barrier()
            t0, t1 = timed(run, args.steps * passes)
            barrier()
            ms, _ = combine_ranks(max(t0.elapsed_time(t1), 0.0), [0], device, world)
            return ms

        # Host launches by default: replays of a captured pass do not overlap one pass's last copies
        # with the next pass's first ones, which host launches do.
        e2e_ms = measure(True, args.e2e_graph)
        copy_ms = measure(False, args.e2e_graph)
        h2d = host.h2d_per_pass * len(pass_layers[0]) // layers if args.workload != "box" else host.h2d_per_pass
        d2h = host.d2h_per_pass * len(pass_layers[0]) // layers
        per_pass_s = e2e_ms / 1000 / (args.steps * passes)
        copy_pass_s = copy_ms / 1000 / (args.steps * passes)
        e2e = {"value": counts[0] / (e2e_ms / 1000), "unit": "queries/s",
               "h2d_bytes_per_step": h2d * passes, "d2h_bytes_per_step": d2h * passes,
               "ms_per_step": e2e_ms / args.steps, "ms_per_pass": per_pass_s * 1000,
               "h2d_gbs_per_gpu": h2d / 1e9 / per_pass_s, "d2h_gbs_per_gpu": d2h / 1e9 / per_pass_s,
               "copies_per_layer": "one host-to-device (Q + new KV rows + top-k selections in one pinned staging buffer), one device-to-host (output)",
               "copy_only": {"ms_per_pass": copy_pass_s * 1000, "h2d_gbs_per_gpu": h2d / 1e9 / copy_pass_s,
                             "d2h_gbs_per_gpu": d2h / 1e9 / copy_pass_s, "value": counts[0] / (copy_ms / 1000),
                             "what": "the same pass with the writer and attention launches left out"},
               "fraction_of_copy_only": copy_ms / e2e_ms,
               "launch": "CUDA graph replay of one pass (copies included)" if args.e2e_graph else "host launches on three streams"}

    if rank != 0:
        if world > 1:
            dist.destroy_process_group()
        return
    peak, peak_kind = measured_peaks()
    roof = {}
    for ratio, (ms, launches, rows) in per_kind.items():
        achieved = rows * ROW_BYTES / 1e9 / (ms / 1000)
        roof[ratio] = {"bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s", "frac": achieved / peak,
                       "traffic": int(TRAFFIC_PER_ALGORITHMIC_BYTE[ratio] * rows * ROW_BYTES // launches),
                       "traffic_source": "profiler capture of a smaller launch, scaled by algorithmic bytes",
                       "peak_source": peak_kind, "ms_per_launch": ms / launches,
                       "algorithmic_bytes_per_launch": rows * ROW_BYTES // launches, "launches": launches,
                       "timing": "CUDA events around replays of a graph holding this kind's launches back to back, after the sustained region"}
    dominant = max(per_kind, key=lambda r: per_kind[r][0])
    # the CPU baseline is timed at N = 1 only (under torchrun the host's cores belong to all the ranks)
    cpu_qps, cpu_rows, cpu_n, cpu_kind = time_cpu_path(work.seq_lens_host, [l.ratio for l in work.layers],
                                                       args.cpu_seconds if world == 1 else 0.0, os.cpu_count() or 1)
    timed_s = total_ms / 1000
    line = {
        "metric": METRIC, "value": value, "unit": "queries/s", "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": total_ms / args.steps, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "int8", "data": "synthetic",
        "config": {"workload": label, "requests": args.requests if args.workload == "box" else work.requests,
                   "requests_on_rank0": work.requests, "layers_per_gpu": layers, "passes_per_step": passes,
                   "queries_per_step_rank0": queries_per_pass * passes, "launches_per_pass": launches_per_pass,
                   "kv_resident_gb_rank0": work.kv_bytes_resident / 1e9,
                   "launch": "host launches" if args.no_graph else "CUDA graph replay of one pass", "l2": "inputs larger than L2 (KV touched per pass >> 126 MB)"
                   if args.workload != "c128" else f"rotating {layers} cache copies, each launch reads a region not touched for {layers - 1} launches"},
        "timed_region_s": timed_s, "ms_per_pass": total_ms / (args.steps * passes),
        "per_gpu_value": value / world, "kv_gbs": kv_gbs, "kv_gbs_per_gpu": kv_gbs / world,
        "burst": {"value": burst_counts[0] / (burst_total_ms / 1000), "ms_per_pass": burst_total_ms / args.steps, "passes": args.steps,
                  "clocks": clock_note(burst_clocks, burst_total_ms / args.steps)},
        "roofline": dict(roof[dominant], kernel=f"decode_kernel on C{dominant} layers"),
        "roofline_other": {f"decode_kernel on C{r} layers": v for r, v in roof.items() if r != dominant},
        "writer": writer,
        "cpu_baseline": None if not cpu_n else {
            "value": cpu_qps, "unit": "queries/s", "cores": os.cpu_count() or 1, "kind": cpu_kind,
            "sample": f"{cpu_n} queries, batches of 8 requests per layer kind drawn from rank 0's requests",
            "kv_gbs": cpu_rows * ROW_BYTES / 1e9},
        "e2e": e2e, "gpu_launches": launches_per_pass * passes * args.steps,
        "clocks": clock_note(clocks, total_ms / (args.steps * passes)),
    }
    print(json.dumps(line))
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
