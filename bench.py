"""Benchmark of the INT8 shared-KV decode path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl b200|reference] [--workload box|c128|c4mtp|writer]

Default workload ("box"): the box-scale decode step.  2048 concurrent requests with context
lengths log-uniform over 4k..1M tokens are batch-sharded over the N GPUs (longest-first
greedy by KV rows); every GPU holds the INT8 paged KV of its requests for alternating
C4 (top-k 1024 + window 128) and C128 (all compressed rows + window 128) layers, as many
layer pairs as fill about --kv-gb of its HBM.  A step is one decode pass of the hot path
over all resident layers: one attention launch per layer, T = 1 query token per request.
There is no collective on the path; ranks only meet at the timing barriers.

Printed JSON line (rank 0): `value` = (request, layer) attention evaluations per second
over all GPUs with everything resident in HBM; `e2e` = the same through the prepared
operators with host buffers: per step and layer the new KV row of every request, Q and
(C4) the top-k selections are copied from pinned host memory, the cache writer and the
attention run, and the BF16 output is copied back (three streams, so copies overlap compute).
`roofline` is for the layer kind with the larger share of the step (`roofline_other` for the
other): algorithmic KV bytes per launch over its mean CUDA-event duration (the call's memset included).
`--workload writer` times the paged cache writer instead (65 536 rows into the original cache and
16 384 into the ratio-4 compressed cache per step) and prints rows/s.
`--impl reference` times the CPU restatement of the reference's Python path (the reference
itself is Python and does not travel to the GPU box) on a bounded seeded sample.
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
# DRAM traffic (read + written) per algorithmic KV byte, from ncu captures of smaller launches of the
# same kernels (profiles/decode_kernel_*.md); traffic grows in proportion to the queries processed.
TRAFFIC_PER_ALGORITHMIC_BYTE = {4: 1.076, 128: 1.040}


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
            "c128": "C128 decode, B=64, T=1, ctx U[8k,128k], compact pages (stride 38 x 16384 B, offset 16384 B)",
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
        work = synthetic.build("c128", device, lengths, ratios=ratios, queries=1, seed=200 + rank, stride_slots=38,
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


# --------------------------------------------------------------------------- CPU path (oracle port of the reference)
def cpu_sample_case(ratio, lengths, seed):
    """Small CPU case with the shapes of the workload's requests: every request carries the
    rows it attends to (C4: 1024 selected rows + window; C128: all compressed rows + window)."""
    from npu_sparse_attn_sharedkv_int8.reference import SharedKVCase
    g = torch.Generator().manual_seed(seed)
    batch = len(lengths)
    new_lengths, ori_pages, cmp_pages = [], [], []
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


def time_cpu_path(lengths, ratios, budget_s, threads):
    """Runs the CPU restatement of the reference path on batches of 8 requests per layer kind
    until about `budget_s` seconds are spent.  Returns (queries/s, rows/s, queries timed)."""
    from oracle import sharedkv_oracle as oracle
    torch.set_num_threads(threads)
    scale = torch.full((512,), 0.02)
    g = torch.Generator().manual_seed(7)
    kinds = sorted(set(ratios))
    done, rows, spent = 0, 0, 0.0
    if budget_s <= 0:
        return None, None, 0
    oracle.attention_tiled(cpu_sample_case(kinds[0], [4096] * 2, 1), scale, scale)     # warm the thread pool
    while spent < budget_s:
        for ratio in kinds:
            pick = lengths[torch.randint(len(lengths), (8,), generator=g)].tolist()
            case = cpu_sample_case(ratio, pick, seed=done)
            start = time.perf_counter()
            oracle.attention_tiled(case, scale, scale)
            spent += time.perf_counter() - start
            done += len(pick)
            rows += oracle.kv_rows_attended(case)
    return done / spent, rows / spent, done


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


def run_writer(args, rank, world, local):
    from npu_sparse_attn_sharedkv_int8 import PreparedCacheWrite
    torch.cuda.set_device(local)
    device = torch.device("cuda", local)
    if world > 1:
        import torch.distributed as dist
        dist.init_process_group("nccl", device_id=device)
    copies = max(2, args.rotate)              # each launch touches buffers the previous `copies - 1` did not: > L2 in all
    ops, host_sets = [], []
    for c in range(copies):
        for rows, ratio in WRITER_ROWS:
            updates, slots, inverse, pages, scale = writer_inputs(rows, 1000 * rank + 10 * c + ratio, device)
            cache = torch.zeros(pages, 32, 1, 512, dtype=torch.int8, device=device)
            ops.append((PreparedCacheWrite(cache, updates, slots, inverse), rows))
            if c == 0:
                host_sets.append((updates.cpu().pin_memory(), slots.cpu().pin_memory(), updates, slots, scale))
    per_step = len(WRITER_ROWS)

    def step(i):
        for k in range(per_step):
            ops[(i % copies) * per_step + k][0].run()

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    for i in range(args.warmup):
        step(i)
    torch.cuda.synchronize()
    graphs = None
    if not args.no_graph:                     # one captured step per rotating set, replayed
        side = torch.cuda.Stream(device)
        side.wait_stream(torch.cuda.current_stream(device))
        graphs = []
        with torch.cuda.stream(side):
            for c in range(copies):
                g = torch.cuda.CUDAGraph()
                with torch.cuda.graph(g, stream=side):
                    step(c)
                graphs.append(g)
        torch.cuda.current_stream(device).wait_stream(side)
        for c in range(copies):
            graphs[c].replay()
    barrier()
    sampler = ClockSampler(local) if rank == 0 else None
    begin, finish = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    begin.record()
    for i in range(args.steps):
        if graphs is not None:
            graphs[i % copies].replay()
        else:
            step(i)
    finish.record()
    barrier()
    clocks = sampler.stop() if sampler else None
    rows_per_step = sum(r for r, _ in WRITER_ROWS)
    total_ms, counts = combine_ranks(begin.elapsed_time(finish), [rows_per_step * args.steps], device, world)
    value = counts[0] / (total_ms / 1000)

    # end to end: rows and slots come from pinned host memory every step; a 64-byte probe of the cache goes back
    probe = torch.empty(64, dtype=torch.int8).pin_memory()
    def e2e_step():
        for k, (host_rows, host_slots, dev_rows, dev_slots, _) in enumerate(host_sets):
            dev_rows.copy_(host_rows, non_blocking=True)
            dev_slots.copy_(host_slots, non_blocking=True)
            ops[k][0].run()
        probe.copy_(ops[0][0].cache.view(-1)[:64], non_blocking=True)
    for _ in range(3):
        e2e_step()
    barrier()
    t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    t0.record()
    for _ in range(args.steps):
        e2e_step()
    t1.record()
    barrier()
    e2e_ms, _ = combine_ranks(t0.elapsed_time(t1), [0], device, world)
    if rank != 0:
        if world > 1:
            dist.destroy_process_group()
        return
    from oracle import sharedkv_oracle as oracle
    torch.set_num_threads(os.cpu_count() or 1)
    host_rows, host_slots, _, _, scale = host_sets[0]
    cpu_cache = torch.zeros(ops[0][0].cache.shape, dtype=torch.int8)
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
        "config": {"workload": workload_label(args), "rows_per_step_per_gpu": rows_per_step,
                   "launch": "host launches" if args.no_graph else "CUDA graph replay of one step",
                   "l2": f"rotating {copies} sets of rows and caches ({copies * rows_per_step * 1536 / 1e6:.0f} MB) so no launch finds its data in L2"},
        "roofline": {"bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s", "frac": achieved / peak, "traffic": None,
                     "peak_source": peak_kind, "ms_per_launch": total_ms / args.steps / per_step,
                     "algorithmic_bytes_per_launch": rows_per_step * 1536 // per_step, "kernel": "cache_write_kernel"},
        "cpu_baseline": {"value": cpu_rows / spent, "unit": "rows/s", "cores": os.cpu_count() or 1, "kind": "port",
                         "sample": f"{cpu_rows} rows in calls of 8192"},
        "e2e": {"value": counts[0] / (e2e_ms / 1000), "unit": "rows/s",
                "h2d_bytes_per_step": sum(h.numel() * 2 + sl.numel() * 4 for h, sl, _, _, _ in host_sets), "d2h_bytes_per_step": 64},
        "gpu_launches": per_step * args.steps, "clocks": clocks}))
    if world > 1:
        dist.destroy_process_group()


# --------------------------------------------------------------------------- main
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
    rates, row_rates, counted = [], [], 0
    start = time.perf_counter()
    for _ in range(args.steps):
        qps, rps, n = time_cpu_path(lengths, ratios, per_step, threads)
        rates.append(qps); row_rates.append(rps); counted += n
    elapsed = time.perf_counter() - start
    value = statistics.mean(rates)
    sample = f"{counted} queries in {args.steps} steps, batches of 8 requests per layer kind drawn from the workload's length distribution"
    print(json.dumps({
        "impl": "reference", "metric": METRIC, "value": value, "unit": "queries/s", "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": 1000 * elapsed / max(1, args.steps),
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "int8", "data": "synthetic",
        "config": {"workload": workload_label(args), "requests": args.requests},
        "kv_gbs": statistics.mean(row_rates) * ROW_BYTES / 1e9,
        "cpu_baseline": {"value": value, "unit": "queries/s", "cores": threads, "kind": "port", "sample": sample},
        "e2e": {"value": value, "unit": "queries/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0}))


def main():
    parser = argparse.ArgumentParser()
    parser.add_argument("--gpus", type=int, default=1)
    parser.add_argument("--steps", type=int, default=200)
    parser.add_argument("--warmup", type=int, default=3)
    parser.add_argument("--impl", default="b200", choices=("b200", "reference"))
    parser.add_argument("--workload", default="box", choices=("box", "c128", "c4mtp", "writer"))
    parser.add_argument("--requests", type=int, default=2048)
    parser.add_argument("--kv-gb", type=float, default=150.0)
    parser.add_argument("--max-pairs", type=int, default=0)
    parser.add_argument("--layers", default="pair", choices=("pair", "c4", "c128"),
                        help="box workload: layer kinds per pair (one kind keeps a profiler capture small)")
    parser.add_argument("--rotate", type=int, default=8, help="cache copies rotated through by the small workloads")
    parser.add_argument("--cpu-seconds", type=float, default=12.0)
    parser.add_argument("--no-e2e", action="store_true")
    parser.add_argument("--e2e-graph", action="store_true", help="replay a captured step in the host-buffer measurement too")
    parser.add_argument("--no-host-affinity", action="store_true", help="allocate host buffers without moving next to the GPU")
    parser.add_argument("--no-graph", action="store_true", help="launch every layer from the host instead of replaying a captured step")
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
    from npu_sparse_attn_sharedkv_int8 import PreparedAttention, PreparedCacheWrite
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
    ops = [PreparedAttention(work.case(i), work.layers[i].ori_scale, work.layers[i].cmp_scale) for i in range(layers)]
    rows_per_layer = [work.kv_rows(i) for i in range(layers)]
    queries_per_step = work.tokens * layers if args.workload == "box" else work.tokens
    sequence = list(range(layers)) if args.workload == "box" else None

    def step(index):
        if sequence is not None:
            for i in sequence:
                ops[i].run()
        else:
            ops[index % layers].run()

    # ---- resident-in-HBM timing: K replays of a CUDA graph that holds one step (the serving stack
    # of the reference replays captured decode steps too), then the same K steps launched one by
    # one with events around every layer for the per-kernel roofline figures
    for i in range(args.warmup):
        step(i)
    torch.cuda.synchronize()
    graphs = None
    if not args.no_graph:
        side = torch.cuda.Stream(device)
        side.wait_stream(torch.cuda.current_stream(device))
        graphs = []
        with torch.cuda.stream(side):
            for i in range(1 if sequence is not None else layers):
                g = torch.cuda.CUDAGraph()
                with torch.cuda.graph(g, stream=side):
                    step(i)
                graphs.append(g)
        torch.cuda.current_stream(device).wait_stream(side)
        for i in range(args.warmup):
            graphs[i % len(graphs)].replay()
    barrier()
    sampler = ClockSampler(local) if rank == 0 else None
    begin, finish = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    begin.record()
    for i in range(args.steps):
        if graphs is not None:
            graphs[i % len(graphs)].replay()
        else:
            step(i)
    finish.record()
    barrier()
    elapsed_ms = begin.elapsed_time(finish)
    marks = []
    for i in range(args.steps):
        which = sequence if sequence is not None else [i % layers]
        for layer in which:
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record(); ops[layer].run(); b.record()
            marks.append((layer, a, b))
    barrier()
    clocks = sampler.stop() if sampler else None
    per_kind = {}
    for layer, a, b in marks:
        ratio = work.layers[layer].ratio
        entry = per_kind.setdefault(ratio, [0.0, 0, 0])
        entry[0] += a.elapsed_time(b); entry[1] += 1; entry[2] += rows_per_layer[layer]
    total_ms, counts = combine_ranks(elapsed_ms, [queries_per_step * args.steps, sum(rows_per_layer[l] for l, _, _ in marks)],
                                     device, world)
    value = counts[0] / (total_ms / 1000)
    kv_gbs = counts[1] * ROW_BYTES / 1e9 / (total_ms / 1000)

    # ---- end to end through the prepared operators with host buffers
    e2e = None
    if not args.no_e2e:
        tokens = work.tokens
        with HostMemoryNear(-1 if args.no_host_affinity else local):
            host_q = [torch.randn(tokens, 8, 512).bfloat16().pin_memory() for _ in range(min(layers, 4))]
            host_rows = torch.randn(tokens, 512).bfloat16().pin_memory()
            host_out = [torch.empty(tokens, 8, 512, dtype=torch.bfloat16).pin_memory() for _ in range(2)]
            host_idx_source = next((l.cmp_indices for l in work.layers if l.cmp_indices is not None), None)
            host_idx_early = host_idx_source.cpu().pin_memory() if host_idx_source is not None else None
        host_idx = None
        # the new token of request b lands in the last row of its window: logical row seq_len - 1
        last = (work.seq_lens_host - 1)
        slot_pages = work.ori_table[torch.arange(work.requests, device=device), (last // 32).to(device)].long()
        slots = (slot_pages * 32 + (last % 32).to(device)).to(torch.int32).repeat_interleave(work.queries)
        writers, dev_rows, h2d, d2h = [], [], 0, 0
        for i in range(layers):
            layer = work.layers[i]
            inverse = layer.ori_scale.double().reciprocal().float()
            dev_rows.append(torch.empty(tokens, 512, dtype=torch.bfloat16, device=device))
            writers.append(PreparedCacheWrite(layer.ori, dev_rows[i], slots, inverse))
            if layer.cmp_indices is not None and host_idx is None:
                host_idx = host_idx_early
        # Three streams: inputs of layer i + 1 cross PCIe while layer i computes and layer i - 1's
        # output goes back.  Every layer owns its device-side Q, rows, indices and output, so the only
        # ordering needed is copy-in -> compute -> copy-out per layer, and "the previous use of this
        # layer's buffers is over" before they are overwritten.
        copy_in, copy_out = torch.cuda.Stream(device), torch.cuda.Stream(device)
        staged = [torch.cuda.Event() for _ in range(layers)]
        computed = [torch.cuda.Event() for _ in range(layers)]
        returned = [torch.cuda.Event() for _ in range(layers)]
        used = [False] * layers

        def e2e_layer(i, slot):
            nonlocal h2d, d2h
            layer = work.layers[i]
            main = torch.cuda.current_stream(device)
            with torch.cuda.stream(copy_in):
                if used[i]:
                    copy_in.wait_event(computed[i])
                layer.q.copy_(host_q[i % len(host_q)], non_blocking=True)
                dev_rows[i].copy_(host_rows, non_blocking=True)
                moved = layer.q.numel() * 2 + dev_rows[i].numel() * 2
                if layer.cmp_indices is not None:
                    layer.cmp_indices.copy_(host_idx, non_blocking=True)
                    moved += host_idx.numel() * 4
                staged[i].record(copy_in)
            main.wait_event(staged[i])
            if used[i]:
                main.wait_event(returned[i])              # the output of the previous step has been read
            writers[i].run()
            out = ops[i].run()
            computed[i].record(main)
            with torch.cuda.stream(copy_out):
                copy_out.wait_event(computed[i])
                host_out[slot].copy_(out, non_blocking=True)
                returned[i].record(copy_out)
            used[i] = True
            h2d += moved
            d2h += out.numel() * 2

        def e2e_step(index):
            main = torch.cuda.current_stream(device)
            if torch.cuda.is_current_stream_capturing():  # a captured step forks its copy streams from the capture stream;
                copy_in.wait_stream(main)                 # launched from the host, the copies of step n + 1 may overlap
                copy_out.wait_stream(main)                # the end of step n (buffers are guarded by the events below)
            which = sequence if sequence is not None else [index % layers]
            for n, i in enumerate(which):
                e2e_layer(i, n & 1)
            main.wait_stream(copy_in)
            main.wait_stream(copy_out)                    # the step ends when its last result is on the host

        for i in range(3):
            e2e_step(i)
        torch.cuda.synchronize()
        # Optionally one step (copies, writer and attention launches of every layer, on the three
        # streams) is captured and replayed.  Off by default: replays do not overlap one step's last
        # copies with the next step's first ones, which host launches do (measured 10 % slower at
        # 1 and 2 GPUs); it pays only when the host cannot issue a step's launches fast enough.
        e2e_graphs = None
        if args.e2e_graph:
            side = torch.cuda.Stream(device)
            side.wait_stream(torch.cuda.current_stream(device))
            e2e_graphs = []
            with torch.cuda.stream(side):
                for i in range(1 if sequence is not None else layers):
                    used[:] = [False] * layers            # replays are ordered by the stream; no cross-step events
                    g = torch.cuda.CUDAGraph()
                    with torch.cuda.graph(g, stream=side):
                        e2e_step(i)
                    e2e_graphs.append(g)
            torch.cuda.current_stream(device).wait_stream(side)
            used[:] = [False] * layers
            for i in range(2):
                e2e_graphs[i % len(e2e_graphs)].replay()

        def e2e_run(index):
            if e2e_graphs is not None:
                e2e_graphs[index % len(e2e_graphs)].replay()
            else:
                e2e_step(index)

        barrier()
        h2d = d2h = 0
        used[:] = [False] * layers
        e2e_step(0)                                       # one eager step only to count the bytes a step moves
        torch.cuda.synchronize()
        h2d_step, d2h_step = h2d, d2h
        barrier()
        t0 = torch.cuda.Event(enable_timing=True); t1 = torch.cuda.Event(enable_timing=True)
        t0.record()
        for i in range(args.steps):
            e2e_run(i)
        t1.record()
        barrier()
        h2d, d2h = h2d_step * args.steps, d2h_step * args.steps
        e2e_ms, _ = combine_ranks(max(t0.elapsed_time(t1), 0.0), [0], device, world)
        e2e = {"value": counts[0] / (e2e_ms / 1000), "unit": "queries/s",
               "h2d_bytes_per_step": h2d // args.steps, "d2h_bytes_per_step": d2h // args.steps,
               "ms_per_step": e2e_ms / args.steps,
               "launch": "CUDA graph replay of one step (copies included)" if args.e2e_graph else "host launches on three streams"}

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
                       "traffic_source": "ncu capture of a smaller launch, scaled by algorithmic bytes",
                       "peak_source": peak_kind, "ms_per_launch": ms / launches,
                       "algorithmic_bytes_per_launch": rows * ROW_BYTES // launches, "launches": launches}
    dominant = max(per_kind, key=lambda r: per_kind[r][0])
    cpu_qps, cpu_rows, cpu_n = time_cpu_path(work.seq_lens_host, [l.ratio for l in work.layers], args.cpu_seconds,
                                             os.cpu_count() or 1)
    line = {
        "metric": METRIC, "value": value, "unit": "queries/s", "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": total_ms / args.steps, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "int8", "data": "synthetic",
        "config": {"workload": label, "requests": args.requests if args.workload == "box" else work.requests,
                   "requests_on_rank0": work.requests, "layers_per_gpu": layers, "queries_per_step_rank0": queries_per_step,
                   "kv_resident_gb_rank0": work.kv_bytes_resident / 1e9,
                   "launch": "host launches" if args.no_graph else "CUDA graph replay of one step", "l2": "inputs larger than L2 (KV touched per step >> 126 MB)"
                   if args.workload != "c128" else f"rotating {layers} cache copies, each launch reads a region not touched for {layers - 1} launches"},
        "per_gpu_value": value / world, "kv_gbs": kv_gbs, "kv_gbs_per_gpu": kv_gbs / world,
        "roofline": dict(roof[dominant], kernel=f"decode_kernel<{dominant}> (+ the memset in front of it)"),
        "roofline_other": {f"decode_kernel<{r}>": v for r, v in roof.items() if r != dominant},
        "cpu_baseline": None if not cpu_n else {
            "value": cpu_qps, "unit": "queries/s", "cores": os.cpu_count() or 1, "kind": "port",
            "sample": f"{cpu_n} queries, batches of 8 requests per layer kind drawn from rank 0's requests",
            "kv_gbs": cpu_rows * ROW_BYTES / 1e9},
        "e2e": e2e, "gpu_launches": len(marks), "clocks": clocks,
    }
    print(json.dumps(line))
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
