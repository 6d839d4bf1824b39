"""Calibration of the frozen per-channel scales: observe the BF16 rows a serving stack writes to
its shared-KV caches, then merge the per-rank statistics into a `sharedkv-c8-v1` scale file.

Counterpart of the reference's observer (npu_sparse_attn_sharedkv_int8/calibration.py:17-73) and
of the merge procedure its documentation describes (docs/kv-cache.md:51-66: per layer and cache
kind the channel-wise maximum over ranks, `scale = clamp_min(margin * maximum / 127, 1e-8)`).

Collection is gated by a marker file, `<directory>/collect`: create it after the server has
warmed up, remove it, then send one more request so that every rank writes its statistics.  The
observer synchronises when it saves; it is a calibration mode, never to be benchmarked, and it
refuses to run inside a CUDA-graph capture (serve with eager execution while calibrating).
"""
import atexit
import hashlib
import os
from pathlib import Path
import time

import torch

PROTOCOL = "sharedkv-c8-v1"
DIM = 512


class CacheObserver:
    """Running channel-wise absolute maximum and row count per `<layer prefix>.<ori|cmp>`."""

    def __init__(self, directory, save_interval=10.0):
        self.directory = Path(directory)
        self.directory.mkdir(parents=True, exist_ok=True)
        self.marker = self.directory / "collect"
        self.save_interval = save_interval
        self.stats = {}
        self.dirty = False
        self.last_save = time.monotonic()
        atexit.register(self.flush)

    @torch.inference_mode()
    def observe(self, prefix, kind, cache, updates, slots):
        """Account for the rows of `updates` whose slot the cache writer would accept (flat slots:
        0 <= slot < pages * page size; `[page, offset]` pairs: both in range)."""
        if not self.marker.exists():
            self.flush()
            return
        if updates is None or updates.shape[0] == 0:
            return
        if updates.is_cuda and torch.cuda.is_current_stream_capturing():
            raise RuntimeError("Calibration requires eager execution; the marker must be absent during warmup")
        if updates.shape[-1] != DIM or cache.shape[-1] != DIM:
            raise ValueError("Calibration expects the D=512 shared KV cache")
        if slots.ndim == 1:
            valid = (slots >= 0) & (slots < cache.shape[0] * cache.shape[1])
        else:
            valid = ((slots[:, 0] >= 0) & (slots[:, 0] < cache.shape[0])
                     & (slots[:, 1] >= 0) & (slots[:, 1] < cache.shape[1]))
        values = updates.reshape(-1, DIM).float()
        values = torch.where(valid[:, None], values, torch.zeros((), dtype=values.dtype, device=values.device))
        maximum, rows = values.abs().amax(0), valid.sum()
        key = f"{prefix}.{kind}"
        seen = self.stats.get(key)
        if seen is None:
            self.stats[key] = [maximum, rows]
        else:
            seen[0].copy_(torch.maximum(seen[0], maximum))
            seen[1].add_(rows)
        self.dirty = True
        if time.monotonic() - self.last_save >= self.save_interval:
            self.flush()

    def flush(self):
        """Write `rank_XX.pt` atomically (temporary file, then rename), one file per rank."""
        if not self.dirty:
            return
        keys = sorted(self.stats)
        maxima = torch.stack([self.stats[k][0] for k in keys]).cpu()
        counts = torch.stack([self.stats[k][1] for k in keys]).cpu()
        if not torch.isfinite(maxima).all():
            raise RuntimeError("Non-finite real-model cache values encountered during calibration")
        rank = torch.distributed.get_rank() if torch.distributed.is_available() and torch.distributed.is_initialized() else 0
        payload = {"version": 1, "rank": rank, "pid": os.getpid(),
                   "stats": {k: {"maximum": maxima[i].clone(), "rows": int(counts[i])} for i, k in enumerate(keys)}}
        path = self.directory / f"rank_{rank:02d}.pt"
        temporary = path.with_suffix(f".tmp.{os.getpid()}")
        torch.save(payload, temporary)
        os.replace(temporary, path)
        self.dirty = False
        self.last_save = time.monotonic()


def merge_ranks(paths, *, margin=1.1, provenance=None, required_keys=None):
    """Per-rank statistics files -> a scale-file payload `vllm_adapter.load_scales` accepts.

    For every key the channel-wise maximum over the ranks, then
    `scale = clamp_min(margin * maximum / 127, 1e-8)` in FP32.  The payload records the margin,
    the rows observed across ranks, the SHA-256 of every source file and a free-form provenance.
    `required_keys`, when given, must all have been observed (the keys a target model needs)."""
    paths = [Path(p) for p in paths]
    if not paths:
        raise ValueError("No calibration statistics to merge")
    maxima, rows, hashes, ranks = {}, {}, {}, set()
    for path in sorted(paths):
        raw = path.read_bytes()
        payload = torch.load(path, map_location="cpu", weights_only=True)
        if payload.get("version") != 1 or "stats" not in payload:
            raise ValueError(f"Not a calibration statistics file: {path}")
        if payload["rank"] in ranks:
            raise ValueError(f"Rank {payload['rank']} appears twice; statistics files of different nodes need distinct names")
        ranks.add(payload["rank"])
        hashes[path.name] = hashlib.sha256(raw).hexdigest()
        for key, entry in payload["stats"].items():
            maximum = entry["maximum"]
            if maximum.shape != (DIM,) or maximum.dtype != torch.float32 or not bool(torch.isfinite(maximum).all()):
                raise ValueError(f"Invalid statistics for {key} in {path}")
            maxima[key] = maximum.clone() if key not in maxima else torch.maximum(maxima[key], maximum)
            rows[key] = rows.get(key, 0) + int(entry["rows"])
    missing = sorted(set(required_keys or ()) - set(maxima))
    if missing:
        raise ValueError(f"No observations for {len(missing)} required keys, first: {missing[0]}")
    scales = {key: (maximum * (margin / 127)).clamp_min(1e-8).float().contiguous() for key, maximum in sorted(maxima.items())}
    return {"protocol": PROTOCOL, "scales": scales, "margin": float(margin),
            "observed_rows_across_ranks": {key: rows[key] for key in sorted(rows)},
            "source_sha256": hashes, "provenance": dict(provenance or {})}


def save_scales(payload, path):
    """Write a merged payload atomically."""
    path = Path(path)
    temporary = path.with_suffix(path.suffix + f".tmp.{os.getpid()}")
    torch.save(payload, temporary)
    os.replace(temporary, path)
    return path
