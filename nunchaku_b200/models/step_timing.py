"""Shared timing protocol of the transformer-step benchmarks: the reference's latency script
(``app/flux.1/t2i/latency.py:19-34,65-94``: warm-up runs, then timed runs with the extremes dropped) with CUDA events,
plus a per-kernel-class split of one step's device time from the torch profiler."""
from __future__ import annotations

import torch

CLASSES = (
    ("w4a4_gemm", ("gemm_w4a4_kernel", "lora_partial_reduce", "int4_row_norm")),
    ("quantiser", ("quantize_fuse_lora",)),
    ("rowwise", ("qk_norm_rope", "layernorm_modulate", "litela", "gate_residual", "relayout", "retile")),
    ("attention", ("flash", "fmha", "attention", "sdpa", "cudnn", "mha")),
)


def timed_steps(step, reps: int, warmup: int, host: dict | None = None) -> tuple[float, list[float]]:
    """Runs ``step`` ``warmup`` + ``reps`` times; returns (trimmed mean ms: the 20 % fastest and slowest of the timed runs
    dropped, as the reference's script does, and the per-run times).  Every run is bracketed by its own pair of events;
    nothing synchronises inside the timed sequence.  ``host``, when given, receives the host's enqueue time per step."""
    for _ in range(warmup):
        step()
    torch.cuda.synchronize()
    ev = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(reps)]
    import time
    t0 = time.perf_counter()
    for a, b in ev:
        a.record()
        step()
        b.record()
    if host is not None:   # how long the host needs to enqueue one step (the device lags behind while it does)
        host["enqueue_ms_per_step"] = (time.perf_counter() - t0) * 1e3 / reps
    torch.cuda.synchronize()
    ts = sorted(a.elapsed_time(b) for a, b in ev)
    drop = int(len(ts) * 0.2)
    kept = ts[drop: len(ts) - drop] if len(ts) - 2 * drop > 0 else ts
    return sum(kept) / len(kept), ts


def device_time_split(step) -> dict | None:
    """Device time of one ``step`` by kernel class (milliseconds), or None when the profiler is unavailable."""
    try:
        from torch.profiler import ProfilerActivity, profile

        torch.cuda.synchronize()
        with profile(activities=[ProfilerActivity.CUDA]) as prof:
            step()
            torch.cuda.synchronize()
        out = {name: 0.0 for name, _ in CLASSES}
        out["other"] = 0.0
        launches = {name: 0 for name in out}
        for e in prof.key_averages():
            t = getattr(e, "self_device_time_total", None)
            if t is None:
                t = getattr(e, "self_cuda_time_total", 0.0)
            if not t:
                continue
            key = e.key.lower()
            cls = "other"
            for name, pats in CLASSES:
                if any(p in key for p in pats):
                    cls = name
                    break
            out[cls] += t / 1e3
            launches[cls] += e.count
        total = sum(out.values())
        return {"ms": {k: round(v, 3) for k, v in out.items()}, "launches": launches, "total_ms": round(total, 3)}
    except Exception as exc:   # profiling is a nicety: never fail the benchmark over it
        return {"error": f"{type(exc).__name__}: {exc}"[:200]}
