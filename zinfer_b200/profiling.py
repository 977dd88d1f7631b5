"""Device time per kernel class, behind a switch.

While a :class:`Profiler` is active every kernel launch that goes through
``zinfer_b200.ops`` is bracketed by two CUDA events on the launching stream and filed
under its class (the operation, and for matrix products their shape) together with
the bytes it has to move and the floating-point operations it has to do.
``summary()`` waits for the device and gives, per class: launches, milliseconds,
bytes, flops, and the fraction of the roofline reached, i.e. the time the class
would take at the peak rates (the larger of bytes / memory bandwidth and
flops / tensor throughput) divided by the time it took.

Profiled steps run their kernels one by one: decode steps are not replayed from CUDA
graphs, and an event between two kernels keeps the second from starting under the
first's tail as it does in normal operation, so the sum over classes is a little
above a normal step's time.  So that the figures are device times and not the host's
pace of launching, every profiled step first queues a short spin on the device
(``lead_ms``) behind which the host gets ahead: the step's events and kernels then lie
back to back in the queue.  The figures are for finding where time goes; the
benchmark's numbers are never taken under a profiler.

The reference times its phases on the host and prints nanoseconds per operation
(src/app/cli/tools/bench/runtime.zig:57-71, src/app/cli/tools/bench/ops.zig:531-542).
"""
from __future__ import annotations

import json
from contextlib import contextmanager
from typing import Optional

import torch

ACTIVE: Optional["Profiler"] = None     # read by ops on every launch; None: no cost beyond this test


class Profiler:
    def __init__(self, hbm_gbs: Optional[float] = None, bf16_tflops: Optional[float] = None, lead_ms: float = 8.0):
        self.hbm_gbs = hbm_gbs
        self.bf16_tflops = bf16_tflops
        self.lead_ms = lead_ms
        self._records: list[tuple[str, object, object, int, int]] = []
        self.steps = 0

    def begin_step(self) -> None:
        """Called by the step function before a profiled step's first launch."""
        self.steps += 1
        if self.lead_ms > 0 and torch.cuda.is_available():
            torch.cuda._sleep(int(self.lead_ms * 1.5e6))    # cycles of a bounded spin; about lead_ms at 1.5 GHz

    @contextmanager
    def region(self, name: str, nbytes: int = 0, flops: int = 0):
        """Times what is launched inside the block.  The block may set ``rec["keep"] = False``
        (nothing was launched after all) to drop the record."""
        start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        rec = {"keep": True}
        start.record()
        try:
            yield rec
        finally:
            end.record()
            if rec["keep"]:
                self._records.append((name, start, end, int(nbytes), int(flops)))

    def summary(self) -> dict:
        torch.cuda.synchronize()
        classes: dict[str, dict] = {}
        for name, start, end, nbytes, flops in self._records:
            c = classes.setdefault(name, {"class": name, "launches": 0, "ms": 0.0, "bytes": 0, "flops": 0})
            c["launches"] += 1
            c["ms"] += start.elapsed_time(end)
            c["bytes"] += nbytes
            c["flops"] += flops
        rows = sorted(classes.values(), key=lambda c: -c["ms"])
        total = sum(c["ms"] for c in rows)
        for c in rows:
            c["ms"] = round(c["ms"], 4)
            c["share"] = round(c["ms"] / total, 4) if total > 0 else 0.0
            c["us_per_launch"] = round(1e3 * c["ms"] / c["launches"], 2)
            floor_ms = 0.0
            if self.hbm_gbs:
                floor_ms = max(floor_ms, c["bytes"] / (self.hbm_gbs * 1e9) * 1e3)
            if self.bf16_tflops:
                floor_ms = max(floor_ms, c["flops"] / (self.bf16_tflops * 1e12) * 1e3)
            c["roofline_frac"] = round(floor_ms / c["ms"], 4) if c["ms"] > 0 and floor_ms > 0 else None
        return {"steps": self.steps, "total_ms": round(total, 4), "peaks": {"hbm_gbs": self.hbm_gbs,
                "bf16_tflops": self.bf16_tflops}, "classes": rows}

    def dump(self, path: str) -> dict:
        s = self.summary()
        with open(path, "w") as f:
            json.dump(s, f, indent=1)
        return s


@contextmanager
def profile(hbm_gbs: Optional[float] = None, bf16_tflops: Optional[float] = None):
    """Activates a profiler for the kernel launches made inside the block."""
    global ACTIVE
    prof, before = Profiler(hbm_gbs, bf16_tflops), ACTIVE
    ACTIVE = prof
    try:
        yield prof
    finally:
        ACTIVE = before


class _Null:
    def __enter__(self):
        return {"keep": True}

    def __exit__(self, *exc):
        return False


_NULL = _Null()


def region(name: str, nbytes=0, flops=0):
    """A timed region if a profiler is active, else a context that does nothing.  ``nbytes``
    and ``flops`` may be callables, evaluated only when a profiler is active."""
    if ACTIVE is None:
        return _NULL
    return ACTIVE.region(name, nbytes() if callable(nbytes) else nbytes, flops() if callable(flops) else flops)


# ------------------------------------------------------------------ timeline of a chain
_TRACE_FILES = ("elementwise", "gemm_tcgen05", "attention_mma", "sampling", "attention_tcgen05", "attention_generic",
                "gemm_simt")


def chain_timeline(run_step, warm: int = 2) -> list[dict]:
    """The timeline of the kernels that ``run_step()`` launches, as they run inside their chain.

    Needs the kernel library built with time stamps (environment ``ZINFER_B200_TRACE=1`` from the
    start of the process; it is a second library, built beside the ordinary one).  Every kernel
    stamps the device's clock when its first block starts and when the kernels before it have
    completed.  Returns, in launch order, ``{"start_us", "deps_done_us", "own_us"}`` per kernel,
    times relative to the first stamp: ``start_us`` is when the kernel began (under programmatic
    dependent launch long before it may read its inputs), ``deps_done_us`` when everything before it
    had completed, ``own_us`` the time from there until everything before the NEXT kernel had
    completed, i.e. what this kernel adds to the chain.  Unlike a profiler that runs kernels one at
    a time, this shows the overlaps (weights of the next product fetched under a small kernel)."""
    import ctypes

    from . import ops
    from .csrc import build

    if not build.TRACE:
        raise RuntimeError("chain_timeline needs ZINFER_B200_TRACE=1 in the environment when the process starts")
    lib = ops.lib()
    buf = torch.zeros(8192 + 8, dtype=torch.int64, device="cuda")

    def point_all(ptr):
        for f in _TRACE_FILES:
            rc = getattr(lib, "zi_trace_set_" + f)(ctypes.c_void_p(ptr))
            if rc != 0:
                raise RuntimeError(f"zi_trace_set_{f} failed with CUDA error {rc}")

    try:
        for _ in range(warm):
            run_step()
        torch.cuda.synchronize()
        point_all(buf.data_ptr())
        torch.cuda.synchronize()
        run_step()
        torch.cuda.synchronize()
    finally:
        point_all(0)
        torch.cuda.synchronize()
    raw = buf.cpu().numpy()
    n = min(int(raw[0]) & 0xFFFFFFFF, 8192)
    stamps = sorted((int(v) >> 2, int(v) & 3) for v in raw[1:1 + n])
    if not stamps:
        return []
    t0 = stamps[0][0]
    starts = [(t - t0) / 1e3 for t, w in stamps if w == 0]
    waits = [(t - t0) / 1e3 for t, w in stamps if w == 1]
    out = []
    for i, (s_us, w_us) in enumerate(zip(starts, waits)):
        nxt = waits[i + 1] if i + 1 < len(waits) else None
        out.append({"start_us": round(s_us, 2), "deps_done_us": round(w_us, 2),
                    "own_us": round(nxt - w_us, 2) if nxt is not None else None})
    return out
