"""Counter-driven bounded prefetch window: the scheduler-facing controller.

Drop-in for the reference's experiments/cache_window.py: the same names
(``INITIAL``, ``CacheWindowSpec``, ``interval_difference``,
``CacheWindowController`` with ``update`` / ``due``), the same arguments, the
same commands on the UVM socket and the same accounting dictionary.  The
arithmetic itself lives in the native library (``rt_window_spec_check``,
``rt_window``, ``rt_interval_difference``, ``rt_window_accounting``); this file
only keeps the controller's state machine.
"""
from __future__ import annotations

import ctypes as C
import dataclasses
import math
import time
from typing import Mapping

from . import capi
from .control import ControlError

INITIAL = capi.RT_INITIAL

_INT_FIELDS = ("allocation_bytes", "allocation_count", "bytes_per_token",
               "width_tokens", "lookahead_tokens", "quantum_tokens")


@dataclasses.dataclass(frozen=True)
class CacheWindowSpec:
    """experiments/cache_window.py:19-50"""
    allocation_bytes: int
    allocation_count: int
    bytes_per_token: int
    width_tokens: int = 32768
    lookahead_tokens: int = 16384
    quantum_tokens: int = 8192
    min_update_seconds: float = 1.0
    idle_only: bool = True
    update_mode: str = "incremental"

    def __post_init__(self):
        # The checks that depend on Python types stay here; the numeric rules and
        # their order are the library's.
        for name in _INT_FIELDS:
            value = getattr(self, name)
            if type(value) is not int or value <= 0 or value >= 1 << 63:
                raise ValueError(f"cache_window.{name} must be a positive integer")
        mode_ok = self.update_mode in capi.UPDATE_MODES
        interval = self.min_update_seconds
        interval_ok = isinstance(interval, (int, float)) and math.isfinite(interval)
        raw = capi.WindowSpecStruct(*(getattr(self, n) for n in _INT_FIELDS),
                                    float(interval) if interval_ok else math.nan, 1,
                                    capi.UPDATE_MODES.index(self.update_mode) if mode_ok else 99)
        bad = C.c_int(-1)
        status = capi.lib.rt_window_spec_check(C.byref(raw), C.byref(bad))
        # idle_only sits between the interval and the mode check in the reference
        if status in (0, -26) and type(self.idle_only) is not bool:
            raise ValueError("cache_window.idle_only must be boolean")
        if status:
            raise ValueError(capi.strerror(status))
        object.__setattr__(self, "_raw", raw)

    def _struct(self) -> capi.WindowSpecStruct:
        return self._raw

    def window(self, completed_tokens: float) -> tuple[int, int]:
        """experiments/cache_window.py:52-63"""
        out = (C.c_uint64 * 2)()
        status = capi.lib.rt_window(C.byref(self._raw), float(completed_tokens), out)
        if status:
            raise ValueError(capi.strerror(status))
        return int(out[0]), int(out[1])


def interval_difference(a: tuple[int, int], b: tuple[int, int]) -> list[tuple[int, int]]:
    """experiments/cache_window.py:66-68"""
    out = (C.c_uint64 * 4)()
    n = capi.lib.rt_interval_difference((C.c_uint64 * 2)(*a), (C.c_uint64 * 2)(*b), out)
    return [(int(out[2 * i]), int(out[2 * i + 1])) for i in range(n)]


class CacheWindowController:
    """experiments/cache_window.py:71-148"""

    def __init__(self, spec: CacheWindowSpec):
        self.spec = spec
        self.current: tuple[int, int] | None = None
        self.signature: tuple | None = None
        self.last_update = -math.inf
        self.completed_highwater = 0.0

    def _counters(self, metrics: Mapping[str, float]) -> float:
        names = ("sglang:prompt_tokens_total", "sglang:generation_tokens_total")
        if any(name not in metrics for name in names):
            raise ControlError("cache-window policy requires SGLang completed-token counters")
        values = [metrics[name] for name in names]
        if any(not math.isfinite(v) or v < 0 for v in values):
            raise ControlError("invalid SGLang completed-token counters")
        self.completed_highwater = max(self.completed_highwater, sum(values))
        return self.completed_highwater

    def _idle(self, metrics) -> bool:
        return metrics["sglang:num_running_reqs"] == 0 and metrics["sglang:num_queue_reqs"] == 0

    def due(self, metrics: Mapping[str, float], now: float) -> bool:
        if self.spec.update_mode == "initial_only":
            return False
        window = self.spec.window(self._counters(metrics))
        return (window != self.current and now - self.last_update >= self.spec.min_update_seconds
                and (not self.spec.idle_only or self._idle(metrics)))

    def update(self, uvm, metrics: Mapping[str, float], now: float, *, initial: bool = False):
        spec = self.spec
        completed = self._counters(metrics)
        window = spec.window(completed)
        if not initial:
            if spec.update_mode == "initial_only":
                return None
            if window == self.current or now - self.last_update < spec.min_update_seconds:
                return None
            if spec.idle_only and (metrics["sglang:num_running_reqs"] > 0
                                   or metrics["sglang:num_queue_reqs"] > 0):
                return None
        uvm.wait_idle(timeout=600)
        generation, allocations = uvm._allocation_snapshot()
        cache = [a for a in allocations if a["bytes"] == spec.allocation_bytes]
        if len(cache) != spec.allocation_count:
            raise ControlError(f"cache layout mismatch: expected {spec.allocation_count} "
                               f"blocks of {spec.allocation_bytes}, found {len(cache)}")
        signature = tuple((a["id"], a["bytes"], a["device"]) for a in cache)
        full = initial or signature != self.signature or self.current is None
        old = (INITIAL, INITIAL) if full else self.current
        refresh = not full and spec.update_mode == "full_cache"
        verb = "windowfullv" if refresh else "windowv"
        reply = uvm.command(f"{verb} {generation} {spec.allocation_bytes} {spec.allocation_count} "
                            f"{old[0]} {old[1]} {window[0]} {window[1]}")
        if not reply.get("ok"):
            raise ControlError(f"cache window rejected: {reply}")
        try:
            status = uvm._wait_job(int(reply["job_id"]), timeout=600)
        except Exception:
            self.signature = None
            self.current = None
            raise
        other = sum(a["bytes"] for a in allocations if a["bytes"] != spec.allocation_bytes)
        gpu, cpu = C.c_uint64(), C.c_uint64()
        capi.check(capi.lib.rt_window_accounting(
            C.byref(spec._struct()), len(cache), other, (C.c_uint64 * 2)(*(old if not full else (0, 0))),
            (C.c_uint64 * 2)(*window), int(full), int(refresh), C.byref(gpu), C.byref(cpu)),
            "rt_window_accounting")
        self.current, self.signature, self.last_update = window, signature, now
        return {"audit_plan_started_monotonic_s": now,
                "audit_plan_committed_monotonic_s": time.monotonic(),
                "initial": full, "update_mode": spec.update_mode,
                "full_cache_refresh": refresh, "allocation_generation": generation,
                "cache_allocation_count": len(cache), "cache_allocation_bytes": spec.allocation_bytes,
                "old_window": None if full else list(old), "new_window": list(window),
                "completed_token_highwater": completed, "requested_gpu_bytes": gpu.value,
                "requested_cpu_bytes": cpu.value, "status": dataclasses.asdict(status)}
