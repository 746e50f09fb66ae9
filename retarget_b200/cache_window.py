"""Counter-driven bounded prefetch window: the scheduler-facing controller.

Drop-in for the reference's experiments/cache_window.py: the same names
(``INITIAL``, ``CacheWindowSpec``, ``interval_difference``,
``CacheWindowController`` with ``update`` / ``due``), the same arguments, the
same commands on the UVM socket and the same accounting dictionary.  The
arithmetic and the controller's state machine live in the native library
(``rt_window_spec_check``, ``rt_window``, ``rt_interval_difference``,
``rt_window_controller_*``); this file binds them: it turns the metrics
dictionary and the registry snapshot into plain structures, sends the command
the library wrote, and turns status codes back into the reference's exceptions.
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


_METRIC_NAMES = ("sglang:prompt_tokens_total", "sglang:generation_tokens_total",
                 "sglang:num_running_reqs", "sglang:num_queue_reqs")
_MISSING = {capi.RT_ERR_METRICS_KEY_RUNNING: _METRIC_NAMES[2], capi.RT_ERR_METRICS_KEY_QUEUE: _METRIC_NAMES[3]}


def _metrics_struct(metrics: Mapping[str, float]) -> capi.Metrics:
    """The four names the policy reads; what is absent is marked absent, so that
    the library can fail the way the reference does (a ControlError for the
    counters, a KeyError for the gauges, and only if they are needed)."""
    values, present = [], 0
    for bit, name in enumerate(_METRIC_NAMES):
        if name in metrics:
            values.append(float(metrics[name]))
            present |= 1 << bit
        else:
            values.append(0.0)
    return capi.Metrics(*values, present, 0)


def _raise_policy(status: int):
    if status in _MISSING:
        raise KeyError(_MISSING[status])
    if status in (capi.RT_ERR_METRICS_MISSING, capi.RT_ERR_METRICS_INVALID):
        raise ControlError(capi.strerror(status))
    if status == capi.RT_ERR_COMPLETED_COUNT:
        raise ValueError(capi.strerror(status))
    capi.check(status, "window controller")


def _registry_array(allocations):
    arr = (capi.AllocInfo * max(1, len(allocations)))()
    for k, a in enumerate(allocations):
        arr[k] = capi.AllocInfo(a["id"], a["bytes"], a["device"], 0)
    return arr


class CacheWindowController:
    """experiments/cache_window.py:71-148.  The state (``current``, ``signature``,
    ``last_update``, ``completed_highwater``) is held by the native controller and
    shown here as attributes."""

    def __init__(self, spec: CacheWindowSpec):
        self.spec = spec
        self._owner = True
        handle = C.c_void_p()
        capi.check(capi.lib.rt_window_controller_create(C.byref(spec._struct()), C.byref(handle)),
                   "rt_window_controller_create")
        self._w = handle

    def __del__(self):
        lib = getattr(capi, "lib", None)
        if getattr(self, "_owner", False) and getattr(self, "_w", None) and lib is not None:
            lib.rt_window_controller_destroy(self._w)
            self._w = None

    # ---- state ----
    def _state(self) -> capi.WindowState:
        st = capi.WindowState()
        capi.check(capi.lib.rt_window_controller_get(self._w, C.byref(st)))
        return st

    def _store(self, **fields):
        st = self._state()
        for k, v in fields.items():
            setattr(st, k, v)
        capi.check(capi.lib.rt_window_controller_set(self._w, C.byref(st)))

    @property
    def current(self):
        st = self._state()
        return (int(st.current[0]), int(st.current[1])) if st.has_current else None

    @current.setter
    def current(self, window):
        if window is None:
            self._store(has_current=0)
        else:
            st = self._state()
            st.has_current, st.current[0], st.current[1] = 1, int(window[0]), int(window[1])
            capi.check(capi.lib.rt_window_controller_set(self._w, C.byref(st)))

    @property
    def signature(self):
        n = C.c_size_t()
        cap = max(1, int(self._state().signature_count))
        arr = (capi.AllocInfo * cap)()
        status = capi.check(capi.lib.rt_window_controller_get_signature(self._w, arr, cap, C.byref(n)))
        if status == 1:
            return None
        return tuple((int(a.id), int(a.bytes), int(a.device)) for a in arr[:n.value])

    @signature.setter
    def signature(self, value):
        entries = [] if value is None else [dict(id=i, bytes=b, device=d) for i, b, d in value]
        capi.check(capi.lib.rt_window_controller_set_signature(self._w, _registry_array(entries), len(entries),
                                                               int(value is not None)))

    @property
    def last_update(self):
        return float(self._state().last_update)

    @last_update.setter
    def last_update(self, t):
        self._store(last_update=float(t))

    @property
    def completed_highwater(self):
        return float(self._state().completed_highwater)

    @completed_highwater.setter
    def completed_highwater(self, value):
        self._store(completed_highwater=float(value))

    # ---- policy ----
    def due(self, metrics: Mapping[str, float], now: float) -> bool:
        status = capi.lib.rt_window_controller_due(self._w, C.byref(_metrics_struct(metrics)), float(now))
        if status < 0:
            _raise_policy(status)
        return bool(status)

    def update(self, uvm, metrics: Mapping[str, float], now: float, *, initial: bool = False):
        lib, spec = capi.lib, self.spec
        go = lib.rt_window_controller_begin(self._w, C.byref(_metrics_struct(metrics)), float(now), int(initial))
        if go < 0:
            _raise_policy(go)
        if not go:
            return None
        uvm.wait_idle(timeout=600)
        generation, allocations = uvm._allocation_snapshot()
        command = C.create_string_buffer(512)
        plan = capi.WindowUpdate()
        status = lib.rt_window_controller_plan(self._w, _registry_array(allocations), len(allocations),
                                               int(generation), command, len(command), C.byref(plan))
        if status == capi.RT_ERR_LAYOUT_MISMATCH:
            raise ControlError(f"cache layout mismatch: expected {spec.allocation_count} "
                               f"blocks of {spec.allocation_bytes}, found {plan.cache_count}")
        capi.check(status, "rt_window_controller_plan")
        reply = uvm.command(command.value.decode("ascii"))
        if not reply.get("ok"):
            raise ControlError(f"cache window rejected: {reply}")
        try:
            status = uvm._wait_job(int(reply["job_id"]), timeout=600)
        except Exception:
            lib.rt_window_controller_fail(self._w)
            raise
        capi.check(lib.rt_window_controller_commit(self._w, float(now)), "rt_window_controller_commit")
        full = bool(plan.full)
        return {"audit_plan_started_monotonic_s": now,
                "audit_plan_committed_monotonic_s": time.monotonic(),
                "initial": full, "update_mode": spec.update_mode,
                "full_cache_refresh": bool(plan.refresh), "allocation_generation": generation,
                "cache_allocation_count": int(plan.cache_count), "cache_allocation_bytes": spec.allocation_bytes,
                "old_window": None if full else [int(plan.old_window[0]), int(plan.old_window[1])],
                "new_window": [int(plan.new_window[0]), int(plan.new_window[1])],
                "completed_token_highwater": float(plan.completed_highwater),
                "requested_gpu_bytes": int(plan.gpu_bytes), "requested_cpu_bytes": int(plan.cpu_bytes),
                "status": dataclasses.asdict(status)}
