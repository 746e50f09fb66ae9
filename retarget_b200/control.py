"""Client side of the UVM control socket.

The wire behaviour is the reference's (experiments/control.py:403-544): one
ASCII line per connection, shorter than 512 bytes; one JSON line back; a status
poll every 50 ms while a job runs; no talking to a PID that has been replaced.
How it is done is this package's own:

* the transport, the status parser and the two identity checks (owner and start
  time of the PID) are native (``rt_uvm_client_command``, ``rt_uvm_parse_status``,
  ``rt_process_start_time``, ``rt_process_owner``);
* everything that waits goes through one poller (``_Protocol._poll``): a
  condition on the status, a deadline, and what to say when it passes;
* the prefix plans of the trainer side (``aligned_uvm_target``, ``set_target``,
  ``retarget``, experiments/control.py:379-400,488-654) keep the placement they
  last established as one record and fall back to a full target whenever it
  does not describe the registry any more.

The shared-memory registry, the message-queue doorbell and the timeslice
controls of the reference's file belong to the scheduler's control path and
are not part of this package.

``LocalUvm`` is the in-process twin: the same lines go straight to
``rt_uvm_command`` of the library loaded in this process, for callers that own
the GPU process themselves (tests, the benchmark, an embedded scheduler).
"""
from __future__ import annotations

import ctypes as C
import dataclasses
import errno
import json
import os
import time
from typing import Any, Callable

from . import capi

_REPLY_BYTES = 1 << 20
POLL_SECONDS = 0.05


class ControlError(RuntimeError):
    """The controlled process cannot be driven safely (experiments/control.py:29)."""


class _StatusStruct(C.Structure):
    _fields_ = [("pid", C.c_uint64), ("managed_bytes", C.c_uint64), ("allocation_count", C.c_uint64),
                ("allocation_generation", C.c_uint64), ("busy", C.c_int32), ("last_error", C.c_int32),
                ("job_id", C.c_uint64), ("completed_job", C.c_uint64), ("completed_cpu_bytes", C.c_uint64),
                ("completed_gpu_bytes", C.c_uint64), ("job_completed_bytes", C.c_uint64)]


def _bind():
    lib = capi.lib
    lib.rt_uvm_client_command.restype = C.c_int
    lib.rt_uvm_client_command.argtypes = [C.c_char_p, C.c_char_p, C.c_double, C.c_char_p, C.c_size_t,
                                          C.POINTER(C.c_int)]
    lib.rt_uvm_parse_status.restype = C.c_int
    lib.rt_uvm_parse_status.argtypes = [C.c_char_p, C.POINTER(_StatusStruct)]
    lib.rt_process_start_time.restype = C.c_int
    lib.rt_process_start_time.argtypes = [C.c_uint64, C.POINTER(C.c_uint64), C.POINTER(C.c_int)]
    lib.rt_process_owner.restype = C.c_int
    lib.rt_process_owner.argtypes = [C.c_uint64, C.POINTER(C.c_uint32), C.POINTER(C.c_int)]
    lib.rt_uvm_command.restype = C.c_int
    lib.rt_uvm_command.argtypes = [C.c_char_p, C.c_char_p, C.c_size_t]
    return lib


_lib = _bind()


# The fields of a `status` reply in the order the server writes them
# (select.cpp:24058-24068); `busy` is the one boolean.  The record type is made
# from this list so that it, the native parser's structure and the reply cannot
# drift apart; result dictionaries carry ``dataclasses.asdict(status)``.
STATUS_FIELDS = ("pid", "managed_bytes", "allocation_count", "allocation_generation", "busy", "job_id",
                 "completed_job", "last_error", "completed_cpu_bytes", "completed_gpu_bytes",
                 "job_completed_bytes")
assert set(STATUS_FIELDS) == {name for name, _ in _StatusStruct._fields_}


def _status_from_reply(cls, reply: dict[str, Any]):
    """Builds the record from a reply dictionary; the parsing is the library's."""
    raw = _StatusStruct()
    status = _lib.rt_uvm_parse_status(json.dumps(reply, separators=(",", ":")).encode(), C.byref(raw))
    if status == capi.RT_ERR_PLAN:
        raise ControlError(f"UVM status failed: {reply}")
    if status:
        raise KeyError(next((n for n in STATUS_FIELDS if n not in reply and n != "allocation_generation"), "?"))
    return cls(*((bool(raw.busy) if n == "busy" else int(getattr(raw, n))) for n in STATUS_FIELDS))


UvmStatus = dataclasses.make_dataclass(
    "UvmStatus", [(n, bool if n == "busy" else int) for n in STATUS_FIELDS], frozen=True,
    namespace={"from_reply": classmethod(_status_from_reply),
               "__doc__": "A `status` reply (the reference's UvmStatus, experiments/control.py:53-83)."})
UvmStatus.__module__ = __name__


# What a prefix plan did: the request, the request clamped to the managed bytes,
# the page-aligned target that was sent, the status after the job.  A retarget
# also says which target it moved away from.  (Field names are the reference's:
# its callers read them, experiments/control.py:85-104.)
_TARGET_FIELDS = ("requested_bytes", "clamped_bytes", "submitted_bytes")
UvmTargetResult = dataclasses.make_dataclass(
    "UvmTargetResult", [*((n, int) for n in _TARGET_FIELDS), ("status", UvmStatus)], frozen=True)
UvmRetargetResult = dataclasses.make_dataclass(
    "UvmRetargetResult", [*(("previous_" + n, int) for n in _TARGET_FIELDS[::2]),
                          *((n, int) for n in _TARGET_FIELDS), ("status", UvmStatus)], frozen=True)
for _record in (UvmTargetResult, UvmRetargetResult):
    _record.__module__ = __name__


def aligned_uvm_target(allocation_sizes, desired_bytes: int, page_size: int) -> int:
    """A global residency target rounded down to where the preload library accepts
    it: only the offset inside the one partly resident allocation has to be a
    page multiple (experiments/control.py:379-400).  Arithmetic: rt_aligned_target."""
    if desired_bytes < 0 or page_size <= 0:
        raise ValueError("invalid target or page size")
    sizes = [int(x) for x in allocation_sizes]
    if any(x < 0 for x in sizes):
        raise ValueError("allocation sizes must be non-negative")
    array = (C.c_uint64 * max(len(sizes), 1))(*sizes)
    out = C.c_uint64()
    capi.check(capi.lib.rt_aligned_target(array, len(sizes), desired_bytes, page_size, C.byref(out)),
               "rt_aligned_target")
    return out.value


@dataclasses.dataclass(frozen=True)
class _Placement:
    """The registry a prefix plan was computed for and the target it asked for."""
    signature: tuple
    generation: int
    target: int


def process_start_time(pid: int) -> int:
    """Start time of ``pid`` in clock ticks since boot; guards against PID reuse."""
    ticks, err = C.c_uint64(), C.c_int()
    status = _lib.rt_process_start_time(pid, C.byref(ticks), C.byref(err))
    if status == capi.RT_ERR_IO:
        raise ControlError(f"cannot read process {pid}: {OSError(err.value, os.strerror(err.value))}")
    if status:
        raise ControlError(f"malformed /proc/{pid}/stat starttime")
    return ticks.value


def _wire_form(command: str) -> bytes:
    """The line as it goes out, without its terminator."""
    if any(c in command for c in "\0\n\r"):
        raise ValueError("UVM command must be one line without terminators")
    wire = command.encode("ascii")
    if len(wire) + 1 >= 512:
        raise ValueError("UVM command is too long")
    return wire


def _reply_object(raw: bytes, pid: int) -> dict[str, Any]:
    try:
        reply = json.loads(raw)
    except json.JSONDecodeError as exc:
        raise ControlError(f"invalid UVM response from PID {pid}: {raw!r}") from exc
    if not isinstance(reply, dict):
        raise ControlError(f"unexpected UVM response from PID {pid}: {reply!r}")
    return reply


class _Protocol:
    """Everything above the transport.  A subclass supplies ``command(line) ->
    reply dictionary`` and ``pid``."""

    pid: int
    # prefix plans: the placement the process is known to be in (None: unknown, the
    # next retarget becomes a full target) and a job submitted without waiting
    _placed: _Placement | None = None
    _in_flight: tuple[int, _Placement] | None = None

    def command(self, command: str) -> dict[str, Any]:
        raise NotImplementedError

    @property
    def _submitted_target(self):
        return self._placed.target if self._placed else None

    @property
    def _pending_job(self):
        return self._in_flight[0] if self._in_flight else None

    def _accepted(self, line: str, refusal: str) -> dict[str, Any]:
        """Sends one line; a reply that is not ok becomes ControlError(refusal + reply)."""
        reply = self.command(line)
        if not reply.get("ok"):
            raise ControlError(f"{refusal}: {reply}")
        return reply

    # ---- queries ----
    def status(self) -> UvmStatus:
        answer = UvmStatus.from_reply(self.command("status"))
        if answer.pid != self.pid:
            raise ControlError(f"UVM socket identity mismatch: expected {self.pid}, got {answer.pid}")
        return answer

    def _allocation_snapshot(self) -> tuple[int, list[dict[str, int]]]:
        listing = self._accepted("list", "UVM list failed")
        rows = [{key: int(entry[key]) for key in ("id", "bytes", "device")}
                for entry in listing.get("allocations", [])]
        return int(listing.get("allocation_generation", 0)), rows

    def allocations(self) -> list[dict[str, int]]:
        return self._allocation_snapshot()[1]

    # ---- waiting ----
    def _poll(self, settled: Callable[[UvmStatus], bool], timeout: float, poll_seconds: float,
              gave_up: str) -> UvmStatus:
        """Status polls until ``settled(status)``; ControlError(gave_up) once
        ``timeout`` seconds have passed without it."""
        give_up_at = time.monotonic() + timeout
        answer = self.status()
        while not settled(answer):
            if time.monotonic() >= give_up_at:
                raise ControlError(gave_up)
            time.sleep(poll_seconds)
            answer = self.status()
        return answer

    def _job_error(self, job_id: int, answer: UvmStatus) -> ControlError | None:
        if answer.last_error == 0:
            return None
        return ControlError(f"UVM job {job_id} for PID {self.pid} failed with CUDA error {answer.last_error}")

    def wait_idle(self, timeout: float = 120.0, poll_seconds: float = POLL_SECONDS) -> UvmStatus:
        answer = self._poll(lambda s: not s.busy, timeout, poll_seconds,
                            f"UVM worker for PID {self.pid} remained busy")
        if self._in_flight is not None:
            # an idle worker settles the job that was submitted without waiting
            job_id, placement = self._in_flight
            if answer.completed_job < job_id:
                raise ControlError(f"UVM worker for PID {self.pid} became idle before job {job_id} completed")
            self._in_flight = None
            failure = self._job_error(job_id, answer)
            self._placed = None if failure else placement
            if failure:
                raise failure
        return answer

    def _wait_job(self, job_id: int, timeout: float = 120.0, poll_seconds: float = POLL_SECONDS) -> UvmStatus:
        answer = self._poll(lambda s: not s.busy and s.completed_job >= job_id, timeout, poll_seconds,
                            f"timed out waiting for UVM job {job_id}")
        failure = self._job_error(job_id, answer)
        if failure:
            raise failure
        return answer

    # ---- prefix plans ----
    def _registry(self, status: UvmStatus, *targets: int):
        """Generation, signature and the page-aligned form of each target, clamped
        to what is managed."""
        generation, allocations = self._allocation_snapshot()
        signature = tuple((a["id"], a["bytes"], a["device"]) for a in allocations)
        sizes = [a["bytes"] for a in allocations]
        page = os.sysconf("SC_PAGE_SIZE")
        clamped = [min(t, status.managed_bytes) for t in targets]
        return generation, signature, clamped, [aligned_uvm_target(sizes, c, page) for c in clamped]

    def _submit_prefix_plan(self, line: str, what: str, placement: _Placement, wait: bool, timeout: float):
        job_id = int(self._accepted(line, f"UVM {what} for PID {self.pid} failed")["job_id"])
        if not wait:
            self._in_flight = (job_id, placement)
            return job_id, None
        try:
            completed = self._wait_job(job_id, timeout=timeout)
        except Exception:
            self._placed = None
            raise
        self._placed = placement
        return job_id, completed

    def set_target(self, gpu_bytes: int, *, timeout: float = 120.0, wait: bool = True):
        """Makes the first ``gpu_bytes`` of the managed allocations (registry
        order) GPU resident and the rest CPU resident: ``targetv``
        (experiments/control.py:546-592).  With ``wait=False`` returns the job id;
        the next ``wait_idle`` settles it."""
        if gpu_bytes < 0:
            raise ValueError("gpu_bytes must be non-negative")
        status = self.wait_idle(timeout=timeout)
        generation, signature, (desired,), (target,) = self._registry(status, gpu_bytes)
        job_id, completed = self._submit_prefix_plan(
            f"targetv {generation} {target}", f"target {target}",
            _Placement(signature, generation, target), wait, timeout)
        if completed is None:
            return job_id
        return UvmTargetResult(requested_bytes=gpu_bytes, clamped_bytes=desired, submitted_bytes=target,
                               status=completed)

    def retarget(self, previous_gpu_bytes: int, gpu_bytes: int, *, timeout: float = 120.0, wait: bool = True):
        """Moves only the bytes between the previous target and the new one:
        ``retarget`` (experiments/control.py:594-654).  Falls back to ``set_target``
        whenever the process is not known to be in the previous placement (other
        registry, other generation, other target, or a failed job since)."""
        if previous_gpu_bytes < 0 or gpu_bytes < 0:
            raise ValueError("GPU targets must be non-negative")
        status = self.wait_idle(timeout=timeout)
        generation, signature, (_, desired), (previous_target, target) = self._registry(
            status, previous_gpu_bytes, gpu_bytes)
        if self._placed != _Placement(signature, generation, previous_target):
            return self.set_target(gpu_bytes, timeout=timeout, wait=wait)
        job_id, completed = self._submit_prefix_plan(
            f"retarget {generation} {previous_target} {target}", f"retarget {previous_target}->{target}",
            _Placement(signature, generation, target), wait, timeout)
        if completed is None:
            return job_id
        return UvmRetargetResult(previous_requested_bytes=previous_gpu_bytes,
                                 previous_submitted_bytes=previous_target, requested_bytes=gpu_bytes,
                                 clamped_bytes=desired, submitted_bytes=target, status=completed)

    def prefetch(self, allocation_id: int, offset: int, length: int, where: str,
                 timeout: float = 120.0) -> UvmStatus:
        if where not in ("cpu", "gpu"):
            raise ValueError("where must be 'cpu' or 'gpu'")
        reply = self._accepted(f"prefetch {allocation_id} {offset} {length} {where}", "UVM prefetch rejected")
        return self._wait_job(int(reply["job_id"]), timeout=timeout)


class UvmController(_Protocol):
    """Client for the control socket of another (or this) process: one command
    per connection, through the library's transport."""

    def __init__(self, pid: int, timeout: float = 2.0, path: str | None = None):
        if pid <= 0:
            raise ValueError("pid must be positive")
        owner, err = C.c_uint32(), C.c_int()
        if _lib.rt_process_owner(pid, C.byref(owner), C.byref(err)):
            raise ControlError(f"cannot stat process {pid}: {OSError(err.value, os.strerror(err.value))}")
        if owner.value != os.getuid():
            raise ControlError(f"PID {pid} is owned by another user")
        self.pid = pid
        self._born = process_start_time(pid)
        self.timeout = timeout
        self.path = path or f"/tmp/select-uvm-{os.getuid()}-{pid}.sock"
        self._reply = C.create_string_buffer(_REPLY_BYTES + 2)

    def command(self, command: str) -> dict[str, Any]:
        if process_start_time(self.pid) != self._born:
            raise ControlError(f"PID {self.pid} was replaced; refusing stale UVM control")
        wire = _wire_form(command)
        err = C.c_int()
        n = _lib.rt_uvm_client_command(self.path.encode(), wire, float(self.timeout), self._reply,
                                       len(self._reply), C.byref(err))
        if n == capi.RT_ERR_CAPACITY:
            raise ControlError("oversized UVM response")
        if n == capi.RT_ERR_IO:
            why = "timed out" if err.value == errno.ETIMEDOUT else str(OSError(err.value, os.strerror(err.value)))
            raise ControlError(f"UVM command to PID {self.pid} failed: {why}")
        capi.check(n, "rt_uvm_client_command")
        return _reply_object(self._reply.raw[:n], self.pid)


class LocalUvm(_Protocol):
    """The same protocol against the server inside this process."""

    def __init__(self):
        self.pid = os.getpid()
        self._reply = C.create_string_buffer(_REPLY_BYTES)

    def command(self, command: str) -> dict[str, Any]:
        n = _lib.rt_uvm_command(_wire_form(command), self._reply, len(self._reply))
        capi.check(n, "rt_uvm_command")
        return _reply_object(self._reply.raw[:n], self.pid)
