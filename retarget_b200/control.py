"""Client side of the UVM control socket.

Same wire behaviour as the reference's ``UvmController.command/status/
_allocation_snapshot/wait_idle/_wait_job`` (experiments/control.py:403-544): one
ASCII line per connection (shorter than 512 bytes), one JSON line back, 50 ms
polling while a job runs, and refusal to talk to a PID that has been replaced.
The prefix plans of the trainer side are here too: ``aligned_uvm_target``,
``set_target`` and ``retarget`` with their result records
(experiments/control.py:379-400,488-654).
The shared-memory registry, the message-queue doorbell and the timeslice
controls of that file belong to the scheduler's control path and are not part
of this package.

``LocalUvm`` is the in-process twin: it hands the same lines straight to
``rt_uvm_command`` of the library loaded in this process, for callers that own
the GPU process themselves (tests, the benchmark, an embedded scheduler).
"""
from __future__ import annotations

import ctypes as C
import dataclasses
import json
import os
import pathlib
import socket
import time
from typing import Any

from . import capi


class ControlError(RuntimeError):
    """The controlled process cannot be driven safely (experiments/control.py:29)."""


@dataclasses.dataclass(frozen=True)
class UvmStatus:
    """experiments/control.py:53-83"""
    pid: int
    managed_bytes: int
    allocation_count: int
    allocation_generation: int
    busy: bool
    job_id: int
    completed_job: int
    last_error: int
    completed_cpu_bytes: int
    completed_gpu_bytes: int
    job_completed_bytes: int

    @classmethod
    def from_reply(cls, reply: dict[str, Any]) -> "UvmStatus":
        if not reply.get("ok"):
            raise ControlError(f"UVM status failed: {reply}")
        fields = {f.name: reply.get(f.name, 0) if f.name == "allocation_generation" else reply[f.name]
                  for f in dataclasses.fields(cls)}
        return cls(**{k: (bool(v) if k == "busy" else int(v)) for k, v in fields.items()})


@dataclasses.dataclass(frozen=True)
class UvmTargetResult:
    """What ``set_target`` did: the request, the request clamped to the managed
    bytes, and the page-aligned target that was sent."""
    requested_bytes: int
    clamped_bytes: int
    submitted_bytes: int
    status: UvmStatus


@dataclasses.dataclass(frozen=True)
class UvmRetargetResult:
    """What ``retarget`` did, with the previous target it moved away from."""
    previous_requested_bytes: int
    previous_submitted_bytes: int
    requested_bytes: int
    clamped_bytes: int
    submitted_bytes: int
    status: UvmStatus


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
    """Field 22 of /proc/<pid>/stat; guards against PID reuse."""
    try:
        text = pathlib.Path(f"/proc/{pid}/stat").read_text()
    except OSError as exc:
        raise ControlError(f"cannot read process {pid}: {exc}") from exc
    tail = text[text.rfind(")") + 2:].split()
    try:
        return int(tail[19])
    except (IndexError, ValueError) as exc:
        raise ControlError(f"malformed /proc/{pid}/stat starttime") from exc


class _Protocol:
    """Everything above the transport: what the reference client derives from
    command()."""

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

    def status(self) -> UvmStatus:
        status = UvmStatus.from_reply(self.command("status"))
        if status.pid != self.pid:
            raise ControlError(f"UVM socket identity mismatch: expected {self.pid}, got {status.pid}")
        return status

    def _allocation_snapshot(self) -> tuple[int, list[dict[str, int]]]:
        reply = self.command("list")
        if not reply.get("ok"):
            raise ControlError(f"UVM list failed: {reply}")
        allocations = [{"id": int(a["id"]), "bytes": int(a["bytes"]), "device": int(a["device"])}
                       for a in reply.get("allocations", [])]
        return int(reply.get("allocation_generation", 0)), allocations

    def allocations(self) -> list[dict[str, int]]:
        return self._allocation_snapshot()[1]

    def wait_idle(self, timeout: float = 120.0, poll_seconds: float = 0.05) -> UvmStatus:
        deadline = time.monotonic() + timeout
        while True:
            status = self.status()
            if not status.busy:
                self._settle_in_flight(status)
                return status
            if time.monotonic() >= deadline:
                raise ControlError(f"UVM worker for PID {self.pid} remained busy")
            time.sleep(poll_seconds)

    def _settle_in_flight(self, status: UvmStatus) -> None:
        """An idle worker settles a job that was submitted without waiting
        (experiments/control.py:488-513)."""
        if self._in_flight is None:
            return
        job_id, placement = self._in_flight
        if status.completed_job < job_id:
            raise ControlError(f"UVM worker for PID {self.pid} became idle before job {job_id} completed")
        self._in_flight = None
        if status.last_error != 0:
            self._placed = None
            raise ControlError(f"UVM job {job_id} for PID {self.pid} failed with CUDA error "
                               f"{status.last_error}")
        self._placed = placement

    def _wait_job(self, job_id: int, timeout: float = 120.0, poll_seconds: float = 0.05) -> UvmStatus:
        deadline = time.monotonic() + timeout
        while True:
            status = self.status()
            if not status.busy and status.completed_job >= job_id:
                if status.last_error != 0:
                    raise ControlError(f"UVM job {job_id} for PID {self.pid} failed with CUDA error "
                                       f"{status.last_error}")
                return status
            if time.monotonic() >= deadline:
                raise ControlError(f"timed out waiting for UVM job {job_id}")
            time.sleep(poll_seconds)

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
        reply = self.command(line)
        if not reply.get("ok"):
            raise ControlError(f"UVM {what} for PID {self.pid} failed: {reply}")
        job_id = int(reply["job_id"])
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
        reply = self.command(f"prefetch {allocation_id} {offset} {length} {where}")
        if not reply.get("ok"):
            raise ControlError(f"UVM prefetch rejected: {reply}")
        return self._wait_job(int(reply["job_id"]), timeout=timeout)


def _check_line(command: str) -> bytes:
    if "\0" in command or "\n" in command or "\r" in command:
        raise ValueError("UVM command must be one line without terminators")
    wire = (command + "\n").encode("ascii")
    if len(wire) >= 512:
        raise ValueError("UVM command is too long")
    return wire


def _parse_reply(raw: bytes, pid: int) -> dict[str, Any]:
    try:
        reply = json.loads(raw)
    except json.JSONDecodeError as exc:
        raise ControlError(f"invalid UVM response from PID {pid}: {raw!r}") from exc
    if not isinstance(reply, dict):
        raise ControlError(f"unexpected UVM response from PID {pid}: {reply!r}")
    return reply


class UvmController(_Protocol):
    """One-command-per-connection client for the control socket of another
    (or this) process."""

    def __init__(self, pid: int, timeout: float = 2.0, path: str | None = None):
        if pid <= 0:
            raise ValueError("pid must be positive")
        try:
            owner = pathlib.Path(f"/proc/{pid}").stat().st_uid
        except OSError as exc:
            raise ControlError(f"cannot stat process {pid}: {exc}") from exc
        if owner != os.getuid():
            raise ControlError(f"PID {pid} is owned by another user")
        self.pid = pid
        self._start_time = process_start_time(pid)
        self.timeout = timeout
        self.path = path or f"/tmp/select-uvm-{os.getuid()}-{pid}.sock"

    def command(self, command: str) -> dict[str, Any]:
        if process_start_time(self.pid) != self._start_time:
            raise ControlError(f"PID {self.pid} was replaced; refusing stale UVM control")
        wire = _check_line(command)
        chunks, total = [], 0
        with socket.socket(socket.AF_UNIX, socket.SOCK_STREAM) as client:
            client.settimeout(self.timeout)
            try:
                client.connect(self.path)
                client.sendall(wire)
                while True:
                    chunk = client.recv(4096)
                    if not chunk:
                        break
                    chunks.append(chunk)
                    total += len(chunk)
                    if total > 1024 * 1024:
                        raise ControlError("oversized UVM response")
                    if b"\n" in chunk:
                        break
            except OSError as exc:
                raise ControlError(f"UVM command to PID {self.pid} failed: {exc}") from exc
        return _parse_reply(b"".join(chunks).split(b"\n", 1)[0], self.pid)


class LocalUvm(_Protocol):
    """The same protocol against the server inside this process."""

    def __init__(self):
        self.pid = os.getpid()
        self._buf = C.create_string_buffer(1 << 20)
        capi.lib.rt_uvm_command.restype = C.c_int
        capi.lib.rt_uvm_command.argtypes = [C.c_char_p, C.c_char_p, C.c_size_t]

    def command(self, command: str) -> dict[str, Any]:
        wire = _check_line(command)
        n = capi.lib.rt_uvm_command(wire[:-1], self._buf, len(self._buf))
        capi.check(n, "rt_uvm_command")
        return _parse_reply(self._buf.raw[:n], self.pid)
