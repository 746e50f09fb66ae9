"""Client side of the UVM control socket.

Same wire behaviour as the reference's ``UvmController.command/status/
_allocation_snapshot/wait_idle/_wait_job`` (experiments/control.py:403-544): one
ASCII line per connection (shorter than 512 bytes), one JSON line back, 50 ms
polling while a job runs, and refusal to talk to a PID that has been replaced.
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

    def command(self, command: str) -> dict[str, Any]:
        raise NotImplementedError

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
                return status
            if time.monotonic() >= deadline:
                raise ControlError(f"UVM worker for PID {self.pid} remained busy")
            time.sleep(poll_seconds)

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
