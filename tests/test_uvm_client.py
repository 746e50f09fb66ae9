"""The native client transport of the control socket (rt_uvm_client_command),
the status parser and the PID checks, against small Python servers: a reply
that arrives in pieces, a server that never answers, a reply that never ends,
a socket that is not there."""
import ctypes as C
import os
import socket
import threading
import time

import pytest

from retarget_b200 import capi
from retarget_b200.control import ControlError, UvmController, UvmStatus, process_start_time


class Server:
    """Accepts one connection per command and answers with `behaviour(conn, line)`."""

    def __init__(self, path, behaviour):
        self.path, self.behaviour, self.lines = path, behaviour, []
        self.sock = socket.socket(socket.AF_UNIX, socket.SOCK_STREAM)
        self.sock.bind(path)
        self.sock.listen(4)
        self.sock.settimeout(0.1)
        self.stop = False
        self.thread = threading.Thread(target=self.run, daemon=True)
        self.thread.start()

    def run(self):
        while not self.stop:
            try:
                conn, _ = self.sock.accept()
            except socket.timeout:
                continue
            with conn:
                conn.settimeout(2.0)
                data = b""
                try:
                    while not data.endswith(b"\n"):
                        chunk = conn.recv(600)
                        if not chunk:
                            break
                        data += chunk
                    self.lines.append(data)
                    self.behaviour(conn, data)
                except OSError:
                    pass

    def close(self):
        self.stop = True
        self.thread.join()
        self.sock.close()


STATUS = ('{"ok":true,"pid":%d,"managed_bytes":1048576,"allocation_count":2,"allocation_generation":9,'
          '"busy":false,"job_id":4,"completed_job":4,"last_error":0,"completed_cpu_bytes":5,'
          '"completed_gpu_bytes":6,"job_completed_bytes":7}')


def test_command_round_trip_and_reply_in_pieces(tmp_path):
    text = (STATUS % os.getpid()).encode() + b"\n"

    def in_pieces(conn, line):
        for k in range(0, len(text), 17):
            conn.sendall(text[k:k + 17])
            time.sleep(0.002)
    srv = Server(str(tmp_path / "s.sock"), in_pieces)
    try:
        client = UvmController(os.getpid(), path=srv.path)
        st = client.status()
        assert st == UvmStatus(os.getpid(), 1048576, 2, 9, False, 4, 4, 0, 5, 6, 7)
        assert srv.lines == [b"status\n"]                     # one line, one terminator, nothing else
        reply = client.command("list")
        assert reply["pid"] == os.getpid() and srv.lines[-1] == b"list\n"
    finally:
        srv.close()


def test_transport_failures_become_control_errors(tmp_path):
    client = UvmController(os.getpid(), timeout=0.3, path=str(tmp_path / "missing.sock"))
    with pytest.raises(ControlError, match="No such file or directory"):
        client.command("status")
    silent = Server(str(tmp_path / "silent.sock"), lambda conn, line: time.sleep(1.0))
    endless = Server(str(tmp_path / "endless.sock"),
                     lambda conn, line: [conn.sendall(b"x" * 65536) for _ in range(40)])
    try:
        t0 = time.monotonic()
        with pytest.raises(ControlError, match="timed out"):
            UvmController(os.getpid(), timeout=0.3, path=silent.path).command("status")
        assert 0.25 < time.monotonic() - t0 < 0.9          # ONE deadline covers the whole exchange
        with pytest.raises(ControlError, match="oversized"):
            UvmController(os.getpid(), timeout=5.0, path=endless.path).command("status")
    finally:
        silent.close()
        endless.close()
    for bad in ("two\nlines", "nul\0byte", "x" * 511):
        with pytest.raises(ValueError):
            client.command(bad)
    with pytest.raises(ControlError, match="invalid UVM response"):
        srv = Server(str(tmp_path / "junk.sock"), lambda conn, line: conn.sendall(b"not json\n"))
        try:
            UvmController(os.getpid(), path=srv.path).command("status")
        finally:
            srv.close()


def test_status_parser_and_identity_checks():
    lib = capi.lib

    from retarget_b200.control import _StatusStruct as Status      # the binding's view of rt_uvm_status
    out = Status()
    assert lib.rt_uvm_parse_status((STATUS % 77).replace('"busy":false', '"busy":true')
                                   .replace('"last_error":0', '"last_error":700').encode(), C.byref(out)) == 0
    assert (out.pid, out.busy, out.last_error, out.allocation_generation, out.job_completed_bytes) == \
        (77, 1, 700, 9, 7)
    # an older server that does not report the generation: 0
    assert lib.rt_uvm_parse_status((STATUS % 77).replace('"allocation_generation":9,', "").encode(),
                                   C.byref(out)) == 0 and out.allocation_generation == 0
    assert lib.rt_uvm_parse_status(b'{"ok":false,"error":"busy"}', C.byref(out)) == capi.RT_ERR_PLAN
    assert lib.rt_uvm_parse_status(b'{"ok":true,"pid":1}', C.byref(out)) == capi.RT_ERR_INVALID_ARGUMENT
    with pytest.raises(ControlError, match="UVM status failed"):
        UvmStatus.from_reply({"ok": False, "error": "stopping"})
    # the start time is field 22 of /proc/<pid>/stat, whatever the command name contains
    want = int(open(f"/proc/{os.getpid()}/stat").read().rsplit(")", 1)[1].split()[19])
    assert process_start_time(os.getpid()) == want
    with pytest.raises(ControlError, match="cannot read process"):
        process_start_time(2 ** 22 + 12345)
    with pytest.raises(ControlError, match="cannot stat process"):
        UvmController(2 ** 22 + 12345)
    if os.getuid() != 0:
        with pytest.raises(ControlError, match="owned by another user"):
            UvmController(1)
