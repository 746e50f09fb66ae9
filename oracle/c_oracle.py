"""ctypes wrapper of the C oracle (``oracle/plan_oracle.c``).

TEST INFRASTRUCTURE ONLY -- a checker and the timed CPU baseline; the shipped
package never imports it.
"""
from __future__ import annotations

import ctypes as C
import subprocess
from pathlib import Path

import numpy as np

HERE = Path(__file__).resolve().parent
LIB = HERE / "liborc_plan.so"
RANGE_DTYPE = np.dtype([("buffer", "<u4"), ("dst", "<i4"), ("offset", "<u8"), ("bytes", "<u8")])
MAX_BLOCKS = 1024


def build():
    src = HERE / "plan_oracle.c"
    if not LIB.exists() or LIB.stat().st_mtime < src.stat().st_mtime:
        subprocess.run(["make", "-C", str(HERE), "liborc_plan.so"], check=True, capture_output=True)
    return LIB


def _lib():
    lib = C.CDLL(str(build()))
    lib.orc_plan_step.restype = C.c_int64
    lib.orc_plan_step.argtypes = [C.c_void_p, C.c_void_p, C.c_int, C.c_void_p, C.c_int, C.c_uint64,
                                  C.c_uint64, C.c_uint32, C.c_uint64, C.c_uint32, C.c_int, C.c_int32,
                                  C.c_void_p, C.c_void_p, C.c_int64, C.POINTER(C.c_uint64), C.c_int]
    lib.orc_threads.restype = C.c_int
    return lib


class COracle:
    """Keeps the resident sets of one layout between steps."""

    def __init__(self, layout, device=0):
        self.lib = _lib()
        self.layout = layout
        self.device = device
        self.resident = np.zeros((layout.n_groups, MAX_BLOCKS), dtype=np.uint8)
        self.groups = np.ascontiguousarray(layout.buffer_group(), dtype=np.uint32)
        self.out = np.zeros(1 << 16, dtype=RANGE_DTYPE)

    @property
    def max_threads(self):
        return int(self.lib.orc_threads())

    def step(self, slots, group_off, budget, evict=True, threads=0):
        lay = self.layout
        threads = threads or self.max_threads
        invalid = C.c_uint64()
        n = self.lib.orc_plan_step(slots.ctypes.data, group_off.ctypes.data, lay.n_groups,
                                   self.groups.ctypes.data, lay.n_buffers, lay.alloc_bytes,
                                   lay.block_bytes, lay.block_tokens, lay.capacity, budget,
                                   int(evict), self.device, self.resident.ctypes.data,
                                   self.out.ctypes.data, len(self.out), C.byref(invalid), threads)
        assert n <= len(self.out)
        return self.out[:n], int(invalid.value)

    def resident_sets(self):
        return [set(np.flatnonzero(r).tolist()) for r in self.resident]
