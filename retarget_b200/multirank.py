"""One planner process per GPU.

The placement path shards with no exchange: under tensor parallelism every
rank owns its KV-head shard in its own buffers and plans from its own copy of
the slot table, so ranks never trade data.  What they do share is bookkeeping:
a rendezvous, a barrier around timed regions, the maximum of per-rank timings,
and (as a consistency check) a digest of each rank's plan, which must be the
same everywhere because the slot ids are.  This module holds exactly that, on
top of ``torch.distributed`` -- NCCL on GPUs, gloo on CPU-only hosts -- or, with
backend ``"file"``, on nothing but files in a directory all ranks can see (no
process group, no communicator threads: used to tell what a process group costs
the timed region).
"""
from __future__ import annotations

import hashlib
import os

import numpy as np


class Ranks:
    def __init__(self, backend: str | None = None):
        self.rank = int(os.environ.get("RANK", "0"))
        self.world = int(os.environ.get("WORLD_SIZE", "1"))
        self.local_rank = int(os.environ.get("LOCAL_RANK", "0"))
        self.backend = backend
        self._dist = None
        self._device = None

    def start(self, device=None):
        """Joins the process group (no-op for a single process)."""
        if self.world == 1:
            return self
        if self.backend == "file":
            import tempfile
            # all ranks of one launch have the same parent (the launcher): its PID makes the directory theirs
            tag = os.environ.get("MASTER_PORT", "0") + "-" + str(os.getppid())
            self._dir = os.path.join(tempfile.gettempdir(), f"retarget-ranks-{tag}")
            os.makedirs(self._dir, exist_ok=True)
            self._round = 0
            return self
        import torch
        import torch.distributed as dist
        backend = self.backend or ("nccl" if device is not None else "gloo")
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        kwargs = {"device_id": device} if backend == "nccl" and device is not None else {}
        dist.init_process_group(backend, rank=self.rank, world_size=self.world, **kwargs)
        self._dist, self._device = dist, (device if backend == "nccl" else torch.device("cpu"))
        return self

    def stop(self):
        if self._dist is not None:
            self._dist.destroy_process_group()
            self._dist = None

    # ---- file rendezvous: every rank writes <round>.<rank>, then waits for all of them ----
    def _exchange(self, payload: bytes) -> list[bytes]:
        import time
        self._round += 1
        mine = os.path.join(self._dir, f"{self._round}.{self.rank}")
        with open(mine + ".tmp", "wb") as f:
            f.write(payload)
        os.replace(mine + ".tmp", mine)
        out = []
        deadline = time.monotonic() + 600
        for r in range(self.world):
            path = os.path.join(self._dir, f"{self._round}.{r}")
            while not os.path.exists(path):
                if time.monotonic() > deadline:
                    raise RuntimeError(f"rank {r} never reached rendezvous {self._round}")
                time.sleep(0.0005)
            with open(path, "rb") as f:
                out.append(f.read())
        return out

    def barrier(self):
        if getattr(self, "_dir", None):
            self._exchange(b"")
        elif self._dist is not None:
            self._dist.barrier()

    def max_over_ranks(self, values):
        """Element-wise maximum of a list of floats over all ranks."""
        if getattr(self, "_dir", None):
            rows = [np.frombuffer(x, dtype=np.float64) for x in
                    self._exchange(np.asarray(list(values), dtype=np.float64).tobytes())]
            return [float(v) for v in np.max(np.stack(rows), axis=0)]
        if self._dist is None:
            return [float(v) for v in values]
        import torch
        t = torch.tensor(list(values), dtype=torch.float64, device=self._device)
        self._dist.all_reduce(t, op=self._dist.ReduceOp.MAX)
        return [float(v) for v in t.cpu()]

    def same_everywhere(self, payload: bytes) -> bool:
        """True when every rank holds the same bytes (compared by digest)."""
        if getattr(self, "_dir", None):
            return len(set(self._exchange(hashlib.sha256(payload).digest()))) == 1
        if self._dist is None:
            return True
        import torch
        digest = np.frombuffer(hashlib.sha256(payload).digest(), dtype=np.uint8).astype(np.int64)
        mine = torch.from_numpy(digest.copy()).to(self._device)
        lo, hi = mine.clone(), mine.clone()
        self._dist.all_reduce(lo, op=self._dist.ReduceOp.MIN)
        self._dist.all_reduce(hi, op=self._dist.ReduceOp.MAX)
        return bool((lo == hi).all().item())
