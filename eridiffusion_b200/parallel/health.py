"""Host-side rank-failure detection: heartbeats through a key-value store.

The reference has no heartbeat, rank-failure detection or re-rendezvous (its distributed layer is
a stub: crates/training/src/distributed.rs:141-254). Here every rank bumps a counter in a store
(``torch.distributed.TCPStore`` in a job, any object with ``set`` / ``get`` in tests) from a
background thread, and ``check()`` — called between steps, before the next launch — raises
``RankFailure`` naming the ranks whose counter stopped moving for longer than ``timeout_s``.
Nothing runs on the GPU: a rank learns on the host that a peer is gone and can leave the step loop,
write its checkpoint and exit (or re-join a smaller group) instead of waiting inside a collective.
A rank that leaves on purpose calls ``leave()`` so that its peers see a clean departure.
"""
from __future__ import annotations

import threading
import time


class RankFailure(RuntimeError):
    def __init__(self, dead, left=()):
        self.dead, self.left = sorted(dead), sorted(left)
        super().__init__(f"ranks without heartbeat: {self.dead}" + (f"; ranks that left: {self.left}" if left else ""))


class Heartbeat:
    def __init__(self, store, rank: int, world: int, interval_s: float = 1.0, timeout_s: float = 10.0,
                 prefix: str = "hb", clock=time.monotonic, start: bool = True):
        self.store, self.rank, self.world = store, rank, world
        self.interval, self.timeout, self.prefix, self.clock = interval_s, timeout_s, prefix, clock
        self._count = 0
        self._seen = {}                      # rank -> (last counter value, local time it changed)
        self._stop = threading.Event()
        self._thread = None
        self.beat()
        if start:
            self._thread = threading.Thread(target=self._run, daemon=True)
            self._thread.start()

    def _key(self, r):
        return f"{self.prefix}/{r}"

    def beat(self):
        self._count += 1
        self.store.set(self._key(self.rank), str(self._count))

    def _run(self):
        while not self._stop.wait(self.interval):
            try:
                self.beat()
            except Exception:
                return                       # the store is gone: the job is shutting down

    def _read(self, r):
        try:
            v = self.store.get(self._key(r))
        except Exception:
            return None
        if isinstance(v, bytes):
            v = v.decode()
        return v

    def status(self):
        """{rank: "alive" | "dead" | "left" | "unknown"} from this rank's point of view."""
        now = self.clock()
        out = {}
        for r in range(self.world):
            if r == self.rank:
                out[r] = "alive"
                continue
            v = self._read(r)
            if v is None:
                first = self._seen.setdefault(r, (None, now))
                out[r] = "unknown" if now - first[1] <= self.timeout else "dead"
            elif v == "left":
                out[r] = "left"
            else:
                last = self._seen.get(r)
                if last is None or last[0] != v:
                    self._seen[r] = (v, now)
                    out[r] = "alive"
                else:
                    out[r] = "alive" if now - last[1] <= self.timeout else "dead"
        return out

    def check(self):
        """Raise ``RankFailure`` when a peer is dead or has left; call between steps."""
        st = self.status()
        dead = [r for r, s in st.items() if s == "dead"]
        left = [r for r, s in st.items() if s == "left"]
        if dead or left:
            raise RankFailure(dead, left)

    def leave(self):
        """Announce a clean departure and stop beating."""
        self.close()
        try:
            self.store.set(self._key(self.rank), "left")
        except Exception:
            pass

    def close(self):
        self._stop.set()
        if self._thread is not None:
            self._thread.join(timeout=2 * self.interval + 1.0)
            self._thread = None


def heartbeat_from_env(rank: int, world: int, port_offset: int = 17, **kw):
    """A ``Heartbeat`` over its own ``TCPStore`` next to the job's rendezvous port
    (``MASTER_PORT + port_offset``), rank 0 hosting it."""
    import datetime
    import os

    import torch.distributed as dist
    host = os.environ.get("MASTER_ADDR", "127.0.0.1")
    port = int(os.environ.get("MASTER_PORT", "29500")) + port_offset
    store = dist.TCPStore(host, port, world, is_master=(rank == 0), timeout=datetime.timedelta(seconds=60),
                          wait_for_workers=False)
    return Heartbeat(store, rank, world, **kw)
