"""Host-side liveness: every rank publishes (iteration, phase, wall time) through the rendezvous key-value
store; rank 0 reads all entries and names the ranks whose last beat is older than a deadline.

Nothing here touches the GPU: a rank that is stuck inside a collective stops beating because its training
loop stops calling ``beat``; a rank whose process died keeps its last entry, which ages.  The reference has
no counterpart (it relies on the scheduler noticing a dead job).
"""
from __future__ import annotations

import json
import threading
import time
from typing import Dict, List, Optional


class Heartbeat:
    def __init__(self, store, rank: int, world_size: int, interval_s: float = 10.0, stale_after_s: Optional[float] = None,
                 clock=time.time, prefix: str = "neox_hb"):
        self.store, self.rank, self.world = store, rank, world_size
        self.interval = float(interval_s)
        self.stale_after = float(stale_after_s) if stale_after_s is not None else 3.0 * self.interval
        self.clock, self.prefix = clock, prefix
        self._state = {"iteration": -1, "phase": "init"}
        self._stop = threading.Event()
        self._thread: Optional[threading.Thread] = None
        self._lock = threading.Lock()
        self.last_beat_published = None

    def _key(self, r):
        return f"{self.prefix}/{r}"

    def beat(self, iteration: int, phase: str = "step"):
        """Called by the training loop; cheap (no store traffic), the publisher thread sends the latest value."""
        with self._lock:
            self._state = {"iteration": int(iteration), "phase": phase, "progress_time": self.clock()}

    def publish_once(self):
        with self._lock:
            payload = dict(self._state, time=self.clock(), rank=self.rank)
        self.store.set(self._key(self.rank), json.dumps(payload))
        self.last_beat_published = payload

    def start(self):
        if self._thread is not None or self.interval <= 0:
            return self

        def loop():
            while not self._stop.wait(self.interval):
                try:
                    self.publish_once()
                except Exception:  # noqa: BLE001 - the store goes away at shutdown
                    return
        self.publish_once()
        self._thread = threading.Thread(target=loop, name="neox-heartbeat", daemon=True)
        self._thread.start()
        return self

    def stop(self):
        self._stop.set()
        if self._thread is not None:
            self._thread.join(timeout=2 * self.interval + 1)
            self._thread = None

    # ------------------------------------------------------------------ monitor side (any rank may call it)
    def read_all(self) -> Dict[int, Optional[dict]]:
        out = {}
        for r in range(self.world):
            try:
                if hasattr(self.store, "check") and not self.store.check([self._key(r)]):
                    out[r] = None
                    continue
                out[r] = json.loads(self.store.get(self._key(r)).decode())
            except Exception:  # noqa: BLE001
                out[r] = None
        return out

    def stragglers(self) -> List[dict]:
        """Ranks that never reported, whose publisher went silent, or whose training loop made no progress
        for ``stale_after`` seconds while others did."""
        now = self.clock()
        beats = self.read_all()
        newest_iter = max((b["iteration"] for b in beats.values() if b), default=-1)
        bad = []
        for r, b in beats.items():
            if b is None:
                bad.append({"rank": r, "reason": "no heartbeat"})
            elif now - b["time"] > self.stale_after:
                bad.append({"rank": r, "reason": f"silent for {now - b['time']:.1f}s", "last": b})
            elif b["iteration"] < newest_iter and now - b.get("progress_time", b["time"]) > self.stale_after:
                bad.append({"rank": r, "reason": f"stuck at iteration {b['iteration']} ({b['phase']}) while others "
                                                 f"reached {newest_iter}", "last": b})
        return bad


def from_args(neox_args):
    """Heartbeat over the process group's own store when ``heartbeat_interval`` > 0, else None."""
    import torch.distributed as dist
    if not neox_args.heartbeat_interval or not dist.is_initialized():
        return None
    store = dist.distributed_c10d._get_default_store()
    return Heartbeat(store, dist.get_rank(), dist.get_world_size(), interval_s=neox_args.heartbeat_interval).start()
