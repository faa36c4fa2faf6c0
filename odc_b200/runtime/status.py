"""Error reporting for bounded waits, and host-side liveness.

Every wait in the reference is unbounded (odc/primitives/scatter_accumulate.py:204-206,
odc/primitives/utils.py:254-256): a dead peer hangs the GPU stream for good.  Here each device
wait carries a time budget; when it runs out the kernel writes a status word and returns, the
CUDA context stays usable, and the host turns the word into an exception.  Liveness of peers
between steps is tracked on the host with heartbeats in a key-value store.
"""
from __future__ import annotations

import time
from typing import Dict, List, Optional

OK = 0
ERR_WAIT_TIMEOUT = 1      # an arrival counter did not reach its target in time
ERR_BOUNDS = 2            # a debug bounds check refused an access
ERR_PEER_INDEX = 3        # a peer index outside the group
ERR_PIPELINE_TIMEOUT = 4  # an on-chip barrier inside a GEMM/attention pipeline did not complete

_NAMES = {
    ERR_WAIT_TIMEOUT: "wait timed out",
    ERR_BOUNDS: "bounds check failed",
    ERR_PEER_INDEX: "peer index out of range",
    ERR_PIPELINE_TIMEOUT: "kernel pipeline wait timed out",
}


class OdcError(RuntimeError):
    pass


class OdcTimeoutError(OdcError):
    pass


class OdcBoundsError(OdcError):
    pass


class PeerFailure(OdcError):
    pass


def check_status_word(code: int, detail: int = 0, seen: int = 0) -> None:
    if code == OK:
        return
    msg = f"device reported '{_NAMES.get(code, code)}' (detail={detail}, observed={seen})"
    if code in (ERR_WAIT_TIMEOUT, ERR_PIPELINE_TIMEOUT):
        raise OdcTimeoutError(msg)
    if code in (ERR_BOUNDS, ERR_PEER_INDEX):
        raise OdcBoundsError(msg)
    raise OdcError(msg)


class Heartbeat:
    """Host-side liveness through a ``torch.distributed`` store.

    Each rank publishes ``(step, wall time)`` between steps; before a rank enters a phase that
    depends on its peers it can ask which peers have stopped publishing.  No GPU work is
    involved, so a dead peer is noticed before the next kernel is launched rather than by a
    device wait running out.
    """

    def __init__(self, store, rank: int, world: int, prefix: str = "odc_hb"):
        self.store, self.rank, self.world, self.prefix = store, rank, world, prefix
        self._thread = None
        self._stop = None
        self._step = 0

    def beat(self, step: Optional[int] = None) -> None:
        if step is not None:
            self._step = step
        self.store.set(f"{self.prefix}/{self.rank}", f"{self._step}:{time.time():.3f}")

    def start_background(self, interval_s: float = 1.0) -> None:
        """Publish from a daemon thread every ``interval_s`` seconds until ``stop_background`` (or process exit)."""
        import threading
        if self._thread is not None:
            return
        self._stop = threading.Event()
        self.beat()

        def run():
            while not self._stop.wait(interval_s):
                try:
                    self.beat()
                except Exception:
                    return  # the store went away with the job

        self._thread = threading.Thread(target=run, name="odc-heartbeat", daemon=True)
        self._thread.start()

    def stop_background(self) -> None:
        if self._thread is not None:
            self._stop.set()
            self._thread.join(timeout=2.0)
            self._thread = None

    def mark_leaving(self) -> None:
        self.stop_background()  # or the publishing thread would overwrite the farewell
        self.store.set(f"{self.prefix}/{self.rank}", "gone:0")

    def read(self) -> Dict[int, Optional[tuple]]:
        out: Dict[int, Optional[tuple]] = {}
        for r in range(self.world):
            key = f"{self.prefix}/{r}"
            try:
                if hasattr(self.store, "check") and not self.store.check([key]):
                    out[r] = None
                    continue
                step, ts = self.store.get(key).decode().split(":")
                out[r] = (step, float(ts))
            except Exception:
                out[r] = None
        return out

    def dead_peers(self, max_age_s: float, missing_is_dead: bool = True) -> List[int]:
        """Peers that never published (unless ``missing_is_dead`` is off: a job that is still starting up), said they
        were leaving, or whose last beat is older than ``max_age_s``."""
        now = time.time()
        dead = []
        for r, v in self.read().items():
            if r == self.rank:
                continue
            if v is None:
                if missing_is_dead:
                    dead.append(r)
            elif v[0] == "gone" or now - v[1] > max_age_s:
                dead.append(r)
        return dead

    def assert_alive(self, max_age_s: float, missing_is_dead: bool = True) -> None:
        dead = self.dead_peers(max_age_s, missing_is_dead)
        if dead:
            raise PeerFailure(f"rank {self.rank}: peers {dead} stopped publishing heartbeats")
