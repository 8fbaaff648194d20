"""Host-side failure detection for multi-rank jobs: heartbeats, bounded barriers, clean teardown.

The fused collective kernels of this library spin (bounded) on flags that peers write, so a rank that
has gone away must be noticed on the HOST, before the survivors launch the next step.  This module is
that layer.  It uses only the ``torch.distributed`` key-value store (the rendezvous store every job
already has), so it works the same under NCCL and under gloo and never touches a GPU:

* :class:`RankMonitor` -- every rank publishes ``(step, wall time)`` under its own key;
  ``check_peers()`` reads the others' keys and raises :class:`PeerLostError` naming the ranks whose
  heartbeat is older than the limit or who announced that they are leaving.
* :func:`bounded_barrier` -- a store barrier with a time limit: all ranks arrive or the call raises
  :class:`PeerLostError` with the ranks that did not, instead of hanging in a collective.
* :func:`recover` -- tear down the communication contexts of the fused kernels (symmetric buffers,
  flags) so that the job can rebuild them on a new group (the reference allows the same through
  ``destroy_ub`` and a second ``initialize_ub``, ``pytorch/module/base.py:594-604``).

Reference behaviour for comparison: Userbuffers prints and carries on with wrong data when a device
wait runs out (``common/comm_gemm_overlap/userbuffers/userbuffers.cu:91-97``); here the device wait
records a status word that ``check_status()`` turns into an exception, and this module turns a
missing rank into an exception before the wait is ever launched.
"""
from __future__ import annotations

import time
from typing import Iterable, List, Optional

import torch.distributed as dist


class PeerLostError(RuntimeError):
    """One or more ranks of the job stopped answering (or announced their exit)."""

    def __init__(self, ranks: Iterable[int], what: str):
        self.ranks = sorted(set(ranks))
        super().__init__(f"{what}: rank(s) {self.ranks} did not answer")


def _default_store():
    try:
        return dist.distributed_c10d._get_default_store()
    except Exception as e:  # noqa: BLE001
        raise RuntimeError("torch.distributed is not initialised: no rendezvous store to use") from e


class RankMonitor:
    """Heartbeats over the rendezvous store.

    Call :meth:`beat` once per step (cheap: one ``set``) and :meth:`check_peers` before launching work
    that waits on peers.  A rank that ends on purpose calls :meth:`leave` BETWEEN steps, with none of its
    kernels or collectives in flight; the others then see it at their next check.
    """

    def __init__(self, rank: Optional[int] = None, world_size: Optional[int] = None, *, store=None,
                 prefix: str = "teb200/hb", max_silence_s: float = 30.0):
        self.store = store if store is not None else _default_store()
        self.rank = dist.get_rank() if rank is None else rank
        self.world = dist.get_world_size() if world_size is None else world_size
        self.prefix = prefix
        self.max_silence_s = max_silence_s
        self.step = 0
        self.beat()

    def _key(self, r: int) -> str:
        return f"{self.prefix}/{r}"

    def beat(self, step: Optional[int] = None) -> None:
        self.step = self.step + 1 if step is None else step
        self.store.set(self._key(self.rank), f"{self.step}:{time.time():.3f}:alive")

    def leave(self) -> None:
        """Announce a deliberate exit (call between steps)."""
        self.store.set(self._key(self.rank), f"{self.step}:{time.time():.3f}:left")

    def peer_state(self, r: int):
        """(step, age in seconds, state) of rank ``r``; ``(None, inf, 'never')`` if it never reported."""
        try:
            if not self.store.check([self._key(r)]):
                return None, float("inf"), "never"
            step, t, state = self.store.get(self._key(r)).decode().split(":")
            return int(step), time.time() - float(t), state
        except Exception:  # noqa: BLE001  (store unreachable counts as silence)
            return None, float("inf"), "unreachable"

    def lost_peers(self) -> List[int]:
        lost = []
        for r in range(self.world):
            if r == self.rank:
                continue
            _, age, state = self.peer_state(r)
            if state != "alive" or age > self.max_silence_s:
                lost.append(r)
        return lost

    def check_peers(self) -> None:
        lost = self.lost_peers()
        if lost:
            raise PeerLostError(lost, "heartbeat check")


def bounded_barrier(tag: str, rank: Optional[int] = None, world_size: Optional[int] = None, *, store=None,
                    timeout_s: float = 30.0, poll_s: float = 0.01) -> None:
    """All ranks call this with the same ``tag`` (use a new tag per barrier, e.g. the step number).
    Returns when every rank has arrived; raises :class:`PeerLostError` naming the missing ranks when
    ``timeout_s`` passes first.  Host only: nothing is launched on a GPU."""
    store = store if store is not None else _default_store()
    rank = dist.get_rank() if rank is None else rank
    world = dist.get_world_size() if world_size is None else world_size
    store.set(f"teb200/bar/{tag}/{rank}", "1")
    keys = [f"teb200/bar/{tag}/{r}" for r in range(world)]
    deadline = time.time() + timeout_s
    while True:
        try:
            missing = [r for r, k in enumerate(keys) if not store.check([k])]
        except Exception:  # noqa: BLE001
            missing = [r for r in range(world) if r != rank]
        if not missing:
            return
        if time.time() > deadline:
            raise PeerLostError(missing, f"barrier '{tag}' after {timeout_s:.1f} s")
        time.sleep(poll_s)


def recover() -> None:
    """Drop every communication context of the fused kernels (tensor-parallel GEMM contexts, expert-
    and context-parallel workspaces).  The caller then destroys the process group, forms a new one with
    the surviving ranks and calls ``initialize_ub`` / the model constructors again."""
    from . import comm_gemm

    comm_gemm.destroy_ub()
    try:
        from . import expert_parallel

        expert_parallel._EP_CONTEXTS.clear()
    except Exception:  # noqa: BLE001
        pass
