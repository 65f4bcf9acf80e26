"""Elastic data parallelism on the host: who is still in the job, learned before the next launch.

Ranks never learn of a departure from a hung or failed collective. Each rank announces itself
in the rendezvous store every step (``hb/<rank>`` = last finished step) and a rank that leaves
does so between steps, with none of its kernels or collectives in flight, after writing
``left/<rank>``. Before every step the survivors read the store, tell the controller
(``fail_replica`` -> the replica is dead, the gradient accumulation rises so the tokens per
optimizer step stay what the schedule assumes), and continue on a process group of the
survivors. A rank whose heartbeat lags more than ``stale_steps`` behind without a leave notice
is treated the same way.

``ElasticMembership`` is transport-agnostic: it needs a ``torch.distributed`` store
(``TCPStore`` / ``FileStore`` / the default group's store) and builds the survivors' group with
``dist.new_group``. Reference: control/src/lib.rs:208-226 (grad accumulation from live replicas)
and :294-334 (drop / straggler handling) of the reference; the membership protocol is this
package's own.
"""
from __future__ import annotations

import torch.distributed as dist


class ElasticMembership:
    def __init__(self, store, rank: int, world: int, supervisor, *, stale_steps: int = 0,
                 prefix: str = "elastic"):
        self.store, self.rank, self.world = store, int(rank), int(world)
        self.sup = supervisor
        self.stale_steps = int(stale_steps)
        self.prefix = prefix
        self.live = list(range(self.world))
        self.group = None                 # None = the default group while everyone is in
        self._groups: dict[tuple, object] = {}
        self.store.set(self._k("hb", self.rank), "0")

    def _k(self, kind: str, rank: int) -> str:
        return f"{self.prefix}/{kind}/{rank}"

    def heartbeat(self, step: int) -> None:
        self.store.set(self._k("hb", self.rank), str(int(step)))

    def leave(self, step: int) -> None:
        """Announce departure. Call between steps only; the caller then stops taking part."""
        self.store.set(self._k("left", self.rank), str(int(step)))

    def _has(self, key: str) -> bool:
        try:
            return bool(self.store.check([key]))
        except Exception:          # a store without check(): treat a missing key as absent
            return False

    def refresh(self, step: int) -> dict:
        """Before a step: drop ranks that announced leaving (or went silent), re-form the
        group when the membership changed. Every survivor sees the same store contents at the
        same step boundary (the previous step's collective ordered them), so they agree.
        Returns ``{"live", "changed", "grad_accumulation", "group"}``."""
        gone = []
        for r in list(self.live):
            if r == self.rank:
                continue
            if self._has(self._k("left", r)):
                gone.append(r)
            elif self.stale_steps > 0:
                last = int(self.store.get(self._k("hb", r)).decode())
                if step - last > self.stale_steps:
                    gone.append(r)
        for r in gone:
            self.live.remove(r)
            if self.sup.replicas[r] in self.sup.live():      # not already voted out or drained
                self.sup.replica_left(self.sup.replicas[r])
        if gone:
            key = tuple(self.live)
            if key not in self._groups:
                # new_group is collective over the ranks that call it only when told so
                self._groups[key] = dist.new_group(ranks=list(key), use_local_synchronization=True)
            self.group = self._groups[key]
        return {"live": list(self.live), "changed": bool(gone),
                "grad_accumulation": self.sup.grad_accumulation(), "group": self.group}
