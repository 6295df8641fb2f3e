"""Block-exchange backends for plan interpreters.

A ``CommLaunchInstr`` names, per peer, an ordered list of blocks to send and to receive; both ends
list them in the same order.  Two backends implement that contract:

* ``MailboxComm`` - ranks are threads of one process exchanging tensors through queues.  Used to
  run N-device plans on one CPU (tests, dry runs) and to inject failures without any GPU.
* ``TorchDistComm`` - ``torch.distributed`` point-to-point (gloo on CPU, NCCL on GPU), one
  ``batch_isend_irecv`` per launch.

Waits are bounded: a peer that never sends raises ``CommTimeout`` instead of blocking forever.
"""
from __future__ import annotations

import queue
import threading
from typing import Dict, List, Optional, Sequence, Tuple

import torch


class CommTimeout(RuntimeError):
    pass


class MailboxHub:
    """Shared by all ranks of an in-process run."""

    def __init__(self, world_size: int, timeout_s: float = 30.0):
        self.world_size = world_size
        self.timeout_s = timeout_s
        self._queues: Dict[Tuple[int, int, str], "queue.Queue"] = {}
        self._lock = threading.Lock()
        self._barrier = threading.Barrier(world_size)
        self.dropped: set = set()  # (src, dst, key) messages to swallow (fault injection)

    def q(self, src: int, dst: int, key: str) -> "queue.Queue":
        with self._lock:
            return self._queues.setdefault((src, dst, key), queue.Queue())


class MailboxComm:
    def __init__(self, hub: MailboxHub, rank: int):
        self.hub, self.rank = hub, rank
        self._pending: Dict[str, List[Tuple[int, torch.Tensor]]] = {}

    def launch(self, key: str, sends: Sequence[Tuple[int, torch.Tensor]], recvs: Sequence[Tuple[int, torch.Tensor]]):
        for peer, t in sends:
            if (self.rank, peer, key) in self.hub.dropped:
                continue
            self.hub.q(self.rank, peer, key).put(t.detach().clone())
        self._pending[key] = list(recvs)

    def wait(self, key: str) -> None:
        for peer, dst in self._pending.pop(key, []):
            try:
                src = self.hub.q(peer, self.rank, key).get(timeout=self.hub.timeout_s)
            except queue.Empty:
                raise CommTimeout(f"rank {self.rank}: nothing arrived from rank {peer} for exchange {key!r} "
                                  f"within {self.hub.timeout_s}s") from None
            dst.copy_(src.reshape(dst.shape))

    def barrier(self) -> None:
        try:
            self.hub._barrier.wait(timeout=self.hub.timeout_s)
        except threading.BrokenBarrierError:
            raise CommTimeout(f"rank {self.rank}: barrier not reached by all ranks") from None


class TorchDistComm:
    def __init__(self, group=None, ranks: Optional[Sequence[int]] = None):
        import torch.distributed as dist
        self.dist = dist
        self.group = group
        # plan ranks are group-local; translate to global ranks for p2p calls
        self.ranks = list(ranks) if ranks is not None else None
        self._pending: Dict[str, Tuple[list, List[Tuple[torch.Tensor, torch.Tensor]]]] = {}

    def _global(self, r: int) -> int:
        return self.ranks[r] if self.ranks is not None else r

    def launch(self, key: str, sends, recvs):
        dist = self.dist
        ops, copies = [], []
        for peer, t in sends:
            ops.append(dist.P2POp(dist.isend, t.contiguous(), self._global(peer), group=self.group))
        for peer, dst in recvs:
            tmp = dst if dst.is_contiguous() else torch.empty(dst.shape, dtype=dst.dtype, device=dst.device)
            if tmp is not dst:
                copies.append((tmp, dst))
            ops.append(dist.P2POp(dist.irecv, tmp, self._global(peer), group=self.group))
        reqs = dist.batch_isend_irecv(ops) if ops else []
        self._pending[key] = (reqs, copies)

    def wait(self, key: str) -> None:
        reqs, copies = self._pending.pop(key, ([], []))
        for r in reqs:
            r.wait()
        for tmp, dst in copies:
            dst.copy_(tmp)

    def barrier(self) -> None:
        self.dist.barrier(group=self.group)
