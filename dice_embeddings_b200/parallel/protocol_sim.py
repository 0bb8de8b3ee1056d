"""Host-side replay of the sharded training step's communication protocol with Python threads.

The GPU step (:mod:`dice_embeddings_b200.parallel.sharded_engine`) lets kernels read and write peer memory directly
and orders them with three bounded device barriers per step.  There is no memory checker for that on the target machines, so
the same sequence of reads, writes, reductions and barriers is replayed here on NumPy arrays, one thread per rank:

* :class:`SimHeap` – one named buffer per rank, visible to all ranks; every access is tagged with the *phase* of
  the accessing rank, and an access that races with another rank's access of a conflicting kind in a phase that
  no barrier separates raises :class:`ProtocolHazard` (deterministically: the check uses phase numbers, not timing);
* :class:`SimBarrier` – the signal-counter barrier of ``p2p_barrier_kernel``: add 1 to ``sig[peer][rank]`` on every
  peer, then wait until ``sig[rank][p] >= count`` for all ``p``, giving up after a bounded number of polls with
  status ``TIMEOUT_PEER``;
* :func:`run_sharded_step` – the step itself (lookup by peer reads, broadcast of queries and batch indices by peer
  writes, scoring of the local shard, owner-side backward that sums a query's gradient partials from all ranks where
  its head row lives, replicated update of the relation table from all ranks' gradient buffers) on a toy DistMult model, compared by the
  tests against a single-process computation; faults (a rank that never arrives, a dropped signal, a removed
  barrier) are injected on the host.
"""
from __future__ import annotations

import threading
import time
from typing import Callable, Dict, List, Optional, Sequence

import numpy as np

ST_OK, ST_TIMEOUT_PEER = 0, 4


class ProtocolHazard(RuntimeError):
    pass


class PeerTimeout(RuntimeError):
    def __init__(self, rank: int, missing: Sequence[int]):
        super().__init__(f"rank {rank}: barrier wait gave up, no signal from ranks {list(missing)}")
        self.rank, self.missing = rank, list(missing)


class SimHeap:
    """Symmetric buffers with phase-tagged access tracking.

    For every (name, owner) buffer the heap remembers, per phase, which ranks read, wrote or reduced into it.
    Within one phase these combinations are legal: many readers; many reducers (commutative adds); one writer per
    disjoint region (callers pass ``region`` keys; the same region written twice in a phase is a hazard).  A read in
    a phase in which another rank writes or reduces the same buffer is a hazard, and so is one rank's write next to
    another rank's reduce (a rank's own accesses follow stream order)."""

    def __init__(self, world: int):
        self.world = world
        self.bufs: Dict[str, List[np.ndarray]] = {}
        self.phase = [0] * world
        self._log: Dict[tuple, Dict[str, set]] = {}
        self._lock = threading.Lock()

    def alloc(self, name: str, shape, dtype=np.float64) -> None:
        self.bufs[name] = [np.zeros(shape, dtype=dtype) for _ in range(self.world)]

    def _note(self, kind: str, name: str, owner: int, rank: int, region=None) -> None:
        with self._lock:
            key = (name, owner, self.phase[rank])
            e = self._log.setdefault(key, {"r": set(), "w": set(), "a": set(), "regions": set()})
            if kind == "r" and (e["w"] - {rank} or e["a"] - {rank}):
                raise ProtocolHazard(f"rank {rank} reads {name}@{owner} while {e['w'] | e['a']} modify it (phase {key[2]})")
            if kind in ("w", "a") and e["r"] - {rank}:
                raise ProtocolHazard(f"rank {rank} modifies {name}@{owner} while {e['r']} read it (phase {key[2]})")
            if kind == "w" and e["a"] - {rank} or kind == "a" and e["w"] - {rank}:   # one rank's own accesses are stream-ordered
                raise ProtocolHazard(f"write and reduce of {name}@{owner} in one phase ({key[2]})")
            if kind == "w":
                if region in e["regions"]:
                    raise ProtocolHazard(f"region {region} of {name}@{owner} written twice in phase {key[2]}")
                e["regions"].add(region)
            e[kind].add(rank)

    def read(self, name: str, owner: int, rank: int) -> np.ndarray:
        self._note("r", name, owner, rank)
        return self.bufs[name][owner]

    def write(self, name: str, owner: int, rank: int, index, value, region=None) -> None:
        self._note("w", name, owner, rank, region if region is not None else ("rank", rank))
        self.bufs[name][owner][index] = value

    def add(self, name: str, owner: int, rank: int, index, value) -> None:
        self._note("a", name, owner, rank)
        with self._lock:  # the device uses atomic adds
            np.add.at(self.bufs[name][owner], index, value)

    def next_phase(self, rank: int) -> None:
        self.phase[rank] += 1


class SimBarrier:
    def __init__(self, world: int, poll_limit: int = 20000, poll_sleep: float = 1e-4,
                 drop: Optional[Callable[[int, int, int], bool]] = None):
        self.world, self.poll_limit, self.poll_sleep = world, poll_limit, poll_sleep
        self.sig = np.zeros((world, world), dtype=np.int64)   # sig[owner][sender]
        self.count = [0] * world
        self.drop = drop or (lambda sender, peer, count: False)
        self._lock = threading.Lock()
        self.abort = threading.Event()   # set when a rank has failed: the others stop waiting at once

    def arrive_and_wait(self, rank: int) -> int:
        """Returns ``ST_OK`` or ``ST_TIMEOUT_PEER`` (never blocks for ever)."""
        self.count[rank] += 1
        c = self.count[rank]
        for peer in range(self.world):
            if not self.drop(rank, peer, c):
                with self._lock:
                    self.sig[peer][rank] += 1
        for _ in range(self.poll_limit):
            if all(self.sig[rank][p] >= c for p in range(self.world)):
                return ST_OK
            if self.abort.is_set():
                break
            time.sleep(self.poll_sleep)
        return ST_TIMEOUT_PEER

    def missing(self, rank: int) -> List[int]:
        return [p for p in range(self.world) if self.sig[rank][p] < self.count[rank]]


def reference_step(E, R, h, r, labels, lr):
    """One SGD step of DistMult KvsAll with mean BCE-with-logits on full arrays (the oracle)."""
    q = E[h] * R[r]
    s = q @ E.T
    sig = 1.0 / (1.0 + np.exp(-s))
    loss = np.mean(np.maximum(s, 0) - s * labels + np.log1p(np.exp(-np.abs(s))))
    ds = (sig - labels) / s.size
    gE = ds.T @ q
    dq = ds @ E
    np.add.at(gE, h, dq * R[r])
    gR = np.zeros_like(R)
    np.add.at(gR, r, dq * E[h])
    return E - lr * gE, R - lr * gR, loss


def run_sharded_step(world: int, E, R, h, r, labels, lr, skip_barrier: Optional[str] = None,
                     absent_rank: Optional[int] = None, drop: Optional[Callable[[int, int, int], bool]] = None,
                     poll_limit: int = 20000, steps: int = 1):
    """Replay the sharded step.  ``h, r, labels`` hold the *global* batch (rank ``k`` owns its rows
    ``[k·b, (k+1)·b)``); entity ``e`` lives on rank ``e % world`` at row ``e // world``.

    Four barriers per step, three of them on the critical path of the device code (``S2`` and ``S2b`` run on a
    branch beside the entity-role scoring launch, which needs nothing from the other ranks):

    * ``S1`` after the lookup (peer reads of head rows) and the broadcast of query rows and batch indices,
    * ``S2`` after the query-role scoring pass over the local shard (every rank's partial ``dQ`` is complete),
    * ``S2b`` after the *owner-side* backward (the owner of a head row sums that query's ``dQ`` partials from all
      ranks, applies the chain rule and adds the row gradient to its own shard, so no row gradient crosses the
      fabric); behind it the replicated relation table is updated from all ranks' gradient buffers and ``dQ`` is
      cleared,
    * ``S3`` after the entity-role scoring pass (loss, dense gradient of the shard) and the update of the local
      entity shard; behind it the loss partials are summed.  ``S3`` also orders the next step's peer reads of the
      updated entity rows, so no barrier opens a step.

    Fault injection: ``skip_barrier`` ∈ {"S1","S2","S2b","S3"} removes that barrier on every rank (the phases it
    separated then count as one, which is what the hazard check looks at); ``absent_rank`` never starts;
    ``drop(sender, peer, count)`` suppresses single barrier signals.  ``steps`` repeats the step on the same batch.
    Returns ``(E_new, R_new, loss)`` assembled from the shards, or raises the first rank failure."""
    W = world
    NE, D = E.shape
    B = h.shape[0]
    assert B % W == 0
    b = B // W
    rows = (NE + W - 1) // W
    heap = SimHeap(W)
    for name, shape, dt in (("E", (rows, D), np.float64), ("Q", (B, D), np.float64), ("dQ", (B, D), np.float64),
                            ("gR", R.shape, np.float64), ("loss", (1,), np.float64), ("h", (B,), np.int64),
                            ("r", (B,), np.int64)):
        heap.alloc(name, shape, dt)
    gE = [np.zeros((rows, D)) for _ in range(W)]               # row gradients never leave their owner
    Rrep = [R.copy() for _ in range(W)]
    for e in range(NE):
        heap.bufs["E"][e % W][e // W] = E[e]
    bar = SimBarrier(W, poll_limit=poll_limit, drop=drop)
    errors: List[Optional[BaseException]] = [None] * W
    losses = [0.0] * W

    def barrier(rank: int, name: str) -> None:
        if skip_barrier == name:
            return
        if bar.arrive_and_wait(rank) != ST_OK:
            raise PeerTimeout(rank, bar.missing(rank))
        heap.next_phase(rank)

    def work(rank: int) -> None:
        try:
            lo = rank * b
            my_h, my_r = h[lo:lo + b], r[lo:lo + b]
            own = np.arange(rank, NE, W)                       # global ids of the local rows
            n_own = len(own)
            for _ in range(steps):
                # lookup by peer reads + compose + broadcast of the queries and of the batch indices by peer writes
                hv = np.stack([heap.read("E", int(e) % W, rank)[int(e) // W] for e in my_h])
                q = hv * Rrep[rank][my_r]
                for peer in range(W):
                    heap.write("Q", peer, rank, slice(lo, lo + b), q, region=("rows", lo))
                    heap.write("h", peer, rank, slice(lo, lo + b), my_h, region=("rows", lo))
                    heap.write("r", peer, rank, slice(lo, lo + b), my_r, region=("rows", lo))
                barrier(rank, "S1")                            # all queries have landed; last step's sums were read
                heap.write("gR", rank, rank, slice(None), 0.0)
                heap.write("loss", rank, rank, slice(None), 0.0)
                Eloc = heap.read("E", rank, rank)[:n_own]
                Q = heap.read("Q", rank, rank)
                s = Q @ Eloc.T                                 # [B, local rows]
                y = labels[:, own]
                sig = 1.0 / (1.0 + np.exp(-s))
                ds = (sig - y) / (B * NE)
                heap.add("dQ", rank, rank, np.arange(B), ds @ Eloc)   # query role: partial over this shard, kept locally
                barrier(rank, "S2")                            # every rank's partial of dQ is complete
                # owner-side backward: queries whose head row lives here; their dQ is the sum of all ranks' partials
                h_all, r_all = heap.read("h", rank, rank), heap.read("r", rank, rank)
                mine = np.nonzero(h_all % W == rank)[0]
                dq = sum(heap.read("dQ", p, rank)[mine] for p in range(W)) if len(mine) else np.zeros((0, D))
                hv_own = heap.read("E", rank, rank)[h_all[mine] // W]
                np.add.at(gE[rank], h_all[mine] // W, dq * Rrep[rank][r_all[mine]])
                heap.add("gR", rank, rank, r_all[mine], dq * hv_own)
                barrier(rank, "S2b")                           # every rank's backward is through
                gR = sum(heap.read("gR", p, rank) for p in range(W))     # replicated all-reduce by peer reads
                Rrep[rank] = Rrep[rank] - lr * gR
                heap.write("dQ", rank, rank, slice(None), 0.0)
                # entity role (on the device it runs beside S2, the backward and S2b): loss and dense gradient
                heap.add("loss", rank, rank, 0, np.sum(np.maximum(s, 0) - s * y + np.log1p(np.exp(-np.abs(s)))))
                gE[rank][:n_own] += ds.T @ Q
                g_own = gE[rank].copy()                        # the update follows this rank's own reads in stream order
                heap.write("E", rank, rank, slice(None), heap.bufs["E"][rank] - lr * g_own)
                gE[rank][:] = 0.0
                barrier(rank, "S3")                            # shards updated, loss partials complete
                loss = sum(float(heap.read("loss", p, rank)[0]) for p in range(W)) / (B * NE)
                losses[rank] = loss
        except BaseException as exc:  # noqa: BLE001 - reported to the caller
            errors[rank] = exc
            bar.abort.set()

    threads = [threading.Thread(target=work, args=(k,), daemon=True) for k in range(W) if k != absent_rank]
    for t in threads:
        t.start()
    for t in threads:
        t.join()
    failed = [e for e in errors if e is not None]
    if failed:  # the root cause first: a hazard on one rank makes the others time out at their next barrier
        failed.sort(key=lambda e: 0 if isinstance(e, ProtocolHazard) else 1)
        raise failed[0]
    E_new = np.zeros_like(E)
    for e in range(NE):
        E_new[e] = heap.bufs["E"][e % W][e // W]
    return E_new, Rrep[0], losses[0]
