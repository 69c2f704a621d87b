"""Host-side model of the cross-rank flag protocol of the peer-memory kernels (``csrc/peer_sync.cuh``).

One Python thread stands for one thread block of one rank; the signal pads are plain lists shared by all
threads.  The model follows the device code step by step (entry flags, go word, done counter, exit flags,
epoch comparison with wrap-around, bounded waits that end in a status code) so that the protocol's safety
properties can be checked without a GPU, including the failure cases that must never be provoked on one:
a rank that never arrives, a rank that arrives one launch late, and a stale flag from an earlier epoch.
"""

from __future__ import annotations

import threading
import time
from typing import Callable, List, Optional

MAX_PEERS = 8
GO = 2 * MAX_PEERS
DONE = 2 * MAX_PEERS + 1
NORM_FLAG = 32        # words [32, 40): "rank r's partial sum is in your pad" (epoch)      csrc/zero_fused.cu
NORM_VALUE = 40       # words [40, 48): the partial sums, one slot per rank
PAD_WORDS = 48
OK, ENTRY_TIMEOUT, EXIT_TIMEOUT, GO_TIMEOUT = 0, 1, 2, 3
_MASK = 0xFFFFFFFF


def reached(flag: int, epoch: int) -> bool:
    """``(int32)(flag - epoch) >= 0``: true for the awaited epoch and later ones, across the 2^32 wrap."""
    d = (flag - epoch) & _MASK
    return d < 0x80000000


class World:
    """Signal pads and status words of ``world`` ranks."""

    def __init__(self, world: int):
        self.world = world
        self.pads: List[List[float]] = [[0] * PAD_WORDS for _ in range(world)]
        self.status: List[int] = [OK] * world
        self.lock = threading.Lock()          # stands for the atomicity of single-word accesses and atomicAdd

    def store(self, rank: int, word: int, value: int) -> None:
        with self.lock:
            self.pads[rank][word] = value & _MASK

    def load(self, rank: int, word: int) -> int:
        with self.lock:
            return self.pads[rank][word]

    def store_value(self, rank: int, word: int, value: float) -> None:
        """A 32-bit payload word (the model keeps the number itself instead of its bit pattern)."""
        with self.lock:
            self.pads[rank][word] = value

    def add(self, rank: int, word: int, inc: int) -> int:
        with self.lock:
            old = self.pads[rank][word]
            self.pads[rank][word] = (old + inc) & _MASK
            return old


def _bounded_wait(cond: Callable[[], bool], budget_s: float) -> bool:
    t0 = time.monotonic()
    while not cond():
        if time.monotonic() - t0 > budget_s:
            return False
        time.sleep(0.0002)
    return True


def peer_entry(w: World, rank: int, block: int, epoch: int, budget_s: float) -> bool:
    """Entry round of one thread block; True when every peer arrived at ``epoch``."""
    abort_word = epoch ^ 0x80000000
    if block == 0:
        for r in range(w.world):                                  # threads 0..W-1 of block 0
            w.store(r, rank, epoch)
        ok = all(_bounded_wait(lambda r=r: reached(w.load(rank, r), epoch), budget_s) for r in range(w.world))
        if not ok:
            w.status[rank] = ENTRY_TIMEOUT
        w.store(rank, GO, epoch if ok else abort_word)
    seen: List[int] = [0]

    def verdict() -> bool:
        seen[0] = w.load(rank, GO)
        return seen[0] in (epoch, abort_word)
    if not _bounded_wait(verdict, 2 * budget_s):
        w.status[rank] = GO_TIMEOUT
        return False
    return seen[0] == epoch


def peer_exit(w: World, rank: int, blocks: int, epoch: int, budget_s: float) -> None:
    """Exit round: the last block to finish tells every peer and waits for theirs."""
    if w.add(rank, DONE, 1) != blocks - 1:
        return
    w.store(rank, DONE, 0)
    for r in range(w.world):
        w.store(r, MAX_PEERS + rank, epoch)
    for r in range(w.world):
        if not _bounded_wait(lambda r=r: reached(w.load(rank, MAX_PEERS + r), epoch), budget_s):
            w.status[rank] = EXIT_TIMEOUT


def run_launch(w: World, epoch: int, blocks: int, budget_s: float, body: Callable[[int, int], None],
               ranks: Optional[List[int]] = None, delays: Optional[dict] = None) -> None:
    """One kernel launch on every rank in ``ranks`` (default: all): entry round, ``body(rank, block)``, exit round."""
    ranks = list(range(w.world)) if ranks is None else ranks
    delays = delays or {}

    def block_fn(rank: int, block: int) -> None:
        if delays.get(rank):
            time.sleep(delays[rank])
        if peer_entry(w, rank, block, epoch, budget_s):
            body(rank, block)
            peer_exit(w, rank, blocks, epoch, budget_s)

    threads = [threading.Thread(target=block_fn, args=(r, b)) for r in ranks for b in range(blocks)]
    for t in threads:
        t.start()
    for t in threads:
        t.join()


def norm_exchange(w: World, rank: int, epoch: int, mine: float, budget_s: float,
                  between: Optional[Callable[[int], None]] = None):
    """Model of ``zero_norm_exchange_kernel`` (one thread block per rank, thread r of it talks to rank r): publish
    this rank's partial sum into every rank's pad - value first, then the flag with release semantics -, wait
    (bounded) for every rank's flag in the own pad, add the values up in rank order.  Returns ``(total, ok)``; on a
    wait that ran out the status word is set and the total is zero, as on the device.  ``between(r)`` runs between the
    value store and the flag store towards rank r (tests use it to widen that window)."""
    for r in range(w.world):
        w.store_value(r, NORM_VALUE + rank, mine)
        if between is not None:
            between(r)
        w.store(r, NORM_FLAG + rank, epoch)
    ok, vals = True, []
    for r in range(w.world):
        if _bounded_wait(lambda r=r: reached(w.load(rank, NORM_FLAG + r), epoch), budget_s):
            vals.append(w.load(rank, NORM_VALUE + r))
        else:
            w.status[rank] = ENTRY_TIMEOUT
            ok = False
            vals.append(0.0)
    total = 0.0
    for v in vals:
        total += v
    return (total if ok else 0.0), ok
