"""Status words of the peer-memory kernels, surfaced to the host without a synchronisation.

The kernels that wait on other ranks (fused ZeRO step, distributed Muon gather / scatter) give every wait a
cycle budget; when it runs out they write a code into a device word and return.  Reading that word with
``.item()`` after every step would stall the host once per step, and never reading it lets a failed step pass
unnoticed.  ``StatusMailbox`` does neither: after a step's launches it queues, on the launching stream, a copy of
the words into pinned host memory, a reset of the device words and an event.  The next ``step()`` /
``zero_grad()`` looks at the posts whose event has completed (``Event.query``, no wait) and raises if a code was
recorded; a step that finds the previous post still in flight simply leaves it for the call after.

(The reference has no device-side waits and therefore nothing of this kind; its collectives fail through the
process group's own timeout.)
"""

from __future__ import annotations

from collections import deque
from typing import Callable, Deque, List, Optional, Tuple

import torch

ZS_OK, ZS_ENTRY_TIMEOUT, ZS_EXIT_TIMEOUT, ZS_GO_TIMEOUT = 0, 1, 2, 3
STATUS_TEXT = {ZS_ENTRY_TIMEOUT: "a peer never signalled that its gradients were final (nothing was updated)",
               ZS_EXIT_TIMEOUT: "a peer never signalled that it finished writing parameters",
               ZS_GO_TIMEOUT: "the kernel's own go-word never arrived"}


class PeerStepError(RuntimeError):
    """A bounded wait of a peer-memory kernel ran out.  ``codes`` maps status word index -> code."""

    def __init__(self, message: str, codes):
        super().__init__(message)
        self.codes = dict(codes)


class StatusMailbox:
    def __init__(self, device: torch.device, words: int = 1, depth: int = 4):
        self.device = torch.device(device)
        self.words = torch.zeros(max(1, int(words)), dtype=torch.int32, device=self.device)
        self._cuda = self.device.type == "cuda"
        self._host = [torch.zeros(self.words.numel(), dtype=torch.int32).pin_memory() if self._cuda
                      else torch.zeros(self.words.numel(), dtype=torch.int32) for _ in range(max(2, depth))]
        self._free: Deque[int] = deque(range(len(self._host)))
        self._posts: Deque[Tuple[Optional["torch.cuda.Event"], int, Optional[Callable[[dict], None]]]] = deque()
        self._found: dict = {}      # codes of completed posts that no poll() has reported yet

    def word(self, index: int = 0) -> torch.Tensor:
        """One-element view of status word ``index`` (indices past the end share the last word)."""
        i = min(int(index), self.words.numel() - 1)
        return self.words[i:i + 1]

    def post(self, on_failure: Optional[Callable[[dict], None]] = None) -> None:
        """Queue 'copy the words to the host, then clear them' behind everything launched so far on the current
        stream.  ``on_failure(codes)`` runs on the host when the copy shows a non-zero word, before the error is
        raised (the optimizers use it to take back the step count of launches that updated nothing)."""
        if not self._free:              # every host slot still in flight: fold the oldest post in first
            self._drain(block_oldest=True)
        slot = self._free.popleft()
        if self._cuda:
            self._host[slot].copy_(self.words, non_blocking=True)
            self.words.zero_()
            ev = torch.cuda.Event()
            ev.record(torch.cuda.current_stream(self.device))
        else:
            self._host[slot].copy_(self.words)
            self.words.zero_()
            ev = None
        self._posts.append((ev, slot, on_failure))

    def _drain(self, block_oldest: bool = False, block_all: bool = False) -> None:
        """Fold the codes of completed posts (oldest first) into ``self._found``."""
        found = self._found
        first = True
        while self._posts:
            ev, slot, cb = self._posts[0]
            if ev is not None and not ev.query():
                if block_all or (block_oldest and first):
                    ev.synchronize()
                else:
                    break
            first = False
            self._posts.popleft()
            vals = self._host[slot].tolist()
            self._free.append(slot)
            codes = {i: int(v) for i, v in enumerate(vals) if v != 0}
            if codes:
                if cb is not None:
                    cb(codes)
                for i, v in codes.items():
                    found.setdefault(i, v)

    def poll(self, who: str = "peer kernel", rank: int = 0, wait: bool = False) -> None:
        """Raise ``PeerStepError`` if a completed post recorded a failure.  ``wait=True`` first waits for every
        outstanding post (one host synchronisation: ``check_status()`` of the optimizers)."""
        self._drain(block_all=wait)
        codes, self._found = self._found, {}
        if codes:
            worst = next(iter(codes.values()))
            what = STATUS_TEXT.get(worst, f"status {worst}")
            raise PeerStepError(f"{who} failed on rank {rank}: {what}", codes)

    def read_now(self) -> List[int]:
        """The device words as they are now (host synchronisation; tests and ``check_status``)."""
        return [int(v) for v in self.words.tolist()]
