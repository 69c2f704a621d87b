"""Training-step engine: the public call a user makes to run one optimizer step.

``TrainEngine.step(tokens)`` takes one rank's batch of token ids in pinned host memory,
copies it to the device, runs ``grad_accum`` micro-batches of forward + backward through
the model, applies the optimizer (for ``ApexWZeRO`` this is the fused reduce-scatter +
update + all-gather kernel), and returns the mean loss as a host float.  The reference
library has no trainer (it is an optimizer library); this is the harness its benchmark
configurations need.
"""

from __future__ import annotations


import torch
from torch import Tensor


class TrainEngine:
    def __init__(self, model, optimizer, micro_batch: int, grad_accum: int, seq_len: int, device):
        self.model, self.opt = model, optimizer
        self.micro_batch, self.grad_accum, self.seq_len = micro_batch, grad_accum, seq_len
        self.device = torch.device(device)
        rows = micro_batch * grad_accum
        self._tokens_dev = torch.empty(rows, seq_len + 1, dtype=torch.int64, device=self.device)
        self._loss_host = torch.empty((), dtype=torch.float32).pin_memory() if self.device.type == "cuda" else torch.empty(())
        self.h2d_bytes_per_step = rows * (seq_len + 1) * 8
        self.d2h_bytes_per_step = 4
        self.steps_done = 0
        #: when a list, every step appends a (start, end) pair of CUDA events around ``optimizer.step()``; reading them
        #: is the caller's business (after a synchronisation), so the step itself stays free of host waits
        self.optimizer_events = None
        for o in (optimizer, getattr(optimizer, "adamw_opt", None), getattr(optimizer, "apexw_opt", None)):
            if o is not None and hasattr(o, "_grad_accum_steps"):      # in-backward stepping waits for the last micro-batch
                o._grad_accum_steps, o._grad_accum_steps_known = grad_accum, True

    def step_device(self, tokens_dev: Tensor) -> Tensor:
        """One optimizer step on tokens that already live on the device; returns the loss tensor (device)."""
        self.opt.zero_grad(set_to_none=False)
        total = torch.zeros((), dtype=torch.float32, device=self.device)
        scale = 1.0 / self.grad_accum
        arm = getattr(self.opt, "arm_overlap", None)
        for i in range(self.grad_accum):
            if arm is not None and i == self.grad_accum - 1:
                arm()          # the optimizer may step buckets of parameters beside this last backward
            mb = tokens_dev[i * self.micro_batch:(i + 1) * self.micro_batch]
            loss = self.model(mb[:, :-1], mb[:, 1:], loss_scale=scale)
            loss.backward()
            total += loss.detach()
        if self.optimizer_events is not None and self.device.type == "cuda":
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            self.opt.step()
            e1.record()
            self.optimizer_events.append((e0, e1))
        else:
            self.opt.step()
        self.steps_done += 1
        return total

    def step(self, tokens_pinned: Tensor) -> float:
        """Full step from pinned host tokens: H2D copy, compute, optimizer, D2H read of the loss."""
        self._tokens_dev.copy_(tokens_pinned, non_blocking=True)
        loss = self.step_device(self._tokens_dev)
        self._loss_host.copy_(loss, non_blocking=True)
        torch.cuda.current_stream(self.device).synchronize() if self.device.type == "cuda" else None
        return float(self._loss_host)

    # ------------------------------------------------------------------ checkpoint / resume

    def state_dict(self) -> dict:
        """Model weights, optimizer state (this rank's shard for a sharded optimizer) and the step count."""
        return {"model": self.model.state_dict(), "optimizer": self.opt.state_dict(), "steps_done": self.steps_done}

    def load_state_dict(self, state: dict) -> None:
        self.model.load_state_dict(state["model"])         # in place: parameters may be views of flat buffers
        self.opt.load_state_dict(state["optimizer"])
        self.steps_done = int(state.get("steps_done", 0))

    def save_checkpoint(self, path: str) -> str:
        """Write this rank's checkpoint and return the file name.  With a sharded optimizer every rank writes its own
        file, ``<path>.rank<r>`` (the optimizer part is what ``reshard_zero_checkpoint`` takes to change the world size)."""
        name = self._rank_file(path)
        torch.save(self.state_dict(), name)
        return name

    def load_checkpoint(self, path: str) -> None:
        self.load_state_dict(torch.load(self._rank_file(path), map_location=self.device, weights_only=False))

    def _rank_file(self, path: str) -> str:
        world = int(getattr(self.opt, "world_size", 1) or 1)
        return f"{path}.rank{int(getattr(self.opt, 'rank', 0))}" if world > 1 else path
