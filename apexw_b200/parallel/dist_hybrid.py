"""Distributed hybrid optimizer: DistMuon for the hidden matrices, ApexWZeRO for everything else.

``HybridApexW`` (reference: apexw/hybrid.py) orthogonalises every matrix on every rank; ``DistMuon``
(apexw/fsdp.py:112-272) shards that work but covers matrices only.  Multi-GPU hybrid pretraining needs both
halves sharded, so this class applies the hybrid partition rules once and drives the two sharded optimizers
as one: on CUDA both halves step through peer-memory kernels (gather -> Newton-Schulz -> scatter for the
matrices, reduce-scatter -> update -> all-gather for the rest), with no NCCL call in the step.
"""

from __future__ import annotations

from typing import Any, Dict, Optional

import torch
from torch.optim.optimizer import Optimizer

from ..optim.hybrid import partition_parameters_for_hybrid
from .fsdp import DistMuon
from .zero import ApexWZeRO


class DistHybridApexW(Optimizer):
    """``DistMuon`` + ``ApexWZeRO`` behind one ``step`` / ``zero_grad`` / ``state_dict``.

    A ``torch.optim.Optimizer``: ``param_groups`` are the two halves' own group dictionaries, so learning-rate
    schedulers and manual edits reach them.

    ``lr`` / ``weight_decay`` / ``betas`` / ``precision`` go to the AdamW half; ``muon_lr`` (default 0.02),
    ``muon_momentum``, ``muon_weight_decay``, ``ns_steps`` and ``nesterov`` to the Muon half.  Extra keyword
    arguments are forwarded to ``ApexWZeRO``.
    """

    _step_supports_amp_scaling = True

    def __init__(self, model_or_params, lr: float = 1e-3, weight_decay: float = 1e-2, betas=(0.9, 0.95),
                 precision: str = "compact", muon_lr: float = 2e-2, muon_momentum: float = 0.95,
                 muon_weight_decay: Optional[float] = None, ns_steps: int = 5, nesterov: bool = True,
                 process_group: Optional[Any] = None, min_muon_dim: int = 32, exclude_embeddings: bool = True,
                 fused: Optional[bool] = None, **zero_kwargs):
        muon_params, adamw_params = partition_parameters_for_hybrid(model_or_params, min_muon_dim, exclude_embeddings)
        if not muon_params or not adamw_params:
            raise ValueError("DistHybridApexW needs at least one Muon-eligible matrix and one other parameter; "
                             "use DistMuon or ApexWZeRO directly otherwise")
        self._min_muon_dim, self._exclude_embeddings = min_muon_dim, exclude_embeddings
        super().__init__(list(muon_params) + list(adamw_params), dict(lr=lr, muon_lr=muon_lr, weight_decay=weight_decay))
        self.muon_opt = DistMuon(muon_params, lr=muon_lr, momentum=muon_momentum, nesterov=nesterov,
                                 weight_decay=weight_decay if muon_weight_decay is None else muon_weight_decay,
                                 ns_steps=ns_steps, process_group=process_group, fused=fused,
                                 reduce_gradients=zero_kwargs.get("reduce_gradients", True))   # as the AdamW half
        self.adamw_opt = ApexWZeRO(adamw_params, lr=lr, weight_decay=weight_decay, betas=betas, precision=precision,
                                   process_group=process_group, fused=fused, **zero_kwargs)
        if self.muon_opt._fused and zero_kwargs.get("fused_wgrad"):
            for p in muon_params:              # let grad-accumulating linear layers write into the flat buffer too
                p.main_grad = p.grad
        self.param_groups = self.muon_opt.param_groups + self.adamw_opt.param_groups     # the same dictionaries

    def add_param_group(self, param_group: dict) -> None:
        if not hasattr(self, "muon_opt"):
            return super().add_param_group(param_group)         # the base constructor's own call
        params = param_group["params"]
        params = [params] if isinstance(params, torch.Tensor) else list(params)
        muon, rest = partition_parameters_for_hybrid(params, self._min_muon_dim, self._exclude_embeddings)
        extra = {k: v for k, v in param_group.items() if k != "params"}
        for opt, ps in ((self.muon_opt, muon), (self.adamw_opt, rest)):
            if ps:
                opt.add_param_group({**extra, "params": ps})
        self.param_groups = self.muon_opt.param_groups + self.adamw_opt.param_groups

    @torch.no_grad()
    def step(self, closure=None):
        loss = None
        if closure is not None:
            with torch.enable_grad():
                loss = closure()
        # ``torch.amp.GradScaler`` sets these two attributes before ``step`` and deletes them afterwards (and multiplies
        # into an existing ``grad_scale``), so they are never left behind as None
        grad_scale, found_inf = getattr(self, "grad_scale", None), getattr(self, "found_inf", None)
        try:
            for opt in (self.muon_opt, self.adamw_opt):
                if grad_scale is not None:
                    opt.grad_scale = grad_scale
                if found_inf is not None:
                    opt.found_inf = found_inf
                opt.step()
        finally:
            for opt in (self.muon_opt, self.adamw_opt, self):
                for attr in ("grad_scale", "found_inf"):
                    if getattr(opt, attr, None) is not None:
                        setattr(opt, attr, None)
        return loss

    def zero_grad(self, set_to_none: bool = True) -> None:
        self.muon_opt.zero_grad(set_to_none=set_to_none)
        self.adamw_opt.zero_grad(set_to_none=set_to_none)

    def check_status(self) -> None:
        self.muon_opt.check_status()
        self.adamw_opt.check_status()

    def state_dict(self) -> Dict[str, Any]:
        return {"muon": self.muon_opt.state_dict(), "adamw": self.adamw_opt.state_dict()}

    def load_state_dict(self, state: Dict[str, Any]) -> None:
        self.muon_opt.load_state_dict(state["muon"])
        self.adamw_opt.load_state_dict(state["adamw"])

    def get_state_memory_mb(self) -> float:
        return self.muon_opt.get_state_memory_mb() + self.adamw_opt.get_state_memory_mb()

    # the sharding wrapper's reporting surface, so that code written against ApexWZeRO keeps working
    @property
    def world_size(self) -> int:
        return self.adamw_opt.world_size

    @property
    def rank(self) -> int:
        return self.adamw_opt.rank

    @property
    def _fused(self) -> bool:
        return bool(self.muon_opt._fused and self.adamw_opt._fused)

    def print_summary(self) -> None:
        n_m = sum(p.numel() for g in self.muon_opt.param_groups for p in g["params"])
        n_a = sum(p.numel() for g in self.adamw_opt.param_groups for p in g["params"])
        print("\n" + "=" * 60)
        print(" DistHybridApexW Summary")
        print("=" * 60)
        print(f" World Size         : {self.world_size} (Rank {self.rank})")
        print(f" Muon parameters    : {n_m:,} (whole-matrix Newton-Schulz on an owner rank)")
        print(f" AdamW parameters   : {n_a:,} (ZeRO-1, {self.adamw_opt.defaults.get('precision', 'compact')} state)")
        print(f" Local State Memory : {self.get_state_memory_mb():.2f} MB")
        print(f" Step path          : {'peer-memory kernels' if self._fused else 'torch.distributed collectives'}")
        print("=" * 60 + "\n")
