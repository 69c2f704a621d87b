"""ApexWZeRO: ZeRO-1 optimizer-state sharding with a fused reduce-scatter + update + all-gather step.

API and checkpoint layout follow the reference wrapper (apexw/zero.py:45-546): the same
constructor, the same dim-0 slicing rule (tensors with ``numel >= world_size*256`` are
split in ``ceil(dim0/world_size)`` rows per rank, smaller tensors are owned round-robin),
``state_dict()`` with ``local_opt`` and ``zero_meta.shard_map``.

What differs is the machinery:

* Parameters and gradients live in flat buffers with the same layout on every rank.  A
  rank's shard of a parameter is a *view* of the full parameter, not a clone, so there is
  no second copy of the shard.
* On CUDA the buffers are symmetric (every rank maps every rank's buffers, ``symm.py``) and
  one kernel per format class does the whole step (``csrc/zero_fused.cu``): it reads the
  shard's gradient from every rank over NVLink and sums it in registers, updates the
  compact / 8-bit state, and writes the new bf16 parameters into every rank's buffer.
  There is no NCCL call on that path and gradients need no prior all-reduce.
* The inner optimizer keeps the sub-byte formats (NF4 momentum, shared-by-four variance),
  so the state is 2.50 / 0.754 bytes per parameter in total, i.e. divided by the world
  size per rank.  (The reference forces ``int4_m=False`` on its inner optimizer and ends up
  at 4.0 / 2.0, apexw/zero.py:135-136.)
* Where the fused path cannot run (CPU tensors, exotic modes, no peer access) the same
  class falls back to ``torch.distributed`` collectives on the flat buffers: one
  all-reduce of the gradients, the local step, one all-reduce of the parameters with
  non-owned ranges zeroed.
"""

from __future__ import annotations

import copy
import functools
import os
import warnings
from typing import Any, Callable, Dict, List, Optional, Tuple, Union

import torch
import torch.distributed as dist
import torch.nn as nn
from torch import Tensor
from torch.optim import Optimizer

from .. import _native
from ..utils import table_check as _table_check
from ..optim import engine_torch as _eng
from ..optim.apexw import ApexW, _KC_DENSE, _KC_INT8, _KC_DENSE_QUAD, _KC_NF4_QUAD, _SEG_DECAY, _SEG_QUAD, \
    _STEP_STOCHASTIC, _STEP_NESTEROV, _STEP_CAUTIOUS, _STEP_MAXIMIZE
from ..optim.rules import is_hybrid_alias, _normalize_precision

from .status import STATUS_TEXT as _STATUS_TEXT, StatusMailbox, ZS_ENTRY_TIMEOUT

_ALIGN = 128          # every parameter starts on a multiple of 128 elements in the flat buffers
_STATUS_WORDS = 64    # one status word per launch entry of a step (entries past the end share the last word)


def _dist_on() -> bool:
    return dist.is_available() and dist.is_initialized()


def _to_global_rank(group, rank: int) -> int:
    if group is None or not hasattr(dist, "get_global_rank"):
        return rank
    try:
        return dist.get_global_rank(group, rank)
    except Exception:
        return rank


def _agree_found_inf(found_inf, live: bool, group):
    """An AMP overflow seen by any rank makes every rank skip the step.  Ranks compute ``found_inf`` from their own
    unreduced gradients, and a rank that skipped alone would leave its peers waiting in the fused kernel."""
    if found_inf is None or not live:
        return found_inf
    flag = found_inf.detach().clone().float().reshape(1) if isinstance(found_inf, Tensor) \
        else torch.tensor([float(found_inf)])
    if dist.get_backend(group) == "nccl" and not flag.is_cuda:
        flag = flag.cuda()
    dist.all_reduce(flag, op=dist.ReduceOp.MAX, group=group)
    return flag[0]


class _FlatStore:
    """Flat parameter and gradient buffers of one dtype (symmetric on CUDA when possible)."""

    def __init__(self, params: List[Tensor], dtype: torch.dtype, device: torch.device, group, want_symmetric: bool,
                 multicast: bool = False):
        self.dtype, self.device = dtype, device
        self.offsets: Dict[int, int] = {}
        off = 0
        for p in params:
            self.offsets[id(p)] = off
            off += (p.numel() + _ALIGN - 1) // _ALIGN * _ALIGN
        self.numel = max(off, _ALIGN)
        item = torch.empty((), dtype=dtype).element_size()
        self.symm_param = self.symm_grad = None
        self.multicast = False
        if want_symmetric and multicast:
            # NVLS: buffers with a multicast address; every rank must succeed or all fall back to plain peer mappings
            from .symm import MulticastBuffer
            mp, mg = MulticastBuffer(self.numel * item, device, group), MulticastBuffer(self.numel * item, device, group)
            ok = mp.supported and mg.supported
            if _dist_on():
                votes: List[Any] = [None] * dist.get_world_size(group)
                dist.all_gather_object(votes, bool(ok), group=group)
                ok = all(votes)
            if ok:
                self.symm_param, self.symm_grad, self.multicast = mp, mg, True
            else:
                warnings.warn("ApexWZeRO: no NVSwitch multicast address for the flat buffers on every rank; "
                              "using plain peer loads and stores", UserWarning, stacklevel=4)
                del mp, mg
        if want_symmetric and self.symm_param is None:
            from .symm import SymmetricBuffer
            self.symm_param = SymmetricBuffer(self.numel * item, device, group)
            self.symm_grad = SymmetricBuffer(self.numel * item, device, group)
        if want_symmetric:
            self.param = self.symm_param.tensor(dtype, self.numel)
            self.grad = self.symm_grad.tensor(dtype, self.numel)
        else:
            self.param = torch.zeros(self.numel, dtype=dtype, device=device)
            self.grad = torch.zeros(self.numel, dtype=dtype, device=device)
        with torch.no_grad():
            for p in params:
                o, n = self.offsets[id(p)], p.numel()
                self.param[o:o + n].copy_(p.detach().reshape(-1))
                p.data = self.param[o:o + n].view(p.shape)
                p.grad = self.grad[o:o + n].view(p.shape)
        self._params = list(params)
        self._item = item

    def clear_grads(self) -> None:
        """``zero_grad`` of the flat gradient buffer.  A weight whose layer accumulates its gradient with a GEMM straight
        into ``main_grad`` and has declared that it can also *overwrite* (``_apexw_can_overwrite``, set by the harness's
        linear layers) is not cleared: it is told to overwrite on its next backward (``_apexw_overwrite``), which saves
        the memset of its gradient and the read of the zeros by the first accumulating GEMM.  Everything else - gradients
        that autograd accumulates - is cleared range by range.  ``finish_grads`` covers weights that then saw no backward."""
        deferred = [p for p in self._params if getattr(p, "_apexw_can_overwrite", False)]
        if not deferred:
            self.grad.zero_()
            return
        for p in self._params:
            if getattr(p, "_apexw_can_overwrite", False):
                p._apexw_overwrite = True
            else:
                o, n = self.offsets[id(p)], p.numel()
                self.grad[o:o + n].zero_()

    def finish_grads(self) -> None:
        """Before a step: a weight that was told to overwrite its gradient but saw no backward since holds the previous
        step's gradient; clear it now."""
        for p in self._params:
            if getattr(p, "_apexw_overwrite", False):
                o, n = self.offsets[id(p)], p.numel()
                self.grad[o:o + n].zero_()
                p._apexw_overwrite = False

    def adopt_grads(self) -> int:
        """Bring gradients that autograd (re)allocated outside the flat buffer back into it.

        ``model.zero_grad(set_to_none=True)`` drops the persistent gradient views; the next backward then
        allocates fresh tensors that the peer kernels would never see.  Returns the number of gradients moved.
        """
        moved = 0
        base = self.grad.data_ptr()
        with torch.no_grad():
            for p in self._params:
                o, n = self.offsets[id(p)], p.numel()
                g = p.grad
                if g is not None and g.data_ptr() == base + o * self._item:
                    continue
                view = self.grad[o:o + n].view(p.shape)
                if g is None:
                    view.zero_()
                else:
                    view.copy_(g)
                    moved += 1
                p.grad = view
                if hasattr(p, "main_grad"):
                    p.main_grad = view
        return moved


class ApexWZeRO(Optimizer):
    r"""ZeRO stage-1 wrapper around :class:`ApexW`.

    Extra keyword arguments beyond the reference's: ``reduce_gradients`` (default: True on
    the fused path, where gradients are summed over ranks inside the kernel and divided by
    the world size; pass False when a DDP wrapper has already averaged them),
    ``fused`` (None = automatic, False = collectives only), ``fused_wgrad`` (expose
    ``p.main_grad`` so the harness's linear layers accumulate weight gradients in place),
    ``nvls`` (None = the ``APEXW_B200_NVLS`` environment switch, default off: the fused step moves gradients and
    parameters with ``multimem`` loads and stores through the NVSwitch instead of one peer at a time; needs bf16
    parameters and a platform with multicast support, else it falls back), ``peer_timeout_ms`` and ``seed``.
    """

    _step_supports_amp_scaling = True

    def __new__(cls, params=None, *args, **kwargs):
        """``ApexWZeRO(..., use_muon=True, fused=True)`` (or a hybrid precision alias with ``fused=True``, or
        ``APEXW_B200_ZERO_HYBRID_FUSED=1``) asks for the hybrid on the peer-memory path: the result is a
        :class:`~apexw_b200.parallel.dist_hybrid.DistHybridApexW` - whole-matrix Newton-Schulz on an owner rank
        (``DistMuon``) for the hidden matrices and the fused ZeRO step for everything else, no collective call on the step.
        Without ``fused=True`` the hybrid keeps the reference's behaviour (Newton-Schulz on each rank's row slices through
        collectives, apexw/zero.py:99-105), including its checkpoint layout."""
        if cls is ApexWZeRO and params is not None and not args:
            hybrid = bool(kwargs.get("use_muon", False)) or is_hybrid_alias(kwargs.get("precision", "compact"))
            asked = kwargs.get("fused") is True or os.environ.get("APEXW_B200_ZERO_HYBRID_FUSED", "0") not in ("", "0")
            if hybrid and asked and kwargs.get("fused") is not False:
                built = cls._fused_hybrid(params, dict(kwargs))
                if built is not None:
                    return built
        return super().__new__(cls)

    @staticmethod
    def _fused_hybrid(params, kw: Dict[str, Any]):
        from .dist_hybrid import DistHybridApexW
        plist = list(params.parameters()) if isinstance(params, nn.Module) else None
        if plist is None:
            params = list(params)
            plist = [p for g in params for p in g["params"]] if params and isinstance(params[0], dict) else params
        ws = kw.pop("world_size", None)
        rank = kw.pop("rank", None)
        live_world = dist.get_world_size(kw.get("process_group")) if _dist_on() else 1
        if not plist or not all(isinstance(p, Tensor) and p.is_cuda for p in plist) or not _native.available() \
                or (ws is not None and ws != live_world) or (rank is not None and _dist_on()
                                                             and rank != dist.get_rank(kw.get("process_group"))):
            return None
        kw.pop("use_muon", None)
        kw.pop("fused", None)
        precision = kw.pop("precision", "compact")
        precision = "compact" if is_hybrid_alias(precision) else precision
        betas = kw.pop("betas", (0.9, 0.95))
        muon = {k: kw.pop(k) for k in ("muon_lr", "muon_momentum", "muon_weight_decay", "ns_steps", "min_muon_dim",
                                       "exclude_embeddings") if k in kw}
        for k in ("overlap_comm", "flatten", "scale_mode", "muon_precision"):       # no meaning on this path
            kw.pop(k, None)
        try:
            return DistHybridApexW(params, lr=kw.pop("lr", 1e-3), weight_decay=kw.pop("weight_decay", 1e-2),
                                   betas=(betas[0], betas[1]), precision=precision, fused=True, **muon, **kw)
        except ValueError:
            return None          # nothing for one of the halves: the plain wrapper handles it

    def __init__(
        self,
        params,
        lr: float = 1e-3,
        betas: Union[Tuple[float, float], Tuple[float, float, float]] = (0.9, 0.999),
        eps: float = 1e-8,
        weight_decay: float = 1e-2,
        world_size: Optional[int] = None,
        rank: Optional[int] = None,
        process_group: Optional[Any] = None,
        amsgrad: bool = False,
        nesterov: bool = False,
        cautious: bool = False,
        grad_centralization: bool = False,
        decay_norm_only: bool = True,
        clip_grad_norm: Optional[float] = None,
        beta3: Optional[float] = None,
        alpha: float = 5.0,
        lion: bool = False,
        precision: str = "compact",
        dynamic_scaling: bool = True,
        overlap_comm: bool = True,
        reduce_gradients: Optional[bool] = None,
        fused: Optional[bool] = None,
        fused_wgrad: bool = False,
        flatten: bool = True,
        peer_timeout_ms: Optional[float] = None,
        overlap_backward: bool = False,
        overlap_buckets: int = 8,
        overlap_ctas: int = 48,
        nvls: Optional[bool] = None,
        **apex_kwargs,
    ):
        if _dist_on():
            self.world_size = dist.get_world_size(process_group) if world_size is None else world_size
            self.rank = dist.get_rank(process_group) if rank is None else rank
        else:
            self.world_size = world_size if world_size is not None else 1
            self.rank = rank if rank is not None else 0
        self.process_group = process_group
        self.overlap_comm = overlap_comm
        self._live_dist = _dist_on() and dist.get_world_size(process_group) == self.world_size and self.world_size > 1

        if isinstance(params, nn.Module):
            for name, p in params.named_parameters():
                if not hasattr(p, "_param_name"):
                    p._param_name = name
            ps = [p for p in params.parameters() if p.requires_grad]
            params = ps if ps else list(params.parameters())

        hybrid = bool(apex_kwargs.get("use_muon", False)) or is_hybrid_alias(precision)
        if hybrid:
            apex_kwargs["use_muon"] = True
            precision = "compact"
        if len(betas) > 2 and beta3 is None:
            # (beta1, beta2, beta3) means AdEMAMix here as it does for ApexW; the reference's wrapper keeps the first
            # two and silently drops the third (apexw/zero.py:109, :118)
            beta3 = betas[2]

        defaults = dict(lr=lr, betas=(betas[0], betas[1]), eps=eps, weight_decay=weight_decay, amsgrad=amsgrad,
                        nesterov=nesterov, cautious=cautious, grad_centralization=grad_centralization,
                        decay_norm_only=decay_norm_only, clip_grad_norm=clip_grad_norm, beta3=beta3, alpha=alpha,
                        lion=lion, precision=precision, dynamic_scaling=dynamic_scaling, **apex_kwargs)
        super().__init__(params, defaults)

        self._stores: List[_FlatStore] = []
        self._param_store: Dict[int, _FlatStore] = {}
        self._sharded_param_map: List[Dict[str, Any]] = []
        self._local_params: List[Tensor] = []
        self._local_param_groups: List[Dict[str, Any]] = []
        self._p_index = 0
        self._epoch = 0
        self._zero_plans: Optional[List[Dict[str, Any]]] = None
        self._mailbox: Optional[StatusMailbox] = None
        self._signal = None
        self.fused_wgrad = bool(fused_wgrad)
        # overlap of the fused step with the last micro-batch's backward (opt-in, fused path only)
        self.overlap_backward = bool(overlap_backward)
        self.overlap_buckets = max(1, int(overlap_buckets))
        self.overlap_ctas = max(1, int(overlap_ctas))
        self._bucket_of: Dict[int, int] = {}
        self._armed = False
        self._pending: Dict[int, int] = {}
        self._launched: List[int] = []
        self._fired: Dict[int, str] = {}
        self._ready: set = set()
        self._next_bucket = -1
        self._step_entries: List[Dict[str, Any]] = []
        self._side_stream = None
        self.peer_timeout_ms = float(peer_timeout_ms if peer_timeout_ms is not None
                                     else os.environ.get("APEXW_B200_PEER_TIMEOUT_MS", 5000.0))
        # NVLS transport of the fused step (multimem loads / stores through the switch); off unless asked for
        self.nvls = bool(nvls) if nvls is not None else os.environ.get("APEXW_B200_NVLS", "0") not in ("", "0")

        all_params = [p for g in self.param_groups for p in g["params"]]
        on_cuda = bool(all_params) and all(p.is_cuda for p in all_params)
        self._flatten = bool(flatten) and bool(all_params) and len({p.device for p in all_params}) == 1
        want_fused = (fused is not False) and on_cuda and self._flatten and not hybrid and _native.available() \
            and (self.world_size == 1 or self._live_dist) and self.world_size <= 8
        if fused is True and not want_fused:
            raise RuntimeError("ApexWZeRO(fused=True) needs CUDA parameters on one device, the native library and "
                               "an initialised process group of at most 8 ranks")
        self._fused = want_fused
        if self._flatten:
            self._build_stores(all_params, symmetric=want_fused)

        for gi, group in enumerate(self.param_groups):
            self._local_param_groups.append(self._shard_group(gi, group))

        local_kwargs = dict(apex_kwargs)
        from ..optim.backward_hooks import suppress_auto_runtime
        with suppress_auto_runtime():
            self._local_opt = self._make_inner(lr, betas, eps, weight_decay, amsgrad, nesterov, cautious, grad_centralization,
                                               decay_norm_only, clip_grad_norm, beta3, alpha, lion, precision, dynamic_scaling,
                                               local_kwargs)
        self._mark_managed(self._local_opt)
        self.reduce_gradients = bool(reduce_gradients) if reduce_gradients is not None else True
        if self._fused:
            self._fused = self._agree_on_fused()
        self.overlap_backward = self.overlap_backward and self._fused
        self._assign_buckets(all_params)
        if self.overlap_backward:
            self._install_ready_hooks(all_params)
        self._sync_hyperparameters()      # also records the base learning rates that schedules are measured against

    def _make_inner(self, lr, betas, eps, weight_decay, amsgrad, nesterov, cautious, grad_centralization, decay_norm_only,
                    clip_grad_norm, beta3, alpha, lion, precision, dynamic_scaling, local_kwargs):
        return ApexW(self._local_param_groups, lr=lr, betas=betas, eps=eps, weight_decay=weight_decay,
                                amsgrad=amsgrad, nesterov=nesterov, cautious=cautious,
                                grad_centralization=grad_centralization, decay_norm_only=decay_norm_only,
                                clip_grad_norm=clip_grad_norm, beta3=beta3, alpha=alpha, lion=lion,
                                precision=precision, dynamic_scaling=dynamic_scaling, **local_kwargs)

    # ------------------------------------------------------------------ construction helpers

    @staticmethod
    def _mark_managed(opt) -> None:
        for o in (opt, getattr(opt, "muon_opt", None), getattr(opt, "adamw_opt", None)):
            if o is not None:
                o._managed_externally = True
                if hasattr(o, "_disable_auto_8bit_hooks"):
                    o._disable_auto_8bit_hooks()

    def _build_stores(self, params: List[Tensor], symmetric: bool) -> None:
        by_dtype: Dict[torch.dtype, List[Tensor]] = {}
        for p in params:
            by_dtype.setdefault(p.dtype, []).append(p)
        for dt, ps in by_dtype.items():
            store = _FlatStore(ps, dt, ps[0].device, self.process_group, symmetric,
                               multicast=symmetric and self.nvls and self._live_dist and dt == torch.bfloat16)
            self._stores.append(store)
            for p in ps:
                self._param_store[id(p)] = store
            if self.fused_wgrad:
                for p in ps:
                    p.main_grad = p.grad
        if symmetric:
            from .symm import SymmetricBuffer
            dev = params[0].device
            self._signal = SymmetricBuffer(256, dev, self.process_group)
            self._mailbox = StatusMailbox(dev, _STATUS_WORDS)

    def _store_of(self, p: Tensor) -> Optional[_FlatStore]:
        return self._param_store.get(id(p))

    def _shard_group(self, group_idx: int, group: Dict[str, Any]) -> Dict[str, Any]:
        local = {k: v for k, v in group.items() if k not in ("params", "use_muon")}
        local["params"] = []
        W, R = self.world_size, self.rank
        for p in group["params"]:
            entry: Dict[str, Any] = {"full_param": p, "group_idx": group_idx}
            if p.dim() >= 1 and p.numel() >= W * 256:
                dim0 = p.shape[0]
                chunk = (dim0 + W - 1) // W
                start, end = min(R * chunk, dim0), min((R + 1) * chunk, dim0)
                loc = nn.Parameter(p.data[start:end], requires_grad=True)   # a view: no second copy
                if hasattr(p, "_param_name"):
                    loc._param_name = p._param_name
                entry.update(type="slice", local_slice=loc, start=start, end=end, dim0=dim0, chunk_size=chunk)
                local["params"].append(loc)
                self._local_params.append(loc)
            else:
                owner = self._p_index % W
                loc = None
                if owner == R:
                    loc = nn.Parameter(p.data, requires_grad=True)
                    if hasattr(p, "_param_name"):
                        loc._param_name = p._param_name
                    local["params"].append(loc)
                    self._local_params.append(loc)
                entry.update(type="round_robin", local_slice=loc, owner_rank=owner)
            self._sharded_param_map.append(entry)
            self._p_index += 1
        return local

    def _fused_supported_locally(self) -> bool:
        """Every local shard must be in a mode the fused kernels implement."""
        inner = self._local_opt
        if not isinstance(inner, ApexW):
            return False
        ctx = inner._group_ctx()
        for g in inner.param_groups:
            g["precision"] = _normalize_precision(g.get("precision", "compact"))
            if g["capturable"] or g.get("grad_centralization"):
                return False
            if g["lion"] or g["amsgrad"] or g["beta3"] is not None:
                return False      # extra moments / sign updates: the single-GPU kernel and the NCCL path have them
            if g.get("clip_grad_norm") is not None and any(p.dtype != torch.bfloat16 for p in g["params"]):
                return False      # clipping inside the fused step reduces bf16 gradients in place (two-phase kernels)
            for p in g["params"]:
                if p.numel() == 0:
                    continue
                if not p.is_contiguous():
                    return False
                if inner._flat_decay_ranges(p, g):      # decay of parts of a flat parameter: single-GPU kernel only
                    return False
                if p.dtype not in (torch.float32, torch.bfloat16):     # the peer kernel moves fp32 and bf16 only
                    return False
                st = inner._init_state(p, g, ctx)
                had = p.grad
                p.grad = p.data       # eligibility only looks at dtype/contiguity of the gradient
                try:
                    kc = inner._native_eligible(p, st, g)
                finally:
                    p.grad = had
                if kc is None:
                    return False
                if g["cautious"] and kc in (_KC_DENSE, _KC_DENSE_QUAD):
                    return False      # the whole-tensor kept fraction would span ranks
                if kc > _KC_NF4_QUAD:
                    return False      # layouts that only the single-GPU kernel knows (int8 momentum + dense variance)
        return True

    def _agree_on_fused(self) -> bool:
        ok = self._fused_supported_locally()
        if self._live_dist:
            votes: List[Any] = [None] * self.world_size
            dist.all_gather_object(votes, bool(ok), group=self.process_group)
            ok = all(votes)
        if not ok:
            warnings.warn("ApexWZeRO: a shard uses a mode the fused kernels do not implement; "
                          "falling back to torch.distributed collectives for every rank.", UserWarning, stacklevel=3)
        return ok

    # ------------------------------------------------------------------ Optimizer API

    def zero_grad(self, set_to_none: bool = True):
        self._poll_status()
        if self._stores:
            # gradients are persistent views of the flat buffers: clear them in place
            for store in self._stores:
                store.clear_grads()
            return
        super().zero_grad(set_to_none=set_to_none)
        for item in self._sharded_param_map:
            loc = item["local_slice"]
            if loc is not None:
                if set_to_none:
                    loc.grad = None
                elif loc.grad is not None:
                    loc.grad.zero_()

    def _sync_hyperparameters(self) -> None:
        inner_groups = self._local_opt.param_groups
        if len(self.param_groups) == len(inner_groups):
            for og, ig in zip(self.param_groups, inner_groups):
                for k, v in og.items():
                    if k not in ("params", "use_muon"):
                        ig[k] = v
        else:   # hybrid inner optimizer: groups were re-partitioned; scale learning rates by ratio
            # The base rates are remembered from the first synchronisation (or taken from a scheduler's ``initial_lr``),
            # so that a schedule on the outer group moves the Muon and AdamW rates by the same factor.  (The reference
            # reads a key ``_initial_lr`` that nothing sets, so its ratio is always 1: apexw/zero.py:266-269.)
            base = self.__dict__.setdefault("_base_lrs", {})
            for gi, og in enumerate(self.param_groups):
                for ii, ig in enumerate(inner_groups):
                    for k, v in og.items():
                        if k not in ("params", "lr", "use_muon") and k in ig:
                            ig[k] = v
                    if "lr" in og and "lr" in ig:
                        outer0 = og.get("initial_lr", og.get("_initial_lr", base.setdefault(("outer", gi), og["lr"])))
                        inner0 = ig.get("_initial_lr", base.setdefault(("inner", ii), ig["lr"]))
                        ig["lr"] = inner0 * (og["lr"] / max(outer0, 1e-12))

    def _full_grad(self, p: Tensor) -> Optional[Tensor]:
        return p.grad

    @torch.no_grad()
    def step(self, closure: Optional[Callable] = None):
        loss = None
        if closure is not None:
            with torch.enable_grad():
                loss = closure()
        grad_scale = getattr(self, "grad_scale", None)
        found_inf = getattr(self, "found_inf", None)
        try:
            self._poll_status()       # a wait that ran out in an earlier step surfaces here, without a host sync
            found_inf = _agree_found_inf(found_inf, self._live_dist, self.process_group)
            if found_inf is not None and bool(found_inf):
                return loss
            self._sync_hyperparameters()
            if self._fused:
                self._step_fused(grad_scale)
                if _table_check.enabled():
                    _table_check.check()        # debug mode: one device synchronisation per step
            else:
                self._step_collectives(grad_scale, found_inf)
        finally:
            for o in (self._local_opt, self):
                if hasattr(o, "grad_scale"):
                    o.grad_scale = None
                if hasattr(o, "found_inf"):
                    o.found_inf = None
        return loss

    # ------------------------------------------------------------------ overlap with backward

    def _assign_buckets(self, params: List[Tensor]) -> None:
        """Contiguous runs of parameters (registration order) of roughly equal size; one bucket when overlap is off."""
        n_b = self.overlap_buckets if self.overlap_backward else 1
        total = sum(p.numel() for p in params) or 1
        seen = 0
        for p in params:
            self._bucket_of[id(p)] = min(n_b - 1, seen * n_b // total)
            seen += p.numel()

    def _install_ready_hooks(self, params: List[Tensor]) -> None:
        """A parameter reports that its gradient of the current backward is final either through autograd's
        post-accumulate hook or, for weights whose gradient GEMM accumulates into ``main_grad`` (autograd never
        sees that gradient), through the ``_apexw_grad_ready`` callback that the harness's linear layers call."""
        for p in params:
            p._apexw_grad_ready = functools.partial(self._on_grad_ready, p, "callback")
            if hasattr(p, "register_post_accumulate_grad_hook"):
                p.register_post_accumulate_grad_hook(functools.partial(self._on_grad_ready, source="autograd hook"))

    def arm_overlap(self) -> None:
        """Call before the LAST micro-batch of a step (``TrainEngine`` does): from now until ``step()`` a bucket of
        parameters is stepped on a side stream as soon as all of its gradients are final, beside the rest of the
        backward pass.  Every rank must arm the same steps.  AMP loss scaling is not combined with this mode."""
        if not self.overlap_backward:
            return
        if any(g.get("clip_grad_norm") is not None for g in self.param_groups):
            return        # the clip coefficient needs every gradient of the group: nothing can step before backward ends
        self._sync_hyperparameters()
        self._prepare_fused()
        self._pending = {}
        for g in self.param_groups:
            for p in g["params"]:
                if p.requires_grad:
                    b = self._bucket_of[id(p)]
                    self._pending[b] = self._pending.get(b, 0) + 1
        self._launched, self._fired = [], {}
        self._step_entries = []
        self._next_bucket = max(self._bucket_of.values(), default=-1)
        self._ready = {b for b in range(self._next_bucket + 1) if b not in self._pending}   # nothing to wait for
        self._armed = True

    def _on_grad_ready(self, p: Tensor, source: str = "callback") -> None:
        if not self._armed:
            return
        b = self._bucket_of.get(id(p))
        if b is None:
            return
        if id(p) in self._fired:
            # the explicit callback and autograd's hook may both report the same gradient (recent torch versions
            # run the hook even when a backward function returns no gradient for the weight); the same source
            # reporting twice means the parameter is used twice in the graph
            if self._fired[id(p)] == source and b in self._launched:
                raise RuntimeError(f"a parameter of shape {tuple(p.shape)} received a second gradient contribution "
                                   f"through the {source} after its bucket was stepped; parameters used more than once "
                                   f"per backward need overlap_backward=False")
            return
        self._fired[id(p)] = source
        self._pending[b] -= 1
        if self._pending[b] == 0:
            self._ready.add(b)
            self._launch_ready_buckets()

    def _launch_ready_buckets(self) -> None:
        """Buckets go out in one fixed order on every rank - from the last bucket (whose gradients a backward pass
        finishes first) down to bucket 0 - because ranks pair their launches by a running epoch counter: a bucket that
        is ready waits until every higher-numbered bucket has been launched.  Gradients that arrive in another order on
        some rank (unused parameters, data-dependent graphs) then cost overlap, never correctness."""
        while self._next_bucket >= 0 and self._next_bucket in self._ready:
            self._launch_bucket(self._next_bucket, capped=True)
            self._next_bucket -= 1

    def _launch_bucket(self, b: int, capped: bool) -> None:
        dev = self._stores[0].device
        if self._side_stream is None:
            self._side_stream = torch.cuda.Stream(device=dev)
        side = self._side_stream
        side.wait_stream(torch.cuda.current_stream(dev))       # the gradients of this bucket are final on the main stream
        with torch.cuda.stream(side):
            self._launch_entries([e for e in self._zero_plans if e["bucket"] == b], None,
                                 self.overlap_ctas if capped else 0)
        self._launched.append(b)

    def _finish_overlapped_step(self) -> None:
        """``step()`` of an armed pass: buckets that are still held back (their gradients, or those of a higher bucket,
        never reported: unused parameters) go now, in the same descending order, and the main stream waits for all."""
        dev = self._stores[0].device
        while self._next_bucket >= 0:
            self._launch_bucket(self._next_bucket, capped=False)
            self._next_bucket -= 1
        if self._side_stream is not None:
            torch.cuda.current_stream(dev).wait_stream(self._side_stream)
        self._armed = False
        self._post_status()
        self._empty_step = getattr(self, "_empty_step", 0) + 1
        self._local_opt._has_stepped = True

    # ------------------------------------------------------------------ fused path

    def _build_zero_plans(self) -> List[Dict[str, Any]]:
        """One plan per (inner group, kernel class) present on ANY rank, in an order all ranks share."""
        nat = _native.require()
        inner = self._local_opt
        ctx = inner._group_ctx()
        bucket_of_local = {id(item["local_slice"]): self._bucket_of.get(id(item["full_param"]), 0)
                           for item in self._sharded_param_map if item["local_slice"] is not None}
        mine: Dict[Tuple[int, int, int, str], List[Tensor]] = {}
        for gi, g in enumerate(inner.param_groups):
            for p in g["params"]:
                if p.numel() == 0:
                    continue
                st = inner._init_state(p, g, ctx)
                p.grad = p.data
                try:
                    kc = inner._native_eligible(p, st, g)
                finally:
                    p.grad = None
                mine.setdefault((bucket_of_local.get(id(p), 0), gi, kc, str(p.dtype)), []).append(p)
        keys = set(mine)
        if self._live_dist:
            gathered: List[Any] = [None] * self.world_size
            dist.all_gather_object(gathered, sorted(keys), group=self.process_group)
            keys = set(k for ks in gathered for k in map(tuple, ks))
        offset_of = {}
        for item in self._sharded_param_map:
            loc, full = item["local_slice"], item["full_param"]
            if loc is None:
                continue
            store = self._store_of(full)
            base = store.offsets[id(full)]
            if item["type"] == "slice":
                base += item["start"] * (full.numel() // max(full.shape[0], 1))
            offset_of[id(loc)] = (base, store)
        plans = []
        dev = self._stores[0].device
        for (bk, gi, kc, dt) in sorted(keys):
            ps = mine.get((bk, gi, kc, dt), [])
            g = inner.param_groups[gi]
            quant = kc >= _KC_INT8
            flags = []
            for p in ps:
                f = 0
                if g["weight_decay"] != 0 and (not g["decay_norm_only"] or p.dim() >= 2):
                    f |= _SEG_DECAY
                if kc in (_KC_DENSE_QUAD, _KC_NF4_QUAD):
                    f |= _SEG_QUAD
                flags.append(f)
            store = next(s for s in self._stores if str(s.dtype) == dt)
            if os.environ.get("APEXW_B200_DEBUG", "0") not in ("", "0"):
                from ..optim.apexw import assert_disjoint_write_sets
                assert_disjoint_write_sets([p.data for p in ps] + [inner.state[p][k] for p in ps
                                                                   for k in ("exp_avg", "exp_avg_sq")])
            plan = nat.StatePlan(
                kc, [p.data for p in ps], [inner.state[p]["exp_avg"] for p in ps],
                [inner.state[p]["exp_avg_sq"] for p in ps],
                [inner.state[p]["exp_avg_scales"].view(-1) for p in ps] if quant else [],
                [inner.state[p]["exp_avg_sq_scales"].view(-1) for p in ps] if quant else [],
                flags, [inner._salt_of(p) for p in ps],
                [int(inner.state[p].get("block_size_8bit", 0)) for p in ps],
                [offset_of[id(p)][0] for p in ps], dev.index if dev.index is not None else torch.cuda.current_device())
            plans.append({"plan": plan, "group": gi, "params": ps, "store": store, "bucket": bk})
        return plans

    def _prepare_fused(self) -> None:
        if self._zero_plans is None:
            self._zero_plans = self._build_zero_plans()
            if self._live_dist:
                dist.barrier(group=self.process_group)   # align ranks once before the first in-kernel wait
        for store in self._stores:
            store.adopt_grads()
            store.finish_grads()

    def _step_fused(self, grad_scale: Optional[Tensor]) -> None:
        if self._armed:
            if grad_scale is not None:
                raise RuntimeError("overlap_backward does not combine with AMP loss scaling (grad_scale is set)")
            self._finish_overlapped_step()
            return
        self._prepare_fused()
        self._step_entries = []
        self._launch_entries(self._zero_plans, grad_scale, 0)
        self._post_status()
        self._empty_step = getattr(self, "_empty_step", 0) + 1
        self._local_opt._has_stepped = True

    def _launch_entries(self, entries: List[Dict[str, Any]], grad_scale: Optional[Tensor], cta_cap: int) -> None:
        inner = self._local_opt
        clip_totals = self._reduce_for_clipping(entries, grad_scale)
        for entry in entries:
            g = inner.param_groups[entry["group"]]
            ps = entry["params"]
            store: _FlatStore = entry["store"]
            if ps:
                from ..optim.apexw import _bump_steps
                _bump_steps([inner.state[p]["step"] for p in ps])
                step = float(inner.state[ps[0]]["step"])
            else:
                step = float(getattr(self, "_empty_step", 0)) + 1.0
            sc = _eng.make_scalars(g, max(step, 1.0), inner.seed)
            flags = 0
            if g.get("stochastic_rounding", True):
                flags |= _STEP_STOCHASTIC
            if g["nesterov"]:
                flags |= _STEP_NESTEROV
            if g["cautious"]:
                flags |= _STEP_CAUTIOUS
            if g["maximize"]:
                flags |= _STEP_MAXIMIZE
            self._epoch += 1
            code = 1 if store.dtype == torch.bfloat16 else 0
            grads, params, signals = self._peer_pointers(store)
            clip_total = clip_totals.get(entry["group"])
            if clip_total is not None:
                # phase 2 of a clipped step: the shard's gradient was reduced, scaled and written back in phase 1
                grads, inv = [store.symm_grad.local_ptr], 1.0
            else:
                inv = 1.0 / len(grads)
                if grad_scale is not None:
                    inv = inv / float(grad_scale)
            mc_g, mc_p = (store.symm_grad.multicast_ptr, store.symm_param.multicast_ptr) \
                if (store.multicast and len(grads) > 1) else (0, 0)
            entry["plan"].set_cta_cap(int(cta_cap))
            word = self._status_word_of(entry)
            with _native.nvtx_range("apexw_b200.zero_fused"):
                entry["plan"].step_zero(grads, params, signals, self.rank,
                                        self._epoch, self.peer_timeout_ms, self._mailbox.word(word), code, code,
                                        sc.beta1, sc.beta2, sc.step_size, sc.eps_scaled, sc.eps, sc.eps_quad,
                                        sc.eps_quad_scaled, sc.decay_factor, inv,
                                        1.0 + _eng.GAIN_ALIGNED * sc.beta1, 1.0 - _eng.GAIN_OPPOSED * sc.beta1,
                                        sc.key, flags, mc_g, mc_p, clip_total,
                                        float(g["clip_grad_norm"]) if clip_total is not None else 0.0)
            _native.count(1)

    def _status_word_of(self, entry: Dict[str, Any]) -> int:
        """Index of the status word of ``entry`` in this step (assigned at its first launch of the step)."""
        for i, e in enumerate(self._step_entries):
            if e is entry:
                return i
        self._step_entries.append(entry)
        return len(self._step_entries) - 1

    def _reduce_for_clipping(self, entries: List[Dict[str, Any]], grad_scale: Optional[Tensor]) -> Dict[int, Tensor]:
        """Phase 1 of a clipped fused step, for every parameter group with ``clip_grad_norm``: each launch plan's shard is
        reduce-scattered in place (peer loads, the sum scaled and written back over this rank's own copy) while its
        squares are summed; then the ranks swap their partial sums through the signal pads.  Returns, per group index,
        the device scalar that holds the squared norm of the group's WHOLE reduced gradient - the norm an unsharded run
        would clip by.  Still no collective-library call on the step."""
        inner = self._local_opt
        groups = sorted({e["group"] for e in entries if inner.param_groups[e["group"]].get("clip_grad_norm") is not None})
        if not groups:
            return {}
        nat = _native.require()
        dev = self._stores[0].device
        if getattr(self, "_clip_scratch", None) is None:
            sms = torch.cuda.get_device_properties(dev).multi_processor_count
            self._clip_scratch = torch.zeros(4 * sms, dtype=torch.float32, device=dev)
            self._clip_acc: Dict[int, Tensor] = {}
            self._clip_total: Dict[int, Tensor] = {}
        totals: Dict[int, Tensor] = {}
        for gi in groups:
            acc = self._clip_acc.setdefault(gi, torch.zeros(1, dtype=torch.float32, device=dev))
            total = self._clip_total.setdefault(gi, torch.zeros(1, dtype=torch.float32, device=dev))
            mine = [e for e in entries if e["group"] == gi]
            for entry in mine:
                store: _FlatStore = entry["store"]
                grads, _params, signals = self._peer_pointers(store)
                if len(grads) == 1:                      # gradients arrive already reduced: only scale and measure them
                    signals = [self._signal.local_ptr]
                inv = 1.0 / len(grads)
                if grad_scale is not None:
                    inv = inv / float(grad_scale)
                self._epoch += 1
                word = self._status_word_of(entry)
                with _native.nvtx_range("apexw_b200.zero_reduce"):
                    entry["plan"].reduce_zero(grads, signals, self.rank if len(grads) > 1 else 0, self._epoch,
                                              self.peer_timeout_ms, self._mailbox.word(word), inv, self._clip_scratch, acc)
                _native.count(1)
            self._epoch += 1
            nat.zero_norm_exchange(self._signal.peer_ptrs, self.rank, self._epoch, self.peer_timeout_ms,
                                   self._mailbox.word(self._status_word_of(mine[0])), acc, total)
            _native.count(1)
            totals[gi] = total
        return totals

    def _peer_pointers(self, store: "_FlatStore") -> Tuple[List[int], List[int], List[int]]:
        """Addresses, as mapped on this rank, of every rank's gradient buffer (only this rank's when gradients
        arrive already reduced), parameter buffer and signal pad."""
        grads = store.symm_grad.peer_ptrs if self.reduce_gradients else [store.symm_grad.local_ptr]
        return grads, store.symm_param.peer_ptrs, self._signal.peer_ptrs

    def _post_status(self) -> None:
        """After a step's launches: queue the asynchronous read-back of their status words."""
        if self._mailbox is None:
            return
        inner = self._local_opt
        entries = list(getattr(self, "_step_entries", []))

        def take_back(codes: Dict[int, int]) -> None:
            # a launch whose entry wait ran out updated nothing: its parameters have not taken that step
            from ..optim.apexw import _unbump_steps
            last = _STATUS_WORDS - 1
            for i, entry in enumerate(entries):
                if codes.get(min(i, last)) == ZS_ENTRY_TIMEOUT and entry["params"]:
                    _unbump_steps([inner.state[p]["step"] for p in entry["params"]])

        self._mailbox.post(take_back)

    def _poll_status(self, wait: bool = False) -> None:
        if self._mailbox is not None:
            self._mailbox.poll("ApexWZeRO fused step", self.rank, wait=wait)

    def check_status(self) -> None:
        """Wait for the status words of every step issued so far (one host sync) and raise on a timeout.  Not needed
        in a training loop: ``step()`` and ``zero_grad()`` report a failed earlier step by themselves, without a sync."""
        self._poll_status(wait=True)

    # ------------------------------------------------------------------ collectives path

    def _owned_ranges(self, store: _FlatStore) -> List[Tuple[int, int]]:
        out = []
        for item in self._sharded_param_map:
            full, loc = item["full_param"], item["local_slice"]
            if loc is None or self._store_of(full) is not store:
                continue
            base = store.offsets[id(full)]
            if item["type"] == "slice":
                cols = full.numel() // max(full.shape[0], 1)
                out.append((base + item["start"] * cols, base + item["end"] * cols))
            else:
                out.append((base, base + full.numel()))
        return out

    def _step_collectives(self, grad_scale, found_inf) -> None:
        inner = self._local_opt
        live = self._live_dist
        if self.world_size > 1 and not live and not getattr(self, "_warned_unsynced", False):
            warnings.warn(f"ApexWZeRO: world_size={self.world_size} specified, but torch.distributed is not "
                          f"initialized. Shards on other ranks will not be synchronized across processes.",
                          UserWarning, stacklevel=3)
            self._warned_unsynced = True
        for store in self._stores:
            store.finish_grads()
        if live and self.reduce_gradients:
            if self._stores:
                for store in self._stores:
                    dist.all_reduce(store.grad, op=dist.ReduceOp.SUM, group=self.process_group)
                    store.grad.div_(self.world_size)
            else:
                for item in self._sharded_param_map:
                    g = item["full_param"].grad
                    if g is not None:
                        dist.all_reduce(g, op=dist.ReduceOp.SUM, group=self.process_group)
                        g.div_(self.world_size)
        for item in self._sharded_param_map:
            full, loc = item["full_param"], item["local_slice"]
            if loc is None:
                continue
            g = full.grad
            if g is None:
                loc.grad = None
            elif item["type"] == "slice":
                loc.grad = g.data[item["start"]:item["end"]] if item["end"] > item["start"] else None
            else:
                loc.grad = g.data
        grad_scale, restore = self._clip_by_the_whole_norm(grad_scale)
        if grad_scale is not None:
            inner.grad_scale = grad_scale
        if found_inf is not None:
            inner.found_inf = found_inf
        try:
            inner.step()
        finally:
            for ig, clip, cent in restore:
                ig["clip_grad_norm"], ig["grad_centralization"] = clip, cent
        for loc in self._local_params:
            loc.grad = None
        if not live:
            return
        if self._stores:
            for store in self._stores:
                keep = sorted(self._owned_ranges(store))
                pos = 0
                for a, b in keep:
                    if a > pos:
                        store.param[pos:a].zero_()
                    pos = max(pos, b)
                if pos < store.numel:
                    store.param[pos:].zero_()
                dist.all_reduce(store.param, op=dist.ReduceOp.SUM, group=self.process_group)
            return
        handles = []
        for item in self._sharded_param_map:
            full = item["full_param"]
            if item["type"] == "slice":
                s, e = item["start"], item["end"]
                if s > 0:
                    full.data[:s].zero_()
                if e < item["dim0"]:
                    full.data[e:].zero_()
                handles.append(dist.all_reduce(full.data, op=dist.ReduceOp.SUM, group=self.process_group,
                                               async_op=self.overlap_comm))
            else:
                src = _to_global_rank(self.process_group, item["owner_rank"])
                handles.append(dist.broadcast(full.data, src=src, group=self.process_group, async_op=self.overlap_comm))
        for h in handles:
            if h is not None and hasattr(h, "wait"):
                h.wait()

    def _clip_by_the_whole_norm(self, grad_scale):
        """Gradient clipping under sharding: the norm is that of the whole (already reduced) gradients of a group, not
        of this rank's slices, so a sharded run clips exactly like the unsharded optimizer.  (The reference hands
        ``clip_grad_norm`` to the inner optimizer, which then sees the slices only: apexw/zero.py:117, :148.)

        Unscaling, centralisation and clipping are done here on the full gradients, in place, and switched off in the
        inner groups for this step.  Returns the loss scale still to be applied and what to restore afterwards."""
        inner = self._local_opt
        if not isinstance(inner, ApexW) or len(inner.param_groups) != len(self.param_groups) \
                or all(g.get("clip_grad_norm") is None for g in self.param_groups):
            return grad_scale, []
        scale = None
        if grad_scale is not None:
            scale = grad_scale if torch.is_tensor(grad_scale) else torch.tensor(float(grad_scale), dtype=torch.float32)
        restore = []
        for og, ig in zip(self.param_groups, inner.param_groups):
            grads = [p.grad for p in og["params"] if p.grad is not None]
            if grads:
                _, left = ApexW._prepare_grads(grads, og, scale)
                if left is not None:          # a group without clipping or centralisation: only the loss scale
                    torch._foreach_mul_(grads, left.to(grads[0].device).reciprocal())
            restore.append((ig, ig.get("clip_grad_norm"), ig.get("grad_centralization", False)))
            ig["clip_grad_norm"], ig["grad_centralization"] = None, False
        return None, restore

    # ------------------------------------------------------------------ reports

    def get_state_memory_mb(self) -> float:
        return self._local_opt.get_state_memory_mb()

    def _adam_equiv_mb(self) -> float:
        return sum(p.numel() * 8 for g in self.param_groups for p in g["params"]) / (1024 * 1024)

    def get_rank_saved_mb(self) -> float:
        return max(0.0, self._adam_equiv_mb() - self.get_state_memory_mb())

    def get_total_cluster_saved_mb(self) -> float:
        w = max(1, self.world_size)
        return max(0.0, w * self._adam_equiv_mb() - w * self.get_state_memory_mb())

    def print_summary(self) -> None:
        total = sum(p.numel() for g in self.param_groups for p in g["params"])
        adam = self._adam_equiv_mb()
        saved = self.get_rank_saved_mb()
        print("\n" + "=" * 60)
        print(" ApexWZeRO Optimizer Summary")
        print("=" * 60)
        print(f" World Size         : {self.world_size} (Rank {self.rank})")
        print(f" Total Parameters   : {total:,}")
        print(f" Local State Memory : {self.get_state_memory_mb():.2f} MB")
        print(f" AdamW Equivalent   : {adam:.2f} MB")
        print(f" Memory Saved / Rank: {saved:.2f} MB ({saved / max(1e-6, adam) * 100.0:.1f}% reduction)")
        print(f" Cluster Memory Save: {self.get_total_cluster_saved_mb():.2f} MB across {self.world_size} ranks")
        path = 'torch.distributed collectives'
        if self._fused:
            path = 'fused peer-memory kernel' + (' (NVLS multimem)' if any(st.multicast for st in self._stores) else '')
        print(f" Step path          : {path}")
        print("=" * 60 + "\n")

    # ------------------------------------------------------------------ checkpoint

    def state_dict(self):
        local_sd = self._local_opt.state_dict()
        is_hybrid = hasattr(self._local_opt, "muon_opt")
        locals_flat = [p for g in self._local_opt.param_groups for p in g["params"]]
        state_id = {id(p): i for i, p in enumerate(locals_flat)}
        group_of = {id(p): gi for gi, g in enumerate(self._local_opt.param_groups) for p in g["params"]}
        shard_meta = []
        for e in self._sharded_param_map:
            entry = {"type": e["type"], "group_idx": e.get("group_idx", 0)}
            loc = e.get("local_slice")
            if loc is not None and id(loc) in state_id:
                entry["local_state_id"] = state_id[id(loc)]
                entry["local_group_idx"] = group_of[id(loc)]
            elif is_hybrid:
                from ..optim.hybrid import _is_muon_eligible
                n_m = len(self._local_opt.muon_opt.param_groups) if getattr(self._local_opt, "muon_opt", None) else 1
                entry["local_group_idx"] = 0 if _is_muon_eligible(e["full_param"], exclude_embeddings=True, min_muon_dim=32) else n_m
                entry["local_state_id"] = None
            else:
                entry["local_group_idx"] = e.get("group_idx", 0)
                entry["local_state_id"] = None
            if e["type"] == "slice":
                entry.update(start=e["start"], end=e["end"], dim0=e["dim0"])
            else:
                entry["owner_rank"] = e.get("owner_rank")
            shard_meta.append(entry)
        return {
            "state": local_sd.get("state", {}),
            "param_groups": copy.deepcopy(local_sd.get("param_groups", [])),
            "local_opt": local_sd,
            "zero_meta": {"rank": self.rank, "world_size": self.world_size, "shard_map": shard_meta,
                          "is_hybrid": is_hybrid},
        }

    def load_state_dict(self, state_dict: Dict[str, Any]):
        meta = state_dict.get("zero_meta", {})
        if meta.get("world_size") is not None and meta["world_size"] != self.world_size:
            warnings.warn(f"ApexWZeRO: checkpoint was saved with world_size={meta['world_size']}, but current "
                          f"world_size={self.world_size}. Use reshard_zero_checkpoint() to convert it.",
                          UserWarning, stacklevel=2)
        if meta.get("rank") is not None and meta["rank"] != self.rank:
            warnings.warn(f"ApexWZeRO: checkpoint rank={meta['rank']} loaded on rank={self.rank}.",
                          UserWarning, stacklevel=2)
        if "local_opt" in state_dict:
            self._local_opt.load_state_dict(state_dict["local_opt"])
        elif "state" in state_dict:
            self._local_opt.load_state_dict(state_dict)
        self._zero_plans = None
        for og, ig in zip(self.param_groups, self._local_opt.param_groups):
            for k, v in ig.items():
                if k != "params":
                    og[k] = v
        for p, st in self._local_opt.state.items():
            if isinstance(p, Tensor):
                for k, v in list(st.items()):
                    if isinstance(v, Tensor) and v.device != p.device and k != "step":
                        st[k] = v.to(p.device)

    def add_param_group(self, param_group: dict):
        super().add_param_group(param_group)
        if not hasattr(self, "_local_opt"):
            return
        group = self.param_groups[-1]
        if self._stores:
            # new parameters join the flat layout in a store of their own
            self._fused = False   # the symmetric layout does not cover the new parameters
            by_dtype: Dict[torch.dtype, List[Tensor]] = {}
            for p in group["params"]:
                by_dtype.setdefault(p.dtype, []).append(p)
            for dt, ps in by_dtype.items():
                store = _FlatStore(ps, dt, ps[0].device, self.process_group, False)
                self._stores.append(store)
                for p in ps:
                    self._param_store[id(p)] = store
        local = self._shard_group(len(self.param_groups) - 1, group)
        self._local_param_groups.append(local)
        self._local_opt.add_param_group(local)
        self._zero_plans = None
