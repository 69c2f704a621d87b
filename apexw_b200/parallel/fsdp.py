"""FSDP helpers and DistMuon (distributed Muon).

``is_fsdp_flat_param`` / ``extract_fsdp_param_infos`` recognise FSDP1 flat parameters and
list the original tensors packed in them (reference: apexw/fsdp.py:38-109).

``DistMuon`` orthogonalises each matrix on exactly one rank.  Differences from the reference
implementation (apexw/fsdp.py:112-272), which keeps a full fp32 momentum copy on every rank
and broadcasts the whole updated parameter:

* the momentum of a matrix exists only on its owner rank (state is 4/world bytes per
  parameter per rank instead of 4);
* ownership is balanced by Newton-Schulz cost (greedy by ``min(m,n)^2 * max(m,n)``) instead of
  index modulo world size, with ties broken by index so every rank computes the same map
  (``balance=False`` gives the reference's index modulo world size, ``balance="shape"`` keeps equal shapes on
  one rank so that they form few large batches);
* same-shaped matrices owned by a rank are orthogonalised as one batch (tcgen05 kernels on
  CUDA, ``ops/newton_schulz.py``);
* the owner sends the updated parameter; with ``torch.distributed`` that is a broadcast per
  parameter, issued asynchronously while the next matrices are being orthogonalised.

On CUDA with bf16 parameters the default is the fused path: parameters and gradients live in flat buffers
that every rank has mapped (CUDA IPC), and a step is, per parameter group, three stages on the owner:
``muon_gather`` (peer loads of the gradient from every rank, averaged in fp32 registers, momentum update,
bf16 Newton-Schulz input staged), the tcgen05 Newton-Schulz kernels, and ``muon_scatter`` (decay + update,
stored into every rank's parameter buffer).  No NCCL call is made on that path; gradients need not be
all-reduced beforehand (``reduce_gradients=True``, the fused default).

On the collectives path gradients are expected to be identical on all ranks (DDP-averaged), as in the
reference, unless ``reduce_gradients=True`` is given: then the step averages them over the group first.
"""

from __future__ import annotations

import math
import os
import warnings
from collections import defaultdict
from typing import Any, Dict, List, Optional, Tuple, Union

import torch
import torch.distributed as dist
import torch.nn as nn
from torch import Tensor
from torch.optim import Optimizer

from .. import _native
from ..ops.newton_schulz import deferred_errors, zeropower_via_newtonschulz5, zeropower_via_newtonschulz5_batched

_STATUS_TEXT = {1: "a peer did not arrive at the step within the time limit (entry round)",
                2: "a peer did not finish writing parameters within the time limit (exit round)",
                3: "the entry verdict did not reach every thread block within the time limit"}


def _to_global_rank(group, rank: int) -> int:
    if group is None or not hasattr(dist, "get_global_rank"):
        return rank
    try:
        return dist.get_global_rank(group, rank)
    except Exception:
        return rank


def is_fsdp_flat_param(param: Tensor) -> bool:
    """True for an FSDP1 ``FlatParameter`` (by flag, class name or ``_param_infos``)."""
    if getattr(param, "_is_flat_param", False):
        return True
    return "FlatParameter" in type(param).__name__ or hasattr(param, "_param_infos")


def extract_fsdp_param_infos(flat_param: Tensor) -> List[Dict[str, Any]]:
    """Name, shape, numel, dtype, offset and ``is_2d`` of every tensor packed in a flat parameter."""
    infos_in = getattr(flat_param, "_param_infos", None)
    if infos_in is None:
        return []
    shapes = getattr(flat_param, "_shapes", None)
    numels = getattr(flat_param, "_numels", None)
    fqns = getattr(flat_param, "_fqns", None)

    def pick(seq, i, info, attr, default):
        if seq is not None and i < len(seq):
            return seq[i]
        return getattr(info, attr, default)

    out, offset = [], 0
    for i, info in enumerate(infos_in):
        shape = pick(shapes, i, info, "shape", None)
        numel = pick(numels, i, info, "numel", None)
        if numel is None:
            numel = math.prod(shape) if shape is not None else 0
        is_2d = False
        if shape is not None and len(shape) >= 2 and shape[0] > 0:
            is_2d = min(shape[0], numel // shape[0]) >= 32
        out.append({
            "param_name": pick(fqns, i, info, "param_name", str(i)),
            "shape": shape,
            "numel": numel,
            "dtype": getattr(info, "dtype", getattr(flat_param, "dtype", torch.float32)),
            "offset": offset,
            "is_2d": is_2d,
        })
        offset += numel
    return out


def fsdp_decay_mask(flat_param: Tensor, shard_offset: int = 0, shard_numel: Optional[int] = None) -> Tensor:
    """0/1 mask over a flat shard marking elements that belong to tensors with dim >= 2.

    ``decay_norm_only`` keys on ``p.dim()``, so a 1-D flat shard is never decayed by the optimizer
    itself.  Multiply the shard by ``1 - lr*wd*mask`` before the step (or pass
    ``adamw_compat=True`` to decay everything) to apply decay to the matrices inside it.
    """
    infos = extract_fsdp_param_infos(flat_param)
    total = sum(i["numel"] for i in infos)
    n = shard_numel if shard_numel is not None else max(total - shard_offset, 0)
    mask = torch.zeros(n, dtype=torch.float32, device=flat_param.device)
    for info in infos:
        if info["shape"] is None or len(info["shape"]) < 2:
            continue
        a = max(info["offset"] - shard_offset, 0)
        b = min(info["offset"] + info["numel"] - shard_offset, n)
        if b > a:
            mask[a:b] = 1.0
    return mask


def fsdp_decay_ranges(flat_param: Tensor) -> Optional[List[Tuple[int, int]]]:
    """Element ranges of this rank's flat shard that belong to tensors with two or more dimensions (the ones that
    ``decay_norm_only`` decays), merged where adjacent; None when the shard's position cannot be told.

    Uses FSDP's own per-parameter shard records (``_shard_param_infos``: offset and length of each original tensor's
    part inside this rank's shard) next to ``_shapes``; an unsharded flat parameter falls back to the offsets of
    ``extract_fsdp_param_infos``.
    """
    shapes = getattr(flat_param, "_shapes", None)
    shard_infos = getattr(flat_param, "_shard_param_infos", None)
    ranges: List[Tuple[int, int]] = []
    if shapes is not None and shard_infos is not None and len(shapes) == len(shard_infos):
        for shape, info in zip(shapes, shard_infos):
            if getattr(info, "in_shard", False) and len(shape) >= 2:
                a = int(info.offset_in_shard)
                ranges.append((a, a + int(info.numel_in_shard)))
    else:
        infos = extract_fsdp_param_infos(flat_param)
        if not infos or sum(i["numel"] for i in infos) > flat_param.numel():
            return None                      # a shard of unknown position
        ranges = [(i["offset"], i["offset"] + i["numel"]) for i in infos if i["shape"] is not None and len(i["shape"]) >= 2]
    ranges.sort()
    merged: List[Tuple[int, int]] = []
    for a, b in ranges:
        if merged and a <= merged[-1][1]:
            merged[-1] = (merged[-1][0], max(merged[-1][1], b))
        elif b > a:
            merged.append((a, min(b, flat_param.numel())))
    return merged


def _is_matrix(t: Tensor) -> bool:
    return t.ndim >= 2 and min(t.shape[0], t.numel() // max(t.shape[0], 1)) >= 16


def _ns_cost(p: Tensor) -> float:
    if not _is_matrix(p):
        return float(p.numel())
    m = p.shape[0]
    n = p.numel() // m
    lo, hi = min(m, n), max(m, n)
    return float(4 * lo * lo * hi + 2 * lo * lo * lo)


def assign_owners_by_shape(params: List[Tensor], world_size: int) -> List[int]:
    """Owner map that keeps equal shapes together: the parameters, ordered by cost and shape, are cut into
    ``world_size`` consecutive runs of about equal Newton-Schulz cost.  A rank then owns one or two shapes and
    orthogonalises them as few large batches (better tensor-core wave fill than many batches of two or three), at
    the price of a load imbalance of up to half of the largest matrix's cost."""
    cost = _ns_cost
    order = sorted(range(len(params)), key=lambda i: (-cost(params[i]), tuple(params[i].shape), i))
    total = sum(cost(p) for p in params)
    owners = [0] * len(params)
    done, rank = 0.0, 0
    for i in order:
        c = cost(params[i])
        if rank < world_size - 1 and done + c / 2 > total * (rank + 1) / world_size:
            rank += 1
        owners[i] = rank
        done += c
    return owners


def assign_owners(params: List[Tensor], world_size: int) -> List[int]:
    """Deterministic cost-balanced owner map: largest Newton-Schulz cost first onto the least loaded rank."""
    cost = _ns_cost
    order = sorted(range(len(params)), key=lambda i: (-cost(params[i]), i))
    load = [0.0] * world_size
    owners = [0] * len(params)
    for i in order:
        r = min(range(world_size), key=lambda k: (load[k], k))
        owners[i] = r
        load[r] += cost(params[i])
    return owners


class DistMuon(Optimizer):
    _step_supports_amp_scaling = True

    def __init__(self, params, lr: float = 2e-2, momentum: float = 0.95, nesterov: bool = True,
                 weight_decay: float = 1e-2, ns_steps: int = 4, world_size: Optional[int] = None,
                 rank: Optional[int] = None, process_group: Optional[Any] = None, balance: Union[bool, str] = "auto",
                 fused: Optional[bool] = None, reduce_gradients: Optional[bool] = None,
                 peer_timeout_ms: Optional[float] = None):
        if dist.is_available() and dist.is_initialized():
            self.world_size = dist.get_world_size(process_group) if world_size is None else world_size
            self.rank = dist.get_rank(process_group) if rank is None else rank
        else:
            self.world_size = world_size or 1
            self.rank = rank or 0
        self.process_group = process_group
        self.balance = balance
        if isinstance(params, nn.Module):
            params = [p for p in params.parameters() if p.requires_grad]
        super().__init__(params, dict(lr=lr, momentum=momentum, nesterov=nesterov, weight_decay=weight_decay,
                                      ns_steps=ns_steps))
        self._live = self.world_size > 1 and dist.is_available() and dist.is_initialized()
        self.peer_timeout_ms = float(peer_timeout_ms if peer_timeout_ms is not None
                                     else os.environ.get("APEXW_B200_PEER_TIMEOUT_MS", 5000.0))
        self._fused = self._setup_fused(fused)
        self.reduce_gradients = bool(reduce_gradients) if reduce_gradients is not None else self._fused

    def add_param_group(self, param_group: dict) -> None:
        super().add_param_group(param_group)
        if getattr(self, "_fused", False):
            # the flat peer-memory buffers were laid out at construction and do not cover the new parameters
            warnings.warn("DistMuon: a parameter group was added after construction; continuing on the collectives path",
                          UserWarning, stacklevel=2)
            self._fused = False
            self._plans = None

    # ------------------------------------------------------------------ fused path (peer memory)

    def _fused_ok_locally(self) -> bool:
        ps = [p for g in self.param_groups for p in g["params"]]
        return (bool(ps) and all(p.is_cuda and p.dtype == torch.bfloat16 and p.numel() % 8 == 0 and p.is_contiguous()
                                 for p in ps)
                and len({p.device for p in ps}) == 1 and _native.available()
                and (self.world_size == 1 or self._live) and self.world_size <= 8)

    def _setup_fused(self, fused: Optional[bool]) -> bool:
        self._store = self._signal = self._status = self._mailbox = None
        self._plans: Optional[List[Dict[str, Any]]] = None
        self._epoch = 0
        ok = fused is not False and self._fused_ok_locally()
        if self._live:   # the symmetric allocation below is collective: decide together first
            votes: List[Any] = [None] * self.world_size
            dist.all_gather_object(votes, bool(ok), group=self.process_group)
            ok = all(votes)
        if fused is True and not ok:
            raise RuntimeError("DistMuon(fused=True) needs contiguous bf16 CUDA parameters on one device with element "
                               "counts divisible by 8, the native library, and a process group of at most 8 ranks")
        if not ok:
            return False
        from .symm import SymmetricBuffer
        from .zero import _FlatStore
        ps = [p for g in self.param_groups for p in g["params"]]
        self._store = _FlatStore(ps, torch.bfloat16, ps[0].device, self.process_group, True)
        self._signal = SymmetricBuffer(256, ps[0].device, self.process_group)
        from .status import StatusMailbox
        self._mailbox = StatusMailbox(ps[0].device, 2)       # word 0: gather / scatter waits, word 1: Newton-Schulz kernels
        self._status, self._ns_status = self._mailbox.word(0), self._mailbox.word(1)
        return True

    def _build_plans(self) -> List[Dict[str, Any]]:
        nat = _native.require()
        dev = self._store.device
        plans = []
        for group in self.param_groups:
            params = list(group["params"])
            owners = self.owners_of(params)
            mine = [p for p, o in zip(params, owners) if o == self.rank]
            mine.sort(key=lambda p: (0 if _is_matrix(p) else 1, tuple(p.shape)))   # equal shapes become neighbours
            total = sum(p.numel() for p in mine)
            staged = torch.zeros(max(total, 8), dtype=torch.bfloat16, device=dev)
            momentum = torch.zeros(max(total, 8), dtype=torch.float32, device=dev)
            m_views, s_views, offsets, scales, batches = [], [], [], [], []
            off = 0
            for p in mine:
                n = p.numel()
                mv = momentum[off:off + n]
                st = self.state[p]
                if "momentum" in st:            # state loaded from a checkpoint before the first step
                    mv.copy_(st["momentum"].reshape(-1))
                st.setdefault("step", 0)
                st["momentum"] = mv.view(p.shape)
                m_views.append(mv)
                s_views.append(staged[off:off + n])
                offsets.append(self._store.offsets[id(p)])
                if _is_matrix(p):
                    rows, cols = p.shape[0], n // p.shape[0]
                    scales.append(max(1.0, math.sqrt(rows / cols)))
                    key = ("matrix", rows, cols)
                else:
                    scales.append(0.05)
                    key = ("vector", n, 1)
                if batches and batches[-1]["key"] == key and batches[-1]["count"] < self._batch_limit(key, len(mine)):
                    batches[-1]["count"] += 1
                else:
                    batches.append({"key": key, "start": off, "count": 1})
                off += n
            dev_index = dev.index if dev.index is not None else torch.cuda.current_device()
            first = 0
            for b in batches:
                kind, rows, cols = b["key"]
                b["view"] = staged[b["start"]:b["start"] + b["count"] * rows * cols].view(b["count"], rows, cols)
                # a launch plan of its own, so that this batch's gather and scatter can run beside the
                # Newton-Schulz kernels of the other batches
                sl = slice(first, first + b["count"])
                b["plan"] = nat.MuonPlan(m_views[sl], s_views[sl], offsets[sl], scales[sl], dev_index)
                b["gathered"], b["done"] = torch.cuda.Event(), torch.cuda.Event()
                first += b["count"]
            plans.append({"plan": nat.MuonPlan(m_views, s_views, offsets, scales, dev.index if dev.index is not None
                                               else torch.cuda.current_device()),
                          "mine": mine, "batches": batches, "staged": staged, "momentum": momentum})
        if self._live:
            dist.barrier(group=self.process_group)   # align ranks once before the first in-kernel wait
        return plans

    def _batch_limit(self, key, owned: int) -> int:
        """Largest number of equally shaped matrices orthogonalised as ONE batch.  A rank that owns a single long run of
        one shape (the shape-keeping owner map on many ranks) would otherwise gather everything, iterate, then scatter
        everything, with the links idle during the tensor-core work and the tensor cores idle during the transfers.
        Cutting the run into about three batches lets gather(i+1) and scatter(i-1) run beside the Newton-Schulz
        kernels of batch i; a batch of four or more 2048-wide matrices still fills the tensor-core grid."""
        env = os.environ.get("APEXW_B200_MUON_BATCH")
        if env:
            return max(1, int(env))
        if key[0] != "matrix":
            return 1 << 30
        return max(4, (owned + 2) // 3)

    def _step_fused(self, inv_scale: Optional[float]) -> None:
        if self._plans is None:
            self._plans = self._build_plans()
        self._store.adopt_grads()
        self._store.finish_grads()
        W = self.world_size
        inv = (1.0 / W if self.reduce_gradients else 1.0) * (inv_scale if inv_scale is not None else 1.0)
        grads = self._store.symm_grad.peer_ptrs if self.reduce_gradients else [self._store.symm_grad.local_ptr]
        params, signal = self._store.symm_param.peer_ptrs, self._signal.peer_ptrs
        timing = os.environ.get("APEXW_B200_MUON_TIMING", "0") not in ("", "0")
        marks = []

        def mark():
            if timing:
                ev = torch.cuda.Event(enable_timing=True)
                ev.record()
                marks.append(ev)

        pipeline = (not timing) and os.environ.get("APEXW_B200_MUON_PIPELINE", "1") not in ("", "0")
        main = torch.cuda.current_stream(self._store.device)
        for group, entry in zip(self.param_groups, self._plans):
            lr, mu, wd = float(group["lr"]), float(group["momentum"]), float(group["weight_decay"])
            self._epoch += 1
            batches = entry["batches"]
            if pipeline and len(batches) >= 2:
                self._step_group_pipelined(group, entry, grads, params, signal, inv, lr, mu, wd, main)
            else:
                mark()
                with _native.nvtx_range("apexw_b200.muon_gather"):
                    entry["plan"].gather(grads, params, signal, self.rank, self._epoch, self.peer_timeout_ms, self._status,
                                         mu, inv, bool(group["nesterov"]))
                mark()
                for b in batches:
                    self._orthogonalise_batch(b, group)
                mark()
                with _native.nvtx_range("apexw_b200.muon_scatter"):
                    entry["plan"].scatter(params, signal, self.rank, self._epoch, self.peer_timeout_ms, self._status,
                                          lr, 1.0 - lr * wd)
                mark()
                _native.count(2)
            for p in entry["mine"]:
                self.state[p]["step"] += 1
        # read-back of the status words behind this step's kernels; the words are cleared for the next step, so one
        # expired wait costs one step, not every later one (within a step the kernels do skip after a failure)
        mine = [p for entry in self._plans for p in entry["mine"]]

        def take_back(codes):
            if codes.get(0) == 1:            # entry round failed: momentum and parameters were left as they were
                for p in mine:
                    self.state[p]["step"] -= 1

        self._mailbox.post(take_back)
        if timing and marks:
            torch.cuda.synchronize()
            #: per group: (gather, orthogonalise, scatter) milliseconds of the last step, when APEXW_B200_MUON_TIMING=1
            self.last_phase_ms = [tuple(marks[i + k].elapsed_time(marks[i + k + 1]) for k in range(3))
                                  for i in range(0, len(marks), 4)]

    def _orthogonalise_batch(self, b: Dict[str, Any], group: Dict[str, Any]) -> None:
        X = b["view"]
        if b["key"][0] == "matrix":
            with deferred_errors(self._ns_status):          # no host sync per batch; check_status() reads the word
                zeropower_via_newtonschulz5_batched(X, steps=group["ns_steps"], out=X)
        else:
            s = X.float()
            spread = s.abs() if s.shape[1] <= 1 else s.std(dim=(1, 2), unbiased=False, keepdim=True)
            X.copy_(s / (spread + 1e-7))

    def _step_group_pipelined(self, group, entry, grads, params, signal, inv, lr, mu, wd, main) -> None:
        """Batches of equally shaped matrices flow through gather -> Newton-Schulz -> scatter with the two
        memory-bound ends on a side stream, so they run beside the tensor-core kernels of the neighbouring batches.
        Only the first gather runs the entry round and only the last scatter the exit round; the scatters share one
        stream, so the exit flag follows all of this step's parameter stores."""
        if getattr(self, "_side", None) is None:
            self._side = torch.cuda.Stream(device=self._store.device)
        side, batches = self._side, entry["batches"]
        side.wait_stream(main)                               # gradients of this step are final on the main stream
        with torch.cuda.stream(side):
            for i, b in enumerate(batches):
                b["plan"].gather(grads, params, signal, self.rank, self._epoch, self.peer_timeout_ms, self._status,
                                 mu, inv, bool(group["nesterov"]), i == 0)
                b["gathered"].record(side)
        for i, b in enumerate(batches):
            main.wait_event(b["gathered"])
            self._orthogonalise_batch(b, group)
            b["done"].record(main)
            with torch.cuda.stream(side):
                side.wait_event(b["done"])
                b["plan"].scatter(params, signal, self.rank, self._epoch, self.peer_timeout_ms, self._status,
                                  lr, 1.0 - lr * wd, i == len(batches) - 1)
        main.wait_stream(side)
        _native.count(2 * len(batches))

    def _poll_status(self, wait: bool = False) -> None:
        if self._mailbox is None:
            return
        from .status import PeerStepError
        try:
            self._mailbox.poll("DistMuon fused step", self.rank, wait=wait)
        except PeerStepError as exc:
            if 0 not in exc.codes and 1 in exc.codes:
                raise PeerStepError(f"DistMuon fused step failed on rank {self.rank}: a bounded wait expired inside the "
                                    f"Newton-Schulz GEMM kernel (code {exc.codes[1]})", exc.codes) from None
            raise

    def check_status(self) -> None:
        """Wait for the status words of every step issued so far (one host sync) and raise if a wait ran out.  Not
        needed in a training loop: ``step()`` and ``zero_grad()`` report a failed earlier step by themselves."""
        self._poll_status(wait=True)

    def zero_grad(self, set_to_none: bool = True):
        if self._fused:
            self._poll_status()
            self._store.clear_grads()    # gradients are persistent views of the flat buffer
            return
        super().zero_grad(set_to_none=set_to_none)

    def load_state_dict(self, state_dict):
        super().load_state_dict(state_dict)
        if self._fused and self._plans is not None:   # re-seat loaded momenta into the flat fp32 buffer
            for entry in self._plans:
                off = 0
                for p in entry["mine"]:
                    n, st = p.numel(), self.state[p]
                    mv = entry["momentum"][off:off + n].view(p.shape)
                    if "momentum" in st and st["momentum"].data_ptr() != mv.data_ptr():
                        mv.copy_(st["momentum"])
                    st["momentum"] = mv
                    off += n

    # ------------------------------------------------------------------ collectives path

    def owners_of(self, params: List[Tensor]) -> List[int]:
        # "auto" is the cost-balanced map.  Measured for the 1.1B model's 88 matrices on 8 GPUs: 9.7 ms cost-balanced
        # (batches of two or three matrices per shape), 10.3 ms with equal shapes kept together and cut into three
        # batches, 10.2 ms uncut - the tighter balance wins by a little, so shape-keeping stays an option.
        if self.balance == "shape":
            return assign_owners_by_shape(params, self.world_size)
        if self.balance:
            return assign_owners(params, self.world_size)
        return [i % self.world_size for i in range(len(params))]

    @staticmethod
    def _update_source(p: Tensor, st: dict, momentum: float, nesterov: bool) -> Tensor:
        g = torch.nan_to_num(p.grad, nan=0.0, posinf=65504.0, neginf=-65504.0).float()
        buf = st["momentum"]
        buf.mul_(momentum).add_(g, alpha=1.0 - momentum)
        return g.lerp(buf, momentum) if nesterov else buf

    @torch.no_grad()
    def step(self, closure=None):
        loss = None
        if closure is not None:
            with torch.enable_grad():
                loss = closure()
        found_inf = getattr(self, "found_inf", None)
        if found_inf is not None and self._live:
            from .zero import _agree_found_inf
            found_inf = _agree_found_inf(found_inf, True, self.process_group)
        if found_inf is not None and float(found_inf) > 0:
            return loss
        grad_scale = getattr(self, "grad_scale", None)
        inv = None if grad_scale is None else (1.0 / float(grad_scale))
        live = self._live
        if self._fused:
            try:
                self._poll_status()          # a wait that ran out in an earlier step surfaces here, without a host sync
                self._step_fused(inv)
            finally:
                self.grad_scale = None
                self.found_inf = None
            return loss
        try:
            for group in self.param_groups:
                lr, mu, wd = group["lr"], group["momentum"], group["weight_decay"]
                params = [p for p in group["params"] if p.grad is not None]
                if not params:
                    continue
                if live and self.reduce_gradients:
                    handles = [dist.all_reduce(p.grad, op=dist.ReduceOp.SUM, group=self.process_group, async_op=True)
                               for p in params]
                    for h in handles:
                        h.wait()
                    for p in params:
                        p.grad.div_(self.world_size)
                if inv is not None and inv != 1.0:
                    for p in params:
                        p.grad.mul_(inv)
                owners = self.owners_of(params)
                mine = [p for p, o in zip(params, owners) if o == self.rank]
                by_shape: Dict[Tuple[int, ...], List[Tensor]] = defaultdict(list)
                for p in mine:
                    st = self.state[p]
                    if not st:
                        st["step"] = 0
                        st["momentum"] = torch.zeros_like(p, dtype=torch.float32)
                    st["step"] += 1
                    by_shape[tuple(p.shape)].append(p)
                for shape, ps in by_shape.items():
                    srcs = [self._update_source(p, self.state[p], mu, group["nesterov"]) for p in ps]
                    if _is_matrix(ps[0]):
                        if len(ps) > 1:
                            X = torch.stack([s.reshape(shape[0], -1) for s in srcs])
                            X = X.to(torch.bfloat16) if X.is_cuda else X
                            Us = zeropower_via_newtonschulz5_batched(X, steps=group["ns_steps"]).float()
                            Us = [Us[i].reshape(shape) for i in range(len(ps))]
                        else:
                            # tensors with more than two dimensions are orthogonalised as (shape[0], -1), the view
                            # that the eligibility test and the update scale already assume
                            Us = [zeropower_via_newtonschulz5(srcs[0].reshape(shape[0], -1),
                                                              steps=group["ns_steps"]).reshape(shape)]
                        m_dim, n_dim = shape[0], ps[0].numel() // shape[0]
                        scale = max(1.0, math.sqrt(m_dim / n_dim))
                    else:
                        Us = [s / ((s.abs() if s.numel() <= 1 else s.std(unbiased=False)) + 1e-7) for s in srcs]
                        scale = 0.05
                    for p, U in zip(ps, Us):
                        if wd != 0.0:
                            p.mul_(1.0 - lr * wd)
                        p.add_(U.to(p.dtype), alpha=-lr * scale)
                if live:
                    handles = [dist.broadcast(p.data, src=_to_global_rank(self.process_group, o),
                                              group=self.process_group, async_op=True)
                               for p, o in zip(params, owners)]
                    for h in handles:
                        h.wait()
                elif self.world_size > 1 and not getattr(self, "_warned_unsynced", False):
                    warnings.warn(f"DistMuon: world_size={self.world_size} specified, but torch.distributed is not "
                                  f"initialized. Parameters on non-owner ranks will not be synchronized.",
                                  UserWarning, stacklevel=2)
                    self._warned_unsynced = True
        finally:
            self.grad_scale = None
            self.found_inf = None
        return loss

    def get_state_memory_mb(self) -> float:
        total = sum(v.numel() * v.element_size() for st in self.state.values() for v in st.values() if isinstance(v, Tensor))
        if total == 0:
            total = sum(p.numel() * 4.0 for g in self.param_groups for p in g["params"]) / max(1, self.world_size)
        return total / (1024 * 1024)
