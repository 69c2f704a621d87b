"""ApexW: memory-efficient AdamW with compact (2.50 B/param) and 8-bit (0.754 B/param) state.

Drop-in for ``torch.optim.AdamW`` with the constructor, parameter-group keys,
state layout and ``state_dict`` format of the reference optimizer
(apexw/optimizer.py:1510-1839 constructor, :2473-2572 checkpoint, :2574-2957
state layout, :3358-4094 step dispatch).

Execution model (this is where the design departs from the reference): there
are two engines and no backend chain.

* CUDA tensors in the hot modes (dense fp32/bf16 moments with or without the
  shared-by-four variance; NF4/int8 momentum with log-uint8 variance) are
  stepped by the fused sm_100a kernels through a resident ``StatePlan`` per
  parameter group: one persistent launch per format class, no per-step
  metadata upload, no host synchronisation.
* Everything else (CPU tensors, fp16/fp64/complex parameters, Lion, AMSGrad,
  AdEMAMix, factored variance, ``ultra``, capturable mode ...) runs through
  ``engine_torch.update_tensor``, which is also the kernels' test oracle.

Both engines draw stochastic-rounding bits from the same counter-based
generator, so a run is reproducible from ``seed`` alone and a CPU run makes the
same rounding decisions as a GPU run.
"""

from __future__ import annotations

import math
import os
import sys
import warnings
from collections import defaultdict
from typing import Any, Callable, Dict, List, Optional, Tuple, Union

import torch
import torch.nn as nn
from torch import Tensor
from torch.optim import Optimizer

from .. import _native
from ..utils import table_check as _table_check
from . import engine_torch as _eng
from .packing import StateDictWrapper, setup_auto_packing, gather_packed_grads
from .rules import (
    BETA2_V_FP32_THRESHOLD,
    BETA2_WARN_THRESHOLD,
    Layout,
    _detect_peft_context,
    _get_scalar_dtype,
    _normalize_precision,
    choose_layout,
    is_hybrid_alias,
)

_VALID_BACKENDS = (None, "auto", "triton", "cuda", "mps", "foreach", "_multi_tensor", "xla")

# kernel classes of csrc/fused_state.cu
_KC_DENSE, _KC_DENSE_QUAD, _KC_INT8, _KC_NF4, _KC_NF4_QUAD, _KC_ULTRA, _KC_FACTORED, _KC_LION8 = range(8)
_SEG_DECAY, _SEG_QUAD = 1, 2
_STEP_STOCHASTIC, _STEP_NESTEROV, _STEP_CAUTIOUS, _STEP_MAXIMIZE = 1, 2, 4, 8
_STEP_LION, _STEP_SLOW, _STEP_AMSGRAD = 16, 32, 64


def _debug(msg: str) -> None:
    if os.environ.get("APEXW_B200_DEBUG"):
        print(f"[apexw_b200] {msg}")


#: launch plans kept per optimizer.  Whole groups need one each; in-backward stepping steps sub-sets of a group (one
#: plan per sub-set: a model with a few hundred tensors flushed fourteen at a time needs dozens), so the bound is
#: generous and eviction takes the least recently used plan.
_MAX_CACHED_PLANS = 512


class _GroupPlan:
    """Cached native launch plans of one parameter group (one per kernel class)."""

    __slots__ = ("param_ids", "classes", "fallback", "stochastic", "signature", "dynamic")

    def __init__(self):
        self.dynamic = False          # some launch plan was switched to device-resident step / learning-rate scalars
        self.param_ids: Tuple[int, ...] = ()
        self.classes: List[Tuple[Any, List[Tensor]]] = []   # (StatePlan, params in plan order)
        self.fallback: List[Tensor] = []                      # params stepped by the torch engine
        self.stochastic = True


class ApexW(Optimizer):
    r"""Memory-efficient AdamW.

    Args mirror the reference (apexw/optimizer.py:1632-1668), in the same
    positional order.  ``seed`` (keyword only) is an addition: it keys the
    counter-based stochastic-rounding generator.
    """

    _step_supports_amp_scaling = True

    def __new__(cls, *args, **kwargs):
        first = args[0] if args else kwargs.get("params")
        use_muon = kwargs.get("use_muon", args[26] if len(args) > 26 else False)
        prec = kwargs.get("precision", args[16] if len(args) > 16 else None)
        if bool(use_muon) or is_hybrid_alias(prec):
            from .hybrid import HybridApexW
            a = list(args)
            kw = dict(kwargs)
            kw.pop("use_muon", None)
            if len(a) > 26:
                a.pop(26)
            if is_hybrid_alias(kw.get("precision")):
                kw["precision"] = "compact"
            if len(a) > 16 and is_hybrid_alias(a[16]):
                a[16] = "compact"
            return HybridApexW(*a, **kw)
        return super().__new__(cls)

    def __init__(
        self,
        params,
        lr: float = 1e-3,
        betas: Optional[Union[Tuple[float, float], Tuple[float, float, float]]] = None,
        eps: float = 1e-8,
        weight_decay: float = 1e-2,
        amsgrad: bool = False,
        nesterov: bool = False,
        cautious: bool = False,
        grad_centralization: bool = False,
        decay_norm_only: bool = True,
        adamw_compat: bool = False,
        clip_grad_norm: Optional[float] = None,
        beta3: Optional[float] = None,
        alpha: float = 5.0,
        lion: bool = False,
        fused: Optional[bool] = None,
        precision: Union[str, torch.dtype] = "compact",
        threshold: int = 65536,
        maximize: bool = False,
        foreach: Optional[bool] = None,
        capturable: bool = False,
        dynamic_scaling: bool = True,
        differentiable: bool = False,
        backend: Optional[str] = None,
        auto_pack: bool = False,
        pack_threshold: int = 50000,
        use_muon: bool = False,
        amp: Optional[bool] = None,
        stochastic_rounding: bool = True,
        block_size: Optional[int] = None,
        force_compact_v: bool = False,
        factored_v: bool = False,
        int4_m: Optional[bool] = None,
        six_bit: bool = False,
        *,
        seed: int = 0,
    ):
        precision = _normalize_precision(precision)
        if precision == "hybrid":
            precision = "compact"
        if betas is None:
            betas = (0.9, 0.999) if precision in ("8bit", "full") else (0.9, 0.99)
        if isinstance(params, nn.Module):
            if amp is None and any(p.dtype in (torch.float16, torch.bfloat16) for p in params.parameters()):
                amp = True
            for name, p in params.named_parameters():
                if not hasattr(p, "_param_name"):
                    p._param_name = name
            trainable = [p for p in params.parameters() if p.requires_grad]
            params = trainable if trainable else list(params.parameters())
        if differentiable:
            raise NotImplementedError("ApexW does not currently support differentiable=True.")
        if not 0.0 <= lr:
            raise ValueError(f"Invalid learning rate: {lr}")
        if not 0.0 <= eps:
            raise ValueError(f"Invalid epsilon value: {eps}")
        if not 0.0 <= betas[0] < 1.0:
            raise ValueError(f"Invalid beta1 parameter: {betas[0]}")
        if not 0.0 <= betas[1] < 1.0:
            raise ValueError(f"Invalid beta2 parameter: {betas[1]}")
        if len(betas) > 2 and beta3 is None:
            beta3 = betas[2]
        if beta3 is not None and not 0.0 <= beta3 < 1.0:
            raise ValueError(f"Invalid beta3 parameter: {beta3}")
        if not 0.0 <= weight_decay:
            raise ValueError(f"Invalid weight_decay value: {weight_decay}")
        if clip_grad_norm is not None and clip_grad_norm <= 0.0:
            raise ValueError(f"Invalid clip_grad_norm value: {clip_grad_norm}")
        if block_size is not None and (isinstance(block_size, bool) or not isinstance(block_size, int) or block_size <= 0):
            raise ValueError(f"Invalid block_size value: {block_size}. Must be a positive integer.")
        if threshold <= 0:
            raise ValueError(f"Invalid threshold value: {threshold}. Must be positive.")
        if alpha < 0.0:
            raise ValueError(f"Invalid alpha value: {alpha}")
        if backend not in _VALID_BACKENDS:
            raise ValueError(f"Invalid backend '{backend}'. Must be 'auto', 'triton', 'cuda', 'mps', 'foreach', or 'xla'.")

        if adamw_compat:
            decay_norm_only = False
            if tuple(betas[:2]) in ((0.9, 0.95), (0.9, 0.99)):
                betas = (0.9, 0.999)

        beta2 = betas[1]
        if (not adamw_compat and precision in ("auto", "compact") and beta2 >= BETA2_WARN_THRESHOLD
                and not stochastic_rounding):
            margin = (1.0 - beta2) * 128
            if beta2 >= BETA2_V_FP32_THRESHOLD:
                warnings.warn(
                    f"ApexW: beta2={beta2} with precision='{precision}' and stochastic_rounding=False causes severe "
                    f"bf16 second-moment stagnation (bf16 margin ≈ {margin:.2f}×). exp_avg_sq (v) is automatically "
                    f"stored in float32. Keep stochastic_rounding=True for the full memory saving.",
                    UserWarning, stacklevel=2)
            else:
                warnings.warn(
                    f"ApexW: beta2={beta2} with precision='{precision}' and stochastic_rounding=False may cause mild "
                    f"bf16 second-moment precision loss (bf16 margin ≈ {margin:.2f}×) on long runs.",
                    UserWarning, stacklevel=2)

        defaults = dict(
            lr=lr, betas=(betas[0], betas[1]), eps=eps, weight_decay=weight_decay, amsgrad=amsgrad,
            nesterov=nesterov, cautious=cautious, grad_centralization=grad_centralization,
            decay_norm_only=decay_norm_only, clip_grad_norm=clip_grad_norm, beta3=beta3, alpha=alpha, lion=lion,
            fused=fused, precision=precision, threshold=threshold, maximize=maximize, foreach=foreach,
            capturable=capturable, dynamic_scaling=dynamic_scaling, differentiable=differentiable, backend=backend,
            auto_pack=auto_pack, pack_threshold=pack_threshold, amp=amp, stochastic_rounding=stochastic_rounding,
            block_size=block_size, force_compact_v=force_compact_v, factored_v=factored_v, int4_m=int4_m,
            six_bit=six_bit,
        )
        super().__init__(params, defaults)
        self.seed = int(seed)
        self._workspace_pool: Dict[Any, Any] = {}
        self._execution_plans: Dict[int, _GroupPlan] = {}
        self._salts: Dict[int, int] = {}
        self.auto_pack = auto_pack
        self.pack_threshold = pack_threshold
        self.packed_param_groups: List[Dict[str, Any]] = []
        self._param_to_packed: Dict[int, Tuple] = {}
        if self.auto_pack:
            self.state = StateDictWrapper(self, self.state)
            setup_auto_packing(self)

        if (precision == "auto" and amp is not True and not _detect_peft_context(self.param_groups)
                and any(isinstance(p, Tensor) and p.is_cuda and p.dtype == torch.float32
                        for g in self.param_groups for p in g["params"])
                and not any(isinstance(p, Tensor) and p.dtype in (torch.float16, torch.bfloat16)
                            for g in self.param_groups for p in g["params"])):
            warnings.warn(
                "ApexW detected FP32 parameters on CUDA. With precision='auto', optimizer states use float32. "
                "Train with 16-bit Mixed Precision (AMP) to halve optimizer state memory; in pure FP32 training "
                "precision='compact' forces bf16 states.",
                UserWarning, stacklevel=2)

        if any(isinstance(p, Tensor) and p.dtype == torch.float16 for g in self.param_groups for p in g["params"]):
            from .runtime_hooks import set_fp16_active
            set_fp16_active(True, owner=self)    # GradScaler then accepts fp16 gradients; loss scale <= 256 while this lives

        self._has_stepped = False
        self._native_ok = True           # cleared when a native launch raised; the torch engine takes over
        self._native_launches = 0
        self._fused_backward_enabled = False
        self._fused_backward_handles: List[Any] = []
        self._auto_hook_handles: List[Any] = []
        self._auto_hook_queue: List[Tuple[Tensor, dict]] = []
        self._grad_accum_steps = 1
        self._managed_externally = False  # set by ZeRO/FSDP wrappers: no automatic in-backward stepping
        if precision == "8bit":
            from . import backward_hooks
            backward_hooks.maybe_enable_8bit_runtime(self)

    # ------------------------------------------------------------------ bookkeeping

    def __setstate__(self, state):
        super().__setstate__(state)
        for group in self.param_groups:
            for k, v in (("amsgrad", False), ("nesterov", False), ("cautious", False), ("grad_centralization", False),
                         ("decay_norm_only", True), ("dynamic_scaling", True), ("clip_grad_norm", None),
                         ("beta3", None), ("alpha", 5.0), ("lion", False), ("fused", None), ("precision", "compact"),
                         ("threshold", 65536), ("maximize", False), ("foreach", None), ("capturable", False),
                         ("differentiable", False), ("backend", None), ("amp", None), ("stochastic_rounding", True),
                         ("force_compact_v", False), ("factored_v", False), ("int4_m", False), ("six_bit", False)):
                group.setdefault(k, v)
        self._execution_plans = {}
        if not hasattr(self, "_salts"):
            self._salts = {}
        if not hasattr(self, "seed"):
            self.seed = 0

    def add_param_group(self, param_group):
        super().add_param_group(param_group)
        if hasattr(self, "_execution_plans"):
            self._execution_plans = {}

    def zero_grad(self, set_to_none: bool = True):
        super().zero_grad(set_to_none=set_to_none)
        if hasattr(self, "_auto_hook_queue"):
            self._auto_hook_queue.clear()
        if getattr(self, "auto_pack", False):
            for packed in self.packed_param_groups:
                for p in packed["individual_params"]:
                    if set_to_none:
                        p.grad = None
                    elif p.grad is not None:
                        p.grad.zero_()

    def _salt_of(self, p: Tensor) -> int:
        """Stable per-parameter salt of the rounding generator: position in param_groups order."""
        s = self._salts.get(id(p))
        if s is None:
            self._salts = {}
            i = 0
            for g in self.param_groups:
                for q in g["params"]:
                    self._salts[id(q)] = i
                    i += 1
            s = self._salts.get(id(p), 0)
        return s

    # ------------------------------------------------------------------ memory reports

    def get_state_memory_mb(self) -> float:
        total = 0
        for st in self.state.values():
            for v in st.values():
                if torch.is_tensor(v) and v.ndim >= 1:
                    total += v.nelement() * v.element_size()
        return total / (1024 * 1024)

    def get_memory_summary(self) -> str:
        actual = self.get_state_memory_mb()
        count = sum(p.numel() for g in self.param_groups for p in g["params"])
        adamw = count * 8 / (1024 * 1024)
        saved = adamw - actual
        pct = (saved / adamw * 100.0) if adamw > 0 else 50.0
        return ("Optimizer State Memory:\n"
                f"  - ApexW Current State : {actual:.2f} MB\n"
                f"  - PyTorch AdamW Equiv : {adamw:.2f} MB\n"
                f"  - Memory Reduction    : {pct:.1f}% ({saved:.2f} MB saved)")

    def print_summary(self) -> None:
        print(self.get_memory_summary())

    def __repr__(self) -> str:
        count = sum(p.numel() for g in self.param_groups for p in g["params"])
        state_mb = self.get_state_memory_mb()
        adamw = count * 8 / (1024 * 1024)
        g0 = self.param_groups[0]
        if state_mb > 0:
            saved = (adamw - state_mb) / max(adamw, 1e-6) * 100.0
        else:
            saved = {"full": 0.0, "8bit": 75.0, "ultra": 62.5}.get(g0.get("precision", "compact"), 50.0)
        return (f"ApexW(lr={g0['lr']}, betas={g0['betas']}, weight_decay={g0['weight_decay']}, "
                f"precision='{g0['precision']}', params={count:,}, state_memory={state_mb:.2f}MB, "
                f"vram_saved={saved:.1f}%)")

    # ------------------------------------------------------------------ in-backward stepping

    def enable_fused_backward(self, model: Optional[Any] = None, grad_accum_steps: int = 1) -> None:
        from . import backward_hooks
        backward_hooks.enable_fused_backward(self, model, grad_accum_steps)

    def disable_fused_backward(self) -> None:
        from . import backward_hooks
        backward_hooks.disable_fused_backward(self)

    def _disable_auto_8bit_hooks(self) -> None:
        from . import backward_hooks
        backward_hooks.disable_auto_hooks(self)

    # ------------------------------------------------------------------ checkpoint

    def state_dict(self) -> Dict[str, Any]:
        sd = super().state_dict()
        meta = {}
        for p, s in self.state.items():
            if "scale_v" in s:
                meta[id(p)] = {"scale_v": s["scale_v"], "sqrt_scale_v": s.get("sqrt_scale_v", math.sqrt(s["scale_v"]))}
        sd["_dynamic_scaling_meta"] = meta
        return sd

    def load_state_dict(self, state_dict: Dict[str, Any]) -> None:
        """Load a checkpoint written by this class or by the reference optimizer.

        ``Optimizer.load_state_dict`` casts floating state to the parameter dtype;
        every moment is therefore re-copied from the saved dict in its recorded
        storage dtype, and quantised moments / scales are forced back to
        uint8/int8/float32 (reference: apexw/optimizer.py:2486-2572).
        """
        clean = dict(state_dict)
        clean.pop("_dynamic_scaling_meta", None)
        saved_state = clean.get("state", {})
        saved_groups = clean.get("param_groups", [])
        self._check_saved_state_fits(saved_state, saved_groups)     # before anything is mutated
        super().load_state_dict(clean)
        self._workspace_pool = {}
        self._execution_plans = {}
        self._salts = {}

        origin: Dict[Tensor, dict] = {}
        for sg, cg in zip(saved_groups, self.param_groups):
            for old_id, p in zip(sg.get("params", ()), cg.get("params", ())):
                if old_id in saved_state:
                    origin[p] = saved_state[old_id]

        def _restore(s, src_state, key, dtype):
            if key in s and torch.is_tensor(s[key]):
                src = src_state.get(key)
                if torch.is_tensor(src):
                    s[key] = src.to(device=s[key].device, dtype=dtype).clone()
                elif s[key].dtype != dtype:
                    s[key] = s[key].to(dtype)

        for p, s in self.state.items():
            src = origin.get(p, {})
            m_dt, v_dt = s.get("state_dtype"), s.get("state_dtype_v")
            if s.get("is_4bit_m", False) or s.get("is_6bit_m", False):
                _restore(s, src, "exp_avg", torch.uint8)
                _restore(s, src, "exp_avg_slow", torch.int8)
            elif s.get("is_8bit", False) or s.get("is_ultra", False) or m_dt == torch.int8:
                _restore(s, src, "exp_avg", torch.int8)
                _restore(s, src, "exp_avg_slow", torch.int8)
            elif isinstance(m_dt, torch.dtype):
                _restore(s, src, "exp_avg", m_dt)
                _restore(s, src, "exp_avg_slow", m_dt)
            for k in ("exp_avg_scales", "exp_avg_slow_scales", "exp_avg_sq_scales", "exp_avg_sq_row", "exp_avg_sq_col"):
                _restore(s, src, k, torch.float32)
            if (s.get("is_8bit", False) and not s.get("is_factored_v", False)) or v_dt == torch.uint8:
                _restore(s, src, "exp_avg_sq", torch.uint8)
                if "max_exp_avg_sq" in s:
                    _restore(s, src, "max_exp_avg_sq", torch.float32)
            elif isinstance(v_dt, torch.dtype):
                _restore(s, src, "exp_avg_sq", v_dt)
                _restore(s, src, "max_exp_avg_sq", torch.float32 if s.get("is_ultra", False) else v_dt)
            if torch.is_tensor(s.get("step")) and torch.is_tensor(src.get("step")):
                s["step"] = src["step"].to(device=s["step"].device, dtype=src["step"].dtype).clone()

    def _check_saved_state_fits(self, saved_state: Dict[Any, dict], saved_groups: List[dict]) -> None:
        """Reject a checkpoint whose moment tensors do not fit this optimizer's parameters.

        A file written for another shard layout (a ZeRO checkpoint of a different world size that was not
        resharded, a model of other dimensions) would otherwise load silently and fail inside the next
        step.  Runs before any state is replaced, so a rejected file leaves the optimizer as it was.
        """
        from ..ops.formats import six_bit_padded_len
        for gi, (sg, cg) in enumerate(zip(saved_groups, self.param_groups)):
            for pi, (old_id, p) in enumerate(zip(sg.get("params", ()), cg.get("params", ()))):
                src = saved_state.get(old_id)
                if not isinstance(src, dict):
                    continue
                n = p.numel()
                bs = int(src.get("block_size_8bit", src.get("ultra_block_size", 0)) or 0)
                want: Dict[str, int] = {}
                if src.get("is_6bit_m", False) and bs:
                    want["exp_avg"] = six_bit_padded_len(n, bs) * 3 // 4
                elif src.get("is_4bit_m", False):
                    want["exp_avg"] = (n + 1) // 2
                else:
                    want["exp_avg"] = n
                want["exp_avg_sq"] = n // 4 if src.get("is_quad_v", False) else n
                if bs and not src.get("is_6bit_m", False):
                    want["exp_avg_scales"] = want["exp_avg_sq_scales"] = (n + bs - 1) // bs
                for key, expect in want.items():
                    t = src.get(key)
                    if torch.is_tensor(t) and t.numel() != expect:
                        raise ValueError(
                            f"checkpoint does not fit: state '{key}' of parameter {pi} in group {gi} holds {t.numel()} "
                            f"elements, but the parameter (shape {tuple(p.shape)}) needs {expect}. The file was written "
                            f"for another model or shard layout (a ZeRO checkpoint of another world size has to go "
                            f"through reshard_zero_checkpoint first).")

    # ------------------------------------------------------------------ state allocation

    def _init_state(self, p: Tensor, group: Dict[str, Any], ctx: Dict[str, Any]) -> Dict[str, Any]:
        """Allocate the per-parameter state in the reference's layout (apexw/optimizer.py:2611-2931)."""
        st = self.state[p]
        if len(st) != 0:
            self._late_init(p, group, st)
            return st
        fused = bool(group.get("fused", False))
        st["stochastic_rounding"] = bool(group.get("stochastic_rounding", True))
        on_device = bool(group["capturable"] or fused)
        st["step"] = (torch.zeros((), dtype=_get_scalar_dtype(is_fused=fused), device=p.device) if on_device
                      else torch.tensor(0.0, dtype=_get_scalar_dtype(), device="cpu"))
        lay: Layout = choose_layout(p, group, n_group_params=len(group["params"]),
                                    has_16bit_params=ctx["has_16bit"], peft_ctx=ctx["peft"],
                                    auto_pack=bool(getattr(self, "auto_pack", False)))
        for name in lay.flags_present:
            st[name] = bool(getattr(lay, name))
        if lay.is_quad_v:
            st["is_quad_v"] = True
        if lay.is_8bit:
            st["block_size_8bit"] = lay.block_size
            st["m_numel"] = p.numel()
        if lay.is_ultra:
            st["ultra_block_size"] = lay.block_size
        st["state_dtype"] = lay.m_dtype
        st["state_dtype_v"] = lay.v_dtype
        n, dev = p.numel(), p.device
        lion = bool(group["lion"])
        has_slow = group["beta3"] is not None

        if lay.is_8bit or lay.is_ultra:
            bs = lay.block_size
            nblk = (n + bs - 1) // bs
            if lay.is_6bit_m:
                from ..ops.formats import six_bit_padded_len
                padded = six_bit_padded_len(n, bs)
                st["exp_avg"] = torch.tensor([0xDF, 0xF7, 0x7D], dtype=torch.uint8, device=dev).repeat(padded // 4)
                st["exp_avg_scales"] = torch.full((padded // bs, 1), 1e-12 / 31.0, dtype=torch.float32, device=dev)
            elif lay.is_4bit_m:
                st["exp_avg"] = torch.full(((n + 1) // 2,), 0x77, dtype=torch.uint8, device=dev)
                st["exp_avg_scales"] = torch.full((nblk, 1), 1e-12, dtype=torch.float32, device=dev)
            else:
                st["exp_avg"] = torch.zeros_like(p, dtype=torch.int8)
                st["exp_avg_scales"] = torch.full((nblk, 1), 1e-12 / 127.0, dtype=torch.float32, device=dev)
            if has_slow:
                st["exp_avg_slow"] = torch.zeros_like(p, dtype=torch.int8)
                st["exp_avg_slow_scales"] = torch.full((nblk, 1), 1e-12 / 127.0, dtype=torch.float32, device=dev)
        else:
            st["exp_avg"] = torch.zeros_like(p, dtype=lay.m_dtype, memory_format=torch.preserve_format)
            if has_slow:
                st["exp_avg_slow"] = torch.zeros_like(p, dtype=lay.m_dtype, memory_format=torch.preserve_format)

        if not lion:
            if lay.is_factored_v:
                rows = p.shape[0]
                st["exp_avg_sq_row"] = torch.zeros(rows, dtype=torch.float32, device=dev)
                st["exp_avg_sq_col"] = torch.zeros(n // rows, dtype=torch.float32, device=dev)
            elif lay.is_8bit:
                nblk = (n + lay.block_size - 1) // lay.block_size
                st["exp_avg_sq"] = (torch.zeros((n // 4,), dtype=torch.uint8, device=dev) if lay.is_quad_v
                                    else torch.zeros_like(p, dtype=torch.uint8))
                st["exp_avg_sq_scales"] = torch.full((nblk, 1), 1e-12, dtype=torch.float32, device=dev)
            elif lay.is_quad_v:
                st["exp_avg_sq"] = torch.zeros((n // 4,), dtype=lay.v_dtype, device=dev)
            else:
                st["exp_avg_sq"] = torch.zeros_like(p, dtype=lay.v_dtype, memory_format=torch.preserve_format)
            if group["amsgrad"]:
                mx_dt = torch.float32 if (lay.is_8bit or lay.is_ultra) else lay.v_dtype
                st["max_exp_avg_sq"] = torch.zeros(n, dtype=mx_dt, device=dev).reshape(p.shape)

        if not (lay.is_8bit or lay.is_ultra):
            if group.get("dynamic_scaling", True) and not lion and lay.v_dtype == torch.float16:
                st["scale_v"], st["sqrt_scale_v"] = 1024.0, 32.0
            else:
                st["scale_v"], st["sqrt_scale_v"] = 1.0, 1.0
        return st

    def _late_init(self, p: Tensor, group: Dict[str, Any], st: Dict[str, Any]) -> None:
        """Buffers for options switched on after the first step (AMSGrad, AdEMAMix)."""
        m_dt = st.get("state_dtype", p.dtype)
        v_dt = st.get("state_dtype_v", m_dt)
        quantised = st.get("is_8bit", False) or st.get("is_ultra", False)
        if group["beta3"] is not None and "exp_avg_slow" not in st:
            if quantised:
                bs = st.get("block_size_8bit", st.get("ultra_block_size", 2048))
                st["exp_avg_slow"] = torch.zeros_like(p, dtype=torch.int8)
                st["exp_avg_slow_scales"] = torch.full(((p.numel() + bs - 1) // bs, 1), 1e-12 / 127.0,
                                                       dtype=torch.float32, device=p.device)
            else:
                st["exp_avg_slow"] = torch.zeros_like(p, dtype=m_dt, memory_format=torch.preserve_format)
        if not group["lion"] and group["amsgrad"] and "max_exp_avg_sq" not in st and "exp_avg_sq" in st:
            if st.get("is_quad_v", False):
                raise RuntimeError("amsgrad cannot be enabled after state with a shared second moment was created")
            mx_dt = torch.float32 if quantised else v_dt
            st["max_exp_avg_sq"] = torch.zeros(p.numel(), dtype=mx_dt, device=p.device).reshape(p.shape)

    # ------------------------------------------------------------------ gradient preparation

    @staticmethod
    def _prepare_grads(grads: List[Tensor], group: Dict[str, Any], grad_scale: Optional[Tensor]):
        """Centralisation and global-norm clipping (with AMP unscale first when either is on).

        Works on ``p.grad`` in place, as the reference does for finite gradients (its tests read the
        centralised gradient back from ``p.grad`` after the step), so no second copy of the gradients is
        held.  Element-wise NaN/Inf sanitising is done inside both engines, so no separate finiteness pass
        is needed here (reference: apexw/optimizer.py:136-258).
        """
        clip = group.get("clip_grad_norm")
        cent = group.get("grad_centralization", False)
        if not grads or (clip is None and not cent):
            return grads, grad_scale
        out = list(grads)
        if grad_scale is not None:
            inv = grad_scale.to(out[0].device).reciprocal()
            torch._foreach_mul_(out, inv)
            grad_scale = None
        if cent:
            for g in out:
                if g.dim() >= 2:
                    g.sub_(g.mean(dim=tuple(range(1, g.dim())), keepdim=True))
        if clip is not None:
            norms = torch._foreach_norm(out, 2.0)
            dev = out[0].device
            total = torch.linalg.vector_norm(torch.stack([n.to(device=dev, dtype=torch.float32) for n in norms]), 2.0)
            coef = torch.clamp(clip / (total + 1e-6), max=1.0)
            torch._foreach_mul_(out, coef)
        return out, grad_scale

    # ------------------------------------------------------------------ step

    def step(self, closure: Optional[Callable] = None):
        if "torch._dynamo" in sys.modules:        # torch.compile is in use somewhere: keep the tracer out of the step
            return _untraced_step()(self, closure)
        return self._step_impl(closure)

    @torch.no_grad()
    def _step_impl(self, closure: Optional[Callable] = None):
        loss = None
        if closure is not None:
            with torch.enable_grad():
                loss = closure()
        if self._auto_hook_queue:
            from . import backward_hooks
            backward_hooks.flush_auto_queue(self)
        self._auto_flush_pending = False      # (a backward pass that raised never ran its end-of-pass callback)
        if getattr(self, "auto_pack", False):
            gather_packed_grads(self)

        grad_scale = getattr(self, "grad_scale", None)
        found_inf = getattr(self, "found_inf", None)
        if grad_scale is not None and not torch.is_tensor(grad_scale):      # plain numbers are accepted too
            grad_scale = torch.tensor(float(grad_scale), dtype=torch.float32)
        if found_inf is not None and not torch.is_tensor(found_inf):
            found_inf = torch.tensor(float(found_inf), dtype=torch.float32)
        if found_inf is not None and not _is_capturing() and float(found_inf) > 0:
            return loss
        self._has_stepped = True
        for group in self.param_groups:
            self._step_group(group, grad_scale, found_inf)
        return loss

    def _group_ctx(self) -> Dict[str, Any]:
        return {
            "has_16bit": any(isinstance(q, Tensor) and q.dtype in (torch.float16, torch.bfloat16)
                             for g in self.param_groups for q in g.get("params", [])),
            "peft": _detect_peft_context(self.param_groups),
        }

    def _step_group(self, group, grad_scale, found_inf, only: Optional[List[Tensor]] = None) -> None:
        """Step every parameter of ``group`` that has a gradient (or just those in ``only``)."""
        group["precision"] = _normalize_precision(group.get("precision", "compact"))
        params = [p for p in (group["params"] if only is None else only) if p.grad is not None]
        if not params:
            return
        ctx = None
        if group.get("differentiable", False):
            raise NotImplementedError("ApexW does not currently support differentiable=True.")
        if group["capturable"]:
            from . import rules as _rules
            for p in params:      # as torch.optim: device-resident step counters need an accelerator
                if p.device.type not in _rules.CAPTURABLE_SUPPORTED_DEVICES:
                    raise RuntimeError(f"capturable is not supported on {p.device.type}")
        for p in params:
            if p.grad.is_sparse:
                raise RuntimeError("ApexW does not support sparse gradients")
            st = self.state[p]
            if len(st) == 0 or (group["amsgrad"] and "max_exp_avg_sq" not in st) or \
                    (group["beta3"] is not None and "exp_avg_slow" not in st):
                if ctx is None:
                    ctx = self._group_ctx()
                self._init_state(p, group, ctx)
            if group.get("foreach") and torch.is_tensor(group["lr"]) and not group["capturable"]:
                raise RuntimeError("lr as a Tensor is not supported for capturable=False and foreach=True")

        grads, remaining_scale = self._prepare_grads([p.grad for p in params], group, grad_scale)
        inv_scale = None
        if remaining_scale is not None:
            inv_scale = remaining_scale.reciprocal()

        capturable = bool(group["capturable"])
        steps = [self.state[p]["step"] for p in params]
        _bump_steps(steps)

        plan = self._plan_for(group, params)        # capturable groups too: their kernels read step and lr on the device
        done: set = set()
        if plan is not None and plan.classes:
            try:
                self._run_native(plan, group, params, grads, remaining_scale, found_inf)
                done = {id(p) for _, ps in plan.classes for p in ps}
            except Exception as exc:
                # contract: a failed native launch leaves the step to the torch engine
                self._native_ok = False
                self._execution_plans = {}
                _debug(f"native step failed, falling back to the torch engine: {exc}")
                if params[0].is_cuda and not _native.disabled_by_env() and not os.environ.get("APEXW_B200_ALLOW_FALLBACK"):
                    _unbump_steps(steps)
                    raise

        scal_cache: Dict[Any, _eng.StepScalars] = {}
        for p, g in zip(params, grads):
            if id(p) in done:
                continue
            st = self.state[p]
            step_t = st["step"]
            if capturable or step_t.device.type != "cpu":
                key = ("t", id(step_t)) if capturable else float(step_t)
                step_val = step_t if capturable else float(step_t)
            else:
                key = step_val = float(step_t)
            sc = scal_cache.get(key)
            if sc is None:
                sc = _eng.make_scalars(group, step_val, self.seed)
                scal_cache[key] = sc
            inv = inv_scale
            if inv is not None and inv.device != p.device:
                inv = inv.to(p.device)
            _eng.update_tensor(p, g, st, group, sc, self._salt_of(p), inv, decay_mask=self._flat_decay_mask(p, group))

    def _flat_decay_ranges(self, p: Tensor, group: Dict[str, Any]) -> Optional[List[Tuple[int, int]]]:
        """Element ranges of a flat one-dimensional parameter that hold matrices (FSDP flat shards, the flat parameter
        of ``flatten_parameters``), or None when ``p`` is not such a parameter or decays as a whole anyway.

        ``decay_norm_only`` decides by ``p.dim()``, and a flat parameter is one-dimensional whatever it holds, so a
        plain rule would never decay it; both engines instead decay exactly these ranges inside the update (the
        kernels through a per-chunk side table of the launch plan, the torch engine through an element mask).  The
        ranges come from the flattening utility or from FSDP's own records and are cached per parameter and shard size."""
        if p.dim() != 1 or group["weight_decay"] == 0 or not group["decay_norm_only"] or torch.is_tensor(group["lr"]):
            return None
        own = getattr(p, "_apexw_decay_ranges", None)       # set by utils.flatten.flatten_parameters
        if own is not None:
            return [(int(a), int(b)) for a, b in own]
        if not hasattr(p, "_param_infos"):
            return None
        cache = self.__dict__.setdefault("_flat_decay_ranges_cache", {})
        key = (id(p), p.numel())
        if key not in cache:
            from ..parallel.fsdp import fsdp_decay_ranges, is_fsdp_flat_param
            cache[key] = fsdp_decay_ranges(p) if is_fsdp_flat_param(p) else []
            if cache[key] is None:
                warnings.warn("ApexW: cannot locate this rank's part of an FSDP flat parameter; its matrices get no "
                              "weight decay under decay_norm_only=True (use adamw_compat=True to decay everything)",
                              UserWarning, stacklevel=3)
        found = cache[key]
        return [(int(a), int(b)) for a, b in found] if found else None

    def _flat_decay_mask(self, p: Tensor, group: Dict[str, Any]) -> Optional[Tensor]:
        """The same ranges as a boolean element mask (torch engine)."""
        ranges = self._flat_decay_ranges(p, group)
        if not ranges:
            return None
        cache = self.__dict__.setdefault("_flat_decay_mask_cache", {})
        key = (id(p), p.numel(), p.device)
        mask = cache.get(key)
        if mask is None:
            mask = torch.zeros(p.numel(), dtype=torch.bool, device=p.device)
            for a, b in ranges:
                mask[a:b] = True
            cache[key] = mask
        return mask

    # ------------------------------------------------------------------ native plan

    def _native_eligible(self, p: Tensor, st: Dict[str, Any], group: Dict[str, Any]) -> Optional[int]:
        """Return the kernel class for ``p`` or None when the torch engine must take it."""
        floats = (torch.float32, torch.bfloat16, torch.float16)
        if not p.is_cuda or not p.is_contiguous() or p.dtype not in floats:
            return None
        if st.get("is_6bit_m", False):
            return None
        exotic = bool(group["lion"]) or bool(group["amsgrad"]) or group["beta3"] is not None
        lion8 = (bool(group["lion"]) and (st.get("is_8bit", False) or st.get("is_ultra", False)) and not group["cautious"]
                 and not group["nesterov"] and st.get("exp_avg") is not None and st["exp_avg"].dtype == torch.int8
                 and "exp_avg_scales" in st and not st.get("is_4bit_m", False))
        if exotic and not lion8 and (st.get("is_8bit", False) or st.get("is_ultra", False) or st.get("is_quad_v", False)
                                     or group["cautious"]):
            return None       # AMSGrad / AdEMAMix run on the kernel's dense general path only; Lion also on int8 momentum
        if group["nesterov"] and group["cautious"]:
            return None
        g = p.grad
        if g is None or g.dtype not in floats or not g.is_contiguous() or g.device != p.device:
            return None
        lr = group["lr"]
        if torch.is_tensor(lr) and (lr.numel() != 1 or (lr.is_cuda and (lr.device != p.device or lr.dtype != torch.float32))):
            return None       # a learning rate on this device is read by the kernels; anything else goes to the torch engine
        step_t = st.get("step")
        on_device = torch.is_tensor(step_t) and step_t.is_cuda
        if on_device and (step_t.device != p.device or step_t.dtype != torch.float32):
            return None
        if (on_device or (torch.is_tensor(lr) and lr.is_cuda)) and st.get("exp_avg_sq") is not None \
                and st["exp_avg_sq"].dtype == torch.float16 and "scale_v" in st:
            return None       # the fp16 rescaling schedule is driven by the step count on the host
        if group["capturable"] and not on_device:
            return None
        if lion8:
            bs = st.get("block_size_8bit", st.get("ultra_block_size", 0))
            return _KC_LION8 if (64 <= bs <= 2048 and not (bs & (bs - 1))) else None
        if st.get("is_factored_v", False):     # row / column statistics; first moment dense or int8 with block scales
            if torch.are_deterministic_algorithms_enabled():
                return None       # the statistics kernel adds with fp32 atomics: sums vary in their last bits run to run
            r, c, m = st.get("exp_avg_sq_row"), st.get("exp_avg_sq_col"), st.get("exp_avg")
            if (exotic or group["cautious"] or r is None or c is None or m is None or r.dtype != torch.float32
                    or c.dtype != torch.float32 or r.numel() * c.numel() != p.numel()):
                return None
            if m.dtype == torch.int8:
                bs = st.get("block_size_8bit", 0)
                if "exp_avg_scales" not in st or bs < 64 or bs > 2048 or (bs & (bs - 1)):
                    return None
            elif m.dtype not in floats:
                return None
            return _KC_FACTORED
        if st.get("is_8bit", False):
            bs = st["block_size_8bit"]
            if bs < 64 or bs > 2048 or (bs & (bs - 1)):
                return None
            if st.get("is_4bit_m", False):
                if p.numel() % 4:
                    return None
                return _KC_NF4_QUAD if st.get("is_quad_v", False) else _KC_NF4
            return _KC_INT8
        if st.get("is_ultra", False):      # int8 first moment with block scales + a dense second moment per element
            bs = st.get("ultra_block_size", 0)
            m, v = st.get("exp_avg"), st.get("exp_avg_sq")
            if (group["cautious"] or bs < 64 or bs > 2048 or (bs & (bs - 1)) or m is None or m.dtype != torch.int8
                    or "exp_avg_scales" not in st or v is None or v.dtype not in floats or v.numel() != p.numel()):
                return None
            return _KC_ULTRA
        # (dense cautious runs as two launches: a count of what each tensor keeps, then the update)
        m, v = st.get("exp_avg"), st.get("exp_avg_sq")
        if group["lion"]:
            return _KC_DENSE if (m is not None and m.dtype in floats) else None
        if m is None or v is None or m.dtype not in floats or v.dtype not in floats:
            return None
        if group["beta3"] is not None and (st.get("exp_avg_slow") is None or st["exp_avg_slow"].dtype != m.dtype):
            return None
        if group["amsgrad"] and (st.get("max_exp_avg_sq") is None or st["max_exp_avg_sq"].dtype != v.dtype
                                 or v.dtype == torch.float16):
            return None       # a rescaled fp16 v would need its maximum rescaled with it: the torch engine's job
        if float(st.get("scale_v", 1.0)) != 1.0 and v.dtype != torch.float16:
            return None       # only fp16 second moments carry a scale (4^k, k <= 8: the kernel takes the exponent)
        return _KC_DENSE_QUAD if st.get("is_quad_v", False) else _KC_DENSE

    def _plan_for(self, group, params: List[Tensor]) -> Optional[_GroupPlan]:
        if not self._native_ok or not params[0].is_cuda:
            return None
        if _native.disabled_by_env():
            return None
        native = _native.require()   # CUDA tensors without the library: fail loudly
        ids = tuple(id(p) for p in params)
        plan_key = (id(group), ids) if len(ids) < len(group["params"]) else id(group)
        # What a cached plan froze: where each parameter's data lives, its dtype, and which parameters share a step
        # count (one launch applies one bias correction).  ``model.to()``, ``.bfloat16()``, ``flatten_parameters`` or
        # a wrapper that re-homes ``p.data`` moves the first two; a parameter that sat out some steps (gradient None)
        # and comes back moves the third.  Any of them makes the plan stale, so it is rebuilt.
        step0 = self.state[params[0]]["step"]
        host_steps = step0.device.type == "cpu"
        base = float(step0) if host_steps else 0.0
        signature = tuple((p.data_ptr(), p.dtype, (float(self.state[p]["step"]) - base) if host_steps else 0.0)
                          for p in params)
        # options that decide the kernel class or which extra state tensors a plan carries (they can be switched on
        # after the first step: the extra buffers are then created late and the plan must be rebuilt around them)
        signature += ((bool(group["lion"]), bool(group["amsgrad"]), group["beta3"] is not None, bool(group["cautious"]),
                       bool(group["nesterov"]), bool(group["capturable"]), torch.is_tensor(group["lr"])),)
        plan = self._execution_plans.get(plan_key)
        if plan is not None and plan.param_ids == ids and plan.signature == signature:
            self._execution_plans[plan_key] = self._execution_plans.pop(plan_key)      # most recently used goes last
            return plan
        self._execution_plans.pop(plan_key, None)                     # stale: rebuilt below
        while len(self._execution_plans) >= _MAX_CACHED_PLANS:        # sub-sets of a group each get a key: keep it bounded
            self._execution_plans.pop(next(iter(self._execution_plans)))
        plan = _GroupPlan()
        plan.param_ids = ids
        plan.signature = signature
        buckets: Dict[Tuple[int, int, float], List[Tensor]] = defaultdict(list)
        for p in params:
            st = self.state[p]
            kc = self._native_eligible(p, st, group)
            if kc is None:
                plan.fallback.append(p)
            else:
                # device-resident counters of a capturable group cannot be read without a sync: they are taken to agree
                same = 0.0 if (group["capturable"] and st["step"].is_cuda) else float(st["step"])
                int8_m = kc == _KC_FACTORED and st["exp_avg"].dtype == torch.int8      # one first-moment kind per launch
                buckets[(kc, p.device.index, same, int8_m)].append(p)
        for (kc, _dev, _step, int8_m), ps in buckets.items():
            ms = [self.state[p]["exp_avg"] for p in ps]
            quant = _KC_INT8 <= kc <= _KC_NF4_QUAD
            if kc == _KC_FACTORED:
                vs = [self.state[p]["exp_avg_sq_row"] for p in ps]
                vsc = [self.state[p]["exp_avg_sq_col"] for p in ps]
                msc = [self.state[p]["exp_avg_scales"].view(-1) for p in ps] if int8_m else []
            else:
                vs = [self.state[p]["exp_avg"] if group["lion"] else self.state[p]["exp_avg_sq"] for p in ps]   # Lion keeps no v
                msc = [self.state[p]["exp_avg_scales"].view(-1) for p in ps] if (quant or kc in (_KC_ULTRA, _KC_LION8)) else []
                vsc = [self.state[p]["exp_avg_sq_scales"].view(-1) for p in ps] if quant else []
            if not quant and group["beta3"] is not None and not group["lion"]:
                msc = [self.state[p]["exp_avg_slow"] for p in ps]          # dense plans carry the slow moments ...
            if not quant and group["amsgrad"] and not group["lion"]:
                vsc = [self.state[p]["max_exp_avg_sq"] for p in ps]        # ... and AMSGrad's running maxima in these slots
            decay_all = group["weight_decay"] != 0
            flags = []
            for p in ps:
                f = 0
                if decay_all and (not group["decay_norm_only"] or p.dim() >= 2):
                    f |= _SEG_DECAY
                if kc in (_KC_DENSE_QUAD, _KC_NF4_QUAD):
                    f |= _SEG_QUAD
                flags.append(f)
            salts = [self._salt_of(p) for p in ps]
            bss = [int(self.state[p].get("block_size_8bit", self.state[p].get("ultra_block_size", 0))) for p in ps]
            # flat parameters (FSDP shards, flattened models): decay the matrices inside them, chunk by chunk, in the kernel
            partial = [self._flat_decay_ranges(p, group) or [] for p in ps]
            ranges = [[x for ab in r for x in ab] for r in partial] if any(partial) else []
            if os.environ.get("APEXW_B200_DEBUG", "0") not in ("", "0"):
                # (Lion keeps no second moment: its plans repeat the first moment in that slot)
                assert_disjoint_write_sets([p.data for p in ps] + ms + ([] if group["lion"] else vs) + msc + vsc)
            sp = native.StatePlan(kc, [p.data for p in ps], ms, vs, msc, vsc, flags, salts, bss, [], -1, ranges)
            plan.classes.append((sp, ps))
        self._execution_plans[plan_key] = plan
        return plan

    def _run_native(self, plan: _GroupPlan, group, params, grads, grad_scale, found_inf) -> None:
        grad_of = {id(p): g for p, g in zip(params, grads)}
        flags = 0
        if group.get("stochastic_rounding", True):
            flags |= _STEP_STOCHASTIC
        if group["nesterov"]:
            flags |= _STEP_NESTEROV
        if group["cautious"]:
            flags |= _STEP_CAUTIOUS
        if group["maximize"]:
            flags |= _STEP_MAXIMIZE
        if group["lion"]:
            flags |= _STEP_LION
        else:
            if group["beta3"] is not None:
                flags |= _STEP_SLOW
            if group["amsgrad"]:
                flags |= _STEP_AMSGRAD
        lr = group["lr"]
        lr_dev = lr.reshape(()) if (torch.is_tensor(lr) and lr.is_cuda) else None
        for sp, ps in plan.classes:
            step_t = self.state[ps[0]]["step"]
            step_dev = step_t if (step_t.is_cuda and (group["capturable"] or lr_dev is not None or _is_capturing())) else None
            if step_dev is not None or lr_dev is not None:
                # what depends on the step count or the learning rate is derived on the device (no host read, so the
                # step can be captured in a CUDA graph); the host passes the constants and placeholders for the rest
                host_step = 1.0 if step_dev is not None else float(step_t)
                host_lr = 0.0 if lr_dev is not None else float(lr)
                sc = _eng.make_scalars(dict(group, lr=host_lr), host_step, self.seed)
                sp.set_device_scalars(step_dev, lr_dev, host_step, host_lr, float(group["alpha"]),
                                      float(group["weight_decay"]), int(self.seed) & 0xFFFFFFFF)
                plan.dynamic = True
            else:
                if getattr(plan, "dynamic", False):
                    sp.clear_device_scalars()
                sc = _eng.make_scalars(dict(group, lr=float(lr)) if torch.is_tensor(lr) else group, float(step_t), self.seed)
            gs = grad_scale.to(ps[0].device, torch.float32) if grad_scale is not None else None
            fi = found_inf.to(ps[0].device, torch.float32) if (found_inf is not None and _is_capturing()) else None
            if not group["lion"] and any("exp_avg_sq" in self.state[p] and self.state[p]["exp_avg_sq"].dtype == torch.float16
                                         and "scale_v" in self.state[p] for p in ps):
                # fp16 second moments: the per-tensor scale is re-centred on the host every 100 steps (as in the torch
                # engine) and reaches the kernel as an exponent in the segment table
                ks = []
                for p in ps:
                    st = self.state[p]
                    k = 0
                    if st["exp_avg_sq"].dtype == torch.float16 and "scale_v" in st:
                        scale_v, _ = _eng._recalibrate_fp16_v(st, st["exp_avg_sq"], sc, group)
                        k = int(round(math.log(scale_v, 4.0))) if scale_v > 1.0 else 0
                    ks.append(k)
                sp.set_v_scale_log4(ks)
            with _native.nvtx_range("apexw_b200.fused_state"):
                sp.step([grad_of[id(p)] for p in ps], sc.beta1, sc.beta2, sc.step_size, sc.eps_scaled, sc.eps,
                        sc.eps_quad, sc.eps_quad_scaled, sc.decay_factor, 1.0,
                        1.0 + _eng.GAIN_ALIGNED * sc.beta1, 1.0 - _eng.GAIN_OPPOSED * sc.beta1,
                        sc.key, flags, fi, gs, 0, float(sc.beta3 or 0.0), float(sc.slow_ratio or 0.0), float(sc.lr))
            self._native_launches += 1
            # kernels behind this call: the update, plus the scalar kernel of the device-resident mode, the counting
            # pass of a dense cautious step, the two statistics kernels of the factored layout
            kc = getattr(sp, "kernel_class", None)
            _native.count(1 + (1 if (step_dev is not None or lr_dev is not None) else 0)
                          + (1 if (group["cautious"] and kc in (_KC_DENSE, _KC_DENSE_QUAD)) else 0)
                          + (2 if kc == _KC_FACTORED else 0))
        if _table_check.enabled() and not _is_capturing():
            _table_check.check()        # debug mode: one device synchronisation per step


_UNTRACED_STEP = None


def _untraced_step():
    """``ApexW._step_impl`` wrapped so that ``torch.compile(opt.step)`` runs it eagerly (the step is hand-written kernels
    and host-side planning, not a graph to trace).  Built on first use: importing the tracer costs seconds, and only
    programs that already imported it get here."""
    global _UNTRACED_STEP
    if _UNTRACED_STEP is None:
        import torch._dynamo
        _UNTRACED_STEP = torch._dynamo.disable(ApexW._step_impl)
    return _UNTRACED_STEP


def assert_disjoint_write_sets(tensors) -> None:
    """Host-side race check of a launch plan: no two tensors that one launch writes may overlap in memory
    (every chunk of every segment is written by exactly one thread block, so disjoint tensors mean disjoint
    write sets).  Enabled with ``APEXW_B200_DEBUG=1`` when plans are built; raises ``RuntimeError``."""
    spans = sorted((t.data_ptr(), t.data_ptr() + t.numel() * t.element_size(), i)
                   for i, t in enumerate(tensors) if t.numel() > 0)
    for (a0, a1, i), (b0, b1, j) in zip(spans, spans[1:]):
        if b0 < a1:
            raise RuntimeError(f"launch plan writes overlapping memory: tensor {i} [{a0:#x}, {a1:#x}) and tensor {j} "
                               f"[{b0:#x}, {b1:#x})")


def _is_capturing() -> bool:
    return torch.cuda.is_available() and torch.cuda.is_current_stream_capturing()


def _bump_steps(steps: List[Tensor]) -> None:
    cpu = [s for s in steps if s.device.type == "cpu"]
    dev = [s for s in steps if s.device.type != "cpu"]
    if cpu:
        torch._foreach_add_(cpu, 1.0)
    if dev:
        torch._foreach_add_(dev, 1)


def _unbump_steps(steps: List[Tensor]) -> None:
    for s in steps:
        s.sub_(1)


def build_llm_param_groups(model: nn.Module, weight_decay: float = 0.1, no_decay_embeddings: bool = False):
    """Two groups for LLM training: ``decayed`` (matrices) and ``non_decayed`` (1-D tensors,
    norms, biases and, on request, embeddings).  Always returns both groups, in that order
    (reference: apexw/optimizer.py:5890-5920)."""
    groups = {"decayed": [], "non_decayed": []}
    for name, p in model.named_parameters():
        if not p.requires_grad:
            continue
        lname = name.lower()
        skip = p.ndim < 2 or name.endswith(".bias") or "norm" in lname
        if not skip and no_decay_embeddings:
            skip = "embed" in lname or "wte" in lname
        groups["non_decayed" if skip else "decayed"].append(p)
    return [
        {"params": groups["decayed"], "weight_decay": weight_decay, "group_name": "decayed"},
        {"params": groups["non_decayed"], "weight_decay": 0.0, "group_name": "non_decayed"},
    ]
