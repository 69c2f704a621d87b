"""Per-tensor update engine in plain torch ops.

This is both the any-device implementation of every mode of the optimizer and
the oracle the fused sm_100a kernels are tested against.  For the modes the
kernels implement (dense 16/32-bit moments with optional shared-by-four
variance; NF4/int8 momentum with log-uint8 variance) the arithmetic below is
written operation by operation in the same order as ``csrc/fused_state.cu``,
in fp32 without fused multiply-adds, and draws its rounding bits from the same
counter-based generator (``ops/rng.py``), so with or without stochastic
rounding the two paths agree bit for bit except where device ``log2f`` differs
from the host's in the last place.

Mathematical content follows the reference (apexw/optimizer.py:4313-4735 for the
quantised modes, :5297-5887 for the dense ones, apexw/csrc/apexw_cuda_kernel.cu
for which stores are stochastically rounded).
"""

from __future__ import annotations

import math
import struct
from dataclasses import dataclass
from typing import Any, Dict, Optional, Union

import torch
from torch import Tensor

from ..ops import formats as F
from ..ops import rng

Scalar = Union[float, Tensor]

GAIN_ALIGNED = 0.20   # lookahead gain when momentum and gradient agree: 1 + 0.20*beta1
GAIN_OPPOSED = 0.35   # ... and when they disagree: 1 - 0.35*beta1
QUAD_EPS_SWITCH = 1e-6
QUAD_EPS_VALUE = 1e-8


@dataclass
class StepScalars:
    """Per-(group, step) scalars; floats on the normal path, 0-dim tensors when capturable."""
    step: Scalar
    lr: Scalar
    beta1: float
    beta2: float
    beta3: Optional[float]
    alpha: float
    eps: float
    bc1: Scalar
    bc2_sqrt: Scalar
    step_size: Scalar          # lr * sqrt(bc2) / bc1
    eps_scaled: Scalar         # eps * sqrt(bc2)
    eps_quad: float            # eps used by the shared-variance 8-bit path
    eps_quad_scaled: Scalar
    slow_ratio: Scalar         # alpha * bc1 / bc3 (AdEMAMix)
    decay_factor: Scalar       # max(1 - lr*wd, 0)
    weight_decay: float
    key: Optional[int]         # rng step key; None -> torch's generator


def make_scalars(group: Dict[str, Any], step: Scalar, seed: int) -> StepScalars:
    lr = group["lr"]
    beta1, beta2 = group["betas"]
    beta3 = group["beta3"]
    eps = group["eps"]
    wd = group["weight_decay"]
    tensor_mode = isinstance(step, Tensor)
    if tensor_mode:
        stepf = step.to(torch.float32)
        bc1 = 1.0 - beta1 ** stepf
        bc2_sqrt = (1.0 - beta2 ** stepf).sqrt()
        step_size = lr * bc2_sqrt / bc1
        slow = group["alpha"] * (bc1 / (1.0 - beta3 ** stepf)) if beta3 is not None else 0.0
        key = None
    else:
        bc1 = 1.0 - beta1 ** step
        bc2_sqrt = math.sqrt(1.0 - beta2 ** step)
        step_size = lr * bc2_sqrt / bc1
        slow = group["alpha"] * (bc1 / (1.0 - beta3 ** step)) if beta3 is not None else 0.0
        key = rng.step_key(seed, int(step))
    eps_q = QUAD_EPS_VALUE if eps > QUAD_EPS_SWITCH else eps
    if isinstance(lr, Tensor):
        decay = (1.0 - lr * wd).clamp_min(0.0)
    else:
        decay = max(1.0 - lr * wd, 0.0)
    return StepScalars(step=step, lr=lr, beta1=beta1, beta2=beta2, beta3=beta3, alpha=group["alpha"], eps=eps,
                       bc1=bc1, bc2_sqrt=bc2_sqrt, step_size=step_size, eps_scaled=eps * bc2_sqrt,
                       eps_quad=eps_q, eps_quad_scaled=eps_q * bc2_sqrt, slow_ratio=slow,
                       decay_factor=decay, weight_decay=wd, key=key)


class _Bits:
    """Lazily produced rounding bits for one tensor."""

    def __init__(self, numel: int, device, key: Optional[int], salt: int, enabled: bool):
        self.numel, self.device, self.enabled = numel, device, enabled
        self._seg = rng.segment_key(key, salt) if key is not None else None
        self._w = None
        self._w2 = None

    def _words(self) -> Tensor:
        if self._w is None:
            if self._seg is None:
                self._w = torch.randint(0, 2 ** 32, (self.numel,), dtype=torch.int64, device=self.device)
            else:
                self._w = rng.element_words(self.numel, self._seg, device=self.device)
        return self._w

    def param(self) -> Optional[Tensor]:
        return rng.u16_low(self._words()) if self.enabled else None

    def moment1(self) -> Optional[Tensor]:
        return rng.u16_high(self._words()) if self.enabled else None

    def moment2(self, shared_by_four: bool) -> Optional[Tensor]:
        if not self.enabled:
            return None
        if self._w2 is None:
            w = self._words()
            self._w2 = rng.second_words(w[::4] if shared_by_four else w)
        return rng.u16_low(self._w2)


def _sanitize(g: Tensor) -> Tensor:
    return torch.nan_to_num(g, nan=0.0, posinf=65504.0, neginf=-65504.0)


def _f32(x: float) -> float:
    """Round a Python float to float32 (what a kernel argument of type float holds)."""
    return struct.unpack("f", struct.pack("f", float(x)))[0]


def _fma(a: Tensor, b, c: Tensor) -> Tensor:
    """fused multiply-add with a single rounding, emulated through float64 for float32 inputs."""
    if a.dtype != torch.float32:
        return a * b + c
    bb = b.double() if isinstance(b, Tensor) else _f32(b)
    return (a.double() * bb + c.double()).float()


def _lerp_to(m: Tensor, g: Tensor, beta: Scalar) -> Tensor:
    """fma(m, beta, g*(1-beta)): the kernels' order."""
    return _fma(m, beta, g * (1.0 - beta))


def _sum_sq4(g: Tensor) -> Tensor:
    """Sum of squares over consecutive groups of four, accumulated left to right with fma."""
    g4 = g.reshape(-1, 4)
    acc = g4[:, 0] * g4[:, 0]
    for j in (1, 2, 3):
        acc = _fma(g4[:, j], g4[:, j], acc)
    return acc


def _store_param(p: Tensor, new_f32: Tensor, bits: _Bits) -> None:
    if p.dtype in (torch.bfloat16, torch.float16):
        F.store_rounded(p, new_f32, bits.param())
    else:
        p.copy_(new_f32.reshape(p.shape))


def _cautious(num: Tensor, g: Tensor, group_size: Optional[int] = None) -> Tensor:
    """Zero components that oppose the gradient, renormalised by the kept fraction.

    ``group_size`` None: one mean over the tensor.  Otherwise one mean per
    consecutive ``group_size`` elements (the quantisation block), as the fused
    8-bit kernel does.
    """
    mask = (num * g >= 0).to(num.dtype)
    if group_size is None:
        return num * (mask / mask.mean().clamp(min=1e-3))
    flat = mask.reshape(-1)
    n = flat.numel()
    blocks, _ = F.as_blocks(flat, group_size)
    counts = torch.full((blocks.shape[0], 1), float(group_size), device=num.device)
    tail = n % group_size
    if tail:
        counts[-1, 0] = float(tail)
    mean = (blocks.sum(dim=1, keepdim=True) / counts).clamp(min=1e-3)
    scale = (blocks / mean).reshape(-1)[:n].reshape(num.shape)
    return num * scale


# ---------------------------------------------------------------------------
# the update
# ---------------------------------------------------------------------------

@torch.no_grad()
def update_tensor(p: Tensor, grad: Tensor, st: Dict[str, Any], group: Dict[str, Any], sc: StepScalars,
                  salt: int, inv_scale: Optional[Scalar] = None, decay_mask: Optional[Tensor] = None) -> None:
    """Apply one optimizer step to ``p`` in place given its state dict ``st``.  ``decay_mask`` (flat boolean, one entry
    per element): the decoupled weight decay applies to exactly these elements, whatever the parameter's rank - the
    matrices inside a flat parameter - instead of to the whole tensor or to none of it."""
    if torch.is_complex(p):
        _update_complex(p, grad, st, group, sc, salt, inv_scale)
        return

    work = torch.float64 if p.dtype == torch.float64 else torch.float32
    g = grad.detach().to(work)
    if g.shape != p.shape:
        g = g.reshape(p.shape)
    g = _sanitize(g)
    if group["maximize"]:
        g = -g
    if inv_scale is not None:
        g = g * inv_scale

    stochastic = bool(st.get("stochastic_rounding", group.get("stochastic_rounding", True)))
    bits = _Bits(p.numel(), p.device, sc.key, salt, stochastic)
    decay = group["weight_decay"] != 0 and (not group["decay_norm_only"] or p.dim() >= 2)
    pf = p.detach().to(work)
    if decay_mask is not None:
        pf = torch.where(decay_mask.reshape(p.shape), pf * sc.decay_factor, pf)
    elif decay:
        pf = pf * sc.decay_factor

    if group["lion"]:
        _lion(p, pf, g, st, sc, bits)
    elif st.get("is_factored_v", False):
        _factored(p, pf, g, st, group, sc, bits)
    elif st.get("is_8bit", False):
        _eight_bit(p, pf, g, st, group, sc, bits)
    elif st.get("is_ultra", False):
        _ultra(p, pf, g, st, group, sc, bits)
    else:
        _dense(p, pf, g, st, group, sc, bits)


def _update_complex(p, grad, st, group, sc, salt, inv_scale):
    real_state = dict(st)
    for k in ("exp_avg", "exp_avg_sq", "exp_avg_slow", "max_exp_avg_sq"):
        if k in st and torch.is_tensor(st[k]) and torch.is_complex(st[k]):
            real_state[k] = torch.view_as_real(st[k])
    update_tensor(torch.view_as_real(p), torch.view_as_real(grad.to(p.dtype)), real_state, group, sc, salt, inv_scale)
    for k in ("scale_v", "sqrt_scale_v"):
        if k in real_state:
            st[k] = real_state[k]


# -- first-moment storage ----------------------------------------------------

def _m_block(st) -> int:
    return st.get("block_size_8bit", st.get("ultra_block_size", 256))


def _load_m(st, key: str, shape, quantised: bool) -> Tensor:
    buf = st[key]
    if not quantised:
        return buf.to(torch.float64 if buf.dtype == torch.float64 else torch.float32)
    bs = _m_block(st)
    sc = st[key + "_scales"]
    if key == "exp_avg" and st.get("is_6bit_m", False):
        n = math.prod(shape)
        return F._dequantize_blockwise_6bit(buf, sc, numel=n, block_size=bs).view(shape)
    if key == "exp_avg" and st.get("is_4bit_m", False):
        n = st.get("m_numel", math.prod(shape))
        return F._dequantize_blockwise_int4(buf, sc, numel=n, block_size=bs).view(shape)
    return F._dequantize_blockwise_int8(buf, sc, block_size=bs)


def _store_m(st, key: str, m: Tensor, quantised: bool, bits16: Optional[Tensor], ema: bool = True) -> None:
    buf = st[key]
    if not quantised:
        if buf.dtype in (torch.bfloat16, torch.float16):
            F.store_rounded(buf, m.to(torch.float32), bits16)
        else:
            buf.copy_(m.reshape(buf.shape))
        return
    bs = _m_block(st)
    sc = st[key + "_scales"]
    old = sc if ema else None
    stoch = bits16 is not None
    if key == "exp_avg" and st.get("is_6bit_m", False):
        F._quantize_blockwise_6bit(m, bs, stoch, out_q=buf, out_scales=sc, old_scales=old, bits16=bits16)
    elif key == "exp_avg" and st.get("is_4bit_m", False):
        F._quantize_blockwise_int4(m, bs, stoch, out_q=buf, out_scales=sc, old_scales=old, bits16=bits16)
    else:
        F._quantize_blockwise_int8(m, bs, stoch, out_q=buf, out_scales=sc, old_scales=old, bits16=bits16)


# -- modes -------------------------------------------------------------------

def _lion(p, pf, g, st, sc, bits):
    quant = bool(st.get("is_8bit", False) or st.get("is_ultra", False))
    m = _load_m(st, "exp_avg", p.shape, quant)
    update = _lerp_to(m, g, sc.beta1).sign()
    _store_param(p, pf - update * sc.lr, bits)
    m = _lerp_to(m, g, sc.beta2)
    _store_m(st, "exp_avg", m, quant, bits.moment1(), ema=False)


def _numerator(m, m_slow, g, group, sc, lookahead: bool):
    """Pick the update direction: AdEMAMix mix, Nesterov, lookahead with gain, or plain m."""
    if m_slow is not None:
        return m + m_slow * sc.slow_ratio
    if group["nesterov"]:
        return _lerp_to(m, g, sc.beta1)
    if lookahead and not group["cautious"]:
        look = _lerp_to(m, g, sc.beta1)
        gain_hi = 1.0 + GAIN_ALIGNED * sc.beta1
        gain_lo = 1.0 - GAIN_OPPOSED * sc.beta1
        gain = torch.where(m * g >= 0, torch.full_like(m, gain_hi), torch.full_like(m, gain_lo))
        return look * gain
    return m


def _dense(p, pf, g, st, group, sc, bits):
    """fp32 / 16-bit moments, optionally one variance per four elements."""
    m_buf = st["exp_avg"]
    v_buf = st["exp_avg_sq"]
    quad = bool(st.get("is_quad_v", False))
    work = pf.dtype
    scale_v = float(st.get("scale_v", 1.0))
    sqrt_scale_v = float(st.get("sqrt_scale_v", 1.0))

    m = _lerp_to(m_buf.to(work), g, sc.beta1)
    m_slow = None
    if sc.beta3 is not None:
        m_slow = _lerp_to(st["exp_avg_slow"].to(work), g, sc.beta3)

    if v_buf.dtype == torch.float16 and "scale_v" in st:
        scale_v, sqrt_scale_v = _recalibrate_fp16_v(st, v_buf, sc, group)

    omb2 = 1.0 - sc.beta2
    if quad:
        v = _fma(v_buf.to(work).reshape(-1), sc.beta2, _sum_sq4(g) * (0.25 * omb2 * scale_v))
        v = torch.where(torch.isfinite(v), v, torch.zeros_like(v))
    else:
        v = _fma(v_buf.to(work), sc.beta2, (g * g) * (omb2 * scale_v))

    v_used = v
    if group["amsgrad"]:
        mx = st["max_exp_avg_sq"]
        mxf = torch.maximum(mx.to(work).reshape(v.shape), v)
        mx.copy_(mxf.reshape(mx.shape))
        v_used = mxf

    root = v_used.clamp_min(0).sqrt()
    if sqrt_scale_v != 1.0:
        root = root / sqrt_scale_v
    denom = root + sc.eps_scaled     # exactly AdamW's sqrt(v)/sqrt(bc2) + eps, times sqrt(bc2)
    inv = denom.reciprocal() * sc.step_size   # reciprocal then scale: the kernels' order
    if quad:
        inv = inv.unsqueeze(1).expand(-1, 4).reshape(p.shape)

    num = _numerator(m, m_slow, g, group, sc, lookahead=False)
    if group["cautious"]:
        num = _cautious(num, g)
    _store_param(p, _fma(-num, inv, pf), bits)

    _store_m(st, "exp_avg", m, False, bits.moment1())
    if m_slow is not None:
        _store_m(st, "exp_avg_slow", m_slow, False, bits.moment1())
    if v_buf.dtype in (torch.bfloat16, torch.float16):
        F.store_rounded(v_buf, v.to(torch.float32), bits.moment2(quad))
    else:
        v_buf.copy_(v.reshape(v_buf.shape))


def _recalibrate_fp16_v(st, v_buf, sc, group):
    """fp16 second moments carry a per-tensor scale, re-centred every 100 steps."""
    scale_v = float(st.get("scale_v", 1.0))
    if (group.get("dynamic_scaling", True) and not isinstance(sc.step, Tensor)
            and int(sc.step) > 1 and int(sc.step) % 100 == 0 and v_buf.numel() > 0):
        vmax = float(v_buf.max())
        factor = None
        if vmax < 0.25 and scale_v < 65536.0:
            factor = 4.0
        elif vmax > 16384.0 and scale_v > 1.0:
            factor = 0.25
        if factor is not None:
            v_buf.mul_(factor)
            scale_v *= factor
            st["scale_v"] = scale_v
            st["sqrt_scale_v"] = math.sqrt(scale_v)
    return scale_v, float(st.get("sqrt_scale_v", math.sqrt(scale_v)))


def _eight_bit(p, pf, g, st, group, sc, bits):
    """NF4 or int8 first moment, log-uint8 second moment (per element or per four)."""
    bs = st["block_size_8bit"]
    n = p.numel()
    quad = bool(st.get("is_quad_v", False))
    m = _lerp_to(_load_m(st, "exp_avg", p.shape, True), g, sc.beta1)
    m_slow = None
    if sc.beta3 is not None and "exp_avg_slow_scales" in st:
        m_slow = _lerp_to(_load_m(st, "exp_avg_slow", p.shape, True), g, sc.beta3)

    v_q = st["exp_avg_sq"]
    v_sc = st["exp_avg_sq_scales"]
    omb2 = 1.0 - sc.beta2
    if quad:
        v_bs = max(1, bs // 4)
        v = F._dequantize_blockwise_uint8(v_q, v_sc, block_size=v_bs)
        v = _fma(v, sc.beta2, _sum_sq4(g) * (0.25 * omb2))
        v = torch.where(torch.isfinite(v), v, torch.zeros_like(v))
        eps_floor, eps_add = sc.eps_quad, sc.eps_quad_scaled
    else:
        v_bs = bs
        v = F._dequantize_blockwise_uint8(v_q, v_sc, block_size=bs)
        v = _fma(v, sc.beta2, (g * g) * omb2)
        v = torch.where(torch.isfinite(v), v, torch.zeros_like(v))
        eps_floor, eps_add = sc.eps, sc.eps_scaled

    v_used = v
    if group["amsgrad"] and not quad:
        mx = st["max_exp_avg_sq"]
        torch.maximum(mx, v.reshape(mx.shape), out=mx)
        v_used = mx.reshape(v.shape)

    denom = torch.maximum(v_used.clamp_min(0).sqrt() + eps_add,
                          torch.as_tensor(eps_floor, dtype=torch.float32, device=v.device))
    inv = denom.reciprocal() * sc.step_size   # reciprocal then scale: the kernels' order
    if quad:
        inv = inv.unsqueeze(1).expand(-1, 4).reshape(p.shape)

    num = _numerator(m, m_slow, g, group, sc, lookahead=True)
    if group["cautious"]:
        num = _cautious(num, g, group_size=bs)
    _store_param(p, _fma(-num, inv, pf), bits)

    _store_m(st, "exp_avg", m, True, bits.moment1())
    if m_slow is not None:
        _store_m(st, "exp_avg_slow", m_slow, True, bits.moment1())
    F._quantize_blockwise_uint8(v, v_bs, stochastic=bits.enabled, out_q=v_q, out_scales=v_sc,
                                old_scales=v_sc, bits16=bits.moment2(quad))


def _ultra(p, pf, g, st, group, sc, bits):
    """int8 first moment + 16/32-bit second moment."""
    m = _lerp_to(_load_m(st, "exp_avg", p.shape, True), g, sc.beta1)
    m_slow = None
    if sc.beta3 is not None and "exp_avg_slow_scales" in st:
        m_slow = _lerp_to(_load_m(st, "exp_avg_slow", p.shape, True), g, sc.beta3)
    v_buf = st["exp_avg_sq"]
    v = v_buf.float() * sc.beta2 + (g * g) * (1.0 - sc.beta2)
    v_used = v
    if group["amsgrad"]:
        mx = st["max_exp_avg_sq"]
        mxf = torch.maximum(mx.float(), v)
        mx.copy_(mxf)
        v_used = mxf
    denom = v_used.clamp_min(0).sqrt() + sc.eps_scaled
    num = _numerator(m, m_slow, g, group, sc, lookahead=False)
    if group["cautious"]:
        num = _cautious(num, g)
    _store_param(p, pf - num * (denom.reciprocal() * sc.step_size), bits)
    _store_m(st, "exp_avg", m, True, bits.moment1())
    if m_slow is not None:
        _store_m(st, "exp_avg_slow", m_slow, True, bits.moment1())
    if v_buf.dtype in (torch.bfloat16, torch.float16):
        F.store_rounded(v_buf, v, bits.moment2(False))
    else:
        v_buf.copy_(v)


def _factored(p, pf, g, st, group, sc, bits):
    """Row/column second-moment statistics (Adafactor-style) with any first-moment storage
    (reference: apexw/state.py:300-323 for the denominator)."""
    r_t, c_t = st["exp_avg_sq_row"], st["exp_avg_sq_col"]
    rows, cols = r_t.numel(), c_t.numel()
    g2 = g.reshape(rows, cols)
    gsq = g2 * g2
    r_t.mul_(sc.beta2).add_(gsq.mean(dim=1), alpha=1.0 - sc.beta2)
    c_t.mul_(sc.beta2).add_(gsq.mean(dim=0), alpha=1.0 - sc.beta2)
    r_t.nan_to_num_(nan=0.0, posinf=0.0, neginf=0.0)
    c_t.nan_to_num_(nan=0.0, posinf=0.0, neginf=0.0)
    row = (r_t / r_t.mean().clamp_min(1e-30)).sqrt().unsqueeze(1)
    denom = (row * c_t.sqrt().unsqueeze(0) + sc.eps_scaled).clamp_min(sc.eps).reshape(p.shape)

    m_buf = st["exp_avg"]
    quant = m_buf.dtype in (torch.int8, torch.uint8)
    m = _lerp_to(_load_m(st, "exp_avg", p.shape, quant), g, sc.beta1)
    num = _lerp_to(m, g, sc.beta1) if group["nesterov"] else m
    if group["cautious"]:
        num = _cautious(num, g)
    _store_param(p, pf - num * (denom.reciprocal() * sc.step_size), bits)
    _store_m(st, "exp_avg", m, quant, bits.moment1())
