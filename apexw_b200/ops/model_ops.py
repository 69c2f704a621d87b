"""Fused model-side ops used by the training harness (no counterpart in the reference,
which ships no models): RMSNorm (+residual add), SwiGLU, rotary embedding, softmax
cross-entropy, and a linear layer whose weight gradient accumulates straight into a
preallocated gradient buffer.

On CUDA tensors each op calls one hand-written sm_100a kernel from
``csrc/model_ops.cu``; on CPU tensors (tests, tiny models) the same autograd
functions run an fp32 torch formulation, which is also the numerical reference in
the GPU tests.
"""

from __future__ import annotations

from typing import Optional, Tuple

import torch
import torch.nn.functional as Fnn
from torch import Tensor

from .. import _native


def _use_native(x: Tensor) -> bool:
    if not x.is_cuda:
        return False
    if _native.disabled_by_env():
        return False
    _native.require()
    return x.dtype in (torch.bfloat16, torch.float32)


# ---------------------------------------------------------------------------
# RMSNorm with optional fused residual add
# ---------------------------------------------------------------------------

class _RMSNorm(torch.autograd.Function):
    """y = rmsnorm(x + residual) * w ; also returns h = x + residual (the new residual stream)."""

    @staticmethod
    def forward(ctx, x: Tensor, residual: Optional[Tensor], weight: Tensor, eps: float):
        shape = x.shape
        x2 = x.reshape(-1, shape[-1])
        r2 = residual.reshape(-1, shape[-1]) if residual is not None else None
        if _use_native(x2):
            nat = _native.load()
            x2 = x2.contiguous()
            r2 = r2.contiguous() if r2 is not None else None
            y, h, rstd = nat.rmsnorm_fwd(x2, r2, weight, eps)
            _native.count(1)
        else:
            h32 = x2.float() + (r2.float() if r2 is not None else 0.0)
            h = h32.to(x.dtype) if r2 is not None else x2
            h32 = h.float()
            rstd = torch.rsqrt(h32.pow(2).mean(dim=-1) + eps)
            y = (h32 * rstd.unsqueeze(-1) * weight.float()).to(x.dtype)
        ctx.save_for_backward(h, weight, rstd)
        ctx.has_residual = residual is not None
        ctx.shape = shape
        if residual is None:
            return y.view(shape), x
        return y.view(shape), h.view(shape)

    @staticmethod
    def backward(ctx, dy: Tensor, dh_out: Optional[Tensor]):
        h, weight, rstd = ctx.saved_tensors
        H = h.shape[-1]
        dy2 = dy.reshape(-1, H)
        dh2 = dh_out.reshape(-1, H) if dh_out is not None else None
        if _use_native(h):
            nat = _native.load()
            dy2 = dy2.contiguous()
            dh2 = dh2.contiguous() if dh2 is not None else None
            dx, dw = nat.rmsnorm_bwd(dy2, dh2, h, weight, rstd)
            _native.count(2)
            dw = dw.to(weight.dtype)
        else:
            h32 = h.float()
            g = dy2.float() * weight.float()
            xhat = h32 * rstd.unsqueeze(-1)
            dw = (dy2.float() * xhat).sum(dim=0).to(weight.dtype)
            dx32 = (g - xhat * (g * xhat).mean(dim=-1, keepdim=True)) * rstd.unsqueeze(-1)
            if dh2 is not None:
                dx32 = dx32 + dh2.float()
            dx = dx32.to(h.dtype)
        dx = dx.view(ctx.shape)
        return dx, (dx if ctx.has_residual else None), dw, None


def rms_norm(x: Tensor, weight: Tensor, eps: float = 1e-5, residual: Optional[Tensor] = None) -> Tuple[Tensor, Tensor]:
    """Returns (normed, new_residual_stream)."""
    return _RMSNorm.apply(x, residual, weight, eps)


# ---------------------------------------------------------------------------
# SwiGLU on a fused [gate | up] projection
# ---------------------------------------------------------------------------

class _SwiGLU(torch.autograd.Function):
    """gu: (..., 2*F) with gate in the first half -> silu(gate) * up."""

    @staticmethod
    def forward(ctx, gu: Tensor):
        ctx.save_for_backward(gu)
        if _use_native(gu):
            _native.count(1)
            return _native.load().swiglu_fwd(gu.contiguous())
        gate, up = gu.float().chunk(2, dim=-1)
        return (Fnn.silu(gate) * up).to(gu.dtype)

    @staticmethod
    def backward(ctx, dy: Tensor):
        (gu,) = ctx.saved_tensors
        if _use_native(gu):
            _native.count(1)
            return _native.load().swiglu_bwd(dy.contiguous(), gu.contiguous())
        gate, up = gu.float().chunk(2, dim=-1)
        sig = torch.sigmoid(gate)
        silu = gate * sig
        dyf = dy.float()
        dgate = dyf * up * (sig + silu * (1 - sig))
        dup = dyf * silu
        return torch.cat([dgate, dup], dim=-1).to(gu.dtype)


def swiglu(gu: Tensor) -> Tensor:
    return _SwiGLU.apply(gu)


# ---------------------------------------------------------------------------
# rotary embedding, applied to q and k of a fused qkv projection
# ---------------------------------------------------------------------------

def rope_tables(seq_len: int, head_dim: int, theta: float, device, dtype=torch.float32) -> Tuple[Tensor, Tensor]:
    inv = 1.0 / (theta ** (torch.arange(0, head_dim, 2, device=device, dtype=torch.float32) / head_dim))
    ang = torch.outer(torch.arange(seq_len, device=device, dtype=torch.float32), inv)
    return ang.cos().to(dtype).contiguous(), ang.sin().to(dtype).contiguous()


def _rope_torch(x: Tensor, cos: Tensor, sin: Tensor, sign: float) -> Tensor:
    # x: (B, S, H, D); rotate-half convention
    d2 = x.shape[-1] // 2
    xf = x.float()
    x1, x2 = xf[..., :d2], xf[..., d2:]
    c = cos[: x.shape[1]].view(1, x.shape[1], 1, d2)
    s = sin[: x.shape[1]].view(1, x.shape[1], 1, d2) * sign
    return torch.cat([x1 * c - x2 * s, x2 * c + x1 * s], dim=-1).to(x.dtype)


class _RoPE(torch.autograd.Function):
    """Rotate the q and k heads of a packed (B, S, Hq+2*Hkv, D) tensor; v heads pass through."""

    @staticmethod
    def forward(ctx, qkv: Tensor, cos: Tensor, sin: Tensor, n_rot_heads: int):
        ctx.save_for_backward(cos, sin)
        ctx.n_rot = n_rot_heads
        if _use_native(qkv):
            _native.count(1)
            return _native.load().rope_apply(qkv.contiguous(), cos, sin, n_rot_heads, False)
        out = qkv.clone()
        out[:, :, :n_rot_heads] = _rope_torch(qkv[:, :, :n_rot_heads], cos, sin, 1.0)
        return out

    @staticmethod
    def backward(ctx, d: Tensor):
        cos, sin = ctx.saved_tensors
        if _use_native(d):
            _native.count(1)
            return _native.load().rope_apply(d.contiguous(), cos, sin, ctx.n_rot, True), None, None, None
        out = d.clone()
        out[:, :, :ctx.n_rot] = _rope_torch(d[:, :, :ctx.n_rot], cos, sin, -1.0)
        return out, None, None, None


def rope_qkv(qkv: Tensor, cos: Tensor, sin: Tensor, n_rot_heads: int) -> Tensor:
    return _RoPE.apply(qkv, cos, sin, n_rot_heads)


# ---------------------------------------------------------------------------
# softmax cross-entropy: loss and d(logits) in one pass, logits overwritten by their gradient
# ---------------------------------------------------------------------------

def _ce_fwd_bwd(logits: Tensor, targets: Tensor, grad_scale: float, scale_dev: Optional[Tensor] = None) -> Tensor:
    """Returns per-row losses (fp32) and overwrites ``logits`` with grad_scale * scale_dev * dloss/dlogits.
    A target outside ``[0, V)`` (``ignore_index`` -100 included) marks an ignored row: loss 0, zero gradient row."""
    if _use_native(logits):
        _native.count(1)
        return _native.load().cross_entropy_fwd_bwd(logits, targets, grad_scale, scale_dev)
    lf = logits.float()
    counted = (targets >= 0) & (targets < lf.shape[1])
    safe = torch.where(counted, targets, torch.zeros_like(targets)).view(-1, 1)
    lse = torch.logsumexp(lf, dim=-1)
    loss = (lse - lf.gather(1, safe).squeeze(1)) * counted
    prob = torch.exp(lf - lse.unsqueeze(1))
    prob.scatter_add_(1, safe, torch.full((targets.numel(), 1), -1.0, dtype=prob.dtype, device=prob.device))
    prob = prob * counted.unsqueeze(1)
    scale = grad_scale if scale_dev is None else grad_scale * scale_dev.float()
    logits.copy_((prob * scale).to(logits.dtype))
    return loss


class _LinearCrossEntropy(torch.autograd.Function):
    """mean CE( h @ W^T , targets ) computed in row chunks so full fp32 logits never exist.

    Forward also computes the gradients (they only need the chunk's logits), so
    backward is two scalings.  With ``ignore_index`` set, rows whose target equals it (or lies outside the
    vocabulary) contribute neither loss nor gradient and the mean runs over the remaining rows, as
    ``torch.nn.functional.cross_entropy`` does; the row count stays on the device.
    """

    @staticmethod
    def forward(ctx, h: Tensor, weight: Tensor, targets: Tensor, chunk_rows: int, main_grad: Optional[Tensor],
                loss_scale: float, ignore_index: Optional[int]):
        T = h.shape[0]
        dh = torch.empty_like(h)
        dw = main_grad if main_grad is not None else torch.zeros_like(weight)
        total = torch.zeros((), dtype=torch.float32, device=h.device)
        if ignore_index is None:
            inv_T, inv_dev = loss_scale / T, None
        else:
            n = ((targets >= 0) & (targets < weight.shape[0])).sum().clamp_min(1).to(torch.float32)
            inv_T, inv_dev = loss_scale, n.reciprocal().reshape(1)
        need_grad = torch.is_grad_enabled() or h.requires_grad or weight.requires_grad
        if main_grad is not None:
            weight._apexw_can_overwrite = True
        for s in range(0, T, chunk_rows):
            e = min(s + chunk_rows, T)
            logits = h[s:e] @ weight.t()
            losses = _ce_fwd_bwd(logits, targets[s:e], inv_T, inv_dev)
            total += losses.sum()
            if need_grad:
                torch.mm(logits, weight, out=dh[s:e])
                if main_grad is not None and getattr(weight, "_apexw_overwrite", False):
                    torch.mm(logits.t(), h[s:e], out=dw)        # first contribution since zero_grad: no read of zeros
                    weight._apexw_overwrite = False
                else:
                    dw.addmm_(logits.t(), h[s:e])
        ctx.save_for_backward(dh, dw if main_grad is None else torch.empty(0))
        ctx.fused_wgrad = main_grad is not None
        ctx.ready_cb = getattr(weight, "_apexw_grad_ready", None) if main_grad is not None else None
        return total * inv_T if inv_dev is None else total * inv_T * inv_dev[0]

    @staticmethod
    def backward(ctx, dloss: Tensor):
        dh, dw = ctx.saved_tensors
        # The gradients were formed in forward for d(loss) = 1.  An upstream factor is applied
        # here without a host sync; with ``main_grad`` the weight gradient is already
        # accumulated, so scale the loss through ``loss_scale`` instead of multiplying it later.
        dh = dh * dloss.to(dh.dtype)
        if not ctx.fused_wgrad:
            dw = dw * dloss.to(dw.dtype)
        elif ctx.ready_cb is not None:
            ctx.ready_cb()            # the accumulated weight gradient is final for this backward
        return dh, (None if ctx.fused_wgrad else dw), None, None, None, None, None


def linear_cross_entropy(h: Tensor, weight: Tensor, targets: Tensor, chunk_rows: int = 4096,
                         main_grad: Optional[Tensor] = None, loss_scale: float = 1.0,
                         ignore_index: Optional[int] = None) -> Tensor:
    """mean cross-entropy of ``h @ weight.T`` against ``targets``, times ``loss_scale``.  ``ignore_index`` (e.g.
    -100): the mean is over the rows with a target inside the vocabulary.  Without it the mean is over all rows;
    out-of-vocabulary targets still count as ignored rows (zero loss and gradient), they are never used as an index."""
    return _LinearCrossEntropy.apply(h, weight, targets, chunk_rows, main_grad, loss_scale, ignore_index)


# ---------------------------------------------------------------------------
# linear layer with gradient accumulation fused into the weight-gradient GEMM
# ---------------------------------------------------------------------------

class _LinearAccum(torch.autograd.Function):
    """y = x @ W^T.  When the weight carries ``main_grad`` the weight gradient is
    accumulated into it by the GEMM itself (beta = 1) and autograd sees no gradient,
    which removes one read-modify-write of every weight gradient per micro-batch."""

    @staticmethod
    def forward(ctx, x: Tensor, weight: Tensor):
        ctx.save_for_backward(x, weight)
        weight._apexw_can_overwrite = True      # this layer can write its gradient with beta = 0 (see _FlatStore.clear_grads)
        return x @ weight.t()

    @staticmethod
    def backward(ctx, dy: Tensor):
        x, weight = ctx.saved_tensors
        dy2 = dy.reshape(-1, dy.shape[-1])
        x2 = x.reshape(-1, x.shape[-1])
        dx = (dy2 @ weight).view(x.shape) if ctx.needs_input_grad[0] else None
        main = getattr(weight, "main_grad", None)
        if main is not None:
            if getattr(weight, "_apexw_overwrite", False):
                torch.mm(dy2.t(), x2, out=main)                 # first contribution since zero_grad: no read of zeros
                weight._apexw_overwrite = False
            else:
                main.addmm_(dy2.t(), x2)
            ready = getattr(weight, "_apexw_grad_ready", None)
            if ready is not None:
                ready()               # autograd never sees this gradient: tell an overlapping optimizer it is final
            return dx, None
        return dx, dy2.t() @ x2


def linear(x: Tensor, weight: Tensor) -> Tensor:
    if getattr(weight, "main_grad", None) is not None:
        return _LinearAccum.apply(x, weight)
    return Fnn.linear(x, weight)
