"""Matrix orthogonalisation for Muon: quintic Newton-Schulz and Polar Express.

One iteration is ``A = X X^T ; B = b A + c A^2 ; X = a X + B X`` on the wide orientation of
the matrix (rows <= cols), after dividing by the Frobenius norm.  Coefficients and calling
conventions follow the reference (apexw/muon.py:46-340): (a, b, c) = (3.4445, -4.7750,
2.0315) for Newton-Schulz; eight per-iteration triples with a 1.01 safety factor for Polar
Express.

On CUDA in bf16 the iteration runs on the hand-written tcgen05 kernels of
``csrc/ns_gemm.cu`` when they are available (``ns_backend()`` reports which path is
active); elsewhere it is plain matmuls.
"""

from __future__ import annotations

import os
from typing import Optional, Sequence, Tuple

import torch
from torch import Tensor

from .. import _native

NS_COEFFS: Tuple[float, float, float] = (3.4445, -4.7750, 2.0315)

_PE_RAW = (
    (8.28721201814563, -23.595886519098837, 17.300387312530933),
    (4.107059111542203, -2.9478499167379106, 0.5448431082926601),
    (3.9486908534822946, -2.908902115962949, 0.5518191394370137),
    (3.3184196573706015, -2.488488024314874, 0.51004894012372),
    (2.300652019954817, -1.6689039845747493, 0.4188073119525673),
    (1.891301407787398, -1.2679958271945868, 0.37680408948524835),
    (1.8750014808534479, -1.2500016453999487, 0.3750001645474248),
    (1.875, -1.25, 0.375),
)
_SAFETY = 1.01
POLAR_EXPRESS_COEFFS = tuple((a / _SAFETY, b / _SAFETY ** 3, c / _SAFETY ** 5) for a, b, c in _PE_RAW[:-1]) + (_PE_RAW[-1],)


def _work_dtype(t: Tensor) -> torch.dtype:
    return torch.bfloat16 if t.device.type == "cuda" else torch.float32


_SUPPORTED_ON: dict = {}        # device index -> does the tcgen05 path run there (asked once per device)


def _native_ns_ok(X: Tensor) -> bool:
    """The tcgen05 path takes bf16 CUDA matrices whose dimensions are multiples of 128."""
    if not X.is_cuda or X.dtype != torch.bfloat16 or _native.disabled_by_env():
        return False
    if os.environ.get("APEXW_B200_NS_BACKEND", "auto") == "torch":
        return False
    ok = _SUPPORTED_ON.get(X.device.index)
    if ok is None:
        nat = _native.load()
        with torch.cuda.device(X.device):
            ok = nat is not None and hasattr(nat, "ns_iterate") and bool(nat.ns_supported())
        _SUPPORTED_ON[X.device.index] = ok
    if not ok:
        return False
    m, n = X.shape[-2], X.shape[-1]
    return m % 128 == 0 and n % 128 == 0 and m >= 128 and n >= 128


def ns_backend(X: Tensor) -> str:
    return "tcgen05" if _native_ns_ok(X) else "torch"


#: optional int32 CUDA tensor; while set, the tcgen05 path records wait-expired codes there instead of
#: synchronising with the host after every call (set by callers that check it once per optimizer step)
_deferred_error_word: Optional[Tensor] = None


class deferred_errors:
    """Context manager: route the kernels' error codes of every Newton-Schulz call inside to ``word``."""

    def __init__(self, word: Tensor):
        self.word = word

    def __enter__(self):
        global _deferred_error_word
        self._prev, _deferred_error_word = _deferred_error_word, self.word
        return self

    def __exit__(self, *exc):
        global _deferred_error_word
        _deferred_error_word = self._prev
        return False


def _iterate(X: Tensor, coeffs: Sequence[Tuple[float, float, float]]) -> Tensor:
    """X: (..., m, n) with m <= n, already normalised."""
    if _native_ns_ok(X):
        nat = _native.load()
        flat = [c for triple in coeffs for c in triple]
        word = _deferred_error_word
        if word is not None and word.device == X.device:
            return nat.ns_iterate(X.contiguous(), flat, word)
        return nat.ns_iterate(X.contiguous(), flat)
    if X.dim() == 2:
        for a, b, c in coeffs:
            A = X @ X.T
            B = torch.addmm(A, A, A, beta=b, alpha=c)
            X = torch.addmm(X, B, X, beta=a, alpha=1.0)
        return X
    for a, b, c in coeffs:
        A = torch.bmm(X, X.transpose(-2, -1))
        B = torch.baddbmm(A, A, A, beta=b, alpha=c)
        X = torch.baddbmm(X, B, X, beta=a, alpha=1.0)
    return X


def _fused_orthogonalize(M: Tensor, coeffs, eps: float, out: Optional[Tensor]) -> Optional[Tensor]:
    """The whole map in native code (norm, scale + transpose in one pass, tcgen05 iteration, result written in
    place of a copy) when the tensor-core path applies; None otherwise."""
    Xb = M if M.dtype == torch.bfloat16 else (M.to(torch.bfloat16) if M.is_cuda else M)
    if not _native_ns_ok(Xb):       # checks device, dtype, the backend switch and the multiples of 128
        return None
    nat = _native.load()
    if not hasattr(nat, "ns_orthogonalize"):
        return None
    flat = [c for triple in coeffs for c in triple]
    word = _deferred_error_word
    if word is not None and word.device != Xb.device:
        word = None
    dst = out if (out is not None and out.dtype == torch.bfloat16 and out.is_contiguous() and out.shape == Xb.shape
                  and out.device == Xb.device) else None
    return nat.ns_orthogonalize(Xb.contiguous(), flat, float(eps), dst, word)


def _fold_input_scale(coeffs, s: float):
    """Coefficients that give, on X, what ``coeffs`` give on X / s: the first step's odd polynomial
    a(X/s) + b(X/s)^3 + c(X/s)^5 is a/s, b/s^3, c/s^5 applied to X; later steps are unchanged."""
    if s == 1.0 or not coeffs:
        return coeffs
    a, b, c = coeffs[0]
    return [(a / s, b / s ** 3, c / s ** 5)] + list(coeffs[1:])


def _orthogonalize(G: Tensor, coeffs, eps: float, work_dtype: Optional[torch.dtype], out: Optional[Tensor] = None,
                   norm_margin: float = 1.0) -> Tensor:
    """``norm_margin`` > 1 divides by ``norm * norm_margin + eps`` (Polar Express keeps the spectrum strictly inside
    its coefficients' interval this way, reference: apexw/muon.py:287, :320)."""
    shape = G.shape
    batched = G.dim() == 3
    M = G if (batched or G.dim() == 2) else G.reshape(shape[0], -1)
    wd = work_dtype or _work_dtype(M)
    if wd == torch.bfloat16 and M.dim() in (2, 3):
        # the native map normalises by the plain norm; the margin goes into the first step's coefficients
        U = _fused_orthogonalize(M, _fold_input_scale(coeffs, norm_margin), eps,
                                 out if out is not None and out.shape == M.shape else None)
        if U is not None:
            U = U.reshape(shape) if (not batched and len(shape) > 2) else U
            if out is not None and U.data_ptr() != out.data_ptr():
                out.copy_(U)
                return out
            return U if U.dtype == G.dtype else U.to(G.dtype)
    X = M.to(wd)
    if batched:
        nrm = torch.linalg.norm(X, dim=(-2, -1), keepdim=True)
    else:
        nrm = X.norm()
    X = X / ((nrm * norm_margin if norm_margin != 1.0 else nrm) + eps)
    tall = X.shape[-2] > X.shape[-1]
    if tall:
        X = X.transpose(-2, -1)
    X = _iterate(X.contiguous(), coeffs)
    if tall:
        X = X.transpose(-2, -1)
    if not batched and len(shape) > 2:
        X = X.reshape(shape)
    if out is not None:
        out.copy_(X)
        return out
    return X.to(G.dtype)


#: Polar Express divides by 1.01 x the Frobenius norm
PE_NORM_MARGIN = 1.01


def _pe_schedule(steps: int):
    n = len(POLAR_EXPRESS_COEFFS)
    return [POLAR_EXPRESS_COEFFS[i if i < n else -1] for i in range(steps)]


def zeropower_via_newtonschulz5(G: Tensor, steps: int = 5, eps: float = 1e-7,
                                work_dtype: Optional[torch.dtype] = None, compiled: bool = False, *,
                                out: Optional[Tensor] = None) -> Tensor:
    """Approximate polar factor of ``G`` (2-D, or flattened to 2-D) by ``steps`` quintic iterations.
    ``compiled`` is accepted for API compatibility; launch overhead is handled by the fused kernels.
    ``out`` (same shape and dtype as ``G``, may be ``G``) receives the result without an extra copy on the
    tensor-core path."""
    return _orthogonalize(G, [NS_COEFFS] * steps, eps, work_dtype, out)


def zeropower_via_newtonschulz5_batched(X_batch: Tensor, steps: int = 4, eps: float = 1e-7, *,
                                        out: Optional[Tensor] = None) -> Tensor:
    """Same for a stack ``(K, m, n)`` of equally shaped matrices."""
    return _orthogonalize(X_batch, [NS_COEFFS] * steps, eps, None, out)


def zeropower_via_polar_express(G: Tensor, steps: int = 4, eps: float = 1e-7,
                                work_dtype: Optional[torch.dtype] = None, compiled: bool = False) -> Tensor:
    return _orthogonalize(G, _pe_schedule(steps), eps, work_dtype, norm_margin=PE_NORM_MARGIN)


def zeropower_via_polar_express_batched(X_batch: Tensor, steps: int = 4, eps: float = 1e-7) -> Tensor:
    return _orthogonalize(X_batch, _pe_schedule(steps), eps, None, norm_margin=PE_NORM_MARGIN)
