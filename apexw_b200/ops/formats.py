"""State storage formats: blockwise int8, packed 6-bit, NF4, log-uint8 and 16-bit SR.

These are the torch (any-device) codecs.  They define the storage formats that
the fused sm_100a kernels in ``csrc/fused_state.cu`` read and write, and they
are what the CPU engine uses, so a checkpoint written on either path loads on
the other.  The byte layouts are those of the reference library
(apexw/quantization.py:66-482): int8 absmax/127 blocks, four 6-bit values in
three bytes, two NF4 nibbles per byte with the even element in the high nibble,
and a 24-octave logarithmic uint8 for the non-negative second moment with code
0 reserved for "v <= 0".

Rounding convention used throughout (kernels and engine alike):
``code = floor(x + 0.5 + noise)`` with ``noise = u - 0.5`` for ``u`` uniform in
[0, 1) when stochastic, and ``noise = 0`` otherwise.
"""

from __future__ import annotations

from typing import Optional, Tuple

import torch
from torch import Tensor

# ----------------------------------------------------------------------------
# code books
# ----------------------------------------------------------------------------

#: magnitudes of the 15-level symmetric NF4 momentum code book (index 7 is 0,
#: index 14 is 1, index 15 is an unused duplicate of 1).
NF4_MAGNITUDES = (0.0, 0.0911, 0.1848, 0.2844, 0.3949, 0.5251, 0.6962, 1.0)
NF4_CODEBOOK = torch.tensor(
    [-m for m in reversed(NF4_MAGNITUDES[1:])] + list(NF4_MAGNITUDES) + [1.0],
    dtype=torch.float32,
)
assert NF4_CODEBOOK.numel() == 16 and float(NF4_CODEBOOK[7]) == 0.0

_NF4_MAG_T = torch.tensor(NF4_MAGNITUDES, dtype=torch.float32)
# 1 / (c[j+1] - c[j]) as float32, with a dummy for the top level
_NF4_INV_GAP_T = torch.cat(
    [1.0 / (_NF4_MAG_T[1:] - _NF4_MAG_T[:-1]), torch.ones(1)]
).to(torch.float32)

LOGV_OCTAVES = 24.0
LOGV_STEPS_PER_OCTAVE = 254.0 / LOGV_OCTAVES
LOGV_MIN_RATIO = 2.0 ** (-LOGV_OCTAVES)
#: decode table of the log-uint8 variance format: code q>0 maps to
#: 2**((q-1)*24/254 - 24); code 0 maps to exactly 0.
LOGV_DECODE = torch.tensor(
    [0.0] + [2.0 ** ((q - 1) * LOGV_OCTAVES / 254.0 - LOGV_OCTAVES) for q in range(1, 256)],
    dtype=torch.float32,
)

M_SCALE_DECAY = 0.9    # EMA-MAX factor for first-moment block scales
V_SCALE_DECAY = 0.95   # EMA-MAX factor for second-moment block scales
SCALE_FLOOR = 1e-12

_LUT_CACHE: dict = {}


def _on(device, name: str, src: Tensor) -> Tensor:
    key = (name, str(device))
    t = _LUT_CACHE.get(key)
    if t is None:
        t = src.to(device)
        _LUT_CACHE[key] = t
    return t


def nf4_codebook(device) -> Tensor:
    return _on(device, "nf4", NF4_CODEBOOK)


def logv_table(device) -> Tensor:
    return _on(device, "logv", LOGV_DECODE)


# ----------------------------------------------------------------------------
# helpers
# ----------------------------------------------------------------------------

def _random_bits16(shape, device, generator=None) -> Tensor:
    return torch.randint(0, 65536, tuple(shape), dtype=torch.int64, device=device, generator=generator)


def _noise_from_bits(bits16: Optional[Tensor]) -> Optional[Tensor]:
    """16 random bits -> dither in [-0.5, 0.5)."""
    if bits16 is None:
        return None
    return bits16.to(torch.float32) * (1.0 / 65536.0) - 0.5


def as_blocks(x: Tensor, block_size: int, fill: float = 0.0) -> Tuple[Tensor, int]:
    """Flatten ``x`` to fp32 rows of ``block_size`` (last row padded). Returns (blocks, numel)."""
    flat = x.reshape(-1).to(torch.float32)
    n = flat.numel()
    pad = (-n) % block_size
    if pad:
        flat = torch.nn.functional.pad(flat, (0, pad), value=fill)
    return flat.view(-1, block_size), n


def _pad_bits(bits16: Optional[Tensor], rows: int, block_size: int) -> Optional[Tensor]:
    if bits16 is None:
        return None
    flat = bits16.reshape(-1)
    pad = rows * block_size - flat.numel()
    if pad:
        flat = torch.nn.functional.pad(flat, (0, pad))
    return flat.view(rows, block_size)


def _ema_max(target: Tensor, old: Optional[Tensor], decay: float) -> Tensor:
    if old is not None:
        target = torch.maximum(target, old.reshape(-1, 1).to(torch.float32) * decay)
    return target.clamp_min(SCALE_FLOOR)


def round_dither(x: Tensor, noise: Optional[Tensor]) -> Tensor:
    """floor(x + 0.5 + noise): the one rounding rule of every integer codec here."""
    if noise is None:
        return torch.floor(x + 0.5)
    return torch.floor((x + 0.5) + noise)


# ----------------------------------------------------------------------------
# int8 absmax blocks
# ----------------------------------------------------------------------------

def int8_encode(blocks: Tensor, old_scales: Optional[Tensor], bits16: Optional[Tensor], levels: float = 127.0):
    """blocks: (nb, bs) fp32 -> (codes fp32 in [-levels, levels], scales (nb,1))."""
    absmax = blocks.abs().amax(dim=1, keepdim=True)
    scales = _ema_max(absmax / levels, old_scales, M_SCALE_DECAY)
    inv = 1.0 / scales
    q = round_dither(blocks * inv, _noise_from_bits(bits16)).clamp_(-levels, levels)
    return q, scales


def _quantize_blockwise_int8(tensor, block_size: int = 256, stochastic: bool = False,
                             out_q=None, out_scales=None, old_scales=None, bits16=None):
    """Blockwise int8 with EMA-MAX scales (reference: apexw/quantization.py:66-110)."""
    n = tensor.numel()
    if n == 0:
        return (torch.empty_like(tensor, dtype=torch.int8),
                torch.empty((0, 1), device=tensor.device, dtype=torch.float32))
    blocks, _ = as_blocks(tensor, block_size)
    if stochastic and bits16 is None:
        bits16 = _random_bits16(blocks.shape, tensor.device)
    bits16 = _pad_bits(bits16, blocks.shape[0], block_size) if stochastic else None
    q, scales = int8_encode(blocks, old_scales, bits16)
    q = q.to(torch.int8).view(-1)[:n].view(tensor.shape)
    if out_q is not None:
        out_q.copy_(q)
        q = out_q
    if out_scales is not None:
        out_scales.copy_(scales.view_as(out_scales))
        scales = out_scales
    return q, scales


def _dequantize_blockwise_int8(q, scales, block_size: int = 256):
    n = q.numel()
    if n == 0:
        return torch.empty_like(q, dtype=torch.float32)
    blocks, _ = as_blocks(q, block_size)
    out = blocks * scales.reshape(-1, 1).to(torch.float32)
    return out.view(-1)[:n].view(q.shape)


# ----------------------------------------------------------------------------
# packed 6-bit (4 values -> 3 bytes), levels -31..31 stored with +31 bias
# ----------------------------------------------------------------------------

def six_bit_padded_len(numel: int, block_size: int) -> int:
    padded = numel + ((-numel) % block_size)
    return padded + ((-padded) % 4)


def _quantize_blockwise_6bit(tensor, block_size: int = 256, stochastic: bool = False,
                             out_q=None, out_scales=None, old_scales=None, bits16=None):
    """Packed 6-bit momentum (reference: apexw/quantization.py:129-186)."""
    n = tensor.numel()
    if n == 0:
        return (torch.empty(0, dtype=torch.uint8, device=tensor.device),
                torch.empty((0, 1), device=tensor.device, dtype=torch.float32))
    blocks, _ = as_blocks(tensor, block_size)
    if stochastic and bits16 is None:
        bits16 = _random_bits16(blocks.shape, tensor.device)
    bits16 = _pad_bits(bits16, blocks.shape[0], block_size) if stochastic else None
    q, scales = int8_encode(blocks, old_scales, bits16, levels=31.0)
    u = (q + 31.0).to(torch.uint8).reshape(-1)
    extra = (-u.numel()) % 4
    if extra:
        u = torch.nn.functional.pad(u, (0, extra), value=31)
    u = u.view(-1, 4).to(torch.int32)
    b0 = (u[:, 0] & 0x3F) | ((u[:, 1] & 0x03) << 6)
    b1 = ((u[:, 1] >> 2) & 0x0F) | ((u[:, 2] & 0x0F) << 4)
    b2 = ((u[:, 2] >> 4) & 0x03) | ((u[:, 3] & 0x3F) << 2)
    packed = torch.stack([b0, b1, b2], dim=1).to(torch.uint8).reshape(-1)
    if out_q is not None:
        out_q.view(-1).copy_(packed)
        packed = out_q
    if out_scales is not None:
        out_scales.copy_(scales.view_as(out_scales))
        scales = out_scales
    return packed, scales


def _dequantize_blockwise_6bit(q_packed, scales, numel: Optional[int] = None, block_size: int = 256):
    nbytes = q_packed.numel()
    if nbytes == 0:
        return torch.empty(0, dtype=torch.float32, device=q_packed.device)
    b = q_packed.reshape(-1, 3).to(torch.int32)
    u0 = b[:, 0] & 0x3F
    u1 = ((b[:, 0] >> 6) & 0x03) | ((b[:, 1] & 0x0F) << 2)
    u2 = ((b[:, 1] >> 4) & 0x0F) | ((b[:, 2] & 0x03) << 4)
    u3 = (b[:, 2] >> 2) & 0x3F
    vals = torch.stack([u0, u1, u2, u3], dim=1).reshape(-1).to(torch.float32) - 31.0
    nb = scales.numel()
    vals = vals[: nb * block_size].view(nb, block_size) * scales.reshape(-1, 1).to(torch.float32)
    flat = vals.reshape(-1)
    if numel is not None and numel < flat.numel():
        flat = flat[:numel]
    return flat


# ----------------------------------------------------------------------------
# NF4 momentum
# ----------------------------------------------------------------------------

def _round_to_f16(v: Tensor) -> Tensor:
    """float64 -> float16 with ONE rounding to nearest-even (a cast through float32 would round twice)."""
    _, e = torch.frexp(v)                                   # |v| = f * 2**e with f in [0.5, 1)
    q = torch.ldexp(torch.ones_like(v), e.clamp_min(-13) - 11)   # spacing of float16 at |v| (2**-24 below 2**-14)
    return (torch.round(v / q) * q).to(torch.float16)


# F maps magnitude level c_j to j and is linear in between; the gaps grow, so F is concave and equals the minimum of
# its seven lines S_j * a + B_j.  The constants are the half-precision values the kernel uses (csrc/codec.cuh), with
# 0.5 already taken off the intercepts.
_NF4_LINE_S = torch.tensor([0x497d, 0x4956, 0x4905, 0x4886, 0x47ae, 0x45d8, 0x4295], dtype=torch.int16).view(torch.float16)
_NF4_LINE_B = torch.tensor([-0x4800, -0x4872, -0x4a50, -0x5348, 0x3779, 0x3db9, 0x426b], dtype=torch.int16).view(torch.float16)


def nf4_encode_unit(x: Tensor, bits16: Optional[Tensor]) -> Tensor:
    """Encode values already divided by their block scale (clamped to [-1, 1]).

    Works on magnitudes in half precision, step by step as the kernels do (``csrc/codec.cuh``): ``F - 0.5`` is the
    minimum of seven fused multiply-adds, ``u = (2r + 1)/2048`` with ``r`` the low 10 of the 16 random bits is added
    (stochastic: the upper neighbour is then chosen with probability ``(|x| - c_j)/(c_{j+1} - c_j)``), or ``u = 0.5``
    (nearest), and ``1543 +- (F - 0.5 + u)`` is rounded to an integer, ties to even, whose low four bits are the
    code.  Returns int64 code indices 0..14.
    """
    s_h = _on(x.device, "nf4_line_s", _NF4_LINE_S).double()
    b_h = _on(x.device, "nf4_line_b", _NF4_LINE_B).double()
    xh = x.to(torch.float16)
    a = xh.abs().clamp_max(1.0).double()
    f = _round_to_f16(a * s_h[0] + b_h[0])
    for j in range(1, 7):
        f = torch.minimum(f, _round_to_f16(a * s_h[j] + b_h[j]))
    if bits16 is not None:
        u = (2 * (bits16.to(torch.int64) & 0x3FF) + 1).to(torch.float64) / 2048.0     # exact in half precision
    else:
        u = torch.full_like(a, 0.5)
    w = _round_to_f16(f.double() + u).double()
    neg = torch.signbit(xh)
    code = torch.round(1543.0 + torch.where(neg, -w, w))      # half precision has a spacing of one in [1024, 2048)
    return (code.to(torch.int64) - 1024) & 0xF


def nf4_encode(blocks: Tensor, old_scales: Optional[Tensor], bits16: Optional[Tensor]):
    absmax = blocks.abs().amax(dim=1, keepdim=True)
    scales = _ema_max(absmax, old_scales, M_SCALE_DECAY)
    inv = 1.0 / scales
    x = (blocks * inv).clamp_(-1.0, 1.0)
    return nf4_encode_unit(x, bits16), scales


def nf4_pack(codes: Tensor, numel: int) -> Tensor:
    flat = codes.reshape(-1)[:numel].to(torch.uint8)
    if numel % 2:
        flat = torch.nn.functional.pad(flat, (0, 1), value=7)
    pairs = flat.view(-1, 2)
    return (pairs[:, 0] << 4) | pairs[:, 1]


def nf4_unpack(packed: Tensor, numel: int) -> Tensor:
    b = packed.reshape(-1).to(torch.int64)
    codes = torch.stack([(b >> 4) & 0xF, b & 0xF], dim=1).reshape(-1)
    return codes[:numel]


def _quantize_blockwise_int4(tensor, block_size: int = 256, stochastic: bool = False,
                             out_q=None, out_scales=None, old_scales=None, bits16=None):
    """NF4 packed momentum, absmax scale (reference: apexw/quantization.py:278-335)."""
    n = tensor.numel()
    if n == 0:
        return (torch.empty(0, dtype=torch.uint8, device=tensor.device),
                torch.empty((0, 1), device=tensor.device, dtype=torch.float32))
    blocks, _ = as_blocks(tensor, block_size)
    if stochastic and bits16 is None:
        bits16 = _random_bits16(blocks.shape, tensor.device)
    bits16 = _pad_bits(bits16, blocks.shape[0], block_size) if stochastic else None
    codes, scales = nf4_encode(blocks, old_scales, bits16)
    packed = nf4_pack(codes, n)
    if out_q is not None:
        out_q.view(-1).copy_(packed)
        packed = out_q
    if out_scales is not None:
        out_scales.copy_(scales.view_as(out_scales))
        scales = out_scales
    return packed, scales


def _dequantize_blockwise_int4(q_packed, scales, numel: int, block_size: int = 256):
    if numel == 0:
        return torch.empty(0, dtype=torch.float32, device=q_packed.device)
    vals = nf4_codebook(q_packed.device)[nf4_unpack(q_packed, numel)]
    blocks, _ = as_blocks(vals, block_size)
    out = blocks * scales.reshape(-1, 1).to(torch.float32)
    return out.view(-1)[:numel]


# ----------------------------------------------------------------------------
# log-uint8 second moment
# ----------------------------------------------------------------------------

def logv_encode(blocks: Tensor, old_scales: Optional[Tensor], bits16: Optional[Tensor]):
    """blocks (nb, bs) of non-negative fp32 -> (codes int64 0..255, scales (nb,1))."""
    blocks = torch.nan_to_num(blocks, nan=0.0, posinf=0.0, neginf=0.0)
    vmax = blocks.amax(dim=1, keepdim=True)
    scales = _ema_max(vmax, old_scales, V_SCALE_DECAY)
    inv = 1.0 / scales
    r = (blocks * inv).clamp_min(LOGV_MIN_RATIO)
    pos = (torch.log2(r).double() * float(torch.tensor(LOGV_STEPS_PER_OCTAVE, dtype=torch.float32)) + 255.0).float()  # one fma
    q = round_dither(pos, _noise_from_bits(bits16)).clamp_(1.0, 255.0).to(torch.int64)
    q = torch.where(blocks > 0, q, torch.zeros_like(q))
    return q, scales


def _quantize_blockwise_uint8(tensor, block_size: int = 256, stochastic: bool = True,
                              out_q=None, out_scales=None, old_scales=None, bits16=None):
    """24-octave logarithmic uint8 for v >= 0 (reference: apexw/quantization.py:378-430)."""
    n = tensor.numel()
    if n == 0:
        return (torch.empty_like(tensor, dtype=torch.uint8),
                torch.empty((0, 1), device=tensor.device, dtype=torch.float32))
    blocks, _ = as_blocks(tensor, block_size)
    if stochastic and bits16 is None:
        bits16 = _random_bits16(blocks.shape, tensor.device)
    bits16 = _pad_bits(bits16, blocks.shape[0], block_size) if stochastic else None
    q, scales = logv_encode(blocks, old_scales, bits16)
    q = q.to(torch.uint8).view(-1)[:n].view(tensor.shape)
    if out_q is not None:
        out_q.copy_(q)
        q = out_q
    if out_scales is not None:
        out_scales.copy_(scales.view_as(out_scales))
        scales = out_scales
    return q, scales


def _dequantize_blockwise_uint8(q, scales, block_size: int = 256):
    n = q.numel()
    if n == 0:
        return torch.empty_like(q, dtype=torch.float32)
    vals = logv_table(q.device)[q.reshape(-1).to(torch.int64)]
    blocks, _ = as_blocks(vals, block_size)
    out = blocks * scales.reshape(-1, 1).to(torch.float32)
    return out.view(-1)[:n].view(q.shape)


# ----------------------------------------------------------------------------
# 16-bit stochastic rounding
# ----------------------------------------------------------------------------

def bf16_round_sr(x: Tensor, bits16: Tensor) -> Tensor:
    """fp32 -> bf16 by adding 16 random bits below the kept mantissa, then truncating.

    This is bit for bit what the Blackwell conversion unit does (``cvt.rs.bf16x2.f32``, used by the kernels): finite
    values may carry into the next binade, the largest one into Inf; Inf stays Inf; NaN becomes the canonical 0x7FFF.
    """
    u = x.contiguous().view(torch.int32).to(torch.int64) & 0xFFFFFFFF
    out = ((u + bits16.reshape(x.shape)) & 0xFFFFFFFF) & 0xFFFF0000
    out = torch.where((u & 0x7FFFFFFF) > 0x7F800000, torch.full_like(out, 0x7FFF0000), out)
    out = torch.where(out >= 0x80000000, out - 0x100000000, out).to(torch.int32)
    return out.view(torch.float32).to(torch.bfloat16)


def fp16_round_sr(x: Tensor, bits16: Tensor) -> Tensor:
    """fp32 -> fp16 with stochastic rounding; saturates at +-65504.

    Follows ``cvt.rs.satfinite.f16x2.f32``: the low 13 of the random bits are added below the kept mantissa and the
    sum is truncated; in the sub-normal half range (spacing 2**-24) the value is first cut to 13 fractional bits of
    that spacing and the same 13 random bits decide the step; NaN becomes the canonical 0x7FFF.
    """
    bits13 = (bits16.reshape(x.shape) & 0x1FFF)
    ax = x.abs()
    # sub-normal half range
    y = ax.double() * 16777216.0
    sub = torch.floor(torch.floor(y * 8192.0) / 8192.0 + bits13.double() / 8192.0) * (2.0 ** -24)
    u = ax.contiguous().view(torch.int32).to(torch.int64) & 0x7FFFFFFF
    t = ((u + bits13) & 0xFFFFFFFF) & 0xFFFFE000
    normal = t.to(torch.int32).view(torch.float32).clamp_max(65504.0)
    out = torch.where(ax < 6.103515625e-5, sub.float(), normal)
    out = torch.copysign(out, x)
    out = torch.where(torch.isnan(x), x, out)
    return out.to(torch.float16)


def store_rounded(dst: Tensor, value_f32: Tensor, bits16: Optional[Tensor]) -> None:
    """Write fp32 ``value`` into ``dst`` (any float dtype); SR when bits are given and dst is 16-bit."""
    value_f32 = value_f32.reshape(dst.shape)
    if dst.dtype == torch.bfloat16 and bits16 is not None:
        dst.copy_(bf16_round_sr(value_f32, bits16))
    elif dst.dtype == torch.float16 and bits16 is not None:
        dst.copy_(fp16_round_sr(value_f32, bits16))
    elif dst.dtype == torch.float16:
        dst.copy_(value_f32.clamp(-65504.0, 65504.0))
    else:
        dst.copy_(value_f32)


def _copy_fp32_to_16bit_sr_(p: Tensor, p_f: Tensor, stochastic: bool = True, in_place_src: bool = False) -> None:
    """Store fp32 ``p_f`` into ``p`` with stochastic rounding when ``p`` is 16-bit
    (reference: apexw/quantization.py:451-482)."""
    bits = _random_bits16(p.shape, p_f.device) if (stochastic and p.dtype in (torch.bfloat16, torch.float16)) else None
    store_rounded(p, p_f.to(torch.float32), bits)
