// Shared device code of the fused optimizer-state kernels.
//
// One work item is a chunk of 2048 consecutive elements of one segment (a
// parameter tensor, or the slice of it that this rank owns).  A CTA of 256
// threads handles one chunk at a time, 8 consecutive elements per thread, in a
// single pass over HBM: decode moments -> AdamW update with decoupled decay ->
// re-encode with stochastic rounding -> store.
//
// The chunk body is a template over an IO policy so that the same arithmetic
// serves the single-GPU kernel (local gradient in, local parameter out) and the
// ZeRO kernel (gradient reduced from peers' memory in registers, parameter
// written to every peer).
//
// Two code paths produce identical values:
//   * the fast path (segment flagged SEG_FAST, full chunk): everything bf16 and
//     16-byte aligned, no per-element predication, no dtype dispatch;
//   * the general path: any of fp32/bf16, any alignment, ragged tail.
// These kernels are bound by instruction issue before HBM, so the arithmetic is
// written with explicit fused multiply-adds, MUFU approximations for the one
// square root and reciprocal per denominator, and a 3-instruction random word per
// element.  The torch engine mirrors the same formula order (fma emulated in
// float64); only the approximate sqrt/rcp/log2 differ from it in the last place.
//
// Replaces, in function, the reference's three elementwise kernels
// (apexw/csrc/apexw_cuda_kernel.cu:113-460, :580-649, :908-1336).
#pragma once
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <cstdint>
#include "plan_types.h"
#include "codec.cuh"
#include "rng.cuh"

namespace apexb {

// ---------------------------------------------------------------------------
// small math helpers
// ---------------------------------------------------------------------------

__device__ __forceinline__ float fast_sqrt(float x) {
    float r;
    asm("sqrt.approx.ftz.f32 %0, %1;" : "=f"(r) : "f"(x));
    return r;
}
__device__ __forceinline__ float fast_rcp(float x) {
    float r;
    asm("rcp.approx.ftz.f32 %0, %1;" : "=f"(r) : "f"(x));
    return r;
}

__device__ __forceinline__ float lo_bf16(uint32_t w) { return __uint_as_float(w << 16); }
__device__ __forceinline__ float hi_bf16(uint32_t w) { return __uint_as_float(w & 0xFFFF0000u); }

__device__ __forceinline__ void unpack8(const uint4& r, float (&o)[8]) {
    o[0] = lo_bf16(r.x); o[1] = hi_bf16(r.x); o[2] = lo_bf16(r.y); o[3] = hi_bf16(r.y);
    o[4] = lo_bf16(r.z); o[5] = hi_bf16(r.z); o[6] = lo_bf16(r.w); o[7] = hi_bf16(r.w);
}

// two fp32 -> one word of two bf16 (a in the low half) with stochastic rounding by the conversion unit:
// cvt.rs adds 16 random bits below the kept mantissa and truncates, the high half of `rbits` serving b and
// the low half a.  Finite values may carry up to the next binade (and the largest one into Inf), Inf stays
// Inf, NaN becomes the canonical 0x7FFF.  One instruction per pair; ops/formats.py::bf16_round_sr states
// the same rule bit for bit.
__device__ __forceinline__ uint32_t pack2_sr_bits(float a, float b, uint32_t rbits) {
    uint32_t d;
    asm("cvt.rs.bf16x2.f32 %0, %1, %2, %3;" : "=r"(d) : "f"(b), "f"(a), "r"(rbits));
    return d;
}
__device__ __forceinline__ uint32_t pack2_sr(float a, float b, uint32_t ra, uint32_t rb) {
    return pack2_sr_bits(a, b, (ra & 0xFFFFu) | (rb << 16));
}
// |x0| + ... + |x7|: eight additions on the FMA pipe.  A finite sum proves that none of the elements is Inf or NaN.
__device__ __forceinline__ float sum_abs8(const float (&x)[8]) {
    return ((fabsf(x[0]) + fabsf(x[1])) + (fabsf(x[2]) + fabsf(x[3]))) + ((fabsf(x[4]) + fabsf(x[5])) + (fabsf(x[6]) + fabsf(x[7])));
}

__device__ __forceinline__ uint32_t pack2_rn(float a, float b) {
    const __nv_bfloat162 h = __floats2bfloat162_rn(a, b);
    return *reinterpret_cast<const uint32_t*>(&h);
}

// ---------------------------------------------------------------------------
// general 8-wide loads and stores (any dtype, any alignment, ragged tail)
// ---------------------------------------------------------------------------

__device__ __forceinline__ bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

// two fp32 -> one word of two fp16 (a in the low half), stochastic rounding by the conversion unit: the low 13 of each
// half of `rbits` are added below the kept mantissa (sub-normal results take their step from the same 13 bits), values
// beyond +-65504 saturate, NaN becomes 0x7FFF.  ops/formats.py::fp16_round_sr states the same rule.
__device__ __forceinline__ uint32_t pack2_f16_sr_bits(float a, float b, uint32_t rbits) {
    uint32_t d;
    asm("cvt.rs.satfinite.f16x2.f32 %0, %1, %2, %3;" : "=r"(d) : "f"(b), "f"(a), "r"(rbits));
    return d;
}
__device__ __forceinline__ uint32_t pack2_f16_rn(float a, float b) {
    const __half2 h = __floats2half2_rn(fminf(fmaxf(a, -65504.0f), 65504.0f), fminf(fmaxf(b, -65504.0f), 65504.0f));
    return *reinterpret_cast<const uint32_t*>(&h);
}
__device__ __forceinline__ float f16_bits_to_float(uint16_t bits) {
    return __half2float(__ushort_as_half(bits));
}

__device__ __forceinline__ void load8(const void* base, int dt, long long idx, int nvalid, float (&out)[8]) {
    if (dt == DT_F16) {
        const uint16_t* p = reinterpret_cast<const uint16_t*>(base) + idx;
        if (nvalid == 8 && aligned16(p)) {
            const uint4 r = __ldcs(reinterpret_cast<const uint4*>(p));
            const uint32_t w[4] = {r.x, r.y, r.z, r.w};
#pragma unroll
            for (int k = 0; k < 4; ++k) {
                const float2 f = __half22float2(*reinterpret_cast<const __half2*>(&w[k]));
                out[2 * k] = f.x; out[2 * k + 1] = f.y;
            }
        } else {
#pragma unroll
            for (int k = 0; k < 8; ++k) out[k] = (k < nvalid) ? f16_bits_to_float(p[k]) : 0.0f;
        }
    } else if (dt == DT_BF16) {
        const uint16_t* p = reinterpret_cast<const uint16_t*>(base) + idx;
        if (nvalid == 8 && aligned16(p)) {
            unpack8(__ldcs(reinterpret_cast<const uint4*>(p)), out);
        } else {
#pragma unroll
            for (int k = 0; k < 8; ++k) out[k] = (k < nvalid) ? bf16_bits_to_float(p[k]) : 0.0f;
        }
    } else {
        const float* p = reinterpret_cast<const float*>(base) + idx;
        if (nvalid == 8 && aligned16(p)) {
            const float4 a = __ldcs(reinterpret_cast<const float4*>(p));
            const float4 b = __ldcs(reinterpret_cast<const float4*>(p) + 1);
            out[0] = a.x; out[1] = a.y; out[2] = a.z; out[3] = a.w;
            out[4] = b.x; out[5] = b.y; out[6] = b.z; out[7] = b.w;
        } else {
#pragma unroll
            for (int k = 0; k < 8; ++k) out[k] = (k < nvalid) ? p[k] : 0.0f;
        }
    }
}

// r16[k]: 16 rounding bits per element (ignored unless sr)
__device__ __forceinline__ void store8(void* base, int dt, long long idx, int nvalid, const float (&val)[8],
                                       const uint32_t (&r16)[8], bool sr) {
    if (dt == DT_BF16 || dt == DT_F16) {
        uint16_t* p = reinterpret_cast<uint16_t*>(base) + idx;
        uint32_t w[4];
#pragma unroll
        for (int k = 0; k < 4; ++k) {
            const uint32_t rbits = (r16[2 * k] & 0xFFFFu) | (r16[2 * k + 1] << 16);
            if (dt == DT_BF16) w[k] = sr ? pack2_sr_bits(val[2 * k], val[2 * k + 1], rbits) : pack2_rn(val[2 * k], val[2 * k + 1]);
            else w[k] = sr ? pack2_f16_sr_bits(val[2 * k], val[2 * k + 1], rbits) : pack2_f16_rn(val[2 * k], val[2 * k + 1]);
        }
        if (nvalid == 8 && aligned16(p)) {
            __stcs(reinterpret_cast<uint4*>(p), make_uint4(w[0], w[1], w[2], w[3]));
        } else {
#pragma unroll
            for (int k = 0; k < 8; ++k)
                if (k < nvalid) p[k] = static_cast<uint16_t>((k & 1) ? (w[k >> 1] >> 16) : (w[k >> 1] & 0xFFFFu));
        }
    } else {
        float* p = reinterpret_cast<float*>(base) + idx;
        if (nvalid == 8 && aligned16(p)) {
            __stcs(reinterpret_cast<float4*>(p), make_float4(val[0], val[1], val[2], val[3]));
            __stcs(reinterpret_cast<float4*>(p) + 1, make_float4(val[4], val[5], val[6], val[7]));
        } else {
#pragma unroll
            for (int k = 0; k < 8; ++k)
                if (k < nvalid) p[k] = val[k];
        }
    }
}

// ---------------------------------------------------------------------------
// reductions inside a group of T = block_size/8 threads (T is a power of two,
// 8 <= T <= 256, uniform over the CTA)
// ---------------------------------------------------------------------------

struct ReduceScratch {
    float a[kThreads / 32];
    float b[kThreads / 32];
    // maxima of the quantisation blocks of one chunk: three rotating sets of (block-in-chunk, moment) slots, see
    // group_max2.  Zero-initialised by the kernel before the first chunk.
    uint32_t mx[3][kThreads / 64][2];
};

// to be followed by a CTA barrier before the first chunk
__device__ __forceinline__ void init_scratch(ReduceScratch& s) {
    uint32_t* w = &s.mx[0][0][0];
    if (threadIdx.x < 3 * (kThreads / 64) * 2) w[threadIdx.x] = 0u;
}

template <bool IS_MAX>
__device__ __forceinline__ float combine(float x, float y) { return IS_MAX ? fmaxf(x, y) : (x + y); }

template <bool IS_MAX>
__device__ __forceinline__ void group_reduce2(float& a, float& b, int T, ReduceScratch& s) {
    if (IS_MAX && T >= 32) {
        // maxima of non-negative floats order like their bit patterns: one warp-wide redux.sync each instead of
        // five shuffle + max pairs
        a = __uint_as_float(__reduce_max_sync(0xFFFFFFFFu, __float_as_uint(a)));
        b = __uint_as_float(__reduce_max_sync(0xFFFFFFFFu, __float_as_uint(b)));
    } else {
        const int w = (T < 32) ? T : 32;
        for (int off = w >> 1; off > 0; off >>= 1) {
            a = combine<IS_MAX>(a, __shfl_xor_sync(0xFFFFFFFFu, a, off));
            b = combine<IS_MAX>(b, __shfl_xor_sync(0xFFFFFFFFu, b, off));
        }
    }
    if (T > 32) {
        const int warp = threadIdx.x >> 5;
        if ((threadIdx.x & 31) == 0) { s.a[warp] = a; s.b[warp] = b; }
        __syncthreads();
        const int warps_per_group = T >> 5;
        const int first = (warp / warps_per_group) * warps_per_group;
        float ra = s.a[first], rb = s.b[first];
        for (int i = 1; i < warps_per_group; ++i) {
            ra = combine<IS_MAX>(ra, s.a[first + i]);
            rb = combine<IS_MAX>(rb, s.b[first + i]);
        }
        a = ra; b = rb;
        __syncthreads();
    }
}

// Maxima of two non-negative quantities over each group of T threads (T a power of two, 8 <= T <= 256, uniform over
// the CTA), for groups wider than a warp through shared-memory atomics: one redux per warp, one atomic max per warp
// and quantity, ONE barrier, one read.  `turn` counts the calls of this CTA that took this route (uniform over the
// CTA, advanced here).  Three sets of slots rotate: a call clears the set of the next call before its barrier - every
// thread has read that set (two such calls ago) before it passed the previous call's barrier, and nobody writes it
// before this call's barrier - then publishes into its own set.
__device__ __forceinline__ void group_max2(float& a, float& b, int log2T, ReduceScratch& s, uint32_t& turn) {
    const int T = 1 << log2T;
    if (T <= 32) {
        for (int off = T >> 1; off > 0; off >>= 1) {
            a = fmaxf(a, __shfl_xor_sync(0xFFFFFFFFu, a, off));
            b = fmaxf(b, __shfl_xor_sync(0xFFFFFFFFu, b, off));
        }
        return;
    }
    const uint32_t ua = __reduce_max_sync(0xFFFFFFFFu, __float_as_uint(a));
    const uint32_t ub = __reduce_max_sync(0xFFFFFFFFu, __float_as_uint(b));
    const uint32_t set = turn;
    const uint32_t nxt = set == 2u ? 0u : set + 1u;
    turn = nxt;
    const int grp = threadIdx.x >> log2T;
    if (threadIdx.x < (kThreads / 64) * 2) (&s.mx[nxt][0][0])[threadIdx.x] = 0u;
    if ((threadIdx.x & 31) == 0) {
        atomicMax(&s.mx[set][grp][0], ua);
        atomicMax(&s.mx[set][grp][1], ub);
    }
    __syncthreads();
    a = __uint_as_float(s.mx[set][grp][0]);
    b = __uint_as_float(s.mx[set][grp][1]);
}

// ---------------------------------------------------------------------------
// IO policy of the single-GPU kernel
// ---------------------------------------------------------------------------

struct LocalIO {
    __device__ __forceinline__ void load_grad(const SegDesc& s, long long idx, int nvalid, float (&g)[8]) const {
        load8(s.g, s.g_dtype, idx, nvalid, g);
    }
    __device__ __forceinline__ void store_param(const SegDesc& s, long long idx, int nvalid, const float (&p)[8],
                                                const uint32_t (&r16)[8], bool sr) const {
        store8(s.p, s.p_dtype, idx, nvalid, p, r16, sr);
    }
    // fast path: bf16, aligned, full vector
    __device__ __forceinline__ void load_grad_fast(const SegDesc& s, long long idx, float (&g)[8]) const {
        unpack8(__ldcs(reinterpret_cast<const uint4*>(reinterpret_cast<const uint16_t*>(s.g) + idx)), g);
    }
    __device__ __forceinline__ void store_param_fast(const SegDesc& s, long long idx, const uint4& packed) const {
        __stcs(reinterpret_cast<uint4*>(reinterpret_cast<uint16_t*>(s.p) + idx), packed);
    }
};

// ---------------------------------------------------------------------------
// the arithmetic, shared by both paths
// ---------------------------------------------------------------------------

// gradient front end + first moment; g becomes the prepared gradient, p the decayed
// parameter, m the updated first moment
// g_finite: the caller has shown that none of the eight gradients is Inf or NaN (sanitising is then the identity)
// plain: the step's flags are the common set (stochastic rounding only), known at compile time in the caller
// decay_mask: bit k set = element k gets the decoupled weight decay (0xFF / 0 for whole vectors: the compiler folds
// the tests when the caller passes a uniform constant pair through `decay ? 0xFFu : 0u` of a hoisted bool)
template <bool PER_ELEMENT = false>
__device__ __forceinline__ void front8(const StepArgs& a, uint32_t decay_mask, float (&p)[8], float (&g)[8], float (&m)[8],
                                       bool g_finite = false, bool plain = false) {
    const bool maximize = plain ? false : (a.flags & STEP_MAXIMIZE) != 0;
    if (!g_finite) {
#pragma unroll
        for (int k = 0; k < 8; ++k) g[k] = sanitize_grad(g[k]);
    }
#pragma unroll
    for (int k = 0; k < 8; ++k) {
        float gk = g[k];
        if (maximize) gk = -gk;
        gk = gk * a.inv_scale;
        g[k] = gk;
        if (PER_ELEMENT ? ((decay_mask >> k) & 1u) != 0 : decay_mask != 0) p[k] = p[k] * a.decay_factor;
        m[k] = fmaf(m[k], a.beta1, gk * a.omb1);
    }
}

// shared variance of one group of four; returns the update multiplier step_size / den
__device__ __forceinline__ float quad_variance(const StepArgs& a, const float* g4, float& v, float eps_add, float eps_floor) {
    float acc = g4[0] * g4[0];
    acc = fmaf(g4[1], g4[1], acc);
    acc = fmaf(g4[2], g4[2], acc);
    acc = fmaf(g4[3], g4[3], acc);
    float vn = fmaf(v, a.beta2, acc * a.omb2_quarter);
    if (!(fabsf(vn) < INFINITY)) vn = 0.0f;
    v = vn;
    const float den = fmaxf(fast_sqrt(fmaxf(vn, 0.0f)) + eps_add, eps_floor);
    return fast_rcp(den) * a.step_size;
}

__device__ __forceinline__ float elem_variance(const StepArgs& a, float g, float& v, float eps_add, float eps_floor,
                                               bool zero_nonfinite) {
    float vn = fmaf(v, a.beta2, (g * g) * a.omb2);
    if (zero_nonfinite && !(fabsf(vn) < INFINITY)) vn = 0.0f;
    v = vn;
    const float den = fmaxf(fast_sqrt(fmaxf(vn, 0.0f)) + eps_add, eps_floor);
    return fast_rcp(den) * a.step_size;
}

// The same two for a second moment that is stored times `vs` = 4^k (fp16 storage, kept in range by a per-tensor scale):
// the increment is scaled on the way in and the root by `irs` = 2^-k on the way out.  With k = 0 these reduce to the
// functions above bit for bit (multiplications by one).
__device__ __forceinline__ float quad_variance_scaled(const StepArgs& a, const float* g4, float& v, float vs, float irs) {
    float acc = g4[0] * g4[0];
    acc = fmaf(g4[1], g4[1], acc);
    acc = fmaf(g4[2], g4[2], acc);
    acc = fmaf(g4[3], g4[3], acc);
    float vn = fmaf(v, a.beta2, acc * (a.omb2_quarter * vs));
    if (!(fabsf(vn) < INFINITY)) vn = 0.0f;
    v = vn;
    return fast_rcp(fast_sqrt(fmaxf(vn, 0.0f)) * irs + a.eps_scaled) * a.step_size;
}
__device__ __forceinline__ float elem_variance_scaled(const StepArgs& a, float g, float& v, float vs, float irs) {
    const float vn = fmaf(v, a.beta2, (g * g) * (a.omb2 * vs));
    v = vn;
    return fast_rcp(fast_sqrt(fmaxf(vn, 0.0f)) * irs + a.eps_scaled) * a.step_size;
}

// ---------------------------------------------------------------------------
// dense moments (fp32 / bf16 / fp16), optionally one variance per four elements
// ---------------------------------------------------------------------------

// fast path: p, g, m, v all bf16; everything aligned; all 8 elements valid
// PLAIN: flags == STEP_STOCHASTIC exactly (no Nesterov / maximize / cautious), folded at compile time; the caller
// picks the instantiation with one uniform branch per chunk, which removes the per-element flag tests.
template <bool QUAD, bool PLAIN, class IO>
__device__ __forceinline__ void dense_fast(const SegDesc& s, const StepArgs& a, uint32_t chunk, const IO& io, bool decay) {
    const long long idx = static_cast<long long>(chunk) * kChunk + threadIdx.x * kPerThread;
    const bool sr = PLAIN ? true : (a.flags & STEP_STOCHASTIC) != 0;
    const uint4 praw = __ldcs(reinterpret_cast<const uint4*>(reinterpret_cast<const uint16_t*>(s.p) + idx));
    const uint4 mraw = __ldcs(reinterpret_cast<const uint4*>(reinterpret_cast<const uint16_t*>(s.m) + idx));
    float p[8], g[8], m[8], inv[8];
    io.load_grad_fast(s, idx, g);
    uint4 vraw4 = make_uint4(0, 0, 0, 0);
    uint32_t vraw2 = 0;
    if (QUAD) vraw2 = __ldcs(reinterpret_cast<const uint32_t*>(reinterpret_cast<const uint16_t*>(s.v) + (idx >> 2)));
    else vraw4 = __ldcs(reinterpret_cast<const uint4*>(reinterpret_cast<const uint16_t*>(s.v) + idx));
    unpack8(praw, p);
    unpack8(mraw, m);
    front8(a, decay ? 0xFFu : 0u, p, g, m, sum_abs8(g) < INFINITY, PLAIN);

    uint32_t word[8];
    uint32_t state = thread_state(chunk_key(a.step_key, s.salt, chunk), threadIdx.x);
#pragma unroll
    for (int k = 0; k < 8; ++k) word[k] = next_word(state);

    if (QUAD) {
        float v0 = lo_bf16(vraw2), v1 = hi_bf16(vraw2);
        const float i0 = quad_variance(a, g, v0, a.eps_scaled, 0.0f);
        const float i1 = quad_variance(a, g + 4, v1, a.eps_scaled, 0.0f);
#pragma unroll
        for (int k = 0; k < 4; ++k) { inv[k] = i0; inv[4 + k] = i1; }
        const uint32_t vw = sr ? pack2_sr(v0, v1, second_word(word[0]) & 0xFFFFu, second_word(word[4]) & 0xFFFFu)
                               : pack2_rn(v0, v1);
        __stcs(reinterpret_cast<uint32_t*>(reinterpret_cast<uint16_t*>(s.v) + (idx >> 2)), vw);
    } else {
        float v[8];
        unpack8(vraw4, v);
#pragma unroll
        for (int k = 0; k < 8; ++k) inv[k] = elem_variance(a, g[k], v[k], a.eps_scaled, 0.0f, false);
        uint32_t w[4];
#pragma unroll
        for (int k = 0; k < 4; ++k)
            w[k] = sr ? pack2_sr(v[2 * k], v[2 * k + 1], second_word(word[2 * k]) & 0xFFFFu, second_word(word[2 * k + 1]) & 0xFFFFu)
                      : pack2_rn(v[2 * k], v[2 * k + 1]);
        __stcs(reinterpret_cast<uint4*>(reinterpret_cast<uint16_t*>(s.v) + idx), make_uint4(w[0], w[1], w[2], w[3]));
    }
    const bool nesterov = PLAIN ? false : (a.flags & STEP_NESTEROV) != 0;
#pragma unroll
    for (int k = 0; k < 8; ++k) {
        const float num = nesterov ? fmaf(m[k], a.beta1, g[k] * a.omb1) : m[k];
        p[k] = fmaf(-num, inv[k], p[k]);
    }
    uint32_t pw[4], mw[4];
#pragma unroll
    for (int k = 0; k < 4; ++k) {
        if (sr) {   // low halves of the two words round the parameters, high halves the first moments
            pw[k] = pack2_sr_bits(p[2 * k], p[2 * k + 1], __byte_perm(word[2 * k], word[2 * k + 1], 0x5410));
            mw[k] = pack2_sr_bits(m[2 * k], m[2 * k + 1], __byte_perm(word[2 * k], word[2 * k + 1], 0x7632));
        } else {
            pw[k] = pack2_rn(p[2 * k], p[2 * k + 1]);
            mw[k] = pack2_rn(m[2 * k], m[2 * k + 1]);
        }
    }
    io.store_param_fast(s, idx, make_uint4(pw[0], pw[1], pw[2], pw[3]));
    __stcs(reinterpret_cast<uint4*>(reinterpret_cast<uint16_t*>(s.m) + idx), make_uint4(mw[0], mw[1], mw[2], mw[3]));
}

// CAUTIOUS: components of the update that oppose the gradient are dropped and the rest is multiplied by `inv_keep`,
// the reciprocal of the kept fraction of the whole tensor (counted by `dense_keep_count` in a pass of its own)
template <bool QUAD, class IO, bool CAUTIOUS = false>
__device__ __forceinline__ void dense_general(const SegDesc& s, const StepArgs& a, uint32_t chunk, const IO& io,
                                              uint32_t decay_mask, float inv_keep = 1.0f) {
    const long long idx = static_cast<long long>(chunk) * kChunk + threadIdx.x * kPerThread;
    const long long left = s.numel - idx;
    const int nvalid = left >= 8 ? 8 : (left > 0 ? static_cast<int>(left) : 0);
    if (nvalid == 0) return;
    const bool sr = (a.flags & STEP_STOCHASTIC) != 0;
    float p[8], g[8], m[8], inv[8];
    load8(s.p, s.p_dtype, idx, nvalid, p);
    io.load_grad(s, idx, nvalid, g);
    load8(s.m, s.m_fmt, idx, nvalid, m);

    uint32_t word[8];
    uint32_t state = thread_state(chunk_key(a.step_key, s.salt, chunk), threadIdx.x);
#pragma unroll
    for (int k = 0; k < 8; ++k) word[k] = next_word(state);

    front8<true>(a, decay_mask, p, g, m);
    // fp16 second moments carry a per-tensor scale 4^k (k = 0 for every other format)
    const float vs = __uint_as_float((127u + 2u * s.v_scale_log4) << 23);
    const float irs = __uint_as_float((127u - s.v_scale_log4) << 23);
    if (QUAD) {
        // numel % 4 == 0 is guaranteed by the host for shared-variance segments
        const long long qidx = idx >> 2;
        const int nq = nvalid >> 2;
        float vq[2] = {0.f, 0.f};
#pragma unroll
        for (int q = 0; q < 2; ++q) {
            if (q < nq) {
                const uint16_t* v16 = reinterpret_cast<const uint16_t*>(s.v);
                vq[q] = (s.v_fmt == V_BF16) ? bf16_bits_to_float(v16[qidx + q])
                      : (s.v_fmt == V_F16) ? f16_bits_to_float(v16[qidx + q])
                                           : reinterpret_cast<const float*>(s.v)[qidx + q];
            }
            const float iv = quad_variance_scaled(a, g + 4 * q, vq[q], vs, irs);
#pragma unroll
            for (int k = 0; k < 4; ++k) inv[4 * q + k] = iv;
            if (q < nq) {
                const uint32_t rb = second_word(word[4 * q]) & 0xFFFFu;
                if (s.v_fmt == V_BF16) {
                    const uint32_t w = sr ? pack2_sr(vq[q], 0.0f, rb, 0u) : pack2_rn(vq[q], 0.0f);
                    reinterpret_cast<uint16_t*>(s.v)[qidx + q] = static_cast<uint16_t>(w & 0xFFFFu);
                } else if (s.v_fmt == V_F16) {
                    const uint32_t w = sr ? pack2_f16_sr_bits(vq[q], 0.0f, rb) : pack2_f16_rn(vq[q], 0.0f);
                    reinterpret_cast<uint16_t*>(s.v)[qidx + q] = static_cast<uint16_t>(w & 0xFFFFu);
                } else {
                    reinterpret_cast<float*>(s.v)[qidx + q] = vq[q];
                }
            }
        }
    } else {
        float v[8];
        uint32_t vbits[8];
        load8(s.v, s.v_fmt, idx, nvalid, v);
#pragma unroll
        for (int k = 0; k < 8; ++k) {
            inv[k] = elem_variance_scaled(a, g[k], v[k], vs, irs);
            vbits[k] = second_word(word[k]) & 0xFFFFu;
        }
        store8(s.v, s.v_fmt, idx, nvalid, v, vbits, sr);
    }
    const bool nesterov = (a.flags & STEP_NESTEROV) != 0;
    uint32_t pbits[8], mbits[8];
#pragma unroll
    for (int k = 0; k < 8; ++k) {
        float num = nesterov ? fmaf(m[k], a.beta1, g[k] * a.omb1) : m[k];
        if (CAUTIOUS) num = (m[k] * g[k] >= 0.0f) ? m[k] * inv_keep : 0.0f;
        p[k] = fmaf(-num, inv[k], p[k]);
        pbits[k] = word[k] & 0xFFFFu;
        mbits[k] = word[k] >> 16;
    }
    io.store_param(s, idx, nvalid, p, pbits, sr);
    store8(s.m, s.m_fmt, idx, nvalid, m, mbits, sr);
}

// How many of this thread's eight elements a cautious update keeps: the new first moment (not stored here) agrees in
// sign with the gradient.  Same arithmetic as `front8`, so that the count matches what the update pass then does.
template <class IO>
__device__ __forceinline__ uint32_t dense_keep_count(const SegDesc& s, const StepArgs& a, uint32_t chunk, const IO& io) {
    const long long idx = static_cast<long long>(chunk) * kChunk + threadIdx.x * kPerThread;
    const long long left = s.numel - idx;
    const int nvalid = left >= 8 ? 8 : (left > 0 ? static_cast<int>(left) : 0);
    if (nvalid == 0) return 0u;
    float g[8], m[8];
    io.load_grad(s, idx, nvalid, g);
    load8(s.m, s.m_fmt, idx, nvalid, m);
    uint32_t kept = 0;
#pragma unroll
    for (int k = 0; k < 8; ++k) {
        float gk = sanitize_grad(g[k]);
        if (a.flags & STEP_MAXIMIZE) gk = -gk;
        gk = gk * a.inv_scale;
        const float mk = fmaf(m[k], a.beta1, gk * a.omb1);
        kept += (k < nvalid && mk * gk >= 0.0f) ? 1u : 0u;
    }
    return kept;
}

// Lion, AdEMAMix (a second, slow first moment) and AMSGrad (running maximum of the second moment) on per-element
// dense state.  A kernel instantiation of its own runs it, so that the registers of these rarely used branches stay
// out of the common paths.
template <class IO>
__device__ __forceinline__ void dense_exotic(const SegDesc& s, const StepArgs& a, uint32_t chunk, const IO& io,
                                              uint32_t decay_mask) {
    const long long idx = static_cast<long long>(chunk) * kChunk + threadIdx.x * kPerThread;
    const long long left = s.numel - idx;
    const int nvalid = left >= 8 ? 8 : (left > 0 ? static_cast<int>(left) : 0);
    if (nvalid == 0) return;
    const bool sr = (a.flags & STEP_STOCHASTIC) != 0;
    float p[8], g[8], m[8], inv[8];
    load8(s.p, s.p_dtype, idx, nvalid, p);
    io.load_grad(s, idx, nvalid, g);
    load8(s.m, s.m_fmt, idx, nvalid, m);

    uint32_t word[8];
    uint32_t state = thread_state(chunk_key(a.step_key, s.salt, chunk), threadIdx.x);
#pragma unroll
    for (int k = 0; k < 8; ++k) word[k] = next_word(state);

    if (a.flags & STEP_LION) {
        // Lion: p <- p * decay - lr * sign(beta1 m + (1 - beta1) g);  m <- beta2 m + (1 - beta2) g;  no second moment
        uint32_t pb[8], mb[8];
#pragma unroll
        for (int k = 0; k < 8; ++k) {
            float gk = sanitize_grad(g[k]);
            if (a.flags & STEP_MAXIMIZE) gk = -gk;
            gk = gk * a.inv_scale;
            if ((decay_mask >> k) & 1u) p[k] = p[k] * a.decay_factor;
            const float c = fmaf(m[k], a.beta1, gk * a.omb1);
            const float u = c > 0.0f ? 1.0f : (c < 0.0f ? -1.0f : 0.0f);
            p[k] = p[k] - u * a.lr;
            m[k] = fmaf(m[k], a.beta2, gk * a.omb2);
            pb[k] = word[k] & 0xFFFFu;
            mb[k] = word[k] >> 16;
        }
        io.store_param(s, idx, nvalid, p, pb, sr);
        store8(s.m, s.m_fmt, idx, nvalid, m, mb, sr);
        return;
    }
    front8<true>(a, decay_mask, p, g, m);
    float ms[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
    if (a.flags & STEP_SLOW) {          // AdEMAMix: the slow momentum lives in the m_scale slot, in m's format
        load8(s.m_scale, s.m_fmt, idx, nvalid, ms);
#pragma unroll
        for (int k = 0; k < 8; ++k) ms[k] = fmaf(ms[k], a.beta3, g[k] * a.omb3);
    }

    // fp16 second moments carry a per-tensor scale 4^k (k = 0 for every other format)
    const float vs = __uint_as_float((127u + 2u * s.v_scale_log4) << 23);
    const float irs = __uint_as_float((127u - s.v_scale_log4) << 23);
    {
        float v[8];
        uint32_t vbits[8];
        load8(s.v, s.v_fmt, idx, nvalid, v);
#pragma unroll
        for (int k = 0; k < 8; ++k) {
            inv[k] = elem_variance_scaled(a, g[k], v[k], vs, irs);
            vbits[k] = second_word(word[k]) & 0xFFFFu;
        }
        store8(s.v, s.v_fmt, idx, nvalid, v, vbits, sr);
        if (a.flags & STEP_AMSGRAD) {   // running maximum of v in the v_scale slot (v's format, round to nearest)
            float mx[8];
            load8(s.v_scale, s.v_fmt, idx, nvalid, mx);
#pragma unroll
            for (int k = 0; k < 8; ++k) {
                mx[k] = fmaxf(mx[k], v[k]);
                inv[k] = fast_rcp(fast_sqrt(fmaxf(mx[k], 0.0f)) * irs + a.eps_scaled) * a.step_size;
            }
            store8(s.v_scale, s.v_fmt, idx, nvalid, mx, vbits, false);
        }
    }
    const bool nesterov = (a.flags & STEP_NESTEROV) != 0;
    uint32_t pbits[8], mbits[8];
#pragma unroll
    for (int k = 0; k < 8; ++k) {
        float num = nesterov ? fmaf(m[k], a.beta1, g[k] * a.omb1) : m[k];
        if (a.flags & STEP_SLOW) num = m[k] + ms[k] * a.slow_ratio;
        p[k] = fmaf(-num, inv[k], p[k]);
        pbits[k] = word[k] & 0xFFFFu;
        mbits[k] = word[k] >> 16;
    }
    io.store_param(s, idx, nvalid, p, pbits, sr);
    store8(s.m, s.m_fmt, idx, nvalid, m, mbits, sr);
    if (a.flags & STEP_SLOW) store8(s.m_scale, s.m_fmt, idx, nvalid, ms, mbits, sr);
}

// How one chunk decays.  sel: kDecayByFlag (the segment's SEG_DECAY flag decides), 0 (nothing), 1 (everything) or
// k >= 2 (mixed chunk: bit mask number k - 2 of `masks`, one byte per thread).  Mixed chunks take the general path.
struct ChunkDecay {
    uint32_t sel;
    const uint8_t* masks;
    __device__ __forceinline__ bool mixed() const { return sel != kDecayByFlag && sel >= 2u; }
    __device__ __forceinline__ bool uniform(const SegDesc& s) const {
        return sel == kDecayByFlag ? (s.flags & SEG_DECAY) != 0 : sel == 1u;
    }
    __device__ __forceinline__ uint32_t mask8(const SegDesc& s) const {
        if (mixed()) return masks[static_cast<size_t>(sel - 2u) * (kChunk / 8) + threadIdx.x];
        return uniform(s) ? 0xFFu : 0u;
    }
};
__device__ __forceinline__ ChunkDecay decay_by_flag() { return ChunkDecay{kDecayByFlag, nullptr}; }

template <bool QUAD, class IO>
__device__ __forceinline__ void dense_chunk(const SegDesc& s, const StepArgs& a, uint32_t chunk, const IO& io,
                                            const ChunkDecay& dec = decay_by_flag()) {
    const bool full = (static_cast<long long>(chunk) + 1) * kChunk <= s.numel;
    if ((s.flags & SEG_FAST) && full && !dec.mixed()) {
        const bool decay = dec.uniform(s);
        if (a.flags == STEP_STOCHASTIC) dense_fast<QUAD, true>(s, a, chunk, io, decay);
        else dense_fast<QUAD, false>(s, a, chunk, io, decay);
    }
    else dense_general<QUAD>(s, a, chunk, io, dec.mask8(s));
}

// ---------------------------------------------------------------------------
// quantised moments: NF4 or int8 first moment, log-uint8 second moment
// ---------------------------------------------------------------------------

// update direction for the quantised formats (lookahead with gain, Nesterov, or cautious)
__device__ __forceinline__ void quant_direction(const StepArgs& a, const float (&m)[8], const float (&g)[8], int nvalid,
                                                float (&num)[8], float& kept, float& counted, bool plain = false) {
    const bool cautious = plain ? false : (a.flags & STEP_CAUTIOUS) != 0;
    const bool nesterov = plain ? false : (a.flags & STEP_NESTEROV) != 0;
#pragma unroll
    for (int k = 0; k < 8; ++k) {
        const bool agree = (m[k] * g[k] >= 0.0f);
        if (cautious) {
            num[k] = agree ? m[k] : 0.0f;
            if (k < nvalid) { counted += 1.0f; kept += agree ? 1.0f : 0.0f; }
        } else {
            const float look = fmaf(m[k], a.beta1, g[k] * a.omb1);
            num[k] = nesterov ? look : look * (agree ? a.gain_hi : a.gain_lo);
        }
    }
}

template <bool NF4, bool QUAD, bool FAST, bool PLAIN, class IO>
__device__ __forceinline__ void quant_body(const SegDesc& s, const StepArgs& a, uint32_t chunk, const IO& io,
                                           const CodecTables& tab, ReduceScratch& scratch, uint32_t& turn, uint32_t decay_mask) {
    const long long idx = static_cast<long long>(chunk) * kChunk + threadIdx.x * kPerThread;
    const long long left = s.numel - idx;
    const int nvalid = FAST ? 8 : (left >= 8 ? 8 : (left > 0 ? static_cast<int>(left) : 0));
    const bool sr = PLAIN ? true : (a.flags & STEP_STOCHASTIC) != 0;
    const bool cautious = PLAIN ? false : (a.flags & STEP_CAUTIOUS) != 0;
    const int T = 1 << (s.bs_log2 - 3);
    const long long blk = idx >> s.bs_log2;
    const bool blk_ok = FAST || (nvalid > 0);

    float p[8], g[8], m[8], v[8];
    const float sm_old = blk_ok ? s.m_scale[blk] : 1.0f;
    const float sv_old = blk_ok ? s.v_scale[blk] : 1.0f;

#pragma unroll
    for (int k = 0; k < 8; ++k) { p[k] = 0.f; g[k] = 0.f; m[k] = 0.f; v[k] = 0.f; }
    if (FAST) {
        const uint4 praw = __ldcs(reinterpret_cast<const uint4*>(reinterpret_cast<const uint16_t*>(s.p) + idx));
        io.load_grad_fast(s, idx, g);
        unpack8(praw, p);
    } else if (nvalid > 0) {
        load8(s.p, s.p_dtype, idx, nvalid, p);
        io.load_grad(s, idx, nvalid, g);
    }
    // ---- first moment decode
    if (NF4) {
        const uint8_t* mp = reinterpret_cast<const uint8_t*>(s.m) + (idx >> 1);
        uint32_t raw = 0x77777777u;
        if (FAST || (nvalid == 8 && (reinterpret_cast<uintptr_t>(mp) & 3u) == 0)) {
            raw = __ldcs(reinterpret_cast<const uint32_t*>(mp));
        } else {
            const int nb = (nvalid + 1) >> 1;
#pragma unroll
            for (int b = 0; b < 4; ++b)
                if (b < nb) raw = (raw & ~(0xFFu << (8 * b))) | (static_cast<uint32_t>(mp[b]) << (8 * b));
        }
#pragma unroll
        for (int b = 0; b < 4; ++b) {       // one 8-byte table read per packed byte instead of two index computations
            const float2 pair = tab.nf4_pair[__byte_perm(raw, 0u, 0x4440u + b)];
            m[2 * b] = pair.x * sm_old;
            m[2 * b + 1] = pair.y * sm_old;
        }
    } else {
        const int8_t* mp = reinterpret_cast<const int8_t*>(s.m) + idx;
        if (nvalid == 8 && (reinterpret_cast<uintptr_t>(mp) & 7u) == 0) {
            const uint2 raw = __ldcs(reinterpret_cast<const uint2*>(mp));
#pragma unroll
            for (int k = 0; k < 4; ++k) {
                m[k] = static_cast<float>(static_cast<int8_t>((raw.x >> (8 * k)) & 0xFFu)) * sm_old;
                m[4 + k] = static_cast<float>(static_cast<int8_t>((raw.y >> (8 * k)) & 0xFFu)) * sm_old;
            }
        } else {
#pragma unroll
            for (int k = 0; k < 8; ++k) m[k] = (k < nvalid) ? static_cast<float>(mp[k]) * sm_old : 0.0f;
        }
    }
    // ---- second moment decode
    const uint8_t* vbase = reinterpret_cast<const uint8_t*>(s.v);
    if (QUAD) {
        const uint8_t* vp = vbase + (idx >> 2);
        uint32_t codes = 0;
        if (FAST) {
            codes = __ldcs(reinterpret_cast<const uint16_t*>(vp));
        } else {
            const int nq = nvalid >> 2;
            if (nq > 0) codes = vp[0];
            if (nq > 1) codes |= static_cast<uint32_t>(vp[1]) << 8;
        }
        v[0] = tab.logv[codes & 0xFFu] * sv_old;
        v[4] = tab.logv[(codes >> 8) & 0xFFu] * sv_old;
    } else {
        const uint8_t* vp = vbase + idx;
        if (nvalid == 8 && (reinterpret_cast<uintptr_t>(vp) & 7u) == 0) {
            const uint2 raw = __ldcs(reinterpret_cast<const uint2*>(vp));
#pragma unroll
            for (int k = 0; k < 4; ++k) {
                v[k] = tab.logv[(raw.x >> (8 * k)) & 0xFFu] * sv_old;
                v[4 + k] = tab.logv[(raw.y >> (8 * k)) & 0xFFu] * sv_old;
            }
        } else {
#pragma unroll
            for (int k = 0; k < 8; ++k) v[k] = (k < nvalid) ? tab.logv[vp[k]] * sv_old : 0.0f;
        }
    }

    uint32_t word[8];
    uint32_t state = thread_state(chunk_key(a.step_key, s.salt, chunk), threadIdx.x);
#pragma unroll
    for (int k = 0; k < 8; ++k) word[k] = next_word(state);

    front8<!FAST>(a, decay_mask, p, g, m, FAST && (sum_abs8(g) < INFINITY), PLAIN);
    float max_m = 0.0f, max_v = 0.0f;
#pragma unroll
    for (int k = 0; k < 8; ++k)
        if (k < nvalid) max_m = fmaxf(max_m, fabsf(m[k]));

    float inv[8];
    if (QUAD) {
        const float i0 = quad_variance(a, g, v[0], a.eps_quad_scaled, a.eps_quad);
        const float i1 = quad_variance(a, g + 4, v[4], a.eps_quad_scaled, a.eps_quad);
#pragma unroll
        for (int k = 0; k < 4; ++k) { inv[k] = i0; inv[4 + k] = i1; }
        if (nvalid > 0) max_v = v[0];
        if (nvalid > 4) max_v = fmaxf(max_v, v[4]);
    } else {
#pragma unroll
        for (int k = 0; k < 8; ++k) {
            inv[k] = elem_variance(a, g[k], v[k], a.eps_scaled, a.eps, true);
            if (k < nvalid) max_v = fmaxf(max_v, v[k]);
        }
    }

    float num[8];
    float kept = 0.0f, counted = 0.0f;
    quant_direction(a, m, g, nvalid, num, kept, counted, PLAIN);
    if (cautious) {
        group_reduce2<false>(kept, counted, T, scratch);
        const float scale = 1.0f / fmaxf(kept / fmaxf(counted, 1.0f), 1e-3f);
#pragma unroll
        for (int k = 0; k < 8; ++k) num[k] = num[k] * scale;
    }
    group_max2(max_m, max_v, s.bs_log2 - 3, scratch, turn);

    const float sm_new = fmaxf(fmaxf(NF4 ? max_m : (max_m / 127.0f), sm_old * 0.9f), 1e-12f);
    const float sv_new = fmaxf(fmaxf(max_v, sv_old * 0.95f), 1e-12f);
    const float inv_sm = 1.0f / sm_new;
    const float inv_sv = 1.0f / sv_new;
    if (!FAST && nvalid == 0) return;

    // ---- parameter
#pragma unroll
    for (int k = 0; k < 8; ++k) p[k] = fmaf(-num[k], inv[k], p[k]);
    if (FAST) {
        uint32_t pw[4];
#pragma unroll
        for (int k = 0; k < 4; ++k)
            pw[k] = sr ? pack2_sr_bits(p[2 * k], p[2 * k + 1], __byte_perm(word[2 * k], word[2 * k + 1], 0x5410))
                       : pack2_rn(p[2 * k], p[2 * k + 1]);
        io.store_param_fast(s, idx, make_uint4(pw[0], pw[1], pw[2], pw[3]));
    } else {
        uint32_t pbits[8];
#pragma unroll
        for (int k = 0; k < 8; ++k) pbits[k] = word[k] & 0xFFFFu;
        io.store_param(s, idx, nvalid, p, pbits, sr);
    }

    // ---- first moment encode
    if (NF4) {
        uint32_t pr[4];
#pragma unroll
        for (int q = 0; q < 4; ++q) {
            // |m| <= sm_new, so |x| <= 1 up to one rounding; nf4_encode_pair clamps the magnitude in half precision
            const float x0 = m[2 * q] * inv_sm;
            const float x1 = m[2 * q + 1] * inv_sm;
            pr[q] = nf4_encode_pair(x0, x1, __byte_perm(word[2 * q], word[2 * q + 1], 0x7632), sr);
            if (!FAST) {
                if (2 * q >= nvalid) pr[q] = (pr[q] & 0xFFFF0000u) | 7u;
                if (2 * q + 1 >= nvalid) pr[q] = (pr[q] & 0x0000FFFFu) | (7u << 16);
            }
        }
        // pr[q] holds the code of element 2q in bits 0-3 and of element 2q+1 in bits 16-19; a byte of the packed
        // format is (even element << 4) | odd element.  Multiply-adds stand in for shift-and-or (no bits overlap).
        const uint32_t a01 = pr[1] * 256u + pr[0];                 // codes of elements 0, 2, 1, 3 in the low nibbles of bytes 0..3
        const uint32_t a23 = pr[3] * 256u + pr[2];
        const uint32_t b01 = a01 * 16u + (a01 >> 16);               // bytes 0, 1: (e0 << 4) | e1, (e2 << 4) | e3
        const uint32_t b23 = a23 * 16u + (a23 >> 16);
        const uint32_t packed = __byte_perm(b01, b23, 0x5410);
        uint8_t* mp = reinterpret_cast<uint8_t*>(s.m) + (idx >> 1);
        if (FAST || (nvalid == 8 && (reinterpret_cast<uintptr_t>(mp) & 3u) == 0)) {
            __stcs(reinterpret_cast<uint32_t*>(mp), packed);
        } else {
            const int nb = (nvalid + 1) >> 1;
#pragma unroll
            for (int b = 0; b < 4; ++b)
                if (b < nb) mp[b] = static_cast<uint8_t>((packed >> (8 * b)) & 0xFFu);
        }
    } else {
        uint32_t lo = 0, hi = 0;
#pragma unroll
        for (int k = 0; k < 8; ++k) {
            const float noise = sr ? (static_cast<float>(word[k] >> 16) * (1.0f / 65536.0f) - 0.5f) : 0.0f;
            float q = floorf((m[k] * inv_sm + 0.5f) + noise);
            q = fminf(fmaxf(q, -127.0f), 127.0f);
            const uint32_t byte = static_cast<uint32_t>(static_cast<int>(q)) & 0xFFu;
            if (k < 4) lo |= byte << (8 * k); else hi |= byte << (8 * (k - 4));
        }
        int8_t* mp = reinterpret_cast<int8_t*>(s.m) + idx;
        if (nvalid == 8 && (reinterpret_cast<uintptr_t>(mp) & 7u) == 0) {
            __stcs(reinterpret_cast<uint2*>(mp), make_uint2(lo, hi));
        } else {
#pragma unroll
            for (int k = 0; k < 8; ++k)
                if (k < nvalid) mp[k] = static_cast<int8_t>(((k < 4 ? lo >> (8 * k) : hi >> (8 * (k - 4))) & 0xFFu));
        }
    }

    // ---- second moment encode
    uint8_t* vout = reinterpret_cast<uint8_t*>(s.v);
    if (QUAD) {
        uint8_t* vp = vout + (idx >> 2);
        const float n0 = sr ? (static_cast<float>(second_word(word[0]) & 0xFFFFu) * (1.0f / 65536.0f) - 0.5f) : 0.0f;
        const float n1 = sr ? (static_cast<float>(second_word(word[4]) & 0xFFFFu) * (1.0f / 65536.0f) - 0.5f) : 0.0f;
        const uint32_t c0 = logv_encode(v[0], inv_sv, n0), c1 = logv_encode(v[4], inv_sv, n1);
        if (FAST) {
            __stcs(reinterpret_cast<uint16_t*>(vp), static_cast<uint16_t>(c0 | (c1 << 8)));
        } else {
            if (nvalid > 0) vp[0] = static_cast<uint8_t>(c0);
            if (nvalid > 4) vp[1] = static_cast<uint8_t>(c1);
        }
    } else {
        uint32_t lo = 0, hi = 0;
#pragma unroll
        for (int k = 0; k < 8; ++k) {
            const float noise = sr ? (static_cast<float>(second_word(word[k]) & 0xFFFFu) * (1.0f / 65536.0f) - 0.5f) : 0.0f;
            const uint32_t code = logv_encode(v[k], inv_sv, noise);
            if (k < 4) lo |= code << (8 * k); else hi |= code << (8 * (k - 4));
        }
        uint8_t* vp = vout + idx;
        if (nvalid == 8 && (reinterpret_cast<uintptr_t>(vp) & 7u) == 0) {
            __stcs(reinterpret_cast<uint2*>(vp), make_uint2(lo, hi));
        } else {
#pragma unroll
            for (int k = 0; k < 8; ++k)
                if (k < nvalid) vp[k] = static_cast<uint8_t>(((k < 4 ? lo >> (8 * k) : hi >> (8 * (k - 4))) & 0xFFu));
        }
    }

    if ((threadIdx.x & (T - 1)) == 0) {
        s.m_scale[blk] = sm_new;
        s.v_scale[blk] = sv_new;
    }
}

// "ultra" layout: int8 first moment with one scale per block, second moment per element in bf16 / fp16 / fp32
// (the reference's counterpart: apexw/triton_kernel.py:754-825, `_adamw_kernel_triton_8bit_m_16bit_v`).
// v <- v * beta2 + g^2 * (1 - beta2) and p <- p - num * (step_size / (sqrt(v) + eps)) are written as separate
// multiplies and adds (no fused multiply-add), which is the order of the torch engine for this layout.
template <class IO>
__device__ __forceinline__ void ultra_chunk(const SegDesc& s, const StepArgs& a, uint32_t chunk, const IO& io,
                                            ReduceScratch& scratch, uint32_t& turn, uint32_t decay_mask) {
    const long long idx = static_cast<long long>(chunk) * kChunk + threadIdx.x * kPerThread;
    const long long left = s.numel - idx;
    const int nvalid = left >= 8 ? 8 : (left > 0 ? static_cast<int>(left) : 0);
    const bool sr = (a.flags & STEP_STOCHASTIC) != 0;
    const long long blk = idx >> s.bs_log2;
    const float sm_old = nvalid > 0 ? s.m_scale[blk] : 1.0f;

    float p[8], g[8], m[8], v[8];
#pragma unroll
    for (int k = 0; k < 8; ++k) { p[k] = 0.f; g[k] = 0.f; m[k] = 0.f; v[k] = 0.f; }
    if (nvalid > 0) {
        load8(s.p, s.p_dtype, idx, nvalid, p);
        io.load_grad(s, idx, nvalid, g);
        load8(s.v, s.v_fmt, idx, nvalid, v);
        const int8_t* mp = reinterpret_cast<const int8_t*>(s.m) + idx;
        if (nvalid == 8 && (reinterpret_cast<uintptr_t>(mp) & 7u) == 0) {
            const uint2 raw = __ldcs(reinterpret_cast<const uint2*>(mp));
#pragma unroll
            for (int k = 0; k < 4; ++k) {
                m[k] = static_cast<float>(static_cast<int8_t>((raw.x >> (8 * k)) & 0xFFu)) * sm_old;
                m[4 + k] = static_cast<float>(static_cast<int8_t>((raw.y >> (8 * k)) & 0xFFu)) * sm_old;
            }
        } else {
#pragma unroll
            for (int k = 0; k < 8; ++k) m[k] = (k < nvalid) ? static_cast<float>(mp[k]) * sm_old : 0.0f;
        }
    }

    uint32_t word[8];
    uint32_t state = thread_state(chunk_key(a.step_key, s.salt, chunk), threadIdx.x);
#pragma unroll
    for (int k = 0; k < 8; ++k) word[k] = next_word(state);

    front8<true>(a, decay_mask, p, g, m);
    float max_m = 0.0f, unused = 0.0f;
    const bool nesterov = (a.flags & STEP_NESTEROV) != 0;
#pragma unroll
    for (int k = 0; k < 8; ++k) {
        if (k < nvalid) max_m = fmaxf(max_m, fabsf(m[k]));
        v[k] = v[k] * a.beta2 + (g[k] * g[k]) * a.omb2;
        const float inv = fast_rcp(fast_sqrt(fmaxf(v[k], 0.0f)) + a.eps_scaled) * a.step_size;
        const float num = nesterov ? fmaf(m[k], a.beta1, g[k] * a.omb1) : m[k];
        p[k] = p[k] - num * inv;
    }
    group_max2(max_m, unused, s.bs_log2 - 3, scratch, turn);
    if (nvalid == 0) return;
    const float sm_new = fmaxf(fmaxf(max_m / 127.0f, sm_old * 0.9f), 1e-12f);
    const float inv_sm = 1.0f / sm_new;

    uint32_t pbits[8], vbits[8];
#pragma unroll
    for (int k = 0; k < 8; ++k) { pbits[k] = word[k] & 0xFFFFu; vbits[k] = second_word(word[k]) & 0xFFFFu; }
    io.store_param(s, idx, nvalid, p, pbits, sr);
    store8(s.v, s.v_fmt, idx, nvalid, v, vbits, sr);

    uint32_t lo = 0, hi = 0;
#pragma unroll
    for (int k = 0; k < 8; ++k) {
        const float noise = sr ? (static_cast<float>(word[k] >> 16) * (1.0f / 65536.0f) - 0.5f) : 0.0f;
        float q = floorf((m[k] * inv_sm + 0.5f) + noise);
        q = fminf(fmaxf(q, -127.0f), 127.0f);
        const uint32_t byte = static_cast<uint32_t>(static_cast<int>(q)) & 0xFFu;
        if (k < 4) lo |= byte << (8 * k); else hi |= byte << (8 * (k - 4));
    }
    int8_t* mp = reinterpret_cast<int8_t*>(s.m) + idx;
    if (nvalid == 8 && (reinterpret_cast<uintptr_t>(mp) & 7u) == 0) {
        __stcs(reinterpret_cast<uint2*>(mp), make_uint2(lo, hi));
    } else {
#pragma unroll
        for (int k = 0; k < 8; ++k)
            if (k < nvalid) mp[k] = static_cast<int8_t>(((k < 4 ? lo >> (8 * k) : hi >> (8 * (k - 4))) & 0xFFu));
    }
    if ((threadIdx.x & ((1 << (s.bs_log2 - 3)) - 1)) == 0) s.m_scale[blk] = sm_new;
}

// eight int8 codes of one thread: one 8-byte access when the address allows it
__device__ __forceinline__ void load8_int8(const int8_t* mp, int nvalid, float scale, float (&m)[8]) {
    if (nvalid == 8 && (reinterpret_cast<uintptr_t>(mp) & 7u) == 0) {
        const uint2 raw = __ldcs(reinterpret_cast<const uint2*>(mp));
#pragma unroll
        for (int k = 0; k < 4; ++k) {
            m[k] = static_cast<float>(static_cast<int8_t>((raw.x >> (8 * k)) & 0xFFu)) * scale;
            m[4 + k] = static_cast<float>(static_cast<int8_t>((raw.y >> (8 * k)) & 0xFFu)) * scale;
        }
    } else {
#pragma unroll
        for (int k = 0; k < 8; ++k) m[k] = (k < nvalid) ? static_cast<float>(mp[k]) * scale : 0.0f;
    }
}
// m * inv_scale rounded to int8 codes (dither from the high halves of `word` when sr) and stored
__device__ __forceinline__ void store8_int8(int8_t* mp, int nvalid, const float (&m)[8], float inv_scale,
                                            const uint32_t (&word)[8], bool sr) {
    uint32_t lo = 0, hi = 0;
#pragma unroll
    for (int k = 0; k < 8; ++k) {
        const float noise = sr ? (static_cast<float>(word[k] >> 16) * (1.0f / 65536.0f) - 0.5f) : 0.0f;
        float q = floorf((m[k] * inv_scale + 0.5f) + noise);
        q = fminf(fmaxf(q, -127.0f), 127.0f);
        const uint32_t byte = static_cast<uint32_t>(static_cast<int>(q)) & 0xFFu;
        if (k < 4) lo |= byte << (8 * k); else hi |= byte << (8 * (k - 4));
    }
    if (nvalid == 8 && (reinterpret_cast<uintptr_t>(mp) & 7u) == 0) {
        __stcs(reinterpret_cast<uint2*>(mp), make_uint2(lo, hi));
    } else {
#pragma unroll
        for (int k = 0; k < 8; ++k)
            if (k < nvalid) mp[k] = static_cast<int8_t>(((k < 4 ? lo >> (8 * k) : hi >> (8 * (k - 4))) & 0xFFu));
    }
}

// Lion with an int8 first moment (one scale per block, no second moment; the reference has no kernel for Lion and
// runs it as torch operations, dense form at apexw/optimizer.py:1213-1225): p <- p * decay - lr * sign(beta1 m +
// (1 - beta1) g); m <- beta2 m + (1 - beta2) g, re-encoded against the block's new maximum (no carry-over of the old
// scale: the torch engine's rule for Lion).
template <class IO>
__device__ __forceinline__ void lion8_chunk(const SegDesc& s, const StepArgs& a, uint32_t chunk, const IO& io,
                                            ReduceScratch& scratch, uint32_t& turn, uint32_t decay_mask) {
    const long long idx = static_cast<long long>(chunk) * kChunk + threadIdx.x * kPerThread;
    const long long left = s.numel - idx;
    const int nvalid = left >= 8 ? 8 : (left > 0 ? static_cast<int>(left) : 0);
    const bool sr = (a.flags & STEP_STOCHASTIC) != 0;
    const long long blk = idx >> s.bs_log2;
    const float sm_old = nvalid > 0 ? s.m_scale[blk] : 1.0f;
    float p[8], g[8], m[8];
#pragma unroll
    for (int k = 0; k < 8; ++k) { p[k] = 0.f; g[k] = 0.f; m[k] = 0.f; }
    int8_t* mp = reinterpret_cast<int8_t*>(s.m) + idx;
    if (nvalid > 0) {
        load8(s.p, s.p_dtype, idx, nvalid, p);
        io.load_grad(s, idx, nvalid, g);
        load8_int8(mp, nvalid, sm_old, m);
    }
    uint32_t word[8];
    uint32_t state = thread_state(chunk_key(a.step_key, s.salt, chunk), threadIdx.x);
#pragma unroll
    for (int k = 0; k < 8; ++k) word[k] = next_word(state);
    float max_m = 0.0f, unused = 0.0f;
    uint32_t pbits[8];
#pragma unroll
    for (int k = 0; k < 8; ++k) {
        float gk = sanitize_grad(g[k]);
        if (a.flags & STEP_MAXIMIZE) gk = -gk;
        gk = gk * a.inv_scale;
        if ((decay_mask >> k) & 1u) p[k] = p[k] * a.decay_factor;
        const float c = fmaf(m[k], a.beta1, gk * a.omb1);
        const float u = c > 0.0f ? 1.0f : (c < 0.0f ? -1.0f : 0.0f);
        p[k] = p[k] - u * a.lr;
        m[k] = fmaf(m[k], a.beta2, gk * a.omb2);
        if (k < nvalid) max_m = fmaxf(max_m, fabsf(m[k]));
        pbits[k] = word[k] & 0xFFFFu;
    }
    group_max2(max_m, unused, s.bs_log2 - 3, scratch, turn);       // every thread of the CTA takes part
    if (nvalid == 0) return;
    io.store_param(s, idx, nvalid, p, pbits, sr);
    const float sm_new = fmaxf(max_m / 127.0f, 1e-12f);
    store8_int8(mp, nvalid, m, 1.0f / sm_new, word, sr);
    if ((threadIdx.x & ((1 << (s.bs_log2 - 3)) - 1)) == 0) s.m_scale[blk] = sm_new;
}

// Factored second moment (the reference's counterpart: apexw/triton_kernel.py:1722-1800 and its host driver
// `triton_factored_v_step`, :3059-3212; denominator as in apexw/state.py:300-323): the update of one chunk.  s.v points at the row factors sqrt(r_i / mean(r)) and s.v_scale
// at the column factors sqrt(c_j) that `fact_finish_kernel` left in the plan's scratch; s.offset holds the number of
// columns.  The first moment is dense (fp32 / bf16 / fp16) or int8 with one scale per block (s.m_fmt decides, uniform
// over the launch).  denominator = max(row * col + eps_scaled, eps); p <- p - num * (step_size / denominator) without
// fused multiply-add, the torch engine's order for this layout.
template <class IO>
__device__ __forceinline__ void factored_chunk(const SegDesc& s, const StepArgs& a, uint32_t chunk, const IO& io,
                                               ReduceScratch& scratch, uint32_t& turn, uint32_t decay_mask) {
    const long long idx = static_cast<long long>(chunk) * kChunk + threadIdx.x * kPerThread;
    const long long left = s.numel - idx;
    const int nvalid = left >= 8 ? 8 : (left > 0 ? static_cast<int>(left) : 0);
    const bool sr = (a.flags & STEP_STOCHASTIC) != 0;
    const bool int8m = s.m_fmt == M_INT8;
    const long long blk = int8m ? (idx >> s.bs_log2) : 0;
    const float sm_old = (int8m && nvalid > 0) ? s.m_scale[blk] : 1.0f;

    float p[8], g[8], m[8];
#pragma unroll
    for (int k = 0; k < 8; ++k) { p[k] = 0.f; g[k] = 0.f; m[k] = 0.f; }
    if (nvalid > 0) {
        load8(s.p, s.p_dtype, idx, nvalid, p);
        io.load_grad(s, idx, nvalid, g);
        if (int8m) {
            load8_int8(reinterpret_cast<const int8_t*>(s.m) + idx, nvalid, sm_old, m);
        } else {
            load8(s.m, s.m_fmt, idx, nvalid, m);
        }
    }
    uint32_t word[8];
    uint32_t state = thread_state(chunk_key(a.step_key, s.salt, chunk), threadIdx.x);
#pragma unroll
    for (int k = 0; k < 8; ++k) word[k] = next_word(state);

    front8<true>(a, decay_mask, p, g, m);

    const long long cols = s.offset;
    long long row = nvalid > 0 ? idx / cols : 0;
    long long col = nvalid > 0 ? idx - row * cols : 0;
    const float* rowf = reinterpret_cast<const float*>(s.v);
    const float* colf = s.v_scale;
    const bool nesterov = (a.flags & STEP_NESTEROV) != 0;
    float max_m = 0.0f, unused = 0.0f;
    float rf = nvalid > 0 ? rowf[row] : 1.0f;
#pragma unroll
    for (int k = 0; k < 8; ++k) {
        if (k < nvalid) {
            max_m = fmaxf(max_m, fabsf(m[k]));
            const float den = fmaxf(rf * colf[col] + a.eps_scaled, a.eps);
            const float inv = fast_rcp(den) * a.step_size;
            const float num = nesterov ? fmaf(m[k], a.beta1, g[k] * a.omb1) : m[k];
            p[k] = p[k] - num * inv;
            if (++col == cols) {                 // the eight elements may run into the next row
                col = 0; ++row;
                if (k + 1 < nvalid) rf = rowf[row];
            }
        }
    }
    uint32_t pbits[8], mbits[8];
#pragma unroll
    for (int k = 0; k < 8; ++k) { pbits[k] = word[k] & 0xFFFFu; mbits[k] = word[k] >> 16; }
    if (!int8m) {
        if (nvalid == 0) return;
        io.store_param(s, idx, nvalid, p, pbits, sr);
        store8(s.m, s.m_fmt, idx, nvalid, m, mbits, sr);
        return;
    }
    group_max2(max_m, unused, s.bs_log2 - 3, scratch, turn);       // every thread of the CTA takes part
    if (nvalid == 0) return;
    io.store_param(s, idx, nvalid, p, pbits, sr);
    const float sm_new = fmaxf(fmaxf(max_m / 127.0f, sm_old * 0.9f), 1e-12f);
    store8_int8(reinterpret_cast<int8_t*>(s.m) + idx, nvalid, m, 1.0f / sm_new, word, sr);
    if ((threadIdx.x & ((1 << (s.bs_log2 - 3)) - 1)) == 0) s.m_scale[blk] = sm_new;
}

// turn: number of quantised chunks this CTA has processed before this one (uniform over the CTA)
template <bool NF4, bool QUAD, class IO>
__device__ __forceinline__ void quant_chunk(const SegDesc& s, const StepArgs& a, uint32_t chunk, const IO& io,
                                            const CodecTables& tab, ReduceScratch& scratch, uint32_t& turn,
                                            const ChunkDecay& dec = decay_by_flag()) {
    const bool full = (static_cast<long long>(chunk) + 1) * kChunk <= s.numel;
    // the fast body exists for the flagship layout only (NF4 momentum + shared variance)
    if (NF4 && QUAD && (s.flags & SEG_FAST) && full && !dec.mixed()) {
        const uint32_t all = dec.uniform(s) ? 0xFFu : 0u;
        if (a.flags == STEP_STOCHASTIC) quant_body<NF4, QUAD, true, true>(s, a, chunk, io, tab, scratch, turn, all);
        else quant_body<NF4, QUAD, true, false>(s, a, chunk, io, tab, scratch, turn, all);
    } else {
        quant_body<NF4, QUAD, false, false>(s, a, chunk, io, tab, scratch, turn, dec.mask8(s));
    }
}

// ---------------------------------------------------------------------------
// work distribution
// ---------------------------------------------------------------------------

// segment lookup: last segment whose chunk_begin <= chunk
__device__ __forceinline__ int find_segment(const SegDesc* __restrict__ segs, int n, uint32_t chunk) {
    int lo = 0, hi = n - 1;
    while (lo < hi) {
        const int mid = (lo + hi + 1) >> 1;
        if (segs[mid].chunk_begin <= chunk) lo = mid; else hi = mid - 1;
    }
    return lo;
}

// Contiguous range of chunks owned by one CTA, walked with a running segment cursor so the
// table is searched once per CTA instead of once per chunk.
struct ChunkCursor {
    const SegDesc* segs;
    int n;
    uint32_t total;
    int si;
    uint32_t seg_end;
    SegDesc s;

    __device__ __forceinline__ void init(const SegDesc* segments, int count, uint32_t total_chunks, uint32_t first) {
        segs = segments; n = count; total = total_chunks;
        si = find_segment(segs, n, first);
        load();
    }
    __device__ __forceinline__ void load() {
        s = segs[si];
        seg_end = (si + 1 < n) ? segs[si + 1].chunk_begin : total;
    }
    __device__ __forceinline__ void seek(uint32_t chunk) {
        while (chunk >= seg_end && si + 1 < n) { ++si; load(); }
    }
};

// ---- table checks (debug mode) ----------------------------------------------------------------------------------
// With bit 1 of StepArgs::interleave set (APEXW_B200_DEBUG_BOUNDS=1 on the host) the persistent kernels validate, per
// chunk and before any access, what they are about to index with: the segment number, the chunk's place inside its
// segment, the pointers, their alignment and the quantisation block.  A chunk that fails is skipped (no access is
// made) and the first failure is recorded in a device word that the host reads after the step.
constexpr uint32_t kTuneCheckTable = 2u;
enum TableFault : uint32_t {
    TF_NONE = 0, TF_SEGMENT_INDEX = 1, TF_CHUNK_BEFORE_SEGMENT = 2, TF_CHUNK_PAST_SEGMENT = 3, TF_CHUNK_PAST_NUMEL = 4,
    TF_NULL_POINTER = 5, TF_ALIGNMENT = 6, TF_BLOCK_SIZE = 7, TF_NULL_SCALES = 8, TF_FORMAT = 9, TF_OFFSET = 10
};

__device__ __forceinline__ uint32_t float_width(int dt) { return dt == DT_F32 ? 4u : 2u; }

// quant: the class stores block-quantised moments (scales per block); need_local_grad: the gradient is read through s.g
__device__ __forceinline__ uint32_t table_fault(const SegDesc& s, int si, int nseg, uint32_t chunk, uint32_t seg_end,
                                                bool quant, bool need_local_grad) {
    if (si < 0 || si >= nseg) return TF_SEGMENT_INDEX;
    if (chunk < s.chunk_begin) return TF_CHUNK_BEFORE_SEGMENT;
    if (chunk >= seg_end) return TF_CHUNK_PAST_SEGMENT;
    if (s.numel <= 0 || static_cast<long long>(chunk - s.chunk_begin) * kChunk >= s.numel) return TF_CHUNK_PAST_NUMEL;
    if (s.offset < 0) return TF_OFFSET;
    if (s.p == nullptr || s.m == nullptr || s.v == nullptr || (need_local_grad && s.g == nullptr)) return TF_NULL_POINTER;
    if (s.p_dtype > DT_F16 || (need_local_grad && s.g_dtype > DT_F16)) return TF_FORMAT;
    if ((reinterpret_cast<uintptr_t>(s.p) & (float_width(s.p_dtype) - 1u)) != 0) return TF_ALIGNMENT;
    if (need_local_grad && (reinterpret_cast<uintptr_t>(s.g) & (float_width(s.g_dtype) - 1u)) != 0) return TF_ALIGNMENT;
    if (quant) {
        if (s.bs_log2 < 6 || s.bs_log2 > 11) return TF_BLOCK_SIZE;
        if (s.m_scale == nullptr || s.v_scale == nullptr) return TF_NULL_SCALES;
        if ((reinterpret_cast<uintptr_t>(s.m_scale) & 3u) != 0 || (reinterpret_cast<uintptr_t>(s.v_scale) & 3u) != 0) return TF_ALIGNMENT;
        if (s.m_fmt != M_INT8 && s.m_fmt != M_NF4) return TF_FORMAT;
    } else {
        if (s.m_fmt > M_F16 || s.v_fmt > V_F16) return TF_FORMAT;
        if ((reinterpret_cast<uintptr_t>(s.m) & (float_width(s.m_fmt) - 1u)) != 0) return TF_ALIGNMENT;
        if ((reinterpret_cast<uintptr_t>(s.v) & (float_width(s.v_fmt) - 1u)) != 0) return TF_ALIGNMENT;
    }
    return TF_NONE;
}

// word[0]: first fault code, word[1]: segment, word[2]: chunk (of the launch), word[3]: how many chunks were skipped
__device__ __forceinline__ void record_table_fault(unsigned* word, uint32_t code, int si, uint32_t chunk) {
    if (threadIdx.x != 0) return;
    if (atomicCAS(&word[0], 0u, code) == 0u) {
        word[1] = static_cast<unsigned>(si);
        word[2] = chunk;
    }
    atomicAdd(&word[3], 1u);
}

// Ask the copy engine to pull [ptr, ptr+bytes) from HBM into L2 ahead of use.  Has no
// completion to wait for; silently skipped when the range is not 16-byte granular.
__device__ __forceinline__ void l2_prefetch(const void* ptr, uint32_t bytes) {
    if (bytes == 0 || (bytes & 15u) || (reinterpret_cast<uintptr_t>(ptr) & 15u)) return;
    asm volatile("cp.async.bulk.prefetch.L2.global [%0], %1;" ::"l"(ptr), "r"(bytes) : "memory");
}

// Prefetch the local arrays of chunk `c` of segment `s` (one thread per array).
__device__ __forceinline__ void prefetch_chunk(const SegDesc& s, uint32_t c, bool want_grad) {
    const long long first = static_cast<long long>(c) * kChunk;
    if (first >= s.numel) return;
    const long long left = s.numel - first;
    const uint32_t n = left >= kChunk ? kChunk : static_cast<uint32_t>(left);
    const bool quad = (s.flags & SEG_QUAD_V) != 0;
    const int t = threadIdx.x;
    if (t == 0) {
        const uint32_t w = s.p_dtype == DT_F32 ? 4u : 2u;
        l2_prefetch(static_cast<const char*>(s.p) + first * w, n * w);
    } else if (t == 32 && want_grad && s.g != nullptr) {
        const uint32_t w = s.g_dtype == DT_F32 ? 4u : 2u;
        l2_prefetch(static_cast<const char*>(s.g) + first * w, n * w);
    } else if (t == 64) {
        if (s.m_fmt == M_NF4) l2_prefetch(static_cast<const char*>(s.m) + (first >> 1), n >> 1);
        else if (s.m_fmt == M_INT8) l2_prefetch(static_cast<const char*>(s.m) + first, n);
        else { const uint32_t w = s.m_fmt == M_F32 ? 4u : 2u; l2_prefetch(static_cast<const char*>(s.m) + first * w, n * w); }
    } else if (t == 96 && !(s.flags & SEG_NO_V_STREAM)) {
        const long long vf = quad ? (first >> 2) : first;
        const uint32_t vn = quad ? (n >> 2) : n;
        const uint32_t w = s.v_fmt == V_LOGU8 ? 1u : (s.v_fmt == V_F32 ? 4u : 2u);
        l2_prefetch(static_cast<const char*>(s.v) + vf * w, vn * w);
    }
}

__device__ __forceinline__ void load_tables(CodecTables& dst, const CodecTables* __restrict__ src) {
    const float* s = reinterpret_cast<const float*>(src);
    float* d = reinterpret_cast<float*>(&dst);
    for (int i = threadIdx.x; i < static_cast<int>(sizeof(CodecTables) / sizeof(float)); i += blockDim.x) d[i] = s[i];
}

}  // namespace apexb
