// Model-side fused kernels of the training harness: RMSNorm (+residual add) forward and
// backward, SwiGLU forward and backward, rotary embedding on a packed qkv tensor, and
// softmax cross-entropy with the gradient written over the logits.  All are single-pass,
// HBM-bound kernels: 16-byte vector accesses, fp32 math in registers, bf16 or fp32 storage.
// (The reference has no model code; these exist so that the end-to-end benchmark measures
// the optimizer inside a training step whose elementwise work is already fused.)
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <cstdint>
#include "api.h"

namespace apexb {
namespace {

template <typename T> struct Vec8;

template <> struct Vec8<__nv_bfloat16> {
    static __device__ __forceinline__ void load(const __nv_bfloat16* p, float (&o)[8]) {
        const uint4 r = *reinterpret_cast<const uint4*>(p);
        const uint32_t w[4] = {r.x, r.y, r.z, r.w};
#pragma unroll
        for (int k = 0; k < 4; ++k) {
            o[2 * k] = __uint_as_float(w[k] << 16);
            o[2 * k + 1] = __uint_as_float(w[k] & 0xFFFF0000u);
        }
    }
    static __device__ __forceinline__ void store(__nv_bfloat16* p, const float (&v)[8]) {
        uint32_t w[4];
#pragma unroll
        for (int k = 0; k < 4; ++k) {
            const __nv_bfloat162 h = __floats2bfloat162_rn(v[2 * k], v[2 * k + 1]);
            w[k] = *reinterpret_cast<const uint32_t*>(&h);
        }
        *reinterpret_cast<uint4*>(p) = make_uint4(w[0], w[1], w[2], w[3]);
    }
    static __device__ __forceinline__ float round(float x) { return __bfloat162float(__float2bfloat16_rn(x)); }
};

template <> struct Vec8<float> {
    static __device__ __forceinline__ void load(const float* p, float (&o)[8]) {
        const float4 a = *reinterpret_cast<const float4*>(p);
        const float4 b = *reinterpret_cast<const float4*>(p + 4);
        o[0] = a.x; o[1] = a.y; o[2] = a.z; o[3] = a.w; o[4] = b.x; o[5] = b.y; o[6] = b.z; o[7] = b.w;
    }
    static __device__ __forceinline__ void store(float* p, const float (&v)[8]) {
        *reinterpret_cast<float4*>(p) = make_float4(v[0], v[1], v[2], v[3]);
        *reinterpret_cast<float4*>(p + 4) = make_float4(v[4], v[5], v[6], v[7]);
    }
    static __device__ __forceinline__ float round(float x) { return x; }
};

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xFFFFFFFFu, v, o);
    return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xFFFFFFFFu, v, o));
    return v;
}

// block-wide sum; every thread gets the result. smem: >= 33 floats
__device__ __forceinline__ float block_sum(float v, float* smem) {
    v = warp_sum(v);
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nw = (blockDim.x + 31) >> 5;
    if (lane == 0) smem[warp] = v;
    __syncthreads();
    if (warp == 0) {
        float t = lane < nw ? smem[lane] : 0.0f;
        t = warp_sum(t);
        if (lane == 0) smem[32] = t;
    }
    __syncthreads();
    const float r = smem[32];
    __syncthreads();
    return r;
}

constexpr int kNormThreads = 256;
constexpr int kNormMaxVec = 4;  // rows up to 256 * 8 * 4 = 8192 elements stay in registers

// ---------------------------------------------------------------------------
// RMSNorm forward: h = x (+ residual), y = h * rsqrt(mean(h^2) + eps) * w
// ---------------------------------------------------------------------------
template <typename T>
__global__ void __launch_bounds__(kNormThreads)
rmsnorm_fwd_kernel(const T* __restrict__ x, const T* __restrict__ res, const T* __restrict__ w, T* __restrict__ y,
                   T* __restrict__ h_out, float* __restrict__ rstd_out, int rows, int H, float eps) {
    __shared__ float smem[33];
    const int nvec = H / 8;
    for (int row = blockIdx.x; row < rows; row += gridDim.x) {
        const size_t base = static_cast<size_t>(row) * H;
        float h[kNormMaxVec][8];
        float ss = 0.0f;
#pragma unroll
        for (int it = 0; it < kNormMaxVec; ++it) {
            const int v = threadIdx.x + it * kNormThreads;
            if (v < nvec) {
                Vec8<T>::load(x + base + v * 8, h[it]);
                if (res != nullptr) {
                    float r[8];
                    Vec8<T>::load(res + base + v * 8, r);
#pragma unroll
                    for (int k = 0; k < 8; ++k) h[it][k] = Vec8<T>::round(h[it][k] + r[k]);
                    Vec8<T>::store(h_out + base + v * 8, h[it]);
                }
#pragma unroll
                for (int k = 0; k < 8; ++k) ss += h[it][k] * h[it][k];
            }
        }
        const float total = block_sum(ss, smem);
        const float rstd = rsqrtf(total / static_cast<float>(H) + eps);
        if (threadIdx.x == 0) rstd_out[row] = rstd;
#pragma unroll
        for (int it = 0; it < kNormMaxVec; ++it) {
            const int v = threadIdx.x + it * kNormThreads;
            if (v < nvec) {
                float wv[8], o[8];
                Vec8<T>::load(w + v * 8, wv);
#pragma unroll
                for (int k = 0; k < 8; ++k) o[k] = h[it][k] * rstd * wv[k];
                Vec8<T>::store(y + base + v * 8, o);
            }
        }
    }
}

// ---------------------------------------------------------------------------
// RMSNorm backward.  Persistent CTAs loop over rows; each thread keeps its columns'
// weight-gradient partial sums in registers and writes them once to `partial`
// ([gridDim.x, H] fp32 scratch); rmsnorm_dw_reduce_kernel then sums over CTAs.
// ---------------------------------------------------------------------------
// NV = 8-element vectors per thread (1, 2 or 4, from the row width): sizing the register arrays for the actual width
// instead of the maximum takes the H = 4096 case from 161 registers (one CTA per SM) to two resident CTAs per SM.
template <typename T, int NV>
__global__ void __launch_bounds__(kNormThreads, NV == 1 ? 4 : (NV == 2 ? 2 : 1))
rmsnorm_bwd_kernel(const T* __restrict__ dy, const T* __restrict__ dres, const T* __restrict__ h, const T* __restrict__ w,
                   const float* __restrict__ rstd_in, T* __restrict__ dx, float* __restrict__ partial, int rows, int H) {
    __shared__ float smem[33];
    const int nvec = H / 8;
    float dw[NV][8];
    float wv[NV][8];
#pragma unroll
    for (int it = 0; it < NV; ++it) {
        const int v = threadIdx.x + it * kNormThreads;
#pragma unroll
        for (int k = 0; k < 8; ++k) { dw[it][k] = 0.0f; wv[it][k] = 0.0f; }
        if (v < nvec) Vec8<T>::load(w + v * 8, wv[it]);
    }
    for (int row = blockIdx.x; row < rows; row += gridDim.x) {
        const size_t base = static_cast<size_t>(row) * H;
        const float rstd = rstd_in[row];
        float g[NV][8], xh[NV][8];
        float dot = 0.0f;
#pragma unroll
        for (int it = 0; it < NV; ++it) {
            const int v = threadIdx.x + it * kNormThreads;
            if (v < nvec) {
                float d[8], hv[8];
                Vec8<T>::load(dy + base + v * 8, d);
                Vec8<T>::load(h + base + v * 8, hv);
#pragma unroll
                for (int k = 0; k < 8; ++k) {
                    xh[it][k] = hv[k] * rstd;
                    g[it][k] = d[k] * wv[it][k];
                    dot += g[it][k] * xh[it][k];
                    dw[it][k] += d[k] * xh[it][k];
                }
            }
        }
        const float c = block_sum(dot, smem) / static_cast<float>(H);
#pragma unroll
        for (int it = 0; it < NV; ++it) {
            const int v = threadIdx.x + it * kNormThreads;
            if (v < nvec) {
                float o[8];
#pragma unroll
                for (int k = 0; k < 8; ++k) o[k] = (g[it][k] - xh[it][k] * c) * rstd;
                if (dres != nullptr) {
                    float r[8];
                    Vec8<T>::load(dres + base + v * 8, r);
#pragma unroll
                    for (int k = 0; k < 8; ++k) o[k] += r[k];
                }
                Vec8<T>::store(dx + base + v * 8, o);
            }
        }
    }
#pragma unroll
    for (int it = 0; it < NV; ++it) {
        const int v = threadIdx.x + it * kNormThreads;
        if (v < nvec) {
            float* dst = partial + static_cast<size_t>(blockIdx.x) * H + v * 8;
            *reinterpret_cast<float4*>(dst) = make_float4(dw[it][0], dw[it][1], dw[it][2], dw[it][3]);
            *reinterpret_cast<float4*>(dst + 4) = make_float4(dw[it][4], dw[it][5], dw[it][6], dw[it][7]);
        }
    }
}

// dw[col] = sum over CTAs of partial[cta][col].  A CTA of 256 threads takes 32 columns; its 8 warps each sum every
// eighth partial row (128-byte coalesced reads), then the 8 partial sums meet in shared memory.
__global__ void __launch_bounds__(256)
rmsnorm_dw_reduce_kernel(const float* __restrict__ partial, float* __restrict__ dw, int nparts, int H) {
    __shared__ float acc_s[8][33];
    const int lane = threadIdx.x & 31, grp = threadIdx.x >> 5;
    const int col = blockIdx.x * 32 + lane;
    float acc = 0.0f;
    if (col < H)
        for (int i = grp; i < nparts; i += 8) acc += partial[static_cast<size_t>(i) * H + col];
    acc_s[grp][lane] = acc;
    __syncthreads();
    if (grp == 0 && col < H) {
        float t = 0.0f;
#pragma unroll
        for (int k = 0; k < 8; ++k) t += acc_s[k][lane];
        dw[col] = t;
    }
}

// ---------------------------------------------------------------------------
// SwiGLU on a packed [gate | up] row of width 2F
// ---------------------------------------------------------------------------
template <typename T>
__global__ void swiglu_fwd_kernel(const T* __restrict__ gu, T* __restrict__ y, long long rows, int F) {
    const long long nvec = rows * (F / 8);
    for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < nvec;
         i += static_cast<long long>(gridDim.x) * blockDim.x) {
        const long long row = i / (F / 8);
        const int col = static_cast<int>(i % (F / 8)) * 8;
        float g[8], u[8], o[8];
        Vec8<T>::load(gu + row * 2 * F + col, g);
        Vec8<T>::load(gu + row * 2 * F + F + col, u);
#pragma unroll
        for (int k = 0; k < 8; ++k) o[k] = g[k] / (1.0f + __expf(-g[k])) * u[k];
        Vec8<T>::store(y + row * F + col, o);
    }
}

template <typename T>
__global__ void swiglu_bwd_kernel(const T* __restrict__ dy, const T* __restrict__ gu, T* __restrict__ dgu, long long rows, int F) {
    const long long nvec = rows * (F / 8);
    for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < nvec;
         i += static_cast<long long>(gridDim.x) * blockDim.x) {
        const long long row = i / (F / 8);
        const int col = static_cast<int>(i % (F / 8)) * 8;
        float g[8], u[8], d[8], dg[8], du[8];
        Vec8<T>::load(gu + row * 2 * F + col, g);
        Vec8<T>::load(gu + row * 2 * F + F + col, u);
        Vec8<T>::load(dy + row * F + col, d);
#pragma unroll
        for (int k = 0; k < 8; ++k) {
            const float sig = 1.0f / (1.0f + __expf(-g[k]));
            const float silu = g[k] * sig;
            dg[k] = d[k] * u[k] * (sig + silu * (1.0f - sig));
            du[k] = d[k] * silu;
        }
        Vec8<T>::store(dgu + row * 2 * F + col, dg);
        Vec8<T>::store(dgu + row * 2 * F + F + col, du);
    }
}

// ---------------------------------------------------------------------------
// RoPE (rotate-half) on the first n_rot heads of a (tokens, heads, D) tensor; other heads copied.
// cos/sin: (S, D/2) fp32; token t uses position t % S.
// ---------------------------------------------------------------------------
template <typename T>
__global__ void rope_kernel(const T* __restrict__ in, T* __restrict__ out, const float* __restrict__ cosv,
                            const float* __restrict__ sinv, long long tokens, int S, int heads, int D, int n_rot, float sign) {
    const int half_vecs = D / 16;  // vectors of 8 in one half of a head
    const long long total = tokens * heads * half_vecs;
    for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < total;
         i += static_cast<long long>(gridDim.x) * blockDim.x) {
        const int hv = static_cast<int>(i % half_vecs);
        const long long th = i / half_vecs;
        const int head = static_cast<int>(th % heads);
        const long long tok = th / heads;
        const size_t base = static_cast<size_t>(th) * D + hv * 8;
        float a[8], b[8];
        Vec8<T>::load(in + base, a);
        Vec8<T>::load(in + base + D / 2, b);
        if (head < n_rot) {
            const int pos = static_cast<int>(tok % S);
            const float* c = cosv + static_cast<size_t>(pos) * (D / 2) + hv * 8;
            const float* s = sinv + static_cast<size_t>(pos) * (D / 2) + hv * 8;
            float oa[8], ob[8];
#pragma unroll
            for (int k = 0; k < 8; ++k) {
                const float sk = s[k] * sign;
                oa[k] = a[k] * c[k] - b[k] * sk;
                ob[k] = b[k] * c[k] + a[k] * sk;
            }
            Vec8<T>::store(out + base, oa);
            Vec8<T>::store(out + base + D / 2, ob);
        } else {
            Vec8<T>::store(out + base, a);
            Vec8<T>::store(out + base + D / 2, b);
        }
    }
}

// ---------------------------------------------------------------------------
// cross-entropy: per row, online max/sum pass then gradient pass (second read hits L2)
// logits row is overwritten with scale * (softmax - onehot)
// A target outside [0, V) (the usual ignore_index = -100, or any stray value) marks an ignored row: loss 0 and
// an all-zero gradient row; the target is never used as an index then.  scale_dev (optional, one device float)
// multiplies scale, so that a mean over the rows that count needs no host round trip.
// ---------------------------------------------------------------------------
constexpr int kCEThreads = 512;

template <typename T>
__global__ void __launch_bounds__(kCEThreads)
cross_entropy_kernel(T* __restrict__ logits, const long long* __restrict__ targets, float* __restrict__ losses, int V, float scale,
                     const float* __restrict__ scale_dev) {
    __shared__ float smem[33];
    __shared__ float s_max;
    const size_t base = static_cast<size_t>(blockIdx.x) * V;
    T* row = logits + base;
    const int nvec = V / 8;
    float m = -INFINITY, s = 0.0f;
    for (int v = threadIdx.x; v < nvec; v += kCEThreads) {
        float x[8];
        Vec8<T>::load(row + v * 8, x);
        float lm = x[0];
#pragma unroll
        for (int k = 1; k < 8; ++k) lm = fmaxf(lm, x[k]);
        if (lm > m) { s *= __expf(m - lm); m = lm; }
#pragma unroll
        for (int k = 0; k < 8; ++k) s += __expf(x[k] - m);
    }
    for (int j = nvec * 8 + threadIdx.x; j < V; j += kCEThreads) {
        const float x = static_cast<float>(row[j]);
        if (x > m) { s *= __expf(m - x); m = x; }
        s += __expf(x - m);
    }
    // block max
    float wm = warp_max(m);
    if ((threadIdx.x & 31) == 0) smem[threadIdx.x >> 5] = wm;
    __syncthreads();
    if (threadIdx.x < 32) {
        float t = threadIdx.x < kCEThreads / 32 ? smem[threadIdx.x] : -INFINITY;
        t = warp_max(t);
        if (threadIdx.x == 0) s_max = t;
    }
    __syncthreads();
    const float gmax = s_max;
    const float total = block_sum(s * __expf(m - gmax), smem);
    const float lse = gmax + __logf(total);
    const long long tgt = targets[blockIdx.x];
    const bool counted = tgt >= 0 && tgt < V;
    if (threadIdx.x == 0) losses[blockIdx.x] = counted ? lse - static_cast<float>(row[tgt]) : 0.0f;
    if (scale_dev != nullptr) scale *= *scale_dev;
    __syncthreads();
    for (int v = threadIdx.x; v < nvec; v += kCEThreads) {
        float x[8], g[8];
        Vec8<T>::load(row + v * 8, x);
#pragma unroll
        for (int k = 0; k < 8; ++k) {
            const float p = __expf(x[k] - lse);
            g[k] = counted ? (p - ((v * 8 + k) == tgt ? 1.0f : 0.0f)) * scale : 0.0f;
        }
        Vec8<T>::store(row + v * 8, g);
    }
    for (int j = nvec * 8 + threadIdx.x; j < V; j += kCEThreads) {
        const float p = __expf(static_cast<float>(row[j]) - lse);
        row[j] = static_cast<T>(counted ? (p - (j == tgt ? 1.0f : 0.0f)) * scale : 0.0f);
    }
}

int grid_for(long long work_items, int threads, int sm_count, int per_sm) {
    long long blocks = (work_items + threads - 1) / threads;
    const long long cap = static_cast<long long>(sm_count) * per_sm;
    if (blocks > cap) blocks = cap;
    if (blocks < 1) blocks = 1;
    return static_cast<int>(blocks);
}

}  // namespace
}  // namespace apexb

using namespace apexb;

#define DISPATCH_T(is_bf16, ...)                          \
    if (is_bf16) { using T = __nv_bfloat16; __VA_ARGS__; } \
    else { using T = float; __VA_ARGS__; }

extern "C" int apexb_rmsnorm_fwd(const void* x, const void* res, const void* w, void* y, void* h_out, float* rstd, int rows,
                                 int H, float eps, int is_bf16, int sm_count, cudaStream_t stream) {
    if (H % 8 != 0 || H > kNormThreads * 8 * kNormMaxVec) return cudaErrorInvalidValue;
    const int grid = rows < sm_count * 8 ? rows : sm_count * 8;
    DISPATCH_T(is_bf16, rmsnorm_fwd_kernel<T><<<grid, kNormThreads, 0, stream>>>(
        static_cast<const T*>(x), static_cast<const T*>(res), static_cast<const T*>(w), static_cast<T*>(y),
        static_cast<T*>(h_out), rstd, rows, H, eps));
    return static_cast<int>(cudaGetLastError());
}

extern "C" int apexb_rmsnorm_bwd_parts(int rows, int sm_count) {
    const int cap = sm_count * 2;      // two CTAs are resident per SM at H = 4096; more would only enlarge the scratch
    return rows < cap ? rows : cap;
}

namespace {
template <typename T, int NV>
void launch_rmsnorm_bwd_nv(const void* dy, const void* dres, const void* h, const void* w, const float* rstd, void* dx,
                           float* partial, int nparts, int rows, int H, cudaStream_t stream) {
    apexb::rmsnorm_bwd_kernel<T, NV><<<nparts, apexb::kNormThreads, 0, stream>>>(
        static_cast<const T*>(dy), static_cast<const T*>(dres), static_cast<const T*>(h), static_cast<const T*>(w), rstd,
        static_cast<T*>(dx), partial, rows, H);
}

// backward kernel sized for the row width, then the reduction of the per-CTA weight-gradient partial sums
void launch_rmsnorm_bwd(const void* dy, const void* dres, const void* h, const void* w, const float* rstd, void* dx, float* dw,
                        float* partial, int nparts, int rows, int H, int is_bf16, cudaStream_t stream) {
    const int nv = (H / 8 + apexb::kNormThreads - 1) / apexb::kNormThreads;
    if (is_bf16) {
        if (nv <= 1) launch_rmsnorm_bwd_nv<__nv_bfloat16, 1>(dy, dres, h, w, rstd, dx, partial, nparts, rows, H, stream);
        else if (nv == 2) launch_rmsnorm_bwd_nv<__nv_bfloat16, 2>(dy, dres, h, w, rstd, dx, partial, nparts, rows, H, stream);
        else launch_rmsnorm_bwd_nv<__nv_bfloat16, 4>(dy, dres, h, w, rstd, dx, partial, nparts, rows, H, stream);
    } else {
        if (nv <= 1) launch_rmsnorm_bwd_nv<float, 1>(dy, dres, h, w, rstd, dx, partial, nparts, rows, H, stream);
        else if (nv == 2) launch_rmsnorm_bwd_nv<float, 2>(dy, dres, h, w, rstd, dx, partial, nparts, rows, H, stream);
        else launch_rmsnorm_bwd_nv<float, 4>(dy, dres, h, w, rstd, dx, partial, nparts, rows, H, stream);
    }
    apexb::rmsnorm_dw_reduce_kernel<<<(H + 31) / 32, 256, 0, stream>>>(partial, dw, nparts, H);
}
}  // namespace

extern "C" int apexb_rmsnorm_bwd(const void* dy, const void* dres, const void* h, const void* w, const float* rstd, void* dx,
                                 float* dw, float* partial, int nparts, int rows, int H, int is_bf16, cudaStream_t stream) {
    if (H % 8 != 0 || H > kNormThreads * 8 * kNormMaxVec) return cudaErrorInvalidValue;
    launch_rmsnorm_bwd(dy, dres, h, w, rstd, dx, dw, partial, nparts, rows, H, is_bf16, stream);
    return static_cast<int>(cudaGetLastError());
}

extern "C" int apexb_swiglu_fwd(const void* gu, void* y, long long rows, int F, int is_bf16, int sm_count, cudaStream_t stream) {
    if (F % 8 != 0) return cudaErrorInvalidValue;
    const int grid = grid_for(rows * (F / 8), 256, sm_count, 16);
    DISPATCH_T(is_bf16, swiglu_fwd_kernel<T><<<grid, 256, 0, stream>>>(static_cast<const T*>(gu), static_cast<T*>(y), rows, F));
    return static_cast<int>(cudaGetLastError());
}

extern "C" int apexb_swiglu_bwd(const void* dy, const void* gu, void* dgu, long long rows, int F, int is_bf16, int sm_count,
                                cudaStream_t stream) {
    if (F % 8 != 0) return cudaErrorInvalidValue;
    const int grid = grid_for(rows * (F / 8), 256, sm_count, 16);
    DISPATCH_T(is_bf16, swiglu_bwd_kernel<T><<<grid, 256, 0, stream>>>(static_cast<const T*>(dy), static_cast<const T*>(gu),
                                                                      static_cast<T*>(dgu), rows, F));
    return static_cast<int>(cudaGetLastError());
}

extern "C" int apexb_rope(const void* in, void* out, const float* cosv, const float* sinv, long long tokens, int S, int heads,
                          int D, int n_rot, int inverse, int is_bf16, int sm_count, cudaStream_t stream) {
    if (D % 16 != 0) return cudaErrorInvalidValue;
    const int grid = grid_for(tokens * heads * (D / 16), 256, sm_count, 16);
    const float sign = inverse ? -1.0f : 1.0f;
    DISPATCH_T(is_bf16, rope_kernel<T><<<grid, 256, 0, stream>>>(static_cast<const T*>(in), static_cast<T*>(out), cosv, sinv,
                                                                 tokens, S, heads, D, n_rot, sign));
    return static_cast<int>(cudaGetLastError());
}

extern "C" int apexb_cross_entropy(void* logits, const long long* targets, float* losses, int rows, int V, float scale,
                                   const float* scale_dev, int is_bf16, cudaStream_t stream) {
    if (rows <= 0) return 0;
    // rows must start 16-byte aligned for the vector path
    if ((static_cast<long long>(V) * (is_bf16 ? 2 : 4)) % 16 != 0) return cudaErrorInvalidValue;
    DISPATCH_T(is_bf16, cross_entropy_kernel<T><<<rows, kCEThreads, 0, stream>>>(static_cast<T*>(logits), targets, losses, V, scale, scale_dev));
    return static_cast<int>(cudaGetLastError());
}

// ---------------------------------------------------------------------------
// RMSNorm backward with library-owned scratch (see no_alloc.h)
// ---------------------------------------------------------------------------
#include <cstdio>
#include <cstring>
#include "no_alloc.h"

namespace apexb {
// Per-CTA partial sums of the weight gradient, [CTAs, H] floats.  Device code could name this
// array directly; host code must not pass the symbol itself to a kernel (on the host it is only a
// stand-in), so the launcher below asks the runtime for its device address once per device.
static __device__ __align__(256) float g_noalloc_scratch[APEXB_NOALLOC_SCRATCH_FLOATS];
static float* g_noalloc_scratch_ptr[64] = {};
}  // namespace apexb

static int noalloc_fail(int code, char* err, int err_len, const char* msg) {
    if (err != nullptr && err_len > 0) {
        std::strncpy(err, msg, static_cast<size_t>(err_len) - 1);
        err[err_len - 1] = '\0';
    }
    return code;
}

extern "C" int apexb_rmsnorm_bwd_noalloc(const void* dy, const void* dres, const void* h, const void* w, const float* rstd,
                                          void* dx, float* dw, int rows, int H, int is_bf16, cudaStream_t stream, char* err,
                                          int err_len) {
    if (err != nullptr && err_len > 0) err[0] = '\0';
    if (rows <= 0 || H <= 0 || H % 8 != 0 || H > kNormThreads * 8 * kNormMaxVec)
        return noalloc_fail(1, err, err_len, "rmsnorm_bwd_noalloc: rows must be positive and H a multiple of 8 not above 8192");
    if (H > APEXB_NOALLOC_SCRATCH_FLOATS)
        return noalloc_fail(1, err, err_len, "rmsnorm_bwd_noalloc: H exceeds the built-in scratch array");
    if (dy == nullptr || h == nullptr || w == nullptr || rstd == nullptr || dx == nullptr || dw == nullptr)
        return noalloc_fail(2, err, err_len, "rmsnorm_bwd_noalloc: null pointer");
    const uintptr_t bits = reinterpret_cast<uintptr_t>(dy) | reinterpret_cast<uintptr_t>(h) | reinterpret_cast<uintptr_t>(w) |
                           reinterpret_cast<uintptr_t>(dx) | reinterpret_cast<uintptr_t>(dres);
    if (bits & 15u) return noalloc_fail(2, err, err_len, "rmsnorm_bwd_noalloc: dy, dres, h, w and dx must be 16-byte aligned");

    int device = 0;
    cudaError_t e = cudaGetDevice(&device);
    if (e != cudaSuccess || device < 0 || device >= 64)
        return noalloc_fail(1000 + static_cast<int>(e), err, err_len, "rmsnorm_bwd_noalloc: cudaGetDevice failed");
    if (g_noalloc_scratch_ptr[device] == nullptr) {
        // set-up, once per device, with that device current: device address of the scratch symbol
        float* ptr = nullptr;
        e = cudaGetSymbolAddress(reinterpret_cast<void**>(&ptr), g_noalloc_scratch);
        if (e != cudaSuccess || ptr == nullptr)
            return noalloc_fail(1000 + static_cast<int>(e), err, err_len, "rmsnorm_bwd_noalloc: cudaGetSymbolAddress failed");
        g_noalloc_scratch_ptr[device] = ptr;
    }
    float* partial = g_noalloc_scratch_ptr[device];

    int nparts = rows < 256 ? rows : 256;
    const int fit = APEXB_NOALLOC_SCRATCH_FLOATS / H;
    if (nparts > fit) nparts = fit;
    // every launched CTA writes its whole [H] row of partials before the reduction reads it,
    // so the array needs no clearing even though it keeps the previous call's contents
    launch_rmsnorm_bwd(dy, dres, h, w, rstd, dx, dw, partial, nparts, rows, H, is_bf16, stream);
    e = cudaGetLastError();
    if (e != cudaSuccess) return noalloc_fail(1000 + static_cast<int>(e), err, err_len, cudaGetErrorString(e));
    return 0;
}
