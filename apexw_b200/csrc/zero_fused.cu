// Fused ZeRO-1 step: reduce-scatter of gradients, optimizer-state update and all-gather of
// parameters in ONE kernel over NVLink peer memory.
//
// Every rank holds the same flat layout of gradients and parameters in buffers that all
// ranks have mapped (CUDA IPC).  A rank's kernel walks the segments of the shard it owns:
//   gradient  : 16-byte loads of the same 8 elements from every rank's gradient buffer,
//               summed in fp32 registers in rank order (the reduce-scatter),
//   update    : the same decode -> AdamW -> re-encode body as the single-GPU kernel,
//   parameter : the rounded 16-byte result stored to every rank's parameter buffer
//               (the all-gather).
// No NCCL call, no staging buffer, no separate elementwise kernel.  It replaces the
// reference's DDP all-reduce + per-parameter zero-fill/all-reduce/broadcast sequence
// (apexw/zero.py:232-347).
//
// Cross-rank ordering uses two rounds of flags in a small symmetric signal pad:
//   entry: "my gradients are final"  - a rank reads peers' gradients only after all flags,
//   exit : "I wrote all my parameters to you" - a rank's kernel ends only after all flags,
// so stream order on each rank gives the next forward complete parameters.  All waits are
// bounded by a cycle budget; on expiry the kernel records a status code and returns (the
// entry wait is decided once by CTA 0 and broadcast, so either every chunk is updated or none).
//
// Two transports for the bulk data, chosen per launch:
//   * plain peer loads / stores (default): every rank's buffer is addressed through its own mapping;
//   * NVLS (ZeroPeers::mc_grad / mc_param set): `multimem.ld_reduce` returns the gradient already summed over ranks by
//     the switch and `multimem.st` writes all ranks' parameter copies with one store, which roughly halves the bytes
//     that cross this GPU's links (each gradient byte leaves its GPU once instead of being pulled by one peer at a
//     time, each parameter byte enters the switch once instead of W - 1 times).  The switch hands the sum back
//     rounded to bf16, so this path is not bit-identical to the peer-load path.
// Flags always travel as plain release / acquire stores and loads.  No TMA, no cluster multicast anywhere.
#include <cuda_runtime.h>
#include <cstdint>
#include "api.h"
#include "fused_state.cuh"
#include "peer_sync.cuh"

namespace apexb {

__device__ CodecTables g_zero_codec_tables;
__device__ unsigned g_zero_table_fault[4];     // debug mode: first table fault of this module's kernels

// WORLD > 0: world size known at compile time (1, 2, 4, 8 are instantiated): peer loops unroll without
// predication and keep only WORLD vectors live.  WORLD == 0: any world size up to kMaxPeers, predicated.
// sixteen bytes (eight bf16) summed over all ranks by the switch, accumulated in fp32 there
__device__ __forceinline__ uint4 multimem_sum_bf16x8(const void* mc_addr) {
    uint4 r;
    asm volatile("multimem.ld_reduce.relaxed.sys.global.add.acc::f32.v4.bf16x2 {%0, %1, %2, %3}, [%4];"
                 : "=r"(r.x), "=r"(r.y), "=r"(r.z), "=r"(r.w) : "l"(mc_addr) : "memory");
    return r;
}
// sixteen bytes stored into every rank's copy
__device__ __forceinline__ void multimem_store16(void* mc_addr, const uint4& v) {
    asm volatile("multimem.st.relaxed.sys.global.v4.f32 [%0], {%1, %2, %3, %4};"
                 :: "l"(mc_addr), "r"(v.x), "r"(v.y), "r"(v.z), "r"(v.w) : "memory");
}

// MC: the aligned bf16 vector path goes through the multicast addresses; ragged and fp32 accesses stay on peer pointers
template <int WORLD, bool MC = false>
struct PeerIO {
    const ZeroPeers* peers;
    int g_dtype;
    int p_dtype;

    __device__ __forceinline__ void load_grad(const SegDesc& s, long long idx, int nvalid, float (&g)[8]) const {
        const int W = peers->grad_sources;
        const long long e = s.offset + idx;
        if (g_dtype == DT_BF16 && nvalid == 8 && ((e & 7) == 0)) {
            load_grad_fast(s, idx, g);
            return;
        }
        load8(peers->grad[0], g_dtype, e, nvalid, g);
        for (int r = 1; r < W; ++r) {
            float t[8];
            load8(peers->grad[r], g_dtype, e, nvalid, t);
#pragma unroll
            for (int k = 0; k < 8; ++k) g[k] += t[k];
        }
    }

    __device__ __forceinline__ void store_param(const SegDesc& s, long long idx, int nvalid, const float (&p)[8],
                                                const uint32_t (&r16)[8], bool sr) const {
        const int W = peers->world;
        const long long e = s.offset + idx;
        if (p_dtype == DT_BF16 && nvalid == 8 && ((e & 7) == 0)) {
            uint32_t w[4];
#pragma unroll
            for (int k = 0; k < 4; ++k)
                w[k] = sr ? pack2_sr(p[2 * k], p[2 * k + 1], r16[2 * k], r16[2 * k + 1]) : pack2_rn(p[2 * k], p[2 * k + 1]);
            store_param_fast(s, idx, make_uint4(w[0], w[1], w[2], w[3]));
        } else {
            for (int r = 0; r < W; ++r) store8(peers->param[r], p_dtype, e, nvalid, p, r16, sr);
        }
    }

    // fast path: bf16 buffers, s.offset a multiple of 8 elements.  The sum runs in rank order on every path.
    __device__ __forceinline__ void load_grad_fast(const SegDesc& s, long long idx, float (&g)[8]) const {
        const long long e = s.offset + idx;
        const int sources = peers->grad_sources;
        if (sources == 1) {
            unpack8(__ldcs(reinterpret_cast<const uint4*>(reinterpret_cast<const uint16_t*>(peers->grad[0]) + e)), g);
        } else if (MC) {
            unpack8(multimem_sum_bf16x8(reinterpret_cast<const uint16_t*>(peers->mc_grad) + e), g);
        } else if (WORLD > 0) {
            uint4 raw[WORLD > 0 ? WORLD : 1];
#pragma unroll
            for (int r = 0; r < WORLD; ++r)
                raw[r] = __ldcs(reinterpret_cast<const uint4*>(reinterpret_cast<const uint16_t*>(peers->grad[r]) + e));
            unpack8(raw[0], g);
#pragma unroll
            for (int r = 1; r < WORLD; ++r) {
                float t[8];
                unpack8(raw[r], t);
#pragma unroll
                for (int k = 0; k < 8; ++k) g[k] += t[k];
            }
        } else {
            uint4 raw[kMaxPeers];
#pragma unroll
            for (int r = 0; r < kMaxPeers; ++r)
                if (r < sources) raw[r] = __ldcs(reinterpret_cast<const uint4*>(reinterpret_cast<const uint16_t*>(peers->grad[r]) + e));
            unpack8(raw[0], g);
#pragma unroll
            for (int r = 1; r < kMaxPeers; ++r) {
                if (r < sources) {
                    float t[8];
                    unpack8(raw[r], t);
#pragma unroll
                    for (int k = 0; k < 8; ++k) g[k] += t[k];
                }
            }
        }
    }
    __device__ __forceinline__ void store_param_fast(const SegDesc& s, long long idx, const uint4& packed) const {
        const long long e = s.offset + idx;
        if (MC) {
            multimem_store16(reinterpret_cast<uint16_t*>(peers->mc_param) + e, packed);
        } else if (WORLD > 0) {
#pragma unroll
            for (int r = 0; r < WORLD; ++r) *reinterpret_cast<uint4*>(reinterpret_cast<uint16_t*>(peers->param[r]) + e) = packed;
        } else {
            const int W = peers->world;
#pragma unroll
            for (int r = 0; r < kMaxPeers; ++r)
                if (r < W) *reinterpret_cast<uint4*>(reinterpret_cast<uint16_t*>(peers->param[r]) + e) = packed;
        }
    }
};

template <int KC, int WORLD, bool MC>
__global__ void __launch_bounds__(kThreads, (WORLD > 0 || MC) ? 3 : 2)
zero_fused_kernel(const SegDesc* __restrict__ segs, StepArgs a, ZeroPeers peers, uint32_t epoch, long long budget,
                  uint32_t* __restrict__ status, int g_dtype, int p_dtype, const float* __restrict__ clip_total_sq,
                  float clip_max_norm) {
    __shared__ CodecTables tab;
    __shared__ ReduceScratch scratch;
    __shared__ uint32_t s_go;
    __shared__ uint32_t s_last;
    if (KC >= 2) { load_tables(tab, &g_zero_codec_tables); init_scratch(scratch); }   // the entry round ends with a barrier
    uint32_t turn = 0;
    // ---- entry: publish "gradients final", wait for every peer (decided once by CTA 0) ----
    if (!peer_entry(peers, epoch, budget, status, &s_go)) return;   // nothing was touched
    if (clip_total_sq != nullptr) {
        // a failed first phase (status already set) left the gradient unreduced: update nothing
        if (*reinterpret_cast<const volatile uint32_t*>(status) != ZS_OK) return;
        // global-norm clipping: the squared norm of the whole reduced gradient was exchanged between the ranks by
        // zero_norm_exchange_kernel; every rank reads the same total and so applies the same coefficient
        const float total = sqrtf(*clip_total_sq);
        a.inv_scale *= fminf(clip_max_norm / (total + 1e-6f), 1.0f);
    }

    // ---- the shard: reduce, update, broadcast ----
    // (A cp.async look-ahead ring for the remote gradients was tried and removed: on 2 GPUs it took 18.0 ms
    // against 11.6 ms for plain peer loads on the same 3.49 G parameters.  The plain path already runs the
    // links at ~600 GB/s per direction there: each direction carries one rank's parameter stores plus the
    // responses to the other rank's gradient loads.)
    PeerIO<WORLD, MC> io{&peers, g_dtype, p_dtype};
    {
        // chunk walk: round-robin by default (every CTA then works inside the same few megabytes of each
        // rank's buffers), else one contiguous range per CTA
        const uint32_t per_cta = (a.total_chunks + gridDim.x - 1) / gridDim.x;
        const bool rr = (a.interleave & 1u) != 0;
        const uint32_t stride = rr ? gridDim.x : 1u;
        const uint32_t begin = rr ? blockIdx.x : blockIdx.x * per_cta;
        const uint32_t end = rr ? a.total_chunks : min(begin + per_cta, a.total_chunks);
        if (begin < end) {
            ChunkCursor cur;
            cur.init(segs, a.num_segments, a.total_chunks, begin);
            for (uint32_t chunk = begin; chunk < end; chunk += stride) {
                cur.seek(chunk);
                if (a.interleave & kTuneCheckTable) {     // debug mode: a bad record is skipped, the flag rounds still complete
                    const uint32_t fault = table_fault(cur.s, cur.si, a.num_segments, chunk, cur.seg_end, KC >= 2, false);
                    if (fault != TF_NONE) { record_table_fault(g_zero_table_fault, fault, cur.si, chunk); continue; }
                }
                const uint32_t c = chunk - cur.s.chunk_begin;
                const uint32_t ahead = chunk + 2 * stride;
                if (ahead < cur.seg_end && ahead < end) {
                    const uint32_t ca = ahead - cur.s.chunk_begin;
                    prefetch_chunk(cur.s, ca, false);
                    if (threadIdx.x == 32 && g_dtype == DT_BF16 && (cur.s.flags & SEG_FAST) &&
                        (static_cast<long long>(ca) + 1) * kChunk <= cur.s.numel)                 // this rank's own gradient, full chunks only
                        l2_prefetch(reinterpret_cast<const uint16_t*>(peers.grad[peers.grad_sources == 1 ? 0 : peers.rank]) +
                                        cur.s.offset + static_cast<long long>(ca) * kChunk, kChunk * 2);
                }
                if (KC == 0) dense_chunk<false>(cur.s, a, c, io);
                else if (KC == 1) dense_chunk<true>(cur.s, a, c, io);
                else if (KC == 2) quant_chunk<false, false>(cur.s, a, c, io, tab, scratch, turn);
                else if (KC == 3) quant_chunk<true, false>(cur.s, a, c, io, tab, scratch, turn);
                else quant_chunk<true, true>(cur.s, a, c, io, tab, scratch, turn);
            }
        }
    }

    // ---- exit: last CTA tells every peer "my writes to you are complete" and waits for theirs ----
    peer_exit(peers, epoch, budget, status, &s_last);
}

// ---------------------------------------------------------------------------
// Global-norm clipping inside the fused step needs the norm of the REDUCED gradient before any parameter moves, so a
// clipped step runs in two phases:
//   1. zero_reduce_kernel: reduce-scatter only - sum the shard's gradient over the ranks (peer loads), scale it,
//      write it back over this rank's own copy of the shard (bf16) and add up its squares;
//      zero_norm_exchange_kernel: the ranks swap their partial sums through the signal pads (4 bytes each way);
//   2. zero_fused_kernel with the total: update with the clip coefficient and all-gather, reading the already reduced
//      local gradient (grad_sources = 1).
// No collective library call anywhere on the step.
// ---------------------------------------------------------------------------
constexpr int kNormFlagBase = 32;      // signal pad words [32, 40): "my partial sum is in your pad" flags (epoch)
constexpr int kNormValueBase = 40;     // signal pad words [40, 48): the partial sums (fp32 bits), one slot per rank

template <int WORLD>
__global__ void __launch_bounds__(kThreads, 3)
zero_reduce_kernel(const SegDesc* __restrict__ segs, int num_segments, uint32_t total_chunks, ZeroPeers peers, uint32_t epoch,
                   long long budget, uint32_t* __restrict__ status, float inv_scale, float* __restrict__ cta_partials,
                   float* __restrict__ group_acc) {
    __shared__ uint32_t s_go;
    __shared__ uint32_t s_last;
    __shared__ float s_red[kThreads / 32];
    if (!peer_entry(peers, epoch, budget, status, &s_go)) return;
    const int W = WORLD > 0 ? WORLD : peers.world;
    uint16_t* own = reinterpret_cast<uint16_t*>(const_cast<void*>(peers.grad[peers.rank]));
    float sq = 0.0f;
    if (blockIdx.x < total_chunks) {
        ChunkCursor cur;
        cur.init(segs, num_segments, total_chunks, blockIdx.x);
        for (uint32_t chunk = blockIdx.x; chunk < total_chunks; chunk += gridDim.x) {
            cur.seek(chunk);
            const long long idx = static_cast<long long>(chunk - cur.s.chunk_begin) * kChunk + threadIdx.x * kPerThread;
            const long long left = cur.s.numel - idx;
            const int nvalid = left >= 8 ? 8 : (left > 0 ? static_cast<int>(left) : 0);
            if (nvalid == 0) continue;
            const long long e = cur.s.offset + idx;
            float g[8];
            if (nvalid == 8 && (e & 7) == 0) {
                uint4 raw[kMaxPeers];
#pragma unroll
                for (int r = 0; r < kMaxPeers; ++r)
                    if (r < W) raw[r] = __ldcs(reinterpret_cast<const uint4*>(reinterpret_cast<const uint16_t*>(peers.grad[r]) + e));
                unpack8(raw[0], g);
#pragma unroll
                for (int r = 1; r < kMaxPeers; ++r) {
                    if (r < W) {
                        float t[8];
                        unpack8(raw[r], t);
#pragma unroll
                        for (int k = 0; k < 8; ++k) g[k] += t[k];
                    }
                }
                uint32_t w[4];
#pragma unroll
                for (int k = 0; k < 4; ++k) {
                    w[k] = pack2_rn(sanitize_grad(g[2 * k]) * inv_scale, sanitize_grad(g[2 * k + 1]) * inv_scale);
                    const float lo = lo_bf16(w[k]), hi = hi_bf16(w[k]);     // the values the update will read back
                    sq = fmaf(lo, lo, sq);
                    sq = fmaf(hi, hi, sq);
                }
                *reinterpret_cast<uint4*>(own + e) = make_uint4(w[0], w[1], w[2], w[3]);
            } else {
                for (int k = 0; k < nvalid; ++k) {
                    float acc = 0.0f;
                    for (int r = 0; r < W; ++r) acc += bf16_bits_to_float(reinterpret_cast<const uint16_t*>(peers.grad[r])[e + k]);
                    const uint32_t w = pack2_rn(sanitize_grad(acc) * inv_scale, 0.0f);
                    const float v = lo_bf16(w);
                    sq = fmaf(v, v, sq);
                    own[e + k] = static_cast<uint16_t>(w & 0xFFFFu);
                }
            }
        }
    }
    // CTA sum in a fixed order, one slot per CTA; the last CTA adds the slots up in index order (deterministic)
    for (int off = 16; off > 0; off >>= 1) sq += __shfl_xor_sync(0xFFFFFFFFu, sq, off);
    if ((threadIdx.x & 31) == 0) s_red[threadIdx.x >> 5] = sq;
    __syncthreads();
    if (threadIdx.x == 0) {
        float t = 0.0f;
        for (int i = 0; i < kThreads / 32; ++i) t += s_red[i];
        cta_partials[blockIdx.x] = t;
        __threadfence();
        uint32_t* done = peers.signal[peers.rank] + 2 * kMaxPeers + 1;
        s_last = (atomicAdd(done, 1u) == gridDim.x - 1) ? 1u : 0u;
    }
    __syncthreads();
    if (s_last && threadIdx.x == 0) {
        __threadfence();
        float t = 0.0f;
        for (unsigned i = 0; i < gridDim.x; ++i) t += *reinterpret_cast<volatile float*>(cta_partials + i);
        *group_acc += t;                                   // launches of one group follow each other on one stream
        *(peers.signal[peers.rank] + 2 * kMaxPeers + 1) = 0u;
    }
}

// One CTA: publish this rank's partial sum of squares into every rank's pad, wait (bounded) for everybody's, add them
// up in rank order and leave the total in *total_out.  On a timeout the status word is set and the total is left at
// zero (no clipping); the status word tells the host that the step must not be trusted.
__global__ void zero_norm_exchange_kernel(ZeroPeers peers, uint32_t epoch, long long budget, uint32_t* __restrict__ status,
                                          float* __restrict__ group_acc, float* __restrict__ total_out) {
    __shared__ float s_val[kMaxPeers];
    __shared__ int s_ok;
    const int W = peers.world;
    const int r = threadIdx.x;
    if (r == 0) s_ok = 1;
    __syncthreads();
    if (r < W) {
        const float mine = *group_acc;
        uint32_t* theirs = peers.signal[r];
        *reinterpret_cast<volatile uint32_t*>(theirs + kNormValueBase + peers.rank) = __float_as_uint(mine);
        __threadfence_system();
        st_release_sys(theirs + kNormFlagBase + peers.rank, epoch);
        uint32_t* pad = peers.signal[peers.rank];
        if (!bounded_wait(pad + kNormFlagBase + r, epoch, budget)) {
            atomicExch(status, ZS_ENTRY_TIMEOUT);
            s_ok = 0;
            s_val[r] = 0.0f;
        } else {
            s_val[r] = __uint_as_float(*reinterpret_cast<volatile uint32_t*>(pad + kNormValueBase + r));
        }
    }
    __syncthreads();
    if (r == 0) {
        float t = 0.0f;
        for (int i = 0; i < W; ++i) t += s_val[i];
        *total_out = s_ok ? t : 0.0f;
        *group_acc = 0.0f;                                  // ready for the next step
    }
}

static bool g_zero_tables_ready[64] = {};
void fill_codec_tables(CodecTables& t);   // fused_state.cu

template <int KC, int WORLD, bool MC = false>
int launch_zero_w(const SegDesc* segs, const StepArgs& a, const ZeroPeers& peers, uint32_t epoch, long long budget,
                  uint32_t* status, int g_dtype, int p_dtype, int sm_count, cudaStream_t stream, const float* clip_total_sq,
                  float clip_max_norm) {
    int per_sm = 0;
    cudaError_t e = cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, zero_fused_kernel<KC, WORLD, MC>, kThreads, 0);
    if (e != cudaSuccess) return static_cast<int>(e);
    if (per_sm < 1) return static_cast<int>(cudaErrorLaunchOutOfResources);
    // every CTA must be resident: CTAs wait on a word that CTA 0 writes
    const int sm_cap = static_cast<int>((a.interleave >> 8) & 0xFFu);      // tuning word: CTAs per SM ...
    const unsigned total_cap = a.interleave >> 16;                          // ... and CTAs in total (launches beside other work)
    if (sm_cap > 0 && sm_cap < per_sm) per_sm = sm_cap;
    unsigned grid = static_cast<unsigned>(per_sm) * sm_count;
    if (total_cap > 0 && total_cap < grid) grid = total_cap;
    if (a.total_chunks < grid) grid = a.total_chunks > 0 ? a.total_chunks : 1;
    zero_fused_kernel<KC, WORLD, MC><<<grid, kThreads, 0, stream>>>(segs, a, peers, epoch, budget, status, g_dtype, p_dtype,
                                                                    clip_total_sq, clip_max_norm);
    return static_cast<int>(cudaGetLastError());
}

template <int KC>
int launch_zero(const SegDesc* segs, const StepArgs& a, const ZeroPeers& peers, uint32_t epoch, long long budget,
                uint32_t* status, int g_dtype, int p_dtype, int sm_count, cudaStream_t stream, const float* clip_total_sq,
                float clip_max_norm) {
    if (peers.mc_grad != nullptr && peers.mc_param != nullptr && peers.world > 1 && peers.grad_sources == peers.world &&
        g_dtype == DT_BF16 && p_dtype == DT_BF16)      // NVLS transport: one instantiation serves every world size
        return launch_zero_w<KC, 0, true>(segs, a, peers, epoch, budget, status, g_dtype, p_dtype, sm_count, stream, clip_total_sq, clip_max_norm);
    switch (peers.world) {
        case 1: return launch_zero_w<KC, 1>(segs, a, peers, epoch, budget, status, g_dtype, p_dtype, sm_count, stream, clip_total_sq, clip_max_norm);
        case 2: return launch_zero_w<KC, 2>(segs, a, peers, epoch, budget, status, g_dtype, p_dtype, sm_count, stream, clip_total_sq, clip_max_norm);
        case 4: return launch_zero_w<KC, 4>(segs, a, peers, epoch, budget, status, g_dtype, p_dtype, sm_count, stream, clip_total_sq, clip_max_norm);
        case 8: return launch_zero_w<KC, 8>(segs, a, peers, epoch, budget, status, g_dtype, p_dtype, sm_count, stream, clip_total_sq, clip_max_norm);
        default: return launch_zero_w<KC, 0>(segs, a, peers, epoch, budget, status, g_dtype, p_dtype, sm_count, stream, clip_total_sq, clip_max_norm);
    }
}

}  // namespace apexb

using namespace apexb;

extern "C" int apexb_zero_init(int device) {
    if (device < 0 || device >= 64) return cudaErrorInvalidDevice;
    if (g_zero_tables_ready[device]) return 0;
    CodecTables t;
    fill_codec_tables(t);
    cudaError_t e = cudaMemcpyToSymbol(g_zero_codec_tables, &t, sizeof(t));
    if (e != cudaSuccess) return static_cast<int>(e);
    g_zero_tables_ready[device] = true;
    return 0;
}

// Debug mode: copy out (and clear, when asked) this module's table-fault word: code, segment, chunk, skipped chunks.
extern "C" int apexb_zero_table_fault(unsigned out[4], int clear) {
    cudaError_t e = cudaMemcpyFromSymbol(out, g_zero_table_fault, 4 * sizeof(unsigned));
    if (e != cudaSuccess) return static_cast<int>(e);
    if (clear) {
        const unsigned zero[4] = {0, 0, 0, 0};
        e = cudaMemcpyToSymbol(g_zero_table_fault, zero, sizeof(zero));
    }
    return static_cast<int>(e);
}

extern "C" int apexb_zero_fused_launch(int kernel_class, const void* d_segments, const StepArgs* args, const ZeroPeers* peers,
                                        uint32_t epoch, long long wait_budget_cycles, uint32_t* status, int g_dtype,
                                        int p_dtype, int sm_count, const float* clip_total_sq, float clip_max_norm,
                                        cudaStream_t stream) {
    if (peers->world < 1 || peers->world > kMaxPeers) return cudaErrorInvalidValue;
    if (peers->grad_sources != 1 && peers->grad_sources != peers->world) return cudaErrorInvalidValue;
    const SegDesc* segs = static_cast<const SegDesc*>(d_segments);
    switch (kernel_class) {
        case 0: return launch_zero<0>(segs, *args, *peers, epoch, wait_budget_cycles, status, g_dtype, p_dtype, sm_count, stream, clip_total_sq, clip_max_norm);
        case 1: return launch_zero<1>(segs, *args, *peers, epoch, wait_budget_cycles, status, g_dtype, p_dtype, sm_count, stream, clip_total_sq, clip_max_norm);
        case 2: return launch_zero<2>(segs, *args, *peers, epoch, wait_budget_cycles, status, g_dtype, p_dtype, sm_count, stream, clip_total_sq, clip_max_norm);
        case 3: return launch_zero<3>(segs, *args, *peers, epoch, wait_budget_cycles, status, g_dtype, p_dtype, sm_count, stream, clip_total_sq, clip_max_norm);
        case 4: return launch_zero<4>(segs, *args, *peers, epoch, wait_budget_cycles, status, g_dtype, p_dtype, sm_count, stream, clip_total_sq, clip_max_norm);
        default: return cudaErrorInvalidValue;
    }
}

extern "C" int apexb_zero_reduce_launch(const void* d_segments, int num_segments, unsigned total_chunks, const ZeroPeers* peers,
                                         uint32_t epoch, long long wait_budget_cycles, uint32_t* status, float inv_scale,
                                         float* cta_partials, int cta_partials_len, float* group_acc, int sm_count,
                                         cudaStream_t stream) {
    if (peers->world < 1 || peers->world > kMaxPeers || peers->grad_sources != peers->world) return cudaErrorInvalidValue;
    int per_sm = 0;
    cudaError_t e = cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, zero_reduce_kernel<0>, kThreads, 0);
    if (e != cudaSuccess) return static_cast<int>(e);
    if (per_sm < 1) return static_cast<int>(cudaErrorLaunchOutOfResources);
    if (per_sm > 3) per_sm = 3;
    unsigned grid = static_cast<unsigned>(per_sm) * sm_count;       // every CTA resident: CTAs wait on CTA 0's verdict
    if (total_chunks < grid) grid = total_chunks > 0 ? total_chunks : 1;
    if (static_cast<int>(grid) > cta_partials_len) return cudaErrorInvalidValue;
    const SegDesc* segs = static_cast<const SegDesc*>(d_segments);
    switch (peers->world) {
        case 2: zero_reduce_kernel<2><<<grid, kThreads, 0, stream>>>(segs, num_segments, total_chunks, *peers, epoch, wait_budget_cycles, status, inv_scale, cta_partials, group_acc); break;
        case 4: zero_reduce_kernel<4><<<grid, kThreads, 0, stream>>>(segs, num_segments, total_chunks, *peers, epoch, wait_budget_cycles, status, inv_scale, cta_partials, group_acc); break;
        case 8: zero_reduce_kernel<8><<<grid, kThreads, 0, stream>>>(segs, num_segments, total_chunks, *peers, epoch, wait_budget_cycles, status, inv_scale, cta_partials, group_acc); break;
        default: zero_reduce_kernel<0><<<grid, kThreads, 0, stream>>>(segs, num_segments, total_chunks, *peers, epoch, wait_budget_cycles, status, inv_scale, cta_partials, group_acc); break;
    }
    return static_cast<int>(cudaGetLastError());
}

extern "C" int apexb_zero_norm_exchange(const ZeroPeers* peers, uint32_t epoch, long long wait_budget_cycles, uint32_t* status,
                                         float* group_acc, float* total_out, cudaStream_t stream) {
    if (peers->world < 1 || peers->world > kMaxPeers) return cudaErrorInvalidValue;
    zero_norm_exchange_kernel<<<1, 32, 0, stream>>>(*peers, epoch, wait_budget_cycles, status, group_acc, total_out);
    return static_cast<int>(cudaGetLastError());
}
