// Newton-Schulz GEMMs on the 5th-generation tensor cores (tcgen05 + TMEM), sm_100a only.
//
// One kernel serves the three products of a quintic Newton-Schulz step through
//     C[M,N] = alpha * A[M,K] * B[N,K]^T + beta * D[M,N]        (bf16 in/out, fp32 accumulate)
// with both operands K-major (the "TN" form), an optional transposed second output
// Ct[N,M] = C^T, and a batch index in grid.z:
//     A_ = X X^T              : A = X,  B = X,  alpha = 1, beta = 0
//     B_ = b A_ + c A_ A_     : A = A_, B = A_ (A_ is symmetric), alpha = c, beta = b, D = A_
//     X' = a X + B_ X         : A = B_, B = X^T kept as Y[N,M], alpha = 1, beta = a, D = X, Ct = Y'
// Keeping Y = X^T alongside X makes every operand K-major, so no MN-major descriptors are needed;
// Y' comes for free from the epilogue's transposed store.  The reference runs these products
// through cuBLAS (apexw/muon.py:102-108, :203-206).
//
// Persistent kernel, one CTA per SM (320 threads), looping over 128 x 256 (or 128 x 128) output tiles:
//   warp 0   : TMA producer  - cp.async.bulk.tensor (no multicast) into a 4-stage smem ring that runs across tiles
//   warp 1   : MMA issuer    - tcgen05.mma.cta_group::1.kind::f16 into one of two TMEM accumulators (2 x 256 columns)
//   warps 2-9: epilogue      - tcgen05.ld from the other accumulator, alpha/beta math, bf16 stores (plain, and
//                              transposed through a shared-memory staging block), overlapped with the next tile's MMAs;
//                              eight warps (two per TMEM lane quarter, half the columns each) keep it shorter than
//                              the main loop of the K = m products
// X X^T and b A + c A A are symmetric: their tiles strictly below the diagonal are not computed; the transposed
// store (Ct == C) fills them in, which removes 25-45 % of the tensor work of those two products.
// Every mbarrier wait is bounded; on expiry the CTA records an error code, frees its TMEM and leaves.
#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <cstdint>
#include <cstdlib>
#include "api.h"

namespace apexb {
namespace ns {

constexpr int BM = 128;
constexpr int BK = 64;                 // 64 bf16 = 128 bytes = one swizzle atom row
constexpr int UMMA_K = 16;
constexpr int EPI_WARPS = 8;                                 // two warps per TMEM lane quarter, each takes half of the tile's columns
constexpr int THREADS = 64 + EPI_WARPS * 32;                 // TMA warp, MMA warp, epilogue warps
constexpr uint32_t A_BYTES = BM * BK * 2;   // 16 KB

// Tile width BN is 256 (large problems) or 128 (more, smaller tiles when 256-wide tiles would leave most of
// the last wave of the 148 persistent CTAs idle).
template <int BN> struct Cfg {
    static constexpr int STAGES = BN == 256 ? 4 : 6;
    static constexpr uint32_t B_BYTES = BN * BK * 2;              // 32 KB or 16 KB
    static constexpr uint32_t STAGE_BYTES = A_BYTES + B_BYTES;
    static constexpr uint32_t ACC_COLS = BN;                      // fp32 accumulator columns of one tile
    static constexpr uint32_t TMEM_COLS = 2 * BN;                 // two accumulators: epilogue of tile i overlaps MMAs of tile i+1
};
constexpr int TPITCH = 40;                                   // staging row pitch in bf16 (32 rows + pad, 80 bytes: 16-byte aligned)
constexpr uint32_t TRANSPOSE_BYTES = EPI_WARPS * 32 * TPITCH * 2;   // one 32 x 32 staging block per epilogue warp
template <int BN> constexpr uint32_t smem_bytes() {
    return Cfg<BN>::STAGES * Cfg<BN>::STAGE_BYTES + TRANSPOSE_BYTES + 1024 /*alignment slack*/ + 256 /*barriers*/;
}
constexpr int MAX_STAGES = 6;
constexpr uint32_t kSpinLimit = 1u << 22;   // ~ a second of polling with back-off before giving up

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return static_cast<uint32_t>(__cvta_generic_to_shared(p)); }

__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count));
}
__device__ __forceinline__ void mbar_expect_tx(uint64_t* bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint64_t* bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n.reg .pred p;\n"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n"
        "selp.u32 %0, 1, 0, p;\n}"
        : "=r"(ok) : "r"(smem_u32(bar)), "r"(parity) : "memory");
    return ok != 0;
}
// bounded wait: false when the limit is reached
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity) {
    for (uint32_t i = 0; i < kSpinLimit; ++i) {
        if (mbar_try_wait(bar, parity)) return true;
        if (i > 64) __nanosleep(128);
    }
    return false;
}

__device__ __forceinline__ void tma_load_3d(void* dst, const CUtensorMap* map, uint64_t* bar, int c0, int c1, int c2) {
    asm volatile(
        "cp.async.bulk.tensor.3d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5}], [%2];"
        :: "r"(smem_u32(dst)), "l"(reinterpret_cast<uint64_t>(map)), "r"(smem_u32(bar)), "r"(c0), "r"(c1), "r"(c2)
        : "memory");
}

// shared-memory matrix descriptor: K-major operand, 128-byte swizzle, 8-row groups 1024 bytes apart
__device__ __forceinline__ uint64_t umma_desc_k_sw128(uint32_t smem_addr) {
    uint64_t d = 0;
    d |= static_cast<uint64_t>((smem_addr & 0x3FFFFu) >> 4);          // start address
    d |= static_cast<uint64_t>(1) << 16;                              // leading byte offset (unused with swizzle)
    d |= static_cast<uint64_t>(1024 >> 4) << 32;                      // stride byte offset
    d |= static_cast<uint64_t>(1) << 46;                              // descriptor version (sm_100)
    d |= static_cast<uint64_t>(2) << 61;                              // SWIZZLE_128B
    return d;
}

// instruction descriptor: D = fp32, A = B = bf16, both K-major, M x N
__host__ __device__ constexpr uint32_t umma_idesc(int M, int N) {
    return (1u << 4) | (1u << 7) | (1u << 10) | (static_cast<uint32_t>(N >> 3) << 17) | (static_cast<uint32_t>(M >> 4) << 24);
}

__device__ __forceinline__ void umma_bf16(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n.reg .pred p;\n"
        "setp.ne.b32 p, %4, 0;\n"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n}"
        :: "r"(tmem_d), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate) : "memory");
}
__device__ __forceinline__ void umma_commit(uint64_t* bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void tmem_ld32(uint32_t taddr, uint32_t (&r)[32]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
        "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
          "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]),
          "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]),
          "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
        : "r"(taddr) : "memory");
    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}

struct GemmArgs {
    const __nv_bfloat16* D;     // beta operand, [batch, M, N] (may be null when beta == 0)
    __nv_bfloat16* C;           // [batch, M, N]
    __nv_bfloat16* Ct;          // [batch, N, M] or null; equal to C when the output is symmetric
    long long strideD, strideC, strideCt;   // elements between batch entries
    int M, N, K, batch;
    int symmetric;              // M == N and C == C^T: tiles strictly below the diagonal are skipped and mirrored
    int tiles_per_batch;
    float alpha, beta;
};

// Tile t of a batch entry -> (row tile, column tile).  Symmetric outputs enumerate, for each BN-wide column
// tile j, only the row tiles i < (j + 1) * BN / BM (the others lie strictly below the diagonal).
template <int BN>
__device__ __forceinline__ void decode_tile(const GemmArgs& g, int t, int& mi, int& nj) {
    const int m_tiles = g.M / BM;
    if (!g.symmetric) { nj = t / m_tiles; mi = t - nj * m_tiles; return; }
    int j = 0;
    while (true) {
        const int rows = min(m_tiles, (j + 1) * (BN / BM));
        if (t < rows) break;
        t -= rows;
        ++j;
    }
    nj = j; mi = t;
}

struct Shared {
    uint64_t full_bar[MAX_STAGES];
    uint64_t empty_bar[MAX_STAGES];
    uint64_t tmem_full[2];
    uint64_t tmem_empty[2];
    uint32_t tmem_slot;
    uint32_t abort_flag;
};

// bounded wait that also gives up when another role of this CTA has aborted
__device__ __forceinline__ bool mbar_wait_or_abort(uint64_t* bar, uint32_t parity, const uint32_t* abort_flag) {
    // the producer and the MMA issuer sit on the critical path of the smem ring: poll without sleeping for a
    // long while (a sleep of 128 ns is a quarter of one k-block of tensor work), back off only when really idle
    for (uint32_t i = 0; i < kSpinLimit; ++i) {
        if (mbar_try_wait(bar, parity)) return true;
        if (i > 8192) {
            __nanosleep(256);
            if ((i & 1023u) == 0 && *reinterpret_cast<const volatile uint32_t*>(abort_flag)) return false;
        }
    }
    return false;
}
__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}

template <int BN>
__global__ void __launch_bounds__(THREADS, 1)
ns_gemm_kernel(const __grid_constant__ CUtensorMap mapA, const __grid_constant__ CUtensorMap mapB, GemmArgs g,
               uint32_t* __restrict__ error_flag) {
    constexpr int STAGES = Cfg<BN>::STAGES;
    constexpr uint32_t B_BYTES = Cfg<BN>::B_BYTES, STAGE_BYTES = Cfg<BN>::STAGE_BYTES;
    constexpr uint32_t ACC_COLS = Cfg<BN>::ACC_COLS, TMEM_COLS = Cfg<BN>::TMEM_COLS;
    extern __shared__ uint8_t smem_raw[];
    // 1024-byte alignment for the swizzled tiles
    uint8_t* tiles = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~static_cast<uintptr_t>(1023));
    uint16_t* stage_t = reinterpret_cast<uint16_t*>(tiles + STAGES * STAGE_BYTES);                 // transposed-store staging
    Shared* sh = reinterpret_cast<Shared*>(tiles + STAGES * STAGE_BYTES + TRANSPOSE_BYTES);

    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;
    const int k_blocks = (g.K + BK - 1) / BK;
    const int total_tiles = g.tiles_per_batch * g.batch;

    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; ++s) { mbar_init(&sh->full_bar[s], 1); mbar_init(&sh->empty_bar[s], 1); }
        for (int a = 0; a < 2; ++a) { mbar_init(&sh->tmem_full[a], 1); mbar_init(&sh->tmem_empty[a], EPI_WARPS); }
        sh->abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 1) {   // one warp allocates both accumulators (one CTA per SM)
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&sh->tmem_slot)), "r"(TMEM_COLS) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tmem_base = sh->tmem_slot;

    if (warp == 0) {
        // ---------------- TMA producer ----------------
        if (lane == 0) {
            uint32_t it = 0;
            bool ok = true;
            for (int tile = blockIdx.x; tile < total_tiles && ok; tile += gridDim.x) {
                const int batch = tile / g.tiles_per_batch;
                int mi, nj;
                decode_tile<BN>(g, tile - batch * g.tiles_per_batch, mi, nj);
                for (int kb = 0; kb < k_blocks; ++kb, ++it) {
                    const uint32_t s = it % STAGES;
                    const uint32_t parity = ((it / STAGES) & 1u) ^ 1u;
                    if (!mbar_wait_or_abort(&sh->empty_bar[s], parity, &sh->abort_flag)) {
                        atomicExch(error_flag, 1u); sh->abort_flag = 1; ok = false; break;
                    }
                    uint8_t* a_dst = tiles + s * STAGE_BYTES;
                    uint8_t* b_dst = a_dst + A_BYTES;
                    (void)B_BYTES;
                    mbar_expect_tx(&sh->full_bar[s], STAGE_BYTES);
                    tma_load_3d(a_dst, &mapA, &sh->full_bar[s], kb * BK, mi * BM, batch);
                    tma_load_3d(b_dst, &mapB, &sh->full_bar[s], kb * BK, nj * BN, batch);
                }
            }
        }
    } else if (warp == 1) {
        // ---------------- MMA issuer ----------------
        if (lane == 0) {
            constexpr uint32_t idesc = umma_idesc(BM, BN);
            uint32_t it = 0, tcount = 0;
            bool ok = true;
            for (int tile = blockIdx.x; tile < total_tiles && ok; tile += gridDim.x, ++tcount) {
                const uint32_t acc = tcount & 1u;
                // the epilogue must have drained this accumulator (used two tiles ago)
                if (!mbar_wait_or_abort(&sh->tmem_empty[acc], ((tcount >> 1) & 1u) ^ 1u, &sh->abort_flag)) {
                    atomicExch(error_flag, 4u); sh->abort_flag = 1; break;
                }
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                const uint32_t tmem_d = tmem_base + acc * ACC_COLS;
                for (int kb = 0; kb < k_blocks; ++kb, ++it) {
                    const uint32_t s = it % STAGES;
                    if (!mbar_wait_or_abort(&sh->full_bar[s], (it / STAGES) & 1u, &sh->abort_flag)) {
                        atomicExch(error_flag, 2u); sh->abort_flag = 1; ok = false; break;
                    }
                    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                    const uint32_t a_addr = smem_u32(tiles + s * STAGE_BYTES);
                    const uint32_t b_addr = a_addr + A_BYTES;
#pragma unroll
                    for (int k = 0; k < BK / UMMA_K; ++k) {
                        const uint64_t adesc = umma_desc_k_sw128(a_addr + k * UMMA_K * 2);
                        const uint64_t bdesc = umma_desc_k_sw128(b_addr + k * UMMA_K * 2);
                        umma_bf16(tmem_d, adesc, bdesc, idesc, (kb > 0 || k > 0) ? 1u : 0u);
                    }
                    umma_commit(&sh->empty_bar[s]);      // frees the smem stage once these MMAs have read it
                }
                if (ok) umma_commit(&sh->tmem_full[acc]);   // accumulator complete
            }
        }
    } else {
        // ---------------- epilogue (warps 2..5), overlapped with the next tile's main loop ----------------
        const int lane_group = warp & 3;                       // TMEM lanes 32*lane_group .. +31 belong to this warp
        constexpr int HALF = BN / 2;
        const int cbase = ((warp - 2) >> 2) * HALF;            // this warp's half of the tile's columns
        uint16_t* my_stage = stage_t + (warp - 2) * (32 * TPITCH);
        uint32_t tcount = 0;
        for (int tile = blockIdx.x; tile < total_tiles; tile += gridDim.x, ++tcount) {
            const int batch = tile / g.tiles_per_batch;
            int mi, nj;
            decode_tile<BN>(g, tile - batch * g.tiles_per_batch, mi, nj);
            const int m0 = mi * BM, n0 = nj * BN;
            const uint32_t acc = tcount & 1u;
            const int row = m0 + lane_group * 32 + lane;        // always < M (M is a multiple of BM)
            const __nv_bfloat16* Drow = g.D ? g.D + batch * g.strideD + static_cast<long long>(row) * g.N : nullptr;
            __nv_bfloat16* Crow = g.C + batch * g.strideC + static_cast<long long>(row) * g.N;
            uint16_t* Ctb = g.Ct ? reinterpret_cast<uint16_t*>(g.Ct + batch * g.strideCt) : nullptr;
            // the beta operand does not depend on the accumulator: fetch the first block before waiting for it
            uint4 dnext[4];
            if (Drow != nullptr) {
#pragma unroll
                for (int q = 0; q < 4; ++q)
                    dnext[q] = (n0 + cbase + q * 8 < g.N) ? __ldg(reinterpret_cast<const uint4*>(Drow + n0 + cbase + q * 8))
                                                          : make_uint4(0, 0, 0, 0);
            }
            bool ok = mbar_wait_or_abort(&sh->tmem_full[acc], (tcount >> 1) & 1u, &sh->abort_flag);
            if (!ok && lane == 0) { atomicExch(error_flag, 3u); sh->abort_flag = 1; }
            ok = __shfl_sync(0xFFFFFFFFu, ok ? 1 : 0, 0) != 0;
            if (!ok) break;
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            const uint32_t taddr = tmem_base + acc * ACC_COLS + (static_cast<uint32_t>(lane_group * 32) << 16);
#pragma unroll 1
            for (int c0 = cbase; c0 < cbase + HALF; c0 += 32) {
                const int col = n0 + c0;
                if (col >= g.N) break;                 // uniform over the warp
                uint32_t accv[32];
                tmem_ld32(taddr + static_cast<uint32_t>(c0), accv);
                uint4 dcur[4];
                if (Drow != nullptr) {
#pragma unroll
                    for (int q = 0; q < 4; ++q) dcur[q] = dnext[q];
                    if (c0 + 32 < cbase + HALF) {
#pragma unroll
                        for (int q = 0; q < 4; ++q)
                            dnext[q] = (col + 32 + q * 8 < g.N) ? __ldg(reinterpret_cast<const uint4*>(Drow + col + 32 + q * 8))
                                                                : make_uint4(0, 0, 0, 0);
                    }
                }
                float v[32];
#pragma unroll
                for (int j = 0; j < 32; ++j) v[j] = __uint_as_float(accv[j]) * g.alpha;
                if (Drow != nullptr) {
#pragma unroll
                    for (int q = 0; q < 4; ++q) {
                        const uint32_t w[4] = {dcur[q].x, dcur[q].y, dcur[q].z, dcur[q].w};
#pragma unroll
                        for (int t = 0; t < 4; ++t) {
                            v[q * 8 + 2 * t] = fmaf(g.beta, __uint_as_float(w[t] << 16), v[q * 8 + 2 * t]);
                            v[q * 8 + 2 * t + 1] = fmaf(g.beta, __uint_as_float(w[t] & 0xFFFF0000u), v[q * 8 + 2 * t + 1]);
                        }
                    }
                }
                uint32_t packed[16];
#pragma unroll
                for (int j = 0; j < 16; ++j) {
                    const __nv_bfloat162 h = __floats2bfloat162_rn(v[2 * j], v[2 * j + 1]);
                    packed[j] = *reinterpret_cast<const uint32_t*>(&h);
                }
#pragma unroll
                for (int q = 0; q < 4; ++q)
                    if (col + q * 8 < g.N)
                        *reinterpret_cast<uint4*>(Crow + col + q * 8) =
                            make_uint4(packed[4 * q], packed[4 * q + 1], packed[4 * q + 2], packed[4 * q + 3]);
                if (Ctb != nullptr) {
                    // transposed copy through shared memory: stage[c][r] <- value(row r, column c), then 16-byte
                    // row segments of C^T (8 consecutive rows of one column) go out as vector stores
                    __syncwarp();
#pragma unroll
                    for (int j = 0; j < 16; ++j) {
                        my_stage[(2 * j) * TPITCH + lane] = static_cast<uint16_t>(packed[j] & 0xFFFFu);
                        my_stage[(2 * j + 1) * TPITCH + lane] = static_cast<uint16_t>(packed[j] >> 16);
                    }
                    __syncwarp();
                    const int r8 = (lane & 3) * 8;                   // 8-row segment inside the warp's 32 rows
#pragma unroll
                    for (int pass = 0; pass < 4; ++pass) {
                        const int c = pass * 8 + (lane >> 2);
                        if (col + c < g.N) {
                            const uint4 seg = *reinterpret_cast<const uint4*>(my_stage + c * TPITCH + r8);
                            *reinterpret_cast<uint4*>(Ctb + static_cast<long long>(col + c) * g.M + (m0 + lane_group * 32 + r8)) = seg;
                        }
                    }
                }
            }
            // all of this warp's TMEM reads are complete (tcgen05.wait::ld inside tmem_ld32): hand the accumulator back
            asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
            __syncwarp();
            if (lane == 0) mbar_arrive(&sh->tmem_empty[acc]);
        }
    }

    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (*reinterpret_cast<volatile uint32_t*>(&sh->abort_flag)) {
        // give bulk copies that may still be in flight time to land before the CTA's smem goes away
        for (int i = 0; i < 2000; ++i) __nanosleep(1000);
        __syncthreads();
    }
    if (warp == 1) {
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(TMEM_COLS) : "memory");
    }
}

// ---------------------------------------------------------------------------
// Two-CTA variant: a pair of CTAs on the two SMs of one TPC (a cluster of two) computes one 256 x 256 tile with
// tcgen05.mma.cta_group::2.  Each CTA loads ITS 128 rows of A and ITS 128 rows of B per k-block (its own TMA, no
// multicast), holds the 128 x 256 fp32 accumulator of its rows in its own TMEM and runs its own epilogue.  Per SM
// and k-block that is 32 KB of operands for 128 x 256 x 64 multiply-adds instead of 48 KB: the one-CTA kernel is
// bound by the L2 -> SM operand stream, not by the tensor pipe.  The smaller stage also buys a 6-deep ring.
//   both CTAs, warp 0 : TMA producer; the transaction bytes of both CTAs land on the LEADER's full barrier
//   leader,    warp 1 : MMA issuer (one thread); tcgen05.commit with a cluster mask frees the stage in both CTAs and
//                       publishes a finished accumulator to both epilogues
//   both CTAs, warps 2-9 : epilogue of their own rows; "accumulator drained" arrives on the leader's barrier
// Barrier traffic between the CTAs goes through shared::cluster addresses from mapa; every wait is bounded.
// ---------------------------------------------------------------------------
namespace two {

constexpr int BN2 = 256;                    // tile width; the pair covers 256 rows
constexpr int STAGES2 = 6;
constexpr uint32_t HALF_B_BYTES = 128 * BK * 2;                       // this CTA's half of B: 16 KB
constexpr uint32_t STAGE2_BYTES = A_BYTES + HALF_B_BYTES;            // 32 KB
constexpr uint32_t TMEM_COLS2 = 2 * BN2;
constexpr uint32_t smem_bytes2() { return STAGES2 * STAGE2_BYTES + TRANSPOSE_BYTES + 1024 + 256; }

__device__ __forceinline__ uint32_t cluster_ctarank() {
    uint32_t r;
    asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
    return r;
}
// shared::cluster address of `local` (a shared::cta address of this CTA) in the CTA of rank `rank`
__device__ __forceinline__ uint32_t map_to_cta(uint32_t local, uint32_t rank) {
    uint32_t r;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(local), "r"(rank));
    return r;
}
__device__ __forceinline__ void cluster_sync() {
    asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
    asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
}
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t cluster_addr) {
    asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(cluster_addr) : "memory");
}
// this CTA's TMA load whose completion bytes are counted on the barrier at `bar_cluster_addr` (the leader's)
__device__ __forceinline__ void tma_load_3d_pair(void* dst, const CUtensorMap* map, uint32_t bar_cluster_addr, int c0, int c1, int c2) {
    asm volatile(
        "cp.async.bulk.tensor.3d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5}], [%2];"
        :: "r"(smem_u32(dst)), "l"(reinterpret_cast<uint64_t>(map)), "r"(bar_cluster_addr), "r"(c0), "r"(c1), "r"(c2)
        : "memory");
}
__device__ __forceinline__ void umma_bf16_pair(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n.reg .pred p;\n"
        "setp.ne.b32 p, %4, 0;\n"
        "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n}"
        :: "r"(tmem_d), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate) : "memory");
}
// arrive on the barrier at the same offset in both CTAs of the pair once the MMAs issued so far have completed
__device__ __forceinline__ void umma_commit_pair(uint64_t* bar) {
    const uint16_t mask = 3;
    asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;"
                 ::"r"(smem_u32(bar)), "h"(mask) : "memory");
}

// Tile t of a batch entry -> (row tile, column tile) of 256 x 256 tiles; symmetric outputs keep i <= j only.
__device__ __forceinline__ void decode_tile2(const GemmArgs& g, int t, int& mi, int& nj) {
    const int m_tiles = g.M / 256;
    if (!g.symmetric) { nj = t / m_tiles; mi = t - nj * m_tiles; return; }
    int j = 0;
    while (t > j) { t -= j + 1; ++j; }
    nj = j; mi = t;
}

__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(THREADS, 1)
ns_gemm2_kernel(const __grid_constant__ CUtensorMap mapA, const __grid_constant__ CUtensorMap mapB, GemmArgs g,
                uint32_t* __restrict__ error_flag) {
    extern __shared__ uint8_t smem_raw[];
    uint8_t* tiles = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~static_cast<uintptr_t>(1023));
    uint16_t* stage_t = reinterpret_cast<uint16_t*>(tiles + STAGES2 * STAGE2_BYTES);
    Shared* sh = reinterpret_cast<Shared*>(tiles + STAGES2 * STAGE2_BYTES + TRANSPOSE_BYTES);

    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;
    const uint32_t rank = cluster_ctarank();            // 0: leader (issues the MMAs), 1: peer
    const int pair = blockIdx.x >> 1;
    const int pairs = gridDim.x >> 1;
    const int k_blocks = (g.K + BK - 1) / BK;
    const int total_tiles = g.tiles_per_batch * g.batch;

    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES2; ++s) { mbar_init(&sh->full_bar[s], 1); mbar_init(&sh->empty_bar[s], 1); }
        for (int a = 0; a < 2; ++a) { mbar_init(&sh->tmem_full[a], 1); mbar_init(&sh->tmem_empty[a], 2 * EPI_WARPS); }
        sh->abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 1) {   // the same warp of both CTAs allocates the pair's accumulators
        asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&sh->tmem_slot)), "r"(TMEM_COLS2) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    cluster_sync();                                       // both CTAs' barriers exist before anyone signals across
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tmem_base = sh->tmem_slot;

    if (warp == 0) {
        // ---------------- TMA producer (both CTAs) ----------------
        if (lane == 0) {
            uint32_t it = 0;
            bool ok = true;
            for (int tile = pair; tile < total_tiles && ok; tile += pairs) {
                const int batch = tile / g.tiles_per_batch;
                int mi, nj;
                decode_tile2(g, tile - batch * g.tiles_per_batch, mi, nj);
                for (int kb = 0; kb < k_blocks; ++kb, ++it) {
                    const uint32_t s = it % STAGES2;
                    const uint32_t parity = ((it / STAGES2) & 1u) ^ 1u;
                    if (!mbar_wait_or_abort(&sh->empty_bar[s], parity, &sh->abort_flag)) {
                        atomicExch(error_flag, 11u); sh->abort_flag = 1; ok = false; break;
                    }
                    uint8_t* a_dst = tiles + s * STAGE2_BYTES;
                    uint8_t* b_dst = a_dst + A_BYTES;
                    if (rank == 0) mbar_expect_tx(&sh->full_bar[s], 2 * STAGE2_BYTES);      // both CTAs' bytes
                    const uint32_t bar = map_to_cta(smem_u32(&sh->full_bar[s]), 0);
                    tma_load_3d_pair(a_dst, &mapA, bar, kb * BK, mi * 256 + static_cast<int>(rank) * 128, batch);
                    tma_load_3d_pair(b_dst, &mapB, bar, kb * BK, nj * 256 + static_cast<int>(rank) * 128, batch);
                }
            }
        }
    } else if (warp == 1) {
        // ---------------- MMA issuer (leader only) ----------------
        if (rank == 0 && lane == 0) {
            constexpr uint32_t idesc = umma_idesc(256, BN2);
            uint32_t it = 0, tcount = 0;
            bool ok = true;
            for (int tile = pair; tile < total_tiles && ok; tile += pairs, ++tcount) {
                const uint32_t acc = tcount & 1u;
                if (!mbar_wait_or_abort(&sh->tmem_empty[acc], ((tcount >> 1) & 1u) ^ 1u, &sh->abort_flag)) {
                    atomicExch(error_flag, 14u); sh->abort_flag = 1; break;
                }
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                const uint32_t tmem_d = tmem_base + acc * BN2;
                for (int kb = 0; kb < k_blocks; ++kb, ++it) {
                    const uint32_t s = it % STAGES2;
                    if (!mbar_wait_or_abort(&sh->full_bar[s], (it / STAGES2) & 1u, &sh->abort_flag)) {
                        atomicExch(error_flag, 12u); sh->abort_flag = 1; ok = false; break;
                    }
                    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                    const uint32_t a_addr = smem_u32(tiles + s * STAGE2_BYTES);
                    const uint32_t b_addr = a_addr + A_BYTES;
#pragma unroll
                    for (int k = 0; k < BK / UMMA_K; ++k) {
                        const uint64_t adesc = umma_desc_k_sw128(a_addr + k * UMMA_K * 2);
                        const uint64_t bdesc = umma_desc_k_sw128(b_addr + k * UMMA_K * 2);
                        umma_bf16_pair(tmem_d, adesc, bdesc, idesc, (kb > 0 || k > 0) ? 1u : 0u);
                    }
                    umma_commit_pair(&sh->empty_bar[s]);      // frees the stage in both CTAs
                }
                if (ok) umma_commit_pair(&sh->tmem_full[acc]);   // accumulator complete, for both epilogues
            }
        }
    } else {
        // ---------------- epilogue of this CTA's 128 rows ----------------
        const int lane_group = warp & 3;
        constexpr int HALF = BN2 / 2;
        const int cbase = ((warp - 2) >> 2) * HALF;
        uint16_t* my_stage = stage_t + (warp - 2) * (32 * TPITCH);
        uint32_t tcount = 0;
        for (int tile = pair; tile < total_tiles; tile += pairs, ++tcount) {
            const int batch = tile / g.tiles_per_batch;
            int mi, nj;
            decode_tile2(g, tile - batch * g.tiles_per_batch, mi, nj);
            const int m0 = mi * 256 + static_cast<int>(rank) * 128, n0 = nj * BN2;
            const uint32_t acc = tcount & 1u;
            const int row = m0 + lane_group * 32 + lane;
            const __nv_bfloat16* Drow = g.D ? g.D + batch * g.strideD + static_cast<long long>(row) * g.N : nullptr;
            __nv_bfloat16* Crow = g.C + batch * g.strideC + static_cast<long long>(row) * g.N;
            uint16_t* Ctb = g.Ct ? reinterpret_cast<uint16_t*>(g.Ct + batch * g.strideCt) : nullptr;
            uint4 dnext[4];
            if (Drow != nullptr) {
#pragma unroll
                for (int q = 0; q < 4; ++q)
                    dnext[q] = (n0 + cbase + q * 8 < g.N) ? __ldg(reinterpret_cast<const uint4*>(Drow + n0 + cbase + q * 8))
                                                          : make_uint4(0, 0, 0, 0);
            }
            bool ok = mbar_wait_or_abort(&sh->tmem_full[acc], (tcount >> 1) & 1u, &sh->abort_flag);
            if (!ok && lane == 0) { atomicExch(error_flag, 13u); sh->abort_flag = 1; }
            ok = __shfl_sync(0xFFFFFFFFu, ok ? 1 : 0, 0) != 0;
            if (!ok) break;
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            const uint32_t taddr = tmem_base + acc * BN2 + (static_cast<uint32_t>(lane_group * 32) << 16);
#pragma unroll 1
            for (int c0 = cbase; c0 < cbase + HALF; c0 += 32) {
                const int col = n0 + c0;
                if (col >= g.N) break;
                uint32_t accv[32];
                tmem_ld32(taddr + static_cast<uint32_t>(c0), accv);
                uint4 dcur[4];
                if (Drow != nullptr) {
#pragma unroll
                    for (int q = 0; q < 4; ++q) dcur[q] = dnext[q];
                    if (c0 + 32 < cbase + HALF) {
#pragma unroll
                        for (int q = 0; q < 4; ++q)
                            dnext[q] = (col + 32 + q * 8 < g.N) ? __ldg(reinterpret_cast<const uint4*>(Drow + col + 32 + q * 8))
                                                                : make_uint4(0, 0, 0, 0);
                    }
                }
                float v[32];
#pragma unroll
                for (int j = 0; j < 32; ++j) v[j] = __uint_as_float(accv[j]) * g.alpha;
                if (Drow != nullptr) {
#pragma unroll
                    for (int q = 0; q < 4; ++q) {
                        const uint32_t w[4] = {dcur[q].x, dcur[q].y, dcur[q].z, dcur[q].w};
#pragma unroll
                        for (int t = 0; t < 4; ++t) {
                            v[q * 8 + 2 * t] = fmaf(g.beta, __uint_as_float(w[t] << 16), v[q * 8 + 2 * t]);
                            v[q * 8 + 2 * t + 1] = fmaf(g.beta, __uint_as_float(w[t] & 0xFFFF0000u), v[q * 8 + 2 * t + 1]);
                        }
                    }
                }
                uint32_t packed[16];
#pragma unroll
                for (int j = 0; j < 16; ++j) {
                    const __nv_bfloat162 h = __floats2bfloat162_rn(v[2 * j], v[2 * j + 1]);
                    packed[j] = *reinterpret_cast<const uint32_t*>(&h);
                }
#pragma unroll
                for (int q = 0; q < 4; ++q)
                    if (col + q * 8 < g.N)
                        *reinterpret_cast<uint4*>(Crow + col + q * 8) =
                            make_uint4(packed[4 * q], packed[4 * q + 1], packed[4 * q + 2], packed[4 * q + 3]);
                if (Ctb != nullptr) {
                    __syncwarp();
#pragma unroll
                    for (int j = 0; j < 16; ++j) {
                        my_stage[(2 * j) * TPITCH + lane] = static_cast<uint16_t>(packed[j] & 0xFFFFu);
                        my_stage[(2 * j + 1) * TPITCH + lane] = static_cast<uint16_t>(packed[j] >> 16);
                    }
                    __syncwarp();
                    const int r8 = (lane & 3) * 8;
#pragma unroll
                    for (int pass = 0; pass < 4; ++pass) {
                        const int c = pass * 8 + (lane >> 2);
                        if (col + c < g.N) {
                            const uint4 seg = *reinterpret_cast<const uint4*>(my_stage + c * TPITCH + r8);
                            *reinterpret_cast<uint4*>(Ctb + static_cast<long long>(col + c) * g.M + (m0 + lane_group * 32 + r8)) = seg;
                        }
                    }
                }
            }
            asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
            __syncwarp();
            if (lane == 0) mbar_arrive_cluster(map_to_cta(smem_u32(&sh->tmem_empty[acc]), 0));   // the leader's barrier
        }
    }

    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (*reinterpret_cast<volatile uint32_t*>(&sh->abort_flag)) {
        for (int i = 0; i < 2000; ++i) __nanosleep(1000);    // let bulk copies in flight land
        __syncthreads();
    }
    cluster_sync();        // neither CTA leaves (or frees TMEM) while its partner may still touch its smem / TMEM
    if (warp == 1) {
        asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(TMEM_COLS2) : "memory");
    }
}

}  // namespace two

// Newton-Schulz input preparation in one pass: Xs = G * inv[batch] and its transpose XsT, both bf16.
// (The iteration keeps X and Y = X^T side by side so that every GEMM operand is K-major.)
// 64 x 64 tiles, 256 threads, two elements per thread and access; rows and cols are multiples of 64.
constexpr int PT = 64;
__global__ void __launch_bounds__(256)
ns_prep_kernel(const __nv_bfloat16* __restrict__ G, const float* __restrict__ inv, __nv_bfloat16* __restrict__ Xs,
               __nv_bfloat16* __restrict__ XsT, int rows, int cols) {
    __shared__ uint16_t tile[PT][PT + 2];
    const int b = blockIdx.z;
    const int r0 = blockIdx.y * PT, c0 = blockIdx.x * PT;
    const int tx = threadIdx.x & 31, ty = threadIdx.x >> 5;          // 32 x 8
    const float scale = inv[b];
    const long long base = static_cast<long long>(b) * rows * cols;
#pragma unroll
    for (int j = 0; j < PT / 8; ++j) {
        const int r = ty + 8 * j;
        const long long idx = base + static_cast<long long>(r0 + r) * cols + c0 + 2 * tx;
        const uint32_t w = *reinterpret_cast<const uint32_t*>(G + idx);
        const __nv_bfloat162 h = __floats2bfloat162_rn(__uint_as_float(w << 16) * scale, __uint_as_float(w & 0xFFFF0000u) * scale);
        const uint32_t o = *reinterpret_cast<const uint32_t*>(&h);
        *reinterpret_cast<uint32_t*>(Xs + idx) = o;
        tile[r][2 * tx] = static_cast<uint16_t>(o & 0xFFFFu);
        tile[r][2 * tx + 1] = static_cast<uint16_t>(o >> 16);
    }
    __syncthreads();
    const long long tbase = static_cast<long long>(b) * rows * cols;
#pragma unroll
    for (int j = 0; j < PT / 8; ++j) {
        const int tr = ty + 8 * j;                                  // row of the transpose = column of G
        const uint32_t o = static_cast<uint32_t>(tile[2 * tx][tr]) | (static_cast<uint32_t>(tile[2 * tx + 1][tr]) << 16);
        *reinterpret_cast<uint32_t*>(XsT + tbase + static_cast<long long>(c0 + tr) * rows + r0 + 2 * tx) = o;
    }
}

}  // namespace ns
}  // namespace apexb

using namespace apexb::ns;

namespace {

int tiles_per_batch(int M, int N, int bn, int symmetric) {
    const int m_tiles = M / BM, n_tiles = (N + bn - 1) / bn;
    if (!symmetric) return m_tiles * n_tiles;
    int total = 0;
    for (int j = 0; j < n_tiles; ++j) {
        const int rows = (j + 1) * (bn / BM);
        total += rows < m_tiles ? rows : m_tiles;
    }
    return total;
}

template <int BN>
int launch(const void* map_a, const void* map_b, const GemmArgs& g, long long total, int sm_count, unsigned* error_flag,
           cudaStream_t stream) {
    static bool configured = false;
    if (!configured) {
        cudaError_t e = cudaFuncSetAttribute(ns_gemm_kernel<BN>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem_bytes<BN>());
        if (e != cudaSuccess) return static_cast<int>(e);
        configured = true;
    }
    const unsigned grid = static_cast<unsigned>(total < sm_count ? total : sm_count);
    ns_gemm_kernel<BN><<<grid, THREADS, smem_bytes<BN>(), stream>>>(*static_cast<const CUtensorMap*>(map_a),
                                                                    *static_cast<const CUtensorMap*>(map_b), g, error_flag);
    return static_cast<int>(cudaGetLastError());
}

}  // namespace

namespace {

// time of one round of 256 x 256 pair tiles relative to one round of 128 x 256 one-CTA tiles (both are 128 x 256 per SM)
constexpr double kPairCostPerColumn = 0.90;

int tiles_per_batch2(int M, int N, int symmetric) {
    const int m_tiles = M / 256, n_tiles = (N + 255) / 256;
    if (!symmetric) return m_tiles * n_tiles;
    return n_tiles * (n_tiles + 1) / 2;          // M == N: row tiles i <= j for every column tile j
}

// clusters of two that can be resident at once (one CTA per SM, so at most half the SMs)
int max_pairs(int sm_count) {
    static int cached = -1;
    if (cached < 0) {
        cudaError_t e = cudaFuncSetAttribute(apexb::ns::two::ns_gemm2_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                             apexb::ns::two::smem_bytes2());
        if (e != cudaSuccess) { cudaGetLastError(); return 0; }
        cudaLaunchConfig_t cfg = {};
        cfg.gridDim = dim3(static_cast<unsigned>(sm_count & ~1), 1, 1);
        cfg.blockDim = dim3(THREADS, 1, 1);
        cfg.dynamicSmemBytes = apexb::ns::two::smem_bytes2();
        cudaLaunchAttribute attr;
        attr.id = cudaLaunchAttributeClusterDimension;
        attr.val.clusterDim.x = 2; attr.val.clusterDim.y = 1; attr.val.clusterDim.z = 1;
        cfg.attrs = &attr;
        cfg.numAttrs = 1;
        int n = 0;
        e = cudaOccupancyMaxActiveClusters(&n, apexb::ns::two::ns_gemm2_kernel, &cfg);
        if (e != cudaSuccess) { cudaGetLastError(); n = 0; }
        cached = n;
    }
    return cached < sm_count / 2 ? cached : sm_count / 2;
}

int launch2(const void* map_a, const void* map_b, const GemmArgs& g, long long total, int sm_count, unsigned* error_flag,
            cudaStream_t stream) {
    const int pairs_cap = max_pairs(sm_count);
    if (pairs_cap < 1) return static_cast<int>(cudaErrorLaunchOutOfResources);
    const unsigned pairs = static_cast<unsigned>(total < pairs_cap ? total : pairs_cap);
    apexb::ns::two::ns_gemm2_kernel<<<2 * pairs, THREADS, apexb::ns::two::smem_bytes2(), stream>>>(
        *static_cast<const CUtensorMap*>(map_a), *static_cast<const CUtensorMap*>(map_b), g, error_flag);
    return static_cast<int>(cudaGetLastError());
}

}  // namespace

extern "C" int apexb_ns_prep(const void* G, const float* inv, void* Xs, void* XsT, int batch, int rows, int cols,
                             cudaStream_t stream) {
    if (rows % PT != 0 || cols % PT != 0 || batch < 1 || batch > 65535) return cudaErrorInvalidValue;
    dim3 grid(cols / PT, rows / PT, batch);
    ns_prep_kernel<<<grid, 256, 0, stream>>>(static_cast<const __nv_bfloat16*>(G), inv, static_cast<__nv_bfloat16*>(Xs),
                                             static_cast<__nv_bfloat16*>(XsT), rows, cols);
    return static_cast<int>(cudaGetLastError());
}

extern "C" int apexb_ns_smem_bytes() { return static_cast<int>(smem_bytes<256>()); }

// Tile width for a problem: the 256-wide tile has the better operand reuse, the 128-wide one fills the last
// wave better.  Cost model: rounds of the persistent grid x tile width, 128-wide tiles charged 35 % extra
// (measured: at equal round counts a 128-wide launch takes 1.25-1.5x the time of a 256-wide one; the narrow
// tile only wins where it saves a whole round, e.g. batches of 1024-row matrices).
extern "C" int apexb_ns_pick_bn(int M, int N, int batch, int symmetric, int sm_count) {
    if (N <= 128) return 128;
    const long long t256 = static_cast<long long>(tiles_per_batch(M, N, 256, symmetric)) * batch;
    const long long t128 = static_cast<long long>(tiles_per_batch(M, N, 128, symmetric)) * batch;
    const double c256 = static_cast<double>((t256 + sm_count - 1) / sm_count) * 256.0;
    const double c128 = static_cast<double>((t128 + sm_count - 1) / sm_count) * 128.0 * 1.35;
    return c128 < c256 ? 128 : 256;
}

extern "C" int apexb_ns_pick_tile(int M, int N, int K, int batch, int symmetric, int sm_count) {
    static int mode = -1;                         // 0 never, 1 whenever legal, 2 by the cost model
    if (mode < 0) {
        const char* e = std::getenv("APEXW_B200_NS_PAIR");
        mode = e == nullptr ? 2 : (e[0] == '0' ? 0 : (e[0] == '1' ? 1 : 2));
    }
    const int bn = apexb_ns_pick_bn(M, N, batch, symmetric, sm_count);
    if (mode == 0 || M % 256 != 0 || N < 256) return bn;
    const int pairs = max_pairs(sm_count);
    if (pairs < 1) return bn;
    if (mode == 1) return 512;
    // rounds of the persistent grid, weighted by tile area; a CTA pair moves 2/3 of the operand bytes per FLOP of the
    // one-CTA 128 x 256 tile, which is what bounds that kernel
    const long long t2 = static_cast<long long>(tiles_per_batch2(M, N, symmetric)) * batch;
    const long long t1 = static_cast<long long>(tiles_per_batch(M, N, bn, symmetric)) * batch;
    const double c2 = static_cast<double>((t2 + pairs - 1) / pairs) * 256.0 * kPairCostPerColumn;
    const double c1 = static_cast<double>((t1 + sm_count - 1) / sm_count) * bn * (bn == 128 ? 1.35 : 1.0);
    (void)K;
    return c2 < c1 ? 512 : bn;
}

extern "C" int apexb_ns_gemm(const void* tensor_map_a, const void* tensor_map_b, const void* D, void* C, void* Ct,
                             long long strideD, long long strideC, long long strideCt, int M, int N, int K, int batch,
                             float alpha, float beta, int symmetric, int bn, int sm_count, unsigned* error_flag,
                             cudaStream_t stream) {
    if (M % BM != 0 || N % 8 != 0 || K % 8 != 0 || batch < 1 || sm_count < 1) return cudaErrorInvalidValue;
    if (bn != 128 && bn != 256 && bn != 512) return cudaErrorInvalidValue;
    if (bn == 512 && M % 256 != 0) return cudaErrorInvalidValue;
    if (Ct != nullptr && M % 8 != 0) return cudaErrorInvalidValue;
    if (symmetric && (M != N || Ct != C || strideCt != strideC)) return cudaErrorInvalidValue;
    GemmArgs g;
    g.D = static_cast<const __nv_bfloat16*>(D);
    g.C = static_cast<__nv_bfloat16*>(C);
    g.Ct = static_cast<__nv_bfloat16*>(Ct);
    g.strideD = strideD; g.strideC = strideC; g.strideCt = strideCt;
    g.M = M; g.N = N; g.K = K; g.batch = batch; g.alpha = alpha; g.beta = beta;
    g.symmetric = symmetric ? 1 : 0;
    g.tiles_per_batch = bn == 512 ? tiles_per_batch2(M, N, g.symmetric) : tiles_per_batch(M, N, bn, g.symmetric);
    const long long total = static_cast<long long>(g.tiles_per_batch) * batch;
    if (total > 0x7FFFFFFFLL) return cudaErrorInvalidValue;
    if (bn == 512) return launch2(tensor_map_a, tensor_map_b, g, total, sm_count, error_flag, stream);
    return bn == 256 ? launch<256>(tensor_map_a, tensor_map_b, g, total, sm_count, error_flag, stream)
                     : launch<128>(tensor_map_a, tensor_map_b, g, total, sm_count, error_flag, stream);
}
