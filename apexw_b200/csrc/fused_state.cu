// Single-GPU fused optimizer-state kernel (dense and quantised moments in one
// persistent launch over a resident segment table) and its host launcher.
//
// Compile with -fmad=false: the torch engine that serves as the oracle rounds
// every product and sum separately.
#include <cuda_runtime.h>
#include <cmath>
#include <cstdio>
#include "api.h"
#include "fused_state.cuh"

namespace apexb {

__device__ CodecTables g_codec_tables;
__device__ unsigned g_table_fault[4];          // debug mode: first table fault of this module's kernels

// KC_DENSE_EXTRA is chosen at launch for KC_DENSE plans whose step asks for Lion, AdEMAMix or AMSGrad; the two
// ..._CAUTIOUS classes for dense plans whose step is cautious (they need the kept counts of `keep_count_kernel`);
// KC_ULTRA (host class 5) is the int8-momentum + dense-variance layout, KC_FACTORED (host class 6) the row / column
// factored second moment, whose statistics kernels run before the update, KC_LION8 (host class 7) Lion on an int8
// first moment
enum KernelClass : int { KC_DENSE = 0, KC_DENSE_QUAD = 1, KC_INT8 = 2, KC_NF4 = 3, KC_NF4_QUAD = 4, KC_DENSE_EXTRA = 5,
                         KC_DENSE_CAUTIOUS = 6, KC_DENSE_QUAD_CAUTIOUS = 7, KC_ULTRA = 8, KC_FACTORED = 9, KC_LION8 = 10, KC_COUNT = 11 };

#ifndef APEXB_STATE_CTAS_PER_SM
#define APEXB_STATE_CTAS_PER_SM 3
#endif

// PARTIAL: some segment carries a side record for decay over parts of a flat parameter; the common instantiation
// (false) does not pay for the extra state in registers
template <int KC, bool PARTIAL>
__global__ void __launch_bounds__(kThreads, APEXB_STATE_CTAS_PER_SM)
fused_state_kernel(const SegDesc* __restrict__ segs, StepArgs a, const float* __restrict__ found_inf,
                   const float* __restrict__ grad_scale, const SegExtra* __restrict__ extras,
                   const unsigned long long* __restrict__ keep_counts, const DynScalars* __restrict__ dyn) {
    __shared__ CodecTables tab;
    __shared__ ReduceScratch scratch;
    if (found_inf != nullptr && *found_inf > 0.0f) return;  // AMP: overflow seen, skip the step
    if (grad_scale != nullptr) a.inv_scale = 1.0f / *grad_scale;
    if (dyn != nullptr) {       // step count or learning rate live on the device
        a.step_size = dyn->step_size; a.eps_scaled = dyn->eps_scaled; a.eps_quad_scaled = dyn->eps_quad_scaled;
        a.decay_factor = dyn->decay_factor; a.slow_ratio = dyn->slow_ratio; a.lr = dyn->lr; a.step_key = dyn->step_key;
    }
    if (KC >= KC_INT8 && KC <= KC_NF4_QUAD) {
        load_tables(tab, &g_codec_tables);
        init_scratch(scratch);
        __syncthreads();
    }
    if (KC == KC_ULTRA || KC == KC_FACTORED || KC == KC_LION8) {
        init_scratch(scratch);
        __syncthreads();
    }
    uint32_t turn = 0;
    const LocalIO io;
    // chunk walk: one contiguous range per CTA, or round-robin over the whole table
    const uint32_t per_cta = (a.total_chunks + gridDim.x - 1) / gridDim.x;
    const bool rr = (a.interleave & 1u) != 0;
    const uint32_t stride = rr ? gridDim.x : 1u;
    const uint32_t begin = rr ? blockIdx.x : blockIdx.x * per_cta;
    const uint32_t end = rr ? a.total_chunks : min(begin + per_cta, a.total_chunks);
    if (begin >= end) return;
    ChunkCursor cur;
    cur.init(segs, a.num_segments, a.total_chunks, begin);
    if (!rr && !(a.interleave & kTuneCheckTable) && begin + 1 < cur.seg_end && begin + 1 < end) prefetch_chunk(cur.s, begin + 1 - cur.s.chunk_begin, true);
    for (uint32_t chunk = begin; chunk < end; chunk += stride) {
        cur.seek(chunk);
        if (a.interleave & kTuneCheckTable) {        // debug mode: validate before anything is indexed
            uint32_t fault = table_fault(cur.s, cur.si, a.num_segments, chunk, cur.seg_end,
                                         KC >= KC_INT8 && KC <= KC_NF4_QUAD, true);
            if ((KC == KC_ULTRA || KC == KC_FACTORED || KC == KC_LION8) && fault == TF_FORMAT && cur.s.m_fmt == M_INT8) fault = TF_NONE;   // int8 m, no log-u8 v
            if (KC == KC_FACTORED && fault == TF_NONE) {
                if (cur.s.v_scale == nullptr) fault = TF_NULL_POINTER;               // the column factors
                else if (cur.s.offset <= 0 || cur.s.numel % cur.s.offset != 0) fault = TF_OFFSET;   // columns per row
                else if (cur.s.m_fmt == M_INT8 && (cur.s.m_scale == nullptr)) fault = TF_NULL_SCALES;
                else if (cur.s.m_fmt == M_INT8 && (cur.s.bs_log2 < 6 || cur.s.bs_log2 > 11)) fault = TF_BLOCK_SIZE;
            }
            if ((KC == KC_ULTRA || KC == KC_LION8) && fault == TF_NONE) {
                if (cur.s.m_scale == nullptr) fault = TF_NULL_SCALES;
                else if (cur.s.bs_log2 < 6 || cur.s.bs_log2 > 11) fault = TF_BLOCK_SIZE;
            }
            if (fault != TF_NONE) { record_table_fault(g_table_fault, fault, cur.si, chunk); continue; }
        }
        const uint32_t c = chunk - cur.s.chunk_begin;
        const uint32_t ahead = chunk + 2 * stride;
        if (ahead < cur.seg_end && ahead < end) prefetch_chunk(cur.s, ahead - cur.s.chunk_begin, true);
        ChunkDecay dec = decay_by_flag();
        if (PARTIAL) {                      // flat parameters whose decay covers some of their ranges only
            const SegExtra e = extras[cur.si];
            if (e.chunk_decay != nullptr) dec = ChunkDecay{e.chunk_decay[c], e.masks};
        }
        if (KC == KC_DENSE) dense_chunk<false>(cur.s, a, c, io, dec);
        else if (KC == KC_DENSE_QUAD) dense_chunk<true>(cur.s, a, c, io, dec);
        else if (KC == KC_INT8) quant_chunk<false, false>(cur.s, a, c, io, tab, scratch, turn, dec);
        else if (KC == KC_NF4) quant_chunk<true, false>(cur.s, a, c, io, tab, scratch, turn, dec);
        else if (KC == KC_LION8) lion8_chunk(cur.s, a, c, io, scratch, turn, dec.mask8(cur.s));
        else if (KC == KC_FACTORED) factored_chunk(cur.s, a, c, io, scratch, turn, dec.mask8(cur.s));
        else if (KC == KC_ULTRA) ultra_chunk(cur.s, a, c, io, scratch, turn, dec.mask8(cur.s));
        else if (KC == KC_DENSE_EXTRA) dense_exotic(cur.s, a, c, io, dec.mask8(cur.s));
        else if (KC == KC_DENSE_CAUTIOUS || KC == KC_DENSE_QUAD_CAUTIOUS) {
            // mean of the keep mask over the whole tensor, floored at 1e-3, as a multiplier
            const float mean = static_cast<float>(keep_counts[cur.si]) * (1.0f / static_cast<float>(cur.s.numel));
            const float inv_keep = 1.0f / fmaxf(mean, 1e-3f);
            dense_general<KC == KC_DENSE_QUAD_CAUTIOUS, LocalIO, true>(cur.s, a, c, io, dec.mask8(cur.s), inv_keep);
        }
        else quant_chunk<true, true>(cur.s, a, c, io, tab, scratch, turn, dec);
    }
}

// ---- factored second moment: statistics --------------------------------------------------------------------------
__device__ __forceinline__ float grad_elem(const void* g, int dt, long long i) {
    if (dt == DT_F32) return reinterpret_cast<const float*>(g)[i];
    const uint16_t bits = reinterpret_cast<const uint16_t*>(g)[i];
    return dt == DT_BF16 ? bf16_bits_to_float(bits) : f16_bits_to_float(bits);
}

// Sums of squared (sanitised, scaled) gradients per row and per column, added into the zeroed work vectors.  One tile
// = 32 rows x 1024 columns; a thread owns four adjacent columns and walks the rows, so its column sums are private
// and a row's sum over the tile goes through one shared-memory word.  One global atomic per row and per column of a
// tile (fp32 additions in arrival order: the sums can differ in their last bits from run to run).
__global__ void __launch_bounds__(kThreads)
fact_stats_kernel(const SegDesc* __restrict__ segs, const FactAux* __restrict__ aux, int num_segments, uint32_t total_tiles,
                  float inv_scale, uint32_t flags, const float* __restrict__ found_inf, const float* __restrict__ grad_scale) {
    __shared__ float s_row[kFactTileRows];
    if (found_inf != nullptr && *found_inf > 0.0f) return;
    if (grad_scale != nullptr) inv_scale = 1.0f / *grad_scale;
    for (uint32_t tile = blockIdx.x; tile < total_tiles; tile += gridDim.x) {
        int lo = 0, hi = num_segments - 1;
        while (lo < hi) {                           // last segment whose first tile is <= tile
            const int mid = (lo + hi + 1) >> 1;
            if (aux[mid].tile_begin <= tile) lo = mid; else hi = mid - 1;
        }
        const FactAux ax = aux[lo];
        const SegDesc& sg = segs[lo];
        const void* g = sg.g;
        const int gdt = sg.g_dtype;
        const uint32_t local = tile - ax.tile_begin;
        const int row0 = static_cast<int>(local / ax.tiles_c) * kFactTileRows;
        const int col0 = static_cast<int>(local % ax.tiles_c) * kFactTileCols + static_cast<int>(threadIdx.x) * 4;
        if (threadIdx.x < kFactTileRows) s_row[threadIdx.x] = 0.0f;
        __syncthreads();
        float csum[4] = {0.f, 0.f, 0.f, 0.f};
        const int nrows = min(kFactTileRows, ax.rows - row0);
        for (int r = 0; r < nrows; ++r) {
            const long long base = static_cast<long long>(row0 + r) * ax.cols;
            float rsum = 0.0f;
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                if (col0 + j < ax.cols) {
                    float x = sanitize_grad(grad_elem(g, gdt, base + col0 + j));
                    if (flags & STEP_MAXIMIZE) x = -x;
                    x = x * inv_scale;
                    const float sq = x * x;
                    csum[j] += sq;
                    rsum += sq;
                }
            }
            rsum += __shfl_xor_sync(0xFFFFFFFFu, rsum, 16);
            rsum += __shfl_xor_sync(0xFFFFFFFFu, rsum, 8);
            rsum += __shfl_xor_sync(0xFFFFFFFFu, rsum, 4);
            rsum += __shfl_xor_sync(0xFFFFFFFFu, rsum, 2);
            rsum += __shfl_xor_sync(0xFFFFFFFFu, rsum, 1);
            if ((threadIdx.x & 31) == 0 && rsum != 0.0f) atomicAdd(&s_row[r], rsum);
        }
#pragma unroll
        for (int j = 0; j < 4; ++j)
            if (col0 + j < ax.cols && csum[j] != 0.0f) atomicAdd(&ax.col_work[col0 + j], csum[j]);
        __syncthreads();
        if (static_cast<int>(threadIdx.x) < nrows && s_row[threadIdx.x] != 0.0f)
            atomicAdd(&ax.row_work[row0 + threadIdx.x], s_row[threadIdx.x]);
        __syncthreads();
    }
}

// One CTA per segment: moving averages of the row / column means (non-finite values become zero), the mean of the row
// statistics, and the two factor vectors that the update multiplies, written over the sums.
__global__ void __launch_bounds__(kThreads)
fact_finish_kernel(const FactAux* __restrict__ aux, float beta2, float omb2, const float* __restrict__ found_inf) {
    __shared__ float s_part[kThreads / 32];
    __shared__ float s_mean;
    if (found_inf != nullptr && *found_inf > 0.0f) return;
    const FactAux ax = aux[blockIdx.x];
    float part = 0.0f;
    for (int i = threadIdx.x; i < ax.rows; i += kThreads) {
        float r = ax.row_stat[i] * beta2 + (ax.row_work[i] / static_cast<float>(ax.cols)) * omb2;
        if (!(fabsf(r) < INFINITY)) r = 0.0f;
        ax.row_stat[i] = r;
        part += r;
    }
    for (int j = threadIdx.x; j < ax.cols; j += kThreads) {
        float c = ax.col_stat[j] * beta2 + (ax.col_work[j] / static_cast<float>(ax.rows)) * omb2;
        if (!(fabsf(c) < INFINITY)) c = 0.0f;
        ax.col_stat[j] = c;
        ax.col_work[j] = sqrtf(c);
    }
    for (int off = 16; off > 0; off >>= 1) part += __shfl_xor_sync(0xFFFFFFFFu, part, off);
    if ((threadIdx.x & 31) == 0) s_part[threadIdx.x >> 5] = part;
    __syncthreads();
    if (threadIdx.x == 0) {
        float total = 0.0f;
        for (int w = 0; w < kThreads / 32; ++w) total += s_part[w];
        s_mean = fmaxf(total / static_cast<float>(ax.rows), 1e-30f);
    }
    __syncthreads();
    const float mean = s_mean;
    for (int i = threadIdx.x; i < ax.rows; i += kThreads) ax.row_work[i] = sqrtf(ax.row_stat[i] / mean);
}

// Derives the step-dependent scalars on the device (see DynScalars).  Bias corrections in double precision.
__global__ void dyn_scalars_kernel(DynInputs in, DynScalars* __restrict__ out) {
    if (threadIdx.x != 0 || blockIdx.x != 0) return;
    const double step = in.step_dev != nullptr ? static_cast<double>(*in.step_dev) : in.step_host;
    // a learning rate tensor holds an fp32 value; the host value is a double, as on the host path
    const double lr = in.lr_dev != nullptr ? static_cast<double>(*in.lr_dev) : in.lr_host;
    const double bc1 = 1.0 - pow(in.beta1, step);
    const double bc2_sqrt = sqrt(1.0 - pow(in.beta2, step));
    DynScalars d;
    d.step_size = static_cast<float>(lr * bc2_sqrt / bc1);
    d.eps_scaled = static_cast<float>(in.eps * bc2_sqrt);
    d.eps_quad_scaled = static_cast<float>(in.eps_quad * bc2_sqrt);
    d.decay_factor = static_cast<float>(fmax(1.0 - lr * in.weight_decay, 0.0));
    d.slow_ratio = in.beta3 > 0.0 ? static_cast<float>(in.alpha * (bc1 / (1.0 - pow(in.beta3, step)))) : 0.0f;
    d.lr = static_cast<float>(lr);
    d.step_key = mix32(in.seed ^ (static_cast<uint32_t>(static_cast<long long>(step)) * kGolden));
    d.pad = 0;
    *out = d;
}

// First pass of a cautious step on dense state: per segment, how many elements keep their update.  Every CTA walks a
// contiguous range of chunks and adds one total per segment it crosses.
__global__ void __launch_bounds__(kThreads)
keep_count_kernel(const SegDesc* __restrict__ segs, StepArgs a, const float* __restrict__ found_inf,
                  const float* __restrict__ grad_scale, unsigned long long* __restrict__ keep_counts) {
    if (found_inf != nullptr && *found_inf > 0.0f) return;
    if (grad_scale != nullptr) a.inv_scale = 1.0f / *grad_scale;
    const LocalIO io;
    const uint32_t per_cta = (a.total_chunks + gridDim.x - 1) / gridDim.x;
    const uint32_t begin = blockIdx.x * per_cta;
    const uint32_t end = min(begin + per_cta, a.total_chunks);
    if (begin >= end) return;
    ChunkCursor cur;
    cur.init(segs, a.num_segments, a.total_chunks, begin);
    uint32_t kept = 0;
    int seg = -1;
    for (uint32_t chunk = begin; chunk < end; ++chunk) {
        cur.seek(chunk);
        if ((a.interleave & kTuneCheckTable) &&
            table_fault(cur.s, cur.si, a.num_segments, chunk, cur.seg_end, false, true) != TF_NONE)
            continue;       // the update pass records it
        if (static_cast<int>(cur.si) != seg) {
            if (seg >= 0) {
                const uint32_t total = __reduce_add_sync(0xFFFFFFFFu, kept);      // one atomic per warp and segment
                if ((threadIdx.x & 31) == 0 && total) atomicAdd(&keep_counts[seg], static_cast<unsigned long long>(total));
                kept = 0;
            }
            seg = static_cast<int>(cur.si);
        }
        kept += dense_keep_count(cur.s, a, chunk - cur.s.chunk_begin, io);
    }
    const uint32_t total = __reduce_add_sync(0xFFFFFFFFu, kept);
    if ((threadIdx.x & 31) == 0 && total) atomicAdd(&keep_counts[seg], static_cast<unsigned long long>(total));
}

// Exercises `table_fault` on descriptors that are wrong in one way each.  Nothing is dereferenced: the descriptors
// live in registers and their pointers are only compared and masked.  Bit i of *caught: case i gave the expected code.
__global__ void table_check_selftest_kernel(unsigned* caught, void* some_aligned_address) {
    if (threadIdx.x != 0 || blockIdx.x != 0) return;
    SegDesc ok{};
    ok.p = ok.m = ok.v = some_aligned_address;
    ok.g = some_aligned_address;
    ok.m_scale = ok.v_scale = static_cast<float*>(some_aligned_address);
    ok.numel = 5000; ok.offset = 0; ok.chunk_begin = 10; ok.p_dtype = DT_BF16; ok.g_dtype = DT_BF16;
    ok.m_fmt = M_NF4; ok.v_fmt = V_LOGU8; ok.bs_log2 = 8;
    unsigned bits = 0;
    int i = 0;
    auto expect = [&](const SegDesc& d, int si, int nseg, uint32_t chunk, uint32_t seg_end, bool quant, uint32_t want) {
        if (table_fault(d, si, nseg, chunk, seg_end, quant, true) == want) bits |= 1u << i;
        ++i;
    };
    expect(ok, 0, 1, 10, 13, true, TF_NONE);
    expect(ok, 0, 1, 12, 13, true, TF_NONE);                       // the partial last chunk (5000 = 2 * 2048 + 904)
    expect(ok, 1, 1, 10, 13, true, TF_SEGMENT_INDEX);
    expect(ok, -1, 1, 10, 13, true, TF_SEGMENT_INDEX);
    expect(ok, 0, 1, 9, 13, true, TF_CHUNK_BEFORE_SEGMENT);
    expect(ok, 0, 1, 13, 13, true, TF_CHUNK_PAST_SEGMENT);
    expect(ok, 0, 1, 13, 20, true, TF_CHUNK_PAST_NUMEL);           // inside the chunk range, past the elements
    SegDesc d = ok; d.g = nullptr;
    expect(d, 0, 1, 10, 13, true, TF_NULL_POINTER);
    d = ok; d.p = reinterpret_cast<void*>(reinterpret_cast<uintptr_t>(some_aligned_address) + 1);
    expect(d, 0, 1, 10, 13, true, TF_ALIGNMENT);
    d = ok; d.bs_log2 = 5;
    expect(d, 0, 1, 10, 13, true, TF_BLOCK_SIZE);
    d = ok; d.v_scale = nullptr;
    expect(d, 0, 1, 10, 13, true, TF_NULL_SCALES);
    d = ok; d.m_fmt = M_BF16;
    expect(d, 0, 1, 10, 13, true, TF_FORMAT);
    d = ok; d.m_fmt = M_BF16; d.v_fmt = V_BF16;
    expect(d, 0, 1, 10, 13, false, TF_NONE);                       // the same record is a valid dense one
    d = ok; d.offset = -8;
    expect(d, 0, 1, 10, 13, true, TF_OFFSET);
    d = ok; d.numel = 0;
    expect(d, 0, 1, 10, 13, true, TF_CHUNK_PAST_NUMEL);
    *caught = bits;
}

static bool g_tables_ready[64] = {};

void fill_codec_tables(CodecTables& t) {
    static const float mags[8] = {0.0f, 0.0911f, 0.1848f, 0.2844f, 0.3949f, 0.5251f, 0.6962f, 1.0f};
    for (int i = 0; i < 8; ++i) t.nf4_mag[i] = mags[i];
    for (int i = 0; i < 7; ++i) t.nf4_inv_gap[i] = 1.0f / (mags[i + 1] - mags[i]);
    t.nf4_inv_gap[7] = 1.0f;
    for (int i = 0; i < 7; ++i) t.nf4[i] = -mags[7 - i];
    for (int i = 0; i < 8; ++i) t.nf4[7 + i] = mags[i];
    t.nf4[15] = 1.0f;
    for (int b = 0; b < 256; ++b) t.nf4_pair[b] = make_float2(t.nf4[b >> 4], t.nf4[b & 15]);
    t.logv[0] = 0.0f;
    for (int q = 1; q < 256; ++q) t.logv[q] = static_cast<float>(std::pow(2.0, (q - 1) * 24.0 / 254.0 - 24.0));
}

}  // namespace apexb

using namespace apexb;

extern "C" int apexb_fused_state_ctas_per_sm() { return APEXB_STATE_CTAS_PER_SM; }

// Debug mode: copy out (and clear, when asked) this module's table-fault word: code, segment, chunk, skipped chunks.
extern "C" int apexb_fused_state_table_fault(unsigned out[4], int clear) {
    cudaError_t e = cudaMemcpyFromSymbol(out, g_table_fault, 4 * sizeof(unsigned));
    if (e != cudaSuccess) return static_cast<int>(e);
    if (clear) {
        const unsigned zero[4] = {0, 0, 0, 0};
        e = cudaMemcpyToSymbol(g_table_fault, zero, sizeof(zero));
    }
    return static_cast<int>(e);
}

// Factored second moment, before the update launch: row / column sums of g^2 into the (zeroed) work vectors, then the
// moving averages and the factor vectors.  d_aux: one FactAux per segment of the same plan.
extern "C" int apexb_factored_stats_launch(const void* d_segments, const void* d_aux, int num_segments, unsigned total_tiles,
                                            const StepArgs* args, const float* found_inf, const float* grad_scale, int max_ctas,
                                            cudaStream_t stream) {
    if (num_segments == 0 || total_tiles == 0) return 0;
    const unsigned grid = total_tiles < static_cast<unsigned>(max_ctas) ? total_tiles : static_cast<unsigned>(max_ctas);
    fact_stats_kernel<<<grid, kThreads, 0, stream>>>(static_cast<const SegDesc*>(d_segments), static_cast<const FactAux*>(d_aux),
                                                     num_segments, total_tiles, args->inv_scale, args->flags, found_inf, grad_scale);
    fact_finish_kernel<<<num_segments, kThreads, 0, stream>>>(static_cast<const FactAux*>(d_aux), args->beta2, args->omb2, found_inf);
    return static_cast<int>(cudaGetLastError());
}

extern "C" int apexb_dyn_scalars_launch(const DynInputs* in, DynScalars* d_out, cudaStream_t stream) {
    dyn_scalars_kernel<<<1, 32, 0, stream>>>(*in, d_out);
    return static_cast<int>(cudaGetLastError());
}

// Runs the checker on 15 hand-made descriptors (none is dereferenced); *d_caught gets one bit per case that behaved.
extern "C" int apexb_table_check_selftest(unsigned* d_caught, void* some_aligned_address, cudaStream_t stream) {
    table_check_selftest_kernel<<<1, 32, 0, stream>>>(d_caught, some_aligned_address);
    return static_cast<int>(cudaGetLastError());
}

extern "C" int apexb_fused_state_init(int device) {
    if (device < 0 || device >= 64) return cudaErrorInvalidDevice;
    if (g_tables_ready[device]) return 0;
    CodecTables t;
    fill_codec_tables(t);
    cudaError_t e = cudaMemcpyToSymbol(g_codec_tables, &t, sizeof(t));
    if (e != cudaSuccess) return static_cast<int>(e);
    g_tables_ready[device] = true;
    return 0;
}

extern "C" int apexb_fused_state_launch(int kernel_class, const void* d_segments, const StepArgs* args,
                                         const float* found_inf, const float* grad_scale, int max_ctas,
                                         const void* d_extras, unsigned long long* d_keep_counts,
                                         const DynScalars* d_dyn, cudaStream_t stream) {
    if (args->total_chunks == 0 || args->num_segments == 0) return 0;
    const unsigned grid = args->total_chunks < static_cast<unsigned>(max_ctas) ? args->total_chunks : max_ctas;
    const SegDesc* segs = static_cast<const SegDesc*>(d_segments);
    const SegExtra* ex = static_cast<const SegExtra*>(d_extras);
    const bool extra = (args->flags & (STEP_LION | STEP_SLOW | STEP_AMSGRAD)) != 0;
    bool lion8 = false;
    if (kernel_class == 7) {       // host class 7: Lion on an int8 first moment
        if (!(args->flags & STEP_LION) || (args->flags & (STEP_SLOW | STEP_AMSGRAD | STEP_CAUTIOUS | STEP_NESTEROV)))
            return static_cast<int>(cudaErrorInvalidValue);
        kernel_class = KC_LION8;
        lion8 = true;
    } else if (kernel_class == 6) {       // host class 6: factored second moment (the statistics launch has run); plain, Nesterov, maximize
        if (extra || (args->flags & STEP_CAUTIOUS)) return static_cast<int>(cudaErrorInvalidValue);
        kernel_class = KC_FACTORED;
    } else if (kernel_class == 5) {       // host class 5: int8 first moment + dense second moment; plain, Nesterov, maximize only
        if (extra || (args->flags & STEP_CAUTIOUS)) return static_cast<int>(cudaErrorInvalidValue);
        kernel_class = KC_ULTRA;
    } else if (kernel_class > KC_NF4_QUAD) {
        return static_cast<int>(cudaErrorInvalidValue);
    }
    if (extra && !lion8 && kernel_class != KC_DENSE) return static_cast<int>(cudaErrorInvalidValue);
    if (extra && !lion8) kernel_class = KC_DENSE_EXTRA;
    if ((args->flags & STEP_CAUTIOUS) && (kernel_class == KC_DENSE || kernel_class == KC_DENSE_QUAD)) {
        // dense cautious: count what the whole tensor keeps (the counts were zeroed by the caller), then update
        if (d_keep_counts == nullptr) return static_cast<int>(cudaErrorInvalidValue);
        keep_count_kernel<<<grid, kThreads, 0, stream>>>(segs, *args, found_inf, grad_scale, d_keep_counts);
        kernel_class = kernel_class == KC_DENSE ? KC_DENSE_CAUTIOUS : KC_DENSE_QUAD_CAUTIOUS;
    }
#define APEXB_LAUNCH(KC)                                                                                                   \
    case KC:                                                                                                               \
        if (ex) fused_state_kernel<KC, true><<<grid, kThreads, 0, stream>>>(segs, *args, found_inf, grad_scale, ex, d_keep_counts, d_dyn); \
        else fused_state_kernel<KC, false><<<grid, kThreads, 0, stream>>>(segs, *args, found_inf, grad_scale, ex, d_keep_counts, d_dyn);   \
        break;
    switch (kernel_class) {
        APEXB_LAUNCH(KC_DENSE)
        APEXB_LAUNCH(KC_DENSE_QUAD)
        APEXB_LAUNCH(KC_INT8)
        APEXB_LAUNCH(KC_NF4)
        APEXB_LAUNCH(KC_NF4_QUAD)
        APEXB_LAUNCH(KC_DENSE_EXTRA)
        APEXB_LAUNCH(KC_DENSE_CAUTIOUS)
        APEXB_LAUNCH(KC_DENSE_QUAD_CAUTIOUS)
        APEXB_LAUNCH(KC_ULTRA)
        APEXB_LAUNCH(KC_FACTORED)
        APEXB_LAUNCH(KC_LION8)
        default: return static_cast<int>(cudaErrorInvalidValue);
    }
#undef APEXB_LAUNCH
    return static_cast<int>(cudaGetLastError());
}
