// Plain-old-data records shared by host code (bindings, plan builder) and the
// device code of the fused optimizer-state kernels.
#pragma once
#include <cstdint>
#include <vector_types.h>

namespace apexb {

enum DType : int { DT_F32 = 0, DT_BF16 = 1, DT_F16 = 2 };
enum MFmt : int { M_F32 = 0, M_BF16 = 1, M_F16 = 2, M_INT8 = 3, M_NF4 = 4 };
enum VFmt : int { V_F32 = 0, V_BF16 = 1, V_F16 = 2, V_LOGU8 = 3 };

constexpr int kChunk2048 = 2048;  // elements per work item (same value as rng.cuh kChunk)
constexpr int kThreads = 256;
constexpr int kPerThread = 8;

// SEG_FAST: every array of the segment is 16-bit (bf16 / packed codes), 16-byte aligned and
// the gradient is bf16, so full chunks take the unpredicated fast path.
// SEG_NO_V_STREAM: s.v is not one value per element (per four) of the tensor - factored statistics, Lion - so the
// look-ahead prefetch must not touch it.
enum SegFlags : uint32_t { SEG_DECAY = 1u, SEG_QUAD_V = 2u, SEG_FAST = 4u, SEG_NO_V_STREAM = 8u };
// STEP_LION / STEP_SLOW / STEP_AMSGRAD: dense formats only, general path.  Lion keeps no second moment; AdEMAMix keeps a
// slow first moment in the segment's `m_scale` slot and AMSGrad a running maximum of v in its `v_scale` slot (both slots
// are otherwise unused by dense segments; same dtypes as m and v).
enum StepFlags : uint32_t { STEP_STOCHASTIC = 1u, STEP_NESTEROV = 2u, STEP_CAUTIOUS = 4u, STEP_MAXIMIZE = 8u,
                            STEP_LION = 16u, STEP_SLOW = 32u, STEP_AMSGRAD = 64u };

struct SegDesc {
    void* p;
    const void* g;
    void* m;
    void* v;
    float* m_scale;
    float* v_scale;
    long long numel;
    long long offset;        // element offset of this segment in the flat (symmetric) buffers; ZeRO only
    uint32_t chunk_begin;    // index of this segment's first chunk within the launch
    uint32_t salt;
    uint8_t p_dtype, g_dtype, m_fmt, v_fmt;
    uint8_t flags;
    uint8_t bs_log2;         // log2 of the quantisation block (6..11); 0 for dense formats
    uint8_t v_scale_log4;    // dense fp16 second moments are stored times 4^k (k = 0..8) so that they stay in range
    uint8_t pad1;
};
static_assert(sizeof(SegDesc) == 80, "SegDesc layout is mirrored by the host code");

// Optional side record of a segment (single-GPU kernel): decoupled weight decay that applies to PARTS of a flat
// parameter only - the matrices inside an FSDP flat shard or a flattened model - decided per 2048-element chunk.
struct SegExtra {
    const uint32_t* chunk_decay;   // per chunk: 0 = no element decays, 1 = all do, k >= 2 = mixed, bit mask number k - 2
    const uint8_t* masks;          // 256 bytes per mixed chunk: bit j of byte t says whether element 8 * t + j decays
};
constexpr uint32_t kDecayByFlag = 0xFFFFFFFFu;   // no side record: the segment's SEG_DECAY flag decides

struct StepArgs {
    float beta1, omb1, beta2, omb2;
    float omb2_quarter;          // 0.25 * (1 - beta2): weight of the summed squares of four gradients
    float step_size, eps_scaled, eps;
    float eps_quad, eps_quad_scaled;
    float decay_factor, inv_scale;
    float gain_hi, gain_lo;
    uint32_t step_key;
    uint32_t flags;
    int num_segments;
    uint32_t total_chunks;
    float beta3, omb3, slow_ratio;   // AdEMAMix: slow momentum coefficient and its weight alpha * bc1 / bc3 in the numerator
    float lr;                        // Lion steps by lr * sign(...)
    uint32_t interleave;     // tuning word.  bit 0: CTAs take chunks round-robin (else one contiguous range each);
                             // bits 8-15 (peer kernel): cap on resident CTAs per SM, 0 = as many as fit;
                             // bits 16-31 (peer kernel): cap on the CTAs of the launch in total, 0 = none
};


constexpr int kMaxPeers = 8;
constexpr int kSignalWords = 2 * kMaxPeers + 2;   // entry flags, exit flags, go word, done counter

// Peer view of one rank for the fused ZeRO kernel: every rank's flat gradient buffer,
// flat parameter buffer and signal pad as mapped into this process.
// Scalars of a step that depend on the step count or on the learning rate, when either lives on the device (step
// counters of a capturable optimizer, a tensor learning rate): a one-thread kernel derives them and the update kernel
// reads them in place of the corresponding StepArgs fields, so a step never needs the values on the host.
struct DynScalars {
    float step_size, eps_scaled, eps_quad_scaled, decay_factor, slow_ratio, lr;
    uint32_t step_key;
    uint32_t pad;
};
struct DynInputs {
    const float* step_dev;    // null: step_host
    const float* lr_dev;      // null: lr_host
    // doubles: 1 - beta2^step loses five digits when beta2 = 0.999 is first rounded to fp32, and the host path
    // (which this must reproduce bit for bit) works in double precision
    double step_host, lr_host;
    double beta1, beta2, beta3;  // beta3 <= 0: no slow moment
    double alpha, eps, eps_quad, weight_decay;
    uint32_t seed;
    uint32_t pad;
};

// Factored second moment (one statistic per row and one per column of a matrix): side record of a segment for the two
// kernels that run before the update - sums of squared gradients per row and column, then the moving averages and the
// two factor vectors that the update multiplies.
struct FactAux {
    float* row_stat;         // moving average of the row means of g^2     (rows entries, optimizer state)
    float* col_stat;         // moving average of the column means of g^2  (cols entries, optimizer state)
    float* row_work;         // scratch: sums of g^2 per row, then sqrt(row_stat / mean(row_stat))
    float* col_work;         // scratch: sums of g^2 per column, then sqrt(col_stat)
    int rows, cols;
    uint32_t tile_begin;     // first tile of this segment in the statistics launch
    uint32_t tiles_c;        // tiles per row band (column strips)
};
constexpr int kFactTileRows = 32;       // a statistics tile: 32 rows x 1024 columns, four columns per thread
constexpr int kFactTileCols = 1024;

struct ZeroPeers {
    const void* grad[kMaxPeers];
    void* param[kMaxPeers];
    uint32_t* signal[kMaxPeers];
    int world;
    int rank;
    int grad_sources;   // world when gradients are reduced here; 1 when they arrive already reduced (grad[0] = local)
    int pad;
    // NVSwitch multicast addresses of the same two buffers (null: plain peer loads / stores).  A multimem.ld_reduce on
    // mc_grad sums all ranks' gradients inside the switch; a multimem.st on mc_param writes every rank's copy.
    const void* mc_grad;
    void* mc_param;
};

// One matrix owned by this rank in the distributed Muon kernels.
struct MuonSeg {
    float* momentum;         // fp32 momentum, owner only                      (gather)
    uint16_t* staged;        // bf16 staging: Newton-Schulz input (gather) or orthogonalised update (scatter)
    long long numel;         // multiple of 8
    long long offset;        // element offset in the flat symmetric buffers, multiple of 8
    uint32_t chunk_begin;
    float scale;             // update scale of this tensor, multiplied by lr   (scatter)
};
static_assert(sizeof(MuonSeg) == 40, "MuonSeg layout is mirrored by the host code");

struct CodecTables {
    float nf4[16];       // code -> value
    float nf4_mag[8];    // magnitudes 0 .. 1
    float nf4_inv_gap[8];
    float logv[256];     // code -> value (code 0 -> 0)
    float2 nf4_pair[256]; // packed byte -> (value of the high nibble = even element, value of the low nibble)
};

}  // namespace apexb
