// StatePlan: resident launch plan of the fused optimizer-state kernels (shared by the
// single-GPU bindings and the ZeRO bindings).
#pragma once
#include <torch/extension.h>
#include <ATen/cuda/CUDAContext.h>
#include <c10/cuda/CUDAGuard.h>
#include <algorithm>
#include <cstdlib>
#include <cstring>
#include <vector>
#include "api.h"

namespace apexb_host {

using apexb::SegDesc;
using apexb::StepArgs;

inline void check_cuda(int err, const char* what) {
    TORCH_CHECK(err == 0, what, " failed: ", cudaGetErrorString(static_cast<cudaError_t>(err)));
}

// Chunk order of the persistent kernels: "blocked" (one contiguous range per CTA) or "interleaved" (round-robin,
// all CTAs inside one window of the arrays).  APEXW_B200_CHUNK_ORDER overrides the default of the call site.
inline uint32_t chunk_order(bool default_interleaved) {
    static int cached = -1;
    if (cached < 0) {
        const char* e = std::getenv("APEXW_B200_CHUNK_ORDER");
        cached = (e == nullptr) ? 2 : (std::strcmp(e, "interleaved") == 0 ? 1 : 0);
    }
    return cached == 2 ? (default_interleaved ? 1u : 0u) : static_cast<uint32_t>(cached);
}

// Debug mode: APEXW_B200_DEBUG_BOUNDS=1 makes the persistent kernels validate every chunk's table record before they
// index with it (bit 1 of StepArgs::interleave).  Read at every step, so a test can switch it.
inline uint32_t table_check_bit() {
    const char* e = std::getenv("APEXW_B200_DEBUG_BOUNDS");
    return (e != nullptr && e[0] != '\0' && e[0] != '0') ? 2u : 0u;
}

// {code, segment, chunk, skipped chunks} of the single-GPU kernels, then of the peer kernels; synchronises the device.
inline std::vector<int64_t> table_fault_report(bool clear) {
    unsigned a[4] = {0, 0, 0, 0}, b[4] = {0, 0, 0, 0};
    check_cuda(cudaDeviceSynchronize(), "table_fault_report");
    check_cuda(apexb_fused_state_table_fault(a, clear ? 1 : 0), "table_fault_report (state)");
    check_cuda(apexb_zero_table_fault(b, clear ? 1 : 0), "table_fault_report (zero)");
    return {a[0], a[1], a[2], a[3], b[0], b[1], b[2], b[3]};
}

// Bit mask of the checker's self-test cases that behaved (all 15: 0x7FFF).
inline int64_t table_check_selftest(at::Tensor scratch) {
    TORCH_CHECK(scratch.is_cuda() && scratch.scalar_type() == at::kInt && scratch.numel() >= 8 && scratch.is_contiguous(),
                "table_check_selftest: an int32 CUDA tensor of at least 8 elements");
    c10::cuda::CUDAGuard guard(scratch.device());
    cudaStream_t stream = at::cuda::getCurrentCUDAStream(scratch.device().index()).stream();
    unsigned* word = reinterpret_cast<unsigned*>(scratch.data_ptr<int>());
    check_cuda(apexb_table_check_selftest(word, word + 4, stream), "table_check_selftest");      // word + 4: 16-byte aligned
    return static_cast<int64_t>(scratch.select(0, 0).item<int>());
}

// Peer-kernel tuning: APEXW_B200_ZERO_CTAS=n// Peer-kernel tuning: APEXW_B200_ZERO_CTAS=n caps the resident CTAs per SM (bits 8+ of StepArgs::interleave).
inline uint32_t zero_tuning() {
    const char* c = std::getenv("APEXW_B200_ZERO_CTAS");
    const int ctas = c == nullptr ? 0 : std::atoi(c);
    return static_cast<uint32_t>((ctas > 0 && ctas < 64 ? ctas : 0) << 8);
}

// Single-GPU state kernel: APEXW_B200_STATE_CTAS=n sets the resident CTAs per SM that the grid is sized for
// (default: what the kernel was compiled for).
inline int state_ctas_per_sm(int compiled_default) {
    static int cached = -1;
    if (cached < 0) {
        const char* c = std::getenv("APEXW_B200_STATE_CTAS");
        const int v = c == nullptr ? 0 : std::atoi(c);
        cached = (v > 0 && v <= 8) ? v : 0;
    }
    return cached > 0 ? cached : compiled_default;
}

inline int float_code(const at::Tensor& t, const char* what) {
    if (t.scalar_type() == at::kFloat) return apexb::DT_F32;
    if (t.scalar_type() == at::kBFloat16) return apexb::DT_BF16;
    if (t.scalar_type() == at::kHalf) return apexb::DT_F16;
    TORCH_CHECK(false, what, ": unsupported dtype ", t.scalar_type(), " (fp32, bf16 and fp16 only)");
    return -1;
}

inline StepArgs make_step_args(double beta1, double beta2, double step_size, double eps_scaled, double eps, double eps_quad,
                               double eps_quad_scaled, double decay_factor, double inv_scale, double gain_hi, double gain_lo,
                               int64_t step_key, int64_t flags, size_t nseg, uint32_t total_chunks,
                               double beta3 = 0.0, double slow_ratio = 0.0, double lr = 0.0) {
    StepArgs a;
    a.beta1 = static_cast<float>(beta1);
    a.omb1 = static_cast<float>(1.0 - beta1);
    a.beta2 = static_cast<float>(beta2);
    a.omb2 = static_cast<float>(1.0 - beta2);
    a.omb2_quarter = static_cast<float>(0.25 * (1.0 - beta2));
    a.step_size = static_cast<float>(step_size);
    a.eps_scaled = static_cast<float>(eps_scaled);
    a.eps = static_cast<float>(eps);
    a.eps_quad = static_cast<float>(eps_quad);
    a.eps_quad_scaled = static_cast<float>(eps_quad_scaled);
    a.decay_factor = static_cast<float>(decay_factor);
    a.inv_scale = static_cast<float>(inv_scale);
    a.gain_hi = static_cast<float>(gain_hi);
    a.gain_lo = static_cast<float>(gain_lo);
    a.step_key = static_cast<uint32_t>(step_key);
    a.flags = static_cast<uint32_t>(flags);
    a.num_segments = static_cast<int>(nseg);
    a.total_chunks = total_chunks;
    a.beta3 = static_cast<float>(beta3);
    a.omb3 = static_cast<float>(1.0 - beta3);
    a.slow_ratio = static_cast<float>(slow_ratio);
    a.lr = static_cast<float>(lr);
    a.interleave = 0;
    return a;
}

class StatePlan {
  public:
    StatePlan(int kernel_class, std::vector<at::Tensor> params, std::vector<at::Tensor> m, std::vector<at::Tensor> v,
              std::vector<at::Tensor> m_scale, std::vector<at::Tensor> v_scale, std::vector<int64_t> flags,
              std::vector<int64_t> salts, std::vector<int64_t> block_sizes, std::vector<int64_t> offsets,
              int64_t device_index, std::vector<std::vector<int64_t>> decay_ranges = {})
        : kernel_class_(kernel_class), params_(std::move(params)), m_(std::move(m)), v_(std::move(v)),
          m_scale_(std::move(m_scale)), v_scale_(std::move(v_scale)) {
        const size_t n = params_.size();
        TORCH_CHECK(n > 0 || device_index >= 0, "StatePlan needs at least one tensor or an explicit device");
        TORCH_CHECK(m_.size() == n && v_.size() == n && flags.size() == n && salts.size() == n && block_sizes.size() == n,
                    "StatePlan: list lengths differ");
        TORCH_CHECK(offsets.empty() || offsets.size() == n, "StatePlan: offsets length differs");
        TORCH_CHECK(kernel_class_ >= 0 && kernel_class_ <= 7, "StatePlan: unknown kernel class");
        const bool factored = kernel_class_ == 6;    // v = row statistics, v_scale = column statistics; m dense, or int8 with m_scale
        TORCH_CHECK(!factored || (v_scale_.size() == n && (m_scale_.empty() || m_scale_.size() == n)),
                    "StatePlan: the factored layout takes row statistics (v), column statistics (v_scale) and optional int8 scales");
        const bool quant = kernel_class_ >= 2 && kernel_class_ <= 4;
        const bool lion8 = kernel_class_ == 7;       // Lion: int8 first moment with block scales, no second moment (v repeats m)
        const bool ultra = kernel_class_ == 5 || lion8;   // int8 first moment with block scales, dense second moment
        TORCH_CHECK(!quant || (m_scale_.size() == n && v_scale_.size() == n), "StatePlan: scale lists missing");
        TORCH_CHECK(!ultra || (m_scale_.size() == n && v_scale_.empty()), "StatePlan: the int8 + dense layout has first-moment scales only");
        device_ = n > 0 ? params_[0].device() : at::Device(at::kCUDA, static_cast<c10::DeviceIndex>(device_index));
        TORCH_CHECK(device_.is_cuda(), "StatePlan: tensors must be on a CUDA device");
        segs_.resize(n);
        uint64_t chunks = 0;
        for (size_t i = 0; i < n; ++i) {
            const at::Tensor& p = params_[i];
            TORCH_CHECK(p.device() == device_ && m_[i].device() == device_ && v_[i].device() == device_,
                        "StatePlan: all tensors of a plan live on one device");
            TORCH_CHECK(p.is_contiguous() && m_[i].is_contiguous() && v_[i].is_contiguous(),
                        "StatePlan: tensors must be contiguous");
            SegDesc& s = segs_[i];
            std::memset(&s, 0, sizeof(s));
            s.p = p.data_ptr();
            s.m = m_[i].data_ptr();
            s.v = v_[i].data_ptr();
            s.numel = p.numel();
            s.offset = offsets.empty() ? 0 : offsets[i];
            s.p_dtype = static_cast<uint8_t>(float_code(p, "param"));
            s.flags = static_cast<uint8_t>(flags[i]);
            s.salt = static_cast<uint32_t>(salts[i]);
            const bool quad = (s.flags & apexb::SEG_QUAD_V) != 0;
            if (quant) {
                const int64_t bs = block_sizes[i];
                TORCH_CHECK(bs >= 64 && bs <= 2048 && (bs & (bs - 1)) == 0, "StatePlan: block size must be a power of two in [64, 2048]");
                int lg = 0;
                while ((int64_t(1) << lg) < bs) ++lg;
                s.bs_log2 = static_cast<uint8_t>(lg);
                const int64_t nblk = (s.numel + bs - 1) / bs;
                TORCH_CHECK(m_scale_[i].scalar_type() == at::kFloat && v_scale_[i].scalar_type() == at::kFloat &&
                                m_scale_[i].numel() == nblk && v_scale_[i].numel() == nblk &&
                                m_scale_[i].is_contiguous() && v_scale_[i].is_contiguous(),
                            "StatePlan: scale tensors must be contiguous fp32 with one entry per block");
                s.m_scale = m_scale_[i].data_ptr<float>();
                s.v_scale = v_scale_[i].data_ptr<float>();
                const bool nf4 = kernel_class_ >= 3;
                s.m_fmt = nf4 ? apexb::M_NF4 : apexb::M_INT8;
                s.v_fmt = apexb::V_LOGU8;
                TORCH_CHECK(m_[i].element_size() == 1 && v_[i].element_size() == 1, "StatePlan: quantised moments are byte tensors");
                TORCH_CHECK(m_[i].numel() == (nf4 ? (s.numel + 1) / 2 : s.numel), "StatePlan: first-moment size mismatch");
                TORCH_CHECK(!nf4 || s.numel % 4 == 0, "StatePlan: NF4 segments need numel % 4 == 0");
                TORCH_CHECK(v_[i].numel() == (quad ? s.numel / 4 : s.numel), "StatePlan: second-moment size mismatch");
            } else if (factored) {
                TORCH_CHECK(v_[i].scalar_type() == at::kFloat && v_scale_[i].scalar_type() == at::kFloat && v_scale_[i].is_contiguous() &&
                                v_scale_[i].device() == device_, "StatePlan: row / column statistics are contiguous fp32 tensors");
                const int64_t rows = v_[i].numel(), cols = v_scale_[i].numel();
                TORCH_CHECK(rows > 0 && cols > 0 && rows * cols == s.numel && rows < (int64_t(1) << 31) && cols < (int64_t(1) << 31),
                            "StatePlan: rows x columns of the statistics must give the parameter's size");
                TORCH_CHECK(offsets.empty(), "StatePlan: the factored layout is single-GPU only");
                TORCH_CHECK(!quad, "StatePlan: segment/class mismatch");
                if (!m_scale_.empty()) {
                    const int64_t bs = block_sizes[i];
                    TORCH_CHECK(bs >= 64 && bs <= 2048 && (bs & (bs - 1)) == 0, "StatePlan: block size must be a power of two in [64, 2048]");
                    int lg = 0;
                    while ((int64_t(1) << lg) < bs) ++lg;
                    s.bs_log2 = static_cast<uint8_t>(lg);
                    TORCH_CHECK(m_scale_[i].scalar_type() == at::kFloat && m_scale_[i].numel() == (s.numel + bs - 1) / bs &&
                                    m_scale_[i].is_contiguous() && m_scale_[i].device() == device_,
                                "StatePlan: scale tensors must be contiguous fp32 with one entry per block");
                    TORCH_CHECK(m_[i].element_size() == 1 && m_[i].numel() == s.numel, "StatePlan: the int8 first moment has one byte per element");
                    s.m_scale = m_scale_[i].data_ptr<float>();
                    s.m_fmt = apexb::M_INT8;
                } else {
                    s.m_fmt = static_cast<uint8_t>(float_code(m_[i], "exp_avg"));
                    TORCH_CHECK(m_[i].numel() == s.numel, "StatePlan: first-moment size mismatch");
                }
                s.v_fmt = apexb::V_F32;
                s.flags |= apexb::SEG_NO_V_STREAM;
                s.offset = cols;             // the update kernel finds row and column of an element from this
                fact_rows_.push_back(rows);
                fact_cols_.push_back(cols);
            } else if (ultra) {
                const int64_t bs = block_sizes[i];
                TORCH_CHECK(bs >= 64 && bs <= 2048 && (bs & (bs - 1)) == 0, "StatePlan: block size must be a power of two in [64, 2048]");
                int lg = 0;
                while ((int64_t(1) << lg) < bs) ++lg;
                s.bs_log2 = static_cast<uint8_t>(lg);
                const int64_t nblk = (s.numel + bs - 1) / bs;
                TORCH_CHECK(m_scale_[i].scalar_type() == at::kFloat && m_scale_[i].numel() == nblk && m_scale_[i].is_contiguous() &&
                                m_scale_[i].device() == device_,
                            "StatePlan: scale tensors must be contiguous fp32 with one entry per block");
                s.m_scale = m_scale_[i].data_ptr<float>();
                s.m_fmt = apexb::M_INT8;
                s.v_fmt = lion8 ? static_cast<uint8_t>(apexb::V_F32) : static_cast<uint8_t>(float_code(v_[i], "exp_avg_sq"));
                if (lion8) s.flags |= apexb::SEG_NO_V_STREAM;
                TORCH_CHECK(m_[i].element_size() == 1 && m_[i].numel() == s.numel, "StatePlan: the int8 first moment has one byte per element");
                TORCH_CHECK(v_[i].numel() == s.numel && !quad, "StatePlan: second-moment size mismatch");
            } else {
                // dense formats: the two scale slots may carry auxiliary moments instead - the slow first moment of
                // AdEMAMix (m's dtype and size) and AMSGrad's running maximum of v (v's dtype and size)
                if (!m_scale_.empty()) {
                    TORCH_CHECK(m_scale_.size() == n && m_scale_[i].scalar_type() == m_[i].scalar_type() &&
                                    m_scale_[i].numel() == m_[i].numel() && m_scale_[i].is_contiguous() && m_scale_[i].device() == device_,
                                "StatePlan: the slow first moment must match exp_avg");
                    s.m_scale = reinterpret_cast<float*>(m_scale_[i].data_ptr());
                }
                if (!v_scale_.empty()) {
                    TORCH_CHECK(v_scale_.size() == n && v_scale_[i].scalar_type() == v_[i].scalar_type() &&
                                    v_scale_[i].numel() == v_[i].numel() && v_scale_[i].is_contiguous() && v_scale_[i].device() == device_ && !quad,
                                "StatePlan: the running maximum must match exp_avg_sq (and needs a per-element variance)");
                    s.v_scale = reinterpret_cast<float*>(v_scale_[i].data_ptr());
                }
                s.m_fmt = static_cast<uint8_t>(float_code(m_[i], "exp_avg"));
                s.v_fmt = static_cast<uint8_t>(float_code(v_[i], "exp_avg_sq"));
                TORCH_CHECK(m_[i].numel() == s.numel, "StatePlan: first-moment size mismatch");
                TORCH_CHECK(v_[i].numel() == (quad ? s.numel / 4 : s.numel), "StatePlan: second-moment size mismatch");
                TORCH_CHECK(!quad || s.numel % 4 == 0, "StatePlan: shared-variance segments need numel % 4 == 0");
            }
            TORCH_CHECK(quad == (kernel_class_ == 1 || kernel_class_ == 4), "StatePlan: segment/class mismatch");
            TORCH_CHECK(chunks < (1ull << 32), "StatePlan: too many chunks for one launch");
            s.chunk_begin = static_cast<uint32_t>(chunks);
            chunks += static_cast<uint64_t>((s.numel + apexb::kChunk2048 - 1) / apexb::kChunk2048);
        }
        TORCH_CHECK(chunks < (1ull << 32), "StatePlan: too many chunks for one launch");
        total_chunks_ = static_cast<uint32_t>(chunks);
        c10::cuda::CUDAGuard guard(device_);
        check_cuda(apexb_fused_state_init(device_.index()), "codec table upload");
        d_segs_ = at::empty({static_cast<int64_t>((n > 0 ? n : 1) * sizeof(SegDesc))}, at::TensorOptions().dtype(at::kByte).device(device_));
        clock_khz_ = at::cuda::getDeviceProperties(device_.index())->clockRate;
        sm_count_ = at::cuda::getDeviceProperties(device_.index())->multiProcessorCount;
        dirty_ = true;
        build_partial_decay(decay_ranges);
        if (factored) build_factored();
    }

    // Factored layout: scratch for the row / column sums (later the factor vectors) and the side table of the statistics
    // kernels; the segment records point s.v / s.v_scale at that scratch.
    void build_factored() {
        const size_t n = segs_.size();
        int64_t floats = 0;
        for (size_t i = 0; i < n; ++i) floats += fact_rows_[i] + fact_cols_[i];
        d_fact_work_ = at::zeros({std::max<int64_t>(floats, 1)}, at::TensorOptions().dtype(at::kFloat).device(device_));
        std::vector<apexb::FactAux> aux(n);
        float* w = d_fact_work_.data_ptr<float>();
        uint64_t tiles = 0;
        for (size_t i = 0; i < n; ++i) {
            apexb::FactAux& x = aux[i];
            x.row_stat = v_[i].data_ptr<float>();
            x.col_stat = v_scale_[i].data_ptr<float>();
            x.row_work = w; w += fact_rows_[i];
            x.col_work = w; w += fact_cols_[i];
            x.rows = static_cast<int>(fact_rows_[i]);
            x.cols = static_cast<int>(fact_cols_[i]);
            x.tiles_c = static_cast<uint32_t>((fact_cols_[i] + apexb::kFactTileCols - 1) / apexb::kFactTileCols);
            x.tile_begin = static_cast<uint32_t>(tiles);
            tiles += static_cast<uint64_t>((fact_rows_[i] + apexb::kFactTileRows - 1) / apexb::kFactTileRows) * x.tiles_c;
            segs_[i].v = x.row_work;
            segs_[i].v_scale = x.col_work;
        }
        TORCH_CHECK(tiles < (1ull << 32), "StatePlan: too many statistics tiles for one launch");
        fact_tiles_ = static_cast<uint32_t>(tiles);
        d_fact_aux_ = at::empty({static_cast<int64_t>(std::max<size_t>(n, 1) * sizeof(apexb::FactAux))}, at::TensorOptions().dtype(at::kByte).device(device_));
        c10::cuda::CUDAGuard guard(device_);
        if (n > 0)
            check_cuda(cudaMemcpy(d_fact_aux_.data_ptr(), aux.data(), n * sizeof(apexb::FactAux), cudaMemcpyHostToDevice), "statistics table upload");
    }

    // decay_ranges[i]: empty, or sorted disjoint element ranges a0, b0, a1, b1, ... of segment i that get the decoupled
    // weight decay while the rest of the segment does not (the matrices inside a flat parameter).  Per 2048-element
    // chunk the kernel then reads one word: nothing / everything decays, or the number of a 256-byte bit mask.
    void build_partial_decay(const std::vector<std::vector<int64_t>>& decay_ranges) {
        const size_t n = segs_.size();
        bool any = false;
        for (const auto& r : decay_ranges) any = any || !r.empty();
        if (!any) return;
        TORCH_CHECK(decay_ranges.size() == n, "StatePlan: one (possibly empty) list of decay ranges per tensor");
        std::vector<uint32_t> words;           // chunk words of all segments with ranges, back to back
        std::vector<uint8_t> masks;            // bit masks of the mixed chunks
        std::vector<int64_t> first_word(n, -1);
        const int64_t C = apexb::kChunk2048;
        for (size_t i = 0; i < n; ++i) {
            const auto& r = decay_ranges[i];
            if (r.empty()) continue;
            TORCH_CHECK(r.size() % 2 == 0, "StatePlan: decay ranges come as pairs");
            TORCH_CHECK((segs_[i].flags & apexb::SEG_DECAY) == 0, "StatePlan: a tensor decays as a whole or by ranges, not both");
            const int64_t numel = segs_[i].numel;
            int64_t prev = 0;
            for (size_t k = 0; k < r.size(); k += 2) {
                TORCH_CHECK(r[k] >= prev && r[k + 1] >= r[k] && r[k + 1] <= numel, "StatePlan: decay ranges must be sorted, disjoint and inside the tensor");
                prev = r[k + 1];
            }
            const int64_t chunks = (numel + C - 1) / C;
            first_word[i] = static_cast<int64_t>(words.size());
            size_t k = 0;
            for (int64_t c = 0; c < chunks; ++c) {
                const int64_t lo = c * C, hi = std::min(numel, lo + C);
                while (k < r.size() && r[k + 1] <= lo) k += 2;            // ranges that end before this chunk
                int64_t covered = 0;
                for (size_t j = k; j < r.size() && r[j] < hi; j += 2)
                    covered += std::max<int64_t>(0, std::min(hi, r[j + 1]) - std::max(lo, r[j]));
                if (covered == 0) { words.push_back(0u); continue; }
                if (covered == hi - lo) { words.push_back(1u); continue; }
                const size_t base = masks.size();
                masks.resize(base + C / 8, 0);
                for (size_t j = k; j < r.size() && r[j] < hi; j += 2)
                    for (int64_t e = std::max(lo, r[j]); e < std::min(hi, r[j + 1]); ++e)
                        masks[base + (e - lo) / 8] |= static_cast<uint8_t>(1u << ((e - lo) % 8));
                words.push_back(static_cast<uint32_t>(base / (C / 8)) + 2u);
            }
        }
        auto bytes = at::TensorOptions().dtype(at::kByte).device(device_);
        c10::cuda::CUDAGuard guard(device_);
        d_decay_words_ = at::empty({static_cast<int64_t>(words.size() * sizeof(uint32_t))}, bytes);
        d_decay_masks_ = at::empty({static_cast<int64_t>(std::max<size_t>(masks.size(), 1))}, bytes);
        check_cuda(cudaMemcpy(d_decay_words_.data_ptr(), words.data(), words.size() * sizeof(uint32_t), cudaMemcpyHostToDevice), "decay table upload");
        if (!masks.empty())
            check_cuda(cudaMemcpy(d_decay_masks_.data_ptr(), masks.data(), masks.size(), cudaMemcpyHostToDevice), "decay mask upload");
        std::vector<apexb::SegExtra> extras(n);
        for (size_t i = 0; i < n; ++i) {
            extras[i].chunk_decay = first_word[i] < 0 ? nullptr
                : reinterpret_cast<const uint32_t*>(d_decay_words_.data_ptr()) + first_word[i];
            extras[i].masks = reinterpret_cast<const uint8_t*>(d_decay_masks_.data_ptr());
        }
        d_extras_ = at::empty({static_cast<int64_t>(n * sizeof(apexb::SegExtra))}, bytes);
        check_cuda(cudaMemcpy(d_extras_.data_ptr(), extras.data(), n * sizeof(apexb::SegExtra), cudaMemcpyHostToDevice), "decay record upload");
        mixed_chunks_ = static_cast<int64_t>(masks.size() / (C / 8));
    }
    int64_t mixed_decay_chunks() const { return mixed_chunks_; }
    int64_t kernel_class() const { return kernel_class_; }

    // Host table -> device.  Outside a stream capture: an ordinary copy from pageable memory (the driver has taken its
    // copy of the source when the call returns, so the next step may edit the table at once).  While the stream is
    // being captured into a CUDA graph the source must stay put: the table goes through a pinned mirror that only
    // captures write, and every replay of the graph copies that mirror again.
    void upload_table(cudaStream_t stream) {
        const size_t bytes = segs_.size() * sizeof(SegDesc);
        cudaStreamCaptureStatus cap = cudaStreamCaptureStatusNone;
        check_cuda(cudaStreamIsCapturing(stream, &cap), "capture query");
        const void* src = segs_.data();
        if (cap != cudaStreamCaptureStatusNone && bytes > 0) {
            if (!h_segs_pinned_.defined() || static_cast<size_t>(h_segs_pinned_.numel()) < bytes)
                h_segs_pinned_ = at::empty({static_cast<int64_t>(bytes)}, at::TensorOptions().dtype(at::kByte).pinned_memory(true));
            std::memcpy(h_segs_pinned_.data_ptr(), segs_.data(), bytes);
            src = h_segs_pinned_.data_ptr();
        }
        if (bytes > 0)
            check_cuda(cudaMemcpyAsync(d_segs_.data_ptr(), src, bytes, cudaMemcpyHostToDevice, stream), "segment table upload");
        dirty_ = false;
    }

    // Decide per segment whether full chunks may take the unpredicated bf16 path.
    // `zero` = gradients and parameter stores go through the symmetric flat buffers at s.offset.
    void refresh_fast_flags(bool zero) {
        for (auto& s : segs_) {
            auto al = [](const void* p, uintptr_t a) { return (reinterpret_cast<uintptr_t>(p) % a) == 0; };
            const bool quad = (s.flags & apexb::SEG_QUAD_V) != 0;
            bool fast = s.p_dtype == apexb::DT_BF16 && al(s.p, 16);
            fast = fast && (zero ? (s.offset % 8 == 0) : (s.g != nullptr && s.g_dtype == apexb::DT_BF16 && al(s.g, 16)));
            if (kernel_class_ >= 5) {
                fast = false;
            } else if (kernel_class_ <= 1) {
                fast = fast && s.m_fmt == apexb::M_BF16 && s.v_fmt == apexb::V_BF16 && al(s.m, 16) && al(s.v, quad ? 4 : 16);
            } else {
                fast = fast && kernel_class_ == 4 && al(s.m, 4) && al(s.v, 2);
            }
            const uint8_t want = static_cast<uint8_t>(fast ? (s.flags | apexb::SEG_FAST) : (s.flags & ~apexb::SEG_FAST));
            if (want != s.flags) { s.flags = want; dirty_ = true; }
        }
    }

    // Dense fp16 second moments are stored times 4^k; k per tensor (0..8), set again whenever the host re-centres a scale.
    void set_v_scale_log4(const std::vector<int64_t>& ks) {
        TORCH_CHECK(ks.size() == segs_.size(), "set_v_scale_log4: one exponent per tensor");
        for (size_t i = 0; i < ks.size(); ++i) {
            TORCH_CHECK(ks[i] >= 0 && ks[i] <= 8, "set_v_scale_log4: exponent out of range");
            TORCH_CHECK(ks[i] == 0 || segs_[i].v_fmt == apexb::V_F16, "set_v_scale_log4: only fp16 second moments are scaled");
            if (segs_[i].v_scale_log4 != static_cast<uint8_t>(ks[i])) { segs_[i].v_scale_log4 = static_cast<uint8_t>(ks[i]); dirty_ = true; }
        }
    }

    // The following step() calls take the step count and / or the learning rate from device tensors (0-dim fp32 on the
    // plan's device; undefined = the host value given here).  Nothing of the step then needs a value on the host, so
    // the step can be captured in a CUDA graph and replayed while the counters advance on the device.
    void set_device_scalars(c10::optional<at::Tensor> step_dev, c10::optional<at::Tensor> lr_dev, double step_host, double lr_host,
                            double alpha, double weight_decay, int64_t seed) {
        auto check = [&](const c10::optional<at::Tensor>& t, const char* what) {
            if (!t.has_value() || !t->defined()) return at::Tensor();
            TORCH_CHECK(t->device() == device_ && t->scalar_type() == at::kFloat && t->numel() == 1, "set_device_scalars: ", what,
                        " must be one fp32 value on the plan's device");
            return *t;
        };
        dyn_step_ = check(step_dev, "step");
        dyn_lr_ = check(lr_dev, "lr");
        TORCH_CHECK(dyn_step_.defined() || dyn_lr_.defined(), "set_device_scalars: neither scalar is a device tensor");
        dyn_step_host_ = step_host; dyn_lr_host_ = lr_host; dyn_alpha_ = alpha; dyn_weight_decay_ = weight_decay; dyn_seed_ = seed;
        dyn_on_ = true;
        if (!d_dyn_.defined())
            d_dyn_ = at::empty({static_cast<int64_t>(sizeof(apexb::DynScalars))}, at::TensorOptions().dtype(at::kByte).device(device_));
    }
    void clear_device_scalars() { dyn_on_ = false; dyn_step_ = at::Tensor(); dyn_lr_ = at::Tensor(); }

    // cap on the total number of CTAs of the next peer-kernel launches (0 = as many as are resident at once)
    void set_cta_cap(int64_t cap) { cta_cap_ = cap > 0 && cap < 65535 ? static_cast<uint32_t>(cap) : 0u; }
    int64_t total_chunks() const { return total_chunks_; }
    int64_t num_segments() const { return static_cast<int64_t>(segs_.size()); }
    int64_t launches() const { return launches_; }

    // Returns false (and launches nothing) when validation fails; raises on CUDA errors.
    void step(const std::vector<at::Tensor>& grads, double beta1, double beta2, double step_size, double eps_scaled,
              double eps, double eps_quad, double eps_quad_scaled, double decay_factor, double inv_scale, double gain_hi,
              double gain_lo, int64_t step_key, int64_t flags, c10::optional<at::Tensor> found_inf,
              c10::optional<at::Tensor> grad_scale, int64_t ctas_per_sm, double beta3, double slow_ratio, double lr) {
        const size_t n = segs_.size();
        TORCH_CHECK(grads.size() == n, "StatePlan.step: expected ", n, " gradients, got ", grads.size());
        // phase 1: validate everything before touching device state
        for (size_t i = 0; i < n; ++i) {
            const at::Tensor& g = grads[i];
            TORCH_CHECK(g.device() == device_, "StatePlan.step: gradient on another device");
            TORCH_CHECK(g.is_contiguous() && g.numel() == segs_[i].numel, "StatePlan.step: gradient must be contiguous and match its parameter");
            const int code = float_code(g, "grad");
            if (segs_[i].g != g.data_ptr() || segs_[i].g_dtype != code) {
                segs_[i].g = g.data_ptr();
                segs_[i].g_dtype = static_cast<uint8_t>(code);
                dirty_ = true;
            }
        }
        const float* fi = nullptr;
        const float* gs = nullptr;
        if (found_inf.has_value() && found_inf->defined()) {
            TORCH_CHECK(found_inf->device() == device_ && found_inf->scalar_type() == at::kFloat, "found_inf must be fp32 on the plan's device");
            fi = found_inf->data_ptr<float>();
        }
        if (grad_scale.has_value() && grad_scale->defined()) {
            TORCH_CHECK(grad_scale->device() == device_ && grad_scale->scalar_type() == at::kFloat, "grad_scale must be fp32 on the plan's device");
            gs = grad_scale->data_ptr<float>();
        }
        if (dirty_) refresh_fast_flags(false);
        // phase 2: launch
        c10::cuda::CUDAGuard guard(device_);
        cudaStream_t stream = at::cuda::getCurrentCUDAStream(device_.index()).stream();
        if (dirty_) upload_table(stream);
        TORCH_CHECK((flags & (apexb::STEP_LION | apexb::STEP_SLOW | apexb::STEP_AMSGRAD)) == 0 || kernel_class_ == 0 ||
                        (kernel_class_ == 7 && (flags & (apexb::STEP_SLOW | apexb::STEP_AMSGRAD)) == 0),
                    "StatePlan.step: AdEMAMix / AMSGrad run on the dense formats only, Lion on dense or int8 momentum");
        TORCH_CHECK(kernel_class_ != 7 || (flags & apexb::STEP_LION), "StatePlan.step: class 7 is Lion's");
        TORCH_CHECK(kernel_class_ < 5 || !(flags & apexb::STEP_CAUTIOUS), "StatePlan.step: this layout has no cautious mode on the kernel");
        TORCH_CHECK(!(flags & apexb::STEP_SLOW) || (n == 0 || segs_[0].m_scale != nullptr), "StatePlan.step: AdEMAMix needs the slow moments");
        TORCH_CHECK(!(flags & apexb::STEP_AMSGRAD) || (n == 0 || segs_[0].v_scale != nullptr), "StatePlan.step: AMSGrad needs the running maxima");
        StepArgs a = make_step_args(beta1, beta2, step_size, eps_scaled, eps, eps_quad, eps_quad_scaled, decay_factor,
                                          inv_scale, gain_hi, gain_lo, step_key, flags, n, total_chunks_, beta3, slow_ratio, lr);
        a.interleave = chunk_order(true) | table_check_bit();
        const int max_ctas = sm_count_ * static_cast<int>(ctas_per_sm > 0 ? ctas_per_sm : state_ctas_per_sm(apexb_fused_state_ctas_per_sm()));
        unsigned long long* keep = nullptr;
        if ((flags & apexb::STEP_CAUTIOUS) && kernel_class_ <= 1) {      // dense cautious: per-tensor kept counts
            TORCH_CHECK(!(flags & (apexb::STEP_NESTEROV | apexb::STEP_LION | apexb::STEP_SLOW | apexb::STEP_AMSGRAD)),
                        "StatePlan.step: dense cautious combines with neither Nesterov nor Lion / AdEMAMix / AMSGrad");
            if (!d_keep_counts_.defined())
                d_keep_counts_ = at::empty({static_cast<int64_t>(n)}, at::TensorOptions().dtype(at::kLong).device(device_));
            keep = reinterpret_cast<unsigned long long*>(d_keep_counts_.data_ptr());
            check_cuda(cudaMemsetAsync(keep, 0, n * sizeof(unsigned long long), stream), "kept-count reset");
        }
        if (kernel_class_ == 6 && n > 0) {     // factored second moment: row / column statistics of this step's gradients first
            check_cuda(cudaMemsetAsync(d_fact_work_.data_ptr(), 0, static_cast<size_t>(d_fact_work_.numel()) * sizeof(float), stream),
                       "statistics reset");
            check_cuda(apexb_factored_stats_launch(d_segs_.data_ptr(), d_fact_aux_.data_ptr(), static_cast<int>(n), fact_tiles_, &a, fi, gs,
                                                   max_ctas, stream), "factored statistics launch");
        }
        const apexb::DynScalars* dyn = nullptr;
        if (dyn_on_) {       // step count and / or learning rate are device tensors: derive what depends on them there
            if (!d_dyn_.defined())
                d_dyn_ = at::empty({static_cast<int64_t>(sizeof(apexb::DynScalars))}, at::TensorOptions().dtype(at::kByte).device(device_));
            apexb::DynInputs in;
            in.step_dev = dyn_step_.defined() ? dyn_step_.data_ptr<float>() : nullptr;
            in.lr_dev = dyn_lr_.defined() ? dyn_lr_.data_ptr<float>() : nullptr;
            in.step_host = dyn_step_host_;
            in.lr_host = dyn_lr_host_;
            in.beta1 = beta1; in.beta2 = beta2; in.beta3 = beta3;
            in.alpha = dyn_alpha_; in.eps = eps; in.eps_quad = eps_quad;
            in.weight_decay = dyn_weight_decay_;
            in.pad = 0;
            in.seed = static_cast<uint32_t>(dyn_seed_);
            apexb::DynScalars* out = reinterpret_cast<apexb::DynScalars*>(d_dyn_.data_ptr());
            check_cuda(apexb_dyn_scalars_launch(&in, out, stream), "dyn_scalars launch");
            dyn = out;
        }
        check_cuda(apexb_fused_state_launch(kernel_class_, d_segs_.data_ptr(), &a, fi, gs, max_ctas,
                                            d_extras_.defined() ? d_extras_.data_ptr() : nullptr, keep, dyn, stream), "fused_state launch");
        ++launches_;
    }

    // Fused ZeRO step of this rank's shard (see zero_fused.cu).  Pointers are raw addresses of
    // every rank's flat gradient buffer, flat parameter buffer and signal pad as mapped here.
    void step_zero(const std::vector<int64_t>& peer_grad, const std::vector<int64_t>& peer_param,
                   const std::vector<int64_t>& peer_signal, int64_t rank, int64_t epoch, double timeout_ms, at::Tensor status,
                   int64_t grad_dtype_code, int64_t param_dtype_code, double beta1, double beta2, double step_size,
                   double eps_scaled, double eps, double eps_quad, double eps_quad_scaled, double decay_factor, double inv_scale,
                   double gain_hi, double gain_lo, int64_t step_key, int64_t flags, int64_t mc_grad, int64_t mc_param,
                   c10::optional<at::Tensor> clip_total_sq, double clip_max_norm) {
        const size_t W = peer_param.size();
        TORCH_CHECK(W >= 1 && W <= static_cast<size_t>(apexb::kMaxPeers) && peer_signal.size() == W &&
                        (peer_grad.size() == W || peer_grad.size() == 1),
                    "step_zero: between 1 and ", apexb::kMaxPeers, " peers expected (gradient sources: all peers or just the local one)");
        TORCH_CHECK(rank >= 0 && static_cast<size_t>(rank) < W, "step_zero: bad rank");
        TORCH_CHECK((flags & (apexb::STEP_LION | apexb::STEP_SLOW | apexb::STEP_AMSGRAD)) == 0,
                    "step_zero: Lion / AdEMAMix / AMSGrad are not part of the peer-memory step");
        TORCH_CHECK(!(flags & apexb::STEP_CAUTIOUS) || kernel_class_ >= 2, "step_zero: dense cautious is not part of the peer-memory step");
        TORCH_CHECK(kernel_class_ <= 4, "step_zero: the int8 + dense layout is not part of the peer-memory step");
        TORCH_CHECK(status.device() == device_ && status.scalar_type() == at::kInt && status.numel() >= 1, "step_zero: status must be an int32 tensor on the plan's device");
        apexb::ZeroPeers peers;
        std::memset(&peers, 0, sizeof(peers));
        for (size_t r = 0; r < peer_grad.size(); ++r) {
            TORCH_CHECK(peer_grad[r] != 0 && peer_grad[r] % 16 == 0, "step_zero: gradient buffers must be non-null and 16-byte aligned");
            peers.grad[r] = reinterpret_cast<const void*>(peer_grad[r]);
        }
        for (size_t r = 0; r < W; ++r) {
            TORCH_CHECK(peer_param[r] != 0 && peer_signal[r] != 0, "step_zero: null peer pointer");
            TORCH_CHECK(peer_param[r] % 16 == 0, "step_zero: peer buffers must be 16-byte aligned");
            peers.param[r] = reinterpret_cast<void*>(peer_param[r]);
            peers.signal[r] = reinterpret_cast<uint32_t*>(peer_signal[r]);
        }
        peers.grad_sources = static_cast<int>(peer_grad.size());
        peers.world = static_cast<int>(W);
        peers.rank = static_cast<int>(rank);
        TORCH_CHECK((mc_grad == 0) == (mc_param == 0) && mc_grad % 16 == 0 && mc_param % 16 == 0,
                    "step_zero: multicast addresses come as a 16-byte aligned pair (or not at all)");
        peers.mc_grad = reinterpret_cast<const void*>(mc_grad);
        peers.mc_param = reinterpret_cast<void*>(mc_param);
        c10::cuda::CUDAGuard guard(device_);
        check_cuda(apexb_zero_init(device_.index()), "codec table upload");
        cudaStream_t stream = at::cuda::getCurrentCUDAStream(device_.index()).stream();
        const size_t n = segs_.size();
        if (dirty_) refresh_fast_flags(true);
        if (dirty_ && n > 0) upload_table(stream);
        StepArgs a = make_step_args(beta1, beta2, step_size, eps_scaled, eps, eps_quad, eps_quad_scaled, decay_factor,
                                          inv_scale, gain_hi, gain_lo, step_key, flags, n, total_chunks_);
        a.interleave = chunk_order(true) | table_check_bit() | zero_tuning() | (cta_cap_ << 16);
        const long long budget = static_cast<long long>(timeout_ms * static_cast<double>(clock_khz_));
        const float* clip = nullptr;
        if (clip_total_sq.has_value() && clip_total_sq->defined()) {
            TORCH_CHECK(clip_total_sq->device() == device_ && clip_total_sq->scalar_type() == at::kFloat && clip_total_sq->numel() == 1,
                        "step_zero: clip_total_sq must be one fp32 value on the plan's device");
            clip = clip_total_sq->data_ptr<float>();
        }
        check_cuda(apexb_zero_fused_launch(kernel_class_, d_segs_.data_ptr(), &a, &peers, static_cast<uint32_t>(epoch), budget,
                                           reinterpret_cast<uint32_t*>(status.data_ptr<int>()), static_cast<int>(grad_dtype_code),
                                           static_cast<int>(param_dtype_code), sm_count_, clip, static_cast<float>(clip_max_norm),
                                           stream),
                   "zero_fused launch");
        ++launches_;
    }

    // Phase 1 of a clipped step: reduce-scatter of this plan's shard (bf16 gradients) with its sum of squares added to
    // group_acc (see zero_fused.cu).  scratch: fp32, at least 3 x SM count entries.
    void reduce_zero(const std::vector<int64_t>& peer_grad, const std::vector<int64_t>& peer_signal, int64_t rank, int64_t epoch,
                     double timeout_ms, at::Tensor status, double inv_scale, at::Tensor scratch, at::Tensor group_acc) {
        const size_t W = peer_grad.size();
        TORCH_CHECK(W >= 1 && W <= static_cast<size_t>(apexb::kMaxPeers) && peer_signal.size() == W && rank >= 0 &&
                        static_cast<size_t>(rank) < W, "reduce_zero: between 1 and ", apexb::kMaxPeers, " peers expected");
        TORCH_CHECK(status.device() == device_ && status.scalar_type() == at::kInt && status.numel() >= 1, "reduce_zero: status must be an int32 tensor on the plan's device");
        TORCH_CHECK(scratch.device() == device_ && scratch.scalar_type() == at::kFloat && scratch.is_contiguous() &&
                        group_acc.device() == device_ && group_acc.scalar_type() == at::kFloat && group_acc.numel() == 1,
                    "reduce_zero: fp32 scratch and a one-element fp32 accumulator on the plan's device expected");
        apexb::ZeroPeers peers;
        std::memset(&peers, 0, sizeof(peers));
        for (size_t r = 0; r < W; ++r) {
            TORCH_CHECK(peer_grad[r] != 0 && peer_grad[r] % 16 == 0 && peer_signal[r] != 0, "reduce_zero: bad peer pointer");
            peers.grad[r] = reinterpret_cast<const void*>(peer_grad[r]);
            peers.signal[r] = reinterpret_cast<uint32_t*>(peer_signal[r]);
        }
        peers.grad_sources = peers.world = static_cast<int>(W);
        peers.rank = static_cast<int>(rank);
        c10::cuda::CUDAGuard guard(device_);
        cudaStream_t stream = at::cuda::getCurrentCUDAStream(device_.index()).stream();
        const size_t n = segs_.size();
        if (dirty_) refresh_fast_flags(true);
        if (dirty_ && n > 0) upload_table(stream);
        const long long budget = static_cast<long long>(timeout_ms * static_cast<double>(clock_khz_));
        check_cuda(apexb_zero_reduce_launch(d_segs_.data_ptr(), static_cast<int>(n), total_chunks_, &peers, static_cast<uint32_t>(epoch),
                                            budget, reinterpret_cast<uint32_t*>(status.data_ptr<int>()), static_cast<float>(inv_scale),
                                            scratch.data_ptr<float>(), static_cast<int>(scratch.numel()), group_acc.data_ptr<float>(),
                                            sm_count_, stream),
                   "zero_reduce launch");
        ++launches_;
    }

  private:
    int clock_khz_ = 1000000;
    int kernel_class_;
    std::vector<at::Tensor> params_, m_, v_, m_scale_, v_scale_;
    std::vector<SegDesc> segs_;
    at::Tensor d_segs_;
    at::Tensor d_extras_, d_decay_words_, d_decay_masks_;     // partial decay of flat parameters (undefined when unused)
    at::Tensor dyn_step_, dyn_lr_, d_dyn_;                    // device-resident step count / learning rate and what is derived from them
    bool dyn_on_ = false;
    double dyn_step_host_ = 0, dyn_lr_host_ = 0, dyn_alpha_ = 0, dyn_weight_decay_ = 0;
    int64_t dyn_seed_ = 0;
    std::vector<int64_t> fact_rows_, fact_cols_;              // factored layout: matrix shape per segment
    at::Tensor d_fact_work_, d_fact_aux_;
    uint32_t fact_tiles_ = 0;
    at::Tensor h_segs_pinned_;                                // table mirror for uploads inside a stream capture
    at::Tensor d_keep_counts_;                                // dense cautious: kept elements per segment (lazily allocated)
    int64_t mixed_chunks_ = 0;
    at::Device device_{at::kCPU};
    uint32_t total_chunks_ = 0;
    uint32_t cta_cap_ = 0;
    int sm_count_ = 148;
    bool dirty_ = true;
    int64_t launches_ = 0;
};


// Ranks swap their partial sums of squares through the signal pads; total_out = sum over ranks (see zero_fused.cu).
inline void zero_norm_exchange(const std::vector<int64_t>& peer_signal, int64_t rank, int64_t epoch, double timeout_ms,
                               at::Tensor status, at::Tensor group_acc, at::Tensor total_out) {
    const size_t W = peer_signal.size();
    TORCH_CHECK(W >= 1 && W <= static_cast<size_t>(apexb::kMaxPeers) && rank >= 0 && static_cast<size_t>(rank) < W, "zero_norm_exchange: bad peers");
    TORCH_CHECK(group_acc.is_cuda() && group_acc.scalar_type() == at::kFloat && group_acc.numel() == 1 &&
                    total_out.device() == group_acc.device() && total_out.scalar_type() == at::kFloat && total_out.numel() == 1 &&
                    status.device() == group_acc.device() && status.scalar_type() == at::kInt,
                "zero_norm_exchange: one-element fp32 tensors and an int32 status word on one CUDA device expected");
    apexb::ZeroPeers peers;
    std::memset(&peers, 0, sizeof(peers));
    for (size_t r = 0; r < W; ++r) {
        TORCH_CHECK(peer_signal[r] != 0, "zero_norm_exchange: null signal pad");
        peers.signal[r] = reinterpret_cast<uint32_t*>(peer_signal[r]);
    }
    peers.world = static_cast<int>(W);
    peers.rank = static_cast<int>(rank);
    c10::cuda::CUDAGuard guard(group_acc.device());
    const int dev = group_acc.device().index();
    const long long budget = static_cast<long long>(timeout_ms * static_cast<double>(at::cuda::getDeviceProperties(dev)->clockRate));
    check_cuda(apexb_zero_norm_exchange(&peers, static_cast<uint32_t>(epoch), budget, reinterpret_cast<uint32_t*>(status.data_ptr<int>()),
                                        group_acc.data_ptr<float>(), total_out.data_ptr<float>(),
                                        at::cuda::getCurrentCUDAStream(dev).stream()),
               "zero_norm_exchange launch");
}

}  // namespace apexb_host
