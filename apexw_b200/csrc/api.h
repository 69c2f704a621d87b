// C entry points of the native library.  The .cu translation units implement
// them with raw pointers and a stream; bindings.cpp wraps them for Python.
// Every function returns 0 on success or a cudaError_t value.
#pragma once
#include <cuda_runtime.h>
#include <cstdint>
#include "plan_types.h"

extern "C" {

// ---- fused optimizer state (fused_state.cu) --------------------------------
// Upload the codec tables to the current device (idempotent per device).
int apexb_fused_state_init(int device);
// resident CTAs per SM the state kernels were compiled for (their register budget)
int apexb_fused_state_ctas_per_sm();
// One persistent launch over a device-resident array of SegDesc.
// found_inf / grad_scale may be null; when given they are read on the device.
// kernel_class: 0 dense, 1 dense with one variance per four elements, 2 int8+log-u8,
// 3 NF4+log-u8, 4 NF4 + log-u8 shared by four, 5 int8 + dense second moment ("ultra"), 6 row / column factored second moment
// (after apexb_factored_stats_launch), 7 Lion on an int8 first moment.  All segments of a launch
// share the class.
// d_extras: null, or one apexb::SegExtra per segment (decay that covers parts of a flat parameter only).
// d_keep_counts: one zeroed 64-bit counter per segment when the step is cautious and the class is 0 or 1 (a counting
// pass runs first and the update scales by the kept fraction of each tensor); null otherwise.
// Lion / AdEMAMix / AMSGrad flags are honoured for class 0 only.
int apexb_fused_state_launch(int kernel_class, const void* d_segments, const apexb::StepArgs* args,
                             const float* found_inf, const float* grad_scale, int max_ctas, const void* d_extras,
                             unsigned long long* d_keep_counts, const apexb::DynScalars* d_dyn, cudaStream_t stream);
// d_dyn: null, or step-dependent scalars that a preceding apexb_dyn_scalars_launch derived on the device (the step
// count or the learning rate is a device tensor); they replace the corresponding fields of *args inside the kernel.
// Host class 6 (factored second moment): this launch pair runs before apexb_fused_state_launch of the same plan; the
// work vectors named by the FactAux records must have been zeroed on the same stream.
int apexb_factored_stats_launch(const void* d_segments, const void* d_aux, int num_segments, unsigned total_tiles,
                                const apexb::StepArgs* args, const float* found_inf, const float* grad_scale, int max_ctas,
                                cudaStream_t stream);
int apexb_dyn_scalars_launch(const apexb::DynInputs* in, apexb::DynScalars* d_out, cudaStream_t stream);

// Debug mode (bit 1 of StepArgs::interleave): the kernels validate every chunk's table record before indexing with
// it, skip what fails and record the first failure.  out: {code (apexb::TableFault), segment, chunk, skipped chunks}.
int apexb_fused_state_table_fault(unsigned out[4], int clear);
int apexb_zero_table_fault(unsigned out[4], int clear);
// The checker on hand-made records (nothing is dereferenced): bit i of *d_caught = case i behaved; 15 cases.
int apexb_table_check_selftest(unsigned* d_caught, void* some_aligned_address, cudaStream_t stream);

// ---- fused ZeRO step over peer memory (zero_fused.cu) -------------------------
int apexb_zero_init(int device);
// One launch per kernel class.  Every rank must issue the same sequence of launches with
// the same epochs (epoch grows by one per launch); a rank without work in a class still
// launches (total_chunks = 0) so that the flag rounds match.  status: one device word,
// 0 = ok, 1 = entry wait expired (nothing updated), 2 = exit wait expired, 3 = internal.
// clip_total_sq (nullable, one device float): squared global norm of the reduced gradient; the kernel then multiplies the
// gradient scale by min(1, clip_max_norm / (sqrt(total) + 1e-6)).
int apexb_zero_fused_launch(int kernel_class, const void* d_segments, const apexb::StepArgs* args,
                            const apexb::ZeroPeers* peers, uint32_t epoch, long long wait_budget_cycles, uint32_t* status,
                            int g_dtype, int p_dtype, int sm_count, const float* clip_total_sq, float clip_max_norm,
                            cudaStream_t stream);
// Clipped steps, phase 1: reduce-scatter only (bf16 gradients).  The shard's gradient is summed over the ranks, times
// inv_scale, written back over this rank's own copy, and its squares are added to *group_acc (cta_partials: scratch
// of at least 3 x SM count floats).  Same epoch / status rules as the fused launch.
int apexb_zero_reduce_launch(const void* d_segments, int num_segments, unsigned total_chunks, const apexb::ZeroPeers* peers,
                             uint32_t epoch, long long wait_budget_cycles, uint32_t* status, float inv_scale,
                             float* cta_partials, int cta_partials_len, float* group_acc, int sm_count, cudaStream_t stream);
// ... and the exchange of the ranks' partial sums through the signal pads: *total_out = sum over ranks of *group_acc
// (which is cleared for the next step).
int apexb_zero_norm_exchange(const apexb::ZeroPeers* peers, uint32_t epoch, long long wait_budget_cycles, uint32_t* status,
                             float* group_acc, float* total_out, cudaStream_t stream);

// ---- distributed Muon over peer memory (muon_dist.cu) ---------------------------
// gather: peer-reduce gradients of the owned matrices, update the owner's fp32 momentum, stage the bf16
// Newton-Schulz input (entry flag round inside).  scatter: apply decay + update and store the parameters
// into every rank's buffer (exit flag round inside).  Same status codes and epoch rule as the ZeRO kernel.
// do_entry / do_exit: a step may be split into several gathers and scatters (one pair per batch of matrices, so that
// they overlap with the Newton-Schulz kernels of other batches); only the first gather runs the entry round and only
// the last scatter, on the same stream as the other scatters, runs the exit round.
int apexb_muon_gather(const void* d_segments, int nseg, unsigned total_chunks, const apexb::ZeroPeers* peers, float momentum,
                      float inv_world, int nesterov, int do_entry, uint32_t epoch, long long wait_budget_cycles,
                      uint32_t* status, int sm_count, cudaStream_t stream);
int apexb_muon_scatter(const void* d_segments, int nseg, unsigned total_chunks, const apexb::ZeroPeers* peers, float lr, float decay,
                       int do_exit, uint32_t epoch, long long wait_budget_cycles, uint32_t* status, int sm_count,
                       cudaStream_t stream);

// ---- Newton-Schulz GEMM on tcgen05 (ns_gemm.cu) --------------------------------
int apexb_ns_smem_bytes();
// Xs = G * inv[batch] and XsT = Xs^T in one pass (bf16 [batch, rows, cols], rows and cols multiples of 64)
int apexb_ns_prep(const void* G, const float* inv, void* Xs, void* XsT, int batch, int rows, int cols, cudaStream_t stream);
// tile width (128 or 256) that apexb_ns_gemm should be given for a problem
int apexb_ns_pick_bn(int M, int N, int batch, int symmetric, int sm_count);
// kernel and tile for a problem: 128 or 256 = one CTA per 128 x bn tile; 512 = a pair of CTAs (cluster of two,
// tcgen05.mma.cta_group::2) per 256 x 256 tile.  APEXW_B200_NS_PAIR=0 / 1 forces the choice where it is legal.
int apexb_ns_pick_tile(int M, int N, int K, int batch, int symmetric, int sm_count);
// C = alpha * A * B^T + beta * D (+ optional Ct = C^T); tensor maps describe A [batch, M, K] and
// B [batch, N, K] as 3-D bf16 tensors with boxes 64 x 128 and 64 x bn and 128-byte swizzle (bn = 512: CTA pairs on
// 256 x 256 tiles, M a multiple of 256, B box 64 x 128).
// symmetric != 0 (needs M == N and Ct == C): only tiles that touch the upper triangle are computed and the
// transposed store mirrors them.  The kernel is persistent: sm_count CTAs at most.
// error_flag: one device word, set non-zero when a bounded wait expired.
int apexb_ns_gemm(const void* tensor_map_a, const void* tensor_map_b, const void* D, void* C, void* Ct, long long strideD,
                  long long strideC, long long strideCt, int M, int N, int K, int batch, float alpha, float beta,
                  int symmetric, int bn, int sm_count, unsigned* error_flag, cudaStream_t stream);

// ---- model-side fused ops (model_ops.cu) ------------------------------------
int apexb_rmsnorm_fwd(const void* x, const void* res, const void* w, void* y, void* h_out, float* rstd, int rows, int H,
                      float eps, int is_bf16, int sm_count, cudaStream_t stream);
// number of [H]-sized fp32 partial rows the backward kernel needs as scratch
int apexb_rmsnorm_bwd_parts(int rows, int sm_count);
int apexb_rmsnorm_bwd(const void* dy, const void* dres, const void* h, const void* w, const float* rstd, void* dx, float* dw,
                      float* partial, int nparts, int rows, int H, int is_bf16, cudaStream_t stream);
int apexb_swiglu_fwd(const void* gu, void* y, long long rows, int F, int is_bf16, int sm_count, cudaStream_t stream);
int apexb_swiglu_bwd(const void* dy, const void* gu, void* dgu, long long rows, int F, int is_bf16, int sm_count,
                     cudaStream_t stream);
int apexb_rope(const void* in, void* out, const float* cosv, const float* sinv, long long tokens, int S, int heads, int D,
               int n_rot, int inverse, int is_bf16, int sm_count, cudaStream_t stream);
// targets outside [0, V) mark ignored rows (loss 0, zero gradient row); scale_dev: optional device float that multiplies scale
int apexb_cross_entropy(void* logits, const long long* targets, float* losses, int rows, int V, float scale,
                        const float* scale_dev, int is_bf16, cudaStream_t stream);

}  // extern "C"
