// Internal launcher declarations shared by the kernel translation units and the C ABI.
#pragma once

#include <cuda_runtime.h>
#include <stdint.h>

#include "../../include/nvfp4_b200.h"

namespace nvfp4 {

// quant_kernels.cu --------------------------------------------------------------------------
int launch_row_amax(cudaStream_t s, const void* x, int dtype, float* out, uint32_t rows, uint32_t row_len);
int launch_tensor_amax(cudaStream_t s, const void* x, int dtype, float* chunk_amax, float* out, uint64_t n);
int launch_nvfp4_amax(cudaStream_t s, const uint8_t* bytes, const uint8_t* scales, const float* gscales, uint32_t rows,
                      uint32_t cols, int rowwise, int packed, float* chunk_amax, float* out);
// transform 0: out[0] = max(chunks); 1: out[0] = MS-EDEN global scale of that max
int launch_amax_from_chunks(cudaStream_t s, const float* chunk_amax, float* out, uint32_t chunk_count, int transform);
int launch_ms_eden_scale_from_amax(cudaStream_t s, const float* amax, float* out);
// relu2: quantize relu(x)^2 computed on load; decoded_amax (optional f32[1]): max |decoded value| of the result
int launch_four_six(cudaStream_t s, const void* x, int dtype, const float* amax, int rowwise, uint32_t rows,
                    uint32_t cols, uint8_t* out_fp4, uint8_t* out_scales, int packed, float* out_gs, int relu2 = 0,
                    float* decoded_amax = nullptr);
int launch_four_six_rowwise_fused(cudaStream_t s, const void* x, int dtype, uint32_t rows, uint32_t cols,
                                  uint8_t* out_fp4, uint8_t* out_scales, int packed, float* out_gs, float* out_amax,
                                  float* decoded_amax, int relu2 = 0);
int launch_four_six_padded(cudaStream_t s, const float* x, const float* amax, uint8_t* out_fp4, uint8_t* out_scales,
                           float* out_gs, uint32_t rows, uint32_t cols, uint32_t padded_rows, uint32_t padded_cols,
                           int transposed);
int launch_packed_scale_pad(cudaStream_t s, uint8_t* packed, uint32_t rows, uint32_t k_dim);
// y = z + beta * (x - z) -> tensor amax -> four-six (tensor scale); chunk_amax optional
int launch_schedule_free_materialize(cudaStream_t s, const float* z, const float* x, float beta, float* chunk_amax,
                                     float* amax, uint8_t* out_fp4, uint8_t* out_scales, int packed, float* out_gs,
                                     uint32_t rows, uint32_t cols);
// amax_in / gs_out (optional): the global scale is the MS-EDEN scale of amax_in[0] (derived inside the kernel
// where the kernel supports it, by a one-thread kernel otherwise) and is written to gs_out[0]; a.global_scale
// and a.host_global_scale are then not read.
int launch_ms_eden(cudaStream_t s, const nvfp4_ms_eden_args& a, const float* amax_in = nullptr, float* gs_out = nullptr);
// Pair quantization; when col_sum_partials != nullptr (and ms_eden_pair_is_tiled) it also writes the
// per-row-tile column sums [ms_eden_pair_row_tiles(rows)][cols] for launch_col_sum_reduce.
// amax_in / gs_out (only when ms_eden_pair_takes_amax): the kernel derives the global scale from amax_in[0]
// itself and writes it to gs_out[0]; rows.global_scale / transposed.global_scale are then not read.
int launch_ms_eden_pair(cudaStream_t s, const nvfp4_ms_eden_args& rows, const nvfp4_ms_eden_args& transposed,
                        float* col_sum_partials = nullptr, const float* amax_in = nullptr, float* gs_out = nullptr);
bool ms_eden_pair_takes_amax(const nvfp4_ms_eden_args& rows, const nvfp4_ms_eden_args& transposed);
bool ms_eden_pair_is_tiled(const nvfp4_ms_eden_args& rows, const nvfp4_ms_eden_args& transposed);
uint32_t ms_eden_pair_row_tiles(uint32_t rows);
int launch_col_sum_reduce(cudaStream_t s, const float* partials, float* dbias, uint32_t tiles, uint32_t n);
int launch_decode(cudaStream_t s, const uint8_t* bytes, const uint8_t* scales, const float* gscales, int rowwise,
                  int transpose, float* out, uint32_t rows, uint32_t cols);
int launch_scale_pack(cudaStream_t s, const uint8_t* logical, uint8_t* packed, uint32_t mn, uint32_t k_dim);
int launch_pad_u4_rows(cudaStream_t s, const uint8_t* src, uint8_t* dst, uint32_t rows, uint32_t padded_rows,
                       uint32_t cols);
int launch_pad_f32(cudaStream_t s, const float* src, float* dst, uint32_t rows, uint32_t cols, uint32_t padded_rows,
                   uint32_t padded_cols, int transpose);
int launch_crop_f32(cudaStream_t s, const float* src, float* dst, uint32_t rows, uint32_t src_cols, uint32_t dst_cols);
int launch_postop(cudaStream_t s, float* raw, float* other, const uint8_t* bias_bytes, const uint8_t* bias_scales,
                  const float* bias_gs, uint32_t rows, uint32_t cols, int mode);
int launch_bias_grad(cudaStream_t s, const void* e, int dtype, float* dbias, uint32_t tokens, uint32_t n);
// d_pre = (d_out * 2) * max(pre, 0); pre_kind 0 f32, 1 bf16, 2 f16; gradients f32 or (grad_bf16) bf16.
// chunk_amax (optional, relu2_backward_grid(n) floats): per-CTA amax of the stored gradient.
int launch_relu2_backward(cudaStream_t s, const void* pre, int pre_kind, const void* d_out, void* d_pre, int grad_bf16,
                          uint64_t n, float* chunk_amax = nullptr);
uint32_t relu2_backward_grid(uint64_t n);

// gemm_tcgen05.cu ---------------------------------------------------------------------------
int launch_gemm(cudaStream_t s, const nvfp4_gemm_args& a);
// What launch_gemm would choose for these arguments on the current device (no launch).
int gemm_plan_query(const nvfp4_gemm_args& a, nvfp4_gemm_plan* out);
// Encodes (and keeps in the calling thread's cache) the operand tensor maps of a GEMM ahead of its launch.
int gemm_prepare_operand_maps(const uint8_t* a_bytes, const uint8_t* b_bytes, uint32_t m, uint32_t k, uint32_t n);
// Measurement / test aids: forced tile shape (block_n 0 = automatic), limit of the kernel's bounded waits,
// debug flags (bit 0: CTA 0 of every GEMM never loads its first k-tile), tensor-map cache counters.
void gemm_set_tile_override(int block_m, int block_n);
void gemm_set_wait_timeout_ns(uint64_t ns);
void gemm_set_debug_flags(uint32_t flags);
void gemm_map_cache_stats(uint64_t* hits, uint64_t* misses);
// 1: split-K never uses more than two splits (run-to-run identical sums); 0 (default): as many as fill the SMs
void gemm_set_deterministic(int on);
int gemm_get_deterministic();
int gemm_timing_begin(uint32_t max_records);
int gemm_timing_end(uint32_t* count, double* total_ms, double* total_flops, float* per_launch_ms,
                    double* per_launch_flops, uint32_t capacity);
// Device status word written by kernels whose bounded waits expired (0 = never).
uint32_t* device_status_word();

void set_last_error(const char* msg);
// Host-side tally of kernel launches made by this library (read through nvfp4_launch_count).
void count_launch();

}  // namespace nvfp4
