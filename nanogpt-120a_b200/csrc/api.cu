// extern "C" boundary of the NVFP4 projection path: argument checks, composition of the
// kernels into the reference's host-level operations, and nothing else.  Each entry cites
// the reference method it replaces in include/nvfp4_b200.h.
#include <atomic>
#include <cstdio>
#include <cstring>

#include "kernels.h"

namespace nvfp4 {

static thread_local char g_last_error[256] = "";
static std::atomic<uint64_t> g_launches{0};

void count_launch() { g_launches.fetch_add(1, std::memory_order_relaxed); }

void set_last_error(const char* msg) {
  std::strncpy(g_last_error, msg, sizeof(g_last_error) - 1);
  g_last_error[sizeof(g_last_error) - 1] = '\0';
}

static int invalid(const char* msg) {
  set_last_error(msg);
  return static_cast<int>(cudaErrorInvalidValue);
}

static inline cudaStream_t S(void* stream) { return static_cast<cudaStream_t>(stream); }

static inline uint32_t padded_k(uint32_t k) { return (k + 63u) / 64u * 64u; }
static inline uint32_t chunks1024(uint64_t n) { return static_cast<uint32_t>((n + 1023) / 1024); }
static const float kQuartetSO = (17.0f / 16.0f) * 0.93f;  // utils/quartet.rs:1

}  // namespace nvfp4

using namespace nvfp4;

extern "C" {

int nvfp4_abi_version(void) { return 3; }
uint64_t nvfp4_launch_count(void) { return g_launches.load(std::memory_order_relaxed); }
const char* nvfp4_last_error(void) { return g_last_error; }

int nvfp4_read_device_status(void* stream, uint32_t* status_out) {
  uint32_t* word = device_status_word();
  if (!word || !status_out) return invalid("device status word unavailable");
  cudaError_t e = cudaMemcpyAsync(status_out, word, sizeof(uint32_t), cudaMemcpyDeviceToHost, S(stream));
  if (e == cudaSuccess) e = cudaMemsetAsync(word, 0, sizeof(uint32_t), S(stream));
  if (e == cudaSuccess) e = cudaStreamSynchronize(S(stream));
  return static_cast<int>(e);
}

uint32_t nvfp4_padded_k(uint32_t k) { return padded_k(k); }
uint32_t nvfp4_scale_padded_mn_extent(uint32_t mn) { return (mn + 127u) / 128u * 128u; }
size_t nvfp4_scale_packed_len(uint32_t mn, uint32_t k) {
  return static_cast<size_t>((mn + 127u) / 128u) * (k / 64u) * 512u;
}
uint32_t nvfp4_tensor_amax_chunks(uint64_t n) { return chunks1024(n); }

// ---- amax -------------------------------------------------------------------------------
int nvfp4_row_amax_f32(void* stream, const float* x, float* out, uint32_t rows, uint32_t row_len) {
  return launch_row_amax(S(stream), x, NVFP4_DTYPE_F32, out, rows, row_len);
}
int nvfp4_row_amax_bf16(void* stream, const void* x, float* out, uint32_t rows, uint32_t row_len) {
  return launch_row_amax(S(stream), x, NVFP4_DTYPE_BF16, out, rows, row_len);
}
int nvfp4_tensor_amax_f32(void* stream, const float* x, float* chunk_amax, float* out, uint64_t n) {
  return launch_tensor_amax(S(stream), x, NVFP4_DTYPE_F32, chunk_amax, out, n);
}
int nvfp4_tensor_amax_bf16(void* stream, const void* x, float* chunk_amax, float* out, uint64_t n) {
  return launch_tensor_amax(S(stream), x, NVFP4_DTYPE_BF16, chunk_amax, out, n);
}
int nvfp4_tensor_amax_from_chunks_f32(void* stream, const float* chunk_amax, float* out, uint32_t chunk_count) {
  return launch_amax_from_chunks(S(stream), chunk_amax, out, chunk_count, 0);
}

// ---- four-six ---------------------------------------------------------------------------
int nvfp4_fp32_to_nvfp4_four_six(void* stream, const float* x, const float* amax, uint8_t* out_fp4,
                                 uint8_t* out_scales, float* out_gs, uint32_t group_count) {
  if (group_count > 0x0fffffffu) return invalid("fp32_to_nvfp4_four_six: more than 2^32 - 16 elements in one call");
  return launch_four_six(S(stream), x, NVFP4_DTYPE_F32, amax, 0, 1, group_count * 16u, out_fp4, out_scales, 0, out_gs);
}
int nvfp4_fp32_to_nvfp4_four_six_rowwise(void* stream, const float* x, const float* amax, uint8_t* out_fp4,
                                         uint8_t* out_scales, float* out_gs, uint32_t group_count, uint32_t row_len) {
  if (row_len == 0 || row_len % 16 != 0 || (static_cast<uint64_t>(group_count) * 16) % row_len != 0)
    return invalid("four_six_rowwise: row_len must be a multiple of 16 dividing the element count");
  const uint32_t rows = static_cast<uint32_t>(static_cast<uint64_t>(group_count) * 16 / row_len);
  return launch_four_six(S(stream), x, NVFP4_DTYPE_F32, amax, 1, rows, row_len, out_fp4, out_scales, 0, out_gs);
}
int nvfp4_fp32_to_nvfp4_four_six_padded(void* stream, const float* x, const float* amax, uint8_t* out_fp4,
                                        uint8_t* out_scales, float* out_gs, uint32_t rows, uint32_t cols,
                                        uint32_t padded_rows, uint32_t padded_cols) {
  if (padded_cols % 16 != 0 || padded_rows < rows || padded_cols < cols) return invalid("four_six_padded: bad padding");
  return launch_four_six_padded(S(stream), x, amax, out_fp4, out_scales, out_gs, rows, cols, padded_rows, padded_cols, 0);
}
int nvfp4_fp32_transpose_to_nvfp4_four_six_padded(void* stream, const float* x, const float* amax, uint8_t* out_fp4,
                                                  uint8_t* out_scales, float* out_gs, uint32_t source_rows,
                                                  uint32_t source_cols, uint32_t padded_rows, uint32_t padded_cols) {
  if (padded_cols % 16 != 0 || padded_rows < source_cols || padded_cols < source_rows)
    return invalid("four_six_transpose_padded: bad padding");
  return launch_four_six_padded(S(stream), x, amax, out_fp4, out_scales, out_gs, source_rows, source_cols, padded_rows,
                                padded_cols, 1);
}
int nvfp4_quantize_four_six(void* stream, const void* x, int dtype, const float* amax, int rowwise, uint32_t rows,
                            uint32_t cols, uint8_t* out_fp4, uint8_t* out_scales, int scale_layout, float* out_gs) {
  if (cols % 16 != 0) return invalid("quantize_four_six: cols must be a multiple of 16");
  if (scale_layout == NVFP4_SCALES_PACKED && cols % 64 != 0)
    return invalid("quantize_four_six: the packed scale layout needs cols % 64 == 0");
  if (dtype != NVFP4_DTYPE_F32 && dtype != NVFP4_DTYPE_BF16) return invalid("quantize_four_six: unknown dtype");
  if (reinterpret_cast<uintptr_t>(x) & 15u) return invalid("quantize_four_six: input must be 16-byte aligned");
  return launch_four_six(S(stream), x, dtype, amax, rowwise, rows, cols, out_fp4, out_scales,
                         scale_layout == NVFP4_SCALES_PACKED, out_gs);
}

int nvfp4_quantize_four_six_rowwise_fused(void* stream, const void* x, int dtype, uint32_t rows, uint32_t cols,
                                          uint8_t* out_fp4, uint8_t* out_scales, int scale_layout,
                                          float* out_global_scale, float* out_row_amax,
                                          float* out_decoded_amax) {
  if (cols % 16 != 0) return invalid("quantize_four_six_rowwise_fused: cols must be a multiple of 16");
  if (scale_layout == NVFP4_SCALES_PACKED && cols % 64 != 0)
    return invalid("quantize_four_six_rowwise_fused: the packed scale layout needs cols % 64 == 0");
  if (dtype != NVFP4_DTYPE_F32 && dtype != NVFP4_DTYPE_BF16) return invalid("quantize_four_six_rowwise_fused: dtype");
  if (reinterpret_cast<uintptr_t>(x) & 15u) return invalid("quantize_four_six_rowwise_fused: input must be 16-byte aligned");
  const int packed = scale_layout == NVFP4_SCALES_PACKED;
  int rc = launch_four_six_rowwise_fused(S(stream), x, dtype, rows, cols, out_fp4, out_scales, packed,
                                         out_global_scale, out_row_amax, out_decoded_amax);
  if (rc != -1) return rc;
  // rows too long for one thread block: a row amax pass, then the rowwise quantizer
  if (!out_row_amax) return invalid("quantize_four_six_rowwise_fused: rows longer than 4096 need out_row_amax");
  rc = launch_row_amax(S(stream), x, dtype, out_row_amax, rows, cols);
  if (rc) return rc;
  rc = launch_four_six(S(stream), x, dtype, out_row_amax, 1, rows, cols, out_fp4, out_scales, packed,
                       out_global_scale);
  if (rc || !out_decoded_amax) return rc;
  return launch_nvfp4_amax(S(stream), out_fp4, out_scales, out_global_scale, rows, cols, 1, packed, nullptr,
                           out_decoded_amax);
}

int nvfp4_quantize_relu2_four_six_rowwise(void* stream, const void* pre_activation, int dtype, uint32_t rows,
                                          uint32_t cols, const float* row_amax_in, uint8_t* out_fp4,
                                          uint8_t* out_scales, int scale_layout, float* out_global_scale,
                                          float* out_row_amax, float* out_decoded_amax) {
  if (cols % 16 != 0) return invalid("quantize_relu2_four_six_rowwise: cols must be a multiple of 16");
  if (scale_layout == NVFP4_SCALES_PACKED && cols % 64 != 0)
    return invalid("quantize_relu2_four_six_rowwise: the packed scale layout needs cols % 64 == 0");
  if (dtype != NVFP4_DTYPE_F32 && dtype != NVFP4_DTYPE_BF16) return invalid("quantize_relu2_four_six_rowwise: dtype");
  if (reinterpret_cast<uintptr_t>(pre_activation) & 15u)
    return invalid("quantize_relu2_four_six_rowwise: input must be 16-byte aligned");
  const int packed = scale_layout == NVFP4_SCALES_PACKED;
  if (row_amax_in) {
    // the producer (the GEMM epilogue) already has the row amax of relu(pre)^2: one flat pass, no reduction
    if (out_row_amax && out_row_amax != row_amax_in) {
      const cudaError_t e = cudaMemcpyAsync(out_row_amax, row_amax_in, static_cast<size_t>(rows) * sizeof(float),
                                            cudaMemcpyDeviceToDevice, S(stream));
      if (e != cudaSuccess) return static_cast<int>(e);
    }
    return launch_four_six(S(stream), pre_activation, dtype, row_amax_in, 1, rows, cols, out_fp4, out_scales, packed,
                           out_global_scale, 1, out_decoded_amax);
  }
  int rc = launch_four_six_rowwise_fused(S(stream), pre_activation, dtype, rows, cols, out_fp4, out_scales, packed,
                                         out_global_scale, out_row_amax, out_decoded_amax, 1);
  if (rc != -1) return rc;
  return invalid("quantize_relu2_four_six_rowwise: rows longer than 4096 need row_amax_in");
}

// ---- ReLU^2 backward -------------------------------------------------------------------------
int nvfp4_relu2_backward(void* stream, const float* pre_activation, const float* d_out, float* d_pre_activation,
                         uint32_t len) {
  return launch_relu2_backward(S(stream), pre_activation, 0, d_out, d_pre_activation, 0, len);
}
int nvfp4_relu2_backward_f16(void* stream, const uint16_t* pre_activation, const float* d_out, float* d_pre_activation,
                             uint32_t len) {
  return launch_relu2_backward(S(stream), pre_activation, 2, d_out, d_pre_activation, 0, len);
}
int nvfp4_relu2_backward_bf16(void* stream, const void* pre_activation, const void* d_out, void* d_pre_activation,
                              uint64_t len) {
  return launch_relu2_backward(S(stream), pre_activation, 1, d_out, d_pre_activation, 1, len);
}

uint32_t nvfp4_relu2_backward_amax_chunks(uint64_t len) { return len ? relu2_backward_grid(len) : 0; }
int nvfp4_relu2_backward_amax(void* stream, const void* pre_activation, int pre_kind, const void* d_out,
                              void* d_pre_activation, int grad_dtype, uint64_t len, float* chunk_amax,
                              uint32_t chunk_capacity, uint32_t* out_chunks) {
  if (pre_kind < 0 || pre_kind > 2) return invalid("relu2_backward_amax: pre_kind must be 0 (f32), 1 (bf16) or 2 (f16)");
  if (grad_dtype != NVFP4_DTYPE_F32 && grad_dtype != NVFP4_DTYPE_BF16)
    return invalid("relu2_backward_amax: grad_dtype must be NVFP4_DTYPE_F32 or NVFP4_DTYPE_BF16");
  if (!chunk_amax || !out_chunks) return invalid("relu2_backward_amax: null chunk_amax / out_chunks");
  if (len && (!pre_activation || !d_out || !d_pre_activation)) return invalid("relu2_backward_amax: null pointer");
  const uint32_t chunks = nvfp4_relu2_backward_amax_chunks(len);
  if (chunks > chunk_capacity) return invalid("relu2_backward_amax: chunk_amax holds fewer than the chunks of len");
  *out_chunks = chunks;
  return launch_relu2_backward(S(stream), pre_activation, pre_kind, d_out, d_pre_activation,
                               grad_dtype == NVFP4_DTYPE_BF16, len, chunk_amax);
}

// ---- schedule-free weight materialisation ---------------------------------------------------
int nvfp4_materialize_schedule_free(void* stream, const float* z_master, const float* x_master, float* chunk_amax,
                                    float* amax, uint8_t* bytes, uint8_t* scales, float* global_scale, float beta,
                                    uint32_t len) {
  if (len % 16 != 0) return invalid("materialize_schedule_free: len must be a multiple of 16");
  if (!amax || !bytes || !scales || !global_scale || (len && (!z_master || !x_master)))
    return invalid("materialize_schedule_free: null pointer");
  if ((reinterpret_cast<uintptr_t>(z_master) | reinterpret_cast<uintptr_t>(x_master)) & 15u)
    return invalid("materialize_schedule_free: the masters must be 16-byte aligned");
  return launch_schedule_free_materialize(S(stream), z_master, x_master, beta, chunk_amax, amax, bytes, scales, 0,
                                          global_scale, 1, len);
}
int nvfp4_materialize_schedule_free_matrix(void* stream, const float* z_master, const float* x_master,
                                           float* chunk_amax, float* amax, uint8_t* bytes, uint8_t* scales,
                                           int scale_layout, float* global_scale, float beta, uint32_t rows,
                                           uint32_t cols) {
  if (cols % 16 != 0) return invalid("materialize_schedule_free_matrix: cols must be a multiple of 16");
  if (scale_layout == NVFP4_SCALES_PACKED && cols % 64 != 0)
    return invalid("materialize_schedule_free_matrix: the packed scale layout needs cols % 64 == 0");
  if (!amax || !bytes || !scales || !global_scale || (rows && cols && (!z_master || !x_master)))
    return invalid("materialize_schedule_free_matrix: null pointer");
  if ((reinterpret_cast<uintptr_t>(z_master) | reinterpret_cast<uintptr_t>(x_master)) & 15u)
    return invalid("materialize_schedule_free_matrix: the masters must be 16-byte aligned");
  return launch_schedule_free_materialize(S(stream), z_master, x_master, beta, chunk_amax, amax, bytes, scales,
                                          scale_layout == NVFP4_SCALES_PACKED, global_scale, rows, cols);
}

// ---- MS-EDEN ----------------------------------------------------------------------------
static int validate_ms_eden(const nvfp4_ms_eden_args* a);

int nvfp4_ms_eden_quantize(void* stream, const nvfp4_ms_eden_args* a) {
  int rc = validate_ms_eden(a);
  if (rc) return rc;
  return launch_ms_eden(S(stream), *a);
}

static int validate_ms_eden(const nvfp4_ms_eden_args* a) {
  if (!a) return invalid("ms_eden: null args");
  if (a->dst_row_len % 32 != 0) return invalid("ms_eden: dst_row_len must be a multiple of 32");
  if (a->scale_layout == NVFP4_SCALES_PACKED && a->dst_row_len % 64 != 0)
    return invalid("ms_eden: the packed scale layout needs dst_row_len % 64 == 0");
  if (a->group_offset & 1u) return invalid("ms_eden: group_offset must be even");
  const uint32_t src_len = a->src_kind == NVFP4_SRC_F32_ROWS ? a->cols : a->rows;
  if (src_len > a->dst_row_len) return invalid("ms_eden: source row longer than dst_row_len");
  if (!a->host_global_scale_valid && !a->global_scale) return invalid("ms_eden: no global scale given");
  return 0;
}

// Row operand + transposed operand of one matrix in a single pass (same scale, same signs).
static int ms_eden_pair(void* stream, nvfp4_ms_eden_args rows, nvfp4_ms_eden_args transposed,
                        float* col_sum_partials = nullptr, const float* amax_in = nullptr, float* gs_out = nullptr) {
  rows.src_kind = NVFP4_SRC_F32_ROWS;
  transposed.src_kind = NVFP4_SRC_F32_TRANSPOSED;
  int rc = validate_ms_eden(&rows);
  if (rc) return rc;
  rc = validate_ms_eden(&transposed);
  if (rc) return rc;
  return launch_ms_eden_pair(S(stream), rows, transposed, col_sum_partials, amax_in, gs_out);
}

static nvfp4_ms_eden_args rows_args(const float* x, uint8_t* out_fp4, uint8_t* out_scales, float* out_gss,
                                    float* out_chunk_amax, uint32_t row_count, uint32_t src_row_len,
                                    uint32_t dst_row_len, float so, uint32_t sign_seed, uint32_t scale_seed) {
  nvfp4_ms_eden_args a;
  std::memset(&a, 0, sizeof(a));
  a.src_kind = NVFP4_SRC_F32_ROWS;
  a.src_dtype = NVFP4_DTYPE_F32;
  a.x = x;
  a.rows = row_count;
  a.cols = src_row_len;
  a.dst_row_len = dst_row_len;
  a.scale_override = so;
  a.sign_seed = sign_seed;
  a.scale_seed = scale_seed;
  a.out_fp4 = out_fp4;
  a.out_scales = out_scales;
  a.scale_layout = NVFP4_SCALES_LOGICAL;
  a.out_global_scales = out_gss;
  a.out_chunk_amax = out_chunk_amax;
  return a;
}

int nvfp4_fp32_to_nvfp4_ms_eden(void* stream, const float* x, uint8_t* out_fp4, uint8_t* out_scales,
                                float* out_global_scales, float* out_chunk_amax, uint32_t row_count,
                                uint32_t src_row_len, uint32_t dst_row_len, float global_scale, float scale_override,
                                uint32_t sign_seed, uint32_t scale_seed) {
  nvfp4_ms_eden_args a = rows_args(x, out_fp4, out_scales, out_global_scales, out_chunk_amax, row_count, src_row_len,
                                   dst_row_len, scale_override, sign_seed, scale_seed);
  a.host_global_scale = global_scale;
  a.host_global_scale_valid = 1;
  return nvfp4_ms_eden_quantize(stream, &a);
}
int nvfp4_fp32_to_nvfp4_ms_eden_device_scale(void* stream, const float* x, uint8_t* out_fp4, uint8_t* out_scales,
                                             float* out_global_scales, float* out_chunk_amax,
                                             const float* global_scale, uint32_t row_count, uint32_t src_row_len,
                                             uint32_t dst_row_len, float scale_override, uint32_t sign_seed,
                                             uint32_t scale_seed) {
  nvfp4_ms_eden_args a = rows_args(x, out_fp4, out_scales, out_global_scales, out_chunk_amax, row_count, src_row_len,
                                   dst_row_len, scale_override, sign_seed, scale_seed);
  a.global_scale = global_scale;
  return nvfp4_ms_eden_quantize(stream, &a);
}
int nvfp4_fp32_to_nvfp4_ms_eden_device_scale_no_chunk_amax(void* stream, const float* x, uint8_t* out_fp4,
                                                           uint8_t* out_scales, float* out_global_scales,
                                                           const float* global_scale, uint32_t row_count,
                                                           uint32_t src_row_len, uint32_t dst_row_len,
                                                           float scale_override, uint32_t sign_seed,
                                                           uint32_t scale_seed) {
  return nvfp4_fp32_to_nvfp4_ms_eden_device_scale(stream, x, out_fp4, out_scales, out_global_scales, nullptr,
                                                  global_scale, row_count, src_row_len, dst_row_len, scale_override,
                                                  sign_seed, scale_seed);
}
int nvfp4_fp32_transpose_to_nvfp4_ms_eden_device_scale(void* stream, const float* x, uint8_t* out_fp4,
                                                       uint8_t* out_scales, float* out_global_scales,
                                                       float* out_chunk_amax, const float* global_scale,
                                                       uint32_t source_rows, uint32_t source_cols,
                                                       uint32_t dst_row_len, float scale_override, uint32_t sign_seed,
                                                       uint32_t scale_seed) {
  nvfp4_ms_eden_args a = rows_args(x, out_fp4, out_scales, out_global_scales, out_chunk_amax, source_rows, source_cols,
                                   dst_row_len, scale_override, sign_seed, scale_seed);
  a.src_kind = NVFP4_SRC_F32_TRANSPOSED;
  a.global_scale = global_scale;
  return nvfp4_ms_eden_quantize(stream, &a);
}
int nvfp4_fp32_transpose_to_nvfp4_ms_eden_device_scale_no_chunk_amax(
    void* stream, const float* x, uint8_t* out_fp4, uint8_t* out_scales, float* out_global_scales,
    const float* global_scale, uint32_t source_rows, uint32_t source_cols, uint32_t dst_row_len, float scale_override,
    uint32_t sign_seed, uint32_t scale_seed) {
  return nvfp4_fp32_transpose_to_nvfp4_ms_eden_device_scale(stream, x, out_fp4, out_scales, out_global_scales, nullptr,
                                                            global_scale, source_rows, source_cols, dst_row_len,
                                                            scale_override, sign_seed, scale_seed);
}
int nvfp4_quartet_backward_ms_eden_global_scale_from_chunks(void* stream, const float* chunk_amax,
                                                            float* out_global_scale, uint32_t chunk_count) {
  return launch_amax_from_chunks(S(stream), chunk_amax, out_global_scale, chunk_count, 1);
}

// tensor chunk amax -> global scale -> rows.  The chunk-amax buffer first receives the
// 1024-value chunk maxima and, in the first form, is then overwritten by the 32-chunk maxima
// (utils/nvfp4/quant/global_scale.rs:76-93 followed by ms_eden.rs:35-60).
static int quartet_derived(void* stream, const float* x, uint8_t* out_fp4, uint8_t* out_scales, float* out_gss,
                           float* out_chunk_amax, float* out_gs, uint32_t row_count, uint32_t src_row_len,
                           uint32_t dst_row_len, uint32_t sign_seed, uint32_t scale_seed, bool chunk_amax_out) {
  const uint64_t n = static_cast<uint64_t>(row_count) * src_row_len;
  int rc = launch_tensor_amax(S(stream), x, NVFP4_DTYPE_F32, out_chunk_amax, out_gs, n);
  if (rc) return rc;
  rc = launch_amax_from_chunks(S(stream), out_chunk_amax, out_gs, chunks1024(n), 1);
  if (rc) return rc;
  return nvfp4_fp32_to_nvfp4_ms_eden_device_scale(stream, x, out_fp4, out_scales, out_gss,
                                                  chunk_amax_out ? out_chunk_amax : nullptr, out_gs, row_count,
                                                  src_row_len, dst_row_len, kQuartetSO, sign_seed, scale_seed);
}
int nvfp4_fp32_to_nvfp4_quartet_backward_ms_eden_derived_device_scale(
    void* stream, const float* x, uint8_t* out_fp4, uint8_t* out_scales, float* out_global_scales,
    float* out_chunk_amax, float* out_global_scale, uint32_t row_count, uint32_t src_row_len, uint32_t dst_row_len,
    uint32_t sign_seed, uint32_t scale_seed) {
  return quartet_derived(stream, x, out_fp4, out_scales, out_global_scales, out_chunk_amax, out_global_scale, row_count,
                         src_row_len, dst_row_len, sign_seed, scale_seed, true);
}
int nvfp4_fp32_to_nvfp4_quartet_backward_ms_eden_derived_device_scale_no_chunk_amax(
    void* stream, const float* x, uint8_t* out_fp4, uint8_t* out_scales, float* out_global_scales,
    float* out_chunk_amax, float* out_global_scale, uint32_t row_count, uint32_t src_row_len, uint32_t dst_row_len,
    uint32_t sign_seed, uint32_t scale_seed) {
  return quartet_derived(stream, x, out_fp4, out_scales, out_global_scales, out_chunk_amax, out_global_scale, row_count,
                         src_row_len, dst_row_len, sign_seed, scale_seed, false);
}
int nvfp4_fp32_to_nvfp4_quartet_backward_ms_eden_with_global_scale(
    void* stream, const float* x, uint8_t* out_fp4, uint8_t* out_scales, float* out_global_scales,
    float* out_chunk_amax, uint32_t row_count, uint32_t src_row_len, uint32_t dst_row_len, uint32_t sign_seed,
    uint32_t scale_seed, float global_scale) {
  return nvfp4_fp32_to_nvfp4_ms_eden(stream, x, out_fp4, out_scales, out_global_scales, out_chunk_amax, row_count,
                                     src_row_len, dst_row_len, global_scale, kQuartetSO, sign_seed, scale_seed);
}

int nvfp4_fp32_pair_to_nvfp4_quartet_backward_ms_eden_derived_device_scale_no_chunk_amax(
    void* stream, const float* x, uint8_t* out_fp4, uint8_t* out_scales, float* out_global_scales,
    uint8_t* transpose_out_fp4, uint8_t* transpose_out_scales, float* transpose_out_global_scales,
    float* out_chunk_amax, float* out_global_scale, uint32_t row_count, uint32_t src_row_len, uint32_t dst_row_len,
    uint32_t transpose_dst_row_len, uint32_t sign_seed, uint32_t scale_seed, uint32_t transpose_scale_seed,
    uint32_t precomputed_chunk_count) {
  const uint64_t n = static_cast<uint64_t>(row_count) * src_row_len;
  uint32_t chunk_count = precomputed_chunk_count;
  int rc;
  if (chunk_count == 0) {
    rc = launch_tensor_amax(S(stream), x, NVFP4_DTYPE_F32, out_chunk_amax, out_global_scale, n);
    if (rc) return rc;
    chunk_count = chunks1024(n);
  }
  rc = launch_amax_from_chunks(S(stream), out_chunk_amax, out_global_scale, chunk_count, 1);
  if (rc) return rc;
  nvfp4_ms_eden_args r = rows_args(x, out_fp4, out_scales, out_global_scales, nullptr, row_count, src_row_len,
                                   dst_row_len, kQuartetSO, sign_seed, scale_seed);
  r.global_scale = out_global_scale;
  nvfp4_ms_eden_args t = rows_args(x, transpose_out_fp4, transpose_out_scales, transpose_out_global_scales, nullptr,
                                   row_count, src_row_len, transpose_dst_row_len, kQuartetSO, sign_seed,
                                   transpose_scale_seed);
  t.global_scale = out_global_scale;
  return ms_eden_pair(stream, r, t);
}

static int nvfp4_source_transpose(void* stream, int kind, const uint8_t* in_bytes, const uint8_t* in_scales,
                                  const float* in_global, uint8_t* out_fp4, uint8_t* out_scales, float* out_gss,
                                  float* out_chunk_amax, float* out_gs, uint32_t source_rows, uint32_t source_cols,
                                  uint32_t dst_row_len, uint32_t sign_seed, uint32_t scale_seed, bool chunk_amax_out,
                                  int scale_layout, uint32_t col_offset, uint32_t group_offset,
                                  int src_scale_layout = NVFP4_SCALES_LOGICAL,
                                  const float* precomputed_amax = nullptr, uint32_t group_row_stride = 0) {
  const uint64_t n = static_cast<uint64_t>(source_rows) * source_cols;
  if (source_cols % 16 != 0) return invalid("nvfp4 transpose: source_cols must be a multiple of 16");
  if (src_scale_layout == NVFP4_SCALES_PACKED && source_cols % 64 != 0)
    return invalid("nvfp4 transpose: a packed source scale layout needs source_cols % 64 == 0");
  // The amax of the decoded source, unless the caller already holds it (the forward quantizer can emit it).
  // When the chunk scratch is free (no chunk amax asked for) the amax accumulates in its word 0, away from
  // out_gs, so that the transposer can derive the scale from it by itself.
  int rc = 0;
  const bool amax_in_scratch = !precomputed_amax && !chunk_amax_out && out_chunk_amax != nullptr;
  if (!precomputed_amax)
    rc = launch_nvfp4_amax(S(stream), in_bytes, in_scales, in_global, source_rows, source_cols,
                           kind == NVFP4_SRC_ROWWISE_NVFP4_TRANSPOSED, src_scale_layout == NVFP4_SCALES_PACKED,
                           amax_in_scratch ? nullptr : out_chunk_amax, amax_in_scratch ? out_chunk_amax : out_gs);
  if (rc) return rc;
  (void)n;
  nvfp4_ms_eden_args a;
  std::memset(&a, 0, sizeof(a));
  a.src_kind = kind;
  a.src_bytes = in_bytes;
  a.src_scales = in_scales;
  a.src_scale_layout = src_scale_layout;
  a.src_global = in_global;
  a.rows = source_rows;
  a.cols = source_cols;
  a.dst_row_len = dst_row_len;
  a.global_scale = out_gs;
  a.scale_override = kQuartetSO;
  a.sign_seed = sign_seed;
  a.scale_seed = scale_seed;
  a.col_offset = col_offset;
  a.group_offset = group_offset;
  a.group_row_stride = group_row_stride;
  a.out_fp4 = out_fp4;
  a.out_scales = out_scales;
  a.scale_layout = scale_layout;
  a.out_global_scales = out_gss;
  a.out_chunk_amax = chunk_amax_out ? out_chunk_amax : nullptr;
  rc = validate_ms_eden(&a);
  if (rc) return rc;
  // amax -> global scale inside the transposer where it can (whole tiles), by a one-thread kernel otherwise;
  // out_gs receives the scale either way
  const float* amax_ptr = precomputed_amax ? precomputed_amax : (amax_in_scratch ? out_chunk_amax : out_gs);
  if (amax_ptr == out_gs) {
    // the amax sits where the scale will go: deriving it inside the kernel would race across CTAs
    rc = launch_ms_eden_scale_from_amax(S(stream), out_gs, out_gs);
    return rc ? rc : launch_ms_eden(S(stream), a);
  }
  return launch_ms_eden(S(stream), a, amax_ptr, out_gs);
}

int nvfp4_nvfp4_transpose_to_quartet_backward_ms_eden_derived_device_scale(
    void* stream, const uint8_t* in_bytes, const uint8_t* in_scales, const float* in_global_scale, uint8_t* out_fp4,
    uint8_t* out_scales, float* out_global_scales, float* out_chunk_amax, float* out_global_scale,
    uint32_t source_rows, uint32_t source_cols, uint32_t dst_row_len, uint32_t sign_seed, uint32_t scale_seed) {
  return nvfp4_source_transpose(stream, NVFP4_SRC_NVFP4_TRANSPOSED, in_bytes, in_scales, in_global_scale, out_fp4,
                                out_scales, out_global_scales, out_chunk_amax, out_global_scale, source_rows,
                                source_cols, dst_row_len, sign_seed, scale_seed, true, NVFP4_SCALES_LOGICAL, 0, 0);
}
int nvfp4_nvfp4_transpose_to_quartet_backward_ms_eden_derived_device_scale_no_chunk_amax(
    void* stream, const uint8_t* in_bytes, const uint8_t* in_scales, const float* in_global_scale, uint8_t* out_fp4,
    uint8_t* out_scales, float* out_global_scales, float* out_chunk_amax, float* out_global_scale,
    uint32_t source_rows, uint32_t source_cols, uint32_t dst_row_len, uint32_t sign_seed, uint32_t scale_seed) {
  return nvfp4_source_transpose(stream, NVFP4_SRC_NVFP4_TRANSPOSED, in_bytes, in_scales, in_global_scale, out_fp4,
                                out_scales, out_global_scales, out_chunk_amax, out_global_scale, source_rows,
                                source_cols, dst_row_len, sign_seed, scale_seed, false, NVFP4_SCALES_LOGICAL, 0, 0);
}
int nvfp4_rowwise_nvfp4_transpose_to_quartet_backward_ms_eden_derived_device_scale(
    void* stream, const uint8_t* in_bytes, const uint8_t* in_scales, const float* in_global_scales, uint8_t* out_fp4,
    uint8_t* out_scales, float* out_global_scales, float* out_chunk_amax, float* out_global_scale,
    uint32_t source_rows, uint32_t source_cols, uint32_t dst_row_len, uint32_t sign_seed, uint32_t scale_seed) {
  return nvfp4_source_transpose(stream, NVFP4_SRC_ROWWISE_NVFP4_TRANSPOSED, in_bytes, in_scales, in_global_scales,
                                out_fp4, out_scales, out_global_scales, out_chunk_amax, out_global_scale, source_rows,
                                source_cols, dst_row_len, sign_seed, scale_seed, true, NVFP4_SCALES_LOGICAL, 0, 0);
}
int nvfp4_rowwise_nvfp4_transpose_to_quartet_backward_ms_eden_derived_device_scale_no_chunk_amax(
    void* stream, const uint8_t* in_bytes, const uint8_t* in_scales, const float* in_global_scales, uint8_t* out_fp4,
    uint8_t* out_scales, float* out_global_scales, float* out_chunk_amax, float* out_global_scale,
    uint32_t source_rows, uint32_t source_cols, uint32_t dst_row_len, uint32_t sign_seed, uint32_t scale_seed) {
  return nvfp4_source_transpose(stream, NVFP4_SRC_ROWWISE_NVFP4_TRANSPOSED, in_bytes, in_scales, in_global_scales,
                                out_fp4, out_scales, out_global_scales, out_chunk_amax, out_global_scale, source_rows,
                                source_cols, dst_row_len, sign_seed, scale_seed, false, NVFP4_SCALES_LOGICAL, 0, 0);
}

// ---- decode / layout --------------------------------------------------------------------
int nvfp4_decode_transpose_f32(void* stream, const uint8_t* bytes, const uint8_t* scales, const float* global_scale,
                               float* output, uint32_t rows, uint32_t cols) {
  return launch_decode(S(stream), bytes, scales, global_scale, 0, 1, output, rows, cols);
}
int nvfp4_decode_rowwise_transpose_f32(void* stream, const uint8_t* bytes, const uint8_t* scales,
                                       const float* global_scales, float* output, uint32_t rows, uint32_t cols) {
  return launch_decode(S(stream), bytes, scales, global_scales, 1, 1, output, rows, cols);
}
int nvfp4_decode_f32(void* stream, const uint8_t* bytes, const uint8_t* scales, const float* global_scales,
                     int rowwise, float* output, uint32_t rows, uint32_t cols) {
  return launch_decode(S(stream), bytes, scales, global_scales, rowwise, 0, output, rows, cols);
}
int nvfp4_scale_pack(void* stream, const uint8_t* logical, uint8_t* packed, uint32_t mn_extent, uint32_t k_dim) {
  if (k_dim % 64 != 0) return invalid("scale_pack: k_dim must be a multiple of 64");
  return launch_scale_pack(S(stream), logical, packed, mn_extent, k_dim);
}
int nvfp4_pad_u4_rows(void* stream, const uint8_t* src, uint8_t* dst, uint32_t rows, uint32_t padded_rows,
                      uint32_t cols) {
  if (padded_rows < rows || cols % 2 != 0) return invalid("pad_u4_rows: bad shape");
  return launch_pad_u4_rows(S(stream), src, dst, rows, padded_rows, cols);
}
int nvfp4_pad_f32(void* stream, const float* src, float* dst, uint32_t rows, uint32_t cols, uint32_t padded_rows,
                  uint32_t padded_cols) {
  if (padded_rows < rows || padded_cols < cols) return invalid("pad_f32: bad shape");
  return launch_pad_f32(S(stream), src, dst, rows, cols, padded_rows, padded_cols, 0);
}
int nvfp4_transpose_pad_f32(void* stream, const float* src, float* dst, uint32_t rows, uint32_t cols,
                            uint32_t padded_rows, uint32_t padded_cols) {
  if (padded_rows < cols || padded_cols < rows) return invalid("transpose_pad_f32: bad shape");
  return launch_pad_f32(S(stream), src, dst, rows, cols, padded_rows, padded_cols, 1);
}
int nvfp4_crop_f32(void* stream, const float* src, float* dst, uint32_t rows, uint32_t src_cols, uint32_t dst_cols) {
  if (dst_cols > src_cols) return invalid("crop_f32: dst_cols > src_cols");
  return launch_crop_f32(S(stream), src, dst, rows, src_cols, dst_cols);
}

// ---- GEMM -------------------------------------------------------------------------------
int nvfp4_gemm(void* stream, const nvfp4_gemm_args* args) {
  if (!args) return invalid("nvfp4_gemm: null args");
  return launch_gemm(S(stream), *args);
}

int nvfp4_gemm_plan_query(const nvfp4_gemm_args* args, nvfp4_gemm_plan* out) {
  if (!args || !out) return invalid("nvfp4_gemm_plan_query: null pointer");
  return gemm_plan_query(*args, out);
}
int nvfp4_prepare_tma_nvfp4_device_scales_into(void* stream, const uint8_t* input_bytes,
                                               const uint8_t* input_scale_data, const uint8_t* weight_bytes,
                                               const uint8_t* weight_scale_data, uint32_t token_count,
                                               uint32_t input_dim, uint32_t output_dim, void* descriptors) {
  (void)stream;
  (void)descriptors;  // tensor maps travel as kernel parameters; the device copies of the reference are not needed
  if (!input_bytes || !weight_bytes || !input_scale_data || !weight_scale_data)
    return invalid("prepare_tma_nvfp4_device_scales: null operand");
  if ((reinterpret_cast<uintptr_t>(input_bytes) | reinterpret_cast<uintptr_t>(weight_bytes) |
       reinterpret_cast<uintptr_t>(input_scale_data) | reinterpret_cast<uintptr_t>(weight_scale_data)) & 15u)
    return invalid("prepare_tma_nvfp4_device_scales: operand and scale pointers must be 16-byte aligned");
  if (token_count == 0 || output_dim == 0) return 0;
  return gemm_prepare_operand_maps(input_bytes, weight_bytes, token_count, input_dim, output_dim);
}
int nvfp4_prepare_tma_nvfp4_device_scales(void* stream, const uint8_t* input_bytes, const uint8_t* input_scale_data,
                                          const uint8_t* weight_bytes, const uint8_t* weight_scale_data,
                                          uint32_t token_count, uint32_t input_dim, uint32_t output_dim) {
  return nvfp4_prepare_tma_nvfp4_device_scales_into(stream, input_bytes, input_scale_data, weight_bytes,
                                                    weight_scale_data, token_count, input_dim, output_dim, nullptr);
}
int nvfp4_tensor_map_cache_stats(uint64_t* hits, uint64_t* misses) {
  gemm_map_cache_stats(hits, misses);
  return 0;
}
int nvfp4_gemm_set_tile_override(int block_m, int block_n) {
  const bool ok = block_n == 0 || (block_m == 128 && (block_n == 128 || block_n == 192 || block_n == 256)) ||
                  (block_m == 256 && block_n == 192);
  if (!ok) return invalid("gemm_set_tile_override: 128 x {128, 192, 256}, 256 x 192, or block_n = 0 for automatic");
  gemm_set_tile_override(block_m, block_n);
  return 0;
}
int nvfp4_gemm_set_wait_timeout_ns(uint64_t ns) {
  gemm_set_wait_timeout_ns(ns);
  return 0;
}
int nvfp4_gemm_set_debug_flags(uint32_t flags) {
  gemm_set_debug_flags(flags);
  return 0;
}

// ---- forward projections (reference argument lists) ------------------------------------------
// Packed scale plane of an operand: the caller's plane if it is packed already, else packed into the scratch.
static int packed_plane(void* stream, const uint8_t* scales, int layout, uint8_t* scratch, uint32_t rows, uint32_t k,
                        const uint8_t** out, const char* who) {
  if (layout == NVFP4_SCALES_PACKED) {
    *out = scales;
    return 0;
  }
  if (layout != NVFP4_SCALES_LOGICAL) return invalid("unknown scale layout");
  if (!scratch) {
    set_last_error(who);
    return static_cast<int>(cudaErrorInvalidValue);
  }
  *out = scratch;
  return launch_scale_pack(S(stream), scales, scratch, rows, k);
}

enum ProjectionKind { kProjPlain, kProjResidual, kProjRelu2, kProjLogits };

static int projection(void* stream, const nvfp4_projection_args* a, ProjectionKind kind) {
  if (!a) return invalid("projection: null args");
  if (a->token_count == 0 || a->output_dim == 0) return 0;
  if (a->input_dim == 0 || a->input_dim % 64 != 0) return invalid("projection: input_dim must be a non-zero multiple of 64");
  if (!a->input_bytes || !a->input_scales || !a->input_global_scales || !a->weight_bytes || !a->weight_scales ||
      !a->weight_global_scale)
    return invalid("projection: null operand");
  const bool has_bias = a->bias_bytes && a->bias_scales && a->bias_global_scale;
  if (kind != kProjLogits && !has_bias) return invalid("projection: this method takes an NVFP4 bias");
  if (kind == kProjResidual && a->out_dtype != NVFP4_DTYPE_F32) return invalid("projection: the residual stream is f32");
  if (kind == kProjRelu2 ? (!a->pre_activation && !a->out) : !a->out) return invalid("projection: null output");
  const uint8_t *xs = nullptr, *ws = nullptr;
  int rc = packed_plane(stream, a->input_scales, a->input_scale_layout, a->input_scales_packed_scratch, a->token_count,
                        a->input_dim, &xs, "projection: logical input scales need input_scales_packed_scratch");
  if (rc) return rc;
  rc = packed_plane(stream, a->weight_scales, a->weight_scale_layout, a->weight_scales_packed_scratch, a->output_dim,
                    a->input_dim, &ws, "projection: logical weight scales need weight_scales_packed_scratch");
  if (rc) return rc;
  nvfp4_gemm_args g;
  std::memset(&g, 0, sizeof(g));
  g.a_bytes = a->input_bytes;
  g.a_scales = xs;
  g.a_global = a->input_global_scales;
  g.b_bytes = a->weight_bytes;
  g.b_scales = ws;
  g.b_global = a->weight_global_scale;
  g.m = a->token_count;
  g.n = a->output_dim;
  g.k = a->input_dim;
  g.ldo = a->output_dim;
  g.global_scale_mode = NVFP4_GS_ROWWISE_A;
  g.weight_global_scale = 1.0f;
  g.out_dtype = a->out_dtype;
  g.out = a->out;
  if (has_bias) {
    g.bias_nvfp4_bytes = a->bias_bytes;
    g.bias_nvfp4_scales = a->bias_scales;
    g.bias_nvfp4_global = a->bias_global_scale;
  }
  switch (kind) {
    case kProjPlain:
      g.epilogue = NVFP4_EPI_BIAS;
      break;
    case kProjResidual:
      g.epilogue = NVFP4_EPI_RESIDUAL;
      break;
    case kProjLogits:
      g.epilogue = has_bias ? NVFP4_EPI_BIAS : NVFP4_EPI_NONE;
      break;
    case kProjRelu2:
      if (a->out) {
        g.epilogue = NVFP4_EPI_RELU2;
        g.aux = a->pre_activation;
      } else {  // only the pre-activation is kept: a plain biased projection into it
        g.epilogue = NVFP4_EPI_BIAS;
        g.out = a->pre_activation;
      }
      g.relu2_row_amax = a->relu2_row_amax;
      break;
  }
  return launch_gemm(S(stream), g);
}

int nvfp4_qkv_projection(void* stream, const nvfp4_projection_args* a) { return projection(stream, a, kProjPlain); }
int nvfp4_c_proj(void* stream, const nvfp4_projection_args* a) {
  if (a && a->input_dim != a->output_dim) return invalid("c_proj: output_dim must equal input_dim (embedding_dim)");
  return projection(stream, a, kProjResidual);
}
int nvfp4_mlp_up_relu2(void* stream, const nvfp4_projection_args* a) { return projection(stream, a, kProjRelu2); }
int nvfp4_mlp_down_residual(void* stream, const nvfp4_projection_args* a) { return projection(stream, a, kProjResidual); }
int nvfp4_lm_head_logits(void* stream, const nvfp4_projection_args* a) { return projection(stream, a, kProjLogits); }
int nvfp4_lm_head_logits_tma(void* stream, const nvfp4_projection_args* a) { return projection(stream, a, kProjLogits); }
int nvfp4_nextlat_projection(void* stream, const nvfp4_projection_args* a) { return projection(stream, a, kProjPlain); }

static int gemm_plain(void* stream, const uint8_t* a_bytes, const uint8_t* a_scales, const uint8_t* b_bytes,
                      const uint8_t* b_scales, float* out, uint32_t m, uint32_t k, uint32_t n, uint32_t ldo, int mode,
                      const float* ag, const float* bg) {
  nvfp4_gemm_args g;
  std::memset(&g, 0, sizeof(g));
  g.a_bytes = a_bytes;
  g.a_scales = a_scales;
  g.a_global = ag;
  g.b_bytes = b_bytes;
  g.b_scales = b_scales;
  g.b_global = bg;
  g.out = out;
  g.m = m;
  g.n = n;
  g.k = k;
  g.ldo = ldo;
  g.global_scale_mode = mode;
  g.weight_global_scale = 1.0f;
  g.epilogue = NVFP4_EPI_NONE;
  g.out_dtype = NVFP4_DTYPE_F32;
  return launch_gemm(S(stream), g);
}
int nvfp4_gemm_tma_nvfp4_device_scales_and_global_scale_buffers(
    void* stream, const uint8_t* a_bytes, const uint8_t* a_scales_packed, const uint8_t* b_bytes,
    const uint8_t* b_scales_packed, float* out, uint32_t token_count, uint32_t input_dim, uint32_t output_dim,
    const float* a_global_scale, const float* b_global_scale) {
  return gemm_plain(stream, a_bytes, a_scales_packed, b_bytes, b_scales_packed, out, token_count, input_dim,
                    output_dim, output_dim, NVFP4_GS_TENSOR, a_global_scale, b_global_scale);
}
int nvfp4_gemm_tma_nvfp4_rowwise_a_scale_and_global_scale_buffer(
    void* stream, const uint8_t* a_bytes, const uint8_t* a_scales_packed, const uint8_t* b_bytes,
    const uint8_t* b_scales_packed, float* out, uint32_t token_count, uint32_t input_dim, uint32_t output_dim,
    const float* a_global_scales, const float* b_global_scale) {
  return gemm_plain(stream, a_bytes, a_scales_packed, b_bytes, b_scales_packed, out, token_count, input_dim,
                    output_dim, output_dim, NVFP4_GS_ROWWISE_A, a_global_scales, b_global_scale);
}
int nvfp4_gemm_tma_nvfp4_rowwise_a_scale_padded_output(
    void* stream, const uint8_t* a_bytes, const uint8_t* a_scales_packed, const uint8_t* b_bytes,
    const uint8_t* b_scales_packed, float* out, uint32_t token_count, uint32_t input_dim, uint32_t output_dim,
    uint32_t padded_output_dim, const float* a_global_scales, const float* b_global_scale) {
  if (output_dim > padded_output_dim) return invalid("gemm padded_output: output_dim > padded_output_dim");
  // Only output_dim columns exist in `out`; the pad rows of B are simply never stored.
  return gemm_plain(stream, a_bytes, a_scales_packed, b_bytes, b_scales_packed, out, token_count, input_dim,
                    output_dim, output_dim, NVFP4_GS_ROWWISE_A, a_global_scales, b_global_scale);
}

int nvfp4_set_deterministic_reductions(int on) {
  gemm_set_deterministic(on);
  return 0;
}
int nvfp4_get_deterministic_reductions(void) { return gemm_get_deterministic(); }
int nvfp4_gemm_timing_begin(uint32_t max_records) { return gemm_timing_begin(max_records); }
int nvfp4_gemm_timing_end(uint32_t* count, double* total_ms, double* total_flops, float* per_launch_ms,
                          double* per_launch_flops, uint32_t capacity) {
  return gemm_timing_end(count, total_ms, total_flops, per_launch_ms, per_launch_flops, capacity);
}

// ---- post-ops ---------------------------------------------------------------------------
int nvfp4_projection_bias_inplace(void* stream, float* raw, const uint8_t* bias_bytes, const uint8_t* bias_scales,
                                  const float* bias_gs, uint32_t rows, uint32_t cols) {
  return launch_postop(S(stream), raw, nullptr, bias_bytes, bias_scales, bias_gs, rows, cols, 0);
}
int nvfp4_projection_residual_add(void* stream, const float* raw, const uint8_t* bias_bytes,
                                  const uint8_t* bias_scales, const float* bias_gs, float* residual, uint32_t rows,
                                  uint32_t cols) {
  return launch_postop(S(stream), const_cast<float*>(raw), residual, bias_bytes, bias_scales, bias_gs, rows, cols, 1);
}
int nvfp4_projection_relu2_inplace(void* stream, float* pre_activation, float* out, const uint8_t* bias_bytes,
                                   const uint8_t* bias_scales, const float* bias_gs, uint32_t rows, uint32_t cols) {
  return launch_postop(S(stream), pre_activation, out, bias_bytes, bias_scales, bias_gs, rows, cols, 2);
}

// ---- linear backward --------------------------------------------------------------------
int nvfp4_linear_bias_grad(void* stream, const float* e, float* dbias, uint32_t token_count, uint32_t output_dim) {
  return launch_bias_grad(S(stream), e, NVFP4_DTYPE_F32, dbias, token_count, output_dim);
}
int nvfp4_linear_bias_grad_bf16(void* stream, const void* e, float* dbias, uint32_t token_count, uint32_t output_dim) {
  return launch_bias_grad(S(stream), e, NVFP4_DTYPE_BF16, dbias, token_count, output_dim);
}

// ---- generic MS-EDEN matmul ---------------------------------------------------------------------
int nvfp4_tc_matmul_ms_eden(void* stream, const float* a, const float* b_t, float* out,
                            const nvfp4_ms_eden_operand* a_q, float a_global_scale,
                            const nvfp4_ms_eden_operand* b_q, float b_global_scale, uint32_t m, uint32_t n, uint32_t k,
                            uint32_t sign_seed, uint32_t scale_seed) {
  if (!a_q || !b_q || !out || (m && k && !a) || (n && k && !b_t)) return invalid("tc_matmul_ms_eden: null pointer");
  if (m == 0 || n == 0) return 0;
  if (k == 0) return invalid("tc_matmul_ms_eden: k must be non-zero");
  const uint32_t pk = padded_k(k);
  // both operands: MS-EDEN rows with the caller's global scale, K zero-padded to a multiple of 64 on the
  // fly (utils/nvfp4_tc_matmul/{launcher.rs:23-69,quantize.rs:6-32}; no padded f32 copies are made)
  nvfp4_ms_eden_args qa = rows_args(a, a_q->bytes, a_q->scales_packed, a_q->global_scales, a_q->chunk_amax, m, k, pk,
                                    kQuartetSO, sign_seed, scale_seed);
  qa.scale_layout = NVFP4_SCALES_PACKED;
  qa.host_global_scale = a_global_scale;
  qa.host_global_scale_valid = 1;
  int rc = nvfp4_ms_eden_quantize(stream, &qa);
  if (rc) return rc;
  nvfp4_ms_eden_args qb = rows_args(b_t, b_q->bytes, b_q->scales_packed, b_q->global_scales, b_q->chunk_amax, n, k, pk,
                                    kQuartetSO, sign_seed, scale_seed ^ 0x9e3779b9u);
  qb.scale_layout = NVFP4_SCALES_PACKED;
  qb.host_global_scale = b_global_scale;
  qb.host_global_scale_valid = 1;
  rc = nvfp4_ms_eden_quantize(stream, &qb);
  if (rc) return rc;
  // out = acc * a_scale[row] * b_scale (launcher.rs:71-86); every row of b carries the same scale
  nvfp4_gemm_args g;
  std::memset(&g, 0, sizeof(g));
  g.a_bytes = a_q->bytes;
  g.a_scales = a_q->scales_packed;
  g.a_global = a_q->global_scales;
  g.b_bytes = b_q->bytes;
  g.b_scales = b_q->scales_packed;
  g.b_global = b_q->global_scales;
  g.out = out;
  g.m = m;
  g.n = n;
  g.k = pk;
  g.ldo = n;
  g.global_scale_mode = NVFP4_GS_ROWWISE_A;
  g.weight_global_scale = 1.0f;
  g.epilogue = NVFP4_EPI_NONE;
  g.out_dtype = NVFP4_DTYPE_F32;
  return nvfp4_gemm(stream, &g);
}

// The gradient GEMMs over quantized operands: dX = e_h . weight_t_h^T, dW = e_t_h . input_t_h^T.
static int backward_gemms(cudaStream_t s, const uint8_t* eh_b, const uint8_t* eh_s, const float* eh_g,
                          const uint8_t* wt_b, const uint8_t* wt_s, const float* wt_g, const uint8_t* et_b,
                          const uint8_t* et_s, const float* et_g, const uint8_t* xt_b, const uint8_t* xt_s,
                          const float* xt_g, void* dinput, int dinput_dtype, void* dweight, int dweight_dtype,
                          uint32_t T, uint32_t I, uint32_t O) {
  const uint32_t ok = padded_k(O), tk = padded_k(T);
  nvfp4_gemm_args g;
  std::memset(&g, 0, sizeof(g));
  g.global_scale_mode = NVFP4_GS_ROWWISE_A;
  g.weight_global_scale = 1.0f;
  g.epilogue = NVFP4_EPI_NONE;
  g.out_dtype = dinput_dtype;
  g.a_bytes = eh_b;
  g.a_scales = eh_s;
  g.a_global = eh_g;
  g.b_bytes = wt_b;
  g.b_scales = wt_s;
  g.b_global = wt_g;
  g.out = dinput;
  g.m = T;
  g.n = I;
  g.k = ok;
  g.ldo = I;
  int rc = launch_gemm(s, g);
  if (rc) return rc;
  g.a_bytes = et_b;
  g.a_scales = et_s;
  g.a_global = et_g;
  g.b_bytes = xt_b;
  g.b_scales = xt_s;
  g.b_global = xt_g;
  g.out = dweight;
  g.out_dtype = dweight_dtype;
  g.m = O;
  g.n = I;
  g.k = tk;
  return launch_gemm(s, g);
}

static int backward_device_scale(void* stream, const nvfp4_linear_backward_device_scale_args* a) {
  if (!a) return invalid("backward_device_scale: null args");
  const uint32_t T = a->token_count, I = a->input_dim, O = a->output_dim;
  if (T == 0 || I == 0 || O == 0) return 0;
  if (!a->dinput || !a->dweight) return invalid("backward_device_scale: null gradient buffer");
  const uint32_t ok = padded_k(O), tk = padded_k(T);
  const nvfp4_backward_operand* ops[4] = {&a->e_h, &a->weight_t_h, &a->e_t_h, &a->input_t_h};
  const uint32_t rows[4] = {T, I, O, I}, ks[4] = {ok, ok, tk, tk};
  const uint8_t* planes[4];
  for (int i = 0; i < 4; ++i) {
    if (!ops[i]->bytes || !ops[i]->scales || !ops[i]->global_scales) return invalid("backward_device_scale: null operand");
    const int rc = packed_plane(stream, ops[i]->scales, ops[i]->scale_layout, ops[i]->scales_packed_scratch, rows[i],
                                ks[i], &planes[i], "backward_device_scale: logical scales need scales_packed_scratch");
    if (rc) return rc;
  }
  return backward_gemms(S(stream), a->e_h.bytes, planes[0], a->e_h.global_scales, a->weight_t_h.bytes, planes[1],
                        a->weight_t_h.global_scales, a->e_t_h.bytes, planes[2], a->e_t_h.global_scales,
                        a->input_t_h.bytes, planes[3], a->input_t_h.global_scales, a->dinput, a->dinput_dtype,
                        a->dweight, a->dweight_dtype, T, I, O);
}
int nvfp4_linear_backward_device_scale_tma(void* stream, const nvfp4_linear_backward_device_scale_args* a) {
  return backward_device_scale(stream, a);
}
int nvfp4_linear_backward_device_scale(void* stream, const nvfp4_linear_backward_device_scale_args* a) {
  return backward_device_scale(stream, a);
}
int nvfp4_linear_backward_device_scale_cta(void* stream, const nvfp4_linear_backward_device_scale_args* a) {
  return backward_device_scale(stream, a);
}
int nvfp4_linear_backward(void* stream, const nvfp4_linear_backward_device_scale_args* a) {
  return backward_device_scale(stream, a);
}

static int backward_weight_t(void* stream, const nvfp4_linear_backward_args* a) {
  const uint32_t I = a->input_dim, O = a->output_dim;
  return nvfp4_source_transpose(stream, NVFP4_SRC_NVFP4_TRANSPOSED, a->w_bytes, a->w_scales, a->w_global,
                                a->weight_t_h.bytes, a->weight_t_h.scales_packed, a->weight_t_h.global_scales,
                                a->weight_t_h.chunk_amax, a->weight_t_h.global_scale, O, I, padded_k(O), a->sign_seed,
                                a->scale_seed ^ 0x9e3779b9u, false, NVFP4_SCALES_PACKED, 0, 0, a->w_scale_layout);
}

int nvfp4_linear_backward_prepare_weight_t(void* stream, const nvfp4_linear_backward_args* a) {
  if (!a) return invalid("linear_backward_prepare_weight_t: null args");
  if (a->input_dim % 16 != 0) return invalid("linear_backward_prepare_weight_t: input_dim must be a multiple of 16");
  const nvfp4_ms_eden_operand& op = a->weight_t_h;
  if (!a->w_bytes || !a->w_scales || !a->w_global || !op.bytes || !op.scales_packed || !op.global_scales ||
      !op.global_scale || !op.chunk_amax)
    return invalid("linear_backward_prepare_weight_t: null pointer");
  return backward_weight_t(stream, a);
}

// Everything of nvfp4_linear_backward_ms_eden that runs between the fork onto the caller's side stream and the
// join; `ts` is the stream the two transposers go to (the side stream, or the main one when there is none).
static int backward_ms_eden_quantize(void* stream, void* ts, const nvfp4_linear_backward_args* a) {
  const uint32_t T = a->token_count, I = a->input_dim, O = a->output_dim;
  const uint32_t ok = padded_k(O), tk = padded_k(T);
  cudaStream_t s = S(stream);
  // Scale-RNG index space of the transposed operands (K = tokens): a shard addresses the groups of the
  // unsharded operand, row * (K_total / 16) + first_token / 16 + local group.
  const uint32_t total_tk = a->total_token_count ? padded_k(a->total_token_count) : tk;
  const uint32_t t_stride = total_tk / 16u, t_offset = a->total_token_count ? a->token_offset / 16u : 0u;
  int rc;

  // 3. W^T and 4. X^T from their NVFP4 forms (quantize/transpose.rs:14-93).  Enqueued first: they depend on
  //    nothing computed below and are ALU bound, so on a side stream they run beside the HBM-bound dY amax
  //    pass of step 2.
  rc = nvfp4_source_transpose(ts, NVFP4_SRC_ROWWISE_NVFP4_TRANSPOSED, a->x_bytes, a->x_scales, a->x_globals,
                              a->input_t_h.bytes, a->input_t_h.scales_packed, a->input_t_h.global_scales,
                              a->input_t_h.chunk_amax, a->input_t_h.global_scale, T, I, tk, a->sign_seed,
                              a->scale_seed ^ 0xc2b2ae35u, false, NVFP4_SCALES_PACKED, a->token_offset, t_offset,
                              a->x_scale_layout, a->x_decoded_amax, t_stride);
  if (rc) return rc;
  if (!a->weight_t_prepared) {
    rc = backward_weight_t(ts, a);
    if (rc) return rc;
  }

  // 1. dbias.  When the dY quantization below runs tiled, the column sums ride along with it:
  //    each row tile leaves its partial sums in the (not yet written) dinput buffer and a small
  //    kernel adds them up in tile order -- no extra pass over dY.  Otherwise the sum is done
  //    by the stand-alone kernel in the reference's order.
  const size_t dx_bytes = static_cast<size_t>(T) * I * (a->dinput_dtype == NVFP4_DTYPE_F32 ? 4 : 2);
  const size_t partial_bytes = static_cast<size_t>(ms_eden_pair_row_tiles(T)) * O * sizeof(float);
  bool fuse_dbias = a->dbias != nullptr && partial_bytes <= dx_bytes &&
                    (reinterpret_cast<uintptr_t>(a->dinput) & 3u) == 0;

  // 2. dY: tensor amax -> one global scale shared by the row and the transposed operand.  The amax
  //    pass is enqueued further down, once it is known whether the pair kernel can turn the amax into
  //    the scale by itself (whole tiles) or a one-thread kernel has to do it.
  const uint64_t ne = static_cast<uint64_t>(T) * O;
  const float* e_gs = a->e_global_scale_override ? a->e_global_scale_override : a->e_h.global_scale;
  nvfp4_ms_eden_args q;
  std::memset(&q, 0, sizeof(q));
  q.src_dtype = a->e_dtype;
  q.x = a->e;
  q.rows = T;
  q.cols = O;
  q.global_scale = e_gs;
  q.scale_override = kQuartetSO;
  q.sign_seed = a->sign_seed;
  q.scale_layout = NVFP4_SCALES_PACKED;
  //    rows of dY (K = output features): sign index = feature, scale RNG index = flat group id
  q.src_kind = NVFP4_SRC_F32_ROWS;
  q.dst_row_len = ok;
  q.scale_seed = a->scale_seed;
  q.col_offset = 0;
  q.group_offset = a->token_offset * (ok / 16);
  q.out_fp4 = a->e_h.bytes;
  q.out_scales = a->e_h.scales_packed;
  q.out_global_scales = a->e_h.global_scales;
  //    rows of dY^T (K = tokens): sign index = token
  nvfp4_ms_eden_args qt = q;
  qt.src_kind = NVFP4_SRC_F32_TRANSPOSED;
  qt.dst_row_len = tk;
  qt.scale_seed = a->scale_seed ^ 0x85ebca6bu;  // gpt/linear_backward/ms_eden/quantize/pair.rs:36
  qt.col_offset = a->token_offset;
  qt.group_offset = t_offset;
  qt.group_row_stride = t_stride;
  qt.out_fp4 = a->e_t_h.bytes;
  qt.out_scales = a->e_t_h.scales_packed;
  qt.out_global_scales = a->e_t_h.global_scales;
  fuse_dbias = fuse_dbias && ms_eden_pair_is_tiled(q, qt);
  if (a->dbias && !fuse_dbias) {
    rc = launch_bias_grad(s, a->e, a->e_dtype, a->dbias, T, O);
    if (rc) return rc;
  }
  const float* amax_in = nullptr;
  if (!a->e_global_scale_override) {
    if (a->precomputed_e_amax_chunks != 0) {
      rc = launch_amax_from_chunks(s, a->e_h.chunk_amax, a->e_h.global_scale, a->precomputed_e_amax_chunks, 1);
    } else if (ms_eden_pair_takes_amax(q, qt)) {
      // the amax accumulates in word 0 of the (otherwise unused) chunk scratch; the pair kernel derives the
      // scale from it and publishes it in e_h.global_scale
      rc = launch_tensor_amax(s, a->e, a->e_dtype, nullptr, a->e_h.chunk_amax, ne);
      amax_in = a->e_h.chunk_amax;
    } else {
      rc = launch_tensor_amax(s, a->e, a->e_dtype, a->e_h.chunk_amax, a->e_h.global_scale, ne);
      if (rc) return rc;
      rc = launch_ms_eden_scale_from_amax(s, a->e_h.global_scale, a->e_h.global_scale);
    }
    if (rc) return rc;
  }
  float* partials = fuse_dbias ? static_cast<float*>(a->dinput) : nullptr;
  // one pass over dY for both orientations (+ column sums)
  rc = ms_eden_pair(stream, q, qt, partials, amax_in, amax_in ? a->e_h.global_scale : nullptr);
  if (rc) return rc;
  if (fuse_dbias) rc = launch_col_sum_reduce(s, partials, a->dbias, ms_eden_pair_row_tiles(T), O);
  return rc;
}

int nvfp4_linear_backward_ms_eden(void* stream, const nvfp4_linear_backward_args* a) {
  if (!a) return invalid("linear_backward: null args");
  const uint32_t T = a->token_count, I = a->input_dim, O = a->output_dim;
  if (I % 16 != 0) return invalid("linear_backward: input_dim must be a multiple of 16");
  if (!a->e || !a->w_bytes || !a->w_scales || !a->w_global || !a->x_bytes || !a->x_scales || !a->x_globals ||
      !a->dinput || !a->dweight)
    return invalid("linear_backward: null tensor pointer");
  const nvfp4_ms_eden_operand* ops[4] = {&a->e_h, &a->e_t_h, &a->weight_t_h, &a->input_t_h};
  for (const nvfp4_ms_eden_operand* op : ops)
    if (!op->bytes || !op->scales_packed || !op->global_scales || !op->global_scale || !op->chunk_amax)
      return invalid("linear_backward: null scratch pointer");
  if ((a->e_dtype != NVFP4_DTYPE_F32 && a->e_dtype != NVFP4_DTYPE_BF16) ||
      (a->dinput_dtype != NVFP4_DTYPE_F32 && a->dinput_dtype != NVFP4_DTYPE_BF16) ||
      (a->dweight_dtype != NVFP4_DTYPE_F32 && a->dweight_dtype != NVFP4_DTYPE_BF16))
    return invalid("linear_backward: unknown dtype code");
  if (a->total_token_count && (a->token_offset % 128 != 0 || a->token_offset + T > a->total_token_count))
    return invalid("linear_backward: a token shard starts on a multiple of 128 and ends inside the batch");
  if (a->side_stream && (!a->fork_event || !a->join_event))
    return invalid("linear_backward: side_stream needs fork_event and join_event");
  cudaStream_t s = S(stream);

  // fork: every failure above happens before it, and every path below goes through the join
  void* ts = stream;
  bool forked = false;
  if (a->side_stream) {
    cudaError_t e = cudaEventRecord(static_cast<cudaEvent_t>(a->fork_event), s);
    if (e == cudaSuccess) e = cudaStreamWaitEvent(S(a->side_stream), static_cast<cudaEvent_t>(a->fork_event), 0);
    if (e != cudaSuccess) return static_cast<int>(e);
    ts = a->side_stream;
    forked = true;
  }
  int rc = backward_ms_eden_quantize(stream, ts, a);
  if (forked) {
    // join: the GEMMs need W^T and X^T; on an error path this leaves neither stream (nor a capture in
    // progress) dangling
    cudaError_t e = cudaEventRecord(static_cast<cudaEvent_t>(a->join_event), S(a->side_stream));
    if (e == cudaSuccess) e = cudaStreamWaitEvent(s, static_cast<cudaEvent_t>(a->join_event), 0);
    if (rc == 0 && e != cudaSuccess) rc = static_cast<int>(e);
  }
  if (rc) return rc;

  // 5. dX = dY . W   (contraction over output features) and dW = dY^T . X (over tokens)
  return backward_gemms(s, a->e_h.bytes, a->e_h.scales_packed, a->e_h.global_scales, a->weight_t_h.bytes,
                        a->weight_t_h.scales_packed, a->weight_t_h.global_scale, a->e_t_h.bytes, a->e_t_h.scales_packed,
                        a->e_t_h.global_scales, a->input_t_h.bytes, a->input_t_h.scales_packed,
                        a->input_t_h.global_scale, a->dinput, a->dinput_dtype, a->dweight, a->dweight_dtype, T, I, O);
}

}  // extern "C"
