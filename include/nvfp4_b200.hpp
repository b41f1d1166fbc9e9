// nvfp4_b200.hpp -- C++ host layer over the C ABI of nvfp4_b200.h.
//
// The reference drives its kernels through per-operation module structs: `XxxModule::from_module(..)`
// builds one, each operation is a `&self` method that takes one args struct of borrowed device buffers
// plus u32 dimensions, is asynchronous on the caller's stream, and returns `Result<(), DriverError>`
// (crates/cuda-kernels/src/utils/nvfp4/quant/launcher.rs:18-34, utils/nvfp4_tma_matmul/launcher.rs:23-33,
// gpt/linear_backward.rs:31-38).  This header gives C++ callers the same shape: the same module and
// method names, `DeviceBuffer<T>` views that carry their element count, length checks where the
// reference asserts, and a `DriverError` value instead of a panic or an exception.  Nothing here owns
// memory, allocates or synchronises; every method forwards to exactly one C-ABI call.
//
// Header only; needs nvfp4_b200.h and the C++ standard library, not the CUDA headers (streams travel as
// `void*`, i.e. a cudaStream_t / CUstream).
#ifndef NVFP4_B200_HPP_
#define NVFP4_B200_HPP_

#include <cstddef>
#include <cstdint>
#include <string>

#include "nvfp4_b200.h"

namespace nvfp4_b200 {

using Stream = void*;

// `DriverError(u32)` of the reference: 0 is success, anything else a CUDA error number
// (1 = invalid value for shape, alignment and buffer-length violations).
struct DriverError {
  int code = 0;
  std::string message;
  bool ok() const { return code == 0; }
  explicit operator bool() const { return code != 0; }  // `if (auto err = module.op(..)) return err;`
};

namespace detail {
inline DriverError from_rc(int rc) {
  if (rc == 0) return {};
  return DriverError{rc, nvfp4_last_error()};
}
inline DriverError invalid(const char* what) { return DriverError{1, what}; }
}  // namespace detail

// A borrowed device buffer: pointer and element count (`&DeviceBuffer<T>` of the reference).
template <typename T>
struct DeviceBuffer {
  T* ptr = nullptr;
  size_t len = 0;
  DeviceBuffer() = default;
  DeviceBuffer(T* p, size_t n) : ptr(p), len(n) {}
  // a mutable view converts to a read-only one
  template <typename U, typename = decltype(static_cast<T*>(static_cast<U*>(nullptr)))>
  DeviceBuffer(const DeviceBuffer<U>& o) : ptr(o.ptr), len(o.len) {}
};

// Element type tag of f32 / bf16 tensors (bf16 travels as uint16_t bit patterns).
template <typename T> struct dtype_of;
template <> struct dtype_of<float> { static constexpr int value = NVFP4_DTYPE_F32; };
template <> struct dtype_of<const float> { static constexpr int value = NVFP4_DTYPE_F32; };
template <> struct dtype_of<uint16_t> { static constexpr int value = NVFP4_DTYPE_BF16; };
template <> struct dtype_of<const uint16_t> { static constexpr int value = NVFP4_DTYPE_BF16; };

inline uint32_t padded_k(uint32_t k) { return nvfp4_padded_k(k); }
inline size_t scale_packed_len(uint32_t mn_extent, uint32_t k) { return nvfp4_scale_packed_len(mn_extent, k); }
inline uint32_t tensor_amax_chunks(uint32_t element_count) { return nvfp4_tensor_amax_chunks(element_count); }

// utils/nvfp4/tensor.rs:5-45: `Nvfp4DeviceTensor` (one global scale) and `Nvfp4RowwiseDeviceTensor`
// (one per row) as views.  `scale_layout` says whether `scales` is row-major [rows][cols/16] or the
// packed plane the GEMM reads (scale_packed_len(rows, cols) bytes).
struct Nvfp4TensorView {
  DeviceBuffer<uint8_t> bytes;          // rows * cols / 2
  DeviceBuffer<uint8_t> scales;         // rows * cols / 16, or scale_packed_len(rows, cols)
  DeviceBuffer<float> global_scales;    // 1 (tensor scale) or rows (rowwise)
  uint32_t rows = 0, cols = 0;
  int scale_layout = NVFP4_SCALES_PACKED;
  bool rowwise = false;
  DeviceBuffer<float> decoded_amax;     // optional f32[1]: max |decoded value| (forward quantizer -> backward)

  static size_t bytes_len(uint32_t rows, uint32_t cols) { return static_cast<size_t>(rows) * cols / 2; }
  static size_t scales_len(uint32_t rows, uint32_t cols, int layout) {
    return layout == NVFP4_SCALES_PACKED ? scale_packed_len(rows, cols) : static_cast<size_t>(rows) * cols / 16;
  }
  DriverError check() const {
    if (cols % 16 != 0) return detail::invalid("Nvfp4TensorView: cols must be a multiple of 16");
    if (bytes.len < bytes_len(rows, cols)) return detail::invalid("Nvfp4TensorView: bytes buffer too short");
    if (scales.len < scales_len(rows, cols, scale_layout)) return detail::invalid("Nvfp4TensorView: scales buffer too short");
    if (global_scales.len < (rowwise ? rows : 1u)) return detail::invalid("Nvfp4TensorView: global scale buffer too short");
    return {};
  }
};

// utils/nvfp4/quant/launcher.rs:18-34 `Nvfp4QuantModule`.
class Nvfp4QuantModule {
 public:
  static Nvfp4QuantModule from_module() { return {}; }

  // quant/amax.rs:8-17
  DriverError row_amax_f32(Stream s, DeviceBuffer<const float> x, DeviceBuffer<float> out, uint32_t row_count,
                           uint32_t row_len) const {
    if (x.len < static_cast<size_t>(row_count) * row_len || out.len < row_count)
      return detail::invalid("row_amax_f32: buffer too short");
    return detail::from_rc(nvfp4_row_amax_f32(s, x.ptr, out.ptr, row_count, row_len));
  }
  // quant/amax.rs:19-23
  DriverError tensor_amax_f32(Stream s, DeviceBuffer<const float> x, DeviceBuffer<float> chunk_amax,
                              DeviceBuffer<float> out) const {
    if (x.len > 0xffffffffu) return detail::invalid("tensor_amax_f32: more than 2^32 - 1 elements");
    const uint32_t n = static_cast<uint32_t>(x.len);
    if (chunk_amax.len < tensor_amax_chunks(n) || out.len < 1) return detail::invalid("tensor_amax_f32: buffer too short");
    return detail::from_rc(nvfp4_tensor_amax_f32(s, x.ptr, chunk_amax.ptr, out.ptr, n));
  }
  // quant/amax.rs:25-39
  DriverError tensor_amax_from_chunks_f32(Stream s, DeviceBuffer<const float> chunk_amax, DeviceBuffer<float> out,
                                          uint32_t chunk_count) const {
    if (chunk_amax.len < chunk_count || out.len < 1) return detail::invalid("tensor_amax_from_chunks_f32: buffer too short");
    return detail::from_rc(nvfp4_tensor_amax_from_chunks_f32(s, chunk_amax.ptr, out.ptr, chunk_count));
  }
  // quant/four_six.rs:25-58: rowwise four-six from a row amax computed earlier (logical scales)
  DriverError fp32_to_nvfp4_four_six_rowwise(Stream s, DeviceBuffer<const float> x, DeviceBuffer<const float> amax,
                                             const Nvfp4TensorView& out) const {
    if (auto e = out.check()) return e;
    if (!out.rowwise || out.scale_layout != NVFP4_SCALES_LOGICAL)
      return detail::invalid("fp32_to_nvfp4_four_six_rowwise: output must be rowwise with logical scales");
    const size_t n = static_cast<size_t>(out.rows) * out.cols;
    if (x.len < n || amax.len < out.rows) return detail::invalid("fp32_to_nvfp4_four_six_rowwise: buffer too short");
    return detail::from_rc(nvfp4_fp32_to_nvfp4_four_six_rowwise(s, x.ptr, amax.ptr, out.bytes.ptr, out.scales.ptr,
                                                                out.global_scales.ptr, static_cast<uint32_t>(n / 16),
                                                                out.cols));
  }
  // Tensor-scale or rowwise four-six of an f32 / bf16 matrix from a given amax, scales in `out.scale_layout`
  // (quant/four_six.rs:12-58 followed by nvfp4_tma_matmul/scale_pack.rs:54-78 when packed).
  template <typename T>
  DriverError quantize_four_six(Stream s, DeviceBuffer<const T> x, DeviceBuffer<const float> amax,
                                const Nvfp4TensorView& out) const {
    if (auto e = out.check()) return e;
    if (x.len < static_cast<size_t>(out.rows) * out.cols || amax.len < (out.rowwise ? out.rows : 1u))
      return detail::invalid("quantize_four_six: buffer too short");
    return detail::from_rc(nvfp4_quantize_four_six(s, x.ptr, dtype_of<T>::value, amax.ptr, out.rowwise ? 1 : 0, out.rows,
                                                   out.cols, out.bytes.ptr, out.scales.ptr, out.scale_layout,
                                                   out.global_scales.ptr));
  }
  // `RowwiseNvfp4Scratch::quantize_row_amax` (crates/gpt2-nvfp4/src/types/nvfp4_scratch/scratch.rs:35-52):
  // row amax and rowwise four-six in one pass.  `row_amax` may be empty for rows of up to 4096 values;
  // `out.decoded_amax`, when set, receives max |decoded value| for the backward pass.
  template <typename T>
  DriverError quantize_row_amax(Stream s, DeviceBuffer<const T> x, const Nvfp4TensorView& out,
                                DeviceBuffer<float> row_amax = {}) const {
    if (auto e = out.check()) return e;
    if (!out.rowwise) return detail::invalid("quantize_row_amax: output must be rowwise");
    if (x.len < static_cast<size_t>(out.rows) * out.cols) return detail::invalid("quantize_row_amax: input too short");
    if (row_amax.ptr && row_amax.len < out.rows) return detail::invalid("quantize_row_amax: row_amax too short");
    return detail::from_rc(nvfp4_quantize_four_six_rowwise_fused(s, x.ptr, dtype_of<T>::value, out.rows, out.cols,
                                                                 out.bytes.ptr, out.scales.ptr, out.scale_layout,
                                                                 out.global_scales.ptr, row_amax.ptr,
                                                                 out.decoded_amax.ptr));
  }
  // The same quantizer applied to relu(pre)^2 computed on load: the MLP activation is never stored
  // (`RowwiseNvfp4Scratch::quantize_precomputed_amax` fed by the ReLU^2 post-op's row amax in the reference,
  // crates/gpt2-nvfp4/src/types/l3_mlp/forward.rs:60-76).  `row_amax_in` may be empty.
  template <typename T>
  DriverError quantize_relu2(Stream s, DeviceBuffer<const T> pre_activation, DeviceBuffer<const float> row_amax_in,
                             const Nvfp4TensorView& out) const {
    if (auto e = out.check()) return e;
    if (!out.rowwise) return detail::invalid("quantize_relu2: output must be rowwise");
    if (pre_activation.len < static_cast<size_t>(out.rows) * out.cols) return detail::invalid("quantize_relu2: input too short");
    if (row_amax_in.ptr && row_amax_in.len < out.rows) return detail::invalid("quantize_relu2: row_amax_in too short");
    return detail::from_rc(nvfp4_quantize_relu2_four_six_rowwise(s, pre_activation.ptr, dtype_of<T>::value, out.rows,
                                                                 out.cols, row_amax_in.ptr, out.bytes.ptr, out.scales.ptr,
                                                                 out.scale_layout, out.global_scales.ptr, nullptr,
                                                                 out.decoded_amax.ptr));
  }
  // Tensor amax of an f32 / bf16 tensor (quant/amax.rs:19-23)
  template <typename T>
  DriverError tensor_amax(Stream s, DeviceBuffer<const T> x, DeviceBuffer<float> chunk_amax, DeviceBuffer<float> out) const {
    if (chunk_amax.len < (x.len + 1023) / 1024 || out.len < 1) return detail::invalid("tensor_amax: buffer too short");
    if (dtype_of<T>::value == NVFP4_DTYPE_F32)
      return detail::from_rc(nvfp4_tensor_amax_f32(s, reinterpret_cast<const float*>(x.ptr), chunk_amax.ptr, out.ptr, x.len));
    return detail::from_rc(nvfp4_tensor_amax_bf16(s, x.ptr, chunk_amax.ptr, out.ptr, x.len));
  }
};

// An NVFP4-encoded bias [n]: bytes n/2, logical scale bytes n/16, one global scale
// (the `bias: Nvfp4DeviceTensor` of the reference's projection args, gpt/mlp/args.rs:6-27).
struct Nvfp4BiasView {
  DeviceBuffer<const uint8_t> bytes, scales;
  DeviceBuffer<const float> global_scale;
  bool present() const { return bytes.ptr && scales.ptr && global_scale.ptr; }
};

// Fused epilogue of a projection (gpt/projection_postop.rs:97-162 as separate passes in the reference).
enum class Epilogue : int {
  None = NVFP4_EPI_NONE,
  Bias = NVFP4_EPI_BIAS,
  Relu2 = NVFP4_EPI_RELU2,
  Residual = NVFP4_EPI_RESIDUAL,
};

// utils/nvfp4_tma_matmul/launcher.rs:23-328 `Nvfp4GemmModule`.
class Nvfp4GemmModule {
 public:
  static Nvfp4GemmModule from_module() { return {}; }

  // out[m][n] = epilogue((A . B^T) * ga * gb): A = quantized activation [m][k] (rowwise or tensor scale),
  // B = quantized weight [n][k] (tensor scale), both with packed scales.  `aux` receives the
  // pre-activation of the ReLU^2 epilogue when set.
  template <typename T>
  DriverError gemm(Stream s, const Nvfp4TensorView& a, const Nvfp4TensorView& b, DeviceBuffer<T> out,
                   Epilogue epilogue = Epilogue::None, DeviceBuffer<const float> bias = {},
                   DeviceBuffer<T> aux = {}, DeviceBuffer<float> relu2_row_amax = {}) const {
    if (auto e = a.check()) return e;
    if (auto e = b.check()) return e;
    if (a.cols != b.cols) return detail::invalid("gemm: A and B must share K");
    if (a.scale_layout != NVFP4_SCALES_PACKED || b.scale_layout != NVFP4_SCALES_PACKED)
      return detail::invalid("gemm: operands need packed scales");
    if (b.rowwise) return detail::invalid("gemm: B takes a tensor scale");
    const size_t mn = static_cast<size_t>(a.rows) * b.rows;
    if (out.len < mn || (aux.ptr && aux.len < mn)) return detail::invalid("gemm: output buffer too short");
    if (epilogue != Epilogue::None && bias.len < b.rows) return detail::invalid("gemm: bias too short");
    nvfp4_gemm_args g{};
    g.a_bytes = a.bytes.ptr, g.a_scales = a.scales.ptr, g.a_global = a.global_scales.ptr;
    g.b_bytes = b.bytes.ptr, g.b_scales = b.scales.ptr, g.b_global = b.global_scales.ptr;
    g.out = out.ptr, g.aux = aux.ptr, g.bias = bias.ptr;
    g.m = a.rows, g.n = b.rows, g.k = a.cols, g.ldo = b.rows;
    g.global_scale_mode = a.rowwise ? NVFP4_GS_ROWWISE_A : NVFP4_GS_TENSOR;
    g.weight_global_scale = 1.0f;
    g.epilogue = static_cast<int>(epilogue);
    g.out_dtype = dtype_of<T>::value;
    if (relu2_row_amax.ptr && relu2_row_amax.len < a.rows) return detail::invalid("gemm: relu2_row_amax too short");
    g.relu2_row_amax = relu2_row_amax.ptr;
    return detail::from_rc(nvfp4_gemm(s, &g));
  }
  // launcher.rs:39-166: validates the operands and puts their tensor maps into the calling thread's cache
  DriverError prepare_tma_nvfp4_device_scales(Stream s, const Nvfp4TensorView& a, const Nvfp4TensorView& b) const {
    if (auto e = a.check()) return e;
    if (auto e = b.check()) return e;
    if (a.cols != b.cols) return detail::invalid("prepare_tma: A and B must share K");
    return detail::from_rc(nvfp4_prepare_tma_nvfp4_device_scales(s, a.bytes.ptr, a.scales.ptr, b.bytes.ptr, b.scales.ptr,
                                                                 a.rows, a.cols, b.rows));
  }
  // launcher.rs:224-274, the reference's own entry (f32 output, no epilogue)
  DriverError gemm_tma_nvfp4_rowwise_a_scale_and_global_scale_buffer(Stream s, const Nvfp4TensorView& a,
                                                                     const Nvfp4TensorView& b,
                                                                     DeviceBuffer<float> out) const {
    if (auto e = a.check()) return e;
    if (auto e = b.check()) return e;
    if (a.cols != b.cols || !a.rowwise || b.rowwise) return detail::invalid("gemm_tma: operand kinds / K mismatch");
    if (out.len < static_cast<size_t>(a.rows) * b.rows) return detail::invalid("gemm_tma: output buffer too short");
    return detail::from_rc(nvfp4_gemm_tma_nvfp4_rowwise_a_scale_and_global_scale_buffer(
        s, a.bytes.ptr, a.scales.ptr, b.bytes.ptr, b.scales.ptr, out.ptr, a.rows, a.cols, b.rows, a.global_scales.ptr,
        b.global_scales.ptr));
  }
};

namespace detail {
// One forward projection with the reference's argument list; scale planes in the logical layout need the
// packed scratch of the same operand (`LmHeadTmaArgs`, gpt/lm_head.rs:41-54).
struct ProjectionScratch {
  DeviceBuffer<uint8_t> input_scales_packed, weight_scales_packed;
};
inline DriverError fill_projection(nvfp4_projection_args& c, const Nvfp4TensorView& input, const Nvfp4TensorView& weight,
                                   const Nvfp4BiasView& bias, const ProjectionScratch& scratch) {
  if (auto e = input.check()) return e;
  if (auto e = weight.check()) return e;
  if (!input.rowwise || weight.rowwise || input.cols != weight.cols)
    return invalid("projection: rowwise input, tensor-scale weight, common input_dim");
  if (input.scale_layout == NVFP4_SCALES_LOGICAL &&
      scratch.input_scales_packed.len < scale_packed_len(input.rows, input.cols))
    return invalid("projection: input_scales_packed scratch too short");
  if (weight.scale_layout == NVFP4_SCALES_LOGICAL &&
      scratch.weight_scales_packed.len < scale_packed_len(weight.rows, weight.cols))
    return invalid("projection: weight_scales_packed scratch too short");
  if (bias.present() && (bias.bytes.len < weight.rows / 2 || bias.scales.len < weight.rows / 16))
    return invalid("projection: bias too short");
  c.input_bytes = input.bytes.ptr, c.input_scales = input.scales.ptr, c.input_scale_layout = input.scale_layout;
  c.input_global_scales = input.global_scales.ptr;
  c.weight_bytes = weight.bytes.ptr, c.weight_scales = weight.scales.ptr, c.weight_scale_layout = weight.scale_layout;
  c.weight_global_scale = weight.global_scales.ptr;
  c.bias_bytes = bias.bytes.ptr, c.bias_scales = bias.scales.ptr, c.bias_global_scale = bias.global_scale.ptr;
  c.token_count = input.rows, c.input_dim = input.cols, c.output_dim = weight.rows;
  c.input_scales_packed_scratch = scratch.input_scales_packed.ptr;
  c.weight_scales_packed_scratch = scratch.weight_scales_packed.ptr;
  return {};
}
}  // namespace detail
using ProjectionScratch = detail::ProjectionScratch;

// gpt/attention/qkv_projection/launcher.rs:8-42 `AttentionModule` (its two projections).
class AttentionModule {
 public:
  static AttentionModule from_module() { return {}; }
  template <typename T>
  DriverError qkv_projection(Stream s, const Nvfp4TensorView& input, const Nvfp4TensorView& weight,
                             const Nvfp4BiasView& bias, DeviceBuffer<T> out, const ProjectionScratch& scratch = {}) const {
    nvfp4_projection_args c{};
    if (auto e = detail::fill_projection(c, input, weight, bias, scratch)) return e;
    if (out.len < static_cast<size_t>(input.rows) * weight.rows) return detail::invalid("qkv_projection: out too short");
    c.out = out.ptr, c.out_dtype = dtype_of<T>::value;
    return detail::from_rc(nvfp4_qkv_projection(s, &c));
  }
  // residual (f32, in place) = fma(1, X . W^T + b, residual)
  DriverError c_proj(Stream s, const Nvfp4TensorView& input, const Nvfp4TensorView& weight, const Nvfp4BiasView& bias,
                     DeviceBuffer<float> residual, const ProjectionScratch& scratch = {}) const {
    nvfp4_projection_args c{};
    if (auto e = detail::fill_projection(c, input, weight, bias, scratch)) return e;
    if (residual.len < static_cast<size_t>(input.rows) * weight.rows) return detail::invalid("c_proj: residual too short");
    c.out = residual.ptr, c.out_dtype = NVFP4_DTYPE_F32;
    return detail::from_rc(nvfp4_c_proj(s, &c));
  }
};

// gpt/lm_head.rs:65-125 `LmHeadModule`.
class LmHeadModule {
 public:
  static LmHeadModule from_module() { return {}; }
  template <typename T>
  DriverError logits(Stream s, const Nvfp4TensorView& input, const Nvfp4TensorView& weight, DeviceBuffer<T> logits_out,
                     const ProjectionScratch& scratch = {}, bool tma = false) const {
    nvfp4_projection_args c{};
    if (auto e = detail::fill_projection(c, input, weight, Nvfp4BiasView{}, scratch)) return e;
    if (logits_out.len < static_cast<size_t>(input.rows) * weight.rows) return detail::invalid("logits: output too short");
    c.out = logits_out.ptr, c.out_dtype = dtype_of<T>::value;
    return detail::from_rc(tma ? nvfp4_lm_head_logits_tma(s, &c) : nvfp4_lm_head_logits(s, &c));
  }
  template <typename T>
  DriverError logits_tma(Stream s, const Nvfp4TensorView& input, const Nvfp4TensorView& weight, DeviceBuffer<T> logits_out,
                         const ProjectionScratch& scratch = {}) const {
    return logits<T>(s, input, weight, logits_out, scratch, true);
  }
};

// gpt/next_latent/launch_projection.rs:10-29 `NextLatModule::projection`.
class NextLatModule {
 public:
  static NextLatModule from_module() { return {}; }
  template <typename T>
  DriverError projection(Stream s, const Nvfp4TensorView& input, const Nvfp4TensorView& weight, const Nvfp4BiasView& bias,
                         DeviceBuffer<T> out, const ProjectionScratch& scratch = {}) const {
    nvfp4_projection_args c{};
    if (auto e = detail::fill_projection(c, input, weight, bias, scratch)) return e;
    if (out.len < static_cast<size_t>(input.rows) * weight.rows) return detail::invalid("projection: out too short");
    c.out = out.ptr, c.out_dtype = dtype_of<T>::value;
    return detail::from_rc(nvfp4_nextlat_projection(s, &c));
  }
};

// gpt/mlp/launcher.rs:53-76 `MlpModule`: the two MLP projections and the element-wise step between the
// two linear backwards.
class MlpModule {
 public:
  static MlpModule from_module() { return {}; }

  // up_relu2: hidden = relu(x . Wfc^T + b)^2, pre-activation kept for backward
  template <typename T>
  DriverError up_relu2(Stream s, const Nvfp4TensorView& x, const Nvfp4TensorView& w_fc, DeviceBuffer<const float> bias,
                       DeviceBuffer<T> pre_activation, DeviceBuffer<T> hidden) const {
    return Nvfp4GemmModule{}.gemm<T>(s, x, w_fc, hidden, Epilogue::Relu2, bias, pre_activation);
  }
  // down projection with bias (the residual form is Epilogue::Residual on an f32 stream)
  template <typename T>
  DriverError down(Stream s, const Nvfp4TensorView& hidden, const Nvfp4TensorView& w_proj, DeviceBuffer<const float> bias,
                   DeviceBuffer<T> out) const {
    return Nvfp4GemmModule{}.gemm<T>(s, hidden, w_proj, out, Epilogue::Bias, bias);
  }
  // launcher.rs:53-59 with the reference's argument list (NVFP4 bias): pre = X . W^T + b, hidden = relu(pre)^2;
  // an empty `hidden` keeps only the pre-activation, `relu2_row_amax` (optional) receives the row amax of relu(pre)^2
  template <typename T>
  DriverError up_relu2(Stream s, const Nvfp4TensorView& input, const Nvfp4TensorView& weight, const Nvfp4BiasView& bias,
                       DeviceBuffer<T> pre_activation, DeviceBuffer<T> hidden, DeviceBuffer<float> relu2_row_amax = {},
                       const ProjectionScratch& scratch = {}) const {
    nvfp4_projection_args c{};
    if (auto e = detail::fill_projection(c, input, weight, bias, scratch)) return e;
    const size_t mn = static_cast<size_t>(input.rows) * weight.rows;
    if (pre_activation.len < mn || (hidden.ptr && hidden.len < mn)) return detail::invalid("up_relu2: output too short");
    if (relu2_row_amax.ptr && relu2_row_amax.len < input.rows) return detail::invalid("up_relu2: relu2_row_amax too short");
    c.out = hidden.ptr, c.pre_activation = pre_activation.ptr, c.out_dtype = dtype_of<T>::value;
    c.relu2_row_amax = relu2_row_amax.ptr;
    return detail::from_rc(nvfp4_mlp_up_relu2(s, &c));
  }
  // launcher.rs:60-66: residual (f32, in place) += X . W^T + b
  DriverError down_residual(Stream s, const Nvfp4TensorView& input, const Nvfp4TensorView& weight,
                            const Nvfp4BiasView& bias, DeviceBuffer<float> residual,
                            const ProjectionScratch& scratch = {}) const {
    nvfp4_projection_args c{};
    if (auto e = detail::fill_projection(c, input, weight, bias, scratch)) return e;
    if (residual.len < static_cast<size_t>(input.rows) * weight.rows) return detail::invalid("down_residual: residual too short");
    c.out = residual.ptr, c.out_dtype = NVFP4_DTYPE_F32;
    return detail::from_rc(nvfp4_mlp_down_residual(s, &c));
  }
  // launcher.rs:66-76: d_pre = (d_out * 2) * max(pre, 0)
  DriverError relu2_backward(Stream s, DeviceBuffer<const float> pre_activation, DeviceBuffer<const float> d_out,
                             DeviceBuffer<float> d_pre_activation) const {
    if (pre_activation.len > 0xffffffffu || d_out.len < pre_activation.len || d_pre_activation.len < pre_activation.len)
      return detail::invalid("relu2_backward: buffer lengths");
    return detail::from_rc(nvfp4_relu2_backward(s, pre_activation.ptr, d_out.ptr, d_pre_activation.ptr,
                                                static_cast<uint32_t>(pre_activation.len)));
  }
  // The same pass that also leaves the chunk amax of d_pre in `chunk_amax` (point it at the fc backward's
  // e_h.chunk_amax and pass *chunk_count as precomputed_e_amax_chunks).
  template <typename T>
  DriverError relu2_backward_amax(Stream s, DeviceBuffer<const T> pre_activation, DeviceBuffer<const T> d_out,
                                  DeviceBuffer<T> d_pre_activation, DeviceBuffer<float> chunk_amax,
                                  uint32_t* chunk_count) const {
    if (d_out.len < pre_activation.len || d_pre_activation.len < pre_activation.len)
      return detail::invalid("relu2_backward_amax: buffer lengths");
    const int kind = dtype_of<T>::value;  // pre_kind uses the same numbering for f32 / bf16
    return detail::from_rc(nvfp4_relu2_backward_amax(s, pre_activation.ptr, kind, d_out.ptr, d_pre_activation.ptr, kind,
                                                     pre_activation.len, chunk_amax.ptr,
                                                     static_cast<uint32_t>(chunk_amax.len), chunk_count));
  }
};

// One MS-EDEN operand of the backward scratch (gpt/linear_backward/args/ms_eden/scratch.rs:11-89).
struct MsEdenOperandBuffers {
  DeviceBuffer<uint8_t> bytes, scales_packed;
  DeviceBuffer<float> global_scales, global_scale, chunk_amax;
  nvfp4_ms_eden_operand c() const {
    return nvfp4_ms_eden_operand{bytes.ptr, scales_packed.ptr, global_scales.ptr, global_scale.ptr, chunk_amax.ptr};
  }
};

// Element counts of every scratch buffer of one linear backward, the sizing rule of
// `LinearBackwardMsEdenScratchBuffers::new` (args/ms_eden/scratch.rs:91-115); the caller allocates.
struct MsEdenOperandSizes {
  size_t bytes, scales_packed, global_scales, global_scale, chunk_amax;
  bool fits(const MsEdenOperandBuffers& b) const {
    return b.bytes.len >= bytes && b.scales_packed.len >= scales_packed && b.global_scales.len >= global_scales &&
           b.global_scale.len >= global_scale && b.chunk_amax.len >= chunk_amax;
  }
};
struct LinearBackwardMsEdenScratchSizes {
  MsEdenOperandSizes e_h, e_t_h, weight_t_h, input_t_h;
  LinearBackwardMsEdenScratchSizes(uint32_t token_count, uint32_t input_dim, uint32_t output_dim) {
    const uint32_t ok = padded_k(output_dim), tk = padded_k(token_count);
    auto operand = [](uint32_t rows, uint32_t k, size_t amax_elems) {
      const size_t chunks = (amax_elems + 1023) / 1024;
      return MsEdenOperandSizes{static_cast<size_t>(rows) * k / 2, scale_packed_len(rows, k), rows, 1,
                                chunks ? chunks : 1};
    };
    e_h = operand(token_count, ok, static_cast<size_t>(token_count) * output_dim);
    e_t_h = operand(output_dim, tk, 1);
    weight_t_h = operand(input_dim, ok, static_cast<size_t>(output_dim) * input_dim);
    input_t_h = operand(input_dim, tk, static_cast<size_t>(token_count) * input_dim);
  }
};
struct LinearBackwardMsEdenScratchBuffers {
  MsEdenOperandBuffers e_h, e_t_h, weight_t_h, input_t_h;
};

// gpt/linear_backward/args/ms_eden/call.rs:8-36
template <typename T>
struct LinearBackwardMsEdenArgs {
  DeviceBuffer<const T> e;              // dY [token][out]
  Nvfp4TensorView weight;               // W [out][in], tensor scale
  Nvfp4TensorView input;                // saved X [token][in], rowwise
  LinearBackwardMsEdenScratchBuffers scratch;
  DeviceBuffer<T> dinput;               // [token][in]
  DeviceBuffer<float> dweight;          // [out][in]
  DeviceBuffer<float> dbias;            // [out] or empty
  uint32_t token_count = 0, input_dim = 0, output_dim = 0;
  uint32_t sign_seed = 0, scale_seed = 0;
  uint32_t precomputed_e_amax_chunks = 0;
  uint32_t token_offset = 0;
  DeviceBuffer<const float> e_global_scale_override;  // empty = derive from dY here
  DeviceBuffer<const float> x_decoded_amax;           // empty = input.decoded_amax, or a pass over X
  uint32_t total_token_count = 0;                     // tokens of the unsharded batch (0 = not sharded)
  // caller-owned second stream with its fork / join events (cudaStream_t, cudaEvent_t); null = serial
  Stream side_stream = nullptr;
  void* fork_event = nullptr;
  void* join_event = nullptr;
  bool weight_t_prepared = false;  // scratch.weight_t_h was filled by prepare_weight_t with these seeds
};

// gpt/linear_backward.rs:31-67, gpt/linear_backward/ms_eden.rs:15-55 `LinearBackwardModule`.
class LinearBackwardModule {
 public:
  static LinearBackwardModule from_module() { return {}; }

  // gpt/linear_backward/bias.rs:18-69
  DriverError linear_bias_grad(Stream s, DeviceBuffer<const float> e, DeviceBuffer<float> dbias, uint32_t token_count,
                               uint32_t output_dim) const {
    if (e.len < static_cast<size_t>(token_count) * output_dim || dbias.len < output_dim)
      return detail::invalid("linear_bias_grad: buffer too short");
    return detail::from_rc(nvfp4_linear_bias_grad(s, e.ptr, dbias.ptr, token_count, output_dim));
  }

  // The W^T step alone, for callers that run it early (it reads only the weight and the seeds).
  template <typename T>
  DriverError prepare_weight_t(Stream s, const LinearBackwardMsEdenArgs<T>& a) const {
    return run(s, a, true);
  }
  template <typename T>
  DriverError backward_ms_eden(Stream s, const LinearBackwardMsEdenArgs<T>& a) const {
    return run(s, a, false);
  }

 private:
  template <typename T>
  DriverError run(Stream s, const LinearBackwardMsEdenArgs<T>& a, bool weight_t_only) const {
    if (auto e = a.weight.check()) return e;
    if (auto e = a.input.check()) return e;
    if (a.weight.rows != a.output_dim || a.weight.cols != a.input_dim || a.weight.rowwise)
      return detail::invalid("backward_ms_eden: weight must be the tensor-scale W[out][in]");
    if (a.input.rows != a.token_count || a.input.cols != a.input_dim || !a.input.rowwise)
      return detail::invalid("backward_ms_eden: input must be the rowwise X[token][in]");
    const size_t te = static_cast<size_t>(a.token_count) * a.output_dim;
    const size_t ti = static_cast<size_t>(a.token_count) * a.input_dim;
    const size_t oi = static_cast<size_t>(a.output_dim) * a.input_dim;
    if (a.e.len < te || a.dinput.len < ti || a.dweight.len < oi || (a.dbias.ptr && a.dbias.len < a.output_dim))
      return detail::invalid("backward_ms_eden: gradient buffer too short");
    const LinearBackwardMsEdenScratchSizes need(a.token_count, a.input_dim, a.output_dim);
    if (!need.e_h.fits(a.scratch.e_h) || !need.e_t_h.fits(a.scratch.e_t_h) ||
        !need.weight_t_h.fits(a.scratch.weight_t_h) || !need.input_t_h.fits(a.scratch.input_t_h))
      return detail::invalid("backward_ms_eden: scratch smaller than LinearBackwardMsEdenScratchSizes");
    nvfp4_linear_backward_args c{};
    c.e = a.e.ptr, c.e_dtype = dtype_of<T>::value;
    c.w_bytes = a.weight.bytes.ptr, c.w_scales = a.weight.scales.ptr, c.w_scale_layout = a.weight.scale_layout;
    c.w_global = a.weight.global_scales.ptr;
    c.x_bytes = a.input.bytes.ptr, c.x_scales = a.input.scales.ptr, c.x_scale_layout = a.input.scale_layout;
    c.x_globals = a.input.global_scales.ptr;
    c.e_h = a.scratch.e_h.c(), c.e_t_h = a.scratch.e_t_h.c();
    c.weight_t_h = a.scratch.weight_t_h.c(), c.input_t_h = a.scratch.input_t_h.c();
    c.dinput = a.dinput.ptr, c.dinput_dtype = dtype_of<T>::value;
    c.dweight = a.dweight.ptr, c.dweight_dtype = NVFP4_DTYPE_F32;
    c.dbias = a.dbias.ptr;
    c.token_count = a.token_count, c.input_dim = a.input_dim, c.output_dim = a.output_dim;
    c.sign_seed = a.sign_seed, c.scale_seed = a.scale_seed;
    c.precomputed_e_amax_chunks = a.precomputed_e_amax_chunks;
    c.token_offset = a.token_offset;
    c.e_global_scale_override = a.e_global_scale_override.ptr;
    c.x_decoded_amax = a.x_decoded_amax.ptr ? a.x_decoded_amax.ptr : a.input.decoded_amax.ptr;
    c.total_token_count = a.total_token_count;
    c.side_stream = a.side_stream, c.fork_event = a.fork_event, c.join_event = a.join_event;
    c.weight_t_prepared = a.weight_t_prepared ? 1 : 0;
    if (weight_t_only) return detail::from_rc(nvfp4_linear_backward_prepare_weight_t(s, &c));
    return detail::from_rc(nvfp4_linear_backward_ms_eden(s, &c));
  }
};

// ---- checkpoint container (src/checkpoint/format/{writer,reader}.rs of the reference) -------------------
// CheckpointWriter::{write_header (the constructor's `open`), write_tensor, finish} and
// CheckpointReader::{read_header, read_tensor}; tensors live on the device as in save/tensor.rs and
// load/tensor.rs.  Scale bytes in a checkpoint are row-major (NVFP4_SCALES_LOGICAL).
class CheckpointWriter {
 public:
  CheckpointWriter() = default;
  CheckpointWriter(const CheckpointWriter&) = delete;
  CheckpointWriter& operator=(const CheckpointWriter&) = delete;
  ~CheckpointWriter() {
    if (handle_) nvfp4_checkpoint_writer_close(handle_);
  }
  DriverError write_header(const std::string& path, uint32_t tensor_count) {
    return detail::from_rc(nvfp4_checkpoint_writer_open(path.c_str(), tensor_count, &handle_));
  }
  DriverError write_tensor(Stream s, const std::string& name, const Nvfp4TensorView& t) {
    if (t.rowwise || t.scale_layout != NVFP4_SCALES_LOGICAL)
      return detail::invalid("checkpoint tensors carry one global scale and row-major scale bytes");
    return detail::from_rc(nvfp4_checkpoint_write_tensor_device(handle_, s, name.c_str(),
                                                                static_cast<uint64_t>(t.rows) * t.cols, t.global_scales.ptr,
                                                                t.bytes.ptr, t.bytes.len, t.scales.ptr, t.scales.len));
  }
  DriverError finish() {
    void* h = handle_;
    handle_ = nullptr;
    return detail::from_rc(nvfp4_checkpoint_writer_close(h));
  }

 private:
  void* handle_ = nullptr;
};

class CheckpointReader {
 public:
  CheckpointReader() = default;
  CheckpointReader(const CheckpointReader&) = delete;
  CheckpointReader& operator=(const CheckpointReader&) = delete;
  ~CheckpointReader() {
    if (handle_) nvfp4_checkpoint_reader_close(handle_);
  }
  DriverError read_header(const std::string& path, uint32_t* tensor_count) {
    return detail::from_rc(nvfp4_checkpoint_reader_open(path.c_str(), &handle_, tensor_count));
  }
  // header and name of the next tensor; the caller sizes its device buffers from `info`
  DriverError next_tensor(nvfp4_checkpoint_tensor_info* info) {
    return detail::from_rc(nvfp4_checkpoint_next_tensor(handle_, info));
  }
  // payload of that tensor into device buffers (bytes.len >= info.byte_len, scales.len >= info.scale_len)
  DriverError read_tensor(Stream s, DeviceBuffer<uint8_t> bytes, DeviceBuffer<uint8_t> scales, DeviceBuffer<float> global_scale) {
    return detail::from_rc(nvfp4_checkpoint_read_payload_device(handle_, s, bytes.ptr, scales.ptr, global_scale.ptr));
  }

 private:
  void* handle_ = nullptr;
};

// Caps split-K at two splits so that dW is bit-identical from run to run (process-wide; off by default).
inline void set_deterministic_reductions(bool on) { nvfp4_set_deterministic_reductions(on ? 1 : 0); }
inline bool deterministic_reductions() { return nvfp4_get_deterministic_reductions() != 0; }

// Reads and clears the device status word written by kernels whose bounded waits gave up
// (0 = none did).  Synchronises the stream.
inline DriverError read_device_status(Stream s, uint32_t* status) {
  return detail::from_rc(nvfp4_read_device_status(s, status));
}

}  // namespace nvfp4_b200

#endif  // NVFP4_B200_HPP_
