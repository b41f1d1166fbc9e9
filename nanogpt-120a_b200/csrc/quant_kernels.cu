// Bandwidth kernels of the NVFP4 projection path for sm_100a: amax reductions, the
// four-six quantizer, the MS-EDEN quantizer (row, transposed, NVFP4-source variants),
// decode, scale-plane packing, padding, post-ops and the bias gradient.
//
// Compiled with -fmad=false: the arithmetic below must round exactly like the
// reference's device code (one rounding per operation, no contraction).
//
// Work decomposition differs from the reference on purpose.  The reference gives each
// element its own lane and reduces 16-groups with shuffles; here one thread owns a whole
// 16-group (four-six) or 32-chunk (MS-EDEN) in registers, loads it with 128-bit
// transactions and writes nibbles as 8/16-byte words.  The reduction trees are evaluated
// in the same order as the reference's xor butterflies, so the bytes are identical.
#include <cuda_fp16.h>

#include <cstdlib>
#include <atomic>
#include <mutex>

#include "common.cuh"
#include "kernels.h"

namespace nvfp4 {

// ============================================================================
// amax
// ============================================================================

template <typename T>
struct VecTraits;
template <>
struct VecTraits<float> {
  static constexpr int kPerVec = 4;
};
template <>
struct VecTraits<__nv_bfloat16> {
  static constexpr int kPerVec = 8;
};

template <typename T>
__device__ __forceinline__ float vec_amax(const T* p);  // 16-byte aligned, kPerVec elements
template <>
__device__ __forceinline__ float vec_amax<float>(const float* p) {
  float4 t = __ldg(reinterpret_cast<const float4*>(p));
  return max_f32(max_f32(fabsf(t.x), fabsf(t.y)), max_f32(fabsf(t.z), fabsf(t.w)));
}
template <>
__device__ __forceinline__ float vec_amax<__nv_bfloat16>(const __nv_bfloat16* p) {
  uint4 t = __ldg(reinterpret_cast<const uint4*>(p));
  uint32_t w[4] = {t.x, t.y, t.z, t.w};
  float m = 0.0f;
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    m = max_f32(m, fabsf(__uint_as_float(w[j] << 16)));
    m = max_f32(m, fabsf(__uint_as_float(w[j] & 0xffff0000u)));
  }
  return m;
}

__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int s = 16; s > 0; s >>= 1) v = max_f32(v, __shfl_xor_sync(0xffffffffu, v, s));
  return v;
}

// One warp per row.  utils/nvfp4/quant/kernels/row_amax.rs:43-64 (max is order independent).
template <typename T>
__global__ void __launch_bounds__(256) row_amax_kernel(const T* __restrict__ x, float* __restrict__ out,
                                                        uint32_t rows, uint32_t row_len) {
  const uint32_t row = blockIdx.x * 8 + (threadIdx.x >> 5);
  const uint32_t lane = threadIdx.x & 31;
  if (row >= rows) return;
  const T* p = x + static_cast<size_t>(row) * row_len;
  constexpr int V = VecTraits<T>::kPerVec;
  float m = 0.0f;
  const bool aligned = (reinterpret_cast<uintptr_t>(p) & 15u) == 0;
  uint32_t done = 0;
  if (aligned) {
    const uint32_t vecs = row_len / V;
    for (uint32_t v = lane; v < vecs; v += 32) m = max_f32(m, vec_amax<T>(p + static_cast<size_t>(v) * V));
    done = vecs * V;
  }
  for (uint32_t c = done + lane; c < row_len; c += 32) m = max_f32(m, fabsf(load_as_f32<T>(p, c)));
  m = warp_max(m);
  if (lane == 0) out[row] = m;
}

// Block max of per-warp values followed by ONE atomic max per CTA into out[0] (which the
// launcher zeroes first; non-negative floats order like their bit patterns).
__device__ __forceinline__ void cta_atomic_max(float warp_value, float* out) {
  __shared__ float partial[8];
  const uint32_t lane = threadIdx.x & 31, w = threadIdx.x >> 5;
  if (lane == 0) partial[w] = warp_value;
  __syncthreads();
  if (threadIdx.x == 0) {
    float r = 0.0f;
#pragma unroll
    for (int i = 0; i < 8; ++i) r = max_f32(r, partial[i]);
    atomicMax(reinterpret_cast<unsigned int*>(out), __float_as_uint(r));
  }
}

// amax of one full, 16-byte aligned 1024-value chunk, 32 lanes cooperating (result in every lane).
// bf16: the maximum is taken on packed bf16 pairs (exact -- a maximum rounds nothing -- and NaN
// operands are dropped like max.f32 drops them), four instructions per eight values.
template <typename T>
__device__ __forceinline__ float chunk_amax_1024(const T* p, uint32_t lane);
template <>
__device__ __forceinline__ float chunk_amax_1024<float>(const float* p, uint32_t lane) {
  float m = 0.0f;
#pragma unroll
  for (int i = 0; i < 8; ++i) m = max_f32(m, vec_amax<float>(p + (static_cast<size_t>(i) * 32 + lane) * 4));
  return warp_max(m);
}
template <>
__device__ __forceinline__ float chunk_amax_1024<__nv_bfloat16>(const __nv_bfloat16* p, uint32_t lane) {
  uint4 t[4];
#pragma unroll
  for (int i = 0; i < 4; ++i) t[i] = __ldg(reinterpret_cast<const uint4*>(p) + i * 32 + lane);
  __nv_bfloat162 m = __floats2bfloat162_rn(0.0f, 0.0f);
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const uint32_t w[4] = {t[i].x, t[i].y, t[i].z, t[i].w};
#pragma unroll
    for (int j = 0; j < 4; ++j) m = __hmax2(m, __habs2(*reinterpret_cast<const __nv_bfloat162*>(&w[j])));
  }
  return warp_max(max_f32(__low2float(m), __high2float(m)));
}

// Tensor amax: warps stride over 1024-value chunks (chunk amax written when requested).
// utils/nvfp4/quant/kernels/row_amax.rs:67-101.
template <typename T>
__global__ void __launch_bounds__(256) tensor_amax_kernel(const T* __restrict__ x, float* __restrict__ chunk_amax,
                                                           float* __restrict__ out, uint64_t n) {
  const uint32_t lane = threadIdx.x & 31;
  const uint64_t warps = static_cast<uint64_t>(gridDim.x) * 8;
  const uint64_t chunks = (n + 1023) / 1024;
  float running = 0.0f;
  for (uint64_t chunk = static_cast<uint64_t>(blockIdx.x) * 8 + (threadIdx.x >> 5); chunk < chunks; chunk += warps) {
    const uint64_t base = chunk * 1024;
    const T* p = x + base;
    float m = 0.0f;
    if (base + 1024 <= n && (reinterpret_cast<uintptr_t>(p) & 15u) == 0) {
      m = chunk_amax_1024<T>(p, lane);
    } else {
      const uint32_t count = static_cast<uint32_t>(min(static_cast<uint64_t>(1024), n - base));
      for (uint32_t i = lane; i < count; i += 32) m = max_f32(m, fabsf(load_as_f32<T>(p, i)));
      m = warp_max(m);
    }
    if (lane == 0 && chunk_amax) chunk_amax[chunk] = m;
    running = max_f32(running, m);
  }
  cta_atomic_max(running, out);
}

// amax of a decoded NVFP4 tensor [n/cols][cols], warps striding over 1024-value chunks.
// utils/nvfp4/quant/kernels/ms_eden/amax.rs:23-64.  rowwise: one global scale per row;
// packed: the scale bytes are in the packed tile layout.
__global__ void __launch_bounds__(256) nvfp4_amax_kernel(const uint8_t* __restrict__ bytes,
                                                          const uint8_t* __restrict__ scales,
                                                          const float* __restrict__ gscales, uint64_t n, uint32_t cols,
                                                          int rowwise, int packed, float* __restrict__ chunk_amax,
                                                          float* __restrict__ out) {
  const uint32_t lane = threadIdx.x & 31;
  const uint64_t warps = static_cast<uint64_t>(gridDim.x) * 8;
  const uint64_t chunks = (n + 1023) / 1024;
  float running = 0.0f;
  for (uint64_t chunk = static_cast<uint64_t>(blockIdx.x) * 8 + (threadIdx.x >> 5); chunk < chunks; chunk += warps) {
    const uint64_t base = chunk * 1024;
    float m = 0.0f;
    const uint64_t end = min(n, base + 1024);
    // one 16-group (8 bytes, 1 scale) per lane per step
    for (uint64_t g0 = base + lane * 16ull; g0 < end; g0 += 512) {
      const uint32_t srow = static_cast<uint32_t>(g0 / cols);
      const uint32_t skg = static_cast<uint32_t>(g0 - static_cast<uint64_t>(srow) * cols) >> 4;
      const float gs = rowwise ? gscales[srow] : gscales[0];
      const float sc = e4m3_value(packed ? scales[packed_scale_offset(srow, skg, cols >> 6)] : scales[g0 >> 4]);
      const uint2 raw = __ldg(reinterpret_cast<const uint2*>(bytes + (g0 >> 1)));
      // |e2m1| grows with its 3-bit magnitude code and (q * sc) * gs is monotonic in q >= 0, so
      // the group's largest decoded magnitude is that of its largest code: one decode per group
      uint32_t mx = __vmaxu4(__vmaxu4(raw.x & 0x07070707u, (raw.x >> 4) & 0x07070707u),
                             __vmaxu4(raw.y & 0x07070707u, (raw.y >> 4) & 0x07070707u));
      mx = __vmaxu4(mx, mx >> 16);
      mx = __vmaxu4(mx, mx >> 8) & 0x7u;
      m = max_f32(m, fabsf(e2m1_value(mx) * sc * gs));
    }
    m = warp_max(m);
    if (lane == 0 && chunk_amax) chunk_amax[chunk] = m;
    running = max_f32(running, m);
  }
  cta_atomic_max(running, out);
}

// max over chunk values -> out[0] (transform 0) or the MS-EDEN global scale (transform 1).
// utils/nvfp4/quant/kernels/row_amax.rs:86-101, ms_eden/amax.rs:67-104, utils/quartet.rs:6-12.
__global__ void __launch_bounds__(256) amax_from_chunks_kernel(const float* __restrict__ chunk_amax,
                                                                float* __restrict__ out, uint32_t chunk_count,
                                                                int transform) {
  __shared__ float partial[8];
  float m = 0.0f;
  for (uint32_t i = threadIdx.x; i < chunk_count; i += 256) m = max_f32(m, chunk_amax[i]);
  m = warp_max(m);
  if ((threadIdx.x & 31) == 0) partial[threadIdx.x >> 5] = m;
  __syncthreads();
  if (threadIdx.x == 0) {
    float r = 0.0f;
#pragma unroll
    for (int i = 0; i < 8; ++i) r = max_f32(r, partial[i]);
    if (transform == 1) {
      const float so = (17.0f / 16.0f) * 0.93f;
      r = (r == 0.0f) ? 1.0f : r * so / (256.0f * 6.0f);
    }
    out[0] = r;
  }
}

// out[0] = MS-EDEN global scale of amax[0] (single thread).
// utils/quartet.rs:1-12: global scale of an MS-EDEN operand from the amax of its source.
__device__ __forceinline__ float ms_eden_scale_of_amax(float a) {
  const float so = (17.0f / 16.0f) * 0.93f;
  return (a == 0.0f) ? 1.0f : a * so / (256.0f * 6.0f);
}
__global__ void ms_eden_scale_from_amax_kernel(const float* __restrict__ amax, float* __restrict__ out) {
  out[0] = ms_eden_scale_of_amax(amax[0]);
}

// ============================================================================
// four-six
// ============================================================================

__device__ __forceinline__ float four_six_global_scale(float amax) {
  // utils/nvfp4/quant/kernels/four_six/helpers.rs:33-39 with scale_override = 1.0
  return nz(amax == 0.0f ? 1.0f : amax * 1.0f / (256.0f * 6.0f));
}

// Squared quantization error of the group for the 6-anchored (low lane) and the 4-anchored
// (high lane) candidate scale at once: sum of (v - q(v*inv) * (s*gs))^2 in butterfly order
// (utils/nvfp4/quant/kernels/convert.rs:27-35), each lane with its own inv / dequant scale.
// The nibble bytes of both candidates come back too: the winner's bytes are the output.
__device__ __forceinline__ f32x2_t candidate_errors16(const float (&v)[16], float s6, float s4, float gs, uint2& nib6,
                                                      uint2& nib4, float& inv6, float& inv4) {
  inv6 = inv_scale(s6, gs);
  inv4 = inv_scale(s4, gs);
  const f32x2_t inv = pack2(inv6, inv4);
  const f32x2_t dq = pack2(s6 * gs, s4 * gs);
  float x6[16], x4[16];
#pragma unroll
  for (int i = 0; i < 16; ++i) unpack2(mul2(pack2(v[i], v[i]), inv), x6[i], x4[i]);
  nib6 = make_uint2(cvt_e2m1x8(x6[0], x6[1], x6[2], x6[3], x6[4], x6[5], x6[6], x6[7]),
                    cvt_e2m1x8(x6[8], x6[9], x6[10], x6[11], x6[12], x6[13], x6[14], x6[15]));
  nib4 = make_uint2(cvt_e2m1x8(x4[0], x4[1], x4[2], x4[3], x4[4], x4[5], x4[6], x4[7]),
                    cvt_e2m1x8(x4[8], x4[9], x4[10], x4[11], x4[12], x4[13], x4[14], x4[15]));
  float q6a[8], q6b[8], q4a[8], q4b[8];
  e2m1x8_values(nib6.x, q6a);
  e2m1x8_values(nib6.y, q6b);
  e2m1x8_values(nib4.x, q4a);
  e2m1x8_values(nib4.y, q4b);
  f32x2_t a8[8];  // first butterfly level: a8[i] = e[i] + e[i + 8]
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    const f32x2_t d0 = sub2(pack2(v[i], v[i]), mul2_rounded(pack2(q6a[i], q4a[i]), dq));
    const f32x2_t d8 = sub2(pack2(v[i + 8], v[i + 8]), mul2_rounded(pack2(q6b[i], q4b[i]), dq));
    a8[i] = add2(mul2_rounded(d0, d0), mul2_rounded(d8, d8));
  }
  return add2(add2(add2(a8[0], a8[4]), add2(a8[2], a8[6])), add2(add2(a8[1], a8[5]), add2(a8[3], a8[7])));
}

// v: one 16-group.  Returns the scale byte and writes the 8 nibble bytes into `packed`.
// helpers.rs:42-76 and four_six.rs:309-344 of utils/nvfp4/quant/kernels.  The output nibbles
// are cvt(v * inv) with the chosen candidate's inv, i.e. exactly that candidate's trial bytes.
__device__ __forceinline__ uint32_t four_six_group(const float (&v)[16], float gs, uint2& packed,
                                                   float* decoded_amax = nullptr) {
  float ga = 0.0f;
#pragma unroll
  for (int i = 0; i < 16; i += 2) ga = max3_abs(ga, v[i], v[i + 1]);
  const float gsn = nz(gs);
  const uint32_t b6 = cvt_e4m3(ga * 1.0f / (6.0f * gsn + kDenomEps));
  const uint32_t b4 = cvt_e4m3(ga * 1.0f / (4.0f * gsn + kDenomEps));
  const float s6 = e4m3_value(b6);
  const float s4 = e4m3_value(b4);
  float err6, err4, inv6, inv4;
  uint2 nib6, nib4;
  unpack2(candidate_errors16(v, s6, s4, gsn, nib6, nib4, inv6, inv4), err6, err4);
  const bool six = err6 <= err4;
  packed = six ? nib6 : nib4;
  if (decoded_amax) {
    // Largest decoded magnitude of the group, (q * scale) * gs as the stand-alone NVFP4 amax kernel
    // evaluates it (utils/nvfp4/quant/kernels/ms_eden/amax.rs:23-64): rounding to E2M1 is monotonic
    // in |x|, so the largest nibble is the one of the element with the largest magnitude, ga.
    const float q = e2m1x2_values(cvt_e2m1x2(0.0f, ga * (six ? inv6 : inv4))).x;
    *decoded_amax = fabsf(q * (six ? s6 : s4) * gs);
  }
  return six ? b6 : b4;
}

// relu(x)^2 of the values a quantizer has just loaded (the MLP activation computed on load from the stored
// pre-activation): max(x, 0) drops NaN like the reference's max_f32, the square is one rounded multiply.
__device__ __forceinline__ void relu2_inplace16(float (&v)[16]) {
#pragma unroll
  for (int i = 0; i < 16; ++i) {
    const float r = max_f32(v[i], 0.0f);
    v[i] = r * r;
  }
}

// One thread per 16-group of a [rows][cols] tensor.  kRelu2: the tensor quantized is relu(x)^2.
// decoded_amax (optional, zeroed by the launcher): max |decoded value| of the quantized tensor.
template <typename T, bool kRowwise, bool kPacked, bool kRelu2>
__global__ void __launch_bounds__(256) four_six_kernel(const T* __restrict__ x, const float* __restrict__ amax,
                                                        uint8_t* __restrict__ out_fp4, uint8_t* __restrict__ out_scales,
                                                        float* __restrict__ out_gs, float* __restrict__ decoded_amax,
                                                        uint64_t group_count, uint32_t groups_per_row) {
  const uint64_t g = static_cast<uint64_t>(blockIdx.x) * 256 + threadIdx.x;
  float dec = 0.0f;
  if (g < group_count) {
    const uint32_t row = static_cast<uint32_t>(g / groups_per_row);
    const uint32_t kg = static_cast<uint32_t>(g - static_cast<uint64_t>(row) * groups_per_row);
    const float gs = four_six_global_scale(amax[kRowwise ? row : 0]);
    float v[16];
    Load16<T>::run(x + g * 16, v);
    if (kRelu2) relu2_inplace16(v);
    uint2 packed;
    const uint32_t b = four_six_group(v, gs, packed, decoded_amax ? &dec : nullptr);
    *reinterpret_cast<uint2*>(out_fp4 + g * 8) = packed;
    if (kPacked)
      out_scales[packed_scale_offset(row, kg, groups_per_row >> 2)] = static_cast<uint8_t>(b);
    else
      out_scales[g] = static_cast<uint8_t>(b);
    if (kRowwise ? (kg == 0) : (g == 0)) out_gs[kRowwise ? row : 0] = gs;
  }
  if (decoded_amax) cta_atomic_max(warp_max(dec), decoded_amax);  // uniform across the CTA
}

// Row amax and rowwise four-six in ONE pass over the input: a CTA owns whole rows (one thread
// per 16-group), the row amax is the shared-memory max of the group amaxes the quantizer needs
// anyway, and the groups are quantized from registers.  Same bytes as row_amax followed by the
// rowwise kernel (crates/gpt2-nvfp4/src/types/nvfp4_scratch/scratch.rs:35-52 issues those two).
// decoded_amax (optional, zeroed by the launcher): max |decoded value| of the whole quantized
// tensor, i.e. what utils/nvfp4/quant/kernels/ms_eden/amax.rs:23-64 computes from the stored
// tensor before the backward transposer -- handed over so that pass can be skipped.
template <typename T, bool kPacked, bool kRelu2>
__global__ void __launch_bounds__(256) four_six_rowwise_fused_kernel(const T* __restrict__ x,
                                                                      uint8_t* __restrict__ out_fp4,
                                                                      uint8_t* __restrict__ out_scales,
                                                                      float* __restrict__ out_gs,
                                                                      float* __restrict__ out_amax,
                                                                      float* __restrict__ decoded_amax, uint32_t rows,
                                                                      uint32_t groups_per_row, uint32_t rows_per_cta) {
  extern __shared__ unsigned int row_amax_bits[];  // [rows_per_cta] row amax, then one word for the CTA's decoded amax
  const uint32_t t = threadIdx.x;
  for (uint32_t i = t; i <= rows_per_cta; i += blockDim.x) row_amax_bits[i] = 0u;
  __syncthreads();
  const uint32_t local_row = t / groups_per_row;
  const uint32_t kg = t - local_row * groups_per_row;
  const uint32_t row = blockIdx.x * rows_per_cta + local_row;
  const bool active = local_row < rows_per_cta && row < rows;
  float v[16];
  float ga = 0.0f;
  if (active) {
    Load16<T>::run(x + (static_cast<size_t>(row) * groups_per_row + kg) * 16, v);
    if (kRelu2) relu2_inplace16(v);
#pragma unroll
    for (int i = 0; i < 16; i += 2) ga = max3_abs(ga, v[i], v[i + 1]);
  }
  // Row max: non-negative floats order like their bit patterns.  With at least 32 groups per row a
  // warp touches at most two rows, so two warp-wide integer maxima and two shared-memory atomics
  // replace up to 32 atomics on the same word.
  const uint32_t ga_bits = active ? __float_as_uint(ga) : 0u;
  if (groups_per_row >= 32) {
    const uint32_t first_row = __shfl_sync(0xffffffffu, local_row, 0);
    const bool in_first = local_row == first_row;
    const uint32_t m_first = __reduce_max_sync(0xffffffffu, in_first ? ga_bits : 0u);
    const uint32_t m_other = __reduce_max_sync(0xffffffffu, in_first ? 0u : ga_bits);
    const uint32_t other_lanes = __ballot_sync(0xffffffffu, !in_first && active);
    const uint32_t lane_id = t & 31u;
    if (lane_id == 0 && active) atomicMax(&row_amax_bits[local_row], m_first);
    if (other_lanes != 0u && lane_id == static_cast<uint32_t>(__ffs(other_lanes) - 1))
      atomicMax(&row_amax_bits[local_row], m_other);
  } else if (active) {
    atomicMax(&row_amax_bits[local_row], ga_bits);
  }
  __syncthreads();
  uint32_t dec_bits = 0u;
  if (active) {
    const float amax = __uint_as_float(row_amax_bits[local_row]);
    const float gs = four_six_global_scale(amax);
    uint2 packed;
    float dec = 0.0f;
    const uint32_t b = four_six_group(v, gs, packed, decoded_amax ? &dec : nullptr);
    const size_t g = static_cast<size_t>(row) * groups_per_row + kg;
    *reinterpret_cast<uint2*>(out_fp4 + g * 8) = packed;
    if (kPacked)
      out_scales[packed_scale_offset(row, kg, groups_per_row >> 2)] = static_cast<uint8_t>(b);
    else
      out_scales[g] = static_cast<uint8_t>(b);
    if (kg == 0) {
      out_gs[row] = gs;
      if (out_amax) out_amax[row] = amax;
    }
    dec_bits = __float_as_uint(dec);
  }
  if (decoded_amax) {  // uniform across the CTA
    dec_bits = __reduce_max_sync(0xffffffffu, dec_bits);
    if ((t & 31) == 0) atomicMax(&row_amax_bits[rows_per_cta], dec_bits);
    __syncthreads();
    if (t == 0) atomicMax(reinterpret_cast<unsigned int*>(decoded_amax), row_amax_bits[rows_per_cta]);
  }
}

// Raw 16-element group as loaded (two or four 128-bit words) and its widening to f32: kept apart so that
// the next group's words can be in flight while the current one is quantized.
template <typename T>
struct RawGroup;
template <>
struct RawGroup<float> {
  uint4 w[4];
  __device__ __forceinline__ void load(const float* p) {
#pragma unroll
    for (int i = 0; i < 4; ++i) w[i] = __ldg(reinterpret_cast<const uint4*>(p) + i);
  }
  __device__ __forceinline__ void widen(float (&v)[16]) const {
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      v[4 * i] = __uint_as_float(w[i].x);
      v[4 * i + 1] = __uint_as_float(w[i].y);
      v[4 * i + 2] = __uint_as_float(w[i].z);
      v[4 * i + 3] = __uint_as_float(w[i].w);
    }
  }
};
template <>
struct RawGroup<__nv_bfloat16> {
  uint4 w[2];
  __device__ __forceinline__ void load(const __nv_bfloat16* p) {
#pragma unroll
    for (int i = 0; i < 2; ++i) w[i] = __ldg(reinterpret_cast<const uint4*>(p) + i);
  }
  __device__ __forceinline__ void widen(float (&v)[16]) const {
#pragma unroll
    for (int i = 0; i < 2; ++i) {
      const uint32_t t[4] = {w[i].x, w[i].y, w[i].z, w[i].w};
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        v[8 * i + 2 * j] = __uint_as_float(t[j] << 16);
        v[8 * i + 2 * j + 1] = __uint_as_float(t[j] & 0xffff0000u);
      }
    }
  }
};

// The same outputs as four_six_rowwise_fused_kernel from persistent CTAs: a CTA walks row blocks
// blockIdx.x, blockIdx.x + gridDim.x, ... and every thread has the raw words of its next group in flight
// while it quantizes the current one, so global-load latency no longer sits in front of the row-amax
// barrier (one CTA-wide barrier per row block; the per-row maxima rotate through three shared-memory
// buffers so that clearing a buffer is always separated from its next use by a barrier).
constexpr int kStreamMaxRowsPerCta = 256;
template <typename T, bool kPacked, bool kRelu2>
__global__ void __launch_bounds__(256) four_six_rowwise_stream_kernel(const T* __restrict__ x,
                                                                       uint8_t* __restrict__ out_fp4,
                                                                       uint8_t* __restrict__ out_scales,
                                                                       float* __restrict__ out_gs,
                                                                       float* __restrict__ out_amax,
                                                                       float* __restrict__ decoded_amax, uint32_t rows,
                                                                       uint32_t groups_per_row, uint32_t rows_per_cta,
                                                                       uint32_t row_blocks) {
  __shared__ unsigned int row_amax_bits[3][kStreamMaxRowsPerCta];
  const uint32_t t = threadIdx.x, lane_id = t & 31u;
  for (uint32_t i = t; i < 3 * kStreamMaxRowsPerCta; i += blockDim.x) (&row_amax_bits[0][0])[i] = 0u;
  __syncthreads();
  const uint32_t local_row = t / groups_per_row;
  const uint32_t kg = t - local_row * groups_per_row;
  const bool in_use = local_row < rows_per_cta;
  const bool quads = (groups_per_row & 3u) == 0;  // four neighbouring lanes hold four neighbouring scale bytes
  RawGroup<T> raw;
  uint32_t blk = blockIdx.x;
  {
    const uint32_t row = blk * rows_per_cta + local_row;
    if (blk < row_blocks && in_use && row < rows) raw.load(x + (static_cast<size_t>(row) * groups_per_row + kg) * 16);
  }
  float dec_running = 0.0f;
  uint32_t buf = 0;
  for (; blk < row_blocks; blk += gridDim.x) {
    const uint32_t row = blk * rows_per_cta + local_row;
    const bool active = in_use && row < rows;
    float v[16];
    float ga = 0.0f;
    if (active) {
      raw.widen(v);
      if (kRelu2) relu2_inplace16(v);
#pragma unroll
      for (int i = 0; i < 16; i += 2) ga = max3_abs(ga, v[i], v[i + 1]);
    }
    {
      // the next row block's words: in flight across the barrier and the whole quantization below
      const uint32_t nblk = blk + gridDim.x;
      const uint32_t nrow = nblk * rows_per_cta + local_row;
      if (nblk < row_blocks && in_use && nrow < rows) raw.load(x + (static_cast<size_t>(nrow) * groups_per_row + kg) * 16);
    }
    // Row max: non-negative floats order like their bit patterns.  With at least 32 groups per row a warp
    // touches at most two rows: two warp-wide integer maxima and two shared-memory atomics.
    const uint32_t ga_bits = active ? __float_as_uint(ga) : 0u;
    if (groups_per_row >= 32) {
      const uint32_t first_row = __shfl_sync(0xffffffffu, local_row, 0);
      const bool in_first = local_row == first_row;
      const uint32_t m_first = __reduce_max_sync(0xffffffffu, in_first ? ga_bits : 0u);
      const uint32_t m_other = __reduce_max_sync(0xffffffffu, in_first ? 0u : ga_bits);
      const uint32_t other_lanes = __ballot_sync(0xffffffffu, !in_first && active);
      if (lane_id == 0 && active) atomicMax(&row_amax_bits[buf][local_row], m_first);
      if (other_lanes != 0u && lane_id == static_cast<uint32_t>(__ffs(other_lanes) - 1))
        atomicMax(&row_amax_bits[buf][local_row], m_other);
    } else if (active) {
      atomicMax(&row_amax_bits[buf][local_row], ga_bits);
    }
    __syncthreads();
    // every thread is past its reads of the buffer of the previous row block: clear it for the block after next
    const uint32_t stale = buf == 0 ? 2u : buf - 1u;
    if (t < rows_per_cta) row_amax_bits[stale][t] = 0u;
    uint32_t b = 0;
    if (active) {
      const float amax = __uint_as_float(row_amax_bits[buf][local_row]);
      const float gs = four_six_global_scale(amax);
      uint2 packed;
      float dec = 0.0f;
      b = four_six_group(v, gs, packed, decoded_amax ? &dec : nullptr);
      const size_t g = static_cast<size_t>(row) * groups_per_row + kg;
      *reinterpret_cast<uint2*>(out_fp4 + g * 8) = packed;
      if (!quads) {
        if (kPacked)
          out_scales[packed_scale_offset(row, kg, groups_per_row >> 2)] = static_cast<uint8_t>(b);
        else
          out_scales[g] = static_cast<uint8_t>(b);
      }
      if (kg == 0) {
        out_gs[row] = gs;
        if (out_amax) out_amax[row] = amax;
      }
      dec_running = max_f32(dec_running, dec);
    }
    if (quads) {
      // lanes 4j .. 4j+3 hold k-groups 4i .. 4i+3 of one row (one k-atom): one 32-bit store instead of four bytes
      uint32_t word = b | (__shfl_down_sync(0xffffffffu, b, 1) << 8);
      word |= __shfl_down_sync(0xffffffffu, word, 2) << 16;
      if (active && (kg & 3u) == 0) {
        const size_t off = kPacked ? packed_scale_offset(row, kg, groups_per_row >> 2)
                                   : static_cast<size_t>(row) * groups_per_row + kg;
        *reinterpret_cast<uint32_t*>(out_scales + off) = word;
      }
    }
    buf = buf == 2 ? 0u : buf + 1u;
  }
  if (decoded_amax) {  // uniform across the CTA; the CTA may have fewer than eight warps
    __shared__ unsigned int dec_bits;
    if (t == 0) dec_bits = 0u;
    __syncthreads();
    const uint32_t m = __reduce_max_sync(0xffffffffu, __float_as_uint(dec_running));
    if (lane_id == 0) atomicMax(&dec_bits, m);
    __syncthreads();
    if (t == 0) atomicMax(reinterpret_cast<unsigned int*>(decoded_amax), dec_bits);
  }
}

// Schedule-free weight materialisation (gpt/optimizer/schedule_free/{value,amax,four_six}.rs):
// the weight quantized every step is y = z + beta * (x - z) of the two f32 masters; it is never
// written out in f32.  Kernel 1: tensor amax of y (1024-value chunks per warp, chunk amax kept for
// callers that want it); kernel 2: four-six of y with the tensor scale, one thread per 16-group.
__device__ __forceinline__ float schedule_free_value(float z, float x, float beta) { return z + beta * (x - z); }

__global__ void __launch_bounds__(256) schedule_free_amax_kernel(const float* __restrict__ z,
                                                                  const float* __restrict__ x,
                                                                  float* __restrict__ chunk_amax,
                                                                  float* __restrict__ out, float beta, uint64_t n) {
  const uint32_t lane = threadIdx.x & 31;
  const uint64_t warps = static_cast<uint64_t>(gridDim.x) * 8;
  const uint64_t chunks = (n + 1023) / 1024;
  float running = 0.0f;
  for (uint64_t chunk = static_cast<uint64_t>(blockIdx.x) * 8 + (threadIdx.x >> 5); chunk < chunks; chunk += warps) {
    const uint64_t base = chunk * 1024;
    float m = 0.0f;
    if (base + 1024 <= n && ((reinterpret_cast<uintptr_t>(z + base) | reinterpret_cast<uintptr_t>(x + base)) & 15u) == 0) {
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        const float4 a = __ldg(reinterpret_cast<const float4*>(z + base) + i * 32 + lane);
        const float4 b = __ldg(reinterpret_cast<const float4*>(x + base) + i * 32 + lane);
        m = max3_abs(m, schedule_free_value(a.x, b.x, beta), schedule_free_value(a.y, b.y, beta));
        m = max3_abs(m, schedule_free_value(a.z, b.z, beta), schedule_free_value(a.w, b.w, beta));
      }
    } else {
      const uint32_t count = static_cast<uint32_t>(min(static_cast<uint64_t>(1024), n - base));
      for (uint32_t i = lane; i < count; i += 32)
        m = max_f32(m, fabsf(schedule_free_value(__ldg(z + base + i), __ldg(x + base + i), beta)));
    }
    m = warp_max(m);
    if (lane == 0 && chunk_amax) chunk_amax[chunk] = m;
    running = max_f32(running, m);
  }
  cta_atomic_max(running, out);
}

template <bool kPacked>
__global__ void __launch_bounds__(256) schedule_free_four_six_kernel(const float* __restrict__ z,
                                                                      const float* __restrict__ x,
                                                                      const float* __restrict__ amax,
                                                                      uint8_t* __restrict__ out_fp4,
                                                                      uint8_t* __restrict__ out_scales,
                                                                      float* __restrict__ out_gs, float beta,
                                                                      uint64_t group_count, uint32_t groups_per_row) {
  const uint64_t g = static_cast<uint64_t>(blockIdx.x) * 256 + threadIdx.x;
  if (g >= group_count) return;
  const float gs = four_six_global_scale(amax[0]);
  float zv[16], xv[16], v[16];
  Load16<float>::run(z + g * 16, zv);
  Load16<float>::run(x + g * 16, xv);
#pragma unroll
  for (int i = 0; i < 16; ++i) v[i] = schedule_free_value(zv[i], xv[i], beta);
  uint2 packed;
  const uint32_t b = four_six_group(v, gs, packed);
  *reinterpret_cast<uint2*>(out_fp4 + g * 8) = packed;
  if (kPacked) {
    const uint32_t row = static_cast<uint32_t>(g / groups_per_row);
    const uint32_t kg = static_cast<uint32_t>(g - static_cast<uint64_t>(row) * groups_per_row);
    out_scales[packed_scale_offset(row, kg, groups_per_row >> 2)] = static_cast<uint8_t>(b);
  } else {
    out_scales[g] = static_cast<uint8_t>(b);
  }
  if (g == 0) out_gs[0] = gs;
}

// Padded / transposed-padded variants: generic gather, zero outside the source extent.
// utils/nvfp4/quant/kernels/four_six.rs:110-142,173-211,346-395.
template <bool kTransposed>
__global__ void __launch_bounds__(256)
    four_six_padded_kernel(const float* __restrict__ x, const float* __restrict__ amax, uint8_t* __restrict__ out_fp4,
                           uint8_t* __restrict__ out_scales, float* __restrict__ out_gs, uint32_t rows, uint32_t cols,
                           uint32_t padded_cols, uint64_t group_count) {
  const uint64_t g = static_cast<uint64_t>(blockIdx.x) * 256 + threadIdx.x;
  if (g >= group_count) return;
  const float gs = four_six_global_scale(amax[0]);
  float v[16];
#pragma unroll
  for (int i = 0; i < 16; ++i) {
    const uint64_t idx = g * 16 + i;
    const uint32_t r = static_cast<uint32_t>(idx / padded_cols);
    const uint32_t c = static_cast<uint32_t>(idx - static_cast<uint64_t>(r) * padded_cols);
    if (!kTransposed)
      v[i] = (r < rows && c < cols) ? x[static_cast<size_t>(r) * cols + c] : 0.0f;
    else
      v[i] = (r < cols && c < rows) ? x[static_cast<size_t>(c) * cols + r] : 0.0f;
  }
  uint2 packed;
  const uint32_t b = four_six_group(v, gs, packed);
  *reinterpret_cast<uint2*>(out_fp4 + g * 8) = packed;
  out_scales[g] = static_cast<uint8_t>(b);
  if (g == 0) out_gs[0] = gs;
}

// Fills the pad rows [rows, padded_rows) of a packed scale plane with 0x38 (= 1.0).
__global__ void __launch_bounds__(256) packed_scale_pad_kernel(uint8_t* __restrict__ packed, uint32_t rows,
                                                                uint32_t padded_rows, uint32_t k_groups) {
  const uint64_t total = static_cast<uint64_t>(padded_rows - rows) * k_groups;
  for (uint64_t i = static_cast<uint64_t>(blockIdx.x) * 256 + threadIdx.x; i < total;
       i += static_cast<uint64_t>(gridDim.x) * 256) {
    const uint32_t r = rows + static_cast<uint32_t>(i / k_groups);
    const uint32_t kg = static_cast<uint32_t>(i % k_groups);
    packed[packed_scale_offset(r, kg, k_groups >> 2)] = 0x38;
  }
}

// ============================================================================
// MS-EDEN
// ============================================================================

// nz(decode(encode_e4m3(v))) for v >= 0: the value of the nearest E4M3 code (ties to the even
// code, saturating at 448), with zero mapped to one.  Inside the normal range [2^-6, 448) this is
// a round-to-nearest-even of the f32 mantissa at bit 20 and never zero (checked against the CPU
// restatement for every seventh f32 in the range); outside it the conversions are used.
__device__ __forceinline__ float e4m3_rounded_value_nz(float v) {
  const uint32_t bits = __float_as_uint(v);
  if (bits - 0x3c800000u < 0x43e00000u - 0x3c800000u)
    return __uint_as_float((bits + 0x0007ffffu + ((bits >> 20) & 1u)) & 0xfff00000u);
  return nz(e4m3_value(cvt_e4m3(v)));
}

// pack/scale.rs:7-30 of utils/nvfp4/quant/kernels/ms_eden.
__device__ __forceinline__ uint32_t stochastic_e4m3_scale(float value, uint32_t seed, uint32_t group) {
  // Values inside the normal E4M3 range [2^-6, 448) -- every block scale of a tensor whose groups
  // are within 2^14 of its amax -- need no conversions at all: the lower neighbour keeps the top
  // three mantissa bits, its code is (exponent, those bits) rebased, the upper neighbour is the
  // next code, and p = (value - down) / (up - down) is exactly the low 20 mantissa bits / 2^20.
  // The draw is 24 hash bits / 2^24, so `draw < p` is an integer comparison.  Identical to the
  // general path below for every value in the range (checked against the CPU restatement over
  // 7.7 million values including every grid point and its neighbours).
  const uint32_t vbits = __float_as_uint(value);
  if (vbits - 0x3c800000u < 0x43e00000u - 0x3c800000u) {
    const uint32_t draw = hash_u32(seed ^ group) & 0x00ffffffu;
    return (vbits >> 20) - 960u + (draw < ((vbits & 0x000fffffu) << 4) ? 1u : 0u);
  }
  const uint32_t cb = cvt_e4m3(value);
  const float cur = e4m3_value(cb);
  const bool above = cur > value;
  // Only the neighbour on the far side of `value` is needed: the code below when the nearest
  // code lies above the value, the code above otherwise (clamped like the reference's prev / next).
  const uint32_t ob = above ? (cb == 0 ? 0u : cb - 1u) : (cb == 255u ? 255u : cb + 1u);
  const float other = e4m3_value(ob);
  const float up = above ? cur : other;
  const float down = above ? other : cur;
  const uint32_t up_bits = above ? cb : ob;
  const uint32_t down_bits = above ? ob : cb;
  // p = (value - down) / (up - down).  Two E4M3 codes one step apart differ by +-2^e with
  // -9 <= e <= 5 unless one of them is the NaN code or the step was clamped, so the difference is
  // a power of two, zero or NaN.  For a power of two the quotient equals the product with the
  // exact reciprocal (both round the same real number); for zero the reference takes p = 0 and
  // for NaN the quotient is NaN: either way the draw is not below p and the lower code is kept.
  const uint32_t dbits = __float_as_uint(up - down);
  const uint32_t mag = dbits & 0x7fffffffu;
  const bool pow2 = (mag & 0x007fffffu) == 0u && mag - 0x00800000u <= 0x7e000000u - 0x00800000u;
  const float p = (value - down) * __uint_as_float((0x7f000000u - mag) | (dbits & 0x80000000u));
  return (pow2 && random_unit_f32(seed, group) < p) ? up_bits : down_bits;
}

// a / b by the IEEE division instruction, issued unconditionally (the compiler would otherwise
// wrap it in a branch where its result is selected away, and a branch per group costs more
// than the quotient).
__device__ __forceinline__ float div_rn_always(float a, float b) {
  float r;
  asm volatile("div.rn.f32 %0, %1, %2;" : "=f"(r) : "f"(a), "f"(b));
  return r;
}

// In-register 32-point Walsh-Hadamard butterfly in the reference's order
// (pack/hadamard.rs:6-19): stride 1,2,4,8,16; low lane a+b, high lane a-b; then * 1/sqrt(32).
// The chunk is held as 16 packed pairs P[i] = (u[i], u[i+16]): strides 1..8 act between
// registers on both halves at once (packed add / sub), stride 16 inside each register.
__device__ __forceinline__ void hadamard32_x2(f32x2_t (&P)[16]) {
#pragma unroll
  for (int stride = 1; stride < 16; stride <<= 1) {
#pragma unroll
    for (int i = 0; i < 16; ++i) {
      if ((i & stride) == 0) {
        const f32x2_t a = P[i], b = P[i | stride];
        P[i] = add2(a, b);
        P[i | stride] = sub2(a, b);
      }
    }
  }
  const f32x2_t c = pack2(0.17677669f, 0.17677669f);
#pragma unroll
  for (int i = 0; i < 16; ++i) {
    float lo, hi;
    unpack2(P[i], lo, hi);
    P[i] = mul2(pack2(lo + hi, lo - hi), c);  // after this: low lane = group 0, high lane = group 1
  }
}

// Two rotated 16-groups at once, one per packed lane (they may belong to one chunk or to two
// different chunks): block scale, RTN nibbles, EDEN correction and the stochastic scale byte
// of each (pack/payload.rs:15-69).  H points at the 16 packed values.  Returns the two scale
// bytes (low lane in bits 0..7) and the 8 nibble bytes of each lane.
__device__ __forceinline__ uint32_t ms_eden_group_lanes(const f32x2_t* H, float safe_gs, float so, float inv6,
                                                        uint32_t scale_seed, uint32_t group_lo, uint32_t group_hi,
                                                        uint2& nib_lo, uint2& nib_hi) {
  float ga0 = 0.0f, ga1 = 0.0f;
#pragma unroll
  for (int i = 0; i < 16; i += 2) {
    float a0, a1, b0, b1;
    unpack2(H[i], a0, a1);
    unpack2(H[i + 1], b0, b1);
    ga0 = max3_abs(ga0, a0, b0);
    ga1 = max3_abs(ga1, a1, b1);
  }
  const float s0a = e4m3_rounded_value_nz(ga0 * so * inv6);
  const float s0b = e4m3_rounded_value_nz(ga1 * so * inv6);
  const f32x2_t inv = pack2(inv_scale(s0a, safe_gs), inv_scale(s0b, safe_gs));
  f32x2_t x[16];
  float xa[16], xb[16];
#pragma unroll
  for (int i = 0; i < 16; ++i) {
    x[i] = mul2(H[i], inv);
    unpack2(x[i], xa[i], xb[i]);
  }
  nib_lo = make_uint2(cvt_e2m1x8(xa[0], xa[1], xa[2], xa[3], xa[4], xa[5], xa[6], xa[7]),
                      cvt_e2m1x8(xa[8], xa[9], xa[10], xa[11], xa[12], xa[13], xa[14], xa[15]));
  nib_hi = make_uint2(cvt_e2m1x8(xb[0], xb[1], xb[2], xb[3], xb[4], xb[5], xb[6], xb[7]),
                      cvt_e2m1x8(xb[8], xb[9], xb[10], xb[11], xb[12], xb[13], xb[14], xb[15]));
  float qa0[8], qa1[8], qb0[8], qb1[8];  // decoded nibbles: lane a / b, elements 0..7 / 8..15
  e2m1x8_values(nib_lo.x, qa0);
  e2m1x8_values(nib_lo.y, qa1);
  e2m1x8_values(nib_hi.x, qb0);
  e2m1x8_values(nib_hi.y, qb1);
  // first level of the xor-8 butterfly sums formed on the spot: entry i = e[i] + e[i + 8]
  f32x2_t num8[8], den8[8];
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    num8[i] = add2(mul2_rounded(x[i], x[i]), mul2_rounded(x[i + 8], x[i + 8]));
    den8[i] = add2(mul2_rounded(x[i], pack2(qa0[i], qb0[i])), mul2_rounded(x[i + 8], pack2(qa1[i], qb1[i])));
  }
  float num_a, num_b, den_a, den_b;
  unpack2(add2(add2(add2(num8[0], num8[4]), add2(num8[2], num8[6])), add2(add2(num8[1], num8[5]), add2(num8[3], num8[7]))),
          num_a, num_b);
  unpack2(add2(add2(add2(den8[0], den8[4]), add2(den8[2], den8[6])), add2(add2(den8[1], den8[5]), add2(den8[3], den8[7]))),
          den_a, den_b);
  const float qa = div_rn_always(num_a, den_a), qb = div_rn_always(num_b, den_b);
  const float sa = nz(s0a * (den_a == 0.0f ? 1.0f : qa));
  const float sb = nz(s0b * (den_b == 0.0f ? 1.0f : qb));
  return stochastic_e4m3_scale(sa, scale_seed, group_lo) | (stochastic_e4m3_scale(sb, scale_seed, group_hi) << 8);
}

// Both 16-groups of one rotated chunk (low lane = group 0, high lane = group 1).
__device__ __forceinline__ uint32_t ms_eden_groups_x2(const f32x2_t (&H)[16], float safe_gs, float so, float inv6,
                                                      uint32_t scale_seed, uint32_t group0, uint4& packed) {
  uint2 lo, hi;
  const uint32_t sb = ms_eden_group_lanes(&H[0], safe_gs, so, inv6, scale_seed, group0, group0 + 1, lo, hi);
  packed = make_uint4(lo.x, lo.y, hi.x, hi.y);
  return sb;
}

// Where one orientation of an MS-EDEN result goes.
struct MsEdenOut {
  uint8_t* fp4;
  uint8_t* scales;
  float* global_scales;
  float* chunk_amax;      // optional
  uint32_t rows;          // valid output rows
  uint32_t dst_row_len;   // output K (multiple of 32)
  uint32_t scale_seed;
  uint32_t group_offset;  // added to the flat group id of the scale RNG
  uint32_t group_row_stride;  // 16-groups per row in the scale RNG's index space (dst_row_len / 16 unless sharded)
  uint32_t sign_offset;   // added to the K index of the sign hash
  int packed;             // scale bytes in the packed tile layout
};

struct MsEdenParams {
  const void* x;
  const uint8_t* src_bytes;
  const uint8_t* src_scales;
  const float* src_global;
  int src_packed;  // NVFP4 sources: scale bytes in the packed tile layout
  uint32_t a;      // F32_ROWS: src_row_len; transposed kinds: source_rows
  uint32_t b;      // transposed kinds: source_cols
  const float* global_scale_dev;
  float global_scale_host;
  int use_host_scale;
  float scale_override;
  uint32_t sign_seed;
  MsEdenOut out;
};

// Finishes one chunk whose signed inputs are in P (P[i] = (u[i], u[i+16])): rotation, two
// groups, stores.
__device__ __forceinline__ void ms_eden_emit_chunk(f32x2_t (&P)[16], const MsEdenOut& o, float gs, float so,
                                                   uint32_t row, uint32_t chunk_in_row) {
  const uint64_t chunk = static_cast<uint64_t>(row) * (o.dst_row_len >> 5) + chunk_in_row;
  hadamard32_x2(P);
  if (o.chunk_amax) {
    float m = 0.0f;
#pragma unroll
    for (int i = 0; i < 16; ++i) {
      float lo, hi;
      unpack2(P[i], lo, hi);
      m = max3_abs(m, lo, hi);
    }
    o.chunk_amax[chunk] = m;
  }
  const float safe_gs = nz(gs);
  const float inv6 = inv_scale(6.0f, safe_gs);
  const uint32_t group0 = row * o.group_row_stride + chunk_in_row * 2u + o.group_offset;
  uint4 nibbles;
  const uint32_t sb = ms_eden_groups_x2(P, safe_gs, so, inv6, o.scale_seed, group0, nibbles);
  *reinterpret_cast<uint4*>(o.fp4 + chunk * 16) = nibbles;
  // two consecutive k-groups of one k-atom: adjacent bytes in either layout, 2-byte aligned
  const size_t off = o.packed ? packed_scale_offset(row, chunk_in_row * 2, o.dst_row_len >> 6) : chunk * 2;
  *reinterpret_cast<uint16_t*>(o.scales + off) = static_cast<uint16_t>(sb);
  if (chunk_in_row == 0) o.global_scales[row] = gs;
}

// Two chunks at once, one per packed lane (low lane = chunk of row_lo, high lane = chunk of
// row_hi, both at chunk_in_row): P[k] holds the signed inputs of K position k of both, so all
// five butterfly strides act between registers.
__device__ __forceinline__ void ms_eden_emit_chunk_lanes(f32x2_t (&P)[32], const MsEdenOut& o, float gs, float so,
                                                         uint32_t row_lo, uint32_t row_hi, uint32_t chunk_in_row) {
  const uint32_t chunks_per_row = o.dst_row_len >> 5;
  const uint64_t chunk_lo = static_cast<uint64_t>(row_lo) * chunks_per_row + chunk_in_row;
  const uint64_t chunk_hi = static_cast<uint64_t>(row_hi) * chunks_per_row + chunk_in_row;
#pragma unroll
  for (int stride = 1; stride < 32; stride <<= 1) {
#pragma unroll
    for (int i = 0; i < 32; ++i) {
      if ((i & stride) == 0) {
        const f32x2_t a = P[i], b = P[i | stride];
        P[i] = add2(a, b);
        P[i | stride] = sub2(a, b);
      }
    }
  }
  const f32x2_t c = pack2(0.17677669f, 0.17677669f);
#pragma unroll
  for (int i = 0; i < 32; ++i) P[i] = mul2(P[i], c);
  if (o.chunk_amax) {
    float m_lo = 0.0f, m_hi = 0.0f;
#pragma unroll
    for (int i = 0; i < 32; i += 2) {
      float a0, a1, b0, b1;
      unpack2(P[i], a0, a1);
      unpack2(P[i + 1], b0, b1);
      m_lo = max3_abs(m_lo, a0, b0);
      m_hi = max3_abs(m_hi, a1, b1);
    }
    o.chunk_amax[chunk_lo] = m_lo;
    o.chunk_amax[chunk_hi] = m_hi;
  }
  const float safe_gs = nz(gs);
  const float inv6 = inv_scale(6.0f, safe_gs);
  const uint32_t g_lo = row_lo * o.group_row_stride + chunk_in_row * 2u + o.group_offset;
  const uint32_t g_hi = row_hi * o.group_row_stride + chunk_in_row * 2u + o.group_offset;
  uint2 lo0, hi0, lo1, hi1;
  const uint32_t sb0 = ms_eden_group_lanes(&P[0], safe_gs, so, inv6, o.scale_seed, g_lo, g_hi, lo0, hi0);
  const uint32_t sb1 = ms_eden_group_lanes(&P[16], safe_gs, so, inv6, o.scale_seed, g_lo + 1, g_hi + 1, lo1, hi1);
  *reinterpret_cast<uint4*>(o.fp4 + chunk_lo * 16) = make_uint4(lo0.x, lo0.y, lo1.x, lo1.y);
  *reinterpret_cast<uint4*>(o.fp4 + chunk_hi * 16) = make_uint4(hi0.x, hi0.y, hi1.x, hi1.y);
  const uint32_t k_atoms = o.dst_row_len >> 6;
  const size_t off_lo = o.packed ? packed_scale_offset(row_lo, chunk_in_row * 2, k_atoms) : chunk_lo * 2;
  const size_t off_hi = o.packed ? packed_scale_offset(row_hi, chunk_in_row * 2, k_atoms) : chunk_hi * 2;
  *reinterpret_cast<uint16_t*>(o.scales + off_lo) = static_cast<uint16_t>((sb0 & 0xffu) | ((sb1 & 0xffu) << 8));
  *reinterpret_cast<uint16_t*>(o.scales + off_hi) = static_cast<uint16_t>(((sb0 >> 8) & 0xffu) | (sb1 & 0xff00u));
  if (chunk_in_row == 0) {
    o.global_scales[row_lo] = gs;
    o.global_scales[row_hi] = gs;
  }
}

// Signed input pair (u[i], u[i+16]) from two values and the chunk's 32 sign bits.
__device__ __forceinline__ f32x2_t signed_pair(float lo, float hi, uint32_t neg_mask, int i) {
  const uint32_t a = __float_as_uint(lo) ^ ((neg_mask << (31 - i)) & 0x80000000u);
  const uint32_t b = __float_as_uint(hi) ^ ((neg_mask << (15 - i)) & 0x80000000u);
  return pack2(__uint_as_float(a), __uint_as_float(b));
}

// Generic one-thread-per-chunk kernel (row sources, and the fallback for odd transposed
// shapes).  Input gathers follow utils/nvfp4/quant/kernels/ms_eden/input/padded.rs:9-96.
template <int kKind, typename T>
__global__ void __launch_bounds__(128) ms_eden_kernel(const MsEdenParams p) {
  const uint32_t chunks_per_row = p.out.dst_row_len >> 5;
  const uint64_t chunk_count = static_cast<uint64_t>(p.out.rows) * chunks_per_row;
  const uint64_t chunk = static_cast<uint64_t>(blockIdx.x) * 128 + threadIdx.x;
  if (chunk >= chunk_count) return;
  const uint32_t row = static_cast<uint32_t>(chunk / chunks_per_row);
  const uint32_t chunk_in_row = static_cast<uint32_t>(chunk - static_cast<uint64_t>(row) * chunks_per_row);
  const uint32_t col0 = chunk_in_row * 32;
  const float gs = p.use_host_scale ? p.global_scale_host : p.global_scale_dev[0];
  float u[32];
  if (kKind == 0) {
    const T* x = static_cast<const T*>(p.x) + static_cast<size_t>(row) * p.a;
    const bool full = col0 + 32 <= p.a && ((reinterpret_cast<uintptr_t>(x + col0) & 15u) == 0);
    if (full) {
      float lo[16], hi[16];
      Load16<T>::run(x + col0, lo);
      Load16<T>::run(x + col0 + 16, hi);
#pragma unroll
      for (int j = 0; j < 16; ++j) {
        u[j] = lo[j];
        u[16 + j] = hi[j];
      }
    } else {
#pragma unroll
      for (int j = 0; j < 32; ++j) u[j] = (col0 + j < p.a) ? load_as_f32<T>(x, col0 + j) : 0.0f;
    }
  } else if (kKind == 1) {
    const T* x = static_cast<const T*>(p.x);
#pragma unroll
    for (int j = 0; j < 32; ++j) {
      const uint32_t c = col0 + j;
      u[j] = (c < p.a) ? load_as_f32<T>(x, static_cast<size_t>(c) * p.b + row) : 0.0f;
    }
  } else {
#pragma unroll
    for (int j = 0; j < 32; ++j) {
      const uint32_t c = col0 + j;
      if (c < p.a) {
        const float sg = (kKind == 2) ? p.src_global[0] : p.src_global[c];
        const size_t index = static_cast<size_t>(c) * p.b + row;
        const uint32_t byte = p.src_bytes[index >> 1];
        const uint32_t nib = (index & 1) ? (byte >> 4) : (byte & 0xfu);
        const size_t sidx = p.src_packed ? packed_scale_offset(c, row >> 4, p.b >> 6) : (index >> 4);
        u[j] = e2m1_value(nib) * e4m3_value(p.src_scales[sidx]) * sg;
      } else {
        u[j] = 0.0f;
      }
    }
  }
  uint32_t neg_mask = 0;  // x * (-1) == -x exactly: the random signs are applied as sign-bit flips
#pragma unroll
  for (int j = 0; j < 32; ++j)
    neg_mask |= (random_sign_negative(p.sign_seed, col0 + j + p.out.sign_offset) ? 1u : 0u) << j;
  f32x2_t P[16];
#pragma unroll
  for (int i = 0; i < 16; ++i) P[i] = signed_pair(u[i], u[i + 16], neg_mask, i);
  ms_eden_emit_chunk(P, p.out, gs, p.scale_override, row, chunk_in_row);
}

// Tiled kernel for the transposed operands.  A CTA stages a [128 source rows x 64 source
// columns] tile in shared memory with coalesced 128-bit loads (decoding NVFP4 sources on the
// way), then each thread takes one 32-chunk DOWN a column (the transposed operand, K = source
// row) and, in pair mode, one 32-chunk ALONG a row (the row operand, K = source column): the
// source is read from memory once for both orientations, where the reference reads it twice
// and gathers the transposed half with a row-pitch stride
// (utils/nvfp4/quant/kernels/ms_eden/fp32_pair/dispatch.rs:13-43, input/padded.rs:9-96).
struct MsEdenTileParams {
  const void* x;
  const uint8_t* src_bytes;
  const uint8_t* src_scales;
  const float* src_global;
  int src_packed;
  uint32_t src_rows, src_cols;
  const float* global_scale_dev;
  float global_scale_host;
  int use_host_scale;
  float scale_override;
  uint32_t sign_seed;
  MsEdenOut t;  // transposed operand: rows = src_cols, K = src_rows (padded)
  MsEdenOut r;  // row operand (pair mode): rows = src_rows, K = src_cols (padded)
  float* col_sum_partials;  // pair mode, optional: [row tiles][src_cols] column sums of each tile
  // whole-tile pair kernel, optional: take the global scale from the source amax (every thread
  // evaluates the same two operations) and publish it, instead of a one-thread kernel in between
  const float* amax_in;
  float* gs_out;
};

constexpr int kTileRows = 128, kTileCols = 64, kTileLd = kTileCols + 1;

template <int kSrc, typename T, bool kPair>
__global__ void __launch_bounds__(256) ms_eden_tile_kernel(const MsEdenTileParams p) {
  __shared__ float tile[kTileRows * kTileLd];
  __shared__ uint32_t neg_r[kTileRows / 32];  // sign bits of the tile's rows (K of the transposed operand)
  __shared__ uint32_t neg_c[kTileCols / 32];  // sign bits of the tile's columns (K of the row operand)
  const uint32_t tid = threadIdx.x;
  const uint32_t c0 = blockIdx.x * kTileCols, r0 = blockIdx.y * kTileRows;
  if (tid < kTileRows) {
    const uint32_t bits = __ballot_sync(0xffffffffu, random_sign_negative(p.sign_seed, r0 + tid + p.t.sign_offset));
    if ((tid & 31) == 0) neg_r[tid >> 5] = bits;
  } else if (kPair && tid < kTileRows + kTileCols) {
    const uint32_t bits =
        __ballot_sync(0xffffffffu, random_sign_negative(p.sign_seed, c0 + (tid - kTileRows) + p.r.sign_offset));
    if ((tid & 31) == 0) neg_c[(tid - kTileRows) >> 5] = bits;
  }

  if (kSrc == 0) {
    const T* x = static_cast<const T*>(p.x);
    constexpr int V = VecTraits<T>::kPerVec;
    constexpr int kVecPerRow = kTileCols / V;
    const bool vec_ok = (p.src_cols % V == 0) && ((reinterpret_cast<uintptr_t>(x) & 15u) == 0) &&
                        (c0 + kTileCols <= p.src_cols);
    for (uint32_t i = tid; i < kTileRows * kVecPerRow; i += 256) {
      const uint32_t row = i / kVecPerRow, v = i % kVecPerRow;
      const uint32_t r = r0 + row;
      float vals[V];
#pragma unroll
      for (int k = 0; k < V; ++k) vals[k] = 0.0f;
      if (r < p.src_rows) {
        const T* src = x + static_cast<size_t>(r) * p.src_cols + c0 + v * V;
        if (vec_ok) {
          if (V == 4) {
            const float4 t = __ldg(reinterpret_cast<const float4*>(src));
            vals[0] = t.x, vals[1] = t.y, vals[2] = t.z, vals[3] = t.w;
          } else {
            const uint4 t = __ldg(reinterpret_cast<const uint4*>(src));
            const uint32_t w[4] = {t.x, t.y, t.z, t.w};
#pragma unroll
            for (int k = 0; k < 4; ++k) {
              vals[(2 * k) % V] = __uint_as_float(w[k] << 16);
              vals[(2 * k + 1) % V] = __uint_as_float(w[k] & 0xffff0000u);
            }
          }
        } else {
#pragma unroll
          for (int k = 0; k < V; ++k)
            if (c0 + v * V + k < p.src_cols) vals[k] = load_as_f32<T>(src, k);
        }
      }
#pragma unroll
      for (int k = 0; k < V; ++k) tile[row * kTileLd + v * V + k] = vals[k];
    }
  } else {
    // NVFP4 source: per row of the tile 32 nibble bytes and 4 scale bytes; two threads per row
    const uint32_t row = tid >> 1, half = tid & 1;
    const uint32_t r = r0 + row, c = c0 + half * 32;
    float vals[32];
#pragma unroll
    for (int k = 0; k < 32; ++k) vals[k] = 0.0f;
    if (r < p.src_rows) {
      const float sg = kSrc == 2 ? p.src_global[0] : p.src_global[r];
      const size_t index = static_cast<size_t>(r) * p.src_cols + c;
#pragma unroll
      for (int g = 0; g < 2; ++g) {
        if (c + 16 * g < p.src_cols) {
          const uint2 raw = __ldg(reinterpret_cast<const uint2*>(p.src_bytes + ((index + 16 * g) >> 1)));
          const size_t sidx = p.src_packed ? packed_scale_offset(r, (c >> 4) + g, p.src_cols >> 6) : (index >> 4) + g;
          const float sc = e4m3_value(p.src_scales[sidx]);
          const uint32_t w[2] = {raw.x, raw.y};
#pragma unroll
          for (int j = 0; j < 8; ++j) {
            const float2 q = e2m1x2_values((w[j >> 2] >> (8 * (j & 3))) & 0xffu);
            vals[16 * g + 2 * j] = q.x * sc * sg;
            vals[16 * g + 2 * j + 1] = q.y * sc * sg;
          }
        }
      }
    }
#pragma unroll
    for (int k = 0; k < 32; ++k) tile[row * kTileLd + half * 32 + k] = vals[k];
  }
  __syncthreads();

  if (kPair && p.col_sum_partials) {
    // Column sums of this tile (the bias gradient's partial sums), in a fixed order: four
    // sequential 32-row sums per column, then ((q0 + q1) + q2) + q3.
    __shared__ float quarter_sum[4][kTileCols];
    const uint32_t c = tid & 63, quarter = tid >> 6;
    float acc = 0.0f;
#pragma unroll 8
    for (int j = 0; j < 32; ++j) acc += tile[(quarter * 32 + j) * kTileLd + c];
    quarter_sum[quarter][c] = acc;
    __syncthreads();
    if (tid < kTileCols && c0 + tid < p.src_cols)
      p.col_sum_partials[static_cast<size_t>(blockIdx.y) * p.src_cols + c0 + tid] =
          ((quarter_sum[0][tid] + quarter_sum[1][tid]) + quarter_sum[2][tid]) + quarter_sum[3][tid];
  }

  const float gs = p.use_host_scale ? p.global_scale_host : p.global_scale_dev[0];
  {
    const uint32_t c = tid & 63, chunk = tid >> 6;
    const uint32_t out_row = c0 + c, k0 = r0 + chunk * 32;
    if (out_row < p.t.rows && k0 < p.t.dst_row_len) {
      const uint32_t mask = neg_r[chunk];
      f32x2_t P[16];
#pragma unroll
      for (int i = 0; i < 16; ++i)
        P[i] = signed_pair(tile[(chunk * 32 + i) * kTileLd + c], tile[(chunk * 32 + i + 16) * kTileLd + c], mask, i);
      ms_eden_emit_chunk(P, p.t, gs, p.scale_override, out_row, k0 >> 5);
    }
  }
  if (kPair) {
    const uint32_t row = tid >> 1, chunk = tid & 1;
    const uint32_t out_row = r0 + row, k0 = c0 + chunk * 32;
    if (out_row < p.r.rows && k0 < p.r.dst_row_len) {
      const uint32_t mask = neg_c[chunk];
      f32x2_t P[16];
#pragma unroll
      for (int i = 0; i < 16; ++i)
        P[i] = signed_pair(tile[row * kTileLd + chunk * 32 + i], tile[row * kTileLd + chunk * 32 + i + 16], mask, i);
      ms_eden_emit_chunk(P, p.r, gs, p.scale_override, out_row, k0 >> 5);
    }
  }
}

// Pair kernel for sources whose extents are whole tiles (rows % 128 == 0, cols % 64 == 0):
// the same outputs as ms_eden_tile_kernel<0, T, true>, organised for instruction count.
//  * Persistent CTAs walk the tiles; the next tile's 128 x 128-byte rows arrive through
//    cp.async into the other shared-memory stage while the current one is being quantized.
//    The tile stays bf16; the 144-byte row pitch makes all three access patterns conflict-free.
//  * Every thread quantizes TWO chunks at once, one per f32x2 lane, chosen so that both lanes
//    share their K positions: warps 0-3 take two adjacent source columns down 32 rows (the
//    transposed operand), warps 4-7 take rows r and r+32 along 32 columns (the row operand).
//    One 32-bit shared load then feeds both lanes, the random signs are one xor on the raw
//    bf16 pair, and all five Hadamard strides are packed register-to-register operations.
constexpr int kPairPitch = 144;                          // bytes per staged row
constexpr int kPairStageBytes = kTileRows * kPairPitch;  // 18432

__device__ __forceinline__ void cp_async_16(uint32_t smem_addr, const void* gmem) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(smem_addr), "l"(gmem) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
__device__ __forceinline__ void cp_async_wait_all_but_one() { asm volatile("cp.async.wait_group 1;" ::: "memory"); }

// f32 sources use the same kernel with a [128 x 64] f32 tile (272-byte pitch, dynamic shared
// memory): a 64-bit load is the two lanes of the transposed role, two 32-bit values of rows r and
// r + 32 those of the row role, and the signs are xors on the f32 sign bits.
template <typename T>
struct PairTile {
  static constexpr bool kBf16 = sizeof(T) == 2;
  static constexpr int kPitch = kBf16 ? kPairPitch : kTileCols * 4 + 16;  // bytes per staged row
  static constexpr int kStageBytes = kTileRows * kPitch;
  static constexpr int kPiecesPerRow = kTileCols * static_cast<int>(sizeof(T)) / 16;
  static constexpr int kPiecesPerThread = kTileRows * kPiecesPerRow / 256;
};

template <typename T>
__global__ void __launch_bounds__(256, 2) ms_eden_pair_kernel(const MsEdenTileParams p, uint32_t tiles_x,
                                                               uint32_t tile_count) {
  using PT = PairTile<T>;
  constexpr bool kBf16 = PT::kBf16;
  extern __shared__ __align__(16) uint8_t pair_stage[];       // [2][PT::kStageBytes]
  __shared__ __align__(16) uint32_t flip_row[kTileRows];      // sign-bit mask of the row (both bf16 halves)
  __shared__ __align__(16) uint32_t flip_col[kTileCols];      // bf16: per column pair; f32: per column
  __shared__ __align__(16) float2 unflip_row[kTileRows];      // (-1, -1) where the row's sign is negative, else (1, 1)
  __shared__ __align__(8) float quarter_sum[4][kTileCols];
  const uint32_t tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const T* x = static_cast<const T*>(p.x);
  float gs;
  if (p.amax_in) {
    gs = ms_eden_scale_of_amax(p.amax_in[0]);
    if (blockIdx.x == 0 && tid == 0) p.gs_out[0] = gs;
  } else {
    gs = p.use_host_scale ? p.global_scale_host : p.global_scale_dev[0];
  }
  const uint32_t stage_base = static_cast<uint32_t>(__cvta_generic_to_shared(pair_stage));

  // 16-byte pieces of the tile, row-major, PT::kPiecesPerThread per thread
  auto issue_tile = [&](uint32_t tile, uint32_t buf) {
    const uint32_t r0 = (tile / tiles_x) * kTileRows, c0 = (tile % tiles_x) * kTileCols;
#pragma unroll
    for (int k = 0; k < PT::kPiecesPerThread; ++k) {
      const uint32_t i = tid + 256 * k, row = i / PT::kPiecesPerRow, piece = i % PT::kPiecesPerRow;
      cp_async_16(stage_base + buf * PT::kStageBytes + row * PT::kPitch + piece * 16,
                  x + static_cast<size_t>(r0 + row) * p.src_cols + c0 + piece * (16 / sizeof(T)));
    }
  };

  uint32_t tile = blockIdx.x, buf = 0;
  if (tile < tile_count) issue_tile(tile, 0);
  cp_async_commit();
  for (; tile < tile_count; tile += gridDim.x, buf ^= 1) {
    const uint32_t next = tile + gridDim.x;
    if (next < tile_count) issue_tile(next, buf ^ 1);
    cp_async_commit();
    const uint32_t ty = tile / tiles_x, r0 = ty * kTileRows, c0 = (tile % tiles_x) * kTileCols;
    if (tid < kTileRows) {
      const bool neg = random_sign_negative(p.sign_seed, r0 + tid + p.t.sign_offset);
      flip_row[tid] = neg ? (kBf16 ? 0x80008000u : 0x80000000u) : 0u;
      unflip_row[tid] = neg ? make_float2(-1.0f, -1.0f) : make_float2(1.0f, 1.0f);
    } else if (kBf16 && tid < kTileRows + kTileCols / 2) {
      const uint32_t col = c0 + 2 * (tid - kTileRows) + p.r.sign_offset;
      flip_col[tid - kTileRows] = (random_sign_negative(p.sign_seed, col) ? 0x00008000u : 0u) |
                                  (random_sign_negative(p.sign_seed, col + 1) ? 0x80000000u : 0u);
    } else if (!kBf16 && tid < kTileRows + kTileCols) {
      const uint32_t col = c0 + (tid - kTileRows) + p.r.sign_offset;
      flip_col[tid - kTileRows] = random_sign_negative(p.sign_seed, col) ? 0x80000000u : 0u;
    }
    cp_async_wait_all_but_one();
    __syncthreads();
    const uint8_t* t = pair_stage + buf * PT::kStageBytes;

    f32x2_t P[32];
    uint32_t row_lo, row_hi, chunk_in_row;
    if (warp < 4) {
      // transposed operand: source columns c0 + 2*lane (+1), K = source rows r0 + 32*warp ..
      const uint8_t* src = t + warp * 32 * PT::kPitch + lane * 2 * sizeof(T);
#pragma unroll
      for (int i = 0; i < 32; ++i) {
        const uint32_t f = flip_row[warp * 32 + i];
        if (kBf16) {
          const uint32_t w = *reinterpret_cast<const uint32_t*>(src + i * PT::kPitch) ^ f;
          P[i] = pack2(__uint_as_float(w << 16), __uint_as_float(w & 0xffff0000u));
        } else {
          const uint2 w = *reinterpret_cast<const uint2*>(src + i * PT::kPitch);
          P[i] = pack2(__uint_as_float(w.x ^ f), __uint_as_float(w.y ^ f));
        }
      }
      if (p.col_sum_partials) {
        // Column sums of this tile (dbias partials) in their fixed order -- per column four
        // sequential 32-row sums, combined below as ((q0 + q1) + q2) + q3 -- from the values this
        // thread already holds: x = P * (+-1) exactly, so acc + x is one fused multiply-add.
        f32x2_t acc = pack2(0.0f, 0.0f);
#pragma unroll
        for (int i = 0; i < 32; ++i) {
          const float2 u = unflip_row[warp * 32 + i];
          acc = fma2(P[i], pack2(u.x, u.y), acc);
        }
        float a0, a1;
        unpack2(acc, a0, a1);
        *reinterpret_cast<float2*>(&quarter_sum[warp][2 * lane]) = make_float2(a0, a1);
      }
      row_lo = c0 + 2 * lane;
      row_hi = row_lo + 1;
      chunk_in_row = (r0 >> 5) + warp;
    } else {
      // row operand: rows r0 + base + lane and + 32 more, K = source columns c0 + 32*chunk ..
      const uint32_t chunk = warp & 1, row = ((warp - 4) >> 1) * 64 + lane;
      const uint8_t* src_lo = t + row * PT::kPitch + chunk * 32 * sizeof(T);
      const uint8_t* src_hi = src_lo + 32 * PT::kPitch;
      if (kBf16) {
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const uint4 a = *reinterpret_cast<const uint4*>(src_lo + 16 * j);
          const uint4 b = *reinterpret_cast<const uint4*>(src_hi + 16 * j);
          const uint4 f = *reinterpret_cast<const uint4*>(&flip_col[chunk * 16 + 4 * j]);
          const uint32_t wa[4] = {a.x ^ f.x, a.y ^ f.y, a.z ^ f.z, a.w ^ f.w};
          const uint32_t wb[4] = {b.x ^ f.x, b.y ^ f.y, b.z ^ f.z, b.w ^ f.w};
#pragma unroll
          for (int k = 0; k < 4; ++k) {
            P[8 * j + 2 * k] = pack2(__uint_as_float(wa[k] << 16), __uint_as_float(wb[k] << 16));
            P[8 * j + 2 * k + 1] = pack2(__uint_as_float(wa[k] & 0xffff0000u), __uint_as_float(wb[k] & 0xffff0000u));
          }
        }
      } else {
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          const uint4 a = *reinterpret_cast<const uint4*>(src_lo + 16 * j);
          const uint4 b = *reinterpret_cast<const uint4*>(src_hi + 16 * j);
          const uint4 f = *reinterpret_cast<const uint4*>(&flip_col[chunk * 32 + 4 * j]);
          P[4 * j] = pack2(__uint_as_float(a.x ^ f.x), __uint_as_float(b.x ^ f.x));
          P[4 * j + 1] = pack2(__uint_as_float(a.y ^ f.y), __uint_as_float(b.y ^ f.y));
          P[4 * j + 2] = pack2(__uint_as_float(a.z ^ f.z), __uint_as_float(b.z ^ f.z));
          P[4 * j + 3] = pack2(__uint_as_float(a.w ^ f.w), __uint_as_float(b.w ^ f.w));
        }
      }
      row_lo = r0 + row;
      row_hi = row_lo + 32;
      chunk_in_row = (c0 >> 5) + chunk;
    }
    // one copy of the quantizer body for both roles (the role is warp-uniform)
    ms_eden_emit_chunk_lanes(P, warp < 4 ? p.t : p.r, gs, p.scale_override, row_lo, row_hi, chunk_in_row);
    __syncthreads();
    if (p.col_sum_partials && tid < kTileCols)
      p.col_sum_partials[static_cast<size_t>(ty) * p.src_cols + c0 + tid] =
          ((quarter_sum[0][tid] + quarter_sum[1][tid]) + quarter_sum[2][tid]) + quarter_sum[3][tid];
  }
}

// Transposer for NVFP4 sources whose extents are whole 128 x 128 tiles and whose scale bytes are
// in the packed layout: the same outputs as ms_eden_tile_kernel<2 | 3, float, false>, organised
// like the pair kernel above.  One nibble byte holds two adjacent source columns of one row,
// which are exactly the two f32x2 lanes of a thread (two output rows, the same K position):
// per K position a thread does one byte load, one E2M1x2 decode and two packed multiplies,
// (q * scale) * global_scale as utils/nvfp4/tensor.rs:48-57 decodes.  The random sign of the K
// position (the source row) is folded into that row's global scale, (q*s) * (-g) == -((q*s) * g).
constexpr int kNvTileCols = 128;                          // source columns per tile
constexpr int kNvBytePitch = kNvTileCols / 2 + 16;        // staged bytes per source row
constexpr int kNvStageBytes = kTileRows * kNvBytePitch;   // 10240

// Register budget of three CTAs per SM (80 registers, a few spilled words, same speed as the
// unconstrained 113), launched two per SM: the free third of the register file lets the
// bandwidth-bound dY amax kernel of the same backward call run beside it on another stream.
template <bool kRowwise>
__global__ void __launch_bounds__(256, 3) ms_eden_nvfp4_transpose_kernel(const MsEdenTileParams p, uint32_t tiles_x,
                                                                          uint32_t tile_count) {
  __shared__ __align__(16) uint8_t stage[2][kNvStageBytes];
  __shared__ __align__(16) float2 scale2[kTileRows][kNvTileCols / 16];  // block scale of (row, group), duplicated
  __shared__ __align__(16) float2 sgs2[kTileRows];                      // signed global scale of the row, duplicated
  const uint32_t tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  float gs;
  if (p.amax_in) {
    // the global scale from the amax of the decoded source (every thread evaluates the same two operations),
    // published for the GEMM that follows: no one-thread kernel in between
    gs = ms_eden_scale_of_amax(p.amax_in[0]);
    if (blockIdx.x == 0 && tid == 0) p.gs_out[0] = gs;
  } else {
    gs = p.use_host_scale ? p.global_scale_host : p.global_scale_dev[0];
  }
  const uint32_t stage_base = static_cast<uint32_t>(__cvta_generic_to_shared(&stage[0][0]));
  const uint32_t k_atoms = p.src_cols >> 6;

  // 512 16-byte pieces per tile, two per thread: piece i = row i/4, 16-byte column i%4
  auto issue_tile = [&](uint32_t tile, uint32_t buf) {
    const uint32_t r0 = (tile / tiles_x) * kTileRows, c0 = (tile % tiles_x) * kNvTileCols;
#pragma unroll
    for (int k = 0; k < 2; ++k) {
      const uint32_t i = tid + 256 * k, row = i >> 2, piece = i & 3;
      cp_async_16(stage_base + buf * kNvStageBytes + row * kNvBytePitch + piece * 16,
                  p.src_bytes + ((static_cast<size_t>(r0 + row) * p.src_cols + c0) >> 1) + piece * 16);
    }
  };
  // The tile's 1024 scale bytes are two adjacent 512-byte blocks of the packed plane; thread t
  // takes word t: block t/128, and inside it the four groups of row (w%4)*32 + w/4, w = t%128.
  auto scale_word = [&](uint32_t tile) {
    const uint32_t rb = tile / tiles_x, atom0 = (tile % tiles_x) * 2;
    return __ldg(reinterpret_cast<const uint32_t*>(p.src_scales + (static_cast<size_t>(rb) * k_atoms + atom0) * 512u) + tid);
  };

  uint32_t tile = blockIdx.x, buf = 0;
  uint32_t sw = 0;
  if (tile < tile_count) {
    issue_tile(tile, 0);
    sw = scale_word(tile);
  }
  cp_async_commit();
  for (; tile < tile_count; tile += gridDim.x, buf ^= 1) {
    const uint32_t next = tile + gridDim.x;
    uint32_t sw_next = 0;
    if (next < tile_count) {
      issue_tile(next, buf ^ 1);
      sw_next = scale_word(next);
    }
    cp_async_commit();
    const uint32_t r0 = (tile / tiles_x) * kTileRows, c0 = (tile % tiles_x) * kNvTileCols;
    {
      const uint32_t w = tid & 127, row = (w & 3) * 32 + (w >> 2), g0 = (tid >> 7) * 4;
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const float sc = e4m3_value((sw >> (8 * j)) & 0xffu);
        scale2[row][g0 + j] = make_float2(sc, sc);
      }
    }
    if (tid < kTileRows) {
      const float g = kRowwise ? p.src_global[r0 + tid] : p.src_global[0];
      const float sg = random_sign_negative(p.sign_seed, r0 + tid + p.t.sign_offset) ? -g : g;
      sgs2[tid] = make_float2(sg, sg);
    }
    cp_async_wait_all_but_one();
    __syncthreads();

    // thread: source columns c0 + 2*cp (+1), K = source rows r0 + 32*q ..
    const uint32_t cp = tid & 63, q = tid >> 6;
    const uint8_t* src = stage[buf] + q * 32 * kNvBytePitch + cp;
    f32x2_t P[32];
#pragma unroll
    for (int i = 0; i < 32; ++i) {
      const float2 qv = e2m1x2_values(src[i * kNvBytePitch]);
      const float2 sc = scale2[q * 32 + i][cp >> 3];
      const float2 sg = sgs2[q * 32 + i];
      // the last product feeds the butterfly's packed adds: it has to be the rounded form
      P[i] = mul2_rounded(mul2(pack2(qv.x, qv.y), pack2(sc.x, sc.y)), pack2(sg.x, sg.y));
    }
    const uint32_t out_row = c0 + 2 * cp;
    ms_eden_emit_chunk_lanes(P, p.t, gs, p.scale_override, out_row, out_row + 1, (r0 >> 5) + q);
    __syncthreads();
    sw = sw_next;
  }
  (void)lane;
  (void)warp;
}

// ReLU^2 backward between the two MLP linears (gpt/mlp/kernels.rs:72-104):
// d_pre = (d_out * 2) * max(pre, 0).  Element types: pre f32 / f16 / bf16, d_out and d_pre f32 / bf16
// (the reference has pre f32 | f16 with f32 gradients).  Eight elements per thread and step.
enum { kPreF32 = 0, kPreBf16 = 1, kPreF16 = 2 };

template <int kPre>
__device__ __forceinline__ void load8_pre(const void* p, size_t i, float (&v)[8]) {
  if (kPre == kPreF32) {
    const float4 a = __ldg(reinterpret_cast<const float4*>(static_cast<const float*>(p) + i));
    const float4 b = __ldg(reinterpret_cast<const float4*>(static_cast<const float*>(p) + i) + 1);
    v[0] = a.x, v[1] = a.y, v[2] = a.z, v[3] = a.w, v[4] = b.x, v[5] = b.y, v[6] = b.z, v[7] = b.w;
  } else {
    const uint4 t = __ldg(reinterpret_cast<const uint4*>(static_cast<const uint16_t*>(p) + i));
    const uint32_t w[4] = {t.x, t.y, t.z, t.w};
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      if (kPre == kPreBf16) {
        v[2 * k] = __uint_as_float(w[k] << 16);
        v[2 * k + 1] = __uint_as_float(w[k] & 0xffff0000u);
      } else {
        const float2 f = __half22float2(*reinterpret_cast<const __half2*>(&w[k]));
        v[2 * k] = f.x;
        v[2 * k + 1] = f.y;
      }
    }
  }
}
template <int kPre>
__device__ __forceinline__ float load1_pre(const void* p, size_t i) {
  if (kPre == kPreF32) return __ldg(static_cast<const float*>(p) + i);
  const uint16_t h = __ldg(static_cast<const uint16_t*>(p) + i);
  if (kPre == kPreBf16) return __uint_as_float(static_cast<uint32_t>(h) << 16);
  return __half2float(__ushort_as_half(h));
}
template <bool kBf16>
__device__ __forceinline__ void store8_grad(void* p, size_t i, const float (&v)[8]) {
  if (!kBf16) {
    float4* q = reinterpret_cast<float4*>(static_cast<float*>(p) + i);
    q[0] = make_float4(v[0], v[1], v[2], v[3]);
    q[1] = make_float4(v[4], v[5], v[6], v[7]);
  } else {
    uint32_t w[4];
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      const __nv_bfloat162 h = __floats2bfloat162_rn(v[2 * k], v[2 * k + 1]);
      w[k] = *reinterpret_cast<const uint32_t*>(&h);
    }
    *reinterpret_cast<uint4*>(static_cast<uint16_t*>(p) + i) = make_uint4(w[0], w[1], w[2], w[3]);
  }
}

// With chunk_amax set the kernel also emits, per CTA, the amax of the values it stored (after their rounding to
// the gradient type): the chunk list nvfp4_linear_backward_ms_eden accepts in place of its own amax pass over dY
// (the hand-over gpt/loss/kernels.rs:67-88 -> backward/final_head/run.rs:34,54 makes for the loss gradient).
template <int kPre, bool kGradBf16, bool kAmax>
__global__ void __launch_bounds__(256) relu2_backward_kernel(const void* __restrict__ pre, const void* __restrict__ d_out,
                                                              void* __restrict__ d_pre, uint64_t n, int vectorized,
                                                              float* __restrict__ chunk_amax) {
  const uint64_t stride = static_cast<uint64_t>(gridDim.x) * 256;
  const uint64_t tid = static_cast<uint64_t>(blockIdx.x) * 256 + threadIdx.x;
  const uint64_t vec_n = vectorized ? n / 8 : 0;
  float m = 0.0f;
  for (uint64_t i = tid; i < vec_n; i += stride) {
    float p[8], d[8], r[8];
    load8_pre<kPre>(pre, i * 8, p);
    load8_pre<kGradBf16 ? kPreBf16 : kPreF32>(d_out, i * 8, d);
#pragma unroll
    for (int k = 0; k < 8; ++k) r[k] = (d[k] * 2.0f) * max_f32(p[k], 0.0f);
    store8_grad<kGradBf16>(d_pre, i * 8, r);
    if (kAmax) {
#pragma unroll
      for (int k = 0; k < 8; ++k) {
        const float stored = kGradBf16 ? __bfloat162float(__float2bfloat16_rn(r[k])) : r[k];
        m = max_f32(m, fabsf(stored));
      }
    }
  }
  for (uint64_t i = vec_n * 8 + tid; i < n; i += stride) {
    const float p = load1_pre<kPre>(pre, i);
    const float d = load1_pre<kGradBf16 ? kPreBf16 : kPreF32>(d_out, i);
    const float r = (d * 2.0f) * max_f32(p, 0.0f);
    float stored = r;
    if (kGradBf16) {
      const __nv_bfloat16 h = __float2bfloat16_rn(r);
      static_cast<__nv_bfloat16*>(d_pre)[i] = h;
      stored = __bfloat162float(h);
    } else {
      static_cast<float*>(d_pre)[i] = r;
    }
    if (kAmax) m = max_f32(m, fabsf(stored));
  }
  if (kAmax) {
    __shared__ float partial[8];
    m = warp_max(m);
    if ((threadIdx.x & 31) == 0) partial[threadIdx.x >> 5] = m;
    __syncthreads();
    if (threadIdx.x == 0) {
      float r = 0.0f;
#pragma unroll
      for (int i = 0; i < 8; ++i) r = max_f32(r, partial[i]);
      chunk_amax[blockIdx.x] = r;
    }
  }
}

// ============================================================================
// decode, scale pack, padding, post-ops, bias gradient
// ============================================================================

// utils/nvfp4/decode/kernels.rs:11-57
__global__ void __launch_bounds__(256) decode_kernel(const uint8_t* __restrict__ bytes,
                                                      const uint8_t* __restrict__ scales,
                                                      const float* __restrict__ gscales, float* __restrict__ out,
                                                      uint32_t rows, uint32_t cols, int rowwise, int transpose) {
  const uint64_t idx = static_cast<uint64_t>(blockIdx.x) * 256 + threadIdx.x;
  const uint64_t n = static_cast<uint64_t>(rows) * cols;
  if (idx >= n) return;
  const uint32_t r = static_cast<uint32_t>(idx / cols), c = static_cast<uint32_t>(idx % cols);
  const float v = nvfp4_value(bytes, scales, rowwise ? gscales[r] : gscales[0], idx);
  out[transpose ? static_cast<size_t>(c) * rows + r : idx] = v;
}

// utils/nvfp4_tma_matmul/scale_pack.rs:14-40
__global__ void __launch_bounds__(256) scale_pack_kernel(const uint8_t* __restrict__ logical,
                                                          uint8_t* __restrict__ packed, uint32_t mn, uint32_t padded_mn,
                                                          uint32_t k_groups) {
  const uint64_t total = static_cast<uint64_t>(padded_mn) * k_groups;
  for (uint64_t i = static_cast<uint64_t>(blockIdx.x) * 256 + threadIdx.x; i < total;
       i += static_cast<uint64_t>(gridDim.x) * 256) {
    const uint32_t r = static_cast<uint32_t>(i / k_groups), kg = static_cast<uint32_t>(i % k_groups);
    packed[packed_scale_offset(r, kg, k_groups >> 2)] = r < mn ? logical[i] : 0x38;
  }
}

// utils/nvfp4_tma_matmul/pad.rs:115-210
__global__ void __launch_bounds__(256) pad_u4_rows_kernel(const uint8_t* __restrict__ src, uint8_t* __restrict__ dst,
                                                           uint64_t src_bytes, uint64_t dst_bytes) {
  for (uint64_t i = static_cast<uint64_t>(blockIdx.x) * 256 + threadIdx.x; i < dst_bytes;
       i += static_cast<uint64_t>(gridDim.x) * 256)
    dst[i] = i < src_bytes ? src[i] : 0;
}
template <bool kTranspose>
__global__ void __launch_bounds__(256) pad_f32_kernel(const float* __restrict__ src, float* __restrict__ dst,
                                                       uint32_t rows, uint32_t cols, uint32_t padded_rows,
                                                       uint32_t padded_cols) {
  const uint64_t total = static_cast<uint64_t>(padded_rows) * padded_cols;
  for (uint64_t i = static_cast<uint64_t>(blockIdx.x) * 256 + threadIdx.x; i < total;
       i += static_cast<uint64_t>(gridDim.x) * 256) {
    const uint32_t r = static_cast<uint32_t>(i / padded_cols), c = static_cast<uint32_t>(i % padded_cols);
    float v = 0.0f;
    if (!kTranspose) {
      if (r < rows && c < cols) v = src[static_cast<size_t>(r) * cols + c];
    } else {
      if (r < cols && c < rows) v = src[static_cast<size_t>(c) * cols + r];
    }
    dst[i] = v;
  }
}
__global__ void __launch_bounds__(256) crop_f32_kernel(const float* __restrict__ src, float* __restrict__ dst,
                                                        uint32_t rows, uint32_t src_cols, uint32_t dst_cols) {
  const uint64_t total = static_cast<uint64_t>(rows) * dst_cols;
  for (uint64_t i = static_cast<uint64_t>(blockIdx.x) * 256 + threadIdx.x; i < total;
       i += static_cast<uint64_t>(gridDim.x) * 256) {
    const uint32_t r = static_cast<uint32_t>(i / dst_cols), c = static_cast<uint32_t>(i % dst_cols);
    dst[i] = src[static_cast<size_t>(r) * src_cols + c];
  }
}

// gpt/projection_postop.rs:97-162.  mode 0: raw += bias; 1: residual = fma(1, raw + bias, residual);
// 2: pre = raw + bias (in place), out = max(pre, 0)^2.
__global__ void __launch_bounds__(256) postop_kernel(float* __restrict__ raw, float* __restrict__ other,
                                                      const uint8_t* __restrict__ bias_bytes,
                                                      const uint8_t* __restrict__ bias_scales,
                                                      const float* __restrict__ bias_gs, uint64_t n, uint32_t cols,
                                                      int mode) {
  for (uint64_t i = static_cast<uint64_t>(blockIdx.x) * 256 + threadIdx.x; i < n;
       i += static_cast<uint64_t>(gridDim.x) * 256) {
    const uint32_t col = static_cast<uint32_t>(i % cols);
    const float bias = nvfp4_value(bias_bytes, bias_scales, bias_gs[0], col);
    if (mode == 0) {
      raw[i] = raw[i] + bias;
    } else if (mode == 1) {
      other[i] = __fmaf_rn(1.0f, raw[i] + bias, other[i]);
    } else {
      const float pre = raw[i] + bias;
      const float r = max_f32(pre, 0.0f);
      raw[i] = pre;
      other[i] = r * r;
    }
  }
}

// gpt/linear_backward/bias.rs:18-69: 8 row lanes x 32 columns per CTA; each row lane sums
// rows lane, lane+8, ... in order; the 8 lane sums are then added left to right.
template <typename T>
__global__ void __launch_bounds__(256) bias_grad_kernel(const T* __restrict__ e, float* __restrict__ dbias,
                                                         uint32_t tokens, uint32_t n) {
  __shared__ float sums[256];
  const uint32_t lane = threadIdx.x & 31, w = threadIdx.x >> 5;
  const uint32_t col = blockIdx.x * 32 + lane;
  float local = 0.0f;
  if (col < n) {
    uint32_t row = w;
    for (; row + 8 * 7 < tokens; row += 64) {
      float t[8];
#pragma unroll
      for (int i = 0; i < 8; ++i) t[i] = load_as_f32<T>(e, static_cast<size_t>(row + 8 * i) * n + col);
#pragma unroll
      for (int i = 0; i < 8; ++i) local += t[i];
    }
    for (; row < tokens; row += 8) local += load_as_f32<T>(e, static_cast<size_t>(row) * n + col);
  }
  sums[threadIdx.x] = local;
  __syncthreads();
  if (w == 0 && col < n) {
    float s = sums[lane];
#pragma unroll
    for (int i = 1; i < 8; ++i) s = s + sums[lane + 32 * i];
    dbias[col] = s;
  }
}

// dbias[c] = sum over row tiles of the tile column sums in a fixed order: eight lanes per
// column each add tiles lane, lane+8, ... in sequence, then the lane sums are added 0..7.
__global__ void __launch_bounds__(256) col_sum_reduce_kernel(const float* __restrict__ partials,
                                                              float* __restrict__ dbias, uint32_t tiles, uint32_t n) {
  __shared__ float sums[256];
  const uint32_t lane = threadIdx.x & 31, w = threadIdx.x >> 5;
  const uint32_t c = blockIdx.x * 32 + lane;
  float acc = 0.0f;
  if (c < n) {
    // sixteen loads in flight per thread, added in tile order (the loads dominate: few CTAs, long latency)
    uint32_t t = w;
    for (; t + 8 * 15 < tiles; t += 8 * 16) {
      float v[16];
#pragma unroll
      for (int j = 0; j < 16; ++j) v[j] = __ldg(partials + static_cast<size_t>(t + 8 * j) * n + c);
#pragma unroll
      for (int j = 0; j < 16; ++j) acc += v[j];
    }
    for (; t < tiles; t += 8) acc += __ldg(partials + static_cast<size_t>(t) * n + c);
  }
  sums[threadIdx.x] = acc;
  __syncthreads();
  if (w == 0 && c < n) {
    float r = sums[lane];
#pragma unroll
    for (int i = 1; i < 8; ++i) r = r + sums[lane + 32 * i];
    dbias[c] = r;
  }
}

// ============================================================================
// launchers
// ============================================================================

static inline uint32_t blocks_for(uint64_t n, uint32_t per_block, uint32_t cap = 0x7fffffffu) {
  uint64_t b = (n + per_block - 1) / per_block;
  if (b == 0) b = 1;
  return static_cast<uint32_t>(b > cap ? cap : b);
}

#define NVFP4_RETURN_LAST() \
  do {                       \
    count_launch();          \
    return static_cast<int>(cudaGetLastError()); \
  } while (0)

int launch_row_amax(cudaStream_t s, const void* x, int dtype, float* out, uint32_t rows, uint32_t row_len) {
  if (rows == 0) return 0;
  if (dtype == 0)
    row_amax_kernel<float><<<blocks_for(rows, 8), 256, 0, s>>>(static_cast<const float*>(x), out, rows, row_len);
  else
    row_amax_kernel<__nv_bfloat16>
        <<<blocks_for(rows, 8), 256, 0, s>>>(static_cast<const __nv_bfloat16*>(x), out, rows, row_len);
  NVFP4_RETURN_LAST();
}

int launch_tensor_amax(cudaStream_t s, const void* x, int dtype, float* chunk_amax, float* out, uint64_t n) {
  cudaError_t err = cudaMemsetAsync(out, 0, sizeof(float), s);
  if (err != cudaSuccess) return static_cast<int>(err);
  if (n == 0) return 0;
  const uint32_t grid = blocks_for((n + 1023) / 1024, 8, 148 * 8);
  if (dtype == 0)
    tensor_amax_kernel<float><<<grid, 256, 0, s>>>(static_cast<const float*>(x), chunk_amax, out, n);
  else
    tensor_amax_kernel<__nv_bfloat16><<<grid, 256, 0, s>>>(static_cast<const __nv_bfloat16*>(x), chunk_amax, out, n);
  NVFP4_RETURN_LAST();
}

int launch_nvfp4_amax(cudaStream_t s, const uint8_t* bytes, const uint8_t* scales, const float* gscales, uint32_t rows,
                      uint32_t cols, int rowwise, int packed, float* chunk_amax, float* out) {
  const uint64_t n = static_cast<uint64_t>(rows) * cols;
  cudaError_t err = cudaMemsetAsync(out, 0, sizeof(float), s);
  if (err != cudaSuccess) return static_cast<int>(err);
  if (n == 0) return 0;
  nvfp4_amax_kernel<<<blocks_for((n + 1023) / 1024, 8, 148 * 8), 256, 0, s>>>(bytes, scales, gscales, n, cols, rowwise, packed,
                                                                     chunk_amax, out);
  NVFP4_RETURN_LAST();
}

int launch_amax_from_chunks(cudaStream_t s, const float* chunk_amax, float* out, uint32_t chunk_count, int transform) {
  amax_from_chunks_kernel<<<1, 256, 0, s>>>(chunk_amax, out, chunk_count, transform);
  NVFP4_RETURN_LAST();
}

int launch_ms_eden_scale_from_amax(cudaStream_t s, const float* amax, float* out) {
  ms_eden_scale_from_amax_kernel<<<1, 1, 0, s>>>(amax, out);
  NVFP4_RETURN_LAST();
}

template <typename T, bool kRelu2>
static int launch_four_six_t(cudaStream_t s, const T* x, const float* amax, int rowwise, uint32_t rows, uint32_t cols,
                             uint8_t* out_fp4, uint8_t* out_scales, int packed, float* out_gs, float* decoded_amax) {
  const uint32_t gpr = cols / 16;
  const uint64_t groups = static_cast<uint64_t>(rows) * gpr;
  const uint32_t grid = blocks_for(groups, 256);
#define NVFP4_LAUNCH_FS(R, P) \
  four_six_kernel<T, R, P, kRelu2><<<grid, 256, 0, s>>>(x, amax, out_fp4, out_scales, out_gs, decoded_amax, groups, gpr)
  if (rowwise) {
    if (packed) NVFP4_LAUNCH_FS(true, true);
    else NVFP4_LAUNCH_FS(true, false);
  } else {
    if (packed) NVFP4_LAUNCH_FS(false, true);
    else NVFP4_LAUNCH_FS(false, false);
  }
#undef NVFP4_LAUNCH_FS
  count_launch();
  return static_cast<int>(cudaGetLastError());
}

int launch_four_six(cudaStream_t s, const void* x, int dtype, const float* amax, int rowwise, uint32_t rows,
                    uint32_t cols, uint8_t* out_fp4, uint8_t* out_scales, int packed, float* out_gs, int relu2,
                    float* decoded_amax) {
  if (decoded_amax) {
    const cudaError_t err = cudaMemsetAsync(decoded_amax, 0, sizeof(float), s);
    if (err != cudaSuccess) return static_cast<int>(err);
  }
  if (rows == 0 || cols == 0) return 0;
  int rc;
  if (dtype == 0) {
    const float* xf = static_cast<const float*>(x);
    rc = relu2 ? launch_four_six_t<float, true>(s, xf, amax, rowwise, rows, cols, out_fp4, out_scales, packed, out_gs, decoded_amax)
               : launch_four_six_t<float, false>(s, xf, amax, rowwise, rows, cols, out_fp4, out_scales, packed, out_gs, decoded_amax);
  } else {
    const __nv_bfloat16* xb = static_cast<const __nv_bfloat16*>(x);
    rc = relu2 ? launch_four_six_t<__nv_bfloat16, true>(s, xb, amax, rowwise, rows, cols, out_fp4, out_scales, packed, out_gs, decoded_amax)
               : launch_four_six_t<__nv_bfloat16, false>(s, xb, amax, rowwise, rows, cols, out_fp4, out_scales, packed, out_gs, decoded_amax);
  }
  if (rc) return rc;
  if (packed) return launch_packed_scale_pad(s, out_scales, rows, cols);
  return 0;
}

// Fused row amax + rowwise four-six.  Returns -1 when the row is too long for one CTA (the
// caller then runs the two-kernel path).
int launch_four_six_rowwise_fused(cudaStream_t s, const void* x, int dtype, uint32_t rows, uint32_t cols,
                                  uint8_t* out_fp4, uint8_t* out_scales, int packed, float* out_gs, float* out_amax,
                                  float* decoded_amax, int relu2) {
  const uint32_t gpr = cols / 16;
  if (gpr == 0 || gpr > 256) return -1;
  if (decoded_amax) {
    const cudaError_t err = cudaMemsetAsync(decoded_amax, 0, sizeof(float), s);
    if (err != cudaSuccess) return static_cast<int>(err);
  }
  if (rows == 0) return 0;
  const uint32_t rpc = 256 / gpr;
  const uint32_t threads = (rpc * gpr + 31) / 32 * 32;
  const uint32_t row_blocks = (rows + rpc - 1) / rpc;
  const size_t smem = (rpc + 1) * sizeof(unsigned int);
  // Persistent CTAs (three fit an SM) once there are more row blocks than resident CTAs and a CTA holds several
  // rows (measured on B200 at 65536 rows: 768 columns 62 against 67 us; rows of 3072 columns, one per CTA,
  // are faster with one CTA per row: 207 against 228 us); the grid is sized so that every CTA walks the same
  // number of row blocks.
  const uint32_t resident = 148u * 3u;  // 80 registers x 256 threads: three CTAs per SM
  const bool stream = row_blocks > resident && gpr <= 64 && ((reinterpret_cast<uintptr_t>(out_scales) & 3u) == 0);
  const uint32_t per_cta = (row_blocks + resident - 1) / resident;
  const uint32_t grid = stream ? (row_blocks + per_cta - 1) / per_cta : row_blocks;
#define NVFP4_LAUNCH_FUSED(T, P, R)                                                                                   \
  do {                                                                                                                \
    if (stream)                                                                                                       \
      four_six_rowwise_stream_kernel<T, P, R><<<grid, threads, 0, s>>>(static_cast<const T*>(x), out_fp4, out_scales, \
                                                                       out_gs, out_amax, decoded_amax, rows, gpr, rpc, \
                                                                       row_blocks);                                   \
    else                                                                                                              \
      four_six_rowwise_fused_kernel<T, P, R><<<grid, threads, smem, s>>>(static_cast<const T*>(x), out_fp4,           \
                                                                         out_scales, out_gs, out_amax, decoded_amax,  \
                                                                         rows, gpr, rpc);                             \
  } while (0)
#define NVFP4_LAUNCH_FUSED_R(T, P)       \
  do {                                   \
    if (relu2) NVFP4_LAUNCH_FUSED(T, P, true); \
    else NVFP4_LAUNCH_FUSED(T, P, false);      \
  } while (0)
  if (dtype == NVFP4_DTYPE_F32) {
    if (packed) NVFP4_LAUNCH_FUSED_R(float, true);
    else NVFP4_LAUNCH_FUSED_R(float, false);
  } else {
    if (packed) NVFP4_LAUNCH_FUSED_R(__nv_bfloat16, true);
    else NVFP4_LAUNCH_FUSED_R(__nv_bfloat16, false);
  }
#undef NVFP4_LAUNCH_FUSED_R
#undef NVFP4_LAUNCH_FUSED
  count_launch();
  int rc = static_cast<int>(cudaGetLastError());
  if (rc) return rc;
  if (packed) return launch_packed_scale_pad(s, out_scales, rows, cols);
  return 0;
}

int launch_schedule_free_materialize(cudaStream_t s, const float* z, const float* x, float beta, float* chunk_amax,
                                     float* amax, uint8_t* out_fp4, uint8_t* out_scales, int packed, float* out_gs,
                                     uint32_t rows, uint32_t cols) {
  const uint64_t n = static_cast<uint64_t>(rows) * cols;
  cudaError_t err = cudaMemsetAsync(amax, 0, sizeof(float), s);
  if (err != cudaSuccess) return static_cast<int>(err);
  if (n == 0) return 0;
  schedule_free_amax_kernel<<<blocks_for((n + 1023) / 1024, 8, 148 * 8), 256, 0, s>>>(z, x, chunk_amax, amax, beta, n);
  count_launch();
  const uint64_t groups = n / 16;
  const uint32_t gpr = cols / 16;
  if (packed)
    schedule_free_four_six_kernel<true><<<blocks_for(groups, 256), 256, 0, s>>>(z, x, amax, out_fp4, out_scales, out_gs,
                                                                               beta, groups, gpr);
  else
    schedule_free_four_six_kernel<false><<<blocks_for(groups, 256), 256, 0, s>>>(z, x, amax, out_fp4, out_scales, out_gs,
                                                                                beta, groups, gpr);
  count_launch();
  int rc = static_cast<int>(cudaGetLastError());
  if (rc) return rc;
  if (packed) return launch_packed_scale_pad(s, out_scales, rows, cols);
  return 0;
}

int launch_packed_scale_pad(cudaStream_t s, uint8_t* packed, uint32_t rows, uint32_t k_dim) {
  const uint32_t padded = (rows + 127u) / 128u * 128u;
  if (padded == rows) return 0;
  const uint32_t kg = k_dim / 16;
  packed_scale_pad_kernel<<<blocks_for(static_cast<uint64_t>(padded - rows) * kg, 256, 1024), 256, 0, s>>>(packed, rows,
                                                                                                         padded, kg);
  NVFP4_RETURN_LAST();
}

int launch_four_six_padded(cudaStream_t s, const float* x, const float* amax, uint8_t* out_fp4, uint8_t* out_scales,
                           float* out_gs, uint32_t rows, uint32_t cols, uint32_t padded_rows, uint32_t padded_cols,
                           int transposed) {
  const uint64_t groups = static_cast<uint64_t>(padded_rows) * padded_cols / 16;
  if (groups == 0) return 0;
  if (transposed)
    four_six_padded_kernel<true>
        <<<blocks_for(groups, 256), 256, 0, s>>>(x, amax, out_fp4, out_scales, out_gs, rows, cols, padded_cols, groups);
  else
    four_six_padded_kernel<false>
        <<<blocks_for(groups, 256), 256, 0, s>>>(x, amax, out_fp4, out_scales, out_gs, rows, cols, padded_cols, groups);
  NVFP4_RETURN_LAST();
}

static MsEdenOut make_out(const nvfp4_ms_eden_args& a, uint32_t out_rows) {
  MsEdenOut o;
  o.fp4 = a.out_fp4;
  o.scales = a.out_scales;
  o.global_scales = a.out_global_scales;
  o.chunk_amax = a.out_chunk_amax;
  o.rows = out_rows;
  o.dst_row_len = a.dst_row_len;
  o.scale_seed = a.scale_seed;
  o.group_offset = a.group_offset;
  o.group_row_stride = a.group_row_stride ? a.group_row_stride : a.dst_row_len / 16u;
  o.sign_offset = a.col_offset;
  o.packed = a.scale_layout == NVFP4_SCALES_PACKED;
  return o;
}

template <int kSrc, typename T, bool kPair>
static void launch_tile(cudaStream_t s, const MsEdenTileParams& p) {
  dim3 grid((p.src_cols + kTileCols - 1) / kTileCols, (p.src_rows + kTileRows - 1) / kTileRows);
  ms_eden_tile_kernel<kSrc, T, kPair><<<grid, 256, 0, s>>>(p);
}

// The tile kernel covers K positions [0, ceil(rows/128)*128) of the transposed operand and
// [0, ceil(cols/64)*64) of the row operand; longer destinations use the generic kernel.
static bool tile_covers(uint32_t src_rows, uint32_t dst_row_len) {
  return dst_row_len <= (src_rows + kTileRows - 1) / kTileRows * kTileRows;
}

int launch_ms_eden(cudaStream_t s, const nvfp4_ms_eden_args& a_in, const float* amax_in, float* gs_out) {
  nvfp4_ms_eden_args a = a_in;
  if (amax_in) {
    // the whole-tile NVFP4 transposers derive the scale from the amax themselves; every other kernel gets it
    // from a one-thread kernel first
    const bool nv_kind = a.src_kind == NVFP4_SRC_NVFP4_TRANSPOSED || a.src_kind == NVFP4_SRC_ROWWISE_NVFP4_TRANSPOSED;
    const bool whole = nv_kind && a.src_scale_layout == NVFP4_SCALES_PACKED && a.rows % kTileRows == 0 &&
                       a.cols % kNvTileCols == 0 && a.dst_row_len == a.rows &&
                       (reinterpret_cast<uintptr_t>(a.src_bytes) & 15u) == 0 &&
                       (reinterpret_cast<uintptr_t>(a.src_scales) & 3u) == 0 && a.rows != 0 && a.cols != 0;
    if (!whole) {
      const int rc = launch_ms_eden_scale_from_amax(s, amax_in, gs_out);
      if (rc) return rc;
      amax_in = nullptr;
    }
    a.global_scale = gs_out;
    a.host_global_scale_valid = 0;
  }
  const bool rows_kind = a.src_kind == NVFP4_SRC_F32_ROWS;
  const uint32_t out_rows = rows_kind ? a.rows : a.cols;
  const uint64_t chunks = static_cast<uint64_t>(out_rows) * (a.dst_row_len / 32);
  if (chunks == 0) return 0;
  const bool bf16 = a.src_dtype == NVFP4_DTYPE_BF16;
  const int packed = a.scale_layout == NVFP4_SCALES_PACKED;
  if (!rows_kind && tile_covers(a.rows, a.dst_row_len)) {
    MsEdenTileParams p;
    p.x = a.x;
    p.src_bytes = a.src_bytes;
    p.src_scales = a.src_scales;
    p.src_global = a.src_global;
    p.src_packed = a.src_scale_layout == NVFP4_SCALES_PACKED;
    p.src_rows = a.rows;
    p.src_cols = a.cols;
    p.global_scale_dev = a.global_scale;
    p.global_scale_host = a.host_global_scale;
    p.use_host_scale = a.host_global_scale_valid;
    p.scale_override = a.scale_override;
    p.sign_seed = a.sign_seed;
    p.t = make_out(a, out_rows);
    p.r = p.t;
    p.col_sum_partials = nullptr;
    p.amax_in = amax_in;
    p.gs_out = gs_out;
    const bool nv_whole_tiles = p.src_packed && a.rows % kTileRows == 0 && a.cols % kNvTileCols == 0 &&
                                a.dst_row_len == a.rows && (reinterpret_cast<uintptr_t>(a.src_bytes) & 15u) == 0 &&
                                (reinterpret_cast<uintptr_t>(a.src_scales) & 3u) == 0;
    const uint32_t nv_tiles_x = a.cols / kNvTileCols, nv_tiles = nv_tiles_x * (a.rows / kTileRows);
    switch (a.src_kind) {
      case NVFP4_SRC_F32_TRANSPOSED:
        if (bf16) launch_tile<0, __nv_bfloat16, false>(s, p);
        else launch_tile<0, float, false>(s, p);
        break;
      case NVFP4_SRC_NVFP4_TRANSPOSED:
        if (nv_whole_tiles)
          ms_eden_nvfp4_transpose_kernel<false><<<min(nv_tiles, 148u * 2u), 256, 0, s>>>(p, nv_tiles_x, nv_tiles);
        else
          launch_tile<2, float, false>(s, p);
        break;
      case NVFP4_SRC_ROWWISE_NVFP4_TRANSPOSED:
        if (nv_whole_tiles)
          ms_eden_nvfp4_transpose_kernel<true><<<min(nv_tiles, 148u * 2u), 256, 0, s>>>(p, nv_tiles_x, nv_tiles);
        else
          launch_tile<3, float, false>(s, p);
        break;
      default:
        return 1;
    }
  } else {
    MsEdenParams p;
    p.x = a.x;
    p.src_bytes = a.src_bytes;
    p.src_scales = a.src_scales;
    p.src_global = a.src_global;
    p.src_packed = a.src_scale_layout == NVFP4_SCALES_PACKED;
    p.a = rows_kind ? a.cols : a.rows;
    p.b = a.cols;
    p.global_scale_dev = a.global_scale;
    p.global_scale_host = a.host_global_scale;
    p.use_host_scale = a.host_global_scale_valid;
    p.scale_override = a.scale_override;
    p.sign_seed = a.sign_seed;
    p.out = make_out(a, out_rows);
    const uint32_t grid = blocks_for(chunks, 128);
    switch (a.src_kind) {
      case NVFP4_SRC_F32_ROWS:
        if (bf16) ms_eden_kernel<0, __nv_bfloat16><<<grid, 128, 0, s>>>(p);
        else ms_eden_kernel<0, float><<<grid, 128, 0, s>>>(p);
        break;
      case NVFP4_SRC_F32_TRANSPOSED:
        if (bf16) ms_eden_kernel<1, __nv_bfloat16><<<grid, 128, 0, s>>>(p);
        else ms_eden_kernel<1, float><<<grid, 128, 0, s>>>(p);
        break;
      case NVFP4_SRC_NVFP4_TRANSPOSED:
        ms_eden_kernel<2, float><<<grid, 128, 0, s>>>(p);
        break;
      case NVFP4_SRC_ROWWISE_NVFP4_TRANSPOSED:
        ms_eden_kernel<3, float><<<grid, 128, 0, s>>>(p);
        break;
      default:
        return 1;
    }
  }
  count_launch();
  int rc = static_cast<int>(cudaGetLastError());
  if (rc) return rc;
  if (packed) return launch_packed_scale_pad(s, a.out_scales, out_rows, a.dst_row_len);
  return 0;
}

// Row operand and transposed operand of one f32 / bf16 matrix in a single pass over it.
// `rows_args` describes the row operand (src_kind F32_ROWS), `t_args` the transposed one
// (src_kind F32_TRANSPOSED) of the same matrix; both use the same global scale and sign seed.
uint32_t ms_eden_pair_row_tiles(uint32_t rows) { return (rows + kTileRows - 1) / kTileRows; }

bool ms_eden_pair_is_tiled(const nvfp4_ms_eden_args& r, const nvfp4_ms_eden_args& t) {
  return r.rows != 0 && r.cols != 0 && tile_covers(r.rows, t.dst_row_len) &&
         r.dst_row_len <= (r.cols + kTileCols - 1) / kTileCols * kTileCols;
}

int launch_col_sum_reduce(cudaStream_t s, const float* partials, float* dbias, uint32_t tiles, uint32_t n) {
  if (n == 0) return 0;
  col_sum_reduce_kernel<<<blocks_for(n, 32), 256, 0, s>>>(partials, dbias, tiles, n);
  NVFP4_RETURN_LAST();
}

static bool pair_whole_tiles(const nvfp4_ms_eden_args& r, const nvfp4_ms_eden_args& t) {
  return r.rows % kTileRows == 0 && r.cols % kTileCols == 0 && t.dst_row_len == r.rows && r.dst_row_len == r.cols &&
         (reinterpret_cast<uintptr_t>(r.x) & 15u) == 0;
}

bool ms_eden_pair_takes_amax(const nvfp4_ms_eden_args& r, const nvfp4_ms_eden_args& t) {
  return ms_eden_pair_is_tiled(r, t) && pair_whole_tiles(r, t);
}

int launch_ms_eden_pair(cudaStream_t s, const nvfp4_ms_eden_args& r, const nvfp4_ms_eden_args& t,
                        float* col_sum_partials, const float* amax_in, float* gs_out) {
  const uint32_t rows = r.rows, cols = r.cols;
  if (amax_in && !ms_eden_pair_takes_amax(r, t)) return static_cast<int>(cudaErrorInvalidValue);
  if (!ms_eden_pair_is_tiled(r, t)) {
    int rc = launch_ms_eden(s, r);
    return rc ? rc : launch_ms_eden(s, t);
  }
  MsEdenTileParams p;
  p.x = r.x;
  p.src_bytes = nullptr;
  p.src_scales = nullptr;
  p.src_global = nullptr;
  p.src_packed = 0;
  p.src_rows = rows;
  p.src_cols = cols;
  p.global_scale_dev = r.global_scale;
  p.global_scale_host = r.host_global_scale;
  p.use_host_scale = r.host_global_scale_valid;
  p.scale_override = r.scale_override;
  p.sign_seed = r.sign_seed;
  p.t = make_out(t, cols);
  p.r = make_out(r, rows);
  p.col_sum_partials = col_sum_partials;
  p.amax_in = amax_in;
  p.gs_out = gs_out;
  const bool whole_tiles = pair_whole_tiles(r, t);
  if (whole_tiles) {
    const uint32_t tiles_x = cols / kTileCols, tile_count = tiles_x * (rows / kTileRows);
    const uint32_t grid = min(tile_count, 148u * 2u);
    if (r.src_dtype == NVFP4_DTYPE_BF16) {
      ms_eden_pair_kernel<__nv_bfloat16>
          <<<grid, 256, 2 * PairTile<__nv_bfloat16>::kStageBytes, s>>>(p, tiles_x, tile_count);
    } else {
      // the opt-in to more than 48 KB of dynamic shared memory is a per-device attribute of the kernel
      static std::atomic<int> attr_state[64];  // per device ordinal: 0 = not set, 1 = set, -(error) = failed
      int dev = 0;
      if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return static_cast<int>(cudaErrorInvalidDevice);
      int st = attr_state[dev].load(std::memory_order_acquire);
      if (st == 0) {
        const cudaError_t e = cudaFuncSetAttribute(ms_eden_pair_kernel<float>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                                   2 * PairTile<float>::kStageBytes);
        st = e == cudaSuccess ? 1 : -static_cast<int>(e);
        attr_state[dev].store(st, std::memory_order_release);
      }
      if (st < 0) return -st;
      ms_eden_pair_kernel<float><<<grid, 256, 2 * PairTile<float>::kStageBytes, s>>>(p, tiles_x, tile_count);
    }
  } else if (r.src_dtype == NVFP4_DTYPE_BF16) {
    launch_tile<0, __nv_bfloat16, true>(s, p);
  } else {
    launch_tile<0, float, true>(s, p);
  }
  count_launch();
  int rc = static_cast<int>(cudaGetLastError());
  if (rc) return rc;
  if (p.r.packed) rc = launch_packed_scale_pad(s, r.out_scales, rows, r.dst_row_len);
  if (rc) return rc;
  if (p.t.packed) rc = launch_packed_scale_pad(s, t.out_scales, cols, t.dst_row_len);
  return rc;
}

uint32_t relu2_backward_grid(uint64_t n) { return blocks_for((n + 7) / 8, 256, 148 * 8); }

int launch_relu2_backward(cudaStream_t s, const void* pre, int pre_kind, const void* d_out, void* d_pre, int grad_bf16,
                          uint64_t n, float* chunk_amax) {
  if (n == 0) return 0;
  const int vectorized = ((reinterpret_cast<uintptr_t>(pre) | reinterpret_cast<uintptr_t>(d_out) |
                           reinterpret_cast<uintptr_t>(d_pre)) & 15u) == 0;
  const uint32_t grid = relu2_backward_grid(n);
#define NVFP4_RELU2_BWD_A(K, G, A) \
  relu2_backward_kernel<K, G, A><<<grid, 256, 0, s>>>(pre, d_out, d_pre, n, vectorized, chunk_amax)
#define NVFP4_RELU2_BWD(K, G)                     \
  do {                                            \
    if (chunk_amax) NVFP4_RELU2_BWD_A(K, G, true); \
    else NVFP4_RELU2_BWD_A(K, G, false);          \
  } while (0)
  if (grad_bf16) {
    if (pre_kind == kPreF32) NVFP4_RELU2_BWD(kPreF32, true);
    else if (pre_kind == kPreBf16) NVFP4_RELU2_BWD(kPreBf16, true);
    else NVFP4_RELU2_BWD(kPreF16, true);
  } else {
    if (pre_kind == kPreF32) NVFP4_RELU2_BWD(kPreF32, false);
    else if (pre_kind == kPreBf16) NVFP4_RELU2_BWD(kPreBf16, false);
    else NVFP4_RELU2_BWD(kPreF16, false);
  }
#undef NVFP4_RELU2_BWD
#undef NVFP4_RELU2_BWD_A
  NVFP4_RETURN_LAST();
}

int launch_decode(cudaStream_t s, const uint8_t* bytes, const uint8_t* scales, const float* gscales, int rowwise,
                  int transpose, float* out, uint32_t rows, uint32_t cols) {
  const uint64_t n = static_cast<uint64_t>(rows) * cols;
  if (n == 0) return 0;
  decode_kernel<<<blocks_for(n, 256), 256, 0, s>>>(bytes, scales, gscales, out, rows, cols, rowwise, transpose);
  NVFP4_RETURN_LAST();
}

int launch_scale_pack(cudaStream_t s, const uint8_t* logical, uint8_t* packed, uint32_t mn, uint32_t k_dim) {
  const uint32_t padded = (mn + 127u) / 128u * 128u, kg = k_dim / 16;
  const uint64_t total = static_cast<uint64_t>(padded) * kg;
  if (total == 0) return 0;
  scale_pack_kernel<<<blocks_for(total, 256, 148 * 16), 256, 0, s>>>(logical, packed, mn, padded, kg);
  NVFP4_RETURN_LAST();
}

int launch_pad_u4_rows(cudaStream_t s, const uint8_t* src, uint8_t* dst, uint32_t rows, uint32_t padded_rows,
                       uint32_t cols) {
  const uint64_t sb = static_cast<uint64_t>(rows) * cols / 2, db = static_cast<uint64_t>(padded_rows) * cols / 2;
  if (db == 0) return 0;
  pad_u4_rows_kernel<<<blocks_for(db, 256, 148 * 16), 256, 0, s>>>(src, dst, sb, db);
  NVFP4_RETURN_LAST();
}

int launch_pad_f32(cudaStream_t s, const float* src, float* dst, uint32_t rows, uint32_t cols, uint32_t padded_rows,
                   uint32_t padded_cols, int transpose) {
  const uint64_t total = static_cast<uint64_t>(padded_rows) * padded_cols;
  if (total == 0) return 0;
  if (transpose)
    pad_f32_kernel<true><<<blocks_for(total, 256, 148 * 16), 256, 0, s>>>(src, dst, rows, cols, padded_rows, padded_cols);
  else
    pad_f32_kernel<false><<<blocks_for(total, 256, 148 * 16), 256, 0, s>>>(src, dst, rows, cols, padded_rows, padded_cols);
  NVFP4_RETURN_LAST();
}

int launch_crop_f32(cudaStream_t s, const float* src, float* dst, uint32_t rows, uint32_t src_cols, uint32_t dst_cols) {
  const uint64_t total = static_cast<uint64_t>(rows) * dst_cols;
  if (total == 0) return 0;
  crop_f32_kernel<<<blocks_for(total, 256, 148 * 16), 256, 0, s>>>(src, dst, rows, src_cols, dst_cols);
  NVFP4_RETURN_LAST();
}

int launch_postop(cudaStream_t s, float* raw, float* other, const uint8_t* bias_bytes, const uint8_t* bias_scales,
                  const float* bias_gs, uint32_t rows, uint32_t cols, int mode) {
  const uint64_t n = static_cast<uint64_t>(rows) * cols;
  if (n == 0) return 0;
  postop_kernel<<<blocks_for(n, 256, 148 * 16), 256, 0, s>>>(raw, other, bias_bytes, bias_scales, bias_gs, n, cols, mode);
  NVFP4_RETURN_LAST();
}

int launch_bias_grad(cudaStream_t s, const void* e, int dtype, float* dbias, uint32_t tokens, uint32_t n) {
  if (n == 0) return 0;
  if (dtype == NVFP4_DTYPE_F32)
    bias_grad_kernel<float><<<blocks_for(n, 32), 256, 0, s>>>(static_cast<const float*>(e), dbias, tokens, n);
  else
    bias_grad_kernel<__nv_bfloat16>
        <<<blocks_for(n, 32), 256, 0, s>>>(static_cast<const __nv_bfloat16*>(e), dbias, tokens, n);
  NVFP4_RETURN_LAST();
}

}  // namespace nvfp4
