// Device helpers shared by the NVFP4 quantizer / codec kernels (sm_100a).
//
// Bit-exactness contract: every translation unit that includes this header for
// quantizer math is compiled with -fmad=false, so `a * b + c` is never
// contracted; divisions are IEEE (nvcc default -prec-div=true); denormals are
// kept (-ftz=false).  The narrow-format conversions are the same PTX
// instructions the reference's kernels issue (crates/cuda-kernels/src/utils/
// nvfp4/cast.rs:4-32 and utils/nvfp4/quant/kernels/convert.rs:66-93).
#pragma once

#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace nvfp4 {

constexpr float kDenomEps = 1.0e-20f;  // convert.rs:5

// ---- narrow-format conversions ---------------------------------------------

// cvt.rn.satfinite.e2m1x2.f32 d, hi, lo : `hi` lands in the upper nibble.
__device__ __forceinline__ uint32_t cvt_e2m1x2(float hi, float lo) {
  uint16_t r;
  asm("{ .reg .b8 t; cvt.rn.satfinite.e2m1x2.f32 t, %1, %2; cvt.u16.u8 %0, t; }" : "=h"(r) : "f"(hi), "f"(lo));
  return r;
}

// One value to an E4M3 byte (cvt.rn.satfinite.e4m3x2.f32 d, 0, v -> low byte).
__device__ __forceinline__ uint32_t cvt_e4m3(float v) {
  uint16_t r;
  asm("cvt.rn.satfinite.e4m3x2.f32 %0, %1, %2;" : "=h"(r) : "f"(0.0f), "f"(v));
  return r & 0xffu;
}

// A byte holding two E2M1 nibbles -> the two values (low nibble first).
__device__ __forceinline__ float2 e2m1x2_values(uint32_t byte) {
  uint32_t h2;
  asm("{ .reg .b8 t; cvt.u8.u32 t, %1; cvt.rn.f16x2.e2m1x2 %0, t; }" : "=r"(h2) : "r"(byte));
  __half2 h = *reinterpret_cast<__half2*>(&h2);
  return __half22float2(h);
}

// Eight values to four E2M1x2 bytes in one word (byte k holds elements 2k and 2k+1, the even
// element in the low nibble).  The bytes are packed in PTX so that no separate mask or shift
// instruction is needed after the conversions.
__device__ __forceinline__ uint32_t cvt_e2m1x8(float x0, float x1, float x2, float x3, float x4, float x5, float x6,
                                               float x7) {
  uint32_t r;
  asm("{\n\t.reg .b8 b0, b1, b2, b3;\n\t"
      "cvt.rn.satfinite.e2m1x2.f32 b0, %2, %1;\n\t"
      "cvt.rn.satfinite.e2m1x2.f32 b1, %4, %3;\n\t"
      "cvt.rn.satfinite.e2m1x2.f32 b2, %6, %5;\n\t"
      "cvt.rn.satfinite.e2m1x2.f32 b3, %8, %7;\n\t"
      "mov.b32 %0, {b0, b1, b2, b3};\n\t}"
      : "=r"(r)
      : "f"(x0), "f"(x1), "f"(x2), "f"(x3), "f"(x4), "f"(x5), "f"(x6), "f"(x7));
  return r;
}
// Decoding goes byte by byte through an explicit byte extract: unpacking the word with
// mov.b32 {b0,b1,b2,b3} right after the pack above was measured to return zeros for some bytes
// (the assembler forwards the 8-bit temporaries without their masking).
__device__ __forceinline__ void e2m1x8_values(uint32_t word, float (&q)[8]) {
#pragma unroll
  for (int k = 0; k < 4; ++k) {
    const float2 f = e2m1x2_values(__byte_perm(word, 0u, 0x4440u | k));
    q[2 * k] = f.x;
    q[2 * k + 1] = f.y;
  }
}

__device__ __forceinline__ float e2m1_value(uint32_t nibble) { return e2m1x2_values(nibble & 0xfu).x; }

__device__ __forceinline__ float e4m3_value(uint32_t bits) {
  uint32_t h2;
  asm("cvt.rn.f16x2.e4m3x2 %0, %1;" : "=r"(h2) : "h"(static_cast<uint16_t>(bits & 0xffu)));
  __half2 h = *reinterpret_cast<__half2*>(&h2);
  return __low2float(h);
}

// ---- small math helpers (convert.rs:8-35, float_ptx.rs:113-115) -------------

__device__ __forceinline__ float nz(float v) { return v == 0.0f ? 1.0f : v; }

__device__ __forceinline__ float inv_scale(float scale, float gs) {
  return 1.0f / (nz(scale) * nz(gs) + kDenomEps);
}

// max.f32: a NaN operand is dropped, exactly like the reference's max_f32.
__device__ __forceinline__ float max_f32(float a, float b) {
  float r;
  asm("max.f32 %0, %1, %2;" : "=f"(r) : "f"(a), "f"(b));
  return r;
}

// Sum of 16 values in the order of the reference's xor-8,4,2,1 shuffle butterfly
// (utils/warp_reduce.rs:33-38): every lane of that butterfly ends with this value.
__device__ __forceinline__ float butterfly_sum16(const float (&e)[16]) {
  float a0 = e[0] + e[8], a1 = e[1] + e[9], a2 = e[2] + e[10], a3 = e[3] + e[11];
  float a4 = e[4] + e[12], a5 = e[5] + e[13], a6 = e[6] + e[14], a7 = e[7] + e[15];
  float b0 = a0 + a4, b1 = a1 + a5, b2 = a2 + a6, b3 = a3 + a7;
  float c0 = b0 + b2, c1 = b1 + b3;
  return c0 + c1;
}

// ---- packed f32x2 arithmetic (sm_100): two independent IEEE f32 operations per instruction.
// Each lane rounds exactly like the scalar add / sub / mul, so results stay bit-exact; the
// quantizers are instruction-issue bound and this halves their FP32 instruction count.
typedef unsigned long long f32x2_t;
__device__ __forceinline__ f32x2_t pack2(float lo, float hi) {
  f32x2_t r;
  asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "f"(lo), "f"(hi));
  return r;
}
__device__ __forceinline__ void unpack2(f32x2_t v, float& lo, float& hi) {
  asm("mov.b64 {%0, %1}, %2;" : "=f"(lo), "=f"(hi) : "l"(v));
}
__device__ __forceinline__ f32x2_t add2(f32x2_t a, f32x2_t b) {
  f32x2_t r;
  asm("add.rn.f32x2 %0, %1, %2;" : "=l"(r) : "l"(a), "l"(b));
  return r;
}
__device__ __forceinline__ f32x2_t sub2(f32x2_t a, f32x2_t b) {
  f32x2_t r;
  asm("sub.rn.f32x2 %0, %1, %2;" : "=l"(r) : "l"(a), "l"(b));
  return r;
}
__device__ __forceinline__ f32x2_t mul2(f32x2_t a, f32x2_t b) {
  f32x2_t r;
  asm("mul.rn.f32x2 %0, %1, %2;" : "=l"(r) : "l"(a), "l"(b));
  return r;
}
// A packed product that is going to feed a packed add / sub.  The assembler contracts
// mul.rn.f32x2 followed by add.rn.f32x2 into one fused multiply-add even with contraction
// switched off (measured: the scalar forms are left alone), which would skip the rounding of
// the product.  Written as fma(a, b, -0) with the -0 pair read from constant memory, the
// product is rounded once, exactly like a multiply (x + -0 == x for every x, signed zeros
// included), and a fused multiply-add cannot be contracted any further.
static __constant__ unsigned long long kNegZeroPair = 0x8000000080000000ull;
__device__ __forceinline__ f32x2_t mul2_rounded(f32x2_t a, f32x2_t b) {
  f32x2_t r;
  asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(r) : "l"(a), "l"(b), "l"(kNegZeroPair));
  return r;
}
__device__ __forceinline__ f32x2_t fma2(f32x2_t a, f32x2_t b, f32x2_t c) {
  f32x2_t r;
  asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(r) : "l"(a), "l"(b), "l"(c));
  return r;
}
// Packed form of butterfly_sum16: both lanes in the xor-8,4,2,1 order.
__device__ __forceinline__ f32x2_t butterfly_sum16_x2(const f32x2_t (&e)[16]) {
  f32x2_t a0 = add2(e[0], e[8]), a1 = add2(e[1], e[9]), a2 = add2(e[2], e[10]), a3 = add2(e[3], e[11]);
  f32x2_t a4 = add2(e[4], e[12]), a5 = add2(e[5], e[13]), a6 = add2(e[6], e[14]), a7 = add2(e[7], e[15]);
  f32x2_t b0 = add2(a0, a4), b1 = add2(a1, a5), b2 = add2(a2, a6), b3 = add2(a3, a7);
  return add2(add2(b0, b2), add2(b1, b3));
}
// max(m, |a|, |b|) with max.f32 semantics (NaN operands dropped).
__device__ __forceinline__ float max3_abs(float m, float a, float b) {
  float r;
  asm("{\n\t.reg .f32 x, y;\n\tabs.f32 x, %2;\n\tabs.f32 y, %3;\n\tmax.f32 %0, %1, x, y;\n\t}"
      : "=f"(r)
      : "f"(m), "f"(a), "f"(b));
  return r;
}

// NVFP4 element: (e2m1 * e4m3) * global_scale, even index = low nibble
// (utils/nvfp4/tensor.rs:48-57).
__device__ __forceinline__ float nvfp4_value(const uint8_t* __restrict__ bytes, const uint8_t* __restrict__ scales,
                                             float gs, size_t index) {
  uint32_t byte = bytes[index >> 1];
  uint32_t nib = (index & 1) ? (byte >> 4) : (byte & 0xfu);
  return e2m1_value(nib) * e4m3_value(scales[index >> 4]) * gs;
}

// ---- counter RNG (utils/nvfp4/quant/kernels/ms_eden/random.rs) --------------

__device__ __forceinline__ uint32_t hash_u32(uint32_t v) {
  v ^= v >> 16;
  v *= 0x7feb352du;
  v ^= v >> 15;
  v *= 0x846ca68bu;
  return v ^ (v >> 16);
}
__device__ __forceinline__ bool random_sign_negative(uint32_t seed, uint32_t index) {
  return (hash_u32(seed ^ index) & 1u) != 0;
}
__device__ __forceinline__ float random_unit_f32(uint32_t seed, uint32_t index) {
  return static_cast<float>(hash_u32(seed ^ index) & 0x00ffffffu) * 5.9604645e-8f;
}

// ---- packed scale-factor layout ---------------------------------------------
// 512-byte tiles ordered [row_block of 128][k_atom of 64 elements]; inside a tile the byte
// of (row, k_group) is (row % 32) * 16 + (row / 32 % 4) * 4 + k_group % 4.  This is the
// layout tcgen05.cp (32x128b.warpx4) moves into tensor memory unchanged, and it is byte
// identical to the reference's block-major packed plane
// (utils/nvfp4_tma_matmul/cute.rs:448-467).
__host__ __device__ __forceinline__ size_t packed_scale_offset(uint32_t row, uint32_t k_group, uint32_t k_atoms) {
  uint32_t blk = row >> 7, in_blk = row & 127u;
  return (static_cast<size_t>(blk) * k_atoms + (k_group >> 2)) * 512u + (in_blk & 31u) * 16u + (in_blk >> 5) * 4u +
         (k_group & 3u);
}

// ---- loads -------------------------------------------------------------------

template <typename T>
struct Load16;  // loads 16 consecutive elements (64-byte / 32-byte aligned) as f32

template <>
struct Load16<float> {
  __device__ __forceinline__ static void run(const float* p, float (&v)[16]) {
    const float4* q = reinterpret_cast<const float4*>(p);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      float4 t = __ldg(q + i);
      v[4 * i] = t.x;
      v[4 * i + 1] = t.y;
      v[4 * i + 2] = t.z;
      v[4 * i + 3] = t.w;
    }
  }
};

template <>
struct Load16<__nv_bfloat16> {
  __device__ __forceinline__ static void run(const __nv_bfloat16* p, float (&v)[16]) {
    const uint4* q = reinterpret_cast<const uint4*>(p);
#pragma unroll
    for (int i = 0; i < 2; ++i) {
      uint4 t = __ldg(q + i);
      uint32_t w[4] = {t.x, t.y, t.z, t.w};
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        v[8 * i + 2 * j] = __uint_as_float(w[j] << 16);
        v[8 * i + 2 * j + 1] = __uint_as_float(w[j] & 0xffff0000u);
      }
    }
  }
};

template <typename T>
__device__ __forceinline__ float load_as_f32(const T* p, size_t i);
template <>
__device__ __forceinline__ float load_as_f32<float>(const float* p, size_t i) {
  return __ldg(p + i);
}
template <>
__device__ __forceinline__ float load_as_f32<__nv_bfloat16>(const __nv_bfloat16* p, size_t i) {
  return __uint_as_float(static_cast<uint32_t>(__ldg(reinterpret_cast<const unsigned short*>(p) + i)) << 16);
}

}  // namespace nvfp4
