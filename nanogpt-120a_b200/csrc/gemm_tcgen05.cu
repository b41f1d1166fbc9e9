// NVFP4 block-scaled projection GEMM for sm_100a.
//
//   out[m][n] = epilogue( (sum_k A[m][k]*sa[m][k/16] * B[n][k]*sb[n][k/16]) * weight * ga * gb )
//
// Semantics follow the reference's TMA GEMM and its post-op kernels
// (crates/cuda-kernels/src/utils/nvfp4_tma_matmul/kernels.rs:310-351,538-568 and
// gpt/projection_postop.rs:97-162); the engine is new: a persistent, warp-specialised
// kernel in which
//   warp 0      streams A / B nibble tiles with TMA (128-byte swizzle) and the packed
//               scale-factor tiles with bulk copies into a shared-memory ring,
//   warp 1      issues tcgen05.mma.kind::mxf4nvf4.block_scale (128 x BLOCK_N x 64 per
//               instruction), FP32 accumulators in tensor memory,
//   warp 2      owns the tensor-memory allocation,
//   warps 4..7 and 12..15  two epilogue groups: drain accumulators (tcgen05.ld), apply global
//               scales / bias / ReLU^2 / residual, cast and store; the groups take alternate
//               128-byte column sub-tiles of a tile (a warp reaches the tensor-memory lanes of
//               its index modulo four, so warps w and w + 8 share a lane quadrant),
//   warps 8..11 move the scale factors shared -> tensor memory (tcgen05.st).
// Three tile widths.  BLOCK_N = 128 and 192 double buffer the accumulator (2 x 192 accumulator
// columns + 3 x 40 scale-factor columns fill the 512 columns of tensor memory), so the epilogue of
// one tile overlaps the main loop of the next; the 256-column tile has one accumulator buffer,
// which every epilogue warp hands back as soon as its last tcgen05.ld of the tile has landed in
// registers.  Every mbarrier wait is bounded: on expiry the kernel records a status word, drains,
// frees its tensor memory and returns.
//
// No thread-block clusters, no multicast: every load reads this GPU's own memory.
#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_runtime.h>

#include <atomic>
#include <cstdlib>
#include <cstring>
#include <mutex>
#include <unordered_map>
#include <vector>

#include "kernels.h"

namespace nvfp4 {

__device__ uint32_t g_device_status = 0;

namespace {

constexpr int kRowBlock = 128;                    // rows of one MMA, one scale-factor block, one epilogue sub-tile
constexpr int kBlockKBytes = 128;                 // 256 nibbles = one 128-byte swizzle row
constexpr int kKAtomsPerStage = 4;                // 64-element k-atoms (one MMA each per row block) per stage
constexpr int kAHalfBytes = kRowBlock * kBlockKBytes;  // A rows of one MMA in a stage
constexpr int kSfTileBytes = 512;                 // 128 rows x 4 scale bytes
constexpr int kSfBlockStageBytes = kKAtomsPerStage * kSfTileBytes;  // one 128-row scale block of a stage
constexpr int kStoreStageBytes = kRowBlock * 128;  // one epilogue sub-tile: 128 rows x 128 bytes
constexpr int kTmemCols = 512;
constexpr int kMaxStages = 8;
constexpr int kSmemBudget = 227 * 1024;
constexpr int kThreads = 512;
constexpr uint64_t kDefaultWaitTimeoutNs = 2000000000ull;  // 2 s

constexpr uint32_t kStatusProducerTimeout = 1u, kStatusMmaTimeout = 2u, kStatusEpilogueTimeout = 4u;

// Tile shapes: 128 x {128, 192, 256} and the tall 256 x 192.  The tall tile issues two MMAs per k-atom (rows
// 0..127 and 128..255 of the A stage against the same B stage), so a stage's B bytes feed twice the flops:
// streaming GEMMs are bound by the operand bytes an SM can pull from L2, and the tall tile moves 21 % fewer of
// them per flop than 128 x 256.  Its two 192-column accumulators and two scale-factor column sets fill tensor
// memory (2 x 192 + 2 x 56 = 496 of 512 columns), so the accumulator is single buffered.
template <int kBlockM, int kBlockN>
struct Cfg {
  static constexpr int kMHalves = kBlockM / kRowBlock;
  static_assert(kBlockM == 128 || (kBlockM == 256 && kBlockN == 192), "unsupported tile shape");
  static constexpr int kAStageBytes = kMHalves * kAHalfBytes;
  static constexpr int kSfaStageBytes = kMHalves * kSfBlockStageBytes;
  // 128-row scale-factor blocks of B a tile can touch: a 192-column tile starts either on a block
  // boundary or in the middle of a block, and spans two blocks either way
  static constexpr int kSfBlocks = (kBlockN + 127) / 128;
  static constexpr int kBStageBytes = kBlockN * kBlockKBytes;
  static constexpr int kSfbStageBytes = kSfBlocks * kSfBlockStageBytes;
  static constexpr int kAccStages = (kBlockN == 256 || kMHalves == 2) ? 1 : 2;
  static constexpr int kAccCols = kMHalves * kBlockN;  // columns of one accumulator buffer (row halves side by side)
  // Scale factors live in a ring of column sets behind the accumulators (one set per k-tile), so
  // the copies for the next k-tile never overwrite columns an MMA in flight reads.
  static constexpr int kSfaSetCols = kMHalves * 4 * kKAtomsPerStage;
  static constexpr int kSfbColsPerAtom = kBlockN / 32;
  static constexpr int kSfSetCols = kSfaSetCols + kSfbColsPerAtom * kKAtomsPerStage;
  static constexpr int kSfSets = kMHalves == 2 ? 2 : (kBlockN == 192 ? 3 : 4);
  static constexpr int kTmemSfa = kAccStages * kAccCols;   // A scale factors of set 0
  static constexpr int kTmemSfb = kTmemSfa + kSfaSetCols;  // B scale factors of set 0
  static constexpr int kStreamStageBytes = kAStageBytes + kBStageBytes + kSfaStageBytes + kSfbStageBytes;
  static constexpr int kResidentStageBytes = kAStageBytes + kSfaStageBytes;
  static constexpr int kPanelSlotBytes = kBStageBytes + kSfbStageBytes;
  // epilogue staging ring: deep for the narrow tile (short-K GEMMs are epilogue bound), shallow for
  // the wide ones (long-K GEMMs need the shared memory for pipeline stages)
  static constexpr int kStoreBufs = kBlockN == 128 ? 4 : 2;
  static constexpr int kBiasSlots = (kBlockN + 127) / 128;  // bias values a thread of an epilogue group fetches
  static constexpr int kFixedBytes =
      1024 /*alignment slack*/ + kStoreBufs * kStoreStageBytes + 512 /*barriers*/ +
      2 * kBlockN * 4 /*bias of the tile, one copy per epilogue group*/;
  static_assert(kTmemSfa + kSfSets * kSfSetCols <= kTmemCols, "tensor memory overflow");
};

struct GemmParams {
  const uint8_t* sfa;
  const uint8_t* sfb;
  const float* a_global;
  const float* b_global;
  const float* bias;
  // NVFP4-encoded bias [n] (bytes, logical scale bytes, f32[1] global scale): used when bias == nullptr
  const uint8_t* bias_bytes;
  const uint8_t* bias_scales;
  const float* bias_global;
  float* row_amax;  // optional f32[m]: max over the row of relu(stored value)^2 (red.max, zeroed by the launcher)
  void* out;
  void* aux;
  uint32_t m, n, k, ldo;
  uint32_t num_m_blocks, num_n_blocks, k_atoms, sfa_blocks128, sfb_blocks128;
  uint32_t k_splits, k_tiles_per_split, num_k_tiles;
  uint32_t stages;  // depth of the A (and, when streaming, B) ring
  int b_resident;   // the B panel of a column block stays in shared memory (short K)
  uint32_t resident_cpn;  // resident mode: CTAs per column block (0 = contiguous tile ranges instead)
  int mode, epilogue, vec_store, tma_store;
  float weight;
  uint64_t wait_timeout_ns;  // limit of every mbarrier wait
  uint32_t debug_flags;      // bit 0: CTA 0 never loads its first k-tile (exercises the bounded waits)
#ifdef NVFP4_GEMM_TRACE
  unsigned long long* trace;  // measurement builds only: [5 roles][1024] (clock << 8 | tag) records of CTA 0
#endif
};

// Measurement builds (-DNVFP4_GEMM_TRACE) record a time line of CTA 0: one (SM clock, tag) word per event and
// role (0 producer, 1 MMA issuer, 2 first scale-factor warp, 3 / 4 epilogue groups).  Product builds compile
// the macro away.
#ifdef NVFP4_GEMM_TRACE
#define GEMM_TRACE(role, tag, leader)                                                                      \
  do {                                                                                                     \
    if (p.trace && blockIdx.x == 0 && (leader)) {                                                          \
      const uint32_t trace_i = trace_n++;                                                                  \
      if (trace_i < 1024u) p.trace[(role) * 1024u + trace_i] = (static_cast<unsigned long long>(clock64()) << 8) | (tag); \
    }                                                                                                      \
  } while (0)
#else
#define GEMM_TRACE(role, tag, leader) do { } while (0)
#endif

// ---- PTX wrappers ---------------------------------------------------------------------------

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return static_cast<uint32_t>(__cvta_generic_to_shared(p)); }

__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(bar), "r"(parity)
      : "memory");
  return ok != 0;
}
__device__ __forceinline__ uint64_t global_timer_ns() {
  uint64_t t;
  asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
  return t;
}

// Bounded wait.  Returns false when the CTA is aborting (this waiter timed out, or another
// role already did); the caller then leaves its loop and goes to the common teardown.
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, volatile uint32_t* abort_flag,
                                          uint32_t status_bit, uint64_t timeout_ns) {
  if (mbar_try_wait(bar, parity)) return true;
  const uint64_t t0 = global_timer_ns();
  uint32_t polls = 0;
  while (true) {
    if (mbar_try_wait(bar, parity)) return true;
    if ((++polls & 255u) == 0) {
      if (*abort_flag) return false;
      if (global_timer_ns() - t0 > timeout_ns) {
        *abort_flag = 1;
        atomicOr(&g_device_status, status_bit);
        return false;
      }
    }
  }
}

__device__ __forceinline__ void tma_load_2d(uint32_t dst, const CUtensorMap* map, uint32_t bar, int32_t x, int32_t y) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];" ::"r"(dst),
      "l"(reinterpret_cast<uint64_t>(map)), "r"(bar), "r"(x), "r"(y)
      : "memory");
}
__device__ __forceinline__ void bulk_load(uint32_t dst, const void* src, uint32_t bytes, uint32_t bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(dst),
               "l"(reinterpret_cast<uint64_t>(src)), "r"(bytes), "r"(bar)
               : "memory");
}

__device__ __forceinline__ void tma_store_2d(const CUtensorMap* map, uint32_t src, int32_t x, int32_t y) {
  asm volatile("cp.async.bulk.tensor.2d.global.shared::cta.bulk_group [%0, {%2, %3}], [%1];" ::"l"(
                   reinterpret_cast<uint64_t>(map)),
               "r"(src), "r"(x), "r"(y)
               : "memory");
}
__device__ __forceinline__ void tma_reduce_add_2d(const CUtensorMap* map, uint32_t src, int32_t x, int32_t y) {
  asm volatile("cp.reduce.async.bulk.tensor.2d.global.shared::cta.add.tile.bulk_group [%0, {%2, %3}], [%1];" ::"l"(
                   reinterpret_cast<uint64_t>(map)),
               "r"(src), "r"(x), "r"(y)
               : "memory");
}
__device__ __forceinline__ void bulk_commit_group() { asm volatile("cp.async.bulk.commit_group;" ::: "memory"); }
template <int kPending>
__device__ __forceinline__ void bulk_wait_group_read() {
  asm volatile("cp.async.bulk.wait_group.read %0;" ::"n"(kPending) : "memory");
}
__device__ __forceinline__ void bulk_wait_group0() { asm volatile("cp.async.bulk.wait_group 0;" ::: "memory"); }
__device__ __forceinline__ void fence_proxy_async_smem() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }
// one named barrier per epilogue warp group (ids 1 and 2), 128 threads each
__device__ __forceinline__ void epilogue_barrier(uint32_t group) {
  asm volatile("bar.sync %0, 128;" ::"r"(group + 1u) : "memory");
}

// Named barrier of one epilogue group that also ANDs a predicate over its 128 threads: the decision to
// go on with a tile or to leave for the teardown is then the same in every thread of the group, so no
// thread can be left alone in a later bar.sync.
__device__ __forceinline__ bool epilogue_all(uint32_t group, bool pred) {
  uint32_t r;
  asm volatile(
      "{\n\t.reg .pred p, q;\n\t"
      "setp.ne.b32 p, %2, 0;\n\t"
      "bar.red.and.pred q, %1, 128, p;\n\t"
      "selp.u32 %0, 1, 0, q;\n\t}"
      : "=r"(r)
      : "r"(group + 1u), "r"(static_cast<uint32_t>(pred))
      : "memory");
  return r != 0;
}

__device__ __forceinline__ bool elect_one() {
  uint32_t pred;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "elect.sync _|p, 0xffffffff;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(pred));
  return pred != 0;
}
__device__ __forceinline__ void tcgen05_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tcgen05_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tcgen05_commit(uint32_t bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void tcgen05_mma_nvf4(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b, uint32_t idesc,
                                                 uint32_t accumulate, uint32_t tmem_sfa, uint32_t tmem_sfb) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::mxf4nvf4.block_scale.block16 [%0], %1, %2, %3, [%5], [%6], p;\n\t}" ::"r"(tmem_d),
      "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate), "r"(tmem_sfa), "r"(tmem_sfb)
      : "memory");
}
__device__ __forceinline__ void tcgen05_ld_32x32b_x32(uint32_t taddr, uint32_t (&r)[32]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
      "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
        "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]),
        "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]),
        "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
      : "r"(taddr)
      : "memory");
}
// Packed FP32 pairs for the epilogue arithmetic: one instruction per two accumulator columns, each lane
// rounded exactly like the scalar operation.
__device__ __forceinline__ uint64_t pack_f32x2(float lo, float hi) {
  uint64_t r;
  asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "f"(lo), "f"(hi));
  return r;
}
__device__ __forceinline__ void fma_f32x2(float& lo, float& hi, uint32_t a_lo, uint32_t a_hi, uint64_t b, uint64_t c) {
  asm("{\n\t.reg .b64 a, d;\n\tmov.b64 a, {%2, %3};\n\tfma.rn.f32x2 d, a, %4, %5;\n\tmov.b64 {%0, %1}, d;\n\t}"
      : "=f"(lo), "=f"(hi)
      : "r"(a_lo), "r"(a_hi), "l"(b), "l"(c));
}
__device__ __forceinline__ void mul_f32x2(float& lo, float& hi, float a_lo, float a_hi, uint64_t b) {
  asm("{\n\t.reg .b64 a, d;\n\tmov.b64 a, {%2, %3};\n\tmul.rn.f32x2 d, a, %4;\n\tmov.b64 {%0, %1}, d;\n\t}"
      : "=f"(lo), "=f"(hi)
      : "f"(a_lo), "f"(a_hi), "l"(b));
}
__device__ __forceinline__ void square_f32x2(float& lo, float& hi) {
  asm("{\n\t.reg .b64 a;\n\tmov.b64 a, {%0, %1};\n\tmul.rn.f32x2 a, a, a;\n\tmov.b64 {%0, %1}, a;\n\t}"
      : "+f"(lo), "+f"(hi));
}
__device__ __forceinline__ void tcgen05_st_x4(uint32_t taddr, const uint32_t* r) {
  asm volatile("tcgen05.st.sync.aligned.32x32b.x4.b32 [%0], {%1, %2, %3, %4};" ::"r"(taddr), "r"(r[0]), "r"(r[1]),
               "r"(r[2]), "r"(r[3])
               : "memory");
}
__device__ __forceinline__ void tcgen05_st_x2(uint32_t taddr, const uint32_t* r) {
  asm volatile("tcgen05.st.sync.aligned.32x32b.x2.b32 [%0], {%1, %2};" ::"r"(taddr), "r"(r[0]), "r"(r[1]) : "memory");
}
__device__ __forceinline__ void tcgen05_st_x8(uint32_t taddr, const uint32_t* r) {
  asm volatile("tcgen05.st.sync.aligned.32x32b.x8.b32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8};" ::"r"(taddr), "r"(r[0]),
               "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7])
               : "memory");
}
__device__ __forceinline__ void tcgen05_st_x16(uint32_t taddr, const uint32_t* r) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], "
      "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16};" ::"r"(taddr),
      "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]), "r"(r[8]), "r"(r[9]),
      "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15])
      : "memory");
}
__device__ __forceinline__ void tcgen05_wait_ld() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }

// Shared-memory matrix descriptors (sm_100 format: version 1 in bits 46..47).
// A / B tiles: K-major, 128-byte swizzle, 8-row groups 1024 bytes apart; the K offset of a
// 64-element MMA inside the swizzle row (32 bytes) is added to the start address.
__device__ __forceinline__ uint64_t make_ab_desc(uint32_t smem_addr) {
  uint64_t d = 0;
  d |= static_cast<uint64_t>((smem_addr & 0x3FFFFu) >> 4);
  d |= static_cast<uint64_t>(1024u >> 4) << 32;  // stride byte offset
  d |= 1ull << 46;                               // descriptor version
  d |= 2ull << 61;                               // SWIZZLE_128B
  return d;
}
// Instruction descriptor of kind::mxf4nvf4: E2M1 x E2M1, UE4M3 scales, K-major A and B,
// M = 128, N = kBlockN, K = 64.
template <int kBlockN>
__device__ __forceinline__ constexpr uint32_t make_idesc() {
  return (1u << 7) | (1u << 10) | (static_cast<uint32_t>(kBlockN >> 3) << 17) | (0u << 23) |
         (static_cast<uint32_t>(kRowBlock >> 4) << 24);
}

// Bias of one output column: an f32 vector, or an NVFP4-encoded one decoded as the reference's post-op
// kernels decode it, (e2m1 * e4m3) * global_scale (utils/nvfp4/tensor.rs:48-57, gpt/projection_postop.rs:97-115).
__device__ __forceinline__ float bias_value(const GemmParams& p, uint32_t col) {
  if (p.bias) return __ldg(p.bias + col);
  const uint32_t byte = __ldg(p.bias_bytes + (col >> 1));
  const uint32_t nib = (col & 1u) ? (byte >> 4) : (byte & 0xfu);
  uint32_t h2;
  asm("{ .reg .b8 t; cvt.u8.u32 t, %1; cvt.rn.f16x2.e2m1x2 %0, t; }" : "=r"(h2) : "r"(nib));
  const float q = __low2float(*reinterpret_cast<__half2*>(&h2));
  uint32_t s2;
  asm("cvt.rn.f16x2.e4m3x2 %0, %1;" : "=r"(s2) : "h"(static_cast<uint16_t>(__ldg(p.bias_scales + (col >> 4)))));
  const float sc = __low2float(*reinterpret_cast<__half2*>(&s2));
  return __fmul_rn(__fmul_rn(q, sc), __ldg(p.bias_global));
}

// ---- epilogue stores ------------------------------------------------------------------------

template <typename OutT>
__device__ __forceinline__ void store_row32(OutT* dst, const float (&v)[32], uint32_t valid, bool vec);

template <>
__device__ __forceinline__ void store_row32<float>(float* dst, const float (&v)[32], uint32_t valid, bool vec) {
  if (vec && valid == 32) {
#pragma unroll
    for (int i = 0; i < 8; ++i)
      reinterpret_cast<float4*>(dst)[i] = make_float4(v[4 * i], v[4 * i + 1], v[4 * i + 2], v[4 * i + 3]);
  } else {
#pragma unroll
    for (int i = 0; i < 32; ++i)
      if (static_cast<uint32_t>(i) < valid) dst[i] = v[i];
  }
}
template <>
__device__ __forceinline__ void store_row32<__nv_bfloat16>(__nv_bfloat16* dst, const float (&v)[32], uint32_t valid,
                                                           bool vec) {
  if (vec && valid == 32) {
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      uint32_t w[4];
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        __nv_bfloat162 h = __floats2bfloat162_rn(v[8 * i + 2 * j], v[8 * i + 2 * j + 1]);
        w[j] = *reinterpret_cast<uint32_t*>(&h);
      }
      reinterpret_cast<uint4*>(dst)[i] = make_uint4(w[0], w[1], w[2], w[3]);
    }
  } else {
#pragma unroll
    for (int i = 0; i < 32; ++i)
      if (static_cast<uint32_t>(i) < valid) dst[i] = __float2bfloat16_rn(v[i]);
  }
}

template <typename OutT>
__device__ __forceinline__ float load_out(const OutT* p);
template <>
__device__ __forceinline__ float load_out<float>(const float* p) {
  return *p;
}
template <>
__device__ __forceinline__ float load_out<__nv_bfloat16>(const __nv_bfloat16* p) {
  return __bfloat162float(*p);
}

// One row (128 bytes) of an epilogue sub-tile into the staging buffer, 16-byte chunks XOR-swizzled
// with the row index exactly as the SWIZZLE_128B tensor map of the output expects.
template <typename OutT>
struct SubTile;
template <>
struct SubTile<float> {
  static constexpr int kCols = 32;
  __device__ __forceinline__ static void stage(uint32_t row_addr, uint32_t row, const float* v) {
#pragma unroll
    for (uint32_t c = 0; c < 8; ++c) {
      const uint32_t dst = row_addr + ((c ^ (row & 7u)) << 4);
      asm volatile("st.shared.v4.f32 [%0], {%1, %2, %3, %4};" ::"r"(dst), "f"(v[4 * c]), "f"(v[4 * c + 1]),
                   "f"(v[4 * c + 2]), "f"(v[4 * c + 3])
                   : "memory");
    }
  }
};
template <>
struct SubTile<__nv_bfloat16> {
  static constexpr int kCols = 64;
  __device__ __forceinline__ static void stage(uint32_t row_addr, uint32_t row, const float* v) {
#pragma unroll
    for (uint32_t c = 0; c < 8; ++c) {
      uint32_t w[4];
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        __nv_bfloat162 h = __floats2bfloat162_rn(v[8 * c + 2 * j], v[8 * c + 2 * j + 1]);
        w[j] = *reinterpret_cast<uint32_t*>(&h);
      }
      const uint32_t dst = row_addr + ((c ^ (row & 7u)) << 4);
      asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(dst), "r"(w[0]), "r"(w[1]), "r"(w[2]), "r"(w[3])
                   : "memory");
    }
  }
};

// ---- the kernel -----------------------------------------------------------------------------

// Shared-memory plan of one launch, chosen on the host (all offsets from the 1024-byte aligned
// base): A stages, B slots, SFA stages, SFB slots, two epilogue staging buffers, barriers.
// Streaming mode: one B slot per pipeline stage.  Resident mode (short K): the whole
// [kBlockN x K] B panel of the current column block stays in shared memory -- one slot per
// k-tile -- while a CTA walks down the row blocks, so only A tiles stream through the ring.
template <int kBlockM, int kBlockN, typename OutT, bool kTmaStore>
__global__ void __launch_bounds__(kThreads, 1)
    nvfp4_gemm_tcgen05_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_b,
                              const __grid_constant__ CUtensorMap tmap_out,
                              const __grid_constant__ CUtensorMap tmap_aux, const GemmParams p) {
  using C = Cfg<kBlockM, kBlockN>;
  constexpr int kMHalves = C::kMHalves;
  constexpr int kAStageBytes = C::kAStageBytes;
  constexpr int kSfaStageBytes = C::kSfaStageBytes;
  extern __shared__ uint8_t smem_raw[];
  const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t* smem_gen = smem_raw + (smem_base - smem_u32(smem_raw));

  const uint32_t stages = p.stages;
  const uint32_t b_slots = p.b_resident ? p.num_k_tiles : stages;
  const uint32_t smem_a = smem_base;
  const uint32_t smem_b = smem_a + stages * kAStageBytes;
  const uint32_t smem_sfa = smem_b + b_slots * C::kBStageBytes;
  const uint32_t smem_sfb = smem_sfa + stages * kSfaStageBytes;
  const uint32_t smem_store = smem_sfb + b_slots * C::kSfbStageBytes;  // staging ring, 16 KB buffers, 1024-byte aligned
  const uint32_t smem_bar = smem_store + C::kStoreBufs * kStoreStageBytes;
  // barrier block: full[8], empty[8], tmem_full[2], tmem_empty[2], b_full, b_empty, sf_full[4], sf_empty[4],
  // tmem base, abort flag
  const uint32_t smem_bias = smem_bar + 512;  // kBlockN floats per epilogue group
  const uint32_t bar_full = smem_bar;
  const uint32_t bar_empty = bar_full + 8 * kMaxStages;
  const uint32_t bar_tmem_full = bar_empty + 8 * kMaxStages;
  const uint32_t bar_tmem_empty = bar_tmem_full + 16;
  const uint32_t bar_b_full = bar_tmem_empty + 16;
  const uint32_t bar_b_empty = bar_b_full + 8;
  const uint32_t bar_sf_full = bar_b_empty + 8;
  const uint32_t bar_sf_empty = bar_sf_full + 8 * C::kSfSets;
  const uint32_t bar_mma_drain = bar_sf_empty + 8 * C::kSfSets;  // abort path only: issued MMAs have retired
  uint32_t* tmem_base_ptr =
      reinterpret_cast<uint32_t*>(smem_gen + (smem_bar - smem_base) + 8 * (2 * kMaxStages + 7 + 2 * C::kSfSets));
  volatile uint32_t* abort_flag = tmem_base_ptr + 1;

  const uint32_t warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
#ifdef NVFP4_GEMM_TRACE
  uint32_t trace_n = 0;
#endif

  if (threadIdx.x == 0) {
    asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(&tmap_a)) : "memory");
    asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(&tmap_b)) : "memory");
    if (kTmaStore) {
      asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(&tmap_out)) : "memory");
      if (p.aux) asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(&tmap_aux)) : "memory");
    }
    for (int s = 0; s < kMaxStages; ++s) {
      mbar_init(bar_full + 8 * s, 1);
      mbar_init(bar_empty + 8 * s, 1 + 4);  // the MMA commit and the four scale-factor warps
    }
    for (int s = 0; s < C::kSfSets; ++s) {
      mbar_init(bar_sf_full + 8 * s, 4);
      mbar_init(bar_sf_empty + 8 * s, 1);
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(bar_tmem_full + 8 * a, 1);
      mbar_init(bar_tmem_empty + 8 * a, 8);
    }
    mbar_init(bar_b_full, 1);
    mbar_init(bar_b_empty, 1);
    mbar_init(bar_mma_drain, 1);
    *abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 2) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_base_ptr)),
                 "r"(static_cast<uint32_t>(kTmemCols))
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    tcgen05_fence_before();
  }
  __syncthreads();
  tcgen05_fence_after();
  const uint32_t tmem_base = *tmem_base_ptr;

  // Work list, identical in every role.  Streaming: work items (tile, k-split) strided over the
  // grid, column block fastest (neighbouring CTAs share A rows in L2).  Resident: each CTA owns a
  // contiguous range of tiles ordered column block major, so its B panel changes at most a
  // couple of times.
  const uint32_t tiles_mn = p.num_m_blocks * p.num_n_blocks;
  uint32_t w_begin, w_end, w_step;
  if (p.b_resident && p.resident_cpn) {
    // Column block c / cpn, row blocks j, j + cpn, j + 2 cpn, ...: at any moment the CTAs of all
    // column blocks work on the same band of cpn row blocks, so whole output rows are written at
    // about the same time (full DRAM pages when L2 writes them back).
    const bool has_work = blockIdx.x < p.resident_cpn * p.num_n_blocks;
    w_begin = blockIdx.x % p.resident_cpn;
    w_end = has_work ? p.num_m_blocks : 0;
    w_step = p.resident_cpn;
  } else if (p.b_resident) {
    w_begin = static_cast<uint32_t>(static_cast<uint64_t>(tiles_mn) * blockIdx.x / gridDim.x);
    w_end = static_cast<uint32_t>(static_cast<uint64_t>(tiles_mn) * (blockIdx.x + 1) / gridDim.x);
    w_step = 1;
  } else {
    w_begin = blockIdx.x;
    w_end = tiles_mn * p.k_splits;
    w_step = gridDim.x;
  }
  auto decode = [&](uint32_t w, uint32_t& m_blk, uint32_t& n_blk, uint32_t& split) {
    if (p.b_resident && p.resident_cpn) {
      n_blk = blockIdx.x / p.resident_cpn;
      m_blk = w;
      split = 0;
    } else if (p.b_resident) {
      n_blk = w / p.num_m_blocks;
      m_blk = w - n_blk * p.num_m_blocks;
      split = 0;
    } else {
      const uint32_t tile = w % tiles_mn;
      split = w / tiles_mn;
      m_blk = tile / p.num_n_blocks;
      n_blk = tile - m_blk * p.num_n_blocks;
    }
  };

  if (warp == 0) {
    // ===================== TMA producer =====================
    if (lane == 0) {
      uint32_t stage = 0, phase = 0, issued = 0, runs = 0, prev_n = 0xffffffffu;
      bool ok = true;
      for (uint32_t w = w_begin; w < w_end && ok; w += w_step) {
        uint32_t m_blk, n_blk, split;
        decode(w, m_blk, n_blk, split);
        const uint32_t kt_begin = split * p.k_tiles_per_split;
        const uint32_t kt_end = min(p.num_k_tiles, kt_begin + p.k_tiles_per_split);
        const uint32_t first_blk128 = n_blk * kBlockN / 128u;
        const uint32_t blks128 = min(static_cast<uint32_t>(C::kSfBlocks), p.sfb_blocks128 - first_blk128);
        if (p.b_resident && n_blk != prev_n) {
          // new column block: wait until the MMAs of the previous run have retired, then load the panel
          if (runs > 0 && !mbar_wait(bar_b_empty, (runs - 1) & 1u, abort_flag, kStatusProducerTimeout, p.wait_timeout_ns)) {
            ok = false;
            break;
          }
          const uint32_t sf_total = p.k_atoms * kSfTileBytes * blks128;
          mbar_expect_tx(bar_b_full, p.num_k_tiles * C::kBStageBytes + sf_total);
          for (uint32_t kt = 0; kt < p.num_k_tiles; ++kt) {
            const uint32_t atoms = min(static_cast<uint32_t>(kKAtomsPerStage), p.k_atoms - kt * kKAtomsPerStage);
            tma_load_2d(smem_b + kt * C::kBStageBytes, &tmap_b, bar_b_full, static_cast<int32_t>(kt * kBlockKBytes),
                        static_cast<int32_t>(n_blk * kBlockN));
            for (uint32_t i = 0; i < blks128; ++i)
              bulk_load(smem_sfb + kt * C::kSfbStageBytes + i * kSfBlockStageBytes,
                        p.sfb + (static_cast<size_t>(first_blk128 + i) * p.k_atoms + kt * kKAtomsPerStage) * kSfTileBytes,
                        atoms * kSfTileBytes, bar_b_full);
          }
          prev_n = n_blk;
          ++runs;
        }
        for (uint32_t kt = kt_begin; kt < kt_end; ++kt) {
          if (!mbar_wait(bar_empty + 8 * stage, phase ^ 1u, abort_flag, kStatusProducerTimeout, p.wait_timeout_ns)) {
            ok = false;
            break;
          }
          GEMM_TRACE(0, 1, true);
          const uint32_t atoms = min(static_cast<uint32_t>(kKAtomsPerStage), p.k_atoms - kt * kKAtomsPerStage);
          const uint32_t sf_bytes = atoms * kSfTileBytes;
          const uint32_t full = bar_full + 8 * stage;
          if ((p.debug_flags & 1u) && blockIdx.x == 0 && issued == 0) {
            // test hook: this stage is never armed nor loaded, so its consumers' waits run out
            ++issued;
            if (++stage == stages) {
              stage = 0;
              phase ^= 1u;
            }
            continue;
          }
          // scale blocks of A inside the matrix (the second row half of a tall tile may lie below it)
          const uint32_t a_blks = min(static_cast<uint32_t>(kMHalves), p.sfa_blocks128 - m_blk * kMHalves);
          if (p.b_resident) {
            mbar_expect_tx(full, kAStageBytes + sf_bytes * a_blks);
          } else {
            mbar_expect_tx(full, kAStageBytes + C::kBStageBytes + sf_bytes * (a_blks + blks128));
            tma_load_2d(smem_b + stage * C::kBStageBytes, &tmap_b, full, static_cast<int32_t>(kt * kBlockKBytes),
                        static_cast<int32_t>(n_blk * kBlockN));
            for (uint32_t i = 0; i < blks128; ++i)
              bulk_load(smem_sfb + stage * C::kSfbStageBytes + i * kSfBlockStageBytes,
                        p.sfb + (static_cast<size_t>(first_blk128 + i) * p.k_atoms + kt * kKAtomsPerStage) * kSfTileBytes,
                        sf_bytes, full);
          }
          tma_load_2d(smem_a + stage * kAStageBytes, &tmap_a, full, static_cast<int32_t>(kt * kBlockKBytes),
                      static_cast<int32_t>(m_blk * kBlockM));
          for (uint32_t h = 0; h < a_blks; ++h)
            bulk_load(smem_sfa + stage * kSfaStageBytes + h * kSfBlockStageBytes,
                      p.sfa + (static_cast<size_t>(m_blk * kMHalves + h) * p.k_atoms + kt * kKAtomsPerStage) * kSfTileBytes,
                      sf_bytes, full);
          GEMM_TRACE(0, 2, true);
          ++issued;
          if (++stage == stages) {
            stage = 0;
            phase ^= 1u;
          }
        }
      }
      if (!ok) {
        // aborting: give copies already in flight a bounded chance to land before the CTA exits
        const uint32_t pending = min(issued, stages);
        for (uint32_t i = 0; i < pending; ++i) {
          const uint32_t s = (stage + stages - 1 - i) % stages;
          const uint32_t ph = (s < stage) ? phase : (phase ^ 1u);
          for (int spin = 0; spin < 4096 && !mbar_try_wait(bar_full + 8 * s, ph); ++spin) {
          }
        }
      }
    }
  } else if (warp == 1) {
    // ===================== MMA issuer =====================
    // The whole warp walks the loops so that tile / stage bookkeeping and the descriptors stay warp
    // uniform (uniform registers); one elected lane issues the tensor-core instructions.  Issuing
    // from inside a single-lane branch instead costs ~140 cycles per tcgen05.mma.
    {
      constexpr uint32_t idesc = make_idesc<kBlockN>();
      uint32_t stage = 0, phase = 0, acc = 0, acc_phase = 0, runs = 0, prev_n = 0xffffffffu, sf_set = 0, sf_phase = 0;
      bool ok = true;
      for (uint32_t w = w_begin; w < w_end && ok; w += w_step) {
        uint32_t m_blk, n_blk, split;
        decode(w, m_blk, n_blk, split);
        const uint32_t kt_begin = split * p.k_tiles_per_split;
        const uint32_t kt_end = min(p.num_k_tiles, kt_begin + p.k_tiles_per_split);
        if (p.b_resident && n_blk != prev_n) {
          if (!__all_sync(0xffffffffu, mbar_wait(bar_b_full, runs & 1u, abort_flag, kStatusMmaTimeout, p.wait_timeout_ns))) {
            ok = false;
            break;
          }
          prev_n = n_blk;
          ++runs;
        }
        GEMM_TRACE(1, 10, lane == 0);
        if (!__all_sync(0xffffffffu, mbar_wait(bar_tmem_empty + 8 * acc, acc_phase ^ 1u, abort_flag, kStatusMmaTimeout, p.wait_timeout_ns))) {
          ok = false;
          break;
        }
        GEMM_TRACE(1, 11, lane == 0);
        tcgen05_fence_after();
        const uint32_t tmem_acc = tmem_base + acc * C::kAccCols;
        for (uint32_t kt = kt_begin; kt < kt_end; ++kt) {
          // The scale-factor warps arrive on `sf_full` only after they have seen the stage's `full` barrier
          // complete (operands and scale tiles share it), so this one wait covers both: operands in
          // shared memory and column set `sf_set` filled.
          const bool ready = mbar_wait(bar_sf_full + 8 * sf_set, sf_phase, abort_flag, kStatusMmaTimeout, p.wait_timeout_ns);
          if (!__all_sync(0xffffffffu, ready)) {
            ok = false;
            break;
          }
          GEMM_TRACE(1, 12, lane == 0);
          tcgen05_fence_after();
          const uint32_t atoms = min(static_cast<uint32_t>(kKAtomsPerStage), p.k_atoms - kt * kKAtomsPerStage);
          const uint32_t b_slot = p.b_resident ? kt : stage;
          const uint32_t tsfa = tmem_base + C::kTmemSfa + sf_set * C::kSfSetCols;
          const uint32_t tsfb = tmem_base + C::kTmemSfb + sf_set * C::kSfSetCols;
          const uint64_t desc_a = make_ab_desc(smem_a + stage * kAStageBytes);
          const uint64_t desc_b = make_ab_desc(smem_b + b_slot * C::kBStageBytes);
          if (elect_one()) {
#pragma unroll
            for (uint32_t kb = 0; kb < kKAtomsPerStage; ++kb) {
              // 64 nibbles = 32 bytes further along the swizzled row: +2 in the 16-byte start field; the
              // second row half of a tall tile sits 16 KB further in the A stage and has its own accumulator
              // and A scale columns
              if (kb < atoms) {
#pragma unroll
                for (uint32_t h = 0; h < static_cast<uint32_t>(kMHalves); ++h)
                  tcgen05_mma_nvf4(tmem_acc + h * kBlockN, desc_a + h * (kAHalfBytes >> 4) + kb * 2, desc_b + kb * 2, idesc,
                                   (kt > kt_begin || kb > 0) ? 1u : 0u, tsfa + h * 4 * kKAtomsPerStage + kb * 4,
                                   tsfb + kb * C::kSfbColsPerAtom);
              }
            }
            tcgen05_commit(bar_empty + 8 * stage);       // frees the smem stage once these MMAs retire
            tcgen05_commit(bar_sf_empty + 8 * sf_set);   // ... and the scale-factor column set
          }
          __syncwarp();
          GEMM_TRACE(1, 13, lane == 0);
          if (++sf_set == C::kSfSets) {
            sf_set = 0;
            sf_phase ^= 1u;
          }
          if (++stage == stages) {
            stage = 0;
            phase ^= 1u;
          }
        }
        if (!ok) break;
        // last tile of this column block (or of this CTA): the resident panel may be replaced once
        // everything issued so far has retired
        bool release_panel = false;
        if (p.b_resident) {
          uint32_t nm, nn = n_blk, ns;
          const bool last = (w + w_step >= w_end);
          if (!last) decode(w + w_step, nm, nn, ns);
          release_panel = last || nn != n_blk;
        }
        if (elect_one()) {
          tcgen05_commit(bar_tmem_full + 8 * acc);  // accumulator complete
          if (release_panel) tcgen05_commit(bar_b_empty);
        }
        __syncwarp();
        GEMM_TRACE(1, 14, lane == 0);
        if (++acc == C::kAccStages) {
          acc = 0;
          acc_phase ^= 1u;
        }
      }
      if (!ok) {
        // aborting: give the MMAs already issued a bounded chance to retire before tensor memory is freed
        if (elect_one()) tcgen05_commit(bar_mma_drain);
        __syncwarp();
        for (int spin = 0; spin < (1 << 16) && !mbar_try_wait(bar_mma_drain, 0); ++spin) {
        }
      }
    }
  } else if (warp >= 8 && warp < 12) {
    // ===================== scale-factor warps =====================
    // Four warps (one per 32-lane quadrant of tensor memory) read the 512-byte scale tiles of each
    // k-tile from shared memory -- lane l takes the 16 bytes of rows l, l+32, l+64, l+96 -- and write
    // them with tcgen05.st into the four columns per k-atom the MMA expects, replicated in every
    // quadrant.  This keeps scale-factor transport off the tensor pipe (tcgen05.cp runs in order
    // with the MMAs and costs about a third of a wide-tile main loop).
    const uint32_t quad = warp & 3u;
    uint32_t stage = 0, phase = 0, sf_set = 0, sf_phase = 0, runs = 0, prev_n = 0xffffffffu;
    bool ok = true;
    for (uint32_t w = w_begin; w < w_end && ok; w += w_step) {
      uint32_t m_blk, n_blk, split;
      decode(w, m_blk, n_blk, split);
      const uint32_t kt_begin = split * p.k_tiles_per_split;
      const uint32_t kt_end = min(p.num_k_tiles, kt_begin + p.k_tiles_per_split);
      if (p.b_resident && n_blk != prev_n) {
        if (!mbar_wait(bar_b_full, runs & 1u, abort_flag, kStatusMmaTimeout, p.wait_timeout_ns)) break;
        prev_n = n_blk;
        ++runs;
      }
      for (uint32_t kt = kt_begin; kt < kt_end; ++kt) {
        if (!mbar_wait(bar_full + 8 * stage, phase, abort_flag, kStatusMmaTimeout, p.wait_timeout_ns) ||
            !mbar_wait(bar_sf_empty + 8 * sf_set, sf_phase ^ 1u, abort_flag, kStatusMmaTimeout, p.wait_timeout_ns)) {
          ok = false;
          break;
        }
        GEMM_TRACE(2, 20, warp == 8 && lane == 0);
        tcgen05_fence_after();
        const uint32_t atoms = min(static_cast<uint32_t>(kKAtomsPerStage), p.k_atoms - kt * kKAtomsPerStage);
        const uint32_t b_slot = p.b_resident ? kt : stage;
        const uint32_t sfa_s = smem_sfa + stage * kSfaStageBytes + lane * 16;
        const uint32_t sfb_s = smem_sfb + b_slot * C::kSfbStageBytes + lane * 16;
        const uint32_t tsfa = tmem_base + C::kTmemSfa + sf_set * C::kSfSetCols + ((quad * 32u) << 16);
        const uint32_t tsfb = tmem_base + C::kTmemSfb + sf_set * C::kSfSetCols + ((quad * 32u) << 16);
        // all shared-memory reads first (independent, pipelined), then the tensor-memory stores
        uint32_t ra[kMHalves][kKAtomsPerStage][4];
        uint32_t rb[kKAtomsPerStage][C::kSfBlocks * 4];
#pragma unroll
        for (uint32_t kb = 0; kb < kKAtomsPerStage; ++kb) {
          if (kb < atoms) {
#pragma unroll
            for (int h = 0; h < kMHalves; ++h)
              asm volatile("ld.shared.v4.b32 {%0, %1, %2, %3}, [%4];"
                           : "=r"(ra[h][kb][0]), "=r"(ra[h][kb][1]), "=r"(ra[h][kb][2]), "=r"(ra[h][kb][3])
                           : "r"(sfa_s + h * kSfBlockStageBytes + kb * kSfTileBytes));
#pragma unroll
            for (int i = 0; i < C::kSfBlocks; ++i)
              asm volatile("ld.shared.v4.b32 {%0, %1, %2, %3}, [%4];"
                           : "=r"(rb[kb][4 * i]), "=r"(rb[kb][4 * i + 1]), "=r"(rb[kb][4 * i + 2]), "=r"(rb[kb][4 * i + 3])
                           : "r"(sfb_s + i * kSfBlockStageBytes + kb * kSfTileBytes));
          }
        }
        if constexpr (kBlockN == 192) {
          // Six scale words (192 rows of B) per k-atom out of the eight loaded: words 0..5 when the tile
          // starts on a 128-row block boundary (even column block), words 2..7 when it starts in the
          // middle of the first block (odd column block).
          const bool odd = (n_blk & 1u) != 0;
          uint32_t sel[kKAtomsPerStage][6];
#pragma unroll
          for (uint32_t kb = 0; kb < kKAtomsPerStage; ++kb)
#pragma unroll
            for (int j = 0; j < 6; ++j) sel[kb][j] = odd ? rb[kb][j + 2] : rb[kb][j];
          if (atoms == kKAtomsPerStage) {
#pragma unroll
            for (int h = 0; h < kMHalves; ++h) tcgen05_st_x16(tsfa + h * 4 * kKAtomsPerStage, &ra[h][0][0]);
            tcgen05_st_x16(tsfb, &sel[0][0]);
            tcgen05_st_x8(tsfb + 16, &sel[0][0] + 16);
          } else {
#pragma unroll
            for (uint32_t kb = 0; kb < kKAtomsPerStage; ++kb) {
              if (kb < atoms) {
#pragma unroll
                for (int h = 0; h < kMHalves; ++h) tcgen05_st_x4(tsfa + h * 4 * kKAtomsPerStage + kb * 4, ra[h][kb]);
                tcgen05_st_x4(tsfb + kb * 6, sel[kb]);
                tcgen05_st_x2(tsfb + kb * 6 + 4, sel[kb] + 4);
              }
            }
          }
        } else if (atoms == kKAtomsPerStage) {
          // one 16-column store for the A scales, one 16- or 32-column store for the B scales
          tcgen05_st_x16(tsfa, &ra[0][0][0]);
          tcgen05_st_x16(tsfb, &rb[0][0]);
          if constexpr (C::kSfBlocks == 2) tcgen05_st_x16(tsfb + 16, &rb[2][0]);
        } else {
#pragma unroll
          for (uint32_t kb = 0; kb < kKAtomsPerStage; ++kb) {
            if (kb < atoms) {
              tcgen05_st_x4(tsfa + kb * 4, ra[0][kb]);
#pragma unroll
              for (int i = 0; i < C::kSfBlocks; ++i) tcgen05_st_x4(tsfb + kb * C::kSfbColsPerAtom + i * 4, &rb[kb][4 * i]);
            }
          }
        }
        asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
        tcgen05_fence_before();
        __syncwarp();
        if (lane == 0) {
          mbar_arrive(bar_sf_full + 8 * sf_set);  // scale factors visible to the MMA issuer
          mbar_arrive(bar_empty + 8 * stage);     // this warp no longer reads the smem stage
        }
        GEMM_TRACE(2, 21, warp == 8 && lane == 0);
        if (++sf_set == C::kSfSets) {
          sf_set = 0;
          sf_phase ^= 1u;
        }
        if (++stage == stages) {
          stage = 0;
          phase ^= 1u;
        }
      }
    }
  } else if (warp >= 4) {
    // ===================== epilogue (two groups of four warps) =====================
    const uint32_t ew = warp & 3u;               // lane quadrant of tensor memory this warp reaches
    const uint32_t eg = warp >= 12 ? 1u : 0u;    // epilogue group
    const uint32_t gtid = ew * 32 + lane;        // thread index inside the group, also the tile row
    const bool elected = gtid == 0;
    constexpr uint32_t kRing = C::kStoreBufs / 2;  // staging buffers per group
    OutT* out = static_cast<OutT*>(p.out);
    OutT* aux = static_cast<OutT*>(p.aux);
    uint32_t acc = 0, acc_phase = 0, store_buf = 0, tile_iter = 0;
    const uint32_t my_bias = smem_bias + eg * kBlockN * 4;
    const float* my_bias_gen = reinterpret_cast<const float*>(smem_gen + (my_bias - smem_base));
    const uint32_t my_store = smem_store + eg * kRing * kStoreStageBytes;
    const float gb = p.mode == NVFP4_GS_NONE ? 1.0f : __ldg(p.b_global);
    const float ga_scalar = p.mode == NVFP4_GS_TENSOR ? __ldg(p.a_global) : 1.0f;
    // the rows' global scales of a tile are fetched one tile ahead: their load latency would
    // otherwise sit between the accumulator becoming ready and the first store
    auto row_scale = [&](uint32_t w, uint32_t h) {
      uint32_t mb, nb, sp;
      decode(w, mb, nb, sp);
      const uint32_t r = mb * kBlockM + h * kRowBlock + gtid;
      return (p.mode == NVFP4_GS_ROWWISE_A && r < p.m) ? __ldg(p.a_global + r) : 0.0f;
    };
    // The bias slice of a tile travels the same way: its values are fetched into registers one tile ahead
    // and reach shared memory only when the column block changes (a banded schedule keeps a CTA on one
    // column block for many tiles).
    float bias_next[C::kBiasSlots];
    uint32_t staged_bias_blk = 0xffffffffu;
    auto fetch_bias = [&](uint32_t w) {
      uint32_t mb, nb, sp;
      decode(w, mb, nb, sp);
#pragma unroll
      for (int j = 0; j < C::kBiasSlots; ++j) {
        const uint32_t in_tile = gtid + 128 * j;
        const uint32_t col = nb * kBlockN + in_tile;
        bias_next[j] = (kTmaStore && p.epilogue != NVFP4_EPI_NONE && in_tile < static_cast<uint32_t>(kBlockN) && col < p.n)
                           ? bias_value(p, col)
                           : 0.0f;
      }
    };
    if (w_begin < w_end) fetch_bias(w_begin);
    float ga_next[kMHalves];
#pragma unroll
    for (int h = 0; h < kMHalves; ++h) ga_next[h] = w_begin < w_end ? row_scale(w_begin, h) : 0.0f;
    for (uint32_t w = w_begin; w < w_end; w += w_step, ++tile_iter) {
      uint32_t m_blk, n_blk, split;
      decode(w, m_blk, n_blk, split);
      float ga_row[kMHalves];
#pragma unroll
      for (int h = 0; h < kMHalves; ++h) {
        ga_row[h] = ga_next[h];
        if (w + w_step < w_end) ga_next[h] = row_scale(w + w_step, h);
      }
      // the tile's bias slice goes through shared memory once (every row then reads it broadcast); it is
      // fetched before the wait for the accumulator so that its latency hides behind the main loop.  The
      // group's last barrier of the previous tile comes after that tile's last read of the slice.
      const bool add_bias = kTmaStore && p.epilogue != NVFP4_EPI_NONE && (p.k_splits == 1 || split == 0);
      if (add_bias && n_blk != staged_bias_blk) {  // uniform across the group
#pragma unroll
        for (int j = 0; j < C::kBiasSlots; ++j)
          if (gtid + 128 * j < static_cast<uint32_t>(kBlockN))
            asm volatile("st.shared.f32 [%0], %1;" ::"r"(my_bias + (gtid + 128 * j) * 4), "f"(bias_next[j]) : "memory");
        epilogue_barrier(eg);
        staged_bias_blk = n_blk;
      }
      if (w + w_step < w_end) fetch_bias(w + w_step);
      // go on only if every thread of the group saw the accumulator arrive (no thread may be left in a
      // later barrier of the group when another one gives up)
      GEMM_TRACE(3 + eg, 30, elected);
      if (!epilogue_all(eg, mbar_wait(bar_tmem_full + 8 * acc, acc_phase, abort_flag, kStatusEpilogueTimeout,
                                      p.wait_timeout_ns)))
        break;
      GEMM_TRACE(3 + eg, 31, elected);
      tcgen05_fence_after();
      // reference order: (weight * a_scale) * b_scale, then acc * scale
      float scale_h[kMHalves];
#pragma unroll
      for (int h = 0; h < kMHalves; ++h)
        scale_h[h] = __fmul_rn(__fmul_rn(p.weight, p.mode == NVFP4_GS_ROWWISE_A ? ga_row[h] : ga_scalar), gb);
      const uint32_t taddr_row = tmem_base + acc * C::kAccCols + ((ew * 32u) << 16);
      // The accumulator buffer goes back to the MMA warp as soon as this warp's last tcgen05.ld of the
      // tile has landed in registers: scaling, staging and the stores of that last sub-tile then run
      // beside the next tile's main loop.
      auto release_accumulator = [&]() {
        tcgen05_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(bar_tmem_empty + 8 * acc);
      };
      if (kTmaStore) {
        // Sub-tiles of 128 rows x 128 bytes go through the group's shared-memory ring and leave
        // with TMA stores (TMA reduce-add for split-K partial sums); rows / columns outside the
        // matrix are clipped by the tensor map.  The items of a tile -- (row half, column sub-tile) --
        // alternate between the two groups; with an odd number of items per tile (192 bf16 columns = 3)
        // the group that takes two alternates from tile to tile, which the double-buffered accumulator
        // evens out.
        constexpr int kSub = SubTile<OutT>::kCols;
        constexpr int kNumSub = kBlockN / kSub;
        constexpr int kItems = kMHalves * kNumSub;
        const int first_item = static_cast<int>((kItems & 1) ? (eg ^ (tile_iter & 1u)) : eg);
        auto item_valid = [&](int item) {  // uniform across the group
          const uint32_t h = static_cast<uint32_t>(item / kNumSub), sub = static_cast<uint32_t>(item % kNumSub);
          return n_blk * kBlockN + sub * kSub < p.n && m_blk * kBlockM + h * kRowBlock < p.m;
        };
        int last_item = -1;
#pragma unroll
        for (int item = first_item; item < kItems; item += 2)
          if (item_valid(item)) last_item = item;
        if (last_item < 0) release_accumulator();  // nothing of this tile is for this group to read
        float row_max = -INFINITY;  // largest value this thread stores for its row in the current row half
        uint32_t max_h = 0;
        auto flush_row_max = [&]() {
          const uint32_t r = m_blk * kBlockM + max_h * kRowBlock + gtid;
          if (p.row_amax && r < p.m && row_max > 0.0f) {
            // max over the row of relu(stored value)^2: rounding to the stored type and relu^2 are both
            // monotonic, so they apply to the maximum instead of to every element; a reduction without a
            // return value, so the thread does not wait for it
            const float stored = sizeof(OutT) == 2 ? __bfloat162float(__float2bfloat16_rn(row_max)) : row_max;
            const uint32_t bits = __float_as_uint(__fmul_rn(stored, stored));
            asm volatile("red.global.max.u32 [%0], %1;" ::"l"(reinterpret_cast<unsigned int*>(p.row_amax) + r), "r"(bits)
                         : "memory");
          }
          row_max = -INFINITY;
        };
#pragma unroll 1
        for (int item = first_item; item < kItems; item += 2) {
          if (!item_valid(item)) continue;
          const uint32_t h = static_cast<uint32_t>(item / kNumSub);
          const int c = (item % kNumSub) * kSub;
          const uint32_t col0 = n_blk * kBlockN + c;
          const uint32_t row0 = m_blk * kBlockM + h * kRowBlock;
          if (h != max_h) {
            flush_row_max();
            max_h = h;
          }
          const float scale = kMHalves == 1 ? scale_h[0] : (h == 0 ? scale_h[0] : scale_h[kMHalves - 1]);
          const uint64_t scale2 = pack_f32x2(scale, scale);
          float v[kSub];
          {
            uint32_t r[kSub / 32][32];
#pragma unroll
            for (int q = 0; q < kSub / 32; ++q) tcgen05_ld_32x32b_x32(taddr_row + h * kBlockN + c + 32 * q, r[q]);
            tcgen05_wait_ld();
            GEMM_TRACE(3 + eg, 32, elected);
            if (item == last_item) release_accumulator();  // the group's last read of this tile
            if (add_bias) {
              // acc * scale + bias in one rounding (the reference rounds the product first; the
              // difference is below the f32 ulp and far inside the GEMM tolerance)
#pragma unroll
              for (int i = 0; i < kSub; i += 4) {
                const float4 b = *reinterpret_cast<const float4*>(my_bias_gen + c + i);
                fma_f32x2(v[i], v[i + 1], r[i / 32][i % 32], r[i / 32][i % 32 + 1], scale2, pack_f32x2(b.x, b.y));
                fma_f32x2(v[i + 2], v[i + 3], r[i / 32][i % 32 + 2], r[i / 32][i % 32 + 3], scale2, pack_f32x2(b.z, b.w));
              }
            } else {
#pragma unroll
              for (int i = 0; i < kSub; i += 2)
                mul_f32x2(v[i], v[i + 1], __uint_as_float(r[i / 32][i % 32]), __uint_as_float(r[i / 32][i % 32 + 1]),
                          scale2);
            }
          }
          if (p.row_amax) {
            // columns past n hold zero-filled operands (acc = 0): only real columns count
            const uint32_t valid = min(static_cast<uint32_t>(kSub), p.n - col0);
            if (valid == static_cast<uint32_t>(kSub)) {
              // four independent chains instead of one of kSub dependent maxima
              float m0 = v[0], m1 = v[1], m2 = v[2], m3 = v[3];
#pragma unroll
              for (int i = 4; i < kSub; i += 4) {
                m0 = fmaxf(m0, v[i]);
                m1 = fmaxf(m1, v[i + 1]);
                m2 = fmaxf(m2, v[i + 2]);
                m3 = fmaxf(m3, v[i + 3]);
              }
              row_max = fmaxf(row_max, fmaxf(fmaxf(m0, m1), fmaxf(m2, m3)));
            } else {
#pragma unroll
              for (int i = 0; i < kSub; ++i)
                if (static_cast<uint32_t>(i) < valid) row_max = fmaxf(row_max, v[i]);
            }
          }
          const int passes = (p.epilogue == NVFP4_EPI_RELU2 && p.aux) ? 2 : 1;
          for (int pass = 0; pass < passes; ++pass) {
            const bool is_pre = passes == 2 && pass == 0;
            if (p.epilogue == NVFP4_EPI_RELU2 && !is_pre) {
#pragma unroll
              for (int i = 0; i < kSub; i += 2) {
                v[i] = fmaxf(v[i], 0.0f);
                v[i + 1] = fmaxf(v[i + 1], 0.0f);
                square_f32x2(v[i], v[i + 1]);
              }
            }
            const uint32_t buf = my_store + store_buf * kStoreStageBytes;
            if (kRing == 1) {
              // single staging buffer: the previous store must have read it before it is rewritten
              if (elected) bulk_wait_group_read<0>();
              epilogue_barrier(eg);
            }
            GEMM_TRACE(3 + eg, 36, elected);
            SubTile<OutT>::stage(buf + gtid * 128, gtid, v);
            fence_proxy_async_smem();
            GEMM_TRACE(3 + eg, 33, elected);
            // deeper rings: the buffer written next was last used kRing - 1 stores ago
            if (kRing > 1 && elected) bulk_wait_group_read<(kRing > 1 ? kRing - 2 : 0)>();
            epilogue_barrier(eg);
            GEMM_TRACE(3 + eg, 34, elected);
            if (elected) {
              const CUtensorMap* map = is_pre ? &tmap_aux : &tmap_out;
              if (p.k_splits > 1)
                tma_reduce_add_2d(map, buf, static_cast<int32_t>(col0), static_cast<int32_t>(row0));
              else
                tma_store_2d(map, buf, static_cast<int32_t>(col0), static_cast<int32_t>(row0));
              bulk_commit_group();
            }
            GEMM_TRACE(3 + eg, 35, elected);
            store_buf = (store_buf + 1) % kRing;
          }
        }
        flush_row_max();
      } else {
#pragma unroll 1
        for (uint32_t h = 0; h < static_cast<uint32_t>(kMHalves); ++h) {
          const uint32_t row = m_blk * kBlockM + h * kRowBlock + gtid;
          const bool row_ok = row < p.m;
          const float scale = kMHalves == 1 ? scale_h[0] : (h == 0 ? scale_h[0] : scale_h[kMHalves - 1]);
#pragma unroll 1
          for (int c = eg * 32; c < kBlockN; c += 64) {
            uint32_t r[32];
            tcgen05_ld_32x32b_x32(taddr_row + h * kBlockN + c, r);
            tcgen05_wait_ld();
            if (h + 1 == static_cast<uint32_t>(kMHalves) && c + 64 >= kBlockN) release_accumulator();
            const uint32_t col0 = n_blk * kBlockN + c;
            if (row_ok && col0 < p.n) {
              const uint32_t valid = min(32u, p.n - col0);
              float v[32];
#pragma unroll
              for (int i = 0; i < 32; ++i) v[i] = __fmul_rn(__uint_as_float(r[i]), scale);
              const size_t off = static_cast<size_t>(row) * p.ldo + col0;
              if (p.k_splits > 1) {
                // split-K partial sums: f32 reduction into a zero-initialised output; bias joins once
#pragma unroll
                for (int i = 0; i < 32; ++i)
                  if (static_cast<uint32_t>(i) < valid) {
                    float t = v[i];
                    if (p.epilogue == NVFP4_EPI_BIAS && split == 0) t = __fadd_rn(t, bias_value(p, col0 + i));
                    atomicAdd(reinterpret_cast<float*>(p.out) + off + i, t);
                  }
              } else {
                if (p.epilogue != NVFP4_EPI_NONE) {
#pragma unroll
                  for (int i = 0; i < 32; ++i)
                    if (static_cast<uint32_t>(i) < valid) v[i] = __fadd_rn(v[i], bias_value(p, col0 + i));
                }
                if (p.epilogue == NVFP4_EPI_RELU2) {
                  if (aux) store_row32<OutT>(aux + off, v, valid, p.vec_store != 0);
#pragma unroll
                  for (int i = 0; i < 32; ++i) {
                    const float t = fmaxf(v[i], 0.0f);
                    v[i] = __fmul_rn(t, t);
                  }
                } else if (p.epilogue == NVFP4_EPI_RESIDUAL) {
#pragma unroll
                  for (int i = 0; i < 32; ++i)
                    if (static_cast<uint32_t>(i) < valid) v[i] = __fmaf_rn(1.0f, v[i], load_out<OutT>(out + off + i));
                }
                store_row32<OutT>(out + off, v, valid, p.vec_store != 0);
              }
            }
          }
        }
      }  // direct-store path
      if (++acc == C::kAccStages) {
        acc = 0;
        acc_phase ^= 1u;
      }
    }
    if (kTmaStore && elected) bulk_wait_group0();  // stores complete before the CTA exits
  }

  // ===================== teardown =====================
  tcgen05_fence_before();
  __syncthreads();
  if (warp == 2) {
    tcgen05_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base),
                 "r"(static_cast<uint32_t>(kTmemCols))
                 : "memory");
  }
}

// ---- host side ------------------------------------------------------------------------------

using EncodeTiledFn = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                   const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                   CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn encode_tiled_fn() {
  static EncodeTiledFn fn = nullptr;
  static std::once_flag once;
  std::call_once(once, [] {
    void* ptr = nullptr;
    cudaDriverEntryPointQueryResult qres;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &qres) == cudaSuccess &&
        qres == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeTiledFn>(ptr);
  });
  return fn;
}

// Tensor maps are pure functions of (address, extents, pitch, box): they say nothing about the bytes in
// memory.  Buffers of a training step never move, so every host thread keeps the maps it has encoded
// (the reference encodes four maps and copies them to the device before every GEMM,
// utils/nvfp4_tma_matmul/launcher.rs:106-166).
struct MapKey {
  uint64_t base;
  uint32_t kind, rows, cols, ld_or_box;
  bool operator==(const MapKey& o) const {
    return base == o.base && kind == o.kind && rows == o.rows && cols == o.cols && ld_or_box == o.ld_or_box;
  }
};
struct MapKeyHash {
  size_t operator()(const MapKey& k) const {
    uint64_t h = k.base * 0x9E3779B97F4A7C15ull;
    h ^= (static_cast<uint64_t>(k.kind) << 56) ^ (static_cast<uint64_t>(k.rows) << 24) ^ k.cols;
    h = (h ^ (h >> 29)) * 0xBF58476D1CE4E5B9ull;
    h ^= k.ld_or_box;
    return static_cast<size_t>(h ^ (h >> 32));
  }
};
struct MapCache {
  std::unordered_map<MapKey, CUtensorMap, MapKeyHash> maps;
  uint64_t hits = 0, misses = 0;
};
MapCache& map_cache() {
  static thread_local MapCache cache;
  return cache;
}
constexpr size_t kMapCacheLimit = 8192;  // entries per host thread; the cache starts over when it is full

// Nibble matrix [rows][k] seen as bytes [rows][k/2]; box = 128 bytes x box_rows, 128-byte swizzle.
int encode_operand_map(CUtensorMap* map, const uint8_t* base, uint32_t rows, uint32_t k, uint32_t box_rows) {
  MapCache& cache = map_cache();
  const MapKey key{reinterpret_cast<uint64_t>(base), 0u, rows, k, box_rows};
  auto it = cache.maps.find(key);
  if (it != cache.maps.end()) {
    ++cache.hits;
    *map = it->second;
    return 0;
  }
  EncodeTiledFn fn = encode_tiled_fn();
  if (!fn) {
    set_last_error("cuTensorMapEncodeTiled is not available from the CUDA driver");
    return static_cast<int>(cudaErrorNotSupported);
  }
  const cuuint64_t dims[2] = {k / 2, rows};
  const cuuint64_t strides[1] = {k / 2};
  const cuuint32_t box[2] = {kBlockKBytes, box_rows};
  const cuuint32_t elem_strides[2] = {1, 1};
  CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<uint8_t*>(base), dims, strides, box, elem_strides,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) {
    set_last_error("cuTensorMapEncodeTiled rejected the operand (base must be 16-byte aligned, k % 32 == 0)");
    return static_cast<int>(cudaErrorInvalidValue);
  }
  ++cache.misses;
  if (cache.maps.size() >= kMapCacheLimit) cache.maps.clear();
  cache.maps.emplace(key, *map);
  return 0;
}

// Output matrix [rows][ld] of f32 / bf16; box = 128 bytes x 128 rows, 128-byte swizzle.
int encode_output_map(CUtensorMap* map, void* base, int dtype, uint32_t rows, uint32_t cols, uint32_t ld) {
  MapCache& cache = map_cache();
  const MapKey key{reinterpret_cast<uint64_t>(base), dtype == NVFP4_DTYPE_F32 ? 1u : 2u, rows, cols, ld};
  auto it = cache.maps.find(key);
  if (it != cache.maps.end()) {
    ++cache.hits;
    *map = it->second;
    return 0;
  }
  EncodeTiledFn fn = encode_tiled_fn();
  if (!fn) return static_cast<int>(cudaErrorNotSupported);
  const size_t esz = dtype == NVFP4_DTYPE_F32 ? 4 : 2;
  const cuuint64_t dims[2] = {cols, rows};
  const cuuint64_t strides[1] = {static_cast<cuuint64_t>(ld) * esz};
  const cuuint32_t box[2] = {static_cast<cuuint32_t>(128 / esz), kRowBlock};
  const cuuint32_t elem_strides[2] = {1, 1};
  CUresult r = fn(map, dtype == NVFP4_DTYPE_F32 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT32 : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2,
                  base, dims, strides, box, elem_strides, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                  CU_TENSOR_MAP_L2_PROMOTION_NONE, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return static_cast<int>(cudaErrorInvalidValue);
  ++cache.misses;
  if (cache.maps.size() >= kMapCacheLimit) cache.maps.clear();
  cache.maps.emplace(key, *map);
  return 0;
}

constexpr int kMaxDevices = 64;

int current_device() {
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) return -1;
  return dev;
}

// SM count of the current device (cached per device ordinal).
int sm_count() {
  static std::atomic<int> counts[kMaxDevices];
  const int dev = current_device();
  if (dev < 0) return 148;
  int c = counts[dev].load(std::memory_order_relaxed);
  if (c == 0) {
    if (cudaDeviceGetAttribute(&c, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || c <= 0) c = 148;
    counts[dev].store(c, std::memory_order_relaxed);
  }
  return c;
}

// Optional event timing of GEMM launches (off by default; a measurement aid for benchmarks).
struct GemmTimingRecord {
  cudaEvent_t start, stop;
  double flops;
};
struct GemmTiming {
  std::mutex mu;
  bool enabled = false;
  std::vector<GemmTimingRecord> pool;  // events created once by timing_begin
  size_t used = 0;
} g_timing;

// Everything the host decides about one launch.
struct GemmPlan {
  uint32_t block_m = 128, block_n = 128, num_n_blocks = 0, k_splits = 1, k_tiles_per_split = 0;
  uint32_t stages = 0, grid = 0, b_resident = 0, resident_cpn = 0, tma_store = 0, vec_store = 0;
  size_t smem_bytes = 0;
};

struct TileBytes {
  int fixed, stream_stage, resident_stage, panel_slot, a_stage;
};
template <int kBlockM, int kBlockN>
constexpr TileBytes tile_bytes_of() {
  using C = Cfg<kBlockM, kBlockN>;
  return {C::kFixedBytes, C::kStreamStageBytes, C::kResidentStageBytes, C::kPanelSlotBytes,
          C::kAStageBytes + C::kSfaStageBytes};
}
TileBytes tile_bytes(uint32_t block_m, uint32_t block_n) {
  if (block_m == 256) return tile_bytes_of<256, 192>();
  return block_n == 256 ? tile_bytes_of<128, 256>() : block_n == 192 ? tile_bytes_of<128, 192>() : tile_bytes_of<128, 128>();
}

template <int kBlockM, int kBlockN, typename OutT, bool kTmaStore>
int launch_store_variant(cudaStream_t s, const CUtensorMap& ma, const CUtensorMap& mb, const CUtensorMap& mo,
                         const CUtensorMap& mx, const GemmParams& p, const GemmPlan& pl) {
  // the opt-in to more than 48 KB of dynamic shared memory is a per-device attribute of the kernel
  static std::atomic<int> attr_state[kMaxDevices];  // 0 = not set, 1 = set, -(error) = failed
  const int dev = current_device();
  if (dev < 0) return static_cast<int>(cudaErrorInvalidDevice);
  int st = attr_state[dev].load(std::memory_order_acquire);
  if (st == 0) {
    const cudaError_t e = cudaFuncSetAttribute(nvfp4_gemm_tcgen05_kernel<kBlockM, kBlockN, OutT, kTmaStore>,
                                               cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemBudget);
    st = e == cudaSuccess ? 1 : -static_cast<int>(e);
    attr_state[dev].store(st, std::memory_order_release);
  }
  if (st < 0) return -st;
  GemmTimingRecord* rec = nullptr;
  if (g_timing.enabled) {
    std::lock_guard<std::mutex> lock(g_timing.mu);
    if (g_timing.enabled && g_timing.used < g_timing.pool.size()) rec = &g_timing.pool[g_timing.used++];
  }
  if (rec) {
    rec->flops = 2.0 * p.m * p.n * p.k;
    cudaEventRecord(rec->start, s);
  }
  nvfp4_gemm_tcgen05_kernel<kBlockM, kBlockN, OutT, kTmaStore><<<pl.grid, kThreads, pl.smem_bytes, s>>>(ma, mb, mo, mx, p);
  count_launch();
  const int rc = static_cast<int>(cudaGetLastError());
  if (rec) cudaEventRecord(rec->stop, s);
  return rc;
}

// The store path is a compile-time property of the kernel (TMA stores through the staging ring, or direct
// stores for outputs a tensor map cannot describe and for the in-place residual epilogue): each variant
// carries only its own epilogue code.
template <int kBlockM, int kBlockN, typename OutT>
int launch_variant(cudaStream_t s, const CUtensorMap& ma, const CUtensorMap& mb, const CUtensorMap& mo,
                   const CUtensorMap& mx, const GemmParams& p, const GemmPlan& pl) {
  return p.tma_store ? launch_store_variant<kBlockM, kBlockN, OutT, true>(s, ma, mb, mo, mx, p, pl)
                     : launch_store_variant<kBlockM, kBlockN, OutT, false>(s, ma, mb, mo, mx, p, pl);
}

std::atomic<int> g_tile_override{-1};  // -1 = read NVFP4_GEMM_TILE once, 0 = automatic, else (block_m << 16) | block_n
std::atomic<bool> g_allow_tall{true};  // the automatic choice may take the 256 x 192 tile
std::atomic<uint64_t> g_wait_timeout_ns{kDefaultWaitTimeoutNs};
std::atomic<uint32_t> g_debug_flags{0};
#ifdef NVFP4_GEMM_TRACE
std::atomic<unsigned long long*> g_trace_buffer{nullptr};
#endif
bool tile_shape_ok(int bm, int bn) {
  return (bm == 128 && (bn == 128 || bn == 192 || bn == 256)) || (bm == 256 && bn == 192);
}

int tile_override() {
  int v = g_tile_override.load(std::memory_order_relaxed);
  if (v < 0) {
    // NVFP4_GEMM_TILE = "<width>" (128-row tile) or "<height>x<width>"
    const char* env = std::getenv("NVFP4_GEMM_TILE");
    int bm = 128, bn = 0;
    if (env) {
      const char* x = std::strchr(env, 'x');
      if (x) {
        bm = std::atoi(env);
        bn = std::atoi(x + 1);
      } else {
        bn = std::atoi(env);
      }
    }
    v = tile_shape_ok(bm, bn) ? ((bm << 16) | bn) : 0;
    g_tile_override.store(v, std::memory_order_relaxed);
  }
  return v;
}

int validate_gemm(const nvfp4_gemm_args& a) {
  if (a.k == 0 || a.k % 64 != 0 || a.ldo < a.n) {
    set_last_error("nvfp4_gemm: k must be a non-zero multiple of 64 and ldo >= n");
    return static_cast<int>(cudaErrorInvalidValue);
  }
  if ((reinterpret_cast<uintptr_t>(a.a_bytes) | reinterpret_cast<uintptr_t>(a.b_bytes) |
       reinterpret_cast<uintptr_t>(a.a_scales) | reinterpret_cast<uintptr_t>(a.b_scales)) & 15u) {
    set_last_error("nvfp4_gemm: operand and scale pointers must be 16-byte aligned");
    return static_cast<int>(cudaErrorInvalidValue);
  }
  const bool has_bias = a.bias || (a.bias_nvfp4_bytes && a.bias_nvfp4_scales && a.bias_nvfp4_global);
  if (a.epilogue < NVFP4_EPI_NONE || a.epilogue > NVFP4_EPI_RESIDUAL || (a.epilogue != NVFP4_EPI_NONE && !has_bias) ||
      a.global_scale_mode < NVFP4_GS_NONE || a.global_scale_mode > NVFP4_GS_ROWWISE_A ||
      (a.global_scale_mode != NVFP4_GS_NONE && (!a.a_global || !a.b_global)) ||
      (a.out_dtype != NVFP4_DTYPE_F32 && a.out_dtype != NVFP4_DTYPE_BF16) || !a.out) {
    set_last_error("nvfp4_gemm: inconsistent epilogue / scale mode / dtype arguments");
    return static_cast<int>(cudaErrorInvalidValue);
  }
  return 0;
}

// Tile width, split-K count, shared-memory plan and grid of one GEMM on `sms` SMs.
void plan_gemm(const nvfp4_gemm_args& a, int sms, GemmPlan& pl) {
  const uint32_t k_atoms = a.k / 64;
  const uint32_t num_k_tiles = (k_atoms + kKAtomsPerStage - 1) / kKAtomsPerStage;
  const uint32_t m_blocks128 = (a.m + kRowBlock - 1) / kRowBlock;
  const uint32_t usms = static_cast<uint32_t>(sms);
  // Tile shape.  A block-scaled FP4 tcgen05.mma occupies the tensor pipe for about as long at N = 128 as
  // at N = 256 (the 128-column form is bound by shared-memory operand reads), so wide tiles do more work
  // per instruction and are preferred whenever the shape can still fill the SMs:
  //  * long K: enough wide tiles, or (f32 output, linear epilogue) enough tiles x K splits;
  //  * short K with many row blocks: wide tile with its whole B panel resident in shared memory.
  // 128 x 192 keeps a double-buffered accumulator (the drain of one tile hides behind the next main loop);
  // 128 x 256 has one buffer; the tall 256 x 192 tile moves the fewest operand bytes per flop and is for
  // streamed long-K GEMMs; 128 x 128 remains for everything else.
  const bool can_split = a.out_dtype == NVFP4_DTYPE_F32 &&
                         (a.epilogue == NVFP4_EPI_NONE || a.epilogue == NVFP4_EPI_BIAS) && num_k_tiles >= 16;
  // Work items, waves and an estimated duration (SM cycles) of a candidate shape.  The constants are fits to
  // B200 measurements of the training step's shapes: a streamed k-tile costs what its operand bytes take
  // through the SM's L2 port (about 47 bytes per cycle: 128 x 128 700, 128 x 192 980, 128 x 256 1150,
  // 256 x 192 1360 cycles), a tile adds the part of its epilogue that the next main loop does not hide (one
  // accumulator buffer: all of the drain).
  struct Candidate {
    uint32_t splits;
    uint64_t cost;
  };
  auto tiles_of = [&](uint32_t bm, uint32_t bn) { return ((a.m + bm - 1) / bm) * ((a.n + bn - 1) / bn); };
  auto evaluate = [&](uint32_t bm, uint32_t bn) {
    const uint32_t tiles = tiles_of(bm, bn);
    const uint64_t ck = bm == 256 ? 1360 : bn == 256 ? 1150 : bn == 192 ? 980 : 700;
    const uint64_t ce = bm == 256 ? 5000 : bn == 256 ? 3500 : bn == 192 ? 2000 : 1500;
    Candidate best{1, ~0ull};
    uint32_t max_splits = 1;
    if (can_split && tiles < 2 * usms) {
      max_splits = num_k_tiles / 8;
      if (max_splits > 32) max_splits = 32;
      if (max_splits > 2 && gemm_get_deterministic()) max_splits = 2;
      if (max_splits < 1) max_splits = 1;
    }
    for (uint32_t sp = 1; sp <= max_splits; ++sp) {
      const uint32_t per = (num_k_tiles + sp - 1) / sp;
      const uint32_t real = (num_k_tiles + per - 1) / per;
      const uint64_t waves = (static_cast<uint64_t>(tiles) * real + usms - 1) / usms;
      const uint64_t cost = waves * (per * ck + ce);
      if (cost < best.cost) best = Candidate{real, cost};  // ties go to fewer splits
    }
    return best;
  };
  uint32_t block_m = 128, block_n = 128;
  const int forced = tile_override();
  if (forced) {
    block_m = static_cast<uint32_t>(forced) >> 16;
    block_n = static_cast<uint32_t>(forced) & 0xffffu;
  } else {
    const uint32_t tiles192 = tiles_of(128, 192), tiles256 = tiles_of(128, 256);
    // columns of the last 192-wide block that lie outside the matrix, as a share of all columns computed
    const uint32_t cols192 = (a.n + 191) / 192 * 192;
    const bool fits192 = (cols192 - a.n) * 16u <= cols192 && a.n >= 192;  // at most 1/16 wasted
    const bool ok192 = fits192 && (tiles192 >= usms || can_split);
    const bool wide_shape = a.n % 256 == 0 || a.n > 1024;
    const bool ok256 = wide_shape && ((num_k_tiles >= 4 && (tiles256 >= usms || can_split)) ||
                                      (a.n % 256 == 0 && num_k_tiles <= 3 && tiles256 >= 4u * usms));
    // the tall tile: streamed long-K GEMMs only (its A stages leave no room for a resident panel, and short-K
    // GEMMs are bound by writing their output); the wave count in the estimate decides against it when its
    // tiles are too few
    const bool ok_tall = fits192 && num_k_tiles >= 6;
    if (ok192 && ok256) {
      // short K (resident B panel, bound by writing the output): the wider tile; otherwise the cheaper estimate
      if (num_k_tiles <= 3)
        block_n = a.n % 256 == 0 ? 256 : 192;
      else
        block_n = evaluate(128, 192).cost < evaluate(128, 256).cost ? 192 : 256;
    } else if (ok256) {
      block_n = 256;
    } else if (ok192) {
      block_n = 192;
    }
    if (ok_tall && g_allow_tall.load(std::memory_order_relaxed) && evaluate(256, 192).cost < evaluate(128, block_n).cost) {
      block_m = 256;
      block_n = 192;
    }
  }
  pl.block_m = block_m;
  pl.block_n = block_n;
  pl.num_n_blocks = (a.n + block_n - 1) / block_n;
  const uint32_t num_m_blocks = (a.m + block_m - 1) / block_m;
  (void)m_blocks128;
  const uint32_t tiles = num_m_blocks * pl.num_n_blocks;

  // split-K for long GEMMs with few tiles (dW = dY^T.X): f32 output, linear epilogue only; the split count is
  // the one that minimises waves x (main loop + exposed epilogue) of one work item
  pl.k_splits = evaluate(block_m, block_n).splits;
  pl.k_tiles_per_split = (num_k_tiles + pl.k_splits - 1) / pl.k_splits;
  pl.k_splits = (num_k_tiles + pl.k_tiles_per_split - 1) / pl.k_tiles_per_split;

  const size_t esz = a.out_dtype == NVFP4_DTYPE_F32 ? 4 : 2;
  const uint32_t vec_elems = 16 / static_cast<uint32_t>(esz);
  pl.vec_store = ((reinterpret_cast<uintptr_t>(a.out) & 15u) == 0 && a.ldo % vec_elems == 0 &&
                  (!a.aux || (reinterpret_cast<uintptr_t>(a.aux) & 15u) == 0))
                     ? 1
                     : 0;
  // TMA-store epilogue whenever the output satisfies the tensor-map rules (16-byte aligned base
  // and row pitch); the in-place residual epilogue and odd layouts use direct stores.
  pl.tma_store = (pl.vec_store && a.epilogue != NVFP4_EPI_RESIDUAL) ? 1 : 0;

  const uint32_t work = tiles * pl.k_splits;
  pl.grid = work < usms ? work : usms;
  // Short K and many row blocks: keep the B panel resident and stream only A (halves the
  // operand traffic per tile; these shapes are otherwise bound by L2 -> SM bandwidth).
  const bool want_resident =
      block_m == 128 && pl.k_splits == 1 && num_k_tiles <= (block_n == 256 ? 3u : 4u) && tiles >= 4 * pl.grid;
  const TileBytes tb = tile_bytes(block_m, block_n);
  const int budget = kSmemBudget - tb.fixed;
  pl.b_resident = 0;
  pl.resident_cpn = 0;
  if (want_resident) {
    const int left = budget - static_cast<int>(num_k_tiles) * tb.panel_slot;
    const int st = left / tb.resident_stage;
    if (st >= 4) {
      pl.b_resident = 1;
      pl.stages = static_cast<uint32_t>(st > kMaxStages ? kMaxStages : st);
      // banded schedule when the column blocks divide the grid almost evenly
      const uint32_t cpn = pl.grid / pl.num_n_blocks;
      if (cpn >= 1 && cpn * pl.num_n_blocks * 20 >= pl.grid * 19 && num_m_blocks >= 4 * cpn) pl.resident_cpn = cpn;
    }
  }
  if (!pl.b_resident) {
    const int st = budget / tb.stream_stage;
    pl.stages = static_cast<uint32_t>(st > kMaxStages ? kMaxStages : st);
  }
  const uint32_t b_slots = pl.b_resident ? num_k_tiles : pl.stages;
  pl.smem_bytes = tb.fixed + static_cast<size_t>(pl.stages) * tb.a_stage + static_cast<size_t>(b_slots) * tb.panel_slot;
}

}  // namespace

// Split-K sums its partial tiles with TMA reduce-add in arrival order: with two splits the sum is
// order-free (0 + a + b), with more it can differ in the last bits from run to run.  The switch below
// caps the split count at two for callers that need run-to-run identical dW.
static std::atomic<int> g_deterministic_splits{0};
void gemm_set_deterministic(int on) { g_deterministic_splits.store(on ? 1 : 0, std::memory_order_relaxed); }
int gemm_get_deterministic() { return g_deterministic_splits.load(std::memory_order_relaxed); }

#ifdef NVFP4_GEMM_TRACE
extern "C" void nvfp4_gemm_set_trace_buffer(unsigned long long* device_words) {
  g_trace_buffer.store(device_words, std::memory_order_relaxed);
}
#endif

int gemm_timing_begin(uint32_t max_records) {
  std::lock_guard<std::mutex> lock(g_timing.mu);
  while (g_timing.pool.size() < max_records) {
    GemmTimingRecord r;
    r.flops = 0;
    cudaError_t e = cudaEventCreate(&r.start);
    if (e == cudaSuccess) e = cudaEventCreate(&r.stop);
    if (e != cudaSuccess) return static_cast<int>(e);
    g_timing.pool.push_back(r);
  }
  g_timing.used = 0;
  g_timing.enabled = true;
  return 0;
}

int gemm_timing_end(uint32_t* count, double* total_ms, double* total_flops, float* per_launch_ms,
                    double* per_launch_flops, uint32_t capacity) {
  std::lock_guard<std::mutex> lock(g_timing.mu);
  g_timing.enabled = false;
  double ms_sum = 0, fl_sum = 0;
  for (size_t i = 0; i < g_timing.used; ++i) {
    float ms = 0;
    cudaError_t e = cudaEventSynchronize(g_timing.pool[i].stop);
    if (e == cudaSuccess) e = cudaEventElapsedTime(&ms, g_timing.pool[i].start, g_timing.pool[i].stop);
    if (e != cudaSuccess) return static_cast<int>(e);
    ms_sum += ms;
    fl_sum += g_timing.pool[i].flops;
    if (per_launch_ms && i < capacity) per_launch_ms[i] = ms;
    if (per_launch_flops && i < capacity) per_launch_flops[i] = g_timing.pool[i].flops;
  }
  if (count) *count = static_cast<uint32_t>(g_timing.used);
  if (total_ms) *total_ms = ms_sum;
  if (total_flops) *total_flops = fl_sum;
  g_timing.used = 0;
  return 0;
}

uint32_t* device_status_word() {
  uint32_t* ptr = nullptr;
  if (cudaGetSymbolAddress(reinterpret_cast<void**>(&ptr), g_device_status) != cudaSuccess) return nullptr;
  return ptr;
}

int gemm_plan_query(const nvfp4_gemm_args& a, nvfp4_gemm_plan* out) {
  if (!out) return static_cast<int>(cudaErrorInvalidValue);
  std::memset(out, 0, sizeof(*out));
  if (a.m == 0 || a.n == 0) return 0;
  const int rc = validate_gemm(a);
  if (rc) return rc;
  GemmPlan pl;
  plan_gemm(a, sm_count(), pl);
  // the kernel falls back to direct stores when the output map cannot be encoded; that cannot happen for
  // outputs that pass the alignment test above, so the plan reports the test's verdict
  out->block_m = pl.block_m;
  out->block_n = pl.block_n;
  out->acc_stages = (pl.block_n == 256 || pl.block_m == 256) ? 1 : 2;
  out->k_splits = pl.k_splits;
  out->b_resident = pl.b_resident;
  out->resident_cpn = pl.resident_cpn;
  out->stages = pl.stages;
  out->grid = pl.grid;
  out->tma_store = pl.tma_store;
  out->smem_bytes = static_cast<uint32_t>(pl.smem_bytes);
  return 0;
}

void gemm_set_tile_override(int block_m, int block_n) {
  g_tile_override.store(tile_shape_ok(block_m, block_n) ? ((block_m << 16) | block_n) : 0, std::memory_order_relaxed);
}
void gemm_set_wait_timeout_ns(uint64_t ns) { g_wait_timeout_ns.store(ns ? ns : kDefaultWaitTimeoutNs, std::memory_order_relaxed); }
void gemm_set_debug_flags(uint32_t flags) { g_debug_flags.store(flags, std::memory_order_relaxed); }
void gemm_map_cache_stats(uint64_t* hits, uint64_t* misses) {
  if (hits) *hits = map_cache().hits;
  if (misses) *misses = map_cache().misses;
}

int gemm_prepare_operand_maps(const uint8_t* a_bytes, const uint8_t* b_bytes, uint32_t m, uint32_t k, uint32_t n) {
  if (k == 0 || k % 64 != 0) {
    set_last_error("prepare_tma: input_dim must be a non-zero multiple of 64");
    return static_cast<int>(cudaErrorInvalidValue);
  }
  CUtensorMap tmp;
  // operands are read with boxes as tall as the tile the launch will choose: encode every candidate
  int rc = 0;
  for (uint32_t box : {128u, 256u})
    if (!rc) rc = encode_operand_map(&tmp, a_bytes, m, k, box);
  for (uint32_t box : {128u, 192u, 256u})
    if (!rc) rc = encode_operand_map(&tmp, b_bytes, n, k, box);
  return rc;
}

int launch_gemm(cudaStream_t s, const nvfp4_gemm_args& a) {
  if (a.m == 0 || a.n == 0) return 0;
  int rc = validate_gemm(a);
  if (rc) return rc;
  GemmPlan pl;
  plan_gemm(a, sm_count(), pl);
  if (a.relu2_row_amax && !pl.tma_store) {
    set_last_error("nvfp4_gemm: relu2_row_amax needs a 16-byte aligned output and row pitch and no residual epilogue");
    return static_cast<int>(cudaErrorInvalidValue);
  }

  GemmParams p;
  p.sfa = a.a_scales;
  p.sfb = a.b_scales;
  p.a_global = a.a_global;
  p.b_global = a.b_global;
  p.bias = a.bias;
  p.bias_bytes = a.bias_nvfp4_bytes;
  p.bias_scales = a.bias_nvfp4_scales;
  p.bias_global = a.bias_nvfp4_global;
  p.row_amax = a.relu2_row_amax;
  p.out = a.out;
  p.aux = a.aux;
  p.m = a.m;
  p.n = a.n;
  p.k = a.k;
  p.ldo = a.ldo;
  p.mode = a.global_scale_mode;
  p.epilogue = a.epilogue;
  p.weight = a.weight_global_scale;
  p.k_atoms = a.k / 64;
  p.num_k_tiles = (p.k_atoms + kKAtomsPerStage - 1) / kKAtomsPerStage;
  p.num_m_blocks = (a.m + pl.block_m - 1) / pl.block_m;
  p.num_n_blocks = pl.num_n_blocks;
  p.sfa_blocks128 = (a.m + 127) / 128;
  p.sfb_blocks128 = (a.n + 127) / 128;
  p.k_splits = pl.k_splits;
  p.k_tiles_per_split = pl.k_tiles_per_split;
  p.stages = pl.stages;
  p.b_resident = static_cast<int>(pl.b_resident);
  p.resident_cpn = pl.resident_cpn;
  p.vec_store = static_cast<int>(pl.vec_store);
  p.tma_store = static_cast<int>(pl.tma_store);
  p.wait_timeout_ns = g_wait_timeout_ns.load(std::memory_order_relaxed);
  p.debug_flags = g_debug_flags.load(std::memory_order_relaxed);
#ifdef NVFP4_GEMM_TRACE
  p.trace = g_trace_buffer.load(std::memory_order_relaxed);
#endif

  CUtensorMap ma, mb, mo, mx;
  rc = encode_operand_map(&ma, a.a_bytes, a.m, a.k, pl.block_m);
  if (rc) return rc;
  rc = encode_operand_map(&mb, a.b_bytes, a.n, a.k, pl.block_n);
  if (rc) return rc;
  mo = ma;
  mx = ma;
  if (p.tma_store) {
    if (encode_output_map(&mo, a.out, a.out_dtype, a.m, a.n, a.ldo) != 0) p.tma_store = 0;
    if (p.tma_store && a.aux && encode_output_map(&mx, a.aux, a.out_dtype, a.m, a.n, a.ldo) != 0) p.tma_store = 0;
    if (!p.tma_store && a.relu2_row_amax) {
      set_last_error("nvfp4_gemm: relu2_row_amax needs an output the TMA store path accepts");
      return static_cast<int>(cudaErrorInvalidValue);
    }
  }

  const size_t esz = a.out_dtype == NVFP4_DTYPE_F32 ? 4 : 2;
  if (p.k_splits > 1) {
    cudaError_t e = cudaMemset2DAsync(a.out, static_cast<size_t>(a.ldo) * esz, 0, static_cast<size_t>(a.n) * esz, a.m, s);
    if (e != cudaSuccess) return static_cast<int>(e);
  }
  if (a.relu2_row_amax) {
    cudaError_t e = cudaMemsetAsync(a.relu2_row_amax, 0, static_cast<size_t>(a.m) * sizeof(float), s);
    if (e != cudaSuccess) return static_cast<int>(e);
  }

  const bool f32 = a.out_dtype == NVFP4_DTYPE_F32;
  if (pl.block_m == 256)
    return f32 ? launch_variant<256, 192, float>(s, ma, mb, mo, mx, p, pl)
               : launch_variant<256, 192, __nv_bfloat16>(s, ma, mb, mo, mx, p, pl);
  switch (pl.block_n) {
    case 256:
      return f32 ? launch_variant<128, 256, float>(s, ma, mb, mo, mx, p, pl)
                 : launch_variant<128, 256, __nv_bfloat16>(s, ma, mb, mo, mx, p, pl);
    case 192:
      return f32 ? launch_variant<128, 192, float>(s, ma, mb, mo, mx, p, pl)
                 : launch_variant<128, 192, __nv_bfloat16>(s, ma, mb, mo, mx, p, pl);
    default:
      return f32 ? launch_variant<128, 128, float>(s, ma, mb, mo, mx, p, pl)
                 : launch_variant<128, 128, __nv_bfloat16>(s, ma, mb, mo, mx, p, pl);
  }
}

}  // namespace nvfp4
