/*
 * nvfp4_b200.h -- C ABI of the B200 (sm_100a) NVFP4 projection path.
 *
 * Drop-in boundary for the quantization and projection entry points of the
 * reference's `crates/cuda-kernels` (a Rust crate whose host methods launch
 * device kernels).  Each function below replaces one reference host method; the
 * comment in front of it gives that method's file:line (paths relative to
 * crates/cuda-kernels/src/).  A Rust `extern "C"` block binding these symbols
 * reproduces the reference's module structs one to one.
 *
 * Conventions (same as the reference):
 *   - every pointer is a DEVICE pointer owned by the caller unless stated otherwise;
 *     the library allocates nothing per call and keeps no per-call state;
 *   - every call is asynchronous on `stream` (a cudaStream_t / CUstream) and is
 *     ordered only by that stream; no call synchronises;
 *   - the return value is 0 on success or a CUDA error number (1 =
 *     cudaErrorInvalidValue for shape / alignment violations); nothing aborts;
 *   - an NVFP4 tensor is the triple (bytes u8[rows*cols/2], scales u8[rows*cols/16],
 *     global scale f32[1] or f32[rows]); element i is in byte i/2, even index = low
 *     nibble; value = e2m1 * e4m3(scales[i/16]) * global_scale.
 *
 * Scale-factor layouts:
 *   NVFP4_SCALES_LOGICAL  row-major bytes [rows][cols/16]  (the reference's tensor format)
 *   NVFP4_SCALES_PACKED   512-byte tiles [row_block128][k_atom64], byte
 *                         (r%32)*16 + (r/32%4)*4 + g%4 inside a tile, rows padded to 128 with
 *                         0x38 by whoever fills the buffer -- the order tcgen05.cp consumes
 *                         and byte-identical to the reference's packed plane
 *                         (utils/nvfp4_tma_matmul/cute.rs:448-467).
 */
#ifndef NVFP4_B200_H_
#define NVFP4_B200_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define NVFP4_DTYPE_F32 0
#define NVFP4_DTYPE_BF16 1

#define NVFP4_SCALES_LOGICAL 0
#define NVFP4_SCALES_PACKED 1

/* GEMM global-scale modes (utils/nvfp4_tma_matmul/kernels.rs:310-351). */
#define NVFP4_GS_NONE 0        /* out = acc * weight                                   */
#define NVFP4_GS_TENSOR 1      /* out = acc * weight * a_global[0] * b_global[0]       */
#define NVFP4_GS_ROWWISE_A 2   /* out = acc * weight * a_global[row] * b_global[0]     */

/* GEMM epilogues (gpt/projection_postop.rs:97-162). */
#define NVFP4_EPI_NONE 0       /* out = raw                                            */
#define NVFP4_EPI_BIAS 1       /* out = raw + bias[col]                                */
#define NVFP4_EPI_RELU2 2      /* pre = raw + bias; out = max(pre,0)^2; pre stored if `aux` != NULL */
#define NVFP4_EPI_RESIDUAL 3   /* out = fma(1, raw + bias, out)   (in-place residual add, f32 only)  */

/* MS-EDEN source kinds. */
#define NVFP4_SRC_F32_ROWS 0            /* x[rows][src_row_len], zero padded to dst_row_len    */
#define NVFP4_SRC_F32_TRANSPOSED 1      /* x[source_rows][source_cols], output row = source col */
#define NVFP4_SRC_NVFP4_TRANSPOSED 2    /* NVFP4 tensor-scale source, transposed               */
#define NVFP4_SRC_ROWWISE_NVFP4_TRANSPOSED 3 /* NVFP4 rowwise-scale source, transposed          */

/* Library / device ------------------------------------------------------------------------ */

/* Version of this ABI (bumped on incompatible change).  2: nvfp4_linear_backward_args gained
 * x_decoded_amax, nvfp4_quantize_four_six_rowwise_fused gained out_decoded_amax. */
int nvfp4_abi_version(void);
/* Number of kernels this library has launched in this process (host-side tally). */
uint64_t nvfp4_launch_count(void);
/* Text for the last error recorded on the calling thread (host pointer, never NULL). */
const char* nvfp4_last_error(void);
/* Reads and clears the device-side status word written by kernels whose bounded waits gave
 * up (0 = no kernel ever timed out on this device).  Synchronises `stream`.               */
int nvfp4_read_device_status(void* stream, uint32_t* status_out /* host */);

/* Sizes ----------------------------------------------------------------------------------- */

/* utils/nvfp4_tc_matmul/args.rs:37-39 -- K padded to a multiple of 64. */
uint32_t nvfp4_padded_k(uint32_t k);
/* utils/nvfp4_tma_matmul/scale_layout.rs:26-28 -- rows padded to a multiple of 128. */
uint32_t nvfp4_scale_padded_mn_extent(uint32_t mn_extent);
/* utils/nvfp4_tma_matmul/scale_layout.rs:109-112 -- bytes of a packed scale plane
 * (mn_extent is padded to 128 internally). */
size_t nvfp4_scale_packed_len(uint32_t mn_extent, uint32_t k_dim);
/* utils/nvfp4/quant/mod.rs:36-39 -- number of 1024-value chunks of a tensor amax. */
uint32_t nvfp4_tensor_amax_chunks(uint32_t element_count);

/* amax ------------------------------------------------------------------------------------ */

/* utils/nvfp4/quant/amax.rs:8-17  Nvfp4QuantModule::row_amax_f32 */
int nvfp4_row_amax_f32(void* stream, const float* x, float* out, uint32_t row_count, uint32_t row_len);
/* bf16-input variant of the above (no reference counterpart: the reference is f32-only). */
int nvfp4_row_amax_bf16(void* stream, const void* x, float* out, uint32_t row_count, uint32_t row_len);
/* utils/nvfp4/quant/amax.rs:19-23  Nvfp4QuantModule::tensor_amax_f32
 * chunk_amax[ceil(n/1024)] and out[1] are both written. */
int nvfp4_tensor_amax_f32(void* stream, const float* x, float* chunk_amax, float* out, uint32_t element_count);
int nvfp4_tensor_amax_bf16(void* stream, const void* x, float* chunk_amax, float* out, uint32_t element_count);
/* No counterpart in the reference.  Same out[0] as nvfp4_tensor_amax_f32, for callers that cannot
 * supply the chunk_amax scratch because they cannot allocate at the point of the call (device
 * handed to an arena sized earlier, a loop where an allocation would synchronise the device, a
 * full GPU).  Allocates nothing: the per-chunk scratch is a fixed 256 KiB array inside the
 * library, one per device.  Limits: element_count <= 67108864 (2^26), larger returns 1 with a
 * message; calls that overlap in time on one device race on the array (order them on a stream);
 * the first call on a device does one-time set-up (address look-up), so make it during
 * initialisation and before any stream capture. */
int nvfp4_tensor_amax_f32_static_scratch(void* stream, const float* x, float* out, uint64_t element_count);
/* utils/nvfp4/quant/amax.rs:25-39  Nvfp4QuantModule::tensor_amax_from_chunks_f32 */
int nvfp4_tensor_amax_from_chunks_f32(void* stream, const float* chunk_amax, float* out, uint32_t chunk_count);

/* four-six quantizer (round-to-nearest-even nibbles, error-minimising 4/6 block scale) ---- */

/* utils/nvfp4/quant/four_six.rs:12-23  Nvfp4QuantModule::fp32_to_nvfp4_four_six
 * One tensor scale from amax[0]; flat tensor of group_count*16 values; logical scales. */
int nvfp4_fp32_to_nvfp4_four_six(void* stream, const float* x, const float* amax, uint8_t* out_fp4,
                                 uint8_t* out_scales, float* out_global_scale, uint32_t group_count);
/* utils/nvfp4/quant/four_six.rs:25-58  Nvfp4QuantModule::fp32_to_nvfp4_four_six_rowwise
 * One scale per row from amax[row]; out_global_scale[row]. */
int nvfp4_fp32_to_nvfp4_four_six_rowwise(void* stream, const float* x, const float* amax, uint8_t* out_fp4,
                                         uint8_t* out_scales, float* out_global_scale, uint32_t group_count,
                                         uint32_t row_len);
/* utils/nvfp4/quant/four_six.rs:60-82  Nvfp4QuantModule::fp32_to_nvfp4_four_six_padded
 * Output is [padded_rows][padded_cols], zero outside [rows][cols]; tensor scale. */
int nvfp4_fp32_to_nvfp4_four_six_padded(void* stream, const float* x, const float* amax, uint8_t* out_fp4,
                                        uint8_t* out_scales, float* out_global_scale, uint32_t rows,
                                        uint32_t cols, uint32_t padded_rows, uint32_t padded_cols);
/* utils/nvfp4/quant/four_six.rs:84-123  Nvfp4QuantModule::fp32_transpose_to_nvfp4_four_six_padded
 * x is [source_rows][source_cols]; output row r, col c = x[c][r]. */
int nvfp4_fp32_transpose_to_nvfp4_four_six_padded(void* stream, const float* x, const float* amax,
                                                  uint8_t* out_fp4, uint8_t* out_scales,
                                                  float* out_global_scale, uint32_t source_rows,
                                                  uint32_t source_cols, uint32_t padded_rows,
                                                  uint32_t padded_cols);
/* B200-native form of the four-six quantizer: f32 or bf16 input [rows][cols] (cols % 16 == 0),
 * tensor (rowwise = 0, amax[0]) or rowwise (amax[row]) global scale, scales written either in
 * the logical layout or directly in the packed layout the GEMM consumes (cols % 64 == 0 then;
 * pad rows up to the next multiple of 128 are filled with 0x38).  Same bytes as the entries
 * above; replaces quantize + Sm120ScalePackModule::pack (scale_pack.rs:54-78) in one pass. */
int nvfp4_quantize_four_six(void* stream, const void* x, int dtype, const float* amax, int rowwise,
                            uint32_t rows, uint32_t cols, uint8_t* out_fp4, uint8_t* out_scales,
                            int scale_layout, float* out_global_scale);

/* Row amax and rowwise four-six in one pass over the input (the caller pattern
 * RowwiseNvfp4Scratch::quantize_row_amax, crates/gpt2-nvfp4/src/types/nvfp4_scratch/scratch.rs:35-52,
 * issues row_amax_f32 then fp32_to_nvfp4_four_six_rowwise).  Same bytes as those two calls.
 * out_row_amax (f32[rows]) is optional for rows of up to 4096 elements and required beyond.
 * out_decoded_amax (f32[1], optional): max |decoded value| of the quantized tensor, the number
 * rowwise_nvfp4_chunk_amax + its reduction (utils/nvfp4/quant/kernels/ms_eden/amax.rs:23-104) derive
 * from the stored tensor in the backward pass; pass it on as x_decoded_amax to skip that pass. */
int nvfp4_quantize_four_six_rowwise_fused(void* stream, const void* x, int dtype, uint32_t rows, uint32_t cols,
                                          uint8_t* out_fp4, uint8_t* out_scales, int scale_layout,
                                          float* out_global_scale, float* out_row_amax, float* out_decoded_amax);

/* gpt/mlp/launcher.rs:66-76  MlpModule::relu2_backward / relu2_backward_f16 (kernels gpt/mlp/kernels.rs:72-104):
 * d_pre = (d_out * 2) * max(pre, 0) between the two MLP linears of the backward pass. */
int nvfp4_relu2_backward(void* stream, const float* pre_activation, const float* d_out, float* d_pre_activation,
                         uint32_t len);
int nvfp4_relu2_backward_f16(void* stream, const uint16_t* pre_activation /* IEEE f16 bits */, const float* d_out,
                             float* d_pre_activation, uint32_t len);
/* all three tensors bf16 (the B200 data flow; no reference counterpart): f32 arithmetic, one rounding to bf16 */
int nvfp4_relu2_backward_bf16(void* stream, const void* pre_activation, const void* d_out, void* d_pre_activation,
                              uint64_t len);

/* The same element-wise pass that also emits the amax of what it stores, as a chunk list (one value per
 * CTA, nvfp4_relu2_backward_amax_chunks(len) of them, written to chunk_amax and counted in *out_chunks).
 * Point chunk_amax at nvfp4_linear_backward_args.e_h.chunk_amax of the MLP fc backward and pass *out_chunks
 * as precomputed_e_amax_chunks: the linear backward then skips its own amax pass over dY, the hand-over the
 * reference makes for the loss gradient (gpt/loss/kernels.rs:67-88 -> backward/final_head/run.rs:34,54).
 * Outputs of the linear backward are bit-identical either way.  pre_kind: 0 f32, 1 bf16, 2 IEEE f16;
 * grad_dtype (d_out and d_pre_activation): NVFP4_DTYPE_F32 or NVFP4_DTYPE_BF16. */
uint32_t nvfp4_relu2_backward_amax_chunks(uint64_t len);
int nvfp4_relu2_backward_amax(void* stream, const void* pre_activation, int pre_kind, const void* d_out,
                              void* d_pre_activation, int grad_dtype, uint64_t len, float* chunk_amax,
                              uint32_t chunk_capacity, uint32_t* out_chunks);

/* gpt/optimizer/launcher/update.rs:11-58  OptimizerModule::materialize_schedule_free
 * (kernels gpt/optimizer/schedule_free/{value,amax,four_six}.rs): the weight a schedule-free optimizer
 * evaluates with, y = z + beta * (x - z) of the two f32 masters, quantized four-six with a tensor scale
 * without ever being written in f32.  amax[1] receives max|y|; chunk_amax[ceil(len/1024)] is optional.
 * len % 16 == 0; scales in the logical layout. */
int nvfp4_materialize_schedule_free(void* stream, const float* z_master, const float* x_master, float* chunk_amax,
                                    float* amax, uint8_t* bytes, uint8_t* scales, float* global_scale, float beta,
                                    uint32_t len);
/* Same for a [rows x cols] weight with the scale bytes written in either layout (NVFP4_SCALES_PACKED is what
 * nvfp4_gemm reads; no reference counterpart for that layout choice). */
int nvfp4_materialize_schedule_free_matrix(void* stream, const float* z_master, const float* x_master,
                                           float* chunk_amax, float* amax, uint8_t* bytes, uint8_t* scales,
                                           int scale_layout, float* global_scale, float beta, uint32_t rows,
                                           uint32_t cols);

/* MS-EDEN quantizer (random-sign Hadamard-32 rotation, RTN nibbles, EDEN-corrected block
 * scale rounded stochastically with a counter RNG) ---------------------------------------- */

typedef struct nvfp4_ms_eden_args {
  int src_kind;                 /* NVFP4_SRC_*                                               */
  int src_dtype;                /* NVFP4_DTYPE_* for the f32/bf16 source kinds               */
  const void* x;                /* f32 / bf16 source                                         */
  const uint8_t* src_bytes;     /* NVFP4 source kinds                                        */
  const uint8_t* src_scales;    /*   scale bytes, layout given by src_scale_layout           */
  int src_scale_layout;         /*   NVFP4_SCALES_* (packed needs source cols % 64 == 0)     */
  const float* src_global;      /*   f32[1] or f32[source_rows]                              */
  uint32_t rows;                /* F32_ROWS: row_count;  transposed kinds: source_rows       */
  uint32_t cols;                /* F32_ROWS: src_row_len; transposed kinds: source_cols      */
  uint32_t dst_row_len;         /* multiple of 32 (64 for the packed layout)                 */
  const float* global_scale;    /* device f32[1] used when host_global_scale_valid == 0      */
  float host_global_scale;      /* used when host_global_scale_valid != 0                    */
  int host_global_scale_valid;
  float scale_override;
  uint32_t sign_seed;
  uint32_t scale_seed;
  uint32_t col_offset;          /* added to the K index of the sign hash (token sharding)    */
  uint32_t group_offset;        /* added to the flat group id of the scale RNG (even)        */
  uint8_t* out_fp4;
  uint8_t* out_scales;
  int scale_layout;             /* NVFP4_SCALES_*                                            */
  float* out_global_scales;     /* f32[out_rows], every entry = the global scale             */
  float* out_chunk_amax;        /* f32[out_rows*dst_row_len/32] or NULL                      */
} nvfp4_ms_eden_args;

/* Generic MS-EDEN entry: every reference variant below is a thin wrapper over it. */
int nvfp4_ms_eden_quantize(void* stream, const nvfp4_ms_eden_args* args /* host */);

/* utils/nvfp4/quant/ms_eden.rs:8-33  Nvfp4QuantModule::fp32_to_nvfp4_ms_eden */
int nvfp4_fp32_to_nvfp4_ms_eden(void* stream, const float* x, uint8_t* out_fp4, uint8_t* out_scales,
                                float* out_global_scales, float* out_chunk_amax, uint32_t row_count,
                                uint32_t src_row_len, uint32_t dst_row_len, float global_scale,
                                float scale_override, uint32_t sign_seed, uint32_t scale_seed);
/* utils/nvfp4/quant/ms_eden.rs:35-60  ..._device_scale  (global_scale read from device) */
int nvfp4_fp32_to_nvfp4_ms_eden_device_scale(void* stream, const float* x, uint8_t* out_fp4,
                                             uint8_t* out_scales, float* out_global_scales,
                                             float* out_chunk_amax, const float* global_scale,
                                             uint32_t row_count, uint32_t src_row_len, uint32_t dst_row_len,
                                             float scale_override, uint32_t sign_seed, uint32_t scale_seed);
/* utils/nvfp4/quant/ms_eden.rs:62-91  ..._device_scale_no_chunk_amax */
int nvfp4_fp32_to_nvfp4_ms_eden_device_scale_no_chunk_amax(void* stream, const float* x, uint8_t* out_fp4,
                                                           uint8_t* out_scales, float* out_global_scales,
                                                           const float* global_scale, uint32_t row_count,
                                                           uint32_t src_row_len, uint32_t dst_row_len,
                                                           float scale_override, uint32_t sign_seed,
                                                           uint32_t scale_seed);
/* utils/nvfp4/quant/ms_eden_fp32_transpose.rs  ..._fp32_transpose_to_nvfp4_ms_eden_device_scale */
int nvfp4_fp32_transpose_to_nvfp4_ms_eden_device_scale(void* stream, const float* x, uint8_t* out_fp4,
                                                       uint8_t* out_scales, float* out_global_scales,
                                                       float* out_chunk_amax, const float* global_scale,
                                                       uint32_t source_rows, uint32_t source_cols,
                                                       uint32_t dst_row_len, float scale_override,
                                                       uint32_t sign_seed, uint32_t scale_seed);
int nvfp4_fp32_transpose_to_nvfp4_ms_eden_device_scale_no_chunk_amax(
    void* stream, const float* x, uint8_t* out_fp4, uint8_t* out_scales, float* out_global_scales,
    const float* global_scale, uint32_t source_rows, uint32_t source_cols, uint32_t dst_row_len,
    float scale_override, uint32_t sign_seed, uint32_t scale_seed);
/* utils/nvfp4/quant/global_scale.rs:11-26  quartet_backward_ms_eden_global_scale_from_chunks
 * out[0] = amax == 0 ? 1 : amax * (17/16*0.93) / 1536 with amax = max(chunk_amax). */
int nvfp4_quartet_backward_ms_eden_global_scale_from_chunks(void* stream, const float* chunk_amax,
                                                            float* out_global_scale, uint32_t chunk_count);
/* utils/nvfp4/quant/ms_eden_quartet.rs:10-31  tensor amax -> global scale -> MS-EDEN rows.
 * out_chunk_amax needs max(ceil(row_count*src_row_len/1024), row_count*dst_row_len/32) floats for
 * the first form (it receives the 32-chunk amax) and ceil(n/1024) floats for the second. */
int nvfp4_fp32_to_nvfp4_quartet_backward_ms_eden_derived_device_scale(
    void* stream, const float* x, uint8_t* out_fp4, uint8_t* out_scales, float* out_global_scales,
    float* out_chunk_amax, float* out_global_scale, uint32_t row_count, uint32_t src_row_len,
    uint32_t dst_row_len, uint32_t sign_seed, uint32_t scale_seed);
int nvfp4_fp32_to_nvfp4_quartet_backward_ms_eden_derived_device_scale_no_chunk_amax(
    void* stream, const float* x, uint8_t* out_fp4, uint8_t* out_scales, float* out_global_scales,
    float* out_chunk_amax, float* out_global_scale, uint32_t row_count, uint32_t src_row_len,
    uint32_t dst_row_len, uint32_t sign_seed, uint32_t scale_seed);
/* utils/nvfp4/quant/ms_eden_quartet.rs:33-56  ..._with_global_scale (host scalar scale). */
int nvfp4_fp32_to_nvfp4_quartet_backward_ms_eden_with_global_scale(
    void* stream, const float* x, uint8_t* out_fp4, uint8_t* out_scales, float* out_global_scales,
    float* out_chunk_amax, uint32_t row_count, uint32_t src_row_len, uint32_t dst_row_len,
    uint32_t sign_seed, uint32_t scale_seed, float global_scale);
/* utils/nvfp4/quant/ms_eden_pair.rs:13-45  one call quantizes dY rows (for dX) and dY
 * transposed (for dW) with one shared tensor scale.  precomputed_chunk_count = 0 computes
 * the 1024-value chunk amax of x into out_chunk_amax first; otherwise out_chunk_amax already
 * holds that many chunk values. */
int nvfp4_fp32_pair_to_nvfp4_quartet_backward_ms_eden_derived_device_scale_no_chunk_amax(
    void* stream, const float* x, uint8_t* out_fp4, uint8_t* out_scales, float* out_global_scales,
    uint8_t* transpose_out_fp4, uint8_t* transpose_out_scales, float* transpose_out_global_scales,
    float* out_chunk_amax, float* out_global_scale, uint32_t row_count, uint32_t src_row_len,
    uint32_t dst_row_len, uint32_t transpose_dst_row_len, uint32_t sign_seed, uint32_t scale_seed,
    uint32_t transpose_scale_seed, uint32_t precomputed_chunk_count);
/* utils/nvfp4/quant/ms_eden_transpose.rs:9-84  NVFP4 weight W[source_rows][source_cols] ->
 * amax of the decoded tensor -> global scale -> MS-EDEN of the transpose. */
int nvfp4_nvfp4_transpose_to_quartet_backward_ms_eden_derived_device_scale(
    void* stream, const uint8_t* in_bytes, const uint8_t* in_scales, const float* in_global_scale,
    uint8_t* out_fp4, uint8_t* out_scales, float* out_global_scales, float* out_chunk_amax,
    float* out_global_scale, uint32_t source_rows, uint32_t source_cols, uint32_t dst_row_len,
    uint32_t sign_seed, uint32_t scale_seed);
int nvfp4_nvfp4_transpose_to_quartet_backward_ms_eden_derived_device_scale_no_chunk_amax(
    void* stream, const uint8_t* in_bytes, const uint8_t* in_scales, const float* in_global_scale,
    uint8_t* out_fp4, uint8_t* out_scales, float* out_global_scales, float* out_chunk_amax,
    float* out_global_scale, uint32_t source_rows, uint32_t source_cols, uint32_t dst_row_len,
    uint32_t sign_seed, uint32_t scale_seed);
/* utils/nvfp4/quant/ms_eden_transpose_rowwise.rs:14-54  same for a rowwise-scaled NVFP4
 * activation X[source_rows][source_cols] saved on the tape. */
int nvfp4_rowwise_nvfp4_transpose_to_quartet_backward_ms_eden_derived_device_scale(
    void* stream, const uint8_t* in_bytes, const uint8_t* in_scales, const float* in_global_scales,
    uint8_t* out_fp4, uint8_t* out_scales, float* out_global_scales, float* out_chunk_amax,
    float* out_global_scale, uint32_t source_rows, uint32_t source_cols, uint32_t dst_row_len,
    uint32_t sign_seed, uint32_t scale_seed);
int nvfp4_rowwise_nvfp4_transpose_to_quartet_backward_ms_eden_derived_device_scale_no_chunk_amax(
    void* stream, const uint8_t* in_bytes, const uint8_t* in_scales, const float* in_global_scales,
    uint8_t* out_fp4, uint8_t* out_scales, float* out_global_scales, float* out_chunk_amax,
    float* out_global_scale, uint32_t source_rows, uint32_t source_cols, uint32_t dst_row_len,
    uint32_t sign_seed, uint32_t scale_seed);

/* decode / layout helpers ----------------------------------------------------------------- */

/* utils/nvfp4/decode/launcher.rs  Nvfp4DecodeModule::decode_transpose_f32 : out[c][r] = value(r,c) */
int nvfp4_decode_transpose_f32(void* stream, const uint8_t* bytes, const uint8_t* scales,
                               const float* global_scale, float* output, uint32_t rows, uint32_t cols);
/* utils/nvfp4/decode/launcher.rs  Nvfp4DecodeModule::decode_rowwise_transpose_f32 */
int nvfp4_decode_rowwise_transpose_f32(void* stream, const uint8_t* bytes, const uint8_t* scales,
                                       const float* global_scales, float* output, uint32_t rows,
                                       uint32_t cols);
/* Untransposed decode (rowwise = 0/1); used for NVFP4-encoded biases. */
int nvfp4_decode_f32(void* stream, const uint8_t* bytes, const uint8_t* scales, const float* global_scales,
                     int rowwise, float* output, uint32_t rows, uint32_t cols);
/* utils/nvfp4_tma_matmul/scale_pack.rs:54-78  Sm120ScalePackModule::pack : logical -> packed,
 * pad rows filled with 0x38. */
int nvfp4_scale_pack(void* stream, const uint8_t* logical, uint8_t* packed, uint32_t mn_extent,
                     uint32_t k_dim);
/* utils/nvfp4_tma_matmul/pad.rs:49-107  TmaMatrixPadModule */
int nvfp4_pad_u4_rows(void* stream, const uint8_t* src, uint8_t* dst, uint32_t rows, uint32_t padded_rows,
                      uint32_t cols);
int nvfp4_pad_f32(void* stream, const float* src, float* dst, uint32_t rows, uint32_t cols,
                  uint32_t padded_rows, uint32_t padded_cols);
int nvfp4_transpose_pad_f32(void* stream, const float* src, float* dst, uint32_t rows, uint32_t cols,
                            uint32_t padded_rows, uint32_t padded_cols);
int nvfp4_crop_f32(void* stream, const float* src, float* dst, uint32_t rows, uint32_t src_cols,
                   uint32_t dst_cols);

/* block-scaled GEMM ----------------------------------------------------------------------- */

typedef struct nvfp4_gemm_args {
  const uint8_t* a_bytes;       /* A [m][k] nibbles, K-major, row pitch k/2 bytes (16-byte aligned) */
  const uint8_t* a_scales;      /* packed layout, rows padded to 128                          */
  const float* a_global;        /* f32[1] (mode 1) or f32[m] (mode 2); unused in mode 0       */
  const uint8_t* b_bytes;       /* B [n][k] nibbles, K-major                                  */
  const uint8_t* b_scales;      /* packed layout                                              */
  const float* b_global;        /* f32[1]; unused in mode 0                                   */
  void* out;                    /* [m][ldo] f32 or bf16                                       */
  void* aux;                    /* RELU2: pre-activation [m][ldo] (same dtype) or NULL        */
  const float* bias;            /* f32[n] for epilogues 1..3, else NULL                       */
  uint32_t m, n, k;             /* k % 64 == 0                                                */
  uint32_t ldo;                 /* output row pitch in elements (>= n)                        */
  int global_scale_mode;        /* NVFP4_GS_*                                                 */
  float weight_global_scale;    /* the reference passes 1.0                                   */
  int epilogue;                 /* NVFP4_EPI_*                                                */
  int out_dtype;                /* NVFP4_DTYPE_*                                              */
} nvfp4_gemm_args;

/* out[m][n] = epilogue( (sum_k A*sa * B*sb) * weight * ga * gb ), FP32 accumulation in tensor
 * memory by tcgen05.mma kind::mxf4nvf4.  Replaces pack + prepare_tma + gemm_tma + post-op
 * (utils/nvfp4_tma_matmul/launcher.rs:106-328, gpt/projection_postop.rs:50-162).           */
int nvfp4_gemm(void* stream, const nvfp4_gemm_args* args /* host */);

/* utils/nvfp4_tma_matmul/launcher.rs:172-222  gemm_tma_nvfp4_device_scales_and_global_scale_buffers */
int nvfp4_gemm_tma_nvfp4_device_scales_and_global_scale_buffers(
    void* stream, const uint8_t* a_bytes, const uint8_t* a_scales_packed, const uint8_t* b_bytes,
    const uint8_t* b_scales_packed, float* out, uint32_t token_count, uint32_t input_dim,
    uint32_t output_dim, const float* a_global_scale, const float* b_global_scale);
/* utils/nvfp4_tma_matmul/launcher.rs:224-274  gemm_tma_nvfp4_rowwise_a_scale_and_global_scale_buffer */
int nvfp4_gemm_tma_nvfp4_rowwise_a_scale_and_global_scale_buffer(
    void* stream, const uint8_t* a_bytes, const uint8_t* a_scales_packed, const uint8_t* b_bytes,
    const uint8_t* b_scales_packed, float* out, uint32_t token_count, uint32_t input_dim,
    uint32_t output_dim, const float* a_global_scales, const float* b_global_scale);
/* utils/nvfp4_tma_matmul/launcher.rs:276-328  gemm_tma_nvfp4_rowwise_a_scale_padded_output
 * (B holds padded_output_dim rows; only output_dim columns are written, row pitch output_dim). */
int nvfp4_gemm_tma_nvfp4_rowwise_a_scale_padded_output(
    void* stream, const uint8_t* a_bytes, const uint8_t* a_scales_packed, const uint8_t* b_bytes,
    const uint8_t* b_scales_packed, float* out, uint32_t token_count, uint32_t input_dim,
    uint32_t output_dim, uint32_t padded_output_dim, const float* a_global_scales,
    const float* b_global_scale);

/* Run-to-run reproducibility of split-K GEMMs (no reference counterpart: the reference's GEMM never splits K).
 * Long-K f32 GEMMs with few output tiles (dW = dY^T.X) split K over several CTAs whose partial tiles are summed
 * with TMA reduce-add in arrival order: with two splits the sum is order-free, with more (small dW such as
 * 768 x 768) the last bits can differ from run to run, always inside the GEMM tolerance.  on = 1 caps the split
 * count at two (process-wide; those GEMMs then fill fewer SMs); the default 0 takes as many splits as fill the
 * SMs.  Quantizer outputs, dbias and every unsplit GEMM are reproducible either way. */
int nvfp4_set_deterministic_reductions(int on);
int nvfp4_get_deterministic_reductions(void);

/* Measurement aid (no reference counterpart; off by default).  Between begin and end every GEMM
 * launch of this process is bracketed by a CUDA event pair recorded on the launch stream (up to
 * max_records launches; the events are created by begin, once).  end waits for the recorded
 * launches and returns their count, summed duration and summed 2*m*n*k, and optionally the
 * per-launch values (host arrays of `capacity` entries). */
int nvfp4_gemm_timing_begin(uint32_t max_records);
int nvfp4_gemm_timing_end(uint32_t* count, double* total_ms, double* total_flops, float* per_launch_ms,
                          double* per_launch_flops, uint32_t capacity);

/* post-ops as separate passes (gpt/projection_postop.rs:50-162); bias is NVFP4 encoded ----- */
int nvfp4_projection_bias_inplace(void* stream, float* raw, const uint8_t* bias_bytes,
                                  const uint8_t* bias_scales, const float* bias_global_scale,
                                  uint32_t rows, uint32_t cols);
int nvfp4_projection_residual_add(void* stream, const float* raw, const uint8_t* bias_bytes,
                                  const uint8_t* bias_scales, const float* bias_global_scale,
                                  float* residual, uint32_t rows, uint32_t cols);
int nvfp4_projection_relu2_inplace(void* stream, float* pre_activation, float* out,
                                   const uint8_t* bias_bytes, const uint8_t* bias_scales,
                                   const float* bias_global_scale, uint32_t rows, uint32_t cols);

/* linear backward ------------------------------------------------------------------------- */

/* gpt/linear_backward/bias.rs:18-69 + kernels/bias.rs:10  dbias[col] = sum_rows e[row][col],
 * summed in the reference's fixed order (bit-exact). */
int nvfp4_linear_bias_grad(void* stream, const float* e, float* dbias, uint32_t token_count,
                           uint32_t output_dim);
/* Same sum, same order, for a bf16 dY (no reference counterpart: the reference is f32-only). */
int nvfp4_linear_bias_grad_bf16(void* stream, const void* e, float* dbias, uint32_t token_count,
                                uint32_t output_dim);

/* Scratch of one linear backward (gpt/linear_backward/args/ms_eden/scratch.rs:11-160).  All
 * buffers are caller owned; sizes with ok = padded_k(output_dim), tk = padded_k(token_count):
 *   e_h      : bytes token*ok/2, scales_packed packed_len(token, ok), global_scales token
 *   e_t_h    : bytes out*tk/2,   scales_packed packed_len(out, tk),   global_scales out
 *   weight_t : bytes in*ok/2,    scales_packed packed_len(in, ok),    global_scales in
 *   input_t  : bytes in*tk/2,    scales_packed packed_len(in, tk),    global_scales in
 *   chunk_amax: max over the operands of ceil(elements/1024) floats; global_scale f32[1] each */
typedef struct nvfp4_ms_eden_operand {
  uint8_t* bytes;
  uint8_t* scales_packed;
  float* global_scales;
  float* global_scale;   /* f32[1] */
  float* chunk_amax;
} nvfp4_ms_eden_operand;

typedef struct nvfp4_linear_backward_args {
  const void* e;                     /* dY [token][out], f32 or bf16 (e_dtype)                */
  int e_dtype;
  /* weight: NVFP4 tensor-scale W[out][in] */
  const uint8_t* w_bytes;
  const uint8_t* w_scales;
  int w_scale_layout;                /* NVFP4_SCALES_*                                        */
  const float* w_global;
  /* saved activation: NVFP4 rowwise X[token][in] */
  const uint8_t* x_bytes;
  const uint8_t* x_scales;
  int x_scale_layout;                /* NVFP4_SCALES_*                                        */
  const float* x_globals;
  nvfp4_ms_eden_operand e_h, e_t_h, weight_t_h, input_t_h;
  void* dinput;                      /* [token][in]                                           */
  int dinput_dtype;                  /* NVFP4_DTYPE_*                                         */
  void* dweight;                     /* [out][in]                                             */
  int dweight_dtype;                 /* NVFP4_DTYPE_* (f32 lets long-K GEMMs split K)         */
  float* dbias;                      /* f32[out] or NULL                                      */
  uint32_t token_count, input_dim, output_dim;
  uint32_t sign_seed, scale_seed;
  uint32_t precomputed_e_amax_chunks; /* 0 = compute the dY chunk amax here                   */
  uint32_t token_offset;             /* first token of this shard (sign / RNG index spaces)   */
  const float* e_global_scale_override; /* device f32[1] shared across shards, or NULL        */
  const float* x_decoded_amax;       /* device f32[1]: max |decoded X| (from the forward quantizer),
                                        or NULL = compute it here with a pass over X             */
} nvfp4_linear_backward_args;

/* gpt/linear_backward/ms_eden.rs:15-55  LinearBackwardModule::backward_ms_eden :
 * dbias, MS-EDEN quantization of dY (rows + transposed), W^T, X^T, then
 * dX = dY.W and dW = dY^T.X on the tcgen05 GEMM. */
int nvfp4_linear_backward_ms_eden(void* stream, const nvfp4_linear_backward_args* args /* host */);

/* utils/nvfp4_tc_matmul/launcher.rs:23-87  Nvfp4TcMatmulModule::matmul_ms_eden : out[m][n] (f32) = a[m][k] . b_t[n][k]^T
 * with both operands MS-EDEN quantized (caller-given global scales, the second with scale_seed ^ 0x9e3779b9) and K
 * zero-padded to a multiple of 64.  The operand structs are caller scratch: bytes [rows * padded_k / 2], scales_packed
 * [nvfp4_scale_packed_len(rows, padded_k)], global_scales [rows], chunk_amax [rows * padded_k / 32]; their global_scale
 * member is not used.  The reference's padded f32 copies of the operands are not needed. */
int nvfp4_tc_matmul_ms_eden(void* stream, const float* a, const float* b_t, float* out,
                            const nvfp4_ms_eden_operand* a_q, float a_global_scale,
                            const nvfp4_ms_eden_operand* b_q, float b_global_scale, uint32_t m, uint32_t n, uint32_t k,
                            uint32_t sign_seed, uint32_t scale_seed);


#ifdef __cplusplus
}
#endif
#endif /* NVFP4_B200_H_ */
