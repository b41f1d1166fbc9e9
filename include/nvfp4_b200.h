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
 * x_decoded_amax, nvfp4_quantize_four_six_rowwise_fused gained out_decoded_amax.  3: nvfp4_gemm_args gained
 * the NVFP4 bias and relu2_row_amax members, nvfp4_linear_backward_args gained side_stream / fork_event /
 * join_event, total_token_count and weight_t_prepared, nvfp4_ms_eden_args gained group_row_stride, element counts of the
 * tensor-amax entries became 64-bit. */
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
uint32_t nvfp4_tensor_amax_chunks(uint64_t element_count);

/* amax ------------------------------------------------------------------------------------ */

/* utils/nvfp4/quant/amax.rs:8-17  Nvfp4QuantModule::row_amax_f32 */
int nvfp4_row_amax_f32(void* stream, const float* x, float* out, uint32_t row_count, uint32_t row_len);
/* bf16-input variant of the above (no reference counterpart: the reference is f32-only). */
int nvfp4_row_amax_bf16(void* stream, const void* x, float* out, uint32_t row_count, uint32_t row_len);
/* utils/nvfp4/quant/amax.rs:19-23  Nvfp4QuantModule::tensor_amax_f32
 * chunk_amax[ceil(n/1024)] and out[1] are both written. */
int nvfp4_tensor_amax_f32(void* stream, const float* x, float* chunk_amax, float* out, uint64_t element_count);
int nvfp4_tensor_amax_bf16(void* stream, const void* x, float* chunk_amax, float* out, uint64_t element_count);
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

/* The same quantizer applied to relu(pre)^2 computed on load (f32 arithmetic: max(pre, 0) then one multiply),
 * for an MLP whose up projection stored only its pre-activation: the activation relu(pre)^2 is never written
 * to memory (the reference writes both, gpt/projection_postop.rs:140-162, and hands the row amax of the
 * activation to this quantizer, crates/gpt2-nvfp4/src/types/l3_mlp/forward.rs:60-76).  row_amax_in (f32[rows],
 * optional): the row amax of relu(pre)^2 if the producer already has it (nvfp4_gemm_args.relu2_row_amax);
 * NULL = computed here.  Same bytes as materialising relu(pre)^2 in f32 and quantizing that. */
int nvfp4_quantize_relu2_four_six_rowwise(void* stream, const void* pre_activation, int dtype, uint32_t rows,
                                          uint32_t cols, const float* row_amax_in, uint8_t* out_fp4,
                                          uint8_t* out_scales, int scale_layout, float* out_global_scale,
                                          float* out_row_amax, float* out_decoded_amax);

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
  uint32_t group_row_stride;    /* 16-groups per output row in the scale RNG's index space; 0 = dst_row_len / 16.
                                   A token shard of a transposed operand passes the unsharded K / 16 here and
                                   first_token / 16 as group_offset to draw the unsharded tensor's bits.    */
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
  /* Optional members (zero the struct first).  An NVFP4-encoded bias [n], the form the reference's
   * projections take it in (gpt/attention/qkv_projection/launcher.rs:8-25: bias.bytes, bias.scales,
   * bias.global_scale), decoded in the epilogue as (e2m1 * e4m3) * global_scale; read when `bias` is NULL. */
  const uint8_t* bias_nvfp4_bytes;   /* u8[n/2]                                               */
  const uint8_t* bias_nvfp4_scales;  /* u8[n/16], logical layout                              */
  const float* bias_nvfp4_global;    /* f32[1]                                                */
  /* f32[m] or NULL: receives, per output row, max over the columns of relu(stored value)^2 -- the row amax
   * of the activation a ReLU^2 MLP feeds to its down projection, handed to the next quantizer the way the
   * reference's post-op hands it over (gpt/projection_postop.rs:140-162,
   * crates/gpt2-nvfp4/src/types/l3_mlp/forward.rs:60-76).  Needs a 16-byte aligned output / row pitch. */
  float* relu2_row_amax;
} nvfp4_gemm_args;

/* out[m][n] = epilogue( (sum_k A*sa * B*sb) * weight * ga * gb ), FP32 accumulation in tensor
 * memory by tcgen05.mma kind::mxf4nvf4.  Replaces pack + prepare_tma + gemm_tma + post-op
 * (utils/nvfp4_tma_matmul/launcher.rs:106-328, gpt/projection_postop.rs:50-162).           */
int nvfp4_gemm(void* stream, const nvfp4_gemm_args* args /* host */);

/* What nvfp4_gemm would choose for `args` on the current device, without launching (no reference
 * counterpart: the reference has one tile shape, utils/nvfp4_tma_matmul/kernels.rs:1314).  Lets a caller
 * or a test see which kernel instantiation and schedule a shape takes. */
typedef struct nvfp4_gemm_plan {
  uint32_t block_m;       /* tile height: 128 rows, or 256 (two MMAs per k-atom sharing the B stage)       */
  uint32_t block_n;       /* tile width: 128, 192 or 256 output columns (256 x 192 is the only tall shape) */
  uint32_t acc_stages;    /* accumulator buffers in tensor memory: 2 (128 x 128, 128 x 192) or 1           */
  uint32_t k_splits;      /* > 1: K split over CTAs, partial tiles summed with TMA reduce-add              */
  uint32_t b_resident;    /* 1: the B panel of a column block stays in shared memory (short K)             */
  uint32_t resident_cpn;  /* resident mode: CTAs per column block of the banded schedule, 0 = contiguous   */
  uint32_t stages;        /* depth of the shared-memory operand ring                                       */
  uint32_t grid;          /* CTAs (persistent, at most one per SM)                                         */
  uint32_t tma_store;     /* 1: epilogue stores through shared memory + TMA, 0: direct stores              */
  uint32_t smem_bytes;    /* dynamic shared memory of the launch                                           */
} nvfp4_gemm_plan;
int nvfp4_gemm_plan_query(const nvfp4_gemm_args* args /* host */, nvfp4_gemm_plan* out /* host */);

/* utils/nvfp4_tma_matmul/launcher.rs:39-166  Nvfp4GemmModule::prepare_tma_nvfp4_device_scales{,_into}.
 * The reference encodes four tensor maps per GEMM on the host and copies them into caller-owned device
 * memory (4 x 128 bytes, TmaNvfp4DeviceScaleDescriptors, tma.rs:8-13) before every launch.  Here tensor
 * maps travel as kernel parameters and the scale planes need no map at all (a k-tile's scales are
 * contiguous in the packed layout), so `descriptors` is accepted and left untouched.  The call validates
 * the shapes like the reference (input_dim % 64, 16-byte aligned operands; 1 = invalid value) and encodes
 * the two operand maps into the calling thread's tensor-map cache, where every later nvfp4_gemm* call on
 * the same buffers finds them: persistent buffers are encoded once, not once per launch.  Optional --
 * a GEMM call on buffers it has not seen encodes and caches the maps itself. */
int nvfp4_prepare_tma_nvfp4_device_scales(void* stream, const uint8_t* input_bytes, const uint8_t* input_scale_data,
                                          const uint8_t* weight_bytes, const uint8_t* weight_scale_data,
                                          uint32_t token_count, uint32_t input_dim, uint32_t output_dim);
int nvfp4_prepare_tma_nvfp4_device_scales_into(void* stream, const uint8_t* input_bytes,
                                               const uint8_t* input_scale_data, const uint8_t* weight_bytes,
                                               const uint8_t* weight_scale_data, uint32_t token_count,
                                               uint32_t input_dim, uint32_t output_dim,
                                               void* descriptors /* device, 4 x 128 bytes, may be NULL */);
/* Tensor maps encoded (misses) and reused (hits) by the calling thread so far. */
int nvfp4_tensor_map_cache_stats(uint64_t* hits, uint64_t* misses);

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

/* Measurement aid (no reference counterpart): forces the tile shape of every following GEMM of this process
 * (128 x 128, 128 x 192, 128 x 256 or 256 x 192; block_n = 0 = automatic choice, the default; the environment
 * variable NVFP4_GEMM_TILE = "<width>" or "<height>x<width>" sets the initial value). */
int nvfp4_gemm_set_tile_override(int block_m, int block_n);
/* Limit of every bounded wait inside the GEMM kernel in nanoseconds (default 2 s; 0 restores it).  A wait
 * that runs out sets a bit of the device status word (nvfp4_read_device_status: 1 producer, 2 MMA /
 * scale-factor warps, 4 epilogue), all roles of that CTA leave their loops, tensor memory is freed and
 * the kernel returns; the CTA's output tiles are then unspecified.  The reference's waits spin without a
 * limit (utils/nvfp4_tma_matmul/kernels.rs:172-174). */
int nvfp4_gemm_set_wait_timeout_ns(uint64_t ns);
/* Test aid: bit 0 makes CTA 0 of every following GEMM skip the loads of its first k-tile, so that the
 * waits on that stage run out (the safe way to exercise the time-out path: nothing faults, the kernel
 * returns).  0 (default) = normal operation. */
int nvfp4_gemm_set_debug_flags(uint32_t flags);

/* Measurement aid (no reference counterpart; off by default).  Between begin and end every GEMM
 * launch of this process is bracketed by a CUDA event pair recorded on the launch stream (up to
 * max_records launches; the events are created by begin, once).  end waits for the recorded
 * launches and returns their count, summed duration and summed 2*m*n*k, and optionally the
 * per-launch values (host arrays of `capacity` entries). */
int nvfp4_gemm_timing_begin(uint32_t max_records);
int nvfp4_gemm_timing_end(uint32_t* count, double* total_ms, double* total_flops, float* per_launch_ms,
                          double* per_launch_flops, uint32_t capacity);

/* forward projections with the reference's argument lists -------------------------------------- */

/* One forward projection Y = X . W^T + b the way the reference's module methods take it: X a rowwise NVFP4
 * activation, W an NVFP4 tensor-scale weight, b an NVFP4-encoded bias (bytes, logical scales, global_scale),
 * dimensions as u32.  Scale bytes of X and W may be logical (the reference's tensor format; the matching
 * *_scales_packed_scratch must then hold nvfp4_scale_packed_len(rows, input_dim) bytes and is filled by the
 * call -- the scratch LmHeadTmaArgs carries, gpt/lm_head.rs:41-54) or already packed (what this library's
 * quantizers write; no scratch).  One fused launch: global scales, bias, activation / residual and the cast
 * all happen in the GEMM epilogue. */
typedef struct nvfp4_projection_args {
  const uint8_t* input_bytes;          /* X [token_count][input_dim] nibbles                       */
  const uint8_t* input_scales;
  int input_scale_layout;              /* NVFP4_SCALES_*                                           */
  const float* input_global_scales;    /* f32[token_count]                                         */
  const uint8_t* weight_bytes;         /* W [output_dim][input_dim] nibbles                        */
  const uint8_t* weight_scales;
  int weight_scale_layout;
  const float* weight_global_scale;    /* f32[1]                                                   */
  const uint8_t* bias_bytes;           /* NVFP4 bias [output_dim]; all three NULL = no bias        */
  const uint8_t* bias_scales;
  const float* bias_global_scale;
  void* out;                           /* the method's output (see each entry), [token_count][output_dim] */
  void* pre_activation;                /* up_relu2 only                                            */
  int out_dtype;                       /* NVFP4_DTYPE_F32 (the reference's type) or NVFP4_DTYPE_BF16 */
  float* relu2_row_amax;               /* up_relu2 only, optional f32[token_count]                 */
  uint32_t token_count, input_dim, output_dim;
  uint8_t* input_scales_packed_scratch;
  uint8_t* weight_scales_packed_scratch;
} nvfp4_projection_args;
/* gpt/attention/qkv_projection/launcher.rs:8-25  AttentionModule::qkv_projection : out = X . W^T + b */
int nvfp4_qkv_projection(void* stream, const nvfp4_projection_args* args /* host */);
/* gpt/attention/qkv_projection/launcher.rs:27-42  AttentionModule::c_proj : out (the f32 residual stream, in
 * place) = fma(1, X . W^T + b, out); output_dim = input_dim = embedding_dim */
int nvfp4_c_proj(void* stream, const nvfp4_projection_args* args);
/* gpt/mlp/launcher.rs:53-59  MlpModule::up_relu2 : pre_activation = X . W^T + b, out = max(pre, 0)^2.  `out`
 * may be NULL: only the pre-activation is stored (see nvfp4_quantize_relu2_four_six_rowwise). */
int nvfp4_mlp_up_relu2(void* stream, const nvfp4_projection_args* args);
/* gpt/mlp/launcher.rs:60-66  MlpModule::down_residual : out (residual, f32, in place) += X . W^T + b */
int nvfp4_mlp_down_residual(void* stream, const nvfp4_projection_args* args);
/* gpt/lm_head.rs:65-87  LmHeadModule::logits : out = X . W^T (no bias; weight_global_scale as given) */
int nvfp4_lm_head_logits(void* stream, const nvfp4_projection_args* args);
/* gpt/lm_head.rs:89-125  LmHeadModule::logits_tma : the same product through the reference's pack +
 * prepare_tma + TMA GEMM sequence; one launch here */
int nvfp4_lm_head_logits_tma(void* stream, const nvfp4_projection_args* args);
/* gpt/next_latent/launch_projection.rs:10-29  NextLatModule::projection : out = X . W^T + b */
int nvfp4_nextlat_projection(void* stream, const nvfp4_projection_args* args);

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
  /* Optional second stream (cudaStream_t) with two events (cudaEvent_t), all caller owned: the two NVFP4
   * transposers (W^T, X^T) depend on nothing else in the call and are ALU bound, so they can run beside the
   * bandwidth-bound dY amax pass.  The call forks onto side_stream after recording fork_event on `stream` and
   * joins through join_event before the GEMMs, on every path including errors; NULL side_stream = everything
   * in order on `stream`.  The library owns no stream, event or lock. */
  void* side_stream;
  void* fork_event;
  void* join_event;
  /* Token sharding: tokens of the unsharded batch (0 = token_count, i.e. not sharded).  With token_offset,
   * e_global_scale_override and x_decoded_amax (both derived from the all-reduced amax) a shard then draws
   * exactly the bits of the unsharded operands, so the shards' dW partial sums add up to the unsharded dW
   * up to f32 summation order. */
  uint32_t total_token_count;
  /* 1: weight_t_h already holds W^T quantized for this call's seeds by nvfp4_linear_backward_prepare_weight_t
   * (that step depends on the weight and the seeds only); the call then skips it. */
  int weight_t_prepared;
} nvfp4_linear_backward_args;

/* gpt/linear_backward/ms_eden.rs:15-55  LinearBackwardModule::backward_ms_eden :
 * dbias, MS-EDEN quantization of dY (rows + transposed), W^T, X^T, then
 * dX = dY.W and dW = dY^T.X on the tcgen05 GEMM. */
int nvfp4_linear_backward_ms_eden(void* stream, const nvfp4_linear_backward_args* args /* host */);
/* The W^T step of backward_ms_eden alone (gpt/linear_backward/ms_eden/quantize/transpose.rs:14-93, weight half):
 * amax of the decoded weight -> global scale -> MS-EDEN of W^T into args->weight_t_h, with the seeds of `args`.
 * It reads only the weight, so a caller may enqueue it early and on another stream (beside the forward pass,
 * right after the weight was quantized) and pass weight_t_prepared = 1 to the backward call: the replicated
 * weight-side work of a token-sharded step then leaves the critical path. */
int nvfp4_linear_backward_prepare_weight_t(void* stream, const nvfp4_linear_backward_args* args /* host */);

/* gpt/linear_backward/device_scale.rs:38-187  LinearBackwardModule::backward_device_scale_tma,
 * backward_device_scale, backward_device_scale_cta and gpt/linear_backward.rs:40-67 backward: the two gradient
 * GEMMs over operands that are already MS-EDEN quantized, dX[token][in] = e_h . weight_t_h^T and
 * dW[out][in] = e_t_h . input_t_h^T (K = padded_k(output_dim) and padded_k(token_count)).  The reference's
 * three variants differ only in which of its kernels runs (TMA, warp, CTA pair); all three names resolve to
 * the one tcgen05 GEMM here.  Operand scale bytes may be logical (the reference's layout; scales_packed_scratch
 * of that operand must then hold nvfp4_scale_packed_len(rows, k) bytes, the LinearBackwardTmaScratch of the
 * reference) or already packed (scratch unused).  e_h / e_t_h carry per-row global scales, weight_t_h /
 * input_t_h one scale (global_scale[0]). */
typedef struct nvfp4_backward_operand {
  const uint8_t* bytes;
  const uint8_t* scales;
  int scale_layout;                /* NVFP4_SCALES_*                                            */
  const float* global_scales;      /* f32[rows] (e_h, e_t_h) or f32[1] (weight_t_h, input_t_h)  */
  uint8_t* scales_packed_scratch;  /* used when scale_layout == NVFP4_SCALES_LOGICAL            */
} nvfp4_backward_operand;
typedef struct nvfp4_linear_backward_device_scale_args {
  nvfp4_backward_operand e_h, weight_t_h, e_t_h, input_t_h;
  void* dinput;                    /* [token][in]                                               */
  int dinput_dtype;
  void* dweight;                   /* [out][in]                                                 */
  int dweight_dtype;
  uint32_t token_count, input_dim, output_dim;
} nvfp4_linear_backward_device_scale_args;
int nvfp4_linear_backward_device_scale_tma(void* stream, const nvfp4_linear_backward_device_scale_args* args);
int nvfp4_linear_backward_device_scale(void* stream, const nvfp4_linear_backward_device_scale_args* args);
int nvfp4_linear_backward_device_scale_cta(void* stream, const nvfp4_linear_backward_device_scale_args* args);
int nvfp4_linear_backward(void* stream, const nvfp4_linear_backward_device_scale_args* args);

/* utils/nvfp4_tc_matmul/launcher.rs:23-87  Nvfp4TcMatmulModule::matmul_ms_eden : out[m][n] (f32) = a[m][k] . b_t[n][k]^T
 * with both operands MS-EDEN quantized (caller-given global scales, the second with scale_seed ^ 0x9e3779b9) and K
 * zero-padded to a multiple of 64.  The operand structs are caller scratch: bytes [rows * padded_k / 2], scales_packed
 * [nvfp4_scale_packed_len(rows, padded_k)], global_scales [rows], chunk_amax [rows * padded_k / 32]; their global_scale
 * member is not used.  The reference's padded f32 copies of the operands are not needed. */
int nvfp4_tc_matmul_ms_eden(void* stream, const float* a, const float* b_t, float* out,
                            const nvfp4_ms_eden_operand* a_q, float a_global_scale,
                            const nvfp4_ms_eden_operand* b_q, float b_global_scale, uint32_t m, uint32_t n, uint32_t k,
                            uint32_t sign_seed, uint32_t scale_seed);


/* ---- NVFP4 checkpoint container ----------------------------------------------------------------------------
 * src/checkpoint/format/writer.rs:15-38 (CheckpointWriter::write_header / write_tensor / finish),
 * src/checkpoint/format/reader.rs:22-67 (CheckpointReader::read_header / read_tensor), constants
 * src/checkpoint/format.rs:7-8.  Little-endian: magic "GPT2_NVFP4_CHECKPOINT\n", u32 version (2), u32 tensor
 * count; per tensor u32 name_len, u64 len, u64 byte_len, u64 scale_len, f32 global_scale, name, bytes, scales.
 * Scale bytes in a checkpoint are in the logical row-major layout.  Files are byte-identical to the reference's
 * for the same tensors.  The *_device forms copy each member through pinned host memory and synchronize the
 * stream, as src/checkpoint/save/tensor.rs:14-20 and load/tensor.rs:17-23 do; reading for the device also applies
 * the length checks of load/tensor.rs:27-39 (bytes = len / 2, scales = len / 16). */
typedef struct nvfp4_checkpoint_tensor_info {
  char name[256];        /* NUL-terminated copy of the tensor's name                          */
  uint64_t len;          /* elements                                                           */
  uint64_t byte_len;     /* nibble bytes stored                                                */
  uint64_t scale_len;    /* scale bytes stored                                                 */
  float global_scale;
} nvfp4_checkpoint_tensor_info;
int nvfp4_checkpoint_writer_open(const char* path, uint32_t tensor_count, void** writer_out);
int nvfp4_checkpoint_write_tensor(void* writer, const char* name, uint64_t len, float global_scale,
                                  const uint8_t* bytes /* host */, uint64_t byte_len, const uint8_t* scales /* host */,
                                  uint64_t scale_len);
int nvfp4_checkpoint_write_tensor_device(void* writer, void* stream, const char* name, uint64_t len,
                                         const float* global_scale /* device f32[1] */, const uint8_t* bytes /* device */,
                                         uint64_t byte_len, const uint8_t* scales /* device */, uint64_t scale_len);
/* Flushes and closes; an error if fewer tensors were written than the header declares. */
int nvfp4_checkpoint_writer_close(void* writer);
int nvfp4_checkpoint_reader_open(const char* path, void** reader_out, uint32_t* tensor_count_out);
/* Reads the next tensor's header and name; its payload must then be taken with one of the two calls below. */
int nvfp4_checkpoint_next_tensor(void* reader, nvfp4_checkpoint_tensor_info* info);
int nvfp4_checkpoint_read_payload(void* reader, uint8_t* bytes /* host */, uint64_t byte_capacity,
                                  uint8_t* scales /* host */, uint64_t scale_capacity);
int nvfp4_checkpoint_read_payload_device(void* reader, void* stream, uint8_t* bytes /* device */,
                                         uint8_t* scales /* device */, float* global_scale /* device f32[1] */);
int nvfp4_checkpoint_reader_close(void* reader);


#ifdef __cplusplus
}
#endif
#endif /* NVFP4_B200_H_ */
