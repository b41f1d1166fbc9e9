/*
 * nvfp4_b200_step.h -- C ABI of the C++ training-step driver (include/nvfp4_b200_step.hpp), for callers that
 * are not C++ (the benchmark binds it with ctypes; a Rust trainer would bind it with an extern "C" block).
 *
 * This is caller-side glue, not part of the kernel library: it owns buffers, streams and (optionally) an NCCL
 * communicator, and sequences the calls of nvfp4_b200.h the way crates/gpt2-nvfp4 sequences the reference's
 * kernels (types/{l2_attention,l3_mlp}/forward.rs, types/model/final_logits.rs, backward/{linear,mlp/run,
 * attention/*,final_head/run}.rs), restricted to the projections of a GPT-2 shaped model.  Everything is
 * asynchronous on the stream passed to nvfp4_step_run; return values are 0 or a CUDA error number, with the
 * text of the last failure in nvfp4_step_error.
 */
#ifndef NVFP4_B200_STEP_H_
#define NVFP4_B200_STEP_H_

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef struct nvfp4_step_config {
  uint32_t n_layer, d_model, d_mlp, vocab;
  uint32_t tokens;          /* rows this rank holds (multiple of 128)                           */
  uint32_t token_offset;    /* first token of this rank's shard                                 */
  uint32_t total_tokens;    /* tokens of the whole batch (0 = tokens)                           */
  uint64_t seed;            /* MS-EDEN seed stream (crates/gpt2-nvfp4/src/random.rs:1-27)       */
  int fused_mlp;            /* 1: fc stores only its pre-activation, relu^2 applied on load     */
  int reproducible_sharding;/* 1: all-reduce(max) of the step's amaxes, unsharded RNG indices   */
} nvfp4_step_config;

/* weights[i] bf16 [out][in], biases[i] f32 [out] or NULL, for linear i = layer * 4 + {c_attn, attn c_proj,
 * mlp fc, mlp proj}, then the LM head (n_linears = 4 * n_layer + 1).  x / dy: one bf16 [tokens][width] device
 * tensor per activation width (d_model, d_mlp) and per gradient width (3 d_model, d_model, d_mlp, vocab).
 * All pointers are device pointers owned by the caller and must outlive the handle.  NULL on failure
 * (nvfp4_step_error(NULL) has the reason). */
void* nvfp4_step_create(const nvfp4_step_config* cfg, const void* const* weights, const void* const* biases,
                        uint32_t n_linears, const uint32_t* x_widths, const void* const* x_ptrs, uint32_t n_x,
                        const uint32_t* dy_widths, const void* const* dy_ptrs, uint32_t n_dy);
void nvfp4_step_destroy(void* handle);
const char* nvfp4_step_error(void* handle);
/* One forward + backward pass (weight quantization included unless weights_changed == 0). */
int nvfp4_step_run(void* handle, void* stream, int weights_changed);
/* Swaps the activation / gradient inputs (double-buffered loaders). */
int nvfp4_step_set_inputs(void* handle, const uint32_t* x_widths, const void* const* x_ptrs, uint32_t n_x,
                          const uint32_t* dy_widths, const void* const* dy_ptrs, uint32_t n_dy);
/* Gradient bucket i (0 .. n_layer: a layer's dW and dbias, the last one the LM head's dW), f32. */
int nvfp4_step_bucket(void* handle, uint32_t index, float** ptr, uint64_t* len);
/* dX of the linears with this input width (bf16 [tokens][width]); outputs of the linears of an output width. */
int nvfp4_step_dx(void* handle, uint32_t width, void** ptr);
int nvfp4_step_y(void* handle, uint32_t width, void** ptr);
uint64_t nvfp4_step_flops(void* handle);
/* NCCL: rank 0 makes an id (128 bytes), every rank attaches with it (collective).  Without a communicator the
 * step reduces nothing. */
int nvfp4_step_nccl_unique_id(uint8_t* id128);
int nvfp4_step_attach_nccl(void* handle, const uint8_t* id128, int rank, int world);

#ifdef __cplusplus
}
#endif
#endif /* NVFP4_B200_STEP_H_ */
