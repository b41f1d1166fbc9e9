// nvfp4_b200_step.hpp -- the training-step projection set of a GPT-2 shaped model, driven from C++.
//
// The caller side of the C ABI: what crates/gpt2-nvfp4 does around the kernels of crates/cuda-kernels --
// own the buffers, quantize the weights, walk the linears forward (types/l2_attention/forward.rs:12-192,
// types/l3_mlp/forward.rs:7-130, types/model/final_logits.rs:33-68) and backward (backward/linear.rs:54-98,
// backward/mlp/run.rs:34-80, backward/attention/{output_projection.rs:21-39,qkv_projection.rs:25-43},
// backward/final_head/run.rs:38-55, backward/linear_scratch.rs:10-76), hand out the MS-EDEN seeds
// (random.rs:1-27) -- restricted to the projections, and extended by what the reference does not have:
// token sharding over the GPUs of one node, one process (or host thread) per GPU, with one NCCL all-reduce
// of every layer's dW / dbias bucket per step, issued on a communication stream as soon as the layer's
// backward has been enqueued.  No PyTorch anywhere: CUDA runtime for memory, streams and events, the C ABI
// of nvfp4_b200.h for every kernel, NCCL (loaded at run time, only when a communicator is attached) for the
// one collective.
//
// The attention core, LayerNorm, loss and optimizer are outside this path; their outputs (the activation of
// every input width, the upstream gradient of every output width) and the bf16 master weights are
// caller-provided device buffers.
#ifndef NVFP4_B200_STEP_HPP_
#define NVFP4_B200_STEP_HPP_

#include <cuda_runtime.h>
#include <dlfcn.h>

#include <cstdint>
#include <cstring>
#include <map>
#include <memory>
#include <string>
#include <utility>
#include <vector>

#include "nvfp4_b200.hpp"

namespace nvfp4_b200 {

// splitmix64 stream handing out the (sign, scale) seeds of each linear backward
// (crates/gpt2-nvfp4/src/random.rs:1-27).
class SeedStream {
 public:
  explicit SeedStream(uint64_t seed) : state_(seed) {}
  uint64_t next_u64() {
    state_ += 0x9E3779B97F4A7C15ull;
    uint64_t z = state_;
    z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ull;
    z = (z ^ (z >> 27)) * 0x94D049BB133111EBull;
    return z ^ (z >> 31);
  }
  uint32_t next_u32() { return static_cast<uint32_t>(next_u64() & 0xffffffffu); }

 private:
  uint64_t state_;
};

// NCCL through dlopen: a single-GPU user needs no NCCL at all, and a process that already holds a copy of
// the library (for instance one loaded by another framework) shares it.
class NcclApi {
 public:
  struct UniqueId {
    char bytes[128];
  };
  static NcclApi* get(std::string* error) {
    static NcclApi api;
    if (!api.handle_) {
      for (const char* name : {"libnccl.so.2", "libnccl.so"}) {
        api.handle_ = dlopen(name, RTLD_NOW | RTLD_GLOBAL);
        if (api.handle_) break;
      }
      if (!api.handle_) {
        if (error) *error = "libnccl.so.2 could not be loaded";
        return nullptr;
      }
      api.get_unique_id = reinterpret_cast<int (*)(UniqueId*)>(dlsym(api.handle_, "ncclGetUniqueId"));
      api.comm_init_rank = reinterpret_cast<int (*)(void**, int, UniqueId, int)>(dlsym(api.handle_, "ncclCommInitRank"));
      api.all_reduce = reinterpret_cast<int (*)(const void*, void*, size_t, int, int, void*, cudaStream_t)>(
          dlsym(api.handle_, "ncclAllReduce"));
      api.comm_destroy = reinterpret_cast<int (*)(void*)>(dlsym(api.handle_, "ncclCommDestroy"));
      api.error_string = reinterpret_cast<const char* (*)(int)>(dlsym(api.handle_, "ncclGetErrorString"));
      if (!api.get_unique_id || !api.comm_init_rank || !api.all_reduce || !api.comm_destroy) {
        if (error) *error = "libnccl.so.2 lacks a required symbol";
        return nullptr;
      }
    }
    return &api;
  }
  int (*get_unique_id)(UniqueId*) = nullptr;
  int (*comm_init_rank)(void**, int, UniqueId, int) = nullptr;
  int (*all_reduce)(const void*, void*, size_t, int, int, void*, cudaStream_t) = nullptr;
  int (*comm_destroy)(void*) = nullptr;
  const char* (*error_string)(int) = nullptr;
  static constexpr int kFloat32 = 7, kSum = 0, kMax = 2;  // ncclDataType_t / ncclRedOp_t values of nccl.h

 private:
  void* handle_ = nullptr;
};

// Owning device allocation (the kernel library itself never allocates).
class DeviceBlock {
 public:
  DeviceBlock() = default;
  explicit DeviceBlock(size_t bytes) : bytes_(bytes) {
    if (cudaMalloc(&ptr_, bytes ? bytes : 1) != cudaSuccess) ptr_ = nullptr;
  }
  DeviceBlock(const DeviceBlock&) = delete;
  DeviceBlock& operator=(const DeviceBlock&) = delete;
  DeviceBlock(DeviceBlock&& o) noexcept : ptr_(o.ptr_), bytes_(o.bytes_) { o.ptr_ = nullptr; }
  DeviceBlock& operator=(DeviceBlock&& o) noexcept {
    if (this != &o) {
      release();
      ptr_ = o.ptr_, bytes_ = o.bytes_, o.ptr_ = nullptr;
    }
    return *this;
  }
  ~DeviceBlock() { release(); }
  bool ok() const { return ptr_ != nullptr; }
  size_t bytes() const { return bytes_; }
  template <typename T>
  DeviceBuffer<T> as() const {
    return {static_cast<T*>(ptr_), bytes_ / sizeof(T)};
  }

 private:
  void release() {
    if (ptr_) cudaFree(ptr_);
    ptr_ = nullptr;
  }
  void* ptr_ = nullptr;
  size_t bytes_ = 0;
};

struct StepShape {
  uint32_t n_layer = 12, d_model = 768, d_mlp = 3072, vocab = 32000;
  uint64_t macs_per_token() const {
    const uint64_t d = d_model, h = d_mlp;
    return n_layer * (d * 3 * d + d * d + d * h + h * d) + d * static_cast<uint64_t>(vocab);
  }
};

struct StepOptions {
  uint32_t tokens = 0;        // rows of X / dY this rank holds (multiple of 128)
  uint32_t token_offset = 0;  // first token of this rank's shard
  uint32_t total_tokens = 0;  // tokens of the whole batch (0 = tokens)
  uint64_t seed = 1234;       // MS-EDEN seed stream
  bool fused_mlp = true;      // fc stores only its pre-activation; relu^2 is applied on load by the next quantizer
  bool reproducible_sharding = false;  // all-reduce(max) every amax that feeds a per-tensor scale (one collective per step)
};

// Caller-provided device tensors.  Linear index: layer * 4 + {0 c_attn, 1 attn c_proj, 2 mlp fc, 3 mlp proj};
// the LM head is index 4 * n_layer (no bias).  Widths: activations d_model and d_mlp; gradients 3 d_model,
// d_model, d_mlp, vocab.
struct StepInputs {
  std::vector<const uint16_t*> weight;  // bf16 [out][in] per linear
  std::vector<const float*> bias;       // f32 [out] per linear (nullptr for the LM head)
  std::map<uint32_t, const uint16_t*> x;   // bf16 [tokens][width] per input width
  std::map<uint32_t, const uint16_t*> dy;  // bf16 [tokens][width] per output width
};

class ProjectionStep {
 public:
  struct Linear {
    uint32_t in = 0, out = 0;
    int epilogue = NVFP4_EPI_BIAS;
    bool is_fc = false, is_proj = false;
    const uint16_t* weight = nullptr;
    const float* bias = nullptr;
    Nvfp4TensorView wq, xq;
    DeviceBuffer<float> w_amax, w_chunk, dweight, dbias;
    MsEdenOperandBuffers weight_t_h;      // W^T of this step, quantized early on the weight stream
    cudaEvent_t wq_ready = nullptr, wt_ready = nullptr;
    uint32_t sign_seed = 0, scale_seed = 0;  // this step's MS-EDEN seeds
    uint32_t bucket = 0;
  };

  ProjectionStep(const StepShape& shape, const StepOptions& opt, const StepInputs& in) : shape_(shape), opt_(opt), rng_(opt.seed) {
    build(in);
  }
  ~ProjectionStep() {
    if (comm_ && nccl_) nccl_->comm_destroy(comm_);
    for (auto& l : linears_) {
      if (l.wq_ready) cudaEventDestroy(l.wq_ready);
      if (l.wt_ready) cudaEventDestroy(l.wt_ready);
    }
    for (cudaEvent_t e : {fork_, join_, weights_free_, layer_done_, comm_done_})
      if (e) cudaEventDestroy(e);
    for (cudaStream_t s : {weight_stream_, side_stream_, comm_stream_})
      if (s) cudaStreamDestroy(s);
  }
  ProjectionStep(const ProjectionStep&) = delete;
  ProjectionStep& operator=(const ProjectionStep&) = delete;

  const std::string& error() const { return error_; }
  bool ok() const { return error_.empty(); }
  uint64_t flops_per_step() const { return 6ull * shape_.macs_per_token() * opt_.tokens; }
  size_t bucket_count() const { return buckets_.size(); }
  DeviceBuffer<float> bucket(size_t i) const { return buckets_[i].as<float>(); }
  DeviceBuffer<uint16_t> dx(uint32_t width) const { return dx_.at(width).as<uint16_t>(); }
  DeviceBuffer<uint16_t> y(uint32_t width) const { return y_.at(width).as<uint16_t>(); }
  const std::vector<Linear>& linears() const { return linears_; }
  // Replaces the activation / gradient inputs (for callers that double-buffer their inputs).
  void set_inputs(const std::map<uint32_t, const uint16_t*>& x, const std::map<uint32_t, const uint16_t*>& dy) {
    x_ = x;
    dy_ = dy;
  }

  static DriverError nccl_unique_id(NcclApi::UniqueId* id) {
    std::string err;
    NcclApi* api = NcclApi::get(&err);
    if (!api) return DriverError{static_cast<int>(cudaErrorNotSupported), err};
    const int rc = api->get_unique_id(id);
    return rc == 0 ? DriverError{} : DriverError{static_cast<int>(cudaErrorUnknown), "ncclGetUniqueId failed"};
  }
  // Joins the communicator of this step's ranks (collective: every rank calls it with the same id).
  DriverError attach_nccl(const NcclApi::UniqueId& id, int rank, int world) {
    std::string err;
    nccl_ = NcclApi::get(&err);
    if (!nccl_) return DriverError{static_cast<int>(cudaErrorNotSupported), err};
    const int rc = nccl_->comm_init_rank(&comm_, world, id, rank);
    if (rc != 0) {
      comm_ = nullptr;
      return DriverError{static_cast<int>(cudaErrorUnknown),
                         std::string("ncclCommInitRank: ") + (nccl_->error_string ? nccl_->error_string(rc) : "failed")};
    }
    world_ = world;
    return {};
  }

  // One forward + backward pass over this rank's tokens, enqueued on `s`; returns without synchronising.
  DriverError step(cudaStream_t s, bool weights_changed = true) {
    if (!ok()) return DriverError{static_cast<int>(cudaErrorInvalidValue), error_};
    // this step's seeds, in the order the backward pass uses them (the forward pass draws none)
    for (size_t i : backward_order()) {
      linears_[i].sign_seed = rng_.next_u32();
      linears_[i].scale_seed = rng_.next_u32();
    }
    if (auto e = weight_side(s, weights_changed || !weights_quantized_)) return e;
    weights_quantized_ = true;
    for (auto& l : linears_)
      if (auto e = forward(s, l)) return e;
    return backward(s);
  }

 private:
  static DriverError cuda(cudaError_t e, const char* what) {
    if (e == cudaSuccess) return {};
    return DriverError{static_cast<int>(e), std::string(what) + ": " + cudaGetErrorString(e)};
  }
  DeviceBlock& alloc(size_t bytes) {
    blocks_.emplace_back(bytes);
    if (!blocks_.back().ok() && error_.empty()) error_ = "cudaMalloc failed";
    return blocks_.back();
  }
  Nvfp4TensorView alloc_tensor(uint32_t rows, uint32_t cols, bool rowwise, bool decoded) {
    Nvfp4TensorView t;
    t.rows = rows, t.cols = cols, t.rowwise = rowwise, t.scale_layout = NVFP4_SCALES_PACKED;
    t.bytes = alloc(Nvfp4TensorView::bytes_len(rows, cols)).as<uint8_t>();
    t.scales = alloc(scale_packed_len(rows, cols)).as<uint8_t>();
    t.global_scales = alloc(sizeof(float) * (rowwise ? rows : 1)).as<float>();
    if (decoded) t.decoded_amax = alloc(sizeof(float)).as<float>();
    return t;
  }
  MsEdenOperandBuffers alloc_operand(const MsEdenOperandSizes& n) {
    MsEdenOperandBuffers b;
    b.bytes = alloc(n.bytes).as<uint8_t>();
    b.scales_packed = alloc(n.scales_packed).as<uint8_t>();
    b.global_scales = alloc(n.global_scales * sizeof(float)).as<float>();
    b.global_scale = alloc(n.global_scale * sizeof(float)).as<float>();
    b.chunk_amax = alloc(n.chunk_amax * sizeof(float)).as<float>();
    return b;
  }

  void build(const StepInputs& in) {
    const uint32_t T = opt_.tokens, d = shape_.d_model, h = shape_.d_mlp, v = shape_.vocab;
    if (T == 0 || T % 128 != 0) {
      error_ = "token shards are multiples of 128 rows";
      return;
    }
    const size_t n_lin = 4ull * shape_.n_layer + 1;
    if (in.weight.size() != n_lin || in.bias.size() != n_lin) {
      error_ = "StepInputs: one weight and one bias entry per linear";
      return;
    }
    x_ = in.x;
    dy_ = in.dy;
    struct Kind {
      uint32_t in, out;
      int epi;
    };
    const Kind kinds[4] = {{d, 3 * d, NVFP4_EPI_BIAS}, {d, d, NVFP4_EPI_BIAS}, {d, h, NVFP4_EPI_RELU2}, {h, d, NVFP4_EPI_BIAS}};
    linears_.resize(n_lin);
    for (size_t i = 0; i < n_lin; ++i) {
      Linear& l = linears_[i];
      const bool head = i + 1 == n_lin;
      const Kind k = head ? Kind{d, v, NVFP4_EPI_NONE} : kinds[i % 4];
      l.in = k.in, l.out = k.out, l.epilogue = k.epi;
      l.is_fc = !head && i % 4 == 2, l.is_proj = !head && i % 4 == 3;
      l.weight = in.weight[i], l.bias = in.bias[i];
      l.bucket = head ? shape_.n_layer : static_cast<uint32_t>(i / 4);
      l.wq = alloc_tensor(l.out, l.in, false, false);
      l.xq = alloc_tensor(T, l.in, true, true);
      l.w_amax = alloc(sizeof(float)).as<float>();
      l.w_chunk = alloc(sizeof(float) * ((static_cast<size_t>(l.out) * l.in + 1023) / 1024)).as<float>();
      l.weight_t_h = alloc_operand(LinearBackwardMsEdenScratchSizes(T, l.in, l.out).weight_t_h);
      if (cudaEventCreateWithFlags(&l.wq_ready, cudaEventDisableTiming) != cudaSuccess ||
          cudaEventCreateWithFlags(&l.wt_ready, cudaEventDisableTiming) != cudaSuccess)
        error_ = "cudaEventCreate failed";
      if (!x_.count(l.in) || !dy_.count(l.out)) error_ = "StepInputs: an activation / gradient width is missing";
    }
    // gradient buckets: dW (+ dbias) of a layer's four linears in one flat f32 buffer, the LM head in its own
    for (uint32_t b = 0; b <= shape_.n_layer; ++b) {
      size_t floats = 0;
      for (auto& l : linears_)
        if (l.bucket == b) floats += static_cast<size_t>(l.out) * l.in + (l.bias ? l.out : 0);
      buckets_.emplace_back(floats * sizeof(float));
      if (!buckets_.back().ok()) error_ = "cudaMalloc failed";
      float* base = buckets_.back().as<float>().ptr;
      size_t off = 0;
      for (auto& l : linears_) {
        if (l.bucket != b) continue;
        l.dweight = {base + off, static_cast<size_t>(l.out) * l.in};
        off += l.dweight.len;
        if (l.bias) {
          l.dbias = {base + off, l.out};
          off += l.out;
        }
      }
    }
    for (auto& l : linears_) {
      const auto key = std::make_pair(l.in, l.out);
      if (!scratch_.count(key)) {
        const LinearBackwardMsEdenScratchSizes n(T, l.in, l.out);
        LinearBackwardMsEdenScratchBuffers sb;
        sb.e_h = alloc_operand(n.e_h), sb.e_t_h = alloc_operand(n.e_t_h);
        sb.weight_t_h = alloc_operand(n.weight_t_h), sb.input_t_h = alloc_operand(n.input_t_h);
        scratch_[key] = sb;
      }
      if (!y_.count(l.out)) y_.emplace(l.out, DeviceBlock(static_cast<size_t>(T) * l.out * 2));
      if (!dx_.count(l.in)) dx_.emplace(l.in, DeviceBlock(static_cast<size_t>(T) * l.in * 2));
    }
    pre_ = DeviceBlock(static_cast<size_t>(T) * h * 2);
    pre_row_amax_ = DeviceBlock(static_cast<size_t>(T) * sizeof(float));
    amax_vec_ = DeviceBlock(2 * n_lin * sizeof(float));
    e_scales_ = DeviceBlock(n_lin * sizeof(float));
    bool streams = cudaStreamCreateWithFlags(&weight_stream_, cudaStreamNonBlocking) == cudaSuccess &&
                   cudaStreamCreateWithFlags(&side_stream_, cudaStreamNonBlocking) == cudaSuccess &&
                   cudaStreamCreateWithFlags(&comm_stream_, cudaStreamNonBlocking) == cudaSuccess;
    for (cudaEvent_t* e : {&fork_, &join_, &weights_free_, &layer_done_, &comm_done_})
      streams = streams && cudaEventCreateWithFlags(e, cudaEventDisableTiming) == cudaSuccess;
    if (!streams && error_.empty()) error_ = "could not create the step's streams / events";
    if (!pre_.ok() || !pre_row_amax_.ok() || !amax_vec_.ok() || !e_scales_.ok()) error_ = "cudaMalloc failed";
  }

  // The weight side of a step, on its own stream beside the forward pass: (when the masters changed) four-six of
  // every weight in the order the forward pass needs them -- each forward GEMM waits for its own weight's event
  // -- and then, always, the MS-EDEN form of every W^T with this step's seeds in the order the backward pass
  // needs them.  This work is replicated on every rank of a token-sharded step; here it is off the critical path.
  DriverError weight_side(cudaStream_t s, bool requantize) {
    if (auto e = cuda(cudaEventRecord(weights_free_, s), "event record")) return e;  // the previous step is done with the old operands
    if (auto e = cuda(cudaStreamWaitEvent(weight_stream_, weights_free_, 0), "stream wait")) return e;
    if (requantize) {
      for (auto& l : linears_) {
        const DeviceBuffer<const uint16_t> w{l.weight, static_cast<size_t>(l.out) * l.in};
        if (auto e = quant_.tensor_amax<uint16_t>(weight_stream_, w, l.w_chunk, l.w_amax)) return e;
        if (auto e = quant_.quantize_four_six<uint16_t>(weight_stream_, w, l.w_amax, l.wq)) return e;
        if (auto e = cuda(cudaEventRecord(l.wq_ready, weight_stream_), "event record")) return e;
      }
    }
    for (size_t i : backward_order()) {
      Linear& l = linears_[i];
      if (auto e = backward_.prepare_weight_t<uint16_t>(weight_stream_, backward_args(l, 0))) return e;
      if (auto e = cuda(cudaEventRecord(l.wt_ready, weight_stream_), "event record")) return e;
    }
    return {};
  }

  // The arguments of one linear's backward call (`index` = its position in the backward order).
  LinearBackwardMsEdenArgs<uint16_t> backward_args(Linear& l, size_t index) {
    LinearBackwardMsEdenArgs<uint16_t> a;
    a.e = {dy_.at(l.out), static_cast<size_t>(opt_.tokens) * l.out};
    a.weight = l.wq, a.input = l.xq;
    a.scratch = scratch_.at({l.in, l.out});
    a.scratch.weight_t_h = l.weight_t_h;
    a.weight_t_prepared = true;
    a.dinput = dx_.at(l.in).as<uint16_t>();
    a.dweight = l.dweight, a.dbias = l.dbias;
    a.token_count = opt_.tokens, a.input_dim = l.in, a.output_dim = l.out;
    a.sign_seed = l.sign_seed, a.scale_seed = l.scale_seed;
    a.token_offset = opt_.token_offset;
    a.side_stream = side_stream_, a.fork_event = fork_, a.join_event = join_;
    if (opt_.reproducible_sharding) {
      const size_t n = linears_.size();
      a.total_token_count = opt_.total_tokens ? opt_.total_tokens : opt_.tokens;
      a.e_global_scale_override = {e_scales_.as<float>().ptr + index, 1};
      a.x_decoded_amax = {amax_vec_.as<float>().ptr + n + index, 1};
    }
    return a;
  }

  DriverError forward(cudaStream_t s, Linear& l) {
    const uint32_t T = opt_.tokens;
    if (opt_.fused_mlp && l.is_proj) {
      // the MLP activation relu(pre)^2 is computed on load from the fc projection's pre-activation; its row
      // amax came out of that GEMM's epilogue
      if (auto e = quant_.quantize_relu2<uint16_t>(s, pre_.as<const uint16_t>(), pre_row_amax_.as<const float>(), l.xq)) return e;
    } else {
      const DeviceBuffer<const uint16_t> x{x_.at(l.in), static_cast<size_t>(T) * l.in};
      if (auto e = quant_.quantize_row_amax<uint16_t>(s, x, l.xq)) return e;
    }
    if (auto e = cuda(cudaStreamWaitEvent(s, l.wq_ready, 0), "stream wait")) return e;
    const DeviceBuffer<const float> bias{l.bias, l.bias ? l.out : 0};
    if (opt_.fused_mlp && l.is_fc)
      return gemm_.gemm<uint16_t>(s, l.xq, l.wq, pre_.as<uint16_t>(), Epilogue::Bias, bias, {}, pre_row_amax_.as<float>());
    const DeviceBuffer<uint16_t> aux = l.is_fc ? pre_.as<uint16_t>() : DeviceBuffer<uint16_t>{};
    return gemm_.gemm<uint16_t>(s, l.xq, l.wq, y_.at(l.out).as<uint16_t>(), static_cast<Epilogue>(l.epilogue), bias, aux);
  }

  std::vector<size_t> backward_order() const {
    std::vector<size_t> order{linears_.size() - 1};
    for (uint32_t layer = shape_.n_layer; layer-- > 0;)
      for (int j = 3; j >= 0; --j) order.push_back(layer * 4 + j);
    return order;
  }

  // Reproducible sharding: the amax of every dY and of every decoded X of this step as ONE f32 vector,
  // all-reduced (max) over the ranks; the dY scales are derived from the reduced values.
  DriverError sync_scales(cudaStream_t s, const std::vector<size_t>& order) {
    const size_t n = order.size();
    float* vec = amax_vec_.as<float>().ptr;
    for (size_t i = 0; i < n; ++i) {
      const Linear& l = linears_[order[i]];
      const DeviceBuffer<const uint16_t> e{dy_.at(l.out), static_cast<size_t>(opt_.tokens) * l.out};
      auto& sc = scratch_.at({l.in, l.out});
      if (auto err = quant_.tensor_amax<uint16_t>(s, e, sc.e_h.chunk_amax, {vec + i, 1})) return err;
      if (auto err = cuda(cudaMemcpyAsync(vec + n + i, l.xq.decoded_amax.ptr, sizeof(float), cudaMemcpyDeviceToDevice, s), "copy"))
        return err;
    }
    if (comm_) {
      const int rc = nccl_->all_reduce(vec, vec, 2 * n, NcclApi::kFloat32, NcclApi::kMax, comm_, s);
      if (rc != 0) return DriverError{static_cast<int>(cudaErrorUnknown), "ncclAllReduce(max) failed"};
    }
    for (size_t i = 0; i < n; ++i)
      if (int rc = nvfp4_quartet_backward_ms_eden_global_scale_from_chunks(s, vec + i, e_scales_.as<float>().ptr + i, 1))
        return detail::from_rc(rc);
    return {};
  }

  DriverError backward(cudaStream_t s) {
    const std::vector<size_t> order = backward_order();
    if (opt_.reproducible_sharding)
      if (auto e = sync_scales(s, order)) return e;
    const size_t n = order.size();
    bool reduced_any = false;
    for (size_t i = 0; i < n; ++i) {
      Linear& l = linears_[order[i]];
      if (auto e = cuda(cudaStreamWaitEvent(s, l.wt_ready, 0), "stream wait")) return e;
      if (auto e = backward_.backward_ms_eden<uint16_t>(s, backward_args(l, i))) return e;
      // last linear of its bucket: the bucket is complete, its all-reduce goes to the communication stream
      const bool bucket_done = i + 1 == n || linears_[order[i + 1]].bucket != l.bucket;
      if (bucket_done && comm_) {
        if (auto e = cuda(cudaEventRecord(layer_done_, s), "event record")) return e;
        if (auto e = cuda(cudaStreamWaitEvent(comm_stream_, layer_done_, 0), "stream wait")) return e;
        const DeviceBuffer<float> b = buckets_[l.bucket].as<float>();
        const int rc = nccl_->all_reduce(b.ptr, b.ptr, b.len, NcclApi::kFloat32, NcclApi::kSum, comm_, comm_stream_);
        if (rc != 0) return DriverError{static_cast<int>(cudaErrorUnknown), "ncclAllReduce failed"};
        reduced_any = true;
      }
    }
    if (reduced_any) {
      if (auto e = cuda(cudaEventRecord(comm_done_, comm_stream_), "event record")) return e;
      if (auto e = cuda(cudaStreamWaitEvent(s, comm_done_, 0), "stream wait")) return e;
    }
    return {};
  }

  StepShape shape_;
  StepOptions opt_;
  SeedStream rng_;
  std::string error_;
  std::vector<Linear> linears_;
  std::vector<DeviceBlock> blocks_, buckets_;
  std::map<std::pair<uint32_t, uint32_t>, LinearBackwardMsEdenScratchBuffers> scratch_;
  std::map<uint32_t, DeviceBlock> y_, dx_;
  std::map<uint32_t, const uint16_t*> x_, dy_;
  DeviceBlock pre_, pre_row_amax_, amax_vec_, e_scales_;
  cudaStream_t weight_stream_ = nullptr, side_stream_ = nullptr, comm_stream_ = nullptr;
  cudaEvent_t fork_ = nullptr, join_ = nullptr, weights_free_ = nullptr, layer_done_ = nullptr, comm_done_ = nullptr;
  bool weights_quantized_ = false;
  Nvfp4QuantModule quant_;
  Nvfp4GemmModule gemm_;
  LinearBackwardModule backward_;
  NcclApi* nccl_ = nullptr;
  void* comm_ = nullptr;
  int world_ = 1;
};

}  // namespace nvfp4_b200

#endif  // NVFP4_B200_STEP_HPP_
