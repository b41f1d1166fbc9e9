// C ABI over the C++ training-step driver of include/nvfp4_b200_step.hpp (see include/nvfp4_b200_step.h).
#include "nvfp4_b200_step.h"

#include <cstring>
#include <stdexcept>
#include <string>

#include "nvfp4_b200_step.hpp"

using namespace nvfp4_b200;

namespace {
thread_local std::string g_create_error;
struct Handle {
  std::unique_ptr<ProjectionStep> step;
  std::string last_error;
};
int fail(Handle* h, const DriverError& e) {
  h->last_error = e.message;
  return e.code ? e.code : 1;
}
void fill(std::map<uint32_t, const uint16_t*>& m, const uint32_t* widths, const void* const* ptrs, uint32_t n) {
  for (uint32_t i = 0; i < n; ++i) m[widths[i]] = static_cast<const uint16_t*>(ptrs[i]);
}
}  // namespace

extern "C" {

void* nvfp4_step_create(const nvfp4_step_config* cfg, const void* const* weights, const void* const* biases,
                        uint32_t n_linears, const uint32_t* x_widths, const void* const* x_ptrs, uint32_t n_x,
                        const uint32_t* dy_widths, const void* const* dy_ptrs, uint32_t n_dy) {
  if (!cfg || !weights || !biases) {
    g_create_error = "nvfp4_step_create: null argument";
    return nullptr;
  }
  StepShape shape;
  shape.n_layer = cfg->n_layer, shape.d_model = cfg->d_model, shape.d_mlp = cfg->d_mlp, shape.vocab = cfg->vocab;
  StepOptions opt;
  opt.tokens = cfg->tokens, opt.token_offset = cfg->token_offset, opt.total_tokens = cfg->total_tokens;
  opt.seed = cfg->seed, opt.fused_mlp = cfg->fused_mlp != 0, opt.reproducible_sharding = cfg->reproducible_sharding != 0;
  StepInputs in;
  for (uint32_t i = 0; i < n_linears; ++i) {
    in.weight.push_back(static_cast<const uint16_t*>(weights[i]));
    in.bias.push_back(static_cast<const float*>(biases[i]));
  }
  fill(in.x, x_widths, x_ptrs, n_x);
  fill(in.dy, dy_widths, dy_ptrs, n_dy);
  auto h = std::make_unique<Handle>();
  h->step = std::make_unique<ProjectionStep>(shape, opt, in);
  if (!h->step->ok()) {
    g_create_error = h->step->error();
    return nullptr;
  }
  return h.release();
}

void nvfp4_step_destroy(void* handle) { delete static_cast<Handle*>(handle); }

const char* nvfp4_step_error(void* handle) {
  return handle ? static_cast<Handle*>(handle)->last_error.c_str() : g_create_error.c_str();
}

int nvfp4_step_run(void* handle, void* stream, int weights_changed) {
  Handle* h = static_cast<Handle*>(handle);
  if (!h) return 1;
  const DriverError e = h->step->step(static_cast<cudaStream_t>(stream), weights_changed != 0);
  return e.ok() ? 0 : fail(h, e);
}

int nvfp4_step_set_inputs(void* handle, const uint32_t* x_widths, const void* const* x_ptrs, uint32_t n_x,
                          const uint32_t* dy_widths, const void* const* dy_ptrs, uint32_t n_dy) {
  Handle* h = static_cast<Handle*>(handle);
  if (!h) return 1;
  std::map<uint32_t, const uint16_t*> x, dy;
  fill(x, x_widths, x_ptrs, n_x);
  fill(dy, dy_widths, dy_ptrs, n_dy);
  h->step->set_inputs(x, dy);
  return 0;
}

int nvfp4_step_bucket(void* handle, uint32_t index, float** ptr, uint64_t* len) {
  Handle* h = static_cast<Handle*>(handle);
  if (!h || index >= h->step->bucket_count() || !ptr || !len) return 1;
  const DeviceBuffer<float> b = h->step->bucket(index);
  *ptr = b.ptr;
  *len = b.len;
  return 0;
}

int nvfp4_step_dx(void* handle, uint32_t width, void** ptr) {
  Handle* h = static_cast<Handle*>(handle);
  if (!h || !ptr) return 1;
  try {
    *ptr = h->step->dx(width).ptr;
  } catch (const std::out_of_range&) {
    return 1;
  }
  return 0;
}

int nvfp4_step_y(void* handle, uint32_t width, void** ptr) {
  Handle* h = static_cast<Handle*>(handle);
  if (!h || !ptr) return 1;
  try {
    *ptr = h->step->y(width).ptr;
  } catch (const std::out_of_range&) {
    return 1;
  }
  return 0;
}

uint64_t nvfp4_step_flops(void* handle) {
  Handle* h = static_cast<Handle*>(handle);
  return h ? h->step->flops_per_step() : 0;
}

int nvfp4_step_nccl_unique_id(uint8_t* id128) {
  if (!id128) return 1;
  NcclApi::UniqueId id;
  const DriverError e = ProjectionStep::nccl_unique_id(&id);
  if (!e.ok()) {
    g_create_error = e.message;
    return e.code ? e.code : 1;
  }
  std::memcpy(id128, id.bytes, sizeof(id.bytes));
  return 0;
}

int nvfp4_step_attach_nccl(void* handle, const uint8_t* id128, int rank, int world) {
  Handle* h = static_cast<Handle*>(handle);
  if (!h || !id128) return 1;
  NcclApi::UniqueId id;
  std::memcpy(id.bytes, id128, sizeof(id.bytes));
  const DriverError e = h->step->attach_nccl(id, rank, world);
  return e.ok() ? 0 : fail(h, e);
}

}  // extern "C"
