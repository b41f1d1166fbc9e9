// Reader and writer of the NVFP4 checkpoint container: a flat little-endian file of (bytes, scales,
// global_scale) triples, the interchange format of every quantized tensor on the projection path.
//
// Layout (src/checkpoint/format.rs:7-8, format/writer.rs:15-38, format/reader.rs:22-67 of the reference):
//   magic "GPT2_NVFP4_CHECKPOINT\n" | u32 version = 2 | u32 tensor_count
//   per tensor: u32 name_len | u64 len (elements) | u64 byte_len | u64 scale_len | f32 global_scale |
//               name (UTF-8, no terminator) | bytes | scales
// A tensor read back for the device must hold len / 2 nibble bytes and len / 16 scale bytes
// (src/checkpoint/load/tensor.rs:27-39).  The device variants stage through pinned host memory exactly as
// the reference's save/tensor.rs:14-20 and load/tensor.rs:17-23 copy each member through the host.
#include <cstdio>
#include <cstring>
#include <string>
#include <vector>

#include "kernels.h"

namespace nvfp4 {
namespace {

constexpr char kMagic[] = "GPT2_NVFP4_CHECKPOINT\n";  // 22 bytes, no terminator in the file
constexpr size_t kMagicLen = sizeof(kMagic) - 1;
constexpr uint32_t kVersion = 2;

struct Checkpoint {
  FILE* file = nullptr;
  bool writing = false;
  uint32_t declared = 0;   // tensor count of the header
  uint32_t done = 0;       // tensors written / fully read so far
  // reader: the tensor whose header was read and whose payload is still in the file
  bool pending = false;
  uint64_t pending_len = 0, pending_bytes = 0, pending_scales = 0;
  float pending_global = 0.0f;
  std::string pending_name;
  // pinned staging for the device variants (grown on demand)
  void* pinned = nullptr;
  size_t pinned_size = 0;
};

int fail(const char* msg) {
  set_last_error(msg);
  return static_cast<int>(cudaErrorInvalidValue);
}

bool put(FILE* f, const void* p, size_t n) { return n == 0 || std::fwrite(p, 1, n, f) == n; }
bool get(FILE* f, void* p, size_t n) { return n == 0 || std::fread(p, 1, n, f) == n; }
bool put_u32(FILE* f, uint32_t v) {
  const uint8_t b[4] = {uint8_t(v), uint8_t(v >> 8), uint8_t(v >> 16), uint8_t(v >> 24)};
  return put(f, b, 4);
}
bool put_u64(FILE* f, uint64_t v) { return put_u32(f, uint32_t(v)) && put_u32(f, uint32_t(v >> 32)); }
bool get_u32(FILE* f, uint32_t& v) {
  uint8_t b[4];
  if (!get(f, b, 4)) return false;
  v = uint32_t(b[0]) | (uint32_t(b[1]) << 8) | (uint32_t(b[2]) << 16) | (uint32_t(b[3]) << 24);
  return true;
}
bool get_u64(FILE* f, uint64_t& v) {
  uint32_t lo, hi;
  if (!get_u32(f, lo) || !get_u32(f, hi)) return false;
  v = uint64_t(lo) | (uint64_t(hi) << 32);
  return true;
}

int ensure_pinned(Checkpoint* c, size_t bytes) {
  if (bytes <= c->pinned_size) return 0;
  if (c->pinned) cudaFreeHost(c->pinned);
  c->pinned = nullptr;
  c->pinned_size = 0;
  const cudaError_t e = cudaMallocHost(&c->pinned, bytes);
  if (e != cudaSuccess) {
    set_last_error("checkpoint: pinned staging allocation failed");
    return static_cast<int>(e);
  }
  c->pinned_size = bytes;
  return 0;
}

void destroy(Checkpoint* c) {
  if (c->file) std::fclose(c->file);
  if (c->pinned) cudaFreeHost(c->pinned);
  delete c;
}

}  // namespace
}  // namespace nvfp4

using namespace nvfp4;

extern "C" {

int nvfp4_checkpoint_writer_open(const char* path, uint32_t tensor_count, void** writer_out) {
  if (!path || !writer_out) return fail("checkpoint writer: null argument");
  FILE* f = std::fopen(path, "wb");
  if (!f) return fail("checkpoint writer: cannot create the file");
  Checkpoint* c = new Checkpoint;
  c->file = f;
  c->writing = true;
  c->declared = tensor_count;
  if (!put(f, kMagic, kMagicLen) || !put_u32(f, kVersion) || !put_u32(f, tensor_count)) {
    destroy(c);
    return fail("checkpoint writer: short write of the header");
  }
  *writer_out = c;
  return 0;
}

int nvfp4_checkpoint_write_tensor(void* writer, const char* name, uint64_t len, float global_scale, const uint8_t* bytes,
                                  uint64_t byte_len, const uint8_t* scales, uint64_t scale_len) {
  Checkpoint* c = static_cast<Checkpoint*>(writer);
  if (!c || !c->writing || !name || (byte_len && !bytes) || (scale_len && !scales))
    return fail("checkpoint writer: null argument or not a writer");
  if (c->done >= c->declared) return fail("checkpoint writer: more tensors than the header declares");
  const size_t name_len = std::strlen(name);
  uint8_t gs[4];
  std::memcpy(gs, &global_scale, 4);  // the hosts this library runs on are little-endian
  if (!put_u32(c->file, static_cast<uint32_t>(name_len)) || !put_u64(c->file, len) || !put_u64(c->file, byte_len) ||
      !put_u64(c->file, scale_len) || !put(c->file, gs, 4) || !put(c->file, name, name_len) ||
      !put(c->file, bytes, byte_len) || !put(c->file, scales, scale_len))
    return fail("checkpoint writer: short write");
  ++c->done;
  return 0;
}

int nvfp4_checkpoint_write_tensor_device(void* writer, void* stream, const char* name, uint64_t len,
                                         const float* global_scale, const uint8_t* bytes, uint64_t byte_len,
                                         const uint8_t* scales, uint64_t scale_len) {
  Checkpoint* c = static_cast<Checkpoint*>(writer);
  if (!c || !c->writing || !global_scale) return fail("checkpoint writer: null argument or not a writer");
  const size_t total = static_cast<size_t>(byte_len) + static_cast<size_t>(scale_len) + 16;
  if (int e = ensure_pinned(c, total)) return e;
  uint8_t* host = static_cast<uint8_t*>(c->pinned);
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  cudaError_t e = cudaMemcpyAsync(host, global_scale, sizeof(float), cudaMemcpyDeviceToHost, s);
  if (e == cudaSuccess && byte_len) e = cudaMemcpyAsync(host + 16, bytes, byte_len, cudaMemcpyDeviceToHost, s);
  if (e == cudaSuccess && scale_len)
    e = cudaMemcpyAsync(host + 16 + byte_len, scales, scale_len, cudaMemcpyDeviceToHost, s);
  if (e == cudaSuccess) e = cudaStreamSynchronize(s);
  if (e != cudaSuccess) {
    set_last_error("checkpoint writer: device to host copy failed");
    return static_cast<int>(e);
  }
  float gs;
  std::memcpy(&gs, host, sizeof(float));
  return nvfp4_checkpoint_write_tensor(writer, name, len, gs, host + 16, byte_len, host + 16 + byte_len, scale_len);
}

int nvfp4_checkpoint_writer_close(void* writer) {
  Checkpoint* c = static_cast<Checkpoint*>(writer);
  if (!c || !c->writing) return fail("checkpoint writer: not a writer");
  const bool complete = c->done == c->declared;
  const bool flushed = std::fflush(c->file) == 0;
  destroy(c);
  if (!flushed) return fail("checkpoint writer: flush failed");
  if (!complete) return fail("checkpoint writer: fewer tensors than the header declares");
  return 0;
}

int nvfp4_checkpoint_reader_open(const char* path, void** reader_out, uint32_t* tensor_count_out) {
  if (!path || !reader_out || !tensor_count_out) return fail("checkpoint reader: null argument");
  FILE* f = std::fopen(path, "rb");
  if (!f) return fail("checkpoint reader: cannot open the file");
  Checkpoint* c = new Checkpoint;
  c->file = f;
  char magic[kMagicLen];
  uint32_t version = 0;
  if (!get(f, magic, kMagicLen) || std::memcmp(magic, kMagic, kMagicLen) != 0) {
    destroy(c);
    return fail("invalid GPT2 NVFP4 checkpoint magic");
  }
  if (!get_u32(f, version) || version != kVersion) {
    destroy(c);
    return fail("unsupported checkpoint version");
  }
  if (!get_u32(f, c->declared)) {
    destroy(c);
    return fail("checkpoint reader: truncated header");
  }
  *tensor_count_out = c->declared;
  *reader_out = c;
  return 0;
}

int nvfp4_checkpoint_next_tensor(void* reader, nvfp4_checkpoint_tensor_info* info) {
  Checkpoint* c = static_cast<Checkpoint*>(reader);
  if (!c || c->writing || !info) return fail("checkpoint reader: null argument or not a reader");
  if (c->pending) return fail("checkpoint reader: the previous tensor's payload has not been read");
  if (c->done >= c->declared) return fail("checkpoint reader: no tensor left");
  uint32_t name_len = 0;
  uint8_t gs[4];
  if (!get_u32(c->file, name_len) || !get_u64(c->file, c->pending_len) || !get_u64(c->file, c->pending_bytes) ||
      !get_u64(c->file, c->pending_scales) || !get(c->file, gs, 4))
    return fail("checkpoint reader: truncated tensor header");
  if (name_len >= sizeof(info->name)) return fail("checkpoint reader: tensor name longer than 255 bytes");
  std::memcpy(&c->pending_global, gs, 4);
  c->pending_name.assign(name_len, '\0');
  if (!get(c->file, &c->pending_name[0], name_len)) return fail("checkpoint reader: truncated tensor name");
  c->pending = true;
  std::memset(info, 0, sizeof(*info));
  std::memcpy(info->name, c->pending_name.data(), name_len);
  info->len = c->pending_len;
  info->byte_len = c->pending_bytes;
  info->scale_len = c->pending_scales;
  info->global_scale = c->pending_global;
  return 0;
}

int nvfp4_checkpoint_read_payload(void* reader, uint8_t* bytes, uint64_t byte_capacity, uint8_t* scales,
                                  uint64_t scale_capacity) {
  Checkpoint* c = static_cast<Checkpoint*>(reader);
  if (!c || c->writing || !c->pending) return fail("checkpoint reader: no tensor header has been read");
  if (byte_capacity < c->pending_bytes || scale_capacity < c->pending_scales || (c->pending_bytes && !bytes) ||
      (c->pending_scales && !scales))
    return fail("checkpoint reader: destination smaller than the tensor");
  if (!get(c->file, bytes, c->pending_bytes) || !get(c->file, scales, c->pending_scales))
    return fail("checkpoint reader: truncated tensor payload");
  c->pending = false;
  ++c->done;
  return 0;
}

int nvfp4_checkpoint_read_payload_device(void* reader, void* stream, uint8_t* bytes, uint8_t* scales,
                                         float* global_scale) {
  Checkpoint* c = static_cast<Checkpoint*>(reader);
  if (!c || c->writing || !c->pending) return fail("checkpoint reader: no tensor header has been read");
  if (!global_scale) return fail("checkpoint reader: null global scale destination");
  // load/tensor.rs:27-39: the member lengths have to match the element count
  if (c->pending_bytes != c->pending_len / 2) return fail("checkpoint tensor: byte count is not len / 2");
  if (c->pending_scales != c->pending_len / 16) return fail("checkpoint tensor: scale count is not len / 16");
  const size_t nb = c->pending_bytes, ns = c->pending_scales;
  if (int e = ensure_pinned(c, nb + ns + 16)) return e;
  uint8_t* host = static_cast<uint8_t*>(c->pinned);
  std::memcpy(host, &c->pending_global, sizeof(float));
  if (int e = nvfp4_checkpoint_read_payload(reader, host + 16, nb, host + 16 + nb, ns)) return e;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  cudaError_t e = cudaMemcpyAsync(global_scale, host, sizeof(float), cudaMemcpyHostToDevice, s);
  if (e == cudaSuccess && nb) e = cudaMemcpyAsync(bytes, host + 16, nb, cudaMemcpyHostToDevice, s);
  if (e == cudaSuccess && ns) e = cudaMemcpyAsync(scales, host + 16 + nb, ns, cudaMemcpyHostToDevice, s);
  if (e == cudaSuccess) e = cudaStreamSynchronize(s);  // the staging buffer is reused by the next tensor
  if (e != cudaSuccess) {
    set_last_error("checkpoint reader: host to device copy failed");
    return static_cast<int>(e);
  }
  return 0;
}

int nvfp4_checkpoint_reader_close(void* reader) {
  Checkpoint* c = static_cast<Checkpoint*>(reader);
  if (!c || c->writing) return fail("checkpoint reader: not a reader");
  destroy(c);
  return 0;
}

}  // extern "C"
