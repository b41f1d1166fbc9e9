// One MLP block, forward and backward, driven from C++ through include/nvfp4_b200.hpp in the order the
// reference's model crate calls its kernels (forward: crates/gpt2-nvfp4/src/types/l3_mlp/forward.rs:15-130,
// backward: crates/gpt2-nvfp4/src/backward/mlp/run.rs:30-90): quantize X with its row amax, fc projection
// with the ReLU^2 epilogue, quantize the hidden activation, down projection with bias; then the linear
// backward of the down projection, the ReLU^2 backward (which hands its amax to the next step) and the
// linear backward of fc.  f32 in, f32 out: the reference's own I/O types.
//
//   mlp_layer_driver <input file> <output file>
//
// input : 8 x u32 {magic 0x4d4c5031, tokens, d_model, d_mlp, sign_seed_proj, scale_seed_proj, sign_seed_fc,
//         scale_seed_fc}, then f32 x[T][d], w_fc[h][d], b_fc[h], w_proj[d][h], b_proj[d], dy[T][d]
// output: f32 y[T][d], dx[T][d], dw_fc[h][d], db_fc[h], dw_proj[d][h], db_proj[d], then
//         u32 {relu2 chunk count, device status word}
// Exit code 0 on success; any failing call prints its DriverError and exits 1.
#include <cuda_runtime.h>

#include <cstdint>
#include <cstdio>
#include <cstdlib>
#include <vector>

#include "nvfp4_b200.hpp"

using namespace nvfp4_b200;

namespace {

[[noreturn]] void die(const char* what, const char* detail) {
  std::fprintf(stderr, "mlp_layer_driver: %s: %s\n", what, detail);
  std::exit(1);
}
void cuda_ok(cudaError_t e, const char* what) {
  if (e != cudaSuccess) die(what, cudaGetErrorString(e));
}
void ok(const DriverError& e, const char* what) {
  if (!e.ok()) die(what, e.message.c_str());
}

// Owning device allocation; the library itself never allocates.
template <typename T>
class DeviceVec {
 public:
  explicit DeviceVec(size_t n) : n_(n) { cuda_ok(cudaMalloc(&p_, (n ? n : 1) * sizeof(T)), "cudaMalloc"); }
  DeviceVec(const DeviceVec&) = delete;
  DeviceVec& operator=(const DeviceVec&) = delete;
  DeviceVec(DeviceVec&& o) noexcept : p_(o.p_), n_(o.n_) { o.p_ = nullptr; }
  ~DeviceVec() { if (p_) cudaFree(p_); }
  DeviceBuffer<T> buf() const { return {static_cast<T*>(p_), n_}; }
  DeviceBuffer<const T> cbuf() const { return {static_cast<const T*>(p_), n_}; }
  void upload(const std::vector<T>& h, cudaStream_t s) {
    cuda_ok(cudaMemcpyAsync(p_, h.data(), h.size() * sizeof(T), cudaMemcpyHostToDevice, s), "upload");
  }
  std::vector<T> download(cudaStream_t s) const {
    std::vector<T> h(n_);
    cuda_ok(cudaMemcpyAsync(h.data(), p_, n_ * sizeof(T), cudaMemcpyDeviceToHost, s), "download");
    cuda_ok(cudaStreamSynchronize(s), "sync");
    return h;
  }

 private:
  void* p_ = nullptr;
  size_t n_;
};

// Owning NVFP4 tensor with packed scales.
struct Nvfp4Owned {
  DeviceVec<uint8_t> bytes, scales;
  DeviceVec<float> globals, decoded;
  uint32_t rows, cols;
  bool rowwise;
  Nvfp4Owned(uint32_t r, uint32_t c, bool rw)
      : bytes(Nvfp4TensorView::bytes_len(r, c)), scales(scale_packed_len(r, c)), globals(rw ? r : 1), decoded(1),
        rows(r), cols(c), rowwise(rw) {}
  Nvfp4TensorView view(bool with_decoded_amax) const {
    Nvfp4TensorView v;
    v.bytes = bytes.buf(), v.scales = scales.buf(), v.global_scales = globals.buf();
    v.rows = rows, v.cols = cols, v.scale_layout = NVFP4_SCALES_PACKED, v.rowwise = rowwise;
    if (with_decoded_amax) v.decoded_amax = decoded.buf();
    return v;
  }
};

struct OperandOwned {
  DeviceVec<uint8_t> bytes, scales;
  DeviceVec<float> globals, global, chunks;
  explicit OperandOwned(const MsEdenOperandSizes& z)
      : bytes(z.bytes), scales(z.scales_packed), globals(z.global_scales), global(z.global_scale), chunks(z.chunk_amax) {}
  MsEdenOperandBuffers view() const { return {bytes.buf(), scales.buf(), globals.buf(), global.buf(), chunks.buf()}; }
};
struct ScratchOwned {
  OperandOwned e_h, e_t_h, weight_t_h, input_t_h;
  explicit ScratchOwned(const LinearBackwardMsEdenScratchSizes& z)
      : e_h(z.e_h), e_t_h(z.e_t_h), weight_t_h(z.weight_t_h), input_t_h(z.input_t_h) {}
  LinearBackwardMsEdenScratchBuffers view() const {
    return {e_h.view(), e_t_h.view(), weight_t_h.view(), input_t_h.view()};
  }
};

std::vector<float> read_f32(std::FILE* f, size_t n) {
  std::vector<float> v(n);
  if (std::fread(v.data(), sizeof(float), n, f) != n) die("input", "file too short");
  return v;
}
void write_f32(std::FILE* f, const std::vector<float>& v) {
  if (std::fwrite(v.data(), sizeof(float), v.size(), f) != v.size()) die("output", "short write");
}

}  // namespace

int main(int argc, char** argv) {
  if (argc != 3) die("usage", "mlp_layer_driver <input> <output>");
  std::FILE* in = std::fopen(argv[1], "rb");
  if (!in) die("input", "cannot open");
  uint32_t hdr[8];
  if (std::fread(hdr, sizeof(uint32_t), 8, in) != 8 || hdr[0] != 0x4d4c5031u) die("input", "bad header");
  const uint32_t T = hdr[1], d = hdr[2], h = hdr[3];
  const size_t Td = size_t(T) * d, Th = size_t(T) * h, hd = size_t(h) * d;
  const auto hx = read_f32(in, Td), hwfc = read_f32(in, hd), hbfc = read_f32(in, h), hwproj = read_f32(in, hd),
             hbproj = read_f32(in, d), hdy = read_f32(in, Td);
  std::fclose(in);

  cudaStream_t stream;
  cuda_ok(cudaStreamCreate(&stream), "cudaStreamCreate");
  Stream s = stream;

  DeviceVec<float> x(Td), w_fc(hd), b_fc(h), w_proj(hd), b_proj(d), dy(Td);
  x.upload(hx, stream), w_fc.upload(hwfc, stream), b_fc.upload(hbfc, stream);
  w_proj.upload(hwproj, stream), b_proj.upload(hbproj, stream), dy.upload(hdy, stream);

  const auto quant = Nvfp4QuantModule::from_module();
  const auto mlp = MlpModule::from_module();
  const auto backward = LinearBackwardModule::from_module();

  // ---- weights: tensor amax, then four-six with one tensor scale, scales written packed -------------
  Nvfp4Owned wq_fc(h, d, false), wq_proj(d, h, false);
  DeviceVec<float> w_chunks(tensor_amax_chunks(uint32_t(hd))), w_amax(1);
  ok(quant.tensor_amax_f32(s, w_fc.cbuf(), w_chunks.buf(), w_amax.buf()), "tensor_amax_f32(w_fc)");
  ok(quant.quantize_four_six<float>(s, w_fc.cbuf(), w_amax.cbuf(), wq_fc.view(false)), "quantize_four_six(w_fc)");
  ok(quant.tensor_amax_f32(s, w_proj.cbuf(), w_chunks.buf(), w_amax.buf()), "tensor_amax_f32(w_proj)");
  ok(quant.quantize_four_six<float>(s, w_proj.cbuf(), w_amax.cbuf(), wq_proj.view(false)), "quantize_four_six(w_proj)");

  // ---- forward --------------------------------------------------------------------------------------
  Nvfp4Owned xq(T, d, true), hq(T, h, true);
  DeviceVec<float> pre(Th), hidden(Th), y(Td);
  ok(quant.quantize_row_amax<float>(s, x.cbuf(), xq.view(true)), "quantize_row_amax(x)");
  ok(mlp.up_relu2<float>(s, xq.view(false), wq_fc.view(false), b_fc.cbuf(), pre.buf(), hidden.buf()), "up_relu2");
  ok(quant.quantize_row_amax<float>(s, hidden.cbuf(), hq.view(true)), "quantize_row_amax(hidden)");
  ok(mlp.down<float>(s, hq.view(false), wq_proj.view(false), b_proj.cbuf(), y.buf()), "down");

  // ---- backward -------------------------------------------------------------------------------------
  ScratchOwned sc_proj(LinearBackwardMsEdenScratchSizes(T, h, d)), sc_fc(LinearBackwardMsEdenScratchSizes(T, d, h));
  DeviceVec<float> d_hidden(Th), d_pre(Th), dx(Td), dw_fc(hd), db_fc(h), dw_proj(hd), db_proj(d);

  LinearBackwardMsEdenArgs<float> bp;
  bp.e = dy.cbuf(), bp.weight = wq_proj.view(false), bp.input = hq.view(true), bp.scratch = sc_proj.view();
  bp.dinput = d_hidden.buf(), bp.dweight = dw_proj.buf(), bp.dbias = db_proj.buf();
  bp.token_count = T, bp.input_dim = h, bp.output_dim = d;
  bp.sign_seed = hdr[4], bp.scale_seed = hdr[5];
  ok(backward.backward_ms_eden(s, bp), "backward_ms_eden(proj)");

  uint32_t chunk_count = 0;
  ok(mlp.relu2_backward_amax<float>(s, pre.cbuf(), d_hidden.cbuf(), d_pre.buf(), sc_fc.e_h.chunks.buf(), &chunk_count),
     "relu2_backward_amax");

  LinearBackwardMsEdenArgs<float> bf;
  bf.e = d_pre.cbuf(), bf.weight = wq_fc.view(false), bf.input = xq.view(true), bf.scratch = sc_fc.view();
  bf.dinput = dx.buf(), bf.dweight = dw_fc.buf(), bf.dbias = db_fc.buf();
  bf.token_count = T, bf.input_dim = d, bf.output_dim = h;
  bf.sign_seed = hdr[6], bf.scale_seed = hdr[7];
  bf.precomputed_e_amax_chunks = chunk_count;
  ok(backward.backward_ms_eden(s, bf), "backward_ms_eden(fc)");

  // A deliberately short buffer must come back as an error value, not as a launch.
  LinearBackwardMsEdenArgs<float> bad = bf;
  bad.dweight.len = 1;
  if (backward.backward_ms_eden(s, bad).code != 1) die("length check", "a short dweight buffer was accepted");

  uint32_t status = 0;
  ok(read_device_status(s, &status), "read_device_status");

  std::FILE* out = std::fopen(argv[2], "wb");
  if (!out) die("output", "cannot open");
  write_f32(out, y.download(stream)), write_f32(out, dx.download(stream));
  write_f32(out, dw_fc.download(stream)), write_f32(out, db_fc.download(stream));
  write_f32(out, dw_proj.download(stream)), write_f32(out, db_proj.download(stream));
  const uint32_t tail[2] = {chunk_count, status};
  std::fwrite(tail, sizeof(uint32_t), 2, out);
  std::fclose(out);
  cuda_ok(cudaStreamDestroy(stream), "cudaStreamDestroy");
  return 0;
}
