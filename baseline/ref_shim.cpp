// C shim over the UNMODIFIED reference sources (block codec and .oil reader/writer), compiled out
// of tree into baseline/_ref/ and used only as a test oracle for byte compatibility.
#include <cstring>
#include <string>
#include <vector>

#include "oil/block_codec.h"
#include "oil/oil_format.h"
#include "oil/random.h"
#include "oil/tensor.h"

extern "C" {
int ref_encode_block(int fmt, const float* w, int n, uint8_t* idx_out, uint64_t* idx_len, uint8_t* cb_out, uint64_t* cb_len) {
  std::vector<uint8_t> idx, cb;
  if (!oil::quantize_block_all((oil::Format)fmt, w, n, idx, cb)) return -1;
  std::memcpy(idx_out, idx.data(), idx.size());
  std::memcpy(cb_out, cb.data(), cb.size());
  *idx_len = idx.size();
  *cb_len = cb.size();
  return 0;
}
void ref_decode_block(int fmt, const uint8_t* idx, uint64_t idx_len, const uint8_t* cb, uint64_t cb_len, uint32_t n, float* out) {
  oil::dequantize_block_all((oil::Format)fmt, idx, idx_len, cb, cb_len, n, out);
}
// Reads a tensor with the reference's OILReader; returns its element count or -1.
long ref_read_tensor(const char* path, const char* name, float* out, long cap) {
  oil::OILReader r(path);
  if (!r.valid()) return -1;
  oil::Tensor t = r.read_tensor(name);
  const long n = (long)t.numel();
  if (n > cap) return -2;
  std::memcpy(out, t.data<float>(), (size_t)n * 4);
  return n;
}
// Writes one tensor in 256-weight blocks of one format with the reference's writer and codec.
int ref_write_single(const char* path, const char* name, const float* w, long n, int fmt, int block) {
  std::vector<oil::BlockData> blocks;
  for (long lo = 0; lo < n; lo += block) {
    oil::BlockData b;
    b.format = (oil::Format)fmt;
    b.num_weights = (uint32_t)std::min<long>(block, n - lo);
    oil::quantize_block_all(b.format, w + lo, (int)b.num_weights, b.indices, b.codebook);
    blocks.push_back(std::move(b));
  }
  oil::OILWriter wr(path);
  oil::OILHeader h;
  std::memcpy(h.magic, "OIL1", 4);
  h.version = 1; h.flags = 0; h.config_size = 0;
  wr.write_header(h, nullptr);
  std::vector<oil::FormatBlockEntry> ft;
  for (size_t i = 0; i < blocks.size(); ++i) ft.push_back({(uint32_t)i, (uint8_t)fmt, (uint32_t)blocks[i].codebook.size()});
  wr.write_format_table(ft);
  oil::TensorEntry te; te.name_len = (uint16_t)std::strlen(name); te.block_start = 0; te.num_blocks = (uint32_t)blocks.size();
  wr.write_tensor_table({te}, {std::string(name)});
  for (auto& b : blocks) wr.write_block(b);
  wr.close();
  return 0;
}
// The reference's random stream: n raw words, then n uniforms, n normals and n integers in [lo, hi] from fresh generators.
void ref_rng_stream(uint64_t seed, int n, uint64_t* words, float* uniforms, float* normals, int lo, int hi, int* ints) {
  oil::RNG a(seed), b(seed), c(seed), d(seed);
  for (int i = 0; i < n; i++) words[i] = a.next_u64();
  for (int i = 0; i < n; i++) uniforms[i] = b.uniform();
  for (int i = 0; i < n; i++) normals[i] = c.normal();
  for (int i = 0; i < n; i++) ints[i] = d.uniform_int(lo, hi);
}
// Serialises a tensor of the given dims / dtype code / raw bytes with the reference's Tensor::serialize; returns the size.
long ref_serialize_tensor(const int64_t* dims, int rank, int dtype, const uint8_t* raw, long raw_bytes, uint8_t* out, long cap) {
  oil::Shape sh;
  sh.rank = rank;
  for (int i = 0; i < rank; i++) sh.dims[i] = dims[i];
  oil::Tensor t(sh, (oil::DType)dtype);
  if ((long)t.size_bytes() != raw_bytes) return -1;
  std::memcpy(t.data(), raw, (size_t)raw_bytes);
  if ((long)t.serialized_size() > cap) return -2;
  return (long)t.serialize(out);
}
}
