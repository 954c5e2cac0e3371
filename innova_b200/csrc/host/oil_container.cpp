// The .oil container and its .oilidx companion, byte-compatible with the reference
// (include/oil/oil_format.h:15-35, src/oil_format.cpp:196-277 writer, :289-351 and :378-482 reader,
// :540-622 index file).
//
// Layout (little-endian, unpadded): "OIL1", u32 version, u32 flags, u32 config_size, config bytes,
// format table {u32 N, N x {u32 block_id, u8 format, u32 cb_bytes}}, tensor table {u32 T, T x {u16
// name_len, name, u32 block_start, u32 num_blocks}}, then the blocks in id order, each {u32
// num_weights, u32 cb_bytes, cb, u32 idx_bytes, idx}. Tensor shapes are not stored.
//
// The writer collects encoded tensors in memory (tables precede the blocks in the file, and block
// sizes are known only after encoding) and encodes blocks on all host cores. The reader loads the
// file, bounds-checks every advance, and tolerates what reference-written files contain: raw fp32
// blocks tagged with format 5, format bytes above 14, and tensor entries whose num_blocks is 0.
#include <algorithm>
#include <atomic>
#include <cstdio>
#include <cstring>
#include <functional>
#include <map>
#include <string>
#include <thread>
#include <vector>

#include "oil_codec.h"
#include "sha256.h"

namespace inv {

struct EncodedBlock {
  uint8_t format;
  uint32_t num_weights;
  std::vector<uint8_t> cb, idx;
};
struct PendingTensor {
  std::string name;
  std::vector<EncodedBlock> blocks;
};

static void parallel_for(size_t n, const std::function<void(size_t)>& fn);

class OilWriter {
 public:
  explicit OilWriter(const std::string& path) : path_(path) {}
  void set_header(uint32_t version, uint32_t flags, const uint8_t* cfg, uint32_t cfg_size) {
    version_ = version;
    flags_ = flags;
    config_.assign(cfg, cfg + cfg_size);
  }
  // formats: one byte per block (n_formats == number of blocks) or a single byte for all blocks.
  int add_tensor(const char* name, const float* w, uint64_t n, const uint8_t* formats, size_t n_formats, int block_size) {
    if (block_size <= 0 || n == 0) return -1;
    const size_t nb = (size_t)((n + block_size - 1) / block_size);
    if (n_formats != 1 && n_formats != nb) return -2;
    PendingTensor t;
    t.name = name;
    t.blocks.resize(nb);
    std::atomic<int> bad{0};
    parallel_for(nb, [&](size_t b) {
      const uint64_t lo = (uint64_t)b * block_size;
      const int cnt = (int)std::min<uint64_t>(block_size, n - lo);
      EncodedBlock& e = t.blocks[b];
      e.format = formats[n_formats == 1 ? 0 : b];
      e.num_weights = (uint32_t)cnt;
      if (!encode_block(e.format, w + lo, cnt, e.idx, e.cb)) bad = 1;
    });
    if (bad) return -3;
    tensors_.push_back(std::move(t));
    return 0;
  }
  int add_raw_block_tensor(const char* name, const uint8_t* fmt, const uint32_t* nw, const uint8_t* const* cb, const uint32_t* cb_len,
                           const uint8_t* const* idx, const uint32_t* idx_len, size_t nb) {
    PendingTensor t;
    t.name = name;
    t.blocks.resize(nb);
    for (size_t b = 0; b < nb; ++b) {
      t.blocks[b].format = fmt[b];
      t.blocks[b].num_weights = nw[b];
      t.blocks[b].cb.assign(cb[b], cb[b] + cb_len[b]);
      t.blocks[b].idx.assign(idx[b], idx[b] + idx_len[b]);
    }
    tensors_.push_back(std::move(t));
    return 0;
  }
  int finish() {
    FILE* f = std::fopen(path_.c_str(), "wb");
    if (!f) return -1;
    auto put = [&](const void* p, size_t n) { return n == 0 || std::fwrite(p, 1, n, f) == n; };
    auto put32 = [&](uint32_t v) { return put(&v, 4); };
    bool ok = put("OIL1", 4) && put32(version_) && put32(flags_) && put32((uint32_t)config_.size()) && put(config_.data(), config_.size());
    uint32_t total_blocks = 0;
    for (auto& t : tensors_) total_blocks += (uint32_t)t.blocks.size();
    ok = ok && put32(total_blocks);
    uint32_t id = 0;
    for (auto& t : tensors_)
      for (auto& b : t.blocks) {
        const uint32_t cbn = (uint32_t)b.cb.size();
        ok = ok && put32(id++) && put(&b.format, 1) && put32(cbn);
      }
    ok = ok && put32((uint32_t)tensors_.size());
    uint32_t start = 0;
    for (auto& t : tensors_) {
      const uint16_t nl = (uint16_t)t.name.size();
      ok = ok && put(&nl, 2) && put(t.name.data(), nl) && put32(start) && put32((uint32_t)t.blocks.size());
      start += (uint32_t)t.blocks.size();
    }
    for (auto& t : tensors_)
      for (auto& b : t.blocks)
        ok = ok && put32(b.num_weights) && put32((uint32_t)b.cb.size()) && put(b.cb.data(), b.cb.size()) && put32((uint32_t)b.idx.size()) &&
             put(b.idx.data(), b.idx.size());
    ok = (std::fclose(f) == 0) && ok;
    return ok ? 0 : -2;
  }
  uint64_t payload_bytes() const {
    uint64_t s = 0;
    for (auto& t : tensors_)
      for (auto& b : t.blocks) s += b.cb.size() + b.idx.size();
    return s;
  }

 private:
  std::string path_;
  uint32_t version_ = 1, flags_ = 0;
  std::vector<uint8_t> config_;
  std::vector<PendingTensor> tensors_;
};

struct BlockRef {
  uint8_t format;
  uint32_t num_weights, cb_bytes, idx_bytes;
  size_t cb_off, idx_off;
};
struct TensorRef {
  std::string name;
  uint32_t block_start, num_blocks;
  uint64_t numel;
};

class OilReader {
 public:
  explicit OilReader(const std::string& path) {
    FILE* f = std::fopen(path.c_str(), "rb");
    if (!f) return;
    std::fseek(f, 0, SEEK_END);
    const long sz = std::ftell(f);
    std::fseek(f, 0, SEEK_SET);
    if (sz > 0) {
      data_.resize((size_t)sz);
      if (std::fread(data_.data(), 1, (size_t)sz, f) != (size_t)sz) data_.clear();
    }
    std::fclose(f);
    parse();
  }
  bool valid() const { return valid_; }
  uint32_t version() const { return version_; }
  uint32_t flags() const { return flags_; }
  const std::vector<uint8_t>& config() const { return config_; }
  const std::vector<TensorRef>& tensors() const { return tensors_; }
  const std::vector<BlockRef>& blocks() const { return blocks_; }
  const uint8_t* base() const { return data_.data(); }
  const TensorRef* find(const std::string& name) const {
    auto it = by_name_.find(name);
    return it == by_name_.end() ? nullptr : &tensors_[it->second];
  }
  // The format a block decodes with (reference quirks resolved).
  int effective_format(const BlockRef& b) const {
    if (b.format > 14) return OIL32;
    if (b.format == OIL16 && b.idx_bytes == 4ull * b.num_weights) return OIL32;  // reference save() tags fp32 blocks with 5
    return b.format;
  }
  int read_tensor(const TensorRef& t, float* out) const {
    std::vector<uint64_t> offs(t.num_blocks + 1, 0);
    for (uint32_t i = 0; i < t.num_blocks; ++i) offs[i + 1] = offs[i] + blocks_[t.block_start + i].num_weights;
    parallel_for(t.num_blocks, [&](size_t i) {
      const BlockRef& b = blocks_[t.block_start + i];
      decode_block(effective_format(b), data_.data() + b.idx_off, b.idx_bytes, data_.data() + b.cb_off, b.cb_bytes, b.num_weights,
                   out + offs[i]);
    });
    return 0;
  }

 private:
  void parse() {
    const size_t n = data_.size();
    if (n < 16 || std::memcmp(data_.data(), "OIL1", 4) != 0) return;
    auto rd32 = [&](size_t at) { uint32_t v; std::memcpy(&v, data_.data() + at, 4); return v; };
    version_ = rd32(4);
    flags_ = rd32(8);
    const uint32_t cfg = rd32(12);
    if (16ull + cfg + 4 > n) return;
    config_.assign(data_.begin() + 16, data_.begin() + 16 + cfg);
    size_t at = 16 + (size_t)cfg;
    const uint32_t nb = rd32(at);
    at += 4;
    if (at + 9ull * nb + 4 > n) return;
    std::vector<uint8_t> table_fmt(nb);
    for (uint32_t i = 0; i < nb; ++i) table_fmt[i] = data_[at + 9ull * i + 4];
    at += 9ull * nb;
    const uint32_t nt = rd32(at);
    at += 4;
    for (uint32_t i = 0; i < nt; ++i) {
      if (at + 2 > n) break;
      uint16_t nl;
      std::memcpy(&nl, data_.data() + at, 2);
      at += 2;
      if (at + nl + 8 > n) break;
      TensorRef t;
      t.name.assign(reinterpret_cast<const char*>(data_.data() + at), nl);
      at += nl;
      t.block_start = rd32(at);
      t.num_blocks = rd32(at + 4);
      t.numel = 0;
      at += 8;
      tensors_.push_back(std::move(t));
    }
    blocks_.reserve(nb);
    for (uint32_t i = 0; i < nb; ++i) {
      if (at + 8 > n) break;
      BlockRef b;
      b.format = table_fmt[i];
      b.num_weights = rd32(at);
      b.cb_bytes = rd32(at + 4);
      b.cb_off = at + 8;
      if (b.cb_off + b.cb_bytes + 4 > n) break;
      b.idx_bytes = rd32(b.cb_off + b.cb_bytes);
      b.idx_off = b.cb_off + b.cb_bytes + 4;
      if (b.idx_off + b.idx_bytes > n) break;
      at = b.idx_off + b.idx_bytes;
      blocks_.push_back(b);
    }
    // entries written with num_blocks == 0 (a reference converter quirk): infer from the next start
    std::vector<size_t> order(tensors_.size());
    for (size_t i = 0; i < order.size(); ++i) order[i] = i;
    std::sort(order.begin(), order.end(), [&](size_t a, size_t b) { return tensors_[a].block_start < tensors_[b].block_start; });
    for (size_t k = 0; k < order.size(); ++k) {
      TensorRef& t = tensors_[order[k]];
      if (t.num_blocks == 0) {
        const uint32_t next = k + 1 < order.size() ? tensors_[order[k + 1]].block_start : (uint32_t)blocks_.size();
        t.num_blocks = next > t.block_start ? next - t.block_start : 0;
      }
      if ((uint64_t)t.block_start + t.num_blocks > blocks_.size())
        t.num_blocks = t.block_start < blocks_.size() ? (uint32_t)blocks_.size() - t.block_start : 0;
      for (uint32_t i = 0; i < t.num_blocks; ++i) t.numel += blocks_[t.block_start + i].num_weights;
    }
    for (size_t i = 0; i < tensors_.size(); ++i) by_name_[tensors_[i].name] = i;
    valid_ = true;
  }
  std::vector<uint8_t> data_;
  bool valid_ = false;
  uint32_t version_ = 0, flags_ = 0;
  std::vector<uint8_t> config_;
  std::vector<TensorRef> tensors_;
  std::vector<BlockRef> blocks_;
  std::map<std::string, size_t> by_name_;
};

static void parallel_for(size_t n, const std::function<void(size_t)>& fn) {
  unsigned hw = std::thread::hardware_concurrency();
  size_t nt = std::min<size_t>(hw ? hw : 4, n / 64 + 1);
  if (nt <= 1) {
    for (size_t i = 0; i < n; ++i) fn(i);
    return;
  }
  std::atomic<size_t> next{0};
  std::vector<std::thread> th;
  for (size_t t = 0; t < nt; ++t)
    th.emplace_back([&]() {
      for (;;) {
        const size_t lo = next.fetch_add(256);
        if (lo >= n) return;
        const size_t hi = std::min(n, lo + 256);
        for (size_t i = lo; i < hi; ++i) fn(i);
      }
    });
  for (auto& t : th) t.join();
}

}  // namespace inv

using namespace inv;

extern "C" {

// ---------------------------------------------------------------- codec
int oil_format_count() { return FORMAT_COUNT; }
const char* oil_format_name(int fmt) { return format_name(fmt); }
int oil_format_from_name(const char* name) { return format_from_name(name); }
float oil_format_bpw(int fmt) { return format_bpw(fmt); }
uint64_t oil_claimed_bytes(int fmt, uint32_t n) { return claimed_bytes(fmt, n); }
uint16_t oil_f32_to_f16(float v) { return f32_to_f16(v); }
float oil_f16_to_f32(uint16_t h) { return f16_to_f32(h); }

// Encodes one block. idx_out / cb_out need capacity 4*n + 16. Returns 0, or -1 for an unknown format.
int oil_encode_block(int fmt, const float* w, int n, uint8_t* idx_out, uint64_t* idx_len, uint8_t* cb_out, uint64_t* cb_len) {
  std::vector<uint8_t> idx, cb;
  if (!encode_block(fmt, w, n, idx, cb)) return -1;
  std::memcpy(idx_out, idx.data(), idx.size());
  std::memcpy(cb_out, cb.data(), cb.size());
  *idx_len = idx.size();
  *cb_len = cb.size();
  return 0;
}
void oil_decode_block(int fmt, const uint8_t* idx, uint64_t idx_len, const uint8_t* cb, uint64_t cb_len, uint32_t n, float* out) {
  decode_block(fmt, idx, idx_len, cb, cb_len, n, out);
}
// Quantise + dequantise a whole tensor in blocks (what a stored tensor decodes to); returns stored bytes.
uint64_t oil_roundtrip(int fmt, const float* w, uint64_t n, int block_size, float* out) {
  const size_t nb = (size_t)((n + block_size - 1) / block_size);
  std::vector<uint64_t> bytes(nb, 0);
  parallel_for(nb, [&](size_t b) {
    const uint64_t lo = (uint64_t)b * block_size;
    const int cnt = (int)std::min<uint64_t>(block_size, n - lo);
    std::vector<uint8_t> idx, cb;
    encode_block(fmt, w + lo, cnt, idx, cb);
    decode_block(fmt, idx.data(), idx.size(), cb.data(), cb.size(), (uint32_t)cnt, out + lo);
    bytes[b] = idx.size() + cb.size();
  });
  uint64_t s = 0;
  for (auto v : bytes) s += v;
  return s;
}

// ---------------------------------------------------------------- sha256
void oil_sha256(const void* data, uint64_t size, uint8_t out[32]) {
  Sha256 h = sha256(data, size);
  std::memcpy(out, h.bytes, 32);
}

// ---------------------------------------------------------------- writer
void* oilw_open(const char* path) { return new OilWriter(path); }
void oilw_set_header(void* w, uint32_t version, uint32_t flags, const uint8_t* cfg, uint32_t cfg_size) {
  static_cast<OilWriter*>(w)->set_header(version, flags, cfg, cfg_size);
}
int oilw_add_tensor(void* w, const char* name, const float* data, uint64_t n, const uint8_t* formats, uint64_t n_formats, int block_size) {
  return static_cast<OilWriter*>(w)->add_tensor(name, data, n, formats, n_formats, block_size);
}
uint64_t oilw_payload_bytes(void* w) { return static_cast<OilWriter*>(w)->payload_bytes(); }
int oilw_close(void* w) {
  OilWriter* ow = static_cast<OilWriter*>(w);
  const int rc = ow->finish();
  delete ow;
  return rc;
}

// ---------------------------------------------------------------- reader
void* oilr_open(const char* path) {
  OilReader* r = new OilReader(path);
  if (!r->valid()) {
    delete r;
    return nullptr;
  }
  return r;
}
void oilr_close(void* r) { delete static_cast<OilReader*>(r); }
uint32_t oilr_version(void* r) { return static_cast<OilReader*>(r)->version(); }
uint32_t oilr_flags(void* r) { return static_cast<OilReader*>(r)->flags(); }
uint32_t oilr_config_size(void* r) { return (uint32_t)static_cast<OilReader*>(r)->config().size(); }
void oilr_config(void* r, uint8_t* out) {
  auto& c = static_cast<OilReader*>(r)->config();
  std::memcpy(out, c.data(), c.size());
}
uint32_t oilr_num_tensors(void* r) { return (uint32_t)static_cast<OilReader*>(r)->tensors().size(); }
uint32_t oilr_num_blocks(void* r) { return (uint32_t)static_cast<OilReader*>(r)->blocks().size(); }
const char* oilr_tensor_name(void* r, uint32_t i) { return static_cast<OilReader*>(r)->tensors()[i].name.c_str(); }
uint64_t oilr_tensor_numel(void* r, uint32_t i) { return static_cast<OilReader*>(r)->tensors()[i].numel; }
uint32_t oilr_tensor_block_start(void* r, uint32_t i) { return static_cast<OilReader*>(r)->tensors()[i].block_start; }
uint32_t oilr_tensor_num_blocks(void* r, uint32_t i) { return static_cast<OilReader*>(r)->tensors()[i].num_blocks; }
int oilr_find(void* r, const char* name) {
  auto* rd = static_cast<OilReader*>(r);
  const TensorRef* t = rd->find(name);
  return t ? (int)(t - rd->tensors().data()) : -1;
}
int oilr_read_tensor(void* r, uint32_t i, float* out) {
  auto* rd = static_cast<OilReader*>(r);
  if (i >= rd->tensors().size()) return -1;
  return rd->read_tensor(rd->tensors()[i], out);
}
// Block metadata: out = {format as stored, effective format, num_weights, cb_bytes, idx_bytes}
int oilr_block_info(void* r, uint32_t b, uint32_t out[5]) {
  auto* rd = static_cast<OilReader*>(r);
  if (b >= rd->blocks().size()) return -1;
  const BlockRef& br = rd->blocks()[b];
  out[0] = br.format;
  out[1] = (uint32_t)rd->effective_format(br);
  out[2] = br.num_weights;
  out[3] = br.cb_bytes;
  out[4] = br.idx_bytes;
  return 0;
}
// Raw payload pointers of a block inside the reader's buffer (valid until oilr_close).
int oilr_block_payload(void* r, uint32_t b, const uint8_t** cb, const uint8_t** idx) {
  auto* rd = static_cast<OilReader*>(r);
  if (b >= rd->blocks().size()) return -1;
  const BlockRef& br = rd->blocks()[b];
  *cb = rd->base() + br.cb_off;
  *idx = rd->base() + br.idx_off;
  return 0;
}

// Device-decoder records (csrc/block_codec.cu, 32 bytes each) for the blocks of tensor i. Payload offsets are
// relative to *base_off, the start of the file span [*base_off, *base_off + *span) that holds the tensor's
// blocks; the caller uploads that span once and decodes the whole tensor in one launch.
const uint8_t* oilr_base(void* r) { return static_cast<OilReader*>(r)->base(); }
int oilr_tensor_descs(void* r, uint32_t i, void* descs, uint64_t* base_off, uint64_t* span) {
  auto* rd = static_cast<OilReader*>(r);
  if (i >= rd->tensors().size()) return -1;
  const TensorRef& t = rd->tensors()[i];
  size_t lo = (size_t)-1, hi = 0;
  for (uint32_t b = 0; b < t.num_blocks; ++b) {
    const BlockRef& br = rd->blocks()[t.block_start + b];
    if (br.cb_bytes) { lo = std::min(lo, br.cb_off); hi = std::max(hi, br.cb_off + br.cb_bytes); }
    if (br.idx_bytes) { lo = std::min(lo, br.idx_off); hi = std::max(hi, br.idx_off + br.idx_bytes); }
  }
  if (lo == (size_t)-1) lo = hi = 0;
  if (hi - lo >= (1ull << 32)) return -2;
  *base_off = lo;
  *span = hi - lo;
  if (!descs) return 0;
  struct Desc {
    uint64_t idx_off, out_off;
    uint32_t idx_bytes, cb_off_lo;
    uint16_t cb_bytes;
    uint8_t fmt, pad;
    uint32_t n;
  };
  static_assert(sizeof(Desc) == 32, "record layout");
  Desc* d = static_cast<Desc*>(descs);
  uint64_t out = 0;
  for (uint32_t b = 0; b < t.num_blocks; ++b) {
    const BlockRef& br = rd->blocks()[t.block_start + b];
    d[b].idx_off = br.idx_bytes ? br.idx_off - lo : 0;
    d[b].out_off = out;
    d[b].idx_bytes = br.idx_bytes;
    d[b].cb_off_lo = br.cb_bytes ? (uint32_t)(br.cb_off - lo) : 0;
    d[b].cb_bytes = (uint16_t)std::min<uint32_t>(br.cb_bytes, 65535u);
    d[b].fmt = (uint8_t)rd->effective_format(br);
    d[b].pad = 0;
    d[b].n = br.num_weights;
    out += br.num_weights;
  }
  return 0;
}

// ---------------------------------------------------------------- .oilidx
// names: n NUL-terminated strings back to back.
int oilidx_write(const char* path, uint32_t version, const char* names, uint32_t n) {
  FILE* f = std::fopen(path, "wb");
  if (!f) return -1;
  const char magic[10] = {'I', 'n', 'N', 'o', 'v', 'a', 'I', 'D', 'X', '\0'};
  std::fwrite(magic, 1, 10, f);
  std::fwrite(&version, 4, 1, f);
  std::fwrite(&n, 4, 1, f);
  const char* p = names;
  for (uint32_t i = 0; i < n; ++i) {
    const size_t len = std::strlen(p);
    const uint16_t nl = (uint16_t)len;
    std::fwrite(&nl, 2, 1, f);
    std::fwrite(p, 1, len, f);
    const Sha256 h = sha256(p, len);
    std::fwrite(h.bytes, 1, 32, f);
    p += len + 1;
  }
  return std::fclose(f) == 0 ? 0 : -2;
}
// Verifies every stored hash. Returns the number of names (>= 0) and fills `names_out` (NUL-separated,
// capacity `cap`); -1 unreadable / bad magic, -2 truncated, -(100 + i) when name i fails its hash, in
// which case names_out holds that name.
int oilidx_read(const char* path, uint32_t* version, char* names_out, uint64_t cap) {
  FILE* f = std::fopen(path, "rb");
  if (!f) return -1;
  std::vector<uint8_t> d;
  std::fseek(f, 0, SEEK_END);
  const long sz = std::ftell(f);
  std::fseek(f, 0, SEEK_SET);
  d.resize(sz > 0 ? (size_t)sz : 0);
  if (sz > 0 && std::fread(d.data(), 1, d.size(), f) != d.size()) d.clear();
  std::fclose(f);
  if (d.size() < 18 || std::memcmp(d.data(), "InNovaIDX\0", 10) != 0) return -1;
  uint32_t n;
  std::memcpy(version, d.data() + 10, 4);
  std::memcpy(&n, d.data() + 14, 4);
  size_t at = 18, w = 0;
  for (uint32_t i = 0; i < n; ++i) {
    if (at + 2 > d.size()) return -2;
    uint16_t nl;
    std::memcpy(&nl, d.data() + at, 2);
    at += 2;
    if (at + nl + 32 > d.size()) return -2;
    const Sha256 h = sha256(d.data() + at, nl);
    if (std::memcmp(h.bytes, d.data() + at + nl, 32) != 0) {
      if (cap > (uint64_t)nl) {
        std::memcpy(names_out, d.data() + at, nl);
        names_out[nl] = 0;
      }
      return -(100 + (int)i);
    }
    if (w + nl + 1 <= cap) {
      std::memcpy(names_out + w, d.data() + at, nl);
      names_out[w + nl] = 0;
      w += nl + 1;
    }
    at += nl + 32;
  }
  return (int)n;
}

}  // extern "C"
