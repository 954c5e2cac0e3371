// Native importers: GGUF, safetensors and raw tensor files -> fp32.
//
// The file is mapped read-only; tensors are listed once at open time and decoded on request straight from the mapping
// into the caller's buffer, so a multi-GB checkpoint is never held twice. Covers what the reference's converter reads
// (tools/convert.cpp:175-310, src/adapters/src/gguf_bridge.cpp, src/adapters/src/safetensors_bridge.cpp):
//   GGUF v1-v3   F32, F16, BF16, F64, I8, I16, I32, Q4_0, Q4_1, Q5_0, Q5_1, Q8_0, Q8_1, Q2_K, Q3_K, Q4_K, Q5_K, Q6_K
//                (ggml's block layouts), general.alignment honoured
//   safetensors  F64, F32, F16, BF16, F8_E4M3, F8_E5M2, I64, I32, I16, I8, U8, BOOL
//   raw          flat little-endian fp32 / fp16 / bf16 / fp8-e4m3 / fp8-e5m2
// Every read is bounds-checked against the mapping; a malformed file gives an error string, never a fault.
#include <fcntl.h>
#include <sys/mman.h>
#include <sys/stat.h>
#include <unistd.h>

#include <cmath>
#include <cstdint>
#include <cstdio>
#include <cstring>
#include <string>
#include <vector>

namespace {

struct Mapping {
  const uint8_t* p = nullptr;
  size_t n = 0;
  int fd = -1;
  bool open(const char* path, std::string& err) {
    fd = ::open(path, O_RDONLY);
    if (fd < 0) { err = std::string("cannot open ") + path; return false; }
    struct stat st;
    if (fstat(fd, &st) != 0) { err = "fstat failed"; return false; }
    n = (size_t)st.st_size;
    if (n == 0) { err = "empty file"; return false; }
    void* m = mmap(nullptr, n, PROT_READ, MAP_PRIVATE, fd, 0);
    if (m == MAP_FAILED) { err = "mmap failed"; return false; }
    p = (const uint8_t*)m;
    return true;
  }
  ~Mapping() {
    if (p) munmap((void*)p, n);
    if (fd >= 0) ::close(fd);
  }
};

inline float half_to_float(uint16_t h) {
  const uint32_t sign = (uint32_t)(h & 0x8000u) << 16;
  uint32_t exp = (h >> 10) & 31u, man = h & 1023u, bits;
  if (exp == 0) {
    if (man == 0) {
      bits = sign;
    } else {  // subnormal: renormalise
      int e = -1;
      do { man <<= 1; ++e; } while (!(man & 1024u));
      bits = sign | ((uint32_t)(127 - 15 - e) << 23) | ((man & 1023u) << 13);
    }
  } else if (exp == 31) {
    bits = sign | 0x7f800000u | (man << 13);
  } else {
    bits = sign | ((exp + 112u) << 23) | (man << 13);
  }
  float f;
  memcpy(&f, &bits, 4);
  return f;
}
inline float bf16_to_float(uint16_t h) {
  const uint32_t bits = (uint32_t)h << 16;
  float f;
  memcpy(&f, &bits, 4);
  return f;
}
inline float e4m3_to_float(uint8_t v) {  // fn variant: no infinities, 0x7f / 0xff are NaN
  const int s = v >> 7, e = (v >> 3) & 15, m = v & 7;
  float r;
  if (e == 15 && m == 7) r = NAN;
  else if (e == 0) r = std::ldexp((float)m, -9);
  else r = std::ldexp(1.f + m / 8.f, e - 7);
  return s ? -r : r;
}
inline float e5m2_to_float(uint8_t v) { return half_to_float((uint16_t)v << 8); }
inline uint16_t rd16(const uint8_t* p) { uint16_t v; memcpy(&v, p, 2); return v; }
inline uint32_t rd32(const uint8_t* p) { uint32_t v; memcpy(&v, p, 4); return v; }

enum Kind { KIND_GGUF = 1, KIND_SAFETENSORS = 2 };
// element codes shared by both containers
enum Elem {
  E_F32, E_F16, E_BF16, E_F64, E_I8, E_U8, E_I16, E_I32, E_I64, E_BOOL, E_F8E4M3, E_F8E5M2,
  E_Q4_0, E_Q4_1, E_Q5_0, E_Q5_1, E_Q8_0, E_Q8_1, E_Q2_K, E_Q3_K, E_Q4_K, E_Q5_K, E_Q6_K
};
struct ElemInfo { int block; int bytes; };  // weights per block, bytes per block
const ElemInfo ELEM[] = {{1, 4}, {1, 2}, {1, 2}, {1, 8}, {1, 1}, {1, 1}, {1, 2}, {1, 4}, {1, 8}, {1, 1}, {1, 1}, {1, 1},
                         {32, 18}, {32, 20}, {32, 22}, {32, 24}, {32, 34}, {32, 36}, {256, 84}, {256, 110}, {256, 144}, {256, 176}, {256, 210}};

struct TensorEntry {
  std::string name;
  std::vector<int64_t> dims;   // outermost first
  int elem = E_F32;
  int64_t numel = 0;
  size_t offset = 0, nbytes = 0;
};

struct Importer {
  Mapping map;
  int kind = 0;
  std::vector<TensorEntry> tensors;
  std::string meta;            // safetensors "__metadata__" object text / GGUF "general.architecture"
};

// ------------------------------------------------------------------------------------------------ GGUF
struct Cursor {
  const uint8_t* p; size_t n, at = 0; bool ok = true;
  bool need(size_t k) { if (!ok || k > n - at) { ok = false; return false; } return true; }
  template <class T> T get() { T v{}; if (need(sizeof(T))) { memcpy(&v, p + at, sizeof(T)); at += sizeof(T); } return v; }
  uint64_t count(bool wide) { return wide ? get<uint64_t>() : (uint64_t)get<uint32_t>(); }
  std::string str(bool wide) {
    const uint64_t k = count(wide);
    if (!need(k)) return {};
    std::string s((const char*)p + at, (size_t)k);
    at += (size_t)k;
    return s;
  }
};

bool gguf_skip_value(Cursor& c, uint32_t t, bool wide, int depth) {
  static const int sz[13] = {1, 1, 2, 2, 4, 4, 4, 1, 0, 0, 8, 8, 8};
  if (t == 8) { c.str(wide); return c.ok; }
  if (t == 9) {
    if (depth > 4) return false;
    const uint32_t et = c.get<uint32_t>();
    const uint64_t k = c.count(wide);
    if (et != 8 && et != 9) {
      if (et > 12) return false;
      if (k > (c.n - c.at) / (sz[et] ? sz[et] : 1)) return false;
      c.at += (size_t)k * sz[et];
      return c.ok;
    }
    for (uint64_t i = 0; i < k && c.ok; ++i)
      if (!gguf_skip_value(c, et, wide, depth + 1)) return false;
    return c.ok;
  }
  if (t > 12) return false;
  if (!c.need(sz[t])) return false;
  c.at += sz[t];
  return true;
}

int ggml_to_elem(uint32_t t) {
  switch (t) {
    case 0: return E_F32; case 1: return E_F16; case 2: return E_Q4_0; case 3: return E_Q4_1; case 6: return E_Q5_0;
    case 7: return E_Q5_1; case 8: return E_Q8_0; case 9: return E_Q8_1; case 10: return E_Q2_K; case 11: return E_Q3_K;
    case 12: return E_Q4_K; case 13: return E_Q5_K; case 14: return E_Q6_K; case 24: return E_I8; case 25: return E_I16;
    case 26: return E_I32; case 27: return E_I64; case 28: return E_F64; case 30: return E_BF16;
    default: return -1;
  }
}

bool parse_gguf(Importer& im, std::string& err) {
  Cursor c{im.map.p, im.map.n};
  if (im.map.n < 16 || memcmp(im.map.p, "GGUF", 4) != 0) { err = "not a GGUF file"; return false; }
  c.at = 4;
  const uint32_t ver = c.get<uint32_t>();
  if (ver < 1 || ver > 3) { err = "unsupported GGUF version " + std::to_string(ver); return false; }
  const bool wide = ver >= 2;
  const uint64_t n_tensors = c.count(wide), n_kv = c.count(wide);
  if (n_tensors > (1u << 24) || n_kv > (1u << 24)) { err = "implausible GGUF header"; return false; }
  uint64_t align = 32;
  for (uint64_t i = 0; i < n_kv; ++i) {
    const std::string key = c.str(wide);
    const uint32_t t = c.get<uint32_t>();
    if (!c.ok) break;
    if (key == "general.alignment" && t == 4) {
      if (c.need(4)) align = rd32(c.p + c.at);
    } else if (key == "general.architecture" && t == 8) {
      Cursor peek = c;
      im.meta = peek.str(wide);
    }
    if (!gguf_skip_value(c, t, wide, 0)) { err = "malformed GGUF metadata at key '" + key + "'"; return false; }
  }
  if (!c.ok) { err = "truncated GGUF metadata"; return false; }
  if (align == 0 || (align & (align - 1))) { err = "GGUF alignment is not a power of two"; return false; }
  im.tensors.reserve((size_t)n_tensors);
  for (uint64_t i = 0; i < n_tensors; ++i) {
    TensorEntry e;
    e.name = c.str(wide);
    const uint32_t nd = c.get<uint32_t>();
    if (!c.ok || nd > 8) { err = "malformed GGUF tensor record"; return false; }
    e.numel = 1;
    std::vector<int64_t> ne(nd);
    for (uint32_t d = 0; d < nd; ++d) {
      ne[d] = (int64_t)c.count(wide);
      if (ne[d] < 0 || (ne[d] > 0 && e.numel > INT64_MAX / ne[d])) { err = e.name + ": dimension overflow"; return false; }
      e.numel *= ne[d];
    }
    e.dims.assign(ne.rbegin(), ne.rend());  // GGUF lists the innermost dimension first
    const uint32_t typ = c.get<uint32_t>();
    e.offset = (size_t)c.get<uint64_t>();
    if (!c.ok) { err = "truncated GGUF tensor table"; return false; }
    e.elem = ggml_to_elem(typ);
    if (e.elem < 0) { err = e.name + ": GGUF tensor type " + std::to_string(typ) + " is not supported"; return false; }
    const ElemInfo ei = ELEM[e.elem];
    if (e.numel % ei.block) { err = e.name + ": element count is not a whole number of blocks"; return false; }
    e.nbytes = (size_t)(e.numel / ei.block) * ei.bytes;
    im.tensors.push_back(std::move(e));
  }
  const size_t base = (c.at + align - 1) / align * align;
  for (auto& e : im.tensors) {
    if (e.offset > im.map.n || base > im.map.n - e.offset || e.nbytes > im.map.n - base - e.offset) {
      err = e.name + ": data outside the file";
      return false;
    }
    e.offset += base;
  }
  return true;
}

// ------------------------------------------------------------------------------------------------ safetensors (JSON header)
struct Json {
  const char* s; size_t n, at = 0; bool ok = true;
  void ws() { while (at < n && (s[at] == ' ' || s[at] == '\n' || s[at] == '\t' || s[at] == '\r')) ++at; }
  bool eat(char c) { ws(); if (at < n && s[at] == c) { ++at; return true; } return false; }
  char peek() { ws(); return at < n ? s[at] : 0; }
  std::string str() {
    std::string out;
    if (!eat('"')) { ok = false; return out; }
    while (at < n && s[at] != '"') {
      char ch = s[at++];
      if (ch == '\\' && at < n) {
        const char e = s[at++];
        switch (e) {
          case 'n': out += '\n'; break; case 't': out += '\t'; break; case 'r': out += '\r'; break;
          case 'b': out += '\b'; break; case 'f': out += '\f'; break;
          case 'u': {
            if (at + 4 > n) { ok = false; return out; }
            unsigned cp = 0;
            for (int i = 0; i < 4; ++i) {
              const char h = s[at++];
              cp = cp * 16 + (h >= '0' && h <= '9' ? h - '0' : h >= 'a' && h <= 'f' ? h - 'a' + 10 : h >= 'A' && h <= 'F' ? h - 'A' + 10 : 0);
            }
            if (cp < 0x80) out += (char)cp;
            else if (cp < 0x800) { out += (char)(0xC0 | (cp >> 6)); out += (char)(0x80 | (cp & 63)); }
            else { out += (char)(0xE0 | (cp >> 12)); out += (char)(0x80 | ((cp >> 6) & 63)); out += (char)(0x80 | (cp & 63)); }
            break;
          }
          default: out += e;
        }
      } else {
        out += ch;
      }
    }
    if (at >= n) { ok = false; return out; }
    ++at;
    return out;
  }
  int64_t integer() {
    ws();
    int64_t v = 0; bool any = false, neg = false;
    if (at < n && s[at] == '-') { neg = true; ++at; }
    while (at < n && s[at] >= '0' && s[at] <= '9') {
      if (v > (INT64_MAX - 9) / 10) { ok = false; return 0; }
      v = v * 10 + (s[at++] - '0');
      any = true;
    }
    if (!any) ok = false;
    return neg ? -v : v;
  }
  void skip(int depth = 0) {  // any value
    if (depth > 32) { ok = false; return; }
    const char c = peek();
    if (c == '"') { str(); return; }
    if (c == '{' || c == '[') {
      const char close = c == '{' ? '}' : ']';
      ++at;
      if (eat(close)) return;
      do {
        if (c == '{') { str(); if (!eat(':')) { ok = false; return; } }
        skip(depth + 1);
        if (!ok) return;
      } while (eat(','));
      if (!eat(close)) ok = false;
      return;
    }
    while (at < n && s[at] != ',' && s[at] != '}' && s[at] != ']') ++at;  // number / true / false / null
  }
};

int st_elem(const std::string& d) {
  static const struct { const char* n; int e; } T[] = {{"F32", E_F32}, {"F16", E_F16}, {"BF16", E_BF16}, {"F64", E_F64}, {"I8", E_I8},
      {"U8", E_U8}, {"I16", E_I16}, {"I32", E_I32}, {"I64", E_I64}, {"BOOL", E_BOOL}, {"F8_E4M3", E_F8E4M3}, {"F8_E5M2", E_F8E5M2}};
  for (auto& t : T) if (d == t.n) return t.e;
  return -1;
}

bool parse_safetensors(Importer& im, std::string& err) {
  if (im.map.n < 8) { err = "not a safetensors file"; return false; }
  uint64_t hn;
  memcpy(&hn, im.map.p, 8);
  if (hn > im.map.n - 8 || hn < 2) { err = "safetensors header length outside the file"; return false; }
  Json j{(const char*)im.map.p + 8, (size_t)hn};
  const size_t base = 8 + (size_t)hn, data_bytes = im.map.n - base;
  if (!j.eat('{')) { err = "safetensors header is not a JSON object"; return false; }
  if (j.peek() != '}') {
    do {
      std::string name = j.str();
      if (!j.ok || !j.eat(':')) { err = "malformed safetensors header"; return false; }
      if (name == "__metadata__") {
        const size_t a = j.at;
        j.skip();
        im.meta.assign(j.s + a, j.at - a);
        continue;
      }
      TensorEntry e;
      e.name = std::move(name);
      std::string dtype;
      int64_t lo = -1, hi = -1;
      if (!j.eat('{')) { err = e.name + ": tensor record is not an object"; return false; }
      do {
        const std::string key = j.str();
        if (!j.ok || !j.eat(':')) { err = e.name + ": malformed record"; return false; }
        if (key == "dtype") dtype = j.str();
        else if (key == "shape") {
          if (!j.eat('[')) { err = e.name + ": shape is not an array"; return false; }
          if (j.peek() != ']') do { e.dims.push_back(j.integer()); } while (j.eat(','));
          if (!j.eat(']')) { err = e.name + ": malformed shape"; return false; }
        } else if (key == "data_offsets") {
          if (!j.eat('[')) { err = e.name + ": data_offsets is not an array"; return false; }
          lo = j.integer();
          if (!j.eat(',')) { err = e.name + ": malformed data_offsets"; return false; }
          hi = j.integer();
          if (!j.eat(']')) { err = e.name + ": malformed data_offsets"; return false; }
        } else {
          j.skip();
        }
      } while (j.ok && j.eat(','));
      if (!j.ok || !j.eat('}')) { err = e.name + ": malformed record"; return false; }
      e.elem = st_elem(dtype);
      if (e.elem < 0) { err = e.name + ": dtype " + dtype + " is not supported"; return false; }
      e.numel = 1;
      for (int64_t d : e.dims) {
        if (d < 0 || (d > 0 && e.numel > INT64_MAX / d)) { err = e.name + ": bad shape"; return false; }
        e.numel *= d;
      }
      if (lo < 0 || hi < lo || (uint64_t)hi > data_bytes) { err = e.name + ": data_offsets outside the file"; return false; }
      e.offset = base + (size_t)lo;
      e.nbytes = (size_t)(hi - lo);
      if (e.nbytes != (size_t)e.numel * ELEM[e.elem].bytes) { err = e.name + ": byte range does not match shape and dtype"; return false; }
      im.tensors.push_back(std::move(e));
    } while (j.ok && j.eat(','));
  }
  if (!j.ok || !j.eat('}')) { err = "malformed safetensors header"; return false; }
  return true;
}

// ------------------------------------------------------------------------------------------------ block decoders (ggml layouts)
inline void k4_scale_min(int j, const uint8_t* q, uint8_t& d, uint8_t& m) {
  if (j < 4) { d = q[j] & 63; m = q[j + 4] & 63; }
  else { d = (uint8_t)((q[j + 4] & 0xF) | ((q[j - 4] >> 6) << 4)); m = (uint8_t)((q[j + 4] >> 4) | ((q[j] >> 6) << 4)); }
}

void decode_blocks(int elem, const uint8_t* src, int64_t nblocks, float* y) {
  for (int64_t b = 0; b < nblocks; ++b) {
    const uint8_t* x = src + b * ELEM[elem].bytes;
    switch (elem) {
      case E_Q4_0: {
        const float d = half_to_float(rd16(x));
        for (int i = 0; i < 16; ++i) { y[i] = ((x[2 + i] & 15) - 8) * d; y[i + 16] = ((x[2 + i] >> 4) - 8) * d; }
        y += 32; break;
      }
      case E_Q4_1: {
        const float d = half_to_float(rd16(x)), m = half_to_float(rd16(x + 2));
        for (int i = 0; i < 16; ++i) { y[i] = (x[4 + i] & 15) * d + m; y[i + 16] = (x[4 + i] >> 4) * d + m; }
        y += 32; break;
      }
      case E_Q5_0: {
        const float d = half_to_float(rd16(x));
        const uint32_t qh = rd32(x + 2);
        for (int i = 0; i < 16; ++i) {
          const int h0 = ((qh >> i) << 4) & 16, h1 = (qh >> (i + 12)) & 16;
          y[i] = (((x[6 + i] & 15) | h0) - 16) * d;
          y[i + 16] = (((x[6 + i] >> 4) | h1) - 16) * d;
        }
        y += 32; break;
      }
      case E_Q5_1: {
        const float d = half_to_float(rd16(x)), m = half_to_float(rd16(x + 2));
        const uint32_t qh = rd32(x + 4);
        for (int i = 0; i < 16; ++i) {
          const int h0 = ((qh >> i) << 4) & 16, h1 = (qh >> (i + 12)) & 16;
          y[i] = ((x[8 + i] & 15) | h0) * d + m;
          y[i + 16] = ((x[8 + i] >> 4) | h1) * d + m;
        }
        y += 32; break;
      }
      case E_Q8_0: {
        const float d = half_to_float(rd16(x));
        for (int i = 0; i < 32; ++i) y[i] = (int8_t)x[2 + i] * d;
        y += 32; break;
      }
      case E_Q8_1: {  // d, sum (unused for decoding), 32 int8
        const float d = half_to_float(rd16(x));
        for (int i = 0; i < 32; ++i) y[i] = (int8_t)x[4 + i] * d;
        y += 32; break;
      }
      case E_Q2_K: {  // scales[16] (4-bit scale | 4-bit min), qs[64], d, dmin
        const uint8_t* sc = x; const uint8_t* q = x + 16;
        const float d = half_to_float(rd16(x + 80)), dmin = half_to_float(rd16(x + 82));
        int is = 0;
        for (int n = 0; n < 256; n += 128, q += 32)
          for (int j = 0, shift = 0; j < 4; ++j, shift += 2)
            for (int half = 0; half < 2; ++half) {
              const uint8_t s = sc[is++];
              const float dl = d * (s & 15), ml = dmin * (s >> 4);
              for (int l = 0; l < 16; ++l) *y++ = dl * ((q[l + 16 * half] >> shift) & 3) - ml;
            }
        break;
      }
      case E_Q3_K: {  // hmask[32], qs[64], scales[12] (6-bit, packed), d
        const uint8_t* hm = x; const uint8_t* q = x + 32;
        const float d_all = half_to_float(rd16(x + 108));
        uint32_t aux[4];
        memcpy(aux, x + 96, 12);
        const uint32_t k1 = 0x03030303u, k2 = 0x0f0f0f0fu, tmp = aux[2];
        aux[2] = ((aux[0] >> 4) & k2) | (((tmp >> 4) & k1) << 4);
        aux[3] = ((aux[1] >> 4) & k2) | (((tmp >> 6) & k1) << 4);
        aux[0] = (aux[0] & k2) | (((tmp >> 0) & k1) << 4);
        aux[1] = (aux[1] & k2) | (((tmp >> 2) & k1) << 4);
        int8_t scales[16];
        memcpy(scales, aux, 16);
        int is = 0;
        uint8_t m = 1;
        for (int n = 0; n < 256; n += 128, q += 32)
          for (int j = 0, shift = 0; j < 4; ++j, shift += 2, m <<= 1)
            for (int half = 0; half < 2; ++half) {
              const float dl = d_all * (scales[is++] - 32);
              for (int l = 0; l < 16; ++l) {
                const int i = l + 16 * half;
                *y++ = dl * ((int)((q[i] >> shift) & 3) - ((hm[i] & m) ? 0 : 4));
              }
            }
        break;
      }
      case E_Q4_K: {  // d, dmin, scales[12], qs[128]
        const float d = half_to_float(rd16(x)), dmin = half_to_float(rd16(x + 2));
        const uint8_t* sc = x + 4; const uint8_t* q = x + 16;
        for (int j = 0, is = 0; j < 256; j += 64, q += 32, is += 2) {
          uint8_t s, m;
          k4_scale_min(is, sc, s, m);
          const float d1 = d * s, m1 = dmin * m;
          k4_scale_min(is + 1, sc, s, m);
          const float d2 = d * s, m2 = dmin * m;
          for (int l = 0; l < 32; ++l) *y++ = d1 * (q[l] & 15) - m1;
          for (int l = 0; l < 32; ++l) *y++ = d2 * (q[l] >> 4) - m2;
        }
        break;
      }
      case E_Q5_K: {  // d, dmin, scales[12], qh[32], qs[128]
        const float d = half_to_float(rd16(x)), dmin = half_to_float(rd16(x + 2));
        const uint8_t* sc = x + 4; const uint8_t* qh = x + 16; const uint8_t* ql = x + 48;
        uint8_t u1 = 1, u2 = 2;
        for (int j = 0, is = 0; j < 256; j += 64, ql += 32, is += 2, u1 <<= 2, u2 <<= 2) {
          uint8_t s, m;
          k4_scale_min(is, sc, s, m);
          const float d1 = d * s, m1 = dmin * m;
          k4_scale_min(is + 1, sc, s, m);
          const float d2 = d * s, m2 = dmin * m;
          for (int l = 0; l < 32; ++l) *y++ = d1 * ((ql[l] & 15) + ((qh[l] & u1) ? 16 : 0)) - m1;
          for (int l = 0; l < 32; ++l) *y++ = d2 * ((ql[l] >> 4) + ((qh[l] & u2) ? 16 : 0)) - m2;
        }
        break;
      }
      case E_Q6_K: {  // ql[128], qh[64], scales[16] (int8), d
        const uint8_t* ql = x; const uint8_t* qh = x + 128; const int8_t* sc = (const int8_t*)(x + 192);
        const float d = half_to_float(rd16(x + 208));
        for (int n = 0; n < 256; n += 128, y += 128, ql += 64, qh += 32, sc += 8)
          for (int l = 0; l < 32; ++l) {
            const int is = l / 16;
            const int q1 = (int)((ql[l] & 15) | (((qh[l] >> 0) & 3) << 4)) - 32;
            const int q2 = (int)((ql[l + 32] & 15) | (((qh[l] >> 2) & 3) << 4)) - 32;
            const int q3 = (int)((ql[l] >> 4) | (((qh[l] >> 4) & 3) << 4)) - 32;
            const int q4 = (int)((ql[l + 32] >> 4) | (((qh[l] >> 6) & 3) << 4)) - 32;
            y[l] = d * sc[is] * q1;
            y[l + 32] = d * sc[is + 2] * q2;
            y[l + 64] = d * sc[is + 4] * q3;
            y[l + 96] = d * sc[is + 6] * q4;
          }
        break;
      }
      default: break;
    }
  }
}

void decode_plain(int elem, const uint8_t* src, int64_t n, float* y) {
  switch (elem) {
    case E_F32: memcpy(y, src, (size_t)n * 4); break;
    case E_F16: for (int64_t i = 0; i < n; ++i) y[i] = half_to_float(rd16(src + 2 * i)); break;
    case E_BF16: for (int64_t i = 0; i < n; ++i) y[i] = bf16_to_float(rd16(src + 2 * i)); break;
    case E_F64: for (int64_t i = 0; i < n; ++i) { double v; memcpy(&v, src + 8 * i, 8); y[i] = (float)v; } break;
    case E_I8: for (int64_t i = 0; i < n; ++i) y[i] = (float)(int8_t)src[i]; break;
    case E_U8: for (int64_t i = 0; i < n; ++i) y[i] = (float)src[i]; break;
    case E_BOOL: for (int64_t i = 0; i < n; ++i) y[i] = src[i] ? 1.f : 0.f; break;
    case E_I16: for (int64_t i = 0; i < n; ++i) y[i] = (float)(int16_t)rd16(src + 2 * i); break;
    case E_I32: for (int64_t i = 0; i < n; ++i) y[i] = (float)(int32_t)rd32(src + 4 * i); break;
    case E_I64: for (int64_t i = 0; i < n; ++i) { int64_t v; memcpy(&v, src + 8 * i, 8); y[i] = (float)v; } break;
    case E_F8E4M3: for (int64_t i = 0; i < n; ++i) y[i] = e4m3_to_float(src[i]); break;
    case E_F8E5M2: for (int64_t i = 0; i < n; ++i) y[i] = e5m2_to_float(src[i]); break;
    default: break;
  }
}

void set_err(char* err, int errlen, const std::string& msg) {
  if (err && errlen > 0) snprintf(err, (size_t)errlen, "%s", msg.c_str());
}

}  // namespace

extern "C" {

// kind: 0 = decide by content (GGUF magic, else safetensors), 1 = GGUF, 2 = safetensors. Returns a handle or null
// (the reason is written to err).
void* inv_import_open(const char* path, int kind, char* err, int errlen) {
  auto* im = new Importer();
  std::string e;
  if (!im->map.open(path, e)) { set_err(err, errlen, e); delete im; return nullptr; }
  if (kind == 0) kind = (im->map.n >= 4 && memcmp(im->map.p, "GGUF", 4) == 0) ? KIND_GGUF : KIND_SAFETENSORS;
  im->kind = kind;
  const bool ok = kind == KIND_GGUF ? parse_gguf(*im, e) : kind == KIND_SAFETENSORS ? parse_safetensors(*im, e) : false;
  if (!ok) { set_err(err, errlen, e.empty() ? "unknown container kind" : e); delete im; return nullptr; }
  return im;
}
void inv_import_close(void* h) { delete (Importer*)h; }
int inv_import_kind(void* h) { return ((Importer*)h)->kind; }
int inv_import_count(void* h) { return (int)((Importer*)h)->tensors.size(); }
const char* inv_import_meta(void* h) { return ((Importer*)h)->meta.c_str(); }
const char* inv_import_name(void* h, int i) {
  auto* im = (Importer*)h;
  return i >= 0 && i < (int)im->tensors.size() ? im->tensors[i].name.c_str() : "";
}
long inv_import_numel(void* h, int i) {
  auto* im = (Importer*)h;
  return i >= 0 && i < (int)im->tensors.size() ? (long)im->tensors[i].numel : -1;
}
int inv_import_ndim(void* h, int i) {
  auto* im = (Importer*)h;
  return i >= 0 && i < (int)im->tensors.size() ? (int)im->tensors[i].dims.size() : -1;
}
long inv_import_dim(void* h, int i, int d) {
  auto* im = (Importer*)h;
  if (i < 0 || i >= (int)im->tensors.size() || d < 0 || d >= (int)im->tensors[i].dims.size()) return -1;
  return (long)im->tensors[i].dims[d];
}
long inv_import_stored_bytes(void* h, int i) {
  auto* im = (Importer*)h;
  return i >= 0 && i < (int)im->tensors.size() ? (long)im->tensors[i].nbytes : -1;
}
// Decode tensor i into out (numel floats). 0 on success.
int inv_import_read_f32(void* h, int i, float* out) {
  auto* im = (Importer*)h;
  if (i < 0 || i >= (int)im->tensors.size() || out == nullptr) return -1;
  const TensorEntry& e = im->tensors[i];
  const uint8_t* src = im->map.p + e.offset;
  if (ELEM[e.elem].block == 1) decode_plain(e.elem, src, e.numel, out);
  else decode_blocks(e.elem, src, e.numel / ELEM[e.elem].block, out);
  return 0;
}

// Raw files. dtype: 0 fp32, 1 fp16, 2 bf16, 3 fp8-e4m3, 4 fp8-e5m2. Returns the number of values, or -1.
long inv_import_raw_count(const char* path, int dtype) {
  struct stat st;
  if (dtype < 0 || dtype > 4 || stat(path, &st) != 0) return -1;
  static const int bytes[5] = {4, 2, 2, 1, 1};
  return (long)(st.st_size / bytes[dtype]);
}
int inv_import_raw_f32(const char* path, int dtype, float* out, long n) {
  if (dtype < 0 || dtype > 4 || n < 0) return -1;
  Mapping m;
  std::string e;
  if (n == 0) return 0;
  if (!m.open(path, e)) return -2;
  static const int elem[5] = {E_F32, E_F16, E_BF16, E_F8E4M3, E_F8E5M2};
  if ((size_t)n * ELEM[elem[dtype]].bytes > m.n) return -3;
  decode_plain(elem[dtype], m.p, n, out);
  return 0;
}

}  // extern "C"
