// Block codec for the 15 .oil wire formats. The arithmetic (level tables, rounding, slot
// positions, tail rules, bit order) follows the reference's canonical codec
// (src/block_codec.cpp:14-23 tables, :122-126 slots, :157-182 lattice, :189-364 grouped lattice,
// :406-570 sign / sparse formats) so that payloads are byte-identical; the code is organised as
// one small encoder/decoder per payload family on top of a shared LSB-first bit stream.
#include "oil_codec.h"

#include <algorithm>
#include <cmath>
#include <cstring>

namespace inv {

const float kLevels2[4] = {-1.5104f, -0.4528f, 0.4528f, 1.5104f};
const float kLevels4[16] = {-2.7178f, -2.0522f, -1.5995f, -1.2392f, -0.9275f, -0.6508f, -0.3976f, -0.1260f,
                            0.1260f,  0.3976f,  0.6508f,  0.9275f,  1.2392f,  1.5995f,  2.0522f,  2.7178f};

namespace {

struct FormatInfo {
  const char* name;
  float bpw;
};
const FormatInfo kInfo[FORMAT_COUNT] = {
    {"OIL1", 1.0f},      {"SPARK_Q0", 1.5f},  {"OIL2", 2.0f},       {"OIL4", 4.0f},          {"OIL8", 8.0f},
    {"OIL16", 16.0f},    {"OIL32", 32.0f},    {"OIL1_GRP", 1.0f},   {"SPARK_Q0_GRP", 1.5f},  {"OIL2_GRP", 2.5f},
    {"OIL4_GRP", 4.5f},  {"OIL8_GRP", 8.5f},  {"OIL16_GRP", 16.0f}, {"SPARK_SPARSE", 2.0f},  {"SPARK_SPARSE_GRP", 2.0f},
};

constexpr int kGroup = 64;     // window of the *_GRP lattice formats
constexpr int kSubBlock = 32;  // window of OIL1 means and SPARK_Q0 scales

// LSB-first bit stream over a pre-sized byte vector. Writes past the end are dropped and reads
// past the end return zero bits, which is what gives tiny tail blocks their defined behaviour.
class BitSink {
 public:
  explicit BitSink(std::vector<uint8_t>& b) : buf_(b) {}
  void put(uint32_t v, int nbits) {
    for (int i = 0; i < nbits; ++i, ++pos_) {
      if (pos_ >= buf_.size() * 8) return;
      if ((v >> i) & 1u) buf_[pos_ >> 3] |= (uint8_t)(1u << (pos_ & 7));
    }
  }
 private:
  std::vector<uint8_t>& buf_;
  size_t pos_ = 0;
};
class BitSource {
 public:
  BitSource(const uint8_t* p, size_t n) : p_(p), nbits_(n * 8) {}
  uint32_t get(int nbits) {
    uint32_t v = 0;
    for (int i = 0; i < nbits; ++i, ++pos_) {
      if (pos_ >= nbits_) break;
      if ((p_[pos_ >> 3] >> (pos_ & 7)) & 1u) v |= 1u << i;
    }
    return v;
  }
 private:
  const uint8_t* p_;
  size_t nbits_, pos_ = 0;
};

// A position is a "slot" (skipped on encode, zero on decode) when the running count
// floor((i+1)*slots/n) advances at i. The slots of a block pay for its 16-bit scale.
inline bool slot_at(int64_t i, int64_t n, int slots) {
  if (slots <= 0 || n <= 0) return false;
  return ((i + 1) * slots) / n != (i * slots) / n;
}

inline float lattice_value(int bits, uint32_t idx) {
  if (bits == 2) return kLevels2[idx > 3 ? 3 : idx];
  if (bits == 4) return kLevels4[idx > 15 ? 15 : idx];
  return level8(idx);
}
inline uint32_t lattice_index(float v, int bits) {
  if (bits == 8) {
    const float c = std::max(-8.0f, std::min(8.0f, v));
    return (uint32_t)std::lround((c + 8.0f) * 255.0f / 16.0f);
  }
  const int count = bits == 2 ? 4 : 16;
  uint32_t best = 0;
  float best_d = std::fabs(v - lattice_value(bits, 0));
  for (int i = 1; i < count; ++i) {
    const float d = std::fabs(v - lattice_value(bits, (uint32_t)i));
    if (d < best_d) {
      best_d = d;
      best = (uint32_t)i;
    }
  }
  return best;
}
// round(t * 255) with the reference's conversion: a negative result wraps and is clamped to 255.
inline uint32_t range_index(float t, float mul) {
  const uint32_t idx = (uint32_t)std::lround(t * mul);
  return idx > 255u ? 255u : idx;
}
inline float rms(const float* w, int n) {
  if (n <= 0) return 0.0f;
  double s = 0.0;
  for (int i = 0; i < n; ++i) s += (double)w[i] * w[i];
  return (float)std::sqrt(s / (double)n);
}
inline void put_u16le(std::vector<uint8_t>& v, size_t at, uint16_t h) {
  v[at] = (uint8_t)(h & 0xFF);
  v[at + 1] = (uint8_t)(h >> 8);
}
inline uint16_t get_u16le(const uint8_t* p) { return (uint16_t)p[0] | ((uint16_t)p[1] << 8); }

// ---------------------------------------------------------------- OIL8 / OIL4 / OIL2
void encode_lattice(const float* w, int n, int bits, std::vector<uint8_t>& out) {
  const int slots = 16 / bits;
  out.assign(((size_t)bits * (size_t)n + 7) / 8, 0);
  BitSink bs(out);
  const float scale = rms(w, n);
  bs.put(f32_to_f16(scale), 16);
  const bool dead = scale <= 1e-12f;
  for (int i = 0; i < n; ++i) {
    if (slot_at(i, n, slots)) continue;
    bs.put(lattice_index(dead ? 0.0f : w[i] / scale, bits), bits);
  }
}
void decode_lattice(const uint8_t* p, size_t size, int n, int bits, float* out) {
  const int slots = 16 / bits;
  BitSource src(p, size);
  const float scale = f16_to_f32((uint16_t)src.get(16));
  for (int i = 0; i < n; ++i) out[i] = slot_at(i, n, slots) ? 0.0f : lattice_value(bits, src.get(bits)) * scale;
}

// ---------------------------------------------------------------- OIL8_GRP / OIL4_GRP / OIL2_GRP
// Full 64-weight groups carry fp16 zero-point + fp16 scale. A block shorter than one group carries
// a scale only (n >= 8) or nothing (n < 8); a partial tail after full groups reuses the last header.
struct GroupParams {
  float zp, scale;
};
inline GroupParams fit_group(const float* w, int count, bool is8) {
  GroupParams g;
  if (is8) {
    float lo = w[0], hi = w[0];
    for (int i = 1; i < count; ++i) {
      if (w[i] < lo) lo = w[i];
      if (w[i] > hi) hi = w[i];
    }
    g.zp = lo;
    g.scale = hi - lo;
  } else {
    double mu = 0.0, ss = 0.0;
    for (int i = 0; i < count; ++i) mu += w[i];
    mu /= (double)count;
    for (int i = 0; i < count; ++i) {
      const double d = (double)w[i] - mu;
      ss += d * d;
    }
    g.zp = (float)mu;
    g.scale = ss > 0.0 ? (float)std::sqrt(ss / (double)count) : 0.0f;
  }
  return g;
}
inline void put_grouped(BitSink& bs, float w, const GroupParams& g, int bits, bool is8) {
  if (g.scale == 0.0f) {
    bs.put(0, bits);
  } else if (is8) {
    bs.put(range_index((w - g.zp) / g.scale, 255.0f), 8);
  } else {
    bs.put(lattice_index((float)(((double)w - g.zp) / (double)g.scale), bits), bits);
  }
}
void encode_grouped(int bits, const float* w, int n, std::vector<uint8_t>& out) {
  const bool is8 = bits == 8;
  const int nfull = n / kGroup;
  const size_t header_bits = nfull == 0 ? (n < 8 ? 0 : 16) : (size_t)nfull * 32;
  out.assign((header_bits + (size_t)n * (size_t)bits + 7) / 8, 0);
  BitSink bs(out);
  GroupParams last{0.0f, 1.0f};
  for (int g = 0; g < nfull; ++g) {
    const float* gw = w + g * kGroup;
    last = fit_group(gw, kGroup, is8);
    bs.put(f32_to_f16(last.zp), 16);
    bs.put(f32_to_f16(last.scale), 16);
    for (int i = 0; i < kGroup; ++i) put_grouped(bs, gw[i], last, bits, is8);
  }
  const int tail0 = nfull * kGroup;
  if (tail0 == n) return;
  if (nfull > 0) {
    for (int i = tail0; i < n; ++i) put_grouped(bs, w[i], last, bits, is8);
    return;
  }
  if (n < 8) {  // headerless: implicit scale 1, zero-point 0
    for (int i = 0; i < n; ++i) {
      if (is8) bs.put(range_index(w[i] + 1.0f, 127.5f), 8);
      else bs.put(lattice_index(w[i], bits), bits);
    }
    return;
  }
  float scale;
  if (is8) {
    scale = std::fabs(w[0]);
    for (int i = 1; i < n; ++i) scale = std::max(scale, std::fabs(w[i]));
  } else {
    double ss = 0.0;
    for (int i = 0; i < n; ++i) ss += (double)w[i] * (double)w[i];
    scale = ss > 0.0 ? (float)std::sqrt(ss / (double)n) : 0.0f;
  }
  bs.put(f32_to_f16(scale), 16);
  if (scale == 0.0f) return;  // all index bits stay zero
  for (int i = 0; i < n; ++i) {
    if (is8) bs.put(range_index(w[i] / scale + 1.0f, 127.5f), 8);
    else bs.put(lattice_index(w[i] / scale, bits), bits);
  }
}
void decode_grouped(const uint8_t* p, size_t size, int bits, int n, float* out) {
  const bool is8 = bits == 8;
  BitSource src(p, size);
  const int nfull = n / kGroup;
  GroupParams last{0.0f, 1.0f};
  auto one = [&](const GroupParams& g) -> float {
    const uint32_t idx = src.get(bits);
    if (g.scale == 0.0f) return g.zp;
    return is8 ? g.zp + (float)idx / 255.0f * g.scale : lattice_value(bits, idx) * g.scale + g.zp;
  };
  for (int g = 0; g < nfull; ++g) {
    last.zp = f16_to_f32((uint16_t)src.get(16));
    last.scale = f16_to_f32((uint16_t)src.get(16));
    for (int i = 0; i < kGroup; ++i) out[g * kGroup + i] = one(last);
  }
  const int tail0 = nfull * kGroup;
  if (tail0 == n) return;
  if (nfull > 0) {
    for (int i = tail0; i < n; ++i) out[i] = one(last);
    return;
  }
  if (n < 8) {
    for (int i = 0; i < n; ++i) out[i] = is8 ? (float)src.get(8) / 127.5f - 1.0f : lattice_value(bits, src.get(bits));
    return;
  }
  const float scale = f16_to_f32((uint16_t)src.get(16));
  if (scale == 0.0f) {
    for (int i = 0; i < n; ++i) out[i] = 0.0f;
    return;
  }
  for (int i = 0; i < n; ++i)
    out[i] = is8 ? ((float)src.get(8) / 127.5f - 1.0f) * scale : lattice_value(bits, src.get(bits)) * scale;
}

// ---------------------------------------------------------------- sign formats
inline uint32_t sign_bit(float v) { return v >= 0.0f ? 1u : 0u; }

void encode_signs_only(const float* w, int n, std::vector<uint8_t>& out) {
  out.assign((size_t)(n + 7) / 8, 0);
  BitSink bs(out);
  for (int i = 0; i < n; ++i) bs.put(sign_bit(w[i]), 1);
}
void decode_signs_only(const uint8_t* p, size_t size, int n, float* out) {
  BitSource src(p, size);
  for (int i = 0; i < n; ++i) out[i] = src.get(1) ? 1.0f : -1.0f;
}

// ---------------------------------------------------------------- sparse formats
struct Ranked {
  float mag;
  int idx;
};
// Largest `keep` magnitudes, descending. Ties are left to std::partial_sort on the index-ordered
// input, which is what the reference does, so equal magnitudes come out in the same order as there
// when both are built against the same standard library.
void top_magnitudes(const float* w, int n, int keep, std::vector<Ranked>& r) {
  r.resize((size_t)n);
  for (int i = 0; i < n; ++i) r[(size_t)i] = {std::fabs(w[i]), i};
  if (keep > 0)
    std::partial_sort(r.begin(), r.begin() + keep, r.end(),
                      [](const Ranked& a, const Ranked& b) { return a.mag > b.mag; });
}
inline void put_record(std::vector<uint8_t>& out, int slot, int idx, float normalised) {
  int q = (int)std::lround(normalised * 127.0f);
  q = std::max(-127, std::min(127, q));
  const size_t at = 4 + (size_t)slot * 3;
  put_u16le(out, at, (uint16_t)idx);
  out[at + 2] = (uint8_t)q;
}

}  // namespace

const char* format_name(int fmt) { return (fmt >= 0 && fmt < FORMAT_COUNT) ? kInfo[fmt].name : "unknown"; }
int format_from_name(const std::string& name) {
  std::string u;
  for (char c : name) u.push_back((char)std::toupper((unsigned char)c));
  for (int i = 0; i < FORMAT_COUNT; ++i)
    if (u == kInfo[i].name) return i;
  return -1;
}
float format_bpw(int fmt) { return (fmt >= 0 && fmt < FORMAT_COUNT) ? kInfo[fmt].bpw : 0.0f; }
size_t claimed_bytes(int fmt, uint32_t n) { return (size_t)std::ceil(format_bpw(fmt) * (float)n / 8.0f); }

// fp32 -> fp16, round to nearest even, subnormals kept, magnitudes below 2^-24 flushed to zero,
// everything with an exponent above 15 (inf and NaN included) becomes infinity.
uint16_t f32_to_f16(float v) {
  uint32_t u;
  std::memcpy(&u, &v, 4);
  const uint16_t sign = (uint16_t)((u >> 16) & 0x8000u);
  const int e = (int)((u >> 23) & 0xFF) - 127;
  const uint32_t frac = u & 0x7FFFFFu;
  if (e > 15) return sign | 0x7C00u;
  if (e >= -14) {
    uint32_t m = (frac >> 13) | 0x400u;  // 11-bit significand
    const uint32_t rest = frac & 0x1FFFu;
    if (rest > 0x1000u || (rest == 0x1000u && (m & 1u))) ++m;
    int eh = e;
    if (m >= 0x800u) {
      m >>= 1;
      if (++eh > 15) return sign | 0x7C00u;
    }
    return (uint16_t)(sign | ((uint32_t)(eh + 15) << 10) | (m & 0x3FFu));
  }
  if (e < -24) return sign;
  const uint32_t full = frac | 0x800000u;
  const int shift = -e - 1;  // 14 .. 23
  uint32_t m = full >> shift;
  const uint32_t half = 1u << (shift - 1);
  const uint32_t rest = full & ((1u << shift) - 1u);
  if (rest > half || (rest == half && (m & 1u))) ++m;
  return (uint16_t)(sign | m);  // m == 0x400 is the smallest normal, which is the right encoding
}
float f16_to_f32(uint16_t h) {
  const uint32_t sign = (uint32_t)(h & 0x8000u) << 16;
  const int e = (h >> 10) & 0x1F;
  uint32_t m = h & 0x3FFu;
  uint32_t u;
  if (e == 0) {
    if (m == 0) {
      u = sign;
    } else {
      int ex = -14;
      while (!(m & 0x400u)) {
        m <<= 1;
        --ex;
      }
      u = sign | ((uint32_t)(ex + 127) << 23) | ((m & 0x3FFu) << 13);
    }
  } else if (e == 31) {
    u = sign | 0x7F800000u | (m << 13);
  } else {
    u = sign | ((uint32_t)(e - 15 + 127) << 23) | (m << 13);
  }
  float f;
  std::memcpy(&f, &u, 4);
  return f;
}

bool encode_block(int fmt, const float* w, int n, std::vector<uint8_t>& idx, std::vector<uint8_t>& cb) {
  if (!w || n <= 0) return false;
  idx.clear();
  cb.clear();
  switch (fmt) {
    case OIL32:
      idx.resize((size_t)n * 4);
      std::memcpy(idx.data(), w, (size_t)n * 4);
      return true;
    case OIL16:
    case OIL16_GRP:
      idx.resize((size_t)n * 2);
      for (int i = 0; i < n; ++i) put_u16le(idx, (size_t)i * 2, f32_to_f16(w[i]));
      return true;
    case OIL8: encode_lattice(w, n, 8, idx); return true;
    case OIL4: encode_lattice(w, n, 4, idx); return true;
    case OIL2: encode_lattice(w, n, 2, idx); return true;
    case OIL8_GRP: encode_grouped(8, w, n, idx); return true;
    case OIL4_GRP: encode_grouped(4, w, n, idx); return true;
    case OIL2_GRP: encode_grouped(2, w, n, idx); return true;
    case OIL1: {  // fp16 mean of every 32 weights, in the codebook channel
      const int nb = (n + kSubBlock - 1) / kSubBlock;
      cb.resize((size_t)nb * 2);
      for (int b = 0; b < nb; ++b) {
        const int lo = b * kSubBlock, hi = std::min(lo + kSubBlock, n);
        double s = 0.0;
        for (int i = lo; i < hi; ++i) s += w[i];
        put_u16le(cb, (size_t)b * 2, f32_to_f16((float)(s / (double)(hi - lo))));
      }
      return true;
    }
    case OIL1_GRP: {
      if (n < 32) {
        encode_signs_only(w, n, idx);
        return true;
      }
      idx.assign((size_t)(n + 7) / 8, 0);
      BitSink bs(idx);
      bs.put(f32_to_f16(rms(w, n)), 16);
      for (int i = 0; i < n; ++i)
        if (!slot_at(i, n, 16)) bs.put(sign_bit(w[i]), 1);
      return true;
    }
    case SPARK_Q0: {
      idx.assign(((size_t)n * 3 + 15) / 16, 0);
      BitSink bs(idx);
      for (int lo = 0; lo < n; lo += kSubBlock) {
        const int hi = std::min(lo + kSubBlock, n);
        if (hi - lo == kSubBlock) bs.put(f32_to_f16(rms(w + lo, kSubBlock)), 16);
        for (int i = lo; i < hi; ++i) bs.put(sign_bit(w[i]), 1);
      }
      return true;
    }
    case SPARK_Q0_GRP: {
      if (n < 32) {
        encode_signs_only(w, n, idx);
        return true;
      }
      idx.assign((size_t)(n * 3 + 15) / 16, 0);
      BitSink bs(idx);
      const float scale = rms(w, n);
      bs.put(f32_to_f16(scale), 16);
      for (int i = 0; i < n; ++i) bs.put(sign_bit(w[i]), 1);
      const int refined = std::max(0, n / 2 - 16);
      const float thr = scale * 1.23f;
      for (int i = 0; i < n; ++i)
        if (slot_at(i, n, refined)) bs.put(std::fabs(w[i]) > thr ? 1u : 0u, 1);
      return true;
    }
    case SPARK_SPARSE: {
      const size_t budget = (size_t)n / 4;
      if (budget < 4) return true;
      const int keep = std::min(20, (int)((budget - 4) / 3));
      float scale = 0.0f;
      for (int i = 0; i < n; ++i) scale = std::max(scale, std::fabs(w[i]));
      if (scale <= 1e-12f) {
        idx.assign(4, 0);
        return true;
      }
      std::vector<Ranked> r;
      top_magnitudes(w, n, keep, r);
      idx.assign((size_t)4 + (size_t)keep * 3, 0);
      std::memcpy(idx.data(), &scale, 4);
      for (int i = 0; i < keep; ++i) put_record(idx, i, r[(size_t)i].idx, w[r[(size_t)i].idx] / scale);
      return true;
    }
    case SPARK_SPARSE_GRP: {
      const size_t budget = (size_t)n / 4;
      if (budget < 8) return true;
      const int keep = (int)((budget - 4) / 3);
      if (keep <= 0) return true;
      const int half = n / 2;
      float s0 = 0.0f, s1 = 0.0f;
      for (int i = 0; i < n; ++i) {
        const float a = std::fabs(w[i]);
        if (i < half) s0 = std::max(s0, a);
        else s1 = std::max(s1, a);
      }
      if (s0 <= 1e-12f) s0 = 1.0f;
      if (s1 <= 1e-12f) s1 = 1.0f;
      std::vector<Ranked> r;
      top_magnitudes(w, n, keep, r);
      idx.assign((size_t)4 + (size_t)keep * 3, 0);
      put_u16le(idx, 0, f32_to_f16(s0));
      put_u16le(idx, 2, f32_to_f16(s1));
      for (int i = 0; i < keep; ++i) {
        const int at = r[(size_t)i].idx;
        put_record(idx, i, at, w[at] / (at < half ? s0 : s1));
      }
      return true;
    }
    default:
      return false;
  }
}

void decode_block(int fmt, const uint8_t* idx, size_t idx_bytes, const uint8_t* cb, size_t cb_bytes, uint32_t nw, float* out) {
  if (!out || nw == 0) return;
  std::fill(out, out + nw, 0.0f);
  const int n = (int)std::min<uint32_t>(nw, 1u << 24);
  switch (fmt) {
    case OIL32:
      if (idx_bytes >= (size_t)n * 4) std::memcpy(out, idx, (size_t)n * 4);
      return;
    case OIL16:
    case OIL16_GRP:
      for (int i = 0; i < n && (size_t)i * 2 + 1 < idx_bytes; ++i) out[i] = f16_to_f32(get_u16le(idx + (size_t)i * 2));
      return;
    case OIL8: decode_lattice(idx, idx_bytes, n, 8, out); return;
    case OIL4: decode_lattice(idx, idx_bytes, n, 4, out); return;
    case OIL2: decode_lattice(idx, idx_bytes, n, 2, out); return;
    case OIL8_GRP: decode_grouped(idx, idx_bytes, 8, n, out); return;
    case OIL4_GRP: decode_grouped(idx, idx_bytes, 4, n, out); return;
    case OIL2_GRP: decode_grouped(idx, idx_bytes, 2, n, out); return;
    case OIL1:
      for (int b = 0; b * kSubBlock < n && (size_t)b * 2 + 1 < cb_bytes; ++b) {
        const float mean = f16_to_f32(get_u16le(cb + (size_t)b * 2));
        std::fill(out + b * kSubBlock, out + std::min((b + 1) * kSubBlock, n), mean);
      }
      return;
    case OIL1_GRP: {
      if (n < 32) {
        decode_signs_only(idx, idx_bytes, n, out);
        return;
      }
      BitSource src(idx, idx_bytes);
      const float scale = f16_to_f32((uint16_t)src.get(16));
      for (int i = 0; i < n; ++i) out[i] = slot_at(i, n, 16) ? 0.0f : (src.get(1) ? scale : -scale);
      return;
    }
    case SPARK_Q0: {
      BitSource src(idx, idx_bytes);
      for (int lo = 0; lo < n; lo += kSubBlock) {
        const int hi = std::min(lo + kSubBlock, n);
        const float scale = (hi - lo == kSubBlock) ? f16_to_f32((uint16_t)src.get(16)) : 1.0f;
        for (int i = lo; i < hi; ++i) out[i] = src.get(1) ? scale : -scale;
      }
      return;
    }
    case SPARK_Q0_GRP: {
      if (n < 32) {
        decode_signs_only(idx, idx_bytes, n, out);
        return;
      }
      BitSource src(idx, idx_bytes);
      const float scale = f16_to_f32((uint16_t)src.get(16));
      const int refined = std::max(0, n / 2 - 16);
      std::vector<uint8_t> neg((size_t)n);
      for (int i = 0; i < n; ++i) neg[(size_t)i] = src.get(1) ? 0 : 1;
      for (int i = 0; i < n; ++i) {
        float mag = scale;
        if (slot_at(i, n, refined)) mag = scale * (src.get(1) ? 1.893f : 0.567f);
        out[i] = neg[(size_t)i] ? -mag : mag;
      }
      return;
    }
    case SPARK_SPARSE: {
      if (idx_bytes < 4) return;
      float scale;
      std::memcpy(&scale, idx, 4);
      if (scale == 0.0f) return;
      for (size_t at = 4; at + 2 < idx_bytes; at += 3) {
        const uint32_t rel = get_u16le(idx + at);
        if (rel < (uint32_t)n) out[rel] = (float)(int8_t)idx[at + 2] / 127.0f * scale;
      }
      return;
    }
    case SPARK_SPARSE_GRP: {
      if (idx_bytes < 7) return;
      const float s0 = f16_to_f32(get_u16le(idx)), s1 = f16_to_f32(get_u16le(idx + 2));
      if (s0 == 0.0f && s1 == 0.0f) return;
      const int half = n / 2;
      for (size_t at = 4; at + 2 < idx_bytes; at += 3) {
        const uint32_t rel = get_u16le(idx + at);
        if (rel < (uint32_t)n) out[rel] = (float)(int8_t)idx[at + 2] / 127.0f * ((int)rel < half ? s0 : s1);
      }
      return;
    }
    default:
      return;
  }
}

}  // namespace inv
