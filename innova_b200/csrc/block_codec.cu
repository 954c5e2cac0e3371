// .oil wire-format block codec on the device: decode of all 15 formats (any block length) and encode of
// the dense formats for full 256-weight blocks, byte-identical to the host codec in csrc/host/oil_codec.cpp
// and therefore to the reference's quantize_block_all / dequantize_block_all (src/block_codec.cpp:368-720).
//
// Decode: one warp per block. Every format's bit stream has a closed-form bit position per element (the
// "slot" positions that pay for a block's header are floor(i*slots/n) steps), so the 32 lanes decode
// elements independently with unaligned LSB-first bit reads; the two sparse formats are a short serial
// scatter. A block is described by a 32-byte record (format, count, payload / codebook / output offsets),
// so a whole tensor, or a whole file, decodes in one launch straight into bf16 or fp32 device memory.
// Encode: one warp per full block; the statistics that feed rounding decisions (rms, group mean / deviation)
// are summed in the same order and precision as the host code (sequential fp64 in one lane) so the index
// bytes match bit for bit; indices are packed through shared memory with word-wide OR.
// Division and square root are the IEEE-rounded intrinsics: the file is compiled with fast-math like the
// rest of the library, and the approximate forms would move rounding boundaries.
#include "sm100_common.cuh"
#include "inv_api.h"

namespace inv {
namespace bc {

enum { OIL1 = 0, SPARK_Q0 = 1, OIL2 = 2, OIL4 = 3, OIL8 = 4, OIL16 = 5, OIL32 = 6, OIL1_GRP = 7, SPARK_Q0_GRP = 8, OIL2_GRP = 9,
       OIL4_GRP = 10, OIL8_GRP = 11, OIL16_GRP = 12, SPARK_SPARSE = 13, SPARK_SPARSE_GRP = 14 };

struct BlockDesc {          // 32 bytes
  uint64_t idx_off;         // payload offset in the byte buffer
  uint64_t out_off;         // first output element
  uint32_t idx_bytes;
  uint32_t cb_off_lo;       // codebook offset (low 32 bits; codebooks live in the first 4 GiB window given by cb_base)
  uint16_t cb_bytes;
  uint8_t fmt;
  uint8_t pad;
  uint32_t n;
};

__constant__ float kL2[4] = {-1.5104f, -0.4528f, 0.4528f, 1.5104f};
__constant__ float kL4[16] = {-2.7178f, -2.0522f, -1.5995f, -1.2392f, -0.9275f, -0.6508f, -0.3976f, -0.1260f,
                              0.1260f,  0.3976f,  0.6508f,  0.9275f,  1.2392f,  1.5995f,  2.0522f,  2.7178f};

__device__ __forceinline__ float level(int bits, uint32_t i) {
  if (bits == 2) return kL2[i & 3];
  if (bits == 4) return kL4[i & 15];
  return __fadd_rn(-8.0f, __fdiv_rn(__fmul_rn(16.0f, (float)(i > 255u ? 255u : i)), 255.0f));
}
__device__ __forceinline__ uint32_t nearest_level(float v, int bits) {
  if (bits == 8) {
    const float c = fmaxf(-8.0f, fminf(8.0f, v));
    return (uint32_t)lroundf(__fmul_rn(__fadd_rn(c, 8.0f), 255.0f) * 0.0625f);
  }
  const int count = bits == 2 ? 4 : 16;
  uint32_t best = 0;
  float bd = fabsf(__fsub_rn(v, level(bits, 0)));
  for (int i = 1; i < count; ++i) {
    const float d = fabsf(__fsub_rn(v, level(bits, i)));
    if (d < bd) { bd = d; best = i; }
  }
  return best;
}
__device__ __forceinline__ uint32_t range_index(float t, float mul) {
  const uint32_t idx = (uint32_t)lroundf(__fmul_rn(t, mul));
  return idx > 255u ? 255u : idx;
}
__device__ uint16_t f32_to_f16_wire(float v) {
  const uint32_t u = __float_as_uint(v);
  const uint16_t sign = (uint16_t)((u >> 16) & 0x8000u);
  const int e = (int)((u >> 23) & 0xFF) - 127;
  const uint32_t frac = u & 0x7FFFFFu;
  if (e > 15) return sign | 0x7C00u;
  if (e >= -14) {
    uint32_t m = (frac >> 13) | 0x400u;
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
  const int shift = -e - 1;
  uint32_t m = full >> shift;
  const uint32_t half = 1u << (shift - 1);
  const uint32_t rest = full & ((1u << shift) - 1u);
  if (rest > half || (rest == half && (m & 1u))) ++m;
  return (uint16_t)(sign | m);
}
__device__ float f16_to_f32_wire(uint32_t h) {
  const uint32_t sign = (h & 0x8000u) << 16;
  const int e = (h >> 10) & 0x1F;
  uint32_t m = h & 0x3FFu;
  if (e == 0) {
    if (m == 0) return __uint_as_float(sign);
    int ex = -14;
    while (!(m & 0x400u)) { m <<= 1; --ex; }
    return __uint_as_float(sign | ((uint32_t)(ex + 127) << 23) | ((m & 0x3FFu) << 13));
  }
  if (e == 31) return __uint_as_float(sign | 0x7F800000u | (m << 13));
  return __uint_as_float(sign | ((uint32_t)(e - 15 + 127) << 23) | (m << 13));
}

// LSB-first read of nbits (<= 16) at bit position pos; bits past the payload read as zero.
__device__ __forceinline__ uint32_t get_bits(const uint8_t* p, uint32_t size, uint32_t pos, int nbits) {
  const uint32_t byte = pos >> 3;
  uint32_t v = 0;
#pragma unroll
  for (int j = 0; j < 3; ++j)
    if (byte + j < size) v |= (uint32_t)p[byte + j] << (8 * j);
  return (v >> (pos & 7)) & ((1u << nbits) - 1u);
}
__device__ __forceinline__ bool slot_at(long i, long n, int slots) {
  if (slots <= 0 || n <= 0) return false;
  return ((i + 1) * slots) / n != (i * slots) / n;
}
__device__ __forceinline__ uint32_t slots_before(long i, long n, int slots) { return slots > 0 ? (uint32_t)((i * slots) / n) : 0u; }

template <bool BF16>
__device__ __forceinline__ void put_out(void* out, uint64_t at, float v) {
  if (BF16) reinterpret_cast<__nv_bfloat16*>(out)[at] = __float2bfloat16_rn(v);
  else reinterpret_cast<float*>(out)[at] = v;
}

template <bool BF16>
__global__ void codec_decode_kernel(const uint8_t* __restrict__ bytes, const uint8_t* __restrict__ cb_base, const BlockDesc* __restrict__ descs,
                                    long nblocks, void* __restrict__ out) {
  const int lane = threadIdx.x & 31;
  const long warp0 = (blockIdx.x * (long)blockDim.x + threadIdx.x) >> 5, nwarps = ((long)gridDim.x * blockDim.x) >> 5;
  for (long b = warp0; b < nblocks; b += nwarps) {
    const BlockDesc d = descs[b];
    const uint8_t* p = bytes + d.idx_off;
    const uint32_t size = d.idx_bytes;
    const int n = (int)d.n;
    const int fmt = d.fmt;
    const uint64_t o0 = d.out_off;
    if (fmt == SPARK_SPARSE || fmt == SPARK_SPARSE_GRP) {
      for (int i = lane; i < n; i += 32) put_out<BF16>(out, o0 + i, 0.f);
      __syncwarp();
      if (lane == 0) {
        float s0 = 0.f, s1 = 0.f;
        bool live = false;
        if (fmt == SPARK_SPARSE && size >= 4) {
          s0 = s1 = __uint_as_float(get_bits(p, size, 0, 16) | (get_bits(p, size, 16, 16) << 16));
          live = s0 != 0.0f;
        } else if (fmt == SPARK_SPARSE_GRP && size >= 7) {
          s0 = f16_to_f32_wire(get_bits(p, size, 0, 16));
          s1 = f16_to_f32_wire(get_bits(p, size, 16, 16));
          live = !(s0 == 0.0f && s1 == 0.0f);
        }
        if (live) {
          const int half = n / 2;
          for (uint32_t at = 4; at + 2 < size; at += 3) {
            const uint32_t rel = (uint32_t)p[at] | ((uint32_t)p[at + 1] << 8);
            if (rel < (uint32_t)n) {
              const float sc = (fmt == SPARK_SPARSE || (int)rel < half) ? s0 : s1;
              put_out<BF16>(out, o0 + rel, __fmul_rn(__fdiv_rn((float)(int8_t)p[at + 2], 127.0f), sc));
            }
          }
        }
      }
      continue;
    }
    const uint8_t* cb = cb_base + d.cb_off_lo;
    const bool grp = fmt == OIL2_GRP || fmt == OIL4_GRP || fmt == OIL8_GRP;
    const int bits = (fmt == OIL8 || fmt == OIL8_GRP) ? 8 : (fmt == OIL4 || fmt == OIL4_GRP) ? 4 : 2;
    for (int i = lane; i < n; i += 32) {
      float v = 0.f;
      switch (fmt) {
        case OIL32:
          if (size >= (uint32_t)n * 4) v = __uint_as_float(get_bits(p, size, i * 32, 16) | (get_bits(p, size, i * 32 + 16, 16) << 16));
          break;
        case OIL16:
        case OIL16_GRP:
          if ((uint32_t)i * 2 + 1 < size) v = f16_to_f32_wire(get_bits(p, size, i * 16, 16));
          break;
        case OIL8: case OIL4: case OIL2: {
          const int slots = 16 / bits;
          if (!slot_at(i, n, slots)) {
            const float scale = f16_to_f32_wire(get_bits(p, size, 0, 16));
            v = __fmul_rn(level(bits, get_bits(p, size, 16 + bits * (i - slots_before(i, n, slots)), bits)), scale);
          }
          break;
        }
        case OIL1: {
          const int sb = i / 32;
          if ((uint32_t)sb * 2 + 1 < d.cb_bytes) v = f16_to_f32_wire((uint32_t)cb[sb * 2] | ((uint32_t)cb[sb * 2 + 1] << 8));
          break;
        }
        case OIL1_GRP:
          if (n < 32) v = get_bits(p, size, i, 1) ? 1.0f : -1.0f;
          else if (!slot_at(i, n, 16)) {
            const float scale = f16_to_f32_wire(get_bits(p, size, 0, 16));
            v = get_bits(p, size, 16 + i - slots_before(i, n, 16), 1) ? scale : -scale;
          }
          break;
        case SPARK_Q0: {
          const int sb = i / 32, nfull = n / 32;
          const bool full = sb < nfull;
          const uint32_t base = full ? sb * 48 : nfull * 48;
          const float scale = full ? f16_to_f32_wire(get_bits(p, size, base, 16)) : 1.0f;
          v = get_bits(p, size, base + (full ? 16 : 0) + (i - sb * 32), 1) ? scale : -scale;
          break;
        }
        case SPARK_Q0_GRP:
          if (n < 32) v = get_bits(p, size, i, 1) ? 1.0f : -1.0f;
          else {
            const float scale = f16_to_f32_wire(get_bits(p, size, 0, 16));
            const int refined = max(0, n / 2 - 16);
            float mag = scale;
            if (slot_at(i, n, refined)) mag = __fmul_rn(scale, get_bits(p, size, 16 + n + slots_before(i, n, refined), 1) ? 1.893f : 0.567f);
            v = get_bits(p, size, 16 + i, 1) ? mag : -mag;
          }
          break;
        default:
          if (grp) {
            const int nfull = n / 64, gbits = 32 + 64 * bits;
            const bool is8 = bits == 8;
            if (nfull > 0) {
              const int g = min(i / 64, nfull - 1);  // a partial tail reuses the last full group's header
              const uint32_t hdr = g * gbits;
              const uint32_t pos = (i < nfull * 64) ? hdr + 32 + (i - g * 64) * bits : nfull * gbits + (i - nfull * 64) * bits;
              const float zp = f16_to_f32_wire(get_bits(p, size, hdr, 16)), sc = f16_to_f32_wire(get_bits(p, size, hdr + 16, 16));
              const uint32_t q = get_bits(p, size, pos, bits);
              if (sc == 0.0f) v = zp;
              else v = is8 ? __fadd_rn(zp, __fmul_rn(__fdiv_rn((float)q, 255.0f), sc)) : __fadd_rn(__fmul_rn(level(bits, q), sc), zp);
            } else if (n < 8) {
              const uint32_t q = get_bits(p, size, i * bits, bits);
              v = is8 ? __fsub_rn(__fdiv_rn((float)q, 127.5f), 1.0f) : level(bits, q);
            } else {
              const float sc = f16_to_f32_wire(get_bits(p, size, 0, 16));
              if (sc != 0.0f) {
                const uint32_t q = get_bits(p, size, 16 + i * bits, bits);
                v = is8 ? __fmul_rn(__fsub_rn(__fdiv_rn((float)q, 127.5f), 1.0f), sc) : __fmul_rn(level(bits, q), sc);
              }
            }
          }
          break;
      }
      put_out<BF16>(out, o0 + i, v);
    }
  }
}

// ------------------------------------------------------------------------------------------ encode (full 256 blocks)
constexpr int EB = 256;           // weights per block
constexpr int WARPS = 4;          // blocks per CTA
constexpr int PAY_WORDS = 72;     // 288 bytes >= the largest packed payload (OIL8_GRP: 272)

__device__ __forceinline__ void or_bits(uint32_t* words, uint32_t pos, uint32_t v, int nbits) {
  const uint32_t w = pos >> 5, s = pos & 31;
  atomicOr(&words[w], v << s);
  if (s + nbits > 32) atomicOr(&words[w + 1], v >> (32 - s));
}
__device__ double seq_sumsq(const float* w, int n) {
  double s = 0.0;
  for (int i = 0; i < n; ++i) s = __dadd_rn(s, __dmul_rn((double)w[i], (double)w[i]));
  return s;
}
__device__ __forceinline__ float rms_of(const float* w, int n) { return (float)__dsqrt_rn(__ddiv_rn(seq_sumsq(w, n), (double)n)); }

// out: nblocks x stride bytes (stride = payload size of the format for 256 weights); cb_out (OIL1 only): nblocks x 16 bytes.
__global__ void __launch_bounds__(WARPS * 32)
codec_encode_kernel(const float* __restrict__ w, long nblocks, int fmt, uint8_t* __restrict__ out, int stride, uint8_t* __restrict__ cb_out) {
  __shared__ float sw[WARPS][EB];
  __shared__ uint32_t pay[WARPS][PAY_WORDS];
  __shared__ float stat[WARPS][8];
  const int lane = threadIdx.x & 31, wp = threadIdx.x >> 5;
  for (long b = blockIdx.x * (long)WARPS + wp; b < nblocks; b += (long)gridDim.x * WARPS) {
    const float* src = w + b * EB;
    for (int i = lane; i < EB; i += 32) sw[wp][i] = src[i];
    for (int i = lane; i < PAY_WORDS; i += 32) pay[wp][i] = 0;
    __syncwarp();
    const float* x = sw[wp];
    uint32_t* pw = pay[wp];
    uint8_t* dst = out + (size_t)b * stride;
    if (fmt == OIL32 || fmt == OIL16 || fmt == OIL16_GRP) {
      for (int i = lane; i < EB; i += 32) {
        if (fmt == OIL32) reinterpret_cast<uint32_t*>(dst)[i] = __float_as_uint(x[i]);
        else reinterpret_cast<uint16_t*>(dst)[i] = f32_to_f16_wire(x[i]);
      }
      __syncwarp();
      continue;
    }
    if (fmt == OIL1) {  // fp16 means of 32-weight sub-blocks in the codebook channel; lane s sums sub-block s in order
      if (lane < 8) {
        double s = 0.0;
        for (int i = 0; i < 32; ++i) s = __dadd_rn(s, (double)x[lane * 32 + i]);
        reinterpret_cast<uint16_t*>(cb_out + (size_t)b * 16)[lane] = f32_to_f16_wire((float)__ddiv_rn(s, 32.0));
      }
      __syncwarp();
      continue;
    }
    const bool lattice = fmt == OIL8 || fmt == OIL4 || fmt == OIL2;
    const bool grp = fmt == OIL8_GRP || fmt == OIL4_GRP || fmt == OIL2_GRP;
    const int bits = (fmt == OIL8 || fmt == OIL8_GRP) ? 8 : (fmt == OIL4 || fmt == OIL4_GRP) ? 4 : 2;
    if (lattice || fmt == OIL1_GRP || fmt == SPARK_Q0_GRP) {
      if (lane == 0) stat[wp][0] = rms_of(x, EB);
      __syncwarp();
      const float scale = stat[wp][0];
      if (lane == 0) or_bits(pw, 0, f32_to_f16_wire(scale), 16);
      if (lattice) {
        const int slots = 16 / bits;
        const bool dead = scale <= 1e-12f;
        for (int i = lane; i < EB; i += 32)
          if (!slot_at(i, EB, slots))
            or_bits(pw, 16 + bits * (i - slots_before(i, EB, slots)), nearest_level(dead ? 0.0f : __fdiv_rn(x[i], scale), bits), bits);
      } else if (fmt == OIL1_GRP) {
        for (int i = lane; i < EB; i += 32)
          if (!slot_at(i, EB, 16)) or_bits(pw, 16 + i - slots_before(i, EB, 16), x[i] >= 0.0f ? 1u : 0u, 1);
      } else {
        const int refined = EB / 2 - 16;
        const float thr = __fmul_rn(scale, 1.23f);
        for (int i = lane; i < EB; i += 32) {
          or_bits(pw, 16 + i, x[i] >= 0.0f ? 1u : 0u, 1);
          if (slot_at(i, EB, refined)) or_bits(pw, 16 + EB + slots_before(i, EB, refined), fabsf(x[i]) > thr ? 1u : 0u, 1);
        }
      }
    } else if (fmt == SPARK_Q0) {
      if (lane < 8) stat[wp][lane] = rms_of(x + lane * 32, 32);
      __syncwarp();
      if (lane < 8) or_bits(pw, lane * 48, f32_to_f16_wire(stat[wp][lane]), 16);
      for (int i = lane; i < EB; i += 32) or_bits(pw, (i / 32) * 48 + 16 + (i & 31), x[i] >= 0.0f ? 1u : 0u, 1);
    } else if (grp) {
      const bool is8 = bits == 8;
      if (lane < 4) {  // one lane per 64-weight group, sequential like the host code
        const float* gw = x + lane * 64;
        float zp, sc;
        if (is8) {
          float lo = gw[0], hi = gw[0];
          for (int i = 1; i < 64; ++i) { lo = gw[i] < lo ? gw[i] : lo; hi = gw[i] > hi ? gw[i] : hi; }
          zp = lo;
          sc = __fsub_rn(hi, lo);
        } else {
          double mu = 0.0, ss = 0.0;
          for (int i = 0; i < 64; ++i) mu = __dadd_rn(mu, (double)gw[i]);
          mu = __ddiv_rn(mu, 64.0);
          for (int i = 0; i < 64; ++i) {
            const double dd = __dsub_rn((double)gw[i], mu);
            ss = __dadd_rn(ss, __dmul_rn(dd, dd));
          }
          zp = (float)mu;
          sc = ss > 0.0 ? (float)__dsqrt_rn(__ddiv_rn(ss, 64.0)) : 0.0f;
        }
        stat[wp][lane * 2] = zp;
        stat[wp][lane * 2 + 1] = sc;
        const uint32_t hdr = lane * (32 + 64 * bits);
        or_bits(pw, hdr, f32_to_f16_wire(zp), 16);
        or_bits(pw, hdr + 16, f32_to_f16_wire(sc), 16);
      }
      __syncwarp();
      for (int i = lane; i < EB; i += 32) {
        const int g = i / 64;
        const float zp = stat[wp][g * 2], sc = stat[wp][g * 2 + 1];
        uint32_t q = 0;
        if (sc != 0.0f) {
          if (is8) q = range_index(__fdiv_rn(__fsub_rn(x[i], zp), sc), 255.0f);
          else q = nearest_level((float)__ddiv_rn(__dsub_rn((double)x[i], (double)zp), (double)sc), bits);
        }
        or_bits(pw, g * (32 + 64 * bits) + 32 + (i - g * 64) * bits, q, bits);
      }
    }
    __syncwarp();
    for (int i = lane; i < stride; i += 32) dst[i] = (uint8_t)(pw[i >> 2] >> (8 * (i & 3)));
    __syncwarp();
  }
}

}  // namespace bc
}  // namespace inv

using namespace inv::bc;

extern "C" int inv_codec_desc_bytes() { return (int)sizeof(BlockDesc); }

// descs: device array of nblocks records (see BlockDesc); bytes / cb_base: device copies of the index and codebook payloads.
extern "C" int inv_codec_decode(const void* bytes, const void* cb_base, const void* descs, long nblocks, void* out, int out_bf16, void* stream) {
  if (nblocks <= 0) return 0;
  long g = (nblocks * 32 + 255) / 256;
  if (g > 148L * 16) g = 148L * 16;
  if (out_bf16) codec_decode_kernel<true><<<(int)g, 256, 0, (cudaStream_t)stream>>>((const uint8_t*)bytes, (const uint8_t*)cb_base,
                                                                                  (const BlockDesc*)descs, nblocks, out);
  else codec_decode_kernel<false><<<(int)g, 256, 0, (cudaStream_t)stream>>>((const uint8_t*)bytes, (const uint8_t*)cb_base,
                                                                            (const BlockDesc*)descs, nblocks, out);
  cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? 0 : -(int)e;
}
// Payload bytes of one full 256-weight block (0 for formats the device encoder does not write).
extern "C" int inv_codec_encode_stride(int fmt) {
  switch (fmt) {
    case OIL32: return 1024; case OIL16: case OIL16_GRP: return 512; case OIL8: return 256; case OIL4: return 128; case OIL2: return 64;
    case OIL8_GRP: return 272; case OIL4_GRP: return 144; case OIL2_GRP: return 80; case OIL1_GRP: return 32; case SPARK_Q0: return 48;
    case SPARK_Q0_GRP: return 48; case OIL1: return 0;
    default: return -1;
  }
}
extern "C" int inv_codec_encode(const float* w, long nblocks, int fmt, void* out, void* cb_out, void* stream) {
  if (nblocks <= 0) return 0;
  const int stride = inv_codec_encode_stride(fmt);
  if (stride < 0 || (fmt == OIL1 && !cb_out)) return -inv::ERR_BAD_ARG;
  long g = (nblocks + WARPS - 1) / WARPS;
  if (g > 148L * 12) g = 148L * 12;
  codec_encode_kernel<<<(int)g, WARPS * 32, 0, (cudaStream_t)stream>>>(w, nblocks, fmt, (uint8_t*)out, stride, (uint8_t*)cb_out);
  cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? 0 : -(int)e;
}
