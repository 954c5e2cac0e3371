// Canonical .oil block codec: the payload bytes of every wire format.
//
// Byte-compatible with the reference's quantize_block_all / dequantize_block_all
// (src/block_codec.cpp:368-720). Format ids are the reference's (include/oil/types.h:19-35).
#pragma once
#include <cstddef>
#include <cstdint>
#include <string>
#include <vector>

namespace inv {

enum Format : uint8_t {
  OIL1 = 0, SPARK_Q0 = 1, OIL2 = 2, OIL4 = 3, OIL8 = 4, OIL16 = 5, OIL32 = 6, OIL1_GRP = 7, SPARK_Q0_GRP = 8, OIL2_GRP = 9,
  OIL4_GRP = 10, OIL8_GRP = 11, OIL16_GRP = 12, SPARK_SPARSE = 13, SPARK_SPARSE_GRP = 14, FORMAT_COUNT = 15,
};

const char* format_name(int fmt);
int format_from_name(const std::string& name);  // -1 if unknown
float format_bpw(int fmt);                      // claimed bits per weight
size_t claimed_bytes(int fmt, uint32_t n);      // ceil(bpw * n / 8)

uint16_t f32_to_f16(float v);
float f16_to_f32(uint16_t h);

// Encode one block of n weights. `codebook` is used by OIL1 only (fp16 means per 32 weights).
bool encode_block(int fmt, const float* w, int n, std::vector<uint8_t>& indices, std::vector<uint8_t>& codebook);
// Decode; reads past the payload yield zeros, unknown formats all zeros.
void decode_block(int fmt, const uint8_t* indices, size_t idx_bytes, const uint8_t* codebook, size_t cb_bytes, uint32_t n, float* out);

// Fixed Gaussian lattices of the 2- and 4-bit formats, and the 8-bit uniform lattice on [-8, 8].
extern const float kLevels2[4];
extern const float kLevels4[16];
inline float level8(uint32_t i) { return -8.0f + 16.0f * (float)(i > 255u ? 255u : i) / 255.0f; }

}  // namespace inv
