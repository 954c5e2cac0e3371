// SHA-256 (FIPS 180-4). Used for the .oilidx name hashes, content-addressed block dedup and
// checkpoint shard manifests, like the reference's in-file implementation (src/oil_format.cpp:17-114).
#pragma once
#include <cstddef>
#include <cstdint>
#include <string>

namespace inv {
struct Sha256 {
  uint8_t bytes[32];
  std::string hex() const;
};
Sha256 sha256(const void* data, size_t size);
}  // namespace inv
