// Host-side artifact primitives: LSB-first bit packing of quantised codes, IEEE CRC-32 and the PGRS tensor container.
// Native counterparts of the reference's Rust serializer (parameter-golf-rs/crates/pg-quant/src/serialize.rs:6-99,
// export.rs:542-558); byte formats are identical so artifacts written by either side load in the other.
#pragma once
#include <cstdint>
#include <string>
#include <vector>

namespace pgb {

// `count` signed codes of `bits` width (2..8), stored as (q - qmin) back to back, least significant bit first.
// Throws std::runtime_error when a code is outside [qmin, qmax].
std::string pack_bits(const int8_t* q, size_t count, int bits);
// Inverse; `out` receives `count` codes. Throws when `data` is too short.
void unpack_bits(const uint8_t* data, size_t len, size_t count, int bits, int8_t* out);
uint32_t crc32_ieee(const uint8_t* data, size_t len);

struct PgrsTensor {
  std::string name;
  std::vector<uint32_t> dims;
  uint8_t dtype = 0;        // BF16=0, F16=1, F32=2, I8=3, I32=4, U16=5, U32=6
  std::string data;         // raw payload
};
std::string write_pgrs(const std::vector<PgrsTensor>& tensors, const std::string& metadata);
// Parses and checks every tensor's CRC; throws std::runtime_error with the reason on any malformed input.
std::vector<PgrsTensor> read_pgrs(const std::string& buf, std::string* metadata);

}  // namespace pgb
