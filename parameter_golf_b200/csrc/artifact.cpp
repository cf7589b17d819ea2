#include "artifact.h"

#include <cstring>
#include <stdexcept>

namespace pgb {

std::string pack_bits(const int8_t* q, size_t count, int bits) {
  if (bits < 2 || bits > 8) throw std::runtime_error("pack_bits: bit width must be 2..8");
  const int qmin = -(1 << (bits - 1));
  const uint32_t limit = 1u << bits;
  std::string out((count * (size_t)bits + 7) / 8, '\0');
  uint8_t* o = reinterpret_cast<uint8_t*>(&out[0]);
  uint64_t acc = 0;       // bit accumulator, least significant bit = next bit to emit
  int have = 0;
  size_t pos = 0;
  for (size_t i = 0; i < count; ++i) {
    const uint32_t e = (uint32_t)((int)q[i] - qmin);
    if (e >= limit) throw std::runtime_error("quantised value out of range for bit width");
    acc |= (uint64_t)e << have;
    have += bits;
    while (have >= 8) {
      o[pos++] = (uint8_t)(acc & 0xFF);
      acc >>= 8;
      have -= 8;
    }
  }
  if (have > 0) o[pos++] = (uint8_t)(acc & 0xFF);
  return out;
}

void unpack_bits(const uint8_t* data, size_t len, size_t count, int bits, int8_t* out) {
  if (bits < 2 || bits > 8) throw std::runtime_error("unpack_bits: bit width must be 2..8");
  if (len < (count * (size_t)bits + 7) / 8) throw std::runtime_error("packed tensor is shorter than its shape requires");
  const int qmin = -(1 << (bits - 1));
  const uint32_t mask = (1u << bits) - 1;
  uint64_t acc = 0;
  int have = 0;
  size_t pos = 0;
  for (size_t i = 0; i < count; ++i) {
    while (have < bits) {
      acc |= (uint64_t)data[pos++] << have;
      have += 8;
    }
    out[i] = (int8_t)((int)(acc & mask) + qmin);
    acc >>= bits;
    have -= bits;
  }
}

namespace {
struct CrcTable {
  uint32_t t[8][256];
  CrcTable() {
    for (uint32_t i = 0; i < 256; ++i) {
      uint32_t c = i;
      for (int k = 0; k < 8; ++k) c = (c & 1) ? (0xEDB88320u ^ (c >> 1)) : (c >> 1);
      t[0][i] = c;
    }
    for (uint32_t i = 0; i < 256; ++i)
      for (int s = 1; s < 8; ++s) t[s][i] = (t[s - 1][i] >> 8) ^ t[0][t[s - 1][i] & 0xFF];
  }
};
const CrcTable& crc_table() {
  static const CrcTable tab;
  return tab;
}
void put_u32(std::string& s, uint32_t v) {
  const char b[4] = {(char)(v & 0xFF), (char)((v >> 8) & 0xFF), (char)((v >> 16) & 0xFF), (char)((v >> 24) & 0xFF)};
  s.append(b, 4);
}
}  // namespace

uint32_t crc32_ieee(const uint8_t* data, size_t len) {
  const CrcTable& T = crc_table();
  uint32_t c = 0xFFFFFFFFu;
  while (len >= 8) {      // slicing-by-8
    uint32_t lo, hi;
    std::memcpy(&lo, data, 4);
    std::memcpy(&hi, data + 4, 4);
    lo ^= c;
    c = T.t[7][lo & 0xFF] ^ T.t[6][(lo >> 8) & 0xFF] ^ T.t[5][(lo >> 16) & 0xFF] ^ T.t[4][lo >> 24] ^ T.t[3][hi & 0xFF] ^ T.t[2][(hi >> 8) & 0xFF] ^
        T.t[1][(hi >> 16) & 0xFF] ^ T.t[0][hi >> 24];
    data += 8;
    len -= 8;
  }
  while (len--) c = T.t[0][(c ^ *data++) & 0xFF] ^ (c >> 8);
  return c ^ 0xFFFFFFFFu;
}

std::string write_pgrs(const std::vector<PgrsTensor>& tensors, const std::string& metadata) {
  size_t total = 12 + 4 + metadata.size();
  for (const auto& t : tensors) total += 4 + t.name.size() + 4 + 4 * t.dims.size() + 1 + 4 + t.data.size() + 4;
  std::string out;
  out.reserve(total);
  out.append("PGRS", 4);
  put_u32(out, 1);
  put_u32(out, (uint32_t)tensors.size());
  for (const auto& t : tensors) {
    if (t.dtype > 7) throw std::runtime_error("write_pgrs: unknown dtype code");
    put_u32(out, (uint32_t)t.name.size());
    out.append(t.name);
    put_u32(out, (uint32_t)t.dims.size());
    for (uint32_t d : t.dims) put_u32(out, d);
    out.push_back((char)t.dtype);
    put_u32(out, (uint32_t)t.data.size());
    out.append(t.data);
    put_u32(out, crc32_ieee(reinterpret_cast<const uint8_t*>(t.data.data()), t.data.size()));
  }
  put_u32(out, (uint32_t)metadata.size());
  out.append(metadata);
  return out;
}

std::vector<PgrsTensor> read_pgrs(const std::string& buf, std::string* metadata) {
  if (buf.size() < 12 || std::memcmp(buf.data(), "PGRS", 4) != 0) throw std::runtime_error("not a PGRS file");
  size_t pos = 4;
  auto take = [&](size_t n) -> const char* {
    if (pos + n > buf.size()) throw std::runtime_error("truncated PGRS file");
    const char* p = buf.data() + pos;
    pos += n;
    return p;
  };
  auto u32 = [&]() -> uint32_t {
    const uint8_t* p = reinterpret_cast<const uint8_t*>(take(4));
    return (uint32_t)p[0] | ((uint32_t)p[1] << 8) | ((uint32_t)p[2] << 16) | ((uint32_t)p[3] << 24);
  };
  const uint32_t version = u32(), count = u32();
  if (version != 1) throw std::runtime_error("unsupported PGRS version " + std::to_string(version));
  std::vector<PgrsTensor> tensors;
  for (uint32_t i = 0; i < count; ++i) {
    PgrsTensor t;
    const uint32_t nl = u32();
    t.name.assign(take(nl), nl);
    const uint32_t nd = u32();
    if (nd > 8) throw std::runtime_error("tensor " + t.name + ": too many dimensions");
    for (uint32_t k = 0; k < nd; ++k) t.dims.push_back(u32());
    t.dtype = (uint8_t)*take(1);
    if (t.dtype > 7) throw std::runtime_error("tensor " + t.name + ": unknown dtype code " + std::to_string((int)t.dtype));
    const uint32_t dl = u32();
    t.data.assign(take(dl), dl);
    const uint32_t crc = u32();
    if (crc != crc32_ieee(reinterpret_cast<const uint8_t*>(t.data.data()), t.data.size()))
      throw std::runtime_error("tensor " + t.name + ": CRC mismatch");
    tensors.push_back(std::move(t));
  }
  const uint32_t ml = u32();
  const char* m = take(ml);
  if (metadata) metadata->assign(m, ml);
  return tensors;
}

}  // namespace pgb
