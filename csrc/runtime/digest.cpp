// Streaming FNV-1a 64 digest: the hash behind plan hashes, mesh ids and autotune identities.
//
// Every rank derives its collective plan independently and the 64-bit hashes are compared before any communicator
// or peer mapping exists (the reference hashes "incin.collective.plan.v2" plus every descriptor field the same way:
// crates/incin-core/src/dist/collective.rs:843-866).  The encoding is fixed: `number` = 8 little-endian bytes,
// `field` = number(length) followed by the bytes, `text` = field(utf-8).  The Python package carries the same digest
// in pure Python; a parity test keeps the two identical.
#include <cstddef>
#include <cstdint>

#define API extern "C" __attribute__((visibility("default")))

namespace {
constexpr uint64_t kOffset = 0xCBF29CE484222325ull;
constexpr uint64_t kPrime = 0x100000001B3ull;

inline uint64_t mix(uint64_t s, const uint8_t* p, size_t n) {
  for (size_t i = 0; i < n; ++i) s = (s ^ p[i]) * kPrime;
  return s;
}
}  // namespace

API uint64_t incin_digest_init(void) { return kOffset; }

API uint64_t incin_digest_bytes(uint64_t state, const void* data, int64_t n) {
  if (!data || n <= 0) return state;
  return mix(state, static_cast<const uint8_t*>(data), static_cast<size_t>(n));
}

API uint64_t incin_digest_number(uint64_t state, uint64_t v) {
  uint8_t le[8];
  for (int i = 0; i < 8; ++i) le[i] = static_cast<uint8_t>(v >> (8 * i));
  return mix(state, le, 8);
}

API uint64_t incin_digest_field(uint64_t state, const void* data, int64_t n) {
  if (n < 0) n = 0;
  state = incin_digest_number(state, static_cast<uint64_t>(n));
  return incin_digest_bytes(state, data, n);
}

// One call for the common case: hash of a whole buffer from the initial state.
API uint64_t incin_fnv1a64(const void* data, int64_t n) { return incin_digest_bytes(kOffset, data, n); }
