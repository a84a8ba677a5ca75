// TEST INFRASTRUCTURE ONLY -- exposes the reference's committed Hadamard tables (src/qtip_constants.hpp) so that the
// test suite can compare the constructed Paley matrices with them entry by entry.
#include <cstdint>
#include <cstring>

#include "qtip_constants.hpp"

extern "C" int ref_had_table(int K, int8_t* out) {
  const int8_t* h = qtip::had_table(K);
  if (!h) return 0;
  std::memcpy(out, h, size_t(K) * K);
  return 1;
}
