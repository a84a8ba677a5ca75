// TEST INFRASTRUCTURE ONLY -- C-ABI wrappers around the reference runtime's host decode oracle
// (runtime/src/qtip.cpp), compiled from the reference tree where it lies (see Makefile target `ref`).
#include <cstdint>
#include <cstring>
#include <filesystem>
#include <span>
#include <string>
#include <vector>

#include "behemoth/checkpoint.hpp"
#include "behemoth/qtip.hpp"

using namespace behemoth::qtip;

static HostLinear make(const uint16_t* trellis, const float* su, const float* sv, const uint16_t* tlut, int in, int out) {
  HostLinear l;
  l.in = in;
  l.out = out;
  l.trellis.assign(trellis, trellis + size_t(out / 16) * size_t(in / 16) * 32);
  l.su.assign(su, su + in);
  l.sv.assign(sv, sv + out);
  l.tlut.assign(tlut, tlut + 1024);
  return l;
}

extern "C" {
// make_codebook, runtime/src/qtip.cpp:62-80.
int rref_codebook(const uint16_t* tlut, float* c0, float* c1, uint32_t* bf16x2) {
  try {
    Codebook cb = make_codebook(std::span<const uint16_t>(tlut, 1024));
    std::memcpy(c0, cb.c0.data(), 4096);
    std::memcpy(c1, cb.c1.data(), 4096);
    std::memcpy(bf16x2, cb.bf16x2.data(), 4096);
    return 0;
  } catch (...) { return -1; }
}
int rref_had_k(int n) {
  try { return had_k(n); } catch (...) { return 0; }
}
int rref_hadamard(double* x, int n, int transpose) {
  try { hadamard(x, n, transpose != 0); return 0; } catch (...) { return -1; }
}
// decode_rows / decode_rows_bf16, runtime/src/qtip.cpp:83-128.
int rref_decode_rows(const uint16_t* trellis, const uint16_t* tlut, int in, int out, int row0, int rows, int bf16,
                     float* w) {
  try {
    std::vector<float> su(size_t(in), 1.f), sv(size_t(out), 1.f);
    HostLinear l = make(trellis, su.data(), sv.data(), tlut, in, out);
    Codebook cb = make_codebook(l.tlut);
    if (bf16) decode_rows_bf16(l, cb, row0, rows, w);
    else decode_rows(l, cb, row0, rows, w);
    return 0;
  } catch (...) { return -1; }
}
// reference_forward, runtime/src/qtip.cpp:129-192.
int rref_forward(const uint16_t* trellis, const float* su, const float* sv, const uint16_t* tlut, int in, int out,
                 const float* x, int rows, int device_rounding, int round_z, float* y) {
  try {
    HostLinear l = make(trellis, su, sv, tlut, in, out);
    auto r = reference_forward(l, std::span<const float>(x, size_t(rows) * size_t(in)), device_rounding != 0, round_z != 0);
    std::memcpy(y, r.data(), r.size() * 4);
    return 0;
  } catch (...) { return -1; }
}
// load_linear(SafeTensorFile, layer, name, config), runtime/src/qtip.cpp:231-289: the runtime's loader with its checks,
// on a layer file at `path`; geometry from a configuration with the given hidden / intermediate / kv_heads / dim.
// Returns 0 and fills the caller's arrays (sized from the geometry), or -1 with the message in rref_last_error().
static thread_local std::string g_load_error;
const char* rref_last_error() { return g_load_error.c_str(); }
int rref_load_linear(const char* path, int layer, const char* name, int hidden, int intermediate, int kv_heads, int dim,
                     int* in, int* out, uint16_t* trellis, float* su, float* sv, uint16_t* tlut) {
  try {
    behemoth::SafeTensorFile file{std::filesystem::path(path)};
    behemoth::ModelConfig cfg;
    cfg.hidden = hidden, cfg.intermediate = intermediate, cfg.kv_heads = kv_heads, cfg.dim = dim;
    HostLinear l = load_linear(file, layer, name, &cfg);
    *in = l.in, *out = l.out;
    std::memcpy(trellis, l.trellis.data(), l.trellis.size() * 2);
    std::memcpy(su, l.su.data(), l.su.size() * 4);
    std::memcpy(sv, l.sv.data(), l.sv.size() * 4);
    std::memcpy(tlut, l.tlut.data(), l.tlut.size() * 2);
    return 0;
  } catch (const std::exception& e) {
    g_load_error = e.what();
    return -1;
  }
}
}
