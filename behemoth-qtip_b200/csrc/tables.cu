// Error plumbing, per-device set-up and the codebook tables of the qtip_b200 library.
#include <cmath>
#include <cstdarg>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <atomic>
#include <mutex>

#include "common.cuh"

namespace qb {

static thread_local char g_error[512] = "";

int fail(int code, const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  std::vsnprintf(g_error, sizeof g_error, fmt, ap);
  va_end(ap);
  return code;
}
int cuda_fail(cudaError_t e, const char* what, const char* file, int line) {
  const char* base = std::strrchr(file, '/');
  std::snprintf(g_error, sizeof g_error, "%s:%d: %s -> %s", base ? base + 1 : file, line, what, cudaGetErrorString(e));
  return int(e);
}

static std::mutex g_mu;
static DeviceInfo g_dev[64];
// Published with release order after g_dev[dev] is complete and read with acquire order, so that a thread calling an
// entry point while another thread initialises the device sees either "not ready" or the whole record.
static std::atomic<bool> g_dev_ready[64];

DeviceInfo* device_info() {
  int dev = -1;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) {
    fail(QTIP_E_DEVICE, "no current CUDA device");
    return nullptr;
  }
  if (!g_dev_ready[dev].load(std::memory_order_acquire)) {
    fail(QTIP_E_DEVICE, "qtip_init() has not been called on device %d", dev);
    return nullptr;
  }
  return &g_dev[dev];
}

// Quadratic character mod p (p prime).
static int chi(int a, int p) {
  a = ((a % p) + p) % p;
  if (a == 0) return 0;
  for (int x = 1; x < p; ++x)
    if ((x * x) % p == a) return 1;
  return -1;
}
// The order-12 and order-20 factors are Paley-I matrices (q = 11, 19) in the normalisation the QTIP checkpoints use:
// first row (1, -1, ..., -1), first column all ones, circulant core with 1 on the diagonal and -chi(j - i) elsewhere.
// The order-28 factor is the Paley-II matrix for q = 13 as a 2x2 arrangement of bordered 14x14 circulants.
bool had_factor(int K, int8_t* H) {
  if (K == 12 || K == 20) {
    const int q = K - 1;
    for (int i = 0; i < K; ++i)
      for (int j = 0; j < K; ++j) {
        int v;
        if (i == 0) v = j == 0 ? 1 : -1;
        else if (j == 0) v = 1;
        else {
          int k = ((j - i) % q + q) % q;
          v = k == 0 ? 1 : -chi(k, q);
        }
        H[i * K + j] = int8_t(v);
      }
    return true;
  }
  if (K == 28) {
    const int q = 13, h = 14;
    for (int i = 0; i < K; ++i)
      for (int j = 0; j < K; ++j) {
        const int bi = i / h, bj = j / h, r = i % h, c = j % h;
        const bool core = r >= 1 && c >= 1;
        const int k = ((c - r) % q + q) % q;
        const int x = (core && k != 0) ? chi(k, q) : 0;
        int v;
        if (bi == 0 && bj == 0) v = !core ? 1 : (k == 0 ? 1 : x);
        else if (bi != bj) v = r == 0 ? (c == 0 ? -1 : 1) : (c == 0 ? 1 : (k == 0 ? -1 : x));
        else v = !core ? -1 : (k == 0 ? -1 : -x);
        H[i * K + j] = int8_t(v);
      }
    return true;
  }
  return false;
}
int had_order(long n) {
  static const int order[12] = {172, 156, 140, 124, 116, 108, 60, 52, 36, 28, 20, 12};
  for (int K : order)
    if (n % K == 0) {
      long p = n / K;
      if (p <= 0 || (p & (p - 1))) return 0;
      return (K == 28 || K == 20 || K == 12) ? K : 0;
    }
  return (n > 0 && (n & (n - 1)) == 0) ? 1 : 0;
}

static float half_bits_to_float(uint16_t h) {
  const uint32_t s = (h >> 15) & 1, e = (h >> 10) & 0x1f, m = h & 0x3ff;
  float v;
  if (e == 0) v = std::ldexp(float(m), -24);
  else if (e == 31) v = m ? NAN : INFINITY;
  else v = std::ldexp(float(m | 0x400), int(e) - 25);
  return s ? -v : v;
}
static uint16_t float_to_bf16_bits(float f) {
  uint32_t u;
  std::memcpy(&u, &f, 4);
  if ((u & 0x7fffffffu) > 0x7f800000u) return uint16_t((u >> 16) | 0x40);
  u += 0x7fffu + ((u >> 16) & 1u);
  return uint16_t(u >> 16);
}

}  // namespace qb

using namespace qb;

namespace qb {
bool chained_launches_enabled() {
  static const bool on = [] {
    const char* e = std::getenv("QTIP_PDL");
    return !(e && e[0] == '0');
  }();
  return on;
}
}  // namespace qb

extern "C" const char* qtip_last_error(void) { return g_error; }
extern "C" int qtip_abi_version(void) { return 1; }

extern "C" int qtip_init(void) {
  int dev = -1;
  QB_CUDA(cudaGetDevice(&dev));
  QB_REQUIRE(dev >= 0 && dev < 64, QTIP_E_DEVICE, "device index %d out of range", dev);
  std::lock_guard<std::mutex> lk(g_mu);
  if (g_dev_ready[dev].load(std::memory_order_acquire)) return QTIP_OK;
  cudaDeviceProp prop{};
  QB_CUDA(cudaGetDeviceProperties(&prop, dev));
  QB_REQUIRE(prop.major == 10, QTIP_E_DEVICE, "device %d is sm_%d%d; this library is built for sm_100a only", dev,
             prop.major, prop.minor);
  DeviceInfo info;
  info.sm_count = prop.multiProcessorCount;
  int rc = hadamard_device_setup();
  if (rc) return rc;
  rc = viterbi_device_setup(&info);
  if (rc) return rc;
  rc = decode_device_setup(&info);
  if (rc) return rc;
  rc = gemm_tc_device_setup();
  if (rc) return rc;
  rc = trellis_tc_device_setup();
  if (rc) return rc;
  rc = block_ldl_device_setup();
  if (rc) return rc;
  info.ready = true;
  g_dev[dev] = info;
  g_dev_ready[dev].store(true, std::memory_order_release);
  return QTIP_OK;
}

// The two table uploads copy from pageable host memory: cudaMemcpyAsync then returns only after the source has been
// consumed, so the host buffer may be reused at once. Not legal during stream capture: build tables at load time.
static int upload_table(const void* host, size_t bytes, void* dev_dst, void* stream) {
  QB_CUDA(cudaMemcpyAsync(dev_dst, host, bytes, cudaMemcpyHostToDevice, as_stream(stream)));
  return QTIP_OK;
}

extern "C" int qtip_encoder_lut(const uint16_t* tlut_h, uint32_t* lut_h2_d, double* lut_rms_h, void* stream) {
  QB_REQUIRE(tlut_h && lut_h2_d, QTIP_E_ARG, "qtip_encoder_lut: null pointer");
  static thread_local uint32_t table[65536];
  double ss = 0;
  for (uint32_t s = 0; s < 65536; ++s) {
    const uint64_t p = uint64_t(s + 1) * uint64_t(s);
    const int idx = int((p >> 6) & 511);
    uint16_t h0 = tlut_h[idx * 2], h1 = tlut_h[idx * 2 + 1];
    if ((p >> 15) & 1) h0 ^= 0x8000;
    table[s] = uint32_t(h0) | (uint32_t(h1) << 16);
    const double a = half_bits_to_float(h0), b = half_bits_to_float(h1);
    ss += a * a + b * b;
  }
  if (lut_rms_h) *lut_rms_h = std::sqrt(ss / (2.0 * 65536));
  return upload_table(table, sizeof table, lut_h2_d, stream);
}

extern "C" int qtip_runtime_lut(const uint16_t* tlut_h, uint32_t* lut_d, void* stream) {
  QB_REQUIRE(tlut_h && lut_d, QTIP_E_ARG, "qtip_runtime_lut: null pointer");
  uint32_t table[1024];
  for (int e = 0; e < 1024; ++e) {
    const int idx = e & 511;
    uint16_t h0 = tlut_h[idx * 2], h1 = tlut_h[idx * 2 + 1];
    if (e >> 9) h0 ^= 0x8000u;
    const float c0 = half_bits_to_float(h0), c1 = half_bits_to_float(h1);
    QB_REQUIRE(std::isfinite(c0) && std::isfinite(c1), QTIP_E_ARG, "qtip_runtime_lut: non-finite tlut entry %d", idx);
    table[e] = uint32_t(float_to_bf16_bits(c0)) | (uint32_t(float_to_bf16_bits(c1)) << 16);
  }
  return upload_table(table, sizeof table, lut_d, stream);
}
