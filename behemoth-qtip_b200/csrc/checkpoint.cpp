// Layer files of a QTIP checkpoint (safetensors container): the writer of the quantizer (write_layer_file,
// src/pipeline.cpp:314-352, container code src/safetensors.cpp:93-136) and the loader of the runtime with its checks
// (load_linear, runtime/src/qtip.cpp:231-289). Host code only. Per linear `model.layers.<L>.<name>.`:
//   trellis I16 [(m/16)(n/16), 32]  kernel-layout words      SU  BF16 [n]  +-1
//   SV      F32 [m]  sign * Wscale                            tlut F16 [512, 2]
//   rcp     I64 [] = 0                                        tp_rank I64 [] = 8
// Container: 8-byte little-endian header length, JSON header padded with spaces to a multiple of 8 bytes, tensor data in
// header order (names sorted), offsets relative to the end of the header.
#include <cerrno>
#include <cmath>
#include <cstdio>
#include <cstring>
#include <map>
#include <string>
#include <vector>

#include <sys/stat.h>

#include "../../include/qtip_b200.h"

namespace qb {
int fail(int code, const char* fmt, ...);
}
#define CK_REQUIRE(cond, code, ...)                   \
  do {                                                \
    if (!(cond)) return qb::fail(code, __VA_ARGS__); \
  } while (0)

namespace {

struct Entry {
  std::string dtype;
  std::vector<long> shape;
  const void* data = nullptr;
  std::vector<unsigned char> owned;  // scalars
  size_t bytes = 0;
  size_t begin = 0, end = 0;  // reader: offsets relative to the data section
};

std::string json_string(const std::string& s) {
  std::string o = "\"";
  for (char c : s) {
    if (c == '"' || c == '\\') o.push_back('\\');
    o.push_back(c);
  }
  return o + "\"";
}

// ---- a reader for the flat JSON of a safetensors header: {"name": {"dtype": "..", "shape": [..], "data_offsets": [a, b]}, ...}
struct Cursor {
  const char* p;
  const char* end;
  bool ok = true;
  void ws() {
    while (p < end && (*p == ' ' || *p == '\n' || *p == '\t' || *p == '\r')) ++p;
  }
  bool eat(char c) {
    ws();
    if (p < end && *p == c) {
      ++p;
      return true;
    }
    return false;
  }
  std::string str() {
    ws();
    std::string s;
    if (p >= end || *p != '"') {
      ok = false;
      return s;
    }
    for (++p; p < end && *p != '"'; ++p) {
      if (*p == '\\' && p + 1 < end) ++p;
      s.push_back(*p);
    }
    if (p >= end) ok = false;
    else ++p;
    return s;
  }
  long integer() {
    ws();
    char* e = nullptr;
    const long v = std::strtol(p, &e, 10);
    if (e == p) ok = false;
    p = e;
    return v;
  }
  void skip_value() {  // strings, numbers, arrays and objects of strings / numbers
    ws();
    if (p >= end) {
      ok = false;
      return;
    }
    if (*p == '"') {
      str();
    } else if (*p == '{' || *p == '[') {
      const char close = *p == '{' ? '}' : ']';
      ++p;
      if (eat(close)) return;
      do {
        if (close == '}') {
          str();
          if (!eat(':')) ok = false;
        }
        skip_value();
      } while (ok && eat(','));
      if (!eat(close)) ok = false;
    } else {
      while (p < end && *p != ',' && *p != '}' && *p != ']') ++p;
    }
  }
};

bool parse_header(const std::string& h, std::map<std::string, Entry>* out) {
  Cursor c{h.data(), h.data() + h.size()};
  if (!c.eat('{')) return false;
  if (c.eat('}')) return true;
  do {
    const std::string name = c.str();
    if (!c.ok || !c.eat(':')) return false;
    if (name == "__metadata__") {
      c.skip_value();
      continue;
    }
    Entry e;
    if (!c.eat('{')) return false;
    do {
      const std::string key = c.str();
      if (!c.ok || !c.eat(':')) return false;
      if (key == "dtype") {
        e.dtype = c.str();
      } else if (key == "shape" || key == "data_offsets") {
        std::vector<long> v;
        if (!c.eat('[')) return false;
        if (!c.eat(']')) {
          do v.push_back(c.integer());
          while (c.ok && c.eat(','));
          if (!c.eat(']')) return false;
        }
        if (key == "shape") e.shape = v;
        else if (v.size() == 2 && v[0] >= 0 && v[1] >= v[0]) e.begin = size_t(v[0]), e.end = size_t(v[1]);
        else return false;
      } else {
        c.skip_value();
      }
    } while (c.ok && c.eat(','));
    if (!c.ok || !c.eat('}')) return false;
    (*out)[name] = e;
  } while (c.ok && c.eat(','));
  return c.ok && c.eat('}');
}

float bf16_bits_to_float(uint16_t b) {
  uint32_t u = uint32_t(b) << 16;
  float f;
  std::memcpy(&f, &u, 4);
  return f;
}
float f16_bits_to_float(uint16_t h) {
  const uint32_t s = (h >> 15) & 1, e = (h >> 10) & 0x1f, m = h & 0x3ff;
  float v;
  if (e == 0) v = std::ldexp(float(m), -24);
  else if (e == 31) v = m ? NAN : INFINITY;
  else v = std::ldexp(float(m | 0x400), int(e) - 25);
  return s ? -v : v;
}

struct File {
  std::FILE* f = nullptr;
  ~File() {
    if (f) std::fclose(f);
  }
};

}  // namespace

extern "C" int qtip_write_layer_file(const char* path, int layer, const qtip_checkpoint_linear* lins, int count) {
  CK_REQUIRE(path && lins && count >= 1 && layer >= 0, QTIP_E_ARG, "qtip_write_layer_file: bad argument");
  std::map<std::string, Entry> entries;  // sorted by name, like the reference's writer
  const int64_t zero = 0, eight = 8;
  for (int i = 0; i < count; ++i) {
    const qtip_checkpoint_linear& l = lins[i];
    CK_REQUIRE(l.name && l.trellis_h && l.su_bf16_h && l.sv_h && l.tlut_h, QTIP_E_ARG, "qtip_write_layer_file: linear %d has a null field", i);
    CK_REQUIRE(l.m > 0 && l.n > 0 && l.m % 32 == 0 && l.n % 32 == 0, QTIP_E_GEOMETRY,
               "qtip_write_layer_file: %s is %d x %d (multiples of 32 needed for the kernel layout)", l.name, l.m, l.n);
    for (int r = 0; r < l.m; ++r)
      CK_REQUIRE(std::isfinite(l.sv_h[r]), QTIP_E_ARG, "qtip_write_layer_file: %s has a non-finite SV entry", l.name);
    const std::string b = "model.layers." + std::to_string(layer) + "." + l.name + ".";
    auto add = [&](const char* suffix, const char* dtype, std::vector<long> shape, const void* data, size_t bytes) {
      Entry e;
      e.dtype = dtype, e.shape = std::move(shape), e.data = data, e.bytes = bytes;
      entries[b + suffix] = std::move(e);
    };
    const long tiles = long(l.m / 16) * (l.n / 16);
    add("trellis", "I16", {tiles, 32}, l.trellis_h, size_t(tiles) * 64);
    add("SU", "BF16", {l.n}, l.su_bf16_h, size_t(l.n) * 2);
    add("SV", "F32", {l.m}, l.sv_h, size_t(l.m) * 4);
    add("tlut", "F16", {512, 2}, l.tlut_h, 2048);
    add("rcp", "I64", {}, &zero, 8);       // the sign vector already carries Wscale
    add("tp_rank", "I64", {}, &eight, 8);
  }
  std::string h = "{\"__metadata__\":{\"format\":\"pt\"}";
  size_t off = 0;
  for (auto& kv : entries) {
    h += "," + json_string(kv.first) + ":{\"data_offsets\":[" + std::to_string(off) + "," +
         std::to_string(off + kv.second.bytes) + "],\"dtype\":" + json_string(kv.second.dtype) + ",\"shape\":[";
    for (size_t d = 0; d < kv.second.shape.size(); ++d) h += (d ? "," : "") + std::to_string(kv.second.shape[d]);
    h += "]}";
    off += kv.second.bytes;
  }
  h += "}";
  while ((h.size() + 8) % 8) h.push_back(' ');
  const std::string tmp = std::string(path) + ".tmp";
  {
    File out;
    out.f = std::fopen(tmp.c_str(), "wb");
    CK_REQUIRE(out.f, QTIP_E_ARG, "qtip_write_layer_file: cannot write %s (%s)", tmp.c_str(), std::strerror(errno));
    const uint64_t hl = h.size();
    bool ok = std::fwrite(&hl, 8, 1, out.f) == 1 && std::fwrite(h.data(), 1, h.size(), out.f) == h.size();
    for (auto& kv : entries)
      ok = ok && std::fwrite(kv.second.data, 1, kv.second.bytes, out.f) == kv.second.bytes;
    ok = ok && std::fflush(out.f) == 0;
    CK_REQUIRE(ok, QTIP_E_ARG, "qtip_write_layer_file: write to %s failed", tmp.c_str());
  }
  CK_REQUIRE(std::rename(tmp.c_str(), path) == 0, QTIP_E_ARG, "qtip_write_layer_file: cannot rename %s (%s)", tmp.c_str(),
             std::strerror(errno));
  return QTIP_OK;
}

extern "C" int qtip_read_layer_linear(const char* path, int layer, const char* name, int m, int n, uint16_t* trellis_h,
                                      float* su_h, float* sv_h, uint16_t* tlut_h) {
  CK_REQUIRE(path && name && trellis_h && su_h && sv_h && tlut_h && layer >= 0 && m > 0 && n > 0, QTIP_E_ARG,
             "qtip_read_layer_linear: bad argument");
  File in;
  in.f = std::fopen(path, "rb");
  CK_REQUIRE(in.f, QTIP_E_ARG, "qtip_read_layer_linear: cannot open %s (%s)", path, std::strerror(errno));
  struct stat sb;
  CK_REQUIRE(stat(path, &sb) == 0, QTIP_E_ARG, "qtip_read_layer_linear: cannot stat %s", path);
  uint64_t hl = 0;
  CK_REQUIRE(std::fread(&hl, 8, 1, in.f) == 1 && hl >= 2 && hl + 8 <= uint64_t(sb.st_size), QTIP_E_ARG,
             "qtip_read_layer_linear: %s is not a safetensors file", path);
  std::string h(size_t(hl), '\0');
  CK_REQUIRE(std::fread(&h[0], 1, h.size(), in.f) == h.size(), QTIP_E_ARG, "qtip_read_layer_linear: short header in %s", path);
  std::map<std::string, Entry> entries;
  CK_REQUIRE(parse_header(h, &entries), QTIP_E_ARG, "qtip_read_layer_linear: malformed header in %s", path);
  const size_t data0 = 8 + size_t(hl), data_bytes = size_t(sb.st_size) - data0;
  const std::string base = "model.layers." + std::to_string(layer) + "." + name + ".";
  auto find = [&](const char* suffix, const char* dtype, const std::vector<long>& shape, size_t bytes,
                  const Entry** out) -> int {
    auto it = entries.find(base + suffix);
    CK_REQUIRE(it != entries.end(), QTIP_E_ARG, "%s%s is missing from %s", base.c_str(), suffix, path);
    const Entry& e = it->second;
    CK_REQUIRE(e.dtype == dtype && e.shape == shape && e.end - e.begin == bytes && e.end <= data_bytes, QTIP_E_GEOMETRY,
               "Invalid QTIP %s%s: dtype %s, %zu bytes (expected %s, %zu bytes)", base.c_str(), suffix, e.dtype.c_str(),
               e.end - e.begin, dtype, bytes);
    *out = &e;
    return QTIP_OK;
  };
  auto read = [&](const Entry* e, void* dst) -> int {
    CK_REQUIRE(std::fseek(in.f, long(data0 + e->begin), SEEK_SET) == 0 &&
                   std::fread(dst, 1, e->end - e->begin, in.f) == e->end - e->begin,
               QTIP_E_ARG, "qtip_read_layer_linear: short read in %s", path);
    return QTIP_OK;
  };
  const Entry* e = nullptr;
  int rc;
  const long tiles = long(m / 16) * (n / 16);
  if ((rc = find("trellis", "I16", {tiles, 32}, size_t(tiles) * 64, &e)) || (rc = read(e, trellis_h))) return rc;
  {
    std::vector<uint16_t> su(static_cast<size_t>(n));
    if ((rc = find("SU", "BF16", {n}, size_t(n) * 2, &e)) || (rc = read(e, su.data()))) return rc;
    for (int i = 0; i < n; ++i) {
      su_h[i] = bf16_bits_to_float(su[size_t(i)]);
      CK_REQUIRE(std::isfinite(su_h[i]), QTIP_E_ARG, "Nonfinite QTIP vector %sSU", base.c_str());
    }
  }
  if ((rc = find("SV", "F32", {m}, size_t(m) * 4, &e)) || (rc = read(e, sv_h))) return rc;
  for (int i = 0; i < m; ++i) CK_REQUIRE(std::isfinite(sv_h[i]), QTIP_E_ARG, "Nonfinite QTIP vector %sSV", base.c_str());
  if ((rc = find("tlut", "F16", {512, 2}, 2048, &e)) || (rc = read(e, tlut_h))) return rc;
  for (int i = 0; i < 1024; ++i)
    CK_REQUIRE(std::isfinite(f16_bits_to_float(tlut_h[i])), QTIP_E_ARG, "Nonfinite QTIP tlut in %s", base.c_str());
  int64_t rcp = 0, tp = 0;
  if ((rc = find("rcp", "I64", {}, 8, &e)) || (rc = read(e, &rcp))) return rc;
  if ((rc = find("tp_rank", "I64", {}, 8, &e)) || (rc = read(e, &tp))) return rc;
  CK_REQUIRE(rcp == 0, QTIP_E_GEOMETRY, "QTIP rcp != 0 in %s (checkpoints split for tensor parallelism are not supported)",
             base.c_str());
  return QTIP_OK;
}
