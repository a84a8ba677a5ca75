/*
 * TEST INFRASTRUCTURE ONLY -- CPU restatement of the reference's QTIP trellis codec hot path.
 *
 * This file is the checker that the CUDA kernels are compared against. It is never linked into, imported by or
 * called from the product library; only the test suite, the smoke check and the CPU-baseline leg of the benchmark
 * load it.
 *
 * Parity is pinned: the functions below are checked against the reference's committed golden vectors
 * (tests/refvec/{vit_x,vit_states,vit_hat,lut,perm,pack_*,had_*,ldl_*}.bin of the reference tree) and against the
 * reference's own C++ compiled in place (see the Makefile target `ref`), by tests/test_oracle_*.py.
 *
 * Each function cites the reference file:line it restates (paths relative to the reference project root).
 * Plain C, fp32 arithmetic written so that the compiler cannot re-associate it (-ffp-contract=off, fmaf = one
 * rounding).
 */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

#define QO_STATES 65536
#define QO_GROUPS 4096
#define QO_STEPS 128
#define QO_SEQ 256

/* ------------------------------------------------------------------------------------------------ conversions */

static inline uint32_t f2u(float f) { uint32_t u; memcpy(&u, &f, 4); return u; }
static inline float u2f(uint32_t u) { float f; memcpy(&f, &u, 4); return f; }

/* fp16 <-> fp32, round to nearest even. Follows src/common.hpp:50-79. */
float qo_f16_to_f32(uint16_t h) {
  uint32_t s = (h >> 15) & 1, e = (h >> 10) & 0x1f, m = h & 0x3ff;
  float v;
  if (e == 0) v = ldexpf((float)m, -24);
  else if (e == 31) v = m ? NAN : INFINITY;
  else v = ldexpf((float)(m | 0x400), (int)e - 25);
  return s ? -v : v;
}
uint16_t qo_f32_to_f16(float f) {
  uint32_t u = f2u(f);
  uint32_t sign = (u >> 16) & 0x8000u, a = u & 0x7fffffffu;
  if (a >= 0x7f800000u) return (uint16_t)(sign | 0x7c00u | (a > 0x7f800000u ? 0x200u : 0u));
  if (a >= 0x477ff000u) return (uint16_t)(sign | 0x7c00u);
  if (a < 0x38800000u) { /* subnormal or zero in fp16: value / 2^-24 rounded to nearest even */
    float q = u2f(a) * 16777216.0f;
    float r = nearbyintf(q);
    return (uint16_t)(sign | (uint32_t)r);
  }
  uint32_t e = (a >> 23) - 112, m = a & 0x7fffffu;
  uint32_t h = (e << 10) | (m >> 13), rem = m & 0x1fffu;
  if (rem > 0x1000u || (rem == 0x1000u && (h & 1u))) h++;
  return (uint16_t)(sign | h);
}
static inline float round_f16(float f) { return qo_f16_to_f32(qo_f32_to_f16(f)); }

/* bf16 <-> fp32 RNE. Follows src/common.hpp:38-49 and runtime/cuda/kernels.cu:11-14. */
uint16_t qo_f32_to_bf16(float f) {
  uint32_t u = f2u(f);
  if ((u & 0x7fffffffu) > 0x7f800000u) return (uint16_t)((u >> 16) | 0x40);
  u += 0x7fffu + ((u >> 16) & 1u);
  return (uint16_t)(u >> 16);
}
float qo_bf16_to_f32(uint16_t h) { return u2f((uint32_t)h << 16); }

/* ------------------------------------------------------------------------------------------------ codebook */

/* quantlut_sym expansion of a tlut (fp16 bits, [512][2]) to the 65,536-entry packed half2 table.
 * Follows src/qtip_core.cpp:18-46 (build_codebook). lut_rms may be NULL. */
void qo_build_lut(const uint16_t* tlut_h, uint32_t* lut_h2, double* lut_rms) {
  double ss = 0;
  for (uint32_t s = 0; s < QO_STATES; ++s) {
    uint64_t p = (uint64_t)(s + 1) * (uint64_t)s;
    int flip = (int)((p >> 15) & 1);
    int idx = (int)((p >> 6) & 511);
    uint16_t h0 = tlut_h[idx * 2], h1 = tlut_h[idx * 2 + 1];
    if (flip) h0 ^= 0x8000;
    lut_h2[s] = (uint32_t)h0 | ((uint32_t)h1 << 16);
    double a = qo_f16_to_f32(h0), b = qo_f16_to_f32(h1);
    ss += a * a + b * b;
  }
  if (lut_rms) *lut_rms = sqrt(ss / (2.0 * QO_STATES));
}

/* Runtime codebook: 1,024 sign-folded entries e = sign<<9 | idx with fp16-exact floats and the bf16x2 device word.
 * Follows runtime/src/qtip.cpp:62-80 (make_codebook). Returns 0, or -1 on a non-finite entry. */
int qo_runtime_codebook(const uint16_t* tlut_h, float* c0, float* c1, uint32_t* bf16x2) {
  for (int e = 0; e < 1024; ++e) {
    int idx = e & 511, flip = e >> 9;
    uint16_t h0 = tlut_h[idx * 2], h1 = tlut_h[idx * 2 + 1];
    if (flip) h0 ^= 0x8000u;
    c0[e] = qo_f16_to_f32(h0);
    c1[e] = qo_f16_to_f32(h1);
    if (!isfinite(c0[e]) || !isfinite(c1[e])) return -1;
    bf16x2[e] = (uint32_t)qo_f32_to_bf16(c0[e]) | ((uint32_t)qo_f32_to_bf16(c1[e]) << 16);
  }
  return 0;
}

/* LUT entry of a 16-bit state; bits above 15 of `state` are ignored. runtime/include/behemoth/qtip.hpp:39-42. */
int qo_lut_entry(uint32_t state) {
  uint32_t s = state & 0xffffu;
  return (int)(((s * (s + 1)) >> 6) & 1023u);
}

/* _PERMUTE: sequence position p -> tile index 16 r + c, and its inverse. src/qtip_core.cpp:54-73,
 * src/viterbi.hip:40-47. */
static inline int perm_fwd(int p) {
  int e = p & 1, a = (p >> 1) & 1, c = (p >> 2) & 1, d = (p >> 3) & 3, b = (p >> 5) & 7;
  return a * 128 + b * 16 + c * 8 + d * 2 + e;
}
static inline int perm_inv(int q) {
  int a = q >> 7, b = (q >> 4) & 7, c = (q >> 3) & 1, d = (q >> 1) & 3, e = q & 1;
  return (((b * 4 + d) * 2 + c) * 2 + a) * 2 + e;
}
void qo_perm(int* perm, int* inv) {
  for (int p = 0; p < 256; ++p) { perm[p] = perm_fwd(p); inv[p] = perm_inv(p); }
}

/* ------------------------------------------------------------------------------------------------ exact Viterbi */

typedef struct {
  float* l0;  /* [65536] component 0 as fp32 */
  float* l1;  /* [65536] component 1 */
  float* nrm; /* [65536] l0*l0 + l1*l1, one rounding */
} lut_f32;

static lut_f32 expand_lut(const uint32_t* lut_h2) {
  lut_f32 t;
  t.l0 = (float*)malloc(QO_STATES * 4);
  t.l1 = (float*)malloc(QO_STATES * 4);
  t.nrm = (float*)malloc(QO_STATES * 4);
  for (int s = 0; s < QO_STATES; ++s) {
    float a = qo_f16_to_f32((uint16_t)lut_h2[s]), b = qo_f16_to_f32((uint16_t)(lut_h2[s] >> 16));
    t.l0[s] = a;
    t.l1[s] = b;
    t.nrm[s] = a * a + b * b;
  }
  return t;
}
static void free_lut(lut_f32* t) { free(t->l0); free(t->l1); free(t->nrm); }

/* One forward pass for one sequence: the arithmetic of the CUDA branch of viterbi_fwd_kernel,
 * src/viterbi.hip:49-188. A: [127][1024] uint16 (4 nibbles), returns the final state. */
static uint16_t viterbi_fwd_one(const float* xb, int ov, int roll, uint16_t* A, const lut_f32* t) {
  float xs[QO_SEQ];
  float M[2][QO_GROUPS], t0[QO_GROUPS];
  for (int i = 0; i < QO_SEQ; ++i) xs[i] = round_f16(roll ? xb[(i + 128) & 255] : xb[i]); /* :59 */
  for (int k = 0; k < QO_GROUPS; ++k) M[0][k] = (ov < 0 || k == ov) ? 0.f : 1e30f;       /* :100-101 */
  int cur = 0;
  for (int i = 0; i < 127; ++i) { /* :105-143 */
    const float x0 = xs[2 * i], x1 = xs[2 * i + 1];
    const float m0 = round_f16(-2.f * x0), m1 = round_f16(-2.f * x1);
    const float xx = x0 * x0 + x1 * x1;
    float* best = M[cur ^ 1];
    for (int k = 0; k < QO_GROUPS; ++k) { t0[k] = M[cur][k] + xx; best[k] = 3e30f; }
    for (int d = 0; d < 16; ++d) {
      const float *l0 = t->l0 + (d << 12), *l1 = t->l1 + (d << 12), *nr = t->nrm + (d << 12);
      for (int g = 0; g < 256; ++g) {
        const float mp = t0[(d << 8) | g];
        for (int q = 0; q < 16; ++q) {
          int j = (g << 4) | q;
          float c = fmaf(l1[j], m1, fmaf(l0[j], m0, nr[j] + mp)); /* q_dot2(v, xm2, norm + mp), :26-28,128 */
          float tg = u2f((f2u(c) & ~15u) | (uint32_t)d);          /* :132 */
          best[j] = tg < best[j] ? tg : best[j];                   /* fminf, no NaN can occur */
        }
      }
    }
    for (int tq = 0; tq < 1024; ++tq) { /* :136-142 */
      uint32_t pk = 0;
      for (int q = 0; q < 4; ++q) {
        uint32_t bb = f2u(best[(tq << 2) | q]);
        pk |= (bb & 15u) << (4 * q);
        best[(tq << 2) | q] = u2f(bb & ~15u);
      }
      A[i * 1024 + tq] = (uint16_t)pk;
    }
    cur ^= 1;
  }
  /* last step: untagged costs, end constraint, lowest state on ties, :145-187 */
  const float x0 = xs[254], x1 = xs[255];
  const float m0 = round_f16(-2.f * x0), m1 = round_f16(-2.f * x1);
  const float xx = x0 * x0 + x1 * x1;
  float bv = 3e30f;
  uint32_t bs = 0;
  for (uint32_t s = 0; s < QO_STATES; ++s) {
    if (ov >= 0 && (int)(s & 0xfff) != ov) continue;
    float mp = M[cur][s >> 4] + xx;
    float c = fmaf(t->l1[s], m1, fmaf(t->l0[s], m0, t->nrm[s] + mp));
    if (c < bv) { bv = c; bs = s; } /* ascending s: strict < keeps the lowest state */
  }
  return (uint16_t)bs;
}

static inline uint32_t prev_state(const uint16_t* Ab, int i, uint32_t s) { /* src/viterbi.hip:190-195 */
  uint32_t j = s >> 4;
  uint32_t w = Ab[i * 1024 + (j >> 2)];
  uint32_t d = (w >> (4 * (j & 3))) & 15u;
  return j | (d << 12);
}

/* k_viterbi_fwd, src/viterbi.hip:275-279: B sequences, same buffers as the device kernel. */
void qo_viterbi_fwd(const float* X, const int* overlap, int roll, int B, uint16_t* A, uint16_t* final_state,
                    const uint32_t* lut_h2) {
  lut_f32 t = expand_lut(lut_h2);
#pragma omp parallel for schedule(dynamic, 1)
  for (int b = 0; b < B; ++b)
    final_state[b] =
        viterbi_fwd_one(X + (size_t)b * 256, overlap ? overlap[b] : -1, roll, A + (size_t)b * 127 * 1024, &t);
  free_lut(&t);
}
/* k_viterbi_overlap, src/viterbi.hip:197-205. */
void qo_viterbi_overlap(const uint16_t* A, const uint16_t* final_state, int B, int* overlap) {
  for (int b = 0; b < B; ++b) {
    const uint16_t* Ab = A + (size_t)b * 127 * 1024;
    uint32_t s = final_state[b];
    for (int i = 126; i >= 64; --i) s = prev_state(Ab, i, s);
    overlap[b] = (int)(s >> 4);
  }
}
/* k_viterbi_finish, src/viterbi.hip:207-229. Q and hatWT may each be NULL. */
void qo_viterbi_finish(const uint16_t* A, const uint16_t* final_state, int B, int b0, uint16_t* Q, int nblk, int blk,
                       float* hatWT, long m, int col0, const uint32_t* lut_h2) {
  for (int b = 0; b < B; ++b) {
    const uint16_t* Ab = A + (size_t)b * 127 * 1024;
    long row0 = (long)(b0 + b) * 16;
    uint16_t* q = Q ? Q + ((size_t)(b0 + b) * nblk + blk) * 128 : NULL;
    uint32_t s = final_state[b];
    for (int i = 127; i >= 0; --i) {
      if (i < 127) s = prev_state(Ab, i, s);
      if (q) q[i] = (uint16_t)s;
      if (hatWT) {
        uint32_t u = lut_h2[s];
        for (int e = 0; e < 2; ++e) {
          int tq = perm_fwd(2 * i + e), r = tq >> 4, c = tq & 15;
          hatWT[(long)(col0 + c) * m + row0 + r] = qo_f16_to_f32((uint16_t)(e ? u >> 16 : u));
        }
      }
    }
  }
}
/* k_decode_states, src/viterbi.hip:231-238. */
void qo_decode_states(const uint16_t* st, int B, float* hat, const uint32_t* lut_h2) {
  for (long i = 0; i < (long)B * 128; ++i) {
    uint32_t u = lut_h2[st[i]];
    hat[2 * i] = qo_f16_to_f32((uint16_t)u);
    hat[2 * i + 1] = qo_f16_to_f32((uint16_t)(u >> 16));
  }
}

/* Two-pass tail-biting quantisation of B sequences with the exact kernel arithmetic: the call sequence of
 * src/quantizer.cpp:59-62 (fwd roll=1 -> overlap -> fwd with overlap -> finish). states [B][128], hat [B][256]
 * (sequence order); either output may be NULL. */
void qo_quantize_tiles(const float* X, int B, const uint32_t* lut_h2, uint16_t* states, float* hat) {
  lut_f32 t = expand_lut(lut_h2);
#pragma omp parallel
  {
    uint16_t* A = (uint16_t*)malloc((size_t)127 * 1024 * 2);
#pragma omp for schedule(dynamic, 1)
    for (int b = 0; b < B; ++b) {
      const float* xb = X + (size_t)b * 256;
      uint16_t fs = viterbi_fwd_one(xb, -1, 1, A, &t);
      int ov;
      qo_viterbi_overlap(A, &fs, 1, &ov);
      fs = viterbi_fwd_one(xb, ov, 0, A, &t);
      uint16_t st[128];
      qo_viterbi_finish(A, &fs, 1, 0, st, 1, 0, NULL, 0, 0, lut_h2);
      if (states) memcpy(states + (size_t)b * 128, st, 256);
      if (hat) qo_decode_states(st, 1, hat + (size_t)b * 256, lut_h2);
    }
    free(A);
  }
  free_lut(&t);
}

/* ------------------------------------------------------------------------------------------------ fp64 Viterbi */

static inline double sq_err(const lut_f32* t, uint32_t s, double x0, double x1) { /* src/qtip_core.cpp:123-127 */
  double a = t->l0[s] - x0, b = t->l1[s] - x1;
  return a * a + b * b;
}
/* viterbi_ref, src/qtip_core.cpp:129-170: exact fp64 Viterbi, strict '<' tie-breaks. */
static double viterbi_ref_one(const lut_f32* t, const float* X, int overlap, uint16_t* states) {
  double* cost = (double*)malloc(QO_STATES * 8);
  double* ncost = (double*)malloc(QO_STATES * 8);
  double* M = (double*)malloc(QO_GROUPS * 8);
  uint8_t* A = (uint8_t*)malloc((size_t)QO_STEPS * QO_GROUPS);
  for (uint32_t s = 0; s < QO_STATES; ++s) {
    cost[s] = sq_err(t, s, X[0], X[1]);
    if (overlap >= 0 && (int)(s >> 4) != overlap) cost[s] = INFINITY;
  }
  for (int i = 1; i < QO_STEPS; ++i) {
    for (int j = 0; j < QO_GROUPS; ++j) {
      double best = cost[j];
      int bd = 0;
      for (int d = 1; d < 16; ++d) {
        double c = cost[j | (d << 12)];
        if (c < best) { best = c; bd = d; }
      }
      M[j] = best;
      A[(size_t)i * QO_GROUPS + j] = (uint8_t)bd;
    }
    double x0 = X[2 * i], x1 = X[2 * i + 1];
    for (uint32_t s = 0; s < QO_STATES; ++s) ncost[s] = sq_err(t, s, x0, x1) + M[s >> 4];
    double* tmp = cost; cost = ncost; ncost = tmp;
  }
  double best = INFINITY;
  uint32_t bs = 0;
  for (uint32_t s = 0; s < QO_STATES; ++s) {
    if (overlap >= 0 && (int)(s & 0xfff) != overlap) continue;
    if (cost[s] < best) { best = cost[s]; bs = s; }
  }
  states[QO_STEPS - 1] = (uint16_t)bs;
  for (int i = QO_STEPS - 1; i > 0; --i) {
    uint32_t j = states[i] >> 4;
    states[i - 1] = (uint16_t)(j | ((uint32_t)A[(size_t)i * QO_GROUPS + j] << 12));
  }
  free(cost); free(ncost); free(M); free(A);
  return best;
}
/* quantize_seq_ref, src/qtip_core.cpp:180-191, over B sequences. cost may be NULL. */
void qo_quantize_seq_ref(const float* X, int B, const uint32_t* lut_h2, uint16_t* states, float* hat, double* cost) {
  lut_f32 t = expand_lut(lut_h2);
#pragma omp parallel for schedule(dynamic, 1)
  for (int b = 0; b < B; ++b) {
    const float* x = X + (size_t)b * 256;
    float R[QO_SEQ];
    for (int i = 0; i < QO_SEQ; ++i) R[i] = x[(i - 128 + QO_SEQ) % QO_SEQ];
    uint16_t st1[QO_STEPS];
    viterbi_ref_one(&t, R, -1, st1);
    int overlap = st1[64] >> 4;
    uint16_t* st = states + (size_t)b * 128;
    double c = viterbi_ref_one(&t, x, overlap, st);
    if (cost) cost[b] = c;
    if (hat) qo_decode_states(st, 1, hat + (size_t)b * 256, lut_h2);
  }
  free_lut(&t);
}
/* path_cost, src/qtip_core.cpp:174-178. */
double qo_path_cost(const float* X, const uint16_t* states, const uint32_t* lut_h2) {
  double c = 0;
  for (int i = 0; i < QO_STEPS; ++i) {
    uint32_t u = lut_h2[states[i]];
    double a = qo_f16_to_f32((uint16_t)u) - (double)X[2 * i], b = qo_f16_to_f32((uint16_t)(u >> 16)) - (double)X[2 * i + 1];
    c += a * a + b * b;
  }
  return c;
}

/* ------------------------------------------------------------------------------------------------ packing */

/* pack_trellis, src/qtip_core.cpp:194-208: state 0 (16 bits, MSB first) then the low 4 bits of each later state;
 * the first 512 bits are kept. */
void qo_pack_trellis(const uint16_t* states, long B, uint16_t* packed) {
  for (long b = 0; b < B; ++b) {
    const uint16_t* st = states + b * 128;
    uint16_t* out = packed + b * 32;
    memset(out, 0, 64);
    int pos = 0;
    for (int i = 15; i >= 0; --i, ++pos)
      if ((st[0] >> i) & 1) out[pos >> 4] |= (uint16_t)(1u << (15 - (pos & 15)));
    for (int t = 1; t < 128; ++t)
      for (int i = 3; i >= 0; --i, ++pos)
        if (pos < 512 && ((st[t] >> i) & 1)) out[pos >> 4] |= (uint16_t)(1u << (15 - (pos & 15)));
  }
}
/* unpack_trellis, src/qtip_core.cpp:210-228: bit positions wrap modulo 512. */
void qo_unpack_trellis(const uint16_t* packed, long B, uint16_t* states) {
  for (long b = 0; b < B; ++b) {
    const uint16_t* in = packed + b * 32;
    uint16_t* st = states + b * 128;
    uint32_t s = 0;
    for (int i = 0; i < 16; ++i) s = (s << 1) | ((in[i >> 4] >> (15 - (i & 15))) & 1u);
    st[0] = (uint16_t)s;
    for (int t = 1; t < 128; ++t) {
      uint32_t e = 0;
      for (int i = 0; i < 4; ++i) {
        int pos = (16 + (t - 1) * 4 + i) % 512;
        e = (e << 1) | ((in[pos >> 4] >> (15 - (pos & 15))) & 1u);
      }
      s = ((s << 4) & 0xffffu) | e;
      st[t] = (uint16_t)s;
    }
  }
}
/* swizzle_for_kernel / unswizzle_for_kernel, src/qtip_core.cpp:233-253. Returns -1 unless m, n are multiples of 32. */
int qo_swizzle(const uint16_t* packed, int m, int n, uint16_t* out) {
  if (m % 32 || n % 32) return -1;
  long nb = n / 16, M2 = m / 32, N2 = n / 32;
  for (long i0 = 0; i0 < M2; ++i0)
    for (long j0 = 0; j0 < N2; ++j0)
      for (int c = 0; c < 32; ++c)
        for (int j1 = 0; j1 < 2; ++j1)
          for (int i1 = 0; i1 < 2; ++i1)
            out[(((i0 * N2 + j0) * 32 + c) * 2 + j1) * 2 + i1] = packed[((2 * i0 + i1) * nb + 2 * j0 + j1) * 32 + c];
  return 0;
}
int qo_unswizzle(const uint16_t* in, int m, int n, uint16_t* packed) {
  if (m % 32 || n % 32) return -1;
  long nb = n / 16, M2 = m / 32, N2 = n / 32;
  for (long i0 = 0; i0 < M2; ++i0)
    for (long j0 = 0; j0 < N2; ++j0)
      for (int c = 0; c < 32; ++c)
        for (int j1 = 0; j1 < 2; ++j1)
          for (int i1 = 0; i1 < 2; ++i1)
            packed[((2 * i0 + i1) * nb + 2 * j0 + j1) * 32 + c] = in[(((i0 * N2 + j0) * 32 + c) * 2 + j1) * 2 + i1];
  return 0;
}

/* ------------------------------------------------------------------------------------------------ Hadamard */

/* The order-12, order-20 and order-28 factors used by the codec are Paley matrices; they are constructed here from
 * quadratic residues and compared entry by entry with the reference's committed tables (kHad12, kHad20, kHad28 of
 * src/qtip_constants.hpp) by the test suite. Returns 0, or -1 for an unsupported order. H is K x K row-major +-1. */
static int legendre(int a, int p) {
  a %= p;
  if (a < 0) a += p;
  if (a == 0) return 0;
  for (int x = 1; x < p; ++x)
    if ((x * x) % p == a) return 1;
  return -1;
}
int qo_had_table(int K, int8_t* H) {
  if (K == 12 || K == 20) { /* Paley I, q = K-1: bordered circulant with first row [1, -chi(k)] */
    int q = K - 1;
    for (int i = 0; i < K; ++i)
      for (int j = 0; j < K; ++j) {
        int v;
        if (i == 0) v = j == 0 ? 1 : -1;
        else if (j == 0) v = 1;
        else { int k = ((j - i) % q + q) % q; v = k == 0 ? 1 : -legendre(k, q); }
        H[i * K + j] = (int8_t)v;
      }
    return 0;
  }
  if (K == 28) { /* Paley II, q = 13: 2x2 arrangement of bordered 14x14 circulants */
    const int q = 13, h = 14;
    for (int i = 0; i < K; ++i)
      for (int j = 0; j < K; ++j) {
        int bi = i / h, bj = j / h, r = i % h, c = j % h, v;
        int k = ((c - r) % q + q) % q; /* circulant offset for the 13x13 core (r, c >= 1) */
        int chi = (r >= 1 && c >= 1 && k != 0) ? legendre(k, q) : 0;
        if (bi == 0 && bj == 0) v = (r == 0 || c == 0) ? 1 : (k == 0 ? 1 : chi);
        else if (bi != bj) v = (r == 0) ? (c == 0 ? -1 : 1) : (c == 0 ? 1 : (k == 0 ? -1 : chi));
        else v = (r == 0 || c == 0) ? -1 : (k == 0 ? -1 : -chi);
        H[i * K + j] = (int8_t)v;
      }
    return 0;
  }
  return -1;
}
/* get_hadK restricted to the orders this build carries (12, 20, 28; 1 for a power of two; 0 = unsupported).
 * Divisibility order as src/qtip_core.cpp:77-81 with kHadOrder = {172,...,28,20,12}: a larger listed order that
 * divides n but is not carried here makes the size unsupported. */
int qo_had_K(int n) {
  static const int order[12] = {172, 156, 140, 124, 116, 108, 60, 52, 36, 28, 20, 12};
  for (int i = 0; i < 12; ++i)
    if (n % order[i] == 0) {
      long p = n / order[i];
      if (p <= 0 || (p & (p - 1))) return 0;
      return (order[i] == 28 || order[i] == 20 || order[i] == 12) ? order[i] : 0;
    }
  return (n > 0 && (n & (n - 1)) == 0) ? 1 : 0;
}
/* hadamard_rows_ref, src/qtip_core.cpp:83-120: x <- (hadK^(T) (x) H_P) x / sqrt(n) per row, fp64. */
int qo_hadamard_rows_ref(double* X, long rows, int n, long ld, int transpose) {
  int K = qo_had_K(n);
  if (K <= 0) return -1;
  int8_t hk[28 * 28];
  if (K > 1) qo_had_table(K, hk);
  int P = n / K;
  double sc = 1.0 / sqrt((double)n);
#pragma omp parallel for schedule(static)
  for (long r = 0; r < rows; ++r) {
    double* x = X + r * ld;
    double* y = (double*)malloc((size_t)n * 8);
    double* z = (double*)malloc((size_t)n * 8);
    memcpy(y, x, (size_t)n * 8);
    for (int c = 0; c < K; ++c) {
      double* v = y + (long)c * P;
      for (int h = 1; h < P; h <<= 1)
        for (int i = 0; i < P; i += 2 * h)
          for (int j = i; j < i + h; ++j) {
            double a = v[j], b = v[j + h];
            v[j] = a + b;
            v[j + h] = a - b;
          }
    }
    if (K > 1) {
      for (int k2 = 0; k2 < K; ++k2)
        for (int i = 0; i < P; ++i) {
          double s = 0;
          for (int k = 0; k < K; ++k) s += (transpose ? hk[k * K + k2] : hk[k2 * K + k]) * y[(long)k * P + i];
          z[(long)k2 * P + i] = s;
        }
      for (int i = 0; i < n; ++i) x[i] = z[i] * sc;
    } else {
      for (int i = 0; i < n; ++i) x[i] = y[i] * sc;
    }
    free(y); free(z);
  }
  return 0;
}

/* ------------------------------------------------------------------------------------------------ LDLQ */

/* k_ldlq_prep, src/viterbi.hip:241-267: in-buffer feedback in fp32 (fmaf, k ascending), permuted into sequences. */
void qo_ldlq_prep(const float* WT, const float* hatWT, const float* prod, const float* L, long n, long m, int col0,
                  int bufend, float* X) {
  const int k0 = col0 + 16, nk = bufend - k0;
#pragma omp parallel for schedule(static)
  for (long j = 0; j < m; ++j) {
    float acc[16];
    for (int c = 0; c < 16; ++c) acc[c] = WT[(long)(col0 + c) * m + j] + prod[(long)(col0 + c) * m + j];
    for (int kk = 0; kk < nk; ++kk) {
      long o = (long)(k0 + kk) * m + j;
      float dk = WT[o] - hatWT[o];
      for (int c = 0; c < 16; ++c) acc[c] = fmaf(L[(long)(k0 + kk) * n + col0 + c], dk, acc[c]);
    }
    float* xb = X + (j >> 4) * 256;
    int r = (int)(j & 15);
    for (int c = 0; c < 16; ++c) xb[perm_inv(r * 16 + c)] = acc[c];
  }
}

/* ldlq_gpu, src/quantizer.cpp:30-89, with the device kernels replaced by their restatements above. The
 * cross-buffer update prod[0:c0] += L[c0:c0+128, 0:c0]^T (WT - hatWT)[c0:c0+128] is done with one fp32 fmaf per
 * term, k ascending (the reference uses a split-bf16 library GEMM there, which is not bit-reproducible; any
 * scheme at least as accurate as fp32 is an accepted replacement). hatWT [n][m], Q [(m/16)(n/16)][128]. */
int qo_ldlq_f32(const float* WT, const float* L, long n, long m, float* hatWT, uint16_t* Q, const uint32_t* lut_h2) {
  if (n % 128 || m % 16) return -1;
  const long ntr = m / 16;
  const int nblk = (int)(n / 16);
  float* prod = (float*)calloc((size_t)n * m, 4);
  float* X = (float*)malloc((size_t)ntr * 256 * 4);
  uint16_t* st = (uint16_t*)malloc((size_t)ntr * 128 * 2);
  float* hat = (float*)malloc((size_t)ntr * 256 * 4);
  memset(hatWT, 0, (size_t)n * m * 4);
  for (long cur = n / 16; cur > 0; cur -= 8) {
    const int bufend = (int)(16 * cur), c0 = bufend - 128;
    for (int i = 7; i >= 0; --i) {
      const int col0 = c0 + 16 * i;
      qo_ldlq_prep(WT, hatWT, prod, L, n, m, col0, bufend, X);
      qo_quantize_tiles(X, (int)ntr, lut_h2, st, hat);
      for (long b = 0; b < ntr; ++b) {
        memcpy(Q + ((size_t)b * nblk + col0 / 16) * 128, st + b * 128, 256);
        for (int p = 0; p < 256; ++p) {
          int tq = perm_fwd(p), r = tq >> 4, c = tq & 15;
          hatWT[(long)(col0 + c) * m + b * 16 + r] = hat[b * 256 + p];
        }
      }
    }
    if (c0 > 0) {
#pragma omp parallel for schedule(static)
      for (long r = 0; r < c0; ++r)
        for (long j = 0; j < m; ++j) {
          float acc = prod[r * m + j];
          for (long k = c0; k < bufend; ++k) acc = fmaf(L[k * n + r], WT[k * m + j] - hatWT[k * m + j], acc);
          prod[r * m + j] = acc;
        }
    }
  }
  free(prod); free(X); free(st); free(hat);
  return 0;
}

/* ldlq_ref, tests/test_gpu.cpp:181-225: fp64 port of the upstream LDLQ (128-column buffers) on top of the fp64
 * Viterbi; each sequence is rounded to fp16 before quantisation. Wr [m][n] row-major, hatWr [m][n]. */
int qo_ldlq_ref(const float* Wr, const float* L, int m, int n, float* hatWr, uint16_t* Q, const uint32_t* lut_h2) {
  if (n % 128 || m % 16) return -1;
  size_t nm = (size_t)n * m;
  double* WT = (double*)malloc(nm * 8);
  double* hT = (double*)calloc(nm, 8);
  double* prod = (double*)calloc(nm, 8);
  double* WX = (double*)malloc((size_t)16 * m * 8);
  float* X = (float*)malloc((size_t)(m / 16) * 256 * 4);
  float* H = (float*)malloc((size_t)(m / 16) * 256 * 4);
  uint16_t* st = (uint16_t*)malloc((size_t)(m / 16) * 128 * 2);
  for (int i = 0; i < m; ++i)
    for (int j = 0; j < n; ++j) WT[(size_t)j * m + i] = Wr[(size_t)i * n + j];
  for (int cur = n / 16; cur > 0; cur -= 8) {
    int bufend = 16 * cur, c0 = bufend - 128;
    for (int bi = 7; bi >= 0; --bi) {
      int col0 = c0 + 16 * bi;
      for (int c = 0; c < 16; ++c)
        for (int j = 0; j < m; ++j) {
          double v = WT[(size_t)(col0 + c) * m + j] + prod[(size_t)(col0 + c) * m + j];
          for (int k = col0 + 16; k < bufend; ++k)
            v += (double)L[(size_t)k * n + col0 + c] * (WT[(size_t)k * m + j] - hT[(size_t)k * m + j]);
          WX[(size_t)c * m + j] = v;
        }
      for (int b = 0; b < m / 16; ++b)
        for (int p = 0; p < 256; ++p) {
          int q = perm_fwd(p), r = q >> 4, c = q & 15;
          X[(size_t)b * 256 + p] = round_f16((float)WX[(size_t)c * m + 16 * b + r]);
        }
      qo_quantize_seq_ref(X, m / 16, lut_h2, st, H, NULL);
      for (int b = 0; b < m / 16; ++b) {
        for (int p = 0; p < 256; ++p) {
          int q = perm_fwd(p), r = q >> 4, c = q & 15;
          hT[(size_t)(col0 + c) * m + 16 * b + r] = H[(size_t)b * 256 + p];
        }
        memcpy(Q + ((size_t)b * (n / 16) + col0 / 16) * 128, st + (size_t)b * 128, 256);
      }
    }
    for (int r = 0; r < c0; ++r)
      for (int k = c0; k < bufend; ++k) {
        double l = L[(size_t)k * n + r];
        if (l == 0) continue;
        for (int j = 0; j < m; ++j) prod[(size_t)r * m + j] += l * (WT[(size_t)k * m + j] - hT[(size_t)k * m + j]);
      }
  }
  for (int i = 0; i < m; ++i)
    for (int j = 0; j < n; ++j) hatWr[(size_t)i * n + j] = (float)hT[(size_t)j * m + i];
  free(WT); free(hT); free(prod); free(WX); free(X); free(H); free(st);
  return 0;
}

/* block_ldl_to_L, src/qtip_core.cpp:444-487, with an unblocked fp64 Cholesky in place of the reference's blocked
 * AVX-512 one (same factor up to rounding). A: n x n fp64 row-major, lower triangle used, destroyed.
 * L_out: strictly block-lower fp32. Returns 0, -1 if not positive definite, -2 for a bad size. */
int qo_block_ldl(double* A, int n, float* L_out) {
  if (n % 16) return -2;
  for (int j = 0; j < n; ++j) {
    double d = A[(size_t)j * n + j];
    for (int p = 0; p < j; ++p) d -= A[(size_t)j * n + p] * A[(size_t)j * n + p];
    if (!(d > 0)) return -1;
    d = sqrt(d);
    A[(size_t)j * n + j] = d;
#pragma omp parallel for schedule(static) if (n - j > 256)
    for (int i = j + 1; i < n; ++i) {
      double s = A[(size_t)i * n + j];
      for (int p = 0; p < j; ++p) s -= A[(size_t)i * n + p] * A[(size_t)j * n + p];
      A[(size_t)i * n + j] = s / d;
    }
  }
  int nb = n / 16;
  double* inv = (double*)malloc((size_t)nb * 256 * 8);
  for (int bi = 0; bi < nb; ++bi) {
    double D[16][16], Iv[16][16];
    for (int i = 0; i < 16; ++i)
      for (int j = 0; j < 16; ++j) D[i][j] = j <= i ? A[(size_t)(bi * 16 + i) * n + bi * 16 + j] : 0.0;
    for (int c = 0; c < 16; ++c)
      for (int i = 0; i < 16; ++i) {
        double s = (i == c) ? 1.0 : 0.0;
        for (int p = 0; p < i; ++p) s -= D[i][p] * Iv[p][c];
        Iv[i][c] = s / D[i][i];
      }
    for (int i = 0; i < 16; ++i)
      for (int j = 0; j < 16; ++j) inv[(size_t)bi * 256 + i * 16 + j] = Iv[i][j];
  }
  for (int r = 0; r < n; ++r) {
    int rb = r / 16;
    for (int bj = 0; bj < nb; ++bj) {
      float* o = L_out + (size_t)r * n + bj * 16;
      if (bj >= rb) { memset(o, 0, 64); continue; }
      const double* a = A + (size_t)r * n + bj * 16;
      const double* iv = inv + (size_t)bj * 256;
      for (int j = 0; j < 16; ++j) {
        double s = 0;
        for (int p = j; p < 16; ++p) s += a[p] * iv[p * 16 + j];
        o[j] = (float)s;
      }
    }
  }
  free(inv);
  return 0;
}

/* ------------------------------------------------------------------------------------------------ decode side */

/* Kernel-layout word c of tile (tr, tc): HostLinear::word, runtime/include/behemoth/qtip.hpp:63-67. */
static inline uint16_t kword(const uint16_t* trellis, int in, int tr, int tc, int c) {
  size_t i0 = (size_t)(tr / 2), i1 = (size_t)(tr % 2), j0 = (size_t)(tc / 2), j1 = (size_t)(tc % 2), n2 = (size_t)(in / 32);
  return trellis[(((i0 * n2 + j0) * 32 + (size_t)c) * 2 + j1) * 2 + i1];
}
/* decode_rows / decode_rows_bf16, runtime/src/qtip.cpp:83-128: rows [row0, row0+rows) of the rotated weight,
 * row-major rows x in, from component tables c0/c1 (1,024 entries each; fp16-exact or bf16-exact values).
 * Returns -1 on a geometry violation. */
int qo_decode_rows(const uint16_t* trellis, int in, int out, const float* c0, const float* c1, int row0, int rows,
                   float* w) {
  if (row0 % 16 || rows % 16 || row0 < 0 || row0 + rows > out || in % 32 || out % 32) return -1;
  const int tiles_c = in / 16;
#pragma omp parallel for schedule(static)
  for (int tr = row0 / 16; tr < (row0 + rows) / 16; ++tr)
    for (int tc = 0; tc < tiles_c; ++tc) {
      uint16_t wd[32];
      for (int c = 0; c < 32; ++c) wd[c] = kword(trellis, in, tr, tc, c);
      for (int t = 0; t < 128; ++t) {
        int i = t >> 2, s = 4 * (t & 3);
        uint32_t u = (uint32_t)wd[i] << 16 | wd[(i + 1) & 31];
        int e = qo_lut_entry(u >> (16 - s));
        int A = t >> 4, B = (t >> 2) & 3, C = (t >> 1) & 1, D = t & 1;
        int r = D * 8 + A, col = C * 8 + B * 2;
        float* o = w + (size_t)(tr * 16 - row0 + r) * (size_t)in + (size_t)(tc * 16 + col);
        o[0] = c0[e];
        o[1] = c1[e];
      }
    }
  return 0;
}

/* hadamard, runtime/src/qtip.cpp:25-56: one vector in place, fp64 (orders 1, 12, 28 only, as the runtime). */
static int rt_hadamard(double* x, int n, int transpose, double* y) {
  int k = qo_had_K(n);
  if (k != 1 && k != 12 && k != 28) return -1;
  int p = n / k;
  int8_t h[28 * 28];
  if (k > 1) qo_had_table(k, h);
  for (int c = 0; c < k; ++c) {
    double* v = x + (size_t)c * p;
    for (int s = 1; s < p; s <<= 1)
      for (int i = 0; i < p; i += 2 * s)
        for (int j = i; j < i + s; ++j) {
          double a = v[j], b = v[j + s];
          v[j] = a + b;
          v[j + s] = a - b;
        }
  }
  double scale = 1 / sqrt((double)n);
  if (k == 1) {
    for (int i = 0; i < n; ++i) x[i] *= scale;
    return 0;
  }
  memset(y, 0, (size_t)n * 8);
  for (int r = 0; r < k; ++r)
    for (int c = 0; c < k; ++c) {
      int sign = transpose ? h[c * k + r] : h[r * k + c];
      const double* src = x + (size_t)c * p;
      double* dst = y + (size_t)r * p;
      for (int i = 0; i < p; ++i) dst[i] += sign * src[i];
    }
  for (int i = 0; i < n; ++i) x[i] = y[i] * scale;
  return 0;
}
int qo_rt_hadamard(double* x, int n, int transpose) {
  double* y = (double*)malloc((size_t)n * 8);
  int r = rt_hadamard(x, n, transpose, y);
  free(y);
  return r;
}

/* reference_forward, runtime/src/qtip.cpp:129-192 (QTIP branch): y = SV (.) hadU_out(hadUt_in(x (.) SU) . What^T)
 * in double; device_rounding = bf16 rotated input + bf16 LUT; round_z_bf16 rounds z before the output transform.
 * x [rows][in] f32 -> y [rows][out] f32. Optional z_out [rows][out] receives the rotated products (as float).
 * Returns 0 or -1. */
int qo_reference_forward(const uint16_t* trellis, const float* su, const float* sv, const uint16_t* tlut_h, int in,
                         int out, const float* x, int rows, int device_rounding, int round_z_bf16, float* y,
                         float* z_out) {
  float c0[1024], c1[1024];
  uint32_t b2[1024];
  if (qo_runtime_codebook(tlut_h, c0, c1, b2)) return -1;
  if (device_rounding)
    for (int e = 0; e < 1024; ++e) { c0[e] = u2f((b2[e] & 0xffffu) << 16); c1[e] = u2f(b2[e] & 0xffff0000u); }
  int nmax = in > out ? in : out;
  double* u = (double*)malloc((size_t)rows * in * 8);
  double* tmp = (double*)malloc((size_t)nmax * 8);
  for (int r = 0; r < rows; ++r) {
    double* v = u + (size_t)r * in;
    for (int i = 0; i < in; ++i) v[i] = (double)x[(size_t)r * in + i] * su[i];
    if (rt_hadamard(v, in, 1, tmp)) { free(u); free(tmp); return -1; }
    if (device_rounding)
      for (int i = 0; i < in; ++i) v[i] = (double)qo_bf16_to_f32(qo_f32_to_bf16((float)v[i]));
  }
  double* z = (double*)calloc((size_t)rows * out, 8);
  const int block = 256;
  float* w = (float*)malloc((size_t)block * in * 4);
  for (int r0 = 0; r0 < out; r0 += block) {
    int nr = block < out - r0 ? block : out - r0;
    if (qo_decode_rows(trellis, in, out, c0, c1, r0, nr, w)) { free(u); free(tmp); free(z); free(w); return -1; }
#pragma omp parallel for schedule(static)
    for (int o = 0; o < nr; ++o)
      for (int r = 0; r < rows; ++r) {
        double s = 0;
        const float* wr = w + (size_t)o * in;
        const double* ur = u + (size_t)r * in;
        for (int i = 0; i < in; ++i) s += (double)wr[i] * ur[i];
        z[(size_t)r * out + r0 + o] = s;
      }
  }
  for (int r = 0; r < rows; ++r) {
    double* v = z + (size_t)r * out;
    if (round_z_bf16)
      for (int o = 0; o < out; ++o) v[o] = (double)qo_bf16_to_f32(qo_f32_to_bf16((float)v[o]));
    if (z_out)
      for (int o = 0; o < out; ++o) z_out[(size_t)r * out + o] = (float)v[o];
    if (rt_hadamard(v, out, 0, tmp)) { free(u); free(tmp); free(z); free(w); return -1; }
    for (int o = 0; o < out; ++o) y[(size_t)r * out + o] = (float)(v[o] * sv[o]);
  }
  free(u); free(tmp); free(z); free(w);
  return 0;
}

/* FP8 e4m3 (OCP fn: 0x7f/0xff NaN, bias 7) -> fp32. src/common.hpp:81-88, runtime/cuda/kernels.cu:15-22. */
float qo_fp8e4m3_to_f32(uint8_t b) {
  uint32_t s = b >> 7, e = (b >> 3) & 0xf, m = b & 7;
  float v;
  if (e == 0) v = ldexpf((float)m, -9);
  else if (e == 15 && m == 7) v = NAN;
  else v = ldexpf((float)(m | 8), (int)e - 10);
  return s ? -v : v;
}
/* FP8 branch of reference_forward, runtime/src/qtip.cpp:134-149: y = float(sum_i bf16(x_i) * fp8(w_oi)) * scale_o. */
void qo_fp8_forward(const uint8_t* w, const float* scale, int in, int out, const float* x, int rows,
                    int device_rounding, float* y) {
#pragma omp parallel for schedule(static)
  for (int o = 0; o < out; ++o)
    for (int r = 0; r < rows; ++r) {
      double sum = 0;
      for (int i = 0; i < in; ++i) {
        float v = x[(size_t)r * in + i];
        if (device_rounding) v = qo_bf16_to_f32(qo_f32_to_bf16(v));
        sum += (double)v * qo_fp8e4m3_to_f32(w[(size_t)o * in + i]);
      }
      y[(size_t)r * out + o] = (float)sum * scale[o];
    }
}
