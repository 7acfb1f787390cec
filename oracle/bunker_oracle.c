/*
 * bunker_oracle.c -- CPU oracle for the hybrid decode hot path.
 *
 * TEST INFRASTRUCTURE ONLY.  Nothing in the shipped library links, loads or
 * calls this file; it is the checker for the CUDA path (tests, the smoke
 * check, and the reported CPU baseline of the benchmark).
 *
 * PARITY STATUS: "parity unpinned".  The reference (skyne98/bunker) holds no
 * golden vectors for this path: its Q4 tests draw unseeded Math.random()
 * inputs (tests/test_dequant.ts:16-17), its token check needs the real
 * Qwen3.5-0.8B weights (prototypes/decode.ts:933), and it has no 144-byte
 * llama.cpp-layout Q4_K code at all.  No bun/node exists to run its
 * TypeScript.  This file restates the reference's per-op math in C and is
 * pinned by hand-derived known-answer vectors (tests/golden/).
 *
 * Two kinds of function live here:
 *   orc_*_plain : straight restatement of the reference loop (double
 *                 accumulation where the reference relies on JS doubles).
 *                 Pins the semantics; compared at 1e-3 relative.
 *   orc_*       : the same math with every f32 rounding point and every
 *                 reduction order fixed ("canonical order"), so that a GPU
 *                 kernel that uses the same order is bit-identical.  This is
 *                 what makes 256-step greedy token identity a stable test.
 *
 * Build: gcc -O2 -ffp-contract=off -fopenmp -shared -fPIC (see Makefile).
 * -ffp-contract=off is REQUIRED: a*b+c must round twice unless fmaf is spelled.
 *
 * Reference citations are paths inside skyne98/bunker.
 */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>
#ifdef _OPENMP
#include <omp.h>
#endif

#define ORC_API __attribute__((visibility("default")))

/* Threads of the OpenMP loops below.  A launcher may have exported OMP_NUM_THREADS=1 for its worker processes; a
 * caller that times this library as a CPU baseline sets the count it wants and reads back the one in effect. */
ORC_API int orc_set_threads(int n) {
#ifdef _OPENMP
  if (n > 0) omp_set_num_threads(n);
  return omp_get_max_threads();
#else
  (void)n;
  return 1;
#endif
}

/* ------------------------------------------------------------------------ */
/* Number formats                                                           */
/* ------------------------------------------------------------------------ */

static inline uint32_t f2u(float f) { uint32_t u; memcpy(&u, &f, 4); return u; }
static inline float u2f(uint32_t u) { float f; memcpy(&f, &u, 4); return f; }

/* IEEE binary16 -> binary32, subnormals kept.  Used for the Q4_K superblock
 * d / dmin (ggml's Q4_K is a third-party format, absent from the reference;
 * its halves are IEEE). */
ORC_API float orc_f16_to_f32(uint16_t h) {
  uint32_t s = (uint32_t)(h & 0x8000u) << 16;
  uint32_t e = (h >> 10) & 0x1fu, m = h & 0x3ffu;
  if (e == 0) {
    if (m == 0) return u2f(s);
    /* subnormal: m * 2^-24 */
    float v = (float)m * 5.9604644775390625e-08f;
    return (s ? -v : v);
  }
  if (e == 31) return u2f(s | 0x7f800000u | (m << 13));
  return u2f(s | ((e + 112u) << 23) | (m << 13));
}

/* Q8_1 scale encode: the reference's encodeHalf truncates the mantissa and
 * flushes anything below the smallest normal half to signed zero
 * (bench/bench.ts:41-51). */
ORC_API uint16_t orc_f32_to_f16_trunc(float v) {
  if (v == 0.0f) return 0;
  uint32_t bits = f2u(v);
  uint32_t s = (bits >> 16) & 0x8000u, e = (bits >> 23) & 0xffu, m = bits & 0x7fffffu;
  int ne = (int)e - 127 + 15;
  if (ne >= 31) return (uint16_t)(s | 0x7c00u);
  if (ne <= 0) return (uint16_t)s;
  return (uint16_t)(s | ((uint32_t)ne << 10) | (m >> 13));
}

/* Q8_1 scale decode: the reference's half_to_float returns 0 for a zero
 * exponent field (src/dsl.ts:955-975). */
ORC_API float orc_q8half_to_f32(uint16_t h) {
  uint32_t e = (h >> 10) & 0x1fu;
  if (e == 0) return 0.0f;
  return orc_f16_to_f32(h);
}

/* bf16 <-> f32.  Device truncation in the reference is MLIR arith.truncf,
 * round-to-nearest-even (src/ttir.ts:846). */
ORC_API uint16_t orc_f32_to_bf16(float f) {
  uint32_t u = f2u(f);
  if ((u & 0x7fffffffu) > 0x7f800000u) return 0x7fffu; /* canonical NaN, as cvt.rn.bf16.f32 gives */
  u += 0x7fffu + ((u >> 16) & 1u);
  return (uint16_t)(u >> 16);
}
ORC_API float orc_bf16_to_f32(uint16_t h) { return u2f((uint32_t)h << 16); }

/* ------------------------------------------------------------------------ */
/* Deterministic transcendentals (same operation sequence on the GPU)        */
/* ------------------------------------------------------------------------ */

/* exp(x): x clamped to [-87, 88]; n = rint(x*log2e); Cody-Waite reduction in
 * two fmaf steps; Cephes degree-5 polynomial in Horner form with fmaf. */
ORC_API float orc_expf(float x) {
  if (x > 88.0f) x = 88.0f;
  if (x < -87.0f) x = -87.0f;
  float t = x * 1.44269504088896341f;
  float n = rintf(t);
  float r = fmaf(n, -0.693359375f, x);
  r = fmaf(n, 2.12194440e-4f, r);
  float p = 1.9875691500e-4f;
  p = fmaf(p, r, 1.3981999507e-3f);
  p = fmaf(p, r, 8.3334519073e-3f);
  p = fmaf(p, r, 4.1665795894e-2f);
  p = fmaf(p, r, 1.6666665459e-1f);
  p = fmaf(p, r, 5.0000001201e-1f);
  float r2 = r * r;
  float y = fmaf(p, r2, r);
  y = y + 1.0f;
  int32_t ni = (int32_t)n;
  float scale = u2f((uint32_t)(ni + 127) << 23);
  return y * scale;
}

/* log(x) for positive normal x (only ever called on 1+exp(.) >= 1).
 * Cephes logf: mantissa in [sqrt(1/2), sqrt(2)), degree-8 polynomial. */
ORC_API float orc_logf(float x) {
  uint32_t u = f2u(x);
  int32_t e = (int32_t)((u >> 23) & 0xffu) - 126;
  float m = u2f((u & 0x007fffffu) | 0x3f000000u); /* [0.5, 1) */
  if (m < 0.707106781186547524f) {
    e -= 1;
    m = m + m;
  }
  m = m - 1.0f;
  float z = m * m;
  float p = 7.0376836292e-2f;
  p = fmaf(p, m, -1.1514610310e-1f);
  p = fmaf(p, m, 1.1676998740e-1f);
  p = fmaf(p, m, -1.2420140846e-1f);
  p = fmaf(p, m, 1.4249322787e-1f);
  p = fmaf(p, m, -1.6668057665e-1f);
  p = fmaf(p, m, 2.0000714765e-1f);
  p = fmaf(p, m, -2.4999993993e-1f);
  p = fmaf(p, m, 3.3333331174e-1f);
  float y = (m * z) * p;
  float fe = (float)e;
  y = fmaf(fe, -2.12194440e-4f, y);
  y = fmaf(-0.5f, z, y);
  float r = m + y;
  r = fmaf(fe, 0.693359375f, r);
  return r;
}

/* sigmoid as the reference spells it: 1/(1+exp(-x)) (src/emitters.ts:65). */
ORC_API float orc_sigmoidf(float x) { return 1.0f / (1.0f + orc_expf(-x)); }

/* softplus: the reference computes log2(1+e^x)*ln2 (src/emitters.ts:93);
 * here the natural log directly. */
ORC_API float orc_softplusf(float x) { return orc_logf(1.0f + orc_expf(x)); }

/* ------------------------------------------------------------------------ */
/* Canonical reductions                                                     */
/* ------------------------------------------------------------------------ */

/* 32 partials combined the way a warp xor-butterfly (16,8,4,2,1) does. */
static float warp_tree32(const float* p_in) {
  float p[32], q[32];
  memcpy(p, p_in, sizeof(p));
  for (int off = 16; off >= 1; off >>= 1) {
    for (int i = 0; i < 32; i++) q[i] = p[i] + p[i ^ off];
    memcpy(p, q, sizeof(p));
  }
  return p[0];
}

/* Sum of squares over a head of D elements (D = 32*c): lane l owns the c
 * contiguous elements [l*c, l*c+c), accumulates with fmaf, then the tree. */
static float head_sumsq(const float* x, int D) {
  int c = D / 32;
  float part[32];
  for (int l = 0; l < 32; l++) {
    float a = 0.0f;
    for (int e = 0; e < c; e++) a = fmaf(x[l * c + e], x[l * c + e], a);
    part[l] = a;
  }
  return warp_tree32(part);
}

/* Sum of squares over a row of H elements in the 256-thread block order:
 * 8-element chunk q goes to thread q mod 256 (chunks ascending, fmaf inside),
 * each warp reduced by the butterfly, the 8 warp sums added in order. */
static float row_sumsq_block256(const float* x, int H) {
  float part[256];
  for (int t = 0; t < 256; t++) part[t] = 0.0f;
  int nchunk = (H + 7) / 8;
  for (int q = 0; q < nchunk; q++) {
    int t = q & 255;
    float a = part[t];
    for (int e = 0; e < 8; e++) {
      int i = q * 8 + e;
      if (i < H) a = fmaf(x[i], x[i], a);
    }
    part[t] = a;
  }
  float total = 0.0f;
  for (int w = 0; w < 8; w++) {
    float ws = warp_tree32(part + 32 * w);
    total = (w == 0) ? ws : total + ws;
  }
  return total;
}

/* ------------------------------------------------------------------------ */
/* Q4_K (ggml layout, 144-byte superblock of 256 weights)                    */
/* ------------------------------------------------------------------------ */
/* bytes [0,2) f16 d, [2,4) f16 dmin, [4,16) 6-bit scales/mins, [16,144)
 * quants; every 32 quant bytes serve two sub-blocks (low nibbles -> even,
 * high nibbles -> odd).  w = d*sc_j*q - dmin*m_j.  The format is ggml's
 * (third-party, un-pinned by the reference, no version in any lock file);
 * restated from its published description. */

ORC_API void orc_q4k_scales(const uint8_t* sb, uint8_t* sc, uint8_t* mn) {
  const uint8_t* b = sb + 4;
  for (int j = 0; j < 8; j++) {
    if (j < 4) {
      sc[j] = b[j] & 63;
      mn[j] = b[j + 4] & 63;
    } else {
      sc[j] = (uint8_t)((b[j + 4] & 0x0f) | ((b[j - 4] >> 6) << 4));
      mn[j] = (uint8_t)((b[j + 4] >> 4) | ((b[j] >> 6) << 4));
    }
  }
}

static inline uint16_t rd16(const uint8_t* p) { return (uint16_t)(p[0] | (p[1] << 8)); }

/* Dequantise one row of K weights.  Expression form is part of the contract:
 * dl = d*sc, ml = dmin*m, w = dl*q - ml, each operation rounded to f32. */
ORC_API void orc_q4k_dequant_row(const uint8_t* row, int K, float* out) {
  int nsb = K / 256;
  for (int s = 0; s < nsb; s++) {
    const uint8_t* sb = row + (size_t)s * 144;
    float d = orc_f16_to_f32(rd16(sb)), dmin = orc_f16_to_f32(rd16(sb + 2));
    uint8_t sc[8], mn[8];
    orc_q4k_scales(sb, sc, mn);
    const uint8_t* qs = sb + 16;
    for (int p = 0; p < 4; p++) {
      float dl0 = d * (float)sc[2 * p], ml0 = dmin * (float)mn[2 * p];
      float dl1 = d * (float)sc[2 * p + 1], ml1 = dmin * (float)mn[2 * p + 1];
      for (int i = 0; i < 32; i++) {
        uint8_t q = qs[p * 32 + i];
        float lo = dl0 * (float)(q & 15);
        float hi = dl1 * (float)(q >> 4);
        out[s * 256 + p * 64 + i] = lo - ml0;
        out[s * 256 + p * 64 + 32 + i] = hi - ml1;
      }
    }
  }
}


/* ------------------------------------------------------------------------ */
/* f32 -> Q4_K quantiser (the weight side of the loader)                      */
/* ------------------------------------------------------------------------ */
/* The reference loads bf16 safetensors weights and never quantises them (prototypes/decode.ts:64-76); the Q4_K model
 * of this build needs a quantiser, restated here from the published description of the format, not from any
 * implementation: per 32-weight sub-block  lo = min(min x, 0), scale = (max x - lo)/15, mn = -lo;  per 256-weight
 * superblock  d = f16(max scale / 63), dmin = f16(max mn / 63) (round to nearest even), sc = round(scale/d),
 * m = round(mn/dmin) (6 bits each, half up);  q = clamp(round((x + dmin*m) / (d*sc)), 0, 15).  Every operation is a
 * single rounded f32 operation in the order written, so the CUDA quantiser gives the same bytes. */
static uint16_t f32_to_f16_rne(float v) {
  uint32_t x = f2u(v);
  uint32_t sign = (x >> 16) & 0x8000u;
  uint32_t e = (x >> 23) & 0xffu, m = x & 0x7fffffu;
  if (e == 0xffu) return (uint16_t)(sign | 0x7c00u | (m ? 0x200u : 0u));
  int ne = (int)e - 127 + 15;
  if (ne >= 31) return (uint16_t)(sign | 0x7c00u);
  if (ne <= 0) {
    if (ne < -10) return (uint16_t)sign;
    m |= 0x800000u;
    int shift = 14 - ne;                       /* 14..24 */
    uint32_t h = m >> shift;
    uint32_t rem = m & ((1u << shift) - 1u), half = 1u << (shift - 1);
    if (rem > half || (rem == half && (h & 1u))) h++;
    return (uint16_t)(sign | h);
  }
  uint32_t h = ((uint32_t)ne << 10) | (m >> 13);
  uint32_t rem = m & 0x1fffu;
  if (rem > 0x1000u || (rem == 0x1000u && (h & 1u))) h++;   /* a carry into the exponent is the right result */
  return (uint16_t)(sign | h);
}

ORC_API uint16_t orc_f32_to_f16_rne(float v) { return f32_to_f16_rne(v); }

ORC_API void orc_q4k_quantize_row(const float* x, int K, uint8_t* out) {
  int nsb = K / 256;
  for (int s = 0; s < nsb; s++) {
    const float* xs = x + (size_t)s * 256;
    uint8_t* sb = out + (size_t)s * 144;
    float scale[8], mn[8], max_scale = 0.0f, max_min = 0.0f;
    for (int j = 0; j < 8; j++) {
      float lo = xs[j * 32], hi = xs[j * 32];
      for (int i = 1; i < 32; i++) {
        float v = xs[j * 32 + i];
        if (v < lo) lo = v;
        if (v > hi) hi = v;
      }
      if (lo > 0.0f) lo = 0.0f;
      scale[j] = (hi - lo) / 15.0f;
      if (!(scale[j] > 0.0f)) scale[j] = 0.0f;
      mn[j] = 0.0f - lo;
      if (scale[j] > max_scale) max_scale = scale[j];
      if (mn[j] > max_min) max_min = mn[j];
    }
    uint16_t dh = f32_to_f16_rne(max_scale / 63.0f), mh = f32_to_f16_rne(max_min / 63.0f);
    float d = orc_f16_to_f32(dh), dm = orc_f16_to_f32(mh);
    float inv_d = d > 0.0f ? 1.0f / d : 0.0f, inv_dm = dm > 0.0f ? 1.0f / dm : 0.0f;
    uint8_t sc6[8], m6[8];
    for (int j = 0; j < 8; j++) {
      int a = (int)floorf(scale[j] * inv_d + 0.5f), b = (int)floorf(mn[j] * inv_dm + 0.5f);
      sc6[j] = (uint8_t)(a > 63 ? 63 : a);
      m6[j] = (uint8_t)(b > 63 ? 63 : b);
    }
    sb[0] = (uint8_t)(dh & 0xff); sb[1] = (uint8_t)(dh >> 8);
    sb[2] = (uint8_t)(mh & 0xff); sb[3] = (uint8_t)(mh >> 8);
    for (int j = 0; j < 4; j++) {
      sb[4 + j] = (uint8_t)(sc6[j] | ((sc6[j + 4] >> 4) << 6));
      sb[8 + j] = (uint8_t)(m6[j] | ((m6[j + 4] >> 4) << 6));
      sb[12 + j] = (uint8_t)((sc6[j + 4] & 0x0f) | ((m6[j + 4] & 0x0f) << 4));
    }
    for (int p = 0; p < 4; p++) {
      float dl0 = d * (float)sc6[2 * p], ml0 = dm * (float)m6[2 * p];
      float dl1 = d * (float)sc6[2 * p + 1], ml1 = dm * (float)m6[2 * p + 1];
      for (int i = 0; i < 32; i++) {
        int q0 = 0, q1 = 0;
        if (dl0 > 0.0f) {
          q0 = (int)floorf((xs[p * 64 + i] + ml0) / dl0 + 0.5f);
          q0 = q0 < 0 ? 0 : (q0 > 15 ? 15 : q0);
        }
        if (dl1 > 0.0f) {
          q1 = (int)floorf((xs[p * 64 + 32 + i] + ml1) / dl1 + 0.5f);
          q1 = q1 < 0 ? 0 : (q1 > 15 ? 15 : q1);
        }
        sb[16 + p * 32 + i] = (uint8_t)(q0 | (q1 << 4));
      }
    }
  }
}

/* Embedding gather from the tied Q4_K table: X = bf16(dequant(E[id,:]))
 * (reference gathers a bf16 row, src/emitters.ts:31-45). */
ORC_API void orc_embed_q4k(const uint8_t* table, int H, const int32_t* ids, int B, uint16_t* x) {
  float* tmp = (float*)malloc(sizeof(float) * (size_t)H);
  size_t rowb = (size_t)(H / 256) * 144;
  for (int b = 0; b < B; b++) {
    orc_q4k_dequant_row(table + rowb * (size_t)ids[b], H, tmp);
    for (int i = 0; i < H; i++) x[(size_t)b * H + i] = orc_f32_to_bf16(tmp[i]);
  }
  free(tmp);
}

/* ------------------------------------------------------------------------ */
/* Q8_1 activation blocks (reference layout: q[32], f16 d, f16 s = 36 bytes) */
/* ------------------------------------------------------------------------ */
/* packQ8_1, bench/bench.ts:53-72: d = amax/127, q = round-half-up(x/d)
 * clamped to [-128,127], s = (sum q)*d; both halves by truncation.  The JS
 * arithmetic is double; here it is f32, and the quotient is taken as
 * x * (1/d) with one fused multiply-add, q = floor(fma(x, 1/d, 0.5)), which is
 * what the GPU computes (one IEEE division per block instead of 32).  The two
 * forms differ only when x/d lies within an ulp of a half-integer. */
ORC_API void orc_q8_1_quantize(const float* x, int K, uint8_t* out) {
  int nb = K / 32;
  for (int b = 0; b < nb; b++) {
    const float* xb = x + b * 32;
    float amax = 0.0f;
    for (int i = 0; i < 32; i++) {
      float a = fabsf(xb[i]);
      if (a > amax) amax = a;
    }
    float d = amax / 127.0f;
    float id = (d == 0.0f) ? 1.0f : 1.0f / d;
    int32_t sum = 0;
    uint8_t* ob = out + (size_t)b * 36;
    for (int i = 0; i < 32; i++) {
      float v = floorf(fmaf(xb[i], id, 0.5f));
      int32_t q = (int32_t)v;
      sum += q; /* the reference sums before clamping (bench.ts:66-67) */
      if (q > 127) q = 127;
      if (q < -128) q = -128;
      ob[i] = (uint8_t)(int8_t)q;
    }
    uint16_t hd = orc_f32_to_f16_trunc(d);
    uint16_t hs = orc_f32_to_f16_trunc((float)sum * d);
    ob[32] = (uint8_t)(hd & 0xff);
    ob[33] = (uint8_t)(hd >> 8);
    ob[34] = (uint8_t)(hs & 0xff);
    ob[35] = (uint8_t)(hs >> 8);
  }
}

/* bf16 rows -> Q8_1 (the form the fused kernels use between ops). */
ORC_API void orc_q8_1_quantize_bf16(const uint16_t* x, int K, int B, uint8_t* out) {
  float* tmp = (float*)malloc(sizeof(float) * (size_t)K);
  for (int b = 0; b < B; b++) {
    for (int i = 0; i < K; i++) tmp[i] = orc_bf16_to_f32(x[(size_t)b * K + i]);
    orc_q8_1_quantize(tmp, K, out + (size_t)b * (K / 32) * 36);
  }
  free(tmp);
}

/* ------------------------------------------------------------------------ */
/* Integer block dots (bit-exact stage)                                      */
/* ------------------------------------------------------------------------ */
/* Per 32-weight sub-block j of a row: isum_j = sum q4*q8, qsum_j = sum q8
 * (the s1/s2 of the reference's scalar kernel, bench/bench.ts:24-33, with
 * ggml's nibble-to-sub-block assignment instead of the 20-byte toy block). */
ORC_API void orc_block_dots(const uint8_t* wrow, const uint8_t* xq, int K, int32_t* isum, int32_t* qsum) {
  int nsb = K / 256;
  for (int s = 0; s < nsb; s++) {
    const uint8_t* qs = wrow + (size_t)s * 144 + 16;
    for (int p = 0; p < 4; p++) {
      const int8_t* x0 = (const int8_t*)(xq + (size_t)(s * 8 + 2 * p) * 36);
      const int8_t* x1 = (const int8_t*)(xq + (size_t)(s * 8 + 2 * p + 1) * 36);
      int32_t i0 = 0, i1 = 0, s0 = 0, s1 = 0;
      for (int i = 0; i < 32; i++) {
        uint8_t q = qs[p * 32 + i];
        i0 += (int32_t)(q & 15) * x0[i];
        i1 += (int32_t)(q >> 4) * x1[i];
        s0 += x0[i];
        s1 += x1[i];
      }
      isum[s * 8 + 2 * p] = i0;
      isum[s * 8 + 2 * p + 1] = i1;
      qsum[s * 8 + 2 * p] = s0;
      qsum[s * 8 + 2 * p + 1] = s1;
    }
  }
}

/* ------------------------------------------------------------------------ */
/* Q4_K x Q8_1 GEMV                                                          */
/* ------------------------------------------------------------------------ */

/* Canonical row dot.  The row is cut into 64-weight units (one 32-byte quant
 * group = sub-blocks 2p, 2p+1 of superblock s; unit index u = 4s+p).  Unit u
 * belongs to lane u mod 32.  Per unit:
 *   accd = fma(d8_b, f32(sc_b*isum_b), accd)   for b = 2p, 2p+1 (accd from 0)
 *   accm = fma(s8_b, f32(m_b),        accm)    with s8_b = d8_b*f32(qsum_b)
 *   val  = fma(d, accd, -(dmin*accm))
 * Each lane adds its unit values in ascending u, then the butterfly tree.
 * s8_b is exact in f32 (11-bit x 13-bit). */
static float gemv_row_canonical(const uint8_t* wrow, const uint8_t* xq, int K) {
  float lane[32];
  for (int l = 0; l < 32; l++) lane[l] = 0.0f;
  int nunits = K / 64;
  for (int u = 0; u < nunits; u++) {
    int s = u >> 2, p = u & 3;
    const uint8_t* sb = wrow + (size_t)s * 144;
    float d = orc_f16_to_f32(rd16(sb)), dmin = orc_f16_to_f32(rd16(sb + 2));
    uint8_t sc[8], mn[8];
    orc_q4k_scales(sb, sc, mn);
    const uint8_t* qs = sb + 16 + p * 32;
    float accd = 0.0f, accm = 0.0f;
    for (int h = 0; h < 2; h++) {
      int j = 2 * p + h;
      const uint8_t* xb = xq + (size_t)(s * 8 + j) * 36;
      const int8_t* x8 = (const int8_t*)xb;
      int32_t isum = 0, qsum = 0;
      for (int i = 0; i < 32; i++) {
        int q4 = h ? (qs[i] >> 4) : (qs[i] & 15);
        isum += q4 * x8[i];
        qsum += x8[i];
      }
      float d8 = orc_q8half_to_f32(rd16(xb + 32));
      float s8 = d8 * (float)qsum;
      accd = fmaf(d8, (float)((int32_t)sc[j] * isum), accd);
      accm = fmaf(s8, (float)mn[j], accm);
    }
    float t = dmin * accm;
    float val = fmaf(d, accd, -t);
    lane[u & 31] = lane[u & 31] + val;
  }
  return warp_tree32(lane);
}

/* y[b][n] for W[N][K/256][144], xq[B][K/32][36]; f32 pre-epilogue value.
 * Accumulate in f32 as the reference GEMM does (prototypes/decode.ts:141-145). */
ORC_API void orc_gemv_q4k_q8(const uint8_t* W, int N, int K, const uint8_t* xq, int B, float* y) {
  size_t rowb = (size_t)(K / 256) * 144, xb = (size_t)(K / 32) * 36;
#pragma omp parallel for schedule(static)
  for (int n = 0; n < N; n++)
    for (int b = 0; b < B; b++) y[(size_t)b * N + n] = gemv_row_canonical(W + rowb * n, xq + xb * b, K);
}


/* The order of the dense tile path (batch >= 16, tensor-core integer dots): per (row, column) one chain per chunk
 * of four superblocks.  Inside a superblock the eight sub-blocks in ascending order,
 * accd = fma(d8_j, f32(sc_j*isum_j), accd) and accm = fma(s8_j, f32(m_j), accm) from zero; then
 * val = fma(d, accd, -(dmin*accm)); yc = yc + val over the (up to four) superblocks of a chunk in ascending order from
 * zero; y = y + yc over the chunks in ascending order from zero.  (The chunks are what lets a launch of few rows be
 * cut along K over several thread blocks without changing a bit.)  Integer sums are exact either way; only this f32
 * order differs from the lane / butterfly order above (by a few ulp). */
static float gemv_row_tile(const uint8_t* wrow, const uint8_t* xq, int K) {
  float y = 0.0f, yc = 0.0f;
  int nsb = K / 256;
  for (int s = 0; s < nsb; s++) {
    const uint8_t* sb = wrow + (size_t)s * 144;
    float d = orc_f16_to_f32(rd16(sb)), dmin = orc_f16_to_f32(rd16(sb + 2));
    uint8_t sc[8], mn[8];
    orc_q4k_scales(sb, sc, mn);
    float accd = 0.0f, accm = 0.0f;
    for (int j = 0; j < 8; j++) {
      const uint8_t* qs = sb + 16 + (j >> 1) * 32;
      const uint8_t* xb = xq + (size_t)(s * 8 + j) * 36;
      const int8_t* x8 = (const int8_t*)xb;
      int32_t isum = 0, qsum = 0;
      for (int i = 0; i < 32; i++) {
        int q4 = (j & 1) ? (qs[i] >> 4) : (qs[i] & 15);
        isum += q4 * x8[i];
        qsum += x8[i];
      }
      float d8 = orc_q8half_to_f32(rd16(xb + 32));
      float s8 = d8 * (float)qsum;
      accd = fmaf(d8, (float)((int32_t)sc[j] * isum), accd);
      accm = fmaf(s8, (float)mn[j], accm);
    }
    float t = dmin * accm;
    float val = fmaf(d, accd, -t);
    yc = yc + val;
    if ((s & 3) == 3 || s == nsb - 1) {
      y = y + yc;
      yc = 0.0f;
    }
  }
  return y;
}

ORC_API void orc_gemv_q4k_q8_tile(const uint8_t* W, int N, int K, const uint8_t* xq, int B, float* y) {
  size_t rowb = (size_t)(K / 256) * 144, xb = (size_t)(K / 32) * 36;
#pragma omp parallel for schedule(static)
  for (int n = 0; n < N; n++)
    for (int b = 0; b < B; b++) y[(size_t)b * N + n] = gemv_row_tile(W + rowb * n, xq + xb * b, K);
}

/* Plain restatement: dequantise both sides and accumulate in double, the way
 * the reference's host loops run on JS numbers (bench/bench.ts:18-35). */
ORC_API void orc_gemv_q4k_q8_plain(const uint8_t* W, int N, int K, const uint8_t* xq, int B, double* y) {
  size_t rowb = (size_t)(K / 256) * 144, xb = (size_t)(K / 32) * 36;
#pragma omp parallel
  {
    float* w = (float*)malloc(sizeof(float) * (size_t)K);
#pragma omp for schedule(static)
    for (int n = 0; n < N; n++) {
      orc_q4k_dequant_row(W + rowb * n, K, w);
      for (int b = 0; b < B; b++) {
        const uint8_t* xr = xq + xb * b;
        double acc = 0.0;
        for (int k = 0; k < K; k++) {
          const uint8_t* blk = xr + (size_t)(k / 32) * 36;
          double xv = (double)orc_q8half_to_f32(rd16(blk + 32)) * (double)((const int8_t*)blk)[k % 32];
          acc += (double)w[k] * xv;
        }
        y[(size_t)b * N + n] = acc;
      }
    }
    free(w);
  }
}

/* Sum of tensor-parallel partials in rank order, ((p0+p1)+p2)+... */
ORC_API void orc_sum_ranks(const float* parts, int nranks, int n, float* out) {
  for (int i = 0; i < n; i++) {
    float a = parts[i];
    for (int r = 1; r < nranks; r++) a = a + parts[(size_t)r * n + i];
    out[i] = a;
  }
}

/* Epilogues of the fused GEMM kernels (prototypes/decode.ts:148-156):
 * cast = bf16(acc); add = bf16(acc + f32(res)), one rounding. */
ORC_API void orc_epilogue_cast(const float* y, int n, uint16_t* out) {
  for (int i = 0; i < n; i++) out[i] = orc_f32_to_bf16(y[i]);
}
ORC_API void orc_epilogue_add(const float* y, const uint16_t* res, int n, uint16_t* out) {
  for (int i = 0; i < n; i++) out[i] = orc_f32_to_bf16(y[i] + orc_bf16_to_f32(res[i]));
}
/* SwiGLU: bf16((g*sigmoid(g))*u) (prototypes/decode.ts:117-119, src/fusion.ts:324-330). */
ORC_API void orc_swiglu(const float* g, const float* u, int n, uint16_t* out) {
  for (int i = 0; i < n; i++) {
    float sig = orc_sigmoidf(g[i]);
    out[i] = orc_f32_to_bf16((g[i] * sig) * u[i]);
  }
}

/* ------------------------------------------------------------------------ */
/* RMSNorm (Gemma form)                                                     */
/* ------------------------------------------------------------------------ */
/* y = bf16((x * rstd) * (1 + w)), rstd = 1/sqrt(mean(x^2)+eps)
 * (prototypes/decode.ts:208-214, src/fusion.ts:310-322).  The reference uses
 * rsqrt.approx; here IEEE sqrt and divide. */
ORC_API void orc_rmsnorm(const uint16_t* x, const uint16_t* w, int H, int B, float eps, uint16_t* y) {
  float* xf = (float*)malloc(sizeof(float) * (size_t)H);
  for (int b = 0; b < B; b++) {
    for (int i = 0; i < H; i++) xf[i] = orc_bf16_to_f32(x[(size_t)b * H + i]);
    float ss = row_sumsq_block256(xf, H);
    float ms = ss / (float)H;
    float rstd = 1.0f / sqrtf(ms + eps);
    for (int i = 0; i < H; i++) {
      float v = (xf[i] * rstd) * (1.0f + orc_bf16_to_f32(w[i]));
      y[(size_t)b * H + i] = orc_f32_to_bf16(v);
    }
  }
  free(xf);
}

/* Plain: prototypes/rmsnorm.ts:59-67 (double accumulation, exact sqrt). */
ORC_API void orc_rmsnorm_plain(const uint16_t* x, const uint16_t* w, int H, int B, double eps, double* y) {
  for (int b = 0; b < B; b++) {
    double ss = 0.0;
    for (int i = 0; i < H; i++) {
      double v = orc_bf16_to_f32(x[(size_t)b * H + i]);
      ss += v * v;
    }
    double rstd = 1.0 / sqrt(ss / H + eps);
    for (int i = 0; i < H; i++)
      y[(size_t)b * H + i] = orc_bf16_to_f32(x[(size_t)b * H + i]) * rstd * (1.0 + orc_bf16_to_f32(w[i]));
  }
}

/* ------------------------------------------------------------------------ */
/* Causal depthwise conv1d, k=4, SiLU, one decode step                       */
/* ------------------------------------------------------------------------ */
/* src/emitters.ts:48-72.  State is [B][3][C] bf16, oldest first; weights
 * [C][4] bf16.  raw = (w0*s0 + w1*s1) + (w2*s2 + w3*x); out = bf16(raw*sig(raw));
 * new state = [s1, s2, x]. */
ORC_API void orc_conv1d_step(const uint16_t* x, const uint16_t* state, const uint16_t* w, int C, int B,
                             uint16_t* out, uint16_t* state_new) {
  for (int b = 0; b < B; b++) {
    const uint16_t* st = state + (size_t)b * 3 * C;
    uint16_t* sn = state_new + (size_t)b * 3 * C;
    for (int c = 0; c < C; c++) {
      float s0 = orc_bf16_to_f32(st[c]), s1 = orc_bf16_to_f32(st[C + c]), s2 = orc_bf16_to_f32(st[2 * C + c]);
      float xv = orc_bf16_to_f32(x[(size_t)b * C + c]);
      float w0 = orc_bf16_to_f32(w[4 * c]), w1 = orc_bf16_to_f32(w[4 * c + 1]);
      float w2 = orc_bf16_to_f32(w[4 * c + 2]), w3 = orc_bf16_to_f32(w[4 * c + 3]);
      float a0 = w0 * s0, a1 = w1 * s1, a2 = w2 * s2, a3 = w3 * xv;
      float raw = (a0 + a1) + (a2 + a3);
      float o = raw * orc_sigmoidf(raw);
      out[(size_t)b * C + c] = orc_f32_to_bf16(o);
      uint16_t n0 = st[C + c], n1 = st[2 * C + c], n2 = x[(size_t)b * C + c];
      sn[c] = n0;
      sn[C + c] = n1;
      sn[2 * C + c] = n2;
    }
  }
}

/* ------------------------------------------------------------------------ */
/* Gated DeltaNet decode step                                               */
/* ------------------------------------------------------------------------ */
/* src/emitters.ts:75-120 / prototypes/decode.ts:314-388; CPU twin
 * prototypes/gdn_gated.ts:67-88.  conv_out is [B][2*Hk*Dk + Hv*Dv] bf16 laid
 * out q | k | v; S is [B][Hv][Dk][Dv] f32, row = k index.  The reference has
 * Hk == Hv; for Hv > Hk value head hv uses key head hv / (Hv/Hk).
 * Column j (value index) is independent of the others; its two reductions over
 * the Dk = 128 rows use four row groups of 32 rows (serial fmaf inside a
 * group, groups added in order).
 * o_raw receives the un-normalised head output (f32). */
ORC_API void orc_gdn_step(const uint16_t* conv_out, const float* a_in, const float* b_in, const float* A_log,
                          const uint16_t* dt_bias, const float* S_in, int B, int Hk, int Hv, float* S_out,
                          float* o_raw) {
  const int D = 128;
  int keydim = Hk * D, width = 2 * keydim + Hv * D, ratio = Hv / Hk;
#pragma omp parallel for collapse(2) schedule(static)
  for (int b = 0; b < B; b++) {
    for (int hv = 0; hv < Hv; hv++) {
      int hk = hv / ratio;
      const uint16_t* co = conv_out + (size_t)b * width;
      float q[128], k[128], v[128], qn[128], kn[128];
      for (int i = 0; i < D; i++) {
        q[i] = orc_bf16_to_f32(co[hk * D + i]);
        k[i] = orc_bf16_to_f32(co[keydim + hk * D + i]);
        v[i] = orc_bf16_to_f32(co[2 * keydim + hv * D + i]);
      }
      float qr = 1.0f / sqrtf(head_sumsq(q, D) + 1e-6f);
      float kr = 1.0f / sqrtf(head_sumsq(k, D) + 1e-6f);
      float qs = qr * 0.088388347648318441f; /* 1/sqrt(128) */
      for (int i = 0; i < D; i++) {
        qn[i] = q[i] * qs;
        kn[i] = k[i] * kr;
      }
      float sp = orc_softplusf(a_in[(size_t)b * Hv + hv] + orc_bf16_to_f32(dt_bias[hv]));
      float decay = orc_expf(-(orc_expf(A_log[hv]) * sp));
      float beta = orc_sigmoidf(b_in[(size_t)b * Hv + hv]);
      const float* S = S_in + ((size_t)b * Hv + hv) * D * D;
      float* Sn = S_out + ((size_t)b * Hv + hv) * D * D;
      for (int j = 0; j < D; j++) {
        float sd[128];
        float part[4];
        for (int r = 0; r < 4; r++) {
          float acc = 0.0f;
          for (int i = 32 * r; i < 32 * r + 32; i++) {
            sd[i] = S[i * D + j] * decay;
            acc = fmaf(kn[i], sd[i], acc);
          }
          part[r] = acc;
        }
        float kS = ((part[0] + part[1]) + part[2]) + part[3];
        float delta = (v[j] - kS) * beta;
        for (int r = 0; r < 4; r++) {
          float acc = 0.0f;
          for (int i = 32 * r; i < 32 * r + 32; i++) {
            float sn = fmaf(kn[i], delta, sd[i]);
            Sn[i * D + j] = sn;
            acc = fmaf(qn[i], sn, acc);
          }
          part[r] = acc;
        }
        o_raw[((size_t)b * Hv + hv) * D + j] = ((part[0] + part[1]) + part[2]) + part[3];
      }
    }
  }
}

/* Gated RMSNorm of the head output: bf16(((o*rstd)*nw) * (z*sigmoid(z)))
 * (src/emitters.ts:109-118). z is [B][Hv*128] bf16, norm_w f32[128]. */
ORC_API void orc_gdn_gate_norm(const float* o_raw, const uint16_t* z, const float* norm_w, int B, int Hv,
                               uint16_t* out) {
  const int D = 128;
  for (int bh = 0; bh < B * Hv; bh++) {
    const float* o = o_raw + (size_t)bh * D;
    float ms = head_sumsq(o, D) / (float)D;
    float rstd = 1.0f / sqrtf(ms + 1e-6f);
    for (int j = 0; j < D; j++) {
      float zv = orc_bf16_to_f32(z[(size_t)bh * D + j]);
      float zs = zv * orc_sigmoidf(zv);
      float ow = (o[j] * rstd) * norm_w[j];
      out[(size_t)bh * D + j] = orc_f32_to_bf16(ow * zs);
    }
  }
}

/* Plain recurrence in double: prototypes/gdn_gated.ts:67-88 with the gating
 * of src/emitters.ts:88-97 (exact libm). Inputs already f32. */
ORC_API void orc_gdn_step_plain(const float* q, const float* k, const float* v, double decay, double beta,
                                const float* S_in, double* S_out, double* o) {
  const int D = 128;
  double qss = 1e-6, kss = 1e-6;
  for (int i = 0; i < D; i++) {
    qss += (double)q[i] * q[i];
    kss += (double)k[i] * k[i];
  }
  double qr = 1.0 / sqrt(qss) / sqrt((double)D), kr = 1.0 / sqrt(kss);
  for (int j = 0; j < D; j++) {
    double kS = 0.0;
    for (int i = 0; i < D; i++) kS += k[i] * kr * (S_in[i * D + j] * decay);
    double delta = (v[j] - kS) * beta;
    double acc = 0.0;
    for (int i = 0; i < D; i++) {
      double sn = S_in[i * D + j] * decay + k[i] * kr * delta;
      S_out[i * D + j] = sn;
      acc += q[i] * qr * sn;
    }
    o[j] = acc;
  }
}

/* ------------------------------------------------------------------------ */
/* Per-head q/k RMSNorm + partial rotary                                     */
/* ------------------------------------------------------------------------ */
/* qnorm/knorm: src/emitters.ts:123-147 -> bf16((x*rstd)*(1+w)) over HD dims;
 * then RoPE in place on the bf16 buffer, src/emitters.ts:150-183: pairs
 * (i, i+rot_half), x1' = x1*c - x2*s, x2' = x2*c + x1*s, f32 tables
 * [max_len][rot_half] (prototypes/decode.ts:865-871).
 * in: [B][nheads][in_stride] bf16 starting at in_off inside each head slot
 * (q_proj output interleaves q and gate per head: stride 2*HD). */
ORC_API void orc_headnorm_rope(const uint16_t* in, int in_stride, const uint16_t* w, const float* cos_t,
                               const float* sin_t, int rot_half, const int32_t* pos, int B, int nheads, int HD,
                               uint16_t* out) {
  float x[512];
  for (int b = 0; b < B; b++) {
    for (int h = 0; h < nheads; h++) {
      const uint16_t* src = in + ((size_t)b * nheads + h) * in_stride;
      uint16_t* dst = out + ((size_t)b * nheads + h) * HD;
      for (int i = 0; i < HD; i++) x[i] = orc_bf16_to_f32(src[i]);
      float ms = head_sumsq(x, HD) / (float)HD;
      float rstd = 1.0f / sqrtf(ms + 1e-6f);
      for (int i = 0; i < HD; i++) dst[i] = orc_f32_to_bf16((x[i] * rstd) * (1.0f + orc_bf16_to_f32(w[i])));
      const float* c = cos_t + (size_t)pos[b] * rot_half;
      const float* s = sin_t + (size_t)pos[b] * rot_half;
      for (int i = 0; i < rot_half; i++) {
        float x1 = orc_bf16_to_f32(dst[i]), x2 = orc_bf16_to_f32(dst[i + rot_half]);
        float a = x1 * c[i], bb = x2 * s[i], cc = x2 * c[i], dd = x1 * s[i];
        dst[i] = orc_f32_to_bf16(a - bb);
        dst[i + rot_half] = orc_f32_to_bf16(cc + dd);
      }
    }
  }
}

/* Table builder used by tests (double math, rounded to f32), as the reference
 * fills its Float32Array (prototypes/decode.ts:865-871). */
ORC_API void orc_rope_tables(int max_len, int rot_dim, double theta, float* cos_t, float* sin_t) {
  int half = rot_dim / 2;
  for (int p = 0; p < max_len; p++)
    for (int i = 0; i < half; i++) {
      double freq = 1.0 / pow(theta, 2.0 * i / rot_dim);
      cos_t[(size_t)p * half + i] = (float)cos(p * freq);
      sin_t[(size_t)p * half + i] = (float)sin(p * freq);
    }
}

/* ------------------------------------------------------------------------ */
/* Decode attention over a bf16 KV cache (GQA, split-KV)                     */
/* ------------------------------------------------------------------------ */
/* Math of src/emitters.ts:188-226 restricted to the valid rows 0..pos:
 * s_j = (q.K_j)*scale, softmax, o = sum w_j V_j, out = bf16(o*sigmoid(gate)).
 * Cache is per KV head: [B][Hkv][max_len][HD] bf16 (the reference replicates
 * it per q head, emitters.ts:202).  The caller appends K/V at row pos first.
 *
 * Canonical order.  n = pos+1 rows are cut into splits of split_len rows.
 * Inside a split, row jj (relative) belongs to warp jj mod W.  A score is the
 * per-lane fmaf chain over the lane's 8 contiguous dims (lane l: dims
 * [l*HD/32, ...)), butterfly tree, times scale.  m = max over the split
 * (order-free).  p = exp(s-m).  Each warp adds p (for l) and fmaf(p, v, acc)
 * (for o) over its rows in ascending order; warps are added in order 0..W-1.
 * Splits are merged with M = max m_s, w_s = exp(m_s-M), L = fma(w_s,l_s,L),
 * O = fma(w_s,o_s,O) in ascending s; out = (O/L)*sigmoid(gate). */
static void attn_split(const float* q, const uint16_t* Kc, const uint16_t* Vc, int HD, int j0, int j1, float scale,
                       int W, float* m_out, float* l_out, float* o_out, float* sbuf) {
  int c = HD / 32;
  int n = j1 - j0;
  float m = -INFINITY;
  for (int jj = 0; jj < n; jj++) {
    const uint16_t* kr = Kc + (size_t)(j0 + jj) * HD;
    float part[32];
    for (int l = 0; l < 32; l++) {
      float a = 0.0f;
      for (int e = 0; e < c; e++) a = fmaf(q[l * c + e], orc_bf16_to_f32(kr[l * c + e]), a);
      part[l] = a;
    }
    float s = warp_tree32(part) * scale;
    sbuf[jj] = s;
    if (s > m) m = s;
  }
  float l_tot = 0.0f;
  for (int d = 0; d < HD; d++) o_out[d] = 0.0f;
  float* acc = (float*)malloc(sizeof(float) * (size_t)HD);
  for (int w = 0; w < W; w++) {
    float lw = 0.0f;
    for (int d = 0; d < HD; d++) acc[d] = 0.0f;
    for (int jj = w; jj < n; jj += W) {
      float p = orc_expf(sbuf[jj] - m);
      lw = lw + p;
      const uint16_t* vr = Vc + (size_t)(j0 + jj) * HD;
      for (int d = 0; d < HD; d++) acc[d] = fmaf(p, orc_bf16_to_f32(vr[d]), acc[d]);
    }
    if (w == 0) {
      l_tot = lw;
      for (int d = 0; d < HD; d++) o_out[d] = acc[d];
    } else {
      l_tot = l_tot + lw;
      for (int d = 0; d < HD; d++) o_out[d] = o_out[d] + acc[d];
    }
  }
  free(acc);
  *m_out = m;
  *l_out = l_tot;
}

ORC_API void orc_attn_decode(const uint16_t* q, const uint16_t* gate, int gate_stride, const uint16_t* Kc,
                             const uint16_t* Vc, const int32_t* pos, int B, int Hq, int Hkv, int HD, int max_len,
                             int split_len, int W, float scale, uint16_t* out) {
  int G = Hq / Hkv;
#pragma omp parallel for collapse(2) schedule(dynamic)
  for (int b = 0; b < B; b++) {
    for (int h = 0; h < Hq; h++) {
      int n = pos[b] + 1;
      int nsplit = (n + split_len - 1) / split_len;
      int kvh = h / G;
      const uint16_t* Kb = Kc + ((size_t)b * Hkv + kvh) * (size_t)max_len * HD;
      const uint16_t* Vb = Vc + ((size_t)b * Hkv + kvh) * (size_t)max_len * HD;
      float qf[512];
      for (int d = 0; d < HD; d++) qf[d] = orc_bf16_to_f32(q[((size_t)b * Hq + h) * HD + d]);
      float* ms = (float*)malloc(sizeof(float) * (size_t)nsplit * (2 + HD));
      float* ls = ms + nsplit;
      float* os = ls + nsplit;
      float* sbuf = (float*)malloc(sizeof(float) * (size_t)split_len);
      float M = -INFINITY;
      for (int s = 0; s < nsplit; s++) {
        int j0 = s * split_len, j1 = j0 + split_len;
        if (j1 > n) j1 = n;
        attn_split(qf, Kb, Vb, HD, j0, j1, scale, W, &ms[s], &ls[s], os + (size_t)s * HD, sbuf);
        if (ms[s] > M) M = ms[s];
      }
      float L = 0.0f;
      float O[512];
      for (int d = 0; d < HD; d++) O[d] = 0.0f;
      for (int s = 0; s < nsplit; s++) {
        float w = orc_expf(ms[s] - M);
        L = fmaf(w, ls[s], L);
        for (int d = 0; d < HD; d++) O[d] = fmaf(w, os[(size_t)s * HD + d], O[d]);
      }
      for (int d = 0; d < HD; d++) {
        float g = orc_bf16_to_f32(gate[((size_t)b * Hq + h) * gate_stride + d]);
        out[((size_t)b * Hq + h) * HD + d] = orc_f32_to_bf16((O[d] / L) * orc_sigmoidf(g));
      }
      free(sbuf);
      free(ms);
    }
  }
}

/* Plain: prototypes/fa2_vllm.ts:114-139 for the last row, double math, plus
 * the output gate of src/emitters.ts:221-224; ungated f64 output. */
ORC_API void orc_attn_decode_plain(const uint16_t* q, const uint16_t* Kc, const uint16_t* Vc, int n, int HD,
                                   double scale, double* out) {
  double* s = (double*)malloc(sizeof(double) * (size_t)n);
  double m = -1e300;
  for (int j = 0; j < n; j++) {
    double a = 0.0;
    for (int d = 0; d < HD; d++) a += (double)orc_bf16_to_f32(q[d]) * orc_bf16_to_f32(Kc[(size_t)j * HD + d]);
    s[j] = a * scale;
    if (s[j] > m) m = s[j];
  }
  double l = 0.0;
  for (int j = 0; j < n; j++) {
    s[j] = exp(s[j] - m);
    l += s[j];
  }
  for (int d = 0; d < HD; d++) {
    double a = 0.0;
    for (int j = 0; j < n; j++) a += s[j] / l * orc_bf16_to_f32(Vc[(size_t)j * HD + d]);
    out[d] = a;
  }
  free(s);
}


/* ------------------------------------------------------------------------ */
/* Sampling (temperature / top-k / top-p)                                     */
/* ------------------------------------------------------------------------ */
/* The reference decodes greedily only (prototypes/decode.ts:749-791).  Sampling as the library defines it: the top_k
 * largest logits (ties to the lower index) in descending order; p_i = exp((l_i - l_0)/T) summed in that order; the
 * shortest prefix reaching top_p * total; u from splitmix64 of (seed, step, sequence); first i whose running sum
 * exceeds u * prefix total. */
static uint64_t splitmix64(uint64_t x) {
  x += 0x9E3779B97F4A7C15ull;
  x = (x ^ (x >> 30)) * 0xBF58476D1CE4E5B9ull;
  x = (x ^ (x >> 27)) * 0x94D049BB133111EBull;
  return x ^ (x >> 31);
}

ORC_API void orc_sample(const float* logits, int V, int B, float temperature, int top_k, float top_p, uint64_t seed,
                        const int32_t* step, uint32_t step_add, int32_t* idx, float* val) {
  for (int b = 0; b < B; b++) {
    const float* l = logits + (size_t)b * V;
    float cv[64];
    int ci[64];
    float pv = INFINITY;
    int pi = -1, k = 0;
    for (int r = 0; r < top_k && r < 64; r++) {
      float bv = -INFINITY;
      int bi = 0x7fffffff;
      for (int i = 0; i < V; i++) {
        float v = l[i];
        if (v != v) continue;
        if (!(v < pv || (v == pv && i > pi))) continue;
        if (v > bv || (v == bv && i < bi)) { bv = v; bi = i; }
      }
      if (bi == 0x7fffffff) break;
      cv[r] = bv; ci[r] = bi; pv = bv; pi = bi; k = r + 1;
    }
    if (k == 0) { idx[b] = 0; if (val) val[b] = -INFINITY; continue; }
    int pick = 0;
    if (temperature > 0.0f && k > 1) {
      float pr[64];
      float inv_t = 1.0f / temperature, total = 0.0f;
      for (int i = 0; i < k; i++) { pr[i] = orc_expf((cv[i] - cv[0]) * inv_t); total = total + pr[i]; }
      float need = top_p * total, run = 0.0f;
      int n = k;
      for (int i = 0; i < k; i++) { run = run + pr[i]; if (run >= need) { n = i + 1; break; } }
      float prefix = 0.0f;
      for (int i = 0; i < n; i++) prefix = prefix + pr[i];
      uint32_t st = (step ? (uint32_t)step[b] : 0u) + step_add;
      uint64_t h = splitmix64(splitmix64(seed ^ ((uint64_t)st << 20)) + (uint64_t)b);
      float u = (float)(uint32_t)(h >> 40) * 5.9604644775390625e-8f;
      float target = u * prefix;
      pick = n - 1;
      run = 0.0f;
      for (int i = 0; i < n; i++) { run = run + pr[i]; if (run > target) { pick = i; break; } }
    }
    idx[b] = ci[pick];
    if (val) val[b] = cv[pick];
  }
}

/* ------------------------------------------------------------------------ */
/* Argmax                                                                   */
/* ------------------------------------------------------------------------ */
/* Exact maximum, lowest index on ties (strict '>' scan,
 * prototypes/decode.ts:776-784).  The reference's per-chunk index-sum quirk
 * (decode.ts:760-763) and the -1000 initial value (src/emitters.ts:235) are
 * not reproduced. */
ORC_API void orc_argmax(const float* logits, int V, int B, int32_t* idx, float* val) {
  for (int b = 0; b < B; b++) {
    const float* l = logits + (size_t)b * V;
    float best = l[0];
    int32_t bi = 0;
    for (int i = 1; i < V; i++)
      if (l[i] > best) {
        best = l[i];
        bi = i;
      }
    idx[b] = bi;
    val[b] = best;
  }
}
