// bk_common.cuh -- device-side numerics shared by every kernel of libbunker_cuda.
//
// Every f32 rounding point is spelled out (explicit __fmul_rn/__fadd_rn/fmaf)
// and the file is compiled with -fmad=false, so a*b+c never fuses by accident.
// The CPU checker mirrors the same operation sequences; that is what makes the
// kernels bit-reproducible on a host.
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

#define BK_DEVINL __device__ __forceinline__

// ---- programmatic dependent launch -------------------------------------------
// trigger: lets the next kernel on the stream start its own pre-wait part now.
// wait   : returns once every earlier kernel has completed and its writes are visible.
BK_DEVINL void bk_pdl_trigger() { asm volatile("griddepcontrol.launch_dependents;"); }
BK_DEVINL void bk_pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }

// ---- device-side timeline (bkTraceEnable): thread 0 of CTA 0 stamps the global timer ----
BK_DEVINL void bk_stamp(unsigned long long* rec, int slot) {
  if (rec && blockIdx.x == 0 && blockIdx.y == 0 && blockIdx.z == 0 && threadIdx.x == 0) {
    unsigned long long t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    rec[slot] = t;
  }
}

// lane 0 of every warp folds its exit time into the record (slot = latest exit of the whole grid)
BK_DEVINL void bk_stamp_max(unsigned long long* rec, int slot) {
  if (rec && (threadIdx.x & 31) == 0) {
    unsigned long long t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    atomicMax(rec + slot, t);
  }
}

// ---- mbarrier + bulk async copy (global -> this CTA's shared memory, no multicast) ----
BK_DEVINL uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
BK_DEVINL void mbar_init(uint32_t bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
BK_DEVINL void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
BK_DEVINL void bulk_g2s(uint32_t dst, const void* src, uint32_t bytes, uint32_t bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(dst),
               "l"(src), "r"(bytes), "r"(bar)
               : "memory");
}
BK_DEVINL bool mbar_try_wait(uint32_t bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{ .reg .pred p; mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2; selp.u32 %0, 1, 0, p; }"
      : "=r"(ok)
      : "r"(bar), "r"(parity)
      : "memory");
  return ok != 0;
}
// bounded: a copy that never lands sets the status word instead of hanging the GPU
BK_DEVINL void mbar_wait_bounded(uint32_t bar, uint32_t parity, int* status) {
  for (int it = 0; it < (1 << 22); it++)
    if (mbar_try_wait(bar, parity)) return;
  if (status) atomicExch(status, 10003 /* BK_ERR_TIMEOUT */);
}

// {a.x*b.x + c.x, a.y*b.y + c.y}: two IEEE fused multiply-adds in one instruction (one issue slot instead of two)
BK_DEVINL float2 bk_fma2(float2 a, float2 b, float2 c) {
  unsigned long long ra, rb, rc, rd;
  asm("mov.b64 %0, {%1, %2};" : "=l"(ra) : "f"(a.x), "f"(a.y));
  asm("mov.b64 %0, {%1, %2};" : "=l"(rb) : "f"(b.x), "f"(b.y));
  asm("mov.b64 %0, {%1, %2};" : "=l"(rc) : "f"(c.x), "f"(c.y));
  asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(rd) : "l"(ra), "l"(rb), "l"(rc));
  float2 d;
  asm("mov.b64 {%0, %1}, %2;" : "=f"(d.x), "=f"(d.y) : "l"(rd));
  return d;
}

// ---- bf16 / f16 -----------------------------------------------------------

BK_DEVINL float bk_bf16_to_f32(uint16_t h) { return __uint_as_float((uint32_t)h << 16); }

// round-to-nearest-even, NaN kept quiet (MLIR arith.truncf semantics of the
// reference's device casts, src/ttir.ts:846)
BK_DEVINL uint16_t bk_f32_to_bf16(float f) {
  uint16_t h;
  asm("cvt.rn.bf16.f32 %0, %1;" : "=h"(h) : "f"(f));
  return h;
}
// two values -> packed pair (lo in the low half), one instruction
BK_DEVINL uint32_t bk_f32x2_to_bf16x2(float lo, float hi) {
  uint32_t r;
  asm("cvt.rn.bf16x2.f32 %0, %1, %2;" : "=r"(r) : "f"(hi), "f"(lo));
  return r;
}

// IEEE half -> float, subnormals kept (Q4_K superblock d / dmin)
BK_DEVINL float bk_f16_to_f32(uint16_t h) {
  float f;
  asm("{ .reg .b16 t; mov.b16 t, %1; cvt.f32.f16 %0, t; }" : "=f"(f) : "h"(h));
  return f;
}

// Q8_1 scale encode: truncate the mantissa, flush below-normal to signed zero
// (the reference's encodeHalf, bench/bench.ts:41-51)
BK_DEVINL uint16_t bk_f32_to_f16_trunc(float v) {
  if (v == 0.0f) return 0;
  uint32_t bits = __float_as_uint(v);
  uint32_t s = (bits >> 16) & 0x8000u, e = (bits >> 23) & 0xffu, m = bits & 0x7fffffu;
  int ne = (int)e - 127 + 15;
  if (ne >= 31) return (uint16_t)(s | 0x7c00u);
  if (ne <= 0) return (uint16_t)s;
  return (uint16_t)(s | ((uint32_t)ne << 10) | (m >> 13));
}

// Q8_1 scale decode: zero exponent field reads as 0 (the reference's
// half_to_float, src/dsl.ts:955-975)
BK_DEVINL float bk_q8half_to_f32(uint16_t h) {
  if (((h >> 10) & 0x1fu) == 0) return 0.0f;
  return bk_f16_to_f32(h);
}

// ---- deterministic transcendentals ----------------------------------------

BK_DEVINL float bk_expf(float x) {
  if (x > 88.0f) x = 88.0f;
  if (x < -87.0f) x = -87.0f;
  float t = __fmul_rn(x, 1.44269504088896341f);
  float n = rintf(t);
  float r = fmaf(n, -0.693359375f, x);
  r = fmaf(n, 2.12194440e-4f, r);
  float p = 1.9875691500e-4f;
  p = fmaf(p, r, 1.3981999507e-3f);
  p = fmaf(p, r, 8.3334519073e-3f);
  p = fmaf(p, r, 4.1665795894e-2f);
  p = fmaf(p, r, 1.6666665459e-1f);
  p = fmaf(p, r, 5.0000001201e-1f);
  float r2 = __fmul_rn(r, r);
  float y = fmaf(p, r2, r);
  y = __fadd_rn(y, 1.0f);
  int ni = (int)n;
  float scale = __uint_as_float((uint32_t)(ni + 127) << 23);
  return __fmul_rn(y, scale);
}

// log(x), x positive and normal
BK_DEVINL float bk_logf(float x) {
  uint32_t u = __float_as_uint(x);
  int e = (int)((u >> 23) & 0xffu) - 126;
  float m = __uint_as_float((u & 0x007fffffu) | 0x3f000000u);
  if (m < 0.707106781186547524f) {
    e -= 1;
    m = __fadd_rn(m, m);
  }
  m = __fadd_rn(m, -1.0f);
  float z = __fmul_rn(m, m);
  float p = 7.0376836292e-2f;
  p = fmaf(p, m, -1.1514610310e-1f);
  p = fmaf(p, m, 1.1676998740e-1f);
  p = fmaf(p, m, -1.2420140846e-1f);
  p = fmaf(p, m, 1.4249322787e-1f);
  p = fmaf(p, m, -1.6668057665e-1f);
  p = fmaf(p, m, 2.0000714765e-1f);
  p = fmaf(p, m, -2.4999993993e-1f);
  p = fmaf(p, m, 3.3333331174e-1f);
  float y = __fmul_rn(__fmul_rn(m, z), p);
  float fe = (float)e;
  y = fmaf(fe, -2.12194440e-4f, y);
  y = fmaf(-0.5f, z, y);
  float r = __fadd_rn(m, y);
  r = fmaf(fe, 0.693359375f, r);
  return r;
}

BK_DEVINL float bk_rcp_sqrt(float x) { return __fdiv_rn(1.0f, __fsqrt_rn(x)); }
BK_DEVINL float bk_sigmoidf(float x) { return __fdiv_rn(1.0f, __fadd_rn(1.0f, bk_expf(-x))); }
BK_DEVINL float bk_softplusf(float x) { return bk_logf(__fadd_rn(1.0f, bk_expf(x))); }

// ---- warp reductions --------------------------------------------------------

// xor butterfly 16,8,4,2,1: every lane ends with the same bits
BK_DEVINL float bk_warp_sum(float v) {
#pragma unroll
  for (int off = 16; off >= 1; off >>= 1) v = __fadd_rn(v, __shfl_xor_sync(0xffffffffu, v, off));
  return v;
}
BK_DEVINL float bk_warp_max(float v) {
#pragma unroll
  for (int off = 16; off >= 1; off >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, off));
  return v;
}

// ---- Q8_1 block stores from registers (packQ8_1, bench/bench.ts:53-72, in f32) ----
// `group` consecutive lanes hold one 32-value block, 32/group consecutive values each (group = 32 or 4).
// All lanes of the warp must call.  blk points at the 36-byte block of the calling lane.
template <int PER>
BK_DEVINL void bk_q8_1_store(uint8_t* blk, const float (&y)[PER], int idx_in_block) {
  constexpr int GROUP = 32 / PER;
  float amax = 0.0f;
#pragma unroll
  for (int e = 0; e < PER; e++) amax = fmaxf(amax, fabsf(y[e]));
#pragma unroll
  for (int off = GROUP / 2; off >= 1; off >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, off));
  const float d = __fdiv_rn(amax, 127.0f);
  const float id = (d == 0.0f) ? 1.0f : __fdiv_rn(1.0f, d);
  int sum = 0;
  int qs[PER];
#pragma unroll
  for (int e = 0; e < PER; e++) {
    int v = __float2int_rd(fmaf(y[e], id, 0.5f));
    sum += v;  // the reference sums before clamping
    qs[e] = max(-128, min(127, v));
  }
#pragma unroll
  for (int off = GROUP / 2; off >= 1; off >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, off);
  if (PER == 1) {
    blk[idx_in_block] = (uint8_t)(int8_t)qs[0];
  } else {
    static_assert(PER == 1 || PER % 4 == 0, "values per lane");
    uint32_t* w = reinterpret_cast<uint32_t*>(blk + idx_in_block);
#pragma unroll
    for (int e = 0; e < PER / 4 * 4; e += 4)
      w[e >> 2] = (uint32_t)(qs[e] & 0xff) | ((uint32_t)(qs[e + 1] & 0xff) << 8) | ((uint32_t)(qs[e + 2] & 0xff) << 16) |
                  ((uint32_t)(qs[e + 3] & 0xff) << 24);
  }
  if (idx_in_block == 0) {
    const uint32_t hd = bk_f32_to_f16_trunc(d), hs = bk_f32_to_f16_trunc(__fmul_rn((float)sum, d));
    *reinterpret_cast<uint32_t*>(blk + 32) = hd | (hs << 16);
  }
}

// ---- fused tensor-parallel exchange (descriptors: BkPush / BkReduce in bk_internal.h) ------------------
BK_DEVINL unsigned int bk_exchange_tag(const unsigned int* epoch, unsigned int tag_add) {
  return *reinterpret_cast<const volatile unsigned int*>(epoch) * 256u + tag_add;
}
BK_DEVINL void bk_push_store(uint2* dst, float y, unsigned int tag) {
  asm volatile("st.volatile.global.v2.u32 [%0], {%1, %2};" ::"l"(dst), "r"(__float_as_uint(y)), "r"(tag) : "memory");
}
BK_DEVINL uint4 bk_ld_volatile_v4(const uint2* p) {
  uint4 v;
  asm volatile("ld.volatile.global.v4.u32 {%0, %1, %2, %3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p) : "memory");
  return v;
}
// 8 consecutive values at element offset o (a multiple of 8): ((p0 + p1) + ...) + residual, rounded to bf16 (returned
// as f32).  Two ranks are polled per pass so that their loads are in flight together; sums stay in rank order.
// limit: polls before the wait gives up (0 = the default of 2^20).
BK_DEVINL void bk_reduce_load8(const uint2* src, unsigned long long stride, int n, unsigned int tag, const uint16_t* res,
                               uint16_t* out, size_t o, bool write_out, int* status, float (&y)[8], int limit = 0) {
  const int max_it = limit > 0 ? limit : (1 << 20);
  float a[8];
  for (int r = 0; r < n; r += 2) {
    const bool two = r + 1 < n;
    const uint2* s0 = src + r * stride + o;
    const uint2* s1 = s0 + (two ? stride : 0);
    uint4 w0[4], w1[4];
    for (int it = 0;; it++) {
#pragma unroll
      for (int k = 0; k < 4; k++) w0[k] = bk_ld_volatile_v4(s0 + 2 * k);
#pragma unroll
      for (int k = 0; k < 4; k++) w1[k] = bk_ld_volatile_v4(s1 + 2 * k);
      bool ok = true;
#pragma unroll
      for (int k = 0; k < 4; k++) ok = ok && w0[k].y == tag && w0[k].w == tag && w1[k].y == tag && w1[k].w == tag;
      if (ok) break;
      if (it > max_it || (status && (it & 255) == 255 && *reinterpret_cast<volatile int*>(status) != 0)) {
        if (status) atomicExch(status, 10003 /* BK_ERR_TIMEOUT */);
        break;
      }
    }
#pragma unroll
    for (int k = 0; k < 4; k++) {
      if (r == 0) {
        a[2 * k] = __uint_as_float(w0[k].x);
        a[2 * k + 1] = __uint_as_float(w0[k].z);
      } else {
        a[2 * k] = __fadd_rn(a[2 * k], __uint_as_float(w0[k].x));
        a[2 * k + 1] = __fadd_rn(a[2 * k + 1], __uint_as_float(w0[k].z));
      }
      if (two) {
        a[2 * k] = __fadd_rn(a[2 * k], __uint_as_float(w1[k].x));
        a[2 * k + 1] = __fadd_rn(a[2 * k + 1], __uint_as_float(w1[k].z));
      }
    }
  }
  const uint4 rv = *reinterpret_cast<const uint4*>(res + o);
  uint4 ov;
  ov.x = bk_f32x2_to_bf16x2(__fadd_rn(a[0], __uint_as_float(rv.x << 16)), __fadd_rn(a[1], __uint_as_float(rv.x & 0xffff0000u)));
  ov.y = bk_f32x2_to_bf16x2(__fadd_rn(a[2], __uint_as_float(rv.y << 16)), __fadd_rn(a[3], __uint_as_float(rv.y & 0xffff0000u)));
  ov.z = bk_f32x2_to_bf16x2(__fadd_rn(a[4], __uint_as_float(rv.z << 16)), __fadd_rn(a[5], __uint_as_float(rv.z & 0xffff0000u)));
  ov.w = bk_f32x2_to_bf16x2(__fadd_rn(a[6], __uint_as_float(rv.w << 16)), __fadd_rn(a[7], __uint_as_float(rv.w & 0xffff0000u)));
  if (write_out) *reinterpret_cast<uint4*>(out + o) = ov;
  y[0] = __uint_as_float(ov.x << 16); y[1] = __uint_as_float(ov.x & 0xffff0000u);
  y[2] = __uint_as_float(ov.y << 16); y[3] = __uint_as_float(ov.y & 0xffff0000u);
  y[4] = __uint_as_float(ov.z << 16); y[5] = __uint_as_float(ov.z & 0xffff0000u);
  y[6] = __uint_as_float(ov.w << 16); y[7] = __uint_as_float(ov.w & 0xffff0000u);
}

// ---- staged activation image of the tensor-core GEMV (batch 2..8) ---------------------
// The exact bytes that kernel keeps in shared memory, so that its prologue is one bulk copy:
//   words  [B][K/4 + 8]   Q8_1 quants, the eight words of a block in the order 0,4,1,5,2,6,3,7
//   float4 [K/64][8]      per 64-value unit u and column b: {d8 of block 2u, d8 of block 2u+1 / 16,
//                          s8 of 2u, s8 of 2u+1}, d8 = the block scale after its f16 round trip, s8 = d8 * sum(q)
__host__ __device__ __forceinline__ size_t bk_staged_row_words(int K) { return (size_t)K / 4 + 8; }
// More than 8 batch rows: one image per group of 8 rows (the last group may be smaller), each at a stride of the
// 8-row image size; the GEMV then runs once per group.
__host__ __device__ __forceinline__ size_t bk_staged_group_stride(int K) { return (size_t)8 * bk_staged_row_words(K) * 4 + (size_t)(K / 64) * 8 * 16; }
__host__ __device__ __forceinline__ size_t bk_staged_total_bytes(int K, int B);
__host__ __device__ __forceinline__ size_t bk_staged_bytes(int K, int B) { return (size_t)B * bk_staged_row_words(K) * 4 + (size_t)(K / 64) * 8 * 16; }

__host__ __device__ __forceinline__ size_t bk_staged_total_bytes(int K, int B) {
  return B <= 8 ? bk_staged_bytes(K, B) : (size_t)((B + 7) / 8) * bk_staged_group_stride(K);
}

// Same contract as bk_q8_1_store, writing block blk of column b into a staged image (grouped when B > 8).
template <int PER>
BK_DEVINL void bk_staged_store(uint8_t* img, int K, int B, int b, int blk, const float (&y)[PER], int idx_in_block) {
  if (B > 8) {
    img += (size_t)(b >> 3) * bk_staged_group_stride(K);
    B = min(8, B - (b & ~7));
    b &= 7;
  }
  constexpr int GROUP = 32 / PER;
  float amax = 0.0f;
#pragma unroll
  for (int e = 0; e < PER; e++) amax = fmaxf(amax, fabsf(y[e]));
#pragma unroll
  for (int off = GROUP / 2; off >= 1; off >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, off));
  const float d = __fdiv_rn(amax, 127.0f);
  const float id = (d == 0.0f) ? 1.0f : __fdiv_rn(1.0f, d);
  int sum = 0;
  int qs[PER];
#pragma unroll
  for (int e = 0; e < PER; e++) {
    int v = __float2int_rd(fmaf(y[e], id, 0.5f));
    qs[e] = max(-128, min(127, v));
    sum += qs[e];  // of the stored quants, as a reader of the blocks would recompute it
  }
#pragma unroll
  for (int off = GROUP / 2; off >= 1; off >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, off);
  uint32_t* xw = reinterpret_cast<uint32_t*>(img) + (size_t)b * bk_staged_row_words(K) + (blk >> 1) * 16 + (blk & 1) * 8;
  if (PER == 1) {
    // byte idx of the block lives in word idx/4, stored at position (w&3)*2 + (w>>2)
    const int w = idx_in_block >> 2;
    reinterpret_cast<uint8_t*>(xw + ((w & 3) * 2 + (w >> 2)))[idx_in_block & 3] = (uint8_t)(int8_t)qs[0];
  } else {
    static_assert(PER == 1 || PER % 4 == 0, "values per lane");
#pragma unroll
    for (int e = 0; e < PER / 4 * 4; e += 4) {
      const int w = (idx_in_block + e) >> 2;
      xw[(w & 3) * 2 + (w >> 2)] = (uint32_t)(qs[e] & 0xff) | ((uint32_t)(qs[e + 1] & 0xff) << 8) |
                                   ((uint32_t)(qs[e + 2] & 0xff) << 16) | ((uint32_t)(qs[e + 3] & 0xff) << 24);
    }
  }
  if (idx_in_block == 0) {
    const float d8 = bk_q8half_to_f32(bk_f32_to_f16_trunc(d));
    float* e4 = reinterpret_cast<float*>(img + (size_t)B * bk_staged_row_words(K) * 4) + ((size_t)((blk >> 1) * 8 + b) * 4 + (blk & 1));
    e4[0] = (blk & 1) ? __fmul_rn(d8, 0.0625f) : d8;
    e4[2] = __fmul_rn(d8, (float)sum);
  }
}

// ---- Q4_K superblock header -------------------------------------------------
// bytes [4,16) of a superblock as three words w0,w1,w2; sub-block j in 0..7
BK_DEVINL void bk_q4k_scale_min(uint32_t w0, uint32_t w1, uint32_t w2, int j, int& sc, int& mn) {
  // b[i] = byte i of the 12
  uint32_t lo = (j & 1) * 8 + ((j & 2) ? 16 : 0);  // shift of byte (j&3) in a word
  if (j < 4) {
    sc = (w0 >> lo) & 63;
    mn = (w1 >> lo) & 63;
  } else {
    uint32_t b8 = (w2 >> lo) & 0xffu;   // b[j+4]
    uint32_t b0 = (w0 >> lo) & 0xffu;   // b[j-4]
    uint32_t b4 = (w1 >> lo) & 0xffu;   // b[j]
    sc = (int)((b8 & 0x0fu) | ((b0 >> 6) << 4));
    mn = (int)((b8 >> 4) | ((b4 >> 6) << 4));
  }
}

// scales and mins of the two sub-blocks 2p, 2p+1 (p = 0..3) in one go, branch-free:
// byte 0 of the results belongs to sub-block 2p, byte 1 to 2p+1
BK_DEVINL void bk_q4k_scale_min_pair(uint32_t w0, uint32_t w1, uint32_t w2, int p, uint32_t& sc2, uint32_t& mn2) {
  // the 16-bit half (p & 1) of each word, by one byte permute (selector bytes 0,1 or 2,3; upper half zero)
  const uint32_t sel = (p & 1) ? 0x4432u : 0x4410u;
  const uint32_t h0 = __byte_perm(w0, 0u, sel), h1 = __byte_perm(w1, 0u, sel), h2 = __byte_perm(w2, 0u, sel);
  const uint32_t sc_lo = h0 & 0x3f3fu, mn_lo = h1 & 0x3f3fu;
  const uint32_t sc_hi = (h2 & 0x0f0fu) | ((h0 >> 2) & 0x3030u);
  const uint32_t mn_hi = ((h2 >> 4) & 0x0f0fu) | ((h1 >> 2) & 0x3030u);
  sc2 = p >= 2 ? sc_hi : sc_lo;
  mn2 = p >= 2 ? mn_hi : mn_lo;
}

// One 64-weight unit u (sub-blocks 2p, 2p+1 of superblock u>>2, p = u&3) of a Q4_K row dequantised to bf16:
// dl = d*sc, ml = dmin*m, w = dl*q - ml, each product and the difference rounded once (emitEmbed, src/emitters.ts:31-45,
// on the tied Q4_K table).
BK_DEVINL void bk_q4k_unit_to_bf16(const uint8_t* row, int u, uint16_t* o) {
  const uint8_t* sb = row + (size_t)(u >> 2) * 144;
  const uint4 hdr = __ldg(reinterpret_cast<const uint4*>(sb));
  const uint4* q = reinterpret_cast<const uint4*>(sb + 16 + (u & 3) * 32);
  const uint4 qa = __ldg(q), qb = __ldg(q + 1);
  const int p = u & 3;
  const float d = bk_f16_to_f32((uint16_t)(hdr.x & 0xffffu)), dmin = bk_f16_to_f32((uint16_t)(hdr.x >> 16));
  int sc0, mn0, sc1, mn1;
  bk_q4k_scale_min(hdr.y, hdr.z, hdr.w, 2 * p, sc0, mn0);
  bk_q4k_scale_min(hdr.y, hdr.z, hdr.w, 2 * p + 1, sc1, mn1);
  const float dl0 = __fmul_rn(d, (float)sc0), ml0 = __fmul_rn(dmin, (float)mn0);
  const float dl1 = __fmul_rn(d, (float)sc1), ml1 = __fmul_rn(dmin, (float)mn1);
  const uint32_t qw[8] = {qa.x, qa.y, qa.z, qa.w, qb.x, qb.y, qb.z, qb.w};
#pragma unroll
  for (int k = 0; k < 8; k++)
#pragma unroll
    for (int e = 0; e < 4; e++) {
      const uint32_t byte = (qw[k] >> (8 * e)) & 0xffu;
      o[k * 4 + e] = bk_f32_to_bf16(__fsub_rn(__fmul_rn(dl0, (float)(byte & 15u)), ml0));
      o[32 + k * 4 + e] = bk_f32_to_bf16(__fsub_rn(__fmul_rn(dl1, (float)(byte >> 4)), ml1));
    }
}

BK_DEVINL int bk_dp4a(uint32_t a, uint32_t b, int c) {
  // a: four unsigned bytes (nibble values), b: four signed bytes
  int d;
  asm("dp4a.u32.s32 %0, %1, %2, %3;" : "=r"(d) : "r"(a), "r"(b), "r"(c));
  return d;
}
BK_DEVINL int bk_dp4a_ss(uint32_t a, uint32_t b, int c) {
  int d;
  asm("dp4a.s32.s32 %0, %1, %2, %3;" : "=r"(d) : "r"(a), "r"(b), "r"(c));
  return d;
}
