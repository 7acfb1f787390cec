// bk_quantize.cu -- f32 / bf16 weight rows -> Q4_K superblocks on the device: the quantiser behind the weight loader.
//
// bunker uploads its safetensors weights as they are, bf16 (loadWeights, prototypes/decode.ts:64-76); the Q4_K model
// served here needs them quantised once at load time.  One warp per 256-weight superblock, lane l holding weights
// [8l, 8l+8) (a quarter of sub-block l/4).  The arithmetic is the CPU checker's, operation for operation:
//   sub-block:  lo = min(min x, 0), scale = (max x - lo) / 15, mn = 0 - lo
//   superblock: d = f16_rn(max scale / 63), dmin = f16_rn(max mn / 63), sc = floor(scale * (1/d) + 0.5) (<= 63),
//               m = floor(mn * (1/dmin) + 0.5) (<= 63)
//   weight:     q = clamp(floor((x + dmin*m) / (d*sc) + 0.5), 0, 15)
// Output layout: bytes [0,2) d, [2,4) dmin, [4,16) the twelve 6-bit scale/min bytes, [16,144) quants, every 32 bytes
// serving sub-blocks 2p (low nibbles) and 2p+1 (high nibbles).
#include "bk_common.cuh"
#include "bk_internal.h"

namespace {

template <bool BF16>
__global__ void __launch_bounds__(256) quantize_q4k_kernel(const void* x, size_t n_superblocks, uint8_t* out) {
  const int lane = threadIdx.x & 31;
  const size_t sb_idx = (size_t)blockIdx.x * 8 + (threadIdx.x >> 5);
  if (sb_idx >= n_superblocks) return;   // whole warps leave together
  float v[8];
  if (BF16) {
    const uint4 r = *reinterpret_cast<const uint4*>(reinterpret_cast<const uint16_t*>(x) + sb_idx * 256 + lane * 8);
    v[0] = __uint_as_float(r.x << 16); v[1] = __uint_as_float(r.x & 0xffff0000u);
    v[2] = __uint_as_float(r.y << 16); v[3] = __uint_as_float(r.y & 0xffff0000u);
    v[4] = __uint_as_float(r.z << 16); v[5] = __uint_as_float(r.z & 0xffff0000u);
    v[6] = __uint_as_float(r.w << 16); v[7] = __uint_as_float(r.w & 0xffff0000u);
  } else {
    const float4* s = reinterpret_cast<const float4*>(reinterpret_cast<const float*>(x) + sb_idx * 256 + lane * 8);
    const float4 a = s[0], c = s[1];
    v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w;
    v[4] = c.x; v[5] = c.y; v[6] = c.z; v[7] = c.w;
  }
  float lo = v[0], hi = v[0];
#pragma unroll
  for (int e = 1; e < 8; e++) {
    lo = fminf(lo, v[e]);
    hi = fmaxf(hi, v[e]);
  }
#pragma unroll
  for (int off = 1; off <= 2; off <<= 1) {   // the four lanes of a sub-block
    lo = fminf(lo, __shfl_xor_sync(0xffffffffu, lo, off));
    hi = fmaxf(hi, __shfl_xor_sync(0xffffffffu, hi, off));
  }
  if (lo > 0.0f) lo = 0.0f;
  float scale = __fdiv_rn(__fsub_rn(hi, lo), 15.0f);
  if (!(scale > 0.0f)) scale = 0.0f;
  const float mn = __fsub_rn(0.0f, lo);   // 0 - lo, not -lo: a zero minimum stays +0 (its sign would reach the f16 dmin)
  float max_scale = scale, max_min = mn;
#pragma unroll
  for (int off = 4; off <= 16; off <<= 1) {
    max_scale = fmaxf(max_scale, __shfl_xor_sync(0xffffffffu, max_scale, off));
    max_min = fmaxf(max_min, __shfl_xor_sync(0xffffffffu, max_min, off));
  }
  uint16_t dh, mh;
  asm("cvt.rn.f16.f32 %0, %1;" : "=h"(dh) : "f"(__fdiv_rn(max_scale, 63.0f)));
  asm("cvt.rn.f16.f32 %0, %1;" : "=h"(mh) : "f"(__fdiv_rn(max_min, 63.0f)));
  const float d = bk_f16_to_f32(dh), dm = bk_f16_to_f32(mh);
  const float inv_d = d > 0.0f ? __fdiv_rn(1.0f, d) : 0.0f, inv_dm = dm > 0.0f ? __fdiv_rn(1.0f, dm) : 0.0f;
  const int sc = min(63, (int)floorf(__fadd_rn(__fmul_rn(scale, inv_d), 0.5f)));
  const int m6 = min(63, (int)floorf(__fadd_rn(__fmul_rn(mn, inv_dm), 0.5f)));
  const float dl = __fmul_rn(d, (float)sc), ml = __fmul_rn(dm, (float)m6);
  uint32_t q[2] = {0u, 0u};   // eight 4-bit quants, one per byte
#pragma unroll
  for (int e = 0; e < 8; e++) {
    int qi = 0;
    if (dl > 0.0f) {
      qi = (int)floorf(__fadd_rn(__fdiv_rn(__fadd_rn(v[e], ml), dl), 0.5f));
      qi = max(0, min(15, qi));
    }
    q[e >> 2] |= (uint32_t)qi << (8 * (e & 3));
  }
  // quant bytes: lanes 8p..8p+3 hold sub-block 2p (low nibbles), lanes 8p+4..8p+7 sub-block 2p+1 (high nibbles) of
  // the same 32 bytes
  const uint32_t h0 = __shfl_down_sync(0xffffffffu, q[0], 4), h1 = __shfl_down_sync(0xffffffffu, q[1], 4);
  uint8_t* sb = out + sb_idx * 144;
  if ((lane & 4) == 0) {
    uint32_t* dst = reinterpret_cast<uint32_t*>(sb + 16 + (lane >> 3) * 32 + (lane & 3) * 8);
    dst[0] = q[0] | (h0 << 4);
    dst[1] = q[1] | (h1 << 4);
  }
  // header: sub-block j's scale and min sit in lane 4j
  const int j = lane & 3;   // lanes 0..3 assemble bytes j, j+4, j+8 of the twelve
  const int sc_lo = __shfl_sync(0xffffffffu, sc, 4 * j), sc_hi = __shfl_sync(0xffffffffu, sc, 4 * (j + 4));
  const int m_lo = __shfl_sync(0xffffffffu, m6, 4 * j), m_hi = __shfl_sync(0xffffffffu, m6, 4 * (j + 4));
  if (lane < 4) {
    sb[4 + j] = (uint8_t)(sc_lo | ((sc_hi >> 4) << 6));
    sb[8 + j] = (uint8_t)(m_lo | ((m_hi >> 4) << 6));
    sb[12 + j] = (uint8_t)((sc_hi & 0x0f) | ((m_hi & 0x0f) << 4));
  }
  if (lane == 0) *reinterpret_cast<uint32_t*>(sb) = (uint32_t)dh | ((uint32_t)mh << 16);
}

}  // namespace

extern "C" int32_t bkQuantizeQ4K(uint64_t x, int32_t dtype, int64_t n_rows, int32_t K, uint64_t out) {
  BK_REQUIRE_INIT();
  BK_ARG(dtype == BK_DTYPE_F32 || dtype == BK_DTYPE_BF16, "bkQuantizeQ4K: dtype %d (BK_DTYPE_F32 or BK_DTYPE_BF16)", dtype);
  BK_ARG(n_rows > 0 && K > 0 && K % 256 == 0, "bkQuantizeQ4K: bad shape rows=%lld K=%d (K a multiple of 256)", (long long)n_rows, K);
  BK_ARG(x && out && (x & 15) == 0 && (out & 15) == 0, "bkQuantizeQ4K: null or misaligned pointer");
  const size_t nsb = (size_t)n_rows * (K / 256);
  const unsigned grid = (unsigned)((nsb + 7) / 8);
  if (dtype == BK_DTYPE_BF16)
    quantize_q4k_kernel<true><<<grid, 256, 0, bk_ctx().stream>>>(bk_ptr<void>(x), nsb, bk_ptr<uint8_t>(out));
  else
    quantize_q4k_kernel<false><<<grid, 256, 0, bk_ctx().stream>>>(bk_ptr<void>(x), nsb, bk_ptr<uint8_t>(out));
  BK_CHECK_LAUNCH();
  return BK_OK;
}
