// bk_gemv_shared.cuh -- pieces common to the two Q4_K x Q8_1 GEMV kernels (dp4a for batch <= 2, int8 MMA above):
// launch parameters, the activation prologues (Q8_1 staging, bf16 -> Q8_1, RMSNorm -> Q8_1), virtual-row decoding,
// mbarrier / bulk-copy helpers and the fused epilogues.
#pragma once
#include "bk_common.cuh"
#include "bk_internal.h"

namespace {


constexpr int kThreads = 256;   // threads of the canonical sum-of-squares order (and of the small kernels below)
constexpr int kWarps = kThreads / 32;
constexpr int kUnitWords = 20;  // 16 data words + 4 pad

struct SegDev {
  const uint8_t* W;
  const uint8_t* W2;
  void* out;
  const uint16_t* res;
  int n_rows;
  int epi;
  int ld_out;
  int col_off;
  int vrow_begin;  // first virtual row of this segment
};

struct GemvParams {
  int K;
  int n_segs;
  int prologue;
  int total_vrows;
  int rows_per_cta;
  int n_slots;       // weight slots (and mbarriers) per CTA
  int depth;         // 0: one slot per group, all requested up front; >0: per-warp ring of this depth
  int group_rows;    // rows one warp processes together (even when a SwiGLU segment is present)
  int x_unit_words;  // words one 64-value unit of the staged activation occupies (16 data + padding)
  int x_row_words;   // words between batch rows of the staged activation
  int x_scale_ld;    // floats between batch rows of the staged block scales d8 / s8
  int tiles_base;    // tensor-core path: every CTA owns tiles_base 16-row tiles, the first tiles_extra CTAs one more
  int tiles_extra;
  const void* x;
  const uint16_t* norm_w;
  float eps;
  int* status;       // device status word: set when a bounded wait gives up
  unsigned long long* trace;  // timeline record of this launch, or null
  unsigned long long* cta_trace;  // per-CTA timeline of this launch, or null
  SegDev segs[4];
  // K view of a split launch (batch >= 2, rows too wide for shared memory): K above is the part's width
  unsigned int row_stride;   // bytes between weight rows in memory; 0 = the part is the whole row
  unsigned int row_off;      // byte offset of the part inside each row
  int xq_ld, xq_off;         // BK_PRO_Q8 input: blocks between batch rows (0 = K/32) and first block of the part
  const float* carry_in;     // class accumulators of the parts before this one, or null
  float* carry_out;          // where to leave them for the next part (then no epilogue runs), or null
  BkPush push;     // n = 0 unless a segment has the BK_EPI_PUSH_F32 epilogue
  BkReduce red;    // n = 0 unless the prologue is BK_PRO_REDUCE_RMSNORM
};

// ---- staged activation layouts ---------------------------------------------------
// Plain (dp4a kernel): quants of block blk at xs[b*x_row_words + (blk>>1)*x_unit_words + (blk&1)*8 + w], w = 0..7;
// scales d8s[b*x_scale_ld + blk] (odd blocks divided by 16, like the MMA layout), s8s likewise (undivided).
// MMA (TC = true): the eight words of a block are stored in the order 0,4,1,5,2,6,3,7 so that the two words a lane
// feeds to one mma (w = j and j+4) are one 64-bit load; the scales of unit u = blk>>1 and column b form one float4
// {d8 of block 2u, d8 of block 2u+1 divided by 16, s8 of 2u, s8 of 2u+1} at sc4[u*8 + b] (s8s is unused).
// The division by 16 pairs with high nibbles left in place (16*q) in the integer dot: the product is unchanged.
template <bool TC>
__device__ __forceinline__ uint32_t* x_block_ptr(const GemvParams& p, uint32_t* xs, int b, int blk) {
  return xs + (size_t)b * p.x_row_words + (blk >> 1) * p.x_unit_words + (blk & 1) * 8;
}
template <bool TC>
__device__ __forceinline__ int x_word_pos(int w) { return TC ? ((w & 3) * 2 + (w >> 2)) : w; }
template <bool TC>
__device__ __forceinline__ void store_block_scales(const GemvParams& p, float* d8s, float* s8s, int b, int blk, float d8,
                                                   float s8) {
  if (TC) {
    float* e = d8s + ((size_t)((blk >> 1) * 8 + b) * 4 + (blk & 1));
    e[0] = (blk & 1) ? __fmul_rn(d8, 0.0625f) : d8;
    e[2] = s8;
  } else {
    d8s[b * p.x_scale_ld + blk] = (blk & 1) ? __fmul_rn(d8, 0.0625f) : d8;   // see unit_val() of the dp4a kernel
    s8s[b * p.x_scale_ld + blk] = s8;
  }
}

// ---- prologues ---------------------------------------------------------------

// Q8_1 blocks [B][nblk][36] -> shared layout
template <bool TC>
__device__ void prologue_q8(const GemvParams& p, const int B, uint32_t* xs, float* d8s, float* s8s) {
  const int nblk = p.K / 32;
  const uint32_t* src = reinterpret_cast<const uint32_t*>(p.x);
  for (int i = threadIdx.x; i < B * nblk; i += blockDim.x) {
    int b = i / nblk, blk = i - b * nblk;
    const uint32_t* s = src + ((size_t)b * (p.xq_ld ? p.xq_ld : nblk) + p.xq_off + blk) * 9;
    uint32_t* dst = x_block_ptr<TC>(p, xs, b, blk);
    int qsum = 0;
#pragma unroll
    for (int k = 0; k < 8; k++) {
      uint32_t w = s[k];
      dst[x_word_pos<TC>(k)] = w;
      qsum = bk_dp4a_ss(w, 0x01010101u, qsum);
    }
    float d8 = bk_q8half_to_f32((uint16_t)(s[8] & 0xffffu));
    store_block_scales<TC>(p, d8s, s8s, b, blk, d8, __fmul_rn(d8, (float)qsum));
  }
}

// quantise 8 consecutive values held by this thread; the 4 threads of an aligned
// lane group hold one 32-element block (packQ8_1, bench/bench.ts:53-72, in f32)
template <bool TC>
__device__ __forceinline__ void quant_chunk(const GemvParams& p, const float (&y)[8], int q, int b, int nblk, uint32_t* xs,
                                            float* d8s, float* s8s) {
  float amax = 0.0f;
#pragma unroll
  for (int e = 0; e < 8; e++) amax = fmaxf(amax, fabsf(y[e]));
  amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 1));
  amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 2));
  float d = __fdiv_rn(amax, 127.0f);
  float id = (d == 0.0f) ? 1.0f : __fdiv_rn(1.0f, d);
  int qs[8];
  int qsum = 0;
#pragma unroll
  for (int e = 0; e < 8; e++) {
    int v = __float2int_rd(fmaf(y[e], id, 0.5f));
    v = max(-128, min(127, v));
    qs[e] = v;
    qsum += v;
  }
  qsum += __shfl_xor_sync(0xffffffffu, qsum, 1);
  qsum += __shfl_xor_sync(0xffffffffu, qsum, 2);
  uint32_t w0 = (uint32_t)(qs[0] & 0xff) | ((uint32_t)(qs[1] & 0xff) << 8) | ((uint32_t)(qs[2] & 0xff) << 16) |
                ((uint32_t)(qs[3] & 0xff) << 24);
  uint32_t w1 = (uint32_t)(qs[4] & 0xff) | ((uint32_t)(qs[5] & 0xff) << 8) | ((uint32_t)(qs[6] & 0xff) << 16) |
                ((uint32_t)(qs[7] & 0xff) << 24);
  int blk = q >> 2;
  uint32_t* dst = x_block_ptr<TC>(p, xs, b, blk);
  dst[x_word_pos<TC>((q & 3) * 2)] = w0;
  dst[x_word_pos<TC>((q & 3) * 2 + 1)] = w1;
  if ((q & 3) == 0) {
    float d8 = bk_q8half_to_f32(bk_f32_to_f16_trunc(d));
    store_block_scales<TC>(p, d8s, s8s, b, blk, d8, __fmul_rn(d8, (float)qsum));
  }
}

__device__ __forceinline__ void load_chunk_bf16(const uint16_t* row, int q, float (&y)[8]) {
  uint4 v = *reinterpret_cast<const uint4*>(row + (size_t)q * 8);
  y[0] = __uint_as_float(v.x << 16);
  y[1] = __uint_as_float(v.x & 0xffff0000u);
  y[2] = __uint_as_float(v.y << 16);
  y[3] = __uint_as_float(v.y & 0xffff0000u);
  y[4] = __uint_as_float(v.z << 16);
  y[5] = __uint_as_float(v.z & 0xffff0000u);
  y[6] = __uint_as_float(v.w << 16);
  y[7] = __uint_as_float(v.w & 0xffff0000u);
}

// chunk q (8 values) of batch row b.  SRC 0: from the bf16 row.  SRC 1: from the ranks' partial sums + residual
// (tensor-parallel reduce; also writes the bf16 result to p.red.out).  SRC 2: from p.red.out as written by CTA 0 of
// this same launch (L2 loads: the L1 of this SM knows nothing of another CTA's stores).  SRC 3: from the bf16 row as
// written by other CTAs earlier in this same launch (persistent step kernel), again past L1.
template <int SRC>
__device__ __forceinline__ void load_chunk_in(const GemvParams& p, const uint16_t* row, int b, int q, float (&y)[8]) {
  if (SRC == 2) {
    const uint4 v = __ldcg(reinterpret_cast<const uint4*>(p.red.out + (size_t)b * p.K) + q);
    y[0] = __uint_as_float(v.x << 16); y[1] = __uint_as_float(v.x & 0xffff0000u);
    y[2] = __uint_as_float(v.y << 16); y[3] = __uint_as_float(v.y & 0xffff0000u);
    y[4] = __uint_as_float(v.z << 16); y[5] = __uint_as_float(v.z & 0xffff0000u);
    y[6] = __uint_as_float(v.w << 16); y[7] = __uint_as_float(v.w & 0xffff0000u);
  } else if (SRC == 3) {
    const uint4 v = __ldcg(reinterpret_cast<const uint4*>(row) + q);
    y[0] = __uint_as_float(v.x << 16); y[1] = __uint_as_float(v.x & 0xffff0000u);
    y[2] = __uint_as_float(v.y << 16); y[3] = __uint_as_float(v.y & 0xffff0000u);
    y[4] = __uint_as_float(v.z << 16); y[5] = __uint_as_float(v.z & 0xffff0000u);
    y[6] = __uint_as_float(v.w << 16); y[7] = __uint_as_float(v.w & 0xffff0000u);
  } else if (SRC == 1) bk_reduce_load8(p.red.src, p.red.stride, p.red.n, bk_exchange_tag(p.red.epoch, p.red.tag_add), p.red.res, p.red.out,
                              (size_t)b * p.K + (size_t)q * 8, true, p.status, y, p.red.spin_limit);
  else load_chunk_bf16(row, q, y);
}

// bf16 rows -> (optional RMSNorm -> bf16) -> Q8_1 in shared memory.
// SRC: where the row comes from (see load_chunk_in).
// Sum of squares in the 256-thread block order: chunk q (8 elements) belongs to
// thread q mod 256, fmaf chain inside; warp butterflies; the 8 warp sums in order.
// wpre: the norm weights of chunk threadIdx.x, loaded by the caller before the dependency wait.
template <bool NORM, int SRC = 0>
__device__ void prologue_bf16(const GemvParams& p, const int B, uint32_t* xs, float* d8s, float* s8s, float* red, const uint4 wpre) {
  const int K = p.K, nblk = K / 32, nchunk = K / 8;
  const uint16_t* x = reinterpret_cast<const uint16_t*>(p.x);
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  for (int b = 0; b < B; b++) {
    const uint16_t* row = x + (size_t)b * K;
    float rstd = 1.0f;
    float y0[8];
    const bool have0 = (int)threadIdx.x < nchunk;
    if (have0) load_chunk_in<SRC>(p, row, b, threadIdx.x, y0);
    if (NORM) {
      float acc = 0.0f;
      if (threadIdx.x < kThreads) {  // the fixed 256-thread order, whatever the CTA size
        if (have0) {
#pragma unroll
          for (int e = 0; e < 8; e++) acc = fmaf(y0[e], y0[e], acc);
        }
        for (int q = threadIdx.x + kThreads; q < nchunk; q += kThreads) {
          float y[8];
          load_chunk_in<SRC>(p, row, b, q, y);
#pragma unroll
          for (int e = 0; e < 8; e++) acc = fmaf(y[e], y[e], acc);
        }
        acc = bk_warp_sum(acc);
      }
      __syncthreads();  // red[] reuse across batch rows
      if (lane == 0 && warp < kWarps) red[warp] = acc;
      __syncthreads();
      float total = red[0];
#pragma unroll
      for (int w = 1; w < kWarps; w++) total = __fadd_rn(total, red[w]);
      float ms = __fdiv_rn(total, (float)K);
      rstd = bk_rcp_sqrt(__fadd_rn(ms, p.eps));
    }
    for (int q = threadIdx.x; q < nchunk; q += blockDim.x) {
      float y[8];
      if (q == (int)threadIdx.x) {
#pragma unroll
        for (int e = 0; e < 8; e++) y[e] = y0[e];
      } else {
        load_chunk_in<SRC>(p, row, b, q, y);
      }
      if (NORM) {
        float wv[8];
        if (q == (int)threadIdx.x) {
          wv[0] = __uint_as_float(wpre.x << 16); wv[1] = __uint_as_float(wpre.x & 0xffff0000u);
          wv[2] = __uint_as_float(wpre.y << 16); wv[3] = __uint_as_float(wpre.y & 0xffff0000u);
          wv[4] = __uint_as_float(wpre.z << 16); wv[5] = __uint_as_float(wpre.z & 0xffff0000u);
          wv[6] = __uint_as_float(wpre.w << 16); wv[7] = __uint_as_float(wpre.w & 0xffff0000u);
        } else {
          load_chunk_bf16(p.norm_w, q, wv);
        }
#pragma unroll
        for (int e = 0; e < 8; e += 2) {
          float v0 = __fmul_rn(__fmul_rn(y[e], rstd), __fadd_rn(1.0f, wv[e]));
          float v1 = __fmul_rn(__fmul_rn(y[e + 1], rstd), __fadd_rn(1.0f, wv[e + 1]));
          uint32_t pk = bk_f32x2_to_bf16x2(v0, v1);
          y[e] = __uint_as_float(pk << 16);
          y[e + 1] = __uint_as_float(pk & 0xffff0000u);
        }
      }
      quant_chunk<false>(p, y, q, b, nblk, xs, d8s, s8s);
    }
  }
}

// The same prologue for several batch rows at once (batch 2..8 path).  Row b's sum of squares still uses the
// canonical 256-thread order, but each aligned block of 256 threads takes a different row, the per-row warp sums
// land in red[b*8 + w], and one barrier serves all rows; the quantisation then runs over the flattened
// (row, chunk) items so that every thread has several independent items in flight.
// red: 8*B + B floats.
template <bool NORM>
__device__ void prologue_bf16_batched(const GemvParams& p, const int B, uint32_t* xs, float* d8s, float* s8s, float* red) {
  const int K = p.K, nblk = K / 32, nchunk = K / 8;
  const uint16_t* x = reinterpret_cast<const uint16_t*>(p.x);
  const int lane = threadIdx.x & 31;
  float* rstd_s = red + 8 * B;
  if (NORM) {
    const int nsl = blockDim.x / kThreads;          // row slots of 256 threads
    const int r = threadIdx.x / kThreads, t256 = threadIdx.x % kThreads;
    if (r < nsl) {
      for (int b = r; b < B; b += nsl) {
        const uint16_t* row = x + (size_t)b * K;
        float acc = 0.0f;
        for (int q = t256; q < nchunk; q += kThreads) {
          float y[8];
          load_chunk_bf16(row, q, y);
#pragma unroll
          for (int e = 0; e < 8; e++) acc = fmaf(y[e], y[e], acc);
        }
        acc = bk_warp_sum(acc);
        if (lane == 0) red[b * 8 + (t256 >> 5)] = acc;
      }
    }
    __syncthreads();
    if ((int)threadIdx.x < B) {
      const float* rb = red + threadIdx.x * 8;
      float total = rb[0];
#pragma unroll
      for (int w = 1; w < kWarps; w++) total = __fadd_rn(total, rb[w]);
      rstd_s[threadIdx.x] = bk_rcp_sqrt(__fadd_rn(__fdiv_rn(total, (float)K), p.eps));
    }
    __syncthreads();
  }
  const int items = B * nchunk;
  for (int i = threadIdx.x; i < items; i += blockDim.x) {
    const int b = i / nchunk, q = i - b * nchunk;
    float y[8];
    load_chunk_bf16(x + (size_t)b * K, q, y);
    if (NORM) {
      float wv[8];
      load_chunk_bf16(p.norm_w, q, wv);
      const float rstd = rstd_s[b];
#pragma unroll
      for (int e = 0; e < 8; e += 2) {
        float v0 = __fmul_rn(__fmul_rn(y[e], rstd), __fadd_rn(1.0f, wv[e]));
        float v1 = __fmul_rn(__fmul_rn(y[e + 1], rstd), __fadd_rn(1.0f, wv[e + 1]));
        uint32_t pk = bk_f32x2_to_bf16x2(v0, v1);
        y[e] = __uint_as_float(pk << 16);
        y[e + 1] = __uint_as_float(pk & 0xffff0000u);
      }
    }
    quant_chunk<true>(p, y, q, b, nblk, xs, d8s, s8s);
  }
}

// ---- virtual rows --------------------------------------------------------------
// The rows of all segments of a launch are numbered consecutively.  A SwiGLU segment contributes
// 2*n_rows virtual rows: even = gate row, odd = the up row of the same output column.
struct VRow {
  const uint8_t* row;
  int si;  // segment
  int n;   // output column within the segment
};

__device__ __forceinline__ VRow decode_vrow(const GemvParams& p, int v) {
  int si = 0;
#pragma unroll
  for (int s = 1; s < 4; s++)
    if (s < p.n_segs && v >= p.segs[s].vrow_begin) si = s;
  const SegDev& sg = p.segs[si];
  const int t = v - sg.vrow_begin;
  const size_t rowb = p.row_stride ? (size_t)p.row_stride : (size_t)(p.K / 256) * 144;
  VRow r;
  r.si = si;
  if (sg.epi == BK_EPI_SWIGLU) {
    r.n = t >> 1;
    r.row = ((t & 1) ? sg.W2 : sg.W) + rowb * (size_t)r.n + p.row_off;
  } else {
    r.n = t;
    r.row = sg.W + rowb * (size_t)t + p.row_off;
  }
  return r;
}

// CG: the residual was written by another CTA earlier in the same launch (persistent step kernel): read it past L1.
template <bool TP = true, bool CG = false>
__device__ __forceinline__ void store_epilogue(const GemvParams& p, const SegDev& sg, size_t o, float y, float yup) {
  if (TP && sg.epi == BK_EPI_PUSH_F32) {
    const unsigned int tag = bk_exchange_tag(p.push.epoch, p.push.tag_add);
    for (int r = 0; r < p.push.n; r++) bk_push_store(p.push.dst[r] + o, y, tag);   // remote stores over NVLink, fire and forget
  } else if (sg.epi == BK_EPI_SWIGLU) {
    float sig = bk_sigmoidf(y);
    reinterpret_cast<uint16_t*>(sg.out)[o] = bk_f32_to_bf16(__fmul_rn(__fmul_rn(y, sig), yup));
  } else if (sg.epi == BK_EPI_F32) {
    reinterpret_cast<float*>(sg.out)[o] = y;
  } else if (sg.epi == BK_EPI_BF16) {
    reinterpret_cast<uint16_t*>(sg.out)[o] = bk_f32_to_bf16(y);
  } else {  // BK_EPI_ADD_BF16
    reinterpret_cast<uint16_t*>(sg.out)[o] = bk_f32_to_bf16(__fadd_rn(y, bk_bf16_to_f32(CG ? __ldcg(sg.res + o) : sg.res[o])));
  }
}

}  // namespace
