// bk_ops.cu -- the non-GEMV decode ops: embed, RMSNorm, SwiGLU, conv1d, the fused
// conv1d + gated-DeltaNet step, q/k head norm + partial rotary, argmax.
// Math follows bunker's emitters (src/emitters.ts) and tuned decode kernels
// (prototypes/decode.ts); reduction orders are fixed so a host can reproduce the bits.
#include <math.h>

#include "bk_common.cuh"
#include "bk_internal.h"
#include "bk_gdn.cuh"

namespace {

// ---- embed: x[b] = bf16(dequant(E[ids[b]])) (src/emitters.ts:31-45) ------------
__global__ void embed_q4k_kernel(const uint8_t* table, int H, const int32_t* ids, uint16_t* x) {
  bk_pdl_trigger();
  bk_pdl_wait();
  const int b = blockIdx.x;
  const int nunits = H / 64;
  const uint8_t* row = table + (size_t)ids[b] * (H / 256) * 144;
  for (int u = threadIdx.x; u < nunits; u += blockDim.x) bk_q4k_unit_to_bf16(row, u, x + (size_t)b * H + (size_t)u * 64);
}

__device__ __forceinline__ void load8_bf16(const uint16_t* p, float (&y)[8]) {
  uint4 v = *reinterpret_cast<const uint4*>(p);
  y[0] = __uint_as_float(v.x << 16);
  y[1] = __uint_as_float(v.x & 0xffff0000u);
  y[2] = __uint_as_float(v.y << 16);
  y[3] = __uint_as_float(v.y & 0xffff0000u);
  y[4] = __uint_as_float(v.z << 16);
  y[5] = __uint_as_float(v.z & 0xffff0000u);
  y[6] = __uint_as_float(v.w << 16);
  y[7] = __uint_as_float(v.w & 0xffff0000u);
}

// ---- RMSNorm (buildRMS, prototypes/decode.ts:201-216), one CTA of 256 per row ----
__global__ void __launch_bounds__(256) rmsnorm_kernel(const uint16_t* x, const uint16_t* w, int H, float eps,
                                                      uint16_t* y) {
  __shared__ float red[8];
  const uint16_t* row = x + (size_t)blockIdx.x * H;
  uint16_t* out = y + (size_t)blockIdx.x * H;
  const int nchunk = H / 8;
  float acc = 0.0f;
  for (int q = threadIdx.x; q < nchunk; q += 256) {
    float v[8];
    load8_bf16(row + (size_t)q * 8, v);
#pragma unroll
    for (int e = 0; e < 8; e++) acc = fmaf(v[e], v[e], acc);
  }
  acc = bk_warp_sum(acc);
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = acc;
  __syncthreads();
  float total = red[0];
#pragma unroll
  for (int i = 1; i < 8; i++) total = __fadd_rn(total, red[i]);
  float rstd = bk_rcp_sqrt(__fadd_rn(__fdiv_rn(total, (float)H), eps));
  for (int q = threadIdx.x; q < nchunk; q += 256) {
    float v[8], wv[8];
    load8_bf16(row + (size_t)q * 8, v);
    load8_bf16(w + (size_t)q * 8, wv);
    uint32_t o[4];
#pragma unroll
    for (int e = 0; e < 8; e += 2) {
      uint32_t lo = bk_f32_to_bf16(__fmul_rn(__fmul_rn(v[e], rstd), __fadd_rn(1.0f, wv[e])));
      uint32_t hi = bk_f32_to_bf16(__fmul_rn(__fmul_rn(v[e + 1], rstd), __fadd_rn(1.0f, wv[e + 1])));
      o[e >> 1] = lo | (hi << 16);
    }
    *reinterpret_cast<uint4*>(out + (size_t)q * 8) = make_uint4(o[0], o[1], o[2], o[3]);
  }
}

// ---- (RMSNorm ->) Q8_1 rows, computed once for all consumers ------------------------
// At batch >= 2 the projection kernels read their activation as ready Q8_1 blocks instead of each of the
// 148 CTAs normalising and quantising all batch rows again.  NORM: one CTA per batch row (the canonical
// 256-thread sum of squares).  Plain: 256 chunks of 8 values per CTA.  Output blocks [B][K/32][36].
// STAGED: the output is the staged image of the tensor-core GEMV instead of 36-byte blocks.
// rd.n > 0 (NORM only): row b is not read from x but formed from the tensor-parallel partial sums + residual.
template <bool NORM, bool STAGED>
__global__ void __launch_bounds__(256) quant_rows_kernel(const uint16_t* x, const uint16_t* w, int K, float eps,
                                                         uint8_t* out, const BkReduce rd, int* status) {
  bk_pdl_trigger();
  __shared__ float red[8];
  const int b = blockIdx.y, nchunk = K / 8, tid = threadIdx.x;
  const uint16_t* row = x + (size_t)b * K;
  uint8_t* orow = out + (size_t)b * (K / 32) * 36;
  if (NORM) {
    float wv0[8];
    const bool have0 = tid < nchunk;
    if (have0) load8_bf16(w + (size_t)tid * 8, wv0);
    if (!rd.n) bk_pdl_wait();   // a reducing launch synchronises through the tagged words instead (see gemv_q4k_kernel)
    const unsigned int tag = rd.n ? bk_exchange_tag(rd.epoch, rd.tag_add) : 0u;
    auto load_in = [&](int q, float (&y)[8]) {
      if (rd.n) bk_reduce_load8(rd.src, rd.stride, rd.n, tag, rd.res, rd.out, (size_t)b * K + (size_t)q * 8, true, status, y, rd.spin_limit);
      else load8_bf16(row + (size_t)q * 8, y);
    };
    float y0[8];
    float acc = 0.0f;
    if (have0) {
      load_in(tid, y0);
#pragma unroll
      for (int e = 0; e < 8; e++) acc = fmaf(y0[e], y0[e], acc);
    }
    for (int q = tid + 256; q < nchunk; q += 256) {
      float v[8];
      load_in(q, v);
#pragma unroll
      for (int e = 0; e < 8; e++) acc = fmaf(v[e], v[e], acc);
    }
    acc = bk_warp_sum(acc);
    if ((tid & 31) == 0) red[tid >> 5] = acc;
    __syncthreads();
    float total = red[0];
#pragma unroll
    for (int i = 1; i < 8; i++) total = __fadd_rn(total, red[i]);
    const float rstd = bk_rcp_sqrt(__fadd_rn(__fdiv_rn(total, (float)K), eps));
    for (int q = tid; q < nchunk; q += 256) {  // nchunk is a multiple of 32: whole warps enter together
      float v[8], wv[8];
      if (q == tid) {
#pragma unroll
        for (int e = 0; e < 8; e++) { v[e] = y0[e]; wv[e] = wv0[e]; }
      } else {
        load_in(q, v);
        load8_bf16(w + (size_t)q * 8, wv);
      }
      float y[8];
#pragma unroll
      for (int e = 0; e < 8; e++)
        y[e] = bk_bf16_to_f32(bk_f32_to_bf16(__fmul_rn(__fmul_rn(v[e], rstd), __fadd_rn(1.0f, wv[e]))));
      if (STAGED) bk_staged_store<8>(out, K, gridDim.y, b, q >> 2, y, (q & 3) * 8);
      else bk_q8_1_store<8>(orow + (size_t)(q >> 2) * 36, y, (q & 3) * 8);
    }
  } else {
    bk_pdl_wait();
    const int q = blockIdx.x * 256 + tid;
    if (q < nchunk) {
      float y[8];
      load8_bf16(row + (size_t)q * 8, y);
      if (STAGED) bk_staged_store<8>(out, K, gridDim.y, b, q >> 2, y, (q & 3) * 8);
      else bk_q8_1_store<8>(orow + (size_t)(q >> 2) * 36, y, (q & 3) * 8);
    }
  }
}

// ---- SwiGLU (src/fusion.ts:324-330) ---------------------------------------------
__global__ void swiglu_kernel(const float* g, const float* u, int n, uint16_t* out) {
  int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n) return;
  float gv = g[i];
  out[i] = bk_f32_to_bf16(__fmul_rn(__fmul_rn(gv, bk_sigmoidf(gv)), u[i]));
}

// ---- conv1d decode step (src/emitters.ts:48-72) ----------------------------------
__device__ __forceinline__ float conv_tap4(float s0, float s1, float s2, float xv, const uint16_t* w4) {
  uint2 wv = *reinterpret_cast<const uint2*>(w4);
  float w0 = __uint_as_float(wv.x << 16), w1 = __uint_as_float(wv.x & 0xffff0000u);
  float w2 = __uint_as_float(wv.y << 16), w3 = __uint_as_float(wv.y & 0xffff0000u);
  float raw = __fadd_rn(__fadd_rn(__fmul_rn(w0, s0), __fmul_rn(w1, s1)), __fadd_rn(__fmul_rn(w2, s2), __fmul_rn(w3, xv)));
  return __fmul_rn(raw, bk_sigmoidf(raw));
}

__global__ void conv1d_step_kernel(const uint16_t* x, const uint16_t* st, const uint16_t* w, int C, int B,
                                   uint16_t* out, uint16_t* sn) {
  int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= B * C) return;
  int b = i / C, c = i - b * C;
  const uint16_t* s = st + (size_t)b * 3 * C;
  uint16_t h0 = s[c], h1 = s[C + c], h2 = s[2 * C + c], hx = x[i];
  float o = conv_tap4(bk_bf16_to_f32(h0), bk_bf16_to_f32(h1), bk_bf16_to_f32(h2), bk_bf16_to_f32(hx), w + 4 * (size_t)c);
  out[i] = bk_f32_to_bf16(o);
  uint16_t* d = sn + (size_t)b * 3 * C;
  d[c] = h1;
  d[C + c] = h2;
  d[2 * C + c] = hx;
}

__global__ void __launch_bounds__(576) gdn_step_kernel(const GdnParams p) {
  __shared__ GdnSmem sm;
  gdn_step_body<false>(p, sm, blockIdx.x, blockIdx.y);
}
__global__ void __launch_bounds__(512, 2) gdn_step_kernel_x2(const GdnParams p) {
  __shared__ GdnSmem sm;
  gdn_step_body<false>(p, sm, blockIdx.x, blockIdx.y);
}
__global__ void __launch_bounds__(576) gdn_step_kernel_multi(const GdnParams p) {
  __shared__ GdnSmem sm;
  gdn_step_body<true>(p, sm, blockIdx.x, blockIdx.y);
}
// ---- q/k head RMSNorm + partial rotary, one warp per (batch, head) ----------------
// (src/emitters.ts:123-183).  Lane l owns the HD/32 contiguous dims of the head.
template <int C>
__device__ __forceinline__ void headnorm_rope_warp(const uint16_t* src, const uint16_t* w, const float* cos_row,
                                                   const float* sin_row, int rot_half, uint16_t* stage,
                                                   uint16_t* dst) {
  const int lane = threadIdx.x & 31;
  float x[C];
#pragma unroll
  for (int e = 0; e < C; e++) x[e] = bk_bf16_to_f32(src[lane * C + e]);
  float acc = 0.0f;
#pragma unroll
  for (int e = 0; e < C; e++) acc = fmaf(x[e], x[e], acc);
  acc = bk_warp_sum(acc);
  float rstd = bk_rcp_sqrt(__fadd_rn(__fdiv_rn(acc, (float)(32 * C)), 1e-6f));
#pragma unroll
  for (int e = 0; e < C; e++) {
    float wv = bk_bf16_to_f32(w[lane * C + e]);
    stage[lane * C + e] = bk_f32_to_bf16(__fmul_rn(__fmul_rn(x[e], rstd), __fadd_rn(1.0f, wv)));
  }
  __syncwarp();
  for (int i = lane; i < rot_half; i += 32) {
    float x1 = bk_bf16_to_f32(stage[i]), x2 = bk_bf16_to_f32(stage[i + rot_half]);
    float c = cos_row[i], s = sin_row[i];
    uint16_t r1 = bk_f32_to_bf16(__fsub_rn(__fmul_rn(x1, c), __fmul_rn(x2, s)));
    uint16_t r2 = bk_f32_to_bf16(__fadd_rn(__fmul_rn(x2, c), __fmul_rn(x1, s)));
    stage[i] = r1;  // each pair (i, i+rot_half) is read and written by this lane only
    stage[i + rot_half] = r2;
  }
  __syncwarp();
  if (dst != stage) {
#pragma unroll
    for (int e = 0; e < C; e++) dst[lane * C + e] = stage[lane * C + e];
  }
}

__global__ void __launch_bounds__(128) headnorm_rope_kernel(const uint16_t* in, int in_stride, const uint16_t* w,
                                                            const float* cos_t, const float* sin_t, int rot_half,
                                                            const int32_t* pos, int B, int nheads, int HD,
                                                            uint16_t* out) {
  __shared__ uint16_t stage[4][512];
  const int warp = threadIdx.x >> 5;
  const int idx = blockIdx.x * 4 + warp;
  if (idx >= B * nheads) return;
  const int b = idx / nheads;
  const uint16_t* src = in + (size_t)idx * in_stride;
  uint16_t* dst = out + (size_t)idx * HD;
  const float* c = cos_t + (size_t)pos[b] * rot_half;
  const float* s = sin_t + (size_t)pos[b] * rot_half;
  if (HD == 256) headnorm_rope_warp<8>(src, w, c, s, rot_half, stage[warp], dst);
  else headnorm_rope_warp<4>(src, w, c, s, rot_half, stage[warp], dst);
}

// ---- argmax: exact max, lowest index on ties (prototypes/decode.ts:776-784) -------
__device__ __forceinline__ void argmax_merge(float& v, int& i, float ov, int oi) {
  if (ov > v || (ov == v && oi < i)) {
    v = ov;
    i = oi;
  }
}

constexpr int kArgmaxBlocks = 64;

// pos/hist (optional): the finishing block also records the token at hist[pos[b]*hist_ld + b] and advances
// pos[b], which is how the model-level decode step feeds the next token without a host round trip.
__global__ void __launch_bounds__(256) argmax_kernel(const float* logits, int V, int32_t* idx, float* val,
                                                     float* part_v, int32_t* part_i, unsigned int* counter,
                                                     int32_t* pos, int32_t* hist, int hist_ld, int hist_rows,
                                                     int32_t* host_out) {
  __shared__ float sv[8];
  __shared__ int si[8];
  __shared__ bool last;
  bk_pdl_trigger();
  bk_pdl_wait();
  const int b = blockIdx.y;
  const float* l = logits + (size_t)b * V;
  const int per = (V + gridDim.x - 1) / gridDim.x;
  const int lo = blockIdx.x * per, hi = min(V, lo + per);
  float bv = -INFINITY;
  int bi = 0x7fffffff;
  for (int i = lo + threadIdx.x; i < hi; i += 256) {
    float v = l[i];
    if (v > bv) {
      bv = v;
      bi = i;
    }
  }
  for (int off = 16; off >= 1; off >>= 1) {
    float ov = __shfl_xor_sync(0xffffffffu, bv, off);
    int oi = __shfl_xor_sync(0xffffffffu, bi, off);
    argmax_merge(bv, bi, ov, oi);
  }
  if ((threadIdx.x & 31) == 0) {
    sv[threadIdx.x >> 5] = bv;
    si[threadIdx.x >> 5] = bi;
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    for (int w = 1; w < 8; w++) argmax_merge(bv, bi, sv[w], si[w]);
    part_v[b * kArgmaxBlocks + blockIdx.x] = bv;
    part_i[b * kArgmaxBlocks + blockIdx.x] = bi;
    __threadfence();
    unsigned int done = atomicAdd(&counter[b], 1u);
    last = (done == gridDim.x - 1);
  }
  __syncthreads();
  if (last && threadIdx.x == 0) {
    __threadfence();
    volatile float* pv = part_v;
    volatile int32_t* pi = part_i;
    float v = -INFINITY;
    int i = 0x7fffffff;
    for (unsigned k = 0; k < gridDim.x; k++) argmax_merge(v, i, pv[b * kArgmaxBlocks + k], pi[b * kArgmaxBlocks + k]);
    if (i == 0x7fffffff) i = 0;
    idx[b] = i;
    val[b] = v;
    if (host_out) {   // pinned host memory mapped into the device: the result reaches the host without a copy engine
      host_out[b] = i;
      host_out[gridDim.y + b] = __float_as_int(v);
    }
    counter[b] = 0;
    if (pos) {
      int pcur = pos[b];
      if (hist && pcur < hist_rows) hist[(size_t)pcur * hist_ld + b] = i;
      pos[b] = pcur + 1;
    }
  }
}

}  // namespace

extern "C" {

int32_t bkEmbedQ4K(uint64_t table, int32_t H, uint64_t ids, int32_t B, uint64_t x_out) {
  BK_REQUIRE_INIT();
  BK_ARG(H > 0 && H % 256 == 0 && B > 0, "bkEmbedQ4K: bad shape H=%d B=%d", H, B);
  BK_ARG(table && ids && x_out && (table & 15) == 0, "bkEmbedQ4K: null or misaligned pointer");
  BK_CUDA(bk_launch_pdl(embed_q4k_kernel, dim3(B), dim3(64), 0, bk_ptr<uint8_t>(table), H, bk_ptr<int32_t>(ids),
                        bk_ptr<uint16_t>(x_out)));
  BK_CHECK_LAUNCH();
  return BK_OK;
}

int32_t bkRmsNorm(uint64_t x, uint64_t w, int32_t H, int32_t B, float eps, uint64_t y) {
  BK_REQUIRE_INIT();
  BK_ARG(H > 0 && H % 8 == 0 && B > 0, "bkRmsNorm: bad shape H=%d B=%d", H, B);
  BK_ARG(x && w && y && ((x | w | y) & 15) == 0, "bkRmsNorm: null or misaligned pointer");
  rmsnorm_kernel<<<B, 256, 0, bk_ctx().stream>>>(bk_ptr<uint16_t>(x), bk_ptr<uint16_t>(w), H, eps,
                                                bk_ptr<uint16_t>(y));
  BK_CHECK_LAUNCH();
  return BK_OK;
}

}  // extern "C"

int32_t bk_quant_rows_launch(uint64_t x, uint64_t w, int32_t K, int32_t B, float eps, uint64_t out, int32_t layout,
                             const BkReduce* reduce) {
  BK_ARG(K > 0 && K % 256 == 0 && B > 0, "bkRmsNormQuantQ8_1: bad shape K=%d B=%d (K a multiple of 256)", K, B);
  BK_ARG((x || reduce) && out && ((x | w) & 15) == 0 && (out & 3) == 0, "bkRmsNormQuantQ8_1: null or misaligned pointer");
  BK_ARG(layout == BK_Q8_BLOCKS || layout == BK_Q8_STAGED, "bkRmsNormQuantQ8_1: unknown layout %d", layout);
  BK_ARG(!reduce || w, "bkRmsNormQuantQ8_1: the reduce input exists with the norm only");
  if (layout == BK_Q8_STAGED) BK_ARG((out & 15) == 0, "bkRmsNormQuantQ8_1: a staged image is 16-byte aligned");
  const dim3 grid = w ? dim3(1, B) : dim3((K / 8 + 255) / 256, B);
  auto* px = bk_ptr<uint16_t>(x);
  auto* pw = bk_ptr<uint16_t>(w);
  auto* po = bk_ptr<uint8_t>(out);
  BkReduce red;
  memset(&red, 0, sizeof(red));
  if (reduce) red = *reduce;
  red.spin_limit = bk_ctx().spin_limit;
  int* st = bk_ctx().d_status;
  if (w) {
    if (layout == BK_Q8_STAGED) BK_CUDA(bk_launch_pdl(quant_rows_kernel<true, true>, grid, dim3(256), 0, px, pw, K, eps, po, red, st));
    else BK_CUDA(bk_launch_pdl(quant_rows_kernel<true, false>, grid, dim3(256), 0, px, pw, K, eps, po, red, st));
  } else {
    if (layout == BK_Q8_STAGED) BK_CUDA(bk_launch_pdl(quant_rows_kernel<false, true>, grid, dim3(256), 0, px, pw, K, eps, po, red, st));
    else BK_CUDA(bk_launch_pdl(quant_rows_kernel<false, false>, grid, dim3(256), 0, px, pw, K, eps, po, red, st));
  }
  BK_CHECK_LAUNCH();
  return BK_OK;
}

extern "C" {
int32_t bkRmsNormQuantQ8_1(uint64_t x, uint64_t w, int32_t K, int32_t B, float eps, uint64_t out, int32_t layout) {
  BK_REQUIRE_INIT();
  BK_ARG(x != 0, "bkRmsNormQuantQ8_1: x is null");
  return bk_quant_rows_launch(x, w, K, B, eps, out, layout, nullptr);
}

int32_t bkReduceRmsNormQuantQ8_1(uint64_t words, int32_t n_ranks, uint64_t stride_words, uint64_t epoch, uint32_t tag_add,
                                 uint64_t residual, uint64_t sum_out, uint64_t w, int32_t K, int32_t B, float eps, uint64_t out,
                                 int32_t layout) {
  BK_REQUIRE_INIT();
  BK_ARG(words && epoch && residual && sum_out && w && n_ranks >= 1 && n_ranks <= 8 && (words & 15) == 0 && stride_words % 2 == 0,
         "bkReduceRmsNormQuantQ8_1: bad arguments");
  BkReduce rd;
  memset(&rd, 0, sizeof(rd));
  rd.src = bk_ptr<uint2>(words);
  rd.epoch = bk_ptr<unsigned int>(epoch);
  rd.res = bk_ptr<uint16_t>(residual);
  rd.out = bk_ptr<uint16_t>(sum_out);
  rd.stride = stride_words;
  rd.tag_add = tag_add;
  rd.n = n_ranks;
  return bk_quant_rows_launch(sum_out, w, K, B, eps, out, layout, &rd);
}

uint64_t bkStagedBytes(int32_t K, int32_t B) { return (K > 0 && B > 0) ? (uint64_t)bk_staged_total_bytes(K, B) : 0; }

int32_t bkSwiglu(uint64_t g_f32, uint64_t u_f32, int32_t n, uint64_t out_bf16) {
  BK_REQUIRE_INIT();
  BK_ARG(n > 0 && g_f32 && u_f32 && out_bf16, "bkSwiglu: bad arguments");
  swiglu_kernel<<<(n + 255) / 256, 256, 0, bk_ctx().stream>>>(bk_ptr<float>(g_f32), bk_ptr<float>(u_f32), n,
                                                             bk_ptr<uint16_t>(out_bf16));
  BK_CHECK_LAUNCH();
  return BK_OK;
}

int32_t bkConv1dStep(uint64_t x, uint64_t state_in, uint64_t w, int32_t C, int32_t B, uint64_t out,
                     uint64_t state_new) {
  BK_REQUIRE_INIT();
  BK_ARG(C > 0 && B > 0, "bkConv1dStep: bad shape C=%d B=%d", C, B);
  BK_ARG(x && state_in && w && out && state_new && (w & 7) == 0, "bkConv1dStep: null or misaligned pointer");
  BK_ARG(state_in != state_new, "bkConv1dStep: state_in and state_new must be distinct buffers");
  int n = B * C;
  conv1d_step_kernel<<<(n + 255) / 256, 256, 0, bk_ctx().stream>>>(bk_ptr<uint16_t>(x), bk_ptr<uint16_t>(state_in),
                                                                  bk_ptr<uint16_t>(w), C, B, bk_ptr<uint16_t>(out),
                                                                  bk_ptr<uint16_t>(state_new));
  BK_CHECK_LAUNCH();
  return BK_OK;
}

int32_t bkGdnStep(const bkGdnArgs* args) {
  BK_REQUIRE_INIT();
  BK_ARG(args != nullptr, "bkGdnStep: args is null");
  bkGdnArgs a = *args;
  BK_ARG(a.B > 0 && a.Hk > 0 && a.Hv > 0 && a.Hv % a.Hk == 0, "bkGdnStep: bad head counts B=%d Hk=%d Hv=%d", a.B, a.Hk,
         a.Hv);
  BK_ARG(a.qkv && a.z && a.a && a.b && a.A_log && a.dt_bias && a.norm_w && a.S_in && a.S_new && a.out,
         "bkGdnStep: null pointer among required arguments");
  if (a.apply_conv) {
    BK_ARG(a.conv_w && a.conv_state_in && a.conv_state_new && (a.conv_w & 7) == 0,
           "bkGdnStep: conv weights/state missing or misaligned");
    BK_ARG(a.conv_state_in != a.conv_state_new, "bkGdnStep: conv state buffers must be distinct");
  }
  GdnParams p;
  p.qkv = bk_ptr<uint16_t>(a.qkv);
  p.z = bk_ptr<uint16_t>(a.z);
  p.a = bk_ptr<float>(a.a);
  p.b = bk_ptr<float>(a.b);
  p.conv_w = bk_ptr<uint16_t>(a.conv_w);
  p.cs_in = bk_ptr<uint16_t>(a.conv_state_in);
  p.cs_new = bk_ptr<uint16_t>(a.conv_state_new);
  p.A_log = bk_ptr<float>(a.A_log);
  p.dt_bias = bk_ptr<uint16_t>(a.dt_bias);
  p.norm_w = bk_ptr<float>(a.norm_w);
  p.S_in = bk_ptr<float>(a.S_in);
  p.S_new = bk_ptr<float>(a.S_new);
  p.out = bk_ptr<uint16_t>(a.out);
  p.o_raw = bk_ptr<float>(a.o_raw);
  p.conv_out = bk_ptr<uint16_t>(a.conv_out);
  p.out_q8 = bk_ptr<uint8_t>(a.out_q8);
  p.out_q8_staged = a.out_q8_layout == BK_Q8_STAGED;
  BK_ARG(a.out_q8_layout == BK_Q8_BLOCKS || (a.out_q8_layout == BK_Q8_STAGED && (a.Hv * 128) % 256 == 0),
         "bkGdnStep: out_q8_layout %d (a staged image needs Hv*128 a multiple of 256)", a.out_q8_layout);
  p.B = a.B;
  p.Hk = a.Hk;
  p.Hv = a.Hv;
  p.apply_conv = a.apply_conv;
  p.early = a.state_is_settled;
  p.T = a.n_tokens > 1 ? a.n_tokens : 1;
  BK_ARG(a.n_tokens >= 0 && (p.out_q8_staged == 0 || (size_t)a.B * p.T <= 64), "bkGdnStep: n_tokens=%d", a.n_tokens);
  p.trace = bk_trace_slot();
  if (p.T > 1) BK_CUDA(bk_launch_pdl(gdn_step_kernel_multi, dim3(a.Hv, a.B), dim3(576), 0, p));
  else if (a.Hv * a.B > bk_ctx().sm_count) BK_CUDA(bk_launch_pdl(gdn_step_kernel_x2, dim3(a.Hv, a.B), dim3(512), 0, p));
  else BK_CUDA(bk_launch_pdl(gdn_step_kernel, dim3(a.Hv, a.B), dim3(576), 0, p));
  BK_CHECK_LAUNCH();
  return BK_OK;
}

int32_t bkRopeTables(int32_t max_len, int32_t rot_dim, double theta, float* cos_out, float* sin_out) {
  if (max_len <= 0 || rot_dim <= 0 || (rot_dim & 1) || !cos_out || !sin_out)
    return bk_fail(BK_ERR_ARG, "bkRopeTables: bad arguments");
  int half = rot_dim / 2;
  for (int p = 0; p < max_len; p++)
    for (int i = 0; i < half; i++) {
      double freq = 1.0 / pow(theta, 2.0 * i / rot_dim);
      cos_out[(size_t)p * half + i] = (float)cos(p * freq);
      sin_out[(size_t)p * half + i] = (float)sin(p * freq);
    }
  return BK_OK;
}

int32_t bkHeadNormRope(uint64_t in, int32_t in_stride, uint64_t w, uint64_t cos_t, uint64_t sin_t, int32_t rot_half,
                       uint64_t pos, int32_t B, int32_t nheads, int32_t HD, uint64_t out) {
  BK_REQUIRE_INIT();
  BK_ARG(HD == 256 || HD == 128, "bkHeadNormRope: HD=%d unsupported (128 or 256)", HD);
  BK_ARG(B > 0 && nheads > 0 && in_stride >= HD && rot_half > 0 && 2 * rot_half <= HD, "bkHeadNormRope: bad shape");
  BK_ARG(rot_half <= 256, "bkHeadNormRope: rot_half=%d too large", rot_half);
  BK_ARG(in && w && cos_t && sin_t && pos && out, "bkHeadNormRope: null pointer");
  int n = B * nheads;
  headnorm_rope_kernel<<<(n + 3) / 4, 128, 0, bk_ctx().stream>>>(
      bk_ptr<uint16_t>(in), in_stride, bk_ptr<uint16_t>(w), bk_ptr<float>(cos_t), bk_ptr<float>(sin_t), rot_half,
      bk_ptr<int32_t>(pos), B, nheads, HD, bk_ptr<uint16_t>(out));
  BK_CHECK_LAUNCH();
  return BK_OK;
}

uint64_t bkArgmaxScratchBytes(int32_t B) { return (uint64_t)(B > 0 ? B : 1) * (kArgmaxBlocks * 8 + 4); }

int32_t bkArgmax(uint64_t logits, int32_t V, int32_t B, uint64_t idx, uint64_t val, uint64_t scratch) {
  return bk_argmax_launch(logits, V, B, idx, val, scratch, 0, 0, 0, 0);
}

}  // extern "C"

int32_t bk_argmax_launch(uint64_t logits, int32_t V, int32_t B, uint64_t idx, uint64_t val, uint64_t scratch,
                         uint64_t pos, uint64_t hist, int32_t hist_ld, int32_t hist_rows, uint64_t host_out) {
  BK_REQUIRE_INIT();
  BK_ARG(V > 0 && B > 0 && logits && idx && val && scratch, "bkArgmax: bad arguments");
  // scratch: [B][64] f32, [B][64] i32, [B] counters (zero before first use; the kernel re-zeroes them)
  float* pv = bk_ptr<float>(scratch);
  int32_t* pi = reinterpret_cast<int32_t*>(pv + (size_t)B * kArgmaxBlocks);
  unsigned int* cnt = reinterpret_cast<unsigned int*>(pi + (size_t)B * kArgmaxBlocks);
  int blocks = (V + 2047) / 2048;
  if (blocks > kArgmaxBlocks) blocks = kArgmaxBlocks;
  BK_CUDA(bk_launch_pdl(argmax_kernel, dim3(blocks, B), dim3(256), 0, bk_ptr<float>(logits), V, bk_ptr<int32_t>(idx),
                        bk_ptr<float>(val), pv, pi, cnt, bk_ptr<int32_t>(pos), bk_ptr<int32_t>(hist), hist_ld,
                        hist_rows, bk_ptr<int32_t>(host_out)));
  BK_CHECK_LAUNCH();
  return BK_OK;
}

// ---- argmax for callers that may not allocate -----------------------------------------------------
// bkArgmax needs a caller-provided scratch buffer (per-block partial results and a completion counter per
// batch row).  Some hosts cannot provide one: a decode loop that was handed a fixed memory budget at
// start-up and has spent it, code that runs where cudaMalloc is off limits (it synchronises the whole
// device and is not permitted while a stream is being captured), or an embedding runtime that owns every
// byte of device memory itself.  For them the scratch lives in the library image: a file-scope array of
// kArgmaxStaticMaxB * 516 = 33,024 bytes that every GPU loading the library carries until the process
// exits.  All calls share it and it keeps whatever the last call left, so the counters are cleared at the
// start of every call, and two calls that overlap on the GPU would corrupt each other.
constexpr int kArgmaxStaticMaxB = 64;
static __device__ __align__(256) unsigned char g_argmax_static_scratch[kArgmaxStaticMaxB * (kArgmaxBlocks * 8 + 4)];

extern "C" int32_t bkArgmaxStatic(uint64_t logits, int32_t V, int32_t B, uint64_t idx, uint64_t val) {
  BK_REQUIRE_INIT();
  BK_ARG(V > 0 && B > 0 && logits && idx && val, "bkArgmaxStatic: bad arguments");
  BK_ARG(B <= kArgmaxStaticMaxB, "bkArgmaxStatic: B=%d exceeds the built-in scratch, which holds at most %d rows; use bkArgmax with your own scratch",
         B, kArgmaxStaticMaxB);
  // The array's name is only a host-side stand-in; the kernel needs its device address.  Looked up once per
  // device, with that device current (the first call on a device does this, so make that call before any
  // stream capture).
  static unsigned char* dev_addr[64] = {nullptr};
  const int dev = bk_ctx().device;
  BK_ARG(dev >= 0 && dev < 64, "bkArgmaxStatic: device index %d out of range", dev);
  if (!dev_addr[dev]) {
    int cur = -1;
    BK_CUDA(cudaGetDevice(&cur));
    if (cur != dev) BK_CUDA(cudaSetDevice(dev));
    void* p = nullptr;
    const cudaError_t e = cudaGetSymbolAddress(&p, g_argmax_static_scratch);
    if (cur != dev && cur >= 0) cudaSetDevice(cur);   // the caller's current device is left as it was
    if (e != cudaSuccess) return bk_fail((int32_t)e, "bkArgmaxStatic: cudaGetSymbolAddress -> %s", cudaGetErrorString(e));
    dev_addr[dev] = static_cast<unsigned char*>(p);
  }
  float* pv = reinterpret_cast<float*>(dev_addr[dev]);
  int32_t* pi = reinterpret_cast<int32_t*>(pv + (size_t)B * kArgmaxBlocks);
  unsigned int* cnt = reinterpret_cast<unsigned int*>(pi + (size_t)B * kArgmaxBlocks);
  BK_CUDA(cudaMemsetAsync(cnt, 0, (size_t)B * sizeof(unsigned int), bk_ctx().stream));  // counters must start at zero
  int blocks = (V + 2047) / 2048;
  if (blocks > kArgmaxBlocks) blocks = kArgmaxBlocks;
  BK_CUDA(bk_launch_pdl(argmax_kernel, dim3(blocks, B), dim3(256), 0, bk_ptr<float>(logits), V, bk_ptr<int32_t>(idx),
                        bk_ptr<float>(val), pv, pi, cnt, (int32_t*)nullptr, (int32_t*)nullptr, 0, 0, (int32_t*)nullptr));
  BK_CHECK_LAUNCH();
  return BK_OK;
}
