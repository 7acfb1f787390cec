// bk_gdn.cuh -- the fused conv1d + gated-DeltaNet step body (emitConv1d + emitGDN, src/emitters.ts:48-120;
// buildGDNDecode, prototypes/decode.ts:314-388), shared by the per-op kernels (bk_ops.cu) and the persistent
// decode-step kernel (bk_persist.cu).
#pragma once
#include "bk_common.cuh"
#include "bk_internal.h"

namespace {

// ---- fused conv1d + gated DeltaNet step ------------------------------------------
// One CTA of 512 threads per (batch, value head).  Thread (r = t>>7, j = t&127)
// keeps rows 32r..32r+31 of column j of the 128x128 state in registers: one read
// and one write of the state per step.  Column sums over the 128 rows use the four
// row groups in order ((g0+g1)+g2)+g3.
struct GdnParams {
  const uint16_t* qkv;
  const uint16_t* z;
  const float* a;
  const float* b;
  const uint16_t* conv_w;
  const uint16_t* cs_in;
  uint16_t* cs_new;
  const float* A_log;
  const uint16_t* dt_bias;
  const float* norm_w;
  const float* S_in;
  float* S_new;
  uint16_t* out;
  float* o_raw;
  uint16_t* conv_out;
  uint8_t* out_q8;
  int out_q8_staged;
  int B, Hk, Hv, apply_conv;
  int T;      // tokens per sequence handled by this launch, in order (1 in the decode step)
  int early;  // state / conv state / weights are not outputs of the immediately preceding launch
  unsigned long long* trace;
};

// Two builds of this body.  gdn_step_kernel: launched with 576 threads when the grid has at most one CTA per SM; the
// two extra warps only keep a second CTA of this grid off the SM (register file), so no SM finishes last with two.
// gdn_step_kernel_x2: 64 registers, two CTAs per SM, for grids larger than the SM count (batch 8: 256 CTAs, one wave).
// MULTI = false compiles the single-token body of the decode step (no loop, no carried taps).
// PERSIST: the body runs as one phase of the persistent decode-step kernel (bk_persist.cu): head and sequence come
// from the caller, no programmatic-launch calls, and the activations another CTA of the same launch produced
// (qkv, z, a, b) are read past this SM's L1.
struct GdnSmem {
  float s_q[128], s_k[128], s_v[128], s_o[128];
  float s_part[4][128];
  float s_scal[4];  // q scale, k rstd, decay, beta
};

template <bool PERSIST, typename T>
__device__ __forceinline__ T gdn_ld_act(const T* p) { return PERSIST ? __ldcg(p) : *p; }

template <bool MULTI, bool PERSIST = false>
__device__ __forceinline__ void gdn_step_body(const GdnParams& p, GdnSmem& sm, const int hv, const int b) {
  constexpr int D = 128;
  float (&s_q)[D] = sm.s_q;
  float (&s_k)[D] = sm.s_k;
  float (&s_v)[D] = sm.s_v;
  float (&s_o)[D] = sm.s_o;
  float (&s_part)[4][D] = sm.s_part;
  float (&s_scal)[4] = sm.s_scal;
  if (!PERSIST) {
    bk_pdl_trigger();
    bk_stamp(p.trace, 0);
  }
  const int t = threadIdx.x;
  const int ratio = p.Hv / p.Hk, hk = hv / ratio;
  const int keydim = p.Hk * D, C = 2 * keydim + p.Hv * D;
  const int warp = t >> 5, lane = t & 31;
  const bool active = t < 4 * D;            // threads beyond 512 only occupy registers (see the launch)
  const int r = active ? t >> 7 : 0, j = t & 127;
  const int which = t >> 7, ci = t & 127;
  int ch = 0;
  if (which == 0) ch = hk * D + ci;
  else if (which == 1) ch = keydim + hk * D + ci;
  else ch = 2 * keydim + hv * D + ci;
  const float* S = p.S_in + (((size_t)b * p.Hv + hv) * D + 32 * r) * D + j;
  float* Sn = p.S_new + (((size_t)b * p.Hv + hv) * D + 32 * r) * D + j;

  // State, conv taps and per-head constants do not come from the kernel that runs just before this one
  // (p.early != 0 asserts that), so they are requested before the dependency wait and arrive while the
  // projection GEMV is still finishing.
  float sd[32];
  uint16_t h0 = 0, h1 = 0, h2 = 0;
  uint2 cw = make_uint2(0, 0);
  float alog = 0.0f, dtb = 0.0f, nw = 0.0f;
  auto load_static = [&]() {
    if (active) {
#pragma unroll
      for (int i = 0; i < 32; i++) sd[i] = S[(size_t)i * D];
    }
    if (t < 3 * D && p.apply_conv) {
      const uint16_t* st = p.cs_in + (size_t)b * 3 * C;
      h0 = st[ch];
      h1 = st[C + ch];
      h2 = st[2 * C + ch];
      cw = *reinterpret_cast<const uint2*>(p.conv_w + 4 * (size_t)ch);
    }
    if (t == 3 * D) {
      alog = p.A_log[hv];
      dtb = bk_bf16_to_f32(p.dt_bias[hv]);
    }
    if (t < D) nw = p.norm_w[t];
  };
  if (PERSIST) {
    load_static();
  } else {
    if (p.early) load_static();
    bk_pdl_wait();
    bk_stamp(p.trace, 2);
    if (!p.early) load_static();
  }

  // Tokens tk = 0..T-1 of this sequence in order (T = 1 in the decode step): rows tk*B + b of the per-token inputs and
  // outputs.  The state and the three conv taps stay in registers between tokens; both are written back after the last.
  const int T = MULTI ? p.T : 1;
  for (int tk = 0; tk < T; tk++) {
    const size_t row = (size_t)tk * p.B + b;
    const bool last = !MULTI || tk == T - 1;
    float zv = 0.0f;
    if (t < D) zv = bk_bf16_to_f32(gdn_ld_act<PERSIST>(p.z + (row * p.Hv + hv) * D + t));
    if (t < 3 * D) {
      uint16_t hx = gdn_ld_act<PERSIST>(p.qkv + row * C + ch);
      float val;
      if (p.apply_conv) {
        float w0 = __uint_as_float(cw.x << 16), w1 = __uint_as_float(cw.x & 0xffff0000u);
        float w2 = __uint_as_float(cw.y << 16), w3 = __uint_as_float(cw.y & 0xffff0000u);
        float raw = __fadd_rn(__fadd_rn(__fmul_rn(w0, bk_bf16_to_f32(h0)), __fmul_rn(w1, bk_bf16_to_f32(h1))),
                              __fadd_rn(__fmul_rn(w2, bk_bf16_to_f32(h2)), __fmul_rn(w3, bk_bf16_to_f32(hx))));
        uint16_t ob = bk_f32_to_bf16(__fmul_rn(raw, bk_sigmoidf(raw)));
        val = bk_bf16_to_f32(ob);
        // q/k channels are shared by `ratio` value heads: the first of them writes
        if (which == 2 || hv % ratio == 0) {
          if (last) {
            uint16_t* d = p.cs_new + (size_t)b * 3 * C;
            d[ch] = h1;
            d[C + ch] = h2;
            d[2 * C + ch] = hx;
          }
          if (p.conv_out) p.conv_out[row * C + ch] = ob;
        }
        if (MULTI) {
          h0 = h1;
          h1 = h2;
          h2 = hx;
        }
      } else {
        val = bk_bf16_to_f32(hx);
      }
      if (which == 0) s_q[ci] = val;
      else if (which == 1) s_k[ci] = val;
      else s_v[ci] = val;
    } else if (t == 3 * D) {
      // gates on an otherwise idle warp, overlapping the conv above
      float sp = bk_softplusf(__fadd_rn(gdn_ld_act<PERSIST>(p.a + row * p.Hv + hv), dtb));
      s_scal[2] = bk_expf(-__fmul_rn(bk_expf(alog), sp));
      s_scal[3] = bk_sigmoidf(gdn_ld_act<PERSIST>(p.b + row * p.Hv + hv));
    }
    __syncthreads();
    if (warp < 2) {
      const float* src = warp == 0 ? s_q : s_k;
      float acc = 0.0f;
#pragma unroll
      for (int e = 0; e < 4; e++) acc = fmaf(src[lane * 4 + e], src[lane * 4 + e], acc);
      acc = bk_warp_sum(acc);
      float rr = bk_rcp_sqrt(__fadd_rn(acc, 1e-6f));
      if (lane == 0) s_scal[warp] = (warp == 0) ? __fmul_rn(rr, 0.088388347648318441f) : rr;
    }
    __syncthreads();
    if (t < D) s_q[t] = __fmul_rn(s_q[t], s_scal[0]);
    else if (t < 2 * D) s_k[t - D] = __fmul_rn(s_k[t - D], s_scal[1]);
    __syncthreads();

    const float decay = s_scal[2], beta = s_scal[3];
    float acc = 0.0f;
    if (active) {
#pragma unroll
      for (int i = 0; i < 32; i++) {
        sd[i] = __fmul_rn(sd[i], decay);
        acc = fmaf(s_k[32 * r + i], sd[i], acc);
      }
      s_part[r][j] = acc;
    }
    __syncthreads();
    float kS = __fadd_rn(__fadd_rn(__fadd_rn(s_part[0][j], s_part[1][j]), s_part[2][j]), s_part[3][j]);
    float delta = __fmul_rn(__fsub_rn(s_v[j], kS), beta);
    __syncthreads();
    acc = 0.0f;
    if (active) {
#pragma unroll
      for (int i = 0; i < 32; i++) {
        sd[i] = fmaf(s_k[32 * r + i], delta, sd[i]);
        if (last) Sn[(size_t)i * D] = sd[i];
        acc = fmaf(s_q[32 * r + i], sd[i], acc);
      }
      s_part[r][j] = acc;
    }
    __syncthreads();
    if (t < D) {
      float o = __fadd_rn(__fadd_rn(__fadd_rn(s_part[0][t], s_part[1][t]), s_part[2][t]), s_part[3][t]);
      s_o[t] = o;
      if (p.o_raw) p.o_raw[(row * p.Hv + hv) * D + t] = o;
    }
    __syncthreads();
    if (warp == 0) {
      float a2 = 0.0f;
#pragma unroll
      for (int e = 0; e < 4; e++) a2 = fmaf(s_o[lane * 4 + e], s_o[lane * 4 + e], a2);
      a2 = bk_warp_sum(a2);
      if (lane == 0) s_scal[0] = bk_rcp_sqrt(__fadd_rn(__fdiv_rn(a2, (float)D), 1e-6f));
    }
    __syncthreads();
    if (t < D) {
      float zs = __fmul_rn(zv, bk_sigmoidf(zv));
      float ow = __fmul_rn(__fmul_rn(s_o[t], s_scal[0]), nw);
      const uint16_t ob = bk_f32_to_bf16(__fmul_rn(ow, zs));
      p.out[(row * p.Hv + hv) * D + t] = ob;
      if (p.out_q8) {  // warp w of the first four holds block w of this head
        const float y[1] = {bk_bf16_to_f32(ob)};
        if (p.out_q8_staged) bk_staged_store<1>(p.out_q8, p.Hv * D, p.B * T, (int)row, hv * 4 + warp, y, lane);
        else bk_q8_1_store<1>(p.out_q8 + ((row * p.Hv + hv) * 4 + warp) * 36, y, lane);
      }
    }
    if (!last) __syncthreads();   // s_scal[0] and s_o are rewritten by the next token
  }
  if (!PERSIST) bk_stamp(p.trace, 5);
}

}  // namespace
