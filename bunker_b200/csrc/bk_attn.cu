// bk_attn.cu -- split-KV flash-decode GQA attention over a bf16 KV cache.
//
// Replaces bunker's single-tile decode attention (emitFA2Attn, src/emitters.ts:188-226;
// buildFA2Attn, prototypes/decode.ts:427-468), whose cache is capped at 128 rows and
// replicated per query head.  Here the cache is per KV head, [B][Hkv][max_len][256],
// and a (batch, KV head) pair is cut into splits of split_len rows, one CTA each, so
// every SM streams K/V.  The same kernel applies the q/k head RMSNorm and the partial
// rotary (emitQNorm/emitKNorm/emitRoPE/emitRoPEK, src/emitters.ts:123-183) and appends
// the new K/V row, so one launch replaces five of the reference's.
//
// Per split: scores for all rows (each K row is read once for the G query heads of
// the group), exact max, p = exp(s-m), then o = sum p*V with each V row read once.
// The CTA that finishes a (batch, KV head) last merges its splits and applies the sigmoid output gate.
// Orders are fixed (see the CPU checker): lane l owns dims [8l,8l+8); row jj of a
// split belongs to warp jj mod 8; warps and splits are added in ascending order.
#include "bk_common.cuh"
#include "bk_internal.h"

namespace {

constexpr int kW = 8;        // warps per split CTA
constexpr int kHD = 256;     // head dim (8 per lane)
constexpr int kMaxSplits = 1024;
constexpr int kCh = 4;       // rows of one warp per register chunk (two chunks are live: the one in use and the next)

struct AttnParams {
  const uint16_t* qg;
  const uint16_t* k;
  const uint16_t* v;
  const uint16_t* q_norm_w;
  const uint16_t* k_norm_w;
  const float* cos_t;
  const float* sin_t;
  uint16_t* k_cache;
  uint16_t* v_cache;
  const int32_t* pos;
  uint16_t* out;
  uint8_t* out_q8;
  int out_q8_staged;
  float* scratch;
  const uint16_t* gate;
  int B, Hq, Hkv, rot_half, max_len, split_len, max_splits, fused;
  int settled;  // cache rows of earlier steps and pos[] are not outputs of the immediately preceding launch
  int layout_B; // entries the scratch buffer is laid out for (>= B): partials of all entries, then the completion counters,
                // which must stay where they are from launch to launch (they reset themselves)
  int n_seq;    // > 0: prompt columns.  Entry b of the launch is token b / n_seq of sequence b mod n_seq: it reads that
                // sequence's cache, and its own K/V row has already been appended (attn_append_kernel)
  float scale;
  unsigned long long* trace;
};

__device__ __forceinline__ void bf16x8_to_f32(uint4 v, float (&y)[8]) {
  y[0] = __uint_as_float(v.x << 16);
  y[1] = __uint_as_float(v.x & 0xffff0000u);
  y[2] = __uint_as_float(v.y << 16);
  y[3] = __uint_as_float(v.y & 0xffff0000u);
  y[4] = __uint_as_float(v.z << 16);
  y[5] = __uint_as_float(v.z & 0xffff0000u);
  y[6] = __uint_as_float(v.w << 16);
  y[7] = __uint_as_float(v.w & 0xffff0000u);
}

// head RMSNorm*(1+w) -> bf16 -> rotary on the first 2*rot_half dims, result in `stage`
__device__ __forceinline__ void norm_rope_256(const uint16_t* src, const uint16_t* w, const float* cos_row,
                                              const float* sin_row, int rot_half, uint16_t* stage) {
  const int lane = threadIdx.x & 31;
  float x[8], wv[8];
  bf16x8_to_f32(*reinterpret_cast<const uint4*>(src + lane * 8), x);
  bf16x8_to_f32(*reinterpret_cast<const uint4*>(w + lane * 8), wv);
  float acc = 0.0f;
#pragma unroll
  for (int e = 0; e < 8; e++) acc = fmaf(x[e], x[e], acc);
  acc = bk_warp_sum(acc);
  float rstd = bk_rcp_sqrt(__fadd_rn(__fdiv_rn(acc, (float)kHD), 1e-6f));
#pragma unroll
  for (int e = 0; e < 8; e++)
    stage[lane * 8 + e] = bk_f32_to_bf16(__fmul_rn(__fmul_rn(x[e], rstd), __fadd_rn(1.0f, wv[e])));
  __syncwarp();
  for (int i = lane; i < rot_half; i += 32) {
    float x1 = bk_bf16_to_f32(stage[i]), x2 = bk_bf16_to_f32(stage[i + rot_half]);
    float c = cos_row[i], s = sin_row[i];
    uint16_t r1 = bk_f32_to_bf16(__fsub_rn(__fmul_rn(x1, c), __fmul_rn(x2, s)));
    uint16_t r2 = bk_f32_to_bf16(__fadd_rn(__fmul_rn(x2, c), __fmul_rn(x1, s)));
    stage[i] = r1;
    stage[i + rot_half] = r2;
  }
  __syncwarp();
}

// Sum 8 per-lane values over the warp with 9 shuffles instead of 40: at each of the
// first three levels a lane keeps half of its values and trades the other half with
// its xor partner.  The additions are the butterfly's, so the bits are too.
// On return lane l holds the total of value index 4*bit4(l) + 2*bit3(l) + bit2(l).
__device__ __forceinline__ float warp_sum8(const float (&v)[8]) {
  const int lane = threadIdx.x & 31;
  const bool b4 = lane & 16, b3 = lane & 8, b2 = lane & 4;
  float w[4], x[2];
#pragma unroll
  for (int i = 0; i < 4; i++) {
    float send = b4 ? v[i] : v[i + 4];
    float keep = b4 ? v[i + 4] : v[i];
    w[i] = __fadd_rn(keep, __shfl_xor_sync(0xffffffffu, send, 16));
  }
#pragma unroll
  for (int i = 0; i < 2; i++) {
    float send = b3 ? w[i] : w[i + 2];
    float keep = b3 ? w[i + 2] : w[i];
    x[i] = __fadd_rn(keep, __shfl_xor_sync(0xffffffffu, send, 8));
  }
  float send = b2 ? x[0] : x[1];
  float keep = b2 ? x[1] : x[0];
  float y = __fadd_rn(keep, __shfl_xor_sync(0xffffffffu, send, 4));
  y = __fadd_rn(y, __shfl_xor_sync(0xffffffffu, y, 2));
  y = __fadd_rn(y, __shfl_xor_sync(0xffffffffu, y, 1));
  return y;
}

// merge the splits of one (batch, q head) by one warp; lane l owns output dims [8l, 8l+8).
// w_s: ns floats of shared memory private to the warp.  M = max m_s; w_s = exp(m_s - M);
// L = fma(w_s, l_s, L) and O = fma(w_s, o_s, O) in ascending s; out = (O/L) * sigmoid(gate).
__device__ void combine_head_warp(const AttnParams& p, int b, int h, int ns, float* w_s) {
  const int lane = threadIdx.x & 31;
  const float* sc_ml = p.scratch + ((size_t)b * p.Hq + h) * p.max_splits * 2;
  const float* sc_o = p.scratch + (size_t)p.layout_B * p.Hq * p.max_splits * 2 + ((size_t)b * p.Hq + h) * p.max_splits * kHD;
  float m = -INFINITY;
  for (int s = lane; s < ns; s += 32) {
    float ms = __ldcg(sc_ml + 2 * s);
    w_s[s] = ms;
    m = fmaxf(m, ms);
  }
  const float M = bk_warp_max(m);
  for (int s = lane; s < ns; s += 32) w_s[s] = bk_expf(__fsub_rn(w_s[s], M));
  __syncwarp();
  float L = 0.0f, O[8];
#pragma unroll
  for (int e = 0; e < 8; e++) O[e] = 0.0f;
  for (int s = 0; s < ns; s++) {
    const float w = w_s[s];
    L = fmaf(w, __ldcg(sc_ml + 2 * s + 1), L);
    const float4 a = __ldcg(reinterpret_cast<const float4*>(sc_o + (size_t)s * kHD + lane * 8));
    const float4 c = __ldcg(reinterpret_cast<const float4*>(sc_o + (size_t)s * kHD + lane * 8) + 1);
    O[0] = fmaf(w, a.x, O[0]); O[1] = fmaf(w, a.y, O[1]); O[2] = fmaf(w, a.z, O[2]); O[3] = fmaf(w, a.w, O[3]);
    O[4] = fmaf(w, c.x, O[4]); O[5] = fmaf(w, c.y, O[5]); O[6] = fmaf(w, c.z, O[6]); O[7] = fmaf(w, c.w, O[7]);
  }
  const uint16_t* gp = p.fused ? p.qg + ((size_t)b * p.Hq + h) * 2 * kHD + kHD + lane * 8
                               : p.gate + ((size_t)b * p.Hq + h) * kHD + lane * 8;
  float gf[8];
  bf16x8_to_f32(*reinterpret_cast<const uint4*>(gp), gf);
  uint32_t o[4];
#pragma unroll
  for (int e = 0; e < 8; e += 2) {
    float v0 = __fmul_rn(__fdiv_rn(O[e], L), bk_sigmoidf(gf[e]));
    float v1 = __fmul_rn(__fdiv_rn(O[e + 1], L), bk_sigmoidf(gf[e + 1]));
    o[e >> 1] = bk_f32x2_to_bf16x2(v0, v1);
  }
  *reinterpret_cast<uint4*>(p.out + ((size_t)b * p.Hq + h) * kHD + lane * 8) = make_uint4(o[0], o[1], o[2], o[3]);
  if (p.out_q8) {  // four lanes hold one 32-value block
    float y[8];
#pragma unroll
    for (int e = 0; e < 4; e++) {
      y[2 * e] = __uint_as_float(o[e] << 16);
      y[2 * e + 1] = __uint_as_float(o[e] & 0xffff0000u);
    }
    if (p.out_q8_staged) bk_staged_store<8>(p.out_q8, p.Hq * kHD, p.B, b, (h * kHD + lane * 8) >> 5, y, (lane & 3) * 8);
    else bk_q8_1_store<8>(p.out_q8 + ((((size_t)b * p.Hq + h) * kHD + lane * 8) >> 5) * 36, y, (lane & 3) * 8);
  }
}

// dynamic shared memory layout (bytes):
//   q_st  : 8*256 bf16                 4096
//   k_st  : 256 bf16                    512
//   m_s   : 8 f32 (+8 spare)             64
//   l_s   : kW*8 f32                    256
//   s_s   : split_len*8 f32
//   o_s   : kW*8*256 f32              65536   (reused by the split merge)
// One CTA per (split, KV head, batch).  Rows of the cache that were written in earlier steps do not depend on
// the kernel running just before this one, so (p.settled) the first 8 K rows and 8 V rows of every warp are
// requested before the dependency wait; longer splits stream further chunks of 8 rows per warp with the next
// chunk in flight while the current one is reduced.  The CTA that finishes a (batch, KV head) last merges the splits.
// Two CTAs per SM (at most 128 registers): with one CTA of 8 warps an SM cannot hide the latency of the per-row
// shuffle reductions and the stream stalls.
// Prompt columns: every column's K row (head norm + RoPE at its own position, the arithmetic of the decode step) and V
// row go into its sequence's cache before the attention launch, since a later token of the same pass attends to them.
// One warp per (KV head, column).
__global__ void __launch_bounds__(32) attn_append_kernel(const AttnParams p) {
  bk_pdl_trigger();
  __shared__ __align__(16) uint16_t k_st[kHD];
  const int kvh = blockIdx.x, b = blockIdx.y, lane = threadIdx.x;
  bk_pdl_wait();
  const int pos = __ldcg(p.pos + b);
  const int cb = b % p.n_seq;
  uint16_t* Kb = p.k_cache + ((size_t)cb * p.Hkv + kvh) * (size_t)p.max_len * kHD;
  uint16_t* Vb = p.v_cache + ((size_t)cb * p.Hkv + kvh) * (size_t)p.max_len * kHD;
  norm_rope_256(p.k + ((size_t)b * p.Hkv + kvh) * kHD, p.k_norm_w, p.cos_t + (size_t)pos * p.rot_half,
                p.sin_t + (size_t)pos * p.rot_half, p.rot_half, k_st);
  __syncwarp();
  *reinterpret_cast<uint4*>(Kb + (size_t)pos * kHD + lane * 8) = *reinterpret_cast<const uint4*>(k_st + lane * 8);
  *reinterpret_cast<uint4*>(Vb + (size_t)pos * kHD + lane * 8) =
      *reinterpret_cast<const uint4*>(p.v + ((size_t)b * p.Hkv + kvh) * kHD + lane * 8);
}

template <int G>
__global__ void __launch_bounds__(kW * 32, 2) attn_split_kernel(const AttnParams p) {
  bk_pdl_trigger();
  bk_stamp(p.trace, 0);
  extern __shared__ __align__(16) uint8_t smem[];
  uint16_t* q_st = reinterpret_cast<uint16_t*>(smem);
  uint16_t* k_st = q_st + 8 * kHD;
  float* m_s = reinterpret_cast<float*>(k_st + kHD);
  float* l_s = m_s + 16;
  float* s_s = l_s + kW * 8;
  float* o_s = s_s + (size_t)p.split_len * 8;
  __shared__ int s_last;

  const int split = blockIdx.x, kvh = blockIdx.y, b = blockIdx.z;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, tid = threadIdx.x;
  const int cb = p.n_seq > 0 ? b % p.n_seq : b;   // whose cache
  uint16_t* Kb = p.k_cache + ((size_t)cb * p.Hkv + kvh) * (size_t)p.max_len * kHD;
  uint16_t* Vb = p.v_cache + ((size_t)cb * p.Hkv + kvh) * (size_t)p.max_len * kHD;
  const int j0 = split * p.split_len;

  // rows of this warp: jj = warp + 8*i; chunk c holds i in [kCh*c, kCh*c + kCh)
  uint4 kc[kCh], vc[kCh];
  int pos = 0, ns = 0;
  auto load_chunk = [&](const uint16_t* base, int c, uint4 (&dst)[kCh], bool skip_pos) {
#pragma unroll
    for (int e = 0; e < kCh; e++) {
      const int jj = warp + 8 * (kCh * c + e);
      const bool ok = jj < ns && !(skip_pos && j0 + jj == pos);
      dst[e] = ok ? *reinterpret_cast<const uint4*>(base + (size_t)(j0 + jj) * kHD + lane * 8) : make_uint4(0, 0, 0, 0);
    }
  };
  bool early = false;   // the first chunks were requested before the dependency wait and are still the right ones
  if (p.settled) {
    pos = p.pos[b];
    ns = min(pos + 1, j0 + p.split_len) - j0;   // <= 0: nothing to do for this split
    if (ns > 0) {
      load_chunk(Kb, 0, kc, true);
      load_chunk(Vb, 0, vc, true);
    }
    early = true;
  }
  bk_pdl_wait();
  bk_stamp(p.trace, 2);
  {
    // The position is taken (again) after the wait: the kernel that advances it may be only a few launches back and
    // still have been running when the early part above read it.  A changed value discards the early loads.
    const int pos_now = __ldcg(p.pos + b);
    if (!early || pos_now != pos) {
      early = false;
      pos = pos_now;
      ns = min(pos + 1, j0 + p.split_len) - j0;
    }
  }
  if (ns <= 0) return;
  const int nsplits = (pos + p.split_len) / p.split_len;

  // ---- phase 0: q (and, in the split that owns row pos, k/v append) ----
  if (p.fused) {
    const float* cr = p.cos_t + (size_t)pos * p.rot_half;
    const float* sr = p.sin_t + (size_t)pos * p.rot_half;
    if (warp < G) {
      const uint16_t* src = p.qg + ((size_t)b * p.Hq + kvh * G + warp) * 2 * kHD;
      norm_rope_256(src, p.q_norm_w, cr, sr, p.rot_half, q_st + warp * kHD);
    }
    if (p.n_seq == 0 && warp == kW - 1 && pos >= j0 && pos < j0 + ns) {
      norm_rope_256(p.k + ((size_t)b * p.Hkv + kvh) * kHD, p.k_norm_w, cr, sr, p.rot_half, k_st);
      *reinterpret_cast<uint4*>(Kb + (size_t)pos * kHD + lane * 8) = *reinterpret_cast<const uint4*>(k_st + lane * 8);
      *reinterpret_cast<uint4*>(Vb + (size_t)pos * kHD + lane * 8) =
          *reinterpret_cast<const uint4*>(p.v + ((size_t)b * p.Hkv + kvh) * kHD + lane * 8);
    }
  } else {
    if (warp < G)
      *reinterpret_cast<uint4*>(q_st + warp * kHD + lane * 8) =
          *reinterpret_cast<const uint4*>(p.qg + ((size_t)b * p.Hq + kvh * G + warp) * kHD + lane * 8);
  }
  __syncthreads();  // the appended K/V row is visible to this CTA from here on
  bk_stamp(p.trace, 3);
  if (!early) {
    load_chunk(Kb, 0, kc, false);
    load_chunk(Vb, 0, vc, false);
  } else {
    // the row appended above was left out of the early loads
    const int jp = pos - j0;
    if (jp >= 0 && jp < ns && (jp & 7) == warp && (jp >> 3) < kCh) {
      const int e = jp >> 3;
#pragma unroll
      for (int i = 0; i < kCh; i++)
        if (i == e) {
          kc[i] = *reinterpret_cast<const uint4*>(Kb + (size_t)pos * kHD + lane * 8);
          vc[i] = *reinterpret_cast<const uint4*>(Vb + (size_t)pos * kHD + lane * 8);
        }
    }
  }
  const int nchunks = (ns + 8 * kCh - 1) / (8 * kCh);

  // ---- phase 1: scores ----
  {
    // query heads in pairs {q_g[d], q_g+1[d]}: one packed FMA advances the dot products of two heads (each its own
    // chain over d, as before)
    float2 qp[(G + 1) / 2][8];
#pragma unroll
    for (int g = 0; g < G; g += 2) {
      float q0[8], q1[8];
      bf16x8_to_f32(*reinterpret_cast<const uint4*>(q_st + g * kHD + lane * 8), q0);
      if (g + 1 < G) bf16x8_to_f32(*reinterpret_cast<const uint4*>(q_st + (g + 1) * kHD + lane * 8), q1);
#pragma unroll
      for (int d = 0; d < 8; d++) qp[g >> 1][d] = make_float2(q0[d], g + 1 < G ? q1[d] : 0.0f);
    }
    const int hsel = ((lane >> 4) & 1) * 4 + ((lane >> 3) & 1) * 2 + ((lane >> 2) & 1);
    for (int c = 0; c < nchunks; c++) {
      uint4 kn[kCh];
      if (c + 1 < nchunks) load_chunk(Kb, c + 1, kn, false);
#pragma unroll
      for (int e = 0; e < kCh; e++) {
        const int jj = warp + 8 * (kCh * c + e);
        if (jj < ns) {   // warp-uniform
          float kf[8], pa[8];
          bf16x8_to_f32(kc[e], kf);
#pragma unroll
          for (int g = 0; g < 8; g += 2) {
            float2 a2 = make_float2(0.0f, 0.0f);
            if (g < G) {
#pragma unroll
              for (int d = 0; d < 8; d++) a2 = bk_fma2(qp[(g < G ? g : 0) >> 1][d], make_float2(kf[d], kf[d]), a2);
            }
            pa[g] = a2.x;
            pa[g + 1] = a2.y;
          }
          const float s1 = warp_sum8(pa);
          if ((lane & 3) == 0) s_s[(size_t)jj * 8 + hsel] = __fmul_rn(s1, p.scale);
        }
      }
      if (c + 1 < nchunks) {
#pragma unroll
        for (int e = 0; e < kCh; e++) kc[e] = kn[e];
      }
    }
  }
  __syncthreads();
  bk_stamp(p.trace, 4);

  // ---- phase 2: exact max per head, p = exp(s - m) in place ----
  {
    const int g = tid & 7;
    float m = -INFINITY;
    for (int jj = tid >> 3; jj < ns; jj += (kW * 32) >> 3) m = fmaxf(m, s_s[(size_t)jj * 8 + g]);
    m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, 8));
    m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, 16));
    if (lane < 8) l_s[warp * 8 + lane] = m;  // l_s doubles as the cross-warp max buffer
    __syncthreads();
    if (tid < 8) {
      float mm = l_s[tid];
#pragma unroll
      for (int w = 1; w < kW; w++) mm = fmaxf(mm, l_s[w * 8 + tid]);
      m_s[tid] = mm;
    }
    __syncthreads();
    const float mg = m_s[g];
    for (int jj = tid >> 3; jj < ns; jj += (kW * 32) >> 3) {
      float sv = s_s[(size_t)jj * 8 + g];
      s_s[(size_t)jj * 8 + g] = (g < G) ? bk_expf(__fsub_rn(sv, mg)) : 0.0f;
    }
  }
  __syncthreads();

  // ---- phase 3: o = sum p * V ----
  {
    float2 acc[G][4];   // dims (2i, 2i+1) side by side: one packed FMA per pair
    float lw[G];
#pragma unroll
    for (int g = 0; g < G; g++) {
      lw[g] = 0.0f;
#pragma unroll
      for (int e = 0; e < 4; e++) acc[g][e] = make_float2(0.0f, 0.0f);
    }
    for (int c = 0; c < nchunks; c++) {
      uint4 vn[kCh];
      if (c + 1 < nchunks) load_chunk(Vb, c + 1, vn, false);
#pragma unroll
      for (int e = 0; e < kCh; e++) {
        const int jj = warp + 8 * (kCh * c + e);
        if (jj < ns) {
          float vf[8];
          bf16x8_to_f32(vc[e], vf);
          const float4 p0 = *reinterpret_cast<const float4*>(s_s + (size_t)jj * 8);
          const float4 p1 = *reinterpret_cast<const float4*>(s_s + (size_t)jj * 8 + 4);
          const float pp[8] = {p0.x, p0.y, p0.z, p0.w, p1.x, p1.y, p1.z, p1.w};
#pragma unroll
          for (int g = 0; g < G; g++) {
            lw[g] = __fadd_rn(lw[g], pp[g]);
            const float2 p2 = make_float2(pp[g], pp[g]);
#pragma unroll
            for (int d = 0; d < 4; d++) acc[g][d] = bk_fma2(p2, make_float2(vf[2 * d], vf[2 * d + 1]), acc[g][d]);
          }
        }
      }
      if (c + 1 < nchunks) {
#pragma unroll
        for (int e = 0; e < kCh; e++) vc[e] = vn[e];
      }
    }
#pragma unroll
    for (int g = 0; g < G; g++) {
      float4* d = reinterpret_cast<float4*>(o_s + ((size_t)(warp * 8 + g)) * kHD + lane * 8);
      d[0] = make_float4(acc[g][0].x, acc[g][0].y, acc[g][1].x, acc[g][1].y);
      d[1] = make_float4(acc[g][2].x, acc[g][2].y, acc[g][3].x, acc[g][3].y);
      if (lane == 0) l_s[warp * 8 + g] = lw[g];
    }
  }
  __syncthreads();
  bk_stamp(p.trace, 6);

  // ---- cross-warp sums in warp order, partial out ----
  float* sc_ml = p.scratch;
  float* sc_o = p.scratch + (size_t)p.layout_B * p.Hq * p.max_splits * 2;
  for (int idx = tid; idx < G * kHD; idx += kW * 32) {
    const int g = idx >> 8, d = idx & 255;
    float o = o_s[(size_t)g * kHD + d];
#pragma unroll
    for (int w = 1; w < kW; w++) o = __fadd_rn(o, o_s[((size_t)(w * 8 + g)) * kHD + d]);
    sc_o[(((size_t)b * p.Hq + kvh * G + g) * p.max_splits + split) * kHD + d] = o;
  }
  if (tid < G) {
    float l = l_s[tid];
#pragma unroll
    for (int w = 1; w < kW; w++) l = __fadd_rn(l, l_s[w * 8 + tid]);
    size_t o = (((size_t)b * p.Hq + kvh * G + tid) * p.max_splits + split) * 2;
    sc_ml[o] = m_s[tid];
    sc_ml[o + 1] = l;
  }

  // ---- the CTA that completes this (batch, KV head) merges its splits ----
  __threadfence();
  __syncthreads();
  bk_stamp(p.trace, 7);
  unsigned int* cnt = reinterpret_cast<unsigned int*>(p.scratch + (size_t)p.layout_B * p.Hq * p.max_splits * (kHD + 2)) + b * p.Hkv + kvh;
  if (tid == 0) {
    const unsigned int done = atomicAdd(cnt, 1u);
    s_last = (done == (unsigned int)(nsplits - 1));
  }
  __syncthreads();
  if (s_last) {
    __threadfence();
    if (warp < G) combine_head_warp(p, b, kvh * G + warp, nsplits, o_s + warp * kMaxSplits);  // one head per warp
    if (tid == 0) *cnt = 0;
  }
  bk_stamp(p.trace, 5);
}

size_t attn_smem_bytes(int split_len) { return 4096 + 512 + 64 + 256 + (size_t)split_len * 32 + (size_t)kW * 8 * kHD * 4; }

template <int G>
int32_t launch_split(const AttnParams& p, dim3 grid, size_t smem) {
  static size_t configured = 0;
  if (smem > configured) {
    BK_CUDA(cudaFuncSetAttribute(attn_split_kernel<G>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    configured = smem;
  }
  BK_CUDA(bk_launch_pdl(attn_split_kernel<G>, grid, dim3(kW * 32), smem, p));
  BK_CHECK_LAUNCH();
  return BK_OK;
}

}  // namespace

extern "C" {

int32_t bkAttnPlan(int32_t n_rows, int32_t B, int32_t Hkv, int32_t* split_len, int32_t* warps) {
  BK_REQUIRE_INIT();
  BK_ARG(n_rows > 0 && B > 0 && Hkv > 0 && split_len, "bkAttnPlan: bad arguments");
  // enough splits for about two CTAs per SM, rows per split a multiple of 64 in [64, 512]
  int target = (2 * bk_ctx().sm_count + B * Hkv - 1) / (B * Hkv);
  int len = (n_rows + target - 1) / target;
  len = ((len + 63) / 64) * 64;
  if (len < 64) len = 64;
  if (len > 512) len = 512;
  *split_len = len;
  if (warps) *warps = kW;
  return BK_OK;
}

uint64_t bkAttnScratchBytes(int32_t B, int32_t Hq, int32_t HD, int32_t max_len, int32_t split_len) {
  if (split_len <= 0) return 0;
  uint64_t ms = (uint64_t)(max_len + split_len - 1) / split_len;
  return (uint64_t)B * Hq * ms * (uint64_t)(HD + 2) * 4 + (uint64_t)B * Hq * 4;  // partials + completion counters
}

int32_t bkAttnDecode(const bkAttnArgs* args) {
  BK_REQUIRE_INIT();
  BK_ARG(args != nullptr, "bkAttnDecode: args is null");
  return bk_attn_launch(*args, 0, 0);
}

}  // extern "C"

// n_seq > 0: the B entries are prompt columns of n_seq sequences (entry b = token b / n_seq of sequence b mod n_seq,
// pos[b] its position): one launch appends every column's K/V row, a second one attends -- the same arithmetic per
// column as B / n_seq decode steps.  layout_B > 0: the scratch buffer was sized for that many entries (launches with
// different B then share one buffer).
int32_t bk_attn_launch(const bkAttnArgs& args, int n_seq, int layout_B) {
  bkAttnArgs a = args;
  BK_ARG(layout_B == 0 || layout_B >= a.B, "attention: scratch laid out for %d entries, %d given", layout_B, a.B);
  BK_ARG(n_seq >= 0 && (n_seq == 0 || (a.B % n_seq == 0 && a.fused_norm_rope)), "attention: %d columns of %d sequences", a.B, n_seq);
  BK_ARG(a.HD == kHD, "bkAttnDecode: head_dim %d unsupported (256 only)", a.HD);
  BK_ARG(a.B > 0 && a.Hq > 0 && a.Hkv > 0 && a.Hq % a.Hkv == 0 && a.Hq / a.Hkv <= 8,
         "bkAttnDecode: bad head counts B=%d Hq=%d Hkv=%d (group size 1..8)", a.B, a.Hq, a.Hkv);
  BK_ARG(a.max_len > 0 && a.max_pos >= 0 && a.max_pos < a.max_len, "bkAttnDecode: max_pos=%d outside cache of %d rows",
         a.max_pos, a.max_len);
  BK_ARG(a.qg && a.k_cache && a.v_cache && a.pos && a.out && a.scratch, "bkAttnDecode: null pointer");
  BK_ARG(((a.qg | a.k_cache | a.v_cache | a.out) & 15) == 0, "bkAttnDecode: pointers must be 16-byte aligned");
  if (a.fused_norm_rope) {
    BK_ARG(a.k && a.v && a.q_norm_w && a.k_norm_w && a.cos_t && a.sin_t, "bkAttnDecode: fused mode needs k, v, norm weights and tables");
    BK_ARG(((a.k | a.v | a.q_norm_w | a.k_norm_w) & 15) == 0, "bkAttnDecode: pointers must be 16-byte aligned");
    BK_ARG(a.rot_half > 0 && 2 * a.rot_half <= kHD, "bkAttnDecode: rot_half=%d", a.rot_half);
  } else {
    BK_ARG(a.gate != 0, "bkAttnDecode: gate is null");
  }
  int split_len = a.split_len;
  if (split_len <= 0) {
    int32_t rc = bkAttnPlan(a.max_pos + 1, a.B, a.Hkv, &split_len, nullptr);
    if (rc) return rc;
  }
  BK_ARG(split_len % 8 == 0 && split_len <= 2048, "bkAttnDecode: split_len=%d must be a multiple of 8, at most 2048", split_len);
  int max_splits = (a.max_len + split_len - 1) / split_len;
  BK_ARG(max_splits <= kMaxSplits, "bkAttnDecode: %d splits exceed the limit of %d", max_splits, kMaxSplits);
  int nsplit = (a.max_pos + split_len) / split_len;
  AttnParams p;
  p.qg = bk_ptr<uint16_t>(a.qg);
  p.k = bk_ptr<uint16_t>(a.k);
  p.v = bk_ptr<uint16_t>(a.v);
  p.q_norm_w = bk_ptr<uint16_t>(a.q_norm_w);
  p.k_norm_w = bk_ptr<uint16_t>(a.k_norm_w);
  p.cos_t = bk_ptr<float>(a.cos_t);
  p.sin_t = bk_ptr<float>(a.sin_t);
  p.k_cache = bk_ptr<uint16_t>(a.k_cache);
  p.v_cache = bk_ptr<uint16_t>(a.v_cache);
  p.pos = bk_ptr<int32_t>(a.pos);
  p.out = bk_ptr<uint16_t>(a.out);
  p.out_q8 = bk_ptr<uint8_t>(a.out_q8);
  p.out_q8_staged = a.out_q8_layout == BK_Q8_STAGED;
  BK_ARG(a.out_q8_layout == BK_Q8_BLOCKS || a.out_q8_layout == BK_Q8_STAGED, "bkAttnDecode: out_q8_layout %d", a.out_q8_layout);
  p.scratch = bk_ptr<float>(a.scratch);
  p.gate = bk_ptr<uint16_t>(a.gate);
  p.B = a.B;
  p.Hq = a.Hq;
  p.Hkv = a.Hkv;
  p.rot_half = a.rot_half;
  p.max_len = a.max_len;
  p.split_len = split_len;
  p.max_splits = max_splits;
  p.fused = a.fused_norm_rope;
  p.scale = a.scale;
  p.trace = bk_trace_slot();
  p.settled = n_seq ? 0 : a.cache_is_settled;
  p.n_seq = n_seq;
  p.layout_B = layout_B ? layout_B : a.B;
  if (n_seq) {
    BK_CUDA(bk_launch_pdl(attn_append_kernel, dim3(a.Hkv, a.B), dim3(32), 0, p));
    BK_CHECK_LAUNCH();
  }
  size_t smem = attn_smem_bytes(split_len);
  dim3 grid(nsplit, a.Hkv, a.B);
  int32_t rc;
  switch (a.Hq / a.Hkv) {
    case 1: rc = launch_split<1>(p, grid, smem); break;
    case 2: rc = launch_split<2>(p, grid, smem); break;
    case 3: rc = launch_split<3>(p, grid, smem); break;
    case 4: rc = launch_split<4>(p, grid, smem); break;
    case 5: rc = launch_split<5>(p, grid, smem); break;
    case 6: rc = launch_split<6>(p, grid, smem); break;
    case 7: rc = launch_split<7>(p, grid, smem); break;
    default: rc = launch_split<8>(p, grid, smem); break;
  }
  if (rc) return rc;
  return BK_OK;
}
