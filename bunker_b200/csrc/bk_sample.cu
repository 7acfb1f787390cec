// bk_sample.cu -- temperature / top-k / top-p sampling over f32 logits, deterministic and reproducible on a host.
//
// bunker only has the greedy tail (buildArgmax + buildArgmaxComb, prototypes/decode.ts:749-791); this is the sampling
// step that stands beside it.  Per sequence:
//   1. the top_k (<= 64) largest logits, ties to the lower index, in descending order (exact selection: round r finds
//      the largest element that comes after round r-1's pick in that order);
//   2. p_i = exp((l_i - l_0) / T) with the library's own exp, summed in that order;
//   3. nucleus: the shortest prefix whose running sum reaches top_p * total;
//   4. u in [0,1) from a counter-based hash of (seed, step, sequence); the first i whose running sum exceeds u * prefix
//      total is the token.
// One CTA of 1024 threads per sequence; the k selection rounds scan the logits from L2.
#include <math.h>

#include "bk_common.cuh"
#include "bk_internal.h"

namespace {

constexpr int kSampleMaxK = 64;

// order of candidates: larger logit first, then lower index
BK_DEVINL bool cand_after(float v, int i, float pv, int pi) { return v < pv || (v == pv && i > pi); }
BK_DEVINL bool cand_better(float v, int i, float bv, int bi) { return v > bv || (v == bv && i < bi); }

BK_DEVINL unsigned long long splitmix64(unsigned long long x) {
  x += 0x9E3779B97F4A7C15ull;
  x = (x ^ (x >> 30)) * 0xBF58476D1CE4E5B9ull;
  x = (x ^ (x >> 27)) * 0x94D049BB133111EBull;
  return x ^ (x >> 31);
}

__global__ void __launch_bounds__(1024) sample_kernel(const float* logits, int V, float temperature, int top_k, float top_p,
                                                      unsigned long long seed, const int32_t* step_dev, unsigned int step_add,
                                                      int32_t* idx_out, float* val_out) {
  __shared__ float sv[32];
  __shared__ int si[32];
  __shared__ float cv[kSampleMaxK];
  __shared__ int ci[kSampleMaxK];
  const int b = blockIdx.x, tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const float* l = logits + (size_t)b * V;
  float pv = INFINITY;
  int pi = -1;
  for (int r = 0; r < top_k; r++) {
    float bv = -INFINITY;
    int bi = 0x7fffffff;
    for (int i = tid; i < V; i += 1024) {
      const float v = __ldcg(l + i);
      if (v == v && cand_after(v, i, pv, pi) && cand_better(v, i, bv, bi)) {
        bv = v;
        bi = i;
      }
    }
    for (int off = 16; off >= 1; off >>= 1) {
      const float ov = __shfl_xor_sync(0xffffffffu, bv, off);
      const int oi = __shfl_xor_sync(0xffffffffu, bi, off);
      if (cand_better(ov, oi, bv, bi)) {
        bv = ov;
        bi = oi;
      }
    }
    if (lane == 0) {
      sv[warp] = bv;
      si[warp] = bi;
    }
    __syncthreads();
    if (warp == 0) {
      bv = sv[lane];
      bi = si[lane];
      for (int off = 16; off >= 1; off >>= 1) {
        const float ov = __shfl_xor_sync(0xffffffffu, bv, off);
        const int oi = __shfl_xor_sync(0xffffffffu, bi, off);
        if (cand_better(ov, oi, bv, bi)) {
          bv = ov;
          bi = oi;
        }
      }
      if (lane == 0) {
        cv[r] = bv;
        ci[r] = bi;
      }
    }
    __syncthreads();
    pv = cv[r];
    pi = ci[r];
    if (pi == 0x7fffffff) {   // fewer than top_k finite logits
      top_k = r;
      break;
    }
  }
  if (tid == 0) {
    int pick = 0;
    if (top_k <= 0) {
      idx_out[b] = 0;
      if (val_out) val_out[b] = -INFINITY;
      return;
    }
    if (temperature > 0.0f && top_k > 1) {
      float pr[kSampleMaxK];
      const float inv_t = __fdiv_rn(1.0f, temperature);
      float total = 0.0f;
      for (int i = 0; i < top_k; i++) {
        pr[i] = bk_expf(__fmul_rn(__fsub_rn(cv[i], cv[0]), inv_t));
        total = __fadd_rn(total, pr[i]);
      }
      const float need = __fmul_rn(top_p, total);
      int n = top_k;
      float run = 0.0f;
      for (int i = 0; i < top_k; i++) {
        run = __fadd_rn(run, pr[i]);
        if (run >= need) {
          n = i + 1;
          break;
        }
      }
      float prefix = 0.0f;
      for (int i = 0; i < n; i++) prefix = __fadd_rn(prefix, pr[i]);
      const unsigned int step = (step_dev ? (unsigned int)step_dev[b] : 0u) + step_add;
      const unsigned long long h = splitmix64(splitmix64(seed ^ ((unsigned long long)step << 20)) + (unsigned long long)b);
      const float u = __fmul_rn((float)(unsigned int)(h >> 40), 5.9604644775390625e-8f);   // 24 bits -> [0,1)
      const float target = __fmul_rn(u, prefix);
      pick = n - 1;
      run = 0.0f;
      for (int i = 0; i < n; i++) {
        run = __fadd_rn(run, pr[i]);
        if (run > target) {
          pick = i;
          break;
        }
      }
    }
    idx_out[b] = ci[pick];
    if (val_out) val_out[b] = cv[pick];
  }
}

}  // namespace

extern "C" int32_t bkSample(uint64_t logits, int32_t V, int32_t B, float temperature, int32_t top_k, float top_p, uint64_t seed,
                            uint64_t step_dev, uint32_t step_add, uint64_t idx, uint64_t val) {
  BK_REQUIRE_INIT();
  BK_ARG(logits && idx && V > 0 && B > 0, "bkSample: bad arguments");
  BK_ARG(top_k >= 1 && top_k <= kSampleMaxK, "bkSample: top_k=%d outside 1..%d", top_k, kSampleMaxK);
  BK_ARG(temperature >= 0.0f && top_p > 0.0f && top_p <= 1.0f, "bkSample: temperature=%g top_p=%g", (double)temperature, (double)top_p);
  sample_kernel<<<B, 1024, 0, bk_ctx().stream>>>(bk_ptr<float>(logits), V, temperature, top_k, top_p, (unsigned long long)seed,
                                                 bk_ptr<int32_t>(step_dev), step_add, bk_ptr<int32_t>(idx), bk_ptr<float>(val));
  BK_CHECK_LAUNCH();
  return BK_OK;
}
