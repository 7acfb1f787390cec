// bk_launch.cu -- cuLaunch-shaped entry: an op id plus 8-byte argument slots, the way
// bunker's cuLaunch packs kernel arguments (src/ttir.ts:321-348: every argument in one
// 8-byte slot, pointers as u64, integers as i64).  Floats travel as their f32 bits.
#include <string.h>

#include "bk_internal.h"

static inline float slot_f32(uint64_t s) {
  uint32_t u = (uint32_t)s;
  float f;
  memcpy(&f, &u, 4);
  return f;
}

extern "C" int32_t bkLaunch(int32_t op, const uint64_t* s, int32_t n) {
  BK_REQUIRE_INIT();
  BK_ARG(s != nullptr || n == 0, "bkLaunch: slots is null");
  switch (op) {
    case BK_OP_EMBED:  // table, x_out, ids, H, B
      BK_ARG(n == 5, "bkLaunch(embed): expected 5 slots, got %d", n);
      return bkEmbedQ4K(s[0], (int32_t)s[3], s[2], (int32_t)s[4], s[1]);
    case BK_OP_RMSNORM:  // x, w, y, H, B, eps
      BK_ARG(n == 6, "bkLaunch(rmsnorm): expected 6 slots, got %d", n);
      return bkRmsNorm(s[0], s[1], (int32_t)s[3], (int32_t)s[4], slot_f32(s[5]), s[2]);
    case BK_OP_GEMV: {  // A(q8_1), W, C, N, K, B, epilogue, R, W2
      BK_ARG(n == 9, "bkLaunch(gemm): expected 9 slots, got %d", n);
      bkGemvArgs a;
      memset(&a, 0, sizeof(a));
      a.K = (int32_t)s[4];
      a.B = (int32_t)s[5];
      a.n_segs = 1;
      a.prologue = BK_PRO_Q8;
      a.x = s[0];
      a.segs[0].W = s[1];
      a.segs[0].out = s[2];
      a.segs[0].n_rows = (int32_t)s[3];
      a.segs[0].epilogue = (int32_t)s[6];
      a.segs[0].residual = s[7];
      a.segs[0].W2 = s[8];
      a.segs[0].ld_out = (int32_t)s[3];
      return bkGemvQ4K(&a);
    }
    case BK_OP_SWIGLU:  // g, u, out, n
      BK_ARG(n == 4, "bkLaunch(swiglu): expected 4 slots, got %d", n);
      return bkSwiglu(s[0], s[1], (int32_t)s[3], s[2]);
    case BK_OP_CONV1D:  // x, state_in, w, out, state_new, C, B
      BK_ARG(n == 7, "bkLaunch(conv1d_decode): expected 7 slots, got %d", n);
      return bkConv1dStep(s[0], s[1], s[2], (int32_t)s[5], (int32_t)s[6], s[3], s[4]);
    case BK_OP_ARGMAX:  // logits, idx, val, scratch, V, B
      BK_ARG(n == 6, "bkLaunch(argmax): expected 6 slots, got %d", n);
      return bkArgmax(s[0], (int32_t)s[4], (int32_t)s[5], s[1], s[2], s[3]);
    case BK_OP_QUANT_Q8_1:  // x_f32, out, K, B
      BK_ARG(n == 4, "bkLaunch(quant_q8_1): expected 4 slots, got %d", n);
      return bkQuantQ8_1(s[0], (int32_t)s[2], (int32_t)s[3], s[1]);
    case BK_OP_QUANT_Q8_1_BF16:  // x_bf16, out, K, B
      BK_ARG(n == 4, "bkLaunch(quant_q8_1_bf16): expected 4 slots, got %d", n);
      return bkQuantQ8_1Bf16(s[0], (int32_t)s[2], (int32_t)s[3], s[1]);
    case BK_OP_HEADNORM_ROPE:  // x, in_stride, w, cos_t, sin_t, rot_half, pos, B, nheads, HD, out
      BK_ARG(n == 11, "bkLaunch(headnorm_rope): expected 11 slots, got %d", n);
      return bkHeadNormRope(s[0], (int32_t)s[1], s[2], s[3], s[4], (int32_t)s[5], s[6], (int32_t)s[7], (int32_t)s[8],
                            (int32_t)s[9], s[10]);
    case BK_OP_GDN: {  // qkv, z, a, b, conv_w, conv_state_in, conv_state_new, A_log, dt_bias, norm_w, S_in, S_new, out,
                       // B, Hk, Hv, apply_conv, state_is_settled
      BK_ARG(n == 18, "bkLaunch(gdn): expected 18 slots, got %d", n);
      bkGdnArgs a;
      memset(&a, 0, sizeof(a));
      a.qkv = s[0]; a.z = s[1]; a.a = s[2]; a.b = s[3]; a.conv_w = s[4]; a.conv_state_in = s[5]; a.conv_state_new = s[6];
      a.A_log = s[7]; a.dt_bias = s[8]; a.norm_w = s[9]; a.S_in = s[10]; a.S_new = s[11]; a.out = s[12];
      a.B = (int32_t)s[13]; a.Hk = (int32_t)s[14]; a.Hv = (int32_t)s[15]; a.apply_conv = (int32_t)s[16];
      a.state_is_settled = (int32_t)s[17];
      return bkGdnStep(&a);
    }
    case BK_OP_ATTN: {  // qg, k, v, q_norm_w, k_norm_w, cos_t, sin_t, k_cache, v_cache, pos, out, scratch,
                        // B, Hq, Hkv, HD, rot_half, max_len, split_len, max_pos, scale (f32 bits), cache_is_settled
      BK_ARG(n == 22, "bkLaunch(attn): expected 22 slots, got %d", n);
      bkAttnArgs a;
      memset(&a, 0, sizeof(a));
      a.qg = s[0]; a.k = s[1]; a.v = s[2]; a.q_norm_w = s[3]; a.k_norm_w = s[4]; a.cos_t = s[5]; a.sin_t = s[6];
      a.k_cache = s[7]; a.v_cache = s[8]; a.pos = s[9]; a.out = s[10]; a.scratch = s[11];
      a.B = (int32_t)s[12]; a.Hq = (int32_t)s[13]; a.Hkv = (int32_t)s[14]; a.HD = (int32_t)s[15]; a.rot_half = (int32_t)s[16];
      a.max_len = (int32_t)s[17]; a.split_len = (int32_t)s[18]; a.max_pos = (int32_t)s[19]; a.scale = slot_f32(s[20]);
      a.fused_norm_rope = 1;
      a.cache_is_settled = (int32_t)s[21];
      return bkAttnDecode(&a);
    }
    default:
      return bk_fail(BK_ERR_ARG, "bkLaunch: unknown op id %d", op);
  }
}
