// bk_gemv_mma.cu -- Q4_K x Q8_1 GEMV for batch 3..8 on the int8 tensor-core path (mma.sync m16n8k32).
//
// At these batch sizes 16 dp4a per 64 weights per batch column no longer fit under the HBM stream; one
// m16n8k32 computes a 32-value sub-block dot for 16 rows and all 8 batch columns, with exact int32 sums,
// so the integer stage stays bit-identical to the scalar one.  (north star: "integer dp4a-style block dots";
// the tcgen05 tile path starts at batch 16, where a CTA-wide tile pays for its TMEM round trip.)
//
// Work split.  A tile = 16 virtual rows; a warp task = (tile, p) with p = 0..3 the sub-block pair
// (sub-blocks 2p, 2p+1 of every superblock).  The low nibbles of a 32-byte quant group are sub-block 2p and
// the high nibbles 2p+1, and a lane's A fragment wants bytes 4j..4j+3 and 16+4j..19+4j of rows R and R+8
// (R = lane/4, j = lane%4): four 32-bit loads give both fragments.  B fragments come from the staged Q8_1
// activation, [batch][K] int8.  Per (row, column) the warp forms exactly the unit values of the scalar kernel,
//     val(s,p) = fma(d, fma(d8_1, f32(sc1*i1), d8_0*f32(sc0*i0)), -(dmin * fma(s8_1, m1, s8_0*m0)))
// and adds them in the order the 32-lane scheme defines: class c = s mod 8 collects s = c, c+8, ... in
// ascending order; T_p = ((P0+P4)+(P2+P6)) + ((P1+P5)+(P3+P7)); row total = (T0+T2) + (T1+T3) across the four
// p-warps through shared memory.  The result is bit-identical to gemv_q4k_kernel and to the CPU checker.
//
// Rows of a tile sit in shared memory at a stride of rowb+16 bytes (one bulk copy per row): with the natural
// stride (a multiple of 128 bytes) the eight rows of an A fragment would hit the same banks.
// A SwiGLU tile holds 8 gate rows then their 8 up rows, so a lane's (row R, row R+8) pair is one output.
#include "bk_gemv_shared.cuh"

namespace {

constexpr int kTileRows = 16;
constexpr int kMaxTilesPerRound = 4;  // a round = tiles_per_round tiles x 4 sub-block pairs = up to 16 warps

__device__ __forceinline__ void mma_s8(int (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1) {
  asm volatile("mma.sync.aligned.m16n8k32.row.col.s32.s8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
               : "+r"(c[0]), "+r"(c[1]), "+r"(c[2]), "+r"(c[3])
               : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

struct RowHdr {
  float d, dmin, fm0, fm1;
  int sc0, sc1;
};

__device__ __forceinline__ RowHdr decode_hdr(const uint8_t* sb, int p) {
  const uint4 h = *reinterpret_cast<const uint4*>(sb);
  RowHdr r;
  r.d = bk_f16_to_f32((uint16_t)(h.x & 0xffffu));
  r.dmin = bk_f16_to_f32((uint16_t)(h.x >> 16));
  uint32_t sc2, mn2;
  bk_q4k_scale_min_pair(h.y, h.z, h.w, p, sc2, mn2);
  r.sc0 = (int)(sc2 & 0xffu);
  r.sc1 = (int)(sc2 >> 8);
  r.fm0 = (float)(int)(mn2 & 0xffu);
  r.fm1 = (float)(int)(mn2 >> 8);
  return r;
}

// unit value for one (row, column): i0/i1 exact sub-block sums, d8/s8 of the column's two Q8_1 blocks
__device__ __forceinline__ float unit_value(const RowHdr& h, int i0, int i1, float2 d8, float2 s8) {
  float accd = __fmul_rn(d8.x, (float)(h.sc0 * i0));
  accd = fmaf(d8.y, (float)(h.sc1 * i1), accd);
  float accm = __fmul_rn(s8.x, h.fm0);
  accm = fmaf(s8.y, h.fm1, accm);
  const float t = __fmul_rn(h.dmin, accm);
  return fmaf(h.d, accd, -t);
}

// Shared memory: xs [B][K/4 + 4] words | d8s [B][K/32+2] | s8s [B][K/32+2] | red[72] | bars[n_slots] | part[2][4 tiles][4 p][16][8] f32 |
// tile slots [n_slots][16 rows][rowb+16].
__global__ void __launch_bounds__(kMaxTilesPerRound * 128, 1) gemv_q4k_mma_kernel(const GemvParams p, const int B) {
  bk_pdl_trigger();
  bk_stamp(p.trace, 0);
  extern __shared__ __align__(128) uint8_t smem_raw[];
  const int K = p.K, nsb = K / 256;
  uint32_t* xs = reinterpret_cast<uint32_t*>(smem_raw);
  float* d8s = reinterpret_cast<float*>(xs + (size_t)B * p.x_row_words);
  float* s8s = d8s + (size_t)B * p.x_scale_ld;
  float* red = s8s + (size_t)B * p.x_scale_ld;
  uint64_t* bars = reinterpret_cast<uint64_t*>(red + 72);   // red: 8 warp sums per batch row + one rstd per row
  const int tpr = blockDim.x >> 7;   // tiles per round (4 or 2): four warps per tile
  const int nwarps = blockDim.x >> 5;
  float* part = reinterpret_cast<float*>((reinterpret_cast<uintptr_t>(bars + p.n_slots) + 15) & ~(uintptr_t)15);
  uint8_t* slots = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(part + 2 * tpr * 4 * 128) + 127) & ~(uintptr_t)127);

  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, tid = threadIdx.x;
  // tiles are dealt out evenly: the first tiles_extra CTAs own one tile more than the others
  const int cta = blockIdx.x;
  const int tile0 = cta < p.tiles_extra ? cta * (p.tiles_base + 1) : p.tiles_extra + cta * p.tiles_base;
  const int n_tiles = p.tiles_base + (cta < p.tiles_extra ? 1 : 0);
  const int c0 = tile0 * kTileRows;
  const int n_rows_cta = min(p.total_vrows, c0 + n_tiles * kTileRows) - c0;
  const uint32_t rowb = (uint32_t)nsb * 144, rstride = rowb + 16;
  const uint32_t slot_bytes = kTileRows * rstride;
  const int n_slots = p.n_slots;      // >= tiles of the CTA (pool) or a multiple of 4 (ring)
  const uint32_t bar_base = smem_u32(bars), slot_base = smem_u32(slots);
  const bool swiglu = p.segs[0].epi == BK_EPI_SWIGLU;

  // one bulk copy per row (padded stride); requested by lane 0 of the warp with p == 0 of the tile's round position
  auto request_tile = [&](int t, int slot) {
    const int nr = min(kTileRows, n_rows_cta - t * kTileRows);
    mbar_expect_tx(bar_base + 8 * slot, nr * rowb);
    for (int r = 0; r < kTileRows; r++) {
      // SwiGLU: slot rows 0..7 are the gate rows of the tile's 8 outputs, rows 8..15 their up rows
      const int vv = swiglu ? 2 * (r & 7) + (r >> 3) : r;
      if (vv < nr) {
        const VRow vr = decode_vrow(p, c0 + t * kTileRows + vv);
        bulk_g2s(slot_base + slot * slot_bytes + r * rstride, vr.row, rowb, bar_base + 8 * slot);
      }
    }
  };
  // ---- before the dependency wait: weights only ----
  if (lane == 0) {
    for (int s = warp; s < n_slots; s += nwarps) mbar_init(bar_base + 8 * s, 1);
  }
  asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
  __syncthreads();
  if (lane == 0) {
    for (int t = warp; t < n_tiles && t < n_slots; t += nwarps) request_tile(t, t);
  }
  bk_stamp(p.trace, 1);
  bk_pdl_wait();
  bk_stamp(p.trace, 2);

  if (p.prologue == BK_PRO_Q8) prologue_q8(p, B, xs, d8s, s8s);
  else if (p.prologue == BK_PRO_BF16) prologue_bf16_batched<false>(p, B, xs, d8s, s8s, red);
  else prologue_bf16_batched<true>(p, B, xs, d8s, s8s, red);
  __syncthreads();
  bk_stamp(p.trace, 3);

  const int R = lane >> 2, j = lane & 3;      // fragment coordinates
  const int tp = warp & 3;                    // sub-block pair of this warp
  const int tq = warp >> 2;                   // tile position inside a round
  const int col0 = 2 * j, col1 = 2 * j + 1;   // C columns of this lane
  // columns beyond the batch read the last real column; their results are never stored
  const int cR = min(R, B - 1), ca = min(col0, B - 1), cb = min(col1, B - 1);
  const uint32_t* xbase = xs + (size_t)cR * p.x_row_words + tp * 16 + j;
  const int ld8 = p.x_scale_ld;
  const float* d8a = d8s + ca * ld8 + 2 * tp;
  const float* s8a = s8s + ca * ld8 + 2 * tp;
  const float* d8b = d8s + cb * ld8 + 2 * tp;
  const float* s8b = s8s + cb * ld8 + 2 * tp;
  const int n_rounds = (n_tiles + tpr - 1) / tpr;

  for (int rd = 0; rd < n_rounds; rd++) {
    const int t = rd * tpr + tq;
    float T[4] = {0.0f, 0.0f, 0.0f, 0.0f};    // (R,col0) (R,col1) (R+8,col0) (R+8,col1)
    if (t < n_tiles) {
      const int slot = t % n_slots;
      const uint32_t parity = (uint32_t)((t / n_slots) & 1);
      mbar_wait_bounded(bar_base + 8 * slot, parity, p.status);
      if (rd == 0) bk_stamp(p.trace, 4);
      const uint8_t* rowA = slots + (size_t)slot * slot_bytes + R * rstride;
      const uint8_t* rowB = rowA + 8 * rstride;
      const uint32_t qoff = 16 + tp * 32 + 4 * j;
      // classes in the order 0,4,2,6,1,5,3,7 so the tree closes with three live partial sums per value
      float stk0[4], stk1[4];
#pragma unroll
      for (int ci = 0; ci < 8; ci++) {
        const int c = ((ci & 1) << 2) | (ci & 2) | ((ci >> 2) & 1);
        float P[4] = {0.0f, 0.0f, 0.0f, 0.0f};
        for (int s = c; s < nsb; s += 8) {
          const uint8_t* sa = rowA + s * 144;
          const uint8_t* sb = rowB + s * 144;
          const uint32_t qa0 = *reinterpret_cast<const uint32_t*>(sa + qoff);
          const uint32_t qa2 = *reinterpret_cast<const uint32_t*>(sa + qoff + 16);
          const uint32_t qb0 = *reinterpret_cast<const uint32_t*>(sb + qoff);
          const uint32_t qb2 = *reinterpret_cast<const uint32_t*>(sb + qoff + 16);
          const uint32_t* xr = xbase + s * 64;
          const uint32_t x00 = xr[0], x01 = xr[4], x10 = xr[8], x11 = xr[12];
          int ilo[4] = {0, 0, 0, 0}, ihi[4] = {0, 0, 0, 0};
          mma_s8(ilo, qa0 & 0x0f0f0f0fu, qb0 & 0x0f0f0f0fu, qa2 & 0x0f0f0f0fu, qb2 & 0x0f0f0f0fu, x00, x01);
          mma_s8(ihi, (qa0 >> 4) & 0x0f0f0f0fu, (qb0 >> 4) & 0x0f0f0f0fu, (qa2 >> 4) & 0x0f0f0f0fu, (qb2 >> 4) & 0x0f0f0f0fu,
                 x10, x11);
          const RowHdr ha = decode_hdr(sa, tp), hb = decode_hdr(sb, tp);
          const float2 da = *reinterpret_cast<const float2*>(d8a + 8 * s);
          const float2 sa8 = *reinterpret_cast<const float2*>(s8a + 8 * s);
          const float2 db = *reinterpret_cast<const float2*>(d8b + 8 * s);
          const float2 sb8 = *reinterpret_cast<const float2*>(s8b + 8 * s);
          P[0] = __fadd_rn(P[0], unit_value(ha, ilo[0], ihi[0], da, sa8));
          P[1] = __fadd_rn(P[1], unit_value(ha, ilo[1], ihi[1], db, sb8));
          P[2] = __fadd_rn(P[2], unit_value(hb, ilo[2], ihi[2], da, sa8));
          P[3] = __fadd_rn(P[3], unit_value(hb, ilo[3], ihi[3], db, sb8));
        }
        // tree: ci 0,1 -> a = P0+P4; ci 2,3 -> b = P2+P6, ab = a+b; ci 4,5 -> a'; ci 6,7 -> b', T = ab + (a'+b')
#pragma unroll
        for (int v = 0; v < 4; v++) {
          if ((ci & 1) == 0) {
            stk1[v] = P[v];
          } else {
            const float pair = __fadd_rn(stk1[v], P[v]);
            if (ci == 1 || ci == 5) {
              stk0[v] = pair;
            } else {
              const float quad = __fadd_rn(stk0[v], pair);
              if (ci == 3) T[v] = quad;
              else T[v] = __fadd_rn(T[v], quad);
            }
          }
        }
      }
    }
    __syncwarp();
    // ring refill: once the four p-warps of a tile are done with a slot the round barrier below releases it
    float* pw = part + (size_t)(rd & 1) * (tpr * 4 * 128) + (size_t)(tq * 4 + tp) * 128;
    pw[R * 8 + col0] = T[0];
    pw[R * 8 + col1] = T[1];
    pw[(R + 8) * 8 + col0] = T[2];
    pw[(R + 8) * 8 + col1] = T[3];
    __syncthreads();   // all partial totals of the round are in shared memory; its weight slots are free
    if (lane == 0 && tp == 0) {
      const int t2 = t + n_slots;
      if (t < n_tiles && t2 < n_tiles) request_tile(t2, t % n_slots);
    }
    // epilogue: thread -> (tile position, row, column)
    {
      const int eq = tid >> 7, er = (tid >> 3) & 15, ec = tid & 7;
      const int et = rd * tpr + eq;
      const float* pr = part + (size_t)(rd & 1) * (tpr * 4 * 128) + (size_t)(eq * 4) * 128 + er * 8 + ec;
      if (et < n_tiles && ec < B) {
        const int nr = min(kTileRows, n_rows_cta - et * kTileRows);
        const float y = __fadd_rn(__fadd_rn(pr[0], pr[2 * 128]), __fadd_rn(pr[1 * 128], pr[3 * 128]));
        if (swiglu) {
          if (er < 8 && 2 * er < nr) {
            const float* pu = pr + 8 * 8;   // the up row of the same output
            const float yup = __fadd_rn(__fadd_rn(pu[0], pu[2 * 128]), __fadd_rn(pu[1 * 128], pu[3 * 128]));
            const VRow vr = decode_vrow(p, c0 + et * kTileRows + 2 * er);
            const SegDev& sg = p.segs[vr.si];
            store_epilogue(sg, (size_t)ec * sg.ld_out + sg.col_off + vr.n, y, yup);
          }
        } else if (er < nr) {
          const VRow vr = decode_vrow(p, c0 + et * kTileRows + er);
          const SegDev& sg = p.segs[vr.si];
          store_epilogue(sg, (size_t)ec * sg.ld_out + sg.col_off + vr.n, y, 0.0f);
        }
      }
    }
  }
  bk_stamp(p.trace, 5);
  bk_stamp_max(p.trace, 6);
}

size_t mma_fixed_smem(int K, int B, int n_slots, int tpr) {
  return (size_t)B * (K / 4 + 4) * 4 + (size_t)B * (K / 32 + 2) * 8 + 288 + (size_t)n_slots * 8 + 16 +
         (size_t)2 * tpr * 4 * 128 * 4 + 128;
}

}  // namespace

// Whether one 16-row tile round plus the staged activation fits an SM's shared memory on this path.
bool bk_gemv_mma_fits(int K, int B) {
  const size_t rowb = (size_t)(K / 256) * 144, tile_bytes = (size_t)kTileRows * (rowb + 16);
  const size_t limit = bk_ctx().smem_optin - 1024;
  return mma_fixed_smem(K, B, 64, 2) + (size_t)2 * tile_bytes <= limit;
}

// Launch shape for the MMA path; `p` arrives with segments, prologue and trace already filled in.
int32_t bk_gemv_mma_launch(void* params, int K, int B, int vrows, bool has_swiglu) {
  GemvParams& p = *static_cast<GemvParams*>(params);
  BkContext& c = bk_ctx();
  const size_t rowb = (size_t)(K / 256) * 144, tile_bytes = (size_t)kTileRows * (rowb + 16);
  const size_t limit = c.smem_optin - 1024;
  const int tiles = (vrows + kTileRows - 1) / kTileRows;
  const int grid = tiles < c.sm_count ? tiles : c.sm_count;
  const int base = tiles / grid, extra = tiles % grid;
  const int tpc = base + (extra ? 1 : 0);         // most tiles any CTA owns
  // tiles per round: as many as fit (4, 2 or 1); slots: the CTA's whole share if it fits (every copy is then
  // requested before the dependency wait), else a ring of whole rounds
  int tpr = kMaxTilesPerRound;
  while (tpr > 2 && mma_fixed_smem(K, B, 64, tpr) + (size_t)tpr * tile_bytes > limit) tpr >>= 1;  // >= 256 threads for the prologue
  BK_ARG(mma_fixed_smem(K, B, 64, tpr) + (size_t)tpr * tile_bytes <= limit,
         "bkGemvQ4K: K=%d with batch %d needs more shared memory than an SM has on the tensor-core path (batch <= 2 has no such limit)", K, B);
  int n_slots = (tpc + tpr - 1) / tpr * tpr;
  if (mma_fixed_smem(K, B, n_slots, tpr) + (size_t)n_slots * tile_bytes > limit) {
    int rounds = (int)((limit - mma_fixed_smem(K, B, 64, tpr)) / ((size_t)tpr * tile_bytes));
    if (rounds > 8) rounds = 8;
    n_slots = rounds * tpr;
  }
  p.tiles_base = base;
  p.tiles_extra = extra;
  (void)has_swiglu;
  p.rows_per_cta = tpc * kTileRows;
  p.n_slots = n_slots;
  p.depth = 0;
  p.group_rows = kTileRows;
  p.x_unit_words = 16;
  p.x_row_words = K / 4 + 4;
  p.x_scale_ld = K / 32 + 2;   // two floats of padding: the four column pairs of a quad land in different banks
  const size_t smem = mma_fixed_smem(K, B, n_slots, tpr) + (size_t)n_slots * tile_bytes;
  static size_t configured = 0;
  if (smem > configured) {
    BK_CUDA(cudaFuncSetAttribute(gemv_q4k_mma_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    configured = smem;
  }
  BK_CUDA(bk_launch_pdl(gemv_q4k_mma_kernel, dim3(grid), dim3(tpr * 128), smem, p, B));
  BK_CHECK_LAUNCH();
  return BK_OK;
}
