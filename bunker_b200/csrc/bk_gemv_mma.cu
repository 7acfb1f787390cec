// bk_gemv_mma.cu -- Q4_K x Q8_1 GEMV for batch 2..8 on the int8 tensor-core path (mma.sync m16n8k32).
//
// At these batch sizes 16 dp4a per 64 weights per batch column no longer fit under the HBM stream; one
// m16n8k32 computes a 32-value sub-block dot for 16 rows and all 8 batch columns, with exact int32 sums,
// so the integer stage stays bit-identical to the scalar one.
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

// A: unsigned bytes (nibbles, or nibbles left in the high half = 16*q), B: signed Q8_1 quants
__device__ __forceinline__ void mma_u8s8(int (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1) {
  asm volatile("mma.sync.aligned.m16n8k32.row.col.s32.u8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
               : "+r"(c[0]), "+r"(c[1]), "+r"(c[2]), "+r"(c[3])
               : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

// Decoded header of one (row, superblock) for the warp's sub-block pair: {d, dmin, sc0, sc1 (int bits)} and {m0, m1}.
// unit value for one (row, column): i0 exact sum of sub-block 2p, i1x16 = 16 * exact sum of sub-block 2p+1 (the high
// nibbles stay in place); sc.y already carries the matching 1/16, so fma(d8_1/16, f32(16*sc1*i1), .) rounds the same
// real number as fma(d8_1, f32(sc1*i1), .).  16*sc1*i1 < 2^26 is a multiple of 16, hence exact in f32.
__device__ __forceinline__ float unit_value(const float4 h, const float2 m, int i0, int i1x16, const float4 sc) {
  float accd = __fmul_rn(sc.x, (float)(__float_as_int(h.z) * i0));
  accd = fmaf(sc.y, (float)(__float_as_int(h.w) * i1x16), accd);
  float accm = __fmul_rn(sc.z, m.x);
  accm = fmaf(sc.w, m.y, accm);
  const float t = __fmul_rn(h.y, accm);
  return fmaf(h.x, accd, -t);
}

constexpr int kChunk = 4;                       // superblocks whose headers a warp decodes at a time
constexpr int kTabBytes = kChunk * 16 * 24;     // per warp: float4 + float2 per (superblock of the chunk, row)

// Shared memory: xs [B][K/4 + 8] words | sc4 [K/64][8] float4 | red[72] | bars[n_slots] | part[2][tiles][4 p][16][8] f32 |
// header tables [warps][kTabBytes] | tile slots [n_slots][16 rows][rowb+16].
// ALIGNED: K is a multiple of 2048 (whole groups of 8 superblocks), so the per-superblock range checks fold away.
// CARRY: a part of a launch cut along K (class accumulators come from / go to a scratch buffer).
template <bool ALIGNED, bool CARRY>
__global__ void __launch_bounds__(kMaxTilesPerRound * 128, 1) gemv_q4k_mma_kernel(const GemvParams p, const int B) {
  bk_pdl_trigger();
  bk_stamp(p.trace, 0);
  extern __shared__ __align__(128) uint8_t smem_raw[];
  const int K = p.K, nsb = K / 256;
  uint32_t* xs = reinterpret_cast<uint32_t*>(smem_raw);
  float* sc4f = reinterpret_cast<float*>(xs + (size_t)B * p.x_row_words);
  float* red = sc4f + (size_t)(K / 64) * 32;
  uint64_t* bars = reinterpret_cast<uint64_t*>(red + 72);   // red: 8 warp sums per batch row + one rstd per row
  const int tpr = blockDim.x >> 7;   // tiles per round (4 or 2): four warps per tile
  const int nwarps = blockDim.x >> 5;
  float* part = reinterpret_cast<float*>((reinterpret_cast<uintptr_t>(bars + p.n_slots + 1) + 15) & ~(uintptr_t)15);
  uint8_t* tabs = reinterpret_cast<uint8_t*>(part + 2 * tpr * 4 * 128);
  uint8_t* slots = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(tabs + (size_t)nwarps * kTabBytes) + 127) & ~(uintptr_t)127);

  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, tid = threadIdx.x;
  // tiles are dealt out evenly: the first tiles_extra CTAs own one tile more than the others
  const int cta = blockIdx.x;
  const int tile0 = cta < p.tiles_extra ? cta * (p.tiles_base + 1) : p.tiles_extra + cta * p.tiles_base;
  const int n_tiles = p.tiles_base + (cta < p.tiles_extra ? 1 : 0);
  const int c0 = tile0 * kTileRows;
  const int n_rows_cta = min(p.total_vrows, c0 + n_tiles * kTileRows) - c0;
  const uint32_t rowb = (uint32_t)nsb * 144, rstride = rowb + 16;
  const uint32_t slot_bytes = kTileRows * rstride;
  const int n_slots = p.n_slots;      // >= tiles of the CTA (pool) or a multiple of tiles-per-round (ring)
  const uint32_t bar_base = smem_u32(bars), slot_base = smem_u32(slots);
  const bool swiglu = p.segs[0].epi == BK_EPI_SWIGLU;

  // one bulk copy per row (padded stride), issued by the first 16 lanes of the calling warp
  auto request_tile = [&](int t, int slot) {
    const int nr = min(kTileRows, n_rows_cta - t * kTileRows);
    if (lane == 0) mbar_expect_tx(bar_base + 8 * slot, nr * rowb);
    __syncwarp();
    if (lane < kTileRows) {
      // SwiGLU: slot rows 0..7 are the gate rows of the tile's 8 outputs, rows 8..15 their up rows
      const int vv = swiglu ? 2 * (lane & 7) + (lane >> 3) : lane;
      if (vv < nr) {
        const VRow vr = decode_vrow(p, c0 + t * kTileRows + vv);
        bulk_g2s(slot_base + slot * slot_bytes + lane * rstride, vr.row, rowb, bar_base + 8 * slot);
      }
    }
  };
  // ---- before the dependency wait: weights only ----
  const uint32_t xbar = bar_base + 8 * n_slots;   // arrival of a staged activation image
  if (lane == 0) {
    for (int s = warp; s < n_slots + 1; s += nwarps) mbar_init(bar_base + 8 * s, 1);
  }
  asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
  __syncthreads();
  for (int t = warp; t < n_tiles && t < n_slots; t += nwarps) request_tile(t, t);
  bk_stamp(p.trace, 1);
  bk_pdl_wait();
  bk_stamp(p.trace, 2);

  if (p.prologue == BK_PRO_STAGED) {
    // the producer wrote exactly the bytes of xs | sc4: one bulk copy, nothing to compute
    if (tid == 0) {
      const uint32_t bytes = (uint32_t)bk_staged_bytes(K, B);
      mbar_expect_tx(xbar, bytes);
      bulk_g2s(smem_u32(xs), p.x, bytes, xbar);
    }
    mbar_wait_bounded(xbar, 0, p.status);
  } else if (p.prologue == BK_PRO_Q8) prologue_q8<true>(p, B, xs, sc4f, nullptr);
  else if (p.prologue == BK_PRO_BF16) prologue_bf16_batched<false>(p, B, xs, sc4f, nullptr, red);
  else prologue_bf16_batched<true>(p, B, xs, sc4f, nullptr, red);
  __syncthreads();
  bk_stamp(p.trace, 3);

  const int R = lane >> 2, j = lane & 3;      // fragment coordinates
  const int tp = warp & 3;                    // sub-block pair of this warp
  const int tq = warp >> 2;                   // tile position inside a round
  const int col0 = 2 * j, col1 = 2 * j + 1;   // C columns of this lane
  // columns beyond the batch read the last real column; their results are never stored
  const int cR = min(R, B - 1), ca = min(col0, B - 1), cb = min(col1, B - 1);
  const uint2* xbase = reinterpret_cast<const uint2*>(xs + (size_t)cR * p.x_row_words + tp * 16) + j;
  const float4* sc4 = reinterpret_cast<const float4*>(sc4f) + tp * 8;
  float4* tabA = reinterpret_cast<float4*>(tabs + (size_t)warp * kTabBytes);
  float2* tabB = reinterpret_cast<float2*>(tabA + kChunk * 16);
  const int n_rounds = (n_tiles + tpr - 1) / tpr;

  for (int rd = 0; rd < n_rounds; rd++) {
    const int t = rd * tpr + tq;
    float T[4] = {0.0f, 0.0f, 0.0f, 0.0f};    // (R,col0) (R,col1) (R+8,col0) (R+8,col1)
    if (t < n_tiles) {
      const int slot = t % n_slots;
      const uint32_t parity = (uint32_t)((t / n_slots) & 1);
      mbar_wait_bounded(bar_base + 8 * slot, parity, p.status);
      if (rd == 0) bk_stamp(p.trace, 4);
      const uint8_t* tile = slots + (size_t)slot * slot_bytes;
      const uint8_t* rowA = tile + R * rstride + 16 + tp * 32 + 4 * j;
      const uint8_t* rowB = rowA + 8 * rstride;
      // class c = s mod 8 collects the unit values of s = c, c+8, ... in ascending order
      float P[8][4];
      // class accumulators of (global tile, pair): 8 x float4 per lane, carried between the K parts of a split launch
      const size_t carry_idx = ((size_t)(tile0 + t) * 4 + tp) * 8 * 32 + lane;
#pragma unroll
      for (int c = 0; c < 8; c++) {
        float4 v4 = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
        if (CARRY && p.carry_in) v4 = __ldcg(reinterpret_cast<const float4*>(p.carry_in) + carry_idx + c * 32);
        P[c][0] = v4.x; P[c][1] = v4.y; P[c][2] = v4.z; P[c][3] = v4.w;
      }
      for (int s0 = 0; s0 < nsb; s0 += 8) {
#pragma unroll
        for (int h = 0; h < 8 / kChunk; h++) {
          const int sbase = s0 + kChunk * h;
          if (ALIGNED || sbase < nsb) {
            __syncwarp();   // the previous chunk's table has been read by every lane
#pragma unroll
            for (int k = 0; k < kChunk * 16 / 32; k++) {
              const int e = lane + 32 * k, row = e & 15, s = sbase + (e >> 4);
              if (ALIGNED || s < nsb) {
                const uint4 hw = *reinterpret_cast<const uint4*>(tile + row * rstride + s * 144);
                uint32_t sc2, mn2;
                bk_q4k_scale_min_pair(hw.y, hw.z, hw.w, tp, sc2, mn2);
                tabA[e] = make_float4(bk_f16_to_f32((uint16_t)(hw.x & 0xffffu)), bk_f16_to_f32((uint16_t)(hw.x >> 16)),
                                      __int_as_float((int)(sc2 & 0xffu)), __int_as_float((int)(sc2 >> 8)));
                tabB[e] = make_float2((float)(int)(mn2 & 0xffu), (float)(int)(mn2 >> 8));
              }
            }
            __syncwarp();
#pragma unroll
            for (int sl = 0; sl < kChunk; sl++) {
              const int s = sbase + sl;
              if (ALIGNED || s < nsb) {
                const uint32_t qa0 = *reinterpret_cast<const uint32_t*>(rowA + s * 144);
                const uint32_t qa2 = *reinterpret_cast<const uint32_t*>(rowA + s * 144 + 16);
                const uint32_t qb0 = *reinterpret_cast<const uint32_t*>(rowB + s * 144);
                const uint32_t qb2 = *reinterpret_cast<const uint32_t*>(rowB + s * 144 + 16);
                const uint2 xlo = xbase[s * 32], xhi = xbase[s * 32 + 4];
                int ilo[4] = {0, 0, 0, 0}, ihi[4] = {0, 0, 0, 0};
                mma_u8s8(ilo, qa0 & 0x0f0f0f0fu, qb0 & 0x0f0f0f0fu, qa2 & 0x0f0f0f0fu, qb2 & 0x0f0f0f0fu, xlo.x, xlo.y);
                mma_u8s8(ihi, qa0 & 0xf0f0f0f0u, qb0 & 0xf0f0f0f0u, qa2 & 0xf0f0f0f0u, qb2 & 0xf0f0f0f0u, xhi.x, xhi.y);
                const float4 ha = tabA[sl * 16 + R], hb = tabA[sl * 16 + R + 8];
                const float2 ma = tabB[sl * 16 + R], mb = tabB[sl * 16 + R + 8];
                const float4 sa = sc4[s * 32 + ca], sb = sc4[s * 32 + cb];
                float* Pc = P[kChunk * h + sl];
                Pc[0] = __fadd_rn(Pc[0], unit_value(ha, ma, ilo[0], ihi[0], sa));
                Pc[1] = __fadd_rn(Pc[1], unit_value(ha, ma, ilo[1], ihi[1], sb));
                Pc[2] = __fadd_rn(Pc[2], unit_value(hb, mb, ilo[2], ihi[2], sa));
                Pc[3] = __fadd_rn(Pc[3], unit_value(hb, mb, ilo[3], ihi[3], sb));
              }
            }
          }
        }
      }
      if (CARRY && p.carry_out) {
#pragma unroll
        for (int c = 0; c < 8; c++)
          reinterpret_cast<float4*>(p.carry_out)[carry_idx + c * 32] = make_float4(P[c][0], P[c][1], P[c][2], P[c][3]);
      }
      // T_p = ((P0+P4)+(P2+P6)) + ((P1+P5)+(P3+P7))
#pragma unroll
      for (int v = 0; v < 4; v++)
        T[v] = __fadd_rn(__fadd_rn(__fadd_rn(P[0][v], P[4][v]), __fadd_rn(P[2][v], P[6][v])),
                         __fadd_rn(__fadd_rn(P[1][v], P[5][v]), __fadd_rn(P[3][v], P[7][v])));
    }
    // The four p-warps of a tile position form a group with its own named barrier: groups drift apart freely,
    // so one group's barrier, epilogue and refill overlap the other groups' dot products.
    if (t < n_tiles) {   // uniform within the group
      float* pw = part + (size_t)(rd & 1) * (tpr * 4 * 128) + (size_t)(tq * 4 + tp) * 128;
      pw[R * 8 + col0] = T[0];
      pw[R * 8 + col1] = T[1];
      pw[(R + 8) * 8 + col0] = T[2];
      pw[(R + 8) * 8 + col1] = T[3];
      asm volatile("bar.sync %0, 128;" ::"r"(1 + tq) : "memory");   // the tile's partial totals are in shared memory; its slot is free
      if (tp == 0) {
        const int t2 = t + n_slots;
        if (t2 < n_tiles) request_tile(t2, t % n_slots);
      }
      // epilogue: the group's 128 threads -> (row, column) of the tile.  The other half of `part` is written in the
      // next round only after every warp of the group has passed that round's barrier, i.e. finished reading here.
      const int g = tid & 127, er = g >> 3, ec = g & 7;
      const float* pr = part + (size_t)(rd & 1) * (tpr * 4 * 128) + (size_t)(tq * 4) * 128 + er * 8 + ec;
      if (ec < B && !(CARRY && p.carry_out)) {
        const int nr = min(kTileRows, n_rows_cta - t * kTileRows);
        const float y = __fadd_rn(__fadd_rn(pr[0], pr[2 * 128]), __fadd_rn(pr[1 * 128], pr[3 * 128]));
        if (swiglu) {
          if (er < 8 && 2 * er < nr) {
            const float* pu = pr + 8 * 8;   // the up row of the same output
            const float yup = __fadd_rn(__fadd_rn(pu[0], pu[2 * 128]), __fadd_rn(pu[1 * 128], pu[3 * 128]));
            const VRow vr = decode_vrow(p, c0 + t * kTileRows + 2 * er);
            const SegDev& sg = p.segs[vr.si];
            store_epilogue(p, sg, (size_t)ec * sg.ld_out + sg.col_off + vr.n, y, yup);
          }
        } else if (er < nr) {
          const VRow vr = decode_vrow(p, c0 + t * kTileRows + er);
          const SegDev& sg = p.segs[vr.si];
          store_epilogue(p, sg, (size_t)ec * sg.ld_out + sg.col_off + vr.n, y, 0.0f);
        }
      }
    }
  }
  bk_stamp(p.trace, 5);
  bk_stamp_max(p.trace, 6);
}

size_t mma_fixed_smem(int K, int B, int n_slots, int tpr) {
  return (size_t)B * (K / 4 + 8) * 4 + (size_t)(K / 64) * 8 * 16 + 288 + (size_t)(n_slots + 1) * 8 + 16 +
         (size_t)2 * tpr * 4 * 128 * 4 + (size_t)tpr * 4 * kTabBytes + 128;
}

}  // namespace

// Whether one 16-row tile round plus the staged activation fits an SM's shared memory on this path.
bool bk_gemv_mma_fits(int K, int B) {
  const size_t rowb = (size_t)(K / 256) * 144, tile_bytes = (size_t)kTileRows * (rowb + 16);
  const size_t limit = bk_ctx().smem_optin - 1024;
  return mma_fixed_smem(K, B, 64, 2) + (size_t)2 * tile_bytes <= limit;
}

// Launch shape for the MMA path; `p` arrives with segments, prologue and trace already filled in.
int32_t bk_gemv_mma_launch(void* params, int K, int B, int vrows, bool has_swiglu, int* ctas_out) {
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
  if (ctas_out) *ctas_out = grid;
  p.tiles_base = base;
  p.tiles_extra = extra;
  (void)has_swiglu;
  p.rows_per_cta = tpc * kTileRows;
  p.n_slots = n_slots;
  p.depth = 0;
  p.group_rows = kTileRows;
  p.x_unit_words = 16;
  p.x_row_words = K / 4 + 8;   // 8 words of padding: the 64-bit loads of a half-warp (4 columns x 4 j) tile the 32 banks
  p.x_scale_ld = 0;            // scales live in the float4 layout of the tensor-core path
  const size_t smem = mma_fixed_smem(K, B, n_slots, tpr) + (size_t)n_slots * tile_bytes;
  static size_t configured[4] = {0, 0, 0, 0};
  const bool aligned = (K / 256) % 8 == 0;
  const bool carry = p.carry_in != nullptr || p.carry_out != nullptr;
  auto kernel = carry ? (aligned ? gemv_q4k_mma_kernel<true, true> : gemv_q4k_mma_kernel<false, true>)
                      : (aligned ? gemv_q4k_mma_kernel<true, false> : gemv_q4k_mma_kernel<false, false>);
  const int ki = (carry ? 2 : 0) + (aligned ? 1 : 0);
  if (smem > configured[ki]) {
    BK_CUDA(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    configured[ki] = smem;
  }
  BK_CUDA(bk_launch_pdl(kernel, dim3(grid), dim3(tpr * 128), smem, p, B));
  BK_CHECK_LAUNCH();
  return BK_OK;
}
