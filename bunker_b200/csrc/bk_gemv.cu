// bk_gemv.cu -- Q4_K x Q8_1 dequant-GEMV: the batch-1 kernel (also batch 2 when K is too wide for the tensor-core
// kernel of bk_gemv_mma.cu) and the host-side launch logic of both kernels.
//
// Replaces the bf16 tt.dot GEMMs of bunker's decode loop (buildMM / buildGateSwiglu,
// prototypes/decode.ts:101-186; emitGemm, src/fusion.ts:276-293) with integer block
// dots on 4-bit weights.
//
// Work split.  A weight row of K columns is K/64 "units": one 32-byte quant group
// (sub-blocks 2p, 2p+1 of superblock s; u = 4s+p).  A warp owns whole rows; lane l
// owns the units u = l (mod 32).  All loads are 128-bit: per unit two for the quants
// and one for the 16-byte superblock header (shared by the 4 lanes of a superblock,
// one transaction).  A warp therefore reads a row as one contiguous, fully used span.
//
// Arithmetic per unit and batch column: 16 dp4a (nibbles x int8) -> two exact int32
// sub-block sums; then the fixed f32 form
//     accd = fma(d8_b, f32(sc_b*isum_b), accd), accm = fma(s8_b, f32(m_b), accm)
//     val  = fma(d, accd, -(dmin*accm));  lane_sum += val   (ascending u)
// and the xor-butterfly over the 32 lanes.  The order is fixed so a host can
// reproduce the result bit for bit.
//
// Weight staging.  One CTA per SM owning a contiguous range of rows, handled in groups of G rows per warp.
// Every group has a slot in shared memory (all groups at once when the CTA's rows fit, else a per-warp ring)
// that lane 0 fills with one bulk async copy per contiguous run of rows (cp.async.bulk, completion on an
// mbarrier).  The first copies are issued before the programmatic-dependency wait, so the weight stream of
// this launch is in flight while the previous kernel drains and while the activation prologue runs; the
// dot products then read weights from shared memory.  High nibbles stay in place (16*q as unsigned bytes);
// the staged scale of odd blocks carries the 1/16.
//
// The activation lives in shared memory for the whole CTA: int8 quants padded to
// 80 bytes per 64 (conflict-free 128-bit reads at lane stride), plus per-block
// d8 and s8 = d8*sum(q8) (exact in f32).  Three prologues fill it: ready-made
// Q8_1 blocks, bf16 rows quantised in place, or bf16 rows through RMSNorm first.
#include "bk_gemv_shared.cuh"
#include "bk_gemv_dp4a.cuh"

namespace {

// ---- main kernel -------------------------------------------------------------

// One CTA per SM owns the contiguous virtual rows [c*rows_per_cta, ...).  Rows are processed in
// groups of G by one warp (group g of the CTA belongs to warp g mod nw).  Each group has a slot of
// G rows in shared memory and an mbarrier.  depth == 0 ("pool"): every group has its own slot and all
// copies are issued before the dependency wait.  depth > 0 ("ring"): a warp owns `depth` slots and
// refills a slot with its next group as soon as the slot is consumed.
// TP: the build with the tensor-parallel reduce prologue and push epilogue (kept out of the single-GPU build, whose
// register allocation they would disturb).
template <int B, int GMAX, bool TP>
__global__ void __maxnreg__(64) gemv_q4k_kernel(const GemvParams p) {
  static_assert(B <= 2, "batch >= 3 runs on the tensor-core kernel (bk_gemv_mma.cu) or as column pairs of this one");
  bk_pdl_trigger();
  bk_stamp(p.trace, 0);
  unsigned long long* ctr = p.cta_trace ? p.cta_trace + 4 * blockIdx.x : nullptr;
  if (ctr && threadIdx.x == 0) { unsigned int sm_; asm volatile("mov.u32 %0, %%smid;" : "=r"(sm_)); ctr[0] = sm_; ctr[3] = 0; }
  extern __shared__ __align__(128) uint8_t smem_raw[];
  const int K = p.K, nunits = K / 64, nblk = K / 32;
  const int nw = blockDim.x >> 5;
  uint32_t* xs = reinterpret_cast<uint32_t*>(smem_raw);
  float* d8s = reinterpret_cast<float*>(xs + (size_t)B * nunits * kUnitWords);
  float* s8s = d8s + (size_t)B * nblk;
  float* red = s8s + (size_t)B * nblk;
  uint64_t* bars = reinterpret_cast<uint64_t*>(red + 8);
  uint8_t* slots = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(bars + p.n_slots) + 127) & ~(uintptr_t)127);

  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int c0 = blockIdx.x * p.rows_per_cta;
  const int n_rows_cta = min(p.total_vrows, c0 + p.rows_per_cta) - c0;
  const int G = p.group_rows;  // rows per group, 1..GMAX
  const int n_groups = (n_rows_cta + G - 1) / G;
  const uint32_t rowb = (uint32_t)(K / 256) * 144;
  const uint32_t slot_bytes = G * rowb;
  const int depth = p.depth;
  const uint32_t bar_base = smem_u32(bars);
  const uint32_t slot_base = smem_u32(slots);

  // ---- before the dependency wait: weights only ----
  if (lane == 0) {
    int first = depth == 0 ? (n_groups - warp + nw - 1) / nw : depth;  // groups to request now
    for (int gi = 0; gi < first; gi++) {
      const int g = warp + gi * nw;
      const int slot = depth == 0 ? g : gi * nw + warp;
      mbar_init(bar_base + 8 * slot, 1);
    }
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    for (int gi = 0; gi < first; gi++) {
      const int g = warp + gi * nw;
      if (g >= n_groups) break;
      const int slot = depth == 0 ? g : gi * nw + warp;
      const int nr = min(G, n_rows_cta - g * G);
      request_group(p, c0 + g * G, nr, rowb, slot_base + slot * slot_bytes, bar_base + 8 * slot);
    }
  }
  uint4 wpre = make_uint4(0, 0, 0, 0);  // norm weights are weights: fetched before the wait as well
  if ((p.prologue == BK_PRO_RMSNORM || p.prologue == BK_PRO_REDUCE_RMSNORM) && (int)threadIdx.x < K / 8)
    wpre = __ldg(reinterpret_cast<const uint4*>(p.norm_w) + threadIdx.x);
  __syncwarp();
  bk_stamp(p.trace, 1);
  // A reducing launch depends on its predecessor (the pushing GEMV) only through the tagged exchange words, which it
  // polls; it does not wait for that grid to complete, because completion includes the acknowledgement of the
  // predecessor's remote stores -- an NVLink round trip.  Everything older is complete: the predecessor passed its own
  // dependency wait before it pushed anything.  Nothing is written here before every tag of the row has been seen,
  // i.e. before every CTA of the predecessor has finished reading its inputs.
  if (!(TP && p.prologue == BK_PRO_REDUCE_RMSNORM)) bk_pdl_wait();
  bk_stamp(p.trace, 2);
  if (ctr && threadIdx.x == 0) { unsigned long long t_; asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t_)); ctr[1] = t_; }

  if (p.prologue == BK_PRO_Q8)
    prologue_q8<false>(p, B, xs, d8s, s8s);
  else if (p.prologue == BK_PRO_BF16)
    prologue_bf16<false>(p, B, xs, d8s, s8s, red, wpre);
  else if (p.prologue == BK_PRO_RMSNORM)
    prologue_bf16<true>(p, B, xs, d8s, s8s, red, wpre);
  else if constexpr (TP) {
    // Tensor-parallel input.  CTA 0 gathers the ranks' partial sums (tagged words, polled), adds the residual and
    // writes the bf16 row; it then publishes the exchange tag in a local word.  The other CTAs wait for that word
    // and read the 4 KB row from L2 -- 148 CTAs polling the tagged words themselves would flood L2.
    const unsigned int tag = bk_exchange_tag(p.red.epoch, p.red.tag_add);
    if (blockIdx.x == 0) {
      prologue_bf16<true, 1>(p, B, xs, d8s, s8s, red, wpre);
      __syncthreads();
      if (threadIdx.x == 0) {
        __threadfence();
        asm volatile("st.release.gpu.global.u32 [%0], %1;" ::"l"(p.red.ready), "r"(tag) : "memory");
      }
    } else {
      if (threadIdx.x == 0) {
        unsigned int v;
        for (int it = 0;; it++) {
          asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p.red.ready) : "memory");
          if (v == tag) break;
          if (it > (1 << 22)) {
            if (p.status) atomicExch(p.status, BK_ERR_TIMEOUT);
            break;
          }
        }
      }
      __syncthreads();
      prologue_bf16<true, 2>(p, B, xs, d8s, s8s, red, wpre);
    }
  }
  __syncthreads();
  bk_stamp(p.trace, 3);
  bk_stamp_max(p.trace, 1);  // (reuses slot 1) latest prologue end over all CTAs

  const int ri = ((lane >> 4) & 1) * 4 + ((lane >> 3) & 1) * 2 + ((lane >> 2) & 1);  // row this lane reports
  const bool swiglu = p.segs[0].epi == BK_EPI_SWIGLU;  // such a segment is always alone in its launch
  for (int gi = 0, g = warp; g < n_groups; gi++, g += nw) {
    const int slot = depth == 0 ? g : (gi % depth) * nw + warp;
    const uint32_t parity = depth == 0 ? 0u : (uint32_t)((gi / depth) & 1);
    const int nr = min(G, n_rows_cta - g * G);
    mbar_wait_bounded(bar_base + 8 * slot, parity, p.status);
    if (gi == 0) {
      bk_stamp(p.trace, 4);
      bk_stamp_max(p.trace, 7);  // latest "first weights landed" over all warps
      if (ctr && threadIdx.x == 0) { unsigned long long t_; asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t_)); ctr[2] = t_; }
    }
    const uint8_t* wbase = slots + slot * slot_bytes;
    float acc[GMAX][B];
#pragma unroll
    for (int r = 0; r < GMAX; r++)
#pragma unroll
      for (int b = 0; b < B; b++) acc[r][b] = 0.0f;
    for (int u = lane; u < nunits; u += 32) {
      const int pp = u & 3;
      // one or two columns: the activation of this unit stays in registers across the G rows
      XRegs xr[B];
#pragma unroll
      for (int b = 0; b < B; b++) xr[b] = load_x(xs, d8s, s8s, b, u, nunits, nblk);
#pragma unroll
      for (int r = 0; r < GMAX; r++) {
        if (r < nr) {
          const WRegs w = decode_unit(load_unit_smem(wbase + slot_row(swiglu, r, nr) * rowb, u), pp);
#pragma unroll
          for (int b = 0; b < B; b++) acc[r][b] = __fadd_rn(acc[r][b], unit_val(w, xr[b]));
        }
      }
    }
    __syncwarp();  // every lane has consumed the slot
    if (depth > 0 && lane == 0) {
      const int g2 = g + depth * nw;
      if (g2 < n_groups) {
        const int nr2 = min(G, n_rows_cta - g2 * G);
        request_group(p, c0 + g2 * G, nr2, rowb, slot_base + slot * slot_bytes, bar_base + 8 * slot);
      }
    }
    // reduce over lanes; lane (lane&3)==0 ends up with the sum of row ri of the group
    const int v = c0 + g * G + ri;
    const bool mine = (lane & 3) == 0 && ri < nr;
    VRow vr = {nullptr, 0, 0};
    if (mine) vr = decode_vrow(p, v);
    const SegDev& sg = p.segs[vr.si];
#pragma unroll
    for (int b = 0; b < B; b++) {
      float pa[8];
#pragma unroll
      for (int r = 0; r < 8; r++) pa[r] = r < GMAX ? acc[r < GMAX ? r : 0][b] : 0.0f;
      const float y = warp_sum8(pa);
      const float yup = __shfl_xor_sync(0xffffffffu, y, 4);  // the odd neighbour row (the "up" row of a SwiGLU pair)
      if (mine && !(sg.epi == BK_EPI_SWIGLU && (ri & 1))) store_epilogue<TP>(p, sg, (size_t)b * sg.ld_out + sg.col_off + vr.n, y, yup);
    }
  }
  bk_stamp(p.trace, 5);
  bk_stamp_max(p.trace, 6);  // latest exit over all warps of all CTAs
  if (ctr) bk_stamp_max(ctr, 3);
}

// bytes of shared memory before the weight slots: activation, scales, reduction scratch, barriers (+ alignment slack)
size_t gemv_fixed_smem(int K, int B, int n_slots) {
  size_t nunits = K / 64, nblk = K / 32;
  return (size_t)B * nunits * kUnitWords * 4 + (size_t)B * nblk * 8 + 8 * 4 + (size_t)n_slots * 8 + 128;
}

template <int B, int GMAX, bool TP>
int32_t launch_gemv(const GemvParams& p, int grid, int threads, size_t smem) {
  static size_t configured = 0;
  if (smem > configured) {
    BK_CUDA((cudaFuncSetAttribute(gemv_q4k_kernel<B, GMAX, TP>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem)));
    configured = smem;
  }
  BK_CUDA((bk_launch_pdl(gemv_q4k_kernel<B, GMAX, TP>, dim3(grid), dim3(threads), smem, p)));
  BK_CHECK_LAUNCH();
  return BK_OK;
}

// widest row group the register budget of batch B allows
constexpr int gemv_gmax(int) { return 8; }

// ---- dequant / block-dot check kernels ---------------------------------------

// One thread per (row, unit): writes 64 f32 weights, dl = d*sc, ml = dmin*m, w = dl*q - ml
__global__ void dequant_q4k_kernel(const uint8_t* W, int N, int K, float* out) {
  const int nunits = K / 64;
  size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= (size_t)N * nunits) return;
  int n = (int)(idx / nunits), u = (int)(idx - (size_t)n * nunits);
  const uint8_t* row = W + (size_t)n * (K / 256) * 144;
  RowRegs r = load_unit(row, u);
  int p = u & 3;
  float d = bk_f16_to_f32((uint16_t)(r.hdr.x & 0xffffu));
  float dmin = bk_f16_to_f32((uint16_t)(r.hdr.x >> 16));
  int sc0, mn0, sc1, mn1;
  bk_q4k_scale_min(r.hdr.y, r.hdr.z, r.hdr.w, 2 * p, sc0, mn0);
  bk_q4k_scale_min(r.hdr.y, r.hdr.z, r.hdr.w, 2 * p + 1, sc1, mn1);
  float dl0 = __fmul_rn(d, (float)sc0), ml0 = __fmul_rn(dmin, (float)mn0);
  float dl1 = __fmul_rn(d, (float)sc1), ml1 = __fmul_rn(dmin, (float)mn1);
  const uint32_t qw[8] = {r.qa.x, r.qa.y, r.qa.z, r.qa.w, r.qb.x, r.qb.y, r.qb.z, r.qb.w};
  float* o = out + (size_t)n * K + (size_t)u * 64;
#pragma unroll
  for (int k = 0; k < 8; k++)
#pragma unroll
    for (int e = 0; e < 4; e++) {
      uint32_t byte = (qw[k] >> (8 * e)) & 0xffu;
      o[k * 4 + e] = __fsub_rn(__fmul_rn(dl0, (float)(byte & 15u)), ml0);
      o[32 + k * 4 + e] = __fsub_rn(__fmul_rn(dl1, (float)(byte >> 4)), ml1);
    }
}

// One thread per (row, unit): the two int32 sub-block sums and the q8 sums
__global__ void block_dots_kernel(const uint8_t* W, int N, int K, const uint32_t* xq, int32_t* isum, int32_t* qsum) {
  const int nunits = K / 64, nblk = K / 32;
  size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= (size_t)N * nunits) return;
  int n = (int)(idx / nunits), u = (int)(idx - (size_t)n * nunits);
  const uint8_t* row = W + (size_t)n * (K / 256) * 144;
  RowRegs r = load_unit(row, u);
  const uint32_t qw[8] = {r.qa.x, r.qa.y, r.qa.z, r.qa.w, r.qb.x, r.qb.y, r.qb.z, r.qb.w};
  const uint32_t* x0 = xq + (size_t)(2 * u) * 9;
  const uint32_t* x1 = xq + (size_t)(2 * u + 1) * 9;
  int i0 = 0, i1 = 0, s0 = 0, s1 = 0;
#pragma unroll
  for (int k = 0; k < 8; k++) {
    i0 = bk_dp4a(qw[k] & 0x0f0f0f0fu, x0[k], i0);
    i1 = bk_dp4a((qw[k] >> 4) & 0x0f0f0f0fu, x1[k], i1);
    s0 = bk_dp4a_ss(x0[k], 0x01010101u, s0);
    s1 = bk_dp4a_ss(x1[k], 0x01010101u, s1);
  }
  isum[(size_t)n * nblk + 2 * u] = i0;
  isum[(size_t)n * nblk + 2 * u + 1] = i1;
  qsum[(size_t)n * nblk + 2 * u] = s0;
  qsum[(size_t)n * nblk + 2 * u + 1] = s1;
}

// packQ8_1 on the device: one aligned group of 4 lanes per 32-element block
template <bool BF16>
__global__ void quant_q8_1_kernel(const void* x, int K, int B, uint8_t* out) {
  const int nchunk = K / 8;
  size_t gid = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  bool active = gid < (size_t)B * nchunk;
  size_t g = active ? gid : 0;
  int b = (int)(g / nchunk), q = (int)(g - (size_t)b * nchunk);
  float y[8];
  if (BF16) {
    load_chunk_bf16(reinterpret_cast<const uint16_t*>(x) + (size_t)b * K, q, y);
  } else {
    const float4* s = reinterpret_cast<const float4*>(reinterpret_cast<const float*>(x) + (size_t)b * K + (size_t)q * 8);
    float4 a = s[0], c = s[1];
    y[0] = a.x; y[1] = a.y; y[2] = a.z; y[3] = a.w;
    y[4] = c.x; y[5] = c.y; y[6] = c.z; y[7] = c.w;
  }
  float amax = 0.0f;
#pragma unroll
  for (int e = 0; e < 8; e++) amax = fmaxf(amax, fabsf(y[e]));
  amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 1));
  amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 2));
  float d = __fdiv_rn(amax, 127.0f);
  float id = (d == 0.0f) ? 1.0f : __fdiv_rn(1.0f, d);
  int sum = 0;
  uint32_t w[2] = {0, 0};
#pragma unroll
  for (int e = 0; e < 8; e++) {
    int v = __float2int_rd(fmaf(y[e], id, 0.5f));
    sum += v;  // the reference sums before clamping (bench/bench.ts:66-67)
    v = max(-128, min(127, v));
    w[e >> 2] |= (uint32_t)(v & 0xff) << (8 * (e & 3));
  }
  sum += __shfl_xor_sync(0xffffffffu, sum, 1);
  sum += __shfl_xor_sync(0xffffffffu, sum, 2);
  if (!active) return;
  int blk = q >> 2;
  uint32_t* ob = reinterpret_cast<uint32_t*>(out + ((size_t)b * (K / 32) + blk) * 36);
  ob[(q & 3) * 2] = w[0];
  ob[(q & 3) * 2 + 1] = w[1];
  if ((q & 3) == 0) {
    uint32_t hd = bk_f32_to_f16_trunc(d);
    uint32_t hs = bk_f32_to_f16_trunc(__fmul_rn((float)sum, d));
    ob[8] = hd | (hs << 16);
  }
}

}  // namespace

// ---- host entry points ---------------------------------------------------------

int32_t bk_gemv_mma_launch(void* params, int K, int B, int vrows, bool has_swiglu, int* ctas_out);  // bk_gemv_mma.cu
int32_t bk_gemv_umma_launch(void* params, int B);                                                   // bk_gemv_umma.cu
static bool g_umma_group = false;   // the launch being set up is one group of <= 32 columns of the dense tile path
// BK_GEMV_ORDER_AUTO takes the tile path from g_tile_min_rows launch rows on, and from g_tile_min_rows_cut rows on when K is
// at least 2048 (such a launch has few 128-row tiles and is cut along K over several thread blocks); bkTuneTileMinRows
static int g_tile_min_rows = 4096, g_tile_min_rows_cut = 1024;

static int g_tune_warps = 0, g_tune_rows = 0, g_tune_depth = 0;

// K view of the launch being set up by the split-K driver below (null otherwise)
struct KView {
  unsigned int row_stride, row_off;
  int xq_ld, xq_off;
  const float* carry_in;
  float* carry_out;
};
static const KView* g_view = nullptr;

int32_t bk_gemv_launch(const bkGemvArgs& a) { return bk_gemv_launch_tp(a, nullptr, nullptr, nullptr); }

int32_t bk_gemv_launch_tp(const bkGemvArgs& a, const BkPush* push, const BkReduce* reduce, int* ctas_out) {
  BkContext& c = bk_ctx();
  BK_ARG(a.K > 0 && a.K % 256 == 0, "bkGemvQ4K: K=%d is not a positive multiple of 256", a.K);
  BK_ARG(a.B >= 1 && a.B <= 64, "bkGemvQ4K: B=%d outside 1..64", a.B);
  // From 16 columns on, ready-made Q8_1 blocks go to the dense tile kernel (tcgen05 int8 MMA, bk_gemv_umma.cu): the
  // weights are streamed once per 32 columns.  Its f32 order differs from the batch <= 8 kernels' (see there);
  // order = BK_GEMV_ORDER_LANES keeps the columns on those kernels.
  // A launch of very few rows (or few rows and a short K) has too few 128-row tiles to fill the machine and its
  // weights stay in L2 between groups of 8 columns anyway, so AUTO sends it to the batch <= 8 kernels; the rule
  // depends on the shapes only.
  int launch_rows = 0;
  for (int i = 0; i < a.n_segs && i < 4; i++) launch_rows += a.segs[i].n_rows * (a.segs[i].epilogue == BK_EPI_SWIGLU ? 2 : 1);
  const bool tile_path = !g_umma_group && a.B >= 16 && a.prologue == BK_PRO_Q8 && !push && !reduce && !g_view &&
                         (a.order == BK_GEMV_ORDER_TILE || (a.order == BK_GEMV_ORDER_AUTO && bk_gemv_auto_tile(launch_rows, a.K)));
  if (a.B > 8 && !g_umma_group) {
    // More than 8 columns without the tile path: groups of 8 on the mma.sync kernel, one launch per group (the weights
    // of the later groups come from L2 when they fit there).
    BK_ARG(a.prologue != BK_PRO_REDUCE_RMSNORM, "bkGemvQ4K: the reduce prologue is a batch-1 path");
    if (ctas_out) *ctas_out = 0;
    const int gsz = tile_path ? 32 : 8;
    for (int b0 = 0; b0 < a.B; b0 += gsz) {
      bkGemvArgs s = a;
      s.B = a.B - b0 < gsz ? a.B - b0 : gsz;
      if (a.prologue == BK_PRO_STAGED) s.x = a.x + (uint64_t)(b0 / 8) * bk_staged_group_stride(a.K);
      else s.x = a.x + (uint64_t)b0 * (a.prologue == BK_PRO_Q8 ? (uint64_t)(a.K / 32) * 36 : (uint64_t)a.K * 2);
      if (s.B == 1 && a.prologue == BK_PRO_STAGED && !tile_path) return bk_fail(BK_ERR_ARG, "bkGemvQ4K: a staged activation cannot end in a group of one column (B=%d)", a.B);
      BkPush ps;
      if (push) {
        ps = *push;
        for (int r = 0; r < ps.n; r++) ps.dst[r] += (size_t)b0 * a.segs[0].ld_out;
      }
      for (int i = 0; i < a.n_segs && i < 4; i++) {
        const uint64_t esz = a.segs[i].epilogue == BK_EPI_F32 ? 4 : 2;
        if (a.segs[i].out) s.segs[i].out = a.segs[i].out + (uint64_t)b0 * a.segs[i].ld_out * esz;
        if (a.segs[i].residual) s.segs[i].residual = a.segs[i].residual + (uint64_t)b0 * a.segs[i].ld_out * 2;
      }
      int ctas = 0;
      g_umma_group = tile_path;
      const int32_t rc = bk_gemv_launch_tp(s, push ? &ps : nullptr, nullptr, &ctas);
      g_umma_group = false;
      if (rc != BK_OK) return rc;
      if (ctas_out) *ctas_out += ctas;
    }
    return BK_OK;
  }
  BK_ARG(a.n_segs >= 1 && a.n_segs <= 4, "bkGemvQ4K: n_segs=%d outside 1..4", a.n_segs);
  BK_ARG((a.prologue >= BK_PRO_Q8 && a.prologue <= BK_PRO_STAGED) || (a.prologue == BK_PRO_REDUCE_RMSNORM && reduce && reduce->n > 0),
         "bkGemvQ4K: unknown prologue %d", a.prologue);
  const bool tc_path = !g_umma_group && a.B >= 2 && bk_gemv_mma_fits(a.K, a.B);
  BK_ARG(a.prologue != BK_PRO_REDUCE_RMSNORM || !tc_path, "bkGemvQ4K: the reduce prologue exists on the batch-1 kernel only");
  if (a.prologue == BK_PRO_STAGED)
    BK_ARG(a.B >= 2 && bk_gemv_mma_fits(a.K, a.B),
           "bkGemvQ4K: a staged activation needs batch 2..8 and a K that fits the tensor-core path (K=%d B=%d)", a.K, a.B);
  BK_ARG(a.x != 0 && (a.x & 15) == 0, "bkGemvQ4K: x must be a non-null 16-byte aligned device pointer");
  if (a.prologue == BK_PRO_RMSNORM || a.prologue == BK_PRO_REDUCE_RMSNORM)
    BK_ARG(a.norm_w != 0 && (a.norm_w & 15) == 0, "bkGemvQ4K: norm_w must be non-null and 16-byte aligned");
  if (!g_umma_group && a.B >= 2 && !g_view && a.prologue == BK_PRO_Q8 && !bk_gemv_mma_fits(a.K, a.B)) {
    // Rows too wide for the tensor-core path's shared memory (FFN 17408 of the 64-layer configuration): the launch is
    // cut along K into parts of whole 8-superblock groups.  The canonical order adds a row's unit values per class
    // (superblock mod 8) in ascending order, so a part starts from the class accumulators its predecessor left in a
    // scratch buffer and only the last part closes the tree and runs the epilogue: same bits as one launch.
    int psb = 0;
    for (int cand = 32; cand >= 8; cand -= 8)
      if (bk_gemv_mma_fits(cand * 256, a.B)) { psb = cand; break; }
    if (psb) {
      const int nsb = a.K / 256, nparts = (nsb + psb - 1) / psb;
      int per = ((nsb + nparts - 1) / nparts + 7) & ~7;   // even parts, whole groups of 8
      int vr = 0;
      for (int i = 0; i < a.n_segs && i < 4; i++) vr += a.segs[i].epilogue == BK_EPI_SWIGLU ? 2 * a.segs[i].n_rows : a.segs[i].n_rows;
      const size_t need = (size_t)((vr + 15) / 16) * 16384;
      if (c.gemv_carry_bytes < need) {
        if (c.capturing) return bk_fail(BK_ERR_STATE, "bkGemvQ4K: the split-K scratch must be sized by an eager launch before a capture");
        if (c.gemv_carry) cudaFree(c.gemv_carry);
        c.gemv_carry = nullptr;
        c.gemv_carry_bytes = 0;
        void* q = nullptr;
        BK_CUDA(cudaMalloc(&q, need));
        c.gemv_carry = static_cast<float*>(q);
        c.gemv_carry_bytes = need;
      }
      for (int s0 = 0, i = 0; s0 < nsb; s0 += per, i++) {
        const int s1 = s0 + per < nsb ? s0 + per : nsb;
        const bool last = s1 == nsb;
        bkGemvArgs s = a;
        s.K = (s1 - s0) * 256;
        const KView v = {(unsigned int)(nsb * 144), (unsigned int)(s0 * 144), a.K / 32, s0 * 8, i ? c.gemv_carry : nullptr,
                         last ? nullptr : c.gemv_carry};
        g_view = &v;
        const int32_t rc = bk_gemv_launch_tp(s, push, nullptr, last ? ctas_out : nullptr);
        g_view = nullptr;
        if (rc != BK_OK) return rc;
      }
      return BK_OK;
    }
  }
  if (!g_umma_group && a.B >= 3 && !g_view && !bk_gemv_mma_fits(a.K, a.B)) {
    // A K this wide (FFN 17408 of the 64-layer configuration) leaves no room for a 16-row tile beside the staged
    // activation of 3..8 columns.  The columns are independent, so the launch is cut into column pairs on the
    // small-batch kernel (same arithmetic, same bits); the weights of the later pairs come mostly from L2.
    if (ctas_out) *ctas_out = 0;
    for (int b0 = 0; b0 < a.B; b0 += 2) {
      bkGemvArgs s = a;
      BkPush ps;
      if (push) {
        ps = *push;
        for (int r = 0; r < ps.n; r++) ps.dst[r] += (size_t)b0 * a.segs[0].ld_out;
      }
      s.B = a.B - b0 < 2 ? a.B - b0 : 2;
      s.x = a.x + (uint64_t)b0 * (a.prologue == BK_PRO_Q8 ? (uint64_t)(a.K / 32) * 36 : (uint64_t)a.K * 2);
      for (int i = 0; i < a.n_segs && i < 4; i++) {
        const uint64_t esz = a.segs[i].epilogue == BK_EPI_F32 ? 4 : 2;
        s.segs[i].out = a.segs[i].out + (uint64_t)b0 * a.segs[i].ld_out * esz;
        if (a.segs[i].residual) s.segs[i].residual = a.segs[i].residual + (uint64_t)b0 * a.segs[i].ld_out * 2;
      }
      int ctas = 0;
      int32_t rc = bk_gemv_launch_tp(s, push ? &ps : nullptr, reduce, &ctas);
      if (rc != BK_OK) return rc;
      if (ctas_out) *ctas_out += ctas;
    }
    return BK_OK;
  }
  GemvParams p;
  p.K = a.K;
  p.n_segs = a.n_segs;
  p.prologue = a.prologue;
  p.x = bk_ptr<void>(a.x);
  p.row_stride = g_view ? g_view->row_stride : 0;
  p.row_off = g_view ? g_view->row_off : 0;
  p.xq_ld = g_view ? g_view->xq_ld : 0;
  p.xq_off = g_view ? g_view->xq_off : 0;
  p.carry_in = g_view ? g_view->carry_in : nullptr;
  p.carry_out = g_view ? g_view->carry_out : nullptr;
  memset(&p.push, 0, sizeof(p.push));
  memset(&p.red, 0, sizeof(p.red));
  if (reduce && a.prologue == BK_PRO_REDUCE_RMSNORM) p.red = *reduce;
  p.norm_w = bk_ptr<uint16_t>(a.norm_w);
  p.eps = a.eps;
  int vrows = 0;
  bool has_swiglu = false;
  for (int s = 0; s < 4; s++) {
    SegDev& d = p.segs[s];
    if (s >= a.n_segs) {
      d = SegDev{nullptr, nullptr, nullptr, nullptr, 0, 0, 0, 0, 0x7fffffff};
      continue;
    }
    const bkGemvSeg& g = a.segs[s];
    BK_ARG(g.n_rows > 0, "bkGemvQ4K: segment %d has n_rows=%d", s, g.n_rows);
    BK_ARG(g.W != 0 && (g.W & 15) == 0, "bkGemvQ4K: segment %d W must be non-null and 16-byte aligned", s);
    if (g.epilogue == BK_EPI_PUSH_F32) {
      BK_ARG(push && push->n > 0 && a.n_segs == 1, "bkGemvQ4K: segment %d: the push epilogue needs an exchange and a single segment", s);
      p.push = *push;
    } else {
      BK_ARG(g.out != 0, "bkGemvQ4K: segment %d out is null", s);
      BK_ARG(g.epilogue >= BK_EPI_F32 && g.epilogue <= BK_EPI_SWIGLU, "bkGemvQ4K: segment %d unknown epilogue %d", s,
             g.epilogue);
    }
    BK_ARG(g.ld_out >= g.col_off + g.n_rows, "bkGemvQ4K: segment %d ld_out=%d < col_off+n_rows", s, g.ld_out);
    if (g.epilogue == BK_EPI_SWIGLU) {
      BK_ARG(g.W2 != 0 && (g.W2 & 15) == 0, "bkGemvQ4K: segment %d needs a 16-byte aligned W2 for SwiGLU", s);
      has_swiglu = true;
    }
    if (g.epilogue == BK_EPI_ADD_BF16) BK_ARG(g.residual != 0, "bkGemvQ4K: segment %d needs a residual", s);
    d.W = bk_ptr<uint8_t>(g.W);
    d.W2 = bk_ptr<uint8_t>(g.W2);
    d.out = bk_ptr<void>(g.out);
    d.res = bk_ptr<uint16_t>(g.residual);
    d.n_rows = g.n_rows;
    d.epi = g.epilogue;
    d.ld_out = g.ld_out;
    d.col_off = g.col_off;
    d.vrow_begin = vrows;
    vrows += (g.epilogue == BK_EPI_SWIGLU) ? 2 * g.n_rows : g.n_rows;
  }
  // gate/up pairs must sit at even virtual rows so that a pair never straddles a group
  BK_ARG(!has_swiglu || a.n_segs == 1, "bkGemvQ4K: a SwiGLU segment must be the only segment of its launch");
  p.total_vrows = vrows;
  p.status = c.d_status;
  p.trace = bk_trace_slot();
  p.cta_trace = nullptr;
  if (c.cta_trace && c.cta_trace_seen++ == c.cta_trace_launch) p.cta_trace = c.cta_trace;

  if (g_umma_group) {
    if (ctas_out) *ctas_out = 0;
    return bk_gemv_umma_launch(&p, a.B);
  }
  if (tc_path) return bk_gemv_mma_launch(&p, a.K, a.B, vrows, has_swiglu, ctas_out);

  // ---- launch shape ----
  const size_t rowb = (size_t)(a.K / 256) * 144;
  const size_t limit = c.smem_optin - 1024;
  int grid = (vrows + 7) / 8;
  if (grid > c.sm_count) grid = c.sm_count;
  int rpc = (vrows + grid - 1) / grid;
  rpc = (rpc + 1) & ~1;
  grid = (vrows + rpc - 1) / rpc;
  // Occupancy classes.  The hardware may put two CTAs of one grid on the same SM when two slots are free, which
  // makes that SM finish last.  Two classes keep every GEMV grid at one CTA per SM while still letting the NEXT
  // kernel's CTA share the SM (so its weight copies run under this kernel):
  //   class A (large weight slice): > half of the SM's shared memory, <= 14 warps  -> two A CTAs never share an SM
  //   class B (small weight slice): 18 warps (> half of the register file at 64 registers) -> nor do two B CTAs
  // and A + B fit together (65,536 registers, < 227 KB).  A decode layer alternates A and B launches.
  const size_t slice_bytes = (size_t)rpc * rowb;
  const bool class_a = slice_bytes > 56 * 1024;
  const int max_warps = class_a ? 14 : 16;
  // rows per group: one group per warp when the CTA's rows allow it (a single round, evenly loaded), capped by the
  // register budget; a SwiGLU launch keeps gate/up pairs together (even group size)
  const int gmax = gemv_gmax(a.B);
  int G = (rpc + max_warps - 1) / max_warps;
  if (G < 1) G = 1;
  if (has_swiglu) G = (G + 1) & ~1;
  if (G > gmax) G = gmax;
  int n_groups = (rpc + G - 1) / G;
  int nw = n_groups < 8 ? 8 : (n_groups > max_warps ? max_warps : n_groups);
  // pool if the CTA's whole slice fits in about half of the SM's shared memory, else a per-warp ring
  int depth = 0, n_slots = n_groups;
  const size_t half = limit / 2;
  if (gemv_fixed_smem(a.K, a.B, n_groups) + (size_t)n_groups * G * rowb > half + 8 * 1024) {
    // Ring: the CTA's rows do not fit at once.  Measured on K = 2048 ... 17408: 16 warps with as many rows per group as
    // fit beat fewer warps with wider groups (more independent copy/compute chains); single-row groups take 18 warps.
    const int min_g = has_swiglu ? 2 : 1, step_g = has_swiglu ? 2 : 1;
    nw = 16;
    G = (rpc + nw - 1) / nw;
    if (has_swiglu) G = (G + 1) & ~1;
    if (G > gmax) G = gmax;
    if (G < min_g) G = min_g;
    while (G > min_g && gemv_fixed_smem(a.K, a.B, nw * 8) + (size_t)nw * G * rowb > limit) G -= step_g;
    if (G == 1 && gemv_fixed_smem(a.K, a.B, 18 * 8) + (size_t)18 * rowb <= limit) nw = 18;
    while (nw > 8 && gemv_fixed_smem(a.K, a.B, nw * 8) + (size_t)nw * G * rowb > limit) nw -= 2;
    size_t per_level = (size_t)nw * G * rowb;
    size_t fixed = gemv_fixed_smem(a.K, a.B, nw * 8);
    BK_ARG(fixed + per_level <= limit, "bkGemvQ4K: K=%d B=%d does not fit in shared memory", a.K, a.B);
    n_groups = (rpc + G - 1) / G;
    depth = (int)((limit - fixed) / per_level);
    if (g_tune_warps > 0 && g_tune_rows > 0) {   // bkTuneGemvRing: measurement aid
      nw = g_tune_warps;
      G = g_tune_rows;
      if (has_swiglu) G = (G + 1) & ~1;
      per_level = (size_t)nw * G * rowb;
      fixed = gemv_fixed_smem(a.K, a.B, nw * 8);
      BK_ARG(fixed + per_level <= limit, "bkTuneGemvRing: %d warps x %d rows of K=%d do not fit in shared memory", nw, G, a.K);
      n_groups = (rpc + G - 1) / G;
      depth = (int)((limit - fixed) / per_level);
      if (g_tune_depth > 0 && depth > g_tune_depth) depth = g_tune_depth;
    }
    const int max_depth = (n_groups + nw - 1) / nw;
    if (depth > max_depth) depth = max_depth;
    if (depth > 8) depth = 8;
    n_slots = depth * nw;
  }
  p.group_rows = G;
  p.x_unit_words = kUnitWords;
  p.x_row_words = (a.K / 64) * kUnitWords;
  p.x_scale_ld = a.K / 32;
  p.rows_per_cta = rpc;
  p.n_slots = n_slots;
  p.depth = depth;
  size_t smem = gemv_fixed_smem(a.K, a.B, n_slots) + (size_t)n_slots * G * rowb;
  int threads = nw * 32;
  {
    if (class_a) {
      if (smem < limit / 2 + 2048) smem = limit / 2 + 2048;   // > half: one class-A CTA per SM
    } else if (smem <= limit / 2 - 4096) {
      // > half of the register file: one class-B CTA per SM.  18 warps at the 64 registers the kernel is built with;
      // should a compiler allocate fewer, as many warps more as that takes.
      static int regs = 0;
      if (!regs) {
        cudaFuncAttributes fa;
        BK_CUDA(cudaFuncGetAttributes(&fa, gemv_q4k_kernel<1, gemv_gmax(1), false>));
        regs = fa.numRegs > 0 ? fa.numRegs : 64;
      }
      const int per_warp = (regs * 32 + 255) / 256 * 256;
      int wb = 32768 / per_warp + 1;
      if (wb < 18) wb = 18;
      if (wb > 32) wb = 32;
      threads = wb * 32;
    }
  }
  if (ctas_out) *ctas_out = grid;
  const bool tp = p.push.n > 0 || p.red.n > 0;
  if (a.B == 1) return tp ? launch_gemv<1, gemv_gmax(1), true>(p, grid, threads, smem) : launch_gemv<1, gemv_gmax(1), false>(p, grid, threads, smem);
  // batch 2 only when K is too wide for the tensor-core path
  return tp ? launch_gemv<2, gemv_gmax(2), true>(p, grid, threads, smem) : launch_gemv<2, gemv_gmax(2), false>(p, grid, threads, smem);
}

bool bk_gemv_auto_tile(int rows, int K) { return rows >= g_tile_min_rows || (rows >= g_tile_min_rows_cut && K >= 2048); }

extern "C" {

int32_t bkTuneGemvRing(int32_t warps, int32_t rows_per_group, int32_t max_depth) {
  BK_ARG(warps == 0 || (warps >= 8 && warps <= 18 && rows_per_group >= 1 && rows_per_group <= 8), "bkTuneGemvRing: bad shape");
  g_tune_warps = warps;
  g_tune_rows = rows_per_group;
  g_tune_depth = max_depth;
  return BK_OK;
}

int32_t bkTuneTileMinRows(int32_t rows) {
  BK_ARG(rows >= 0, "bkTuneTileMinRows: rows=%d", rows);
  g_tile_min_rows = rows == 0 ? 4096 : rows;
  g_tile_min_rows_cut = rows == 0 ? 1024 : rows;
  return BK_OK;
}

int32_t bkGemvQ4K(const bkGemvArgs* args) {
  BK_REQUIRE_INIT();
  BK_ARG(args != nullptr, "bkGemvQ4K: args is null");
  bkGemvArgs a = *args;  // copied before any asynchronous use
  return bk_gemv_launch(a);
}

int32_t bkGemvQ4KSimple(uint64_t W, int32_t N, int32_t K, uint64_t xq, int32_t B, uint64_t y) {
  BK_REQUIRE_INIT();
  bkGemvArgs a = {};
  a.K = K;
  a.B = B;
  a.n_segs = 1;
  a.prologue = BK_PRO_Q8;
  a.x = xq;
  a.segs[0].W = W;
  a.segs[0].out = y;
  a.segs[0].n_rows = N;
  a.segs[0].epilogue = BK_EPI_F32;
  a.segs[0].ld_out = N;
  return bk_gemv_launch(a);
}

int32_t bkDequantQ4K(uint64_t W, int32_t N, int32_t K, uint64_t out_f32) {
  BK_REQUIRE_INIT();
  BK_ARG(K > 0 && K % 256 == 0 && N > 0, "bkDequantQ4K: bad shape N=%d K=%d", N, K);
  BK_ARG(W && out_f32 && (W & 15) == 0, "bkDequantQ4K: null or misaligned pointer");
  size_t total = (size_t)N * (K / 64);
  dequant_q4k_kernel<<<(unsigned)((total + 255) / 256), 256, 0, bk_ctx().stream>>>(bk_ptr<uint8_t>(W), N, K,
                                                                                  bk_ptr<float>(out_f32));
  BK_CHECK_LAUNCH();
  return BK_OK;
}

int32_t bkBlockDotsQ4K(uint64_t W, int32_t N, int32_t K, uint64_t xq, uint64_t isum, uint64_t qsum) {
  BK_REQUIRE_INIT();
  BK_ARG(K > 0 && K % 256 == 0 && N > 0, "bkBlockDotsQ4K: bad shape N=%d K=%d", N, K);
  BK_ARG(W && xq && isum && qsum && (W & 15) == 0 && (xq & 3) == 0, "bkBlockDotsQ4K: null or misaligned pointer");
  size_t total = (size_t)N * (K / 64);
  block_dots_kernel<<<(unsigned)((total + 255) / 256), 256, 0, bk_ctx().stream>>>(
      bk_ptr<uint8_t>(W), N, K, bk_ptr<uint32_t>(xq), bk_ptr<int32_t>(isum), bk_ptr<int32_t>(qsum));
  BK_CHECK_LAUNCH();
  return BK_OK;
}

static int32_t quant_common(uint64_t x, int32_t K, int32_t B, uint64_t out, bool bf16) {
  BK_ARG(K > 0 && K % 32 == 0 && B > 0, "bkQuantQ8_1: bad shape K=%d B=%d", K, B);
  BK_ARG(x && out && (x & 15) == 0 && (out & 3) == 0, "bkQuantQ8_1: null or misaligned pointer");
  size_t total = (size_t)B * (K / 8);
  unsigned grid = (unsigned)((total + 255) / 256);
  if (bf16)
    quant_q8_1_kernel<true><<<grid, 256, 0, bk_ctx().stream>>>(bk_ptr<void>(x), K, B, bk_ptr<uint8_t>(out));
  else
    quant_q8_1_kernel<false><<<grid, 256, 0, bk_ctx().stream>>>(bk_ptr<void>(x), K, B, bk_ptr<uint8_t>(out));
  BK_CHECK_LAUNCH();
  return BK_OK;
}

int32_t bkQuantQ8_1(uint64_t x_f32, int32_t K, int32_t B, uint64_t out_blocks) {
  BK_REQUIRE_INIT();
  return quant_common(x_f32, K, B, out_blocks, false);
}

int32_t bkQuantQ8_1Bf16(uint64_t x_bf16, int32_t K, int32_t B, uint64_t out_blocks) {
  BK_REQUIRE_INIT();
  return quant_common(x_bf16, K, B, out_blocks, true);
}

}  // extern "C"
