// bk_gemv_umma.cu -- Q4_K x Q8_1 GEMM for 16 or more activation columns on the 5th-generation tensor cores:
// tcgen05.mma kind::i8 with the accumulators in tensor memory (TMEM).
//
// From 16 columns on the product is a dense contraction: the weights are streamed ONCE for all columns (the batch 2..8
// kernel would stream them once per group of 8).  The reference's nearest thing is its int8 tensor-core GEMM experiment
// (src/kernel.ts:396-456: 4-bit blocks expanded to int8 tiles, int32 accumulators, scales applied afterwards,
// experiments/q4k_q81_final.ts:217); this is that scheme on the 144-byte Q4_K layout.
//
// One CTA of 256 threads per 128-row tile; threads t and t+128 <-> tile row t <-> TMEM lane t, each owning half of the
// row's sub-blocks (expansion) and half of the columns (f32 part).  Per 256-weight superblock column:
//   1. every thread copies its 64 quant bytes of the row into shared memory (cp.async, three superblocks in flight) and
//      reads the 16-byte superblock header straight into registers, one superblock ahead;
//   2. it expands the quant bytes into four 32-byte rows of unsigned int8 (one per sub-block) and stores them in the
//      K-major "core matrix" layout the MMA reads (8 rows x 16 bytes contiguous, no swizzle);
//   3. the Q8_1 activation blocks of the superblock are staged the same way (signed int8, N = columns);
//   4. one thread issues eight MMAs (M = 128, N = 16 or 32, K = 32: exactly one sub-block each) into eight separate
//      TMEM accumulators -- the integer dot of every (row, column, sub-block), exact -- and commits to an mbarrier;
//   5. while the tensor core works on superblock s, all threads run the f32 part of superblock s-1: tcgen05.ld brings a
//      thread its row's int32 sums, and  accd = fma(d8, f32(sc*isum), accd), accm = fma(s8, f32(m), accm)  over the
//      sub-blocks in ascending order, then  y += fma(d, accd, -(dmin*accm)).
// That f32 order ("tile order": one chain per (row, column)) is fixed and mirrored by the CPU checker; it differs from
// the batch <= 8 kernels' lane / butterfly order by a few ulp.
//
// Single CTA per tile, no cluster, no multicast, no tensor maps.  Every wait is bounded; TMEM is released on every
// path out of the kernel.
#include "bk_gemv_shared.cuh"

namespace {

constexpr int kTileM = 128;
constexpr int kUT = 256;            // threads: warps w and w+4 share TMEM lane quarter w (rows 32w..32w+31) and split the columns
constexpr int kRawStages = 3;       // superblock columns of raw Q4_K rows in flight
constexpr int kTmemCols = 512;

struct UmmaParams {
  GemvParams g;   // K, segments, total_vrows, x = Q8_1 blocks [B][K/32][36], status
  int B;          // activation columns of this launch, 1..32
  int Npad;       // MMA N: 16 or 32
};

BK_DEVINL uint64_t umma_desc(uint32_t smem_addr, uint32_t lbo_bytes, uint32_t sbo_bytes) {
  // K-major, no swizzle: 8 rows x 16 bytes contiguous; lbo = bytes between the two 16-byte K chunks of a 32-byte row,
  // sbo = bytes between groups of 8 rows.  Bits [46,48) = 1: the descriptor version of this architecture.
  return (uint64_t)((smem_addr >> 4) & 0x3fffu) | ((uint64_t)((lbo_bytes >> 4) & 0x3fffu) << 16) |
         ((uint64_t)((sbo_bytes >> 4) & 0x3fffu) << 32) | (1ull << 46);
}

BK_DEVINL void cp_async16(uint32_t dst, const void* src) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst), "l"(src) : "memory");
}

// {a.x*b.x + c.x, a.y*b.y + c.y}: two IEEE fused multiply-adds in one instruction
BK_DEVINL float2 fma2(float2 a, float2 b, float2 c) {
  unsigned long long ra, rb, rc, rd;
  asm("mov.b64 %0, {%1, %2};" : "=l"(ra) : "f"(a.x), "f"(a.y));
  asm("mov.b64 %0, {%1, %2};" : "=l"(rb) : "f"(b.x), "f"(b.y));
  asm("mov.b64 %0, {%1, %2};" : "=l"(rc) : "f"(c.x), "f"(c.y));
  asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(rd) : "l"(ra), "l"(rb), "l"(rc));
  float2 d;
  asm("mov.b64 {%0, %1}, %2;" : "=f"(d.x), "=f"(d.y) : "l"(rd));
  return d;
}

// NC: accumulator columns per thread (Npad / 2): 8 or 16
template <int NC>
__global__ void __launch_bounds__(kUT, 1) gemv_q4k_umma_kernel(const UmmaParams P) {
  bk_pdl_trigger();
  const GemvParams& p = P.g;
  extern __shared__ __align__(1024) uint8_t smem[];
  constexpr int Npad = 2 * NC;
  uint8_t* raw = smem;                                              // [kRawStages][128][144]
  uint8_t* As = raw + (size_t)kRawStages * kTileM * 144;            // [2][8][4096]
  As = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(As) + 1023) & ~(uintptr_t)1023);
  uint8_t* Bs = As + 2 * 8 * 4096;                                  // [2][8][Npad*32]
  float2* scs = reinterpret_cast<float2*>(Bs + 2 * 8 * 32 * 32);    // [2][8][32] {d8, s8}
  uint64_t* mbar = reinterpret_cast<uint64_t*>(scs + 2 * 8 * 32);   // [2]
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(mbar + 2);

  const int t = threadIdx.x, warp = t >> 5;
  const int row_t = t & (kTileM - 1);       // tile row (= TMEM lane) of this thread
  const int half = t >> 7;                  // 0: sub-blocks 0..3 and columns [0, NC); 1: sub-blocks 4..7 and columns [NC, 2NC)
  const int K = p.K, nsb = K / 256, nblk = K / 32;

  if (t == 0) {
    mbar_init(smem_u32(mbar), 1);
    mbar_init(smem_u32(mbar + 1), 1);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 0) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)), "r"(kTmemCols)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
  const uint32_t tmem = *reinterpret_cast<volatile uint32_t*>(tmem_slot);
  // M = 128, N = Npad, int32 accumulators, A unsigned 8-bit, B signed 8-bit, both K-major
  const uint32_t idesc = (2u << 4) | (0u << 7) | (1u << 10) | ((uint32_t)(Npad >> 3) << 17) | ((uint32_t)(kTileM >> 4) << 24);

  const int n_tiles = (p.total_vrows + kTileM - 1) / kTileM;
  uint32_t uses[2] = {0u, 0u};   // completed commits per accumulator buffer (mbarrier phase)
  const uint32_t* xq = reinterpret_cast<const uint32_t*>(p.x);
  bool waited = false;           // the dependency wait has been executed (weights are requested before it)

  for (int tile = blockIdx.x; tile < n_tiles; tile += gridDim.x) {
    const int vrow = tile * kTileM + row_t;
    const bool have_row = vrow < p.total_vrows;
    VRow vr = {nullptr, 0, 0};
    if (have_row) vr = decode_vrow(p, vrow);
    const uint8_t* wrow = vr.row;

    float y[NC];
#pragma unroll
    for (int c = 0; c < NC; c++) y[c] = 0.0f;

    // this thread's share of its row's superblock s: the four 16-byte quant chunks of two 32-byte groups
    // (half 0: groups 0,1 = sub-blocks 0..3; half 1: groups 2,3 = sub-blocks 4..7)
    auto request_raw = [&](int s) {
      if (s < nsb && have_row) {
        const uint32_t dst = smem_u32(raw + ((size_t)(s % kRawStages) * kTileM + row_t) * 144) + 16 + half * 64;
        const uint8_t* src = wrow + (size_t)s * 144 + 16 + half * 64;
#pragma unroll
        for (int k = 0; k < 4; k++) cp_async16(dst + 16 * k, src + 16 * k);
      }
      asm volatile("cp.async.commit_group;" ::: "memory");
    };
    // activation block (j, b) of superblock s for this thread: item i = j*Npad + b, Npad*8 <= 256 items
    uint32_t xw[9];
    const int xi_j = t / Npad, xi_b = t - (t / Npad) * Npad;
    auto load_x = [&](int s) {
      const bool ok = s < nsb && t < Npad * 8 && xi_b < P.B;
#pragma unroll
      for (int k = 0; k < 9; k++) xw[k] = ok ? __ldcg(xq + ((size_t)xi_b * nblk + (size_t)s * 8 + xi_j) * 9 + k) : 0u;
    };
    auto store_x = [&](int s) {
      if (t < Npad * 8) {
        uint8_t* tile_j = Bs + (size_t)(s & 1) * 8 * (Npad * 32) + (size_t)xi_j * (Npad * 32) + (xi_b >> 3) * 128 + (xi_b & 7) * 16;
        *reinterpret_cast<uint4*>(tile_j) = make_uint4(xw[0], xw[1], xw[2], xw[3]);
        *reinterpret_cast<uint4*>(tile_j + Npad * 16) = make_uint4(xw[4], xw[5], xw[6], xw[7]);
        int qsum = 0;
#pragma unroll
        for (int k = 0; k < 8; k++) qsum = bk_dp4a_ss(xw[k], 0x01010101u, qsum);
        const float d8 = bk_q8half_to_f32((uint16_t)(xw[8] & 0xffffu));
        scs[(size_t)(s & 1) * 8 * 32 + xi_j * 32 + xi_b] = make_float2(d8, __fmul_rn(d8, (float)qsum));
      }
    };
    // superblock header (d, dmin, scales, mins) of this thread's row, read straight from global memory one superblock
    // ahead: next (in flight), current (being multiplied), previous (being scaled)
    uint4 h_next = make_uint4(0, 0, 0, 0), h_cur = make_uint4(0, 0, 0, 0), h_prev = make_uint4(0, 0, 0, 0);
    auto load_hdr = [&](int s) { h_next = (s < nsb && have_row) ? __ldg(reinterpret_cast<const uint4*>(wrow + (size_t)s * 144)) : make_uint4(0, 0, 0, 0); };

    auto epilogue = [&](int s) {   // f32 part of superblock s from accumulator buffer s&1, this thread's NC columns
      const int buf = s & 1;
      mbar_wait_bounded(smem_u32(mbar + buf), (uses[buf] & 1u), p.status);
      uses[buf]++;
      asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
      const float d = bk_f16_to_f32((uint16_t)(h_prev.x & 0xffffu)), dmin = bk_f16_to_f32((uint16_t)(h_prev.x >> 16));
      const float2* sb_ = scs + (size_t)buf * 8 * 32 + half * NC;
      float2 acc[NC];   // {accd, accm}
#pragma unroll
      for (int c = 0; c < NC; c++) acc[c] = make_float2(0.0f, 0.0f);
#pragma unroll
      for (int j = 0; j < 8; j++) {
        int sc, mn;
        bk_q4k_scale_min(h_prev.y, h_prev.z, h_prev.w, j, sc, mn);
        const float fsc = (float)sc, fm = (float)mn;
        uint32_t r[NC];
        const uint32_t taddr = tmem + ((uint32_t)((warp & 3) * 32) << 16) + (uint32_t)(buf * 256 + j * Npad + half * NC);
        if constexpr (NC == 16) {
          asm volatile(
              "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
              : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
                "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
              : "r"(taddr)
              : "memory");
        } else {
          asm volatile("tcgen05.ld.sync.aligned.32x32b.x8.b32 {%0, %1, %2, %3, %4, %5, %6, %7}, [%8];"
                       : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7])
                       : "r"(taddr)
                       : "memory");
        }
        asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
        for (int c = 0; c < NC; c++) {
          // accd = fma(d8, f32(sc*isum), accd) and accm = fma(s8, f32(m), accm) as one packed instruction; sc*isum < 2^22
          // is exact as the f32 product of the two integers
          acc[c] = fma2(sb_[j * 32 + c], make_float2(__fmul_rn(fsc, (float)(int)r[c]), fm), acc[c]);
        }
      }
#pragma unroll
      for (int c = 0; c < NC; c++) y[c] = __fadd_rn(y[c], fmaf(d, acc[c].x, -__fmul_rn(dmin, acc[c].y)));
      asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    };

    // ---- pipeline over the superblock columns of this tile ----
    for (int s = 0; s < kRawStages; s++) request_raw(s);   // weights depend on nothing: requested before the wait
    load_hdr(0);
    if (!waited) {
      bk_pdl_wait();
      waited = true;
    }
    load_x(0);
    store_x(0);
    for (int s = 0; s < nsb; s++) {
      h_prev = h_cur;
      h_cur = h_next;
      load_hdr(s + 1);
      load_x(s + 1);   // in flight during the expansion below
      // (1) this thread's 64 quant bytes of superblock s have landed (it copied them itself)
      asm volatile("cp.async.wait_group %0;" ::"n"(kRawStages - 1) : "memory");
      const uint8_t* rw = raw + ((size_t)(s % kRawStages) * kTileM + row_t) * 144 + 16 + half * 64;
      uint4 q[4];
#pragma unroll
      for (int k = 0; k < 4; k++) q[k] = have_row ? *reinterpret_cast<const uint4*>(rw + 16 * k) : make_uint4(0, 0, 0, 0);
      request_raw(s + kRawStages);   // refills the stage just read
      // (2) 4-bit quants -> unsigned int8 rows of this thread's four sub-block tiles
      uint8_t* Ab = As + (size_t)(s & 1) * 8 * 4096 + (row_t >> 3) * 128 + (row_t & 7) * 16;
#pragma unroll
      for (int g = 0; g < 2; g++) {
        const int grp = half * 2 + g;
        const uint4 a = q[2 * g], b = q[2 * g + 1];
        const uint4 lo0 = make_uint4(a.x & 0x0f0f0f0fu, a.y & 0x0f0f0f0fu, a.z & 0x0f0f0f0fu, a.w & 0x0f0f0f0fu);
        const uint4 lo1 = make_uint4(b.x & 0x0f0f0f0fu, b.y & 0x0f0f0f0fu, b.z & 0x0f0f0f0fu, b.w & 0x0f0f0f0fu);
        const uint4 hi0 = make_uint4((a.x >> 4) & 0x0f0f0f0fu, (a.y >> 4) & 0x0f0f0f0fu, (a.z >> 4) & 0x0f0f0f0fu, (a.w >> 4) & 0x0f0f0f0fu);
        const uint4 hi1 = make_uint4((b.x >> 4) & 0x0f0f0f0fu, (b.y >> 4) & 0x0f0f0f0fu, (b.z >> 4) & 0x0f0f0f0fu, (b.w >> 4) & 0x0f0f0f0fu);
        *reinterpret_cast<uint4*>(Ab + (2 * grp) * 4096) = lo0;
        *reinterpret_cast<uint4*>(Ab + (2 * grp) * 4096 + 2048) = lo1;
        *reinterpret_cast<uint4*>(Ab + (2 * grp + 1) * 4096) = hi0;
        *reinterpret_cast<uint4*>(Ab + (2 * grp + 1) * 4096 + 2048) = hi1;
      }
      asm volatile("fence.proxy.async.shared::cta;" ::: "memory");   // the MMA reads shared memory through the async proxy
      __syncthreads();
      // (3) eight MMAs, one per sub-block, into accumulator buffer s&1
      if (t == 0) {
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        const uint32_t a0 = smem_u32(As + (size_t)(s & 1) * 8 * 4096);
        const uint32_t b0 = smem_u32(Bs + (size_t)(s & 1) * 8 * (Npad * 32));
#pragma unroll
        for (int j = 0; j < 8; j++) {
          const uint64_t ad = umma_desc(a0 + j * 4096, 2048, 128);
          const uint64_t bd = umma_desc(b0 + j * (Npad * 32), (uint32_t)Npad * 16, 128);
          const uint32_t dcol = tmem + (uint32_t)((s & 1) * 256 + j * Npad);
          asm volatile(
              "{\n\t.reg .pred pz;\n\tsetp.ne.b32 pz, %4, 0;\n\t"
              "tcgen05.mma.cta_group::1.kind::i8 [%0], %1, %2, %3, {%5, %5, %5, %5}, pz;\n\t}"
              ::"r"(dcol), "l"(ad), "l"(bd), "r"(idesc), "r"(0u), "r"(0u)
              : "memory");
        }
        asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(mbar + (s & 1)))
                     : "memory");
      }
      // (4) f32 part of the previous superblock while the tensor core works on this one
      if (s > 0) epilogue(s - 1);
      // (5) activations of the next superblock into the buffers the previous one has released -- once every thread
      //     has finished reading that one's block scales
      __syncthreads();
      store_x(s + 1);
    }
    h_prev = h_cur;
    epilogue(nsb - 1);
    asm volatile("cp.async.wait_group 0;" ::: "memory");

    // ---- fused epilogues: this thread's columns [half*NC, half*NC + NC) of its row ----
    const SegDev& sg = p.segs[vr.si];
    const bool swiglu = have_row && sg.epi == BK_EPI_SWIGLU;
#pragma unroll
    for (int c = 0; c < NC; c++) {
      const int b = half * NC + c;
      const float yup = __shfl_xor_sync(0xffffffffu, y[c], 1);   // the odd neighbour row: the "up" row of a SwiGLU pair
      if (b < P.B && have_row && !(swiglu && (row_t & 1)))
        store_epilogue<false>(p, sg, (size_t)b * sg.ld_out + sg.col_off + vr.n, y[c], yup);
    }
    __syncthreads();   // shared buffers and accumulators are reused by the next tile
  }
  if (!waited) bk_pdl_wait();

  // ---- release tensor memory (every thread gets here, whatever happened above) ----
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  if (warp == 0) {
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(kTmemCols) : "memory");
  }
}

size_t umma_smem_bytes() {
  return (size_t)kRawStages * kTileM * 144 + 1024 + 2 * 8 * 4096 + 2 * 8 * 32 * 32 + 2 * 8 * 32 * 8 + 64;
}

}  // namespace

// Launch for at most 32 columns (the caller cuts wider batches into groups of 32).  p: a filled GemvParams.
int32_t bk_gemv_umma_launch(void* params, int B) {
  BkContext& c = bk_ctx();
  UmmaParams P;
  P.g = *static_cast<GemvParams*>(params);
  BK_ARG(B >= 1 && B <= 32, "tile GEMV: %d columns per launch (1..32)", B);
  P.B = B;
  P.Npad = B <= 16 ? 16 : 32;
  static bool configured = false;
  const size_t smem = umma_smem_bytes();
  if (!configured) {
    BK_CUDA(cudaFuncSetAttribute(gemv_q4k_umma_kernel<8>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    BK_CUDA(cudaFuncSetAttribute(gemv_q4k_umma_kernel<16>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    configured = true;
  }
  const int tiles = (P.g.total_vrows + kTileM - 1) / kTileM;
  const int grid = tiles < c.sm_count ? tiles : c.sm_count;
  if (P.Npad == 16) BK_CUDA(bk_launch_pdl(gemv_q4k_umma_kernel<8>, dim3(grid), dim3(kUT), smem, P));
  else BK_CUDA(bk_launch_pdl(gemv_q4k_umma_kernel<16>, dim3(grid), dim3(kUT), smem, P));
  BK_CHECK_LAUNCH();
  return BK_OK;
}
