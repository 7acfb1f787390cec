// bk_gemv_umma.cu -- Q4_K x Q8_1 GEMM for 16 or more activation columns on the 5th-generation tensor cores:
// tcgen05.mma kind::i8 with the accumulators in tensor memory (TMEM).
//
// From 16 columns on the product is a dense contraction: the weights are streamed ONCE for all columns (the batch 2..8
// kernel would stream them once per group of 8).  The reference's nearest thing is its int8 tensor-core GEMM experiment
// (src/kernel.ts:396-456: 4-bit blocks expanded to int8 tiles, int32 accumulators, scales applied afterwards,
// experiments/q4k_q81_final.ts:217); this is that scheme on the 144-byte Q4_K layout.
//
// One CTA of 128 threads per 128-row tile; thread t <-> tile row t <-> TMEM lane t.  Per 256-weight superblock column:
//   1. every thread copies its row's 144 bytes into shared memory (cp.async, three superblocks in flight);
//   2. it expands the 128 quant bytes into eight 32-byte rows of unsigned int8 (one per sub-block) and stores them in
//      the K-major "core matrix" layout the MMA reads (8 rows x 16 bytes contiguous, no swizzle);
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
constexpr int kUT = 128;            // threads
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

__global__ void __launch_bounds__(kUT, 1) gemv_q4k_umma_kernel(const UmmaParams P) {
  bk_pdl_trigger();
  const GemvParams& p = P.g;
  extern __shared__ __align__(1024) uint8_t smem[];
  const int Npad = P.Npad;
  uint8_t* raw = smem;                                              // [kRawStages][128][144]
  uint8_t* As = raw + (size_t)kRawStages * kTileM * 144;            // [2][8][4096]
  As = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(As) + 1023) & ~(uintptr_t)1023);
  uint8_t* Bs = As + 2 * 8 * 4096;                                  // [2][8][Npad*32]
  float2* scs = reinterpret_cast<float2*>(Bs + 2 * 8 * 32 * 32);    // [2][8][32] {d8, s8}
  uint64_t* mbar = reinterpret_cast<uint64_t*>(scs + 2 * 8 * 32);   // [2]
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(mbar + 2);

  const int t = threadIdx.x, warp = t >> 5, lane = t & 31;
  const int K = p.K, nsb = K / 256, nblk = K / 32;
  const uint32_t rowb = (uint32_t)nsb * 144;

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

  bk_pdl_wait();

  const int n_tiles = (p.total_vrows + kTileM - 1) / kTileM;
  const int nhalves = Npad / 16;
  uint32_t uses[2] = {0u, 0u};   // completed commits per accumulator buffer (mbarrier phase)
  const uint32_t* xq = reinterpret_cast<const uint32_t*>(p.x);

  for (int tile = blockIdx.x; tile < n_tiles; tile += gridDim.x) {
    const int vrow = tile * kTileM + t;
    const bool have_row = vrow < p.total_vrows;
    VRow vr = {nullptr, 0, 0};
    if (have_row) vr = decode_vrow(p, vrow);
    const uint8_t* wrow = vr.row;

    float y[32];
#pragma unroll
    for (int c = 0; c < 32; c++) y[c] = 0.0f;

    auto request_raw = [&](int s) {   // this thread's 144 bytes of superblock s
      if (s < nsb && have_row) {
        const uint32_t dst = smem_u32(raw + ((size_t)(s % kRawStages) * kTileM + t) * 144);
        const uint8_t* src = wrow + (size_t)s * 144;
#pragma unroll
        for (int k = 0; k < 9; k++) cp_async16(dst + 16 * k, src + 16 * k);
      }
      asm volatile("cp.async.commit_group;" ::: "memory");
    };
    // activation blocks of superblock s: item i = j*Npad + b, two per thread at most (Npad*8 <= 256)
    uint32_t xw[2][9];
    auto load_x = [&](int s) {
#pragma unroll
      for (int r = 0; r < 2; r++) {
        const int i = t + r * kUT;
        const int j = i / Npad, b = i - j * Npad;
        const bool ok = s < nsb && i < Npad * 8 && b < P.B;
#pragma unroll
        for (int k = 0; k < 9; k++) xw[r][k] = ok ? __ldcg(xq + ((size_t)b * nblk + (size_t)s * 8 + j) * 9 + k) : 0u;
      }
    };
    auto store_x = [&](int s) {
      uint8_t* Bb = Bs + (size_t)(s & 1) * 8 * (Npad * 32);
      float2* sb_ = scs + (size_t)(s & 1) * 8 * 32;
#pragma unroll
      for (int r = 0; r < 2; r++) {
        const int i = t + r * kUT;
        if (i < Npad * 8) {
          const int j = i / Npad, b = i - j * Npad;
          uint8_t* tile_j = Bb + (size_t)j * (Npad * 32) + (b >> 3) * 128 + (b & 7) * 16;
          *reinterpret_cast<uint4*>(tile_j) = make_uint4(xw[r][0], xw[r][1], xw[r][2], xw[r][3]);
          *reinterpret_cast<uint4*>(tile_j + Npad * 16) = make_uint4(xw[r][4], xw[r][5], xw[r][6], xw[r][7]);
          int qsum = 0;
#pragma unroll
          for (int k = 0; k < 8; k++) qsum = bk_dp4a_ss(xw[r][k], 0x01010101u, qsum);
          const float d8 = bk_q8half_to_f32((uint16_t)(xw[r][8] & 0xffffu));
          sb_[j * 32 + b] = make_float2(d8, __fmul_rn(d8, (float)qsum));
        }
      }
    };

    // superblock header of this thread's row: current (being multiplied) and previous (being scaled)
    uint32_t h_cur[4] = {0, 0, 0, 0}, h_prev[4] = {0, 0, 0, 0};

    auto epilogue = [&](int s) {   // f32 part of superblock s from accumulator buffer s&1
      const int buf = s & 1;
      mbar_wait_bounded(smem_u32(mbar + buf), (uses[buf] & 1u), p.status);
      uses[buf]++;
      asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
      const float d = bk_f16_to_f32((uint16_t)(h_prev[0] & 0xffffu)), dmin = bk_f16_to_f32((uint16_t)(h_prev[0] >> 16));
      const float2* sb_ = scs + (size_t)buf * 8 * 32;
      for (int h = 0; h < nhalves; h++) {
        float accd[16], accm[16];
#pragma unroll
        for (int c = 0; c < 16; c++) accd[c] = accm[c] = 0.0f;
#pragma unroll
        for (int j = 0; j < 8; j++) {
          int sc, mn;
          bk_q4k_scale_min(h_prev[1], h_prev[2], h_prev[3], j, sc, mn);
          const float fm = (float)mn;
          uint32_t r[16];
          const uint32_t taddr = tmem + ((uint32_t)(warp * 32) << 16) + (uint32_t)(buf * 256 + j * Npad + h * 16);
          asm volatile(
              "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
              : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
                "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
              : "r"(taddr)
              : "memory");
          asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
          for (int c = 0; c < 16; c++) {
            const float2 f = sb_[j * 32 + h * 16 + c];
            accd[c] = fmaf(f.x, (float)(sc * (int)r[c]), accd[c]);
            accm[c] = fmaf(f.y, fm, accm[c]);
          }
        }
#pragma unroll
        for (int c = 0; c < 16; c++) {
          const float val = fmaf(d, accd[c], -__fmul_rn(dmin, accm[c]));
          if (h == 0) y[c] = __fadd_rn(y[c], val);
          else y[16 + c] = __fadd_rn(y[16 + c], val);
        }
      }
      asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    };

    // ---- pipeline over the superblock columns of this tile ----
    for (int s = 0; s < kRawStages; s++) request_raw(s);
    load_x(0);
    store_x(0);
    for (int s = 0; s < nsb; s++) {
      load_x(s + 1);   // in flight during the expansion below
      // (1) this row's raw superblock s has landed (each thread copied its own bytes)
      asm volatile("cp.async.wait_group %0;" ::"n"(kRawStages - 1) : "memory");
      const uint8_t* rw = raw + ((size_t)(s % kRawStages) * kTileM + t) * 144;
      uint4 q[9];
#pragma unroll
      for (int k = 0; k < 9; k++) q[k] = have_row ? *reinterpret_cast<const uint4*>(rw + 16 * k) : make_uint4(0, 0, 0, 0);
      request_raw(s + kRawStages);   // refills the stage just read (every later group keeps the count of 2 pending valid)
#pragma unroll
      for (int k = 0; k < 4; k++) h_prev[k] = h_cur[k];
      h_cur[0] = q[0].x; h_cur[1] = q[0].y; h_cur[2] = q[0].z; h_cur[3] = q[0].w;
      // (2) 4-bit quants -> unsigned int8 rows of the eight sub-block tiles
      uint8_t* Ab = As + (size_t)(s & 1) * 8 * 4096 + (t >> 3) * 128 + (t & 7) * 16;
#pragma unroll
      for (int g = 0; g < 4; g++) {
        const uint4 a = q[1 + 2 * g], b = q[2 + 2 * g];
        const uint4 lo0 = make_uint4(a.x & 0x0f0f0f0fu, a.y & 0x0f0f0f0fu, a.z & 0x0f0f0f0fu, a.w & 0x0f0f0f0fu);
        const uint4 lo1 = make_uint4(b.x & 0x0f0f0f0fu, b.y & 0x0f0f0f0fu, b.z & 0x0f0f0f0fu, b.w & 0x0f0f0f0fu);
        const uint4 hi0 = make_uint4((a.x >> 4) & 0x0f0f0f0fu, (a.y >> 4) & 0x0f0f0f0fu, (a.z >> 4) & 0x0f0f0f0fu, (a.w >> 4) & 0x0f0f0f0fu);
        const uint4 hi1 = make_uint4((b.x >> 4) & 0x0f0f0f0fu, (b.y >> 4) & 0x0f0f0f0fu, (b.z >> 4) & 0x0f0f0f0fu, (b.w >> 4) & 0x0f0f0f0fu);
        *reinterpret_cast<uint4*>(Ab + (2 * g) * 4096) = lo0;
        *reinterpret_cast<uint4*>(Ab + (2 * g) * 4096 + 2048) = lo1;
        *reinterpret_cast<uint4*>(Ab + (2 * g + 1) * 4096) = hi0;
        *reinterpret_cast<uint4*>(Ab + (2 * g + 1) * 4096 + 2048) = hi1;
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
#pragma unroll
    for (int k = 0; k < 4; k++) h_prev[k] = h_cur[k];
    epilogue(nsb - 1);
    asm volatile("cp.async.wait_group 0;" ::: "memory");

    // ---- fused epilogues (the column loop is the batch) ----
    const SegDev& sg = p.segs[vr.si];
    const bool swiglu = have_row && sg.epi == BK_EPI_SWIGLU;
#pragma unroll
    for (int b = 0; b < 32; b++) {
      const float yup = __shfl_xor_sync(0xffffffffu, y[b], 1);   // the odd neighbour row: the "up" row of a SwiGLU pair
      if (b < P.B && have_row && !(swiglu && (t & 1)))
        store_epilogue<false>(p, sg, (size_t)b * sg.ld_out + sg.col_off + vr.n, y[b], yup);
    }
    __syncthreads();   // shared buffers and accumulators are reused by the next tile
  }

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
    BK_CUDA(cudaFuncSetAttribute(gemv_q4k_umma_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    configured = true;
  }
  const int tiles = (P.g.total_vrows + kTileM - 1) / kTileM;
  const int grid = tiles < c.sm_count ? tiles : c.sm_count;
  BK_CUDA(bk_launch_pdl(gemv_q4k_umma_kernel, dim3(grid), dim3(kUT), smem, P));
  BK_CHECK_LAUNCH();
  return BK_OK;
}
