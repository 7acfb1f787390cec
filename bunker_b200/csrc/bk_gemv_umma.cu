// bk_gemv_umma.cu -- Q4_K x Q8_1 GEMM for 16 or more activation columns on the 5th-generation tensor cores:
// tcgen05.mma kind::i8 with the accumulators in tensor memory (TMEM).
//
// From 16 columns on the product is a dense contraction: the weights are streamed ONCE for all columns (the batch 2..8
// kernel would stream them once per group of 8).  The reference's nearest thing is its int8 tensor-core GEMM experiment
// (src/kernel.ts:396-456: 4-bit blocks expanded to int8 tiles, int32 accumulators, scales applied afterwards,
// experiments/q4k_q81_final.ts:217); this is that scheme on the 144-byte Q4_K layout.
//
// One CTA of 768 threads per SM walks over its 128-row tiles, as five groups of warps that meet only at mbarriers:
//   * one PRODUCER warp keeps a ring of two stages filled: a stage holds two superblock columns (288 bytes) of each of
//     the 128 rows; the ring runs ahead across tile boundaries and starts before the dependency wait (see "Weight
//     feed" below for the two ways a stage is filled);
//   * four EXPANDER warps (thread <-> tile row).  Per 256-weight superblock column every expander thread
//     unpacks its row's 128 quant bytes into eight 32-byte rows of unsigned int8 (one per sub-block), stored in the
//     K-major "core matrix" layout the MMA reads (8 rows x 16 bytes contiguous, no swizzle), and decodes the eight
//     6-bit scales and mins into a table;
//   * two STAGER warps put the superblock's Q8_1 activation blocks into the same layout (signed int8, N = columns)
//     with their d8 and s8 scales, reading one superblock ahead;
//   * one MMA warp: when all 128 expander threads have arrived, one thread issues eight MMAs (M = 128, N = 16 or 32,
//     K = 32: exactly one sub-block each) into eight separate TMEM accumulators -- the integer dot of every (row,
//     column, sub-block), exact -- and commits to an mbarrier (issue and commit keep that thread busy for about a
//     thousand cycles per superblock, which is why it is not an expander);
//   * sixteen SCALER warps (four per TMEM lane quarter, each a quarter of the columns) run the f32 part of a
//     superblock as soon as its MMAs have completed: tcgen05.ld brings a thread its row's int32 sums, and
//     accd = fma(d8, f32(sc*isum), accd), accm = fma(s8, f32(m), accm)  over the sub-blocks in ascending order, then
//     yc += fma(d, accd, -(dmin*accm));  every four superblocks  y += yc.  They hand the buffers back through two more
//     mbarriers: the shared-memory side (tiles and tables, three buffers, so that the unpacking runs up to two steps
//     ahead) to the expanders and stagers, the accumulators (two buffers of 256 TMEM columns) to the MMA warp.
// That f32 order ("tile order": per (row, column) one chain per chunk of four superblocks, chunks added in order) is
// fixed and mirrored by the CPU checker; it differs from the batch <= 8 kernels' lane / butterfly order by a few ulp.
//
// A launch of few tiles (fewer than half the SMs) is cut along K: thread block (tile, part) runs a contiguous range of
// whole chunks and leaves each chunk's partial sums in a scratch buffer; the block that arrives last at the tile's
// counter adds the chunks in ascending order -- the same chain as an uncut launch -- and runs the epilogue.
//
// Weight feed: when every segment's row count is a multiple of 32 (all shapes of the model) a stage is filled with one
// tiled TMA load per 32-row box and superblock column (cp.async.bulk.tensor.2d through a tensor map of the weight
// matrix; 8 instructions per stage instead of 128 row copies -- the row copies cap the feed at about 7 GB/s per SM
// and cost 5 us before the first stage has landed).  A SwiGLU launch then keeps its 64 gate rows in tile rows 0..63
// and the 64 up rows in 64..127 (boxes are contiguous rows of one matrix), and the epilogue passes the up values to
// the gate rows' threads through shared memory.  Other shapes keep the per-row copies.
//
// No cluster, no multicast.  Every wait is bounded (and may sleep between polls); TMEM is released on every path out
// of the kernel.
#include <cuda.h>   // CUtensorMap and the types of its encoder; the encoder itself is looked up at run time

#include "bk_gemv_shared.cuh"

namespace {

constexpr int kTileM = 128;
// The supporting roles come first: their work per step is short but the scalers wait for it
constexpr int kExpanderWarps = 4;   // warps 0..3: thread <-> tile row
constexpr int kStagerWarp0 = 4;     // warps 4, 5 stage the activation blocks
constexpr int kStagerWarps = 2;
constexpr int kProducerWarp = 6;    // keeps the weight ring filled
constexpr int kMmaWarp = 7;         // issues the MMAs
constexpr int kScalerWarp0 = 8;     // warps 8..23: warp w reads TMEM lanes 32*(w mod 4)..+31, columns of quarter (w - 8) / 4
constexpr int kScalerWarps = 16;
constexpr int kUT = (kScalerWarp0 + kScalerWarps) * 32;
constexpr int kStages = 2;          // ring stages, two superblock columns each
constexpr int kSB = 3;              // shared-memory buffers (A / B tiles, scale tables): the unpacking runs up to two steps
                                    // ahead of the two TMEM accumulator buffers
constexpr int kRowPitch = 2 * 144 + 16;   // bytes between rows of a stage: 76 words, so 16-byte reads of 8 rows hit 8 bank groups
constexpr int kStageBytes = kTileM * kRowPitch;
constexpr int kPlaneBytes = kTileM * 144;   // tensor-map feed: a stage is two planes [128 rows][144 bytes], one per superblock column
constexpr int kTmemCols = 512;
constexpr int kScsLd = 72;          // floats per sub-block of the column scales: 32 d8, 32 s8, 8 of padding (bank spread)

// dynamic shared memory without the SwiGLU exchange buffer, which follows it: ring, A tiles (3 x 8 x 4 KB), B tiles,
// column scales, row scale table, row {d, dmin}, barriers and flags
__host__ __device__ constexpr size_t umma_smem_core_bytes() {
  return (size_t)kStages * kStageBytes + kSB * 8 * 4096 + kSB * 8 * 32 * 32 + kSB * 8 * kScsLd * 4 + kSB * 8 * kTileM * 2 +
         kSB * kTileM * 8 + 160;
}

struct UmmaParams {
  GemvParams g;   // K, segments, total_vrows, x = Q8_1 blocks [B][K/32][36], status
  int B;          // activation columns of this launch, 1..32
  int Npad;       // MMA N: 16 or 32
  int use_maps;   // weights are fed by tiled TMA loads through maps[] (segment i -> maps[i]; the up matrix of a SwiGLU launch -> maps[4])
  int ksplit;     // > 1: every tile is cut along K over ksplit thread blocks (launches of few tiles)
  float* scratch; // ksplit > 1: per-chunk partial sums [tile][chunk][32 columns][128 rows]
  int* counters;  // ksplit > 1: arrivals per tile; the last block to arrive adds the chunks in order and resets the count
  CUtensorMap maps[5];   // use_maps: uint8 [n_rows][row bytes], box 32 rows x 144 bytes
};

BK_DEVINL uint64_t umma_desc(uint32_t smem_addr, uint32_t lbo_bytes, uint32_t sbo_bytes) {
  // K-major, no swizzle: 8 rows x 16 bytes contiguous; lbo = bytes between the two 16-byte K chunks of a 32-byte row,
  // sbo = bytes between groups of 8 rows.  Bits [46,48) = 1: the descriptor version of this architecture.
  return (uint64_t)((smem_addr >> 4) & 0x3fffu) | ((uint64_t)((lbo_bytes >> 4) & 0x3fffu) << 16) |
         ((uint64_t)((sbo_bytes >> 4) & 0x3fffu) << 32) | (1ull << 46);
}

// f32 of the integer sc*isum, |sc*isum| < 2^22: the product lands in the mantissa of 1.5 * 2^23, which is then
// subtracted -- both steps exact, so the value equals the integer-to-float conversion
BK_DEVINL float scaled_sum_f32(int sc, int isum) { return __fsub_rn(__int_as_float(sc * isum + 0x4B400000), 12582912.0f); }

// NC accumulator columns of this thread's TMEM lane, starting at column taddr; the load is complete after tmem_wait.
// No memory clobber on either: they touch tensor memory only, their order among themselves is kept by `volatile`, and
// without the clobber the compiler may move shared-memory loads of later sub-blocks across them (their latency was
// the largest stall of the scaler warps).
template <int NC>
BK_DEVINL void tmem_ld(uint32_t taddr, uint32_t (&r)[NC]) {
  if constexpr (NC == 8) {
    asm volatile("tcgen05.ld.sync.aligned.32x32b.x8.b32 {%0, %1, %2, %3, %4, %5, %6, %7}, [%8];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7])
                 : "r"(taddr));
  } else {
    asm volatile("tcgen05.ld.sync.aligned.32x32b.x4.b32 {%0, %1, %2, %3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
                 : "r"(taddr));
  }
}
// the registers are operands so that no use of them can be scheduled before the wait
template <int NC>
BK_DEVINL void tmem_wait(uint32_t (&r)[NC]) {
  if constexpr (NC == 8) {
    asm volatile("tcgen05.wait::ld.sync.aligned;"
                 : "+r"(r[0]), "+r"(r[1]), "+r"(r[2]), "+r"(r[3]), "+r"(r[4]), "+r"(r[5]), "+r"(r[6]), "+r"(r[7]));
  } else {
    asm volatile("tcgen05.wait::ld.sync.aligned;" : "+r"(r[0]), "+r"(r[1]), "+r"(r[2]), "+r"(r[3]));
  }
}

// Bounded wait whose polls may sleep: the hint lets the hardware keep the warp suspended for up to a millisecond per
// try (it wakes as soon as the phase completes), so that waiting roles do not spend issue slots on polling.  2048 tries
// bound a wait to about two seconds; the first wait of a CTA that gives up sets the status word and a flag in shared
// memory, after which every other wait of that CTA returns at once -- the kernel then runs to its end (results
// undefined, status BK_ERR_TIMEOUT) instead of timing out step after step.
BK_DEVINL void mbar_wait_idle(uint32_t bar, uint32_t parity, int* status, volatile int* dead) {
  for (int it = 0; it < 2048; it++) {
    uint32_t ok;
    asm volatile(
        "{ .reg .pred p; mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2, %3; selp.u32 %0, 1, 0, p; }"
        : "=r"(ok)
        : "r"(bar), "r"(parity), "r"(1000000u)
        : "memory");
    if (ok || *dead) return;
  }
  *dead = 1;
  if (status) atomicExch(status, 10003 /* BK_ERR_TIMEOUT */);
}

BK_DEVINL void mbar_arrive(uint32_t bar) { asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory"); }

// NC: accumulator columns per scaler thread (MMA N / 4): 4 or 8
template <int NC>
__global__ void __launch_bounds__(kUT, 1) gemv_q4k_umma_kernel(const __grid_constant__ UmmaParams P) {
  bk_pdl_trigger();
  const GemvParams& p = P.g;
  extern __shared__ __align__(1024) uint8_t smem[];
  constexpr int Npad = 4 * NC;
  uint8_t* raw = smem;                                             // [kStages][128 rows][kRowPitch]
  uint8_t* As = raw + (size_t)kStages * kStageBytes;               // [kSB][8][4096]
  uint8_t* Bs = As + kSB * 8 * 4096;                               // [kSB][8][Npad*32]
  float* scs = reinterpret_cast<float*>(Bs + kSB * 8 * 32 * 32);   // [kSB][8][d8 of 32 columns | s8 of 32 columns | pad]
  uint16_t* scm = reinterpret_cast<uint16_t*>(scs + kSB * 8 * kScsLd);   // [kSB][8][128] sc | m << 8 of (sub-block, row)
  float2* dd = reinterpret_cast<float2*>(scm + kSB * 8 * kTileM);  // [kSB][128] {d, dmin} of a row's superblock
  uint64_t* full = reinterpret_cast<uint64_t*>(dd + kSB * kTileM); // [kStages] weights of a stage have landed
  uint64_t* empty = full + kStages;                                // [kStages] every row of a stage has been unpacked (4 arrivals)
  uint64_t* ab_full = empty + kStages;                             // [kSB] tiles and tables of a step written (192 arrivals)
  uint64_t* smem_free = ab_full + kSB;                             // [kSB] the scalers are done with a shared-memory buffer (16 arrivals)
  uint64_t* mma_done = smem_free + kSB;                            // [2] the step's MMAs have completed
  uint64_t* tmem_free = mma_done + 2;                              // [2] the scalers have read an accumulator buffer (16 arrivals)
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(tmem_free + 2);
  int* last_flag = reinterpret_cast<int*>(tmem_slot + 1);   // K cut: this block arrived last at its tile's counter
  volatile int* dead = last_flag + 1;                        // a bounded wait of this CTA has given up
  float* xchg = reinterpret_cast<float*>(smem + umma_smem_core_bytes());   // [32 columns][64]: up values of a SwiGLU tile (tensor-map feed)
  const bool swiglu_halves = P.use_maps && p.segs[0].epi == BK_EPI_SWIGLU;   // tile rows 0..63 gate, 64..127 up

  const int t = threadIdx.x, warp = t >> 5, lane = t & 31;
  const int K = p.K, nsb = K / 256, nblk = K / 32;

  if (t == 0) {
    *dead = 0;
    for (int i = 0; i < kStages; i++) {
      mbar_init(smem_u32(full + i), 1);
      mbar_init(smem_u32(empty + i), kExpanderWarps);
    }
    for (int i = 0; i < kSB; i++) {
      mbar_init(smem_u32(ab_full + i), (kExpanderWarps + kStagerWarps) * 32);
      mbar_init(smem_u32(smem_free + i), kScalerWarps);
    }
    for (int i = 0; i < 2; i++) {
      mbar_init(smem_u32(mma_done + i), 1);
      mbar_init(smem_u32(tmem_free + i), kScalerWarps);
    }
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

  const int n_tiles = (p.total_vrows + kTileM - 1) / kTileM;
  const int n_chunks = (nsb + 3) / 4;
  // this CTA's tiles tile0, tile0 + tile_step, ... (n_my of them) and, of each, superblocks [s_begin, s_begin + n_s)
  int tile0 = (int)blockIdx.x, tile_step = (int)gridDim.x, s_begin = 0, n_s = nsb;
  int n_my = (n_tiles - (int)blockIdx.x + (int)gridDim.x - 1) / (int)gridDim.x;
  if (P.ksplit > 1) {
    const int part = (int)blockIdx.x % P.ksplit;
    const int c0 = part * n_chunks / P.ksplit, c1 = (part + 1) * n_chunks / P.ksplit;   // whole chunks, at least one
    tile0 = (int)blockIdx.x / P.ksplit;
    tile_step = 0;
    n_my = 1;
    s_begin = 4 * c0;
    n_s = min(nsb, 4 * c1) - s_begin;
  }
  const int npairs = (n_s + 1) / 2;
  const int G = n_my * n_s;       // superblock steps of this CTA, tile after tile
  const int Q = n_my * npairs;    // ring fills: pairs of superblock columns, never across a tile boundary

  if (warp >= kStagerWarp0 && warp < kStagerWarp0 + kStagerWarps) {
    // ================= stagers: Q8_1 activation blocks of step g -> B tiles and scales of buffer g&1 =================
    const int te = t - kStagerWarp0 * 32;
    const uint32_t* xq = reinterpret_cast<const uint32_t*>(p.x);
    // activation blocks of a superblock: Npad*8 items (column b, sub-block j); eight neighbouring threads take eight
    // neighbouring columns of one sub-block, whose 16-byte rows are contiguous in the B tile (no bank conflicts);
    // stager thread te takes items te, te + 64, ...
    constexpr int kXI = Npad * 8 / 64;   // 2 or 4
    uint32_t xw[kXI][9];
    auto load_x = [&](int s) {
#pragma unroll
      for (int i = 0; i < kXI; i++) {
        const int it = te + 64 * i, j = (it >> 3) & 7, b = (it & 7) + 8 * (it >> 6);
#pragma unroll
        for (int k = 0; k < 9; k++) xw[i][k] = b < P.B ? __ldcg(xq + ((size_t)b * nblk + (size_t)s * 8 + j) * 9 + k) : 0u;
      }
    };
    auto store_x = [&](int buf) {
#pragma unroll
      for (int i = 0; i < kXI; i++) {
        const int it = te + 64 * i, j = (it >> 3) & 7, b = (it & 7) + 8 * (it >> 6);
        uint8_t* tile_j = Bs + (size_t)buf * 8 * (Npad * 32) + (size_t)j * (Npad * 32) + (b >> 3) * 128 + (b & 7) * 16;
        *reinterpret_cast<uint4*>(tile_j) = make_uint4(xw[i][0], xw[i][1], xw[i][2], xw[i][3]);
        *reinterpret_cast<uint4*>(tile_j + Npad * 16) = make_uint4(xw[i][4], xw[i][5], xw[i][6], xw[i][7]);
        int qsum = 0;
#pragma unroll
        for (int k = 0; k < 8; k++) qsum = bk_dp4a_ss(xw[i][k], 0x01010101u, qsum);
        const float d8 = bk_q8half_to_f32((uint16_t)(xw[i][8] & 0xffffu));
        scs[(size_t)buf * 8 * kScsLd + j * kScsLd + b] = d8;
        scs[(size_t)buf * 8 * kScsLd + j * kScsLd + 32 + b] = __fmul_rn(d8, (float)qsum);
      }
    };

    bk_pdl_wait();
    load_x(s_begin);
    int s = 0;
    int buf = 0;          // shared-memory buffer g mod kSB, and the parity of its use number g / kSB
    uint32_t upar = 0;
    for (int g = 0; g < G; g++) {
      if (g >= kSB) mbar_wait_idle(smem_u32(smem_free + buf), upar ^ 1u, p.status, dead);   // the scalers have finished step g - kSB
      store_x(buf);
      s = s + 1 == n_s ? 0 : s + 1;
      if (g + 1 < G) load_x(s_begin + s);   // in flight until the next step
      asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
      mbar_arrive(smem_u32(ab_full + buf));
      if (++buf == kSB) {
        buf = 0;
        upar ^= 1u;
      }
    }
  } else if (warp == kMmaWarp) {
    // ================= MMA issue: eight MMAs, one per sub-block, into accumulator buffer g&1 =================
    // M = 128, N = Npad, int32 accumulators, A unsigned 8-bit, B signed 8-bit, both K-major
    const uint32_t idesc = (2u << 4) | (0u << 7) | (1u << 10) | ((uint32_t)(Npad >> 3) << 17) | ((uint32_t)(kTileM >> 4) << 24);
    int buf = 0;
    uint32_t upar = 0;
    for (int g = 0; g < G; g++) {
      const int tb = g & 1;   // accumulator buffer
      mbar_wait_idle(smem_u32(ab_full + buf), upar, p.status, dead);   // all 128 rows and the activations are in place
      if (g >= 2) mbar_wait_idle(smem_u32(tmem_free + tb), (uint32_t)(((g >> 1) & 1) ^ 1), p.status, dead);   // step g-2 has been read out
      if (lane == 0) {
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        const uint32_t a0 = smem_u32(As + (size_t)buf * 8 * 4096);
        const uint32_t b0 = smem_u32(Bs + (size_t)buf * 8 * (Npad * 32));
#pragma unroll
        for (int j = 0; j < 8; j++) {
          const uint64_t ad = umma_desc(a0 + j * 4096, 2048, 128);
          const uint64_t bd = umma_desc(b0 + j * (Npad * 32), (uint32_t)Npad * 16, 128);
          const uint32_t dcol = tmem + (uint32_t)(tb * 256 + j * Npad);
          asm volatile(
              "{\n\t.reg .pred pz;\n\tsetp.ne.b32 pz, %4, 0;\n\t"
              "tcgen05.mma.cta_group::1.kind::i8 [%0], %1, %2, %3, {%5, %5, %5, %5}, pz;\n\t}"
              ::"r"(dcol), "l"(ad), "l"(bd), "r"(idesc), "r"(0u), "r"(0u)
              : "memory");
        }
        asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(mma_done + tb))
                     : "memory");
      }
      __syncwarp();
      if (++buf == kSB) {
        buf = 0;
        upar ^= 1u;
      }
    }
  } else if (warp == kProducerWarp) {
    // ================= producer: fill ring stage q mod kStages with pair q (weights depend on no earlier kernel) ==========
    for (int q = 0; q < Q; q++) {
      if (q >= kStages) mbar_wait_idle(smem_u32(empty + q % kStages), (uint32_t)((q / kStages - 1) & 1), p.status, dead);
      const int tl = q / npairs, pp = q - tl * npairs;
      const int tile = tile0 + tl * tile_step;
      const uint32_t bytes = (uint32_t)((n_s - 2 * pp) >= 2 ? 288 : 144);
      const int rows_here = min(kTileM, p.total_vrows - tile * kTileM);
      const uint32_t bar = smem_u32(full + q % kStages);
      const uint32_t dst0 = smem_u32(raw + (size_t)(q % kStages) * kStageBytes);
      if (P.use_maps) {
        // lane l < 8: 32-row box l & 3 of the tile, superblock column l >> 2 of the pair
        const int k = lane & 3, sbi = lane >> 2;
        bool valid = lane < 8 && (uint32_t)sbi * 144 < bytes;
        int mi = 0, row0 = 0;
        if (swiglu_halves) {   // boxes 0, 1: gate rows tile*64 + 32k; boxes 2, 3: the same rows of the up matrix
          row0 = tile * 64 + 32 * (k & 1);
          mi = k < 2 ? 0 : 4;
          valid = valid && row0 < p.segs[0].n_rows;
        } else {
          const int v0 = tile * kTileM + 32 * k;
          valid = valid && v0 < p.total_vrows;
#pragma unroll
          for (int i = 1; i < 4; i++)
            if (i < p.n_segs && v0 >= p.segs[i].vrow_begin) mi = i;
          row0 = v0 - p.segs[mi].vrow_begin;
        }
        const unsigned n_valid = __popc(__ballot_sync(0xffffffffu, valid));
        if (lane == 0) mbar_expect_tx(bar, n_valid * 32u * 144u);
        __syncwarp();
        if (valid) {
          const int x = (s_begin + 2 * pp + sbi) * 144;
          asm volatile(
              "cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
              ::"r"(dst0 + (uint32_t)(sbi * kPlaneBytes + 32 * k * 144)), "l"(reinterpret_cast<uint64_t>(&P.maps[mi])), "r"(x), "r"(row0),
              "r"(bar)
              : "memory");
        }
        continue;
      }
      if (lane == 0) mbar_expect_tx(bar, (uint32_t)rows_here * bytes);
      __syncwarp();
#pragma unroll
      for (int k = 0; k < 4; k++) {
        const int r = lane + 32 * k;
        if (r < rows_here) bulk_g2s(dst0 + r * kRowPitch, decode_vrow(p, tile * kTileM + r).row + (size_t)s_begin * 144 + (size_t)pp * 288, bytes, bar);
      }
    }
  } else if (warp >= kScalerWarp0) {
    // ================= scalers: f32 part of step g from accumulator buffer g&1 =================
    const int row_t = t & (kTileM - 1);   // tile row (= TMEM lane) of this thread
    const int qd = (t >> 7) - kScalerWarp0 / 4;   // which quarter of the columns
    bk_pdl_wait();
    float y[NC], yc[NC];
#pragma unroll
    for (int c = 0; c < NC; c++) y[c] = yc[c] = 0.0f;
    int s = 0, tl = 0;
    int buf = 0;
    uint32_t upar = 0;
    for (int g = 0; g < G; g++) {
      const int tb = g & 1;   // accumulator buffer
      mbar_wait_idle(smem_u32(ab_full + buf), upar, p.status, dead);    // the tables of this step are visible
      mbar_wait_idle(smem_u32(mma_done + tb), (uint32_t)((g >> 1) & 1), p.status, dead);
      asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
      const float2 dm = dd[buf * kTileM + row_t];
      const float4* sb4 = reinterpret_cast<const float4*>(scs + (size_t)buf * 8 * kScsLd + qd * NC);   // d8 of this thread's columns; s8 8 float4 further
      const uint16_t* sm_ = scm + (size_t)buf * 8 * kTileM + row_t;
      const uint32_t taddr = tmem + ((uint32_t)((warp & 3) * 32) << 16) + (uint32_t)(tb * 256 + qd * NC);
      float2 accd[NC / 2], accm[NC / 2];   // columns (2i, 2i+1) side by side: one packed FMA serves both
#pragma unroll
      for (int c = 0; c < NC / 2; c++) accd[c] = accm[c] = make_float2(0.0f, 0.0f);
      uint32_t r[NC], rn[NC];
      tmem_ld<NC>(taddr, r);
      tmem_wait<NC>(r);
#pragma unroll
      for (int j = 0; j < 8; j++) {
        if (j < 7) tmem_ld<NC>(taddr + (uint32_t)((j + 1) * Npad), rn);   // in flight during this sub-block's arithmetic
        const uint32_t scmv = sm_[j * kTileM];
        const int2 s2 = make_int2((int)(scmv & 0xffu), 0);
        const float fm = __fsub_rn(__int_as_float((int)(scmv >> 8) + 0x4B400000), 12582912.0f);   // f32(m), exact
        const float2 fm2 = make_float2(fm, fm);
#pragma unroll
        for (int c = 0; c < NC; c += 4) {
          const float4 d4 = sb4[j * (kScsLd / 4) + (c >> 2)], s4 = sb4[j * (kScsLd / 4) + 8 + (c >> 2)];   // d8, s8 of columns c..c+3
          accd[c / 2] = bk_fma2(make_float2(d4.x, d4.y),
                             make_float2(scaled_sum_f32(s2.x, (int)r[c]), scaled_sum_f32(s2.x, (int)r[c + 1])), accd[c / 2]);
          accd[c / 2 + 1] = bk_fma2(make_float2(d4.z, d4.w),
                                 make_float2(scaled_sum_f32(s2.x, (int)r[c + 2]), scaled_sum_f32(s2.x, (int)r[c + 3])), accd[c / 2 + 1]);
          accm[c / 2] = bk_fma2(make_float2(s4.x, s4.y), fm2, accm[c / 2]);
          accm[c / 2 + 1] = bk_fma2(make_float2(s4.z, s4.w), fm2, accm[c / 2 + 1]);
        }
        if (j < 7) {
          tmem_wait<NC>(rn);
#pragma unroll
          for (int c = 0; c < NC; c++) r[c] = rn[c];
        }
      }
      asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
      __syncwarp();
      if (lane == 0) {   // tables and accumulators of this step may be overwritten
        mbar_arrive(smem_u32(smem_free + buf));
        mbar_arrive(smem_u32(tmem_free + tb));
      }
      if (++buf == kSB) {
        buf = 0;
        upar ^= 1u;
      }
#pragma unroll
      for (int c = 0; c < NC; c += 2) {
        yc[c] = __fadd_rn(yc[c], fmaf(dm.x, accd[c / 2].x, -__fmul_rn(dm.y, accm[c / 2].x)));
        yc[c + 1] = __fadd_rn(yc[c + 1], fmaf(dm.x, accd[c / 2].y, -__fmul_rn(dm.y, accm[c / 2].y)));
      }
      const bool last = s == n_s - 1;
      const int tile = tile0 + tl * tile_step;
      if ((s & 3) == 3 || last) {   // a chunk of four superblocks ends
        if (P.ksplit > 1) {         // its partial sums go to the scratch buffer; the last block of the tile adds them up
          float* dst = P.scratch + (((size_t)tile * n_chunks + ((s_begin + s) >> 2)) * 32 + qd * NC) * kTileM + row_t;
#pragma unroll
          for (int c = 0; c < NC; c++) {
            __stcg(dst + c * kTileM, yc[c]);
            yc[c] = 0.0f;
          }
        } else {
#pragma unroll
          for (int c = 0; c < NC; c++) {
            y[c] = __fadd_rn(y[c], yc[c]);
            yc[c] = 0.0f;
          }
        }
      }
      bool merge = true;
      if (last && P.ksplit > 1) {
        __threadfence();                                   // this thread's partial sums before the arrival
        asm volatile("bar.sync 1, %0;" ::"n"(kScalerWarps * 32) : "memory");
        if (t == kScalerWarp0 * 32) {
          const int old = atomicAdd(P.counters + tile, 1);
          if (old == P.ksplit - 1) P.counters[tile] = 0;   // everyone has arrived: ready for the next launch
          *last_flag = old == P.ksplit - 1;
        }
        asm volatile("bar.sync 1, %0;" ::"n"(kScalerWarps * 32) : "memory");
        merge = *last_flag != 0;
        if (merge) {
          __threadfence();
          const float* src = P.scratch + (((size_t)tile * n_chunks) * 32 + qd * NC) * kTileM + row_t;
          for (int ch = 0; ch < n_chunks; ch++)
#pragma unroll
            for (int c = 0; c < NC; c++) y[c] = __fadd_rn(y[c], __ldcg(src + ((size_t)ch * 32 + c) * kTileM));
        }
      }
      if (last && merge && swiglu_halves) {   // gate rows in tile rows 0..63, their up rows 64 further on (other warps)
        if (row_t >= 64) {
#pragma unroll
          for (int c = 0; c < NC; c++) xchg[(qd * NC + c) * 64 + row_t - 64] = y[c];
        }
        asm volatile("bar.sync 1, %0;" ::"n"(kScalerWarps * 32) : "memory");
        const SegDev& sg = p.segs[0];
        const int n = tile * 64 + row_t;
#pragma unroll
        for (int c = 0; c < NC; c++) {
          const int b = qd * NC + c;
          if (row_t < 64 && b < P.B && n < sg.n_rows)
            store_epilogue<false>(p, sg, (size_t)b * sg.ld_out + sg.col_off + n, y[c], xchg[b * 64 + row_t]);
          y[c] = 0.0f;
        }
        asm volatile("bar.sync 1, %0;" ::"n"(kScalerWarps * 32) : "memory");   // the values have been read: the next tile may overwrite them
        s = 0;
        tl++;
      } else if (last && merge) {   // fused epilogue of the tile; uniform over the CTA
        const int vrow = tile * kTileM + row_t;
        const bool have_row = vrow < p.total_vrows;
        VRow vr = {nullptr, 0, 0};
        if (have_row) vr = decode_vrow(p, vrow);
        const SegDev& sg = p.segs[vr.si];
        const bool swiglu = have_row && sg.epi == BK_EPI_SWIGLU;
#pragma unroll
        for (int c = 0; c < NC; c++) {
          const int b = qd * NC + c;
          const float yup = __shfl_xor_sync(0xffffffffu, y[c], 1);   // the odd neighbour row: the "up" row of a SwiGLU pair
          if (b < P.B && have_row && !(swiglu && (row_t & 1)))
            store_epilogue<false>(p, sg, (size_t)b * sg.ld_out + sg.col_off + vr.n, y[c], yup);
          y[c] = 0.0f;
        }
        s = 0;
        tl++;
      } else {
        s++;
      }
    }
  } else {
    // ================= expanders: unpacking, scale tables =================
    const int te = t;                 // tile row of this thread
    bk_pdl_wait();
    int s = 0, tl = 0;
    int buf = 0;
    uint32_t upar = 0;
    for (int g = 0; g < G; g++) {
      const int q = tl * npairs + (s >> 1);
      const int stage = q % kStages;
      if ((s & 1) == 0) mbar_wait_idle(smem_u32(full + stage), (uint32_t)((q / kStages) & 1), p.status, dead);
      if (g >= kSB) mbar_wait_idle(smem_u32(smem_free + buf), upar ^ 1u, p.status, dead);   // the scalers have finished step g - kSB
      const int s_next = s + 1 == n_s ? 0 : s + 1;
      // header -> scale table; 4-bit quants -> unsigned int8 rows, sub-block 2p from the low nibbles of group p,
      //     2p+1 from the high nibbles
      const uint8_t* rw = raw + (size_t)stage * kStageBytes +
                          (P.use_maps ? (size_t)(s & 1) * kPlaneBytes + (size_t)te * 144 : (size_t)te * kRowPitch + (s & 1) * 144);
      const uint4 hdr = *reinterpret_cast<const uint4*>(rw);
      dd[buf * kTileM + te] = make_float2(bk_f16_to_f32((uint16_t)(hdr.x & 0xffffu)), bk_f16_to_f32((uint16_t)(hdr.x >> 16)));
      uint16_t* sm_w = scm + (size_t)buf * 8 * kTileM + te;
      uint8_t* Ab = As + (size_t)buf * 8 * 4096 + (te >> 3) * 128 + (te & 7) * 16;
      uint4 qv[8];
#pragma unroll
      for (int k = 0; k < 8; k++) qv[k] = *reinterpret_cast<const uint4*>(rw + 16 + 16 * k);
      if ((s & 1) || s == n_s - 1) {   // this warp's rows of the stage are in registers: hand the stage back
        __syncwarp();
        if (lane == 0) mbar_arrive(smem_u32(empty + stage));
      }
#pragma unroll
      for (int pq = 0; pq < 4; pq++) {
        uint32_t sc2, mn2;
        bk_q4k_scale_min_pair(hdr.y, hdr.z, hdr.w, pq, sc2, mn2);
        sm_w[(2 * pq) * kTileM] = (uint16_t)((sc2 & 0xffu) | ((mn2 & 0xffu) << 8));
        sm_w[(2 * pq + 1) * kTileM] = (uint16_t)((sc2 >> 8) | (mn2 & 0xff00u));
        const uint4 qa = qv[2 * pq], qb = qv[2 * pq + 1];
        uint8_t* A0 = Ab + (size_t)(2 * pq) * 4096;
        *reinterpret_cast<uint4*>(A0) = make_uint4(qa.x & 0x0f0f0f0fu, qa.y & 0x0f0f0f0fu, qa.z & 0x0f0f0f0fu, qa.w & 0x0f0f0f0fu);
        *reinterpret_cast<uint4*>(A0 + 2048) = make_uint4(qb.x & 0x0f0f0f0fu, qb.y & 0x0f0f0f0fu, qb.z & 0x0f0f0f0fu, qb.w & 0x0f0f0f0fu);
        *reinterpret_cast<uint4*>(A0 + 4096) =
            make_uint4((qa.x >> 4) & 0x0f0f0f0fu, (qa.y >> 4) & 0x0f0f0f0fu, (qa.z >> 4) & 0x0f0f0f0fu, (qa.w >> 4) & 0x0f0f0f0fu);
        *reinterpret_cast<uint4*>(A0 + 4096 + 2048) =
            make_uint4((qb.x >> 4) & 0x0f0f0f0fu, (qb.y >> 4) & 0x0f0f0f0fu, (qb.z >> 4) & 0x0f0f0f0fu, (qb.w >> 4) & 0x0f0f0f0fu);
      }
      asm volatile("fence.proxy.async.shared::cta;" ::: "memory");   // the MMA reads shared memory through the async proxy
      mbar_arrive(smem_u32(ab_full + buf));
      if (++buf == kSB) {
        buf = 0;
        upar ^= 1u;
      }
      s = s_next;
      if (s == 0) tl++;
    }
  }

  // ---- release tensor memory (every thread gets here, whatever happened above) ----
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  if (warp == 0) {
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(kTmemCols) : "memory");
  }
}

size_t umma_smem_bytes() { return umma_smem_core_bytes() + 32 * 64 * sizeof(float); }

// cuTensorMapEncodeTiled, looked up through the runtime so that the library needs no link against the driver
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                  const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
EncodeTiledFn encode_tiled_fn() {
  static EncodeTiledFn fn = nullptr;
  static bool looked = false;
  if (!looked) {
    void* ptr = nullptr;
    cudaDriverEntryPointQueryResult qr;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &qr) == cudaSuccess && qr == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeTiledFn>(ptr);
    looked = true;
  }
  return fn;
}

// uint8 matrix [n_rows][row_bytes], box = 32 rows x 144 bytes (one superblock column of 32 rows), no swizzle
bool encode_weight_map(CUtensorMap* m, const uint8_t* W, int n_rows, size_t row_bytes) {
  EncodeTiledFn fn = encode_tiled_fn();
  if (!fn || (reinterpret_cast<uintptr_t>(W) & 15) || row_bytes % 16) return false;
  const cuuint64_t dims[2] = {(cuuint64_t)row_bytes, (cuuint64_t)n_rows};
  const cuuint64_t strides[1] = {(cuuint64_t)row_bytes};
  const cuuint32_t box[2] = {144, 32};
  const cuuint32_t estr[2] = {1, 1};
  return fn(m, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<uint8_t*>(W), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
            CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
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
  // tensor-map feed: whole rows in memory, 32-row boxes that never straddle two segments, and a SwiGLU segment alone
  {
    const GemvParams& g = P.g;
    bool ok = g.row_stride == 0 && g.row_off == 0;
    bool any_swiglu = false;
    for (int i = 0; i < g.n_segs; i++) {
      ok = ok && g.segs[i].n_rows % 32 == 0;
      any_swiglu = any_swiglu || g.segs[i].epi == BK_EPI_SWIGLU;
    }
    ok = ok && (!any_swiglu || g.n_segs == 1);
    const size_t row_bytes = (size_t)(g.K / 256) * 144;
    for (int i = 0; ok && i < g.n_segs; i++) {
      ok = encode_weight_map(&P.maps[i], g.segs[i].W, g.segs[i].n_rows, row_bytes);
      if (ok && g.segs[i].epi == BK_EPI_SWIGLU) ok = encode_weight_map(&P.maps[4], g.segs[i].W2, g.segs[i].n_rows, row_bytes);
    }
    P.use_maps = ok ? 1 : 0;
  }
  static bool configured = false;
  const size_t smem = umma_smem_bytes();
  if (!configured) {
    BK_CUDA(cudaFuncSetAttribute(gemv_q4k_umma_kernel<4>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    BK_CUDA(cudaFuncSetAttribute(gemv_q4k_umma_kernel<8>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    configured = true;
  }
  const int tiles = (P.g.total_vrows + kTileM - 1) / kTileM;
  int grid = tiles < c.sm_count ? tiles : c.sm_count;
  // few tiles: cut each along K into parts of whole chunks (four superblocks), as many as there are SMs for
  const int n_chunks = (P.g.K / 256 + 3) / 4;
  P.ksplit = 1;
  P.scratch = c.tile_scratch;
  P.counters = c.tile_counters;
  if (tiles * 2 <= c.sm_count && n_chunks >= 2 && tiles <= 256 &&
      (size_t)tiles * n_chunks * 32 * kTileM * sizeof(float) <= c.tile_scratch_bytes) {
    P.ksplit = c.sm_count / tiles < n_chunks ? c.sm_count / tiles : n_chunks;
    if (P.ksplit > 1) grid = tiles * P.ksplit;
  }
  if (P.Npad == 16) BK_CUDA(bk_launch_pdl(gemv_q4k_umma_kernel<4>, dim3(grid), dim3(kUT), smem, P));
  else BK_CUDA(bk_launch_pdl(gemv_q4k_umma_kernel<8>, dim3(grid), dim3(kUT), smem, P));
  BK_CHECK_LAUNCH();
  return BK_OK;
}
