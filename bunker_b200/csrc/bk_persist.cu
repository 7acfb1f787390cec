// bk_persist.cu -- the batch-1 decode step as a persistent kernel: one cooperative launch of one CTA per SM runs a
// list of phases (projection GEMVs, conv1d + gated-DeltaNet steps, lm_head + argmax) separated by device-side grid
// barriers, instead of one launch per op.
//
// Replaces the launch loop of bunker's executor (runGraphDecode, src/runner.ts:133-160: ~287 cuLaunch calls per token,
// LOG.md:580,712) on the single-GPU, single-sequence path.  The arithmetic of every phase is the per-op kernels' own
// (bk_gemv_dp4a.cuh, bk_gemv_shared.cuh, bk_gdn.cuh), so results are bit-identical to the per-op step.
//
// Weight stream.  Every warp owns a byte ring in shared memory and walks the list of its row groups over ALL phases
// of the launch: lane 0 requests a group with one bulk async copy per contiguous run of rows (cp.async.bulk, completion
// on an mbarrier) as soon as the ring has room, so the weights of the next phases are in flight or resident while the
// current phase computes and while the grid waits at a barrier.  Weights depend on nothing, only activations do.
//
// Grid barrier.  flags[c] = generation, one word per CTA; a CTA stores its word after its phase (release) and warp 0
// polls all words (bounded: a barrier that never completes sets the status word, the CTA drains its copies and
// returns).  The launch is cooperative, so all CTAs are resident and waiting inside one launch is legal.
// Activations written by other CTAs of the launch are read past L1 (ld.global.cg).
#include <string.h>

#include <vector>

#include "bk_gemv_dp4a.cuh"
#include "bk_gdn.cuh"

namespace {

constexpr int kPW = 16;            // warps per CTA
constexpr int kPT = kPW * 32;
constexpr int kRingBars = 8;       // row groups a warp may have requested and not yet consumed
constexpr int kMaxK = 8192;        // widest activation row the staging area holds
constexpr int kBarrierPolls = 1 << 21;
constexpr int kDescSlots = 8;      // phase descriptors kept in shared memory: the current phase and the next six valid,
                                   // the seventh being copied

enum { PH_GEMV = 1, PH_GDN = 2 };

struct __align__(16) Phase {
  int type, flags, pad0, pad1;
  GemvParams g;
  GdnParams d;
};

struct StepIO {
  const uint8_t* embed;   // tied Q4_K table (BK_PF_EMBED)
  const int32_t* ids_in;  // token of this step (device or mapped host memory)
  uint16_t* x0;           // residual stream buffer that receives the embedded row
  int H;
  // argmax tail (BK_PF_ARGMAX)
  float* part_v;
  int32_t* part_i;
  unsigned int* counter;
  int32_t* ids_out;
  float* val_out;
  int32_t* pos;
  int32_t* hist;
  int hist_ld, hist_rows;
  int32_t* host_out;
  int vocab_offset;
};

struct PersistParams {
  const Phase* phases;
  int first, count;
  unsigned int* flags;
  unsigned int* epoch;
  unsigned int* counter;        // barrier_mode 1: monotonic arrival counter and the value it had when the launch began
  unsigned int* counter_base;
  int barrier_mode;
  int barrier_polls;            // polls before a barrier gives up
  int* status;
  unsigned long long* trace;   // 8 slots per phase of the plan, or null
  uint32_t ring_bytes;         // per warp
  uint32_t scratch_bytes;
  StepIO io;
};

// shared memory carve-up, the same on host and device
struct SmemLayout {
  size_t desc, xs, d8s, s8s, red, bars, ent, misc, scratch, ring, total;
};
__host__ __device__ inline SmemLayout smem_layout(uint32_t scratch_bytes, uint32_t ring_bytes) {
  SmemLayout L;
  size_t o = 0;
  L.desc = o; o += kDescSlots * ((sizeof(Phase) + 127) & ~(size_t)127);
  L.xs = o; o += (size_t)kMaxK / 64 * kUnitWords * 4;
  L.d8s = o; o += (size_t)kMaxK / 32 * 4;
  L.s8s = o; o += (size_t)kMaxK / 32 * 4;
  L.red = o; o += 128;
  L.bars = o; o += (size_t)kPW * kRingBars * 8;
  L.ent = o; o += (size_t)kPW * kRingBars * 8;
  L.misc = o; o += 256;
  L.scratch = o; o += (scratch_bytes + 127) & ~(size_t)127;
  L.ring = o; o += (size_t)kPW * ring_bytes;
  L.total = o;
  return L;
}

struct Ring {
  uint32_t base, bar0, size, head, used, issued, consumed;
  int pp, pg, end;                 // producer cursor: phase (absolute index), group of this CTA; end of the launch
  int G, ngroups, nrows, c0;       // geometry of phase pp for this CTA
  uint32_t rowb;
  bool ready;                      // the cursor stands on a group that can be requested
};

// descriptor of phase pp (absolute index) in the shared-memory window
struct DescWin {
  const uint8_t* base;
  size_t stride;
  __device__ __forceinline__ const Phase& at(int pp) const {
    return *reinterpret_cast<const Phase*>(base + (size_t)(pp & (kDescSlots - 1)) * stride);
  }
};

// position the producer on the first phase >= R.pp in which this warp has a row group (never beyond `limit`, the
// last phase whose descriptor is in the window)
__device__ __forceinline__ void ring_seek(Ring& R, const DescWin& win, int limit, int warp) {
  R.ready = false;
  while (R.pp < R.end && R.pp <= limit) {
    const Phase& ph = win.at(R.pp);
    if (ph.type == PH_GEMV) {
      const int rpc = ph.g.rows_per_cta;
      const int c0 = blockIdx.x * rpc;
      const int nrows = min(ph.g.total_vrows, c0 + rpc) - c0;
      if (nrows > 0) {
        const int G = ph.g.group_rows;
        const int ngroups = (nrows + G - 1) / G;
        if (warp < ngroups) {
          R.G = G;
          R.ngroups = ngroups;
          R.nrows = nrows;
          R.c0 = c0;
          R.rowb = (uint32_t)(ph.g.K / 256) * 144;
          R.pg = warp;
          R.ready = true;
          return;
        }
      }
    }
    R.pp++;
  }
}

// request as many of this warp's next groups as the ring and its mbarriers have room for
__device__ __forceinline__ void ring_fill(Ring& R, const DescWin& win, int limit, uint32_t* ent, int warp, int lane) {
  if (!R.ready) ring_seek(R, win, limit, warp);
  while (R.ready && R.issued - R.consumed < (uint32_t)kRingBars) {
    const int nr = min(R.G, R.nrows - R.pg * R.G);
    const uint32_t bytes = (uint32_t)nr * R.rowb;
    if (R.used == 0) R.head = 0;
    uint32_t off = R.head, pad = 0;
    if (off + bytes > R.size) {   // does not fit before the end: skip the tail, place at the start
      pad = R.size - off;
      off = 0;
    }
    if (R.used + pad + bytes > R.size) break;
    const uint32_t e = R.issued % kRingBars;
    if (lane == 0) {
      ent[2 * e] = off;
      ent[2 * e + 1] = pad + bytes;
      request_group(win.at(R.pp).g, R.c0 + R.pg * R.G, nr, R.rowb, R.base + off, R.bar0 + 8 * e);
    }
    R.head = off + bytes;
    R.used += pad + bytes;
    R.issued++;
    R.pg += kPW;
    if (R.pg >= R.ngroups) {
      R.pp++;
      ring_seek(R, win, limit, warp);
    }
  }
  __syncwarp();
}

BK_DEVINL unsigned int ld_relaxed_gpu(const unsigned int* p) {
  unsigned int v;
  asm volatile("ld.relaxed.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
// bounded wait for a requested row group; gives up early once the status word is set (some wait already failed)
BK_DEVINL bool wait_group(uint32_t bar, uint32_t parity, int* status) {
  for (int it = 0; it < (1 << 20); it++) {
    if (mbar_try_wait(bar, parity)) return true;
    if ((it & 1023) == 1023 && *reinterpret_cast<volatile int*>(status) != 0) return false;
  }
  atomicExch(status, BK_ERR_TIMEOUT);
  return false;
}
// On the way out after a failed barrier: the copies this warp has requested must have landed before the CTA may
// exit (they write its shared memory), whatever the status word says.  Bounded all the same.
BK_DEVINL void drain_group(uint32_t bar, uint32_t parity) {
  for (int it = 0; it < (1 << 22); it++)
    if (mbar_try_wait(bar, parity)) return;
}
BK_DEVINL unsigned long long global_timer() {
  unsigned long long t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}

// All CTAs of the launch meet.  Warp kPW-1 publishes this CTA's arrival and polls; the other warps use the wait to
// request the weight groups their rings have room for.  Returns false when the barrier gave up (status word set):
// the caller must leave.
// mode 0: one word per CTA (flags[c] = generation), the poller reads all of them.
// mode 1: one counter, an atomic add per CTA, the poller reads that word (target = base + (k+1) * CTAs).
__device__ __forceinline__ bool grid_barrier(const PersistParams& P, unsigned int gen, unsigned int target, int* s_abort,
                                             unsigned long long* trec, Ring& R, const DescWin& win, int limit, uint32_t* ent) {
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  __syncthreads();   // every warp of this CTA has finished the phase (and its global stores precede the release below)
  if (warp == kPW - 1) {
    if (lane == 0) {
      if (trec) atomicMax(trec + 3, global_timer());   // latest CTA to finish the phase
      __threadfence();
      if (P.barrier_mode == 0) asm volatile("st.release.gpu.global.u32 [%0], %1;" ::"l"(P.flags + blockIdx.x), "r"(gen) : "memory");
      else atomicAdd(P.counter, 1u);
    }
    __syncwarp();
  }
  if (warp == kPW - 1) {
    bool ok = false;
    for (int it = 0; it < P.barrier_polls; it++) {
      unsigned int behind = 0;   // all loads of a poll are in flight together
      if (P.barrier_mode == 0) {
        for (int i = lane; i < (int)gridDim.x; i += 32) behind |= (ld_relaxed_gpu(P.flags + i) - gen) >> 31;
      } else {
        if (lane == 0) behind = (ld_relaxed_gpu(P.counter) - target) >> 31;
      }
      if (__all_sync(0xffffffffu, behind == 0)) {
        ok = true;
        break;
      }
      // another CTA gave up: stop waiting for it (checked only long after any healthy barrier has completed)
      if (it >= 1024 && (it & 1023) == 0) {   // warp-uniform condition: the vote below is taken by all lanes
        const int st = *reinterpret_cast<volatile int*>(P.status);
        if (__any_sync(0xffffffffu, st != 0)) break;
      }
    }
    __threadfence();   // acquire: what the other CTAs wrote before their release is visible to this CTA from here
    if (lane == 0) {
      if (!ok) atomicExch(P.status, BK_ERR_TIMEOUT);
      *s_abort = ok ? 0 : 1;
    }
  }
  __syncthreads();
  return *s_abort == 0;
}

__device__ __forceinline__ void argmax_merge_p(float& v, int& i, float ov, int oi) {
  if (ov > v || (ov == v && oi < i)) {
    v = ov;
    i = oi;
  }
}

__global__ void __launch_bounds__(kPT, 1) decode_persist_kernel(const PersistParams P) {
  extern __shared__ __align__(128) uint8_t smem[];
  const SmemLayout L = smem_layout(P.scratch_bytes, P.ring_bytes);
  const size_t desc_stride = (sizeof(Phase) + 127) & ~(size_t)127;
  uint32_t* xs = reinterpret_cast<uint32_t*>(smem + L.xs);
  float* d8s = reinterpret_cast<float*>(smem + L.d8s);
  float* s8s = reinterpret_cast<float*>(smem + L.s8s);
  float* red = reinterpret_cast<float*>(smem + L.red);
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + L.bars);
  int* misc = reinterpret_cast<int*>(smem + L.misc);   // [0] abort flag, [8..24) argmax values, [24..40) indices
  uint8_t* scratch = smem + L.scratch;

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  uint32_t* ent = reinterpret_cast<uint32_t*>(smem + L.ent) + warp * kRingBars * 2;
  const unsigned int ep = *reinterpret_cast<const volatile unsigned int*>(P.epoch);
  const unsigned int cbase = *reinterpret_cast<const volatile unsigned int*>(P.counter_base);
  unsigned long long* const trace = (P.trace && blockIdx.x == 0 && tid == 0) ? P.trace : nullptr;
  const DescWin win = {smem + L.desc, desc_stride};
  const int last_phase = P.first + P.count - 1;

  // descriptors of the first phases of the launch
  auto copy_desc = [&](int pp) {
    const uint4* src = reinterpret_cast<const uint4*>(P.phases + pp);
    uint4* dst = reinterpret_cast<uint4*>(smem + L.desc + (size_t)(pp & (kDescSlots - 1)) * desc_stride);
    for (int i = tid; i < (int)(sizeof(Phase) / 16); i += kPT) dst[i] = src[i];
  };
  for (int pp = P.first; pp <= last_phase && pp < P.first + kDescSlots - 1; pp++) copy_desc(pp);

  // ---- weight ring of this warp ----
  Ring R;
  R.base = smem_u32(smem + L.ring + (size_t)warp * P.ring_bytes);
  R.bar0 = smem_u32(bars + warp * kRingBars);
  R.size = P.ring_bytes;
  R.head = R.used = R.issued = R.consumed = 0;
  R.pp = P.first;
  R.end = P.first + P.count;
  R.pg = 0;
  R.G = R.ngroups = R.nrows = R.c0 = 0;
  R.rowb = 0;
  R.ready = false;
  if (lane == 0) {
    for (int e = 0; e < kRingBars; e++) mbar_init(R.bar0 + 8 * e, 1);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
  }
  uint4 wpre = make_uint4(0, 0, 0, 0);
  {
    const Phase& f = P.phases[P.first];
    if (f.type == PH_GEMV && f.g.prologue == BK_PRO_RMSNORM && tid < f.g.K / 8)
      wpre = __ldg(reinterpret_cast<const uint4*>(f.g.norm_w) + tid);
  }
  __syncthreads();
  ring_fill(R, win, P.first + kDescSlots - 2, ent, warp, lane);
  const uint8_t* ring_mem = smem + L.ring + (size_t)warp * P.ring_bytes;

  float best_v = -INFINITY;
  int best_i = 0x7fffffff;
  bool has_argmax = false;
  bool dead = false;   // a wait for weights gave up: no further row groups are consumed by this warp

  for (int k = 0; k < P.count; k++) {
    const int cur = P.first + k;
    const int limit = cur + kDescSlots - 2;   // last phase whose descriptor is valid in the window during this phase
    Phase& ph = *reinterpret_cast<Phase*>(smem + L.desc + (size_t)(cur & (kDescSlots - 1)) * desc_stride);
    unsigned long long* trec = P.trace ? P.trace + (size_t)cur * 8 : nullptr;
    if (trace) trec[0] = global_timer();
    // one more descriptor into the slot the previous phase has left (valid after the next barrier)
    if (cur + kDescSlots - 1 <= last_phase) copy_desc(cur + kDescSlots - 1);

    if (ph.type == PH_GEMV) {
      const GemvParams& p = ph.g;
      const bool embed = (ph.flags & BK_PF_EMBED) != 0;
      if (embed) {
        // the token's row of the tied table, dequantised by every CTA for itself; CTA 0 also stores it as the
        // residual stream
        uint16_t* erow = reinterpret_cast<uint16_t*>(scratch);
        const int id = P.io.ids_in[0];
        const uint8_t* row = P.io.embed + (size_t)id * (P.io.H / 256) * 144;
        for (int u = tid; u < P.io.H / 64; u += kPT) bk_q4k_unit_to_bf16(row, u, erow + (size_t)u * 64);
        if (tid == 0) ph.g.x = erow;
        __syncthreads();
        if (blockIdx.x == 0)
          for (int q = tid; q < P.io.H / 8; q += kPT)
            reinterpret_cast<uint4*>(P.io.x0)[q] = reinterpret_cast<const uint4*>(erow)[q];
      }
      if (p.prologue == BK_PRO_RMSNORM) {
        if (embed) prologue_bf16<true, 0>(p, 1, xs, d8s, s8s, red, wpre);
        else prologue_bf16<true, 3>(p, 1, xs, d8s, s8s, red, wpre);
      } else {
        prologue_bf16<false, 3>(p, 1, xs, d8s, s8s, red, wpre);
      }
      __syncthreads();
      if (trace) trec[1] = global_timer();
      // The activation is staged: from here to the end of the phase this CTA needs nothing from global memory, so this
      // is where the weights of the coming phases are requested (not during the barrier or the activation loads,
      // whose latency the burst would stretch).
      ring_fill(R, win, limit, ent, warp, lane);

      const int K = p.K, nunits = K / 64, nblk = K / 32;
      const int c0 = blockIdx.x * p.rows_per_cta;
      const int n_rows_cta = max(0, min(p.total_vrows, c0 + p.rows_per_cta) - c0);
      const int G = p.group_rows;
      const int n_groups = (n_rows_cta + G - 1) / G;
      const uint32_t rowb = (uint32_t)(K / 256) * 144;
      const int ri = ((lane >> 4) & 1) * 4 + ((lane >> 3) & 1) * 2 + ((lane >> 2) & 1);  // row this lane reports
      const bool swiglu = p.segs[0].epi == BK_EPI_SWIGLU;
      const bool argmax = (ph.flags & BK_PF_ARGMAX) != 0;
      has_argmax = has_argmax || argmax;
      for (int g = warp; g < n_groups && !dead; g += kPW) {
        const int nr = min(G, n_rows_cta - g * G);
        const uint32_t e = R.consumed % kRingBars;
        const uint32_t parity = (R.consumed / kRingBars) & 1u;
        const uint32_t off = ent[2 * e], fp = ent[2 * e + 1];
        if (!wait_group(R.bar0 + 8 * e, parity, P.status)) {
          // the weights did not arrive (or another wait already failed): this warp stops consuming; the next barrier
          // sees the status word and winds the launch down
          dead = true;
          break;
        }
        if (trace && g == warp) trec[4] = global_timer();
        const uint8_t* wbase = ring_mem + off;
        float acc[8];
#pragma unroll
        for (int r = 0; r < 8; r++) acc[r] = 0.0f;
        for (int u = lane; u < nunits; u += 32) {
          const int pp = u & 3;
          const XRegs xr = load_x(xs, d8s, s8s, 0, u, nunits, nblk);
#pragma unroll
          for (int r = 0; r < 8; r++) {
            if (r < nr) {
              const WRegs w = decode_unit(load_unit_smem(wbase + slot_row(swiglu, r, nr) * rowb, u), pp);
              acc[r] = __fadd_rn(acc[r], unit_val(w, xr));
            }
          }
        }
        __syncwarp();   // every lane has consumed the group
        if (trace && g == warp) trec[5] = global_timer();
        R.used -= fp;
        R.consumed++;
        // more groups of this phase to come: keep the ring full; after the last one the refill waits for the next phase
        if (g + kPW < n_groups) ring_fill(R, win, limit, ent, warp, lane);
        const int v = c0 + g * G + ri;
        const bool mine = (lane & 3) == 0 && ri < nr;
        VRow vr = {nullptr, 0, 0};
        if (mine) vr = decode_vrow(p, v);
        const SegDev& sg = p.segs[vr.si];
        if (trace && g == warp) trec[6] = global_timer();
        const float y = warp_sum8(acc);
        const float yup = __shfl_xor_sync(0xffffffffu, y, 4);   // the odd neighbour row (the "up" row of a SwiGLU pair)
        if (mine && !(sg.epi == BK_EPI_SWIGLU && (ri & 1))) {
          store_epilogue<false, true>(p, sg, (size_t)sg.col_off + vr.n, y, yup);
          if (argmax) argmax_merge_p(best_v, best_i, y, P.io.vocab_offset + vr.n);
        }
        if (trace && g == warp) trec[7] = global_timer();
      }
    } else if (ph.type == PH_GDN) {
      const GdnParams& d = ph.d;
      GdnSmem& gsm = *reinterpret_cast<GdnSmem*>(scratch);
      ring_fill(R, win, limit, ent, warp, lane);
      for (int i = blockIdx.x; i < d.Hv * d.B; i += gridDim.x) {
        gdn_step_body<false, true>(d, gsm, i % d.Hv, i / d.Hv);
        __syncthreads();
      }
      if (trace) trec[1] = global_timer();
    }
    if (trace) trec[2] = global_timer();
    if (trec && tid == 0 && cur == last_phase) atomicMax(trec + 3, global_timer());

    if (cur < last_phase) {
      const Phase& nx = win.at(cur + 1);
      if (nx.type == PH_GEMV && nx.g.prologue == BK_PRO_RMSNORM && tid < nx.g.K / 8)
        wpre = __ldg(reinterpret_cast<const uint4*>(nx.g.norm_w) + tid);
      const unsigned int gen = ep * 4096u + (unsigned int)k + 1u;
      const unsigned int target = cbase + (unsigned int)(k + 1) * gridDim.x;
      if (!grid_barrier(P, gen, target, misc, trec, R, win, limit + 1, ent)) {
        // leave: wait (bounded) for the copies this warp still has in flight, then return
        while (R.consumed != R.issued) {
          drain_group(R.bar0 + 8 * (R.consumed % kRingBars), (R.consumed / kRingBars) & 1u);
          R.consumed++;
        }
        return;
      }
    }
  }

  while (dead && R.consumed != R.issued) {
    drain_group(R.bar0 + 8 * (R.consumed % kRingBars), (R.consumed / kRingBars) & 1u);
    R.consumed++;
  }

  // ---- argmax over the lm_head rows of this launch: per CTA, then the CTA that arrives last merges ----
  if (has_argmax) {
    for (int off = 16; off >= 1; off >>= 1) {
      const float ov = __shfl_xor_sync(0xffffffffu, best_v, off);
      const int oi = __shfl_xor_sync(0xffffffffu, best_i, off);
      argmax_merge_p(best_v, best_i, ov, oi);
    }
    float* sv = reinterpret_cast<float*>(misc + 8);
    int* si = misc + 8 + kPW;
    if (lane == 0) {
      sv[warp] = best_v;
      si[warp] = best_i;
    }
    __syncthreads();
    if (tid == 0) {
      for (int w = 1; w < kPW; w++) argmax_merge_p(best_v, best_i, sv[w], si[w]);
      P.io.part_v[blockIdx.x] = best_v;
      P.io.part_i[blockIdx.x] = best_i;
      __threadfence();
      const unsigned int done = atomicAdd(P.io.counter, 1u);
      if (done == gridDim.x - 1) {
        __threadfence();
        const volatile float* pv = P.io.part_v;
        const volatile int32_t* pi = P.io.part_i;
        float v = -INFINITY;
        int i = 0x7fffffff;
        for (unsigned c = 0; c < gridDim.x; c++) argmax_merge_p(v, i, pv[c], pi[c]);
        if (i == 0x7fffffff) i = 0;
        P.io.ids_out[0] = i;
        P.io.val_out[0] = v;
        if (P.io.host_out) {   // pinned host memory mapped into the device
          P.io.host_out[0] = i;
          P.io.host_out[1] = __float_as_int(v);
        }
        *P.io.counter = 0;
        if (P.io.pos) {
          const int pcur = P.io.pos[0];
          if (P.io.hist && pcur < P.io.hist_rows) P.io.hist[(size_t)pcur * P.io.hist_ld] = i;
          P.io.pos[0] = pcur + 1;
        }
      }
    }
  }
  // The next launch needs a new generation / counter base.  Every CTA has read the old ones: it has passed this
  // launch's barriers, or the launch has none.
  if (blockIdx.x == 0 && tid == 0) {
    *P.epoch = ep + 1;
    *P.counter_base = cbase + (unsigned int)(P.count - 1) * gridDim.x;
  }
}

struct Plan {
  std::vector<Phase> ph[2];   // conv-state parity 0 / 1
  Phase* d_ph[2] = {nullptr, nullptr};
  unsigned int* d_flags = nullptr;   // [grid] barrier words, then the epoch word, then the argmax counter
  float* d_part_v = nullptr;
  int32_t* d_part_i = nullptr;
  int grid = 0;
  uint32_t ring_bytes = 0, scratch_bytes = 0;
  size_t smem = 0;
  bool finished = false;
};

Plan* as_plan(uint64_t h) { return reinterpret_cast<Plan*>(static_cast<uintptr_t>(h)); }

}  // namespace

int32_t bk_plan_create(uint64_t* out, int hidden) {
  BkContext& c = bk_ctx();
  BK_ARG(out && hidden > 0 && hidden % 256 == 0 && hidden <= kMaxK, "step plan: hidden=%d unsupported", hidden);
  Plan* pl = new Plan();
  pl->grid = c.sm_count;
  size_t scratch = sizeof(GdnSmem);
  if ((size_t)hidden * 2 > scratch) scratch = (size_t)hidden * 2;
  pl->scratch_bytes = (uint32_t)scratch;
  const size_t fixed = smem_layout(pl->scratch_bytes, 0).total;
  const size_t limit = c.smem_optin;
  if (fixed + (size_t)kPW * 4096 > limit) {
    delete pl;
    return bk_fail(BK_ERR_UNSUPPORTED, "step plan: %zu bytes of shared memory leave no room for the weight rings", limit);
  }
  pl->ring_bytes = (uint32_t)(((limit - fixed) / kPW) & ~(size_t)127);
  pl->smem = smem_layout(pl->scratch_bytes, pl->ring_bytes).total;
  *out = (uint64_t)(uintptr_t)pl;
  return BK_OK;
}

bool bk_plan_gemv_fits(uint64_t plan, int K) {
  Plan* pl = as_plan(plan);
  return pl && K > 0 && K % 256 == 0 && K <= kMaxK && (size_t)(K / 256) * 144 * 2 <= pl->ring_bytes;
}

int32_t bk_plan_add_gemv(uint64_t plan, const bkGemvArgs& a, int flags) {
  Plan* pl = as_plan(plan);
  BK_ARG(pl && !pl->finished, "step plan: closed");
  BK_ARG(a.B == 1, "step plan: batch %d (the persistent step is a batch-1 path)", a.B);
  BK_ARG(bk_plan_gemv_fits(plan, a.K), "step plan: K=%d does not fit", a.K);
  BK_ARG(a.prologue == BK_PRO_RMSNORM || a.prologue == BK_PRO_BF16, "step plan: prologue %d unsupported", a.prologue);
  BK_ARG(a.n_segs >= 1 && a.n_segs <= 4, "step plan: n_segs=%d", a.n_segs);
  BK_ARG((flags & BK_PF_EMBED) || (a.x != 0 && (a.x & 15) == 0), "step plan: x must be a 16-byte aligned device pointer");
  if (a.prologue == BK_PRO_RMSNORM) BK_ARG(a.norm_w != 0 && (a.norm_w & 15) == 0, "step plan: norm_w missing or misaligned");
  Phase ph;
  memset(&ph, 0, sizeof(ph));
  ph.type = PH_GEMV;
  ph.flags = flags;
  GemvParams& p = ph.g;
  p.K = a.K;
  p.n_segs = a.n_segs;
  p.prologue = a.prologue;
  p.x = bk_ptr<void>(a.x);
  p.norm_w = bk_ptr<uint16_t>(a.norm_w);
  p.eps = a.eps;
  p.status = bk_ctx().d_status;
  int vrows = 0;
  bool has_swiglu = false;
  for (int s = 0; s < 4; s++) {
    SegDev& d = p.segs[s];
    if (s >= a.n_segs) {
      d = SegDev{nullptr, nullptr, nullptr, nullptr, 0, 0, 0, 0, 0x7fffffff};
      continue;
    }
    const bkGemvSeg& g = a.segs[s];
    BK_ARG(g.n_rows > 0 && g.W != 0 && (g.W & 15) == 0 && g.out != 0, "step plan: segment %d is malformed", s);
    BK_ARG(g.epilogue >= BK_EPI_F32 && g.epilogue <= BK_EPI_SWIGLU, "step plan: segment %d epilogue %d", s, g.epilogue);
    BK_ARG(g.ld_out >= g.col_off + g.n_rows, "step plan: segment %d ld_out=%d < col_off+n_rows", s, g.ld_out);
    if (g.epilogue == BK_EPI_SWIGLU) {
      BK_ARG(g.W2 != 0 && (g.W2 & 15) == 0 && a.n_segs == 1, "step plan: a SwiGLU segment needs W2 and must be alone");
      has_swiglu = true;
    }
    if (g.epilogue == BK_EPI_ADD_BF16) BK_ARG(g.residual != 0, "step plan: segment %d needs a residual", s);
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
  if (flags & BK_PF_ARGMAX) BK_ARG(a.n_segs == 1 && a.segs[0].epilogue == BK_EPI_F32, "step plan: argmax needs one f32 segment");
  p.total_vrows = vrows;
  // rows per CTA (even: gate/up pairs stay together) and rows per warp group: one group per warp when the CTA's rows
  // allow it, at most 8 rows, and never more than half of a warp's ring so that the next group can be in flight
  const size_t rowb = (size_t)(a.K / 256) * 144;
  int rpc = (vrows + pl->grid - 1) / pl->grid;
  rpc = (rpc + 1) & ~1;
  int G = (rpc + kPW - 1) / kPW;
  if (G > 8) G = 8;
  const int min_g = has_swiglu ? 2 : 1;
  if (has_swiglu) G = (G + 1) & ~1;
  while (G > min_g && (size_t)G * rowb * 2 > pl->ring_bytes) G -= min_g;
  BK_ARG((size_t)G * rowb <= pl->ring_bytes, "step plan: a group of %d rows of K=%d exceeds the ring", G, a.K);
  p.rows_per_cta = rpc;
  p.group_rows = G;
  p.x_unit_words = kUnitWords;
  p.x_row_words = (a.K / 64) * kUnitWords;
  p.x_scale_ld = a.K / 32;
  pl->ph[0].push_back(ph);
  pl->ph[1].push_back(ph);
  return BK_OK;
}

int32_t bk_plan_add_gdn(uint64_t plan, const bkGdnArgs& a) {
  Plan* pl = as_plan(plan);
  BK_ARG(pl && !pl->finished, "step plan: closed");
  BK_ARG(a.B == 1 && a.Hk > 0 && a.Hv > 0 && a.Hv % a.Hk == 0, "step plan: bad GDN shape B=%d Hk=%d Hv=%d", a.B, a.Hk, a.Hv);
  BK_ARG(a.qkv && a.z && a.a && a.b && a.A_log && a.dt_bias && a.norm_w && a.S_in && a.S_new && a.out && a.apply_conv &&
             a.conv_w && a.conv_state_in && a.conv_state_new && a.conv_state_in != a.conv_state_new && (a.conv_w & 7) == 0,
         "step plan: GDN arguments missing");
  Phase ph;
  memset(&ph, 0, sizeof(ph));
  ph.type = PH_GDN;
  GdnParams& p = ph.d;
  p.qkv = bk_ptr<uint16_t>(a.qkv);
  p.z = bk_ptr<uint16_t>(a.z);
  p.a = bk_ptr<float>(a.a);
  p.b = bk_ptr<float>(a.b);
  p.conv_w = bk_ptr<uint16_t>(a.conv_w);
  p.cs_in = bk_ptr<uint16_t>(a.conv_state_in);
  p.cs_new = bk_ptr<uint16_t>(a.conv_state_new);
  p.A_log = bk_ptr<float>(a.A_log);
  p.dt_bias = bk_ptr<uint16_t>(a.dt_bias);
  p.norm_w = bk_ptr<float>(a.norm_w);
  p.S_in = bk_ptr<float>(a.S_in);
  p.S_new = bk_ptr<float>(a.S_new);
  p.out = bk_ptr<uint16_t>(a.out);
  p.B = a.B;
  p.Hk = a.Hk;
  p.Hv = a.Hv;
  p.apply_conv = 1;
  p.T = 1;
  p.early = 1;
  pl->ph[0].push_back(ph);
  p.cs_in = bk_ptr<uint16_t>(a.conv_state_new);   // odd steps read what even steps wrote
  p.cs_new = bk_ptr<uint16_t>(a.conv_state_in);
  pl->ph[1].push_back(ph);
  return BK_OK;
}

int32_t bk_plan_count(uint64_t plan) { return plan ? (int32_t)as_plan(plan)->ph[0].size() : 0; }

int32_t bk_plan_finish(uint64_t plan) {
  Plan* pl = as_plan(plan);
  BK_ARG(pl && !pl->finished && !pl->ph[0].empty(), "step plan: nothing to finish");
  BK_ARG(pl->ph[0].size() < 4000, "step plan: too many phases");
  cudaStream_t st = bk_ctx().stream;
  const size_t bytes = pl->ph[0].size() * sizeof(Phase);
  for (int i = 0; i < 2; i++) {
    void* p = nullptr;
    BK_CUDA(cudaMalloc(&p, bytes));
    pl->d_ph[i] = static_cast<Phase*>(p);
    BK_CUDA(cudaMemcpyAsync(p, pl->ph[i].data(), bytes, cudaMemcpyHostToDevice, st));
  }
  {
    void* p = nullptr;
    const size_t n = (size_t)pl->grid + 8;
    BK_CUDA(cudaMalloc(&p, n * 4));
    BK_CUDA(cudaMemsetAsync(p, 0, n * 4, st));
    pl->d_flags = static_cast<unsigned int*>(p);
    BK_CUDA(cudaMalloc(&p, (size_t)pl->grid * 4));
    pl->d_part_v = static_cast<float*>(p);
    BK_CUDA(cudaMalloc(&p, (size_t)pl->grid * 4));
    pl->d_part_i = static_cast<int32_t*>(p);
  }
  BK_CUDA(cudaStreamSynchronize(st));
  BK_CUDA(cudaFuncSetAttribute(decode_persist_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)pl->smem));
  int per_sm = 0;
  BK_CUDA(cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, decode_persist_kernel, kPT, pl->smem));
  if (per_sm < 1) return bk_fail(BK_ERR_UNSUPPORTED, "step plan: the persistent kernel does not fit on an SM");
  pl->finished = true;
  return BK_OK;
}

int32_t bk_plan_launch(uint64_t plan, int first, int count, int parity, const BkStepIO& io) {
  Plan* pl = as_plan(plan);
  BK_ARG(pl && pl->finished, "step plan: not finished");
  BK_ARG(first >= 0 && count >= 1 && first + count <= (int)pl->ph[0].size(), "step plan: phases [%d, %d) out of range", first, first + count);
  BkContext& c = bk_ctx();
  PersistParams P;
  memset(&P, 0, sizeof(P));
  P.phases = pl->d_ph[parity & 1];
  P.first = first;
  P.count = count;
  P.flags = pl->d_flags;
  P.epoch = pl->d_flags + pl->grid;
  P.counter = pl->d_flags + pl->grid + 2;
  P.counter_base = pl->d_flags + pl->grid + 3;
  P.barrier_mode = c.step_barrier_mode;
  P.barrier_polls = c.spin_limit > 0 ? c.spin_limit : kBarrierPolls;
  P.status = c.d_status;
  P.trace = (c.step_trace && c.step_trace_phases >= (int)pl->ph[0].size()) ? c.step_trace : nullptr;
  P.ring_bytes = pl->ring_bytes;
  P.scratch_bytes = pl->scratch_bytes;
  P.io.embed = bk_ptr<uint8_t>(io.embed);
  P.io.ids_in = bk_ptr<int32_t>(io.ids_in);
  P.io.x0 = bk_ptr<uint16_t>(io.x0);
  P.io.H = io.H;
  P.io.part_v = pl->d_part_v;
  P.io.part_i = pl->d_part_i;
  P.io.counter = pl->d_flags + pl->grid + 1;
  P.io.ids_out = bk_ptr<int32_t>(io.ids_out);
  P.io.val_out = bk_ptr<float>(io.val_out);
  P.io.pos = bk_ptr<int32_t>(io.pos);
  P.io.hist = bk_ptr<int32_t>(io.hist);
  P.io.hist_ld = io.hist_ld;
  P.io.hist_rows = io.hist_rows;
  P.io.host_out = bk_ptr<int32_t>(io.host_out);
  P.io.vocab_offset = io.vocab_offset;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(pl->grid);
  cfg.blockDim = dim3(kPT);
  cfg.dynamicSmemBytes = pl->smem;
  cfg.stream = c.stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeCooperative;
  attr[0].val.cooperative = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  BK_CUDA(cudaLaunchKernelEx(&cfg, decode_persist_kernel, P));
  BK_CHECK_LAUNCH();
  return BK_OK;
}

// Barrier words, generation bases and the argmax counter back to zero (after a launch that gave up they are in an
// unknown state).  Enqueued on the library stream.
int32_t bk_plan_reset(uint64_t plan) {
  Plan* pl = as_plan(plan);
  BK_ARG(pl && pl->finished, "step plan: not finished");
  BK_CUDA(cudaMemsetAsync(pl->d_flags, 0, ((size_t)pl->grid + 8) * 4, bk_ctx().stream));
  return BK_OK;
}

void bk_plan_destroy(uint64_t plan) {
  Plan* pl = as_plan(plan);
  if (!pl) return;
  for (int i = 0; i < 2; i++)
    if (pl->d_ph[i]) cudaFree(pl->d_ph[i]);
  if (pl->d_flags) cudaFree(pl->d_flags);
  if (pl->d_part_v) cudaFree(pl->d_part_v);
  if (pl->d_part_i) cudaFree(pl->d_part_i);
  delete pl;
}
