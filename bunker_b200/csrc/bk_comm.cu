// bk_comm.cu -- tensor-parallel exchange between the ranks of one NVLink/NVSwitch box.
//
// The reference has no multi-GPU path (one context on device 0, src/ttir.ts:249-252); this is the
// sharded decode step's only communication: after each row-parallel GEMV (out_proj / o_proj / down)
// the ranks' f32 partial rows are summed in rank order, the residual is added and the result rounded
// to bf16 once; after the vocabulary-sharded lm_head the per-rank (max, index) pairs are merged.
//
// One process per GPU.  Every rank allocates one exchange buffer and publishes it with a CUDA IPC
// handle (the host passes the handles around, e.g. with torch.distributed); peers map it and read it
// with plain loads over NVLink.  No multicast, no multimem, no NCCL on this path.
//
// Protocol (all ranks run the same sequence of exchanges, so a sequence number identifies one):
//   the payload of an exchange lives in one of three slots of the owner's buffer (written by the
//   preceding kernel; the slot is fixed per call site, so it can be baked into a CUDA graph);
//   the owner then stores the sequence number s into flag[owner] of every peer's buffer (remote store
//   after a system fence); a reader waits until its local flag[p] >= s for every p, then loads p's payload.
//   Consecutive exchanges must use different slots: nobody can start exchange s+2 before it finished
//   s+1, which needs every peer's flag s+1, which a peer only raises after it has finished reading s.
// Every wait is bounded; on timeout the kernel sets the status word and returns.
//
// Fused exchange (the model's row-parallel GEMVs): a second region, push[2 slots][ranks][payload as {value, tag}
// words], receives the partial sums of ALL ranks by remote 8-byte stores from the producing GEMV itself.  The
// consumer -- the prologue of the next projection, or the norm+quantise launch -- polls the words it needs in
// local memory until their tag is the current one and sums them: one NVLink store latency per exchange, no extra
// launch, no fence, no remote load.  The tag is epoch*256 + (index of the exchange in the step) + 1; the epoch
// word is advanced by the last kernel of every step (argmax_merge_kernel), identically on all ranks.  Slots
// alternate: nobody can push exchange e+2 before it has consumed e+1, which needs every rank's e+1 words, which
// a rank only sends after it has consumed e.
#include <string.h>

#include "bk_common.cuh"
#include "bk_internal.h"

struct BkComm {
  int rank = 0, nranks = 1;
  size_t payload_bytes = 0;       // per slot
  uint8_t* local = nullptr;       // [3 slots][payload] | flags[8] u64 | counter u64 | pad | push [2][nranks][2*payload] | epoch u32
  size_t push_off = 0, epoch_off = 0; // byte offsets of the push region and the step counter (same on every rank)
  uint8_t* peer[8] = {nullptr};   // mapped bases, peer[rank] == local
  bool imported = false;
};

namespace {

constexpr int kMaxRanks = 8;
constexpr int kSlots = 3;
constexpr int kSpinLimit = 1 << 24;

struct CommDev {
  uint8_t* peer[kMaxRanks];
  int rank, nranks;
  unsigned long long payload_bytes;
};

__device__ __forceinline__ unsigned long long* flags_of(uint8_t* base, unsigned long long payload_bytes) {
  return reinterpret_cast<unsigned long long*>(base + kSlots * payload_bytes);
}

__device__ __forceinline__ unsigned long long ld_volatile_u64(const unsigned long long* p) {
  unsigned long long v;
  asm volatile("ld.volatile.global.u64 %0, [%1];" : "=l"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ float ld_volatile_f32(const float* p) {
  float v;
  asm volatile("ld.volatile.global.f32 %0, [%1];" : "=f"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ float4 ld_volatile_f32x4(const float* p) {
  float4 v;
  asm volatile("ld.volatile.global.v4.f32 {%0,%1,%2,%3}, [%4];" : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w) : "l"(p) : "memory");
  return v;
}

// announce exchange `seq` to every peer and wait for theirs; returns false on timeout
__device__ bool exchange_barrier(const CommDev& c, unsigned long long seq, int* status) {
  __shared__ int ok;
  if (threadIdx.x == 0) ok = 1;
  __syncthreads();
  if (threadIdx.x < c.nranks) {
    const int p = threadIdx.x;
    __threadfence_system();
    unsigned long long* remote = flags_of(c.peer[p], c.payload_bytes) + c.rank;
    asm volatile("st.volatile.global.u64 [%0], %1;" ::"l"(remote), "l"(seq) : "memory");
    const unsigned long long* mine = flags_of(c.peer[c.rank], c.payload_bytes) + p;
    int it = 0;
    while (ld_volatile_u64(mine) < seq) {
      if (++it > kSpinLimit) {
        ok = 0;
        if (status) atomicExch(status, BK_ERR_TIMEOUT);
        break;
      }
    }
    __threadfence_system();
  }
  __syncthreads();
  return ok != 0;
}

// out[i] = bf16( ((p0[i] + p1[i]) + ...) + f32(res[i]) ), i < n; one CTA
__global__ void __launch_bounds__(1024) allreduce_residual_kernel(const CommDev c, int slot_id, int n, const uint16_t* res,
                                                                  uint16_t* out, int* status, unsigned long long* trace) {
  bk_pdl_trigger();
  bk_stamp(trace, 0);
  bk_pdl_wait();
  bk_stamp(trace, 2);
  unsigned long long* counter = flags_of(c.peer[c.rank], c.payload_bytes) + kMaxRanks;
  const unsigned long long seq = *counter + 1;
  const bool ok = exchange_barrier(c, seq, status);
  bk_stamp(trace, 3);
  if (ok) {
    const size_t slot = (size_t)slot_id * c.payload_bytes;
    for (int i = threadIdx.x * 4; i < n; i += blockDim.x * 4) {
      float4 acc = ld_volatile_f32x4(reinterpret_cast<const float*>(c.peer[0] + slot) + i);
      for (int r = 1; r < c.nranks; r++) {
        float4 v = ld_volatile_f32x4(reinterpret_cast<const float*>(c.peer[r] + slot) + i);
        acc.x = __fadd_rn(acc.x, v.x);
        acc.y = __fadd_rn(acc.y, v.y);
        acc.z = __fadd_rn(acc.z, v.z);
        acc.w = __fadd_rn(acc.w, v.w);
      }
      uint2 rv = *reinterpret_cast<const uint2*>(res + i);
      uint32_t lo = bk_f32x2_to_bf16x2(__fadd_rn(acc.x, __uint_as_float(rv.x << 16)),
                                       __fadd_rn(acc.y, __uint_as_float(rv.x & 0xffff0000u)));
      uint32_t hi = bk_f32x2_to_bf16x2(__fadd_rn(acc.z, __uint_as_float(rv.y << 16)),
                                       __fadd_rn(acc.w, __uint_as_float(rv.y & 0xffff0000u)));
      *reinterpret_cast<uint2*>(out + i) = make_uint2(lo, hi);
    }
  }
  __syncthreads();
  if (threadIdx.x == 0) *counter = seq;
  bk_stamp(trace, 5);
}

// merge per-rank (value, index) pairs: payload of rank r = B pairs {f32 val, i32 idx (already global)}.
// Strict '>' in rank order keeps the lowest index on ties because rank order is vocabulary order.
__global__ void __launch_bounds__(32) argmax_merge_kernel(const CommDev c, int slot_id, int B, int32_t* idx, float* val, int32_t* pos,
                                                          int32_t* hist, int hist_ld, int hist_rows, int* status,
                                                          unsigned int* epoch) {
  bk_pdl_trigger();
  bk_pdl_wait();
  unsigned long long* counter = flags_of(c.peer[c.rank], c.payload_bytes) + kMaxRanks;
  const unsigned long long seq = *counter + 1;
  const bool ok = exchange_barrier(c, seq, status);
  if (ok) {
    const size_t slot = (size_t)slot_id * c.payload_bytes;
    for (int b = threadIdx.x; b < B; b += blockDim.x) {
      float bv = -INFINITY;
      int bi = 0;
      for (int r = 0; r < c.nranks; r++) {
        const float* pr = reinterpret_cast<const float*>(c.peer[r] + slot) + 2 * b;
        float v = ld_volatile_f32(pr);
        int i = __float_as_int(ld_volatile_f32(pr + 1));
        if (r == 0 || v > bv) {
          bv = v;
          bi = i;
        }
      }
      idx[b] = bi;
      val[b] = bv;
      if (pos) {
        int pcur = pos[b];
        if (hist && pcur < hist_rows) hist[(size_t)pcur * hist_ld + b] = bi;
        pos[b] = pcur + 1;
      }
    }
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    *counter = seq;
    if (epoch) *epoch = *epoch + 1;   // last kernel of a decode step: the tags of the next step's fused exchanges change
  }
}

// local (val, idx) of this rank -> {val, idx + offset} pairs in the exchange slot of the next sequence number
__global__ void pack_argmax_kernel(const CommDev c, int slot_id, int B, const float* val, const int32_t* idx, int offset) {
  bk_pdl_trigger();
  bk_pdl_wait();
  float* dst = reinterpret_cast<float*>(c.peer[c.rank] + (size_t)slot_id * c.payload_bytes);
  for (int b = threadIdx.x; b < B; b += blockDim.x) {
    dst[2 * b] = val[b];
    dst[2 * b + 1] = __int_as_float(idx[b] + offset);
  }
}

CommDev dev_view(const BkComm& c) {
  CommDev d;
  for (int i = 0; i < kMaxRanks; i++) d.peer[i] = c.peer[i];
  d.rank = c.rank;
  d.nranks = c.nranks;
  d.payload_bytes = c.payload_bytes;
  return d;
}

BkComm* as_comm(uint64_t h) { return reinterpret_cast<BkComm*>(static_cast<uintptr_t>(h)); }

}  // namespace

// ---- internal API used by the model -------------------------------------------------------------

uint64_t bk_comm_slot_ptr(uint64_t comm, int slot) {
  BkComm* c = as_comm(comm);
  return (uint64_t)(uintptr_t)(c->local + (size_t)slot * c->payload_bytes);
}

int32_t bk_comm_allreduce_residual(uint64_t comm, int slot, int n, uint64_t residual, uint64_t out) {
  BkComm* c = as_comm(comm);
  BK_ARG(c && c->imported, "allreduce: communicator has no peers mapped (bkCommImportPeers)");
  BK_ARG(n > 0 && n % 4 == 0 && (size_t)n * 4 <= c->payload_bytes, "allreduce: n=%d does not fit the exchange slot", n);
  BK_ARG(slot >= 0 && slot < kSlots, "allreduce: slot %d out of range", slot);
  BK_CUDA(bk_launch_pdl(allreduce_residual_kernel, dim3(1), dim3(1024), 0, dev_view(*c), slot, n, bk_ptr<uint16_t>(residual),
                        bk_ptr<uint16_t>(out), bk_ctx().d_status, bk_trace_slot()));
  BK_CHECK_LAUNCH();
  return BK_OK;
}

int32_t bk_comm_argmax_merge(uint64_t comm, int slot, int B, uint64_t local_val, uint64_t local_idx, int offset, uint64_t idx,
                             uint64_t val, uint64_t pos, uint64_t hist, int hist_ld, int hist_rows) {
  BkComm* c = as_comm(comm);
  BK_ARG(c && c->imported, "argmax merge: communicator has no peers mapped (bkCommImportPeers)");
  BK_ARG((size_t)B * 8 <= c->payload_bytes, "argmax merge: B=%d does not fit the exchange slot", B);
  BK_CUDA(bk_launch_pdl(pack_argmax_kernel, dim3(1), dim3(32), 0, dev_view(*c), slot, B, bk_ptr<float>(local_val),
                        bk_ptr<int32_t>(local_idx), offset));
  BK_CHECK_LAUNCH();
  BK_CUDA(bk_launch_pdl(argmax_merge_kernel, dim3(1), dim3(32), 0, dev_view(*c), slot, B, bk_ptr<int32_t>(idx), bk_ptr<float>(val),
                        bk_ptr<int32_t>(pos), bk_ptr<int32_t>(hist), hist_ld, hist_rows, bk_ctx().d_status,
                        reinterpret_cast<unsigned int*>(c->local + c->epoch_off)));
  BK_CHECK_LAUNCH();
  return BK_OK;
}

int32_t bk_comm_push_desc(uint64_t comm, int slot, BkPush* out) {
  BkComm* c = as_comm(comm);
  BK_ARG(c && c->imported && out && (slot == 0 || slot == 1), "push descriptor: bad communicator or slot");
  memset(out, 0, sizeof(*out));
  for (int r = 0; r < c->nranks; r++)
    out->dst[r] = reinterpret_cast<uint2*>(c->peer[r] + c->push_off + ((size_t)slot * c->nranks + c->rank) * 2 * c->payload_bytes);
  out->epoch = reinterpret_cast<const unsigned int*>(c->local + c->epoch_off);
  out->n = c->nranks;
  return BK_OK;
}

uint64_t bk_comm_epoch_ptr(uint64_t comm) {
  BkComm* c = as_comm(comm);
  return c ? (uint64_t)(uintptr_t)(c->local + c->epoch_off) : 0;
}

int32_t bk_comm_reduce_desc(uint64_t comm, int slot, BkReduce* out) {
  BkComm* c = as_comm(comm);
  BK_ARG(c && c->imported && out && (slot == 0 || slot == 1), "reduce descriptor: bad communicator or slot");
  memset(out, 0, sizeof(*out));
  out->src = reinterpret_cast<const uint2*>(c->local + c->push_off + (size_t)slot * c->nranks * 2 * c->payload_bytes);
  out->epoch = reinterpret_cast<const unsigned int*>(c->local + c->epoch_off);
  out->stride = c->payload_bytes / 4;   // one 8-byte word per f32 of the payload
  out->ready = reinterpret_cast<unsigned int*>(c->local + c->epoch_off + 64) + slot;
  out->spin_limit = bk_ctx().spin_limit;
  out->n = c->nranks;
  return BK_OK;
}

int32_t bk_comm_info(uint64_t comm, int* rank, int* nranks) {
  BkComm* c = as_comm(comm);
  if (!c) return bk_fail(BK_ERR_ARG, "null communicator");
  *rank = c->rank;
  *nranks = c->nranks;
  return BK_OK;
}

// ---- C ABI ------------------------------------------------------------------------------------------

extern "C" {

int32_t bkCommCreate(int32_t rank, int32_t nranks, uint64_t payload_bytes, uint64_t* out_comm) {
  BK_REQUIRE_INIT();
  BK_ARG(out_comm != nullptr, "bkCommCreate: out_comm is null");
  BK_ARG(nranks >= 1 && nranks <= kMaxRanks && rank >= 0 && rank < nranks, "bkCommCreate: rank %d of %d (at most %d ranks)", rank,
         nranks, kMaxRanks);
  BK_ARG(payload_bytes >= 64, "bkCommCreate: payload_bytes=%llu too small", (unsigned long long)payload_bytes);
  BkComm* c = new BkComm();
  c->rank = rank;
  c->nranks = nranks;
  c->payload_bytes = (payload_bytes + 255) / 256 * 256;
  c->push_off = (kSlots * c->payload_bytes + (kMaxRanks + 1) * sizeof(unsigned long long) + 255) / 256 * 256;
  c->epoch_off = c->push_off + (size_t)2 * nranks * 2 * c->payload_bytes;
  size_t total = c->epoch_off + 256;
  void* p = nullptr;
  cudaError_t e = cudaMalloc(&p, total);
  if (e != cudaSuccess) {
    delete c;
    return bk_fail((int32_t)e, "bkCommCreate: cudaMalloc -> %s", cudaGetErrorString(e));
  }
  // tags, flags and the epoch start at zero; the zeroing is ordered on the library stream and awaited, so no peer's
  // store and no later launch can overtake it
  cudaMemsetAsync(p, 0, total, bk_ctx().stream);
  cudaStreamSynchronize(bk_ctx().stream);
  c->local = static_cast<uint8_t*>(p);
  c->peer[rank] = c->local;
  c->imported = (nranks == 1);
  *out_comm = (uint64_t)(uintptr_t)c;
  return BK_OK;
}

int32_t bkCommExportHandle(uint64_t comm, uint8_t* out_handle64) {
  BK_REQUIRE_INIT();
  BkComm* c = as_comm(comm);
  BK_ARG(c && out_handle64, "bkCommExportHandle: null argument");
  static_assert(sizeof(cudaIpcMemHandle_t) == 64, "IPC handle size");
  cudaIpcMemHandle_t h;
  BK_CUDA(cudaIpcGetMemHandle(&h, c->local));
  memcpy(out_handle64, &h, 64);
  return BK_OK;
}

int32_t bkCommImportPeers(uint64_t comm, const uint8_t* handles) {
  BK_REQUIRE_INIT();
  BkComm* c = as_comm(comm);
  BK_ARG(c && handles, "bkCommImportPeers: null argument");
  for (int r = 0; r < c->nranks; r++) {
    if (r == c->rank) continue;
    cudaIpcMemHandle_t h;
    memcpy(&h, handles + (size_t)r * 64, 64);
    void* p = nullptr;
    cudaError_t e = cudaIpcOpenMemHandle(&p, h, cudaIpcMemLazyEnablePeerAccess);
    if (e != cudaSuccess)
      return bk_fail(BK_ERR_COMM, "bkCommImportPeers: cannot map the buffer of rank %d: %s", r, cudaGetErrorString(e));
    c->peer[r] = static_cast<uint8_t*>(p);
  }
  c->imported = true;
  return BK_OK;
}

int32_t bkCommDestroy(uint64_t comm) {
  BK_REQUIRE_INIT();
  BkComm* c = as_comm(comm);
  if (!c) return BK_OK;
  cudaStreamSynchronize(bk_ctx().stream);
  for (int r = 0; r < c->nranks; r++)
    if (r != c->rank && c->peer[r]) cudaIpcCloseMemHandle(c->peer[r]);
  if (c->local) cudaFree(c->local);
  delete c;
  return BK_OK;
}

// Standalone exchange (every rank calls it with the same slot and n): out bf16[n] = (sum of the ranks'
// partial f32[n] in rank order) + residual.  Consecutive calls must alternate slots (0, 1, 2).
int32_t bkCommAllReduceResidual(uint64_t comm, int32_t slot, uint64_t partial_f32, int32_t n, uint64_t residual_bf16,
                                uint64_t out_bf16) {
  BK_REQUIRE_INIT();
  BkComm* c = as_comm(comm);
  BK_ARG(c && partial_f32 && residual_bf16 && out_bf16, "bkCommAllReduceResidual: null argument");
  BK_ARG(slot >= 0 && slot < kSlots, "bkCommAllReduceResidual: slot %d out of range", slot);
  BK_ARG(n > 0 && n % 4 == 0 && (size_t)n * 4 <= c->payload_bytes, "bkCommAllReduceResidual: n=%d does not fit", n);
  BK_CUDA(cudaMemcpyAsync(c->local + (size_t)slot * c->payload_bytes, bk_ptr<void>(partial_f32), (size_t)n * 4,
                          cudaMemcpyDeviceToDevice, bk_ctx().stream));
  return bk_comm_allreduce_residual(comm, slot, n, residual_bf16, out_bf16);
}

}  // extern "C"
