// bk_internal.h -- host-side state shared by the translation units of libbunker_cuda.
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>
#include <stdio.h>

#include "../../include/bunker_cuda_diag.h"

struct BkContext {
  bool ready = false;
  int device = -1;
  int sm_count = 0;
  int cc_major = 0, cc_minor = 0;
  size_t total_mem = 0;
  size_t smem_optin = 0;
  cudaStream_t stream = nullptr;
  unsigned long long launches = 0;   // kernels enqueued outside graphs + graph kernels replayed
  bool capturing = false;            // true while a graph capture is open on `stream`
  unsigned long long captured = 0;   // kernels recorded into the open capture
  unsigned long long* trace = nullptr;  // device trace buffer (bkTraceEnable), 8 slots per launch
  int trace_cap = 0;                  // launches the buffer can hold
  int trace_seq = 0;                  // next launch index
  unsigned long long* cta_trace = nullptr;  // per-CTA timeline of one chosen GEMV launch (bkTraceCtas)
  int cta_trace_launch = -1;          // index (among GEMV launches since bkTraceCtas) of the launch to record
  int cta_trace_seen = 0;
  unsigned long long* step_trace = nullptr;  // per-phase timeline of the persistent step kernel (bkStepTraceEnable)
  int step_trace_phases = 0;          // phases the buffer can hold (4 slots each)
  int spin_limit = 0;                 // polls a bounded device-side wait may take (bkSetSpinLimit; 0 = built-in limits)
  int step_barrier_mode = 1;          // grid barrier of the persistent step kernel: 0 one word per CTA, 1 one counter (faster, measured)
  int* d_status = nullptr;           // device word set by kernels whose bounded waits gave up
  float* tile_scratch = nullptr;     // dense tile GEMV cut along K: per-chunk partial sums [tile][chunk][32 columns][128 rows]
  int* tile_counters = nullptr;      // ... and one arrival counter per tile (self-resetting)
  size_t tile_scratch_bytes = 0;
  float* gemv_carry = nullptr;       // class accumulators handed from one K part of a split GEMV to the next
  size_t gemv_carry_bytes = 0;
  char err[512] = {0};
};

BkContext& bk_ctx();
int32_t bk_fail(int32_t code, const char* fmt, ...);

// count one kernel launch (directly executed or recorded into a capture)
inline void bk_count_launch() {
  BkContext& c = bk_ctx();
  if (c.capturing) c.captured++; else c.launches++;
}

#define BK_REQUIRE_INIT()                                                            \
  do {                                                                               \
    if (!bk_ctx().ready) return bk_fail(BK_ERR_STATE, "%s: bkInit has not been called", __func__); \
  } while (0)

#define BK_CUDA(expr)                                                                \
  do {                                                                               \
    cudaError_t _e = (expr);                                                         \
    if (_e != cudaSuccess)                                                           \
      return bk_fail((int32_t)_e, "%s: %s -> %s", __func__, #expr, cudaGetErrorString(_e)); \
  } while (0)

#define BK_CHECK_LAUNCH()                                                            \
  do {                                                                               \
    cudaError_t _e = cudaGetLastError();                                             \
    if (_e != cudaSuccess)                                                           \
      return bk_fail((int32_t)_e, "%s: kernel launch -> %s", __func__, cudaGetErrorString(_e)); \
    bk_count_launch();                                                               \
  } while (0)

#define BK_ARG(cond, ...)                                                            \
  do {                                                                               \
    if (!(cond)) return bk_fail(BK_ERR_ARG, __VA_ARGS__);                             \
  } while (0)

template <typename T>
static inline T* bk_ptr(uint64_t p) { return reinterpret_cast<T*>(static_cast<uintptr_t>(p)); }

// ---- tensor-parallel exchange fused into the GEMV (descriptors filled by bk_comm.cu) --------------------
// Push: a row-parallel GEMV stores its f32 partial result into the exchange region of EVERY rank (its own included)
// as 8-byte words {value, tag}: an aligned 8-byte store arrives whole, so a reader that sees the tag has the value --
// no fence, flag or counter, one NVLink store latency.  (Forwarding from the reducer instead of pushing from the GEMV
// epilogue was measured slower: the words leave later, and the reducer's successor still waits for the acknowledgement
// of the remote stores before the grid counts as complete.)  tag = epoch*256 + index of the exchange in the step + 1;
// the epoch is a device word every rank advances once per step, so a tag never repeats in a slot.
// Reduce: the consumer (the next projection's prologue, or the norm+quantise launch at batch >= 2) polls -- bounded --
// the words it needs in LOCAL memory, sums the partials in rank order, adds the residual, rounds to bf16 once.
// Two slots alternate so that a rank running ahead cannot overwrite words a slower rank has not read yet.
#define BK_EPI_PUSH_F32 4        /* internal epilogue: f32 partial pushed to all ranks */
#define BK_PRO_REDUCE_RMSNORM 4  /* internal prologue: reduce + residual -> bf16 -> RMSNorm -> Q8_1 */
struct BkPush {
  uint2* dst[8];               // [r]: rank r's region for this rank's {value, tag} words
  const unsigned int* epoch;   // local step counter
  unsigned int tag_add;        // index of the exchange in the step + 1
  int n;                       // ranks; 0 = no push
};
struct BkReduce {
  const uint2* src;            // local region [n][stride] {value, tag} words
  const unsigned int* epoch;
  const uint16_t* res;         // residual bf16, same indexing as the partials
  uint16_t* out;               // sum + residual as bf16 (materialised for later residual adds)
  unsigned long long stride;   // words between ranks' partials
  unsigned int tag_add;
  int n;                       // ranks; 0 = no reduce
  unsigned int* ready;         // local word: CTA 0 of a reducing GEMV stores the tag here once `out` is complete
  int spin_limit;              // polls before the bounded wait gives up (0 = default)
};

// internal launchers shared between translation units
bool bk_gemv_mma_fits(int K, int B);   // whether the batch-3..8 tensor-core GEMV can hold this K (else column pairs)
bool bk_gemv_auto_tile(int rows, int K);   // whether BK_GEMV_ORDER_AUTO sends a launch of these shapes (>= 16 columns) to the dense tile path
int32_t bk_gemv_launch(const bkGemvArgs& a);
// decode attention; n_seq > 0: the B entries are prompt columns of n_seq sequences (append launch + attention launch)
int32_t bk_attn_launch(const bkAttnArgs& a, int n_seq, int layout_B);
// same with the fused exchange: push (may be null) for BK_EPI_PUSH_F32 segments, reduce (may be null) for
// BK_PRO_REDUCE_RMSNORM; ctas_out (may be null) receives the number of CTAs that will signal arrival
int32_t bk_gemv_launch_tp(const bkGemvArgs& a, const BkPush* push, const BkReduce* reduce, int* ctas_out);
int32_t bk_quant_rows_launch(uint64_t x, uint64_t w, int32_t K, int32_t B, float eps, uint64_t out, int32_t layout,
                             const BkReduce* reduce);
int32_t bk_argmax_launch(uint64_t logits, int32_t V, int32_t B, uint64_t idx, uint64_t val, uint64_t scratch,
                         uint64_t pos, uint64_t hist, int32_t hist_ld, int32_t hist_rows, uint64_t host_out = 0);

// Launch with programmatic dependent launch: the kernel may start while its predecessor on the
// stream is still running; it must execute bk_pdl_wait() (bk_common.cuh) before it touches anything
// an earlier kernel wrote or may still read.  Works eagerly and under stream capture.
template <typename... KArgs, typename... Args>
static inline cudaError_t bk_launch_pdl(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, Args&&... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = bk_ctx().stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  return cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...);
}

// next trace record for a launch (nullptr when tracing is off or the buffer is full)
inline unsigned long long* bk_trace_slot() {
  BkContext& c = bk_ctx();
  if (!c.trace || c.trace_seq >= c.trace_cap) return nullptr;
  return c.trace + (size_t)(c.trace_seq++) * 8;
}

// tensor-parallel exchange (bk_comm.cu)
uint64_t bk_comm_slot_ptr(uint64_t comm, int slot);
int32_t bk_comm_push_desc(uint64_t comm, int slot, BkPush* out);       // slot 0 or 1 of the push region; tag_add left 0
int32_t bk_comm_reduce_desc(uint64_t comm, int slot, BkReduce* out);   // src/epoch/stride/n filled in
uint64_t bk_comm_epoch_ptr(uint64_t comm);                             // device word to advance once per step
int32_t bk_comm_allreduce_residual(uint64_t comm, int slot, int n, uint64_t residual, uint64_t out);
int32_t bk_comm_argmax_merge(uint64_t comm, int slot, int B, uint64_t local_val, uint64_t local_idx, int offset, uint64_t idx,
                             uint64_t val, uint64_t pos, uint64_t hist, int hist_ld, int hist_rows);
int32_t bk_comm_info(uint64_t comm, int* rank, int* nranks);

// ---- persistent decode step (bk_persist.cu) ----------------------------------------------------------------
// A plan is the list of phases of one batch-1 decode step on one GPU: GEMV phases (bkGemvArgs, prologues
// BK_PRO_RMSNORM / BK_PRO_BF16) and conv1d + gated-DeltaNet phases (bkGdnArgs).  bk_plan_launch runs phases
// [first, first+count) in ONE cooperative launch with device-side barriers between them.
#define BK_PF_EMBED 1    /* GEMV phase: the activation is the embedded row of token ids_in[0] (also stored to x0) */
#define BK_PF_ARGMAX 2   /* GEMV phase with one f32 segment: the launch ends with the argmax tail over its rows */
struct BkStepIO {
  uint64_t embed, ids_in, x0;                            // BK_PF_EMBED
  uint64_t ids_out, val_out, pos, hist, host_out;        // BK_PF_ARGMAX tail (as bk_argmax_launch)
  int32_t H, hist_ld, hist_rows, vocab_offset;
};
int32_t bk_plan_create(uint64_t* out, int hidden);
bool bk_plan_gemv_fits(uint64_t plan, int K);
int32_t bk_plan_add_gemv(uint64_t plan, const bkGemvArgs& a, int flags);
int32_t bk_plan_add_gdn(uint64_t plan, const bkGdnArgs& a);   // odd conv-state parity swaps conv_state_in / _new
int32_t bk_plan_count(uint64_t plan);
int32_t bk_plan_finish(uint64_t plan);
int32_t bk_plan_launch(uint64_t plan, int first, int count, int parity, const BkStepIO& io);
int32_t bk_plan_reset(uint64_t plan);
void bk_plan_destroy(uint64_t plan);
