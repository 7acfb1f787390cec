/*
 * bunker_cuda.h -- C ABI of libbunker_cuda.so, the sm_100a replacement for
 * bunker's Triton lowering (shim/triton_shim.c) and raw-driver runtime
 * (src/ttir.ts:223-348) on the hybrid decode hot path.
 *
 * Conventions (chosen for bun:ffi, see bunker's LOG.md:725-733):
 *   - every entry point returns int32: 0 = success, otherwise a CUDA runtime
 *     error number or one of the BK_ERR_* codes below; bkLastError() gives text
 *   - device pointers, events and handles travel as uint64_t, never as `ptr`
 *   - host buffers are borrowed for the duration of the call only
 *   - argument structs are copied before the call returns
 *   - nothing is read from the environment (bun's process.env never reaches
 *     getenv, LOG.md:605-607)
 *   - one context per process, one library-owned stream; every op enqueues on
 *     that stream and returns without waiting (src/ttir.ts:342 uses stream 0)
 *
 * Citations name files of skyne98/bunker.
 */
#ifndef BUNKER_CUDA_H
#define BUNKER_CUDA_H

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#if defined(__GNUC__)
#define BK_API __attribute__((visibility("default")))
#else
#define BK_API
#endif

#define BK_OK 0
#define BK_ERR_ARG 10001       /* bad argument (size, alignment, null, range) */
#define BK_ERR_STATE 10002     /* call made in the wrong state (not initialised, ...) */
#define BK_ERR_TIMEOUT 10003   /* a bounded device-side wait gave up */
#define BK_ERR_UNSUPPORTED 10004
#define BK_ERR_COMM 10005      /* communicator / peer-mapping failure */

/* ---- runtime: replaces cu()/cuAlloc/cuHtoD/cuDtoH/cuFree/cuSync ---------- */

/* src/ttir.ts:223-261 cu(): open the driver, create the context on `device`. */
BK_API int32_t bkInit(int32_t device);
BK_API int32_t bkShutdown(void);
/* Text of the most recent failure on this thread's library context. */
BK_API const char* bkLastError(void);
BK_API int32_t bkDeviceInfo(int32_t* sm_count, int32_t* cc_major, int32_t* cc_minor, uint64_t* total_mem);

/* src/ttir.ts:266 cuAlloc */
BK_API int32_t bkAlloc(uint64_t bytes, uint64_t* out_ptr);
/* src/ttir.ts:283 cuFree */
BK_API int32_t bkFree(uint64_t ptr);
/* src/ttir.ts:273 cuHtoD (ordered after queued ops; returns when the host buffer may be reused) */
BK_API int32_t bkHtoD(uint64_t dst, const void* src, uint64_t bytes);
/* src/ttir.ts:278 cuDtoH (synchronous: doubles as the per-token barrier, prototypes/decode.ts:1042-1049) */
BK_API int32_t bkDtoH(void* dst, uint64_t src, uint64_t bytes);
/* src/ttir.ts:305-317 async copies; host memory must stay valid until bkSync */
BK_API int32_t bkHtoDAsync(uint64_t dst, const void* src, uint64_t bytes);
BK_API int32_t bkDtoHAsync(void* dst, uint64_t src, uint64_t bytes);
BK_API int32_t bkDtoD(uint64_t dst, uint64_t src, uint64_t bytes);
BK_API int32_t bkMemset(uint64_t dst, int32_t byte_value, uint64_t bytes);
/* pinned host staging for bkHtoDAsync/bkDtoHAsync */
BK_API int32_t bkHostAlloc(uint64_t bytes, void** out);
BK_API int32_t bkHostFree(void* p);
/* src/ttir.ts:285 cuSync */
BK_API int32_t bkSync(void);

/* src/ttir.ts:352-417 CUDA-event profiler: events on the library stream. */
BK_API int32_t bkEventCreate(uint64_t* out_event);
BK_API int32_t bkEventRecord(uint64_t event);
BK_API int32_t bkEventSync(uint64_t event);
BK_API int32_t bkEventElapsedMs(uint64_t start, uint64_t stop, float* out_ms);
BK_API int32_t bkEventDestroy(uint64_t event);
/* Number of kernels this library has launched since bkInit (graph replays count their kernels). */
BK_API int32_t bkLaunchCount(uint64_t* out_count);

/* ---- Q4_K x Q8_1 GEMV: replaces buildMM/buildGateSwiglu (prototypes/decode.ts:101-186),
 *      emitGemm (src/fusion.ts:276-293) ------------------------------------- */

/* prologues: how the activation reaches the kernel */
#define BK_PRO_Q8 0       /* x = Q8_1 blocks [B][K/32][36] (bench/bench.ts:7 layout) */
#define BK_PRO_BF16 1     /* x = bf16 [B][K]; quantised to Q8_1 inside the kernel */
#define BK_PRO_STAGED 3   /* x = staged image (BK_Q8_STAGED) for this K and B; batch 2..8 only */
#define BK_PRO_RMSNORM 2  /* x = bf16 [B][K]; RMSNorm(x, norm_w, eps) -> bf16 -> Q8_1 inside the kernel
                             (buildRMS, prototypes/decode.ts:201-216, fused) */
/* epilogues */
#define BK_EPI_F32 0      /* out f32 */
#define BK_EPI_BF16 1     /* out bf16(acc)                      (decode.ts cast) */
#define BK_EPI_ADD_BF16 2 /* out bf16(acc + f32(residual))      (decode.ts:152-154 add) */
#define BK_EPI_SWIGLU 3   /* out bf16((g*sigmoid(g))*u), g from W, u from W2 (decode.ts:117-119) */

/* Layouts of a quantised activation handed from one op to the next.
 * BK_Q8_BLOCKS: the reference's Q8_1 blocks [B][K/32][36] (bench/bench.ts:7), read with BK_PRO_Q8.
 * BK_Q8_STAGED: the image the batch-2..8 GEMV keeps in shared memory (bkStagedBytes(K, B) bytes, 16-byte aligned):
 *   words [B][K/4+8] with the eight words of each block in the order 0,4,1,5,2,6,3,7, then float4 [K/64][8] =
 *   {d8 of block 2u, d8 of block 2u+1 / 16, s8 of 2u, s8 of 2u+1} per 64-value unit u and batch column.  The GEMV
 *   prologue is then a single bulk copy (BK_PRO_STAGED).  No counterpart in the reference. */
#define BK_Q8_BLOCKS 0
#define BK_Q8_STAGED 1
BK_API uint64_t bkStagedBytes(int32_t K, int32_t B);

/* f32 accumulation order of a row's result (the integer block dots are exact either way).  LANES: the order of the
 * batch <= 8 kernels (64-weight units over 32 lanes, butterfly).  TILE: from 16 columns on, with BK_PRO_Q8 input, the
 * dense tile kernel (tcgen05 int8 MMA, accumulators in tensor memory) and its order: one chain per (row, column),
 * sub-blocks ascending, superblocks ascending within a chunk of four, chunks ascending; below 16 columns TILE means
 * LANES.  AUTO: TILE when the launch has at least 4096 rows (all segments together, a SwiGLU pair counting twice), or
 * at least 1024 rows and K >= 2048; else LANES -- a rule of the shapes alone, so a host can mirror it.  Both orders are
 * within a few ulp of each other and of the reference's f32 accumulation (prototypes/decode.ts:141-145). */
#define BK_GEMV_ORDER_AUTO 0
#define BK_GEMV_ORDER_LANES 1
#define BK_GEMV_ORDER_TILE 2

typedef struct bkGemvSeg {
  uint64_t W;        /* Q4_K rows [n_rows][K/256][144] */
  uint64_t W2;       /* BK_EPI_SWIGLU: the up_proj rows, else 0 */
  uint64_t out;      /* [B][ld_out] of the epilogue's element type */
  uint64_t residual; /* BK_EPI_ADD_BF16: bf16 [B][ld_out] */
  int32_t n_rows;
  int32_t epilogue;
  int32_t ld_out;    /* elements between consecutive batch rows of out / residual */
  int32_t col_off;   /* column of out that receives this segment's row 0 */
} bkGemvSeg;

typedef struct bkGemvArgs {
  int32_t K;         /* multiple of 256 */
  int32_t B;         /* 1..64 */
  int32_t n_segs;    /* 1..4 row segments that share the activation (qkv|z|a|b, gate|up, ...) */
  int32_t prologue;
  uint64_t x;
  uint64_t norm_w;   /* bf16 [K], BK_PRO_RMSNORM only */
  float eps;
  int32_t order;     /* BK_GEMV_ORDER_AUTO, _LANES or _TILE */
  bkGemvSeg segs[4];
} bkGemvArgs;

BK_API int32_t bkGemvQ4K(const bkGemvArgs* args);
/* config-0 convenience: y f32 [B][N] = W[N][K] (Q4_K) x xq (Q8_1 blocks) */
BK_API int32_t bkGemvQ4KSimple(uint64_t W, int32_t N, int32_t K, uint64_t xq, int32_t B, uint64_t y);

/* dequant (kernel.ts:422 / tests/test_dequant.ts:13-21 analogue for the 144-byte layout): f32 [N][K] */
BK_API int32_t bkDequantQ4K(uint64_t W, int32_t N, int32_t K, uint64_t out_f32);
/* integer stage alone (bench/bench.ts:24-33 s1/s2): int32 [N][K/32] each, for one Q8_1 row */
BK_API int32_t bkBlockDotsQ4K(uint64_t W, int32_t N, int32_t K, uint64_t xq, uint64_t isum, uint64_t qsum);

/* Weight loader's quantiser (no counterpart in the reference, which uploads its safetensors weights as bf16 --
 * loadWeights, prototypes/decode.ts:64-76 -- and keeps them bf16): rows of f32 or bf16 [n_rows][K] -> Q4_K rows
 * [n_rows][K/256][144].  Per 32-weight sub-block lo = min(min x, 0), scale = (max x - lo)/15, min = -lo; per superblock
 * d = f16(max scale/63), dmin = f16(max min/63); 6-bit sc = round(scale/d), m = round(min/dmin);
 * q = clamp(round((x + dmin*m)/(d*sc)), 0, 15). */
#define BK_DTYPE_F32 0
#define BK_DTYPE_BF16 1
BK_API int32_t bkQuantizeQ4K(uint64_t x, int32_t dtype, int64_t n_rows, int32_t K, uint64_t out_q4k);

/* packQ8_1 (bench/bench.ts:53-72) on the device: f32 or bf16 [B][K] -> blocks [B][K/32][36] */
BK_API int32_t bkQuantQ8_1(uint64_t x_f32, int32_t K, int32_t B, uint64_t out_blocks);
BK_API int32_t bkQuantQ8_1Bf16(uint64_t x_bf16, int32_t K, int32_t B, uint64_t out_blocks);

/* ---- small decode ops ------------------------------------------------------- */

/* emitEmbed (src/emitters.ts:31-45): x bf16 [B][H] = dequant(table[ids[b]]); ids int32 on the device */
BK_API int32_t bkEmbedQ4K(uint64_t table, int32_t H, uint64_t ids, int32_t B, uint64_t x_out);
/* buildRMS (prototypes/decode.ts:201-216): y = bf16((x*rstd)*(1+w)) */
BK_API int32_t bkRmsNorm(uint64_t x, uint64_t w, int32_t H, int32_t B, float eps, uint64_t y);
/* buildRMS followed by packQ8_1 (prototypes/decode.ts:201-216, bench/bench.ts:53-72) in one launch: bf16 rows
 * x [B][K] -> Q8_1 of bf16((x*rstd)*(1+w)) in `layout` (BK_Q8_BLOCKS or BK_Q8_STAGED); w = 0 skips the norm
 * (plain bf16 -> Q8_1).  Used between ops at batch >= 2. */
BK_API int32_t bkRmsNormQuantQ8_1(uint64_t x, uint64_t w, int32_t K, int32_t B, float eps, uint64_t out, int32_t layout);
/* The consumer side of the tensor-parallel exchange as a stand-alone call (no counterpart in the reference; the model
 * enqueues it internally at batch >= 2): `words` holds, for each of n_ranks ranks at a stride of stride_words, B*K 8-byte
 * words {f32 partial sum, tag}; the launch polls (bounded) until every word carries the tag *epoch * 256 + tag_add, adds the
 * partials in rank order, adds the bf16 residual, rounds to bf16 (written to sum_out), then RMSNorm(w) and Q8_1 as above. */
BK_API int32_t bkReduceRmsNormQuantQ8_1(uint64_t words, int32_t n_ranks, uint64_t stride_words, uint64_t epoch, uint32_t tag_add,
                                        uint64_t residual, uint64_t sum_out, uint64_t w, int32_t K, int32_t B, float eps,
                                        uint64_t out, int32_t layout);
/* emitSwiGLU (src/fusion.ts:324-330): out bf16 [n] from f32 g,u */
BK_API int32_t bkSwiglu(uint64_t g_f32, uint64_t u_f32, int32_t n, uint64_t out_bf16);
/* emitConv1d (src/emitters.ts:48-72): state [B][3][C] bf16 oldest first, w [C][4] bf16 */
BK_API int32_t bkConv1dStep(uint64_t x, uint64_t state_in, uint64_t w, int32_t C, int32_t B, uint64_t out,
                     uint64_t state_new);

/* emitConv1d + emitGDN fused (src/emitters.ts:48-120, prototypes/decode.ts:272-388).
 * qkv: bf16 [B][2*Hk*128+Hv*128] (pre-conv projection); z bf16 [B][Hv*128]; a,b f32 [B][Hv];
 * conv state [B][3][C]; S f32 [B][Hv][128][128]; out bf16 [B][Hv*128] (normed and gated);
 * o_raw (optional, 0 to skip) f32 [B][Hv*128] un-normalised head output.
 * conv_out (optional) bf16 [B][C] receives the post-conv activations. */
typedef struct bkGdnArgs {
  uint64_t qkv, z, a, b;
  uint64_t conv_w, conv_state_in, conv_state_new;
  uint64_t A_log, dt_bias, norm_w;
  uint64_t S_in, S_new;
  uint64_t out, o_raw, conv_out;
  int32_t B, Hk, Hv, apply_conv; /* apply_conv=0: qkv already holds conv output */
  int32_t state_is_settled;      /* 1: S_in, conv_state_in and the weights were NOT written by the launch that
                                    immediately precedes this one on the stream, so the kernel may read them while that
                                    launch is still running (programmatic dependent launch).  0: read everything after it. */
  int32_t out_q8_layout;         /* BK_Q8_BLOCKS or BK_Q8_STAGED */
  uint64_t out_q8;               /* optional (0 to skip): the same output quantised for the output projection */
  int32_t n_tokens;              /* 0 or 1: one token per sequence (the decode step).  T > 1: T consecutive tokens of every
                                    sequence in one launch; token t of sequence b is row t*B + b of qkv, z, a, b and of
                                    every output ([T*B][...]); the state stays in registers between tokens. */
  int32_t reserved;
} bkGdnArgs;
BK_API int32_t bkGdnStep(const bkGdnArgs* args);

/* f32 tables [max_len][rot_dim/2], filled on the host in double as prototypes/decode.ts:865-871 */
BK_API int32_t bkRopeTables(int32_t max_len, int32_t rot_dim, double theta, float* cos_out, float* sin_out);

/* emitQNorm/emitKNorm + emitRoPE/emitRoPEK (src/emitters.ts:123-183):
 * in bf16 [B][nheads][in_stride] (first HD of each slot), out bf16 [B][nheads*HD]; pos int32 [B] on device */
BK_API int32_t bkHeadNormRope(uint64_t in, int32_t in_stride, uint64_t w, uint64_t cos_t, uint64_t sin_t,
                       int32_t rot_half, uint64_t pos, int32_t B, int32_t nheads, int32_t HD, uint64_t out);

/* emitFA2Attn (src/emitters.ts:188-226) as split-KV flash-decode over a per-KV-head cache.
 * qg: bf16 [B][Hq][2*HD] = per head q | gate (q_proj output); k, v: bf16 [B][Hkv*HD] projections.
 * The kernel norms+rotates q and k, appends k,v at row pos[b], attends over rows 0..pos[b],
 * and writes out bf16 [B][Hq*HD] = attention * sigmoid(gate).
 * caches: bf16 [B][Hkv][max_len][HD].  scratch: bkAttnScratchBytes() bytes, zeroed once before its first use
 * (it ends with completion counters that the kernel re-arms itself). */
typedef struct bkAttnArgs {
  uint64_t qg, k, v;
  uint64_t q_norm_w, k_norm_w, cos_t, sin_t;
  uint64_t k_cache, v_cache;
  uint64_t pos;      /* int32 [B] on the device */
  uint64_t out;
  uint64_t scratch;
  int32_t B, Hq, Hkv, HD, rot_half, max_len;
  int32_t split_len; /* rows per split; 0 = library default from bkAttnPlan */
  int32_t max_pos;   /* upper bound of pos[] this call may see (sizes the grid) */
  float scale;
  int32_t fused_norm_rope; /* 1: as above. 0: qg holds ready q in [B][Hq*HD], gate in `gate`, cache already appended */
  uint64_t gate;     /* only for fused_norm_rope=0: bf16 [B][Hq*HD] */
  int32_t cache_is_settled; /* 1: pos[] and the cache rows below pos[b] were NOT written by the launch that immediately
                               precedes this one on the stream, so they may be read while that launch is still running */
  int32_t out_q8_layout; /* BK_Q8_BLOCKS or BK_Q8_STAGED */
  uint64_t out_q8;   /* optional (0 to skip): the same output quantised for the output projection */
} bkAttnArgs;
BK_API int32_t bkAttnDecode(const bkAttnArgs* args);
/* split length and warps per split the library uses for n rows */
BK_API int32_t bkAttnPlan(int32_t n_rows, int32_t B, int32_t Hkv, int32_t* split_len, int32_t* warps);
BK_API uint64_t bkAttnScratchBytes(int32_t B, int32_t Hq, int32_t HD, int32_t max_len, int32_t split_len);

/* buildArgmax+buildArgmaxComb (prototypes/decode.ts:749-791): exact max, lowest index on ties.
 * logits f32 [B][V]; idx int32 [B]; val f32 [B]; scratch >= bkArgmaxScratchBytes(B) bytes */
BK_API int32_t bkArgmax(uint64_t logits, int32_t V, int32_t B, uint64_t idx, uint64_t val, uint64_t scratch);
BK_API uint64_t bkArgmaxScratchBytes(int32_t B);
/* No counterpart in the reference.  Same result as bkArgmax for callers that cannot allocate device memory
 * (a host with a fixed memory budget, code running where cudaMalloc is forbidden such as during stream
 * capture, a runtime that owns all device memory): the scratch is a 33,024-byte array built into the
 * library, enough for B <= 64; larger B is rejected with BK_ERR_ARG.  Nothing is allocated or freed.  The
 * first call on a device looks up the array's device address, so make it before any stream capture.  All
 * calls share the array: calls that overlap on the GPU race. */
BK_API int32_t bkArgmaxStatic(uint64_t logits, int32_t V, int32_t B, uint64_t idx, uint64_t val);

/* Sampling beside the greedy tail (no counterpart in the reference, which only takes the argmax,
 * prototypes/decode.ts:749-791).  logits f32 [B][V].  Per sequence: the top_k (1..64) largest logits, ties to the lower
 * index, in descending order; p_i = exp((l_i - l_0)/temperature) summed in that order; the shortest prefix reaching
 * top_p * total; u in [0,1) from splitmix64(splitmix64(seed ^ (step << 20)) + sequence) >> 40; the first candidate whose
 * running sum exceeds u * (prefix total).  step = (step_dev ? step_dev[b] : 0) + step_add (step_dev: device int32 [B],
 * e.g. the model's position buffer, or 0).  temperature 0 or top_k 1 is the argmax.  idx int32 [B]; val f32 [B] (the
 * chosen logit; 0 to skip).  Deterministic: the same inputs give the same tokens, on any GPU and on the CPU checker. */
BK_API int32_t bkSample(uint64_t logits, int32_t V, int32_t B, float temperature, int32_t top_k, float top_p, uint64_t seed,
                        uint64_t step_dev, uint32_t step_add, uint64_t idx, uint64_t val);

/* ---- whole decode step: replaces buildModelGraph + compileStep + runGraphDecode
 *      (src/model.ts:46-204, src/runner.ts:94-162) --------------------------------
 * One call per token; the CUDA graph lives inside the library because replaying a graph
 * through bun:ffi crashed the reference (LOG.md:710-738).  Dims follow src/model.ts:14-18. */
typedef struct bkModelConfig {
  int32_t hidden;             /* H */
  int32_t n_layers;           /* NL */
  int32_t full_attn_interval; /* FAI: layer % FAI == FAI-1 is gated attention (src/model.ts:61) */
  int32_t vocab;              /* VOCAB; embedding and lm_head are tied (src/model.ts:196) */
  int32_t gdn_k_heads;        /* LKH, head dim 128 */
  int32_t gdn_v_heads;        /* LVH, head dim 128 */
  int32_t attn_q_heads;       /* NH */
  int32_t attn_kv_heads;      /* NKV */
  int32_t head_dim;           /* HD = 256 */
  int32_t rot_dim;            /* ROT_DIM = 64 */
  int32_t intermediate;       /* INTER */
  int32_t max_len;            /* KV cache rows per sequence (the reference fixes 128) */
  int32_t batch;              /* sequences decoded in lockstep, 1..8 */
  int32_t tp_rank, tp_size;   /* tensor-parallel rank / world (1 = single GPU) */
  float eps;                  /* EPS = 1e-6 */
  double rope_theta;          /* 1e7 (prototypes/decode.ts:868) */
} bkModelConfig;

BK_API int32_t bkModelCreate(const bkModelConfig* cfg, uint64_t* out_model);
/* Register a weight that already sits in device memory (the caller uploads one slab and addresses
 * it by offset, prototypes/decode.ts:64-75).  Names are the reference's graph names
 * (src/model.ts:72-196): "embed.weight", "final.norm.weight", "model.layers.N.input_layernorm.weight",
 * "...linear_attn.in_proj_qkv.weight" and so on.  Linear weights are Q4_K rows. */
BK_API int32_t bkModelSetTensor(uint64_t model, const char* name, uint64_t dev_ptr, uint64_t bytes);
/* Tensor parallelism (tp_size > 1): give the model its exchange object before bkModelFinalize.  Each rank registers
 * only its shard of every weight: column-parallel matrices keep the rows of the rank's heads / FFN columns /
 * vocabulary rows, row-parallel matrices (out_proj, o_proj, down_proj) keep all rows and the rank's K slice; the
 * embedding table is registered whole (replicated).  Shard shapes are derived from the config by the rule in
 * bunker_b200/model.py `shard_weights`. */
BK_API int32_t bkModelSetComm(uint64_t model, uint64_t comm);
/* How the decode step is issued (before bkModelFinalize).  0: the library's choice (currently 1); 1: one launch per
 * op, the shape of the reference's loop (src/runner.ts:146-149), chained with programmatic dependent launch; 2: the
 * persistent step kernel -- a few cooperative launches per token that run the ops as phases with device-side barriers
 * (batch 1 on one GPU only; bkModelFinalize fails if the model's shapes do not fit it).  All modes give the same bits. */
BK_API int32_t bkModelSetStepMode(uint64_t model, int32_t mode);
/* Checks the tensor set, allocates state and activations, captures the step graphs.  With tp_size > 1 every rank
 * must call it at about the same time: it runs one step, which exchanges with the peers. */
BK_API int32_t bkModelFinalize(uint64_t model);
/* Zero the recurrent state, conv state, KV cache and position.  Also the way back after bkSync reported
 * BK_ERR_TIMEOUT for a decode step (a step that gave up leaves the state half-written). */
BK_API int32_t bkModelReset(uint64_t model);
/* One decode step (runGraphDecode's loop body, src/runner.ts:133-160).  tokens: B host ints, or NULL to
 * feed back the previous step's argmax on the device.  out_ids / out_vals: B host values each, or NULL to
 * skip the read-back (and its synchronisation). */
BK_API int32_t bkDecodeStep(uint64_t model, const int32_t* tokens, int32_t* out_ids, float* out_vals);
/* T prompt tokens of every sequence in one call (tokens host int32 [T][B], T*B <= 64; longer prompts in chunks):
 * the projections run once over T*B columns, the recurrent parts (conv1d + GDN state, KV append + attention) token
 * after token.  State and results are bit-identical to T calls of bkDecodeStep; out_ids/out_vals (optional) are the
 * argmax after the last token.  Replaces the token-by-token prompt loop of prototypes/decode.ts:952-1061.
 * Single-GPU models only. */
BK_API int32_t bkModelPrefill(uint64_t model, const int32_t* tokens, int32_t T, int32_t* out_ids, float* out_vals);
/* n_steps greedy steps with device-side token feedback and no host traffic. */
BK_API int32_t bkDecodeRun(uint64_t model, int32_t n_steps);
/* One eagerly launched step with a CUDA-event pair around every op (the BUNKER_GPU_PROF=1 profiler of
 * src/ttir.ts:352-417).  ms_out/count_out[n_classes >= 11]: 0 embed, 1 projection GEMV (qkv|z|a|b, q|k|v),
 * 2 conv1d+GDN, 3 attention (2 kernels per call), 4 out/o_proj GEMV, 5 gate|up GEMV, 6 down GEMV, 7 lm_head GEMV, 8 argmax,
 * 9 tensor-parallel exchanges, 10 stand-alone norm+quantise launches (batch >= 2 only). */
BK_API int32_t bkDecodeStepProfiled(uint64_t model, float* ms_out, int32_t* count_out, int32_t n_classes);
/* Tokens produced by steps [first_step, first_step+n_steps): out[n_steps][B] host ints. */
BK_API int32_t bkModelTokens(uint64_t model, int32_t first_step, int32_t n_steps, int32_t* out);
BK_API int32_t bkModelInfo(uint64_t model, int32_t* split_len, int32_t* attn_warps, int32_t* kernels_per_step,
                           int64_t* steps);
/* Device address of an internal buffer: "logits" f32 [B][vocab], "ids", "pos", "x0", "x1". */
BK_API int32_t bkModelBuffer(uint64_t model, const char* name, uint64_t* out_ptr);
BK_API int32_t bkModelDestroy(uint64_t model);

/* ---- tensor-parallel exchange over NVLink peer memory (no counterpart in the reference, which is single-GPU) ----
 * One process per GPU.  Each rank creates a communicator, exports its 64-byte IPC handle, the host gathers the handles
 * of all ranks in rank order (nranks x 64 bytes) and hands them to bkCommImportPeers.  payload_bytes must hold the largest
 * exchanged vector: batch x hidden x 4. */
BK_API int32_t bkCommCreate(int32_t rank, int32_t nranks, uint64_t payload_bytes, uint64_t* out_comm);
BK_API int32_t bkCommExportHandle(uint64_t comm, uint8_t* out_handle64);
BK_API int32_t bkCommImportPeers(uint64_t comm, const uint8_t* handles);
BK_API int32_t bkCommDestroy(uint64_t comm);
/* out bf16[n] = (partials of all ranks summed in rank order) + residual; every rank calls it with the same slot (0..2)
 * and n; consecutive calls must use different slots. */
BK_API int32_t bkCommAllReduceResidual(uint64_t comm, int32_t slot, uint64_t partial_f32, int32_t n, uint64_t residual_bf16,
                                       uint64_t out_bf16);

/* cuLaunch-shaped entry (src/ttir.ts:321-348): op id + 8-byte argument slots.
 * Slot lists per op: the comment beside every case of bkLaunch in bunker_b200/csrc/bk_launch.cu. */
BK_API int32_t bkLaunch(int32_t op, const uint64_t* slots, int32_t nslots);
#define BK_OP_EMBED 1
#define BK_OP_RMSNORM 2
#define BK_OP_GEMV 3
#define BK_OP_SWIGLU 4
#define BK_OP_CONV1D 5
#define BK_OP_ARGMAX 6
#define BK_OP_QUANT_Q8_1 7
#define BK_OP_HEADNORM_ROPE 8 /* qnorm+rope / knorm+ropek */
#define BK_OP_GDN 9           /* conv1d_decode + gdn_delta_rule + gated norm */
#define BK_OP_ATTN 10         /* qnorm/knorm/rope + KV append + fa2_attn + gate */
#define BK_OP_QUANT_Q8_1_BF16 11 /* quant_q8_1 on bf16 rows (the activation format between ops) */

#ifdef __cplusplus
}
#endif
#endif /* BUNKER_CUDA_H */
