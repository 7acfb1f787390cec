// bk_model.cu -- the whole hybrid decode step behind one call per token.
//
// Stands where bunker's graph executor stands: buildModelGraph (src/model.ts:46-204) declares the
// per-token DAG and runGraphDecode (src/runner.ts:116-162) launches ~287 kernels per token from
// TypeScript.  bunker found that replaying a CUDA graph through bun:ffi crashes (LOG.md:710-738), so
// here the graph is captured and replayed inside the library and the host makes one call per token.
//
// Step (tp_size = 1), per layer:
//   GDN layer      : [RMSNorm+Q8_1 | qkv,z,a,b GEMV] -> [conv1d+GDN] -> [Q8_1 | out_proj GEMV + residual]
//   attention layer: [RMSNorm+Q8_1 | q,k,v GEMV] -> [norm+rope+append+split attention] -> [combine+gate]
//                    -> [Q8_1 | o_proj GEMV + residual]
//   MLP            : [RMSNorm+Q8_1 | gate,up GEMV + SwiGLU] -> [Q8_1 | down GEMV + residual]
// then [RMSNorm+Q8_1 | lm_head GEMV] -> [argmax, token feedback, pos++].
// Layer kind: layer % interval == interval-1 is full attention (src/model.ts:61).
#include <string.h>

#include <string>
#include <unordered_map>
#include <vector>

#include "bk_common.cuh"
#include "bk_internal.h"

namespace {

struct Tensor {
  uint64_t ptr = 0;
  uint64_t bytes = 0;
};

struct LayerW {
  bool full = false;
  uint64_t in_ln = 0, post_ln = 0;
  // GDN
  uint64_t qkv = 0, z = 0, a = 0, b = 0, conv_w = 0, A_log = 0, dt_bias = 0, gnorm = 0, out_proj = 0;
  // attention
  uint64_t q = 0, k = 0, v = 0, q_norm = 0, k_norm = 0, o = 0;
  // MLP
  uint64_t gate = 0, up = 0, down = 0;
  // state (owned by the model)
  uint64_t conv_state[2] = {0, 0}, S = 0, kc = 0, vc = 0;
};

struct Model {
  bkModelConfig cfg;
  std::unordered_map<std::string, Tensor> tensors;
  std::vector<LayerW> layers;
  uint64_t embed = 0, final_norm = 0;
  bool finalized = false;
  int B = 0;
  // derived, per rank
  int Hk = 0, Hv = 0, Hq = 0, Hkv = 0, Cw = 0, ZD = 0, QG = 0, KVD = 0, inter = 0, vocab_local = 0;
  int split_len = 0;
  int vocab_offset = 0;   // first vocabulary row of this rank's lm_head shard
  uint64_t comm = 0;      // tensor-parallel exchange (bk_comm.cu), 0 for a single GPU
  int tp = 1, rank = 0;
  uint64_t lval = 0, lidx = 0;  // per-rank argmax before the merge
  // device buffers
  std::vector<uint64_t> owned;
  uint64_t x[2] = {0, 0}, h1 = 0, qkv = 0, z = 0, a = 0, b = 0, attn_out = 0, attn_q8 = 0, xq = 0, qg = 0, kbuf = 0, vbuf = 0, act = 0;
  uint64_t logits = 0, ids = 0, val = 0, pos = 0, hist = 0, argmax_scratch = 0, attn_scratch = 0, cos_t = 0, sin_t = 0;
  int32_t* pin_ids = nullptr;  // pinned, mapped into the device: 2 x B ids in (one slot per graph parity), B ids out,
                               // B vals (float bits)
  cudaEvent_t pin_read[2] = {nullptr, nullptr};   // recorded after the step that reads ids slot p
  bool pin_busy[2] = {false, false};
  uint64_t pin_dev = 0;        // device address of pin_ids
  cudaGraphExec_t graph[2] = {nullptr, nullptr};       // token fed back on the device (embed reads m.ids)
  cudaGraphExec_t graph_host[2] = {nullptr, nullptr};  // token from the host (embed reads the mapped pinned ids)
  unsigned long long graph_kernels = 0;
  // persistent step (batch 1, one GPU): the phases of the plan run as a few cooperative launches, with the attention
  // kernel between them
  int step_mode = 0;    // 0 = library's choice, 1 = one launch per op, 2 = persistent step kernel
  uint64_t plan = 0;
  struct StepItem { int kind; int first, count; int layer; };   // kind 0: phases [first, first+count) of the plan; 1: attention of `layer`
  std::vector<StepItem> items;
  long long steps = 0;  // steps taken since the last reset (host mirror of pos)
  int conv_cur = 0;     // which of the two conv-state buffers is current (flips with every decode step / prompt pass)
  // buffers of the multi-token prompt path (bkModelPrefill), sized for `cols` = tokens x sequences columns
  struct Prefill {
    int cols = 0;
    uint64_t x[2] = {0, 0}, h1 = 0, qkv = 0, z = 0, a = 0, b = 0, attn_out = 0, qg = 0, kbuf = 0, vbuf = 0, act = 0, xq = 0;
    uint64_t ids = 0, pos = 0;   // int32 [cols]: token ids, position of every column
    uint64_t attn_scratch = 0;   // split partials and completion counters for `cols` attention entries
  } pf;
};

int32_t dev_alloc(Model& m, size_t bytes, uint64_t* out, bool zero = true) {
  void* p = nullptr;
  BK_CUDA(cudaMalloc(&p, bytes ? bytes : 16));
  if (zero) BK_CUDA(cudaMemsetAsync(p, 0, bytes ? bytes : 16, bk_ctx().stream));
  *out = (uint64_t)(uintptr_t)p;
  m.owned.push_back(*out);
  return BK_OK;
}

int32_t need(Model& m, const std::string& name, uint64_t bytes, uint64_t* out) {
  auto it = m.tensors.find(name);
  if (it == m.tensors.end()) return bk_fail(BK_ERR_STATE, "bkModelFinalize: tensor '%s' was never set", name.c_str());
  if (it->second.bytes != bytes)
    return bk_fail(BK_ERR_ARG, "bkModelFinalize: tensor '%s' has %llu bytes, expected %llu", name.c_str(),
                   (unsigned long long)it->second.bytes, (unsigned long long)bytes);
  if (it->second.ptr & 15) return bk_fail(BK_ERR_ARG, "bkModelFinalize: tensor '%s' is not 16-byte aligned", name.c_str());
  *out = it->second.ptr;
  return BK_OK;
}

inline uint64_t q4k_bytes(uint64_t n, uint64_t k) { return n * (k / 256) * 144; }

#define TRY(expr)            \
  do {                       \
    int32_t _rc = (expr);    \
    if (_rc) return _rc;     \
  } while (0)

// Per-op CUDA-event pairs for one eagerly launched step, the analogue of the reference's
// BUNKER_GPU_PROF=1 profiler (src/ttir.ts:352-417).  Classes index the ms/count arrays of
// bkDecodeStepProfiled.
enum ProfClass { PC_EMBED = 0, PC_GEMV_PROJ, PC_GDN, PC_ATTN, PC_GEMV_OUT, PC_GEMV_GATEUP, PC_GEMV_DOWN, PC_GEMV_LMHEAD,
                 PC_ARGMAX, PC_EXCHANGE, PC_QUANT, PC_COUNT };

struct Prof {
  bool on = false;
  std::vector<cudaEvent_t> ev;
  std::vector<int> cls;
};
Prof g_prof;

struct ProfScope {
  bool on;
  explicit ProfScope(int cls) : on(g_prof.on) {
    if (!on) return;
    cudaEvent_t a, b;
    cudaEventCreate(&a);
    cudaEventCreate(&b);
    cudaEventRecord(a, bk_ctx().stream);
    g_prof.ev.push_back(a);
    g_prof.ev.push_back(b);
    g_prof.cls.push_back(cls);
  }
  ~ProfScope() {
    if (on) cudaEventRecord(g_prof.ev.back(), bk_ctx().stream);
  }
};
#define PROF(cls, expr)    \
  do {                     \
    ProfScope _ps(cls);    \
    TRY(expr);             \
  } while (0)


// arguments of the attention launch of layer L for the decode step (one token per sequence)
bkAttnArgs step_attn_args(Model& m, LayerW& L, bool q8_handoff, bool o_staged) {
  const bkModelConfig& c = m.cfg;
  bkAttnArgs aa;
  memset(&aa, 0, sizeof(aa));
  aa.qg = m.qg; aa.k = m.kbuf; aa.v = m.vbuf; aa.q_norm_w = L.q_norm; aa.k_norm_w = L.k_norm;
  aa.cos_t = m.cos_t; aa.sin_t = m.sin_t; aa.k_cache = L.kc; aa.v_cache = L.vc; aa.pos = m.pos;
  aa.out = m.attn_out; aa.out_q8 = q8_handoff ? m.attn_q8 : 0; aa.out_q8_layout = o_staged ? BK_Q8_STAGED : BK_Q8_BLOCKS;
  aa.scratch = m.attn_scratch;
  aa.B = m.B; aa.Hq = m.Hq; aa.Hkv = m.Hkv; aa.HD = c.head_dim; aa.rot_half = c.rot_dim / 2; aa.max_len = c.max_len;
  aa.split_len = m.split_len; aa.max_pos = c.max_len - 1; aa.scale = 1.0f / sqrtf((float)c.head_dim);
  aa.fused_norm_rope = 1;
  aa.cache_is_settled = 1;  // pos and the older cache rows were written a whole step ago
  return aa;
}

// The batch-1 single-GPU step as a plan for the persistent kernel (bk_persist.cu): the same ops in the same order as
// enqueue_step, every GEMV and GDN launch becoming a phase; the attention kernel stays a launch of its own and cuts
// the plan into segments.  Leaves m.plan = 0 when a shape does not fit the persistent kernel.
int32_t build_plan(Model& m) {
  const bkModelConfig& c = m.cfg;
  const int H = c.hidden, attn_w = m.Hq * c.head_dim;
  if (H > 8192) return BK_OK;
  TRY(bk_plan_create(&m.plan, H));
  if (!bk_plan_gemv_fits(m.plan, H) || !bk_plan_gemv_fits(m.plan, m.ZD) || !bk_plan_gemv_fits(m.plan, attn_w) ||
      !bk_plan_gemv_fits(m.plan, m.inter)) {
    bk_plan_destroy(m.plan);
    m.plan = 0;
    return BK_OK;
  }
  int cur = 0, seg_first = 0;
  auto close_segment = [&]() {
    const int n = bk_plan_count(m.plan) - seg_first;
    if (n > 0) m.items.push_back(Model::StepItem{0, seg_first, n, -1});
    seg_first = bk_plan_count(m.plan);
  };
  auto gemv = [&](uint64_t x, int K, uint64_t norm_w) {
    bkGemvArgs g;
    memset(&g, 0, sizeof(g));
    g.K = K; g.B = 1; g.eps = c.eps; g.x = x; g.norm_w = norm_w;
    g.prologue = norm_w ? BK_PRO_RMSNORM : BK_PRO_BF16;
    return g;
  };
  for (int li = 0; li < c.n_layers; li++) {
    LayerW& L = m.layers[li];
    const int first_flags = li == 0 ? BK_PF_EMBED : 0;
    bkGemvArgs g = gemv(m.x[cur], H, L.in_ln);
    if (!L.full) {
      g.n_segs = 4;
      g.segs[0] = bkGemvSeg{L.qkv, 0, m.qkv, 0, m.Cw, BK_EPI_BF16, m.Cw, 0};
      g.segs[1] = bkGemvSeg{L.z, 0, m.z, 0, m.ZD, BK_EPI_BF16, m.ZD, 0};
      g.segs[2] = bkGemvSeg{L.a, 0, m.a, 0, m.Hv, BK_EPI_F32, m.Hv, 0};
      g.segs[3] = bkGemvSeg{L.b, 0, m.b, 0, m.Hv, BK_EPI_F32, m.Hv, 0};
      TRY(bk_plan_add_gemv(m.plan, g, first_flags));
      bkGdnArgs ga;
      memset(&ga, 0, sizeof(ga));
      ga.qkv = m.qkv; ga.z = m.z; ga.a = m.a; ga.b = m.b;
      ga.conv_w = L.conv_w; ga.conv_state_in = L.conv_state[0]; ga.conv_state_new = L.conv_state[1];
      ga.A_log = L.A_log; ga.dt_bias = L.dt_bias; ga.norm_w = L.gnorm;
      ga.S_in = L.S; ga.S_new = L.S;
      ga.out = m.attn_out; ga.B = 1; ga.Hk = m.Hk; ga.Hv = m.Hv; ga.apply_conv = 1; ga.state_is_settled = 1;
      TRY(bk_plan_add_gdn(m.plan, ga));
      g = gemv(m.attn_out, m.ZD, 0);
      g.n_segs = 1;
      g.segs[0] = bkGemvSeg{L.out_proj, 0, m.h1, m.x[cur], H, BK_EPI_ADD_BF16, H, 0};
      TRY(bk_plan_add_gemv(m.plan, g, 0));
    } else {
      g.n_segs = 3;
      g.segs[0] = bkGemvSeg{L.q, 0, m.qg, 0, m.QG, BK_EPI_BF16, m.QG, 0};
      g.segs[1] = bkGemvSeg{L.k, 0, m.kbuf, 0, m.KVD, BK_EPI_BF16, m.KVD, 0};
      g.segs[2] = bkGemvSeg{L.v, 0, m.vbuf, 0, m.KVD, BK_EPI_BF16, m.KVD, 0};
      TRY(bk_plan_add_gemv(m.plan, g, first_flags));
      close_segment();
      m.items.push_back(Model::StepItem{1, 0, 0, li});
      g = gemv(m.attn_out, attn_w, 0);
      g.n_segs = 1;
      g.segs[0] = bkGemvSeg{L.o, 0, m.h1, m.x[cur], H, BK_EPI_ADD_BF16, H, 0};
      TRY(bk_plan_add_gemv(m.plan, g, 0));
    }
    g = gemv(m.h1, H, L.post_ln);
    g.n_segs = 1;
    g.segs[0] = bkGemvSeg{L.gate, L.up, m.act, 0, m.inter, BK_EPI_SWIGLU, m.inter, 0};
    TRY(bk_plan_add_gemv(m.plan, g, 0));
    g = gemv(m.act, m.inter, 0);
    g.n_segs = 1;
    g.segs[0] = bkGemvSeg{L.down, 0, m.x[cur ^ 1], m.h1, H, BK_EPI_ADD_BF16, H, 0};
    TRY(bk_plan_add_gemv(m.plan, g, 0));
    cur ^= 1;
  }
  bkGemvArgs g = gemv(m.x[cur], H, m.final_norm);
  g.n_segs = 1;
  g.segs[0] = bkGemvSeg{m.embed, 0, m.logits, 0, m.vocab_local, BK_EPI_F32, m.vocab_local, 0};
  TRY(bk_plan_add_gemv(m.plan, g, BK_PF_ARGMAX));
  close_segment();
  TRY(bk_plan_finish(m.plan));
  return BK_OK;
}

int32_t enqueue_step_persist(Model& m, int parity, bool host_tokens) {
  const bkModelConfig& c = m.cfg;
  const bool mapped_io = m.pin_dev != 0;
  BkStepIO io;
  memset(&io, 0, sizeof(io));
  io.embed = m.embed;
  io.ids_in = (host_tokens && mapped_io) ? m.pin_dev + (uint64_t)parity * 4 : m.ids;
  io.x0 = m.x[0];
  io.ids_out = m.ids; io.val_out = m.val; io.pos = m.pos; io.hist = m.hist;
  io.host_out = mapped_io ? m.pin_dev + (uint64_t)2 * 4 : 0;
  io.H = c.hidden; io.hist_ld = 1; io.hist_rows = c.max_len; io.vocab_offset = 0;
  for (const Model::StepItem& it : m.items) {
    if (it.kind == 0) {
      TRY(bk_plan_launch(m.plan, it.first, it.count, parity, io));
    } else {
      bkAttnArgs aa = step_attn_args(m, m.layers[it.layer], false, false);
      TRY(bkAttnDecode(&aa));
    }
  }
  return BK_OK;
}

// enqueue one decode step on the library stream; parity selects the conv-state buffer pair
int32_t enqueue_step(Model& m, int parity, bool host_tokens = false) {
  if (m.plan && !g_prof.on) return enqueue_step_persist(m, parity, host_tokens);
  const bkModelConfig& c = m.cfg;
  const int B = m.B, H = c.hidden;
  int cur = 0;
  // GDN / attention also emit their output as Q8_1 blocks.  Reading those spares the output projection its own
  // quantisation, which pays once that prologue covers several batch rows; at batch 1-2 the bf16 row is as fast.
  const bool q8_handoff = B >= 2;
  // the staged layout serves groups of 2..8 columns on the tensor-core kernel; a last group of one column (B = 9, 17, ...)
  // or a K too wide for that kernel reads plain blocks instead
  // from 16 sequences on (one GPU) the projections of many rows run on the dense tile kernel, which reads plain blocks
  // (the library's rule for BK_GEMV_ORDER_AUTO, bk_gemv_auto_tile)
  const bool tile_path = B >= 16 && m.tp == 1;
  const int gemv_order = tile_path ? BK_GEMV_ORDER_AUTO : BK_GEMV_ORDER_LANES;
  auto staged_ok = [&](int K, int rows) {
    return !(tile_path && bk_gemv_auto_tile(rows, K)) && bk_gemv_mma_fits(K, B < 8 ? B : 8) && !(B > 8 && B % 8 == 1);
  };
  // Input of a projection: fused RMSNorm/quantise prologue at batch 1; at batch >= 2 one small launch
  // normalises and quantises the rows once and every CTA of the projection just copies the blocks.
  // Tensor parallel: a row-parallel GEMV pushes its partial sums to every rank (BK_EPI_PUSH_F32); the sum over ranks,
  // the residual add and the bf16 rounding happen in the prologue of whatever reads the result next (`pending`).
  struct Pending { bool on; int slot; unsigned int tag_add; uint64_t res, out; } pending = {false, 0, 0, 0, 0};
  unsigned int n_exchanges = 0;   // fused exchanges enqueued so far in this step
  BkReduce red_desc;
  bool use_red = false;   // the GEMV being set up carries the reduce prologue (batch 1)
  auto set_input = [&](bkGemvArgs& g, uint64_t x, int K, uint64_t norm_w, int rows) -> int32_t {
    g.K = K; g.B = B; g.eps = c.eps; g.order = gemv_order;
    use_red = false;
    const bool reduce = pending.on && norm_w && x == pending.out;
    if (reduce) {
      TRY(bk_comm_reduce_desc(m.comm, pending.slot, &red_desc));
      red_desc.res = bk_ptr<uint16_t>(pending.res);
      red_desc.out = bk_ptr<uint16_t>(pending.out);
      red_desc.tag_add = pending.tag_add;
      pending.on = false;
    }
    if (q8_handoff) {
      const bool staged = staged_ok(K, rows);   // else the GEMV is cut along K (or runs as column pairs) reading plain blocks
      PROF(PC_QUANT, bk_quant_rows_launch(x, norm_w, K, B, c.eps, m.xq, staged ? BK_Q8_STAGED : BK_Q8_BLOCKS,
                                          reduce ? &red_desc : nullptr));
      g.prologue = staged ? BK_PRO_STAGED : BK_PRO_Q8; g.x = m.xq;
    } else {
      g.prologue = reduce ? BK_PRO_REDUCE_RMSNORM : norm_w ? BK_PRO_RMSNORM : BK_PRO_BF16; g.x = x; g.norm_w = norm_w;
      use_red = reduce;
    }
    return BK_OK;
  };
  auto launch = [&](const bkGemvArgs& g) -> int32_t { return bk_gemv_launch_tp(g, nullptr, use_red ? &red_desc : nullptr, nullptr); };
  // row-parallel GEMV of a tensor-parallel model: push the partials, remember who adds the residual
  auto launch_push = [&](bkGemvArgs& g, uint64_t W, int slot, uint64_t res, uint64_t out) -> int32_t {
    BkPush ps;
    TRY(bk_comm_push_desc(m.comm, slot, &ps));
    ps.tag_add = ++n_exchanges;
    BK_ARG(n_exchanges < 256, "decode step: more than 255 tensor-parallel exchanges");
    g.segs[0] = bkGemvSeg{W, 0, 0, 0, H, BK_EPI_PUSH_F32, H, 0};
    TRY(bk_gemv_launch_tp(g, &ps, use_red ? &red_desc : nullptr, nullptr));
    pending = Pending{true, slot, ps.tag_add, res, out};
    return BK_OK;
  };
  // single GPU: the step talks to the host through mapped pinned memory -- the embed kernel can read the host's
  // tokens there and the argmax kernel always leaves (id, logit) there -- so a step with host I/O is one graph launch
  // and one synchronisation, no copy-engine operations
  const bool mapped_io = m.tp == 1 && m.pin_dev != 0;
  PROF(PC_EMBED, bkEmbedQ4K(m.embed, H, (host_tokens && mapped_io) ? m.pin_dev + (uint64_t)parity * B * 4 : m.ids, B, m.x[0]));
  for (int li = 0; li < c.n_layers; li++) {
    LayerW& L = m.layers[li];
    bkGemvArgs g;
    if (!L.full) {
      memset(&g, 0, sizeof(g));
      TRY(set_input(g, m.x[cur], H, L.in_ln, m.Cw + m.ZD + 2 * m.Hv));
      g.n_segs = 4;
      g.segs[0] = bkGemvSeg{L.qkv, 0, m.qkv, 0, m.Cw, BK_EPI_BF16, m.Cw, 0};
      g.segs[1] = bkGemvSeg{L.z, 0, m.z, 0, m.ZD, BK_EPI_BF16, m.ZD, 0};
      g.segs[2] = bkGemvSeg{L.a, 0, m.a, 0, m.Hv, BK_EPI_F32, m.Hv, 0};
      g.segs[3] = bkGemvSeg{L.b, 0, m.b, 0, m.Hv, BK_EPI_F32, m.Hv, 0};
      PROF(PC_GEMV_PROJ, launch(g));
      bkGdnArgs ga;
      memset(&ga, 0, sizeof(ga));
      ga.qkv = m.qkv; ga.z = m.z; ga.a = m.a; ga.b = m.b;
      ga.conv_w = L.conv_w; ga.conv_state_in = L.conv_state[parity]; ga.conv_state_new = L.conv_state[parity ^ 1];
      ga.A_log = L.A_log; ga.dt_bias = L.dt_bias; ga.norm_w = L.gnorm;
      ga.S_in = L.S; ga.S_new = L.S;  // in place: each thread rewrites exactly the rows it read
      const bool zd_staged = q8_handoff && staged_ok(m.ZD, H);
      ga.out = m.attn_out; ga.out_q8 = q8_handoff ? m.attn_q8 : 0; ga.out_q8_layout = zd_staged ? BK_Q8_STAGED : BK_Q8_BLOCKS;
      ga.B = B; ga.Hk = m.Hk; ga.Hv = m.Hv; ga.apply_conv = 1;
      ga.state_is_settled = 1;  // this layer's state was last written one whole step ago
      PROF(PC_GDN, bkGdnStep(&ga));
      memset(&g, 0, sizeof(g));
      g.K = m.ZD; g.B = B; g.n_segs = 1; g.order = gemv_order;
      g.prologue = zd_staged ? BK_PRO_STAGED : q8_handoff ? BK_PRO_Q8 : BK_PRO_BF16; g.x = q8_handoff ? m.attn_q8 : m.attn_out;
      if (m.tp == 1) {
        g.segs[0] = bkGemvSeg{L.out_proj, 0, m.h1, m.x[cur], H, BK_EPI_ADD_BF16, H, 0};
        PROF(PC_GEMV_OUT, launch(g));
      } else {
        PROF(PC_GEMV_OUT, launch_push(g, L.out_proj, 0, m.x[cur], m.h1));
      }
    } else {
      memset(&g, 0, sizeof(g));
      TRY(set_input(g, m.x[cur], H, L.in_ln, m.QG + 2 * m.KVD));
      g.n_segs = 3;
      g.segs[0] = bkGemvSeg{L.q, 0, m.qg, 0, m.QG, BK_EPI_BF16, m.QG, 0};
      g.segs[1] = bkGemvSeg{L.k, 0, m.kbuf, 0, m.KVD, BK_EPI_BF16, m.KVD, 0};
      g.segs[2] = bkGemvSeg{L.v, 0, m.vbuf, 0, m.KVD, BK_EPI_BF16, m.KVD, 0};
      PROF(PC_GEMV_PROJ, launch(g));
      const bool o_staged = q8_handoff && staged_ok(m.Hq * c.head_dim, H);
      bkAttnArgs aa = step_attn_args(m, L, q8_handoff, o_staged);
      PROF(PC_ATTN, bkAttnDecode(&aa));
      memset(&g, 0, sizeof(g));
      g.K = m.Hq * c.head_dim; g.B = B; g.n_segs = 1; g.order = gemv_order;
      g.prologue = o_staged ? BK_PRO_STAGED : q8_handoff ? BK_PRO_Q8 : BK_PRO_BF16; g.x = q8_handoff ? m.attn_q8 : m.attn_out;
      if (m.tp == 1) {
        g.segs[0] = bkGemvSeg{L.o, 0, m.h1, m.x[cur], H, BK_EPI_ADD_BF16, H, 0};
        PROF(PC_GEMV_OUT, launch(g));
      } else {
        PROF(PC_GEMV_OUT, launch_push(g, L.o, 0, m.x[cur], m.h1));
      }
    }
    memset(&g, 0, sizeof(g));
    TRY(set_input(g, m.h1, H, L.post_ln, 2 * m.inter));
    g.n_segs = 1;
    g.segs[0] = bkGemvSeg{L.gate, L.up, m.act, 0, m.inter, BK_EPI_SWIGLU, m.inter, 0};
    PROF(PC_GEMV_GATEUP, launch(g));
    memset(&g, 0, sizeof(g));
    TRY(set_input(g, m.act, m.inter, 0, H));
    g.n_segs = 1;
    if (m.tp == 1) {
      g.segs[0] = bkGemvSeg{L.down, 0, m.x[cur ^ 1], m.h1, H, BK_EPI_ADD_BF16, H, 0};
      PROF(PC_GEMV_DOWN, launch(g));
    } else {
      PROF(PC_GEMV_DOWN, launch_push(g, L.down, 1, m.h1, m.x[cur ^ 1]));
    }
    cur ^= 1;
  }
  bkGemvArgs g;
  memset(&g, 0, sizeof(g));
  TRY(set_input(g, m.x[cur], H, m.final_norm, m.vocab_local));
  g.n_segs = 1;
  g.segs[0] = bkGemvSeg{m.embed + (uint64_t)m.vocab_offset * (H / 256) * 144, 0, m.logits, 0, m.vocab_local, BK_EPI_F32,
                        m.vocab_local, 0};
  PROF(PC_GEMV_LMHEAD, launch(g));
  if (m.tp == 1) {
    PROF(PC_ARGMAX, bk_argmax_launch(m.logits, m.vocab_local, B, m.ids, m.val, m.argmax_scratch, m.pos, m.hist, B, c.max_len,
                                     mapped_io ? m.pin_dev + (uint64_t)2 * B * 4 : 0));
  } else {
    PROF(PC_ARGMAX, bk_argmax_launch(m.logits, m.vocab_local, B, m.lidx, m.lval, m.argmax_scratch, 0, 0, 0, 0));
    PROF(PC_EXCHANGE, bk_comm_argmax_merge(m.comm, 2, B, m.lval, m.lidx, m.vocab_offset, m.ids, m.val, m.pos, m.hist, B, c.max_len));
  }
  return BK_OK;
}

// pos_cols[t*B + b] = pos[b] + t
__global__ void prefill_positions_kernel(const int32_t* pos, int32_t* pos_cols, int T, int B) {
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i < T * B) pos_cols[i] = pos[i % B] + i / B;
}
__global__ void advance_positions_kernel(int32_t* pos, int B, int delta) {
  const int b = blockIdx.x * blockDim.x + threadIdx.x;
  if (b < B) pos[b] += delta;
}

int32_t alloc_prefill(Model& m, int cols) {
  if (m.pf.cols >= cols) return BK_OK;
  const bkModelConfig& c = m.cfg;
  const int H = c.hidden, attn_w = m.Hq * c.head_dim;
  const size_t C = (size_t)cols;
  Model::Prefill& f = m.pf;
  TRY(dev_alloc(m, C * H * 2, &f.x[0]));
  TRY(dev_alloc(m, C * H * 2, &f.x[1]));
  TRY(dev_alloc(m, C * H * 2, &f.h1));
  TRY(dev_alloc(m, C * m.Cw * 2, &f.qkv));
  TRY(dev_alloc(m, C * m.ZD * 2, &f.z));
  TRY(dev_alloc(m, C * m.Hv * 4, &f.a));
  TRY(dev_alloc(m, C * m.Hv * 4, &f.b));
  TRY(dev_alloc(m, C * (m.ZD > attn_w ? m.ZD : attn_w) * 2, &f.attn_out));
  TRY(dev_alloc(m, C * m.QG * 2, &f.qg));
  TRY(dev_alloc(m, C * m.KVD * 2, &f.kbuf));
  TRY(dev_alloc(m, C * m.KVD * 2, &f.vbuf));
  TRY(dev_alloc(m, C * m.inter * 2, &f.act));
  int kmax = m.inter > H ? m.inter : H;
  if (m.ZD > kmax) kmax = m.ZD;
  if (attn_w > kmax) kmax = attn_w;
  const size_t blocks = C * kmax / 32 * 36, staged = bk_staged_total_bytes(kmax, cols);
  TRY(dev_alloc(m, blocks > staged ? blocks : staged, &f.xq));
  TRY(dev_alloc(m, C * 4, &f.ids));
  TRY(dev_alloc(m, C * 4, &f.pos));
  TRY(dev_alloc(m, bkAttnScratchBytes(cols, m.Hq, c.head_dim, c.max_len, m.split_len), &f.attn_scratch));
  f.cols = cols;
  return BK_OK;
}

// T prompt tokens of every sequence in one pass: the projections see T*B columns (weights streamed once per 8
// columns instead of once per token); the recurrent parts -- conv1d + GDN state, KV append + attention -- run token
// after token with the decode kernels.  Every column goes through the arithmetic of the decode step, so the state
// and the logits of the last token are bit-identical to T decode steps.  Single GPU only.
int32_t enqueue_prefill(Model& m, int T) {
  const bkModelConfig& c = m.cfg;
  const int B = m.B, H = c.hidden, C = T * B;
  Model::Prefill& f = m.pf;
  auto staged_ok = [&](int K, int cols) { return cols >= 2 && bk_gemv_mma_fits(K, cols < 8 ? cols : 8) && !(cols > 8 && cols % 8 == 1); };
  // quantise `cols` rows once (optionally RMSNorm first) and point the GEMV at the result
  auto set_input = [&](bkGemvArgs& g, uint64_t x, int K, uint64_t norm_w, int cols) -> int32_t {
    g.K = K; g.B = cols; g.eps = c.eps;
    g.order = BK_GEMV_ORDER_LANES;   // every column must get the bits of a single decode step
    if (cols == 1) {
      g.prologue = norm_w ? BK_PRO_RMSNORM : BK_PRO_BF16; g.x = x; g.norm_w = norm_w;
      return BK_OK;
    }
    const bool staged = staged_ok(K, cols);
    TRY(bk_quant_rows_launch(x, norm_w, K, cols, c.eps, f.xq, staged ? BK_Q8_STAGED : BK_Q8_BLOCKS, nullptr));
    g.prologue = staged ? BK_PRO_STAGED : BK_PRO_Q8; g.x = f.xq;
    return BK_OK;
  };
  prefill_positions_kernel<<<(C + 127) / 128, 128, 0, bk_ctx().stream>>>(bk_ptr<int32_t>(m.pos), bk_ptr<int32_t>(f.pos), T, B);
  BK_CHECK_LAUNCH();
  int cur = 0;
  TRY(bkEmbedQ4K(m.embed, H, f.ids, C, f.x[0]));
  for (int li = 0; li < c.n_layers; li++) {
    LayerW& L = m.layers[li];
    bkGemvArgs g;
    memset(&g, 0, sizeof(g));
    TRY(set_input(g, f.x[cur], H, L.in_ln, C));
    if (!L.full) {
      g.n_segs = 4;
      g.segs[0] = bkGemvSeg{L.qkv, 0, f.qkv, 0, m.Cw, BK_EPI_BF16, m.Cw, 0};
      g.segs[1] = bkGemvSeg{L.z, 0, f.z, 0, m.ZD, BK_EPI_BF16, m.ZD, 0};
      g.segs[2] = bkGemvSeg{L.a, 0, f.a, 0, m.Hv, BK_EPI_F32, m.Hv, 0};
      g.segs[3] = bkGemvSeg{L.b, 0, f.b, 0, m.Hv, BK_EPI_F32, m.Hv, 0};
      TRY(bk_gemv_launch(g));
      {   // all T tokens in one launch: the state is read and written once, the taps once
        const int parity = m.conv_cur;
        bkGdnArgs ga;
        memset(&ga, 0, sizeof(ga));
        ga.qkv = f.qkv; ga.z = f.z; ga.a = f.a; ga.b = f.b;
        ga.conv_w = L.conv_w; ga.conv_state_in = L.conv_state[parity]; ga.conv_state_new = L.conv_state[parity ^ 1];
        ga.A_log = L.A_log; ga.dt_bias = L.dt_bias; ga.norm_w = L.gnorm;
        ga.S_in = L.S; ga.S_new = L.S;
        ga.out = f.attn_out; ga.B = B; ga.Hk = m.Hk; ga.Hv = m.Hv; ga.apply_conv = 1; ga.n_tokens = T;
        ga.state_is_settled = 1;   // written by the previous pass, many launches ago
        TRY(bkGdnStep(&ga));
      }
      memset(&g, 0, sizeof(g));
      TRY(set_input(g, f.attn_out, m.ZD, 0, C));
      g.n_segs = 1;
      g.segs[0] = bkGemvSeg{L.out_proj, 0, f.h1, f.x[cur], H, BK_EPI_ADD_BF16, H, 0};
      TRY(bk_gemv_launch(g));
    } else {
      g.n_segs = 3;
      g.segs[0] = bkGemvSeg{L.q, 0, f.qg, 0, m.QG, BK_EPI_BF16, m.QG, 0};
      g.segs[1] = bkGemvSeg{L.k, 0, f.kbuf, 0, m.KVD, BK_EPI_BF16, m.KVD, 0};
      g.segs[2] = bkGemvSeg{L.v, 0, f.vbuf, 0, m.KVD, BK_EPI_BF16, m.KVD, 0};
      TRY(bk_gemv_launch(g));
      const int attn_w = m.Hq * c.head_dim;
      {
        // all columns of the pass in two launches: every column's K/V row is appended first, then column (t, b)
        // attends to rows 0..pos[b]+t of sequence b's cache -- per column the arithmetic of a decode step
        bkAttnArgs aa;
        memset(&aa, 0, sizeof(aa));
        aa.qg = f.qg; aa.k = f.kbuf; aa.v = f.vbuf;
        aa.q_norm_w = L.q_norm; aa.k_norm_w = L.k_norm;
        aa.cos_t = m.cos_t; aa.sin_t = m.sin_t; aa.k_cache = L.kc; aa.v_cache = L.vc; aa.pos = f.pos;
        aa.out = f.attn_out; aa.scratch = f.attn_scratch;
        aa.B = C; aa.Hq = m.Hq; aa.Hkv = m.Hkv; aa.HD = c.head_dim; aa.rot_half = c.rot_dim / 2; aa.max_len = c.max_len;
        aa.split_len = m.split_len; aa.max_pos = c.max_len - 1; aa.scale = 1.0f / sqrtf((float)c.head_dim);
        aa.fused_norm_rope = 1;
        TRY(bk_attn_launch(aa, B, m.pf.cols));
      }
      memset(&g, 0, sizeof(g));
      TRY(set_input(g, f.attn_out, attn_w, 0, C));
      g.n_segs = 1;
      g.segs[0] = bkGemvSeg{L.o, 0, f.h1, f.x[cur], H, BK_EPI_ADD_BF16, H, 0};
      TRY(bk_gemv_launch(g));
    }
    memset(&g, 0, sizeof(g));
    TRY(set_input(g, f.h1, H, L.post_ln, C));
    g.n_segs = 1;
    g.segs[0] = bkGemvSeg{L.gate, L.up, f.act, 0, m.inter, BK_EPI_SWIGLU, m.inter, 0};
    TRY(bk_gemv_launch(g));
    memset(&g, 0, sizeof(g));
    TRY(set_input(g, f.act, m.inter, 0, C));
    g.n_segs = 1;
    g.segs[0] = bkGemvSeg{L.down, 0, f.x[cur ^ 1], f.h1, H, BK_EPI_ADD_BF16, H, 0};
    TRY(bk_gemv_launch(g));
    cur ^= 1;
  }
  // logits and argmax of the last token only
  bkGemvArgs g;
  memset(&g, 0, sizeof(g));
  TRY(set_input(g, f.x[cur] + (uint64_t)(C - B) * H * 2, H, m.final_norm, B));
  g.n_segs = 1;
  g.segs[0] = bkGemvSeg{m.embed, 0, m.logits, 0, m.vocab_local, BK_EPI_F32, m.vocab_local, 0};
  TRY(bk_gemv_launch(g));
  if (T > 1) {
    advance_positions_kernel<<<(B + 127) / 128, 128, 0, bk_ctx().stream>>>(bk_ptr<int32_t>(m.pos), B, T - 1);
    BK_CHECK_LAUNCH();
  }
  TRY(bk_argmax_launch(m.logits, m.vocab_local, B, m.ids, m.val, m.argmax_scratch, m.pos, m.hist, B, c.max_len,
                       m.pin_dev ? m.pin_dev + (uint64_t)2 * B * 4 : 0));
  return BK_OK;
}

int32_t capture(Model& m, int parity, bool host_tokens = false) {
  BkContext& c = bk_ctx();
  cudaGraph_t g = nullptr;
  BK_CUDA(cudaStreamBeginCapture(c.stream, cudaStreamCaptureModeThreadLocal));
  c.capturing = true;
  c.captured = 0;
  int32_t rc = enqueue_step(m, parity, host_tokens);
  c.capturing = false;
  cudaError_t e = cudaStreamEndCapture(c.stream, &g);
  if (rc) {
    if (g) cudaGraphDestroy(g);
    return rc;
  }
  if (e != cudaSuccess) return bk_fail((int32_t)e, "bkModelFinalize: graph capture -> %s", cudaGetErrorString(e));
  m.graph_kernels = c.captured;
  e = cudaGraphInstantiate(host_tokens ? &m.graph_host[parity] : &m.graph[parity], g, 0);
  cudaGraphDestroy(g);
  if (e != cudaSuccess) return bk_fail((int32_t)e, "bkModelFinalize: graph instantiate -> %s", cudaGetErrorString(e));
  return BK_OK;
}

int32_t reset_state(Model& m) {
  cudaStream_t st = bk_ctx().stream;
  const bkModelConfig& c = m.cfg;
  for (auto& L : m.layers) {
    if (!L.full) {
      BK_CUDA(cudaMemsetAsync(bk_ptr<void>(L.conv_state[0]), 0, (size_t)m.B * 3 * m.Cw * 2, st));
      BK_CUDA(cudaMemsetAsync(bk_ptr<void>(L.conv_state[1]), 0, (size_t)m.B * 3 * m.Cw * 2, st));
      BK_CUDA(cudaMemsetAsync(bk_ptr<void>(L.S), 0, (size_t)m.B * m.Hv * 128 * 128 * 4, st));
    } else {
      size_t kv = (size_t)m.B * m.Hkv * c.max_len * c.head_dim * 2;
      BK_CUDA(cudaMemsetAsync(bk_ptr<void>(L.kc), 0, kv, st));
      BK_CUDA(cudaMemsetAsync(bk_ptr<void>(L.vc), 0, kv, st));
    }
  }
  BK_CUDA(cudaMemsetAsync(bk_ptr<void>(m.pos), 0, (size_t)m.B * 4, st));
  BK_CUDA(cudaMemsetAsync(bk_ptr<void>(m.ids), 0, (size_t)m.B * 4, st));
  BK_CUDA(cudaMemsetAsync(bk_ptr<void>(m.hist), 0, (size_t)c.max_len * m.B * 4, st));
  if (m.plan) TRY(bk_plan_reset(m.plan));
  m.steps = 0;
  m.conv_cur = 0;
  return BK_OK;
}

Model* as_model(uint64_t h) { return reinterpret_cast<Model*>(static_cast<uintptr_t>(h)); }

}  // namespace

extern "C" {

int32_t bkModelCreate(const bkModelConfig* cfg, uint64_t* out_model) {
  BK_REQUIRE_INIT();
  BK_ARG(cfg && out_model, "bkModelCreate: null argument");
  bkModelConfig c = *cfg;
  BK_ARG(c.hidden > 0 && c.hidden % 256 == 0, "bkModelCreate: hidden=%d must be a positive multiple of 256", c.hidden);
  BK_ARG(c.n_layers > 0 && c.full_attn_interval > 0, "bkModelCreate: bad layer counts");
  BK_ARG(c.intermediate > 0 && c.intermediate % 256 == 0, "bkModelCreate: intermediate=%d must be a multiple of 256", c.intermediate);
  BK_ARG(c.gdn_k_heads > 0 && c.gdn_v_heads % c.gdn_k_heads == 0, "bkModelCreate: bad GDN head counts");
  BK_ARG(c.attn_q_heads > 0 && c.attn_kv_heads > 0 && c.attn_q_heads % c.attn_kv_heads == 0 &&
             c.attn_q_heads / c.attn_kv_heads <= 8, "bkModelCreate: bad attention head counts");
  BK_ARG(c.head_dim == 256, "bkModelCreate: head_dim=%d unsupported (256)", c.head_dim);
  BK_ARG(c.rot_dim > 0 && c.rot_dim % 2 == 0 && c.rot_dim <= c.head_dim, "bkModelCreate: rot_dim=%d", c.rot_dim);
  BK_ARG(c.batch >= 1 && c.batch <= 64, "bkModelCreate: batch=%d outside 1..64", c.batch);
  BK_ARG(c.max_len >= 1, "bkModelCreate: max_len=%d", c.max_len);
  BK_ARG(c.vocab > 0, "bkModelCreate: vocab=%d", c.vocab);
  BK_ARG(c.tp_size >= 1 && c.tp_size <= 8 && c.tp_rank >= 0 && c.tp_rank < c.tp_size, "bkModelCreate: tp rank %d of %d", c.tp_rank, c.tp_size);
  if (c.tp_size > 1) {
    const int n = c.tp_size;
    BK_ARG(c.gdn_k_heads % n == 0 && c.gdn_v_heads % n == 0 && c.attn_q_heads % n == 0,
           "bkModelCreate: head counts (%d,%d,%d) are not divisible by tp_size=%d", c.gdn_k_heads, c.gdn_v_heads, c.attn_q_heads, n);
    BK_ARG(c.attn_kv_heads % n == 0 || n % c.attn_kv_heads == 0, "bkModelCreate: %d KV heads cannot be split or replicated over %d ranks",
           c.attn_kv_heads, n);
    BK_ARG(c.intermediate / 256 >= n, "bkModelCreate: intermediate=%d has fewer superblocks than ranks", c.intermediate);
  }
  Model* m = new Model();
  m->cfg = c;
  m->B = c.batch;
  m->tp = c.tp_size;
  m->rank = c.tp_rank;
  *out_model = (uint64_t)(uintptr_t)m;
  return BK_OK;
}

int32_t bkModelSetTensor(uint64_t model, const char* name, uint64_t dev_ptr, uint64_t bytes) {
  BK_REQUIRE_INIT();
  BK_ARG(model && name && dev_ptr, "bkModelSetTensor: null argument");
  Model* m = as_model(model);
  BK_ARG(!m->finalized, "bkModelSetTensor: model is already finalized");
  m->tensors[std::string(name)] = Tensor{dev_ptr, bytes};
  return BK_OK;
}

int32_t bkModelSetComm(uint64_t model, uint64_t comm) {
  BK_REQUIRE_INIT();
  BK_ARG(model && comm, "bkModelSetComm: null argument");
  Model* m = as_model(model);
  BK_ARG(!m->finalized, "bkModelSetComm: model is already finalized");
  m->comm = comm;
  return BK_OK;
}

int32_t bkModelSetStepMode(uint64_t model, int32_t mode) {
  BK_REQUIRE_INIT();
  BK_ARG(model && mode >= 0 && mode <= 2, "bkModelSetStepMode: bad arguments");
  Model* m = as_model(model);
  BK_ARG(!m->finalized, "bkModelSetStepMode: model is already finalized");
  m->step_mode = mode;
  return BK_OK;
}

int32_t bkModelFinalize(uint64_t model) {
  BK_REQUIRE_INIT();
  BK_ARG(model, "bkModelFinalize: null model");
  Model& m = *as_model(model);
  if (m.finalized) return BK_OK;
  const bkModelConfig& c = m.cfg;
  const int H = c.hidden, B = m.B;
  // per-rank shard shapes: heads split evenly, KV heads split or replicated, FFN and vocabulary rows split with the
  // remainder going to the lowest ranks (FFN in whole 256-column superblocks)
  const int n = m.tp, r = m.rank;
  if (n > 1) {
    BK_ARG(m.comm != 0, "bkModelFinalize: tp_size=%d needs a communicator (bkModelSetComm)", n);
    int cr = -1, cn = -1;
    TRY(bk_comm_info(m.comm, &cr, &cn));
    BK_ARG(cr == r && cn == n, "bkModelFinalize: communicator is rank %d of %d, model is rank %d of %d", cr, cn, r, n);
  }
  m.Hk = c.gdn_k_heads / n; m.Hv = c.gdn_v_heads / n; m.Hq = c.attn_q_heads / n;
  m.Hkv = c.attn_kv_heads >= n ? c.attn_kv_heads / n : 1;
  m.Cw = 2 * m.Hk * 128 + m.Hv * 128; m.ZD = m.Hv * 128; m.QG = m.Hq * 2 * c.head_dim; m.KVD = m.Hkv * c.head_dim;
  {
    const int nsb = c.intermediate / 256;
    m.inter = (nsb / n + (r < nsb % n ? 1 : 0)) * 256;
    const int vb = c.vocab / n, ve = c.vocab % n;
    m.vocab_local = vb + (r < ve ? 1 : 0);
    m.vocab_offset = r * vb + (r < ve ? r : ve);
  }
  TRY(need(m, "embed.weight", q4k_bytes(c.vocab, H), &m.embed));
  TRY(need(m, "final.norm.weight", (uint64_t)H * 2, &m.final_norm));
  m.layers.resize(c.n_layers);
  for (int li = 0; li < c.n_layers; li++) {
    LayerW& L = m.layers[li];
    L.full = (li % c.full_attn_interval) == c.full_attn_interval - 1;
    std::string p = "model.layers." + std::to_string(li) + ".";
    TRY(need(m, p + "input_layernorm.weight", (uint64_t)H * 2, &L.in_ln));
    TRY(need(m, p + "post_attention_layernorm.weight", (uint64_t)H * 2, &L.post_ln));
    TRY(need(m, p + "mlp.gate_proj.weight", q4k_bytes(m.inter, H), &L.gate));
    TRY(need(m, p + "mlp.up_proj.weight", q4k_bytes(m.inter, H), &L.up));
    TRY(need(m, p + "mlp.down_proj.weight", q4k_bytes(H, m.inter), &L.down));
    if (!L.full) {
      std::string q = p + "linear_attn.";
      TRY(need(m, q + "in_proj_qkv.weight", q4k_bytes(m.Cw, H), &L.qkv));
      TRY(need(m, q + "in_proj_z.weight", q4k_bytes(m.ZD, H), &L.z));
      TRY(need(m, q + "in_proj_a.weight", q4k_bytes(m.Hv, H), &L.a));
      TRY(need(m, q + "in_proj_b.weight", q4k_bytes(m.Hv, H), &L.b));
      TRY(need(m, q + "conv1d.weight", (uint64_t)m.Cw * 4 * 2, &L.conv_w));
      TRY(need(m, q + "A_log", (uint64_t)m.Hv * 4, &L.A_log));
      TRY(need(m, q + "dt_bias", (uint64_t)m.Hv * 2, &L.dt_bias));
      TRY(need(m, q + "norm.weight", 128 * 4, &L.gnorm));
      TRY(need(m, q + "out_proj.weight", q4k_bytes(H, m.ZD), &L.out_proj));
      TRY(dev_alloc(m, (size_t)B * 3 * m.Cw * 2, &L.conv_state[0]));
      TRY(dev_alloc(m, (size_t)B * 3 * m.Cw * 2, &L.conv_state[1]));
      TRY(dev_alloc(m, (size_t)B * m.Hv * 128 * 128 * 4, &L.S));
    } else {
      std::string q = p + "self_attn.";
      TRY(need(m, q + "q_proj.weight", q4k_bytes(m.QG, H), &L.q));
      TRY(need(m, q + "k_proj.weight", q4k_bytes(m.KVD, H), &L.k));
      TRY(need(m, q + "v_proj.weight", q4k_bytes(m.KVD, H), &L.v));
      TRY(need(m, q + "q_norm.weight", (uint64_t)c.head_dim * 2, &L.q_norm));
      TRY(need(m, q + "k_norm.weight", (uint64_t)c.head_dim * 2, &L.k_norm));
      TRY(need(m, q + "o_proj.weight", q4k_bytes(H, (uint64_t)m.Hq * c.head_dim), &L.o));
      size_t kv = (size_t)B * m.Hkv * c.max_len * c.head_dim * 2;
      TRY(dev_alloc(m, kv, &L.kc));
      TRY(dev_alloc(m, kv, &L.vc));
    }
  }
  int attn_w = m.Hq * c.head_dim;
  TRY(dev_alloc(m, (size_t)B * H * 2, &m.x[0]));
  TRY(dev_alloc(m, (size_t)B * H * 2, &m.x[1]));
  TRY(dev_alloc(m, (size_t)B * H * 2, &m.h1));
  TRY(dev_alloc(m, (size_t)B * m.Cw * 2, &m.qkv));
  TRY(dev_alloc(m, (size_t)B * m.ZD * 2, &m.z));
  TRY(dev_alloc(m, (size_t)B * m.Hv * 4, &m.a));
  TRY(dev_alloc(m, (size_t)B * m.Hv * 4, &m.b));
  TRY(dev_alloc(m, (size_t)B * (m.ZD > attn_w ? m.ZD : attn_w) * 2, &m.attn_out));
  {  // quantised handoff buffers: room for either layout
    const int ka = m.ZD > attn_w ? m.ZD : attn_w, kx = m.inter > H ? m.inter : H;
    const size_t ba = (size_t)B * ka / 32 * 36, bx = (size_t)B * kx / 32 * 36;
    const size_t sa = bk_staged_total_bytes(ka, B), sx = bk_staged_total_bytes(kx, B);
    TRY(dev_alloc(m, ba > sa ? ba : sa, &m.attn_q8));
    TRY(dev_alloc(m, bx > sx ? bx : sx, &m.xq));
  }
  TRY(dev_alloc(m, (size_t)B * m.QG * 2, &m.qg));
  TRY(dev_alloc(m, (size_t)B * m.KVD * 2, &m.kbuf));
  TRY(dev_alloc(m, (size_t)B * m.KVD * 2, &m.vbuf));
  TRY(dev_alloc(m, (size_t)B * m.inter * 2, &m.act));
  TRY(dev_alloc(m, (size_t)B * m.vocab_local * 4, &m.logits));
  TRY(dev_alloc(m, (size_t)B * 4, &m.ids));
  TRY(dev_alloc(m, (size_t)B * 4, &m.val));
  TRY(dev_alloc(m, (size_t)B * 4, &m.lval));
  TRY(dev_alloc(m, (size_t)B * 4, &m.lidx));
  TRY(dev_alloc(m, (size_t)B * 4, &m.pos));
  TRY(dev_alloc(m, (size_t)c.max_len * B * 4, &m.hist));
  TRY(dev_alloc(m, bkArgmaxScratchBytes(B), &m.argmax_scratch));
  int32_t sl = 0;
  TRY(bkAttnPlan(c.max_len, B, m.Hkv, &sl, nullptr));
  m.split_len = sl;
  TRY(dev_alloc(m, bkAttnScratchBytes(B, m.Hq, c.head_dim, c.max_len, sl), &m.attn_scratch));
  {
    int half = c.rot_dim / 2;
    std::vector<float> ct((size_t)c.max_len * half), st((size_t)c.max_len * half);
    TRY(bkRopeTables(c.max_len, c.rot_dim, c.rope_theta, ct.data(), st.data()));
    TRY(dev_alloc(m, ct.size() * 4, &m.cos_t, false));
    TRY(dev_alloc(m, st.size() * 4, &m.sin_t, false));
    BK_CUDA(cudaMemcpyAsync(bk_ptr<void>(m.cos_t), ct.data(), ct.size() * 4, cudaMemcpyHostToDevice, bk_ctx().stream));
    BK_CUDA(cudaMemcpyAsync(bk_ptr<void>(m.sin_t), st.data(), st.size() * 4, cudaMemcpyHostToDevice, bk_ctx().stream));
    BK_CUDA(cudaStreamSynchronize(bk_ctx().stream));
  }
  BK_CUDA(cudaHostAlloc((void**)&m.pin_ids, (size_t)B * 4 * 4, cudaHostAllocMapped));
  memset(m.pin_ids, 0, (size_t)B * 4 * 4);
  for (int i = 0; i < 2; i++) BK_CUDA(cudaEventCreateWithFlags(&m.pin_read[i], cudaEventDisableTiming));
  {
    void* dp = nullptr;
    BK_CUDA(cudaHostGetDevicePointer(&dp, m.pin_ids, 0));
    m.pin_dev = (uint64_t)(uintptr_t)dp;
  }
  BK_ARG(m.step_mode != 2 || (B == 1 && m.tp == 1), "bkModelFinalize: the persistent step needs batch 1 on one GPU");
  // The library's own choice (mode 0) is one launch per op: on B200 the programmatic hand-off between dependent
  // launches measures 0.7 us, a device-side barrier over 148 CTAs 1.8 us, and the step is a chain of ~120 of them.
  if (m.step_mode == 2) TRY(build_plan(m));
  BK_ARG(m.step_mode != 2 || m.plan, "bkModelFinalize: this model's shapes do not fit the persistent step kernel");
  // one eager step sets the kernels' shared-memory attributes and validates every pointer, then the
  // state is cleared and the two parity graphs are captured
  TRY(enqueue_step(m, 0));
  BK_CUDA(cudaStreamSynchronize(bk_ctx().stream));
  TRY(reset_state(m));
  TRY(capture(m, 0));
  TRY(capture(m, 1));
  if (m.tp == 1) {
    TRY(capture(m, 0, true));
    TRY(capture(m, 1, true));
  }
  BK_CUDA(cudaStreamSynchronize(bk_ctx().stream));
  m.finalized = true;
  return BK_OK;
}

int32_t bkModelReset(uint64_t model) {
  BK_REQUIRE_INIT();
  BK_ARG(model, "bkModelReset: null model");
  Model& m = *as_model(model);
  BK_ARG(m.finalized, "bkModelReset: model is not finalized");
  return reset_state(m);
}

int32_t bkModelInfo(uint64_t model, int32_t* split_len, int32_t* attn_warps, int32_t* kernels_per_step, int64_t* steps) {
  BK_REQUIRE_INIT();
  BK_ARG(model, "bkModelInfo: null model");
  Model& m = *as_model(model);
  if (split_len) *split_len = m.split_len;
  if (attn_warps) *attn_warps = 8;
  if (kernels_per_step) *kernels_per_step = (int32_t)m.graph_kernels;
  if (steps) *steps = m.steps;
  return BK_OK;
}

static int32_t launch_step(Model& m, bool host_tokens = false) {
  BkContext& c = bk_ctx();
  BK_ARG(m.steps < m.cfg.max_len, "bkDecodeStep: position %lld reached max_len=%d", m.steps, m.cfg.max_len);
  BK_CUDA(cudaGraphLaunch((host_tokens && m.graph_host[m.conv_cur]) ? m.graph_host[m.conv_cur] : m.graph[m.conv_cur], c.stream));
  c.launches += m.graph_kernels;
  m.steps++;
  m.conv_cur ^= 1;
  return BK_OK;
}

int32_t bkDecodeStep(uint64_t model, const int32_t* tokens, int32_t* out_ids, float* out_vals) {
  BK_REQUIRE_INIT();
  BK_ARG(model, "bkDecodeStep: null model");
  Model& m = *as_model(model);
  BK_ARG(m.finalized, "bkDecodeStep: model is not finalized");
  cudaStream_t st = bk_ctx().stream;
  const int B = m.B;
  const bool mapped_io = m.tp == 1 && m.graph_host[0] != nullptr;
  int32_t* const out_slot = m.pin_ids + 2 * B;   // ids out, then vals
  if (tokens) {
    const int p = m.conv_cur;                     // the graph about to run reads ids slot p
    int32_t* in_slot = m.pin_ids + (mapped_io ? p * B : 0);
    if (mapped_io && m.pin_busy[p]) {              // the step before last may still be reading this slot
      BK_CUDA(cudaEventSynchronize(m.pin_read[p]));
      m.pin_busy[p] = false;
    }
    for (int b = 0; b < B; b++) {
      BK_ARG(tokens[b] >= 0 && tokens[b] < m.cfg.vocab, "bkDecodeStep: token %d outside the vocabulary", tokens[b]);
      in_slot[b] = tokens[b];
    }
    if (!mapped_io) BK_CUDA(cudaMemcpyAsync(bk_ptr<void>(m.ids), in_slot, (size_t)B * 4, cudaMemcpyHostToDevice, st));
    TRY(launch_step(m, true));
    if (mapped_io) {
      BK_CUDA(cudaEventRecord(m.pin_read[p], st));
      m.pin_busy[p] = true;
    }
  } else {
    TRY(launch_step(m, false));
  }
  if (out_ids || out_vals) {
    if (!mapped_io) {
      BK_CUDA(cudaMemcpyAsync(out_slot, bk_ptr<void>(m.ids), (size_t)B * 4, cudaMemcpyDeviceToHost, st));
      if (out_vals) BK_CUDA(cudaMemcpyAsync(out_slot + B, bk_ptr<void>(m.val), (size_t)B * 4, cudaMemcpyDeviceToHost, st));
    }
    BK_CUDA(cudaStreamSynchronize(st));
    m.pin_busy[0] = m.pin_busy[1] = false;
    if (out_ids) memcpy(out_ids, out_slot, (size_t)B * 4);
    if (out_vals) memcpy(out_vals, out_slot + B, (size_t)B * 4);
  }
  return BK_OK;
}

int32_t bkDecodeStepProfiled(uint64_t model, float* ms_out, int32_t* count_out, int32_t n_classes) {
  BK_REQUIRE_INIT();
  BK_ARG(model && ms_out && count_out && n_classes >= PC_COUNT, "bkDecodeStepProfiled: need %d classes", (int)PC_COUNT);
  Model& m = *as_model(model);
  BK_ARG(m.finalized, "bkDecodeStepProfiled: model is not finalized");
  BK_ARG(m.steps < m.cfg.max_len, "bkDecodeStepProfiled: position reached max_len");
  g_prof.on = true;
  g_prof.ev.clear();
  g_prof.cls.clear();
  int32_t rc = enqueue_step(m, m.conv_cur);
  g_prof.on = false;
  cudaError_t e = cudaStreamSynchronize(bk_ctx().stream);
  for (int i = 0; i < n_classes; i++) {
    ms_out[i] = 0.0f;
    count_out[i] = 0;
  }
  for (size_t i = 0; i < g_prof.cls.size(); i++) {
    float ms = 0.0f;
    if (!rc && e == cudaSuccess) cudaEventElapsedTime(&ms, g_prof.ev[2 * i], g_prof.ev[2 * i + 1]);
    ms_out[g_prof.cls[i]] += ms;
    count_out[g_prof.cls[i]] += 1;
    cudaEventDestroy(g_prof.ev[2 * i]);
    cudaEventDestroy(g_prof.ev[2 * i + 1]);
  }
  g_prof.ev.clear();
  g_prof.cls.clear();
  if (rc) return rc;
  if (e != cudaSuccess) return bk_fail((int32_t)e, "bkDecodeStepProfiled: %s", cudaGetErrorString(e));
  m.steps++;
  m.conv_cur ^= 1;
  return BK_OK;
}

int32_t bkDecodeStepEager(uint64_t model) {
  BK_REQUIRE_INIT();
  BK_ARG(model, "bkDecodeStepEager: null model");
  Model& m = *as_model(model);
  BK_ARG(m.finalized, "bkDecodeStepEager: model is not finalized");
  BK_ARG(m.steps < m.cfg.max_len, "bkDecodeStepEager: position reached max_len");
  TRY(enqueue_step(m, m.conv_cur));
  m.steps++;
  m.conv_cur ^= 1;
  return BK_OK;
}

int32_t bkModelPrefill(uint64_t model, const int32_t* tokens, int32_t T, int32_t* out_ids, float* out_vals) {
  BK_REQUIRE_INIT();
  BK_ARG(model && tokens && T >= 1, "bkModelPrefill: bad arguments");
  Model& m = *as_model(model);
  BK_ARG(m.finalized, "bkModelPrefill: model is not finalized");
  BK_ARG(m.tp == 1, "bkModelPrefill: single-GPU models only");
  const int B = m.B, C = T * B;
  BK_ARG(C <= 64, "bkModelPrefill: %d tokens x %d sequences exceed 64 columns; feed the prompt in chunks", T, B);
  BK_ARG(m.steps + T <= m.cfg.max_len, "bkModelPrefill: position %lld + %d tokens exceeds max_len=%d", m.steps, T, m.cfg.max_len);
  for (int i = 0; i < C; i++)
    BK_ARG(tokens[i] >= 0 && tokens[i] < m.cfg.vocab, "bkModelPrefill: token %d outside the vocabulary", tokens[i]);
  cudaStream_t st = bk_ctx().stream;
  TRY(alloc_prefill(m, C));
  BK_CUDA(cudaMemcpyAsync(bk_ptr<void>(m.pf.ids), tokens, (size_t)C * 4, cudaMemcpyHostToDevice, st));
  BK_CUDA(cudaStreamSynchronize(st));   // the caller may reuse `tokens` as soon as this returns
  TRY(enqueue_prefill(m, T));
  m.steps += T;
  m.conv_cur ^= 1;
  if (out_ids || out_vals) {
    // the argmax kernel left (id, logit) in the mapped pinned buffer
    BK_CUDA(cudaStreamSynchronize(st));
    if (out_ids) memcpy(out_ids, m.pin_ids + 2 * B, (size_t)B * 4);
    if (out_vals) memcpy(out_vals, m.pin_ids + 3 * B, (size_t)B * 4);
  }
  return BK_OK;
}

int32_t bkDecodeRun(uint64_t model, int32_t n_steps) {
  BK_REQUIRE_INIT();
  BK_ARG(model && n_steps >= 0, "bkDecodeRun: bad arguments");
  Model& m = *as_model(model);
  BK_ARG(m.finalized, "bkDecodeRun: model is not finalized");
  for (int i = 0; i < n_steps; i++) TRY(launch_step(m));
  return BK_OK;
}

int32_t bkModelTokens(uint64_t model, int32_t first_step, int32_t n_steps, int32_t* out) {
  BK_REQUIRE_INIT();
  BK_ARG(model && out, "bkModelTokens: null argument");
  Model& m = *as_model(model);
  BK_ARG(first_step >= 0 && n_steps >= 0 && first_step + n_steps <= m.cfg.max_len, "bkModelTokens: range outside max_len");
  BK_CUDA(cudaMemcpyAsync(out, bk_ptr<int32_t>(m.hist) + (size_t)first_step * m.B, (size_t)n_steps * m.B * 4,
                          cudaMemcpyDeviceToHost, bk_ctx().stream));
  BK_CUDA(cudaStreamSynchronize(bk_ctx().stream));
  return BK_OK;
}

int32_t bkModelBuffer(uint64_t model, const char* name, uint64_t* out_ptr) {
  BK_REQUIRE_INIT();
  BK_ARG(model && name && out_ptr, "bkModelBuffer: null argument");
  Model& m = *as_model(model);
  std::string n(name);
  if (n == "logits") *out_ptr = m.logits;
  else if (n == "ids") *out_ptr = m.ids;
  else if (n == "pos") *out_ptr = m.pos;
  else if (n == "x0") *out_ptr = m.x[0];
  else if (n == "x1") *out_ptr = m.x[1];
  else return bk_fail(BK_ERR_ARG, "bkModelBuffer: unknown buffer '%s'", name);
  return BK_OK;
}

int32_t bkModelDestroy(uint64_t model) {
  BK_REQUIRE_INIT();
  if (!model) return BK_OK;
  Model* m = as_model(model);
  cudaStreamSynchronize(bk_ctx().stream);
  for (int i = 0; i < 2; i++) {
    if (m->graph[i]) cudaGraphExecDestroy(m->graph[i]);
    if (m->graph_host[i]) cudaGraphExecDestroy(m->graph_host[i]);
    if (m->pin_read[i]) cudaEventDestroy(m->pin_read[i]);
  }
  for (uint64_t p : m->owned) cudaFree(bk_ptr<void>(p));
  if (m->plan) bk_plan_destroy(m->plan);
  if (m->pin_ids) cudaFreeHost(m->pin_ids);
  delete m;
  return BK_OK;
}

}  // extern "C"
