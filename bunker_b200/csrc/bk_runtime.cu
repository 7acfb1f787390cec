// bk_runtime.cu -- context, memory, copies, events: the runtime half of the C ABI.
// Replaces the driver-API wrappers of bunker's src/ttir.ts:223-417.
#include <stdarg.h>
#include <string.h>

#include "bk_internal.h"

static BkContext g_ctx;
BkContext& bk_ctx() { return g_ctx; }

int32_t bk_fail(int32_t code, const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(g_ctx.err, sizeof(g_ctx.err), fmt, ap);
  va_end(ap);
  return code;
}

extern "C" {

int32_t bkInit(int32_t device) {
  if (g_ctx.ready) {
    if (g_ctx.device == device) return BK_OK;
    return bk_fail(BK_ERR_STATE, "bkInit: already initialised on device %d", g_ctx.device);
  }
  int n = 0;
  BK_CUDA(cudaGetDeviceCount(&n));
  BK_ARG(device >= 0 && device < n, "bkInit: device %d out of range (%d visible)", device, n);
  BK_CUDA(cudaSetDevice(device));
  cudaDeviceProp prop;
  BK_CUDA(cudaGetDeviceProperties(&prop, device));
  if (prop.major < 10)
    return bk_fail(BK_ERR_UNSUPPORTED, "bkInit: device %d is sm_%d%d; this library holds sm_100a code only", device,
                   prop.major, prop.minor);
  g_ctx.device = device;
  g_ctx.sm_count = prop.multiProcessorCount;
  g_ctx.cc_major = prop.major;
  g_ctx.cc_minor = prop.minor;
  g_ctx.total_mem = prop.totalGlobalMem;
  g_ctx.smem_optin = prop.sharedMemPerBlockOptin;
  BK_CUDA(cudaStreamCreateWithFlags(&g_ctx.stream, cudaStreamNonBlocking));
  BK_CUDA(cudaMalloc((void**)&g_ctx.d_status, sizeof(int)));
  BK_CUDA(cudaMemsetAsync(g_ctx.d_status, 0, sizeof(int), g_ctx.stream));   // ordered on the library stream, then awaited
  g_ctx.tile_scratch_bytes = (size_t)24 << 20;
  BK_CUDA(cudaMalloc((void**)&g_ctx.tile_scratch, g_ctx.tile_scratch_bytes));
  BK_CUDA(cudaMalloc((void**)&g_ctx.tile_counters, 256 * sizeof(int)));
  BK_CUDA(cudaMemsetAsync(g_ctx.tile_counters, 0, 256 * sizeof(int), g_ctx.stream));
  BK_CUDA(cudaStreamSynchronize(g_ctx.stream));
  g_ctx.launches = 0;
  g_ctx.ready = true;
  return BK_OK;
}

int32_t bkShutdown(void) {
  if (!g_ctx.ready) return BK_OK;
  cudaStreamSynchronize(g_ctx.stream);
  cudaStreamDestroy(g_ctx.stream);
  cudaFree(g_ctx.d_status);
  cudaFree(g_ctx.tile_scratch);
  cudaFree(g_ctx.tile_counters);
  g_ctx.d_status = nullptr;
  g_ctx.tile_scratch = nullptr;
  g_ctx.tile_counters = nullptr;
  g_ctx.stream = nullptr;
  g_ctx.ready = false;
  return BK_OK;
}

const char* bkLastError(void) { return g_ctx.err; }

int32_t bkDeviceInfo(int32_t* sm_count, int32_t* cc_major, int32_t* cc_minor, uint64_t* total_mem) {
  BK_REQUIRE_INIT();
  if (sm_count) *sm_count = g_ctx.sm_count;
  if (cc_major) *cc_major = g_ctx.cc_major;
  if (cc_minor) *cc_minor = g_ctx.cc_minor;
  if (total_mem) *total_mem = g_ctx.total_mem;
  return BK_OK;
}

int32_t bkAlloc(uint64_t bytes, uint64_t* out_ptr) {
  BK_REQUIRE_INIT();
  BK_ARG(out_ptr != nullptr, "bkAlloc: out_ptr is null");
  void* p = nullptr;
  BK_CUDA(cudaMalloc(&p, bytes ? bytes : 1));
  *out_ptr = (uint64_t)(uintptr_t)p;
  return BK_OK;
}

int32_t bkFree(uint64_t ptr) {
  BK_REQUIRE_INIT();
  if (!ptr) return BK_OK;
  BK_CUDA(cudaFree(bk_ptr<void>(ptr)));
  return BK_OK;
}

int32_t bkHtoD(uint64_t dst, const void* src, uint64_t bytes) {
  BK_REQUIRE_INIT();
  BK_ARG(dst && src, "bkHtoD: null pointer");
  BK_CUDA(cudaMemcpyAsync(bk_ptr<void>(dst), src, bytes, cudaMemcpyHostToDevice, g_ctx.stream));
  BK_CUDA(cudaStreamSynchronize(g_ctx.stream));
  return BK_OK;
}

int32_t bkDtoH(void* dst, uint64_t src, uint64_t bytes) {
  BK_REQUIRE_INIT();
  BK_ARG(dst && src, "bkDtoH: null pointer");
  BK_CUDA(cudaMemcpyAsync(dst, bk_ptr<void>(src), bytes, cudaMemcpyDeviceToHost, g_ctx.stream));
  BK_CUDA(cudaStreamSynchronize(g_ctx.stream));
  return BK_OK;
}

int32_t bkHtoDAsync(uint64_t dst, const void* src, uint64_t bytes) {
  BK_REQUIRE_INIT();
  BK_ARG(dst && src, "bkHtoDAsync: null pointer");
  BK_CUDA(cudaMemcpyAsync(bk_ptr<void>(dst), src, bytes, cudaMemcpyHostToDevice, g_ctx.stream));
  return BK_OK;
}

int32_t bkDtoHAsync(void* dst, uint64_t src, uint64_t bytes) {
  BK_REQUIRE_INIT();
  BK_ARG(dst && src, "bkDtoHAsync: null pointer");
  BK_CUDA(cudaMemcpyAsync(dst, bk_ptr<void>(src), bytes, cudaMemcpyDeviceToHost, g_ctx.stream));
  return BK_OK;
}

int32_t bkDtoD(uint64_t dst, uint64_t src, uint64_t bytes) {
  BK_REQUIRE_INIT();
  BK_ARG(dst && src, "bkDtoD: null pointer");
  BK_CUDA(cudaMemcpyAsync(bk_ptr<void>(dst), bk_ptr<void>(src), bytes, cudaMemcpyDeviceToDevice, g_ctx.stream));
  return BK_OK;
}

int32_t bkMemset(uint64_t dst, int32_t byte_value, uint64_t bytes) {
  BK_REQUIRE_INIT();
  BK_ARG(dst, "bkMemset: null pointer");
  BK_CUDA(cudaMemsetAsync(bk_ptr<void>(dst), byte_value, bytes, g_ctx.stream));
  return BK_OK;
}

int32_t bkHostAlloc(uint64_t bytes, void** out) {
  BK_REQUIRE_INIT();
  BK_ARG(out != nullptr, "bkHostAlloc: out is null");
  BK_CUDA(cudaHostAlloc(out, bytes ? bytes : 1, cudaHostAllocDefault));
  return BK_OK;
}

int32_t bkHostFree(void* p) {
  BK_REQUIRE_INIT();
  if (p) BK_CUDA(cudaFreeHost(p));
  return BK_OK;
}

int32_t bkSync(void) {
  BK_REQUIRE_INIT();
  BK_CUDA(cudaStreamSynchronize(g_ctx.stream));
  int st = 0;
  BK_CUDA(cudaMemcpy(&st, g_ctx.d_status, sizeof(int), cudaMemcpyDeviceToHost));
  if (st != 0) {
    cudaMemsetAsync(g_ctx.d_status, 0, sizeof(int), g_ctx.stream);
    cudaStreamSynchronize(g_ctx.stream);
    return bk_fail(st, "bkSync: a kernel reported status %d (a bounded device-side wait gave up)", st);
  }
  return BK_OK;
}

int32_t bkEventCreate(uint64_t* out_event) {
  BK_REQUIRE_INIT();
  BK_ARG(out_event != nullptr, "bkEventCreate: out_event is null");
  cudaEvent_t ev;
  BK_CUDA(cudaEventCreate(&ev));
  *out_event = (uint64_t)(uintptr_t)ev;
  return BK_OK;
}

int32_t bkEventRecord(uint64_t event) {
  BK_REQUIRE_INIT();
  BK_CUDA(cudaEventRecord((cudaEvent_t)(uintptr_t)event, g_ctx.stream));
  return BK_OK;
}

int32_t bkEventSync(uint64_t event) {
  BK_REQUIRE_INIT();
  BK_CUDA(cudaEventSynchronize((cudaEvent_t)(uintptr_t)event));
  return BK_OK;
}

int32_t bkEventElapsedMs(uint64_t start, uint64_t stop, float* out_ms) {
  BK_REQUIRE_INIT();
  BK_ARG(out_ms != nullptr, "bkEventElapsedMs: out_ms is null");
  BK_CUDA(cudaEventElapsedTime(out_ms, (cudaEvent_t)(uintptr_t)start, (cudaEvent_t)(uintptr_t)stop));
  return BK_OK;
}

int32_t bkEventDestroy(uint64_t event) {
  BK_REQUIRE_INIT();
  BK_CUDA(cudaEventDestroy((cudaEvent_t)(uintptr_t)event));
  return BK_OK;
}

int32_t bkTraceEnable(uint64_t dev_buf, int32_t max_launches) {
  BK_REQUIRE_INIT();
  BK_ARG(dev_buf && max_launches > 0, "bkTraceEnable: bad arguments");
  g_ctx.trace = bk_ptr<unsigned long long>(dev_buf);
  g_ctx.trace_cap = max_launches;
  g_ctx.trace_seq = 0;
  return BK_OK;
}

int32_t bkTraceCtas(uint64_t dev_buf, int32_t gemv_launch_index) {
  BK_REQUIRE_INIT();
  g_ctx.cta_trace = bk_ptr<unsigned long long>(dev_buf);
  g_ctx.cta_trace_launch = gemv_launch_index;
  g_ctx.cta_trace_seen = 0;
  return BK_OK;
}

int32_t bkStepTraceEnable(uint64_t dev_buf, int32_t max_phases) {
  BK_REQUIRE_INIT();
  BK_ARG(dev_buf && max_phases > 0, "bkStepTraceEnable: bad arguments");
  g_ctx.step_trace = bk_ptr<unsigned long long>(dev_buf);
  g_ctx.step_trace_phases = max_phases;
  return BK_OK;
}

int32_t bkSetSpinLimit(int32_t polls) {
  BK_REQUIRE_INIT();
  BK_ARG(polls >= 0, "bkSetSpinLimit: polls=%d", polls);
  g_ctx.spin_limit = polls;
  return BK_OK;
}

int32_t bkStepBarrierMode(int32_t mode) {
  BK_REQUIRE_INIT();
  BK_ARG(mode == 0 || mode == 1, "bkStepBarrierMode: mode %d", mode);
  g_ctx.step_barrier_mode = mode;
  return BK_OK;
}

int32_t bkTraceDisable(void) {
  BK_REQUIRE_INIT();
  g_ctx.step_trace = nullptr;
  g_ctx.step_trace_phases = 0;
  g_ctx.trace = nullptr;
  g_ctx.trace_cap = 0;
  g_ctx.cta_trace = nullptr;
  return BK_OK;
}

int32_t bkLaunchCount(uint64_t* out_count) {
  BK_REQUIRE_INIT();
  BK_ARG(out_count != nullptr, "bkLaunchCount: out_count is null");
  *out_count = g_ctx.launches;
  return BK_OK;
}

}  // extern "C"
