/*
 * bunker_cuda_diag.h -- diagnostic entry points of libbunker_cuda.so: device-side timelines and tuning overrides used
 * to analyse the kernels.  They are NOT part of the drop-in ABI (nothing in bunker binds them), they keep process-wide
 * state, and like the rest of the library they expect a single caller thread.
 */
#ifndef BUNKER_CUDA_DIAG_H
#define BUNKER_CUDA_DIAG_H

#include "bunker_cuda.h"

#ifdef __cplusplus
extern "C" {
#endif

/* Device-side timeline.  While enabled, every kernel launched (or captured into a graph) gets the next
 * 64-byte record of dev_buf and thread 0 of its CTA 0 stamps %globaltimer (ns) into slots:
 * 0 entry, 1 own weight copies issued, 2 dependency wait returned, 3 prologue done, 4 first weights landed, 5 exit.
 * A graph replays the records it was captured with.  Off by default. */
BK_API int32_t bkTraceEnable(uint64_t dev_buf, int32_t max_launches);
/* Per-CTA timeline of ONE GEMV launch: the gemv_launch_index-th bkGemvQ4K-class launch issued (or captured) after
 * this call records, for every CTA c, dev_buf[4c..4c+3] = {entry, dependency wait returned, first weights landed in
 * warp 0, latest warp exit} in %globaltimer ns.  dev_buf must hold 4 x 8 bytes per SM. */
BK_API int32_t bkTraceCtas(uint64_t dev_buf, int32_t gemv_launch_index);
BK_API int32_t bkTraceDisable(void);
/* Measurement aid, no counterpart in the reference: force the batch-1 kernel's weight ring (warps per CTA, rows per
 * warp group, maximum ring depth) for launches whose rows do not fit in shared memory at once; warps = 0 restores the
 * library's own choice. */
BK_API int32_t bkTuneGemvRing(int32_t warps, int32_t rows_per_group, int32_t max_depth);
/* Row count from which BK_GEMV_ORDER_AUTO takes the dense tile path (default 4096, or 1024 when K >= 2048; 0 restores both).  Lets a small test
 * model run every GEMV of its step on the tile kernel.  Captured graphs keep the choice they were captured with. */
BK_API int32_t bkTuneTileMinRows(int32_t rows);
/* Per-phase timeline of the persistent step kernel.  While enabled, every launch of that kernel stamps %globaltimer
 * (ns) into dev_buf[8*phase + k] for each phase it runs: 0 phase entered (CTA 0), 1 activation staged (CTA 0),
 * 2 CTA 0 finished its rows, 3 the latest CTA finished (atomic max; clear the buffer between steps), and for warp 0's
 * first row group of a GEMV phase 4 weights landed, 5 dot products done, 6 ring refilled, 7 epilogue stored.  Takes effect
 * for launches issued eagerly after the call (bkDecodeStepEager); captured graphs keep what they were captured with. */
BK_API int32_t bkStepTraceEnable(uint64_t dev_buf, int32_t max_phases);
/* Polls a bounded device-side wait may take before it gives up and sets the status word that bkSync reports as
 * BK_ERR_TIMEOUT (0 restores the built-in limits).  Applies to the tensor-parallel exchange consumer
 * (bkReduceRmsNormQuantQ8_1 and the model's reducing launches) and the persistent step kernel's grid barrier, for
 * launches issued after the call.  Lets a test make a wait run out in microseconds without hanging anything. */
BK_API int32_t bkSetSpinLimit(int32_t polls);
/* Grid barrier of the persistent step kernel, for models finalized after the call: 0 = one arrival word per CTA
 * , 1 = one atomic counter (the default: 1.8 us against 3-5 us per barrier on 148 CTAs). */
BK_API int32_t bkStepBarrierMode(int32_t mode);
/* One decode step enqueued without the CUDA graph (device-side token feedback), so that timelines enabled after
 * bkModelFinalize apply to it. */
BK_API int32_t bkDecodeStepEager(uint64_t model);

#ifdef __cplusplus
}
#endif
#endif /* BUNKER_CUDA_DIAG_H */
