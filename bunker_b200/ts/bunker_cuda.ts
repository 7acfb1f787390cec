// bunker_cuda.ts -- the TypeScript side of the drop-in: libbunker_cuda.so bound through bun:ffi behind the names of
// bunker's runtime (src/ttir.ts:223-417): cu / cuAlloc / cuHtoD / cuDtoH / cuFree / cuSync / cuHtoDAsync / cuDtoHAsync /
// cuCopySync / cuLaunch / LoadedKernel / profGpuReset / profGpuReport, with `compileAndLoad(ttir, ...)` replaced by
// `loadOp(name)` (the kernels are in the library, nothing is compiled at run time), plus the whole-step calls that
// keep the CUDA graph inside the library (one FFI call per token; replaying a graph through bun:ffi crashed bunker,
// LOG.md:710-738).
//
// Binding rules taken from bunker's own experience with bun:ffi (LOG.md:605-607, 725-733): device pointers, events and
// handles travel as u64 (a "ptr" argument below 2^32 is rejected), argument structs are packed into a Buffer that the
// callee copies before it returns, nothing depends on process.env, host buffers only need to live for the call.
//
// Usage in bunker:   import { cuAlloc, cuHtoD, cuDtoH, cuSync, cuLaunch, loadOp } from "./bunker_cuda";
// in place of the same names from "./ttir" in src/runner.ts:18, prototypes/decode_graph.ts:15 and prototypes/decode.ts:5.
import { dlopen, ptr as ffiPtr, CString } from "bun:ffi";

export const BK_OK = 0, BK_ERR_ARG = 10001, BK_ERR_STATE = 10002, BK_ERR_TIMEOUT = 10003, BK_ERR_UNSUPPORTED = 10004, BK_ERR_COMM = 10005;
export const BK_PRO_Q8 = 0, BK_PRO_BF16 = 1, BK_PRO_RMSNORM = 2, BK_PRO_STAGED = 3;
export const BK_EPI_F32 = 0, BK_EPI_BF16 = 1, BK_EPI_ADD_BF16 = 2, BK_EPI_SWIGLU = 3;
export const BK_Q8_BLOCKS = 0, BK_Q8_STAGED = 1, BK_DTYPE_F32 = 0, BK_DTYPE_BF16 = 1, BK_GEMV_ORDER_AUTO = 0, BK_GEMV_ORDER_LANES = 1, BK_GEMV_ORDER_TILE = 2;
export const OPS: Record<string, number> = {
  embed: 1, rmsnorm: 2, gemm: 3, swiglu: 4, conv1d_decode: 5, argmax: 6, quant_q8_1: 7, headnorm_rope: 8,
  gdn_delta_rule: 9, fa2_attn: 10, quant_q8_1_bf16: 11,
};

const SYMBOLS = {
  bkInit: { args: ["i32"], returns: "i32" },
  bkShutdown: { args: [], returns: "i32" },
  bkLastError: { args: [], returns: "cstring" },
  bkDeviceInfo: { args: ["ptr", "ptr", "ptr", "ptr"], returns: "i32" },
  bkAlloc: { args: ["u64", "ptr"], returns: "i32" },
  bkFree: { args: ["u64"], returns: "i32" },
  bkHtoD: { args: ["u64", "ptr", "u64"], returns: "i32" },
  bkDtoH: { args: ["ptr", "u64", "u64"], returns: "i32" },
  bkHtoDAsync: { args: ["u64", "ptr", "u64"], returns: "i32" },
  bkDtoHAsync: { args: ["ptr", "u64", "u64"], returns: "i32" },
  bkDtoD: { args: ["u64", "u64", "u64"], returns: "i32" },
  bkMemset: { args: ["u64", "i32", "u64"], returns: "i32" },
  bkHostAlloc: { args: ["u64", "ptr"], returns: "i32" },
  bkHostFree: { args: ["ptr"], returns: "i32" },
  bkSync: { args: [], returns: "i32" },
  bkEventCreate: { args: ["ptr"], returns: "i32" },
  bkEventRecord: { args: ["u64"], returns: "i32" },
  bkEventSync: { args: ["u64"], returns: "i32" },
  bkEventElapsedMs: { args: ["u64", "u64", "ptr"], returns: "i32" },
  bkEventDestroy: { args: ["u64"], returns: "i32" },
  bkLaunchCount: { args: ["ptr"], returns: "i32" },
  bkStagedBytes: { args: ["i32", "i32"], returns: "u64" },
  bkGemvQ4K: { args: ["ptr"], returns: "i32" },
  bkGemvQ4KSimple: { args: ["u64", "i32", "i32", "u64", "i32", "u64"], returns: "i32" },
  bkDequantQ4K: { args: ["u64", "i32", "i32", "u64"], returns: "i32" },
  bkBlockDotsQ4K: { args: ["u64", "i32", "i32", "u64", "u64", "u64"], returns: "i32" },
  bkQuantizeQ4K: { args: ["u64", "i32", "i64", "i32", "u64"], returns: "i32" },
  bkQuantQ8_1: { args: ["u64", "i32", "i32", "u64"], returns: "i32" },
  bkQuantQ8_1Bf16: { args: ["u64", "i32", "i32", "u64"], returns: "i32" },
  bkEmbedQ4K: { args: ["u64", "i32", "u64", "i32", "u64"], returns: "i32" },
  bkRmsNorm: { args: ["u64", "u64", "i32", "i32", "f32", "u64"], returns: "i32" },
  bkRmsNormQuantQ8_1: { args: ["u64", "u64", "i32", "i32", "f32", "u64", "i32"], returns: "i32" },
  bkReduceRmsNormQuantQ8_1: { args: ["u64", "i32", "u64", "u64", "u32", "u64", "u64", "u64", "i32", "i32", "f32", "u64", "i32"], returns: "i32" },
  bkSwiglu: { args: ["u64", "u64", "i32", "u64"], returns: "i32" },
  bkConv1dStep: { args: ["u64", "u64", "u64", "i32", "i32", "u64", "u64"], returns: "i32" },
  bkGdnStep: { args: ["ptr"], returns: "i32" },
  bkRopeTables: { args: ["i32", "i32", "f64", "ptr", "ptr"], returns: "i32" },
  bkHeadNormRope: { args: ["u64", "i32", "u64", "u64", "u64", "i32", "u64", "i32", "i32", "i32", "u64"], returns: "i32" },
  bkAttnDecode: { args: ["ptr"], returns: "i32" },
  bkAttnPlan: { args: ["i32", "i32", "i32", "ptr", "ptr"], returns: "i32" },
  bkAttnScratchBytes: { args: ["i32", "i32", "i32", "i32", "i32"], returns: "u64" },
  bkArgmax: { args: ["u64", "i32", "i32", "u64", "u64", "u64"], returns: "i32" },
  bkArgmaxScratchBytes: { args: ["i32"], returns: "u64" },
  bkArgmaxStatic: { args: ["u64", "i32", "i32", "u64", "u64"], returns: "i32" },
  bkSample: { args: ["u64", "i32", "i32", "f32", "i32", "f32", "u64", "u64", "u32", "u64", "u64"], returns: "i32" },
  bkModelCreate: { args: ["ptr", "ptr"], returns: "i32" },
  bkModelSetTensor: { args: ["u64", "ptr", "u64", "u64"], returns: "i32" },
  bkModelSetComm: { args: ["u64", "u64"], returns: "i32" },
  bkModelSetStepMode: { args: ["u64", "i32"], returns: "i32" },
  bkModelFinalize: { args: ["u64"], returns: "i32" },
  bkModelReset: { args: ["u64"], returns: "i32" },
  bkDecodeStep: { args: ["u64", "ptr", "ptr", "ptr"], returns: "i32" },
  bkModelPrefill: { args: ["u64", "ptr", "i32", "ptr", "ptr"], returns: "i32" },
  bkDecodeRun: { args: ["u64", "i32"], returns: "i32" },
  bkDecodeStepProfiled: { args: ["u64", "ptr", "ptr", "i32"], returns: "i32" },
  bkModelTokens: { args: ["u64", "i32", "i32", "ptr"], returns: "i32" },
  bkModelInfo: { args: ["u64", "ptr", "ptr", "ptr", "ptr"], returns: "i32" },
  bkModelBuffer: { args: ["u64", "ptr", "ptr"], returns: "i32" },
  bkModelDestroy: { args: ["u64"], returns: "i32" },
  bkCommCreate: { args: ["i32", "i32", "u64", "ptr"], returns: "i32" },
  bkCommExportHandle: { args: ["u64", "ptr"], returns: "i32" },
  bkCommImportPeers: { args: ["u64", "ptr"], returns: "i32" },
  bkCommDestroy: { args: ["u64"], returns: "i32" },
  bkCommAllReduceResidual: { args: ["u64", "i32", "u64", "i32", "u64", "u64"], returns: "i32" },
  bkLaunch: { args: ["i32", "ptr", "i32"], returns: "i32" },
  bkTraceEnable: { args: ["u64", "i32"], returns: "i32" },
  bkTraceCtas: { args: ["u64", "i32"], returns: "i32" },
  bkTraceDisable: { args: [], returns: "i32" },
  bkTuneGemvRing: { args: ["i32", "i32", "i32"], returns: "i32" },
  bkTuneTileMinRows: { args: ["i32"], returns: "i32" },
  bkStepTraceEnable: { args: ["u64", "i32"], returns: "i32" },
  bkSetSpinLimit: { args: ["i32"], returns: "i32" },
  bkStepBarrierMode: { args: ["i32"], returns: "i32" },
  bkDecodeStepEager: { args: ["u64"], returns: "i32" },
} as const;

let _lib: any = null;
let _device = 0;
/** Open the library and create the context on `device` (src/ttir.ts:223-261 `cu()`).  There is no CPU fallback. */
export function cu(libPath = "./bunker_b200/libbunker_cuda.so", device = 0) {
  if (!_lib) {
    _lib = dlopen(libPath, SYMBOLS).symbols;
    const rc = _lib.bkInit(device);
    if (rc !== 0) throw new Error(`bkInit failed (rc=${rc}): ${lastError()}`);
    _device = device;
  }
  return _lib;
}
export function lastError(): string { const s = _lib?.bkLastError(); return s ? s.toString() : ""; }
function check(rc: number, what: string): void { if (rc !== 0) throw new Error(`${what} failed (rc=${rc}): ${lastError()}`); }
const hostBuf = (h: Buffer | ArrayBuffer): Buffer => (h instanceof ArrayBuffer ? Buffer.from(h) : h);

/** Allocate a device buffer; returns the device pointer as a BigInt (src/ttir.ts:266). */
export function cuAlloc(bytes: number | bigint): bigint {
  const b = Buffer.alloc(8);
  if (cu().bkAlloc(BigInt(bytes), b) !== 0) throw new Error(`cuMemAlloc failed (${bytes} bytes)`);
  return b.readBigUInt64LE(0);
}
export function cuHtoD(devPtr: bigint, host: Buffer | ArrayBuffer, bytes?: number | bigint): void {
  const buf = hostBuf(host);
  if (cu().bkHtoD(devPtr, buf, BigInt(bytes ?? buf.byteLength)) !== 0) throw new Error("cuMemcpyHtoD failed");
}
/** Synchronous: doubles as the per-token barrier of the decode loop (prototypes/decode.ts:1042-1049). */
export function cuDtoH(host: Buffer | ArrayBuffer, devPtr: bigint, bytes?: number | bigint): void {
  const buf = hostBuf(host);
  if (cu().bkDtoH(buf, devPtr, BigInt(bytes ?? buf.byteLength)) !== 0) throw new Error("cuMemcpyDtoH failed");
}
export function cuFree(devPtr: bigint): void { cu().bkFree(devPtr); }
/** Returns the rc instead of throwing, like the reference (src/ttir.ts:285).  BK_ERR_TIMEOUT = a bounded device wait gave up. */
export function cuSync(): number { return cu().bkSync(); }
/** Async copies (src/ttir.ts:305-317); the host buffer must be pinned (bkHostAlloc) and stay alive until cuCopySync. */
export function cuHtoDAsync(devPtr: bigint, host: Buffer | ArrayBuffer, bytes?: number | bigint): void {
  const buf = hostBuf(host);
  const rc = cu().bkHtoDAsync(devPtr, buf, BigInt(bytes ?? buf.byteLength));
  if (rc !== 0) throw new Error(`cuMemcpyHtoDAsync failed (rc=${rc})`);
}
export function cuDtoHAsync(host: Buffer | ArrayBuffer, devPtr: bigint, bytes?: number | bigint): void {
  const buf = hostBuf(host);
  const rc = cu().bkDtoHAsync(buf, devPtr, BigInt(bytes ?? buf.byteLength));
  if (rc !== 0) throw new Error(`cuMemcpyDtoHAsync failed (rc=${rc})`);
}
export function cuCopySync(): number { return cu().bkSync(); }

/** src/ttir.ts:350.  `fn` is the library's op id; module and shmem exist for shape parity only. */
export interface LoadedKernel { module: number; fn: number; shmem: number; }
/** Stands where compileAndLoad(ttir, func, numWarps) stood (src/ttir.ts:488): the op's kernel is already in the library. */
export function loadOp(name: string): LoadedKernel {
  const fn = OPS[name];
  if (fn === undefined) throw new Error(`loadOp: the library has no op '${name}'`);
  return { module: 0, fn, shmem: 0 };
}

// ── per-op timing, the BUNKER_GPU_PROF=1 profiler of src/ttir.ts:352-417 on the library's events ──
let GPU_PROF = false;
export function profGpuEnable(on: boolean): void { GPU_PROF = on; }   // process.env never reaches the library
const _profTotal = new Map<string, { ms: number; count: number }>();
let _pending: { start: bigint; end: bigint; key: string }[] = [];
const newEvent = (): bigint => { const b = Buffer.alloc(8); check(cu().bkEventCreate(b), "bkEventCreate"); return b.readBigUInt64LE(0); };
export function profGpuReset(): void { _pending = []; _profTotal.clear(); }
export function profGpuReport(): void {
  if (!GPU_PROF) return;
  const L = cu();
  L.bkSync();
  const ms = new Float32Array(1);
  for (const pe of _pending) {
    if (L.bkEventElapsedMs(pe.start, pe.end, ms) === 0) {
      const cur = _profTotal.get(pe.key) ?? { ms: 0, count: 0 };
      cur.ms += ms[0]; cur.count += 1; _profTotal.set(pe.key, cur);
    }
    L.bkEventDestroy(pe.start); L.bkEventDestroy(pe.end);
  }
  _pending = [];
  const rows = [..._profTotal.entries()].sort((a, b) => b[1].ms - a[1].ms);
  const total = rows.reduce((a, r) => a + r[1].ms, 0);
  console.log("\n── BUNKER_GPU_PROF (kernel elapsed, library stream) ──");
  for (const [key, v] of rows)
    console.log(`  ${v.ms.toFixed(2).padStart(8)}ms  ${(total ? v.ms / total * 100 : 0).toFixed(1).padStart(5)}%  x${String(v.count).padStart(4)}  avg ${(v.ms / v.count * 1e3).toFixed(1).padStart(6)}us  ${key}`);
  console.log(`  ${total.toFixed(2)}ms total GPU (${rows.length} distinct ops)\n`);
}

/** Launch an op: every argument in one 8-byte slot, BigInt = device pointer, number = integer; floats as their f32 bits
 *  (f32Slot).  grid and block are accepted for signature parity and ignored.  Returns the rc, does not throw
 *  (src/ttir.ts:321-348). */
export function cuLaunch(k: LoadedKernel, _grid: [number, number, number], _block: [number, number, number], args: (bigint | number)[]): number {
  const L = cu();
  const slot = Buffer.alloc(Math.max(args.length, 1) * 8);
  for (let i = 0; i < args.length; i++) {
    const a = args[i];
    if (typeof a === "bigint") slot.writeBigUInt64LE(a, i * 8); else slot.writeBigInt64LE(BigInt(a), i * 8);
  }
  let pe: { start: bigint; end: bigint } | null = null;
  if (GPU_PROF) { pe = { start: newEvent(), end: newEvent() }; L.bkEventRecord(pe.start); }
  const rc = L.bkLaunch(k.fn, slot, args.length);
  if (pe) { L.bkEventRecord(pe.end); _pending.push({ ...pe, key: Object.keys(OPS).find(n => OPS[n] === k.fn) ?? `op${k.fn}` }); }
  return rc;
}
/** A float argument of cuLaunch: its f32 bit pattern as an integer slot. */
export function f32Slot(x: number): number { const b = Buffer.alloc(4); b.writeFloatLE(x, 0); return b.readUInt32LE(0); }

// ── argument structs (layouts of include/bunker_cuda.h; the library copies them before returning) ──
export interface GemvSeg { W: bigint; W2?: bigint; out: bigint; residual?: bigint; nRows: number; epilogue: number; ldOut?: number; colOff?: number; }
export function packGemvArgs(K: number, B: number, prologue: number, x: bigint, segs: GemvSeg[], normW = 0n, eps = 1e-6, order = 0): Buffer {
  const b = Buffer.alloc(40 + 4 * 48);
  b.writeInt32LE(K, 0); b.writeInt32LE(B, 4); b.writeInt32LE(segs.length, 8); b.writeInt32LE(prologue, 12);
  b.writeBigUInt64LE(x, 16); b.writeBigUInt64LE(normW, 24); b.writeFloatLE(eps, 32); b.writeInt32LE(order, 36);
  segs.forEach((s, i) => {
    const o = 40 + i * 48, col = s.colOff ?? 0;
    b.writeBigUInt64LE(s.W, o); b.writeBigUInt64LE(s.W2 ?? 0n, o + 8); b.writeBigUInt64LE(s.out, o + 16); b.writeBigUInt64LE(s.residual ?? 0n, o + 24);
    b.writeInt32LE(s.nRows, o + 32); b.writeInt32LE(s.epilogue, o + 36); b.writeInt32LE(s.ldOut ?? s.nRows + col, o + 40); b.writeInt32LE(col, o + 44);
  });
  return b;
}
export function gemvQ4K(args: Buffer): void { check(cu().bkGemvQ4K(args), "bkGemvQ4K"); }

export interface ModelDims {
  hidden: number; nLayers: number; fullAttnInterval: number; vocab: number; gdnKHeads: number; gdnVHeads: number;
  attnQHeads: number; attnKvHeads: number; headDim: number; rotDim: number; intermediate: number; maxLen: number;
  batch: number; tpRank?: number; tpSize?: number; eps?: number; ropeTheta?: number;
}
/** bkModelConfig: 15 int32, float eps, double rope_theta (72 bytes). */
export function packModelConfig(d: ModelDims): Buffer {
  const b = Buffer.alloc(72);
  [d.hidden, d.nLayers, d.fullAttnInterval, d.vocab, d.gdnKHeads, d.gdnVHeads, d.attnQHeads, d.attnKvHeads, d.headDim, d.rotDim,
   d.intermediate, d.maxLen, d.batch, d.tpRank ?? 0, d.tpSize ?? 1].forEach((v, i) => b.writeInt32LE(v, 4 * i));
  b.writeFloatLE(d.eps ?? 1e-6, 60); b.writeDoubleLE(d.ropeTheta ?? 1e7, 64);
  return b;
}

/** The whole decode step behind one call per token: stands where buildModelGraph + compileStep + runGraphDecode stand
 *  (src/model.ts:46-204, src/runner.ts:94-162).  Weights are registered under the graph's tensor names. */
export class BunkerModel {
  handle: bigint;
  private ids: Int32Array; private out: Int32Array; private val: Float32Array;
  constructor(public dims: ModelDims) {
    const h = Buffer.alloc(8);
    check(cu().bkModelCreate(packModelConfig(dims), h), "bkModelCreate");
    this.handle = h.readBigUInt64LE(0);
    this.ids = new Int32Array(dims.batch); this.out = new Int32Array(dims.batch); this.val = new Float32Array(dims.batch);
  }
  /** name as in src/model.ts:72-196 ("embed.weight", "model.layers.3.self_attn.q_proj.weight", ...); linear weights are Q4_K rows. */
  setTensor(name: string, devPtr: bigint, bytes: number | bigint): void {
    check(cu().bkModelSetTensor(this.handle, Buffer.from(name + "\0"), devPtr, BigInt(bytes)), `bkModelSetTensor(${name})`);
  }
  setStepMode(mode: 0 | 1 | 2): void { check(cu().bkModelSetStepMode(this.handle, mode), "bkModelSetStepMode"); }
  finalize(): void { check(cu().bkModelFinalize(this.handle), "bkModelFinalize"); }
  reset(): void { check(cu().bkModelReset(this.handle), "bkModelReset"); }
  /** One token per sequence in, (argmax id, its logit) per sequence out: runGraphDecode's loop body (src/runner.ts:133-160). */
  step(tokens: ArrayLike<number> | null): { ids: Int32Array; vals: Float32Array } {
    if (tokens) for (let i = 0; i < this.ids.length; i++) this.ids[i] = tokens[i];
    check(cu().bkDecodeStep(this.handle, tokens ? this.ids : null, this.out, this.val), "bkDecodeStep");
    return { ids: this.out, vals: this.val };
  }
  /** n greedy steps with the token fed back on the device, no host traffic. */
  run(n: number): void { check(cu().bkDecodeRun(this.handle, n), "bkDecodeRun"); }
  /** T prompt tokens of every sequence in one call (tokens laid out [T][batch], T*batch <= 64). */
  prefill(tokens: Int32Array, T: number): { ids: Int32Array; vals: Float32Array } {
    check(cu().bkModelPrefill(this.handle, tokens, T, this.out, this.val), "bkModelPrefill");
    return { ids: this.out, vals: this.val };
  }
  tokens(firstStep: number, nSteps: number): Int32Array {
    const o = new Int32Array(nSteps * this.dims.batch);
    check(cu().bkModelTokens(this.handle, firstStep, nSteps, o), "bkModelTokens");
    return o;
  }
  destroy(): void { cu().bkModelDestroy(this.handle); this.handle = 0n; }
}

/** src/runner.ts:116-162 on top of BunkerModel: prompt one token at a time, then genLen-1 greedy steps; onToken as in the reference. */
export function runGraphDecode(model: BunkerModel, prompt: number[], genLen: number, onToken?: (pos: number, id: number, val: number) => void): number[] {
  const out: number[] = [];
  let id = 0, pos = 0;
  for (const t of prompt) { const r = model.step([t]); id = r.ids[0]; onToken?.(pos++, id, r.vals[0]); }
  out.push(id);
  for (let g = 1; g < genLen; g++) { const r = model.step([id]); id = r.ids[0]; onToken?.(pos++, id, r.vals[0]); out.push(id); }
  return out;
}

/** Weight loader's quantiser: f32 / bf16 rows already on the device -> Q4_K rows (prototypes/decode.ts:64-76 uploads bf16). */
export function quantizeQ4K(x: bigint, dtype: number, nRows: number | bigint, K: number, outQ4K: bigint): void {
  check(cu().bkQuantizeQ4K(x, dtype, BigInt(nRows), K, outQ4K), "bkQuantizeQ4K");
}
