// `CudaBackend`: the reference's `Backend` interface (src/backend.ts:158-211) over libjaxcuda.so.
//
// Drop this file in src/backend/cuda.ts of jax-js, add "cuda" to the `Device` union and the
// `devices` list (src/backend.ts:18-19) and an arm to `createBackend` (src/backend.ts:72-142):
//
//     } else if (device === "cuda") {
//       const { CudaBackend } = await import("./backend/cuda");
//       return CudaBackend.create();
//     }
//
// The native calls go through a Node-API addon (addon.cc beside this file) that forwards each
// function of include/jaxcuda.h unchanged.  Lowering stays in TypeScript: `tuneNullopt`
// (src/tuner.ts:219-240) binds gidx/ridx, rewrites GlobalView to guarded GlobalIndex loads and
// simplifies; this file only serialises the lowered DAG into the wire image of
// include/jaxcuda_ir.h.  Skeleton choice and tiling happen in the library, so `tuneWebgpu` is
// not used for this device.
//
// This file is not compiled in this repository (no Node toolchain in the build image); the Python
// class jax_js_b200/backend.py drives the same C ABI in the tests.

import { AluExp, AluOp, DType, Kernel } from "../alu";
import { Backend, Device, Executable, Slot, SlotError, UnsupportedOpError, UnsupportedRoutineError } from "../backend";
import { Routine } from "../routine";
import { emitTrace, isTracing, onFlushTrace, traceSourceInfo, type TraceInfo } from "../tracing";
import { tuneNullopt } from "../tuner";
import { FpHash } from "../utils";

interface Native {
  create(device: number): bigint;                      // jaxcuda_create -> ctx handle
  destroy(ctx: bigint): void;
  lastError(ctx: bigint): string;
  malloc(ctx: bigint, bytes: number, init?: Uint8Array): number;
  incref(ctx: bigint, slot: number): number;           // returns jaxcuda_status
  decref(ctx: bigint, slot: number): number;
  read(ctx: bigint, slot: number, start: number, count: number): Uint8Array<ArrayBuffer>;
  readAsync(ctx: bigint, slot: number, start: number, count: number): Promise<Uint8Array<ArrayBuffer>>;
  prepareKernel(ctx: bigint, image: Uint8Array, hash: bigint): bigint;
  prepareRoutine(ctx: bigint, name: string, type: unknown, params: string): bigint;
  dispatch(ctx: bigint, exe: bigint, inputs: Uint32Array, outputs: Uint32Array): number;
  captureBegin(ctx: bigint): void;
  captureEnd(ctx: bigint): bigint;
  graphLaunch(ctx: bigint, graph: bigint): void;
  graphDestroy(ctx: bigint, graph: bigint): void;
  graphCost(graph: bigint): { launches: number; bytes: number; fusedRuns: number };
  traceStart(ctx: bigint): void;                       // jaxcuda_trace_start
  traceStop(ctx: bigint): { startMs: number; durationMs: number }[];   // jaxcuda_trace_stop + jaxcuda_trace_record
}

// Codes of include/jaxcuda_ir.h, in the declaration order of AluOp (src/alu.ts:1365-1407).
const OP_CODE: Record<string, number> = Object.fromEntries(
  ["Add", "Sub", "Mul", "Idiv", "Mod", "Min", "Max", "Sin", "Cos", "Asin", "Atan", "Exp", "Log", "Erf", "Erfc",
   "Sqrt", "Floor", "Ceil", "Reciprocal", "Cast", "Bitcast", "BitCombine", "BitInvert", "BitShift", "Cmplt",
   "Cmpne", "Where", "Threefry2x32", "Const", "Special", "Variable", "GlobalIndex"].map((n, i) => [n, i]));
const DTYPE_CODE: Record<string, number> = { float32: 0, int32: 1, uint32: 2, bool: 3, float16: 4, float64: 5 };
const NODE_WORDS = 10, HEADER_WORDS = 10, MAGIC = 0x314b584a;

function isFloat(d: DType) { return d === DType.Float32 || d === DType.Float16 || d === DType.Float64; }

/** Topologically ordered node list of one expression DAG, shared nodes emitted once. */
function encodeDag(root: AluExp, words: number[]): number {
  const index = new Map<AluExp, number>();
  const order: AluExp[] = [];
  const visit = (e: AluExp) => {
    if (index.has(e)) return;
    for (const s of e.src) visit(s);
    index.set(e, order.length);
    order.push(e);
  };
  visit(root);
  const f64 = new Float64Array(1), u32 = new Uint32Array(f64.buffer);
  for (const e of order) {
    let lo = 0, hi = 0, arg1 = 0;
    switch (e.op) {
      case AluOp.Const:
        if (isFloat(e.dtype)) { f64[0] = e.arg; lo = u32[0]; hi = u32[1]; }
        else { lo = e.arg >>> 0; hi = e.arg < 0 ? 0xffffffff : 0; }
        break;
      case AluOp.Special: lo = e.arg[0] === "gidx" ? 0 : 1; arg1 = e.arg[1]; break;
      case AluOp.Variable: if (e.arg !== "acc") throw new Error(`unbound variable ${e.arg}`); break;
      case AluOp.GlobalIndex: lo = e.arg[0]; arg1 = e.arg[1]; break;
      case AluOp.BitCombine: lo = { and: 0, or: 1, xor: 2 }[e.arg as string]!; break;
      case AluOp.BitShift: lo = e.arg === "shl" ? 0 : 1; break;
      case AluOp.Threefry2x32: lo = e.arg === "xor" ? 0 : e.arg === 0 ? 1 : 2; break;
      case AluOp.GlobalView: throw new Error("GlobalView must be lowered before serialisation");
    }
    const src = e.src.map((s) => index.get(s)!);
    while (src.length < 4) src.push(0);
    words.push(OP_CODE[e.op], DTYPE_CODE[e.dtype], e.src.length, ...src, lo, hi, arg1 >>> 0);
  }
  return order.length;
}

/** Wire image of a Kernel (layout: include/jaxcuda_ir.h). */
export function serializeKernel(kernel: Kernel): Uint8Array {
  const tune = tuneNullopt(kernel);
  const r = kernel.reduction;
  const body: number[] = [];
  const nExp = encodeDag(tune.exp, body);
  const nEpi = tune.epilogue ? encodeDag(tune.epilogue, body) : 0;
  const head = [MAGIC, kernel.nargs, kernel.size >>> 0, Math.floor(kernel.size / 2 ** 32), r ? 1 : 0,
                r ? DTYPE_CODE[r.dtype] : 0, r ? OP_CODE[r.op] : 0, r ? r.size : 0, nExp, nEpi];
  if (head.length !== HEADER_WORDS || body.length !== (nExp + nEpi) * NODE_WORDS) throw new Error("bad image");
  return new Uint8Array(new Uint32Array([...head, ...body]).buffer);
}

const STATUS = { OK: 0, ESLOT: 1, EUNSUPPORTED: 2, EINVAL: 3, ECOMPILE: 4, ECUDA: 5, ENOMEM: 6 };

export class CudaBackend implements Backend {
  readonly type = "cuda" as Device;
  readonly maxArgs = 64;                     // jaxcuda_max_args(); the Wasm backend's value (src/backend/wasm.ts:38)
  #exes = new Map<bigint, Executable<bigint>>();

  private constructor(private native: Native, private ctx: bigint) {}

  static async create(device = Number(process.env.JAXCUDA_DEVICE ?? 0)): Promise<CudaBackend | null> {
    let native: Native;
    try {
      native = (await import("node:module")).createRequire(import.meta.url)("./jaxcuda_addon.node");
    } catch {
      return null;                           // addon not built: the device is simply unavailable (init() skips it)
    }
    return new CudaBackend(native, native.create(device));
  }

  #check(status: number, slot?: Slot): void {
    if (status === STATUS.OK) return;
    const msg = this.native.lastError(this.ctx);
    if (status === STATUS.ESLOT) throw new SlotError(slot ?? -1);
    throw new Error(msg);
  }

  malloc(size: number, initialData?: Uint8Array): Slot {
    if (initialData && initialData.byteLength !== size) throw new Error("initialData size does not match buffer size");
    return this.native.malloc(this.ctx, size, initialData);
  }
  incRef(slot: Slot): void { this.#check(this.native.incref(this.ctx, slot), slot); }
  decRef(slot: Slot): void { this.#check(this.native.decref(this.ctx, slot), slot); }

  // The copy starts at once on the library's download stream; the Promise resolves on a worker thread,
  // so the event loop keeps dispatching (and uploading) the next step meanwhile.
  read(slot: Slot, start = 0, count = -1): Promise<Uint8Array<ArrayBuffer>> {
    return this.native.readAsync(this.ctx, slot, start, count);
  }
  readSync(slot: Slot, start = 0, count = -1): Uint8Array<ArrayBuffer> {
    return this.native.read(this.ctx, slot, start, count);   // count -1: to the end; 0: barrier only
  }

  async prepareKernel(kernel: Kernel) { return this.prepareKernelSync(kernel); }
  prepareKernelSync(kernel: Kernel): Executable<bigint> {
    const hash = FpHash.hash(kernel);                         // the cache key the other backends use
    const hit = this.#exes.get(hash);
    if (hit) return hit;
    let handle: bigint;
    try {
      handle = this.native.prepareKernel(this.ctx, serializeKernel(kernel), hash);
    } catch (e) {
      const msg = this.native.lastError(this.ctx);
      const m = /^(\w*)<(\w+)> not supported in cuda backend/.exec(msg);
      if (m) throw new UnsupportedOpError((m[1] || null) as AluOp | null, m[2] as DType, this.type);
      throw new Error(msg);                                   // NVRTC log plus generated source
    }
    const exe = new Executable(kernel, handle);
    this.#exes.set(hash, exe);
    return exe;
  }

  async prepareRoutine(routine: Routine) { return this.prepareRoutineSync(routine); }
  prepareRoutineSync(routine: Routine): Executable<bigint> {
    try {
      return new Executable(routine, this.native.prepareRoutine(this.ctx, routine.name, routine.type,
                                                                JSON.stringify(routine.params ?? {})));
    } catch {
      // an unknown routine name (src/backend.ts:236-240); anything else is a shape or dtype the
      // reference's own routine rejects, with its message (src/routine.ts:305-313, :341-346)
      const msg = this.native.lastError(this.ctx);
      if (/^routine '.*' is not supported in cuda backend/.test(msg)) throw new UnsupportedRoutineError(routine.name, this.type);
      throw new Error(msg);
    }
  }

  // Tracing (src/tracing.ts:15-33): the library times every dispatch with a pair of CUDA events while
  // a trace is on; the records are turned into `performance.measure` entries when the profiler
  // flushes (the webgpu backend resolves its timestamp queries at the same point,
  // src/backend/webgpu/tracing.ts:61-70), placed on the host clock from the moment the trace began.
  #traceInfos: TraceInfo[] | null = null;
  #traceAnchor = 0;
  #recording = false;
  #flushRegistered = false;

  #flushTrace(): void {
    const infos = this.#traceInfos;
    if (!infos) return;
    this.#traceInfos = null;
    const records = this.native.traceStop(this.ctx);
    for (let i = 0; i < records.length && i < infos.length; i++) {
      const start = this.#traceAnchor + records[i].startMs;
      emitTrace("cuda", infos[i], start, start + records[i].durationMs);
    }
  }

  dispatch(exe: Executable<bigint>, inputs: Slot[], outputs: Slot[]): void {
    // dispatches inside a recording are fused and replayed as one graph: the library leaves no record of them
    const traced = isTracing() && !this.#recording;
    if (traced && !this.#traceInfos) {
      this.native.traceStart(this.ctx);
      this.#traceAnchor = performance.now();
      this.#traceInfos = [];
      if (!this.#flushRegistered) onFlushTrace(() => this.#flushTrace());   // stopTrace runs every callback ever registered
      this.#flushRegistered = true;
    } else if (!isTracing() && this.#traceInfos) {
      this.#flushTrace();
    }
    this.#check(this.native.dispatch(this.ctx, exe.data, Uint32Array.from(inputs), Uint32Array.from(outputs)));
    if (traced) this.#traceInfos!.push(traceSourceInfo(exe.source));   // a dispatch that failed left no record either
  }

  /**
   * Beyond `Backend`: records `steps` (the malloc / dispatch / decRef calls of one
   * `JitProgram.execute`, src/frontend/jit.ts:111-162) as a CUDA graph and returns a function that
   * replays it.  Slots alive when `steps` returns keep their addresses and are rewritten by every
   * replay.  Inside the recording the backend fuses what the list allows (rows of softmax-like
   * chains, producers into their only consumer, runs of small kernels).
   */
  record(steps: () => void): { replay: () => void; destroy: () => void; cost: { launches: number; bytes: number; fusedRuns: number } } {
    this.native.captureBegin(this.ctx);
    this.#recording = true;
    let graph: bigint;
    try {
      steps();
    } finally {
      this.#recording = false;
      graph = this.native.captureEnd(this.ctx);
    }
    return {
      replay: () => this.native.graphLaunch(this.ctx, graph),
      destroy: () => this.native.graphDestroy(this.ctx, graph),
      cost: this.native.graphCost(graph),
    };
  }
}
