/**
 * `BackendCuda`: the B200 kernel backend of tfjs-core, reference side.
 *
 * A `KernelBackend` subclass (tfjs-core/src/backends/backend.ts:91-649) whose methods are thin
 * marshalling over the N-API addon (js/binding.cc), which in turn is one function per entry
 * point of the C ABI (include/tfjs_cuda.h).  Tensor data lives in device memory owned by the
 * native library; it reaches the host only in readSync() / read().  Every kernel method only
 * enqueues work on the context's stream and returns.
 *
 * Methods outside the reference's surface are extensions (named as such below): a clip / relu6
 * activation for the fused ops, fusedDepthwiseConv2D, fusedSeparableConv2d, softmax, quantised
 * weight registration, asynchronous writes, CUDA-graph capture, per-kernel profiling.  Each has
 * an unfused equivalent through the plain methods, which is what unmodified tf.* code reaches.
 *
 * The Python class tfjs-core_b200/backend_cuda.py mirrors this file method for method; it is the
 * form the test-suite executes on machines without a JavaScript runtime.
 */
import {backend_util, DataType, ENV, engine, KernelBackend, Rank, ShapeMap, Tensor, Tensor3D, Tensor4D, util} from '@tensorflow/tfjs-core';
import {DataStorage} from '@tensorflow/tfjs-core/dist/backends/backend';

import * as binding from './binding';

type DataId = object;
type Conv2DInfo = backend_util.Conv2DInfo;
/** 'linear' | 'relu' | 'prelu' (ops/fused_util.ts:20) plus the extensions. */
export type CudaActivation = backend_util.Activation|'relu6'|['clip', number, number];

const EPSILON_FLOAT32 = 1e-7;   // backends/backend.ts:23
const EPSILON_FLOAT16 = 1e-4;   // backends/backend.ts:24

// enums of include/tfjs_cuda.h
const DTYPE: {[d: string]: number} = {float32: 0, int32: 1, bool: 2};
const STORAGE_F16 = 3;   // TFJS_F16: a float32 tensor stored as IEEE half
const ACT: {[a: string]: number} = {linear: 0, relu: 1, prelu: 2, clip: 3};
const MATH: {[m: string]: number} = {'3xtf32': 0, tf32: 1};
const BINARY = {add: 0, sub: 1, mul: 2, div: 3, prelu: 4, notEqual: 5};
const UNARY = {relu: 0, clip: 1, exp: 2, log: 3, int: 4, step: 5};
const REDUCE = {sum: 0, max: 1, argMax: 2};
const ERR_UNSUPPORTED = -5;

interface TensorRecord {
  id: number;             // tfjs_tensor_id
  dtype: DataType;        // dtype the storage was registered with
  half?: boolean;         // float32 values stored as IEEE half (16-bit activation storage)
  shape: number[];
  quantized?: boolean;    // uint8 bytes + scale/min (registerQuantized)
}

function typedArrayFor(dtype: DataType, size: number): Float32Array|Int32Array|Uint8Array {
  if (dtype === 'float32') return new Float32Array(size);
  if (dtype === 'int32') return new Int32Array(size);
  if (dtype === 'bool') return new Uint8Array(size);
  throw new Error(`cuda backend does not support dtype ${dtype}`);
}

export class BackendCuda extends KernelBackend {
  private ctx: binding.Handle;
  /** dataId -> device record.  A miss asks the engine to move the tensor here through host
   * memory (backends/backend.ts:47-70, engine.ts:361-363). */
  private data: DataStorage<TensorRecord>;
  mathMode: '3xtf32'|'tf32' = '3xtf32';
  activationStorage: 'float32'|'float16' = 'float32';
  private pendingStorage: 'float32'|'float16'|null = null;

  constructor(readonly device = 0, mathMode: '3xtf32'|'tf32' = '3xtf32') {
    super();
    const r = binding.ctxCreate(device);
    if (r.status !== 0) {
      // the factory throws, the engine warns and falls back by priority (engine.ts:302-306)
      throw new Error(`cuda backend initialisation failed (${r.status}): ${binding.lastError(null)}`);
    }
    this.ctx = r.out;
    this.data = new DataStorage(this, engine());
    this.setMathMode(mathMode);
  }

  // ---- helpers ---------------------------------------------------------------------------
  private check(rc: number): void {
    if (rc === 0) return;
    const msg = binding.lastError(this.ctx);
    if (rc === ERR_UNSUPPORTED) throw new Error(`Not yet implemented: ${msg}`);
    throw new Error(`cuda backend [${rc}]: ${msg}`);
  }

  private newId(shape: number[], dtype: DataType): number {
    if (!(dtype in DTYPE)) throw new Error(`cuda backend does not support dtype ${dtype}`);
    const r = binding.tensorRegister(this.ctx, shape.length, shape, DTYPE[dtype]);
    this.check(r.status);
    return r.out_id;
  }

  /** Device id of `t` read as `want`.  A cast-up alias shares its source's storage
   * (backend_util.ts:50-54), so the stored dtype can differ from the dtype the tensor claims;
   * then a converted temporary is returned as the second element and must be freed. */
  private id(t: Tensor, want: DataType = 'float32'): [number, number|null] {
    const rec = this.data.get(t.dataId);
    if (rec.dtype === want && !rec.half) return [rec.id, null];
    const tmp = this.newId(t.shape, want);
    this.check(binding.cast(this.ctx, rec.id, tmp));
    return [tmp, tmp];
  }

  /** Device id of an activation operand for the kernels that read float32 and half storage alike. */
  private activationId(t: Tensor): [number, number|null] {
    const rec = this.data.get(t.dataId);
    if (rec.half) return [rec.id, null];
    return this.id(t);
  }

  private freeTmp(...ids: Array<number|null>): void {
    for (const i of ids) {
      if (i != null) binding.tensorDispose(this.ctx, i);
    }
  }

  private makeOutput<T extends Tensor>(shape: number[], dtype: DataType = 'float32'): T {
    return Tensor.make(shape, {}, dtype, this) as T;   // re-enters register()
  }

  /** Output of a convolution: float32 values whose storage follows the activation-storage mode
   * (or `storage` when the caller names one). */
  private makeActivation<T extends Tensor>(shape: number[], storage?: 'float32'|'float16'): T {
    this.pendingStorage = storage || this.activationStorage;
    try {
      return Tensor.make(shape, {}, 'float32', this) as T;
    } finally {
      this.pendingStorage = null;
    }
  }

  private outId(t: Tensor): number {
    return this.data.get(t.dataId).id;
  }

  private assertNumeric(tensors: Array<Tensor|undefined|null>, op: string): void {
    for (const t of tensors) {
      if (t != null && !(t.dtype in DTYPE)) {
        throw new Error(`${op}: cuda backend does not support ${t.dtype} tensors`);
      }
    }
  }

  // ---- storage (backend.ts:92-126; CPU backend_cpu.ts:102-129, 199-254) --------------------
  register(dataId: DataId, shape: number[], dtype: DataType): void {
    if (this.data.has(dataId)) {
      throw new Error('Data buffer is already registered');   // backend_cpu.ts:119-121
    }
    if (this.pendingStorage === 'float16' && dtype === 'float32') {
      // a float32 tensor stored as IEEE half: the native library converts on write / read
      const r = binding.tensorRegister(this.ctx, shape.length, shape, STORAGE_F16);
      this.check(r.status);
      this.data.set(dataId, {id: r.out_id, dtype, shape: shape.slice(), half: true});
      return;
    }
    this.data.set(dataId, {id: this.newId(shape, dtype), dtype, shape: shape.slice()});
  }

  write(dataId: DataId, values: backend_util.BackendValues): void {
    if (values == null) {
      throw new Error('MathBackendCUDA.write(): values can not be null');   // backend_cpu.ts:125-127
    }
    const rec = this.data.get(dataId);
    let host = values as backend_util.TypedArray;
    if (rec.quantized) {
      // a quantised tensor is refilled with its raw bytes (e.g. the next batch of pixels)
      this.check(binding.tensorWrite(this.ctx, rec.id, host as Uint8Array));
      return;
    }
    const want = typedArrayFor(rec.dtype, 0).constructor;
    if (host.constructor !== want) {
      const conv = typedArrayFor(rec.dtype, host.length);
      conv.set(host as ArrayLike<number>);
      host = conv;
    }
    this.check(binding.tensorWrite(this.ctx, rec.id, host));
  }

  /** Extension: upload from pinned host memory (allocPinned) on the copy stream, overlapping the
   * kernels enqueued next; consumers wait for it (pass the tensor to graphLaunch's `inputs`). */
  writeAsync(dataId: DataId, pinned: ArrayBufferView): void {
    this.check(binding.tensorWriteAsync(this.ctx, this.data.get(dataId).id, pinned));
  }

  /** Extension: page-locked host memory for writeAsync / read. */
  allocPinned(nbytes: number): ArrayBuffer {
    const r = binding.hostAlloc(nbytes);
    if (r.status !== 0) throw new Error('pinned host allocation failed');
    return r.buffer;
  }

  readSync(dataId: DataId): backend_util.BackendValues {
    const rec = this.data.get(dataId);
    const out = typedArrayFor(rec.quantized ? 'float32' : rec.dtype, util.sizeFromShape(rec.shape));
    this.check(binding.tensorRead(this.ctx, rec.id, out));   // half storage arrives as float32
    return out;
  }

  /** The copy is enqueued now; the returned promise resolves when its event has completed,
   * without blocking the event loop (the wait runs in the addon's async work). */
  read(dataId: DataId): Promise<backend_util.BackendValues> {
    const rec = this.data.get(dataId);
    const out = typedArrayFor(rec.quantized ? 'float32' : rec.dtype, util.sizeFromShape(rec.shape));
    return binding.tensorReadPromise(this.ctx, rec.id, out);
  }

  /** Extension: read() into caller-owned (pinned) memory, e.g. a slice of a gather buffer. */
  readInto<T extends ArrayBufferView>(dataId: DataId, into: T): Promise<T> {
    return binding.tensorReadPromise(this.ctx, this.data.get(dataId).id, into);
  }

  disposeData(dataId: DataId): void {
    if (!this.data.has(dataId)) return;   // idempotent, backend_cpu.ts:228-237
    const rec = this.data.get(dataId);
    if (this.ctx != null) binding.tensorDispose(this.ctx, rec.id);
    this.data.delete(dataId);
  }

  memory() {
    const m = binding.ctxMemory(this.ctx);
    this.check(m.status);
    return {
      unreliable: false,
      numBytesInGPU: m.bytes_in_use,
      numBytesInGPUAllocated: m.bytes_reserved,
      numBuffersFree: m.num_buffers_cached,
      numDeviceAllocs: m.num_device_allocs,
      numDeviceTensors: m.num_tensors
    };
  }

  /** backend.ts:92-94 / BackendTimingInfo: device time between two events around f(). */
  async time(f: () => void): Promise<backend_util.BackendTimingInfo> {
    this.check(binding.ctxTimeBegin(this.ctx));
    f();
    const r = binding.ctxTimeEnd(this.ctx);
    this.check(r.status);
    return {kernelMs: r.kernel_ms, getExtraProfileInfo: () => `${r.num_launches} kernel launches`};
  }

  /** backend.ts:120-126: 16 while activations are stored as IEEE half, else 32. */
  floatPrecision(): 16|32 {
    return this.activationStorage === 'float16' ? 16 : 32;
  }

  epsilon(): number {
    return this.floatPrecision() === 32 ? EPSILON_FLOAT32 : EPSILON_FLOAT16;
  }

  dispose(): void {
    if (this.ctx != null) {
      binding.ctxDestroy(this.ctx);
      this.ctx = null;
    }
  }

  fromPixels(): Tensor3D {
    throw new Error('Not yet implemented.');
  }

  // ---- options / diagnostics (extensions) --------------------------------------------------
  /** '3xtf32' (default, float32-level accuracy) or 'tf32' (one tensor-core pass). */
  setMathMode(mode: '3xtf32'|'tf32'): void {
    this.mathMode = mode;
    this.check(binding.ctxSetOption(this.ctx, 'math_mode', MATH[mode]));
  }

  /** Extension: 'float32' (default) or 'float16'.  With 'float16' the outputs of the convolution
   * methods are stored as IEEE half, which halves the bytes every layer moves; the arithmetic
   * stays float32 / tf32 with float32 accumulation.  This is the reference's 16-bit precision
   * class (floatPrecision() == 16, test tolerance 1e-1: test_util.ts:23-39). */
  setActivationStorage(storage: 'float32'|'float16'): void {
    this.activationStorage = storage;
  }

  setOption(key: string, value: number): void {
    this.check(binding.ctxSetOption(this.ctx, key, value));
  }

  sync(timeoutMs = -1): void {
    this.check(binding.ctxSync(this.ctx, timeoutMs));
  }

  profileBegin(maxLaunches = 4096): void {
    this.check(binding.profileBegin(this.ctx, maxLaunches));
  }

  /** [kernel name, device milliseconds] of every launch since profileBegin(). */
  profileEnd(): Array<[string, number]> {
    const n = binding.profileEnd(this.ctx);
    this.check(n.status);
    const rows: Array<[string, number]> = [];
    for (let i = 0; i < n.num_launches; i++) {
      const r = binding.profileGet(this.ctx, i);
      this.check(r.status);
      rows.push([r.name, r.ms]);
    }
    return rows;
  }

  launchCount(): number {
    return binding.ctxLaunchCount(this.ctx);
  }

  stream(): bigint {
    return binding.ctxStream(this.ctx);
  }

  /** Extension: a float32 tensor stored as uint8 affine-quantised bytes, w = q*scale + min
   * (io/io_utils.ts:122-146).  Usable as the filter / b operand of the contractions and as a
   * depthwise filter; readSync returns the dequantised float32 values. */
  registerQuantized(shape: number[], q: Uint8Array, scale: number, min: number): Tensor {
    if (q.length !== util.sizeFromShape(shape)) {
      throw new Error('quantised byte count does not match the shape');
    }
    // The engine creates and tracks the tensor like any other backend output (Tensor.make
    // re-enters register(), which allocates a float32 buffer); that buffer is then swapped for
    // the uint8 storage, so that id, refcount, scopes and the tape all see a normal tensor.
    const t = this.makeOutput<Tensor>(shape, 'float32');
    const rec = this.data.get(t.dataId);
    const r = binding.tensorRegisterQuantized(this.ctx, shape.length, shape, q, scale, min);
    if (r.status !== 0) {
      t.dispose();
      this.check(r.status);
    }
    binding.tensorDispose(this.ctx, rec.id);
    this.data.set(t.dataId, {id: r.out_id, dtype: 'float32', shape: shape.slice(), quantized: true});
    return t;
  }

  // ---- fused epilogue marshalling ------------------------------------------------------------
  /** True when `t` broadcasts along the inner-most axis only: a scalar, or [.., 1, C]. */
  private static isChannelVector(t: Tensor, channels: number): boolean {
    if (t.size === 1) return true;
    return t.size === channels && t.shape[t.shape.length - 1] === channels;
  }

  /** The bias shapes the reference's own tests exercise are a full [M, N] matrix, [N], [1, N]
   * against a batched result, a scalar and [[1]] (ops/fused_test.ts:80-122, 242-268, 501-529).
   * A per-channel vector or a scalar goes into the kernel's epilogue; anything else is composed
   * from the linear op followed by add / activation, as MathBackendCPU does. */
  private epilogue(bias: Tensor|undefined, activation: CudaActivation|undefined, prelu: Tensor|undefined,
                   channels: number): {epi: binding.EpilogueLike|null, tmps: Array<number|null>, compose: boolean} {
    const tmps: Array<number|null> = [];
    let act: string = activation == null ? 'linear' : (activation as string);
    let clip: [number, number]|null = null;
    if (activation === 'relu6') {
      act = 'clip';
      clip = [0, 6];
    } else if (Array.isArray(activation)) {
      act = 'clip';
      clip = [activation[1], activation[2]];
    }
    if (!(act in ACT)) {
      throw new Error(`Activation ${act} has not been implemented for the cuda backend.`);
    }
    let fusable = true;
    if (bias != null && !BackendCuda.isChannelVector(bias, channels)) fusable = false;
    if (act === 'prelu') {
      if (prelu == null) throw new Error('prelu activation needs preluActivationWeights');
      if (!BackendCuda.isChannelVector(prelu, channels)) fusable = false;
    }
    if (!fusable) return {epi: null, tmps, compose: true};
    const epi: binding.EpilogueLike =
        {bias: 0, biasLen: 0, activation: ACT[act], prelu: 0, preluLen: 0, clipLo: 0, clipHi: 0};
    if (bias != null) {
      const [bid, tmp] = this.id(bias);
      tmps.push(tmp);
      epi.bias = bid;
      epi.biasLen = bias.size;
    }
    if (act === 'prelu') {
      const [pid, tmp] = this.id(prelu);
      tmps.push(tmp);
      epi.prelu = pid;
      epi.preluLen = prelu.size;
    }
    if (clip) {
      epi.clipLo = clip[0];
      epi.clipHi = clip[1];
    }
    return {epi, tmps, compose: false};
  }

  /** The unfused order of MathBackendCPU (backend_cpu.ts:542-555, 1536-1550). */
  private composeEpilogue<T extends Tensor>(result: T, bias: Tensor|undefined, activation: CudaActivation|undefined,
                                            prelu: Tensor|undefined): T {
    if (bias != null) {
      const r2 = this.add(result, bias) as T;
      result.dispose();
      result = r2;
    }
    if (activation == null || activation === 'linear') return result;
    let r2: T;
    if (activation === 'relu') {
      r2 = this.relu(result);
    } else if (activation === 'prelu') {
      r2 = this.prelu(result, prelu as T);
    } else if (activation === 'relu6') {
      r2 = this.clip(result, 0, 6);
    } else if (Array.isArray(activation)) {
      r2 = this.clip(result, activation[1], activation[2]);
    } else {
      throw new Error(`Activation ${activation} has not been implemented for the cuda backend.`);
    }
    result.dispose();
    return r2;
  }

  // ---- contractions --------------------------------------------------------------------------
  batchMatMul(a: Tensor3D, b: Tensor3D, transposeA: boolean, transposeB: boolean): Tensor3D {
    return this.fusedBatchMatMul({a, b, transposeA, transposeB});
  }

  /** backend.ts:134-138; CPU backend_cpu.ts:542-555. */
  fusedBatchMatMul({a, b, transposeA, transposeB, bias, activation, preluActivationWeights}: {
    a: Tensor3D, b: Tensor3D, transposeA: boolean, transposeB: boolean, bias?: Tensor,
    activation?: CudaActivation, preluActivationWeights?: Tensor
  }): Tensor3D {
    this.assertNumeric([a, b, bias], 'matMul');
    const batch = a.shape[0];
    const M = transposeA ? a.shape[2] : a.shape[1];
    const N = transposeB ? b.shape[1] : b.shape[2];
    const {epi, tmps, compose} = this.epilogue(bias, activation, preluActivationWeights, N);
    const [aid, ta] = this.id(a);
    const [bid, tb] = this.id(b);
    let out = this.makeOutput<Tensor3D>([batch, M, N]);
    this.check(binding.batchMatmul(
        this.ctx, aid, bid, this.outId(out), batch, a.shape[1], a.shape[2], b.shape[1], b.shape[2],
        transposeA ? 1 : 0, transposeB ? 1 : 0, epi));
    this.freeTmp(ta, tb, ...tmps);
    if (compose) out = this.composeEpilogue(out, bias, activation, preluActivationWeights);
    return out;
  }

  conv2d(x: Tensor4D, filter: Tensor4D, convInfo: Conv2DInfo): Tensor4D {
    return this.fusedConv2d(x, filter, convInfo);
  }

  /** backend.ts:414-418; CPU backend_cpu.ts:1536-1616. */
  fusedConv2d(x: Tensor4D, filter: Tensor4D, convInfo: Conv2DInfo, bias?: Tensor, activation?: CudaActivation,
              preluActivationWeights?: Tensor, outputStorage?: 'float32'|'float16'): Tensor4D {
    this.assertNumeric([x, filter, bias], 'conv2d');
    const {epi, tmps, compose} = this.epilogue(bias, activation, preluActivationWeights, convInfo.outChannels);
    const [xid, tx] = this.activationId(x);
    const [fid, tf] = this.id(filter);
    let out = this.makeActivation<Tensor4D>(convInfo.outShape, outputStorage);
    this.check(binding.conv2d(this.ctx, xid, fid, this.outId(out), convInfo, epi));
    this.freeTmp(tx, tf, ...tmps);
    if (compose) out = this.composeEpilogue(out, bias, activation, preluActivationWeights);
    return out;
  }

  /** backend.ts:431-434; CPU backend_cpu.ts:1979-2035. */
  depthwiseConv2D(x: Tensor4D, filter: Tensor4D, convInfo: Conv2DInfo): Tensor4D {
    return this.fusedDepthwiseConv2D(x, filter, convInfo);
  }

  /** Extension: depthwiseConv2D + add(bias) + activation in one kernel. */
  fusedDepthwiseConv2D(x: Tensor4D, filter: Tensor4D, convInfo: Conv2DInfo, bias?: Tensor,
                       activation?: CudaActivation): Tensor4D {
    this.assertNumeric([x, filter, bias], 'depthwiseConv2D');
    const {epi, tmps, compose} = this.epilogue(bias, activation, undefined, convInfo.outChannels);
    const [xid, tx] = this.activationId(x);
    const [fid, tf] = this.id(filter);
    let out = this.makeActivation<Tensor4D>(convInfo.outShape);
    this.check(binding.depthwiseConv2d(this.ctx, xid, fid, this.outId(out), convInfo, epi));
    this.freeTmp(tx, tf, ...tmps);
    if (compose) out = this.composeEpilogue(out, bias, activation, undefined);
    return out;
  }

  /** Extension: tf.separableConv2d's op pair (ops/conv.ts:574-654) with bias + activation after
   * each half; `convInfo` is the depthwise Conv2DInfo, pointwiseFilter is
   * [1, 1, convInfo.outChannels, outDepth].  Eligible shapes run as one kernel that never writes
   * the depthwise result to device memory; results equal the two separate calls. */
  fusedSeparableConv2d(x: Tensor4D, depthwiseFilter: Tensor4D, pointwiseFilter: Tensor4D, convInfo: Conv2DInfo,
                       dwBias?: Tensor, dwActivation?: CudaActivation, pwBias?: Tensor,
                       pwActivation?: CudaActivation): Tensor4D {
    this.assertNumeric([x, depthwiseFilter, pointwiseFilter, dwBias, pwBias], 'separableConv2d');
    const outDepth = pointwiseFilter.shape[3];
    if (pointwiseFilter.shape[0] !== 1 || pointwiseFilter.shape[1] !== 1 ||
        pointwiseFilter.shape[2] !== convInfo.outChannels) {
      throw new Error(
          `Error in separableConv2d: the third dimension of pointwise filter must be ` +
          `${convInfo.outChannels}, but got ${pointwiseFilter.shape[2]}.`);
    }
    const dw = this.epilogue(dwBias, dwActivation, undefined, convInfo.outChannels);
    const pw = this.epilogue(pwBias, pwActivation, undefined, outDepth);
    if (dw.compose || pw.compose) {
      // a bias that is not a channel vector: the two-call form handles the broadcast
      this.freeTmp(...dw.tmps, ...pw.tmps);
      const mid = this.fusedDepthwiseConv2D(x, depthwiseFilter, convInfo, dwBias, dwActivation);
      const ci = backend_util.computeConv2DInfo(mid.shape, pointwiseFilter.shape, 1, 1, 'valid');
      const out = this.fusedConv2d(mid, pointwiseFilter, ci, pwBias, pwActivation);
      mid.dispose();
      return out;
    }
    const [xid, tx] = this.activationId(x);
    const [did, td] = this.id(depthwiseFilter);
    const [pid, tp] = this.id(pointwiseFilter);
    const out = this.makeActivation<Tensor4D>([convInfo.batchSize, convInfo.outHeight, convInfo.outWidth, outDepth]);
    this.check(binding.separableConv2d(this.ctx, xid, did, pid, this.outId(out), convInfo, outDepth, dw.epi, pw.epi));
    this.freeTmp(tx, td, tp, ...dw.tmps, ...pw.tmps);
    return out;
  }

  // ---- pooling (backend.ts:453-466) --------------------------------------------------------------
  private pool(x: Tensor4D, convInfo: Conv2DInfo, isAvg: boolean): Tensor4D {
    this.assertNumeric([x], 'pool');
    const [xid, tx] = this.activationId(x);
    const out = this.makeOutput<Tensor4D>(convInfo.outShape);
    this.check(binding.pool2d(this.ctx, xid, this.outId(out), convInfo, isAvg ? 1 : 0));
    this.freeTmp(tx);
    return out;
  }

  maxPool(x: Tensor4D, convInfo: Conv2DInfo): Tensor4D {
    return this.pool(x, convInfo, false);
  }

  avgPool(x: Tensor4D, convInfo: Conv2DInfo): Tensor4D {
    return this.pool(x, convInfo, true);
  }

  // ---- element-wise (backend.ts:164-178, 300-346, 410) -------------------------------------------
  private binary(op: number, name: string, a: Tensor, b: Tensor, outDtype: DataType = 'float32'): Tensor {
    this.assertNumeric([a, b], name);
    const shape = backend_util.assertAndGetBroadcastShape(a.shape, b.shape);
    const [aid, ta] = this.id(a);
    const [bid, tb] = this.id(b);
    const out = this.makeOutput(shape, outDtype);
    this.check(binding.binary(this.ctx, op, aid, a.shape.length, a.shape, bid, b.shape.length, b.shape, this.outId(out)));
    this.freeTmp(ta, tb);
    return out;
  }

  add(a: Tensor, b: Tensor): Tensor {
    return this.binary(BINARY.add, 'add', a, b);
  }

  subtract(a: Tensor, b: Tensor): Tensor {
    return this.binary(BINARY.sub, 'subtract', a, b);
  }

  multiply(a: Tensor, b: Tensor): Tensor {
    return this.binary(BINARY.mul, 'multiply', a, b);
  }

  realDivide(a: Tensor, b: Tensor): Tensor {
    return this.binary(BINARY.div, 'realDivide', a, b);
  }

  prelu<T extends Tensor>(x: T, a: T): T {
    return this.binary(BINARY.prelu, 'prelu', x, a) as T;
  }

  notEqual(a: Tensor, b: Tensor): Tensor {
    return this.binary(BINARY.notEqual, 'notEqual', a, b, 'bool');
  }

  private unary<T extends Tensor>(op: number, name: string, x: T, p0 = 0, p1 = 0, outDtype: DataType = 'float32'): T {
    this.assertNumeric([x], name);
    const [xid, tx] = this.id(x);
    const out = this.makeOutput<T>(x.shape, outDtype);
    this.check(binding.unary(this.ctx, op, xid, this.outId(out), p0, p1));
    this.freeTmp(tx);
    return out;
  }

  relu<T extends Tensor>(x: T): T {
    return this.unary(UNARY.relu, 'relu', x);
  }

  clip<T extends Tensor>(x: T, min: number, max: number): T {
    return this.unary(UNARY.clip, 'clip', x, min, max);
  }

  exp<T extends Tensor>(x: T): T {
    return this.unary(UNARY.exp, 'exp', x);
  }

  log<T extends Tensor>(x: T): T {
    return this.unary(UNARY.log, 'log', x);
  }

  int<T extends Tensor>(x: T): T {
    return this.unary(UNARY.int, 'int', x, 0, 0, 'int32');
  }

  /** backend.ts:410; CPU backend_cpu.ts:1520-1534 (the gradient of relu). */
  step<T extends Tensor>(x: T, alpha = 0): T {
    return this.unary(UNARY.step, 'step', x, alpha);
  }

  // ---- gradient kernels (backend.ts:424-442, 456-466, 497) -----------------------------------------
  private convGradient(fn: (ctx: binding.Handle, a: number, b: number, out: number, info: Conv2DInfo) => number,
                       first: Tensor, second: Tensor, outShape: number[], convInfo: Conv2DInfo, name: string): Tensor4D {
    this.assertNumeric([first, second], name);
    const [aid, ta] = this.id(first);
    const [bid, tb] = this.id(second);
    const out = this.makeOutput<Tensor4D>(outShape);
    this.check(fn(this.ctx, aid, bid, this.outId(out), convInfo));
    this.freeTmp(ta, tb);
    return out;
  }

  conv2dDerInput(dy: Tensor4D, filter: Tensor4D, convInfo: Conv2DInfo): Tensor4D {
    return this.convGradient(binding.conv2dDerInput, dy, filter, convInfo.inShape, convInfo, 'conv2dDerInput');
  }

  conv2dDerFilter(x: Tensor4D, dy: Tensor4D, convInfo: Conv2DInfo): Tensor4D {
    const shape = [convInfo.filterHeight, convInfo.filterWidth, convInfo.inChannels, convInfo.outChannels];
    return this.convGradient(binding.conv2dDerFilter, x, dy, shape, convInfo, 'conv2dDerFilter');
  }

  depthwiseConv2DDerInput(dy: Tensor4D, filter: Tensor4D, convInfo: Conv2DInfo): Tensor4D {
    return this.convGradient(binding.depthwiseConv2dDerInput, dy, filter, convInfo.inShape, convInfo,
                             'depthwiseConv2DDerInput');
  }

  depthwiseConv2DDerFilter(x: Tensor4D, dy: Tensor4D, convInfo: Conv2DInfo): Tensor4D {
    const shape = [convInfo.filterHeight, convInfo.filterWidth, convInfo.inChannels,
                   Math.floor(convInfo.outChannels / Math.max(convInfo.inChannels, 1))];
    return this.convGradient(binding.depthwiseConv2dDerFilter, x, dy, shape, convInfo, 'depthwiseConv2DDerFilter');
  }

  private poolBackprop(dy: Tensor4D, x: Tensor4D, convInfo: Conv2DInfo, isAvg: boolean): Tensor4D {
    this.assertNumeric([dy, x], 'poolBackprop');
    const [did, td] = this.id(dy);
    const [xid, tx] = this.id(x);
    const out = this.makeOutput<Tensor4D>(x.shape);
    this.check(binding.pool2dBackprop(this.ctx, did, xid, this.outId(out), convInfo, isAvg ? 1 : 0));
    this.freeTmp(td, tx);
    return out;
  }

  maxPoolBackprop(dy: Tensor4D, x: Tensor4D, y: Tensor4D, convInfo: Conv2DInfo): Tensor4D {
    return this.poolBackprop(dy, x, convInfo, false);
  }

  avgPoolBackprop(dy: Tensor4D, x: Tensor4D, convInfo: Conv2DInfo): Tensor4D {
    return this.poolBackprop(dy, x, convInfo, true);
  }

  /** Extension: dy where lo <= x <= hi, else 0 (the gradient of clip as one kernel). */
  clipBackprop<T extends Tensor>(dy: T, x: T, lo: number, hi: number): T {
    this.assertNumeric([dy, x], 'clipBackprop');
    const [did, td] = this.id(dy);
    const [xid, tx] = this.id(x);
    const out = this.makeOutput<T>(x.shape);
    this.check(binding.clipBackprop(this.ctx, did, xid, this.outId(out), lo, hi));
    this.freeTmp(td, tx);
    return out;
  }

  transpose<T extends Tensor>(x: T, perm: number[]): T {
    this.assertNumeric([x], 'transpose');
    const [xid, tx] = this.id(x);
    const out = this.makeOutput<T>(perm.map(p => x.shape[p]));
    this.check(binding.transpose(this.ctx, xid, this.outId(out), perm.length, x.shape, perm));
    this.freeTmp(tx);
    return out;
  }

  // ---- reductions over the inner-most axes (backend.ts:183, 198, 255) ------------------------------
  private reduce(op: number, name: string, x: Tensor, axes: number[], outDtype: DataType): Tensor {
    this.assertNumeric([x], name);
    backend_util.assertAxesAreInnerMostDims(name, axes, x.rank);
    const [outShape, reduceShape] = backend_util.computeOutAndReduceShapes(x.shape, axes);
    const inner = util.sizeFromShape(reduceShape);
    const outer = util.sizeFromShape(outShape);
    const [xid, tx] = this.id(x);
    const out = this.makeOutput(outShape, outDtype);
    this.check(binding.reduceLast(this.ctx, op, xid, this.outId(out), outer, inner));
    this.freeTmp(tx);
    return out;
  }

  sum(x: Tensor, axes: number[]): Tensor {
    return this.reduce(REDUCE.sum, 'sum', x, axes, 'float32');
  }

  max(x: Tensor, axes: number[]): Tensor {
    return this.reduce(REDUCE.max, 'max', x, axes, 'float32');
  }

  argMax(x: Tensor, axis: number): Tensor {
    return this.reduce(REDUCE.argMax, 'argMax', x, [axis], 'int32');
  }

  /** Extension: tf.softmax over the last axis in one kernel (same per-stage rounding as the
   * op-layer chain max, sub, exp, sum, log, add, sub, exp: ops/softmax.ts:57-63,
   * ops/reduction_ops.ts:56-73). */
  softmax<T extends Tensor>(logits: T): T {
    this.assertNumeric([logits], 'softmax');
    const inner = logits.shape.length ? logits.shape[logits.shape.length - 1] : 1;
    const outer = inner ? logits.size / inner : 0;
    const [xid, tx] = this.id(logits);
    const out = this.makeOutput<T>(logits.shape);
    this.check(binding.softmaxLast(this.ctx, xid, this.outId(out), outer, inner));
    this.freeTmp(tx);
    return out;
  }

  // ---- metadata ops (backend.ts:480-486; backend_util.ts:36-76): free, no device work -------------
  reshape<T extends Tensor, R extends Rank>(x: T, shape: ShapeMap[R]): Tensor<R> {
    return backend_util.reshapeTensor(x, shape);
  }

  cast<T extends Tensor>(x: T, dtype: DataType): T {
    return backend_util.castTensor(x, dtype, this);
  }

  // ---- CUDA graph capture (extension) ------------------------------------------------------------------
  graphBegin(): void {
    this.check(binding.graphBegin(this.ctx));
  }

  graphEnd(): binding.Handle {
    const r = binding.graphEnd(this.ctx);
    this.check(r.status);
    return r.out;
  }

  /** Replays a captured graph.  `inputs`: tensors the graph reads that may have an asynchronous
   * upload (writeAsync) in flight; the replay is ordered after those uploads. */
  graphLaunch(graph: binding.Handle, inputs: Tensor[] = []): void {
    for (const t of inputs) {
      this.check(binding.tensorWait(this.ctx, this.data.get(t.dataId).id));
    }
    this.check(binding.graphLaunch(this.ctx, graph));
  }

  graphDestroy(graph: binding.Handle): void {
    binding.graphDestroy(this.ctx, graph);
  }
}

/** Flags of the backend, registered the way out-of-tree backends do
 * (tfjs-webgpu/src/flags_webgpu.ts:21-34); each mirrors a key of tfjs_cuda_ctx_set_option. */
export function registerCudaFlags(): void {
  ENV.registerFlag('CUDA_DEVICE', () => 0);
  ENV.registerFlag('CUDA_MATH_MODE', () => '3xtf32');
  ENV.registerFlag('CUDA_FUSE_SEPARABLE', () => 1);
  ENV.registerFlag('CUDA_DEQUANT_IN_GEMM', () => false);
}
