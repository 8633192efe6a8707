// The `Backend` of alpha (packages/core/src/interfaces.ts:38-151) on libalpha_cuda.so.
//
// This is the file a maintainer drops into `packages/cuda/src/backend.ts` beside
// `packages/helios`: it replaces HeliosBackend (packages/helios/src/backend.ts:1221) method for
// method and calls the C ABI through the generated table in ./ffi.ts.  It was written against
// the interface text; the build machines of this library have no JavaScript runtime, so it has
// not been executed — tests/test_ffi_tables.py checks every `C.alpha_*` call below against
// the header (name and argument count), and alpha2_b200/backend.py is the same class in Python,
// which every test of the library runs through.
//
// Lifetime model (the one helios uses): a TensorData is a plain object; its device buffer
// lives in a WeakMap side table keyed by the object (backend.ts:599); `data` is a lazy getter
// that copies back and caches (backend.ts:1143-1171); in-place ops invalidate the cache
// (backend.ts:706-729); releaseGpuTensor drops a reference, a FinalizationRegistry is the
// backstop (backend.ts:629-639, 688-699).  reshape shares the buffer through a reference count.
import { ptr } from "bun:ffi";
import type { Backend, TensorData, Shape, Dtype } from "@alpha/core";
import { C, check } from "./ffi";

type DType = Dtype | "bf16";
const CODE: Record<string, number> = { f32: 0, bf16: 1, i32: 2 };
const SIZE: Record<string, number> = { f32: 4, bf16: 2, i32: 4 };
const OP = { ADD: 0, SUB: 1, MUL: 2, DIV: 3 };
const UN = { NEG: 0, EXP: 1, LOG: 2, SQRT: 3, RELU: 4, SILU: 5, GELU: 6, SCALE: 7, CLAMP: 8, POW: 9, SOFTCAP: 10 };
const GEMM = { NT: 0, NN: 1, TN: 2 };
const EPI = { NONE: 0, GELU: 1, ADD: 2, GELU_BWD: 3 };

const sizeOf = (s: Shape) => s.reduce((a, b) => a * b, 1);

/** One device allocation, shared by the TensorData objects that view it. */
class Buf {
  refs = 1;
  constructor(readonly addr: bigint, readonly bytes: number) {}
}

const finalizer = new FinalizationRegistry<Buf>((b) => {
  if (--b.refs === 0) C.alpha_free(b.addr);
});

export class CudaBackend implements Backend {
  readonly name = "alpha_cuda";
  private side = new WeakMap<object, { buf: Buf; host: Float32Array | Int32Array | null }>();
  private opsMark = 0n;

  constructor(device = 0) {
    check(C.alpha_init(device));
  }

  // ── storage ────────────────────────────────────────────────────────────────
  private alloc(bytes: number): Buf {
    const out = new BigUint64Array(1);
    check(C.alpha_alloc(BigInt(Math.max(bytes, 1)), ptr(out)));
    return new Buf(out[0], bytes);
  }

  /** A new device tensor; `.data` reads it back on first access. */
  private make(shape: Shape, dtype: DType, buf?: Buf): TensorData {
    const self = this;
    const b = buf ?? this.alloc(sizeOf(shape) * SIZE[dtype]);
    const td = {
      shape: [...shape],
      dtype,
      get data() {
        return self.readBack(td as unknown as TensorData);
      },
    } as unknown as TensorData;
    this.side.set(td, { buf: b, host: null });
    finalizer.register(td, b);
    return td;
  }

  /** Device address of a tensor; host-created tensors (plain `{shape,dtype,data}`) upload on first use. */
  private addr(t: TensorData): bigint {
    let s = this.side.get(t);
    if (!s) {
      const dtype = t.dtype as DType;
      const host = t.data as Float32Array | Int32Array; // i32 indices go up as raw bits (backend.ts:298-313)
      const b = this.alloc(host.byteLength);
      check(C.alpha_h2d(b.addr, ptr(host), BigInt(host.byteLength)));
      s = { buf: b, host };
      this.side.set(t, s);
      finalizer.register(t, b);
      if (dtype === "bf16") throw new Error("host tensors are f32 or i32; cast on the device with castDtype");
    }
    return s.buf.addr;
  }

  private readBack(t: TensorData): Float32Array | Int32Array {
    const s = this.side.get(t)!;
    if (s.host) return s.host;
    const n = sizeOf(t.shape);
    if ((t.dtype as DType) === "bf16") {
      const raw = new Uint16Array(n);
      check(C.alpha_d2h(ptr(raw), s.buf.addr, BigInt(raw.byteLength)));
      const bits = new Uint32Array(n);
      for (let i = 0; i < n; i++) bits[i] = raw[i] << 16;
      s.host = new Float32Array(bits.buffer);
    } else {
      s.host = t.dtype === "i32" ? new Int32Array(n) : new Float32Array(n);
      check(C.alpha_d2h(ptr(s.host), s.buf.addr, BigInt(s.host.byteLength))); // waits for the stream
    }
    return s.host;
  }

  private invalidate(t: TensorData): void {
    const s = this.side.get(t);
    if (s) s.host = null;
  }

  private i64(values: number[]): BigInt64Array {
    return BigInt64Array.from(values.map((v) => BigInt(v)));
  }

  // ── duck-typed extras the trainer and CLI probe (trainer.ts:623-641,998-1044; train.ts:284-318) ──
  releaseGpuTensor(t: TensorData): void {
    const s = this.side.get(t);
    if (!s) return;
    this.side.delete(t);
    finalizer.unregister(t);
    if (--s.buf.refs === 0) check(C.alpha_free(s.buf.addr)); // the block returns to the library's pool
  }
  flush(): void {} // every call is already enqueued on the stream
  syncGpu(): void {
    check(C.alpha_stream_sync());
  }
  purgeBufferPools(): void {
    check(C.alpha_purge_pools());
  }
  checkAsyncError(): void {
    check(C.alpha_check_async_error());
  }
  private launchCount(): bigint {
    const out = new BigUint64Array(1);
    check(C.alpha_launch_count(ptr(out)));
    return out[0];
  }
  resetStepOps(): void {
    this.opsMark = this.launchCount();
  }
  get gpuOpsThisStep(): number {
    return Number(this.launchCount() - this.opsMark);
  }
  gpuMemStats() {
    const s = new BigUint64Array(5);
    check(C.alpha_mem_stats(ptr(s)));
    return { bytesInUse: Number(s[0]), bytesCached: Number(s[1]), peakInUse: Number(s[2]), deviceMallocs: Number(s[3]), allocs: Number(s[4]) };
  }
  getDeviceInfo() {
    const raw = new Uint8Array(128 + 4 * 4 + 8 * 2);
    check(C.alpha_device_info(ptr(raw)));
    const v = new DataView(raw.buffer);
    const name = new TextDecoder().decode(raw.subarray(0, raw.indexOf(0)));
    return { deviceName: name, vendorId: v.getInt32(128, true), smCount: v.getInt32(132, true) }; // vendorId 0x10de
  }
  smokeTest(): boolean {
    const c = this.matmul(this.fromArray([1, 2, 3, 4], [2, 2]), this.fromArray([5, 6, 7, 8], [2, 2]));
    return Array.from(c.data as Float32Array).map(Math.round).join() === "19,22,43,50";
  }
  setMinGpuSize(_n: number): void {} // every tensor lives on the device; there is no CPU path
  readonly coopMatmulPaused = false;
  getMatmulCoopStats() {
    return { coopDispatches: 0, fallbackDispatches: 0 };
  }

  // ── creation (interfaces.ts:42-46) ───────────────────────────────────────────
  zeros(shape: Shape, dtype: Dtype = "f32"): TensorData {
    const t = this.make(shape, dtype);
    check(C.alpha_memset(this.addr(t), 0, BigInt(sizeOf(shape) * SIZE[dtype])));
    return t;
  }
  full(shape: Shape, value: number, dtype: Dtype = "f32"): TensorData {
    const t = this.make(shape, dtype);
    check(C.alpha_fill(this.addr(t), BigInt(sizeOf(shape)), value, CODE[dtype]));
    return t;
  }
  ones(shape: Shape, dtype: Dtype = "f32"): TensorData {
    return this.full(shape, 1, dtype);
  }
  fromArray(data: number[], shape: Shape, dtype: Dtype = "f32"): TensorData {
    if (data.length !== sizeOf(shape)) throw new Error(`Data length ${data.length} does not match shape size ${sizeOf(shape)}`);
    const host = dtype === "i32" ? Int32Array.from(data) : Float32Array.from(data);
    const t = this.make(shape, dtype);
    check(C.alpha_h2d(this.addr(t), ptr(host), BigInt(host.byteLength)));
    return t;
  }
  randn(shape: Shape, dtype: Dtype = "f32"): TensorData {
    // cpu_ref.ts:134-140 draws from SeededRng(42); the same generator is exported by the library
    const rng = new Uint8Array(24);
    check(C.alpha_rng_seed(ptr(rng), 42));
    const host = new Float32Array(sizeOf(shape));
    check(C.alpha_rng_fill_gauss(ptr(rng), ptr(host), BigInt(host.length), 1.0));
    const t = this.make(shape, dtype);
    check(C.alpha_h2d(this.addr(t), ptr(host), BigInt(host.byteLength)));
    return t;
  }

  // ── elementwise (interfaces.ts:49-71) ─────────────────────────────────────────
  private binary(op: number, a: TensorData, b: TensorData): TensorData {
    const same = a.shape.length === b.shape.length && a.shape.every((d, i) => d === b.shape[i]);
    if (same) {
      const out = this.make(a.shape, a.dtype as DType);
      check(C.alpha_binary(op, this.addr(a), this.addr(b), this.addr(out), BigInt(sizeOf(a.shape)), CODE[a.dtype]));
      return out;
    }
    const nd = Math.max(a.shape.length, b.shape.length);
    const pad = (s: Shape) => [...Array(nd - s.length).fill(1), ...s];
    const sa = pad(a.shape), sb = pad(b.shape);
    const shape = sa.map((d, i) => Math.max(d, sb[i]));
    const strides = (s: number[]) => {
      const st = Array(nd).fill(0);
      let acc = 1;
      for (let d = nd - 1; d >= 0; d--) { st[d] = s[d] === 1 ? 0 : acc; acc *= s[d]; }
      return st;
    };
    const out = this.make(shape, a.dtype as DType);
    check(C.alpha_binary_bcast(op, this.addr(a), this.addr(b), this.addr(out), nd, ptr(this.i64(shape)), ptr(this.i64(strides(sa))), ptr(this.i64(strides(sb))), CODE[a.dtype]));
    return out;
  }
  add(a: TensorData, b: TensorData) { return this.binary(OP.ADD, a, b); }
  sub(a: TensorData, b: TensorData) { return this.binary(OP.SUB, a, b); }
  mul(a: TensorData, b: TensorData) { return this.binary(OP.MUL, a, b); }
  div(a: TensorData, b: TensorData) { return this.binary(OP.DIV, a, b); }

  private unary(op: number, a: TensorData, p0 = 0, p1 = 0): TensorData {
    const out = this.make(a.shape, a.dtype as DType);
    check(C.alpha_unary(op, this.addr(a), this.addr(out), BigInt(sizeOf(a.shape)), p0, p1, CODE[a.dtype]));
    return out;
  }
  neg(a: TensorData) { return this.unary(UN.NEG, a); }
  exp(a: TensorData) { return this.unary(UN.EXP, a); }
  log(a: TensorData) { return this.unary(UN.LOG, a); }
  sqrt(a: TensorData) { return this.unary(UN.SQRT, a); }
  pow(a: TensorData, e: number) { return this.unary(UN.POW, a, e); }
  scale(a: TensorData, s: number) { return this.unary(UN.SCALE, a, s); }
  clamp(a: TensorData, lo: number, hi: number) { return this.unary(UN.CLAMP, a, lo, hi); }
  gelu(a: TensorData) { return this.unary(UN.GELU, a); }
  relu(a: TensorData) { return this.unary(UN.RELU, a); }
  silu(a: TensorData) { return this.unary(UN.SILU, a); }
  softCap(a: TensorData, cap: number) { return this.unary(UN.SOFTCAP, a, cap); }

  private unaryBwd(op: number, x: TensorData, g: TensorData, p0 = 0, p1 = 0): TensorData {
    const out = this.make(x.shape, x.dtype as DType);
    check(C.alpha_unary_bwd(op, this.addr(x), this.addr(g), this.addr(out), BigInt(sizeOf(x.shape)), p0, p1, CODE[x.dtype]));
    return out;
  }
  geluBackward(x: TensorData, g: TensorData) { return this.unaryBwd(UN.GELU, x, g); }
  reluBackward(x: TensorData, g: TensorData) { return this.unaryBwd(UN.RELU, x, g); }
  siluBackward(x: TensorData, g: TensorData) { return this.unaryBwd(UN.SILU, x, g); }
  clampBackward(x: TensorData, g: TensorData, lo: number, hi: number) { return this.unaryBwd(UN.CLAMP, x, g, lo, hi); }
  softCapBackward(g: TensorData, x: TensorData, cap: number) { return this.unaryBwd(UN.SOFTCAP, x, g, cap); }

  siluMul(a: TensorData, b: TensorData): TensorData {
    const out = this.make(a.shape, a.dtype as DType);
    check(C.alpha_silu_mul_fwd(this.addr(a), this.addr(b), this.addr(out), BigInt(sizeOf(a.shape)), CODE[a.dtype]));
    return out;
  }
  siluMulBackward(a: TensorData, b: TensorData, g: TensorData): TensorData[] {
    const da = this.make(a.shape, a.dtype as DType), db = this.make(a.shape, a.dtype as DType);
    check(C.alpha_silu_mul_bwd(this.addr(a), this.addr(b), this.addr(g), this.addr(da), this.addr(db), BigInt(sizeOf(a.shape)), CODE[a.dtype]));
    return [da, db];
  }
  addInplace(a: TensorData, b: TensorData): void {
    check(C.alpha_add_inplace(this.addr(a), this.addr(b), BigInt(sizeOf(a.shape)), CODE[a.dtype], CODE[b.dtype]));
    this.invalidate(a);
  }
  scaleInplace(a: TensorData, s: number): void {
    check(C.alpha_scale_inplace(this.addr(a), s, BigInt(sizeOf(a.shape)), CODE[a.dtype]));
    this.invalidate(a);
  }
  castDtype(a: TensorData, dtype: Dtype): TensorData {
    const out = this.make(a.shape, dtype as DType);
    check(C.alpha_cast(this.addr(a), CODE[a.dtype], this.addr(out), CODE[dtype], BigInt(sizeOf(a.shape))));
    return out;
  }
  broadcast(a: TensorData, target: Shape): TensorData {
    const nd = target.length;
    const s = [...Array(nd - a.shape.length).fill(1), ...a.shape];
    const st = Array(nd).fill(0);
    let acc = 1;
    for (let d = nd - 1; d >= 0; d--) { st[d] = s[d] === 1 && target[d] !== 1 ? 0 : acc; acc *= s[d]; }
    const out = this.make(target, a.dtype as DType);
    check(C.alpha_broadcast(this.addr(a), this.addr(out), nd, ptr(this.i64([...target])), ptr(this.i64(st)), CODE[a.dtype]));
    return out;
  }
  clone(a: TensorData): TensorData {
    const out = this.make(a.shape, a.dtype as DType);
    check(C.alpha_d2d(this.addr(out), this.addr(a), BigInt(sizeOf(a.shape) * SIZE[a.dtype])));
    return out;
  }

  // ── matmul family (interfaces.ts:53,111-112) ────────────────────────────────────
  private gemm(layout: number, a: TensorData, b: TensorData, M: number, N: number, K: number, lda: number, ldb: number, outShape: Shape, outDtype: DType = a.dtype as DType, epilogue = EPI.NONE, aux: TensorData | null = null, out: TensorData | null = null, accumulate = false): TensorData {
    const c = out ?? this.make(outShape, outDtype);
    check(C.alpha_gemm(layout, this.addr(a), this.addr(b), this.addr(c), BigInt(M), BigInt(N), BigInt(K), BigInt(lda), BigInt(ldb), BigInt(N), CODE[a.dtype], CODE[outDtype], epilogue, aux ? this.addr(aux) : 0n, BigInt(N), accumulate ? 1 : 0));
    this.invalidate(c);
    return c;
  }
  matmul(a: TensorData, b: TensorData): TensorData {
    const [M, K] = a.shape.slice(-2), [K2, N] = b.shape.slice(-2);
    if (K !== K2) throw new Error(`matmul shape mismatch: [${a.shape}] x [${b.shape}]`);
    const ab = a.shape.slice(0, -2), bb = b.shape.slice(0, -2);
    if (bb.length === 0) return this.gemm(GEMM.NN, a, b, sizeOf(ab) * M, N, K, K, N, [...ab, M, N]);
    const nb = Math.max(sizeOf(ab), sizeOf(bb)); // batched fp32 (the unfused attention branch)
    const out = this.make([...(sizeOf(ab) >= sizeOf(bb) ? ab : bb), M, N], "f32");
    check(C.alpha_gemm_batched_f32(GEMM.NN, this.addr(a), this.addr(b), this.addr(out), BigInt(M), BigInt(N), BigInt(K), BigInt(K), BigInt(N), BigInt(N), BigInt(nb), BigInt(sizeOf(ab) === nb ? M * K : 0), BigInt(sizeOf(bb) === nb ? K * N : 0), BigInt(M * N)));
    return out;
  }
  matmulTransposed(a: TensorData, b: TensorData): TensorData {
    const K = a.shape[a.shape.length - 1], N = b.shape[0];
    return this.gemm(GEMM.NT, a, b, sizeOf(a.shape) / K, N, K, K, K, [...a.shape.slice(0, -1), N]);
  }
  /** A^T B with A [K, M], B [K, N]; weight gradients of bf16 GEMMs come out in f32. */
  matmulTransposedA(a: TensorData, b: TensorData, into?: TensorData): TensorData {
    const M = a.shape[a.shape.length - 1], N = b.shape[b.shape.length - 1], K = sizeOf(a.shape) / M;
    const outDtype: DType = (a.dtype as DType) === "bf16" ? "f32" : (a.dtype as DType);
    return this.gemm(GEMM.TN, a, b, M, N, K, M, N, [M, N], outDtype, EPI.NONE, null, into ?? null, into !== undefined);
  }
  /** Fused forms this backend adds (probed with `typeof backend.x === "function"`). */
  matmulTransposedGelu(a: TensorData, b: TensorData): [TensorData, TensorData] {
    const K = a.shape[a.shape.length - 1], N = b.shape[0], shape = [...a.shape.slice(0, -1), N];
    const pre = this.make(shape, a.dtype as DType);
    const act = this.gemm(GEMM.NT, a, b, sizeOf(a.shape) / K, N, K, K, K, shape, a.dtype as DType, EPI.GELU, pre);
    return [pre, act];
  }
  matmulTransposedAdd(a: TensorData, b: TensorData, residual: TensorData): TensorData {
    const K = a.shape[a.shape.length - 1], N = b.shape[0];
    return this.gemm(GEMM.NT, a, b, sizeOf(a.shape) / K, N, K, K, K, residual.shape, a.dtype as DType, EPI.ADD, residual);
  }
  matmulGeluBackward(g: TensorData, w: TensorData, pre: TensorData): TensorData {
    const [N, K] = w.shape;
    return this.gemm(GEMM.NN, g, w, sizeOf(g.shape) / N, K, N, N, K, pre.shape, g.dtype as DType, EPI.GELU_BWD, pre);
  }
  matmulInto(a: TensorData, b: TensorData, into: TensorData): TensorData {
    const [K, N] = b.shape;
    return this.gemm(GEMM.NN, a, b, sizeOf(a.shape) / K, N, K, K, N, into.shape, a.dtype as DType, EPI.ADD, into, into);
  }

  // ── reductions (interfaces.ts:54-55,72-73,144-146) ────────────────────────────────
  sum(a: TensorData, axis?: number, keepdims = false, scaleBy = 1): TensorData {
    if (axis === undefined) {
      const out = this.make(keepdims ? a.shape.map(() => 1) : [], a.dtype as DType);
      check(C.alpha_sum_axis(this.addr(a), this.addr(out), 1n, BigInt(sizeOf(a.shape)), 1n, scaleBy, CODE[a.dtype]));
      return out;
    }
    const ax = axis < 0 ? axis + a.shape.length : axis;
    const outer = sizeOf(a.shape.slice(0, ax)), dim = a.shape[ax], inner = sizeOf(a.shape.slice(ax + 1));
    const out = this.make([...a.shape.slice(0, ax), ...(keepdims ? [1] : []), ...a.shape.slice(ax + 1)], a.dtype as DType);
    check(C.alpha_sum_axis(this.addr(a), this.addr(out), BigInt(outer), BigInt(dim), BigInt(inner), scaleBy, CODE[a.dtype]));
    return out;
  }
  mean(a: TensorData, axis?: number, keepdims = false): TensorData {
    return this.sum(a, axis, keepdims, 1 / (axis === undefined ? sizeOf(a.shape) : a.shape[axis < 0 ? axis + a.shape.length : axis]));
  }
  private softmaxImpl(a: TensorData, logMode: number): TensorData {
    const cols = a.shape[a.shape.length - 1];
    const out = this.make(a.shape, a.dtype as DType);
    check(C.alpha_softmax(this.addr(a), this.addr(out), BigInt(sizeOf(a.shape) / cols), BigInt(cols), logMode, CODE[a.dtype]));
    return out;
  }
  softmax(a: TensorData, _axis?: number) { return this.softmaxImpl(a, 0); }
  logSoftmax(a: TensorData, _axis?: number) { return this.softmaxImpl(a, 1); }
  totalSumOfSquares(tensors: TensorData[]): TensorData {
    const out = this.make([], "f32");
    const ptrs = BigUint64Array.from(tensors.map((t) => this.addr(t)));
    const counts = this.i64(tensors.map((t) => sizeOf(t.shape)));
    const dts = Int32Array.from(tensors.map((t) => CODE[t.dtype]));
    check(C.alpha_sumsq_multi(ptr(ptrs), ptr(counts), ptr(dts), tensors.length, this.addr(out)));
    return out;
  }
  sumOfSquares(t: TensorData) { return this.totalSumOfSquares([t]); }
  checkFinite(t: TensorData): TensorData {
    const out = this.make([], "f32");
    check(C.alpha_check_finite(this.addr(t), BigInt(sizeOf(t.shape)), CODE[t.dtype], this.addr(out)));
    return out;
  }

  // ── nn (interfaces.ts:67-74,103-105) ───────────────────────────────────────────
  embedding(weight: TensorData, indices: TensorData): TensorData {
    const [vocab, dim] = weight.shape;
    const out = this.make([...indices.shape, dim], weight.dtype as DType);
    check(C.alpha_embedding_fwd(this.addr(weight), this.addr(indices), this.addr(out), BigInt(sizeOf(indices.shape)), BigInt(dim), BigInt(vocab), CODE[weight.dtype]));
    return out;
  }
  embeddingBackward(indices: TensorData, g: TensorData, vocabSize: number): TensorData {
    const dim = g.shape[g.shape.length - 1];
    const out = this.make([vocabSize, dim], "f32");
    check(C.alpha_embedding_bwd(this.addr(indices), this.addr(g), this.addr(out), BigInt(sizeOf(indices.shape)), BigInt(dim), BigInt(vocabSize), CODE[g.dtype], 0));
    return out;
  }
  layerNorm(x: TensorData, w: TensorData, b: TensorData, eps: number): TensorData {
    const dim = x.shape[x.shape.length - 1];
    const out = this.make(x.shape, x.dtype as DType);
    check(C.alpha_layernorm_fwd(this.addr(x), this.addr(w), this.addr(b), this.addr(out), BigInt(sizeOf(x.shape) / dim), BigInt(dim), eps, CODE[x.dtype]));
    return out;
  }
  layerNormBackward(x: TensorData, w: TensorData, g: TensorData, eps: number) {
    const dim = x.shape[x.shape.length - 1];
    const dx = this.make(x.shape, x.dtype as DType), dw = this.make(w.shape, "f32"), db = this.make(w.shape, "f32");
    check(C.alpha_layernorm_bwd(this.addr(x), this.addr(w), this.addr(g), this.addr(dx), this.addr(dw), this.addr(db), BigInt(sizeOf(x.shape) / dim), BigInt(dim), eps, CODE[x.dtype], 0, 0n));
    return { dx, dw, db };
  }
  crossEntropy(logits: TensorData, targets: TensorData): TensorData {
    const [N, V] = logits.shape;
    const out = this.make([], "f32");
    check(C.alpha_cross_entropy_fwd(this.addr(logits), this.addr(targets), this.addr(out), BigInt(N), BigInt(V), BigInt(V), CODE[logits.dtype]));
    return out;
  }
  crossEntropyBackward(logits: TensorData, targets: TensorData, gradOutput: TensorData): TensorData {
    const [N, V] = logits.shape;
    const out = this.make(logits.shape, logits.dtype as DType);
    check(C.alpha_cross_entropy_bwd(this.addr(logits), this.addr(targets), this.addr(gradOutput), this.addr(out), BigInt(N), BigInt(V), BigInt(V), CODE[logits.dtype]));
    return out;
  }

  // ── views / layout (interfaces.ts:77-80,117-121) ────────────────────────────────
  reshape(a: TensorData, shape: Shape): TensorData {
    if (sizeOf(shape) !== sizeOf(a.shape)) throw new Error(`Cannot reshape [${a.shape}] to [${shape}]: size mismatch`);
    this.addr(a);
    const s = this.side.get(a)!;
    s.buf.refs++; // shared storage, as helios does (backend.ts:669-676)
    return this.make(shape, a.dtype as DType, s.buf);
  }
  transpose(a: TensorData, dim0: number, dim1: number): TensorData {
    const nd = a.shape.length, d0 = dim0 < 0 ? dim0 + nd : dim0, d1 = dim1 < 0 ? dim1 + nd : dim1;
    const shape = [...a.shape];
    [shape[d0], shape[d1]] = [shape[d1], shape[d0]];
    const out = this.make(shape, a.dtype as DType);
    check(C.alpha_transpose(this.addr(a), this.addr(out), nd, ptr(this.i64([...a.shape])), d0, d1, CODE[a.dtype]));
    return out;
  }
  slice(a: TensorData, starts: number[], ends: number[]): TensorData {
    const [rows, cols] = a.shape;
    const out = this.make([rows, ends[1] - starts[1]], a.dtype as DType);
    check(C.alpha_slice_cols(this.addr(a), this.addr(out), BigInt(rows), BigInt(cols), BigInt(starts[1]), BigInt(ends[1]), CODE[a.dtype]));
    return out;
  }
  scatterSlice(g: TensorData, origShape: Shape, starts: number[], ends: number[]): TensorData {
    const [rows, cols] = origShape;
    const out = this.make(origShape, g.dtype as DType);
    check(C.alpha_scatter_cols(this.addr(g), this.addr(out), BigInt(rows), BigInt(cols), BigInt(starts[1]), BigInt(ends[1]), CODE[g.dtype]));
    return out;
  }
  sliceQkv(a: TensorData): [TensorData, TensorData, TensorData] {
    const [rows, c3] = a.shape, d = c3 / 3;
    const q = this.make([rows, d], a.dtype as DType), k = this.make([rows, d], a.dtype as DType), v = this.make([rows, d], a.dtype as DType);
    check(C.alpha_slice_qkv(this.addr(a), this.addr(q), this.addr(k), this.addr(v), BigInt(rows), BigInt(d), CODE[a.dtype]));
    return [q, k, v];
  }
  causalMask(size: number): TensorData {
    const out = this.make([size, size], "f32");
    check(C.alpha_causal_mask(this.addr(out), BigInt(size)));
    return out;
  }
  maskedFill(a: TensorData, mask: TensorData, value: number): TensorData {
    const out = this.make(a.shape, a.dtype as DType);
    check(C.alpha_masked_fill(this.addr(a), this.addr(mask), this.addr(out), BigInt(sizeOf(a.shape)), BigInt(sizeOf(mask.shape)), value, CODE[a.dtype]));
    return out;
  }
  dropoutMask(shape: Shape, seed: number, counter: number, p: number): TensorData {
    const out = this.make(shape, "f32");
    check(C.alpha_dropout_mask(this.addr(out), BigInt(sizeOf(shape)), seed, counter, p, CODE.f32));
    return out;
  }
  residualDropoutAdd(residual: TensorData, projected: TensorData, mask: TensorData): TensorData {
    const out = this.make(residual.shape, residual.dtype as DType);
    check(C.alpha_residual_dropout_add(this.addr(residual), this.addr(projected), this.addr(mask), this.addr(out), BigInt(sizeOf(residual.shape)), CODE[residual.dtype]));
    return out;
  }

  // ── fused attention (interfaces.ts:127-135) ─────────────────────────────────────
  /** alpha_attn_params_t: 10 x i64, 2 x f32, 1 x i32 (96 bytes with tail padding). */
  private attnParams(batch: number, heads: number, T: number, D: number, q: number[], o: number[], scale: number, cap: number, dtype: DType): Uint8Array {
    const raw = new Uint8Array(96), v = new DataView(raw.buffer);
    [batch, heads, T, D, ...q, ...o].forEach((x, i) => v.setBigInt64(8 * i, BigInt(x), true));
    v.setFloat32(80, scale, true);
    v.setFloat32(84, cap, true);
    v.setInt32(88, CODE[dtype], true);
    return raw;
  }
  flashAttention(Q: TensorData, K: TensorData, V: TensorData, T: number, scale: number, softCap: number) {
    const [BH, , D] = Q.shape;
    const p = this.attnParams(BH, 1, T, D, [T * D, 0, D], [T * D, 0, D], scale, softCap, Q.dtype as DType);
    const output = this.make(Q.shape, Q.dtype as DType), lse = this.make([BH, T], "f32");
    check(C.alpha_flash_attn_fwd(this.addr(Q), this.addr(K), this.addr(V), this.addr(output), this.addr(lse), ptr(p)));
    return { output, lse };
  }
  flashAttentionBackward(Q: TensorData, K: TensorData, V: TensorData, O: TensorData, dO: TensorData, lse: TensorData, T: number, scale: number, softCap: number) {
    const [BH, , D] = Q.shape;
    const p = this.attnParams(BH, 1, T, D, [T * D, 0, D], [T * D, 0, D], scale, softCap, Q.dtype as DType);
    const dQ = this.make(Q.shape, Q.dtype as DType), dK = this.make(Q.shape, Q.dtype as DType), dV = this.make(Q.shape, Q.dtype as DType);
    check(C.alpha_flash_attn_bwd(this.addr(Q), this.addr(K), this.addr(V), this.addr(O), this.addr(dO), this.addr(lse), this.addr(dQ), this.addr(dK), this.addr(dV), ptr(p)));
    return { dQ, dK, dV };
  }
  /** Causal attention reading q, k, v in place from the fused projection [B*T, 3E] (optional hook). */
  attentionQkv(qkv: TensorData, B: number, T: number, H: number, scale: number, softCap: number): [TensorData, TensorData] {
    const E3 = qkv.shape[1], E = E3 / 3, D = E / H, es = BigInt(SIZE[qkv.dtype]);
    const p = this.attnParams(B, H, T, D, [T * E3, D, E3], [T * E, D, E], scale, softCap, qkv.dtype as DType);
    const out = this.make([B * T, E], qkv.dtype as DType), lse = this.make([B * H, T], "f32");
    const base = this.addr(qkv);
    check(C.alpha_flash_attn_fwd(base, base + BigInt(E) * es, base + BigInt(2 * E) * es, this.addr(out), this.addr(lse), ptr(p)));
    return [out, lse];
  }

  /** Two weight gradients A_i^T B_i over the same K in one launch (each argument as for
   *  matmulTransposedA: a [K, M], b [K, N] bf16, an existing f32 gradient to add into or
   *  undefined); two GEMMs that would each fill half of the device need no split over K this way. */
  matmulTransposedAPair(first: [TensorData, TensorData, TensorData?], second: [TensorData, TensorData, TensorData?]): TensorData[] {
    const K = sizeOf(first[0].shape) / first[0].shape[first[0].shape.length - 1];
    const outs: TensorData[] = [];
    const a: (bigint | number)[] = [];
    for (const [x, y, into] of [first, second]) {
      const M = x.shape[x.shape.length - 1], N = y.shape[y.shape.length - 1];
      const out = into ?? this.make([M, N], "f32");
      outs.push(out);
      a.push(this.addr(x), this.addr(y), this.addr(out), BigInt(M), BigInt(N), BigInt(M), BigInt(N), BigInt(N), into ? 1 : 0);
    }
    check((C.alpha_gemm_tn_pair as (...args: (bigint | number)[]) => number)(...a, BigInt(K)));
    outs.forEach((t) => this.invalidate(t));
    return outs;
  }
  /** Rotary embedding of `heads` heads of width D in the column block that starts at column
   *  `colOffset` of x [B*T, ld], in place (`inverse`: the transposed rotation, i.e. the backward).
   *  For the fused projection [B*T, 3E]: heads = 2H, ld = 3E, colOffset = 0 rotates q and k. */
  rope(x: TensorData, B: number, T: number, heads: number, D: number, ld: number, colOffset = 0, theta = 10000, inverse = false): void {
    const p = this.addr(x) + BigInt(colOffset * SIZE[x.dtype]);
    check(C.alpha_rope(p, p, BigInt(B), BigInt(T), BigInt(heads), BigInt(D), BigInt(ld), theta, inverse ? 1 : 0, CODE[x.dtype]));
    this.invalidate(x);
  }
  /** The same for q and k of a fused [B*T, 3E] activation into a new tensor (v copied). */
  ropeQkv(qkv: TensorData, B: number, T: number, H: number, theta = 10000, inverse = false): TensorData {
    const D = qkv.shape[1] / 3 / H;
    const out = this.make(qkv.shape, qkv.dtype as DType);
    check(C.alpha_rope_qkv(this.addr(qkv), this.addr(out), BigInt(B), BigInt(T), BigInt(H), BigInt(D), theta, inverse ? 1 : 0, CODE[qkv.dtype]));
    return out;
  }

  // ── optimizer (interfaces.ts:149-150) ────────────────────────────────────────────
  adamwStep(params: TensorData, grads: TensorData, m: TensorData, v: TensorData, lr: number, beta1: number, beta2: number, eps: number, weightDecay: number, bc1: number, bc2: number, gradScale = 1, shadow?: TensorData): void {
    check(C.alpha_adamw(this.addr(params), this.addr(grads), this.addr(m), this.addr(v), BigInt(sizeOf(params.shape)), lr, beta1, beta2, eps, weightDecay, bc1, bc2, gradScale, CODE[grads.dtype], shadow ? this.addr(shadow) : 0n));
    [params, m, v].forEach((t) => this.invalidate(t));
    if (shadow) this.invalidate(shadow);
  }

  // ── comparison and sampling utilities: host reads, off the train-step path ─────────────
  equal(a: TensorData, b: TensorData): boolean {
    const x = a.data, y = b.data;
    return x.length === y.length && x.every((v, i) => v === y[i]);
  }
  allClose(a: TensorData, b: TensorData, atol = 1e-5, rtol = 1e-8): boolean {
    const x = a.data, y = b.data;
    return x.length === y.length && x.every((v, i) => Math.abs(v - y[i]) <= atol + rtol * Math.abs(y[i]));
  }
  private offPath(name: string): never {
    throw new Error(`${name} is not part of the train-step path this backend implements`);
  }
  cat(_t: TensorData[], _axis: number): TensorData { return this.offPath("cat"); }
  argmax(_a: TensorData, _axis?: number): TensorData { return this.offPath("argmax"); }
  topk(_a: TensorData, _k: number, _axis?: number): { values: TensorData; indices: TensorData } { return this.offPath("topk"); }
  gather(_a: TensorData, _axis: number, _i: TensorData): TensorData { return this.offPath("gather"); }
}

// Registration, as packages/helios/src/index.ts:29-30 does for "helios"
// (resolved by apps/cli/src/resolve.ts:12-19):
//   import { backendRegistry } from "@alpha/core";
//   backendRegistry.register("cuda", () => new CudaBackend(Number(process.env.ALPHA_CUDA_DEVICE ?? 0)));
