/**
 * Batch sharding over the GPUs of one machine: one backend context per device, contiguous slices
 * of the batch, weights replicated, no exchange between devices, host-side gather of the results
 * into one pinned buffer.  (The path has no collective: inference over a batch is independent per
 * image -- every loop of MathBackendCPU on the path has the batch outermost,
 * tfjs-core/src/backends/cpu/backend_cpu.ts:1578, 1995, 2299.)
 *
 * JavaScript is single-threaded, so the issue order is: for every device enqueue the upload of
 * its slice and the replay of its captured graph (each call only enqueues and returns), then
 * enqueue every device's read of its [B/G, classes] slice straight into its place in the output
 * buffer, then await the reads.  All devices compute concurrently; the host thread never blocks
 * before the awaits.
 *
 * tfjs-core_b200/sharded.py is the Python mirror (one host thread per device instead of the
 * event loop) that the test-suite and the benchmark execute.
 */
import {Tensor, Tensor2D, tensor4d} from '@tensorflow/tfjs-core';

import {BackendCuda} from './backend_cuda';
import * as binding from './binding';

/** Builds the network on one backend and returns its forward function. */
export type ModelFactory = (backend: BackendCuda) => {
  forward: (x: Tensor) => Tensor2D,
  dispose: () => void
};

interface Shard {
  backend: BackendCuda;
  model: {forward: (x: Tensor) => Tensor2D, dispose: () => void};
  rows: number;          // images of this device's slice
  input: Tensor;         // device tensor [rows, ...imageShape]
  output: Tensor2D;      // device tensor [rows, classes], rewritten by every replay
  graph: binding.Handle; // captured forward pass
}

export class ShardedRunner {
  private shards: Shard[] = [];
  private pinnedIn: ArrayBuffer;
  private pinnedOut: ArrayBuffer;
  readonly classes: number;

  /**
   * `backends`: one BackendCuda per device (e.g. the instances behind 'cuda:0' ... 'cuda:7').
   * `batch` must divide evenly over them.  Builds the model on every device, runs one eager pass
   * (which prepares the tensor-core layouts of the weights) and captures the forward pass of
   * every device into a CUDA graph.
   */
  constructor(private backends: BackendCuda[], factory: ModelFactory, readonly batch: number,
              readonly imageShape: [number, number, number]) {
    if (backends.length === 0 || batch % backends.length !== 0) {
      throw new Error(`a batch of ${batch} does not divide evenly over ${backends.length} devices`);
    }
    const rows = batch / backends.length;
    const imageSize = imageShape[0] * imageShape[1] * imageShape[2];
    this.pinnedIn = backends[0].allocPinned(batch * imageSize * 4);
    let classes = 0;
    for (const backend of backends) {
      const model = factory(backend);
      const input = tensor4d(new Float32Array(rows * imageSize), [rows, ...imageShape] as [number, number, number, number]);
      backend.write(input.dataId, new Float32Array(rows * imageSize));   // moves the tensor to this device
      const warm = model.forward(input);
      classes = warm.shape[1];
      warm.dispose();
      backend.graphBegin();
      const output = model.forward(input);
      const graph = backend.graphEnd();
      this.shards.push({backend, model, rows, input, output, graph});
    }
    this.classes = classes;
    this.pinnedOut = backends[0].allocPinned(batch * classes * 4);
  }

  /** Pinned staging buffer for the whole batch: fill it, then call run(). */
  get input(): Float32Array {
    return new Float32Array(this.pinnedIn);
  }

  /** Runs the batch in `input`; resolves to the gathered [batch, classes] result, a view of one
   * pinned buffer that the next run() overwrites. */
  async run(): Promise<Float32Array> {
    const imageSize = this.imageShape[0] * this.imageShape[1] * this.imageShape[2];
    let row = 0;
    for (const s of this.shards) {
      const slice = new Float32Array(this.pinnedIn, row * imageSize * 4, s.rows * imageSize);
      s.backend.writeAsync(s.input.dataId, slice);
      s.backend.graphLaunch(s.graph, [s.input]);
      row += s.rows;
    }
    const reads: Array<Promise<ArrayBufferView>> = [];
    row = 0;
    for (const s of this.shards) {
      const into = new Float32Array(this.pinnedOut, row * this.classes * 4, s.rows * this.classes);
      reads.push(s.backend.readInto(s.output.dataId, into));
      row += s.rows;
    }
    await Promise.all(reads);
    return new Float32Array(this.pinnedOut);
  }

  dispose(): void {
    for (const s of this.shards) {
      s.backend.graphDestroy(s.graph);
      s.input.dispose();
      s.output.dispose();
      s.model.dispose();
    }
    this.shards = [];
    binding.hostFree(this.pinnedIn);
    binding.hostFree(this.pinnedOut);
  }
}

/** One-shot convenience: shard `images` ([batch, h, w, c] values) over `backends`. */
export async function runSharded(backends: BackendCuda[], factory: ModelFactory, images: Float32Array,
                                 batch: number, imageShape: [number, number, number]): Promise<Float32Array> {
  const runner = new ShardedRunner(backends, factory, batch, imageShape);
  try {
    runner.input.set(images);
    return (await runner.run()).slice();
  } finally {
    runner.dispose();
  }
}
