/**
 * Registers the B200 backend with tfjs-core's engine.
 *
 *   import '@tensorflow/tfjs-core';
 *   import 'tfjs-backend-cuda';            // this file
 *   await tf.setBackend('cuda');           // or leave it to the priority order
 *
 * Registration follows the out-of-tree precedents tfjs-backend-wasm/src/backend_wasm.ts:154-157
 * and tfjs-webgpu/src/index.ts:23-29: `tf.registerBackend(name, factory, priority)`
 * (tfjs-core/src/globals.ts:325-329, engine.ts:220-232).  A factory that throws (no usable
 * device, library missing) makes the engine warn and fall back to the next backend by priority
 * (engine.ts:302-306); the addon has no CPU path of its own.
 *
 * One backend per device: 'cuda' is device CUDA_DEVICE (default 0) and 'cuda:k' is device k, for
 * every device the driver reports.  The registry is keyed by name (engine.ts:132-138), so the
 * instances coexist and tensors move between them through host memory (DataStorage.get miss ->
 * engine.moveData, backends/backend.ts:52-57).  `runSharded` below uses them to spread a batch.
 */
import {ENV, registerBackend} from '@tensorflow/tfjs-core';

import {BackendCuda, registerCudaFlags} from './backend_cuda';
import * as binding from './binding';

export {BackendCuda, CudaActivation} from './backend_cuda';
export {runSharded, ShardedRunner} from './sharded';

/** Above 'cpu' (1) and 'webgl' (2). */
const CUDA_PRIORITY = 3;

registerCudaFlags();

function configured(device: number): BackendCuda {
  const b = new BackendCuda(device, ENV.get('CUDA_MATH_MODE') as '3xtf32' | 'tf32');
  b.setOption('fuse_separable', ENV.getNumber('CUDA_FUSE_SEPARABLE'));
  b.setOption('dequant_in_gemm', ENV.getBool('CUDA_DEQUANT_IN_GEMM') ? 1 : 0);
  return b;
}

registerBackend('cuda', () => configured(ENV.getNumber('CUDA_DEVICE')), CUDA_PRIORITY);

/** Number of CUDA devices the addon sees (0 when there is none). */
export function deviceCount(): number {
  const r = binding.deviceCount();
  return r.status === 0 ? r.out : 0;
}

// 'cuda:k' never wins the priority order by itself: it is selected by name.
for (let k = 0; k < deviceCount(); k++) {
  registerBackend(`cuda:${k}`, () => configured(k), 0);
}
