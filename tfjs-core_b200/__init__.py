"""B200-native `cuda` kernel backend for tfjs-core's MobileNet inference path.

Importing the package registers the backend under the name 'cuda' the way an out-of-tree
tfjs backend does (tf.registerBackend(name, factory, priority), tfjs-core/src/globals.ts:
325-329; precedent tfjs-backend-wasm/src/backend_wasm.ts:154-157).  The factory creates the
device context lazily, so importing works on a machine without a GPU; using the backend
there fails loudly (there is no CPU fallback inside it).
"""
from . import _ffi, conv_util, ops, weights_loader  # noqa: F401
from .backend_cuda import BackendCuda, CudaError  # noqa: F401
from .engine import ENGINE, Tensor  # noqa: F401
from .sharded import ShardedRunner, device_count, run_sharded  # noqa: F401


def register_backend(name="cuda", device=0, priority=3, math_mode="3xtf32"):
    """tf.registerBackend('cuda', () => new BackendCuda(device), priority)."""
    return ENGINE.registerBackend(name, lambda: BackendCuda(device, math_mode), priority)


def set_backend(name="cuda"):
    return ENGINE.setBackend(name)


register_backend()
