"""A minimal host-memory KernelBackend in numpy, for testing the engine (tape, scopes, registry)
without a GPU.  Test infrastructure only: float32 tensors, the handful of methods the tape tests
reach.  It is not a fallback of the cuda backend and nothing in the package imports it."""
import numpy as np

from tfjs_core_b200.engine import Tensor


class NumpyBackend:
    def __init__(self):
        self.data = {}

    # ---- storage ----
    def register(self, data_id, shape, dtype):
        self.data[data_id] = None

    def write(self, data_id, values):
        self.data[data_id] = np.array(values, copy=True).reshape(-1)

    def readSync(self, data_id):
        return self.data[data_id]

    def disposeData(self, data_id):
        self.data.pop(data_id, None)

    def memory(self):
        return {"unreliable": True}

    def dispose(self):
        self.data.clear()

    # ---- helpers ----
    def _v(self, t):
        return self.data[t.dataId].reshape(t.shape).astype(np.float32)

    def _make(self, arr):
        arr = np.asarray(arr, np.float32)
        return Tensor(list(arr.shape), "float32", arr, None, self)

    # ---- kernels ----
    def add(self, a, b):
        return self._make(self._v(a) + self._v(b))

    def subtract(self, a, b):
        return self._make(self._v(a) - self._v(b))

    def multiply(self, a, b):
        return self._make(self._v(a) * self._v(b))

    def realDivide(self, a, b):
        return self._make(self._v(a) / self._v(b))

    def relu(self, x):
        return self._make(np.maximum(self._v(x), 0))

    def step(self, x, alpha=0.0):
        v = self._v(x)
        return self._make(np.where(np.isnan(v), v, np.where(v > 0, 1.0, alpha)))

    def exp(self, x):
        return self._make(np.exp(self._v(x).astype(np.float64)))

    def log(self, x):
        return self._make(np.log(self._v(x).astype(np.float64)))

    def sum(self, x, axes):
        return self._make(self._v(x).sum(tuple(axes)))

    def transpose(self, x, perm):
        return self._make(self._v(x).transpose(perm))

    def reshape(self, x, shape):
        return Tensor(list(shape), x.dtype, None, x.dataId)

    def cast(self, x, dtype):
        return Tensor(list(x.shape), dtype, None, x.dataId)

    def fusedBatchMatMul(self, a, b, transposeA=False, transposeB=False, bias=None, activation=None,
                         preluActivationWeights=None):
        av, bv = self._v(a).astype(np.float64), self._v(b).astype(np.float64)
        if transposeA:
            av = av.transpose(0, 2, 1)
        if transposeB:
            bv = bv.transpose(0, 2, 1)
        y = av @ bv
        if bias is not None:
            y = y + self._v(bias)
        if activation == "relu":
            y = np.maximum(y, 0)
        return self._make(y)
