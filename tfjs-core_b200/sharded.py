"""Batch sharding over the GPUs of one machine, inside one process.

One backend context per device (registered with the engine as 'cuda:0' ... 'cuda:N-1': the
registry is keyed by name, tfjs-core/src/engine.ts:132-138, 220-232), contiguous slices of the
batch, weights replicated, no exchange between devices, and a host-side gather: every device
copies its [rows, classes] slice of the result straight into its place in ONE pinned host
buffer.  The path has no collective: inference over a batch is independent per image (every loop
of MathBackendCPU on the path has the batch outermost, backend_cpu.ts:1578, 1995, 2299).

Set-up (model building, one eager pass that prepares the tensor-core layouts of the weights,
CUDA-graph capture) runs on the calling thread, device by device, because the engine is a
single-threaded object exactly as in JavaScript.  A step then runs on one host thread per
device: upload of the device's slice from the pinned input buffer, graph replay, asynchronous
read into the output buffer, wait for that read (run_pipelined streams batches through two
slots so that the upload of the next batch overlaps the kernels of the current one).  Those calls go straight to the C ABI of the
device's own context (ctypes releases the GIL), touch no engine state, and contexts are
independent of each other, so the threads need no lock.

js/sharded.ts is the same runner on the JavaScript side, where the event loop takes the place
of the threads.
"""
import ctypes as C
import threading

import numpy as np

from . import _ffi
from .backend_cuda import BackendCuda, CudaError
from .engine import ENGINE


def device_count():
    """Number of CUDA devices the library can use (0 when there is none)."""
    n = C.c_int()
    if _ffi.load().tfjs_cuda_device_count(C.byref(n)) != 0:
        return 0
    return n.value


def plan_shards(batch, num_devices):
    """[(first row, rows)] per device: contiguous, equal slices."""
    if num_devices < 1 or batch % num_devices != 0:
        raise ValueError(f"a batch of {batch} does not divide evenly over {num_devices} devices")
    rows = batch // num_devices
    return [(d * rows, rows) for d in range(num_devices)]


class _PinnedBuffer:
    """Page-locked host memory viewed as a numpy array."""

    def __init__(self, lib, shape, dtype=np.float32):
        self._lib = lib
        self.nbytes = int(np.prod(shape)) * np.dtype(dtype).itemsize
        self.ptr = C.c_void_p()
        if lib.tfjs_cuda_host_alloc(C.byref(self.ptr), max(self.nbytes, 1)) != 0:
            raise CudaError("pinned host allocation failed")
        raw = (C.c_uint8 * self.nbytes).from_address(self.ptr.value)
        self.array = np.frombuffer(raw, dtype=dtype).reshape(shape)

    def address(self, first_row):
        return C.c_void_p(self.ptr.value + first_row * self.array.strides[0])

    def free(self):
        if self.ptr:
            self.array = None
            self._lib.tfjs_cuda_host_free(self.ptr)
            self.ptr = None


class _Shard:
    def __init__(self, backend, name, first, rows):
        self.backend, self.name, self.first, self.rows = backend, name, first, rows
        self.net = None
        # Two slots, so that the upload of batch k + 1 overlaps the kernels of batch k: each has
        # its own input tensor, captured graph and output tensor (a graph is tied to the buffers
        # it was captured with).
        self.inputs = [None, None]    # device tensors [rows, *image_shape]
        self.outputs = [None, None]   # device tensors [rows, classes], rewritten by every replay
        self.graphs = [None, None]
        self.forward = None           # eager forward of slot 0 (no graph capture)


class ShardedRunner:
    """Runs `forward` of a model over a batch split across devices.

    build(backend) -> model      builds the model (its weights) on one backend;
    forward(model, x) -> (logits, probabilities) or one tensor: the result that is gathered is
                                 the LAST tensor returned, of shape [rows, classes].
    devices: device ordinals, one context each (an ordinal may repeat: two contexts on one
             device behave like two devices, which is how the gather is tested on one GPU).
    backend_factory: how a context is made (tests inject a host-memory fake).
    """

    def __init__(self, build, forward, batch, image_shape, devices=None, math_mode="3xtf32",
                 options=None, backend_factory=None, use_graph=True):
        self._lib = None
        devices = list(range(device_count())) if devices is None else list(devices)
        self.plan = plan_shards(batch, len(devices))
        self.batch, self.image_shape = batch, tuple(image_shape)
        self.shards, self.classes = [], None
        self.pinned_in, self.pinned_out = [], []
        self._errors = []
        make = backend_factory or (lambda dev: BackendCuda(dev, math_mode))
        previous = ENGINE.backendName
        try:
            for k, (dev, (first, rows)) in enumerate(zip(devices, self.plan)):
                name = f"cuda:{dev}" if devices.count(dev) == 1 else f"cuda:{dev}#{k}"
                backend = ENGINE.registry.get(name)
                if backend is None:
                    ENGINE.registerBackend(name, (lambda d=dev: make(d)), 0)
                    if not ENGINE.setBackend(name):
                        raise CudaError(f"backend {name} failed to initialise")
                    backend = ENGINE.registry[name]
                else:
                    ENGINE.setBackend(name)
                    if hasattr(backend, "setMathMode"):
                        backend.setMathMode(math_mode)
                for key, value in (options or {}).items():
                    backend.setOption(key, value)
                shard = _Shard(backend, name, first, rows)
                self.shards.append(shard)
                self._prepare(shard, build, forward, use_graph)
        except Exception:
            self.dispose()
            raise
        finally:
            if previous is not None and previous in ENGINE.registryFactory:
                ENGINE.setBackend(previous)
        self._lib = getattr(self.shards[0].backend, "_lib", None)
        if self._lib is not None:
            self.pinned_in = [_PinnedBuffer(self._lib, (batch,) + self.image_shape) for _ in range(2)]
            self.pinned_out = [_PinnedBuffer(self._lib, (batch, self.classes)) for _ in range(2)]
            self.input = self.pinned_in[0].array
        else:  # a host-memory fake backend: plain arrays
            self.input = np.zeros((batch,) + self.image_shape, np.float32)
            self._out = np.zeros((batch, self.classes), np.float32)

    # ---- set-up, on the calling thread (the engine is single-threaded) ---------------------
    def _prepare(self, shard, build, forward, use_graph):
        from . import ops
        bk = shard.backend
        shard.net = build(bk)

        def run(x):
            out = forward(shard.net, x)
            outs = list(out) if isinstance(out, (tuple, list)) else [out]
            for t in outs[:-1]:
                t.dispose()
            return outs[-1]

        graphs = use_graph and hasattr(bk, "graphBegin")
        for slot in range(2 if graphs else 1):
            shard.inputs[slot] = ops.tensor(np.zeros((shard.rows,) + self.image_shape, np.float32))
        warm = run(shard.inputs[0])       # eager: prepares the weights' tensor-core layouts
        classes = int(np.prod(warm.shape[1:]))
        if self.classes not in (None, classes):
            raise ValueError("the model returns different shapes on different devices")
        self.classes = classes
        if graphs:
            warm.dispose()
            for slot in range(2):
                bk.graphBegin()
                shard.outputs[slot] = run(shard.inputs[slot])
                shard.graphs[slot] = bk.graphEnd()
        else:
            shard.outputs[0] = warm
            shard.forward = lambda: run(shard.inputs[0])

    # ---- the calls of one step, each of which only enqueues ----------------------------------
    def _check(self, shard, rc):
        if rc:
            raise CudaError(f"shard {shard.name}: " + self._lib.tfjs_cuda_last_error(shard.backend._ctx).decode())

    def _upload(self, shard, slot):
        bk, lib = shard.backend, self._lib
        buf = self.pinned_in[slot]
        self._check(shard, lib.tfjs_cuda_tensor_write_async(
            bk._ctx, bk._rec(shard.inputs[slot].dataId)["id"], buf.address(shard.first),
            shard.rows * buf.array.strides[0]))

    def _launch(self, shard, slot):
        bk, lib = shard.backend, self._lib
        self._check(shard, lib.tfjs_cuda_tensor_wait(bk._ctx, bk._rec(shard.inputs[slot].dataId)["id"]))
        self._check(shard, lib.tfjs_cuda_graph_launch(bk._ctx, shard.graphs[slot]))

    def _read(self, shard, slot, out_tensor=None):
        """Enqueues the copy of the shard's result into its rows of the gather buffer."""
        bk, lib = shard.backend, self._lib
        out = out_tensor if out_tensor is not None else shard.outputs[slot]
        ev = C.c_void_p()
        self._check(shard, lib.tfjs_cuda_tensor_read_async(
            bk._ctx, bk._rec(out.dataId)["id"], self.pinned_out[slot].address(shard.first),
            shard.rows * self.classes * 4, C.byref(ev)))
        return ev

    def _wait(self, shard, ev):
        rc = self._lib.tfjs_cuda_event_wait(ev, -1)
        self._lib.tfjs_cuda_event_destroy(ev)
        if rc:
            raise CudaError(f"read of shard {shard.name} failed with status {rc}")

    def _step_on(self, shard):
        bk = shard.backend
        try:
            if self._lib is None:         # fake backend: synchronous host arrays
                bk.write(shard.inputs[0].dataId, self.input[shard.first:shard.first + shard.rows])
                out = shard.forward()
                self._out[shard.first:shard.first + shard.rows] = out.dataSync().reshape(shard.rows, -1)
                out.dispose()
                return
            self._upload(shard, 0)
            if shard.graphs[0] is not None:
                self._launch(shard, 0)
                self._wait(shard, self._read(shard, 0))
            else:                         # eager: a fresh result tensor every step
                out = shard.forward()
                self._wait(shard, self._read(shard, 0, out))
                out.dispose()
        except Exception as err:  # surfaced by run() on the calling thread
            self._errors.append((shard.name, err))

    def _threaded(self):
        # Threads only for graph replays, which touch nothing but their own context.  An eager
        # forward goes through the engine (scopes, tensor registry), which is single-threaded.
        return (self._lib is not None and len(self.shards) > 1 and
                all(s.graphs[0] is not None for s in self.shards))

    def _raise_errors(self):
        if self._errors:
            name, err = self._errors[0]
            raise CudaError(f"shard {name}: {err}") from err

    def run(self, images=None):
        """Runs one batch.  `images` ([batch, *image_shape] float32) is copied into the pinned
        input buffer first; without it the buffer's current contents (self.input) are used.
        Returns the gathered [batch, classes] array, a view of the pinned output buffer that the
        next run() overwrites."""
        if images is not None:
            np.copyto(self.input, np.asarray(images, np.float32).reshape(self.input.shape))
        self._errors = []
        if not self._threaded():
            previous = ENGINE.backendName
            for s in self.shards:
                if s.graphs[0] is None:
                    ENGINE.setBackend(s.name)  # an eager forward may create tensors through the op layer
                self._step_on(s)
            if previous is not None and previous != ENGINE.backendName and previous in ENGINE.registryFactory:
                ENGINE.setBackend(previous)
        else:
            threads = [threading.Thread(target=self._step_on, args=(s,)) for s in self.shards]
            for t in threads:
                t.start()
            for t in threads:
                t.join()
        self._raise_errors()
        return self.pinned_out[0].array if self._lib is not None else self._out

    def run_pipelined(self, num_batches, fill=None, consume=None):
        """Streams `num_batches` batches through the devices with the upload of batch k + 1
        overlapping the kernels of batch k.

        fill(k, buffer): write batch k into `buffer` ([batch, *image_shape], pinned); called on
        the calling thread before the batch is uploaded.  Without it the slots' current contents
        are used (self.input_slots).  consume(k, result): called with the gathered
        [batch, classes] result of batch k (a view that is overwritten two batches later).
        Needs captured graphs (use_graph=True on a real backend)."""
        if self._lib is None or any(g is None for s in self.shards for g in s.graphs):
            raise CudaError("run_pipelined needs captured graphs on every device")
        if num_batches < 1:
            return
        self._errors = []
        n = len(self.shards)
        ready = threading.Barrier(n + 1)   # calling thread + one thread per device
        done = threading.Barrier(n + 1)

        def device_loop(shard):
            try:
                self._upload(shard, 0)
                for k in range(num_batches):
                    ready.wait()                       # batch k + 1 is in its pinned slot
                    if k + 1 < num_batches:
                        self._upload(shard, (k + 1) % 2)   # issued BEFORE the kernels of batch k, so it overlaps them
                    self._launch(shard, k % 2)
                    self._wait(shard, self._read(shard, k % 2))
                    done.wait()
            except Exception as err:
                self._errors.append((shard.name, err))
                ready.abort()
                done.abort()

        if fill is not None:
            fill(0, self.pinned_in[0].array)
        threads = [threading.Thread(target=device_loop, args=(s,)) for s in self.shards]
        for t in threads:
            t.start()
        try:
            for k in range(num_batches):
                if fill is not None and k + 1 < num_batches:
                    # slot (k + 1) % 2 is free: batch k - 1, its last user, has been computed
                    fill(k + 1, self.pinned_in[(k + 1) % 2].array)
                ready.wait()
                done.wait()
                if consume is not None:
                    consume(k, self.pinned_out[k % 2].array)
        except threading.BrokenBarrierError:
            pass
        for t in threads:
            t.join()
        self._raise_errors()

    @property
    def input_slots(self):
        """The two pinned input buffers of run_pipelined (batch k uses slot k % 2)."""
        return [b.array for b in self.pinned_in]

    def dispose(self):
        for s in self.shards:
            bk = s.backend
            for slot in range(2):
                if s.graphs[slot] is not None:
                    bk.graphDestroy(s.graphs[slot])
                    s.graphs[slot] = None
            for t in s.inputs + s.outputs:
                if t is not None and not t.isDisposed:
                    t.dispose()
            if s.net is not None and hasattr(s.net, "dispose"):
                s.net.dispose()
            s.net = None
            s.inputs, s.outputs = [None, None], [None, None]
        self.shards = []
        for buf in list(self.pinned_in) + list(self.pinned_out):
            buf.free()
        self.pinned_in, self.pinned_out = [], []


def run_sharded(build, forward, images, devices=None, **kwargs):
    """One-shot convenience: shard `images` over the devices and return a copy of the result."""
    images = np.asarray(images, np.float32)
    runner = ShardedRunner(build, forward, images.shape[0], images.shape[1:], devices, **kwargs)
    try:
        return runner.run(images).copy()
    finally:
        runner.dispose()
