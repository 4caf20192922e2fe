"""A small host-side stand-in for the parts of tfjs-core's Engine that call the backend.

The real engine (tfjs-core/src/engine.ts) is TypeScript and runs unchanged on top of a
KernelBackend; it cannot run here (no JavaScript toolchain), so this module replays its
calling sequence against the same backend interface: backend registry with priorities and
fallback on failed initialisation (engine.ts:220-359), tensor registry with per-dataId
reference counts (engine.ts:502-572), tidy scopes (engine.ts:365-399, 675-718) and the
runKernel dispatcher (engine.ts:435-498), the gradient tape (engine.ts:660-669, 726-774;
tape.ts) including nested tapes for higher-order gradients.
"""
import warnings

import numpy as np

NP_DTYPE = {"float32": np.float32, "int32": np.int32, "bool": np.uint8}


class DataId:
    """Opaque storage key; plays the role of the `dataId` object (tensor.ts:408-416)."""
    __slots__ = ("__weakref__",)


def size_from_shape(shape):
    n = 1
    for s in shape:
        n *= int(s)
    return n


class Tensor:
    """tensor.ts:419-484: a shape, a dtype and a dataId registered with the engine."""

    def __init__(self, shape, dtype, values=None, data_id=None, backend=None):
        self.shape = [int(s) for s in shape]
        self.dtype = dtype
        self.size = size_from_shape(self.shape)
        self.dataId = data_id if data_id is not None else DataId()
        self.isDisposed = False
        self.kept = False
        Tensor._next_id += 1
        self.id = Tensor._next_id   # tensor.ts:421: unique per Tensor object, the tape's key
        ENGINE.registerTensor(self, backend)
        if values is not None:
            ENGINE.write(backend, self.dataId, values)

    _next_id = 0

    def clone(self):
        """A second Tensor over the same storage (shares the dataId).  While a tape records, the
        clone is a node of it (identity, gradient dy), so that gradients flow through clones."""
        self._throw_if_disposed()
        return ENGINE.runKernel(lambda backend: Tensor(self.shape, self.dtype, None, self.dataId), "clone",
                                {"x": self}, lambda dy, saved: {"x": lambda: dy.clone()})

    @staticmethod
    def make(shape, data=None, dtype="float32", backend=None):
        """Tensor.make (tensor.ts:474-484): data is {} for a backend-created output,
        {'dataId': id} for an alias, {'values': array} for host data."""
        data = data or {}
        return Tensor(shape, dtype, data.get("values"), data.get("dataId"), backend)

    @property
    def rank(self):
        return len(self.shape)

    def dataSync(self):
        self._throw_if_disposed()
        return ENGINE.readSync(self.dataId)

    def data(self):
        """Asynchronous read: returns a handle whose .result() blocks (tensor.ts:616-630)."""
        self._throw_if_disposed()
        return ENGINE.read(self.dataId)

    def dispose(self):
        if self.isDisposed:
            return
        ENGINE.disposeTensor(self)
        self.isDisposed = True

    def _throw_if_disposed(self):
        if self.isDisposed:
            raise RuntimeError("Tensor is disposed.")

    def reshape(self, shape):
        from . import ops
        return ops.reshape(self, shape)


class Engine:
    def __init__(self):
        self.reset()

    def reset(self):
        for b in getattr(self, "registry", {}).values():
            b.dispose()
        self.registryFactory = {}   # name -> (factory, priority)
        self.registry = {}          # name -> initialised backend
        self.backendName = None
        self.backendInstance = None
        self.tensorInfo = {}        # DataId -> {backend, refCount, shape, dtype, bytes}
        self.numTensors = 0
        self.numBytes = 0
        self.numDataBuffers = 0
        self.scopeStack = []
        self.kernelDepth = 0
        self.kernelNames = []       # runKernel trace (profile-like): one entry per backend call
        self.activeTape = None      # list of tape nodes while a gradient scope records
        self.gradientDepth = 0
        self.nextTapeNodeId = 0

    # ---- backend registry (engine.ts:220-359) ----
    def registerBackend(self, name, factory, priority=1):
        if name in self.registryFactory:
            warnings.warn(f"{name} backend was already registered. Reusing existing backend factory.")
            return False
        self.registryFactory[name] = (factory, priority)
        return True

    def findBackend(self, name):
        if name not in self.registry:
            if name in self.registryFactory:
                return self.registry[name] if self.initializeBackend(name) else None
            return None
        return self.registry[name]

    def initializeBackend(self, name):
        if name not in self.registryFactory:
            raise ValueError(f"Cannot initialize backend {name}, no registration found.")
        factory, _ = self.registryFactory[name]
        try:
            self.registry[name] = factory()
            return True
        except Exception as err:  # engine.ts:302-306: warn and let the caller fall back
            warnings.warn(f"Initialization of backend {name} failed: {err}")
            return False

    def setBackend(self, name):
        if name not in self.registryFactory:
            raise ValueError(f"Backend name '{name}' not found in registry")
        self.backendName = name
        if name not in self.registry:
            self.backendInstance = None
            if not self.initializeBackend(name):
                return False
        self.backendInstance = self.registry[name]
        return True

    def initializeBackendsAndReturnBest(self):
        """engine.ts:334-359: try factories by descending priority."""
        if not self.registryFactory:
            raise RuntimeError("No backend found in registry.")
        for name in sorted(self.registryFactory, key=lambda n: -self.registryFactory[n][1]):
            if self.initializeBackend(name):
                return name, self.registry[name]
        raise RuntimeError("Could not initialize any backends, all backend initializations failed.")

    @property
    def backend(self):
        if self.backendInstance is None:
            name, inst = self.initializeBackendsAndReturnBest()
            self.backendName, self.backendInstance = name, inst
        return self.backendInstance

    def removeBackend(self, name):
        self.registryFactory.pop(name, None)
        b = self.registry.pop(name, None)
        if b is not None:
            b.dispose()
            if self.backendInstance is b:
                self.backendInstance = None
                self.backendName = None

    # ---- tensor registry (engine.ts:502-572) ----
    def registerTensor(self, t, backend=None):
        info = self.tensorInfo.get(t.dataId)
        self.numTensors += 1
        if info is None:
            b = backend or self.backend
            nbytes = t.size * (1 if t.dtype == "bool" else 4)
            self.tensorInfo[t.dataId] = {"backend": b, "refCount": 0, "shape": t.shape,
                                         "dtype": t.dtype, "bytes": nbytes}
            self.numBytes += nbytes
            self.numDataBuffers += 1
            b.register(t.dataId, t.shape, t.dtype)
            info = self.tensorInfo[t.dataId]
        info["refCount"] += 1
        if self.scopeStack:
            self.scopeStack[-1]["track"].append(t)

    def disposeTensor(self, t):
        info = self.tensorInfo.get(t.dataId)
        if info is None:
            return
        self.numTensors -= 1
        if info["refCount"] <= 1:
            self.numBytes -= info["bytes"]
            self.numDataBuffers -= 1
            info["backend"].disposeData(t.dataId)
            del self.tensorInfo[t.dataId]
        else:
            info["refCount"] -= 1

    def write(self, backend, data_id, values):
        info = self.tensorInfo[data_id]
        dest = backend or self.backend
        if dest is not info["backend"]:
            # engine.ts:843-851: the tensor migrates to the destination backend
            info["backend"].disposeData(data_id)
            info["backend"] = dest
            dest.register(data_id, info["shape"], info["dtype"])
        dest.write(data_id, values)

    def readSync(self, data_id):
        return self.tensorInfo[data_id]["backend"].readSync(data_id)

    def read(self, data_id):
        return self.tensorInfo[data_id]["backend"].read(data_id)

    def moveData(self, dest_backend, data_id):
        """engine.ts:361-363: host-staged copy between backends (DataStorage miss)."""
        self.write(dest_backend, data_id, self.readSync(data_id))

    # ---- scopes (engine.ts:365-399, 675-718) ----
    def startScope(self, name=None):
        self.scopeStack.append({"track": [], "name": name})

    def endScope(self, result=None):
        keep = set()
        for t in _tensors_in(result):
            keep.add(id(t))
        scope = self.scopeStack.pop()
        for t in scope["track"]:
            if id(t) in keep or t.isDisposed or t.kept:
                continue
            t.dispose()
        if self.scopeStack:
            for t in _tensors_in(result):
                self.scopeStack[-1]["track"].append(t)

    def tidy(self, fn):
        self.startScope()
        result = None
        try:
            result = fn()
            return result
        finally:
            self.endScope(result)

    # ---- kernel dispatch (engine.ts:435-498) ----
    def runKernel(self, forward, name=None, inputs=None, backward=None):
        """engine.ts:435-498.  `forward(backend)` or `forward(backend, save)` computes the result;
        `inputs` is {name: Tensor}; `backward(dy, saved)` returns {name: () -> Tensor}, the gradient
        with respect to each input.  While a tape records (engine.gradients), a node with the
        inputs, the output and the gradient function is appended to it; `save(tensors)` keeps
        clones of the tensors the gradient needs, so the caller may dispose its own handles."""
        # engine.ts:427-429 isTapeOn: only kernels called directly from user code are recorded,
        # not the kernels a kernel calls, and only while some gradients() scope is open
        tape_on = self.gradientDepth > 0 and self.kernelDepth == 0
        self.kernelDepth += 1
        saved = []

        def save(tensors):
            # not saved unless recording: nothing would ever dispose the kept clones
            if tape_on:
                for t in tensors:
                    saved.append(self.keep(self._clone_on_tape(t)))
        try:
            if name:
                self.kernelNames.append(name)
            try:
                takes_save = forward.__code__.co_argcount >= 2
            except AttributeError:
                takes_save = False
            result = forward(self.backend, save) if takes_save else forward(self.backend)
        finally:
            self.kernelDepth -= 1
        if tape_on and inputs and backward is not None:
            self.nextTapeNodeId += 1
            self.activeTape.append({"id": self.nextTapeNodeId, "name": name, "inputs": dict(inputs),
                                    "outputs": [result], "saved": saved,
                                    "gradient": (lambda dy, _s=saved: backward(dy, _s))})
        return result

    def _clone_on_tape(self, x):
        """engine.ts:401-409 clone(): an alias of x recorded on the tape as an identity node.  The
        saved tensors of a kernel are such clones; the node keeps them connected to x, which is
        what lets an outer gradients() differentiate through an inner backward pass."""
        y = Tensor(x.shape, x.dtype, None, x.dataId)
        self.nextTapeNodeId += 1
        self.activeTape.append({"id": self.nextTapeNodeId, "name": "clone", "inputs": {"x": x}, "outputs": [y],
                                "saved": [], "gradient": (lambda dy: {"x": lambda: dy.clone()})})
        return y

    def keep(self, t):
        """tf.keep (engine.ts:720-731): the tensor survives the enclosing tidy scopes."""
        t.kept = True
        return t

    # ---- gradients (engine.ts:739-812, tape.ts) ----
    def gradients(self, f, xs, dy=None):
        """Returns (value, grads): value = f(), grads[i] = d sum(value * dy) / d xs[i].  f must
        return one float32 Tensor computed from xs through ops that define gradients."""
        from . import ops
        assert xs, "gradients() received an empty list of xs."
        if dy is not None and dy.dtype != "float32":
            raise ValueError(f"dy must have 'float32' dtype, but has '{dy.dtype}'")
        # engine.ts:660-669 startTape / endTape: a fresh tape only for the outermost gradients();
        # a nested call records onto the same tape, so that the outer call can differentiate
        # through the inner call's backward pass (higher-order gradients)
        if self.gradientDepth == 0:
            self.activeTape = []
        self.gradientDepth += 1
        try:
            y = self.tidy(f)   # engine.ts:737: the forward pass runs in its own scope
        finally:
            self.gradientDepth -= 1
        if not isinstance(y, Tensor):
            if self.gradientDepth == 0:
                self._dispose_tape(self.activeTape)
                self.activeTape = None
            raise ValueError("The result y returned by f() must be a tensor.")
        tape = self.activeTape
        filtered = get_filtered_nodes_x_to_y(tape, xs, y)
        if not filtered and xs:
            if self.gradientDepth == 0:
                self._dispose_tape(tape)
                self.activeTape = None
            raise ValueError("Cannot compute gradient of y=f(x) with respect to x. Make sure that the f "
                             "you passed encloses all operations that lead from x to y.")
        # Back-propagation runs in its own scope: every temporary it creates (clones, masks,
        # partial sums, the gradients of intermediates) is disposed when the scope ends, only the
        # gradients of xs survive (engine.ts:751-773 wraps this in tidy).  With an outer
        # gradients() still open (gradientDepth > 0) these kernels are recorded too.
        self.startScope("backward")
        grads = None
        try:
            acc = {y.id: dy if dy is not None else ops.tensor(np.ones(y.shape, np.float32), y.shape)}
            backpropagate_gradients(acc, filtered)
            grads = []
            for x in xs:
                g = acc.get(x.id)
                if g is None:
                    g = ops.tensor(np.zeros(x.shape, np.float32), x.shape)
                elif g is dy:
                    g = dy.clone()   # x is y itself: hand back a tensor the caller may dispose
                grads.append(g)
        finally:
            self.endScope(grads)
            if self.gradientDepth == 0:
                # not computing higher-order gradients: the tape can go (engine.ts:762-771)
                self._dispose_tape(tape)
                self.activeTape = None
        return y, grads

    @staticmethod
    def _dispose_tape(tape):
        for node in tape:
            for t in node["saved"]:
                if not t.isDisposed:
                    t.kept = False
                    t.dispose()
            node["saved"] = []

    def memory(self):
        info = dict(self.backend.memory())
        info.update(numTensors=self.numTensors, numDataBuffers=self.numDataBuffers,
                    numBytes=self.numBytes)
        return info

    def time(self, fn):
        return self.backend.time(fn)


def get_filtered_nodes_x_to_y(tape, xs, y):
    """tape.ts:38-125: the nodes on a path from any x to y, each with only the inputs that lie
    on such a path."""
    from_x = {x.id for x in xs}
    nodes_from_x = set()
    for i, node in enumerate(tape):
        if any(t.id in from_x for t in node["inputs"].values()):
            for out in node["outputs"]:
                from_x.add(out.id)
            nodes_from_x.add(i)
    to_y = {y.id}
    nodes_to_y = set()
    for i in range(len(tape) - 1, -1, -1):
        node = tape[i]
        if any(out.id in to_y for out in node["outputs"]):
            for t in node["inputs"].values():
                to_y.add(t.id)
            nodes_to_y.add(i)
    filtered = []
    for i, node in enumerate(tape):
        if i in nodes_from_x and i in nodes_to_y:
            pruned = {k: t for k, t in node["inputs"].items() if t.id in from_x}
            filtered.append(dict(node, inputs=pruned))
    return filtered


def backpropagate_gradients(acc, filtered_tape):
    """tape.ts:134-190: walks the tape backwards; `acc` maps tensor id -> accumulated gradient."""
    from . import ops
    for node in reversed(filtered_tape):
        out = node["outputs"][0]
        dy = acc.get(out.id)
        if dy is None:
            continue   # this output does not influence y
        input_gradients = node["gradient"](dy)
        for name, x in node["inputs"].items():
            if name not in input_gradients:
                raise ValueError(f"Cannot backprop through input {name}. Available gradients found: "
                                 f"{list(input_gradients)}.")
            dx = input_gradients[name]()
            if dx.dtype != "float32":
                raise ValueError(f"Error in gradient for op {node['name']}. The gradient of input "
                                 f"{name} must have 'float32' dtype, but has '{dx.dtype}'")
            if dx.shape != x.shape:
                raise ValueError(f"Error in gradient for op {node['name']}. The gradient of input "
                                 f"'{name}' has shape '{dx.shape}', which does not match the shape of "
                                 f"the input '{x.shape}'")
            cur = acc.get(x.id)
            if cur is None:
                acc[x.id] = dx
            else:
                acc[x.id] = ops.add(cur, dx)
                cur.dispose()
                dx.dispose()


def _tensors_in(result):
    if result is None:
        return []
    if isinstance(result, Tensor):
        return [result]
    if isinstance(result, (list, tuple)):
        out = []
        for r in result:
            out.extend(_tensors_in(r))
        return out
    if isinstance(result, dict):
        out = []
        for r in result.values():
            out.extend(_tensors_in(r))
        return out
    return []


ENGINE = Engine()
