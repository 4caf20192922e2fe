"""The in-process batch sharder on host memory: the plan, the slicing of the input buffer and the
gather of the per-device results, with a fake backend standing in for the devices."""
import numpy as np
import pytest

from numpy_backend import NumpyBackend
from tfjs_core_b200 import ENGINE, ops
from tfjs_core_b200.sharded import ShardedRunner, plan_shards


def test_plan_is_contiguous_and_even():
    assert plan_shards(1024, 8) == [(i * 128, 128) for i in range(8)]
    assert plan_shards(6, 1) == [(0, 6)]
    with pytest.raises(ValueError, match="does not divide evenly"):
        plan_shards(10, 4)
    with pytest.raises(ValueError):
        plan_shards(8, 0)


class _Model:
    """y = relu(x_flat * w + device_tag): the tag shows which context produced a row."""

    def __init__(self, backend, tag):
        self.backend, self.tag = backend, tag
        self.w = ops.tensor(np.arange(1, 13, dtype=np.float32).reshape(1, 12, 1).repeat(3, axis=2))

    def dispose(self):
        self.w.dispose()


def test_slices_and_gather_with_a_fake_backend():
    ENGINE.reset()
    made = []

    def factory(dev):
        b = NumpyBackend()
        b.tag = float(len(made))
        made.append(b)
        return b

    def build(backend):
        return _Model(backend, backend.tag)

    def forward(model, x):
        bk = model.backend
        rows = x.shape[0]
        flat = bk.reshape(x, [1, rows, 12])
        y = bk.fusedBatchMatMul(flat, model.w)                 # [1, rows, 3]
        tag = ops.tensor(np.full((1, 1, 3), model.tag, np.float32))
        out = bk.add(y, tag)
        y.dispose()
        tag.dispose()
        return bk.reshape(out, [rows, 3])

    batch = 8
    runner = ShardedRunner(build, forward, batch, (2, 2, 3), devices=[0, 1, 2, 3], backend_factory=factory,
                           use_graph=False)
    try:
        assert len(made) == 4 and runner.classes == 3
        assert [(s.first, s.rows) for s in runner.shards] == [(0, 2), (2, 2), (4, 2), (6, 2)]
        rng = np.random.Generator(np.random.PCG64(5))
        x = rng.uniform(-1, 1, (batch, 2, 2, 3)).astype(np.float32)
        got = runner.run(x)
        w = np.arange(1, 13, dtype=np.float32)
        want = (x.reshape(batch, 12) @ w)[:, None].repeat(3, axis=1) + (np.arange(batch) // 2)[:, None]
        np.testing.assert_allclose(got, want, rtol=1e-6, atol=1e-5)
        # a second batch reuses the buffers and overwrites the gathered result
        x2 = rng.uniform(-1, 1, (batch, 2, 2, 3)).astype(np.float32)
        got2 = runner.run(x2)
        want2 = (x2.reshape(batch, 12) @ w)[:, None].repeat(3, axis=1) + (np.arange(batch) // 2)[:, None]
        np.testing.assert_allclose(got2, want2, rtol=1e-6, atol=1e-5)
    finally:
        runner.dispose()
        ENGINE.reset()
        import tfjs_core_b200
        tfjs_core_b200.register_backend()


def test_uneven_batch_is_refused_before_any_device_is_touched():
    with pytest.raises(ValueError, match="does not divide evenly"):
        ShardedRunner(lambda b: None, lambda m, x: None, 10, (1, 1, 1), devices=[0, 1, 2],
                      backend_factory=lambda d: (_ for _ in ()).throw(AssertionError("must not be created")))
