"""The in-process sharded runner on real contexts: a batch split over several backend contexts
(several devices where the machine has them, several contexts of one device otherwise) must give
the gathered result of the single-context forward, bit for bit, on repeated runs."""
import numpy as np
import pytest

from gpu_util import tf  # noqa: F401

pytestmark = pytest.mark.gpu


def _build_and_forward(params):
    from tfjs_core_b200 import mobilenet

    def build(backend):
        return mobilenet.MobileNetV1(params, backend)

    def forward(net, x):
        return net.forward_separable(x)
    return build, forward


@pytest.mark.parametrize("math_mode", ["tf32", "3xtf32"])
def test_sharded_equals_single_context(tf, math_mode):
    from tfjs_core_b200 import ShardedRunner, device_count, mobilenet
    n_dev = device_count()
    assert n_dev >= 1
    contexts = 4
    devices = [k % n_dev for k in range(contexts)]
    params = mobilenet.make_weights(3, gain=1.5)
    build, forward = _build_and_forward(params)
    batch = 8
    x = mobilenet.make_input(7, batch)
    single = ShardedRunner(build, forward, batch, x.shape[1:], devices=[0], math_mode=math_mode)
    try:
        want = single.run(x).copy()
    finally:
        single.dispose()
    runner = ShardedRunner(build, forward, batch, x.shape[1:], devices=devices, math_mode=math_mode)
    try:
        assert [s.rows for s in runner.shards] == [2, 2, 2, 2]
        got = runner.run(x).copy()
        assert np.array_equal(got, want)
        assert np.allclose(got.sum(1), 1.0, atol=1e-5)
        # a second, different batch through the same graphs and buffers
        x2 = mobilenet.make_input(8, batch)
        got2 = runner.run(x2).copy()
        assert not np.array_equal(got2, got)
        # and back: the gathered result depends on the input only
        assert np.array_equal(runner.run(x), want)
    finally:
        runner.dispose()
    assert tf.set_backend("cuda")


def test_sharded_result_matches_the_oracle(tf):
    from oracle import mobilenet as oracle_net
    from tfjs_core_b200 import device_count, mobilenet, run_sharded
    params = mobilenet.make_weights(3, gain=1.5)
    build, forward = _build_and_forward(params)
    x = mobilenet.make_input(9, 4)
    n_dev = device_count()
    got = run_sharded(build, forward, x, devices=[k % n_dev for k in range(2)])
    _, want = oracle_net.forward(x, params)
    assert np.abs(got - want).max() <= 1e-5
    assert (got.argmax(1) == want.argmax(1)).all()
    assert tf.set_backend("cuda")


def test_pipelined_stream_equals_batch_by_batch(tf):
    """run_pipelined: five different batches through two slots per device (upload of the next batch
    overlapping the kernels of the current one) give, batch for batch, what run() gives."""
    from tfjs_core_b200 import ShardedRunner, device_count, mobilenet
    n_dev = device_count()
    params = mobilenet.make_weights(3, gain=1.5)
    build, forward = _build_and_forward(params)
    batch, steps = 4, 5
    batches = [mobilenet.make_input(20 + k, batch) for k in range(steps)]
    runner = ShardedRunner(build, forward, batch, batches[0].shape[1:], devices=[k % n_dev for k in range(2)],
                           math_mode="tf32")
    try:
        want = [runner.run(b).copy() for b in batches]
        got = {}
        runner.run_pipelined(steps, fill=lambda k, buf: np.copyto(buf, batches[k]),
                             consume=lambda k, res: got.__setitem__(k, res.copy()))
        assert sorted(got) == list(range(steps))
        for k in range(steps):
            assert np.array_equal(got[k], want[k]), k
    finally:
        runner.dispose()
    assert tf.set_backend("cuda")
