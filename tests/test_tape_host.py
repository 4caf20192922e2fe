"""The engine's gradient tape (engine.ts:435-498, 739-812; tape.ts) on a numpy stand-in backend:
node recording, pruning to the paths from x to y, accumulation, saved-tensor lifetime, errors."""
import numpy as np
import pytest

import tfjs_core_b200 as tfb
from numpy_backend import NumpyBackend
from tfjs_core_b200 import ops
from tfjs_core_b200.engine import ENGINE, get_filtered_nodes_x_to_y


@pytest.fixture()
def host():
    prev = ENGINE.backendName
    bk = NumpyBackend()
    ENGINE.registerBackend("numpy-test", lambda: bk, 1000)
    assert ENGINE.setBackend("numpy-test")
    yield bk
    ENGINE.removeBackend("numpy-test")
    if prev:
        ENGINE.setBackend(prev)


def test_grad_of_elementwise_chain(host):
    x = ops.tensor(np.array([-2.0, 0.5, 3.0], np.float32))
    # f = relu(x) * x + exp(x): f' = 2x (x > 0) + exp(x)
    g = ops.grad(lambda v: ops.add(ops.mul(ops.relu(v), v), ops.exp(v)))(x)
    xv = np.array([-2.0, 0.5, 3.0])
    np.testing.assert_allclose(g.dataSync(), np.where(xv > 0, 2 * xv, 0) + np.exp(xv), rtol=1e-6)


def test_dy_scales_the_gradient_and_value_is_returned(host):
    x = ops.tensor(np.array([[1.0, 2.0], [3.0, 4.0]], np.float32))
    dy = ops.tensor(np.array([[10.0, 0.0], [0.0, 1.0]], np.float32))
    value, (g,) = ops.value_and_grads(lambda v: ops.square(v))([x], dy)
    np.testing.assert_allclose(value.dataSync(), [1, 4, 9, 16])
    np.testing.assert_allclose(g.dataSync(), [20, 0, 0, 8])
    with pytest.raises(ValueError, match="float32"):
        ENGINE.gradients(lambda: ops.square(x), [x], ops.tensor(np.ones((2, 2)), None, "int32"))


def test_broadcast_gradients_reduce_to_the_operand_shape(host):
    a = ops.tensor(np.ones((2, 3, 4), np.float32))
    b = ops.tensor(np.array([1.0, 2.0, 3.0, 4.0], np.float32))       # [4] broadcast over [2,3,4]
    c = ops.tensor(np.full((3, 1), 2.0, np.float32))                  # [3,1]
    ga, gb, gc = ops.grads(lambda p, q, r: ops.mul(ops.add(p, q), r))([a, b, c])
    assert ga.shape == [2, 3, 4] and gb.shape == [4] and gc.shape == [3, 1]
    np.testing.assert_allclose(ga.dataSync(), np.full(24, 2.0))
    np.testing.assert_allclose(gb.dataSync(), np.full(4, 12.0))       # 2 * 3 positions, times c = 2
    np.testing.assert_allclose(gc.dataSync().reshape(3), [(2 + 3 + 4 + 5) * 2] * 3)


def test_matmul_and_sum_over_outer_axes(host):
    rng = np.random.default_rng(0)
    a = rng.normal(size=(3, 4)).astype(np.float32)
    b = rng.normal(size=(4, 2)).astype(np.float32)
    ga, gb = ops.grads(lambda p, q: ops.sum(ops.matmul(p, q), 0))([ops.tensor(a), ops.tensor(b)])
    np.testing.assert_allclose(ga.dataSync().reshape(3, 4), np.ones((3, 2)) @ b.T, rtol=1e-5)
    np.testing.assert_allclose(gb.dataSync().reshape(4, 2), a.T @ np.ones((3, 2)), rtol=1e-5)


def test_a_tensor_used_twice_accumulates_and_unrelated_ops_are_pruned(host):
    x = ops.tensor(np.array([1.0, 2.0], np.float32))
    other = ops.tensor(np.array([5.0, 5.0], np.float32))

    def f(v):
        ops.exp(other)                      # recorded, but not on a path from v to the result
        return ops.add(ops.mul(v, v), v)    # v used three times
    g = ops.grad(f)(x)
    np.testing.assert_allclose(g.dataSync(), [3.0, 5.0])
    # tape.ts getFilteredNodesXToY on a hand-made tape
    t = [ops.tensor(np.zeros(1, np.float32)) for _ in range(5)]
    tape = [{"id": 0, "name": "n0", "inputs": {"a": t[0]}, "outputs": [t[1]], "saved": [], "gradient": None},
            {"id": 1, "name": "n1", "inputs": {"a": t[4]}, "outputs": [t[3]], "saved": [], "gradient": None},
            {"id": 2, "name": "n2", "inputs": {"a": t[1], "b": t[4]}, "outputs": [t[2]], "saved": [], "gradient": None}]
    filtered = get_filtered_nodes_x_to_y(tape, [t[0]], t[2])
    assert [n["name"] for n in filtered] == ["n0", "n2"] and list(filtered[1]["inputs"]) == ["a"]


def test_y_not_reachable_from_x_raises(host):
    x = ops.tensor(np.array([1.0], np.float32))
    y = ops.tensor(np.array([2.0], np.float32))
    with pytest.raises(ValueError, match="Cannot compute gradient"):
        ops.grad(lambda v: ops.exp(y))(x)


def test_saved_tensors_do_not_leak(host):
    x = ops.tensor(np.array([[0.5, -1.0], [2.0, 3.0]], np.float32))
    w = ops.tensor(np.array([[1.0, 2.0], [3.0, 4.0]], np.float32))
    before, buffers_before = ENGINE.numTensors, len(host.data)

    def f(p, q):
        return ENGINE.tidy(lambda: ops.sum(ops.relu(ops.fused_matmul(p, q, activation="relu"))))
    for _ in range(3):
        value, grads = ops.value_and_grads(f)([x, w])
        value.dispose()
        for g in grads:
            g.dispose()
    assert ENGINE.numTensors == before
    assert len(host.data) == buffers_before


def test_kernels_without_a_gradient_cannot_be_backpropagated(host):
    x = ops.tensor(np.array([1.0, 4.0], np.float32))
    # max has no gradient on this path: the tape has no node for it, so y is unreachable
    with pytest.raises((ValueError, AttributeError)):
        ops.grad(lambda v: ops.max(v))(x)


def test_grad_does_not_leak_without_a_caller_side_tidy(host):
    """tf.grad wraps the forward pass in its own scope (engine.ts:737, gradients.ts:68-80): the value
    of f and every intermediate are disposed, only the gradient survives."""
    x = ops.tensor(np.array([1.0, -2.0, 3.0], np.float32))
    before = ENGINE.numTensors
    g = ops.grad(lambda v: ops.mul(ops.relu(v), ops.exp(v)))(x)
    assert ENGINE.numTensors == before + 1
    g.dispose()
    z = ops.tensor(np.array([2.0, 2.0, 2.0], np.float32))
    gs = ops.grads(lambda p, q: ops.mul(ops.add(p, q), p))([x, z])
    assert ENGINE.numTensors == before + 3
    for t in gs + [z]:
        t.dispose()
    assert ENGINE.numTensors == before and ENGINE.activeTape is None


def test_second_derivative_through_a_nested_tape(host):
    """grad(grad(f)): the inner call records onto the outer call's tape (engine.ts:660-665), so the
    outer call differentiates through the inner backward pass.  f = x^3: f'' = 6x."""
    x = ops.tensor(np.array([0.5, -1.0, 2.0], np.float32))
    cube = lambda v: ops.mul(ops.mul(v, v), v)  # noqa: E731
    before = ENGINE.numTensors
    first = ops.grad(cube)(x)
    np.testing.assert_allclose(first.dataSync(), 3 * np.array([0.5, -1.0, 2.0]) ** 2, rtol=1e-6)
    second = ops.grad(lambda v: ops.grad(cube)(v))(x)
    np.testing.assert_allclose(second.dataSync(), 6 * np.array([0.5, -1.0, 2.0]), rtol=1e-6)
    first.dispose()
    second.dispose()
    assert ENGINE.numTensors == before and ENGINE.activeTape is None and ENGINE.gradientDepth == 0
