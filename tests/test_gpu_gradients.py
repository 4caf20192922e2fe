"""The engine's gradient tape on the cuda backend: tf.grad / tf.grads / tf.valueAndGrads over the
ops of the MobileNet path, against the reference's own gradient spec values (transcribed with
their line numbers) and against a hand-written chain rule over the oracle's gradient kernels.
"""
import numpy as np
import pytest

import oracle
from gpu_util import rel_err, tf  # noqa: F401

pytestmark = pytest.mark.gpu


def _rng(seed):
    return np.random.Generator(np.random.PCG64(seed))


def test_conv2d_gradient_specs(tf):
    ops = tf.ops
    # ops/conv2d_test.ts:398-423 "gradient with clones input=[3,3,1] f=[2,2,1,1] s=1 p=0"
    x = ops.tensor(np.arange(1, 10, dtype=np.float32), [3, 3, 1])
    filt = ops.tensor(np.ones(4, np.float32), [2, 2, 1, 1])
    dy = ops.tensor(np.array([3, 1, 2, 0], np.float32), [2, 2, 1])
    dx, dfilter = ops.grads(lambda a, f: ops.clone(ops.conv2d(ops.clone(a), ops.clone(f), 1, 0)))([x, filt], dy)
    assert dx.shape == [3, 3, 1] and dfilter.shape == [2, 2, 1, 1]
    np.testing.assert_allclose(dx.dataSync(), [3, 4, 1, 5, 6, 1, 2, 2, 0], atol=1e-3)
    np.testing.assert_allclose(dfilter.dataSync(), [13, 19, 31, 37], atol=1e-3)
    # :425-452 batch of two
    x2 = ops.tensor(np.tile(np.arange(1, 10, dtype=np.float32), 2), [2, 3, 3, 1])
    dy2 = ops.tensor(np.array([3, 1, 2, 0] * 2, np.float32), [2, 2, 2, 1])
    dx2, df2 = ops.grads(lambda a, f: ops.conv2d(a, f, 1, 0))([x2, filt], dy2)
    np.testing.assert_allclose(dx2.dataSync(), [3, 4, 1, 5, 6, 1, 2, 2, 0] * 2, atol=1e-3)
    np.testing.assert_allclose(df2.dataSync(), [26, 38, 62, 74], atol=1e-3)


def test_depthwise_gradient_specs(tf):
    ops = tf.ops
    # ops/conv2d_depthwise_test.ts:580-650
    images = ops.tensor(np.array([[[[2, 3, 1], [3, 0, 2]], [[0, 4, 1], [3, 1, 3]]],
                                  [[[2, 1, 0], [0, 3, 3]], [[4, 0, 1], [1, 4, 1]]]], np.float32))
    filt = ops.tensor(np.array([[[[1, 1], [1, 1], [0, 0]], [[0, 1], [1, 1], [1, 1]]],
                                [[[1, 0], [1, 1], [0, 0]], [[0, 1], [1, 0], [0, 0]]]], np.float32))
    value, (gx,) = ops.value_and_grads(lambda a: ops.depthwise_conv2d(a, filt, 1, "same"))([images])
    want_value = [2, 8, 8, 7, 2, 2, 6, 3, 1, 1, 0, 0, 0, 3, 5, 5, 3, 3, 3, 3, 1, 1, 0, 0,
                  6, 3, 8, 4, 3, 3, 1, 0, 7, 7, 0, 0, 4, 5, 4, 4, 1, 1, 1, 1, 4, 4, 0, 0]
    np.testing.assert_allclose(value.dataSync(), want_value, atol=1e-3)
    np.testing.assert_allclose(gx.dataSync(), [2, 2, 0, 3, 4, 2, 3, 4, 0, 5, 7, 2] * 2, atol=1e-3)
    # "wrt input, squared output" :612-623
    g2 = ops.grad(lambda a: ops.square(ops.depthwise_conv2d(a, filt, 1, "same")))(images)
    np.testing.assert_allclose(g2.dataSync(), [20, 30, 0, 34, 34, 8, 10, 50, 0, 46, 44, 12,
                                               18, 24, 0, 8, 52, 12, 30, 40, 0, 22, 76, 4], atol=1e-3)
    # "wrt filter" :625-638
    gf = ops.grad(lambda f: ops.depthwise_conv2d(images, f, 1, "same"))(filt)
    np.testing.assert_allclose(gf.dataSync(), [15, 15, 16, 16, 12, 12, 7, 7, 8, 8, 9, 9,
                                               8, 8, 9, 9, 6, 6, 4, 4, 5, 5, 4, 4], atol=1e-3)


def test_pool_gradient_specs(tf):
    ops = tf.ops
    dy = ops.tensor(np.array([1, 2, 3, 4], np.float32), [2, 2, 1])
    # ops/pool_test.ts:141-150
    x = ops.tensor(np.arange(1, 10, dtype=np.float32), [3, 3, 1])
    dx = ops.grad(lambda a: ops.max_pool(a, 2, 1, 0))(x, dy)
    np.testing.assert_allclose(dx.dataSync(), [0, 0, 0, 0, 1, 2, 0, 3, 4], atol=1e-3)
    # :188-197 duplicate maximum: the whole gradient lands on it
    x = ops.tensor(np.array([0, 0, 0, 0, 5, 0, 0, 0, 0], np.float32), [3, 3, 1])
    dx = ops.grad(lambda a: ops.max_pool(a, 2, 1, 0))(x, dy)
    np.testing.assert_allclose(dx.dataSync(), [0, 0, 0, 0, 10, 0, 0, 0, 0], atol=1e-3)
    # :468-482 average pool
    x = ops.tensor(np.array([1, 2, 3, 4, 5, 6, 7, 9, 8], np.float32), [3, 3, 1])
    dx = ops.grad(lambda a: ops.avg_pool(a, 2, 1, 0))(x, dy)
    np.testing.assert_allclose(dx.dataSync(), np.array([1, 3, 2, 4, 10, 6, 3, 7, 4]) / 4, atol=1e-3)


def test_elementwise_and_matmul_gradients(tf):
    ops = tf.ops
    rng = _rng(4)
    a = rng.normal(0, 1, (3, 4)).astype(np.float32)
    b = rng.normal(0, 1, (4, 5)).astype(np.float32)
    bias = rng.normal(0, 1, (5,)).astype(np.float32)
    dy = rng.normal(0, 1, (3, 5)).astype(np.float32)
    ta, tb, tbias, tdy = (ops.tensor(v) for v in (a, b, bias, dy))
    # y = relu(a @ b + bias) * 2 - a @ b ; compare with numpy
    def f(x, w, c):
        m = ops.matmul(x, w)
        r = ops.relu(ops.add(m, c))
        return ops.sub(ops.mul(r, ops.scalar(2.0)), m)
    ga, gb, gc = ops.grads(f)([ta, tb, tbias], tdy)
    m = a.astype(np.float64) @ b
    mask = (m + bias > 0).astype(np.float64)
    dm = 2 * dy * mask - dy
    np.testing.assert_allclose(ga.dataSync().reshape(3, 4), dm @ b.T, atol=2e-5)
    np.testing.assert_allclose(gb.dataSync().reshape(4, 5), a.T @ dm, atol=2e-5)
    np.testing.assert_allclose(gc.dataSync(), (2 * dy * mask).sum(0), atol=2e-5)
    # softmax, both forms, exp / log / div / sum over a non-inner axis
    z = rng.normal(0, 1, (4, 6)).astype(np.float32)
    t = rng.normal(0, 1, (4, 6)).astype(np.float32)
    p = np.exp(z - z.max(1, keepdims=True))
    p /= p.sum(1, keepdims=True)
    want = p * t - (p * t).sum(1, keepdims=True) * p
    for sm in (ops.softmax, ops.fused_softmax):
        g = ops.grad(lambda v: sm(v))(ops.tensor(z), ops.tensor(t))
        np.testing.assert_allclose(g.dataSync().reshape(4, 6), want, atol=1e-6)
    g = ops.grad(lambda v: ops.sum(ops.div(ops.log(ops.exp(v)), ops.tensor(t)), 0))(ops.tensor(z))
    np.testing.assert_allclose(g.dataSync().reshape(4, 6), 1.0 / t, rtol=1e-5)


def test_small_separable_network_gradients_match_the_oracle_chain_rule(tf):
    """loss = sum(softmax(fc(avgpool(block(block(stem(x)))))) * target) differentiated by the tape
    with respect to the image and all eight parameter tensors, against the same chain written
    out with the oracle's gradient kernels."""
    ops = tf.ops
    rng = _rng(12)
    B, H, C1, C2, NCLS = 2, 12, 8, 16, 10
    v = dict(
        x=rng.uniform(-1, 1, (B, H, H, 3)), w1=rng.normal(0, 0.4, (3, 3, 3, C1)), b1=rng.normal(0.5, 0.2, C1),
        wd=rng.normal(0, 0.4, (3, 3, C1, 1)), bd=rng.normal(0.5, 0.2, C1), wp=rng.normal(0, 0.4, (1, 1, C1, C2)),
        bp=rng.normal(0.5, 0.2, C2), wf=rng.normal(0, 0.5, (C2, NCLS)), bf=rng.normal(0, 0.1, NCLS))
    v = {k: a.astype(np.float32) for k, a in v.items()}
    target = rng.normal(0, 1, (B, NCLS)).astype(np.float32)
    names = list(v)
    tensors = [ops.tensor(v[k]) for k in names]

    def net(x, w1, b1, wd, bd, wp, bp, wf, bf):
        h = ops.clip_by_value(ops.add(ops.conv2d(x, w1, 2, "same"), b1), 0, 6)
        h = ops.clip_by_value(ops.add(ops.depthwise_conv2d(h, wd, 1, "same"), bd), 0, 6)
        h = ops.clip_by_value(ops.add(ops.conv2d(h, wp, 1, "valid"), bp), 0, 6)
        h = ops.avg_pool(h, [h.shape[1], h.shape[2]], 1, "valid")
        logits = ops.add(ops.matmul(ops.reshape(h, [B, C2]), wf), bf)
        return ops.sum(ops.mul(ops.softmax(logits), ops.tensor(target)))
    loss, got = ops.value_and_grads(net)(tensors)

    # ---- the same chain on the CPU oracle ----
    o = oracle
    ci1 = o.compute_conv2d_info(v["x"].shape, v["w1"].shape, 2, 1, "same")
    a1 = o.binary("add", o.conv2d(v["x"], v["w1"], ci1), v["b1"])
    h1 = o.unary("clip", a1, 0, 6)
    cid = o.compute_conv2d_info(h1.shape, v["wd"].shape, 1, 1, "same", None, True)
    a2 = o.binary("add", o.depthwise_conv2d(h1, v["wd"], cid), v["bd"])
    h2 = o.unary("clip", a2, 0, 6)
    cip = o.compute_conv2d_info(h2.shape, v["wp"].shape, 1, 1, "valid")
    a3 = o.binary("add", o.conv2d(h2, v["wp"], cip), v["bp"])
    h3 = o.unary("clip", a3, 0, 6)
    cpool = o.compute_pool2d_info(h3.shape, [h3.shape[1], h3.shape[2]], 1, 1, "valid")
    pooled = o.pool(h3, cpool, "avg").reshape(B, C2)
    logits = o.fused_matmul(pooled[None], v["wf"][None], bias=v["bf"])[0]
    probs = o.softmax_last(logits)
    assert abs(float(loss.dataSync()[0]) - float((probs.astype(np.float64) * target).sum())) < 1e-4
    dyy = probs * target
    dlogits = (dyy - dyy.sum(1, keepdims=True) * probs).astype(np.float32)
    want = {"bf": dlogits.sum(0), "wf": pooled.T @ dlogits}
    dpooled = (dlogits @ v["wf"].T).astype(np.float32).reshape(B, 1, 1, C2)
    d3 = o.pool_backprop(dpooled, h3, cpool, "avg") * ((a3 >= 0) & (a3 <= 6))
    want["bp"] = d3.sum((0, 1, 2))
    want["wp"] = o.conv2d_der_filter(h2, d3, cip)
    d2 = o.conv2d_der_input(d3, v["wp"], cip) * ((a2 >= 0) & (a2 <= 6))
    want["bd"] = d2.sum((0, 1, 2))
    want["wd"] = o.depthwise_der_filter(h1, d2, cid)
    d1 = o.depthwise_der_input(d2, v["wd"], cid) * ((a1 >= 0) & (a1 <= 6))
    want["b1"] = d1.sum((0, 1, 2))
    want["w1"] = o.conv2d_der_filter(v["x"], d1, ci1)
    want["x"] = o.conv2d_der_input(d1, v["w1"], ci1)
    for k, g in zip(names, got):
        assert g.shape == list(v[k].shape), k
        assert rel_err(g.dataSync().reshape(v[k].shape), want[k]) <= 1e-4, k
