"""GPU: a launch-bound training step recorded once and replayed (CUDA graph).

Config 1 of the benchmark (MLP 784-128-64-10, batch 32) and the reference
trainer's batch-1 loop (src/main.cpp:20-46) are chains of ~20 dependent
micro-kernels.  `RecordedStep` records the step as it is written on the Tensor
API and replays it with one launch.  The replays must produce exactly what the
same steps produce when run one launch at a time — same kernels, same order, so
the comparison is bit for bit — and agree with the CPU oracle within the parity
bar (1e-10).
"""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu

SIZES = [784, 128, 64, 10]


def _model(api, params, lr):
    layers = []
    for W, b in params:
        lin = api.Linear(W.shape[0], W.shape[1])
        lin.weights().set_data(W)
        lin.bias().set_data(b)
        layers.append(lin)
    return layers, api.SGD([t for lin in layers for t in (lin.weights(), lin.bias())], lr)


def _step(api, layers, opt, x, y):
    h = layers[1].forward_relu(layers[0].forward_relu(x))
    loss = api.softmax_cross_entropy(layers[2].forward(h), y)
    opt.zero_grad()
    loss.backward()
    opt.step()
    return loss


def test_recorded_step_equals_eager_steps_and_the_oracle(api, abi, fast):
    rng = np.random.default_rng(42)
    batch, steps, lr = 32, 6, 0.05
    params = [(rng.standard_normal((i, o)) / np.sqrt(i), np.zeros(o)) for i, o in zip(SIZES[:-1], SIZES[1:])]
    Xs = [rng.random((batch, 784)) for _ in range(steps)]
    ys = [rng.integers(0, 10, batch).astype(np.float64) for _ in range(steps)]

    # one launch at a time
    layers, opt = _model(api, params, lr)
    eager = []
    for X, y in zip(Xs, ys):
        x = api.Tensor([batch, 784], X)
        x.set_requires_grad(False)
        eager.append(_step(api, layers, opt, x, api.Tensor([batch], y)).data()[0])
    eager_params = [(lin.weights().data().copy(), lin.bias().data().copy()) for lin in layers]

    # recorded: step 0 runs normally (it also creates the GEMM tables and scratch
    # buffers), step 1 is recorded, steps 1..5 are replays
    layers, opt = _model(api, params, lr)
    x = api.Tensor([batch, 784], Xs[0])
    x.set_requires_grad(False)
    y = api.Tensor([batch], ys[0])
    first = _step(api, layers, opt, x, y)
    got = [first.data()[0]]
    del first                                   # nothing made before begin() may die while recording
    rec = api.RecordedStep()
    rec.begin()
    loss = _step(api, layers, opt, x, y)        # recorded, not executed
    with pytest.raises(RuntimeError):
        loss.data()                             # host reads are refused while recording ...
    rec.end()                                   # ... and leave the recording intact
    assert rec.kernels() >= 15
    for X, yy in zip(Xs[1:], ys[1:]):
        x.copy_from_host(X)
        y.copy_from_host(yy)
        before = abi.mg_launch_count()
        rec.replay()
        assert abi.mg_launch_count() - before == rec.kernels()
        got.append(loss.data()[0])              # same tensor, new value after every replay
    abi.mg_check_kernel_status()
    assert got == eager
    for lin, (W, b) in zip(layers, eager_params):
        assert np.array_equal(lin.weights().data(), W) and np.array_equal(lin.bias().data(), b)

    # and the oracle
    ref = [(W.copy(), b.copy()) for W, b in params]
    for s in range(steps):
        ref_loss, _, _ = fast.mlp_train_step(ref, Xs[s], ys[s].astype(np.int32), lr)
        assert abs(got[s] - ref_loss) <= 1e-10 * abs(ref_loss)
    for lin, (W, b) in zip(layers, ref):
        assert np.abs(lin.weights().data() - W.reshape(-1)).max() <= 1e-10 * np.abs(W).max()


def test_recorded_per_sample_trainer_step(api, abi, fast):
    """The reference trainer's loop body at batch 1: avg_pool -> Linear -> relu ->
    Linear -> mse_loss, zero_grad, backward, SGD step; the loss is read after
    each replay as src/main.cpp:45 reads it."""
    rng = np.random.default_rng(7)
    l1, l2 = api.Linear(196, 100), api.Linear(100, 10)
    W1, W2 = rng.uniform(-0.1, 0.1, (196, 100)), rng.uniform(-0.1, 0.1, (100, 10))
    images = rng.random((5, 784))
    targets = np.eye(10)[rng.integers(0, 10, 5)]

    def run(recorded):
        l1.weights().set_data(W1); l1.bias().set_data(np.zeros(100))
        l2.weights().set_data(W2); l2.bias().set_data(np.zeros(10))
        opt = api.SGD([l1.weights(), l1.bias(), l2.weights(), l2.bias()], 0.01)
        img, tgt = api.Tensor([1, 784], images[0]), api.Tensor([1, 10], targets[0])

        def body():
            out = l2.forward(l1.forward(api.avg_pool_2x2(img)).relu())
            loss = api.mse_loss(out, tgt)
            opt.zero_grad()
            loss.backward()
            opt.step()
            return loss

        losses = []
        if not recorded:
            for i in range(5):
                img.copy_from_host(images[i]); tgt.copy_from_host(targets[i])
                losses.append(body().at([0]))
            return losses, l1.weights().data().copy()
        warm = body()
        losses.append(warm.at([0]))
        del warm
        rec = api.RecordedStep()
        rec.begin()
        loss = body()
        rec.end()
        for i in range(1, 5):
            img.copy_from_host(images[i]); tgt.copy_from_host(targets[i])
            rec.replay()
            losses.append(loss.at([0]))
        return losses, l1.weights().data().copy()

    eager_losses, eager_w = run(False)
    rec_losses, rec_w = run(True)
    abi.mg_check_kernel_status()
    assert rec_losses == eager_losses
    assert np.array_equal(rec_w, eager_w)


def test_abandoned_recording_is_closed(api, abi):
    """A RecordedStep dropped between begin() and end() ends the recording: work
    enqueued afterwards executes again."""
    rec = api.RecordedStep()
    a = api.Tensor([4], [1.0, 2.0, 3.0, 4.0])
    warm = a.mul(2.0).sum()
    assert warm.data()[0] == 20.0
    del warm
    rec.begin()
    pending = a.mul(3.0).sum()                 # recorded only
    rec.abandon()
    del pending
    assert a.mul(3.0).sum().data()[0] == 30.0  # executes
    abi.mg_check_kernel_status()


def test_replay_survives_scratch_buffers_outgrown_after_the_recording(api, abi):
    """A recorded bias-gradient column sum carries the address of the library's
    scratch buffer for partial sums.  A larger column sum after the recording makes
    the library take a bigger buffer; the old one must stay alive for the replay,
    which is checked here with fresh allocations in between that would otherwise
    land on the freed memory."""
    rng = np.random.default_rng(3)
    rows, cols = 4096, 256                        # several row chunks: partials + second stage
    X = rng.standard_normal((rows, cols))
    x = api.Tensor([rows, cols], X)
    bias = api.Tensor([1, cols], np.zeros((1, cols)))

    def bias_grad():
        bias.zero_grad()
        out = x.add(bias).sum()                   # row-broadcast add; backward = column sum of ones
        out.backward()
        return out

    first = bias_grad()                           # normal run: scratch buffers get their first size
    want = np.array(bias.grad()).copy()
    assert np.array_equal(want, np.full(cols, float(rows)))
    del first
    rec = api.RecordedStep()
    rec.begin()
    out = bias_grad()
    rec.end()
    # outgrow the scratch buffer (wider and taller), then churn the pool
    wide = api.Tensor([8192, 4096], np.ones((8192, 4096)))
    wide_bias = api.Tensor([1, 4096], np.zeros((1, 4096)))
    wide.add(wide_bias).sum().backward()
    assert np.array_equal(np.array(wide_bias.grad()), np.full(4096, 8192.0))
    junk = [api.Tensor([1 << 16], np.full(1 << 16, 7.0)) for _ in range(32)]
    for t in junk:
        t.mul(2.0)
    for _ in range(3):
        rec.replay()
        assert np.array_equal(np.array(bias.grad()), want)
        assert abs(out.data()[0] - X.sum()) <= 1e-10 * np.abs(X).sum()
    abi.mg_check_kernel_status()
    del junk
