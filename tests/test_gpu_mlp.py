"""GPU: the MLP hot path end to end (benchmark configs 1, 4, 5 at test sizes).

Linear (fused bias / bias+ReLU GEMM epilogues) -> softmax cross-entropy ->
backward -> SGD, compared with the reference-generated golden vectors of config
1 and with the CPU oracle; batched inference argmax compared bit-exactly.
Tolerances: <= 1e-10 (matmul/reduction bound), stated per assertion.
"""
import numpy as np
import pytest

from conftest import golden, norm_err

pytestmark = pytest.mark.gpu


def build_mlp(api, params):
    layers = []
    for W, b in params:
        lin = api.Linear(W.shape[0], W.shape[1])
        lin.weights().set_data(W)
        lin.bias().set_data(b)
        layers.append(lin)
    return layers


def forward(api, layers, x, fused):
    h = x
    for i, lin in enumerate(layers):
        last = i + 1 == len(layers)
        if last:
            h = lin.forward(h)
        elif fused:
            h = lin.forward_relu(h)
        else:
            h = lin.forward(h).relu()
    return h


@pytest.mark.parametrize("fused", [False, True])
def test_config1_training_step_matches_reference_golden(api, fused):
    """784-128-64-10, batch 32, lr 0.01: loss, all gradients, the input gradient
    and the updated parameters against vectors produced by the reference code."""
    g = golden("mlp_c1.npz")
    params = [(g[f"W{i}"], g[f"b{i}"]) for i in range(3)]
    layers = build_mlp(api, params)
    flat = [t for lin in layers for t in (lin.weights(), lin.bias())]
    opt = api.SGD(flat, 0.01)
    x = api.Tensor([32, 784], g["X"])
    logits = forward(api, layers, x, fused)
    loss = api.softmax_cross_entropy(logits, g["y"])
    opt.zero_grad()
    loss.backward()
    assert abs(loss.data()[0] - float(g["loss"])) <= 1e-10 * abs(float(g["loss"]))
    for i, lin in enumerate(layers):
        assert norm_err(lin.weights().grad(), g[f"gW{i}"].reshape(-1)) <= 1e-10, i
        assert norm_err(lin.bias().grad(), g[f"gb{i}"]) <= 1e-10, i
    assert norm_err(x.grad(), g["gX"].reshape(-1)) <= 1e-10
    opt.step()
    for i, lin in enumerate(layers):
        assert norm_err(lin.bias().data(), g[f"b{i}_new"]) <= 1e-10, i
        assert abs(lin.weights().data().sum() - float(g[f"W{i}_new_sum"])) <= 1e-9, i


def test_labels_as_tensor_and_skipped_input_gradient(api):
    g = golden("mlp_c1.npz")
    layers = build_mlp(api, [(g[f"W{i}"], g[f"b{i}"]) for i in range(3)])
    x = api.Tensor([32, 784], g["X"])
    x.set_requires_grad(False)
    labels = api.Tensor([32], g["y"].astype(np.float64))
    loss = api.softmax_cross_entropy(forward(api, layers, x, True), labels)
    loss.backward()
    assert abs(loss.data()[0] - float(g["loss"])) <= 1e-10 * abs(float(g["loss"]))
    assert not x.grad().any()
    assert norm_err(layers[0].weights().grad(), g["gW0"].reshape(-1)) <= 1e-10


@pytest.mark.parametrize("batch,sizes", [(256, [784, 128, 64, 10]), (192, [784, 1024, 1024, 10])])
def test_multi_step_training_tracks_oracle(api, fast, batch, sizes):
    """Five SGD steps (config-4 architecture at a reduced batch): loss curve and
    final weights against the oracle, normwise <= 1e-9 after five steps."""
    rng = np.random.default_rng(sizes[1])
    params = [(rng.standard_normal((i, o)) / np.sqrt(i), np.zeros(o)) for i, o in zip(sizes[:-1], sizes[1:])]
    X, y = rng.random((batch, sizes[0])), rng.integers(0, 10, batch).astype(np.int32)
    layers = build_mlp(api, params)
    flat = [t for lin in layers for t in (lin.weights(), lin.bias())]
    opt = api.SGD(flat, 0.01)
    opt.enable_allreduce()          # flat parameter/gradient buffers; single process: no exchange
    ref = [(W.copy(), b.copy()) for W, b in params]
    x = api.Tensor([batch, sizes[0]], X)
    x.set_requires_grad(False)
    for step in range(5):
        loss = api.softmax_cross_entropy(forward(api, layers, x, True), y)
        opt.zero_grad()
        loss.backward()
        opt.step()
        ref_loss, _, _ = fast.mlp_train_step(ref, X, y, 0.01)
        assert abs(loss.data()[0] - ref_loss) <= 1e-10 * abs(ref_loss), step
    for lin, (W, b) in zip(layers, ref):
        assert norm_err(lin.weights().data(), W.reshape(-1)) <= 1e-9
        assert norm_err(lin.bias().data(), b) <= 1e-9


def test_batched_inference_argmax_bit_exact(api, fast):
    """Config 5 at 16384 inputs: class ids equal the oracle's on every row."""
    rng = np.random.default_rng(5)
    sizes = [784, 128, 64, 10]
    params = [(rng.standard_normal((i, o)) / np.sqrt(i), np.zeros(o)) for i, o in zip(sizes[:-1], sizes[1:])]
    X = rng.random((16384, 784))
    layers = build_mlp(api, params)
    x = api.Tensor([16384, 784], X)
    x.set_requires_grad(False)
    ids = api.argmax_rows(forward(api, layers, x, True))
    logits, _ = fast.mlp_forward(params, X)
    ref_ids = fast.argmax_rows(logits)
    mism = np.nonzero(ids != ref_ids)[0]
    if mism.size:  # report the top-2 gap of any flipped row
        top2 = np.sort(logits[mism], axis=1)[:, -2:]
        raise AssertionError(f"{mism.size} argmax flips; top-2 gaps {top2[:, 1] - top2[:, 0]}")
    # row sharding does not change the ids (inference shards by rows across GPUs)
    half = api.Tensor([8192, 784], X[8192:])
    assert np.array_equal(api.argmax_rows(forward(api, layers, half, True)), ids[8192:])


def test_from_host_upload_matches_constructor(api):
    rng = np.random.default_rng(1)
    X = np.ascontiguousarray(rng.random((64, 784)))
    a = api.Tensor([64, 784], X)
    b = api.from_host([64, 784], X.ctypes.data)
    api.synchronize()
    assert np.array_equal(a.data(), b.data())


def _train_both(api, fast, sizes, batch, steps, lr=0.01, seed=0):
    rng = np.random.default_rng(seed)
    params = [(rng.standard_normal((i, o)) / np.sqrt(i), np.zeros(o)) for i, o in zip(sizes[:-1], sizes[1:])]
    X, y = rng.random((batch, sizes[0])), rng.integers(0, 10, batch).astype(np.int32)
    layers = build_mlp(api, params)
    opt = api.SGD([t for lin in layers for t in (lin.weights(), lin.bias())], lr)
    opt.enable_allreduce()
    ref = [(W.copy(), b.copy()) for W, b in params]
    x = api.Tensor([batch, sizes[0]], X)
    x.set_requires_grad(False)
    labels = api.Tensor([batch], y.astype(np.float64))
    got, want = [], []
    for _ in range(steps):
        loss = api.softmax_cross_entropy(forward(api, layers, x, True), labels)
        opt.zero_grad()
        loss.backward()
        opt.step()
        got.append(loss)
        want.append(fast.mlp_train_step(ref, X, y, lr)[0])
    got = np.array([t.data()[0] for t in got])
    return got, np.array(want), layers, ref


def test_hundred_steps_of_config4_architecture_at_reduced_batch(api, fast):
    """784-1024-1024-10, 100 SGD steps (benchmark config 4's step count) at batch 256:
    the whole loss curve and the final parameters against the oracle."""
    got, want, layers, ref = _train_both(api, fast, [784, 1024, 1024, 10], 256, 100)
    assert np.max(np.abs(got - want) / np.abs(want)) <= 1e-9
    assert want[-1] < want[0]                                  # it does learn its batch
    for lin, (W, b) in zip(layers, ref):
        assert norm_err(lin.weights().data(), W.reshape(-1)) <= 1e-9
        assert norm_err(lin.bias().data(), b) <= 1e-9


def test_two_full_batch_steps_of_config4(api, fast):
    """Benchmark config 4 at its full size (global batch 65536): two SGD steps against
    the multi-threaded order-preserving oracle (about half a minute of host time)."""
    got, want, layers, ref = _train_both(api, fast, [784, 1024, 1024, 10], 65536, 2)
    assert np.max(np.abs(got - want) / np.abs(want)) <= 1e-10
    for lin, (W, b) in zip(layers, ref):
        assert norm_err(lin.weights().data(), W.reshape(-1)) <= 1e-10
        assert norm_err(lin.bias().data(), b) <= 1e-10
