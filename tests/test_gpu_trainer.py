"""GPU: the reference's own application pattern — the per-sample MNIST trainer of
src/main.cpp and inference with the weights of its models/mnist.bin — on the
B200 backend, against vectors produced by the reference's compiled code
(tests/golden/trainer_mnist_bin.npz, made by tests/golden/make_golden.py).
"""
import os
import re

import numpy as np
import pytest

from conftest import golden, norm_err

import oracle

pytestmark = pytest.mark.gpu


def _load_reference_weights(api, g, tmp_path):
    """Writes W1,b1,W2,b2 in the raw fp64 layout of save_model (src/nn.cpp:79-101)
    and loads them with load_model — the file has the size of models/mnist.bin."""
    path = str(tmp_path / "mnist.bin")
    with open(path, "wb") as f:
        for key in ("W1", "b1", "W2", "b2"):
            f.write(np.ascontiguousarray(g[key], dtype=np.float64).tobytes())
    assert os.path.getsize(path) == 165680
    l1, l2 = api.Linear(196, 100), api.Linear(100, 10)
    api.load_model(path, l1, l2)
    return l1, l2


def test_inference_with_reference_model_file(api, tmp_path):
    g = golden("trainer_mnist_bin.npz")
    l1, l2 = _load_reference_weights(api, g, tmp_path)
    images = g["infer_images"]
    # per sample, exactly as the reference drives it
    for i in range(8):
        x = api.Tensor([1, 784], images[i])
        got = l2.forward(l1.forward(api.avg_pool_2x2(x)).relu()).data()
        assert norm_err(got, g["infer_logits"][i]) <= 1e-10
    # and as one batch of 64 (batched Linear, device pooling)
    xb = api.Tensor([64, 784], images)
    logits = l2.forward(l1.forward_relu(api.avg_pool_2x2(xb)))
    assert norm_err(logits.data().reshape(64, 10), g["infer_logits"]) <= 1e-10
    assert np.array_equal(api.argmax_rows(logits), g["infer_logits"].argmax(axis=1))


def test_avg_pool_matches_reference_order(api):
    rng = np.random.default_rng(0)
    img = rng.random((5, 784))
    got = api.avg_pool_2x2(api.Tensor([5, 784], img)).data().reshape(5, 196)
    v = img.reshape(5, 14, 2, 14, 2).transpose(0, 1, 3, 2, 4).reshape(5, 196, 4)
    ref = (((v[..., 0] + v[..., 1]) + v[..., 2]) + v[..., 3]) / 4.0
    assert np.array_equal(got, ref)
    one = api.avg_pool_2x2(api.Tensor([1, 784], img[3]))
    assert one.shape() == [1, 196] and np.array_equal(one.data(), ref[3])


def test_per_sample_trainer_loop_matches_reference(api, tmp_path):
    """src/main.cpp:20-46, two epochs over 24 samples: every loss, every host-side
    prediction and the final parameters."""
    g = golden("trainer_mnist_bin.npz")
    l1, l2 = _load_reference_weights(api, g, tmp_path)
    opt = api.SGD([l1.weights(), l1.bias(), l2.weights(), l2.bias()], 0.01)
    losses, preds = [], []
    for epoch in range(2):
        for i in range(24):
            onehot = np.zeros(10)
            onehot[g["train_labels"][i]] = 1.0
            x = l1.forward(api.avg_pool_2x2(api.Tensor([1, 784], g["train_images"][i]))).relu()
            o = l2.forward(x)
            loss = api.mse_loss(o, api.Tensor([1, 10], onehot))
            pred = 0
            for j in range(10):
                if o.at([0, j]) > o.at([0, pred]):
                    pred = j
            preds.append(pred)
            opt.zero_grad()
            loss.backward()
            opt.step()
            losses.append(loss.at([0]))
    assert np.max(np.abs(np.array(losses) - g["losses"]) / g["losses"]) <= 1e-10
    assert np.array_equal(np.array(preds), g["preds"])
    for key, t in (("W1", l1.weights()), ("b1", l1.bias()), ("W2", l2.weights()), ("b2", l2.bias())):
        assert norm_err(t.data(), g[key + "_final"].reshape(-1)) <= 1e-10, key


@pytest.mark.skipif(not os.path.exists(oracle.REF_TRUE_PATH), reason="reference library not built")
def test_to_dot_text_equals_reference(api):
    """Same graph in both implementations: the Graphviz text is identical line for
    line once node addresses are renamed in order of appearance."""
    def build(a):
        x = a.Tensor([2], [2.0, -1.0])
        w = a.Tensor([2], [0.5, 3.0])
        y = x.mul(w).add(x).relu().mul(2.0).sum()
        y.backward()
        return y.to_dot()

    def normalise(text):
        names = {}
        return re.sub(r"0x[0-9a-f]+", lambda m: names.setdefault(m.group(0), f"n{len(names)}"), text)

    assert normalise(build(api)) == normalise(build(oracle.ref_true()))
