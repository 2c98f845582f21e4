"""Generates tests/golden/*.npz by running the reference project's own compiled
code (oracle/_ref/libref_true.so, built by `make -C oracle` from the mounted
reference tree) on seeded inputs.

    python tests/golden/make_golden.py

The fixtures hold inputs AND outputs, so the tests never depend on a random
generator reproducing the same stream.  They are consumed by
tests/test_oracle.py (ref_fast must reproduce them bit for bit, without the
reference tree) and by the GPU parity tests.
"""
from __future__ import annotations

import os
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(os.path.dirname(HERE)))

import oracle  # noqa: E402


def elementwise_cases(api, rng):
    out = {}
    shape = [3, 5]
    a = rng.standard_normal(shape)
    b = rng.standard_normal(shape) + 3.0  # keep divisors away from zero
    ga0 = rng.standard_normal(shape)
    gb0 = rng.standard_normal(shape)
    seed = rng.standard_normal(shape)  # upstream gradient, injected via mul(seed).sum()
    out.update(a=a, b=b, ga0=ga0, gb0=gb0, seed=seed)
    for op in ("add", "sub", "mul", "div"):
        ta, tb, ts = api.Tensor(shape, a), api.Tensor(shape, b), api.Tensor(shape, seed)
        ta.set_grad(ga0)
        tb.set_grad(gb0)
        c = getattr(ta, op)(tb)
        c.mul(ts).sum().backward()
        out[f"{op}_out"] = c.data().reshape(shape)
        out[f"{op}_ga"] = ta.grad().reshape(shape)
        out[f"{op}_gb"] = tb.grad().reshape(shape)
    scal = 1.75
    pos = np.abs(a) + 0.5  # pow with a fractional exponent needs a positive base
    out["scalar"] = np.float64(scal)
    out["pos"] = pos
    for op, arg in (("add", scal), ("sub", scal), ("mul", scal), ("div", scal)):
        ta, ts = api.Tensor(shape, a), api.Tensor(shape, seed)
        ta.set_grad(ga0)
        c = getattr(ta, op)(arg)
        c.mul(ts).sum().backward()
        out[f"s{op}_out"] = c.data().reshape(shape)
        out[f"s{op}_ga"] = ta.grad().reshape(shape)
    for expo, tag in ((2.0, "pow2"), (2.5, "pow25"), (3.0, "pow3")):
        ta, ts = api.Tensor(shape, pos), api.Tensor(shape, seed)
        ta.set_grad(ga0)
        c = ta.pow(expo)
        c.mul(ts).sum().backward()
        out[f"{tag}_out"] = c.data().reshape(shape)
        out[f"{tag}_ga"] = ta.grad().reshape(shape)
    for op in ("relu", "sigmoid", "tanh"):
        ta, ts = api.Tensor(shape, a), api.Tensor(shape, seed)
        ta.set_grad(ga0)
        c = getattr(ta, op)()
        c.mul(ts).sum().backward()
        out[f"{op}_out"] = c.data().reshape(shape)
        out[f"{op}_ga"] = ta.grad().reshape(shape)
    # x (op) x: both gradient updates land on one tensor
    ta = api.Tensor(shape, a)
    ta.set_grad(ga0)
    c = ta.mul(ta)
    c.sum().backward()
    out["square_out"] = c.data().reshape(shape)
    out["square_ga"] = ta.grad().reshape(shape)
    return out


def matmul_cases(api, rng):
    out = {}
    for tag, (m, k, n) in {"small": (5, 7, 4), "odd": (33, 17, 9), "even": (32, 48, 16)}.items():
        A = rng.standard_normal((m, k)) / np.sqrt(k)
        B = rng.standard_normal((k, n)) / np.sqrt(k)
        gA0 = rng.standard_normal((m, k))
        gB0 = rng.standard_normal((k, n))
        seed = rng.standard_normal((m, n))
        ta, tb, ts = api.Tensor([m, k], A), api.Tensor([k, n], B), api.Tensor([m, n], seed)
        ta.set_grad(gA0)
        tb.set_grad(gB0)
        c = ta.matmul(tb)
        loss = c.mul(ts).sum()
        loss.backward()
        out.update({f"{tag}_A": A, f"{tag}_B": B, f"{tag}_gA0": gA0, f"{tag}_gB0": gB0,
                    f"{tag}_seed": seed, f"{tag}_C": c.data().reshape(m, n),
                    f"{tag}_gA": ta.grad().reshape(m, k), f"{tag}_gB": tb.grad().reshape(k, n),
                    f"{tag}_loss": loss.data()})
    # sum(): 1000 values, and the reference test's 1..10000 ramp
    x = rng.standard_normal(1000)
    t = api.Tensor([1000], x)
    s = t.sum()
    s.backward()
    out.update(sum_x=x, sum_out=s.data(), sum_gx=t.grad())
    return out


def axis_sum_cases(api, rng):
    """Encodings of two ops the reference lacks, run by the reference's own matmul
    loop (src/ops/Matmul.cpp:30-58): the last-axis sum of X is X.matmul(ones[N,1])
    (0.0 + x*1.0 left to right along the row) and the column sum is
    ones[1,M].matmul(X) (ascending rows).  Their backward closures give the
    gradients of the two sums: gx[i,j] += g[i] and gx[i,j] += g[j]."""
    out = {}
    M, N = 37, 23
    X = rng.standard_normal((M, N))
    gx0 = rng.standard_normal((M, N))
    seed_rows, seed_cols = rng.standard_normal((M, 1)), rng.standard_normal((1, N))
    tx, ones = api.Tensor([M, N], X), api.Tensor([N, 1], np.ones(N))
    tx.set_grad(gx0)
    rows = tx.matmul(ones)
    rows.mul(api.Tensor([M, 1], seed_rows)).sum().backward()
    out.update(X=X, gx0=gx0, seed_rows=seed_rows.reshape(M), seed_cols=seed_cols.reshape(N),
               row_sums=rows.data().reshape(M), row_sums_gx=tx.grad().reshape(M, N))
    tx, ones = api.Tensor([M, N], X), api.Tensor([1, M], np.ones(M))
    tx.set_grad(gx0)
    cols = ones.matmul(tx)
    cols.mul(api.Tensor([1, N], seed_cols)).sum().backward()
    out.update(col_sums=cols.data().reshape(N), col_sums_gx=tx.grad().reshape(M, N))
    return out


def mse_case(api, rng):
    pred = rng.standard_normal((1, 10))
    target = np.zeros((1, 10))
    target[0, 3] = 1.0
    tp, tt = api.Tensor([1, 10], pred), api.Tensor([1, 10], target)
    loss = api.mse_loss(tp, tt)
    loss.backward()
    return dict(pred=pred, target=target, loss=loss.data(), gpred=tp.grad().reshape(1, 10),
                gtarget=tt.grad().reshape(1, 10))


def mlp_case(rng):
    """Benchmark config 1: 784-128-64-10, batch 32, one SGD step, lr 0.01."""
    sizes = [784, 128, 64, 10]
    batch = 32
    params = [(rng.standard_normal((i, o)) / np.sqrt(i), np.zeros(o))
              for i, o in zip(sizes[:-1], sizes[1:])]
    X = rng.random((batch, 784))
    y = rng.integers(0, 10, batch).astype(np.int32)
    work = [(W.copy(), b.copy()) for W, b in params]
    loss, grads, gX = oracle.mlp_train_step_true(work, X, y, 0.01)
    out = dict(X=X, y=y, loss=np.float64(loss), gX=gX)
    for i, ((W, b), (gW, gb), (W1, b1)) in enumerate(zip(params, grads, work)):
        # The updated parameters are W - lr*gW exactly (src/nn.cpp:74); a checksum of
        # them is enough to pin the SGD step without doubling the fixture size.
        out.update({f"W{i}": W, f"b{i}": b, f"gW{i}": gW, f"gb{i}": gb,
                    f"W{i}_new_sum": np.float64(oracle.fast.sum(W1.reshape(-1))),
                    f"b{i}_new": b1})
    return out


REFERENCE_MODEL = os.path.join(
    os.environ.get("MICROGRAD_REFERENCE") or os.path.join(os.path.dirname(os.path.dirname(os.path.dirname(HERE))), "reference"),
    "models", "mnist.bin")


def trainer_cases(api, rng):
    """The reference trainer's per-sample loop (src/main.cpp:20-46) on synthetic
    images: avg_pool -> Linear(196,100) -> relu -> Linear(100,10) -> mse_loss,
    host argmax, zero_grad, backward, SGD step lr 0.01 — two epochs over 24
    samples, starting from the weights of the reference's models/mnist.bin.
    Also plain inference with those weights on 64 images."""
    l1, l2 = api.Linear(196, 100), api.Linear(100, 10)
    api.load_model(REFERENCE_MODEL, l1, l2)
    out = {"W1": l1.weights().data().reshape(196, 100), "b1": l1.bias().data(),
           "W2": l2.weights().data().reshape(100, 10), "b2": l2.bias().data()}
    images = rng.random((64, 784))
    logits = []
    for i in range(64):
        x = api.Tensor([1, 784], images[i])
        logits.append(l2.forward(l1.forward(api.avg_pool_2x2(x)).relu()).data())
    out["infer_images"] = images
    out["infer_logits"] = np.array(logits)
    train_images = rng.random((24, 784))
    train_labels = rng.integers(0, 10, 24)
    opt = api.SGD([l1.weights(), l1.bias(), l2.weights(), l2.bias()], 0.01)
    losses, preds = [], []
    for epoch in range(2):
        for i in range(24):
            onehot = np.zeros(10)
            onehot[train_labels[i]] = 1.0
            x = l1.forward(api.avg_pool_2x2(api.Tensor([1, 784], train_images[i]))).relu()
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
    out.update(train_images=train_images, train_labels=train_labels, losses=np.array(losses),
               preds=np.array(preds), W1_final=l1.weights().data().reshape(196, 100),
               b1_final=l1.bias().data(), W2_final=l2.weights().data().reshape(100, 10),
               b2_final=l2.bias().data())
    return out


def main():
    api = oracle.ref_true()
    rng = np.random.default_rng(20240611)
    np.savez(os.path.join(HERE, "elementwise.npz"), **elementwise_cases(api, rng))
    np.savez(os.path.join(HERE, "matmul_sum.npz"), **matmul_cases(api, rng))
    np.savez(os.path.join(HERE, "mse.npz"), **mse_case(api, rng))
    np.savez(os.path.join(HERE, "mlp_c1.npz"), **mlp_case(rng))
    np.savez(os.path.join(HERE, "trainer_mnist_bin.npz"), **trainer_cases(api, rng))
    # separate generator: adding cases must not shift the stream the files above were drawn from
    np.savez(os.path.join(HERE, "axis_sums.npz"), **axis_sum_cases(api, np.random.default_rng(20240612)))
    for f in sorted(os.listdir(HERE)):
        if f.endswith(".npz"):
            print(f, os.path.getsize(os.path.join(HERE, f)), "bytes")


if __name__ == "__main__":
    main()
