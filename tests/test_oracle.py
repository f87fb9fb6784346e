"""The CPU oracle against the fixtures produced by the reference's own numpy code
(tests/golden/make_golden.py).  Runs without a GPU."""

import os
import sys

import numpy as np
import pytest

sys.path.insert(0, os.path.join(os.path.dirname(__file__), "golden"))
import make_golden as mg  # noqa: E402
from oracle import vkgrad_numpy as orc  # noqa: E402

GOLD = os.path.join(os.path.dirname(__file__), "golden")


def relerr(a, b):
    return float(np.abs(a - b).max() / max(np.abs(b).max(), 1e-8))


def test_matmul_against_reference_fixture():
    z = np.load(os.path.join(GOLD, "matmul.npz"))
    for i, (m, n, k, ta, tb) in enumerate(mg.MATMUL_CASES):
        a, b = mg.matmul_inputs(m, n, k, ta, tb)
        assert mg.digest(a, b) == z[f"c{i}_in"][0], "seeded inputs drifted from the fixture"
        c = orc.matmul16(a, b, ta, tb)
        assert np.array_equal(c[::7, ::5], z[f"c{i}_sample"])
        assert np.isclose(c.astype(np.float64).sum(), z[f"c{i}_sum"][0], rtol=1e-9, atol=1e-6)


def test_matmul_known_answer_k1024():
    """All-ones 64x64x1024 is exactly 1024 (test_kernels.py:69-100)."""
    z = np.load(os.path.join(GOLD, "matmul.npz"))
    c = orc.matmul16(np.ones((64, 1024), np.float16), np.ones((1024, 64), np.float16))
    assert c.min() == c.max() == 1024.0
    assert tuple(z["ones_k1024"]) == (1024.0, 1024.0)


@pytest.mark.parametrize("seed", range(5))
def test_mlp_against_reference_fixture(seed):
    z = np.load(os.path.join(GOLD, "mlp.npz"))
    x, y, params = mg.mlp_inputs(seed=seed)
    assert mg.digest(x, y, *params) == z[f"s{seed}_in"][0]
    loss, grads = orc.mlp_forward_backward(x, params, y, 4)
    assert abs(loss - z[f"s{seed}_loss"][0]) < 1e-6
    for g, nm in zip(grads, ("dW1", "db1", "dW2", "db2")):
        assert relerr(g, z[f"s{seed}_{nm}"]) < 1e-5, nm


def test_mlp_against_hetero_cpu_worker():
    """examples/hetero_mnist.py:cpu_backward is a second statement of the same model."""
    z = np.load(os.path.join(GOLD, "mlp.npz"))
    x, y, params = mg.mlp_inputs(seed=0)
    loss, grads = orc.mlp_forward_backward(x, params, y, 4)
    assert abs(loss - z["hetero_loss"][0]) < 1e-6
    for g, nm in zip(grads, ("dW1", "db1", "dW2", "db2")):
        assert relerr(g, z[f"hetero_{nm}"]) < 1e-5, nm


@pytest.mark.parametrize("name", list(mg.GPT_CASES))
def test_gpt_against_reference_fixture(name):
    z = np.load(os.path.join(GOLD, f"{name}.npz"))
    cfg, P, ids, tgt, seg, w = mg.gpt_inputs(name)
    assert mg.digest(ids, tgt, P["tok"], P["b0"]["qkv.W"]) == z["inputs_digest"][0]
    loss, G, _ = orc.gpt_forward_backward(P, ids, tgt, cfg["B"], cfg["T"], cfg["D"], cfg["H"],
                                          cfg["L"], cfg["vocab"], seg=seg, weights=w)
    assert abs(loss - z["loss"][0]) <= 2e-6 * abs(z["loss"][0])
    flat = mg.flatten_grads(G, cfg["L"])
    assert set(flat) == set(z.files) - {"loss", "inputs_digest"}
    for k, v in flat.items():
        assert relerr(v, z[k]) < 2e-5, k


def test_faithful_mode_stays_close_to_fp32():
    """Rounding at the fp16 storage points moves results by ~1e-3, not more."""
    cfg, P, ids, tgt, seg, w = mg.gpt_inputs("gpt_tied")
    a = orc.gpt_forward_backward(P, ids, tgt, cfg["B"], cfg["T"], cfg["D"], cfg["H"], cfg["L"],
                                 cfg["vocab"])
    b = orc.gpt_forward_backward(P, ids, tgt, cfg["B"], cfg["T"], cfg["D"], cfg["H"], cfg["L"],
                                 cfg["vocab"], faithful=True)
    assert abs(a[0] - b[0]) < 5e-3 * abs(a[0])
    fa, fb = mg.flatten_grads(a[1], cfg["L"]), mg.flatten_grads(b[1], cfg["L"])
    worst = max(relerr(fb[k], fa[k]) for k in fa)
    assert 0 < worst < 3e-2


def test_adamw_matches_scalar_restatement():
    """AdamW has no numpy twin in the reference; check the vector form against a
    scalar transcription of the shader body (kernels.py:836-850)."""
    rng = np.random.default_rng(3)
    n = 64
    w = rng.standard_normal(n).astype(np.float32)
    g = rng.standard_normal(n).astype(np.float32)
    m = (0.1 * rng.standard_normal(n)).astype(np.float32)
    v = np.abs(0.01 * rng.standard_normal(n)).astype(np.float32)
    lr, b1, b2, eps, wd, t = 1e-3, 0.9, 0.999, 1e-8, 0.01, 3
    w2, m2, v2, w16 = orc.adamw_step(w, g, m, v, t, lr, b1, b2, eps, wd)
    bc1, bc2 = 1 - b1 ** t, 1 - b2 ** t
    for i in range(n):
        mi = b1 * float(m[i]) + (1 - b1) * float(g[i])
        vi = b2 * float(v[i]) + (1 - b2) * float(g[i]) ** 2
        wi = float(w[i])
        wi -= lr * ((mi / bc1) / (np.sqrt(vi / bc2) + eps) + wd * wi)
        assert abs(m2[i] - mi) < 1e-6 and abs(v2[i] - vi) < 1e-7
        assert abs(w2[i] - wi) < 2e-6
    assert w16.dtype == np.float16
    assert orc.adamw_bias_corrections(0) == orc.adamw_bias_corrections(1)


def test_dp_reduce_is_mean_of_workers():
    gs = [np.full(8, float(i + 1), np.float32) for i in range(4)]
    assert np.allclose(orc.dp_reduce(gs), 2.5)


def test_softmax_ce_masks_padding_and_zero_weights():
    rng = np.random.default_rng(0)
    logits = rng.standard_normal((6, 16)).astype(np.float32)
    labels = rng.integers(0, 10, 6)
    loss, g = orc.softmax_ce(logits, labels, 10)
    assert np.all(g[:, 10:] == 0)
    assert np.allclose(g.sum(axis=1), 0, atol=1e-6)
    w = np.array([1, 0, 2, 0, 1, 1], np.float32)
    loss_w, gw = orc.softmax_ce(logits, labels, 10, weights=w)
    assert np.all(loss_w[w == 0] == 0) and np.all(gw[w == 0] == 0)
    assert np.allclose(gw[2], g[2] * 6 * 2, rtol=1e-5)
