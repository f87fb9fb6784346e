"""Parity at the shapes the benchmark times, not only at toy sizes.

* the GPT-2-small-shaped model (12 layers, d_model 768, 12 heads, ctx 1024, vocab
  50257 tied, loss scale 4096, non-zero biases) at batch 1: loss, every gradient
  tensor and one AdamW step against the rounding-faithful CPU oracle;
* the 24-layer d_model 1024 / 16 heads shape at 2 layers;
* every case of the GEMM-trio microbench (M in {4096, 16384} x four (K, N) x Y / dX / dW)
  and the three vocabulary-sized GEMMs of the tied head on CTA-pair tiles, against
  the fp32 matmul of the widened fp16 operands (kernels.py:606-610, tolerance of
  test_kernels.py:34);
* the reference's in-process data parallelism: two replicas adding into one arena,
  sum of two workers, weights bit-identical afterwards (examples/ddp_mnist.py:79-105,
  test_shared.py:109-145);
* autotune_matmul: the tuned configuration is correct and its cache round-trips
  (test_kernels.py:103-118, kernels.py:459-466, 594-596).
"""

import json
import os
import sys

import numpy as np
import pytest

sys.path.insert(0, os.path.join(os.path.dirname(__file__), "golden"))
import make_golden as mg  # noqa: E402
from oracle import vkgrad_numpy as orc  # noqa: E402
from test_transformer_gpu import expected, load_params, model_grads, relerr, shared  # noqa: E402

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _report(name, payload):
    """Leave the measured errors in the folder VKG_TEST_REPORT_DIR names, when it is set."""
    out = os.environ.get("VKG_TEST_REPORT_DIR")
    if out and os.path.isdir(out):
        with open(os.path.join(out, f"parity_{name}.json"), "w") as f:
            json.dump(payload, f, indent=1, sort_keys=True)


def _gpt_step_case(dev, name, B, T, D, H, L, V, loss_scale, seed):
    from vkgrad_b200.autograd import AdamW
    from vkgrad_b200.dataparallel import DataParallelStep, Replica
    from vkgrad_b200.transformer import GPT, TCtx
    Vp = (V + 15) // 16 * 16
    P = orc.make_gpt_params(D, H, L, T, Vp, seed=seed, std=0.02, bias_std=0.02, tie=True)
    rng = np.random.default_rng(seed + 100)
    ids = rng.integers(0, V, B * T).astype(np.uint32)
    tgt = rng.integers(0, V, B * T).astype(np.uint32)
    lr, wd = 6e-4, 0.01

    def build(d):
        ctx = TCtx(d)
        model = GPT(ctx, B, T, D, H, L, V, tie=True, loss_scale=loss_scale)
        load_params(model, P)
        opt = AdamW(ctx, model.params(), lr=lr, wd=wd)
        return ctx, model, opt, ctx.buf(B * T * 4, "shared"), ctx.buf(B * T * 4, "shared")

    rep = Replica(dev, build)
    try:
        model = rep.model
        assert model.blocks[0].attn.fused
        idb, tgb = shared(rep.ctx, ids), shared(rep.ctx, tgt)
        # gradients first (AdamW would be free to overwrite nothing, but keep the check clean)
        g = dev.graph(name)
        model.record(idb, tgb, g)
        g.finish()
        g.submit()
        loss = model.read_loss()
        got = model_grads(model)
        ref_loss, G, _ = orc.gpt_forward_backward(P, ids, tgt, B, T, D, H, L, V, faithful=True,
                                                  grad_scale=loss_scale / (B * T))
        exp = expected(mg.flatten_grads(G, L), True)
        assert set(exp) == set(got)
        errs = {k: relerr(got[k], exp[k].reshape(got[k].shape)) for k in exp}
        assert all(np.isfinite(v) for v in errs.values())
        worst = sorted(errs.items(), key=lambda kv: -kv[1])[:8]
        # one full recorded step: the same backward, then AdamW with 1/loss_scale folded in
        step = DataParallelStep(rep, idb, tgb, name=name + "_step")
        step_loss, _ = step(lr)
        chk = {}
        for key, prm, w0 in (("b0.fc1.W", model.blocks[0].fc1.W, P["b0"]["fc1.W"]),
                             (f"b{L - 1}.qkv.W", model.blocks[L - 1].attn.qkv.W,
                              P[f"b{L - 1}"]["qkv.W"]),
                             ("tok", model.tok, P["tok"]),
                             ("lnf.g", model.lnf.g, P["lnf.g"])):
            gg = prm.grad_numpy()
            w_ref, _, _, _ = orc.adamw_step(w0, gg, 0 * gg, 0 * gg, 1, lr=lr,
                                            wd=wd if w0.ndim == 2 else 0.0,
                                            gscale=1.0 / loss_scale)
            chk[key] = float(np.abs(prm.numpy() - w_ref).max())
        _report(name, {"loss": loss, "oracle_loss": ref_loss,
                       "loss_rel_err": abs(loss - ref_loss) / abs(ref_loss),
                       "worst_tensors": worst, "median_err": float(np.median(list(errs.values()))),
                       "adamw_max_abs_diff": chk})
        assert abs(loss - ref_loss) < 1e-3 * abs(ref_loss), (loss, ref_loss)
        assert abs(step_loss - loss) <= 1e-6 * abs(loss)
        # the bar for fp32-accumulated gradients: 1e-3 of each tensor's largest entry, every tensor
        assert max(errs.values()) < 1e-3, worst
        assert max(chk.values()) < 1e-6, chk
    finally:
        rep.destroy()


def test_gpt2_small_dims_step_against_faithful_oracle(dev):
    _gpt_step_case(dev, "gpt2_small_b1", 1, 1024, 768, 12, 12, 50257, 4096.0, seed=11)


def test_gpt_d1024_h16_dims_step_against_faithful_oracle(dev):
    _gpt_step_case(dev, "gpt_d1024_l2_b1", 1, 1024, 1024, 16, 2, 50257, 4096.0, seed=12)


def test_weighted_loss_keeps_the_static_loss_scale(dev):
    """Per-row loss weights and a static loss scale together: gradients carry exactly the
    factor S that AdamW's gradient scale divides out again."""
    from vkgrad_b200.transformer import GPT, TCtx
    cfg, P, ids, tgt, seg, w = mg.gpt_inputs("gpt_packed")
    grads = []
    for S in (1.0, 256.0):
        ctx = TCtx(dev)
        try:
            model = GPT(ctx, cfg["B"], cfg["T"], cfg["D"], cfg["H"], cfg["L"], cfg["vocab"],
                        tie=cfg["tie"], loss_scale=S)
            load_params(model, P)
            g = dev.graph("w")
            model.record(shared(ctx, ids), shared(ctx, tgt), g, seg=shared(ctx, seg),
                         weights=shared(ctx, w))
            g.finish()
            g.submit()
            grads.append(model.blocks[0].attn.qkv.W.grad_numpy())
        finally:
            ctx.destroy()
    assert np.abs(grads[1]).max() > 100 * np.abs(grads[0]).max()
    assert relerr(grads[1] / 256.0, grads[0]) < 2e-3


# ---- GEMM trio --------------------------------------------------------------------------------

TRIO = [(m, k, n) for m in (4096, 16384)
        for (k, n) in ((768, 768), (768, 3072), (3072, 768), (1024, 4096))]


def _upload16(dev, arr):
    from vkgrad_b200.vk import _check
    a = np.ascontiguousarray(arr, dtype=np.float16)
    buf = dev.buffer(a.nbytes, "device")
    _check(dev.lib.vkg_upload(dev.handle, buf.dptr, a.ctypes.data, a.nbytes), "upload")
    return buf


def _download32(dev, buf, shape):
    from vkgrad_b200.vk import _check
    out = np.empty(shape, np.float32)
    _check(dev.lib.vkg_download(dev.handle, out.ctypes.data, buf.dptr, out.nbytes), "download")
    return out


def _check_gemm(dev, a, b, m, n, k, ta, tb, **kw):
    from vkgrad_b200.kernels import gemm
    ba, bb = _upload16(dev, a), _upload16(dev, b)
    bc = dev.buffer(m * n * 4, "device")
    try:
        # poison: a tile that is never written shows up as NaN
        nan = np.full(1 << 20, np.nan, np.float32)
        for off in range(0, m * n * 4, nan.nbytes):
            dev.lib.vkg_upload(dev.handle, bc.dptr + off, nan.ctypes.data,
                               min(nan.nbytes, m * n * 4 - off))
        gemm(dev, ba, bb, bc, m, n, k, trans_a=ta, trans_b=tb, **kw)
        got = _download32(dev, bc, (m, n))
    finally:
        for x in (ba, bb, bc):
            x.destroy()
    ref = orc.matmul16(a, b, ta, tb)
    assert np.isfinite(got).all()
    return float(np.abs(got - ref).max() / max(np.abs(ref).max(), 1e-6))


@pytest.mark.parametrize("m,k,n", TRIO)
def test_gemm_trio_shapes_against_oracle(dev, m, k, n):
    rng = np.random.default_rng(m + k + n)
    x = rng.standard_normal((m, k)).astype(np.float16)
    dy = rng.standard_normal((m, n)).astype(np.float16)
    w = (rng.standard_normal((k, n)) * k ** -0.5).astype(np.float16)
    errs = {"Y": _check_gemm(dev, x, w, m, n, k, False, False),
            "dX": _check_gemm(dev, dy, w, m, k, n, False, True),
            "dW": _check_gemm(dev, x, dy, k, n, m, True, False)}
    assert max(errs.values()) < 2e-3, errs


@pytest.mark.parametrize("which", ["logits", "dh", "dtok"])
def test_vocabulary_sized_gemms_on_cta_pairs(dev, which):
    """The three GEMMs of the tied head at 8 x 1024 rows: 197 column tiles with a ragged last
    one (50272 = 196 * 256 + 96), on 256 x 256 CTA-pair tiles."""
    R, D, Vp = 8192, 768, 50272
    rng = np.random.default_rng(3)
    h = rng.standard_normal((R, D)).astype(np.float16)
    tok = (rng.standard_normal((Vp, D)) * 0.02).astype(np.float16)
    if which == "logits":
        err = _check_gemm(dev, h, tok, R, Vp, D, False, True, cta_pair=1)
    else:
        dl = (rng.standard_normal((R, Vp)) * 0.01).astype(np.float16)
        if which == "dh":
            err = _check_gemm(dev, dl, tok, R, D, Vp, False, False, cta_pair=1)
        else:
            err = _check_gemm(dev, dl, h, Vp, D, R, True, False, cta_pair=1)
    assert err < 2e-3, err


# ---- in-process replicas on one arena -----------------------------------------------------------

def test_two_replicas_one_arena_sum_and_no_drift(dev):
    from vkgrad_b200.autograd import MLP, AdamW, Ctx
    from vkgrad_b200.dataparallel import HostArena, Replica
    batch, sizes, ncls, pad = 64, (48, 32), 5, 16
    x, y, params = orc.make_mlp_case(2 * batch, sizes, ncls, pad, seed=4)

    def build(d):
        ctx = Ctx(d)
        model = MLP(ctx, batch, list(sizes), ncls, pad_classes=pad)
        for p, w in zip(model.params(), params):
            p.set(w)
        opt = AdamW(ctx, model.params(), lr=1e-2)
        return ctx, model, opt, ctx.buf(batch * sizes[0] * 2, "shared"), ctx.buf(batch * 4, "shared")

    n_params = sum(int(np.prod(w.shape)) for w in params)
    arena = HostArena(n_params)
    reps = [Replica(dev, build, arena) for _ in range(2)]
    try:
        assert all(np.array_equal(reps[0].params[0].numpy(), r.params[0].numpy()) for r in reps[1:])
        rng = np.random.default_rng(0)
        for step in range(3):
            idx = rng.permutation(2 * batch)
            reps[0].zero_arena()
            local = []
            for s, r in enumerate(reps):
                sl = idx[s * batch:(s + 1) * batch]
                r.xbuf.array(np.float16, (batch, sizes[0]))[:] = x[sl].astype(np.float16)
                r.ybuf.array(np.uint32, (batch,))[:] = y[sl]
                r.model.forward_backward(r.xbuf, r.ybuf)
                local.append([p.grad_numpy().copy() for p in r.params])
                r.push_gradients()
            dev.sync()
            # the arena holds the two workers' sum, tensor by tensor at the bucket offsets
            tmp = dev.buffer(reps[0].total * 4, "cached")
            dev.copy(reps[0].arena_buf, tmp, reps[0].total * 4)
            tmp.invalidate()
            flat = tmp.array(np.float32).copy()
            tmp.destroy()
            for i, (p, off) in enumerate(zip(reps[0].params, reps[0].offsets)):
                want = (local[0][i] + local[1][i]).ravel()
                assert np.array_equal(flat[off:off + p.n], want), p.name
            for r in reps:
                r.step_from_arena(1e-2, n_workers=2)
            # the update used the mean of the two workers
            for i, p in enumerate(reps[0].params):
                assert np.allclose(p.grad_numpy(), (local[0][i] + local[1][i]) * 0.5, rtol=0, atol=1e-7)
        drift = 0.0
        for r in reps[1:]:
            for a, b in zip(reps[0].params, r.params):
                drift = max(drift, float(np.abs(a.numpy() - b.numpy()).max()))
        assert drift == 0.0
        assert not np.array_equal(reps[0].params[0].numpy(), params[0])     # and they did move
    finally:
        for r in reps:
            r.destroy()
        arena.destroy()


# ---- autotune -------------------------------------------------------------------------------------

def test_autotune_matmul_is_correct_and_caches(dev, tmp_path, monkeypatch):
    from vkgrad_b200 import kernels
    monkeypatch.setattr(kernels, "_TUNE_CACHE", str(tmp_path / "autotune.json"))
    m = n = k = 512
    mm, best = kernels.autotune_matmul(dev, m, n, k, use_cache=True)
    assert best["tflops"] > 0 and best["evaluated"] >= 1 and best["tile"][0] == 128
    assert best["tile"][1] in kernels.TILE_N_CHOICES and mm.tile_n == best["tile"][1]
    rng = np.random.default_rng(1)
    a = rng.standard_normal((m, k)).astype(np.float16)
    b = rng.standard_normal((k, n)).astype(np.float16)
    ba, bb, bc = _upload16(dev, a), _upload16(dev, b), dev.buffer(m * n * 4, "device")
    try:
        mm(ba, bb, bc, m, n, k)
        got = _download32(dev, bc, (m, n))
    finally:
        for t in (ba, bb, bc):
            t.destroy()
    ref = kernels.matmul_reference(a, b)
    assert np.abs(got - ref).max() / np.abs(ref).max() < 2e-3
    # the cache file has the reference's schema and answers the second call without timing
    with open(kernels._TUNE_CACHE) as f:
        cache = json.load(f)
    (key, entry), = cache.items()
    assert f"{m}x{n}x{k}" in key and dev.name in key
    assert {"config", "lds", "tflops", "ms", "tile", "group_m", "evaluated", "pruned"} <= set(entry)
    monkeypatch.setattr(kernels, "warmup", lambda *a, **k: pytest.fail("cache was not used"))
    mm2, again = kernels.autotune_matmul(dev, m, n, k, use_cache=True)
    assert again == entry and mm2.tile_n == mm.tile_n
