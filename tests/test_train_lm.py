"""Gradient accumulation, evaluation and checkpoints of the language-model driver
(reference: test_accum.py over examples/train_lm.py and dataparallel.GradAccum).

Accumulating N microbatches of B rows and stepping once must give the gradient of one
batch of N*B rows; evaluation must train nothing; a resumed run must continue as the
uninterrupted one would."""

import json
import os
import sys

import numpy as np
import pytest

sys.path.insert(0, os.path.join(os.path.dirname(__file__), "golden"))
import make_golden as mg  # noqa: E402
from vkgrad_b200 import train_lm  # noqa: E402

GOLD = os.path.join(os.path.dirname(__file__), "golden")


# ---- CPU ---------------------------------------------------------------------------------

def test_encode_against_reference_fixture():
    gold = np.load(os.path.join(GOLD, "lm_encode.npz"))
    data = mg.lm_bytes()
    assert gold["data_digest"][0] == mg.digest(data)
    ids, itos = train_lm.encode(data, 48)
    assert ids.dtype == np.uint16 and np.array_equal(ids, gold["ids"])
    assert sorted(itos) == gold["itos_ids"].tolist()
    assert [ord(itos[k]) for k in sorted(itos)] == gold["itos_chars"].tolist()
    assert ids.max() == 47 and len(itos) == 47          # the last id is "everything else"


def test_warmup_schedule():
    assert train_lm.lr_at(1, 6e-4, 200) == pytest.approx(3e-6)
    assert train_lm.lr_at(100, 6e-4, 200) == pytest.approx(3e-4)
    assert train_lm.lr_at(200, 6e-4, 200) == train_lm.lr_at(5000, 6e-4, 200) == 6e-4
    assert train_lm.lr_at(1, 1e-3, 0) == 1e-3


def test_synthetic_corpus_is_seeded_and_predictable():
    a, b = train_lm.synthetic_corpus(4096, seed=1), train_lm.synthetic_corpus(4096, seed=1)
    assert a.dtype == np.uint8 and np.array_equal(a, b)
    assert not np.array_equal(a, train_lm.synthetic_corpus(4096, seed=2))
    assert a.min() >= 32 and a.max() < 96


class _HostParam:
    def __init__(self, shape):
        self.shape, self.n, self.name, self.value = shape, int(np.prod(shape)), "p", None

    def set(self, arr):
        self.value = np.array(arr, np.float32)


def test_weights_only_checkpoint_is_accepted(tmp_path):
    """The reference's checkpoints hold p<i> and step only (train_lm.py:251-252)."""
    path = str(tmp_path / "ckpt.npz")
    w = [np.arange(6, dtype=np.float32).reshape(2, 3), np.ones(4, np.float32)]
    np.savez(path, step=17, p0=w[0], p1=w[1].reshape(2, 2))
    params = [_HostParam((2, 3)), _HostParam((4,))]
    assert train_lm.load_checkpoint(path, params) == 17
    assert np.array_equal(params[0].value, w[0]) and params[1].value.shape == (4,)
    with pytest.raises(ValueError, match="needs 5"):
        train_lm.load_checkpoint(path, [_HostParam((2, 3)), _HostParam((5,))])
    with pytest.raises(ValueError, match="more tensors"):
        train_lm.load_checkpoint(path, params[:1])


# ---- GPU: accumulation == one large batch (test_accum.py:21-70, 139-170) -------------------

def _arena(dev, ctx, ga):
    tmp = ctx.buf(ga.total * 4, "cached")
    dev.copy(ga.arena, tmp, ga.total * 4)
    tmp.invalidate()
    return tmp.array(np.float32, (ga.total,)).copy()


def _accumulated_gradients(dev, batch, accum, data, labels, in_f, hidden, n_cls, dirty=False):
    from vkgrad_b200.autograd import AdamW, Ctx, MLP
    from vkgrad_b200.dataparallel import GradAccum
    ctx = Ctx(dev)
    try:
        model = MLP(ctx, batch, [in_f, hidden], n_cls, pad_classes=16)
        params = list(model.params())
        opt = AdamW(ctx, params, lr=1e-3)
        rng = np.random.default_rng(7)
        for p in params:
            p.set(rng.standard_normal(p.shape).astype(np.float32) * 0.05)
        ga = GradAccum(ctx, params, accum=accum)
        xb, yb = ctx.buf(batch * in_f * 2, "shared"), ctx.buf(batch * 4, "shared")
        xv, yv = xb.array(np.float16, (batch, in_f)), yb.array(np.uint32, (batch,))
        if dirty:   # stale values, as reused device memory would hold
            src = ctx.buf(ga.total * 4, "shared")
            src.array(np.float32, (ga.total,))[:] = \
                np.random.default_rng(11).standard_normal(ga.total)
            src.flush()
            dev.copy(src, ga.arena, ga.total * 4)
            assert np.abs(_arena(dev, ctx, ga)).max() > 0.5
        gmicro, _ = train_lm.accum_graphs(dev, model, opt, ga, xb, yb)
        for i in range(accum):
            xv[:] = data[i * batch:(i + 1) * batch]
            yv[:] = labels[i * batch:(i + 1) * batch]
            xb.flush()
            yb.flush()
            gmicro.submit()
        return _arena(dev, ctx, ga)
    finally:
        ctx.destroy()


@pytest.mark.gpu
def test_accumulation_equals_one_large_batch(dev):
    in_f, hidden, n_cls, total = 64, 32, 8, 64
    rng = np.random.default_rng(3)
    data = rng.standard_normal((total, in_f)).astype(np.float16)
    labels = rng.integers(0, n_cls, total).astype(np.uint32)
    ref = _accumulated_gradients(dev, total, 1, data, labels, in_f, hidden, n_cls)
    assert np.abs(ref).max() > 0
    for accum, dirty in ((2, False), (4, False), (4, True)):
        got = _accumulated_gradients(dev, total // accum, accum, data, labels, in_f, hidden,
                                     n_cls, dirty=dirty)
        # each microbatch's loss is a mean over its own rows, so the sum is accum times
        # the large batch's gradient (test_accum.py:158-161)
        err = np.abs(got / accum - ref).max() / np.abs(ref).max()
        assert err < 2e-3, (accum, dirty, err)


@pytest.mark.gpu
def test_evaluation_trains_nothing(dev):
    """test_accum.py:73-136: the evaluation graph leaves weights and arena alone and reports
    the training forward's loss; the training graphs, submitted instead, do move them."""
    from vkgrad_b200.autograd import AdamW
    from vkgrad_b200.dataparallel import GradAccum
    from vkgrad_b200.transformer import GPT, TCtx
    B, T, D, H, L, V = 2, 16, 32, 2, 2, 16
    rows = B * T
    ctx = TCtx(dev)
    try:
        model = GPT(ctx, B, T, D, H, L, V)
        params = list(model.params())
        opt = AdamW(ctx, params, lr=6e-4, wd=0.01)
        idb, tgb = ctx.buf(rows * 4, "shared"), ctx.buf(rows * 4, "shared")
        idv, tgv = idb.array(np.uint32, (rows,)), tgb.array(np.uint32, (rows,))
        gtrain = dev.graph("train")
        model.record(idb, tgb, gtrain)
        opt.record(gtrain)
        gtrain.finish()
        ga = GradAccum(ctx, params, accum=2)
        gmicro, gstep = train_lm.accum_graphs(dev, model, opt, ga, idb, tgb)
        geval = train_lm.eval_graph(dev, model, idb, tgb)
        opt.advance(6e-4)
        rng = np.random.default_rng(5)
        batches = [(rng.integers(0, V, rows).astype(np.uint32),
                    rng.integers(0, V, rows).astype(np.uint32)) for _ in range(3)]

        def state():
            return [p.numpy().copy() for p in params], _arena(dev, ctx, ga)

        def run(g):
            w0, a0 = state()
            loss = train_lm.evaluate(g, model, idv, tgv, batches)
            w1, a1 = state()
            return (loss, max(float(np.abs(x - y).max()) for x, y in zip(w0, w1)),
                    float(np.abs(a1 - a0).max()))

        loss, dw, da = run(geval)
        assert dw == 0 and da == 0
        ref, dw_micro, da_micro = run(gmicro)
        assert dw_micro == 0 and da_micro > 0
        assert abs(loss - ref) <= 1e-6 * abs(ref)
        _, dw_train, _ = run(gtrain)
        assert dw_train > 0
        # the step graph applies the sum and leaves a zeroed arena behind
        opt.advance(6e-4)
        w0, _ = state()
        gstep.submit()
        w1, a1 = state()
        assert max(float(np.abs(x - y).max()) for x, y in zip(w0, w1)) > 0
        assert not a1.any()
    finally:
        ctx.destroy()


# ---- GPU: the run loop, its log and its checkpoints --------------------------------------

def _tokens(vocab=48):
    ids, _ = train_lm.encode(train_lm.synthetic_corpus(1 << 16, seed=4, order=1), vocab)
    return ids[:60000], ids[60000:]


def _trainer(dev, accum=1, **kw):
    tr_tok, va_tok = _tokens()
    return train_lm.Trainer(dev, tr_tok, va_tok, 48, dmodel=64, layers=2, heads=2, seq=64,
                            batch=4, accum=accum, lr=3e-3, warmup_steps=10, **kw)


@pytest.mark.gpu
@pytest.mark.parametrize("accum", [1, 2])
def test_run_loop_learns_and_logs(dev, tmp_path, accum):
    tr = _trainer(dev, accum)
    try:
        first = tr.val_loss(4)
        assert abs(first - np.log(48)) < 0.5          # untrained: close to uniform
        recs = train_lm.train(tr, minutes=2.0, eval_every=40, max_steps=120,
                              log_path=str(tmp_path / "log.jsonl"),
                              ckpt_path=str(tmp_path / "ckpt.npz"), out=lambda s: None)
        assert [r["step"] for r in recs] == [40, 80, 120]
        assert recs[-1]["val"] < first - 0.3 and recs[-1]["train"] < recs[0]["train"]
        assert recs[-1]["tokens"] == 120 * 4 * 64 * accum
        lines = [json.loads(x) for x in (tmp_path / "log.jsonl").read_text().splitlines()]
        assert lines == recs
        assert set(lines[0]) == {"step", "train", "val", "tokens", "elapsed", "tok_per_s"}
        z = np.load(str(tmp_path / "ckpt.npz"))
        assert int(z["step"]) == 120 and int(z["opt_t"]) == 120
        assert f"m{len(tr.params) - 1}" in z and f"p{len(tr.params)}" not in z
    finally:
        tr.destroy()


@pytest.mark.gpu
def test_resume_continues_the_uninterrupted_run(dev, tmp_path):
    ckpt = str(tmp_path / "ckpt.npz")
    weights_only = str(tmp_path / "weights.npz")

    def finish(tr):
        tr.rng = np.random.default_rng(99)       # the same batches after the save point
        for _ in range(10):
            tr.step()
        return [p.numpy().copy() for p in tr.params]

    tr = _trainer(dev)
    try:
        for _ in range(10):
            tr.step()
        tr.save(ckpt)
        z = np.load(ckpt)
        np.savez(weights_only, step=z["step"], **{k: z[k] for k in z.files if k.startswith("p")})
        straight = finish(tr)
    finally:
        tr.destroy()

    def resumed(path):
        t2 = _trainer(dev)
        try:
            assert t2.resume(path) == 10
            return finish(t2), t2.opt.t
        finally:
            t2.destroy()

    full, t_full = resumed(ckpt)
    bare, _ = resumed(weights_only)
    assert t_full == 20
    saved = [z[f"p{i}"] for i in range(len(straight))]
    norm = lambda xs, ys: float(np.sqrt(sum(float(((x - y) ** 2).sum()) for x, y in zip(xs, ys))))
    moved = norm(straight, saved)
    assert moved > 0
    # Not bit for bit: float atomics in the embedding gradient change low bits from run to run,
    # and AdamW turns rounding noise into +-lr moves where the true gradient is zero (the key
    # bias: softmax ignores a shift of every score in a row).  Measured against the distance
    # the ten steps moved the weights, the resumed run must land on the uninterrupted one.
    assert norm(full, straight) < 0.05 * moved, (norm(full, straight), moved)
    # without the moments the continued run is a different one
    assert norm(bare, straight) > 0.25 * moved, (norm(bare, straight), moved)
