"""Language-model training driver pieces (reference: examples/train_lm.py).

`accum_graphs`, `eval_graph`, `evaluate` and `encode` keep the reference's names and
behaviour; the run loop is `train()`.  Additions the reference's script lacks: the
checkpoint also carries the Adam moments and the optimiser's step count
(the reference saves weights only, train_lm.py:251-252, so a resumed run restarts its
moment estimates), and the corpus may be synthetic (the reference reads the Python
standard library's sources, train_lm.py:37-57; any uint8 array works here).

  python -m vkgrad_b200.train_lm --minutes 1 --dmodel 128 --layers 2 --heads 2
"""

import argparse
import json
import os
import time

import numpy as np

from .autograd import AdamW
from .dataparallel import GradAccum
from .transformer import GPT, TCtx
from .vk import Device


# ---- corpus ------------------------------------------------------------------------------

def synthetic_corpus(n_bytes=1 << 20, seed=0, order=2):
    """A byte stream with learnable structure, standing in for the text corpus of
    train_lm.py:37-57: a random Markov chain over 64 printable symbols whose context is the
    last `order` (1 or 2) symbols; the favoured successor is taken 85 % of the time."""
    rng = np.random.default_rng(seed)
    mask = 64 ** order - 1
    successors = rng.integers(0, 64, (mask + 1, 4)).astype(np.int64)
    choice = np.where(rng.random(n_bytes) < 0.85, 0, rng.integers(0, 4, n_bytes))
    out = np.empty(n_bytes, np.uint8)
    state = 0
    for i in range(n_bytes):
        s = successors[state, choice[i]]
        out[i] = 32 + s
        state = (state * 64 + s) & mask
    return out


def encode(data, vocab):
    """The vocab-1 most frequent bytes get ids in byte order, everything else shares the
    last id (train_lm.py:60-67).  Returns (ids uint16, {id: character})."""
    counts = np.bincount(np.asarray(data, np.uint8), minlength=256)
    kept = np.sort(np.argsort(-counts)[:vocab - 1])
    lut = np.full(256, vocab - 1, np.uint16)
    lut[kept] = np.arange(len(kept), dtype=np.uint16)
    return lut[data], {int(lut[b]): chr(int(b)) for b in kept}


def lr_at(step, base_lr, warmup_steps):
    """Linear warm-up to base_lr over warmup_steps steps, flat after (train_lm.py:220)."""
    return base_lr * min(1.0, step / max(warmup_steps, 1))


# ---- graphs ------------------------------------------------------------------------------

def accum_graphs(dev, model, opt, ga, idb, tgb):
    """(microbatch graph, step graph) for gradient accumulation (train_lm.py:70-88).

    The arena is device memory with stale contents, so it is zeroed here once before the
    first microbatch; the step graph zeroes it again after applying the sum."""
    gz = dev.graph("zero")
    ga.record_zero(gz)
    gz.finish()
    gz.submit()
    gmicro = dev.graph("micro")
    model.record(idb, tgb, gmicro)
    ga.record_push(gmicro)
    gmicro.finish()
    gstep = dev.graph("step")
    ga.record_apply(gstep, opt)
    ga.record_zero(gstep)
    gstep.finish()
    return gmicro, gstep


def eval_graph(dev, model, idb, tgb):
    """Forward and loss only: evaluation must not train (train_lm.py:91-101)."""
    g = dev.graph("eval")
    model.record(idb, tgb, g, backward=False)
    g.finish()
    return g


def evaluate(g, model, idv, tgv, batches):
    """Mean loss over (ids, targets) batches, one submit of g each (train_lm.py:104-111)."""
    total = 0.0
    for x, y in batches:
        idv[:] = x
        tgv[:] = y
        g.submit()
        total += model.read_loss()
    return total / len(batches)


# ---- checkpoints --------------------------------------------------------------------------

def _device_to_numpy(dev, buf, n):
    tmp = dev.buffer(n * 4, "cached")
    try:
        dev.copy(buf, tmp, n * 4)
        tmp.invalidate()
        return tmp.array(np.float32, (n,)).copy()
    finally:
        tmp.destroy()


def _numpy_to_device(dev, arr, buf):
    flat = np.ascontiguousarray(arr, np.float32).reshape(-1)
    tmp = dev.buffer(flat.nbytes, "cached")
    try:
        tmp.array(np.float32, flat.shape)[:] = flat
        tmp.flush()
        dev.copy(tmp, buf, flat.nbytes)
    finally:
        tmp.destroy()


def save_checkpoint(path, params, opt, step, extra=None):
    """npz with p<i> (weights, the reference's keys, train_lm.py:251-252), m<i> / v<i> (Adam
    moments), `step` and `opt_t`.  Written to a temporary name and renamed, so a run killed
    in the middle leaves the previous checkpoint intact."""
    dev = opt.ctx.dev
    blob = {"step": np.int64(step), "opt_t": np.int64(opt.t)}
    for i, p in enumerate(params):
        blob[f"p{i}"] = p.numpy().copy()
        blob[f"m{i}"] = _device_to_numpy(dev, p.m, p.n).reshape(p.shape)
        blob[f"v{i}"] = _device_to_numpy(dev, p.v, p.n).reshape(p.shape)
    for k, v in (extra or {}).items():
        blob[f"x_{k}"] = np.asarray(v)
    tmp = path + ".tmp.npz"
    np.savez(tmp, **blob)
    os.replace(tmp, path)


def load_checkpoint(path, params, opt=None):
    """Restore weights (and, when present and opt is given, moments and step count).
    A weights-only file, as the reference writes, is accepted.  Returns the step."""
    z = np.load(path)
    params = list(params)
    for i, p in enumerate(params):
        w = z[f"p{i}"]
        if w.size != p.n:
            raise ValueError(f"{path}: p{i} has {w.size} values, {p.name} needs {p.n}")
    if f"p{len(params)}" in z:
        raise ValueError(f"{path}: holds more tensors than the model")
    for i, p in enumerate(params):
        p.set(z[f"p{i}"].reshape(p.shape))
        if opt is not None and f"m{i}" in z:
            _numpy_to_device(opt.ctx.dev, z[f"m{i}"], p.m)
            _numpy_to_device(opt.ctx.dev, z[f"v{i}"], p.v)
    if opt is not None and "opt_t" in z:
        opt.t = int(z["opt_t"])
    return int(z["step"])


# ---- run loop -----------------------------------------------------------------------------

class Trainer:
    """Model, optimiser and recorded graphs of one training run; `step()` takes one
    optimiser step over `accum` microbatches drawn from `train_tokens`."""

    def __init__(self, dev, train_tokens, val_tokens, vocab, dmodel=384, layers=6, heads=6,
                 seq=256, batch=8, accum=1, lr=6e-4, warmup_steps=200, wd=0.01, seed=1234):
        self.dev, self.ctx = dev, TCtx(dev)
        self.B, self.T, self.accum = batch, seq, max(int(accum), 1)
        self.lr, self.warmup_steps = lr, warmup_steps
        self.train_tokens, self.val_tokens = train_tokens, val_tokens
        self.model = GPT(self.ctx, batch, seq, dmodel, heads, layers, vocab)
        self.params = list(self.model.params())
        self.opt = AdamW(self.ctx, self.params, lr=lr, wd=wd)
        rows = self.rows = batch * seq
        self.idb = self.ctx.buf(rows * 4, "shared")
        self.tgb = self.ctx.buf(rows * 4, "shared")
        self.idv = self.idb.array(np.uint32, (rows,))
        self.tgv = self.tgb.array(np.uint32, (rows,))
        self.ga = None
        if self.accum == 1:
            self.g = dev.graph("train")
            self.model.record(self.idb, self.tgb, self.g)
            self.opt.record(self.g)
            self.g.finish()
        else:
            self.ga = GradAccum(self.ctx, self.params, accum=self.accum)
            self.g, self.gstep = accum_graphs(dev, self.model, self.opt, self.ga, self.idb, self.tgb)
        self.geval = eval_graph(dev, self.model, self.idb, self.tgb)
        self.rng = np.random.default_rng(seed)
        self.step_no = 0

    def batch_from(self, tokens):
        starts = self.rng.integers(0, len(tokens) - self.T - 1, self.B)
        idx = starts[:, None] + np.arange(self.T)[None, :]
        return (tokens[idx].reshape(-1).astype(np.uint32),
                tokens[idx + 1].reshape(-1).astype(np.uint32))

    def step(self):
        """One optimiser step; returns (mean microbatch loss, tokens consumed)."""
        self.step_no += 1
        lr = lr_at(self.step_no, self.lr, self.warmup_steps)
        total = 0.0
        for _ in range(self.accum):
            self.idv[:], self.tgv[:] = self.batch_from(self.train_tokens)
            if self.accum == 1:
                self.opt.advance(lr)
            self.g.submit()
            total += self.model.read_loss()
        if self.accum > 1:
            self.opt.advance(lr)
            self.gstep.submit()
        return total / self.accum, self.rows * self.accum

    def val_loss(self, n_batches=20):
        return evaluate(self.geval, self.model, self.idv, self.tgv,
                        [self.batch_from(self.val_tokens) for _ in range(n_batches)])

    def save(self, path):
        save_checkpoint(path, self.params, self.opt, self.step_no)

    def resume(self, path):
        self.step_no = load_checkpoint(path, self.params, self.opt)
        return self.step_no

    def destroy(self):
        if self.ga:
            self.ga.destroy()
        self.ctx.destroy()


def train(trainer, minutes, eval_every, log_path=None, ckpt_path=None, max_steps=None, out=print):
    """Run for a wall-clock budget; every eval_every steps append one JSON line with the keys
    the reference logs (step, train, val, tokens, elapsed, tok_per_s; train_lm.py:236-245)
    and write the checkpoint.  Returns the list of records."""
    budget, t0 = minutes * 60.0, time.perf_counter()
    losses, records, tokens_done = [], [], 0
    log = open(log_path, "a", encoding="utf-8") if log_path else None
    try:
        while time.perf_counter() - t0 < budget and (max_steps is None or len(losses) < max_steps):
            loss, ntok = trainer.step()
            losses.append(loss)
            tokens_done += ntok
            if trainer.step_no % eval_every == 0:
                elapsed = time.perf_counter() - t0
                rec = {"step": trainer.step_no, "train": float(np.mean(losses[-eval_every:])),
                       "val": trainer.val_loss(), "tokens": tokens_done, "elapsed": elapsed,
                       "tok_per_s": tokens_done / elapsed}
                records.append(rec)
                out(f"{rec['step']:7d}{rec['train']:9.4f}{rec['val']:9.4f}{rec['tok_per_s']:12,.0f}")
                if log:
                    log.write(json.dumps(rec) + "\n")
                    log.flush()
                if ckpt_path:
                    trainer.save(ckpt_path)
    finally:
        if log:
            log.close()
    return records


def main(argv=None):
    ap = argparse.ArgumentParser(description=__doc__.split("\n")[0])
    ap.add_argument("--dmodel", type=int, default=384)
    ap.add_argument("--layers", type=int, default=6)
    ap.add_argument("--heads", type=int, default=6)
    ap.add_argument("--seq", type=int, default=256)
    ap.add_argument("--batch", type=int, default=8, help="microbatch size")
    ap.add_argument("--accum", type=int, default=1, help="microbatches per optimiser step")
    ap.add_argument("--vocab", type=int, default=96)
    ap.add_argument("--lr", type=float, default=6e-4)
    ap.add_argument("--warmup-steps", type=int, default=200)
    ap.add_argument("--minutes", type=float, default=20.0)
    ap.add_argument("--eval-every", type=int, default=250)
    ap.add_argument("--corpus", default=None, help=".npy of uint8; default: a synthetic stream")
    ap.add_argument("--out", default=None, help="run folder (log.jsonl, ckpt.npz)")
    ap.add_argument("--resume", default=None, help="run folder to continue")
    a = ap.parse_args(argv)

    tag = a.resume or a.out or os.path.join("runs", f"lm_{a.dmodel}x{a.layers}")
    os.makedirs(tag, exist_ok=True)
    ckpt = os.path.join(tag, "ckpt.npz")
    data = np.load(a.corpus) if a.corpus else synthetic_corpus()
    tokens, _ = encode(data, a.vocab)
    split = int(len(tokens) * 0.98)
    dev = Device()
    tr = Trainer(dev, tokens[:split], tokens[split:], a.vocab, a.dmodel, a.layers, a.heads,
                 a.seq, a.batch, a.accum, a.lr, a.warmup_steps)
    try:
        print(dev)
        print(f"model d={a.dmodel} L={a.layers} H={a.heads} seq={a.seq} batch={a.batch}: "
              f"{tr.model.n_params():,} params; {tr.g.n_dispatch} launches per microbatch")
        if a.resume and os.path.exists(ckpt):
            print(f"resumed from step {tr.resume(ckpt)}")
        print(f"{'step':>7}{'loss':>9}{'val':>9}{'tok/s':>12}")
        recs = train(tr, a.minutes, a.eval_every, os.path.join(tag, "log.jsonl"), ckpt)
        if recs:
            print(f"  loss {recs[0]['train']:.4f} -> {recs[-1]['train']:.4f}, val {recs[-1]['val']:.4f}; "
                  f"checkpoint {ckpt}")
    finally:
        tr.destroy()
        dev.destroy()


if __name__ == "__main__":
    main()
