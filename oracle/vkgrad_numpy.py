"""CPU oracle for the vkgrad training-step hot path (TEST INFRASTRUCTURE ONLY).

A numpy restatement of the arithmetic BrettKnox/vkgrad performs in one
training step, used only as the checker in tests/, in __graft_entry__.smoke()
and as the timed CPU baseline of bench.py.  Nothing in the vkgrad_b200 package
imports this module; the product path has no CPU fallback.

Parity is pinned: tests/golden/make_golden.py imports the reference's own numpy
functions (kernels.matmul_reference, test_autograd.numpy_forward_backward,
test_transformer.np_model, ...) behind a stub `vk` module, runs them on seeded
inputs and stores the results; tests/test_oracle.py checks every function here
against those stored results.  The AdamW, gradient-exchange and rounding rules
have no numpy twin in the reference and follow its GLSL, cited per function.

Two precisions:
  faithful=False  everything in fp32, like the reference's test oracles.
  faithful=True   values are rounded to fp16 wherever the GPU path stores fp16
                  (matmul operands, activations that feed a matmul, the logit
                  gradient), so a kernel bug is not hidden inside the 1e-2 gap
                  between fp32 and mixed precision.
"""

import numpy as np

SQRT_2_OVER_PI = np.float32(0.7978845608028654)
GELU_CUBIC = np.float32(0.044715)


def r16(x):
    """Round to fp16 and widen back: the storage rounding of an f16 buffer."""
    return np.asarray(x, dtype=np.float32).astype(np.float16).astype(np.float32)


def _maybe16(x, faithful):
    return r16(x) if faithful else np.asarray(x, dtype=np.float32)


# -- matmul (kernels.py:606-610) ------------------------------------------------

def matmul16(a, b, trans_a=False, trans_b=False):
    """fp16 operands widened to fp32, fp32 product: what every GEMM computes."""
    lhs = np.asarray(a, dtype=np.float32)
    rhs = np.asarray(b, dtype=np.float32)
    lhs = lhs.T if trans_a else lhs
    rhs = rhs.T if trans_b else rhs
    return lhs @ rhs


# -- activations (kernels.py:624-636) ---------------------------------------------

def gelu(x):
    x = np.asarray(x)
    inner = SQRT_2_OVER_PI * (x + GELU_CUBIC * x * x * x)
    return 0.5 * x * (1.0 + np.tanh(inner))


def dgelu(x):
    x = np.asarray(x)
    t = np.tanh(SQRT_2_OVER_PI * (x + GELU_CUBIC * x * x * x))
    return (0.5 * (1.0 + t)
            + 0.5 * x * (1.0 - t * t) * SQRT_2_OVER_PI * (1.0 + 3.0 * GELU_CUBIC * x * x))


def relu(x):
    return np.maximum(x, 0)


def drelu(x):
    return (np.asarray(x) > 0).astype(np.asarray(x).dtype)


ACTS = {"gelu": (gelu, dgelu), "relu": (relu, drelu)}


# -- softmax + cross entropy (kernels.py:766-827) ----------------------------------

def softmax_ce(logits, labels, n_cls, weights=None, grad_scale=None):
    """Per-row loss and the logit gradient.

    Columns >= n_cls are padding: masked out of the softmax, gradient exactly 0.
    Row gradient scale is 1/rows (kernels.py:780-785) unless per-row weights are
    given (kernels.py:800-827), in which case rows with weight 0 report loss 0.
    """
    logits = np.asarray(logits)
    rows = logits.shape[0]
    valid = logits[:, :n_cls]
    top = valid.max(axis=1, keepdims=True)
    log_z = top + np.log(np.exp(valid - top).sum(axis=1, keepdims=True))
    picked = valid[np.arange(rows), labels]
    loss_rows = log_z[:, 0] - picked
    grad = np.zeros_like(logits)
    grad[:, :n_cls] = np.exp(valid - log_z)
    grad[np.arange(rows), labels] -= 1.0
    if weights is None:
        scale = (1.0 / rows) if grad_scale is None else grad_scale
        grad[:, :n_cls] *= scale
    else:
        w = np.asarray(weights, dtype=logits.dtype)
        grad[:, :n_cls] *= w[:, None]
        loss_rows = np.where(w == 0, 0.0, loss_rows).astype(logits.dtype)
    return loss_rows, grad


# -- MLP step (autograd.py:159-293, test_autograd.py:21-46) ------------------------

def mlp_forward_backward(x, params, labels, n_cls, act="gelu", faithful=False):
    """Loss and gradients of MLP(sizes) with a linear head padded to params[-2].shape[1].

    params = [W0, b0, W1, b1, ..., Whead, bhead]; hidden layers use `act`.
    Returns (loss, [dW0, db0, ...]).  With one hidden layer and act='gelu' this is
    the reference's numpy_forward_backward.
    """
    fwd, bwd = ACTS[act]
    n_layers = len(params) // 2
    h = _maybe16(x, faithful)
    inputs, pre = [], []
    for i in range(n_layers):
        W, b = _maybe16(params[2 * i], faithful), np.asarray(params[2 * i + 1])
        inputs.append(h)
        z = h @ W + b
        pre.append(z)
        h = _maybe16(fwd(z), faithful) if i < n_layers - 1 else z
    loss_rows, dlog = softmax_ce(h, labels, n_cls)
    loss = float(loss_rows.mean())
    grads = [None] * len(params)
    g = dlog
    for i in reversed(range(n_layers)):
        if i < n_layers - 1:
            g = g * bwd(pre[i])
        g16 = _maybe16(g, faithful)
        grads[2 * i] = inputs[i].T @ g16
        grads[2 * i + 1] = g.sum(axis=0)
        if i > 0:
            g = g16 @ _maybe16(params[2 * i], faithful).T
    return loss, grads


# -- AdamW (kernels.py:832-851, schedule autograd.py:319-329) ----------------------

def adamw_bias_corrections(t, b1=0.9, b2=0.999):
    """bc1, bc2 for step t (t counts from 1; t=0 is clamped to 1)."""
    tt = max(int(t), 1)
    return 1.0 - b1 ** tt, 1.0 - b2 ** tt


def adamw_step(w, g, m, v, t, lr=1e-3, b1=0.9, b2=0.999, eps=1e-8, wd=0.01, gscale=1.0):
    """One fused update in fp32, returning (w, m, v, w16).

    m = b1 m + (1-b1) g ; v = b2 v + (1-b2) g^2 ;
    w -= lr * ((m/bc1) / (sqrt(v/bc2) + eps) + wd * w); w16 = fp16(w).
    gscale multiplies the gradient first (grad_pull's scale, dataparallel.py:69-73).
    """
    f = np.float32
    bc1, bc2 = adamw_bias_corrections(t, b1, b2)
    g = np.asarray(g, dtype=f) * f(gscale)
    m = f(b1) * np.asarray(m, dtype=f) + f(1.0 - f(b1)) * g
    v = f(b2) * np.asarray(v, dtype=f) + f(1.0 - f(b2)) * g * g
    mh = m / f(bc1)
    vh = v / f(bc2)
    w = np.asarray(w, dtype=f)
    w = w - f(lr) * (mh / (np.sqrt(vh) + f(eps)) + f(wd) * w)
    return w.astype(f), m.astype(f), v.astype(f), w.astype(np.float16)


# -- data-parallel exchange (dataparallel.py:40-73, 131-144) -------------------------

def dp_reduce(worker_grads):
    """Sum over workers then scale by 1/W: push (atomic add) followed by pull."""
    total = np.zeros_like(np.asarray(worker_grads[0], dtype=np.float32))
    for g in worker_grads:
        total = total + np.asarray(g, dtype=np.float32)
    return total * np.float32(1.0 / max(len(worker_grads), 1))


# -- layernorm (tkernels.py:32-88) --------------------------------------------------

def layernorm_fwd(x, gamma, beta, eps=1e-5):
    mean = x.mean(axis=-1, keepdims=True)
    centred = x - mean
    rstd = 1.0 / np.sqrt((centred * centred).mean(axis=-1, keepdims=True) + eps)
    xhat = centred * rstd
    return xhat * gamma + beta, xhat, rstd[..., 0]


def layernorm_bwd(dy, xhat, rstd, gamma):
    dxhat = dy * gamma
    a = dxhat.mean(axis=-1, keepdims=True)
    b = (dxhat * xhat).mean(axis=-1, keepdims=True)
    dx = rstd[:, None] * (dxhat - a - xhat * b)
    return dx, (dy * xhat).sum(axis=0), dy.sum(axis=0)


# -- GPT step (transformer.py:189-386, test_transformer.py:38-151) --------------------

def _heads(mat, B, T, H, hd):
    """(B*T, H*hd) -> (B, H, T, hd)"""
    return mat.reshape(B, T, H, hd).transpose(0, 2, 1, 3)


def _unheads(t, B, T, H, hd):
    """(B, H, T, hd) -> (B*T, H*hd)"""
    return t.transpose(0, 2, 1, 3).reshape(B * T, H * hd)


def gpt_forward_backward(P, ids, targets, B, T, D, H, n_layer, vocab, seg=None, weights=None,
                         faithful=False, grad_scale=None, want_grads=True):
    """Loss and all gradients of the pre-LN decoder.

    P: {"tok","pos","lnf.g","lnf.b","head.W","head.b", "b<i>": {ln1.g, ln1.b, ln2.g,
    ln2.b, qkv.W, qkv.b, proj.W, proj.b, fc1.W, fc1.b, fc2.W, fc2.b}}.  For a tied
    head pass head.W = tok.T and head.b = 0, and add G["head.W"].T to G["tok"]
    (test_transformer.py:185-192).  seg[b*T+t] is the start of token t's packed
    sample; weights are per-row loss weights.  Returns (loss, G, loss_rows).
    """
    R, hd = B * T, D // H
    q_ = (lambda a: r16(a)) if faithful else (lambda a: a)
    scale = np.float32(1.0 / np.sqrt(hd))
    ids = np.asarray(ids).astype(np.int64)
    targets = np.asarray(targets).astype(np.int64)
    tpos = np.arange(R) % T
    allowed = np.tril(np.ones((T, T), dtype=bool))[None, None]
    if seg is not None:
        seg = np.asarray(seg).astype(np.int64)
        tpos = tpos - seg
        allowed = allowed & (np.arange(T)[None, None, None, :] >= seg.reshape(B, 1, T, 1))

    x = P["tok"][ids] + P["pos"][tpos]
    saved = []
    for l in range(n_layer):
        p = P[f"b{l}"]
        c = {"x_in": x}
        y, c["xh1"], c["r1"] = layernorm_fwd(x, p["ln1.g"], p["ln1.b"])
        c["h"] = q_(y)
        c["qkv"] = q_(c["h"] @ q_(p["qkv.W"]) + p["qkv.b"])
        c["q"], c["k"], c["v"] = (_heads(c["qkv"][:, i * D:(i + 1) * D], B, T, H, hd)
                                  for i in range(3))
        s = (c["q"] @ c["k"].transpose(0, 1, 3, 2)) * scale
        s = np.where(allowed, s, np.float32(-1e30))
        e = np.exp(s - s.max(axis=-1, keepdims=True)) * allowed
        c["p"] = q_(e / e.sum(axis=-1, keepdims=True))
        c["ao"] = q_(_unheads(c["p"] @ c["v"], B, T, H, hd))
        c["res1"] = x + (c["ao"] @ q_(p["proj.W"]) + p["proj.b"])
        y2, c["xh2"], c["r2"] = layernorm_fwd(c["res1"], p["ln2.g"], p["ln2.b"])
        c["h2"] = q_(y2)
        c["z1"] = c["h2"] @ q_(p["fc1.W"]) + p["fc1.b"]
        c["hh"] = q_(gelu(c["z1"]))
        x = c["res1"] + (c["hh"] @ q_(p["fc2.W"]) + p["fc2.b"])
        saved.append(c)

    yf, xhf, rf = layernorm_fwd(x, P["lnf.g"], P["lnf.b"])
    hf = q_(yf)
    logits = hf @ q_(P["head.W"]) + P["head.b"]
    loss_rows, dlog = softmax_ce(logits, targets, vocab, weights=weights, grad_scale=grad_scale)
    if weights is None:
        loss = float(loss_rows.mean())
    else:
        loss = float((loss_rows * np.asarray(weights)).sum())
    if not want_grads:
        return loss, None, loss_rows
    dlog16 = q_(dlog)

    G = {"head.W": hf.T @ dlog16, "head.b": dlog.sum(axis=0)}
    d, G["lnf.g"], G["lnf.b"] = layernorm_bwd(dlog16 @ q_(P["head.W"]).T, xhf, rf, P["lnf.g"])
    for l in reversed(range(n_layer)):
        p, c, g = P[f"b{l}"], saved[l], {}
        d16 = q_(d)
        g["fc2.W"] = c["hh"].T @ d16
        g["fc2.b"] = d16.sum(axis=0)
        dz1 = q_((d16 @ q_(p["fc2.W"]).T) * dgelu(c["z1"]))
        g["fc1.W"] = c["h2"].T @ dz1
        g["fc1.b"] = dz1.sum(axis=0)
        dln2, g["ln2.g"], g["ln2.b"] = layernorm_bwd(dz1 @ q_(p["fc1.W"]).T, c["xh2"], c["r2"],
                                                    p["ln2.g"])
        dres1 = d + dln2
        dres1_16 = q_(dres1)
        g["proj.W"] = c["ao"].T @ dres1_16
        g["proj.b"] = dres1_16.sum(axis=0)
        dao = _heads(q_(dres1_16 @ q_(p["proj.W"]).T), B, T, H, hd)
        dv = c["p"].transpose(0, 1, 3, 2) @ dao
        dp = dao @ c["v"].transpose(0, 1, 3, 2)
        row_dot = (dp * c["p"]).sum(axis=-1, keepdims=True)
        ds = q_(c["p"] * (dp - row_dot) * scale)
        dq = ds @ c["k"]
        dk = ds.transpose(0, 1, 3, 2) @ c["q"]
        dqkv = q_(np.concatenate([_unheads(t, B, T, H, hd) for t in (dq, dk, dv)], axis=1))
        g["qkv.W"] = c["h"].T @ dqkv
        g["qkv.b"] = dqkv.sum(axis=0)
        dln1, g["ln1.g"], g["ln1.b"] = layernorm_bwd(dqkv @ q_(p["qkv.W"]).T, c["xh1"], c["r1"],
                                                    p["ln1.g"])
        d = dres1 + dln1
        G[f"b{l}"] = g

    G["pos"] = np.zeros_like(P["pos"])
    np.add.at(G["pos"], tpos, d)
    G["tok"] = np.zeros_like(P["tok"])
    np.add.at(G["tok"], ids, d)
    return loss, G, loss_rows


# -- seeded synthetic inputs for the benchmark configurations ---------------------------

def make_mlp_case(batch=256, sizes=(784, 256, 256), n_cls=10, pad=16, seed=0):
    """Inputs uniform[0,1) rounded to fp16, labels uniform, weights N(0, 1/sqrt(fan_in)),
    biases 0.1*N(0,1) (non-zero so a dropped bias add shows)."""
    rng = np.random.default_rng(seed)
    x = rng.random((batch, sizes[0]), dtype=np.float32).astype(np.float16)
    y = rng.integers(0, n_cls, batch).astype(np.uint32)
    dims = list(sizes) + [pad]
    params = []
    for fan_in, fan_out in zip(dims[:-1], dims[1:]):
        params.append((rng.standard_normal((fan_in, fan_out)) / np.sqrt(fan_in)).astype(np.float32))
        params.append((0.1 * rng.standard_normal(fan_out)).astype(np.float32))
    return x, y, params


def make_gpt_params(D, H, n_layer, T, pad_vocab, seed=0, std=0.02, bias_std=0.0, tie=True):
    """All weights N(0, std); LN gamma 1, beta 0; biases N(0, bias_std)."""
    rng = np.random.default_rng(seed)
    nrm = lambda *s: (rng.standard_normal(s) * std).astype(np.float32)
    bias = lambda n: (rng.standard_normal(n) * bias_std).astype(np.float32)
    P = {"tok": nrm(pad_vocab, D), "pos": nrm(T, D),
         "lnf.g": np.ones(D, np.float32), "lnf.b": bias(D)}
    for l in range(n_layer):
        P[f"b{l}"] = {
            "ln1.g": np.ones(D, np.float32), "ln1.b": bias(D),
            "ln2.g": np.ones(D, np.float32), "ln2.b": bias(D),
            "qkv.W": nrm(D, 3 * D), "qkv.b": bias(3 * D),
            "proj.W": nrm(D, D), "proj.b": bias(D),
            "fc1.W": nrm(D, 4 * D), "fc1.b": bias(4 * D),
            "fc2.W": nrm(4 * D, D), "fc2.b": bias(D)}
    if tie:
        P["head.W"] = P["tok"].T.copy()
        P["head.b"] = np.zeros(pad_vocab, np.float32)
    else:
        P["head.W"] = nrm(D, pad_vocab)
        P["head.b"] = bias(pad_vocab)
    return P


# -- GPT-2 forward from a Hugging Face state dict (test_hf_gpt2.py:33-66) ----------------

def gpt2_logits(W, H, ids):
    """Logits (n, vocab) of GPT-2 for one sequence of n token ids, straight from tensors
    under GPT2Model names (wte.weight, h.<i>.attn.c_attn.weight, ...): Conv1D is
    x @ weight + bias with weight (in, out); c_attn yields q, k, v in that order; a head is
    a contiguous slice of D/H columns; tanh GELU; layernorm eps 1e-5; the head is wte^T.
    Deliberately independent of the name mapping the package's loader uses."""
    ids = np.asarray(ids).astype(np.int64)
    n = len(ids)
    wte = np.asarray(W["wte.weight"], np.float64)
    D = wte.shape[1]
    hd = D // H
    get = lambda name: np.asarray(W[name], np.float64)
    norm = lambda x, name: layernorm_fwd(x, get(name + ".weight"), get(name + ".bias"))[0]
    lin = lambda x, name: x @ get(name + ".weight") + get(name + ".bias")
    causal = np.tril(np.ones((n, n), dtype=bool))
    x = wte[ids] + get("wpe.weight")[:n]
    i = 0
    while f"h.{i}.ln_1.weight" in W:
        pre = f"h.{i}."
        qkv = lin(norm(x, pre + "ln_1"), pre + "attn.c_attn")
        q, k, v = (qkv[:, j * D:(j + 1) * D].reshape(n, H, hd).transpose(1, 0, 2) for j in range(3))
        s = np.where(causal, (q @ k.transpose(0, 2, 1)) / np.sqrt(hd), -np.inf)
        p = np.exp(s - s.max(axis=-1, keepdims=True))
        p = p / p.sum(axis=-1, keepdims=True)
        x = x + lin((p @ v).transpose(1, 0, 2).reshape(n, D), pre + "attn.c_proj")
        x = x + lin(gelu(lin(norm(x, pre + "ln_2"), pre + "mlp.c_fc")), pre + "mlp.c_proj")
        i += 1
    return norm(x, "ln_f") @ wte.T


def perplexity(logits, ids):
    """exp(mean next-token cross entropy) of logits (n, vocab) on ids (n,)
    (test_hf_gpt2.py:69-73)."""
    lg = np.asarray(logits[:-1], np.float64)
    top = lg.max(axis=-1, keepdims=True)
    lse = top[:, 0] + np.log(np.exp(lg - top).sum(axis=-1))
    nxt = np.asarray(ids)[1:]
    return float(np.exp((lse - lg[np.arange(len(nxt)), nxt]).mean()))


def make_hf_gpt2_tensors(D, H, n_layer, n_ctx, vocab, seed=0, std=0.08, prefix="", dtype=np.float32):
    """A synthetic GPT-2 state dict under Hugging Face names (a stand-in for the real
    checkpoints, which are not available offline): weights N(0, std), layernorm gains
    1 + N(0, 0.1), biases N(0, 0.1); includes the attn.bias mask buffers real files carry."""
    rng = np.random.default_rng(seed)
    nrm = lambda *s, sd=std: (rng.standard_normal(s) * sd).astype(dtype)
    W = {"wte.weight": nrm(vocab, D), "wpe.weight": nrm(n_ctx, D)}
    for i in range(n_layer):
        p = f"h.{i}."
        for ln in ("ln_1", "ln_2"):
            W[p + ln + ".weight"] = (1 + nrm(D, sd=0.1)).astype(dtype)
            W[p + ln + ".bias"] = nrm(D, sd=0.1)
        for name, (fi, fo) in (("attn.c_attn", (D, 3 * D)), ("attn.c_proj", (D, D)),
                               ("mlp.c_fc", (D, 4 * D)), ("mlp.c_proj", (4 * D, D))):
            W[p + name + ".weight"] = nrm(fi, fo)
            W[p + name + ".bias"] = nrm(fo, sd=0.1)
        W[p + "attn.bias"] = np.tril(np.ones((1, 1, n_ctx, n_ctx), np.uint8))
    W["ln_f.weight"] = (1 + nrm(D, sd=0.1)).astype(dtype)
    W["ln_f.bias"] = nrm(D, sd=0.1)
    return {prefix + k: v for k, v in W.items()}


# -- timed CPU twins the reference itself reports next to its GPU numbers -----------------

def mlp_train_step_seconds(x, labels, params, n_cls, act="gelu", optimizer="sgd", steps=20,
                           lr=1e-3):
    """Best-of-`steps` wall time of one full numpy training step of the MLP: forward,
    backward and the update, like examples/mnist.py:83-118 (which updates with plain SGD,
    mnist.py:115-116).  optimizer="adamw" replaces the update by the AdamW restatement
    above on every tensor (weight decay on matrices only, autograd.py:334)."""
    import time
    P = [np.array(p, dtype=np.float32) for p in params]
    M = [np.zeros_like(p) for p in P]
    V = [np.zeros_like(p) for p in P]
    x32 = np.asarray(x, dtype=np.float32)
    best = float("inf")
    for t in range(1, steps + 1):
        t0 = time.perf_counter()
        _, grads = mlp_forward_backward(x32, P, labels, n_cls, act=act)
        for i, g in enumerate(grads):
            if optimizer == "sgd":
                P[i] -= np.float32(lr) * g.astype(np.float32)
            else:
                P[i], M[i], V[i], _ = adamw_step(P[i], g, M[i], V[i], t, lr=lr,
                                                 wd=0.01 if P[i].ndim == 2 else 0.0)
        best = min(best, time.perf_counter() - t0)
    return best


def matmuls_only_step_seconds(B, T, D, H, n_layer, vocab, reps=1):
    """The reference's own lower bound for a CPU transformer step (examples/charlm.py:60-96):
    only the dominant matmuls and the attention of a forward pass plus two stand-in
    backward matmuls per layer, in fp32 numpy; best of `reps`."""
    import time
    rows, hd = B * T, D // H
    rng = np.random.default_rng(0)
    f = np.float32
    x = rng.standard_normal((rows, D)).astype(f)
    w_qkv = rng.standard_normal((D, 3 * D)).astype(f)
    w_proj = rng.standard_normal((D, D)).astype(f)
    w_fc1 = rng.standard_normal((D, 4 * D)).astype(f)
    w_fc2 = rng.standard_normal((4 * D, D)).astype(f)
    w_head = rng.standard_normal((D, vocab)).astype(f)
    best = float("inf")
    for _ in range(reps):
        t0 = time.perf_counter()
        for _ in range(n_layer):
            qkv = x @ w_qkv
            q, k, v = (_heads(qkv[:, i * D:(i + 1) * D], B, T, H, hd) for i in range(3))
            s = q @ k.transpose(0, 1, 3, 2)
            s = np.exp(s - s.max(-1, keepdims=True))
            s /= s.sum(-1, keepdims=True)
            a = _unheads(s @ v, B, T, H, hd) @ w_proj
            h = (a @ w_fc1) @ w_fc2
            _ = h.T @ x          # the two matmuls the reference lets stand for the backward
            _ = h @ w_fc2.T
        _ = x @ w_head
        best = min(best, time.perf_counter() - t0)
    return best
