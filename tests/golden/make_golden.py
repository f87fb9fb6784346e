"""Generates the golden fixtures in this folder from the reference's own numpy code.

    python tests/golden/make_golden.py [/path/to/vkgrad]

The reference (BrettKnox/vkgrad) loads libvulkan when `vk` is imported, and every
module imports `vk`, so a stub `vk` module is placed in sys.modules first; only
the reference's numpy functions are executed:

  kernels.matmul_reference                 (kernels.py:606-610)
  test_autograd.numpy_forward_backward     (test_autograd.py:21-46)
  test_transformer.np_model                (test_transformer.py:38-151)
  examples.hetero_mnist.cpu_backward       (examples/hetero_mnist.py:38-68)
  test_hf_gpt2.ref_logits, perplexity      (test_hf_gpt2.py:33-73)
  hf_gpt2.read_safetensors                 (hf_gpt2.py:36-59; reads tiny_gpt2.safetensors back)
  examples.train_lm.encode                 (examples/train_lm.py:60-67)

Inputs come from numpy seeds with the same draws the reference's tests make
(test_kernels.py:10-16, test_autograd.py:53-75, test_transformer.py:222-243),
so the fixtures store the reference's outputs plus a digest of the inputs.
The fixtures are what travels: the GPU box has no copy of the reference.
"""

import hashlib
import os
import sys
import types

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
sys.path.insert(0, ROOT)

from oracle import vkgrad_numpy as orc  # noqa: E402  (input generators only)


def import_reference(path):
    stub = types.ModuleType("vk")

    class VkError(RuntimeError):
        pass

    class Device:
        def __init__(self, *a, **k):
            raise VkError("stub: no Vulkan here")

    stub.VkError, stub.Device = VkError, Device
    sys.modules["vk"] = stub
    sys.path.insert(0, path)
    import kernels as ref_kernels
    import test_autograd as ref_test_autograd
    import test_transformer as ref_test_transformer
    from examples import hetero_mnist as ref_hetero
    import hf_gpt2 as ref_hf
    import test_hf_gpt2 as ref_test_hf
    from examples import train_lm as ref_lm
    return (ref_kernels, ref_test_autograd, ref_test_transformer, ref_hetero, ref_hf, ref_test_hf,
            ref_lm)


def digest(*arrays):
    h = hashlib.sha256()
    for a in arrays:
        h.update(np.ascontiguousarray(a).tobytes())
    return np.frombuffer(h.digest()[:8], dtype=np.uint64)[0]


MATMUL_CASES = [  # (m, n, k, trans_a, trans_b): test_kernels.py:47-66
    (256, 256, 256, False, False), (128, 128, 128, False, False),
    (512, 256, 128, False, False), (256, 512, 256, False, False),
    (64, 64, 512, False, False), (256, 256, 256, True, False),
    (256, 256, 256, False, True)]


def matmul_inputs(m, n, k, ta, tb, seed=0):
    rng = np.random.default_rng(seed)
    a = rng.standard_normal((k, m) if ta else (m, k)).astype(np.float16)
    b = rng.standard_normal((n, k) if tb else (k, n)).astype(np.float16)
    return a, b


def mlp_inputs(batch=16, n_in=32, n_hid=16, n_cls=4, pad=16, seed=0):
    """Same draws, in the same order, as test_autograd.build (test_autograd.py:53-68)."""
    rng = np.random.default_rng(seed)
    x = rng.standard_normal((batch, n_in)).astype(np.float16).astype(np.float32)
    y = rng.integers(0, n_cls, batch).astype(np.uint32)
    params = []
    for shape in ((n_in, n_hid), (n_hid,), (n_hid, pad), (pad,)):
        std = np.sqrt(2.0 / shape[0]) if len(shape) == 2 else 0.1
        params.append(rng.standard_normal(shape).astype(np.float32) * np.float32(std))
    return x, y, params


GPT_CASES = {  # name: (B, T, D, H, L, vocab, tie, packed)
    "gpt_untied": (2, 16, 32, 2, 2, 16, False, False),
    "gpt_tied": (2, 16, 32, 2, 2, 16, True, False),
    "gpt_packed": (2, 64, 32, 2, 2, 16, True, True),
}


def gpt_inputs(name):
    B, T, D, H, L, vocab, tie, packed = GPT_CASES[name]
    rows = B * T
    pad_vocab = ((vocab + 15) // 16) * 16
    P = orc.make_gpt_params(D, H, L, T, pad_vocab, seed=7, std=0.08, bias_std=0.1, tie=tie)
    if not tie:
        P["head.b"] = (np.random.default_rng(8).standard_normal(pad_vocab)).astype(np.float32)
    rng = np.random.default_rng(0)
    ids = rng.integers(0, vocab, rows).astype(np.uint32)
    tgt = rng.integers(0, vocab, rows).astype(np.uint32)
    seg = w = None
    if packed:  # test_transformer.py:282-287
        seg = np.zeros(rows, np.uint32)
        for b, starts in enumerate(((0, 23, 40, 57), (0, 5, 33))):
            for s, e in zip(starts, starts[1:] + (T,)):
                seg[b * T + s:b * T + e] = s
        w = rng.uniform(0.5, 2.0, rows).astype(np.float32)
        w[rng.random(rows) < 0.3] = 0.0
    return dict(B=B, T=T, D=D, H=H, L=L, vocab=vocab, pad_vocab=pad_vocab, tie=tie), P, ids, tgt, seg, w


HF_CASES = {  # name: (D, H, n_layer, n_ctx, vocab, tokens in the prompt)
    "hf_small": (32, 2, 2, 32, 80, 24),
    "hf_hd64": (128, 2, 2, 128, 96, 100),   # head dimension 64: the fused attention kernels
}


def hf_inputs(name):
    """Synthetic GPT-2 state dict under Hugging Face names and a prompt (stand-ins for the
    real checkpoint and the tokenised paragraph of test_hf_gpt2.py:20-30)."""
    D, H, L, n_ctx, vocab, n = HF_CASES[name]
    W = orc.make_hf_gpt2_tensors(D, H, L, n_ctx, vocab, seed=21)
    ids = np.random.default_rng(22).integers(0, vocab, n)
    return dict(D=D, H=H, n_layer=L, n_ctx=n_ctx, vocab=vocab), W, ids


def lm_bytes(n=8192, seed=31):
    """Bytes with a skewed, text-like frequency profile (more distinct values than ids)."""
    rng = np.random.default_rng(seed)
    return np.clip(rng.normal(100, 22, n), 0, 255).astype(np.uint8)


def flatten_grads(G, L):
    out = {}
    for k, v in G.items():
        if isinstance(v, dict):
            for kk, vv in v.items():
                out[f"{k}.{kk}"] = np.asarray(vv, np.float32)
        else:
            out[k] = np.asarray(v, np.float32)
    return out


def main():
    if len(sys.argv) < 2:
        raise SystemExit("usage: python make_golden.py <path to a checkout of the reference>")
    ref_path = sys.argv[1]
    rk, rta, rtt, rh, rhf, rthf, rlm = import_reference(ref_path)

    mm = {}
    for i, (m, n, k, ta, tb) in enumerate(MATMUL_CASES):
        a, b = matmul_inputs(m, n, k, ta, tb)
        c = rk.matmul_reference(a, b, ta, tb)
        mm[f"c{i}_shape"] = np.array([m, n, k, int(ta), int(tb)])
        mm[f"c{i}_in"] = np.array([digest(a, b)], dtype=np.uint64)
        mm[f"c{i}_sample"] = c[::7, ::5].astype(np.float32)
        mm[f"c{i}_sum"] = np.array([c.astype(np.float64).sum(), np.abs(c).astype(np.float64).sum()])
    ones = rk.matmul_reference(np.ones((64, 1024), np.float16), np.ones((1024, 64), np.float16))
    mm["ones_k1024"] = np.array([ones.min(), ones.max()], np.float32)  # test_kernels.py:69-100
    np.savez_compressed(os.path.join(HERE, "matmul.npz"), **mm)

    mlp = {}
    for seed in range(5):
        x, y, params = mlp_inputs(seed=seed)
        loss, dW1, db1, dW2, db2 = rta.numpy_forward_backward(x, *params, y, 4)
        mlp[f"s{seed}_in"] = np.array([digest(x, y, *params)], dtype=np.uint64)
        mlp[f"s{seed}_loss"] = np.array([loss], np.float64)
        for nm, g in zip(("dW1", "db1", "dW2", "db2"), (dW1, db1, dW2, db2)):
            mlp[f"s{seed}_{nm}"] = g.astype(np.float32)
    # the heterogeneous example's CPU worker: same model, different code
    x, y, params = mlp_inputs(seed=0)
    loss_h, grads_h = rh.cpu_backward(x, y.astype(np.int64), *params, 4)
    mlp["hetero_loss"] = np.array([loss_h], np.float64)
    for nm, g in zip(("dW1", "db1", "dW2", "db2"), grads_h):
        mlp[f"hetero_{nm}"] = np.asarray(g, np.float32)
    np.savez_compressed(os.path.join(HERE, "mlp.npz"), **mlp)

    for name in GPT_CASES:
        cfg, P, ids, tgt, seg, w = gpt_inputs(name)
        loss, G = rtt.np_model(P, ids.astype(np.int64), tgt.astype(np.int64), cfg["B"], cfg["T"],
                               cfg["D"], cfg["H"], cfg["L"], cfg["vocab"], cfg["pad_vocab"],
                               seg=seg, weights=w)
        flat = flatten_grads(G, cfg["L"])
        flat["loss"] = np.array([loss], np.float64)
        flat["inputs_digest"] = np.array([digest(ids, tgt, P["tok"], P["b0"]["qkv.W"])], np.uint64)
        np.savez_compressed(os.path.join(HERE, f"{name}.npz"), **flat)
        print(f"{name}: loss {loss:.6f}, {len(flat) - 2} gradient tensors")
    hf = {}
    for name in HF_CASES:
        cfg, W, ids = hf_inputs(name)
        logits = rthf.ref_logits(W, cfg["H"], ids)
        hf[f"{name}_logits"] = logits.astype(np.float32)
        hf[f"{name}_ppl"] = np.array([rthf.perplexity(logits, ids)], np.float64)
        hf[f"{name}_in"] = np.array([digest(ids, W["wte.weight"], W["h.1.mlp.c_fc.weight"])], np.uint64)
        print(f"{name}: logits {logits.shape}, perplexity {hf[f'{name}_ppl'][0]:.4f}")
    np.savez_compressed(os.path.join(HERE, "hf_gpt2.npz"), **hf)

    # a checkpoint file written by this repo's writer and read back by the reference's reader
    from vkgrad_b200 import hf_gpt2 as our_hf
    tiny = orc.make_hf_gpt2_tensors(32, 2, 1, 16, 48, seed=23, prefix="transformer.")
    tiny["lm_head.weight"] = tiny["transformer.wte.weight"].copy()   # tied, as CodeGPT ships it
    path = os.path.join(HERE, "tiny_gpt2.safetensors")
    our_hf.write_safetensors(path, tiny, metadata={"format": "pt"})
    back = rhf.read_safetensors(path)
    assert set(back) == set(tiny)
    assert all(back[k].dtype == tiny[k].dtype and np.array_equal(back[k], tiny[k]) for k in tiny)
    stripped = rhf.gpt2_tensors(path)
    assert "lm_head.weight" not in stripped and "h.0.attn.bias" not in stripped
    print(f"tiny_gpt2.safetensors: {os.path.getsize(path)} bytes, {len(back)} tensors, "
          f"{len(stripped)} after the reference's gpt2_tensors")
    # byte -> id table of the language-model driver on a skewed byte stream
    data = lm_bytes()
    ids, itos = rlm.encode(data, 48)
    np.savez_compressed(os.path.join(HERE, "lm_encode.npz"), ids=ids.astype(np.uint16),
                        itos_ids=np.array(sorted(itos), np.int64),
                        itos_chars=np.array([ord(itos[k]) for k in sorted(itos)], np.int64),
                        data_digest=np.array([digest(data)], np.uint64))
    print("fixtures written to", HERE)


if __name__ == "__main__":
    main()
