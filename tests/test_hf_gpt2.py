"""GPT-2 checkpoint loading and forward parity (reference: hf_gpt2.py, test_hf_gpt2.py).

The real GPT-2 / CodeGPT files are not available offline; synthetic state dicts under the
same Hugging Face names stand in.  The expected logits in tests/golden/hf_gpt2.npz were
produced by the reference's own test_hf_gpt2.ref_logits (see tests/golden/make_golden.py),
and tests/golden/tiny_gpt2.safetensors was read back by the reference's reader when it was
written.  Tolerances are the reference's (test_hf_gpt2.py:120-124): argmax agreement
>= 98 %, perplexity within 5e-3 relative; max |logit diff| is scaled to this model's range.
"""

import json
import os
import struct
import sys

import numpy as np
import pytest

sys.path.insert(0, os.path.join(os.path.dirname(__file__), "golden"))
import make_golden as mg  # noqa: E402
from oracle import vkgrad_numpy as orc  # noqa: E402
from vkgrad_b200 import hf_gpt2  # noqa: E402

GOLD = os.path.join(os.path.dirname(__file__), "golden")
TINY = os.path.join(GOLD, "tiny_gpt2.safetensors")


# ---- CPU: oracle against the reference's outputs, file format, name mapping -------------

@pytest.mark.parametrize("name", sorted(mg.HF_CASES))
def test_oracle_logits_against_reference_fixture(name):
    gold = np.load(os.path.join(GOLD, "hf_gpt2.npz"))
    cfg, W, ids = mg.hf_inputs(name)
    assert gold[f"{name}_in"][0] == mg.digest(ids, W["wte.weight"], W["h.1.mlp.c_fc.weight"])
    got = orc.gpt2_logits(W, cfg["H"], ids)
    ref = gold[f"{name}_logits"]
    assert got.shape == ref.shape
    assert np.abs(got - ref).max() < 1e-4 * np.abs(ref).max()
    assert abs(orc.perplexity(got, ids) - gold[f"{name}_ppl"][0]) < 1e-4 * gold[f"{name}_ppl"][0]


def test_reads_the_committed_checkpoint():
    expect = orc.make_hf_gpt2_tensors(32, 2, 1, 16, 48, seed=23, prefix="transformer.")
    raw = hf_gpt2.read_safetensors(TINY)
    assert set(raw) == set(expect) | {"lm_head.weight"}
    for k, v in expect.items():
        assert raw[k].dtype == v.dtype and np.array_equal(raw[k], v)
    assert not raw["transformer.wte.weight"].flags.writeable
    W = hf_gpt2.gpt2_tensors(TINY)
    assert "wte.weight" in W and "lm_head.weight" not in W
    assert not any(k.endswith(".attn.bias") or k.startswith("transformer.") for k in W)
    assert len(W) == 16


@pytest.mark.parametrize("dtype", [np.float64, np.float32, np.float16, np.int64, np.int32,
                                   np.int16, np.int8, np.uint8, np.bool_])
def test_write_read_round_trip(tmp_path, dtype):
    rng = np.random.default_rng(3)
    a = (rng.standard_normal((5, 3, 2)) * 10).astype(dtype)
    path = str(tmp_path / "t.safetensors")
    hf_gpt2.write_safetensors(path, {"a": a, "scalar": np.asarray(7, dtype), "empty": a[:0]})
    back = hf_gpt2.read_safetensors(path)
    assert back["a"].dtype == np.dtype(dtype) and np.array_equal(back["a"], a)
    assert back["scalar"].shape == () and back["scalar"] == np.asarray(7, dtype)
    assert back["empty"].shape == (0, 3, 2)


def _write_raw(path, header, payload=b""):
    text = json.dumps(header).encode()
    with open(path, "wb") as fh:
        fh.write(struct.pack("<Q", len(text)) + text + payload)


def test_malformed_files_are_rejected(tmp_path):
    p = str(tmp_path / "bad.safetensors")
    with open(p, "wb") as fh:   # header length larger than the file
        fh.write(struct.pack("<Q", 1 << 40) + b"{}")
    with pytest.raises(ValueError, match="header length"):
        hf_gpt2.read_safetensors(p)
    _write_raw(p, {"x": {"dtype": "BF16", "shape": [2], "data_offsets": [0, 4]}}, b"\0" * 4)
    with pytest.raises(ValueError, match="unsupported dtype"):
        hf_gpt2.read_safetensors(p)
    _write_raw(p, {"x": {"dtype": "F32", "shape": [3], "data_offsets": [0, 8]}}, b"\0" * 8)
    with pytest.raises(ValueError, match="do not match"):
        hf_gpt2.read_safetensors(p)
    _write_raw(p, {"x": {"dtype": "F32", "shape": [4], "data_offsets": [0, 16]}}, b"\0" * 8)
    with pytest.raises(ValueError, match="do not match"):
        hf_gpt2.read_safetensors(p)
    W = orc.make_hf_gpt2_tensors(32, 2, 1, 16, 48, seed=1)
    W["lm_head.weight"] = W["wte.weight"] + 1
    hf_gpt2.write_safetensors(p, W)
    with pytest.raises(ValueError, match="untied lm_head"):
        hf_gpt2.gpt2_tensors(p)


def test_config_accepts_only_what_the_kernels_implement(tmp_path):
    good = {"model_type": "gpt2", "activation_function": "gelu_new", "layer_norm_epsilon": 1e-5,
            "n_embd": 768, "n_head": 12, "n_layer": 12, "vocab_size": 50257, "n_positions": 1024}
    (tmp_path / "config.json").write_text(json.dumps(good))
    assert hf_gpt2.config(str(tmp_path)) == dict(D=768, H=12, n_layer=12, vocab=50257, n_ctx=1024)
    for key, bad in (("activation_function", "gelu"), ("layer_norm_epsilon", 1e-6),
                     ("model_type", "gpt_neo")):
        (tmp_path / "config.json").write_text(json.dumps({**good, key: bad}))
        with pytest.raises(ValueError, match="not a GPT-2 config"):
            hf_gpt2.config(str(tmp_path))


class _FakeParam:
    def __init__(self, name, shape):
        self.name, self.shape, self.value = name, tuple(shape), None

    def set(self, arr):
        assert tuple(np.shape(arr)) == self.shape
        self.value = np.array(arr, np.float32)


def _fake_model(D, L, T, vocab, tie=True):
    """An object with the attributes `load` touches, so the name mapping is checked on CPU."""
    from types import SimpleNamespace as NS
    P = _FakeParam
    pad_vocab = (vocab + 15) // 16 * 16
    blocks = [NS(ln1=NS(g=P("ln1.g", (D,)), b=P("ln1.b", (D,))),
                 ln2=NS(g=P("ln2.g", (D,)), b=P("ln2.b", (D,))),
                 attn=NS(qkv=NS(W=P("qkv.W", (D, 3 * D)), b=P("qkv.b", (3 * D,))),
                         proj=NS(W=P("proj.W", (D, D)), b=P("proj.b", (D,)))),
                 fc1=NS(W=P("fc1.W", (D, 4 * D)), b=P("fc1.b", (4 * D,))),
                 fc2=NS(W=P("fc2.W", (4 * D, D)), b=P("fc2.b", (D,)))) for _ in range(L)]
    m = NS(vocab=vocab, pad_vocab=pad_vocab, D=D, T=T, blocks=blocks, tie=tie,
           tok=P("tok", (pad_vocab, D)), pos=P("pos", (T, D)),
           lnf=NS(g=P("lnf.g", (D,)), b=P("lnf.b", (D,))))
    if not tie:
        m.head = NS(W=P("head.W", (D, pad_vocab)), b=P("head.b", (pad_vocab,)))
    return m


def test_load_maps_every_tensor_and_checks_shapes():
    D, H, L, n_ctx, vocab = 32, 2, 2, 32, 80 - 3      # 77: exercises the vocabulary padding
    W = orc.make_hf_gpt2_tensors(D, H, L, n_ctx, vocab, seed=4)
    W = {k: v for k, v in W.items() if not k.endswith(".attn.bias")}
    m = _fake_model(D, L, 24, vocab, tie=False)
    hf_gpt2.load(m, W)
    assert np.array_equal(m.tok.value[:vocab], W["wte.weight"]) and not m.tok.value[vocab:].any()
    assert np.array_equal(m.pos.value, W["wpe.weight"][:24])
    assert np.array_equal(m.blocks[1].attn.qkv.W.value, W["h.1.attn.c_attn.weight"])
    assert np.array_equal(m.blocks[0].fc2.b.value, W["h.0.mlp.c_proj.bias"])
    assert np.array_equal(m.head.W.value[:, :vocab], W["wte.weight"].T)
    assert not m.head.W.value[:, vocab:].any() and not m.head.b.value.any()
    # a transposed non-square Conv1D is caught by its shape (hf_gpt2.py:6-11)
    bad = dict(W)
    bad["h.0.mlp.c_fc.weight"] = W["h.0.mlp.c_fc.weight"].T
    with pytest.raises(ValueError, match="h.0.mlp.c_fc.weight"):
        hf_gpt2.load(_fake_model(D, L, 24, vocab), bad)
    with pytest.raises(ValueError, match="unmapped tensors"):
        hf_gpt2.load(_fake_model(D, L, 24, vocab), {**W, "h.0.extra": np.zeros(1)})
    for wrong in (_fake_model(D, L + 1, 24, vocab), _fake_model(D, L - 1, 24, vocab),
                  _fake_model(D, L, n_ctx + 8, vocab), _fake_model(D, L, 24, vocab + 1)):
        with pytest.raises(ValueError, match="does not match the model shape"):
            hf_gpt2.load(wrong, W)


# ---- GPU: the forward of a loaded checkpoint against the reference's logits --------------

def _checkpoint_dir(tmp_path, cfg, W, prefix=""):
    d = tmp_path / "ckpt"
    d.mkdir(exist_ok=True)
    (d / "config.json").write_text(json.dumps({
        "model_type": "gpt2", "activation_function": "gelu_new", "layer_norm_epsilon": 1e-5,
        "n_embd": cfg["D"], "n_head": cfg["H"], "n_layer": cfg["n_layer"],
        "vocab_size": cfg["vocab"], "n_positions": cfg["n_ctx"]}))
    hf_gpt2.write_safetensors(str(d / "model.safetensors"), {prefix + k: v for k, v in W.items()})
    return str(d)


@pytest.mark.gpu
@pytest.mark.parametrize("name,tie", [("hf_small", True), ("hf_small", False), ("hf_hd64", True)])
def test_forward_matches_reference_logits(dev, tmp_path, name, tie):
    from vkgrad_b200.transformer import TCtx
    gold = np.load(os.path.join(GOLD, "hf_gpt2.npz"))
    cfg, W, ids = mg.hf_inputs(name)
    ref = gold[f"{name}_logits"]
    model_dir = _checkpoint_dir(tmp_path, cfg, W, prefix="transformer." if tie else "")
    ctx = TCtx(dev)
    try:
        model = hf_gpt2.build(ctx, 1, cfg["n_ctx"], model_dir, tie=tie)
        assert model.blocks[0].attn.fused == (cfg["D"] // cfg["H"] == 64)
        fwd = hf_gpt2.Forward(model)
        got = fwd([ids])[0]
        assert got.shape == ref.shape
        span = float(np.abs(ref).max())
        dmax = float(np.abs(got - ref).max())
        agree = (got.argmax(-1) == ref.argmax(-1)).mean()
        p_got, p_ref = orc.perplexity(got, ids), float(gold[f"{name}_ppl"][0])
        assert dmax < 2e-2 * span, (dmax, span)
        assert agree >= 0.98, agree
        assert abs(p_got - p_ref) / p_ref < 5e-3, (p_got, p_ref)
        # last=True is the final row; a shorter prompt is unaffected by the right padding
        assert np.array_equal(fwd([ids], last=True)[0], got[-1])
        half = len(ids) // 2
        short = fwd([ids[:half]])[0]
        assert short.shape == (half, cfg["vocab"])
        assert np.abs(short - ref[:half]).max() < 2e-2 * span
        # attn.c_proj is square: only the logits can show a transposed copy
        for b in model.blocks:
            b.attn.proj.W.set(b.attn.proj.W.numpy().T.copy())
        bad = fwd([ids])[0]
        assert np.abs(bad - ref).max() > 10 * dmax
    finally:
        ctx.destroy()


@pytest.mark.gpu
def test_forward_of_the_committed_checkpoint_against_the_oracle(dev, tmp_path):
    """tiny_gpt2.safetensors ('transformer.' prefix, tied lm_head, mask buffers) through
    `build`, batch of two different prompts."""
    import shutil
    from vkgrad_b200.transformer import TCtx
    cfg = dict(D=32, H=2, n_layer=1, n_ctx=16, vocab=48)
    d = _checkpoint_dir(tmp_path, cfg, {})
    shutil.copy(TINY, os.path.join(d, "model.safetensors"))
    W = hf_gpt2.gpt2_tensors(TINY)
    ids = np.random.default_rng(9).integers(0, 48, (2, 12))
    ctx = TCtx(dev)
    try:
        fwd = hf_gpt2.Forward(hf_gpt2.build(ctx, 2, 16, d))
        got = fwd(ids)
    finally:
        ctx.destroy()
    for b in range(2):
        ref = orc.gpt2_logits(W, 2, ids[b])
        assert np.abs(got[b] - ref).max() < 2e-2 * np.abs(ref).max()
        assert (got[b].argmax(-1) == ref.argmax(-1)).mean() >= 0.9
