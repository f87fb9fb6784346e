"""Hugging Face GPT-2 checkpoints into this package's GPT, numpy only (reference: hf_gpt2.py).

Same surface as the reference module: `read_safetensors`, `gpt2_tensors`, `config`, `load`,
`build`, `Forward`.  `write_safetensors` is an addition: the real GPT-2 / CodeGPT files are
not available offline, so checkpoints of the same format with synthetic weights are written
and read back through the same loader.  The tokenizer helpers of the reference
(hf_gpt2.py:177-211: tiktoken cache seeding, hub download) need files from the network and
are not provided.

File format (hf_gpt2.py:3-4, 36-59): u64 little-endian header length, a JSON header
{name: {dtype, shape, data_offsets}}, then the raw little-endian tensor bytes.

Weight layout (hf_gpt2.py:6-11): HF's Conv1D stores weight as (in, out) and computes
x @ weight + bias, exactly what Dense does with W (in_f, out_f): nothing is transposed.
"""

import json
import os
import struct

import numpy as np

_NP_OF = {"F64": "<f8", "F32": "<f4", "F16": "<f2", "I64": "<i8", "I32": "<i4",
          "I16": "<i2", "I8": "i1", "U8": "u1", "BOOL": "?"}
_ST_OF = {np.dtype(v).str.lstrip("<|="): k for k, v in _NP_OF.items()}
_MAX_HEADER = 100 << 20

_BLOCK_TENSORS = (  # (attribute path inside a Block, HF name inside h.<i>.)
    ("ln1.g", "ln_1.weight"), ("ln1.b", "ln_1.bias"),
    ("attn.qkv.W", "attn.c_attn.weight"), ("attn.qkv.b", "attn.c_attn.bias"),
    ("attn.proj.W", "attn.c_proj.weight"), ("attn.proj.b", "attn.c_proj.bias"),
    ("ln2.g", "ln_2.weight"), ("ln2.b", "ln_2.bias"),
    ("fc1.W", "mlp.c_fc.weight"), ("fc1.b", "mlp.c_fc.bias"),
    ("fc2.W", "mlp.c_proj.weight"), ("fc2.b", "mlp.c_proj.bias"))


def read_safetensors(path):
    """{name: read-only array} viewing a memory map of the file (hf_gpt2.py:36-59).
    Raises ValueError for a header that does not fit the file, an unknown dtype, or
    offsets that disagree with shape x itemsize."""
    file_size = os.path.getsize(path)
    with open(path, "rb") as fh:
        raw = fh.read(8)
        if len(raw) != 8:
            raise ValueError(f"{path}: shorter than its 8-byte header length")
        hlen = struct.unpack("<Q", raw)[0]
        if hlen > min(file_size - 8, _MAX_HEADER):
            raise ValueError(f"{path}: header length {hlen} does not fit a {file_size}-byte file")
        header = json.loads(fh.read(hlen))
    payload = np.memmap(path, np.uint8, "r", offset=8 + hlen) if file_size > 8 + hlen \
        else np.zeros(0, np.uint8)
    tensors = {}
    for name, entry in header.items():
        if name == "__metadata__":
            continue
        code = entry["dtype"]
        if code not in _NP_OF:
            raise ValueError(f"{path}: {name} has unsupported dtype {code}")
        dt = np.dtype(_NP_OF[code])
        lo, hi = entry["data_offsets"]
        count = int(np.prod(entry["shape"], dtype=np.int64))
        if not (0 <= lo <= hi <= payload.size) or hi - lo != count * dt.itemsize:
            raise ValueError(f"{path}: {name} bytes {lo}..{hi} do not match "
                             f"{entry['shape']} {code}")
        tensors[name] = np.frombuffer(payload, dt, count, lo).reshape(entry["shape"])
    return tensors


def write_safetensors(path, tensors, metadata=None):
    """Write {name: array} in the format `read_safetensors` reads (tensor data in the
    order given, offsets 8-byte aligned through header padding as the format asks)."""
    header, offset, blobs = {}, 0, []
    if metadata:
        header["__metadata__"] = {str(k): str(v) for k, v in metadata.items()}
    for name, arr in tensors.items():
        a = np.asarray(arr)       # tobytes() below is C order whatever the strides
        key = a.dtype.newbyteorder("<").str.lstrip("<|=")
        if key not in _ST_OF:
            raise ValueError(f"{name}: dtype {a.dtype} has no safetensors code")
        blob = a.astype(a.dtype.newbyteorder("<"), copy=False).tobytes()
        header[name] = {"dtype": _ST_OF[key], "shape": list(a.shape),
                        "data_offsets": [offset, offset + len(blob)]}
        offset += len(blob)
        blobs.append(blob)
    text = json.dumps(header, separators=(",", ":")).encode()
    text += b" " * (-len(text) % 8)
    with open(path, "wb") as fh:
        fh.write(struct.pack("<Q", len(text)))
        fh.write(text)
        for blob in blobs:
            fh.write(blob)


def gpt2_tensors(path):
    """Tensors under HF GPT2Model names (wte.weight, h.0.ln_1.weight, ...): the
    'transformer.' prefix some checkpoints carry is removed, the causal-mask buffers
    attn.bias / attn.masked_bias are dropped, and an lm_head.weight is accepted only
    when it equals wte.weight (hf_gpt2.py:62-76)."""
    out = {}
    for name, arr in read_safetensors(path).items():
        if name.startswith("transformer."):
            name = name[len("transformer."):]
        if name.endswith(".attn.bias") or name.endswith(".attn.masked_bias"):
            continue
        out[name] = arr
    head = out.pop("lm_head.weight", None)
    if head is not None and not np.array_equal(head, out["wte.weight"]):
        raise ValueError(f"{path}: untied lm_head.weight is not supported")
    return out


def config(model_dir):
    """Shape of the checkpoint from its config.json; only what the kernels implement is
    accepted: tanh GELU ('gelu_new') and LayerNorm eps 1e-5 (hf_gpt2.py:79-88)."""
    with open(os.path.join(model_dir, "config.json")) as fh:
        c = json.load(fh)
    if c.get("model_type") != "gpt2" or c.get("activation_function") != "gelu_new" \
            or c.get("layer_norm_epsilon") != 1e-5:
        raise ValueError(f"{model_dir}: not a GPT-2 config vkgrad implements")
    return {"D": c["n_embd"], "H": c["n_head"], "n_layer": c["n_layer"],
            "vocab": c["vocab_size"], "n_ctx": c["n_positions"]}


def _resolve(obj, dotted):
    for part in dotted.split("."):
        obj = getattr(obj, part)
    return obj


def load(model, W):
    """Copy GPT-2 tensors into a GPT of the matching shape (hf_gpt2.py:91-136).  Every
    tensor of W must find a parameter of exactly its shape; vocabulary padding rows stay
    zero (never looked up, masked out of the softmax)."""
    vocab, D = W["wte.weight"].shape
    L = len(model.blocks)
    if (vocab, D) != (model.vocab, model.D) or W["h.0.ln_1.weight"].shape[0] != model.D \
            or f"h.{L}.ln_1.weight" in W or f"h.{L - 1}.ln_1.weight" not in W \
            or model.T > W["wpe.weight"].shape[0]:
        raise ValueError("checkpoint does not match the model shape")
    pending = set(W)

    def assign(param, name, value=None):
        value = W[name] if value is None else value
        if tuple(value.shape) != tuple(param.shape):
            raise ValueError(f"{name}: {tuple(value.shape)} into {param.name} {param.shape}")
        param.set(value)
        pending.discard(name)

    table = np.zeros((model.pad_vocab, D), np.float32)
    table[:vocab] = W["wte.weight"]
    assign(model.tok, "wte.weight", table)
    assign(model.pos, "wpe.weight", W["wpe.weight"][:model.T])
    for i, block in enumerate(model.blocks):
        for attr, hf_name in _BLOCK_TENSORS:
            assign(_resolve(block, attr), f"h.{i}.{hf_name}")
    assign(model.lnf.g, "ln_f.weight")
    assign(model.lnf.b, "ln_f.bias")
    if not model.tie:
        # GPT-2 ties the head to wte; an untied model starts from a copy.
        head = np.zeros((D, model.pad_vocab), np.float32)
        head[:, :vocab] = np.asarray(W["wte.weight"], np.float32).T
        model.head.W.set(head)
        model.head.b.set(np.zeros(model.pad_vocab, np.float32))
    if pending:
        raise ValueError(f"unmapped tensors: {sorted(pending)}")


def build(ctx, B, T, model_dir, tie=True):
    """A GPT carrying the weights of model_dir/model.safetensors (hf_gpt2.py:139-145)."""
    from .transformer import GPT
    c = config(model_dir)
    model = GPT(ctx, B, T, c["D"], c["H"], c["n_layer"], c["vocab"], tie=tie)
    load(model, gpt2_tensors(os.path.join(model_dir, "model.safetensors")))
    return model


class Forward:
    """The forward pass recorded once; each call copies the logits to the host
    (hf_gpt2.py:148-185).  There is no KV cache: every call runs all T positions."""

    def __init__(self, model):
        ctx = model.ctx
        self.model = model
        self.ids = ctx.buf(model.rows * 4, "shared")
        self.host = ctx.buf(model.rows * model.pad_vocab * 4, "cached")
        self.graph = ctx.dev.graph("forward")
        self.out = model.forward(self.ids, graph=self.graph)
        self.graph.finish()
        self.submit_s = self.copy_s = 0.0

    def __call__(self, ids, pad=50256, last=False):
        """ids (B, n) with n <= T -> logits (B, n, vocab); with last=True only position
        n-1, shape (B, vocab).  Padding goes on the right, where causal attention keeps it
        out of every real position."""
        m = self.model
        ids = np.asarray(ids)
        n = ids.shape[1]
        if ids.shape[0] != m.B or n > m.T or n < 1:
            raise ValueError(f"ids {ids.shape} do not fit a ({m.B}, <={m.T}) model")
        grid = np.full((m.B, m.T), pad if pad < m.vocab else 0, np.uint32)
        grid[:, :n] = ids
        self.ids.array(np.uint32, (m.rows,))[:] = grid.reshape(-1)
        self.ids.flush()
        self.submit_s = self.graph.submit()
        self.copy_s = m.ctx.dev.copy(self.out, self.host, m.rows * m.pad_vocab * 4)
        self.host.invalidate()
        full = self.host.array(np.float32, (m.B, m.T, m.pad_vocab))
        if last:
            return full[:, n - 1, :m.vocab].copy()
        return full[:, :n, :m.vocab].copy()
