"""Two real GPUs, one process each, NCCL between them: the data-parallel step of the product.

Skipped on a box with one GPU.  Checks the reference's claims for its data-parallel path
(examples/ddp_mnist.py:79-105): the update uses the mean of the workers' gradients, and the
replicas stay bit-identical (drift == 0) -- for the single all-reduce after the backward and
for the exchange that runs beside the backward, which with two workers must agree with each
other to the last bit (a + b has one order) and with the CPU oracle within the gradient
tolerance.
"""

import multiprocessing as mp
import os
import socket

import numpy as np
import pytest

from oracle import vkgrad_numpy as orc

pytestmark = pytest.mark.gpu

B, T, D, H, L, V = 2, 128, 128, 2, 4, 250
LR, WD, SCALE = 1e-3, 0.01, 256.0


def _gpu_count():
    import ctypes as C
    try:
        from vkgrad_b200 import _lib
        n = C.c_int32(0)
        _lib.load().vkg_device_count(C.byref(n))
        return n.value
    except Exception:       # no library: the GPU tests that need it fail loudly on their own
        return 0


def free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def batch(rank, step):
    rng = np.random.default_rng(1000 * step + rank)
    return (rng.integers(0, V, B * T).astype(np.uint32), rng.integers(0, V, B * T).astype(np.uint32))


def params():
    return orc.make_gpt_params(D, H, L, T, (V + 15) // 16 * 16, seed=21, std=0.05, bias_std=0.05, tie=True)


NAMES = [("tok", None), ("pos", None), ("lnf.g", None), ("b0", "fc1.W"), ("b1", "qkv.b"), ("b3", "proj.W"),
         ("b2", "ln2.g")]


def _worker(rank, world, port, groups, steps, q):
    os.environ.update(RANK=str(rank), WORLD_SIZE=str(world), LOCAL_RANK=str(rank),
                      MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    try:
        from test_transformer_gpu import load_params
        from vkgrad_b200 import vk
        from vkgrad_b200.autograd import AdamW
        from vkgrad_b200.dataparallel import Comm, DataParallelStep, Replica
        from vkgrad_b200.transformer import GPT, TCtx
        dev = vk.Device(rank)
        if groups > 1:
            comm, side = Comm.pair_from_env(dev, 4)
        else:
            comm, side = Comm.from_env(dev), None
        P = params()

        def build(d):
            ctx = TCtx(d)
            model = GPT(ctx, B, T, D, H, L, V, tie=True, loss_scale=SCALE)
            load_params(model, P)
            opt = AdamW(ctx, model.params(), lr=LR, wd=WD)
            return ctx, model, opt, ctx.buf(B * T * 4, "shared"), ctx.buf(B * T * 4, "shared")
        rep = Replica(dev, build, comm=comm)
        ids_dev, tgt_dev = rep.ctx.buf(B * T * 4), rep.ctx.buf(B * T * 4)
        step = DataParallelStep(rep, ids_dev, tgt_dev, host_ids=rep.xbuf, host_targets=rep.ybuf,
                                overlap_groups=groups, side_comm=side, side_sms=8 if groups > 1 else 0)
        losses = []
        for s in range(steps):
            ids, tgt = batch(rank, s)
            rep.xbuf.array(np.uint32)[:] = ids
            rep.ybuf.array(np.uint32)[:] = tgt
            loss, _ = step(LR)
            losses.append(loss)
        m = rep.model
        tensors = {"tok": m.tok, "pos": m.pos, "lnf.g": m.lnf.g, "b0.fc1.W": m.blocks[0].fc1.W,
                   "b1.qkv.b": m.blocks[1].attn.qkv.b, "b3.proj.W": m.blocks[3].attn.proj.W,
                   "b2.ln2.g": m.blocks[2].ln2.g}
        out = {k: p.numpy().tobytes() for k, p in tensors.items()}
        out.update({"grad:" + k: p.grad_numpy().tobytes() for k, p in tensors.items()})
        n_parts = len(step.parts) if step.parts is not None else 1
        dev.sync()
        for c in (side, comm):
            if c is not None:
                c.destroy()
        rep.destroy()
        dev.destroy()
        q.put((rank, out, losses, n_parts, None))
    except Exception as e:      # report instead of leaving the parent to time out
        import traceback
        q.put((rank, None, None, 0, traceback.format_exc() + repr(e)))


def _run(groups, steps):
    port = free_port()
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    procs = [ctx.Process(target=_worker, args=(r, 2, port, groups, steps, q)) for r in range(2)]
    for p in procs:
        p.start()
    got = {}
    try:
        for _ in range(2):
            rank, out, losses, n_parts, err = q.get(timeout=300)
            assert err is None, err
            got[rank] = (out, losses, n_parts)
    finally:
        for p in procs:
            p.join(60)
            if p.is_alive():
                p.kill()
    return got


def _oracle_first_step():
    """The two workers' gradients summed (still carrying the loss scale), and the weights."""
    P = params()
    grads = []
    for rank in range(2):
        ids, tgt = batch(rank, 0)
        _, G, _ = orc.gpt_forward_backward(P, ids, tgt, B, T, D, H, L, V, faithful=True,
                                           grad_scale=SCALE / (B * T))
        G["tok"] = G["tok"] + G.pop("head.W").T
        grads.append(G)
    out = {}
    for k, kk in NAMES:
        w = P[k] if kk is None else P[k][kk]
        g = (grads[0][k] + grads[1][k]) if kk is None else (grads[0][k][kk] + grads[1][k][kk])
        out[k if kk is None else f"{k}.{kk}"] = (g, w)
    return out


@pytest.mark.skipif(_gpu_count() < 2, reason="needs two GPUs")
def test_two_gpu_step_sums_the_workers_and_keeps_replicas_identical():
    one = _run(1, 1)
    ref = _oracle_first_step()
    assert one[0][0] == one[1][0], "replicas diverged after one step"
    for k, (g_ref, w0) in ref.items():
        # what the bucket holds after the exchange is the sum over both workers ...
        g = np.frombuffer(one[0][0]["grad:" + k], np.float32).reshape(g_ref.shape)
        assert np.abs(g - g_ref).max() <= 2e-3 * np.abs(g_ref).max(), k
        # ... and AdamW reads it as the mean, with the loss scale divided out
        w = np.frombuffer(one[0][0][k], np.float32).reshape(w0.shape)
        w_ref = orc.adamw_step(w0, g, 0 * w0, 0 * w0, 1, lr=LR, wd=WD if w0.ndim == 2 else 0.0,
                               gscale=1.0 / (2 * SCALE))[0]
        assert np.abs(w - w_ref).max() < 1e-6, k
    plain, split = _run(1, 3), _run(2, 3)
    assert split[0][2] == 2 and plain[0][2] == 1
    assert plain[0][0] == plain[1][0] and split[0][0] == split[1][0]         # drift == 0
    assert plain[0][0] == split[0][0], "the exchange beside the backward changed the result"
    assert plain[0][1] == split[0][1]


@pytest.mark.skipif(_gpu_count() < 2, reason="needs two GPUs")
def test_two_devices_in_one_process_run_the_same_step():
    """Two vk.Device objects in one process (the reference's examples/ddp_mnist.py opens every
    GPU from one interpreter): kernel attributes such as the opt-in shared-memory size are per
    device, so the second device must launch the big-shared-memory kernels (GEMM, grouped GEMM,
    fused attention) as well as the first, and both must produce the same bits."""
    from test_transformer_gpu import load_params, model_grads, shared
    from vkgrad_b200 import vk
    from vkgrad_b200.transformer import GPT, TCtx
    P = params()
    ids, tgt = batch(0, 0)
    results = []
    for ordinal in (0, 1):
        dev = vk.Device(ordinal)
        ctx = TCtx(dev)
        try:
            model = GPT(ctx, B, T, D, H, L, V, tie=True, loss_scale=SCALE)
            load_params(model, P)
            assert model.blocks[0].attn.fused
            g = dev.graph(f"dev{ordinal}")
            model.record(shared(ctx, ids), shared(ctx, tgt), g)
            g.finish()
            g.submit()
            results.append((model.read_loss(), model_grads(model)))
        finally:
            ctx.destroy()
            dev.destroy()
    assert results[0][0] == results[1][0]
    for k in results[0][1]:
        assert np.array_equal(results[0][1][k], results[1][1][k]), k
    ref_loss, _, _ = orc.gpt_forward_backward(P, ids, tgt, B, T, D, H, L, V, faithful=True,
                                              grad_scale=SCALE / (B * T))
    assert abs(results[0][0] - ref_loss) < 1e-3 * abs(ref_loss)
