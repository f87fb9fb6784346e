"""The product's DataParallelStep on two CPU ranks over gloo.

The class under test is the real one (graph order, the parts of the flat bucket it sums beside
the backward, the points where it lets the model flush a group's gradients, AdamW's gradient
scale).  What stands in for the GPU is small: a device whose graphs replay their thunks on the
host, a communicator that all-reduces numpy memory through torch.distributed (gloo), and a
model of stacked linear blocks whose `record` writes each block's oracle gradient into the
bucket only when that block's backward stage runs -- so a part that was summed before its
gradients were complete, or never summed, shows up as a wrong weight.
"""

import multiprocessing as mp
import os
import socket

import numpy as np

from oracle import vkgrad_numpy as orc

L, D, ROWS = 6, 8, 16


def free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


class View:
    """A tensor's slice of the flat numpy bucket, shaped like Param.g32 is used."""

    def __init__(self, bucket, off, n):
        self.arr = bucket[off:off + n]


class FakeParam:
    def __init__(self, name, w):
        self.name, self.w, self.n, self.shape = name, w.copy(), w.size, w.shape
        self.m, self.v = np.zeros_like(w), np.zeros_like(w)
        self.g32 = None


class FakeBlock:
    def __init__(self, i, rng):
        self.W = FakeParam(f"b{i}.W", (rng.standard_normal((D, D)) * 0.3).astype(np.float32))
        self.b = FakeParam(f"b{i}.b", (rng.standard_normal(D) * 0.1).astype(np.float32))

    def params(self):
        yield self.W
        yield self.b


class FakeModel:
    """y = x; for each block y = tanh(y W + b); loss = mean(y^2) / 2 per rank shard.  `record`
    follows GPT.record's stage numbering and flush contract."""

    def __init__(self, rng, loss_scale):
        self.tok = FakeParam("tok", (rng.standard_normal((4, D)) * 0.2).astype(np.float32))
        self.blocks = [FakeBlock(i, rng) for i in range(L)]
        self.lnf = FakeParam("lnf.g", np.ones(D, np.float32))
        self.loss_scale = loss_scale
        self.flushes = []

    def params(self):
        yield self.tok
        for b in self.blocks:
            yield from b.params()
        yield self.lnf

    def grads(self, x):
        acts, y = [], x + self.tok.w.sum(0)
        for b in self.blocks:
            acts.append(y)
            y = np.tanh(y @ b.W.w + b.b.w)
        out = y * self.lnf.w
        g = {"lnf.g": (out / ROWS * y).sum(0) * self.loss_scale}
        d = out / ROWS * self.lnf.w * self.loss_scale
        for i in reversed(range(L)):
            b, a = self.blocks[i], acts[i]
            dz = d * (1.0 - np.tanh(a @ b.W.w + b.b.w) ** 2)
            g[b.W.name], g[b.b.name] = a.T @ dz, dz.sum(0)
            d = dz @ b.W.w.T
        g["tok"] = np.tile(d.sum(0), (4, 1))
        return {k: v.astype(np.float32) for k, v in g.items()}

    def record(self, x_buf, _targets, graph, flush_after=(), sm_limit_after_flush=0):
        g = graph if callable(graph) else (lambda s: graph)
        state, pending = {}, []

        def forward():
            state["g"] = self.grads(x_buf)
        g(0).add(forward, "forward")

        def write(p):
            # a gradient becomes visible in the bucket only at its flush point
            pending.append(p)
        g(L + 1).add(lambda: write(self.lnf), "lnf.bwd")
        for k in range(L):
            i = L - 1 - k
            gk = g(L + 2 + k)
            gk.add(lambda b=self.blocks[i]: (write(b.W), write(b.b)), f"b{i}.bwd")
            if i in set(flush_after) and i > 0:
                def flush(i=i):
                    self.flushes.append(i)
                    for p in pending:
                        p.g32.arr[:] = state["g"][p.name].ravel()
                    pending.clear()
                gk.add(flush, "flush")
        ge = g(2 * L + 2)

        def last():
            pending.append(self.tok)
            for p in pending:
                p.g32.arr[:] = state["g"][p.name].ravel()
            pending.clear()
        ge.add(last, "embed_bwd + finals")


class FakeGraph:
    def __init__(self, name, log):
        self.name, self.ops, self.log = name, [], log
        self.n_dispatch = self.n_kernels = 0

    def add(self, thunk, name="op", nbytes=0, hint=None):
        self.ops.append(thunk)
        self.n_dispatch += 1

    def finish(self):
        return self

    def submit_async(self):
        self.log.append(("graph", self.name))
        for op in self.ops:
            op()


class FakeDev:
    sm_count = 148
    lib = handle = None

    def __init__(self):
        self.log = []

    def graph(self, name):
        return FakeGraph(name, self.log)


class GlooComm:
    def __init__(self, world, log):
        self.world, self.log = world, log

    def _reduce(self, bucket, count, offset_bytes):
        import torch
        import torch.distributed as dist
        first = offset_bytes // 4
        dist.all_reduce(torch.from_numpy(bucket.arr[first:first + count]))

    def allreduce_sum(self, bucket, count, dtype=0, offset_bytes=0):
        self.log.append(("allreduce", offset_bytes // 4, count))
        self._reduce(bucket, count, offset_bytes)

    def side_begin(self):
        self.log.append(("side_begin",))

    def allreduce_sum_side(self, bucket, count, slot, dtype=0, offset_bytes=0):
        self.log.append(("allreduce_side", offset_bytes // 4, count, slot))
        self._reduce(bucket, count, offset_bytes)

    def side_wait(self, slot):
        self.log.append(("side_wait", slot))


class FakeOpt:
    def __init__(self, params):
        self.params, self.t, self.grad_scale, self.lr = list(params), 0, 0.0, 1e-2

    def advance(self, lr=None):
        self.t += 1
        self.lr = self.lr if lr is None else lr

    def record(self, graph, params=None):
        ps = self.params if params is None else list(params)

        def go():
            for p in ps:
                w, p.m, p.v, _ = orc.adamw_step(p.w, p.g32.arr.reshape(p.shape), p.m, p.v, self.t,
                                                lr=self.lr, wd=0.01 if p.w.ndim == 2 else 0.0,
                                                gscale=self.grad_scale)
                p.w[...] = w
        graph.add(go, "adamw")


class FakeReplica:
    def __init__(self, world, loss_scale, log):
        self.dev = FakeDev()
        self.dev.log = log
        self.model = FakeModel(np.random.default_rng(3), loss_scale)
        self.params = list(self.model.params())
        self.offsets, off = [], 0
        for p in self.params:
            self.offsets.append(off)
            off += (p.n + 3) // 4 * 4
        self.total = off
        self.bucket = View(np.zeros(off, np.float32), 0, off)
        for p, o in zip(self.params, self.offsets):
            p.g32 = View(self.bucket.arr, o, p.n)
        self.opt = FakeOpt(self.params)
        self.comm = GlooComm(world, log) if world > 1 else None
        self.loss_scale = loss_scale

    def push_gradients(self, graph=None):
        pass


def shard(rank, step):
    return np.random.default_rng(100 * step + rank).standard_normal((ROWS, D)).astype(np.float32)


def _worker(rank, world, port, groups, q):
    import torch.distributed as dist
    from vkgrad_b200.dataparallel import DataParallelStep
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    log = []
    rep = FakeReplica(world, 64.0, log)
    x = shard(rank, 0)
    step = DataParallelStep(rep, x, None, overlap_groups=groups, side_comm=None, side_sms=8)
    for s in range(2):
        x[...] = shard(rank, s)
        step.enqueue(1e-2)
    q.put((rank, [p.w.tobytes() for p in rep.params], log, rep.model.flushes))
    dist.barrier()
    dist.destroy_process_group()


def _run(groups):
    port = free_port()
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    procs = [ctx.Process(target=_worker, args=(r, 2, port, groups, q)) for r in range(2)]
    for p in procs:
        p.start()
    got = {}
    for _ in range(2):
        r, w, log, fl = q.get(timeout=180)
        got[r] = (w, log, fl)
    for p in procs:
        p.join(60)
    return got


def _single_process_reference():
    rep = FakeReplica(1, 64.0, [])
    m, opt = rep.model, rep.opt
    for s in range(2):
        gs = [m.grads(shard(r, s)) for r in range(2)]
        opt.t += 1
        for p in rep.params:
            summed = gs[0][p.name] + gs[1][p.name]
            p.w[...], p.m, p.v, _ = orc.adamw_step(p.w, summed, p.m, p.v, opt.t, lr=1e-2,
                                                    wd=0.01 if p.w.ndim == 2 else 0.0,
                                                    gscale=1.0 / (2 * 64.0))
    return [p.w.copy() for p in rep.params]


def test_overlapped_exchange_equals_one_all_reduce_and_the_single_process_oracle():
    ref = _single_process_reference()
    plain, split = _run(1), _run(3)
    for got in (plain, split):
        assert got[0][0] == got[1][0], "replicas diverged"            # drift == 0
        for w, r in zip(got[0][0], ref):
            assert np.allclose(np.frombuffer(w, np.float32).reshape(r.shape), r, atol=1e-6)
    assert plain[0][0] == split[0][0], "the split exchange must equal the single all-reduce bit for bit"
    # the unsplit step: backward graph, ONE all-reduce of the whole bucket, optimiser graph
    kinds = [e[0] for e in plain[0][1][:3]]
    assert kinds == ["graph", "allreduce", "graph"] and plain[0][1][1][1:] == (0, FakeReplica(1, 1.0, []).total)
    # the split step of 6 blocks in 3 groups: flushes after blocks 4 and 2; every part goes to a
    # side stream right after the graph that completes it; the optimiser over the two upper
    # parts waits for their sums only and runs while the last part is still being summed
    log = split[0][1]
    per_step = len(log) // 2
    names = [e[0] for e in log[:per_step]]
    assert names == ["graph", "side_begin", "allreduce_side", "graph", "side_begin", "allreduce_side",
                     "graph", "side_begin", "allreduce_side", "side_wait", "side_wait", "graph",
                     "side_wait", "graph"]
    assert [e[1] for e in log[:per_step] if e[0] == "side_wait"] == [0, 1, 2]
    assert split[0][2][:2] == [4, 2]
    sides = [e for e in log[:per_step] if e[0] == "allreduce_side"]
    total = FakeReplica(1, 1.0, []).total
    assert sides[0][1] + sides[0][2] == total                      # top part reaches the bucket's end
    assert sides[1][1] + sides[1][2] == sides[0][1]                # parts tile the bucket downwards
    assert sides[2][1] == 0 and sides[2][2] == sides[1][1]
