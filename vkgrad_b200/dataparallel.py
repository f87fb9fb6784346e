"""Data-parallel training: replicated weights, summed gradients, identical steps.

Same classes as the reference's dataparallel.py -- `HostArena` (77), `Replica`
(102: push_gradients, zero_arena, step_from_arena), `GradAccum` (153),
`make_reduce_kernels` (28) -- and the same arithmetic: gradients of all workers
are summed, scaled by 1/workers when they are read back (dataparallel.py:63-73,
131-144), and every replica applies the identical AdamW step, so replicas that
start identical stay bit-identical.

What carries the sum is different.  The reference imports one host allocation
into every device and lets each device atomicAdd its gradients into it
(dataparallel.py:40-47).  Here there is one process per GPU and the sum is an
NCCL all-reduce over NVLink/NVSwitch of ONE flat fp32 bucket: `Replica` re-homes
every parameter's gradient buffer into a single contiguous allocation (params()
order, the reference's offset table, dataparallel.py:110-117), so the dW GEMMs
write straight into the bucket and no pack/unpack pass exists.  The 1/workers
(and 1/loss_scale) factor is folded into AdamW's gradient read instead of a
separate pull pass.

Several logical replicas inside one process (the reference's
examples/ddp_mnist.py) still work: without a communicator, `HostArena` is a
device buffer the replicas of that process add into, with the reference's
zero / push / pull sequence.
"""

import ctypes as C
import os
import socket
import struct
import time

import numpy as np

from ._lib import F32
from .kernels import Elementwise
from .vk import VkError, _check


def make_reduce_kernels(dev):
    """push / add / zero / pull under the reference's names (dataparallel.py:28-74).
    One process drives one stream here, so push needs no atomics and equals add."""
    lib, h = dev.lib, dev.handle
    K = {}
    add = lambda b, n, off: _check(lib.vkg_grad_add(h, b[0].dptr, b[1].dptr, n, int(off)), "grad_add")
    K["push"] = Elementwise(dev, "grad_push", add, 2)
    K["add"] = Elementwise(dev, "grad_add", add, 2)
    K["zero"] = Elementwise(dev, "arena_zero", lambda b, n: _check(
        lib.vkg_memset0(h, b[0].dptr, n * 4), "arena_zero"), 1)
    K["pull"] = Elementwise(dev, "grad_pull", lambda b, n, off, scale: _check(
        lib.vkg_grad_pull(h, b[0].dptr, b[1].dptr, n, int(off), float(scale)), "grad_pull"), 2)
    return K


# ---- communicator ---------------------------------------------------------------------

def exchange_unique_id(rank, world, make_id, addr="127.0.0.1", port=29617, timeout=120.0):
    """Rank 0 makes the 128-byte NCCL id and hands it to every other rank over TCP.

    make_id is called on rank 0 only.  No torch, no files: a listener on
    (addr, port) that serves world-1 connections."""
    if world == 1:
        return make_id()
    if rank == 0:
        uid = make_id()
        srv = socket.socket(socket.AF_INET, socket.SOCK_STREAM)
        srv.setsockopt(socket.SOL_SOCKET, socket.SO_REUSEADDR, 1)
        srv.bind((addr, port))
        srv.listen(world)
        srv.settimeout(timeout)
        served = 0
        try:
            while served < world - 1:
                conn, _ = srv.accept()
                with conn:
                    conn.sendall(struct.pack("<I", len(uid)) + uid)
                served += 1
        except socket.timeout:
            raise VkError(f"rendezvous: only {served} of {world - 1} ranks connected "
                          f"within {timeout:.0f} s")
        finally:
            srv.close()
        return uid
    deadline = time.monotonic() + timeout
    last = None
    while time.monotonic() < deadline:
        try:
            with socket.create_connection((addr, port), timeout=5.0) as s:
                head = _recv_exact(s, 4)
                (n,) = struct.unpack("<I", head)
                return _recv_exact(s, n)
        except (ConnectionRefusedError, socket.timeout, OSError) as e:
            last = e
            time.sleep(0.2)
    raise VkError(f"rendezvous: rank {rank} could not reach rank 0 at {addr}:{port}: {last}")


def _recv_exact(s, n):
    out = b""
    while len(out) < n:
        chunk = s.recv(n - len(out))
        if not chunk:
            raise OSError("connection closed during rendezvous")
        out += chunk
    return out


class Comm:
    """An NCCL communicator bound to one Device (one process per GPU)."""

    def __init__(self, dev, rank, world, unique_id, max_ctas=0):
        """max_ctas > 0 holds NCCL to that many CTAs: for a communicator whose collectives run
        beside the compute stream."""
        self.dev, self.rank, self.world = dev, rank, world
        uid = (C.c_uint8 * 128).from_buffer_copy(unique_id)
        h = C.c_void_p()
        _check(dev.lib.vkg_comm_create_limited(dev.handle, rank, world, uid, int(max_ctas),
                                               C.byref(h)), "comm_create")
        self.handle = h
        self.max_ctas = int(max_ctas)

    @staticmethod
    def make_unique_id(lib):
        uid = (C.c_uint8 * 128)()
        _check(lib.vkg_comm_unique_id(uid), "comm_unique_id")
        return bytes(uid)

    @classmethod
    def from_env(cls, dev, port_offset=101, max_ctas=0):
        """Build from RANK / WORLD_SIZE / MASTER_ADDR / MASTER_PORT (torchrun's variables)."""
        rank = int(os.environ.get("RANK", "0"))
        world = int(os.environ.get("WORLD_SIZE", "1"))
        addr = os.environ.get("MASTER_ADDR", "127.0.0.1")
        port = (int(os.environ.get("MASTER_PORT", "29500")) + port_offset) % 65536
        uid = exchange_unique_id(rank, world, lambda: cls.make_unique_id(dev.lib), addr, port)
        return cls(dev, rank, world, uid, max_ctas=max_ctas)

    @classmethod
    def pair_from_env(cls, dev, side_max_ctas, port_offset=101):
        """(main, side): the communicator for the compute stream and one held to
        side_max_ctas CTAs for collectives beside it, from ONE rendezvous (both ids travel in
        the same message)."""
        rank = int(os.environ.get("RANK", "0"))
        world = int(os.environ.get("WORLD_SIZE", "1"))
        addr = os.environ.get("MASTER_ADDR", "127.0.0.1")
        port = (int(os.environ.get("MASTER_PORT", "29500")) + port_offset) % 65536
        ids = exchange_unique_id(rank, world,
                                 lambda: cls.make_unique_id(dev.lib) + cls.make_unique_id(dev.lib),
                                 addr, port)
        main = cls(dev, rank, world, ids[:128])
        try:
            side = cls(dev, rank, world, ids[128:256], max_ctas=side_max_ctas)
        except VkError:
            # an NCCL that does not take the CTA limit refuses on every rank alike: the caller
            # exchanges on the main communicator alone
            side = None
        return main, side

    def allreduce_sum(self, buf, count, dtype=F32, offset_bytes=0):
        _check(self.dev.lib.vkg_allreduce_sum(self.handle, buf.dptr + offset_bytes, count, dtype),
               "allreduce")

    def side_begin(self):
        """Order the side stream after everything enqueued on the compute stream so far."""
        _check(self.dev.lib.vkg_comm_side_begin(self.handle), "comm_side_begin")

    def allreduce_sum_side(self, buf, count, slot, dtype=F32, offset_bytes=0):
        """All-reduce on the side stream; event `slot` marks its end."""
        _check(self.dev.lib.vkg_allreduce_sum_side(self.handle, buf.dptr + offset_bytes, count, dtype,
                                                   slot), "allreduce_side")

    def side_wait(self, slot):
        """The compute stream waits for the side-stream all-reduce that used `slot`."""
        _check(self.dev.lib.vkg_comm_side_wait(self.handle, slot), "comm_side_wait")

    def max_double(self, value):
        v = C.c_double(float(value))
        _check(self.dev.lib.vkg_comm_max_double(self.handle, C.byref(v)), "comm_max")
        return v.value

    def barrier(self):
        _check(self.dev.lib.vkg_comm_barrier(self.handle), "barrier")

    def destroy(self):
        if self.handle:
            self.dev.lib.vkg_comm_destroy(self.handle)
            self.handle = None


# ---- arena / replicas --------------------------------------------------------------------

class HostArena:
    """The flat gradient exchange buffer (dataparallel.py:77-99).

    In the reference this is host memory imported by every device.  Here it is
    device memory, allocated on first use by a replica's device, that logical
    replicas inside one process add into; with a communicator it is not used at
    all (the bucket is all-reduced in place)."""

    def __init__(self, n_floats, alignment=4096):
        self.n = int(n_floats)
        # room for the 16-byte alignment padding between tensors of the flat bucket
        self.nbytes = ((self.n * 4 + 16384 + alignment - 1) // alignment) * alignment
        self._buffers = {}

    def buffer_for(self, dev):
        key = dev.ordinal
        if key not in self._buffers:
            if self._buffers:
                # device memory of one GPU: replicas on another GPU would each sum into a
                # private arena and still divide by n_workers
                raise VkError(f"HostArena already lives on GPU {next(iter(self._buffers))}; "
                              f"replicas on GPU {key} exchange gradients through a Comm "
                              f"(NCCL all-reduce), not through the arena")
            self._buffers[key] = dev.buffer(self.nbytes, "device")
        return self._buffers[key]

    def destroy(self):
        for b in self._buffers.values():
            b.destroy()
        self._buffers = {}


def flatten_gradients(ctx, params):
    """Re-home every p.g32 into one contiguous device buffer, in params() order.
    Returns (bucket, offsets_in_floats, total_floats).  Must run before a step is
    recorded: recorded launches keep the pointers they were recorded with."""
    offs, off = [], 0
    for p in params:
        offs.append(off)
        off += (p.n + 3) // 4 * 4          # keep every tensor 16-byte aligned
    bucket = ctx.buf(max(off, 4) * 4, "device")
    _check(ctx.dev.lib.vkg_memset0(ctx.dev.handle, bucket.dptr, bucket.size), "zero bucket")
    for p, o in zip(params, offs):
        old = p.g32
        p.g32 = bucket.view(o * 4, p.n * 4)
        if old in ctx._owned:
            ctx._owned.remove(old)
            old.destroy()
    return bucket, offs, off


class Replica:
    """One device's copy of the model plus its part in the exchange (dataparallel.py:102-150).

    build(dev) -> (ctx, model, opt, xbuf, ybuf).  With `comm`, push_gradients is an
    all-reduce of the flat bucket; with `arena` the replica adds into it; with
    neither it is a single worker."""

    def __init__(self, dev, build, arena=None, comm=None):
        self.dev = dev
        self.comm = comm
        self.ctx, self.model, self.opt, self.xbuf, self.ybuf = build(dev)
        self.K = make_reduce_kernels(dev)
        self.params = list(self.model.params())
        self.bucket, self.offsets, self.total = flatten_gradients(self.ctx, self.params)
        self.arena = arena
        self.arena_buf = None
        if comm is None and arena is not None:
            assert self.total <= arena.nbytes // 4, \
                f"arena too small: need {self.total}, have {arena.nbytes // 4}"
            self.arena_buf = arena.buffer_for(dev)
        self.loss_scale = float(getattr(self.model, "loss_scale", 1.0))

    def zero_arena(self, graph=None):
        if self.arena_buf is not None:
            self.K["zero"]([self.arena_buf], self.total, graph=graph)

    def push_gradients(self, graph=None):
        """Contribute this replica's gradients to the sum."""
        if self.comm is not None:
            comm, bucket, total = self.comm, self.bucket, self.total
            if comm.world > 1:
                thunk = lambda: comm.allreduce_sum(bucket, total)
                if graph is not None:
                    graph.add(thunk, "nccl_allreduce", total * 4)
                else:
                    thunk()
            return
        if self.arena_buf is None:
            return                      # a single worker: its gradient is the sum
        self.dev.sync()
        self.K["push"]([self.bucket, self.arena_buf], self.total, 0, graph=graph)

    def record_step(self, graph, n_workers=None):
        """Record all-reduce + AdamW after a recorded forward/backward."""
        w = n_workers if n_workers is not None else (self.comm.world if self.comm else 1)
        self.opt.grad_scale = 1.0 / (max(w, 1) * self.loss_scale)
        self.push_gradients(graph=graph)
        self.opt.record(graph)

    def step_from_arena(self, lr, n_workers=1):
        """AdamW from the summed gradient, scaled back to a mean (dataparallel.py:131-144)."""
        scale = 1.0 / (max(n_workers, 1) * self.loss_scale)
        if self.arena_buf is not None:
            self.opt.grad_scale = 0.0
            self.K["pull"]([self.arena_buf, self.bucket], self.total, 0, scale)
        else:
            self.opt.grad_scale = scale
        self.opt.step(lr)

    def destroy(self):
        self.ctx.destroy()


class DataParallelStep:
    """One recorded data-parallel training step: (inputs up) -> forward/backward ->
    all-reduce of the flat gradient bucket -> AdamW.

    The multi-GPU counterpart of autograd.TrainStep; with one worker it is the same
    step without the all-reduce.  host_ids/host_targets, when given, are pinned
    host buffers copied to the device inside the step, so per-step data written by
    the caller is picked up by every replay.

    With more than one worker the step is several CUDA graphs with the NCCL calls enqueued
    between them (no host synchronisation in between); in_graph=True captures the one
    all-reduce into a single graph instead.

    overlap_groups=k > 1 hides most of the exchange under the backward (the reference's
    workers push each tensor as soon as it exists, dataparallel.py:119-126).  The blocks are
    cut into k groups from the top; as soon as the backward of a group is done, its dW GEMMs
    and final passes run (GPT.record(flush_after=...)), which completes that part of the flat
    bucket, and its all-reduce starts on a side stream while the compute stream goes on with
    the blocks below.  Only the last part -- the lowest blocks and the embedding tables,
    whose gradient is final only after the embedding backward -- is summed after the
    backward, and AdamW over the parameters of the earlier parts runs meanwhile (the
    optimiser is one launch per set of parts).  The sums are the same fp32 NCCL sums over the
    same bytes, so replicas stay bit-identical; with two workers the result also equals the
    unsplit exchange bit for bit, with more it agrees to rounding (the order in which NCCL adds
    the ranks' values of an element depends on where the element sits in its message).
    The side stream should use `side_comm`, a communicator held to a few CTAs
    (Comm(..., max_ctas=n)); the persistent kernels recorded after the first flush then launch
    sm_count - side_sms CTAs so that NCCL's CTAs find free SMs instead of delaying a statically
    scheduled grid by a whole wave.
    """

    def __init__(self, replica, ids_dev, targets_dev, host_ids=None, host_targets=None,
                 name="dp_step", in_graph=False, overlap_groups=1, side_comm=None, side_sms=0,
                 **record_kwargs):
        self.replica = replica
        self.model, self.opt = replica.model, replica.opt
        dev = self.dev = replica.dev
        lib, h = dev.lib, dev.handle
        comm = replica.comm
        workers = comm.world if comm is not None else 1
        blocks = getattr(self.model, "blocks", None)
        k = int(overlap_groups)
        split = (comm is not None and comm.world > 1 and not in_graph and k > 1
                 and blocks is not None and len(blocks) >= k)
        self.between = None
        self.parts = None
        upload = None
        if host_ids is not None:
            pairs = [(ids_dev, host_ids), (targets_dev, host_targets)]

            def upload():
                for d, s in pairs:
                    _check(lib.vkg_copy_h2d_async(h, d.dptr, s.hptr, min(d.size, s.size)), "h2d")
            upload.nbytes = sum(min(d.size, s.size) for d, s in pairs)

        def first_graph(g):
            if upload is not None:
                g.add(upload, "h2d_inputs", upload.nbytes)
                g.n_dispatch -= 1
            return g

        self.opt.grad_scale = 1.0 / (workers * replica.loss_scale)
        if split:
            L = len(blocks)
            flush = backward_flush_points(L, k)
            gs = [dev.graph(f"{name}_{j}") for j in range(len(flush) + 1)]
            first_graph(gs[0])

            def stage(s):
                if s < L + 2:
                    return gs[0]
                i = L - 1 - (s - (L + 2))          # block whose backward this stage is
                return gs[sum(1 for f in flush if f > i)]
            sm_limit = dev.sm_count - int(side_sms) if side_sms > 0 else 0
            self.model.record(ids_dev, targets_dev, stage, flush_after=flush,
                              sm_limit_after_flush=sm_limit, **record_kwargs)
            for g in gs:
                g.finish()
            self.parts = bucket_parts_for_flush(replica.params, replica.offsets, replica.total,
                                                blocks, flush)
            self.side = side_comm if side_comm is not None else comm
            # the optimiser in two launches: the parameters whose sums arrive during the
            # backward, then those of the last part
            last_first = self.parts[-1][0] + self.parts[-1][1]
            early = [p for p, o in zip(replica.params, replica.offsets) if o >= last_first]
            late = [p for p, o in zip(replica.params, replica.offsets) if o < last_first]
            self.opt_graphs = []
            for tag, ps in (("a", early), ("b", late)):
                if ps:
                    go = dev.graph(f"{name}_opt{tag}")
                    self.opt.record(go, params=ps)
                    go.finish()
                    self.opt_graphs.append(go)
            if not early:
                self.opt_graphs.insert(0, None)
            self.graphs = gs + [g for g in self.opt_graphs if g is not None]
        elif comm is not None and comm.world > 1 and not in_graph:
            g = first_graph(dev.graph(name))
            self.model.record(ids_dev, targets_dev, g, **record_kwargs)
            g.finish()
            bucket, total = replica.bucket, replica.total
            self.between = lambda: comm.allreduce_sum(bucket, total)
            g_opt = dev.graph(name + "_opt")
            self.opt.record(g_opt)
            g_opt.finish()
            self.graphs = [g, g_opt]
        else:
            g = first_graph(dev.graph(name))
            self.model.record(ids_dev, targets_dev, g, **record_kwargs)
            replica.push_gradients(graph=g)
            self.opt.record(g)
            g.finish()
            self.graphs = [g]
        self.n_dispatch = sum(x.n_dispatch for x in self.graphs)
        self.n_kernels = sum(x.n_kernels for x in self.graphs)

    def enqueue(self, lr=None):
        """Advance the schedule and launch without waiting (pair with dev.sync())."""
        self.opt.advance(lr)
        if self.parts is not None:
            comm, side, bucket = self.replica.comm, self.side, self.replica.bucket
            n = len(self.parts)
            for j, (first, count) in enumerate(self.parts):
                self.graphs[j].submit_async()
                # this part of the bucket is complete: sum it beside what follows on the compute
                # stream -- the rest of the backward, or, for the last part, the optimiser over
                # the earlier parts (on the main communicator: nothing persistent runs then)
                c = side if j < n - 1 else comm
                c.side_begin()
                c.allreduce_sum_side(bucket, count, j, offset_bytes=4 * first)
            for j in range(n - 1):
                side.side_wait(j)
            if self.opt_graphs[0] is not None:
                self.opt_graphs[0].submit_async()
            comm.side_wait(n - 1)
            self.opt_graphs[1].submit_async()
            return
        self.graphs[0].submit_async()
        if self.between is not None:
            self.between()
            self.graphs[1].submit_async()

    def __call__(self, lr=None):
        lib, h = self.dev.lib, self.dev.handle
        _check(lib.vkg_timer_begin(h), "timer")
        self.enqueue(lr)
        s = C.c_double(0.0)
        _check(lib.vkg_timer_end(h, C.byref(s)), "step")
        return self.model.read_loss(), s.value


def backward_flush_points(n_blocks, groups):
    """Block indices after whose backward a group's gradients are complete: the blocks are cut
    into `groups` runs of (almost) equal length from the top; the lowest run has no flush point
    (it ends with the embedding backward).  12 blocks in 3 groups -> [8, 4]."""
    groups = max(1, min(int(groups), n_blocks))
    pts = []
    for j in range(1, groups):
        i = n_blocks - (n_blocks * j) // groups
        if 0 < i < n_blocks and i not in pts:
            pts.append(i)
    return pts


def bucket_parts_for_flush(params, offsets, total, blocks, flush):
    """[(first_float, n_floats)] of the flat bucket, in the order the parts complete during the
    backward: part 0 = blocks flush[0].. and everything after them in params() order (the final
    layernorm), part j = blocks flush[j] .. flush[j-1]-1, last part = everything below
    flush[-1] (embedding tables first in params() order, and the lowest blocks)."""
    params = list(params)
    index = {id(p): n for n, p in enumerate(params)}
    starts = []
    for f in flush:
        first = next(iter(blocks[f].params()))
        starts.append(offsets[index[id(first)]])
    parts, hi = [], total
    for st in starts:
        parts.append((st, hi - st))
        hi = st
    parts.append((0, hi))
    assert all(c > 0 for _, c in parts) and sum(c for _, c in parts) == total
    return parts


class GradAccum:
    """Gradient accumulation over microbatches on one device (dataparallel.py:153-207):
    the same sum with the workers separated in time."""

    def __init__(self, ctx, params, accum=1):
        self.ctx, self.params, self.accum = ctx, list(params), accum
        self.K = make_reduce_kernels(ctx.dev)
        offs, off = [], 0
        for p in self.params:
            offs.append(off)
            off += p.n
        self.offsets, self.total = offs, off
        self.arena = ctx.buf(off * 4, "device")

    def record_push(self, graph):
        for p, o in zip(self.params, self.offsets):
            self.K["add"]([p.g32, self.arena], p.n, o, graph=graph)

    def record_zero(self, graph):
        self.K["zero"]([self.arena], self.total, graph=graph)

    def record_apply(self, graph, opt, scale=None):
        sc = (1.0 / self.accum) if scale is None else scale
        for p, o in zip(self.params, self.offsets):
            self.K["pull"]([self.arena, p.g32], p.n, o, sc, graph=graph)
        opt.record(graph)

    def destroy(self):
        pass
