"""Host-side logic that needs no GPU: tile planning mirrors, gradient-bucket layout,
the unique-id rendezvous between two processes, and a world-size-2 data-parallel step
over gloo checked against the single-process oracle."""

import multiprocessing as mp
import os
import socket
import sys

import numpy as np
import pytest

from oracle import vkgrad_numpy as orc

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def test_pick_config_reports_reference_tiles():
    from vkgrad_b200.autograd import pick_config
    from vkgrad_b200.vk import VkError
    sg, wm, wn, lds = pick_config(256, 256, 256)
    assert 256 % (sg * wm * 16) == 0 and 256 % (wn * 16) == 0 and lds is False
    with pytest.raises(VkError):
        pick_config(24, 24, 24)


def test_matmul_reference_matches_oracle():
    from vkgrad_b200.kernels import matmul_reference
    rng = np.random.default_rng(0)
    a = rng.standard_normal((24, 40)).astype(np.float16)
    b = rng.standard_normal((40, 16)).astype(np.float16)
    assert np.array_equal(matmul_reference(a, b), orc.matmul16(a, b))
    assert np.array_equal(matmul_reference(a.T.copy(), b, trans_a=True), orc.matmul16(a, b))


def test_step_flops_matches_the_reference_dispatch_count():
    """Sum of 2*M*N*K over the 219 matmuls of a GPT-2-small step: 7.0001e12."""
    sys.path.insert(0, ROOT)
    import bench
    assert abs(bench.step_flops(8, 1024, 768, 12, 12, 50257) - 7.0001e12) < 1e9
    assert abs(bench.step_flops(4, 1024, 1024, 16, 24, 50257) - 9.9238e12) < 2e9
    table = bench.gemm_shape_table(8, 1024, 768, 12, 12, 50257, fused_attention=False)
    total = sum(c * 2.0 * s["m"] * s["n"] * s["k"] * s.get("nb", 1) for c, s in table)
    assert abs(total - bench.step_flops(8, 1024, 768, 12, 12, 50257)) < 1e6
    assert sum(c for c, _ in table) == 219
    # with the fused attention kernels the six batched matmuls per layer are not GEMM launches
    assert sum(c for c, _ in bench.gemm_shape_table(8, 1024, 768, 12, 12, 50257)) == 219 - 72


def _rdzv_worker(rank, world, port, q):
    from vkgrad_b200.dataparallel import exchange_unique_id
    uid = exchange_unique_id(rank, world, lambda: bytes(range(128)), "127.0.0.1", port, timeout=30)
    q.put((rank, uid))


def test_unique_id_rendezvous_three_processes():
    port = free_port()
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    procs = [ctx.Process(target=_rdzv_worker, args=(r, 3, port, q)) for r in range(3)]
    for p in procs:
        p.start()
    got = dict(q.get(timeout=60) for _ in range(3))
    for p in procs:
        p.join(30)
    assert all(got[r] == bytes(range(128)) for r in range(3))


def test_rendezvous_reports_a_missing_rank():
    """A rank that never joins makes rank 0 fail with an error instead of waiting forever."""
    from vkgrad_b200.dataparallel import exchange_unique_id
    from vkgrad_b200.vk import VkError
    with pytest.raises(VkError, match="only 0 of 1"):
        exchange_unique_id(0, 2, lambda: b"x" * 128, "127.0.0.1", free_port(), timeout=1.0)


def _dp_worker(rank, world, port, q):
    """One data-parallel rank on CPU: oracle gradients of its shard, gloo all-reduce of
    the flat bucket, 1/world folded into AdamW's gradient scale (as Replica does)."""
    import torch
    import torch.distributed as dist
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    x, y, params = orc.make_mlp_case(32, (32, 16), 4, 16, seed=1)
    shard = slice(rank * 16, (rank + 1) * 16)
    _, grads = orc.mlp_forward_backward(x[shard].astype(np.float32), params, y[shard], 4)
    offs, off = [], 0
    for g in grads:
        offs.append(off)
        off += (g.size + 3) // 4 * 4
    bucket = np.zeros(off, np.float32)
    for g, o in zip(grads, offs):
        bucket[o:o + g.size] = g.ravel()
    t = torch.from_numpy(bucket)
    dist.all_reduce(t)
    new = []
    for w, g, o in zip(params, grads, offs):
        summed = bucket[o:o + g.size].reshape(g.shape)
        new.append(orc.adamw_step(w, summed, 0 * w, 0 * w, 1, gscale=1.0 / world)[0])
    q.put((rank, [n.tobytes() for n in new]))
    dist.barrier()
    dist.destroy_process_group()


def test_world_size_two_step_over_gloo():
    port = free_port()
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    procs = [ctx.Process(target=_dp_worker, args=(r, 2, port, q)) for r in range(2)]
    for p in procs:
        p.start()
    got = dict(q.get(timeout=120) for _ in range(2))
    for p in procs:
        p.join(60)
    assert got[0] == got[1], "replicas diverged"                 # the reference's drift == 0
    x, y, params = orc.make_mlp_case(32, (32, 16), 4, 16, seed=1)
    shards = [orc.mlp_forward_backward(x[s].astype(np.float32), params, y[s], 4)[1]
              for s in (slice(0, 16), slice(16, 32))]
    for i, w in enumerate(params):
        mean = orc.dp_reduce([shards[0][i], shards[1][i]])
        ref = orc.adamw_step(w, mean, 0 * w, 0 * w, 1)[0]
        assert np.allclose(np.frombuffer(got[0][i], np.float32).reshape(w.shape), ref, atol=1e-6)
    # and the mean of the shard gradients is the big-batch gradient (each shard's loss is a
    # mean over its own rows, dataparallel.py:63-68)
    _, big = orc.mlp_forward_backward(x.astype(np.float32), params, y, 4)
    assert np.allclose(orc.dp_reduce([shards[0][0], shards[1][0]]), big[0], atol=1e-6)


def test_bench_reference_arm_line_shape(monkeypatch, capsys):
    """--impl reference prints one JSON line with the contract's keys (tiny workload)."""
    import json
    sys.path.insert(0, ROOT)
    import bench
    monkeypatch.setitem(bench.WORKLOADS, "tiny", (2, 32, 32, 2, 1, 50))
    monkeypatch.setattr(sys, "argv", ["bench.py", "--impl", "reference", "--steps", "2",
                                      "--warmup", "1", "--workload", "tiny"])
    ap_choices = sorted(bench.WORKLOADS)
    assert "tiny" in ap_choices
    bench.main()
    line = json.loads(capsys.readouterr().out.strip().splitlines()[-1])
    assert line["impl"] == "reference" and line["cpu_baseline"]["kind"] == "port"
    assert line["e2e"]["h2d_bytes_per_step"] == 0 and line["value"] > 0
    assert line["cpu_baseline"]["cores"] == os.cpu_count()


def test_bucket_parts_follow_the_backward_order():
    """The parts of the flat bucket a data-parallel step sums while the backward still runs:
    whole tensors, disjoint, covering the bucket, in the order their gradients complete."""
    from vkgrad_b200.dataparallel import backward_flush_points, bucket_parts_for_flush

    class P:
        def __init__(self, n):
            self.n = n

    class Blk:
        def __init__(self, ps):
            self._ps = ps

        def params(self):
            return iter(self._ps)
    tok, pos, lnf = P(1000), P(64), [P(8), P(8)]
    blocks = [Blk([P(8), P(30), P(7)]) for _ in range(12)]
    params = [tok, pos] + [p for b in blocks for p in b.params()] + lnf
    offs, off = [], 0
    for p in params:
        offs.append(off)
        off += (p.n + 3) // 4 * 4
    assert backward_flush_points(12, 3) == [8, 4]
    assert backward_flush_points(12, 1) == [] and backward_flush_points(1, 3) == []
    assert backward_flush_points(2, 8) == [1]
    parts = bucket_parts_for_flush(params, offs, off, blocks, [8, 4])
    per_block = 8 + 32 + 8
    assert parts[0] == (1000 + 64 + 8 * per_block, 4 * per_block + 16)      # blocks 8..11 + lnf
    assert parts[1] == (1000 + 64 + 4 * per_block, 4 * per_block)           # blocks 4..7
    assert parts[2] == (0, 1000 + 64 + 4 * per_block)                       # tables + blocks 0..3
    assert sum(c for _, c in parts) == off
    assert bucket_parts_for_flush(params, offs, off, blocks, []) == [(0, off)]


def test_arena_refuses_a_second_gpu_without_communicator():
    from vkgrad_b200.dataparallel import HostArena
    from vkgrad_b200.vk import VkError

    class FakeDev:
        def __init__(self, o):
            self.ordinal = o

        def buffer(self, n, kind):
            return object()
    arena = HostArena(16)
    arena.buffer_for(FakeDev(0))
    arena.buffer_for(FakeDev(0))
    with pytest.raises(VkError):
        arena.buffer_for(FakeDev(1))


# ---- bounded host waits (the analogue of the reference's 10 s fence timeout, vk.py:884-888) ----

def _wait_selftest(ready_after, error_at, timeout_s):
    import ctypes as C
    from vkgrad_b200 import _lib
    lib = _lib.load()
    aborted = C.c_int32(-1)
    rc = lib.vkg_selftest_wait_deadline(ready_after, error_at, timeout_s, C.byref(aborted))
    return rc, aborted.value, _lib.last_error()


def test_host_wait_returns_when_the_device_finishes():
    rc, aborted, _ = _wait_selftest(500, -1, 5.0)
    assert rc == 0 and aborted == 0


def test_host_wait_gives_up_at_the_deadline_and_aborts_the_communicator():
    import time
    t0 = time.perf_counter()
    rc, aborted, msg = _wait_selftest(-1, -1, 0.2)
    dt = time.perf_counter() - t0
    assert rc != 0 and aborted == 1
    assert "did not finish within" in msg and "aborted" in msg
    assert 0.2 <= dt < 2.0


def test_host_wait_reports_an_asynchronous_communicator_error_before_the_deadline():
    import time
    t0 = time.perf_counter()
    rc, aborted, msg = _wait_selftest(-1, 3, 30.0)
    assert rc != 0 and aborted == 1 and "asynchronous error" in msg
    assert time.perf_counter() - t0 < 5.0
