#!/usr/bin/env python3
"""Headline benchmark: GPT-2-small-shaped full training steps (forward + backward +
all-reduce + AdamW, fp16 operands / fp32 accumulate) on N B200s, tokens per second.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]
                    [--workload gpt2-small|gpt-24l] [--gemm-trio] [--trio-table]

N > 1 is launched one process per GPU by torch.distributed.run (RANK / LOCAL_RANK /
WORLD_SIZE / MASTER_ADDR / MASTER_PORT from the environment); ranks find each other
over a TCP socket and exchange gradients with NCCL.  Rank 0 prints ONE JSON line.

Keys beyond the base contract:
  value     device-timed (CUDA events, max over ranks) tokens/s, inputs resident in HBM
  e2e       wall-clock tokens/s through DataParallelStep.__call__ with pinned host
            inputs copied up and the per-row loss copied down every step
  roofline  all tcgen05 GEMM launches of one step, each shape timed with CUDA events
            in this process: achieved = algorithmic FLOP / time, peak = measured
            cuBLAS bf16 burst TFLOP/s of MEASURED_PEAKS.json
  kernels   the HBM-bound kernels of the step timed alone (CUDA events), against the
            measured copy bandwidth
  gaps_ms   ms_per_step minus the sum over every kernel family of count x isolated time
  gemm_trio the GEMM-trio microbench (BASELINE config 2) with numpy's sgemm beside it
  c1_mlp    the MLP step of BASELINE config 1 with its numpy twins (SGD and AdamW)
  cpu_baseline  the CPU oracle (numpy restatement of the reference's step) on a
            bounded sample, rank 0 only
`--impl reference` times that CPU oracle alone with all host threads.
"""

import argparse
import json
import os
import subprocess
import sys
import threading
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

WORKLOADS = {
    # name: (B, T, D, H, L, vocab)
    "gpt2-small": (8, 1024, 768, 12, 12, 50257),
    "gpt-24l": (4, 1024, 1024, 16, 24, 50257),
}
FALLBACK_PEAKS = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0,
                  "nvlink_gbs": 770.0}   # nvlink: peer copy per direction measured on this pool


def profile_traffic():
    """DRAM read + write bytes of one launch of the 8192x3072x768 fp32-out GEMM, read from the
    committed ncu summary of that capture (profiles/); None when the summary is absent."""
    import re
    path = os.path.join(ROOT, "profiles", "gemm_tcgen05_8192x3072x768_ncu_full.md")
    note = ("ncu dram__bytes_read.sum + dram__bytes_write.sum of ONE launch of the 8192x3072x768 "
            "fp32-out shape (algorithmic minimum 118 MB; much of the output is still in L2 when "
            "the kernel ends), parsed from profiles/gemm_tcgen05_8192x3072x768_ncu_full.md")
    try:
        with open(path) as f:
            m = re.search(r"traffic \(read \+ write\)\s*\|\s*([0-9.]+)\s*MB", f.read())
        if m:
            return float(m.group(1)) * 1e6, note
    except OSError:
        pass
    return None, "no ncu summary of the GEMM found under profiles/"


def load_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            return json.load(f), "measured"
    return dict(FALLBACK_PEAKS), "fallback"


def step_flops(B, T, D, H, L, V):
    """Algorithmic FLOP of one step: 2*M*N*K over every matmul the reference records
    (full T x T attention, tied head)."""
    R, hd, Vp = B * T, D // H, (V + 15) // 16 * 16
    per_layer = 3 * 2 * R * D * (3 * D + D + 4 * D + 4 * D)      # fwd + dW + dX of four linears
    per_layer += 6 * 2 * (B * H) * T * T * hd                     # six batched attention matmuls
    head = 3 * 2 * R * D * Vp
    return L * per_layer + head


class ClockSampler:
    """nvidia-smi clock / throttle samples while the timed region runs."""
    Q = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
         "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
         "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index):
        self.rows, self.proc = [], None
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits",
                 "-i", str(index), "-lms", "100"], stdout=subprocess.PIPE, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append((time.perf_counter(), [c.strip() for c in line.split(",")]))

    def stop(self, t0, t1):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.15)
        self.proc.terminate()
        rows = [r for t, r in self.rows if t0 <= t <= t1 + 0.2] or [r for _, r in self.rows[-3:]]
        sm = [float(r[0]) for r in rows if r and r[0].replace(".", "").isdigit()]
        mx = [float(r[1]) for r in rows if len(r) > 1 and r[1].replace(".", "").isdigit()]
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        reasons = set()
        for r in rows:
            for nm, v in zip(names, r[4:8]):
                if v.lower().startswith("active"):
                    reasons.add(nm)
        return {"sm_mhz": float(np.median(sm)) if sm else None,
                "sm_max_mhz": max(mx) if mx else None, "reasons": sorted(reasons),
                "samples": len(rows)}


# ---- CPU oracle arm ---------------------------------------------------------------------
#
# The CPU figure is one number, taken one way by both arms: forward + backward of the full
# model on ONE sequence of the real context length (1 x T tokens; fewer only if the time
# budget forces it), and AdamW over every parameter timed by itself, because the optimiser
# is paid once per step whatever the batch.  tokens/s is then quoted for the benchmark's
# batch: B*T / (B * t_fwd_bwd(1 x T) + t_adamw).

_CPU_STATE = {}


def _cpu_state(T, D, H, L, V, seed=0):
    from oracle import vkgrad_numpy as orc
    Vp = (V + 15) // 16 * 16
    key = (T, D, H, L, Vp, seed)
    if _CPU_STATE.get("key") != key:
        _CPU_STATE.clear()
        P = orc.make_gpt_params(D, H, L, T, Vp, seed=seed, tie=True)
        flat = [("tok", None), ("pos", None), ("lnf.g", None), ("lnf.b", None)]
        flat += [(f"b{l}", k) for l in range(L) for k in P[f"b{l}"]]
        get = lambda k, kk: P[k] if kk is None else P[k][kk]
        _CPU_STATE.update(key=key, P=P, flat=flat, t=0,
                          m={f: np.zeros_like(get(*f)) for f in flat},
                          v={f: np.zeros_like(get(*f)) for f in flat})
    return _CPU_STATE


def cpu_step_seconds(B, T, D, H, L, V, seed=0):
    """One oracle step at batch B: (seconds forward+backward, seconds AdamW, loss)."""
    from oracle import vkgrad_numpy as orc
    st = _cpu_state(T, D, H, L, V, seed)
    P = st["P"]
    rng = np.random.default_rng(seed + 1 + st["t"])
    ids = rng.integers(0, V, B * T).astype(np.uint32)
    tgt = rng.integers(0, V, B * T).astype(np.uint32)
    t0 = time.perf_counter()
    loss, G, _ = orc.gpt_forward_backward(P, ids, tgt, B, T, D, H, L, V)
    G["tok"] = G["tok"] + G.pop("head.W").T
    G.pop("head.b")
    t1 = time.perf_counter()
    st["t"] += 1
    for k, kk in st["flat"]:
        w, g = (P[k], G[k]) if kk is None else (P[k][kk], G[k][kk])
        out = orc.adamw_step(w, g, st["m"][(k, kk)], st["v"][(k, kk)], st["t"], lr=6e-4,
                             wd=0.01 if w.ndim == 2 else 0.0)
        if kk is None:
            P[k] = out[0]
        else:
            P[k][kk] = out[0]
        st["m"][(k, kk)], st["v"][(k, kk)] = out[1], out[2]
    P["head.W"] = P["tok"].T
    t2 = time.perf_counter()
    return t1 - t0, t2 - t1, loss


def cpu_sample_T(name, budget_s, n_steps):
    """Longest sequence (the real context length if it fits) whose n_steps fit the budget.
    The probe step is a real one and is returned so that it is not wasted."""
    B, T, D, H, L, V = WORKLOADS[name]
    fb, ad, _ = cpu_step_seconds(1, T, D, H, L, V)
    if (fb + ad) * n_steps <= budget_s:
        return T, (fb, ad)
    for cand in (T // 2, T // 4, T // 8):
        # forward/backward shrink about linearly with the tokens, AdamW does not shrink
        if (fb * cand / T + ad) * n_steps <= budget_s:
            return cand, None
    return T // 16, None


def cpu_line_fields(name, fb, ad, st):
    """tokens/s for the benchmark's batch from the per-sequence and per-step parts."""
    B, T, D, H, L, V = WORKLOADS[name]
    seqs = B * T / st                     # samples of st tokens in one step of the real batch
    step_s = seqs * fb + ad
    sample = (f"forward+backward of the full {L}-layer model on 1x{st} tokens "
              f"({fb * 1e3:.0f} ms) and AdamW over every parameter ({ad * 1e3:.0f} ms), "
              f"numpy oracle restating the reference's np_model; quoted for the batch of "
              f"{B}x{T} tokens as {B * T} / ({seqs:.0f} x fwd_bwd + adamw)")
    return B * T / step_s, step_s, sample


def run_reference_arm(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    name = args.workload
    B, T, D, H, L, V = WORKLOADS[name]
    st, probe = cpu_sample_T(name, 240.0, args.steps + args.warmup)
    done = 1 if (probe is not None and st == T) else 0     # the probe was a warm-up step
    for _ in range(max(args.warmup - done, 0)):
        cpu_step_seconds(1, st, D, H, L, V)
    fb_sum = ad_sum = 0.0
    t0 = time.perf_counter()
    for _ in range(args.steps):
        fb, ad, _ = cpu_step_seconds(1, st, D, H, L, V)
        fb_sum += fb
        ad_sum += ad
    dt = time.perf_counter() - t0
    fb, ad = fb_sum / args.steps, ad_sum / args.steps
    tok_s, step_s, sample = cpu_line_fields(name, fb, ad, st)
    cores = os.cpu_count()
    from oracle import vkgrad_numpy as orc
    mm_only = orc.matmuls_only_step_seconds(1, st, D, H, L, (V + 15) // 16 * 16)
    line = {
        "impl": "reference", "metric": "gpt_train_tokens_per_s", "value": tok_s, "unit": "tokens/s",
        "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": step_s * 1e3, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": workload_config(name, 1, float(args.loss_scale)),
        "cpu_baseline": {"value": tok_s, "unit": "tokens/s", "cores": cores, "kind": "port",
                         "sample": sample, "fwd_bwd_s": fb, "adamw_s": ad, "sample_tokens": st,
                         "measured_s": dt,
                         "matmuls_only_tokens_per_s": st / mm_only,
                         "matmuls_only_note": "examples/charlm.py:60-96 restated: the reference's "
                                              "own lower bound, dominant forward matmuls only"},
        "e2e": {"value": tok_s, "unit": "tokens/s", "h2d_bytes_per_step": 0,
                "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


def workload_config(name, world, loss_scale):
    B, T, D, H, L, V = WORKLOADS[name]
    return {"workload": name, "layers": L, "d_model": D, "heads": H, "ctx": T, "vocab": V,
            "tied": True, "batch_per_gpu": f"{B}x{T}", "global_batch_tokens": B * T * world,
            "parallelism": f"dp{world}", "loss_scale": loss_scale, "optimizer": "AdamW",
            "l2": "working set per step >> 126 MB L2 (no flush needed)"}


# ---- GPU arm ---------------------------------------------------------------------------------

def gemm_shape_table(B, T, D, H, L, V, fused_attention=True):
    """(count per step, shape) for every distinct launch of gemm_tcgen05_kernel in a step.
    With head dimension 64 attention runs in the fused attention kernels, so the six
    batched matmuls per layer of the reference's plan are not GEMM launches here."""
    R, hd, Vp = B * T, D // H, (V + 15) // 16 * 16
    t = []
    for (i, o) in ((D, 3 * D), (D, D), (D, 4 * D), (4 * D, D)):
        t.append((L, dict(m=R, n=o, k=i, ta=False, tb=False)))          # Y  = X W
        t.append((L, dict(m=i, n=o, k=R, ta=True, tb=False, grouped=True)))   # dW = X^T dY
        t.append((L, dict(m=R, n=i, k=o, ta=False, tb=True)))           # dX = dY W^T
    if not fused_attention:
        nb = B * H
        t.append((2 * L, dict(m=T, n=T, k=hd, ta=False, tb=True, nb=nb, causal=1)))   # QK^T, dP
        t.append((2 * L, dict(m=T, n=hd, k=T, ta=False, tb=False, nb=nb, causal=2)))  # PV, dQ
        t.append((2 * L, dict(m=T, n=hd, k=T, ta=True, tb=False, nb=nb, causal=3)))   # dV, dK
    t.append((1, dict(m=R, n=Vp, k=D, ta=False, tb=True)))              # logits
    t.append((1, dict(m=R, n=D, k=Vp, ta=False, tb=False)))             # dh
    t.append((1, dict(m=Vp, n=D, k=R, ta=True, tb=False)))              # dtok (head share)
    return t


def time_attention(dev, B, T, H, hd):
    """CUDA-event time of the fused attention forward and backward for one layer, on N(0,1)
    q/k/v and dO, with the qkv bias-gradient sums folded in as in the training step (their
    short final pass is collected, not launched, also as in the step)."""
    from vkgrad_b200.vk import _check
    D = H * hd
    lib, h = dev.lib, dev.handle
    qkv = dev.buffer(B * T * 3 * D * 2, "device")
    dout = dev.buffer(B * T * D * 2, "device")
    out = dev.buffer(B * T * D * 2, "device")
    dqkv = dev.buffer(B * T * 3 * D * 2, "device")
    lse = dev.buffer(B * H * T * 4, "device")
    delta = dev.buffer(B * H * T * 4, "device")
    dbias = dev.buffer(3 * D * 4, "device")
    scratch = dev.buffer(4 * lib.vkg_attn_bwd_dbias_scratch_floats(B, T, H, hd), "device")
    fill_random16(dev, qkv)
    fill_random16(dev, dout)
    scale = 1.0 / np.sqrt(hd)

    def fwd():
        _check(lib.vkg_attn_fwd(h, qkv.dptr, None, out.dptr, lse.dptr, B, T, H, hd, scale), "fwd")

    def bwd():
        _check(lib.vkg_attn_bwd(h, qkv.dptr, dout.dptr, out.dptr, lse.dptr, None, dqkv.dptr,
                                delta.dptr, dbias.dptr, scratch.dptr, B, T, H, hd, scale), "bwd")
    res = {}
    _check(lib.vkg_finals_defer(h, 1), "defer")
    for name, fn in (("fwd_us", fwd), ("bwd_us", bwd)):
        dev.run_op(fn, 2)
        res[name] = min(dev.run_op(fn, 10) / 10 for _ in range(3)) * 1e6
    _check(lib.vkg_finals_defer(h, -1), "defer off")
    flop = 2.0 * (B * H) * T * T * hd
    res["fwd_tflops_full_TxT"] = 2 * flop / res["fwd_us"] / 1e6
    res["bwd_tflops_full_TxT"] = 4 * flop / res["bwd_us"] / 1e6
    for b in (qkv, dout, out, dqkv, lse, delta, dbias, scratch):
        b.destroy()
    return res


def time_row_kernels(dev, rep, hbm_gbs):
    """The HBM-bound kernels of the step timed alone on the model's own buffers (rotating over
    the layers so that the working set is larger than L2).  Returns {name: {us, count,
    bytes, gbs, frac_hbm}}; bytes are the algorithmic bytes per launch."""
    from vkgrad_b200.vk import _check
    lib, h = dev.lib, dev.handle
    m, opt = rep.model, rep.opt
    R, D, V, Vp, L, T = m.rows, m.D, m.vocab, m.pad_vocab, len(m.blocks), m.T
    out = {}

    def timed(fns, reps=4):
        def go():
            for f in fns:
                f()
        dev.run_op(go, 1)
        return min(dev.run_op(go, reps) / (reps * len(fns)) for _ in range(3))

    def entry(name, t, count, nbytes):
        out[name] = {"us": t * 1e6, "count": count, "bytes": nbytes, "gbs": nbytes / t / 1e9,
                     "frac_hbm": nbytes / t / 1e9 / hbm_gbs}

    lns = [ln for b in m.blocks for ln in (b.ln1, b.ln2)] + [m.lnf]
    fwd = [lambda ln=ln: _check(lib.vkg_layernorm(h, ln.x32.dptr, ln.g.w32.dptr, ln.b.w32.dptr,
                                                  ln.y16.dptr, ln.mu.dptr, ln.rstd.dptr, R, D), "ln")
           for ln in lns]
    entry("layernorm", timed(fwd), len(lns), R * D * 6 + R * 8)
    if all(ln._scratch is not None for ln in lns):
        _check(lib.vkg_finals_defer(h, 1), "defer")
        n = len(lns)
        bwd = [lambda ln=ln, dy=lns[(i + 1) % n].dx, dres=lns[(i + 2) % n].dx: _check(
            lib.vkg_layernorm_bwd(h, dy.dptr, ln.x32.dptr, ln.g.w32.dptr, ln.mu.dptr, ln.rstd.dptr,
                                  dres.dptr, ln.dx.dptr, ln.dx16.dptr, None, None, ln.g.g32.dptr,
                                  ln.b.g32.dptr, None, ln._scratch.dptr, R, D), "ln_bwd")
               for i, ln in enumerate(lns)]
        entry("layernorm_bwd", timed(bwd, reps=2), len(lns), R * D * 18)
        # the collected final passes: as many entries as a step collects (2 per block + 1
        # from layernorm, 1 per block each from attention and the fc2-dX epilogue)
        _check(lib.vkg_finals_defer(h, -1), "drop")
        n_fin = (2 * L + 1) + 2 * L
        _check(lib.vkg_finals_defer(h, 1), "defer")
        for f in (bwd * 3)[:n_fin]:
            f()
        dev.sync()
        t_fin = dev.run_op(lambda: _check(lib.vkg_finals_flush(h), "flush"), 1)
        entry("finals", t_fin, 1, n_fin * 3 * D * 4 * 256)
    scale = m.loss_scale / R
    ce = lambda: _check(lib.vkg_softmax_ce(h, m.logits.dptr, rep_targets(rep).dptr, None,
                                           m.dlog16.dptr, None, m.loss.dptr, R, Vp, V, scale), "ce")
    entry("softmax_ce", timed([ce], reps=3), 1, R * Vp * 6)
    table = opt._get_table(opt.params)
    n_par = sum(p.n for p in opt.params)
    ad = lambda: _check(lib.vkg_adamw_multi(h, table, opt.hp.dptr), "adamw")
    entry("adamw", timed([ad], reps=3), 1, n_par * 30)
    ids = rep_ids(rep)
    emb = lambda: _check(lib.vkg_embed(h, m.tok.w32.dptr, m.pos.w32.dptr, ids.dptr, None,
                                       m.x0.dptr, R * D, D, T), "embed")
    entry("embed", timed([emb]), 1, R * D * 12)

    def emb_bwd():
        _check(lib.vkg_memset0(h, m.pos.g32.dptr, m.pos.n * 4), "zero")
        _check(lib.vkg_embed_bwd(h, m.x0.dptr, ids.dptr, None, m.tok.g32.dptr, m.pos.g32.dptr,
                                 R * D, D, T), "embed_bwd")
    entry("embed_bwd", timed([emb_bwd]), 1, R * D * 12)
    return out


def rep_ids(rep):
    return rep._bench_ids


def rep_targets(rep):
    return rep._bench_targets


_RANDOM_BLOCKS = {}


def fill_random16(dev, buf, scale=1.0):
    """Fill a device buffer with N(0, scale^2) fp16 values: timings on zero operands would
    flatter a power-limited tensor core."""
    blk = _RANDOM_BLOCKS.get(scale)
    if blk is None:
        blk = (np.random.default_rng(7).standard_normal(8 << 20) * scale).astype(np.float16)
        _RANDOM_BLOCKS[scale] = blk
    for off in range(0, buf.size, blk.nbytes):
        n = min(blk.nbytes, buf.size - off)
        rc = dev.lib.vkg_upload(dev.handle, buf.dptr + off, blk.ctypes.data, n)
        if rc:
            raise RuntimeError("upload of random operands failed")


def time_gemm_shapes(dev, table):
    """CUDA-event time of each shape (back-to-back launches on the device stream)."""
    from vkgrad_b200.kernels import gemm, gemm_group
    total_t, total_f, rows = 0.0, 0.0, []
    # the blocks' dW GEMMs run as ONE grouped launch in the step: time them that way, every
    # problem on its own operands
    grouped = [(count, s) for count, s in table if s.get("grouped")]
    if grouped:
        probs, bufs, fl = [], [], 0.0
        for count, s in grouped:
            m, n, k = s["m"], s["n"], s["k"]
            for _ in range(count):
                a, b, c = dev.buffer(m * k * 2, "device"), dev.buffer(k * n * 2, "device"), \
                    dev.buffer(m * n * 4, "device")
                fill_random16(dev, a)
                fill_random16(dev, b)
                bufs += [a, b, c]
                probs.append((a, b, c, m, n, k, dict(trans_a=True)))
                fl += 2.0 * m * n * k
        gemm_group(dev, probs, repeat=2)
        t = min(gemm_group(dev, probs, repeat=5) / 5 for _ in range(3))
        rows.append({"grouped_dw_problems": len(probs), "us": t * 1e6, "tflops": fl / t / 1e12})
        total_t += t
        total_f += fl
        for x in bufs:
            x.destroy()
    for count, s in table:
        if s.get("grouped"):
            continue
        nb = s.get("nb", 1)
        m, n, k = s["m"], s["n"], s["k"]
        a = dev.buffer(nb * m * k * 2, "device")
        b = dev.buffer(nb * k * n * 2, "device")
        c = dev.buffer(nb * m * n * 4, "device")
        fill_random16(dev, a)
        fill_random16(dev, b)
        kw = dict(trans_a=s["ta"], trans_b=s["tb"], nb0=nb, sa=(m * k, 0), sb=(k * n, 0),
                  sc=(m * n, 0), causal=s.get("causal", 0))
        gemm(dev, a, b, c, m, n, k, repeat=2, **kw)
        reps = 10
        t = min(gemm(dev, a, b, c, m, n, k, repeat=reps, **kw) / reps for _ in range(3))
        fl = 2.0 * m * n * k * nb
        rows.append({"m": m, "n": n, "k": k, "ta": int(s["ta"]), "tb": int(s["tb"]), "batch": nb,
                     "count": count, "us": t * 1e6, "tflops": fl / t / 1e12})
        total_t += count * t
        total_f += count * fl
        for x in (a, b, c):
            x.destroy()
    return total_f, total_t, rows


def library_gemm_rows(dev):
    """Four of the step's GEMM shapes through vkg_gemm (the fastest of its own choice and the two
    kernels a caller may force) and through the library GEMM (torch.mm -> cuBLAS)
    in the same process, with fp32 and with fp16 outputs: like for like, since an fp32 output
    costs both the same 64 KB more per 128 x 256 tile.  For orientation only: torch is on no
    path of the product, and the section says so if it cannot be imported."""
    from vkgrad_b200._lib import F16, F32
    from vkgrad_b200.kernels import gemm
    try:
        import torch
        torch.backends.cuda.matmul.allow_fp16_reduced_precision_reduction = False
        torch.zeros(1, device="cuda")
    except Exception as e:      # no torch, or torch without this GPU: report, do not fail the bench
        return {"unavailable": repr(e)[:120]}

    def lib_time(f):
        for _ in range(3):
            f()
        torch.cuda.synchronize()
        best = None
        for _ in range(3):
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            for _ in range(10):
                f()
            e1.record()
            torch.cuda.synchronize()
            t = e0.elapsed_time(e1) / 10 * 1e3
            best = t if best is None else min(best, t)
        return best

    rows = []
    for m, n, k, tb in ((8192, 2304, 768, False), (8192, 3072, 768, False), (8192, 768, 768, False),
                        (8192, 768, 3072, True)):
        a, b, c = dev.buffer(m * k * 2, "device"), dev.buffer(k * n * 2, "device"), \
            dev.buffer(m * n * 4, "device")
        fill_random16(dev, a)
        fill_random16(dev, b)
        row = {"m": m, "n": n, "k": k, "tb": int(tb)}
        for tag, cd in (("f32", F32), ("f16", F16)):
            best = None
            for pair in (0, -1, 1):
                kw = dict(trans_b=tb, c_dtype=cd, cta_pair=pair)
                gemm(dev, a, b, c, m, n, k, repeat=2, **kw)
                t = min(gemm(dev, a, b, c, m, n, k, repeat=10, **kw) / 10 for _ in range(3)) * 1e6
                best = t if best is None else min(best, t)
            row["ours_%s_us" % tag] = best
        for x in (a, b, c):
            x.destroy()
        ta_ = torch.randn(m, k, device="cuda", dtype=torch.float16)
        tb_ = torch.randn((n, k) if tb else (k, n), device="cuda", dtype=torch.float16)
        rhs = tb_.t() if tb else tb_
        row["lib_f16_us"] = lib_time(lambda: torch.mm(ta_, rhs))
        try:
            row["lib_f32_us"] = lib_time(lambda: torch.mm(ta_, rhs, out_dtype=torch.float32))
        except Exception as e:  # an older torch without out_dtype
            row["lib_f32_us"] = None
            row["lib_f32_note"] = repr(e)[:80]
        del ta_, tb_, rhs
        rows.append(row)
    return {"rows": rows, "note": "us per launch, best of 3 rounds of 10, N(0,1) operands; ours = "
            "the best of vkg_gemm's own choice, the single-CTA kernel and 256x256 CTA-pair tiles; "
            "lib = torch.mm (cuBLAS)"}


TRIO_SHAPES = [(m, k, n) for m in (4096, 16384)
               for (k, n) in ((768, 768), (768, 3072), (3072, 768), (1024, 4096))]


def trio_summary(dev, peak, warm=3, reps=11, with_cpu=True):
    """The GEMM-trio microbench: Y = X W, dX = dY W^T, dW = X^T dY with fp32 outputs on
    M in {4096, 16384} x four (K, N); X, dY ~ N(0,1), W ~ N(0, 1/K).  With with_cpu the same
    products through numpy's sgemm on the widened operands (kernels.py:606-610), one pass."""
    from vkgrad_b200.kernels import gemm
    rows, tot_f, tot_t, cpu_f, cpu_t = [], 0.0, 0.0, 0.0, 0.0
    rng = np.random.default_rng(5)
    for m, k, n in TRIO_SHAPES:
        x, w, dy = dev.buffer(m * k * 2, "device"), dev.buffer(k * n * 2, "device"), \
            dev.buffer(m * n * 2, "device")
        out = dev.buffer(4 * max(m * n, m * k, k * n), "device")
        fill_random16(dev, x)
        fill_random16(dev, dy)
        fill_random16(dev, w, scale=float(k) ** -0.5)
        ops = [("Y", (x, w, out, m, n, k), {}),
               ("dX", (dy, w, out, m, k, n), {"trans_b": True}),
               ("dW", (x, dy, out, k, n, m), {"trans_a": True})]
        for name, a, kw in ops:
            gemm(dev, *a, repeat=warm, **kw)
            t = min(gemm(dev, *a, repeat=reps, **kw) / reps for _ in range(3))
            fl = 2.0 * m * n * k
            rows.append({"op": name, "m": m, "k": k, "n": n, "us": t * 1e6, "tflops": fl / t / 1e12,
                         "frac_of_peak": fl / t / 1e12 / peak})
            tot_f += fl
            tot_t += t
        for b in (x, w, dy, out):
            b.destroy()
        if with_cpu:
            xs = rng.standard_normal((m, k)).astype(np.float16).astype(np.float32)
            ws = rng.standard_normal((k, n)).astype(np.float16).astype(np.float32)
            ds = rng.standard_normal((m, n)).astype(np.float16).astype(np.float32)
            for a, b in ((xs, ws), (ds, ws.T), (xs.T, ds)):
                t0 = time.perf_counter()
                np.matmul(a, b)
                cpu_t += time.perf_counter() - t0
                cpu_f += 2.0 * m * n * k
    worst = min(rows, key=lambda r: r["tflops"])
    best = max(rows, key=lambda r: r["tflops"])
    res = {"tflops": tot_f / tot_t / 1e12, "frac_of_peak": tot_f / tot_t / 1e12 / peak,
           "cases": len(rows), "out_dtype": "f32", "worst": worst, "best": best, "rows": rows}
    if with_cpu:
        res["cpu_baseline"] = {"value": cpu_f / cpu_t / 1e12, "unit": "TFLOP/s",
                               "cores": os.cpu_count(), "kind": "port",
                               "sample": "the same 24 products once each through numpy sgemm"}
    return res


def run_trio_table(args):
    """--trio-table: the GEMM-trio microbench alone, one JSON line."""
    from vkgrad_b200 import vk
    dev = vk.Device(0)
    peaks, peak_src = load_peaks()
    peak = float(peaks.get("bf16_tflops", FALLBACK_PEAKS["bf16_tflops"]))
    r = trio_summary(dev, peak, max(args.warmup, 3), max(args.steps, 11), not args.no_cpu)
    print(json.dumps({"metric": "gemm_trio_tflops", "value": r["tflops"], "unit": "TFLOP/s",
                      "n_gpus": 1, "higher_is_better": True, "dtype": "f16", "data": "synthetic",
                      "config": {"workload": "gemm-trio", "shapes": len(TRIO_SHAPES), "ops": 3,
                                 "out_dtype": "f32"},
                      "roofline": {"bound": "tensor", "achieved": r["tflops"], "peak": peak,
                                   "unit": "TFLOP/s", "frac": r["frac_of_peak"],
                                   "peak_source": peak_src},
                      "cpu_baseline": r.get("cpu_baseline"), "rows": r["rows"]}), flush=True)
    dev.destroy()


def c5_summary(dev, steps=5, warmup=3):
    """BASELINE config 5: the 24-layer d_model 1024 / 16 heads decoder (354.8 M parameters with
    the tied embedding), 4 x 1024 tokens, one recorded step (forward + backward + AdamW)
    replayed `steps` times with resident inputs."""
    import ctypes as C
    from vkgrad_b200 import vk
    from vkgrad_b200.autograd import AdamW
    from vkgrad_b200.dataparallel import DataParallelStep, Replica
    from vkgrad_b200.transformer import GPT, TCtx
    B, T, D, H, L, V = WORKLOADS["gpt-24l"]
    R = B * T

    def build(d):
        ctx = TCtx(d)
        model = GPT(ctx, B, T, D, H, L, V, tie=True, loss_scale=4096.0)
        rng = np.random.default_rng(0)
        for p in model.params():
            if p.name.endswith(".g"):
                p.set(np.ones(p.shape, np.float32))
            elif len(p.shape) == 1:
                p.set(np.zeros(p.shape, np.float32))
            else:
                p.set((rng.standard_normal(p.shape) * 0.02).astype(np.float32))
        opt = AdamW(ctx, model.params(), lr=6e-4, wd=0.01)
        return ctx, model, opt, ctx.buf(R * 4, "shared"), ctx.buf(R * 4, "shared")
    rep = Replica(dev, build)
    try:
        ids, tgt = rep.ctx.buf(R * 4), rep.ctx.buf(R * 4)
        rng = np.random.default_rng(5)
        rep.xbuf.array(np.uint32)[:] = rng.integers(0, V, R)
        rep.ybuf.array(np.uint32)[:] = rng.integers(0, V, R)
        dev.copy(rep.xbuf, ids, R * 4)
        dev.copy(rep.ybuf, tgt, R * 4)
        step = DataParallelStep(rep, ids, tgt, name="c5")
        for _ in range(warmup):
            step.enqueue(6e-4)
        dev.sync()
        vk._check(dev.lib.vkg_timer_begin(dev.handle), "timer")
        for _ in range(steps):
            step.enqueue(6e-4)
        sec = C.c_double(0.0)
        vk._check(dev.lib.vkg_timer_end(dev.handle, C.byref(sec)), "timer")
        ms = sec.value / steps * 1e3
        n_par = rep.model.n_params()
        return {"workload": "gpt-24l: 24 layers, d_model 1024, 16 heads, ctx 1024, vocab 50257 tied, "
                            "batch 4x1024", "params": n_par, "ms_per_step": ms,
                "tokens_per_s": R / (ms * 1e-3), "launches_per_step": step.n_kernels,
                "algorithmic_tflop_per_step": step_flops(B, T, D, H, L, V) / 1e12,
                "loss": rep.model.read_loss()}
    finally:
        rep.destroy()


def c1_mlp_summary(dev, with_cpu=True, steps=200):
    """BASELINE config 1: MLP 784-256-256-10 (ReLU, softmax cross-entropy, AdamW lr 1e-3),
    batch 256, one recorded training step replayed `steps` times; beside it the numpy step of
    examples/mnist.py:83-118 on the same shape, with its SGD update and with AdamW."""
    import ctypes as C
    from oracle import vkgrad_numpy as orc
    from vkgrad_b200.autograd import MLP, AdamW, Ctx, TrainStep
    from vkgrad_b200.vk import _check
    x, y, params = orc.make_mlp_case(256, (784, 256, 256), 10, 16, seed=0)
    ctx = Ctx(dev)
    try:
        model = MLP(ctx, 256, [784, 256, 256], 10, pad_classes=16, act="relu")
        for p, w in zip(model.params(), params):
            p.set(w)
        xb, yb = ctx.buf(x.size * 2, "shared"), ctx.buf(256 * 4, "shared")
        xb.array(np.float16, x.shape)[:] = x
        yb.array(np.uint32, (256,))[:] = y
        opt = AdamW(ctx, model.params(), lr=1e-3)
        step = TrainStep(model, opt, xb, yb)
        first, _ = step(1e-3)
        for _ in range(20):
            opt.advance(1e-3)
            step.graph.submit_async()
        dev.sync()
        _check(dev.lib.vkg_timer_begin(dev.handle), "timer")
        for _ in range(steps):
            opt.advance(1e-3)
            step.graph.submit_async()
        sec = C.c_double(0.0)
        _check(dev.lib.vkg_timer_end(dev.handle, C.byref(sec)), "timer")
        res = {"workload": "mlp 784-256-256-10 relu, batch 256, AdamW", "us_per_step":
               sec.value / steps * 1e6, "samples_per_s": 256 * steps / sec.value,
               "launches_per_step": step.graph.n_kernels, "loss_first": first,
               "loss_last": model.read_loss()}
    finally:
        ctx.destroy()
    if with_cpu:
        sgd = orc.mlp_train_step_seconds(x, y, params, 10, act="relu", optimizer="sgd")
        adw = orc.mlp_train_step_seconds(x, y, params, 10, act="relu", optimizer="adamw")
        res["cpu_baseline"] = {"sgd_us_per_step": sgd * 1e6, "adamw_us_per_step": adw * 1e6,
                               "value": 256 / adw, "unit": "samples/s", "cores": os.cpu_count(),
                               "kind": "port", "sample": "best of 20 numpy steps, same shape"}
    return res


def run_single_gemm(args):
    """--gemm M,N,K,ta,tb,batch[,c16]: one GEMM shape, `steps` launches; for ncu captures."""
    from vkgrad_b200 import vk
    from vkgrad_b200._lib import F16, F32
    from vkgrad_b200.kernels import gemm
    vals = [int(x) for x in args.gemm.split(",")]
    m, n, k, ta, tb, nb = vals[:6]
    c16 = len(vals) > 6 and vals[6]
    dev = vk.Device(0)
    a = dev.buffer(nb * m * k * 2, "device")
    b = dev.buffer(nb * k * n * 2, "device")
    c = dev.buffer(nb * m * n * 4, "device")
    fill_random16(dev, a)
    fill_random16(dev, b)
    kw = dict(trans_a=bool(ta), trans_b=bool(tb), nb0=nb, sa=(m * k, 0), sb=(k * n, 0),
              sc=(m * n, 0), c_dtype=F16 if c16 else F32, tile_n=args.tile_n, split_k=args.split_k,
              max_ctas=args.max_ctas, cta_pair=args.cta_pair)
    gemm(dev, a, b, c, m, n, k, repeat=max(args.warmup, 1), **kw)
    t = gemm(dev, a, b, c, m, n, k, repeat=args.steps, **kw) / args.steps
    print(json.dumps({"gemm": args.gemm, "us": t * 1e6,
                      "tflops": 2.0 * m * n * k * nb / t / 1e12}), flush=True)
    dev.destroy()


def run_single_attention(args):
    """--attn B,T,H: the fused attention forward and backward of one layer alone, `steps`
    launches each on N(0,1) q/k/v and dO; for ncu captures with a small footprint."""
    from vkgrad_b200 import vk
    B, T, H = [int(x) for x in args.attn.split(",")[:3]]
    dev = vk.Device(0)
    res = None
    for _ in range(max(args.steps, 1)):
        res = time_attention(dev, B, T, H, 64)
    print(json.dumps({"attn": args.attn, **res}), flush=True)
    dev.destroy()


def run_gpu_arm(args):
    from vkgrad_b200 import vk
    from vkgrad_b200.autograd import AdamW
    from vkgrad_b200.dataparallel import Comm, DataParallelStep, Replica
    from vkgrad_b200.transformer import GPT, TCtx

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if world > 1:
        # a rank stuck in rendezvous or a collective dumps every thread's stack and exits
        import faulthandler
        faulthandler.dump_traceback_later(args.watchdog, exit=True)
    if world != args.gpus:
        if world == 1 and args.gpus > 1:
            raise SystemExit("--gpus N > 1 needs one process per GPU: launch with "
                             "python -m torch.distributed.run --nproc-per-node N bench.py ...")
    name = args.workload
    B, T, D, H, L, V = WORKLOADS[name]
    R = B * T
    peaks, peak_src = load_peaks()

    dev = vk.Device(local)
    if args.pdl is not None:
        vk._check(dev.lib.vkg_set_pdl(dev.handle, int(args.pdl)), "set_pdl")
    # N > 1: the communicator of the compute stream and, for the parts of the exchange that run
    # beside the backward, a second one held to a few CTAs
    comm = side = None
    groups = args.overlap_groups if world > 1 else 1
    if world > 1 and groups > 1 and args.side_ctas > 0:
        comm, side = Comm.pair_from_env(dev, args.side_ctas)
        if side is None:
            groups = 1          # no limited communicator: one all-reduce after the backward
    elif world > 1:
        comm = Comm.from_env(dev)
    loss_scale = float(args.loss_scale)

    def build(d):
        ctx = TCtx(d)
        model = GPT(ctx, B, T, D, H, L, V, tie=True, loss_scale=loss_scale)
        rng = np.random.default_rng(0)          # identical weights on every rank
        for p in model.params():
            if p.name.endswith(".g"):
                p.set(np.ones(p.shape, np.float32))
            elif len(p.shape) == 1:
                p.set(np.zeros(p.shape, np.float32))
            else:
                p.set((rng.standard_normal(p.shape) * 0.02).astype(np.float32))
        opt = AdamW(ctx, model.params(), lr=6e-4, wd=0.01)
        return ctx, model, opt, ctx.buf(R * 4, "shared"), ctx.buf(R * 4, "shared")

    rep = Replica(dev, build, comm=comm)
    ctx, model = rep.ctx, rep.model
    ids_dev, tgt_dev = ctx.buf(R * 4), ctx.buf(R * 4)
    rep._bench_ids, rep._bench_targets = ids_dev, tgt_dev
    ids_host, tgt_host = rep.xbuf, rep.ybuf
    rng = np.random.default_rng(1000 + rank)    # each rank its own token stream
    batches = [(rng.integers(0, V, R).astype(np.uint32), rng.integers(0, V, R).astype(np.uint32))
               for _ in range(4)]
    ids_host.array(np.uint32)[:] = batches[0][0]
    tgt_host.array(np.uint32)[:] = batches[0][1]
    dev.copy(ids_host, ids_dev, R * 4)
    dev.copy(tgt_host, tgt_dev, R * 4)

    dp_kw = dict(overlap_groups=groups, side_comm=side, side_sms=args.side_ctas if groups > 1 else 0)
    core = DataParallelStep(rep, ids_dev, tgt_dev, name="step_resident", **dp_kw)
    e2e = DataParallelStep(rep, ids_dev, tgt_dev, host_ids=ids_host, host_targets=tgt_host,
                           name="step_e2e", **dp_kw)
    lr = 6e-4

    def barrier():
        dev.sync()
        if comm is not None:
            comm.barrier()
        dev.sync()

    # ---- device-timed: K steps back to back, inputs resident -------------------------------
    for _ in range(args.warmup):
        core.enqueue(lr)
    barrier()
    sampler = ClockSampler(local) if rank == 0 else None
    t_wall0 = time.perf_counter()
    import ctypes as C
    vk._check(dev.lib.vkg_timer_begin(dev.handle), "timer")
    for _ in range(args.steps):
        core.enqueue(lr)
    sec = C.c_double(0.0)
    vk._check(dev.lib.vkg_timer_end(dev.handle, C.byref(sec)), "timer")
    barrier()
    t_wall1 = time.perf_counter()
    dt = comm.max_double(sec.value) if comm is not None else sec.value
    loss_core = model.read_loss()

    if args.profile:
        # launch-list runs: only the resident steps above, nothing else on the device
        if rank == 0:
            print(json.dumps({"profile_only": True, "ms_per_step": dt / args.steps * 1e3,
                              "launches_per_step": core.n_kernels}), flush=True)
        barrier()
        for c_ in (side, comm):
            if c_ is not None:
                c_.destroy()
        rep.destroy()
        dev.destroy()
        return

    # ---- end to end: host inputs in, loss out, every step ----------------------------------
    for i in range(max(1, min(args.warmup, 3))):
        e2e(lr)
    barrier()
    t0 = time.perf_counter()
    last_loss = None
    for i in range(args.steps):
        bi, bt = batches[i % len(batches)]
        ids_host.array(np.uint32)[:] = bi
        tgt_host.array(np.uint32)[:] = bt
        last_loss, _ = e2e(lr)
    dev.sync()
    dt_e2e = time.perf_counter() - t0
    t_wall2 = time.perf_counter()
    if comm is not None:
        dt_e2e = comm.max_double(dt_e2e)
    clocks = sampler.stop(t_wall0, t_wall2) if sampler else None

    # replicas must still be bit-identical (the reference's drift == 0 claim); the sums also
    # let two runs with the same arguments be compared: every kernel of the step adds in a
    # fixed order, so they agree to the last bit
    sums = {nm: float(np.abs(p.numpy().astype(np.float64)).sum())
            for nm, p in (("b0.fc1.W", model.blocks[0].fc1.W), ("tok", model.tok),
                          ("pos", model.pos))}
    drift = 0.0
    if comm is not None:
        for chk in sums.values():
            drift = max(drift, comm.max_double(chk) - (-comm.max_double(-chk)))

    # the exchange step alone: fp32 all-reduce of the flat gradient bucket, max over ranks
    nvlink = None
    if comm is not None:
        reps = 5
        barrier()
        t_ar = dev.run_op(lambda: comm.allreduce_sum(rep.bucket, rep.total), reps) / reps
        t_ar = comm.max_double(t_ar)
        bucket_bytes = rep.total * 4
        wire = 2.0 * (world - 1) / world * bucket_bytes      # per GPU, per direction
        nv_peak = float(peaks.get("nvlink_gbs", FALLBACK_PEAKS["nvlink_gbs"]))
        nvlink = {"bucket_bytes": bucket_bytes, "wire_bytes_per_gpu": wire,
                  "allreduce_ms": t_ar * 1e3, "achieved": wire / t_ar / 1e9, "peak": nv_peak,
                  "unit": "GB/s", "frac": wire / t_ar / 1e9 / nv_peak,
                  "peak_note": "peer-copy bandwidth per direction measured on this pool",
                  "overlapped": core.parts is not None, "exposed_ms": t_ar * 1e3}
        if core.parts is not None:
            # what still runs on the compute stream after the backward: the last part alone
            first, count = core.parts[-1]
            barrier()
            t_last = dev.run_op(lambda: comm.allreduce_sum(rep.bucket, count, offset_bytes=4 * first),
                                reps) / reps
            nvlink["exposed_ms"] = comm.max_double(t_last) * 1e3
            nvlink["parts_bytes"] = [4 * c for _, c in core.parts]
            nvlink["side_ctas"] = args.side_ctas

    tokens_step = R * world
    line = None
    if rank == 0:
        fused = (D // H) == 64
        flops_total, gemm_t, rows = time_gemm_shapes(
            dev, gemm_shape_table(B, T, D, H, L, V, fused_attention=fused))
        attn = time_attention(dev, B, T, H, D // H) if fused else None
        achieved = flops_total / gemm_t / 1e12
        peak = float(peaks.get("bf16_tflops", FALLBACK_PEAKS["bf16_tflops"]))
        hbm = float(peaks.get("hbm_gbs", FALLBACK_PEAKS["hbm_gbs"]))
        alg = step_flops(B, T, D, H, L, V)
        ms = dt / args.steps * 1e3
        kernels = time_row_kernels(dev, rep, hbm)
        # what the launches of a step lose between kernels: step time minus every kernel
        # family timed alone (same process, same clocks regime, CUDA events)
        parts = {"gemm": gemm_t * 1e3}
        if attn is not None:
            parts["attention"] = L * (attn["fwd_us"] + attn["bwd_us"]) * 1e-3
        for k, v in kernels.items():
            parts[k] = v["count"] * v["us"] * 1e-3
        comm_ms = nvlink["exposed_ms"] if nvlink is not None else 0.0
        gaps = ms - sum(parts.values()) - comm_ms
        cpu = None
        if not args.no_cpu:
            st, probe = cpu_sample_T(name, 40.0, 1)
            fb, ad = probe if (probe is not None and st == T) else cpu_step_seconds(1, st, D, H, L, V)[:2]
            tok_s, _, sample = cpu_line_fields(name, fb, ad, st)
            cpu = {"value": tok_s, "unit": "tokens/s", "cores": os.cpu_count(), "kind": "port",
                   "sample": sample, "fwd_bwd_s": fb, "adamw_s": ad, "sample_tokens": st}
        traffic, traffic_note = profile_traffic()
        line = {
            "metric": "gpt_train_tokens_per_s", "value": tokens_step * args.steps / dt,
            "unit": "tokens/s", "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
            "ms_per_step": ms, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
            "dtype": "f16", "data": "synthetic",
            "config": workload_config(name, world, loss_scale),
            "e2e": {"value": tokens_step * args.steps / dt_e2e, "unit": "tokens/s",
                    "h2d_bytes_per_step": 2 * R * 4, "d2h_bytes_per_step": R * 4,
                    "ms_per_step": dt_e2e / args.steps * 1e3},
            "gpu_launches": core.n_kernels * args.steps,
            "launches_per_step": core.n_kernels,
            "clocks": clocks,
            "roofline": {"bound": "tensor", "achieved": achieved, "peak": peak, "unit": "TFLOP/s",
                         "frac": achieved / peak, "traffic": traffic, "peak_source": peak_src,
                         "kernel": "gemm_tcgen05_kernel, gemm_cta_pair_kernel and gemm_group_kernel "
                                   "(all their launches in one step)",
                         "traffic_note": traffic_note,
                         "gemm_ms_per_step": gemm_t * 1e3,
                         "gemm_tflop_per_step": flops_total / 1e12},
            "attention_per_layer": attn,
            "kernels": kernels,
            "parts_ms": parts,
            "gaps_ms": gaps,
            "pdl": bool(args.pdl) if args.pdl is not None else os.environ.get("VKG_PDL", "0") == "1",
            "step_tensor_frac": alg / (dt / args.steps) / 1e12 / peak,
            "algorithmic_tflop_per_step": alg / 1e12,
            "cpu_baseline": cpu,
            "loss": {"resident": loss_core, "e2e": last_loss},
            "replica_drift": drift,
            "weight_abs_sums": {k: repr(v) for k, v in sums.items()},
            "nvlink": nvlink,
        }
        if world == 1 and not args.no_extras:
            line["gemm_trio"] = trio_summary(dev, peak, with_cpu=not args.no_cpu)
            if not args.gemm_trio:
                line["gemm_trio"].pop("rows")
            line["c1_mlp"] = c1_mlp_summary(dev, with_cpu=not args.no_cpu)
        if args.gemm_trio:
            line["gemm_shapes"] = rows
    barrier()
    for c_ in (side, comm):
        if c_ is not None:
            c_.destroy()
    rep.destroy()
    if line is not None and world == 1 and not args.no_extras and name == "gpt2-small":
        peak = float(peaks.get("bf16_tflops", FALLBACK_PEAKS["bf16_tflops"]))
        line["c5_gpt_24l"] = c5_summary(dev)
        line["c5_gpt_24l"]["step_tensor_frac"] = (line["c5_gpt_24l"]["algorithmic_tflop_per_step"] /
                                                  (line["c5_gpt_24l"]["ms_per_step"] * 1e-3) / peak)
    if line is not None and world == 1 and not args.no_extras:
        line["library_gemm"] = library_gemm_rows(dev)
    dev.destroy()
    if line is not None:
        print(json.dumps(line), flush=True)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="gpt2-small", choices=sorted(WORKLOADS))
    ap.add_argument("--loss-scale", type=float, default=4096.0)
    ap.add_argument("--overlap-groups", type=int, default=4,
                    help="N>1: groups of blocks whose gradients are all-reduced beside the rest of "
                         "the backward (1 = one all-reduce after the backward)")
    ap.add_argument("--side-ctas", type=int, default=8,
                    help="N>1: CTAs NCCL may use for the overlapped parts (SMs the persistent "
                         "kernels leave free meanwhile); 0 = share the main communicator")
    ap.add_argument("--cta-pair", type=int, default=0,
                    help="with --gemm: 1 = 256x256 tiles on CTA pairs, -1 = never, 0 = library's choice")
    ap.add_argument("--max-ctas", type=int, default=0, help="with --gemm: cap the persistent grid")
    ap.add_argument("--trio-table", action="store_true",
                    help="GEMM-trio microbench over M in {4096,16384} x four (K,N); one JSON line")
    ap.add_argument("--gemm-trio", action="store_true", help="add per-shape GEMM timings")
    ap.add_argument("--no-cpu", action="store_true", help="skip the CPU oracle timing")
    ap.add_argument("--no-extras", action="store_true",
                    help="skip the GEMM-trio and MLP (BASELINE configs 1 and 2) parts of the line")
    ap.add_argument("--pdl", type=int, default=None, choices=[0, 1],
                    help="programmatic dependent launch off / on (default: the library's, off)")
    ap.add_argument("--profile", action="store_true",
                    help="run only the device-resident steps (for an ncu launch list)")
    ap.add_argument("--attn", default=None,
                    help="B,T,H: time the fused attention kernels of one layer instead of the step")
    ap.add_argument("--gemm", default=None,
                    help="M,N,K,ta,tb,batch[,c16]: time one GEMM shape instead of the step")
    ap.add_argument("--watchdog", type=int, default=900,
                    help="seconds after which a multi-GPU rank dumps its stacks and exits")
    ap.add_argument("--tile-n", type=int, default=0)
    ap.add_argument("--split-k", type=int, default=0)
    args = ap.parse_args()
    if args.attn:
        run_single_attention(args)
    elif args.gemm:
        run_single_gemm(args)
    elif args.trio_table:
        run_trio_table(args)
    elif args.impl == "reference":
        run_reference_arm(args)
    else:
        run_gpu_arm(args)


if __name__ == "__main__":
    main()
