#!/usr/bin/env python
"""Benchmark of the R-SWA KV-cache hot path: batched decode (ring append + decode attention).

Workload ("cfg2", the configuration the headline metric is quoted on): 64 sequences, 12 layers,
10 heads x 128, bf16 KV in paged blocks of 16 tokens, one 256-token vision prefix shared by all 64
sequences (refcount 64), ring window W = 1024, current text positions uniform in [1, 4096]; a step
appends one token per sequence per layer and runs decode attention; values N(0,1), synthetic.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]

One JSON line on stdout (rank 0).  Under torchrun every rank owns one GPU and an independent replica
of the workload (sequences shard by request; no collective on the data path); the timed region is
bracketed by a barrier + synchronize, timed on the device, max over ranks.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
for _p in (ROOT, os.path.join(ROOT, "tests")):
    if _p not in sys.path:
        sys.path.insert(0, _p)

import numpy as np  # noqa: E402

CFG = dict(seqs=64, layers=12, heads=10, kv_heads=10, head_dim=128, window=1024, prefixes=(256,),
           pos_lo=1, pos_hi=4096, block_tokens=16, seed=1234, total_seqs=None, name="cfg2")
# Other configurations of the same path, selectable with --workload (cfg2 is the headline and the default):
CFG4 = dict(CFG, window=4096, prefixes=(256, 656, 1056, 1456), pos_hi=16384, total_seqs=512, name="cfg4")
METRIC = "rswa_decode_tokens_per_s"
UNIT = "tokens/s"
NOMINAL_HBM_GBS = 8000.0


def load_pkg():
    import importlib.util
    if "uocr_b200" in sys.modules:
        return sys.modules["uocr_b200"]
    spec = importlib.util.spec_from_file_location("uocr_b200", os.path.join(ROOT, "unlimited-ocr.cpp_b200", "__init__.py"))
    mod = importlib.util.module_from_spec(spec)
    sys.modules["uocr_b200"] = mod
    spec.loader.exec_module(mod)
    return mod


def strong_plan(world: int):
    """Strong-scaling workloads: positions and prefix ids are drawn once for the whole job and the sequences
    are dealt to the ranks.  Returns (positions, prefix ids, order, bounds): rank r owns order[bounds[r]:bounds[r+1]]."""
    import synth
    total, n = CFG["total_seqs"], len(CFG["prefixes"])
    pos = synth.integers(CFG["seed"], 77, CFG["pos_lo"], CFG["pos_hi"], (total,)).astype(np.int64)
    ids = synth.integers(CFG["seed"], 177, 0, n - 1, (total,)).astype(np.int64) if n > 1 else np.zeros(total, np.int64)
    order, bounds = balanced_shards(ids, np.minimum(pos, CFG["window"]), total, world)
    return pos, ids, order, bounds


def _global_shard(rank: int):
    """(positions, prefix ids) of this rank's sequences."""
    world = int(os.environ.get("WORLD_SIZE", 1))
    pos, ids, order, bounds = strong_plan(world)
    mine = order[bounds[rank]:bounds[rank + 1]]
    return pos[mine], ids[mine]


def balanced_shards(ids, load, total, world, balance=True):
    """Contiguous shards of the prefix-sorted sequence order for a strong-scaling job (requests are
    independent, so any partition is valid).  Affinity first: the order is sorted by prefix id, so a rank
    holds as few distinct prefixes as possible, one copy of each.  Then bytes: `load` is the window tokens
    a sequence streams per step; the shard boundaries are put where the cumulated load of the groups' mean
    crosses multiples of total / world (a rank whose sequences have long windows gets a few sequences
    fewer), and inside every prefix group the sequences are dealt to the shards that cut the group largest
    first, each to the segment whose mean load is lowest.  With balance=False: equal counts, no dealing."""
    order = np.argsort(ids, kind="stable")
    if not balance or world == 1:
        return order, [shard_sequences(total, world, r)[0] for r in range(world)] + [total]
    load = np.asarray(load, np.float64)
    gmean = np.zeros(total)
    for g in set(ids.tolist()):
        gmean[ids == g] = load[ids == g].mean()
    cum = np.concatenate([[0.0], np.cumsum(gmean[order])])
    bounds = [0]
    for r in range(1, world):
        b = int(np.argmin(np.abs(cum - r * cum[-1] / world)))
        bounds.append(min(max(b, bounds[-1] + 1), total - (world - r)))
    bounds.append(total)
    out = order.copy()
    g0 = 0
    while g0 < total:
        g1 = g0
        while g1 < total and ids[order[g1]] == ids[order[g0]]:
            g1 += 1
        cuts = sorted({g0, g1} | {b for b in bounds if g0 < b < g1})
        segs = list(zip(cuts, cuts[1:]))
        members = sorted(order[g0:g1].tolist(), key=lambda i: (-load[i], i))
        fill = [[] for _ in segs]
        sums = [0.0] * len(segs)
        for i in members:
            open_ = [k for k, (a, b) in enumerate(segs) if len(fill[k]) < b - a]
            k = min(open_, key=lambda k: (sums[k] / (segs[k][1] - segs[k][0]), k))
            fill[k].append(i)
            sums[k] += load[i]
        for (a, b), f in zip(segs, fill):
            out[a:b] = f
        g0 = g1
    return out, bounds


def draw_positions(rank: int):
    import synth
    if CFG["total_seqs"]:
        return _global_shard(rank)[0][:CFG["seqs"]]
    # weak scaling: every replica gets the SAME positions (the work per GPU is fixed exactly as the GPU count
    # grows; only the random KV contents differ by rank), so the slowest rank is a slower GPU, not a longer job
    return synth.integers(CFG["seed"], 77, CFG["pos_lo"], CFG["pos_hi"], (CFG["seqs"],)).astype(np.int64)


def draw_prefix_ids(rank: int):
    """Which of the distinct prefixes each sequence of this GPU uses (uniform; one prefix -> all 0)."""
    import synth
    n = len(CFG["prefixes"])
    if CFG["total_seqs"]:
        return _global_shard(rank)[1][:CFG["seqs"]]
    if n == 1:
        return np.zeros(CFG["seqs"], np.int64)
    return synth.integers(CFG["seed"], 177, 0, n - 1, (CFG["seqs"],)).astype(np.int64)


def algorithmic_bytes_per_layer(pos_after_append: np.ndarray, prefix_ids: np.ndarray) -> float:
    """Unique bytes one layer of one decode step must move: window tokens read + every distinct
    prefix on this GPU once + appended rows written (bf16 K+V = 5120 B per token), plus q read, out
    written and new k, v read in fp32."""
    row = CFG["kv_heads"] * CFG["head_dim"]
    kv_tok = row * 2 * 2
    n = np.minimum(pos_after_append, CFG["window"])
    B = len(pos_after_append)
    distinct = sum(CFG["prefixes"][i] for i in set(prefix_ids.tolist()))
    return float(kv_tok * (n.sum() + distinct + B) + B * row * 4 * 4)


def measured_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        try:
            return float(json.load(open(path))["hbm_gbs"]), "measured"
        except Exception:
            pass
    return 6650.0, "fallback"


class Ranks:
    """The multi-GPU plumbing of the benchmark: one process per GPU, no collective on the data path.
    torch.distributed is used for exactly two things -- the barrier that brackets the timed region and
    the MAX over ranks of the device-measured time.  `backend="gloo"` runs the same logic on CPU."""

    def __init__(self, rank: int, world: int, backend: str = "nccl", device=None):
        self.rank, self.world, self.dist, self.device = rank, world, None, device
        if world > 1:
            import torch.distributed as dist
            kw = {"device_id": device} if (backend == "nccl" and device is not None) else {}
            dist.init_process_group(backend, rank=rank, world_size=world, **kw)
            self.dist = dist

    def barrier(self):
        if self.dist:
            self.dist.barrier()

    def max_over_ranks(self, value: float) -> float:
        if not self.dist:
            return value
        import torch
        t = torch.tensor([value], dtype=torch.float64, device=self.device if self.device is not None else "cpu")
        self.dist.all_reduce(t, op=self.dist.ReduceOp.MAX)
        return float(t[0])

    def gather(self, values):
        """Every rank's list of floats, as a list of lists indexed by rank (same on all ranks)."""
        if not self.dist:
            return [list(values)]
        import torch
        dev = self.device if self.device is not None else "cpu"
        mine = torch.tensor(list(values), dtype=torch.float64, device=dev)
        out = [torch.zeros_like(mine) for _ in range(self.world)]
        self.dist.all_gather(out, mine)
        return [[float(x) for x in t.tolist()] for t in out]

    def close(self):
        if self.dist:
            self.dist.barrier()
            self.dist.destroy_process_group()


def shard_sequences(total_seqs: int, world: int, rank: int):
    """Strong-scaling workloads: sequences are dealt to ranks in contiguous, near-equal shards
    (requests are independent, so any partition is valid)."""
    base, extra = divmod(total_seqs, world)
    start = rank * base + min(rank, extra)
    return start, base + (1 if rank < extra else 0)


def aggregate_tokens_per_s(seqs_per_rank, steps: int, max_ms: float) -> float:
    """Whole-job throughput: tokens produced by all ranks divided by the slowest rank's time."""
    return sum(seqs_per_rank) * steps / (max_ms * 1e-3)


class ClockSampler:
    """nvidia-smi clocks / throttle reasons sampled every 50 ms while the timed region runs."""
    Q = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
         "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
         "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index: int):
        self.idx = gpu_index
        self.proc = None
        self.lines = []

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits",
                                          "-lms", "50", "-i", str(self.idx)], stdout=subprocess.PIPE, text=True)
            self.t = threading.Thread(target=self._read, daemon=True)
            self.t.start()
        except Exception:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.lines.append(line.strip())

    def stop(self):
        if not self.proc:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except Exception:
            self.proc.kill()
        sm, mx, reasons = [], [], set()
        for ln in self.lines:
            f = [x.strip() for x in ln.split(",")]
            if len(f) < 9:
                continue
            try:
                sm.append(float(f[1]))
                mx.append(float(f[2]))
            except ValueError:
                continue
            for name, val in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), f[5:9]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": sorted(reasons), "samples": len(sm)}


# ---------------------------------------------------------------------------------------------
# our arm
# ---------------------------------------------------------------------------------------------
class DecodeWorkload:
    """Device state of the cfg2 workload on the current GPU, driven through the C ABI."""

    def __init__(self, pkg, rank: int, fused: bool = True, overlap: bool = True,
                 rope: bool = False):
        self.rope = rope
        import torch
        self.pkg, self.torch = pkg, torch
        self.fused = fused
        c = CFG
        B, L, W, bt = c["seqs"], c["layers"], c["window"], c["block_tokens"]
        self.B, self.L = B, L
        self.row = c["kv_heads"] * c["head_dim"]
        self.prefix_ids = draw_prefix_ids(rank)
        plen = np.array([c["prefixes"][i] for i in self.prefix_ids], np.int64)
        pbs = [p // bt for p in c["prefixes"]]
        pstart = np.concatenate([[0], np.cumsum(pbs)])  # every distinct prefix stored once
        rb = W // bt
        self.num_blocks = int(pstart[-1]) + B * rb
        table = np.full((B, max(pbs) + rb), -1, np.int32)
        for s in range(B):
            i = self.prefix_ids[s]
            table[s, :pbs[i]] = pstart[i] + np.arange(pbs[i])  # physically shared prefix blocks
            table[s, pbs[i]:pbs[i] + rb] = pstart[-1] + s * rb + np.arange(rb)
        self.table = torch.from_numpy(table).cuda()
        g = torch.Generator(device="cuda")
        g.manual_seed(c["seed"] + rank)
        self.layers = []
        for _ in range(L):
            lay = pkg.PagedLayer(self.num_blocks, c["kv_heads"], c["head_dim"], pkg.BF16, self.table)
            lay.k.copy_(torch.randn(lay.k.shape, generator=g, device="cuda", dtype=torch.float32))
            lay.v.copy_(torch.randn(lay.v.shape, generator=g, device="cuda", dtype=torch.float32))
            self.layers.append(lay)
        self.pos0 = draw_positions(rank)
        self.plen = plen
        self.d_prefill = torch.from_numpy(plen.astype(np.int32)).cuda()
        self.d_slots = torch.arange(B, dtype=torch.int32, device="cuda")
        self.d_len = torch.zeros((L, B), dtype=torch.int32, device="cuda")
        self.d_ring = torch.zeros((L, B), dtype=torch.int32, device="cuda")
        self.set_positions(self.pos0)
        self.d_positions = torch.from_numpy((plen + self.pos0).astype(np.int32)).cuda()  # rotary positions (--rope)
        # q, k, v of a layer sit next to each other so that the end-to-end step can bring the inputs of
        # several layers over in one copy
        self.qkv = torch.randn((L, 3, B, self.row), generator=g, device="cuda")
        self.q, self.k, self.v = self.qkv[:, 0], self.qkv[:, 1], self.qkv[:, 2]
        self.out = torch.zeros((L, B, self.row), device="cuda")
        self.ws = pkg.Workspace(B)
        self.ws.set_overlap(overlap)  # consecutive launches belong to different layers: overlap is safe
        self.graph = None
        self.launches_per_step = 0
        self.steps_done = 0

    def set_positions(self, pos):
        """Cursor state after `pos` appends (closed form of the ring state machine)."""
        torch = self.torch
        W, P = CFG["window"], self.plen
        ln = P + np.minimum(pos, W)
        rp = np.where(pos < W, 0, (pos - W) % W)
        self.d_len.copy_(torch.from_numpy(np.tile(ln.astype(np.int32), (self.L, 1))))
        self.d_ring.copy_(torch.from_numpy(np.tile(rp.astype(np.int32), (self.L, 1))))

    def layer_step(self, l, out=None):
        p = self.pkg
        out = self.out[l] if out is None else out
        if self.fused and self.rope:
            p.decode_step_rope_paged(self.layers[l], self.q[l], self.k[l], self.v[l], self.d_positions, 10000.0,
                                     self.d_len[l], self.d_ring[l], self.d_prefill, self.d_slots, self.B,
                                     CFG["window"], CFG["heads"], out, self.ws)
        elif self.fused:
            p.decode_step_paged(self.layers[l], self.q[l], self.k[l], self.v[l], self.d_len[l], self.d_ring[l],
                                self.d_prefill, self.d_slots, self.B, CFG["window"], CFG["heads"], out,
                                self.ws)
        else:
            p.append_decode_batch_paged(self.layers[l], self.k[l], self.v[l], self.d_len[l], self.d_ring[l],
                                        self.d_prefill, self.d_slots, self.B, CFG["window"], self.ws)
            p.attention_batch_paged(self.layers[l], self.q[l], self.d_len[l], self.d_prefill, self.d_slots,
                                    self.B, CFG["heads"], out, self.ws)

    def step_plain(self, per_layer_hook=None):
        for l in range(self.L):
            self.layer_step(l)
            if per_layer_hook:
                per_layer_hook(l)

    def capture(self):
        torch = self.torch
        before = self.pkg.launch_count()
        self.step_plain()  # also sets kernel attributes outside capture
        self.launches_per_step = self.pkg.launch_count() - before
        self.steps_done += 1
        torch.cuda.synchronize()
        self.graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(self.graph):
            self.step_plain()

    def step(self):
        self.graph.replay()
        self.steps_done += 1

    def capture_e2e(self, hqkv, hout, chunks=(1, 3, 8), mapped_out=False):
        """One graph for a whole step fed from pinned host memory, three streams.  The inputs come over in
        a few copies of growing size (layer 0 alone, so that compute starts early; the rest behind the
        kernels of the layers before them); every layer's result goes back as soon as its kernel is done.
        Few cross-stream waits keep the kernels of one chunk back to back on the compute stream."""
        torch = self.torch
        assert sum(chunks) == self.L
        h2d, d2h = torch.cuda.Stream(), torch.cuda.Stream()
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g):
            main = torch.cuda.current_stream()
            h2d.wait_stream(main)
            d2h.wait_stream(main)
            ready, l0 = [], 0
            with torch.cuda.stream(h2d):
                for n in chunks:
                    self.qkv[l0:l0 + n].copy_(hqkv[l0:l0 + n], non_blocking=True)
                    ev = torch.cuda.Event()
                    ev.record(h2d)
                    ready.append(ev)
                    l0 += n
            l0 = 0
            for ci, n in enumerate(chunks):
                main.wait_event(ready[ci])
                for l in range(l0, l0 + n):
                    if mapped_out:
                        # the kernel stores the layer's result straight into the caller's pinned (mapped)
                        # host buffer: no copy node, no cross-stream edge behind the kernel
                        self.layer_step(l, hout[l])
                        continue
                    self.layer_step(l)
                    done = torch.cuda.Event()
                    done.record(main)
                    d2h.wait_event(done)
                    with torch.cuda.stream(d2h):
                        hout[l].copy_(self.out[l], non_blocking=True)
                l0 += n
            main.wait_stream(h2d)
            main.wait_stream(d2h)
        return g


def parity_check(pkg, wl, n_seqs=4):
    """After the timed region: one more decode step of layer 0 on the device, and the same step on the CPU
    oracle (the checker, never the thing timed) for a few sampled sequences.  The oracle caches are filled
    with what the device holds -- read back through the block-table gather -- driven to the same cursors
    through the reference's own calls (reset, write_prefill, append_decode), then append + attention.
    Cursors must agree exactly, outputs within max-abs 2e-2 / rel-L2 1e-3 (bf16 KV)."""
    import torch
    import synth
    from oracle import oracle
    if wl.rope:
        return None
    orc = oracle.load("orc")
    c, W, B = CFG, CFG["window"], wl.B
    sel = sorted({int(round(x)) for x in np.linspace(0, B - 1, n_seqs)})
    cap = int(max(c["prefixes"])) + W
    ds = torch.tensor(sel, dtype=torch.int32, device="cuda")
    gk = torch.empty((len(sel), cap, wl.row), device="cuda")
    gv = torch.empty_like(gk)
    pkg.gather_paged(wl.layers[0], wl.d_len[0], wl.d_prefill, ds, len(sel), cap, gk, gv, pkg.F32, wl.ws)
    len0, ring0 = wl.d_len[0].cpu().numpy(), wl.d_ring[0].cpu().numpy()
    hk, hv = gk.cpu().numpy(), gv.cpu().numpy()
    q, k, v = (x[0].cpu().numpy() for x in (wl.q, wl.k, wl.v))
    out = torch.full((B, wl.row), float("nan"), device="cuda")
    wl.layer_step(0, out)
    got = out.cpu().numpy()
    len1, ring1 = wl.d_len[0].cpu().numpy(), wl.d_ring[0].cpu().numpy()
    want, cursors_ok = [], True
    for i, s_ in enumerate(sel):
        P = int(wl.plen[s_])
        n = int(len0[s_]) - P
        cache = orc.Cache(1, c["kv_heads"], c["head_dim"], W)
        cache.reset(P)
        cache.write_prefill(0, hk[i, :P], hv[i, :P])
        for j in range(n):
            cache.append_decode(0, hk[i, P + j], hv[i, P + j])
        if n == W:  # steady state: the same rows once more up to the device's ring position
            for j in range(int(ring0[s_])):
                cache.append_decode(0, hk[i, P + j], hv[i, P + j])
        cache.append_decode(0, synth.round_bf16(k[s_]), synth.round_bf16(v[s_]))
        cursors_ok &= cache.len(0) == int(len1[s_]) and cache.ring_pos(0) == int(ring1[s_])
        want.append(cache.attention(0, q[s_:s_ + 1], cache.len(0) - 1, c["heads"], False)[0])
    want = np.stack(want)
    g = got[sel]
    max_abs = float(np.abs(g - want).max())
    rel_l2 = float(np.linalg.norm(g - want) / max(np.linalg.norm(want), 1e-30))
    ok = bool(np.isfinite(g).all() and cursors_ok and max_abs <= 2e-2 and rel_l2 <= 1e-3)
    assert ok, f"parity check failed: max-abs {max_abs}, rel-L2 {rel_l2}, cursors ok {cursors_ok}"
    return {"ok": ok, "max_abs": max_abs, "rel_l2": rel_l2, "rows": len(sel), "sequences": sel, "layer": 0,
            "window_tokens": [int(len0[x] - wl.plen[x]) for x in sel], "cursors_bit_exact": bool(cursors_ok),
            "tolerance": {"max_abs": 2e-2, "rel_l2": 1e-3}, "checker": "CPU oracle (restatement of RSWACache)"}


def kernel_source_sha():
    """Hash of the sources the dominant kernel is compiled from; ties an ncu traffic record to the code."""
    import hashlib
    h = hashlib.sha256()
    for f in ("rswa_attention.cuh", "rswa_device.cuh"):
        h.update(open(os.path.join(ROOT, "unlimited-ocr.cpp_b200", "csrc", f), "rb").read())
    return h.hexdigest()[:16]


def traffic_record(name="rswa_attn_kernel_fused_bf16_hd128_cfg2.md"):
    """DRAM traffic of one launch of the dominant kernel from the committed ncu summary: a line
    `traffic-record: kernel_sha=<hash> dram_bytes=<read+write> algorithmic_bytes=<bytes at the captured step>`.
    Returned only while the kernel sources still hash to the recorded value; otherwise the record is stale
    and the traffic is reported as null."""
    import re
    path = os.path.join(ROOT, "profiles", name)
    try:
        m = re.search(r"traffic-record:\s*kernel_sha=(\w+)\s+dram_bytes=([\d.e+]+)\s+algorithmic_bytes=([\d.e+]+)", open(path).read())
    except OSError:
        m = None
    if not m:
        return None, None, "no traffic record"
    if m.group(1) != kernel_source_sha():
        return None, None, f"stale: profiles/{name} was captured at kernel sources {m.group(1)}, now {kernel_source_sha()}"
    return float(m.group(2)), float(m.group(3)), f"profiles/{name} @ kernel sources {m.group(1)}"


def workload_config(world):
    """The workload both arms run (the GPU arm and the reference's CPU code): same dict in both lines."""
    return {"workload": "%s: batched decode, %d seqs/GPU x %d layers, 10 heads x 128, bf16 paged KV "
                        "(16-token blocks), shared prefixes %s, W=%d, pos~U[%d,%d]"
                        % (CFG["name"], CFG["seqs"], CFG["layers"], list(CFG["prefixes"]), CFG["window"],
                           CFG["pos_lo"], CFG["pos_hi"]),
            "seqs_per_gpu": CFG["seqs"], "layers": CFG["layers"], "window": CFG["window"],
            "prefixes": list(CFG["prefixes"]),
            "l2_policy": "inputs larger than L2: the KV every step streams is resident and far larger than the "
                         "126 MB L2 (bf16 pools on the GPU, fp32 caches on the host arm)",
            "parallelism": f"replicas x{world} (sequences shard by request, no collective)"}


def run_ours(args, rank, world):
    import torch
    pkg = load_pkg()
    pkg.lib()  # fails loudly when the CUDA library is missing
    local = int(os.environ.get("LOCAL_RANK", 0))
    torch.cuda.set_device(local)
    ranks = Ranks(rank, world, "nccl", torch.device("cuda", local))
    wl = DecodeWorkload(pkg, rank, fused=not args.separate, overlap=not args.no_overlap,
                        rope=args.rope)
    wl.capture()
    for _ in range(max(args.warmup - 1, 0)):
        wl.step()
    torch.cuda.synchronize()

    def barrier():
        ranks.barrier()
        torch.cuda.synchronize()

    # ---- timed region: K whole steps (12 layers x (append + attention)), one graph launch each.  The
    # K-step train is timed `repeats` times in this one invocation, every time from the same cursor state
    # (a short launch train is a thin sample: the median over the repeats is the reported value, min and
    # max stand beside it); each repeat is bracketed by barrier + synchronize and is the MAX over ranks ----
    stream = torch.cuda.current_stream()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start()
        time.sleep(0.15)
    start_pos = wl.pos0 + wl.steps_done
    rep_ms_local = []
    for _ in range(args.repeats):
        wl.set_positions(start_pos)
        barrier()
        e0.record(stream)
        for _ in range(args.steps):
            wl.step()
        e1.record(stream)
        barrier()
        rep_ms_local.append(e0.elapsed_time(e1))
    clocks = sampler.stop() if rank == 0 else None
    by_rank = ranks.gather(rep_ms_local)  # [rank][repeat]
    rep_ms = [max(r[i] for r in by_rank) for i in range(args.repeats)]
    ms = statistics.median(rep_ms)
    per_rank_ms = [statistics.median(r) / args.steps for r in by_rank]
    dev_status = wl.ws.status()
    assert dev_status == 0, f"device status {dev_status}"

    # ---- roofline of the dominant kernel: per-launch duration of the partial-attention kernel ------
    pos_mid = start_pos + np.arange(args.steps)[:, None] + 1  # after each timed append
    bytes_layer = float(np.mean([algorithmic_bytes_per_layer(p, wl.prefix_ids) for p in pos_mid]))
    parity = parity_check(pkg, wl) if rank == 0 and not args.no_parity_check else None
    wl.ws.set_timing(True)
    kms = []
    wl.step_plain(lambda l: kms.append(wl.ws.last_kernel_ms()))
    kms = []
    for _ in range(min(args.steps, 10)):
        wl.step_plain(lambda l: kms.append(wl.ws.last_kernel_ms()))
        wl.steps_done += 1
    wl.ws.set_timing(False)
    wl.set_positions(start_pos + args.steps)  # all layers back on one cursor state
    k_ms_isolated = float(np.mean(kms))  # one launch between two events on an idle stream (includes launch latency)
    # The fused step is ONE launch per layer, so the timed region is a back-to-back train of identical
    # launches of the dominant kernel: its average launch duration is the region's time per launch.
    # With separate entry points the region also holds the append and plan kernels, so the per-launch
    # event pair is used there.
    k_ms = (ms / args.steps / CFG["layers"]) if wl.fused else k_ms_isolated
    peak, peak_kind = measured_peaks()
    achieved = bytes_layer / (k_ms * 1e-3) / 1e9

    # ---- e2e: the same step from HOST buffers (pinned): per layer, H2D of q/k/v on a copy stream, the
    # fused kernel on the compute stream, D2H of out on a third stream -- all captured in one graph so
    # the copies of later layers overlap the kernels of earlier ones; the caller reads the result every step ----
    hqkv = torch.randn(wl.qkv.shape).pin_memory()
    hout = torch.empty(wl.out.shape).pin_memory()
    chunks = (1, 3, 8) if CFG["layers"] == 12 else (1,) * CFG["layers"]
    e2e_graph = wl.capture_e2e(hqkv, hout, chunks, mapped_out=(args.e2e_out == "mapped"))
    for _ in range(2):
        e2e_graph.replay()
    e2e_local = []
    for _ in range(args.repeats):
        wl.set_positions(start_pos)
        barrier()
        e0.record(stream)
        for _ in range(args.steps):
            e2e_graph.replay()
            stream.synchronize()  # the caller reads the step's result before the next step
        e1.record(stream)
        barrier()
        e2e_local.append(e0.elapsed_time(e1))
    e2e_by_rank = ranks.gather(e2e_local)
    e2e_rep = [max(r[i] for r in e2e_by_rank) for i in range(args.repeats)]
    e2e_ms = statistics.median(e2e_rep)
    h2d = int(hqkv.numel() * 4)
    d2h = int(hout.numel() * 4)

    # ---- read-only streaming rate of this GPU through the same copy engine path the kernel uses (one CTA
    # per SM, 4 KB bulk copies into shared memory): a second denominator beside the read+write copy peak ----
    stream_read_gbs = wl.ws.stream_read_gbs() if rank == 0 else None

    secondary = None
    if rank == 0 and world == 1 and not args.no_secondary and CFG["name"] == "cfg2":
        del e2e_graph, hqkv, hout
        secondary = {"cfg3_ragged_prefill": prefill_record(pkg, torch, layers=2, steps=3, warmup=2),
                     "gather_batched": gather_batched_gbs(pkg, torch, reps=5)}
    cpu = None
    if rank == 0 and world == 1 and not args.no_cpu_baseline:
        # cfg2: every sequence (fp32 caches of 64 sequences are about 10 GB of host memory); the W=4096
        # configuration would need hundreds of GB, so a sample of 8 sequences stands for it
        cpu = cpu_baseline(sample_seqs=CFG["seqs"] if CFG["name"] == "cfg2" else min(8, CFG["seqs"]), steps=4,
                           threads=host_threads())
    ranks.close()
    if rank != 0:
        return
    traffic, traffic_alg, traffic_source = traffic_record() if (CFG["name"] == "cfg2" and CFG["seqs"] == 64 and not args.separate
                                                                  and not args.rope) else (None, None, "no capture of this workload")
    if CFG["total_seqs"]:
        bounds = strong_plan(world)[3]
        seqs_all = [bounds[r + 1] - bounds[r] for r in range(world)]
    else:
        seqs_all = [CFG["seqs"]] * world
    tokens = sum(seqs_all) * args.steps
    line = {
        "metric": METRIC, "value": tokens / (ms * 1e-3), "unit": UNIT, "n_gpus": world, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": ms / args.steps, "higher_is_better": True,
        "repeats": args.repeats, "ms_per_step_min": min(rep_ms) / args.steps, "ms_per_step_max": max(rep_ms) / args.steps,
        "per_rank_ms": per_rank_ms,
        "scaling": "strong" if CFG["total_seqs"] else "weak",
        "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
        "config": workload_config(world),
        "run": {"kv_resident_gb": round(wl.num_blocks * 81920 * CFG["layers"] / 1e9, 2),
                "step": ("cuda graph of %d x (append; plan; attention)" % CFG["layers"] if args.separate else
                         "cuda graph of %d fused decode-step launches (append + attention in one kernel)" % CFG["layers"])},
        "roofline": {"bound": "hbm", "kernel": "rswa_attn_kernel<BF16,128,paged,%s>" % ("separate" if args.separate else "fused"), "achieved": achieved,
                     "peak": peak, "unit": "GB/s", "frac": achieved / peak, "peak_kind": peak_kind,
                     "frac_of_nominal_8TBs": achieved / NOMINAL_HBM_GBS, "kernel_ms": k_ms,
                     "kernel_ms_isolated_launch": k_ms_isolated,
                     # one launch alone between two events (no neighbour hides its prologue): in a decoder the
                     # neighbours are other kernels, so the drop-in figure lies between frac_isolated and frac
                     "frac_isolated": bytes_layer / (k_ms_isolated * 1e-3) / 1e9 / peak,
                     "algorithmic_bytes_per_launch": bytes_layer,
                     # dram__bytes_read.sum + dram__bytes_write.sum of one launch of this kernel from the ncu
                     # capture summarised in the file named by traffic_source (null when the kernel sources
                     # changed since); the capture sits at the workload's first steps, hence its own byte count
                     "traffic": traffic, "traffic_capture_algorithmic_bytes": traffic_alg, "traffic_source": traffic_source,
                     "stream_read_gbs": stream_read_gbs,
                     "frac_of_stream_read": (achieved / stream_read_gbs) if stream_read_gbs else None,
                     "step_gbs": bytes_layer * CFG["layers"] / (ms / args.steps * 1e-3) / 1e9},
        "e2e": {"value": tokens / (e2e_ms * 1e-3), "unit": UNIT, "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h,
                "ms_per_step": e2e_ms / args.steps, "ms_per_step_min": min(e2e_rep) / args.steps,
                "per_rank_ms": [statistics.median(r) / args.steps for r in e2e_by_rank],
                "ms_per_step_max": max(e2e_rep) / args.steps,
                "how": "per step: q/k/v of all layers from pinned host memory in %s host-to-device copies behind the "
                       "kernels, results %s, host synchronises after every step"
                       % (len(chunks), "stored by the kernels straight into the pinned host buffer (device-mapped)"
                          if args.e2e_out == "mapped" else "returned by one device-to-host copy per layer")},
        "gpu_launches": wl.launches_per_step * args.steps,  # per timed K-step train (there are `repeats` of them)
        "clocks": clocks,
    }
    if parity:
        line["parity_check"] = parity
    if secondary:
        line["secondary"] = secondary
    if cpu:
        line["cpu_baseline"] = cpu
    print(json.dumps(line))


# ---------------------------------------------------------------------------------------------
# CPU arm: the reference's own RSWACache (compiled, unmodified) or the oracle port
# ---------------------------------------------------------------------------------------------
def host_threads() -> int:
    """All host cores this process may use (torchrun exports OMP_NUM_THREADS=1, which would otherwise
    silently make the CPU arm single-threaded)."""
    try:
        return len(os.sched_getaffinity(0))
    except AttributeError:
        return os.cpu_count() or 1


def cpu_baseline(sample_seqs: int, steps: int, threads: int = 0):
    from oracle import oracle
    kind = "reference" if oracle.available("ref") else "port"
    o = oracle.load("ref" if kind == "reference" else "orc")
    pos = draw_positions(0)[:sample_seqs]
    pl = np.array([CFG["prefixes"][i] for i in draw_prefix_ids(0)[:sample_seqs]], np.int32)
    sec, used, _ = o.run_decode_bench(pl, pos, CFG["layers"], CFG["kv_heads"], CFG["head_dim"], CFG["window"],
                                      steps, threads=threads, seed=CFG["seed"])
    return {"value": sample_seqs * steps / sec, "unit": UNIT, "cores": used, "kind": kind,
            "sample": f"{'all' if sample_seqs >= CFG['seqs'] else 'first'} {sample_seqs} of the {CFG['seqs']} sequences, "
                      f"all {CFG['layers']} layers, {steps} decode steps, fp32 KV "
                      f"holding the bf16-rounded values; OpenMP over (sequence, layer) in the harness",
            "seconds": sec}


def run_reference(args, rank, world):
    if rank != 0:
        return
    seqs = CFG["seqs"]  # every sequence of the configuration (fp32 caches: about 10 GB of host memory for cfg2)
    steps = max(args.steps, 1)
    # warm-up steps are part of the same call (state set-up dominates); time K steps
    cpu = cpu_baseline(sample_seqs=seqs, steps=steps, threads=host_threads())
    line = {
        "impl": "reference", "metric": METRIC, "value": cpu["value"], "unit": UNIT, "n_gpus": world,
        "steps": steps, "warmup": args.warmup, "ms_per_step": cpu["seconds"] / steps * 1e3,
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": workload_config(world),
        "run": {"how": "the reference's RSWACache on host cores (rank 0 only): " + cpu["sample"]},
        "cpu_baseline": cpu,
        "e2e": {"value": cpu["value"], "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }
    print(json.dumps(line))


def run_prefill(args, rank, world):
    """Configuration 3: ragged prefill + ring fill.  16 sequences, 12 layers, 10 heads x 128, bf16;
    vision prefix lengths from {256, 656, 1056}, text prompt lengths uniform in [64, 2048], W=1024
    (prompts longer than W wrap).  Per layer: scatter of the vision K/V into the prefix blocks and of
    the text K/V into the text pool, attention (vision rows causal over the prefix; text rows over
    prefix + window) on the tcgen05 kernel, ring fill.  Reports prefill tokens/s and TFLOP/s
    (4*D*H = 5120 flop per attended (query, key) pair).  Tensor-core pass: vision scatter; text scatter + ring
    fill + cursor publication in one kernel; attention.  Parity of this path: tests/test_gpu_prefill.py."""
    if rank != 0:
        return
    import torch
    pkg = load_pkg()
    print(json.dumps(prefill_record(pkg, torch, layers=args.layers or CFG["layers"], steps=max(1, min(args.steps, 20)),
                                    warmup=max(args.warmup, 1))))


def prefill_record(pkg, torch, layers, steps, warmup):
    """The cfg3 measurement as a dict (see run_prefill); `layers` < 12 gives a compact record for the default line."""
    import synth
    c = CFG
    S, L, W, H, D, bt = 16, layers, 1024, c["heads"], c["head_dim"], 16
    row = H * D
    pv = np.array([(256, 656, 1056)[i] for i in synth.integers(c["seed"], 301, 0, 2, (S,))])
    tl = synth.integers(c["seed"], 302, 64, 2048, (S,)).astype(np.int64)
    pb, rb = pv // bt, W // bt
    pstart = np.concatenate([[0], np.cumsum(pb)])
    num_blocks = int(pstart[-1]) + S * rb
    table = np.full((S, int(pb.max()) + rb), -1, np.int32)
    for s in range(S):
        table[s, :pb[s]] = pstart[s] + np.arange(pb[s])
        table[s, pb[s]:pb[s] + rb] = pstart[-1] + s * rb + np.arange(rb)
    d_table = torch.from_numpy(table).cuda()
    layers = [pkg.PagedLayer(num_blocks, H, D, pkg.BF16, d_table) for _ in range(L)]
    tb = -(-tl // bt)
    block0 = np.concatenate([[0], np.cumsum(tb)])[:-1]
    text_blocks = int(tb.sum())
    text_k = torch.zeros((text_blocks, H, bt, D), dtype=torch.bfloat16, device="cuda")
    text_v = torch.zeros_like(text_k)
    nv, nt = int(pv.sum()), int(tl.sum())
    d = lambda a: torch.from_numpy(np.ascontiguousarray(a)).cuda()
    v_slots = d(np.concatenate([np.full(pv[s], s) for s in range(S)]).astype(np.int32))
    v_pos = d(np.concatenate([np.arange(pv[s]) for s in range(S)]).astype(np.int32))
    t_slots = d(np.concatenate([np.full(tl[s], s) for s in range(S)]).astype(np.int32))
    t_pos = d(np.concatenate([np.arange(tl[s]) for s in range(S)]).astype(np.int32))
    t_b0 = d(np.concatenate([np.full(tl[s], block0[s]) for s in range(S)]).astype(np.int32))
    t_len = d(np.concatenate([np.full(tl[s], tl[s]) for s in range(S)]).astype(np.int32))
    d_prefill = d(pv.astype(np.int32))
    d_len = torch.zeros((L, S), dtype=torch.int32, device="cuda")
    d_ring = torch.zeros((L, S), dtype=torch.int32, device="cuda")
    g = torch.Generator(device="cuda")
    g.manual_seed(c["seed"])
    q = torch.randn((nv + nt, row), generator=g, device="cuda")
    k = torch.randn((nv + nt, row), generator=g, device="cuda")
    v = torch.randn((nv + nt, row), generator=g, device="cuda")
    out = torch.zeros((nv + nt, row), device="cuda")
    reqs, at = [], 0
    for s in range(S):
        reqs.append((at, int(pv[s]), s, 0, 0, 0))
        at += int(pv[s])
    for s in range(S):
        reqs.append((at, int(tl[s]), s, 1, 0, int(block0[s])))
        at += int(tl[s])
    tiles = pkg.make_prefill_tiles(reqs)
    ws = pkg.Workspace(nv + nt)
    pairs = sum(int(p) * (int(p) + 1) // 2 for p in pv) + sum(
        int(t) * int(p) + (int(t) * (int(t) + 1) // 2 if t <= W else W * (W + 1) // 2 + (int(t) - W) * W)
        for t, p in zip(tl, pv))
    flops = pairs * 4.0 * D * H

    def layer_pass(l, tc=True):
        pkg.write_prefill_ragged_paged(layers[l], k[:nv], v[:nv], v_slots, v_pos, nv, ws)
        if tc:
            pkg.text_scatter_fill_paged(layers[l], text_k, text_v, text_blocks, k[nv:], v[nv:], t_slots, t_pos, t_b0, t_len,
                                        d_prefill, d_len[l], d_ring[l], nt, W, ws)
            # one plan of the query tiles per pass, shared by its layers (the prefix lengths do not change)
            pkg.prefill_attention_tc(layers[l], text_k, text_v, text_blocks, q, d_prefill, tiles, W, H, out, ws, reuse_plan=l > 0)
            return
        else:
            pkg.attention_ragged_paged(layers[l], q[:nv], d_prefill, v_slots, v_pos, nv, H, out[:nv], ws)
            pkg.prefill_text_paged(layers[l], text_k, text_v, text_blocks, q[nv:], k[nv:], v[nv:], d_prefill, t_slots,
                                   t_pos, t_b0, nt, W, H, out[nv:], ws)
        pkg.ring_fill_paged(layers[l], text_k, text_v, text_blocks, t_slots, t_pos, t_b0, t_len, d_prefill, d_len[l],
                            d_ring[l], nt, W, ws)

    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    for _ in range(warmup):
        layer_pass(0)
    torch.cuda.synchronize()
    e0.record()
    for _ in range(steps):
        for l in range(L):
            layer_pass(l)
    e1.record()
    torch.cuda.synchronize()
    ms = e0.elapsed_time(e1) / steps
    layer_pass(0, tc=False)
    torch.cuda.synchronize()
    e0.record()
    layer_pass(0, tc=False)
    e1.record()
    torch.cuda.synchronize()
    ms_cuda_core_layer = e0.elapsed_time(e1)
    assert ws.status() == 0
    peaks = json.load(open(os.path.join(ROOT, "MEASURED_PEAKS.json"))) if os.path.exists(os.path.join(ROOT, "MEASURED_PEAKS.json")) else {}
    tf = flops * L / (ms * 1e-3) / 1e12
    # the attention kernel alone (the dominant kernel of the pass), per layer
    pkg.prefill_plan_tc(tiles, d_prefill, W, ws)
    torch.cuda.synchronize()
    n_attn = max(steps, 40)  # short trains scatter by several percent
    e0.record()
    for _ in range(n_attn):
        pkg.prefill_attention_tc(layers[0], text_k, text_v, text_blocks, q, d_prefill, tiles, W, H, out, ws, reuse_plan=True)
    e1.record()
    torch.cuda.synchronize()
    ms_attn = e0.elapsed_time(e1) / n_attn
    tf_attn = flops / (ms_attn * 1e-3) / 1e12
    return ({
        "metric": "rswa_prefill_tokens_per_s", "value": (nv + nt) / (ms * 1e-3), "unit": "tokens/s", "n_gpus": 1,
        "steps": steps, "ms_per_step": ms, "dtype": "bf16", "data": "synthetic",
        "config": {"workload": "cfg3: ragged prefill + ring fill, 16 seqs x %d layers, prefixes {256,656,1056}, "
                               "text U[64,2048], W=1024" % L, "vision_tokens": nv, "text_tokens": nt,
                   "query_tiles": int(tiles.shape[0]), "attended_pairs_per_layer": pairs},
        "roofline": {"bound": "tensor", "kernel": "rswa_prefill_tc_kernel", "achieved": tf_attn, "unit": "TFLOP/s",
                     "peak": peaks.get("bf16_tflops"), "frac": (tf_attn / peaks["bf16_tflops"]) if peaks.get("bf16_tflops") else None,
                     "kernel_ms": ms_attn, "whole_pass_tflops": tf,
                     "note": "useful flops (5120 per attended query-key pair) over the attention kernel's own time; "
                             "whole_pass_tflops divides by the pass including the scatter kernels"},
        "cuda_core_path_ms_per_layer": ms_cuda_core_layer, "tensor_core_path_ms_per_layer": ms / L})


def gather_batched_gbs(pkg, torch, seqs=256, prefix=656, window=1024, reps=10):
    """One gather launch over `seqs` full sequences of one layer that share one prefix (bf16 in, bf16 out):
    unique bytes read + bytes written over the CUDA-event time, against the measured copy peak (which
    counts read + write bytes too)."""
    bt, kvh, hd = 16, CFG["kv_heads"], CFG["head_dim"]
    pb, rb = prefix // bt, window // bt
    num_blocks = pb + seqs * rb
    table = np.zeros((seqs, pb + rb), np.int32)
    rng = np.random.default_rng(7)
    ring = rng.permutation(seqs * rb).reshape(seqs, rb) + pb  # ring blocks scattered over the pool
    table[:, :pb] = np.arange(pb)
    table[:, pb:] = ring
    lay = pkg.PagedLayer(num_blocks, kvh, hd, pkg.BF16, torch.from_numpy(table).cuda())
    lay.k.normal_()
    lay.v.normal_()
    cap = prefix + window
    d_len = torch.full((seqs,), cap, dtype=torch.int32, device="cuda")
    d_prefill = torch.full((seqs,), prefix, dtype=torch.int32, device="cuda")
    slots = torch.arange(seqs, dtype=torch.int32, device="cuda")
    gk = torch.empty((seqs, cap, kvh * hd), dtype=torch.bfloat16, device="cuda")
    gv = torch.empty_like(gk)
    ws = pkg.Workspace(seqs)
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    for _ in range(3):
        pkg.gather_paged(lay, d_len, d_prefill, slots, seqs, cap, gk, gv, pkg.BF16, ws)
    torch.cuda.synchronize()
    e0.record()
    for _ in range(reps):
        pkg.gather_paged(lay, d_len, d_prefill, slots, seqs, cap, gk, gv, pkg.BF16, ws)
    e1.record()
    torch.cuda.synchronize()
    ms = e0.elapsed_time(e1) / reps
    row = 2 * kvh * hd * 2  # K and V of one token, bf16
    # unique bytes: every sequence's ring rows and the shared prefix once are read, every row is written
    nbytes = row * (seqs * window + prefix) + row * seqs * cap
    peak, kind = measured_peaks()
    gbs = nbytes / (ms * 1e-3) / 1e9
    return {"gbs": gbs, "ms_per_launch": ms, "bytes_per_launch": nbytes, "frac_of_copy_peak": gbs / peak,
            "peak_kind": kind, "seqs": seqs, "rows_per_seq": cap}


def run_churn(args, rank, world):
    """Configuration 5: pool of 65536 blocks x 12 layers (64 GB), 1000 requests on a seeded Poisson
    schedule, 8 prefixes, W=1024; reports append and block-table gather bandwidth (algorithmic bytes:
    append reads the fp32 k, v rows and writes them as bf16; gather reads and writes len x 5120 B per
    layer).  Table parity for this workload at full size is asserted by tests/test_host_classes.py (host
    integers only) and with device values at reduced size by tests/test_gpu_churn.py."""
    if rank != 0:
        return
    import torch
    import churn_driver
    pkg = load_pkg()
    host = pkg.host_classes()  # the library's own MemoryPool / BlockManager / scheduler through its C ABI
    t0 = time.time()
    legs = {}
    for name, all_layers in (("one_launch_per_layer", False), ("one_launch_for_all_layers", True)):
        cfg = churn_driver.ChurnConfig(layers=args.layers or 12, all_layer_launches=all_layers)
        res = churn_driver.run(cfg, host, check=None, time_kernels=True)
        st = res["stats"]
        append_gb = st["append_rows"] * (res["row_bytes_in"] + res["row_bytes_out"]) / 1e9
        gather_gb = st["gather_tokens"] * res["row_bytes_out"] * 2 / 1e9
        launches = st["steps"] * (1 if all_layers else cfg.layers)
        legs[name] = {"append_gbs": append_gb / (st["append_ms"] * 1e-3), "append_us_per_launch": st["append_ms"] * 1e3 / max(launches, 1),
                      "gather_gbs": gather_gb / max(st["gather_ms"] * 1e-3, 1e-9)}
    batched = gather_batched_gbs(pkg, torch)
    best = legs["one_launch_for_all_layers"]
    print(json.dumps({
        "metric": "rswa_churn_append_gather", "unit": "GB/s", "n_gpus": 1, "data": "synthetic",
        "config": {"workload": "cfg5: 65536-block pool x %d layers, 1000 requests, 8 prefixes 256..1456, "
                               "out-len U[32,2048], W=1024, exponential inter-arrival mean 2 steps" % cfg.layers},
        "append_gbs": best["append_gbs"], "gather_gbs": best["gather_gbs"], "append_rows": st["append_rows"],
        "gather_tokens": st["gather_tokens"], "legs": legs,
        "note": "a step appends one row per running sequence per layer (~190 rows x 15 KB per layer) and a retiring "
                "sequence is gathered once (10-25 MB per layer): both are launches of microseconds, issued from Python, "
                "so one launch per layer is bound by launch latency; the all-layer entry points move the same bytes in one "
                "launch per step / per retiring sequence; gather_batched is the gather kernel over 256 sequences at once",
        "gather_batched": batched,
        "steps": st["steps"], "peak_running": st["peak_running"], "prefix_hits": st["prefix_hits"],
        "prefix_misses": st["prefix_misses"], "arenas_empty_at_end": res["final"][0][0] == 0 and res["final"][0][3] == 0,
        "wall_s": time.time() - t0}))


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=500)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--repeats", type=int, default=10,
                    help="how many times the K-step train is timed (median reported, min / max beside it)")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-parity-check", action="store_true", help="skip the oracle check of 4 sequences after the timed region")
    ap.add_argument("--no-secondary", action="store_true", help="skip the compact cfg3 / gather records of the default line")
    ap.add_argument("--separate", action="store_true",
                    help="issue append and attention as the reference does (two entry points per layer) "
                         "instead of the fused one-launch decode step")
    ap.add_argument("--workload", default="cfg2", choices=["cfg2", "cfg3", "cfg4", "churn", "gather"],
                    help="cfg2 (default, headline): 64 seqs/GPU, W=1024, one shared prefix, weak scaling; "
                         "cfg4: 512 seqs in total sharded over the GPUs, W=4096, 4 prefixes, strong scaling; "
                         "churn: block-manager churn on a 65536-block pool (append + gather GB/s)")
    ap.add_argument("--rope", action="store_true",
                    help="fused step with the rotary embedding folded in (q, k un-rotated; one position per row)")
    ap.add_argument("--e2e-out", default="mapped", choices=["copy", "mapped"],
                    help="end-to-end step: results return by one device-to-host copy per layer, or the kernels "
                         "store them straight into the pinned host buffer")
    ap.add_argument("--no-overlap", action="store_true",
                    help="launch the fused steps without programmatic dependent launch")
    ap.add_argument("--seqs", type=int, default=None, help="profiling aid only: sequences per GPU (not a bench number)")
    ap.add_argument("--layers", type=int, default=None,
                    help="profiling aid only: fewer layers so an ncu capture holds < 1 GB (not a bench number)")
    args = ap.parse_args()
    if args.workload == "cfg4":
        CFG.update(CFG4)
    if args.layers:
        CFG["layers"] = args.layers
    if args.seqs:
        CFG["seqs"] = args.seqs
    args.warmup = max(args.warmup, 3)
    args.repeats = max(args.repeats, 1)
    rank = int(os.environ.get("RANK", 0))
    world = int(os.environ.get("WORLD_SIZE", 1))
    if CFG["total_seqs"]:
        bounds = strong_plan(world)[3]
        CFG["seqs"] = bounds[rank + 1] - bounds[rank]
    if args.workload == "gather":
        if rank == 0:
            import torch
            pkg = load_pkg()
            pkg.lib()
            print(json.dumps({"metric": "rswa_gather_batched", "unit": "GB/s", "n_gpus": 1, "data": "synthetic",
                              "config": {"workload": "block-table gather of 256 sequences (656-token shared prefix + "
                                                     "W=1024 ring each, bf16) in one launch"},
                              **gather_batched_gbs(pkg, torch, reps=max(args.steps, 1) if args.steps < 500 else 10)}))
    elif args.workload == "churn":
        run_churn(args, rank, world)
    elif args.workload == "cfg3":
        run_prefill(args, rank, world)
    elif args.impl == "reference":
        run_reference(args, rank, world)
    else:
        run_ours(args, rank, world)


if __name__ == "__main__":
    main()
