"""Trace drivers shared by the golden-vector generator and the parity tests.

Each driver replays a list of operations on any object exposing the oracle's Python surface
(`oracle.oracle.Oracle` back ends, or the CUDA library's host classes wrapped the same way) and
returns plain integer / float arrays, so two implementations can be compared entry by entry.
"""
from __future__ import annotations

import random

import numpy as np

import synth

# ---------------------------------------------------------------------------------------------
# arena traces
# ---------------------------------------------------------------------------------------------

def make_pool_ops(seed, n_ops, total, max_size, aligns=(0,)):
    """ops rows: (kind, a, b): kind 0 = allocate(size=a, align=b); 1 = free(the a-th live one)."""
    rng = random.Random(seed)
    ops, live = [], 0
    for _ in range(n_ops):
        if live and rng.random() < 0.45:
            ops.append((1, rng.randrange(live), 0))
            live -= 1
        else:
            ops.append((0, rng.randrange(0, max_size + 1), rng.choice(aligns)))
            live += 1  # corrected during replay if the allocation fails
    return np.array(ops, dtype=np.int64), total


def run_pool_trace(lib, ops, total, alignment):
    pool = lib.Pool(total, alignment)
    live, out = [], []
    for kind, a, b in ops.tolist():
        if kind == 0:
            off = pool.allocate(a, b)
            if off >= 0 and a > 0:
                live.append((off, a))
            res = off
        else:
            if not live:
                res = -2
            else:
                off, size = live.pop(a % len(live))
                pool.free(off, size)
                res = off
        t, used, peak, nfree, frag = pool.state()
        out.append((res, used, peak, nfree, int(round(frag * 1e12))))
    return np.array(out, dtype=np.int64)


# ---------------------------------------------------------------------------------------------
# block-manager traces (arena units: 1 block == 256 arena bytes)
# ---------------------------------------------------------------------------------------------

def make_bm_ops(seed, n_ops, n_keys, max_prefix_blocks, ring_blocks):
    """ops rows: (kind, a, b): 0 acquire(key a, blocks b); 1 release(key a); 2 allocate_ring(b);
    3 free_ring(a-th live ring)."""
    rng = random.Random(seed)
    sizes = [rng.randrange(1, max_prefix_blocks + 1) for _ in range(n_keys)]
    ops = []
    for _ in range(n_ops):
        r = rng.random()
        if r < 0.3:
            k = rng.randrange(n_keys)
            ops.append((0, k, sizes[k]))
        elif r < 0.55:
            ops.append((1, rng.randrange(n_keys + 1), 0))  # n_keys == a key never acquired
        elif r < 0.8:
            ops.append((2, 0, ring_blocks))
        else:
            ops.append((3, rng.randrange(1 << 16), 0))
    return np.array(ops, dtype=np.int64)


def run_bm_trace(lib, ops, prefix_blocks, ring_pool_blocks):
    bm = lib.BlockManager(prefix_blocks * 256, ring_pool_blocks * 256)
    rings, out = [], []
    for kind, a, b in ops.tolist():
        res, rc = 0, 0
        if kind == 0:
            res, rc = bm.acquire_prefix(f"doc{a}", b * 16, b * 256)
        elif kind == 1:
            bm.release_prefix(f"doc{a}")
        elif kind == 2:
            res = bm.allocate_ring(b * 256)
            if res >= 0:
                rings.append((res, b * 256))
        elif rings:
            off, size = rings.pop(a % len(rings))
            bm.free_ring(off, size)
            res = off
        st = bm.stats()
        cnt = bm.counters()
        out.append((res, rc) + tuple(int(x) for x in st[:5]) +
                   (int(round(st[5] * 1e12)), int(round(st[6] * 1e12)), int(st[7])) +
                   tuple(int(x) for x in cnt))
    return np.array(out, dtype=np.int64)


# ---------------------------------------------------------------------------------------------
# scheduler traces
# ---------------------------------------------------------------------------------------------

def make_sched_script(seed, n_req, max_new_hi):
    rng = random.Random(seed)
    arrivals = sorted(rng.randrange(0, n_req * 2) for _ in range(n_req))
    return np.array([(arrivals[i], rng.randrange(1, 40), rng.randrange(1, max_new_hi + 1))
                     for i in range(n_req)], dtype=np.int64)


def run_sched_trace(lib, script, max_batch, early_finish_every=0):
    """Engine-style loop (src/engine/engine.cpp:328-413): admit arrivals, build a batch, prefill
    wave -> mark_prefilled + first token, decode wave -> add_token.  Returns one row per step."""
    s = lib.Scheduler(max_batch, 4)
    rows, step, nxt = [], 0, 0
    script = script.tolist()
    while nxt < len(script) or s.has_work():
        while nxt < len(script) and script[nxt][0] <= step:
            s.add_request(script[nxt][1], script[nxt][2])
            nxt += 1
        pf, dc = s.build_batch()
        for i in pf:
            s.mark_prefilled(i)
            s.add_token(i, 7)
        for j, i in enumerate(dc):
            if early_finish_every and (step + j) % early_finish_every == 0:
                s.finish(i)
            else:
                s.add_token(i, 7)
        st = s.stats()
        h = 0
        for i in pf:
            h = (h * 1000003 + i + 1) % (1 << 61)
        for i in dc:
            h = (h * 1000003 + i + 7) % (1 << 61)
        for i in s.running():
            h = (h * 1000003 + i + 13) % (1 << 61)
        rows.append((len(pf), len(dc), h) + tuple(int(x) for x in st[:6]))
        step += 1
        if step > 100000:
            raise RuntimeError("scheduler trace did not terminate")
    return np.array(rows, dtype=np.int64)


# ---------------------------------------------------------------------------------------------
# cache traces
# ---------------------------------------------------------------------------------------------

def run_cache_trace(lib, layers, kv_heads, head_dim, window, prefix, n_append, heads, seed,
                    attn_steps, bf16=False, causal_prefill=True):
    """reset(P) + write_prefill + n appends; decode attention (non-causal, seq=1) at the listed
    steps; returns bookkeeping per step, final logical K/V, and the attention outputs."""
    row = kv_heads * head_dim
    rnd = synth.round_bf16 if bf16 else (lambda x: x)
    c = lib.Cache(layers, kv_heads, head_dim, window)
    c.reset(prefix)
    out = {"book": [], "attn": [], "prefill_attn": []}
    for l in range(layers):
        pk = rnd(synth.normal(seed, 10 + l, (prefix, row)))
        pv = rnd(synth.normal(seed, 20 + l, (prefix, row)))
        if prefix > 0:
            c.write_prefill(l, pk, pv)
            if causal_prefill:
                q = synth.normal(seed, 30 + l, (prefix, heads * head_dim))
                out["prefill_attn"].append(c.attention(l, q, 0, heads, True))
    for t in range(n_append):
        for l in range(layers):
            k = rnd(synth.normal(seed, 1000 + t * 64 + l, (row,)))
            v = rnd(synth.normal(seed, 500000 + t * 64 + l, (row,)))
            c.append_decode(l, k, v)
            out["book"].append((c.len(l), c.ring_pos(l), int(c.ring_started(l))))
            if t in attn_steps:
                q = synth.normal(seed, 900000 + t * 64 + l, (1, heads * head_dim))
                out["attn"].append(c.attention(l, q, c.len(l) - 1, heads, False)[0])
    out["book"] = np.array(out["book"], dtype=np.int32)
    out["attn"] = np.array(out["attn"], dtype=np.float32)
    out["keys"] = np.stack([c.keys(l, full=True) for l in range(layers)])
    out["values"] = np.stack([c.values(l, full=True) for l in range(layers)])
    if out["prefill_attn"]:
        out["prefill_attn"] = np.stack(out["prefill_attn"])
    else:
        out["prefill_attn"] = np.zeros((0,), np.float32)
    out["meta"] = np.array([c.capacity(), c.prefill_len(), c.bytes()], dtype=np.int64)
    return out


ROPE_CASES = {
    # name: (seq, heads, kv_heads, head_dim, theta, max_position, seed)
    "hd128": (19, 10, 10, 128, 10000.0, 6000, 31),
    "hd16_gqa": (7, 4, 2, 16, 1000000.0, 300000, 32),
}


def run_rope_case(o, seq, heads, kv_heads, hd, theta, max_pos, seed):
    """RoPE of seeded q / k at seeded positions through back end `o`: (q_out, k_out)."""
    q = synth.normal(seed, 0, (seq, heads * hd))
    k = synth.normal(seed, 1, (seq, kv_heads * hd))
    pos = synth.integers(seed, 2, 0, max_pos, (seq,)).astype(np.int32)
    return o.apply_rope(q, k, pos, heads, kv_heads, hd, theta)
