"""Block-manager churn workload: seeded Poisson arrivals, 1 of 8 shared prefixes per request, random
output lengths; every scheduler step admits, appends one token per running sequence per layer, and
retires finished sequences (ring freed, prefix reference dropped).

`impl` is the allocator/scheduler under test (the CUDA library's host classes through their C ABI);
`check` is an optional second implementation (the CPU oracle or the compiled reference) run in
lockstep: every block-table row handed out, every stats tuple and every scheduler batch must be
equal.  Device work (append, and a gather of each retiring sampled sequence) runs through the C ABI.
"""
from __future__ import annotations

import math

import numpy as np

import synth
from paged_fixture import ceil_div, load_b200

PREFIX_LENS = (256, 416, 576, 752, 912, 1088, 1264, 1456)  # multiples of 16 between 256 and 1456


class ChurnConfig:
    def __init__(self, **kw):
        self.requests = 1000
        self.slots = 256
        self.layers = 12
        self.kv_heads, self.head_dim = 10, 128
        self.window = 1024
        self.prefix_lens = PREFIX_LENS
        self.out_lo, self.out_hi = 32, 2048
        self.prefix_arena_blocks = 1024
        self.ring_arena_blocks = 64512
        self.mean_interarrival = 2.0
        self.seed = 1234
        self.sample_every = 0      # value-check every n-th request against an oracle cache (0 = off)
        self.gather_on_finish = True
        self.all_layer_launches = False  # append / gather of every layer in one launch instead of one per layer
        self.__dict__.update(kw)


def arrivals(cfg):
    """Exponential inter-arrival times (mean cfg.mean_interarrival scheduler steps) from the integer
    hash generator: u -> -mean * ln(1 - u)."""
    u = (synth.integers(cfg.seed, 901, 0, (1 << 24) - 1, (cfg.requests,)).astype(np.float64) + 0.5) / (1 << 24)
    gaps = -cfg.mean_interarrival * np.log1p(-u)
    return np.floor(np.cumsum(gaps)).astype(np.int64)


def run(cfg, impl, check=None, oracle_caches=None, time_kernels=False, device=True):
    """`device=False` replays the bookkeeping alone (allocator, scheduler, slots, block-table rows: host
    integers) with no KV writes, so the full-size schedule can be checked without a GPU."""
    b = load_b200()
    bt = b.BLOCK_TOKENS
    L, row, W = cfg.layers, cfg.kv_heads * cfg.head_dim, cfg.window
    rb = ceil_div(W, bt)
    stride = ceil_div(max(cfg.prefix_lens), bt) + rb
    num_blocks = cfg.prefix_arena_blocks + cfg.ring_arena_blocks
    host_table = np.full((cfg.slots, stride), -1, np.int32)
    host_len = np.zeros(cfg.slots, np.int64)       # tokens appended so far, per slot (closed-form cursors)
    host_prefill = np.zeros(cfg.slots, np.int64)
    if device:
        import torch
        table = torch.full((cfg.slots, stride), -1, dtype=torch.int32, device="cuda")
        layers = [b.PagedLayer(num_blocks, cfg.kv_heads, cfg.head_dim, b.BF16, table) for _ in range(L)]
        d_len = torch.zeros((L, cfg.slots), dtype=torch.int32, device="cuda")
        d_ring = torch.zeros((L, cfg.slots), dtype=torch.int32, device="cuda")
        d_prefill = torch.zeros(cfg.slots, dtype=torch.int32, device="cuda")
        ws = b.Workspace(max(cfg.slots, 64))

    arr = arrivals(cfg)
    pkey = synth.integers(cfg.seed, 902, 0, len(cfg.prefix_lens) - 1, (cfg.requests,))
    olen = synth.integers(cfg.seed, 903, cfg.out_lo, cfg.out_hi, (cfg.requests,))

    impls = [impl] + ([check] if check is not None else [])
    bms = [x.BlockManager(cfg.prefix_arena_blocks * 256, cfg.ring_arena_blocks * 256) for x in impls]
    scheds = [x.Scheduler(cfg.slots, 4) for x in impls]
    free_slots = list(range(cfg.slots))  # handed out from the back, released slots reused first
    slot_of, ring_of, rows_log, mismatches = {}, {}, [], 0
    cap = max(cfg.prefix_lens) + W
    if device:
        k_in = torch.randn((L, cfg.slots, row), device="cuda")
        v_in = torch.randn((L, cfg.slots, row), device="cuda")
        gk = torch.empty((1, cap, row), dtype=torch.bfloat16, device="cuda")
        gv = torch.empty_like(gk)
        if cfg.all_layer_launches:
            gk_all = torch.empty((L, 1, cap, row), dtype=torch.bfloat16, device="cuda")
            gv_all = torch.empty_like(gk_all)
    stats = dict(steps=0, append_rows=0, append_ms=0.0, gather_tokens=0, gather_ms=0.0, peak_running=0,
                 prefix_hits=0, prefix_misses=0)
    ev = [torch.cuda.Event(enable_timing=True) for _ in range(4)] if device else []
    sampled = {}
    nxt, step = 0, 0
    while nxt < cfg.requests or scheds[0].has_work():
        while nxt < cfg.requests and arr[nxt] <= step:
            for s in scheds:
                s.add_request(int(cfg.prefix_lens[pkey[nxt]]), int(olen[nxt]))
            nxt += 1
        batches = [s.build_batch() for s in scheds]
        if check is not None and batches[0] != batches[1]:
            mismatches += 1
        pf, dc = batches[0]
        # ---- admissions: slot, shared prefix, ring; one table row each ------------------------------
        for rid in pf:
            slot = free_slots.pop()
            slot_of[rid] = slot
            P = int(cfg.prefix_lens[pkey[rid]])
            pb = ceil_div(P, bt)
            got = []
            for bm in bms:
                off, rc = bm.acquire_prefix(f"doc{pkey[rid]}", P, pb * 256)
                roff = bm.allocate_ring(rb * 256)
                assert off >= 0 and roff >= 0, "arena exhausted"
                got.append((off, rc, roff))
            if check is not None and got[0] != got[1]:
                mismatches += 1
            off, rc, roff = got[0]
            stats["prefix_hits" if rc > 1 else "prefix_misses"] += 1
            ring_of[rid] = roff
            r = np.full(stride, -1, np.int32)
            r[:pb] = off // 256 + np.arange(pb)
            r[pb:pb + rb] = cfg.prefix_arena_blocks + roff // 256 + np.arange(rb)
            rows_log.append((rid, slot, r.copy()))
            host_table[slot] = r
            host_len[slot] = 0
            host_prefill[slot] = P
            if device:
                table[slot].copy_(torch.from_numpy(r))
                d_len[:, slot] = P
                d_ring[:, slot] = 0
                d_prefill[slot] = P
            if oracle_caches is not None and cfg.sample_every and rid % cfg.sample_every == 0:
                c = oracle_caches.Cache(L, cfg.kv_heads, cfg.head_dim, W)
                c.reset(P)
                if rc == 1:  # first user of this prefix writes it (values: zeros stay zeros in both)
                    pass
                sampled[rid] = c
            for s in scheds:
                s.mark_prefilled(rid)
        # ---- one token per running sequence per layer ---------------------------------------------------
        run_ids = [i for i in dc] + [i for i in pf]
        stats["peak_running"] = max(stats["peak_running"], len(run_ids))
        for i in run_ids:
            host_len[slot_of[i]] += 1
        if run_ids and not device:
            stats["append_rows"] += len(run_ids) * L
        if run_ids and device:
            rows = torch.tensor([slot_of[i] for i in run_ids], dtype=torch.int32, device="cuda")
            n = len(run_ids)
            if time_kernels:
                ev[0].record()
            if cfg.all_layer_launches:  # one launch for the append of every layer
                b.append_decode_batch_paged_layers(layers, k_in, v_in, d_len, d_ring, d_prefill, rows, n, W, ws)
            else:
                for l in range(L):
                    b.append_decode_batch_paged(layers[l], k_in[l], v_in[l], d_len[l], d_ring[l], d_prefill, rows, n, W, ws)
            if time_kernels:
                ev[1].record()
                ev[1].synchronize()
                stats["append_ms"] += ev[0].elapsed_time(ev[1])
            stats["append_rows"] += n * L
            if sampled:
                kh = synth.round_bf16(k_in[:, :n].float().cpu().numpy())
                vh = synth.round_bf16(v_in[:, :n].float().cpu().numpy())
                for j, i in enumerate(run_ids):
                    if i in sampled:
                        for l in range(L):
                            sampled[i].append_decode(l, kh[l, j], vh[l, j])
        # ---- retire ---------------------------------------------------------------------------------------------
        for i in run_ids:
            done = [s.add_token(i, 1) for s in scheds]
            if check is not None and done[0] != done[1]:
                mismatches += 1
            if not done[0]:
                continue
            slot = slot_of.pop(i)
            P = int(cfg.prefix_lens[pkey[i]])
            if device:  # device cursors equal the closed form of the ring state machine for this slot
                n_app = int(host_len[slot])
                want_len = P + min(n_app, W)
                want_ring = 0 if n_app < W else (n_app - W) % W
                assert int(d_len[0, slot]) == want_len and int(d_ring[0, slot]) == want_ring
            if cfg.gather_on_finish and device:
                sl = torch.tensor([slot], dtype=torch.int32, device="cuda")
                if time_kernels:
                    ev[2].record()
                if cfg.all_layer_launches and i not in sampled:
                    b.gather_paged_layers(layers, d_len, d_prefill, sl, 1, cap, gk_all, gv_all, b.BF16, ws)
                for l in range(0 if (cfg.all_layer_launches and i not in sampled) else (L if (time_kernels or i in sampled) else 1)):
                    b.gather_paged(layers[l], d_len[l], d_prefill, sl, 1, cap, gk, gv, b.BF16, ws)
                    if i in sampled:
                        c = sampled[i]
                        nn = c.len(l)
                        assert int(d_len[l, slot]) == nn and int(d_ring[l, slot]) == c.ring_pos(l)
                        assert np.array_equal(gk[0, P:nn].float().cpu().numpy(), c.keys(l)[P:])
                        assert np.array_equal(gv[0, P:nn].float().cpu().numpy(), c.values(l)[P:])
                if time_kernels:
                    ev[3].record()
                    ev[3].synchronize()
                    stats["gather_ms"] += ev[2].elapsed_time(ev[3])
                    stats["gather_tokens"] += int(d_len[0, slot]) * L
            sampled.pop(i, None)
            for bm in bms:
                bm.free_ring(ring_of[i], rb * 256)
                bm.release_prefix(f"doc{pkey[i]}")
            ring_of.pop(i)
            free_slots.append(slot)
            host_table[slot] = -1
            if device:
                table[slot] = -1
        if check is not None and bms[0].stats() != bms[1].stats():
            mismatches += 1
        step += 1
        stats["steps"] = step
        assert step < 10_000_000
    if device:
        assert ws.status() == 0
        assert np.array_equal(table.cpu().numpy(), host_table)
    final = [bm.stats() for bm in bms]
    sched_final = [s.stats() for s in scheds]
    return dict(stats=stats, rows=rows_log, mismatches=mismatches, final=final, sched=sched_final, table=host_table,
                row_bytes_in=row * 4 * 2, row_bytes_out=row * 2 * 2)
