"""Test helper: a batch of paged R-SWA sequences on the device next to one CPU-oracle cache per slot.

Block ids are handed out the way the parity rule for paging prescribes: the oracle's BlockManager is
run in block units (1 block == 256 arena bytes, the arena's alignment), prefix arena ids come first,
ring ids follow (`ring_id = n_prefix_blocks_total + offset / 256`).
"""
from __future__ import annotations

import importlib.util
import os

import numpy as np

import synth

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def load_b200():
    import sys
    if "uocr_b200" in sys.modules:
        return sys.modules["uocr_b200"]
    spec = importlib.util.spec_from_file_location(
        "uocr_b200", os.path.join(ROOT, "unlimited-ocr.cpp_b200", "__init__.py"))
    mod = importlib.util.module_from_spec(spec)
    sys.modules["uocr_b200"] = mod
    spec.loader.exec_module(mod)
    return mod


def ceil_div(a, b):
    return (a + b - 1) // b


class PagedBatch:
    def __init__(self, orc, slots, layers, kv_heads, head_dim, window, dtype, prefix_lens,
                 prefix_keys=None, heads=None, seed=1, prefix_arena_blocks=None, extra_blocks=0):
        import torch
        self.b = load_b200()
        self.torch = torch
        self.orc = orc
        self.slots, self.layers, self.kvh, self.hd, self.W = slots, layers, kv_heads, head_dim, window
        self.heads = heads or kv_heads
        self.dtype = dtype
        self.row = kv_heads * head_dim
        self.P = list(prefix_lens)
        self.keys = list(prefix_keys) if prefix_keys is not None else [f"slot{i}" for i in range(slots)]
        self.seed = seed
        self.rnd = synth.round_bf16 if dtype == self.b.BF16 else (lambda x: x)
        bt = self.b.BLOCK_TOKENS
        distinct = {}
        for s in range(slots):
            distinct.setdefault(self.keys[s], self.P[s])
            assert distinct[self.keys[s]] == self.P[s]
        n_pref = sum(ceil_div(p, bt) for p in distinct.values())
        self.n_pref_arena = prefix_arena_blocks or max(n_pref, 1)
        ring_blocks = ceil_div(window, bt)
        n_ring = slots * ring_blocks
        self.num_blocks = self.n_pref_arena + n_ring + extra_blocks
        self.bm = orc.BlockManager(self.n_pref_arena * 256, (n_ring + extra_blocks) * 256)
        self.stride = max(ceil_div(p, bt) for p in self.P) + ring_blocks
        table = np.full((slots, self.stride), -1, np.int32)
        self.prefix_first_slot = {}
        for s in range(slots):
            nb = ceil_div(self.P[s], bt)
            if nb:
                off, _ = self.bm.acquire_prefix(self.keys[s], self.P[s], nb * 256)
                assert off >= 0
                table[s, :nb] = off // 256 + np.arange(nb)
            self.prefix_first_slot.setdefault(self.keys[s], s)
            roff = self.bm.allocate_ring(ring_blocks * 256)
            assert roff >= 0
            table[s, nb:nb + ring_blocks] = self.n_pref_arena + roff // 256 + np.arange(ring_blocks)
        self.table_np = table
        dev = "cuda"
        self.table = torch.from_numpy(table).to(dev)
        self.layer = [self.b.PagedLayer(self.num_blocks, kv_heads, head_dim, dtype, self.table) for _ in range(layers)]
        self.d_prefill = torch.tensor(self.P, dtype=torch.int32, device=dev)
        self.d_len = torch.tensor([self.P] * layers, dtype=torch.int32, device=dev).contiguous()
        self.d_ring = torch.zeros((layers, slots), dtype=torch.int32, device=dev)
        self.ws = self.b.Workspace(max(slots, max(self.P + [1]) * 2, 64))
        self.cache = [orc.Cache(layers, kv_heads, head_dim, window) for _ in range(slots)]
        for s in range(slots):
            self.cache[s].reset(self.P[s])

    # ---- prefix -------------------------------------------------------------------------------
    def prefix_kv(self, key, layer):
        p = self.P[self.prefix_first_slot[key]]
        h = abs(hash(key)) % 100000 if False else sum(ord(c) for c in key)
        k = self.rnd(synth.normal(self.seed, 7000 + h * 64 + layer, (p, self.row)))
        v = self.rnd(synth.normal(self.seed, 9000 + h * 64 + layer, (p, self.row)))
        return k, v

    def write_prefixes(self):
        torch = self.torch
        for l in range(self.layers):
            for key, s0 in self.prefix_first_slot.items():
                p = self.P[s0]
                if p == 0:
                    continue
                k, v = self.prefix_kv(key, l)
                dk, dv = torch.from_numpy(k).cuda(), torch.from_numpy(v).cuda()
                slots = torch.full((p,), s0, dtype=torch.int32, device="cuda")
                pos = torch.arange(p, dtype=torch.int32, device="cuda")
                self.b.write_prefill_ragged_paged(self.layer[l], dk, dv, slots, pos, p, self.ws)
            for s in range(self.slots):
                if self.P[s]:
                    k, v = self.prefix_kv(self.keys[s], l)
                    self.cache[s].write_prefill(l, k, v)
        torch.cuda.synchronize()

    # ---- decode ---------------------------------------------------------------------------------
    def step_inputs(self, t, layer, rows):
        k = self.rnd(synth.normal(self.seed, 100000 + t * 64 + layer, (self.slots, self.row)))[rows]
        v = self.rnd(synth.normal(self.seed, 300000 + t * 64 + layer, (self.slots, self.row)))[rows]
        q = synth.normal(self.seed, 500000 + t * 64 + layer, (self.slots, self.heads * self.hd))[rows]
        return np.ascontiguousarray(k), np.ascontiguousarray(v), np.ascontiguousarray(q)

    def append(self, layer, k, v, row_slots):
        """row i of k/v goes to slot row_slots[i]; device + oracle."""
        torch = self.torch
        dk, dv = torch.from_numpy(k).cuda(), torch.from_numpy(v).cuda()
        ds = torch.tensor(row_slots, dtype=torch.int32, device="cuda")
        self.b.append_decode_batch_paged(self.layer[layer], dk, dv, self.d_len[layer], self.d_ring[layer],
                                         self.d_prefill, ds, len(row_slots), self.W, self.ws)
        for i, s in enumerate(row_slots):
            self.cache[s].append_decode(layer, k[i], v[i])

    def attend(self, layer, q, row_slots):
        torch = self.torch
        dq = torch.from_numpy(q).cuda()
        ds = torch.tensor(row_slots, dtype=torch.int32, device="cuda")
        out = torch.full((len(row_slots), self.heads * self.hd), float("nan"), device="cuda")
        self.b.attention_batch_paged(self.layer[layer], dq, self.d_len[layer], self.d_prefill, ds,
                                     len(row_slots), self.heads, out, self.ws)
        got = out.cpu().numpy()
        want = np.stack([self.cache[s].attention(layer, q[i:i + 1], self.cache[s].len(layer) - 1, self.heads, False)[0]
                         for i, s in enumerate(row_slots)])
        return got, want

    def step_fused(self, layer, k, v, q, row_slots, host_out=False):
        """append + attention in one launch (decode_step_paged); oracle advanced alongside.  With
        `host_out` the kernel stores the result straight into pinned (device-mapped) host memory."""
        torch = self.torch
        dk, dv, dq = (torch.from_numpy(x).cuda() for x in (k, v, q))
        ds = torch.tensor(row_slots, dtype=torch.int32, device="cuda")
        shape = (len(row_slots), self.heads * self.hd)
        if host_out:
            out = torch.full(shape, float("nan")).pin_memory()
        else:
            out = torch.full(shape, float("nan"), device="cuda")
        self.b.decode_step_paged(self.layer[layer], dq, dk, dv, self.d_len[layer], self.d_ring[layer],
                                 self.d_prefill, ds, len(row_slots), self.W, self.heads, out, self.ws)
        if host_out:
            torch.cuda.synchronize()
            got = out.numpy().copy()
        else:
            got = out.cpu().numpy()
        want = []
        for i, s in enumerate(row_slots):
            self.cache[s].append_decode(layer, k[i], v[i])
            want.append(self.cache[s].attention(layer, q[i:i + 1], self.cache[s].len(layer) - 1, self.heads, False)[0])
        return got, np.stack(want)

    def gather(self, layer, slot_ids, out_dtype=0):
        torch = self.torch
        cap = max(self.P) + self.W
        ds = torch.tensor(slot_ids, dtype=torch.int32, device="cuda")
        tdt = torch.float32 if out_dtype == 0 else torch.bfloat16
        ok = torch.full((len(slot_ids), cap, self.row), float("nan"), dtype=tdt, device="cuda")
        ov = torch.full((len(slot_ids), cap, self.row), float("nan"), dtype=tdt, device="cuda")
        self.b.gather_paged(self.layer[layer], self.d_len[layer], self.d_prefill, ds, len(slot_ids), cap, ok, ov,
                            out_dtype, self.ws)
        return ok.float().cpu().numpy(), ov.float().cpu().numpy()

    def check_logical_view(self, layer):
        """gather == oracle keys()/values() bit for bit, zero beyond len; cursors equal."""
        gk, gv = self.gather(layer, list(range(self.slots)))
        dl = self.d_len[layer].cpu().numpy()
        dr = self.d_ring[layer].cpu().numpy()
        for s in range(self.slots):
            c = self.cache[s]
            n = c.len(layer)
            assert dl[s] == n, (s, dl[s], n)
            assert dr[s] == c.ring_pos(layer), (s, dr[s], c.ring_pos(layer))
            assert np.array_equal(gk[s, :n], c.keys(layer)), f"K mismatch slot {s}"
            assert np.array_equal(gv[s, :n], c.values(layer)), f"V mismatch slot {s}"
            assert not gk[s, n:].any() and not gv[s, n:].any()


def assert_attention_close(got, want, max_abs, rel_l2):
    assert np.isfinite(got).all(), "non-finite attention output"
    err = np.abs(got - want).max()
    rl2 = np.linalg.norm(got - want) / max(np.linalg.norm(want), 1e-30)
    assert err <= max_abs, f"max-abs {err} > {max_abs}"
    assert rl2 <= rel_l2, f"rel-L2 {rl2} > {rel_l2}"
    return err, rl2
