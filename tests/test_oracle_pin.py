"""Pins the CPU oracle (oracle/rswa_oracle.c) before anything is checked against it.

Three anchors:
 1. the known answers asserted by the reference's own unit tests for this path
    (tests/test_kv_ring_buffer.cpp, tests/test_memory_budget.cpp, tests/test_scheduler.cpp);
 2. the golden vectors in tests/golden/rswa_golden.npz, produced by the compiled reference;
 3. when the compiled reference is present, a live side-by-side run on fresh seeded traces.
"""
import math
import os

import numpy as np
import pytest

import synth
import traces
from golden.make_golden import CACHE_CASES

GOLD = np.load(os.path.join(os.path.dirname(__file__), "golden", "rswa_golden.npz"))


# ---- 1. known answers from the reference's tests --------------------------------------------

def test_ring_buffer_lifecycle_known_answers(orc):
    # tests/test_kv_ring_buffer.cpp:59-98
    L, kvh, hd, W, P = 1, 2, 4, 4, 3
    c = orc.Cache(L, kvh, hd, W)
    c.reset(P)
    assert (c.capacity(), c.prefill_len(), c.len(0)) == (P + W, P, P)
    pk, pv = synth.normal(42, 0, (P, kvh * hd)), synth.normal(42, 1, (P, kvh * hd))
    c.write_prefill(0, pk, pv)
    for i in range(W):
        c.append_decode(0, synth.normal(42, 10 + i, (kvh * hd,)), synth.normal(42, 50 + i, (kvh * hd,)))
    assert c.len(0) == P + W and c.ring_started(0)
    for i in range(5):
        c.append_decode(0, synth.normal(42, 100 + i, (kvh * hd,)), synth.normal(42, 150 + i, (kvh * hd,)))
    assert c.len(0) == P + W
    assert c.ring_pos(0) == 5 % W
    assert np.array_equal(c.keys(0)[:P], pk) and np.array_equal(c.values(0)[:P], pv)


def test_ring_attention_matches_naive(orc):
    # tests/test_kv_ring_buffer.cpp:100-124 (two-pass softmax, tolerance 1e-4)
    L, kvh, heads, hd, W, P = 1, 2, 2, 4, 4, 5
    c = orc.Cache(L, kvh, hd, W)
    c.reset(P)
    c.write_prefill(0, synth.normal(7, 0, (P, kvh * hd)), synth.normal(7, 1, (P, kvh * hd)))
    for i in range(13):
        c.append_decode(0, synth.normal(7, 10 + i, (kvh * hd,)), synth.normal(7, 50 + i, (kvh * hd,)))
    q = synth.normal(7, 99, (1, heads * hd))
    got = c.attention(0, q, c.len(0) - 1, heads, False)[0].reshape(heads, hd)
    K = c.keys(0).reshape(-1, kvh, hd).astype(np.float64)
    V = c.values(0).reshape(-1, kvh, hd).astype(np.float64)
    for h in range(heads):
        s = K[:, h] @ q.reshape(heads, hd)[h].astype(np.float64) / math.sqrt(hd)
        p = np.exp(s - s.max())
        want = (p / p.sum()) @ V[:, h]
        assert np.abs(got[h] - want).max() < 1e-4


def test_prefill_causal_attention(orc):
    # tests/test_kv_ring_buffer.cpp:126-161
    hd, W, P = 4, 4, 6
    c = orc.Cache(1, 1, hd, W)
    c.reset(P)
    k, v = synth.normal(3, 0, (P, hd)), synth.normal(3, 1, (P, hd))
    c.write_prefill(0, k, v)
    q = synth.normal(3, 2, (P, hd))
    got = c.attention(0, q, 0, 1, True)
    for s in range(P):
        sc = (k[: s + 1].astype(np.float64) @ q[s].astype(np.float64)) / math.sqrt(hd)
        p = np.exp(sc - sc.max())
        want = (p / p.sum()) @ v[: s + 1].astype(np.float64)
        assert np.abs(got[s] - want).max() < 1e-4


def test_memory_pool_known_answers(orc):
    # tests/test_memory_budget.cpp:7-41
    p = orc.Pool(1024, 64)
    assert p.state()[:2] == (1024, 0)
    a = p.allocate(100)
    assert a >= 0 and a % 64 == 0
    b = p.allocate(200)
    assert b > a
    assert p.state()[1] == 328  # alignment pad (28) is counted
    p.free(a, 100)
    assert p.state()[1] == 228
    assert p.allocate(50) >= 0 and p.state()[3] <= 3
    f = orc.Pool(1000, 1)
    offs = [f.allocate(200) for _ in range(4)]
    f.free(offs[0], 200)
    f.free(offs[2], 200)
    assert f.state()[4] > 0.5
    assert f.allocate(300) == -1
    assert f.allocate(200) >= 0
    assert orc.Pool(64, 1).allocate(0) == 0


def test_block_manager_known_answers(orc):
    # tests/test_memory_budget.cpp:43-66
    m = orc.BlockManager(1 << 20, 1 << 20)
    assert m.acquire_prefix("docA", 100, 4096)[1] == 1
    assert m.stats()[2] == 0
    assert m.acquire_prefix("docA", 100, 4096)[1] == 2
    assert m.stats()[7] == 1 and m.stats()[2] == 4096
    m.acquire_prefix("docB", 50, 2048)
    assert m.stats()[7] == 2
    m.release_prefix("docA")
    assert m.stats()[7] == 2
    m.release_prefix("docA")
    assert m.stats()[7] == 1
    m.release_prefix("docB")
    assert m.stats()[7] == 0
    m.release_prefix("never-seen")  # no-op
    small = orc.BlockManager(512, 512)
    assert small.acquire_prefix("x", 1, 1024)[0] == -1  # "prefix pool exhausted"


def test_scheduler_known_answers(orc):
    # tests/test_scheduler.cpp:6-58 -- batch sizes 4/4/4/2
    s = orc.Scheduler(4, 2)
    for _ in range(6):
        s.add_request(3, 2)
    assert s.stats()[4] == 6
    pf, dc = s.build_batch()
    assert (len(pf), len(dc)) == (4, 0)
    for i in pf:
        s.mark_prefilled(i)
    pf, dc = s.build_batch()
    assert (len(pf), len(dc)) == (0, 4)
    assert not any(s.add_token(i, 10) for i in dc)
    pf, dc = s.build_batch()
    assert len(dc) == 4 and all(s.add_token(i, 11) for i in dc)
    assert s.stats()[1] == 4
    pf, dc = s.build_batch()
    assert len(pf) == 2
    for i in pf:
        s.mark_prefilled(i)
    for i in s.build_batch()[1]:
        assert not s.add_token(i, 10)
    for i in s.build_batch()[1]:
        assert s.add_token(i, 11)
    assert s.stats()[1] == 6 and not s.has_work()
    one = orc.Scheduler(16, 4)
    one.add_request(1, 4096)
    assert len(one.build_batch()[0]) == 1


def test_closed_form_state_machine(orc):
    # after n appends: len = P + min(n, W); ring_pos = 0 if n < W else (n - W) % W
    for P, W in ((0, 1), (0, 4), (3, 4), (16, 16), (17, 48), (33, 32)):
        c = orc.Cache(1, 1, 4, W)
        c.reset(P)
        z = np.zeros(4, np.float32)
        for n in range(1, 3 * W + 3):
            c.append_decode(0, z, z)
            assert c.len(0) == P + min(n, W)
            assert c.ring_pos(0) == (0 if n < W else (n - W) % W)
            assert c.ring_started(0) == (n >= W)
    # the CPU-runnable benchmark configuration ends at len 384, ring_pos 44
    book = GOLD["cache/cfg1/book"]
    assert tuple(book[-1]) == (384, 44, 1)


# ---- 2. golden vectors from the compiled reference ---------------------------------------------

def _check_cache_case(lib, name, exact):
    L, kvh, hd, W, P, n, heads, seed, steps, bf16 = CACHE_CASES[name]
    r = traces.run_cache_trace(lib, L, kvh, hd, W, P, n, heads, seed, steps, bf16=bf16,
                               causal_prefill=(P <= 64))
    g = lambda k: GOLD[f"cache/{name}/{k}"]
    assert np.array_equal(r["book"], g("book"))
    assert np.array_equal(r["meta"], g("meta"))
    if f"cache/{name}/keys" in GOLD:
        assert np.array_equal(r["keys"], g("keys")) and np.array_equal(r["values"], g("values"))
    else:
        assert np.array_equal(r["keys"].astype(np.float64).sum(-1), g("keys_rowsum"))
        assert np.array_equal(r["values"].astype(np.float64).sum(-1), g("values_rowsum"))
    if exact:
        assert np.array_equal(r["attn"], g("attn"))
        assert np.array_equal(r["prefill_attn"], g("prefill_attn"))
    else:
        assert np.abs(r["attn"] - g("attn")).max() <= 1e-5
        if r["prefill_attn"].size:
            assert np.abs(r["prefill_attn"] - g("prefill_attn")).max() <= 1e-5


@pytest.mark.parametrize("name", list(CACHE_CASES))
def test_oracle_cache_matches_golden(orc, name):
    # cache contents and cursors bit-exact; attention to 1e-5 (libm expf may differ in the last ulp
    # between a C and a C++ build; in practice the two agree exactly here)
    _check_cache_case(orc, name, exact=False)


@pytest.mark.parametrize("key,align", [("pool", 256), ("pool1", 1)])
def test_oracle_pool_matches_golden(orc, key, align):
    total, al = GOLD[f"{key}/cfg"].tolist()
    assert al == align
    assert np.array_equal(traces.run_pool_trace(orc, GOLD[f"{key}/ops"], total, al), GOLD[f"{key}/res"])


def test_oracle_block_manager_matches_golden(orc):
    pb, rb = GOLD["bm/cfg"].tolist()
    res = traces.run_bm_trace(orc, GOLD["bm/ops"], pb, rb)
    assert np.array_equal(res, GOLD["bm/res"])
    assert (GOLD["bm/res"][:, 0] % 256 == 0)[GOLD["bm/res"][:, 0] > 0].all()  # block-unit offsets


def test_oracle_scheduler_matches_golden(orc):
    assert np.array_equal(traces.run_sched_trace(orc, GOLD["sched/script"], 16), GOLD["sched/res"])
    assert np.array_equal(traces.run_sched_trace(orc, GOLD["sched/script"], 5, early_finish_every=7),
                          GOLD["sched/res_early"])


@pytest.mark.parametrize("name", list(traces.ROPE_CASES))
def test_oracle_rope_matches_golden(orc, name):
    # the restatement calls the same libm float functions as the reference build: bit-exact
    q, k = traces.run_rope_case(orc, *traces.ROPE_CASES[name])
    assert np.array_equal(q, GOLD[f"rope/{name}/q"]) and np.array_equal(k, GOLD[f"rope/{name}/k"])


# ---- 3. live comparison with the compiled reference ---------------------------------------------

def test_golden_is_what_the_reference_produces(ref):
    for name in ("tiny", "p0", "ragged_p17"):
        _check_cache_case(ref, name, exact=True)


@pytest.mark.parametrize("seed", [101, 102, 103])
def test_live_reference_vs_oracle_random(orc, ref, seed):
    P = int(synth.integers(seed, 1, 0, 40, (1,))[0])
    W = int(synth.integers(seed, 2, 1, 24, (1,))[0])
    a = traces.run_cache_trace(orc, 2, 2, 8, W, P, 3 * W + 5, 4, seed, tuple(range(0, 3 * W + 5, 3)))
    b = traces.run_cache_trace(ref, 2, 2, 8, W, P, 3 * W + 5, 4, seed, tuple(range(0, 3 * W + 5, 3)))
    for k in ("book", "keys", "values", "meta"):
        assert np.array_equal(a[k], b[k])
    assert np.abs(a["attn"] - b["attn"]).max() <= 1e-6
    ops, total = traces.make_pool_ops(seed, 1500, 1 << 14, 900, aligns=(0, 16, 256))
    assert np.array_equal(traces.run_pool_trace(orc, ops, total, 256), traces.run_pool_trace(ref, ops, total, 256))
    bops = traces.make_bm_ops(seed, 1500, 8, 40, 16)
    assert np.array_equal(traces.run_bm_trace(orc, bops, 256, 400), traces.run_bm_trace(ref, bops, 256, 400))
    sc = traces.make_sched_script(seed, 80, 12)
    assert np.array_equal(traces.run_sched_trace(orc, sc, 7, 5), traces.run_sched_trace(ref, sc, 7, 5))


def test_bf16_rounding_rule(orc):
    x = np.concatenate([synth.normal(5, 0, (4096,)) * 37.0,
                        np.array([0.0, -0.0, 1.0, np.inf, -np.inf, 1.00390625, 1.01171875, 3.3895314e38], np.float32)])
    assert np.array_equal(orc.round_bf16(x), synth.round_bf16(x))
    assert orc.f32_to_bf16(1.00390625) == 0x3F80  # tie -> even
    assert orc.f32_to_bf16(1.01171875) == 0x3F82  # tie -> even (odd neighbour rounds up)
