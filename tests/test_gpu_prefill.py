"""Ragged prefill with ring fill (the configuration whose prompts can exceed the window) against the
composed oracle: reset(Pv), write_prefill(vision), causal attention for the vision queries, then for
every text token in order append_decode + attention(seq=1) -- only reference calls
(src/scheduler/kv_cache.cpp:45-130).  Outputs within the attention tolerance (bf16: 2e-2 / 1e-3; the
observed 2e-5 / 1e-5 is asserted too), final cache contents and cursors bit-exact, and decode steps
that follow the prefill keep agreeing."""
import numpy as np
import pytest

import synth
from paged_fixture import PagedBatch, assert_attention_close, ceil_div, load_b200

pytestmark = pytest.mark.gpu
TIGHT = (2e-5, 1e-5)
TC_TIGHT = (2e-4, 1e-4)  # tensor-core path: Q and P enter as bf16 hi+lo pairs (~16 mantissa bits)


@pytest.fixture(scope="module")
def b():
    import torch
    if not torch.cuda.is_available():
        pytest.skip("needs a CUDA device")
    return load_b200()


def run_prefill_case(orc, b, dtype, kvh, hd, heads, W, prefixes, text_lens, seed, decode_after=5, engine="cuda"):
    import torch
    slots = len(prefixes)
    pb = PagedBatch(orc, slots, 1, kvh, hd, W, dtype, prefixes, heads=heads, seed=seed)
    row = kvh * hd
    rnd = pb.rnd
    # ---- vision prefix: scatter + causal attention over packed rows of all requests ----------------
    pb.write_prefixes()
    vis_rows = [(s, p) for s in range(slots) for p in range(prefixes[s])]
    if vis_rows:
        rs = torch.tensor([s for s, _ in vis_rows], dtype=torch.int32, device="cuda")
        pos = torch.tensor([p for _, p in vis_rows], dtype=torch.int32, device="cuda")
        qv = synth.normal(seed, 41, (len(vis_rows), heads * hd))
        out = torch.full((len(vis_rows), heads * hd), float("nan"), device="cuda")
        big = b.Workspace(max(len(vis_rows), sum(text_lens), 64))
        if engine in ("tc", "tc_fused"):
            reqs, at = [], 0
            for s in range(slots):
                if prefixes[s]:
                    reqs.append((at, prefixes[s], s, 0, 0, 0))
                at += prefixes[s]
            b.prefill_attention_tc(pb.layer[0], None, None, 0, torch.from_numpy(qv).cuda(), pb.d_prefill,
                                   b.make_prefill_tiles(reqs), W, heads, out, big)
        else:
            b.attention_ragged_paged(pb.layer[0], torch.from_numpy(qv).cuda(), pb.d_prefill, rs, pos, len(vis_rows), heads, out, big)
        got = out.cpu().numpy()
        at = 0
        for s in range(slots):
            n = prefixes[s]
            if n:
                want = pb.cache[s].attention(0, qv[at:at + n], 0, heads, True)
                assert_attention_close(got[at:at + n], want, *(TC_TIGHT if engine != "cuda" else TIGHT))
            at += n
    else:
        big = b.Workspace(max(sum(text_lens), 64))
    # ---- text tokens: packed rows, window may wrap ------------------------------------------------------
    total = sum(text_lens)
    block0, nb = [], 0
    for T in text_lens:
        block0.append(nb)
        nb += ceil_div(max(T, 1), 16)
    tdt = torch.bfloat16 if dtype == b.BF16 else torch.float32
    text_k = torch.zeros((nb, kvh, 16, hd), dtype=tdt, device="cuda")
    text_v = torch.zeros_like(text_k)
    k = rnd(synth.normal(seed, 51, (total, row)))
    v = rnd(synth.normal(seed, 52, (total, row)))
    q = synth.normal(seed, 53, (total, heads * hd))
    rs = np.concatenate([np.full(T, s) for s, T in enumerate(text_lens)]).astype(np.int32)
    pos = np.concatenate([np.arange(T) for T in text_lens]).astype(np.int32)
    b0 = np.concatenate([np.full(T, block0[s]) for s, T in enumerate(text_lens)]).astype(np.int32)
    tl = np.concatenate([np.full(T, T) for T in text_lens]).astype(np.int32)
    d = lambda a: torch.from_numpy(np.ascontiguousarray(a)).cuda()
    drs, dpos, db0, dtl = d(rs), d(pos), d(b0), d(tl)
    out = torch.full((total, heads * hd), float("nan"), device="cuda")
    tc = engine in ("tc", "tc_fused")
    if tc:
        if engine == "tc_fused":  # scatter, ring fill and cursor publication in one pass, before the attention
            b.text_scatter_fill_paged(pb.layer[0], text_k, text_v, nb, d(k), d(v), drs, dpos, db0, dtl, pb.d_prefill,
                                      pb.d_len[0], pb.d_ring[0], total, W, big)
        else:
            b.text_scatter_paged(pb.layer[0], text_k, text_v, nb, d(k), d(v), dpos, db0, total, big)
        reqs, at = [], 0
        for s, T in enumerate(text_lens):
            if T:
                reqs.append((at, T, s, 1, 0, block0[s]))
            at += T
        b.prefill_attention_tc(pb.layer[0], text_k, text_v, nb, d(q), pb.d_prefill, b.make_prefill_tiles(reqs), W, heads,
                               out, big)
    else:
        b.prefill_text_paged(pb.layer[0], text_k, text_v, nb, d(q), d(k), d(v), pb.d_prefill, drs, dpos, db0, total, W,
                             heads, out, big)
    if engine != "tc_fused":
        b.ring_fill_paged(pb.layer[0], text_k, text_v, nb, drs, dpos, db0, dtl, pb.d_prefill, pb.d_len[0], pb.d_ring[0],
                          total, W, big)
    got = out.cpu().numpy()
    at = 0
    for s, T in enumerate(text_lens):
        want = []
        for i in range(T):
            pb.cache[s].append_decode(0, k[at + i], v[at + i])
            want.append(pb.cache[s].attention(0, q[at + i:at + i + 1], pb.cache[s].len(0) - 1, heads, False)[0])
        if T:
            tol = (2e-2, 1e-3) if dtype == b.BF16 else (1e-3, 1e-3)
            assert_attention_close(got[at:at + T], np.array(want), *tol)
            assert_attention_close(got[at:at + T], np.array(want), *(TC_TIGHT if engine != "cuda" else TIGHT))
        at += T
    pb.check_logical_view(0)  # ring contents + len + ring_pos bit-exact after the fill
    # ---- decode continues from the prefilled state -----------------------------------------------------------
    rows = list(range(slots))
    for t in range(decode_after):
        kk, vv, qq = pb.step_inputs(t, 0, rows)
        g, w = pb.step_fused(0, kk, vv, qq, rows)
        assert_attention_close(g, w, *TIGHT)
    pb.check_logical_view(0)
    assert big.status() == 0 and pb.ws.status() == 0


@pytest.mark.parametrize("dtype_name", ["bf16", "f32"])
@pytest.mark.parametrize("W", [16, 24])
def test_prefill_text_window_wraps_tiny(orc, b, dtype_name, W):
    dtype = b.BF16 if dtype_name == "bf16" else b.F32
    run_prefill_case(orc, b, dtype, 2, 8, 4, W, prefixes=[0, 7, 16, 33, 5, 16, 1],
                     text_lens=[40, 1, 0, 70, 16, 17, W], seed=600 + W)


def test_prefill_text_real_head_geometry(orc, b):
    # 10 heads x 128; prefixes like "256 global + crops" scaled down; prompts shorter and longer than W
    run_prefill_case(orc, b, b.BF16, 10, 128, 10, 32, prefixes=[48, 20, 65], text_lens=[80, 12, 33], seed=77)


def test_prefill_tensor_core_small(orc, b):
    # tcgen05 path, one head, short rows: every mask shape (causal prefix, partial tiles, window wrap)
    run_prefill_case(orc, b, b.BF16, 1, 128, 1, 32, prefixes=[20, 0, 130], text_lens=[40, 7, 150], seed=91, engine="tc")


def test_prefill_tensor_core_fused_scatter_and_fill(orc, b):
    # text scatter + ring fill + cursor publication as one kernel ahead of the attention: same outputs, and
    # ring contents / cursors bit-equal to the appends (checked inside through the logical view); prompts
    # shorter than, equal to and longer than the window, a zero-length prompt, a request without prefix
    run_prefill_case(orc, b, b.BF16, 2, 128, 2, 48, prefixes=[20, 0, 130, 33], text_lens=[40, 48, 150, 0], seed=93,
                     engine="tc_fused")


def test_prefill_tensor_core_real_geometry(orc, b):
    # 10 heads x 128, prefixes and prompts spanning several 128-row / 128-key tiles, window shorter than prompts
    run_prefill_case(orc, b, b.BF16, 10, 128, 10, 160, prefixes=[272, 48, 656], text_lens=[300, 130, 64], seed=92,
                     engine="tc")


def test_prefill_tensor_core_grouped_heads(orc, b):
    # six query heads on two KV heads (three query heads read each KV head's tiles), through both text paths
    run_prefill_case(orc, b, b.BF16, 2, 128, 6, 48, prefixes=[150, 20, 0], text_lens=[70, 130, 49], seed=94, engine="tc")
    run_prefill_case(orc, b, b.BF16, 2, 128, 6, 48, prefixes=[150, 20, 0], text_lens=[70, 130, 49], seed=95, engine="tc_fused")


def test_prefill_tensor_core_bf16_output(orc, b):
    # the workspace's bf16 output option on the tcgen05 path: same rows as fp32, rounded to nearest even
    import torch
    kvh = heads = 2
    hd, W, P, T = 128, 48, 40, 150
    pb = PagedBatch(orc, 1, 1, kvh, hd, W, b.BF16, [P], heads=heads, seed=31)
    pb.write_prefixes()
    ws = b.Workspace(256)
    nb = ceil_div(T, 16)
    text_k = torch.zeros((nb, kvh, 16, hd), dtype=torch.bfloat16, device="cuda")
    text_v = torch.zeros_like(text_k)
    k = pb.rnd(synth.normal(31, 51, (T, kvh * hd)))
    v = pb.rnd(synth.normal(31, 52, (T, kvh * hd)))
    q = synth.normal(31, 53, (P + T, heads * hd))
    d = lambda a: torch.from_numpy(np.ascontiguousarray(a)).cuda()
    pos = np.arange(T, dtype=np.int32)
    b.text_scatter_paged(pb.layer[0], text_k, text_v, nb, d(k), d(v), d(pos), d(np.zeros(T, np.int32)), T, ws)
    tiles = b.make_prefill_tiles([(0, P, 0, 0, 0, 0), (P, T, 0, 1, 0, 0)])
    out32 = torch.full((P + T, heads * hd), float("nan"), device="cuda")
    b.prefill_attention_tc(pb.layer[0], text_k, text_v, nb, d(q), pb.d_prefill, tiles, W, heads, out32, ws)
    ws.set_out_dtype(b.BF16)
    out16 = torch.full((P + T, heads * hd), float("nan"), dtype=torch.bfloat16, device="cuda")
    serial = b.lib().uocr_b200_workspace_prefill_plan_serial(ws.h)
    # the second call shares the first call's plan of the tiles
    b.prefill_attention_tc(pb.layer[0], text_k, text_v, nb, d(q), pb.d_prefill, tiles, W, heads, out16, ws, reuse_plan=True)
    assert b.lib().uocr_b200_workspace_prefill_plan_serial(ws.h) == serial
    a, c = out32.cpu().numpy(), out16.float().cpu().numpy()
    assert np.isfinite(a).all() and np.array_equal(c, synth.round_bf16(a))  # same kernel, same fp32 values, RNE
    # a plan made on its own serves as well; without a matching plan the call is refused
    assert b.prefill_plan_tc(tiles, pb.d_prefill, W, ws) == serial + 1
    out16.fill_(float("nan"))
    b.prefill_attention_tc(pb.layer[0], text_k, text_v, nb, d(q), pb.d_prefill, tiles, W, heads, out16, ws, reuse_plan=True)
    assert np.array_equal(out16.float().cpu().numpy(), c)
    with pytest.raises(b.Error):
        b.prefill_attention_tc(pb.layer[0], text_k, text_v, nb, d(q), pb.d_prefill, tiles[:-1], W, heads, out16, ws, reuse_plan=True)
    assert ws.status() == 0


@pytest.mark.parametrize("W,t_max", [(1024, 1536), (4096, 6000)])
def test_prefill_tensor_core_many_items_per_cta_against_cuda_core_path(orc, b, W, t_max):
    # 12 requests with the benchmark's prefix lengths and prompts up to 1.5 windows: ~150 query tiles x 10 heads,
    # i.e. ten items for every persistent CTA, drawn from the counter in longest-first order, with one plan of
    # the tiles shared by two calls.  Too many rows for the scalar oracle; the reference here is the CUDA-core
    # path on the same pools, which the cases above hold to the oracle (its own error is 1e-5).
    # The second case has windows of 4096 and prompts up to 6000: items of up to 42 key tiles.
    import torch
    heads, kvh, hd = 10, 10, 128
    prefixes = [256, 656, 1056, 256, 656, 1056, 1056, 256, 656, 1056, 256, 656]
    text_lens = [int(x) for x in synth.integers(909 + W, 3, 64, t_max, (len(prefixes),))]
    slots = len(prefixes)
    pb = PagedBatch(orc, slots, 1, kvh, hd, W, b.BF16, prefixes, heads=heads, seed=909)
    row = kvh * hd
    pb.write_prefixes()
    d = lambda a: torch.from_numpy(np.ascontiguousarray(a)).cuda()
    nv, nt = sum(prefixes), sum(text_lens)
    ws = b.Workspace(nv + nt)
    # vision rows
    qv = d(synth.normal(909, 41, (nv, heads * hd)))
    rs = d(np.concatenate([np.full(p, s) for s, p in enumerate(prefixes)]).astype(np.int32))
    pos = d(np.concatenate([np.arange(p) for p in prefixes]).astype(np.int32))
    ref_v = torch.full((nv, heads * hd), float("nan"), device="cuda")
    for a in range(0, nv, 4096):
        n = min(4096, nv - a)
        b.attention_ragged_paged(pb.layer[0], qv[a:a + n], pb.d_prefill, rs[a:a + n], pos[a:a + n], n, heads, ref_v[a:a + n], ws)
    # text rows
    block0, nb = [], 0
    for T in text_lens:
        block0.append(nb)
        nb += ceil_div(T, 16)
    text_k = torch.zeros((nb, kvh, 16, hd), dtype=torch.bfloat16, device="cuda")
    text_v = torch.zeros_like(text_k)
    k = d(pb.rnd(synth.normal(909, 51, (nt, row))))
    v = d(pb.rnd(synth.normal(909, 52, (nt, row))))
    qt = d(synth.normal(909, 53, (nt, heads * hd)))
    trs = d(np.concatenate([np.full(T, s) for s, T in enumerate(text_lens)]).astype(np.int32))
    tpos = d(np.concatenate([np.arange(T) for T in text_lens]).astype(np.int32))
    tb0 = d(np.concatenate([np.full(T, block0[s]) for s, T in enumerate(text_lens)]).astype(np.int32))
    ref_t = torch.full((nt, heads * hd), float("nan"), device="cuda")
    for a in range(0, nt, 4096):
        n = min(4096, nt - a)
        b.prefill_text_paged(pb.layer[0], text_k, text_v, nb, qt[a:a + n], k[a:a + n], v[a:a + n], pb.d_prefill, trs[a:a + n],
                             tpos[a:a + n], tb0[a:a + n], n, W, heads, ref_t[a:a + n], ws)
    # tensor-core path: vision and text tiles in ONE call, then once more on the same plan
    reqs, at = [], 0
    for s, p in enumerate(prefixes):
        reqs.append((at, p, s, 0, 0, 0))
        at += p
    for s, T in enumerate(text_lens):
        reqs.append((at, T, s, 1, 0, block0[s]))
        at += T
    tiles = b.make_prefill_tiles(reqs)
    assert tiles.shape[0] * heads >= 8 * 148
    q_all = torch.cat([qv, qt])
    ref = torch.cat([ref_v, ref_t]).cpu().numpy()
    assert np.isfinite(ref).all()
    for reuse in (False, True):
        out = torch.full((nv + nt, heads * hd), float("nan"), device="cuda")
        b.prefill_attention_tc(pb.layer[0], text_k, text_v, nb, q_all, pb.d_prefill, tiles, W, heads, out, ws, reuse_plan=reuse)
        assert_attention_close(out.cpu().numpy(), ref, 4e-4, 2e-4)  # two paths' errors: 1e-5 and 1e-4 against the oracle
    assert ws.status() == 0


def test_prefill_tensor_core_items_without_key_tiles(orc, b):
    # Query tiles of slots whose prefix length is zero on the device: their rows see no key and come out as
    # zeros (the reference's empty attention), also when such an item follows an ordinary one on the same CTA
    # (190 items for 148 CTAs, the empty ones last in the order).
    import torch
    W, heads, kvh, hd = 64, 10, 10, 128
    prefixes = [128] * 16 + [0, 0, 0]
    pb = PagedBatch(orc, len(prefixes), 1, kvh, hd, W, b.BF16, prefixes, heads=heads, seed=515)
    pb.write_prefixes()
    rows_of = [128] * 16 + [16, 128, 1]  # the packed batch claims vision rows for the empty slots too
    n = sum(rows_of)
    q = synth.normal(515, 41, (n, heads * hd))
    out = torch.full((n, heads * hd), float("nan"), device="cuda")
    reqs, at = [], 0
    for s, r in enumerate(rows_of):
        reqs.append((at, r, s, 0, 0, 0))
        at += r
    tiles = b.make_prefill_tiles(reqs)
    assert tiles.shape[0] * heads > 148
    ws = b.Workspace(n)
    b.prefill_attention_tc(pb.layer[0], None, None, 0, torch.from_numpy(q).cuda(), pb.d_prefill, tiles, W, heads, out, ws)
    got = out.cpu().numpy()
    at = 0
    for s, r in enumerate(rows_of):
        if prefixes[s]:
            want = pb.cache[s].attention(0, q[at:at + r], 0, heads, True)
            assert_attention_close(got[at:at + r], want, *TC_TIGHT)
        else:
            assert not got[at:at + r].any()
        at += r
    assert ws.status() == 0


def test_prefill_tensor_core_waits_give_up_cleanly(orc, b):
    # every wait of the tensor-core kernel is bounded: with a poll limit of zero each role gives up at its first
    # wait, the copies already issued are seen to land, the kernel ends (nothing hangs, nothing faults) and the
    # status word says the launch is void; the same workspace and plan then serve a correct launch
    import torch
    W, heads, kvh, hd = 64, 10, 10, 128
    prefixes = [300, 150]
    pb = PagedBatch(orc, len(prefixes), 1, kvh, hd, W, b.BF16, prefixes, heads=heads, seed=717)
    pb.write_prefixes()
    n = sum(prefixes)
    q = synth.normal(717, 41, (n, heads * hd))
    dq = torch.from_numpy(q).cuda()
    tiles = b.make_prefill_tiles([(0, 300, 0, 0, 0, 0), (300, 150, 1, 0, 0, 0)])
    ws = b.Workspace(n)
    out = torch.full((n, heads * hd), float("nan"), device="cuda")
    ws.set_wait_limit(0)
    b.prefill_attention_tc(pb.layer[0], None, None, 0, dq, pb.d_prefill, tiles, W, heads, out, ws)  # void launch
    torch.cuda.synchronize()
    assert ws.status() & b.STATUS_WAIT_TIMEOUT
    ws.set_wait_limit(1 << 22)
    assert ws.status() == 0
    for reuse in (True, False):
        out.fill_(float("nan"))
        b.prefill_attention_tc(pb.layer[0], None, None, 0, dq, pb.d_prefill, tiles, W, heads, out, ws, reuse_plan=reuse)
        got = out.cpu().numpy()
        at = 0
        for s, p_ in enumerate(prefixes):
            want = pb.cache[s].attention(0, q[at:at + p_], 0, heads, True)
            assert_attention_close(got[at:at + p_], want, *TC_TIGHT)
            at += p_
    assert ws.status() == 0
