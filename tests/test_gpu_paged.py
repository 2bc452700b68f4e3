"""GPU parity of the paged path (append, gather, decode attention) against the CPU oracle.

Bookkeeping (cursors, block-table addressing, cache contents through the gather) is bit-exact.
Attention tolerances: bf16 KV max-abs 2e-2 and rel-L2 1e-3 (the stated bar); because the oracle is
fed the bf16-rounded values, the observed error is fp32 reassociation only, so a far tighter bound
(2e-5 / 1e-5) is asserted as well.  fp32 KV: 1e-3 max-abs is the reference's own GPU-vs-CPU bar
(tests/test_rswa_cuda.cu:98); 2e-5 asserted.
"""
import numpy as np
import pytest

import synth
from paged_fixture import PagedBatch, assert_attention_close, load_b200

pytestmark = pytest.mark.gpu

TIGHT = (2e-5, 1e-5)


def tol_for(b, dtype):
    return (2e-2, 1e-3) if dtype == b.BF16 else (1e-3, 1e-3)


@pytest.fixture(scope="module")
def b():
    import torch
    if not torch.cuda.is_available():
        pytest.skip("needs a CUDA device")
    return load_b200()


@pytest.mark.parametrize("dtype_name", ["bf16", "f32"])
@pytest.mark.parametrize("P,W", [(0, 16), (1, 16), (15, 32), (16, 16), (17, 48), (33, 32)])
def test_append_gather_attention_tiny(orc, b, dtype_name, P, W):
    dtype = b.BF16 if dtype_name == "bf16" else b.F32
    slots, layers, kvh, hd = 3, 2, 2, 8
    pb = PagedBatch(orc, slots, layers, kvh, hd, W, dtype, [P, max(P - 1, 0), P], heads=4, seed=P * 100 + W)
    pb.write_prefixes()
    perm = [2, 0, 1]
    for t in range(3 * W + 5):
        for l in range(layers):
            rows = perm if t % 2 else [0, 1, 2]
            if t % 7 == 3:
                rows = rows[:2]  # a smaller batch: one slot lags behind -> mixed warm-up / steady rows
            k, v, q = pb.step_inputs(t, l, rows)
            pb.append(l, k, v, rows)
            if t % 5 == 0 or t >= 3 * W:
                got, want = pb.attend(l, q, rows)
                assert_attention_close(got, want, *tol_for(b, dtype))
                assert_attention_close(got, want, *TIGHT)
        if t in (0, W - 1, W, 2 * W + 1, 3 * W + 4):
            for l in range(layers):
                pb.check_logical_view(l)
    assert pb.ws.status() == 0


@pytest.mark.parametrize("dtype_name", ["bf16", "f32"])
def test_real_geometry_shared_prefix(orc, b, dtype_name):
    # 10 heads x 128, a 273-token prefix (partial last prefix block) shared by 4 of 5 slots
    dtype = b.BF16 if dtype_name == "bf16" else b.F32
    slots, W, P = 5, 48, 273
    pb = PagedBatch(orc, slots, 1, 10, 128, W, dtype, [P, P, P, 40, P],
                    prefix_keys=["doc", "doc", "doc", "other", "doc"], seed=77)
    pb.write_prefixes()
    assert pb.bm.stats()[7] == 2 and pb.bm.counters()[2] == 18 * 256  # refcount 4 -> shared bytes
    rows = [4, 2, 0, 1, 3]
    for t in range(2 * W + 3):
        k, v, q = pb.step_inputs(t, 0, rows)
        pb.append(0, k, v, rows)
        if t in (0, 1, W - 1, W, 2 * W + 2):
            got, want = pb.attend(0, q, rows)
            assert_attention_close(got, want, *tol_for(b, dtype))
            assert_attention_close(got, want, *TIGHT)
            pb.check_logical_view(0)
    # the shared prefix blocks are physically the same blocks in every sharing slot's table
    assert (pb.table_np[0, :18] == pb.table_np[1, :18]).all() and (pb.table_np[0, :18] == pb.table_np[4, :18]).all()
    assert pb.ws.status() == 0


def test_reference_cuda_case_and_cfg1_golden(orc, b):
    # the reference's own decode case (tests/test_rswa_cuda.cu:52-104: P=257, W=128, 50 appends) and the
    # CPU-runnable benchmark configuration (P=256, W=128, 300 steps) against the committed golden vectors
    import os
    from golden.make_golden import CACHE_CASES
    gold = np.load(os.path.join(os.path.dirname(__file__), "golden", "rswa_golden.npz"))
    import synth
    import torch
    for name, dtype in (("ref_cuda_case", b.F32), ("cfg1", b.F32), ("cfg1_bf16", b.BF16)):
        L, kvh, hd, W, P, n, heads, seed, steps, bf16 = CACHE_CASES[name]
        pb = PagedBatch(orc, 1, L, kvh, hd, W, dtype, [P], heads=heads, seed=seed)
        rnd = synth.round_bf16 if bf16 else (lambda x: x)
        row = kvh * hd
        pk = rnd(synth.normal(seed, 10, (P, row)))
        pv = rnd(synth.normal(seed, 20, (P, row)))
        sl = torch.zeros(P, dtype=torch.int32, device="cuda")
        pos = torch.arange(P, dtype=torch.int32, device="cuda")
        b.write_prefill_ragged_paged(pb.layer[0], torch.from_numpy(pk).cuda(), torch.from_numpy(pv).cuda(), sl, pos, P, pb.ws)
        ds = torch.zeros(1, dtype=torch.int32, device="cuda")
        book, outs = [], []
        for t in range(n):
            k = rnd(synth.normal(seed, 1000 + t * 64, (1, row)))
            v = rnd(synth.normal(seed, 500000 + t * 64, (1, row)))
            b.append_decode_batch_paged(pb.layer[0], torch.from_numpy(k).cuda(), torch.from_numpy(v).cuda(),
                                        pb.d_len[0], pb.d_ring[0], pb.d_prefill, ds, 1, W, pb.ws)
            if t in steps:
                q = synth.normal(seed, 900000 + t * 64, (1, heads * hd))
                out = torch.full((1, heads * hd), float("nan"), device="cuda")
                b.attention_batch_paged(pb.layer[0], torch.from_numpy(q).cuda(), pb.d_len[0], pb.d_prefill, ds, 1, heads, out, pb.ws)
                outs.append(out.cpu().numpy()[0])
            if t in (0, W - 1, W, n - 1):
                book.append((t, int(pb.d_len[0, 0]), int(pb.d_ring[0, 0])))
        g_book = gold[f"cache/{name}/book"]
        for t, ln, rp in book:
            assert (ln, rp) == tuple(g_book[t][:2])
        assert_attention_close(np.array(outs), gold[f"cache/{name}/attn"], *(tol_for(b, dtype)))
        assert_attention_close(np.array(outs), gold[f"cache/{name}/attn"], *TIGHT)
        gk, gv = pb.gather(0, [0])
        assert np.array_equal(gk[0].astype(np.float64).sum(-1), gold[f"cache/{name}/keys_rowsum"][0])
        assert np.array_equal(gv[0].astype(np.float64).sum(-1), gold[f"cache/{name}/values_rowsum"][0])
        assert pb.ws.status() == 0
    assert tuple(gold["cache/cfg1/book"][-1][:2]) == (384, 44)


def test_gather_raw_dtype_and_empty_rows(orc, b):
    import torch
    pb = PagedBatch(orc, 2, 1, 2, 16, 16, b.BF16, [5, 0], seed=3)
    pb.write_prefixes()
    # slot 1 has P = 0 and nothing appended: attention must return exact zeros (nothing attended)
    q = np.ones((2, 2 * 16), np.float32)
    got, want = pb.attend(0, q, [0, 1])
    assert not got[1].any() and not want[1].any()
    assert_attention_close(got, want, *TIGHT)
    k, v, _ = pb.step_inputs(0, 0, [0, 1])
    pb.append(0, k, v, [0, 1])
    raw_k, raw_v = pb.gather(0, [1, 0], out_dtype=b.BF16)
    wide_k, wide_v = pb.gather(0, [1, 0], out_dtype=b.F32)
    assert np.array_equal(raw_k, wide_k) and np.array_equal(raw_v, wide_v)
    assert np.array_equal(wide_k[0, :1], pb.cache[1].keys(0))
    # batch of zero rows is a no-op, like the reference wrappers (src/kernels/cuda/rswa_attention.cu:405,493)
    b.append_decode_batch_paged(pb.layer[0], None, None, pb.d_len[0], pb.d_ring[0], pb.d_prefill, None, 0, 16, pb.ws)
    assert pb.ws.status() == 0


def test_errors_are_loud(orc, b):
    import torch
    pb = PagedBatch(orc, 2, 1, 2, 16, 16, b.BF16, [4, 4], seed=5)
    q = torch.zeros((2, 32), device="cuda")
    out = torch.zeros((2, 32), device="cuda")
    ds = torch.tensor([0, 1], dtype=torch.int32, device="cuda")
    small = b.Workspace(1)
    with pytest.raises(b.Error) as e:
        b.attention_batch_paged(pb.layer[0], q, pb.d_len[0], pb.d_prefill, ds, 2, 2, out, small)
    assert e.value.status == 4
    with pytest.raises(b.Error) as e:  # heads not a multiple of kv_heads
        b.attention_batch_paged(pb.layer[0], q, pb.d_len[0], pb.d_prefill, ds, 2, 3, out, pb.ws)
    assert e.value.status == 1
    bad = b.PagedLayer(pb.num_blocks, 2, 24, b.BF16, pb.table)  # head_dim not a power of two
    with pytest.raises(b.Error) as e:
        b.attention_batch_paged(bad, q, pb.d_len[0], pb.d_prefill, ds, 2, 2, out, pb.ws)
    assert e.value.status == 2
    # a block id outside the pool is recorded in the status word, not dereferenced
    tbl = pb.table.clone()
    tbl[0, 0] = pb.num_blocks + 5
    poisoned = b.PagedLayer(pb.num_blocks, 2, 16, b.BF16, tbl)
    b.attention_batch_paged(poisoned, q, pb.d_len[0], pb.d_prefill, ds, 2, 2, out, pb.ws)
    assert pb.ws.status() & b.STATUS_BAD_BLOCK
    assert pb.ws.status() == 0  # reading clears it


def test_graph_replay_across_ring_boundary(orc, b):
    # one captured (append + attention) step replayed across warm-up -> ring equals the plain run bit
    # for bit (the reference's bar for its graph path, tests/test_rswa_cuda.cu:848-927)
    import torch
    slots, W, P, kvh, hd = 3, 16, 9, 2, 32
    runs = []
    for use_graph in (False, True):
        pb = PagedBatch(orc, slots, 1, kvh, hd, W, b.BF16, [P] * slots, seed=9)
        pb.write_prefixes()
        k = torch.zeros((slots, kvh * hd), device="cuda")
        v = torch.zeros_like(k)
        q = torch.zeros_like(k)
        out = torch.zeros_like(k)
        ds = torch.tensor([1, 2, 0], dtype=torch.int32, device="cuda")

        def step():
            b.append_decode_batch_paged(pb.layer[0], k, v, pb.d_len[0], pb.d_ring[0], pb.d_prefill, ds, slots, W, pb.ws)
            b.attention_batch_paged(pb.layer[0], q, pb.d_len[0], pb.d_prefill, ds, slots, kvh, out, pb.ws)

        graph = None
        if use_graph:
            side = torch.cuda.Stream()
            side.wait_stream(torch.cuda.current_stream())
            with torch.cuda.stream(side):
                k.zero_(); v.zero_(); q.zero_()
            torch.cuda.current_stream().wait_stream(side)
            torch.cuda.synchronize()
            len0, ring0 = pb.d_len.clone(), pb.d_ring.clone()
            kpool0, vpool0 = pb.layer[0].k.clone(), pb.layer[0].v.clone()
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph):
                step()
            # capture does not execute, but restore state anyway so both runs start identically
            pb.d_len.copy_(len0); pb.d_ring.copy_(ring0)
            pb.layer[0].k.copy_(kpool0); pb.layer[0].v.copy_(vpool0)
        outs = []
        for t in range(2 * W + 3):
            kk, vv, qq = pb.step_inputs(t, 0, [0, 1, 2])
            k.copy_(torch.from_numpy(kk)); v.copy_(torch.from_numpy(vv)); q.copy_(torch.from_numpy(qq))
            if graph is not None:
                graph.replay()
            else:
                step()
            outs.append(out.cpu().numpy().copy())
        runs.append((np.array(outs), pb.d_len.cpu().numpy(), pb.d_ring.cpu().numpy(),
                     pb.layer[0].k.float().cpu().numpy(), pb.layer[0].v.float().cpu().numpy()))
        assert pb.ws.status() == 0
    for a, c in zip(*runs):
        assert np.array_equal(a, c)
    assert runs[0][1].max() == P + W


@pytest.mark.parametrize("dtype_name", ["bf16", "f32"])
@pytest.mark.parametrize("P,W", [(0, 16), (15, 32), (17, 48), (33, 32)])
def test_fused_decode_step_tiny(orc, b, dtype_name, P, W):
    # append + attention in ONE launch: outputs, cursors and pool contents equal the oracle at every step
    dtype = b.BF16 if dtype_name == "bf16" else b.F32
    slots, layers, kvh, hd = 3, 2, 2, 8
    pb = PagedBatch(orc, slots, layers, kvh, hd, W, dtype, [P, max(P - 1, 0), P], heads=4, seed=P * 100 + W + 1)
    pb.write_prefixes()
    perm = [2, 0, 1]
    for t in range(3 * W + 5):
        for l in range(layers):
            rows = perm if t % 2 else [0, 1, 2]
            if t % 7 == 3:
                rows = rows[:2]
            k, v, q = pb.step_inputs(t, l, rows)
            got, want = pb.step_fused(l, k, v, q, rows)
            assert_attention_close(got, want, *tol_for(b, dtype))
            assert_attention_close(got, want, *TIGHT)
        if t in (0, 1, W - 1, W, 2 * W + 1, 3 * W + 4):
            for l in range(layers):
                pb.check_logical_view(l)
    assert pb.ws.status() == 0


def test_fused_decode_step_real_geometry_and_mixed_calls(orc, b):
    # real head geometry, shared prefix with a partial last block, GQA off; fused and separate calls
    # interleaved on the same state must agree with the oracle throughout
    slots, W, P = 5, 48, 273
    pb = PagedBatch(orc, slots, 1, 10, 128, W, b.BF16, [P, P, P, 40, P],
                    prefix_keys=["doc", "doc", "doc", "other", "doc"], seed=78)
    pb.write_prefixes()
    rows = [4, 2, 0, 1, 3]
    for t in range(2 * W + 3):
        k, v, q = pb.step_inputs(t, 0, rows)
        if t % 3 == 2:
            pb.append(0, k, v, rows)
            got, want = pb.attend(0, q, rows)
        else:
            got, want = pb.step_fused(0, k, v, q, rows)
        assert_attention_close(got, want, *TIGHT)
        if t in (0, 1, W - 1, W, 2 * W + 2):
            pb.check_logical_view(0)
    assert pb.ws.status() == 0


@pytest.mark.parametrize("dtype_name,hd,kvh,heads", [("bf16", 256, 2, 2), ("f32", 256, 1, 4), ("bf16", 64, 2, 8),
                                                      ("f32", 64, 4, 4), ("bf16", 32, 1, 2)])
def test_head_dims_of_the_reference_dispatch_and_grouped_heads(orc, b, dtype_name, hd, kvh, heads):
    # the reference instantiates its kernels for head_dim 64 / 128 / 256 (rswa_attention.cu:348-359) and maps
    # query head h to kv head h / (heads / kv_heads): fused and separate calls, across the ring wrap
    dtype = b.BF16 if dtype_name == "bf16" else b.F32
    slots, W, P = 5, 32, 21
    pb = PagedBatch(orc, slots, 1, kvh, hd, W, dtype, [P, P, 7, P, 0], prefix_keys=["a", "a", "b", "a", "c"],
                    heads=heads, seed=hd + kvh)
    pb.write_prefixes()
    rows = [3, 0, 4, 1, 2]
    for t in range(2 * W + 3):
        k, v, q = pb.step_inputs(t, 0, rows)
        if t % 4 == 1:
            pb.append(0, k, v, rows)
            got, want = pb.attend(0, q, rows)
        else:
            got, want = pb.step_fused(0, k, v, q, rows)
        assert_attention_close(got, want, *tol_for(b, dtype))
        assert_attention_close(got, want, *TIGHT)
    pb.check_logical_view(0)
    assert pb.ws.status() == 0


def test_fused_decode_step_stores_into_pinned_host_output(orc, b):
    # `out` may be any device-accessible address: pinned host memory receives the same values, from
    # rows written directly by one warp and from rows merged out of partials alike
    slots, W, P = 6, 64, 273
    pb = PagedBatch(orc, slots, 1, 10, 128, W, b.BF16, [P] * slots, prefix_keys=["doc"] * slots, seed=79)
    pb.write_prefixes()
    rows = [5, 3, 1, 0, 2, 4]
    for t in range(W + 4):
        k, v, q = pb.step_inputs(t, 0, rows)
        got, want = pb.step_fused(0, k, v, q, rows, host_out=(t % 2 == 0))
        assert_attention_close(got, want, *TIGHT)
    pb.check_logical_view(0)
    assert pb.ws.status() == 0


@pytest.mark.parametrize("slots,P,W", [(24, 1600, 64), (5, 273, 48)])
def test_long_shared_prefix_many_units_per_warp(orc, b, slots, P, W):
    # the large case gives every warp of the persistent grid ten units (24 rows x 10 heads x 101 tiles over
    # 2368 warps), nearly all of them tiles of one shared prefix; the small one leaves most warps without a
    # piece.  Fused and separate calls, rows in reverse slot order.
    pb = PagedBatch(orc, slots, 1, 10, 128, W, b.BF16, [P] * slots, prefix_keys=["doc"] * slots, seed=91)
    pb.write_prefixes()
    rows = list(range(slots))[::-1]
    for t in range(5):
        k, v, q = pb.step_inputs(t, 0, rows)
        if t == 3:
            pb.append(0, k, v, rows)
            got, want = pb.attend(0, q, rows)
        else:
            got, want = pb.step_fused(0, k, v, q, rows)
        assert_attention_close(got, want, *TIGHT)
    pb.check_logical_view(0)
    assert pb.ws.status() == 0


@pytest.mark.parametrize("dtype_name,hd,theta", [("bf16", 128, 10000.0), ("f32", 16, 10000.0), ("bf16", 16, 1e6)])
def test_fused_decode_step_with_rope(orc, b, dtype_name, hd, theta):
    # rope + append + attention in one launch against the oracle's rope (restating the reference's CPU
    # rope) followed by append_decode and attention.  The device evaluates sin/cos with its own libm, so
    # a rotated k can land on the other side of a bf16 rounding boundary: K is compared to one bf16 ulp
    # on a handful of elements, everything else (V, cursors) bit for bit.
    import torch
    dtype = b.BF16 if dtype_name == "bf16" else b.F32
    slots, W, P, kvh, heads = 4, 32, 17, 2, 4
    pb = PagedBatch(orc, slots, 1, kvh, hd, W, dtype, [P] * slots, heads=heads, seed=55)
    pb.write_prefixes()
    rows = [2, 0, 3, 1]
    ds = torch.tensor(rows, dtype=torch.int32, device="cuda")
    worst = (0.0, 0.0)
    for t in range(2 * W + 3):
        k = np.ascontiguousarray(synth.normal(55, 100000 + t, (slots, kvh * hd)))
        v = np.ascontiguousarray(pb.rnd(synth.normal(55, 300000 + t, (slots, kvh * hd))))
        q = np.ascontiguousarray(synth.normal(55, 500000 + t, (slots, heads * hd)))
        pos = np.array([P + t + 977 * i for i in range(slots)], dtype=np.int32)  # up to ~3000: many turns of the fast pairs
        out = torch.full((slots, heads * hd), float("nan"), device="cuda")
        b.decode_step_rope_paged(pb.layer[0], torch.from_numpy(q).cuda(), torch.from_numpy(k).cuda(),
                                 torch.from_numpy(v).cuda(), torch.from_numpy(pos).cuda(), theta, pb.d_len[0], pb.d_ring[0],
                                 pb.d_prefill, ds, slots, W, heads, out, pb.ws)
        got = out.cpu().numpy()
        q_rot, k_rot = orc.apply_rope(q, k, pos, heads, kvh, hd, theta)
        k_rot = np.ascontiguousarray(pb.rnd(k_rot))
        want = []
        for i, s in enumerate(rows):
            pb.cache[s].append_decode(0, k_rot[i], v[i])
            want.append(pb.cache[s].attention(0, q_rot[i:i + 1], pb.cache[s].len(0) - 1, heads, False)[0])
        e = assert_attention_close(got, np.stack(want), *TIGHT)
        worst = (max(worst[0], e[0]), max(worst[1], e[1]))
    print("rope step worst max-abs / rel-L2:", worst)
    gk, gv = pb.gather(0, list(range(slots)))
    dl, dr = pb.d_len[0].cpu().numpy(), pb.d_ring[0].cpu().numpy()
    for s in range(slots):
        c = pb.cache[s]
        n = c.len(0)
        assert dl[s] == n and dr[s] == c.ring_pos(0)
        assert np.array_equal(gv[s, :n], c.values(0))
        wk = c.keys(0)
        diff = np.abs(gk[s, :n] - wk)
        ulp = np.abs(wk) * 2.0 ** -7 + 1e-30 if dtype_name == "bf16" else np.abs(wk) * 2.0 ** -20 + 1e-6
        assert (diff <= ulp).all(), "rotated K off by more than one ulp of the pool dtype"
        if dtype_name == "bf16":
            assert (diff > 0).mean() < 5e-3, "too many rotated K elements rounded differently"
    assert pb.ws.status() == 0


def test_bf16_attention_output(orc, b):
    # workspace option: results written as bf16 (RNE) for the o-projection.  Separate and fused calls, an
    # item merged from several partials (long rows) and rows written directly; against RNE(oracle).
    import torch
    slots, W, P, kvh, hd = 6, 64, 600, 10, 128
    pb = PagedBatch(orc, slots, 1, kvh, hd, W, b.BF16, [P, P, 40, P, 0, P], prefix_keys=["d", "d", "e", "d", "f", "d"], seed=23)
    pb.write_prefixes()
    pb.ws.set_out_dtype(b.BF16)
    rows = [5, 1, 4, 0, 2, 3]
    ds = torch.tensor(rows, dtype=torch.int32, device="cuda")
    for t in range(4):
        k, v, q = pb.step_inputs(t, 0, rows)
        out = torch.full((slots, kvh * hd), float("nan"), dtype=torch.bfloat16, device="cuda")
        dq = torch.from_numpy(q).cuda()
        if t % 2:
            pb.append(0, k, v, rows)
            b.attention_batch_paged(pb.layer[0], dq, pb.d_len[0], pb.d_prefill, ds, slots, kvh, out, pb.ws)
        else:
            b.decode_step_paged(pb.layer[0], dq, torch.from_numpy(k).cuda(), torch.from_numpy(v).cuda(), pb.d_len[0],
                                pb.d_ring[0], pb.d_prefill, ds, slots, W, kvh, out, pb.ws)
            for i, s in enumerate(rows):
                pb.cache[s].append_decode(0, k[i], v[i])
        got = out.float().cpu().numpy()
        want = np.stack([pb.cache[s].attention(0, q[i:i + 1], pb.cache[s].len(0) - 1, kvh, False)[0]
                         for i, s in enumerate(rows)])
        assert np.isfinite(got).all()
        exact = got == synth.round_bf16(want)
        assert exact.mean() > 0.99                                       # fp32 reassociation flips a rounding now and then
        # never more than half a bf16 ulp (<= |x| / 256) off, plus the fp32 difference that caused a flip
        assert (np.abs(got - want) <= np.abs(want) * 2.0 ** -8 + 2e-6).all()
    pb.ws.set_out_dtype(b.F32)
    k, v, q = pb.step_inputs(9, 0, rows)
    got, want = pb.step_fused(0, k, v, q, rows)
    assert_attention_close(got, want, *TIGHT)
    assert pb.ws.status() == 0


@pytest.mark.parametrize("slots,layers", [(12, 4), (2, 3)])
def test_fused_decode_step_overlapped_launches(orc, b, slots, layers):
    # the step of every layer queued back to back with launch overlap enabled (each kernel may become
    # resident while its predecessor drains): outputs, pool contents and cursors still equal the oracle.
    # The two-slot case leaves most CTAs without a unit (they plan, draw their ticket and leave at once, so
    # CTAs of the next launch move in early) and has an odd number of launches per step.
    import torch
    W, P, kvh, hd = 80, 273, 10, 128
    pb = PagedBatch(orc, slots, layers, kvh, hd, W, b.BF16, [P] * slots, prefix_keys=["doc"] * slots, seed=83)
    pb.write_prefixes()
    pb.ws.set_overlap(True)
    rows = [7, 3, 11, 0, 5, 9, 1, 10, 2, 8, 4, 6] if slots == 12 else [1, 0]
    ds = torch.tensor(rows, dtype=torch.int32, device="cuda")
    for t in range(W + 6):
        ins = [pb.step_inputs(t, l, rows) for l in range(layers)]
        dev = [[torch.from_numpy(x).cuda() for x in kvq] for kvq in ins]
        outs = [torch.full((slots, kvh * hd), float("nan"), device="cuda") for _ in range(layers)]
        torch.cuda.synchronize()
        for l in range(layers):  # no host synchronisation between the launches
            dk, dv, dq = dev[l]
            b.decode_step_paged(pb.layer[l], dq, dk, dv, pb.d_len[l], pb.d_ring[l], pb.d_prefill, ds, slots, W,
                                kvh, outs[l], pb.ws)
        torch.cuda.synchronize()
        check = t in (0, 1, W - 1, W, W + 5) or t % 9 == 0
        for l in range(layers):
            k, v, q = ins[l]
            want = []
            for i, s in enumerate(rows):
                pb.cache[s].append_decode(l, k[i], v[i])
                if check:
                    want.append(pb.cache[s].attention(l, q[i:i + 1], pb.cache[s].len(l) - 1, kvh, False)[0])
            if check:
                assert_attention_close(outs[l].cpu().numpy(), np.stack(want), *TIGHT)
    for l in range(layers):
        pb.check_logical_view(l)
    assert pb.ws.status() == 0


def test_fused_decode_step_overlapped_launches_full_grid(orc, b):
    # enough units that every warp of every CTA holds a piece: the overlapped launch then trims the share
    # of its last CTA (the one that starts late); results must not depend on how the line is cut
    import torch
    slots, layers, W, P, kvh, hd = 64, 2, 32, 512, 10, 128
    pb = PagedBatch(orc, slots, layers, kvh, hd, W, b.BF16, [P] * slots, prefix_keys=["doc"] * slots, seed=84)
    pb.write_prefixes()
    pb.ws.set_overlap(True)
    rows = list(range(slots))[::-1]
    ds = torch.tensor(rows, dtype=torch.int32, device="cuda")
    for t in range(W + 3):
        ins = [pb.step_inputs(t, l, rows) for l in range(layers)]
        dev = [[torch.from_numpy(x).cuda() for x in kvq] for kvq in ins]
        outs = [torch.full((slots, kvh * hd), float("nan"), device="cuda") for _ in range(layers)]
        torch.cuda.synchronize()
        for l in range(layers):
            dk, dv, dq = dev[l]
            b.decode_step_paged(pb.layer[l], dq, dk, dv, pb.d_len[l], pb.d_ring[l], pb.d_prefill, ds, slots, W,
                                kvh, outs[l], pb.ws)
        torch.cuda.synchronize()
        check = t in (0, W - 1, W, W + 2)
        for l in range(layers):
            k, v, q = ins[l]
            want = []
            for i, s in enumerate(rows):
                pb.cache[s].append_decode(l, k[i], v[i])
                if check:
                    want.append(pb.cache[s].attention(l, q[i:i + 1], pb.cache[s].len(l) - 1, kvh, False)[0])
            if check:
                assert_attention_close(outs[l].cpu().numpy(), np.stack(want), *TIGHT)
    for l in range(layers):
        pb.check_logical_view(l)
    assert pb.ws.status() == 0


def test_fused_step_graph_replay(orc, b):
    import torch
    slots, W, P, kvh, hd = 4, 16, 9, 2, 64
    pb = PagedBatch(orc, slots, 1, kvh, hd, W, b.BF16, [P] * slots, prefix_keys=["d"] * slots, seed=19)
    pb.write_prefixes()
    k = torch.zeros((slots, kvh * hd), device="cuda")
    v, q, out = torch.zeros_like(k), torch.zeros_like(k), torch.zeros_like(k)
    ds = torch.tensor([1, 2, 0, 3], dtype=torch.int32, device="cuda")

    def step():
        b.decode_step_paged(pb.layer[0], q, k, v, pb.d_len[0], pb.d_ring[0], pb.d_prefill, ds, slots, W, kvh, out, pb.ws)

    step()  # warm-up outside capture (zeros appended to every slot; mirrored in the oracle below)
    for s in range(slots):
        pb.cache[s].append_decode(0, np.zeros(kvh * hd, np.float32), np.zeros(kvh * hd, np.float32))
    torch.cuda.synchronize()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        step()
    for t in range(2 * W + 3):
        kk, vv, qq = pb.step_inputs(t, 0, [0, 1, 2, 3])
        k.copy_(torch.from_numpy(kk)); v.copy_(torch.from_numpy(vv)); q.copy_(torch.from_numpy(qq))
        graph.replay()
        got = out.cpu().numpy()
        want = []
        for i, s in enumerate([1, 2, 0, 3]):
            pb.cache[s].append_decode(0, kk[i], vv[i])
            want.append(pb.cache[s].attention(0, qq[i:i + 1], pb.cache[s].len(0) - 1, kvh, False)[0])
        assert_attention_close(got, np.stack(want), *TIGHT)
    pb.check_logical_view(0)
    assert pb.ws.status() == 0


def test_wait_that_runs_out_is_reported_and_the_workspace_recovers(orc, b):
    # With the poll limit at zero every tile wait gives up at once: each warp records the fact, lets the
    # copies it has in flight land and leaves; the kernel ends normally (nothing hangs, nothing faults),
    # the status word says the launch is void, and after the status call the same workspace serves the
    # next launch correctly.  Long rows so that items are split over several warps and partials are in play.
    slots, W, P = 12, 96, 400
    pb = PagedBatch(orc, slots, 1, 10, 128, W, b.BF16, [P] * slots, prefix_keys=["doc"] * slots, seed=61)
    pb.write_prefixes()
    rows = list(range(slots))
    for t in range(W + 5):
        k, v, q = pb.step_inputs(t, 0, rows)
        pb.append(0, k, v, rows)
    got, want = pb.attend(0, q, rows)
    assert_attention_close(got, want, *TIGHT)
    pb.ws.set_wait_limit(0)
    pb.attend(0, q, rows)  # void launch
    assert pb.ws.status() & b.STATUS_WAIT_TIMEOUT
    pb.ws.set_wait_limit(1 << 22)
    assert pb.ws.status() == 0
    for _ in range(2):
        got, want = pb.attend(0, q, rows)
        assert_attention_close(got, want, *TIGHT)
    k, v, q = pb.step_inputs(W + 5, 0, rows)
    got, want = pb.step_fused(0, k, v, q, rows)
    assert_attention_close(got, want, *TIGHT)
    pb.check_logical_view(0)
    assert pb.ws.status() == 0


@pytest.mark.parametrize("dtype_name", ["bf16", "f32"])
def test_all_layer_append_and_gather_equal_the_per_layer_calls(orc, b, dtype_name):
    # one launch for every layer of an append step / of a gather: same cursors, same pool contents, same
    # views as one call per layer, and as the oracle; steps alternate between the two forms, rows permuted,
    # one slot lagging, across the ring wrap
    import torch
    dtype = b.BF16 if dtype_name == "bf16" else b.F32
    slots, L, W, kvh, hd = 5, 3, 32, 2, 32
    P = [21, 21, 7, 0, 16]
    pb = PagedBatch(orc, slots, L, kvh, hd, W, dtype, P, prefix_keys=["a", "a", "b", "c", "d"], seed=314)
    pb.write_prefixes()
    for t in range(2 * W + 5):
        rows = [3, 0, 4, 1, 2] if t % 3 else [0, 1, 2, 4]
        kv = [pb.step_inputs(t, l, rows) for l in range(L)]
        if t % 2:
            k = torch.from_numpy(np.stack([x[0] for x in kv])).cuda()
            v = torch.from_numpy(np.stack([x[1] for x in kv])).cuda()
            ds = torch.tensor(rows, dtype=torch.int32, device="cuda")
            b.append_decode_batch_paged_layers(pb.layer, k, v, pb.d_len, pb.d_ring, pb.d_prefill, ds, len(rows), W, pb.ws)
            for l in range(L):
                for i, s in enumerate(rows):
                    pb.cache[s].append_decode(l, kv[l][0][i], kv[l][1][i])
        else:
            for l in range(L):
                pb.append(l, kv[l][0], kv[l][1], rows)
    for l in range(L):
        pb.check_logical_view(l)
    cap = max(P) + W
    ds = torch.tensor([4, 2, 0], dtype=torch.int32, device="cuda")
    for out_dtype, tdt in ((b.F32, torch.float32), (dtype, torch.bfloat16 if dtype == b.BF16 else torch.float32)):
        ak = torch.full((L, 3, cap, pb.row), float("nan"), dtype=tdt, device="cuda")
        av = torch.full_like(ak, float("nan"))
        b.gather_paged_layers(pb.layer, pb.d_len, pb.d_prefill, ds, 3, cap, ak, av, out_dtype, pb.ws)
        for l in range(L):
            ok = torch.full((3, cap, pb.row), float("nan"), dtype=tdt, device="cuda")
            ov = torch.full_like(ok, float("nan"))
            b.gather_paged(pb.layer[l], pb.d_len[l], pb.d_prefill, ds, 3, cap, ok, ov, out_dtype, pb.ws)
            assert torch.equal(ak[l], ok) and torch.equal(av[l], ov)
    with pytest.raises(b.Error):  # layers behind different block tables cannot share a launch
        other = b.PagedLayer(pb.num_blocks, kvh, hd, dtype, pb.table.clone())
        b.gather_paged_layers([pb.layer[0], other], pb.d_len, pb.d_prefill, ds, 3, cap, ak, av, b.F32, pb.ws)
    assert pb.ws.status() == 0


def test_stream_read_rate_and_slot_publication(orc, b):
    # the library's own read-only streaming measurement returns a plausible HBM rate, and the packed slot
    # publication writes exactly the rows and cursors its records name (and flags a slot out of range)
    import ctypes as C
    import torch
    ws = b.Workspace(64)
    gbs = ws.stream_read_gbs()
    assert 1000.0 < gbs < 20000.0
    slots, layers, stride = 6, 3, 5
    table = torch.full((slots, stride), 7, dtype=torch.int32, device="cuda")
    d_len = torch.full((layers, slots), 9, dtype=torch.int32, device="cuda")
    d_ring = torch.full((layers, slots), 9, dtype=torch.int32, device="cuda")
    d_prefill = torch.full((slots,), 9, dtype=torch.int32, device="cuda")
    rec = np.array([[4, 33, 1, 10, 11, 12, -1, -1],     # slot 4: length 33, row written
                    [1, 5, 0, 99, 99, 99, 99, 99],       # slot 1: cursors only, row untouched
                    [2, 0, 1, -1, -1, -1, -1, -1]],      # slot 2: retired
                   dtype=np.int32)
    d_rec = torch.from_numpy(rec).cuda()
    b.check(b.lib().uocr_b200_rswa_publish_slots(d_rec.data_ptr(), 3, table.data_ptr(), stride, d_len.data_ptr(),
                                                 d_ring.data_ptr(), d_prefill.data_ptr(), slots, layers, ws.h,
                                                 b.stream_handle()))
    t, ln, rg, pf = (x.cpu().numpy() for x in (table, d_len, d_ring, d_prefill))
    assert t[4].tolist() == [10, 11, 12, -1, -1] and t[1].tolist() == [7] * 5 and t[2].tolist() == [-1] * 5
    assert (ln[:, 4] == 33).all() and (ln[:, 1] == 5).all() and (ln[:, 2] == 0).all() and (ln[:, [0, 3, 5]] == 9).all()
    assert (rg[:, [4, 1, 2]] == 0).all() and (rg[:, [0, 3, 5]] == 9).all()
    assert pf.tolist() == [9, 5, 0, 9, 33, 9]
    assert ws.status() == 0
    bad = torch.tensor([[slots, 1, 0, 0, 0, 0, 0, 0]], dtype=torch.int32, device="cuda")
    b.check(b.lib().uocr_b200_rswa_publish_slots(bad.data_ptr(), 1, table.data_ptr(), stride, d_len.data_ptr(),
                                                 d_ring.data_ptr(), d_prefill.data_ptr(), slots, layers, ws.h,
                                                 b.stream_handle()))
    assert ws.status() & b.STATUS_BAD_SLOT
