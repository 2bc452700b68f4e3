"""GPU parity at the sizes the benchmark numbers are quoted on, against the CPU oracle.

* the batched-decode configuration itself: 64 sequences, one shared 256-token prefix, W = 1024, the
  benchmark's own seeded positions (uniform in [1, 4096]); cursors reached through the append state
  machine on both sides, then fused decode steps with and without launch overlap -- the split / merge
  geometry (tens of thousands of units over every warp of the grid) of the timed launches;
* a sample of the 8-GPU configuration: 8 sequences at W = 4096 behind the 1456-token prefix;
* the ragged-prefill configuration's shapes on the tensor-core path: a 1056-token vision prefix with
  text prompts of 2048 and 1200 tokens at W = 1024 (window tiles that start several 128-key tiles into
  the prompt, nine-tile windows), plus a small case whose later query tiles start beyond the window.

One layer each (layers are independent replicas of the same launch).  Bookkeeping bit-exact, attention
within max-abs 2e-2 / rel-L2 1e-3 (bf16 KV) and within the observed fp32-reassociation bound as well.
"""
import numpy as np
import pytest

import synth
from paged_fixture import PagedBatch, assert_attention_close, ceil_div, load_b200
from test_gpu_prefill import TC_TIGHT, run_prefill_case

pytestmark = pytest.mark.gpu
BAR = (2e-2, 1e-3)
TIGHT = (2e-5, 1e-5)
POOL_ROWS = 4099  # prime: (slot * 1031 + step) % 4099 gives every slot of a window a distinct row


@pytest.fixture(scope="module")
def b():
    import torch
    if not torch.cuda.is_available():
        pytest.skip("needs a CUDA device")
    return load_b200()


def appends_to_reach(pos, W):
    """Fewest appends that leave the cursors where `pos` appends leave them (len, ring_pos depend on pos
    only through min(pos, W) and (pos - W) mod W)."""
    pos = np.asarray(pos, np.int64)
    return np.where(pos < W, pos, W + (pos - W) % W)


def fill_to_positions(pb, layer, pos, seed):
    """Drives every slot's ring to the state `pos[s]` appends leave, through the batched append on the
    device and append_decode on the oracle, with the same bf16-rounded rows on both sides."""
    import torch
    n_app = appends_to_reach(pos, pb.W)
    pool_k = pb.rnd(synth.normal(seed, 11, (POOL_ROWS, pb.row)))
    pool_v = pb.rnd(synth.normal(seed, 12, (POOL_ROWS, pb.row)))
    dpk, dpv = torch.from_numpy(pool_k).cuda(), torch.from_numpy(pool_v).cuda()
    for t in range(int(n_app.max())):
        rows = np.nonzero(n_app > t)[0]
        idx = (rows * 1031 + t) % POOL_ROWS
        di = torch.from_numpy(idx).cuda()
        ds = torch.from_numpy(rows.astype(np.int32)).cuda()
        pb.b.append_decode_batch_paged(pb.layer[layer], dpk[di].contiguous(), dpv[di].contiguous(), pb.d_len[layer],
                                       pb.d_ring[layer], pb.d_prefill, ds, len(rows), pb.W, pb.ws)
        for s, i in zip(rows, idx):
            pb.cache[s].append_decode(layer, pool_k[i], pool_v[i])
    return n_app


def fused_steps_against_oracle(pb, rows, n_steps, t0):
    worst = (0.0, 0.0)
    for t in range(t0, t0 + n_steps):
        k, v, q = pb.step_inputs(t, 0, rows)
        got, want = pb.step_fused(0, k, v, q, rows)
        assert_attention_close(got, want, *BAR)
        e = assert_attention_close(got, want, *TIGHT)
        worst = (max(worst[0], e[0]), max(worst[1], e[1]))
    return worst


def test_decode_benchmark_state_64_sequences_w1024(orc, b):
    slots, W, P = 64, 1024, 256
    pos = synth.integers(1234, 77, 1, 4096, (slots,)).astype(np.int64)  # the benchmark's draw for rank 0
    pb = PagedBatch(orc, slots, 1, 10, 128, W, b.BF16, [P] * slots, prefix_keys=["doc"] * slots, seed=1234)
    assert pb.bm.stats()[7] == 1 and (pb.table_np[:, :16] == pb.table_np[0, :16]).all()  # one prefix, refcount 64
    pb.write_prefixes()
    fill_to_positions(pb, 0, pos, 1234)
    dl, dr = pb.d_len[0].cpu().numpy(), pb.d_ring[0].cpu().numpy()
    assert np.array_equal(dl, P + np.minimum(pos, W))                       # closed form of the state machine
    assert np.array_equal(dr, np.where(pos < W, 0, (pos - W) % W))
    rows = list(range(slots))
    worst_plain = fused_steps_against_oracle(pb, rows, 3, 0)
    pb.ws.set_overlap(True)
    worst_overlap = fused_steps_against_oracle(pb, rows, 3, 3)
    pb.ws.set_overlap(False)
    # separate entry points on the same state, rows permuted
    perm = rows[::-1]
    k, v, q = pb.step_inputs(9, 0, perm)
    pb.append(0, k, v, perm)
    got, want = pb.attend(0, q, perm)
    assert_attention_close(got, want, *TIGHT)
    pb.check_logical_view(0)  # gathered contents and cursors of all 64 sequences, bit for bit
    assert pb.ws.status() == 0
    print("cfg2 state: worst max-abs / rel-L2 without overlap", worst_plain, "with overlap", worst_overlap)


def test_eight_gpu_configuration_sample_w4096(orc, b):
    slots, W, P = 8, 4096, 1456
    pos = synth.integers(1234, 77, 1, 16384, (512,)).astype(np.int64)[:slots]  # first sequences of the job's draw
    pb = PagedBatch(orc, slots, 1, 10, 128, W, b.BF16, [P] * slots, prefix_keys=["doc1456"] * slots, seed=4321)
    pb.write_prefixes()
    fill_to_positions(pb, 0, pos, 4321)
    rows = [3, 7, 0, 5, 1, 6, 2, 4]
    worst = fused_steps_against_oracle(pb, rows, 2, 0)
    pb.ws.set_overlap(True)
    worst2 = fused_steps_against_oracle(pb, rows, 2, 2)
    pb.check_logical_view(0)
    assert pb.ws.status() == 0
    print("cfg4 sample: worst max-abs / rel-L2", worst, worst2)


def sampled_positions(n, every=16):
    s = set(range(0, n, every)) | set(range(min(n, 40))) | set(range(max(n - 40, 0), n))
    for a in range(0, n, 128):  # both sides of every 128-row query-tile boundary
        s |= {x for x in (a - 1, a, a + 1) if 0 <= x < n}
    return sorted(s)


def test_ragged_prefill_configuration_shapes_tensor_cores(orc, b):
    # Pv = 1056 (a 256-token global view + 8 crops), T = 2048 and 1200, W = 1024: through the fused text
    # scatter + ring fill and the tcgen05 attention.  Every text token is appended to the oracle in order;
    # its attention is compared on a sample of positions (every 16th, the ends, both sides of every query
    # tile boundary) to keep the scalar oracle to seconds.
    import torch
    W, heads, kvh, hd = 1024, 10, 10, 128
    prefixes, text_lens = [1056, 1056], [2048, 1200]
    slots = len(prefixes)
    pb = PagedBatch(orc, slots, 1, kvh, hd, W, b.BF16, prefixes, heads=heads, seed=303)
    row = kvh * hd
    pb.write_prefixes()
    d = lambda a: torch.from_numpy(np.ascontiguousarray(a)).cuda()
    ws = b.Workspace(sum(prefixes) + sum(text_lens))
    # ---- vision rows, causal over the prefix ----
    nv = sum(prefixes)
    qv = synth.normal(303, 41, (nv, heads * hd))
    out = torch.full((nv, heads * hd), float("nan"), device="cuda")
    reqs, at = [], 0
    for s in range(slots):
        reqs.append((at, prefixes[s], s, 0, 0, 0))
        at += prefixes[s]
    b.prefill_attention_tc(pb.layer[0], None, None, 0, d(qv), pb.d_prefill, b.make_prefill_tiles(reqs), W, heads, out, ws)
    got = out.cpu().numpy()
    at = 0
    worst_v = (0.0, 0.0)
    for s in range(slots):
        idx = sampled_positions(prefixes[s], every=32)
        want = np.stack([pb.cache[s].attention(0, qv[at + i:at + i + 1], i, heads, True)[0] for i in idx])
        assert_attention_close(got[at + np.array(idx)], want, *BAR)
        e = assert_attention_close(got[at + np.array(idx)], want, *TC_TIGHT)
        worst_v = (max(worst_v[0], e[0]), max(worst_v[1], e[1]))
        at += prefixes[s]
    # ---- text rows: scatter + ring fill + cursors in one kernel, then the attention ----
    total = sum(text_lens)
    block0, nb = [], 0
    for T in text_lens:
        block0.append(nb)
        nb += ceil_div(T, 16)
    text_k = torch.zeros((nb, kvh, 16, hd), dtype=torch.bfloat16, device="cuda")
    text_v = torch.zeros_like(text_k)
    k = pb.rnd(synth.normal(303, 51, (total, row)))
    v = pb.rnd(synth.normal(303, 52, (total, row)))
    q = synth.normal(303, 53, (total, heads * hd))
    rs = np.concatenate([np.full(T, s) for s, T in enumerate(text_lens)]).astype(np.int32)
    pos = np.concatenate([np.arange(T) for T in text_lens]).astype(np.int32)
    b0 = np.concatenate([np.full(T, block0[s]) for s, T in enumerate(text_lens)]).astype(np.int32)
    tl = np.concatenate([np.full(T, T) for T in text_lens]).astype(np.int32)
    b.text_scatter_fill_paged(pb.layer[0], text_k, text_v, nb, d(k), d(v), d(rs), d(pos), d(b0), d(tl), pb.d_prefill,
                              pb.d_len[0], pb.d_ring[0], total, W, ws)
    reqs, at = [], 0
    for s, T in enumerate(text_lens):
        reqs.append((at, T, s, 1, 0, block0[s]))
        at += T
    tiles = b.make_prefill_tiles(reqs)
    assert (tiles[:, 4] >= 127 + W).any()  # query tiles whose window starts beyond the prompt's first key tile
    out = torch.full((total, heads * hd), float("nan"), device="cuda")
    b.prefill_attention_tc(pb.layer[0], text_k, text_v, nb, d(q), pb.d_prefill, tiles, W, heads, out, ws)
    got = out.cpu().numpy()
    assert np.isfinite(got).all()
    at = 0
    worst_t = (0.0, 0.0)
    for s, T in enumerate(text_lens):
        keep = set(sampled_positions(T))
        rows_i, want = [], []
        for i in range(T):
            pb.cache[s].append_decode(0, k[at + i], v[at + i])
            if i in keep:
                rows_i.append(at + i)
                want.append(pb.cache[s].attention(0, q[at + i:at + i + 1], pb.cache[s].len(0) - 1, heads, False)[0])
        assert_attention_close(got[rows_i], np.array(want), *BAR)
        e = assert_attention_close(got[rows_i], np.array(want), *TC_TIGHT)
        worst_t = (max(worst_t[0], e[0]), max(worst_t[1], e[1]))
        at += T
    pb.check_logical_view(0)  # ring contents, len and ring_pos as 2048 / 1200 appends leave them
    # decode continues from the prefilled state
    rows = [1, 0]
    for t in range(2):
        kk, vv, qq = pb.step_inputs(t, 0, rows)
        g, w = pb.step_fused(0, kk, vv, qq, rows)
        assert_attention_close(g, w, *TIGHT)
    pb.check_logical_view(0)
    assert ws.status() == 0 and pb.ws.status() == 0
    print("cfg3 shapes: worst max-abs / rel-L2 vision", worst_v, "text", worst_t)


def test_prefill_tensor_core_query_tiles_beyond_the_window(orc, b):
    # W = 32, T = 300: from the second query tile on, the window's first key lies beyond text tile 0
    run_prefill_case(orc, b, b.BF16, 2, 128, 2, 32, prefixes=[40, 0], text_lens=[300, 290], seed=95, engine="tc_fused")
