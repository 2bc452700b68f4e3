"""GPU parity of the reference-layout entry points (contiguous fp32 caches, the argument lists of
uocr::cuda::rswa_*) against the CPU oracle.  Scenarios follow the reference's own CUDA tests
(tests/test_rswa_cuda.cu:51-361); its tolerances are 1e-3 (attention) and 1e-5 (cache contents) --
here cache contents must be bit-equal and attention within 2e-5.
"""
import numpy as np
import pytest

import synth
from paged_fixture import assert_attention_close, load_b200

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def b():
    import torch
    if not torch.cuda.is_available():
        pytest.skip("needs a CUDA device")
    return load_b200()


def dev(x):
    import torch
    return torch.from_numpy(np.ascontiguousarray(x)).cuda()


def test_decode_attention_real_geometry(orc, b):
    # tests/test_rswa_cuda.cu:52-104
    import torch
    kvh = heads = 10
    hd, W, P = 128, 128, 257
    row = kvh * hd
    c = orc.Cache(1, kvh, hd, W)
    c.reset(P)
    c.write_prefill(0, synth.normal(1234, 0, (P, row)), synth.normal(1234, 1, (P, row)))
    for i in range(50):
        c.append_decode(0, synth.normal(1234, 10 + i, (row,)), synth.normal(1234, 100 + i, (row,)))
    kv_len = c.len(0)
    q = synth.normal(1234, 999, (1, heads * hd))
    want = c.attention(0, q, kv_len - 1, heads, False)
    dk, dv = dev(c.keys(0, full=True)), dev(c.values(0, full=True))
    ws = b.Workspace(64)
    out = torch.full((1, heads * hd), float("nan"), device="cuda")
    b.attention_f32(dev(q), dk, dv, kv_len, None, 1, 0, heads, kvh, hd, False, out, ws)
    assert_attention_close(out.cpu().numpy(), want, 2e-5, 1e-5)
    # device-length form (rswa_attention_devlen): same answer with the length read on the device
    dlen = torch.tensor([kv_len], dtype=torch.int32, device="cuda")
    out2 = torch.full_like(out, float("nan"))
    b.attention_f32(dev(q), dk, dv, 0, dlen, 1, 0, heads, kvh, hd, False, out2, ws)
    assert np.array_equal(out.cpu().numpy(), out2.cpu().numpy())
    assert ws.status() == 0


def test_single_cache_ring_overwrite_and_causal_prefill(orc, b):
    # tests/test_rswa_cuda.cu:107-221: W=8, P=4, 24 appends (3 wraps), then causal prefill attention
    import torch
    kvh = heads = 10
    hd, W, P = 128, 8, 4
    row = kvh * hd
    cap = P + W
    hc = orc.Cache(1, kvh, hd, W)
    hc.reset(P)
    pk, pv = synth.normal(7, 0, (P, row)), synth.normal(7, 1, (P, row))
    hc.write_prefill(0, pk, pv)
    kc = torch.zeros((cap, row), device="cuda")
    vc = torch.zeros((cap, row), device="cuda")
    zeros = torch.zeros(P, dtype=torch.int32, device="cuda")
    b.write_prefill_ragged_f32(dev(pk), dev(pv), kc, vc, zeros, torch.arange(P, dtype=torch.int32, device="cuda"),
                               P, cap, kvh, hd)
    dlen = torch.tensor([P], dtype=torch.int32, device="cuda")
    dring = torch.zeros(1, dtype=torch.int32, device="cuda")
    for t in range(24):
        k, v = synth.normal(7, 10 + t, (row,)), synth.normal(7, 100 + t, (row,))
        hc.append_decode(0, k, v)
        b.append_decode_f32(dev(k), dev(v), kc, vc, dlen, dring, P, W, kvh, hd)
    assert int(dlen[0]) == hc.len(0) and int(dring[0]) == hc.ring_pos(0)
    assert np.array_equal(kc.cpu().numpy(), hc.keys(0, full=True))
    assert np.array_equal(vc.cpu().numpy(), hc.values(0, full=True))
    ws = b.Workspace(64)
    q = synth.normal(7, 999, (1, heads * hd))
    out = torch.full((1, heads * hd), float("nan"), device="cuda")
    b.attention_f32(dev(q), kc, vc, hc.len(0), None, 1, hc.len(0) - 1, heads, kvh, hd, False, out, ws)
    assert_attention_close(out.cpu().numpy(), hc.attention(0, q, hc.len(0) - 1, heads, False), 2e-5, 1e-5)
    # causal prefill over a fresh cache holding only the prefix
    hp = orc.Cache(1, kvh, hd, W)
    hp.reset(P)
    hp.write_prefill(0, pk, pv)
    qa = synth.normal(7, 555, (P, heads * hd))
    outa = torch.full((P, heads * hd), float("nan"), device="cuda")
    b.attention_f32(dev(qa), dev(hp.keys(0, full=True)), dev(hp.values(0, full=True)), P, None, P, 0, heads, kvh, hd,
                    True, outa, ws)
    assert_attention_close(outa.cpu().numpy(), hp.attention(0, qa, 0, heads, True), 2e-5, 1e-5)
    assert ws.status() == 0


def test_batched_append_attention_with_slot_permutation(orc, b):
    # tests/test_rswa_cuda.cu:224-361: kv_heads=heads=4, hd=64, W=8, prefill {4,6,3}, rows -> slots {2,1,0}
    import torch
    kvh = heads = 4
    hd, W, batch = 64, 8, 3
    prefill = [4, 6, 3]
    cap = 6 + W
    row = kvh * hd
    caches = []
    kb = np.zeros((batch, cap, row), np.float32)
    vb = np.zeros((batch, cap, row), np.float32)
    for s in range(batch):
        c = orc.Cache(1, kvh, hd, W)
        c.reset(prefill[s])
        k, v = synth.normal(21, s, (prefill[s], row)), synth.normal(21, 10 + s, (prefill[s], row))
        c.write_prefill(0, k, v)
        kb[s, :prefill[s]], vb[s, :prefill[s]] = k, v
        caches.append(c)
    dkb, dvb = dev(kb), dev(vb)
    d_len = torch.tensor(prefill, dtype=torch.int32, device="cuda")
    d_ring = torch.zeros(batch, dtype=torch.int32, device="cuda")
    d_pref = torch.tensor(prefill, dtype=torch.int32, device="cuda")
    slots = [2, 1, 0]
    d_slots = torch.tensor(slots, dtype=torch.int32, device="cuda")
    ws = b.Workspace(64)
    for step in range(3 * W):
        k, v = synth.normal(21, 1000 + step, (batch, row)), synth.normal(21, 2000 + step, (batch, row))
        q = synth.normal(21, 3000 + step, (batch, heads * hd))
        b.append_decode_batch_f32(dev(k), dev(v), dkb, dvb, d_len, d_ring, d_pref, d_slots, batch, cap, W, kvh, hd)
        out = torch.full((batch, heads * hd), float("nan"), device="cuda")
        b.attention_batch_f32(dev(q), dkb, dvb, d_len, d_slots, batch, cap, heads, kvh, hd, out, ws)
        want = []
        for r, s in enumerate(slots):
            caches[s].append_decode(0, k[r], v[r])
            want.append(caches[s].attention(0, q[r:r + 1], caches[s].len(0) - 1, heads, False)[0])
        assert_attention_close(out.cpu().numpy(), np.array(want), 2e-5, 1e-5)
    got_k, got_v = dkb.cpu().numpy(), dvb.cpu().numpy()
    for s in range(batch):
        n = caches[s].len(0)
        assert int(d_len[s]) == n and int(d_ring[s]) == caches[s].ring_pos(0)
        assert np.array_equal(got_k[s, :n], caches[s].keys(0)) and np.array_equal(got_v[s, :n], caches[s].values(0))
        assert not got_k[s, n:].any()
    assert ws.status() == 0


def test_ragged_prefill_scatter_and_attention(orc, b):
    # packed rows of several requests, row t -> (slot, pos), causal within its request
    # (src/kernels/cuda/rswa_attention.cu:218-305; call site src/engine/gpu_decoder.cu:1042-1046)
    import torch
    kvh, heads, hd, W = 2, 4, 32, 8
    lengths, slots = [5, 33, 1, 16], [3, 0, 2, 1]
    cap = max(lengths) + W
    row = kvh * hd
    total = sum(lengths)
    k, v = synth.normal(31, 0, (total, row)), synth.normal(31, 1, (total, row))
    q = synth.normal(31, 2, (total, heads * hd))
    pos = np.concatenate([np.arange(n) for n in lengths]).astype(np.int32)
    rs = np.concatenate([np.full(n, s) for n, s in zip(lengths, slots)]).astype(np.int32)
    kb = torch.zeros((4, cap, row), device="cuda")
    vb = torch.zeros((4, cap, row), device="cuda")
    ws = b.Workspace(total)
    b.write_prefill_ragged_f32(dev(k), dev(v), kb, vb, dev(rs), dev(pos), total, cap, kvh, hd)
    out = torch.full((total, heads * hd), float("nan"), device="cuda")
    b.attention_ragged_f32(dev(q), kb, vb, dev(rs), dev(pos), total, cap, heads, kvh, hd, out, ws)
    got = out.cpu().numpy()
    start = 0
    for n, s in zip(lengths, slots):
        c = orc.Cache(1, kvh, hd, W)
        c.reset(n)
        c.write_prefill(0, k[start:start + n], v[start:start + n])
        want = c.attention(0, q[start:start + n], 0, heads, True)
        assert_attention_close(got[start:start + n], want, 2e-5, 1e-5)
        assert np.array_equal(kb[s, :n].cpu().numpy(), k[start:start + n])
        start += n
    assert ws.status() == 0


def test_unaligned_rows_take_the_scalar_copy(orc, b):
    # kv_heads*head_dim not a multiple of 4: append still bit-exact (attention needs 16-byte rows and says so)
    import torch
    kvh, hd, W, P = 1, 6, 4, 2
    c = orc.Cache(1, kvh, hd, W)
    c.reset(P)
    kc = torch.zeros((P + W, 6), device="cuda")
    vc = torch.zeros((P + W, 6), device="cuda")
    dlen = torch.tensor([P], dtype=torch.int32, device="cuda")
    dring = torch.zeros(1, dtype=torch.int32, device="cuda")
    for t in range(11):
        k, v = synth.normal(41, t, (6,)), synth.normal(41, 100 + t, (6,))
        c.append_decode(0, k, v)
        b.append_decode_f32(dev(k), dev(v), kc, vc, dlen, dring, P, W, kvh, hd)
    assert np.array_equal(kc.cpu().numpy()[P:], c.keys(0, full=True)[P:])
    assert (int(dlen[0]), int(dring[0])) == (c.len(0), c.ring_pos(0))
    ws = b.Workspace(4)
    with pytest.raises(b.Error) as e:
        b.attention_f32(kc, kc, vc, P + W, None, 1, 0, 1, 1, 6, False, kc, ws)
    assert e.value.status == 2
