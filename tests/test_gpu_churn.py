"""Block-manager churn (scaled-down form of the 65536-block stress configuration): the library's host
allocator and scheduler run in lockstep with the CPU oracle (and, when present, the compiled
reference); every block-table row, every stats tuple and every batch must be identical, the appended
values of sampled sequences must match an oracle cache bit for bit at retirement, and at the end all
arenas are empty."""
import numpy as np
import pytest

import churn_driver
from oracle import oracle
from paged_fixture import load_b200

pytestmark = pytest.mark.gpu


def small_cfg(**kw):
    base = dict(requests=120, slots=24, layers=2, kv_heads=2, head_dim=16, window=64,
                prefix_lens=(16, 32, 48, 80, 96, 112, 144, 176), out_lo=4, out_hi=200,
                prefix_arena_blocks=64, ring_arena_blocks=24 * 4 + 8, mean_interarrival=2.0, seed=77, sample_every=7)
    base.update(kw)
    return churn_driver.ChurnConfig(**base)


@pytest.mark.parametrize("checker,all_layers", [("orc", False), ("ref", False), ("orc", True)])
def test_churn_tables_bit_exact(orc, checker, all_layers):
    import torch
    if not torch.cuda.is_available():
        pytest.skip("needs a CUDA device")
    if checker == "ref" and not oracle.available("ref"):
        pytest.skip("compiled reference not present")
    b = load_b200()
    host = b.host_classes()
    chk = oracle.load(checker)
    cfg = small_cfg(all_layer_launches=all_layers)  # appends (and unsampled gathers) of every layer in one launch
    res = churn_driver.run(cfg, host, check=chk, oracle_caches=orc)
    assert res["mismatches"] == 0
    assert len(res["rows"]) == cfg.requests
    # block ids stay inside their arenas and live rows never share a ring block
    for rid, slot, row in res["rows"]:
        used = row[row >= 0]
        assert used.max() < cfg.prefix_arena_blocks + cfg.ring_arena_blocks
    a, c = res["final"]
    assert a == c and a[0] == 0 and a[3] == 0 and a[7] == 0  # everything released at the end
    assert res["sched"][0] == res["sched"][1]
    assert res["sched"][0][1] == cfg.requests  # all finished
    assert res["stats"]["prefix_hits"] > 0 and res["stats"]["peak_running"] > 4
