"""The N>1 path of the benchmark on CPU: two gloo ranks exercise the sharding, the barrier and the
max-over-ranks reduction that bracket the timed region (the data path itself has no collective:
sequences shard by request and every GPU owns its pool)."""
import os
import subprocess
import sys
import textwrap

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))

WORKER = textwrap.dedent("""
    import json, os, sys
    sys.path.insert(0, %r)
    import bench
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    r = bench.Ranks(rank, world, backend="gloo")
    r.barrier()
    slow = r.max_over_ranks(10.0 + 5.0 * rank)           # rank 1 is the slow one
    by_rank = r.gather([1.0 + rank, 2.0 + rank, 3.0 + rank])  # per-repeat times of every rank, seen by all
    start, n = bench.shard_sequences(513, world, rank)
    bench.CFG["seqs"] = 8
    pos = bench.draw_positions(rank).tolist()
    r.close()
    print(json.dumps({"rank": rank, "slow": slow, "start": start, "n": n, "pos": pos, "by_rank": by_rank}))
""") % ROOT


def test_two_gloo_ranks(tmp_path):
    script = tmp_path / "worker.py"
    script.write_text(WORKER)
    env = dict(os.environ, MASTER_ADDR="127.0.0.1", MASTER_PORT="29631", WORLD_SIZE="2")
    procs = [subprocess.Popen([sys.executable, str(script)], env=dict(env, RANK=str(r)), stdout=subprocess.PIPE,
                              stderr=subprocess.PIPE, text=True) for r in range(2)]
    outs = []
    for p in procs:
        o, e = p.communicate(timeout=300)
        assert p.returncode == 0, e
        outs.append(__import__("json").loads(o.strip().splitlines()[-1]))
    outs.sort(key=lambda d: d["rank"])
    assert outs[0]["slow"] == outs[1]["slow"] == 15.0          # MAX over ranks, seen by every rank
    assert (outs[0]["start"], outs[0]["n"]) == (0, 257) and (outs[1]["start"], outs[1]["n"]) == (257, 256)
    assert outs[0]["pos"] == outs[1]["pos"]                     # weak scaling: the same work on every replica
    assert outs[0]["by_rank"] == outs[1]["by_rank"] == [[1.0, 2.0, 3.0], [2.0, 3.0, 4.0]]
    import bench
    assert bench.aggregate_tokens_per_s([64, 64], 10, 20.0) == 64000.0
    assert [bench.shard_sequences(512, 8, r)[1] for r in range(8)] == [64] * 8


def test_strong_scaling_shards_keep_prefix_affinity_and_balance_bytes():
    # 512 sequences, 4 prefixes, W = 4096 dealt to 8 ranks: every sequence lands on exactly one rank, a rank
    # holds at most two distinct prefixes, and the window tokens per rank are within 1.5 % of the mean (the
    # plain equal-count split of the prefix-sorted order is several percent off)
    import numpy as np
    import bench
    import synth
    total, world, W = 512, 8, 4096
    pos = synth.integers(1234, 77, 1, 16384, (total,)).astype(np.int64)
    ids = synth.integers(1234, 177, 0, 3, (total,)).astype(np.int64)
    load = np.minimum(pos, W)
    spreads = {}
    for balance in (False, True):
        order, bounds = bench.balanced_shards(ids, load, total, world, balance=balance)
        assert sorted(order.tolist()) == list(range(total)) and bounds[0] == 0 and bounds[-1] == total
        per_rank = []
        for r in range(world):
            mine = order[bounds[r]:bounds[r + 1]]
            assert len(mine) >= 1 and len(set(ids[mine].tolist())) <= 2
            per_rank.append(int(load[mine].sum()))
        spreads[balance] = max(per_rank) / (sum(per_rank) / world) - 1.0
    assert spreads[True] < 0.015 < spreads[False]
    for w in (1, 2, 4):
        order, bounds = bench.balanced_shards(ids, load, total, w)
        assert sorted(order.tolist()) == list(range(total)) and len(bounds) == w + 1
