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
    assert outs[0]["pos"] != outs[1]["pos"]                     # every replica draws its own workload
    assert outs[0]["by_rank"] == outs[1]["by_rank"] == [[1.0, 2.0, 3.0], [2.0, 3.0, 4.0]]
    import bench
    assert bench.aggregate_tokens_per_s([64, 64], 10, 20.0) == 64000.0
    assert [bench.shard_sequences(512, 8, r)[1] for r in range(8)] == [64] * 8
