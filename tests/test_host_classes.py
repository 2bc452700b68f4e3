"""The host-side C++ classes of the CUDA library (MemoryPool, BlockManager,
ContinuousBatchScheduler) against the golden vectors of the compiled reference and, live, against
the CPU oracle.  They are driven through the library's host C ABI with the very scripts that drive
the oracle, so every offset, counter, batch and fragmentation figure is compared entry by entry.
Also compiles the reference's own unit tests for these classes, unmodified, against this library's
headers where the reference checkout is available."""
import os
import subprocess

import numpy as np
import pytest

import traces
from oracle import oracle
from paged_fixture import ROOT, load_b200

GOLD = np.load(os.path.join(os.path.dirname(__file__), "golden", "rswa_golden.npz"))
REF = oracle.reference_root()


@pytest.fixture(scope="module")
def host():
    b = load_b200()
    if not os.path.exists(b.LIB_PATH):
        b.build()
    return b.host_classes()


@pytest.mark.parametrize("key", ["pool", "pool1"])
def test_memory_pool_matches_reference_golden(host, key):
    total, al = GOLD[f"{key}/cfg"].tolist()
    assert np.array_equal(traces.run_pool_trace(host, GOLD[f"{key}/ops"], total, al), GOLD[f"{key}/res"])


def test_block_manager_matches_reference_golden(host):
    pb, rb = GOLD["bm/cfg"].tolist()
    assert np.array_equal(traces.run_bm_trace(host, GOLD["bm/ops"], pb, rb), GOLD["bm/res"])


def test_scheduler_matches_reference_golden(host):
    assert np.array_equal(traces.run_sched_trace(host, GOLD["sched/script"], 16), GOLD["sched/res"])
    assert np.array_equal(traces.run_sched_trace(host, GOLD["sched/script"], 5, early_finish_every=7),
                          GOLD["sched/res_early"])


@pytest.mark.parametrize("seed", [201, 202, 203, 204])
def test_host_classes_vs_oracle_random(host, orc, seed):
    ops, total = traces.make_pool_ops(seed, 2500, 1 << 15, 1500, aligns=(0, 0, 8, 256, 1024))
    assert np.array_equal(traces.run_pool_trace(host, ops, total, 256), traces.run_pool_trace(orc, ops, total, 256))
    ops, total = traces.make_pool_ops(seed + 50, 2500, 4096, 64, aligns=(0,))
    assert np.array_equal(traces.run_pool_trace(host, ops, total, 1), traces.run_pool_trace(orc, ops, total, 1))
    bops = traces.make_bm_ops(seed, 3000, 8, 91, 64)
    assert np.array_equal(traces.run_bm_trace(host, bops, 512, 64 * 30), traces.run_bm_trace(orc, bops, 512, 64 * 30))
    sc = traces.make_sched_script(seed, 150, 25)
    for mb, ef in ((3, 0), (16, 4), (64, 9)):
        assert np.array_equal(traces.run_sched_trace(host, sc, mb, ef), traces.run_sched_trace(orc, sc, mb, ef))


def test_host_failure_points(host):
    # pool exhausted, double release, unknown key, and everything returns to zero afterwards
    bm = host.BlockManager(4 * 256, 2 * 256)
    assert bm.acquire_prefix("a", 48, 3 * 256)[0] == 0
    assert bm.acquire_prefix("b", 32, 2 * 256)[0] == -1  # "prefix pool exhausted"
    assert bm.allocate_ring(2 * 256) == 0
    assert bm.allocate_ring(256) == -1
    bm.release_prefix("a")
    bm.release_prefix("a")  # second release: the key is gone, no-op
    bm.release_prefix("never")
    bm.free_ring(0, 2 * 256)
    st = bm.stats()
    assert st[0] == 0 and st[3] == 0 and st[7] == 0 and st[5] == 0.0 and st[6] == 0.0
    s = host.Scheduler(2, 1)
    i = s.add_request(3, 1)
    s.build_batch()
    s.mark_prefilled(i)
    assert s.add_token(i, 5) is True
    s.finish(i)  # finishing twice is harmless
    assert s.add_token(999, 1) is True  # unknown id reports finished
    assert not s.has_work()


@pytest.mark.skipif(not os.path.isdir(os.path.join(REF, "tests")), reason="reference checkout not present")
def test_reference_unit_tests_compile_and_pass_against_this_library(tmp_path):
    # the reference's own tests for the allocator, the block manager and the scheduler, compiled
    # unmodified from where they lie against this library's headers and linked to this library
    b = load_b200()
    exe = tmp_path / "ref_host_tests"
    inc = [os.path.join(ROOT, "unlimited-ocr.cpp_b200", "include"), os.path.join(ROOT, "include"),
           os.path.join(REF, "tests")]
    srcs = [os.path.join(REF, "tests", f) for f in ("test_main.cpp", "test_memory_budget.cpp", "test_scheduler.cpp")]
    cmd = ["g++", "-std=c++17", "-O1", *[f"-I{i}" for i in inc], *srcs, "-o", str(exe),
           f"-L{os.path.dirname(b.LIB_PATH)}", "-luocr_rswa_b200", f"-Wl,-rpath,{os.path.dirname(b.LIB_PATH)}"]
    subprocess.check_call(cmd)
    out = subprocess.run([str(exe)], capture_output=True, text=True)
    assert out.returncode == 0, out.stdout + out.stderr
    assert "5 passed" in out.stdout or "passed" in out.stdout
    # the KV-cache test file needs a GPU to run, but must at least compile against the same headers
    obj = tmp_path / "kv.o"
    subprocess.check_call(["g++", "-std=c++17", "-c", *[f"-I{i}" for i in inc],
                           os.path.join(REF, "tests", "test_kv_ring_buffer.cpp"), "-o", str(obj)])


@pytest.mark.parametrize("checker", ["orc", "ref"])
def test_churn_full_size_tables_bit_exact(host, checker):
    # The block-manager churn stress at its full size -- pool of 65536 blocks (1024 prefix ids + 64512 ring
    # ids), 1000 requests on the seeded arrival schedule, 8 prefixes, output lengths 32..2048, W=1024 -- with
    # the KV writes switched off: allocator offsets, every block-table row, every stats tuple and every
    # scheduler batch of this library's host classes must equal the checker's (the compiled reference where
    # it is present, the restatement always), the end-of-run table is empty and both arenas are free.
    import churn_driver
    if checker == "ref" and not oracle.available("ref"):
        pytest.skip("compiled reference not present")
    chk = oracle.load(checker)
    cfg = churn_driver.ChurnConfig()
    assert (cfg.requests, cfg.prefix_arena_blocks + cfg.ring_arena_blocks, cfg.window) == (1000, 65536, 1024)
    res = churn_driver.run(cfg, host, check=chk, device=False)
    assert res["mismatches"] == 0
    assert len(res["rows"]) == cfg.requests
    ring_blocks = cfg.window // 16
    live = {}
    for rid, slot, row in res["rows"]:
        used = row[row >= 0]
        assert used.min() >= 0 and used.max() < 65536
        ring = row[row >= cfg.prefix_arena_blocks]
        assert len(ring) == ring_blocks and (np.diff(ring) == 1).all()  # one contiguous first-fit allocation
    a, c = res["final"]
    assert a == c and a[0] == 0 and a[3] == 0 and a[7] == 0
    assert (res["table"] == -1).all()
    assert res["sched"][0] == res["sched"][1] and res["sched"][0][1] == cfg.requests
    assert res["stats"]["prefix_hits"] > 0 and res["stats"]["peak_running"] > 64
