"""Host-side checks of the benchmark's bookkeeping (no GPU): the ncu traffic record the bench line quotes
belongs to the kernel sources as they are now, the algorithmic-byte formula matches its definition, and
both arms print the same workload description."""
import numpy as np

import bench


def test_traffic_record_matches_current_kernel_sources():
    traffic, algorithmic, source = bench.traffic_record()
    assert traffic is not None, source  # stale: re-capture the kernel and update the traffic-record line
    assert bench.kernel_source_sha() in source
    assert 1.0 <= traffic / algorithmic < 1.05  # no wasted re-reads in the captured launch


def test_algorithmic_bytes_formula():
    # 5120 B per token of bf16 K+V: window tokens read + every distinct prefix once + appended rows written,
    # plus q read, out written, new k and v read in fp32 (4 x 1280 x 4 B per row)
    pos = np.array([1, 500, 1024, 4000], np.int64)
    ids = np.zeros(4, np.int64)
    want = 5120 * ((1 + 500 + 1024 + 1024) + 256 + 4) + 4 * 1280 * 4 * 4
    assert bench.algorithmic_bytes_per_layer(pos, ids) == float(want)


def test_both_arms_describe_the_same_workload():
    a, b = bench.workload_config(1), bench.workload_config(1)
    assert a == b and a["seqs_per_gpu"] == 64 and a["window"] == 1024 and "l2_policy" in a
