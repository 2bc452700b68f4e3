"""Generates tests/golden/rswa_golden.npz from the COMPILED, UNMODIFIED reference
(oracle/_ref/libuocr_ref.so, built by `make -C oracle ref` where the reference checkout exists).

Run:  python tests/golden/make_golden.py
The fixture holds the reference's outputs on seeded traces (inputs are regenerated from the seeds by
tests/synth.py, which is integer-only and therefore bit-reproducible; the op lists of the
allocator/scheduler traces are stored in the file itself).
"""
import os
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
sys.path[:0] = [ROOT, os.path.join(ROOT, "tests")]

import traces  # noqa: E402
from oracle import oracle  # noqa: E402

CACHE_CASES = {
    # name: (layers, kvh, hd, W, P, n_append, heads, seed, attn_steps, bf16)
    "tiny": (2, 2, 8, 8, 5, 29, 2, 11, (0, 7, 8, 20, 28), False),
    "tiny_gqa": (1, 2, 8, 4, 3, 13, 4, 12, (0, 3, 4, 12), False),
    "p0": (1, 2, 4, 4, 0, 9, 2, 13, (0, 3, 8), False),
    "ragged_p17": (1, 2, 16, 16, 17, 50, 2, 14, (0, 15, 16, 49), True),
    "ref_cuda_case": (1, 10, 128, 128, 257, 50, 10, 1234, (49,), False),  # tests/test_rswa_cuda.cu:52-104 geometry
    "cfg1": (1, 10, 128, 128, 256, 300, 10, 1234, (0, 127, 128, 299), False),
    "cfg1_bf16": (1, 10, 128, 128, 256, 300, 10, 1234, (0, 127, 128, 299), True),
}


def main():
    ref = oracle.load("ref")
    out = {}
    for name, (L, kvh, hd, W, P, n, heads, seed, steps, bf16) in CACHE_CASES.items():
        r = traces.run_cache_trace(ref, L, kvh, hd, W, P, n, heads, seed, steps, bf16=bf16,
                                   causal_prefill=(P <= 64))
        out[f"cache/{name}/book"] = r["book"]
        out[f"cache/{name}/attn"] = r["attn"]
        out[f"cache/{name}/meta"] = r["meta"]
        out[f"cache/{name}/prefill_attn"] = r["prefill_attn"]
        if r["keys"].size <= 1 << 16:
            out[f"cache/{name}/keys"] = r["keys"]
            out[f"cache/{name}/values"] = r["values"]
        else:  # large: keep float64 per-row sums (order-sensitive bit pin stays in the small cases)
            out[f"cache/{name}/keys_rowsum"] = r["keys"].astype(np.float64).sum(-1)
            out[f"cache/{name}/values_rowsum"] = r["values"].astype(np.float64).sum(-1)

    ops, total = traces.make_pool_ops(5, 3000, 1 << 16, 3000, aligns=(0, 0, 1, 64, 512))
    out["pool/ops"] = ops
    out["pool/cfg"] = np.array([total, 256], dtype=np.int64)
    out["pool/res"] = traces.run_pool_trace(ref, ops, total, 256)
    ops2, total2 = traces.make_pool_ops(6, 2000, 1000, 300, aligns=(0,))
    out["pool1/ops"] = ops2
    out["pool1/cfg"] = np.array([total2, 1], dtype=np.int64)
    out["pool1/res"] = traces.run_pool_trace(ref, ops2, total2, 1)

    bops = traces.make_bm_ops(7, 4000, 8, 91, 64)
    out["bm/ops"] = bops
    out["bm/cfg"] = np.array([1024, 64 * 40], dtype=np.int64)
    out["bm/res"] = traces.run_bm_trace(ref, bops, 1024, 64 * 40)

    script = traces.make_sched_script(8, 200, 30)
    out["sched/script"] = script
    out["sched/res"] = traces.run_sched_trace(ref, script, 16)
    out["sched/res_early"] = traces.run_sched_trace(ref, script, 5, early_finish_every=7)

    for name, case in traces.ROPE_CASES.items():
        out[f"rope/{name}/q"], out[f"rope/{name}/k"] = traces.run_rope_case(ref, *case)

    path = os.path.join(HERE, "rswa_golden.npz")
    np.savez_compressed(path, **out)
    print("wrote", path, os.path.getsize(path), "bytes;", len(out), "arrays")


if __name__ == "__main__":
    main()
