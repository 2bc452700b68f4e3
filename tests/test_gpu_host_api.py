"""GPU tests of the C++ host API: the device-backed uocr::RSWACache driven by the same trace scripts
as the CPU oracle (bit-exact cache contents and cursors against the compiled reference's golden
vectors), the C++ test binary (GpuRSWACache, uocr::cuda::rswa_* with the reference's signatures,
PagedBatchKV, SlotAllocator), and the reference's own test_kv_ring_buffer.cpp compiled unmodified
against this library's headers."""
import os
import subprocess

import numpy as np
import pytest

import build_cpp_tests
import traces
from golden.make_golden import CACHE_CASES
from oracle import oracle
from paged_fixture import load_b200

pytestmark = pytest.mark.gpu
GOLD = np.load(os.path.join(os.path.dirname(__file__), "golden", "rswa_golden.npz"))


@pytest.fixture(scope="module")
def host():
    import torch
    if not torch.cuda.is_available():
        pytest.skip("needs a CUDA device")
    b = load_b200()
    return b.host_classes()


@pytest.mark.parametrize("name", ["tiny", "tiny_gqa", "p0", "ref_cuda_case", "cfg1"])
def test_rswa_cache_class_matches_reference_golden(host, name):
    # fp32 payload (the class default): contents, cursors and capacity bit-equal to the compiled reference
    L, kvh, hd, W, P, n, heads, seed, steps, bf16 = CACHE_CASES[name]
    assert not bf16
    r = traces.run_cache_trace(host, L, kvh, hd, W, P, n, heads, seed, steps, causal_prefill=(P <= 64))
    g = lambda k: GOLD[f"cache/{name}/{k}"]
    assert np.array_equal(r["book"], g("book")) and np.array_equal(r["meta"], g("meta"))
    if f"cache/{name}/keys" in GOLD:
        assert np.array_equal(r["keys"], g("keys")) and np.array_equal(r["values"], g("values"))
    else:
        assert np.array_equal(r["keys"].astype(np.float64).sum(-1), g("keys_rowsum"))
        assert np.array_equal(r["values"].astype(np.float64).sum(-1), g("values_rowsum"))
    assert np.abs(r["attn"] - g("attn")).max() <= 2e-5
    if r["prefill_attn"].size:
        assert np.abs(r["prefill_attn"] - g("prefill_attn")).max() <= 2e-5


def test_cpp_host_api_binary(tmp_path):
    if not os.path.exists(build_cpp_tests.HOST_API_BIN):
        build_cpp_tests.build(ref_root="/nonexistent")
    env = dict(os.environ, UOCR_SNAPSHOT_DIR=str(tmp_path))
    out = subprocess.run([build_cpp_tests.HOST_API_BIN], capture_output=True, text=True, timeout=600, env=env)
    assert out.returncode == 0 and "ALL OK" in out.stdout, out.stdout + out.stderr
    # the snapshot the binary exported (contents already checked there against the oracle): the manifest
    # must be real JSON in the reference's export layout, and every tensor file as large as its shape says
    import json
    man = json.loads((tmp_path / "manifest.json").read_text())
    assert man["cache_layers"] == 2 and man["window"] == 16 and man["final_cache_len"] > 0
    assert sorted(man["tensors"]) == ["final_k_0", "final_k_1", "final_v_0", "final_v_1"]
    for name, entry in man["tensors"].items():
        assert entry["dtype"] == "<f4" and entry["file"] == name + ".bin"
        assert entry["shape"] == [man["kv_heads"], man["final_cache_len"], man["head_dim"]]
        data = np.fromfile(tmp_path / entry["file"], dtype="<f4")
        assert data.size == int(np.prod(entry["shape"])) and np.isfinite(data).all() and np.abs(data).max() > 0


def test_reference_kv_ring_buffer_tests_on_this_library():
    # the reference's tests/test_kv_ring_buffer.cpp (ring_buffer_lifecycle, ring_attention_matches_naive,
    # prefill_causal_attention), compiled unmodified where the checkout was present at build time
    if not os.path.exists(build_cpp_tests.REF_BIN):
        pytest.skip("binary of the reference's test file was not built (no reference checkout at build time)")
    out = subprocess.run([build_cpp_tests.REF_BIN], capture_output=True, text=True, timeout=600)
    assert out.returncode == 0, out.stdout + out.stderr
    assert "3 passed" in out.stdout, out.stdout
