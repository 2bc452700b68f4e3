"""Python plumbing over the C ABI of libuocr_rswa_b200.so (tests and benchmark only).

The product is the shared library (hand-written sm_100a kernels behind `include/uocr_rswa_b200.h`)
plus the C++17 host classes under `include/uocr/`.  This module only loads the library with ctypes,
mirrors the structs of the header, and offers thin wrappers that take torch CUDA tensors (used here
purely as device-memory handles) and launch on torch's current stream.  There is no fallback: if
the library is missing or a call fails, an exception is raised.

The directory name is not a Python identifier; load it with

    importlib.util.spec_from_file_location("uocr_b200", "<repo>/unlimited-ocr.cpp_b200/__init__.py")
"""
from __future__ import annotations

import ctypes as C
import os
import subprocess

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(HERE)
LIB_PATH = os.path.join(HERE, "libuocr_rswa_b200.so")

F32, BF16 = 0, 1
BLOCK_TOKENS = 16
STATUS_BAD_BLOCK, STATUS_WAIT_TIMEOUT, STATUS_BAD_SLOT = 1, 2, 4

NVCC_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
              "-Xcompiler", "-fPIC,-fvisibility=hidden", "-shared"]


def sources():
    csrc = os.path.join(HERE, "csrc")
    return sorted(os.path.join(csrc, f) for f in os.listdir(csrc) if f.endswith((".cu", ".cpp")))


def build(verbose: bool = False) -> str:
    """Compile every source under csrc/ for sm_100a into libuocr_rswa_b200.so (in-tree)."""
    cmd = ["nvcc", *NVCC_FLAGS, "-I", os.path.join(ROOT, "include"), "-I", os.path.join(HERE, "include"),
           "-I", os.path.join(HERE, "csrc"), "-o", LIB_PATH, *sources()]
    if verbose:
        print(" ".join(cmd))
    subprocess.check_call(cmd)
    return LIB_PATH


class PagedKV(C.Structure):
    """uocr_b200_paged_kv"""
    _fields_ = [("k_pool", C.c_void_p), ("v_pool", C.c_void_p), ("block_table", C.c_void_p),
                ("table_stride", C.c_int32), ("num_blocks", C.c_int32), ("kv_heads", C.c_int32),
                ("head_dim", C.c_int32), ("dtype", C.c_int32)]


class Error(RuntimeError):
    def __init__(self, status, msg):
        super().__init__(f"uocr_b200 status {status}: {msg}")
        self.status = status


_LIB = None

_vp, _i, _i64 = C.c_void_p, C.c_int, C.c_int64
_SIGS = {
    "uocr_b200_status_string": (C.c_char_p, [_i]),
    "uocr_b200_last_error": (C.c_char_p, []),
    "uocr_b200_version": (C.c_char_p, []),
    "uocr_b200_launch_count": (C.c_uint64, []),
    "uocr_b200_workspace_create": (_i, [_i, C.POINTER(_vp)]),
    "uocr_b200_workspace_destroy": (_i, [_vp]),
    "uocr_b200_workspace_status": (_i, [_vp, _vp, C.POINTER(_i)]),
    "uocr_b200_workspace_set_timing": (_i, [_vp, _i]),
    "uocr_b200_workspace_set_overlap": (_i, [_vp, _i]),
    "uocr_b200_workspace_set_wait_limit": (_i, [_vp, C.c_uint]),
    "uocr_b200_noalloc_status": (_i, [_vp, C.POINTER(_i)]),
    "uocr_b200_workspace_set_out_dtype": (_i, [_vp, _i]),
    "uocr_b200_workspace_stream_read_gbs": (_i, [_vp, _vp, C.POINTER(C.c_double)]),
    "uocr_b200_workspace_last_kernel_ms": (_i, [_vp, C.POINTER(C.c_float)]),
    "uocr_b200_rswa_append_decode_batch_f32": (_i, [_vp] * 8 + [_i] * 5 + [_vp]),
    "uocr_b200_rswa_append_decode_f32": (_i, [_vp] * 6 + [_i] * 4 + [_vp]),
    "uocr_b200_rswa_append_decode_batch_paged": (_i, [C.POINTER(PagedKV)] + [_vp] * 6 + [_i, _i, _vp, _vp]),
    "uocr_b200_rswa_append_decode_batch_paged_layers": (_i, [_vp, _i, _vp, _vp, C.c_longlong, _vp, _vp, C.c_longlong, _vp, _vp,
                                                              _i, _i, _vp, _vp]),
    "uocr_b200_rswa_gather_paged_layers": (_i, [_vp, _i, _vp, C.c_longlong, _vp, _vp, _i, _i, _vp, _vp, C.c_longlong, _i,
                                                 _vp, _vp]),
    "uocr_b200_rswa_write_prefill_ragged_f32": (_i, [_vp] * 6 + [_i] * 4 + [_vp]),
    "uocr_b200_rswa_write_prefill_ragged_paged": (_i, [C.POINTER(PagedKV)] + [_vp] * 4 + [_i, _vp, _vp]),
    "uocr_b200_rswa_publish_slots": (_i, [_vp, _i, _vp, _i, _vp, _vp, _vp, _i, _i, _vp, _vp]),
    "uocr_b200_rswa_attention_batch_f32": (_i, [_vp] * 5 + [_i] * 5 + [_vp, _vp, _vp]),
    "uocr_b200_rswa_attention_batch_paged": (_i, [C.POINTER(PagedKV)] + [_vp] * 4 + [_i, _i, _vp, _vp, _vp]),
    "uocr_b200_rswa_prefill_text_paged": (_i, [C.POINTER(PagedKV), _vp, _vp, _i] + [_vp] * 7 + [_i, _i, _i, _vp, _vp, _vp]),
    "uocr_b200_rswa_text_scatter_paged": (_i, [C.POINTER(PagedKV), _vp, _vp, _i] + [_vp] * 4 + [_i, _vp, _vp]),
    "uocr_b200_rswa_text_scatter_fill_paged": (_i, [C.POINTER(PagedKV), _vp, _vp, _i] + [_vp] * 9 + [_i, _i, _vp, _vp]),
    "uocr_b200_rswa_prefill_attention_tc": (_i, [C.POINTER(PagedKV), _vp, _vp, _i, _vp, _vp, _vp, _i, _i, _i, _vp, _vp, _vp]),
    "uocr_b200_rswa_prefill_plan_tc": (_i, [_vp, _i, _vp, _i, _vp, _vp]),
    "uocr_b200_workspace_prefill_plan_serial": (C.c_uint, [_vp]),
    "uocr_b200_rswa_ring_fill_paged": (_i, [C.POINTER(PagedKV), _vp, _vp, _i] + [_vp] * 7 + [_i, _i, _vp, _vp]),
    "uocr_b200_rswa_decode_step_paged": (_i, [C.POINTER(PagedKV)] + [_vp] * 7 + [_i, _i, _i, _vp, _vp, _vp]),
    "uocr_b200_rswa_decode_step_rope_paged": (_i, [C.POINTER(PagedKV)] + [_vp] * 4 + [C.c_float] + [_vp] * 4 +
                                              [_i, _i, _i, _vp, _vp, _vp]),
    "uocr_b200_rswa_attention_batch_paged_noalloc": (_i, [C.POINTER(PagedKV)] + [_vp] * 4 + [_i, _i, _vp, _vp]),
    "uocr_b200_rswa_attention_ragged_f32": (_i, [_vp] * 5 + [_i] * 5 + [_vp, _vp, _vp]),
    "uocr_b200_rswa_attention_ragged_paged": (_i, [C.POINTER(PagedKV)] + [_vp] * 4 + [_i, _i, _vp, _vp, _vp]),
    "uocr_b200_rswa_attention_f32": (_i, [_vp] * 3 + [_i, _vp] + [_i] * 6 + [_vp, _vp, _vp]),
    "uocr_b200_rswa_attention_paged": (_i, [C.POINTER(PagedKV), _i, _vp, _i, _vp, _i, _vp] + [_i] * 4 + [_vp, _vp, _vp]),
    "uocr_b200_rswa_gather_paged": (_i, [C.POINTER(PagedKV)] + [_vp] * 3 + [_i, _i, _vp, _vp, _i, _vp, _vp]),
    "uocr_b200_rswa_gather_heads_paged": (_i, [C.POINTER(PagedKV)] + [_vp] * 3 + [_i, _i, _vp, _vp, _vp, _vp]),
}


_HOST_SYMBOLS = [
    "pool_create", "pool_destroy", "pool_reset", "pool_allocate", "pool_free", "pool_total", "pool_used",
    "pool_peak", "pool_num_free_blocks", "pool_fragmentation",
    "bm_create", "bm_destroy", "bm_acquire_prefix", "bm_release_prefix", "bm_allocate_ring", "bm_free_ring",
    "bm_live_prefixes", "bm_total_prefix_bytes", "bm_shared_prefix_bytes", "bm_peak_prefix_bytes", "bm_get_stats",
    "sched_create", "sched_destroy", "sched_add_request", "sched_build_batch", "sched_mark_prefilled",
    "sched_mark_prefilling", "sched_add_token", "sched_finish", "sched_state", "sched_num_outputs",
    "sched_has_work", "sched_running", "sched_get_stats",
    "cache_create", "cache_set_kv_dtype", "cache_destroy", "cache_reset", "cache_write_prefill",
    "cache_append_decode", "cache_attention", "cache_len", "cache_ring_pos", "cache_ring_started",
    "cache_capacity", "cache_prefill_len", "cache_keys", "cache_values", "cache_bytes",
]


def host_symbols():
    """Entry points of include/uocr_rswa_b200_host.h (host classes behind the C ABI)."""
    return ["uocr_b200_" + n for n in _HOST_SYMBOLS]


def declared_symbols():
    """Names of every function declared in include/uocr_rswa_b200.h (parsed from the header)."""
    import re
    out = []
    for name in ("uocr_rswa_b200.h", "uocr_rswa_b200_host.h"):
        text = open(os.path.join(ROOT, "include", name)).read()
        out += re.findall(r"UOCR_B200_API\s+[\w\s\*]+?\b(uocr_b200_\w+)\s*\(", text)
    return sorted(set(out))


def lib() -> C.CDLL:
    """Load the shared library (never builds it: a missing library is an error on a GPU box)."""
    global _LIB
    if _LIB is None:
        if not os.path.exists(LIB_PATH):
            raise FileNotFoundError(f"{LIB_PATH} is missing: run __graft_entry__.build() first "
                                    "(there is no Python or CPU fallback for the CUDA path)")
        L = C.CDLL(LIB_PATH, mode=os.RTLD_LOCAL)
        for name, (res, args) in _SIGS.items():
            f = getattr(L, name)
            f.restype, f.argtypes = res, args
        _LIB = L
    return _LIB


def check(status: int) -> None:
    if status != 0:
        L = lib()
        raise Error(status, f"{L.uocr_b200_status_string(status).decode()}: {L.uocr_b200_last_error().decode()}")


def _p(t):
    """Device (or host) address of a torch tensor / numpy array / None."""
    if t is None:
        return None
    if hasattr(t, "data_ptr"):
        return t.data_ptr()
    return t.ctypes.data


def stream_handle(stream=None):
    import torch
    s = stream if stream is not None else torch.cuda.current_stream()
    return s.cuda_stream


class Workspace:
    def __init__(self, max_rows: int):
        h = _vp()
        check(lib().uocr_b200_workspace_create(max_rows, C.byref(h)))
        self.h = h

    def status(self, stream=None) -> int:
        v = _i(0)
        check(lib().uocr_b200_workspace_status(self.h, stream_handle(stream), C.byref(v)))
        return v.value

    def set_timing(self, enabled: bool) -> None:
        check(lib().uocr_b200_workspace_set_timing(self.h, 1 if enabled else 0))

    def set_out_dtype(self, dtype: int) -> None:
        """F32 (default) or BF16: type of the `out` tensor of every attention call using this workspace."""
        check(lib().uocr_b200_workspace_set_out_dtype(self.h, dtype))

    def set_overlap(self, enabled: bool) -> None:
        check(lib().uocr_b200_workspace_set_overlap(self.h, 1 if enabled else 0))

    def set_wait_limit(self, polls: int) -> None:
        """Polls a tile wait may take before the warp gives up (0: every wait gives up at once)."""
        check(lib().uocr_b200_workspace_set_wait_limit(self.h, polls))

    def stream_read_gbs(self, stream=None) -> float:
        """Read-only HBM -> shared-memory streaming rate of this GPU in GB/s (bulk copies, one CTA per SM)."""
        v = C.c_double(0)
        check(lib().uocr_b200_workspace_stream_read_gbs(self.h, stream_handle(stream), C.byref(v)))
        return v.value

    def last_kernel_ms(self) -> float:
        v = C.c_float(0)
        check(lib().uocr_b200_workspace_last_kernel_ms(self.h, C.byref(v)))
        return v.value

    def close(self):
        if self.h:
            lib().uocr_b200_workspace_destroy(self.h)
            self.h = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


def host_classes():
    """ctypes table + object wrappers over this library's host classes (MemoryPool, BlockManager,
    ContinuousBatchScheduler, RSWACache): see host_classes.py."""
    import importlib.util
    import sys
    name = "uocr_b200_host_classes"
    if name not in sys.modules:
        spec = importlib.util.spec_from_file_location(name, os.path.join(HERE, "host_classes.py"))
        mod = importlib.util.module_from_spec(spec)
        sys.modules[name] = mod
        spec.loader.exec_module(mod)
    lib()  # a missing library is an error
    return sys.modules[name].FunctionTable(LIB_PATH, "uocr_b200")


def launch_count() -> int:
    return int(lib().uocr_b200_launch_count())


class PagedLayer:
    """Device storage of one layer's paged KV plus the descriptor the C ABI takes."""

    def __init__(self, num_blocks, kv_heads, head_dim, dtype, table, device="cuda"):
        import torch
        self.dtype = dtype
        tdt = torch.bfloat16 if dtype == BF16 else torch.float32
        shape = (num_blocks, kv_heads, BLOCK_TOKENS, head_dim)
        self.k = torch.zeros(shape, dtype=tdt, device=device)
        self.v = torch.zeros(shape, dtype=tdt, device=device)
        self.table = table  # int32 [slots, stride], shared between layers
        self.desc = PagedKV(self.k.data_ptr(), self.v.data_ptr(), table.data_ptr(), table.shape[1],
                            num_blocks, kv_heads, head_dim, dtype)

    def ref(self):
        return C.byref(self.desc)


# ---- thin call wrappers (torch tensors in, status checked) ---------------------------------------

def append_decode_batch_paged(layer, k, v, d_len, d_ring, d_prefill, d_slots, batch, window, ws=None, stream=None):
    check(lib().uocr_b200_rswa_append_decode_batch_paged(layer.ref(), _p(k), _p(v), _p(d_len), _p(d_ring),
                                                          _p(d_prefill), _p(d_slots), batch, window,
                                                          ws.h if ws else None, stream_handle(stream)))


def layer_array(layers):
    """Contiguous array of uocr_b200_paged_kv for the entry points that take several layers at once."""
    arr = (PagedKV * len(layers))()
    for i, lay in enumerate(layers):
        arr[i] = lay.desc
    return arr


def append_decode_batch_paged_layers(layers, k, v, d_len, d_ring, d_prefill, d_slots, batch, window, ws=None, stream=None):
    """All layers of an append step in one launch: k, v are [L][rows >= batch][row], d_len / d_ring [L][slots]."""
    check(lib().uocr_b200_rswa_append_decode_batch_paged_layers(
        layer_array(layers), len(layers), _p(k), _p(v), k.stride(0), _p(d_len), _p(d_ring), d_len.stride(0), _p(d_prefill),
        _p(d_slots), batch, window, ws.h if ws else None, stream_handle(stream)))


def gather_paged_layers(layers, d_len, d_prefill, d_slots, n, capacity_rows, out_k, out_v, out_dtype, ws=None, stream=None):
    """All layers of a gather in one launch: out_k, out_v are [L][n][capacity_rows][row], d_len [L][slots]."""
    check(lib().uocr_b200_rswa_gather_paged_layers(
        layer_array(layers), len(layers), _p(d_len), d_len.stride(0), _p(d_prefill), _p(d_slots), n, capacity_rows,
        _p(out_k), _p(out_v), out_k.stride(0) * out_k.element_size(), out_dtype, ws.h if ws else None, stream_handle(stream)))


def attention_batch_paged(layer, q, d_len, d_prefill, d_slots, batch, heads, out, ws, stream=None):
    check(lib().uocr_b200_rswa_attention_batch_paged(layer.ref(), _p(q), _p(d_len), _p(d_prefill), _p(d_slots),
                                                      batch, heads, _p(out), ws.h, stream_handle(stream)))


def prefill_text_paged(layer, text_k, text_v, text_blocks, q, k, v, d_prefill, d_slots, d_pos, d_block0, total, window,
                       heads, out, ws, stream=None):
    check(lib().uocr_b200_rswa_prefill_text_paged(layer.ref(), _p(text_k), _p(text_v), text_blocks, _p(q), _p(k), _p(v),
                                                   _p(d_prefill), _p(d_slots), _p(d_pos), _p(d_block0), total, window,
                                                   heads, _p(out), ws.h, stream_handle(stream)))


def text_scatter_paged(layer, text_k, text_v, text_blocks, k, v, d_pos, d_block0, total, ws=None, stream=None):
    check(lib().uocr_b200_rswa_text_scatter_paged(layer.ref(), _p(text_k), _p(text_v), text_blocks, _p(k), _p(v),
                                                   _p(d_pos), _p(d_block0), total, ws.h if ws else None,
                                                   stream_handle(stream)))


def text_scatter_fill_paged(layer, text_k, text_v, text_blocks, k, v, d_slots, d_pos, d_block0, d_text_len, d_prefill,
                            d_len, d_ring, total, window, ws=None, stream=None):
    """text scatter + ring fill + cursor publication in one pass."""
    check(lib().uocr_b200_rswa_text_scatter_fill_paged(layer.ref(), _p(text_k), _p(text_v), text_blocks, _p(k), _p(v),
                                                        _p(d_slots), _p(d_pos), _p(d_block0), _p(d_text_len), _p(d_prefill),
                                                        _p(d_len), _p(d_ring), total, window, ws.h if ws else None,
                                                        stream_handle(stream)))


def prefill_attention_tc(layer, text_k, text_v, text_blocks, q, d_prefill, tiles, window, heads, out, ws, stream=None,
                         reuse_plan=False):
    """tiles: int32 numpy array [n, 6] = (row0, rows, slot, kind, pos0, block0) per query tile (host).
    reuse_plan: the workspace already holds the plan of exactly these tiles (prefill_plan_tc, or an earlier call)."""
    import numpy as np
    t = np.ascontiguousarray(tiles, dtype=np.int32)
    check(lib().uocr_b200_rswa_prefill_attention_tc(layer.ref(), _p(text_k), _p(text_v), text_blocks, _p(q),
                                                     _p(d_prefill), None if reuse_plan else t.ctypes.data, t.shape[0], window,
                                                     heads, _p(out), ws.h, stream_handle(stream)))


def prefill_plan_tc(tiles, d_prefill, window, ws, stream=None):
    """Uploads and orders the query tiles once; later prefill_attention_tc(..., reuse_plan=True) calls share the plan."""
    import numpy as np
    t = np.ascontiguousarray(tiles, dtype=np.int32)
    check(lib().uocr_b200_rswa_prefill_plan_tc(t.ctypes.data, t.shape[0], _p(d_prefill), window, ws.h, stream_handle(stream)))
    return lib().uocr_b200_workspace_prefill_plan_serial(ws.h)


def make_prefill_tiles(requests):
    """requests: iterable of (row0, n_rows, slot, kind, pos0, block0); cut into tiles of <= 128 rows."""
    import numpy as np
    out = []
    for row0, n, slot, kind, pos0, block0 in requests:
        for a in range(0, n, 128):
            out.append((row0 + a, min(128, n - a), slot, kind, pos0 + a, block0))
    return np.array(out, dtype=np.int32).reshape(-1, 6)


def ring_fill_paged(layer, text_k, text_v, text_blocks, d_slots, d_pos, d_block0, d_text_len, d_prefill, d_len, d_ring,
                    total, window, ws=None, stream=None):
    check(lib().uocr_b200_rswa_ring_fill_paged(layer.ref(), _p(text_k), _p(text_v), text_blocks, _p(d_slots), _p(d_pos),
                                                _p(d_block0), _p(d_text_len), _p(d_prefill), _p(d_len), _p(d_ring),
                                                total, window, ws.h if ws else None, stream_handle(stream)))


def decode_step_rope_paged(layer, q, k, v, d_positions, theta, d_len, d_ring, d_prefill, d_slots, batch, window, heads,
                           out, ws, stream=None):
    """rope + append + decode attention of one layer in one launch (q, k un-rotated)."""
    check(lib().uocr_b200_rswa_decode_step_rope_paged(layer.ref(), _p(q), _p(k), _p(v), _p(d_positions), float(theta),
                                                       _p(d_len), _p(d_ring), _p(d_prefill), _p(d_slots), batch, window,
                                                       heads, _p(out), ws.h, stream_handle(stream)))


def decode_step_paged(layer, q, k, v, d_len, d_ring, d_prefill, d_slots, batch, window, heads, out, ws, stream=None):
    """append + decode attention of one layer in one launch."""
    check(lib().uocr_b200_rswa_decode_step_paged(layer.ref(), _p(q), _p(k), _p(v), _p(d_len), _p(d_ring),
                                                  _p(d_prefill), _p(d_slots), batch, window, heads, _p(out), ws.h,
                                                  stream_handle(stream)))


def attention_batch_paged_noalloc(layer, q, d_len, d_prefill, d_slots, batch, heads, out, stream=None):
    """Same result as attention_batch_paged, scratch in the library's built-in device array."""
    check(lib().uocr_b200_rswa_attention_batch_paged_noalloc(layer.ref(), _p(q), _p(d_len), _p(d_prefill),
                                                              _p(d_slots), batch, heads, _p(out),
                                                              stream_handle(stream)))


def noalloc_status(stream=None) -> int:
    """Reads and clears the device status word of the allocation-free calls (synchronises the stream)."""
    v = _i(0)
    check(lib().uocr_b200_noalloc_status(stream_handle(stream), C.byref(v)))
    return v.value


def write_prefill_ragged_paged(layer, k, v, d_slots, d_pos, total, ws=None, stream=None):
    check(lib().uocr_b200_rswa_write_prefill_ragged_paged(layer.ref(), _p(k), _p(v), _p(d_slots), _p(d_pos), total,
                                                           ws.h if ws else None, stream_handle(stream)))


def attention_ragged_paged(layer, q, d_prefill, d_slots, d_pos, total, heads, out, ws, stream=None):
    check(lib().uocr_b200_rswa_attention_ragged_paged(layer.ref(), _p(q), _p(d_prefill), _p(d_slots), _p(d_pos),
                                                       total, heads, _p(out), ws.h, stream_handle(stream)))


def attention_paged(layer, slot, q, kv_len, d_len, prefill_len, d_prefill, seq, q_start, heads, causal, out, ws,
                    stream=None):
    check(lib().uocr_b200_rswa_attention_paged(layer.ref(), slot, _p(q), kv_len, _p(d_len), prefill_len,
                                                _p(d_prefill), seq, q_start, heads, 1 if causal else 0, _p(out),
                                                ws.h, stream_handle(stream)))


def gather_paged(layer, d_len, d_prefill, d_slots, n, capacity_rows, out_k, out_v, out_dtype, ws=None, stream=None):
    check(lib().uocr_b200_rswa_gather_paged(layer.ref(), _p(d_len), _p(d_prefill), _p(d_slots), n, capacity_rows,
                                             _p(out_k), _p(out_v), out_dtype, ws.h if ws else None,
                                             stream_handle(stream)))


def gather_heads_paged(layer, d_len, d_prefill, d_slots, n, capacity_rows, out_k, out_v, ws=None, stream=None):
    """fp32 out[n][kv_heads][capacity_rows][head_dim]: the layout of the reference's cache snapshots."""
    check(lib().uocr_b200_rswa_gather_heads_paged(layer.ref(), _p(d_len), _p(d_prefill), _p(d_slots), n, capacity_rows,
                                                   _p(out_k), _p(out_v), ws.h if ws else None, stream_handle(stream)))


def append_decode_batch_f32(k, v, kbase, vbase, d_len, d_ring, d_prefill, d_slots, batch, batch_cap, window,
                            kv_heads, head_dim, stream=None):
    check(lib().uocr_b200_rswa_append_decode_batch_f32(_p(k), _p(v), _p(kbase), _p(vbase), _p(d_len), _p(d_ring),
                                                        _p(d_prefill), _p(d_slots), batch, batch_cap, window,
                                                        kv_heads, head_dim, stream_handle(stream)))


def append_decode_f32(k, v, kcache, vcache, d_len, d_ring, prefill_len, window, kv_heads, head_dim, stream=None):
    check(lib().uocr_b200_rswa_append_decode_f32(_p(k), _p(v), _p(kcache), _p(vcache), _p(d_len), _p(d_ring),
                                                  prefill_len, window, kv_heads, head_dim, stream_handle(stream)))


def write_prefill_ragged_f32(k, v, kbase, vbase, d_slots, d_pos, total, batch_cap, kv_heads, head_dim, stream=None):
    check(lib().uocr_b200_rswa_write_prefill_ragged_f32(_p(k), _p(v), _p(kbase), _p(vbase), _p(d_slots), _p(d_pos),
                                                         total, batch_cap, kv_heads, head_dim, stream_handle(stream)))


def attention_batch_f32(q, kbase, vbase, d_len, d_slots, batch, batch_cap, heads, kv_heads, head_dim, out, ws,
                        stream=None):
    check(lib().uocr_b200_rswa_attention_batch_f32(_p(q), _p(kbase), _p(vbase), _p(d_len), _p(d_slots), batch,
                                                    batch_cap, heads, kv_heads, head_dim, _p(out), ws.h,
                                                    stream_handle(stream)))


def attention_ragged_f32(q, kbase, vbase, d_slots, d_pos, total, batch_cap, heads, kv_heads, head_dim, out, ws,
                         stream=None):
    check(lib().uocr_b200_rswa_attention_ragged_f32(_p(q), _p(kbase), _p(vbase), _p(d_slots), _p(d_pos), total,
                                                     batch_cap, heads, kv_heads, head_dim, _p(out), ws.h,
                                                     stream_handle(stream)))


def attention_f32(q, kcache, vcache, kv_len, d_len, seq, q_start, heads, kv_heads, head_dim, causal, out, ws,
                  stream=None):
    check(lib().uocr_b200_rswa_attention_f32(_p(q), _p(kcache), _p(vcache), kv_len, _p(d_len), seq, q_start, heads,
                                              kv_heads, head_dim, 1 if causal else 0, _p(out), ws.h,
                                              stream_handle(stream)))
