"""ctypes driver for the host classes behind the C ABI (include/uocr_rswa_b200_host.h): MemoryPool,
BlockManager, ContinuousBatchScheduler and the device-backed RSWACache of libuocr_rswa_b200.so, with
small object wrappers.  The same table binds any library that exports the same function set under
another prefix, which is how the tests run one script against this library and against a checker.
"""
from __future__ import annotations

import ctypes as C
import os

import numpy as np

_f32p = C.POINTER(C.c_float)
_i32p = C.POINTER(C.c_int)


class BMStats(C.Structure):
    _fields_ = [("prefix_live_bytes", C.c_uint64), ("prefix_peak_bytes", C.c_uint64),
                ("prefix_shared_bytes", C.c_uint64), ("ring_live_bytes", C.c_uint64),
                ("ring_peak_bytes", C.c_uint64), ("prefix_fragmentation", C.c_double),
                ("ring_fragmentation", C.c_double), ("live_prefixes", C.c_uint64)]

    def as_tuple(self):
        return tuple(getattr(self, f) for f, _ in self._fields_)


class SchedStats(C.Structure):
    _fields_ = [("total_requests", C.c_uint64), ("finished_requests", C.c_uint64),
                ("prefill_tokens", C.c_uint64), ("decode_tokens", C.c_uint64),
                ("waiting", C.c_uint64), ("running", C.c_uint64), ("last_batch_size", C.c_double)]

    def as_tuple(self):
        return tuple(getattr(self, f) for f, _ in self._fields_)


def _fp(a: np.ndarray):
    assert a.dtype == np.float32 and a.flags.c_contiguous
    return a.ctypes.data_as(_f32p)


class FunctionTable:
    """ctypes bindings of one shared library exporting `<prefix>_<name>` for the host-class function
    set (cache_*, pool_*, bm_*, sched_*): the CUDA library's own host classes
    (include/uocr_rswa_b200_host.h, prefix `uocr_b200`), or any other library with the same set."""

    def __init__(self, path: str, prefix: str):
        self.path, self.prefix = path, prefix
        self.lib = C.CDLL(path, mode=os.RTLD_LOCAL)
        p = prefix + "_"
        L = self.lib

        def fn(name, res, args):
            f = getattr(L, p + name, None)
            if f is None:  # optional entry (e.g. the timed decode leg)
                return
            f.restype = res
            f.argtypes = args
            setattr(self, name, f)

        vp = C.c_void_p
        fn("f32_to_bf16", C.c_uint16, [C.c_float])
        fn("bf16_to_f32", C.c_float, [C.c_uint16])
        fn("round_bf16_inplace", None, [_f32p, C.c_size_t])
        fn("rope", None, [_f32p, _f32p, _i32p, C.c_int, C.c_int, C.c_int, C.c_int, C.c_float])
        fn("cache_create", vp, [C.c_int] * 4)
        fn("cache_destroy", None, [vp])
        fn("cache_reset", C.c_int, [vp, C.c_int])
        fn("cache_write_prefill", C.c_int, [vp, C.c_int, _f32p, _f32p, C.c_int])
        fn("cache_append_decode", None, [vp, C.c_int, _f32p, _f32p])
        fn("cache_attention", C.c_int, [vp, C.c_int, _f32p, C.c_int, C.c_int, _f32p, C.c_int, C.c_int])
        for g in ("len", "ring_pos", "ring_started"):
            fn("cache_" + g, C.c_int, [vp, C.c_int])
        fn("cache_capacity", C.c_int, [vp])
        fn("cache_prefill_len", C.c_int, [vp])
        fn("cache_keys", _f32p, [vp, C.c_int])
        fn("cache_values", _f32p, [vp, C.c_int])
        fn("cache_bytes", C.c_size_t, [vp])
        fn("pool_create", vp, [C.c_size_t, C.c_size_t])
        fn("pool_destroy", None, [vp])
        fn("pool_reset", None, [vp])
        fn("pool_allocate", C.c_int64, [vp, C.c_size_t, C.c_size_t])
        fn("pool_free", None, [vp, C.c_int64, C.c_size_t])
        for g in ("total", "used", "peak", "num_free_blocks"):
            fn("pool_" + g, C.c_size_t, [vp])
        fn("pool_fragmentation", C.c_double, [vp])
        fn("bm_create", vp, [C.c_size_t, C.c_size_t])
        fn("bm_destroy", None, [vp])
        fn("bm_acquire_prefix", C.c_int64, [vp, C.c_char_p, C.c_int, C.c_size_t, _i32p])
        fn("bm_release_prefix", None, [vp, C.c_char_p])
        fn("bm_allocate_ring", C.c_int64, [vp, C.c_size_t])
        fn("bm_free_ring", None, [vp, C.c_int64, C.c_size_t])
        for g in ("live_prefixes", "total_prefix_bytes", "shared_prefix_bytes", "peak_prefix_bytes"):
            fn("bm_" + g, C.c_uint64, [vp])
        fn("bm_get_stats", None, [vp, C.POINTER(BMStats)])
        fn("sched_create", vp, [C.c_int, C.c_int])
        fn("sched_destroy", None, [vp])
        fn("sched_add_request", C.c_int, [vp, C.c_int, C.c_int])
        fn("sched_build_batch", None, [vp, _i32p, _i32p, _i32p, _i32p, C.c_int])
        fn("sched_mark_prefilled", None, [vp, C.c_int])
        fn("sched_mark_prefilling", None, [vp, C.c_int])
        fn("sched_add_token", C.c_int, [vp, C.c_int, C.c_int])
        fn("sched_finish", None, [vp, C.c_int])
        fn("sched_state", C.c_int, [vp, C.c_int])
        fn("sched_num_outputs", C.c_int, [vp, C.c_int])
        fn("sched_has_work", C.c_int, [vp])
        fn("sched_running", C.c_int, [vp, _i32p, C.c_int])
        fn("sched_get_stats", None, [vp, C.POINTER(SchedStats)])
        fn("decode_bench", C.c_double, [C.c_int] * 5 + [_i32p, _i32p, C.c_int, C.c_int, C.c_uint64,
                                                       C.POINTER(C.c_double), _i32p])

    # ---- convenience object wrappers ---------------------------------------------------------
    def Cache(self, layers, kv_heads, head_dim, window):
        return _Cache(self, layers, kv_heads, head_dim, window)

    def Pool(self, nbytes, alignment=256):
        return _Pool(self, nbytes, alignment)

    def BlockManager(self, prefix_bytes, ring_bytes):
        return _BM(self, prefix_bytes, ring_bytes)

    def Scheduler(self, max_batch=16, min_batch=4):
        return _Sched(self, max_batch, min_batch)

    def apply_rope(self, q: np.ndarray, k, positions: np.ndarray, n_heads: int, n_kv_heads: int, head_dim: int,
                   theta: float):
        """RoPE on copies of q [seq, n_heads*hd] and k [seq, n_kv_heads*hd] (k may be None)."""
        q2 = np.ascontiguousarray(q, dtype=np.float32).copy()
        k2 = None if k is None else np.ascontiguousarray(k, dtype=np.float32).copy()
        pos = np.ascontiguousarray(positions, dtype=np.int32)
        self.rope(_fp(q2), _fp(k2) if k2 is not None else None, pos.ctypes.data_as(_i32p), int(pos.shape[0]), n_heads,
                  n_kv_heads, head_dim, theta)
        return q2, k2

    def round_bf16(self, x: np.ndarray) -> np.ndarray:
        y = np.ascontiguousarray(x, dtype=np.float32).copy()
        self.round_bf16_inplace(_fp(y.reshape(-1)), y.size)
        return y

    def run_decode_bench(self, prefix_len, pos, layers, kv_heads, head_dim, window, steps,
                         threads=0, seed=1234):
        pl = np.ascontiguousarray(prefix_len, dtype=np.int32)
        ps = np.ascontiguousarray(pos, dtype=np.int32)
        cs = C.c_double(0)
        used = C.c_int(0)
        sec = self.decode_bench(len(pl), layers, kv_heads, head_dim, window,
                                pl.ctypes.data_as(_i32p), ps.ctypes.data_as(_i32p), steps, threads,
                                seed, C.byref(cs), C.byref(used))
        return sec, used.value, cs.value


class _Cache:
    def __init__(self, o, layers, kv_heads, head_dim, window):
        self.o, self.layers, self.kv_heads, self.head_dim, self.window = o, layers, kv_heads, head_dim, window
        self.h = o.cache_create(layers, kv_heads, head_dim, window)

    def __del__(self):
        if getattr(self, "h", None):
            self.o.cache_destroy(self.h)
            self.h = None

    @property
    def row(self):
        return self.kv_heads * self.head_dim

    def reset(self, P):
        return self.o.cache_reset(self.h, P)

    def write_prefill(self, layer, k, v):
        k = np.ascontiguousarray(k, np.float32)
        v = np.ascontiguousarray(v, np.float32)
        seq = k.size // self.row
        return self.o.cache_write_prefill(self.h, layer, _fp(k.reshape(-1)), _fp(v.reshape(-1)), seq)

    def append_decode(self, layer, k, v):
        k = np.ascontiguousarray(k, np.float32)
        v = np.ascontiguousarray(v, np.float32)
        self.o.cache_append_decode(self.h, layer, _fp(k.reshape(-1)), _fp(v.reshape(-1)))

    def attention(self, layer, q, q_start, heads, causal):
        q = np.ascontiguousarray(q, np.float32).reshape(-1, heads * self.head_dim)
        out = np.full_like(q, np.nan)
        rc = self.o.cache_attention(self.h, layer, _fp(q.reshape(-1)), q.shape[0], q_start,
                                    _fp(out.reshape(-1)), heads, 1 if causal else 0)
        assert rc == 0
        return out

    def len(self, layer):
        return self.o.cache_len(self.h, layer)

    def ring_pos(self, layer):
        return self.o.cache_ring_pos(self.h, layer)

    def ring_started(self, layer):
        return bool(self.o.cache_ring_started(self.h, layer))

    def capacity(self):
        return self.o.cache_capacity(self.h)

    def prefill_len(self):
        return self.o.cache_prefill_len(self.h)

    def bytes(self):
        return self.o.cache_bytes(self.h)

    def _arr(self, ptr, n_rows):
        n = n_rows * self.row
        if n == 0:
            return np.zeros((0, self.row), np.float32)
        return np.ctypeslib.as_array(ptr, shape=(n,)).reshape(n_rows, self.row).copy()

    def keys(self, layer, full=False):
        """Logical [len, kv_heads*head_dim] view (or all `capacity` rows with full=True)."""
        return self._arr(self.o.cache_keys(self.h, layer), self.capacity() if full else self.len(layer))

    def values(self, layer, full=False):
        return self._arr(self.o.cache_values(self.h, layer), self.capacity() if full else self.len(layer))


class _Pool:
    def __init__(self, o, nbytes, alignment):
        self.o = o
        self.h = o.pool_create(nbytes, alignment)

    def __del__(self):
        if getattr(self, "h", None):
            self.o.pool_destroy(self.h)
            self.h = None

    def allocate(self, n, alignment=0):
        return self.o.pool_allocate(self.h, n, alignment)

    def free(self, off, n):
        self.o.pool_free(self.h, off, n)

    def reset(self):
        self.o.pool_reset(self.h)

    def state(self):
        return (self.o.pool_total(self.h), self.o.pool_used(self.h), self.o.pool_peak(self.h),
                self.o.pool_num_free_blocks(self.h), self.o.pool_fragmentation(self.h))


class _BM:
    def __init__(self, o, prefix_bytes, ring_bytes):
        self.o = o
        self.h = o.bm_create(prefix_bytes, ring_bytes)

    def __del__(self):
        if getattr(self, "h", None):
            self.o.bm_destroy(self.h)
            self.h = None

    def acquire_prefix(self, key, prefill_len, nbytes):
        rc = C.c_int(0)
        off = self.o.bm_acquire_prefix(self.h, key.encode(), prefill_len, nbytes, C.byref(rc))
        return off, rc.value

    def release_prefix(self, key):
        self.o.bm_release_prefix(self.h, key.encode())

    def allocate_ring(self, n):
        return self.o.bm_allocate_ring(self.h, n)

    def free_ring(self, off, n):
        self.o.bm_free_ring(self.h, off, n)

    def stats(self):
        s = BMStats()
        self.o.bm_get_stats(self.h, C.byref(s))
        return s.as_tuple()

    def counters(self):
        return (self.o.bm_live_prefixes(self.h), self.o.bm_total_prefix_bytes(self.h),
                self.o.bm_shared_prefix_bytes(self.h), self.o.bm_peak_prefix_bytes(self.h))


class _Sched:
    def __init__(self, o, max_batch, min_batch):
        self.o = o
        self.h = o.sched_create(max_batch, min_batch)

    def __del__(self):
        if getattr(self, "h", None):
            self.o.sched_destroy(self.h)
            self.h = None

    def add_request(self, prompt_len, max_new):
        return self.o.sched_add_request(self.h, prompt_len, max_new)

    def build_batch(self, cap=4096):
        pf = (C.c_int * cap)()
        dc = (C.c_int * cap)()
        npf, ndc = C.c_int(0), C.c_int(0)
        self.o.sched_build_batch(self.h, pf, C.byref(npf), dc, C.byref(ndc), cap)
        return list(pf[:npf.value]), list(dc[:ndc.value])

    def mark_prefilled(self, i):
        self.o.sched_mark_prefilled(self.h, i)

    def mark_prefilling(self, i):
        self.o.sched_mark_prefilling(self.h, i)

    def add_token(self, i, tok=0):
        return bool(self.o.sched_add_token(self.h, i, tok))

    def finish(self, i):
        self.o.sched_finish(self.h, i)

    def state(self, i):
        return self.o.sched_state(self.h, i)

    def num_outputs(self, i):
        return self.o.sched_num_outputs(self.h, i)

    def has_work(self):
        return bool(self.o.sched_has_work(self.h))

    def running(self, cap=4096):
        buf = (C.c_int * cap)()
        n = self.o.sched_running(self.h, buf, cap)
        return list(buf[:n])

    def stats(self):
        s = SchedStats()
        self.o.sched_get_stats(self.h, C.byref(s))
        return s.as_tuple()
