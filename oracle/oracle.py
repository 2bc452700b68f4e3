"""TEST INFRASTRUCTURE ONLY: ctypes driver for the CPU oracle of the R-SWA KV-cache path.

Two interchangeable back ends export the same C function set:

* ``load("orc")`` -- ``oracle/librswa_oracle.so``, the plain-C restatement (``rswa_oracle.c``);
* ``load("ref")`` -- ``oracle/_ref/libuocr_ref.so``, the unmodified reference sources compiled by
  ``oracle/Makefile`` (only present where the reference checkout was available at build time).

Only the tests, the smoke check and the benchmark's CPU-baseline leg import this module; the shipped
library never does.
"""
from __future__ import annotations

import ctypes as C
import os
import subprocess

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
_PATHS = {
    "orc": os.path.join(HERE, "librswa_oracle.so"),
    "ref": os.path.join(HERE, "_ref", "libuocr_ref.so"),
}
_f32p = C.POINTER(C.c_float)
_i32p = C.POINTER(C.c_int)


def reference_root() -> str:
    """Where the reference checkout lies: $UOCR_REFERENCE_ROOT, else a directory `reference` beside
    this repository (absent on a machine that only runs the prebuilt files)."""
    return os.environ.get("UOCR_REFERENCE_ROOT") or os.path.join(os.path.dirname(os.path.dirname(HERE)), "reference")


def build(ref_root: str | None = None) -> None:
    """Compile the restatement and, when the reference checkout is present, the reference itself."""
    ref_root = ref_root or reference_root()
    subprocess.check_call(["make", "-s", "-C", HERE, "all"])
    if os.path.isdir(os.path.join(ref_root, "src", "scheduler")):
        subprocess.check_call(["make", "-s", "-C", HERE, "ref", f"REF={ref_root}"])


def available(kind: str) -> bool:
    return os.path.exists(_PATHS[kind])


def _host_classes():
    """The generic ctypes table and object wrappers live with the CUDA library's Python plumbing; the
    checker libraries export the same function set under their own prefixes."""
    import importlib.util
    import sys
    name = "uocr_b200_host_classes"
    if name in sys.modules:
        return sys.modules[name]
    path = os.path.join(os.path.dirname(HERE), "unlimited-ocr.cpp_b200", "host_classes.py")
    spec = importlib.util.spec_from_file_location(name, path)
    mod = importlib.util.module_from_spec(spec)
    sys.modules[name] = mod
    spec.loader.exec_module(mod)
    return mod


_hc = _host_classes()
BMStats, SchedStats = _hc.BMStats, _hc.SchedStats


class Oracle(_hc.FunctionTable):
    """Function table of one checker back end (prefix ``orc`` or ``ref``)."""

    def __init__(self, kind: str):
        super().__init__(_PATHS[kind], kind)
        self.kind = kind


_CACHE = {}


def load(kind: str = "orc") -> Oracle:
    if kind not in _CACHE:
        if kind == "orc" and not available("orc"):
            build()
        _CACHE[kind] = Oracle(kind)
    return _CACHE[kind]
