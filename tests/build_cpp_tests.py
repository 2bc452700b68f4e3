"""Builds the C++ test binaries (tests/_bin/, build output):

* test_host_api             -- tests/cpp/test_host_api.cu, this repository's own GPU test of the C++ host API
* (oracle/_ref/) ref_kv_ring_buffer_on_b200 -- the REFERENCE's own tests/test_kv_ring_buffer.cpp and
  tests/test_main.cpp, compiled unmodified from the reference checkout against this library's headers
  and linked to this library; only built where the checkout is present, never copied.
"""
import os
import subprocess

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
PKG = os.path.join(ROOT, "unlimited-ocr.cpp_b200")
BIN = os.path.join(ROOT, "tests", "_bin")
REF_BIN = os.path.join(ROOT, "oracle", "_ref", "ref_kv_ring_buffer_on_b200")
HOST_API_BIN = os.path.join(BIN, "test_host_api")


def build(ref_root=None):
    from oracle import oracle
    ref_root = ref_root or oracle.reference_root()
    os.makedirs(BIN, exist_ok=True)
    subprocess.check_call([
        "nvcc", "-gencode", "arch=compute_100a,code=sm_100a", "-O1", "-std=c++17",
        "-I", os.path.join(ROOT, "include"), "-I", os.path.join(PKG, "include"), "-I", os.path.join(ROOT, "oracle"),
        os.path.join(ROOT, "tests", "cpp", "test_host_api.cu"), "-o", HOST_API_BIN,
        "-L", PKG, "-luocr_rswa_b200", "-L", os.path.join(ROOT, "oracle"), "-lrswa_oracle",
        "-Xlinker", "-rpath,$ORIGIN/../../unlimited-ocr.cpp_b200", "-Xlinker", "-rpath,$ORIGIN/../../oracle"])
    tests = os.path.join(ref_root, "tests")
    if os.path.isfile(os.path.join(tests, "test_kv_ring_buffer.cpp")):
        os.makedirs(os.path.dirname(REF_BIN), exist_ok=True)
        subprocess.check_call([
            "g++", "-std=c++17", "-O1", "-I", os.path.join(PKG, "include"), "-I", os.path.join(ROOT, "include"),
            "-I", tests, os.path.join(tests, "test_main.cpp"), os.path.join(tests, "test_kv_ring_buffer.cpp"),
            "-o", REF_BIN, "-L", PKG, "-luocr_rswa_b200", "-Wl,-rpath,$ORIGIN/../../unlimited-ocr.cpp_b200"])


if __name__ == "__main__":
    build()
