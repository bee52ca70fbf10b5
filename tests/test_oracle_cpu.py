"""CPU suite: pins the oracle against the reference's golden vectors and own CPU code, checks the
host-visible contracts, and that the shared library loads and exports every declared symbol."""
import hashlib
import json
import os
import re

import numpy as np
import pytest

from conftest import GOLDEN, ROOT, bits, glibc_uniform, golden_names


def test_oracle_matches_golden_vectors(oracle, golden):
    for name in golden_names(golden):
        x = golden[name + ".x"]
        s, d = oracle.nf4_quantize(x)
        assert np.array_equal(bits(s), bits(golden[name + ".nf4_scales"])), name
        assert np.array_equal(d, golden[name + ".nf4_data"]), name
        dq, c, d2 = oracle.nf4dq_quantize(x)
        assert bits(np.array([dq]))[0] == bits(golden[name + ".dq"])[0], name
        assert np.array_equal(c, golden[name + ".dq_codes"]), name
        assert np.array_equal(d2, golden[name + ".dq_data"]), name
        assert np.array_equal(bits(oracle.nf4_dequantize(s, d, x.size)), bits(golden[name + ".nf4_deq"])), name
        assert np.array_equal(bits(oracle.nf4dq_dequantize(dq, c, d2, x.size)), bits(golden[name + ".dq_deq"])), name


@pytest.mark.parametrize("seed", [12345, 54321])
def test_oracle_on_reference_test_fixture(oracle, seed):
    """The input of tests/quantization_cuda/test_nf4_cuda.cu / test_nf4_dq_cuda.cu, digests made by the reference."""
    with open(os.path.join(GOLDEN, "rand_fixture.json")) as f:
        want = json.load(f)[str(seed)]
    x = glibc_uniform(seed, 1 << 20)
    sha = lambda a: hashlib.sha256(np.ascontiguousarray(a).tobytes()).hexdigest()
    assert sha(x) == want["input_sha256"]
    s, d = oracle.nf4_quantize(x)
    assert sha(s) == want["nf4_scales_sha256"] and sha(d) == want["nf4_data_sha256"]
    dq, c, d2 = oracle.nf4dq_quantize(x)
    assert int(bits(np.array([dq]))[0]) == want["dq_bits"]
    assert sha(c) == want["dq_codes_sha256"] and sha(d2) == want["dq_data_sha256"]
    assert sha(oracle.nf4_dequantize(s, d, x.size)) == want["nf4_deq_sha256"]
    assert sha(oracle.nf4dq_dequantize(dq, c, d2, x.size)) == want["dq_deq_sha256"]


def test_oracle_matches_reference_cpu_library(oracle, ref_cpu):
    if ref_cpu is None:
        pytest.skip("oracle/_ref not built (reference tree absent)")
    rng = np.random.default_rng(3)
    for n in (1, 63, 65, 4097, 1 << 16):
        for scale in (1.0, 1e-4, 1e5):
            x = (rng.standard_normal(n) * scale).astype(np.float32)
            x[rng.integers(0, n, max(1, n // 40))] = 0
            a, b = oracle.nf4_quantize(x), ref_cpu.nf4_quantize(x)
            assert np.array_equal(bits(a[0]), bits(b[0])) and np.array_equal(a[1], b[1])
            a, b = oracle.nf4dq_quantize(x), ref_cpu.nf4dq_quantize(x)
            assert bits(np.array([a[0]]))[0] == bits(np.array([b[0]]))[0]
            assert np.array_equal(a[1], b[1]) and np.array_equal(a[2], b[2])


def test_nf4_threshold_table_in_kernel_header(oracle):
    """The 15 thresholds baked into the CUDA encoder are where the reference scan changes code."""
    src = open(os.path.join(ROOT, "bitsqueeze-llm_b200", "csrc", "bsq_device.cuh")).read()
    block = src[src.index("c_nf4_bucket_thr[32]"):]
    block = block[:block.index("};")]
    thr = [int(v, 16) for v in re.findall(r"0x[0-9a-fA-F]{8}", block)]
    assert len(thr) == 32
    # buckets without a threshold hold NaN (never +Inf: "v >= +Inf" is true for v = +Inf and would give code 16)
    assert 0x7F800000 not in thr
    real = sorted((np.array([t], np.uint32).view(np.float32)[0] for t in thr if t != 0x7FC00000))
    assert len(real) == 15
    for i, t in enumerate(real):
        below = np.nextafter(np.float32(t), np.float32(-np.inf))
        assert oracle.nf4_code(float(t)) == i + 1 and oracle.nf4_code(float(below)) == i


def test_e4m3_roundtrip_and_saturation(oracle):
    for c in range(0, 127):
        v = oracle.e4m3_decode(c)
        assert oracle.e4m3_encode(v) == c
    assert oracle.e4m3_encode(448.0) == 0x7E and oracle.e4m3_encode(1e9) == 0x7E
    assert oracle.e4m3_encode(float("inf")) == 0x7E and oracle.e4m3_encode(0.0) == 0
    assert oracle.e4m3_encode(2.0 ** -9) == 1 and oracle.e4m3_encode(2.0 ** -11) == 0


def test_topk_num_columns(oracle):
    # values of the configs: round(4096*0.01f)=41, 20/41 at 4096, 72/143 at 14336
    assert oracle.topk_num_columns(4096, 0.01) == 41
    assert oracle.topk_num_columns(4096, 0.005) == 20
    assert oracle.topk_num_columns(14336, 0.005) == 72 and oracle.topk_num_columns(14336, 0.01) == 143
    assert oracle.topk_num_columns(8, 0.01) == 1 and oracle.topk_num_columns(8, 0.0) == 0
    assert oracle.topk_num_columns(8, 1.0) == 8 and oracle.topk_num_columns(6, 0.5) == 3
    assert oracle.topk_num_columns(8, 1.5) == 0xFFFFFFFF


def test_topk_order_ties_and_nan(oracle):
    x = np.array([[1.0, -3.0, 3.0, 0.0, -0.0, np.nan, 2.0, -3.0],
                  [np.nan, np.nan, 0.5, np.nan, -np.inf, 0.5, np.nan, np.nan]], np.float32)
    idx, val, z = oracle.topk_rows(x, 4, zero_selected=True)
    assert idx[0].tolist() == [1, 2, 7, 6]                 # |3| ties by ascending column, then 2
    assert val[0].tolist() == [-3.0, 3.0, -3.0, 2.0]
    assert idx[1].tolist() == [4, 2, 5, 0]                 # inf, the two 0.5 by column, then first NaN
    assert np.isnan(val[1][3]) and val[1][0] == -np.inf
    assert z[0].tolist()[:3] == [1.0, 0.0, 0.0] and z[0][6] == 0.0 and z[0][7] == 0.0
    # properties the reference's own tests assert (tests/topk_cuda/test_topk_cuda_extraction.cpp:132-162)
    rng = np.random.default_rng(5)
    m = rng.standard_normal((3, 6)).astype(np.float32)
    idx, val, _ = oracle.topk_rows(m, 3)
    for r in range(3):
        assert len(set(idx[r].tolist())) == 3
        assert np.array_equal(val[r], m[r, idx[r]])
        assert set(idx[r].tolist()) == set(np.argsort(-np.abs(m[r]), kind="stable")[:3].tolist())


def test_compress_nosvd_layout_and_roundtrip(oracle):
    rows, cols = 64, 256
    rng = np.random.default_rng(11)
    x = rng.standard_normal((rows, cols)).astype(np.float32)
    x[:, 3] *= 50
    p = oracle.compress_nosvd(x, 0.05, 0.10, 10)
    ko, ke = 13, 26
    nb = rows * cols // 64
    assert p.size == 200 + (48 + nb + rows * cols // 2) + (8 + rows * ko * 6) + (8 + rows * ke * 6)
    assert int(np.frombuffer(p[40:44].tobytes(), np.uint32)[0]) == 6          # outlier + error flags
    y = oracle.decompress_nosvd(p, rows, cols)
    # outliers restored exactly, error entries corrected: residual error is small
    assert np.linalg.norm(y - x) / np.linalg.norm(x) < 0.05
    p2 = oracle.compress_nosvd(x, 0.0, 0.0, -1)                                  # dense FP32 section
    assert p2.size == 200 + rows * cols * 4
    assert np.array_equal(oracle.decompress_nosvd(p2, rows, cols), x)


def test_library_exports_every_declared_symbol(pkg, lib):
    header = open(os.path.join(ROOT, "include", "bitsqz_llm_c.h")).read()
    declared = set(re.findall(r"\b(bsq_[a-z0-9_]+)\s*\(", header))
    assert declared == set(pkg.SIGNATURES), declared ^ set(pkg.SIGNATURES)
    for name in declared:
        assert getattr(lib, name) is not None
    import ctypes
    raw = ctypes.CDLL(pkg.LIB_PATH)
    for sym in pkg.CXX_SYMBOLS:                 # the reference's mangled C++ interface (drop-in relink)
        assert getattr(raw, sym) is not None
    assert b"sm_100a" in lib.bsq_build_info()


def test_host_only_entry_points(pkg, lib):
    """Calls that need no GPU: k computation, packed-size / load validation, argument rejection."""
    assert lib.bsq_topk_num_columns(4096, 0.01) == 41 and lib.bsq_topk_num_columns(4096, 2.0) == -1
    assert lib.bsq_get_packed_size(None) == 0
    assert lib.bsq_load_from_buffer(None, 0) is None
    short = np.zeros(100, np.uint8)
    assert lib.bsq_load_from_buffer(short.ctypes.data, short.size) is None
    hdr = pkg.Array()
    hdr.num_rows, hdr.num_columns, hdr.num_elements = 2, 8, 16
    hdr.section_direct.offset, hdr.section_direct.size, hdr.section_direct.storage = 0, 64, pkg.SECTION_FP32
    buf = np.zeros(264, np.uint8)
    buf[:200] = np.frombuffer(bytes(hdr), np.uint8)
    h = lib.bsq_load_from_buffer(buf.ctypes.data, buf.size)
    assert h is not None and lib.bsq_get_packed_size(h) == 264
    lib.bsq_free(h)
    assert lib.bsq_load_from_buffer(buf.ctypes.data, 263) is None          # truncated payload
    hdr.section_direct.storage = 9                                           # unknown storage kind
    buf[:200] = np.frombuffer(bytes(hdr), np.uint8)
    assert lib.bsq_load_from_buffer(buf.ctypes.data, buf.size) is None
    # initialisers reject bad arguments before touching the device (src/bitsqz_llm.cu:796-804)
    assert lib.bsq_compress_initialize(0, 8, 0.0, 0.0, -1, 1, -1, -1, 11, 1) == 1
    assert lib.bsq_compress_initialize(8, 8, 1.5, 0.0, -1, 1, -1, -1, 11, 1) == 1
    assert lib.bsq_compress_initialize(8, 8, 0.0, 0.0, -1, 1, -1, -1, 0, 1) == 1     # Q8_0 is not accepted
    assert lib.bsq_compress_initialize(8, 8, 0.0, 0.0, -1, 0, -1, -1, 11, 1) == 1    # niters < 1
    assert lib.bsq_compress_initialize(8, 8, 0.0, 0.0, -1, 1, -1, -1, 11, 7) == 1    # bad location
    assert lib.bsq_decompress_initialize(8, 0, 0.0, 0.0, -1, -1, -1, 11) == 1
