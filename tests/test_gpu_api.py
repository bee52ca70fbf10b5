"""GPU parity and contract tests of the public interface (bitsqz_llm_compress / decompress and the
lifecycle rules), through the C ABI.  The no-SVD configurations are byte-compared with the CPU
oracle's packed object; the lifecycle and negative cases follow the reference's integration tests
(tests/bitsqz_llm/test_quantization.cpp:129-230,379-430)."""
import ctypes as C

import numpy as np
import pytest

from conftest import bits, make_c2_like

pytestmark = pytest.mark.gpu
torch = pytest.importorskip("torch")


def compress_bytes(pkg, lib, x, outlier, err, q, location, ranks=-1, niters=1, uv=-1, s=-1):
    rows, cols = x.shape
    assert lib.bsq_compress_initialize(rows, cols, outlier, err, ranks, niters, uv, s, q, location) == 0
    if location == pkg.INPUT_HOST:
        res = pkg.compress_to_bytes(x.ctypes.data)
    else:
        d_x = torch.from_numpy(x).cuda()
        keep = d_x.clone()
        res = pkg.compress_to_bytes(d_x.data_ptr())
        torch.cuda.synchronize()
        assert torch.equal(d_x.view(torch.int32), keep.view(torch.int32)), "device input was modified"
    assert res is not None
    return res


def decompress(pkg, lib, packed, rows, cols, outlier, err, q, ranks=-1, uv=-1, s=-1):
    assert lib.bsq_decompress_initialize(rows, cols, outlier, err, ranks, uv, s, q) == 0
    d_y = torch.full((rows, cols), 123.0, dtype=torch.float32, device="cuda")
    assert pkg.decompress_packed(packed, d_y.data_ptr(), rows * cols) == 0
    torch.cuda.synchronize()
    return d_y.cpu().numpy()


def same_bytes(packed, want):
    got = packed.copy()
    got[192:200] = 0
    return got.size == want.size and np.array_equal(got, want)


CASES = [
    # rows, cols, outlier, error, method, location          (benchmark configurations 1 and 2 first)
    (1024, 1024, 0.0, 0.0, 11, 0),
    (4096, 4096, 0.01, 0.0, 10, 1),
    (512, 8192, 0.0, 0.0, 11, 1),
    (512, 8192, 0.0, 0.10, 11, 1),
    (512, 8192, 0.05, 0.0, 10, 1),
    (512, 8192, 0.05, 0.10, 10, 0),
    (100, 200, 0.03, 0.02, 10, 1),          # blocks straddle rows, generic top-k
    (64, 1000, 0.01, 0.0, 11, 1),
    (33, 4096, 0.005, 0.01, 11, 1),
    (192, 14336, 0.005, 0.0, 10, 1),        # row length of benchmark configuration 5 (k = 72): 8 warps per row
    (192, 14336, 0.005, 0.01, 11, 1),       # ... with error correction (k = 143)
    (128, 512, 0.0, 0.0, -1, 1),            # dense FP32 section
    (128, 512, 0.02, 0.0, -1, 0),
]


@pytest.mark.parametrize("case", CASES)
def test_nosvd_compress_bytes_and_roundtrip(pkg, lib, oracle, case):
    rows, cols, outlier, err, q, loc = case
    if (rows, cols) == (1024, 1024):
        x = np.random.default_rng(1).standard_normal((rows, cols)).astype(np.float32)
    else:
        x = make_c2_like(rows, cols, 2)
    hdr, packed = compress_bytes(pkg, lib, x, outlier, err, q, loc)
    want = oracle.compress_nosvd(x, outlier, err, q)
    assert same_bytes(packed, want)
    assert hdr.num_rows == rows and hdr.num_columns == cols and hdr.num_elements == rows * cols
    assert hdr.effective_rank == 0 and hdr.quantization_only_format == q
    y = decompress(pkg, lib, packed, rows, cols, outlier, err, q)
    assert np.array_equal(bits(y), bits(oracle.decompress_nosvd(want, rows, cols)))
    lib.bsq_compress_release()
    lib.bsq_decompress_release()


def test_profile_is_filled(pkg, lib):
    x = make_c2_like(256, 4096, 3)
    assert lib.bsq_compress_initialize(256, 4096, 0.01, 0.0, -1, 1, -1, -1, 10, 1) == 0
    d_x = torch.from_numpy(x).cuda()
    prof = pkg.Profile()
    res = pkg.compress_to_bytes(d_x.data_ptr(), prof)
    assert res is not None
    assert prof.topk_separation_latency_ms > 0.0 and prof.other_latency_ms >= 0.0
    assert prof.svd_lowrank_cuda_latency_ms == 0.0
    lib.bsq_compress_release()


def test_lifecycle_and_negative_paths(pkg, lib):
    rows, cols = 128, 512
    x = make_c2_like(rows, cols, 5)
    d_x = torch.from_numpy(x).cuda()
    d_y = torch.zeros_like(d_x)
    out = C.c_void_p(None)
    lib.bsq_compress_release()
    lib.bsq_decompress_release()
    # before initialisation
    assert lib.bsq_compress(d_x.data_ptr(), C.byref(out), None) == 1 and not out.value
    assert lib.bsq_compress_initialize(rows, cols, 0.05, 0.0, -1, 1, -1, -1, 10, 1) == 0
    assert lib.bsq_compress(None, C.byref(out), None) == 1
    assert lib.bsq_compress(d_x.data_ptr(), None, None) == 1
    res = pkg.compress_to_bytes(d_x.data_ptr())
    assert res is not None
    hdr, packed = res
    assert packed.size > 200 and hdr.flags == pkg.FLAG_OUTLIER
    # *out must be null on entry and stays untouched on failure
    sentinel = C.c_void_p(12345)
    assert lib.bsq_compress(d_x.data_ptr(), C.byref(sentinel), None) == 1 and sentinel.value == 12345
    # decompress before initialisation fails; the compress runtime survives that
    assert pkg.decompress_packed(packed, d_y.data_ptr(), rows * cols) == 1
    assert lib.bsq_decompress_initialize(rows, cols, 0.05, 0.0, -1, -1, -1, 10) == 0
    assert pkg.decompress_packed(packed, d_y.data_ptr(), rows * cols) == 0
    first = d_y.clone()
    # each runtime survives the release of the other
    lib.bsq_compress_release()
    assert pkg.decompress_packed(packed, d_y.data_ptr(), rows * cols) == 0
    assert torch.equal(first, d_y)
    assert lib.bsq_compress(d_x.data_ptr(), C.byref(out), None) == 1
    # destination too small
    assert pkg.decompress_packed(packed, d_y.data_ptr(), rows * cols - 1) == 1
    # wrong shape, missing quantiser runtime, smaller top-k capacity
    assert lib.bsq_decompress_initialize(rows, cols - 64, 0.05, 0.0, -1, -1, -1, 10) == 0
    assert pkg.decompress_packed(packed, d_y.data_ptr(), rows * cols) == 1
    assert lib.bsq_decompress_initialize(rows, cols, 0.05, 0.0, -1, -1, -1, -1) == 0
    assert pkg.decompress_packed(packed, d_y.data_ptr(), rows * cols) == 1
    assert lib.bsq_decompress_initialize(rows, cols, 0.01, 0.0, -1, -1, -1, 10) == 0
    assert pkg.decompress_packed(packed, d_y.data_ptr(), rows * cols) == 1
    assert lib.bsq_decompress_initialize(rows, cols, 0.0, 0.0, -1, -1, -1, 10) == 0      # no outlier runtime at all
    assert pkg.decompress_packed(packed, d_y.data_ptr(), rows * cols) == 1
    # a larger capacity and a different configured method are fine (the object says what it holds)
    assert lib.bsq_decompress_initialize(rows, cols, 0.10, 0.0, -1, -1, -1, 11) == 0
    assert pkg.decompress_packed(packed, d_y.data_ptr(), rows * cols) == 0
    assert torch.equal(first, d_y)
    # corrupted payloads are rejected on the host, never on the device
    bad = packed.copy()
    bad[200] ^= 0xFF                                   # quantiser magic
    assert pkg.decompress_packed(bad, d_y.data_ptr(), rows * cols) == 1
    bad = packed.copy()
    bad[40] |= 1                                       # claims SVD sections that are not there
    assert pkg.decompress_packed(bad, d_y.data_ptr(), rows * cols) == 1
    bad = packed.copy()
    sec = pkg.Array.section_outlier_topk.offset
    bad[sec + 8:sec + 16] = np.frombuffer(np.uint64(10 ** 9).tobytes(), np.uint8)   # section size beyond the buffer
    assert pkg.load_packed(bad) is None
    # re-initialisation works after release
    lib.bsq_decompress_release()
    assert pkg.decompress_packed(packed, d_y.data_ptr(), rows * cols) == 1
    assert lib.bsq_compress_initialize(rows, cols, 0.05, 0.0, -1, 1, -1, -1, 10, 1) == 0
    res2 = pkg.compress_to_bytes(d_x.data_ptr())
    assert res2 is not None and np.array_equal(res2[1][:192], packed[:192]) and np.array_equal(res2[1][200:], packed[200:])
    lib.bsq_compress_release()


def test_error_section_skipped_when_quantisation_is_exact(pkg, lib, oracle):
    """All-zero input: every dequantised value equals the input, so no error section is emitted
    (src/bitsqz_llm.cu:1160-1178) although an error ratio is configured."""
    rows, cols = 64, 512
    x = np.zeros((rows, cols), np.float32)
    hdr, packed = compress_bytes(pkg, lib, x, 0.0, 0.05, 11, 1)
    assert hdr.flags == 0 and hdr.section_error_topk.storage == pkg.SECTION_NONE
    assert same_bytes(packed, oracle.compress_nosvd(x, 0.0, 0.05, 11))
    lib.bsq_compress_release()


@pytest.mark.parametrize("method", [10, 11])
def test_selected_infinity_does_not_spoil_its_neighbour(pkg, lib, oracle, method):
    """A +Inf that the outlier stage selects sits in a block whose other values are ordinary, so the block takes the table
    encoder; the encoder's output for +Inf must stay a nibble, or the value packed into the same byte comes out wrong
    (the selected column itself is overwritten with the code of 0.0 afterwards).  Also rows of NaN, zeros and denormals."""
    from test_gpu_ref_parity import special_matrix
    x = np.ascontiguousarray(special_matrix(48, 256, 3))
    hdr, packed = compress_bytes(pkg, lib, x, 0.04, 0.0, method, pkg.INPUT_DEVICE)
    assert same_bytes(packed, oracle.compress_nosvd(x, 0.04, 0.0, method))
    lib.bsq_compress_release()
