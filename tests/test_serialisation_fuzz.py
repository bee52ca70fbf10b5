"""Malformed packed objects: load_bitsqz_llm_from_buffer (host only) and bitsqz_llm_decompress must reject what does not
add up -- or accept it and stay inside the buffer -- and never crash or fault a kernel.  The checks they make are the
reference's (src/bitsqz_llm.cu:1417-1450 for loading, :654-761 for decompress; quantization_cuda.cu:809-876 and
topk_cuda.cu:271-297 for the section headers); the mutations are random but seeded."""
import ctypes as C

import numpy as np
import pytest

from conftest import make_c2_like


def mutations(valid, rng, count, header_bias=0.8):
    """Seeded corruptions of a valid object: single bytes, 64-bit fields of the section table, truncations."""
    n = valid.size
    for i in range(count):
        bad = valid.copy()
        kind = i % 4
        if kind == 0:                                        # a byte of the 200-byte header
            bad[rng.integers(0, 192)] = rng.integers(0, 256)
        elif kind == 1:                                      # a section's offset or size becomes arbitrary
            sec = 48 + 24 * int(rng.integers(0, 6)) + 8 * int(rng.integers(0, 2))
            value = int(rng.choice([0, 1, n, n + 1, 2 ** 31, 2 ** 63, rng.integers(0, 2 * n)]))
            bad[sec:sec + 8] = np.frombuffer(np.uint64(value).tobytes(), np.uint8)
        elif kind == 2:                                      # bytes of a section header or payload
            lo = 200 if rng.random() < header_bias else int(rng.integers(200, n))
            hi = min(n, lo + 64)
            at = rng.integers(lo, hi, size=4)
            bad[at] = rng.integers(0, 256, size=4)
        else:                                                # storage kinds, flags, formats
            at = int(rng.choice([40, 24, 28, 32, 16, 18, 20, 64, 88, 112, 136, 160, 184]))
            bad[at] = rng.integers(0, 8)
        cut = n if i % 7 else int(rng.integers(0, n))        # sometimes the buffer is shorter than the object
        yield bad[:cut]


def test_load_never_accepts_what_does_not_fit(pkg, lib, oracle):
    x = make_c2_like(64, 256, 11)
    valid = oracle.compress_nosvd(x, 0.05, 0.03, 10)
    rng = np.random.default_rng(2024)
    accepted = 0
    for bad in mutations(valid, rng, 600):
        buf = np.ascontiguousarray(bad)
        h = lib.bsq_load_from_buffer(buf.ctypes.data if buf.size else None, buf.size)
        if not h:
            continue
        accepted += 1
        hdr = pkg.Array.from_buffer_copy(C.string_at(h, 200))
        packed = int(lib.bsq_get_packed_size(h))
        assert 200 <= packed <= buf.size                     # whatever it describes lies inside what was handed in
        for name in ("section_u", "section_s", "section_v", "section_direct", "section_outlier_topk", "section_error_topk"):
            s = getattr(hdr, name)
            if s.storage != pkg.SECTION_NONE:
                assert s.offset + s.size <= packed - 200
        assert hdr.payload == h + 200                        # the payload pointer is rebuilt, never taken from the bytes
        lib.bsq_free(h)
    assert accepted > 0                                      # payload-only corruptions are still well-formed objects


@pytest.mark.gpu
def test_decompress_survives_corrupted_objects(pkg, lib, oracle):
    torch = pytest.importorskip("torch")
    rows, cols = 64, 256
    x = make_c2_like(rows, cols, 11)
    valid = oracle.compress_nosvd(x, 0.05, 0.03, 10)
    want = oracle.decompress_nosvd(valid, rows, cols)
    assert lib.bsq_decompress_initialize(rows, cols, 0.05, 0.03, -1, -1, -1, 10) == 0
    d_y = torch.zeros((rows, cols), dtype=torch.float32, device="cuda")
    rng = np.random.default_rng(7)
    outcomes = {0: 0, 1: 0}
    for bad in mutations(valid, rng, 400):
        rc = pkg.decompress_packed(bad, d_y.data_ptr(), rows * cols) if bad.size else 1
        assert rc in (0, 1)
        outcomes[rc] += 1
    torch.cuda.synchronize()                                 # no kernel faulted: the context still works ...
    assert outcomes[0] > 0 and outcomes[1] > 0
    assert pkg.decompress_packed(valid, d_y.data_ptr(), rows * cols) == 0
    torch.cuda.synchronize()
    assert np.array_equal(d_y.cpu().numpy().view(np.uint32), want.view(np.uint32))      # ... and gives the right answer
    lib.bsq_decompress_release()
