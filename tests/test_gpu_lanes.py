"""GPU tests of the additive entry points around the public calls: lanes (begin / end halves of a call on a stream of
their own), device-resident packed objects, batches over several lanes, and the host-side fault hook.  Everything is
checked bit for bit against the public bitsqz_llm_compress / bitsqz_llm_decompress of the same library, which the other
test files check against the oracle and the reference."""
import ctypes as C

import numpy as np
import pytest

from conftest import make_c2_like

pytestmark = pytest.mark.gpu
torch = pytest.importorskip("torch")

CONFIGS = [
    # rows, cols, outlier, error, rank, niters, uv, s, q
    (256, 4096, 0.01, 0.0, -1, 1, -1, -1, 10),        # fused front end, one list on decompress
    (128, 1024, 0.02, 0.03, -1, 1, -1, -1, 11),       # unfused, two lists
    (96, 320, 0.0, 0.0, -1, 1, -1, -1, -1),           # dense FP32
    (512, 1024, 0.01, 0.02, 64, 2, 11, -1, -1),       # SVD, NF4 factors, error correction
    (300, 700, 0.0, 0.0, 48, 1, -1, 10, -1),          # SVD, FP32 U/V, NF4_DQ S
]


def masked(b):
    out = np.array(b, dtype=np.uint8, copy=True)
    out[192:200] = 0
    return out


def matrix_for(cfg, seed):
    rows, cols = cfg[0], cfg[1]
    x = make_c2_like(rows, cols, seed)
    if cfg[4] >= 1:                                      # something low-rank under the noise for the SVD configurations
        rng = np.random.default_rng(seed + 100)
        x = (rng.standard_normal((rows, 24)) @ rng.standard_normal((24, cols)) + 0.05 * x).astype(np.float32)
        x[:, 3] *= 25.0
    return np.ascontiguousarray(x)


def public_roundtrip(pkg, lib, cfg, x_ptr, loc):
    rows, cols, outlier, err, rank, niters, uv, s, q = cfg
    assert lib.bsq_compress_initialize(rows, cols, outlier, err, rank, niters, uv, s, q, loc) == 0
    res = pkg.compress_to_bytes(x_ptr)
    lib.bsq_compress_release()
    assert res is not None
    hdr, packed = res
    eff = hdr.effective_rank if rank >= 1 else rank
    assert lib.bsq_decompress_initialize(rows, cols, outlier, err, eff, uv, s, q) == 0
    d_y = torch.zeros((rows, cols), dtype=torch.float32, device="cuda")
    assert pkg.decompress_packed(packed, d_y.data_ptr(), rows * cols) == 0
    torch.cuda.synchronize()
    lib.bsq_decompress_release()
    return packed, d_y


@pytest.mark.parametrize("cfg", CONFIGS)
def test_lane_host_and_device_objects_equal_public_call(pkg, lib, cfg):
    rows, cols = cfg[0], cfg[1]
    n = rows * cols
    x = matrix_for(cfg, 11)
    d_x = torch.from_numpy(x).cuda()
    want, want_y = public_roundtrip(pkg, lib, cfg, d_x.data_ptr(), pkg.INPUT_DEVICE)
    lane = lib.bsq_lane_create(*cfg)
    assert lane
    try:
        cap = int(lib.bsq_lane_packed_capacity(lane))
        assert cap >= want.size
        # host object, from a device and from a host input
        pinned = torch.from_numpy(x).pin_memory()
        for ptr, loc in ((d_x.data_ptr(), pkg.INPUT_DEVICE), (pinned.data_ptr(), pkg.INPUT_HOST), (x.ctypes.data, pkg.INPUT_HOST)):
            out, size = C.c_void_p(None), C.c_uint64(0)
            assert lib.bsq_lane_compress_begin(lane, ptr, loc, None, 0) == 0
            assert lib.bsq_lane_compress_begin(lane, ptr, loc, None, 0) == 1          # one call per lane at a time
            assert lib.bsq_lane_compress_end(lane, C.byref(out), None, C.byref(size)) == 0
            got = np.frombuffer(C.string_at(out.value, size.value), np.uint8)
            assert size.value == want.size and np.array_equal(masked(got), masked(want))
            # decompress straight from the host object
            d_y = torch.zeros((rows, cols), dtype=torch.float32, device="cuda")
            assert lib.bsq_lane_decompress_begin(lane, out, 0, d_y.data_ptr(), n) == 0
            assert lib.bsq_lane_decompress_end(lane) == 0
            assert torch.equal(d_y.view(torch.int32), want_y.view(torch.int32))
            lib.bsq_free(out)
        # device-resident object: same bytes in a device buffer, header copy with a device payload pointer
        d_packed = torch.zeros(cap + 64, dtype=torch.uint8, device="cuda")
        hdr, size = pkg.Array(), C.c_uint64(0)
        assert lib.bsq_lane_compress_begin(lane, d_x.data_ptr(), pkg.INPUT_DEVICE, d_packed.data_ptr(), cap - 1) == 1   # too small
        assert lib.bsq_lane_compress_begin(lane, d_x.data_ptr(), pkg.INPUT_DEVICE, d_packed.data_ptr(), cap) == 0
        assert lib.bsq_lane_compress_end(lane, None, C.byref(hdr), C.byref(size)) == 0
        assert size.value == want.size and hdr.payload == d_packed.data_ptr() + 200
        back = d_packed[: size.value].cpu().numpy()
        assert np.array_equal(masked(back), masked(want))
        loaded = pkg.load_packed(back)                       # the device buffer's bytes are a loadable serialised object
        assert loaded
        lib.bsq_free(loaded)
        d_y = torch.zeros((rows, cols), dtype=torch.float32, device="cuda")
        assert lib.bsq_lane_decompress_begin(lane, C.byref(hdr), 1, d_y.data_ptr(), n) == 0
        assert lib.bsq_lane_decompress_end(lane) == 0
        assert torch.equal(d_y.view(torch.int32), want_y.view(torch.int32))
        # a corrupted section header inside the device payload is caught on the host before any kernel runs
        first_sec = hdr.section_u if cfg[4] >= 1 else hdr.section_direct
        if first_sec.storage == pkg.SECTION_QUANT:
            d_packed[200 + first_sec.offset] ^= 0xFF
            assert lib.bsq_lane_decompress_begin(lane, C.byref(hdr), 1, d_y.data_ptr(), n) == 1
            assert lib.bsq_lane_decompress_end(lane) == 1                                # nothing was begun
    finally:
        lib.bsq_lane_destroy(lane)


@pytest.mark.parametrize("cfg", [CONFIGS[0], CONFIGS[3]])
@pytest.mark.parametrize("lanes", [1, 3])
def test_batch_equals_individual_calls(pkg, lib, cfg, lanes):
    rows, cols = cfg[0], cfg[1]
    n, count = rows * cols, 7
    xs = [matrix_for(cfg, 20 + i) for i in range(count)]
    d_xs = [torch.from_numpy(x).cuda() for x in xs]
    wants = [public_roundtrip(pkg, lib, cfg, d.data_ptr(), pkg.INPUT_DEVICE) for d in d_xs]
    batch = lib.bsq_batch_create(*cfg, lanes)
    assert batch and lib.bsq_batch_lanes(batch) == lanes
    try:
        VP = C.c_void_p * count
        outs = VP()
        sizes = (C.c_uint64 * count)()
        # device inputs -> host objects
        assert lib.bsq_batch_compress(batch, VP(*[d.data_ptr() for d in d_xs]), count, pkg.INPUT_DEVICE, None, 0, outs, None, sizes) == 0
        for i in range(count):
            got = np.frombuffer(C.string_at(outs[i], sizes[i]), np.uint8)
            assert np.array_equal(masked(got), masked(wants[i][0])), i
        d_ys = [torch.zeros((rows, cols), dtype=torch.float32, device="cuda") for _ in range(count)]
        assert lib.bsq_batch_decompress(batch, VP(*[outs[i] for i in range(count)]), count, 0, VP(*[y.data_ptr() for y in d_ys]), n) == 0
        for i in range(count):
            assert torch.equal(d_ys[i].view(torch.int32), wants[i][1].view(torch.int32)), i
            lib.bsq_free(outs[i])
        # host inputs -> device-resident objects -> decompress from the device
        cap = int(lib.bsq_lane_packed_capacity(lib.bsq_batch_lane(batch, 0)))
        d_packed = [torch.zeros(cap, dtype=torch.uint8, device="cuda") for _ in range(count)]
        hdrs = (pkg.Array * count)()
        pinned = [torch.from_numpy(x).pin_memory() for x in xs]
        assert lib.bsq_batch_compress(batch, VP(*[p.data_ptr() for p in pinned]), count, pkg.INPUT_HOST,
                                      VP(*[p.data_ptr() for p in d_packed]), cap, None, hdrs, sizes) == 0
        for i in range(count):
            assert np.array_equal(masked(d_packed[i][: sizes[i]].cpu().numpy()), masked(wants[i][0])), i
        for y in d_ys:
            y.zero_()
        hp = VP(*[C.addressof(hdrs[i]) for i in range(count)])
        assert lib.bsq_batch_decompress(batch, hp, count, 1, VP(*[y.data_ptr() for y in d_ys]), n) == 0
        for i in range(count):
            assert torch.equal(d_ys[i].view(torch.int32), wants[i][1].view(torch.int32)), i
        # a null matrix in the list fails the call and leaves no object behind
        bad = VP(*[d.data_ptr() for d in d_xs])
        bad[4] = None
        assert lib.bsq_batch_compress(batch, bad, count, pkg.INPUT_DEVICE, None, 0, outs, None, sizes) == 1
        assert all(not outs[i] for i in range(count))
    finally:
        lib.bsq_batch_destroy(batch)


def test_status_word_set_by_a_stage_fails_the_call(pkg, lib):
    """A kernel that gives up a bounded wait sets a bit in the runtime's status word; compress and decompress must then
    return 1 and hand out nothing.  The bit is set from the host here (bsq_test_inject_status), no kernel fails."""
    cfg = CONFIGS[3]
    rows, cols, outlier, err, rank, niters, uv, s, q = cfg
    x = matrix_for(cfg, 31)
    d_x = torch.from_numpy(x).cuda()
    assert lib.bsq_compress_initialize(rows, cols, outlier, err, rank, niters, uv, s, q, pkg.INPUT_DEVICE) == 0
    good = pkg.compress_to_bytes(d_x.data_ptr())
    assert good is not None
    lib.bsq_test_inject_status(0, 1)                      # "a bounded wait ran out"
    out = C.c_void_p(None)
    assert lib.bsq_compress(d_x.data_ptr(), C.byref(out), None) == 1 and not out.value
    again = pkg.compress_to_bytes(d_x.data_ptr())         # the runtime is usable afterwards
    assert again is not None and np.array_equal(masked(again[1]), masked(good[1]))
    lib.bsq_compress_release()
    assert lib.bsq_decompress_initialize(rows, cols, outlier, err, good[0].effective_rank, uv, s, q) == 0
    d_y = torch.zeros((rows, cols), dtype=torch.float32, device="cuda")
    lib.bsq_test_inject_status(1, 1)
    assert pkg.decompress_packed(good[1], d_y.data_ptr(), rows * cols) == 1
    assert pkg.decompress_packed(good[1], d_y.data_ptr(), rows * cols) == 0
    lib.bsq_decompress_release()
