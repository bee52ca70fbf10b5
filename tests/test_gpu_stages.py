"""GPU parity of the stage kernels, through the C ABI, against the CPU oracle (bit-exact)."""
import hashlib
import json
import os

import numpy as np
import pytest

from conftest import GOLDEN, bits, glibc_uniform, golden_names, make_c2_like

pytestmark = pytest.mark.gpu
torch = pytest.importorskip("torch")


def dev(a):
    return torch.from_numpy(np.ascontiguousarray(a)).cuda()


def quantize_gpu(lib, x, method, want_deq=False, in_place=False):
    n = x.size
    nb = (n + 63) // 64
    d_x = dev(x.ravel())
    d_data = torch.zeros((n + 1) // 2, dtype=torch.uint8, device="cuda")
    d_deq = d_x if in_place else (torch.zeros(n, dtype=torch.float32, device="cuda") if want_deq else None)
    deq_ptr = d_deq.data_ptr() if d_deq is not None else None
    if method == 11:
        d_s = torch.zeros(nb, dtype=torch.float32, device="cuda")
        assert lib.bsq_nf4_quantize(d_x.data_ptr(), n, d_s.data_ptr(), d_data.data_ptr(), deq_ptr, None) == 0
        torch.cuda.synchronize()
        return d_s.cpu().numpy(), d_data.cpu().numpy(), (d_deq.cpu().numpy() if d_deq is not None else None)
    d_dq = torch.zeros(4, dtype=torch.float32, device="cuda")
    d_c = torch.zeros(nb, dtype=torch.uint8, device="cuda")
    d_scr = torch.zeros(lib.bsq_nf4dq_scratch_bytes(n), dtype=torch.uint8, device="cuda")
    assert lib.bsq_nf4dq_quantize(d_x.data_ptr(), n, d_dq.data_ptr(), d_c.data_ptr(), d_data.data_ptr(), deq_ptr,
                                  d_scr.data_ptr(), None) == 0
    torch.cuda.synchronize()
    return d_dq.cpu().numpy()[0], d_c.cpu().numpy(), d_data.cpu().numpy(), (d_deq.cpu().numpy() if d_deq is not None else None)


def check_quant(lib, oracle, x, tag=""):
    n = x.size
    s, d, deq = quantize_gpu(lib, x, 11, want_deq=True)
    so, do = oracle.nf4_quantize(x)
    assert np.array_equal(bits(s), bits(so)), tag
    assert np.array_equal(d, do), tag
    assert np.array_equal(bits(deq), bits(oracle.nf4_dequantize(so, do, n))), tag
    dq, c, d2, deq2 = quantize_gpu(lib, x, 10, want_deq=True)
    dqo, co, d2o = oracle.nf4dq_quantize(x)
    assert bits(np.array([dq]))[0] == bits(np.array([dqo]))[0], tag
    assert np.array_equal(c, co), tag
    assert np.array_equal(d2, d2o), tag
    assert np.array_equal(bits(deq2), bits(oracle.nf4dq_dequantize(dqo, co, d2o, n))), tag
    # stand-alone dequantisers
    d_out = torch.zeros(n, dtype=torch.float32, device="cuda")
    assert lib.bsq_nf4_dequantize(dev(so).data_ptr(), dev(do).data_ptr(), n, d_out.data_ptr(), None) == 0
    torch.cuda.synchronize()
    assert np.array_equal(bits(d_out.cpu().numpy()), bits(oracle.nf4_dequantize(so, do, n))), tag
    d_dq = dev(np.array([dqo, 0, 0, 0], np.float32))
    assert lib.bsq_nf4dq_dequantize(d_dq.data_ptr(), dev(co).data_ptr(), dev(d2o).data_ptr(), n, d_out.data_ptr(), None) == 0
    torch.cuda.synchronize()
    assert np.array_equal(bits(d_out.cpu().numpy()), bits(oracle.nf4dq_dequantize(dqo, co, d2o, n))), tag


def test_quant_golden_vectors(lib, oracle, golden):
    for name in golden_names(golden):
        x = golden[name + ".x"]
        s, d, _ = quantize_gpu(lib, x, 11)
        assert np.array_equal(bits(s), bits(golden[name + ".nf4_scales"])), name
        assert np.array_equal(d, golden[name + ".nf4_data"]), name
        dq, c, d2, _ = quantize_gpu(lib, x, 10)
        assert bits(np.array([dq]))[0] == bits(golden[name + ".dq"])[0], name
        assert np.array_equal(c, golden[name + ".dq_codes"]), name
        assert np.array_equal(d2, golden[name + ".dq_data"]), name
        check_quant(lib, oracle, x, name)


@pytest.mark.parametrize("seed", [12345, 54321])
def test_quant_reference_test_fixture(lib, seed):
    """Same input as the reference's GPU-vs-CPU tests; digests were produced by the reference's CPU code."""
    with open(os.path.join(GOLDEN, "rand_fixture.json")) as f:
        want = json.load(f)[str(seed)]
    x = glibc_uniform(seed, 1 << 20)
    sha = lambda a: hashlib.sha256(np.ascontiguousarray(a).tobytes()).hexdigest()
    s, d, deq = quantize_gpu(lib, x, 11, want_deq=True)
    assert sha(s) == want["nf4_scales_sha256"] and sha(d) == want["nf4_data_sha256"] and sha(deq) == want["nf4_deq_sha256"]
    dq, c, d2, deq2 = quantize_gpu(lib, x, 10, want_deq=True)
    assert int(bits(np.array([dq]))[0]) == want["dq_bits"]
    assert sha(c) == want["dq_codes_sha256"] and sha(d2) == want["dq_data_sha256"] and sha(deq2) == want["dq_deq_sha256"]


def test_quant_ragged_sizes_and_inplace(lib, oracle):
    rng = np.random.default_rng(17)
    for n in (1, 7, 64, 100, 1023, 1024, 1025, 4099, 65536 + 31, (1 << 20) + 5):
        check_quant(lib, oracle, rng.standard_normal(n).astype(np.float32), f"n={n}")
    x = rng.standard_normal(5000).astype(np.float32)
    s, d, deq = quantize_gpu(lib, x, 11, in_place=True)
    so, do = oracle.nf4_quantize(x)
    assert np.array_equal(d, do) and np.array_equal(bits(deq), bits(oracle.nf4_dequantize(so, do, x.size)))


def test_quant_near_every_threshold(lib, oracle):
    """Scaled values within +-256 ulp of each of the 15 code boundaries, in blocks whose absmax is 1."""
    thr = [0xbf591cd8, 0xbf1c5270, 0xbeeb847f, 0xbeadea76, 0xbe703cec, 0xbe0d38bb, 0xbd3a7870, 0x3d22fb00,
           0x3df64863, 0x3e5067e1, 0x3e9582d5, 0x3ec753fa, 0x3f006d04, 0x3f248db0, 0x3f5c89da]
    vals = []
    for t in thr:
        vals.append(np.arange(t - 256, t + 256, dtype=np.uint32).view(np.float32))
    v = np.concatenate(vals)
    pad = (-v.size) % 63
    v = np.concatenate([v, np.zeros(pad, np.float32)]).reshape(-1, 63)
    x = np.concatenate([np.ones((v.shape[0], 1), np.float32), v], axis=1).ravel()
    check_quant(lib, oracle, x, "thresholds")


def topk_gpu(lib, x, k, residual="none"):
    rows, cols = x.shape
    d_x = dev(x)
    d_idx = torch.zeros((rows, max(k, 1)), dtype=torch.int16, device="cuda")
    d_val = torch.zeros((rows, max(k, 1)), dtype=torch.float32, device="cuda")
    d_st = torch.zeros(4, dtype=torch.int32, device="cuda")
    d_res = None
    if residual == "copy":
        d_res = torch.full_like(d_x, 7.0)
    elif residual == "inplace":
        d_res = d_x
    rc = lib.bsq_topk_rows(d_x.data_ptr(), d_res.data_ptr() if d_res is not None else None, rows, cols, k,
                           d_idx.data_ptr(), d_val.data_ptr(), d_st.data_ptr(), None)
    assert rc == 0
    torch.cuda.synchronize()
    assert int(d_st[0]) == 0
    idx = d_idx.cpu().numpy().view(np.uint16)[:, :k]
    val = d_val.cpu().numpy()[:, :k]
    return idx, val, (d_res.cpu().numpy() if d_res is not None else None)


def check_topk(lib, oracle, x, k, tag=""):
    io, vo, zo = oracle.topk_rows(x, k, zero_selected=True)
    for mode in ("none", "copy", "inplace"):
        idx, val, res = topk_gpu(lib, x, k, mode)
        assert np.array_equal(idx, io), (tag, mode)
        assert np.array_equal(bits(val), bits(vo)), (tag, mode)
        if res is not None:
            assert np.array_equal(bits(res), bits(zo)), (tag, mode)


def test_topk_random_shapes(lib, oracle):
    rng = np.random.default_rng(23)
    for rows, cols, k in [(64, 4096, 41), (33, 4096, 20), (16, 14336, 143), (16, 14336, 72), (8, 8192, 123),
                          (300, 1024, 10), (5, 256, 1), (3, 64, 64), (7, 512, 256)]:
        check_topk(lib, oracle, rng.standard_normal((rows, cols)).astype(np.float32), k, f"{rows}x{cols} k={k}")
    check_topk(lib, oracle, make_c2_like(128, 4096, 2), 41, "c2-like")
    t = rng.standard_t(3, (32, 4096)).astype(np.float32)
    check_topk(lib, oracle, t, 41, "student-t")


def test_topk_ties_zeros_nan(lib, oracle):
    rng = np.random.default_rng(29)
    cols = 1024
    x = np.zeros((6, cols), np.float32)                      # rows of zeros and few distinct values
    x[1] = 1.0
    x[2] = rng.integers(-2, 3, cols).astype(np.float32)
    x[3, ::3] = np.nan
    x[3, 1::3] = rng.standard_normal(len(x[3, 1::3])).astype(np.float32)
    x[4] = np.nan
    x[5] = rng.standard_normal(cols).astype(np.float32)
    x[5, 10] = np.inf
    x[5, 20] = -np.inf
    x[5, 30] = -0.0
    for k in (1, 5, 41, 200):
        check_topk(lib, oracle, x, k, f"ties k={k}")
    y = np.round(rng.standard_normal((16, 4096)) * 4).astype(np.float32) / 4        # heavy ties at the cut
    check_topk(lib, oracle, y, 41, "quantised values")


def test_topk_generic_path(lib, oracle):
    """Shapes the shared-memory kernel does not take: cols % 4 != 0, k > 256, tiny literal cases."""
    rng = np.random.default_rng(31)
    for rows, cols, k in [(3, 6, 3), (2, 8, 1), (2, 8, 8), (4, 5, 2), (9, 1001, 17), (4, 8192, 819), (2, 4096, 2500),
                          (3, 3000, 3000)]:
        check_topk(lib, oracle, rng.standard_normal((rows, cols)).astype(np.float32), k, f"{rows}x{cols} k={k}")


def test_topk_apply(lib, oracle):
    rng = np.random.default_rng(37)
    rows, cols, k = 50, 777, 13
    x = rng.standard_normal((rows, cols)).astype(np.float32)
    idx, val, _ = oracle.topk_rows(x, k)
    base = rng.standard_normal((rows, cols)).astype(np.float32)
    d_dense = dev(base)
    d_st = torch.zeros(4, dtype=torch.int32, device="cuda")
    assert lib.bsq_topk_apply(dev(idx.view(np.int16)).data_ptr(), dev(val).data_ptr(), rows, cols, k, d_dense.data_ptr(),
                              d_st.data_ptr(), None) == 0
    torch.cuda.synchronize()
    assert np.array_equal(bits(d_dense.cpu().numpy()), bits(oracle.topk_apply(idx, val, base)))
    bad = idx.copy()
    bad[0, 0] = 60000                                  # out-of-range column: skipped and reported, no fault
    assert lib.bsq_topk_apply(dev(bad.view(np.int16)).data_ptr(), dev(val).data_ptr(), rows, cols, k, d_dense.data_ptr(),
                              d_st.data_ptr(), None) == 0
    torch.cuda.synchronize()
    assert int(d_st[0]) != 0


def frontend_gpu(lib, x, k, method, carried=None, calls=1):
    """carried: bit pattern put into the scratch word that carries the selection bound from call to call."""
    rows, cols = x.shape
    n = rows * cols
    nb = n // 64
    d_x = dev(x)
    d_idx = torch.zeros((rows, k), dtype=torch.int16, device="cuda")
    d_val = torch.zeros((rows, k), dtype=torch.float32, device="cuda")
    d_s = torch.zeros(nb, dtype=torch.float32, device="cuda")
    d_dq = torch.zeros(4, dtype=torch.float32, device="cuda")
    d_c = torch.zeros(nb, dtype=torch.uint8, device="cuda")
    d_data = torch.zeros(n // 2, dtype=torch.uint8, device="cuda")
    d_scr = torch.zeros(lib.bsq_frontend_scratch_bytes(rows, cols), dtype=torch.uint8, device="cuda")
    d_st = torch.zeros(4, dtype=torch.int32, device="cuda")
    assert lib.bsq_frontend_supported(rows, cols, k) == 1
    if carried is not None:
        d_scr.view(torch.int32)[3] = int(np.array([carried], dtype=np.uint32).view(np.int32)[0])
    for _ in range(calls):
        rc = lib.bsq_frontend_quantize(method, d_x.data_ptr(), rows, cols, k, d_idx.data_ptr(), d_val.data_ptr(), d_s.data_ptr(),
                                       d_dq.data_ptr(), d_c.data_ptr(), d_data.data_ptr(), d_scr.data_ptr(), d_st.data_ptr(), None)
        assert rc == 0
    torch.cuda.synchronize()
    assert int(d_st[0]) == 0
    return (d_idx.cpu().numpy().view(np.uint16), d_val.cpu().numpy(), d_s.cpu().numpy(), d_dq.cpu().numpy()[0],
            d_c.cpu().numpy(), d_data.cpu().numpy())


@pytest.mark.parametrize("shape_k", [(128, 4096, 41), (40, 14336, 72), (64, 1024, 10), (16, 8192, 82), (300, 64, 1)])
def test_frontend_matches_oracle(lib, oracle, shape_k):
    rows, cols, k = shape_k
    x = make_c2_like(rows, cols, rows + cols)
    x[1, :64] = 0.0
    x[2, 5] = np.nan
    x[2, 6] = np.inf
    io, vo, zo = oracle.topk_rows(x, k, zero_selected=True)
    for method in (11, 10):
        idx, val, s, dq, c, data = frontend_gpu(lib, x, k, method)
        assert np.array_equal(idx, io) and np.array_equal(bits(val), bits(vo))
        if method == 11:
            so, do = oracle.nf4_quantize(zo)
            assert np.array_equal(bits(s), bits(so)) and np.array_equal(data, do)
        else:
            dqo, co, do = oracle.nf4dq_quantize(zo)
            assert bits(np.array([dq]))[0] == bits(np.array([dqo]))[0]
            assert np.array_equal(c, co) and np.array_equal(data, do)


@pytest.mark.parametrize("method", [10, 11])
def test_frontend_result_does_not_depend_on_the_carried_bound(lib, method):
    # whatever the scratch word holds (nothing, the bound of an earlier call on the same or on a differently scaled
    # matrix, denormal, huge, infinite, NaN, negative), the bytes that come out are the same
    rows, cols, k = 96, 4096, 41
    x = make_c2_like(rows, cols, 77)
    want = frontend_gpu(lib, x, k, method)
    again = frontend_gpu(lib, x, k, method, calls=3)                 # the second and third call start from a carried bound
    cases = [0x00000001, 0x00800000, 0x3A83126F, 0x3F800000, 0x41200000, 0x7F7FFFFF, 0x7F800000, 0x7FC00000, 0xBF800000, 0xFFFFFFFF]
    outs = [again] + [frontend_gpu(lib, x, k, method, carried=c) for c in cases]
    for got in outs:
        for a, b in zip(want, got):
            assert np.array_equal(bits(np.asarray(a)), bits(np.asarray(b))) if np.asarray(a).dtype == np.float32 else np.array_equal(a, b)


@pytest.mark.parametrize("shape_k", [(64, 4096, 41), (37, 192, 5), (300, 64, 1), (5, 14336, 143), (129, 1024, 10)])
@pytest.mark.parametrize("method", [10, 11])
def test_dequantize_add_topk_equals_the_two_stages(lib, shape_k, method):
    # one pass (decode, then the row's k entries added) against bsq_nf4*_dequantize followed by bsq_topk_apply: same bits;
    # rows shorter and longer than a warp's batch of 1024 elements, batches that straddle rows, a ragged last batch
    rows, cols, k = shape_k
    x = make_c2_like(rows, cols, rows * 7 + cols)
    idx, val, s, dq, c, data = frontend_gpu(lib, x, k, method)
    n = rows * cols
    d_idx, d_val = dev(idx.view(np.int16)), dev(val)
    d_s, d_dq, d_c, d_data = dev(s), dev(np.array([dq, 0, 0, 0], np.float32)), dev(c), dev(data)
    want = torch.full((rows, cols), 7.0, dtype=torch.float32, device="cuda")
    got = torch.full((rows, cols), 9.0, dtype=torch.float32, device="cuda")
    d_st = torch.zeros(4, dtype=torch.int32, device="cuda")
    if method == 11:
        assert lib.bsq_nf4_dequantize(d_s.data_ptr(), d_data.data_ptr(), n, want.data_ptr(), None) == 0
    else:
        assert lib.bsq_nf4dq_dequantize(d_dq.data_ptr(), d_c.data_ptr(), d_data.data_ptr(), n, want.data_ptr(), None) == 0
    assert lib.bsq_topk_apply(d_idx.data_ptr(), d_val.data_ptr(), rows, cols, k, want.data_ptr(), d_st.data_ptr(), None) == 0
    assert lib.bsq_dequantize_add_topk(method, d_s.data_ptr(), d_dq.data_ptr(), d_c.data_ptr(), d_data.data_ptr(), rows, cols,
                                       d_idx.data_ptr(), d_val.data_ptr(), k, got.data_ptr(), d_st.data_ptr(), None) == 0
    torch.cuda.synchronize()
    assert int(d_st[0]) == 0
    assert torch.equal(want.view(torch.int32), got.view(torch.int32))
    # and it gives the input back where the input was an outlier
    r0 = got.cpu().numpy()
    assert np.array_equal(bits(r0[np.arange(rows)[:, None], idx.astype(np.int64)]), bits(val))
    # a column out of range is skipped and reported
    bad = idx.copy()
    bad[0, 0] = 65000
    assert lib.bsq_dequantize_add_topk(method, d_s.data_ptr(), d_dq.data_ptr(), d_c.data_ptr(), d_data.data_ptr(), rows, cols,
                                       dev(bad.view(np.int16)).data_ptr(), d_val.data_ptr(), k, got.data_ptr(), d_st.data_ptr(), None) == 0
    torch.cuda.synchronize()
    assert int(d_st[0]) != 0


def test_residual_error(lib, oracle):
    rng = np.random.default_rng(41)
    for n in (5, 64, 1000, 4099):
        a = rng.standard_normal(n).astype(np.float32)
        b = a.copy()
        d_e = torch.zeros(n, dtype=torch.float32, device="cuda")
        d_f = torch.zeros(4, dtype=torch.int32, device="cuda")
        assert lib.bsq_residual_error(dev(a).data_ptr(), dev(b).data_ptr(), n, d_e.data_ptr(), d_f.data_ptr(), None) == 0
        torch.cuda.synchronize()
        assert int(d_f[0]) == 0 and not d_e.any()
        b[n // 2] += np.float32(0.5)
        assert lib.bsq_residual_error(dev(a).data_ptr(), dev(b).data_ptr(), n, d_e.data_ptr(), d_f.data_ptr(), None) == 0
        torch.cuda.synchronize()
        assert int(d_f[0]) == 1 and np.array_equal(d_e.cpu().numpy(), a - b)
