"""The allocation-free NF4_DQ entry point against the ordinary one, through the C ABI.

Callers that may not allocate device memory (a serving loop with a fixed memory budget, code that
runs under a pool owning the whole device) use bsq_nf4dq_quantize_static, whose scratch is a fixed
array inside the library.  It must give exactly the bytes of bsq_nf4dq_quantize, also on a second
call that finds the first call's leftovers in the shared scratch.  Collected last on purpose."""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu
torch = pytest.importorskip("torch")


def _run(lib, x, static):
    n = x.size
    nb = (n + 63) // 64
    d_x = torch.from_numpy(x).cuda()
    d_dq = torch.zeros(4, dtype=torch.float32, device="cuda")
    d_c = torch.full((nb,), 0xAA, dtype=torch.uint8, device="cuda")
    d_d = torch.full(((n + 1) // 2,), 0xAA, dtype=torch.uint8, device="cuda")
    if static:
        rc = lib.bsq_nf4dq_quantize_static(d_x.data_ptr(), n, d_dq.data_ptr(), d_c.data_ptr(), d_d.data_ptr(), None)
    else:
        scr = torch.zeros(lib.bsq_nf4dq_scratch_bytes(n), dtype=torch.uint8, device="cuda")
        rc = lib.bsq_nf4dq_quantize(d_x.data_ptr(), n, d_dq.data_ptr(), d_c.data_ptr(), d_d.data_ptr(), None,
                                    scr.data_ptr(), None)
    assert rc == 0
    torch.cuda.synchronize()
    return d_dq.cpu().numpy()[:1].view(np.uint32)[0], d_c.cpu().numpy(), d_d.cpu().numpy()


def test_static_scratch_variant_matches_on_two_calls_in_a_row(lib):
    rng = np.random.default_rng(99)
    first = (rng.standard_normal(1 << 20) * 37.0).astype(np.float32)      # large values, many blocks
    second = (rng.standard_normal(70001) * 1e-3).astype(np.float32)       # smaller, ragged, tiny values
    for x in (first, second):
        want = _run(lib, x, static=False)
        got = _run(lib, x, static=True)
        assert got[0] == want[0]
        assert np.array_equal(got[1], want[1]) and np.array_equal(got[2], want[2])
    # sizes beyond the built-in scratch are refused, not truncated
    limit = int(lib.bsq_nf4dq_quantize_static_max_elements())
    assert limit == 1 << 24
    d = torch.zeros(16, dtype=torch.uint8, device="cuda")
    assert lib.bsq_nf4dq_quantize_static(d.data_ptr(), limit + 1, d.data_ptr(), d.data_ptr(), d.data_ptr(), None) == 1
    assert lib.bsq_nf4dq_quantize_static(d.data_ptr(), 0, d.data_ptr(), d.data_ptr(), d.data_ptr(), None) == 1
