"""GPU tests of the matrix product under the low-rank stages: the tcgen05 (3xTF32) kernel and the FP32-pipe
kernel against an FP64 product of the same operands, in all four operand orientations.  Floating point:
the tolerance is stated at the assert."""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu
torch = pytest.importorskip("torch")


def operands(M, N, K, a_kmajor, b_kmajor, seed):
    g = torch.Generator(device="cuda").manual_seed(seed)
    a = torch.randn((M, K) if a_kmajor else (K, M), generator=g, device="cuda", dtype=torch.float32)
    b = torch.randn((N, K) if b_kmajor else (K, N), generator=g, device="cuda", dtype=torch.float32)
    # a wide range of magnitudes, so that the hi/lo operand split is exercised on every exponent
    a *= torch.exp2(torch.randint(-8, 9, a.shape, generator=g, device="cuda").float())
    return a, b


def product_fp64(a, b, a_kmajor, b_kmajor):
    opa = a.double() if a_kmajor else a.double().t()
    opb = b.double().t() if b_kmajor else b.double()
    return opa @ opb, opa.abs() @ opb.abs()


def run(lib, a, b, M, N, K, a_kmajor, b_kmajor, tensor_cores, workspace):
    c = torch.full((M, N), float("nan"), device="cuda", dtype=torch.float32)
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    ws_ptr, ws_bytes = (workspace.data_ptr(), workspace.numel() * 4) if workspace is not None else (None, 0)
    rc = lib.bsq_gemm(int(a_kmajor), int(b_kmajor), a.data_ptr(), a.shape[1], b.data_ptr(), b.shape[1], c.data_ptr(), N, M, N, K,
                      ws_ptr, ws_bytes, int(tensor_cores), status.data_ptr(), None)
    torch.cuda.synchronize()
    assert rc == 0
    assert int(status.item()) == 0
    return c


SHAPES = [
    (128, 16, 128), (128, 128, 128), (256, 64, 256), (300, 48, 200), (1000, 128, 1000), (4096, 128, 4096),
    (2048, 256, 1024), (512, 240, 416), (131, 32, 132), (128, 128, 4096),
    (1024, 160, 2008), (640, 256, 4096),      # B split beforehand: K tail, partial last row tile
    (96, 64, 300),      # fewer rows than a tensor-core tile: FP32 pipes
    (256, 40, 256),     # N not a multiple of 16: FP32 pipes
]


@pytest.mark.parametrize("shape", SHAPES)
@pytest.mark.parametrize("a_kmajor", [True, False])
@pytest.mark.parametrize("b_kmajor", [True, False])
def test_gemm_matches_fp64(lib, shape, a_kmajor, b_kmajor):
    M, N, K = shape
    a, b = operands(M, N, K, a_kmajor, b_kmajor, seed=M * 7 + N * 3 + K)
    want, scale = product_fp64(a, b, a_kmajor, b_kmajor)
    workspace = torch.empty(8 * M * N, device="cuda", dtype=torch.float32)
    for tensor_cores in (False, True):
        for ws in (None, workspace):
            got = run(lib, a, b, M, N, K, a_kmajor, b_kmajor, tensor_cores, ws).double()
            # FP32 accumulation over K terms: |error| <= 3e-5 * sum_k |a_ik| |b_kj| elementwise (the forward bound
            # K * 2^-24 would allow far more; the tensor core truncates when it accumulates, the FP32 pipes round)
            # and 2e-6 in the Frobenius norm relative to that scale; a product in plain TF32 (operands cut to
            # 11 bits) misses the second bound by an order of magnitude
            err = (got - want).abs()
            assert bool((err <= 3e-5 * scale).all()), (tensor_cores, ws is not None, float((err / scale).max()))
            assert float(err.norm() / scale.norm()) <= 2e-6, (tensor_cores, ws is not None)


def test_gemm_tensor_core_path_is_repeatable(lib):
    M, N, K = 1024, 128, 2048
    a, b = operands(M, N, K, True, False, seed=5)
    workspace = torch.empty(8 * M * N, device="cuda", dtype=torch.float32)
    first = run(lib, a, b, M, N, K, True, False, True, workspace)
    for _ in range(3):
        assert torch.equal(first, run(lib, a, b, M, N, K, True, False, True, workspace))


def test_gemm_with_b_split_beforehand_for_every_shape():
    """BSQ_GEMM_IMAGE=2 sends every product that can take it (also those of up to 128 columns, which by default
    stay on the kernel that splits B in every CTA) to the kernel fed by bulk copies of pre-split images; the switch
    is read once per process, so the accuracy test runs again in a child process."""
    import os
    import subprocess
    import sys
    env = dict(os.environ, BSQ_GEMM_IMAGE="2")
    here = os.path.dirname(os.path.abspath(__file__))
    res = subprocess.run([sys.executable, "-m", "pytest", os.path.join(here, "test_gpu_gemm.py"), "-q", "-x", "-m", "gpu",
                          "-k", "test_gemm_matches_fp64 or test_gemm_tensor_core_path_is_repeatable"],
                         env=env, capture_output=True, text=True, timeout=600)
    assert res.returncode == 0, res.stdout[-2000:] + res.stderr[-2000:]


@pytest.mark.parametrize("a_kmajor,b_kmajor", [(1, 0), (1, 1), (0, 0), (0, 1)])
@pytest.mark.parametrize("scale_log2", [0, 40, -40])
def test_gemm_fp16_halves_match_fp64_and_follow_the_scale(lib, a_kmajor, b_kmajor, scale_log2):
    """256-column products with a caller-supplied bound on |A| split their operands into two FP16 halves with
    power-of-two scales (bsq_gemm_bounded).  Same tolerance against FP64 as the TF32 halves; scaling A by a power of two
    must scale the result by exactly that power (the split sees the same halves); a bound above the true maximum is
    allowed."""
    M, N, K = 1024, 256, 2048
    a, b = operands(M, N, K, a_kmajor, b_kmajor, 5)
    ws = torch.zeros(64 << 20, dtype=torch.uint8, device="cuda")

    def run_bounded(a_op, bound):
        c = torch.full((M, N), float("nan"), device="cuda", dtype=torch.float32)
        st = torch.zeros(1, dtype=torch.int32, device="cuda")
        word = torch.tensor([bound], dtype=torch.float32, device="cuda")
        rc = lib.bsq_gemm_bounded(int(a_kmajor), int(b_kmajor), a_op.data_ptr(), a_op.shape[1], b.data_ptr(), b.shape[1], c.data_ptr(), N,
                                  M, N, K, ws.data_ptr(), ws.numel(), word.data_ptr(), st.data_ptr(), None)
        torch.cuda.synchronize()
        assert rc == 0 and int(st.item()) == 0
        return c
    base = run_bounded(a, float(a.abs().max()))
    want, mag = product_fp64(a, b, a_kmajor, b_kmajor)
    # 22 significant bits per operand element, FP32 accumulation: a few 1e-6 of sum |a||b|
    assert float(((base.double() - want).abs() / mag).max()) <= 4e-6
    f = float(2.0 ** scale_log2)
    scaled = run_bounded(a * f, float(a.abs().max()) * f * 1.7)        # (a bound that is not tight)
    assert torch.equal(scaled, base * f)
    # elements far below the largest still count: rows of A shrunk by 2^-20 give rows of C shrunk alike, to FP32 accuracy
    a2 = a.clone()
    rows = slice(0, 64)
    if a_kmajor:
        a2[rows, :] *= 2.0 ** -20
    else:
        a2[:, rows] *= 2.0 ** -20
    small = run_bounded(a2, float(a2.abs().max()))
    # (this is the FP16 path: a bound 2^6 below the true maximum leaves FP16's range, and the result says so)
    assert not bool(torch.isfinite(run_bounded(a, float(a.abs().max()) / 64.0)).all())
    assert float(((small[rows].double() - want[rows] * 2.0 ** -20).abs() / (mag[rows] * 2.0 ** -20)).max()) <= 2e-5
