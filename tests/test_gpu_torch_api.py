"""The PyTorch door (bitsqueeze-llm_b200/torch_api.py): CUDA tensors in, packed objects in CUDA memory out, ordered after
PyTorch's current stream; checked against the public bitsqz_llm_compress / decompress of the same library."""
import importlib

import numpy as np
import pytest

from conftest import make_c2_like

pytestmark = pytest.mark.gpu
torch = pytest.importorskip("torch")


def masked(b):
    out = np.array(b, dtype=np.uint8, copy=True)
    out[192:200] = 0
    return out


@pytest.mark.parametrize("cfg", [
    dict(rows=256, cols=4096, outlier=0.01, error=0.0, rank=-1, niters=1, uv=-1, s=-1, q=10),
    dict(rows=512, cols=1024, outlier=0.01, error=0.02, rank=64, niters=2, uv=11, s=-1, q=-1),
])
def test_torch_compressor_matches_public_calls(pkg, lib, cfg):
    T = importlib.import_module(pkg.__name__ + ".torch_api")
    rows, cols = cfg["rows"], cfg["cols"]
    x = make_c2_like(rows, cols, 5)
    if cfg["rank"] >= 1:
        rng = np.random.default_rng(6)
        x = (rng.standard_normal((rows, 16)) @ rng.standard_normal((16, cols)) + 0.05 * x).astype(np.float32)
    args = (rows, cols, cfg["outlier"], cfg["error"], cfg["rank"], cfg["niters"], cfg["uv"], cfg["s"], cfg["q"])
    d_x = torch.from_numpy(x).cuda()
    assert lib.bsq_compress_initialize(*args, pkg.INPUT_DEVICE) == 0
    hdr, want = pkg.compress_to_bytes(d_x.data_ptr())
    lib.bsq_compress_release()
    comp = T.Compressor(**cfg)
    # the input is produced on a side stream just before the call: the compressor must wait for it
    side = torch.cuda.Stream()
    with torch.cuda.stream(side):
        d_in = torch.zeros_like(d_x)
        for _ in range(20):
            d_in.add_(d_x, alpha=0.05)                     # 20 kernels, so that the producer is still running
        d_in.copy_(d_x)
        packed = comp.compress(d_in)
        y = comp.decompress(packed)
        y2 = comp.decompress(packed.to_bytes())             # from serialised bytes as well
    torch.cuda.synchronize()
    assert packed.nbytes == want.size and np.array_equal(masked(packed.to_bytes()), masked(want))
    eff = hdr.effective_rank if cfg["rank"] >= 1 else cfg["rank"]
    assert lib.bsq_decompress_initialize(rows, cols, cfg["outlier"], cfg["error"], eff, cfg["uv"], cfg["s"], cfg["q"]) == 0
    d_y = torch.zeros((rows, cols), dtype=torch.float32, device="cuda")
    assert pkg.decompress_packed(want, d_y.data_ptr(), rows * cols) == 0
    torch.cuda.synchronize()
    lib.bsq_decompress_release()
    assert torch.equal(y.view(torch.int32), d_y.view(torch.int32)) and torch.equal(y2.view(torch.int32), d_y.view(torch.int32))
    # two calls in flight: compress of one matrix while another is being decompressed
    p1 = comp.compress_async(d_x)
    p2 = comp.decompress_async(packed)
    assert np.array_equal(masked(p1.wait().to_bytes()), masked(want)) and torch.equal(p2.wait().view(torch.int32), d_y.view(torch.int32))
    with pytest.raises(ValueError):
        comp.compress(d_x[:, :-1])
    comp.close()
