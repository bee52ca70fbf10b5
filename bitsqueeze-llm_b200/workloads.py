"""Seeded synthetic inputs and settings of the five benchmark configurations of this path.

The reference ships no dataset and names no public benchmark: its workload is a description of matrices
(shape, value distribution, seed).  This module builds those matrices -- on the host with numpy for the
two quantiser-only configurations, on the GPU with torch for the low-rank ones, whose construction needs
QR factorisations of tall Gaussian matrices -- and lists the settings each configuration is run with.
The benchmark and the parity tests both take their inputs from here, so that they measure and check the
same thing.  Nothing in here computes any part of the compress/decompress path.

  C1  1024 x 1024   N(0,1)                                                     NF4, nothing else, host input
  C2  4096 x 4096   N(0,1), 0.1 % of the columns scaled by U[20,100]           outlier 0.01 + NF4_DQ
  C3  8192 x 4096   G1 diag(1/i) G2^T + 0.01 N(0,1), 512 components            rank 128, 2 iterations, FP32 factors
  C4  8192 x 4096   C3's construction + 0.05 % columns x 50 + 1 % Student-t(3)  outlier 0.005, rank 256, NF4 U/V, error 0.01
  C5A 4096 x 14336  C4's construction, one seed per layer, 32 layers            as C4; matrices are independent
  C5B 65536 x 4096  C3's construction, held as row shards                      rank 128, 2 iterations (row-sharded SVD)
"""
import numpy as np

NONE, NF4_DQ, NF4 = -1, 10, 11

# settings of bitsqz_llm_compress_initialize per configuration
CONFIGS = {
    "C1": dict(rows=1024, cols=1024, outlier=0.0, error=0.0, rank=-1, niters=1, uv=NONE, s=NONE, q=NF4),
    "C2": dict(rows=4096, cols=4096, outlier=0.01, error=0.0, rank=-1, niters=1, uv=NONE, s=NONE, q=NF4_DQ),
    "C3": dict(rows=8192, cols=4096, outlier=0.0, error=0.0, rank=128, niters=2, uv=NONE, s=NONE, q=NONE),
    "C4": dict(rows=8192, cols=4096, outlier=0.005, error=0.01, rank=256, niters=2, uv=NF4, s=NONE, q=NONE),
    "C5A": dict(rows=4096, cols=14336, outlier=0.005, error=0.01, rank=256, niters=2, uv=NF4, s=NONE, q=NONE),
}
C5A_LAYERS = 32
C5A_BASE_SEED = 5000
C5B = dict(rows=65536, cols=4096, rank=128, niters=2, seed=77)
SLICE_BAND = 2048          # rows per independently seeded band of a row-sliced matrix (lowrank_matrix)


def c1_matrix(seed=1):
    return np.random.default_rng(seed).standard_normal((1024, 1024)).astype(np.float32)


def c2_matrix(seed=2, rows=4096, cols=4096, outlier_frac=0.001):
    """N(0,1) with round(outlier_frac * cols) columns (at least one) scaled by their own factor from U[20,100]."""
    rng = np.random.default_rng(seed)
    x = rng.standard_normal((rows, cols), dtype=np.float32)
    ncol = max(1, int(round(outlier_frac * cols)))
    for c in rng.choice(cols, size=ncol, replace=False):
        x[:, c] *= np.float32(rng.uniform(20.0, 100.0))
    return x


def lowrank_matrix(torch, rows, cols, seed, llama_like=False, components=512, noise=0.01, device="cuda", row_slice=None):
    """A = G1 diag(1/i) G2^T + noise N(0,1) as FP32 on `device`; G1, G2: Q factors of seeded Gaussian matrices (FP64).

    llama_like adds what configuration 4 describes: round(0.0005 cols) columns times 50 and, on a seeded Bernoulli(0.01)
    mask, an added Student-t(3) sample (scaled like the noise).  row_slice = (first, count) returns only those rows
    of the same matrix (the row shards of C5B are slices of one matrix).
    """
    g = torch.Generator(device=device).manual_seed(int(seed))
    f64 = torch.float64
    g1, _ = torch.linalg.qr(torch.randn(rows, components, device=device, generator=g, dtype=f64))
    g2, _ = torch.linalg.qr(torch.randn(cols, components, device=device, generator=g, dtype=f64))
    sv = torch.arange(1, components + 1, device=device, dtype=f64) ** -1.0
    if row_slice is not None:
        # the noise of a slice is drawn per band of SLICE_BAND rows with a seed of its own, so that every slicing of
        # the same matrix into whole bands sees the same values (32768 rows over 8 ranks are 4096 rows each)
        first, count = row_slice
        if first % SLICE_BAND or count % SLICE_BAND or count <= 0 or first + count > rows or llama_like:
            raise ValueError("row_slice must be whole bands of %d rows inside the matrix (and not llama_like)" % SLICE_BAND)
        out = torch.empty(count, cols, device=device, dtype=torch.float32)
        for b in range(count // SLICE_BAND):
            band = (first // SLICE_BAND) + b
            gb = torch.Generator(device=device).manual_seed(int(seed) * 1000 + band)
            rows_b = slice((first + b * SLICE_BAND), (first + (b + 1) * SLICE_BAND))
            a = (g1[rows_b] * sv) @ g2.T + noise * torch.randn(SLICE_BAND, cols, device=device, generator=gb, dtype=f64)
            out[b * SLICE_BAND:(b + 1) * SLICE_BAND] = a.float()
        return out.contiguous()
    a = (g1 * sv) @ g2.T + noise * torch.randn(rows, cols, device=device, generator=g, dtype=f64)
    if llama_like:
        chosen = torch.randperm(cols, device=device, generator=g)[: max(1, round(0.0005 * cols))]
        a[:, chosen] *= 50.0
        mask = torch.rand(rows, cols, device=device, generator=g) < 0.01
        z = torch.randn(rows, cols, device=device, generator=g, dtype=f64)
        chi = torch.zeros(rows, cols, device=device, dtype=f64)
        for _ in range(3):                                     # chi-square with 3 degrees of freedom, one term at a time
            chi += torch.randn(rows, cols, device=device, generator=g, dtype=f64) ** 2
        a = torch.where(mask, a + noise * z / (chi / 3.0).sqrt(), a)
    return a.float().contiguous()


def config_matrix(torch, name, layer=0, device="cuda"):
    """The input of configuration `name` as an FP32 torch tensor on `device` (C5A: layer 0..31)."""
    name = name.upper()
    cfg = CONFIGS[name]
    if name == "C1":
        return torch.from_numpy(c1_matrix()).to(device)
    if name == "C2":
        return torch.from_numpy(c2_matrix()).to(device)
    if name == "C3":
        return lowrank_matrix(torch, cfg["rows"], cfg["cols"], 3, llama_like=False, device=device)
    if name == "C4":
        return lowrank_matrix(torch, cfg["rows"], cfg["cols"], 4, llama_like=True, device=device)
    if name == "C5A":
        return lowrank_matrix(torch, cfg["rows"], cfg["cols"], C5A_BASE_SEED + int(layer), llama_like=True, device=device)
    raise KeyError(name)


def describe(name):
    cfg = CONFIGS[name.upper()]
    fmt = {NONE: "FP32", NF4: "NF4", NF4_DQ: "NF4_DQ"}
    if cfg["rank"] >= 1:
        core = "rank %d, %d power iterations, U/V %s, S %s" % (cfg["rank"], cfg["niters"], fmt[cfg["uv"]], fmt[cfg["s"]])
    else:
        core = "no SVD, %s" % fmt[cfg["q"]]
    return "%dx%d FP32, outlier_topk=%g, %s, error_correction_topk=%g" % (cfg["rows"], cfg["cols"], cfg["outlier"], core, cfg["error"])
