"""Generates tests/golden/nf4_golden.npz and tests/golden/rand_fixture.json from the REFERENCE's own
CPU quantiser (oracle/_ref/libref_cpu.so = legacy_modules/quantization compiled unmodified).

Run where the reference tree is available:   make -C oracle && python tests/golden/make_golden.py

nf4_golden.npz   small seeded inputs (ragged lengths, specials, outlier-dominated blocks) with the
                 reference's NF4 scales/nibbles and NF4_DQ dq/scale codes/nibbles.
rand_fixture.json  SHA-256 of the reference's outputs on the fixture its own GPU-vs-CPU tests use
                 (tests/quantization_cuda/test_nf4_cuda.cu, test_nf4_dq_cuda.cu: 2^20 values,
                 uniform[-10, 10] from glibc srand(seed)/rand(), seeds 12345 and 54321); the input is
                 regenerated at test time, only digests are stored.
"""
import ctypes
import hashlib
import json
import os
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.join(HERE, "..", "..", "oracle"))
from oracle import RefCpu  # noqa: E402


def glibc_uniform(seed, n, lo=-10.0, hi=10.0):
    """utils/random.hpp:8-35 of the reference: u = (float)rand() / (float)RAND_MAX; lo + u * (hi - lo)."""
    libc = ctypes.CDLL("libc.so.6")
    libc.srand(ctypes.c_uint(seed))
    r = np.fromiter((libc.rand() for _ in range(n)), dtype=np.int64, count=n)
    u = r.astype(np.float32) / np.float32(2147483647)
    return (np.float32(lo) + u * np.float32(hi - lo)).astype(np.float32)


def cases():
    rng = np.random.default_rng(20240611)
    out = {}
    for n in (1, 2, 63, 64, 65, 127, 129, 1000, 4096):
        out[f"normal_{n}"] = rng.standard_normal(n).astype(np.float32)
    x = rng.standard_normal(1024).astype(np.float32)
    x[::7] = 0.0
    x[5] = np.inf
    x[70] = -np.inf
    x[200] = np.nan
    x[640:704] = 0.0                       # an all-zero block
    out["specials_1024"] = x
    x = (rng.standard_normal(2048) * 1e-3).astype(np.float32)
    x[100] = 3.0e4                         # one huge block: other blocks' E4M3 scale codes underflow
    out["outlier_block_2048"] = x
    x = rng.standard_normal(513).astype(np.float32) * np.float32(1e-30)
    out["tiny_513"] = x
    out["denormal_130"] = (rng.standard_normal(130) * 1e-41).astype(np.float32)
    x = rng.standard_normal(777).astype(np.float32)
    x[300] = 2.0e9                          # a scale-1.0 fallback block next to a huge maximum
    x[0:64] *= np.float32(3000.0)
    out["huge_777"] = x
    t = rng.standard_t(3, 3000).astype(np.float32)
    out["student_t_3000"] = t
    return out


def main():
    ref = RefCpu()
    blob = {}
    for name, x in cases().items():
        s, d = ref.nf4_quantize(x)
        dq, c, d2 = ref.nf4dq_quantize(x)
        blob[name + ".x"] = x
        blob[name + ".nf4_scales"] = s
        blob[name + ".nf4_data"] = d
        blob[name + ".dq"] = np.array([dq], np.float32)
        blob[name + ".dq_codes"] = c
        blob[name + ".dq_data"] = d2
        blob[name + ".nf4_deq"] = ref.nf4_roundtrip(x)
        blob[name + ".dq_deq"] = ref.nf4dq_roundtrip(x)
    np.savez_compressed(os.path.join(HERE, "nf4_golden.npz"), **blob)
    fixture = {}
    for seed in (12345, 54321):
        x = glibc_uniform(seed, 1 << 20)
        s, d = ref.nf4_quantize(x)
        dq, c, d2 = ref.nf4dq_quantize(x)
        fixture[str(seed)] = {
            "input_sha256": hashlib.sha256(x.tobytes()).hexdigest(),
            "nf4_scales_sha256": hashlib.sha256(s.tobytes()).hexdigest(),
            "nf4_data_sha256": hashlib.sha256(d.tobytes()).hexdigest(),
            "dq_bits": int(np.array([dq], np.float32).view(np.uint32)[0]),
            "dq_codes_sha256": hashlib.sha256(c.tobytes()).hexdigest(),
            "dq_data_sha256": hashlib.sha256(d2.tobytes()).hexdigest(),
            "nf4_deq_sha256": hashlib.sha256(ref.nf4_roundtrip(x).tobytes()).hexdigest(),
            "dq_deq_sha256": hashlib.sha256(ref.nf4dq_roundtrip(x).tobytes()).hexdigest(),
        }
    with open(os.path.join(HERE, "rand_fixture.json"), "w") as f:
        json.dump(fixture, f, indent=1)
    print("wrote", len(blob), "arrays and", len(fixture), "digests")


if __name__ == "__main__":
    main()
