"""The CMake package of the library: a consumer written for the reference's `find_package(bitsqz_llm)` target configures,
builds and links against this tree's shared library (no GPU needed: the program only calls host-side functions)."""
import os
import shutil
import subprocess

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))

CONSUMER_CMAKE = """cmake_minimum_required(VERSION 3.18)
project(bsq_consumer CXX)
find_package(bitsqz_llm CONFIG REQUIRED)
add_executable(consumer main.cpp)
target_link_libraries(consumer PRIVATE bitsqz_llm::bitsqz_llm)
"""

CONSUMER_MAIN = """#include <bitsqz_llm.hpp>
#include <bitsqz_llm_c.h>
#include <cstdio>
#include <cstring>
#include <vector>
int main() {
    // host-side entry points only: sizes, loading a (malformed) buffer, the helper of the top-k module
    if (bitsqz_llm_get_packed_size(nullptr) != 0) return 1;
    std::vector<unsigned char> junk(sizeof(bitsqz_llm_array_t) + 64, 0xAB);
    if (load_bitsqz_llm_from_buffer(junk.data(), junk.size()) != nullptr) return 2;
    if (topk_compute_num_topk_columns(4096, 0.01f) != 41) return 3;
    if (bsq_topk_num_columns(14336, 0.005f) != 72) return 4;
    std::printf("%s\\n", bsq_build_info());
    return 0;
}
"""


def test_cmake_consumer_builds_and_runs(built, tmp_path):
    cmake = shutil.which("cmake")
    if cmake is None:
        pytest.skip("cmake not on PATH")
    (tmp_path / "CMakeLists.txt").write_text(CONSUMER_CMAKE)
    (tmp_path / "main.cpp").write_text(CONSUMER_MAIN)
    build = tmp_path / "build"
    env = dict(os.environ)
    env.pop("CC", None)
    env.pop("CXX", None)              # a toolchain wrapper named there may lack parts; the default compiler will do
    cfg = subprocess.run([cmake, "-S", str(tmp_path), "-B", str(build),
                          "-Dbitsqz_llm_DIR=" + os.path.join(ROOT, "bitsqueeze-llm_b200", "cmake")],
                         capture_output=True, text=True, env=env)
    assert cfg.returncode == 0, cfg.stdout + cfg.stderr
    bld = subprocess.run([cmake, "--build", str(build)], capture_output=True, text=True, env=env)
    assert bld.returncode == 0, bld.stdout + bld.stderr
    run = subprocess.run([str(build / "consumer")], capture_output=True, text=True)
    assert run.returncode == 0, (run.returncode, run.stdout, run.stderr)
    assert "sm_100a" in run.stdout


def test_row_slices_of_the_sharded_workload_agree():
    """The row shards of the tall matrix (bench.py's row-sharded leg) are slices of ONE matrix: whatever the number of
    ranks, a row must get the same values (the leg's 8-rank parity run slices 32768 rows into 4096-row shards)."""
    torch = pytest.importorskip("torch")
    import importlib
    W = importlib.import_module("bitsqueeze-llm_b200.workloads")
    rows, cols, band = 4 * W.SLICE_BAND, 128, W.SLICE_BAND
    whole = W.lowrank_matrix(torch, rows, cols, 7, components=32, device="cpu", row_slice=(0, rows))
    for ranks in (2, 4):
        per = rows // ranks
        parts = [W.lowrank_matrix(torch, rows, cols, 7, components=32, device="cpu", row_slice=(r * per, per)) for r in range(ranks)]
        assert torch.equal(torch.cat(parts), whole)
    for bad in ((1, band), (0, band + 1), (rows, band), (0, 0)):
        with pytest.raises(ValueError):
            W.lowrank_matrix(torch, rows, cols, 7, components=32, device="cpu", row_slice=bad)
