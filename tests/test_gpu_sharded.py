"""Row-sharded randomized SVD on two GPUs (one process per GPU, NCCL all-reduce of the Gram matrices and
partial products) against the unsharded run on one GPU.  Skipped with fewer than two devices."""
import os
import subprocess
import sys

import numpy as np
import pytest

pytestmark = pytest.mark.gpu
torch = pytest.importorskip("torch")
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))

WORKER = r'''
import os, sys, time, ctypes as C
import numpy as np, torch
sys.path.insert(0, os.environ["BSQ_ROOT"])
import __graft_entry__ as entry
rank, world, tmp = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"]), os.environ["BSQ_TMP"]
torch.cuda.set_device(rank)
pkg = entry.load_package(); L = pkg.lib()
idf = os.path.join(tmp, "id.bin")
if rank == 0:
    buf = (C.c_char * 128)()
    assert L.bsq_shard_unique_id(buf, 128) == 0
    open(idf + ".tmp", "wb").write(bytes(buf)); os.rename(idf + ".tmp", idf)
for _ in range(600):
    if os.path.exists(idf): break
    time.sleep(0.05)
uid = open(idf, "rb").read()
comm = L.bsq_shard_comm_create(uid, rank, world)
assert comm
a = np.load(os.path.join(tmp, "a.npy"))
m, n = a.shape
k, niter = int(os.environ["BSQ_K"]), 2
rows = m // world
mine = torch.from_numpy(a[rank * rows:(rank + 1) * rows].copy()).cuda()
u = torch.zeros((rows, k), device="cuda"); s = torch.zeros(k, device="cuda"); v = torch.zeros((n, k), device="cuda")
assert L.bsq_svd_lowrank_sharded(comm, mine.data_ptr(), rows, m, n, k, niter, 1241, u.data_ptr(), s.data_ptr(), v.data_ptr(), None) == 0
torch.cuda.synchronize()
# the same through a workspace that lives across calls: two calls, both bit-identical to the one-shot call
h = L.bsq_shard_svd_create(comm, rows, m, n, k, niter)
assert h
u2 = torch.zeros_like(u); s2 = torch.zeros_like(s); v2 = torch.zeros_like(v)
for _ in range(2):
    u2.zero_(); s2.zero_(); v2.zero_()
    assert L.bsq_shard_svd_run(h, mine.data_ptr(), 1241, u2.data_ptr(), s2.data_ptr(), v2.data_ptr(), None) == 0
    assert torch.equal(u2.view(torch.int32), u.view(torch.int32)) and torch.equal(s2.view(torch.int32), s.view(torch.int32))
    assert torch.equal(v2.view(torch.int32), v.view(torch.int32))
# this rank's shard as an ordinary packed object, decompressed by the unchanged public call
obj = C.c_void_p(None)
assert L.bsq_shard_compress(h, mine.data_ptr(), 1241, C.byref(obj), None) == 0
hdr = pkg.Array.from_buffer_copy(C.string_at(obj.value, 200))
assert (hdr.num_rows, hdr.num_columns, hdr.effective_rank, hdr.flags) == (rows, n, k, pkg.FLAG_SVD)
assert int(L.bsq_get_packed_size(obj)) == 200 + (rows * k + k + n * k) * 4
assert L.bsq_decompress_initialize(rows, n, 0.0, 0.0, k, -1, -1, -1) == 0
y = torch.zeros((rows, n), device="cuda")
assert L.bsq_decompress(obj, y.data_ptr(), rows * n) == 0
torch.cuda.synchronize()
want = (u.double() * s.double()) @ v.double().T
assert float((y.double() - want).norm() / want.norm()) <= 1e-6
L.bsq_free(obj); L.bsq_decompress_release()
L.bsq_shard_svd_destroy(h)
np.savez(os.path.join(tmp, f"out{rank}.npz"), u=u.cpu().numpy(), s=s.cpu().numpy(), v=v.cpu().numpy(),
         peer=np.int32(L.bsq_shard_uses_peer_exchange(comm)))
L.bsq_shard_comm_destroy(comm)
'''


@pytest.mark.parametrize("peer", ["1", "0"], ids=["peer-exchange", "nccl-only"])
def test_row_sharded_svd_matches_unsharded(lib, tmp_path, peer):
    """peer-exchange: the k x k all-reduces run as one kernel over peer memory where the ranks can map each other's
    memory (falls back to NCCL otherwise, which the saved flag tells); nccl-only: BSQ_SHARD_PEER=0."""
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    from test_gpu_svd import lowrank_plus_noise, rel_frob, svd_gpu
    m, n, k = 4096, 1024, 64
    a = lowrank_plus_noise(m, n, 48, 1e-4, 5)
    np.save(tmp_path / "a.npy", a)
    (tmp_path / "worker.py").write_text(WORKER)
    procs = []
    for rank in range(2):
        env = dict(os.environ, RANK=str(rank), WORLD_SIZE="2", BSQ_ROOT=ROOT, BSQ_TMP=str(tmp_path), BSQ_K=str(k),
                   NCCL_NVLS_ENABLE="0", BSQ_SHARD_PEER=peer)
        procs.append(subprocess.Popen([sys.executable, str(tmp_path / "worker.py")], env=env, stdout=subprocess.PIPE,
                                      stderr=subprocess.PIPE, text=True))
    try:
        outs = [p.communicate(timeout=300) for p in procs]
    finally:
        for p in procs:                      # a rank stuck in communicator set-up must not keep its GPU
            if p.poll() is None:
                p.kill()
    assert all(p.returncode == 0 for p in procs), outs
    r0, r1 = np.load(tmp_path / "out0.npz"), np.load(tmp_path / "out1.npz")
    assert int(r0["peer"]) == int(r1["peer"])                  # both ranks agree on how they exchange
    if peer == "0":
        assert int(r0["peer"]) == 0
    # replicated factors are bit-identical on both ranks
    assert np.array_equal(r0["s"].view(np.uint32), r1["s"].view(np.uint32))
    assert np.array_equal(r0["v"].view(np.uint32), r1["v"].view(np.uint32))
    u = np.concatenate([r0["u"], r1["u"]], axis=0)
    s, v = r0["s"], r0["v"]
    u1, s1, v1 = svd_gpu(lib, a, k, 2)
    e_sharded, e_single = rel_frob(a, (u * s) @ v.T), rel_frob(a, (u1 * s1) @ v1.T)
    assert abs(e_sharded - e_single) <= 1e-4, (e_sharded, e_single)              # same tolerance as against the reference
    assert np.max(np.abs(s[:16] - s1[:16]) / s1[:16]) <= 1e-4
    assert np.abs(u.T @ u - np.eye(k))[:40, :40].max() <= 1e-3
