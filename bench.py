"""Benchmark of the bitsqz_llm compress/decompress hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--lanes L]

Workload (the largest configuration of the path, benchmark configuration 5, configs[4]): a batch of 32 independent FP32 activation
matrices of 4096 x 14336 (per-layer seeds, seeded synthetic: low-rank + noise + outlier channels + heavy-tailed
entries, bitsqueeze-llm_b200/workloads.py), full pipeline: outlier top-k 0.005, randomized SVD rank 256 with 2 power
iterations, U/V in NF4, S in FP32, error-correction top-k 0.01; compress AND decompress.  Matrix i belongs to rank
i % N (one process per GPU, no collective on the data path: the matrices are independent; the batch is fixed, so more
GPUs means fewer matrices per GPU: strong scaling).  A step is one pass over the rank's share of the batch: every matrix compressed, then every object
decompressed.  Inputs (235 MB each) are larger than the L2.

  value   FP32 bytes of the whole batch / time of a step, inputs resident in HBM, packed objects left in device
          memory (device-resident objects through the batch entry points, `lanes` matrices in flight per GPU); CUDA
          events, barrier + synchronize on both sides, max over ranks.  compress / decompress are reported separately
          beside it, and the same with one matrix at a time (lanes = 1).
  e2e     the same step with HOST buffers: matrices in pinned host memory, packed objects returned as host objects
          (the public object format), decompress from those host objects; host<->device copies inside the timed region.
  roofline      the TMA-fed tcgen05 3xTF32 product kernel (gemm_tc_tma_kernel: the six products of the range finder with
                the 4096 x 14336 matrix), timed by CUDA events on its stream in a one-lane pass; FLOPs 2 M N K per launch
                against the TF32 dense rate measured in this run / 3.
  cpu_baseline  rank 0, N=1: the only stage of this pipeline the reference can run on a CPU -- its OpenMP NF4 quantiser
                (oracle/_ref/libref_cpu.so) on arrays of U's and V's size -- on all host cores.

--impl reference times the reference's own CUDA build (oracle/_ref/libref_cuda.so, its five .cu files compiled
unmodified for sm_100) on the same batch through its public calls, on rank 0's GPU (the reference has no multi-GPU
mode and no CPU path for top-k, SVD or reconstruction).
--single C3|C4|C5A times the public compress / decompress calls on one matrix of that configuration (a side
measurement for profiles; with --impl reference through the reference's CUDA build).
"""
import argparse
import ctypes as C
import json
import math
import os
import statistics
import subprocess
import sys
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)
import __graft_entry__ as entry  # noqa: E402

METRIC = "FP32-input GB/s, compress+decompress of 32 x (4096x14336) FP32 matrices, full pipeline"
WORKLOAD = ("configs[4]: 32 independent 4096x14336 FP32 matrices, outlier_topk=0.005, SVD rank 256 (2 power iterations), "
            "U/V NF4, S FP32, error_correction_topk=0.01, compress+decompress, matrix i on rank i % N")
# kernels this library launches per matrix in this configuration, counted from an ncu launch list of
# `python bench.py --single C5A` (all launches of the run, minus the decompress calls', divided by the compress calls)
LAUNCHES_PER_COMPRESS = 59
LAUNCHES_PER_DECOMPRESS = 9
# DRAM bytes of one 4096x14336x256 product launch of gemm_tc_tma_kernel (ncu, read + write): 239.8-242.7 MB for W X (matrix
# read along M), 250.0-251.9 MB for W^T X (read along K); the matrix itself is 234.9 MB, so it is read once.
PRODUCT_DRAM_BYTES_PER_LAUNCH = 245.7e6


def workloads():
    import importlib
    entry.load_package()
    return importlib.import_module(entry.PKG_NAME + ".workloads")


def load_shard():
    import importlib
    entry.load_package()
    return importlib.import_module(entry.PKG_NAME + ".shard")


def measured_peaks():
    try:
        with open(os.path.join(ROOT, "MEASURED_PEAKS.json")) as f:
            d = json.load(f)
        return float(d["hbm_gbs"]), float(d["bf16_tflops"]), "measured"
    except Exception:
        return 6650.0, 1590.0, "fallback"


def host_threads():
    try:
        return len(os.sched_getaffinity(0))
    except AttributeError:
        return os.cpu_count() or 1


class ClockSampler:
    """nvidia-smi clock / throttle-reason samples taken while the timed region runs."""
    Q = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,"
         "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
         "clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index):
        self.gpu = gpu_index
        self.proc = None

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", "-i", str(self.gpu), "--query-gpu=" + self.Q,
                                          "--format=csv,noheader,nounits", "-lms", "100"],
                                         stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
        except OSError:
            self.proc = None

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.25)
        self.proc.terminate()
        try:
            out, _ = self.proc.communicate(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
            out, _ = self.proc.communicate()
        sm, smax, power, reasons = [], [], [], set()
        for line in out.splitlines():
            f = [t.strip() for t in line.split(",")]
            if len(f) < 9:
                continue
            try:
                sm.append(float(f[1]))
                smax.append(float(f[2]))
                power.append(float(f[3]))
            except ValueError:
                continue
            for name, v in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), f[5:9]):
                if v.lower().startswith("active"):
                    reasons.add(name)
        busy = [v for v in sm if v >= 0.5 * max(sm)] if sm else []
        return {"sm_mhz": statistics.median(busy) if busy else None, "sm_max_mhz": max(smax) if smax else None,
                "power_w_max": max(power) if power else None, "samples": len(sm), "reasons": sorted(reasons)}


def bind_near_gpu(gpu_index):
    """Best effort: run this process (and so first-touch its pinned host buffers) on the NUMA node the GPU hangs off.
    Changes only this process's CPU affinity.  Returns a short description for the bench line."""
    try:
        bus = subprocess.run(["nvidia-smi", "-i", str(gpu_index), "--query-gpu=pci.bus_id", "--format=csv,noheader"],
                             capture_output=True, text=True, timeout=20).stdout.strip().lower()
        if not bus:
            return "unknown (no bus id)"
        dom, rest = bus.split(":", 1)
        path = "/sys/bus/pci/devices/%s:%s/numa_node" % (dom[-4:], rest)
        node = int(open(path).read().strip())
        if node < 0:
            return "no NUMA information for %s" % bus
        cpus = set()
        for part in open("/sys/devices/system/node/node%d/cpulist" % node).read().strip().split(","):
            lo, _, hi = part.partition("-")
            cpus.update(range(int(lo), int(hi or lo) + 1))
        allowed = os.sched_getaffinity(0)
        use = cpus & allowed
        if not use:
            return "GPU on node %d, but this process may only run on other nodes' CPUs: left as it is" % node
        os.sched_setaffinity(0, use)
        return "bound to the %d CPUs of NUMA node %d next to the GPU" % (len(use), node)
    except Exception as e:                                   # noqa: BLE001 -- any failure just leaves the affinity alone
        return "not bound (%s)" % type(e).__name__


def rel_frob(x, y):
    return float((x.double() - y.double()).norm() / x.double().norm())


# ----------------------------------------------------------------------------------------------------------------
# the reference arm
# ----------------------------------------------------------------------------------------------------------------
def cpu_nf4_baseline(W, budget_s=12.0):
    """The reference's OpenMP NF4 quantiser on arrays of the size of U and V of one matrix, all host threads."""
    orc = entry.load_oracle()
    try:
        q = orc.RefCpu()
        kind = "reference"
    except (FileNotFoundError, OSError):
        q = orc.Oracle()
        kind = "port"
    threads = host_threads()
    q.set_threads(threads)                   # a launcher may have exported OMP_NUM_THREADS=1
    cfg = W.CONFIGS["C5A"]
    rng = np.random.default_rng(5)
    u = rng.standard_normal(cfg["rows"] * cfg["rank"]).astype(np.float32) / 64
    v = rng.standard_normal(cfg["cols"] * cfg["rank"]).astype(np.float32) / 64
    q.nf4_quantize(u)
    reps, t0 = 0, time.perf_counter()
    while reps < 3 or (time.perf_counter() - t0 < budget_s and reps < 2000):
        q.nf4_quantize(u)
        q.nf4_quantize(v)
        reps += 1
    dt = time.perf_counter() - t0
    return {"value": (u.size + v.size) * 4 * reps / dt / 1e9, "unit": "GB/s (FP32 input of the NF4 stage)", "cores": q.max_threads(),
            "kind": kind,
            "sample": "%d x NF4 of U (%d) and V (%d floats) of one matrix in %.1f s: the reference's legacy OpenMP quantiser, "
                      "the one stage of this pipeline with a CPU path" % (reps, u.size, v.size, dt)}


def run_reference(args, rank):
    """--impl reference: the reference's own CUDA build on the same batch, rank 0 only."""
    if rank != 0:
        return
    W = workloads()
    base = {"impl": "reference", "metric": METRIC, "unit": "GB/s", "n_gpus": args.gpus, "steps": args.steps,
            "warmup": args.warmup, "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "f32",
            "data": "synthetic", "config": {"workload": WORKLOAD}}
    try:
        ref = entry.load_oracle().RefCuda()
    except (FileNotFoundError, OSError) as e:
        print(json.dumps(dict(base, unavailable="oracle/_ref/libref_cuda.so (the reference's CUDA build) is not there: %s" % e)))
        return
    import torch
    torch.cuda.set_device(int(os.environ.get("LOCAL_RANK", "0")))
    cfg = W.CONFIGS["C5A"]
    rows, cols, n = cfg["rows"], cfg["cols"], cfg["rows"] * cfg["cols"]
    mats = [W.config_matrix(torch, "C5A", layer=l) for l in range(W.C5A_LAYERS)]
    L = ref.lib
    assert L.ref_compress_initialize(rows, cols, cfg["outlier"], cfg["error"], cfg["rank"], cfg["niters"], cfg["uv"], cfg["s"], cfg["q"], 1) == 0
    assert L.ref_decompress_initialize(rows, cols, cfg["outlier"], cfg["error"], cfg["rank"], cfg["uv"], cfg["s"], cfg["q"]) == 0
    d_y = torch.zeros((rows, cols), dtype=torch.float32, device="cuda")
    t_c = t_d = 0.0

    def step(timed):
        nonlocal t_c, t_d
        objs = []
        torch.cuda.synchronize()
        t0 = time.perf_counter()
        for m in mats:
            o = C.c_void_p(None)
            if L.ref_compress(m.data_ptr(), C.byref(o), None) != 0:
                raise RuntimeError("reference compress failed")
            objs.append(o)
        torch.cuda.synchronize()
        t1 = time.perf_counter()
        for o in objs:
            if L.ref_decompress(o, d_y.data_ptr(), n) != 0:
                raise RuntimeError("reference decompress failed")
        torch.cuda.synchronize()
        t2 = time.perf_counter()
        for o in objs:
            L.ref_free(o)
        if timed:
            t_c += t1 - t0
            t_d += t2 - t1

    warm = max(1, min(args.warmup, 3))
    for _ in range(warm):
        step(False)
    err = rel_frob(mats[-1], d_y)
    sampler = ClockSampler(torch.cuda.current_device())
    sampler.start()
    t0 = time.perf_counter()
    for _ in range(args.steps):
        step(True)
    dt = time.perf_counter() - t0
    clocks = sampler.stop()
    L.ref_compress_release()
    L.ref_decompress_release()
    total_bytes = len(mats) * n * 4
    gbs = total_bytes * args.steps / dt / 1e9
    cpu = cpu_nf4_baseline(W)
    line = dict(base, value=gbs, ms_per_step=dt / args.steps * 1e3,
                compress={"value": total_bytes * args.steps / t_c / 1e9, "unit": "GB/s", "ms_per_matrix": t_c / args.steps / len(mats) * 1e3},
                decompress={"value": total_bytes * args.steps / t_d / 1e9, "unit": "GB/s (FP32 output)", "ms_per_matrix": t_d / args.steps / len(mats) * 1e3},
                rel_frob_last_layer=err, cpu_baseline=cpu,
                reference_kind="the reference's CUDA build (oracle/_ref/libref_cuda.so) on one B200, device input, its public "
                               "compress / decompress calls, all 32 matrices on rank 0's GPU; wall clock with a device "
                               "synchronise on both sides",
                e2e={"value": gbs, "unit": "GB/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
                gpu_launches=0, clocks=clocks)
    print(json.dumps(line))


# ----------------------------------------------------------------------------------------------------------------
# side measurement: one matrix through the public calls
# ----------------------------------------------------------------------------------------------------------------
def run_single(args):
    import torch
    W = workloads()
    name = args.single.upper()
    cfg = W.CONFIGS[name]
    a = W.config_matrix(torch, name, layer=0)
    m, n = a.shape
    steps, warm = max(3, min(args.steps, 20)), max(2, min(args.warmup, 5))

    def timed(fn):
        for _ in range(warm):
            fn()
        torch.cuda.synchronize()
        ts = []
        for _ in range(steps):
            t0 = time.perf_counter()
            fn()
            torch.cuda.synchronize()
            ts.append((time.perf_counter() - t0) * 1e3)
        return statistics.median(ts)

    out = {"single": name, "impl": args.impl, "shape": [m, n], "steps": steps}
    y = torch.zeros_like(a)
    ci = (m, n, cfg["outlier"], cfg["error"], cfg["rank"], cfg["niters"], cfg["uv"], cfg["s"], cfg["q"], 1)
    di = (m, n, cfg["outlier"], cfg["error"], cfg["rank"], cfg["uv"], cfg["s"], cfg["q"])
    if args.impl == "ours":
        pkg = entry.load_package()
        L = pkg.lib()
        assert L.bsq_compress_initialize(*ci) == 0 and L.bsq_decompress_initialize(*di) == 0
        obj = C.c_void_p(None)
        assert L.bsq_compress(a.data_ptr(), C.byref(obj), None) == 0
        out["bytes"] = int(L.bsq_get_packed_size(obj))

        def compress_call():
            o = C.c_void_p(None)
            assert L.bsq_compress(a.data_ptr(), C.byref(o), None) == 0
            L.bsq_free(o)
        out["compress_ms"] = timed(compress_call)
        out["decompress_ms"] = timed(lambda: L.bsq_decompress(obj, y.data_ptr(), m * n))
        prof = pkg.Profile()
        o = C.c_void_p(None)
        assert L.bsq_compress(a.data_ptr(), C.byref(o), C.byref(prof)) == 0
        L.bsq_free(o)
        out["profile_ms"] = {k: round(getattr(prof, k), 4) for k, _ in prof._fields_}
        L.bsq_free(obj)
        L.bsq_compress_release()
        L.bsq_decompress_release()
    else:
        try:
            ref = entry.load_oracle().RefCuda()
        except (FileNotFoundError, OSError) as e:
            print(json.dumps({"single": name, "impl": "reference", "unavailable": "oracle/_ref/libref_cuda.so not built: %s" % e}))
            return
        R = ref.lib
        assert R.ref_compress_initialize(*ci) == 0 and R.ref_decompress_initialize(*di) == 0
        obj = C.c_void_p(None)
        assert R.ref_compress(a.data_ptr(), C.byref(obj), None) == 0
        out["bytes"] = int(R.ref_get_packed_size(obj))

        def compress_call():
            o = C.c_void_p(None)
            assert R.ref_compress(a.data_ptr(), C.byref(o), None) == 0
            R.ref_free(o)
        out["compress_ms"] = timed(compress_call)
        out["decompress_ms"] = timed(lambda: R.ref_decompress(obj, y.data_ptr(), m * n))
        R.ref_free(obj)
        R.ref_compress_release()
        R.ref_decompress_release()
    out["rel_frob"] = rel_frob(a, y)
    out["fp32_input_gbs_compress"] = m * n * 4 / (out["compress_ms"] * 1e-3) / 1e9
    print(json.dumps(out))


# ----------------------------------------------------------------------------------------------------------------
# extra legs of the main line
# ----------------------------------------------------------------------------------------------------------------
def c2_frontend_leg(torch, pkg, L, W, hbm_peak):
    """Configuration 2 (4096x4096, outlier 0.01 + NF4_DQ): the fused front end's two kernels and the decompress kernel,
    device resident, CUDA events; inputs rotate over 4 matrices (256 MiB > L2)."""
    rows = cols = 4096
    n, nb = rows * cols, rows * cols // 64
    k = L.bsq_topk_num_columns(cols, 0.01)
    d_in = [torch.from_numpy(W.c2_matrix(seed=100 + i)).cuda() for i in range(4)]
    idx = torch.zeros((rows, k), dtype=torch.int16, device="cuda")
    val = torch.zeros((rows, k), dtype=torch.float32, device="cuda")
    dq = torch.zeros(4, dtype=torch.float32, device="cuda")
    codes = torch.zeros(nb, dtype=torch.uint8, device="cuda")
    data = torch.zeros(n // 2, dtype=torch.uint8, device="cuda")
    scr = torch.zeros(L.bsq_frontend_scratch_bytes(rows, cols), dtype=torch.uint8, device="cuda")
    st = torch.zeros(4, dtype=torch.int32, device="cuda")
    outs = [torch.zeros((rows, cols), dtype=torch.float32, device="cuda") for _ in range(4)]
    stream = torch.cuda.current_stream().cuda_stream

    def stage(i):
        if L.bsq_frontend_quantize(10, d_in[i % 4].data_ptr(), rows, cols, k, idx.data_ptr(), val.data_ptr(), None, dq.data_ptr(),
                                   codes.data_ptr(), data.data_ptr(), scr.data_ptr(), st.data_ptr(), stream) != 0:
            raise RuntimeError("bsq_frontend_quantize failed")

    def dstage(i):
        if L.bsq_dequantize_add_topk(10, None, dq.data_ptr(), codes.data_ptr(), data.data_ptr(), rows, cols, idx.data_ptr(),
                                     val.data_ptr(), k, outs[i % 4].data_ptr(), st.data_ptr(), stream) != 0:
            raise RuntimeError("bsq_dequantize_add_topk failed")

    def loop(fn, reps):
        for i in range(10):
            fn(i)
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for i in range(reps):
            fn(i)
        e1.record()
        torch.cuda.synchronize()
        return e0.elapsed_time(e1) / reps
    ms_c = loop(stage, 400)
    ms_d = loop(dstage, 400)

    # two independent matrices in flight on two streams (matrices are the unit of work; outputs and scratch per stream)
    class Out2:
        def __init__(self):
            self.idx, self.val = torch.zeros_like(idx), torch.zeros_like(val)
            self.dq, self.codes, self.data = torch.zeros_like(dq), torch.zeros_like(codes), torch.zeros_like(data)
            self.scr, self.st = torch.zeros_like(scr), torch.zeros_like(st)
            self.stream = torch.cuda.Stream()
    lanes2 = [Out2(), Out2()]

    def stage2(i):
        o = lanes2[i % 2]
        if L.bsq_frontend_quantize(10, d_in[i % 4].data_ptr(), rows, cols, k, o.idx.data_ptr(), o.val.data_ptr(), None, o.dq.data_ptr(),
                                   o.codes.data_ptr(), o.data.data_ptr(), o.scr.data_ptr(), o.st.data_ptr(), o.stream.cuda_stream) != 0:
            raise RuntimeError("bsq_frontend_quantize failed")
    for i in range(10):
        stage2(i)
    torch.cuda.synchronize()
    main = torch.cuda.current_stream()
    f0, f1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    f0.record(main)
    for o in lanes2:
        o.stream.wait_event(f0)
    for i in range(400):
        stage2(i)
    for o in lanes2:
        main.wait_stream(o.stream)
    f1.record(main)
    torch.cuda.synchronize()
    ms_c2 = f0.elapsed_time(f1) / 400
    if int(st[0]) != 0:
        raise RuntimeError("kernel status word set: %d" % int(st[0]))
    ms_pass = (C.c_float * 2)()
    p1, p2 = [], []
    for i in range(16):
        for j in range(3):
            stage(i + j + 1)
        if L.bsq_frontend_quantize_timed(10, d_in[i % 4].data_ptr(), rows, cols, k, idx.data_ptr(), val.data_ptr(), None,
                                         dq.data_ptr(), codes.data_ptr(), data.data_ptr(), scr.data_ptr(), st.data_ptr(), stream,
                                         ms_pass) != 0:
            raise RuntimeError("bsq_frontend_quantize_timed failed")
        p1.append(ms_pass[0])
        p2.append(ms_pass[1])
    bytes_stage = n * 4 + rows * k * 6 + n // 2 + nb + 4
    bytes_p1 = n * 4 + rows * k * 6 + nb * 4
    ach = bytes_stage / (ms_c * 1e-3) / 1e9
    ach_d = bytes_stage / (ms_d * 1e-3) / 1e9
    return {"workload": "configs[1]: " + W.describe("C2") + ", device resident, one stream",
            "compress": {"fp32_input_gbs": n * 4 / (ms_c * 1e-3) / 1e9, "ms": ms_c, "hbm_gbs": ach, "frac_of_hbm_peak": ach / hbm_peak,
                         "two_in_flight": {"ms_per_matrix": ms_c2, "fp32_input_gbs": n * 4 / (ms_c2 * 1e-3) / 1e9,
                                           "frac_of_hbm_peak": bytes_stage / (ms_c2 * 1e-3) / 1e9 / hbm_peak},
                         "select_kernel_ms": statistics.mean(p1), "encode_kernel_ms": statistics.mean(p2),
                         "select_kernel_frac": bytes_p1 / (statistics.mean(p1) * 1e-3) / 1e9 / hbm_peak},
            "decompress": {"fp32_output_gbs": n * 4 / (ms_d * 1e-3) / 1e9, "ms": ms_d, "hbm_gbs": ach_d,
                           "frac_of_hbm_peak": ach_d / hbm_peak, "kernel": "dequantise + outlier add in one kernel"}}


def row_sharded_leg(torch, dist, pkg, L, W, rank, world):
    """The second half of configs[4]: one 65536 x 4096 matrix (seeded, configuration 3's construction) held as `world`
    row shards, rank-128 randomized SVD with 2 power iterations; NCCL all-reduces of the k x k Gram matrices and the
    n x k partial products are the only exchange.  First a smaller matrix (32768 rows, which one GPU can also take
    unsharded) for parity, then the full one for time; every rank also packs its shard as an ordinary object and
    decompresses it through the unchanged public call."""
    cfg = W.C5B
    n, k, niter = cfg["cols"], cfg["rank"], cfg["niters"]
    ids = [None]
    if rank == 0:
        buf = (C.c_char * 128)()
        ids = [bytes(buf) if L.bsq_shard_unique_id(buf, 128) == 0 else None]
    dist.broadcast_object_list(ids, src=0)
    if ids[0] is None:
        return {"error": "bsq_shard_unique_id failed on rank 0 (NCCL not found)"}
    comm = L.bsq_shard_comm_create(ids[0], rank, world)
    if not comm:
        raise RuntimeError("bsq_shard_comm_create failed")
    bad = []                                               # failures of library calls on this rank: reported, never raised --
                                                           # a rank that left early would strand the others in a collective

    def check(ok, what):
        if not ok:
            bad.append(what)
        return ok
    out = {"workload": "65536x4096 FP32 (G1 diag(1/i) G2^T + 0.01 N(0,1)), rank 128, 2 power iterations, %d row shards" % world,
           "gram_allreduce": "one kernel per rank over peer memory (CUDA IPC, plain loads over NVLink, fixed rank order)"
                             if L.bsq_shard_uses_peer_exchange(comm) else "NCCL",
           "partial_product_allreduce": "NCCL"}

    def sq_sums(a, u, s, v):
        r = a.double() - (u.double() * s.double()) @ v.double().T
        t = torch.stack([(r * r).sum(), (a.double() ** 2).sum()])
        dist.all_reduce(t)
        return float((t[0] / t[1]).sqrt())

    def run(m_total, timed_calls):
        m_local = m_total // world
        a = W.lowrank_matrix(torch, m_total, n, cfg["seed"], row_slice=(rank * m_local, m_local))
        u = torch.zeros((m_local, k), device="cuda")
        s = torch.zeros(k, device="cuda")
        v = torch.zeros((n, k), device="cuda")
        h = L.bsq_shard_svd_create(comm, m_local, m_total, n, k, niter)
        if not check(bool(h), "bsq_shard_svd_create"):
            return {"rel_frob": None}, np.zeros(k, np.float32)
        stream = torch.cuda.current_stream().cuda_stream
        res = {}
        for _ in range(2):
            check(L.bsq_shard_svd_run(h, a.data_ptr(), 1241, u.data_ptr(), s.data_ptr(), v.data_ptr(), stream) == 0, "bsq_shard_svd_run")
        res["rel_frob"] = sq_sums(a, u, s, v)
        if timed_calls:
            L.bsq_shard_svd_profile(h, 1)
            dist.barrier()
            torch.cuda.synchronize()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            for _ in range(timed_calls):
                check(L.bsq_shard_svd_run(h, a.data_ptr(), 1241, u.data_ptr(), s.data_ptr(), v.data_ptr(), stream) == 0, "bsq_shard_svd_run")
            e1.record()
            torch.cuda.synchronize()
            ms, kinds = (C.c_float * 32)(), (C.c_int * 32)()
            cnt = L.bsq_shard_svd_profile_read(h, ms, kinds, 32)
            t = torch.tensor([e0.elapsed_time(e1) / timed_calls, sum(ms[i] for i in range(cnt) if kinds[i] == 1),
                              sum(ms[i] for i in range(cnt) if kinds[i] == 0)], dtype=torch.float64, device="cuda")
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            res["ms_per_call"], res["allreduce_ms_per_call"], res["big_products_ms_per_call"] = [float(x) for x in t]
            res["allreduces_per_call"] = sum(1 for i in range(cnt) if kinds[i] == 1)
            res["fp32_input_gbs"] = m_total * n * 4 / (res["ms_per_call"] * 1e-3) / 1e9
            # the shard as an ordinary object, through the unchanged decompress
            obj = C.c_void_p(None)
            y = torch.zeros((m_local, n), device="cuda")
            if check(L.bsq_shard_compress(h, a.data_ptr(), 1241, C.byref(obj), stream) == 0, "bsq_shard_compress"):
                check(L.bsq_decompress_initialize(m_local, n, 0.0, 0.0, k, -1, -1, -1) == 0, "bsq_decompress_initialize")
                check(L.bsq_decompress(obj, y.data_ptr(), m_local * n) == 0, "bsq_decompress of the shard object")
            torch.cuda.synchronize()
            r = (a.double() - y.double())
            t2 = torch.stack([(r * r).sum(), (a.double() ** 2).sum()])
            dist.all_reduce(t2)
            res["rel_frob_from_shard_objects"] = float((t2[0] / t2[1]).sqrt())
            res["shard_object_bytes"] = int(L.bsq_get_packed_size(obj)) if obj.value else 0
            if obj.value:
                L.bsq_free(obj)
            L.bsq_decompress_release()
        L.bsq_shard_svd_destroy(h)
        sv = s.cpu().numpy().copy()
        del a, u, s, v
        return res, sv

    small, s_sharded = run(32768, 0)
    out["parity_32768x4096"] = {"rel_frob_sharded": small["rel_frob"]}
    if rank == 0:
        a = W.lowrank_matrix(torch, 32768, n, cfg["seed"], row_slice=(0, 32768))
        u = torch.zeros((32768, k), device="cuda")
        s = torch.zeros(k, device="cuda")
        v = torch.zeros((n, k), device="cuda")
        check(L.bsq_svd_lowrank(a.data_ptr(), 32768, n, k, niter, 1241, u.data_ptr(), s.data_ptr(), v.data_ptr(), None) == 0, "unsharded bsq_svd_lowrank")
        torch.cuda.synchronize()
        e1 = rel_frob(a, (u * s) @ v.T)
        s1 = s.cpu().numpy()
        out["parity_32768x4096"].update({"rel_frob_unsharded": e1, "abs_diff": abs(e1 - small["rel_frob"]),
                                         "s_lead4_max_rel_diff": float(np.max(np.abs(s_sharded[:4] - s1[:4]) / s1[:4]))})
        del a, u, s, v
    dist.barrier()
    full, _ = run(cfg["rows"], 5)
    out.update(full)
    L.bsq_shard_comm_destroy(comm)
    failures = [None] * world
    dist.all_gather_object(failures, bad)
    if any(failures):
        out["error"] = {"rank %d" % r: f for r, f in enumerate(failures) if f}
    return out


def tf32_peak(torch):
    """Dense TF32 rate of a library matrix product, the denominator of the 3xTF32 roofline: FP32 matmul 8192^3 with TF32
    allowed, best of 10 (a measurement of the device, not part of the path)."""
    old = torch.backends.cuda.matmul.allow_tf32
    torch.backends.cuda.matmul.allow_tf32 = True
    try:
        a = torch.randn(8192, 8192, device="cuda")
        b = torch.randn(8192, 8192, device="cuda")
        for _ in range(3):
            torch.matmul(a, b)
        best = 1e9
        for _ in range(10):
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            torch.matmul(a, b)
            e1.record()
            torch.cuda.synchronize()
            best = min(best, e0.elapsed_time(e1))
        return 2 * 8192 ** 3 / (best * 1e-3) / 1e12
    finally:
        torch.backends.cuda.matmul.allow_tf32 = old


def fp16_peak(torch):
    """Dense FP16 rate of a library matrix product (FP32 accumulation), the denominator of the roofline when the products
    run as three kind::f16 MMAs on operands split into FP16 halves: half matmul 8192^3, best of 10."""
    a = torch.randn(8192, 8192, device="cuda").half()
    b = torch.randn(8192, 8192, device="cuda").half()
    for _ in range(3):
        torch.matmul(a, b)
    best = 1e9
    for _ in range(10):
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        torch.matmul(a, b)
        e1.record()
        torch.cuda.synchronize()
        best = min(best, e0.elapsed_time(e1))
    return 2 * 8192 ** 3 / (best * 1e-3) / 1e12


# ----------------------------------------------------------------------------------------------------------------
# the bench line
# ----------------------------------------------------------------------------------------------------------------
def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=4)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--lanes", type=int, default=8, help="matrices in flight per GPU")
    ap.add_argument("--layers", type=int, default=None, help="batch size (default: the configuration's 32)")
    ap.add_argument("--single", default=None, choices=["C3", "C4", "C5A", "c3", "c4", "c5a"],
                    help="side measurement, not the bench line: public compress / decompress of one matrix")
    ap.add_argument("--skip-extras", action="store_true", help="leave out the configs[1] leg, the row-sharded leg and the CPU baseline")
    ap.add_argument("--sharded-only", action="store_true", help="run only the row-sharded SVD leg (needs torchrun, N >= 2)")
    ap.add_argument("--stage-only", action="store_true",
                    help="run only the configs[1] leg (fused front end and fused decompress kernel, device resident): for "
                         "profiler captures; prints that leg's figures, no bench line")
    args = ap.parse_args()
    if args.single:
        run_single(args)
        return
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    if args.impl == "reference":
        run_reference(args, rank)
        return
    args.warmup = max(args.warmup, 3)

    import torch
    import torch.distributed as dist

    all_cpus = os.sched_getaffinity(0) if hasattr(os, "sched_getaffinity") else None
    numa = bind_near_gpu(local_rank)
    pkg = entry.load_package()
    L = pkg.lib()
    W = workloads()
    shard = load_shard()
    torch.cuda.set_device(local_rank)
    if world > 1:
        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    if args.stage_only:
        if rank == 0:
            print(json.dumps({"stage_only": True, "configs1_frontend": c2_frontend_leg(torch, pkg, L, W, measured_peaks()[0])}))
        return
    if args.sharded_only:
        res = row_sharded_leg(torch, dist, pkg, L, W, rank, world)
        if rank == 0:
            print(json.dumps({"row_sharded_svd": res}))
        dist.barrier()
        dist.destroy_process_group()
        return

    cfg = W.CONFIGS["C5A"]
    rows, cols = cfg["rows"], cfg["cols"]
    n = rows * cols
    n_layers = args.layers or W.C5A_LAYERS
    layers = shard.layers_for_rank(n_layers, rank, world)
    cnt = len(layers)
    mats = [W.config_matrix(torch, "C5A", layer=l) for l in layers]
    lanes = max(1, args.lanes)
    # a rank with fewer matrices than lanes (8 ranks: 4 each) queues `mult` passes over its matrices at a time, every
    # entry with an output buffer of its own, so that the lanes stay full; a pass is still every matrix once
    mult = max(1, lanes // cnt) if cnt else 1
    lanes = min(lanes, max(cnt * mult, 1))
    entries = cnt * mult
    cfg_args = (rows, cols, cfg["outlier"], cfg["error"], cfg["rank"], cfg["niters"], cfg["uv"], cfg["s"], cfg["q"])
    batch = L.bsq_batch_create(*cfg_args, lanes)
    single = L.bsq_batch_create(*cfg_args, 1)
    if not batch or not single:
        raise RuntimeError("bsq_batch_create failed")
    cap = int(L.bsq_lane_packed_capacity(L.bsq_batch_lane(batch, 0)))
    VP = C.c_void_p * max(cnt, 1)
    VPE = C.c_void_p * max(entries, 1)
    d_packed = [torch.empty(cap, dtype=torch.uint8, device="cuda") for _ in range(entries)]
    d_dst = [torch.empty((rows, cols), dtype=torch.float32, device="cuda") for _ in range(lanes)]
    in_ptrs = VPE(*[mats[i % cnt].data_ptr() for i in range(entries)])
    packed_ptrs = VPE(*[p.data_ptr() for p in d_packed])
    dst_ptrs = VPE(*[d_dst[i % lanes].data_ptr() for i in range(entries)])
    hdrs = (pkg.Array * max(entries, 1))()
    hdr_ptrs = VPE(*[C.addressof(hdrs[i]) for i in range(entries)])
    sizes = (C.c_uint64 * max(entries, 1))()
    main_stream = torch.cuda.current_stream()

    def compress_pass(b):
        """`mult` passes over this rank's matrices."""
        if cnt and L.bsq_batch_compress(b, in_ptrs, entries, pkg.INPUT_DEVICE, packed_ptrs, cap, None, hdrs, sizes) != 0:
            raise RuntimeError("bsq_batch_compress failed")

    def decompress_pass(b):
        if cnt and L.bsq_batch_decompress(b, hdr_ptrs, entries, 1, dst_ptrs, n) != 0:
            raise RuntimeError("bsq_batch_decompress failed")

    def timed_steps(b, steps, passes):
        """`steps` steps of `passes` passes each (`passes` a multiple of `mult`); returns (total ms, compress ms, decompress ms)
        from CUDA events."""
        evs = []
        barrier()
        for _ in range(steps * passes // mult):
            e = [torch.cuda.Event(enable_timing=True) for _ in range(3)]
            e[0].record(main_stream)
            compress_pass(b)
            e[1].record(main_stream)
            decompress_pass(b)
            e[2].record(main_stream)
            evs.append(e)
        barrier()
        total = evs[0][0].elapsed_time(evs[-1][2])
        return total, sum(e[0].elapsed_time(e[1]) for e in evs), sum(e[1].elapsed_time(e[2]) for e in evs)

    # ---- warm-up, and how many passes a step needs for a timed region of at least 0.6 s ----
    for _ in range(args.warmup):
        compress_pass(batch)
        decompress_pass(batch)
    t_est, _, _ = timed_steps(batch, 1, mult)
    t_est = shard.max_over_ranks([t_est], device="cuda")[0] / mult
    mult_all = int(shard.max_over_ranks([float(mult)], device="cuda")[0])       # the same pass count on every rank
    passes = max(1, int(math.ceil(600.0 / max(t_est * args.steps, 1e-3))))
    passes = (passes + mult_all - 1) // mult_all * mult_all
    err0 = rel_frob(mats[-1], d_dst[(entries - 1) % lanes]) if cnt else None
    packed_total = int(sum(sizes[i] for i in range(cnt)))

    sampler = ClockSampler(local_rank)
    if rank == 0:
        sampler.start()
    ms_total, ms_c, ms_d = timed_steps(batch, args.steps, passes)

    # ---- one matrix at a time, with the big products timed on the lane's stream (roofline) ----
    lane0 = L.bsq_batch_lane(single, 0)
    L.bsq_lane_profile(lane0, 1)
    prod_ms = []
    one_c = one_d = 0.0
    reps1 = max(1, min(cnt, 4))
    ms_buf, kind_buf = (C.c_float * 32)(), (C.c_int * 32)()
    for w in range(2):
        for i in range(reps1):
            e = [torch.cuda.Event(enable_timing=True) for _ in range(3)]
            torch.cuda.synchronize()
            e[0].record(main_stream)
            if L.bsq_lane_compress_begin(lane0, mats[i].data_ptr(), pkg.INPUT_DEVICE, d_packed[i].data_ptr(), cap) != 0 or \
                    L.bsq_lane_compress_end(lane0, None, C.byref(hdrs[i]), None) != 0:
                raise RuntimeError("lane compress failed")
            e[1].record(main_stream)
            if L.bsq_lane_decompress_begin(lane0, C.byref(hdrs[i]), 1, d_dst[0].data_ptr(), n) != 0 or L.bsq_lane_decompress_end(lane0) != 0:
                raise RuntimeError("lane decompress failed")
            e[2].record(main_stream)
            torch.cuda.synchronize()
            if w == 1:
                one_c += e[0].elapsed_time(e[1]) / reps1
                one_d += e[1].elapsed_time(e[2]) / reps1
                k_ = L.bsq_lane_profile_read(lane0, ms_buf, kind_buf, 32)
                prod_ms += [ms_buf[j] for j in range(k_) if kind_buf[j] == 0]
    L.bsq_lane_profile(lane0, 0)

    # ---- end to end: pinned host matrices in, host objects out, decompress from the host objects ----
    pinned = [torch.empty((rows, cols), dtype=torch.float32).pin_memory() for _ in range(cnt)]
    for p, m in zip(pinned, mats):
        p.copy_(m)
    torch.cuda.synchronize()
    host_ptrs = VP(*[p.data_ptr() for p in pinned])
    outs = VP()
    probe = torch.empty(1, dtype=torch.float32).pin_memory()

    def e2e_pass():
        if cnt == 0:
            return 0
        if L.bsq_batch_compress(batch, host_ptrs, cnt, pkg.INPUT_HOST, None, 0, outs, None, sizes) != 0:
            raise RuntimeError("bsq_batch_compress (host) failed")
        if L.bsq_batch_decompress(batch, outs, cnt, 0, VP(*[d_dst[i % lanes].data_ptr() for i in range(cnt)]), n) != 0:
            raise RuntimeError("bsq_batch_decompress (host objects) failed")
        probe.copy_(d_dst[(cnt - 1) % lanes].view(-1)[:1])            # the step's result is read back
        got = sum(int(sizes[i]) for i in range(cnt))
        for i in range(cnt):
            L.bsq_free(outs[i])
            outs[i] = None
        return got
    for _ in range(2):
        e2e_pass()
    barrier()
    t0 = time.perf_counter()
    for _ in range(args.steps * passes):
        d2h = e2e_pass()
    torch.cuda.synchronize()
    e2e_ms = (time.perf_counter() - t0) * 1e3
    barrier()

    # ---- the same through the reference's own two calls, one matrix at a time (the drop-in path: host matrix in, host
    # object out, decompress from it; every call synchronous) ----
    if L.bsq_compress_initialize(*cfg_args, pkg.INPUT_HOST) != 0 or \
            L.bsq_decompress_initialize(rows, cols, cfg["outlier"], cfg["error"], cfg["rank"], cfg["uv"], cfg["s"], cfg["q"]) != 0:
        raise RuntimeError("public initialisers failed")

    def dropin_pass():
        for i in range(cnt):
            o = C.c_void_p(None)
            if L.bsq_compress(pinned[i].data_ptr(), C.byref(o), None) != 0:
                raise RuntimeError("bitsqz_llm_compress failed")
            if L.bsq_decompress(o, d_dst[0].data_ptr(), n) != 0:
                raise RuntimeError("bitsqz_llm_decompress failed")
            L.bsq_free(o)
    dropin_pass()
    barrier()
    dropin_passes = max(1, min(passes * args.steps, 3))
    t0 = time.perf_counter()
    for _ in range(dropin_passes):
        dropin_pass()
    torch.cuda.synchronize()
    dropin_ms = (time.perf_counter() - t0) * 1e3 / dropin_passes
    barrier()
    L.bsq_compress_release()
    L.bsq_decompress_release()
    clocks = sampler.stop() if rank == 0 else None

    ms_total, ms_c, ms_d, e2e_ms, one_c, one_d, dropin_ms = shard.max_over_ranks([ms_total, ms_c, ms_d, e2e_ms, one_c, one_d, dropin_ms],
                                                                                 device="cuda")
    packed_all = int(sum(shard.gather_objects(packed_total)))
    L.bsq_batch_destroy(batch)
    L.bsq_batch_destroy(single)
    del pinned, d_packed, mats, d_dst
    torch.cuda.empty_cache()
    sharded = None
    if world > 1 and not args.skip_extras:
        # a failure here must not cost the line: what the leg cannot do is reported inside its own object
        try:
            sharded = row_sharded_leg(torch, dist, pkg, L, W, rank, world)
        except Exception as exc:                             # noqa: BLE001 (reported, not hidden)
            sharded = {"error": "%s: %s" % (type(exc).__name__, exc)}

    if rank == 0:
        hbm_peak, bf16_peak, peak_kind = measured_peaks()
        tf32 = tf32_peak(torch)
        batch_bytes = n_layers * n * 4
        per_step = batch_bytes * passes
        nsteps = args.steps
        value = per_step * nsteps / (ms_total * 1e-3) / 1e9
        flops = 2.0 * rows * cols * cfg["rank"]
        prod_mean = statistics.mean(prod_ms) if prod_ms else None
        # products alternate: W X (W read along M: A as stored is K x M) and W^T X (A read along K)
        ach = flops / (prod_mean * 1e-3) / 1e12 if prod_mean else None
        # three MMAs per product either way: on FP16 halves (default) or on TF32 halves (BSQ_GEMM_F16=0)
        split16 = os.environ.get("BSQ_GEMM_F16", "1") != "0"
        fp16 = fp16_peak(torch) if split16 else None
        peak3 = (fp16 if split16 else tf32) / 3.0
        line = {
            "metric": METRIC, "value": value, "unit": "GB/s", "n_gpus": world, "steps": nsteps, "warmup": args.warmup,
            "ms_per_step": ms_total / nsteps, "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
            "dtype": "f32 (products on tcgen05 from operands split into two FP16 halves with power-of-two scales, FP32-level accuracy)", "data": "synthetic",
            "config": {"workload": WORKLOAD, "rows": rows, "cols": cols, "layers": n_layers, "passes_per_step": passes,
                       "lanes_per_gpu": lanes, "passes_queued_together": mult,
                       "parallelism": "matrix i on rank i %% %d, no collective on the data path; %d matrices in flight per GPU" % (world, lanes),
                       "l2": "every input matrix is 235 MB (> 126 MB L2)", "host_memory": "rank 0: " + numa,
                       "timed_region_s": ms_total * 1e-3},
            "compress": {"value": per_step * nsteps / (ms_c * 1e-3) / 1e9, "unit": "GB/s", "ms_per_matrix": ms_c / (nsteps * passes * max(cnt, 1)),
                         "one_at_a_time_ms_per_matrix": one_c},
            "decompress": {"value": per_step * nsteps / (ms_d * 1e-3) / 1e9, "unit": "GB/s (FP32 output)",
                           "ms_per_matrix": ms_d / (nsteps * passes * max(cnt, 1)), "one_at_a_time_ms_per_matrix": one_d,
                           "call": "bsq_batch_decompress on device-resident objects"},
            "rel_frob_last_layer": err0,
            "packed_bytes_per_step": packed_all * passes, "compression_ratio": batch_bytes / max(packed_all, 1),
            "e2e": {"value": per_step * nsteps / (e2e_ms * 1e-3) / 1e9, "unit": "GB/s", "h2d_bytes_per_step": per_step + packed_all * passes,
                    "d2h_bytes_per_step": packed_all * passes + 4 * passes * world, "ms_per_step": e2e_ms / nsteps,
                    "api": "bsq_batch_compress (pinned host matrices -> host objects) + bsq_batch_decompress (host objects -> device "
                           "matrix), the lanes form of bitsqz_llm_compress / bitsqz_llm_decompress; h2d = inputs + objects on their way "
                           "back for decompress",
                    "drop_in_calls": {"value": batch_bytes / (dropin_ms * 1e-3) / 1e9, "unit": "GB/s", "ms_per_pass": dropin_ms,
                                      "api": "bitsqz_llm_compress (BITSQZ_LLM_INPUT_HOST, pinned matrix) + bitsqz_llm_decompress on the "
                                             "returned host object, one matrix at a time, every call synchronous: the calls the "
                                             "reference arm makes"}},
            "gpu_launches": (LAUNCHES_PER_COMPRESS + LAUNCHES_PER_DECOMPRESS) * n_layers * passes * nsteps,
            "roofline": {"bound": "tensor", "kernel": "gemm_tc_tma_kernel<*,256> (TMA-fed tcgen05, operands split into two %s halves: three MMAs per "
                                                       "product, 4096x14336 matrix times a 256-column panel)" % ("FP16" if split16 else "TF32"),
                         "achieved": ach, "peak": peak3, "unit": "TFLOP/s", "frac": (ach / peak3) if ach else None, "traffic": PRODUCT_DRAM_BYTES_PER_LAUNCH,
                         "traffic_unit": "bytes per launch: dram__bytes_read.sum + dram__bytes_write.sum of one ncu capture of this kernel on this "
                                         "matrix (FP16 halves), mean of the six products of a call; the matrix alone is 234.9 MB",
                         "peak_kind": ("FP16 dense matmul measured in this run (%.0f TFLOP/s) / 3; TF32 dense measured %.0f (achieved / (TF32 / 3) = %.2f); BF16 %s %.0f"
                                       % (fp16, tf32, (ach / (tf32 / 3.0)) if ach else 0.0, peak_kind, bf16_peak)) if split16 else
                                      "TF32 dense matmul measured in this run (%.0f TFLOP/s) / 3; BF16 %s %.0f" % (tf32, peak_kind, bf16_peak),
                         "flops_per_launch": flops, "ms_per_launch": prod_mean, "launches_timed": len(prod_ms),
                         "ms_w_x": statistics.mean(prod_ms[0::2]) if prod_ms else None,
                         "ms_wt_x": statistics.mean(prod_ms[1::2]) if prod_ms else None,
                         "timed": "CUDA events on the lane's stream around each product, one matrix in flight"},
            "clocks": clocks,
        }
        if clocks and clocks.get("sm_mhz"):
            # time x clock: comparable between runs whose sampled SM clocks differ (nothing sets the clocks)
            line["clocks"]["ms_per_step_x_sm_ghz"] = ms_total / nsteps * clocks["sm_mhz"] / 1000.0
        if sharded is not None:
            line["row_sharded_svd"] = sharded
        if not args.skip_extras:
            def guarded(leg, *a):                             # a side measurement that fails is reported in its own object
                try:
                    return leg(*a)
                except Exception as exc:                      # noqa: BLE001
                    return {"error": "%s: %s" % (type(exc).__name__, exc)}
            line["configs1_frontend"] = guarded(c2_frontend_leg, torch, pkg, L, W, hbm_peak)
            if world == 1:
                if all_cpus:
                    os.sched_setaffinity(0, all_cpus)         # the CPU baseline runs on every core this process may use
                line["cpu_baseline"] = guarded(cpu_nf4_baseline, W)
        print(json.dumps(line))
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
