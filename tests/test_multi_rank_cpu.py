"""World-size-2 test of the multi-GPU plumbing on CPU (gloo): the round-robin partition over independent
matrices, the max-over-ranks reduction the bench uses, and that sharding changes no bytes -- each rank
compresses its share with the CPU oracle and the gathered digests equal the single-process ones."""
import hashlib
import os
import subprocess
import sys

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))

WORKER = r'''
import hashlib, json, os, sys
import numpy as np
import torch.distributed as dist
sys.path.insert(0, os.environ["BSQ_ROOT"])
import __graft_entry__ as entry
pkg = entry.load_package()
import importlib.util
spec = importlib.util.spec_from_file_location("bsq_shard", os.path.join(os.environ["BSQ_ROOT"], "bitsqueeze-llm_b200", "shard.py"))
shard = importlib.util.module_from_spec(spec); spec.loader.exec_module(shard)
dist.init_process_group("gloo", init_method="tcp://127.0.0.1:" + os.environ["BSQ_PORT"],
                        rank=int(os.environ["RANK"]), world_size=int(os.environ["WORLD_SIZE"]))
rank, world = dist.get_rank(), dist.get_world_size()
oracle = entry.load_oracle().Oracle()
mine = shard.layers_for_rank(7, rank, world)
digests = {}
for layer in mine:
    x = np.random.default_rng(100 + layer).standard_normal((32, 128)).astype(np.float32)
    digests[layer] = hashlib.sha256(oracle.compress_nosvd(x, 0.05, 0.0, 10).tobytes()).hexdigest()
everyone = shard.gather_objects(digests)
slowest = shard.max_over_ranks([float(rank + 1), 10.0 - rank])
dist.barrier()
if rank == 0:
    print(json.dumps({"digests": everyone, "max": slowest, "mine": mine}))
dist.destroy_process_group()
'''


def test_two_ranks_gloo(built, oracle, tmp_path):
    script = tmp_path / "worker.py"
    script.write_text(WORKER)
    port = str(29500 + os.getpid() % 2000)
    procs = []
    for rank in range(2):
        env = dict(os.environ, RANK=str(rank), WORLD_SIZE="2", BSQ_ROOT=ROOT, BSQ_PORT=port, MASTER_ADDR="127.0.0.1")
        procs.append(subprocess.Popen([sys.executable, str(script)], env=env, stdout=subprocess.PIPE, stderr=subprocess.PIPE, text=True))
    outs = [p.communicate(timeout=240) for p in procs]
    assert all(p.returncode == 0 for p in procs), outs
    import json
    res = json.loads(outs[0][0].strip().splitlines()[-1])
    assert res["mine"] == [0, 2, 4, 6]
    assert res["max"] == [2.0, 10.0]                                   # element-wise max over the two ranks
    merged = {}
    for d in res["digests"]:
        for k, v in d.items():
            assert k not in merged                                      # no matrix handled twice
            merged[int(k)] = v
    assert sorted(merged) == list(range(7))                            # every matrix handled
    for layer in range(7):                                              # and bytes identical to an unsharded run
        x = np.random.default_rng(100 + layer).standard_normal((32, 128)).astype(np.float32)
        assert merged[layer] == hashlib.sha256(oracle.compress_nosvd(x, 0.05, 0.0, 10).tobytes()).hexdigest()
