"""The N > 1 path on CPU: two gloo ranks each take their shard of a configuration, evaluate it
(with the CPU oracle standing in for the device), all-gather the outputs along the documented axis
and must reproduce the unsharded result bit for bit. This covers workloads.shard (which slice of
the seeded input streams a rank draws) and the gather step bench.py performs over NCCL."""
import os
import sys
from pathlib import Path

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = Path(__file__).resolve().parent.parent
sys.path.insert(0, str(ROOT / "oracle"))

CASES = {
    "c2": dict(n=4, h=6, w=6, c_in=64, c_mid=64),
    "c3": dict(m=64, k=64, n=64),
    "c4": dict(b=2, h=2, s=16, d=8),
    "c5": dict(batch=4, hq=4, hkv=2, d=16, pages=32, block=8, max_len=64, min_len=8),
}


def _evaluate(workload):
    import graph_oracle
    ins, storage = {}, {}
    for uid, make in workload.inputs.items():
        raw = make()
        data_type = workload.tensor(uid)["data_type"]
        ins[uid] = graph_oracle.widen(raw, data_type)
        storage[uid] = raw
    return graph_oracle.run(workload.document, ins, storage_inputs={u: storage[u] for u in storage if workload.tensor(u)["data_type"] in ("BFLOAT16", "HALF") and workload.config == 3})


def _worker(rank, world, port, name, results):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from deepforge_b200 import workloads
        local = workloads.shard(name, rank, world, **CASES[name])
        values = _evaluate(local)
        gathered = {}
        for uid in workloads.GATHER_AXIS[name]:
            mine = torch.from_numpy(np.ascontiguousarray(values[uid]).view(np.uint8).copy())
            parts = [torch.empty_like(mine) for _ in range(world)]
            dist.all_gather(parts, mine)
            gathered[uid] = torch.cat(parts).numpy()
        if rank == 0:
            full = _evaluate(workloads.BUILDERS[name](**CASES[name]))
            for uid, data in gathered.items():
                expected = np.ascontiguousarray(full[uid]).view(np.uint8)
                assert np.array_equal(data, expected), f"{name}: gathered tensor {uid} differs from the unsharded result"
            results.put((name, "ok"))
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("name", sorted(CASES))
def test_two_rank_shards_gather_to_the_unsharded_result(name):
    context = mp.get_context("spawn")
    results = context.Queue()
    port = 29500 + (os.getpid() + hash(name)) % 2000
    processes = [context.Process(target=_worker, args=(rank, 2, port, name, results)) for rank in range(2)]
    for process in processes:
        process.start()
    for process in processes:
        process.join(timeout=120)
        assert process.exitcode == 0, f"rank exited with {process.exitcode}"
    assert results.get(timeout=5) == (name, "ok")


def test_ranks_take_disjoint_cores_near_their_gpus(monkeypatch):
    """bench.py's host-side placement for multi-GPU runs: ranks whose GPUs hang off the same NUMA node split that
    node's cores between them, ranks on different nodes each stay on their own, and without NVML's answer every rank
    takes an equal share of the allowed cores. (os.sched_setaffinity is intercepted: the test process keeps its cores.)"""
    sys.path.insert(0, str(Path(__file__).resolve().parent.parent))
    import bench
    chosen = {}
    monkeypatch.setattr(os, "sched_getaffinity", lambda pid: set(range(64)))
    monkeypatch.setattr(os, "sched_setaffinity", lambda pid, cores: chosen.__setitem__("cores", sorted(cores)))
    # GPUs 0-3 on node 0 (cores 0-31), GPUs 4-7 on node 1 (cores 32-63)
    monkeypatch.setattr(bench, "cores_near_gpu", lambda index: list(range(0, 32)) if index < 4 else list(range(32, 64)))
    seen = []
    for rank in range(8):
        text = bench.spread_over_cores(rank, 8)
        assert "NUMA node" in text
        seen.append(chosen["cores"])
    assert seen[0] == list(range(0, 8)) and seen[3] == list(range(24, 32)) and seen[4] == list(range(32, 40)) and seen[7] == list(range(56, 64))
    assert sorted(core for cores in seen for core in cores) == list(range(64))
    monkeypatch.setattr(bench, "cores_near_gpu", lambda index: [])
    assert "GPU locality unknown" in bench.spread_over_cores(5, 8) and chosen["cores"] == list(range(40, 48))
    assert bench.spread_over_cores(0, 1) == "unchanged"
