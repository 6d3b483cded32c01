"""Head-parallel host logic on CPU: two gloo ranks each compute their heads (the CPU oracle stands in
for the kernels), all-gather, and must reproduce the single-rank result."""
import os
import sys
from pathlib import Path

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = Path(__file__).resolve().parent.parent


def _worker(rank, world, port, tmp):
    sys.path.insert(0, str(ROOT))
    sys.path.insert(0, str(ROOT / "tests"))
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), OMP_NUM_THREADS="1")
    dist.init_process_group("gloo", rank=rank, world_size=world)
    import oracle
    from mycaffe_b200 import head_shard
    rng = np.random.default_rng(0)            # same global problem on every rank
    B, H, T, D = 2, 4, 24, 8
    q, k, v = (rng.standard_normal((B, H, T, D)).astype(np.float32) for _ in range(3))
    lo, hi = head_shard.head_range(rank, world, H)
    assert (lo, hi) == (rank * H // world, (rank + 1) * H // world)
    ql, kl, vl = (head_shard.shard_heads(torch.from_numpy(a), rank, world).numpy() for a in (q, k, v))
    y_local = torch.from_numpy(oracle.sdpa_forward(ql, kl, vl, None, 3))
    y = head_shard.gather_heads(y_local)
    ref = oracle.sdpa_forward(q, k, v, None, 3)
    np.testing.assert_array_equal(y.numpy(), ref)
    ys = head_shard.gather_heads(y_local, strided=True)     # (B, N, H/N, T, D) view, no copy
    np.testing.assert_array_equal(ys.reshape(B, H, T, D).numpy(), ref)
    # decode: (B, dim/N) slices -> (B, dim); GQA split by kv head
    assert head_shard.head_range(rank, world, 8, n_kv_heads=2) == (rank * 4, rank * 4 + 4)
    full = np.arange(3 * 16, dtype=np.float32).reshape(3, 16)
    part = torch.from_numpy(full[:, rank * 8:(rank + 1) * 8].copy())
    np.testing.assert_array_equal(head_shard.gather_decode_outputs(part).numpy(), full)
    dist.barrier()
    dist.destroy_process_group()
    Path(tmp, f"ok{rank}").write_text("ok")


def test_two_rank_head_parallel_matches_single_rank(tmp_path):
    world = 2
    port = 29600 + os.getpid() % 300
    mp.spawn(_worker, args=(world, port, str(tmp_path)), nprocs=world, join=True)
    assert all((tmp_path / f"ok{r}").exists() for r in range(world))


def test_head_range_rejects_uneven_splits():
    from mycaffe_b200 import head_shard
    assert head_shard.head_range(0, 1, 12) == (0, 12)
    assert head_shard.head_range(3, 4, 12) == (9, 12)
    with pytest.raises(ValueError):
        head_shard.head_range(0, 8, 12)     # 12 heads (GPT-2 small) do not divide over 8 GPUs
    with pytest.raises(ValueError):
        head_shard.head_range(2, 2, 4)


def test_bind_near_pci_uses_the_local_cpulist(tmp_path):
    """The affinity helper: parses sysfs' cpulist, intersects with the allowed set, reports and can be undone;
    a missing entry is a skip."""
    import os

    from mycaffe_b200 import head_shard
    assert head_shard._parse_cpulist("0-3,8,10-11\n") == {0, 1, 2, 3, 8, 10, 11}
    allowed = os.sched_getaffinity(0)
    keep = sorted(allowed)[: max(1, len(allowed) // 2)]
    dev = tmp_path / "0000:1b:00.0"
    dev.mkdir()
    (dev / "local_cpulist").write_text(",".join(str(c) for c in keep) + ",4095\n")
    (dev / "numa_node").write_text("1\n")
    try:
        r = head_shard.bind_near_pci("0000:1b:00.0", str(tmp_path))
        assert r["cpus"] == len(keep) and r["numa_node"] == 1 and r["previous"] == allowed
        assert os.sched_getaffinity(0) == set(keep)
    finally:
        os.sched_setaffinity(0, allowed)
    assert "skipped" in head_shard.bind_near_pci("0000:ff:00.0", str(tmp_path))
    (dev / "local_cpulist").write_text("4095\n")
    assert "skipped" in head_shard.bind_near_pci("0000:1b:00.0", str(tmp_path))
    assert os.sched_getaffinity(0) == allowed
