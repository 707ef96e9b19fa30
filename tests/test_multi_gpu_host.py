"""The N>1 path of bench.py on CPU: two gloo ranks shard the sequences (no data-path collective), agree on the step time
as the maximum over ranks, and rank 0 alone reports. Also the reference arm's rank rule."""
import json
import os
import subprocess
import sys
from pathlib import Path

import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = Path(__file__).resolve().parent.parent


def _worker(rank, world, port, q):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    sys.path.insert(0, str(ROOT))
    from pragnosia_b200 import synth
    import bench
    # every rank draws its own sequences (seed 1 + rank), as the product arm does
    ids = synth.token_ids(bench.B_PER_GPU, 64, bench.CFG["vocab"], seed=1 + rank)
    t = torch.tensor([10.0 + rank, 20.0 - rank], dtype=torch.float64)          # per-rank step / e2e times
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    gathered = [torch.zeros_like(ids) for _ in range(world)]
    dist.all_gather(gathered, ids)                                             # the output gather a caller may do afterwards
    q.put((rank, t.tolist(), int(ids.sum()), [int(g.sum()) for g in gathered]))
    dist.barrier()
    dist.destroy_process_group()


def test_two_ranks_shard_and_take_the_max():
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = 29500 + os.getpid() % 2000
    procs = [ctx.Process(target=_worker, args=(r, 2, port, q)) for r in range(2)]
    for p in procs: p.start()
    res = sorted(q.get(timeout=120) for _ in range(2))
    for p in procs: p.join(60)
    assert all(p.exitcode == 0 for p in procs)
    (r0, t0, s0, g0), (r1, t1, s1, g1) = res
    assert t0 == t1 == [11.0, 20.0]                                             # max over ranks, identical everywhere
    assert s0 != s1 and g0 == g1 == [s0, s1]                                    # different shards, gather in rank order


def test_reference_arm_only_rank_zero_reports():
    env = dict(os.environ, RANK="1", WORLD_SIZE="2")
    r = subprocess.run([sys.executable, str(ROOT / "bench.py"), "--impl", "reference", "--gpus", "2", "--steps", "1", "--warmup", "0"],
                       capture_output=True, text=True, env=env, timeout=120)
    assert r.returncode == 0 and r.stdout.strip() == ""


def test_bench_token_accounting():
    sys.path.insert(0, str(ROOT))
    import bench
    assert bench.B_PER_GPU * bench.T_TOTAL == 32768 and bench.T_TOTAL // bench.WINDOW == 4
    assert bench.CFG == dict(vocab=8192, d=768, layers=12, mlp_mult=4, ctx=512, mixer="aspin", norm="rms")


def _gather_worker(rank, world, port, q):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    sys.path.insert(0, str(ROOT))
    from pragnosia_b200 import sharded
    b0, b1 = sharded.shard_range(6, rank, world)
    # three "windows": each rank's local output carries its global sequence numbers and the window index
    fn = lambda w: (torch.arange(b0, b1, dtype=torch.float32)[:, None] * 10 + w).expand(b1 - b0, 4).contiguous()
    full = sharded.run_windows(fn, 3, sharded.WindowGather(enabled=True))
    local = sharded.run_windows(fn, 3, sharded.WindowGather(enabled=False))
    g = sharded.WindowGather(enabled=True)
    g.submit(fn(0))
    q.put((rank, (b0, b1), [f[:, 0].tolist() for f in full], [tuple(t.shape) for t in local], g.bytes_received))
    g.finish()
    dist.barrier()
    dist.destroy_process_group()


def test_window_outputs_are_gathered_in_rank_and_window_order():
    """pragnosia_b200.sharded on two gloo ranks: contiguous batch shards, per-window all-gather along the batch axis in
    submission order, and the compute-only arm (gather disabled) returning the local tensors."""
    sys.path.insert(0, str(ROOT))
    from pragnosia_b200 import sharded
    assert [sharded.shard_range(7, r, 3) for r in range(3)] == [(0, 3), (3, 5), (5, 7)]
    assert sharded.shard_range(64, 5, 8) == (40, 48) and sharded.shard_range(2, 3, 4) == (2, 2)
    assert [(s.start, s.stop) for s in sharded.windows_of(10, 4)] == [(0, 4), (4, 8), (8, 10)]
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = 31500 + os.getpid() % 2000
    procs = [ctx.Process(target=_gather_worker, args=(r, 2, port, q)) for r in range(2)]
    for p in procs: p.start()
    res = sorted(q.get(timeout=120) for _ in range(2))
    for p in procs: p.join(60)
    assert all(p.exitcode == 0 for p in procs)
    for rank, (b0, b1), full, local_shapes, nbytes in res:
        assert (b0, b1) == ((0, 3), (3, 6))[rank]
        assert full == [[float(10 * s + w) for s in range(6)] for w in range(3)]     # every rank holds the whole batch, per window
        assert local_shapes == [(3, 4)] * 3
        assert nbytes == 3 * 4 * 4                                                  # one peer's window of 3 x 4 floats
