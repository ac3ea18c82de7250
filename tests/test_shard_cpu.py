"""Multi-rank host logic on CPU: world_size-2 and -3 gloo process groups shard a batch, each rank
produces (fake) token streams for its shard, rank 0 gathers them in global order."""
import os

import numpy as np
import pytest
import torch.multiprocessing as mp

from small_llm_b200.shard import balanced_assignment, shard_range


def test_shard_range_covers_everything_once():
    for n in (0, 1, 7, 512, 513):
        for world in (1, 2, 3, 8):
            spans = [shard_range(n, world, r) for r in range(world)]
            assert spans[0][0] == 0 and spans[-1][1] == n
            assert all(spans[i][1] == spans[i + 1][0] for i in range(world - 1))
            sizes = [e - b for b, e in spans]
            assert max(sizes) - min(sizes) <= 1
    with pytest.raises(ValueError):
        shard_range(4, 2, 2)


def test_balanced_assignment_evens_out_total_length():
    rng = np.random.default_rng(4)
    lens = rng.integers(256, 1537, size=512)
    for world in (1, 2, 4, 8):
        parts = balanced_assignment(lens, world)
        assert sorted(np.concatenate(parts).tolist()) == list(range(512))
        assert {len(p) for p in parts} == {512 // world}
        sums = [int(lens[p].sum()) for p in parts]
        assert max(sums) - min(sums) <= 1536                       # within one sequence of each other
    assert [p.tolist() for p in balanced_assignment([5, 9, 1], 2)] == [[1], [0, 2]]


def _stream(i):                       # deterministic fake "generation" of sequence i
    return (np.arange(3 + i % 5, dtype=np.uint32) * 7 + i) % 32768


def _worker(rank, world, port, n_seq, q, balanced=False):
    import torch.distributed as dist
    from small_llm_b200.shard import balanced_assignment, gather_streams, shard_range
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    if balanced:
        parts = balanced_assignment([len(_stream(i)) for i in range(n_seq)], world)
        got = gather_streams([_stream(int(i)) for i in parts[rank]], n_seq, 16, assignment=parts)
    else:
        b, e = shard_range(n_seq, world, rank)
        got = gather_streams([_stream(i) for i in range(b, e)], n_seq, 16)
    if rank == 0:
        q.put([g.tolist() for g in got])
    else:
        assert got is None
    dist.barrier()
    dist.destroy_process_group()


@pytest.mark.parametrize("world,n_seq,balanced", [(2, 5, False), (3, 7, False), (2, 2, False), (2, 7, True)])
def test_gather_streams_gloo(world, n_seq, balanced):
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = 29600 + world * 10 + n_seq + (100 if balanced else 0)
    procs = [ctx.Process(target=_worker, args=(r, world, port, n_seq, q, balanced)) for r in range(world)]
    for p in procs:
        p.start()
    got = q.get(timeout=120)
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    assert got == [_stream(i).tolist() for i in range(n_seq)]
