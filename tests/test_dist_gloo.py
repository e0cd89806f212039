"""CPU-only: the multi-rank plumbing (shards, logits all-gather, max-over-ranks timing) on a
world of 2 gloo processes."""
import os
import socket

import torch
import torch.multiprocessing as mp


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def _worker(rank, world, port, q):
    os.environ.update(RANK=str(rank), WORLD_SIZE=str(world), MASTER_ADDR="127.0.0.1",
                      MASTER_PORT=str(port))
    from tcbnn_b200 import dist as d
    r, w = d.init(backend="gloo")
    assert (r, w) == (rank, world)
    b, e = d.shard_range(8, rank, world)
    local = torch.arange(b, e, dtype=torch.float32).reshape(-1, 1).repeat(1, 3) + 0.5
    full = d.gather_logits(local)
    og = d.OverlappedGather(local.shape[0], local.shape[1], local.dtype, "cpu", world)
    assert og(local).tolist() == full.tolist() and og.finish().tolist() == full.tolist()
    try:
        d.shard_range(7, rank, world)            # a batch that does not split evenly is refused
        raise AssertionError("uneven shard accepted")
    except ValueError:
        pass
    times = d.max_over_ranks([1.0 + rank, 5.0 - rank])
    member = torch.tensor([[1.0, -2.0 + 5 * rank, 3.0 - rank], [0.5 * rank, 0.0, -1.0]])
    voted = d.ensemble_max(member.clone())
    d.barrier()
    q.put((rank, full.tolist(), times, d.shard_seed(100, rank), voted.tolist()))
    d.finish()


def test_two_rank_gather_and_timing():
    world = 2
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    ps = [ctx.Process(target=_worker, args=(r, world, port, q)) for r in range(world)]
    for p in ps:
        p.start()
    res = sorted(q.get(timeout=120) for _ in range(world))
    for p in ps:
        p.join(timeout=60)
        assert p.exitcode == 0
    expect = [[i + 0.5] * 3 for i in range(8)]
    for rank, full, times, seed, voted in res:
        assert full == expect                    # rank-major order, every rank sees all logits
        assert times == [2.0, 5.0]               # max over ranks
        assert seed == 100 + rank
        if rank == 0:                            # ensemble mode: element-wise max lands on the root
            assert voted == [[1.0, 3.0, 3.0], [0.5, 0.0, -1.0]]


def test_single_process_needs_no_group():
    from tcbnn_b200 import dist as d
    for k in ("RANK", "WORLD_SIZE"):
        os.environ.pop(k, None)
    assert d.init() == (0, 1)
    x = torch.ones(2, 3)
    assert d.gather_logits(x) is x
    assert d.max_over_ranks([3.0]) == [3.0]
    assert d.ensemble_max(x) is x
