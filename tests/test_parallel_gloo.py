"""The multi-rank host logic on CPU: two gloo ranks deal out images, time them
independently and agree on the job's figures."""
import os
import socket

import pytest
import torch.multiprocessing as mp


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
    s.close()
    return port


def _rank_main(rank, world, port, q):
    import torch.distributed as dist

    from ace_compiler_b200 import parallel
    os.environ.update(RANK=str(rank), WORLD_SIZE=str(world), MASTER_ADDR="127.0.0.1",
                      MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    mine = parallel.images_of_rank(7, rank, world)
    # a fake per-image cost: rank 1 is the slow one
    ms_local = sum(100.0 + 50.0 * rank for _ in mine)
    ms, steps = parallel.slowest_rank([ms_local, float(len(mine))])
    logits = parallel.gather_logits([float(rank), float(len(mine))])
    dist.barrier()
    q.put((rank, mine, ms, steps, logits, parallel.job_throughput(3, world, ms)))
    dist.destroy_process_group()


def test_two_ranks_agree():
    world, port = 2, _free_port()
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    procs = [ctx.Process(target=_rank_main, args=(r, world, port, q)) for r in range(world)]
    for p in procs:
        p.start()
    got = sorted(q.get(timeout=120) for _ in range(world))
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    (r0, mine0, ms0, steps0, logits0, thr0), (r1, mine1, ms1, steps1, logits1, thr1) = got
    assert mine0 == [0, 2, 4, 6] and mine1 == [1, 3, 5]
    assert sorted(mine0 + mine1) == list(range(7))
    # the slowest rank defines the job: rank 1 has 3 images at 150 ms, rank 0 has 4 at 100 ms
    assert ms0 == ms1 == pytest.approx(450.0)
    assert steps0 == steps1 == 4.0
    assert logits0 == logits1 == [[0.0, 4.0], [1.0, 3.0]]
    assert thr0 == thr1 == pytest.approx(3 * 2 / 0.45)


def test_single_process_needs_no_group():
    from ace_compiler_b200 import parallel
    assert parallel.slowest_rank([12.5]) == [12.5]
    assert parallel.images_of_rank(5, 0, 1) == [0, 1, 2, 3, 4]
    assert parallel.gather_logits([1.0, 2.0]) == [[1.0, 2.0]]
