"""Limb-sharded rotation, multiplication with relinearisation and rescale:
the per-rank phases run for every rank on one GPU (device copies in place of
the collectives) and, where two GPUs are visible, as two ranks whose exchanges
the library issues itself through NCCL; the assembled results equal the
reference runtime's."""
import ctypes as C
import os
import socket

import numpy as np
import pytest

from tests import ref_runtime as rr

pytestmark = pytest.mark.gpu

N, L = 8192, 11
ROTS = (1, 5)


@pytest.fixture(scope="module")
def pair():
    if not rr.available():
        pytest.skip("reference runtime not built")
    import ace_compiler_b200 as rt
    seed = np.arange(16, dtype=np.uint32) + 9
    ref = rr.RefRuntime(N, L, 60, 56, 3, rot_idxs=ROTS, seed=seed, fake_time_us=1_700_000_000_000_009)
    gpu = rt.Runtime(N, L, 60, 56, 3, rot_idxs=ROTS, keygen=True, seed=seed,
                     fake_time_us=1_700_000_000_000_009)
    yield ref, gpu
    gpu.close()
    rr.close_ref(ref)


@pytest.mark.parametrize("world", [1, 2, 3, 4, 8])
def test_all_ranks_on_one_gpu(pair, world):
    from ace_compiler_b200 import sharded
    ref, gpu = pair
    rng = np.random.default_rng(40 + world)
    for level in (L, 7, 3):
        c0 = rr.uniform_limbs(rng, gpu.primes[:level], N)
        c1 = rr.uniform_limbs(rng, gpu.primes[:level], N)
        for rot in ROTS:
            got = sharded.emulate_rotate(gpu, c0, c1, rot, world)
            want = ref.rotate(c0, c1, rot)
            assert np.array_equal(got[0], want[0]) and np.array_equal(got[1], want[1]), (world, level, rot)


@pytest.mark.parametrize("world", [1, 2, 3, 4, 8])
def test_mul_relin_and_rescale_all_ranks_on_one_gpu(pair, world):
    from ace_compiler_b200 import sharded
    ref, gpu = pair
    rng = np.random.default_rng(60 + world)
    for level in (L, 6, 2):
        a0, a1, b0, b1 = (rr.uniform_limbs(rng, gpu.primes[:level], N) for _ in range(4))
        p0, p1 = sharded.emulate_mul_relin(gpu, a0, a1, b0, b1, world)
        r0, r1 = sharded.emulate_rescale(gpu, p0, p1, world)
        w0, w1 = ref.mul_relin_rescale(a0, a1, b0, b1)
        assert np.array_equal(r0, w0) and np.array_equal(r1, w1), (world, level)


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
    s.close()
    return port


def _nccl_rank(rank, world, port, q):
    import torch
    import torch.distributed as dist

    import ace_compiler_b200 as rt
    from ace_compiler_b200 import sharded
    os.environ.update(RANK=str(rank), WORLD_SIZE=str(world), MASTER_ADDR="127.0.0.1",
                      MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    seed = np.arange(16, dtype=np.uint32) + 9
    gpu = rt.Runtime(N, L, 60, 56, 3, rot_idxs=ROTS, keygen=True, seed=seed,
                     fake_time_us=1_700_000_000_000_009)
    rng = np.random.default_rng(77)   # same ciphertext on every rank
    c0 = np.stack([rng.integers(0, p, N, dtype=np.int64) for p in gpu.primes[:L]])
    c1 = np.stack([rng.integers(0, p, N, dtype=np.int64) for p in gpu.primes[:L]])
    whole = rt.CIPHERTEXT()
    full = gpu.new_ciph(c0, c1)
    gpu.lib.Rotate_ciph(C.byref(whole), C.byref(full), ROTS[0])
    want = gpu.ciph_to_host(whole)
    rot = sharded.ShardedRotator(gpu, L, rank, world)
    # foreign limbs of the input are garbage on purpose
    mine = list(sharded.owned_q(L, rank, world, rot.qb))
    d0, d1 = np.full_like(c0, 12345), np.full_like(c1, 54321)
    d0[mine], d1[mine] = c0[mine], c1[mine]
    ct = gpu.new_ciph(d0, d1)
    out = gpu.new_ciph(np.zeros_like(c0), np.zeros_like(c1))
    rot.rotate(ct._c0_poly._data, ct._c1_poly._data, ROTS[0], out._c0_poly._data, out._c1_poly._data)
    got = gpu.ciph_to_host(out)
    ok = all(np.array_equal(got[0][i], want[0][i]) and np.array_equal(got[1][i], want[1][i])
             for i in mine)
    # the same rotation, then a product and a rescale, with the exchanges inside the library
    ops = sharded.ShardedOps(gpu, rank, world)
    res = rt.CIPHERTEXT()
    ops.rotate(res, ct, ROTS[0])
    got = gpu.ciph_to_host(res)
    ok = ok and all(np.array_equal(got[0][i], want[0][i]) and np.array_equal(got[1][i], want[1][i])
                    for i in mine)
    prod_whole, resc_whole = rt.CIPHERTEXT(), rt.CIPHERTEXT()
    gpu.lib.Mul_ciph(C.byref(prod_whole), C.byref(full), C.byref(whole))
    gpu.lib.Rescale_ciph(C.byref(resc_whole), C.byref(prod_whole))
    want2 = gpu.ciph_to_host(resc_whole)
    prod, resc = rt.CIPHERTEXT(), rt.CIPHERTEXT()
    ops.mul_relin(prod, ct, res)
    ops.rescale(resc, prod)
    got2 = gpu.ciph_to_host(resc)
    mine2 = [i for i in mine if i < L - 1]
    ok = ok and all(np.array_equal(got2[0][i], want2[0][i]) and np.array_equal(got2[1][i], want2[1][i])
                    for i in mine2)
    ops.close()
    dist.barrier()
    q.put((rank, ok, mine))
    gpu.close()
    dist.destroy_process_group()


def test_two_nccl_ranks():
    import torch
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    import torch.multiprocessing as mp
    world, port = 2, _free_port()
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    procs = [ctx.Process(target=_nccl_rank, args=(r, world, port, q)) for r in range(world)]
    for p in procs:
        p.start()
    got = sorted(q.get(timeout=600) for _ in range(world))
    for p in procs:
        p.join(timeout=120)
        assert p.exitcode == 0
    assert all(ok for _, ok, _ in got)
    assert sorted(i for _, _, mine in got for i in mine) == list(range(L))
