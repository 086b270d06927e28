"""Limb-sharded rotation across GPUs: the host side of csrc/shard.cu.

One process per GPU (torch.distributed, NCCL).  Every rank holds the
ciphertext in the usual limb-major layout with only its own limbs valid; a
rotation is three local phases with two all-gathers in between, all queued on
the library's stream, so the exchange overlaps nothing it should not and the
received limbs are in local memory before a kernel reads them.

`emulate_rotate` runs the same phases for all ranks inside one process on one
GPU, with plain device copies standing in for the all-gathers: the sharding
logic can be checked where only one GPU is available.
"""
import ctypes as C

import numpy as np


def blocks(lib, level, world):
    qb, pb = C.c_int(), C.c_int()
    lib.Fhert_shard_blocks(level, world, C.byref(qb), C.byref(pb))
    return qb.value, pb.value


def owned_q(level, rank, world, qb):
    return range(min(level, rank * qb), min(level, (rank + 1) * qb))


class ShardedRotator:
    """Rotation of a sharded ciphertext on `world` GPUs (call on every rank)."""

    def __init__(self, gpu, level, rank, world):
        import torch
        self.torch, self.gpu, self.lib = torch, gpu, gpu.lib
        self.level, self.rank, self.world = level, rank, world
        self.qb, self.pb = blocks(self.lib, level, world)
        n, dev = gpu.N, torch.device("cuda", torch.cuda.current_device())
        self.gq = torch.zeros((world * self.qb, n), dtype=torch.int64, device=dev)
        self.gp = [torch.zeros((world * self.pb, n), dtype=torch.int64, device=dev) for _ in (0, 1)]
        self.stream = torch.cuda.ExternalStream(self.lib.Fhert_stream(), device=dev)

    def _gather(self, buf, block):
        import torch.distributed as dist
        mine = buf[self.rank * block:(self.rank + 1) * block]
        with self.torch.cuda.stream(self.stream):
            dist.all_gather_into_tensor(buf, mine)

    def rotate(self, c0_ptr, c1_ptr, rot_idx, out0_ptr, out1_ptr, conj=False):
        """c0/c1/out0/out1: device addresses of full-layout polynomials."""
        lib = self.lib
        st = lib.Fhert_shard_begin(c1_ptr, self.level, self.rank, self.world, self.gq.data_ptr())
        if self.world > 1:
            self._gather(self.gq, self.qb)
        lib.Fhert_shard_mid(st, c1_ptr, self.gq.data_ptr(), rot_idx, int(conj),
                            self.gp[0].data_ptr(), self.gp[1].data_ptr())
        if self.world > 1:
            self._gather(self.gp[0], self.pb)
            self._gather(self.gp[1], self.pb)
        lib.Fhert_shard_end(st, c0_ptr, self.gp[0].data_ptr(), self.gp[1].data_ptr(), rot_idx,
                            int(conj), out0_ptr, out1_ptr)

    def exchange_bytes(self):
        """Bytes this rank receives per rotation."""
        n8 = self.gpu.N * 8
        return (self.world - 1) * (self.qb + 2 * self.pb) * n8


def emulate_rotate(gpu, c0, c1, rot_idx, world, conj=False):
    """All ranks of a `world`-way sharded rotation in this process: returns the
    assembled (c0, c1) of the result as numpy arrays."""
    import ace_compiler_b200 as rt
    lib, n, level = gpu.lib, gpu.N, c0.shape[0]
    qb, pb = blocks(lib, level, world)
    ct = gpu.new_ciph(c0, c1)
    gq = gpu.new_poly(world * qb)
    gp0, gp1 = gpu.new_poly(world * pb), gpu.new_poly(world * pb)
    # per-rank private exchange buffers, then the "gathered" ones every rank reads
    parts = [(gpu.new_poly(world * qb), gpu.new_poly(world * pb), gpu.new_poly(world * pb))
             for _ in range(world)]
    c0p, c1p = ct._c0_poly._data, ct._c1_poly._data
    states = []
    for r in range(world):
        states.append(lib.Fhert_shard_begin(c1p, level, r, world, parts[r][0].contents._data))
    for r in range(world):  # all-gather of the Q blocks
        lo, hi = r * qb, min((r + 1) * qb, world * qb)
        for i in range(lo, hi):
            lib.Set_coeffs(gq, i, n, lib.Coeffs(parts[r][0], i, n))
    for r in range(world):
        lib.Fhert_shard_mid(states[r], c1p, gq.contents._data, rot_idx, int(conj),
                            parts[r][1].contents._data, parts[r][2].contents._data)
    for r in range(world):  # all-gather of the special-limb blocks
        for k in range(r * pb, (r + 1) * pb):
            lib.Set_coeffs(gp0, k, n, lib.Coeffs(parts[r][1], k, n))
            lib.Set_coeffs(gp1, k, n, lib.Coeffs(parts[r][2], k, n))
    outs = [gpu.new_ciph(np.zeros_like(c0), np.zeros_like(c1)) for _ in range(world)]
    for r in range(world):
        lib.Fhert_shard_end(states[r], c0p, gp0.contents._data, gp1.contents._data, rot_idx,
                            int(conj), outs[r]._c0_poly._data, outs[r]._c1_poly._data)
    res0, res1 = np.zeros_like(c0), np.zeros_like(c1)
    for r in range(world):
        h0, h1 = gpu.ciph_to_host(outs[r])
        for i in owned_q(level, r, world, qb):
            res0[i], res1[i] = h0[i], h1[i]
        gpu.free_ciph(outs[r])
    for p in [gq, gp0, gp1] + [x for t in parts for x in t]:
        gpu.free(p)
    gpu.free_ciph(ct)
    return res0, res1
