"""Limb-sharded ciphertext operations across GPUs: the host side of csrc/shard.cu.

One process per GPU.  Every rank holds the ciphertext in the usual limb-major
layout with only its own limbs valid (contiguous blocks of the context's Q
primes, the same owner at every level).  `ShardedOps` drives the library's own
entry points (Fhert_shard_rotate / _mul_relin / _rescale), which issue their
exchanges as NCCL collectives on the library stream; this module only hands the
communicator identifier from rank 0 to the others.  `ShardedRotator` is the
older form in which the host runs the all-gathers between the phases through
torch.distributed.

The `emulate_*` functions run the phases of all ranks inside one process on one
GPU, with plain device copies standing in for the collectives: the sharding
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


class ShardedOps:
    """Rotation, multiplication with relinearisation and rescale of sharded
    ciphertexts with the exchanges inside the library (call on every rank)."""

    def __init__(self, gpu, rank, world, broadcast_bytes=None):
        """broadcast_bytes(buf: bytearray, src=0) must make rank 0's 128 bytes
        appear on every rank (defaults to torch.distributed.broadcast)."""
        self.gpu, self.lib, self.rank, self.world = gpu, gpu.lib, rank, world
        ident = (C.c_char * 128)()
        if world > 1:
            if rank == 0:
                rc = self.lib.Fhert_shard_comm_id(ident)
                if rc != 0:
                    raise RuntimeError(f"NCCL is not available to the library (code {rc})")
            buf = bytearray(ident.raw)
            if broadcast_bytes is None:
                import torch
                import torch.distributed as dist
                t = torch.tensor(list(buf), dtype=torch.uint8)
                if dist.get_backend() == "nccl":
                    t = t.cuda()
                dist.broadcast(t, 0)
                buf = bytearray(t.cpu().tolist())
            else:
                broadcast_bytes(buf, 0)
            ident = (C.c_char * 128).from_buffer_copy(bytes(buf))
        rc = self.lib.Fhert_shard_comm_init(ident, rank, world)
        if rc != 0:
            raise RuntimeError(f"Fhert_shard_comm_init failed (code {rc})")

    def close(self):
        self.lib.Fhert_shard_comm_destroy()

    def rotate(self, res, ct, rot_idx, conj=False):
        self.lib.Fhert_shard_rotate(C.byref(res), C.byref(ct), rot_idx, int(conj))

    def mul_relin(self, res, a, b):
        self.lib.Fhert_shard_mul_relin(C.byref(res), C.byref(a), C.byref(b))

    def rescale(self, res, ct):
        self.lib.Fhert_shard_rescale(C.byref(res), C.byref(ct))

    def exchange_bytes(self, level, op):
        """Bytes this rank receives per operation at `level`."""
        qb, pb = blocks(self.lib, level, self.world)
        n8 = self.gpu.N * 8
        if op == "rescale":
            return 0 if (level - 1) // qb == self.rank else 2 * n8
        return (self.world - 1) * (qb + 2 * pb) * n8


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
        # the zero fills above ran on torch's current stream; the library stream does
        # not order itself against that one
        self.stream.wait_stream(torch.cuda.current_stream())

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


def _gather_blocks(gpu, dst, srcs, block):
    """dst[r*block + j] = srcs[r][r*block + j]: what an all-gather leaves everywhere."""
    lib, n = gpu.lib, gpu.N
    for r, src in enumerate(srcs):
        for i in range(r * block, (r + 1) * block):
            lib.Set_coeffs(dst, i, n, lib.Coeffs(src, i, n))


def emulate_mul_relin(gpu, a0, a1, b0, b1, world):
    """All ranks of a sharded multiplication with relinearisation in this
    process: returns the assembled (c0, c1) of the product (same level)."""
    lib, n, level = gpu.lib, gpu.N, a0.shape[0]
    qb, pb = blocks(lib, level, world)
    ca, cb = gpu.new_ciph(a0, a1), gpu.new_ciph(b0, b1)
    gq, gp0, gp1 = gpu.new_poly(world * qb), gpu.new_poly(world * pb), gpu.new_poly(world * pb)
    per = [dict(d=[gpu.new_poly(level) for _ in range(3)], gq=gpu.new_poly(world * qb),
                gp0=gpu.new_poly(world * pb), gp1=gpu.new_poly(world * pb)) for _ in range(world)]
    states = []
    for r in range(world):
        d = [p.contents._data for p in per[r]["d"]]
        lib.Fhert_shard_tensor(ca._c0_poly._data, ca._c1_poly._data, cb._c0_poly._data,
                               cb._c1_poly._data, level, r, world, d[0], d[1], d[2])
        states.append(lib.Fhert_shard_begin(d[2], level, r, world, per[r]["gq"].contents._data))
    _gather_blocks(gpu, gq, [p["gq"] for p in per], qb)
    for r in range(world):
        lib.Fhert_shard_mid(states[r], per[r]["d"][2].contents._data, gq.contents._data, 0, 2,
                            per[r]["gp0"].contents._data, per[r]["gp1"].contents._data)
    _gather_blocks(gpu, gp0, [p["gp0"] for p in per], pb)
    _gather_blocks(gpu, gp1, [p["gp1"] for p in per], pb)
    outs = [gpu.new_ciph(np.zeros_like(a0), np.zeros_like(a1)) for _ in range(world)]
    for r in range(world):
        lib.Fhert_shard_end2(states[r], per[r]["d"][0].contents._data, per[r]["d"][1].contents._data,
                             gp0.contents._data, gp1.contents._data, 0, 2,
                             outs[r]._c0_poly._data, outs[r]._c1_poly._data)
    res0, res1 = np.zeros_like(a0), np.zeros_like(a1)
    for r in range(world):
        h0, h1 = gpu.ciph_to_host(outs[r])
        for i in owned_q(level, r, world, qb):
            res0[i], res1[i] = h0[i], h1[i]
        gpu.free_ciph(outs[r])
    for p in [gq, gp0, gp1] + [x for t in per for x in t["d"] + [t["gq"], t["gp0"], t["gp1"]]]:
        gpu.free(p)
    gpu.free_ciph(ca)
    gpu.free_ciph(cb)
    return res0, res1


def emulate_rescale(gpu, c0, c1, world):
    """All ranks of a sharded rescale in this process: the assembled result
    (level - 1 limbs)."""
    lib, n, level = gpu.lib, gpu.N, c0.shape[0]
    qb, _ = blocks(lib, level, world)
    ct = gpu.new_ciph(c0, c1)
    bc = gpu.new_poly(2)
    owners = [lib.Fhert_shard_rescale_begin(ct._c0_poly._data, ct._c1_poly._data, level, r, world,
                                            bc.contents._data) for r in range(world)]
    assert sum(owners) == 1
    outs = [gpu.new_ciph(np.zeros_like(c0), np.zeros_like(c1)) for _ in range(world)]
    for r in range(world):
        lib.Fhert_shard_rescale_end(ct._c0_poly._data, ct._c1_poly._data, level, r, world,
                                    bc.contents._data, outs[r]._c0_poly._data,
                                    outs[r]._c1_poly._data)
    res0, res1 = np.zeros_like(c0[:-1]), np.zeros_like(c1[:-1])
    for r in range(world):
        h0, h1 = gpu.ciph_to_host(outs[r])
        for i in owned_q(level - 1, r, world, qb):
            res0[i], res1[i] = h0[i], h1[i]
        gpu.free_ciph(outs[r])
    gpu.free(bc)
    gpu.free_ciph(ct)
    return res0, res1
