"""Deferred per-limb operations: random sequences of Hw_* calls, including
in-place updates, a shared scratch limb reused by every step, dead stores and
limb copies, must leave exactly what running them one by one would."""
import ctypes as C

import numpy as np
import pytest

pytestmark = pytest.mark.gpu

N, L = 1024, 4


@pytest.fixture(scope="module")
def gpu():
    import ace_compiler_b200 as rt
    g = rt.Runtime(N, L, 60, 56, 2, rot_idxs=(1, 3))
    yield g
    g.close()


def run_program(gpu, seed, steps, limbs=10):
    lib = gpu.lib
    rng = np.random.default_rng(seed)
    primes = gpu.primes
    # every limb buffer belongs to one prime; operations stay within a prime
    owner = [int(rng.integers(0, 2)) for _ in range(limbs)]
    poly = gpu.new_poly(limbs)
    host = np.stack([rng.integers(0, primes[owner[i]], N, dtype=np.int64) for i in range(limbs)])
    gpu.upload(poly, host)
    model = [host[i].astype(object) for i in range(limbs)]
    order_dev = lib.Auto_order(1)
    # the permutation itself: rotate the identity vector once
    ident = gpu.new_poly(2)
    gpu.upload(ident, np.stack([np.arange(N, dtype=np.int64), np.zeros(N, np.int64)]))
    lib.Hw_rotate(gpu.limb_ptr(ident, 1), gpu.limb_ptr(ident, 0), order_dev, gpu.modulus(0), N)
    table = gpu.download(ident)[1].astype(np.int64)
    gpu.free(ident)

    def ptr(i):
        return gpu.limb_ptr(poly, i)

    def mod(i):
        return gpu.modulus(owner[i])

    for step in range(steps):
        kind = int(rng.integers(0, 9))
        d = int(rng.integers(0, limbs))
        same = [i for i in range(limbs) if owner[i] == owner[d]]
        a = int(rng.choice(same))
        b = int(rng.choice(same))
        q = primes[owner[d]]
        if step % 5 == 0:
            d = 0 if owner[0] == owner[d] else d  # limb 0 doubles as the shared scratch
            same = [i for i in range(limbs) if owner[i] == owner[d]]
            a, b = int(rng.choice(same)), int(rng.choice(same))
        if kind == 0:
            lib.Hw_modadd(ptr(d), ptr(a), ptr(b), mod(d), N)
            model[d] = (model[a] + model[b]) % q
        elif kind == 1:
            lib.Hw_modsub(ptr(d), ptr(a), ptr(b), mod(d), N)
            model[d] = (model[a] - model[b]) % q
        elif kind == 2:
            lib.Hw_modmul(ptr(d), ptr(a), ptr(b), mod(d), N)
            model[d] = (model[a] * model[b]) % q
        elif kind == 3:
            lib.Hw_modmuladd(ptr(d), ptr(a), ptr(b), mod(d), N)
            model[d] = (model[d] + model[a] * model[b]) % q
        elif kind == 4:
            s = int(rng.integers(-2 ** 40, 2 ** 40))
            lib.Hw_modadd_scalar(ptr(d), ptr(a), s, mod(d), N)
            model[d] = (model[a] + s) % q
        elif kind == 5:
            s = int(rng.integers(-2 ** 40, 2 ** 40))
            lib.Hw_modmul_scalar(ptr(d), ptr(a), s, mod(d), N)
            model[d] = (model[a] * s) % q
        elif kind == 6:
            if a == d:
                continue
            lib.Hw_rotate(ptr(d), ptr(a), order_dev, mod(d), N)
            model[d] = model[a][table]
        elif kind == 7:
            lib.Set_coeffs(poly, d, N, ptr(a))
            model[d] = model[a].copy()
        else:
            if step % 3 == 0:
                lib.Fhert_sync()  # an unrelated entry point in the middle of a sequence
    got = gpu.download(poly)
    want = np.stack([m.astype(np.int64) for m in model])
    gpu.free(poly)
    return got, want


@pytest.mark.parametrize("seed", range(6))
def test_random_limb_programs(gpu, seed):
    before = gpu.lib.Fhert_kernel_launches()
    got, want = run_program(gpu, seed, 400)
    assert np.array_equal(got, want)
    launches = gpu.lib.Fhert_kernel_launches() - before
    assert launches < 400  # recorded calls were merged into fewer launches


@pytest.mark.parametrize("seed", range(20, 26))
def test_random_limb_programs_on_few_limbs(gpu, seed):
    """Four limbs only: nearly every call depends on the one before it, through
    values, overwritten sources and rotated sources alike."""
    got, want = run_program(gpu, seed, 500, limbs=4)
    assert np.array_equal(got, want)


def test_long_accumulation_runs_as_one_chain(gpu):
    """acc[l] += w[i][l] * rot_i(x)[l] over 448 terms with one shared product limb
    and one shared rotated limb per l: the sums of one limb form one chain, which
    here is longer than a launch holds and continues in the next one."""
    lib = gpu.lib
    rng = np.random.default_rng(5)
    limbs, terms = 3, 448
    primes = gpu.primes[:limbs]
    order_dev = lib.Auto_order(1)
    ident = gpu.new_poly(2)
    gpu.upload(ident, np.stack([np.arange(N, dtype=np.int64), np.zeros(N, np.int64)]))
    lib.Hw_rotate(gpu.limb_ptr(ident, 1), gpu.limb_ptr(ident, 0), order_dev, gpu.modulus(0), N)
    table = gpu.download(ident)[1].astype(np.int64)
    gpu.free(ident)
    hx = np.stack([rng.integers(0, p, (terms, N), dtype=np.int64) for p in primes])  # [l][i]
    hw = np.stack([rng.integers(0, p, (terms, N), dtype=np.int64) for p in primes])
    # operand i of limb l lives in limb i % L of the (i // L)-th polynomial of its pool
    pools = {}
    for name, host in (("x", hx), ("w", hw)):
        for l in range(limbs):
            pools[name, l] = [gpu.new_poly(L, data=host[l][k:k + L]) for k in range(0, terms, L)]

    def operand(name, l, i):
        return gpu.limb_ptr(pools[name, l][i // L], i % L)

    acc = gpu.new_poly(limbs); gpu.upload(acc, np.zeros((limbs, N), np.int64))
    rot = gpu.new_poly(1); tmp = gpu.new_poly(1)
    lib.Fhert_sync()
    before = lib.Fhert_kernel_launches()
    for i in range(terms):
        for l in range(limbs):
            m = gpu.modulus(l)
            lib.Hw_rotate(gpu.limb_ptr(rot, 0), operand("x", l, i), order_dev, m, N)
            lib.Hw_modmul(gpu.limb_ptr(tmp, 0), operand("w", l, i), gpu.limb_ptr(rot, 0), m, N)
            lib.Hw_modadd(gpu.limb_ptr(acc, l), gpu.limb_ptr(acc, l), gpu.limb_ptr(tmp, 0), m, N)
    lib.Fhert_sync()
    launches = lib.Fhert_kernel_launches() - before
    assert launches <= 24, launches
    want = np.zeros((limbs, N), dtype=object)
    for l in range(limbs):
        for i in range(terms):
            want[l] = (want[l] + hw[l][i].astype(object) * hx[l][i][table].astype(object)) % primes[l]
    assert np.array_equal(gpu.download(acc), want.astype(np.int64))
    for p in [q for pool in pools.values() for q in pool] + [acc, rot, tmp]:
        gpu.free(p)


def test_key_switch_idiom_is_merged(gpu):
    """tmp = key * digit; acc += tmp for every limb with one shared tmp: two
    launches, not two per limb."""
    lib = gpu.lib
    rng = np.random.default_rng(11)
    limbs = 32
    q = gpu.primes[0]
    key = gpu.new_poly(limbs); dig = gpu.new_poly(limbs); acc = gpu.new_poly(limbs)
    tmp = gpu.new_poly(1)
    hk = rng.integers(0, q, (limbs, N), dtype=np.int64)
    hd = rng.integers(0, q, (limbs, N), dtype=np.int64)
    ha = rng.integers(0, q, (limbs, N), dtype=np.int64)
    gpu.upload(key, hk); gpu.upload(dig, hd); gpu.upload(acc, ha)
    m0 = gpu.modulus(0)
    lib.Fhert_sync()
    before = lib.Fhert_kernel_launches()
    for i in range(limbs):
        lib.Hw_modmul(lib.Coeffs(tmp, 0, N), lib.Coeffs(key, i, N), lib.Coeffs(dig, i, N), m0, N)
        lib.Hw_modadd(lib.Coeffs(acc, i, N), lib.Coeffs(acc, i, N), lib.Coeffs(tmp, 0, N), m0, N)
    lib.Fhert_sync()
    assert lib.Fhert_kernel_launches() - before <= 3
    want = (ha.astype(object) + hk.astype(object) * hd.astype(object)) % q
    assert np.array_equal(gpu.download(acc), want.astype(np.int64))
    last = (hk[-1].astype(object) * hd[-1].astype(object)) % q
    assert np.array_equal(gpu.download(tmp)[0], last.astype(np.int64))
    for p in (key, dig, acc, tmp):
        gpu.free(p)


def test_waiting_rescale_runs_before_younger_limb_calls(gpu):
    """A lone Rescale waits for a sibling; per-limb calls recorded after it read
    its result, so the drain must run the Rescale first."""
    lib = gpu.lib
    rng = np.random.default_rng(31)
    level = 4
    data = np.stack([rng.integers(0, p, N, dtype=np.int64) for p in gpu.primes[:level]])
    src = gpu.new_poly(level, data=data)
    ref_out = gpu.new_poly(level)
    lib.Rescale(ref_out, src)
    want = gpu.download(ref_out)          # the download drains: the plain result
    out = gpu.new_poly(level)
    acc = gpu.new_poly(level - 1)
    gpu.upload(acc, np.zeros((level - 1, N), np.int64))
    lib.Rescale(out, src)                 # waits
    for i in range(level - 1):            # recorded, reads the waiting call's result
        lib.Hw_modadd(gpu.limb_ptr(acc, i), gpu.limb_ptr(acc, i), gpu.limb_ptr(out, i),
                      gpu.modulus(i), N)
    assert np.array_equal(gpu.download(acc), want)
    for p in (src, ref_out, out, acc):
        gpu.free(p)


def _raise_all(gpu, src, level, order):
    """Decomp_modup of every digit in the given order, each into its own result."""
    lib = gpu.lib
    parts = int(lib.Num_decomp(src))
    out = {}
    for p in order:
        ext = gpu.new_poly(level, extended=True)
        lib.Decomp_modup(ext, src, p)
        out[p] = ext
    assert sorted(out) == list(range(parts))
    return out


def test_digits_raised_together_equal_digits_raised_alone(gpu):
    """Digit 0 first makes the library raise all digits at once and hand the others
    out later; any other order raises each digit on its own.  Same residues."""
    lib = gpu.lib
    rng = np.random.default_rng(41)
    level = L
    data = np.stack([rng.integers(0, p, N, dtype=np.int64) for p in gpu.primes[:level]])
    src = gpu.new_poly(level, data=data)
    parts = int(lib.Num_decomp(src))
    assert parts >= 2
    alone = _raise_all(gpu, src, level, list(range(1, parts)) + [0])
    want = {p: gpu.download(alone[p]) for p in alone}
    lib.Fhert_sync()
    before = lib.Fhert_kernel_launches()
    together = _raise_all(gpu, src, level, list(range(parts)))
    launches = lib.Fhert_kernel_launches() - before
    for p in range(parts):
        assert np.array_equal(gpu.download(together[p]), want[p]), p
    assert launches <= 8, launches  # one batch of launches, not one per digit
    for p in list(alone.values()) + list(together.values()) + [src]:
        gpu.free(p)


def test_kept_digits_follow_the_program(gpu):
    """One result polynomial reused for every digit with per-limb calls in between
    (the emitted key-switch loop); then the source changes between two digits, and
    the later digit must come from the changed source."""
    lib = gpu.lib
    rng = np.random.default_rng(43)
    level = L
    primes = gpu.primes
    data = np.stack([rng.integers(0, p, N, dtype=np.int64) for p in primes[:level]])
    src = gpu.new_poly(level, data=data)
    parts = int(lib.Num_decomp(src))
    alone = _raise_all(gpu, src, level, list(range(1, parts)) + [0])
    want = {p: gpu.download(alone[p]) for p in alone}
    # acc_i = sum over digits of ext_i (Q limbs only), ext shared by all digits
    ext = gpu.new_poly(level, extended=True)
    acc = gpu.new_poly(level)
    gpu.upload(acc, np.zeros((level, N), np.int64))
    for p in range(parts):
        lib.Decomp_modup(ext, src, p)
        for i in range(level):
            lib.Hw_modadd(gpu.limb_ptr(acc, i), gpu.limb_ptr(acc, i), gpu.limb_ptr(ext, i),
                          gpu.modulus(i), N)
    total = np.zeros((level, N), dtype=object)
    for p in range(parts):
        total += want[p][:level].astype(object)
    for i in range(level):
        total[i] %= primes[i]
    assert np.array_equal(gpu.download(acc), total.astype(np.int64))
    assert np.array_equal(gpu.download(ext), want[parts - 1])  # the last digit stays in ext
    # the source changes after digit 0 was handed out
    lib.Decomp_modup(ext, src, 0)
    lib.Hw_modadd_scalar(gpu.limb_ptr(src, level - 1), gpu.limb_ptr(src, level - 1), 5,
                         gpu.modulus(level - 1), N)
    lib.Decomp_modup(ext, src, parts - 1)
    got = gpu.download(ext)
    changed = data.copy()
    changed[level - 1] = (changed[level - 1] + 5) % primes[level - 1]
    src2 = gpu.new_poly(level, data=changed)
    ref = gpu.new_poly(level, extended=True)
    lib.Decomp_modup(ref, src2, parts - 1)
    assert np.array_equal(got, gpu.download(ref))
    for p in list(alone.values()) + [src, src2, ext, acc, ref]:
        gpu.free(p)


def test_write_into_a_handed_out_digit_does_not_spoil_later_digits(gpu):
    """A result limb of Decomp_modup is an alias of the digits the library keeps; a
    recorded in-place write to that limb must not change what a second
    Decomp_modup of the same, unchanged polynomial returns."""
    lib = gpu.lib
    rng = np.random.default_rng(44)
    level = L
    data = np.stack([rng.integers(0, p, N, dtype=np.int64) for p in gpu.primes[:level]])
    src = gpu.new_poly(level, data=data)
    fresh = gpu.new_poly(level, extended=True)
    lib.Decomp_modup(fresh, src, 0)
    want = gpu.download(fresh)          # (the download drains the recording: kept digits go)
    ext, ext2 = gpu.new_poly(level, extended=True), gpu.new_poly(level, extended=True)
    lib.Decomp_modup(ext, src, 0)
    limb = level - 1                    # a limb outside digit 0: a converted one
    lib.Hw_modadd_scalar(gpu.limb_ptr(ext, limb), gpu.limb_ptr(ext, limb), 7, gpu.modulus(limb), N)
    lib.Decomp_modup(ext2, src, 0)
    assert np.array_equal(gpu.download(ext2), want)
    changed = want.copy()
    changed[limb] = (changed[limb] + 7) % gpu.primes[limb]
    assert np.array_equal(gpu.download(ext), changed)
    for p in (src, fresh, ext, ext2):
        gpu.free(p)
