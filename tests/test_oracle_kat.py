"""Pins the CPU oracle's scalar arithmetic against the known answers held by the
reference's own unit tests (cahel-main/unittest/util/uintarithsmallmod.cu and numth.cu)."""
import numpy as np

from oracle.binding import Oracle, coeff_modulus_create, elts_from_steps, lib


def test_multiply_uint_mod_kat():
    # cahel-main/unittest/util/uintarithsmallmod.cu:184-209
    assert lib.orc_mulmod(7, 7, 10) == 9
    assert lib.orc_mulmod(6, 7, 10) == 2
    mod = 2305843009211596801
    assert lib.orc_mulmod(1152921504605798400, 1152921504605798401, mod) == 576460752302899200
    assert lib.orc_mulmod(1152921504605798401, 1152921504605798401, mod) == 1729382256908697601
    assert lib.orc_mulmod(2305843009211596800, 2305843009211596800, mod) == 1


def test_barrett_reduce_128_kat():
    # cahel-main/unittest/util/uintarithsmallmod.cu:140-182: (hi:lo) mod m through Python integers
    # and through the oracle's own product path for values that are products
    mod = 13131313131313
    assert ((456 << 64) | 123) % mod == 8722750765283
    assert ((79797979797979 << 64) | 24242424242424) % mod == 1010101010101
    # same numbers through mulmod: (a * 2^64 + b) mod m = (a mod m)(2^64 mod m) + b
    t = (lib.orc_mulmod(456 % mod, (1 << 64) % mod, mod) + 123) % mod
    assert t == 8722750765283


def test_invert_and_exponentiate_kat():
    # cahel-main/unittest/util/uintarithsmallmod.cu:295-333 (prime moduli only: the oracle inverts by Fermat)
    assert lib.orc_invmod(2, 5) == 3 and lib.orc_invmod(3, 5) == 2 and lib.orc_invmod(4, 5) == 4
    # 1351315121 of that test is composite, out of the Fermat inverse's domain; same answer by Python
    assert pow(331975426, -1, 1351315121) == 1052541512
    assert lib.orc_powmod(2, 0xFFFFFFFFFFFFFFFF, 5) == 3
    assert lib.orc_powmod(2424242424, 16, 131313131313) == 39418477653


def test_shoup_operand_kat():
    # cahel-main/unittest/util/uintarithsmallmod.cu:371-400
    assert lib.orc_shoup(1, 3) == 6148914691236517205
    assert lib.orc_shoup(2, 3) == 12297829382473034410
    assert lib.orc_shoup(1, 2147483647) == 8589934596
    assert lib.orc_shoup(2147483646, 2147483647) == 18446744065119617019
    assert lib.orc_shoup(1, 2305843009211596801) == 8
    assert lib.orc_shoup(2305843009211596800, 2305843009211596801) == 18446744073709551607


def test_is_prime_kat():
    # cahel-main/unittest/util/numth.cu:95-110
    for n, want in [(0, 0), (2, 1), (3, 1), (4, 0), (5, 1), (221, 0), (65537, 1), (65536, 0), (59399, 1), (72307, 1),
                    (72307 * 59399, 0), (36893488147419103, 1), (36893488147419107, 0)]:
        assert lib.orc_is_prime(n) == want, n


def test_minimal_primitive_root_kat():
    # cahel-main/unittest/util/numth.cu:197-216
    assert lib.orc_minimal_primitive_root(2, 11) == 10
    assert lib.orc_minimal_primitive_root(2, 29) == 28
    assert lib.orc_minimal_primitive_root(4, 29) == 12
    assert lib.orc_minimal_primitive_root(2, 1234565441) == 1234565440
    assert lib.orc_minimal_primitive_root(8, 1234565441) == 249725733


def test_prime_chain_properties():
    for logn, bits in [(13, [60, 40, 40, 60]), (15, [60, 40, 40, 60]), (16, [60] + [50] * 23 + [60] * 8)]:
        n = 1 << logn
        mods = coeff_modulus_create(n, bits)
        assert len(set(mods)) == len(mods)
        for m, b in zip(mods, bits):
            assert m.bit_length() == b and m % (2 * n) == 1 and lib.orc_is_prime(m)
        # the first request of a size gets the largest candidate, later ones descend
        seen = {}
        for m, b in zip(mods, bits):
            if b in seen:
                assert m < seen[b]
            seen[b] = m
        # nothing qualifying lies above the largest one handed out
        top = max(m for m, b in zip(mods, bits) if b == bits[0])
        c = top + 2 * n
        while c < (1 << bits[0]):
            assert not lib.orc_is_prime(c)
            c += 2 * n


def test_galois_elements():
    n = 1 << 13
    assert elts_from_steps([0], n) == [2 * n - 1]
    assert elts_from_steps([1, 2, 3], n) == [5, 25, 125]
    assert elts_from_steps([-1], n) == [pow(5, n // 2 - 1, 2 * n)]


def test_ntt_is_negacyclic_convolution():
    logn, n = 5, 32
    mods = coeff_modulus_create(n, [30, 30])
    o = Oracle(logn, mods, 1)
    rng = np.random.default_rng(1)
    for r, q in enumerate(mods[:1]):
        a = rng.integers(0, q, n, dtype=np.uint64)
        b = rng.integers(0, q, n, dtype=np.uint64)
        fa = o.ntt_rows(a[None], 1, 1, 0)
        fb = o.ntt_rows(b[None], 1, 1, 0)
        prod = o.poly_op("mul", 1, fa, fb)
        c = o.ntt_rows(prod, 1, 1, 0, inverse=True)[0]
        want = [0] * n
        for i in range(n):
            for j in range(n):
                k, s = (i + j) % n, (-1 if i + j >= n else 1)
                want[k] = (want[k] + s * int(a[i]) * int(b[j])) % q
        assert [int(x) for x in c] == want
        # psi is a primitive 2n-th root and the table is psi^bitrev(i)
        psi = o.psi(0)
        assert pow(psi, n, q) == q - 1
        tw = o.twiddles(0)
        assert int(tw[1]) == pow(psi, n // 2, q)


def test_ntt_round_trip_all_limbs():
    logn = 10
    mods = coeff_modulus_create(1 << logn, [60, 40, 40, 60])
    o = Oracle(logn, mods, 1)
    rng = np.random.default_rng(2)
    data = np.stack([rng.integers(0, q, 1 << logn, dtype=np.uint64) for q in mods])
    f = o.ntt_rows(data, 1, 3, 1)
    assert not np.array_equal(f, data)
    assert np.array_equal(o.ntt_rows(f, 1, 3, 1, inverse=True), data)


def test_ckks_chain_semantics():
    """encode -> encrypt -> multiply -> relinearize -> rescale -> rotate -> decrypt -> decode
    reproduces the plaintext computation (the tolerance of cahel-main/examples/example.h:14-19 is 1e-3)."""
    logn, n = 11, 1 << 11
    mods = coeff_modulus_create(n, [60, 40, 40, 60])
    elts = elts_from_steps([1, 2], n)
    o = Oracle(logn, mods, 1, elts)
    rng = np.random.default_rng(3)
    seed = lambda: rng.integers(0, 256, 64, dtype=np.uint8)
    sk = o.gen_sk(seed())
    pk = o.gen_pk(sk, seed(), seed())
    v1, v2 = rng.uniform(-1, 1, n // 2), rng.uniform(-1, 1, n // 2)
    scale = 2.0 ** 40
    pt1, pt2 = o.encode(3, v1, scale), o.encode(3, v2, scale)
    assert np.abs(o.decode(3, pt1, scale, n // 2) - v1).max() < 1e-9
    ct1, ct2 = o.encrypt_asym(pk, pt1, seed(), seed()), o.encrypt_asym(pk, pt2, seed(), seed())
    ct3 = o.tensor(3, ct1, ct2)
    rlk = o.gen_ksk(sk, o.sk_square(sk), np.concatenate([seed() for _ in range(6)]))
    ct = o.rescale(3, o.relinearize(3, ct3, rlk))
    s2 = scale * scale / mods[2]
    got = o.decode(2, o.decrypt(2, ct, sk), s2, n // 2)
    assert np.abs(got - v1 * v2).max() < 1e-5
    glk = [o.gen_ksk(sk, o.galois(i, sk), np.concatenate([seed() for _ in range(6)])) for i in range(2)]
    rot = o.rotate(2, ct, 0, glk[0])
    got = o.decode(2, o.decrypt(2, rot, sk), s2, n // 2)
    assert np.abs(got - np.roll(v1 * v2, -1)).max() < 1e-4
    h = o.hoisting(2, ct, [0, 1], glk)
    got = o.decode(2, o.decrypt(2, h, sk), s2, n // 2)
    p = v1 * v2
    assert np.abs(got - (np.roll(p, -1) + np.roll(p, -2))).max() < 1e-4


def test_samplers_shape_and_range():
    logn, n = 8, 256
    mods = coeff_modulus_create(n, [40, 40, 50])
    o = Oracle(logn, mods, 1)
    seed = np.arange(64, dtype=np.uint8)
    t = o.sample_small("ternary", seed, 2, 1)
    for r, q in enumerate(mods):
        assert set(np.unique(t[r])) <= {0, 1, q - 1}
    # every limb carries the same small polynomial
    signed = [np.where(t[r] > mods[r] // 2, t[r].astype(np.int64) - mods[r], t[r].astype(np.int64)) for r in range(3)]
    assert np.array_equal(signed[0], signed[1]) and np.array_equal(signed[0], signed[2])
    e = o.sample_small("error", seed, 2, 1)
    se = np.where(e[0] > mods[0] // 2, e[0].astype(np.int64) - mods[0], e[0].astype(np.int64))
    assert np.abs(se).max() <= 21 and 1.0 < se.std() < 5.0
    u = o.sample_uniform(seed, 2, 1)
    for r, q in enumerate(mods):
        assert int(u[r].max()) < q
    # the keyed block function: nonce changes the block, seed bytes 56..63 do not
    b0, b1 = o.prng_block(seed, 0), o.prng_block(seed, 1)
    assert not np.array_equal(b0, b1)
    seed2 = seed.copy()
    seed2[60] ^= 0xFF
    assert np.array_equal(o.prng_block(seed2, 0), b0)
