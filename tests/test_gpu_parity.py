"""Parity of the CUDA path (through the C ABI) against the CPU oracle: bit-exact on the
same seeded inputs.  Needs a B200; run with -m gpu."""
import numpy as np
import pytest

from gpu_util import rand_rows, row_moduli, seeds

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def torch_cuda():
    import torch

    if not torch.cuda.is_available():
        pytest.fail("GPU tests need a CUDA device; there is no CPU fallback")
    return torch


def make(logn, bits, size_p, steps=()):
    from lancelot_b200 import cabi
    from oracle import binding

    n = 1 << logn
    mods = binding.coeff_modulus_create(n, bits)
    elts = binding.elts_from_steps(list(steps), n)
    return binding.Oracle(logn, mods, size_p, elts), cabi.Context(logn, mods, size_p, elts), mods


@pytest.mark.parametrize("logn", [4, 5, 7, 10, 12, 13, 14, 15, 16])
def test_ntt_matches_oracle(torch_cuda, logn):
    from lancelot_b200 import cabi

    o, ctx, mods = make(logn, [60, 40, 50, 60], 1)
    rng = np.random.default_rng(logn)
    groups = 3 if logn <= 13 else 2
    data = rand_rows(rng, row_moduli(mods, 3, 3, 1, groups), 1 << logn)
    d = cabi.to_device(data)
    ctx.ntt_forward(d, groups, 3, 1)
    want = o.ntt_rows(data, groups, 3, 1)
    got = cabi.to_host(d)
    assert np.array_equal(got, want)
    ctx.ntt_inverse(d, groups, 3, 1)
    assert np.array_equal(cabi.to_host(d), data)
    # inverse alone, from the oracle's forward output
    d2 = cabi.to_device(want)
    ctx.ntt_inverse(d2, groups, 3, 1)
    assert np.array_equal(cabi.to_host(d2), data)


def test_ntt_edge_values(torch_cuda):
    """all-zero, all q-1 and a single one: the extremes of the lazy-reduction ranges"""
    from lancelot_b200 import cabi

    logn = 13
    o, ctx, mods = make(logn, [60, 40, 60], 1)
    n = 1 << logn
    rows = []
    for q in [mods[0], mods[1], mods[2]]:
        rows += [np.zeros(n, np.uint64), np.full(n, q - 1, np.uint64)]
    # layout: groups of (2 data + 1 special); build 2 groups: zeros and q-1
    data = np.stack([np.zeros(n, np.uint64)] * 3 + [np.full(n, mods[0] - 1, np.uint64), np.full(n, mods[1] - 1, np.uint64),
                                                    np.full(n, mods[2] - 1, np.uint64)])
    d = cabi.to_device(data)
    ctx.ntt_forward(d, 2, 2, 1)
    assert np.array_equal(cabi.to_host(d), o.ntt_rows(data, 2, 2, 1))
    ctx.ntt_inverse(d, 2, 2, 1)
    assert np.array_equal(cabi.to_host(d), data)


@pytest.mark.parametrize("logn", [11, 13, 16])
def test_ntt_every_butterfly_variant(torch_cuda, logn):
    """primes on both sides of the size limits that select the butterfly variant (2^58, 2^50, 2^46),
    on random residues and on the extremes 0 and q-1"""
    from lancelot_b200 import cabi

    bits = [60, 59, 58, 57, 51, 50, 49, 47, 46, 45, 40, 30]
    o, ctx, mods = make(logn, bits, 0)
    n, L = 1 << logn, len(bits)
    rng = np.random.default_rng(100 + logn)
    rand = rand_rows(rng, row_moduli(mods, L, L, 0, 1), n)
    top = np.stack([np.full(n, q - 1, np.uint64) for q in mods])
    data = np.concatenate([rand, top, np.zeros_like(top)])
    d = cabi.to_device(data)
    ctx.ntt_forward(d, 3, L, 0)
    want = o.ntt_rows(data, 3, L, 0)
    assert np.array_equal(cabi.to_host(d), want)
    ctx.ntt_inverse(d, 3, L, 0)
    assert np.array_equal(cabi.to_host(d), data)


def test_ntt_special_limbs_only_and_empty(torch_cuda):
    from lancelot_b200 import cabi

    logn = 12
    o, ctx, mods = make(logn, [50, 40, 40, 50, 50], 2)
    rng = np.random.default_rng(5)
    data = rand_rows(rng, row_moduli(mods, 3, 0, 2, 2), 1 << logn)
    d = cabi.to_device(data)
    ctx.ntt_forward(d, 2, 0, 2)
    assert np.array_equal(cabi.to_host(d), o.ntt_rows(data, 2, 0, 2))
    ctx.ntt_forward(d, 0, 0, 2)  # empty batch is a no-op
    assert np.array_equal(cabi.to_host(d), o.ntt_rows(data, 2, 0, 2))


@pytest.mark.parametrize("logn", [10, 13])
def test_elementwise_and_tensor(torch_cuda, logn):
    from lancelot_b200 import cabi

    o, ctx, mods = make(logn, [60, 40, 40, 60], 1)
    rng = np.random.default_rng(7)
    n = 1 << logn
    a = rand_rows(rng, row_moduli(mods, 3, 3, 0, 2), n)
    b = rand_rows(rng, row_moduli(mods, 3, 3, 0, 2), n)
    da, db = cabi.to_device(a), cabi.to_device(b)
    assert np.array_equal(cabi.to_host(ctx.add(3, da, db)), o.poly_op("add", 3, a, b))
    assert np.array_equal(cabi.to_host(ctx.sub(3, da, db)), o.poly_op("sub", 3, a, b))
    assert np.array_equal(cabi.to_host(ctx.multiply_poly(3, da, db)), o.poly_op("mul", 3, a, b))
    assert np.array_equal(cabi.to_host(ctx.negate(3, da)), o.poly_op("neg", 3, a))
    assert np.array_equal(cabi.to_host(ctx.multiply(3, da, db)).reshape(3, 3, n), o.tensor(3, a.reshape(2, 3, n), b.reshape(2, 3, n)))
    assert np.array_equal(cabi.to_host(ctx.square(3, da)).reshape(3, 3, n), o.square(3, a.reshape(2, 3, n)))
    # in place
    ctx.add(3, da, db, out=da)
    assert np.array_equal(cabi.to_host(da), o.poly_op("add", 3, a, b))
    # level drop
    assert np.array_equal(cabi.to_host(ctx.mod_switch_drop(3, db)).reshape(2, 2, n), o.drop_last(3, b))


def _keys(o, rng, n_elts):
    sk = o.gen_sk(seeds(rng, 1))
    dnum = o.size_Q // o.size_P
    rlk = o.gen_ksk(sk, o.sk_square(sk), seeds(rng, 2 * dnum))
    glk = [o.gen_ksk(sk, o.galois(i, sk), seeds(rng, 2 * dnum)) for i in range(n_elts)]
    return sk, rlk, glk


CASES = [
    # logn, bits, size_P, levels to test
    (10, [60, 40, 40, 60], 1, [3, 2]),
    (13, [60, 40, 40, 60], 1, [3, 2]),
    (11, [50, 40, 40, 40, 40, 40, 50, 50], 2, [6, 5, 3]),
    (12, [50] + [40] * 8 + [50, 50, 50], 3, [9, 7]),
    (14, [60, 40, 40, 60], 1, [3]),
]


@pytest.mark.parametrize("logn,bits,size_p,levels", CASES)
def test_keyswitch_pieces_and_whole(torch_cuda, logn, bits, size_p, levels):
    from lancelot_b200 import cabi

    steps = [1, 2, 3]
    o, ctx, mods = make(logn, bits, size_p, steps)
    rng = np.random.default_rng(100 + logn)
    n = 1 << logn
    size_Q = len(bits) - size_p
    sk, rlk, glk = _keys(o, rng, len(steps))
    d_rlk = cabi.to_device(rlk)
    d_glk = [cabi.to_device(g) for g in glk]
    for L in levels:
        cks = rand_rows(rng, row_moduli(mods, size_Q, L, 0), n)
        dig = o.modup(L, cks)
        got_dig = cabi.to_host(ctx.modup(L, cabi.to_device(cks)))
        assert np.array_equal(got_dig, dig), "modup L=%d" % L
        cx = o.inner_product(L, dig, rlk)
        got_cx = cabi.to_host(ctx.inner_product(L, cabi.to_device(dig), d_rlk))
        assert np.array_equal(got_cx, cx), "inner product L=%d" % L
        md = o.moddown(L, cx[0])
        assert np.array_equal(cabi.to_host(ctx.moddown(L, cabi.to_device(cx[0]))), md), "moddown L=%d" % L
        ct = rand_rows(rng, row_moduli(mods, size_Q, L, 0, 2), n).reshape(2, L, n)
        want = o.keyswitch(L, ct, cks, rlk)
        got = cabi.to_host(ctx.keyswitch(L, cabi.to_device(ct), cabi.to_device(cks), d_rlk))
        assert np.array_equal(got, want), "keyswitch L=%d" % L
        ct3 = rand_rows(rng, row_moduli(mods, size_Q, L, 0, 3), n).reshape(3, L, n)
        assert np.array_equal(cabi.to_host(ctx.relinearize(L, cabi.to_device(ct3), d_rlk)), o.relinearize(L, ct3, rlk))
        if L >= 2:
            assert np.array_equal(cabi.to_host(ctx.rescale(L, cabi.to_device(ct3))), o.rescale(L, ct3)), "rescale L=%d" % L
        for e in range(2):
            assert np.array_equal(cabi.to_host(ctx.galois_permute(e, cabi.to_device(ct))), o.galois(e, ct))
            want = o.rotate(L, ct, e, glk[e])
            got = cabi.to_host(ctx.rotate(L, cabi.to_device(ct), e, d_glk[e]))
            assert np.array_equal(got, want), "rotate L=%d elt=%d" % (L, e)
        want = o.hoisting(L, ct, [0, 1, 2], glk)
        got = cabi.to_host(ctx.hoisting(L, cabi.to_device(ct), [0, 1, 2], d_glk))
        assert np.array_equal(got, want), "hoisting L=%d" % L
        # decryption of a size-2 and a size-3 ciphertext
        d_sk = cabi.to_device(sk)
        assert np.array_equal(cabi.to_host(ctx.decrypt(L, cabi.to_device(ct), d_sk)), o.decrypt(L, ct, sk))
        assert np.array_equal(cabi.to_host(ctx.decrypt(L, cabi.to_device(ct3), d_sk)), o.decrypt(L, ct3, sk))


@pytest.mark.parametrize("n_chunks", [1, 5, 70])
def test_krum_accumulate(torch_cuda, n_chunks):
    from lancelot_b200 import cabi

    logn, L = 10, 3
    o, ctx, mods = make(logn, [60, 40, 40, 60], 1)
    rng = np.random.default_rng(n_chunks)
    n = 1 << logn
    a = rand_rows(rng, row_moduli(mods, 3, L, 0, 2 * n_chunks), n).reshape(n_chunks, 2, L, n)
    b = rand_rows(rng, row_moduli(mods, 3, L, 0, 2 * n_chunks), n).reshape(n_chunks, 2, L, n)
    want = np.zeros((3, L, n), dtype=np.uint64)
    for c in range(n_chunks):
        want = o.poly_op("add", L, want, o.square(L, o.poly_op("sub", L, b[c], a[c]).reshape(2, L, n)))
    acc = ctx.empty(3, L, n)
    ctx.krum_accumulate(L, cabi.to_device(a), cabi.to_device(b), acc, accumulate=False)
    assert np.array_equal(cabi.to_host(acc), want)
    # accumulate on top of a previous value
    ctx.krum_accumulate(L, cabi.to_device(a), cabi.to_device(b), acc, accumulate=True)
    assert np.array_equal(cabi.to_host(acc), o.poly_op("add", L, want, want))


@pytest.mark.parametrize("n_a,n_b,n_chunks", [(2, 0, 3), (3, 0, 1), (4, 0, 70), (1, 1, 5), (1, 4, 2), (2, 1, 130), (2, 3, 4), (2, 4, 66)])
def test_krum_accumulate_tile(torch_cuda, n_a, n_b, n_chunks):
    """every pair sum of a tile equals the per-chunk sub / square / add sequence of the oracle"""
    from lancelot_b200 import cabi

    logn, L = 10, 3
    o, ctx, mods = make(logn, [60, 40, 40, 60], 1)
    rng = np.random.default_rng(1000 * n_a + 100 * n_b + n_chunks)
    n = 1 << logn
    host = [rand_rows(rng, row_moduli(mods, 3, L, 0, 2 * n_chunks), n).reshape(n_chunks, 2, L, n) for _ in range(n_a + n_b)]
    dev = [cabi.to_device(h) for h in host]
    if n_b:
        pairs = [(i, n_a + j) for i in range(n_a) for j in range(n_b)]
    else:
        pairs = [(i, j) for i in range(n_a) for j in range(i + 1, n_a)]
    outs = [ctx.empty(3, L, n) for _ in pairs]
    ctx.krum_accumulate_tile(L, dev[:n_a], dev[n_a:], outs)
    for (i, j), got in zip(pairs, outs):
        want = np.zeros((3, L, n), dtype=np.uint64)
        for c in range(n_chunks):
            want = o.poly_op("add", L, want, o.square(L, o.poly_op("sub", L, host[j][c], host[i][c]).reshape(2, L, n)))
        assert np.array_equal(cabi.to_host(got), want)


def test_krum_tile_shape_errors(torch_cuda):
    from lancelot_b200 import cabi
    from lancelot_b200._lib import InvalidArgument

    o, ctx, mods = make(10, [60, 40, 40, 60], 1)
    t = [ctx.empty(1, 2, 3, 1 << 10) for _ in range(5)]
    outs = [ctx.empty(3, 3, 1 << 10) for _ in range(10)]
    with pytest.raises(InvalidArgument):
        ctx.krum_accumulate_tile(3, t[:5], [], outs[:10])  # triangle of five
    with pytest.raises(InvalidArgument):
        ctx.krum_accumulate_tile(3, t[:3], t[3:5], outs[:6])  # three rows


def test_sum_groups_equals_repeated_add(torch_cuda):
    from lancelot_b200 import cabi
    from lancelot_b200._lib import InvalidArgument

    logn, L = 10, 2
    o, ctx, mods = make(logn, [60, 40, 40, 60], 1)
    rng = np.random.default_rng(9)
    n = 1 << logn
    items = rand_rows(rng, row_moduli(mods, 3, L, 0, 2 * 7), n).reshape(7, 2, L, n)
    groups = [[0, 3, 6], [], [5], [1, 2, 3, 4, 5, 6, 0]]
    got = cabi.to_host(ctx.sum_groups(L, 2, cabi.to_device(items), groups))
    for g, idx in enumerate(groups):
        want = np.zeros((2, L, n), dtype=np.uint64)
        for i in idx:
            want = o.poly_op("add", L, want, items[i])
        assert np.array_equal(got[g].reshape(-1), np.asarray(want).reshape(-1))
    with pytest.raises(InvalidArgument):
        ctx.sum_groups(L, 2, cabi.to_device(items), [[7]])


def test_error_reporting_on_gpu(torch_cuda):
    from lancelot_b200 import cabi
    from lancelot_b200._lib import InvalidArgument, LancelotError

    o, ctx, mods = make(10, [60, 40, 40, 60], 1, [1])
    n = 1 << 10
    ct = ctx.empty(2, 3, n)
    with pytest.raises(InvalidArgument):
        ctx.rescale(1, ct)  # no next level
    with pytest.raises(LancelotError):
        ctx.galois_permute(5, ct)  # no such Galois key
    with pytest.raises(InvalidArgument):
        ctx.ntt_forward(ct, 1, 7, 0)  # more limbs than the context has


@pytest.mark.parametrize("logn,bits,size_p", [(8, [40, 40, 50], 1), (12, [60, 40, 40, 60], 1), (11, [50, 40, 40, 40, 50, 50], 2)])
def test_samplers_and_keys(torch_cuda, logn, bits, size_p):
    from lancelot_b200 import cabi

    o, ctx, mods = make(logn, bits, size_p, [1, 2])
    rng = np.random.default_rng(17 + logn)
    size_Q = len(bits) - size_p
    s = seeds(rng, 1)
    for kind in ["ternary", "error"]:
        assert np.array_equal(cabi.to_host(ctx.sample(kind, s, size_Q, size_p)), o.sample_small(kind, s, size_Q, size_p)), kind
    assert np.array_equal(cabi.to_host(ctx.sample("uniform", s, size_Q, size_p)), o.sample_uniform(s, size_Q, size_p))
    sk = o.gen_sk(s)
    d_sk = ctx.gen_secret_key(s)
    assert np.array_equal(cabi.to_host(d_sk), sk)
    se, sa = seeds(rng, 1), seeds(rng, 1)
    pk = o.gen_pk(sk, se, sa)
    d_pk = ctx.gen_public_key(d_sk, se, sa)
    assert np.array_equal(cabi.to_host(d_pk), pk)
    dnum = size_Q // size_p
    ss = seeds(rng, 2 * dnum)
    sk2 = o.sk_square(sk)
    assert np.array_equal(cabi.to_host(ctx.multiply_poly_qp(d_sk, d_sk)), sk2)
    rlk = o.gen_ksk(sk, sk2, ss)
    assert np.array_equal(cabi.to_host(ctx.gen_switch_key(d_sk, cabi.to_device(sk2), ss)), rlk)
    skp = o.galois(1, sk)
    assert np.array_equal(cabi.to_host(ctx.galois_permute(1, d_sk)), skp)
    glk = o.gen_ksk(sk, skp, ss)
    assert np.array_equal(cabi.to_host(ctx.gen_switch_key(d_sk, cabi.to_device(skp), ss)), glk)
    # batched public-key encryption, with and without a plaintext
    batch = 3
    es = seeds(rng, 2 * batch)
    n = 1 << logn
    pts = rand_rows(rng, row_moduli(mods, size_Q, size_Q, 0, batch), n).reshape(batch, size_Q, n)
    got = cabi.to_host(ctx.encrypt_asymmetric(d_pk, cabi.to_device(pts), es, batch)).reshape(batch, 2, size_Q, n)
    got0 = cabi.to_host(ctx.encrypt_asymmetric(d_pk, None, es, batch)).reshape(batch, 2, size_Q, n)
    for b in range(batch):
        su, se_ = es[128 * b:128 * b + 64], es[128 * b + 64:128 * b + 128]
        assert np.array_equal(got0[b], o.encrypt_zero_asym(pk, su, se_)), "encrypt zero %d" % b
        assert np.array_equal(got[b], o.encrypt_asym(pk, pts[b], su, se_)), "encrypt %d" % b


@pytest.mark.parametrize("logn,slots", [(5, 16), (10, 512), (12, 2048), (13, 4096), (14, 8192), (15, 16384), (16, 32768), (13, 64)])
def test_encode_decode(torch_cuda, logn, slots):
    import torch
    from lancelot_b200 import cabi

    o, ctx, mods = make(logn, [60, 40, 40, 60], 1)
    rng = np.random.default_rng(logn * 100 + slots)
    scale = 2.0 ** 40
    batch = 2
    vals = rng.uniform(-1, 1, (batch, slots))
    vals[0, : min(8, slots)] = [0.0, -0.0, 1.0, -1.0, 0.5, -0.5, 1e-13, -1e-13][: min(8, slots)]
    d = torch.from_numpy(vals).cuda()
    pt = ctx.encode(3, d, scale, sparse_slots=slots, batch=batch)
    ctx.check_status()
    got = cabi.to_host(pt).reshape(batch, 3, 1 << logn)
    for b in range(batch):
        want = o.encode(3, vals[b], scale, sparse_slots=slots)
        assert np.array_equal(got[b], want), "encode message %d" % b
    # float32 input is widened exactly
    v32 = vals.astype(np.float32)
    pt32 = ctx.encode(3, torch.from_numpy(v32).cuda(), scale, sparse_slots=slots, batch=batch)
    assert np.array_equal(cabi.to_host(pt32).reshape(batch, 3, -1)[1], o.encode(3, v32[1].astype(np.float64), scale, sparse_slots=slots))
    # complex input and short messages (zero padded)
    cv = (rng.uniform(-1, 1, slots) + 1j * rng.uniform(-1, 1, slots))[: max(1, slots - 3)]
    ptc = ctx.encode(3, torch.from_numpy(cv).cuda(), scale, sparse_slots=slots)
    assert np.array_equal(cabi.to_host(ptc), o.encode(3, cv, scale, sparse_slots=slots))
    # decode: floating point, tolerance of the reference's own round-trip tests (1e-5, cahel-main/unittest/evaluator.cu)
    dec = ctx.decode(3, pt[1].contiguous(), scale, slots).cpu().numpy()
    assert np.abs(dec - vals[1]).max() < 1e-7
    want = o.decode(3, got[1], scale, slots)
    assert np.abs(dec - want).max() < 1e-9
    # two-limb plaintext after a level drop decodes too
    dec2 = ctx.decode(2, pt[1, :2].contiguous(), scale, slots).cpu().numpy()
    assert np.abs(dec2 - vals[1]).max() < 1e-7


def test_encode_rejects_values_that_do_not_fit(torch_cuda):
    import torch
    from lancelot_b200._lib import InvalidArgument

    o, ctx, mods = make(10, [30, 30], 1)
    big = torch.full((512,), 1e9, dtype=torch.float64, device="cuda")
    ctx.encode(1, big, 2.0 ** 25, sparse_slots=512)
    with pytest.raises(InvalidArgument):
        ctx.check_status()
    ctx.check_status()  # the flag is cleared once reported
    with pytest.raises(InvalidArgument):
        ctx.encode(1, big, 2.0 ** 40, sparse_slots=512)  # scale out of bounds


@pytest.mark.parametrize("logn,bits,size_p,L", [(10, [60, 40, 40, 60], 1, 2), (11, [50, 40, 40, 40, 40, 40, 50, 50], 2, 5)])
def test_batched_keyswitch_matches_per_ciphertext(torch_cuda, logn, bits, size_p, L):
    from lancelot_b200 import cabi

    steps = [1, 2, 3]
    o, ctx, mods = make(logn, bits, size_p, steps)
    rng = np.random.default_rng(500 + logn)
    n = 1 << logn
    size_Q = len(bits) - size_p
    sk, rlk, glk = _keys(o, rng, len(steps))
    d_rlk = cabi.to_device(rlk)
    d_glk = [cabi.to_device(g) for g in glk]
    batch = 5
    ct3 = rand_rows(rng, row_moduli(mods, size_Q, L, 0, 3 * batch), n).reshape(batch, 3, L, n)
    got = cabi.to_host(ctx.relinearize_batch(L, cabi.to_device(ct3), d_rlk)).reshape(batch, 3, L, n)
    for b in range(batch):
        assert np.array_equal(got[b, :2], o.relinearize(L, ct3[b], rlk)), "relinearize %d" % b
    ct = rand_rows(rng, row_moduli(mods, size_Q, L, 0, 2 * batch), n).reshape(batch, 2, L, n)
    got = cabi.to_host(ctx.rotate_batch(L, cabi.to_device(ct), 1, d_glk[1])).reshape(batch, 2, L, n)
    for b in range(batch):
        assert np.array_equal(got[b], o.rotate(L, ct[b], 1, glk[1])), "rotate %d" % b
    got = cabi.to_host(ctx.hoisting_batch(L, cabi.to_device(ct), [0, 1, 2], d_glk)).reshape(batch, 2, L, n)
    for b in range(batch):
        assert np.array_equal(got[b], o.hoisting(L, ct[b], [0, 1, 2], glk)), "hoisting %d" % b
    # rescale already takes any number of polynomials
    got = cabi.to_host(ctx.rescale(L, cabi.to_device(ct))).reshape(batch, 2, L - 1, n)
    for b in range(batch):
        assert np.array_equal(got[b], o.rescale(L, ct[b]))


@pytest.mark.parametrize("logn,slots", [(12, 2048), (15, 16384), (13, 256)])
def test_fused_encode_encrypt_equals_two_calls(torch_cuda, logn, slots):
    import torch
    from lancelot_b200 import cabi

    o, ctx, mods = make(logn, [60, 40, 40, 60], 1)
    rng = np.random.default_rng(31 + logn)
    batch = 3
    vals = torch.from_numpy(rng.normal(0, 0.01, (batch, slots)).astype(np.float32)).cuda()
    s = seeds(rng, 1)
    sk = ctx.gen_secret_key(s)
    pk = ctx.gen_public_key(sk, seeds(rng, 1), seeds(rng, 1))
    es = seeds(rng, 2 * batch)
    scale = 2.0 ** 40
    pts = ctx.encode(3, vals, scale, sparse_slots=slots, batch=batch)
    two = cabi.to_host(ctx.encrypt_asymmetric(pk, pts, es, batch))
    one = cabi.to_host(ctx.encode_encrypt(pk, vals, scale, es, slots, batch))
    assert np.array_equal(one.reshape(-1), two.reshape(-1))
