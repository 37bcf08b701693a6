"""Bit-exact parity of the CUDA path against the CPU oracle at the sizes the benchmarks run:
N = 2^15 and 2^16 with Lancelot's chain {60,40,40 | 60}, and N = 2^16 with 24 data primes and eight
special primes (alpha = 8, dnum = 3).  These ring degrees take other code paths than the small cases
(clusters of 4 and 8 CTAs per limb, the fixed-schedule transforms and their fused loaders), so the
small-ring digests do not cover them.  Needs a B200; run with -m gpu."""
import numpy as np
import pytest

from gpu_util import rand_rows, row_moduli, seeds

pytestmark = pytest.mark.gpu

KRUM_BITS = [60, 40, 40, 60]
WIDE_BITS = [60] + [50] * 23 + [60] * 8


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


def _keys(o, rng, n_elts):
    sk = o.gen_sk(seeds(rng, 1))
    dnum = o.size_Q // o.size_P
    rlk = o.gen_ksk(sk, o.sk_square(sk), seeds(rng, 2 * dnum))
    glk = [o.gen_ksk(sk, o.galois(i, sk), seeds(rng, 2 * dnum)) for i in range(n_elts)]
    return sk, rlk, glk


@pytest.mark.parametrize("logn,bits,size_p,levels", [
    (15, KRUM_BITS, 1, [3, 2]),
    (16, KRUM_BITS, 1, [3, 2]),
    (16, WIDE_BITS, 8, [24, 23]),  # 23 limbs: the last digit is partial (8 + 8 + 7)
])
def test_keyswitch_chain_at_bench_sizes(torch_cuda, logn, bits, size_p, levels):
    """mod-up, inner product, mod-down, key switch, relinearize, rescale, rotate, hoisting, decrypt"""
    from lancelot_b200 import cabi

    steps = [1, 4]
    o, ctx, mods = make(logn, bits, size_p, steps)
    rng = np.random.default_rng(900 + logn + size_p)
    n = 1 << logn
    size_Q = len(bits) - size_p
    sk, rlk, glk = _keys(o, rng, len(steps))
    # generated keys first: the key generators run their own transforms at the key level
    d_sk = ctx.gen_secret_key(seeds(np.random.default_rng(900 + logn + size_p), 1))
    assert np.array_equal(cabi.to_host(d_sk), sk), "secret key"
    d_rlk = cabi.to_device(rlk)
    d_glk = [cabi.to_device(g) for g in glk]
    for L in levels:
        cks = rand_rows(rng, row_moduli(mods, size_Q, L, 0), n)
        dig = o.modup(L, cks)
        assert np.array_equal(cabi.to_host(ctx.modup(L, cabi.to_device(cks))), dig), "modup L=%d" % L
        cx = o.inner_product(L, dig, rlk)
        assert np.array_equal(cabi.to_host(ctx.inner_product(L, cabi.to_device(dig), d_rlk)), cx), "inner product L=%d" % L
        del dig
        assert np.array_equal(cabi.to_host(ctx.moddown(L, cabi.to_device(cx[0]))), o.moddown(L, cx[0])), "moddown L=%d" % L
        ct = rand_rows(rng, row_moduli(mods, size_Q, L, 0, 2), n).reshape(2, L, n)
        ct3 = rand_rows(rng, row_moduli(mods, size_Q, L, 0, 3), n).reshape(3, L, n)
        assert np.array_equal(cabi.to_host(ctx.relinearize(L, cabi.to_device(ct3), d_rlk)), o.relinearize(L, ct3, rlk)), "relinearize L=%d" % L
        assert np.array_equal(cabi.to_host(ctx.rescale(L, cabi.to_device(ct3))), o.rescale(L, ct3)), "rescale L=%d" % L
        for e in range(2):
            got = cabi.to_host(ctx.rotate(L, cabi.to_device(ct), e, d_glk[e]))
            assert np.array_equal(got, o.rotate(L, ct, e, glk[e])), "rotate L=%d elt=%d" % (L, e)
        got = cabi.to_host(ctx.hoisting(L, cabi.to_device(ct), [0, 1], d_glk))
        assert np.array_equal(got, o.hoisting(L, ct, [0, 1], glk)), "hoisting L=%d" % L
        assert np.array_equal(cabi.to_host(ctx.decrypt(L, cabi.to_device(ct3), d_sk)), o.decrypt(L, ct3, sk)), "decrypt L=%d" % L


@pytest.mark.parametrize("logn,bits,size_p", [(15, KRUM_BITS, 1), (16, KRUM_BITS, 1), (16, WIDE_BITS, 8)])
def test_keys_and_encryption_at_bench_sizes(torch_cuda, logn, bits, size_p):
    """public key, switch key, plain and fused public-key encryption"""
    import torch
    from lancelot_b200 import cabi

    o, ctx, mods = make(logn, bits, size_p, [1])
    rng = np.random.default_rng(70 + logn + size_p)
    n = 1 << logn
    size_Q = len(bits) - size_p
    dnum = size_Q // size_p
    s = seeds(rng, 1)
    sk = o.gen_sk(s)
    d_sk = ctx.gen_secret_key(s)
    se, sa = seeds(rng, 1), seeds(rng, 1)
    pk = o.gen_pk(sk, se, sa)
    d_pk = ctx.gen_public_key(d_sk, se, sa)
    assert np.array_equal(cabi.to_host(d_pk), pk), "public key"
    ss = seeds(rng, 2 * dnum)
    skp = o.galois(0, sk)
    assert np.array_equal(cabi.to_host(ctx.gen_switch_key(d_sk, cabi.to_device(skp), ss)), o.gen_ksk(sk, skp, ss)), "switch key"
    batch = 2
    es = seeds(rng, 2 * batch)
    slots = n // 2
    scale = 2.0 ** (40 if size_p == 1 else 50)
    vals = rng.normal(0, 0.01, (batch, slots)).astype(np.float32)
    d_vals = torch.from_numpy(vals).cuda()
    pts = ctx.encode(size_Q, d_vals, scale, sparse_slots=slots, batch=batch)
    ctx.check_status()
    h_pts = cabi.to_host(pts).reshape(batch, size_Q, n)
    got = cabi.to_host(ctx.encrypt_asymmetric(d_pk, pts, es, batch)).reshape(batch, 2, size_Q, n)
    for b in range(batch):
        want_pt = o.encode(size_Q, vals[b].astype(np.float64), scale, sparse_slots=slots)
        assert np.array_equal(h_pts[b], want_pt), "encode %d" % b
        want = o.encrypt_asym(pk, want_pt, es[128 * b:128 * b + 64], es[128 * b + 64:128 * b + 128])
        assert np.array_equal(got[b], want), "encrypt %d" % b
    # the fused encode + encrypt entry the Krum driver uses
    fused = cabi.to_host(ctx.encode_encrypt(d_pk, d_vals, scale, es, slots, batch)).reshape(batch, 2, size_Q, n)
    assert np.array_equal(fused, got), "fused encode + encrypt"


@pytest.mark.parametrize("logn,n_a,n_b,n_chunks", [(16, 2, 4, 342), (16, 4, 0, 342), (15, 2, 4, 342), (10, 2, 2, 2100), (10, 3, 0, 2100),
                                                   (10, 1, 3, 2049), (5, 2, 4, 9)])
def test_pair_tile_at_bench_sizes(torch_cuda, logn, n_a, n_b, n_chunks):
    """Long tiles against the oracle's per-chunk sub / square / add: 342 chunks at the rings of the benchmark rounds
    (past five in-place reductions of the integer path), more than 2048 chunks (past one window of the FP64 path the
    40-bit limbs take), and a ring shorter than a CTA.  The device holds the full clients; their chunks repeat with
    period 7 so that the host needs only seven chunks per client."""
    import torch
    from lancelot_b200 import cabi

    L, period = 3, 7
    o, ctx, mods = make(logn, KRUM_BITS, 1)
    rng = np.random.default_rng(logn * 100 + n_a * 10 + n_b)
    n = 1 << logn
    host = []
    for k in range(n_a + n_b):
        h = rand_rows(rng, row_moduli(mods, 3, L, 0, 2 * period), n).reshape(period, 2, L, n)
        if k == 0:
            h[0] = 0  # extremes of the unreduced difference range
        if k == (n_a if n_b else 1):
            for r in range(L):
                h[0][:, r, :] = mods[r] - 1
        host.append(h)
    reps = (n_chunks + period - 1) // period
    dev = [cabi.to_device(h).repeat(reps, 1, 1, 1)[:n_chunks].contiguous() for h in host]
    if n_b:
        pairs = [(i, n_a + j) for i in range(n_a) for j in range(n_b)]
    else:
        pairs = [(i, j) for i in range(n_a) for j in range(i + 1, n_a)]
    outs = [ctx.empty(3, L, n) for _ in pairs]
    ctx.krum_accumulate_tile(L, dev[:n_a], dev[n_a:], outs)
    torch.cuda.synchronize()
    for (i, j), got in zip(pairs, outs):
        sq = [o.square(L, o.poly_op("sub", L, host[j][c], host[i][c]).reshape(2, L, n)) for c in range(period)]
        want = np.zeros((3, L, n), dtype=np.uint64)
        for c in range(n_chunks):
            want = o.poly_op("add", L, want, sq[c % period])
        assert np.array_equal(cabi.to_host(got), want), "pair (%d, %d)" % (i, j)
