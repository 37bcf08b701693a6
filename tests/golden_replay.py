"""Replays the chain recorded in tests/golden/ref_fixture.json (outputs of the reference
library itself on a B200) and compares SHA-256 digests stage by stage."""
import hashlib
import json
import os

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))


def load_fixture():
    with open(os.path.join(HERE, "golden", "ref_fixture.json")) as f:
        return json.load(f)


def seeds_of(entry):
    w = np.array(entry["seed_words"], dtype=np.uint32)
    return w.view(np.uint8).reshape(-1, 64)


def digest(a):
    return hashlib.sha256(np.ascontiguousarray(a).tobytes()).hexdigest()


def message(n, salt):
    i = np.arange(n, dtype=np.uint64)
    x = ((i + np.uint64(salt)) * np.uint64(2654435761)) & np.uint64(0xFFFFFFFF)
    return x.astype(np.float64) / 2147483648.0 - 1.0


KRUM_BITS = [60, 40, 40, 60]
CASES = {
    "n4096_a1": dict(logn=12, size_p=1, steps=[1, 2, 3], bits=KRUM_BITS),
    "n8192_a1": dict(logn=13, size_p=1, steps=[1, 2, 3], bits=KRUM_BITS),
    "n4096_a2": dict(logn=12, size_p=2, steps=[1, 5], bits=[50, 40, 40, 40, 40, 40, 50, 50]),
    # the ring degrees and chains the benchmarks run: the two Krum configurations and the hybrid key-switching one
    # (24 data primes, 8 special primes); naf = a rotation step without a key of its own (5 = 1 + 4)
    "n32768_a1": dict(logn=15, size_p=1, steps=[1, 2, 4], bits=KRUM_BITS, naf=[1, 4]),
    "n65536_a1": dict(logn=16, size_p=1, steps=[1, 2, 4], bits=KRUM_BITS, naf=[1, 4]),
    "n65536_a8": dict(logn=16, size_p=8, steps=[1, 4], bits=[60] + [50] * 23 + [60] * 8, naf=[1, 4], scale=2.0 ** 50),
    # scale 2^50: the largest coefficients keep two or three bits below the rounding point, which pins the order of
    # the encoder's floating-point operations (2048 slots: the reference's single-kernel inverse FFT; 4096: one more stage kernel)
    "n4096_s50": dict(logn=12, size_p=1, steps=[1], bits=[60, 60, 60], scale=2.0 ** 50),
    "n8192_s50": dict(logn=13, size_p=1, steps=[1], bits=[60, 60, 60], scale=2.0 ** 50),
}
SCALE = 2.0 ** 40


def moduli_of(case, fix, create):
    """the case's primes from ``create(n, bits)``, checked against the digest the reference recorded"""
    cfg = CASES[case]
    mods = [int(m) for m in create(1 << cfg["logn"], cfg["bits"])]
    arr = np.array(mods, dtype=np.uint64)
    assert arr.nbytes == fix["moduli"]["bytes"] and digest(arr) == fix["moduli"]["sha256"], "moduli differ from the reference's"
    return mods


class Mismatch(AssertionError):
    pass


def check(fix, name, arr, report):
    want = fix[name]
    arr = np.ascontiguousarray(arr)
    ok = arr.nbytes == want["bytes"] and digest(arr) == want["sha256"]
    report.append((name, ok))
    return ok


def replay(case, fix, ops, keep=None):
    """ops: an object with the oracle's method names (the oracle itself, or an adapter that
    runs the CUDA library).  Returns the list of (stage, ok); ``keep`` (a dict) receives the
    public key, first plaintext, first ciphertext and the rescaled product."""
    cfg = CASES[case]
    report = []
    size_QP = fix["moduli"]["bytes"] // 8
    size_p = cfg["size_p"]
    size_Q = size_QP - size_p
    dnum = size_Q // size_p
    n = 1 << cfg["logn"]
    L = size_Q
    scale = cfg.get("scale", SCALE)

    sk = ops.gen_sk(seeds_of(fix["seed_sk"])[0])
    check(fix, "sk", sk, report)
    s = seeds_of(fix["seed_pk"])
    pk = ops.gen_pk(sk, s[0], s[1])
    check(fix, "pk", pk, report)
    s = seeds_of(fix["seed_rlk"])
    rlk = ops.gen_ksk(sk, ops.sk_square(sk), s.reshape(-1))
    for j in range(dnum):
        check(fix, "rlk%d" % j, rlk[j], report)
    s = seeds_of(fix["seed_glk"])
    n_elts = len(cfg["steps"])
    glk = []
    for e in range(n_elts):
        g = ops.gen_ksk(sk, ops.galois(e, sk), s[e * 2 * dnum:(e + 1) * 2 * dnum].reshape(-1))
        glk.append(g)
        for j in range(dnum):
            check(fix, "glk%d_%d" % (e, j), g[j], report)

    m1, m2 = message(n // 2, 1), message(n // 2, 77)
    pt1, pt2 = ops.encode(L, m1, scale), ops.encode(L, m2, scale)
    check(fix, "pt1", pt1, report)
    check(fix, "pt2", pt2, report)
    s = seeds_of(fix["seed_enc"])
    ct1 = ops.encrypt_asym(pk, pt1, s[0], s[1])
    ct2 = ops.encrypt_asym(pk, pt2, s[2], s[3])
    check(fix, "ct1", ct1, report)
    check(fix, "ct2", ct2, report)
    diff = ops.poly_op("sub", L, ct2, ct1)
    check(fix, "sub", diff, report)
    prod = ops.tensor(L, ct1, ct2)
    check(fix, "mul", prod, report)
    check(fix, "square", ops.square(L, diff.reshape(2, L, n)), report)
    rel = ops.relinearize(L, prod, rlk)
    check(fix, "relin", rel, report)
    res = ops.rescale(L, rel)
    check(fix, "rescale", res, report)
    if keep is not None:
        keep.update(pk=pk, pt1=pt1, ct1=ct1, rescaled=res, size_QP=size_QP, size_Q=size_Q, n=n, rlk=rlk, glk=glk, scale=scale)
    L2 = L - 1
    check(fix, "rotate", ops.rotate(L2, res, 0, glk[0]), report)
    if cfg.get("naf"):
        # rotate_internal applies the non-adjacent-form terms least significant first
        # (cahel-main/include/util/numth.h:18-35, src/evaluate.cu:2396-2407)
        r = res
        for step in cfg["naf"]:
            e = cfg["steps"].index(step)
            r = ops.rotate(L2, r, e, glk[e])
        check(fix, "rotate_naf", r, report)
    hoist = ops.hoisting(L2, res, list(range(n_elts)), glk)
    check(fix, "hoisting", hoist, report)
    if L2 >= 2:
        low = ops.drop_last(L2, res)
        check(fix, "drop", low, report)
        check(fix, "rotate_low", ops.rotate(L2 - 1, low, 0, glk[0]), report)
    dec = ops.decrypt(L2, hoist, sk)
    check(fix, "decrypt", dec, report)
    out = ops.decode(L2, dec, scale, n // 2)
    # decode is floating point: compare values, not digests
    want_head = np.array(fix["decode"]["head"], dtype=np.float64)
    got_head = np.asarray(out).view(np.float64)[:8]
    report.append(("decode_head", bool(np.allclose(got_head, want_head, rtol=1e-9, atol=1e-9))))
    return report
