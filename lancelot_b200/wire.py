"""Byte streams of ciphertexts, plaintexts and public keys in the reference library's own format,
so that a client and a server may run different implementations.

Layouts (little endian, no padding; cahel-main/include/ciphertext.h:174-292, plaintext.h:109-213,
secretkey.h:54-60):

    ciphertext / public key:  parms_id[32] | is_ntt_form u8 | chain_index u64 | size u64 |
                              poly_modulus_degree u64 | coeff_modulus_size u64 | scale f64 |
                              data_size u64 | data u64[size * limbs * N] | prng seed u8[64]
    plaintext:                parms_id[32] | coeff_modulus_size u64 | chain_index u64 |
                              poly_modulus_degree u64 | scale f64 | data_size u64 | data u64[limbs * N]

parms_id is the unkeyed 32-byte BLAKE2b digest of the uint64 words (scheme, N, special_modulus_size,
every key-level prime, the primes of the object's chain level, plain modulus = 0), as
cahel-main/include/util/encryptionparams.h:337-381 and util/hash.h:22-38 form it; chain level 0
carries all primes, 1 drops the special ones, every further level drops one more
(cahel-main/src/context.cu:352-403).  A public key is a size-2 ciphertext over all primes with the
key level's parms_id; the reference stores chain index 1 and scale 1.0 in it.

    relinearization key:      parms_id[32] (key level) | generated u8 | pair count u64 | that many key pairs, each a
                              size-2 ciphertext stream over all primes with chain index 0 and scale 1.0
                              (cahel-main/include/secretkey.h:212-256, src/secretkey.cu:322-370)
    Galois keys:              parms_id[32] (key level) | generated u8 | key count u64 | that many relinearization-key
                              streams, one per Galois element of the context (secretkey.h:354-400)

The reference's secret key has no stream of its own.  Its save_seed flags are accepted but never acted on
(cahel-main/src/secretkey.cu:459: "current version not support"), so no seeded form exists to be compatible with.

Pure host code: it packs and unpacks numpy arrays and knows nothing about devices.
"""
import hashlib
import struct

import numpy as np

SCHEME_CKKS = 3
SEED_BYTES = 64


def level_moduli(moduli, size_p, chain_index):
    """primes in use at a chain level of the context built from ``moduli`` (data primes first, then special)"""
    moduli = [int(m) for m in moduli]
    if chain_index == 0:
        return moduli
    size_q = len(moduli) - size_p
    keep = size_q - (chain_index - 1)
    if keep < 1 or chain_index < 0:
        raise ValueError("chain_index is out of range")
    return moduli[:keep]


def parms_id(poly_modulus_degree, moduli, size_p, chain_index):
    words = [SCHEME_CKKS, int(poly_modulus_degree), int(size_p)] + [int(m) for m in moduli]
    words += level_moduli(moduli, size_p, chain_index) + [0]
    data = struct.pack("<%dQ" % len(words), *words)
    return hashlib.blake2b(data, digest_size=32).digest()


def _words(a):
    a = np.ascontiguousarray(a)
    if a.dtype not in (np.uint64, np.int64):
        raise ValueError("residues must be 64-bit words")
    return a.view(np.uint64).reshape(-1)


def pack_ciphertext(pid, chain_index, size, poly_modulus_degree, coeff_modulus_size, scale, data, is_ntt_form=True, seed=None):
    w = _words(data)
    if w.size != size * coeff_modulus_size * poly_modulus_degree:
        raise ValueError("data does not match size * coeff_modulus_size * poly_modulus_degree")
    seed = bytes(SEED_BYTES) if seed is None else bytes(seed)
    if len(pid) != 32 or len(seed) != SEED_BYTES:
        raise ValueError("parms_id is 32 bytes and the seed block 64")
    head = pid + struct.pack("<BQQQQdQ", 1 if is_ntt_form else 0, chain_index, size, poly_modulus_degree, coeff_modulus_size, float(scale),
                             w.size)
    return head + w.astype("<u8", copy=False).tobytes() + seed


def pack_public_key(poly_modulus_degree, moduli, size_p, data):
    return pack_ciphertext(parms_id(poly_modulus_degree, moduli, size_p, 0), 1, 2, poly_modulus_degree, len(moduli), 1.0, data)


def pack_plaintext(pid, chain_index, poly_modulus_degree, coeff_modulus_size, scale, data):
    w = _words(data)
    if w.size != coeff_modulus_size * poly_modulus_degree:
        raise ValueError("data does not match coeff_modulus_size * poly_modulus_degree")
    if len(pid) != 32:
        raise ValueError("parms_id is 32 bytes")
    head = pid + struct.pack("<QQQdQ", coeff_modulus_size, chain_index, poly_modulus_degree, float(scale), w.size)
    return head + w.astype("<u8", copy=False).tobytes()


def _take(buf, off, fmt):
    n = struct.calcsize(fmt)
    if off + n > len(buf):
        raise RuntimeError("I/O error")  # the reference reports a short stream this way
    return struct.unpack_from(fmt, buf, off), off + n


def unpack_ciphertext(buf):
    buf = bytes(buf)
    if len(buf) < 32:
        raise RuntimeError("I/O error")
    pid, off = buf[:32], 32
    (ntt, chain, size, n, limbs, scale, count), off = _take(buf, off, "<BQQQQdQ")
    total = size * n * limbs
    if count != total or off + 8 * total + SEED_BYTES > len(buf):
        raise RuntimeError("I/O error")
    data = np.frombuffer(buf, dtype="<u8", count=total, offset=off).reshape(size, limbs, n).copy()
    off += 8 * total
    return dict(parms_id=pid, is_ntt_form=bool(ntt), chain_index=chain, size=size, poly_modulus_degree=n, coeff_modulus_size=limbs,
                scale=scale, data=data, seed=buf[off:off + SEED_BYTES], consumed=off + SEED_BYTES)


def unpack_plaintext(buf):
    buf = bytes(buf)
    if len(buf) < 32:
        raise RuntimeError("I/O error")
    pid, off = buf[:32], 32
    (limbs, chain, n, scale, count), off = _take(buf, off, "<QQQdQ")
    total = limbs * n
    if count != total or off + 8 * total > len(buf):
        raise RuntimeError("I/O error")
    data = np.frombuffer(buf, dtype="<u8", count=total, offset=off).reshape(limbs, n).copy()
    return dict(parms_id=pid, chain_index=chain, poly_modulus_degree=n, coeff_modulus_size=limbs, scale=scale, data=data,
                consumed=off + 8 * total)


def pack_switch_key(poly_modulus_degree, moduli, size_p, data):
    """data: [dnum][2][size_QP][N] -> the reference's CAHELGPURelinKey stream"""
    a = np.ascontiguousarray(data)
    n_qp = len(moduli)
    dnum = a.size // (2 * n_qp * poly_modulus_degree)
    if dnum * 2 * n_qp * poly_modulus_degree != a.size or dnum < 1:
        raise ValueError("data does not match [dnum][2][size_QP][N]")
    pid = parms_id(poly_modulus_degree, moduli, size_p, 0)
    a = a.reshape(dnum, -1)
    parts = [pid, struct.pack("<BQ", 1, dnum)]
    for j in range(dnum):
        parts.append(pack_ciphertext(pid, 0, 2, poly_modulus_degree, n_qp, 1.0, a[j]))
    return b"".join(parts)


def unpack_switch_key(buf):
    buf = bytes(buf)
    if len(buf) < 41:
        raise RuntimeError("I/O error")
    pid = buf[:32]
    (generated, dnum), off = _take(buf, 32, "<BQ")
    if dnum < 1 or dnum > 64:
        raise RuntimeError("I/O error")
    pairs = []
    for _ in range(dnum):
        f = unpack_ciphertext(buf[off:])
        if f["size"] != 2 or f["parms_id"] != pid:
            raise ValueError("relinearization key data is invalid")
        pairs.append(f["data"])
        off += f["consumed"]
    return dict(parms_id=pid, generated=bool(generated), poly_modulus_degree=pairs[0].shape[2], coeff_modulus_size=pairs[0].shape[1],
                data=np.stack(pairs), consumed=off)


def pack_galois_keys(poly_modulus_degree, moduli, size_p, keys):
    """keys: one [dnum][2][size_QP][N] array per Galois element -> the reference's CAHELGPUGaloisKey stream"""
    pid = parms_id(poly_modulus_degree, moduli, size_p, 0)
    return b"".join([pid, struct.pack("<BQ", 1, len(keys))] + [pack_switch_key(poly_modulus_degree, moduli, size_p, k) for k in keys])


def unpack_galois_keys(buf):
    buf = bytes(buf)
    if len(buf) < 41:
        raise RuntimeError("I/O error")
    pid = buf[:32]
    (generated, count), off = _take(buf, 32, "<BQ")
    if count > 4096:
        raise RuntimeError("I/O error")
    keys = []
    for _ in range(count):
        f = unpack_switch_key(buf[off:])
        if f["parms_id"] != pid:
            raise ValueError("Galois key data is invalid")
        keys.append(f["data"])
        off += f["consumed"]
    return dict(parms_id=pid, generated=bool(generated), keys=keys, consumed=off)
