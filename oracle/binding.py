"""ctypes binding of ``libckks_oracle.so`` (the CPU restatement in ``ckks_oracle.c``).

Test infrastructure only.  All polynomial data are ``numpy.uint64`` arrays laid out as
in the reference library: polynomial ``[limb][N]``, ciphertext ``[poly][limb][N]``,
key pair ``[2][size_QP][N]``, switch key ``[dnum][2][size_QP][N]``.
"""
import ctypes as C
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_SO = os.path.join(_HERE, "libckks_oracle.so")

u64 = C.c_uint64
_p64 = C.POINTER(C.c_uint64)
_p8 = C.POINTER(C.c_uint8)


def build():
    """Compile the checker library with the Makefile beside it."""
    subprocess.check_call(["make", "-C", _HERE, "libckks_oracle.so"], stdout=subprocess.DEVNULL)


def _load():
    if not os.path.exists(_SO):
        build()
    lib = C.CDLL(_SO)
    lib.orc_mulmod.restype = u64
    lib.orc_mulmod.argtypes = [u64, u64, u64]
    lib.orc_powmod.restype = u64
    lib.orc_powmod.argtypes = [u64, u64, u64]
    lib.orc_invmod.restype = u64
    lib.orc_invmod.argtypes = [u64, u64]
    lib.orc_shoup.restype = u64
    lib.orc_shoup.argtypes = [u64, u64]
    lib.orc_is_prime.argtypes = [u64]
    lib.orc_get_primes.argtypes = [u64, C.c_int, C.c_int, _p64]
    lib.orc_coeff_modulus_create.argtypes = [u64, C.POINTER(C.c_int), C.c_int, _p64]
    lib.orc_minimal_primitive_root.restype = u64
    lib.orc_minimal_primitive_root.argtypes = [u64, u64]
    lib.orc_elt_from_step.restype = C.c_uint32
    lib.orc_elt_from_step.argtypes = [C.c_int, u64]
    lib.orc_create.restype = C.c_void_p
    lib.orc_create.argtypes = [C.c_int, _p64, C.c_int, C.c_int, C.POINTER(C.c_uint32), C.c_int]
    lib.orc_destroy.argtypes = [C.c_void_p]
    lib.orc_get_modulus.restype = u64
    lib.orc_get_modulus.argtypes = [C.c_void_p, C.c_int]
    lib.orc_get_psi.restype = u64
    lib.orc_get_psi.argtypes = [C.c_void_p, C.c_int]
    lib.orc_get_perm.restype = C.POINTER(C.c_uint32)
    lib.orc_get_perm.argtypes = [C.c_void_p, C.c_int]
    lib.orc_get_twiddles.restype = _p64
    lib.orc_get_twiddles.argtypes = [C.c_void_p, C.c_int, C.c_int]
    vp = C.c_void_p
    I = C.c_int
    lib.orc_ntt_fwd.argtypes = [vp, _p64, I]
    lib.orc_ntt_inv.argtypes = [vp, _p64, I]
    lib.orc_ntt_rows.argtypes = [vp, _p64, I, I, I, I]
    lib.orc_poly_op.argtypes = [vp, I, I, I, _p64, _p64, _p64]
    lib.orc_tensor.argtypes = [vp, I, _p64, _p64, _p64]
    lib.orc_square.argtypes = [vp, I, _p64, _p64]
    lib.orc_galois.argtypes = [vp, I, I, _p64, _p64]
    lib.orc_modup.argtypes = [vp, I, _p64, _p64]
    lib.orc_inner_product.argtypes = [vp, I, _p64, _p64, _p64]
    lib.orc_moddown.argtypes = [vp, I, _p64, _p64]
    lib.orc_keyswitch.argtypes = [vp, I, _p64, _p64, _p64]
    lib.orc_relinearize.argtypes = [vp, I, _p64, _p64]
    lib.orc_rescale.argtypes = [vp, I, I, _p64, _p64]
    lib.orc_drop_last.argtypes = [vp, I, I, _p64, _p64]
    lib.orc_rotate.argtypes = [vp, I, _p64, I, _p64]
    lib.orc_hoisting.argtypes = [vp, I, _p64, I, C.POINTER(C.c_int), C.POINTER(_p64)]
    lib.orc_prng_block.argtypes = [_p8, u64, C.POINTER(C.c_uint32)]
    lib.orc_sample_small.argtypes = [vp, I, _p8, I, I, _p64]
    lib.orc_sample_uniform.argtypes = [vp, _p8, I, I, _p64]
    lib.orc_gen_sk.argtypes = [vp, _p8, _p64]
    lib.orc_gen_pk.argtypes = [vp, _p64, _p8, _p8, _p64]
    lib.orc_gen_ksk.argtypes = [vp, _p64, _p64, _p8, _p64]
    lib.orc_encrypt_zero_asym.argtypes = [vp, _p64, _p8, _p8, _p64]
    lib.orc_decrypt.argtypes = [vp, I, I, _p64, _p64, _p64]
    pd = C.POINTER(C.c_double)
    lib.orc_encode.argtypes = [vp, I, pd, C.c_size_t, C.c_size_t, C.c_double, _p64]
    lib.orc_decode.argtypes = [vp, I, _p64, C.c_double, C.c_size_t, pd]
    lib.orc_croot.argtypes = [C.c_size_t, C.c_size_t, pd]
    lib.orc_max_threads.restype = I
    lib.orc_set_threads.argtypes = [I]
    lib.orc_encode_encrypt_batch.argtypes = [vp, _p64, pd, C.c_size_t, C.c_double, _p8, I, _p64]
    lib.orc_pair_chunk_batch.argtypes = [vp, I, _p64, _p64, _p64, I]
    lib.orc_relin_rescale_batch.argtypes = [vp, I, _p64, _p64, _p64, I]
    lib.orc_mask_chunk_batch.argtypes = [vp, I, _p64, _p64, _p64, I]
    lib.orc_hmult_batch.argtypes = [vp, I, _p64, _p64, _p64, _p64, I]
    lib.orc_rotate_batch.argtypes = [vp, I, _p64, I, _p64, I]
    lib.orc_ntt_roundtrip_batch.argtypes = [vp, _p64, I, I]
    return lib


lib = _load()


def _u(a):
    assert a.dtype == np.uint64 and a.flags["C_CONTIGUOUS"]
    return a.ctypes.data_as(_p64)


def _s(seed):
    seed = np.ascontiguousarray(seed, dtype=np.uint8)
    assert seed.size % 64 == 0
    return seed, seed.ctypes.data_as(_p8)


def coeff_modulus_create(N, bit_sizes):
    """Primes handed out as the reference does (cahel-main/src/modulus.cu:93-125)."""
    n = len(bit_sizes)
    out = np.zeros(n, dtype=np.uint64)
    bits = (C.c_int * n)(*bit_sizes)
    if lib.orc_coeff_modulus_create(N, bits, n, _u(out)) != 0:
        raise ValueError("failed to find enough qualifying primes")
    return [int(x) for x in out]


def elts_from_steps(steps, N):
    return [int(lib.orc_elt_from_step(int(s), N)) for s in steps]


class Oracle:
    """One parameter set: ring degree, the QP modulus list, special-prime count, Galois elements."""

    def __init__(self, logN, moduli, size_P, galois_elts=()):
        self.logN, self.N = logN, 1 << logN
        self.moduli = [int(m) for m in moduli]
        self.size_QP, self.size_P = len(moduli), size_P
        self.size_Q = self.size_QP - size_P
        self.elts = [int(e) for e in galois_elts]
        m = np.array(self.moduli, dtype=np.uint64)
        e = (C.c_uint32 * max(1, len(self.elts)))(*self.elts)
        self.h = lib.orc_create(logN, _u(m), self.size_QP, size_P, e, len(self.elts))
        if not self.h:
            raise ValueError("invalid modulus for NTT")

    def __del__(self):
        if getattr(self, "h", None):
            lib.orc_destroy(self.h)
            self.h = None

    # -- tables
    def psi(self, i):
        return int(lib.orc_get_psi(self.h, i))

    def perm(self, i):
        return np.ctypeslib.as_array(lib.orc_get_perm(self.h, i), shape=(self.N,)).copy()

    def twiddles(self, mod, inverse=False):
        return np.ctypeslib.as_array(lib.orc_get_twiddles(self.h, mod, int(inverse)), shape=(self.N,)).copy()

    def beta(self, L):
        return (L + self.size_P - 1) // self.size_P

    # -- transforms
    def ntt_rows(self, data, n_groups, size_l, size_p, inverse=False):
        out = np.ascontiguousarray(data, dtype=np.uint64).copy()
        lib.orc_ntt_rows(self.h, _u(out), n_groups, size_l, size_p, int(inverse))
        return out

    # -- element-wise
    def poly_op(self, op, L, a, b=None):
        code = {"add": 0, "sub": 1, "mul": 2, "neg": 3}[op]
        a = np.ascontiguousarray(a, dtype=np.uint64)
        n_polys = a.size // (L * self.N)
        out = np.empty_like(a)
        bb = _u(np.ascontiguousarray(b, dtype=np.uint64)) if b is not None else None
        lib.orc_poly_op(self.h, code, L, n_polys, _u(a), bb, _u(out))
        return out

    def tensor(self, L, a, b):
        out = np.empty((3, L, self.N), dtype=np.uint64)
        lib.orc_tensor(self.h, L, _u(np.ascontiguousarray(a)), _u(np.ascontiguousarray(b)), _u(out))
        return out

    def square(self, L, a):
        return self.tensor(L, a, a)

    def galois(self, elt_idx, data):
        data = np.ascontiguousarray(data, dtype=np.uint64)
        out = np.empty_like(data)
        lib.orc_galois(self.h, elt_idx, data.size // self.N, _u(data), _u(out))
        return out

    # -- key switching
    def modup(self, L, cks):
        out = np.empty((self.beta(L), L + self.size_P, self.N), dtype=np.uint64)
        lib.orc_modup(self.h, L, _u(np.ascontiguousarray(cks)), _u(out))
        return out

    def inner_product(self, L, digits, evk):
        out = np.empty((2, L + self.size_P, self.N), dtype=np.uint64)
        lib.orc_inner_product(self.h, L, _u(np.ascontiguousarray(digits)), _u(np.ascontiguousarray(evk)), _u(out))
        return out

    def moddown(self, L, cx):
        out = np.empty((L, self.N), dtype=np.uint64)
        lib.orc_moddown(self.h, L, _u(np.ascontiguousarray(cx)), _u(out))
        return out

    def keyswitch(self, L, ct, cks, evk):
        ct = np.ascontiguousarray(ct, dtype=np.uint64).copy()
        lib.orc_keyswitch(self.h, L, _u(ct), _u(np.ascontiguousarray(cks)), _u(np.ascontiguousarray(evk)))
        return ct

    def relinearize(self, L, ct3, rlk):
        ct3 = np.ascontiguousarray(ct3, dtype=np.uint64).copy()
        lib.orc_relinearize(self.h, L, _u(ct3), _u(np.ascontiguousarray(rlk)))
        return ct3[:2].copy()

    def rescale(self, L, ct):
        ct = np.ascontiguousarray(ct, dtype=np.uint64)
        k = ct.size // (L * self.N)
        out = np.empty((k, L - 1, self.N), dtype=np.uint64)
        lib.orc_rescale(self.h, L, k, _u(ct), _u(out))
        return out

    def drop_last(self, L, ct):
        ct = np.ascontiguousarray(ct, dtype=np.uint64)
        k = ct.size // (L * self.N)
        out = np.empty((k, L - 1, self.N), dtype=np.uint64)
        lib.orc_drop_last(self.h, L, k, _u(ct), _u(out))
        return out

    def rotate(self, L, ct, elt_idx, glk):
        ct = np.ascontiguousarray(ct, dtype=np.uint64).copy()
        lib.orc_rotate(self.h, L, _u(ct), elt_idx, _u(np.ascontiguousarray(glk)))
        return ct

    def hoisting(self, L, ct, elt_idx, glks):
        ct = np.ascontiguousarray(ct, dtype=np.uint64).copy()
        n = len(elt_idx)
        idx = (C.c_int * n)(*elt_idx)
        keep = [np.ascontiguousarray(k, dtype=np.uint64) for k in glks]
        ptrs = (_p64 * n)(*[_u(k) for k in keep])
        lib.orc_hoisting(self.h, L, _u(ct), n, idx, ptrs)
        return ct

    # -- randomness
    def prng_block(self, seed, nonce):
        seed, sp = _s(seed)
        out = (C.c_uint32 * 16)()
        lib.orc_prng_block(sp, nonce, out)
        return np.array(out[:], dtype=np.uint32)

    def sample_small(self, kind, seed, size_l, size_p):
        seed, sp = _s(seed)
        out = np.empty((size_l + size_p, self.N), dtype=np.uint64)
        lib.orc_sample_small(self.h, {"ternary": 0, "error": 1}[kind], sp, size_l, size_p, _u(out))
        return out

    def sample_uniform(self, seed, size_l, size_p):
        seed, sp = _s(seed)
        out = np.empty((size_l + size_p, self.N), dtype=np.uint64)
        lib.orc_sample_uniform(self.h, sp, size_l, size_p, _u(out))
        return out

    # -- keys / encryption
    def gen_sk(self, seed):
        seed, sp = _s(seed)
        sk = np.empty((self.size_QP, self.N), dtype=np.uint64)
        lib.orc_gen_sk(self.h, sp, _u(sk))
        return sk

    def gen_pk(self, sk, seed_e, seed_a):
        se, pe = _s(seed_e)
        sa, pa = _s(seed_a)
        pk = np.empty((2, self.size_QP, self.N), dtype=np.uint64)
        lib.orc_gen_pk(self.h, _u(sk), pe, pa, _u(pk))
        return pk

    def gen_ksk(self, sk, skp, seeds):
        """seeds: uint8 array [dnum][2][64]"""
        dnum = self.size_Q // self.size_P
        seeds, sp = _s(seeds)
        assert seeds.size == dnum * 128
        out = np.empty((dnum, 2, self.size_QP, self.N), dtype=np.uint64)
        lib.orc_gen_ksk(self.h, _u(sk), _u(np.ascontiguousarray(skp)), sp, _u(out))
        return out

    def sk_square(self, sk):
        return self.poly_op_qp("mul", sk, sk)

    def poly_op_qp(self, op, a, b):
        """element-wise op over the full QP limb list"""
        out = np.empty_like(a)
        for r in range(self.size_QP):
            q = self.moduli[r]
            x = a[r].astype(object)
            y = b[r].astype(object)
            v = {"mul": x * y, "add": x + y, "sub": x - y}[op] % q
            out[r] = np.array(v, dtype=np.uint64)
        return out

    def encrypt_zero_asym(self, pk, seed_u, seed_e):
        su, pu = _s(seed_u)
        se, pe = _s(seed_e)
        ct = np.empty((2, self.size_Q, self.N), dtype=np.uint64)
        lib.orc_encrypt_zero_asym(self.h, _u(np.ascontiguousarray(pk)), pu, pe, _u(ct))
        return ct

    def encrypt_asym(self, pk, pt, seed_u, seed_e):
        ct = self.encrypt_zero_asym(pk, seed_u, seed_e)
        ct[0] = self.poly_op("add", self.size_Q, ct[0], pt)
        return ct

    def decrypt(self, L, ct, sk):
        ct = np.ascontiguousarray(ct, dtype=np.uint64)
        k = ct.size // (L * self.N)
        pt = np.empty((L, self.N), dtype=np.uint64)
        lib.orc_decrypt(self.h, L, k, _u(ct), _u(np.ascontiguousarray(sk)), _u(pt))
        return pt

    # -- encoder
    def encode(self, L, values, scale, sparse_slots=None):
        v = np.ascontiguousarray(np.asarray(values, dtype=np.complex128))
        n = v.size
        if sparse_slots is None:
            sparse_slots = 1 << max(1, int(np.ceil(np.log2(max(n, 2)))))
        pt = np.empty((L, self.N), dtype=np.uint64)
        raw = v.view(np.float64)
        lib.orc_encode(self.h, L, raw.ctypes.data_as(C.POINTER(C.c_double)), n, sparse_slots, float(scale), _u(pt))
        return pt

    def decode(self, L, pt, scale, sparse_slots):
        out = np.empty(sparse_slots, dtype=np.complex128)
        lib.orc_decode(self.h, L, _u(np.ascontiguousarray(pt)), float(scale), sparse_slots,
                       out.view(np.float64).ctypes.data_as(C.POINTER(C.c_double)))
        return out

    # -- batched forms (one OpenMP thread per item) used by the timed CPU baseline
    def encode_encrypt_batch(self, pk, values, scale, seeds):
        values = np.ascontiguousarray(values, dtype=np.float64)
        batch, slots = values.shape
        seeds, sp = _s(seeds)
        assert seeds.size == 128 * batch
        ct = np.empty((batch, 2, self.size_Q, self.N), dtype=np.uint64)
        lib.orc_encode_encrypt_batch(self.h, _u(np.ascontiguousarray(pk)), values.ctypes.data_as(C.POINTER(C.c_double)), slots,
                                     float(scale), sp, batch, _u(ct))
        return ct

    def pair_chunk_batch(self, L, x, y, acc):
        """acc[b] += (y[b] - x[b])^2 in place"""
        lib.orc_pair_chunk_batch(self.h, L, _u(x), _u(y), _u(acc), x.shape[0])
        return acc

    def mask_chunk_batch(self, L, x, mask, acc):
        """acc[b] += x[b] (x) mask in place"""
        lib.orc_mask_chunk_batch(self.h, L, _u(x), _u(np.ascontiguousarray(mask)), _u(acc), x.shape[0])
        return acc

    def relin_rescale_batch(self, L, ct3, rlk):
        ct3 = np.ascontiguousarray(ct3, dtype=np.uint64).copy()
        out = np.empty((ct3.shape[0], 2, L - 1, self.N), dtype=np.uint64)
        lib.orc_relin_rescale_batch(self.h, L, _u(ct3), _u(np.ascontiguousarray(rlk)), _u(out), ct3.shape[0])
        return out

    def hmult_batch(self, L, x, y, rlk):
        out = np.empty((x.shape[0], 2, L - 1, self.N), dtype=np.uint64)
        lib.orc_hmult_batch(self.h, L, _u(x), _u(y), _u(np.ascontiguousarray(rlk)), _u(out), x.shape[0])
        return out

    def rotate_batch(self, L, ct, elt_idx, glk):
        """in place"""
        lib.orc_rotate_batch(self.h, L, _u(ct), elt_idx, _u(np.ascontiguousarray(glk)), ct.shape[0])
        return ct

    def ntt_roundtrip_batch(self, data, size_l):
        """forward then inverse transform in place"""
        lib.orc_ntt_roundtrip_batch(self.h, _u(data), data.shape[0], size_l)
        return data


def set_threads(n):
    """number of OpenMP threads for later calls (overrides whatever OMP_NUM_THREADS said at load time)"""
    lib.orc_set_threads(int(n))


def max_threads():
    """threads the library's OpenMP runtime will use (what OMP_NUM_THREADS resolved to at load time)"""
    return int(lib.orc_max_threads())
