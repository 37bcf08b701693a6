"""Host-side mirror of the reference's ``pyCAHEL`` module (cahel-main/python/src/binding.cu:8-156).

Same names, argument order (``(context, inputs..., output)`` with the output mutated in
place) and error behaviour (``ValueError`` where the reference throws
``std::invalid_argument``, ``RuntimeError`` where it throws ``std::logic_error``), for the
CKKS path that ``lancelot-main-GPU/utils/byzantine_fl.py`` uses.  All arithmetic runs in
``liblancelot_b200.so`` on the GPU through ``lancelot_b200.cabi``; this file only keeps
shapes, levels and scales, as the reference's C++ containers do
(cahel-main/include/ciphertext.h, plaintext.h, secretkey.h).

Differences from the reference that a caller can see:
* seeds: the reference reads /dev/urandom for every key and encryption
  (cahel-main/include/prng.cuh:12-23).  Here they come from ``os.urandom`` unless
  ``set_seed_source`` installs a deterministic generator (needed for bit-exact replays);
* ``encode`` also accepts numpy arrays and CUDA tensors (float32/float64) without a
  Python-list round trip;
* decryption adds no noise-flooding term (the reference's needs OpenFHE,
  cahel-main/src/secretkey.cu:632-649);
* BFV/BGV entry points raise ``ValueError("unsupported scheme")``;
* ``save`` / ``load`` of plaintexts, ciphertexts and public keys exist here although the pybind module
  does not export them: they write and read the byte streams of the reference's C++ classes
  (``lancelot_b200.wire``), and take the context as their first argument.
"""
import enum
import math
import os

import numpy as np
import torch

from . import cabi, wire
from ._lib import InvalidArgument, LancelotError

# ---- enums (binding.cu:9-29, export_values) -------------------------------------------------


class scheme_type(enum.IntEnum):
    none = 0
    bgv = 1
    bfv = 2
    ckks = 3


class mul_tech_type(enum.IntEnum):
    none = 0
    behz = 1
    hps = 2
    hps_overq = 3
    hps_overq_leveled = 4


class sec_level_type(enum.IntEnum):
    none = 0
    tc128 = 128
    tc192 = 192
    tc256 = 256


bgv, bfv, ckks = scheme_type.bgv, scheme_type.bfv, scheme_type.ckks
behz, hps, hps_overq, hps_overq_leveled = (mul_tech_type.behz, mul_tech_type.hps, mul_tech_type.hps_overq,
                                           mul_tech_type.hps_overq_leveled)
tc128, tc192, tc256 = sec_level_type.tc128, sec_level_type.tc192, sec_level_type.tc256

# ---- seed source ----------------------------------------------------------------------------

_seed_source = None


def set_seed_source(fn):
    """fn(count) -> ``count`` * 64 bytes (uint8 array or bytes); None restores os.urandom."""
    global _seed_source
    _seed_source = fn


def _seeds(count):
    raw = os.urandom(64 * count) if _seed_source is None else _seed_source(count)
    a = np.frombuffer(bytes(raw), dtype=np.uint8) if not isinstance(raw, np.ndarray) else raw.astype(np.uint8).reshape(-1)
    if a.size != 64 * count:
        raise RuntimeError("seed source returned %d bytes, expected %d" % (a.size, 64 * count))
    return np.ascontiguousarray(a)


class counter_seed_source:
    """Deterministic seeds for tests: 64-byte blocks from numpy's PCG64 with a fixed seed."""

    def __init__(self, seed=0):
        self.rng = np.random.default_rng(seed)

    def __call__(self, count):
        return self.rng.integers(0, 256, 64 * count, dtype=np.uint8)


# ---- parameters and context ------------------------------------------------------------------


class modulus:
    def __init__(self, value):
        self._value = int(value)

    def value(self):
        return self._value

    def __int__(self):
        return self._value

    def __repr__(self):
        return "modulus(%d)" % self._value


def coeff_modulus_create(poly_modulus_degree, bit_sizes):
    """CoeffModulus::Create (cahel-main/src/modulus.cu:93-125)."""
    return [modulus(v) for v in cabi.coeff_modulus_create(int(poly_modulus_degree), [int(b) for b in bit_sizes])]


def get_elts_from_steps(steps, coeff_count):
    """cahel-main/include/galois.cuh:155-192"""
    return cabi.galois_elts_from_steps([int(s) for s in steps], int(coeff_count))


class params:
    """EncryptionParameters (binding.cu:36-42)."""

    def __init__(self, scheme):
        self.scheme = scheme_type(scheme)
        self.poly_modulus_degree = 0
        self.coeff_modulus = []
        self.special_modulus_size = 1
        self.galois_elts = []
        self.mul_tech = mul_tech_type.none

    def set_mul_tech(self, t):
        self.mul_tech = mul_tech_type(t)

    def set_poly_modulus_degree(self, n):
        self.poly_modulus_degree = int(n)

    def set_special_modulus_size(self, k):
        self.special_modulus_size = int(k)

    def set_galois_elts(self, elts):
        self.galois_elts = [int(e) for e in elts]

    def set_coeff_modulus(self, moduli):
        self.coeff_modulus = [int(m) for m in moduli]


class context:
    """CAHELGPUContext (cahel-main/include/gpucontext.h:53-136): modulus chain, tables on the device.

    chain index 0 is the key level (all primes), 1 the first data level (special primes dropped),
    every further index drops one more prime (cahel-main/src/context.cu:352-403)."""

    def __init__(self, parms, expand_mod_chain=True, sec_level=sec_level_type.tc128, device=None):
        if parms.scheme != scheme_type.ckks:
            raise ValueError("unsupported scheme")
        n = parms.poly_modulus_degree
        if n < 16 or n & (n - 1):
            raise ValueError("invalid poly_modulus_degree")
        if not parms.coeff_modulus:
            raise ValueError("coeff_modulus is not set")
        self.parms = parms
        self.N = n
        self.log_n = n.bit_length() - 1
        self.size_QP = len(parms.coeff_modulus)
        self.size_P = parms.special_modulus_size if self.size_QP > 1 else 0
        self.size_Q = self.size_QP - self.size_P
        self.moduli = list(parms.coeff_modulus)
        self.galois_elts = list(parms.galois_elts)
        self.expand_mod_chain = bool(expand_mod_chain)
        dev = torch.cuda.current_device() if device is None else int(device)
        try:
            self.lb = cabi.Context(self.log_n, self.moduli, self.size_P, self.galois_elts,
                                   check_tc128=(sec_level_type(sec_level) != sec_level_type.none), device=dev)
        except InvalidArgument as e:
            raise ValueError(str(e)) from None
        self.max_chain = self.size_Q if expand_mod_chain else 1

    def size_l(self, chain_index):
        if chain_index == 0:
            return self.size_Q
        if chain_index < 1 or chain_index > self.max_chain:
            raise ValueError("chain_index is out of range")
        return self.size_Q - (chain_index - 1)

    def total_bits(self, chain_index):
        limbs = self.moduli if chain_index == 0 else self.moduli[: self.size_l(chain_index)]
        p = 1
        for m in limbs:
            p *= m
        return p.bit_length()

    def elt_index(self, elt):
        try:
            return self.galois_elts.index(int(elt))
        except ValueError:
            return -1


# ---- containers --------------------------------------------------------------------------------


def _to_device(ctx, words):
    return torch.from_numpy(np.ascontiguousarray(words).view(np.int64)).to("cuda:%d" % ctx.lb.device)


def _stream_bytes(stream, unpack):
    """reads one object from a binary stream that may hold several, leaving the stream after it"""
    start = stream.tell()
    blob = stream.read()
    out = unpack(blob)
    stream.seek(start + out["consumed"])
    return out


class plaintext:
    """CAHELGPUPlaintext: [limb][N] residues in NTT form, a chain index and a scale."""

    def __init__(self, ctx=None):
        self.data = None
        self.chain_index = 0
        self.scale = 1.0
        self.is_ntt_form = True

    def save(self, ctx, stream):
        """cahel-main/include/plaintext.h:109-146, byte for byte (the reference method takes no context; this
        container does not keep one, so it is passed in)"""
        limbs = ctx.size_l(self.chain_index)
        pid = wire.parms_id(ctx.N, ctx.moduli, ctx.size_P, self.chain_index)
        stream.write(wire.pack_plaintext(pid, self.chain_index, ctx.N, limbs, self.scale, self.data.cpu().numpy()))

    def load(self, ctx, stream):
        """cahel-main/include/plaintext.h:148-213"""
        f = _stream_bytes(stream, wire.unpack_plaintext)
        if f["poly_modulus_degree"] != ctx.N or f["parms_id"] != wire.parms_id(ctx.N, ctx.moduli, ctx.size_P, f["chain_index"]) \
                or f["coeff_modulus_size"] != ctx.size_l(f["chain_index"]):
            raise ValueError("plaintext data is invalid")
        self.data = _to_device(ctx, f["data"])
        self.chain_index, self.scale, self.is_ntt_form = int(f["chain_index"]), float(f["scale"]), True


class ciphertext:
    """CAHELGPUCiphertext: [poly][limb][N] residues in NTT form, chain index, scale."""

    def __init__(self, ctx=None):
        self.data = None
        self.size = 0
        self.chain_index = 0
        self.scale = 1.0
        self.is_ntt_form = True

    def set_scale(self, s):
        self.scale = float(s)

    def _assign(self, other):
        self.data = other.data.clone()
        self.size, self.chain_index, self.scale, self.is_ntt_form = other.size, other.chain_index, other.scale, other.is_ntt_form

    def copy(self):
        c = ciphertext()
        c._assign(self)
        return c

    def save(self, ctx, stream):
        """cahel-main/include/ciphertext.h:174-223, byte for byte (seed block zeroed, as the reference leaves it)"""
        limbs = ctx.size_l(self.chain_index)
        pid = wire.parms_id(ctx.N, ctx.moduli, ctx.size_P, self.chain_index)
        stream.write(wire.pack_ciphertext(pid, self.chain_index, self.size, ctx.N, limbs, self.scale, self.data.cpu().numpy(),
                                          is_ntt_form=self.is_ntt_form))

    def load(self, ctx, stream):
        """cahel-main/include/ciphertext.h:225-292"""
        f = _stream_bytes(stream, wire.unpack_ciphertext)
        if f["poly_modulus_degree"] != ctx.N or f["parms_id"] != wire.parms_id(ctx.N, ctx.moduli, ctx.size_P, f["chain_index"]) \
                or f["coeff_modulus_size"] != ctx.size_l(f["chain_index"]) or f["size"] < 2:
            raise ValueError("ciphertext data is invalid")
        self.data = _to_device(ctx, f["data"])
        self.size, self.chain_index, self.scale, self.is_ntt_form = int(f["size"]), int(f["chain_index"]), float(f["scale"]), f["is_ntt_form"]


class public_key:
    def __init__(self, ctx):
        self.data = None

    def save(self, ctx, stream):
        """cahel-main/include/secretkey.h:54-56: the key pair as a size-2 ciphertext over all primes"""
        if self.data is None:
            raise RuntimeError("public key has not been generated")
        stream.write(wire.pack_public_key(ctx.N, ctx.moduli, ctx.size_P, self.data.cpu().numpy()))

    def load(self, ctx, stream):
        """cahel-main/include/secretkey.h:58-60"""
        f = _stream_bytes(stream, wire.unpack_ciphertext)
        if f["poly_modulus_degree"] != ctx.N or f["parms_id"] != wire.parms_id(ctx.N, ctx.moduli, ctx.size_P, 0) \
                or f["coeff_modulus_size"] != ctx.size_QP or f["size"] != 2:
            raise ValueError("public key data is invalid")
        self.data = _to_device(ctx, f["data"])

    def encrypt_asymmetric(self, ctx, plain, save_seed=False):
        """cahel-main/src/secretkey.cu:179-249: encrypt at the key level, divide by P, add the plaintext.
        Like the reference, only plaintexts at the first data level are supported."""
        if self.data is None:
            raise RuntimeError("public key has not been generated")
        if not plain.is_ntt_form:
            raise ValueError("CKKS plain must be in NTT form")
        if plain.chain_index != 1:
            raise ValueError("asymmetric encryption expects a plaintext at the first data level")
        ct = ciphertext()
        ct.data = ctx.lb.encrypt_asymmetric(self.data, plain.data, _seeds(2))
        ct.size, ct.chain_index, ct.scale = 2, 1, plain.scale
        return ct


class relin_key:
    def __init__(self, ctx):
        self.data = None

    def save(self, ctx, stream):
        """cahel-main/include/secretkey.h:212-233: the dnum key pairs, each as a size-2 ciphertext over all primes"""
        if self.data is None:
            raise RuntimeError("relinearization key has not been generated")
        stream.write(wire.pack_switch_key(ctx.N, ctx.moduli, ctx.size_P, self.data.cpu().numpy()))

    def load(self, ctx, stream):
        """cahel-main/include/secretkey.h:235-256"""
        f = _stream_bytes(stream, wire.unpack_switch_key)
        if f["poly_modulus_degree"] != ctx.N or f["parms_id"] != wire.parms_id(ctx.N, ctx.moduli, ctx.size_P, 0) \
                or f["coeff_modulus_size"] != ctx.size_QP or f["data"].shape[0] != ctx.size_Q // ctx.size_P:
            raise ValueError("relinearization key data is invalid")
        self.data = _to_device(ctx, f["data"])


class galois_key:
    def __init__(self, ctx):
        self.keys = []  # one switch key per Galois element of the context

    def save(self, ctx, stream):
        """cahel-main/include/secretkey.h:354-375: one relinearization-key stream per Galois element"""
        if not self.keys:
            raise RuntimeError("Galois keys have not been generated")
        stream.write(wire.pack_galois_keys(ctx.N, ctx.moduli, ctx.size_P, [k.cpu().numpy() for k in self.keys]))

    def load(self, ctx, stream):
        """cahel-main/include/secretkey.h:377-400"""
        f = _stream_bytes(stream, wire.unpack_galois_keys)
        dnum = ctx.size_Q // ctx.size_P
        if f["parms_id"] != wire.parms_id(ctx.N, ctx.moduli, ctx.size_P, 0) or len(f["keys"]) != len(ctx.galois_elts) \
                or any(k.shape != (dnum, 2, ctx.size_QP, ctx.N) for k in f["keys"]):
            raise ValueError("Galois key data is invalid")
        self.keys = [_to_device(ctx, k) for k in f["keys"]]


class secret_key:
    def __init__(self, parms):
        self.data = None
        self.powers = {}

    def gen_secretkey(self, ctx):
        self.data = ctx.lb.gen_secret_key(_seeds(1))
        self.powers = {1: self.data}

    def _need(self):
        if self.data is None:
            raise RuntimeError("cannot generate keys for unspecified secret key")

    def _power(self, ctx, k):
        while max(self.powers) < k:
            top = max(self.powers)
            self.powers[top + 1] = ctx.lb.multiply_poly_qp(self.powers[top], self.data)
        return self.powers[k]

    def gen_publickey(self, ctx, pk, save_seed=True):
        self._need()
        s = _seeds(2)
        pk.data = ctx.lb.gen_public_key(self.data, s[:64], s[64:])

    def gen_relinkey(self, ctx, rlk, save_seed=False):
        self._need()
        dnum = ctx.size_Q // ctx.size_P
        rlk.data = ctx.lb.gen_switch_key(self.data, self._power(ctx, 2), _seeds(2 * dnum))

    def create_galois_keys(self, ctx, glk, save_seed=False):
        self._need()
        dnum = ctx.size_Q // ctx.size_P
        for elt in ctx.galois_elts:
            if not (elt & 1) or elt >= 2 * ctx.N:
                raise ValueError("Galois element is not valid")
        # the seeds are drawn key by key, as separate calls would draw them; the keys come from one batched call
        n = len(ctx.galois_elts)
        seeds = np.concatenate([_seeds(2 * dnum) for _ in range(n)]) if n else np.zeros(0, dtype=np.uint8)
        keys = ctx.lb.gen_galois_keys(self.data, list(range(n)), seeds) if n else []
        glk.keys = [keys[i] for i in range(n)]

    def encrypt_symmetric(self, ctx, plain, save_seed=False):
        """cahel-main/src/secretkey.cu:451-560: (c0, c1) = (-(a s + e) + pt, a) at the plaintext's level."""
        self._need()
        L = ctx.size_l(plain.chain_index)
        s = _seeds(2)
        lb = ctx.lb
        e = lb.sample("error", s[:64], L, 0)
        lb.ntt_forward(e, 1, L, 0)
        a = lb.sample("uniform", s[64:], L, 0)
        c0 = lb.add(L, lb.multiply_poly(L, a, self.data[:L].contiguous()), e)
        c0 = lb.add(L, lb.negate(L, c0), plain.data)
        ct = ciphertext()
        ct.data = torch.stack([c0.reshape(L, ctx.N), a.reshape(L, ctx.N)])
        ct.size, ct.chain_index, ct.scale = 2, plain.chain_index, plain.scale
        return ct

    def decrypt(self, ctx, ct):
        """cahel-main/src/secretkey.cu:594-654 (ckks_decrypt), without noise flooding."""
        self._need()
        if not ct.is_ntt_form:
            raise ValueError("encrypted must be in NTT form")
        L = ctx.size_l(ct.chain_index)
        lb = ctx.lb
        if ct.size <= 2:
            pt_data = lb.decrypt(L, ct.data, self.data)
        else:
            # c0 + c1 s + c2 s^2 + ... with the powers kept at the key level
            acc = ct.data[0].contiguous()
            for p in range(1, ct.size):
                acc = lb.add(L, acc, lb.multiply_poly(L, ct.data[p].contiguous(), self._power(ctx, p)[:L].contiguous()))
            pt_data = acc.reshape(L, ctx.N)
        pt = plaintext()
        pt.data, pt.chain_index, pt.scale = pt_data, ct.chain_index, ct.scale
        return pt


class ckks_encoder:
    """CAHELGPUCKKSEncoder (cahel-main/include/ckks.h, src/ckks.cu)."""

    def __init__(self, ctx):
        self.slots = ctx.N // 2
        self.sparse_slots = 0  # fixed by the first encode, like the reference (ckks.cu:131-142)

    def slot_count(self):
        return self.slots

    def reset_sparse_slots(self):
        self.sparse_slots = 0

    def _values(self, ctx, values):
        if isinstance(values, torch.Tensor):
            v = values
            if v.dtype not in (torch.float32, torch.float64, torch.complex128):
                v = v.to(torch.float64)
            return v.to("cuda:%d" % ctx.lb.device).contiguous()
        a = np.asarray(values)
        if np.iscomplexobj(a):
            a = a.astype(np.complex128)
        elif a.dtype != np.float32:
            a = a.astype(np.float64)
        return torch.from_numpy(np.ascontiguousarray(a)).to("cuda:%d" % ctx.lb.device)

    def encode_to(self, ctx, values, chain_index, scale):
        v = self._values(ctx, values).reshape(-1)
        n = v.numel()
        if n > self.slots:
            raise ValueError("values_size is too large")
        if self.sparse_slots == 0:
            self.sparse_slots = 1 << max(0, math.ceil(math.log2(max(n, 1))))
        elif n > self.sparse_slots:
            raise ValueError("values_size exceeds previous message length")
        if self.sparse_slots < 2:
            raise ValueError("single value encoding is not available")
        L = ctx.size_l(chain_index)
        try:
            data = ctx.lb.encode(L, v, float(scale), sparse_slots=self.sparse_slots)
            ctx.lb.check_status()
        except InvalidArgument as e:
            raise ValueError(str(e)) from None
        pt = plaintext()
        pt.data, pt.chain_index, pt.scale = data, chain_index, float(scale)
        return pt

    def encode(self, ctx, values, scale):
        return self.encode_to(ctx, values, 1, scale)

    def decode(self, ctx, plain):
        if not plain.is_ntt_form:
            raise ValueError("plain is not in NTT form")
        if self.sparse_slots == 0:
            self.sparse_slots = self.slots
        L = ctx.size_l(plain.chain_index)
        out = ctx.lb.decode(L, plain.data.contiguous(), plain.scale, self.sparse_slots)
        return out.real.cpu().tolist()

    def decode_tensor(self, ctx, plain):
        """complex128 CUDA tensor of the decoded slots (no host copy)"""
        if self.sparse_slots == 0:
            self.sparse_slots = self.slots
        return ctx.lb.decode(ctx.size_l(plain.chain_index), plain.data.contiguous(), plain.scale, self.sparse_slots)


# ---- evaluator free functions (cahel-main/include/evaluate.h, src/evaluate.cu) ---------------------


def _same_level(a, b):
    if a.chain_index != b.chain_index:
        raise ValueError("encrypted1 and encrypted2 parameter mismatch")
    if a.is_ntt_form != b.is_ntt_form:
        raise ValueError("NTT form mismatch")
    if not _same_scale(a.scale, b.scale):
        raise ValueError("scale mismatch")


def _same_scale(x, y):
    return abs(x - y) <= 1e-9 * max(abs(x), abs(y), 1.0)


def _check_scale(ctx, scale, chain_index):
    # cahel-main/include/context.h:644-660: valid iff scale > 0 and int(log2(scale)) < total bit count
    if scale <= 0 or int(math.log2(scale)) >= ctx.total_bits(chain_index):
        raise ValueError("scale out of bounds")


def negate_inplace(ctx, ct):
    L = ctx.size_l(ct.chain_index)
    ctx.lb.negate(L, ct.data, out=ct.data)


def negate(ctx, ct, dst):
    dst._assign(ct)
    negate_inplace(ctx, dst)


def _addsub_inplace(ctx, a, b, op):
    """a <- a op b; the result has max(size) polynomials (cahel-main/src/evaluate.cu:42-110,199-260)"""
    _same_level(a, b)
    L = ctx.size_l(a.chain_index)
    fn = ctx.lb.add if op == "add" else ctx.lb.sub
    k = min(a.size, b.size)
    if a.size >= b.size:
        head = a.data[:k]
        fn(L, head, b.data[:k].contiguous(), out=head)
    else:
        new = b.data.clone() if op == "add" else ctx.lb.negate(L, b.data)
        fn(L, a.data, b.data[:k].contiguous(), out=new[:k])
        a.data, a.size = new, b.size


def add_inplace(ctx, a, b):
    _addsub_inplace(ctx, a, b, "add")


def add(ctx, a, b, dst):
    if dst is b and dst is not a:
        add_inplace(ctx, dst, a)
        return
    if dst is not a:
        dst._assign(a)
    add_inplace(ctx, dst, b)


def sub_inplace(ctx, a, b):
    _addsub_inplace(ctx, a, b, "sub")


def sub(ctx, a, b, dst):
    """dst = a - b (cahel-main/include/evaluate.h:52-61)"""
    if dst is b and dst is not a:
        tmp = a.copy()
        sub_inplace(ctx, tmp, b)
        dst._assign(tmp)
        return
    if dst is not a:
        dst._assign(a)
    sub_inplace(ctx, dst, b)


def add_many(ctx, cts, dst):
    if not cts:
        raise ValueError("encrypteds cannot be empty")
    acc = cts[0].copy()
    for c in cts[1:]:
        add_inplace(ctx, acc, c)
    dst._assign(acc)


def _plain_check(ct, pt):
    if ct.chain_index != pt.chain_index:
        raise ValueError("encrypted and plain parameter mismatch")
    if not pt.is_ntt_form:
        raise ValueError("plain must be in NTT form")


def add_plain_inplace(ctx, ct, pt):
    _plain_check(ct, pt)
    if not _same_scale(ct.scale, pt.scale):
        raise ValueError("scale mismatch")
    L = ctx.size_l(ct.chain_index)
    c0 = ct.data[0]
    ctx.lb.add(L, c0, pt.data, out=c0)


def add_plain(ctx, ct, pt, dst):
    dst._assign(ct)
    add_plain_inplace(ctx, dst, pt)


def sub_plain_inplace(ctx, ct, pt):
    _plain_check(ct, pt)
    if not _same_scale(ct.scale, pt.scale):
        raise ValueError("scale mismatch")
    L = ctx.size_l(ct.chain_index)
    c0 = ct.data[0]
    ctx.lb.sub(L, c0, pt.data, out=c0)


def sub_plain(ctx, ct, pt, dst):
    dst._assign(ct)
    sub_plain_inplace(ctx, dst, pt)


def multiply_plain_inplace(ctx, ct, pt):
    _plain_check(ct, pt)
    L = ctx.size_l(ct.chain_index)
    _check_scale(ctx, ct.scale * pt.scale, ct.chain_index)
    for p in range(ct.size):
        cp = ct.data[p]
        ctx.lb.multiply_poly(L, cp, pt.data, out=cp)
    ct.scale *= pt.scale


def multiply_plain(ctx, ct, pt, dst):
    dst._assign(ct)
    multiply_plain_inplace(ctx, dst, pt)


def multiply_inplace(ctx, a, b):
    """ckks_multiply (cahel-main/src/evaluate.cu:447-500) for two size-2 ciphertexts"""
    if a.chain_index != b.chain_index:
        raise ValueError("encrypted1 and encrypted2 parameter mismatch")
    if not (a.is_ntt_form and b.is_ntt_form):
        raise ValueError("encrypted1 or encrypted2 must be in NTT form")
    if a.size != 2 or b.size != 2:
        raise ValueError("only size-2 ciphertexts can be multiplied on this path")
    _check_scale(ctx, a.scale * b.scale, a.chain_index)
    L = ctx.size_l(a.chain_index)
    a.data = ctx.lb.multiply(L, a.data.contiguous(), b.data.contiguous())
    a.size = 3
    a.scale *= b.scale


def multiply(ctx, a, b, dst):
    if dst is b and dst is not a:
        multiply_inplace(ctx, dst, a)
        return
    if dst is not a:
        dst._assign(a)
    multiply_inplace(ctx, dst, b)


def square_inplace(ctx, ct):
    if ct.size != 2:
        raise ValueError("only size-2 ciphertexts can be squared on this path")
    _check_scale(ctx, ct.scale * ct.scale, ct.chain_index)
    L = ctx.size_l(ct.chain_index)
    ct.data = ctx.lb.square(L, ct.data.contiguous())
    ct.size = 3
    ct.scale *= ct.scale


def square(ctx, ct, dst):
    dst._assign(ct)
    square_inplace(ctx, dst)


def relinearize_inplace(ctx, ct, rlk):
    """cahel-main/src/evaluate.cu:2019-2056"""
    if ct.size != 3:
        raise ValueError("destination_size must be 3")
    if not ct.is_ntt_form:
        raise ValueError("CKKS encrypted must be in NTT form")
    if rlk.data is None:
        raise ValueError("relin_keys is not valid for encryption parameters")
    L = ctx.size_l(ct.chain_index)
    ct.data = ctx.lb.relinearize(L, ct.data.contiguous(), rlk.data).clone()
    ct.size = 2


def relinearize(ctx, ct, rlk, dst):
    dst._assign(ct)
    relinearize_inplace(ctx, dst, rlk)


def multiply_and_relin_inplace(ctx, a, b, rlk):
    multiply_inplace(ctx, a, b)
    relinearize_inplace(ctx, a, rlk)


def rescale_to_next_inplace(ctx, ct):
    """cahel-main/src/evaluate.cu:2059,2307-2361: floor-divide by the last prime, scale /= q_last"""
    if not ct.is_ntt_form:
        raise ValueError("CKKS encrypted must be in NTT form")
    if ct.chain_index >= ctx.max_chain:
        raise ValueError("end of modulus switching chain reached")
    L = ctx.size_l(ct.chain_index)
    ct.data = ctx.lb.rescale(L, ct.data.contiguous())
    ct.scale = ct.scale / float(ctx.moduli[L - 1])
    ct.chain_index += 1


def rescale_to_next(ctx, ct, dst):
    dst._assign(ct)
    rescale_to_next_inplace(ctx, dst)


def mod_switch_to_next_inplace(ctx, obj):
    """mod_switch_drop_to_next (cahel-main/src/evaluate.cu:2253-2300): drop the last prime"""
    if obj.chain_index >= ctx.max_chain:
        raise ValueError("end of modulus switching chain reached")
    L = ctx.size_l(obj.chain_index)
    if isinstance(obj, plaintext):
        obj.data = obj.data[: L - 1].contiguous()
    else:
        obj.data = ctx.lb.mod_switch_drop(L, obj.data.contiguous())
    obj.chain_index += 1


def mod_switch_to_next(ctx, obj, dst):
    if isinstance(obj, plaintext):
        dst.data, dst.chain_index, dst.scale = obj.data.clone(), obj.chain_index, obj.scale
    else:
        dst._assign(obj)
    mod_switch_to_next_inplace(ctx, dst)


def mod_switch_to_inplace(ctx, obj, chain_index):
    """cahel-main/src/evaluate.cu:2200-2250"""
    if obj.chain_index > chain_index:
        raise ValueError("cannot switch to higher level modulus")
    while obj.chain_index < chain_index:
        mod_switch_to_next_inplace(ctx, obj)


def mod_switch_to(ctx, obj, dst, chain_index):
    if isinstance(obj, plaintext):
        dst.data, dst.chain_index, dst.scale = obj.data.clone(), obj.chain_index, obj.scale
    else:
        dst._assign(obj)
    mod_switch_to_inplace(ctx, dst, chain_index)


def _naf(value):
    """non-adjacent form, least significant term first, which is also the order rotate_internal applies the terms in
    (cahel-main/include/util/numth.h:18-35, src/evaluate.cu:2396-2407): 5 -> [1, 4], 6 -> [-2, 8], 3 -> [-1, 4]"""
    res = []
    sign = value < 0
    value = abs(value)
    i = 0
    while value:
        zi = 2 - (value & 3) if value & 1 else 0
        value = (value - zi) >> 1
        if zi:
            res.append((-zi if sign else zi) * (1 << i))
        i += 1
    return res


def apply_galois_inplace(ctx, ct, galois_elt_index, glk):
    """cahel-main/src/evaluate.cu:2631-2686"""
    if ct.size > 2:
        raise ValueError("encrypted size must be 2")
    if galois_elt_index < 0 or galois_elt_index >= len(glk.keys):
        raise RuntimeError("Galois key not present")
    L = ctx.size_l(ct.chain_index)
    ct.data = ctx.lb.rotate(L, ct.data.contiguous(), galois_elt_index, glk.keys[galois_elt_index])


def apply_galois(ctx, ct, galois_elt_index, glk, dst):
    dst._assign(ct)
    apply_galois_inplace(ctx, dst, galois_elt_index, glk)


def rotate_vector_inplace(ctx, ct, step, glk):
    """rotate_internal (cahel-main/src/evaluate.cu:2364-2410): direct key or NAF decomposition"""
    if step == 0:
        return
    if abs(step) >= ctx.N // 2:
        raise ValueError("step count too large")
    idx = ctx.elt_index(get_elts_from_steps([step], ctx.N)[0])
    if idx >= 0:
        apply_galois_inplace(ctx, ct, idx, glk)
        return
    parts = _naf(step)
    if len(parts) == 1:
        raise ValueError("Galois key not present")
    for s in parts:
        if abs(s) != ctx.N // 2:
            rotate_vector_inplace(ctx, ct, s, glk)


def rotate_vector(ctx, ct, step, glk, dst):
    """dst = rot(ct, step) (cahel-main/include/evaluate.h:566-574)"""
    dst._assign(ct)
    rotate_vector_inplace(ctx, dst, step, glk)


def complex_conjugate_inplace(ctx, ct, glk):
    idx = ctx.elt_index(2 * ctx.N - 1)
    if idx < 0:
        raise RuntimeError("Galois key not present")
    apply_galois_inplace(ctx, ct, idx, glk)


def complex_conjugate(ctx, ct, glk, dst):
    dst._assign(ct)
    complex_conjugate_inplace(ctx, dst, glk)


def hoisting_inplace(ctx, ct, glk, steps):
    """cahel-main/src/evaluate.cu:2412-2629: ct <- sum over steps of rot(ct, step), one mod-up"""
    if ct.size > 2:
        raise ValueError("ciphertext size must be 2")
    elts = get_elts_from_steps(list(steps), ctx.N)
    idx = [ctx.elt_index(e) for e in elts]
    if any(i < 0 for i in idx):
        raise RuntimeError("Galois key not present in hoisting")
    L = ctx.size_l(ct.chain_index)
    data = ct.data.contiguous()
    # one mod-up and one mod-down for the whole list, as in the reference; the C ABI takes up to 32 steps
    # (the Krum driver uses 15), and splitting a longer list would round in a different place
    if len(idx) > 32:
        raise ValueError("hoisting takes at most 32 rotation steps per call")
    out = ctx.lb.hoisting(L, data.clone(), idx, [glk.keys[i] for i in idx])
    ct.data = out


def hoisting(ctx, ct, glk, steps):
    """returns the rotated sum as a new ciphertext (cahel-main/include/evaluate.h:449-455)"""
    dst = ct.copy()
    hoisting_inplace(ctx, dst, glk, steps)
    return dst


def _unsupported(*a, **k):
    raise ValueError("unsupported scheme")


# BFV/BGV-only entry points of the reference module
multiply_many = exponentiate = exponentiate_inplace = _unsupported
rotate_rows = rotate_rows_inplace = rotate_columns = rotate_columns_inplace = _unsupported
