"""Thin typed wrapper over the C ABI (include/lancelot_b200.h).

Device buffers are ``torch`` tensors of dtype ``int64`` on a CUDA device, holding the
bit patterns of the ``uint64`` residues; torch only provides the memory and the stream.
Every method forwards to exactly one ``lb_*`` entry point.
"""
import ctypes as C

import numpy as np
import torch

from ._lib import check, lib

_u64p = C.POINTER(C.c_uint64)


def _p(t):
    """Device pointer of a CUDA int64 tensor (or None)."""
    if t is None:
        return None
    assert t.is_cuda and t.dtype == torch.int64 and t.is_contiguous(), "need a contiguous CUDA int64 tensor"
    return C.c_void_p(t.data_ptr())


def to_device(a, device="cuda"):
    """numpy uint64 array -> CUDA int64 tensor with the same bits."""
    a = np.ascontiguousarray(a, dtype=np.uint64)
    return torch.from_numpy(a.view(np.int64)).to(device)


def to_host(t):
    """CUDA int64 tensor -> numpy uint64 array with the same bits."""
    return t.detach().cpu().numpy().view(np.uint64)


def coeff_modulus_create(n, bit_sizes):
    k = len(bit_sizes)
    out = (C.c_uint64 * k)()
    check(lib.lb_coeff_modulus_create(C.c_uint64(n), (C.c_int * k)(*bit_sizes), k, out))
    return [int(x) for x in out]


def galois_elts_from_steps(steps, n):
    k = len(steps)
    out = (C.c_uint32 * max(k, 1))()
    check(lib.lb_galois_elts_from_steps((C.c_int * max(k, 1))(*steps), k, C.c_uint64(n), out))
    return [int(out[i]) for i in range(k)]


class Context:
    """Owns one ``lb_context`` (tables on the device, scratch)."""

    def __init__(self, log_n, moduli, special_modulus_size, galois_elts=(), check_tc128=False, device=0):
        self.log_n, self.N = log_n, 1 << log_n
        self.moduli = [int(m) for m in moduli]
        self.size_QP = len(self.moduli)
        self.size_P = special_modulus_size
        self.size_Q = self.size_QP - self.size_P
        self.galois_elts = [int(e) for e in galois_elts]
        self.device = device
        m = (C.c_uint64 * self.size_QP)(*self.moduli)
        ne = len(self.galois_elts)
        e = (C.c_uint32 * max(ne, 1))(*self.galois_elts)
        h = C.c_void_p()
        check(lib.lb_context_create(log_n, m, self.size_QP, special_modulus_size, e, ne, int(check_tc128), device,
                                    C.byref(h)))
        self.h = h

    def close(self):
        if getattr(self, "h", None):
            lib.lb_context_destroy(self.h)
            self.h = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    def _stream(self):
        """the current torch stream of THIS context's device (not of whatever device is current)"""
        return C.c_void_p(torch.cuda.current_stream(self.device).cuda_stream)

    def reserve_workspace(self, nbytes):
        check(lib.lb_context_reserve_workspace(self.h, C.c_size_t(int(nbytes))))

    def beta(self, size_l):
        return (size_l + self.size_P - 1) // self.size_P

    def empty(self, *shape):
        return torch.empty(shape, dtype=torch.int64, device="cuda:%d" % self.device)

    def root(self, i):
        out = C.c_uint64()
        check(lib.lb_context_get_root(self.h, i, C.byref(out)))
        return int(out.value)

    def galois_table(self, i):
        out = np.empty(self.N, dtype=np.uint32)
        check(lib.lb_context_get_galois_table(self.h, i, out.ctypes.data_as(C.POINTER(C.c_uint32))))
        return out

    def butterfly_rate(self, variant=-1):
        """register-only butterfly rate; variant 0..3 (integer strict / lazy, FP64 pipe at a 50-bit / 40-bit prime), -1: the first prime's"""
        out = C.c_double()
        check(lib.lb_probe_butterfly_rate(self.h, int(variant), C.byref(out)))
        return float(out.value)

    # -- transforms
    def ntt_forward(self, data, n_groups, size_l, size_p):
        check(lib.lb_ntt_forward(self.h, _p(data), n_groups, size_l, size_p, self._stream()))

    def ntt_inverse(self, data, n_groups, size_l, size_p):
        check(lib.lb_ntt_inverse(self.h, _p(data), n_groups, size_l, size_p, self._stream()))

    # -- element-wise
    def add(self, size_l, a, b, out=None):
        out = torch.empty_like(a) if out is None else out
        check(lib.lb_add(self.h, size_l, a.numel() // (size_l * self.N), _p(a), _p(b), _p(out), self._stream()))
        return out

    def sub(self, size_l, a, b, out=None):
        out = torch.empty_like(a) if out is None else out
        check(lib.lb_sub(self.h, size_l, a.numel() // (size_l * self.N), _p(a), _p(b), _p(out), self._stream()))
        return out

    def multiply_poly(self, size_l, a, b, out=None):
        out = torch.empty_like(a) if out is None else out
        check(lib.lb_multiply_poly(self.h, size_l, a.numel() // (size_l * self.N), _p(a), _p(b), _p(out), self._stream()))
        return out

    def multiply_poly_qp(self, a, b):
        """element-wise product over the key-level limb list Q || P (used for s^2)"""
        out = torch.empty_like(a)
        check(lib.lb_multiply_poly_key_level(self.h, _p(a), _p(b), _p(out), self._stream()))
        return out

    def negate(self, size_l, a, out=None):
        out = torch.empty_like(a) if out is None else out
        check(lib.lb_negate(self.h, size_l, a.numel() // (size_l * self.N), _p(a), _p(out), self._stream()))
        return out

    def reduce_mod(self, size_l, a, out=None):
        """a mod q per limb for arbitrary 64-bit words (in place unless ``out`` is given)"""
        out = a if out is None else out
        check(lib.lb_reduce_mod(self.h, size_l, a.numel() // (size_l * self.N), _p(a), _p(out), self._stream()))
        return out

    def multiply(self, size_l, a, b, batch=1):
        out = self.empty(batch, 3, size_l, self.N) if batch > 1 else self.empty(3, size_l, self.N)
        check(lib.lb_multiply(self.h, size_l, batch, _p(a), _p(b), _p(out), self._stream()))
        return out

    def square(self, size_l, a, batch=1):
        out = self.empty(batch, 3, size_l, self.N) if batch > 1 else self.empty(3, size_l, self.N)
        check(lib.lb_square(self.h, size_l, batch, _p(a), _p(out), self._stream()))
        return out

    def mod_switch_drop(self, size_l, ct):
        n_polys = ct.numel() // (size_l * self.N)
        out = self.empty(n_polys, size_l - 1, self.N)
        check(lib.lb_mod_switch_drop(self.h, size_l, n_polys, _p(ct), _p(out), self._stream()))
        return out

    def galois_permute(self, elt_index, data):
        out = torch.empty_like(data)
        check(lib.lb_galois_permute(self.h, elt_index, data.numel() // self.N, _p(data), _p(out), self._stream()))
        return out

    # -- key switching
    def modup(self, size_l, cks):
        out = self.empty(self.beta(size_l), size_l + self.size_P, self.N)
        check(lib.lb_modup(self.h, size_l, _p(cks), _p(out), self._stream()))
        return out

    def inner_product(self, size_l, digits, evk):
        out = self.empty(2, size_l + self.size_P, self.N)
        check(lib.lb_keyswitch_inner_product(self.h, size_l, _p(digits), _p(evk), _p(out), self._stream()))
        return out

    def moddown(self, size_l, cx):
        out = self.empty(size_l, self.N)
        check(lib.lb_moddown(self.h, size_l, _p(cx), _p(out), self._stream()))
        return out

    def keyswitch(self, size_l, ct, cks, evk):
        check(lib.lb_keyswitch(self.h, size_l, _p(ct), _p(cks), _p(evk), self._stream()))
        return ct

    def relinearize(self, size_l, ct3, rlk):
        check(lib.lb_relinearize(self.h, size_l, _p(ct3), _p(rlk), self._stream()))
        return ct3[:2]

    def rescale(self, size_l, ct):
        n_polys = ct.numel() // (size_l * self.N)
        out = self.empty(n_polys, size_l - 1, self.N)
        check(lib.lb_rescale(self.h, size_l, n_polys, _p(ct), _p(out), self._stream()))
        return out

    def rescale_strided(self, size_l, ct, batch, polys_per_ct, ct_stride):
        out = self.empty(batch, polys_per_ct, size_l - 1, self.N)
        check(lib.lb_rescale_strided(self.h, size_l, batch, polys_per_ct, _p(ct), C.c_size_t(ct_stride), _p(out), self._stream()))
        return out

    def rotate(self, size_l, ct, elt_index, glk):
        check(lib.lb_rotate(self.h, size_l, _p(ct), elt_index, _p(glk), self._stream()))
        return ct

    def hoisting(self, size_l, ct, elt_indices, glks):
        n = len(elt_indices)
        idx = (C.c_int * n)(*elt_indices)
        ptrs = (C.c_void_p * n)(*[g.data_ptr() for g in glks])
        check(lib.lb_hoisting(self.h, size_l, _p(ct), n, idx, ptrs, self._stream()))
        return ct

    def relinearize_batch(self, size_l, ct3, rlk):
        """ct3: [batch][3][size_l][N]; the first two polynomials of each hold the result"""
        batch = ct3.numel() // (3 * size_l * self.N)
        check(lib.lb_relinearize_batch(self.h, size_l, batch, _p(ct3), _p(rlk), self._stream()))
        return ct3

    def rotate_batch(self, size_l, ct, elt_index, glk):
        batch = ct.numel() // (2 * size_l * self.N)
        check(lib.lb_rotate_batch(self.h, size_l, batch, _p(ct), elt_index, _p(glk), self._stream()))
        return ct

    def hoisting_batch(self, size_l, ct, elt_indices, glks):
        batch = ct.numel() // (2 * size_l * self.N)
        n = len(elt_indices)
        idx = (C.c_int * n)(*elt_indices)
        ptrs = (C.c_void_p * n)(*[g.data_ptr() for g in glks])
        check(lib.lb_hoisting_batch(self.h, size_l, batch, _p(ct), n, idx, ptrs, self._stream()))
        return ct

    def sum_groups(self, size_l, n_polys, items, groups):
        """items: [n_items][n_polys][size_l][N]; groups: list of index lists -> [len(groups)][n_polys][size_l][N] sums"""
        offsets = [0]
        for g in groups:
            offsets.append(offsets[-1] + len(g))
        flat = [int(i) for g in groups for i in g]
        n_items = items.numel() // (n_polys * size_l * self.N)
        out = self.empty(len(groups), n_polys, size_l, self.N)
        off = (C.c_int * len(offsets))(*offsets)
        idx = (C.c_int * max(1, len(flat)))(*flat)
        check(lib.lb_sum_groups(self.h, size_l, n_polys, len(groups), off, idx, n_items, _p(items), _p(out), self._stream()))
        return out

    def krum_accumulate(self, size_l, a, b, acc, accumulate=False, n_chunks=None, stride_a=None, stride_b=None):
        ct_words = 2 * size_l * self.N
        n_chunks = a.numel() // ct_words if n_chunks is None else n_chunks
        stride_a = ct_words if stride_a is None else stride_a
        stride_b = ct_words if stride_b is None else stride_b
        check(lib.lb_krum_accumulate(self.h, size_l, n_chunks, _p(a), _p(b), C.c_size_t(stride_a), C.c_size_t(stride_b),
                                     _p(acc), int(accumulate), self._stream()))
        return acc

    def krum_accumulate_tile(self, size_l, a, b, outs, n_chunks=None):
        """a, b: lists of client tensors [chunks][2][size_l][N] (b empty: all pairs inside a); outs: one
        [3][size_l][N] tensor per pair, triangle order (0,1),(0,2),..,(1,2),.. or rectangle order i * len(b) + j"""
        ct_words = 2 * size_l * self.N
        n_chunks = a[0].numel() // ct_words if n_chunks is None else n_chunks
        pa = (C.c_void_p * len(a))(*[t.data_ptr() for t in a])
        pb = (C.c_void_p * max(1, len(b)))(*[t.data_ptr() for t in b])
        po = (C.c_void_p * len(outs))(*[t.data_ptr() for t in outs])
        n_pairs = len(a) * len(b) if b else len(a) * (len(a) - 1) // 2
        assert len(outs) == n_pairs, "one output per pair"
        check(lib.lb_krum_accumulate_tile(self.h, size_l, n_chunks, len(a), pa, len(b), pb, C.c_size_t(ct_words), po, self._stream()))
        return outs

    def krum_pair_sums(self, size_l, cts, n_clients, pairs, out):
        """cts: client -> [chunks][2][size_l][N] (dict, list or tensor indexed by client; clients in no pair may be
        missing); pairs: list of (i, j), i < j; out: [>= len(pairs)][3][size_l][N], pair p's sums at out[p]"""
        ct_words = 2 * size_l * self.N
        used = sorted({c for p in pairs for c in p})
        n_chunks = cts[used[0]].numel() // ct_words if used else 0
        ptrs = (C.c_void_p * max(1, n_clients))()
        for c in used:
            ptrs[c] = cts[c].data_ptr()
        flat = (C.c_int * max(1, 2 * len(pairs)))(*[int(x) for p in pairs for x in p])
        check(lib.lb_krum_pair_sums(self.h, size_l, n_clients, ptrs, n_chunks, C.c_size_t(ct_words), len(pairs), flat, _p(out),
                                    self._stream()))
        return out

    def krum_scores(self, size_l, acc, rlk, first_elts, first_keys, pow_elts, pow_keys):
        """acc [P][3][size_l][N] (overwritten) -> scores [P][2][size_l-1][N]: relinearize, rescale, hoisted rotations
        by first_elts added, then rotate + add for every element of pow_elts in order"""
        n_pairs = acc.numel() // (3 * size_l * self.N)
        scores = self.empty(n_pairs, 2, size_l - 1, self.N)
        nf, npw = len(first_elts), len(pow_elts)
        fe = (C.c_int * max(1, nf))(*first_elts)
        fk = (C.c_void_p * max(1, nf))(*[g.data_ptr() for g in first_keys])
        pe = (C.c_int * max(1, npw))(*pow_elts)
        pk = (C.c_void_p * max(1, npw))(*[g.data_ptr() for g in pow_keys])
        check(lib.lb_krum_scores(self.h, size_l, n_pairs, _p(acc), _p(rlk), nf, fe, fk, npw, pe, pk, _p(scores), self._stream()))
        return scores

    def decrypt(self, size_l, ct, sk):
        n_polys = ct.numel() // (size_l * self.N)
        pt = self.empty(size_l, self.N)
        check(lib.lb_decrypt(self.h, size_l, n_polys, _p(ct), _p(sk), _p(pt), self._stream()))
        return pt

    # -- samplers, keys, encryption (seeds are host bytes; 64 per seed)
    @staticmethod
    def _seed(seed, count=1):
        s = np.ascontiguousarray(seed, dtype=np.uint8).reshape(-1)
        assert s.size == 64 * count, "need %d seeds of 64 bytes" % count
        return s, s.ctypes.data_as(C.POINTER(C.c_uint8))

    def sample(self, kind, seed, size_l, size_p):
        s, sp = self._seed(seed)
        out = self.empty(size_l + size_p, self.N)
        fn = {"ternary": lib.lb_sample_ternary, "error": lib.lb_sample_error, "uniform": lib.lb_sample_uniform}[kind]
        check(fn(self.h, sp, size_l, size_p, _p(out), self._stream()))
        return out

    def gen_secret_key(self, seed):
        s, sp = self._seed(seed)
        sk = self.empty(self.size_QP, self.N)
        check(lib.lb_gen_secret_key(self.h, sp, _p(sk), self._stream()))
        return sk

    def gen_public_key(self, sk, seed_error, seed_uniform):
        se, pe = self._seed(seed_error)
        su, pu = self._seed(seed_uniform)
        pk = self.empty(2, self.size_QP, self.N)
        check(lib.lb_gen_public_key(self.h, _p(sk), pe, pu, _p(pk), self._stream()))
        return pk

    def gen_switch_key(self, sk, sk_target, seeds):
        dnum = self.size_Q // self.size_P
        s, sp = self._seed(seeds, 2 * dnum)
        out = self.empty(dnum, 2, self.size_QP, self.N)
        check(lib.lb_gen_switch_key(self.h, _p(sk), _p(sk_target), sp, _p(out), self._stream()))
        return out

    def gen_galois_keys(self, sk, elt_indices, seeds, out=None):
        """switch keys of several Galois elements in one call -> [n][dnum][2][size_QP][N]; seeds: 2 dnum per key"""
        dnum = self.size_Q // self.size_P
        n = len(elt_indices)
        s, sp = self._seed(seeds, 2 * dnum * n)
        if out is None:
            out = self.empty(n, dnum, 2, self.size_QP, self.N)
        idx = (C.c_int * max(1, n))(*[int(e) for e in elt_indices])
        check(lib.lb_gen_galois_keys(self.h, _p(sk), n, idx, sp, _p(out), self._stream()))
        return out

    def encrypt_asymmetric(self, pk, pt, seeds, batch=1, out=None):
        s, sp = self._seed(seeds, 2 * batch)
        if out is not None:
            ct = out
        else:
            ct = self.empty(batch, 2, self.size_Q, self.N) if batch > 1 else self.empty(2, self.size_Q, self.N)
        check(lib.lb_encrypt_asymmetric(self.h, _p(pk), _p(pt), sp, batch, _p(ct), self._stream()))
        return ct

    # -- encoder
    def encode(self, size_l, values, scale, sparse_slots=None, batch=1, n_values=None, value_stride=None):
        """values: CUDA tensor float64 / float32 (real) or complex128, shape [batch, n] or [n]."""
        dt = {torch.float64: 0, torch.float32: 1, torch.complex128: 2}[values.dtype]
        assert values.is_cuda and values.is_contiguous()
        n = values.shape[-1] if n_values is None else n_values
        stride = values.shape[-1] if value_stride is None else value_stride
        if sparse_slots is None:
            sparse_slots = 1 << max(1, int(np.ceil(np.log2(max(n, 2)))))
        pt = self.empty(batch, size_l, self.N) if batch > 1 else self.empty(size_l, self.N)
        check(lib.lb_encode(self.h, size_l, C.c_void_p(values.data_ptr()), dt, C.c_size_t(stride), n, sparse_slots, batch,
                            C.c_double(scale), _p(pt), self._stream()))
        return pt

    def encode_encrypt(self, pk, values, scale, seeds, sparse_slots, batch=1, out=None):
        """fused encode + public-key encryption of a batch of messages [batch][n]"""
        dt = {torch.float64: 0, torch.float32: 1, torch.complex128: 2}[values.dtype]
        assert values.is_cuda and values.is_contiguous()
        s, sp = self._seed(seeds, 2 * batch)
        ct = out if out is not None else self.empty(batch, 2, self.size_Q, self.N)
        check(lib.lb_encode_encrypt(self.h, _p(pk), C.c_void_p(values.data_ptr()), dt, C.c_size_t(values.shape[-1]), values.shape[-1],
                                    sparse_slots, batch, C.c_double(scale), sp, _p(ct), self._stream()))
        return ct

    def decode(self, size_l, pt, scale, sparse_slots):
        out = torch.empty(sparse_slots, dtype=torch.complex128, device=pt.device)
        check(lib.lb_decode(self.h, size_l, _p(pt), C.c_double(scale), sparse_slots, C.c_void_p(out.data_ptr()), self._stream()))
        return out

    def decode_batch(self, size_l, pts, scale, sparse_slots, batch):
        out = torch.empty(batch, sparse_slots, dtype=torch.complex128, device=pts.device)
        check(lib.lb_decode_batch(self.h, size_l, batch, _p(pts), C.c_double(scale), sparse_slots, C.c_void_p(out.data_ptr()), self._stream()))
        return out

    def decrypt_batch(self, size_l, cts, sk, n_polys, batch):
        pt = self.empty(batch, size_l, self.N)
        check(lib.lb_decrypt_batch(self.h, size_l, n_polys, batch, _p(cts), _p(sk), _p(pt), self._stream()))
        return pt

    def mask_accumulate(self, size_l, client_cts, masks, n_chunks):
        """client_cts: list of [chunks][2][size_l][N] tensors; masks [n_clients][2][size_l][N] -> [chunks][3][size_l][N]"""
        n = len(client_cts)
        ptrs = (C.c_void_p * n)(*[t.data_ptr() for t in client_cts])
        out = self.empty(n_chunks, 3, size_l, self.N)
        check(lib.lb_mask_accumulate(self.h, size_l, n, n_chunks, ptrs, C.c_size_t(2 * size_l * self.N), _p(masks), _p(out), self._stream()))
        return out

    def check_status(self):
        check(lib.lb_check_status(self.h, self._stream()))


# -- benchmark diagnostics (include/lancelot_b200_diag.h); not part of the drop-in boundary
def launch_count():
    """kernels this library has launched in this process"""
    lib.lb_launch_count.restype = C.c_ulonglong
    return int(lib.lb_launch_count())


def kernel_timing(enable=True):
    """start (and clear) or stop the per-kernel device timer"""
    check(lib.lb_diag_kernel_timing(int(bool(enable))))


def kernel_report():
    """{kernel name: {"launches", "ms", "bytes"}} since the timer was started; synchronises and clears the record"""
    import json

    buf = C.create_string_buffer(1 << 16)
    check(lib.lb_diag_kernel_report(buf, C.c_size_t(len(buf))))
    out = json.loads(buf.value.decode())
    overflow = out.pop("_overflow", False)
    if overflow:
        raise RuntimeError("more launches than the kernel timer records")
    return out
