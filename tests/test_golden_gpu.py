"""The CUDA library replays the chain recorded from the reference library itself
(tests/golden/ref_fixture.json) and must hash identically at every stage."""
import numpy as np
import pytest

from golden_replay import CASES, load_fixture, moduli_of, replay

pytestmark = pytest.mark.gpu


class CudaOps:
    """Adapter: the oracle's method names, executed by the C-ABI library on the GPU."""

    def __init__(self, ctx):
        import torch

        from lancelot_b200 import cabi

        self.ctx, self.cabi, self.torch = ctx, cabi, torch
        self.N = ctx.N

    def _d(self, a):
        return self.cabi.to_device(np.ascontiguousarray(a))

    def _h(self, t):
        return self.cabi.to_host(t)

    def gen_sk(self, seed):
        return self._h(self.ctx.gen_secret_key(seed))

    def gen_pk(self, sk, se, sa):
        return self._h(self.ctx.gen_public_key(self._d(sk), se, sa))

    def sk_square(self, sk):
        # s^2 over the full key modulus (QP limb order = table order at the key level)
        return self._h(self.ctx.multiply_poly_qp(self._d(sk), self._d(sk)))

    def galois(self, e, data):
        return self._h(self.ctx.galois_permute(e, self._d(data)))

    def gen_ksk(self, sk, skp, seeds):
        return self._h(self.ctx.gen_switch_key(self._d(sk), self._d(skp), seeds))

    def encode(self, L, values, scale):
        v = self.torch.from_numpy(np.ascontiguousarray(values, dtype=np.float64)).cuda()
        pt = self.ctx.encode(L, v, scale, sparse_slots=self.N // 2)
        self.ctx.check_status()
        return self._h(pt)

    def encrypt_asym(self, pk, pt, su, se):
        return self._h(self.ctx.encrypt_asymmetric(self._d(pk), self._d(pt), np.concatenate([su, se])))

    def poly_op(self, op, L, a, b):
        fn = {"sub": self.ctx.sub, "add": self.ctx.add}[op]
        return self._h(fn(L, self._d(a), self._d(b)))

    def tensor(self, L, a, b):
        return self._h(self.ctx.multiply(L, self._d(a), self._d(b)))

    def square(self, L, a):
        return self._h(self.ctx.square(L, self._d(a)))

    def relinearize(self, L, ct3, rlk):
        return self._h(self.ctx.relinearize(L, self._d(ct3), self._d(rlk)).contiguous())

    def rescale(self, L, ct):
        return self._h(self.ctx.rescale(L, self._d(ct)))

    def rotate(self, L, ct, e, glk):
        return self._h(self.ctx.rotate(L, self._d(ct), e, self._d(glk)))

    def hoisting(self, L, ct, idx, glks):
        return self._h(self.ctx.hoisting(L, self._d(ct), idx, [self._d(g) for g in glks]))

    def drop_last(self, L, ct):
        return self._h(self.ctx.mod_switch_drop(L, self._d(ct)))

    def decrypt(self, L, ct, sk):
        return self._h(self.ctx.decrypt(L, self._d(ct), self._d(sk)))

    def decode(self, L, pt, scale, slots):
        return self.ctx.decode(L, self._d(pt), scale, slots).cpu().numpy()


@pytest.mark.parametrize("case", sorted(CASES))
def test_cuda_library_reproduces_reference_digests(case):
    import torch

    if not torch.cuda.is_available():
        pytest.fail("GPU tests need a CUDA device; there is no CPU fallback")
    from lancelot_b200 import cabi

    fix = load_fixture()[case]
    cfg = CASES[case]
    mods = moduli_of(case, fix, cabi.coeff_modulus_create)
    elts = [int(x) for x in fix["galois_elts"]["head"]]
    ctx = cabi.Context(cfg["logn"], mods, cfg["size_p"], elts)
    report = replay(case, fix, CudaOps(ctx))
    bad = [name for name, ok in report if not ok]
    assert not bad, "stages that differ from the reference: %s" % bad
