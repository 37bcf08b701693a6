"""The pyCAHEL extension module (lancelot_b200/pybind, bound from include/cahel_b200.hpp with the names of
cahel-main/python/src/binding.cu) on a GPU: Lancelot's own call sequences through it, its ciphertext bytes against
the Python mirror's under the same seeds, and - when a checkout of the reference is at hand - the reference's
unmodified Krum driver running on top of it.  Needs a B200; run with -m gpu."""
import io
import os
import sys

import numpy as np
import pytest

pytestmark = pytest.mark.gpu

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
MODULE_DIR = os.path.join(ROOT, "lancelot_b200", "pybind")


@pytest.fixture(scope="module")
def cahel():
    import torch

    if not torch.cuda.is_available():
        pytest.fail("GPU tests need a CUDA device; there is no CPU fallback")
    if MODULE_DIR not in sys.path:
        sys.path.insert(0, MODULE_DIR)
    try:
        import pyCAHEL
    except ImportError as e:
        pytest.fail("pyCAHEL is not built (python lancelot_b200/pybind/build.py): %s" % e)
    return pyCAHEL


def _setup(cahel, n, steps):
    params = cahel.params(cahel.scheme_type.ckks)
    params.set_poly_modulus_degree(n)
    params.set_coeff_modulus(cahel.coeff_modulus_create(n, [60, 40, 40, 60]))
    params.set_special_modulus_size(1)
    params.set_galois_elts(cahel.get_elts_from_steps(steps, n))
    context = cahel.context(params, True, cahel.sec_level_type.tc128)
    sk = cahel.secret_key(params)
    sk.gen_secretkey(context)
    pk = cahel.public_key(context)
    sk.gen_publickey(context, pk)
    rlk = cahel.relin_key(context)
    sk.gen_relinkey(context, rlk)
    glk = cahel.galois_key(context)
    sk.create_galois_keys(context, glk)
    return params, context, sk, pk, rlk, glk, cahel.ckks_encoder(context)


def test_lancelot_smoke_sequence_on_the_module(cahel):
    """the calls of lancelot-main-GPU/ckks.py:14-57: encode, encrypt, multiply, relinearize, rescale, rotate, decrypt"""
    n = 8192
    params, context, sk, pk, rlk, glk, encoder = _setup(cahel, n, [1, 2, 3])
    slots = encoder.slot_count()
    assert slots == n // 2
    rng = np.random.default_rng(0)
    x, y = rng.uniform(-1, 1, slots), rng.uniform(-1, 1, slots)
    scale = 2.0 ** 40
    cx = pk.encrypt_asymmetric(context, encoder.encode(context, list(x), scale))
    cy = pk.encrypt_asymmetric(context, encoder.encode(context, y, scale))  # numpy array: the added overload
    prod = cahel.ciphertext(context)
    cahel.multiply(context, cx, cy, prod)
    cahel.relinearize_inplace(context, prod, rlk)
    cahel.rescale_to_next_inplace(context, prod)
    got = np.array(encoder.decode(context, sk.decrypt(context, prod)))
    assert np.abs(got - x * y).max() < 1e-5  # the tolerance of cahel-main/unittest/evaluator.cu
    rot = cahel.ciphertext(context)
    cahel.rotate_vector(context, prod, 1, glk, rot)
    got = np.array(encoder.decode(context, sk.decrypt(context, rot)))
    assert np.abs(got - np.roll(x * y, -1)).max() < 1e-5
    h = cahel.hoisting(context, prod, glk, [1, 2, 3])
    got = np.array(encoder.decode(context, sk.decrypt(context, h)))
    assert np.abs(got - sum(np.roll(x * y, -k) for k in (1, 2, 3))).max() < 1e-5
    # error classes of the reference's binding: invalid_argument -> ValueError, logic_error -> RuntimeError
    with pytest.raises(ValueError):
        cahel.relinearize_inplace(context, cx, rlk)  # size 2
    with pytest.raises(RuntimeError):
        cahel.rotate_rows_inplace(context, cx, 1, glk)  # a BFV / BGV operation
    dst = cahel.ciphertext(context)
    cahel.sub(context, cy, cx, dst)
    got = np.array(encoder.decode(context, sk.decrypt(context, dst)))
    assert np.abs(got - (y - x)).max() < 1e-6
    stats = cahel.memory_pool_stats()
    assert stats["reuses"] > 0


def test_module_and_python_mirror_write_the_same_ciphertext_bytes(cahel):
    """same seeds in, same bytes out: keys, a ciphertext and a relinearized product, through save() in the
    reference's stream layout"""
    import lancelot_b200.pycahel as mirror

    n = 4096
    stream = np.random.default_rng(7).integers(0, 256, 64 * 400, dtype=np.uint8).tobytes()

    def feeder():
        pos = [0]

        def take(k):
            b = stream[pos[0]:pos[0] + 64 * k]
            pos[0] += 64 * k
            return b
        return take

    vals = np.random.default_rng(1).uniform(-1, 1, n // 2)
    # -- extension module
    take = feeder()
    cahel.set_seed_source(take)
    try:
        params = cahel.params(cahel.scheme_type.ckks)
        params.set_poly_modulus_degree(n)
        params.set_coeff_modulus(cahel.coeff_modulus_create(n, [60, 40, 40, 60]))
        params.set_special_modulus_size(1)
        params.set_galois_elts(cahel.get_elts_from_steps([1], n))
        context = cahel.context(params, True, cahel.sec_level_type.none)
        sk = cahel.secret_key(params)
        sk.gen_secretkey(context)
        pk = cahel.public_key(context)
        sk.gen_publickey(context, pk)
        rlk = cahel.relin_key(context)
        sk.gen_relinkey(context, rlk)
        glk = cahel.galois_key(context)
        sk.create_galois_keys(context, glk)
        enc = cahel.ckks_encoder(context)
        ct = pk.encrypt_asymmetric(context, enc.encode(context, vals, 2.0 ** 40))
        sq = cahel.ciphertext(context)
        cahel.square(context, ct, sq)
        cahel.relinearize_inplace(context, sq, rlk)
        cahel.rescale_to_next_inplace(context, sq)
        cahel.rotate_vector_inplace(context, sq, 1, glk)
        ext = [pk.save(context), rlk.save(context), glk.save(context), ct.save(context), sq.save(context)]
    finally:
        cahel.set_seed_source(None)
    # -- Python mirror over the same C ABI
    take = feeder()
    prev = mirror._seed_source
    mirror.set_seed_source(lambda k: np.frombuffer(take(k), dtype=np.uint8))
    try:
        p = mirror.params(mirror.scheme_type.ckks)
        p.set_poly_modulus_degree(n)
        p.set_coeff_modulus(mirror.coeff_modulus_create(n, [60, 40, 40, 60]))
        p.set_special_modulus_size(1)
        p.set_galois_elts(mirror.get_elts_from_steps([1], n))
        c = mirror.context(p, True, mirror.sec_level_type.none)
        s = mirror.secret_key(p)
        s.gen_secretkey(c)
        k = mirror.public_key(c)
        s.gen_publickey(c, k)
        r = mirror.relin_key(c)
        s.gen_relinkey(c, r)
        g = mirror.galois_key(c)
        s.create_galois_keys(c, g)
        e = mirror.ckks_encoder(c)
        t = k.encrypt_asymmetric(c, e.encode(c, list(vals), 2.0 ** 40))
        q = mirror.ciphertext(c)
        mirror.square(c, t, q)
        mirror.relinearize_inplace(c, q, r)
        mirror.rescale_to_next_inplace(c, q)
        mirror.rotate_vector_inplace(c, q, 1, g)
        py = []
        for obj in (k, r, g, t, q):
            buf = io.BytesIO()
            obj.save(c, buf)
            py.append(buf.getvalue())
    finally:
        mirror.set_seed_source(prev)
    names = ["public key", "relinearization key", "Galois keys", "ciphertext", "rotated product"]
    for name, a, b in zip(names, ext, py):
        assert a == b, name
    # and the module loads what it saved
    ct2 = cahel.ciphertext(context)
    ct2.load(context, ext[3])
    assert ct2.save(context) == ext[3]


def test_reference_driver_runs_unmodified_on_the_module(cahel):
    """lancelot-main-GPU/utils/byzantine_fl.py, imported as it is from a checkout of the reference
    (LANCELOT_REFERENCE_DIR), finds this module as `pyCAHEL` and runs GPU_init -> GPU_computing_distance_cipher ->
    GPU_decrypt_sort_mask -> GPU_mul_mask_weight on three small clients; the selected client and its weights are
    those of plaintext Krum.  Skipped where no checkout is available."""
    import torch

    ref = os.environ.get("LANCELOT_REFERENCE_DIR")
    if not ref or not os.path.isdir(os.path.join(ref, "lancelot-main-GPU", "utils")):
        pytest.skip("LANCELOT_REFERENCE_DIR does not point at a checkout of the reference")
    sim = os.path.join(ref, "lancelot-main-GPU")
    sys.path.insert(0, sim)
    try:
        import importlib

        bfl = importlib.import_module("utils.byzantine_fl")
        assert os.path.samefile(os.path.dirname(bfl.__file__), os.path.join(sim, "utils"))
        assert bfl.cahel is cahel, "the driver did not pick up the extension module"
        # the driver hard-codes 32768 slots (byzantine_fl.py:33-34); a ring of 8192 keeps the test short
        bfl.Nslot, bfl.log_Nslot = 4096, 12
        torch.manual_seed(0)
        dim = 6000  # two chunks, the second one ragged
        base = torch.randn(dim) * 0.1
        w_locals = [{"layer.weight": (base[:5000] + 0.01 * torch.randn(5000)).reshape(50, 100),
                     "layer.bias": base[5000:] + 0.01 * torch.randn(1000)} for _ in range(3)]
        w_locals[1]["layer.weight"] = w_locals[1]["layer.weight"] + 1.5  # the outlier
        flat = [torch.cat([v.reshape(-1) for v in w.values()]).double() for w in w_locals]
        dist = [sum(float(((flat[i] - flat[j]) ** 2).sum()) for j in range(3)) for i in range(3)]
        chosen = int(np.argmin(dist))
        assert chosen != 1
        context, pk, sk, glk, rlk, encoder, scale = bfl.GPU_init()
        distance_matrix, vectors_final = bfl.GPU_computing_distance_cipher(context, pk, sk, glk, rlk, encoder, scale, w_locals)
        # the encrypted distances themselves (slot 0 of every pair)
        for i in range(3):
            for j in range(3):
                d = encoder.decode(context, sk.decrypt(context, distance_matrix[i][j]))[0]
                want = float(((flat[i] - flat[j]) ** 2).sum())
                assert abs(d - want) <= 1e-5 * want + 1e-3, (i, j, d, want)
        mask, chosen_idx = bfl.GPU_decrypt_sort_mask(context, pk, sk, encoder, scale, distance_matrix)
        assert int(chosen_idx) == chosen
        w_new = bfl.GPU_mul_mask_weight(context, pk, encoder, scale, rlk, vectors_final, mask, sk)
        got = np.array(w_new[:dim])
        assert np.abs(got - flat[chosen].numpy()).max() < 1e-4
    finally:
        sys.path.remove(sim)
