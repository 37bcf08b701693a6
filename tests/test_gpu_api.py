"""The pyCAHEL mirror used the way the reference's own examples and the Lancelot driver use the
original: encode -> encrypt -> evaluate -> decrypt -> decode against the plaintext computation
(tolerance 1e-3 as in cahel-main/examples/example.h:14-19, most checks far tighter), error
classes, and the batched Krum driver against the step-by-step API."""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def env():
    import torch

    if not torch.cuda.is_available():
        pytest.fail("GPU tests need a CUDA device; there is no CPU fallback")
    import lancelot_b200.pycahel as cahel

    cahel.set_seed_source(cahel.counter_seed_source(7))
    n = 1 << 13
    parms = cahel.params(cahel.scheme_type.ckks)
    parms.set_poly_modulus_degree(n)
    parms.set_coeff_modulus(cahel.coeff_modulus_create(n, [60, 40, 40, 60]))
    parms.set_special_modulus_size(1)
    steps = [1, 2, 3, 4, 8, -2]
    parms.set_galois_elts(cahel.get_elts_from_steps(steps, n))
    ctx = cahel.context(parms, True, cahel.sec_level_type.tc128)
    sk = cahel.secret_key(parms)
    sk.gen_secretkey(ctx)
    pk = cahel.public_key(ctx)
    sk.gen_publickey(ctx, pk)
    rlk = cahel.relin_key(ctx)
    sk.gen_relinkey(ctx, rlk)
    glk = cahel.galois_key(ctx)
    sk.create_galois_keys(ctx, glk)
    enc = cahel.ckks_encoder(ctx)
    yield dict(cahel=cahel, ctx=ctx, sk=sk, pk=pk, rlk=rlk, glk=glk, enc=enc, n=n, scale=2.0 ** 40)
    cahel.set_seed_source(None)


def _dec(e, ct):
    return np.array(e["enc"].decode(e["ctx"], e["sk"].decrypt(e["ctx"], ct)))


def test_primitive_chain_config(env):
    """BASELINE configs[0]: encode two 4096-slot vectors, encrypt, multiply, relinearize, rescale, rotate by 1, decrypt."""
    cahel, ctx = env["cahel"], env["ctx"]
    rng = np.random.default_rng(2024)
    x, y = rng.uniform(-1, 1, 4096), rng.uniform(-1, 1, 4096)
    ct1 = env["pk"].encrypt_asymmetric(ctx, env["enc"].encode(ctx, list(x), env["scale"]))
    ct2 = env["pk"].encrypt_asymmetric(ctx, env["enc"].encode(ctx, y, env["scale"]))
    assert np.abs(_dec(env, ct1) - x).max() < 1e-6
    cahel.multiply_inplace(ctx, ct1, ct2)
    assert ct1.size == 3
    assert np.abs(_dec(env, ct1) - x * y).max() < 1e-6  # size-3 decryption uses s^2
    cahel.relinearize_inplace(ctx, ct1, env["rlk"])
    cahel.rescale_to_next_inplace(ctx, ct1)
    assert ct1.chain_index == 2 and abs(np.log2(ct1.scale) - 40) < 1e-3
    assert np.abs(_dec(env, ct1) - x * y).max() < 1e-5
    rot = cahel.ciphertext(ctx)
    cahel.rotate_vector(ctx, ct1, 1, env["glk"], rot)
    assert np.abs(_dec(env, rot) - np.roll(x * y, -1)).max() < 1e-4
    # a step without its own key goes through the non-adjacent form (5 = 4 + 1), a negative one rotates right
    cahel.rotate_vector(ctx, ct1, 5, env["glk"], rot)
    assert np.abs(_dec(env, rot) - np.roll(x * y, -5)).max() < 1e-4
    cahel.rotate_vector(ctx, ct1, -2, env["glk"], rot)
    assert np.abs(_dec(env, rot) - np.roll(x * y, 2)).max() < 1e-4
    h = cahel.hoisting(ctx, ct1, env["glk"], [1, 2, 3])
    p = x * y
    assert np.abs(_dec(env, h) - (np.roll(p, -1) + np.roll(p, -2) + np.roll(p, -3))).max() < 1e-4


def test_lancelot_smoke_script_sequence(env):
    """the operation sequence of lancelot-main-GPU/ckks.py: square, relinearize, rescale, multiply_plain, rescale, add, rotate(-2)"""
    cahel, ctx = env["cahel"], env["ctx"]
    x = np.linspace(-1, 1, 4096)
    ct = env["pk"].encrypt_asymmetric(ctx, env["enc"].encode(ctx, x, env["scale"]))
    cahel.square_inplace(ctx, ct)
    cahel.relinearize_inplace(ctx, ct, env["rlk"])
    cahel.rescale_to_next_inplace(ctx, ct)
    pt = env["enc"].encode_to(ctx, [0.5] * 4096, 2, env["scale"])
    cahel.multiply_plain_inplace(ctx, ct, pt)
    cahel.rescale_to_next_inplace(ctx, ct)
    assert ct.chain_index == 3
    got = _dec(env, ct)
    assert np.abs(got - 0.5 * x * x).max() < 1e-4
    other = ct.copy()
    cahel.add_inplace(ctx, ct, other)
    cahel.rotate_vector_inplace(ctx, ct, -2, env["glk"])
    assert np.abs(_dec(env, ct) - np.roll(x * x, 2)).max() < 1e-3


def test_add_sub_negate_plain_and_errors(env):
    cahel, ctx = env["cahel"], env["ctx"]
    rng = np.random.default_rng(5)
    x, y = rng.uniform(-1, 1, 4096), rng.uniform(-1, 1, 4096)
    pt_x = env["enc"].encode(ctx, x, env["scale"])
    ct1 = env["pk"].encrypt_asymmetric(ctx, pt_x)
    ct2 = env["sk"].encrypt_symmetric(ctx, env["enc"].encode(ctx, y, env["scale"]), False)
    out = cahel.ciphertext(ctx)
    cahel.sub(ctx, ct2, ct1, out)  # out = ct2 - ct1, as the Krum loop uses it
    assert np.abs(_dec(env, out) - (y - x)).max() < 1e-6
    cahel.add(ctx, ct1, ct2, out)
    assert np.abs(_dec(env, out) - (x + y)).max() < 1e-6
    cahel.negate(ctx, ct1, out)
    assert np.abs(_dec(env, out) + x).max() < 1e-6
    cahel.add_plain(ctx, ct2, pt_x, out)
    assert np.abs(_dec(env, out) - (x + y)).max() < 1e-6
    cahel.sub_plain(ctx, ct2, pt_x, out)
    assert np.abs(_dec(env, out) - (y - x)).max() < 1e-6
    many = cahel.ciphertext(ctx)
    cahel.add_many(ctx, [ct1, ct2, ct1], many)
    assert np.abs(_dec(env, many) - (2 * x + y)).max() < 1e-6
    # a size-3 plus a size-2 ciphertext keeps three polynomials
    sq = ct1.copy()
    cahel.square_inplace(ctx, sq)
    with pytest.raises(ValueError):
        cahel.add_inplace(ctx, sq, ct2)  # scale mismatch 2^80 vs 2^40
    low = ct1.copy()
    cahel.mod_switch_to_inplace(ctx, low, 2)
    assert np.abs(_dec(env, low) - x).max() < 1e-6
    with pytest.raises(ValueError):
        cahel.add_inplace(ctx, low, ct1)  # level mismatch
    with pytest.raises(ValueError):
        cahel.relinearize_inplace(ctx, ct1, env["rlk"])  # size must be 3
    with pytest.raises(ValueError):
        cahel.mod_switch_to_inplace(ctx, low, 1)  # cannot go back up
    with pytest.raises(ValueError):
        env["enc"].encode(ctx, [1.0] * 5000, env["scale"])  # more values than slots
    with pytest.raises((RuntimeError, ValueError)):
        cahel.rotate_vector(ctx, ct1, 4095, env["glk"], out)  # no key and no decomposition into available steps
    with pytest.raises(ValueError):
        cahel.params(cahel.scheme_type.bfv) and cahel.context(cahel.params(cahel.scheme_type.bfv))


def test_batched_krum_driver_equals_stepwise_api_and_plaintext():
    """EncryptedKrum (fused accumulate, batched relinearize / rescale / rotations) against the same
    ciphertexts pushed through the one-call-per-operation API of the reference driver: bit-exact;
    and against float64 plaintext Krum: relative error of the distances below 1e-6."""
    import torch

    import lancelot_b200.pycahel as cahel
    from lancelot_b200 import cabi, krum

    torch.manual_seed(3)
    log_slots = 10
    ek = krum.EncryptedKrum(log_slots=log_slots, seed=11)
    n_clients, dim = 5, 3 * 1024 - 100
    upd = torch.randn(n_clients, dim, dtype=torch.float32) * 0.5
    upd[1] += 2.0
    keep = {}
    d, order = ek.round(upd.cuda(), keep=keep)
    want_d, want_order = krum.plaintext_krum(upd)
    rel = max(abs(a - b) / b for a, b in zip(d, want_d))
    assert rel < 1e-6, rel
    assert list(order) == list(want_order) and order[-1] == 1
    # step-by-step API on the very same ciphertexts for one pair
    ctx = ek.context
    i, j = keep["pairs"][2]
    acc = None
    for c in range(keep["cts"][i].shape[0]):
        a, b = cahel.ciphertext(ctx), cahel.ciphertext(ctx)
        for obj, src in ((a, keep["cts"][i][c]), (b, keep["cts"][j][c])):
            obj.data, obj.size, obj.chain_index, obj.scale = src.clone(), 2, 1, ek.scale
        tmp = cahel.ciphertext(ctx)
        cahel.sub(ctx, b, a, tmp)
        cahel.square_inplace(ctx, tmp)
        if acc is None:
            acc = tmp
        else:
            cahel.add_inplace(ctx, acc, tmp)
    cahel.relinearize_inplace(ctx, acc, ek.rlk)
    cahel.rescale_to_next_inplace(ctx, acc)
    acc.set_scale(ek.scale)
    rot = cahel.hoisting(ctx, acc, ek.glk, ek.first_steps)
    cahel.add_inplace(ctx, acc, rot)
    tmp_rot = cahel.ciphertext(ctx)
    for k in ek.pow_steps:
        cahel.rotate_vector(ctx, acc, k, ek.glk, tmp_rot)
        cahel.add_inplace(ctx, acc, tmp_rot)
    assert torch.equal(acc.data.reshape(-1), keep["scores"][2].reshape(-1))


def test_round_from_pinned_host_updates_equals_device_updates():
    """updates left in (pinned) host memory are streamed in one client ahead of the encryption; the
    ciphertexts and the distances are the same as from a device tensor"""
    import torch

    from lancelot_b200 import krum

    torch.manual_seed(5)
    ek = krum.EncryptedKrum(log_slots=10, seed=3)
    upd = (torch.randn(6, 2 * 1024 + 17, dtype=torch.float32) * 0.3).pin_memory()
    k_dev, k_host = {}, {}
    d_dev, o_dev = ek.round(upd.cuda(), keep=k_dev)
    d_host, o_host = ek.round(upd, keep=k_host)
    assert d_dev == d_host and list(o_dev) == list(o_host)
    assert torch.equal(k_dev["cts"], k_host["cts"])


@pytest.mark.parametrize("world", [2, 3, 8])
def test_chunk_sharded_partial_sums_add_up_to_the_single_rank_sums(world):
    """What several GPUs do in EncryptedKrum.round(exchange="chunks"), on one GPU: every "rank" encrypts its chunk range
    of all clients and forms the partial sums of all pairs; the plain 64-bit sum of the partial sums, reduced mod q once
    (lb_reduce_mod), equals the sums one rank forms over all chunks, word for word, and so do the final scores."""
    import torch

    from lancelot_b200 import krum

    torch.manual_seed(9)
    ek = krum.EncryptedKrum(log_slots=10, seed=21)
    n_clients, dim = 4, 11 * 1024 - 300  # 11 chunks, the last one ragged
    upd = (torch.randn(n_clients, dim, dtype=torch.float32) * 0.4).cuda()
    chunks = ek.n_chunks(dim)
    pairs = krum.all_pairs(n_clients)
    # the deterministic test seeds depend on (client, first chunk of the slice): encrypting a slice twice gives the
    # same ciphertexts, so both sums below are formed from identical partial sums
    total, again = None, None
    for r in range(world):
        lo, hi = krum.chunk_range(chunks, r, world)
        part = ek.pair_sums(ek.encrypt_slices(upd, lo, hi), pairs)
        again_part = ek.pair_sums(ek.encrypt_slices(upd, lo, hi), pairs)
        assert torch.equal(part, again_part)
        total = part.clone() if total is None else total + part          # plain 64-bit words, as NCCL sums them
        again = again_part if again is None else ek.lb.add(3, again, again_part)  # modular additions, one rank
    ek.lb.reduce_mod(3, total)
    assert torch.equal(total, again)
    # and the decrypted distances agree with the plaintext rule
    scores = ek.finish_scores(total)
    d, order = ek.select(ek.client_sums(scores, pairs, n_clients))
    want_d, want_order = krum.plaintext_krum(upd.cpu())
    assert max(abs(a - b) / b for a, b in zip(d, want_d)) < 1e-6 and list(order) == list(want_order)



def test_save_load_streams_round_trip_on_the_device(env):
    """objects written with the reference's stream layout come back identical, several per stream"""
    import io

    import torch

    import lancelot_b200.pycahel as cahel

    ctx, sk, pk, rlk, enc, scale = env["ctx"], env["sk"], env["pk"], env["rlk"], env["enc"], env["scale"]
    pt = enc.encode(ctx, [0.5, -0.25, 3.0], scale)
    ct = pk.encrypt_asymmetric(ctx, pt)
    cahel.square_inplace(ctx, ct)
    buf = io.BytesIO()
    pt.save(ctx, buf)
    ct.save(ctx, buf)
    pk.save(ctx, buf)
    buf.seek(0)
    pt2, ct2, pk2 = cahel.plaintext(), cahel.ciphertext(), cahel.public_key(ctx)
    pt2.load(ctx, buf)
    ct2.load(ctx, buf)
    pk2.load(ctx, buf)
    assert buf.read() == b""
    assert torch.equal(pt2.data.reshape(-1), pt.data.reshape(-1)) and pt2.chain_index == pt.chain_index and pt2.scale == pt.scale
    assert torch.equal(ct2.data.reshape(-1), ct.data.reshape(-1)) and (ct2.size, ct2.chain_index, ct2.scale) == (3, ct.chain_index, ct.scale)
    assert torch.equal(pk2.data.reshape(-1), pk.data.reshape(-1))
    # a loaded ciphertext keeps working
    cahel.relinearize_inplace(ctx, ct2, rlk)
    cahel.rescale_to_next_inplace(ctx, ct2)
    out = enc.decode(ctx, sk.decrypt(ctx, ct2))
    assert abs(out[0] - 0.25) < 1e-6 and abs(out[2] - 9.0) < 1e-5
    # a stream of another parameter set is refused
    other = io.BytesIO(buf.getvalue()[:32][::-1] + buf.getvalue()[32:])
    with pytest.raises(ValueError):
        cahel.plaintext().load(ctx, other)


def test_reference_driver_flow_small():
    """GPU_init .. GPU_krum with the reference's call sequence (diagonal pairs, re-encryption per pair, masks)"""
    import torch

    from lancelot_b200 import krum

    krum.set_slots(9)
    try:
        rng = np.random.default_rng(8)
        vecs = [rng.normal(0, 0.1, 700).astype(np.float32) for _ in range(3)]
        vecs[2] = vecs[2] + 1.0
        context, pk, sk, glk, rlk, encoder, scale = krum.GPU_init()
        dm, vf = krum.GPU_computing_distance_cipher(context, pk, sk, glk, rlk, encoder, scale, vecs)
        mask, chosen = krum.GPU_decrypt_sort_mask(context, pk, sk, encoder, scale, dm)
        d01 = float(((vecs[0].astype(np.float64) - vecs[1]) ** 2).sum())
        got = encoder.decode(context, sk.decrypt(context, dm[0][1]))[0]
        assert abs(got - d01) / d01 < 1e-5
        assert chosen in (0, 1)
        w = krum.GPU_mul_mask_weight(context, pk, encoder, scale, rlk, vf, mask, sk)
        assert np.abs(np.array(w[:700]) - vecs[chosen]).max() < 1e-4
    finally:
        krum.set_slots(15)


def test_cpp_class_layer_program():
    """include/cahel_b200.hpp used like the reference's C++ examples use cahel.h (tests/cpp_api_check.cu)"""
    import os
    import subprocess

    import tempfile

    from lancelot_b200 import cabi, wire

    exe = os.path.join(os.path.dirname(os.path.abspath(__file__)), "cpp_api_check")
    assert os.path.exists(exe), "run __graft_entry__.build() first"
    with tempfile.TemporaryDirectory() as tmp:
        path = os.path.join(tmp, "objects.bin")
        r = subprocess.run([exe], capture_output=True, text=True, timeout=120, env=dict(os.environ, CPP_API_CHECK_STREAM=path))
        assert r.returncode == 0, r.stdout + r.stderr
        blob = open(path, "rb").read()
    # the stream the C++ classes wrote (plaintext, rescaled ciphertext, public key) parses with the Python reader
    n = 8192
    mods = cabi.coeff_modulus_create(n, [60, 40, 40, 60])
    pt = wire.unpack_plaintext(blob)
    assert pt["parms_id"] == wire.parms_id(n, mods, 1, 1) and pt["coeff_modulus_size"] == 3 and pt["chain_index"] == 1
    ct = wire.unpack_ciphertext(blob[pt["consumed"]:])
    assert ct["parms_id"] == wire.parms_id(n, mods, 1, 2) and (ct["size"], ct["coeff_modulus_size"], ct["chain_index"]) == (2, 2, 2)
    pk = wire.unpack_ciphertext(blob[pt["consumed"] + ct["consumed"]:])
    assert pk["parms_id"] == wire.parms_id(n, mods, 1, 0) and (pk["size"], pk["coeff_modulus_size"], pk["chain_index"]) == (2, 4, 1)
    assert pt["consumed"] + ct["consumed"] + pk["consumed"] == len(blob)
    assert all(int(x) < m for x, m in zip(ct["data"][0].max(axis=1), mods[:2]))


def test_mask_multiplication_selects_and_averages():
    """aggregation phase: one-hot mask returns the chosen client's update, a k-hot mask with 1/k their mean"""
    import torch

    from lancelot_b200 import cabi, krum

    torch.manual_seed(5)
    ek = krum.EncryptedKrum(log_slots=10, seed=3)
    n_clients, dim = 4, 2 * 1024 + 77
    upd = (torch.randn(n_clients, dim, dtype=torch.float32) * 0.3).cuda()
    cts = {c: ek.encrypt_client(upd[c], client=c) for c in range(n_clients)}
    got = ek.aggregate(cts, [2], dim)
    assert float((got - upd[2].double()).abs().max()) < 1e-6
    got = ek.aggregate(cts, [0, 3], dim)
    assert float((got - (upd[0].double() + upd[3].double()) / 2).abs().max()) < 1e-6
    # the fused accumulation equals multiply + add_inplace per client of the stepwise API, bit for bit
    import lancelot_b200.pycahel as cahel
    ctx = ek.context
    one, zero = ek.encrypt_constant(1.0), ek.encrypt_constant(0.0)
    masks = torch.stack([zero, one, zero, zero]).contiguous()
    fused = ek.lb.mask_accumulate(3, [cts[k] for k in range(n_clients)], masks, cts[0].shape[0])
    acc = None
    for k in range(n_clients):
        a, m, t = cahel.ciphertext(ctx), cahel.ciphertext(ctx), cahel.ciphertext(ctx)
        a.data, a.size, a.chain_index, a.scale = cts[k][1].clone(), 2, 1, ek.scale
        m.data, m.size, m.chain_index, m.scale = masks[k].clone(), 2, 1, ek.scale
        cahel.multiply(ctx, a, m, t)
        if acc is None:
            acc = t
        else:
            cahel.add_inplace(ctx, acc, t)
    assert torch.equal(acc.data.reshape(-1), fused[1].reshape(-1))
    # and against the CPU checker: out[c] = sum over clients of tensor(ct_k[c], mask_k), every chunk, bit for bit
    from oracle import binding
    o = binding.Oracle(ek.log_slots + 1, ctx.moduli, 1)
    h_masks = cabi.to_host(masks)
    h_cts = [cabi.to_host(cts[k]) for k in range(n_clients)]
    h_fused = cabi.to_host(fused)
    for c in range(h_fused.shape[0]):
        want = np.zeros((3, 3, ek.N), dtype=np.uint64)
        for k in range(n_clients):
            want = o.poly_op("add", 3, want, o.tensor(3, h_cts[k][c], h_masks[k]))
        assert np.array_equal(h_fused[c].reshape(-1), want.reshape(-1)), "chunk %d" % c


@pytest.mark.gpu
@pytest.mark.parametrize("n_clients,drop", [(9, 0), (9, 7), (6, 3), (2, 0), (5, 9)])
def test_round_entries_pair_sums_and_scores_equal_the_single_operations(n_clients, drop):
    """lb_krum_pair_sums (tile schedule inside the library) against the one-pair kernel for full and ragged pair
    lists, and lb_krum_scores against relinearize / rescale / hoisting / rotate / add issued one by one: word for word"""
    import random

    import torch

    from lancelot_b200 import krum

    torch.manual_seed(13)
    ek = krum.EncryptedKrum(log_slots=9, seed=5)
    dim = 3 * 512 - 41
    upd = (torch.randn(n_clients, dim, dtype=torch.float32) * 0.2).cuda()
    cts = ek.encrypt_slices(upd, 0, ek.n_chunks(dim))
    pairs = krum.all_pairs(n_clients)
    random.Random(drop).shuffle(pairs)
    pairs = sorted(pairs[: len(pairs) - drop]) if drop < len(pairs) else pairs[:1]
    acc = ek.pair_sums(cts, pairs, n_slots=len(pairs) + 2)
    assert not acc[len(pairs):].any()
    for p, (i, j) in enumerate(pairs):
        one = ek.lb.empty(3, 3, ek.N)
        ek.lb.krum_accumulate(3, cts[i], cts[j], one)
        assert torch.equal(acc[p], one), "pair %d %d" % (i, j)
    fused = ek.finish_scores(acc[: len(pairs)].clone())
    single = ek.finish_scores(acc[: len(pairs)].clone(), stepwise=True)
    assert torch.equal(fused, single)
    # refusals of the entry: a pair out of order, a pair listed twice
    with pytest.raises(ValueError):
        ek.lb.krum_pair_sums(3, cts, n_clients, [(1, 0)], acc)
    if len(pairs) > 1:
        with pytest.raises(ValueError):
            ek.lb.krum_pair_sums(3, cts, n_clients, [pairs[0], pairs[0]], acc)


@pytest.mark.gpu
def test_batched_galois_key_generation_equals_key_by_key():
    """lb_gen_galois_keys against lb_galois_permute + lb_gen_switch_key per element with the same seeds, word for word
    (the key-by-key path is the one the reference-made fixtures pin)"""
    import torch

    from lancelot_b200 import pycahel as cahel

    n = 4096
    params = cahel.params(cahel.scheme_type.ckks)
    params.set_poly_modulus_degree(n)
    params.set_coeff_modulus(cahel.coeff_modulus_create(n, [60, 40, 40, 40, 60, 60]))
    params.set_special_modulus_size(2)  # four data primes, two special ones: dnum = 2, digits of two limbs
    params.set_galois_elts(cahel.get_elts_from_steps([1, 2, 3, 5, 64], n))
    ctx = cahel.context(params, True, cahel.sec_level_type.none)
    cahel.set_seed_source(cahel.counter_seed_source(11))
    try:
        sk = cahel.secret_key(params)
        sk.gen_secretkey(ctx)
        dnum = ctx.size_Q // ctx.size_P
        seeds = [cahel._seeds(2 * dnum) for _ in ctx.galois_elts]
    finally:
        cahel.set_seed_source(None)
    lb = ctx.lb
    single = [lb.gen_switch_key(sk.data, lb.galois_permute(i, sk.data), seeds[i]) for i in range(len(seeds))]
    order = [3, 0, 4]  # any subset, any order
    batched = lb.gen_galois_keys(sk.data, order, np.concatenate([seeds[i] for i in order]))
    for k, i in enumerate(order):
        assert torch.equal(batched[k], single[i]), "element %d" % i
    every = lb.gen_galois_keys(sk.data, list(range(len(seeds))), np.concatenate(seeds))
    assert all(torch.equal(every[i], single[i]) for i in range(len(seeds)))
