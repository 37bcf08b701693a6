"""The save() byte streams of the reference library (ciphertext, plaintext, public key), recorded by
the reference itself in tests/golden/ref_fixture.json, against lancelot_b200.wire on the words the CPU
oracle reproduces.  Runs without a GPU."""
import hashlib

import numpy as np
import pytest

from golden_replay import CASES, load_fixture, moduli_of, replay


# cases in which the reference's memory pool happened to hand the key pairs zeroed seed blocks
ZERO_SEED_BLOCKS = ("n4096_a1", "n4096_a2", "n8192_a1", "n65536_a8")


@pytest.mark.parametrize("case", sorted(CASES))
def test_streams_match_the_reference_byte_for_byte(case):
    from lancelot_b200 import wire
    from oracle import binding

    fix = load_fixture()[case]
    cfg = CASES[case]
    mods = moduli_of(case, fix, binding.coeff_modulus_create)
    elts = [int(x) for x in fix["galois_elts"]["head"]]
    o = binding.Oracle(cfg["logn"], mods, cfg["size_p"], elts)
    keep = {}
    replay(case, fix, o, keep)
    n, size_QP, size_Q, P = keep["n"], keep["size_QP"], keep["size_Q"], cfg["size_p"]

    zero_tail = hashlib.sha256(bytes(64)).hexdigest()

    def same(name, blob, body_only=False):
        """body_only: everything before the trailing 64-byte seed block.  The reference never defines that block for
        objects it did not seed-compress (it is whatever its memory pool held), so the whole stream is compared only
        where the recorded block happens to be zero, which is what this library writes."""
        if not body_only and name + "_tail" in fix and fix[name + "_tail"]["sha256"] != zero_tail:
            assert len(blob) == fix[name]["bytes"], name
            return
        want = fix[name + ("_body" if body_only else "")]
        got = blob[:-64] if body_only else blob
        assert len(got) == want["bytes"], name
        assert hashlib.sha256(got).hexdigest() == want["sha256"], name

    pid1 = wire.parms_id(n, mods, P, 1)
    # the recorded stream starts with the parms_id words
    assert [int(x) for x in fix["stream_ct1"]["head"][:4]] == list(np.frombuffer(pid1, dtype="<u8"))
    pt = wire.pack_plaintext(pid1, 1, n, size_Q, keep["scale"], keep["pt1"])
    same("stream_pt1", pt)
    ct = wire.pack_ciphertext(pid1, 1, 2, n, size_Q, keep["scale"], keep["ct1"])
    same("stream_ct1", ct, body_only=True)
    same("stream_ct1", ct)  # the reference leaves the seed block zeroed for these objects
    # a public key is a size-2 ciphertext over all primes that carries chain index 1 and scale 1
    pk = wire.pack_public_key(n, mods, P, keep["pk"])
    same("stream_pk", pk, body_only=True)
    same("stream_pk", pk)
    res = wire.pack_ciphertext(wire.parms_id(n, mods, P, 2), 2, 2, n, size_Q - 1, keep["scale"], keep["rescaled"])
    same("stream_rescaled", res, body_only=True)

    # relinearization and Galois key streams (cahel-main/include/secretkey.h:212-256, 354-400).  The reference recorded
    # one digest over the whole stream, seed blocks of the inner key pairs included; those blocks are undefined in the
    # reference (see above), so the digest is compared where it left them zero and the length everywhere.
    rlk = wire.pack_switch_key(n, mods, P, keep["rlk"])
    glk = wire.pack_galois_keys(n, mods, P, keep["glk"])
    assert len(rlk) == fix["stream_rlk"]["bytes"] and len(glk) == fix["stream_glk"]["bytes"]
    assert [int(x) for x in fix["stream_rlk"]["head"][:4]] == list(np.frombuffer(wire.parms_id(n, mods, P, 0), dtype="<u8"))
    if case in ZERO_SEED_BLOCKS:
        assert hashlib.sha256(rlk).hexdigest() == fix["stream_rlk"]["sha256"]
        assert hashlib.sha256(glk).hexdigest() == fix["stream_glk"]["sha256"]
    back = wire.unpack_switch_key(rlk)
    assert back["consumed"] == len(rlk) and np.array_equal(back["data"].reshape(-1), np.asarray(keep["rlk"]).reshape(-1))
    gb = wire.unpack_galois_keys(glk)
    assert gb["consumed"] == len(glk) and len(gb["keys"]) == len(keep["glk"])
    assert all(np.array_equal(a.reshape(-1), np.asarray(b).reshape(-1)) for a, b in zip(gb["keys"], keep["glk"]))
    with pytest.raises(RuntimeError):
        wire.unpack_switch_key(rlk[:-1])

    # round trips and error behaviour
    back = wire.unpack_ciphertext(ct)
    assert back["chain_index"] == 1 and back["size"] == 2 and back["scale"] == keep["scale"] and back["consumed"] == len(ct)
    assert np.array_equal(back["data"].reshape(-1), np.asarray(keep["ct1"]).reshape(-1))
    pb = wire.unpack_plaintext(pt)
    assert pb["coeff_modulus_size"] == size_Q and np.array_equal(pb["data"].reshape(-1), np.asarray(keep["pt1"]).reshape(-1))
    with pytest.raises(RuntimeError):
        wire.unpack_ciphertext(ct[:-1])
    with pytest.raises(RuntimeError):
        wire.unpack_plaintext(pt[:100])


def test_cpp_layer_computes_the_same_parms_id():
    """the BLAKE2b of include/cahel_b200.hpp (host-only mode of tests/cpp_api_check) against the recorded ids"""
    import os
    import subprocess

    from lancelot_b200 import wire

    exe = os.path.join(os.path.dirname(os.path.abspath(__file__)), "cpp_api_check")
    if not os.path.exists(exe):
        pytest.skip("tests/cpp_api_check is built by __graft_entry__.build()")
    for case, cfg in CASES.items():
        fix = load_fixture()[case]
        from oracle import binding
        mods = moduli_of(case, fix, binding.coeff_modulus_create)
        n = 1 << cfg["logn"]
        for chain in (0, 1, 2):
            out = subprocess.run([exe, "--parms-id", str(n), str(cfg["size_p"]), str(chain)] + [str(m) for m in mods],
                                 capture_output=True, text=True, check=True).stdout.strip()
            assert out == wire.parms_id(n, mods, cfg["size_p"], chain).hex()
        recorded = np.array([int(x) for x in fix["stream_ct1"]["head"][:4]], dtype="<u8").tobytes().hex()
        assert recorded == wire.parms_id(n, mods, cfg["size_p"], 1).hex()
