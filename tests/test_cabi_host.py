"""CPU-side checks of the C-ABI library: it loads, exports every symbol the header
declares, and its host-only parameter helpers agree with the oracle."""
import ctypes as C
import os
import re

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _declared_symbols():
    names = set()
    for header in ("lancelot_b200.h", "lancelot_b200_diag.h"):
        text = open(os.path.join(ROOT, "include", header)).read()
        names.update(re.findall(r"LB_API[^;(]*?\b(lb_[a-z0-9_]+)\s*\(", text))
    return sorted(names)


def test_library_exports_every_declared_symbol():
    from lancelot_b200 import lib

    names = _declared_symbols()
    assert len(names) >= 30
    for name in names:
        assert hasattr(lib, name), "missing export: " + name


def test_prime_generation_matches_oracle():
    from lancelot_b200 import cabi
    from oracle import binding

    for n, bits in [(1 << 13, [60, 40, 40, 60]), (1 << 15, [60, 40, 40, 60]), (1 << 16, [60] + [50] * 23 + [60] * 8),
                    (1 << 12, [50, 40, 40, 40, 40, 40, 50, 50])]:
        assert cabi.coeff_modulus_create(n, bits) == binding.coeff_modulus_create(n, bits)


def test_roots_and_galois_elements_match_oracle():
    from lancelot_b200 import cabi, lib
    from oracle import binding

    n = 1 << 12
    mods = binding.coeff_modulus_create(n, [60, 40, 60])
    for q in mods:
        assert lib.lb_minimal_primitive_root(2 * n, q) == binding.lib.orc_minimal_primitive_root(2 * n, q)
    steps = [0, 1, 2, 3, 15, 16, 1024, -1, -7]
    assert cabi.galois_elts_from_steps(steps, n) == binding.elts_from_steps(steps, n)
    with pytest.raises(ValueError):
        cabi.galois_elts_from_steps([n // 2], n)


def test_invalid_arguments_are_reported_not_crashed():
    from lancelot_b200 import cabi, lib
    from lancelot_b200._lib import InvalidArgument

    with pytest.raises(InvalidArgument):
        cabi.coeff_modulus_create(1000, [40])  # not a power of two
    with pytest.raises(InvalidArgument):
        cabi.coeff_modulus_create(1 << 12, [61])  # above the 60-bit limit of the reference
    assert lib.lb_max_bit_count_tc128(65536) == 1777 and lib.lb_max_bit_count_tc128(8192) == 218
    # a null context is refused by every compute entry point
    assert lib.lb_ntt_forward(None, None, 1, 1, 0, None) == 1
    assert b"context" in lib.lb_last_error()


def test_context_refuses_primes_of_more_than_60_bits():
    """the kernels' lazy ranges (unreduced differences, 63 products per 128-bit sum, 64-bit sums of eight residues)
    hold for primes below 2^60, the reference's own limit; a larger prime is refused before any device work"""
    from lancelot_b200 import cabi
    from lancelot_b200._lib import InvalidArgument

    n = 1 << 10
    # a 61-bit prime congruent to 1 mod 2n
    q = (1 << 61) - (1 << 61) % (2 * n) + 1
    from oracle import binding
    while not binding.lib.orc_is_prime(q):
        q -= 2 * n
    assert q >> 60
    with pytest.raises(InvalidArgument, match="2\\^60"):
        cabi.Context(10, [q], 0)


def test_pycahel_extension_module_exports_the_reference_binding_names():
    """the pybind11 module loads without a GPU and carries every name cahel-main/python/src/binding.cu:8-156 exports;
    its host-only calls agree with the oracle"""
    import sys

    from oracle import binding

    sys.path.insert(0, os.path.join(ROOT, "lancelot_b200", "pybind"))
    try:
        import pyCAHEL as cahel
    finally:
        sys.path.pop(0)
    names = """scheme_type mul_tech_type sec_level_type modulus coeff_modulus_create params context secret_key public_key
        relin_key galois_key get_elts_from_steps ckks_encoder plaintext ciphertext negate negate_inplace add add_inplace
        add_plain add_plain_inplace add_many sub sub_inplace sub_plain sub_plain_inplace multiply multiply_inplace
        multiply_and_relin_inplace multiply_plain multiply_plain_inplace multiply_many square square_inplace exponentiate
        exponentiate_inplace relinearize relinearize_inplace mod_switch_to mod_switch_to_inplace mod_switch_to_next
        mod_switch_to_next_inplace rescale_to_next rescale_to_next_inplace apply_galois apply_galois_inplace rotate_rows
        rotate_rows_inplace rotate_columns rotate_columns_inplace rotate_vector rotate_vector_inplace hoisting
        hoisting_inplace complex_conjugate complex_conjugate_inplace""".split()
    for name in names:
        assert hasattr(cahel, name), "missing: " + name
    # export_values(): the enumerators are module attributes too
    assert cahel.ckks == cahel.scheme_type.ckks and cahel.tc128 == cahel.sec_level_type.tc128
    for cls, methods in [(cahel.params, "set_mul_tech set_poly_modulus_degree set_special_modulus_size set_galois_elts set_coeff_modulus"),
                         (cahel.secret_key, "gen_secretkey gen_publickey gen_relinkey create_galois_keys encrypt_symmetric decrypt"),
                         (cahel.public_key, "encrypt_asymmetric"), (cahel.ckks_encoder, "slot_count encode encode_to decode"),
                         (cahel.ciphertext, "set_scale")]:
        for m in methods.split():
            assert hasattr(cls, m), "%s.%s" % (cls.__name__, m)
    n = 1 << 13
    mods = cahel.coeff_modulus_create(n, [60, 40, 40, 60])
    assert [m.value() for m in mods] == binding.coeff_modulus_create(n, [60, 40, 40, 60])
    assert list(cahel.get_elts_from_steps([1, 2, -3], n)) == binding.elts_from_steps([1, 2, -3], n)
    with pytest.raises(ValueError):
        cahel.coeff_modulus_create(1000, [40])
