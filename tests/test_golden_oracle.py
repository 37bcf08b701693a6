"""Pins the CPU oracle against outputs of the reference library itself (run on a B200,
tests/golden/ref_fixture.json): every stage of the chain must hash identically."""
import pytest

from golden_replay import CASES, load_fixture, moduli_of, replay


@pytest.mark.parametrize("case", sorted(CASES))
def test_oracle_reproduces_reference_digests(case):
    from oracle import binding

    fix = load_fixture()[case]
    cfg = CASES[case]
    mods = moduli_of(case, fix, binding.coeff_modulus_create)
    n = 1 << cfg["logn"]
    assert mods[:8] == [int(x) for x in fix["moduli"]["head"]]
    elts = binding.elts_from_steps(cfg["steps"], n)
    assert elts == [int(x) for x in fix["galois_elts"]["head"]]
    o = binding.Oracle(cfg["logn"], mods, cfg["size_p"], elts)
    report = replay(case, fix, o)
    bad = [name for name, ok in report if not ok]
    assert not bad, "stages that differ from the reference: %s" % bad
