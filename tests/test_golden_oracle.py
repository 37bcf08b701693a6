"""Pins the CPU oracle against outputs of the reference library itself (run on a B200,
tests/golden/ref_fixture.json): every stage of the chain must hash identically."""
import pytest

from golden_replay import CASES, load_fixture, replay


@pytest.mark.parametrize("case", sorted(CASES))
def test_oracle_reproduces_reference_digests(case):
    from oracle import binding

    fix = load_fixture()[case]
    cfg = CASES[case]
    mods = [int(x) for x in fix["moduli"]["head"]]
    n = 1 << cfg["logn"]
    assert mods == binding.coeff_modulus_create(n, {"n4096_a1": [60, 40, 40, 60], "n8192_a1": [60, 40, 40, 60],
                                                    "n4096_a2": [50, 40, 40, 40, 40, 40, 50, 50]}[case])
    elts = binding.elts_from_steps(cfg["steps"], n)
    assert elts == [int(x) for x in fix["galois_elts"]["head"]]
    o = binding.Oracle(cfg["logn"], mods, cfg["size_p"], elts)
    report = replay(case, fix, o)
    bad = [name for name, ok in report if not ok]
    assert not bad, "stages that differ from the reference: %s" % bad
