"""The CPU oracle against the golden fixtures: the reference's own outputs on seeded inputs, RTX 4060 hardware bits
(epilogue ties and zero-sign / underflow / NaN extracts) and the sha256 of H100 PCIe outputs. CPU only."""
import pytest

import golden_cases as G
from oracle import oracle

H100_CPU_GMAC = 0.12      # the larger H100 calls run in the GPU tier; all of them run in oracle/pin_against_reference.py


def _check(case):
    msg = G.evaluate(case, oracle.scaled_mm, oracle.accumulate)
    assert msg is None, msg


@pytest.mark.parametrize("case", G.reference_cases(), ids=lambda c: c.id)
def test_reference_outputs(case):
    _check(case)


@pytest.mark.parametrize("case", G.late_preset_cases(), ids=lambda c: c.id)
def test_reference_outputs_of_the_late_accumulator_preset(case):
    _check(case)


@pytest.mark.parametrize("case", G.epilogue_tie_cases(), ids=lambda c: c.id)
def test_rtx4060_double_rounding_ties(case):
    _check(case)


@pytest.mark.parametrize("case", G.epilogue_extract_cases(), ids=lambda c: c.id)
def test_rtx4060_zero_sign_underflow_nan(case):
    _check(case)


@pytest.mark.parametrize("case", G.h100_cases(max_gmac=H100_CPU_GMAC), ids=lambda c: c.id)
def test_h100_live_calls(case):
    _check(case)


def test_fixture_coverage():
    ref = G.reference_cases()
    assert {c.out for c in ref} == {"float32", "bfloat16", "float16", "float8_e4m3fn", "float8_e5m2"}
    assert {(c.fa, c.fb) for c in ref} == {("e4m3", "e4m3"), ("e5m2", "e4m3"), ("e4m3", "e5m2")}
    assert {c.scheme for c in ref} == {"none", "serial", "pairwise", "contiguous"}
    assert {c.fast for c in ref} == {True, False} and {c.api for c in ref} == {"scaled_mm", "accumulate"}
    late = G.late_preset_cases()
    assert len(late) == 13 and {c.nfma for c in late} == {288} and all(c.fast and c.S == 1 for c in late)
    assert {(c.fa, c.fb) for c in late} == {("e4m3", "e4m3"), ("e5m2", "e4m3"), ("e4m3", "e5m2")}
    assert len(G.epilogue_tie_cases()) == 64 and len(G.h100_cases()) == 122 and len(G.h100_rejected()) == 2
    assert {c.S for c in G.h100_cases()} == {1, 2, 3, 4, 5, 6}
