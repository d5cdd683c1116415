"""Pins the CPU oracle against the reference's own known-answer vectors (no GPU needed)."""
import pytest

from tests.golden.reference_known_answers import CASES


@pytest.mark.parametrize("case", CASES, ids=[c.__name__ for c in CASES])
def test_oracle_reproduces_reference_vector(ora, case):
    case(ora)
