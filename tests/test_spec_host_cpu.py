"""Host logic of the speculative loop that needs no GPU: option clamping and
prompt-lookup drafting, product (C ABI) against the reference's own vectors
(engine/speculative_test.go:139-151) and against the CPU oracle."""
import numpy as np

from oracle import pyoracle as yo
from yuuka_b200 import cuda


def test_options_normalize_clamps_like_the_reference():
    # engine/speculative.go:21-34: defaults 4 / 2, caps 16 / 8
    assert cuda.spec_options_normalize(0, 0) == (4, 2)
    assert cuda.spec_options_normalize(-3, -1) == (4, 2)
    assert cuda.spec_options_normalize(99, 99) == (16, 8)
    assert cuda.spec_options_normalize(7, 3) == (7, 3)


def test_lookup_draft_reference_vectors():
    # engine/speculative_test.go:139-151
    assert cuda.spec_lookup_draft([1, 2, 3, 4, 1, 2], 3, 2) == [3, 4, 1]
    assert cuda.spec_lookup_draft([1, 2, 3, 4], 3, 2) == []
    assert cuda.spec_lookup_draft([5, 6, 7, 5, 6, 8, 5, 6], 2, 2) == [8, 5]


def test_lookup_draft_matches_oracle_on_random_histories():
    rng = np.random.default_rng(5)
    hits = 0
    for trial in range(400):
        n = int(rng.integers(1, 60))
        alphabet = int(rng.integers(2, 6))
        h = rng.integers(0, alphabet, n).astype(np.int32)
        max_draft, min_match = int(rng.integers(0, 18)), int(rng.integers(0, 10))
        got = cuda.spec_lookup_draft(h, max_draft, min_match)
        want = yo.lookup_draft(h, max_draft, min_match)
        assert got == list(want), (h.tolist(), max_draft, min_match)
        hits += bool(got)
    assert hits > 100


def test_lookup_draft_edge_cases():
    assert cuda.spec_lookup_draft([], 4, 2) == []
    assert cuda.spec_lookup_draft([7, 7], 4, 2) == []          # len(history) <= min_match
    assert cuda.spec_lookup_draft([7, 7, 7], 4, 2) == [7]       # overlap: suffix [7,7] at 0, one follower
    assert cuda.spec_lookup_draft([1, 2, 1, 2, 1, 2], 16, 1) == [1, 2]  # longest suffix wins over later shorter ones
