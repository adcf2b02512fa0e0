"""The oracle's chunkwise (WY-form) Gated-DeltaNet scan against its per-token scan.

Restates TestGDNChunkedMatchesPerToken and TestGDNChunkedLongSequence (model/qwen35/recurrent_test.go:9-126):
same shapes, row counts, input distributions and bar (largest difference relative to the largest magnitude of
the per-token result <= 1e-4, for the outputs and for the state). The reference draws from Go's math/rand, which
cannot be reproduced here; the inputs are seeded numpy draws of the same distributions.
"""
import numpy as np
import pytest

from oracle import pyoracle as yo


def unit_rows(rng, n, size):
    x = rng.standard_normal((n, size))
    return (x / np.sqrt((x * x).sum(-1, keepdims=True))).astype(np.float32)


def rel_diff(a, b):
    peak = float(np.max(np.abs(a)))
    diff = float(np.max(np.abs(a - b)))
    return diff if peak == 0 else diff / peak


def make_inputs(rng, rows, groups, rank, S, v_scale, alpha_lo, beta_lo, beta_span):
    key_dim = groups * S
    conv = np.empty((rows, 2 * key_dim + rank * S), np.float32)
    conv[:, :key_dim] = unit_rows(rng, rows * groups, S).reshape(rows, key_dim)
    conv[:, key_dim:2 * key_dim] = unit_rows(rng, rows * groups, S).reshape(rows, key_dim)
    conv[:, 2 * key_dim:] = (v_scale * rng.standard_normal((rows, rank * S))).astype(np.float32)
    alpha = (alpha_lo * rng.random((rows, rank))).astype(np.float32)
    beta = (beta_span * rng.random((rows, rank)) + beta_lo).astype(np.float32)
    return conv, alpha, beta


@pytest.mark.parametrize("rows", [1, 5, 32, 33, 64, 100])
def test_chunked_matches_per_token(rows):
    S, groups, rank = 128, 4, 8
    rng = np.random.default_rng(20261118 + rows)
    state = (0.5 * rng.standard_normal((rank, S, S))).astype(np.float32)
    conv, alpha, beta = make_inputs(rng, rows, groups, rank, S, 1.0, -0.2, 0.05, 0.9)
    ref_state, chunk_state = state.copy(), state.copy()
    ref_out = yo.gdn_per_token_scan(ref_state, conv, alpha, beta, rows, groups, rank, S)
    chunk_out = yo.gdn_chunked_scan(chunk_state, conv, alpha, beta, rows, groups, rank, S)
    assert rel_diff(ref_out, chunk_out) <= 1e-4
    assert rel_diff(ref_state, chunk_state) <= 1e-4


def test_chunked_long_sequence():
    S, groups, rank, rows = 128, 2, 4, 160
    rng = np.random.default_rng(7)
    conv, alpha, beta = make_inputs(rng, rows, groups, rank, S, 2.0, -0.05, 0.0, 1.0)
    state = rng.standard_normal((rank, S, S)).astype(np.float32)
    ref_state, chunk_state = state.copy(), state.copy()
    ref_out = yo.gdn_per_token_scan(ref_state, conv, alpha, beta, rows, groups, rank, S)
    chunk_out = yo.gdn_chunked_scan(chunk_state, conv, alpha, beta, rows, groups, rank, S)
    assert rel_diff(ref_out, chunk_out) <= 1e-4
    assert rel_diff(ref_state, chunk_state) <= 1e-4


def test_chunked_state_size_64_and_ragged_groups():
    # rank not a multiple of... the head-to-group map h % groups with rank 6 over 3 groups, state 64
    S, groups, rank, rows = 64, 3, 6, 70
    rng = np.random.default_rng(11)
    conv, alpha, beta = make_inputs(rng, rows, groups, rank, S, 1.0, -0.3, 0.05, 0.9)
    state = (0.5 * rng.standard_normal((rank, S, S))).astype(np.float32)
    ref_state, chunk_state = state.copy(), state.copy()
    ref_out = yo.gdn_per_token_scan(ref_state, conv, alpha, beta, rows, groups, rank, S)
    chunk_out = yo.gdn_chunked_scan(chunk_state, conv, alpha, beta, rows, groups, rank, S)
    assert rel_diff(ref_out, chunk_out) <= 1e-4
    assert rel_diff(ref_state, chunk_state) <= 1e-4
