"""Shared helpers for the GPU parity tests."""
import numpy as np


def rand_rows(rng, moduli_for_rows, n):
    return np.stack([rng.integers(0, q, n, dtype=np.uint64) for q in moduli_for_rows])


def row_moduli(moduli, size_Q, size_l, size_p, groups=1):
    one = [moduli[r] for r in range(size_l)] + [moduli[size_Q + i] for i in range(size_p)]
    return one * groups


def seeds(rng, k):
    return rng.integers(0, 256, 64 * k, dtype=np.uint8)
