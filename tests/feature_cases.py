"""Seeded count distributions (non-zeros per row / per column) for the feature-vector tests."""
import numpy as np


def distributions():
    rng = np.random.default_rng(2024)
    yield "poisson", rng.poisson(10, 5000)
    yield "zipf", np.minimum(rng.zipf(2.1, 20000), 20000)
    yield "constant", np.full(777, 64)
    yield "with_zeros", np.concatenate([np.zeros(300, np.int64), rng.integers(1, 50, 700)])
    yield "all_zero", np.zeros(50, np.int64)
    yield "single", np.array([5])
    yield "short", np.array([9, 1, 4])  # fewer entries than most of the top-k ranks
    yield "hot", np.concatenate([np.full(20, 100000), rng.integers(0, 12, 100000)])
    yield "empty", np.zeros(0, np.int64)
