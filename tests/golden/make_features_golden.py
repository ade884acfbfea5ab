"""Generates tests/golden/features.npz: the REFERENCE's computeDistStats (ML/extract_features.cpp, compiled unmodified
into oracle/_ref) on seeded count distributions.  Run in a checkout that has the reference sources:
python tests/golden/make_features_golden.py"""
import sys
from pathlib import Path

import numpy as np

HERE = Path(__file__).resolve().parent
sys.path.insert(0, str(HERE.parent.parent))
sys.path.insert(0, str(HERE.parent))

import oracle  # noqa: E402
from feature_cases import distributions  # noqa: E402


def main():
    out = {}
    for name, counts in distributions():
        out[name] = oracle.ref_dist_stats(counts)
    np.savez_compressed(HERE / "features" / "features.npz", **out)
    print({k: v[:5] for k, v in out.items()})


if __name__ == "__main__":
    main()
