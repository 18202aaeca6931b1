"""Writes tests/golden/batch_slices.json: which sample indices every rank receives from the reference's own
``Dataset.batch_generator`` (pydtnn/datasets/dataset.py:160-197) for a few (samples, local batch, ranks) cases, with
and without shuffling (NumPy's global generator seeded with 1234 before each pass).  Run where the reference checkout
is importable:  PYTHONPATH=<reference root> python tests/golden/make_batch_slices_golden.py"""
import json
import os
import sys

import numpy as np

sys.path.insert(0, os.environ.get("PYDTNN_REFERENCE", "/root/reference"))
from pydtnn.datasets.dataset import Dataset  # noqa: E402

CASES = [(100, 8, 1), (100, 8, 2), (103, 8, 4), (64, 8, 4), (70, 16, 3), (33, 4, 8), (17, 16, 2)]


def main():
    out = []
    for nsamples, local, nprocs in CASES:
        x = np.arange(nsamples, dtype=np.int64).reshape(-1, 1)
        y = np.arange(nsamples, dtype=np.int64).reshape(-1, 1) * 10
        for shuffle in (False, True):
            per_rank = []
            for rank in range(nprocs):
                np.random.seed(1234)
                gen = Dataset.batch_generator(iter([(x, y)]), local, rank, nprocs, shuffle=shuffle)
                per_rank.append([[xb[:, 0].tolist(), (yb[:, 0] // 10).tolist(), int(bs)] for xb, yb, bs in gen])
            out.append({"nsamples": nsamples, "local_batch": local, "nprocs": nprocs, "shuffle": shuffle, "batches": per_rank})
    path = os.path.join(os.path.dirname(os.path.abspath(__file__)), "batch_slices.json")
    with open(path, "w") as f:
        json.dump(out, f)
    print(path, len(out), "cases")


if __name__ == "__main__":
    main()
