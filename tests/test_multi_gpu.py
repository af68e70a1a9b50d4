"""Two-GPU tests: peer-memory collectives against NCCL, and a tensor-parallel
engine run against the single-GPU engine."""
import json
import os
import tempfile

import pytest
import torch

from dist_utils import run_ranks

pytestmark = [pytest.mark.gpu, pytest.mark.multi_gpu]


def test_symmetric_memory_collectives_match_nccl():
    with tempfile.TemporaryDirectory() as d:
        res = run_ranks("symm", 2, d, device="cuda", timeout=600)
    for r in res:
        for name, err in r["max_err"].items():
            tol = 0.13 if name.startswith(("small", "odd", "large")) else 0.07
            assert err <= tol, (name, err)
    print("all-reduce us (symm vs nccl):", res[0]["us_symm_1MiB"], res[0]["us_nccl_1MiB"],
          res[0]["us_symm_64MiB"], res[0]["us_nccl_64MiB"])
