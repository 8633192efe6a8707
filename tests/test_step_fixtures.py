"""The committed train-step fixtures (tests/golden/step_*.npz) belong to the oracle and the
seeds the generator names: the initial-weight samples equal a fresh oracle initialisation bit
for bit, the batches regenerate to the recorded token sums, and the recorded trajectories are
complete and finite.  (Re-running the oracle's steps takes minutes to hours; the generator is
``tests/golden/make_step_fixtures.py``.)"""
import os

import numpy as np
import pytest

from oracle import gpt as ogpt
from oracle.cpu_ref import SeededRng
from tests.golden.make_step_fixtures import CASES, case_batches, sample_index

GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")


@pytest.mark.parametrize("case", list(CASES))
def test_fixture_matches_oracle_init_and_batches(case):
    spec = CASES[case]
    fx = np.load(os.path.join(GOLDEN, f"step_{case}.npz"))
    P = ogpt.init_gpt(ogpt.ModelConfig(**spec["model"]), SeededRng(spec["train"]["seed"]))
    assert [str(n) for n in fx["param_names"]] == list(P)
    for n, v in P.items():
        flat = np.asarray(v.data, np.float32).reshape(-1)
        assert np.array_equal(flat[sample_index(flat.size)], fx[f"init/{n}/sample"]), n
        assert abs(float(np.linalg.norm(flat.astype(np.float64))) - float(fx[f"init/{n}/norm"])) < 1e-9
    batches = case_batches(spec)
    assert np.array_equal(fx["batch_token_sums"], [int(t.sum()) + int(g.sum()) for t, g in batches])
    for k in ("loss", "gradNorm", "lr", "clipCoef"):
        assert fx[k].shape == (spec["steps"],) and np.all(np.isfinite(fx[k]))
    assert fx["loss"][-1] < fx["loss"][0]                       # the oracle's run learns
    for s in spec["snapshots"]:
        for n in P:
            assert f"step{s}/{n}/sample" in fx.files and f"step{s}/{n}/norm" in fx.files
