"""The range-checked build of the kernels (``-DMINTEXT_DEBUG_BOUNDS``, selected with ``MT_DEBUG_BOUNDS=1``): clean on
ragged / odd shapes and on a training step; bad indices come back as a report, never as a fault."""

import json
import os
import subprocess
import sys
from pathlib import Path

import pytest

pytestmark = pytest.mark.gpu
ROOT = Path(__file__).resolve().parents[1]


def test_debug_bounds_build_reports_and_skips_bad_indices():
    env = dict(os.environ, MT_DEBUG_BOUNDS="1", PYTHONPATH=str(ROOT))
    r = subprocess.run([sys.executable, str(ROOT / "tests" / "debug_bounds_worker.py")], env=env, capture_output=True,
                       text=True, timeout=600)
    assert r.returncode == 0, r.stdout[-3000:] + r.stderr[-3000:]
    out = json.loads(r.stdout.strip().splitlines()[-1])
    assert out["units"] >= 4
    assert all(l == l and l > 0 for l in out["clean_losses"])
    assert "embedding.cu" in out["embedding_report"] and "index 100 outside [0, 100)" in out["embedding_report"]
    assert "route.cu" in out["combine_report"] and "index 5 outside [0, 3)" in out["combine_report"]


def test_ordinary_build_has_no_bounds_units():
    from mintext_b200.ops._ext import debug_bounds_enabled, ext

    if debug_bounds_enabled():
        pytest.skip("running under the range-checked build")
    assert ext().debug_bounds_units() == 0 and ext().debug_bounds_report() == []
