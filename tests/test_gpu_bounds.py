"""The index-checking build of the kernel library (`-DRB_BOUNDS`, loaded with RUSTRAL_BOUNDS=1): out-of-range indices are
reported through the status word, with the code of the kernel family that met them, and never trap."""
import json
import os
import subprocess
import sys

import pytest

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_checking_build_reports_out_of_range_indices_and_stays_clean_otherwise():
    env = dict(os.environ, RUSTRAL_BOUNDS="1", PYTHONPATH=ROOT + os.pathsep + os.environ.get("PYTHONPATH", ""))
    res = subprocess.run([sys.executable, os.path.join(ROOT, "tests", "bounds_worker.py")], env=env, capture_output=True,
                         text=True, timeout=300)
    assert res.returncode == 0, res.stdout[-2000:] + res.stderr[-2000:]
    out = json.loads(res.stdout.strip().splitlines()[-1])
    BOUNDS = 8
    for ok in ("embedding_ok", "gather_ok", "ce_ok", "kv_ok", "paged_ok", "train_step"):
        assert out[ok] == [0, 0], (ok, out[ok])
    for bad, where in (("embedding_bad", 101), ("gather_bad", 102), ("kv_bad", 103), ("paged_bad", 104), ("ce_bad", 105)):
        assert out[bad] == [BOUNDS, where], (bad, out[bad])
    assert out["embedding_bad_reads_row0"] and out["gather_bad_row_is_zero"]
    assert 0 < out["loss"] < 20
