"""The benchmark's reference arm: the unmodified reference files run through out-of-tree adapters.

Each case runs in a child process, because the arm must not share an interpreter with the
product package (the repository's ``communication`` alias package would shadow the reference's
directory of that name).
"""
import json
import os
import subprocess
import sys

import pytest

REPO = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
REF_SRC = os.path.join(REPO, "baseline", "_ref", "communication")

pytestmark = pytest.mark.gpu


def _have_reference():
    beside = os.path.join(os.environ.get("CONEF_REFERENCE_SRC") or os.path.join(os.path.dirname(REPO), "reference"), "communication")
    return os.path.isdir(REF_SRC) or os.path.isdir(beside)


@pytest.mark.skipif(not _have_reference(), reason="no copy of the reference tree on this machine")
def test_reference_sketch_kernels_match_numpy_restatement():
    r = subprocess.run([sys.executable, os.path.join(REPO, "baseline", "check_reference_kernels.py")],
                       capture_output=True, text=True, timeout=600, cwd=REPO)
    assert r.returncode == 0, r.stderr[-3000:]
    assert r.stdout.strip().endswith("ok")


@pytest.mark.skipif(not _have_reference(), reason="no copy of the reference tree on this machine")
def test_reference_arm_prints_a_bench_line_without_loading_the_product():
    env = dict(os.environ, MASTER_ADDR="127.0.0.1", MASTER_PORT="29641")
    for k in ("RANK", "WORLD_SIZE", "LOCAL_RANK"):
        env.pop(k, None)
    r = subprocess.run([sys.executable, os.path.join(REPO, "bench.py"), "--impl", "reference", "--small",
                        "--batch", "32", "--steps", "3", "--warmup", "3"],
                       capture_output=True, text=True, timeout=900, cwd=REPO, env=env)
    assert r.returncode == 0, r.stderr[-3000:]
    line = json.loads(r.stdout.strip().splitlines()[-1])
    assert line["impl"] == "reference"
    assert "unavailable" not in line, line
    assert line["value"] > 0 and line["e2e"]["value"] > 0
    assert line["e2e"]["loss_finite"]
    assert line["ef_buffer_mb"] > 0
