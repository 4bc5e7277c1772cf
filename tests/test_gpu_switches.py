"""The run-time switches select other kernel variants and launch modes for the whole process, so
each combination runs the end-to-end check of ``__graft_entry__.smoke`` in a process of its
own: forward, input gradient, weight gradient (fp16), int8 forward and the GPU table builder
against the oracle."""
import os
import subprocess
import sys
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parents[1]

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("env", [
    {"CUMM_B200_GATHER": "0", "CUMM_B200_PDL": "0", "CUMM_B200_STATIC_TILES": "1"},  # cp.async everywhere, plain launches, static tiles
    {"CUMM_B200_GATHER": "2", "CUMM_B200_PDL": "2"},                                  # TMA gather everywhere, PDL for every kernel
], ids=["cp.async+plain-launch+static-tiles", "tma-gather+pdl-everywhere"])
def test_smoke_under_switches(cuda_lib, env):
    r = subprocess.run([sys.executable, "-c", "import __graft_entry__ as g; g.smoke()"], cwd=str(ROOT),
                       env={**os.environ, **env}, capture_output=True, text=True, timeout=600)
    assert r.returncode == 0, r.stdout[-2000:] + r.stderr[-2000:]
    assert "smoke ok" in r.stdout
