"""Every fast path has a switch that turns it off (environment variables read once per process).  The
output sets of a reach must not depend on them beyond the rounding of a different summation order:
windows vs dense columns, window-only writes vs zero-filled columns, the tap-skipping convolution vs the
patch-tiled one, the window-sorted bound reduction vs the chunked dense one, masked rows and implicit
unit-vector columns vs their eager forms, the gathered FC vs the dense one, unit-vector columns carried
through a pooling layer vs written by it, the bound reduction on window-only copies vs on the columns, the persistent
form of the windowed convolution vs one block per tile.  NNVB_POISON fills every layer's
output buffer with NaN patterns before the layer writes its windows: any read outside a window would
surface as NaN in the sets."""
import os
import subprocess
import sys

import numpy as np
import pytest

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
SWITCHES = ["NNVB_NO_WINDOWS", "NNVB_ZERO_FILL", "NNVB_NO_CONV_WIN", "NNVB_NO_RANGE_SKIP", "NNVB_EAGER_RELU",
            "NNVB_EAGER_MASK", "NNVB_NO_FC_GATHER", "NNVB_NO_HOT_POOL", "NNVB_NO_PACK", "NNVB_NO_COMPACT", "NNVB_NO_PERSIST", "NNVB_POOL_ONE_ROW", "NNVB_POISON"]


def _run(tmp_path, switch):
    out = str(tmp_path / ("%s.npz" % (switch or "default")))
    env = dict(os.environ)
    for s in SWITCHES:
        env.pop(s, None)
    if switch:
        env[switch] = "1"
    r = subprocess.run([sys.executable, os.path.join(ROOT, "tests", "variant_worker.py"), out], env=env,
                       capture_output=True, text=True, timeout=600)
    assert r.returncode == 0, r.stdout + r.stderr
    return np.load(out)


@pytest.fixture(scope="module")
def default_run(tmp_path_factory):
    return _run(tmp_path_factory.mktemp("variants"), None)


@pytest.mark.parametrize("switch", SWITCHES)
def test_switch_does_not_change_the_sets(tmp_path, default_run, switch):
    got = _run(tmp_path, switch)
    assert sorted(got.files) == sorted(default_run.files)
    for k in default_run.files:
        a, b = got[k], default_run[k]
        assert a.shape == b.shape, k
        if "cross" in k or "verdict" in k:
            assert np.array_equal(a, b), k                   # index work and verdicts: identical
        else:
            scale = max(np.abs(b).max(), 1e-300)
            assert np.abs(a - b).max() / scale < 1e-12, k
