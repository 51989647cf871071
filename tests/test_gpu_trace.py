"""The step timeline of the trace build: stamps of the three decode-step kernels are in order."""
import json
import os
import subprocess
import sys

import pytest

pytestmark = pytest.mark.gpu

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_timeline_of_a_decode_step(cuda_device):
    from unified_cache_management_b200 import build as ucm_build
    if not os.path.exists(ucm_build.TRACE_LIB_PATH):
        pytest.skip("no trace build (python -m unified_cache_management_b200.build --trace)")
    out = subprocess.run([sys.executable, os.path.join(ROOT, "bench.py"), "--timeline", "tp8"], capture_output=True,
                         text=True, timeout=600, cwd=ROOT)
    assert out.returncode == 0, out.stderr[-2000:]
    pts = json.loads(out.stdout.strip().splitlines()[-1])["points"]
    for kernel, n in (("encode", 4), ("scan", 8), ("select", 6)):
        own = [v for name, v in pts.items() if name.startswith(kernel + ":")]
        assert len(own) == n
        if kernel == "scan":   # the first copy may be issued before or after the dependency wait
            own = own[:3] + [min(own[3], own[4]), max(own[3], own[4])] + own[5:]
        assert own == sorted(own), (kernel, own)
    assert 0 < pts["select: end"] < 200.0   # a step of this shape takes some tens of microseconds
    assert pts["scan: dependency wait passed"] >= pts["encode: end"] - 0.5
    assert pts["select: dependency wait passed"] >= pts["scan: first warp out of items"]
