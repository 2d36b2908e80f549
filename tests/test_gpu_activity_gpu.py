"""The CUPTI activity collector against the real library on a GPU: a small decode through the engine shows up as kernel
records (this package's kernels among them) and copies, stamped inside the host window they ran in."""
import json
import os
import subprocess
import sys

import pytest
import torch

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))

CHILD = """
import json, time
import torch
from onnx_genai_b200.utils.gpu_activity import GpuActivityCollector, GpuActivityError
import __graft_entry__ as entry
try:
    gpu = GpuActivityCollector().start()
except GpuActivityError as exc:
    print(json.dumps({"unavailable": str(exc)}))
    raise SystemExit(0)
t0 = time.perf_counter()
entry.smoke()
torch.cuda.synchronize()
t1 = time.perf_counter()
recs = gpu.stop()
print(json.dumps({"t0": t0, "t1": t1, "kernels": sum(a.kind == "kernel" for a in recs), "copies": sum(a.kind == "memcpy" for a in recs),
                  "names": sorted({a.name for a in recs if a.kind == "kernel"})[:400], "dropped": gpu.dropped, "busy": gpu.busy_fraction(),
                  "inside": sum(t0 - 0.05 <= a.start_s <= a.end_s <= t1 + 0.05 for a in recs), "n": len(recs),
                  "bad": sum(a.end_s < a.start_s for a in recs), "table": gpu.table(12)}))
"""


def test_a_decode_shows_up_as_kernel_and_copy_records():
    if not torch.cuda.is_available():
        pytest.skip("needs a GPU")
    proc = subprocess.run([sys.executable, "-c", CHILD], env=dict(os.environ, PYTHONPATH=ROOT), cwd=ROOT, capture_output=True, text=True, timeout=420)
    assert proc.returncode == 0, proc.stderr[-3000:]
    got = json.loads([l for l in proc.stdout.splitlines() if l.startswith("{")][-1])
    if "unavailable" in got:
        pytest.skip("CUPTI cannot collect here: " + got["unavailable"])
    assert got["kernels"] >= 100 and got["copies"] >= 1 and got["bad"] == 0
    assert any("tcgen05" in n for n in got["names"]), got["names"][:20]
    assert got["inside"] >= 0.98 * got["n"]                 # device stamps mapped onto the host clock fall in the window they ran in
    assert 0 < got["busy"] <= 1
