"""The CUPTI activity collector (csrc/runtime/cupti_collector.cpp, utils/gpu_activity.py) against a stand-in CUPTI library
that plays the buffer protocol with synthetic records: records reach Python with names, streams and launch shapes, land on
the host clock, merge into the trace beside host spans, and every failure is a message rather than a crash."""
import json
import os
import shutil
import subprocess
import sys
import time

import pytest

from onnx_genai_b200.build import cuda_include_dir

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))

if not cuda_include_dir() or not shutil.which("gcc"):
    pytest.skip("needs the CUPTI headers and a C compiler to build the stand-in library", allow_module_level=True)


@pytest.fixture(scope="module")
def fake(tmp_path_factory):
    out = str(tmp_path_factory.mktemp("cupti") / "libfake_cupti.so")
    subprocess.run(["gcc", "-O1", "-shared", "-fPIC", "-I", cuda_include_dir(), os.path.join(ROOT, "tests", "fake_cupti.c"), "-o", out], check=True)
    return out


def _child(code: str, fake: str, **env):
    """The collector keeps process-wide state (one CUPTI per process), so every scenario runs in its own interpreter."""
    full = dict(os.environ, PYTHONPATH=ROOT, FAKE=fake, **env)
    proc = subprocess.run([sys.executable, "-c", code], env=full, capture_output=True, text=True, timeout=300)
    assert proc.returncode == 0, proc.stderr[-3000:]
    return json.loads(proc.stdout.strip().splitlines()[-1])


def test_records_reach_python_on_the_host_clock_and_merge_into_the_trace(fake, tmp_path):
    trace = str(tmp_path / "t.json")
    got = _child(f"""
import json, os, time
from onnx_genai_b200.utils.gpu_activity import GpuActivityCollector, merge_into_trace
from onnx_genai_b200.utils.trace import TRACER
t0 = time.perf_counter()
TRACER.enabled = True
with GpuActivityCollector(library=os.environ["FAKE"]) as gpu:
    with TRACER.span("step"):
        time.sleep(0.002)
    first = len(gpu.poll())
t1 = time.perf_counter()
n = merge_into_trace({trace!r}, gpu)
print(json.dumps({{"first": first, "n": n, "t0": t0, "t1": t1, "dropped": gpu.dropped, "busy": gpu.busy_fraction(),
                  "table": gpu.table(), "summary": gpu.summary(),
                  "records": [[a.kind, a.name, a.start_s, a.end_s, a.stream, a.grid, a.block, a.bytes, a.detail, a.correlation] for a in gpu.records]}}))
""", fake)
    recs = got["records"]
    assert got["first"] == 5 and len(recs) == 10                      # two flushes (poll, stop) of 3 kernels + memcpy + memset
    kernels = [r for r in recs if r[0] == "kernel"]
    assert {r[1] for r in kernels} == {"gemm_bf16_tcgen05_kernel", "paged_decode_kernel"}
    assert kernels[0][5] == [148, 1, 1] and kernels[0][6] == [192, 1, 1] and kernels[0][7] == 1024 + 200704 and kernels[0][8] == 96
    assert {r[4] for r in kernels} == {7, 8}
    copies = [r for r in recs if r[0] == "memcpy"]
    assert copies[0][7] == 4096 and copies[0][8] == 1
    for r in recs:                                                    # the stand-in stamps "within the last millisecond"
        assert got["t0"] - 0.01 < r[2] <= r[3] < got["t1"] + 0.01
    top = got["summary"][0]
    assert top["name"] == "gemm_bf16_tcgen05_kernel" and top["count"] == 4 and abs(top["mean_us"] - 50.0) < 0.5
    assert "gemm_bf16_tcgen05_kernel" in got["table"] and "device busy" in got["table"]
    assert got["dropped"] == 2 and 0 < got["busy"] < 1
    doc = json.load(open(trace))
    tracks = {e["args"]["name"] for e in doc["traceEvents"] if e["ph"] == "M"}
    assert {"engine", "gpu0 stream 7", "gpu0 stream 8"} <= tracks and got["n"] == 11
    assert any(e["name"].startswith("memcpy host to device 4096 B") for e in doc["traceEvents"])


def test_failures_are_messages(fake):
    got = _child("""
import json, os
from onnx_genai_b200.utils.gpu_activity import GpuActivityCollector, GpuActivityError
out = {}
for name, lib in (("missing", "/nonexistent/libcupti.so"), ("refused", os.environ["FAKE"])):
    try:
        GpuActivityCollector(library=lib).start()
        out[name] = "started"
    except GpuActivityError as exc:
        out[name] = str(exc)
print(json.dumps(out))
""", fake, FAKE_CUPTI_FAIL_ENABLE="1")
    assert "INSUFFICIENT_PRIVILEGES" in got["refused"] and "cuptiActivityEnable" in got["refused"]
    assert "/nonexistent/libcupti.so" in got["missing"] or "not found" in got["missing"]


def test_tracer_collects_device_activity_when_asked_by_the_environment(fake, tmp_path):
    trace = str(tmp_path / "env.json")
    got = _child("""
import json, time
from onnx_genai_b200.utils.trace import TRACER
with TRACER.span("prefill"):
    time.sleep(0.001)
TRACER.flush()
print(json.dumps({"gpu": TRACER.gpu is not None, "error": TRACER.gpu_error}))
""", fake, ONNX_GENAI_TRACE=trace, ONNX_GENAI_TRACE_CUPTI="1", ONNX_GENAI_CUPTI_LIB=fake)
    assert got["gpu"] and not got["error"]
    names = {e["name"] for e in json.load(open(trace))["traceEvents"]}
    assert {"prefill", "gemm_bf16_tcgen05_kernel", "paged_decode_kernel"} <= names
