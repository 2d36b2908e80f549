"""The C interface: in-process through ctypes, and from a plain C program that embeds the engine."""
import ctypes
import os
import shutil
import subprocess
import sys

import numpy as np
import pytest

from onnx_genai_b200 import build
from onnx_genai_b200.bench.config_bench import _export

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.fixture(scope="module")
def model_dir(tmp_path_factory):
    d = tmp_path_factory.mktemp("capi_model")
    _export("tiny-llama", str(d), "fp32", layers=1)
    return str(d)


@pytest.fixture(scope="module")
def lib():
    path = build.build_capi()
    lib = ctypes.CDLL(str(path))
    lib.oge_engine_load.restype = ctypes.c_void_p
    lib.oge_engine_load.argtypes = [ctypes.c_char_p]
    lib.oge_engine_free.argtypes = [ctypes.c_void_p]
    lib.oge_engine_generate.restype = ctypes.c_void_p
    lib.oge_engine_generate.argtypes = [ctypes.c_void_p, ctypes.c_char_p, ctypes.c_size_t]
    lib.oge_engine_generate_with_sampler.restype = ctypes.c_void_p
    lib.oge_engine_generate_with_sampler.argtypes = [ctypes.c_void_p, ctypes.c_char_p, ctypes.c_size_t, ctypes.c_void_p]
    lib.oge_string_free.argtypes = [ctypes.c_void_p]
    lib.oge_last_error.restype = ctypes.c_char_p
    lib.oge_sampler_free.argtypes = [ctypes.c_void_p]
    return lib


SAMPLE_FN = ctypes.CFUNCTYPE(ctypes.c_uint32, ctypes.c_void_p, ctypes.POINTER(ctypes.c_float), ctypes.c_size_t,
                             ctypes.POINTER(ctypes.c_uint32), ctypes.c_size_t, ctypes.c_size_t)
FREE_FN = ctypes.CFUNCTYPE(None, ctypes.c_void_p)


class VTable(ctypes.Structure):
    _fields_ = [("user_data", ctypes.c_void_p), ("sample", SAMPLE_FN), ("name", ctypes.c_char_p), ("free", FREE_FN)]


def _take(lib, ptr):
    assert ptr, lib.oge_last_error()
    text = ctypes.string_at(ptr).decode("utf-8")
    lib.oge_string_free(ptr)
    return text


def test_load_generate_and_errors_in_process(lib, model_dir):
    assert not lib.oge_engine_load(b"/nonexistent/model/dir")
    assert b"cannot load" in lib.oge_last_error()
    eng = lib.oge_engine_load(model_dir.encode())
    assert eng, lib.oge_last_error()
    assert lib.oge_last_error() is None
    a = _take(lib, lib.oge_engine_generate(eng, b"hello", 6))
    b = _take(lib, lib.oge_engine_generate(eng, b"hello", 6))
    assert a == b and len(a) > 0                                   # greedy by default: repeatable
    assert not lib.oge_engine_generate(None, b"x", 1) and b"NULL" in lib.oge_last_error()
    lib.oge_engine_free(eng)
    lib.oge_engine_free(None)
    lib.oge_string_free(None)
    lib.oge_sampler_free(None)


def test_foreign_sampler_sees_logits_history_and_is_consumed(lib, model_dir):
    lib.oge_sampler_new.restype = ctypes.c_void_p
    lib.oge_sampler_new.argtypes = [VTable]
    eng = lib.oge_engine_load(model_dir.encode())
    seen = {"steps": [], "hist": [], "freed": 0, "vocab": 0}

    def pick(user, logits, n, generated, gen_len, step):
        seen["steps"].append(step)
        seen["hist"].append([generated[i] for i in range(gen_len)])
        seen["vocab"] = n
        row = np.ctypeslib.as_array(logits, shape=(n,))
        return int(np.argmax(row))

    def freed(user):
        seen["freed"] += 1

    cb, fcb = SAMPLE_FN(pick), FREE_FN(freed)
    smp = lib.oge_sampler_new(VTable(None, cb, b"argmax-from-test", fcb))
    assert smp
    text = _take(lib, lib.oge_engine_generate_with_sampler(eng, b"hello", 5, smp))
    assert seen["steps"] == [0, 1, 2, 3, 4] and seen["freed"] == 1 and seen["vocab"] == 32000
    assert [len(h) for h in seen["hist"]] == [0, 1, 2, 3, 4]
    assert text == _take(lib, lib.oge_engine_generate(eng, b"hello", 5))          # argmax sampler == built-in greedy
    bad_cb = SAMPLE_FN(lambda *a: 10**6)                                           # must outlive the call that uses it
    bad = lib.oge_sampler_new(VTable(None, bad_cb, None, fcb))
    assert not lib.oge_engine_generate_with_sampler(eng, b"hello", 2, bad)
    assert b"outside the vocabulary" in lib.oge_last_error() and seen["freed"] == 2   # consumed on failure too
    assert not lib.oge_sampler_new(VTable(None, SAMPLE_FN(), None, FREE_FN()))    # sample is required
    lib.oge_engine_free(eng)


@pytest.mark.skipif(shutil.which("gcc") is None, reason="needs a C compiler")
def test_c_program_embeds_the_engine(lib, model_dir, tmp_path):
    exe = tmp_path / "custom_sampler"
    libdir = os.path.join(ROOT, "onnx_genai_b200", "_lib")
    subprocess.run(["gcc", os.path.join(ROOT, "examples", "c", "custom_sampler.c"), "-I", os.path.join(ROOT, "csrc", "capi"),
                    "-L", libdir, "-lonnx_genai_b200", f"-Wl,-rpath,{libdir}", "-lm", "-o", str(exe)], check=True)
    env = dict(os.environ, ONNX_GENAI_B200_PYTHON=sys.executable, ONNX_GENAI_B200_ROOT=ROOT, CUDA_VISIBLE_DEVICES="")
    proc = subprocess.run([str(exe), model_dir, "hello", "6"], env=env, capture_output=True, text=True, timeout=300)
    assert proc.returncode == 0, proc.stderr[-2000:]
    assert "calls=6 freed=1" in proc.stderr
    lines = proc.stdout.splitlines()
    assert len(lines) >= 1 and len(proc.stdout.strip()) > 0
