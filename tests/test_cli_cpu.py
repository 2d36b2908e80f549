import json
import subprocess
import sys

import pytest


@pytest.fixture(scope="module")
def pkg_dir(tmp_path_factory):
    out = str(tmp_path_factory.mktemp("cli") / "tiny")
    r = subprocess.run([sys.executable, "-m", "onnx_genai_b200", "export", "--preset", "tiny-llama", "--layers", "1", "--out", out, "--int4"],
                       capture_output=True, text=True)
    assert r.returncode == 0, r.stderr
    return out


def test_version_and_show(pkg_dir):
    r = subprocess.run([sys.executable, "-m", "onnx_genai_b200", "version"], capture_output=True, text=True)
    assert r.stdout.startswith("onnx-genai-b200 ")
    r = subprocess.run([sys.executable, "-m", "onnx_genai_b200", "show", pkg_dir], capture_output=True, text=True)
    assert r.returncode == 0, r.stderr
    info = json.loads(r.stdout)
    assert info["architecture"]["weight_format"] == "int4" and info["operators"]["com.microsoft::MatMulNBits"] >= 7


def test_generate_with_profile_json(pkg_dir, tmp_path):
    prof, trace = str(tmp_path / "p.json"), str(tmp_path / "t.json")
    r = subprocess.run([sys.executable, "-m", "onnx_genai_b200", "--profile-json", prof, "--profile-trace", trace, "generate", pkg_dir,
                        "--prompt", "hello", "--max-new-tokens", "5", "--greedy", "--device", "cpu"], capture_output=True, text=True)
    assert r.returncode == 0, r.stderr
    assert "tok |" in r.stderr
    rep = json.load(open(prof))
    assert rep["completion_tokens"] <= 5 and "itl_ms" in rep and "kv" in rep
    assert json.load(open(trace))["traceEvents"]


def test_validate_reports_problems_and_exit_code(tmp_path):
    import json as _json
    import subprocess
    import sys as _sys

    from onnx_genai_b200.bench.config_bench import _export

    d = tmp_path / "m"
    _export("tiny-llama", str(d), "fp32", layers=1)
    run = lambda: subprocess.run([_sys.executable, "-m", "onnx_genai_b200", "validate", str(d)], capture_output=True, text=True, timeout=300)
    ok = run()
    assert ok.returncode == 0 and _json.loads(ok.stdout)["ok"] is True
    meta = d / "inference_metadata.yaml"
    meta.write_text(meta.read_text().replace("vocab_size: 32000", "vocab_size: 31999"))
    bad = run()
    report = _json.loads(bad.stdout)
    assert bad.returncode == 1 and not report["ok"] and "31999" in report["problems"][0]
    missing = subprocess.run([_sys.executable, "-m", "onnx_genai_b200", "validate", str(tmp_path / "nope")], capture_output=True, text=True)
    assert missing.returncode == 1 and "not a directory" in missing.stdout


@pytest.mark.parametrize("proposer", ["ngram", "mtp", "eagle3", "shared-kv"])
def test_generate_with_each_proposer_keeps_the_greedy_text(pkg_dir, proposer):
    base = [sys.executable, "-m", "onnx_genai_b200", "generate", pkg_dir, "--prompt", "hello hello hello", "--max-new-tokens", "8",
            "--greedy", "--device", "cpu", "--raw"]
    plain = subprocess.run(base, capture_output=True, text=True)
    spec = subprocess.run(base + ["--proposer", proposer, "--draft-tokens", "3", "--cpu-cores", "2", "--host-ram-limit", "2GiB"],
                          capture_output=True, text=True)
    assert plain.returncode == 0 and spec.returncode == 0, spec.stderr
    assert spec.stdout == plain.stdout


def test_proposer_draft_needs_a_draft_model(pkg_dir):
    r = subprocess.run([sys.executable, "-m", "onnx_genai_b200", "generate", pkg_dir, "--prompt", "x", "--proposer", "draft", "--device", "cpu"],
                       capture_output=True, text=True)
    assert r.returncode != 0 and "--draft-model" in r.stderr
    ok = subprocess.run([sys.executable, "-m", "onnx_genai_b200", "generate", pkg_dir, "--prompt", "hello", "--max-new-tokens", "4", "--greedy",
                         "--device", "cpu", "--draft-model", pkg_dir], capture_output=True, text=True)
    assert ok.returncode == 0, ok.stderr


def test_graph_backend_prints_the_same_greedy_text(pkg_dir):
    base = [sys.executable, "-m", "onnx_genai_b200", "generate", pkg_dir, "--prompt", "hello world", "--max-new-tokens", "8", "--greedy",
            "--device", "cpu", "--raw"]
    native = subprocess.run(base, capture_output=True, text=True)
    graph = subprocess.run(base + ["--backend", "graph"], capture_output=True, text=True)
    assert native.returncode == 0 and graph.returncode == 0, graph.stderr
    assert graph.stdout == native.stdout and "backend graph" in graph.stderr


def test_unrecognised_decoder_points_to_the_graph_backend(tmp_path):
    import os

    ref = os.environ.get("OGB_REFERENCE_DIR", os.path.join(os.path.expanduser("~"), "reference"))
    src = os.path.join(ref, "tests", "fixtures", "tiny-llm")
    if not os.path.isdir(src):
        pytest.skip("the upstream tiny-llm fixture is not available on this machine")
    base = [sys.executable, "-m", "onnx_genai_b200", "generate", src, "--prompt", "ab", "--max-new-tokens", "3", "--greedy", "--device", "cpu", "--raw"]
    fast = subprocess.run(base, capture_output=True, text=True)
    assert fast.returncode == 2 and "--backend graph" in fast.stderr
    graph = subprocess.run(base + ["--backend", "graph"], capture_output=True, text=True)
    assert graph.returncode == 0 and "backend graph" in graph.stderr, graph.stderr


def test_repl_commands_media_device_and_backend(tmp_path):
    """The REPL's slash commands, driven without a terminal: attachments go to the media chat with the next prompt, /ep
    reloads the engine on the other device, /backend switches the decode path, unknown input is explained."""
    import argparse

    from onnx_genai_b200 import cli

    class FakeTok:
        def encode(self, text):
            return [ord(c) % 50 for c in text][:8]

        def decode(self, ids):
            return "ids:" + ",".join(str(i) for i in ids)

    class FakeEngine:
        loads = []

        def __init__(self, device):
            self.llm = argparse.Namespace(device=device)
            self.tokenizer = FakeTok()
            self.sessions = 0
            FakeEngine.loads.append(device)

        def create_session(self):
            self.sessions += 1
            return self.sessions

        def reset_session(self, s):
            self.was_reset = s

        def session_len(self, s):
            return 0

        def resource_snapshot(self):
            return {"kv": 1}

    class FakeMedia:
        accepts = {"image": True, "audio": False}

        def __init__(self):
            self.calls = []

        def generate(self, ids, image=None, audio=None, max_new_tokens=64):
            self.calls.append((list(ids), image, audio, max_new_tokens))
            return [7, 8, 9]

    args = argparse.Namespace(device="cpu", backend="native", raw=True, max_tokens=5)
    said = []
    media = FakeMedia()
    prof = argparse.Namespace(enabled=False)
    repl = cli.Repl(args, prof, loader=lambda a: FakeEngine(a.device), media_chat=media, out=said.append)
    repl.command("/help")
    assert "/image PATH|clear" in said[-1] and "/backend [native|graph]" in said[-1] and "/ep [cpu|cuda]" in said[-1]
    img = tmp_path / "cat.png"
    img.write_bytes(b"\x89PNG1234")
    repl.command(f"/image {img}")
    assert "image attached (8 bytes)" in said[-1]
    repl.command("/image")
    assert "8 bytes" in said[-1]
    repl.command(f"/audio {img}")
    assert "no audio pipeline" in said[-1] and "--multimodal-package" in said[-1]
    repl.command("/image /nonexistent/file.png")
    assert "No such file" in said[-1]
    got = []
    assert repl.prompt("what is this", on_text=got.append) is None
    assert got == ["ids:7,8,9"] and media.calls[0][1] == b"\x89PNG1234" and media.calls[0][3] == 5 and repl.images == []
    repl.command("/ep")
    assert "execution device: cpu" in said[-1]
    repl.command("/ep tpu")
    assert "expected cpu or cuda" in said[-1]
    repl.command("/ep cuda")
    assert ("no CUDA device" in said[-1]) or FakeEngine.loads[-1] == "cuda"
    repl.command("/ep cpu")
    assert FakeEngine.loads[-1] == "cpu" and "reloaded on cpu" in said[-1]
    repl.command("/backend")
    assert "decode backend: native" in said[-1]
    repl.command("/backend graph")
    assert args.backend == "graph" and "graph executor" in said[-1]
    repl.command("/backend warp")
    assert "expected native or graph" in said[-1]
    repl.command("/profile")
    assert prof.enabled is True
    repl.command("/bogus")
    assert "unknown command /bogus" in said[-1]
    repl.command("/quit")
    assert repl.done
