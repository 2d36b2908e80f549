"""Gates that are tests: ABI drift between the C header, the ctypes table and the built library; commands that the
documents tell a reader to run; kernels that must not synchronise inside a captured step; machine paths and document names that must not appear."""
import ctypes
import importlib
import os
import re

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
PKG = os.path.join(ROOT, "onnx_genai_b200")


def _read(path):
    with open(path, encoding="utf-8", errors="replace") as f:
        return f.read()


def _sources(exts, roots=("onnx_genai_b200", "csrc", "tests", "examples")):
    for top in roots:
        for dirpath, _dirs, files in os.walk(os.path.join(ROOT, top)):
            if "__pycache__" in dirpath:
                continue
            for name in files:
                if name.endswith(exts):
                    yield os.path.join(dirpath, name)
    for name in ("bench.py", "__graft_entry__.py"):
        if name.endswith(exts):
            yield os.path.join(ROOT, name)


def test_every_kernel_entry_point_in_the_header_is_bound_with_the_same_arity():
    from onnx_genai_b200.ops import _native
    import onnx_genai_b200.ops.moe  # noqa: F401  (registers its entry points)
    import onnx_genai_b200.ops.quant  # noqa: F401
    import onnx_genai_b200.ops.sequence  # noqa: F401
    import onnx_genai_b200.utils.vmm  # noqa: F401

    header = _read(os.path.join(ROOT, "csrc", "kernels", "ogb_kernels.h"))
    decls = re.findall(r"\b(?:int|void\*?|int64_t|uint64_t)\s+(ogb_\w+)\s*\(([^;]*?)\)\s*;", header, flags=re.S)
    assert len(decls) > 20
    missing, arity = [], []
    for name, args in decls:
        n_args = 0 if args.strip() in ("", "void") else len([a for a in args.split(",") if a.strip()])
        sig = _native._SIGNATURES.get(name)
        if sig is None:
            missing.append(name)
        elif len(sig[0]) != n_args:
            arity.append((name, n_args, len(sig[0])))
    assert not arity, f"ctypes argument count differs from the header: {arity}"
    # entry points that only the C++ step executor calls, or that parallel/fused.py binds when a group forms, are not in
    # the table; everything else must be
    internal = {m for m in missing if m.startswith(("ogb_decoder_", "ogb_ipc_", "ogb_tp_", "ogb_moe_", "ogb_cpu_"))
                or m == "ogb_gemm_bf16_scatter"}
    assert set(missing) - internal == set(), sorted(set(missing) - internal)


def test_the_built_library_exports_what_the_bindings_name():
    from onnx_genai_b200.ops import _native
    import onnx_genai_b200.utils.vmm  # noqa: F401

    lib_path = os.path.join(PKG, "_lib", "libogb_cuda.so")
    if not os.path.exists(lib_path):
        pytest.skip("kernel library not built here")
    lib = ctypes.CDLL(lib_path)
    absent = [name for name in _native._SIGNATURES if not hasattr(lib, name)]
    assert absent == [], f"bound but not exported by {lib_path}: {absent}"


def test_documented_module_commands_exist():
    docs = [os.path.join(ROOT, n) for n in ("README.md", "DESIGN.md")] + \
           [os.path.join(ROOT, "profiles", n) for n in os.listdir(os.path.join(ROOT, "profiles"))]
    modules = set()
    for path in docs:
        modules.update(re.findall(r"python3? -m (onnx_genai_b200(?:\.\w+)*)", _read(path)))
    assert len(modules) >= 4
    for mod in sorted(modules):
        spec = importlib.util.find_spec(mod)
        assert spec is not None, f"a document tells the reader to run `python -m {mod}`, which does not exist"
    cli = _read(os.path.join(PKG, "cli.py"))
    for sub in re.findall(r"onnx[-_]genai[-_]b200 (\w[\w-]*)", _read(os.path.join(ROOT, "README.md"))):
        if sub in ("is", "the", "and"):
            continue
        assert f'"{sub}"' in cli, f"README names the CLI subcommand {sub!r}, which cli.py does not define"


def test_a_captured_step_never_synchronises():
    """CUDA-graph capture of the step executor must not meet a stream or device synchronisation, an allocation or a
    blocking copy (a capture that meets one is invalidated)."""
    src = _read(os.path.join(ROOT, "csrc", "kernels", "decoder_step.cu"))
    body = src[src.index("ogb_decoder_step"):]
    for banned in ("cudaStreamSynchronize", "cudaDeviceSynchronize", "cudaMalloc(", "cudaFree(", "cudaMemcpy("):
        assert banned not in body, f"decoder_step.cu calls {banned} inside the step"


def test_sources_name_no_machine_path_and_no_build_document():
    machine = re.compile(r"/root/(repo|reference)|gpurun|SURVEY\.md|DESIGN\.md|VERDICT\.md|ADVICE\.md|BASELINE\.md")
    bad = []
    for path in _sources((".py", ".cu", ".cuh", ".h", ".cpp", ".c")):
        if os.path.basename(path) == "test_lint_gates_cpu.py":
            continue
        m = machine.search(_read(path))
        if m:
            bad.append((os.path.relpath(path, ROOT), m.group(0)))
    assert bad == []


def test_device_waits_are_bounded():
    """Every spin on an mbarrier or a peer flag in the kernels goes through a helper that gives up after a time limit."""
    for path in _sources((".cu", ".cuh"), roots=("csrc",)):
        text = _read(path)
        for m in re.finditer(r"while\s*\(\s*(?:true|1)\s*\)|for\s*\(\s*;\s*;\s*\)", text):
            window = text[m.start():m.start() + 900]
            assert re.search(r"globaltimer|max_spins|kSpinLimit|deadline|timeout|budget|--\s*tries|tries\s*--|spins", window), \
                f"{os.path.relpath(path, ROOT)}: an unconditional loop near offset {m.start()} shows no bound"
