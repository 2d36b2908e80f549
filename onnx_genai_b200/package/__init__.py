"""Model directories and ORT-style model packages.

Two layouts are accepted, as in the reference (crates/onnx-genai-ort/src/loader.rs:28-130,
crates/onnx-model-package/src/lib.rs, docs/genai/MODEL_PACKAGE.md:66-118):

* flat directory: ``tokenizer.json`` (mandatory), ``decoder.onnx`` or the single ``*.onnx``,
  optional ``inference_metadata.{yaml,yml,json}``, ``genai_config.json`` (import only),
  ``chat_template.jinja`` or ``tokenizer_config.json["chat_template"]``, external ``*.onnx.data``;
* package directory: ``manifest.json`` (``schema_version "1.x"``, ``components{model{variants
  {name: {variant_directory, ep, device, compatibility_string, executor_info}}}}``) with
  content-addressed ``shared_assets/sha256-<digest>/`` directories referenced as
  ``sha256:<digest>[/tail]``.  Variant selection prefers an entry whose ``ep`` / ``device`` match.
"""
from __future__ import annotations

import hashlib
import json
import os
from dataclasses import dataclass, field

from .. import metadata as md


class PackageError(ValueError):
    pass


@dataclass
class ModelDirectory:
    root: str
    model_path: str
    tokenizer_path: str | None
    metadata_path: str | None
    chat_template: str | None = None
    genai_config: dict | None = None
    variant: str | None = None
    manifest: dict | None = None
    extra: dict = field(default_factory=dict)

    def load_metadata(self) -> md.InferenceMetadata:
        if self.metadata_path:
            return md.load(self.metadata_path)
        if self.genai_config is not None:
            from .genai_config import graph_ports, import_genai_config

            graph = None
            if self.model_path and os.path.exists(self.model_path):
                try:                                  # ports only: the weights stay on disk (external data is mapped lazily)
                    from .onnx_pb import load_model

                    graph = graph_ports(load_model(self.model_path))
                except Exception:                     # an unreadable graph leaves the declared name patterns in charge
                    graph = None
            return md.parse(import_genai_config(self.genai_config, graph=graph))
        return md.InferenceMetadata()


def directory_hash(path: str) -> str:
    """Canonical hash of a shared-asset directory: sha256 over sorted '<file-sha256>  <relative-path>\\n' lines."""
    lines = []
    for base, dirs, files in os.walk(path):
        for name in files:
            full = os.path.join(base, name)
            if os.path.islink(full):
                raise PackageError(f"{full}: symlinks are not allowed inside shared assets")
            h = hashlib.sha256()
            with open(full, "rb") as f:
                for chunk in iter(lambda: f.read(1 << 20), b""):
                    h.update(chunk)
            rel = os.path.relpath(full, path).replace(os.sep, "/")
            lines.append(f"{h.hexdigest()}  {rel}\n")
    return hashlib.sha256("".join(sorted(lines)).encode()).hexdigest()


def _confined(root: str, rel: str) -> str:
    full = os.path.realpath(os.path.join(root, rel))
    if not (full + os.sep).startswith(os.path.realpath(root) + os.sep) and full != os.path.realpath(root):
        raise PackageError(f"path {rel!r} escapes the package root; portable packages are confined to their directory")
    return full


def resolve_ref(root: str, ref: str, manifest: dict | None = None) -> str:
    """Resolve a ``sha256:<digest>[/tail]`` reference or a package-relative path."""
    if ref.startswith("sha256:"):
        digest, _, tail = ref[len("sha256:"):].partition("/")
        base = ((manifest or {}).get("shared_assets") or {}).get(digest) or os.path.join("shared_assets", "sha256-" + digest)
        return _confined(root, os.path.join(base, tail) if tail else base)
    return _confined(root, ref)


def _find_onnx(d: str) -> str:
    for name in ("decoder.onnx", "decoder.onnx.textproto"):
        if os.path.exists(os.path.join(d, name)):
            return os.path.join(d, name)
    cands = sorted(f for f in os.listdir(d) if f.endswith(".onnx"))
    if not cands:                      # text-format models (fixtures, hand-written graphs)
        cands = sorted(f for f in os.listdir(d) if f.endswith(".onnx.textproto"))
    if len(cands) == 1:
        return os.path.join(d, cands[0])
    if not cands:
        raise PackageError(f"{d}: no decoder.onnx and no *.onnx file found")
    raise PackageError(f"{d}: several *.onnx files {cands} and none is named decoder.onnx; name the decoder graph decoder.onnx")


def _chat_template(d: str) -> str | None:
    p = os.path.join(d, "chat_template.jinja")
    if os.path.exists(p):
        return open(p, encoding="utf-8").read()
    p = os.path.join(d, "tokenizer_config.json")
    if os.path.exists(p):
        try:
            return json.load(open(p, encoding="utf-8")).get("chat_template")
        except Exception:
            return None
    return None


def open_model_directory(path: str, ep: str = "cuda", device: str = "gpu", variant: str | None = None) -> ModelDirectory:
    path = os.path.abspath(path)
    if not os.path.isdir(path):
        raise PackageError(f"{path}: not a directory; pass a model directory or a model package")
    manifest_path = os.path.join(path, "manifest.json")
    if os.path.exists(manifest_path):
        manifest = json.load(open(manifest_path, encoding="utf-8"))
        if "components" in manifest:
            return _open_package(path, manifest, ep, device, variant)
    tok = os.path.join(path, "tokenizer.json")
    gc = os.path.join(path, "genai_config.json")
    return ModelDirectory(root=path, model_path=_find_onnx(path), tokenizer_path=tok if os.path.exists(tok) else None,
                          metadata_path=md.find(path), chat_template=_chat_template(path),
                          genai_config=json.load(open(gc)) if os.path.exists(gc) else None)


def _open_package(root: str, manifest: dict, ep: str, device: str, variant: str | None) -> ModelDirectory:
    ver = str(manifest.get("schema_version", "1.0"))
    if ver.split(".")[0] != "1":
        raise PackageError(f"manifest.json: schema_version {ver!r} has an unsupported major version (this reader handles 1.x)")
    comps = manifest.get("components") or {}
    name = "model" if "model" in comps else ("decoder" if "decoder" in comps else None)
    if name is None:
        raise PackageError(f"manifest.json: no 'model' (or 'decoder') component among {sorted(comps)}")
    comp = comps[name]
    if isinstance(comp, str):  # external component directory with component.json
        comp_dir = _confined(root, comp)
        comp = json.load(open(os.path.join(comp_dir, "component.json"), encoding="utf-8"))
        comp_root = comp_dir
    else:
        comp_root = _confined(root, comp.get("component_directory", name)) if os.path.isdir(os.path.join(root, comp.get("component_directory", name))) else root
    variants = comp.get("variants") or {}
    if not variants:
        raise PackageError(f"manifest.json: component {name!r} has no variants")
    if variant is None:
        def score(item):
            v = item[1]
            return (str(v.get("ep", "")).lower().startswith(ep.lower()), str(v.get("device", "")).lower() == device.lower())
        variant = max(sorted(variants.items()), key=score)[0]
    if variant not in variants:
        raise PackageError(f"manifest.json: variant {variant!r} not found; available: {sorted(variants)}")
    v = variants[variant]
    vdir = _confined(comp_root, v.get("variant_directory", variant))
    info = (v.get("executor_info") or {})
    assets = info.get("assets") or comp.get("assets") or manifest.get("assets") or {}

    def asset(key, default_name):
        ref = assets.get(key)
        if ref:
            return resolve_ref(root, ref, manifest)
        for d in (vdir, comp_root, root):
            p = os.path.join(d, default_name)
            if os.path.exists(p):
                return p
        return None

    tok = asset("tokenizer", "tokenizer.json")
    tmpl_path = asset("chat_template", "chat_template.jinja")
    meta = md.find(vdir) or md.find(comp_root) or md.find(root)
    return ModelDirectory(root=root, model_path=_find_onnx(vdir), tokenizer_path=tok, metadata_path=meta,
                          chat_template=open(tmpl_path, encoding="utf-8").read() if tmpl_path else _chat_template(vdir),
                          variant=variant, manifest=manifest)


def write_package(root: str, variant_dirs: dict, shared_files: dict | None = None, package_name: str = "model") -> dict:
    """Author a package: ``variant_dirs`` = {variant: {"ep":..., "device":..., "directory": existing dir}};
    ``shared_files`` = {"tokenizer": path, "chat_template": path} are stored content-addressed."""
    import shutil

    os.makedirs(root, exist_ok=True)
    assets = {}
    if shared_files:
        stage = os.path.join(root, "shared_assets", "_staging")
        os.makedirs(stage, exist_ok=True)
        for key, src in shared_files.items():
            shutil.copy(src, os.path.join(stage, os.path.basename(src)))
        digest = directory_hash(stage)
        final = os.path.join(root, "shared_assets", "sha256-" + digest)
        if os.path.exists(final):
            shutil.rmtree(stage)
        else:
            os.rename(stage, final)
        for key, src in shared_files.items():
            assets[key] = f"sha256:{digest}/{os.path.basename(src)}"
    variants = {}
    for vname, spec in variant_dirs.items():
        dst = os.path.join(root, "model", vname)
        if os.path.abspath(spec["directory"]) != os.path.abspath(dst):
            shutil.copytree(spec["directory"], dst, dirs_exist_ok=True)
        variants[vname] = {"variant_directory": vname, "ep": spec.get("ep", "cuda"), "device": spec.get("device", "gpu"),
                           "compatibility_string": spec.get("compatibility_string", "sm_100a"),
                           "executor_info": {"onnx_genai_b200": {"kernels": "sm_100a"}, "assets": assets}}
    manifest = {"schema_version": "1.0", "package_name": package_name, "layout": "portable",
                "components": {"model": {"component_directory": "model", "variants": variants}}}
    with open(os.path.join(root, "manifest.json"), "w", encoding="utf-8") as f:
        json.dump(manifest, f, indent=2)
    return manifest
