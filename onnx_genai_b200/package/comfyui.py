"""ComfyUI "Save (API Format)" graphs -> the canonical workflow form of the inference metadata.

ComfyUI exports a text-to-image graph as a JSON object of numbered nodes, each with a ``class_type`` and ``inputs``
whose values are literals or ``[node id, output index]`` links.  The reference converts such a graph into a
``pipeline.workflow`` document so its workflow runtime can execute it
(crates/onnx-genai-comfyui-config, README.md:396-415).  This importer does the same for the classic latent-diffusion
graph::

    CheckpointLoaderSimple -> CLIPTextEncode (positive / negative) -> KSampler <- EmptyLatentImage
                                                                        |
                                                                    VAEDecode -> SaveImage | PreviewImage

and emits a document with one component per model part (``text_encoder``, ``denoiser``, ``vae_decoder``), policy
components for the sampler (``solver_step`` named after ``sampler_name`` / ``scheduler``) and, when ``cfg`` is not 1,
classifier-free guidance (a second denoiser pass on the negative conditioning and a ``guidance`` combine), a
denoising ``loop`` of ``steps`` iterations, the VAE decode and an ``emit`` of the image.  Graph parameters (steps, cfg,
seed, size, sampler) become generation defaults.  Graphs with other node types are rejected with the node id, its
class and the list of supported classes; nothing is guessed.

This build has no diffusion executor: the output is a validated document (see :mod:`onnx_genai_b200.metadata.workflow`)
for tools that consume the standard, not something ``Engine`` can run.
"""
from __future__ import annotations

import os

SUPPORTED = ("CheckpointLoaderSimple", "CLIPTextEncode", "EmptyLatentImage", "KSampler", "VAEDecode", "SaveImage", "PreviewImage")


class ComfyImportError(ValueError):
    pass


def _link(value, what, node_id):
    if not (isinstance(value, (list, tuple)) and len(value) == 2 and isinstance(value[1], int)):
        raise ComfyImportError(f"node {node_id}: input '{what}' must be a link [node id, output index], found {value!r}")
    return str(value[0]), int(value[1])


def _contract(dtype, shape):
    return {"dtype": dtype, "rank": len(shape), "shape": list(shape), "batch_layout": {"kind": "request_aligned", "axis": 0}}


def import_comfyui(graph: dict) -> dict:
    """``graph``: the parsed API-format JSON.  Returns an inference-metadata document (a plain dict)."""
    if not isinstance(graph, dict) or not graph:
        raise ComfyImportError("the ComfyUI API export is a JSON object of nodes keyed by id; this is not one")
    nodes = {}
    for nid, node in graph.items():
        if not isinstance(node, dict) or "class_type" not in node:
            raise ComfyImportError(f"node {nid}: every node needs a 'class_type' (is this the API format, not the UI save format?)")
        if node["class_type"] not in SUPPORTED:
            raise ComfyImportError(f"node {nid} is a {node['class_type']!r}; this importer handles {', '.join(SUPPORTED)}")
        nodes[str(nid)] = node

    def of_class(cls):
        return [(nid, n) for nid, n in nodes.items() if n["class_type"] == cls]

    sinks = of_class("SaveImage") + of_class("PreviewImage")
    if len(sinks) != 1:
        raise ComfyImportError(f"expected one SaveImage / PreviewImage node, found {len(sinks)}")
    sink_id, sink = sinks[0]
    dec_id, _ = _link(sink["inputs"].get("images"), "images", sink_id)
    dec = nodes.get(dec_id)
    if dec is None or dec["class_type"] != "VAEDecode":
        raise ComfyImportError(f"node {sink_id}: 'images' must come from a VAEDecode node")
    ks_id, _ = _link(dec["inputs"].get("samples"), "samples", dec_id)
    ks = nodes.get(ks_id)
    if ks is None or ks["class_type"] != "KSampler":
        raise ComfyImportError(f"node {dec_id}: 'samples' must come from a KSampler node")
    ki = ks["inputs"]
    ckpt_id, model_out = _link(ki.get("model"), "model", ks_id)
    ckpt = nodes.get(ckpt_id)
    if ckpt is None or ckpt["class_type"] != "CheckpointLoaderSimple" or model_out != 0:
        raise ComfyImportError(f"node {ks_id}: 'model' must be output 0 of a CheckpointLoaderSimple node")
    vae_id, vae_out = _link(dec["inputs"].get("vae"), "vae", dec_id)
    if vae_id != ckpt_id or vae_out != 2:
        raise ComfyImportError(f"node {dec_id}: 'vae' must be output 2 of the checkpoint loader (node {ckpt_id})")
    cond = {}
    for side in ("positive", "negative"):
        cid, _ = _link(ki.get(side), side, ks_id)
        c = nodes.get(cid)
        if c is None or c["class_type"] != "CLIPTextEncode":
            raise ComfyImportError(f"node {ks_id}: '{side}' must come from a CLIPTextEncode node")
        clip_id, clip_out = _link(c["inputs"].get("clip"), "clip", cid)
        if clip_id != ckpt_id or clip_out != 1:
            raise ComfyImportError(f"node {cid}: 'clip' must be output 1 of the checkpoint loader (node {ckpt_id})")
        cond[side] = str(c["inputs"].get("text", ""))
    lat_id, _ = _link(ki.get("latent_image"), "latent_image", ks_id)
    lat = nodes.get(lat_id)
    if lat is None or lat["class_type"] != "EmptyLatentImage":
        raise ComfyImportError(f"node {ks_id}: 'latent_image' must come from an EmptyLatentImage node (image-to-image graphs are not handled)")
    width, height = int(lat["inputs"].get("width", 512)), int(lat["inputs"].get("height", 512))
    batch = int(lat["inputs"].get("batch_size", 1))
    if width % 8 or height % 8:
        raise ComfyImportError(f"node {lat_id}: width and height must be multiples of 8 (the VAE's stride), got {width}x{height}")
    steps, cfg = int(ki.get("steps", 20)), float(ki.get("cfg", 7.0))
    denoise = float(ki.get("denoise", 1.0))
    if denoise != 1.0:
        raise ComfyImportError(f"node {ks_id}: denoise={denoise} (partial denoising) is not handled; use 1.0")
    sampler, scheduler = str(ki.get("sampler_name", "euler")), str(ki.get("scheduler", "normal"))
    guided = cfg != 1.0
    stem = os.path.splitext(os.path.basename(str(ckpt["inputs"].get("ckpt_name", "checkpoint"))))[0]

    def onnx(part):
        return {"implementation": {"kind": "onnx", "artifact": f"{stem}/{part}.onnx"}}

    inputs = {
        "request.positive_ids": {"contract": _contract("int64", ["batch", "sequence"]), "source": {"kind": "request"}, "required": True,
                                 "role": {"kind": "runtime", "version": "1.0", "role": "prompt_tokens"}},
        "request.noise": {"contract": _contract("float32", ["batch", 4, height // 8, width // 8]), "source": {"kind": "application", "name": "noise"},
                          "required": True, "role": {"kind": "opaque"}},
        "request.max_iterations": {"contract": {"dtype": "int64", "rank": 1, "shape": [1]}, "source": {"kind": "request"}, "required": False,
                                   "default": steps, "role": {"kind": "runtime", "version": "1.0", "role": "max_output_tokens"}},
        "package.false": {"contract": {"dtype": "bool", "rank": 1, "shape": [1]}, "source": {"kind": "literal"}, "default": False,
                          "role": {"kind": "opaque"}},
        "package.loop_active": {"contract": {"dtype": "bool", "rank": 1, "shape": [1]}, "source": {"kind": "literal"}, "default": True,
                                "role": {"kind": "opaque"}},
    }
    components = {"text_encoder": onnx("text_encoder"), "denoiser": onnx("unet"), "vae_decoder": onnx("vae_decoder"),
                  "schedule": {"implementation": {"kind": "onnx", "artifact": f"policies/schedule_{scheduler}.onnx"}},
                  "solver_step": {"implementation": {"kind": "onnx", "artifact": f"policies/solver_{sampler}.onnx"}},
                  "continue_predicate": {"implementation": {"kind": "onnx", "artifact": "policies/continue.onnx"}}}
    setup = [{"kind": "invoke", "component": "schedule", "inputs": {}, "outputs": {"schedule": "diffusion.schedule"}},
             {"kind": "invoke", "component": "text_encoder", "inputs": {"input_ids": "request.positive_ids"},
              "outputs": {"encoder_hidden_states": "conditioning.positive"}}]
    body = [{"kind": "invoke", "component": "denoiser",
             "inputs": {"sample": "latent_state", "step": "loop.iteration", "schedule": "diffusion.schedule",
                        "encoder_hidden_states": "conditioning.positive"}, "outputs": {"noise_pred": "denoiser.positive"}}]
    estimate = "denoiser.positive"
    if guided:
        inputs["request.negative_ids"] = {"contract": _contract("int64", ["batch", "sequence"]), "source": {"kind": "request"}, "required": True,
                                          "role": {"kind": "runtime", "version": "1.0", "role": "negative_prompt_tokens"}}
        inputs["package.guidance_scale"] = {"contract": {"dtype": "float32", "rank": 1, "shape": [1]}, "source": {"kind": "literal"},
                                            "default": cfg, "role": {"kind": "opaque"}}
        components["guidance"] = {"implementation": {"kind": "onnx", "artifact": "policies/classifier_free_guidance.onnx"}}
        setup.append({"kind": "invoke", "component": "text_encoder", "inputs": {"input_ids": "request.negative_ids"},
                      "outputs": {"encoder_hidden_states": "conditioning.negative"}})
        body.append({"kind": "invoke", "component": "denoiser",
                     "inputs": {"sample": "latent_state", "step": "loop.iteration", "schedule": "diffusion.schedule",
                                "encoder_hidden_states": "conditioning.negative"}, "outputs": {"noise_pred": "denoiser.negative"}})
        body.append({"kind": "invoke", "component": "guidance",
                     "inputs": {"conditional": "denoiser.positive", "unconditional": "denoiser.negative", "scale": "package.guidance_scale"},
                     "outputs": {"guided": "denoiser.guided"}})
        estimate = "denoiser.guided"
    body += [{"kind": "invoke", "component": "solver_step",
              "inputs": {"sample": "latent_state", "step": "loop.iteration", "schedule": "diffusion.schedule", "derivative": estimate},
              "outputs": {"next_state": "latent.body"}},
             {"kind": "invoke", "component": "continue_predicate", "inputs": {"done": "package.false"}, "outputs": {"continue": "loop.continue"}}]
    latent_contract = _contract("float32", ["batch", 4, height // 8, width // 8])
    workflow = {
        "manifest": {"capabilities": ["workflow_ssa", "typed_emit", "loop_induction_values"]},
        "inputs": inputs,
        "outputs": {"image": {"contract": _contract("float32", ["batch", 3, height, width]), "role": "image", "stage": "post_adapter"}},
        "components": components,
        "state": {"latent_state": {"contract": latent_contract, "scope": "invocation", "initializer": "request.noise",
                                   "recurrence": {"kind": "invariant"}},
                  "loop_active": {"contract": {"dtype": "bool", "rank": 1, "shape": [1]}, "scope": "invocation", "initializer": "package.loop_active",
                                  "recurrence": {"kind": "invariant"}}},
        "steps": [
            {"kind": "loop", "setup": setup, "steps": body, "continue_when": "loop_active", "max_iterations": "request.max_iterations",
             "carried": [{"cell": "latent_state", "initial": "request.noise", "next": "latent.body"},
                         {"cell": "loop_active", "next": "loop.continue"}],
             "iteration": {"value": "loop.iteration", "contract": {"dtype": "int64", "rank": 1, "shape": [1]}}},
            {"kind": "invoke", "component": "vae_decoder", "inputs": {"latent": "latent_state"}, "outputs": {"image": "vae.image"}},
            {"kind": "emit", "value": "vae.image", "output": "image", "mode": "replace"},
        ],
    }
    prefix = str(sink["inputs"].get("filename_prefix", "")) if sink["class_type"] == "SaveImage" else ""
    return {
        "schema_version": "1.0",
        "pipeline": {"workflow": workflow},
        "generation": {"defaults": {"steps": steps, "guidance_scale": cfg, "seed": int(ki.get("seed", 0)), "sampler": sampler,
                                    "scheduler": scheduler, "width": width, "height": height, "batch_size": batch,
                                    "positive_prompt": cond["positive"], "negative_prompt": cond["negative"],
                                    **({"filename_prefix": prefix} if prefix else {})}},
    }


def main(argv=None) -> int:
    import argparse
    import json
    import sys

    import yaml

    ap = argparse.ArgumentParser(description="Convert a ComfyUI API-format export into an inference-metadata workflow document")
    ap.add_argument("graph", help="ComfyUI 'Save (API Format)' JSON file")
    ap.add_argument("-o", "--out", default="-", help="output YAML (default: stdout)")
    args = ap.parse_args(argv)
    with open(args.graph, encoding="utf-8") as f:
        doc = import_comfyui(json.load(f))
    text = yaml.safe_dump(doc, sort_keys=False)
    if args.out == "-":
        sys.stdout.write(text)
    else:
        with open(args.out, "w", encoding="utf-8") as f:
            f.write(text)
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
