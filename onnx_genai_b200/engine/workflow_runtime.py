"""Executor for the workflow form of the inference metadata: invoke / sequence / loop / branch / emit over components.

A workflow names components and wires their ports with single-assignment values, state cells carried around loops
and typed emits.  The reference runs such documents for every multi-model package it serves -- vision-language,
speech, text-to-speech, diffusion, video -- by interpreting the step tree over ONNX sessions
(crates/onnx-genai-engine/src/pipeline/workflow.rs: loop handling around lines 1155-1220, value retention 249-267).
This executor interprets the same tree over *bound components*: any callable that maps a dict of input ports to a
dict of output ports.  A component can be a torch module on the GPU, a numpy policy, or an adapter around
:class:`onnx_genai_b200.engine.api.Engine`; the executor owns only the control flow and the value environment:

* ``invoke``   gathers the bound input ports, calls the component, binds its output ports (missing outputs are errors);
* ``sequence`` runs steps in order;
* ``loop``     runs ``setup`` once, seeds the carried cells, then while the ``continue_when`` cell is true and fewer than
  ``max_iterations`` iterations have run: defines the iteration value, runs the body in a fresh scope (so body values
  are single-assignment per iteration), and moves each carried cell to its ``next`` value;
* ``branch``   picks the arm whose label equals the predicate (booleans read ``true`` / ``false``), else ``default``, and
  binds the declared branch outputs from that arm;
* ``emit``     (``replace`` | ``append`` | ``event``), gated by ``when``, trimmed by ``valid_length`` along axis 0.

State cells with ``scope: session`` survive between runs of one :class:`WorkflowSession` and can be checkpointed and
restored; ``invocation`` cells start from their initializer on every run.  Literal inputs take their declared default,
request inputs must be supplied when ``required``.
"""
from __future__ import annotations

import copy

import numpy as np

from ..metadata import workflow as wfm


_NP_DTYPE = {"float32": np.float32, "float16": np.float16, "float64": np.float64, "int64": np.int64, "int32": np.int32, "bool": np.bool_,
             "uint8": np.uint8, "int8": np.int8}


class WorkflowRuntimeError(RuntimeError):
    pass


def _scalar(v, what):
    """First element of a tensor-like as a Python scalar."""
    if hasattr(v, "detach"):
        v = v.detach().reshape(-1)[:1].cpu().numpy()
    a = np.asarray(v).reshape(-1)
    if a.size == 0:
        raise WorkflowRuntimeError(f"{what} is empty; a scalar (or one-element tensor) is needed")
    return a[0].item()


def _all_true(v) -> bool:
    """A per-row boolean cell keeps the loop alive while any row is active."""
    if hasattr(v, "detach"):
        return bool(v.detach().any().item())
    return bool(np.asarray(v).any())


class _Scope:
    """Chained value environment: reads fall through to the parent, writes stay local."""

    def __init__(self, parent=None):
        self.parent, self.values = parent, {}

    def has(self, name):
        s = self
        while s is not None:
            if name in s.values:
                return True
            s = s.parent
        return False

    def get(self, name):
        s = self
        while s is not None:
            if name in s.values:
                return s.values[name]
            s = s.parent
        raise KeyError(name)

    def set(self, name, value):
        self.values[name] = value


def _invoked_components(steps):
    """Names of the components that the step tree calls."""
    for s in steps:
        if s.kind == "invoke":
            yield s.component
        for group in (s.steps, s.setup, list(s.cases.values()), [s.default] if s.default is not None else []):
            yield from _invoked_components(group)


class WorkflowSession:
    def __init__(self, workflow, components: dict, *, validate: bool = True):
        """``workflow``: a parsed :class:`Workflow`, or the mapping under ``pipeline.workflow``.  ``components``: name -> callable(dict) -> dict."""
        self.wf = workflow if isinstance(workflow, wfm.Workflow) else wfm.parse(workflow)
        if validate:
            problems = wfm.validate(self.wf)
            if problems:
                raise WorkflowRuntimeError("the workflow does not validate:\n  " + "\n  ".join(problems))
        missing = sorted(set(self._invoked(self.wf.steps)) - set(components))
        if missing:
            raise WorkflowRuntimeError("no implementation bound for component(s) " + ", ".join(missing) +
                                       f" (bound: {', '.join(sorted(components)) or 'none'})")
        self.components = components
        self.session_cells: dict = {}
        self.stats = {"runs": 0, "invocations": {}, "iterations": 0}

    @classmethod
    def from_package(cls, package_dir: str, device="cpu", dtype=None, components: dict | None = None, metadata_name: str = "inference_metadata.yaml"):
        """Bind every ONNX component of a package directory to the generic graph executor (binary ``.onnx`` or text
        ``.onnx.textproto`` artifacts, resolved against the directory); ``components`` supplies or overrides bindings --
        needed for components that are not ONNX graphs (adapters named by an ABI) and for a decoder that should run on
        the engine instead."""
        import os

        import yaml

        from ..package.graph_executor import as_component
        from ..package.onnx_text import load_any

        with open(os.path.join(package_dir, metadata_name), encoding="utf-8") as f:
            doc = yaml.safe_load(f)
        wf = wfm.load_document(doc)
        if wf is None:
            raise WorkflowRuntimeError(f"{package_dir}/{metadata_name} has no pipeline.workflow")
        bound = dict(components or {})
        invoked = set(_invoked_components(wf.steps))
        for name, comp in wf.components.items():
            if name in bound or name not in invoked:      # a declared component that no step calls needs no implementation
                continue
            if comp.kind == "adapter" and comp.abi == "onnx-genai.image-preprocess" and ((doc.get("preprocessing") or {}).get("image")):
                from ..preprocess import image_preprocess_adapter

                bound[name] = image_preprocess_adapter(doc["preprocessing"]["image"], next(iter(comp.inputs), "encoded"))
                continue
            if comp.kind == "adapter" and comp.abi == "onnx-genai.parameter-overlay" and doc.get("adapters"):
                from ..package.graph_executor import tensor_to_torch
                from .lora import AdapterStore, parameter_overlay_adapter

                adapters_doc = doc["adapters"]
                store = AdapterStore(package_dir, adapters_doc)
                target = store.targets.get(str(comp.params.get("parameter")))
                if target is None:
                    raise WorkflowRuntimeError(f"component '{name}' overlays parameter '{comp.params.get('parameter')}', which the adapter "
                                               f"target manifest does not list (it lists {sorted(store.targets)})")
                owner = wf.components.get(target["component"])
                if owner is None or not owner.artifact:
                    raise WorkflowRuntimeError(f"adapter target '{target['id']}' belongs to component '{target['component']}', which has no graph")
                graph = load_any(os.path.join(package_dir, owner.artifact)).graph
                if target["initializer"] not in graph.initializers:
                    raise WorkflowRuntimeError(f"adapter target '{target['id']}': {owner.artifact} has no initializer '{target['initializer']}'")
                bound[name] = parameter_overlay_adapter(tensor_to_torch(graph.initializers[target["initializer"]]), store, target["id"],
                                                        adapters_doc.get("selection") or {}, next(iter(comp.inputs), "input"),
                                                        next(iter(comp.outputs), "output"))
                continue
            if comp.kind == "adapter" and comp.abi == "onnx-genai.grammar-guidance":
                from .constraints import grammar_guidance_adapter

                bound[name] = grammar_guidance_adapter(str(comp.params.get("action", "lookahead")))
                continue
            if comp.kind != "onnx" or not comp.artifact:
                raise WorkflowRuntimeError(f"component '{name}' is a '{comp.kind}' implementation{' (' + comp.abi + ')' if comp.abi else ''}, "
                                           "not an ONNX graph: pass a callable for it in `components`")
            path = os.path.join(package_dir, comp.artifact)
            if not os.path.exists(path):
                raise WorkflowRuntimeError(f"component '{name}': artifact {path} does not exist")
            bound[name] = as_component(load_any(path), device, dtype)
        return cls(wf, bound)

    def _invoked(self, steps):
        return _invoked_components(steps)

    # -- checkpoint / restore of session-scoped state ---------------------------------------------------
    def checkpoint(self) -> dict:
        return {"cells": {k: (v.clone() if hasattr(v, "clone") else copy.deepcopy(v)) for k, v in self.session_cells.items()},
                "runs": self.stats["runs"]}

    def restore(self, snapshot: dict) -> None:
        self.session_cells = {k: (v.clone() if hasattr(v, "clone") else copy.deepcopy(v)) for k, v in snapshot["cells"].items()}

    def reset(self) -> None:
        self.session_cells = {}

    # -- one run ----------------------------------------------------------------------------------------
    def run(self, inputs: dict | None = None, on_emit=None, eos_token_ids=()) -> dict:
        """Execute the step tree.  ``on_emit(output, value, mode)`` sees every emit as it happens; returning False stops the
        enclosing loops after the current iteration (a client that went away).  A loop whose termination is
        ``generation_eos`` also ends once the value it last emitted is one of ``eos_token_ids``.  Names the ``serving``
        block hands to the runtime (the ``active`` mask) read as true until then.  Returns ``{output: value | [values]}``."""
        inputs = dict(inputs or {})
        root = _Scope()
        unknown = sorted(set(inputs) - set(self.wf.inputs))
        if unknown:
            raise WorkflowRuntimeError(f"unknown input(s) {', '.join(unknown)}; the workflow declares {', '.join(sorted(self.wf.inputs))}")
        # rows of the request: the extent of the request-aligned axis of the first supplied input that declares one
        # (documents without batch layouts: the leading extent of an input whose contract starts with a symbolic dimension)
        self._batch = 1
        for name, spec in self.wf.inputs.items():
            c = spec["contract"]
            axis = c.batch_axis if c.batch_axis is not None else (0 if c.shape and isinstance(c.shape[0], str) else None)
            if name in inputs and axis is not None and hasattr(inputs[name], "shape") and len(inputs[name].shape) > axis:
                self._batch = int(inputs[name].shape[axis])
                break
        for name, spec in self.wf.inputs.items():
            if name in inputs:
                root.set(name, inputs[name])
            elif spec.get("default") is not None:
                default, c = spec["default"], spec["contract"]
                if np.isscalar(default) or isinstance(default, bool):
                    # a scalar default fills the contract's shape: the request-aligned axis takes one entry per row of the
                    # request, other symbolic extents take one entry
                    axis = c.batch_axis if c.batch_axis is not None else (0 if c.shape and c.shape[0] == "batch" else None)
                    dims = [self._batch if i == axis else (d if isinstance(d, int) else 1) for i, d in enumerate(c.shape)] or [1]
                    default = np.full(tuple(dims), default, dtype=_NP_DTYPE.get(c.dtype))
                root.set(name, default)
            elif spec["required"]:
                raise WorkflowRuntimeError(f"required input '{name}' was not supplied")
        for key, name in self.wf.serving.items():
            if isinstance(name, str) and not root.has(name) and name not in self.wf.state:
                root.set(name, np.asarray([True]))
        for cell, value in self.session_cells.items():
            root.set(cell, value)
        self._eos, self._last_emit = set(int(t) for t in eos_token_ids), None
        self._outputs: dict = {}
        self._on_emit, self._stop = on_emit, False
        self.stats["runs"] += 1
        for s in self.wf.steps:
            self._exec(s, root)
        for cell, spec in self.wf.state.items():
            if spec["scope"] == "session" and root.has(cell):
                self.session_cells[cell] = root.get(cell)
        return self._outputs

    def _read(self, scope: _Scope, name: str, step):
        if scope.has(name):
            return scope.get(name)
        spec = self.wf.state.get(name)
        if spec is not None and spec["initializer"] is not None and scope.has(spec["initializer"]):
            return scope.get(spec["initializer"])           # a cell nobody has written yet reads as its initializer
        raise WorkflowRuntimeError(f"{step.where}: value '{name}' has not been produced (did a component skip an output, or a branch arm not run?)")

    def _exec(self, step, scope: _Scope) -> None:
        kind = step.kind
        if kind == "invoke":
            feed = {port: self._read(scope, val, step) for port, val in step.inputs.items()}
            for port, val in (getattr(self.components[step.component], "extra_inputs", None) or {}).items():
                if val and (scope.has(val) or val in self.wf.state):      # values the runtime hands an adapter next to its ports
                    feed[port] = self._read(scope, val, step)
            result = self.components[step.component](feed)
            if not isinstance(result, dict):
                raise WorkflowRuntimeError(f"{step.where}: component '{step.component}' returned {type(result).__name__}; a dict of output ports is needed")
            for port, val in step.outputs.items():
                if port not in result:
                    raise WorkflowRuntimeError(f"{step.where}: component '{step.component}' did not produce output port '{port}' "
                                               f"(it produced: {', '.join(sorted(result)) or 'nothing'})")
                scope.set(val, result[port])
            self.stats["invocations"][step.component] = self.stats["invocations"].get(step.component, 0) + 1
        elif kind == "sequence":
            for s in step.steps:
                self._exec(s, scope)
        elif kind == "loop":
            for s in step.setup:
                self._exec(s, scope)
            for cell, initial, _next in step.carried:
                if initial is not None:
                    scope.set(cell, self._read(scope, initial, step))
                elif not scope.has(cell):
                    scope.set(cell, self._read(scope, cell, step))
            limit = int(_scalar(self._read(scope, step.max_iterations, step), f"{step.where}: max_iterations"))
            it = 0
            while it < limit and not self._stop and _all_true(self._read(scope, step.continue_when, step)):
                body = _Scope(scope)
                if step.iteration_value:
                    rows = self._batch if any(isinstance(d, str) for d in step.iteration_shape) else 1
                    body.set(step.iteration_value, np.full((rows,), it, dtype=np.int64))
                for s in step.steps:
                    self._exec(s, body)
                nxt = [(cell, self._read(body, n, step)) for cell, _i, n in step.carried]
                for cell, v in nxt:                          # all reads before any write: cells may feed one another
                    scope.set(cell, v)
                it += 1
                self.stats["iterations"] += 1
                if step.termination == "generation_eos" and self._eos and self._last_emit is not None:
                    try:
                        if int(_scalar(self._last_emit, "emitted token")) in self._eos:
                            break
                    except (TypeError, ValueError):
                        pass
        elif kind == "branch":
            pred = _scalar(self._read(scope, step.predicate, step), f"{step.where}: predicate")
            label = ("true" if pred else "false") if isinstance(pred, (bool, np.bool_)) else str(pred)
            arm = step.cases.get(label, step.default)
            took_default = label not in step.cases
            if arm is None:
                raise WorkflowRuntimeError(f"{step.where}: predicate is '{label}' but the branch has cases {', '.join(step.cases)} and no default")
            inner = _Scope(scope)
            self._exec(arm, inner)
            for name, o in step.branch_outputs.items():
                src = o["default"] if took_default else o["cases"].get(label)
                if src is None:
                    raise WorkflowRuntimeError(f"{step.where}: branch output '{name}' has no source for the arm '{'default' if took_default else label}'")
                scope.set(name, self._read(inner, src, step))
        else:  # emit
            if step.when is not None and not _all_true(self._read(scope, step.when, step)):
                return
            value = self._read(scope, step.value, step)
            if step.valid_length is not None:
                value = value[: int(_scalar(self._read(scope, step.valid_length, step), f"{step.where}: valid_length"))]
            if step.mode == "replace":
                self._outputs[step.output] = value
            else:
                self._outputs.setdefault(step.output, []).append(value)
            self._last_emit = value
            if self._on_emit is not None and self._on_emit(step.output, value, step.mode) is False:
                self._stop = True


def run_workflow(document: dict, components: dict, inputs: dict | None = None, on_emit=None) -> dict:
    """One-shot helper: ``document`` is a whole inference-metadata document (with ``pipeline.workflow``)."""
    wf = wfm.load_document(document)
    if wf is None:
        raise WorkflowRuntimeError("the document has no pipeline.workflow")
    return WorkflowSession(wf, components).run(inputs, on_emit)
