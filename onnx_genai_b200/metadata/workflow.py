"""The workflow form of the inference-metadata standard (``pipeline.workflow``): parse, validate, lower.

A workflow describes a package as components (ONNX artifacts with typed ports and port roles), named values in
static single assignment form, state cells carried around loops, a serving block that says which port pairs hold
model state, and a tree of steps -- ``invoke``, ``sequence``, ``loop``, ``branch``, ``emit``
(crates/onnx-genai-metadata/src/schema/ir.rs:801-845).  This module

* parses that document into plain dataclasses, rejecting unknown step kinds and malformed steps;
* validates it: every component an ``invoke`` names exists and its bound ports are declared, every value a step
  reads has been defined by then (a request / literal input, a state cell, a loop iteration value, or the output
  of an earlier step), no value is defined twice in one scope, ``emit`` targets are declared outputs, loop
  ``carried`` entries name state cells and defined values;
* lowers a single-decoder workflow to the resolved decoder ABI the executor consumes -- which component is the
  decoder, its token / mask / position inputs and logits output (from the port roles), its per-layer KV input /
  output pairs, layout and aliasing (from the self-attention ``state_service`` group), whether the cache is
  updated by indexed scatter -- the same derivation the reference performs in
  crates/onnx-genai-metadata/src/decoder_abi.rs:1-30, so a package that carries a workflow needs no ``model.io`` block.

Errors say where in the document the problem is and what would fix it.
"""
from __future__ import annotations

from dataclasses import dataclass, field


class WorkflowError(ValueError):
    pass


STEP_KINDS = ("invoke", "sequence", "loop", "branch", "emit")
EMIT_MODES = ("replace", "append", "event")
TOKEN_ROLES = ("token_ids", "input_ids")


@dataclass
class Contract:
    dtype: str = ""
    rank: int | None = None
    shape: list = field(default_factory=list)
    optional: bool = False
    batch_axis: int | None = None     # axis aligned with the rows of the request (batch_layout: request_aligned), if any


@dataclass
class Component:
    name: str
    kind: str
    artifact: str | None
    inputs: dict            # port -> Contract
    outputs: dict
    roles: dict             # port -> role name
    declares_ports: bool = True   # False: the ports are those of the ONNX artifact itself and are not checked here
    abi: str | None = None        # adapter components: the named ABI they implement
    params: dict = field(default_factory=dict)   # adapter components: the contract's parameters (e.g. action)


@dataclass
class Step:
    kind: str
    where: str
    component: str | None = None
    inputs: dict = field(default_factory=dict)       # port -> value
    outputs: dict = field(default_factory=dict)      # port -> value
    steps: list = field(default_factory=list)        # sequence / loop body
    setup: list = field(default_factory=list)        # loop
    continue_when: str | None = None
    max_iterations: str | None = None
    termination: str = "predicate"
    iteration_value: str | None = None
    iteration_shape: list = field(default_factory=lambda: [1])   # [1], or ["batch"] for one counter per request row
    carried: list = field(default_factory=list)      # [(cell, initial | None, next)]
    predicate: str | None = None                     # branch
    cases: dict = field(default_factory=dict)        # label -> Step
    default: "Step | None" = None
    branch_outputs: dict = field(default_factory=dict)   # value -> {"cases": {label: value}, "default": value | None}
    value: str | None = None                         # emit
    output: str | None = None
    mode: str = "replace"
    when: str | None = None
    valid_length: str | None = None


@dataclass
class StateGroup:
    name: str
    kind: str
    layout: str | None
    sequence_axis: int | None
    aliasing: str | None
    update: str | None
    logical_lengths: str | None
    ports: dict            # component -> {alias: {"input", "output", "role", "layer", "access"}}
    capabilities: dict


@dataclass
class Workflow:
    capabilities: list
    inputs: dict           # value name -> {"contract": Contract, "source": str, "role": str | None, "required": bool, "default"}
    outputs: dict          # output name -> Contract
    components: dict       # name -> Component
    state: dict            # cell -> {"contract": Contract, "initializer": str | None, "scope": str, "recurrence": str}
    serving: dict
    groups: dict           # name -> StateGroup
    steps: list            # [Step]


@dataclass
class DecoderAbi:
    component: str
    artifact: str | None
    token_input: str
    attention_mask_input: str | None
    position_ids_input: str | None
    logits_output: str
    kv_pairs: list         # [(input port, output port)] in layer order (key before value within a layer)
    kv_layout: str | None
    kv_sequence_axis: int | None
    kv_aliasing: str | None
    kv_update: str         # "append" | "indexed_scatter"
    num_layers: int
    rollback_positions: int
    prefix_reusable: bool


# ---------------------------------------------------------------------------------------------
# parsing
# ---------------------------------------------------------------------------------------------
def _contract(d, where) -> Contract:
    if d is None:
        return Contract()
    if not isinstance(d, dict):
        raise WorkflowError(f"{where}: a tensor contract must be a mapping with dtype / rank / shape")
    layout = d.get("batch_layout")
    axis = int(layout.get("axis", 0)) if isinstance(layout, dict) and layout.get("kind") == "request_aligned" else None
    return Contract(dtype=str(d.get("dtype", "")), rank=d.get("rank"), shape=list(d.get("shape") or []), optional=bool(d.get("optional", False)),
                    batch_axis=axis)


def _step(d, where) -> Step:
    if not isinstance(d, dict) or "kind" not in d:
        raise WorkflowError(f"{where}: a step is a mapping with a 'kind' ({', '.join(STEP_KINDS)})")
    kind = d["kind"]
    if kind not in STEP_KINDS:
        raise WorkflowError(f"{where}: unknown step kind {kind!r}; use one of {', '.join(STEP_KINDS)}")
    s = Step(kind=kind, where=where)
    if kind == "invoke":
        if not d.get("component"):
            raise WorkflowError(f"{where}: invoke needs a 'component'")
        s.component = str(d["component"])
        s.inputs = {str(k): str(v) for k, v in (d.get("inputs") or {}).items()}
        s.outputs = {str(k): str(v) for k, v in (d.get("outputs") or {}).items()}
    elif kind == "sequence":
        s.steps = [_step(x, f"{where}.steps[{i}]") for i, x in enumerate(d.get("steps") or [])]
    elif kind == "loop":
        for req in ("steps", "continue_when", "max_iterations"):
            if req not in d:
                raise WorkflowError(f"{where}: loop needs '{req}'")
        s.setup = [_step(x, f"{where}.setup[{i}]") for i, x in enumerate(d.get("setup") or [])]
        s.steps = [_step(x, f"{where}.steps[{i}]") for i, x in enumerate(d["steps"])]
        s.continue_when, s.max_iterations = str(d["continue_when"]), str(d["max_iterations"])
        s.termination = str(d.get("termination", "predicate"))
        if s.termination not in ("predicate", "generation_eos"):
            raise WorkflowError(f"{where}: loop termination {s.termination!r} is not predicate or generation_eos")
        it = d.get("iteration")
        s.iteration_value = str(it["value"]) if isinstance(it, dict) and "value" in it else None
        if isinstance(it, dict) and isinstance(it.get("contract"), dict) and it["contract"].get("shape"):
            s.iteration_shape = list(it["contract"]["shape"])
        for i, c in enumerate(d.get("carried") or []):
            if not isinstance(c, dict) or "cell" not in c or "next" not in c:
                raise WorkflowError(f"{where}.carried[{i}]: a carried entry needs 'cell' and 'next'")
            s.carried.append((str(c["cell"]), str(c["initial"]) if c.get("initial") is not None else None, str(c["next"])))
    elif kind == "branch":
        if "predicate" not in d or not d.get("cases"):
            raise WorkflowError(f"{where}: branch needs a 'predicate' and at least one case")
        s.predicate = str(d["predicate"])
        s.cases = {str(k): _step(v, f"{where}.cases[{k}]") for k, v in d["cases"].items()}
        s.default = _step(d["default"], f"{where}.default") if d.get("default") is not None else None
        for name, o in (d.get("outputs") or {}).items():
            s.branch_outputs[str(name)] = {"cases": {str(k): str(v) for k, v in (o.get("cases") or {}).items()},
                                           "default": str(o["default"]) if o.get("default") is not None else None}
    else:  # emit
        for req in ("value", "output", "mode"):
            if req not in d:
                raise WorkflowError(f"{where}: emit needs '{req}'")
        s.value, s.output, s.mode = str(d["value"]), str(d["output"]), str(d["mode"])
        if s.mode not in EMIT_MODES:
            raise WorkflowError(f"{where}: emit mode {s.mode!r} is not one of {', '.join(EMIT_MODES)}")
        s.when = str(d["when"]) if d.get("when") is not None else None
        s.valid_length = str(d["valid_length"]) if d.get("valid_length") is not None else None
    return s


def parse(doc: dict) -> Workflow:
    """``doc`` is the mapping under ``pipeline.workflow``."""
    if not isinstance(doc, dict):
        raise WorkflowError("pipeline.workflow must be a mapping")
    inputs = {}
    for name, d in (doc.get("inputs") or {}).items():
        src = (d.get("source") or {}).get("kind", "request") if isinstance(d, dict) else "request"
        role = d.get("role") if isinstance(d, dict) else None
        role_name = role.get("role") if isinstance(role, dict) else (role if isinstance(role, str) else None)
        inputs[str(name)] = {"contract": _contract(d.get("contract"), f"inputs.{name}"), "source": src, "role": role_name,
                             "required": bool(d.get("required", False)), "default": d.get("default") if isinstance(d, dict) else None}
    outputs = {str(n): _contract((d or {}).get("contract"), f"outputs.{n}") for n, d in (doc.get("outputs") or {}).items()}
    components = {}
    for name, d in (doc.get("components") or {}).items():
        impl = d.get("implementation") or {}
        ports = d.get("ports") or {}
        components[str(name)] = Component(
            name=str(name), kind=str(impl.get("kind", "onnx")), artifact=impl.get("artifact"),
            inputs={str(p): _contract(c, f"components.{name}.ports.inputs.{p}") for p, c in (ports.get("inputs") or {}).items()},
            outputs={str(p): _contract(c, f"components.{name}.ports.outputs.{p}") for p, c in (ports.get("outputs") or {}).items()},
            roles={str(p): str(r) for p, r in (ports.get("roles") or {}).items()},
            declares_ports=bool(ports.get("inputs") or ports.get("outputs")), abi=impl.get("abi"),
            params=dict(((d.get("contract") or {}).get("parameters")) or {}))
    state = {}
    for name, d in (doc.get("state") or {}).items():
        rec = d.get("recurrence") or {}
        state[str(name)] = {"contract": _contract(d.get("contract"), f"state.{name}"), "initializer": d.get("initializer"),
                            "scope": d.get("scope", "invocation"), "recurrence": rec.get("kind", "invariant") if isinstance(rec, dict) else str(rec)}
    serving = doc.get("serving") or {}
    groups = {}
    for name, g in ((serving.get("state_service") or {}).get("groups") or {}).items():
        upd = g.get("update")
        groups[str(name)] = StateGroup(
            name=str(name), kind=str(g.get("kind", "")), layout=g.get("layout"), sequence_axis=g.get("sequence_axis"),
            aliasing=g.get("aliasing"), update=(upd.get("kind") if isinstance(upd, dict) else upd), logical_lengths=g.get("logical_lengths"),
            ports={str(c): {str(a): dict(v) for a, v in (aliases or {}).items()} for c, aliases in (g.get("ports") or {}).items()},
            capabilities=dict(g.get("capabilities") or {}) | {"reuse": dict(g.get("reuse") or {})})
    steps = [_step(x, f"steps[{i}]") for i, x in enumerate(doc.get("steps") or [])]
    if not steps:
        raise WorkflowError("pipeline.workflow.steps is empty: a workflow needs at least one step")
    return Workflow(capabilities=list((doc.get("manifest") or {}).get("capabilities") or []), inputs=inputs, outputs=outputs,
                    components=components, state=state, serving=serving, groups=groups, steps=steps)


# ---------------------------------------------------------------------------------------------
# validation
# ---------------------------------------------------------------------------------------------
def validate(wf: Workflow) -> list:
    """All problems found (empty list = valid).  Checks components, ports, single assignment and definedness."""
    problems: list = []
    state_aliases = {a for g in wf.groups.values() for aliases in g.ports.values() for a in aliases}
    serving_names = {v for k, v in wf.serving.items() if isinstance(v, str)}

    def defined_base():
        return set(wf.inputs) | set(wf.state) | state_aliases | serving_names

    def check(step: Step, scope: set, assigned: set):
        """``scope`` = values readable here; ``assigned`` = values assigned in the enclosing region (for SSA)."""
        def read(val, what):
            if val is not None and val not in scope:
                problems.append(f"{step.where}: {what} reads '{val}', which is not defined at this point (not an input, a state "
                                "cell, or the output of an earlier step)")

        def write(val, what):
            if val in assigned:
                problems.append(f"{step.where}: {what} assigns '{val}' a second time; workflow values are single-assignment")
            assigned.add(val)
            scope.add(val)

        if step.kind == "invoke":
            comp = wf.components.get(step.component)
            if comp is None:
                problems.append(f"{step.where}: invoke names component '{step.component}', which is not declared "
                                f"(declared: {', '.join(sorted(wf.components)) or 'none'})")
            checked = comp is not None and comp.declares_ports
            for port, val in step.inputs.items():
                if checked and port not in comp.inputs:
                    problems.append(f"{step.where}: '{port}' is not an input port of component '{step.component}'")
                read(val, f"input port '{port}'")
            for port, val in step.outputs.items():
                if checked and port not in comp.outputs:
                    problems.append(f"{step.where}: '{port}' is not an output port of component '{step.component}'")
                write(val, f"output port '{port}'")
            if checked:
                for port, c in comp.inputs.items():
                    if port not in step.inputs and not c.optional and port not in _state_bound_ports(wf, comp.name, "input"):
                        problems.append(f"{step.where}: required input port '{port}' of component '{step.component}' is not bound")
        elif step.kind == "sequence":
            for s in step.steps:
                check(s, scope, assigned)
        elif step.kind == "loop":
            for s in step.setup:
                check(s, scope, assigned)
            body_scope, body_assigned = set(scope), set()
            for cell, _initial, _next in step.carried:
                body_scope.add(cell)
            if step.iteration_value:
                body_scope.add(step.iteration_value)
            read_scope = scope
            if step.max_iterations not in read_scope:
                problems.append(f"{step.where}: max_iterations reads '{step.max_iterations}', which is not defined before the loop")
            for s in step.steps:
                check(s, body_scope, body_assigned)
            if step.continue_when not in body_scope:
                problems.append(f"{step.where}: continue_when reads '{step.continue_when}', which the loop body does not define")
            for cell, initial, nxt in step.carried:
                if cell not in wf.state and cell not in state_aliases:
                    problems.append(f"{step.where}: carried cell '{cell}' is not declared under state (or as a state-service alias)")
                if initial is not None and initial not in scope:
                    problems.append(f"{step.where}: carried cell '{cell}' starts from '{initial}', which is not defined before the loop")
                if nxt not in body_scope:
                    problems.append(f"{step.where}: carried cell '{cell}' continues with '{nxt}', which the loop body does not define")
        elif step.kind == "branch":
            if step.predicate not in scope:
                problems.append(f"{step.where}: predicate reads '{step.predicate}', which is not defined at this point")
            arms = list(step.cases.items()) + ([("default", step.default)] if step.default is not None else [])
            arm_scopes = {}
            for label, arm in arms:
                arm_scope, arm_assigned = set(scope), set()
                check(arm, arm_scope, arm_assigned)
                arm_scopes[label] = arm_scope
            for name, o in step.branch_outputs.items():
                for label, val in o["cases"].items():
                    if label not in step.cases:
                        problems.append(f"{step.where}: branch output '{name}' names case '{label}', which the branch does not have")
                    elif val not in arm_scopes[label]:
                        problems.append(f"{step.where}: branch output '{name}' takes '{val}' from case '{label}', which does not define it")
                if o["default"] is not None and step.default is not None and o["default"] not in arm_scopes["default"]:
                    problems.append(f"{step.where}: branch output '{name}' takes '{o['default']}' from the default arm, which does not define it")
                write(name, f"branch output '{name}'")
        else:  # emit
            read(step.value, "emit")
            if step.when is not None:
                read(step.when, "emit 'when'")
            if step.valid_length is not None:
                read(step.valid_length, "emit 'valid_length'")
            if step.output not in wf.outputs:
                problems.append(f"{step.where}: emit targets '{step.output}', which is not a declared output "
                                f"(declared: {', '.join(sorted(wf.outputs)) or 'none'})")

    scope, assigned = defined_base(), set()
    for s in wf.steps:
        check(s, scope, assigned)
    for gname, g in wf.groups.items():
        for comp, aliases in g.ports.items():
            c = wf.components.get(comp)
            if c is None:
                problems.append(f"serving.state_service.groups.{gname}: ports name component '{comp}', which is not declared")
                continue
            for alias, v in aliases.items():
                if not c.declares_ports:
                    continue
                if v.get("input") is not None and v["input"] not in c.inputs:
                    problems.append(f"serving.state_service.groups.{gname}.ports.{comp}.{alias}: '{v['input']}' is not an input port of '{comp}'")
                if v.get("output") is not None and v["output"] not in c.outputs:
                    problems.append(f"serving.state_service.groups.{gname}.ports.{comp}.{alias}: '{v['output']}' is not an output port of '{comp}'")
    return problems


def _state_bound_ports(wf: Workflow, component: str, side: str) -> set:
    out = set()
    for g in wf.groups.values():
        for v in (g.ports.get(component) or {}).values():
            if v.get(side) is not None:
                out.add(v[side])
    return out


# ---------------------------------------------------------------------------------------------
# lowering: the decoder ABI
# ---------------------------------------------------------------------------------------------
def decoder_abi(wf: Workflow) -> DecoderAbi:
    """The decode-step ABI of a single-decoder workflow.  Raises ``WorkflowError`` when the workflow is not one."""
    candidates = [c for c in wf.components.values() if "logits" in c.roles.values() and any(r in TOKEN_ROLES for r in c.roles.values())]
    if not candidates:
        raise WorkflowError("no component declares both a token-id input role and a logits output role, so this workflow has no "
                            "decoder to lower (roles found: " + ", ".join(sorted({r for c in wf.components.values() for r in c.roles.values()}) or ["none"]) + ")")
    with_state = [c for c in candidates if any(c.name in g.ports for g in wf.groups.values() if g.kind in ("full_attention", "self_attention", "sliding_window"))]
    if len(with_state) > 1:
        raise WorkflowError("several components look like decoders with attention state (" + ", ".join(c.name for c in with_state) +
                            "); the single-decoder lowering does not apply (a speculative workflow names a target and a draft)")
    comp = (with_state or candidates)[0]
    by_role = {}
    for port, role in comp.roles.items():
        by_role.setdefault(role, port)
    token = next((by_role[r] for r in TOKEN_ROLES if r in by_role), None)
    group = next((g for g in wf.groups.values() if comp.name in g.ports and g.kind in ("full_attention", "self_attention", "sliding_window")), None)
    pairs, layers = [], 0
    if group is not None:
        role_order = {"key": 0, "combined": 0, "value": 1}
        aliases = []
        for pos, (alias, v) in enumerate(group.ports[comp.name].items()):
            aliases.append((int(v.get("layer", pos)), role_order.get(v.get("role"), 2), alias, v))
        aliases.sort(key=lambda t: (t[0], t[1], t[2]))
        for layer, _r, alias, v in aliases:
            if v.get("access", "read_write") != "read_write":
                continue
            if v.get("input") is None or v.get("output") is None:
                raise WorkflowError(f"serving.state_service.groups.{group.name}.ports.{comp.name}.{alias}: a read-write state port "
                                    "names both an input and an output")
            pairs.append((v["input"], v["output"]))
        layers = len({t[0] for t in aliases})
    caps = group.capabilities if group is not None else {}
    return DecoderAbi(component=comp.name, artifact=comp.artifact, token_input=token, attention_mask_input=by_role.get("attention_mask"),
                      position_ids_input=by_role.get("position_ids"), logits_output=by_role["logits"], kv_pairs=pairs,
                      kv_layout=group.layout if group else None, kv_sequence_axis=group.sequence_axis if group else None,
                      kv_aliasing=group.aliasing if group else None,
                      kv_update="indexed_scatter" if group is not None and group.update == "indexed_scatter" else "append",
                      num_layers=layers, rollback_positions=int(caps.get("rollback_positions", 0) or 0),
                      prefix_reusable=bool((caps.get("reuse") or {}).get("prefix_reusable", False)))


def load_document(doc: dict) -> Workflow | None:
    """The workflow of a whole inference-metadata document, or None when it has none."""
    wf = ((doc or {}).get("pipeline") or {}).get("workflow")
    return parse(wf) if wf is not None else None
