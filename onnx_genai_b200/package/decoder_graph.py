"""Decoder ONNX graph <-> fused executor plan.

``export_decoder`` writes a decoder as the operator set the reference's packages contain
(docs/execution/NATIVE_CUDA_DECODE.md:133-150): Gather, (Skip)SimplifiedLayerNormalization,
MatMul or com.microsoft::MatMulNBits (+Add bias), com.microsoft::GroupQueryAttention with in-op
rotary (cos/sin caches), Sigmoid/Mul SwiGLU glue, with onnxruntime-genai style past/present I/O
names.  ``lower_decoder`` is the inverse and the counterpart of the reference's graph-level
fusion passes (crates/onnx-runtime-ep-cuda/src/optimizer.rs:27-158): it walks the nodes in
topological order and recognises the layer pattern *structurally* (operator types and data
flow, never tensor or model names), producing the ``DecoderConfig`` + ``DecoderWeights`` the fused
executor runs.  A graph that does not match the pattern is rejected with the node that broke it.
"""
from __future__ import annotations

import math

import numpy as np
import torch

from ..models.config import DecoderConfig
from ..models.decoder import DecoderWeights, LayerWeights, pad_mlp, pick_swiglu_half
from ..ops import reference as ref
from . import onnx_pb as pb

MS = "com.microsoft"


def _np_of(t: torch.Tensor, dtype: str):
    if dtype == "bf16":
        return t.detach().to(torch.bfloat16).cpu().contiguous().view(torch.uint16).numpy(), pb.BFLOAT16
    if dtype == "fp16":
        return t.detach().to(torch.float16).cpu().contiguous().numpy(), pb.FLOAT16
    return t.detach().float().cpu().contiguous().numpy(), pb.FLOAT


def _torch_of(t: pb.Tensor) -> torch.Tensor:
    arr = np.ascontiguousarray(t.array)
    if t.data_type == pb.BFLOAT16:
        return torch.from_numpy(arr.view(np.uint16).copy()).view(torch.bfloat16)
    return torch.from_numpy(arr.copy())


class GraphPatternError(ValueError):
    pass


# ---------------------------------------------------------------------------------------------
# export
# ---------------------------------------------------------------------------------------------
def export_decoder(cfg: DecoderConfig, gate_up_unpacked, weights: DecoderWeights, path: str, dtype: str = "fp32",
                   int4: bool = False, int4_symmetric: bool = True, scale_dtype: str = "fp32") -> pb.Model:
    """Write ``path`` (+ ``.data``).  ``gate_up_unpacked(layer) -> (gate_w, up_w)`` returns the MLP
    projections in natural [intermediate, hidden] layout (the executor keeps them tile-interleaved)."""
    g = pb.Graph(name="decoder")
    elem = {"fp32": pb.FLOAT, "bf16": pb.BFLOAT16, "fp16": pb.FLOAT16}[dtype]

    def init(name, t, as_dtype=None):
        arr, dt = _np_of(t, as_dtype or dtype)
        g.initializers[name] = pb.Tensor(name=name, dims=tuple(arr.shape), data_type=dt, array=arr)
        return name

    def raw_init(name, arr, dt):
        g.initializers[name] = pb.Tensor(name=name, dims=tuple(arr.shape), data_type=dt, array=arr)
        return name

    def linear(prefix, x, w, bias=None):
        """y = x @ w^T (+ bias); w is [N, K]."""
        n, k = w.shape
        out = prefix + "/out"
        if int4:
            q, s, zp = ref.quantize_w4(w.float().cpu(), cfg.int4_block, symmetric=int4_symmetric)
            ins = [x, raw_init(prefix + ".qweight", q.numpy(), pb.UINT8), init(prefix + ".scales", s, scale_dtype),
                   raw_init(prefix + ".zp", zp.numpy(), pb.UINT8) if zp is not None else "", "",
                   init(prefix + ".bias", bias) if bias is not None else ""]
            while ins and ins[-1] == "":
                ins.pop()
            g.nodes.append(pb.Node("MatMulNBits", ins, [out], name=prefix, domain=MS,
                                   attrs={"K": k, "N": n, "bits": 4, "block_size": cfg.int4_block, "accuracy_level": 0}))
            return out
        g.nodes.append(pb.Node("MatMul", [x, init(prefix + ".weight", w.t().contiguous())], [out], name=prefix))
        if bias is not None:
            g.nodes.append(pb.Node("Add", [out, init(prefix + ".bias", bias)], [prefix + "/biased"], name=prefix + "/add"))
            return prefix + "/biased"
        return out

    hq, hkv, d, hid = cfg.num_heads, cfg.num_kv_heads, cfg.head_dim, cfg.hidden
    rd = cfg.rotary_dim or d
    cs = ref.rope_table(cfg.max_position, rd, cfg.rope_theta)
    init("cos_cache", cs[..., 0].contiguous(), "fp32")
    init("sin_cache", cs[..., 1].contiguous(), "fp32")
    g.inputs += [pb.ValueInfo("input_ids", pb.INT64, ("batch", "seq")), pb.ValueInfo("attention_mask", pb.INT64, ("batch", "total"))]
    g.nodes.append(pb.Node("Gather", [init("embed.weight", weights.embed), "input_ids"], ["hidden/0"], name="embed"))
    # attention-mask glue -> seqlens_k, total_sequence_length (same shape the reference's graphs carry)
    g.nodes.append(pb.Node("ReduceSum", ["attention_mask", raw_init("axes1", np.array([1], np.int64), pb.INT64)], ["mask_sum"], attrs={"keepdims": 0}))
    g.nodes.append(pb.Node("Sub", ["mask_sum", raw_init("one", np.array(1, np.int64), pb.INT64)], ["seqlens_k64"]))
    g.nodes.append(pb.Node("Cast", ["seqlens_k64"], ["seqlens_k"], attrs={"to": pb.INT32}))
    g.nodes.append(pb.Node("Shape", ["attention_mask"], ["mask_shape"]))
    g.nodes.append(pb.Node("Gather", ["mask_shape", raw_init("idx1", np.array(1, np.int64), pb.INT64)], ["total64"], attrs={"axis": 0}))
    g.nodes.append(pb.Node("Cast", ["total64"], ["total_seq"], attrs={"to": pb.INT32}))
    x, skip = "hidden/0", None
    for li, lw in enumerate(weights.layers):
        p = f"layers.{li}"
        qkv_w = lw.qkv_w.float().cpu()
        qw, kw, vw = qkv_w[: hq * d], qkv_w[hq * d:(hq + hkv) * d], qkv_w[(hq + hkv) * d:]
        qb = kb = vb = None
        if lw.qkv_b is not None:
            b = lw.qkv_b.float().cpu()
            qb, kb, vb = b[: hq * d], b[hq * d:(hq + hkv) * d], b[(hq + hkv) * d:]
        if skip is None:
            g.nodes.append(pb.Node("SimplifiedLayerNormalization", [x, init(p + ".ln1.weight", lw.ln1)], [p + "/ln1"],
                                   attrs={"epsilon": float(cfg.rms_eps), "axis": -1}))
            resid = x
        else:
            g.nodes.append(pb.Node("SkipSimplifiedLayerNormalization", [x, skip, init(p + ".ln1.weight", lw.ln1)],
                                   [p + "/ln1", "", "", p + "/resid1"], domain=MS, attrs={"epsilon": float(cfg.rms_eps)}))
            resid = p + "/resid1"
        q = linear(p + ".attn.q_proj", p + "/ln1", qw, qb)
        k = linear(p + ".attn.k_proj", p + "/ln1", kw, kb)
        v = linear(p + ".attn.v_proj", p + "/ln1", vw, vb)
        pk, pv = f"past_key_values.{li}.key", f"past_key_values.{li}.value"
        g.inputs += [pb.ValueInfo(pk, elem, ("batch", hkv, "past", d)), pb.ValueInfo(pv, elem, ("batch", hkv, "past", d))]
        g.nodes.append(pb.Node("GroupQueryAttention", [q, k, v, pk, pv, "seqlens_k", "total_seq", "cos_cache", "sin_cache"],
                               [p + "/attn", f"present.{li}.key", f"present.{li}.value"], name=p + ".attn", domain=MS,
                               attrs={"num_heads": hq, "kv_num_heads": hkv, "do_rotary": 1,
                                      "rotary_interleaved": int(cfg.rotary_interleaved),
                                      "local_window_size": cfg.sliding_window if cfg.sliding_window > 0 else -1,
                                      "scale": float(1.0 / np.sqrt(d))}))
        o = linear(p + ".attn.o_proj", p + "/attn", lw.o_w.float().cpu())
        g.nodes.append(pb.Node("SkipSimplifiedLayerNormalization", [resid, o, init(p + ".ln2.weight", lw.ln2)],
                               [p + "/ln2", "", "", p + "/resid2"], domain=MS, attrs={"epsilon": float(cfg.rms_eps)}))
        gate_w, up_w = gate_up_unpacked(li)
        gt = linear(p + ".mlp.gate_proj", p + "/ln2", gate_w.float().cpu())
        up = linear(p + ".mlp.up_proj", p + "/ln2", up_w.float().cpu())
        g.nodes.append(pb.Node("Sigmoid", [gt], [p + "/sig"]))
        g.nodes.append(pb.Node("Mul", [gt, p + "/sig"], [p + "/silu"]))
        g.nodes.append(pb.Node("Mul", [p + "/silu", up], [p + "/act"]))
        x = linear(p + ".mlp.down_proj", p + "/act", lw.down_w.float().cpu())
        skip = p + "/resid2"
    g.nodes.append(pb.Node("SkipSimplifiedLayerNormalization", [skip, x, init("final_norm.weight", weights.final_norm)],
                           ["final/normed", "", "", "final/resid"], domain=MS, attrs={"epsilon": float(cfg.rms_eps)}))
    if cfg.tie_embeddings and not int4:
        g.nodes.append(pb.Node("Transpose", ["embed.weight"], ["lm_head_t"], attrs={"perm": [1, 0]}))
        g.nodes.append(pb.Node("MatMul", ["final/normed", "lm_head_t"], ["logits"], name="lm_head"))
    else:
        out = linear("lm_head", "final/normed", weights.lm_head.float().cpu())
        g.nodes.append(pb.Node("Identity", [out], ["logits"]))
    g.outputs.append(pb.ValueInfo("logits", pb.FLOAT if dtype == "fp32" else elem, ("batch", "seq", cfg.vocab)))
    for li in range(cfg.num_layers):
        g.outputs += [pb.ValueInfo(f"present.{li}.key", elem, ("batch", hkv, "total", d)),
                      pb.ValueInfo(f"present.{li}.value", elem, ("batch", hkv, "total", d))]
    model = pb.Model(graph=g)
    pb.save_model(model, path)
    return model


# ---------------------------------------------------------------------------------------------
# lowering (pattern recognition)
# ---------------------------------------------------------------------------------------------
class _Lin:
    """One recognised projection: dense [N, K] weight or MatMulNBits tensors (+ optional bias)."""

    def __init__(self):
        self.w = None
        self.q = self.scales = self.zp = None
        self.bias = None
        self.block = 32
        self.k = None

    def dense(self, dtype) -> torch.Tensor:
        if self.w is not None:
            return self.w.to(dtype)
        return ref.dequant_w4(self.q, self.scales.float(), self.zp, self.block, self.k).to(dtype)


def lower_decoder(model: pb.Model, dtype=torch.float32, device="cpu", keep_int4: bool = False, tp: int = 1, rank: int = 0):
    """Returns (DecoderConfig, DecoderWeights, gate_up_unpacked) recognised from the graph."""
    g = model.graph
    inits = g.initializers
    producer = {}
    for n in g.nodes:
        for o in n.outputs:
            if o:
                producer[o] = n

    def const(name):
        return inits.get(name)

    def as_linear(node) -> _Lin:
        lin = _Lin()
        if node.op_type == "MatMulNBits":
            if int(node.attrs.get("bits", 4)) != 4:
                raise GraphPatternError(f"node {node.name!r}: MatMulNBits with bits={node.attrs.get('bits')} is not supported (int4 only)")
            lin.block = int(node.attrs.get("block_size", 32))
            lin.k = int(node.attrs["K"]) if "K" in node.attrs else None
            lin.q = _torch_of(const(node.inputs[1]))
            lin.scales = _torch_of(const(node.inputs[2]))
            if len(node.inputs) > 3 and node.inputs[3]:
                lin.zp = _torch_of(const(node.inputs[3]))
            if len(node.inputs) > 5 and node.inputs[5]:
                lin.bias = _torch_of(const(node.inputs[5])).float()
        else:
            w = const(node.inputs[1])
            if w is None:
                src = producer.get(node.inputs[1])
                if src is not None and src.op_type == "Transpose" and const(src.inputs[0]) is not None:
                    lin.w = _torch_of(const(src.inputs[0])).float()            # tied lm_head: Transpose(embed)
                    return lin
                raise GraphPatternError(f"node {node.name!r}: MatMul weight {node.inputs[1]!r} is not a constant")
            lin.w = _torch_of(w).float().t().contiguous()
        return lin

    embed = None
    norms, eps = [], 1e-6
    layers_raw = []
    cur = None
    pending_bias_for = {}
    gqa_attrs = None
    cos = sin = None
    lm_head = None
    stage = "pre"
    for n in g.nodes:
        op = n.op_type
        if op == "Gather" and embed is None and const(n.inputs[0]) is not None and const(n.inputs[0]).array.ndim == 2:
            embed = _torch_of(const(n.inputs[0])).float()
        elif op in ("SimplifiedLayerNormalization", "SkipSimplifiedLayerNormalization", "RMSNormalization"):
            w = const(n.inputs[-1])
            if w is None:
                raise GraphPatternError(f"node {n.name!r}: normalisation weight is not a constant")
            eps = float(n.attrs.get("epsilon", eps))
            norms.append(_torch_of(w).float())
            if cur is not None and cur.get("down") is not None:
                layers_raw.append(cur)
                cur = None
            if cur is None:
                cur = {"ln1": norms[-1], "proj": [], "stage": "attn_in"}
            elif cur["stage"] == "attn_out":
                cur["ln2"] = norms[-1]
                cur["stage"] = "mlp_in"
        elif op in ("MatMul", "MatMulNBits"):
            lin = as_linear(n)
            pending_bias_for[n.outputs[0]] = lin
            if cur is None:
                raise GraphPatternError(f"node {n.name!r}: projection before any normalisation")
            if cur["stage"] == "attn_in" and "gqa" not in cur:
                cur["proj"].append(lin)
            elif cur["stage"] == "attn_in":
                cur["o"] = lin
                cur["stage"] = "attn_out"
            elif cur["stage"] == "mlp_in":
                cur.setdefault("mlp", []).append(lin)
                if len(cur["mlp"]) == 3:
                    cur["down"] = lin
            elif cur["stage"] == "attn_out":
                raise GraphPatternError(f"node {n.name!r}: unexpected projection between o_proj and the post-attention norm")
        elif op == "Add":
            for a, b in ((n.inputs[0], n.inputs[1]), (n.inputs[1], n.inputs[0])):
                if a in pending_bias_for and const(b) is not None:
                    pending_bias_for[a].bias = _torch_of(const(b)).float()
                    pending_bias_for[n.outputs[0]] = pending_bias_for[a]
        elif op == "GroupQueryAttention":
            if cur is None or cur["stage"] != "attn_in":
                raise GraphPatternError(f"node {n.name!r}: GroupQueryAttention outside an attention block")
            cur["gqa"] = n
            gqa_attrs = n.attrs
            if len(n.inputs) > 8 and const(n.inputs[7]) is not None:
                cos, sin = _torch_of(const(n.inputs[7])).float(), _torch_of(const(n.inputs[8])).float()
    # the projections after the last norm: the final layer's collected state holds the lm_head
    if cur is not None:
        if cur.get("down") is not None:
            layers_raw.append(cur)
        else:
            # "cur" was opened by the final norm: its single projection is the lm_head
            if cur["proj"]:
                lm_head = cur["proj"][0]
    if embed is None or not layers_raw or gqa_attrs is None:
        raise GraphPatternError("graph is not a recognised decoder: need Gather(embedding), GroupQueryAttention layers and norms")
    if lm_head is None:
        raise GraphPatternError("no lm_head projection found after the final normalisation")
    final_norm = norms[-1]
    hq, hkv = int(gqa_attrs["num_heads"]), int(gqa_attrs["kv_num_heads"])
    hidden = embed.shape[1]
    first = layers_raw[0]
    if len(first["proj"]) == 3:
        q_out = first["proj"][0].dense(torch.float32).shape[0]
    elif len(first["proj"]) == 1:
        q_out = first["proj"][0].dense(torch.float32).shape[0] * hq // (hq + 2 * hkv)
    else:
        raise GraphPatternError(f"attention block has {len(first['proj'])} input projections; expected 3 (q,k,v) or 1 (packed qkv)")
    d = q_out // hq
    inter = first["mlp"][0].dense(torch.float32).shape[0]
    lm_w = lm_head.dense(torch.float32)
    tied = lm_w.shape == embed.shape and torch.equal(lm_w, embed)
    int4 = first["o"].q is not None
    cfg = DecoderConfig(name=g.name or "decoder", num_layers=len(layers_raw), hidden=hidden, num_heads=hq, num_kv_heads=hkv,
                        head_dim=d, intermediate=inter, vocab=embed.shape[0], rms_eps=eps, tie_embeddings=tied,
                        qkv_bias=first["proj"][0].bias is not None,
                        max_position=int(cos.shape[0]) if cos is not None else 8192,
                        rotary_interleaved=bool(int(gqa_attrs.get("rotary_interleaved", 0))),
                        rotary_dim=int(cos.shape[1] * 2) if cos is not None else 0,
                        sliding_window=max(0, int(gqa_attrs.get("local_window_size", -1))),
                        weight_format="int4" if int4 else "bf16", int4_block=first["o"].block if int4 else 32)
    # Tensor parallelism: this rank keeps its query / KV heads (rows of q, k, v; columns of o) and its slice of the MLP's
    # intermediate width (rows of gate / up, columns of down), cut exactly as the seeded weights of the benchmarks are
    # (models/decoder.py random_weights); embeddings, norms and the LM head stay whole.
    q_rows = kv_rows = None
    i0, i1 = 0, inter
    if tp > 1:
        if keep_int4 and int4:
            raise GraphPatternError("tensor parallelism over packed int4 weights is not built: load with keep_int4=False (bf16 shards)")
        from ..parallel.sharding import shard_heads, shard_range

        hs = shard_heads(hq, hkv, tp, rank)
        q_rows = torch.tensor([h * d + i for h in hs.q_heads for i in range(d)])
        kv_rows = torch.tensor([h * d + i for h in hs.kv_heads for i in range(d)])
        i0, i1 = shard_range(inter, tp, rank, math.gcd(inter, 32))        # 32 where the width allows (int4 blocks, MMA tiles)
    inter_local = i1 - i0
    half = pick_swiglu_half(inter_local + (-inter_local) % 64 if inter_local % 32 else inter_local)
    dev = torch.device(device)
    layers, unpacked = [], []
    for lr in layers_raw:
        if "ln2" not in lr or "o" not in lr or len(lr.get("mlp", [])) != 3:
            raise GraphPatternError("layer does not match norm -> qkv -> GroupQueryAttention -> o_proj -> norm -> gate/up/down")
        projs = lr["proj"]
        qkv_w = torch.cat([p.dense(torch.float32) for p in projs], 0)
        qkv_b = None
        if projs[0].bias is not None:
            qkv_b = torch.cat([p.bias if p.bias is not None else torch.zeros(p.dense(torch.float32).shape[0]) for p in projs], 0)
        gate, up, down = (lr["mlp"][i].dense(torch.float32) for i in range(3))
        o_w = lr["o"].dense(dtype)
        if tp > 1:
            q_size, kv_size = hq * d, hkv * d
            rows = torch.cat([q_rows, q_size + kv_rows, q_size + kv_size + kv_rows])
            qkv_w = qkv_w[rows]
            qkv_b = qkv_b[rows] if qkv_b is not None else None
            o_w = o_w[:, q_rows].contiguous()
            gate, up, down = gate[i0:i1], up[i0:i1], down[:, i0:i1]
        unpacked.append((gate, up))
        if inter_local % 32:
            gate, up, down = pad_mlp(gate, up, down)
        lw = LayerWeights(ln1=lr["ln1"].to(dtype).to(dev), qkv_w=qkv_w.to(dtype).to(dev),
                          qkv_b=qkv_b.to(dtype).to(dev) if qkv_b is not None else None,
                          o_w=o_w.to(dev), ln2=lr["ln2"].to(dtype).to(dev),
                          gate_up_w=ref.pack_gate_up(gate, up, half).to(dtype).to(dev), down_w=down.to(dtype).to(dev))
        if keep_int4 and int4:
            lw.quant = {"o": lr["o"], "down": lr["mlp"][2], "gate": lr["mlp"][0], "up": lr["mlp"][1], "qkv": projs}
        layers.append(lw)
    emb = embed.to(dtype).to(dev)
    weights = DecoderWeights(embed=emb, layers=layers, final_norm=final_norm.to(dtype).to(dev),
                             lm_head=emb if tied else lm_w.to(dtype).to(dev), swiglu_half=half)
    if cos is not None:
        weights.cos_sin = torch.stack([cos, sin], dim=-1).contiguous()
    return cfg, weights, (lambda li: unpacked[li])
