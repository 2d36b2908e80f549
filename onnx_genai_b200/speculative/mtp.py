"""Multi-token-prediction proposer: a small head drafts from the target's own hidden state.

The target's last hidden state already encodes most of what the next few tokens will be.  An MTP head takes that state
and the embedding of the token the target just chose, produces the state one position ahead, and reads a draft token
from it through the target's *shared* output projection; feeding its own output back gives the following draft
tokens ("hidden-threaded": the recurrent state is the hidden vector, no KV cache of its own, nothing to rewind when
drafts are rejected).  Same seam as the reference's ``MtpProposer`` -- last hidden state + greedy next token in, a chain
of draft tokens out, the target's embedding table and LM head shared rather than duplicated
(crates/onnx-genai-engine/src/speculative/mod.rs:48-63, 999-1170).

One head step, for hidden ``h`` and token embedding ``e`` (all RMS-normalised with learned gains)::

    z = W_fuse [norm(h) ; norm(e)]
    z = z + W_down ( silu(W_gate norm(z)) * (W_up norm(z)) )
    draft = argmax( LM_head norm_out(z) )          h <- z, e <- embed(draft)

The engine hands every proposer that sets ``wants_hidden`` the final hidden state of the row that produced the last
committed token (after verification: the row of the last accepted draft), so the head always continues from the
verified prefix.  Sequences that share a head are drafted together: one [B, H] pass per draft position.
"""
from __future__ import annotations

import numpy as np
import torch

from . import SpeculativeProposer


def _rms(x, g, eps=1e-6):
    xf = x.float()
    return (xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + eps)).to(x.dtype) * g


class MtpHead:
    """Weights of one hidden-threaded MTP block.  ``embed`` [V, H] and ``lm_head`` [V, H] belong to the target."""

    NAMES = ("fuse", "gate", "up", "down", "norm_h", "norm_e", "norm_m", "norm_out")

    def __init__(self, weights: dict, embed: torch.Tensor, lm_head: torch.Tensor, eps: float = 1e-6):
        missing = [n for n in self.NAMES if n not in weights]
        if missing:
            raise ValueError(f"MTP head is missing tensors {missing}; it needs {list(self.NAMES)}")
        hid = embed.shape[1]
        if tuple(weights["fuse"].shape) != (hid, 2 * hid):
            raise ValueError(f"MTP head hidden size {weights['fuse'].shape[0]} (fuse {tuple(weights['fuse'].shape)}) does not match the "
                             f"target's embedding width {hid}")
        self.w = {n: weights[n].to(device=embed.device, dtype=embed.dtype) for n in self.NAMES}
        self.embed, self.lm_head, self.eps = embed, lm_head, eps
        self.hidden, self.inter = hid, int(weights["gate"].shape[0])

    @classmethod
    def random(cls, embed, lm_head, inter: int | None = None, seed: int = 0, std: float = 0.02) -> "MtpHead":
        hid = embed.shape[1]
        inter = inter or 2 * hid
        g = torch.Generator().manual_seed(seed)
        w = {"fuse": torch.randn(hid, 2 * hid, generator=g) * std, "gate": torch.randn(inter, hid, generator=g) * std,
             "up": torch.randn(inter, hid, generator=g) * std, "down": torch.randn(hid, inter, generator=g) * std,
             "norm_h": torch.ones(hid), "norm_e": torch.ones(hid), "norm_m": torch.ones(hid), "norm_out": torch.ones(hid)}
        return cls(w, embed, lm_head)

    def save(self, path: str) -> None:
        from safetensors.torch import save_file

        save_file({n: t.detach().float().cpu().contiguous() for n, t in self.w.items()}, path)

    @classmethod
    def load(cls, path: str, embed, lm_head) -> "MtpHead":
        from safetensors.torch import load_file

        return cls(load_file(path), embed, lm_head)

    @torch.no_grad()
    def draft(self, hidden: torch.Tensor, tokens: torch.Tensor, k: int) -> torch.Tensor:
        """``hidden`` [B, H] (the target's final-normed states), ``tokens`` [B] (the tokens chosen from them) -> [B, k] drafts."""
        w, out = self.w, []
        h, tok = hidden.to(self.embed.dtype), tokens.long()
        for _ in range(k):
            e = self.embed.index_select(0, tok)
            z = torch.cat([_rms(h, w["norm_h"], self.eps), _rms(e, w["norm_e"], self.eps)], dim=-1) @ w["fuse"].T
            m = _rms(z, w["norm_m"], self.eps)
            z = z + (torch.nn.functional.silu(m @ w["gate"].T) * (m @ w["up"].T)) @ w["down"].T
            tok = (_rms(z, w["norm_out"], self.eps) @ self.lm_head.T).float().argmax(-1)
            out.append(tok)
            h = z
        return torch.stack(out, dim=1)


class MtpProposer(SpeculativeProposer):
    name = "mtp"
    wants_hidden = True

    def __init__(self, head: MtpHead):
        self.head = head
        self.hidden = None           # [H] on the head's device, set by the engine after every committed step

    @property
    def batch_key(self):
        return ("mtp", id(self.head))

    def observe(self, hidden: torch.Tensor) -> None:
        self.hidden = hidden

    def propose(self, token_ids, k):
        return self.propose_many([self], [token_ids], k)[0]

    @staticmethod
    def propose_many(proposers, token_lists, k):
        empty = np.zeros(0, dtype=np.int32)
        live = [i for i, p in enumerate(proposers) if p.hidden is not None and len(token_lists[i])]
        out = [empty] * len(proposers)
        if not live or k <= 0:
            return out
        head = proposers[live[0]].head
        hidden = torch.stack([proposers[i].hidden for i in live])
        last = torch.tensor([int(token_lists[i][-1]) for i in live], device=hidden.device)
        drafts = head.draft(hidden, last, k).to("cpu", torch.int32).numpy()
        for row, i in enumerate(live):
            out[i] = drafts[row]
        return out


class Eagle3Head(MtpHead):
    """EAGLE-3 style head: the draft state starts from a fusion of the target's low-, mid- and high-level features (the
    residual stream entering three chosen layers) instead of the final hidden state alone, then threads through the
    same recurrent block as :class:`MtpHead`.  The reference's ``Eagle3Proposer`` concatenates the three taps into its
    ``fused_hidden`` input in the same order (crates/onnx-genai-engine/src/speculative/mod.rs:886, 1174-1200)."""

    NAMES = MtpHead.NAMES + ("fuse3", "norm_low", "norm_mid", "norm_high")

    def __init__(self, weights: dict, embed, lm_head, tap_layers, eps: float = 1e-6):
        super().__init__(weights, embed, lm_head, eps)
        if len(tap_layers) != 3:
            raise ValueError(f"an EAGLE-3 head reads three layers (low, mid, high), got {list(tap_layers)}")
        if tuple(weights["fuse3"].shape) != (self.hidden, 3 * self.hidden):
            raise ValueError(f"fuse3 is {tuple(weights['fuse3'].shape)}; a head for hidden size {self.hidden} needs ({self.hidden}, {3 * self.hidden})")
        self.tap_layers = [int(l) for l in tap_layers]

    @classmethod
    def random(cls, embed, lm_head, tap_layers, inter: int | None = None, seed: int = 0, std: float = 0.02) -> "Eagle3Head":
        hid = embed.shape[1]
        base = MtpHead.random(embed, lm_head, inter, seed, std)
        g = torch.Generator().manual_seed(seed + 1)
        w = {n: t.float().cpu() for n, t in base.w.items()}
        w.update({"fuse3": torch.randn(hid, 3 * hid, generator=g) * std, "norm_low": torch.ones(hid), "norm_mid": torch.ones(hid),
                  "norm_high": torch.ones(hid)})
        return cls(w, embed, lm_head, tap_layers)

    @staticmethod
    def default_tap_layers(num_layers: int) -> list:
        """Low, middle and high: after roughly 1/8, 1/2 and 7/8 of the stack."""
        return sorted({max(1, num_layers // 8), max(1, num_layers // 2), max(1, num_layers - max(1, num_layers // 8))})[:3] \
            if num_layers >= 4 else [0, max(0, num_layers // 2), num_layers - 1][:3]

    def fuse(self, taps: dict) -> torch.Tensor:
        """``taps``: layer -> [B, H] residual states; returns the fused draft state [B, H]."""
        w = self.w
        lo, mid, hi = (taps[l].to(self.embed.dtype) for l in self.tap_layers)
        cat = torch.cat([_rms(lo, w["norm_low"], self.eps), _rms(mid, w["norm_mid"], self.eps), _rms(hi, w["norm_high"], self.eps)], dim=-1)
        return cat @ w["fuse3"].T


class Eagle3Proposer(MtpProposer):
    name = "eagle3"

    def __init__(self, head: Eagle3Head):
        super().__init__(head)
        self.tap_layers = head.tap_layers
        self.taps = None

    @property
    def batch_key(self):
        return ("eagle3", id(self.head))

    def observe(self, hidden, taps=None) -> None:
        if taps is None:
            raise RuntimeError("the EAGLE-3 proposer needs the target's intermediate states; call model.set_hidden_taps(head.tap_layers)")
        self.taps = taps
        self.hidden = self.head.fuse({l: t[None] for l, t in taps.items()})[0]


def attach_eagle3(engine, head: Eagle3Head | None = None, tap_layers=None, seed: int = 0) -> Eagle3Head:
    """Make ``engine`` draft with an EAGLE-3 style head on speculative requests; switches the target's layer taps on."""
    model = engine.llm.model
    if head is None:
        head = Eagle3Head.random(model.w.embed, model.w.lm_head, tap_layers or Eagle3Head.default_tap_layers(model.cfg.num_layers), seed=seed)
    model.set_hidden_taps(head.tap_layers)
    engine.proposer_factory = lambda: Eagle3Proposer(head)
    return head


class SharedKvHead(MtpHead):
    """A draft block that attends over the *target's* KV cache instead of keeping one of its own: its query is projected
    from the draft state, rotated to the draft position, and run through the same paged-attention kernels against the
    pages of one target layer (by default the last).  No extra cache memory, nothing to rewind.  The reference's
    shared-KV proposer binds target KV slices to its ``shared_kv.*`` inputs for the same purpose
    (crates/onnx-genai-engine/src/speculative/mod.rs:890-891)."""

    NAMES = MtpHead.NAMES + ("q_proj", "o_proj", "norm_q")

    def __init__(self, weights: dict, embed, lm_head, num_heads: int, head_dim: int, layer: int = -1, eps: float = 1e-6):
        super().__init__(weights, embed, lm_head, eps)
        if tuple(weights["q_proj"].shape) != (num_heads * head_dim, self.hidden):
            raise ValueError(f"q_proj is {tuple(weights['q_proj'].shape)}; the target's attention needs ({num_heads * head_dim}, {self.hidden})")
        self.num_heads, self.head_dim, self.layer = num_heads, head_dim, layer

    @classmethod
    def random(cls, embed, lm_head, num_heads: int, head_dim: int, layer: int = -1, inter: int | None = None, seed: int = 0,
               std: float = 0.02) -> "SharedKvHead":
        hid = embed.shape[1]
        base = MtpHead.random(embed, lm_head, inter, seed, std)
        g = torch.Generator().manual_seed(seed + 2)
        w = {n: t.float().cpu() for n, t in base.w.items()}
        w.update({"q_proj": torch.randn(num_heads * head_dim, hid, generator=g) * std,
                  "o_proj": torch.randn(hid, num_heads * head_dim, generator=g) * std, "norm_q": torch.ones(hid)})
        return cls(w, embed, lm_head, num_heads, head_dim, layer)

    @torch.no_grad()
    def draft_shared(self, hidden, tokens, k: int, llm, page_table, ctx_len) -> torch.Tensor:
        """As :meth:`MtpHead.draft`, with one attention read of the target's pages per draft position.
        ``page_table`` [B, P] int32 and ``ctx_len`` [B] int32 describe the computed context of each sequence."""
        from .. import ops
        from ..ops import reference

        w, model, kv = self.w, llm.model, llm.kv
        layer = self.layer % len(kv.pools)
        pool = kv.pools[layer]
        scales = kv.scales[layer] if kv.scales is not None else None
        b, hq, d = hidden.shape[0], self.num_heads, self.head_dim
        stride = (hq + 2 * model.hkv) * d                          # the attention entry points read q from packed qkv rows
        qkv = torch.zeros(b, stride, dtype=self.embed.dtype, device=hidden.device)
        attn = torch.zeros(b, hq * d, dtype=self.embed.dtype, device=hidden.device)
        h, tok, out = hidden.to(self.embed.dtype), tokens.long(), []
        for j in range(k):
            e = self.embed.index_select(0, tok)
            z = torch.cat([_rms(h, w["norm_h"], self.eps), _rms(e, w["norm_e"], self.eps)], dim=-1) @ w["fuse"].T
            q = (_rms(z, w["norm_q"], self.eps) @ w["q_proj"].T).view(b, hq, d)
            pos = (ctx_len.long() + j).clamp(max=model.cos_sin.shape[0] - 1)
            qkv[:, : hq * d] = reference.apply_rope(q, pos, model.cos_sin, model.rotary_dim, model.cfg.rotary_interleaved).reshape(b, hq * d)
            ops.paged_decode(qkv, attn, pool, page_table, ctx_len, hq, model.hkv, d, model.scale, kv_scales=scales)
            z = z + attn[:b] @ w["o_proj"].T
            m = _rms(z, w["norm_m"], self.eps)
            z = z + (torch.nn.functional.silu(m @ w["gate"].T) * (m @ w["up"].T)) @ w["down"].T
            tok = (_rms(z, w["norm_out"], self.eps) @ self.lm_head.T).float().argmax(-1)
            out.append(tok)
            h = z
        return torch.stack(out, dim=1)


class SharedKvProposer(MtpProposer):
    name = "shared_kv"
    wants_sequence = True

    def __init__(self, head: SharedKvHead):
        super().__init__(head)
        self.llm, self.sid = None, None

    @property
    def batch_key(self):
        return ("shared_kv", id(self.head))

    def bind(self, llm, sid: int) -> None:
        self.llm, self.sid = llm, sid

    @staticmethod
    def propose_many(proposers, token_lists, k):
        empty = np.zeros(0, dtype=np.int32)
        live = [i for i, p in enumerate(proposers) if p.hidden is not None and p.llm is not None and len(token_lists[i]) > 1]
        out = [empty] * len(proposers)
        if not live or k <= 0:
            return out
        llm, head = proposers[live[0]].llm, proposers[live[0]].head
        # the last token was sampled but not fed yet: the cache holds every token before it
        ctx = [len(token_lists[i]) - 1 for i in live]
        pages = [llm.core.seq_pages(proposers[i].sid) for i in live]
        need = [-(-c // 16) for c in ctx]
        keep = [j for j in range(len(live)) if len(pages[j]) >= need[j] > 0]
        if not keep:
            return out
        table = np.zeros((len(keep), max(need[j] for j in keep)), dtype=np.int32)
        for row, j in enumerate(keep):
            table[row, : need[j]] = pages[j][: need[j]]
        dev = llm.device
        hidden = torch.stack([proposers[live[j]].hidden for j in keep])
        last = torch.tensor([int(token_lists[live[j]][-1]) for j in keep], device=dev)
        drafts = head.draft_shared(hidden, last, k, llm, torch.from_numpy(table).to(dev),
                                   torch.tensor([ctx[j] for j in keep], dtype=torch.int32, device=dev)).to("cpu", torch.int32).numpy()
        for row, j in enumerate(keep):
            out[live[j]] = drafts[row]
        return out


def attach_shared_kv(engine, head: SharedKvHead | None = None, layer: int = -1, seed: int = 0) -> SharedKvHead:
    """Make ``engine`` draft with a head that reads the target's own KV pages (one GPU or CPU; not tensor parallel)."""
    llm = engine.llm
    if llm.tp != 1:
        raise ValueError("the shared-KV proposer reads whole KV heads; with tensor parallelism each rank holds a slice")
    model = llm.model
    head = head or SharedKvHead.random(model.w.embed, model.w.lm_head, model.hq, model.d, layer, seed=seed)
    engine.proposer_factory = lambda: SharedKvProposer(head)
    return head


def attach_mtp(engine, head: MtpHead | None = None, seed: int = 0) -> MtpHead:
    """Make ``engine`` (an :class:`onnx_genai_b200.engine.api.Engine`) draft with an MTP head on speculative requests.
    With no head given, a randomly initialised one is made (useful for measuring the mechanism, not acceptance)."""
    w = engine.llm.model.w
    head = head or MtpHead.random(w.embed, w.lm_head, seed=seed)
    engine.proposer_factory = lambda: MtpProposer(head)
    return head
