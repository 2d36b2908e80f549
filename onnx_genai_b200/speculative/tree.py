"""Tree-structured speculation: one verification pass scores a branching set of candidate continuations.

A linear draft is a chain; a tree draft lets the proposer hedge (two candidates for the next token, each with its own
continuation) and the verifier keeps the single root-to-leaf path the target agrees with.  This module holds the
parts that do not depend on how the target is run, as the reference's tree core does
(crates/onnx-genai-engine/src/speculative/tree.rs:1-31):

* :class:`SpecTree` -- parent-pointer tree of draft tokens in breadth-compatible order (a parent always precedes its
  children), built from explicit nodes, from several linear drafts that share prefixes, or from per-depth top-k lists;
* :func:`ancestor_attention_mask` -- node i attends node j iff j is i or an ancestor of i (every node also sees the
  whole committed context);
* :func:`relative_position_ids` -- position = depth, so rotary embeddings see path length and not the flattened index;
* :meth:`SpecTree.accept` -- the greedy acceptance walk: from the root, follow the child whose token equals the
  target's choice at the current node, stop when none does, then append the target's choice there (correction or bonus);
* :func:`kv_retention_plan` -- which flattened KV slots survive (the accepted path, in depth order) and where they
  move, so the cache is compacted to a plain prefix after verification;
* :func:`verify_tree` -- scorer + accept + plan in one call.  A scorer is anything that returns one row of logits per
  node given the committed context and the tree.  :class:`PathScorer` builds one from a plain ``context -> next-token
  logits`` function by scoring each node with its own path (what a masked batched forward computes in one pass).

The engine's own verification path feeds linear drafts; this core is the seam for a tree-masked attention pass and is
exercised here against plain next-token functions.

Under greedy acceptance the tokens produced are exactly those of plain greedy decoding, whatever the tree holds.
"""
from __future__ import annotations

from dataclasses import dataclass, field

import numpy as np


@dataclass
class TreeNode:
    token: int
    parent: int            # index of the parent node, -1 for children of the committed context
    depth: int = 0         # 0 for children of the context


@dataclass
class SpecTree:
    nodes: list = field(default_factory=list)

    # -- construction ---------------------------------------------------------------------------------
    def add(self, token: int, parent: int = -1) -> int:
        if parent >= len(self.nodes) or parent < -1:
            raise ValueError(f"parent {parent} does not exist yet; a node is added after its parent (have {len(self.nodes)} nodes)")
        depth = 0 if parent < 0 else self.nodes[parent].depth + 1
        self.nodes.append(TreeNode(int(token), parent, depth))
        return len(self.nodes) - 1

    @classmethod
    def from_paths(cls, paths) -> "SpecTree":
        """Merge linear drafts; common prefixes become shared nodes."""
        tree, index = cls(), {}
        for path in paths:
            parent = -1
            for tok in path:
                key = (parent, int(tok))
                if key not in index:
                    index[key] = tree.add(tok, parent)
                parent = index[key]
        return tree

    @classmethod
    def from_topk(cls, per_depth_candidates, max_nodes: int = 64) -> "SpecTree":
        """``per_depth_candidates[d]`` lists candidate tokens at depth d, best first.  The first candidate of each depth
        continues every branch; the others are leaves hanging off the best path (a "caterpillar": cheap and usually
        where the hedging pays)."""
        tree, spine = cls(), -1
        for cands in per_depth_candidates:
            if not len(cands) or len(tree.nodes) >= max_nodes:
                break
            first = tree.add(cands[0], spine)
            for tok in list(cands[1:]):
                if len(tree.nodes) >= max_nodes:
                    break
                tree.add(tok, spine)
            spine = first
        return tree

    # -- queries ----------------------------------------------------------------------------------------
    def __len__(self):
        return len(self.nodes)

    def children(self, parent: int) -> list:
        return [i for i, n in enumerate(self.nodes) if n.parent == parent]

    def path_to(self, node: int) -> list:
        """Node indices from depth 0 down to ``node``."""
        out = []
        while node >= 0:
            out.append(node)
            node = self.nodes[node].parent
        return out[::-1]

    def leaves(self) -> list:
        parents = {n.parent for n in self.nodes}
        return [i for i in range(len(self.nodes)) if i not in parents]

    def tokens(self) -> np.ndarray:
        return np.asarray([n.token for n in self.nodes], dtype=np.int32)

    # -- acceptance -----------------------------------------------------------------------------------
    def accept(self, root_choice: int, node_choices) -> "TreeAcceptance":
        """``root_choice``: the target's token after the committed context.  ``node_choices[i]``: the target's token after
        the context followed by the path to node i.  Returns the accepted node path and the tokens to commit."""
        path, choice, parent = [], int(root_choice), -1
        while True:
            nxt = next((c for c in self.children(parent) if self.nodes[c].token == choice), None)
            if nxt is None:
                break
            path.append(nxt)
            parent, choice = nxt, int(node_choices[nxt])
        tokens = [self.nodes[i].token for i in path] + [choice]
        return TreeAcceptance(path=path, tokens=np.asarray(tokens, dtype=np.int32), bonus=choice)


@dataclass
class TreeAcceptance:
    path: list             # accepted node indices, depth order
    tokens: np.ndarray     # accepted draft tokens followed by the target's own next token
    bonus: int

    @property
    def accepted(self) -> int:
        return len(self.path)


def ancestor_attention_mask(tree: SpecTree) -> np.ndarray:
    """[n, n] bool: row i may attend column j.  Lower-triangular by construction (parents come first)."""
    n = len(tree)
    mask = np.zeros((n, n), dtype=bool)
    for i, node in enumerate(tree.nodes):
        if node.parent >= 0:
            mask[i] = mask[node.parent]
        mask[i, i] = True
    return mask


def relative_position_ids(tree: SpecTree, context_len: int = 0) -> np.ndarray:
    return np.asarray([context_len + n.depth for n in tree.nodes], dtype=np.int64)


@dataclass
class KvRetentionPlan:
    keep: list             # flattened tree slots (node indices) to keep, in depth order
    moves: list            # (from_slot, to_slot) relative to the first tree slot; only entries that actually move
    new_length: int        # context_len + accepted nodes


def kv_retention_plan(tree: SpecTree, acceptance: TreeAcceptance, context_len: int) -> KvRetentionPlan:
    """After a flattened tree pass the cache holds one slot per node at ``context_len + node index``.  Keep the accepted
    path and slide it down so the cache is a plain prefix again; everything else is dropped."""
    moves = [(src, dst) for dst, src in enumerate(acceptance.path) if src != dst]
    return KvRetentionPlan(keep=list(acceptance.path), moves=moves, new_length=context_len + len(acceptance.path))


class PathScorer:
    """Scores a tree with a plain next-token function: ``logits_fn(token ids) -> logits of the next token``."""

    def __init__(self, logits_fn):
        self.fn = logits_fn
        self.calls = 0

    def score(self, context, tree: SpecTree):
        ctx = [int(t) for t in context]
        self.calls += 1 + len(tree)
        root = np.asarray(self.fn(ctx))
        rows = [np.asarray(self.fn(ctx + [tree.nodes[j].token for j in tree.path_to(i)])) for i in range(len(tree))]
        return root, rows


def verify_tree(context, tree: SpecTree, scorer) -> tuple:
    """Greedy verification: (acceptance, retention plan).  ``scorer.score(context, tree)`` returns the logits after the
    context and one logits row per node."""
    root, rows = scorer.score(context, tree)
    acc = tree.accept(int(np.argmax(root)), [int(np.argmax(r)) for r in rows])
    return acc, kv_retention_plan(tree, acc, len(context))


def greedy_decode_with_trees(logits_fn, prompt, max_new_tokens: int, propose_tree) -> tuple:
    """Reference loop used by the tests and by callers without an engine: repeatedly ``propose_tree(tokens) -> SpecTree``,
    verify, commit.  Returns (tokens generated, verification passes)."""
    scorer = PathScorer(logits_fn)
    toks, out, passes = [int(t) for t in prompt], [], 0
    while len(out) < max_new_tokens:
        tree = propose_tree(toks)
        acc, _plan = verify_tree(toks, tree, scorer)
        passes += 1
        new = [int(t) for t in acc.tokens][: max_new_tokens - len(out)]
        out += new
        toks += new
    return out, passes
