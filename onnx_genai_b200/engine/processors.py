"""Host-side logit processors, warpers and samplers (the path taken when a request cannot use the
fused device sampler).

Order and eligibility follow the reference (crates/onnx-genai-engine/src/processors.rs:18-292):

    repetition penalty -> frequency penalty -> presence penalty -> DRY -> stop-sequence guard ->
    constraint -> [only when sampling] temperature -> top-k / top-p -> min-p -> top-a -> typical-p ->
    mirostat -> XTC

Under greedy selection no warper is built.  A request runs on the device when its chain is a
subset of {temperature, top-k, top-p, min-p}, it asks for no logprobs and brings no custom
sampler; otherwise the engine copies the row's logits to the host and runs this chain.
`Sampler` and `LogitProcessor` are the public extension seams (src/sampling.rs:38-42,
src/logits.rs:72-118).
"""
from __future__ import annotations

import math
from dataclasses import dataclass, field

import numpy as np


class LogitProcessor:
    """``process(token_ids, logits) -> logits`` over one fp32 row; ``preserves_argmax`` lets a greedy
    request stay on the device when every processor in its chain keeps the argmax."""

    preserves_argmax = False

    def process(self, token_ids, logits: np.ndarray) -> np.ndarray:
        raise NotImplementedError


class Sampler:
    """``sample(logits, u) -> token id``; ``u`` is the request's uniform draw for this token."""

    name = "sampler"

    def sample(self, logits: np.ndarray, u: float) -> int:
        raise NotImplementedError


class GreedySampler(Sampler):
    name = "greedy"

    def sample(self, logits, u=0.0):
        l = np.where(np.isnan(logits), -np.inf, logits)
        return int(np.flatnonzero(l == l.max())[0])  # lowest id wins ties


class CategoricalSampler(Sampler):
    name = "categorical"

    def sample(self, logits, u):
        l = np.where(np.isnan(logits), -np.inf, logits).astype(np.float64)
        p = np.exp(l - l.max())
        p /= p.sum()
        c = np.cumsum(p)
        return int(min(np.searchsorted(c, u * c[-1], side="right"), len(p) - 1))


class RepetitionPenalty(LogitProcessor):
    def __init__(self, penalty, window=0):
        self.penalty, self.window = float(penalty), int(window)

    def process(self, token_ids, logits):
        ids = token_ids[-self.window:] if self.window > 0 else token_ids
        if len(ids) == 0:
            return logits
        idx = np.unique(np.asarray(ids, dtype=np.int64))
        idx = idx[(idx >= 0) & (idx < logits.shape[0])]
        v = logits[idx]
        logits[idx] = np.where(v > 0, v / self.penalty, v * self.penalty)
        return logits


class FrequencyPresencePenalty(LogitProcessor):
    def __init__(self, frequency=0.0, presence=0.0, prompt_len=0):
        self.frequency, self.presence, self.prompt_len = float(frequency), float(presence), int(prompt_len)

    def process(self, token_ids, logits):
        gen = np.asarray(token_ids[self.prompt_len:], dtype=np.int64)
        if gen.size == 0:
            return logits
        ids, counts = np.unique(gen[(gen >= 0) & (gen < logits.shape[0])], return_counts=True)
        logits[ids] -= self.frequency * counts + self.presence
        return logits


class DryPenalty(LogitProcessor):
    """DRY ("don't repeat yourself"): penalise tokens that would extend a repeated suffix."""

    def __init__(self, multiplier, base=1.75, allowed_length=2, sequence_breakers=()):
        self.multiplier, self.base, self.allowed = float(multiplier), float(base), int(allowed_length)
        self.breakers = set(int(b) for b in sequence_breakers)

    def process(self, token_ids, logits):
        ids = list(token_ids)
        n = len(ids)
        if n < 2 or self.multiplier <= 0:
            return logits
        last = ids[-1]
        best = {}
        for i in range(n - 1):
            if ids[i] != last:
                continue
            ln = 1
            while i - ln >= 0 and ids[i - ln] == ids[n - 1 - ln] and ids[i - ln] not in self.breakers and ln < 64:
                ln += 1
            nxt = ids[i + 1]
            if ln >= self.allowed:
                best[nxt] = max(best.get(nxt, 0), ln)
        for tok, ln in best.items():
            if 0 <= tok < logits.shape[0]:
                logits[tok] -= self.multiplier * self.base ** (ln - self.allowed)
        return logits


class BanTokens(LogitProcessor):
    def __init__(self, banned):
        self.banned = np.asarray(sorted(set(int(b) for b in banned)), dtype=np.int64)

    def process(self, token_ids, logits):
        if self.banned.size:
            logits[self.banned[self.banned < logits.shape[0]]] = -np.inf
        return logits


class Temperature(LogitProcessor):
    preserves_argmax = True

    def __init__(self, t):
        self.t = max(float(t), 1e-6)

    def process(self, token_ids, logits):
        return logits / self.t


class TopKTopP(LogitProcessor):
    preserves_argmax = True

    def __init__(self, top_k=0, top_p=1.0):
        self.k, self.p = int(top_k), float(top_p)

    def process(self, token_ids, logits):
        v = logits.shape[0]
        if 0 < self.k < v:
            kth = np.partition(logits, v - self.k)[v - self.k]
            logits = np.where(logits < kth, -np.inf, logits)
        if 0.0 < self.p < 1.0:
            order = np.argsort(-logits, kind="stable")
            sl = logits[order].astype(np.float64)
            pr = np.exp(sl - sl[0])
            pr /= pr.sum()
            c = np.cumsum(pr)
            cut = int(np.searchsorted(c, self.p, side="left")) + 1
            drop = order[cut:]
            logits[drop] = -np.inf
        return logits


class MinP(LogitProcessor):
    preserves_argmax = True

    def __init__(self, min_p):
        self.min_p = float(min_p)

    def process(self, token_ids, logits):
        thr = logits.max() + math.log(max(self.min_p, 1e-12))
        return np.where(logits < thr, -np.inf, logits)


class TopA(LogitProcessor):
    preserves_argmax = True

    def __init__(self, a):
        self.a = float(a)

    def process(self, token_ids, logits):
        l = logits.astype(np.float64)
        p = np.exp(l - l.max())
        p /= p.sum()
        return np.where(p < self.a * p.max() ** 2, -np.inf, logits)


class TypicalP(LogitProcessor):
    def __init__(self, p):
        self.p = float(p)

    def process(self, token_ids, logits):
        l = logits.astype(np.float64)
        lp = l - (l.max() + math.log(np.exp(l - l.max()).sum()))
        p = np.exp(lp)
        ent = -(p * np.where(np.isfinite(lp), lp, 0.0)).sum()
        dev = np.abs(-lp - ent)
        order = np.argsort(dev, kind="stable")
        c = np.cumsum(p[order])
        cut = int(np.searchsorted(c, self.p, side="left")) + 1
        logits[order[cut:]] = -np.inf
        return logits


class Mirostat(LogitProcessor):
    """Mirostat v2: truncate to tokens whose surprise is below mu; mu follows the observed surprise."""

    def __init__(self, tau=5.0, eta=0.1):
        self.tau, self.eta, self.mu = float(tau), float(eta), 2.0 * float(tau)
        self._last_probs = None

    def process(self, token_ids, logits):
        l = logits.astype(np.float64)
        p = np.exp(l - l.max())
        p /= p.sum()
        surprise = -np.log2(np.maximum(p, 1e-300))
        keep = surprise <= self.mu
        if not keep.any():
            keep[np.argmax(p)] = True
        self._last_probs = p
        return np.where(keep, logits, -np.inf)

    def observe(self, token):
        if self._last_probs is not None:
            s = -math.log2(max(self._last_probs[token], 1e-300))
            self.mu -= self.eta * (s - self.tau)


class Xtc(LogitProcessor):
    """XTC: with probability `probability`, drop every token above `threshold` except the least likely of them."""

    def __init__(self, probability, threshold, rng):
        self.probability, self.threshold, self.rng = float(probability), float(threshold), rng

    def process(self, token_ids, logits):
        if self.rng.random() >= self.probability:
            return logits
        l = logits.astype(np.float64)
        p = np.exp(l - l.max())
        p /= p.sum()
        above = np.flatnonzero(p >= self.threshold)
        if above.size > 1:
            keep = above[np.argmin(p[above])]
            logits[above[above != keep]] = -np.inf
        return logits


@dataclass
class ProcessorChain:
    processors: list = field(default_factory=list)

    def process(self, token_ids, logits):
        for p in self.processors:
            logits = p.process(token_ids, logits)
        return logits

    @property
    def preserves_argmax(self):
        return all(p.preserves_argmax for p in self.processors)


DEVICE_OK = (Temperature, TopKTopP, MinP)


def build_processor_chain(opt, prompt_len: int, rng=None, extra=(), constraint=None) -> ProcessorChain:
    """Build the chain for ``opt`` (a GenerateOptions) in the fixed order documented above."""
    chain = []
    if opt.repetition_penalty and opt.repetition_penalty != 1.0:
        chain.append(RepetitionPenalty(opt.repetition_penalty, opt.repetition_window))
    if opt.frequency_penalty or opt.presence_penalty:
        chain.append(FrequencyPresencePenalty(opt.frequency_penalty, opt.presence_penalty, prompt_len))
    if opt.dry_multiplier:
        chain.append(DryPenalty(opt.dry_multiplier, opt.dry_base, opt.dry_allowed_length, opt.dry_sequence_breakers))
    if opt.banned_tokens:
        chain.append(BanTokens(opt.banned_tokens))
    chain.extend(extra)
    if constraint is not None:
        chain.append(constraint)
    if not opt.greedy:
        if opt.temperature and opt.temperature != 1.0:
            chain.append(Temperature(opt.temperature))
        if (opt.top_k and opt.top_k > 0) or (opt.top_p is not None and opt.top_p < 1.0):
            chain.append(TopKTopP(opt.top_k or 0, opt.top_p if opt.top_p is not None else 1.0))
        if opt.min_p:
            chain.append(MinP(opt.min_p))
        if opt.top_a:
            chain.append(TopA(opt.top_a))
        if opt.typical_p and opt.typical_p < 1.0:
            chain.append(TypicalP(opt.typical_p))
        if opt.mirostat:
            chain.append(Mirostat(opt.mirostat_tau, opt.mirostat_eta))
        if opt.xtc_probability:
            chain.append(Xtc(opt.xtc_probability, opt.xtc_threshold, rng or np.random.default_rng(opt.seed or None)))
    return ProcessorChain(chain)


def device_sampling_plan(chain: ProcessorChain, opt, has_custom_sampler: bool) -> str:
    """'greedy' | 'sampled' | 'host' -- the single eligibility predicate (processors.rs:229-292)."""
    if has_custom_sampler or opt.logprobs:
        return "host"
    if opt.greedy:
        return "greedy" if chain.preserves_argmax else "host"
    if all(isinstance(p, DEVICE_OK) for p in chain.processors):
        return "sampled"
    return "host"


def log_softmax(logits: np.ndarray) -> np.ndarray:
    l = logits.astype(np.float64)
    m = l.max()
    return l - (m + math.log(np.exp(l - m).sum()))
