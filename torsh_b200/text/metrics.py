"""Text evaluation metrics: BLEU (corpus and sentence, with smoothing), ROUGE-N / ROUGE-L, edit distance and word error
rate, perplexity, token-overlap F1, and an embedding-based greedy-matching score (the BERTScore recipe over any token
embedding function). Reference: crates/torsh-text/src/metrics/{bleu,rouge,edit_distance,perplexity,overlap,bert_score}.rs.
"""
from __future__ import annotations

import math
from collections import Counter

import torch


def _ngrams(tokens, n):
    return Counter(tuple(tokens[i:i + n]) for i in range(len(tokens) - n + 1))


def bleu(candidates, references, max_n: int = 4, smooth: bool = False) -> float:
    """Corpus BLEU. ``candidates``: list of token lists; ``references``: list of lists of reference token lists."""
    match, total = [0] * max_n, [0] * max_n
    c_len = r_len = 0
    for cand, refs in zip(candidates, references):
        c_len += len(cand)
        r_len += min((len(r) for r in refs), key=lambda L: (abs(L - len(cand)), L))
        for n in range(1, max_n + 1):
            cg = _ngrams(cand, n)
            best: Counter = Counter()
            for r in refs:
                for g, k in _ngrams(r, n).items():
                    best[g] = max(best[g], k)
            match[n - 1] += sum(min(k, best[g]) for g, k in cg.items())
            total[n - 1] += max(len(cand) - n + 1, 0)
    prec = []
    for m, t in zip(match, total):
        if smooth:
            m, t = m + 1, t + 1
        if t == 0 or m == 0:
            return 0.0
        prec.append(m / t)
    bp = 1.0 if c_len > r_len else math.exp(1 - r_len / max(c_len, 1))
    return bp * math.exp(sum(math.log(p) for p in prec) / max_n)


def sentence_bleu(candidate, refs, max_n: int = 4, smooth: bool = True) -> float:
    return bleu([candidate], [refs], max_n, smooth)


def _prf(match, c_total, r_total):
    p = match / c_total if c_total else 0.0
    r = match / r_total if r_total else 0.0
    return {"precision": p, "recall": r, "f1": 2 * p * r / (p + r) if p + r else 0.0}


def rouge_n(candidate, reference, n: int = 1) -> dict:
    c, r = _ngrams(candidate, n), _ngrams(reference, n)
    return _prf(sum((c & r).values()), sum(c.values()), sum(r.values()))


def _lcs(a, b) -> int:
    prev = [0] * (len(b) + 1)
    for x in a:
        cur = [0]
        for j, y in enumerate(b):
            cur.append(prev[j] + 1 if x == y else max(prev[j + 1], cur[j]))
        prev = cur
    return prev[-1]


def rouge_l(candidate, reference) -> dict:
    return _prf(_lcs(candidate, reference), len(candidate), len(reference))


def edit_distance(a, b, substitution_cost: int = 1) -> int:
    """Levenshtein distance between two sequences (strings or token lists)."""
    prev = list(range(len(b) + 1))
    for i, x in enumerate(a, 1):
        cur = [i]
        for j, y in enumerate(b, 1):
            cur.append(min(prev[j] + 1, cur[j - 1] + 1, prev[j - 1] + (0 if x == y else substitution_cost)))
        prev = cur
    return prev[-1]


def word_error_rate(hypothesis: str, reference: str) -> float:
    r = reference.split()
    return edit_distance(hypothesis.split(), r) / max(len(r), 1)


def perplexity(logits: torch.Tensor, targets: torch.Tensor, ignore_index: int = -100) -> float:
    """exp of the mean token negative log-likelihood; ``logits`` [..., V], ``targets`` [...]."""
    nll = torch.nn.functional.cross_entropy(logits.reshape(-1, logits.shape[-1]).float(), targets.reshape(-1),
                                            ignore_index=ignore_index, reduction="mean")
    return float(torch.exp(nll))


def token_overlap_f1(candidate, reference) -> dict:
    c, r = Counter(candidate), Counter(reference)
    return _prf(sum((c & r).values()), sum(c.values()), sum(r.values()))


def embedding_match_score(candidate, reference, embed) -> dict:
    """Greedy cosine matching of token embeddings (BERTScore's precision / recall / F1): ``embed(tokens) -> [T, D]``."""
    c = torch.nn.functional.normalize(embed(candidate).float(), dim=-1)
    r = torch.nn.functional.normalize(embed(reference).float(), dim=-1)
    sim = c @ r.t()
    p, rec = float(sim.max(1).values.mean()), float(sim.max(0).values.mean())
    return {"precision": p, "recall": rec, "f1": 2 * p * rec / (p + rec) if p + rec else 0.0}
