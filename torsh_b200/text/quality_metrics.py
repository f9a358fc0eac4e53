"""Text evaluation suite (``crates/torsh-text/src/metrics/``): edit-distance family (``edit_distance.rs``), overlap measures and
clustering (``overlap.rs``), ROUGE-N / L / W / S / SU with multiple references and bootstrap intervals (``rouge.rs``), BLEU
smoothing variants, chrF, a METEOR-style aligner and TER (``bleu.rs``), embedding-based greedy matching with idf weights
(``bert_score.rs``), perplexity from logits / probabilities / cross-entropy with model comparison (``perplexity.rs``), coherence
(entity grid and centering, lexical chains, discourse markers, structure: ``coherence/``), fluency (lexical richness, syntactic
well-formedness, rhythm, pragmatics, language-model fluency: ``fluency/``) and semantic analysis (sentiment trajectories,
emotions, topic models with coherence, domain profiles, syntactic and latent semantic similarity: ``semantic/``)."""
from __future__ import annotations

import math
import re
import statistics
from collections import Counter, defaultdict
from typing import Callable, Sequence

import torch

from .analysis import STOPWORDS, count_syllables, sentences, words

try:
    from ..data.pipeline import PorterStemmer
    _STEM = PorterStemmer().stem
except Exception:                                                                      # pragma: no cover - the data package is part of this tree
    _STEM = lambda w: w


# ================================================================================================ edit distances
def levenshtein(a: Sequence, b: Sequence, insertion: float = 1, deletion: float = 1, substitution: float = 1) -> float:
    prev = [j * insertion for j in range(len(b) + 1)]
    for i, x in enumerate(a, 1):
        cur = [i * deletion]
        for j, y in enumerate(b, 1):
            cur.append(min(prev[j] + deletion, cur[j - 1] + insertion, prev[j - 1] + (0 if x == y else substitution)))
        prev = cur
    return prev[-1]


def optimal_string_alignment(a: Sequence, b: Sequence, transposition: float = 1) -> float:
    """Levenshtein plus adjacent transpositions, no substring edited twice."""
    d = [[0.0] * (len(b) + 1) for _ in range(len(a) + 1)]
    for i in range(len(a) + 1):
        d[i][0] = i
    for j in range(len(b) + 1):
        d[0][j] = j
    for i in range(1, len(a) + 1):
        for j in range(1, len(b) + 1):
            d[i][j] = min(d[i - 1][j] + 1, d[i][j - 1] + 1, d[i - 1][j - 1] + (a[i - 1] != b[j - 1]))
            if i > 1 and j > 1 and a[i - 1] == b[j - 2] and a[i - 2] == b[j - 1]:
                d[i][j] = min(d[i][j], d[i - 2][j - 2] + transposition)
    return d[-1][-1]


def damerau_levenshtein(a: Sequence, b: Sequence) -> int:
    """Unrestricted Damerau-Levenshtein distance (a true metric: transposed characters may be edited again)."""
    last, INF = {}, len(a) + len(b)
    d = [[INF] * (len(b) + 2) for _ in range(len(a) + 2)]
    for i in range(len(a) + 1):
        d[i + 1][1], d[i + 1][0] = i, INF
    for j in range(len(b) + 1):
        d[1][j + 1], d[0][j + 1] = j, INF
    for i in range(1, len(a) + 1):
        db = 0
        for j in range(1, len(b) + 1):
            k, l = last.get(b[j - 1], 0), db
            cost = 1
            if a[i - 1] == b[j - 1]:
                cost, db = 0, j
            d[i + 1][j + 1] = min(d[i][j] + cost, d[i + 1][j] + 1, d[i][j + 1] + 1, d[k][l] + (i - k - 1) + 1 + (j - l - 1))
        last[a[i - 1]] = i
    return d[-1][-1]


def hamming(a: Sequence, b: Sequence) -> int:
    if len(a) != len(b):
        raise ValueError("Hamming distance needs sequences of equal length")
    return sum(x != y for x, y in zip(a, b))


def jaro(a: str, b: str) -> float:
    if a == b:
        return 1.0
    if not a or not b:
        return 0.0
    win = max(len(a), len(b)) // 2 - 1
    ma, mb = [False] * len(a), [False] * len(b)
    m = 0
    for i, c in enumerate(a):
        for j in range(max(0, i - win), min(len(b), i + win + 1)):
            if not mb[j] and b[j] == c:
                ma[i] = mb[j] = True; m += 1
                break
    if not m:
        return 0.0
    sa, sb = [c for c, f in zip(a, ma) if f], [c for c, f in zip(b, mb) if f]
    t = sum(x != y for x, y in zip(sa, sb)) / 2
    return (m / len(a) + m / len(b) + (m - t) / m) / 3


def normalized_distance(fn: Callable, a: Sequence, b: Sequence) -> float: n = max(len(a), len(b)); return fn(a, b) / n if n else 0.0
def similarity(fn: Callable, a: Sequence, b: Sequence) -> float: return 1.0 - normalized_distance(fn, a, b)
def pairwise_distances(items: Sequence, fn: Callable = levenshtein) -> torch.Tensor:
    n = len(items)
    d = torch.zeros(n, n, dtype=torch.float64)
    for i in range(n):
        for j in range(i + 1, n):
            d[i, j] = d[j, i] = fn(items[i], items[j])
    return d


def find_most_similar(query: Sequence, candidates: Sequence[Sequence], fn: Callable = levenshtein, top: int = 1) -> list[tuple[int, float]]:
    return sorted(((i, normalized_distance(fn, query, c)) for i, c in enumerate(candidates)), key=lambda t: t[1])[:top]


# ================================================================================================ overlap
def _ngrams(tokens: Sequence, n: int) -> Counter: return Counter(tuple(tokens[i:i + n]) for i in range(len(tokens) - n + 1))


def ngram_overlap(a: Sequence, b: Sequence, n: int = 1) -> dict:
    ca, cb = _ngrams(a, n), _ngrams(b, n)
    inter, sa, sb = sum((ca & cb).values()), sum(ca.values()), sum(cb.values())
    union = sum((ca | cb).values())
    return {"jaccard": inter / union if union else 0.0, "dice": 2 * inter / (sa + sb) if sa + sb else 0.0, "overlap_coefficient": inter / min(sa, sb) if min(sa, sb) else 0.0, "precision": inter / sa if sa else 0.0, "recall": inter / sb if sb else 0.0}


def positional_overlap(a: Sequence, b: Sequence) -> float:
    """Share of positions (after scaling both to the same length) that hold the same token: sensitive to order."""
    if not a or not b:
        return 0.0
    n = max(len(a), len(b))
    return sum(a[int(i * len(a) / n)] == b[int(i * len(b) / n)] for i in range(n)) / n


def overlap_matrix(texts: Sequence[Sequence], n: int = 1, measure: str = "jaccard") -> torch.Tensor:
    m = torch.eye(len(texts), dtype=torch.float64)
    for i in range(len(texts)):
        for j in range(i + 1, len(texts)):
            m[i, j] = m[j, i] = ngram_overlap(texts[i], texts[j], n)[measure]
    return m


def cluster_by_overlap(texts: Sequence[Sequence], threshold: float = 0.5, n: int = 1) -> list[list[int]]:
    """Connected components of the graph that joins texts whose overlap reaches the threshold."""
    m, parent = overlap_matrix(texts, n), list(range(len(texts)))
    def find(i):
        while parent[i] != i:
            parent[i] = parent[parent[i]]; i = parent[i]
        return i
    for i in range(len(texts)):
        for j in range(i + 1, len(texts)):
            if m[i, j] >= threshold:
                parent[find(i)] = find(j)
    groups = defaultdict(list)
    for i in range(len(texts)):
        groups[find(i)].append(i)
    return sorted(groups.values())


# ================================================================================================ ROUGE
def _prep(tokens: Sequence[str], stem: bool, remove_stopwords: bool) -> list[str]:
    t = [w for w in tokens if not (remove_stopwords and w in STOPWORDS)]
    return [_STEM(w) for w in t] if stem else list(t)


def _prf(match: float, cand: float, ref: float, beta: float = 1.0) -> dict:
    p, r = (match / cand if cand else 0.0), (match / ref if ref else 0.0)
    return {"precision": p, "recall": r, "f": (1 + beta * beta) * p * r / (r + beta * beta * p) if p + r else 0.0}


def _lcs_table(a, b):
    t = [[0] * (len(b) + 1) for _ in range(len(a) + 1)]
    for i, x in enumerate(a, 1):
        for j, y in enumerate(b, 1):
            t[i][j] = t[i - 1][j - 1] + 1 if x == y else max(t[i - 1][j], t[i][j - 1])
    return t


def rouge(candidate: Sequence[str], references: Sequence[Sequence[str]] | Sequence[str], variant: str = "rouge-1", stem: bool = False, remove_stopwords: bool = False, beta: float = 1.0, multi: str = "max", weight: float = 1.2, skip: int | None = None) -> dict:
    """``rouge-N``, ``rouge-l`` (longest common subsequence), ``rouge-w`` (consecutive matches weighted ``k^weight``), ``rouge-s`` (skip
    bigrams within ``skip`` words) and ``rouge-su`` (skip bigrams plus unigrams).  Several references are combined by ``max`` or
    ``mean`` of the F-score."""
    refs = [references] if references and isinstance(references[0], str) else list(references)
    c = _prep(candidate, stem, remove_stopwords)
    rows = []
    for ref in refs:
        r = _prep(ref, stem, remove_stopwords)
        if variant.startswith("rouge-") and variant[6:].isdigit():
            n = int(variant[6:]); cc, rc = _ngrams(c, n), _ngrams(r, n)
            rows.append(_prf(sum((cc & rc).values()), sum(cc.values()), sum(rc.values()), beta))
        elif variant == "rouge-l":
            rows.append(_prf(_lcs_table(c, r)[-1][-1], len(c), len(r), beta))
        elif variant == "rouge-w":
            f = lambda k: k ** weight
            cst = [[0.0] * (len(r) + 1) for _ in range(len(c) + 1)]
            run = [[0] * (len(r) + 1) for _ in range(len(c) + 1)]
            for i, x in enumerate(c, 1):
                for j, y in enumerate(r, 1):
                    if x == y:
                        k = run[i - 1][j - 1]
                        cst[i][j], run[i][j] = cst[i - 1][j - 1] + f(k + 1) - f(k), k + 1
                    else:
                        cst[i][j] = max(cst[i - 1][j], cst[i][j - 1])
            w = cst[-1][-1]
            inv = lambda v: v ** (1 / weight)
            p, rec = (inv(w / f(len(c))) if c else 0.0), (inv(w / f(len(r))) if r else 0.0)
            rows.append({"precision": p, "recall": rec, "f": (1 + beta ** 2) * p * rec / (rec + beta ** 2 * p) if p + rec else 0.0})
        elif variant in ("rouge-s", "rouge-su"):
            def skips(t):
                out = Counter((t[i], t[j]) for i in range(len(t)) for j in range(i + 1, len(t) if skip is None else min(len(t), i + skip + 2)))
                if variant == "rouge-su":
                    out.update((w,) for w in t)
                return out
            cc, rc = skips(c), skips(r)
            rows.append(_prf(sum((cc & rc).values()), sum(cc.values()), sum(rc.values()), beta))
        else:
            raise ValueError(variant)
    if multi == "max":
        return max(rows, key=lambda d: d["f"])
    return {k: statistics.fmean(d[k] for d in rows) for k in rows[0]}


def rouge_l_summary(candidate_sentences: Sequence[Sequence[str]], reference_sentences: Sequence[Sequence[str]], beta: float = 1.0) -> dict:
    """Summary-level ROUGE-L: for every reference sentence the union of its LCS with all candidate sentences."""
    hits = 0
    for r in reference_sentences:
        covered = set()
        for c in candidate_sentences:
            t = _lcs_table(c, r)
            i, j = len(c), len(r)
            while i and j:
                if c[i - 1] == r[j - 1]:
                    covered.add(j - 1); i -= 1; j -= 1
                elif t[i - 1][j] >= t[i][j - 1]:
                    i -= 1
                else:
                    j -= 1
        hits += len(covered)
    return _prf(hits, sum(len(c) for c in candidate_sentences), sum(len(r) for r in reference_sentences), beta)


def bootstrap_interval(scores: Sequence[float], samples: int = 1000, confidence: float = 0.95, seed: int = 0) -> dict:
    g = torch.Generator().manual_seed(seed)
    s = torch.tensor(scores, dtype=torch.float64)
    means = s[torch.randint(len(s), (samples, len(s)), generator=g)].mean(1).sort().values
    lo, hi = means[int((1 - confidence) / 2 * samples)], means[min(samples - 1, int((1 + confidence) / 2 * samples))]
    return {"mean": float(s.mean()), "lower": float(lo), "upper": float(hi), "width": float(hi - lo), "margin_of_error": float(hi - lo) / 2}


# ================================================================================================ BLEU variants, chrF, METEOR-style, TER
def bleu_detailed(candidate: Sequence[str], references: Sequence[Sequence[str]], max_n: int = 4, smoothing: str = "none", weights: Sequence[float] | None = None) -> dict:
    """Sentence BLEU with clipped n-gram precisions, brevity penalty and a smoothing method: ``none``, ``epsilon`` (zero counts
    become 0.1), ``add_one`` (orders above one), ``exponential`` (each zero precision halves the previous floor)."""
    weights = list(weights or [1 / max_n] * max_n)
    precs, floor = [], 1.0
    for n in range(1, max_n + 1):
        cc = _ngrams(candidate, n)
        best = Counter()
        for r in references:
            for g, v in _ngrams(r, n).items():
                best[g] = max(best[g], v)
        m, tot = sum(min(v, best[g]) for g, v in cc.items()), sum(cc.values())
        if smoothing == "add_one" and n > 1:
            m, tot = m + 1, tot + 1
        if m == 0 and tot:
            if smoothing == "epsilon":
                m = 0.1
            elif smoothing == "exponential":
                floor /= 2; m = floor
        precs.append(m / tot if tot else 0.0)
    c = len(candidate)
    r = min((abs(len(x) - c), len(x)) for x in references)[1]
    bp = 1.0 if c > r else math.exp(1 - r / c) if c else 0.0
    score = bp * math.exp(sum(w * math.log(p) for w, p in zip(weights, precs))) if all(p > 0 for p in precs) else 0.0
    return {"bleu": score, "precisions": precs, "brevity_penalty": bp, "length_ratio": c / r if r else 0.0, "candidate_length": c, "reference_length": r}


def chrf(candidate: str, reference: str, max_n: int = 6, beta: float = 2.0, word_n: int = 0) -> float:
    """Character n-gram F-score (``word_n = 2`` gives chrF++): the mean over orders of precision and recall, combined with ``beta``."""
    def grams(s, n): s = s.replace(" ", ""); return Counter(s[i:i + n] for i in range(len(s) - n + 1))
    ps, rs = [], []
    for n in range(1, max_n + 1):
        c, r = grams(candidate, n), grams(reference, n)
        if not c and not r:
            continue
        m = sum((c & r).values())
        ps.append(m / sum(c.values()) if c else 0.0); rs.append(m / sum(r.values()) if r else 0.0)
    for n in range(1, word_n + 1):
        c, r = _ngrams(candidate.split(), n), _ngrams(reference.split(), n)
        if c or r:
            m = sum((c & r).values())
            ps.append(m / sum(c.values()) if c else 0.0); rs.append(m / sum(r.values()) if r else 0.0)
    if not ps:
        return 0.0
    p, r = statistics.fmean(ps), statistics.fmean(rs)
    return (1 + beta ** 2) * p * r / (beta ** 2 * p + r) if p + r else 0.0


def meteor_like(candidate: Sequence[str], reference: Sequence[str], alpha: float = 0.9, beta: float = 3.0, gamma: float = 0.5, synonyms: dict | None = None) -> dict:
    """Unigram alignment in stages (exact, stem, synonym table), recall-weighted harmonic mean and a fragmentation penalty
    ``gamma (chunks / matches)^beta``."""
    used, align = set(), {}
    stages = [lambda a, b: a == b, lambda a, b: _STEM(a) == _STEM(b), lambda a, b: b in (synonyms or {}).get(a, ()) or a in (synonyms or {}).get(b, ())]
    for match in stages:
        for i, w in enumerate(candidate):
            if i in align:
                continue
            for j, v in enumerate(reference):
                if j not in used and match(w, v):
                    align[i] = j; used.add(j)
                    break
    m = len(align)
    if not m:
        return {"score": 0.0, "precision": 0.0, "recall": 0.0, "chunks": 0, "penalty": 0.0}
    p, r = m / len(candidate), m / len(reference)
    fmean = p * r / (alpha * p + (1 - alpha) * r)
    idx = sorted(align)
    chunks = 1 + sum(1 for a, b in zip(idx, idx[1:]) if not (b == a + 1 and align[b] == align[a] + 1))
    pen = gamma * (chunks / m) ** beta
    return {"score": fmean * (1 - pen), "precision": p, "recall": r, "chunks": chunks, "penalty": pen}


def translation_edit_rate(candidate: Sequence[str], reference: Sequence[str], max_shift: int = 10) -> float:
    """Edits (insert, delete, substitute, and block shifts, each round taking the shift that reduces the distance most) per
    reference word."""
    hyp, shifts = list(candidate), 0
    best = levenshtein(hyp, reference)
    while best:
        choice = None                                                               # the single shift that lowers the distance most
        for length in range(min(max_shift, len(hyp) - 1), 0, -1):
            for i in range(len(hyp) - length + 1):
                block, rest = hyp[i:i + length], hyp[:i] + hyp[i + length:]
                for j in range(len(rest) + 1):
                    if j == i:
                        continue
                    cand = rest[:j] + block + rest[j:]
                    d = levenshtein(cand, reference)
                    if d + 1 < best and (choice is None or d < choice[0]):
                        choice = (d, cand)
        if choice is None:
            break
        best, hyp, shifts = choice[0], choice[1], shifts + 1
    return (best + shifts) / max(len(reference), 1)


# ================================================================================================ embedding-based matching
def embedding_score(cand_emb: torch.Tensor, ref_emb: torch.Tensor, cand_idf: torch.Tensor | None = None, ref_idf: torch.Tensor | None = None, baseline: float | None = None) -> dict:
    """Greedy matching of token embeddings by cosine similarity: precision averages every candidate token's best match,
    recall every reference token's; idf weights emphasise rare tokens; ``baseline`` rescales to a more readable range."""
    c, r = torch.nn.functional.normalize(cand_emb.double(), dim=-1), torch.nn.functional.normalize(ref_emb.double(), dim=-1)
    sim = c @ r.T
    wc = torch.ones(len(c), dtype=torch.float64) if cand_idf is None else cand_idf.double()
    wr = torch.ones(len(r), dtype=torch.float64) if ref_idf is None else ref_idf.double()
    p, rec = float((sim.max(1).values * wc).sum() / wc.sum()), float((sim.max(0).values * wr).sum() / wr.sum())
    f = 2 * p * rec / (p + rec) if p + rec else 0.0
    if baseline is not None:
        p, rec, f = [(v - baseline) / (1 - baseline) for v in (p, rec, f)]
    return {"precision": p, "recall": rec, "f": f}


def idf_weights(corpus: Sequence[Sequence[str]]) -> dict:
    n, df = len(corpus), Counter(w for doc in corpus for w in set(doc))
    return defaultdict(lambda: math.log((n + 1) / 1), {w: math.log((n + 1) / (c + 1)) for w, c in df.items()})


# ================================================================================================ perplexity
def perplexity_from_logits(logits: torch.Tensor, targets: torch.Tensor, ignore_index: int = -100, per_sequence: bool = False):
    nll = torch.nn.functional.cross_entropy(logits.reshape(-1, logits.shape[-1]).float(), targets.reshape(-1), ignore_index=ignore_index, reduction="none").reshape(targets.shape)
    mask = targets != ignore_index
    if per_sequence:
        return torch.exp((nll * mask).sum(-1) / mask.sum(-1).clamp_min(1))
    return float(torch.exp(nll[mask].mean()))


def perplexity_from_probabilities(probs: Sequence[float], min_probability: float = 1e-12) -> float: return math.exp(-statistics.fmean(math.log(max(p, min_probability)) for p in probs))
def perplexity_from_cross_entropy(ce: float, base: float = math.e) -> float: return base ** ce
def bits_per_character(total_nll_nats: float, characters: int) -> float: return total_nll_nats / math.log(2) / characters


def compare_perplexities(model1: Sequence[float], model2: Sequence[float]) -> dict:
    """Per-sequence perplexities of two models on the same texts: means, win rate of model 2, relative improvement and a paired
    sign-flip test on the log perplexities."""
    d = [math.log(a) - math.log(b) for a, b in zip(model1, model2)]
    g = torch.Generator().manual_seed(0)
    dt = torch.tensor(d, dtype=torch.float64)
    flips = (torch.randint(0, 2, (2000, len(d)), generator=g) * 2 - 1).double()
    p = float(((flips * dt).mean(1).abs() >= abs(float(dt.mean())) - 1e-15).double().mean())
    m1, m2 = statistics.fmean(model1), statistics.fmean(model2)
    return {"mean1": m1, "mean2": m2, "model2_win_rate": sum(x > 0 for x in d) / len(d), "improvement_percentage": 100 * (m1 - m2) / m1, "is_model2_better": m2 < m1 and p < 0.05, "p_value": p}


def perplexity_quality(ppl: float) -> str: return "excellent" if ppl < 20 else "good" if ppl < 50 else "fair" if ppl < 100 else "poor"


# ================================================================================================ coherence
DISCOURSE_MARKERS = {"additive": {"and", "also", "moreover", "furthermore", "besides", "additionally", "in addition"}, "adversative": {"but", "however", "yet", "nevertheless", "although", "though", "whereas", "on the other hand", "in contrast"},
                     "causal": {"because", "therefore", "thus", "hence", "so", "consequently", "since", "as a result"}, "temporal": {"then", "next", "finally", "meanwhile", "afterwards", "before", "after", "first", "second", "later", "subsequently"},
                     "exemplifying": {"for example", "for instance", "such as", "namely", "specifically"}, "summarising": {"in conclusion", "in summary", "overall", "to sum up", "in short"}}
_PRONOUNS = {"he", "she", "it", "they", "him", "her", "them", "his", "its", "their", "this", "that", "these", "those"}


def _content(sent: str) -> list[str]: return [w for w in words(sent) if w not in STOPWORDS and len(w) > 2]


def entity_grid(text: str, min_mentions: int = 2) -> dict:
    """Entities (content words mentioned in at least ``min_mentions`` sentences) against sentences; a cell is ``S`` when the entity
    opens the sentence (before the first verb-like position: the first third), ``O`` when it follows, ``-`` when absent.  Transition
    probabilities over adjacent sentences and the share of ``continue`` (S->S), ``retain`` (S->O / O->S), ``shift`` (to or from
    absence) describe how the focus moves."""
    sents = sentences(text)
    toks = [_content(s) for s in sents]
    ents = [e for e, c in Counter(w for t in toks for w in set(t)).items() if c >= min_mentions]
    grid = {e: ["-" if e not in t else ("S" if t.index(e) < max(1, len(t) // 3) else "O") for t in toks] for e in ents}
    trans = Counter((r[i], r[i + 1]) for r in grid.values() for i in range(len(r) - 1))
    total = sum(trans.values()) or 1
    probs = {f"{a}{b}": v / total for (a, b), v in trans.items()}
    present = sum(v for (a, b), v in trans.items() if a != "-" and b != "-")
    cont, ret = trans[("S", "S")], trans[("S", "O")] + trans[("O", "S")] + trans[("O", "O")]
    return {"entities": sorted(ents), "grid": grid, "transitions": probs, "continue": cont / total, "retain": ret / total, "shift": 1 - present / total - probs.get("--", 0.0), "density": present / total, "coherence": (2 * cont + ret) / (2 * total)}


def lexical_chains(text: str, max_gap: int = 3) -> list[dict]:
    """Chains of repeated content words (stemmed) whose consecutive mentions are at most ``max_gap`` sentences apart."""
    pos = defaultdict(list)
    for i, s in enumerate(sentences(text)):
        for w in set(_content(s)):
            pos[_STEM(w)].append(i)
    chains = []
    for w, idx in pos.items():
        run = [idx[0]]
        for i in idx[1:]:
            if i - run[-1] <= max_gap:
                run.append(i)
            else:
                if len(run) > 1:
                    chains.append({"word": w, "sentences": run, "span": run[-1] - run[0] + 1, "strength": len(run) / (run[-1] - run[0] + 1)})
                run = [i]
        if len(run) > 1:
            chains.append({"word": w, "sentences": run, "span": run[-1] - run[0] + 1, "strength": len(run) / (run[-1] - run[0] + 1)})
    return sorted(chains, key=lambda c: -len(c["sentences"]))


def discourse_markers(text: str) -> dict:
    low = " " + " ".join(words(text)) + " "
    counts = {k: sum(low.count(f" {m} ") for m in ms) for k, ms in DISCOURSE_MARKERS.items()}
    n_s, total = max(len(sentences(text)), 1), sum(counts.values())
    ent = -sum(c / total * math.log(c / total) for c in counts.values() if c) if total else 0.0
    return {"counts": counts, "per_sentence": total / n_s, "diversity": ent / math.log(len(counts)), "dominant": max(counts, key=counts.get) if total else None}


def local_coherence(text: str) -> dict:
    """Cosine similarity of adjacent sentences' content-word counts (plus pronoun links, which tie a sentence to the previous
    one without repeating words); the minimum locates the weakest transition."""
    sents = sentences(text)
    vecs = [Counter(_STEM(w) for w in _content(s)) for s in sents]
    sims = []
    for i in range(len(vecs) - 1):
        a, b = vecs[i], vecs[i + 1]
        num = sum(a[k] * b[k] for k in a)
        den = math.sqrt(sum(v * v for v in a.values()) * sum(v * v for v in b.values()))
        link = 0.15 if set(words(sents[i + 1])[:3]) & _PRONOUNS else 0.0
        sims.append(min(1.0, (num / den if den else 0.0) + link))
    return {"adjacent": sims, "mean": statistics.fmean(sims) if sims else 1.0, "weakest_transition": min(range(len(sims)), key=sims.__getitem__) if sims else None}


def structural_coherence(text: str) -> dict:
    paras = [p for p in re.split(r"\n\s*\n", text.strip()) if p.strip()]
    lens = [len(words(p)) for p in paras]
    balance = 1 - (statistics.pstdev(lens) / statistics.fmean(lens) if len(lens) > 1 and statistics.fmean(lens) else 0.0)
    topical = []
    for p in paras:
        ss = sentences(p)
        if len(ss) > 1:
            first, rest = set(_content(ss[0])), set(w for s in ss[1:] for w in _content(s))
            topical.append(len(first & rest) / len(first) if first else 0.0)
    return {"paragraphs": len(paras), "paragraph_lengths": lens, "balance": max(0.0, balance), "topic_sentence_support": statistics.fmean(topical) if topical else 0.0,
            "has_introduction_marker": bool(re.search(r"\b(first|introduc|this (paper|essay|article))", paras[0].lower())) if paras else False, "has_conclusion_marker": bool(re.search(r"\b(in conclusion|in summary|overall|finally|to sum up)", paras[-1].lower())) if paras else False}


def coherence_report(text: str, weights: dict | None = None) -> dict:
    w = {"entity": 0.3, "lexical": 0.25, "local": 0.25, "discourse": 0.1, "structure": 0.1, **(weights or {})}
    eg, lc, loc, dm, st = entity_grid(text), lexical_chains(text), local_coherence(text), discourse_markers(text), structural_coherence(text)
    n_s = max(len(sentences(text)), 1)
    parts = {"entity": eg["coherence"], "lexical": min(1.0, sum(len(c["sentences"]) for c in lc) / (2 * n_s)), "local": loc["mean"], "discourse": min(1.0, dm["per_sentence"]), "structure": st["balance"]}
    return {"score": sum(w[k] * parts[k] for k in parts), "components": parts, "weakest_transition": loc["weakest_transition"], "chains": len(lc)}


# ================================================================================================ fluency
def lexical_richness(tokens: Sequence[str]) -> dict:
    n, freq = len(tokens), Counter(tokens)
    v, spec = len(freq), Counter(freq.values())
    v1 = spec[1]
    yule_k = 1e4 * (sum(i * i * c for i, c in spec.items()) - n) / (n * n) if n else 0.0
    return {"tokens": n, "types": v, "ttr": v / n if n else 0.0, "root_ttr": v / math.sqrt(n) if n else 0.0, "log_ttr": math.log(v) / math.log(n) if n > 1 else 0.0, "hapax_ratio": v1 / v if v else 0.0,
            "dis_legomena_ratio": spec[2] / v if v else 0.0, "yule_k": yule_k, "simpson_d": sum(c * (c - 1) for c in freq.values()) / (n * (n - 1)) if n > 1 else 0.0, "honore_r": 100 * math.log(n) / (1 - v1 / v) if v and v1 < v else math.inf,
            "mean_word_length": statistics.fmean(len(w) for w in tokens) if tokens else 0.0}


_IRREGULAR = {"sat", "went", "ran", "saw", "came", "took", "made", "said", "got", "gave", "found", "left", "fell", "rose", "grew", "knew", "wrote", "ate", "began", "broke", "brought", "built", "bought", "caught", "chose", "drew", "drank", "drove",
              "felt", "flew", "forgot", "heard", "held", "kept", "led", "lost", "met", "paid", "put", "read", "rode", "rang", "sang", "sent", "set", "slept", "spoke", "spent", "stood", "swam", "taught", "told", "thought", "threw", "understood", "wore", "won", "lay", "hit", "cut", "let", "run", "go", "see", "come", "take", "make", "say", "get", "give", "find", "know"}


def syntactic_fluency(text: str) -> dict:
    """Surface well-formedness: sentence-length profile, capitalisation and end punctuation, balanced brackets / quotes, doubled
    words, ``a`` / ``an`` agreement, fragments (no finite-verb cue) and run-ons (long sentences without internal punctuation)."""
    sents, issues = sentences(text), []
    lens = [len(words(s)) for s in sents]
    for i, s in enumerate(sents):
        ws = words(s)
        if s and s[0].isalpha() and not s[0].isupper():
            issues.append({"sentence": i, "kind": "capitalisation"})
        if s and s.rstrip()[-1] not in ".!?\"')":
            issues.append({"sentence": i, "kind": "end_punctuation"})
        for a, b in zip(ws, ws[1:]):
            if a == b and a not in ("that", "had", "very"):
                issues.append({"sentence": i, "kind": "doubled_word", "word": a})
            if a in ("a", "an") and b and (b[0] in "aeiou") != (a == "an") and not b.startswith(("uni", "use", "one", "eu")) and not (a == "an" and b.startswith(("hour", "hon"))):
                issues.append({"sentence": i, "kind": "article_agreement", "word": f"{a} {b}"})
        if len(ws) > 40 and not re.search(r"[,;:]", s):
            issues.append({"sentence": i, "kind": "run_on"})
        if 0 < len(ws) < 3 or (ws and not any(w in ws for w in ("is", "are", "was", "were", "be", "has", "have", "had", "do", "does", "did", "will", "can", "could", "would", "should", "may", "might", "must")) and not any(w.endswith(("ed", "es", "s", "ing")) or w in _IRREGULAR for w in ws[1:])):
            issues.append({"sentence": i, "kind": "fragment"})
    for o, c in (("(", ")"), ("[", "]"), ("{", "}")):
        if text.count(o) != text.count(c):
            issues.append({"kind": "unbalanced", "symbol": o + c})
    if text.count('"') % 2:
        issues.append({"kind": "unbalanced", "symbol": '"'})
    n = max(len(sents), 1)
    return {"sentences": len(sents), "mean_length": statistics.fmean(lens) if lens else 0.0, "length_std": statistics.pstdev(lens) if lens else 0.0, "issues": issues, "score": max(0.0, 1 - len(issues) / (2 * n))}


def rhythm_analysis(text: str) -> dict:
    """Prosodic surface features: syllables per word and per sentence, variation of sentence cadence (normalised pairwise
    variability of syllable counts), pauses from punctuation, alliteration and simple end rhyme between adjacent lines."""
    sents = sentences(text)
    syl_w = [count_syllables(w) for w in words(text)]
    syl_s = [sum(count_syllables(w) for w in words(s)) for s in sents]
    npvi = 100 * statistics.fmean(abs(a - b) / ((a + b) / 2) for a, b in zip(syl_s, syl_s[1:]) if a + b) if len(syl_s) > 1 else 0.0
    ws = words(text)
    allit = sum(1 for a, b in zip(ws, ws[1:]) if a[0] == b[0] and a[0].isalpha() and a not in STOPWORDS and b not in STOPWORDS) / max(len(ws) - 1, 1)
    lines = [l for l in text.splitlines() if l.strip()]
    ends = [re.sub(r"[^a-z]", "", l.lower().split()[-1])[-3:] for l in lines if l.split()]
    rhyme = sum(1 for a, b in zip(ends, ends[1:]) if a and a[-2:] == b[-2:]) / max(len(ends) - 1, 1) if len(ends) > 1 else 0.0
    pauses = len(re.findall(r"[,;:—-]", text)) / max(len(ws), 1)
    return {"syllables_per_word": statistics.fmean(syl_w) if syl_w else 0.0, "syllables_per_sentence": syl_s, "polysyllabic_ratio": sum(s >= 3 for s in syl_w) / max(len(syl_w), 1), "cadence_variability": npvi,
            "regularity": 1 / (1 + npvi / 100), "pause_rate": pauses, "alliteration": allit, "end_rhyme": rhyme}


_HEDGES = {"maybe", "perhaps", "possibly", "might", "could", "seems", "appears", "somewhat", "arguably", "likely", "probably", "suggests"}
_POLITE = {"please", "thank", "thanks", "kindly", "appreciate", "grateful", "sorry", "welcome", "would", "could"}
_INFORMAL = {"gonna", "wanna", "kinda", "yeah", "ok", "okay", "stuff", "guys", "cool", "lol", "hey", "awesome", "cuz", "dunno"}
_FORMAL = {"therefore", "furthermore", "moreover", "consequently", "nevertheless", "regarding", "thus", "hence", "whereas", "herein", "pursuant", "notwithstanding"}
_INTENS = {"very", "really", "extremely", "absolutely", "totally", "incredibly", "highly"}


def pragmatic_analysis(text: str) -> dict:
    ws = words(text)
    n = max(len(ws), 1)
    contractions = len(re.findall(r"\b\w+'(t|s|re|ve|ll|d|m)\b", text.lower()))
    second, first = sum(w in ("you", "your", "yours") for w in ws), sum(w in ("i", "me", "my", "we", "our", "us") for w in ws)
    formal = sum(w in _FORMAL for w in ws) + sum(len(w) > 9 for w in ws) * 0.25
    informal = sum(w in _INFORMAL for w in ws) + contractions + text.count("!") * 0.5
    formality = (formal + 1) / (formal + informal + 2)
    return {"hedging": sum(w in _HEDGES for w in ws) / n, "politeness": sum(w in _POLITE for w in ws) / n, "intensifiers": sum(w in _INTENS for w in ws) / n, "formality": formality,
            "register": "formal" if formality > 0.6 else "informal" if formality < 0.4 else "neutral", "questions": text.count("?"), "directness": 1 - min(1.0, 5 * sum(w in _HEDGES for w in ws) / n), "addressee_focus": second / n, "author_presence": first / n}


def fluency_report(text: str, lm=None) -> dict:
    """Combined fluency: lexical, syntactic, rhythmic and (when an n-gram model with ``perplexity(tokens)`` is given) statistical."""
    lex, syn, rhy = lexical_richness(words(text)), syntactic_fluency(text), rhythm_analysis(text)
    parts = {"lexical": min(1.0, lex["root_ttr"] / 8), "syntactic": syn["score"], "rhythm": rhy["regularity"]}
    if lm is not None:
        ppl = lm.perplexity(words(text))
        parts["statistical"] = 1 / (1 + math.log(max(ppl, 1.0)) / 5)
    return {"score": statistics.fmean(parts.values()), "components": parts, "issues": syn["issues"]}


# ================================================================================================ semantics
_POS_W = {"good", "great", "excellent", "happy", "love", "wonderful", "best", "amazing", "positive", "success", "enjoy", "pleasant", "beautiful", "win", "hope", "joy", "delight", "brilliant"}
_NEG_W = {"bad", "terrible", "awful", "sad", "hate", "worst", "horrible", "negative", "failure", "pain", "angry", "ugly", "lose", "fear", "poor", "disaster", "broken", "miserable"}
_NEGATORS = {"not", "no", "never", "n't", "hardly", "without"}
EMOTION_LEXICON = {"joy": {"happy", "joy", "delight", "glad", "cheerful", "love", "enjoy", "smile", "laugh"}, "sadness": {"sad", "cry", "grief", "sorrow", "lonely", "miserable", "tears", "mourn"},
                   "anger": {"angry", "furious", "rage", "hate", "annoyed", "outrage", "hostile"}, "fear": {"afraid", "fear", "scared", "terror", "panic", "anxious", "dread", "worry"},
                   "surprise": {"surprise", "astonished", "amazed", "unexpected", "sudden", "shock"}, "trust": {"trust", "reliable", "honest", "faith", "loyal", "confident", "safe"}}


def sentence_sentiment(sent: str) -> float:
    ws, score, n = words(sent), 0.0, 0
    for i, w in enumerate(ws):
        s = 1.0 if w in _POS_W else -1.0 if w in _NEG_W else 0.0
        if s:
            if any(p in _NEGATORS or p.endswith("n't") for p in ws[max(0, i - 3):i]):
                s = -0.8 * s
            if i and ws[i - 1] in _INTENS:
                s *= 1.5
            score += s; n += 1
    return max(-1.0, min(1.0, score / n)) if n else 0.0


def sentiment_trajectory(text: str) -> dict:
    vals = [sentence_sentiment(s) for s in sentences(text)]
    if len(vals) > 1:
        xs = list(range(len(vals)))
        mx, my = statistics.fmean(xs), statistics.fmean(vals)
        slope = sum((x - mx) * (y - my) for x, y in zip(xs, vals)) / sum((x - mx) ** 2 for x in xs)
    else:
        slope = 0.0
    flips = sum(1 for a, b in zip(vals, vals[1:]) if a * b < 0)
    return {"per_sentence": vals, "mean": statistics.fmean(vals) if vals else 0.0, "slope": slope, "trend": "improving" if slope > 0.05 else "declining" if slope < -0.05 else "stable", "volatility": statistics.pstdev(vals) if vals else 0.0, "polarity_flips": flips}


def emotion_scores(text: str) -> dict:
    ws = [_STEM(w) for w in words(text)]
    lex = {k: {_STEM(w) for w in v} for k, v in EMOTION_LEXICON.items()}
    raw = {k: sum(w in v for w in ws) for k, v in lex.items()}
    tot = sum(raw.values())
    return {"scores": {k: v / tot if tot else 0.0 for k, v in raw.items()}, "dominant": max(raw, key=raw.get) if tot else None, "intensity": tot / max(len(ws), 1)}


def nmf_topics(docs: Sequence[Sequence[str]], k: int = 2, iters: int = 200, top: int = 8, seed: int = 0, min_df: int = 1) -> dict:
    """Non-negative factorisation of the tf-idf matrix by multiplicative updates: ``V ~ W H`` with document-topic ``W`` and
    topic-word ``H``; returns the top words per topic, the document assignments and the UMass coherence of each topic."""
    df = Counter(w for d in docs for w in set(d))
    vocab = sorted(w for w, c in df.items() if c >= min_df and w not in STOPWORDS)
    index = {w: i for i, w in enumerate(vocab)}
    V = torch.zeros(len(docs), len(vocab), dtype=torch.float64)
    for i, d in enumerate(docs):
        for w, c in Counter(d).items():
            if w in index:
                V[i, index[w]] = c * math.log((1 + len(docs)) / (1 + df[w]) + 1)
    g = torch.Generator().manual_seed(seed)
    W, H = torch.rand(len(docs), k, generator=g, dtype=torch.float64) + 0.1, torch.rand(k, len(vocab), generator=g, dtype=torch.float64) + 0.1
    for _ in range(iters):
        H = H * (W.T @ V) / (W.T @ W @ H + 1e-12)
        W = W * (V @ H.T) / (W @ H @ H.T + 1e-12)
    topics = [[vocab[j] for j in H[t].topk(min(top, len(vocab))).indices.tolist()] for t in range(k)]
    sets = [set(d) for d in docs]
    def umass(ws):
        s = 0.0
        for i in range(1, len(ws)):
            for j in range(i):
                co, dj = sum(ws[i] in d and ws[j] in d for d in sets), sum(ws[j] in d for d in sets)
                s += math.log((co + 1) / dj) if dj else 0.0
        return s / max(len(ws) * (len(ws) - 1) / 2, 1)
    return {"topics": topics, "assignments": W.argmax(1).tolist(), "document_topic": W / W.sum(1, keepdim=True).clamp_min(1e-12), "coherence": [umass(t[:5]) for t in topics], "reconstruction_error": float((V - W @ H).norm() / V.norm())}


DOMAIN_PROFILES = {"medical": {"patient", "clinical", "treatment", "disease", "diagnosis", "therapy", "symptoms", "dose", "hospital", "surgery"}, "legal": {"court", "plaintiff", "defendant", "statute", "contract", "liability", "jurisdiction", "appeal", "clause", "law"},
                   "finance": {"market", "stock", "investment", "revenue", "profit", "interest", "bank", "asset", "equity", "inflation"}, "technology": {"software", "algorithm", "data", "network", "computer", "system", "model", "code", "server", "hardware"},
                   "sports": {"team", "game", "player", "score", "season", "coach", "match", "league", "win", "goal"}}


def classify_domain(text: str) -> dict:
    ws = Counter(words(text))
    raw = {d: sum(ws[w] + ws[w + "s"] for w in kw) for d, kw in DOMAIN_PROFILES.items()}
    tot = sum(raw.values())
    return {"domain": max(raw, key=raw.get) if tot else "general", "scores": {d: v / tot if tot else 0.0 for d, v in raw.items()}, "confidence": max(raw.values()) / tot if tot else 0.0}


_FUNCTION = STOPWORDS


def syntactic_similarity(a: str, b: str) -> dict:
    """Similarity of form rather than content: sequences of word classes (function word kept as is, content word replaced by a
    shape: capitalised / number / suffix class) compared by normalised edit distance, plus the similarity of the
    sentence-length and punctuation profiles."""
    def shape(text):
        out = []
        for w in re.findall(r"[A-Za-z']+|\d+|[.,;:!?]", text):
            l = w.lower()
            out.append(l if l in _FUNCTION or not w[0].isalnum() else "NUM" if w.isdigit() else "ING" if l.endswith("ing") else "ED" if l.endswith("ed") else "LY" if l.endswith("ly") else "PL" if l.endswith("s") else "CAP" if w[0].isupper() else "W")
        return out
    sa, sb = shape(a), shape(b)
    struct = similarity(levenshtein, sa, sb)
    la, lb = [len(words(s)) for s in sentences(a)] or [0], [len(words(s)) for s in sentences(b)] or [0]
    length = 1 - abs(statistics.fmean(la) - statistics.fmean(lb)) / max(statistics.fmean(la), statistics.fmean(lb), 1)
    pa, pb = Counter(c for c in a if c in ".,;:!?"), Counter(c for c in b if c in ".,;:!?")
    punct = sum((pa & pb).values()) / max(sum((pa | pb).values()), 1)
    return {"structure": struct, "length": length, "punctuation": punct, "score": 0.6 * struct + 0.2 * length + 0.2 * punct}


def latent_semantic_similarity(docs: Sequence[Sequence[str]], rank: int = 2) -> torch.Tensor:
    """Cosine similarity of documents in the space of the leading singular vectors of the tf-idf matrix (documents sharing no
    word can still be close when their words co-occur elsewhere)."""
    df = Counter(w for d in docs for w in set(d))
    vocab = {w: i for i, w in enumerate(sorted(df))}
    V = torch.zeros(len(docs), len(vocab), dtype=torch.float64)
    for i, d in enumerate(docs):
        for w, c in Counter(d).items():
            V[i, vocab[w]] = c * (math.log((1 + len(docs)) / (1 + df[w])) + 1)
    U, S, _ = torch.linalg.svd(V, full_matrices=False)
    Z = torch.nn.functional.normalize(U[:, :rank] * S[:rank], dim=1)
    return Z @ Z.T
