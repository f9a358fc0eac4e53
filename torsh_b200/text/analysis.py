"""Text analysis and task models (``crates/torsh-text/src/{analysis,utils,convenience,models}.rs`` and ``metrics/``):
sentence and syllable segmentation, readability and lexical-diversity scores, n-gram language models with smoothing,
TF-IDF / BM25 retrieval, similarity measures, keyword extraction (RAKE, TextRank), extractive summarisation, lexicon
sentiment with negation handling, character n-gram language identification, pattern-based entity extraction, lexical
cohesion, and text classifiers (BiLSTM, CNN, Transformer) with a sequence tagger."""
from __future__ import annotations

import math
import re
from collections import Counter, defaultdict
from typing import Iterable, Sequence

import torch
from torch import nn

from ..data.pipeline import STOPWORDS

_WORD = re.compile(r"[A-Za-z0-9]+(?:['-][A-Za-z0-9]+)*")
_ABBREV = {"mr", "mrs", "ms", "dr", "prof", "sr", "jr", "st", "vs", "etc", "e.g", "i.e", "inc", "ltd", "co", "fig", "no"}


def words(text: str, lower: bool = True) -> list[str]: return [w.lower() if lower else w for w in _WORD.findall(text)]


def sentences(text: str) -> list[str]:
    """Splits on ``. ! ?`` followed by whitespace and a capital / quote / digit, but not after known abbreviations,
    initials or inside numbers."""
    out, start = [], 0
    for m in re.finditer(r"[.!?]+[\"')\]]*\s+", text):
        prev = text[start:m.start()].split()
        last = prev[-1].lower().rstrip(".") if prev else ""
        nxt = text[m.end():m.end() + 1]
        if (last in _ABBREV or (len(last) == 1 and last.isalpha() and text[m.start()] == ".")) or not (nxt.isupper() or nxt in "\"'([" or nxt.isdigit()):
            continue
        out.append(text[start:m.end()].strip())
        start = m.end()
    if text[start:].strip():
        out.append(text[start:].strip())
    return out


def count_syllables(word: str) -> int:
    w = re.sub(r"[^a-z]", "", word.lower())
    if not w:
        return 0
    if len(w) <= 3:
        return 1
    if not w.endswith(("le", "les")):                                        # silent endings: -e, -es, -ed (but -ted / -ded are voiced)
        w = re.sub(r"(?:[^laeiouy]es|[^laeiouytd]ed|[^laeiouy]e)$", lambda m: m.group(0)[0], w)
    w = re.sub(r"^y", "", w)
    return max(1, len(re.findall(r"[aeiouy]+", w)))


# ================================================================================================ statistics / readability
def text_statistics(text: str) -> dict:
    ws, ss = words(text), sentences(text)
    syl = [count_syllables(w) for w in ws]
    freq = Counter(ws)
    return {"characters": len(text), "letters": sum(c.isalpha() for c in text), "words": len(ws), "sentences": len(ss), "syllables": sum(syl), "unique_words": len(freq),
            "avg_word_length": sum(map(len, ws)) / max(len(ws), 1), "avg_sentence_length": len(ws) / max(len(ss), 1), "complex_words": sum(s >= 3 for s in syl),
            "hapax_legomena": sum(1 for c in freq.values() if c == 1), "stopword_ratio": sum(w in STOPWORDS for w in ws) / max(len(ws), 1)}


def readability(text: str) -> dict:
    s = text_statistics(text)
    w, se, sy = max(s["words"], 1), max(s["sentences"], 1), s["syllables"]
    L, S = s["letters"] / w * 100, se / w * 100
    return {"flesch_reading_ease": 206.835 - 1.015 * w / se - 84.6 * sy / w, "flesch_kincaid_grade": 0.39 * w / se + 11.8 * sy / w - 15.59,
            "gunning_fog": 0.4 * (w / se + 100 * s["complex_words"] / w), "smog": 1.043 * math.sqrt(s["complex_words"] * 30 / se) + 3.1291,
            "coleman_liau": 0.0588 * L - 0.296 * S - 15.8, "automated_readability": 4.71 * s["letters"] / w + 0.5 * w / se - 21.43}


def lexical_diversity(tokens: Sequence[str], window: int = 50, mtld_threshold: float = 0.72) -> dict:
    n, types = len(tokens), len(set(tokens))
    def mtld_pass(seq):
        factors, seen, count = 0.0, set(), 0
        for t in seq:
            seen.add(t); count += 1
            if len(seen) / count <= mtld_threshold:
                factors, seen, count = factors + 1, set(), 0
        if count:
            factors += (1 - len(seen) / count) / (1 - mtld_threshold)
        return len(seq) / factors if factors else float(len(seq))
    mattr = sum(len(set(tokens[i:i + window])) / window for i in range(n - window + 1)) / (n - window + 1) if n >= window else types / max(n, 1)
    freq = Counter(Counter(tokens).values())
    yule = 1e4 * (sum(m * m * v for m, v in freq.items()) - n) / max(n * n, 1)
    return {"ttr": types / max(n, 1), "root_ttr": types / math.sqrt(max(n, 1)), "log_ttr": math.log(max(types, 1)) / math.log(max(n, 2)), "mattr": mattr,
            "mtld": (mtld_pass(list(tokens)) + mtld_pass(list(tokens)[::-1])) / 2, "yule_k": yule, "hapax_ratio": freq.get(1, 0) / max(types, 1)}


# ================================================================================================ n-gram language model
class NGramLM:
    """Order-``n`` model with ``laplace`` (add-k) or interpolated ``kneser_ney`` smoothing; ``<s>`` / ``</s>`` padding."""

    def __init__(self, n: int = 3, smoothing: str = "kneser_ney", k: float = 1.0, discount: float = 0.75):
        self.n, self.smoothing, self.k, self.d = n, smoothing, k, discount
        self.counts = [Counter() for _ in range(n + 1)]
        self.followers: list[dict] = [defaultdict(set) for _ in range(n + 1)]
        self.preceders: dict = defaultdict(set)
        self.cont_ctx: dict = defaultdict(set)
        self.vocab: set = set()

    def _pad(self, toks): return ["<s>"] * (self.n - 1) + list(toks) + ["</s>"]

    def fit(self, corpus: Iterable[Sequence[str]]):
        for sent in corpus:
            seq = self._pad(sent)
            self.vocab.update(seq)
            for order in range(1, self.n + 1):
                for i in range(len(seq) - order + 1):
                    g = tuple(seq[i:i + order])
                    self.counts[order][g] += 1
                    self.followers[order][g[:-1]].add(g[-1])
            for a, b in zip(seq, seq[1:]):
                self.preceders[b].add(a)
        self.total_bigram_types = sum(len(v) for v in self.preceders.values())
        self.ctx_totals = [Counter() for _ in range(self.n + 1)]
        for order in range(1, self.n + 1):
            for g, c in self.counts[order].items():
                self.ctx_totals[order][g[:-1]] += c
        return self

    def prob(self, word: str, context: Sequence[str] = ()) -> float:
        ctx = tuple((["<s>"] * self.n + list(context))[-(self.n - 1):]) if self.n > 1 else ()
        if self.smoothing == "laplace":
            return (self.counts[self.n][ctx + (word,)] + self.k) / (self.ctx_totals[self.n][ctx] + self.k * len(self.vocab))
        return self._kn(word, ctx)

    def _kn(self, word, ctx):
        if not ctx:
            eps = 0.1                                                         # continuation probability; eps keeps unseen words above zero
            return (len(self.preceders.get(word, ())) + eps) / (self.total_bigram_types + eps * (len(self.vocab) + 1))
        order = len(ctx) + 1
        total = self.ctx_totals[order][ctx]
        lower = self._kn(word, ctx[1:])
        if total == 0:
            return lower
        lam = self.d * len(self.followers[order][ctx]) / total
        return max(self.counts[order][ctx + (word,)] - self.d, 0) / total + lam * lower

    def log_prob(self, sent: Sequence[str]) -> float:
        seq = self._pad(sent)
        return sum(math.log(self.prob(seq[i], seq[max(0, i - self.n + 1):i])) for i in range(self.n - 1, len(seq)))

    def perplexity(self, corpus) -> float:
        lp, n = 0.0, 0
        for s in corpus:
            lp += self.log_prob(s); n += len(s) + 1
        return math.exp(-lp / max(n, 1))

    def generate(self, max_len: int = 20, seed: int = 0) -> list[str]:
        g, ctx, out = torch.Generator().manual_seed(seed), ["<s>"] * (self.n - 1), []
        vocab = sorted(self.vocab - {"<s>"})
        for _ in range(max_len):
            p = torch.tensor([self.prob(w, ctx) for w in vocab])
            w = vocab[int(torch.multinomial(p / p.sum(), 1, generator=g))]
            if w == "</s>":
                break
            out.append(w); ctx = (ctx + [w])[-(self.n - 1):] if self.n > 1 else []
        return out


# ================================================================================================ retrieval / similarity
class TfidfVectorizer:
    """Smoothed idf ``ln((1 + N) / (1 + df)) + 1``, optional sub-linear tf, L2-normalised rows (the common defaults)."""

    def __init__(self, ngram_range=(1, 1), min_df: int = 1, sublinear_tf: bool = False, stop_words=None):
        self.ngrams, self.min_df, self.sub, self.stop = ngram_range, min_df, sublinear_tf, set(stop_words or ())

    def _terms(self, doc):
        ws = [w for w in (words(doc) if isinstance(doc, str) else list(doc)) if w not in self.stop]
        return [" ".join(ws[i:i + n]) for n in range(self.ngrams[0], self.ngrams[1] + 1) for i in range(len(ws) - n + 1)]

    def fit(self, docs):
        df = Counter(t for d in docs for t in set(self._terms(d)))
        self.vocabulary = {t: i for i, t in enumerate(sorted(t for t, c in df.items() if c >= self.min_df))}
        n = len(docs)
        self.idf = torch.tensor([math.log((1 + n) / (1 + df[t])) + 1 for t in self.vocabulary], dtype=torch.float64)
        return self

    def transform(self, docs) -> torch.Tensor:
        m = torch.zeros(len(docs), len(self.vocabulary), dtype=torch.float64)
        for r, d in enumerate(docs):
            for t, c in Counter(self._terms(d)).items():
                if t in self.vocabulary:
                    m[r, self.vocabulary[t]] = 1 + math.log(c) if self.sub else c
        m = m * self.idf
        return m / m.norm(dim=1, keepdim=True).clamp(min=1e-12)

    def fit_transform(self, docs): return self.fit(docs).transform(docs)


class BM25:
    def __init__(self, docs, k1: float = 1.5, b: float = 0.75):
        self.docs = [words(d) if isinstance(d, str) else list(d) for d in docs]
        self.k1, self.b, self.tf = k1, b, [Counter(d) for d in self.docs]
        self.avgdl = sum(map(len, self.docs)) / max(len(self.docs), 1)
        df = Counter(t for d in self.docs for t in set(d))
        n = len(self.docs)
        self.idf = {t: math.log((n - c + 0.5) / (c + 0.5) + 1) for t, c in df.items()}

    def scores(self, query) -> list[float]:
        q = words(query) if isinstance(query, str) else list(query)
        return [sum(self.idf.get(t, 0.0) * tf[t] * (self.k1 + 1) / (tf[t] + self.k1 * (1 - self.b + self.b * len(d) / self.avgdl)) for t in q if t in tf) for d, tf in zip(self.docs, self.tf)]

    def top_k(self, query, k: int = 3): s = self.scores(query); return sorted(range(len(s)), key=lambda i: -s[i])[:k]


def jaccard_similarity(a, b): a, b = set(a), set(b); return len(a & b) / len(a | b) if a | b else 1.0
def dice_similarity(a, b): a, b = set(a), set(b); return 2 * len(a & b) / (len(a) + len(b)) if a or b else 1.0
def cosine_similarity_counts(a, b): ca, cb = Counter(a), Counter(b); num = sum(ca[t] * cb[t] for t in ca); den = math.sqrt(sum(v * v for v in ca.values()) * sum(v * v for v in cb.values())); return num / den if den else 0.0


def jaro_winkler(a: str, b: str, p: float = 0.1) -> float:
    if a == b:
        return 1.0
    la, lb = len(a), len(b)
    if not la or not lb:
        return 0.0
    rng = max(la, lb) // 2 - 1
    ma, mb = [False] * la, [False] * lb
    m = 0
    for i in range(la):
        for j in range(max(0, i - rng), min(lb, i + rng + 1)):
            if not mb[j] and a[i] == b[j]:
                ma[i] = mb[j] = True; m += 1
                break
    if not m:
        return 0.0
    sa, sb = [a[i] for i in range(la) if ma[i]], [b[j] for j in range(lb) if mb[j]]
    t = sum(x != y for x, y in zip(sa, sb)) / 2
    jaro = (m / la + m / lb + (m - t) / m) / 3
    pre = 0
    for x, y in zip(a[:4], b[:4]):
        if x != y:
            break
        pre += 1
    return jaro + pre * p * (1 - jaro)


def minhash_signature(tokens, num_perm: int = 64, seed: int = 1) -> list[int]:
    """Estimates Jaccard similarity: the share of equal positions in two signatures."""
    import hashlib
    prime = (1 << 61) - 1
    g = torch.Generator().manual_seed(seed)
    a = torch.randint(1, 1 << 31, (num_perm,), generator=g).tolist()
    b = torch.randint(0, 1 << 31, (num_perm,), generator=g).tolist()
    hs = [int(hashlib.md5(str(t).encode()).hexdigest()[:15], 16) for t in set(tokens)]
    return [min((ai * h + bi) % prime for h in hs) if hs else prime for ai, bi in zip(a, b)]


# ================================================================================================ keywords / summaries
def rake_keywords(text: str, top: int = 10, stop_words=STOPWORDS) -> list[tuple[str, float]]:
    """Candidate phrases are the runs of non-stop-words between stop words and punctuation; a word scores
    ``degree / frequency`` and a phrase the sum of its words."""
    phrases = []
    for chunk in re.split(r"[.,;:!?()\[\]\"\n]", text.lower()):
        cur = []
        for w in _WORD.findall(chunk):
            if w in stop_words:
                if cur:
                    phrases.append(cur); cur = []
            else:
                cur.append(w)
        if cur:
            phrases.append(cur)
    freq, degree = Counter(), Counter()
    for p in phrases:
        for w in p:
            freq[w] += 1; degree[w] += len(p)
    scores = {" ".join(p): sum(degree[w] / freq[w] for w in p) for p in phrases}
    return sorted(scores.items(), key=lambda kv: (-kv[1], kv[0]))[:top]


def _pagerank(weights: torch.Tensor, damping=0.85, iters=100) -> torch.Tensor:
    n = len(weights)
    out = weights.sum(1, keepdim=True)
    p = torch.where(out > 0, weights / out.clamp(min=1e-12), torch.full_like(weights, 1.0 / n))
    r = torch.full((n,), 1.0 / n, dtype=weights.dtype)
    for _ in range(iters):
        r = (1 - damping) / n + damping * (p.t() @ r)
    return r


def textrank_keywords(text: str, top: int = 10, window: int = 4) -> list[tuple[str, float]]:
    ws = [w for w in words(text) if w not in STOPWORDS and len(w) > 2]
    vocab = sorted(set(ws))
    idx = {w: i for i, w in enumerate(vocab)}
    m = torch.zeros(len(vocab), len(vocab), dtype=torch.float64)
    for i, w in enumerate(ws):
        for u in ws[i + 1:i + window]:
            if u != w:
                m[idx[w], idx[u]] += 1; m[idx[u], idx[w]] += 1
    r = _pagerank(m)
    return sorted(zip(vocab, r.tolist()), key=lambda kv: (-kv[1], kv[0]))[:top]


def summarize(text: str, num_sentences: int = 3, method: str = "textrank") -> list[str]:
    """Extractive summary in document order: ``textrank`` over TF-IDF sentence similarity, or ``frequency`` (mean
    normalised word frequency of each sentence)."""
    ss = sentences(text)
    if len(ss) <= num_sentences:
        return ss
    if method == "frequency":
        freq = Counter(w for w in words(text) if w not in STOPWORDS)
        top = max(freq.values(), default=1)
        score = [sum(freq[w] / top for w in words(s) if w in freq) / max(len(words(s)), 1) for s in ss]
    else:
        v = TfidfVectorizer(stop_words=STOPWORDS).fit_transform(ss)
        sim = v @ v.t()
        sim.fill_diagonal_(0)
        score = _pagerank(sim).tolist()
    keep = sorted(sorted(range(len(ss)), key=lambda i: -score[i])[:num_sentences])
    return [ss[i] for i in keep]


# ================================================================================================ sentiment / language / entities / cohesion
_POS = set("good great excellent amazing wonderful love loved like liked best happy positive fantastic awesome nice enjoy enjoyed perfect brilliant superb pleasant recommend".split())
_NEG = set("bad terrible awful horrible hate hated worst sad negative poor boring disappointing disappointed broken useless slow ugly fail failed failure annoying waste".split())
_NEGATORS, _BOOST, _DAMP = {"not", "no", "never", "n't", "cannot", "without", "hardly"}, {"very": 1.5, "extremely": 2.0, "really": 1.4, "so": 1.3, "absolutely": 1.8}, {"slightly": 0.5, "somewhat": 0.6, "barely": 0.4}


def sentiment(text: str, positive=_POS, negative=_NEG) -> dict:
    """Lexicon score in ``[-1, 1]``: intensifiers scale the next sentiment word, a negator within three words flips it."""
    toks = re.findall(r"n't|[a-z]+", text.lower().replace("n't", " n't"))
    total, hits = 0.0, 0
    for i, w in enumerate(toks):
        pol = 1.0 if w in positive else -1.0 if w in negative else 0.0
        if pol == 0.0:
            continue
        prev = toks[max(0, i - 3):i]
        scale = 1.0
        for p in prev[-1:]:
            scale *= _BOOST.get(p, 1.0) * _DAMP.get(p, 1.0)
        if any(p in _NEGATORS for p in prev):
            pol = -pol
        total += pol * scale; hits += 1
    score = total / math.sqrt(total * total + 4) if hits else 0.0
    return {"score": score, "label": "positive" if score > 0.1 else "negative" if score < -0.1 else "neutral", "matches": hits}


class LanguageIdentifier:
    """Cavnar-Trenkle: rank-order profiles of the most frequent character 1-3-grams; the language with the smallest
    out-of-place distance wins."""

    def __init__(self, profile_size: int = 300): self.size, self.profiles = profile_size, {}

    def _profile(self, text):
        t = " " + re.sub(r"[^\w\s]|\d", "", text.lower()) + " "
        c = Counter(t[i:i + n] for n in (1, 2, 3) for i in range(len(t) - n + 1) if t[i:i + n].strip())
        return [g for g, _ in sorted(c.items(), key=lambda kv: (-kv[1], kv[0]))[:self.size]]

    def fit(self, samples: dict[str, str]):
        self.profiles = {lang: {g: r for r, g in enumerate(self._profile(txt))} for lang, txt in samples.items()}
        return self

    def distances(self, text) -> dict[str, int]:
        prof = self._profile(text)
        return {lang: sum(abs(r - ranks[g]) if g in ranks else self.size for r, g in enumerate(prof)) for lang, ranks in self.profiles.items()}

    def predict(self, text) -> str: d = self.distances(text); return min(d, key=d.get)


_PATTERNS = {"email": r"[\w.+-]+@[\w-]+(?:\.[\w-]+)+", "url": r"https?://[^\s<>\"]+", "date": r"\b\d{4}-\d{2}-\d{2}\b|\b\d{1,2}/\d{1,2}/\d{2,4}\b",
             "time": r"\b\d{1,2}:\d{2}(?::\d{2})?\s?(?:[AaPp][Mm])?\b", "money": r"[$€£]\s?\d[\d,]*(?:\.\d+)?|\b\d[\d,]*(?:\.\d+)?\s?(?:USD|EUR|dollars|euros)\b",
             "percent": r"\b\d+(?:\.\d+)?\s?%", "phone": r"\+?\d{1,3}[\s-]?\(?\d{2,4}\)?[\s-]?\d{3,4}[\s-]?\d{3,4}\b", "hashtag": r"#\w+", "mention": r"@\w+"}


def extract_entities(text: str, kinds: Sequence[str] | None = None) -> list[dict]:
    """Pattern entities plus capitalised multi-word names (``name``) that do not start a sentence alone; spans never overlap
    (earlier pattern kinds win)."""
    out, taken = [], []
    def free(s, e): return all(e <= a or s >= b for a, b in taken)
    for kind in kinds or list(_PATTERNS):
        for m in re.finditer(_PATTERNS[kind], text):
            if free(*m.span()):
                out.append({"type": kind, "text": m.group(0), "start": m.start(), "end": m.end()}); taken.append(m.span())
    if kinds is None or "name" in kinds:
        for m in re.finditer(r"\b[A-Z][a-z]+(?:\s+(?:of|de|van|von)\s+[A-Z][a-z]+|\s+[A-Z][a-z]+)+\b", text):
            s0, e0 = m.span()
            at_start = s0 == 0 or re.search(r"[.!?]\s+$", text[:s0]) is not None
            if at_start and len(m.group(0).split()) >= 3:                      # a capitalised sentence opener in front of a name
                s0 += len(m.group(0).split()[0]) + 1
            if free(s0, e0):
                out.append({"type": "name", "text": text[s0:e0], "start": s0, "end": e0}); taken.append((s0, e0))
    return sorted(out, key=lambda d: d["start"])


def lexical_cohesion(text: str) -> dict:
    """Overlap of content words between adjacent sentences (local) and between every pair (global), plus the positions
    where local overlap drops to zero (candidate topic boundaries)."""
    ss = [set(w for w in words(s) if w not in STOPWORDS) for s in sentences(text)]
    local = [jaccard_similarity(a, b) for a, b in zip(ss, ss[1:])]
    pairs = [jaccard_similarity(ss[i], ss[j]) for i in range(len(ss)) for j in range(i + 1, len(ss))]
    return {"local": sum(local) / max(len(local), 1), "global": sum(pairs) / max(len(pairs), 1), "breaks": [i + 1 for i, v in enumerate(local) if v == 0], "per_transition": local}


# ================================================================================================ task models
class BiLSTMTextClassifier(nn.Module):
    """Embedding -> bidirectional LSTM -> masked max and mean pooling -> linear head; padding id 0."""

    def __init__(self, vocab: int, classes: int, dim: int = 64, hidden: int = 64, layers: int = 1, dropout: float = 0.0):
        super().__init__()
        self.emb, self.rnn = nn.Embedding(vocab, dim, padding_idx=0), nn.LSTM(dim, hidden, layers, batch_first=True, bidirectional=True, dropout=dropout if layers > 1 else 0.0)
        self.head = nn.Linear(4 * hidden, classes)

    def forward(self, ids):
        mask = (ids != 0)[..., None]
        lengths = mask.squeeze(-1).sum(1).clamp(min=1).cpu()                  # packed, so the backward direction starts at the last real token
        packed = nn.utils.rnn.pack_padded_sequence(self.emb(ids), lengths, batch_first=True, enforce_sorted=False)
        h = nn.utils.rnn.pad_packed_sequence(self.rnn(packed)[0], batch_first=True, total_length=ids.shape[1])[0]
        mx = h.masked_fill(~mask, -1e9).amax(1)
        mean = (h * mask).sum(1) / mask.sum(1).clamp(min=1)
        return self.head(torch.cat([mx, mean], -1))


class TextCNN(nn.Module):
    """Parallel convolutions of several widths over the embedded sequence, max over time, linear head (Kim 2014)."""

    def __init__(self, vocab: int, classes: int, dim: int = 64, widths=(2, 3, 4), channels: int = 32):
        super().__init__()
        self.emb = nn.Embedding(vocab, dim, padding_idx=0)
        self.convs, self.head = nn.ModuleList(nn.Conv1d(dim, channels, w, padding=w - 1) for w in widths), nn.Linear(channels * len(widths), classes)

    def forward(self, ids):
        x = self.emb(ids).transpose(1, 2)
        return self.head(torch.cat([torch.relu(c(x)).amax(-1) for c in self.convs], -1))


class TransformerTextClassifier(nn.Module):
    def __init__(self, vocab: int, classes: int, dim: int = 64, heads: int = 4, layers: int = 2, max_len: int = 256):
        super().__init__()
        self.emb, self.pos = nn.Embedding(vocab, dim, padding_idx=0), nn.Parameter(0.02 * torch.randn(max_len, dim))
        self.enc = nn.TransformerEncoder(nn.TransformerEncoderLayer(dim, heads, 2 * dim, dropout=0.0, batch_first=True), layers, enable_nested_tensor=False)
        self.head = nn.Linear(dim, classes)

    def forward(self, ids):
        pad = ids == 0
        h = self.enc(self.emb(ids) + self.pos[:ids.shape[1]], src_key_padding_mask=pad)
        keep = (~pad)[..., None]
        return self.head((h * keep).sum(1) / keep.sum(1).clamp(min=1))


class SequenceTagger(nn.Module):
    """BiLSTM emissions with a linear-chain CRF: ``loss`` is the negative log-likelihood, ``decode`` runs Viterbi."""

    def __init__(self, vocab: int, tags: int, dim: int = 32, hidden: int = 32):
        super().__init__()
        self.emb, self.rnn, self.out = nn.Embedding(vocab, dim, padding_idx=0), nn.LSTM(dim, hidden, batch_first=True, bidirectional=True), nn.Linear(2 * hidden, tags)
        self.trans, self.start, self.end = nn.Parameter(torch.zeros(tags, tags)), nn.Parameter(torch.zeros(tags)), nn.Parameter(torch.zeros(tags))

    def emissions(self, ids): return self.out(self.rnn(self.emb(ids))[0])

    def loss(self, ids, tags):
        em, mask = self.emissions(ids), ids != 0
        b, t, k = em.shape
        score = self.start[tags[:, 0]] + em[:, 0].gather(1, tags[:, :1]).squeeze(1)
        alpha = self.start[None] + em[:, 0]
        for i in range(1, t):
            m = mask[:, i]
            step = self.trans[tags[:, i - 1], tags[:, i]] + em[:, i].gather(1, tags[:, i:i + 1]).squeeze(1)
            score = score + step * m
            nxt = torch.logsumexp(alpha[:, :, None] + self.trans[None], 1) + em[:, i]
            alpha = torch.where(m[:, None], nxt, alpha)
        last = tags.gather(1, (mask.sum(1) - 1).clamp(min=0)[:, None]).squeeze(1)
        return (torch.logsumexp(alpha + self.end[None], 1) - (score + self.end[last])).mean()

    @torch.no_grad()
    def decode(self, ids) -> list[list[int]]:
        em, mask = self.emissions(ids), ids != 0
        out = []
        for e, m in zip(em, mask):
            n = int(m.sum())
            v, back = self.start + e[0], []
            for i in range(1, n):
                s = v[:, None] + self.trans
                back.append(s.argmax(0))
                v = s.amax(0) + e[i]
            best = [int((v + self.end).argmax())]
            for bp in reversed(back):
                best.append(int(bp[best[-1]]))
            out.append(best[::-1])
        return out
