"""Text generation: sampling strategies, repetition controls, beam search with length penalty, and a generator loop over
any ``step_fn(ids [N, T]) -> logits [N, V]`` (the next-token logits of the last position).

Follows the reference's generation module (crates/torsh-text/src/generation.rs: GenerationConfig, TextSampler,
BeamHypothesis / BeamSearchDecoder, RepetitionPenalty, NGramRepetitionFilter, TextGenerator).
"""
from __future__ import annotations

from dataclasses import dataclass

import torch

from . import top_k_top_p_filter


@dataclass
class GenerationConfig:
    max_length: int = 50
    min_length: int = 0
    do_sample: bool = False
    temperature: float = 1.0
    top_k: int = 0
    top_p: float = 1.0
    num_beams: int = 1
    length_penalty: float = 1.0
    repetition_penalty: float = 1.0
    no_repeat_ngram_size: int = 0
    eos_token_id: int | None = None
    pad_token_id: int | None = None
    early_stopping: bool = True
    seed: int | None = None


class TextSampler:
    """Draws one token id from a vector of logits."""

    def __init__(self, seed: int | None = None):
        self.gen = torch.Generator()
        if seed is not None:
            self.gen.manual_seed(seed)

    def _draw(self, logits: torch.Tensor) -> int:
        p = torch.softmax(logits.float().cpu(), -1)
        return int(torch.multinomial(p, 1, generator=self.gen))

    def greedy_sample(self, logits: torch.Tensor) -> int:
        return int(logits.argmax(-1))

    def temperature_sample(self, logits: torch.Tensor, temperature: float) -> int:
        if temperature <= 0:
            raise ValueError("temperature must be positive")
        return self._draw(logits / temperature)

    def top_k_sample(self, logits: torch.Tensor, k: int, temperature: float = 1.0) -> int:
        return self._draw(top_k_top_p_filter(logits / temperature, top_k=k))

    def top_p_sample(self, logits: torch.Tensor, p: float, temperature: float = 1.0) -> int:
        return self._draw(top_k_top_p_filter(logits / temperature, top_p=p))

    def top_k_top_p_sample(self, logits: torch.Tensor, k: int, p: float, temperature: float = 1.0) -> int:
        return self._draw(top_k_top_p_filter(logits / temperature, top_k=k, top_p=p))


class RepetitionPenalty:
    @staticmethod
    def apply(logits: torch.Tensor, generated_tokens, penalty: float) -> torch.Tensor:
        """Divides positive logits of already generated tokens by ``penalty`` and multiplies negative ones (CTRL rule)."""
        if penalty == 1.0 or len(generated_tokens) == 0:
            return logits
        out = logits.clone()
        idx = torch.as_tensor(sorted(set(int(t) for t in generated_tokens)), device=logits.device)
        v = out[..., idx]
        out[..., idx] = torch.where(v > 0, v / penalty, v * penalty)
        return out


class NGramRepetitionFilter:
    """Bans every token that would complete an n-gram already present in the generated sequence."""

    def __init__(self, no_repeat_ngram_size: int):
        self.n = no_repeat_ngram_size

    def banned(self, generated_tokens) -> set:
        n, toks = self.n, [int(t) for t in generated_tokens]
        if n <= 0 or len(toks) < n - 1:
            return set()
        prefix = tuple(toks[len(toks) - (n - 1):]) if n > 1 else ()
        return {toks[i + n - 1] for i in range(len(toks) - n + 1) if tuple(toks[i:i + n - 1]) == prefix}

    def filter_logits(self, logits: torch.Tensor, generated_tokens) -> torch.Tensor:
        ban = self.banned(generated_tokens)
        if not ban:
            return logits
        out = logits.clone()
        out[..., torch.as_tensor(sorted(ban), device=logits.device)] = float("-inf")
        return out


@dataclass
class BeamHypothesis:
    tokens: list
    score: float                       # sum of token log-probabilities
    finished: bool = False

    def normalized_score(self, length_penalty: float) -> float:
        return self.score / (max(len(self.tokens), 1) ** length_penalty)


class BeamSearchDecoder:
    def __init__(self, num_beams: int = 4, max_length: int = 50, length_penalty: float = 1.0, eos_token_id: int | None = None,
                 early_stopping: bool = True, no_repeat_ngram_size: int = 0):
        self.num_beams, self.max_length, self.length_penalty = num_beams, max_length, length_penalty
        self.eos, self.early_stopping = eos_token_id, early_stopping
        self.ngram = NGramRepetitionFilter(no_repeat_ngram_size)

    @torch.no_grad()
    def search(self, step_fn, start_ids) -> list[BeamHypothesis]:
        """Returns the final hypotheses, best first (by length-normalised score)."""
        start = [int(t) for t in torch.as_tensor(start_ids).reshape(-1)]
        device = start_ids.device if isinstance(start_ids, torch.Tensor) else "cpu"
        beams = [BeamHypothesis(list(start), 0.0)]
        done: list[BeamHypothesis] = []
        while beams and len(beams[0].tokens) < self.max_length:
            ids = torch.tensor([b.tokens for b in beams], device=device)
            logp = torch.log_softmax(step_fn(ids).float(), -1)
            cand = []
            for bi, b in enumerate(beams):
                lp = self.ngram.filter_logits(logp[bi], b.tokens[len(start):])
                v, i = lp.topk(min(self.num_beams, lp.shape[-1]))
                for vv, ii in zip(v.tolist(), i.tolist()):
                    if vv == float("-inf"):
                        continue
                    cand.append(BeamHypothesis(b.tokens + [ii], b.score + vv, self.eos is not None and ii == self.eos))
            cand.sort(key=lambda h: -h.normalized_score(self.length_penalty))
            beams = []
            for h in cand:
                (done if h.finished else beams).append(h)
                if len(beams) == self.num_beams:
                    break
            if self.early_stopping and len(done) >= self.num_beams:
                best_open = max((b.normalized_score(self.length_penalty) for b in beams), default=float("-inf"))
                if sorted(h.normalized_score(self.length_penalty) for h in done)[-self.num_beams] >= best_open:
                    break
        return sorted(done + beams, key=lambda h: -h.normalized_score(self.length_penalty))


class TextGenerator:
    def __init__(self, config: GenerationConfig | None = None):
        self.cfg = config or GenerationConfig()
        self.sampler = TextSampler(self.cfg.seed)
        self.ngram = NGramRepetitionFilter(self.cfg.no_repeat_ngram_size)

    @torch.no_grad()
    def generate(self, step_fn, prompt_ids) -> list[int]:
        """Token ids of prompt + continuation (stops at ``eos_token_id`` or ``max_length`` total tokens)."""
        c = self.cfg
        prompt = torch.as_tensor(prompt_ids).reshape(-1)
        if c.num_beams > 1:
            dec = BeamSearchDecoder(c.num_beams, c.max_length, c.length_penalty, c.eos_token_id, c.early_stopping, c.no_repeat_ngram_size)
            return dec.search(step_fn, prompt)[0].tokens
        toks = [int(t) for t in prompt]
        n0 = len(toks)
        while len(toks) < c.max_length:
            logits = step_fn(torch.tensor([toks], device=prompt.device))[0].float()
            gen = toks[n0:]
            logits = RepetitionPenalty.apply(logits, gen, c.repetition_penalty)
            logits = self.ngram.filter_logits(logits, gen)
            if c.eos_token_id is not None and len(gen) < c.min_length:
                logits = logits.clone()
                logits[c.eos_token_id] = float("-inf")
            if c.do_sample:
                nxt = self.sampler.top_k_top_p_sample(logits, c.top_k, c.top_p, c.temperature)
            else:
                nxt = self.sampler.greedy_sample(logits)
            toks.append(nxt)
            if c.eos_token_id is not None and nxt == c.eos_token_id:
                break
        return toks
