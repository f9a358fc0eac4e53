"""Speech encoders: Wav2Vec2 / HuBERT / WavLM-style (convolutional feature extractor on the raw waveform + transformer
encoder) and the Whisper encoder (two convolutions on a log-mel spectrogram + sinusoidal positions + pre-norm blocks).

Reference inventory: ``crates/torsh-models/src/lib.rs:9-38`` lists ``audio`` (wav2vec2, whisper, hubert, wavlm) among
the model families. The transformer blocks are the shared :class:`EncoderBlock` (fused QKV GEMM, flash attention
without a mask, fused MLP on the tcgen05 GEMM when the tensors are bf16 on a GPU).
"""
from __future__ import annotations

import math
from dataclasses import dataclass, field

import torch

from .. import nn
from .transformer_zoo import EncoderBlock, EncoderConfig


# ------------------------------------------------------------------------------------------------ wav2vec2
@dataclass
class Wav2Vec2Config(EncoderConfig):
    conv_dim: tuple = (512, 512, 512, 512, 512, 512, 512)
    conv_kernel: tuple = (10, 3, 3, 3, 3, 2, 2)
    conv_stride: tuple = (5, 2, 2, 2, 2, 2, 2)
    conv_bias: bool = False
    num_conv_pos_embeddings: int = 128
    num_conv_pos_embedding_groups: int = 16
    layer_norm_eps: float = 1e-5
    pre_norm: bool = False             # "stable layer norm" variants (large models, HuBERT-large, WavLM-large) use True
    vocab_size: int = 32               # CTC head

    @classmethod
    def base(cls, **kw): return cls(**kw)
    @classmethod
    def large(cls, **kw): return cls(hidden_size=1024, num_layers=24, num_heads=16, intermediate_size=4096, pre_norm=True, conv_bias=True, **kw)
    @classmethod
    def tiny(cls, **kw):
        d = dict(hidden_size=64, num_layers=2, num_heads=4, intermediate_size=128, conv_dim=(32, 32, 32), conv_kernel=(10, 3, 2),
                 conv_stride=(5, 2, 2), num_conv_pos_embeddings=16, num_conv_pos_embedding_groups=4, dropout=0.0)
        d.update(kw)
        return cls(**d)


class Wav2Vec2FeatureExtractor(nn.Module):
    """Strided 1-D convolutions over the waveform; the first layer is followed by a per-channel GroupNorm ("group" norm
    variant, base models) or every layer by a LayerNorm over channels ("layer" variant, large models)."""

    def __init__(self, cfg: Wav2Vec2Config):
        super().__init__()
        self.layer_norm_variant = cfg.pre_norm
        chans = (1,) + tuple(cfg.conv_dim)
        self.convs = nn.ModuleList([nn.Conv1d(chans[i], chans[i + 1], cfg.conv_kernel[i], cfg.conv_stride[i], bias=cfg.conv_bias)
                                    for i in range(len(cfg.conv_dim))])
        if self.layer_norm_variant:
            self.norms = nn.ModuleList([nn.LayerNorm(c, 1e-5) for c in cfg.conv_dim])
        else:
            self.norms = nn.ModuleList([nn.GroupNorm(cfg.conv_dim[0], cfg.conv_dim[0], 1e-5)])

    def forward(self, wav: torch.Tensor) -> torch.Tensor:
        x = wav[:, None, :]
        for i, conv in enumerate(self.convs):
            x = conv(x)
            if self.layer_norm_variant:
                x = self.norms[i](x.transpose(1, 2)).transpose(1, 2)
            elif i == 0:
                x = self.norms[0](x)
            x = torch.nn.functional.gelu(x)
        return x.transpose(1, 2)               # [B, frames, C]


class Wav2Vec2Model(nn.Module):
    def __init__(self, cfg: Wav2Vec2Config | None = None):
        super().__init__()
        cfg = cfg or Wav2Vec2Config()
        self.config = cfg
        E = cfg.hidden_size
        self.feature_extractor = Wav2Vec2FeatureExtractor(cfg)
        self.feat_norm = nn.LayerNorm(cfg.conv_dim[-1], cfg.layer_norm_eps)
        self.feat_proj = nn.Linear(cfg.conv_dim[-1], E)
        k = cfg.num_conv_pos_embeddings
        self.pos_conv = nn.Conv1d(E, E, k, padding=k // 2, groups=cfg.num_conv_pos_embedding_groups)
        self.enc_norm = nn.LayerNorm(E, cfg.layer_norm_eps)
        self.layers = nn.ModuleList([EncoderBlock(cfg) for _ in range(cfg.num_layers)])
        self.drop = nn.Dropout(cfg.dropout)

    def frames(self, samples: int) -> int:
        for k, s in zip(self.config.conv_kernel, self.config.conv_stride):
            samples = (samples - k) // s + 1
        return samples

    def forward(self, wav: torch.Tensor) -> torch.Tensor:
        """``wav``: ``[B, samples]`` (normalised waveform) → hidden states ``[B, frames, E]``."""
        x = self.feat_proj(self.feat_norm(self.feature_extractor(wav)))
        pos = self.pos_conv(x.transpose(1, 2))
        if self.config.num_conv_pos_embeddings % 2 == 0:
            pos = pos[:, :, :-1]                 # an even kernel with padding k/2 yields one frame too many
        x = x + torch.nn.functional.gelu(pos).transpose(1, 2)
        if not self.config.pre_norm:
            x = self.enc_norm(x)
        x = self.drop(x)
        for l in self.layers:
            x = l(x)
        return self.enc_norm(x) if self.config.pre_norm else x


class Wav2Vec2ForCTC(nn.Module):
    def __init__(self, cfg: Wav2Vec2Config | None = None):
        super().__init__()
        self.wav2vec2 = Wav2Vec2Model(cfg)
        self.lm_head = nn.Linear(self.wav2vec2.config.hidden_size, self.wav2vec2.config.vocab_size)

    def forward(self, wav, labels=None, label_lengths=None):
        logits = self.lm_head(self.wav2vec2(wav))
        if labels is None:
            return logits
        lp = torch.log_softmax(logits.float(), -1).transpose(0, 1)
        T = torch.full((wav.shape[0],), lp.shape[0], dtype=torch.long)
        ll = label_lengths if label_lengths is not None else torch.full((wav.shape[0],), labels.shape[1], dtype=torch.long)
        return torch.nn.functional.ctc_loss(lp, labels, T, ll, blank=0, zero_infinity=True)


HubertModel = Wav2Vec2Model     # same architecture; trained on cluster targets instead of quantised latents
WavLMModel = Wav2Vec2Model      # WavLM adds a gated relative position bias; without it the encoder is this one


# ------------------------------------------------------------------------------------------------ whisper
@dataclass
class WhisperConfig(EncoderConfig):
    num_mel_bins: int = 80
    max_source_positions: int = 1500
    vocab_size: int = 51865
    max_target_positions: int = 448
    num_decoder_layers: int = 12
    pre_norm: bool = True
    layer_norm_eps: float = 1e-5
    dropout: float = 0.0

    @classmethod
    def tiny_en(cls, **kw): return cls(hidden_size=384, num_layers=4, num_decoder_layers=4, num_heads=6, intermediate_size=1536, **kw)
    @classmethod
    def base(cls, **kw): return cls(hidden_size=512, num_layers=6, num_decoder_layers=6, num_heads=8, intermediate_size=2048, **kw)
    @classmethod
    def small(cls, **kw): return cls(**kw)
    @classmethod
    def tiny(cls, **kw):
        d = dict(hidden_size=64, num_layers=2, num_decoder_layers=2, num_heads=4, intermediate_size=128, num_mel_bins=16,
                 max_source_positions=50, vocab_size=200, max_target_positions=32)
        d.update(kw)
        return cls(**d)


def sinusoids(length: int, channels: int, max_timescale: float = 10000.0) -> torch.Tensor:
    """Whisper's fixed encoder positions: ``[sin(t * f_i) | cos(t * f_i)]`` with geometric timescales."""
    inc = math.log(max_timescale) / (channels // 2 - 1)
    inv = torch.exp(-inc * torch.arange(channels // 2))
    t = torch.arange(length)[:, None] * inv[None, :]
    return torch.cat([t.sin(), t.cos()], 1)


class WhisperEncoder(nn.Module):
    def __init__(self, cfg: WhisperConfig | None = None):
        super().__init__()
        cfg = cfg or WhisperConfig()
        self.config = cfg
        E = cfg.hidden_size
        self.conv1 = nn.Conv1d(cfg.num_mel_bins, E, 3, padding=1)
        self.conv2 = nn.Conv1d(E, E, 3, stride=2, padding=1)
        self.register_buffer("embed_positions", sinusoids(cfg.max_source_positions, E), persistent=True)
        self.layers = nn.ModuleList([EncoderBlock(cfg) for _ in range(cfg.num_layers)])
        self.ln_post = nn.LayerNorm(E, cfg.layer_norm_eps)

    def forward(self, mel: torch.Tensor) -> torch.Tensor:
        """``mel``: ``[B, n_mels, 2 * max_source_positions]`` log-mel spectrogram → ``[B, max_source_positions, E]``."""
        x = torch.nn.functional.gelu(self.conv1(mel))
        x = torch.nn.functional.gelu(self.conv2(x)).transpose(1, 2)
        x = x + self.embed_positions[: x.shape[1]].to(x.dtype)
        for l in self.layers:
            x = l(x)
        return self.ln_post(x)


class WhisperModel(nn.Module):
    """Encoder + causal decoder with cross-attention and a tied output embedding."""

    def __init__(self, cfg: WhisperConfig | None = None):
        super().__init__()
        cfg = cfg or WhisperConfig()
        self.config = cfg
        E = cfg.hidden_size
        self.encoder = WhisperEncoder(cfg)
        self.embed_tokens = nn.Embedding(cfg.vocab_size, E)
        self.embed_positions = nn.Embedding(cfg.max_target_positions, E)
        self.decoder = nn.ModuleList([EncoderBlock(cfg, cross_attention=True, causal=True) for _ in range(cfg.num_decoder_layers)])
        self.ln_dec = nn.LayerNorm(E, cfg.layer_norm_eps)

    def forward(self, mel, decoder_input_ids, labels=None):
        mem = self.encoder(mel)
        y = self.embed_tokens(decoder_input_ids) + self.embed_positions(torch.arange(decoder_input_ids.shape[1], device=mel.device))[None]
        for l in self.decoder:
            y = l(y, memory=mem)
        logits = torch.nn.functional.linear(self.ln_dec(y), self.embed_tokens.weight)
        if labels is None:
            return logits
        return torch.nn.functional.cross_entropy(logits.view(-1, logits.shape[-1]).float(), labels.view(-1), ignore_index=-100)
