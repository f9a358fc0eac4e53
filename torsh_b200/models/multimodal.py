"""Contrastive image-text models: CLIP (ViT image tower + causal text transformer, projections into a shared space,
learned temperature) and ALIGN-style dual encoders built from the same parts.

Reference inventory: ``crates/torsh-models/src/lib.rs:9-38`` (``multimodal``: CLIP, ALIGN). Both towers are stacks of the
shared pre-norm :class:`EncoderBlock`.
"""
from __future__ import annotations

import math
from dataclasses import dataclass, field

import torch

from .. import nn
from .transformer_zoo import EncoderBlock, EncoderConfig


@dataclass
class CLIPVisionConfig(EncoderConfig):
    image_size: int = 224
    patch_size: int = 32
    num_channels: int = 3
    pre_norm: bool = True
    activation: str = "quick_gelu"
    layer_norm_eps: float = 1e-5
    dropout: float = 0.0


@dataclass
class CLIPTextConfig(EncoderConfig):
    vocab_size: int = 49408
    max_position_embeddings: int = 77
    hidden_size: int = 512
    num_heads: int = 8
    intermediate_size: int = 2048
    pre_norm: bool = True
    activation: str = "quick_gelu"
    layer_norm_eps: float = 1e-5
    dropout: float = 0.0
    eos_token_id: int = 49407


@dataclass
class CLIPConfig:
    vision: CLIPVisionConfig = field(default_factory=CLIPVisionConfig)
    text: CLIPTextConfig = field(default_factory=CLIPTextConfig)
    projection_dim: int = 512
    logit_scale_init: float = 2.6592

    @classmethod
    def vit_b_32(cls): return cls()
    @classmethod
    def tiny(cls):
        return cls(CLIPVisionConfig(hidden_size=64, num_layers=2, num_heads=4, intermediate_size=128, image_size=32, patch_size=8),
                   CLIPTextConfig(vocab_size=300, max_position_embeddings=16, hidden_size=48, num_layers=2, num_heads=4,
                                  intermediate_size=96, eos_token_id=299), projection_dim=32)


class CLIPVisionTower(nn.Module):
    def __init__(self, cfg: CLIPVisionConfig):
        super().__init__()
        self.config = cfg
        E = cfg.hidden_size
        n = (cfg.image_size // cfg.patch_size) ** 2
        self.patch_embed = nn.Conv2d(cfg.num_channels, E, cfg.patch_size, cfg.patch_size, bias=False)
        self.class_embedding = nn.Parameter(torch.empty(E).normal_(0, 0.02))
        self.position_embedding = nn.Parameter(torch.empty(n + 1, E).normal_(0, 0.02))
        self.pre_ln = nn.LayerNorm(E, cfg.layer_norm_eps)
        self.layers = nn.ModuleList([EncoderBlock(cfg) for _ in range(cfg.num_layers)])
        self.post_ln = nn.LayerNorm(E, cfg.layer_norm_eps)

    def forward(self, pixels: torch.Tensor) -> torch.Tensor:
        x = self.patch_embed(pixels).flatten(2).transpose(1, 2)
        cls = self.class_embedding.to(x.dtype).expand(x.shape[0], 1, -1)
        x = self.pre_ln(torch.cat([cls, x], 1) + self.position_embedding.to(x.dtype))
        for l in self.layers:
            x = l(x)
        return self.post_ln(x[:, 0])            # pooled: the class token


class CLIPTextTower(nn.Module):
    def __init__(self, cfg: CLIPTextConfig):
        super().__init__()
        self.config = cfg
        E = cfg.hidden_size
        self.token_embedding = nn.Embedding(cfg.vocab_size, E)
        self.position_embedding = nn.Parameter(torch.empty(cfg.max_position_embeddings, E).normal_(0, 0.01))
        self.layers = nn.ModuleList([EncoderBlock(cfg, causal=True) for _ in range(cfg.num_layers)])
        self.final_ln = nn.LayerNorm(E, cfg.layer_norm_eps)

    def forward(self, input_ids: torch.Tensor) -> torch.Tensor:
        x = self.token_embedding(input_ids) + self.position_embedding[: input_ids.shape[1]].to(self.token_embedding.weight.dtype)
        for l in self.layers:
            x = l(x)
        x = self.final_ln(x)
        # pooled: the hidden state at the end-of-text token (first occurrence)
        eos = (input_ids == self.config.eos_token_id).int().argmax(-1)
        return x[torch.arange(x.shape[0], device=x.device), eos]


class CLIPModel(nn.Module):
    def __init__(self, cfg: CLIPConfig | None = None):
        super().__init__()
        cfg = cfg or CLIPConfig()
        self.config = cfg
        self.vision = CLIPVisionTower(cfg.vision)
        self.text = CLIPTextTower(cfg.text)
        self.visual_projection = nn.Linear(cfg.vision.hidden_size, cfg.projection_dim, bias=False)
        self.text_projection = nn.Linear(cfg.text.hidden_size, cfg.projection_dim, bias=False)
        self.logit_scale = nn.Parameter(torch.tensor(cfg.logit_scale_init))

    def encode_image(self, pixels):
        e = self.visual_projection(self.vision(pixels))
        return e / e.norm(dim=-1, keepdim=True)

    def encode_text(self, input_ids):
        e = self.text_projection(self.text(input_ids))
        return e / e.norm(dim=-1, keepdim=True)

    def forward(self, input_ids, pixels, return_loss: bool = False):
        """Returns ``(logits_per_image, logits_per_text)``; with ``return_loss`` also the symmetric InfoNCE loss."""
        img, txt = self.encode_image(pixels), self.encode_text(input_ids)
        lt = self.logit_scale.exp() * txt.float() @ img.float().t()
        if not return_loss:
            return lt.t(), lt
        tgt = torch.arange(lt.shape[0], device=lt.device)
        loss = 0.5 * (torch.nn.functional.cross_entropy(lt, tgt) + torch.nn.functional.cross_entropy(lt.t(), tgt))
        return lt.t(), lt, loss


class DualEncoder(nn.Module):
    """ALIGN-style model: any image encoder and any text encoder that return pooled features, linear projections to a
    shared space, a learned temperature and the same symmetric contrastive loss."""

    def __init__(self, image_encoder: torch.nn.Module, text_encoder: torch.nn.Module, image_dim: int, text_dim: int,
                 projection_dim: int = 640, temperature_init: float = 0.07):
        super().__init__()
        self.image_encoder, self.text_encoder = image_encoder, text_encoder
        self.image_projection = nn.Linear(image_dim, projection_dim)
        self.text_projection = nn.Linear(text_dim, projection_dim)
        self.log_temperature = nn.Parameter(torch.tensor(math.log(temperature_init)))

    def forward(self, text_inputs, pixels):
        i = torch.nn.functional.normalize(self.image_projection(self.image_encoder(pixels)), dim=-1)
        t = torch.nn.functional.normalize(self.text_projection(self.text_encoder(text_inputs)), dim=-1)
        logits = t.float() @ i.float().t() / self.log_temperature.exp()
        tgt = torch.arange(logits.shape[0], device=logits.device)
        loss = 0.5 * (torch.nn.functional.cross_entropy(logits, tgt) + torch.nn.functional.cross_entropy(logits.t(), tgt))
        return logits, loss


ALIGNModel = DualEncoder
