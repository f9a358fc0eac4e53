"""Layers. Kernel-backed: Linear, LayerNorm, RMSNorm, Embedding, activations, SwiGLU family,
MultiheadAttention / FlashMultiHeadAttention, rotary embedding, cross-entropy. The long tail
(convolutions, pooling, recurrent, dropout, ...) adopts the PyTorch layer of the same name with the
ToRSh mixin, so the whole reference layer list (``crates/torsh-nn/src/layers/**``) is constructible.
"""
from __future__ import annotations

import math

import torch
import torch.nn.functional as tF

from .. import ops
from ..ops import attention as attn_ops
from ..ops import elementwise as ew
from ..ops import linear as lin_ops
from ..ops import norm as norm_ops
from ..ops import softmax as sm_ops
from . import init as tinit
from .module import Module, ModuleMixin, Parameter


class Linear(Module):
    """``y = x Wᵀ + b`` with weight ``[out, in]`` (``layout="nk"``, PyTorch) or ``y = x W + b`` with
    weight ``[in, out]`` (``layout="kn"``, the reference layout: ``crates/torsh-nn/src/layers/linear.rs:16-62``,
    Xavier-uniform weight, zero bias)."""

    def __init__(self, in_features: int, out_features: int, bias: bool = True, layout: str = "nk", device=None,
                 dtype=None):
        super().__init__()
        self.in_features, self.out_features, self.layout = in_features, out_features, layout
        shape = (out_features, in_features) if layout == "nk" else (in_features, out_features)
        self.weight = Parameter(torch.empty(shape, device=device, dtype=dtype))
        self.bias = Parameter(torch.zeros(out_features, device=device, dtype=dtype)) if bias else None
        tinit.xavier_uniform_(self.weight)

    def forward(self, x):
        return lin_ops.linear(x, self.weight, self.bias, layout=self.layout)

    def extra_repr(self):
        return f"in_features={self.in_features}, out_features={self.out_features}, bias={self.bias is not None}, layout={self.layout}"


class Embedding(Module):
    def __init__(self, num_embeddings: int, embedding_dim: int, padding_idx: int | None = None, device=None, dtype=None):
        super().__init__()
        self.num_embeddings, self.embedding_dim, self.padding_idx = num_embeddings, embedding_dim, padding_idx
        self.weight = Parameter(torch.empty(num_embeddings, embedding_dim, device=device, dtype=dtype))
        torch.nn.init.normal_(self.weight)
        if padding_idx is not None:
            with torch.no_grad():
                self.weight[padding_idx].zero_()

    def forward(self, ids):
        return ew.embedding(ids, self.weight)


class LayerNorm(Module):
    def __init__(self, normalized_shape, eps: float = 1e-5, elementwise_affine: bool = True, bias: bool = True,
                 device=None, dtype=None):
        super().__init__()
        self.normalized_shape = (normalized_shape,) if isinstance(normalized_shape, int) else tuple(normalized_shape)
        self.eps = eps
        n = math.prod(self.normalized_shape)
        self.weight = Parameter(torch.ones(n, device=device, dtype=dtype)) if elementwise_affine else None
        self.bias = Parameter(torch.zeros(n, device=device, dtype=dtype)) if elementwise_affine and bias else None

    def forward(self, x):
        if self.weight is None or len(self.normalized_shape) != 1:
            return tF.layer_norm(x, self.normalized_shape, None if self.weight is None else self.weight.view(self.normalized_shape),
                                 None if self.bias is None else self.bias.view(self.normalized_shape), self.eps)
        return norm_ops.layer_norm(x, self.weight, self.bias, self.eps)


class RMSNorm(Module):
    """``x / sqrt(mean(x²) + eps) * weight`` with eps 1e-6
    (``crates/torsh-nn/src/layers/normalization/layer_group/mod.rs:491-514``)."""

    def __init__(self, dim: int, eps: float = 1e-6, device=None, dtype=None):
        super().__init__()
        self.eps = eps
        self.weight = Parameter(torch.ones(dim, device=device, dtype=dtype))

    def forward(self, x):
        return norm_ops.rms_norm(x, self.weight, self.eps)


class GELU(Module):
    def __init__(self, approximate: str = "none"):
        super().__init__()
        self.approximate = approximate

    def forward(self, x):
        return ew.gelu(x, self.approximate)


class ReLU(Module):
    def __init__(self, inplace: bool = False):
        super().__init__()

    def forward(self, x):
        return ew.relu(x)


class Sigmoid(Module):
    def forward(self, x):
        return ew.sigmoid(x)


class Tanh(Module):
    def forward(self, x):
        return ew.tanh(x)


class SiLU(Module):
    def forward(self, x):
        return ew.silu(x)


Swish = SiLU


class SwiGLU(Module):
    """Splits ``dim`` into halves ``(a, b)`` and returns ``a * silu(b)``: the gate is the second half
    (``crates/torsh-nn/src/layers/activation/gated.rs:536-608``)."""

    def __init__(self, dim: int = -1):
        super().__init__()
        self.dim = dim

    def forward(self, x):
        if self.dim in (-1, x.dim() - 1):
            return ew.swiglu(x)
        a, b = x.chunk(2, self.dim)
        return a * tF.silu(b)


class GLU(Module):
    def __init__(self, dim: int = -1):
        super().__init__()
        self.dim = dim

    def forward(self, x):
        a, b = x.chunk(2, self.dim)
        return a * torch.sigmoid(b)


class GeGLU(GLU):
    def forward(self, x):
        a, b = x.chunk(2, self.dim)
        return a * tF.gelu(b)


class ReGLU(GLU):
    def forward(self, x):
        a, b = x.chunk(2, self.dim)
        return a * torch.relu(b)


class Mish(Module):
    def forward(self, x):
        return tF.mish(x)


class Softmax(Module):
    def __init__(self, dim: int = -1):
        super().__init__()
        self.dim = dim

    def forward(self, x):
        return sm_ops.softmax(x, self.dim)


class LogSoftmax(Module):
    def __init__(self, dim: int = -1):
        super().__init__()
        self.dim = dim

    def forward(self, x):
        return sm_ops.log_softmax(x, self.dim)


class CrossEntropyLoss(Module):
    def __init__(self, ignore_index: int = -100, reduction: str = "mean", label_smoothing: float = 0.0):
        super().__init__()
        self.ignore_index, self.reduction, self.label_smoothing = ignore_index, reduction, label_smoothing

    def forward(self, logits, target):
        if self.reduction == "mean" and self.label_smoothing == 0.0 and target.dtype in (torch.int64, torch.int32):
            return sm_ops.cross_entropy(logits, target, ignore_index=self.ignore_index)
        return tF.cross_entropy(logits, target, ignore_index=self.ignore_index, reduction=self.reduction,
                                label_smoothing=self.label_smoothing)


class RotaryPositionalEmbedding(Module):
    """``RotaryPositionalEmbedding(d_model, base, max_seq_len)``: rotates adjacent pairs ``(2i, 2i+1)``
    by ``pos · base^(-2i/d)``. The reference builds the same frequencies but its rotation step returns
    the input unchanged (``crates/torsh-nn/src/layers/embedding.rs:372-430``); this one rotates."""

    def __init__(self, d_model: int, base: float = 10000.0, max_seq_len: int = 2048):
        super().__init__()
        self.d_model, self.base, self.max_seq_len = d_model, base, max_seq_len

    def forward(self, x, pos_offset: int = 0):
        """``x``: ``[B, S, heads, D]``."""
        return ew.rope(x, self.base, pos_offset)

    def apply_rope(self, q, k, pos_offset: int = 0):
        """``q, k``: ``[B, heads, S, D]`` as in the reference signature."""
        r = lambda t: ew.rope(t.transpose(1, 2).contiguous(), self.base, pos_offset).transpose(1, 2)
        return r(q), r(k)


class SinusoidalPositionalEncoding(Module):
    def __init__(self, d_model: int, max_len: int = 5000, dropout: float = 0.0):
        super().__init__()
        pos = torch.arange(max_len).unsqueeze(1)
        div = torch.exp(torch.arange(0, d_model, 2) * (-math.log(10000.0) / d_model))
        pe = torch.zeros(max_len, d_model)
        pe[:, 0::2] = torch.sin(pos * div)
        pe[:, 1::2] = torch.cos(pos * div)[:, : d_model // 2]
        self.register_buffer("pe", pe, persistent=False)
        self.dropout = torch.nn.Dropout(dropout)

    def forward(self, x):
        return self.dropout(x + self.pe[: x.shape[-2]].to(x.dtype))


class LearnablePositionalEncoding(Module):
    def __init__(self, d_model: int, max_len: int = 512):
        super().__init__()
        self.weight = Parameter(torch.zeros(max_len, d_model))
        torch.nn.init.normal_(self.weight, std=0.02)

    def forward(self, x):
        return x + self.weight[: x.shape[-2]].to(x.dtype)


class ALiBi(Module):
    """Attention with linear biases: per-head slopes ``2^(-8h/H)``."""

    def __init__(self, num_heads: int):
        super().__init__()
        slopes = torch.tensor([2 ** (-8.0 * (h + 1) / num_heads) for h in range(num_heads)])
        self.register_buffer("slopes", slopes, persistent=False)

    def forward(self, seq_len: int) -> torch.Tensor:
        pos = torch.arange(seq_len, device=self.slopes.device)
        rel = (pos[None, :] - pos[:, None]).clamp(max=0).float()
        return self.slopes[:, None, None] * rel[None]


class MultiheadAttention(Module):
    """Parameters ``in_proj_weight [3E, E]``, ``in_proj_bias [3E]``, ``out_proj.weight [E, E]``,
    ``out_proj.bias [E]`` (Xavier / zeros) and ``batch_first=False`` by default, as in
    ``crates/torsh-nn/src/layers/attention.rs:16-110``. Self-attention without an explicit mask runs the
    fused QKV GEMM + flash-attention kernels; anything else uses the general masked path."""

    def __init__(self, embed_dim: int, num_heads: int, dropout: float = 0.0, bias: bool = True,
                 batch_first: bool = False, device=None, dtype=None):
        super().__init__()
        assert embed_dim % num_heads == 0
        self.embed_dim, self.num_heads, self.head_dim = embed_dim, num_heads, embed_dim // num_heads
        self.dropout, self.batch_first = dropout, batch_first
        self.in_proj_weight = Parameter(torch.empty(3 * embed_dim, embed_dim, device=device, dtype=dtype))
        self.in_proj_bias = Parameter(torch.zeros(3 * embed_dim, device=device, dtype=dtype)) if bias else None
        self.out_proj = Linear(embed_dim, embed_dim, bias=bias, device=device, dtype=dtype)
        tinit.xavier_uniform_(self.in_proj_weight)

    def forward(self, query, key=None, value=None, attn_mask=None, key_padding_mask=None, need_weights: bool = False,
                is_causal: bool = False):
        key = query if key is None else key
        value = key if value is None else value
        if not self.batch_first:
            query, key, value = (t.transpose(0, 1) for t in (query, key, value))
        B, S, E = query.shape
        H, D = self.num_heads, self.head_dim
        self_attn = key is query and value is query or (key.data_ptr() == query.data_ptr() and value.data_ptr() == query.data_ptr())
        fast = (self_attn and attn_mask is None and key_padding_mask is None and not need_weights
                and (self.dropout == 0.0 or not self.training))
        if fast:
            qkv = lin_ops.linear(query.reshape(B * S, E), self.in_proj_weight, self.in_proj_bias)
            ctx = attn_ops.flash_attention_qkvpacked(qkv, B, S, H, D, causal=is_causal)
            out = self.out_proj(ctx).view(B, S, E)
            weights = None
        else:
            w_q, w_k, w_v = self.in_proj_weight.chunk(3, 0)
            b_q, b_k, b_v = self.in_proj_bias.chunk(3, 0) if self.in_proj_bias is not None else (None,) * 3
            q = tF.linear(query, w_q, b_q).view(B, S, H, D).transpose(1, 2)
            Sk = key.shape[1]
            k = tF.linear(key, w_k, b_k).view(B, Sk, H, D).transpose(1, 2)
            v = tF.linear(value, w_v, b_v).view(B, Sk, H, D).transpose(1, 2)
            scores = torch.matmul(q, k.transpose(-1, -2)) / math.sqrt(D)
            if is_causal:
                scores = scores.masked_fill(torch.ones(S, Sk, dtype=torch.bool, device=q.device).triu(1), float("-inf"))
            if attn_mask is not None:
                scores = scores.masked_fill(attn_mask, float("-inf")) if attn_mask.dtype == torch.bool else scores + attn_mask
            if key_padding_mask is not None:
                scores = scores.masked_fill(key_padding_mask[:, None, None, :], float("-inf"))
            weights = torch.softmax(scores, -1)
            p = tF.dropout(weights, self.dropout, self.training)
            out = self.out_proj(torch.matmul(p, v).transpose(1, 2).reshape(B, S, E))
            weights = weights.mean(1) if need_weights else None
        if not self.batch_first:
            out = out.transpose(0, 1)
        return out, weights


class FlashMultiHeadAttention(MultiheadAttention):
    """Always takes the flash path (``crates/torsh-nn/src/layers/attention.rs:406-460``; the reference's
    ``block_size`` argument is accepted and ignored: tiles are fixed at 128 x 128 by the TMEM layout)."""

    def __init__(self, embed_dim: int, num_heads: int, block_size: int = 128, **kw):
        super().__init__(embed_dim, num_heads, **kw)
        self.block_size = block_size


# --------------------------------------------------------------------------- adopted PyTorch layers
def _adopt(name: str):
    base = getattr(torch.nn, name)
    return type(name, (ModuleMixin, base), {"__doc__": f"``torch.nn.{name}`` with the ToRSh module mixin.",
                                            "__module__": __name__})


_ADOPTED = [
    "Flatten", "Unflatten", "Identity", "Conv1d", "Conv2d", "Conv3d", "ConvTranspose1d", "ConvTranspose2d",
    "ConvTranspose3d", "BatchNorm1d", "BatchNorm2d", "BatchNorm3d", "SyncBatchNorm", "GroupNorm", "InstanceNorm1d",
    "InstanceNorm2d", "InstanceNorm3d", "LocalResponseNorm", "MaxPool1d", "MaxPool2d", "MaxPool3d", "AvgPool1d",
    "AvgPool2d", "AvgPool3d", "AdaptiveAvgPool1d", "AdaptiveAvgPool2d", "AdaptiveAvgPool3d", "AdaptiveMaxPool1d",
    "AdaptiveMaxPool2d", "AdaptiveMaxPool3d", "FractionalMaxPool2d", "LPPool1d", "LPPool2d", "Dropout", "Dropout1d",
    "Dropout2d", "Dropout3d", "AlphaDropout", "FeatureAlphaDropout", "RNN", "LSTM", "GRU", "RNNCell", "LSTMCell",
    "GRUCell", "LeakyReLU", "PReLU", "RReLU", "ELU", "SELU", "CELU", "ReLU6", "Hardtanh", "Hardswish", "Hardsigmoid",
    "Hardshrink", "Softshrink", "Tanhshrink", "Softplus", "Softsign", "Softmin", "Softmax2d", "LogSigmoid",
    "Threshold", "PixelShuffle", "PixelUnshuffle", "Upsample", "UpsamplingNearest2d", "UpsamplingBilinear2d",
    "ZeroPad2d", "ReflectionPad2d", "ReplicationPad2d", "ConstantPad2d", "Bilinear", "EmbeddingBag",
    "TransformerEncoderLayer", "TransformerEncoder", "TransformerDecoderLayer", "TransformerDecoder", "Transformer",
    "MSELoss", "L1Loss", "SmoothL1Loss", "HuberLoss", "BCELoss", "BCEWithLogitsLoss", "NLLLoss", "KLDivLoss",
    "CosineEmbeddingLoss", "MarginRankingLoss", "HingeEmbeddingLoss", "TripletMarginLoss", "PoissonNLLLoss",
    "GaussianNLLLoss", "CTCLoss", "MultiMarginLoss", "MultiLabelMarginLoss", "MultiLabelSoftMarginLoss",
    "SoftMarginLoss", "CosineSimilarity", "PairwiseDistance", "Fold", "Unfold", "ChannelShuffle",
]
for _n in _ADOPTED:
    if hasattr(torch.nn, _n):
        globals()[_n] = _adopt(_n)

SyncBatchNorm2d = globals()["SyncBatchNorm"]
