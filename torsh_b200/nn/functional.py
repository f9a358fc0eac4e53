"""Functional API (``crates/torsh-functional``, ``crates/torsh-nn/src/functional``).

Kernel-backed entries dispatch to :mod:`torsh_b200.ops`; everything else is the PyTorch function
of the same name, re-exported so ``F.<name>`` covers the reference's list (activations, conv,
pooling, 28 losses, norms, attention variants, fusion helpers).
"""
from __future__ import annotations

import math

import torch
import torch.nn.functional as _tF

from ..ops import attention as _attn
from ..ops import elementwise as _ew
from ..ops import linear as _lin
from ..ops import norm as _norm
from ..ops import softmax as _sm

# ---- kernel-backed -------------------------------------------------------------------------
relu, sigmoid, tanh, silu, gelu, swiglu = _ew.relu, _ew.sigmoid, _ew.tanh, _ew.silu, _ew.gelu, _ew.swiglu
swish = silu
softmax, log_softmax = _sm.softmax, _sm.log_softmax
embedding_lookup = _ew.embedding
rope = _ew.rope
flash_attention = _attn.flash_attention


def linear(x, weight, bias=None):
    return _lin.linear(x, weight, bias)


def layer_norm(x, normalized_shape, weight=None, bias=None, eps: float = 1e-5):
    if weight is not None and (isinstance(normalized_shape, int) or len(normalized_shape) == 1):
        return _norm.layer_norm(x, weight, bias, eps)
    return _tF.layer_norm(x, normalized_shape, weight, bias, eps)


def rms_norm(x, weight, eps: float = 1e-6):
    return _norm.rms_norm(x, weight, eps)


def cross_entropy(logits, target, ignore_index: int = -100, reduction: str = "mean", label_smoothing: float = 0.0,
                  weight=None):
    """log_softmax + NLL (``crates/torsh-nn/src/functional/loss.rs:15-60``)."""
    if reduction == "mean" and label_smoothing == 0.0 and weight is None and not target.is_floating_point():
        return _sm.cross_entropy(logits, target, ignore_index=ignore_index)
    return _tF.cross_entropy(logits, target, weight=weight, ignore_index=ignore_index, reduction=reduction,
                             label_smoothing=label_smoothing)


def scaled_dot_product_attention(q, k, v, attn_mask=None, dropout_p: float = 0.0, is_causal: bool = False,
                                 scale: float | None = None):
    """``[B, H, S, D]`` inputs. Additive mask convention: 0 = keep, ``-inf`` / ``-1e9`` = masked
    (``crates/torsh-functional/src/attention.rs:215-271``)."""
    if attn_mask is None and dropout_p == 0.0 and q.is_cuda and q.dtype == torch.bfloat16 and q.shape[-1] in (64, 128) \
            and k.shape == q.shape:
        o = _attn.flash_attention(q.transpose(1, 2), k.transpose(1, 2), v.transpose(1, 2), causal=is_causal, scale=scale)
        return o.transpose(1, 2)
    return _tF.scaled_dot_product_attention(q, k, v, attn_mask=attn_mask, dropout_p=dropout_p, is_causal=is_causal,
                                            scale=scale)


def multi_head_attention(q, k, v, num_heads: int, attn_mask=None, is_causal: bool = False):
    """``[B, S, E]`` inputs already projected; splits heads, attends, merges."""
    B, S, E = q.shape
    D = E // num_heads
    sp = lambda t: t.view(B, t.shape[1], num_heads, D).transpose(1, 2)
    o = scaled_dot_product_attention(sp(q), sp(k), sp(v), attn_mask=attn_mask, is_causal=is_causal)
    return o.transpose(1, 2).reshape(B, S, E)


self_attention = multi_head_attention


def cross_attention(q, kv, num_heads: int, attn_mask=None):
    return multi_head_attention(q, kv, kv, num_heads, attn_mask)


# ---- fusion helpers (``crates/torsh-functional/src/fusion/operations.rs``) -----------------------
def fused_relu_add(x, y):
    """``relu(x + y)`` (``crates/torsh-functional/src/fusion/operations.rs:28-45``)."""
    return torch.relu(x + y)


def fused_add_relu(x, y):
    return torch.relu(x + y)


def fused_mul_add(x, y, z):
    return torch.addcmul(z, x, y)


def fused_add_mul(x, y, z):
    return (x + y) * z


def fused_sigmoid_mul(x, y):
    return torch.sigmoid(x) * y


def fused_silu(x):
    return silu(x)


def fused_tanh_scale(x, scale: float):
    return torch.tanh(x) * scale


def fused_add_relu_mul(x, y, z):
    return torch.relu(x + y) * z


def fused_batch_norm(x, running_mean, running_var, weight=None, bias=None, eps: float = 1e-5):
    return _tF.batch_norm(x, running_mean, running_var, weight, bias, False, 0.0, eps)


def gelu_exact(x):
    return _tF.gelu(x)


# ---- re-exported long tail -------------------------------------------------------------------
_REEXPORT = [
    "conv1d", "conv2d", "conv3d", "conv_transpose1d", "conv_transpose2d", "conv_transpose3d", "max_pool1d", "max_pool2d",
    "max_pool3d", "avg_pool1d", "avg_pool2d", "avg_pool3d", "adaptive_avg_pool1d", "adaptive_avg_pool2d",
    "adaptive_avg_pool3d", "adaptive_max_pool1d", "adaptive_max_pool2d", "lp_pool2d", "fractional_max_pool2d",
    "batch_norm", "group_norm", "instance_norm", "local_response_norm", "normalize", "dropout", "dropout1d", "dropout2d",
    "dropout3d", "alpha_dropout", "leaky_relu", "elu", "selu", "celu", "prelu", "rrelu", "relu6", "hardtanh", "hardswish",
    "hardsigmoid", "softplus", "softsign", "softmin", "softshrink", "hardshrink", "tanhshrink", "mish", "glu",
    "logsigmoid", "threshold", "gumbel_softmax", "embedding", "embedding_bag", "one_hot", "pad", "interpolate",
    "upsample", "grid_sample", "affine_grid", "unfold", "fold", "pixel_shuffle", "pixel_unshuffle", "mse_loss",
    "l1_loss", "smooth_l1_loss", "huber_loss", "binary_cross_entropy", "binary_cross_entropy_with_logits", "nll_loss",
    "kl_div", "cosine_embedding_loss", "margin_ranking_loss", "hinge_embedding_loss", "triplet_margin_loss",
    "poisson_nll_loss", "gaussian_nll_loss", "ctc_loss", "multi_margin_loss", "multilabel_margin_loss",
    "multilabel_soft_margin_loss", "soft_margin_loss", "cosine_similarity", "pairwise_distance", "pdist",
]
for _n in _REEXPORT:
    if hasattr(_tF, _n):
        globals()[_n] = getattr(_tF, _n)


def focal_loss(logits, target, alpha: float = 0.25, gamma: float = 2.0, reduction: str = "mean"):
    ce = _tF.binary_cross_entropy_with_logits(logits, target, reduction="none")
    p = torch.sigmoid(logits)
    pt = p * target + (1 - p) * (1 - target)
    loss = (alpha * target + (1 - alpha) * (1 - target)) * (1 - pt) ** gamma * ce
    return loss.mean() if reduction == "mean" else loss.sum() if reduction == "sum" else loss


def dice_loss(probs, target, eps: float = 1.0):
    inter = (probs * target).sum()
    return 1 - (2 * inter + eps) / (probs.sum() + target.sum() + eps)


def contrastive_loss(x1, x2, label, margin: float = 1.0):
    d = _tF.pairwise_distance(x1, x2)
    return (label * d.pow(2) + (1 - label) * torch.clamp(margin - d, min=0).pow(2)).mean()
