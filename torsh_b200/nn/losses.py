"""The loss family of the functional API: classification, regression, similarity / metric learning, information-theoretic
and the specialised sequence / GAN losses. All take ``reduction`` in {"none", "mean", "sum"} and are differentiable through
PyTorch autograd; the large-vocabulary cross entropy routes to the fused kernel (``ops.softmax.cross_entropy``).

Names and argument order follow the reference (crates/torsh-functional/src/loss/{classification,regression,similarity,
information,specialized}.rs).
"""
from __future__ import annotations

import torch
import torch.nn.functional as F

EPS = 1e-8


def _reduce(x: torch.Tensor, reduction: str) -> torch.Tensor:
    if reduction == "none":
        return x
    if reduction == "mean":
        return x.mean()
    if reduction == "sum":
        return x.sum()
    raise ValueError(f"unknown reduction {reduction!r}")


def _safe_log(x):
    return torch.log(x.clamp_min(EPS))


# ---- classification ------------------------------------------------------------------------------------------------
def cross_entropy(logits, target, weight=None, ignore_index: int = -100, reduction: str = "mean", label_smoothing: float = 0.0):
    if logits.is_cuda and logits.dtype == torch.bfloat16 and weight is None and label_smoothing == 0.0 and reduction == "mean" \
            and logits.dim() == 2:
        from ..ops.softmax import cross_entropy as fused
        return fused(logits, target, ignore_index=ignore_index)
    return F.cross_entropy(logits, target, weight=weight, ignore_index=ignore_index, reduction=reduction, label_smoothing=label_smoothing)


def cross_entropy_with_label_smoothing(logits, target, smoothing: float = 0.1, reduction: str = "mean"):
    """(1 - s) * NLL(target) + s * mean over classes of NLL."""
    logp = F.log_softmax(logits.float(), -1)
    nll = -logp.gather(-1, target.unsqueeze(-1)).squeeze(-1)
    return _reduce((1 - smoothing) * nll + smoothing * (-logp.mean(-1)), reduction)


def nll_loss(log_probs, target, weight=None, ignore_index: int = -100, reduction: str = "mean"):
    return F.nll_loss(log_probs, target, weight=weight, ignore_index=ignore_index, reduction=reduction)


def binary_cross_entropy(probs, target, weight=None, reduction: str = "mean"):
    return F.binary_cross_entropy(probs, target, weight=weight, reduction=reduction)


def binary_cross_entropy_with_logits(logits, target, weight=None, pos_weight=None, reduction: str = "mean"):
    return F.binary_cross_entropy_with_logits(logits, target, weight=weight, pos_weight=pos_weight, reduction=reduction)


def focal_loss(logits, target, alpha: float = 0.25, gamma: float = 2.0, reduction: str = "mean"):
    """Binary focal loss on logits: alpha_t * (1 - p_t)^gamma * BCE."""
    bce = F.binary_cross_entropy_with_logits(logits, target, reduction="none")
    p = torch.sigmoid(logits)
    pt = p * target + (1 - p) * (1 - target)
    at = alpha * target + (1 - alpha) * (1 - target)
    return _reduce(at * (1 - pt).pow(gamma) * bce, reduction)


def multi_margin_loss(logits, target, p: int = 1, margin: float = 1.0, weight=None, reduction: str = "mean"):
    return F.multi_margin_loss(logits, target, p=p, margin=margin, weight=weight, reduction=reduction)


def hinge_embedding_loss(x, target, margin: float = 1.0, reduction: str = "mean"):
    return F.hinge_embedding_loss(x, target, margin=margin, reduction=reduction)


# ---- regression ----------------------------------------------------------------------------------------------------
def mse_loss(x, target, reduction: str = "mean"):
    return F.mse_loss(x, target, reduction=reduction)


def l1_loss(x, target, reduction: str = "mean"):
    return F.l1_loss(x, target, reduction=reduction)


def smooth_l1_loss(x, target, beta: float = 1.0, reduction: str = "mean"):
    return F.smooth_l1_loss(x, target, beta=beta, reduction=reduction)


def huber_loss(x, target, delta: float = 1.0, reduction: str = "mean"):
    return F.huber_loss(x, target, delta=delta, reduction=reduction)


def gaussian_nll_loss(mean, target, var, full: bool = False, eps: float = 1e-6, reduction: str = "mean"):
    return F.gaussian_nll_loss(mean, target, var, full=full, eps=eps, reduction=reduction)


def poisson_nll_loss(x, target, log_input: bool = True, full: bool = False, eps: float = 1e-8, reduction: str = "mean"):
    return F.poisson_nll_loss(x, target, log_input=log_input, full=full, eps=eps, reduction=reduction)


# ---- similarity / metric learning ----------------------------------------------------------------------------------
def cosine_embedding_loss(x1, x2, target, margin: float = 0.0, reduction: str = "mean"):
    return F.cosine_embedding_loss(x1, x2, target, margin=margin, reduction=reduction)


def margin_ranking_loss(x1, x2, target, margin: float = 0.0, reduction: str = "mean"):
    return F.margin_ranking_loss(x1, x2, target, margin=margin, reduction=reduction)


def triplet_margin_loss(anchor, positive, negative, margin: float = 1.0, p: float = 2.0, swap: bool = False, reduction: str = "mean"):
    return F.triplet_margin_loss(anchor, positive, negative, margin=margin, p=p, swap=swap, reduction=reduction)


def triplet_margin_with_distance_loss(anchor, positive, negative, distance_function=None, margin: float = 1.0, swap: bool = False,
                                      reduction: str = "mean"):
    d = distance_function or (lambda a, b: F.pairwise_distance(a, b))
    dp, dn = d(anchor, positive), d(anchor, negative)
    if swap:
        dn = torch.minimum(dn, d(positive, negative))
    return _reduce((dp - dn + margin).clamp_min(0), reduction)


def contrastive_loss(x1, x2, label, margin: float = 1.0, reduction: str = "mean"):
    """label 1 = similar pair: d^2; label 0 = dissimilar: max(0, margin - d)^2."""
    d = F.pairwise_distance(x1, x2)
    return _reduce(label * d.pow(2) + (1 - label) * (margin - d).clamp_min(0).pow(2), reduction)


# ---- information-theoretic -----------------------------------------------------------------------------------------
def kl_div(log_input, target, reduction: str = "mean", log_target: bool = False):
    return F.kl_div(log_input, target, reduction=reduction, log_target=log_target)


def js_divergence(p, q, reduction: str = "mean"):
    """Jensen-Shannon divergence between distributions given in linear space (last dim sums to one)."""
    m = 0.5 * (p + q)
    js = 0.5 * (p * (_safe_log(p) - _safe_log(m))).sum(-1) + 0.5 * (q * (_safe_log(q) - _safe_log(m))).sum(-1)
    return _reduce(js, reduction)


def cross_entropy_continuous(p_pred, p_true, reduction: str = "mean"):
    """H(true, pred) = -sum true * log(pred), both in linear space."""
    return _reduce(-(p_true * _safe_log(p_pred)), reduction)


def entropy_loss(p, reduction: str = "mean"):
    """-p log p element-wise (sum over the distribution for its entropy)."""
    return _reduce(-(p * _safe_log(p)), reduction)


def mutual_information_loss(joint_scores, marginal_scores, reduction: str = "mean"):
    """Negative Donsker-Varadhan bound: -(E_joint[T] - log E_marginal[exp T]); minimising it maximises the estimate of
    I(X; Y) from critic scores on joint and shuffled pairs."""
    bound = joint_scores.mean() - (torch.logsumexp(marginal_scores.flatten(), 0) - torch.log(torch.tensor(float(marginal_scores.numel()))))
    return _reduce(-bound.reshape(1), reduction) if reduction != "none" else -bound


# ---- specialised ---------------------------------------------------------------------------------------------------
def ctc_loss(log_probs, targets, input_lengths, target_lengths, blank: int = 0, reduction: str = "mean", zero_infinity: bool = False):
    return F.ctc_loss(log_probs, targets, input_lengths, target_lengths, blank=blank, reduction=reduction, zero_infinity=zero_infinity)


def wasserstein_loss(real_scores, fake_scores, reduction: str = "mean"):
    """Critic objective E[D(fake)] - E[D(real)] (to minimise)."""
    if reduction == "none":
        return fake_scores - real_scores
    return _reduce(fake_scores, reduction) - _reduce(real_scores, reduction)


def gradient_penalty_loss(gradients, penalty_weight: float = 10.0, reduction: str = "mean"):
    """WGAN-GP: weight * (||grad||_2 - 1)^2 per sample."""
    if penalty_weight <= 0:
        raise ValueError("penalty_weight must be positive")
    norms = gradients.flatten(1).norm(dim=1)
    return _reduce(penalty_weight * (norms - 1).pow(2), reduction)


def temporal_consistency_loss(predictions, smoothness_weight: float = 1.0, reduction: str = "mean"):
    """Squared difference of consecutive time steps of ``[N, T, ...]`` predictions."""
    if predictions.dim() < 3:
        raise ValueError("temporal_consistency_loss expects [N, T, ...]")
    d = predictions[:, 1:] - predictions[:, :-1]
    return _reduce(smoothness_weight * d.pow(2), reduction)


def seq2seq_loss_with_attention(predictions, targets, attention_weights=None, attention_reg: float = 0.0, ignore_index: int = -100,
                                reduction: str = "mean"):
    """Token cross entropy of ``[N, T, V]`` logits plus ``attention_reg`` times the coverage penalty
    sum_s (1 - sum_t a[t, s])^2 of ``[N, T_out, T_in]`` attention weights (every source position attended about once)."""
    n, t, v = predictions.shape
    ce = F.cross_entropy(predictions.reshape(n * t, v).float(), targets.reshape(n * t), ignore_index=ignore_index,
                         reduction="none").reshape(n, t)
    loss = _reduce(ce, reduction)
    if attention_weights is not None and attention_reg > 0:
        cov = (1 - attention_weights.sum(1)).pow(2).sum(-1)          # [N]
        loss = loss + attention_reg * (_reduce(cov, reduction) if reduction != "none" else cov[:, None])
    return loss


def dice_loss(probs, target, eps: float = 1.0):
    inter = (probs * target).sum()
    return 1 - (2 * inter + eps) / (probs.sum() + target.sum() + eps)


__all__ = [n for n, f in list(globals().items()) if callable(f) and not n.startswith("_") and getattr(f, "__module__", None) == __name__]
