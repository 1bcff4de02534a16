"""Plain PyTorch (fp32) statements of the operators, used as test oracles."""
from __future__ import annotations

import torch
import torch.nn.functional as F


def norm(x, weight, bias, eps):
    v = x.float()
    if bias is not None:
        return F.layer_norm(v, v.shape[-1:], weight.float(), bias.float(), eps)
    return v * torch.rsqrt(v.pow(2).mean(-1, keepdim=True) + eps) * weight.float()


def linear(x, weight, bias=None, act="none"):
    y = F.linear(x.float(), weight.float(), None if bias is None else bias.float())
    return F.gelu(y) if act == "gelu" else y


def linear_cross_entropy(h, weight, targets):
    logits = F.linear(h.float(), weight.float())
    return F.cross_entropy(logits, targets)


def adamw_step(p, g, m, v, lr, beta1, beta2, eps, wd, step):
    """One decoupled-weight-decay Adam step on flat fp32 tensors; returns new (p, m, v)."""
    m = beta1 * m + (1 - beta1) * g
    v = beta2 * v + (1 - beta2) * g * g
    mhat = m / (1 - beta1 ** step)
    vhat = v / (1 - beta2 ** step)
    p = p * (1 - lr * wd) - lr * mhat / (vhat.sqrt() + eps)
    return p, m, v
