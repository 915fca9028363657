"""Plain PyTorch (autograd) statement of the same GPT-2, used only as the numerical oracle.

It consumes the flat llm.c-ordered parameter vector of ``models.gpt2.GPT2`` so gradients can be
compared tensor by tensor (the role ``train_gpt2.py`` + the debug-state file play for the
reference: ``test_gpt2.mojo:218-715``).
"""
from __future__ import annotations

import math
from typing import Dict, Tuple

import torch
import torch.nn.functional as F

from ..config import GPT2Config, PARAM_NAMES


def unflatten(config: GPT2Config, flat: torch.Tensor) -> Dict[str, torch.Tensor]:
    out, off = {}, 0
    for name, shape, size in zip(PARAM_NAMES, config.param_shapes(), config.param_sizes()):
        out[name] = flat[off:off + size].view(shape)
        off += size
    return out


def forward(config: GPT2Config, p: Dict[str, torch.Tensor], tokens: torch.Tensor,
            targets: torch.Tensor | None = None) -> Tuple[torch.Tensor, torch.Tensor | None]:
    """Returns (logits [B,T,Vp], mean loss).  ``p`` holds autograd leaves."""
    B, T = tokens.shape
    C, NH, L, V = config.channels, config.num_heads, config.num_layer, config.vocab_size
    hs = C // NH
    x = p["wte"][tokens.long()] + p["wpe"][:T]
    for l in range(L):
        h = F.layer_norm(x, (C,), p["ln1w"][l], p["ln1b"][l], 1e-5)
        qkv = h @ p["qkvw"][l].t() + p["qkvb"][l]
        q, k, v = (t.view(B, T, NH, hs).transpose(1, 2) for t in qkv.split(C, dim=2))
        att = (q @ k.transpose(-1, -2)) / math.sqrt(hs)
        mask = torch.ones(T, T, dtype=torch.bool, device=x.device).tril()
        att = att.masked_fill(~mask, float("-inf")).softmax(-1)
        y = (att @ v).transpose(1, 2).reshape(B, T, C)
        x = x + y @ p["attprojw"][l].t() + p["attprojb"][l]
        h = F.layer_norm(x, (C,), p["ln2w"][l], p["ln2b"][l], 1e-5)
        h = F.gelu(h @ p["fcw"][l].t() + p["fcb"][l], approximate="tanh")
        x = x + h @ p["fcprojw"][l].t() + p["fcprojb"][l]
    x = F.layer_norm(x, (C,), p["lnfw"], p["lnfb"], 1e-5)
    logits = x @ p["wte"].t()
    loss = None
    if targets is not None:
        loss = F.cross_entropy(logits[..., :V].reshape(-1, V).float(), targets.reshape(-1).long())
    return logits, loss


def loss_and_grads(config: GPT2Config, flat: torch.Tensor, tokens: torch.Tensor, targets: torch.Tensor):
    """(loss, logits, flat fp32 gradient) by autograd."""
    leaf = flat.detach().clone().float().requires_grad_(True)
    p = unflatten(config, leaf)
    logits, loss = forward(config, p, tokens, targets)
    loss.backward()
    return float(loss.detach()), logits.detach(), leaf.grad.detach()
