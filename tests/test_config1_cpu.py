"""BASELINE configuration 1: GPT-2 124M (L=12, NH=12, C=768, padded vocab 50304) in fp32 on the CPU, B=4, T=64,
AdamW lr 1e-4, weight decay 0, random init from the seed, uniform tokens.  Checked against PyTorch autograd: every
parameter tensor's gradient after the first forward/backward and the loss trajectory of the first 10 steps.  The
40-step timing of the same configuration is taken by ``python tests/test_config1_cpu.py`` (prints ms/step).

Marked slow: a 124M-parameter model on host cores takes a minute or two.
"""
import os
import sys
import time

import pytest
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)

from llm_mojo_b200.config import PARAM_NAMES, parse_model_descriptor
from llm_mojo_b200.models import GPT2, random_init_params
from llm_mojo_b200.models import reference as ref


def _tokens(cfg, B=4, T=64):
    g = torch.Generator().manual_seed(20240520)
    toks = torch.randint(0, cfg.vocab_size, (B, T + 1), generator=g, dtype=torch.int32)
    return toks[:, :-1].contiguous(), toks[:, 1:].contiguous()


@pytest.mark.slow
def test_config1_gradients_and_trajectory_match_autograd():
    cfg = parse_model_descriptor("d12")
    flat = random_init_params(cfg)
    x, y = _tokens(cfg)
    model = GPT2(cfg, "fp32", "cpu", params_flat=flat)
    model.forward(x, y)
    model.backward()
    loss0 = model.read_loss()
    exp_loss, _, exp_grad = ref.loss_and_grads(cfg, flat, x, y)
    assert abs(loss0 - float(exp_loss)) < 1e-4
    for name in PARAM_NAMES:
        b, e = model.tensor_range(name)
        got, want = model.g[name].flatten(), exp_grad[b:e]
        scale = want.abs().max().item() + 1e-12
        assert (got - want).abs().max().item() <= 1e-4 + 1e-3 * scale, name
        assert ((got - want).norm() / (want.norm() + 1e-30)).item() < 1e-3, name
    # 10-step trajectory against torch.optim.AdamW on the autograd model
    leaf = flat.clone().requires_grad_(True)
    opt = torch.optim.AdamW([leaf], lr=1e-4, betas=(0.9, 0.999), eps=1e-8, weight_decay=0.0)
    model = GPT2(cfg, "fp32", "cpu", params_flat=flat)
    for step in range(10):
        opt.zero_grad()
        _, l = ref.forward(cfg, ref.unflatten(cfg, leaf), x, y)
        l.backward()
        opt.step()
        model.forward(x, y)
        model.backward()
        model.update(step + 1, 1e-4, 0.0)
        assert abs(model.read_loss() - float(l.detach())) < 2e-3, step


def time_config1(steps=40):
    cfg = parse_model_descriptor("d12")
    model = GPT2(cfg, "fp32", "cpu", params_flat=random_init_params(cfg))
    x, y = _tokens(cfg)
    ms = []
    for step in range(steps):
        t0 = time.perf_counter()
        model.forward(x, y)
        model.backward()
        model.update(step + 1, 1e-4, 0.0)
        loss = model.read_loss()
        ms.append((time.perf_counter() - t0) * 1e3)
        print(f"step {step + 1}/{steps} loss {loss:.6f} {ms[-1]:.1f} ms", flush=True)
    tail = sorted(ms[3:])
    print(f"config 1 (124M fp32 CPU, B=4 T=64, {torch.get_num_threads()} threads): median {tail[len(tail) // 2]:.1f} ms/step, "
          f"{4 * 64 / (tail[len(tail) // 2] / 1e3):.0f} tok/s")


if __name__ == "__main__":
    time_config1()
