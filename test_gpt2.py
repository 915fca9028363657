#!/usr/bin/env python
"""test_gpt2 — end-to-end check against a debug-state file (llm.c style).

Parity: ``test_gpt2.mojo:218-715``: load ``gpt2_124M.bin`` (or a descriptor) and
``gpt2_124M_debug_state.bin`` (256×int32 header: magic 20240520, version 3, ``[2]``=B, ``[3]``=T; then
x, y int32 ``[B,T]``, logits fp32 ``[B,T,V]``, loss fp32, the 16 gradient tensors fp32 in llm.c order with
``dwte`` padded to Vp; ``train_gpt2.py:1580-1627``), compare logits, loss and every gradient tensor
(``check_tensor``: ``|a-b| <= atol + rtol·maxabs`` and a relative-L2 test), then run 10 AdamW steps
(lr 1e-4, wd 0.01) and compare the loss trajectory.

``--write`` produces the two files from the fp32 autograd oracle of this repository (the role
``train_gpt2.py`` plays for the reference), so the check can run without any download:

    python test_gpt2.py --write --model d6 -b 4 -t 64
    python test_gpt2.py --model-file gpt2_d6.bin --state gpt2_d6_debug_state.bin
"""
from __future__ import annotations

import argparse
import struct
import sys

import numpy as np
import torch

from llm_mojo_b200.config import MODEL_MAGIC, PARAM_NAMES, parse_model_descriptor
from llm_mojo_b200.models import GPT2, random_init_params
from llm_mojo_b200.models import reference as ref
from llm_mojo_b200.utils.checkpointing import read_model_checkpoint, write_model_checkpoint

STATE_VERSION = 3
NUM_STEPS = 10


def write_debug_state(path, config, flat, x, y, steps=NUM_STEPS):
    """Forward/backward with autograd, write the state file; returns the expected 10-step losses."""
    loss, logits, grad = ref.loss_and_grads(config, flat, x, y)
    header = np.zeros(256, dtype=np.int32)
    header[0], header[1], header[2], header[3] = MODEL_MAGIC, STATE_VERSION, x.shape[0], x.shape[1]
    # expected loss trajectory with torch AdamW (betas 0.9/0.999, eps 1e-8, lr 1e-4, wd 0.01 on every tensor)
    leaf = flat.clone().float().requires_grad_(True)
    opt = torch.optim.AdamW([leaf], lr=1e-4, betas=(0.9, 0.999), eps=1e-8, weight_decay=0.01)
    losses = []
    for _ in range(steps):
        opt.zero_grad()
        _, l = ref.forward(config, ref.unflatten(config, leaf), x, y)
        l.backward()
        opt.step()
        losses.append(float(l.detach()))
    header[8] = steps
    with open(path, "wb") as f:
        f.write(header.tobytes())
        f.write(x.numpy().astype(np.int32).tobytes())
        f.write(y.numpy().astype(np.int32).tobytes())
        f.write(logits[..., :config.vocab_size].contiguous().float().numpy().tobytes())
        f.write(np.float32(loss).tobytes())
        f.write(grad.float().numpy().tobytes())
        f.write(np.asarray(losses, dtype=np.float32).tobytes())     # extension: expected loss trajectory
    return losses


def read_debug_state(path, config):
    with open(path, "rb") as f:
        header = struct.unpack("<256i", f.read(1024))
        if header[0] != MODEL_MAGIC:
            raise ValueError("Bad magic in debug state file")
        if header[1] != STATE_VERSION:
            raise ValueError(f"Bad version in debug state file: {header[1]}")
        B, T, V, P = header[2], header[3], config.vocab_size, config.num_parameters()
        x = torch.from_numpy(np.frombuffer(f.read(B * T * 4), dtype=np.int32).copy()).view(B, T)
        y = torch.from_numpy(np.frombuffer(f.read(B * T * 4), dtype=np.int32).copy()).view(B, T)
        logits = torch.from_numpy(np.frombuffer(f.read(B * T * V * 4), dtype=np.float32).copy()).view(B, T, V)
        loss = float(np.frombuffer(f.read(4), dtype=np.float32)[0])
        grads = torch.from_numpy(np.frombuffer(f.read(P * 4), dtype=np.float32).copy())
        rest = f.read(header[8] * 4) if header[8] > 0 else b""
        losses = np.frombuffer(rest, dtype=np.float32).tolist() if len(rest) == header[8] * 4 else []
    return x, y, logits, loss, grads, losses


def check_tensor(a, b, name, atol, rtol, l2_tol) -> bool:
    a, b = a.detach().float().cpu().flatten(), b.detach().float().cpu().flatten()
    maxabs = b.abs().max().item()
    err = (a - b).abs().max().item()
    rel_l2 = ((a - b).norm() / (b.norm() + 1e-30)).item()
    ok = err <= atol + rtol * maxabs and rel_l2 <= l2_tol
    print(f"{'OK ' if ok else 'NOT OK'} {name:10s} max|diff| {err:.3e} (maxabs {maxabs:.3e}) relL2 {rel_l2:.3e}")
    return ok


def run_test(model_file, state_file, device, precision) -> bool:
    config, _, flat = read_model_checkpoint(model_file, dtype=torch.float32)
    x, y, exp_logits, exp_loss, exp_grads, exp_losses = read_debug_state(state_file, config)
    model = GPT2(config, precision, device, params_flat=flat)
    lowp = precision != "fp32"
    atol, rtol, l2 = (5e-2, 5e-2, 8e-2) if lowp else (1e-4, 1e-3, 1e-3)
    print(f"[State] batch_size: {x.shape[0]} seq_len: {x.shape[1]} precision: {precision} device: {device}")
    model.forward(x, None)
    ok = check_tensor(model.acts["logits"][..., :config.vocab_size], exp_logits, "logits", atol * 20 if lowp else 1e-3, rtol, l2)
    model.forward(x, y)
    loss = model.read_loss()
    good = abs(loss - exp_loss) < (2e-2 if lowp else 1e-4)
    print(f"{'OK ' if good else 'NOT OK'} loss {loss:.6f} expected {exp_loss:.6f}")
    ok &= good
    model.backward()
    for name in PARAM_NAMES:
        b, e = model.tensor_range(name)
        ok &= check_tensor(model.g[name], exp_grads[b:e], "d" + name, atol, rtol, l2 if name not in ("ln1b", "ln2b", "lnfb", "qkvb") else 4 * l2)
    tol = 0.05 if lowp else 0.01          # bf16 storage drifts over 10 steps on one batch
    for step in range(len(exp_losses)):
        model.forward(x, y)
        model.backward()
        model.update(step + 1, 1e-4, 0.01)
        l = model.read_loss()
        good = abs(l - exp_losses[step]) < tol
        print(f"{'OK ' if good else 'NOT OK'} step {step}: loss {l:.6f} expected {exp_losses[step]:.6f}")
        ok &= good
    print("overall okay:", int(ok))
    return ok


def main(argv=None) -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--write", action="store_true")
    ap.add_argument("--model", default="d12", help="descriptor used by --write")
    ap.add_argument("--model-file", default="")
    ap.add_argument("--state", default="")
    ap.add_argument("-b", type=int, default=4)
    ap.add_argument("-t", type=int, default=64)
    ap.add_argument("--device", default="")
    ap.add_argument("--precision", default="")
    a = ap.parse_args(argv)
    tag = a.model.replace(":", "_")
    model_file = a.model_file or f"gpt2_{tag}.bin"
    state_file = a.state or f"gpt2_{tag}_debug_state.bin"
    if a.write:
        cfg = parse_model_descriptor(a.model)
        flat = random_init_params(cfg)
        g = torch.Generator().manual_seed(7)
        toks = torch.randint(0, cfg.vocab_size, (a.b, a.t + 1), generator=g, dtype=torch.int32)
        write_model_checkpoint(model_file, cfg, flat, 3)
        write_model_checkpoint(model_file.replace(".bin", "_bf16.bin"), cfg, flat.bfloat16(), 5)
        losses = write_debug_state(state_file, cfg, flat, toks[:, :-1].contiguous(), toks[:, 1:].contiguous())
        print(f"wrote {model_file}, {state_file}; expected losses {['%.4f' % l for l in losses]}")
        return 0
    dev = a.device or ("cuda" if torch.cuda.is_available() else "cpu")
    prec = a.precision or ("bf16" if dev.startswith("cuda") else "fp32")
    return 0 if run_test(model_file, state_file, dev, prec) else 1


if __name__ == "__main__":
    sys.exit(main())
