#!/usr/bin/env python
"""infer_gpt2 — text generation and HellaSwag-style evaluation from a checkpoint.

Parity: ``infer_gpt2.mojo:56-144`` (``run_infer``: warm-up forward, then one full forward per
generated token, last-position logits → softmax → CDF sampling → tokenizer decode),
``:147-190`` (``run_eval``: batches of 4 completions, accuracy by lowest masked mean loss),
``:193-278`` (modes: ``.bin`` / ``.safetensors`` / ``--hf <repo>`` / ``--eval <file>``).

    python infer_gpt2.py gpt2_124M.bin --prompt-tokens 50256 --tokens 64
    python infer_gpt2.py d12 --eval hellaswag_val.bin -b 16
"""
from __future__ import annotations

import argparse
import sys
import time

import torch

from llm_mojo_b200.models import GPT2
from llm_mojo_b200 import ops
from llm_mojo_b200.utils.eval_dataloader import EvalDataLoader, eval_stat_correct
from llm_mojo_b200.utils.sampler import SamplerRNG, sample_softmax
from llm_mojo_b200.utils.tokenizer import Tokenizer


def pick_device(arg: str) -> torch.device:
    if arg:
        return torch.device(arg)
    return torch.device("cuda" if torch.cuda.is_available() else "cpu")


def run_infer(model: GPT2, tokenizer: Tokenizer, prompt, gen_tokens: int, seed: int, temperature: float = 1.0,
              out=sys.stdout) -> list:
    cfg = model.config
    T = min(cfg.max_seq_len, max(64, len(prompt) + gen_tokens))
    T = (T + 7) // 8 * 8
    pad = tokenizer.eot_token if tokenizer.has_initialized else 50256
    toks = torch.full((1, T), min(pad, cfg.vocab_size - 1), dtype=torch.int32)      # filler beyond the prompt (never attended to)
    toks[0, :len(prompt)] = torch.tensor(prompt, dtype=torch.int32)
    rng = SamplerRNG(seed)
    model.forward(toks, None, B=1, T=T)                    # warm-up: allocates activations for this shape
    generated = []
    t0 = time.perf_counter()
    for t in range(len(prompt), min(T, len(prompt) + gen_tokens)):
        model.forward(toks, None, B=1, T=T)
        row = model.acts["logits"][0, t - 1:t]
        probs = ops.softmax_rows(row.reshape(1, -1), cfg.vocab_size, temperature)[0].float().cpu()
        coin = rng.random_f32()
        cdf = torch.cumsum(probs, 0)
        nxt = int(min(int(torch.searchsorted(cdf, torch.tensor(coin), right=True)), cfg.vocab_size - 1))
        toks[0, t] = nxt
        generated.append(nxt)
        piece = tokenizer.decode(nxt) if tokenizer.has_initialized else f"{nxt} "
        out.write(piece)
        out.flush()
    dt = time.perf_counter() - t0
    out.write(f"\n---\n{len(generated)} tokens in {dt:.2f} s ({len(generated) / max(dt, 1e-9):.1f} tok/s)\n")
    return generated


def run_eval(model: GPT2, path: str, B: int, T: int) -> float:
    loader = EvalDataLoader(path, B, T)
    correct = 0
    for _ in range(loader.num_batches):
        loader.next_batch()
        model.forward(loader.inputs, loader.targets, B=B, T=T)
        model.read_loss()
        correct += eval_stat_correct(loader, model.acts["losses"])
    total = loader.end_example_index - loader.start_example_index
    acc = correct / max(total, 1)
    print(f"HellaSwag: {correct}/{total} = {acc:.4f}")
    return acc


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("checkpoint", nargs="?", default="gpt2_124M.bin", help=".bin, .safetensors or model descriptor (dX)")
    ap.add_argument("--hf", default="", help="Hugging Face repo id to download (model.safetensors)")
    ap.add_argument("--eval", default="", help="evaluation file in the llm.c eval format (HellaSwag)")
    ap.add_argument("--tokenizer", default="gpt2_tokenizer.bin")
    ap.add_argument("--prompt-tokens", default="", help="comma-separated token ids (default: end-of-text)")
    ap.add_argument("--tokens", type=int, default=64)
    ap.add_argument("--temperature", type=float, default=1.0)
    ap.add_argument("--seed", type=int, default=1337)
    ap.add_argument("-b", type=int, default=16)
    ap.add_argument("-t", type=int, default=1024)
    ap.add_argument("--device", default="")
    args = ap.parse_args(argv)
    dev = pick_device(args.device)
    src = args.checkpoint
    if args.hf:
        from llm_mojo_b200.utils.safetensors_io import fetch_hf_checkpoint
        src = fetch_hf_checkpoint(args.hf)
    model = GPT2(src, "bf16" if dev.type == "cuda" else "fp32", dev)
    if args.eval:
        run_eval(model, args.eval, args.b, min(args.t, model.config.max_seq_len))
        return 0
    tok = Tokenizer(args.tokenizer)
    prompt = [int(x) for x in args.prompt_tokens.split(",")] if args.prompt_tokens else [tok.eot_token]
    run_infer(model, tok, prompt, args.tokens, args.seed, args.temperature)
    return 0


if __name__ == "__main__":
    sys.exit(main())
