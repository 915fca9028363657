"""Whole-model gate on the GPU: bf16 kernels vs the fp32 autograd oracle (logits, loss, all 16
gradient tensors) and a 10-step loss trajectory (test_gpt2.mojo:218-715 in the reference)."""
import pytest
import torch

from llm_mojo_b200.config import GPT2Config
from llm_mojo_b200.models import GPT2
from llm_mojo_b200.models import reference as ref
from llm_mojo_b200.ops import _lib

pytestmark = pytest.mark.gpu


def _cfg():
    return GPT2Config(max_seq_len=256, vocab_size=1000, num_layer=3, num_heads=4, channels=256, padded_vocab_size=1024)


def _batch(cfg, B, T, seed=0):
    g = torch.Generator().manual_seed(seed)
    x = torch.randint(0, cfg.vocab_size, (B, T + 1), generator=g, dtype=torch.int32)
    return x[:, :-1].contiguous(), x[:, 1:].contiguous()


def test_gradients_match_fp32_oracle():
    cfg = _cfg()
    model = GPT2(cfg, "bf16", "cuda")
    x, y = _batch(cfg, 4, 256)
    model.forward(x, y)
    loss = model.read_loss()
    model.backward()
    torch.cuda.synchronize()
    assert _lib.read_status() == 0
    flat = model.params.float().cpu()
    rloss, rlogits, rgrad = ref.loss_and_grads(cfg, flat, x, y)
    assert abs(loss - rloss) < 2e-2, (loss, rloss)
    for name, gv in model.g.items():
        a, b = gv.float().cpu().flatten(), rgrad[slice(*model.tensor_range(name))]
        cos = torch.nn.functional.cosine_similarity(a, b, dim=0).item()
        rel = ((a - b).norm() / (b.norm() + 1e-12)).item()
        assert cos > 0.99 and rel < 0.1, f"{name}: cosine {cos:.4f}, rel L2 {rel:.4f}"


def test_ten_step_loss_trajectory():
    cfg = _cfg()
    model = GPT2(cfg, "bf16", "cuda")
    cpu = GPT2(cfg, "fp32", "cpu", params_flat=model.params.float().cpu())
    x, y = _batch(cfg, 4, 128, seed=1)
    for step in range(1, 11):
        for mdl in (model, cpu):
            mdl.forward(x, y)
            mdl.backward()
            norm = mdl.calculate_grad_norm()
            mdl.update(step, lr=1e-3, weight_decay=0.01, dev_scale=mdl.clip_scale_from_norm(norm))
        lg, lc = model.read_loss(), cpu.read_loss()
        assert abs(lg - lc) < 0.05, (step, lg, lc)
    assert lg < 6.0


def test_chunked_ce_matches_full_logits_on_gpu():
    cfg = GPT2Config(max_seq_len=128, vocab_size=1000, num_layer=2, num_heads=2, channels=128, padded_vocab_size=1024)
    x, y = _batch(cfg, 4, 128, seed=2)
    a = GPT2(cfg, "bf16", "cuda")
    b = GPT2(cfg, "bf16", "cuda", lm_head_chunks=3)          # 3 tiles of 384: the last one is narrower
    for mdl in (a, b):
        mdl.forward(x, y)
        mdl.backward()
    torch.cuda.synchronize()
    assert _lib.read_status() == 0
    assert abs(a.read_loss() - b.read_loss()) < 5e-3
    for name in a.g:
        ga, gb = a.g[name].flatten(), b.g[name].flatten()
        assert torch.nn.functional.cosine_similarity(ga, gb, dim=0).item() > 0.995, name
    assert b.activation_bytes() < a.activation_bytes()


def test_fp32_storage_model_on_gpu_uses_tf32_path():
    cfg = GPT2Config(max_seq_len=128, vocab_size=1000, num_layer=2, num_heads=2, channels=128, padded_vocab_size=1024)
    x, y = _batch(cfg, 2, 128, seed=3)
    model = GPT2(cfg, "tf32", "cuda")
    model.forward(x, y)
    loss = model.read_loss()
    model.backward()
    torch.cuda.synchronize()
    assert _lib.read_status() == 0
    rloss, _, rgrad = ref.loss_and_grads(cfg, model.params.cpu(), x, y)
    assert abs(loss - rloss) < 5e-3
    cos = torch.nn.functional.cosine_similarity(model.grads.cpu(), rgrad, dim=0).item()
    assert cos > 0.999, cos
