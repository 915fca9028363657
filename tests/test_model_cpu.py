"""Whole-model gate on CPU: explicit forward/backward vs autograd, and a short loss trajectory
(the role of test_gpt2.mojo:218-715 in the reference)."""
import torch

from llm_mojo_b200.config import GPT2Config
from llm_mojo_b200.models import GPT2
from llm_mojo_b200.models import reference as ref


def _batch(cfg, B, T, seed=0):
    g = torch.Generator().manual_seed(seed)
    x = torch.randint(0, cfg.vocab_size, (B, T + 1), generator=g, dtype=torch.int32)
    return x[:, :-1].contiguous(), x[:, 1:].contiguous()


def check_tensor(a, b, atol, rtol, name):
    a, b = a.float().flatten(), b.float().flatten()
    maxabs = b.abs().max().item()
    err = (a - b).abs().max().item()
    assert err <= atol + rtol * maxabs, f"{name}: max err {err} vs maxabs {maxabs}"
    denom = b.norm().item()
    if denom > 0:
        assert (a - b).norm().item() / denom < 1e-3, f"{name}: relative L2 too large"


def test_forward_backward_matches_autograd(tiny_config):
    cfg = tiny_config
    model = GPT2(cfg, "fp32", "cpu")
    x, y = _batch(cfg, 2, 8)
    model.forward(x, y)
    loss = model.read_loss()
    model.backward()
    rloss, rlogits, rgrad = ref.loss_and_grads(cfg, model.params, x, y)
    assert abs(loss - rloss) < 1e-5
    for name, gv in model.g.items():
        off0, off1 = model.tensor_range(name)
        check_tensor(gv, rgrad[off0:off1], 1e-6, 1e-4, name)


def test_grad_accumulation_equals_big_batch(tiny_config):
    cfg = tiny_config
    x, y = _batch(cfg, 4, 8, seed=1)
    big = GPT2(cfg, "fp32", "cpu")
    big.forward(x, y)
    big.backward()
    acc = GPT2(cfg, "fp32", "cpu")
    for i in range(2):
        acc.forward(x[2 * i:2 * i + 2], y[2 * i:2 * i + 2], grad_accum_steps=2)
        acc.backward(grad_accum_steps=2, micro_step=i)
    assert abs(big.read_loss() - acc.read_loss()) < 1e-5
    assert torch.allclose(big.grads, acc.grads, atol=1e-6, rtol=1e-4)


def test_loss_decreases_and_matches_torch_adamw(tiny_config):
    cfg = tiny_config
    model = GPT2(cfg, "fp32", "cpu")
    leaf = model.params.clone().requires_grad_(True)
    opt = torch.optim.AdamW([leaf], lr=1e-2, betas=(0.9, 0.999), eps=1e-8, weight_decay=0.01)
    x, y = _batch(cfg, 2, 8, seed=2)
    losses = []
    for step in range(1, 11):
        model.forward(x, y)
        losses.append(model.read_loss())
        model.backward()
        model.update(step, lr=1e-2, weight_decay=0.01)
        opt.zero_grad()
        _, rl = ref.forward(cfg, ref.unflatten(cfg, leaf), x, y)
        rl.backward()
        opt.step()
        assert abs(losses[-1] - float(rl)) < 2e-4, (step, losses[-1], float(rl))
    assert losses[-1] < losses[0]


def test_recompute_matches(tiny_config):
    cfg = tiny_config
    x, y = _batch(cfg, 2, 8, seed=3)
    a = GPT2(cfg, "fp32", "cpu")
    b = GPT2(cfg, "fp32", "cpu", recompute=True)
    for mdl in (a, b):
        mdl.forward(x, y)
        mdl.backward()
    assert torch.allclose(a.grads, b.grads, atol=1e-7)


def test_random_init_statistics():
    cfg = GPT2Config(max_seq_len=32, vocab_size=100, num_layer=4, num_heads=2, channels=32, padded_vocab_size=128)
    model = GPT2(cfg, "fp32", "cpu")
    p = model.p
    assert torch.all(p["ln1w"] == 1) and torch.all(p["lnfb"] == 0) and torch.all(p["qkvb"] == 0)
    assert torch.all(p["wte"][cfg.vocab_size:] == 0)            # padded rows stay zero
    assert abs(p["qkvw"].std().item() - 0.02) < 2e-3
    assert abs(p["fcprojw"].std().item() - 0.02 / (2 * 4) ** 0.5) < 1e-3


def test_chunked_ce_and_lm_head_tiling_match_untiled(tiny_config):
    """Vocabulary-tiled LM head with two-pass chunked cross-entropy against the single-GEMM path
    (tests/test_chunked_cross_entropy.mojo, tests/test_lm_head_vocab_tiling.mojo)."""
    from llm_mojo_b200.config import GPT2Config
    cfg = GPT2Config(max_seq_len=16, vocab_size=300, num_layer=1, num_heads=2, channels=16, padded_vocab_size=384)
    x, y = _batch(cfg, 2, 8, seed=4)
    a = GPT2(cfg, "fp32", "cpu")
    b = GPT2(cfg, "fp32", "cpu", lm_head_chunks=3)
    for mdl in (a, b):
        mdl.forward(x, y)
        mdl.backward()
    assert "logits" not in b.acts and b.acts["logits_tile"].shape[1] == 128
    assert abs(a.read_loss() - b.read_loss()) < 1e-6
    assert torch.allclose(a.grads, b.grads, atol=1e-6, rtol=1e-4)


def test_debug_nan_scan_cpu():
    """The per-tensor census reports exactly the tensors that hold non-finite values."""
    from llm_mojo_b200 import ops
    from llm_mojo_b200.config import GPT2Config
    from llm_mojo_b200.models import GPT2
    cfg = GPT2Config(max_seq_len=16, vocab_size=64, padded_vocab_size=128, num_layer=1, num_heads=2, channels=16)
    m = GPT2(cfg, "fp32", "cpu")
    assert m.debug_nan_scan("params") == {}
    m.g["wpe"].view(-1)[3] = float("nan")
    m.g["lnfw"].view(-1)[0] = float("inf")
    m.g["lnfw"].view(-1)[1] = float("-inf")
    assert m.debug_nan_scan("grads") == {"wpe": (1, 0), "lnfw": (0, 2)}
    assert ops.nan_census(torch.tensor([1.0, float("nan"), float("inf")])) == (1, 1)


def test_unfused_softmax_and_crossentropy_match_autograd():
    """softmax backward and the unfused cross-entropy pair against autograd (the reference's stand-alone ops,
    llmm/softmax.mojo:632 and llmm/crossentropy.mojo:110 / :284)."""
    import torch
    from llm_mojo_b200 import ops
    g = torch.Generator().manual_seed(3)
    rows, V, ld = 6, 37, 40
    logits = torch.randn(rows, ld, generator=g, requires_grad=True)
    tgt = torch.randint(0, V, (rows,), generator=g, dtype=torch.int32)
    probs_v = torch.softmax(logits[:, :V], dim=-1)
    losses = -torch.log(probs_v.gather(1, tgt.long().view(-1, 1))).squeeze(1)
    dloss = torch.randn(rows, generator=g)
    (losses * dloss).sum().backward()
    probs = torch.zeros(rows, ld)
    probs[:, :V] = probs_v.detach()
    assert torch.allclose(ops.softmax_rows(logits.detach(), V), probs[:, :V], atol=1e-6)
    assert torch.allclose(ops.crossentropy_fwd(probs, tgt), losses.detach(), atol=1e-6)
    dprobs = torch.zeros(rows, ld)
    ops.crossentropy_bwd(dprobs, dloss, probs, tgt)
    dlogits = ops.softmax_bwd(dprobs, probs, V)
    assert torch.allclose(dlogits, logits.grad, atol=1e-5)
    assert torch.all(dlogits[:, V:] == 0)
