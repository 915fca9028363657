"""Low-precision training support: amax / delayed scaling, FP8 and NVFP4 quantisation, Hadamard,
stochastic rounding, low-precision GEMMs against a bf16 control, and the cross-precision gradient
gate (after tests/test_amax.mojo, test_nvfp4_quant.mojo, test_hadamard.mojo, test_lowp_gemm*.mojo,
test_lowp_bwd.mojo and tests/compare_grad_dumps.py:49-55 of the reference)."""
import math

import pytest
import torch

from llm_mojo_b200.config import GPT2Config, Precision
from llm_mojo_b200.models import GPT2
from llm_mojo_b200.ops import lowp

CFG = GPT2Config(max_seq_len=32, vocab_size=60, num_layer=6, num_heads=2, channels=32, padded_vocab_size=64)
CFG_BLOCK = GPT2Config(max_seq_len=64, vocab_size=120, num_layer=3, num_heads=2, channels=128, padded_vocab_size=128)


class _Fp32Storage(Precision):
    """Low-precision GEMM numerics on fp32 storage so the emulation runs on CPU."""
    @property
    def storage(self):
        return torch.float32


def _batch(B=2, T=32, seed=0):
    g = torch.Generator().manual_seed(seed)
    t = torch.randint(0, CFG.vocab_size, (B, T + 1), generator=g, dtype=torch.int32)
    return t[:, :-1].contiguous(), t[:, 1:].contiguous()


# ------------------------------------------------------------------------------ CPU
def test_delayed_scaling_uses_prior_steps_only():
    st = lowp.AmaxState("cpu", lowp.E4M3)
    amaxes = [float(i + 1) for i in range(lowp.AMAX_HISTORY + 4)]
    for step, a in enumerate(amaxes):
        st.update_scale(torch.tensor([a, -a / 2]))
        if step < lowp.AMAX_HISTORY:                      # warm-up: the step's own amax
            assert abs(float(st.scale) - 448.0 / a) < 1e-4
        else:                                             # steady state: max of the previous 16, never its own
            prev = max(amaxes[step - lowp.AMAX_HISTORY:step])
            assert abs(float(st.scale) - 448.0 / prev) < 1e-4
        assert abs(float(st.scale) * float(st.scale_inv) - 1) < 1e-6


def test_amax_is_nan_infectious_and_zero_safe():
    out = torch.zeros(1)
    lowp.compute_amax(out, torch.tensor([1.0, float("nan"), -3.0]))
    assert math.isnan(float(out))
    st = lowp.AmaxState("cpu")
    st.update_scale(torch.zeros(8))
    assert float(st.scale) == 1.0


def test_hadamard_is_orthogonal_and_invertible():
    x = torch.randn(8, 64)
    h = lowp.hadamard16(x)
    assert torch.allclose(lowp.hadamard16(h, inverse=True), x, atol=1e-5)
    assert torch.allclose(h.reshape(-1, 16).norm(dim=1), 4.0 * x.reshape(-1, 16).norm(dim=1), rtol=1e-5)


def test_nvfp4_values_lie_on_the_grid_and_error_is_bounded():
    torch.manual_seed(0)
    x = torch.randn(64, 128)
    deq, ts = lowp.nvfp4_fake_quant(x)
    blocks = deq.float().reshape(64, 8, 16)
    grid = (0.5, 1, 1.5, 2, 3, 4, 6)                      # e2m1 magnitudes; the block's smallest value may be any of them
    allowed = sorted({a / b for a in grid for b in grid if a >= b})
    for b in blocks.reshape(-1, 16)[:50]:
        nz = b[b != 0].abs()
        if nz.numel():
            ratios = nz / nz.min()
            assert all(any(abs(r - g) < 1e-3 for g in allowed) for r in ratios.tolist())
    rel = ((deq.float() * ts - x).norm() / x.norm()).item()
    assert rel < 0.15
    deq16, ts16 = lowp.nvfp4_fake_quant(x, block_rows=16)
    assert ((deq16.float() * ts16 - x).norm() / x.norm()).item() < 0.2


def test_nvfp4_stochastic_rounding_is_unbiased():
    x = torch.full((256, 64), 0.7)          # between grid points after scaling
    x[:, 0] = 6.0                           # fixes the block scale
    acc = torch.zeros_like(x)
    n = 64
    for s in range(n):
        deq, ts = lowp.nvfp4_fake_quant(x, sr=True, seed=11, step=s)
        acc += deq.float() * ts
    assert abs((acc / n)[:, 1:].mean().item() - 0.7) < 0.01
    det, ts = lowp.nvfp4_fake_quant(x)
    assert abs((det.float() * ts)[:, 1:].mean().item() - 0.7) > 0.02       # RNE alone is biased here


def test_fp8_block_scales_are_powers_of_two_and_values_lie_on_the_fp8_grid():
    torch.manual_seed(1)
    x = torch.randn(256, 384) * torch.logspace(-3, 3, 384)          # wide dynamic range across the columns
    for mode in (0, 1, 2):
        for fmt, dt in ((lowp.E4M3, torch.float8_e4m3fn), (lowp.E5M2, torch.float8_e5m2)):
            q = lowp.fp8_block_fake_quant(x, mode, fmt)
            # re-quantising is the identity: every value is scale x an fp8 number with the block's own scale
            assert torch.equal(lowp.fp8_block_fake_quant(q, mode, fmt), q)
            rel = ((q - x).norm() / x.norm()).item()
            assert rel < (0.04 if fmt == lowp.E4M3 else 0.08), (mode, fmt, rel)
            assert torch.equal(q.bfloat16().float(), q)               # exactly representable in bf16
    # a per-tensor scale loses the small columns entirely; block scales keep them
    small = x[:, :64]
    per_tensor = (x / (x.abs().max() / 448)).to(torch.float8_e4m3fn).float() * (x.abs().max() / 448)
    assert (per_tensor[:, :64] == 0).float().mean() > 0.5
    assert ((lowp.fp8_block_fake_quant(x, 0)[:, :64] - small).norm() / small.norm()).item() < 0.04


@pytest.mark.parametrize("name,floor", [("fp8", 0.99), ("fp8b", 0.99), ("fp4", 0.93)])
def test_cross_precision_gradient_gate(name, floor):
    """Per-tensor cosine / relative-L2 of the low-precision gradients against the full-precision build."""
    cfg = CFG_BLOCK if name == "fp8b" else CFG               # block scaling needs dimensions that are multiples of 128
    g = torch.Generator().manual_seed(0)
    t = torch.randint(0, cfg.vocab_size, (2, cfg.max_seq_len + 1), generator=g, dtype=torch.int32)
    x, y = t[:, :-1].contiguous(), t[:, 1:].contiguous()
    ref = GPT2(cfg, "fp32", "cpu")
    ref.forward(x, y); ref.backward()
    m = GPT2(cfg, _Fp32Storage(name), "cpu")
    m.forward(x, y); m.backward()
    if name == "fp8b":
        assert m._site_mode("qkv", 0) == "fp8b" and m._site_mode("fcproj", 2) == "fp8b"
    assert abs(m.read_loss() - ref.read_loss()) < 0.02
    rels = []
    for n_, g in m.g.items():
        a, b = g.flatten(), ref.g[n_].flatten()
        if b.norm() == 0:
            continue
        cos = torch.nn.functional.cosine_similarity(a, b, dim=0).item()
        rels.append(((a - b).norm() / b.norm()).item())
        assert cos > floor, (n_, cos)
        assert torch.isfinite(a).all() and a.abs().sum() > 0
    rels.sort()
    assert rels[len(rels) // 2] < 0.20 and rels[-1] < 0.50


def test_fp4_layer_range_matches_reference_policy():
    pr = Precision("fp4")
    L = 12
    assert [l for l in range(L) if pr.layer_in_fp4_range(l, L)] == list(range(2, 10))
    m = GPT2(CFG, _Fp32Storage("fp4"), "cpu")
    assert m._site_mode("fc", 0) == "bf16" and m._site_mode("fc", 2) == "fp4" and m._site_mode("qkv", 2) == "bf16"


# ------------------------------------------------------------------------------ GPU
def test_native_path_switches_and_split_k_choice(monkeypatch):
    from llm_mojo_b200 import ops
    monkeypatch.delenv("LLMM_FP4_NATIVE", raising=False)
    assert lowp.nvfp4_native(768, 65536) and not lowp.nvfp4_native(768, 1000)      # 16-byte rows of packed values
    monkeypatch.setenv("LLMM_FP4_NATIVE", "0")
    assert not lowp.nvfp4_native(768)
    monkeypatch.delenv("LLMM_FP8B_NATIVE", raising=False)
    assert lowp.fp8_block_native()
    monkeypatch.setenv("LLMM_FP8B_NATIVE", "0")
    assert not lowp.fp8_block_native()
    # wgrad of a 124M layer on 128x256 tiles: 6 x 12 = 72 tiles, two splits fill the 148 CTAs once
    assert ops._splits_for(768, 3072, 65536, tile=128, tile_n=256, bk=256, units=148) == 2
    # a 768 x 768 wgrad has 18 tiles: eight splits
    assert ops._splits_for(768, 768, 65536, tile=128, tile_n=256, bk=256, units=148) == 8
    assert 1 <= ops._splits_for(768, 768, 65536) <= 16


gpu = pytest.mark.gpu


@gpu
def test_amax_and_fp8_quantize_match_torch():
    x = (torch.randn(1024, 768) * 3).bfloat16().cuda()
    out = torch.zeros(1, device="cuda")
    lowp.compute_amax(out, x)
    assert float(out) == float(x.float().abs().max())
    x2 = x.clone(); x2[5, 5] = float("nan")
    lowp.compute_amax(out, x2)
    assert math.isnan(float(out))
    for fmt, dt in ((lowp.E4M3, torch.float8_e4m3fn), (lowp.E5M2, torch.float8_e5m2)):
        st = lowp.AmaxState("cuda", fmt)
        st.update_scale(x)
        q = torch.empty(x.shape, dtype=torch.uint8, device="cuda")
        lowp.quantize_fp8(q, x, st.scale, fmt)
        want = (x.float() * st.scale).clamp(-lowp.FMT_MAX[fmt], lowp.FMT_MAX[fmt]).to(dt).view(torch.uint8)
        assert (q != want).float().mean().item() < 1e-3
        back = lowp.dequantize_fp8(q, st.scale_inv, fmt)
        assert ((back - x.float()).norm() / x.float().norm()).item() < (0.04 if fmt == lowp.E4M3 else 0.08)


@gpu
def test_hadamard_kernel_matches_host():
    x = torch.randn(64, 256)
    assert torch.allclose(lowp.hadamard16(x.cuda()).cpu(), lowp.hadamard16(x), atol=1e-5)
    assert torch.allclose(lowp.hadamard16(lowp.hadamard16(x.cuda()), inverse=True).cpu(), x, atol=1e-5)


@gpu
def test_delayed_scaling_state_on_device_matches_host():
    dev, host = lowp.AmaxState("cuda"), lowp.AmaxState("cpu")
    g = torch.Generator().manual_seed(3)
    for _ in range(lowp.AMAX_HISTORY + 5):
        x = torch.randn(512, generator=g) * float(torch.rand(1, generator=g) * 5 + 0.1)
        dev.update_scale(x.cuda()); host.update_scale(x)
        assert abs(float(dev.scale) - float(host.scale)) / float(host.scale) < 1e-5


@gpu
@pytest.mark.parametrize("fmt", [lowp.E4M3, lowp.E5M2])
def test_single_pass_delayed_quantisation_matches_two_passes(fmt, monkeypatch):
    """Once the amax history is full, `_q` reads the tensor once (quantise with the scale from the history, amax on the way,
    push).  Scales, history and fp8 bytes must equal the two-pass order at every step, across the warm-up boundary, with a NaN
    in one step (its amax is NaN: the scale falls back to 1 while it is in the history) and with values that saturate."""
    one, two = lowp.AmaxState("cuda", fmt), lowp.AmaxState("cuda", fmt)
    g = torch.Generator().manual_seed(5)
    for step in range(lowp.AMAX_HISTORY + 24):
        x = (torch.randn(64, 1024, generator=g) * float(torch.rand(1, generator=g) * 20 + 0.05)).bfloat16().cuda()
        if step == lowp.AMAX_HISTORY + 3:
            x[5, 7] = float("nan")
        monkeypatch.setattr(lowp, "FUSED_DELAYED", True)
        q1 = lowp._q("t1", x, one).clone()
        monkeypatch.setattr(lowp, "FUSED_DELAYED", False)
        q2 = lowp._q("t2", x, two).clone()
        torch.cuda.synchronize()
        assert torch.equal(one.state.cpu().nan_to_num(-1.0), two.state.cpu().nan_to_num(-1.0)), step
        keep = ~torch.isnan(x)                      # what a NaN input encodes to is not part of the contract
        assert torch.equal(q1[keep], q2[keep]), step
    assert one.host_step == two.host_step == lowp.AMAX_HISTORY + 24


@gpu
@pytest.mark.parametrize("fmt", [lowp.E4M3, lowp.E5M2])
def test_fp8_block_dual_quantisation_equals_the_two_single_kernels(fmt):
    rows, cols = 384, 640
    x = (torch.randn(rows, cols) * torch.logspace(-3, 3, cols)).bfloat16().cuda()
    q0, s0, q1, s1 = lowp.fp8_block_quant_dual(x, fmt)
    r0, t0 = lowp.fp8_block_quant(x, 0, fmt)
    r1, t1 = lowp.fp8_block_quant(x, 1, fmt, transpose=True)
    torch.cuda.synchronize()
    assert torch.equal(q0, r0) and torch.equal(s0, t0) and torch.equal(q1, r1) and torch.equal(s1, t1)


@gpu
def test_fp8_block_linear_dual_path_is_bit_identical(monkeypatch):
    rows, C, OC = 256, 384, 512
    g = torch.Generator().manual_seed(2)
    x = torch.randn(rows, C, generator=g).bfloat16().cuda()
    w = (torch.randn(OC, C, generator=g) * 0.05).bfloat16().cuda()
    b = torch.randn(OC, generator=g).bfloat16().cuda()
    dy = torch.randn(rows, OC, generator=g).bfloat16().cuda()
    res = {}
    for on in (True, False):
        monkeypatch.setattr(lowp, "FP8B_DUAL", on)
        out = torch.empty(rows, OC, dtype=torch.bfloat16, device="cuda")
        lowp.matmul_fwd_fp8_block(out, x, w, b)
        dx, dw, db = torch.empty_like(x), torch.zeros(OC, C, device="cuda"), torch.zeros(OC, device="cuda")
        lowp.matmul_bwd_fp8_block(dx, dw, db, dy, x, w)
        torch.cuda.synchronize()
        res[on] = (out, dx, dw, db)
    for a, r in zip(res[True], res[False]):
        assert torch.equal(a, r)


@gpu
def test_fp8_linear_site_fast_path_matches_reference_order(monkeypatch):
    """A linear layer in fp8 for more steps than the amax history holds: the fast path (scales of input and weight derived in one
    launch, single-pass quantisation, forward bytes kept for the backward GEMMs, fc bias gradient in the dGELU epilogue) against the
    plain order (amax pass, scale update, quantise pass per operand and per use).  Outputs, input gradients, weight gradients and
    the scaling states must be equal at every step."""
    rows, C, OC = 512, 256, 1024
    g = torch.Generator().manual_seed(9)
    w = (torch.randn(OC, C, generator=g) * 0.05).bfloat16().cuda()
    b = torch.randn(OC, generator=g).bfloat16().cuda()
    fast, ref = lowp.LinearSite("cuda"), lowp.LinearSite("cuda")
    for step in range(lowp.AMAX_HISTORY + 6):
        x = (torch.randn(rows, C, generator=g) * (0.5 + step % 5)).bfloat16().cuda()
        dy = (torch.randn(rows, OC, generator=g) * 10.0 ** (step % 3 - 2)).bfloat16().cuda()
        res = {}
        for name, site, on in (("fast", fast, True), ("ref", ref, False)):
            monkeypatch.setattr(lowp, "FUSED_DELAYED", on)
            monkeypatch.setattr(lowp, "KEEP_OPERANDS", on)
            out, pre = torch.empty(rows, OC, dtype=torch.bfloat16, device="cuda"), torch.empty(rows, OC, dtype=torch.bfloat16, device="cuda")
            lowp.matmul_fwd_fp8(out, x, w, b, site, pre_gelu=pre)
            dx, dw, db = torch.empty_like(x), torch.zeros(OC, C, device="cuda"), torch.zeros(OC, device="cuda")
            lowp.matmul_bwd_fp8(dx, dw, db, dy, x, w, site)
            torch.cuda.synchronize()
            res[name] = (out, pre, dx, dw, db, site.inp.state.clone(), site.weight.state.clone(), site.dout.state.clone())
        for a, r in zip(res["fast"], res["ref"]):
            assert torch.equal(a, r), step
    assert fast.inp.host_step == ref.inp.host_step == lowp.AMAX_HISTORY + 6


@gpu
@pytest.mark.parametrize("axis,block_rows,rht", [(1, 1, False), (1, 16, False), (0, 1, False), (0, 1, True), (0, 16, False)])
def test_nvfp4_kernel_matches_emulation(axis, block_rows, rht):
    x = torch.randn(256, 384).bfloat16()
    d_cpu, ts_cpu = lowp.nvfp4_fake_quant(x.float(), axis=axis, block_rows=block_rows, rht=rht)
    d_gpu, ts_gpu, q, sc = lowp.nvfp4_fake_quant(x.cuda(), axis=axis, block_rows=block_rows, rht=rht, want_packed=True)
    assert abs(float(ts_gpu) - float(ts_cpu)) / float(ts_cpu) < 1e-2
    a, b = d_gpu.float().cpu() * float(ts_gpu), d_cpu.float() * float(ts_cpu)
    assert ((a - b).abs() > 1e-3 * b.abs().max()).float().mean().item() < 0.02      # rounding ties / bf16 hadamard
    # the packed bytes + swizzled scales decode to the same values
    from llm_mojo_b200.ops._lib import lib, ptr, stream, check
    outer, K = (256, 384) if axis == 1 else (384, 256)
    out = torch.empty(outer, K, device="cuda")
    check(lib().llmb_nvfp4_dequantize(ptr(out), ptr(q), ptr(sc), ptr(ts_gpu), outer, K, 1, stream()), "nvfp4_dequantize")
    want = d_gpu.float() * ts_gpu
    want = want if axis == 1 else want.t()
    assert torch.allclose(out, want, atol=1e-6, rtol=1e-5)


@gpu
def test_fp8_gemm_forward_backward_against_bf16_control():
    rows, C, OC = 512, 768, 3072
    x, w = torch.randn(rows, C).bfloat16().cuda(), (torch.randn(OC, C) * 0.02).bfloat16().cuda()
    b, d = torch.randn(OC).bfloat16().cuda(), torch.randn(rows, OC).bfloat16().cuda()
    site = lowp.LinearSite("cuda")
    out = torch.empty(rows, OC, dtype=torch.bfloat16, device="cuda")
    lowp.matmul_fwd_fp8(out, x, w, b, site)
    ref = x.float() @ w.float().t() + b.float()
    assert ((out.float() - ref).norm() / ref.norm()).item() < 0.06
    dinp, dw, db = torch.empty(rows, C, dtype=torch.bfloat16, device="cuda"), torch.zeros(OC, C, device="cuda"), torch.zeros(OC, device="cuda")
    lowp.matmul_bwd_fp8(dinp, dw, db, d, x, w, site)
    rdi, rdw = d.float() @ w.float(), d.float().t() @ x.float()
    assert ((dinp.float() - rdi).norm() / rdi.norm()).item() < 0.1
    assert ((dw - rdw).norm() / rdw.norm()).item() < 0.1
    assert torch.allclose(db, d.float().sum(0), atol=0.5, rtol=1e-2)
    from llm_mojo_b200.ops import _lib
    assert _lib.read_status() == 0


@gpu
def test_fp4_gemm_matches_emulation():
    rows, C, OC = 256, 256, 512
    x, w = torch.randn(rows, C).bfloat16(), (torch.randn(OC, C) * 0.05).bfloat16()
    out_c = torch.empty(rows, OC)
    lowp.matmul_fwd_fp4(out_c, x.float(), w.float(), None)
    out_g = torch.empty(rows, OC, dtype=torch.bfloat16, device="cuda")
    lowp.matmul_fwd_fp4(out_g, x.cuda(), w.cuda(), None)
    assert ((out_g.float().cpu() - out_c).norm() / out_c.norm()).item() < 0.03
    ref = x.float() @ w.float().t()
    assert ((out_g.float().cpu() - ref).norm() / ref.norm()).item() < 0.2


@gpu
@pytest.mark.parametrize("name,floor", [("fp8", 0.97), ("fp4", 0.93)])
def test_low_precision_model_gradients_on_gpu(name, floor):
    cfg = GPT2Config(max_seq_len=128, vocab_size=1000, num_layer=6, num_heads=2, channels=128, padded_vocab_size=1024)
    g = torch.Generator().manual_seed(0)
    t = torch.randint(0, cfg.vocab_size, (4, 129), generator=g, dtype=torch.int32)
    x, y = t[:, :-1].contiguous(), t[:, 1:].contiguous()
    ref = GPT2(cfg, "bf16", "cuda")
    lp = GPT2(cfg, name, "cuda")
    for m in (ref, lp):
        m.forward(x, y); m.backward()
    assert abs(lp.read_loss() - ref.read_loss()) < 0.05
    for n_, gv in lp.g.items():
        a, b = gv.flatten(), ref.g[n_].flatten()
        cos = torch.nn.functional.cosine_similarity(a, b, dim=0).item()
        assert cos > floor, (n_, cos)
    from llm_mojo_b200.ops import _lib
    assert _lib.read_status() == 0


@gpu
@pytest.mark.parametrize("mode", [0, 1, 2])
@pytest.mark.parametrize("fmt", [lowp.E4M3, lowp.E5M2])
def test_fp8_block_kernel_matches_emulation(mode, fmt):
    torch.manual_seed(2)
    x = (torch.randn(256, 384) * torch.logspace(-2, 2, 384)).bfloat16()
    want = lowp.fp8_block_fake_quant(x.float(), mode, fmt)
    got = lowp.fp8_block_fake_quant(x.cuda(), mode, fmt).float().cpu()
    assert torch.equal(got, want.bfloat16().float())


@gpu
def test_fp8_block_training_step_on_gpu():
    from llm_mojo_b200.config import Precision
    cfg = GPT2Config(max_seq_len=128, vocab_size=1000, num_layer=2, num_heads=2, channels=128, padded_vocab_size=1024)
    g = torch.Generator().manual_seed(0)
    t = torch.randint(0, cfg.vocab_size, (2, 129), generator=g, dtype=torch.int32)
    x, y = t[:, :-1].contiguous(), t[:, 1:].contiguous()
    ref = GPT2(cfg, "bf16", "cuda")
    m = GPT2(cfg, Precision("fp8b"), "cuda")
    assert m._site_mode("fc", 1) == "fp8b"
    losses = []
    for model in (ref, m):
        model.forward(x, y); model.backward()
        losses.append(model.read_loss())
    assert abs(losses[0] - losses[1]) < 0.05
    for n_ in ("qkvw", "fcw", "fcprojw", "wte"):
        a, b = m.g[n_].flatten().float(), ref.g[n_].flatten().float()
        assert torch.nn.functional.cosine_similarity(a, b, dim=0).item() > 0.98, n_


def _nvfp4_operands(M, N, K, seed=0):
    g = torch.Generator().manual_seed(seed)
    a = (torch.randn(M, K, generator=g) * (1 + torch.arange(K) % 7)).bfloat16().cuda()
    b = (torch.randn(N, K, generator=g) * 0.05).bfloat16().cuda()
    da, tsa, qa, sa = lowp.nvfp4_fake_quant(a, axis=1, block_rows=1, want_packed=True)
    db, tsb, qb, sb = lowp.nvfp4_fake_quant(b, axis=1, block_rows=16 if N % 16 == 0 else 1, want_packed=True)
    return da, qa, sa, db, qb, sb, tsa * tsb


@gpu
@pytest.mark.parametrize("M,N,K", [(256, 384, 512), (200, 136, 1600), (128, 128, 64), (1024, 768, 3072)])
def test_native_nvfp4_gemm_matches_fp32_product_of_dequantised_operands(M, N, K):
    """tcgen05 kind::mxf4nvf4 on the packed operands == fp32 product of (value x block scale) x tensor scales."""
    from llm_mojo_b200 import ops
    da, qa, sa, db, qb, sb, alpha = _nvfp4_operands(M, N, K)
    want = (da.float() @ db.float().t()) * alpha
    out = torch.empty(M, N, dtype=torch.bfloat16, device="cuda")
    ops.gemm_nvfp4(out, qa, sa, qb, sb, K, alpha=alpha)
    torch.cuda.synchronize()
    err = (out.float() - want).norm() / want.norm()
    assert err.item() < 4e-3, err.item()
    # fp32 store: only the accumulation order differs
    out32 = torch.empty(M, N, dtype=torch.float32, device="cuda")
    ops.gemm_nvfp4(out32, qa, sa, qb, sb, K, epi=ops.EPI_STORE_F32, alpha=alpha)
    assert ((out32 - want).norm() / want.norm()).item() < 1e-5


@gpu
def test_native_nvfp4_gemm_epilogues_and_split_k():
    from llm_mojo_b200 import ops
    M, N, K = 384, 256, 8192
    da, qa, sa, db, qb, sb, alpha = _nvfp4_operands(M, N, K, seed=1)
    base = (da.float() @ db.float().t()) * alpha
    bias = torch.randn(N, device="cuda").bfloat16()
    res = torch.randn(M, N, device="cuda").bfloat16()
    out = torch.empty(M, N, dtype=torch.bfloat16, device="cuda")
    pre = torch.empty_like(out)
    ops.gemm_nvfp4(out, qa, sa, qb, sb, K, epi=ops.EPI_BIAS_GELU, bias=bias, aux=pre, alpha=alpha)
    want_pre = (base + bias.float()).bfloat16()
    assert ((pre.float() - want_pre.float()).norm() / want_pre.float().norm()).item() < 4e-3
    want = torch.nn.functional.gelu(pre.float(), approximate="tanh")
    assert ((out.float() - want).norm() / want.norm()).item() < 4e-3
    ops.gemm_nvfp4(out, qa, sa, qb, sb, K, epi=ops.EPI_BIAS_RESID, bias=bias, aux=res, alpha=alpha)
    want = base + bias.float() + res.float()
    assert ((out.float() - want).norm() / want.norm()).item() < 4e-3
    acc = torch.ones(M, N, dtype=torch.float32, device="cuda")
    ops.gemm_nvfp4(acc, qa, sa, qb, sb, K, epi=ops.EPI_ACC_F32, splits=4, alpha=alpha)
    assert (((acc - 1.0) - base).norm() / base.norm()).item() < 1e-4


@gpu
def test_nvfp4_linear_native_matches_emulated(monkeypatch):
    """One linear layer forward + backward: the block-scaled tensor path against the bf16 path on dequantised operands."""
    rows, C, OC = 512, 256, 384
    g = torch.Generator().manual_seed(3)
    x = torch.randn(rows, C, generator=g).bfloat16().cuda()
    w = (torch.randn(OC, C, generator=g) * 0.05).bfloat16().cuda()
    b = torch.randn(OC, generator=g).bfloat16().cuda()
    d = (torch.randn(rows, OC, generator=g) * 0.01).bfloat16().cuda()
    res = {}
    for mode in ("1", "0"):
        monkeypatch.setenv("LLMM_FP4_NATIVE", mode)
        out = torch.empty(rows, OC, dtype=torch.bfloat16, device="cuda")
        lowp.matmul_fwd_fp4(out, x, w, b)
        dinp = torch.empty(rows, C, dtype=torch.bfloat16, device="cuda")
        dw = torch.zeros(OC, C, dtype=torch.float32, device="cuda")
        db = torch.zeros(OC, dtype=torch.float32, device="cuda")
        lowp.matmul_bwd_fp4(dinp, dw, db, d, x, w, seed=7, step=2)
        res[mode] = (out.float(), dinp.float(), dw, db)
    for got, want in zip(res["1"], res["0"]):
        assert ((got - want).norm() / want.norm()).item() < 5e-3


@gpu
@pytest.mark.parametrize("axis", [1, 0])
def test_nvfp4_stochastic_rounding_on_device_is_unbiased_and_counter_based(axis):
    x = torch.randn(128, 256).bfloat16().cuda()
    acc = torch.zeros(128, 256, device="cuda")
    n = 64
    for s in range(n):
        deq, ts = lowp.nvfp4_fake_quant(x, axis=axis, sr=True, seed=5, step=s)
        acc += deq.float() * ts
    rne, ts = lowp.nvfp4_fake_quant(x, axis=axis)
    err_sr = (acc / n - x.float()).abs().mean().item()
    err_rne = (rne.float() * ts - x.float()).abs().mean().item()
    assert err_sr < 0.5 * err_rne, (err_sr, err_rne)
    a, _ = lowp.nvfp4_fake_quant(x, axis=axis, sr=True, seed=5, step=3)
    b, _ = lowp.nvfp4_fake_quant(x, axis=axis, sr=True, seed=5, step=3)
    c, _ = lowp.nvfp4_fake_quant(x, axis=axis, sr=True, seed=5, step=4)
    assert torch.equal(a, b) and not torch.equal(a, c)
    # neighbouring elements share one draw but use different bits of it: their rounding directions are uncorrelated
    up = ((a.float() * ts) > x.float()).float()
    pairs = up.reshape(-1, 2) if axis == 1 else up.t().reshape(-1, 2)
    corr = torch.corrcoef(pairs.t())[0, 1].abs().item()
    assert corr < 0.05, corr


@gpu
@pytest.mark.parametrize("gran,transpose,fmt", [(0, False, 0), (1, True, 1), (2, False, 0), (2, True, 0)])
def test_fp8_block_quant_bytes_and_scales_decode_to_the_fake_quantised_tensor(gran, transpose, fmt):
    rows, cols = 256, 384
    x = (torch.randn(rows, cols) * torch.logspace(-2, 2, cols)).bfloat16().cuda()
    q, sf = lowp.fp8_block_quant(x, gran, fmt, transpose)
    want = lowp.fp8_block_fake_quant(x, gran, fmt).float()
    vals = q.view(torch.float8_e4m3fn if fmt == 0 else torch.float8_e5m2).float()
    outer, K = vals.shape
    sfc = sf.cpu().view(outer // 128, K // 128, 32, 4, 4)                 # [line block][k atom][line % 32][line / 32][4 equal bytes]
    assert (sfc == sfc[..., :1]).all()
    e = sfc[..., 0].permute(0, 3, 2, 1).reshape(outer, K // 128).float()  # line = lb*128 + (l/32)*32 + l%32
    scale = torch.exp2(e - 127.0).cuda().repeat_interleave(128, dim=1)
    got = vals * scale
    got = got.t() if transpose else got
    assert torch.equal(got, want)


@gpu
@pytest.mark.parametrize("M,N,K", [(256, 384, 512), (128, 128, 128), (1024, 768, 3072)])
def test_native_mxfp8_gemm_matches_product_of_fake_quantised_operands(M, N, K):
    from llm_mojo_b200 import ops
    g = torch.Generator().manual_seed(2)
    a = (torch.randn(M, K, generator=g) * (1 + torch.arange(K) % 5)).bfloat16().cuda()
    b = (torch.randn(N, K, generator=g) * 0.05).bfloat16().cuda()
    qa, sa = lowp.fp8_block_quant(a, 0, lowp.E5M2)
    qb, sb = lowp.fp8_block_quant(b, 2, lowp.E4M3)
    want = lowp.fp8_block_fake_quant(a, 0, lowp.E5M2).float() @ lowp.fp8_block_fake_quant(b, 2, lowp.E4M3).float().t()
    out32 = torch.empty(M, N, dtype=torch.float32, device="cuda")
    ops.gemm_mxfp8(out32, qa, sa, qb, sb, a_fmt=lowp.E5M2, b_fmt=lowp.E4M3, epi=ops.EPI_STORE_F32)
    assert ((out32 - want).norm() / want.norm()).item() < 1e-5
    out = torch.empty(M, N, dtype=torch.bfloat16, device="cuda")
    bias = torch.randn(N, device="cuda").bfloat16()
    ops.gemm_mxfp8(out, qa, sa, qb, sb, a_fmt=lowp.E5M2, b_fmt=lowp.E4M3, epi=ops.EPI_BIAS, bias=bias)
    w2 = want + bias.float()
    assert ((out.float() - w2).norm() / w2.norm()).item() < 4e-3


@gpu
def test_fp8_block_linear_native_matches_fake_quant_path(monkeypatch):
    rows, C, OC = 512, 256, 384
    g = torch.Generator().manual_seed(4)
    x = torch.randn(rows, C, generator=g).bfloat16().cuda()
    w = (torch.randn(OC, C, generator=g) * 0.05).bfloat16().cuda()
    b = torch.randn(OC, generator=g).bfloat16().cuda()
    d = (torch.randn(rows, OC, generator=g) * 0.01).bfloat16().cuda()
    res = {}
    for mode in ("1", "0"):
        monkeypatch.setenv("LLMM_FP8B_NATIVE", mode)
        out = torch.empty(rows, OC, dtype=torch.bfloat16, device="cuda")
        pre = torch.empty_like(out)
        lowp.matmul_fwd_fp8_block(out, x, w, b, pre_gelu=pre)
        dinp = torch.empty(rows, C, dtype=torch.bfloat16, device="cuda")
        dw = torch.zeros(OC, C, dtype=torch.float32, device="cuda")
        db = torch.zeros(OC, dtype=torch.float32, device="cuda")
        lowp.matmul_bwd_fp8_block(dinp, dw, db, d, x, w)
        res[mode] = (out.float(), pre.float(), dinp.float(), dw, db)
    for got, want in zip(res["1"], res["0"]):
        assert ((got - want).norm() / want.norm()).item() < 5e-3


def test_fp8_static_scales_round_trip(tmp_path):
    """calibrate_fp8_scales.py writes a table; a run that loads it trains with frozen scales: one constant per
    (site, operand) = the minimum over layers, and update_scale no longer touches the state (CPU emulation)."""
    import json
    import calibrate_fp8_scales
    from llm_mojo_b200.config import GPT2Config
    from llm_mojo_b200.models import GPT2
    from llm_mojo_b200.ops.lowp import LowpState
    out = tmp_path / "scales.json"
    assert calibrate_fp8_scales.main(["--model", "d6", "--steps", "3", "-b", "2", "-t", "32", "--out", str(out)]) == 0
    table = json.load(open(out))["scales"]
    assert len(table) == 6 * 4 * 3 and all(v > 0 for v in table.values())
    m = GPT2("d6", Precision("fp8", fp32_storage=True), "cpu", fp8_static_scales=str(out))
    for site in LowpState.SITES:
        for role in LowpState.ROLES:
            want = min(table[f"{site}.{l}.{role}"] for l in range(6))
            for l in range(6):
                st = getattr(m.lowp.site(site, l), role)
                assert st.static and abs(float(st.scale) - want) < 1e-6 * want
    g = torch.Generator().manual_seed(0)
    toks = torch.randint(0, m.config.vocab_size, (2, 33), generator=g, dtype=torch.int32)
    losses = []
    for step in range(4):
        m.forward(toks[:, :-1].contiguous(), toks[:, 1:].contiguous())
        m.backward()
        m.update(step + 1, 1e-3)
        losses.append(m.read_loss())
    assert all(l == l for l in losses) and losses[-1] < losses[0]
    st = m.lowp.site("fc", 1).inp
    assert st.host_step == 0                                # the delayed-scaling machinery never ran
    with pytest.raises(ValueError):
        m.lowp.set_static_scales({"qkv.0.inp": 1.0})        # incomplete table
