"""Per-kernel numerics on the GPU: each sm_100a kernel against the fp32 PyTorch statement of
the same op (the CPU path of ``llm_mojo_b200.ops``).  Mirrors the reference's
tests/test_*_equivalence.py tier."""
import math

import pytest
import torch

from llm_mojo_b200 import ops
from llm_mojo_b200.ops import _lib

pytestmark = pytest.mark.gpu
DEV = "cuda"


def rnd(*shape, dtype=torch.bfloat16, scale=1.0, seed=0):
    g = torch.Generator().manual_seed(seed + sum(shape))
    return (torch.randn(*shape, generator=g) * scale).to(dtype)


def close(a, b, atol, rtol, name="", strict=False):
    """``strict``: not a single element may be out of tolerance (otherwise up to 0.1 % may)."""
    a, b = a.float().cpu(), b.float().cpu()
    err = (a - b).abs()
    lim = atol + rtol * b.abs()
    bad = (err > lim).float().mean().item()
    assert bad < (1e-12 if strict else 1e-3), \
        f"{name}: {bad * 100:.4f}% elements out of tolerance, max err {err.max().item():.4g}"
    assert torch.isfinite(a).all(), f"{name}: non-finite output"


def status_ok():
    assert _lib.read_status() == 0, "a bounded device wait expired"


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32])
def test_encoder_fwd_bwd(dtype):
    B, T, C, V = 4, 64, 256, 512
    wte, wpe = rnd(V, C, dtype=dtype), rnd(T, C, dtype=dtype, seed=1)
    tok = torch.randint(0, V, (B, T), dtype=torch.int32)
    tok[0, :8] = 7   # a long run of one token
    out = torch.empty(B, T, C, dtype=dtype, device=DEV)
    ops.encoder_fwd(out, tok.to(DEV), wte.to(DEV), wpe.to(DEV))
    ref = torch.empty(B, T, C)
    ops.encoder_fwd(ref, tok, wte.float(), wpe.float())
    close(out, ref, 1e-2 if dtype == torch.bfloat16 else 1e-6, 1e-2 if dtype == torch.bfloat16 else 1e-6, "encoder_fwd")
    dout = rnd(B, T, C, dtype=dtype, seed=2)
    dwte, dwpe = torch.zeros(V, C), torch.zeros(T, C)
    ops.encoder_bwd(dwte, dwpe, dout.float(), tok)
    gw, gp = torch.zeros(V, C, device=DEV), torch.zeros(T, C, device=DEV)
    ops.encoder_bwd(gw, gp, dout.to(DEV), tok.to(DEV))
    close(gw, dwte, 1e-5, 1e-5, "dwte")
    close(gp, dwpe, 1e-5, 1e-5, "dwpe")
    gw2, gp2 = torch.zeros(V, C, device=DEV), torch.zeros(T, C, device=DEV)
    ops.encoder_bwd(gw2, gp2, dout.to(DEV), tok.to(DEV))
    assert torch.equal(gw, gw2) and torch.equal(gp, gp2), "encoder backward must be bitwise repeatable"


@pytest.mark.parametrize("C", [256, 1600])     # 1600: a row is 200 vectors of 8, not a multiple of the warp size
@pytest.mark.parametrize("kind", ["zipf", "one_token", "aligned_runs"])
def test_encoder_bwd_skewed_tokens(kind, C):
    """Token distributions of real text: a few tokens own thousands of positions.  The kernel cuts the sorted positions
    into segments of 16 and sums the pieces of a run that crosses segment borders in a second pass; here runs span hundreds
    of segments, start and end exactly on segment borders, and the last segment is partial."""
    B, T, V = 5, 1000, 50304
    g = torch.Generator().manual_seed(3)
    if kind == "zipf":
        w = 1.0 / torch.arange(1, 50258, dtype=torch.float64) ** 1.2
        tok = torch.multinomial(w, B * T, replacement=True, generator=g).view(B, T).int()
    elif kind == "one_token":
        tok = torch.full((B, T), 4321, dtype=torch.int32)
    else:       # runs of exactly 16, 32, 48 positions so that runs begin and end on segment borders, then singles
        ids = torch.cat([torch.full((16,), 5), torch.full((32,), 9), torch.full((48,), 11), torch.full((15,), 12), torch.full((17,), 13),
                         torch.arange(100, 100 + B * T - 128)])
        tok = ids[torch.randperm(B * T, generator=g)].view(B, T).int()
    dout = rnd(B, T, C, dtype=torch.bfloat16, seed=4)
    dwte, dwpe = torch.zeros(V, C), torch.zeros(T, C)
    ops.encoder_bwd(dwte, dwpe, dout.float(), tok)
    gw, gp = torch.full((V, C), 0.5, device=DEV), torch.zeros(T, C, device=DEV)
    ops.encoder_bwd(gw, gp, dout.to(DEV), tok.to(DEV))
    torch.cuda.synchronize()
    close(gw, dwte + 0.5, 2e-3, 1e-4, "dwte (skewed)", strict=True)      # sums of up to 5000 bf16 rows in fp32
    gw2, gp2 = torch.full((V, C), 0.5, device=DEV), torch.zeros(T, C, device=DEV)
    ops.encoder_bwd(gw2, gp2, dout.to(DEV), tok.to(DEV))
    assert torch.equal(gw, gw2), "encoder backward must be bitwise repeatable"


@pytest.mark.parametrize("C", [768, 1024, 1280, 1600])
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32])
def test_layernorm_fwd_bwd(C, dtype):
    rows = 384
    x, x2 = rnd(rows, C, dtype=dtype), rnd(rows, C, dtype=dtype, seed=1)
    w, b = (1 + 0.1 * rnd(C, dtype=dtype, seed=2)).to(dtype), rnd(C, dtype=dtype, seed=3)
    tol = (5e-3, 2e-2) if dtype == torch.bfloat16 else (2e-5, 1e-4)
    out = torch.empty(rows, C, dtype=dtype, device=DEV)
    res = torch.empty(rows, C, dtype=dtype, device=DEV)
    mean, rstd = torch.empty(rows, device=DEV), torch.empty(rows, device=DEV)
    ops.residual_layernorm_fwd(res, out, mean, rstd, x.to(DEV), x2.to(DEV), w.to(DEV), b.to(DEV))
    r_out, r_res, r_mean, r_rstd = torch.empty(rows, C), torch.empty(rows, C), torch.empty(rows), torch.empty(rows)
    xs = (x.float() + x2.float()).to(dtype).float()   # residual is stored in the storage dtype
    ops.layernorm_fwd(r_out, r_mean, r_rstd, xs, w.float(), b.float())
    close(res, xs, *tol, "residual")
    close(out, r_out, *tol, "ln out")
    close(mean, r_mean, 1e-4, 1e-3, "mean")
    close(rstd, r_rstd, 1e-4, 1e-3, "rstd")
    out1 = torch.empty(rows, C, dtype=dtype, device=DEV)
    ops.layernorm_fwd(out1, mean, rstd, xs.to(dtype).to(DEV), w.to(DEV), b.to(DEV))
    close(out1, r_out, *tol, "ln out (no residual)")
    # backward
    dout = rnd(rows, C, dtype=dtype, seed=4)
    dres0 = rnd(rows, C, dtype=dtype, seed=5)
    for accumulate in (True, False):
        r_dres, r_dw, r_db = dres0.float().clone(), torch.zeros(C), torch.zeros(C)
        ops.layernorm_bwd(r_dres, r_dw, r_db, dout.float(), xs, w.float(), r_mean, r_rstd, accumulate=accumulate)
        dres, dw, db = dres0.to(DEV).clone(), torch.zeros(C, device=DEV), torch.zeros(C, device=DEV)
        ops.layernorm_bwd(dres, dw, db, dout.to(DEV), xs.to(dtype).to(DEV), w.to(DEV), mean, rstd, accumulate=accumulate)
        close(dres, r_dres, tol[0] * 4, tol[1], f"dres acc={accumulate}")
        close(dw, r_dw, 1e-3 * math.sqrt(rows), 1e-2, "dgamma")
        close(db, r_db, 1e-3 * math.sqrt(rows), 1e-2, "dbeta")
        # the same pass can also return the column sums of the gradient it wrote (the bias gradient of the layer above)
        dres2, dw2, db2 = dres0.to(DEV).clone(), torch.zeros(C, device=DEV), torch.zeros(C, device=DEV)
        cs = torch.full((C,), 0.5, device=DEV)
        ops.layernorm_bwd(dres2, dw2, db2, dout.to(DEV), xs.to(dtype).to(DEV), w.to(DEV), mean, rstd, accumulate=accumulate,
                          dres_colsum=cs)
        assert torch.equal(dres2, dres) and torch.equal(dw2, dw) and torch.equal(db2, db)
        close(cs, 0.5 + dres.float().sum(0), 2e-3 * math.sqrt(rows), 1e-3, f"colsum of dres acc={accumulate}")


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32])
def test_gelu(dtype):
    x, d = rnd(64, 1024, dtype=dtype, scale=2.0), rnd(64, 1024, dtype=dtype, seed=1)
    tol = (5e-3, 2e-2) if dtype == torch.bfloat16 else (2e-5, 1e-4)
    out, dinp = torch.empty_like(x, device=DEV), torch.empty_like(x, device=DEV)
    ops.gelu_fwd(out, x.to(DEV))
    ops.gelu_bwd(dinp, x.to(DEV), d.to(DEV))
    ref = torch.nn.functional.gelu(x.float(), approximate="tanh")
    close(out, ref, *tol, "gelu")
    xr = x.float().requires_grad_(True)
    torch.nn.functional.gelu(xr, approximate="tanh").backward(d.float())
    close(dinp, xr.grad, *tol, "gelu bwd")


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32])
def test_fused_classifier(dtype):
    rows, V, Vp = 96, 50257, 50304
    logits = rnd(rows, Vp, dtype=dtype, scale=3.0)
    tgt = torch.randint(0, V, (rows,), dtype=torch.int32)
    dloss = 1.0 / rows
    r_logits, r_losses = logits.float().clone(), torch.empty(rows)
    ops.fused_classifier(r_logits, r_losses, tgt, dloss, V)
    g_logits, g_losses = logits.to(DEV).clone(), torch.empty(rows, device=DEV)
    ops.fused_classifier(g_logits, g_losses, tgt.to(DEV), dloss, V)
    close(g_losses, r_losses, 1e-3, 1e-3, "losses")
    atol = 2e-4 * dloss if dtype == torch.float32 else 1e-2 * dloss
    close(g_logits, r_logits, atol, 2e-2, "dlogits")
    assert torch.all(g_logits[:, V:] == 0), "padded vocabulary tail must be zeroed"


def test_fused_classifier_every_cta_refills_its_row_buffers():
    """700 rows of the full GPT-2 vocabulary on at most 148 persistent CTAs: every CTA streams four or five rows, so
    both row buffers of the streaming kernel are refilled and their barrier phases wrap.  Oracle: the fp32 statement
    of the op on the GPU (log-softmax minus one-hot, scaled), strict tolerance."""
    rows, V, Vp = 700, 50257, 50304
    logits = rnd(rows, Vp, scale=3.0).to(DEV)
    tgt = torch.randint(0, V, (rows,), dtype=torch.int32, generator=torch.Generator().manual_seed(3)).to(DEV)
    dloss = 1.0 / rows
    x = logits[:, :V].float()
    lse = torch.logsumexp(x, dim=1)
    r_losses = lse - x.gather(1, tgt.long().view(-1, 1)).squeeze(1)
    r_d = torch.softmax(x, dim=1)
    r_d[torch.arange(rows, device=DEV), tgt.long()] -= 1.0
    r_d *= dloss
    losses = torch.empty(rows, device=DEV)
    ops.fused_classifier(logits, losses, tgt, dloss, V)
    torch.cuda.synchronize()
    status_ok()
    close(losses, r_losses, 2e-3, 1e-3, "losses (700 rows)", strict=True)
    close(logits[:, :V], r_d, 1e-2 * dloss, 2e-2, "dlogits (700 rows)", strict=True)
    assert torch.all(logits[:, V:] == 0), "padded vocabulary tail must be zeroed"


def test_dbias_regression():
    """dbias at 124M / 774M widths with a row count that is not a multiple of the slab size
    (the reference's dbias scratch-overrun regression, tests/test_dbias_regression.mojo)."""
    for rows, OC in ((4096 + 17, 3072), (1000, 5120), (256, 768)):
        d = rnd(rows, OC, seed=rows)
        ref = d.float().sum(0)
        out = torch.zeros(OC, device=DEV)
        ops.dbias_reduce(out, d.to(DEV))
        close(out, ref, 1e-3 * math.sqrt(rows), 1e-3, f"dbias {rows}x{OC}")
        ops.dbias_reduce(out, d.to(DEV))
        close(out, 2 * ref, 2e-3 * math.sqrt(rows), 1e-3, "dbias accumulates")


@pytest.mark.parametrize("master", [True, False])
def test_adamw(master):
    n = 100003
    dtype = torch.bfloat16 if master else torch.float32
    p0 = rnd(n, dtype=torch.float32)
    g, m0, v0 = rnd(n, dtype=torch.float32, seed=1), rnd(n, dtype=torch.float32, seed=2) * 0.1, rnd(n, dtype=torch.float32, seed=3).abs() * 0.01
    kw = dict(lr=1e-2, beta1=0.9, beta2=0.95, eps=1e-8, weight_decay=0.1, grad_scale=0.5, step=3)
    rp, rm, rv = p0.clone(), m0.clone(), v0.clone()
    ops.adamw_update(rp, None, g, rm, rv, **kw)
    gp = p0.to(dtype).to(DEV)
    gmaster = p0.to(DEV).clone() if master else None
    gm, gv = m0.to(DEV).clone(), v0.to(DEV).clone()
    scale = torch.tensor([0.5], device=DEV)
    kw2 = dict(kw, grad_scale=1.0)
    ops.adamw_update(gp, gmaster, g.to(DEV), gm, gv, dev_scale=scale, **kw2)
    close(gm, rm, 1e-6, 1e-5, "m")
    close(gv, rv, 1e-7, 1e-5, "v")
    if master:
        close(gmaster, rp, 1e-6, 1e-5, "master")
        close(gp, rp, 1e-2, 1e-2, "bf16 params")
    else:
        close(gp, rp, 1e-6, 1e-5, "params")


def test_global_norm():
    x = rnd(1 << 20, dtype=torch.float32)
    out = torch.zeros(1, device=DEV)
    ops.global_norm_squared(out, x.to(DEV))
    ref = (x.double() ** 2).sum().item()
    assert abs(out.item() - ref) / ref < 1e-5
    ops.global_norm_squared(out, x.to(DEV), accumulate=True)
    assert abs(out.item() - 2 * ref) / ref < 1e-5


def test_stochastic_rounding_is_unbiased():
    L = _lib.lib()
    x = torch.full((1 << 20,), 1.0 + 2 ** -10, device=DEV)   # between two bf16 values (spacing 2^-7)
    out = torch.empty(1 << 20, dtype=torch.bfloat16, device=DEV)
    _lib.check(L.llmb_sr_cast_bf16(out.data_ptr(), x.data_ptr(), x.numel(), 1234, _lib.stream()), "sr")
    vals = out.float()
    assert set(vals.unique().tolist()) <= {1.0, 1.0 + 2 ** -7}
    assert abs(vals.mean().item() - (1.0 + 2 ** -10)) < 2e-4


# ------------------------------------------------------------------------------ GEMM
def _gemm_case(M, N, K, a_mn, b_mn, epi="none", seed=0):
    A = rnd(K, M, seed=seed) if a_mn else rnd(M, K, seed=seed)
    Bm = rnd(K, N, seed=seed + 1) if b_mn else rnd(N, K, seed=seed + 1)
    Af = (A.float().t() if a_mn else A.float())
    Bf = (Bm.float().t() if b_mn else Bm.float())
    ref = Af @ Bf.t()
    A_d, B_d = A.to(DEV), Bm.to(DEV)
    scale = math.sqrt(K)
    if epi == "acc_f32":
        D0 = rnd(M, N, dtype=torch.float32, seed=seed + 2)
        D = D0.to(DEV).clone()
        ops.gemm(D, A_d, B_d, a_mn=a_mn, b_mn=b_mn, epi=ops.EPI_ACC_F32, splits=ops._splits_for(M, N, K))
        close(D, ref + D0, 2e-3 * scale, 1e-3, f"gemm acc {M}x{N}x{K}")
    else:
        D = torch.empty(M, N, dtype=torch.bfloat16, device=DEV)
        bias = rnd(N, seed=seed + 3)
        if epi == "none":
            ops.gemm(D, A_d, B_d, a_mn=a_mn, b_mn=b_mn)
        elif epi == "bias":
            ops.gemm(D, A_d, B_d, a_mn=a_mn, b_mn=b_mn, epi=ops.EPI_BIAS, bias=bias.to(DEV))
            ref = ref + bias.float()
        elif epi == "bias_gelu":
            aux = torch.empty(M, N, dtype=torch.bfloat16, device=DEV)
            ops.gemm(D, A_d, B_d, epi=ops.EPI_BIAS_GELU, bias=bias.to(DEV), aux=aux)
            pre = ref + bias.float()
            close(aux, pre, 1e-2 * scale, 1e-2, "pre-gelu aux")
            ref = torch.nn.functional.gelu(pre, approximate="tanh")
        elif epi == "dgelu":
            aux = rnd(M, N, seed=seed + 4)
            ops.gemm(D, A_d, B_d, a_mn=a_mn, b_mn=b_mn, epi=ops.EPI_DGELU, aux=aux.to(DEV))
            ref = ref * ops._gelu_grad_t(aux.float())
        elif epi == "bias_resid":
            aux = rnd(M, N, seed=seed + 4)
            ops.gemm(D, A_d, B_d, epi=ops.EPI_BIAS_RESID, bias=bias.to(DEV), aux=aux.to(DEV))
            ref = ref + bias.float() + aux.float()
        close(D, ref, 1e-2 * scale, 1e-2, f"gemm {epi} {M}x{N}x{K} a_mn={a_mn} b_mn={b_mn}")
    torch.cuda.synchronize()
    status_ok()


@pytest.fixture(params=[1, 0], ids=["cta_pair", "single_cta"])
def gemm_mode(request):
    """Run every GEMM test with CTA-pair (cta_group::2, 256x256) and single-CTA (128x256) tiles."""
    _lib.lib().llmb_gemm_set_pair_mode(request.param)
    yield request.param
    _lib.lib().llmb_gemm_set_pair_mode(1)


@pytest.mark.parametrize("shape", [(128, 256, 64), (256, 768, 768), (384, 2304, 768), (512, 50304, 768), (200, 1600, 1600),
                                   (1024, 768, 768)])
def test_gemm_tn(shape, gemm_mode):
    _gemm_case(*shape, a_mn=False, b_mn=False)


@pytest.mark.parametrize("epi", ["bias", "bias_gelu", "bias_resid"])
def test_gemm_fwd_epilogues(epi, gemm_mode):
    _gemm_case(384, 3072, 768, False, False, epi=epi)


@pytest.mark.parametrize("epi", ["none", "dgelu"])
def test_gemm_dinp_nn(epi, gemm_mode):
    _gemm_case(384, 768, 3072, a_mn=False, b_mn=True, epi=epi)


@pytest.mark.parametrize("shape", [(768, 768, 4096), (3072, 768, 2048), (768, 3072, 1024 + 64), (50304, 768, 512)])
def test_gemm_dw_tt_splitk(shape, gemm_mode):
    _gemm_case(*shape, a_mn=True, b_mn=True, epi="acc_f32")


def test_gemm_tf32_fp32_storage(gemm_mode):
    """fp32 operands on the kind::tf32 path: forward with bias+GELU, dinp (B stored [K,N]) and dW (both [K,.])."""
    M, N, K = 384, 768, 512
    g = torch.Generator().manual_seed(3)
    A, W, b = torch.randn(M, K, generator=g), torch.randn(N, K, generator=g) * 0.05, torch.randn(N, generator=g)
    D, aux = torch.empty(M, N, device=DEV), torch.empty(M, N, device=DEV)
    ops.gemm(D, A.to(DEV), W.to(DEV), epi=ops.EPI_BIAS_GELU, bias=b.to(DEV), aux=aux, kind=1)
    pre = A @ W.t() + b
    close(aux, pre, 2e-2, 1e-2, "tf32 pre-gelu")
    close(D, torch.nn.functional.gelu(pre, approximate="tanh"), 2e-2, 1e-2, "tf32 gelu")
    d = torch.randn(M, N, generator=g)
    dA = torch.empty(M, K, device=DEV)
    ops.gemm(dA, d.to(DEV), W.to(DEV), b_mn=True, kind=1)
    close(dA, d @ W, 5e-2, 1e-2, "tf32 dinp")
    dW = torch.zeros(N, K, device=DEV)
    ops.gemm(dW, d.to(DEV), A.to(DEV), a_mn=True, b_mn=True, epi=ops.EPI_ACC_F32, splits=2, kind=1)
    close(dW, d.t() @ A, 1e-1, 1e-2, "tf32 dW")
    torch.cuda.synchronize()
    status_ok()


# ------------------------------------------------------------------------------ attention
@pytest.mark.parametrize("bwd", ["fused", "split"])
@pytest.mark.parametrize("B,T,NH", [(2, 128, 2), (1, 256, 3), (2, 1024, 2), (2, 64, 2), (1, 200, 1), (3, 640, 5), (2, 384, 2), (1, 2048, 2),
                                    (1, 1100, 3)])
def test_attention_fwd_bwd(B, T, NH, bwd, monkeypatch):
    monkeypatch.setattr(ops, "ATTN_BWD", bwd)
    C = NH * 64
    qkv = rnd(B, T, 3 * C, scale=1.0)
    dout = rnd(B, T, C, seed=1)
    r_out, r_lse = torch.empty(B, T, C), torch.empty(B, NH, T)
    ops.attention_fwd(r_out, r_lse, qkv.float(), NH)
    out = torch.empty(B, T, C, dtype=torch.bfloat16, device=DEV)
    lse = torch.empty(B, NH, T, device=DEV)
    ops.attention_fwd(out, lse, qkv.to(DEV), NH)
    torch.cuda.synchronize()
    status_ok()
    close(out, r_out, 1e-2, 2e-2, "attention out")
    close(lse, r_lse, 2e-2, 1e-3, "lse")
    r_dqkv = torch.empty(B, T, 3 * C)
    ops.attention_bwd(r_dqkv, dout.float(), qkv.float(), r_out, r_lse, NH)
    dqkv = torch.full((B, T, 3 * C), float("nan"), dtype=torch.bfloat16, device=DEV)
    dbias = torch.full((3 * C,), 0.25, device=DEV)
    ops.attention_bwd(dqkv, dout.to(DEV), qkv.to(DEV), out, lse, NH, dbias=dbias)
    torch.cuda.synchronize()
    status_ok()
    for i, nm in enumerate(("dq", "dk", "dv")):
        close(dqkv[..., i * C:(i + 1) * C], r_dqkv[..., i * C:(i + 1) * C], 2e-2, 3e-2, nm)
    # the qkv bias gradient from the kernels' epilogues: column sums of dqkv (added to what the buffer held)
    close(dbias, 0.25 + r_dqkv.view(B * T, 3 * C).sum(0), 2e-2 * math.sqrt(B * T), 2e-2, "qkv dbias", strict=True)
    if bwd == "fused":
        # the fp32 dQ accumulation scratch is left zeroed, so a second call gives the same result
        acc = ops.scratch("attn_bwd_dq_acc", 4, dqkv.device).view(torch.float32)
        assert int(torch.count_nonzero(acc)) == 0
        again = torch.full_like(dqkv, float("nan"))
        ops.attention_bwd(again, dout.to(DEV), qkv.to(DEV), out, lse, NH)
        torch.cuda.synchronize()
        status_ok()
        close(again[..., :C], dqkv[..., :C], 1e-6, 2e-2, "dq, second call")     # atomic order differs: last-bit differences only
        assert torch.equal(again[..., C:], dqkv[..., C:])


def test_unfused_softmax_bwd_and_crossentropy():
    g = torch.Generator().manual_seed(11)
    rows, V, ld = 300, 50257, 50304
    logits = torch.randn(rows, ld, generator=g) * 2
    tgt = torch.randint(0, V, (rows,), generator=g, dtype=torch.int32)
    dloss = torch.randn(rows, generator=g)
    probs_c = torch.zeros(rows, ld)
    probs_c[:, :V] = ops.softmax_rows(logits, V)
    probs = probs_c.to(DEV)
    close(ops.crossentropy_fwd(probs, tgt.to(DEV)), ops.crossentropy_fwd(probs_c, tgt), 1e-5, 1e-5, "crossentropy fwd", strict=True)
    dprobs_c, dprobs = torch.zeros(rows, ld), torch.zeros(rows, ld, device=DEV)
    ops.crossentropy_bwd(dprobs_c, dloss, probs_c, tgt)
    ops.crossentropy_bwd(dprobs, dloss.to(DEV), probs, tgt.to(DEV))
    close(dprobs, dprobs_c, 1e-3, 1e-5, "crossentropy bwd", strict=True)
    close(ops.softmax_bwd(dprobs, probs, V), ops.softmax_bwd(dprobs_c, probs_c, V), 1e-5, 1e-4, "softmax bwd", strict=True)


@pytest.mark.parametrize("bwd", ["fused", "split"])
def test_attention_persistent_loops_large(bwd, monkeypatch):
    """B=16, NH=12, T=1024: 768 work items on at most 148 CTAs, so every persistent CTA walks several items per
    tile stream (barrier phase wrap, TMEM hand-back between items, the heavy/light tile alternation).  Oracle: the
    fp32 statement of the op with autograd, on the GPU because of its [B,NH,T,T] intermediates.  Strict: no element
    may miss the tolerance."""
    monkeypatch.setattr(ops, "ATTN_BWD", bwd)
    B, T, NH = 16, 1024, 12
    C = NH * 64
    qkv = rnd(B, T, 3 * C, scale=1.0).to(DEV)
    dout = rnd(B, T, C, seed=1).to(DEV)
    leaf = qkv.float().requires_grad_(True)
    q, k, v = (t.view(B, T, NH, 64).transpose(1, 2) for t in leaf.split(C, dim=2))
    sc = (q @ k.transpose(-1, -2)) / 8.0
    sc = sc.masked_fill(~torch.ones(T, T, dtype=torch.bool, device=DEV).tril(), float("-inf"))
    r_lse = torch.logsumexp(sc, dim=-1) * math.log2(math.e)
    r_out = (torch.softmax(sc, dim=-1) @ v).transpose(1, 2).reshape(B, T, C)
    r_out.backward(dout.float())
    r_dqkv = leaf.grad
    del sc
    out = torch.empty(B, T, C, dtype=torch.bfloat16, device=DEV)
    lse = torch.empty(B, NH, T, device=DEV)
    ops.attention_fwd(out, lse, qkv, NH)
    dqkv = torch.full((B, T, 3 * C), float("nan"), dtype=torch.bfloat16, device=DEV)
    ops.attention_bwd(dqkv, dout, qkv, out, lse, NH)
    torch.cuda.synchronize()
    status_ok()
    close(out, r_out.detach(), 1.5e-2, 2e-2, "attention out (large)", strict=True)
    close(lse, r_lse.detach(), 2e-2, 1e-3, "lse (large)", strict=True)
    for i, nm in enumerate(("dq", "dk", "dv")):
        close(dqkv[..., i * C:(i + 1) * C], r_dqkv[..., i * C:(i + 1) * C], 3e-2, 3e-2, nm + " (large)", strict=True)


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_nan_census(dtype):
    x = torch.randn(1_000_003, device="cuda").to(dtype)
    assert ops.nan_census(x) == (0, 0)
    x[5] = float("nan"); x[77777] = float("nan"); x[999_999] = float("inf"); x[123] = float("-inf"); x[124] = float("inf")
    assert ops.nan_census(x) == (2, 3)


@pytest.mark.gpu
@pytest.mark.parametrize("rows,OC,C", [(1024, 768, 3072), (520, 256, 1024)])
def test_dgelu_gemm_adds_the_column_sums_of_its_result(rows, OC, C, monkeypatch):
    """matmul_bwd(dinp_colsum=...): the bias gradient of the layer below, taken in the dGELU epilogue, equals the
    separate reduction over the stored (bf16) result; rows that do not fill the last tile are left out."""
    d, w = rnd(rows, OC, scale=0.1).to(DEV), rnd(OC, C, scale=0.05).to(DEV)
    pre, x = rnd(rows, C).to(DEV), rnd(rows, C).to(DEV)
    res = {}
    for mode in ("1", "0"):
        monkeypatch.setenv("LLMM_FUSED_FC_DBIAS", mode)
        dinp = torch.empty(rows, C, dtype=torch.bfloat16, device=DEV)
        col = torch.full((C,), 0.5, device=DEV)                      # accumulates on top of what is there
        ops.matmul_bwd(dinp, None, None, d, x, w, gelu_pre=pre, dinp_colsum=col)
        res[mode] = (dinp, col)
    assert torch.equal(res["1"][0], res["0"][0])
    want = res["1"][0].float().sum(0) + 0.5
    close(res["1"][1], want, 1e-3 * math.sqrt(rows), 1e-3, "fused column sums")
    close(res["0"][1], want, 1e-3 * math.sqrt(rows), 1e-3, "separate column sums")
