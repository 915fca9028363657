"""The checked build (``-DLLMB_BOUNDS_CHECK``, ``LLMB_BOUNDS_CHECK=1``): indices that come out of data are tested before
they address memory, scratch buffers carry canaries.  Stand-in for a memory checker: a corrupt batch or an overrunning
kernel shows up as a report, and nothing faults.  Each case runs in a child process, because the library variant is
chosen when the package is imported."""
import os
import subprocess
import sys
import textwrap

import pytest

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _child(code: str) -> str:
    env = dict(os.environ, LLMB_BOUNDS_CHECK="1", PYTHONPATH=ROOT)
    r = subprocess.run([sys.executable, "-c", textwrap.dedent(code)], env=env, capture_output=True, text=True, timeout=600)
    assert r.returncode == 0, (r.stdout + r.stderr)[-3000:]
    return r.stdout


def test_checked_library_exists_and_is_the_one_loaded():
    out = _child("""
        from llm_mojo_b200.ops import _lib
        print(_lib.lib_path())
        assert _lib.BOUNDS_CHECK and _lib.lib_path().endswith("libllmb200_check.so")
        _lib.lib()
    """)
    assert "libllmb200_check.so" in out


def test_out_of_range_token_and_target_are_reported_not_dereferenced():
    _child("""
        import torch
        from llm_mojo_b200 import ops
        from llm_mojo_b200.ops import _lib
        V, C, B, T = 512, 256, 2, 64
        wte = torch.randn(V, C, device="cuda").bfloat16(); wpe = torch.randn(T, C, device="cuda").bfloat16()
        tok = torch.randint(0, V, (B, T), dtype=torch.int32, device="cuda")
        tok[1, 5] = V + 70000                      # a corrupt token id
        out = torch.full((B, T, C), 7.0, device="cuda", dtype=torch.bfloat16)
        ops.encoder_fwd(out, tok, wte, wpe)
        torch.cuda.synchronize()
        rep = _lib.bounds_report()
        assert rep == [("encoder_fwd token id", V + 70000, V)], rep
        assert torch.all(out[1, 5] == 7.0)         # the row of the bad token was skipped ...
        assert torch.allclose(out[0, 0].float(), (wte[tok[0, 0]].float() + wpe[0].float()), atol=2e-2)   # ... the others written
        assert _lib.bounds_report() == []          # the record was reset
        # a corrupt target in the fused classifier
        rows, Vp = 64, 512
        logits = torch.randn(rows, Vp, device="cuda").bfloat16()
        losses = torch.empty(rows, device="cuda")
        tgt = torch.randint(0, V, (rows,), dtype=torch.int32, device="cuda")
        tgt[3] = 10 ** 6
        ops.fused_classifier(logits, losses, tgt, 1.0 / rows, V)
        torch.cuda.synchronize()
        rep = _lib.bounds_report()
        assert rep and rep[0][0] == "fused_classifier target id" and rep[0][1] == 10 ** 6, rep
        assert torch.isfinite(losses).all()
        assert float((torch.ones(8, device="cuda") * 2).sum()) == 16.0     # the context is healthy
    """)


def test_scratch_canary_catches_an_overrun():
    _child("""
        import torch
        from llm_mojo_b200 import ops
        from llm_mojo_b200.ops import _lib
        s = ops.scratch("canary_probe", 1000, torch.device("cuda"))
        ops.verify_scratch_canaries()
        full = ops._CANARIES[("canary_probe", "cuda")]
        full[s.numel() + 3] = 0                    # what a kernel writing 4 bytes past its scratch would do
        try:
            ops.verify_scratch_canaries()
            raise SystemExit("overrun not detected")
        except _lib.KernelError as e:
            assert "canary_probe" in str(e)
    """)


def test_training_steps_run_clean_under_the_checked_build():
    _child("""
        from llm_mojo_b200.trainer import TrainArgs, Trainer
        tr = Trainer(TrainArgs(load_filename="d6", batch_size=2, seq_len=128, total_batch_size=512, max_steps=5,
                               synthetic=True, val_loss_every=0, sample_every=0))
        losses = [tr.train_step()["loss"] for _ in range(3)]     # every step verifies the canaries and the index records
        assert all(l == l for l in losses) and losses[-1] < losses[0], losses
    """)
