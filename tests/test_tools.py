"""Smoke tests of the command-line tools on CPU with tiny models (after the reference's generation smoke test,
`make verify-cpu` debug-state gate, `make verify-fp8-grads` gradient gate and per-precision `make smoke` runs)."""
import io
import json
import os
import sys
from contextlib import redirect_stdout

import pytest
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)


def _run(mod_name, argv):
    import importlib
    mod = importlib.import_module(mod_name)
    buf = io.StringIO()
    with redirect_stdout(buf):
        rc = mod.main(argv)
    return rc, buf.getvalue()


def test_infer_generation_smoke(tmp_path):
    """infer_gpt2 samples the requested number of tokens from a checkpoint and is reproducible for a fixed seed."""
    from llm_mojo_b200.config import GPT2Config
    from llm_mojo_b200.models import GPT2
    m = GPT2(GPT2Config(max_seq_len=32, vocab_size=300, num_layer=2, num_heads=2, channels=32, padded_vocab_size=384), "fp32", "cpu")
    from llm_mojo_b200.utils import checkpointing as ckpt
    ck = str(tmp_path / "tiny.bin")
    ckpt.write_model_checkpoint(ck, m.config, m.full_params(), m.precision.checkpoint_version)
    import subprocess
    cmd = [sys.executable, os.path.join(ROOT, "infer_gpt2.py"), ck, "--tokens", "8", "--device", "cpu", "--seed", "7", "-t", "32",
           "--prompt-tokens", "5,6,7"]
    outs = [subprocess.run(cmd, capture_output=True, text=True, timeout=300, cwd=str(tmp_path)) for _ in range(2)]
    assert all(o.returncode == 0 for o in outs), outs[0].stderr
    gen1, gen2 = (o.stdout.split("---")[-2] for o in outs)      # the text between the tokenizer notice and the timing line
    assert gen1 == gen2 and len(gen1.split()) == 8 and all(0 <= int(t) < 300 for t in gen1.split())


def test_debug_state_gate_roundtrip(tmp_path):
    """test_gpt2 --write produces model + debug state from the autograd oracle; the checker passes on our model."""
    mf, sf = str(tmp_path / "m.bin"), str(tmp_path / "s.bin")
    rc, _ = _run("test_gpt2", ["--write", "--model", "d6", "--model-file", mf, "--state", sf, "-b", "2", "-t", "16", "--device", "cpu"])
    assert rc == 0 and os.path.getsize(mf) > 0 and os.path.getsize(sf) > 0
    rc, out = _run("test_gpt2", ["--model-file", mf, "--state", sf, "--device", "cpu", "--precision", "fp32"])
    assert rc == 0, out
    assert "overall okay: 1" in out or "OK" in out.upper()


def test_gradient_dump_gate_fp32_vs_itself(tmp_path):
    """dump_grads_gpt2 writes one file per gradient tensor; compare_grad_dumps accepts identical dumps and rejects noise."""
    import compare_grad_dumps
    a, b = str(tmp_path / "a"), str(tmp_path / "b")
    for d in (a, b):
        rc, _ = _run("dump_grads_gpt2", ["--model", "d6", "--precision", "fp32", "--out", d, "-b", "2", "-t", "16", "--device", "cpu"])
        assert rc == 0
    assert len(os.listdir(a)) >= 16
    assert compare_grad_dumps.compare(a, b, verbose=False)
    victim = sorted(f for f in os.listdir(b) if os.path.isfile(os.path.join(b, f)) and not f.endswith(".json"))[0]
    path = os.path.join(b, victim)
    raw = bytearray(open(path, "rb").read())
    t = torch.frombuffer(raw, dtype=torch.float32, offset=len(raw) % 4)
    t.copy_(torch.randn(t.numel()))
    open(path, "wb").write(bytes(raw))
    assert not compare_grad_dumps.compare(a, b, verbose=False)


def test_bench_reference_arm_line(tmp_path):
    """--impl reference never runs our code.  With the reference tree in place it runs that tree's own trainer (tiny
    config here, on CPU) and reports its step times; without it, it prints the `unavailable` JSON line.  Exit code 0 both ways."""
    import subprocess
    cmd = [sys.executable, os.path.join(ROOT, "bench.py"), "--impl", "reference", "--batch", "1", "--seq", "16",
           "--total-batch", "32", "--steps", "2", "--warmup", "1"]
    r = subprocess.run(cmd, capture_output=True, text=True, timeout=900, cwd=str(tmp_path))
    assert r.returncode == 0
    line = json.loads(r.stdout.strip().splitlines()[-1])
    assert line["impl"] == "reference"
    if os.path.exists(os.path.join(ROOT, "baseline", "_ref", "train_gpt2.py")):
        assert "unavailable" not in line, line
        assert line["steps"] == 2 and line["value"] > 0 and line["e2e"]["value"] > 0
        assert line["config"]["tokens_per_step"] == 32
    else:
        assert "unavailable" in line


def test_tokenizer_standin_shape():
    """The offline stand-in for tiktoken's GPT-2 plugin yields an encoding with GPT-2's size and end-of-text id."""
    sys.path.insert(0, os.path.join(ROOT, "baseline", "tokenizer_standin"))
    try:
        import importlib
        spec = importlib.util.spec_from_file_location(
            "standin_openai_public", os.path.join(ROOT, "baseline", "tokenizer_standin", "tiktoken_ext", "openai_public.py"))
        mod = importlib.util.module_from_spec(spec)
        spec.loader.exec_module(mod)
        c = mod.ENCODING_CONSTRUCTORS["gpt2"]()
        assert c["explicit_n_vocab"] == 50257 and c["special_tokens"]["<|endoftext|>"] == 50256
        assert len(c["mergeable_ranks"]) == 50256 and sorted(c["mergeable_ranks"].values()) == list(range(50256))
    finally:
        sys.path.pop(0)


@pytest.mark.parametrize("precision", ["fp32", "fp8", "fp4"])
def test_short_training_run_per_precision(precision, tmp_path):
    """Five optimizer steps of a tiny model on CPU for every precision the trainer accepts there (fp8 / fp4 run their
    quantise-dequantise emulation on fp32 storage); the loss must fall and stay finite."""
    from llm_mojo_b200.trainer import TrainArgs, Trainer
    args = TrainArgs(load_filename="d6", batch_size=2, seq_len=32, total_batch_size=64, max_steps=5, learning_rate=1e-3,
                     synthetic=True, device="cpu", precision=precision, val_loss_every=0, sample_every=0, overfit_single_batch=1,
                     output_log_dir=str(tmp_path))
    tr = Trainer(args)
    losses = [tr.train_step()["loss"] for _ in range(5)]
    assert all(torch.isfinite(torch.tensor(l)) for l in losses)
    assert losses[-1] < losses[0]


def test_record_run_result_parses_the_trainers_own_lines(tmp_path):
    """The reporting tool reads the trainer's step / val-loss lines and the eval tool's HellaSwag line."""
    import record_run_result as rr
    from llm_mojo_b200.utils.logger import format_step_line
    log = tmp_path / "train.log"
    lines = ["val loss 10.900000"]
    for s in range(1, 9):
        lines.append(format_step_line(s, 8, 11.0 - s * 0.1, float("nan"), 1.5, float("nan"), 3e-4, 100.0 + s, 0.4, "bf16", 5000 + s, 99.0))
    lines.append("val loss 10.100000")
    log.write_text("\n".join(lines) + "\n")
    ev = tmp_path / "eval.log"
    ev.write_text("HellaSwag: 2965/10042 = 0.2953\n")
    res = rr.record("tiny", str(log), str(ev), str(tmp_path / "results"))
    assert res["steps_run"] == 8 and res["val_loss_final"] == 10.1 and res["val_loss_best"] == 10.1
    assert abs(res["ms_per_step_median"] - 106.5) < 1e-6
    lo, hi = res["hellaswag"]["wilson95"]
    assert lo < 0.2953 < hi and hi - lo < 0.02
    assert "| tiny | 8/8 |" in rr.table(str(tmp_path / "results"))


def test_gate_lock_serialises_and_reports_holders(tmp_path, monkeypatch):
    import subprocess, time
    lock = str(tmp_path / "gate.lock")
    env = dict(os.environ, LLMB_GATE_LOCK=lock)
    gate = os.path.join(ROOT, "gate.py")
    holder = subprocess.Popen([sys.executable, gate, "run", sys.executable, "-c", "import time; time.sleep(3)"], env=env,
                              stdout=subprocess.PIPE, text=True)
    time.sleep(1.0)
    st = subprocess.run([sys.executable, gate, "status"], env=env, capture_output=True, text=True)
    assert "held by" in st.stdout and "gate.py run" in st.stdout and st.stdout.count("pid=") >= 2   # runner and its child
    t0 = time.time()
    second = subprocess.run([sys.executable, gate, "run", sys.executable, "-c", "print('second ran')"], env=env,
                            capture_output=True, text=True, timeout=60)
    assert "second ran" in second.stdout and time.time() - t0 > 1.0       # it had to wait for the holder
    holder.wait(timeout=30)


def test_launch_list_summary_buckets_time_dram_and_tensor_pipe(tmp_path):
    """profile_gpt2 --families reads a profiler launch list (csv): per kernel family the time and, when the capture has
    them, the DRAM bytes and the time-weighted tensor-pipe activity."""
    import csv
    import profile_gpt2 as pg
    hdr = ["ID", "Process ID", "Process Name", "Host Name", "Kernel Name", "Context", "Stream", "Block Size", "Grid Size",
           "Device", "CC", "Section Name", "Metric Name", "Metric Unit", "Metric Value"]
    rows = [hdr]

    def add(i, name, metric, unit, value):
        rows.append([str(i), "1", "py", "h", name, "1", "7", "(1,1,1)", "(1,1,1)", "0", "10.0", "x", metric, unit, value])
    tp = "sm__pipe_tensor_cycles_active.avg.pct_of_peak_sustained_elapsed"
    add(0, "gemm_pair_kernel<0,1>", "gpu__time_duration.sum", "us", "100"); add(0, "gemm_pair_kernel<0,1>", "dram__bytes_read.sum", "Mbyte", "50")
    add(0, "gemm_pair_kernel<0,1>", tp, "%", "80")
    add(1, "gemm_pair_kernel<0,4>", "gpu__time_duration.sum", "us", "300"); add(1, "gemm_pair_kernel<0,4>", tp, "%", "40")
    add(2, "attn_fwd3_kernel", "gpu__time_duration.sum", "ns", "200000"); add(2, "attn_fwd3_kernel", "dram__bytes_write.sum", "Kbyte", "1000")
    path = tmp_path / "launches.csv"
    with open(path, "w", newline="") as f:
        csv.writer(f).writerows(rows)
    res = pg.summarize_launch_csv(str(path))
    assert res["matmul"] == 400.0 and res["attention"] == 200.0
    assert res["detail"]["matmul"] == {"launches": 2, "dram_mb": 50.0, "tensor_pipe_pct": 50.0}
    assert abs(res["detail"]["attention"]["dram_mb"] - 1.0) < 1e-9
