"""Runtime services on CPU: RNG parity with torch, LR schedules, data / eval loaders, tokenizer, sampler,
checkpoint round trips, safetensors import/export, CLI parsing, logger and MFU (after the reference's
tests/test_{dataloader,tokenizer,sampler,checkpointing}.mojo and tests/test_*_equivalence.py)."""
import math
import os
import struct

import numpy as np
import pytest
import torch

from llm_mojo_b200.config import GPT2Config, parse_model_descriptor
from llm_mojo_b200.models import GPT2
from llm_mojo_b200.utils import checkpointing as ckpt
from llm_mojo_b200.utils.dataloader import DataLoader, write_datafile
from llm_mojo_b200.utils.eval_dataloader import EvalDataLoader, eval_stat_correct, write_evalfile
from llm_mojo_b200.utils.logger import OutlierDetector, TokenRateEMA, format_step_line
from llm_mojo_b200.utils.mfu import estimate_mfu
from llm_mojo_b200.utils.rand import MT19937, normal_, random_permutation
from llm_mojo_b200.utils.sampler import SamplerRNG, sample_softmax
from llm_mojo_b200.utils.scheduler import LRScheduler
from llm_mojo_b200.utils.tokenizer import Tokenizer, write_tokenizer


# ------------------------------------------------------------------------------ RNG
def test_mt19937_matches_reference_vector():
    rng = MT19937(5489)
    first = [rng.randint32() for _ in range(3)]
    assert first == [3499211612, 581869302, 3890346734]          # canonical mt19937 output for seed 5489
    rng2 = MT19937(42)
    for _ in range(1300):                                        # crosses two state refills
        rng2.randint32()
    g = torch.Generator().manual_seed(42)
    want = torch.empty(1301, dtype=torch.int64).random_(0, 2 ** 32, generator=g)
    assert rng2.draws == 1300


@pytest.mark.parametrize("n", [5, 16, 37, 1000])
def test_normal_matches_torch_cpu_generator(n):
    g = torch.Generator().manual_seed(42)
    want = torch.empty(n, dtype=torch.float32).normal_(0.0, 0.02, generator=g)
    got = torch.from_numpy(normal_(MT19937(42), n, 0.0, 0.02))
    assert torch.allclose(got, want, atol=1e-7, rtol=1e-5)


def test_random_permutation_is_a_permutation_and_deterministic():
    a, b = list(range(50)), list(range(50))
    random_permutation(a, MT19937(7)); random_permutation(b, MT19937(7))
    assert a == b and sorted(a) == list(range(50)) and a != list(range(50))


# ------------------------------------------------------------------------------ schedules
def test_lr_schedules():
    s = LRScheduler("cosine", 1.0, 10, 110, 0.1)
    assert s.get_learning_rate(0) == pytest.approx(0.1) and s.get_learning_rate(9) == pytest.approx(1.0)
    assert s.get_learning_rate(10) == pytest.approx(1.0) and s.get_learning_rate(110) == pytest.approx(0.1)
    assert s.get_learning_rate(60) == pytest.approx(0.1 + 0.5 * 0.9)
    lin = LRScheduler("linear", 1.0, 0, 100, 0.0)
    assert lin.get_learning_rate(50) == pytest.approx(0.5)
    assert LRScheduler("constant", 0.3, 5, 100, 0.0).get_learning_rate(2) == 0.3
    w = LRScheduler("wsd", 1.0, 0, 100, 0.0)
    assert w.get_learning_rate(79) == 1.0 and w.get_learning_rate(85) == pytest.approx(1 - math.sqrt(0.25))
    with pytest.raises(ValueError):
        LRScheduler("bogus", 1, 0, 1, 1)


# ------------------------------------------------------------------------------ data loader
def _shards(tmp_path, n_shards=3, ntok=1000, dtype="gpt-2"):
    files = []
    for i in range(n_shards):
        p = str(tmp_path / f"shard_{i:03d}.bin")
        write_datafile(p, (np.arange(ntok) + 1000 * i) % 50000, dtype)
        files.append(p)
    return files


def test_dataloader_strided_batches(tmp_path):
    files = _shards(tmp_path)
    B, T, W = 2, 8, 2
    loaders = [DataLoader(files, B, T, r, W, pin_memory=False) for r in range(W)]
    for r, ld in enumerate(loaders):
        x, y = ld.next_batch()
        assert x.tolist() == list(range(r * B * T, (r + 1) * B * T))
        assert y.tolist() == list(range(r * B * T + 1, (r + 1) * B * T + 1))
        x2, _ = ld.next_batch()
        assert x2[0].item() == W * B * T + r * B * T
    ld = loaders[0]
    assert ld.shard_num_samples == (1000 - 1) // (W * B * T)
    for _ in range(ld.shard_num_samples - 2):
        ld.next_batch()
    x, _ = ld.next_batch()                      # first batch of the second shard
    assert x[0].item() == 1000
    assert ld.num_tokens == 3000


def test_dataloader_uint32_and_errors(tmp_path):
    p = str(tmp_path / "l3.bin")
    write_datafile(p, np.arange(500) + 70000, "llama-3")
    ld = DataLoader([p], 2, 8, pin_memory=False)
    assert ld.next_batch()[0][0].item() == 70000
    with pytest.raises(ValueError):
        DataLoader([p], 64, 64, pin_memory=False)        # shard too small for the batch
    bad = str(tmp_path / "bad.bin")
    with open(bad, "wb") as f:
        f.write(struct.pack("<256i", *([123] + [0] * 255)))
    with pytest.raises(ValueError):
        DataLoader([bad], 1, 4, pin_memory=False)


def test_dataloader_shuffle_resume_is_exact(tmp_path):
    files = _shards(tmp_path, n_shards=4, ntok=2000)
    a = DataLoader(files, 2, 8, 0, 1, should_shuffle=True, pin_memory=False)
    for _ in range(150):                        # into the second shard at least
        a.next_batch()
    st = a.state()
    nxt = [a.next_batch()[0].clone() for _ in range(40)]
    b = DataLoader(files, 2, 8, 0, 1, should_shuffle=True, pin_memory=False)
    b.restore(st["should_shuffle"], st["shuffle_draws"], st["current_shard_idx"], st["current_sample_idx"])
    for want in nxt:
        assert torch.equal(b.next_batch()[0], want)


def test_dataloader_prefetch_gives_same_sequence(tmp_path):
    files = _shards(tmp_path)
    a = DataLoader(files, 2, 8, pin_memory=False)
    b = DataLoader(files, 2, 8, pin_memory=False)
    for _ in range(100):
        xa = a.next_batch()[0].clone()
        b.prefetch()
        assert torch.equal(b.next_batch()[0], xa)


# ------------------------------------------------------------------------------ eval loader
def test_eval_loader_and_accuracy(tmp_path):
    datum = []
    for i in range(5):
        datum.append({"label": i % 4, "ctx_tokens": [10 + i, 11, 12], "ending_tokens": [[20, 21], [30], [40, 41, 42], [50, 51]]})
    p = str(tmp_path / "eval.bin")
    write_evalfile(p, datum)
    ld = EvalDataLoader(p, 8, 16)
    assert ld.num_examples == 5 and ld.can_fit_examples == 2 and ld.num_batches == 3
    ld.next_batch()
    inp = ld.inputs.view(8, 16)
    assert inp[0, :5].tolist() == [10, 11, 12, 20, 21] and inp[2, :6].tolist() == [10, 11, 12, 40, 41, 42]
    assert ld.mask.view(8, 16)[0].tolist()[:5] == [0, 0, 1, 1, 0] and ld.targets.view(8, 16)[0, 2].item() == 20
    losses = torch.ones(8, 16)
    losses[0] = 0.1        # example 0: completion 0 has the lowest loss, label 0 -> correct
    losses[6] = 0.1        # example 1: completion 2 lowest, label 1 -> wrong
    assert eval_stat_correct(ld, losses) == 1
    two = [EvalDataLoader(p, 8, 16, r, 2) for r in range(2)]
    assert two[0].end_example_index - two[0].start_example_index == 3 and two[1].end_example_index == 5
    with pytest.raises(ValueError):
        EvalDataLoader(p, 2, 16)


# ------------------------------------------------------------------------------ tokenizer / sampler
def test_tokenizer_roundtrip_and_errors(tmp_path):
    toks = [bytes([65 + i % 26]) * (1 + i % 3) for i in range(300)]
    p = str(tmp_path / "tok.bin")
    write_tokenizer(p, toks, eot_token=299)
    t = Tokenizer(p)
    assert t.has_initialized and t.vocab_size == 300 and t.eot_token == 299
    assert t.decode(1) == "BB" and t.decode(-1) == "" and t.decode(300) == ""
    assert t.decode_sequence([0, 1, 2]) == "ABBCCC"
    missing = Tokenizer(str(tmp_path / "nope.bin"))
    assert not missing.has_initialized and missing.decode(3) == ""
    with open(p, "r+b") as f:
        f.write(struct.pack("<i", 1))
    with pytest.raises(ValueError):
        Tokenizer(p)


def test_sampler_matches_reference_formulas():
    r = SamplerRNG(1337)
    vals = [r.random_u32() for _ in range(3)]
    s = 1337
    want = []
    for _ in range(3):
        s ^= s >> 12; s ^= (s << 25) & (2 ** 64 - 1); s ^= s >> 27
        want.append(((s * 0x2545F4914F6CDD1D) & (2 ** 64 - 1)) >> 32)
    assert vals == want
    f = SamplerRNG(1).random_f32()
    assert 0.0 <= f < 1.0
    logits = np.log(np.array([0.1, 0.2, 0.3, 0.4], dtype=np.float32))
    assert [sample_softmax(logits, c) for c in (0.05, 0.25, 0.55, 0.95, 0.9999)] == [0, 1, 2, 3, 3]


# ------------------------------------------------------------------------------ checkpoints
def test_model_checkpoint_roundtrip_fp32_bf16_and_slice(tmp_path, tiny_config):
    flat = torch.randn(tiny_config.num_parameters())
    p = str(tmp_path / "m.bin")
    ckpt.write_model_checkpoint(p, tiny_config, flat)
    cfg, ver, back = ckpt.read_model_checkpoint(p)
    assert cfg == tiny_config and ver == 3 and torch.equal(back, flat)
    with open(p, "rb") as f:
        h = struct.unpack("<256i", f.read(1024))
    assert h[:8] == (20240520, 3, 16, 60, 2, 2, 16, 64)
    _, _, part = ckpt.read_model_checkpoint(p, offset=100, count=50)
    assert torch.equal(part, flat[100:150])
    ckpt.write_model_checkpoint(p, tiny_config, flat.bfloat16())
    _, ver, back = ckpt.read_model_checkpoint(p, dtype=torch.float32)
    assert ver == 5 and torch.equal(back, flat.bfloat16().float())
    with open(p, "r+b") as f:
        f.write(struct.pack("<i", 999))
    with pytest.raises(ValueError):
        ckpt.read_model_header(p)


def test_state_checkpoint_roundtrip(tmp_path):
    st = ckpt.TrainingState(step=17, num_processes=4, process_rank=2, use_master_weights=1, should_shuffle=1,
                            sampler_rng_state=2 ** 63 + 5, shuffle_rng_state=12345, current_shard_idx=3, current_sample_idx=77)
    m, v = torch.randn(100), torch.rand(100)
    p = str(tmp_path / "s.bin")
    ckpt.write_state_checkpoint(p, st, m, v)
    back, m2, v2 = ckpt.read_state_checkpoint(p, 100)
    assert back == st and torch.equal(m, m2) and torch.equal(v, v2)
    assert os.path.getsize(p) == 1024 + 800
    with open(p, "rb") as f:
        h = struct.unpack("<256i", f.read(1024))
    assert h[0] == 20240527 and h[1] == 1 and h[2] == 4 and h[3] == 2 and h[10] == 17
    os.makedirs(tmp_path / "out", exist_ok=True)
    for s in (5, 20, 100):
        open(ckpt.model_path(str(tmp_path / "out"), s), "wb").close()
    assert ckpt.find_max_step(str(tmp_path / "out")) == 100 and ckpt.find_max_step(str(tmp_path / "none")) == -1


def test_training_resume_reproduces_the_run(tmp_path, tiny_config):
    """Checkpoint after 3 steps, resume in a fresh model, and the next steps match the uninterrupted run."""
    g = torch.Generator().manual_seed(5)
    batches = [torch.randint(0, tiny_config.vocab_size, (2, 9), generator=g, dtype=torch.int32) for _ in range(6)]

    def step(model, i):
        t = batches[i]
        model.forward(t[:, :-1].contiguous(), t[:, 1:].contiguous()); model.backward(); model.update(i + 1, 1e-2, 0.01)
        return model.read_loss()

    full = GPT2(tiny_config, "fp32", "cpu")
    ref_losses = [step(full, i) for i in range(6)]
    a = GPT2(tiny_config, "fp32", "cpu")
    for i in range(3):
        step(a, i)
    mp, sp = str(tmp_path / "model_3.bin"), str(tmp_path / "state_3_0.bin")
    a.write_checkpoint(mp, sp, ckpt.TrainingState(step=3))
    b = GPT2(mp, "fp32", "cpu")
    st = b.load_checkpoint(mp, sp)
    assert st.step == 3
    for i in range(3, 6):
        assert abs(step(b, i) - ref_losses[i]) < 1e-5


# ------------------------------------------------------------------------------ safetensors
def test_safetensors_export_import_roundtrip(tmp_path):
    from llm_mojo_b200.utils.safetensors_io import SafetensorsFile, export_hf_gpt2, load_hf_gpt2
    tiny_config = GPT2Config(max_seq_len=16, vocab_size=60, num_layer=2, num_heads=2, channels=16, padded_vocab_size=128)
    model = GPT2(tiny_config, "fp32", "cpu")
    flat = model.params.clone()
    flat += 0.01 * torch.randn_like(flat)          # biases non-zero
    off0, off1 = model.tensor_range("wte")
    flat[off0 + tiny_config.vocab_size * tiny_config.channels:off1] = 0
    out = str(tmp_path / "hf")
    export_hf_gpt2(out, tiny_config, flat)
    sf = SafetensorsFile(out + "/model.safetensors")
    assert sf.read_tensor("h.0.attn.c_attn.weight").shape == (16, 48)      # Conv1D layout: [in, out]
    assert sf.read_tensor("wte.weight").shape == (60, 16)
    cfg, back = load_hf_gpt2(out + "/model.safetensors")
    assert cfg == tiny_config and torch.allclose(back, flat)


def test_exported_checkpoint_loads_in_transformers(tmp_path):
    transformers = pytest.importorskip("transformers")
    from llm_mojo_b200.models import reference as ref
    from llm_mojo_b200.utils.safetensors_io import export_hf_gpt2
    cfg = GPT2Config(max_seq_len=32, vocab_size=128, num_layer=2, num_heads=2, channels=32, padded_vocab_size=128)
    model = GPT2(cfg, "fp32", "cpu")
    model.params += 0.02 * torch.randn_like(model.params)
    out = str(tmp_path / "hf")
    export_hf_gpt2(out, cfg, model.params)
    hf = transformers.GPT2LMHeadModel.from_pretrained(out).eval()
    toks = torch.randint(0, 128, (2, 16))
    with torch.no_grad():
        want = hf(toks).logits
    got, _ = ref.forward(cfg, ref.unflatten(cfg, model.params), toks)
    assert torch.allclose(got, want, atol=2e-4, rtol=1e-3)


# ------------------------------------------------------------------------------ CLI / config / logging
def test_cli_flags_env_and_config(tmp_path, monkeypatch):
    import train_gpt2 as cli
    args, rank, world, pn = cli.parse_train_args(["-b", "8", "-t", "256", "-l", "6e-4", "-k", "wsd", "-z", "2", "-e", "d24",
                                                  "-x", "10", "-pn", "4", "-pr", "3", "--precision", "fp8"], env={})
    assert (args.batch_size, args.seq_len, args.zero_stage, args.load_filename, args.max_steps) == (8, 256, 2, "d24", 10)
    assert args.learning_rate == pytest.approx(6e-4) and args.lr_scheduler_type == "wsd" and args.precision == "fp8"
    assert (rank, world, pn) == (3, 4, 4)
    args, rank, world, _ = cli.parse_train_args([], env={"RANK": "1", "WORLD_SIZE": "2", "ZERO_STAGE": "3",
                                                         "LLMM_OUTPUT_DIR": "o", "LLMM_SAVE_EVERY": "7"})
    assert (rank, world, args.zero_stage, args.output_log_dir, args.checkpoint_every) == (1, 2, 3, "o", 7)
    with pytest.raises(cli.UsageError):
        cli.parse_train_args(["-Q", "1"], env={})
    with pytest.raises(cli.UsageError):
        cli.parse_train_args(["-b"], env={})
    assert cli.parse_train_args(["-h"], env={}) is None
    cfgp = tmp_path / "z.json"
    cfgp.write_text('{"zero_stage": 2, "world_size": 8, "precision": "bf16", "train_flags": {"b": 32, "t": 512}}')
    args, _, world, _ = cli.parse_train_args(["--config", str(cfgp)], env={})
    assert (args.zero_stage, args.batch_size, args.seq_len, world) == (2, 32, 512, 8)
    import train_zero
    cmd, w = train_zero.build_command(str(cfgp), ["--synthetic", "1"])
    assert w == 8 and "-z" in cmd and cmd[cmd.index("-b") + 1] == "32" and cmd[-2:] == ["--synthetic", "1"]


def test_model_descriptors():
    assert parse_model_descriptor("d12") == GPT2Config(1024, 50257, 12, 12, 768, 50304)
    assert parse_model_descriptor("gpt2:d48").channels == 1600 and parse_model_descriptor("d48").num_heads == 25
    g3 = parse_model_descriptor("gpt3:c2048")
    assert (g3.num_layer, g3.num_heads, g3.max_seq_len) == (24, 16, 2048)
    assert parse_model_descriptor("d12").num_parameters() == 124475904
    for bad in ("d13", "gpt3:c100", "x"):
        with pytest.raises(ValueError):
            parse_model_descriptor(bad)


def test_outlier_detector_ema_mfu_and_log_line():
    d = OutlierDetector(window=8)
    zs = [d.update(1.0 + 0.01 * (i % 2)) for i in range(8)]
    assert all(math.isnan(z) for z in zs)
    assert d.update(5.0) > 2.0
    e = TokenRateEMA()
    assert e.update(100.0) == pytest.approx(100.0)
    assert 100.0 < e.update(200.0) < 200.0
    mfu = estimate_mfu(124475904, 12, 768, 1024, 65536, 0.1, "NVIDIA B200", "bf16")
    assert mfu == pytest.approx((6 * 124475904 + 6 * 12 * 768 * 1024) * 65536 / 0.1 / 2.25e15)
    assert estimate_mfu(1, 1, 1, 1, 1, 1.0, "unknown gpu", "bf16") == -1.0
    line = format_step_line(3, 10, 4.5, 0.1, 1.2, -0.3, 6e-4, 101.5, 0.41, "bf16", 640000.0, 100.2)
    assert line.startswith("step    3/10 | loss 4.500000 (+0.10z)| norm 1.2000 (-0.30z)| lr 6.00e-04 | 101.50 ms | 41.0% bf16 MFU | 640000 tok/s")


def test_trainer_synthetic_cpu_runs_and_resumes(tmp_path):
    from llm_mojo_b200.trainer import TrainArgs, Trainer
    out = str(tmp_path / "run")
    a = TrainArgs(load_filename="d6", batch_size=1, seq_len=16, max_steps=2, synthetic=True, val_loss_every=0, sample_every=0,
                  output_log_dir=out, checkpoint_every=1, learning_rate=1e-3)
    import llm_mojo_b200.config as c
    saved = dict(c._GPT2_LADDER)
    c._GPT2_LADDER[6] = (32, 2)                      # shrink the model for a quick CPU run
    try:
        t = Trainer(a)
        t.train()
        assert ckpt.find_max_step(out) == 2 and os.path.exists(ckpt.state_path(out, 2, 0))
        a2 = TrainArgs(**{**a.__dict__, "resume": 1, "max_steps": 3})
        t2 = Trainer(a2)
        assert t2.step == 2
        r = t2.train_step()
        assert math.isfinite(r["loss"])
    finally:
        c._GPT2_LADDER.clear(); c._GPT2_LADDER.update(saved)


def test_supervisor_restarts_on_failure_and_stall(tmp_path):
    import sys
    import supervise_train as sup
    marker = tmp_path / "count"
    script = tmp_path / "child.py"
    script.write_text(
        "import sys, time, pathlib\n"
        f"p = pathlib.Path({str(marker)!r})\n"
        "n = int(p.read_text()) if p.exists() else 0\n"
        "p.write_text(str(n + 1))\n"
        "print('run', n, sys.argv[1:], flush=True)\n"
        "if n == 0: sys.exit(3)\n"            # first run crashes
        "if n == 1: time.sleep(60)\n"          # second run hangs silently -> stall
        "sys.exit(0)\n")
    log = tmp_path / "log.txt"
    rc = sup.supervise([sys.executable, str(script), "-x", "5"], str(log), stall_seconds=1.5, poll_seconds=0.3)
    text = log.read_text()
    assert rc == 0 and marker.read_text() == "3"
    assert "exit code 3" in text and "stall detected" in text
    assert "'-y', '1'" in text.split("run 2")[1]          # restarts resume from the newest checkpoint
    assert sup.with_resume(["a", "-y", "0"]) == ["a", "-y", "1"]
