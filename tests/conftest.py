import os
import sys

import pytest
import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run on the B200 box)")
    config.addinivalue_line("markers", "slow: takes minutes on host cores (the full-size 124M CPU configuration)")


def pytest_collection_modifyitems(config, items):
    if not os.environ.get("LLMB_RUN_SLOW"):
        slow = pytest.mark.skip(reason="slow: set LLMB_RUN_SLOW=1 (minutes on host cores)")
        for item in items:
            if "slow" in item.keywords:
                item.add_marker(slow)
    if torch.cuda.is_available():
        return
    skip = pytest.mark.skip(reason="no CUDA device")
    for item in items:
        if "gpu" in item.keywords:
            item.add_marker(skip)


@pytest.fixture(scope="session")
def tiny_config():
    from llm_mojo_b200.config import GPT2Config
    return GPT2Config(max_seq_len=16, vocab_size=60, num_layer=2, num_heads=2, channels=16, padded_vocab_size=64)


# tolerances by dtype / device, after the reference's tests/_dtypes.py:24-30
TOL = {("fp32", "cpu"): (1e-6, 1e-5), ("fp32", "cuda"): (2e-5, 1e-4), ("bf16", "cuda"): (5e-3, 2e-2)}
