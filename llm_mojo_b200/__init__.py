"""llm_mojo_b200 — a Blackwell (sm_100a) native GPT-2 training framework.

Layout
------
``config``      model hyper-parameters, model descriptors, precision axis
``models``      GPT-2 over flat parameter / gradient / optimizer buffers with
                explicit forward and backward passes (no autograd on the hot path)
``ops``         per-op entry points; CUDA tensors run hand-written sm_100a kernels
                from ``csrc`` (loaded through ctypes), CPU tensors run the fp32 oracle
``parallel``    process-per-GPU runtime: peer-memory symmetric buffers, fused
                collective kernels, DDP and ZeRO stages 1/2/3
``utils``       data/eval loaders, tokenizer, sampler, RNG, LR schedules,
                checkpoints (.bin / state / safetensors), MFU, tracing, logging
"""

from .config import GPT2Config, parse_model_descriptor, Precision  # noqa: F401

__version__ = "0.1.0"
