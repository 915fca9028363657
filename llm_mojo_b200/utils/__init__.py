"""Runtime services: RNG, schedules, loaders, tokenizer, sampler, checkpoints, MFU, tracing."""
