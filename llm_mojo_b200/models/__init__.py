"""Model families.  GPT-2 (and the GPT-3 channel ladder, which shares the architecture)."""
from .gpt2 import GPT2, random_init_params  # noqa: F401
