"""Shared helpers of the dataset scripts (``data/utils.py`` in the reference): GPT-2 encoding, download
with a progress bar, and the shard / eval-file writers (re-exported from the package so the on-disk
formats have a single implementation)."""
from __future__ import annotations

import functools
import os

from llm_mojo_b200.utils.dataloader import write_datafile          # noqa: F401
from llm_mojo_b200.utils.eval_dataloader import write_evalfile     # noqa: F401


@functools.lru_cache(maxsize=1)
def get_gpt2_encoding():
    import tiktoken
    return tiktoken.get_encoding("gpt2")


def download_file(url: str, path: str, chunk: int = 1 << 20) -> None:
    import requests
    from tqdm import tqdm
    os.makedirs(os.path.dirname(os.path.abspath(path)), exist_ok=True)
    with requests.get(url, stream=True, timeout=60) as r:
        r.raise_for_status()
        total = int(r.headers.get("content-length", 0))
        with open(path, "wb") as f, tqdm(total=total, unit="B", unit_scale=True, desc=os.path.basename(path)) as bar:
            for block in r.iter_content(chunk_size=chunk):
                bar.update(f.write(block))


def tokenize_document(text: str):
    """<|endoftext|> followed by the document's tokens, as uint16-range ints."""
    enc = get_gpt2_encoding()
    return [enc.eot_token] + enc.encode_ordinary(text)
