#!/usr/bin/env python
"""Tiny Shakespeare → ``data/.tinyshakespeare/tiny_shakespeare_{train,val}.bin`` (first 32768 tokens are
the validation split, as in ``data/tinyshakespeare.py`` of the reference)."""
import os

from data.common import download_file, get_gpt2_encoding, write_datafile

URL = "https://raw.githubusercontent.com/karpathy/char-rnn/master/data/tinyshakespeare/input.txt"
OUT = os.path.join(os.path.dirname(__file__), ".tinyshakespeare")


def main():
    os.makedirs(OUT, exist_ok=True)
    raw = os.path.join(OUT, "tiny_shakespeare.txt")
    if not os.path.exists(raw):
        download_file(URL, raw)
    text = open(raw).read()
    enc = get_gpt2_encoding()
    parts = text.split("\n\n")
    tokens = []
    for s in parts:
        tokens.append(enc.eot_token)
        tokens.extend(enc.encode_ordinary(s + "\n\n"))
    write_datafile(os.path.join(OUT, "tiny_shakespeare_val.bin"), tokens[:32768])
    write_datafile(os.path.join(OUT, "tiny_shakespeare_train.bin"), tokens[32768:])


if __name__ == "__main__":
    main()
