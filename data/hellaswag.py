#!/usr/bin/env python
"""HellaSwag validation set → ``data/.hellaswag/hellaswag_val.bin`` in the multiple-choice eval format
(``data/hellaswag.py`` of the reference): context tokens plus four tokenised endings (each prefixed by a space)."""
import json
import os

from data.common import download_file, get_gpt2_encoding, write_evalfile

URL = "https://raw.githubusercontent.com/rowanz/hellaswag/master/data/hellaswag_val.jsonl"
OUT = os.path.join(os.path.dirname(__file__), ".hellaswag")


def render(example):
    enc = get_gpt2_encoding()
    return {"label": int(example["label"]), "ctx_tokens": enc.encode(example["ctx"]),
            "ending_tokens": [enc.encode(" " + e) for e in example["endings"]]}


def main():
    os.makedirs(OUT, exist_ok=True)
    raw = os.path.join(OUT, "hellaswag_val.jsonl")
    if not os.path.exists(raw):
        download_file(URL, raw)
    datum = [render(json.loads(line)) for line in open(raw)]
    write_evalfile(os.path.join(OUT, "hellaswag_val.bin"), datum)


if __name__ == "__main__":
    main()
