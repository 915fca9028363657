#!/usr/bin/env python
"""TinyStories → token shards (shard 0 of the JSON archive is the validation split; ``data/tinystories.py``)."""
import glob
import json
import os

from data.common import download_file, tokenize_document, write_datafile

URL = "https://huggingface.co/datasets/roneneldan/TinyStories/resolve/main/TinyStories_all_data.tar.gz"
OUT = os.path.join(os.path.dirname(__file__), ".tinystories")


def main():
    os.makedirs(OUT, exist_ok=True)
    tar = os.path.join(OUT, "TinyStories_all_data.tar.gz")
    if not os.path.exists(tar):
        download_file(URL, tar)
    raw = os.path.join(OUT, "raw")
    if not os.path.isdir(raw):
        import tarfile
        os.makedirs(raw)
        with tarfile.open(tar) as t:
            t.extractall(raw)
    for split, files in (("val", sorted(glob.glob(raw + "/*.json"))[:1]), ("train", sorted(glob.glob(raw + "/*.json"))[1:])):
        tokens = []
        for fn in files:
            for ex in json.load(open(fn)):
                tokens.extend(tokenize_document(ex["story"].strip()))
        write_datafile(os.path.join(OUT, f"TinyStories_{split}.bin"), tokens)


if __name__ == "__main__":
    main()
