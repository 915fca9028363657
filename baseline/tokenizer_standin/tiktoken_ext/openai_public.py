"""Offline stand-in for tiktoken's `tiktoken_ext.openai_public` plugin module.

The reference's PyTorch trainer builds the GPT-2 encoding at start-up
(`train_gpt2.py:2018`, through `data/utils.py:get_gpt2_encoding`), and the real plugin downloads
`vocab.bpe` / `encoder.json` for that.  On a machine without network access the benchmark's
reference arm puts this directory first on PYTHONPATH, so the unmodified trainer gets an encoding
of the right size (50257 tokens, end-of-text = 50256) without any download.  The merge table is
synthetic: 256 single bytes plus 50000 two-byte tokens.  Token ids it produces are NOT GPT-2's;
it only serves runs that never tokenize real text (synthetic token shards, sampling off).
"""

ENDOFTEXT = "<|endoftext|>"


def gpt2():
    ranks = {bytes([i]): i for i in range(256)}
    n = 256
    for a in range(256):
        for b in range(256):
            if n == 50256:
                break
            ranks[bytes([a, b])] = n
            n += 1
    return {
        "name": "gpt2",
        "explicit_n_vocab": 50257,
        "pat_str": r"""\s+|\S+""",
        "mergeable_ranks": ranks,
        "special_tokens": {ENDOFTEXT: 50256},
    }


ENCODING_CONSTRUCTORS = {"gpt2": gpt2}
