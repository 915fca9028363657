"""Dataset preparation: download, GPT-2 tokenisation and shard writing (needs network access and tiktoken)."""
