"""Sub-word tokenisation for the byte-pair-encoded model variants.

The reference always asks ``tiktoken`` for the GPT-2 vocabulary
(reference ``dicee/knowledge_graph.py:103``), which needs a download.  Here the GPT-2
encoder is used only when its vocabulary is already cached locally (or when
``DICE_B200_TIKTOKEN=1`` forces the attempt); otherwise a self-contained UTF-8 byte
tokenizer with the same four-method interface (``encode``, ``decode``, ``encode_batch``,
``n_vocab``) takes its place, so the BPE code paths run without a network.
"""
from __future__ import annotations

import os
from typing import List, Sequence


class ByteTokenizer:
    """One token per UTF-8 byte; ``n_vocab`` = 256."""

    name = "utf8-bytes"
    n_vocab = 256

    def encode(self, text: str) -> List[int]:
        return list(str(text).encode("utf-8"))

    def encode_batch(self, texts: Sequence[str]) -> List[List[int]]:
        return [self.encode(t) for t in texts]

    def decode(self, tokens: Sequence[int]) -> str:
        return bytes(int(t) & 0xFF for t in tokens).decode("utf-8", errors="replace")


_CACHED = None


def get_tokenizer():
    """Return the process-wide tokenizer (GPT-2 BPE if locally available, else bytes)."""
    global _CACHED
    if _CACHED is not None:
        return _CACHED
    enc = None
    cache_dir = os.environ.get("TIKTOKEN_CACHE_DIR") or os.environ.get("DATA_GYM_CACHE_DIR")
    want = os.environ.get("DICE_B200_TIKTOKEN") == "1" or (cache_dir and os.path.isdir(cache_dir)
                                                          and len(os.listdir(cache_dir)) > 0)
    if want:
        try:
            import tiktoken
            enc = tiktoken.get_encoding("gpt2")
        except Exception:  # no vocabulary on this machine
            enc = None
    _CACHED = enc if enc is not None else ByteTokenizer()
    return _CACHED
