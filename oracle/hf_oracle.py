"""TEST INFRASTRUCTURE ONLY - the live Hugging Face tokenizers that define "bit-exact".

Only ``tests/``, ``__graft_entry__.smoke()`` and ``bench.py``'s CPU-baseline legs may import
this module; nothing under ``dnatok_b200/`` does.

The arithmetic the reference checks itself against lives in the third-party Hugging Face
``tokenizers`` package (Rust wheel; the reference pins tokenizers==0.22.1, this image has
0.22.2).  The reference calls it at ``src/dna_tokenizer.py:1708-1714`` (padded batch call),
``src/gputok_bpe_backend.py:653-656`` (fallback) and ``tests/test_gputok_bpe_backend.py:108``
(per-sequence parity).  The builders below construct, for each of the five benchmark shapes,
the HF tokenizer whose output is the parity target.
"""
from __future__ import annotations

import gzip
import itertools
import json
import os
from typing import Iterable

SPECIALS = ["[PAD]", "[UNK]", "[CLS]", "[SEP]", "[MASK]"]


def _wrap(tok, model_max_length: int = 1 << 30):
    from transformers import PreTrainedTokenizerFast
    return PreTrainedTokenizerFast(
        tokenizer_object=tok, pad_token="[PAD]", unk_token="[UNK]", cls_token="[CLS]",
        sep_token="[SEP]", mask_token="[MASK]", model_max_length=model_max_length)


def _template(tok):
    from tokenizers.processors import TemplateProcessing
    tok.post_processor = TemplateProcessing(
        single="[CLS] $A [SEP]", special_tokens=[("[CLS]", 2), ("[SEP]", 3)])


def char_vocab() -> dict:
    v = {s: i for i, s in enumerate(SPECIALS)}
    for c in "ACGTN":
        v[c] = len(v)
    return v


def char_tokenizer(raw: bool = False):
    """Config 1: WordLevel over {specials, A, C, G, T, N}, one token per character,
    ``[CLS] seq [SEP]``."""
    from tokenizers import Tokenizer, Regex
    from tokenizers.models import WordLevel
    from tokenizers.pre_tokenizers import Split
    tok = Tokenizer(WordLevel(char_vocab(), unk_token="[UNK]"))
    tok.pre_tokenizer = Split(Regex("."), "isolated")
    _template(tok)
    return tok if raw else _wrap(tok)


def kmer_vocab(k: int = 6) -> dict:
    v = {s: i for i, s in enumerate(SPECIALS)}
    for t in itertools.product("ACGT", repeat=k):
        v["".join(t)] = len(v)
    for c in "ACGTN":
        v[c] = len(v)
    return v


def kmer_tokenizer(k: int = 6, raw: bool = False):
    """Config 2: non-overlapping k-mers; a window holding anything but ACGT, and the
    ``len % k`` tail, fall back to single characters.  No special tokens."""
    from tokenizers import Tokenizer, Regex
    from tokenizers.models import WordLevel
    from tokenizers.pre_tokenizers import Split, Sequence
    tok = Tokenizer(WordLevel(kmer_vocab(k), unk_token="[UNK]"))
    tok.pre_tokenizer = Sequence([
        Split(Regex(".{1,%d}" % k), "isolated"),
        Split(Regex("[ACGT]{%d}|." % k), "isolated"),
    ])
    return tok if raw else _wrap(tok)


def byte_tokenizer(vocab_size: int = 512, raw: bool = False):
    """Config 4 (fast form): id = code point, as ``Evo2ByteTokenizer`` of the reference
    (``src/dnatok_compat.py:181-218``) defines it; pad = chr(1), unk = chr(0)."""
    from tokenizers import Tokenizer, Regex
    from tokenizers.models import WordLevel
    from tokenizers.pre_tokenizers import Split
    from transformers import PreTrainedTokenizerFast
    vocab = {chr(i): i for i in range(vocab_size)}
    tok = Tokenizer(WordLevel(vocab, unk_token=chr(0)))
    tok.pre_tokenizer = Split(Regex("[\\s\\S]"), "isolated")
    if raw:
        return tok
    return PreTrainedTokenizerFast(tokenizer_object=tok, pad_token=chr(1), unk_token=chr(0),
                                   model_max_length=1 << 30)


def train_bpe(lines: Iterable[str], vocab_size: int):
    """Configs 3 and 5: BPE + Whitespace pre-tokenizer + BpeTrainer, ``[CLS] seq [SEP]``."""
    from tokenizers import Tokenizer
    from tokenizers.models import BPE
    from tokenizers.pre_tokenizers import Whitespace
    from tokenizers.trainers import BpeTrainer
    tok = Tokenizer(BPE(unk_token="[UNK]"))
    tok.pre_tokenizer = Whitespace()
    trainer = BpeTrainer(vocab_size=vocab_size, special_tokens=SPECIALS, show_progress=False)
    tok.train_from_iterator(lines, trainer=trainer)
    _template(tok)
    return tok


GOLDEN_DIR = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))),
                          "tests", "golden")


def load_tokenizer_json(name: str) -> dict:
    """Read a committed ``tokenizer.json`` fixture (gzip) by stem, e.g. ``bpe4096``."""
    with gzip.open(os.path.join(GOLDEN_DIR, name + ".tokenizer.json.gz"), "rt") as f:
        return json.load(f)


def bpe_tokenizer(name: str, raw: bool = False):
    from tokenizers import Tokenizer
    tok = Tokenizer.from_str(json.dumps(load_tokenizer_json(name)))
    return tok if raw else _wrap(tok)
