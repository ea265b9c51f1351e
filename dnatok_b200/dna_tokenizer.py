"""``DNATok``-compatible facade over the CUDA kernels.

Mirrors the part of the reference's ``DNATok`` (``src/dna_tokenizer.py``) that lies on the
tokenisation path, with the same names, argument meaning and error behaviour:

* ``DNATok(embedder, padding_side="left", normalize_case=False, handle_invalid_chars=False)``
  - ``embedder.tokenizer`` is the Hugging Face tokenizer (reference ``:110-243``);
* ``discover()`` (reference ``:864-1110``): picks the path and builds the tables - per-character
  LUT, k-mer table, or the BPE backend; sets ``use_ids_path``, ``kmer_k``, ``id_pad``, ``unk_id``,
  ``vocab_size``, ``bpe_backend``;
* ``encode_batch_to_ids(seqs)`` (reference ``:2049-2148``): CPU pinned int64 ``[B, T]``, no special
  tokens, ragged rows padded with the pad id on ``padding_side``, optional fixed ``token_len``;
  ``ValueError("No sequences provided.")`` on an empty batch;
* ``encode_batch_with_padding(seqs, max_tokens, pad_to_max=False, pad_multiple=16)`` (reference
  ``:2150-2236``): truncation to ``max_tokens`` tokens, width rounded up to ``pad_multiple``, ids in
  the narrowest integer dtype that holds the vocabulary, ``uint8`` mask; ``ValueError("Empty batch")``.

Where the reference computes on the CPU with numpy, everything here runs in the kernels; a
tokenizer the tables cannot express raises (the reference would fall back to the Hugging Face
tokenizer, which this library does not do).

``encode_batch_with_padding`` on a k-mer tokenizer keeps the reference's literal procedure (pad the
strings with ``N`` to the target width, encode, overwrite everything past ``ceil(len/k)`` with the
pad id), because for rows whose windows hold ``N`` that procedure - not the Hugging Face padding
rules - defines the reference's output.
"""
from __future__ import annotations

import logging
from typing import Any, List, Optional, Tuple

import numpy as np

from .tables import UnsupportedTokenizer, spec_from_tokenizer

_ALLOWED_UPPER = frozenset("ACGTN")
_ALLOWED_ALL = frozenset("ACGTNacgtn")


class DNATok:
    def __init__(self, embedder: Any, *args, padding_side: str = "left", normalize_case: bool = False,
                 handle_invalid_chars: bool = False, logger: Optional[logging.Logger] = None, **_unused) -> None:
        if padding_side not in ("left", "right"):
            raise ValueError("padding_side must be 'left' or 'right'")
        self.embedder = embedder
        self.tokenizer = getattr(embedder, "tokenizer", None)
        self.log = logger or logging.getLogger("DNATok")
        self.padding_side = padding_side
        self.normalize_case = normalize_case
        self.handle_invalid_chars = handle_invalid_chars
        self.token_len: Optional[int] = None
        self.use_ids_path = False
        self.kmer_k: Optional[int] = None
        self.id_pad = 0
        self.pad_id = 0
        self.unk_id = 0
        self.vocab_size = 0
        self.bpe_backend = None
        self._tok = None

    # ------------------------------------------------------------------ discovery
    def discover(self) -> None:
        from .tokenizer import B200Tokenizer
        self.use_ids_path = False
        self.kmer_k = None
        self.bpe_backend = None
        self._tok = None
        if self.tokenizer is None:
            raise UnsupportedTokenizer("embedder has no tokenizer")
        spec = spec_from_tokenizer(self.tokenizer)
        self.id_pad = self.pad_id = spec.specials.pad_id
        self.unk_id = spec.specials.unk_id
        self.vocab_size = spec.vocab_size
        if spec.kind == "bpe":
            from .gputok_bpe_backend import GPUTokBPEBackend
            self.bpe_backend = GPUTokBPEBackend(self.tokenizer, engine="dnatok")
            return
        self._tok = B200Tokenizer(spec)
        self.use_ids_path = True
        self.kmer_k = spec.k if spec.kind == "kmer" else None

    # ------------------------------------------------------------------ helpers
    def _normalize_and_clean_seqs(self, seqs: List[str]) -> List[str]:
        if not (self.normalize_case or self.handle_invalid_chars):
            return seqs
        allowed = _ALLOWED_UPPER if self.normalize_case else _ALLOWED_ALL
        out = []
        for s in seqs:
            if self.normalize_case:
                s = s.upper()
            if self.handle_invalid_chars and not allowed.issuperset(s):
                s = "".join(ch if ch in allowed else "N" for ch in s)
            out.append(s)
        return out

    def _encode_device(self, seqs: List[str], pad_left: bool, width: Optional[int] = None):
        tok = self._tok
        tok.padding_side = "left" if pad_left else "right"
        d_bytes, d_off, offsets = tok.to_device(seqs)
        kw = dict(padding="longest") if width is None else dict(padding="max_length", max_length=int(width))
        return tok.encode_device(d_bytes, d_off, host_offsets=offsets, add_special_tokens=False, **kw)

    # ------------------------------------------------------------------ public encode paths
    def encode_batch_to_ids(self, seqs: List[str]):
        import torch
        if not seqs:
            raise ValueError("No sequences provided.")
        if self._tok is None and self.bpe_backend is None:
            raise RuntimeError("discover() has not been run (or found no supported path)")
        seqs = self._normalize_and_clean_seqs(list(seqs))
        left = self.padding_side == "left"
        if not self.use_ids_path:
            ids_dev, mask_dev = self.bpe_backend.encode_batch(seqs, device="cuda")
            ids = ids_dev.cpu()
            if left:                                   # the backend pads on the right; move the padding
                lens = mask_dev.sum(dim=1).cpu()
                out = torch.full_like(ids, self.pad_id)
                T = ids.shape[1]
                for i, n in enumerate(lens.tolist()):
                    out[i, T - n:] = ids[i, :n]
                ids = out
        else:
            ids = self._encode_device(seqs, left)["input_ids"].cpu()
        if self.token_len is not None and ids.shape[1] < int(self.token_len):
            pad = torch.full((ids.shape[0], int(self.token_len) - ids.shape[1]), self.pad_id, dtype=ids.dtype)
            ids = torch.cat([pad, ids], dim=1) if left else torch.cat([ids, pad], dim=1)
        return ids.pin_memory() if torch.cuda.is_available() else ids

    def encode_batch_with_padding(self, seqs: List[str], max_tokens: int, pad_to_max: bool = False,
                                  pad_multiple: int = 16) -> Tuple[Any, Any]:
        import torch
        if not seqs:
            raise ValueError("Empty batch")
        if not self.use_ids_path or self._tok is None:
            raise RuntimeError("encode_batch_with_padding needs a per-character or k-mer tokenizer (run discover())")
        k = int(self.kmer_k) if self.kmer_k else 1
        max_chars = int(max_tokens) * k
        seqs = [s[:max_chars] for s in seqs]
        char_lengths = [len(s) for s in seqs]
        target_chars = max(char_lengths)
        if pad_to_max:
            target_chars = max(target_chars, max_chars)
        if k > 1 and target_chars % k:
            target_chars += k - target_chars % k
        target_tokens = target_chars // k
        if pad_multiple > 1 and target_tokens % pad_multiple:
            target_tokens += pad_multiple - target_tokens % pad_multiple
        target_chars = target_tokens * k
        left = self.padding_side == "left"

        seqs = self._normalize_and_clean_seqs(seqs)
        if k == 1:
            # one token per character: padding the strings with N and overwriting those columns with
            # the pad id equals padding with the pad id directly, which the kernel does in one pass
            ids = self._encode_device(seqs, left, width=target_tokens)["input_ids"].cpu()
        else:
            padded = [s.rjust(target_chars, "N") if left else s.ljust(target_chars, "N") for s in seqs]
            ids = self._encode_device(padded, left)["input_ids"].cpu()
        T = ids.shape[1]
        token_lengths = torch.tensor([(n + k - 1) // k for n in char_lengths], dtype=torch.long)
        cols = torch.arange(T, dtype=torch.long).unsqueeze(0)
        keep = cols >= (T - token_lengths.unsqueeze(1)) if left else cols < token_lengths.unsqueeze(1)
        max_id = max(int(self.vocab_size or 0) - 1, int(self.id_pad))
        dtype = torch.uint8 if max_id <= 255 else torch.int16 if max_id <= 32767 else \
            torch.int32 if max_id <= 2147483647 else torch.int64
        ids = ids.to(dtype)
        ids[~keep] = int(self.id_pad)
        return ids, keep.to(torch.uint8)
