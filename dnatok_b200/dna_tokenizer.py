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
tokenizer, which this library does not do).  No string is rewritten in Python: ``normalize_case``
and ``handle_invalid_chars`` are a byte translation inside the native packer's one copy and a change
of the 256-entry id table, padding sides and masks come from the kernels, and the narrow id type
of ``encode_batch_with_padding`` is a cast on the device before the copy back.

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

_UPPER = bytes((c - 32 if 97 <= c <= 122 else c) for c in range(256))      # what str.upper() does to ASCII


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
        self._spec = None
        self._built_for = None

    # ------------------------------------------------------------------ discovery
    def discover(self) -> None:
        self.use_ids_path = False
        self.kmer_k = None
        self.bpe_backend = None
        self._tok = None
        self._built_for = None
        if self.tokenizer is None:
            raise UnsupportedTokenizer("embedder has no tokenizer")
        spec = spec_from_tokenizer(self.tokenizer)
        self._spec = spec
        self.id_pad = self.pad_id = spec.specials.pad_id
        self.unk_id = spec.specials.unk_id
        self.vocab_size = spec.vocab_size
        if spec.kind == "bpe":
            from .gputok_bpe_backend import GPUTokBPEBackend
            self.bpe_backend = GPUTokBPEBackend(self.tokenizer, engine="dnatok")
            return
        self.use_ids_path = True
        self.kmer_k = spec.k if spec.kind == "kmer" else None

    # ------------------------------------------------------------------ the flags as tables
    def _byte_table(self) -> Optional[bytes]:
        """The text rewriting of the reference's ``_normalize_and_clean_seqs`` (``src/dna_tokenizer.py:1535-1558``)
        as one 256-entry byte translation applied while the rows are packed: upper-casing for
        ``normalize_case``; for the BPE path (which has no invalid-character id) ``handle_invalid_chars``
        turns every character outside the alphabet into ``N``."""
        table = bytearray(range(256))
        if self.normalize_case:
            table = bytearray(_UPPER)
        if self.handle_invalid_chars and not self.use_ids_path:
            allowed = b"ACGTN" if self.normalize_case else b"ACGTNacgtn"
            for c in range(256):
                if table[c] not in allowed:
                    table[c] = ord("N")
        if bytes(table) == bytes(range(256)):
            return None
        return bytes(table)

    def _tokenizer(self):
        """The kernel front end for the current flags.  On the table paths ``handle_invalid_chars`` gives every
        character outside the alphabet the tokenizer's unknown id (the reference's ``invalid_char_id``,
        ``src/dna_tokenizer.py:926,948,1017``; the id of ``N`` only when there is no unknown id), which is a
        change of the 256-entry id table, not of the text (``:1810-1819``)."""
        from .tokenizer import B200Tokenizer
        key = (self.normalize_case, self.handle_invalid_chars)
        if self._tok is not None and self._built_for == key:
            return self._tok
        import copy
        spec = copy.copy(self._spec)
        if self.handle_invalid_chars:
            lut = np.array(spec.lut256, dtype=np.int32, copy=True)
            has_unk = getattr(self.tokenizer, "unk_token_id", None) is not None
            invalid_id = int(self.unk_id) if has_unk else int(lut[ord("N")])
            allowed = b"ACGTN" if self.normalize_case else b"ACGTNacgtn"
            for c in range(256):
                if c not in allowed:
                    lut[c] = invalid_id
            spec.lut256 = lut
        self._tok = B200Tokenizer(spec)
        self._built_for = key
        return self._tok

    def _encode_device(self, seqs: List[str], pad_left: bool, width: Optional[int] = None, *, pad_to_chars: int = 0,
                       trunc_to_chars: int = 0, mask_dtype=None, return_mask: bool = False):
        tok = self._tokenizer()
        tok.padding_side = "left" if pad_left else "right"
        d_bytes, d_off, offsets = tok.to_device(seqs, table=self._byte_table(), pad_to=pad_to_chars, pad_left=pad_left,
                                                trunc_to=trunc_to_chars)
        kw = dict(padding="longest") if width is None else dict(padding="max_length", max_length=int(width))
        if return_mask:
            kw.update(return_attention_mask=True, mask_dtype=mask_dtype)
        return tok.encode_device(d_bytes, d_off, host_offsets=offsets, add_special_tokens=False, **kw)

    # ------------------------------------------------------------------ public encode paths
    def encode_batch_to_ids(self, seqs: List[str]):
        import torch
        if not seqs:
            raise ValueError("No sequences provided.")
        if self._spec is None or (not self.use_ids_path and self.bpe_backend is None):
            raise RuntimeError("discover() has not been run (or found no supported path)")
        seqs = list(seqs)
        left = self.padding_side == "left"
        width = None
        if not self.use_ids_path:
            # the plug-in's own tokenizer, asked to pad on this object's side (the kernels pad on either side)
            tok = self.bpe_backend._tok
            old = tok.padding_side
            tok.padding_side = "left" if left else "right"
            try:
                d_bytes, d_off, offsets = tok.to_device(seqs, table=self._byte_table())
                ids = tok.encode_device(d_bytes, d_off, host_offsets=offsets, padding="longest",
                                        add_special_tokens=False, return_attention_mask=False)["input_ids"]
            finally:
                tok.padding_side = old
        else:
            ids = self._encode_device(seqs, left)["input_ids"]
        if self.token_len is not None and ids.shape[1] < int(self.token_len):
            pad = torch.full((ids.shape[0], int(self.token_len) - ids.shape[1]), self.pad_id, dtype=ids.dtype, device=ids.device)
            ids = torch.cat([pad, ids], dim=1) if left else torch.cat([ids, pad], dim=1)
        out = torch.empty(ids.shape, dtype=ids.dtype, pin_memory=torch.cuda.is_available())
        out.copy_(ids)
        return out

    def encode_batch_with_padding(self, seqs: List[str], max_tokens: int, pad_to_max: bool = False,
                                  pad_multiple: int = 16) -> Tuple[Any, Any]:
        import torch
        if not seqs:
            raise ValueError("Empty batch")
        if not self.use_ids_path or self._spec is None:
            raise RuntimeError("encode_batch_with_padding needs a per-character or k-mer tokenizer (run discover())")
        k = int(self.kmer_k) if self.kmer_k else 1
        max_chars = int(max_tokens) * k
        seqs = list(seqs)
        char_lengths = np.minimum(np.fromiter(map(len, seqs), dtype=np.int64, count=len(seqs)), max_chars)
        target_chars = int(char_lengths.max())
        if pad_to_max:
            target_chars = max(target_chars, max_chars)
        if k > 1 and target_chars % k:
            target_chars += k - target_chars % k
        target_tokens = target_chars // k
        if pad_multiple > 1 and target_tokens % pad_multiple:
            target_tokens += pad_multiple - target_tokens % pad_multiple
        target_chars = target_tokens * k
        left = self.padding_side == "left"
        max_id = max(int(self.vocab_size or 0) - 1, int(self.id_pad))
        dtype = torch.uint8 if max_id <= 255 else torch.int16 if max_id <= 32767 else \
            torch.int32 if max_id <= 2147483647 else torch.int64

        if k == 1:
            # one token per character: padding the strings with N and overwriting those columns with
            # the pad id equals padding with the pad id directly, which the kernel does in one pass,
            # mask included
            enc = self._encode_device(seqs, left, width=target_tokens, trunc_to_chars=max_chars, return_mask=True,
                                      mask_dtype=torch.uint8)
            return enc["input_ids"].to(dtype).cpu(), enc["attention_mask"].cpu()
        # k-mers: the rows are padded with N to the target width while they are packed (the window frame of a
        # left-padded row depends on it), encoded, and everything past ceil(len / k) tokens becomes padding
        ids = self._encode_device(seqs, left, pad_to_chars=target_chars, trunc_to_chars=max_chars)["input_ids"]
        T = ids.shape[1]
        token_lengths = torch.from_numpy((char_lengths + k - 1) // k).to(ids.device)
        cols = torch.arange(T, dtype=torch.long, device=ids.device).unsqueeze(0)
        keep = cols >= (T - token_lengths.unsqueeze(1)) if left else cols < token_lengths.unsqueeze(1)
        ids = torch.where(keep, ids, torch.full((), int(self.id_pad), dtype=ids.dtype, device=ids.device)).to(dtype)
        return ids.cpu(), keep.to(torch.uint8).cpu()
