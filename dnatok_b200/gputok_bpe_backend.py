"""Drop-in for the reference's BPE plug-in slot.

``DNATok.discover`` (reference ``src/dna_tokenizer.py:1098-1110``) does::

    from gputok_bpe_backend import GPUTokBPEBackend
    if GPUTokBPEBackend.is_supported(tok):
        self.bpe_backend = GPUTokBPEBackend(tok, engine="dnatok")

and its callers (``:2065-2087``, ``:3068-3100``) use ``bpe_backend.encode_batch(seqs, device=...)``
-> ``(input_ids int64 [B, T_max] right-padded with the HF pad id, attention_mask uint8 [B, T_max])``
plus the attributes ``vocab_size``, ``pad_id``, ``unk_id`` (reference
``src/gputok_bpe_backend.py:396-679``).  ``GPUTokBPEBackend`` below has the same members and the
same argument meaning and error behaviour (``ValueError`` on an empty batch, ``RuntimeError`` for a
tokenizer it cannot take), so it can be assigned to ``DNATok.bpe_backend`` unchanged.  Like the
reference it never adds special tokens.

``DnatokBpeKernel`` mirrors the native slot (``src/dnatok_bpe_kernel/__init__.py:81-136``):
``DnatokBpeKernel(merges_path, max_iters)``, ``vocab_size()``, ``id_to_token(i)`` and
``tokenize_batch(texts) -> (ids int32 [B, T_max], lengths int32 [B])`` on the GPU, in the
reference's internal id space when built from a merges file.  The tail of each row is zero-filled
as in the reference (``dnatok_bpe.cu:899``), and the returned tensors are freshly allocated rather
than views into a workspace, so ``clone`` is accepted and ignored.

There is no length-based routing to a CPU tokenizer (reference ``:551-564``): every row goes
through the GPU kernel, whatever its length.
"""
from __future__ import annotations

from typing import Any, List, Tuple

import numpy as np

from .tables import (UnsupportedTokenizer, bpe_spec_from_json, compile_normalizer, compile_normalizer_step,
                     extract_merges, read_tokenizer_json, supported_bpe)

# Names the reference module exposes to its tests.
_compile_normalizer_step = compile_normalizer_step
_compile_normalizer = compile_normalizer
_supported_tokenizer = supported_bpe
_read_tokenizer_json = read_tokenizer_json


def _extract_merges(cfg) -> List[str]:
    return ["%s %s" % ab for ab in extract_merges(cfg)]


class GPUTokBPEBackend:
    def __init__(self, hf_tokenizer: Any, *, engine: str = "dnatok") -> None:
        if engine not in ("gputok", "dnatok"):
            raise ValueError("engine must be 'gputok' or 'dnatok', got %r" % (engine,))
        from .tokenizer import B200Tokenizer
        self.tokenizer = hf_tokenizer
        self.engine = engine
        cfg = read_tokenizer_json(hf_tokenizer)
        ok, reason = supported_bpe(cfg)
        if not ok:
            raise RuntimeError("GPUTokBPEBackend cannot accelerate this tokenizer: %s" % reason)
        pad = getattr(hf_tokenizer, "pad_token_id", None)
        try:
            spec = bpe_spec_from_json(cfg, pad_id=int(pad) if pad is not None else None)
        except UnsupportedTokenizer as e:
            raise RuntimeError("GPUTokBPEBackend cannot accelerate this tokenizer: %s" % e) from None
        self._tok = B200Tokenizer(spec)
        self._tok.padding_side = "right"
        self._normalize = spec.normalizer
        self._merges = _extract_merges(cfg)
        self.vocab_size = int(getattr(hf_tokenizer, "vocab_size", 0) or spec.vocab_size)
        self.pad_id = int(pad or 0)
        self.unk_id = int(getattr(hf_tokenizer, "unk_token_id", 0) or 0)

    @staticmethod
    def is_supported(hf_tokenizer: Any) -> bool:
        try:
            cfg = read_tokenizer_json(hf_tokenizer)
            ok, _ = supported_bpe(cfg)
            if ok:
                bpe_spec_from_json(cfg)
            return ok
        except Exception:
            return False

    def encode_batch(self, seqs: List[str], *, device: object = "cuda") -> Tuple[Any, Any]:
        import torch
        if not seqs:
            raise ValueError("No sequences provided.")
        dev = torch.device(device) if not isinstance(device, torch.device) else device
        if dev.type != "cuda":
            raise RuntimeError("GPUTokBPEBackend runs on CUDA devices only")
        old = self._tok.device
        self._tok.device = dev if dev.index is not None else torch.device("cuda", torch.cuda.current_device())
        try:
            d_bytes, d_off, offsets = self._tok.to_device(list(seqs))
            enc = self._tok.encode_device(d_bytes, d_off, host_offsets=offsets, padding="longest",
                                          add_special_tokens=False, mask_dtype=torch.uint8)
        finally:
            self._tok.device = old
        return enc["input_ids"], enc["attention_mask"]

    def encode_batch_ids_only(self, seqs: List[str], *, device: object = "cuda"):
        ids, _ = self.encode_batch(seqs, device=device)
        return ids


def _spec_from_merges_file(merges_path: str):
    """Tables in the id space of the reference's native class: ids 0..255 are the byte symbols, then
    every token named in merges.txt gets the next id at its first appearance (left operand, right
    operand, result), line by line; a line's rank is its index among the merge lines
    (``build_vocab_from_merges``, reference ``src/dnatok_bpe_kernel/dnatok_bpe.cu:761-791``).  The
    first line is the ``#version`` header; blank lines and ``#`` lines are skipped."""
    from .tables import Specials, TokenizerSpec
    id_to_token: List[str] = [chr(b) for b in range(256)]
    token_to_id = {t: i for i, t in enumerate(id_to_token)}

    def add(t: str) -> int:
        i = token_to_id.get(t)
        if i is None:
            i = token_to_id[t] = len(id_to_token)
            id_to_token.append(t)
        return i

    a, b, o = [], [], []
    with open(merges_path, "r", encoding="utf-8") as f:
        lines = f.read().split("\n")
    if not lines or (len(lines) == 1 and not lines[0]):
        raise RuntimeError("Empty merges file")
    for line in lines[1:]:
        if not line or line[0] == "#":
            continue
        parts = line.split()
        if len(parts) < 2:
            continue
        x, y = parts[0], parts[1]
        a.append(add(x)); b.append(add(y)); o.append(add(x + y))
    if not a:
        raise RuntimeError("merges file holds no merges: %s" % merges_path)
    spec = TokenizerSpec("bpe", Specials(pad_id=0, unk_id=0), len(id_to_token), np.arange(256, dtype=np.int32),
                         merge_a=np.asarray(a, np.int32), merge_b=np.asarray(b, np.int32),
                         merge_out=np.asarray(o, np.int32), vocab=dict(token_to_id))
    return spec, id_to_token


class DnatokBpeKernel:
    """The native slot: ``DnatokBpeKernel(merges_path, max_iters=1024)`` as in the reference
    (``src/dnatok_bpe_kernel/__init__.py:81-136`` over the pybind class
    ``DNATokBPE(merges_path, byte_to_id_lut, max_iters)``, ``dnatok_bpe.cu:1042-1055``), with
    ``vocab_size()``, ``id_to_token(i)`` and ``tokenize_batch(texts, clone=False)``.  Built from a
    merges file the ids are the reference's internal ids (byte symbols, then tokens in file order),
    which its callers remap to Hugging Face ids; ``from_spec`` builds the same object directly in
    Hugging Face id space from a tokenizer spec."""

    def __init__(self, merges_path, max_iters: int = 1024):
        import copy
        from .tokenizer import B200Tokenizer
        if isinstance(merges_path, (str, bytes)) or hasattr(merges_path, "__fspath__"):
            import os
            path = os.fspath(merges_path)
            if not os.path.isfile(path):
                raise RuntimeError("Failed to open merges file: %s" % path)
            spec, self._id_to_token = _spec_from_merges_file(path)
        else:
            spec = copy.copy(merges_path)
            spec.specials = copy.copy(spec.specials)
            spec.specials.pad_id = 0                  # the reference zero-fills the tail of each row
            inv = {i: t for t, i in spec.vocab.items()}
            self._id_to_token = [inv.get(i, "") for i in range(spec.vocab_size)]
        self._tok = B200Tokenizer(spec)
        self._tok.padding_side = "right"
        self.max_iters = int(max_iters)   # accepted for signature parity; the pass bound is the word length

    @classmethod
    def from_spec(cls, spec, max_iters: int = 1024) -> "DnatokBpeKernel":
        return cls(spec, max_iters)

    @classmethod
    def from_merges_file(cls, merges_path: str, max_iters: int = 1024) -> "DnatokBpeKernel":
        return cls(merges_path, max_iters)

    def vocab_size(self) -> int:
        return len(self._id_to_token)

    def id_to_token(self, idx: int) -> str:
        idx = int(idx)
        if idx < 0 or idx >= len(self._id_to_token):
            raise IndexError("token id %d outside the vocabulary" % idx)
        return self._id_to_token[idx]

    def tokenize_batch(self, seqs: List[str], clone: bool = False):
        import torch
        if not seqs:
            raise ValueError("No sequences provided.")
        d_bytes, d_off, offsets = self._tok.to_device(list(seqs))
        enc = self._tok.encode_device(d_bytes, d_off, host_offsets=offsets, padding="longest",
                                      add_special_tokens=False, return_attention_mask=False,
                                      ids_dtype=torch.int32)
        return enc["input_ids"], enc["lengths"]
