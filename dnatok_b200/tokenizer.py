"""Hugging Face style front end over the CUDA kernels.

``B200Tokenizer`` keeps the call surface the reference's users reach through ``AutoTokenizer``
objects (``tok(seqs, padding=..., truncation=..., max_length=..., add_special_tokens=...,
return_tensors=..., return_attention_mask=...)`` -> ``input_ids`` / ``attention_mask``;
``encode``; ``batch_encode_plus``; ``pad_token_id``; ``padding_side``; ``vocab_size``;
``get_vocab``) - the calls the reference makes at ``src/dna_tokenizer.py:1708-1714`` and
``src/gputok_bpe_backend.py:653-656`` and that its ``dnatok_compat`` tokenizers
(``src/dnatok_compat.py:181-238``) implement in Python.

Everything numeric happens in ``libdnatok_b200.so``; PyTorch only allocates the tensors that
are handed across and provides the stream.  With ``return_tensors="pt"`` the tensors stay on
the GPU (Hugging Face returns CPU tensors; pass ``device="cpu"`` to copy back).
"""
from __future__ import annotations

import ctypes
from typing import Any, List, Optional, Sequence, Union

import numpy as np

from . import _cabi
from .pack import pack_any
from .tables import TokenizerSpec, spec_from_tokenizer


class BatchEncoding(dict):
    """dict with attribute access, like ``transformers.BatchEncoding``."""

    def __getattr__(self, k):
        try:
            return self[k]
        except KeyError:
            raise AttributeError(k) from None

    def to(self, device):
        import torch
        return BatchEncoding({k: (v.to(device) if isinstance(v, torch.Tensor) else v) for k, v in self.items()})


def _torch():
    import torch
    return torch


class B200Tokenizer:
    model_input_names = ["input_ids", "attention_mask"]

    def __init__(self, spec: TokenizerSpec, device: Union[int, str, None] = None):
        torch = _torch()
        self.spec = spec
        self.handle = _cabi.Handle(spec)
        if device is None:
            device = torch.cuda.current_device() if torch.cuda.is_available() else 0
        self.device = torch.device(device if not isinstance(device, int) else "cuda:%d" % device)
        self.padding_side = spec.specials.padding_side
        self.check_status = True
        self._pins = [None, None]   # two pinned host buffers the native packer fills in turn, so that packing one
        self._pin_done = [None, None]   # batch can overlap the copy of the batch before; events: the last copy out of each
        self._pin_turn = 0

    # ------------------------------------------------------------------ construction
    @classmethod
    def from_hf(cls, hf_tokenizer: Any, device=None) -> "B200Tokenizer":
        return cls(spec_from_tokenizer(hf_tokenizer), device=device)

    # ------------------------------------------------------------------ HF attributes
    @property
    def pad_token_id(self) -> int:
        return self.spec.specials.pad_id

    @property
    def unk_token_id(self) -> int:
        return self.spec.specials.unk_id

    @property
    def cls_token_id(self) -> Optional[int]:
        return self.spec.specials.cls_id if self.spec.specials.cls_id >= 0 else None

    @property
    def sep_token_id(self) -> Optional[int]:
        return self.spec.specials.sep_id if self.spec.specials.sep_id >= 0 else None

    @property
    def vocab_size(self) -> int:
        return self.spec.vocab_size

    def get_vocab(self) -> dict:
        return dict(self.spec.vocab)

    def __len__(self) -> int:
        return self.spec.vocab_size

    # ------------------------------------------------------------------ formats
    def _format(self, *, id_bits, mask_bits, add_special, max_tokens, out_stride, pad_left=None):
        left = (self.padding_side == "left") if pad_left is None else pad_left
        return _cabi.Format(id_bits, mask_bits, 1 if add_special else 0, 1 if left else 0,
                            int(max_tokens), int(out_stride))

    def _n_special(self, add_special: bool) -> int:
        sp = self.spec.specials
        return ((sp.cls_id >= 0) + (sp.sep_id >= 0)) if add_special else 0

    def _normalize(self, seqs):
        fn = self.spec.normalizer
        if fn is None or isinstance(seqs, (np.ndarray, tuple)):
            return seqs
        return [fn(s) for s in seqs]

    # ------------------------------------------------------------------ device-resident path
    def encode_device(self, d_bytes, d_offsets, *, host_offsets: Optional[np.ndarray] = None,
                      padding: Union[bool, str] = "longest", max_length: Optional[int] = None,
                      truncation: bool = False, add_special_tokens: bool = True,
                      return_attention_mask: bool = True, ids_dtype=None, mask_dtype=None,
                      out: Optional[dict] = None, scratch=None, check: Optional[bool] = None):
        """Encode rows already in GPU memory.

        ``d_bytes`` uint8[total] and ``d_offsets`` int64[B+1] are CUDA tensors.  Returns a dict with
        ``input_ids`` (and ``attention_mask``) for padded output, or ``input_ids`` (flat),
        ``offsets`` (int64[B+1]) for ``padding=False``.  ``lengths`` (int32[B]) is always included.
        ``out`` may carry preallocated ``input_ids`` / ``attention_mask`` tensors and ``scratch`` a
        uint8 scratch tensor, which makes the call allocation-free for fixed strides;
        ``scratch=False`` runs a k-mer tokenizer without scratch memory (one warp per row).
        """
        torch = _torch()
        L = _cabi.lib()
        dev = d_bytes.device
        if dev.type != "cuda":
            raise RuntimeError("encode_device needs CUDA tensors; there is no CPU path")
        ids_dtype = ids_dtype or torch.int64
        mask_dtype = mask_dtype or torch.int64
        id_bits = {torch.int64: 64, torch.int32: 32}[ids_dtype]
        mask_bits = {torch.int64: 64, torch.int32: 32, torch.uint8: 8}[mask_dtype] if return_attention_mask else 0
        B = d_offsets.shape[0] - 1
        total = int(d_bytes.shape[0])
        check = self.check_status if check is None else check
        max_tokens = int(max_length) if (truncation and max_length) else 0
        if truncation and not max_length:
            raise ValueError("truncation=True needs max_length")
        if padding is True:
            padding = "longest"
        if padding in (None, "do_not_pad"):
            padding = False
        if padding not in (False, "longest", "max_length"):
            raise ValueError("padding must be False, True/'longest' or 'max_length'")
        if padding == "max_length" and not max_length:
            raise ValueError("padding='max_length' needs max_length")
        ns = self._n_special(add_special_tokens)
        out = out or {}
        # row lengths known on the host bound the length classes the BPE path has to launch and the
        # number of segments the k-mer path cuts a row into (which only batches of few or very long
        # rows use: large batches of ordinary rows skip the scan of the offsets)
        wants_hint = self.spec.kind == "bpe" or (self.spec.kind == "kmer" and (B < 4096 or total > 32768 * B))
        if wants_hint and host_offsets is not None and B:
            lens = np.diff(host_offsets)
            _cabi.check(L.dnatok_set_row_bytes_hint(self.handle.ptr, int(lens.min()), max(int(lens.max()), 1)))
        elif self.spec.kind in ("bpe", "kmer"):
            _cabi.check(L.dnatok_set_row_bytes_hint(self.handle.ptr, 0, 0))
        with torch.cuda.device(dev):
            stream = ctypes.c_void_p(torch.cuda.current_stream(dev).cuda_stream)
            need = L.dnatok_scratch_bytes(self.handle.ptr, B, total)
            if scratch is False:
                if self.spec.kind == "bpe":
                    raise ValueError("the BPE path needs a scratch buffer")
                need = 0                       # k-mer without scratch: one warp (or block) per row
            if need and (scratch is None or scratch.numel() < need):
                scratch = torch.empty(need, dtype=torch.uint8, device=dev)
            sc_ptr = ctypes.c_void_p(scratch.data_ptr()) if need else None
            sc_len = int(scratch.numel()) if need else 0
            lengths = torch.empty(max(B, 1), dtype=torch.int32, device=dev)
            status = torch.empty(max(B, 1), dtype=torch.int32, device=dev)
            args = (self.handle.ptr, ctypes.c_void_p(d_bytes.data_ptr()), ctypes.c_void_p(d_offsets.data_ptr()), B, total)
            res = BatchEncoding()

            if padding is False:
                fmt = self._format(id_bits=id_bits, mask_bits=0, add_special=add_special_tokens,
                                   max_tokens=max_tokens, out_stride=0)
                bound = L.dnatok_max_tokens(self.handle.ptr, B, total, ctypes.byref(fmt))
                ids = torch.empty(max(bound, 1), dtype=ids_dtype, device=dev)
                out_off = torch.empty(B + 1, dtype=torch.int64, device=dev)
                _cabi.check(L.dnatok_encode(*args, ctypes.byref(fmt), ctypes.c_void_p(ids.data_ptr()), None,
                                            ctypes.c_void_p(lengths.data_ptr()), ctypes.c_void_p(out_off.data_ptr()),
                                            ctypes.c_void_p(status.data_ptr()), sc_ptr, sc_len, stream))
                n_out = int(out_off[-1].item())
                res["input_ids"] = ids[:n_out]
                res["offsets"] = out_off
            else:
                prepared = False
                if padding == "max_length":
                    stride = int(max_length)
                elif self.spec.kind == "char" and host_offsets is not None:
                    lens = np.diff(host_offsets)
                    if max_tokens:
                        lens = np.minimum(lens, max_tokens - ns)
                    stride = int(lens.max()) + ns if B else 0
                else:
                    fmt0 = self._format(id_bits=id_bits, mask_bits=0, add_special=add_special_tokens,
                                        max_tokens=max_tokens, out_stride=0)
                    _cabi.check(L.dnatok_prepare(*args, ctypes.byref(fmt0), ctypes.c_void_p(lengths.data_ptr()),
                                                 ctypes.c_void_p(status.data_ptr()), sc_ptr, sc_len, stream))
                    stride = int(lengths[:B].max().item()) if B else 0
                    prepared = True
                fmt = self._format(id_bits=id_bits, mask_bits=mask_bits, add_special=add_special_tokens,
                                   max_tokens=max_tokens, out_stride=stride)
                ids = out.get("input_ids")
                if ids is None or tuple(ids.shape) != (B, stride) or ids.dtype != ids_dtype:
                    ids = torch.empty((B, stride), dtype=ids_dtype, device=dev)
                mask = None
                if mask_bits:
                    mask = out.get("attention_mask")
                    if mask is None or tuple(mask.shape) != (B, stride) or mask.dtype != mask_dtype:
                        mask = torch.empty((B, stride), dtype=mask_dtype, device=dev)
                if B and stride:
                    ids_p = ctypes.c_void_p(ids.data_ptr())
                    mask_p = ctypes.c_void_p(mask.data_ptr()) if mask is not None else None
                    if prepared:
                        _cabi.check(L.dnatok_write(*args, ctypes.byref(fmt), ctypes.c_void_p(lengths.data_ptr()), None,
                                                   ids_p, mask_p, ctypes.c_void_p(status.data_ptr()), sc_ptr, sc_len, stream))
                    else:
                        _cabi.check(L.dnatok_encode(*args, ctypes.byref(fmt), ids_p, mask_p,
                                                    ctypes.c_void_p(lengths.data_ptr()), None,
                                                    ctypes.c_void_p(status.data_ptr()), sc_ptr, sc_len, stream))
                res["input_ids"] = ids
                if mask is not None:
                    res["attention_mask"] = mask
            res["lengths"] = lengths[:B]
            if check and B:
                self._raise_on_status(status[:B], truncation)
        return res

    def embed_device(self, d_bytes, d_offsets, weight, *, host_offsets: Optional[np.ndarray] = None,
                     padding: Union[bool, str] = "longest", max_length: Optional[int] = None,
                     truncation: bool = False, add_special_tokens: bool = True, out=None):
        """Fused tokenise -> embedding lookup for char / byte-level tokenizers: returns
        ``weight[input_ids]`` as a ``[B, T, D]`` CUDA tensor (and ``lengths``) without materialising the
        ids.  ``weight`` is a contiguous ``[vocab, D]`` CUDA tensor whose rows are a multiple of 16 bytes."""
        torch = _torch()
        L = _cabi.lib()
        if self.spec.kind != "char":
            raise RuntimeError("embed_device needs a one-token-per-character tokenizer")
        B = d_offsets.shape[0] - 1
        ns = self._n_special(add_special_tokens)
        max_tokens = int(max_length) if (truncation and max_length) else 0
        if padding in (True, "longest"):
            if host_offsets is None:
                host_offsets = d_offsets.cpu().numpy()
            lens = np.diff(host_offsets)
            if max_tokens:
                lens = np.minimum(lens, max_tokens - ns)
            stride = int(lens.max()) + ns if B else 0
        elif padding == "max_length" and max_length:
            stride = int(max_length)
        else:
            raise ValueError("embed_device needs padding='longest' or 'max_length'")
        if not weight.is_contiguous() or weight.dim() != 2:
            raise ValueError("weight must be a contiguous [vocab, D] tensor")
        row_bytes = weight.shape[1] * weight.element_size()
        dev = d_bytes.device
        if out is None or tuple(out.shape) != (B, stride, weight.shape[1]) or out.dtype != weight.dtype:
            out = torch.empty((B, stride, weight.shape[1]), dtype=weight.dtype, device=dev)
        lengths = torch.empty(max(B, 1), dtype=torch.int32, device=dev)
        status = torch.empty(max(B, 1), dtype=torch.int32, device=dev)
        fmt = self._format(id_bits=64, mask_bits=0, add_special=add_special_tokens, max_tokens=max_tokens,
                           out_stride=stride)
        if B and stride:
            with torch.cuda.device(dev):
                stream = ctypes.c_void_p(torch.cuda.current_stream(dev).cuda_stream)
                _cabi.check(L.dnatok_embed(self.handle.ptr, ctypes.c_void_p(d_bytes.data_ptr()),
                                           ctypes.c_void_p(d_offsets.data_ptr()), B, int(d_bytes.shape[0]),
                                           ctypes.byref(fmt), ctypes.c_void_p(weight.data_ptr()), int(weight.shape[0]),
                                           int(row_bytes), ctypes.c_void_p(out.data_ptr()),
                                           ctypes.c_void_p(lengths.data_ptr()), ctypes.c_void_p(status.data_ptr()), stream))
        return BatchEncoding(embeddings=out, lengths=lengths[:B])

    def _raise_on_status(self, status, truncation: bool) -> None:
        bits = int(status.max().item()) if status.numel() else 0
        if not bits:
            return
        st = status.cpu().numpy()
        if np.any(st & _cabi.ROW_TOO_LONG):
            raise RuntimeError("%d row(s) exceed the BPE kernel's word limit of %d bytes (first: row %d)"
                               % (int(np.count_nonzero(st & _cabi.ROW_TOO_LONG)), _cabi.BPE_MAX_WORD,
                                  int(np.flatnonzero(st & _cabi.ROW_TOO_LONG)[0])))
        if np.any(st & _cabi.ROW_OUTSIDE_HINT):
            raise RuntimeError("row %d is outside the row-length bounds given to dnatok_set_row_bytes_hint"
                               % int(np.flatnonzero(st & _cabi.ROW_OUTSIDE_HINT)[0]))
        if np.any(st & _cabi.ROW_NOT_CONVERGED):
            raise RuntimeError("BPE merge loop hit its pass limit on row %d" %
                               int(np.flatnonzero(st & _cabi.ROW_NOT_CONVERGED)[0]))
        if np.any(st & _cabi.ROW_STALLED):
            raise RuntimeError("k-mer row %d: a row segment gave up waiting for the one before it"
                               % int(np.flatnonzero(st & _cabi.ROW_STALLED)[0]))
        if np.any(st & _cabi.ROW_CLIPPED):
            raise ValueError("row %d has more tokens than max_length and truncation is off "
                             "(Hugging Face cannot build a tensor from such a batch either)"
                             % int(np.flatnonzero(st & _cabi.ROW_CLIPPED)[0]))

    def to_device(self, seqs, *, table: Optional[bytes] = None, pad_to: int = 0, pad_byte: int = ord("N"),
                  pad_left: bool = False, trunc_to: int = 0):
        """Pack rows on the host (after the tokenizer's normalizer) and copy them to the GPU:
        returns (uint8[total] CUDA tensor, int64[B+1] CUDA tensor, host offsets).  Lists of str / bytes go
        through the native packer straight into a pinned buffer that the tokenizer keeps and reuses; ``table``
        (256 bytes) translates every byte on the way and ``pad_to`` pads short rows, both inside that one copy."""
        torch = _torch()
        dev = self.device
        seqs = self._normalize(seqs)
        if isinstance(seqs, (list, tuple)):
            from .pack import pack_sizes, pack_strings
            if len(seqs) == 0:
                return (torch.empty(0, dtype=torch.uint8, device=dev), torch.zeros(1, dtype=torch.int64, device=dev),
                        np.zeros(1, dtype=np.int64))
            need = pack_sizes(seqs, pad_to, trunc_to)
            k = self._pin_turn
            self._pin_turn ^= 1
            if self._pin_done[k] is not None:
                self._pin_done[k].synchronize()          # the copy out of this buffer two calls ago
            if self._pins[k] is None or self._pins[k].numel() < need:
                self._pins[k] = torch.empty(max(need + need // 4, 1 << 16), dtype=torch.uint8).pin_memory()
            pin = self._pins[k]
            flat, offsets = pack_strings(seqs, table=table, pad_to=pad_to, pad_byte=pad_byte, pad_left=pad_left,
                                         trunc_to=trunc_to, out=pin.numpy())
            with torch.cuda.device(dev):
                d_off = torch.from_numpy(offsets).to(dev)        # small, and before the large copy so it does not wait for it
                d_bytes = torch.empty(flat.size, dtype=torch.uint8, device=dev)
                d_bytes.copy_(pin[:flat.size], non_blocking=True)
                if self._pin_done[k] is None:
                    self._pin_done[k] = torch.cuda.Event()
                self._pin_done[k].record()
            return d_bytes, d_off, offsets
        if pad_to or trunc_to:
            raise ValueError("pad_to / trunc_to need a list of rows")
        flat, offsets = pack_any(seqs)
        if table is not None:
            flat = np.frombuffer(table, dtype=np.uint8)[flat]
        d_bytes = torch.from_numpy(flat).to(dev) if flat.size else torch.empty(0, dtype=torch.uint8, device=dev)
        return d_bytes, torch.from_numpy(offsets).to(dev), offsets

    # ------------------------------------------------------------------ HF call surface
    def __call__(self, text, padding: Union[bool, str] = False, truncation: bool = False,
                 max_length: Optional[int] = None, add_special_tokens: bool = True,
                 return_tensors: Optional[str] = None, return_attention_mask: bool = True,
                 device=None, **unused):
        torch = _torch()
        single = isinstance(text, (str, bytes))
        seqs = [text] if single else text
        dev = self.device
        d_bytes, d_off, offsets = self.to_device(seqs)
        want_pad = padding not in (False, None, "do_not_pad")
        if return_tensors in ("pt", "np") and not want_pad and not single:
            lens = np.diff(offsets)
            if lens.size and lens.min() != lens.max() and self.spec.kind == "char":
                raise ValueError("Unable to create tensor: rows have different lengths; use padding=True")
        enc = self.encode_device(d_bytes, d_off, host_offsets=offsets, padding=padding if want_pad else False,
                                 max_length=max_length, truncation=truncation,
                                 add_special_tokens=add_special_tokens,
                                 return_attention_mask=return_attention_mask)
        B = len(offsets) - 1
        if want_pad:
            ids, mask = enc["input_ids"], enc.get("attention_mask")
            if return_tensors == "pt":
                res = BatchEncoding(input_ids=ids)
                if mask is not None:
                    res["attention_mask"] = mask
                return res.to(device) if device is not None else res
            ids_h = ids.cpu().numpy()
            mask_h = mask.cpu().numpy() if mask is not None else None
            if return_tensors == "np":
                res = BatchEncoding(input_ids=ids_h)
                if mask_h is not None:
                    res["attention_mask"] = mask_h
                return res
            res = BatchEncoding(input_ids=ids_h.tolist() if not single else ids_h[0].tolist())
            if mask_h is not None:
                res["attention_mask"] = mask_h.tolist() if not single else mask_h[0].tolist()
            return res
        # no padding: ragged rows
        flat_ids = enc["input_ids"].cpu().numpy()
        oo = enc["offsets"].cpu().numpy()
        rows = [flat_ids[oo[i]:oo[i + 1]] for i in range(B)]
        if return_tensors in ("pt", "np"):
            if B and any(len(r) != len(rows[0]) for r in rows):
                raise ValueError("Unable to create tensor: rows have different lengths; use padding=True")
            arr = np.stack(rows) if B else np.zeros((0, 0), dtype=np.int64)
            res = BatchEncoding(input_ids=arr)
            if return_attention_mask:
                res["attention_mask"] = np.ones_like(arr)
            if return_tensors == "pt":
                res = BatchEncoding({k: torch.from_numpy(v).to(device or dev) for k, v in res.items()})
            return res
        res = BatchEncoding(input_ids=[r.tolist() for r in rows] if not single else rows[0].tolist())
        if return_attention_mask:
            res["attention_mask"] = [[1] * len(r) for r in rows] if not single else [1] * len(rows[0])
        return res

    def batch_encode_plus(self, batch_text, **kw):
        return self(list(batch_text), **kw)

    batch_encode = batch_encode_plus

    def encode_plus(self, text: str, **kw):
        return self(text, **kw)

    def encode(self, text: str, add_special_tokens: bool = True, **kw) -> List[int]:
        return self(text, add_special_tokens=add_special_tokens, return_attention_mask=False, **kw)["input_ids"]

    # ------------------------------------------------------------------ host-buffer path
    def encode_host(self, seqs, *, padding: Union[bool, str] = "longest", max_length: Optional[int] = None,
                    truncation: bool = False, add_special_tokens: bool = True, return_attention_mask: bool = True,
                    ids_dtype=np.int64, mask_dtype=np.int64, out_ids: Optional[np.ndarray] = None,
                    out_mask: Optional[np.ndarray] = None):
        """Host arrays in, host arrays out, through ``dnatok_encode_host`` (copies + kernels inside
        the library).  Pass pinned ``out_ids`` / ``out_mask`` buffers for asynchronous copies."""
        L = _cabi.lib()
        flat, offsets = pack_any(self._normalize(seqs))
        B = len(offsets) - 1
        ns = self._n_special(add_special_tokens)
        max_tokens = int(max_length) if (truncation and max_length) else 0
        if padding is True:
            padding = "longest"
        ragged = padding in (False, None, "do_not_pad")
        stride = 0 if ragged else (int(max_length) if padding == "max_length" else -1)
        id_bits = np.dtype(ids_dtype).itemsize * 8
        mask_bits = np.dtype(mask_dtype).itemsize * 8 if (return_attention_mask and not ragged) else 0
        fmt = self._format(id_bits=id_bits, mask_bits=mask_bits, add_special=add_special_tokens,
                           max_tokens=max_tokens, out_stride=stride)
        if stride > 0:
            cap = B * stride
        elif ragged:
            cap = int(offsets[-1]) + ns * B
        else:                                     # padded to the longest row: no row has more tokens than bytes
            longest = int(np.diff(offsets).max()) if B else 0
            if max_tokens:
                longest = min(longest, max_tokens - ns)
            cap = B * (longest + ns)
        if out_ids is None or out_ids.size < cap:
            out_ids = np.empty(max(cap, 1), dtype=ids_dtype)
        if mask_bits and (out_mask is None or out_mask.size < cap):
            out_mask = np.empty(max(cap, 1), dtype=mask_dtype)
        lengths = np.empty(max(B, 1), dtype=np.int32)
        status = np.zeros(max(B, 1), dtype=np.int32)
        out_off = np.zeros(B + 1, dtype=np.int64)
        used = ctypes.c_int64(0)
        dev_index = self.device.index if self.device.index is not None else 0
        _cabi.check(L.dnatok_encode_host(
            self.handle.ptr, dev_index, _cabi.np_ptr(flat) if flat.size else None, _cabi.np_ptr(offsets), B,
            ctypes.byref(fmt), _cabi.np_ptr(out_ids), int(out_ids.size),
            _cabi.np_ptr(out_mask) if mask_bits else None, _cabi.np_ptr(lengths), _cabi.np_ptr(out_off),
            _cabi.np_ptr(status), ctypes.byref(used)))
        st = status[:B]
        if self.check_status and st.any():
            import torch
            self._raise_on_status(torch.from_numpy(st.copy()), truncation)
        res = BatchEncoding(lengths=lengths[:B])
        if ragged:
            res["input_ids"] = out_ids.reshape(-1)[:used.value]
            res["offsets"] = out_off
        else:
            w = used.value
            res["input_ids"] = out_ids.reshape(-1)[:B * w].reshape(B, w)
            if mask_bits:
                res["attention_mask"] = out_mask.reshape(-1)[:B * w].reshape(B, w)
        return res
