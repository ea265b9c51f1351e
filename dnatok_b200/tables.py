"""Turn a Hugging Face tokenizer into the flat integer tables the CUDA kernels read.

This is the counterpart of the reference's one-time discovery step: ``DNATok.discover``
(reference ``src/dna_tokenizer.py:864-1110``) probes the wrapped tokenizer and builds an ASCII
LUT (``:633-653``), a k-mer LUT (``_discover_kmer_structure`` ``:655-741``, ``_build_kmer_lut``
``:743-822``) or hands the tokenizer to ``GPUTokBPEBackend`` (``src/gputok_bpe_backend.py:412-474``),
which reads ``tokenizer.json`` (``:132-176``), checks the model / pre-tokenizer / normalizer
(``:265-295``) and extracts the merges in rank order (``:251-262``).

Differences by design: BPE tables are built directly in HF id space (the reference keeps a
kernel-id -> HF-id remap, ``:447-466``), and a k-mer vocabulary is stored as a ``4**k`` table of
clean windows plus a single-character table when probing shows that the tokenizer expands every
other window character by character (the form the fast kernels read); any other k-mer tokenizer is
kept as the reference keeps it, as the table of all ``5**k`` windows over ACGTN with runs of ids for
windows that are not one token.  A per-character tokenizer may give a character one id at the start
of a sequence and another later on (start / continuation tables).

Nothing here computes token ids for user input; tables only.
"""
from __future__ import annotations

import itertools
import json
import re as _re
from dataclasses import dataclass, field
from typing import Any, Callable, Dict, List, Optional, Tuple

import numpy as np


class UnsupportedTokenizer(RuntimeError):
    """The tokenizer cannot be expressed as char / k-mer / BPE tables; there is no CPU fallback."""


@dataclass
class Specials:
    pad_id: int = 0
    unk_id: int = 0
    cls_id: int = -1          # id emitted before the sequence when add_special_tokens, -1: none
    sep_id: int = -1          # id emitted after the sequence, -1: none
    padding_side: str = "right"


@dataclass
class TokenizerSpec:
    kind: str                                   # "char" | "kmer" | "bpe"
    specials: Specials
    vocab_size: int
    lut256: np.ndarray                          # int32[256]: byte -> id (char), single ids (kmer), initial symbols (bpe)
    k: int = 0
    kmer_ids: Optional[np.ndarray] = None       # int32[4**k], itertools.product("ACGT", k) order
    # k-mer tokenizers given window by window (any tokenizer the 4**k + singles form cannot express):
    kmer_table5: Optional[np.ndarray] = None    # int32[5**k] over ACGTN: id, or -(e + 1) for run e
    kmer_run_offsets: Optional[np.ndarray] = None   # int32[n_runs + 1]
    kmer_run_ids: Optional[np.ndarray] = None
    kmer_tail_singles: bool = True              # the len % k tail gives one id per character (False: nothing)
    start_lut256: Optional[np.ndarray] = None   # char: ids of a row's first character when they differ from lut256
    merge_a: Optional[np.ndarray] = None        # int32[n_merges] left operand id, rank order
    merge_b: Optional[np.ndarray] = None
    merge_out: Optional[np.ndarray] = None
    normalizer: Optional[Callable[[str], str]] = None
    vocab: Dict[str, int] = field(default_factory=dict)


# --------------------------------------------------------------------------- normalizer
# Same accepted steps and same semantics as the reference's compiler
# (src/gputok_bpe_backend.py:179-248); its known answers are in
# tests/test_gputok_bpe_backend.py:319-425 of the reference.

def compile_normalizer_step(step: Any) -> Optional[Callable[[str], str]]:
    if not isinstance(step, dict):
        return None
    t = step.get("type")
    if t == "Strip":
        left, right = bool(step.get("strip_left", True)), bool(step.get("strip_right", True))
        if left and right:
            return str.strip
        if left:
            return str.lstrip
        if right:
            return str.rstrip
        return lambda s: s
    if t == "Replace":
        pat, content = step.get("pattern"), str(step.get("content", ""))
        if isinstance(pat, dict) and "String" in pat:
            lit = pat["String"]
            return lambda s: s.replace(lit, content)
        if isinstance(pat, dict) and "Regex" in pat:
            rx = _re.compile(pat["Regex"])
            return lambda s: rx.sub(content, s)
        return None
    if t == "Prepend":
        pre = str(step.get("prepend", ""))
        return lambda s: pre + s
    if t in (None, "NFC", "NFKC", "NFD", "NFKD", "StripAccents"):
        return lambda s: s                      # identity on ASCII DNA
    if t == "Lowercase":
        return str.lower
    if t == "Sequence":
        fns = [compile_normalizer_step(x) for x in step.get("normalizers", [])]
        if any(f is None for f in fns):
            return None

        def run(s: str) -> str:
            for f in fns:
                s = f(s)
            return s
        return run
    return None


def compile_normalizer(cfg: Dict[str, Any]) -> Optional[Callable[[str], str]]:
    norm = cfg.get("normalizer")
    if norm is None:
        return None
    fn = compile_normalizer_step(norm)
    if fn is None:
        raise ValueError("Unsupported normalizer config: %r" % (norm.get("type"),))
    return fn


# --------------------------------------------------------------------------- tokenizer.json

def read_tokenizer_json(tok: Any) -> Optional[Dict[str, Any]]:
    """tokenizer.json of a fast tokenizer: from its backend object, else from a local path."""
    import os
    backend = getattr(tok, "backend_tokenizer", None) or (tok if hasattr(tok, "to_str") else None)
    to_str = getattr(backend, "to_str", None)
    if callable(to_str):
        try:
            return json.loads(to_str())
        except Exception:
            pass
    for attr in ("name_or_path", "vocab_file"):
        v = getattr(tok, attr, None)
        if isinstance(v, str) and v:
            for cand in (os.path.join(v, "tokenizer.json"), v):
                if os.path.isfile(cand) and cand.endswith("tokenizer.json"):
                    with open(cand) as f:
                        return json.load(f)
    return None


def supported_bpe(cfg: Optional[Dict[str, Any]]) -> Tuple[bool, str]:
    """Acceptance rule of the reference (src/gputok_bpe_backend.py:265-295) plus the model
    options this engine does not implement."""
    if cfg is None:
        return False, "tokenizer.json not found"
    model = cfg.get("model") or {}
    if model.get("type") != "BPE":
        return False, "model.type=%r (only BPE supported)" % (model.get("type"),)
    pre = cfg.get("pre_tokenizer")
    if pre is not None:
        pt = pre.get("type") if isinstance(pre, dict) else None
        if pt not in (None, "Whitespace", "Split", "WhitespaceSplit"):
            return False, "pre_tokenizer=%r" % (pt,)
    norm = cfg.get("normalizer")
    if norm is not None and compile_normalizer_step(norm) is None:
        return False, "unsupported normalizer=%r" % (norm.get("type"),)
    for opt in ("dropout", "continuing_subword_prefix", "end_of_word_suffix"):
        if model.get(opt):
            return False, "model.%s is set" % opt
    for opt in ("fuse_unk", "byte_fallback", "ignore_merges"):
        if model.get(opt):
            return False, "model.%s is set" % opt
    return True, "ok"


def extract_merges(cfg: Dict[str, Any]) -> List[Tuple[str, str]]:
    out = []
    for m in cfg.get("model", {}).get("merges", []):
        if isinstance(m, str):
            a, b = m.split(" ")
        elif isinstance(m, (list, tuple)) and len(m) == 2:
            a, b = m
        else:
            raise ValueError("Unrecognised merge entry: %r" % (m,))
        out.append((a, b))
    return out


def _template_specials(cfg: Dict[str, Any]) -> Tuple[int, int]:
    """(cls_id, sep_id) of a ``TemplateProcessing`` of the form ``[X] $A [Y]`` (either may be absent)."""
    post = cfg.get("post_processor")
    if post is None:
        return -1, -1
    if post.get("type") != "TemplateProcessing":
        raise UnsupportedTokenizer("post_processor=%r" % (post.get("type"),))
    ids = {k: v["ids"] for k, v in post.get("special_tokens", {}).items()}
    before, after, seen = [], [], False
    for piece in post.get("single", []):
        if "Sequence" in piece:
            seen = True
        else:
            name = piece["SpecialToken"]["id"]
            (after if seen else before).extend(ids[name])
    if len(before) > 1 or len(after) > 1:
        raise UnsupportedTokenizer("more than one special token on a side")
    return (before[0] if before else -1), (after[0] if after else -1)


def bpe_spec_from_json(cfg: Dict[str, Any], *, pad_id: Optional[int] = None,
                       padding_side: str = "right") -> TokenizerSpec:
    ok, why = supported_bpe(cfg)
    if not ok:
        raise UnsupportedTokenizer("cannot accelerate this tokenizer: " + why)
    model = cfg["model"]
    vocab: Dict[str, int] = model["vocab"]
    merges = extract_merges(cfg)
    if not merges:
        raise UnsupportedTokenizer("tokenizer has no merges")
    unk = model.get("unk_token")
    unk_id = vocab.get(unk, -1) if unk is not None else -1
    if unk_id < 0:
        raise UnsupportedTokenizer("BPE model without an unk token: characters outside the "
                                   "alphabet would be dropped, which this engine does not do")
    n = len(merges)
    a = np.empty(n, np.int32)
    b = np.empty(n, np.int32)
    o = np.empty(n, np.int32)
    for r, (x, y) in enumerate(merges):
        try:
            a[r], b[r], o[r] = vocab[x], vocab[y], vocab[x + y]
        except KeyError as e:
            raise UnsupportedTokenizer("merge %d names a token missing from the vocab: %s" % (r, e))
    lut = np.full(256, unk_id, np.int32)
    for tok_str, i in vocab.items():
        if len(tok_str) == 1 and ord(tok_str) < 128:
            lut[ord(tok_str)] = i
    for added in cfg.get("added_tokens", []):
        c = added.get("content", "")
        if len(c) == 1 and ord(c) < 128:
            raise UnsupportedTokenizer("single-character added token %r" % c)
    cls_id, sep_id = _template_specials(cfg)
    if pad_id is None:
        pad_id = vocab.get("[PAD]", vocab.get("<pad>", 0))
    vs = max(max(vocab.values()) + 1, max((t["id"] for t in cfg.get("added_tokens", [])), default=-1) + 1)
    return TokenizerSpec("bpe", Specials(pad_id, unk_id, cls_id, sep_id, padding_side), vs, lut,
                         merge_a=a, merge_b=b, merge_out=o, normalizer=compile_normalizer(cfg),
                         vocab=dict(vocab))


# --------------------------------------------------------------------------- probing (char / k-mer)

def _flat_ids(x) -> List[int]:
    if hasattr(x, "tolist"):
        x = x.tolist()
    while isinstance(x, list) and len(x) == 1 and isinstance(x[0], list):
        x = x[0]
    return [int(v) for v in x]


def _ids(tok: Any, texts: List[str]) -> List[List[int]]:
    """ids of each text without special tokens; tokenizers that cannot take a ragged batch (the
    reference's dict-based ``CharTokenizer``, ``src/dnatok_compat.py:220-238``) are asked one text at a time."""
    try:
        enc = tok(texts, add_special_tokens=False)
        rows = [_flat_ids(r) for r in enc["input_ids"]]
        if len(rows) == len(texts):
            return rows
    except Exception:
        pass
    return [_flat_ids(tok(t, add_special_tokens=False)["input_ids"]) for t in texts]


def _probe_specials(tok: Any) -> Tuple[int, int]:
    plain = _ids(tok, ["A"])[0]
    full = _flat_ids(tok(["A"], add_special_tokens=True)["input_ids"][0])
    if full == plain:
        return -1, -1
    n = len(plain)
    for lead in range(len(full) - n + 1):
        if full[lead:lead + n] == plain:
            before, after = full[:lead], full[lead + n:]
            if len(before) <= 1 and len(after) <= 1:
                return (before[0] if before else -1), (after[0] if after else -1)
    raise UnsupportedTokenizer("special-token layout is not [X] seq [Y]")


def _printable_ascii() -> List[int]:
    return [c for c in range(33, 127)]


def detect_kmer(tok: Any) -> int:
    """k of a non-overlapping k-mer tokenizer, 0 if it is not one (rule of the reference:
    ``"A"*24`` must give 24/k tokens for k in 2..8, likewise C, G, T and a mixed string)."""
    try:
        n = len(_ids(tok, ["A" * 24])[0])
    except Exception:
        return 0
    if n == 0 or 24 % n or not 2 <= 24 // n <= 8:
        return 0
    k = 24 // n
    probes = ["C" * 24, "G" * 24, "T" * 24, ("ACGT" * 6)]
    return k if all(len(r) == n for r in _ids(tok, probes)) else 0


def spec_from_probing(tok: Any) -> TokenizerSpec:
    """Char or k-mer tables by asking the tokenizer, as the reference's discovery does."""
    pad_id = int(getattr(tok, "pad_token_id", 0) or 0)
    unk_id = getattr(tok, "unk_token_id", None)
    unk_id = int(unk_id) if unk_id is not None else 0
    side = getattr(tok, "padding_side", "right")
    cls_id, sep_id = _probe_specials(tok)
    try:
        vocab = dict(tok.get_vocab())
    except Exception:
        vocab = {}
    vs = max(int(getattr(tok, "vocab_size", 0) or 0), (max(vocab.values()) + 1) if vocab else 0)
    sp = Specials(pad_id, unk_id, cls_id, sep_id, side)

    singles = np.full(256, unk_id, np.int32)
    chars = [c for c in range(1, 128) if not chr(c).isspace()]
    got = _ids(tok, [chr(c) for c in chars])
    for c, r in zip(chars, got):
        if len(r) != 1:
            continue          # no single id (k-mer tokenizers that drop short input): the probes below decide
        singles[c] = r[0]
    # bytes >= 128 and whitespace are outside the supported input domain; they read as unk.

    try:
        k = detect_kmer(tok)
    except Exception:
        k = 0
    if k == 0:
        # One token per character.  Where a character's id at the start of a sequence differs from its id
        # later on (word-piece style vocabularies), the later id is read off the second token of the doubled
        # character, as the reference does (_resolve_cont_ids, src/dna_tokenizer.py:527-558), and the single-
        # character ids become the table of column 0.
        cont = singles.copy()
        doubled = _ids(tok, [chr(c) * 2 for c in chars])
        for c, r in zip(chars, doubled):
            if len(r) == 2 and r[0] == singles[c]:
                cont[c] = r[1]
        start = singles if np.any(cont != singles) else None
        probes = ["ACGTACGT", "NNACGTNN", "acgtnACG", "TTTTTTTT", "AN", "NA", "Xx"]
        for p, r in zip(probes, _ids(tok, probes)):
            want = [int(singles[ord(p[0])])] + [int(cont[ord(ch)]) for ch in p[1:]]
            if r != want:
                raise UnsupportedTokenizer("not a per-character tokenizer with at most a start / continuation split "
                                           "(probe %r)" % p)
        return TokenizerSpec("char", sp, vs, cont, vocab=vocab, start_lut256=start)

    clean = ["".join(t) for t in itertools.product("ACGT", repeat=k)]
    kmer_ids = np.empty(4 ** k, np.int32)
    for lo in range(0, len(clean), 4096):
        for j, r in enumerate(_ids(tok, clean[lo:lo + 4096])):
            if len(r) != 1:
                raise UnsupportedTokenizer("k-mer %r gives %d tokens" % (clean[lo + j], len(r)))
            kmer_ids[lo + j] = r[0]
    # Every window holding a non-ACGT character must expand character by character, and the
    # frame must stay aligned after it; check all 5**k windows over ACGTN (as the reference
    # tabulates them) followed by a clean window, plus tails and lower case.
    dirty = ["".join(t) for t in itertools.product("ACGTN", repeat=k) if "N" in t]
    tail = "ACGTAC"[:k - 1] if k > 1 else ""
    probes = [d + clean[(7 * i) % len(clean)] + tail for i, d in enumerate(dirty)]
    probes += [clean[5] + "acgtn"[:k - 1], "a" + clean[9][1:] + clean[3], clean[1][:k - 1], "N" * (2 * k + 1)]
    fast_form = True
    for lo in range(0, len(probes), 4096):
        chunk = probes[lo:lo + 4096]
        for p, r in zip(chunk, _ids(tok, chunk)):
            if r != expected_kmer_ids(p, k, kmer_ids, singles):
                fast_form = False
                break
        if not fast_form:
            break
    if fast_form:
        return TokenizerSpec("kmer", sp, vs, singles, k=k, kmer_ids=kmer_ids, vocab=vocab)
    return _kmer_table_spec(tok, k, sp, vs, singles, vocab)


def _kmer_table_spec(tok: Any, k: int, sp: Specials, vs: int, singles: np.ndarray, vocab: dict) -> TokenizerSpec:
    """The complete window table: every one of the 5**k strings over ACGTN is tokenised once and kept as an id
    or a run of ids (the reference's _build_kmer_lut, src/dna_tokenizer.py:743-822), the tail rule is read off
    two probes, and the table is accepted only if replaying it reproduces the tokenizer on random ACGTN strings
    (the reference's _sanity_compare_kmer_expansion, :1220-1273)."""
    windows = ["".join(t) for t in itertools.product("ACGTN", repeat=k)]
    table5 = np.empty(5 ** k, np.int32)
    offsets, flat = [0], []
    for lo in range(0, len(windows), 4096):
        for j, r in enumerate(_ids(tok, windows[lo:lo + 4096])):
            if len(r) == 1:
                table5[lo + j] = r[0]
            else:
                table5[lo + j] = -len(offsets)
                flat.extend(r)
                offsets.append(len(flat))
    one = windows[7 % len(windows)]
    whole = _ids(tok, [one])[0]
    with_tail = _ids(tok, [one + "C"])[0] if k > 1 else whole
    if k == 1 or with_tail == whole + [int(singles[ord("C")])]:
        tail_singles = True
    elif with_tail == whole:
        tail_singles = False
    else:
        raise UnsupportedTokenizer("the len %% k tail is neither dropped nor tokenised per character")
    spec = TokenizerSpec("kmer", sp, vs, singles, k=k, vocab=vocab, kmer_table5=table5,
                         kmer_run_offsets=np.asarray(offsets, np.int32), kmer_run_ids=np.asarray(flat, np.int32),
                         kmer_tail_singles=tail_singles)
    rng = np.random.default_rng(k)
    probes = ["".join(rng.choice(list("ACGTN"), size=int(n), p=[0.22, 0.22, 0.22, 0.22, 0.12]))
              for n in list(rng.integers(k, 6 * k + 1, size=48)) + [4 * k] * 16]
    for p, r in zip(probes, _ids(tok, probes)):
        if r != expected_kmer_table_ids(p, spec):
            raise UnsupportedTokenizer("replaying the k-mer window table does not reproduce the tokenizer (probe %r)" % p)
    return spec


def expected_kmer_table_ids(s: str, spec: TokenizerSpec) -> List[int]:
    """Window-table semantics spelled out (validates a probed table; also the checker of its tests)."""
    k, digit = spec.k, {"A": 0, "C": 1, "G": 2, "T": 3}
    out: List[int] = []
    n_full = len(s) // k
    for w in range(n_full):
        idx = 0
        for ch in s[w * k:(w + 1) * k]:
            idx = idx * 5 + digit.get(ch, 4)
        e = int(spec.kmer_table5[idx])
        if e >= 0:
            out.append(e)
        else:
            lo, hi = spec.kmer_run_offsets[-e - 1], spec.kmer_run_offsets[-e]
            out.extend(int(v) for v in spec.kmer_run_ids[lo:hi])
    if spec.kmer_tail_singles:
        out.extend(int(spec.lut256[ord(ch)]) for ch in s[n_full * k:])
    return out


def expected_kmer_ids(s: str, k: int, kmer_ids: np.ndarray, singles: np.ndarray) -> List[int]:
    """Table semantics spelled out (used only to validate a probed table)."""
    code = {"A": 0, "C": 1, "G": 2, "T": 3}
    out: List[int] = []
    for w in range(0, len(s), k):
        win = s[w:w + k]
        if len(win) == k and all(ch in code for ch in win):
            idx = 0
            for ch in win:
                idx = idx * 4 + code[ch]
            out.append(int(kmer_ids[idx]))
        else:
            out.extend(int(singles[ord(ch)]) for ch in win)
    return out


def spec_from_tokenizer(tok: Any) -> TokenizerSpec:
    """Pick the path the way the reference does: BPE by its tokenizer.json, else probe."""
    cfg = read_tokenizer_json(tok)
    if cfg is not None and (cfg.get("model") or {}).get("type") == "BPE":
        pad = getattr(tok, "pad_token_id", None)
        spec = bpe_spec_from_json(cfg, pad_id=int(pad) if pad is not None else None,
                                  padding_side=getattr(tok, "padding_side", "right"))
        u = getattr(tok, "unk_token_id", None)
        if u is not None and int(u) != spec.specials.unk_id:
            raise UnsupportedTokenizer("unk id mismatch between tokenizer and tokenizer.json")
        return spec
    return spec_from_probing(tok)
