"""Shared by the CPU and GPU tests: tokenizer specs for the five shapes and oracle calls."""
import functools
import hashlib

import numpy as np

from dnatok_b200 import synth, tables
from oracle import hf_oracle, oracle


def sha(a) -> str:
    return hashlib.sha256(np.ascontiguousarray(a).tobytes()).hexdigest()


@functools.lru_cache(maxsize=None)
def hf(name: str):
    return {"char": hf_oracle.char_tokenizer, "kmer6": hf_oracle.kmer_tokenizer,
            "byte": hf_oracle.byte_tokenizer,
            "bpe4096": lambda: hf_oracle.bpe_tokenizer("bpe4096"),
            "bpe32000": lambda: hf_oracle.bpe_tokenizer("bpe32000")}[name]()


@functools.lru_cache(maxsize=None)
def spec(name: str):
    return tables.spec_from_tokenizer(hf(name))


@functools.lru_cache(maxsize=None)
def bpe_table(name: str):
    s = spec(name)
    return oracle.BpeTable(s.merge_a, s.merge_b, s.merge_out)


def oracle_rows(name: str, flat, offsets, threads: int = 4):
    s = spec(name)
    ids, counts = oracle.encode_ragged(s.kind, flat, offsets, lut256=s.lut256, k=s.k, kmer_ids=s.kmer_ids,
                                       table=bpe_table(name) if s.kind == "bpe" else None, threads=threads)
    return oracle.rows(ids, offsets, counts)


def oracle_batch(name: str, flat, offsets, *, padding="longest", add_special=True, max_length=0,
                 truncation=False, pad_left=False, id_dtype=np.int64, mask_dtype=np.int64):
    s = spec(name)
    return oracle.assemble(oracle_rows(name, flat, offsets), pad_id=s.specials.pad_id, cls_id=s.specials.cls_id,
                           sep_id=s.specials.sep_id, add_special=add_special, max_length=max_length,
                           truncation=truncation, padding=padding, pad_left=pad_left, id_dtype=id_dtype,
                           mask_dtype=mask_dtype)


def config_inputs(cfg: str):
    """The inputs the golden file was generated on."""
    if cfg == "cfg1_char":
        return ("char",) + synth.pack_rows(synth.config1())
    if cfg == "cfg2_kmer6":
        return ("kmer6",) + synth.pack_rows(synth.config2())
    if cfg == "cfg3_bpe4096":
        return ("bpe4096",) + synth.pack_rows(synth.config3())
    if cfg == "cfg4_byte_2x131072":
        return ("byte",) + synth.pack_rows(synth.config4(batch=2, length=131072))
    if cfg == "cfg5_bpe32000_512reads":
        return ("bpe32000",) + synth.config5(n_reads=512)
    raise KeyError(cfg)


def call_to_kwargs(call: dict):
    pad = call.get("padding", False)
    return dict(padding="longest" if pad is True else pad, max_length=call.get("max_length", 0) or 0,
                truncation=bool(call.get("truncation", False)))


ALL_CONFIGS = ["cfg1_char", "cfg2_kmer6", "cfg3_bpe4096", "cfg4_byte_2x131072", "cfg5_bpe32000_512reads"]
TOKENIZERS = ["char", "kmer6", "bpe4096", "byte", "bpe32000"]


def pack_strs(strs):
    from dnatok_b200.pack import pack_strings
    return pack_strings(strs)


COMPAT_TOKENIZERS = ["NTv3Tokenizer", "Evo2ByteTokenizer", "CharTokenizer"]


def compat_spec(g: dict):
    """TokenizerSpec from the table recorded for one of the reference's own tokenizer classes."""
    return tables.TokenizerSpec(kind=g["kind"], vocab_size=g["vocab_size"], lut256=np.asarray(g["lut256"], dtype=np.int32),
                                specials=tables.Specials(pad_id=g["pad_id"], unk_id=g["unk_id"], cls_id=g["cls_id"],
                                                         sep_id=g["sep_id"]))
