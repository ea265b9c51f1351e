"""dnatok_b200 - genomic tokenizers (single-base / byte, k-mer, BPE) as sm_100a CUDA kernels
behind a C ABI, with a Hugging Face style front end.  No CPU fallback: the kernels are the
only implementation of the encode path."""
from .tables import TokenizerSpec, Specials, UnsupportedTokenizer, spec_from_tokenizer, bpe_spec_from_json

__all__ = ["B200Tokenizer", "GPUTokBPEBackend", "DnatokBpeKernel", "TokenizerSpec", "Specials",
           "UnsupportedTokenizer", "spec_from_tokenizer", "bpe_spec_from_json"]


def __getattr__(name):
    if name == "B200Tokenizer":
        from .tokenizer import B200Tokenizer
        return B200Tokenizer
    if name in ("GPUTokBPEBackend", "DnatokBpeKernel"):
        from . import gputok_bpe_backend
        return getattr(gputok_bpe_backend, name)
    raise AttributeError(name)
