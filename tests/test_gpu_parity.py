"""GPU parity: the CUDA kernels, called through the C ABI (ctypes), against the CPU checker,
the committed golden vectors and live Hugging Face.  Bit-exact everywhere (integer work)."""
import numpy as np
import pytest

from dnatok_b200 import synth

import helpers as H

pytestmark = pytest.mark.gpu

torch = pytest.importorskip("torch")


@pytest.fixture(params=["auto", "warp_teams", "block_teams", "teams_of_2", "teams_of_32", "launch_per_class", "table_in_global", "separate_output_pass"])
def bpe_team_mode(request):
    """Run a BPE test under each way of assigning warps to words (small batches would otherwise only
    ever see the wide-team kernels), and with one launch per length class instead of the shared one."""
    from dnatok_b200 import _cabi
    L = _cabi.lib()
    rows, warps, mixed, smem = {"auto": (-1, 0, 1, 1), "warp_teams": (0, 0, 1, 1), "block_teams": (1 << 40, 0, 1, 1),
                                "teams_of_2": (-1, 2, 1, 1), "teams_of_32": (-1, 32, 1, 1), "launch_per_class": (-1, 0, 0, 1),
                                "table_in_global": (-1, 0, 0, 0), "separate_output_pass": (-1, 0, 1, 1)}[request.param]
    _cabi.check(L.dnatok_set_option(b"bpe_fused_output", 0 if request.param == "separate_output_pass" else 1))
    _cabi.check(L.dnatok_set_option(b"bpe_block_team_rows", rows))
    _cabi.check(L.dnatok_set_option(b"bpe_team_warps", warps))
    _cabi.check(L.dnatok_set_option(b"bpe_mixed_launch", mixed))
    _cabi.check(L.dnatok_set_option(b"bpe_smem_table", smem))
    yield request.param
    _cabi.check(L.dnatok_set_option(b"bpe_block_team_rows", -1))
    _cabi.check(L.dnatok_set_option(b"bpe_team_warps", 0))
    _cabi.check(L.dnatok_set_option(b"bpe_mixed_launch", 1))
    _cabi.check(L.dnatok_set_option(b"bpe_smem_table", 1))
    _cabi.check(L.dnatok_set_option(b"bpe_fused_output", 1))


@pytest.fixture(scope="module")
def toks():
    if not torch.cuda.is_available():
        pytest.fail("GPU tests need a CUDA device")
    from dnatok_b200.tokenizer import B200Tokenizer
    return {n: B200Tokenizer(H.spec(n), device=0) for n in H.TOKENIZERS}


def dev(flat, offs):
    d_b = torch.from_numpy(np.ascontiguousarray(flat)).cuda() if len(flat) else torch.empty(0, dtype=torch.uint8, device="cuda")
    return d_b, torch.from_numpy(offs).cuda()


def run_device(tok, flat, offs, **kw):
    d_b, d_o = dev(flat, offs)
    enc = tok.encode_device(d_b, d_o, host_offsets=offs, **kw)
    torch.cuda.synchronize()
    return enc


@pytest.mark.parametrize("name,rows,length", [("bpe4096", 6000, 1024), ("bpe32000", 3000, 2000), ("bpe32000", 100, 2000),
                                              ("bpe4096", 700, 300)])
@pytest.mark.parametrize("side", ["right", "left"])
def test_bpe_rows_of_one_length_class(toks, name, rows, length, side):
    """Batches whose row bounds name one length class are not binned: more words than the GPU holds at once (words
    claimed from a counter), and fewer (every team takes the word its position names), with the merge kernel writing
    ids, mask, lengths and status itself; both padding sides; a few rows shorter than the rest."""
    tok = toks[name]
    flat, offs = synth.pack_rows(synth.config3(batch=rows, length=length, seed=rows))
    lens = np.diff(offs)
    lens[::97] = length - 5                                  # still the same class
    lens[5] = length - 200 if length > 1100 else length - 3
    offs2 = np.concatenate([[0], np.cumsum(lens)]).astype(np.int64)
    flat = np.concatenate([flat[offs[i]:offs[i] + lens[i]] for i in range(rows)])
    width = length // 3
    tok.padding_side = side
    try:
        enc = run_device(tok, flat, offs2, padding="max_length", max_length=width, truncation=True)
    finally:
        tok.padding_side = "right"
    o_ids, o_mask = H.oracle_batch(name, flat, offs2, padding="max_length", max_length=width, truncation=True,
                                   pad_left=(side == "left"))
    assert np.array_equal(enc["input_ids"].cpu().numpy(), o_ids)
    assert np.array_equal(enc["attention_mask"].cpu().numpy(), o_mask)
    assert np.array_equal(enc["lengths"].cpu().numpy(), o_mask.sum(axis=1))


@pytest.mark.parametrize("cfg", H.ALL_CONFIGS)
def test_golden_configs_device(golden, toks, cfg, bpe_team_mode):
    if bpe_team_mode != "auto" and "bpe" not in cfg:
        pytest.skip("team mode only concerns BPE")
    g = golden["configs"][cfg]
    name, flat, offs = H.config_inputs(cfg)
    kw = H.call_to_kwargs(g["call"])
    enc = run_device(toks[name], flat, offs, **kw)
    ids = enc["input_ids"].cpu().numpy()
    mask = enc["attention_mask"].cpu().numpy()
    assert ids.dtype == np.int64 and mask.dtype == np.int64
    assert list(ids.shape) == g["shape"]
    o_ids, o_mask = H.oracle_batch(name, flat, offs, **kw)
    assert np.array_equal(ids, o_ids)
    assert np.array_equal(mask, o_mask)
    assert H.sha(ids) == g["ids_sha256"] and H.sha(mask) == g["mask_sha256"]


@pytest.mark.parametrize("cfg", H.ALL_CONFIGS)
def test_golden_configs_host_entry(golden, toks, cfg):
    """Same through dnatok_encode_host (host buffers in and out)."""
    g = golden["configs"][cfg]
    name, flat, offs = H.config_inputs(cfg)
    kw = H.call_to_kwargs(g["call"])
    enc = toks[name].encode_host((flat, offs), **kw)
    assert H.sha(enc["input_ids"]) == g["ids_sha256"]
    assert H.sha(enc["attention_mask"]) == g["mask_sha256"]


def test_ragged_output_config5(golden, toks, bpe_team_mode):
    g = golden["configs"]["cfg5_bpe32000_512reads"]
    name, flat, offs = H.config_inputs("cfg5_bpe32000_512reads")
    enc = run_device(toks[name], flat, offs, padding=False)
    assert H.sha(enc["input_ids"].cpu().numpy()) == g["ragged_ids_sha256"]
    assert H.sha(enc["offsets"].cpu().numpy()) == g["ragged_offsets_sha256"]
    enc = toks[name].encode_host((flat, offs), padding=False)
    assert H.sha(enc["input_ids"]) == g["ragged_ids_sha256"]
    assert H.sha(enc["offsets"]) == g["ragged_offsets_sha256"]


def test_config4_int32_ids(toks):
    name, flat, offs = H.config_inputs("cfg4_byte_2x131072")
    enc = run_device(toks[name], flat, offs, ids_dtype=torch.int32, return_attention_mask=False)
    ids = enc["input_ids"].cpu().numpy()
    assert ids.dtype == np.int32
    assert np.array_equal(ids.reshape(-1), flat.astype(np.int32))


@pytest.mark.parametrize("name", H.TOKENIZERS)
def test_adversarial_strings(golden, toks, name):
    strs = golden["adversarial_inputs"]
    flat, offs = H.pack_strs(strs)
    for key, special in (("plain", False), ("special", True)):
        enc = run_device(toks[name], flat, offs, padding=False, add_special_tokens=special)
        ids = enc["input_ids"].cpu().numpy()
        oo = enc["offsets"].cpu().numpy()
        got = [ids[oo[i]:oo[i + 1]].tolist() for i in range(len(strs))]
        assert got == golden["adversarial"][name][key]
        # and padded, both sides, with a mask
        for left in (False, True):
            toks[name].padding_side = "left" if left else "right"
            try:
                enc = run_device(toks[name], flat, offs, padding="longest", add_special_tokens=special)
            finally:
                toks[name].padding_side = "right"
            o_ids, o_mask = H.oracle_batch(name, flat, offs, add_special=special, pad_left=left)
            assert np.array_equal(enc["input_ids"].cpu().numpy(), o_ids)
            assert np.array_equal(enc["attention_mask"].cpu().numpy(), o_mask)


@pytest.mark.parametrize("cls", H.COMPAT_TOKENIZERS)
def test_reference_tokenizer_classes(golden, cls):
    """The reference's own tokenizer classes (src/dnatok_compat.py:135-238): the kernel on the table
    discovered from each class reproduces the ids the class itself gave."""
    from dnatok_b200.tokenizer import B200Tokenizer
    g = golden["compat_tokenizers"]["tokenizers"][cls]
    tok = B200Tokenizer(H.compat_spec(g), device=0)
    strs = golden["compat_tokenizers"]["inputs"]
    flat, offs = H.pack_strs(strs)
    enc = run_device(tok, flat, offs, padding=False, add_special_tokens=False)
    ids, oo = enc["input_ids"].cpu().numpy(), enc["offsets"].cpu().numpy()
    assert [ids[oo[i]:oo[i + 1]].tolist() for i in range(len(strs))] == g["ids"]
    enc = run_device(tok, flat, offs, padding="longest", add_special_tokens=True)
    ids, mask = enc["input_ids"].cpu().numpy(), enc["attention_mask"].cpu().numpy()
    for i, want in enumerate(g["ids"]):
        assert ids[i, :len(want)].tolist() == want and mask[i].sum() == len(want)
        assert (ids[i, len(want):] == g["pad_id"]).all()


@pytest.mark.parametrize("name", H.TOKENIZERS)
@pytest.mark.parametrize("ids_dtype,mask_dtype", [("int64", "int64"), ("int32", "uint8"), ("int64", "int32")])
def test_ragged_lengths_truncation_dtypes(toks, name, ids_dtype, mask_dtype):
    rng = np.random.default_rng(3)
    B = 97
    lens = rng.integers(0, 3000, size=B)
    lens[:6] = [0, 1, 5, 6, 7, 2999]
    a = synth.config4(batch=B, length=3000, seed=9) if name == "byte" else synth.config1(batch=B, length=3000, seed=9)
    offs = np.concatenate([[0], np.cumsum(lens)]).astype(np.int64)
    flat = np.concatenate([a[i, :lens[i]] for i in range(B)])
    for kw in (dict(padding="longest"), dict(padding="max_length", max_length=333, truncation=True),
               dict(padding="longest", max_length=101, truncation=True, add_special_tokens=False)):
        enc = run_device(toks[name], flat, offs, ids_dtype=getattr(torch, ids_dtype),
                         mask_dtype=getattr(torch, mask_dtype), **kw)
        okw = dict(kw)
        okw["add_special"] = okw.pop("add_special_tokens", True)
        o_ids, o_mask = H.oracle_batch(name, flat, offs, id_dtype=getattr(np, ids_dtype),
                                       mask_dtype=getattr(np, mask_dtype), **okw)
        assert np.array_equal(enc["input_ids"].cpu().numpy(), o_ids)
        assert np.array_equal(enc["attention_mask"].cpu().numpy(), o_mask)
        assert np.array_equal(enc["lengths"].cpu().numpy(), o_mask.sum(axis=1))


@pytest.mark.parametrize("name", ["bpe4096", "bpe32000"])
def test_bpe_homopolymers_and_long_words(toks, name, bpe_team_mode):
    words = [b"A" * n for n in (1, 2, 3, 4, 5, 8, 9, 31, 32, 33, 64, 100, 255, 256, 257, 1024, 4097)]
    words += [b"AC" * 300, b"ACG" * 333, b"T" * 511 + b"A", b"N" * 70, b"ACGTNNNACGTnnacgt" * 40]
    words += [bytes(synth.config3(batch=1, length=n, seed=n)[0]) for n in (255, 256, 257, 1023, 1024, 1025, 2047, 2048, 2049, 4096, 4097, 8191, 8192, 8193, 16384,
                                                                       16385, 32767, 32768, 32769, 49152)]
    flat, offs = H.pack_strs(words)
    enc = run_device(toks[name], flat, offs, padding=False, add_special_tokens=False)
    ids = enc["input_ids"].cpu().numpy()
    oo = enc["offsets"].cpu().numpy()
    want = H.oracle_rows(name, flat, offs)
    for i in range(len(words)):
        assert ids[oo[i]:oo[i + 1]].tolist() == want[i].tolist(), "word %d (len %d)" % (i, len(words[i]))


@pytest.mark.parametrize("name", ["bpe4096", "bpe32000"])
def test_bpe_words_beyond_shared_memory(toks, name):
    """Words longer than the 32,768 positions a block keeps in shared memory go through the
    global-memory merge kernel (the reference has no per-input cap either:
    src/dnatok_bpe_kernel/dnatok_bpe.cu:276-297, :890-892)."""
    words = [bytes(synth.config3(batch=1, length=n, seed=n)[0]) for n in (32768, 32769, 49153, 100000)]
    words += [b"A" * 200000, b"ACGT" * 13000, b"AC" * 20000 + b"N" + b"T" * 40001, b"ACG"]
    flat, offs = H.pack_strs(words)
    enc = run_device(toks[name], flat, offs, padding=False, add_special_tokens=False)
    ids = enc["input_ids"].cpu().numpy()
    oo = enc["offsets"].cpu().numpy()
    want = H.oracle_rows(name, flat, offs)
    for i in range(len(words)):
        assert ids[oo[i]:oo[i + 1]].tolist() == want[i].tolist(), "word %d (len %d)" % (i, len(words[i]))


def test_bpe_megabase_words(toks):
    """Eight words of 1,048,576 bp (the byte-level shape's sizes) through a BPE tokenizer."""
    rows = synth.config3(batch=8, length=1 << 20, seed=99)
    flat, offs = synth.pack_rows(rows)
    enc = run_device(toks["bpe4096"], flat, offs, padding=False, add_special_tokens=True)
    ids = enc["input_ids"].cpu().numpy()
    oo = enc["offsets"].cpu().numpy()
    want = H.oracle_rows("bpe4096", flat, offs)
    sp = toks["bpe4096"].spec.specials
    for i in range(8):
        got = ids[oo[i]:oo[i + 1]]
        assert got[0] == sp.cls_id and got[-1] == sp.sep_id
        assert np.array_equal(got[1:-1], want[i]), "word %d" % i


def test_clipping_without_truncation_raises(toks):
    flat, offs = H.pack_strs(["ACGT" * 50, "AC"])
    with pytest.raises(ValueError, match="truncation is off"):
        run_device(toks["char"], flat, offs, padding="max_length", max_length=16)


def test_determinism_and_empty_batch(toks):
    name, flat, offs = H.config_inputs("cfg3_bpe4096")
    a = run_device(toks[name], flat, offs)["input_ids"].clone()
    b = run_device(toks[name], flat, offs)["input_ids"]
    assert torch.equal(a, b)
    enc = run_device(toks["char"], np.zeros(0, np.uint8), np.zeros(1, np.int64), padding="longest")
    assert tuple(enc["input_ids"].shape) == (0, 0)


def test_hf_call_surface_matches_live_hf(toks):
    """B200Tokenizer.__call__ against the live Hugging Face tokenizer objects, same kwargs."""
    strs = ["ACGTNACGT" * 7, "ACG", "", "TTTTNNNNACGTACGTAC", "acgtACGT"]
    for name in H.TOKENIZERS:
        hf, mine = H.hf(name), toks[name]
        for kw in (dict(padding=True), dict(padding="max_length", max_length=24, truncation=True),
                   dict(padding=True, add_special_tokens=False)):
            want = hf(strs, return_tensors="np", **kw)
            got = mine(strs, return_tensors="pt", **kw)
            assert got["input_ids"].dtype == torch.int64 and got["attention_mask"].dtype == torch.int64
            assert np.array_equal(got["input_ids"].cpu().numpy(), want["input_ids"]), (name, kw)
            assert np.array_equal(got["attention_mask"].cpu().numpy(), want["attention_mask"]), (name, kw)
        want = hf(strs)
        got = mine(strs)
        assert got["input_ids"] == [list(r) for r in want["input_ids"]]
        assert mine.encode(strs[0]) == hf.encode(strs[0])
        assert mine.pad_token_id == hf.pad_token_id


def test_bpe_backend_dropin(toks):
    """GPUTokBPEBackend / DnatokBpeKernel keep the reference's return contract."""
    from dnatok_b200.gputok_bpe_backend import DnatokBpeKernel, GPUTokBPEBackend
    hf = H.hf("bpe4096")
    assert GPUTokBPEBackend.is_supported(hf)
    be = GPUTokBPEBackend(hf, engine="dnatok")
    strs = synth.rows_to_strings(*synth.pack_rows(synth.config3(batch=33, length=700, seed=4))) + ["ACGTN" * 3, "A"]
    ids, mask = be.encode_batch(strs, device="cuda")
    assert ids.dtype == torch.int64 and mask.dtype == torch.uint8 and ids.is_cuda
    want = hf(strs, padding=True, add_special_tokens=False, return_tensors="np")
    assert np.array_equal(ids.cpu().numpy(), want["input_ids"])
    assert np.array_equal(mask.cpu().numpy(), want["attention_mask"].astype(np.uint8))
    assert (be.pad_id, be.unk_id, be.vocab_size) == (hf.pad_token_id, hf.unk_token_id, hf.vocab_size)
    with pytest.raises(ValueError):
        be.encode_batch([])
    k = DnatokBpeKernel.from_spec(H.spec("bpe4096"))
    kids, klens = k.tokenize_batch(strs)
    assert kids.dtype == torch.int32 and klens.dtype == torch.int32
    lens = want["attention_mask"].sum(axis=1)
    assert np.array_equal(klens.cpu().numpy(), lens)
    kid = kids.cpu().numpy()
    for i, n in enumerate(lens):
        assert np.array_equal(kid[i, :n], want["input_ids"][i, :n]) and not kid[i, n:].any()


def _kmer_spec(k):
    """A synthetic k-mer vocabulary laid out like the 6-mer one: specials, 4**k k-mers, then A C G T N."""
    from dnatok_b200.tables import Specials, TokenizerSpec
    lut = np.full(256, 1, np.int32)
    for i, c in enumerate("ACGTN"):
        lut[ord(c)] = 5 + 4 ** k + i
    rng = np.random.default_rng(k)
    return TokenizerSpec("kmer", Specials(0, 1, 2, 3), 10 + 4 ** k, lut, k=k,
                         kmer_ids=(5 + rng.permutation(4 ** k)).astype(np.int32))


@pytest.mark.parametrize("k,shape", [(6, "mixed"), (6, "uniform"), (3, "mixed"), (5, "long_tail"), (8, "mixed"),
                                     (2, "long_tail"), (1, "uniform"), (7, "mixed")])
def test_kmer_segment_queue_equals_row_per_warp(k, shape):
    """k-mer with scratch (rows cut into segments taken from a ticket queue) against the oracle and
    against the same call without scratch (one warp per row): rows of many segments, N runs that
    change the token parity between segments, a row far longer than the average, every output layout."""
    from dnatok_b200.tokenizer import B200Tokenizer
    from oracle import oracle
    spec = _kmer_spec(k)
    tok = B200Tokenizer(spec, device=0)
    rng = np.random.default_rng(7 * k + len(shape))
    if shape == "uniform":
        lens = np.full(300, 6000)
    elif shape == "mixed":
        lens = rng.integers(0, 40000, size=150)
        lens[:6] = [0, 1, 256 * k, 256 * k + 1, 257 * k, 512 * k + k - 1]
    else:
        lens = rng.integers(0, 3000, size=200)
        lens[17] = 700001 if k >= 5 else 200001
    rows_b = []
    for n in lens:
        r = np.frombuffer(b"ACGT", np.uint8)[rng.integers(0, 4, int(n))].copy()
        for _ in range(int(n) // 1500):
            s0 = int(rng.integers(0, n))
            r[s0:s0 + int(rng.integers(1, 40))] = ord("N")
        rows_b.append(r)
    offs = np.concatenate([[0], np.cumsum(lens)]).astype(np.int64)
    flat = np.concatenate(rows_b) if len(rows_b) else np.zeros(0, np.uint8)
    ids, counts = oracle.encode_ragged("kmer", flat, offs, lut256=spec.lut256, k=k, kmer_ids=spec.kmer_ids)
    rows = oracle.rows(ids, offs, counts)
    calls = [dict(padding="longest"), dict(padding="max_length", max_length=1000, truncation=True),
             dict(padding="longest", add_special_tokens=False, ids_dtype=torch.int32, mask_dtype=torch.uint8),
             dict(padding="max_length", max_length=777, truncation=True, add_special_tokens=False),
             dict(padding="longest", ids_dtype=torch.int32, mask_dtype=torch.int32)]
    for left in (False, True):
        tok.padding_side = "left" if left else "right"
        for kw in calls:
            a = run_device(tok, flat, offs, **kw)
            b = run_device(tok, flat, offs, scratch=False, **kw)
            want_ids, want_mask = oracle.assemble(rows, pad_id=0, cls_id=2, sep_id=3,
                                                  add_special=kw.get("add_special_tokens", True),
                                                  max_length=kw.get("max_length", 0), truncation=kw.get("truncation", False),
                                                  padding=kw["padding"], pad_left=left)
            for enc in (a, b):
                assert np.array_equal(enc["input_ids"].cpu().numpy(), want_ids), (kw, left)
                assert np.array_equal(enc["attention_mask"].cpu().numpy(), want_mask), (kw, left)
                assert np.array_equal(enc["lengths"].cpu().numpy()[:len(lens)], want_mask.sum(axis=1)), (kw, left)
    tok.padding_side = "right"
    want = np.concatenate(oracle.assemble(rows, pad_id=0, cls_id=2, sep_id=3, padding=False))
    for sc in (None, False):
        enc = run_device(tok, flat, offs, padding=False, scratch=sc)
        assert np.array_equal(enc["input_ids"].cpu().numpy()[:len(want)], want)


@pytest.mark.parametrize("k", [1, 2, 3, 4, 5, 7, 8])
def test_kmer_other_k(k):
    """Every window width the kernel is instantiated for, ragged rows, odd byte alignments."""
    from dnatok_b200.tokenizer import B200Tokenizer
    from oracle import oracle
    spec = _kmer_spec(k)
    tok = B200Tokenizer(spec, device=0)
    rng = np.random.default_rng(100 + k)
    B = 61
    lens = rng.integers(0, 1500, size=B)
    lens[:5] = [0, 1, k - 1 if k > 1 else 1, k, k + 1]
    a = synth.config1(batch=B, length=1500, seed=k)
    a[3, :] = np.frombuffer(b"ACGT", np.uint8)[rng.integers(0, 4, 1500)]           # an all-clean row
    a[7, 100:160] |= 0x20                                                          # lower-case stretch
    offs = np.concatenate([[0], np.cumsum(lens)]).astype(np.int64)
    flat = np.concatenate([a[i, :lens[i]] for i in range(B)])
    ids, counts = oracle.encode_ragged("kmer", flat, offs, lut256=spec.lut256, k=k, kmer_ids=spec.kmer_ids)
    rows = oracle.rows(ids, offs, counts)
    for kw in (dict(padding="longest"), dict(padding="max_length", max_length=97, truncation=True),
               dict(padding="longest", add_special_tokens=False, ids_dtype=torch.int32)):
        enc = run_device(tok, flat, offs, **kw)
        want_ids, want_mask = oracle.assemble(rows, pad_id=0, cls_id=2, sep_id=3,
                                              add_special=kw.get("add_special_tokens", True),
                                              max_length=kw.get("max_length", 0), truncation=kw.get("truncation", False),
                                              padding=kw["padding"])
        assert np.array_equal(enc["input_ids"].cpu().numpy(), want_ids), kw
        assert np.array_equal(enc["attention_mask"].cpu().numpy(), want_mask), kw
    enc = run_device(tok, flat, offs, padding=False)
    got = enc["input_ids"].cpu().numpy()
    oo = enc["offsets"].cpu().numpy()
    want = oracle.assemble(rows, pad_id=0, cls_id=2, sep_id=3, padding=False)
    for i in range(B):
        assert np.array_equal(got[oo[i]:oo[i + 1]], want[i]), i


def test_kmer_very_long_rows_use_block_kernel(toks):
    """Average row length above the warp-per-row limit: the block-per-row kernel."""
    a = synth.config2(batch=3, length=100003, seed=77)
    flat, offs = synth.pack_rows(a)
    for kw in (dict(padding="longest", add_special_tokens=False), dict(padding="max_length", max_length=9000, truncation=True)):
        enc = run_device(toks["kmer6"], flat, offs, **kw)
        okw = dict(kw)
        okw["add_special"] = okw.pop("add_special_tokens", True)
        o_ids, o_mask = H.oracle_batch("kmer6", flat, offs, **okw)
        assert np.array_equal(enc["input_ids"].cpu().numpy(), o_ids)
        assert np.array_equal(enc["attention_mask"].cpu().numpy(), o_mask)


def test_bpe_table_with_late_created_operands_single_step(bpe_team_mode):
    """A merge list whose operands are created by LATER ranks (not what BpeTrainer emits): the kernel
    must fall back to one merge per round and still equal the queue semantics of the checker."""
    from dnatok_b200.tables import Specials, TokenizerSpec
    from dnatok_b200.tokenizer import B200Tokenizer
    from oracle import oracle
    lut = np.full(256, 1, np.int32)
    for i, c in enumerate("ACGT"):
        lut[ord(c)] = 5 + i
    # rank 0 names token 10 ("AC"), which only rank 1 creates; rank 4 names 14, created by rank 5
    a = np.array([10, 5, 7, 12, 14, 8, 6, 9], np.int32)
    b = np.array([8, 6, 7, 12, 5, 8, 7, 9], np.int32)
    o = np.array([11, 10, 12, 13, 15, 14, 9, 16], np.int32)
    spec = TokenizerSpec("bpe", Specials(0, 1, 2, 3), 32, lut, merge_a=a, merge_b=b, merge_out=o)
    tok = B200Tokenizer(spec, device=0)
    table = oracle.BpeTable(a, b, o)
    rng = np.random.default_rng(5)
    words = [bytes(np.frombuffer(b"ACGT", np.uint8)[rng.integers(0, 4, int(n))]) for n in rng.integers(1, 400, 40)]
    words += [b"ACT" * 50, b"GGGGGGGGGGGGGGGGG", b"TTA" * 33, b"ACTTTTACGGGG" * 20, b"CGCGCGCGCG" * 9]
    flat, offs = H.pack_strs(words)
    enc = run_device(tok, flat, offs, padding=False, add_special_tokens=False)
    ids = enc["input_ids"].cpu().numpy()
    oo = enc["offsets"].cpu().numpy()
    for i, w in enumerate(words):
        assert ids[oo[i]:oo[i + 1]].tolist() == oracle.bpe_word(table, w, lut), i


@pytest.mark.parametrize("k", [1, 2, 3, 4, 5, 7, 8])
@pytest.mark.parametrize("shuffled", [False, True])
def test_kmer_other_window_lengths(k, shuffled):
    """Every window length the kernels are built for (6 is covered by the benchmark shape), with the table in vocabulary
    order (ids = base + index, no gather) and shuffled (gather): ragged rows with N runs and lower case, padded with both
    sides and ragged, large batch (one warp per row) and few long rows (segments), against the checker."""
    import dataclasses
    from dnatok_b200.tables import Specials, TokenizerSpec
    from dnatok_b200.tokenizer import B200Tokenizer
    from oracle import oracle
    rng = np.random.default_rng(40 + k)
    n = 4 ** k
    kmer_ids = np.arange(10, 10 + n, dtype=np.int32)
    if shuffled:
        kmer_ids = kmer_ids[rng.permutation(n)]
    lut = np.full(256, 1, np.int32)
    for i, c in enumerate(b"ACGTN"):
        lut[c] = 4 + i
    spec = TokenizerSpec("kmer", Specials(0, 1, 2, 3), 10 + n, lut, k=k, kmer_ids=kmer_ids)
    tok = B200Tokenizer(spec, device=0)

    def rows(lens):
        out = []
        for m in lens:
            r = np.frombuffer(b"ACGT", np.uint8)[rng.integers(0, 4, int(m))].copy()
            for _ in range(int(m) // 400 + (1 if m and rng.random() < 0.5 else 0)):
                s0 = int(rng.integers(0, m)); r[s0:s0 + int(rng.integers(1, 30))] = ord("N")
            if m > 3 and rng.random() < 0.3:
                r[int(rng.integers(0, m))] = ord("a")
            out.append(r)
        flat = np.concatenate(out) if out else np.zeros(0, np.uint8)
        return flat, np.concatenate([[0], np.cumsum([len(r) for r in out])]).astype(np.int64)

    def check(flat, offs, **kw):
        ids, counts = oracle.encode_ragged("kmer", flat, offs, lut256=lut, k=k, kmer_ids=kmer_ids, table=None, threads=2)
        want_rows = oracle.rows(ids, offs, counts)
        okw = dict(kw)
        pad_left = okw.pop("pad_left", False)
        tok.padding_side = "left" if pad_left else "right"
        try:
            enc = run_device(tok, flat, offs, **kw_strip(kw))
        finally:
            tok.padding_side = "right"
        if kw.get("padding") is False:
            got, oo = enc["input_ids"].cpu().numpy(), enc["offsets"].cpu().numpy()
            for i, w in enumerate(want_rows):
                assert got[oo[i]:oo[i + 1]].tolist() == list(w), (k, i)
        else:
            o_ids, o_mask = oracle.assemble(want_rows, pad_id=0, cls_id=2, sep_id=3, add_special=True,
                                            max_length=okw.get("max_length", 0), truncation=okw.get("truncation", False),
                                            padding=okw["padding"], pad_left=pad_left, id_dtype=np.int64, mask_dtype=np.int64)
            assert np.array_equal(enc["input_ids"].cpu().numpy(), o_ids), k
            assert np.array_equal(enc["attention_mask"].cpu().numpy(), o_mask), k

    def kw_strip(kw):
        return {a: b for a, b in kw.items() if a != "pad_left"}

    lens = list(rng.integers(0, 3000, 1500)) + [0, 1, k - 1, k, k + 1, 64 * k, 64 * k + 1, 128 * k - 1, 256 * k, 257 * k + 3]
    flat, offs = rows(lens)
    check(flat, offs, padding="max_length", max_length=300, truncation=True)
    check(flat, offs, padding="longest", pad_left=True)
    check(flat, offs, padding=False, add_special_tokens=False)
    flat, offs = rows([70000, 5, 40000 + k, 123457])          # few long rows: the segment encoder
    check(flat, offs, padding="longest")
    check(flat, offs, padding="max_length", max_length=5000, truncation=True, pad_left=True)


@pytest.mark.parametrize("seed", range(12))
def test_bpe_random_merge_tables(seed):
    _random_merge_tables(seed)


@pytest.mark.parametrize("seed", [100, 101, 102])
def test_bpe_random_merge_tables_every_way_of_running(seed, bpe_team_mode):
    _random_merge_tables(seed)


def _random_merge_tables(seed):
    """Merge tables that no trainer produced: random pairs of already created tokens (so operands always come from
    lower ranks), alphabets whose first ids lie below or above the small-id table, 20 to 700 merges; random words with
    homopolymer stretches, one length class (padded, written by the merge kernel) and mixed lengths (ragged), against
    the queue semantics of the checker."""
    from dnatok_b200.tables import Specials, TokenizerSpec
    from dnatok_b200.tokenizer import B200Tokenizer
    from oracle import oracle
    rng = np.random.default_rng(1000 + seed)
    n_sym = int(rng.integers(2, 7))
    first = int(rng.choice([5, 20, 31, 40, 300]))
    lut = np.full(256, 1, np.int32)
    letters = b"ACGTNR"[:n_sym]
    for i, c in enumerate(letters):
        lut[c] = first + i
    tokens = [first + i for i in range(n_sym)]
    n_merges = int(rng.integers(20, 700))
    seen, a, b, o = set(), [], [], []
    nxt = first + n_sym
    while len(a) < n_merges:
        # pairs lean towards early tokens, as a trained vocabulary's do
        x = tokens[int(min(len(tokens) - 1, rng.exponential(len(tokens) / 3)))]
        y = tokens[int(min(len(tokens) - 1, rng.exponential(len(tokens) / 3)))]
        if (x, y) in seen:
            continue
        seen.add((x, y))
        a.append(x); b.append(y); o.append(nxt)
        tokens.append(nxt)
        nxt += 1
    a, b, o = (np.array(v, np.int32) for v in (a, b, o))
    spec = TokenizerSpec("bpe", Specials(0, 1, 2, 3), nxt, lut, merge_a=a, merge_b=b, merge_out=o)
    tok = B200Tokenizer(spec, device=0)
    table = oracle.BpeTable(a, b, o)

    def word(n):
        out = []
        while len(out) < n:
            c = letters[int(rng.integers(0, n_sym))]
            out += [c] * int(rng.choice([1, 1, 1, 2, 3, 7, 40]))
        return bytes(out[:n])

    # mixed lengths, ragged output
    words = [word(int(n)) for n in rng.integers(1, 3000, 60)] + [word(1), word(2), word(1024), word(1025)]
    flat, offs = H.pack_strs(words)
    enc = run_device(tok, flat, offs, padding=False, add_special_tokens=False)
    ids, oo = enc["input_ids"].cpu().numpy(), enc["offsets"].cpu().numpy()
    want = [oracle.bpe_word(table, w, lut) for w in words]
    for i in range(len(words)):
        assert ids[oo[i]:oo[i + 1]].tolist() == want[i], (seed, i)
    # one length class, padded, with special tokens
    words = [word(int(n)) for n in rng.integers(600, 1025, 300)]
    flat, offs = H.pack_strs(words)
    enc = run_device(tok, flat, offs, padding="max_length", max_length=400, truncation=True)
    ids, lens = enc["input_ids"].cpu().numpy(), enc["lengths"].cpu().numpy()
    for i, w in enumerate(words):
        t = oracle.bpe_word(table, w, lut)[:398]
        assert ids[i, :len(t) + 2].tolist() == [2] + t + [3] and lens[i] == len(t) + 2, (seed, i)
        assert (ids[i, len(t) + 2:] == 0).all()


@pytest.mark.parametrize("name,rows,length,kw", [
    ("char", 8192, 1024, dict(padding="longest")),
    ("kmer6", 4096, 6000, dict(padding="max_length", max_length=1000, truncation=True, add_special_tokens=False)),
    ("bpe4096", 6144, 1024, dict(padding="max_length", max_length=768)),
])
@pytest.mark.parametrize("mask_threads", [-1, 0])
def test_host_entry_chunked_pipeline(toks, name, rows, length, kw, mask_threads):
    """Batches large enough for dnatok_encode_host to split into chunks whose copies and kernels overlap,
    with the mask written by host threads chunk by chunk (-1) or copied from the device (0)."""
    gen = {"char": synth.config1, "kmer6": synth.config2, "bpe4096": synth.config3}[name]
    flat, offs = synth.pack_rows(gen(batch=rows, length=length, seed=1234))
    # ragged tail so the chunks differ in size
    lens = np.diff(offs)
    lens[-7:] = [0, 1, 5, length // 2, 17, length - 1, 3]
    offs2 = np.concatenate([[0], np.cumsum(lens)]).astype(np.int64)
    flat2 = np.concatenate([flat[offs[i]:offs[i] + lens[i]] for i in range(rows - 7, rows)])
    flat = np.concatenate([flat[:offs[rows - 7]], flat2])
    from dnatok_b200 import _cabi
    L = _cabi.lib()
    _cabi.check(L.dnatok_set_option(b"host_chunk_bytes", 4 << 20))
    _cabi.check(L.dnatok_set_option(b"host_chunk_threshold", 0))
    _cabi.check(L.dnatok_set_option(b"host_mask_threads", mask_threads))
    try:
        enc = toks[name].encode_host((flat, offs2), **kw)
    finally:
        _cabi.check(L.dnatok_set_option(b"host_chunk_bytes", 64 << 20))
        _cabi.check(L.dnatok_set_option(b"host_chunk_threshold", 128 << 20))
        _cabi.check(L.dnatok_set_option(b"host_mask_threads", -1))
    okw = dict(kw)
    okw["add_special"] = okw.pop("add_special_tokens", True)
    o_ids, o_mask = H.oracle_batch(name, flat, offs2, **okw)
    assert np.array_equal(enc["input_ids"], o_ids)
    assert np.array_equal(enc["attention_mask"], o_mask)
    assert np.array_equal(enc["lengths"], o_mask.sum(axis=1))


@pytest.mark.parametrize("early", [1, 0])
@pytest.mark.parametrize("pad_left", [False, True])
def test_host_entry_mask_from_row_sizes(toks, early, pad_left):
    """Rows whose token count follows from their byte count (k-mer rows with at least max_length complete windows, N runs
    or not): the host writes the mask without waiting for the GPU's lengths, which must agree with it."""
    from dnatok_b200 import _cabi
    L = _cabi.lib()
    tok = toks["kmer6"]
    flat, offs = synth.pack_rows(synth.config2(batch=3000, length=6003, seed=77))
    kw = dict(padding="max_length", max_length=1000, truncation=True, add_special_tokens=False)
    _cabi.check(L.dnatok_set_option(b"host_chunk_bytes", 4 << 20))
    _cabi.check(L.dnatok_set_option(b"host_chunk_threshold", 0))
    _cabi.check(L.dnatok_set_option(b"host_mask_min_bytes", 0))
    _cabi.check(L.dnatok_set_option(b"host_mask_early", early))
    tok.padding_side = "left" if pad_left else "right"
    try:
        enc = tok.encode_host((flat, offs), **kw)
    finally:
        tok.padding_side = "right"
        _cabi.check(L.dnatok_set_option(b"host_chunk_bytes", 64 << 20))
        _cabi.check(L.dnatok_set_option(b"host_chunk_threshold", 128 << 20))
        _cabi.check(L.dnatok_set_option(b"host_mask_min_bytes", 16 << 20))
        _cabi.check(L.dnatok_set_option(b"host_mask_early", 1))
    o_ids, o_mask = H.oracle_batch("kmer6", flat, offs, padding="max_length", max_length=1000, truncation=True,
                                   add_special=False, pad_left=pad_left)
    assert np.array_equal(enc["input_ids"], o_ids)
    assert np.array_equal(enc["attention_mask"], o_mask)
    assert enc["attention_mask"].all() and np.array_equal(enc["lengths"], np.full(3000, 1000))


@pytest.mark.parametrize("name", ["char", "kmer6", "bpe4096"])
@pytest.mark.parametrize("mask_dtype", [np.int64, np.int32, np.uint8])
def test_host_entry_mask_written_by_host_threads(toks, name, mask_dtype):
    """dnatok_encode_host with the attention mask written by host threads from the GPU's row lengths
    (forced here for a small batch) against the same call with the mask copied from the device and
    against the oracle: ragged rows, empty rows, both padding sides, truncation."""
    import ctypes
    from dnatok_b200 import _cabi
    L = _cabi.lib()
    rng = np.random.default_rng(5)
    B = 211
    lens = rng.integers(0, 2000, size=B)
    lens[:4] = [0, 1, 1999, 6]
    a = synth.config3(batch=B, length=2000, seed=77) if name == "bpe4096" else synth.config2(batch=B, length=2000, seed=77)
    offs = np.concatenate([[0], np.cumsum(lens)]).astype(np.int64)
    flat = np.concatenate([a[i, :lens[i]] for i in range(B)])
    tok = toks[name]
    for left in (False, True):
        tok.padding_side = "left" if left else "right"
        try:
            for kw in (dict(padding="longest"), dict(padding="max_length", max_length=150, truncation=True)):
                got = {}
                for threads in (3, 0):
                    _cabi.check(L.dnatok_set_option(b"host_mask_threads", threads))
                    _cabi.check(L.dnatok_set_option(b"host_mask_min_bytes", 0))
                    try:
                        got[threads] = tok.encode_host((flat, offs), mask_dtype=mask_dtype, **kw)
                        h2d, d2h = ctypes.c_int64(0), ctypes.c_int64(0)
                        L.dnatok_host_copy_bytes(ctypes.byref(h2d), ctypes.byref(d2h))
                        got[threads]["d2h"] = d2h.value
                    finally:
                        _cabi.check(L.dnatok_set_option(b"host_mask_threads", -1))
                        _cabi.check(L.dnatok_set_option(b"host_mask_min_bytes", 16 << 20))
                o_ids, o_mask = H.oracle_batch(name, flat, offs, pad_left=left,
                                               **{k: v for k, v in kw.items()})
                for threads in (3, 0):
                    assert got[threads]["attention_mask"].dtype == mask_dtype
                    assert np.array_equal(got[threads]["input_ids"], o_ids), (kw, left, threads)
                    assert np.array_equal(got[threads]["attention_mask"], o_mask), (kw, left, threads)
                # the mask crossed the link only in the second call
                assert got[0]["d2h"] - got[3]["d2h"] == o_mask.size * np.dtype(mask_dtype).itemsize
                # the same with 32-bit ids
                _cabi.check(L.dnatok_set_option(b"host_mask_min_bytes", 0))
                try:
                    e32 = tok.encode_host((flat, offs), mask_dtype=mask_dtype, ids_dtype=np.int32, **kw)
                finally:
                    _cabi.check(L.dnatok_set_option(b"host_mask_min_bytes", 16 << 20))
                assert e32["input_ids"].dtype == np.int32 and np.array_equal(e32["input_ids"], o_ids)
                assert np.array_equal(e32["attention_mask"], o_mask)
        finally:
            tok.padding_side = "right"


def test_dnatok_api_matches_reference_outputs(golden):
    """dnatok_b200.dna_tokenizer.DNATok against what the reference's DNATok returned for the same calls
    (recorded by tests/golden/make_golden.py): encode_batch_to_ids and encode_batch_with_padding."""
    from dnatok_b200.dna_tokenizer import DNATok

    class Embedder:
        def __init__(self, tokenizer):
            self.tokenizer = tokenizer

        def embed_tokens(self, ids):
            return ids

    api = golden["dnatok_api"]
    seqs = api["seqs"]
    for case in api["cases"]:
        helper = DNATok(Embedder(H.hf(case["tokenizer"])), padding_side=case["padding_side"])
        helper.discover()
        assert helper.use_ids_path
        assert (helper.kmer_k or 1) == (6 if case["tokenizer"] == "kmer6" else 1)
        ids = helper.encode_batch_to_ids(seqs)
        assert ids.dtype == torch.int64 and ids.device.type == "cpu" and ids.is_pinned()
        if case["tokenizer"] == "kmer6" and case["padding_side"] == "left":
            # For ragged k-mer rows the reference pads each equal-length group on the left and the merged
            # tensor on the right, so a row's tokens end up in the middle of its row.  Same tokens per
            # row are required here; the placement is a consistent left padding.
            pad = helper.id_pad
            for mine, ref in zip(ids.tolist(), case["encode_batch_to_ids"]):
                assert [t for t in mine if t != pad] == [t for t in ref if t != pad]
                n = sum(t != pad for t in mine)
                assert all(t == pad for t in mine[:len(mine) - n])
        else:
            assert ids.tolist() == case["encode_batch_to_ids"]
        for w in case["with_padding"]:
            i2, m2 = helper.encode_batch_with_padding(seqs, w["max_tokens"], pad_to_max=w["pad_to_max"],
                                                      pad_multiple=w["pad_multiple"])
            assert str(i2.dtype) == w["ids_dtype"] and str(m2.dtype) == w["mask_dtype"]
            assert i2.tolist() == w["ids"], (case["tokenizer"], case["padding_side"], w["max_tokens"])
            assert m2.tolist() == w["mask"]
        with pytest.raises(ValueError, match="No sequences provided"):
            helper.encode_batch_to_ids([])
        with pytest.raises(ValueError, match="Empty batch"):
            helper.encode_batch_with_padding([], 8)
    # BPE goes through the backend slot, as in the reference's discover()
    helper = DNATok(Embedder(H.hf("bpe4096")), padding_side="right")
    helper.discover()
    assert not helper.use_ids_path and helper.bpe_backend is not None
    ids = helper.encode_batch_to_ids(seqs)
    want = H.hf("bpe4096")(seqs, padding=True, add_special_tokens=False, return_tensors="np")["input_ids"]
    assert np.array_equal(ids.numpy(), want)
    helper.padding_side = "left"
    ids_left = helper.encode_batch_to_ids(seqs)
    lens = (want != helper.pad_id).sum(axis=1)
    for i, n in enumerate(lens):
        assert ids_left[i, ids_left.shape[1] - n:].tolist() == want[i, :n].tolist()


def test_full_size_config4_byte_level(toks):
    """Benchmark shape 4 at its full size (8 x 1,048,576 bp, int32 ids): byte-level ids are the bytes themselves."""
    flat, offs = synth.pack_rows(synth.config4())
    enc = run_device(toks["byte"], flat, offs, ids_dtype=torch.int32, return_attention_mask=False)
    ids = enc["input_ids"]
    assert tuple(ids.shape) == (8, 1048576) and ids.dtype == torch.int32
    assert torch.equal(ids.reshape(-1), torch.from_numpy(flat).cuda().to(torch.int32))
    assert int(enc["lengths"].min()) == 1048576


def test_full_size_config5_reads(toks):
    """Benchmark shape 5 at its full size (16,384 reads, ~38 Mbp, ragged output): equal to the CPU checker on
    every read, and decoding the ids through the vocabulary gives back the input bytes."""
    flat, offs = synth.config5()
    enc = run_device(toks["bpe32000"], flat, offs, padding=False, add_special_tokens=False)
    ids = enc["input_ids"].cpu().numpy()
    oo = enc["offsets"].cpu().numpy()
    want = H.oracle_rows("bpe32000", flat, offs, threads=8)
    assert np.array_equal(np.diff(oo), np.array([len(r) for r in want]))
    assert np.array_equal(ids, np.concatenate(want))
    spec = H.spec("bpe32000")
    inv = {v: k for k, v in spec.vocab.items()}
    tok_len = np.zeros(max(inv) + 1, dtype=np.int64)
    for i, t in inv.items():
        tok_len[i] = len(t)
    assert int(tok_len[ids].sum()) == int(offs[-1])            # every base is covered exactly once
    for r in (0, 1, 4097, 16383):
        text = "".join(inv[int(t)] for t in ids[oo[r]:oo[r + 1]])
        assert text.encode() == bytes(flat[offs[r]:offs[r + 1]])


def test_full_size_config3_property(toks):
    """Shape 3 scaled 16x (16,384 words): same ids as the checker on a sample, and the padded tensor is
    consistent with its lengths (mask sum, [CLS] first, [SEP] last, pad after)."""
    flat, offs = synth.pack_rows(synth.config3(batch=16384, seed=31))
    enc = run_device(toks["bpe4096"], flat, offs, padding="longest")
    ids, mask, lens = enc["input_ids"], enc["attention_mask"], enc["lengths"].long()
    assert torch.equal(mask.sum(dim=1), lens)
    assert bool((ids[:, 0] == 2).all()) and bool((ids.gather(1, (lens - 1).unsqueeze(1)) == 3).all())
    assert bool(((ids == 0) == (mask == 0)).all())
    sample = np.arange(0, 16384, 257)
    from dnatok_b200.shard import take_rows
    f2, o2 = take_rows(flat, offs, sample)
    want = H.oracle_rows("bpe4096", f2, o2)
    got = ids.cpu().numpy()
    for j, r in enumerate(sample):
        n = int(lens[r]) - 2
        assert got[r, 1:1 + n].tolist() == want[j].tolist()


@pytest.mark.parametrize("name", H.TOKENIZERS)
def test_seeded_fuzz_against_live_hf(toks, name):
    """Random batches over a dirty alphabet, random lengths and call options, against the live Hugging Face
    tokenizer (not the checker): ids, mask, padding side."""
    import zlib
    rng = np.random.default_rng(zlib.crc32(name.encode()) % 1000 + 17)
    alphabet = np.frombuffer(b"ACGTACGTACGTACGTNNacgtnRYKM-_0xX", np.uint8)
    hf, mine = H.hf(name), toks[name]
    for trial in range(25):
        B = int(rng.integers(1, 24))
        lens = rng.integers(0, 260, size=B)
        if trial % 5 == 0:
            lens[rng.integers(0, B)] = int(rng.integers(1000, 5000))
        strs = [bytes(alphabet[rng.integers(0, len(alphabet), int(n))]).decode() for n in lens]
        if trial % 7 == 3:
            strs[0] = "A" * int(rng.integers(1, 700))
        special = bool(rng.integers(0, 2))
        mode = int(rng.integers(0, 3))
        if mode == 0:
            kw = dict(padding=True)
        elif mode == 1:
            kw = dict(padding="max_length", max_length=int(rng.integers(2, 300)), truncation=True)
        else:
            kw = dict(padding=True, max_length=int(rng.integers(2, 120)), truncation=True)
        for side in ("right", "left"):
            hf.padding_side = side
            mine.padding_side = side
            try:
                want = hf(strs, add_special_tokens=special, return_tensors="np", **kw)
                got = mine(strs, add_special_tokens=special, return_tensors="pt", **kw)
            finally:
                hf.padding_side = "right"
                mine.padding_side = "right"
            assert np.array_equal(got["input_ids"].cpu().numpy(), want["input_ids"]), (name, trial, side, kw, special)
            assert np.array_equal(got["attention_mask"].cpu().numpy(), want["attention_mask"]), (name, trial, side, kw)
        rows = hf(strs, add_special_tokens=special)["input_ids"]
        assert mine(strs, add_special_tokens=special)["input_ids"] == [list(r) for r in rows]


def test_kmer_segment_wait_runs_out_on_one_row_only():
    """The bounded wait of the k-mer segment encoder: one segment is told (test option) to publish nothing
    and the poll limit is set to a few polls, so the later segments of that row give up.  That row gets
    DNATOK_ROW_STALLED, every other row is exact, and the call returns at once.  Nothing waits for ever:
    the wait ends after poll_limit polls whatever happens."""
    import ctypes, time
    from dnatok_b200 import _cabi
    L = _cabi.lib()
    spec = H.spec("kmer6")
    handle = _cabi.Handle(spec)
    rows, length = 12, 6 * 256 * 5 + 77                  # six segments per row
    flat, offs = synth.pack_rows(synth.config2(batch=rows, length=length, seed=77))
    d_b, d_o = dev(flat, offs)
    B, total = rows, len(flat)
    stride = 1400
    need = L.dnatok_scratch_bytes(handle.ptr, B, total)
    scratch = torch.empty(need, dtype=torch.uint8, device="cuda")
    ids = torch.zeros((B, stride), dtype=torch.int64, device="cuda")
    mask = torch.zeros((B, stride), dtype=torch.int64, device="cuda")
    lengths = torch.zeros(B, dtype=torch.int32, device="cuda")
    status = torch.zeros(B, dtype=torch.int32, device="cuda")
    fmt = _cabi.Format(64, 64, 0, 0, stride, stride)
    p = lambda t: ctypes.c_void_p(t.data_ptr())
    victim = 3
    _cabi.check(L.dnatok_set_option(b"kmer_force_segments", 1))
    _cabi.check(L.dnatok_set_option(b"kmer_poll_limit", 8))
    _cabi.check(L.dnatok_set_option(b"kmer_test_withhold_ticket", 1 * rows + victim))    # segment 1 of the victim row
    try:
        t0 = time.perf_counter()
        _cabi.check(L.dnatok_encode(handle.ptr, p(d_b), p(d_o), B, total, ctypes.byref(fmt), p(ids), p(mask), p(lengths),
                                    None, p(status), p(scratch), need, None))
        torch.cuda.synchronize()
        took = time.perf_counter() - t0
    finally:
        _cabi.check(L.dnatok_set_option(b"kmer_force_segments", 0))
        _cabi.check(L.dnatok_set_option(b"kmer_poll_limit", 1 << 20))
        _cabi.check(L.dnatok_set_option(b"kmer_test_withhold_ticket", -1))
    assert took < 1.0
    st = status.cpu().numpy()
    assert st[victim] & _cabi.ROW_STALLED
    assert not (np.delete(st, victim) & _cabi.ROW_STALLED).any()
    want_ids, want_mask = H.oracle_batch("kmer6", flat, offs, padding="max_length", max_length=stride, truncation=True,
                                         add_special=False)
    got_ids, got_mask = ids.cpu().numpy(), mask.cpu().numpy()
    others = [r for r in range(rows) if r != victim]
    assert np.array_equal(got_ids[others], want_ids[others]) and np.array_equal(got_mask[others], want_mask[others])
    # the same call without the test option: every row exact, no status
    status.zero_()
    _cabi.check(L.dnatok_set_option(b"kmer_force_segments", 1))
    try:
        _cabi.check(L.dnatok_encode(handle.ptr, p(d_b), p(d_o), B, total, ctypes.byref(fmt), p(ids), p(mask), p(lengths),
                                    None, p(status), p(scratch), need, None))
        torch.cuda.synchronize()
    finally:
        _cabi.check(L.dnatok_set_option(b"kmer_force_segments", 0))
    assert not status.any()
    assert np.array_equal(ids.cpu().numpy(), want_ids) and np.array_equal(mask.cpu().numpy(), want_mask)
    handle.close()


def test_dnatok_flags_match_reference_outputs(golden):
    """normalize_case, handle_invalid_chars and token_len of the DNATok facade against what the reference
    returned for the same constructor flags (its tests: tests/test_benchmark_correctness.py:146-200)."""
    from dnatok_b200.dna_tokenizer import DNATok

    class Embedder:
        def __init__(self, tokenizer):
            self.tokenizer = tokenizer

        def embed_tokens(self, ids):
            return ids

    flags = golden["dnatok_flags"]
    seqs = flags["seqs"]
    for case in flags["cases"]:
        helper = DNATok(Embedder(H.hf(case["tokenizer"])), padding_side=case["padding_side"],
                        normalize_case=case["normalize_case"], handle_invalid_chars=case["handle_invalid_chars"])
        helper.discover()
        helper.token_len = case["token_len"]
        ids = helper.encode_batch_to_ids(seqs).tolist()
        tag = (case["tokenizer"], case["padding_side"], case["normalize_case"], case["handle_invalid_chars"], case["token_len"])
        if case["tokenizer"] == "kmer6" and case["padding_side"] == "left":
            # ragged k-mer rows: the reference leaves a row's tokens in the middle of the row (see the test
            # above); the tokens per row and a consistent left padding are what is compared
            pad = helper.id_pad
            for mine, ref in zip(ids, case["ids"]):
                assert [t for t in mine if t != pad] == [t for t in ref if t != pad], tag
                assert len(mine) == len(ref), tag
        else:
            assert ids == case["ids"], tag


def test_bpe_padded_encode_without_lengths_or_status():
    """dnatok_encode for a padded BPE batch writes ids and mask from the merge kernel; the row-length and status arrays
    are optional there."""
    import ctypes
    from dnatok_b200 import _cabi
    L = _cabi.lib()
    handle = _cabi.Handle(H.spec("bpe4096"))
    flat, offs = synth.pack_rows(synth.config3(batch=50, length=700, seed=9))
    d_b, d_o = dev(flat, offs)
    B, total, width = 50, len(flat), 200
    need = L.dnatok_scratch_bytes(handle.ptr, B, total)
    scratch = torch.empty(need, dtype=torch.uint8, device="cuda")
    fmt = _cabi.Format(64, 64, 1, 0, width, width)
    p = lambda t: ctypes.c_void_p(t.data_ptr())
    outs = []
    for with_rows in (True, False):
        ids = torch.full((B, width), -7, dtype=torch.int64, device="cuda")
        mask = torch.full((B, width), -7, dtype=torch.int64, device="cuda")
        lengths = torch.zeros(B, dtype=torch.int32, device="cuda")
        status = torch.full((B,), 99, dtype=torch.int32, device="cuda")          # not zeroed by the caller
        _cabi.check(L.dnatok_encode(handle.ptr, p(d_b), p(d_o), B, total, ctypes.byref(fmt), p(ids), p(mask),
                                    p(lengths) if with_rows else None, None, p(status) if with_rows else None,
                                    p(scratch), need, None))
        torch.cuda.synchronize()
        outs.append((ids, mask))
        if with_rows:
            assert status.tolist() == [0] * B
            assert torch.equal(lengths.to(torch.int64), mask.sum(dim=1))
    assert torch.equal(outs[0][0], outs[1][0]) and torch.equal(outs[0][1], outs[1][1])
    o_ids, o_mask = H.oracle_batch("bpe4096", flat, offs, padding="max_length", max_length=width, truncation=True)
    assert np.array_equal(outs[0][0].cpu().numpy(), o_ids) and np.array_equal(outs[0][1].cpu().numpy(), o_mask)


@pytest.mark.parametrize("name", ["char", "byte", "kmer6"])
def test_status_words_need_no_zeroing_by_the_caller(name):
    """dnatok_encode leaves every row's status word defined whatever the array held before: 0 for rows that fit,
    DNATOK_ROW_CLIPPED for rows cut by a stride that no truncation asked for."""
    import ctypes
    from dnatok_b200 import _cabi
    L = _cabi.lib()
    handle = _cabi.Handle(H.spec(name))
    rows = ["ACGT" * 10, "ACGTTGCA" * 300, "AC", "", "ACGTNNACGT" * 150]
    flat, offs = H.pack_strs(rows)
    d_b, d_o = dev(flat, offs)
    B, total, width = len(rows), len(flat), 256
    ids = torch.zeros((B, width), dtype=torch.int64, device="cuda")
    mask = torch.zeros((B, width), dtype=torch.int64, device="cuda")
    lengths = torch.zeros(B, dtype=torch.int32, device="cuda")
    status = torch.full((B,), 0x55, dtype=torch.int32, device="cuda")
    fmt = _cabi.Format(64, 64, 0, 0, 0, width)                  # no truncation asked for: the stride clips
    p = lambda t: ctypes.c_void_p(t.data_ptr())
    _cabi.check(L.dnatok_encode(handle.ptr, p(d_b), p(d_o), B, total, ctypes.byref(fmt), p(ids), p(mask), p(lengths), None,
                                p(status), None, 0, None))
    torch.cuda.synchronize()
    n_tok = [len(r) for r in H.oracle_rows(name, flat, offs)]
    assert status.tolist() == [_cabi.ROW_CLIPPED if n > width else 0 for n in n_tok]
    assert lengths.tolist() == [min(n, width) for n in n_tok]


def test_scan_lengths_at_trip_boundaries():
    """dnatok_scan_lengths (row lengths -> ragged output offsets) around its 4,096-row trips, on a 16-byte aligned array
    and on one that is not."""
    import ctypes
    from dnatok_b200 import _cabi
    L = _cabi.lib()
    for n in (1, 3, 4, 5, 1023, 1024, 4095, 4096, 4097, 8192, 100003):
        a = torch.randint(0, 5000, (n,), dtype=torch.int32, device="cuda")
        out = torch.empty(n + 1, dtype=torch.int64, device="cuda")
        for src in (a, torch.cat([torch.zeros(1, dtype=torch.int32, device="cuda"), a])[1:]):
            _cabi.check(L.dnatok_scan_lengths(ctypes.c_void_p(src.data_ptr()), n, ctypes.c_void_p(out.data_ptr()), None))
            torch.cuda.synchronize()
            want = torch.cat([torch.zeros(1, dtype=torch.int64, device="cuda"), torch.cumsum(src.to(torch.int64), 0)])
            assert torch.equal(out, want), n


def test_row_length_hint_flags_rows_outside_it():
    """A wrong dnatok_set_row_bytes_hint must not lose rows silently: they get a status bit."""
    import ctypes
    from dnatok_b200 import _cabi
    L = _cabi.lib()
    handle = _cabi.Handle(H.spec("bpe4096"))
    flat, offs = H.pack_strs(["ACGT" * 10, "ACGTTGCA" * 400, "AC"])        # the second row belongs to another length class
    d_b, d_o = dev(flat, offs)
    B, total = 3, len(flat)
    need = L.dnatok_scratch_bytes(handle.ptr, B, total)
    scratch = torch.empty(need, dtype=torch.uint8, device="cuda")
    ids = torch.zeros((B, 64), dtype=torch.int64, device="cuda")
    lengths = torch.zeros(B, dtype=torch.int32, device="cuda")
    status = torch.zeros(B, dtype=torch.int32, device="cuda")
    fmt = _cabi.Format(64, 0, 1, 0, 64, 64)
    p = lambda t: ctypes.c_void_p(t.data_ptr())
    _cabi.check(L.dnatok_set_row_bytes_hint(handle.ptr, 1, 256))
    _cabi.check(L.dnatok_encode(handle.ptr, p(d_b), p(d_o), B, total, ctypes.byref(fmt), p(ids), None, p(lengths), None,
                                p(status), p(scratch), need, None))
    torch.cuda.synchronize()
    assert status.tolist() == [0, _cabi.ROW_OUTSIDE_HINT, 0]
    assert lengths.tolist()[1] == 2                      # only the special tokens
    _cabi.check(L.dnatok_set_row_bytes_hint(handle.ptr, 0, 0))
    _cabi.check(L.dnatok_encode(handle.ptr, p(d_b), p(d_o), B, total, ctypes.byref(fmt), p(ids), None, p(lengths), None,
                                p(status), p(scratch), need, None))
    torch.cuda.synchronize()
    assert status.tolist() == [0, 0, 0]
    want, _ = H.oracle_batch("bpe4096", flat, offs, padding="max_length", max_length=64, truncation=True)
    assert np.array_equal(ids.cpu().numpy(), want)
    assert L.dnatok_set_row_bytes_hint(handle.ptr, 5, 2) == -1
    handle.close()


def test_cli_validate_info_encode(capsys):
    """The command line front end: validate exits 0 only when every window matches Hugging Face."""
    import json
    import os
    from dnatok_b200 import cli
    fixture = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "bpe4096.tokenizer.json.gz")
    for spec, path in (("char", "ascii_lut"), ("kmer6", "kmer_lut"), ("byte", "ascii_lut"), (fixture, "gpu_bpe")):
        assert cli.main(["validate", "--tokenizer", spec, "--n", "40", "--window", "515", "--json"]) == 0
        out = json.loads(capsys.readouterr().out.strip().splitlines()[-1])
        assert out["n_match"] == 40 and out["n_mismatch"] == 0 and out["selected_path"] == path
    assert cli.main(["info", "--tokenizer", "kmer6", "--json"]) == 0
    info = json.loads(capsys.readouterr().out.strip().splitlines()[-1])
    assert info["kmer_k"] == 6 and info["vocab_size"] == 4106 and info["id_pad"] == 0
    assert cli.main(["encode", "--tokenizer", "char", "--seq", "ACGTN", "--json"]) == 0
    enc = json.loads(capsys.readouterr().out.strip().splitlines()[-1])
    assert enc["token_ids"] == [5, 6, 7, 8, 9] and enc["n_tokens"] == 5
    assert cli.main(["bench", "--tokenizer", "char", "--n", "64", "--window", "256", "--json"]) == 0
    b = json.loads(capsys.readouterr().out.strip().splitlines()[-1])
    assert b["total_bp"] == 64 * 256 and b["dnatok_mbp_per_s"] > 0
    assert cli.main(["info", "--tokenizer", "/nonexistent/dir"]) == 2
    # the eight read-length scenarios at a reduced read count, ids of a sample checked against Hugging Face
    for spec in ("kmer6", fixture):
        assert cli.main(["scenarios", "--tokenizer", spec, "--reads", "24", "--check", "12", "--chunk", "8", "--json"]) == 0
        sc = json.loads(capsys.readouterr().out.strip().splitlines()[-1])["scenarios"]
        assert len(sc) == 8 and all(v["mismatches"] == 0 and v["dnatok_mbp_per_s"] > 0 for v in sc.values())
        assert sc["nanopore_long"]["length_max"] <= 100000 and sc["illumina_short"]["length_max"] <= 300


@pytest.mark.parametrize("name", ["char", "byte"])
@pytest.mark.parametrize("dim,dtype", [(128, "float16"), (1024, "bfloat16"), (20, "float32"), (8, "float16")])
def test_fused_embedding_gather(toks, name, dim, dtype):
    """dnatok_embed: out == weight[input_ids] bit for bit (rows are copied), ids never materialised."""
    tok = toks[name]
    rng = np.random.default_rng(dim)
    B = 37
    lens = rng.integers(0, 600, size=B)
    a = synth.config4(batch=B, length=600, seed=3) if name == "byte" else synth.config1(batch=B, length=600, seed=3)
    offs = np.concatenate([[0], np.cumsum(lens)]).astype(np.int64)
    flat = np.concatenate([a[i, :lens[i]] for i in range(B)])
    d_b, d_o = dev(flat, offs)
    vocab = tok.vocab_size if name == "char" else 512
    weight = torch.randn((vocab, dim), device="cuda").to(getattr(torch, dtype)).contiguous()
    for kw in (dict(padding="longest"), dict(padding="max_length", max_length=77, truncation=True)):
        for side in ("right", "left"):
            tok.padding_side = side
            try:
                got = tok.embed_device(d_b, d_o, weight, host_offsets=offs, **kw)
                ref = tok.encode_device(d_b, d_o, host_offsets=offs, **kw)
            finally:
                tok.padding_side = "right"
            torch.cuda.synchronize()
            o_ids, _ = H.oracle_batch(name, flat, offs, pad_left=(side == "left"), **kw)
            assert np.array_equal(ref["input_ids"].cpu().numpy(), o_ids)
            want = weight[torch.from_numpy(o_ids).cuda()]
            assert torch.equal(got["embeddings"], want)
            assert torch.equal(got["lengths"], ref["lengths"])
    # a weight matrix that lacks a row for some id the tokenizer can produce is refused, not patched over
    from dnatok_b200 import _cabi
    top = int(max(max(tok.spec.lut256), tok.spec.specials.cls_id, tok.spec.specials.sep_id))
    short = weight[:top].contiguous()
    with pytest.raises(_cabi.DnatokError, match="weight matrix"):
        tok.embed_device(d_b, d_o, short, host_offsets=offs, padding="longest")
