"""The allocation-free BPE entry point (dnatok_encode_bpe_builtin_scratch) against dnatok_encode.

Some hosts cannot call cudaMalloc around a tokenizer call (all device memory already belongs to
their own pool, or an allocation's implicit synchronisation is not acceptable in their loop), so
the library also offers BPE encoding whose working memory is a fixed array inside the library.
This file checks, through the C ABI, that the variant returns exactly what the ordinary entry
point returns, on two calls in a row (the array is shared and keeps the previous call's
contents), and that an oversized batch is refused on the host.  It is collected last so a run
that stops at the first failure has already been through every other test.
"""
import ctypes

import numpy as np
import pytest

from dnatok_b200 import _cabi, synth

import helpers as H

pytestmark = pytest.mark.gpu

torch = pytest.importorskip("torch")


def _ptr(t):
    return ctypes.c_void_p(t.data_ptr()) if t is not None else None


def _encode(L, handle, entry, d_bytes, d_off, fmt, stride, scratch):
    B, total = d_off.shape[0] - 1, int(d_bytes.shape[0])
    ids = torch.full((B, stride), -7, dtype=torch.int64, device="cuda")
    mask = torch.full((B, stride), -7, dtype=torch.int64, device="cuda")
    lengths = torch.zeros(B, dtype=torch.int32, device="cuda")
    status = torch.zeros(B, dtype=torch.int32, device="cuda")
    stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    common = (handle.ptr, _ptr(d_bytes), _ptr(d_off), B, total, ctypes.byref(fmt), _ptr(ids), _ptr(mask),
              _ptr(lengths), None, _ptr(status))
    if entry == "caller_scratch":
        rc = L.dnatok_encode(*common, _ptr(scratch), int(scratch.numel()), stream)
    else:
        rc = L.dnatok_encode_bpe_builtin_scratch(*common, stream)
    _cabi.check(rc)
    torch.cuda.synchronize()
    assert not status.any()
    return ids.cpu().numpy(), mask.cpu().numpy(), lengths.cpu().numpy()


def test_builtin_scratch_matches_caller_scratch_twice():
    assert torch.cuda.is_available()
    L = _cabi.lib()
    handle = _cabi.Handle(H.spec("bpe4096"))
    fmt = _cabi.Format(64, 64, 1, 0, 0, 256)
    batches = [synth.pack_rows(synth.config3(batch=200, length=900, seed=21)),
               synth.config5(n_reads=96, seed=5)]            # second call: other sizes, ragged lengths
    batches[1] = (batches[1][0], batches[1][1])
    fmts = [fmt, _cabi.Format(64, 64, 1, 0, 0, 2600)]
    for (flat, offs), f in zip(batches, fmts):
        if np.diff(offs).max() > 8000:                       # keep the second batch inside the word limit comfortably
            keep = np.flatnonzero(np.diff(offs) <= 8000)
            from dnatok_b200.shard import take_rows
            flat, offs = take_rows(flat, offs, keep)
        d_bytes, d_off = torch.from_numpy(np.ascontiguousarray(flat)).cuda(), torch.from_numpy(offs).cuda()
        need = L.dnatok_scratch_bytes(handle.ptr, len(offs) - 1, len(flat))
        assert 0 < need <= _cabi.BUILTIN_SCRATCH_BYTES
        scratch = torch.empty(need, dtype=torch.uint8, device="cuda")
        # the ordinary entry point first: it also places the handle's tables on the device
        want = _encode(L, handle, "caller_scratch", d_bytes, d_off, f, int(f.out_stride), scratch)
        got = _encode(L, handle, "builtin", d_bytes, d_off, f, int(f.out_stride), None)
        for w, g in zip(want, got):
            assert np.array_equal(w, g)                      # integer ids: bit-exact, as everywhere else
        o_ids, o_mask = H.oracle_batch("bpe4096", flat, offs, padding="max_length", max_length=int(f.out_stride))
        assert np.array_equal(got[0], o_ids) and np.array_equal(got[1], o_mask)
    handle.close()


def test_builtin_scratch_ragged_output():
    """Ragged output (no padding: flat ids plus row offsets) through the variant, against the ordinary entry
    point and the CPU checker."""
    L = _cabi.lib()
    handle = _cabi.Handle(H.spec("bpe4096"))
    flat, offs = synth.config5(n_reads=64, seed=9)
    keep = np.flatnonzero(np.diff(offs) <= 6000)
    from dnatok_b200.shard import take_rows
    flat, offs = take_rows(flat, offs, keep)
    B, total = len(offs) - 1, len(flat)
    d_bytes, d_off = torch.from_numpy(np.ascontiguousarray(flat)).cuda(), torch.from_numpy(offs).cuda()
    need = L.dnatok_scratch_bytes(handle.ptr, B, total)
    assert 0 < need <= _cabi.BUILTIN_SCRATCH_BYTES
    scratch = torch.empty(need, dtype=torch.uint8, device="cuda")
    fmt = _cabi.Format(64, 0, 1, 0, 0, 0)                    # out_stride 0: ragged
    outs = []
    for entry in ("caller_scratch", "builtin", "builtin"):
        ids = torch.full((total + 2 * B,), -7, dtype=torch.int64, device="cuda")
        out_off = torch.zeros(B + 1, dtype=torch.int64, device="cuda")
        lengths = torch.zeros(B, dtype=torch.int32, device="cuda")
        status = torch.zeros(B, dtype=torch.int32, device="cuda")
        stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
        common = (handle.ptr, _ptr(d_bytes), _ptr(d_off), B, total, ctypes.byref(fmt), _ptr(ids), None, _ptr(lengths),
                  _ptr(out_off), _ptr(status))
        if entry == "caller_scratch":
            _cabi.check(L.dnatok_encode(*common, _ptr(scratch), int(scratch.numel()), stream))
        else:
            _cabi.check(L.dnatok_encode_bpe_builtin_scratch(*common, stream))
        torch.cuda.synchronize()
        assert not status.any()
        oo = out_off.cpu().numpy()
        outs.append((ids.cpu().numpy()[:oo[-1]], oo, lengths.cpu().numpy()))
    for got in outs[1:]:
        for w, g in zip(outs[0], got):
            assert np.array_equal(w, g)
    sp = H.spec("bpe4096").specials
    want = H.oracle_rows("bpe4096", flat, offs)
    ids, oo, _ = outs[1]
    for i in range(B):
        assert ids[oo[i]:oo[i + 1]].tolist() == [sp.cls_id] + want[i].tolist() + [sp.sep_id]
    handle.close()


def test_builtin_scratch_refuses_oversized_batch_and_cold_handle():
    L = _cabi.lib()
    handle = _cabi.Handle(H.spec("bpe4096"))
    d_bytes = torch.zeros(16, dtype=torch.uint8, device="cuda")
    d_off = torch.tensor([0, 16], dtype=torch.int64, device="cuda")
    fmt = _cabi.Format(64, 0, 1, 0, 0, 32)
    ids = torch.zeros((1, 32), dtype=torch.int64, device="cuda")
    lengths = torch.zeros(1, dtype=torch.int32, device="cuda")
    # sizes are host-side arguments: claim a batch far beyond the array; nothing may be launched
    rc = L.dnatok_encode_bpe_builtin_scratch(handle.ptr, _ptr(d_bytes), _ptr(d_off), 1, 64 << 20, ctypes.byref(fmt),
                                             _ptr(ids), None, _ptr(lengths), None, None, None)
    assert rc == -5 and b"built-in array holds" in L.dnatok_last_error()
    # a handle that has never run on this device has no tables there
    rc = L.dnatok_encode_bpe_builtin_scratch(handle.ptr, _ptr(d_bytes), _ptr(d_off), 1, 16, ctypes.byref(fmt),
                                             _ptr(ids), None, _ptr(lengths), None, None, None)
    assert rc == -1 and b"tables are not on device" in L.dnatok_last_error()
    char = _cabi.Handle(H.spec("char"))
    rc = L.dnatok_encode_bpe_builtin_scratch(char.ptr, _ptr(d_bytes), _ptr(d_off), 1, 16, ctypes.byref(fmt),
                                             _ptr(ids), None, _ptr(lengths), None, None, None)
    assert rc == -1
    torch.cuda.synchronize()
    handle.close()
    char.close()
