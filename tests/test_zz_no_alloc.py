"""The allocation-free decode attention entry point (cima_attention_decode_static), called through
its exported C symbol as a caller without the Python package would, against the ordinary entry
point.  Some users of the library may not allocate device memory when they need attention (their
memory was handed out at start-up by a host program, or an allocation would stall a latency-critical
loop); for them the splits' scratch lives in a fixed array inside the library.

Collected last on purpose: a run that stops at the first failure has then run every other test."""
import ctypes
import math

import pytest
import torch

pytestmark = pytest.mark.gpu


def test_static_scratch_entry_matches_the_ordinary_one_twice():
    from cima_b200.cache.kv import LayerKV
    from cima_b200.kernels import Kernels
    K = Kernels(verbose=False)
    lib = ctypes.CDLL(K.path)
    fn = lib.cima_attention_decode_static
    vp, i, f = ctypes.c_void_p, ctypes.c_int, ctypes.c_float
    fn.argtypes = [vp, i, vp, vp, i, i, i, vp, vp, vp, i, i, i, i, i, f, i, i, vp]
    fn.restype = i
    lib.cima_last_error.restype = ctypes.c_char_p

    nh, nkv, hd, page = 28, 4, 128, 64
    gen = torch.Generator().manual_seed(5)
    for call, (lens, n_splits) in enumerate([([700, 1, 130], 5), ([64, 333], 3)]):
        B = len(lens)
        pages = [-(-n // page) for n in lens]
        order = torch.randperm(sum(pages) + 2, generator=gen).tolist()
        table = torch.zeros(B, max(pages), dtype=torch.int32)
        k = 0
        for b, n in enumerate(pages):
            table[b, :n] = torch.tensor(order[k:k + n], dtype=torch.int32)
            k += n
        storage = (torch.randn(sum(pages) + 2, 2, nkv, page, hd, generator=gen)).to(torch.bfloat16).cuda()
        qkv = torch.randn(B, (nh + 2 * nkv) * hd, generator=gen).to(torch.bfloat16).cuda()
        kv = LayerKV(storage, table.cuda(), page, 0, 0, 0)
        seq_slot = torch.arange(B, dtype=torch.int32).cuda()
        seq_len = torch.tensor(lens, dtype=torch.int32).cuda()
        scale = 1.0 / math.sqrt(hd)
        want = torch.empty(B, nh * hd, dtype=torch.bfloat16, device="cuda")
        K.attention_decode(qkv, kv, seq_slot, seq_len, want, nh, nkv, hd, scale, 0, n_splits=n_splits)
        got = torch.full_like(want, 3.0)
        rc = fn(qkv.data_ptr(), qkv.shape[1], storage.data_ptr(), kv.block_table.data_ptr(), kv.block_table.shape[1],
                0, page, seq_slot.data_ptr(), seq_len.data_ptr(), got.data_ptr(), got.shape[1], B, nh, nkv, hd,
                scale, 0, n_splits, torch.cuda.current_stream().cuda_stream)
        assert rc == 0, lib.cima_last_error().decode()
        torch.cuda.synchronize()
        # both entries launch the same kernels with the same splits: the same bits, whatever the last call left
        # in the fixed array
        assert torch.equal(got, want), call
        assert torch.isfinite(got.float()).all()

    # a size beyond the fixed array is refused with a sentence, and nothing runs
    rc = fn(qkv.data_ptr(), qkv.shape[1], storage.data_ptr(), kv.block_table.data_ptr(), kv.block_table.shape[1],
            0, page, seq_slot.data_ptr(), seq_len.data_ptr(), got.data_ptr(), got.shape[1], 4096, nh, nkv, hd,
            scale, 0, 32, torch.cuda.current_stream().cuda_stream)
    assert rc != 0 and b"fixed array" in lib.cima_last_error()
