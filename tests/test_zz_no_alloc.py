"""The allocation-free C entry point of the paged decode attention (liboxb_noalloc.so).

Some embedders of the decode kernel cannot allocate device memory at call time (their memory
budget is frozen after start-up, or another runtime owns the device heap), so the library keeps
the split-KV scratch in a built-in device array. This test calls the exported C symbol through
ctypes twice in a row, with different inputs, and compares each result with the regular entry
point, whose scratch the caller allocates. The file sorts last so that it runs after every other
test; it also passes when run alone.
"""
import ctypes
import math

import pytest
import torch

pytestmark = pytest.mark.gpu


def _paged_case(seq_lens, hq, hkv, d, seed):
    g = torch.Generator(device="cpu").manual_seed(seed)
    n_blocks = sum((s + 15) // 16 for s in seq_lens) + 2
    k_cache = torch.randn(n_blocks, hkv, 16, d, generator=g).to("cuda", torch.bfloat16)
    v_cache = torch.randn(n_blocks, hkv, 16, d, generator=g).to("cuda", torch.bfloat16)
    perm = iter(torch.randperm(n_blocks, generator=g).tolist())
    max_blocks = max((s + 15) // 16 for s in seq_lens)
    bt = torch.zeros(len(seq_lens), max_blocks, dtype=torch.int32)
    for i, s in enumerate(seq_lens):
        for j in range((s + 15) // 16):
            bt[i, j] = next(perm)
    q = torch.randn(len(seq_lens), hq, d, generator=g).to("cuda", torch.bfloat16)
    return q, k_cache, v_cache, bt.cuda(), torch.tensor(seq_lens, dtype=torch.int32, device="cuda")


def test_noalloc_entry_point_matches_regular_entry_point():
    from oxide_tech_llm_engine_b200 import _build, ops

    lib = ctypes.CDLL(str(_build.noalloc_lib_path()))
    fn = lib.oxb_paged_decode_noalloc
    fn.restype = ctypes.c_int
    vp, ll, ci = ctypes.c_void_p, ctypes.c_longlong, ctypes.c_int
    fn.argtypes = [vp, ll, vp, vp, vp, vp, vp, ll, ci, ci, ci, ci, ci, ci, ci, ci, ctypes.c_float, vp,
                   ctypes.c_char_p, ci]
    err = ctypes.create_string_buffer(512)
    cases = [([1, 17, 300, 64, 1000], 8, 1, 128, 4), ([90, 31, 257], 32, 4, 64, 2)]
    for n, (seq_lens, hq, hkv, d, pps) in enumerate(cases):
        q, k_cache, v_cache, bt, sl = _paged_case(seq_lens, hq, hkv, d, seed=100 + n)
        B = len(seq_lens)
        max_pages = max((s + 15) // 16 for s in seq_lens)
        max_splits = (max_pages + pps - 1) // pps
        scale = 1.0 / math.sqrt(d)
        # regular entry point: the caller provides the scratch
        part_o = torch.empty(B * hq * max_splits * d, device="cuda", dtype=torch.float32)
        part_ml = torch.empty(B * hq * max_splits * 2, device="cuda", dtype=torch.float32)
        want = torch.empty(B, hq * d, device="cuda", dtype=torch.bfloat16)
        ops.paged_decode(q, k_cache, v_cache, bt, sl, torch.tensor([pps], dtype=torch.int32, device="cuda"),
                         part_o, part_ml, want, batch=B, max_splits=max_splits, scale=scale)
        # allocation-free entry point, on torch's current stream
        got = torch.zeros_like(want)
        stream = torch.cuda.current_stream().cuda_stream
        rc = fn(q.data_ptr(), q.stride(0), k_cache.data_ptr(), v_cache.data_ptr(), bt.data_ptr(),
                sl.data_ptr(), got.data_ptr(), got.stride(0), B, hq, hkv, d, bt.shape[1], pps, max_splits, 0,
                scale, stream, err, len(err))
        assert rc == 0, err.value.decode()
        torch.cuda.synchronize()
        rel = ((got.float() - want.float()).abs().max() / want.float().abs().max()).item()
        assert rel < 2e-2, (n, rel)
    # a request beyond the built-in scratch is refused with a message, nothing is launched
    rc = fn(q.data_ptr(), q.stride(0), k_cache.data_ptr(), v_cache.data_ptr(), bt.data_ptr(), sl.data_ptr(),
            got.data_ptr(), got.stride(0), 4096, 64, 8, 128, bt.shape[1], 1, 64, 0, 0.1, None, err, len(err))
    assert rc == -2 and b"exceeds the built-in scratch" in err.value
