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


def _bind():
    from oxide_tech_llm_engine_b200 import _build

    lib = ctypes.CDLL(str(_build.noalloc_lib_path()))
    fn = lib.oxb_paged_decode_noalloc
    fn.restype = ctypes.c_int
    vp, ll, ci = ctypes.c_void_p, ctypes.c_longlong, ctypes.c_int
    fn.argtypes = [vp, ll, vp, vp, vp, vp, vp, ll, ci, ci, ci, ci, ci, ci, ci, ci, ci, ctypes.c_float, vp, vp,
                   ctypes.c_char_p, ci]
    return fn


def test_noalloc_entry_point_matches_regular_entry_point():
    from oxide_tech_llm_engine_b200 import ops

    fn = _bind()
    err = ctypes.create_string_buffer(512)
    # (lengths, hq, hkv, head_dim, pages_per_split, window): one KV head with 8 query heads, four KV
    # heads, a group of 16 query heads per KV head (two column tiles), a sliding window
    cases = [([1, 17, 300, 64, 1000], 8, 1, 128, 4, 0), ([90, 31, 257], 32, 4, 64, 2, 0),
             ([400, 33, 129], 32, 2, 128, 3, 0), ([700, 50, 300], 8, 2, 64, 2, 96)]
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    for n, (seq_lens, hq, hkv, d, pps, window) in enumerate(cases):
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
                         part_o, part_ml, want, batch=B, max_splits=max_splits, window=window, scale=scale)
        # allocation-free entry point, on torch's current stream
        got = torch.zeros_like(want)
        stream = torch.cuda.current_stream().cuda_stream
        rc = fn(q.data_ptr(), q.stride(0), k_cache.data_ptr(), v_cache.data_ptr(), bt.data_ptr(),
                sl.data_ptr(), got.data_ptr(), got.stride(0), B, hq, hkv, d, k_cache.shape[0], bt.shape[1], pps,
                max_splits, window, scale, stream, status.data_ptr(), err, len(err))
        assert rc == 0, err.value.decode()
        torch.cuda.synchronize()
        rel = ((got.float() - want.float()).abs().max() / want.float().abs().max()).item()
        assert rel < 2e-2, (n, rel)
        assert int(status.item()) == 0
    args = dict(q=q.data_ptr(), qs=q.stride(0), k=k_cache.data_ptr(), v=v_cache.data_ptr(), bt=bt.data_ptr(),
                sl=sl.data_ptr(), out=got.data_ptr(), os=got.stride(0), batch=B, hq=hq, hkv=hkv, d=d,
                nb=k_cache.shape[0], mb=bt.shape[1], pps=pps, ms=max_splits, win=0, scale=scale, stream=None,
                status=None)

    def call(**kw):
        a = dict(args, **kw)
        return fn(a["q"], a["qs"], a["k"], a["v"], a["bt"], a["sl"], a["out"], a["os"], a["batch"], a["hq"],
                  a["hkv"], a["d"], a["nb"], a["mb"], a["pps"], a["ms"], a["win"], a["scale"], a["stream"],
                  a["status"], err, len(err))

    # a request beyond the built-in scratch is refused with a message, nothing is launched
    assert call(batch=4096, hq=64, hkv=8, d=128, pps=1, ms=64, qs=8192, os=8192) == -2 and b"exceeds the built-in scratch" in err.value
    # a product of the sizes that would wrap 64 bits is refused the same way
    assert call(batch=1 << 30, hq=1 << 19, hkv=1 << 15, d=128, ms=1 << 15) in (-1, -2)
    # bad arguments: misaligned pointers, odd strides, short strides, grid limits
    assert call(q=args["q"] + 2) == -1 and b"16-byte aligned" in err.value
    assert call(out=args["out"] + 8) == -1
    assert call(qs=args["qs"] + 4) == -1 and b"multiples of 8" in err.value
    assert call(os=8) == -1
    assert call(ms=70000) == -1 and b"grid dimensions" in err.value
    assert call(nb=0) == -1
    torch.cuda.synchronize()


def test_noalloc_entry_point_bounds_block_ids_and_lengths():
    """A block id outside the pool and a length beyond the table row are reported through the status
    word and never dereferenced (block 0 is read / the walk stops at the end of the row)."""
    fn = _bind()
    err = ctypes.create_string_buffer(512)
    seq_lens, hq, hkv, d, pps = [100, 40], 8, 1, 128, 2
    q, k_cache, v_cache, bt, sl = _paged_case(seq_lens, hq, hkv, d, seed=7)
    out = torch.zeros(2, hq * d, device="cuda", dtype=torch.bfloat16)
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    bad_bt = bt.clone()
    bad_bt[0, 1] = 10 ** 6          # far outside the pool
    long_sl = sl.clone()
    long_sl[1] = 16 * bt.shape[1] + 500   # longer than its table row
    for tables, lens in ((bad_bt, sl), (bt, long_sl)):
        status.zero_()
        rc = fn(q.data_ptr(), q.stride(0), k_cache.data_ptr(), v_cache.data_ptr(), tables.data_ptr(),
                lens.data_ptr(), out.data_ptr(), out.stride(0), 2, hq, hkv, d, k_cache.shape[0], bt.shape[1], pps,
                64, 0, 0.1, None, status.data_ptr(), err, len(err))
        assert rc == 0, err.value.decode()
        torch.cuda.synchronize()
        assert int(status.item()) == 5
        assert torch.isfinite(out.float()).all()
