"""Numerics of every sm_100a kernel against plain PyTorch fp32 references of the same op."""
import math

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu

DEV = "cuda"


@pytest.fixture(scope="module")
def ops():
    from oxide_tech_llm_engine_b200 import ops as o

    return o


def _rel_err(got, ref):
    got, ref = got.float(), ref.float()
    return ((got - ref).abs().max() / ref.abs().max().clamp_min(1e-6)).item()


def _cos(got, ref):
    return torch.nn.functional.cosine_similarity(got.float().flatten(), ref.float().flatten(), dim=0).item()


# ------------------------------------------------------------------------------------------ GEMM
@pytest.mark.parametrize("m,n,k,bn", [
    (128, 128, 64, 128), (128, 128, 256, 128), (256, 512, 1024, 128), (100, 200, 136, 128),
    (1, 1280, 2048, 64), (17, 256, 512, 64), (300, 1024, 512, 256), (129, 4096, 4096, 128),
    (64, 96, 64, 128), (1024, 4096, 512, 128), (2048, 2048, 192, 64), (640, 8192, 256, 256),
])
def test_gemm_store_bf16(ops, m, n, k, bn):
    torch.manual_seed(0)
    a = torch.randn(m, k, device=DEV, dtype=torch.bfloat16)
    w = torch.randn(n, k, device=DEV, dtype=torch.bfloat16)
    out = ops.gemm(a, w, bn=bn)
    torch.cuda.synchronize()
    ops.check_status()
    ref = a.float() @ w.float().T
    assert _rel_err(out, ref) < 1.5e-2, (m, n, k, bn, _rel_err(out, ref))
    assert _cos(out, ref) > 0.9999


def test_gemm_bias_and_f32(ops):
    torch.manual_seed(1)
    m, n, k = 70, 384, 320
    a = torch.randn(m, k, device=DEV, dtype=torch.bfloat16)
    w = torch.randn(n, k, device=DEV, dtype=torch.bfloat16)
    bias = torch.randn(n, device=DEV, dtype=torch.bfloat16)
    ref = a.float() @ w.float().T + bias.float()
    out = ops.gemm(a, w, bias=bias, epi=ops.EPI_STORE_F32)
    torch.cuda.synchronize()
    assert out.dtype == torch.float32
    assert _rel_err(out, ref) < 2e-3
    out2 = ops.gemm(a, w, bias=bias)
    assert _rel_err(out2, ref) < 1.5e-2


@pytest.mark.parametrize("m,n,k,splits,bn", [(256, 1280, 8192, 7, 128), (32, 512, 4096, 16, 64),
                                             (130, 256, 1024, 4, 128), (1500, 2048, 1024, 3, 128)])
def test_gemm_splitk_red(ops, m, n, k, splits, bn):
    torch.manual_seed(2)
    a = torch.randn(m, k, device=DEV, dtype=torch.bfloat16)
    w = torch.randn(n, k, device=DEV, dtype=torch.bfloat16)
    acc = torch.zeros(m, n, device=DEV, dtype=torch.float32)
    ops.gemm(a, w, epi=ops.EPI_RED_F32, dst_ptrs=[acc.data_ptr()], splits=splits, bn=bn)
    torch.cuda.synchronize()
    ops.check_status()
    ref = a.float() @ w.float().T
    assert _rel_err(acc, ref) < 2e-3
    out = torch.empty(m, n, device=DEV, dtype=torch.bfloat16)
    ops.cast_acc_bf16(acc, out, m, n)
    torch.cuda.synchronize()
    assert _rel_err(out, ref) < 1.5e-2
    assert acc.abs().max().item() == 0.0  # the accumulator is re-armed


def test_gemm_slab_reduce_scatter_emulated(ops):
    """Four owners emulated on one GPU: each gets its rows of the partial product in its slab,
    then finalize_norm sums the slabs of all sources."""
    torch.manual_seed(13)
    tp, rpo, n, k = 4, 64, 512, 256
    m = tp * rpo
    a = torch.randn(m, k, device=DEV, dtype=torch.bfloat16)
    w = torch.randn(n, k, device=DEV, dtype=torch.bfloat16)
    slabs = [torch.zeros(tp, rpo, n, device=DEV, dtype=torch.bfloat16) for _ in range(tp)]
    my = 2
    ops.gemm(a, w, epi=ops.EPI_SLAB_BF16, dst_ptrs=[s.data_ptr() for s in slabs], rows_per_owner=rpo,
             my_rank=my, dst_ld=n, bn=128)
    torch.cuda.synchronize()
    ops.check_status()
    ref = a.float() @ w.float().T
    for o in range(tp):
        assert _rel_err(slabs[o][my], ref[o * rpo:(o + 1) * rpo]) < 1.5e-2
        assert slabs[o][my - 1].abs().max().item() == 0
    # owner 1 sums its slabs (pretend every source wrote the same partial)
    own = slabs[1]
    for src in range(tp):
        own[src] = own[my]
    res = torch.randn(rpo, n, device=DEV, dtype=torch.bfloat16)
    wn = torch.rand(n, device=DEV, dtype=torch.bfloat16) + 0.5
    out = torch.empty(rpo, n, device=DEV, dtype=torch.bfloat16)
    res_out = torch.empty_like(res)
    ops.finalize_norm(rows=rpo, n=n, rs_slab=own, n_slabs=tp, slab_stride=rpo * n, residual_in=res,
                      residual_out=res_out, norm_w=wn, eps=1e-5, out_ptrs=[out.data_ptr()])
    torch.cuda.synchronize()
    h = own[my].float() * tp + res.float()
    assert _rel_err(res_out, h) < 1.5e-2
    assert _rel_err(out, _rms(h, wn, 1e-5)) < 2e-2


def test_gemm_swiglu_epilogue(ops):
    torch.manual_seed(3)
    m, i, k, bn = 2100, 1536, 768, 128  # more work items than SMs: exercises the TMEM double buffer
    a = torch.randn(m, k, device=DEV, dtype=torch.bfloat16) * 0.5
    wg = torch.randn(i, k, device=DEV, dtype=torch.bfloat16) * 0.05
    wu = torch.randn(i, k, device=DEV, dtype=torch.bfloat16) * 0.05
    # gate and up rows interleaved in units of 32: [gate 0..32) | up 0..32) | gate 32..64) | ...
    h = 32
    w = torch.stack([wg.view(i // h, h, k), wu.view(i // h, h, k)], 1).reshape(2 * i, k).contiguous()
    out = ops.gemm(a, w, epi=ops.EPI_SWIGLU_BF16, bn=bn)
    torch.cuda.synchronize()
    g = a.float() @ wg.float().T
    u = a.float() @ wu.float().T
    ref = torch.nn.functional.silu(g) * u
    assert out.shape == (m, i)
    assert _rel_err(out, ref) < 2e-2


@pytest.mark.parametrize("m,n,k,bn,splits,tiled", [
    (256, 1024, 1024, 256, 1, False), (256, 768, 2048, 128, 1, True), (200, 512, 512, 64, 1, False),
    (256, 1024, 2048, 256, 4, False), (130, 640, 4096, 128, 5, False), (256, 1280, 8192, 128, 12, True), (256, 1280, 8192, 64, 7, True),
    (255, 1000, 1024, 256, 3, False), (600, 512, 1024, 256, 2, False), (64, 1024, 4096, 256, 6, False),
])
def test_gemm_full_m_tiles_and_in_kernel_splitk(ops, m, n, k, bn, splits, tiled):
    """mt = 2 (both 128-row halves with the CTA that owns the weight tile) and split-K combined
    inside the kernel through bf16 partial slabs, against fp32 matmul; run twice so that the
    tickets are seen re-armed."""
    torch.manual_seed(21)
    a = torch.randn(m, k, device=DEV, dtype=torch.bfloat16)
    w = torch.randn(n, k, device=DEV, dtype=torch.bfloat16)
    bias = torch.randn(n, device=DEV, dtype=torch.bfloat16)
    ww = ops.tile_weight(w) if tiled else w
    ref = a.float() @ w.float().T + bias.float()
    mt = 2 if m > 128 else 1
    for _ in range(2):
        out = ops.gemm(a, ww, bias=bias, bn=bn, mt=mt, splits=splits)
        torch.cuda.synchronize()
        ops.check_status()
        assert _rel_err(out, ref) < 1.5e-2 and _cos(out, ref) > 0.9999, (m, n, k, bn, splits, _rel_err(out, ref))
    out32 = ops.gemm(a, ww, bias=bias, bn=bn, mt=mt, splits=splits, epi=ops.EPI_STORE_F32)
    torch.cuda.synchronize()
    ops.check_status()
    assert _rel_err(out32, ref) < (2e-3 if splits == 1 else 8e-3)
    assert int(ops.gemm_workspace(DEV)[1].abs().max().item()) == 0  # tickets re-armed


@pytest.mark.parametrize("m,i,k,bn,splits", [(256, 1792, 2048, 256, 5), (256, 512, 1024, 128, 1),
                                              (192, 3584, 1024, 256, 5), (96, 1024, 2048, 64, 4), (256, 3584, 8192, 256, 5)])
def test_gemm_swiglu_full_m_splitk(ops, m, i, k, bn, splits):
    torch.manual_seed(22)
    a = torch.randn(m, k, device=DEV, dtype=torch.bfloat16) * 0.5
    wg = torch.randn(i, k, device=DEV, dtype=torch.bfloat16) * 0.05
    wu = torch.randn(i, k, device=DEV, dtype=torch.bfloat16) * 0.05
    w = torch.stack([wg.view(i // 32, 32, k), wu.view(i // 32, 32, k)], 1).reshape(2 * i, k).contiguous()
    out = ops.gemm(a, w, epi=ops.EPI_SWIGLU_BF16, bn=bn, mt=2 if m > 128 else 1, splits=splits)
    torch.cuda.synchronize()
    ops.check_status()
    ref = torch.nn.functional.silu(a.float() @ wg.float().T) * (a.float() @ wu.float().T)
    assert out.shape == (m, i) and _rel_err(out, ref) < 2e-2


def test_gemm_rejects_splits_that_do_not_fit_one_wave(ops):
    a = torch.randn(256, 1024, device=DEV, dtype=torch.bfloat16)
    w = torch.randn(7168, 1024, device=DEV, dtype=torch.bfloat16)
    with pytest.raises(ValueError, match="one wave"):
        ops.gemm(a, w, epi=ops.EPI_SWIGLU_BF16, bn=256, mt=2, splits=6)   # 28 tiles x 6 > 148 SMs
    with pytest.raises(RuntimeError, match="K mismatch"):
        ops.gemm(a, w[:, :512].contiguous(), bn=128)


def test_gemm_slab_full_m_splitk_reduce_scatter_emulated(ops):
    """Row-parallel projection at decode size: 256 rows, 8 owners emulated on one GPU, split-K
    combined locally before ONE bf16 push per row."""
    torch.manual_seed(23)
    tp, rpo, n, k = 8, 32, 1024, 3584
    m = tp * rpo
    a = torch.randn(m, k, device=DEV, dtype=torch.bfloat16)
    w = torch.randn(n, k, device=DEV, dtype=torch.bfloat16)
    slabs = [torch.zeros(tp, rpo, n, device=DEV, dtype=torch.bfloat16) for _ in range(tp)]
    arrive = torch.zeros(tp, dtype=torch.int32, device=DEV)
    ticket = torch.zeros(1, dtype=torch.int32, device=DEV)
    my = 5
    ops.gemm(a, ops.tile_weight(w), epi=ops.EPI_SLAB_BF16, dst_ptrs=[s.data_ptr() for s in slabs],
             rows_per_owner=rpo, my_rank=my, dst_ld=n, bn=256, mt=2, splits=7,
             arrive_ptrs=[arrive[o:o + 1].data_ptr() for o in range(tp)], done_ticket=ticket)
    torch.cuda.synchronize()
    ops.check_status()
    ref = a.float() @ w.float().T
    for o in range(tp):
        assert _rel_err(slabs[o][my], ref[o * rpo:(o + 1) * rpo]) < 1.5e-2
        assert slabs[o][(my + 1) % tp].abs().max().item() == 0
    assert arrive.tolist() == [1] * tp and int(ticket.item()) == 0


def test_gemm_grouped_combine(ops):
    torch.manual_seed(4)
    G, cap, k, n = 4, 256, 512, 384
    counts = torch.tensor([130, 0, 77, 256], dtype=torch.int32, device=DEV)
    a = torch.randn(G, cap, k, device=DEV, dtype=torch.bfloat16)
    w = torch.randn(G, n, k, device=DEV, dtype=torch.bfloat16)
    # plain grouped store
    out = torch.zeros(G, cap, n, device=DEV, dtype=torch.bfloat16)
    m_tiles = sum((int(c) + 127) // 128 for c in counts.tolist()) + 2  # over-provisioned grid
    ops.gemm(a, w, out=out, group_counts=counts, m_tiles=m_tiles, bn=128)
    torch.cuda.synchronize()
    ops.check_status()
    for g in range(G):
        c = int(counts[g])
        if c:
            ref = a[g, :c].float() @ w[g].float().T
            assert _rel_err(out[g, :c], ref) < 1.5e-2
        if c < cap:
            assert out[g, c:].abs().max().item() == 0.0
    # weighted scatter-add through the row meta table (MoE combine on one rank)
    T = 300
    meta = torch.zeros(G, cap, 4, dtype=torch.int32, device=DEV)
    rows = torch.randint(0, T, (G, cap), device=DEV, dtype=torch.int32)
    wts = torch.rand(G, cap, device=DEV)
    meta[:, :, 1] = rows
    meta[:, :, 2] = wts.view(torch.int32)
    acc = torch.zeros(T, n, device=DEV, dtype=torch.float32)
    ticket = torch.zeros(1, dtype=torch.int32, device=DEV)
    cnt_copy = counts.clone()
    ops.gemm(a, w, epi=ops.EPI_RED_F32, dst_ptrs=[acc.data_ptr()], group_counts=cnt_copy,
             row_meta=meta, m_tiles=m_tiles, bn=128, done_ticket=ticket, reset_on_done=cnt_copy)
    torch.cuda.synchronize()
    ops.check_status()
    ref = torch.zeros(T, n, device=DEV)
    for g in range(G):
        c = int(counts[g])
        if c:
            y = (a[g, :c].float() @ w[g].float().T) * wts[g, :c, None]
            ref.index_add_(0, rows[g, :c].long(), y)
    assert _rel_err(acc, ref) < 2e-3
    assert cnt_copy.abs().max().item() == 0 and ticket.item() == 0


# ------------------------------------------------------------------------------------- attention
def _make_paged(seq_lens, hkv, d, extra_blocks=3, seed=0):
    g = torch.Generator(device="cpu").manual_seed(seed)
    n_blocks = sum((s + 15) // 16 for s in seq_lens) + extra_blocks
    k_cache = torch.randn(n_blocks, hkv, 16, d, generator=g).to(DEV, torch.bfloat16)
    v_cache = torch.randn(n_blocks, hkv, 16, d, generator=g).to(DEV, torch.bfloat16)
    perm = torch.randperm(n_blocks, generator=g).tolist()
    max_blocks = max((s + 15) // 16 for s in seq_lens)
    bt = torch.zeros(len(seq_lens), max_blocks, dtype=torch.int32)
    it = iter(perm)
    for i, s in enumerate(seq_lens):
        for j in range((s + 15) // 16):
            bt[i, j] = next(it)
    return k_cache, v_cache, bt.to(DEV)


def _gather_kv(cache, bt_row, n_tok):
    # -> [n_tok, hkv, d]
    blocks = cache[bt_row[: (n_tok + 15) // 16].long()]  # [nb, hkv, 16, d]
    return blocks.permute(0, 2, 1, 3).reshape(-1, cache.shape[1], cache.shape[3])[:n_tok]


def _ref_attn(q, k, v, scale, q_pos=None, window=0):
    # q [Tq, Hq, D], k/v [Tk, Hkv, D]; q_pos = absolute position of each query (causal mask)
    hq, hkv = q.shape[1], k.shape[1]
    k = k.float().repeat_interleave(hq // hkv, dim=1)
    v = v.float().repeat_interleave(hq // hkv, dim=1)
    s = torch.einsum("qhd,khd->hqk", q.float(), k) * scale
    if q_pos is not None:
        kpos = torch.arange(k.shape[0], device=q.device)
        mask = kpos[None, :] <= q_pos[:, None]
        if window > 0:
            mask &= kpos[None, :] > (q_pos[:, None] - window)
        s = s.masked_fill(~mask[None], float("-inf"))
    p = torch.softmax(s, -1)
    return torch.einsum("hqk,khd->qhd", p, v)


@pytest.mark.parametrize("hq,hkv,d,seq_lens,pps,window", [
    (8, 1, 128, [1, 17, 300, 64, 1000], 4, 0),
    (32, 8, 128, [5, 129, 48], 2, 0),
    (32, 4, 64, [33, 2, 257, 16], 8, 0),
    (4, 4, 64, [90, 31], 1, 0),
    (16, 1, 128, [200, 77], 4, 0),
    (8, 2, 128, [500, 130, 40], 4, 64),
])
def test_paged_decode(ops, hq, hkv, d, seq_lens, pps, window):
    torch.manual_seed(5)
    B = len(seq_lens)
    k_cache, v_cache, bt = _make_paged(seq_lens, hkv, d)
    q = torch.randn(B, hq, d, device=DEV, dtype=torch.bfloat16)
    sl = torch.tensor(seq_lens, dtype=torch.int32, device=DEV)
    max_pages = max((s + 15) // 16 for s in seq_lens)
    max_splits = (max_pages + pps - 1) // pps + 1
    part_o = torch.empty(B, hq, max_splits, d, device=DEV, dtype=torch.float32)
    part_ml = torch.empty(B, hq, max_splits, 2, device=DEV, dtype=torch.float32)
    out = torch.empty(B, hq * d, device=DEV, dtype=torch.bfloat16)
    pps_t = torch.tensor([pps], dtype=torch.int32, device=DEV)
    scale = 1.0 / math.sqrt(d)
    ops.paged_decode(q, k_cache, v_cache, bt, sl, pps_t, part_o, part_ml, out, batch=B,
                     max_splits=max_splits, window=window, scale=scale)
    torch.cuda.synchronize()
    for i, s in enumerate(seq_lens):
        k = _gather_kv(k_cache, bt[i], s)
        v = _gather_kv(v_cache, bt[i], s)
        pos = torch.tensor([s - 1], device=DEV)
        ref = _ref_attn(q[i:i + 1], k, v, scale, q_pos=pos, window=window)[0]
        got = out[i].view(hq, d)
        assert _rel_err(got, ref) < 2e-2, (i, s, _rel_err(got, ref))


@pytest.mark.parametrize("hq,hkv,d,seq_lens,pps,window", [
    (8, 1, 128, [1, 17, 300, 64, 1000], 4, 0),
    (32, 8, 128, [5, 129, 48], 2, 0),
    (14, 2, 64, [257, 16, 90], 8, 0),
    (16, 1, 128, [200, 77], 4, 0),
    (8, 2, 128, [500, 130, 40], 4, 64),
])
def test_paged_decode_block_mass(ops, hq, hkv, d, seq_lens, pps, window):
    """The heavy-hitter statistic of the decode kernel: softmax probability per 16-token block, summed
    over heads, against fp32 softmax of the same scores; the attention output itself is unchanged."""
    torch.manual_seed(15)
    B = len(seq_lens)
    k_cache, v_cache, bt = _make_paged(seq_lens, hkv, d)
    q = torch.randn(B, hq, d, device=DEV, dtype=torch.bfloat16) * 1.5
    sl = torch.tensor(seq_lens, dtype=torch.int32, device=DEV)
    W = bt.shape[1]
    max_pages = max((s + 15) // 16 for s in seq_lens)
    max_splits = (max_pages + pps - 1) // pps + 1
    part_o = torch.empty(B, hq, max_splits, d, device=DEV, dtype=torch.float32)
    part_ml = torch.empty(B, hq, max_splits, 2, device=DEV, dtype=torch.float32)
    out = torch.empty(B, hq * d, device=DEV, dtype=torch.bfloat16)
    out_plain = torch.empty_like(out)
    page_ml = torch.full((B, W, hq, 2), float("nan"), device=DEV, dtype=torch.float32)
    mass = torch.full((B, W), float("nan"), device=DEV, dtype=torch.float32)
    pps_t = torch.tensor([pps], dtype=torch.int32, device=DEV)
    scale = 1.0 / math.sqrt(d)
    kw = dict(batch=B, max_splits=max_splits, window=window, scale=scale)
    ops.paged_decode(q, k_cache, v_cache, bt, sl, pps_t, part_o, part_ml, out_plain, **kw)
    ops.paged_decode(q, k_cache, v_cache, bt, sl, pps_t, part_o, part_ml, out, page_ml=page_ml, block_mass=mass, **kw)
    torch.cuda.synchronize()
    assert torch.equal(out, out_plain)
    assert torch.isfinite(mass).all()
    for i, s in enumerate(seq_lens):
        k = _gather_kv(k_cache, bt[i], s).float().repeat_interleave(hq // hkv, dim=1)   # [s, hq, d]
        sc = torch.einsum("hd,khd->hk", q[i].float(), k) * scale
        if window > 0 and s > window:
            sc[:, :s - window] = float("-inf")
        p = torch.softmax(sc, -1).sum(0)                                                 # [s]
        ref = torch.zeros(W * 16, device=DEV)
        ref[:s] = p
        ref = ref.view(W, 16).sum(1)
        assert abs(float(mass[i].sum()) - hq) < 2e-2 * hq, (i, float(mass[i].sum()))
        assert float((mass[i] - ref).abs().max()) < 2e-2 * max(1.0, float(ref.max())), (i, s)


@pytest.mark.parametrize("hq,hkv,d,chunks,window", [
    (8, 2, 128, [(70, 70), (5, 133), (64, 64), (1, 40)], 0),
    (4, 4, 64, [(100, 100), (33, 200)], 0),
    (16, 2, 128, [(130, 400)], 0),
    (8, 1, 128, [(90, 300), (20, 20)], 48),
    (2, 1, 128, [(300, 700), (128, 128), (257, 257)], 0),
    (4, 2, 64, [(200, 500)], 100),
])
def test_paged_prefill(ops, hq, hkv, d, chunks, window):
    torch.manual_seed(6)
    q_lens = [c[0] for c in chunks]
    ctx_lens = [c[1] for c in chunks]
    k_cache, v_cache, bt = _make_paged(ctx_lens, hkv, d, seed=1)
    T = sum(q_lens)
    q = torch.randn(T, hq, d, device=DEV, dtype=torch.bfloat16)
    q_start, tile_seq, tile_q0 = [], [], []
    off = 0
    for s, ql in enumerate(q_lens):
        q_start.append(off)
        off += ql
        for q0 in range(0, ql, 128):
            tile_seq.append(s)
            tile_q0.append(q0)
    ti = lambda x: torch.tensor(x, dtype=torch.int32, device=DEV)
    out = torch.zeros(T, hq * d, device=DEV, dtype=torch.bfloat16)
    scale = 1.0 / math.sqrt(d)
    ops.paged_prefill(q, k_cache, v_cache, bt, ti(tile_seq), ti(tile_q0), ti(q_start), ti(q_lens),
                      ti(ctx_lens), out, n_tiles=len(tile_seq), window=window, scale=scale)
    torch.cuda.synchronize()
    ops.check_status()
    for s, (ql, cl) in enumerate(chunks):
        k = _gather_kv(k_cache, bt[s], cl)
        v = _gather_kv(v_cache, bt[s], cl)
        pos = torch.arange(cl - ql, cl, device=DEV)
        ref = _ref_attn(q[q_start[s]:q_start[s] + ql], k, v, scale, q_pos=pos, window=window)
        got = out[q_start[s]:q_start[s] + ql].view(ql, hq, d)
        assert _rel_err(got, ref) < 2e-2, (s, _rel_err(got, ref))


# ----------------------------------------------------------------------------- fused finalize ops
def _rms(x, w, eps, off=0.0):
    x = x.float()
    return x * torch.rsqrt(x.pow(2).mean(-1, keepdim=True) + eps) * (w.float() + off)


@pytest.mark.parametrize("rows,n", [(1, 2048), (37, 4096), (256, 8192), (3, 1024), (5, 128), (2, 14336), (4, 6152)])
def test_finalize_norm(ops, rows, n):
    torch.manual_seed(7)
    acc = torch.randn(rows, n, device=DEV)
    acc0 = acc.clone()
    res = torch.randn(rows, n, device=DEV, dtype=torch.bfloat16)
    bias = torch.randn(n, device=DEV, dtype=torch.bfloat16)
    w = torch.rand(n, device=DEV, dtype=torch.bfloat16) + 0.5
    res_out = torch.empty_like(res)
    out = torch.empty_like(res)
    ops.finalize_norm(rows=rows, n=n, acc=acc, residual_in=res, residual_out=res_out, bias=bias,
                      norm_w=w, eps=1e-5, out_ptrs=[out.data_ptr()])
    torch.cuda.synchronize()
    h = acc0 + bias.float() + res.float()
    assert _rel_err(res_out, h) < 1e-2
    assert _rel_err(out, _rms(h, w, 1e-5)) < 1.5e-2
    assert acc.abs().max().item() == 0.0
    # plain RMSNorm through the wrapper, Gemma-style weight offset
    y = ops.rmsnorm(res, w, 1e-6, w_offset=1.0)
    torch.cuda.synchronize()
    assert _rel_err(y, _rms(res, w, 1e-6, 1.0)) < 1.5e-2


def test_device_waits_that_run_out_return_a_status_and_leave_the_context_usable(ops):
    """A wait on a counter that nothing bumps (the stand-in for a peer that never arrives) gives
    up after its spin budget: the kernel returns, the status word says 'peer flag', check_status
    raises CollectiveTimeout exactly once, and the same call works once the counters are re-armed."""
    from oxide_tech_llm_engine_b200.errors import CollectiveTimeout

    torch.manual_seed(31)
    old = ops.SPIN_LIMIT
    ops.SPIN_LIMIT = 3000
    try:
        # --- reduce-scatter tail: finalize_norm waits for arrivals that never come ---
        rows, n = 8, 1024
        acc = torch.randn(rows, n, device=DEV)
        acc0 = acc.clone()
        res = torch.randn(rows, n, device=DEV, dtype=torch.bfloat16)
        w = torch.rand(n, device=DEV, dtype=torch.bfloat16) + 0.5
        out = torch.zeros_like(res)
        arrive = torch.zeros(1, dtype=torch.int32, device=DEV)
        ticket = torch.zeros(1, dtype=torch.int32, device=DEV)
        kw = dict(rows=rows, n=n, acc=acc, arrive=arrive, expected=1, ticket=ticket, residual_in=res, norm_w=w,
                  eps=1e-5, out_ptrs=[out.data_ptr()])
        ops.finalize_norm(**kw)
        torch.cuda.synchronize()
        with pytest.raises(CollectiveTimeout):
            ops.check_status()
        ops.check_status()                                   # reported once, then clean
        assert out.abs().max().item() == 0.0                 # nothing was produced from missing data
        assert torch.equal(acc, acc0)                        # and the accumulator was not consumed
        assert int(arrive.item()) == 0 and int(ticket.item()) == 0   # this wait leaves nothing to re-arm
        arrive.fill_(1)                                      # the arrival comes after all
        ops.finalize_norm(**kw)
        torch.cuda.synchronize()
        ops.check_status()
        assert _rel_err(out, _rms(acc0 + res.float(), w, 1e-5)) < 1.5e-2
        assert int(arrive.item()) == 0                       # consumed and re-armed by the kernel

        # --- all-gather -> GEMM: the producer waits for source rows that never arrive; the MMA and
        # epilogue warps then run out of their own waits and the kernel frees its TMEM and returns ---
        m, nn, k = 256, 512, 1024
        a = torch.randn(m, k, device=DEV, dtype=torch.bfloat16)
        wt = torch.randn(nn, k, device=DEV, dtype=torch.bfloat16)
        o = torch.zeros(m, nn, device=DEV, dtype=torch.bfloat16)
        flags = torch.zeros(2, dtype=torch.int32, device=DEV)
        agt = torch.zeros(1, dtype=torch.int32, device=DEV)
        gkw = dict(out=o, bn=128, ag_flags=flags, ag_expected=128, ag_rows_per_src=128, ag_ticket=agt)
        ops.gemm(a, wt, **gkw)
        torch.cuda.synchronize()
        with pytest.raises(CollectiveTimeout):
            ops.check_status()
        ops.check_status()
        # re-arm: the waiters that gave up left the ticket part-way; the owner zeroes flags and ticket
        agt.zero_()
        flags.fill_(128)
        ops.gemm(a, wt, **gkw)
        torch.cuda.synchronize()
        ops.check_status()
        assert _rel_err(o, a.float() @ wt.float().T) < 1.5e-2
        assert flags.tolist() == [0, 0] and int(agt.item()) == 0
    finally:
        ops.SPIN_LIMIT = old


def test_finalize_norm_moe_dispatch(ops):
    torch.manual_seed(8)
    rows, n, E, top_k, cap = 50, 1024, 8, 2, 64
    x = torch.randn(rows, n, device=DEV, dtype=torch.bfloat16)
    w = torch.ones(n, device=DEV, dtype=torch.bfloat16)
    router = (torch.randn(E, n, device=DEV) * 0.1).to(torch.bfloat16)
    slab = torch.zeros(E, cap, n, device=DEV, dtype=torch.bfloat16)
    meta = torch.zeros(E, cap, 4, device=DEV, dtype=torch.int32)
    cnt = torch.zeros(E, device=DEV, dtype=torch.int32)
    ops.finalize_norm(rows=rows, n=n, residual_in=x, norm_w=w, eps=1e-5, router_w=router, top_k=top_k,
                      experts_per_rank=E, slab_ptrs=[slab.data_ptr()], meta_ptrs=[meta.data_ptr()],
                      cnt_ptrs=[cnt.data_ptr()], cap=cap, my_rank=0)
    torch.cuda.synchronize()
    ops.check_status()
    y = _rms(x, w, 1e-5)
    logits = y @ router.float().T
    tv, ti = logits.topk(top_k, dim=-1)
    wt = torch.softmax(tv, -1)
    assert int(cnt.sum()) == rows * top_k
    for e in range(E):
        c = int(cnt[e])
        exp_rows = sorted((ti == e).any(-1).nonzero().flatten().tolist())
        got_rows = sorted(meta[e, :c, 1].tolist())
        assert got_rows == exp_rows, (e, got_rows, exp_rows)
        for s in range(c):
            r = int(meta[e, s, 1])
            assert _rel_err(slab[e, s], y[r]) < 1.5e-2
            kk = (ti[r] == e).nonzero().item()
            got_w = meta[e, s, 2:3].view(torch.float32).item()
            assert abs(got_w - wt[r, kk].item()) < 2e-3


@pytest.mark.parametrize("hq,hkv,d,use_acc,qk_norm", [(8, 2, 128, True, False), (32, 4, 64, False, True),
                                                      (4, 1, 128, True, True)])
def test_qkv_rope_append(ops, hq, hkv, d, use_acc, qk_norm):
    torch.manual_seed(9)
    M, n_blocks = 23, 12
    W = (hq + 2 * hkv) * d
    qkv = torch.randn(M, W, device=DEV)
    bias = torch.randn(W, device=DEV, dtype=torch.bfloat16) * 0.1
    pos = torch.randint(0, 5000, (M,), device=DEV, dtype=torch.int32)
    slots = torch.randperm(n_blocks * 16, device=DEV)[:M].to(torch.int64)
    slots[3] = -1
    inv_freq = (1.0 / (10000.0 ** (torch.arange(0, d, 2, device=DEV).float() / d))).contiguous()
    qn = (torch.rand(d, device=DEV) + 0.5).to(torch.bfloat16) if qk_norm else None
    kn = (torch.rand(d, device=DEV) + 0.5).to(torch.bfloat16) if qk_norm else None
    k_cache = torch.zeros(n_blocks, hkv, 16, d, device=DEV, dtype=torch.bfloat16)
    v_cache = torch.zeros_like(k_cache)
    q_out = torch.empty(M, hq * d, device=DEV, dtype=torch.bfloat16)
    src = qkv.to(torch.bfloat16) if not use_acc else qkv.clone()
    ops.qkv_rope_append(acc_f32=src if use_acc else None, qkv_bf16=None if use_acc else src, bias=bias,
                        q_norm_w=qn, k_norm_w=kn, norm_eps=1e-6, positions=pos, slot_mapping=slots,
                        inv_freq=inv_freq, q_out=q_out, k_cache=k_cache, v_cache=v_cache, m=M, hq=hq,
                        hkv=hkv, d=d)
    torch.cuda.synchronize()
    ops.check_status()
    x = (qkv if use_acc else qkv.to(torch.bfloat16).float()) + bias.float()
    qr = x[:, :hq * d].view(M, hq, d)
    kr = x[:, hq * d:(hq + hkv) * d].view(M, hkv, d)
    vr = x[:, (hq + hkv) * d:].view(M, hkv, d)
    if qk_norm:
        qr = _rms(qr, qn, 1e-6)
        kr = _rms(kr, kn, 1e-6)
    ang = pos.float()[:, None] * inv_freq[None, :]
    cs, sn = ang.cos()[:, None, :], ang.sin()[:, None, :]

    def rot(t):
        a, b = t[..., : d // 2], t[..., d // 2:]
        return torch.cat([a * cs - b * sn, b * cs + a * sn], -1)

    assert _rel_err(q_out.view(M, hq, d), rot(qr)) < 1.5e-2
    kref, vref = rot(kr), vr
    for i in range(M):
        s = int(slots[i])
        if s < 0:
            continue
        assert _rel_err(k_cache[s // 16, :, s % 16], kref[i]) < 1.5e-2
        assert _rel_err(v_cache[s // 16, :, s % 16], vref[i]) < 1.5e-2
    if use_acc:
        assert src.abs().max().item() == 0.0


def test_swiglu_embed_misc(ops):
    torch.manual_seed(10)
    M, I = 33, 1536
    gu = torch.randn(M, 2 * I, device=DEV)
    out = torch.empty(M, I, device=DEV, dtype=torch.bfloat16)
    ops.swiglu(acc_f32=gu.clone(), out=out, m=M, i=I)
    ref = torch.nn.functional.silu(gu[:, :I]) * gu[:, I:]
    assert _rel_err(out, ref) < 1.5e-2
    ops.swiglu(gu_bf16=gu.to(torch.bfloat16), out=out, m=M, i=I, act=1)
    g16 = gu.to(torch.bfloat16).float()
    ref = torch.nn.functional.gelu(g16[:, :I], approximate="tanh") * g16[:, I:]
    assert _rel_err(out, ref) < 1.5e-2
    # embedding gather, vocab-parallel window
    table = torch.randn(1000, 256, device=DEV, dtype=torch.bfloat16)
    toks = torch.tensor([0, 999, 5, 500, 499], dtype=torch.int32, device=DEV)
    e = torch.empty(5, 256, device=DEV, dtype=torch.bfloat16)
    ops.embed_gather(toks, table, e, scale=2.0)
    assert _rel_err(e, table[toks.long()].float() * 2) < 1e-2
    ops.embed_gather(toks, table[500:], e, vocab_start=500)
    exp = table[toks.long()].clone()
    exp[[0, 2, 4]] = 0
    assert torch.equal(e, exp)
    # FWHT
    x = torch.randn(7 * 128, device=DEV)
    ref = x.clone().view(7, 128)
    h = 1
    while h < 128:
        r = ref.view(7, 128 // (2 * h), 2, h)
        ref = torch.stack([r[:, :, 0] + r[:, :, 1], r[:, :, 0] - r[:, :, 1]], 2).reshape(7, 128)
        h *= 2
    ops.fwht128(x)
    assert _rel_err(x.view(7, 128), ref / math.sqrt(128)) < 1e-5
    # KV block copy
    kc = torch.randn(6, 2, 16, 64, device=DEV).to(torch.bfloat16)
    vc = torch.randn(6, 2, 16, 64, device=DEV).to(torch.bfloat16)
    k0, v0 = kc.clone(), vc.clone()
    ops.kv_block_copy(kc, vc, torch.tensor([1, 4], dtype=torch.int32, device=DEV),
                      torch.tensor([0, 5], dtype=torch.int32, device=DEV))
    assert torch.equal(kc[0], k0[1]) and torch.equal(vc[5], v0[4]) and torch.equal(kc[2], k0[2])
    # softcap
    lg = torch.randn(3, 100, device=DEV) * 50
    ref = 30 * torch.tanh(lg / 30)
    ops.softcap(lg, 30.0)
    assert _rel_err(lg, ref) < 1e-5


# --------------------------------------------------------------------------------- quantized ops
QTYPES = ["Q4_0", "Q4_1", "Q5_0", "Q5_1", "Q8_0", "Q2_K", "Q3_K", "Q4_K", "Q5_K", "Q6_K", "IQ4_NL",
          "TQ2_0", "NVFP4"]


@pytest.mark.parametrize("qname", QTYPES)
def test_dequant_and_mmvq(ops, qname):
    from oxide_tech_llm_engine_b200.formats import quants

    rng = np.random.default_rng(11)
    N, K = 72, 1024
    w = (rng.standard_normal((N, K)) * 0.05).astype(np.float32)
    raw = quants.quantize_2d(qname, w)
    wd = quants.dequantize_2d(qname, raw, N, K)  # numpy oracle of the packed weights
    code = quants.TYPES[qname].code
    w_dev = torch.from_numpy(raw).to(DEV)
    out = torch.empty(N, K, device=DEV, dtype=torch.bfloat16)
    ops.dequant_rows(code, w_dev, out, n_src_rows=N, k=K)
    torch.cuda.synchronize()
    ref = torch.from_numpy(wd).to(DEV)
    assert _rel_err(out, ref) < 8e-3, qname  # bf16 rounding of an fp32-exact decode
    ids = torch.tensor([5, 0, 71, 5], dtype=torch.int32, device=DEV)
    g = torch.empty(4, K, device=DEV, dtype=torch.bfloat16)
    ops.dequant_rows(code, w_dev, g, n_src_rows=N, k=K, row_ids=ids, scale=0.5)
    assert _rel_err(g, ref[ids.long()] * 0.5) < 1e-2
    for M in (1, 2, 3, 8, 13):
        x = torch.randn(M, K, device=DEV, dtype=torch.bfloat16)
        y = torch.empty(M, N, device=DEV, dtype=torch.float32)
        ops.mmvq(code, w_dev, x, y, n=N, k=K)
        torch.cuda.synchronize()
        yref = x.float() @ ref.T
        assert _rel_err(y, yref) < 2e-3, (qname, M, _rel_err(y, yref))
    if code in ops.INT8_MMVQ_CODES:
        # integer dot-product path: activations quantised to int8 blocks of 32 (Q8_1 style)
        for M in (1, 2, 3, 8):
            x = torch.randn(M, K, device=DEV, dtype=torch.bfloat16)
            q8, xd, xs = ops.quant_q8_1(x)
            xb = x.float().view(M, K // 32, 32)
            torch.testing.assert_close(xd, xb.abs().amax(-1) / 127.0, rtol=1e-5, atol=1e-12)
            deq = q8.float().view(M, K // 32, 32) * xd[..., None]
            assert (deq - xb).abs().max() <= xd.max() * 0.51
            torch.testing.assert_close(xs, deq.sum(-1), rtol=1e-4, atol=1e-4)
            y = torch.empty(M, N, device=DEV, dtype=torch.float32)
            ops.mmvq(code, w_dev, x, y, n=N, k=K, xq=(q8, xd, xs))
            torch.cuda.synchronize()
            exact = deq.view(M, K) @ ref.T            # exact product of the quantised activations
            assert _rel_err(y, exact) < 2e-3, (qname, M, _rel_err(y, exact))
            assert _rel_err(y, x.float() @ ref.T) < 3e-2
    bias = torch.randn(N, device=DEV, dtype=torch.bfloat16)
    x = torch.randn(4, K, device=DEV, dtype=torch.bfloat16)
    yb = torch.randn(4, N, device=DEV).to(torch.bfloat16)
    y0 = yb.clone()
    ops.mmvq(code, w_dev, x, yb, n=N, k=K, bias=bias, add=True)
    assert _rel_err(yb, x.float() @ ref.T + bias.float() + y0.float()) < 2e-2


@pytest.mark.parametrize("qname", ["Q4_K", "Q6_K", "Q8_0", "Q5_K", "Q5_0", "Q4_0", "Q4_1", "Q5_1"])
def test_gemm_with_gguf_weights_unpacked_in_the_kernel(ops, qname):
    """tcgen05 GEMM whose weight operand stays GGUF-packed in HBM: against fp32 of the activations times
    the decoded weights (rounded to bf16, as the kernel's operand stage holds them)."""
    from oxide_tech_llm_engine_b200.formats import quants

    rng = np.random.default_rng(31)
    N, K = 200, 1024
    w = (rng.standard_normal((N, K)) * 0.05).astype(np.float32)
    raw = quants.quantize_2d(qname, w)
    wd = torch.from_numpy(quants.dequantize_2d(qname, raw, N, K)).to(DEV).to(torch.bfloat16).float()
    code = quants.TYPES[qname].code
    w_dev = torch.from_numpy(raw).to(DEV).view(-1)
    for M, mt, splits in ((17, 1, 1), (128, 1, 2), (300, 2, 1), (300, 1, 4), (513, 2, 2)):
        x = torch.randn(M, K, device=DEV, dtype=torch.bfloat16)
        ref = x.float() @ wd.T
        out = torch.zeros(M, N, device=DEV, dtype=torch.float32)
        ops.gemm_packed(x, code, w_dev, N, out, epi=ops.EPI_RED_F32, mt=mt, splits=splits)
        torch.cuda.synchronize()
        ops.check_status()
        assert _rel_err(out, ref) < 2e-3, (qname, M, mt, splits, _rel_err(out, ref))
    x = torch.randn(140, K, device=DEV, dtype=torch.bfloat16)
    bias = torch.randn(N, device=DEV, dtype=torch.bfloat16)
    out = torch.empty(140, N, device=DEV, dtype=torch.bfloat16)
    ops.gemm_packed(x, code, w_dev, N, out, epi=ops.EPI_STORE_BF16, mt=2, bias=bias)
    torch.cuda.synchronize()
    assert _rel_err(out, x.float() @ wd.T + bias.float()) < 1e-2


def test_norm_and_swiglu_write_the_int8_view_of_their_output(ops):
    """finalize_norm and swiglu with `q8`: the int8 blocks, scales and sums are exactly what the
    stand-alone quantiser makes of the bf16 rows those kernels wrote."""
    torch.manual_seed(41)
    rows, n = 5, 4096
    x = torch.randn(rows, n, device=DEV, dtype=torch.bfloat16)
    w = (torch.rand(n, device=DEV) + 0.5).to(torch.bfloat16)
    out = torch.empty_like(x)
    q8 = (torch.zeros(rows, n, dtype=torch.int8, device=DEV), torch.zeros(rows, n // 32, device=DEV),
          torch.zeros(rows, n // 32, device=DEV))
    ops.finalize_norm(rows=rows, n=n, residual_in=x, norm_w=w, eps=1e-5, out_ptrs=[out.data_ptr()], device=x.device,
                      q8=q8)
    want = ops.quant_q8_1(out)
    torch.cuda.synchronize()
    for got, ref in zip(q8, want):
        assert torch.equal(got, ref)
    m, i = 3, 1024
    gu = torch.randn(m, 2 * i, device=DEV, dtype=torch.bfloat16)
    act = torch.empty(m, i, device=DEV, dtype=torch.bfloat16)
    q8 = (torch.zeros(m, i, dtype=torch.int8, device=DEV), torch.zeros(m, i // 32, device=DEV),
          torch.zeros(m, i // 32, device=DEV))
    ops.swiglu(gu_bf16=gu, out=act, m=m, i=i, q8=q8)
    want = ops.quant_q8_1(act)
    torch.cuda.synchronize()
    for got, ref in zip(q8, want):
        assert torch.equal(got, ref)
    # decode attention: the merge kernel writes the int8 view of the attention output
    seq_lens, hq, hkv, d = [70, 5, 300], 8, 2, 128
    B = len(seq_lens)
    k_cache, v_cache, bt = _make_paged(seq_lens, hkv, d)
    q = torch.randn(B, hq, d, device=DEV, dtype=torch.bfloat16)
    sl = torch.tensor(seq_lens, dtype=torch.int32, device=DEV)
    part_o = torch.empty(B, hq, 8, d, device=DEV, dtype=torch.float32)
    part_ml = torch.empty(B, hq, 8, 2, device=DEV, dtype=torch.float32)
    out = torch.empty(B, hq * d, device=DEV, dtype=torch.bfloat16)
    q8 = (torch.zeros(B, hq * d, dtype=torch.int8, device=DEV), torch.zeros(B, hq * d // 32, device=DEV),
          torch.zeros(B, hq * d // 32, device=DEV))
    ops.paged_decode(q, k_cache, v_cache, bt, sl, torch.tensor([4], dtype=torch.int32, device=DEV), part_o, part_ml, out,
                     batch=B, max_splits=8, scale=1.0 / math.sqrt(d), q8=q8)
    want = ops.quant_q8_1(out)
    torch.cuda.synchronize()
    for got, ref in zip(q8, want):
        assert torch.equal(got, ref)


def test_mmvq_mixed_types_in_one_launch(ops):
    """Q | K | V of a mixed-precision file (Q4_K, Q4_K, Q6_K) and two more combinations as one GEMV
    launch each, against the exact product of the int8 activations with the decoded weights."""
    from oxide_tech_llm_engine_b200.formats import quants

    rng = np.random.default_rng(21)
    K = 1024
    for names, rows in ((("Q4_K", "Q4_K", "Q6_K"), (40, 16, 16)), (("Q5_K", "Q8_0"), (24, 9)),
                        (("Q4_0", "Q5_0", "Q4_1", "Q5_1"), (8, 8, 3, 5))):
        parts, refs = [], []
        for nm, n in zip(names, rows):
            w = (rng.standard_normal((n, K)) * 0.05).astype(np.float32)
            raw = quants.quantize_2d(nm, w)
            refs.append(torch.from_numpy(quants.dequantize_2d(nm, raw, n, K)).to(DEV))
            parts.append((quants.TYPES[nm].code, torch.from_numpy(raw).to(DEV).view(-1), n))
        ref = torch.cat(refs, 0)
        N = ref.shape[0]
        for M in (1, 2, 4, 7):
            x = torch.randn(M, K, device=DEV, dtype=torch.bfloat16)
            xq = ops.quant_q8_1(x)
            deq = (xq[0].float().view(M, K // 32, 32) * xq[1][..., None]).view(M, K)
            y = torch.full((M, N + 3), float("nan"), device=DEV, dtype=torch.float32)
            ops.mmvq_mixed(parts, x, y, k=K, xq=xq)
            torch.cuda.synchronize()
            assert _rel_err(y[:, :N], deq @ ref.T) < 2e-3, (names, M)
            assert torch.isnan(y[:, N:]).all()


# --------------------------------------------------------------------------------------- sampler
def test_argmax_and_sampling(ops):
    torch.manual_seed(12)
    B, V = 9, 128256
    logits = torch.randn(B, V, device=DEV)
    out = torch.empty(B, dtype=torch.int32, device=DEV)
    val = torch.empty(B, device=DEV)
    ops.argmax(logits, out, val)
    assert torch.equal(out.long(), logits.argmax(-1))
    assert torch.allclose(val, logits.max(-1).values)
    # greedy through the sampler (temperature 0) with a mask that bans the argmax
    mask = torch.full((B, (V + 31) // 32), -1, dtype=torch.int32, device=DEV)
    am = logits.argmax(-1)
    for b in range(B):
        w_, bit = int(am[b]) // 32, int(am[b]) % 32
        mask[b, w_] &= ~(1 << bit) if bit < 31 else 0x7FFFFFFF
    temp = torch.zeros(B, device=DEV)
    ops.sample(logits, out, temperature=temp, allow_mask=mask)
    second = logits.clone()
    second[torch.arange(B), am] = float("-inf")
    assert torch.equal(out.long(), second.argmax(-1))
    # stochastic: top-k=4 draws stay inside the top 4 and follow the renormalised distribution
    V2 = 5000
    lg = torch.randn(1, V2, device=DEV).repeat(4000, 1).contiguous()
    n = lg.shape[0]
    temp = torch.full((n,), 0.8, device=DEV)
    tk = torch.full((n,), 4, dtype=torch.int32, device=DEV)
    tp = torch.full((n,), 1.0, device=DEV)
    mp = torch.zeros(n, device=DEV)
    seeds = torch.full((n,), 1234, dtype=torch.int64, device=DEV)
    ctr = torch.arange(n, dtype=torch.int64, device=DEV)
    toks = torch.empty(n, dtype=torch.int32, device=DEV)
    ops.sample(lg, toks, temperature=temp, top_k=tk, top_p=tp, min_p=mp, seeds=seeds, counters=ctr)
    top4 = lg[0].topk(4)
    assert set(toks.tolist()) <= set(top4.indices.tolist())
    p = torch.softmax(top4.values / 0.8, -1)
    freq = torch.stack([(toks == i).float().mean() for i in top4.indices])
    assert (freq - p).abs().max().item() < 0.04
    toks2 = torch.empty_like(toks)
    ops.sample(lg, toks2, temperature=temp, top_k=tk, top_p=tp, min_p=mp, seeds=seeds, counters=ctr)
    assert torch.equal(toks, toks2)  # same seed and counter -> same draw
    # top-p = tiny keeps only the best token; min-p = 1 likewise
    tp2 = torch.full((n,), 1e-4, device=DEV)
    ops.sample(lg, toks, temperature=temp, top_k=torch.zeros_like(tk), top_p=tp2, min_p=mp, seeds=seeds,
               counters=ctr)
    assert (toks == top4.indices[0]).all()
    mp2 = torch.ones(n, device=DEV)
    ops.sample(lg, toks, temperature=temp, top_k=torch.zeros_like(tk), top_p=tp, min_p=mp2, seeds=seeds,
               counters=ctr)
    assert (toks == top4.indices[0]).all()
    # top-k off on a flat, hot distribution: the nucleus is cut where the FULL softmax reaches top_p,
    # not where the softmax over the 1024 candidates does, and the log-probability is the full one
    hot = torch.full((n,), 3.0, device=DEV)
    tp3 = torch.full((n,), 0.10, device=DEV)
    lp = torch.empty(n, device=DEV)
    ops.sample(lg, toks, temperature=hot, top_k=torch.zeros_like(tk), top_p=tp3, min_p=mp, seeds=seeds,
               counters=ctr, out_logit=lp)
    full = torch.softmax(lg[0] / 3.0, -1)
    srt = full.sort(descending=True)
    n_keep = int((srt.values.cumsum(0) < 0.10).sum().item()) + 1
    nucleus = set(srt.indices[:n_keep].tolist())
    drawn = set(toks.tolist())
    assert drawn <= nucleus and len(drawn) > 0.5 * n_keep, (len(drawn), n_keep)
    torch.testing.assert_close(lp, torch.log(full[toks.long()]), rtol=0, atol=2e-3)


def test_argmax_exchange_on_one_rank(ops):
    """The peer-memory argmax exchange with a single rank: the word table is this GPU's own, both slots
    give the argmax (lowest index on ties) and leave the table empty; a word that never arrives ends
    the bounded wait with the peer-flag status instead of hanging."""
    from oxide_tech_llm_engine_b200.errors import CollectiveTimeout

    torch.manual_seed(13)
    rows, V, max_rows = 7, 5000, 16
    logits = torch.randn(rows, V, device=DEV)
    logits[2, 17] = logits[2, 4000] = 50.0                      # a tie: the lower index wins
    tab = torch.zeros(2, 1, max_rows, dtype=torch.int64, device=DEV)
    out = torch.full((rows,), -1, dtype=torch.int32, device=DEV)
    for slot in (0, 1, 0):
        ops.argmax_exchange(logits, out, vocab_start=100, tab_ptrs=[tab.data_ptr()], max_rows=max_rows, my_rank=0,
                            slot=slot)
        torch.cuda.synchronize()
        assert torch.equal(out.long(), logits.argmax(-1) + 100) and int(out[2]) == 117
        assert int(tab.abs().sum()) == 0
    # two ranks declared, the second never writes: rank 0 gives up after the spin budget
    tab2 = torch.zeros(2, 2, max_rows, dtype=torch.int64, device=DEV)
    old = ops.SPIN_LIMIT
    ops.SPIN_LIMIT = 2000
    try:
        ops.argmax_exchange(logits, out, vocab_start=0, tab_ptrs=[tab2.data_ptr(), tab2.data_ptr()], max_rows=max_rows,
                            my_rank=0, slot=0)
        torch.cuda.synchronize()
        with pytest.raises(CollectiveTimeout):
            ops.check_status()
    finally:
        ops.SPIN_LIMIT = old
    ops.check_status()


@pytest.mark.gpu
@pytest.mark.parametrize("M,N,K", [(128, 256, 512), (200, 384, 1024), (8, 1024, 4096), (640, 1152, 2048), (130, 200, 272)])
def test_gemm_fp8_block_scaled(ops, M, N, K):
    """Block-scaled fp8 GEMM against the fp32 product of the dequantised operands."""
    torch.manual_seed(M + N + K)
    x = (torch.randn(M, K, device="cuda") * torch.rand(M, 1, device="cuda") * 3).bfloat16()
    w = torch.randn(N, K, device="cuda") * 0.05
    w8, sw = ops.quant_weight_fp8_block(w)
    a8, sa_t = ops.quant_act_fp8(x)
    # activation quantiser: scales are amax/448 per 1x128 block, values round-trip within e4m3 error
    kb = (K + 127) // 128
    xp = torch.zeros(M, kb * 128, device="cuda")
    xp[:, :K] = x.float()
    amax = xp.view(M, kb, 128).abs().amax(-1)
    torch.testing.assert_close(sa_t.t().contiguous(), amax.clamp_min(1e-10) / 448.0, rtol=1e-5, atol=1e-12)
    a_deq = (a8.float().view(torch.float32) if False else a8.to(torch.float32))
    a_deq = a_deq * sa_t.t().repeat_interleave(128, 1)[:, :K]
    assert (a_deq - x.float()).abs().max() <= 0.07 * x.float().abs().max()
    w_deq = w8.to(torch.float32) * sw.repeat_interleave(128, 0)[:N].repeat_interleave(128, 1)[:, :K]
    ref = a_deq @ w_deq.t()
    bias = torch.randn(N, device="cuda").bfloat16()
    out = ops.gemm_fp8_block(a8, sa_t, w8, sw, bias=bias)
    ops.check_status(out.device)
    ref = ref + bias.float()
    err = (out.float() - ref).abs().max().item()
    assert err <= 2e-2 * ref.abs().max().item() + 1e-3, err


@pytest.mark.gpu
@pytest.mark.parametrize("bn", [64, 128, 256])
@pytest.mark.parametrize("m,n,k", [(200, 512, 256), (256, 1280, 1024), (8, 768, 192)])
def test_gemm_tile_major_weights(ops, m, n, k, bn):
    """Weights stored tile-major ([N/128, K/64, 128, 64]) give the same product as row-major."""
    torch.manual_seed(m + n + k + bn)
    a = torch.randn(m, k, device="cuda").bfloat16()
    w = (torch.randn(n, k, device="cuda") * 0.1).bfloat16()
    wt = ops.tile_weight(w)
    assert wt.dim() == 4 and torch.equal(ops.untile_weight(wt), w)
    ref = a.float() @ w.float().t()
    out = ops.gemm(a, wt, bn=bn)
    ops.check_status(out.device)
    assert _rel_err(out.float(), ref) < 2e-2
    acc = torch.zeros(m, n, device="cuda")
    ops.gemm(a, wt, epi=ops.EPI_RED_F32, dst_ptrs=[acc.data_ptr()], bn=bn, splits=2)
    ops.check_status(out.device)
    assert _rel_err(acc, ref) < 1e-2
    assert ops.tile_weight(w[:100]).dim() == 2   # shapes that do not tile stay row-major


@pytest.mark.gpu
def test_block_table_bounds_are_checked_without_touching_memory(ops):
    """A block id beyond the pool that the kernel was told about is recorded in the status word and
    page 0 is read instead. The 'pool' passed here is a view of the first 8 blocks of a 32-block
    allocation, so even an unchecked read would stay inside allocated memory."""
    torch.manual_seed(0)
    D, hq, hkv, B = 128, 8, 1, 2
    full_k = torch.randn(32, hkv, 16, D, device="cuda").bfloat16()
    full_v = torch.randn(32, hkv, 16, D, device="cuda").bfloat16()
    k, v = full_k[:8], full_v[:8]
    q = torch.randn(B, hq, D, device="cuda").bfloat16()
    bt = torch.tensor([[0, 1, 2, 3], [4, 20, 5, 6]], dtype=torch.int32, device="cuda")   # 20 >= 8
    lens = torch.tensor([40, 50], dtype=torch.int32, device="cuda")
    pps = torch.tensor([4], dtype=torch.int32, device="cuda")
    part_o = torch.zeros(B * hq * 4 * D, device="cuda")
    part_ml = torch.zeros(B * hq * 4 * 2, device="cuda")
    out = torch.zeros(B, hq * D, device="cuda", dtype=torch.bfloat16)
    ops.check_status(q.device)
    old = ops.CHECK_BOUNDS
    ops.CHECK_BOUNDS = True
    try:
        ops.paged_decode(q, k, v, bt, lens, pps, part_o, part_ml, out, batch=B, max_splits=4, scale=D ** -0.5)
    finally:
        ops.CHECK_BOUNDS = old
    torch.cuda.synchronize()
    from oxide_tech_llm_engine_b200.errors import EngineError
    with pytest.raises(EngineError):
        ops.check_status(q.device)
    ops.check_status(q.device)   # the status word was cleared by the failed check
    assert torch.isfinite(out.float()).all()


@pytest.mark.gpu
@pytest.mark.parametrize("tiled", [False, True])
@pytest.mark.parametrize("m,n,k", [(1, 512, 1024), (3, 256, 192), (8, 1280, 4096)])
def test_gemv_bf16_small_batch(ops, m, n, k, tiled):
    torch.manual_seed(m * n + k)
    x = torch.randn(m, k, device="cuda").bfloat16()
    w = (torch.randn(n, k, device="cuda") * 0.05).bfloat16()
    bias = torch.randn(n, device="cuda").bfloat16()
    ww = ops.tile_weight(w) if tiled else w
    if tiled and ww.dim() != 4:
        pytest.skip("shape does not tile")
    ref = x.float() @ w.float().t()
    out = torch.zeros(m, n, device="cuda")
    ops.gemv(x, ww, out, bias=bias)
    assert _rel_err(out, ref + bias.float()) < 2e-3
    outb = torch.zeros(m, n, device="cuda", dtype=torch.bfloat16)
    ops.gemv(x, ww, outb)
    assert _rel_err(outb, ref) < 1e-2
    if n % 64 == 0:
        # gate|up interleaved in units of 32 rows, as the fused SwiGLU GEMM epilogue stores them
        from oxide_tech_llm_engine_b200.models.llama import interleave32
        g, u = w[: n // 2], w[n // 2:]
        wi = interleave32(g, u)
        wi = ops.tile_weight(wi) if tiled else wi
        y = torch.zeros(m, n // 2, device="cuda", dtype=torch.bfloat16)
        ops.gemv(x, wi, y, swiglu=True)
        gr, ur = x.float() @ g.float().t(), x.float() @ u.float().t()
        assert _rel_err(y, torch.nn.functional.silu(gr) * ur) < 1.5e-2


# ------------------------------------------------------------------------------------------ NVFP4
@pytest.mark.gpu
@pytest.mark.parametrize("m", [1, 17, 128, 300])
def test_gemm_nvfp4_block_scaled_against_dequantised_operands(ops, m):
    """The block-scaled fp4 tensor-core GEMM against the fp32 product of the *dequantised* operands
    (so the only difference is the accumulation order), and the quantiser against its own rules."""
    torch.manual_seed(40 + m)
    n, k = 384, 1024
    x = (torch.randn(m, k, device=DEV) * torch.rand(m, 1, device=DEV) * 4).bfloat16()
    w = torch.randn(n, k, device=DEV) * 0.05
    wq = ops.Nvfp4Weight.from_float(w)
    assert _rel_err(wq.dequant(), w) < 0.3 and _cos(wq.dequant(), w) > 0.99      # 4-bit weights
    xq, sfa, gs = ops.quant_act_nvfp4(x)
    xd = ops.dequant_act_nvfp4(xq, sfa, gs)
    assert _cos(xd, x.float()) > 0.99 and (xd.abs().amax(1) <= x.float().abs().amax(1) * 1.001).all()
    ref = xd @ wq.dequant().T
    out = ops.gemm(xq, wq.q, sfa=sfa, sfb=wq.sf, a_gscale=gs, w_gscale=wq.gscale)
    torch.cuda.synchronize()
    ops.check_status()
    assert out.shape == (m, n) and _rel_err(out, ref) < 1.5e-2 and _cos(out, ref) > 0.9999, _rel_err(out, ref)
    out32 = ops.gemm(xq, wq.q, sfa=sfa, sfb=wq.sf, a_gscale=gs, w_gscale=wq.gscale, epi=ops.EPI_STORE_F32)
    torch.cuda.synchronize()
    assert _rel_err(out32, ref) < 2e-3


@pytest.mark.gpu
def test_nvfp4_weights_from_gguf_blocks_keep_the_file_bits(ops):
    from oxide_tech_llm_engine_b200.formats import quants

    rng = np.random.default_rng(3)
    n, k = 256, 512
    w = (rng.standard_normal((n, k)) * 0.05).astype(np.float32)
    raw = quants.quantize("NVFP4", w)
    want = torch.from_numpy(quants.dequantize("NVFP4", raw, n * k).reshape(n, k)).to(DEV)
    wq = ops.Nvfp4Weight.from_gguf_blocks(torch.from_numpy(raw.reshape(-1, 16).copy()).to(DEV), n, k)
    assert torch.equal(wq.dequant(), want)           # the same values, bit for bit
    x = torch.randn(40, k, device=DEV).bfloat16()
    xq, sfa, gs = ops.quant_act_nvfp4(x)
    out = ops.gemm(xq, wq.q, sfa=sfa, sfb=wq.sf, a_gscale=gs, w_gscale=wq.gscale)
    torch.cuda.synchronize()
    ops.check_status()
    assert _rel_err(out, ops.dequant_act_nvfp4(xq, sfa, gs) @ want.T) < 1.5e-2


@pytest.mark.gpu
def test_gemm_nvfp4_grouped_swiglu_and_combine(ops):
    """Expert GEMMs on packed fp4 weights: grouped gate|up with the SwiGLU epilogue over a slab with
    per-expert row counts, then the grouped down projection with the weighted combine epilogue."""
    torch.manual_seed(44)
    G, cap, d, i = 4, 128, 512, 256
    counts = torch.tensor([100, 0, 128, 37], dtype=torch.int32, device=DEV)
    slab = torch.randn(G, cap, d, device=DEV).bfloat16()
    wg = torch.randn(G, i, d, device=DEV) * 0.05
    wu = torch.randn(G, i, d, device=DEV) * 0.05
    w_gu = torch.stack([wg.view(G, i // 32, 32, d), wu.view(G, i // 32, 32, d)], 2).reshape(G, 2 * i, d)
    wq_gu = ops.Nvfp4Weight.from_float(w_gu)
    wq_dn = ops.Nvfp4Weight.from_float(torch.randn(G, d, i, device=DEV) * 0.05)
    sq, ssf, sgs = ops.quant_act_nvfp4(slab, group_counts=counts)
    act = torch.zeros(G, cap, i, device=DEV, dtype=torch.bfloat16)
    ops.gemm(sq, wq_gu.q, out=act, epi=ops.EPI_SWIGLU_BF16, group_counts=counts, m_tiles=G * (cap // 128),
             sfa=ssf, sfb=wq_gu.sf, a_gscale=sgs, w_gscale=wq_gu.gscale)
    torch.cuda.synchronize()
    ops.check_status()
    deq_w = wq_gu.dequant().view(G, i // 32, 2, 32, d)
    for g in range(G):
        c = int(counts[g])
        if c == 0:
            continue
        xd = ops.dequant_act_nvfp4(sq[g], ssf.view(G, -1)[g], sgs.view(G, cap)[g])[:c]
        gate = xd @ deq_w[g, :, 0].reshape(i, d).T
        up = xd @ deq_w[g, :, 1].reshape(i, d).T
        assert _rel_err(act[g, :c], torch.nn.functional.silu(gate) * up) < 2e-2, g
    # down projection + combine: row r of expert g goes home to row meta[g, r].row with its weight
    meta = torch.zeros(G, cap, 4, dtype=torch.int32, device=DEV)
    home = torch.randint(0, 64, (G, cap), device=DEV, dtype=torch.int32)
    wts = torch.rand(G, cap, device=DEV)
    meta[:, :, 1] = home
    meta[:, :, 2] = wts.view(torch.int32)
    acc = torch.zeros(64, d, device=DEV)
    aq, asf, ags = ops.quant_act_nvfp4(act, group_counts=counts)
    ops.gemm(aq, wq_dn.q, epi=ops.EPI_RED_F32, dst_ptrs=[acc.data_ptr()], group_counts=counts, row_meta=meta,
             m_tiles=G * (cap // 128), sfa=asf, sfb=wq_dn.sf, a_gscale=ags, w_gscale=wq_dn.gscale)
    torch.cuda.synchronize()
    ops.check_status()
    ref = torch.zeros(64, d, device=DEV)
    dn = wq_dn.dequant()
    for g in range(G):
        c = int(counts[g])
        if c == 0:
            continue
        ad = ops.dequant_act_nvfp4(aq[g], asf.view(G, -1)[g], ags.view(G, cap)[g])[:c]
        ref.index_add_(0, home[g, :c].long(), (ad @ dn[g].T) * wts[g, :c, None])
    assert _rel_err(acc, ref) < 2e-3
