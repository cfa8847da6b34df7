"""Python front-ends of the sm_100a kernels.

Every function here launches a hand-written kernel from ``csrc/kernels``; there is no PyTorch
fallback on this path. If the CUDA extension cannot be loaded the import error propagates, so a
GPU box never runs these ops on a silent eager substitute.
"""
from __future__ import annotations

import os
from typing import Optional, Sequence

import torch

from .._build import cuda_ext

EPI_STORE_BF16 = 0
EPI_RED_F32 = 1
EPI_STORE_F32 = 2
EPI_SWIGLU_BF16 = 3
EPI_SLAB_BF16 = 4

STATUS_NAMES = {
    0: "ok",
    1: "mbarrier timeout (TMA producer)",
    2: "mbarrier timeout (MMA issuer)",
    3: "mbarrier timeout (epilogue)",
    4: "peer flag timeout",
    5: "index out of range",
}


# number of kernel launches issued through this module (bench.py reports it)
launch_count = 0


def _ext():
    return cuda_ext()


def _bump(n: int = 1) -> None:
    global launch_count
    launch_count += n


_status: dict[int, torch.Tensor] = {}


def status_word(device: torch.device | int | None = None) -> torch.Tensor:
    """Per-device int32 error word that kernels set when a bounded wait expires."""
    dev = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
    key = dev.index if dev.index is not None else torch.cuda.current_device()
    if key not in _status:
        _status[key] = torch.zeros(1, dtype=torch.int32, device=dev)
    return _status[key]


def check_status(device=None) -> None:
    """Host check of the kernel status word (one D2H copy); raises on a recorded timeout."""
    from ..errors import CollectiveTimeout, EngineError

    code = int(status_word(device).item())
    if code != 0:
        status_word(device).zero_()
        msg = STATUS_NAMES.get(code, f"code {code}")
        if code == 4:
            raise CollectiveTimeout(f"device wait expired: {msg}")
        raise EngineError(f"kernel reported: {msg}")


# Iterations of every bounded device-side wait (0 = the compile-time default of about a second).
# Tests of the time-out path set a few thousand.
SPIN_LIMIT = 0



def set_pdl(on: bool) -> None:
    """Programmatic dependent launch of the step's kernels (GEMM, finalize_norm, QKV RoPE/append,
    decode attention + merge): a kernel becomes resident while the one before it drains, runs its
    prologue (and, in the GEMM, requests the first weight tiles of its operand ring) and then waits
    for the earlier kernel to complete before it touches anything that kernel produced. Also holds
    inside CUDA graphs captured afterwards."""
    _ext().set_pdl(bool(on))


def pdl_enabled() -> bool:
    return bool(_ext().pdl_enabled())


_sm_count: dict[int, int] = {}


def sm_count(device=None) -> int:
    dev = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
    key = dev.index if dev.index is not None else torch.cuda.current_device()
    if key not in _sm_count:
        _sm_count[key] = torch.cuda.get_device_properties(key).multi_processor_count
    return _sm_count[key]


def pick_bn(n: int, m_tiles: int = 1, can_split: bool = False) -> int:
    """Output-tile width. Wide tiles move fewer operand bytes per FLOP through the 64 B/clk
    SM<->L2 port, so take the widest tile that still gives about one CTA per SM; GEMMs that can
    split K keep 128-wide tiles and fill the machine with splits instead."""
    if n % 256 == 0 and (n // 256) * m_tiles >= 120:
        return 256
    t128 = (n + 127) // 128 * m_tiles
    if t128 >= 60 or can_split or n % 64 != 0 or n < 64:
        return 128
    return 64


def pick_splits(m: int, n: int, k: int, bn: int, sms: int = 148) -> int:
    """Split-K factor so that small GEMMs still occupy most SMs (needs the fp32 red epilogue)."""
    tiles = ((m + 127) // 128) * ((n + bn - 1) // bn)
    kb = (k + 63) // 64
    if tiles >= 100 or kb < 8:
        return 1
    return min(max(1, sms // tiles), max(1, kb // 4), 16)


def pick_decode_cfg(m: int, n: int, k: int, *, swiglu: bool = False, sms: int = 148) -> tuple[int, int, int]:
    """(bn, mt, splits) for a GEMM with at most 256 rows against a large weight matrix.

    All rows stay with the CTA that loads a weight tile (mt = 2 above 128 rows) and K is split so
    that tiles * splits fills the SMs; the splits are combined inside the kernel. The choice
    minimises a cost model fitted to per-CTA timelines measured on a B200 (bench_gemm --trace):
    a 64-wide k block costs the slower of the CTA's shared-memory traffic (TMA fills plus the
    operand reads of the MMAs at 128 B/clk), its share of an HBM stream of about 4.5 TB/s and its
    share of about 10 TB/s between L2 and the SMs; a
    split costs the store of the partial tile (3 us for 256 x 256), about 1 us at the ticket and
    3 us (6 us with SwiGLU) per 128 x 64 output unit that the CTA then combines; a direct epilogue
    costs 1.4 us (2.2 us with SwiGLU) per unit.
    """
    mt = 2 if m > 128 else 1
    rows = 128 * mt
    kb = (k + 63) // 64
    best = None
    for bn in (256, 128, 64):
        if n % bn and (swiglu or n < bn):
            continue
        tiles = (n + bn - 1) // bn
        if tiles > sms:
            cands = [1]
        else:
            cap = max_fixup_splits(bn, mt, swiglu)
            cands = sorted({1, *(s for s in range(2, min(sms // tiles, kb // 2, cap) + 1))})
        for s in cands:
            per = -(-kb // s)
            s_eff = -(-kb // per)
            n_cta = tiles * s_eff
            waves = -(-n_cta // sms)
            smem_us = ((rows + bn) * 128 + 4 * mt * (128 + bn) * 32) / (128 * 1.9e3)
            hbm_us = min(n_cta, sms) * bn * 128 / 4.5e6
            l2_us = min(n_cta, sms) * (rows + bn) * 128 / 10e6   # both operands cross the L2 -> SM fabric
            main_us = waves * per * 1.1 * max(smem_us, hbm_us, l2_us)
            units = mt * (((bn // 2 if swiglu else bn) + 63) // 64)
            if s_eff > 1:
                tail_us = 0.6 + rows * bn * 2 / 55e3 + 1.0 + -(-units // s_eff) * (6.0 if swiglu else 3.0)
            else:
                tail_us = waves * units * (2.2 if swiglu else 1.4)
            t = main_us + tail_us
            if best is None or t < best[0] - 1e-9:
                best = (t, bn, s_eff)
    if best is None:
        return pick_bn(n, mt), 1, 1
    return best[1], mt, best[2]


def max_fixup_splits(bn: int, mt: int, swiglu: bool) -> int:
    """Largest split-K factor the in-kernel fix-up takes (mirrors gemm_max_fixup_splits in
    csrc/kernels/gemm_bf16.cu): one split's share of an output unit is 16 KB (32 KB with the SwiGLU
    epilogue at bn >= 128) and all of them are landed in the operand ring together."""
    stages = {(2, 64): 5, (2, 128): 4, (2, 256): 3, (1, 64): 8, (1, 128): 6, (1, 256): 4}[(mt, bn)]
    ring = stages * (mt * 128 * 64 * 2 + bn * 64 * 2)
    acc_cols = (128 if bn >= 128 else bn) if swiglu else 64
    return min(32, ring // (acc_cols * 256))


_gemm_ws: dict[int, tuple[torch.Tensor, torch.Tensor]] = {}
GEMM_WS_BYTES = 48 << 20
GEMM_WS_TICKETS = 4096


def gemm_workspace(device) -> tuple[torch.Tensor, torch.Tensor]:
    """Per-device scratch of the split-K fix-up: bf16 partial tiles and their tickets (allocated
    once, so CUDA graphs can capture launches that use it)."""
    dev = torch.device(device)
    key = dev.index if dev.index is not None else torch.cuda.current_device()
    if key not in _gemm_ws:
        _gemm_ws[key] = (torch.empty(GEMM_WS_BYTES // 2, dtype=torch.bfloat16, device=dev),
                         torch.zeros(GEMM_WS_TICKETS, dtype=torch.int32, device=dev))
    return _gemm_ws[key]


def gemm(a: torch.Tensor, w: torch.Tensor, *, out: Optional[torch.Tensor] = None,
         epi: int = EPI_STORE_BF16, bias: Optional[torch.Tensor] = None,
         dst_ptrs: Sequence[int] = (), arrive_ptrs: Sequence[int] = (),
         done_ticket: Optional[torch.Tensor] = None, reset_on_done: Optional[torch.Tensor] = None,
         rows_per_owner: int = 0, group_counts: Optional[torch.Tensor] = None,
         row_meta: Optional[torch.Tensor] = None, ag_flags: Optional[torch.Tensor] = None,
         ag_expected: int = 0, ag_rows_per_src: int = 0, ag_ticket: Optional[torch.Tensor] = None,
         bn: int = 0, splits: int = 1, act: int = 0, m_tiles: int = 0,
         dst_ld: int = 0, my_rank: int = 0, mt: int = 1, fixup: Optional[bool] = None,
         trace: Optional[torch.Tensor] = None, wide_boxes: bool = True,
         sfa: Optional[torch.Tensor] = None, sfb: Optional[torch.Tensor] = None,
         a_gscale: Optional[torch.Tensor] = None, w_gscale: Optional[torch.Tensor] = None) -> Optional[torch.Tensor]:
    """tcgen05 GEMM  out = a @ w^T  (bf16 in, fp32 accumulate). See csrc/kernels/gemm_bf16.cu.
    `mt` = 2 keeps 256 rows with one CTA per weight tile; `splits` > 1 with a store / SwiGLU / slab
    epilogue combines the split partial tiles inside the kernel (`fixup`, default on for those).
    With `sfa` / `sfb` the operands are NVFP4: `a` and `w` hold e2m1 values packed two per byte
    ([.., K / 2] uint8, see quant_act_nvfp4 / Nvfp4Weight) and the product runs on the block-scaled
    fp4 tensor-core path (128 x 128 tiles); `a_gscale` [rows] and `w_gscale` [groups] multiply the rows."""
    M = a.shape[-2]
    tiled = w.dim() == 4  # tile-major weight from tile_weight()
    N = w.shape[0] * 128 if tiled else w.shape[-2]
    if sfa is not None:
        bn, mt, fixup = 128, 1, False
        if splits > 1 and epi != EPI_RED_F32:
            splits = 1
    if bn == 0:
        bn = pick_bn(N, (M + 127) // 128)
    if out is None and epi not in (EPI_RED_F32, EPI_SLAB_BF16):
        n_out = N // 2 if epi == EPI_SWIGLU_BF16 else N
        dt = torch.float32 if epi == EPI_STORE_F32 else torch.bfloat16
        out = torch.empty(*a.shape[:-1], n_out, dtype=dt, device=a.device)
    if fixup is None:
        fixup = splits > 1 and epi != EPI_RED_F32
    if fixup and splits > 1:
        # the launch must be one wave (the splits of a tile wait for each other) and the partial
        # slabs of one output unit must fit the operand ring
        K = a.shape[-1]
        kb = (K + 63) // 64
        per = -(-kb // min(splits, kb))
        s_eff = -(-kb // per)
        tiles = -(-N // bn) * -(-M // (128 * mt))
        cap = max_fixup_splits(bn, mt, epi == EPI_SWIGLU_BF16)
        if tiles * s_eff > sm_count(a.device) or s_eff > cap:
            raise ValueError(f"gemm: {tiles} tiles x {s_eff} splits do not fit one wave of {sm_count(a.device)} SMs "
                             f"or exceed the fix-up limit of {cap} splits")
    ws, tk = gemm_workspace(a.device) if fixup and splits > 1 else (None, None)
    _ext().gemm_bf16(a, w, epi, out, bias, list(dst_ptrs), list(arrive_ptrs), done_ticket,
                     reset_on_done, rows_per_owner, group_counts, row_meta, ag_flags, ag_expected,
                     ag_rows_per_src, ag_ticket, status_word(a.device), bn, splits, act, m_tiles, dst_ld,
                     my_rank, 1 if tiled else 0, mt, ws, tk, SPIN_LIMIT, trace, 1 if wide_boxes else 0, sfa, sfb, a_gscale, w_gscale)
    _bump()
    return out


# ---------------------------------------------------------------------------------------- NVFP4
E2M1_VALUES = (0.0, 0.5, 1.0, 1.5, 2.0, 3.0, 4.0, 6.0)


def _sf_atoms(scales: torch.Tensor) -> torch.Tensor:
    """[rows, K/16] uint8 block scales -> the 512-byte atom layout the tensor cores read:
    [row tile of 128][K / 64][(row % 32) * 16 + (row / 32 % 4) * 4 + (k / 16 % 4)]. Rows are padded
    to a multiple of 128 with zero scales (and K / 16 to a multiple of 4)."""
    rows, nb = scales.shape
    rp, nbp = (rows + 127) // 128 * 128, (nb + 3) // 4 * 4
    s = torch.zeros(rp, nbp, dtype=torch.uint8, device=scales.device)
    s[:rows, :nb] = scales
    s = s.view(rp // 128, 4, 32, nbp // 4, 4)          # tile, row / 32, row % 32, chunk, k / 16 % 4
    return s.permute(0, 3, 2, 1, 4).contiguous().view(-1)


class Nvfp4Weight:
    """A weight matrix (or a stack of expert matrices) in the layout of the block-scaled fp4 GEMM:
    `q` [.., N, K / 2] uint8 (e2m1, even element in the low nibble), `sf` scale atoms, `gscale`
    [groups] fp32 second-level scale. Built from GGUF NVFP4 blocks (`from_gguf_blocks`: the file's
    e4m3 micro-scales and nibbles are kept bit for bit, only re-ordered) or by quantising a float
    matrix (`from_float`)."""

    def __init__(self, q: torch.Tensor, sf: torch.Tensor, gscale: torch.Tensor, n: int, k: int):
        self.q, self.sf, self.gscale, self.n, self.k = q, sf, gscale, n, k

    @property
    def groups(self) -> int:
        return self.q.shape[0] if self.q.dim() == 3 else 1

    @staticmethod
    def from_gguf_blocks(raw: torch.Tensor, n: int, k: int, groups: int = 1) -> "Nvfp4Weight":
        """raw: uint8 GGUF NVFP4 blocks of 16 bytes (byte 0 = e4m3 scale, bytes 1..8 = nibbles with
        element i in the low and element i + 8 in the high nibble), [groups * n * k / 16, 16]."""
        b = raw.view(groups * n, k // 16, 16)
        qs = b[:, :, 1:9]
        el = torch.cat([qs & 0xF, qs >> 4], dim=-1)                      # elements 0..15 of every block
        q = (el[..., 0::2] | (el[..., 1::2] << 4)).reshape(groups, n, k // 2).contiguous()
        sc = b[:, :, 0].reshape(groups, n, k // 16)
        sf = torch.cat([_sf_atoms(sc[g]) for g in range(groups)])
        gs = torch.ones(groups, dtype=torch.float32, device=raw.device)
        return Nvfp4Weight(q if groups > 1 else q[0], sf, gs, n, k)

    @staticmethod
    def from_float(w: torch.Tensor) -> "Nvfp4Weight":
        """Quantises [N, K] or [G, N, K] float weights: per 16 values an e4m3 scale = amax / 6 relative
        to the matrix-wide second-level scale amax_matrix / (448 * 6); values to the nearest e2m1."""
        w3 = w if w.dim() == 3 else w[None]
        G, N, K = w3.shape
        wf = w3.float()
        gs = (wf.abs().amax(dim=(1, 2)) / (448.0 * 6.0)).clamp_min(1e-30)
        blk = wf.view(G, N, K // 16, 16)
        want = (blk.abs().amax(-1) / 6.0 / gs[:, None, None]).clamp_max(448.0)
        sc8 = want.to(torch.float8_e4m3fn)
        sd = sc8.float()
        bump = (sd < want) & (sc8.view(torch.uint8) < 0x7E)              # round the scale up, never down
        sc8 = torch.where(bump, (sc8.view(torch.uint8) + 1).view(torch.float8_e4m3fn), sc8)
        sd = sc8.float() * gs[:, None, None]
        y = blk / sd.clamp_min(1e-30)[..., None]
        lv = torch.tensor(E2M1_VALUES, device=w.device)
        code = (y.abs()[..., None] - lv).abs().argmin(-1).to(torch.uint8) | ((y < 0).to(torch.uint8) << 3)
        code = code.view(G, N, K)
        q = (code[..., 0::2] | (code[..., 1::2] << 4)).contiguous()
        sf = torch.cat([_sf_atoms(sc8.view(torch.uint8)[g]) for g in range(G)])
        return Nvfp4Weight(q if w.dim() == 3 else q[0], sf, gs.float(), N, K)

    def dequant(self) -> torch.Tensor:
        """fp32 values of the packed matrix (test oracle)."""
        q3 = self.q if self.q.dim() == 3 else self.q[None]
        G, N, _ = q3.shape
        K = self.k
        lv = torch.tensor(E2M1_VALUES, device=q3.device)
        code = torch.stack([q3 & 0xF, q3 >> 4], -1).view(G, N, K)
        val = lv[(code & 7).long()] * torch.where((code & 8) != 0, -1.0, 1.0)
        rp, ch = (N + 127) // 128 * 128, (K // 16 + 3) // 4
        sf = self.sf.view(G, rp // 128, ch, 32, 4, 4).permute(0, 1, 4, 3, 2, 5).reshape(G, rp, ch * 4)[:, :N, :K // 16]
        sc = sf.contiguous().view(torch.float8_e4m3fn).float()
        out = val.view(G, N, K // 16, 16) * sc[..., None] * self.gscale.view(G, 1, 1, 1)
        out = out.view(G, N, K)
        return out if self.q.dim() == 3 else out[0]


def quant_act_nvfp4(x: torch.Tensor, bufs=None, group_counts: Optional[torch.Tensor] = None, *,
                    ag_flags: Optional[torch.Tensor] = None, ag_expected: int = 0,
                    ag_ticket: Optional[torch.Tensor] = None):
    """bf16 [rows, K] or [G, cap, K] -> (q [.., K / 2] uint8, scale atoms, gscale [rows] fp32) for the
    NVFP4 GEMM. `bufs` = preallocated (q, sf, gscale) flat buffers (CUDA-graph friendly). With
    `ag_flags` the kernel first waits (bounded) until every source rank has signalled that its rows
    (an MoE dispatch into the slab) and the per-group counts are complete."""
    K = x.shape[-1]
    rows = x.numel() // K
    tiles = (rows + 127) // 128
    if bufs is None:
        q = torch.empty(*x.shape[:-1], K // 2, dtype=torch.uint8, device=x.device)
        sf = torch.zeros(tiles * (K // 64) * 512, dtype=torch.uint8, device=x.device)
        gs = torch.ones(rows, dtype=torch.float32, device=x.device)
    else:
        q = bufs[0][:rows * K // 2].view(*x.shape[:-1], K // 2)
        sf = bufs[1][:tiles * (K // 64) * 512]
        gs = bufs[2][:rows]
    _ext().quant_act_nvfp4(x, q, sf, gs, group_counts, ag_flags, ag_expected, ag_ticket, status_word(x.device),
                           SPIN_LIMIT)
    _bump()
    return q, sf, gs


def dequant_act_nvfp4(q: torch.Tensor, sf: torch.Tensor, gs: torch.Tensor) -> torch.Tensor:
    """fp32 values of quantised activation rows (test oracle); q is [rows, K / 2]."""
    rows, K = q.shape[0], q.shape[1] * 2
    w = Nvfp4Weight(q, sf, torch.ones(1, device=q.device), rows, K).dequant()
    return w * gs[:rows, None]


def quant_weight_fp8_block(w: torch.Tensor) -> tuple[torch.Tensor, torch.Tensor]:
    """[N, K] float weight -> (e4m3 [N, K], fp32 scales [ceil(N/128), ceil(K/128)]), one scale per
    128 x 128 block (amax / 448). Runs wherever `w` lives; a load-time transform."""
    N, K = w.shape
    nb, kb = (N + 127) // 128, (K + 127) // 128
    wp = torch.zeros(nb * 128, kb * 128, dtype=torch.float32, device=w.device)
    wp[:N, :K] = w.float()
    blk = wp.view(nb, 128, kb, 128)
    scale = blk.abs().amax(dim=(1, 3)).clamp_min(1e-10) / 448.0
    q = (blk / scale[:, None, :, None]).view(nb * 128, kb * 128)[:N, :K]
    return q.to(torch.float8_e4m3fn).contiguous(), scale.contiguous()


def quant_act_fp8(x: torch.Tensor, q: Optional[torch.Tensor] = None, sa_t: Optional[torch.Tensor] = None, *,
                  ag_flags: Optional[torch.Tensor] = None, ag_expected: int = 0, ag_rows_per_src: int = 0,
                  ag_ticket: Optional[torch.Tensor] = None) -> tuple[torch.Tensor, torch.Tensor]:
    """bf16 [M, K] -> (e4m3 [M, K], transposed 1 x 128 scales [ceil(K/128), M]). With `ag_flags` the
    kernel first waits (bounded) until the peers have pushed the rows it reads (all-gather consumer)."""
    M, K = x.shape
    if q is None:
        q = torch.empty(M, K, dtype=torch.float8_e4m3fn, device=x.device)
    if sa_t is None:
        sa_t = torch.empty((K + 127) // 128, M, dtype=torch.float32, device=x.device)
    _ext().quant_act_fp8(x, q, sa_t, ag_flags, ag_expected, ag_rows_per_src, ag_ticket, status_word(x.device))
    _bump()
    return q, sa_t


def gemm_fp8_block(a8: torch.Tensor, sa_t: torch.Tensor, w8: torch.Tensor, sw: torch.Tensor, *,
                   out: Optional[torch.Tensor] = None, bias: Optional[torch.Tensor] = None,
                   slab_ptrs: Sequence[int] = (), arrive_ptrs: Sequence[int] = (),
                   done_ticket: Optional[torch.Tensor] = None, rows_per_owner: int = 0, my_rank: int = 0,
                   slab_ld: int = 0) -> Optional[torch.Tensor]:
    """Block-scaled fp8 GEMM on the tcgen05 f8 path. See csrc/kernels/gemm_fp8_block.cu. With
    `slab_ptrs` the epilogue is the reduce-scatter of a row-parallel projection (bf16 partial rows go
    to the row owner's receive slab, the last CTA signals the owners)."""
    if out is None and not slab_ptrs:
        out = torch.empty(a8.shape[0], w8.shape[0], dtype=torch.bfloat16, device=a8.device)
    _ext().gemm_fp8_block(a8, sa_t, w8, sw, out, bias, status_word(a8.device), list(slab_ptrs), list(arrive_ptrs),
                          done_ticket, rows_per_owner, my_rank, slab_ld)
    _bump()
    return out


def tile_weight(w: torch.Tensor) -> torch.Tensor:
    """[N, K] row-major -> tile-major [N/128, K/64, 128, 64] (a load-time transform): each TMA box of
    the weight stream becomes one contiguous 16 KB run. Needs N % 128 == 0 and K % 64 == 0; other
    shapes stay row-major (the GEMM takes either)."""
    N, K = w.shape
    if N % 128 or K % 64:
        return w
    return w.view(N // 128, 128, K // 64, 64).permute(0, 2, 1, 3).contiguous()


def untile_weight(w: torch.Tensor) -> torch.Tensor:
    if w.dim() != 4:
        return w
    nt, kt = w.shape[0], w.shape[1]
    return w.permute(0, 2, 1, 3).reshape(nt * 128, kt * 64)


def paged_decode(q, k_cache, v_cache, block_tables, seq_lens, pages_per_split, part_o, part_ml, out,
                 *, batch: int, max_splits: int, window: int = 0, scale: float,
                 page_ml: Optional[torch.Tensor] = None, block_mass: Optional[torch.Tensor] = None,
                 q8=None) -> None:
    """Paged split-KV decode attention + merge. With `page_ml` [B, max_blocks, Hq, 2] and `block_mass`
    [B, max_blocks] (fp32) the kernels also produce the softmax probability mass per KV block, summed
    over heads: the heavy-hitter score of H2O pruning (the reference accumulates it in its decode
    kernel too, oxide-backend-cuda/src/kernels/megakernel_ops.cu:577-617). `q8` = (int8 [B, Hq*D],
    scales, sums): the merge also writes the int8 view of `out` (see `finalize_norm`)."""
    q8t, q8d, q8s = q8 if q8 is not None else (None, None, None)
    _ext().paged_decode(q, k_cache, v_cache, block_tables, seq_lens, pages_per_split, part_o, part_ml,
                        out, batch, max_splits, window, scale, status_word(q.device) if CHECK_BOUNDS else None,
                        page_ml, block_mass, q8t, q8d, q8s)
    _bump(3 if page_ml is not None else 2)


# OXB_CHECKS=1: the attention kernels verify every block-table id against the pool size (a bad id is
# recorded in the status word and page 0 is read instead); costs ~4 % of the decode attention kernel.
CHECK_BOUNDS = os.environ.get("OXB_CHECKS", "0") != "0"


def paged_prefill(q, k_cache, v_cache, block_tables, tile_seq, tile_q0, q_start, q_lens, ctx_lens, out,
                  *, n_tiles: int, window: int = 0, scale: float) -> None:
    """Causal paged attention over ragged prefill chunks on 128-row query tiles (tcgen05 / TMEM,
    attn_prefill_tc.cu); `tile_q0` entries are multiples of 128."""
    _ext().paged_prefill_tc(q, k_cache, v_cache, block_tables, tile_seq, tile_q0, q_start, q_lens,
                            ctx_lens, out, n_tiles, window, scale, status_word(q.device))
    _bump()


def finalize_norm(*, rows: int, n: int, acc=None, rs_slab=None, n_slabs: int = 0, slab_stride: int = 0,
                  arrive=None, expected: int = 0, ticket=None,
                  residual_in=None, residual_out=None, bias=None, norm_w=None, eps: float = 1e-5,
                  w_offset: float = 0.0, out_ptrs: Sequence[int] = (), out_flag_ptrs: Sequence[int] = (),
                  out_row_off: int = 0, out_row_map=None, router_w=None, top_k: int = 0, experts_per_rank: int = 0,
                  routed_scale: float = 1.0, slab_ptrs: Sequence[int] = (), meta_ptrs: Sequence[int] = (),
                  cnt_ptrs: Sequence[int] = (), cap: int = 0, my_rank: int = 0, device=None, q8=None) -> None:
    """`q8` = (int8 [rows, n], fp32 scales [rows, n/32], fp32 sums [rows, n/32]): the kernel also writes
    the int8 view of its output rows (the numbers `quant_q8_1` would produce from them), so the integer
    GEMV that follows needs no quantiser launch."""
    q8t, q8d, q8s = q8 if q8 is not None else (None, None, None)
    _ext().finalize_norm(acc, rs_slab, n_slabs, slab_stride, arrive, expected, ticket, residual_in, residual_out, bias, norm_w, eps,
                         w_offset, list(out_ptrs), list(out_flag_ptrs), out_row_off, out_row_map, rows, n,
                         status_word(device), router_w, top_k, experts_per_rank, routed_scale,
                         list(slab_ptrs), list(meta_ptrs), list(cnt_ptrs), cap, my_rank, SPIN_LIMIT, q8t, q8d, q8s)
    _bump()


def rmsnorm(x: torch.Tensor, w: torch.Tensor, eps: float, *, residual: Optional[torch.Tensor] = None,
            residual_out: Optional[torch.Tensor] = None, out: Optional[torch.Tensor] = None,
            w_offset: float = 0.0) -> torch.Tensor:
    """out = RMSNorm(x [+ residual]) * (w + w_offset); optionally writes the sum to residual_out.

    Convenience wrapper over the finalize kernel; with a residual the second operand is passed
    through the kernel's fp32 accumulator input.
    """
    rows, n = x.shape
    if out is None:
        out = torch.empty_like(x)
    acc = None if residual is None else x.float()
    finalize_norm(rows=rows, n=n, acc=acc, residual_in=x if residual is None else residual,
                  residual_out=residual_out, norm_w=w, eps=eps, w_offset=w_offset,
                  out_ptrs=[out.data_ptr()], device=x.device)
    return out


def qkv_rope_append(*, acc_f32=None, qkv_bf16=None, bias=None, q_norm_w=None, k_norm_w=None,
                    norm_eps: float = 1e-6, norm_w_offset: float = 0.0, positions, slot_mapping,
                    inv_freq, rope_mscale: float = 1.0, q_out, k_cache, v_cache, m: int, hq: int,
                    hkv: int, d: int) -> None:
    _ext().qkv_rope_append(acc_f32, qkv_bf16, bias, q_norm_w, k_norm_w, norm_eps, norm_w_offset,
                           positions, slot_mapping, inv_freq, rope_mscale, q_out, k_cache, v_cache, m,
                           hq, hkv, d, status_word(q_out.device))
    _bump()


def swiglu(*, acc_f32=None, gu_bf16=None, out, m: int, i: int, act: int = 0, q8=None) -> None:
    """`q8` as in `finalize_norm`: the int8 view of `out` for the integer GEMV that follows."""
    q8t, q8d, q8s = q8 if q8 is not None else (None, None, None)
    _ext().swiglu(acc_f32, gu_bf16, out, m, i, act, q8t, q8d, q8s)
    _bump()


def embed_gather(tokens, table, out, scale: float = 1.0, vocab_start: int = 0) -> None:
    _ext().embed_gather(tokens, table, out, scale, vocab_start)
    _bump()


def cast_acc_bf16(acc, out, m: int, n: int, bias=None) -> None:
    _ext().cast_acc_bf16(acc, bias, out, m, n)
    _bump()


def fwht128(x) -> None:
    _ext().fwht128(x)
    _bump()


def kv_block_copy(k_cache, v_cache, src, dst) -> None:
    _ext().kv_block_copy(k_cache, v_cache, src, dst)
    _bump()


def softcap(logits, cap: float) -> None:
    _ext().softcap(logits, cap)
    _bump()


def gemm_packed(a: torch.Tensor, qtype: int, qw: torch.Tensor, n: int, out: torch.Tensor, *, epi: int = EPI_STORE_BF16,
                mt: int = 1, splits: int = 1, bias: Optional[torch.Tensor] = None) -> None:
    """out[:M, :n] (+)= a @ W^T for a GGUF-packed weight (`qw` = the block bytes of n rows, block type
    `qtype` from INT8_MMVQ_CODES): the tcgen05 GEMM with four extra warps that unpack each 128 x 64
    weight tile into the bf16 operand stage, so the weights stay packed in HBM and no bf16 copy or
    scratch expansion exists (reference: the MMQ kernels, quant_gemm_mmq.cu:191-409, :624-788).
    `epi` EPI_RED_F32 adds into a zeroed fp32 `out` and may split K."""
    _ext().gemm_packed(a, qw, int(qtype), int(n), out, epi, mt, splits, bias, status_word(a.device), SPIN_LIMIT)
    _bump()


def alloc_mapped_host(n_words: int):
    """Page-locked host memory mapped into the device's address space: (int64 host tensor, device
    address). Kernels post results there and the host polls them without a stream synchronisation."""
    return _ext().alloc_mapped_host(int(n_words))


def advance_decode_step(s, sampled, mailbox_dev: int, step_counter, *, rows: int, ring: int) -> None:
    """In-graph step advance (see csrc/kernels/fused_ops.cuh, AdvanceStepParams): rewrites the first
    `rows` rows of the step descriptor `s` for the next decode step from the sampled ids and posts
    the ids to the mapped-host ring at `mailbox_dev`."""
    _ext().advance_decode_step(s.token_ids, s.positions, s.slot_mapping, s.seq_lens, s.block_tables, sampled,
                               int(mailbox_dev), step_counter, rows, ring, status_word(sampled.device))
    _bump()


def mmvq(qtype: int, w, x, out, *, n: int, k: int, bias=None, add: bool = False, xq=None) -> None:
    """Small-batch quantised GEMV. `xq` = (int8 [M, K], scales [M, K/32], sums [M, K/32]) from
    `quant_q8_1(x)`: the block types of `INT8_MMVQ_CODES` then take the integer dot-product (dp4a)
    path, the others expand their weights to fp32."""
    q8, xd, xs = xq if xq is not None else (None, None, None)
    _ext().mmvq(qtype, w, x, bias, out, n, k, add, q8, xd, xs)
    _bump()


# GGUF type codes with an integer (dp4a) GEMV: Q4_0 Q4_1 Q5_0 Q5_1 Q8_0 Q4_K Q5_K Q6_K
INT8_MMVQ_CODES = frozenset((2, 3, 6, 7, 8, 12, 13, 14))


def mmvq_mixed(parts: Sequence, x, out, *, k: int, xq) -> None:
    """One GEMV launch over stacked packed matrices of different block types that share K:
    `parts` = [(type code, packed bytes, rows), ...] (at most four), out[:, :sum(rows)]. This is how
    the Q|K|V and gate|up projections of a mixed-precision GGUF file (Q4_K_M keeps attn_v in Q6_K)
    stay on one launch (reference: gemv_qkv_mixed_*, quant_gemv_kquants.cu:399-917)."""
    q8, xd, xs = xq
    _ext().mmvq_mixed([int(c) for c, _, _ in parts], [w for _, w, _ in parts], [int(n) for _, _, n in parts],
                      x, out, k, q8, xd, xs)
    _bump()


def gemv(x: torch.Tensor, w: torch.Tensor, out: torch.Tensor, *, bias=None, swiglu: bool = False, act: int = 0) -> None:
    """out[:M] = x @ w^T for M <= 8 rows (single-GPU latency-mode decoding); `w` row-major or
    tile-major. `swiglu`: w holds gate|up interleaved by 32 rows and out gets act(gate) * up."""
    _ext().gemv_bf16(x, w, out, bias, swiglu, act)
    _bump()


def quant_q8_1(x: torch.Tensor, bufs=None):
    """bf16 [M, K] -> (int8 [M, K], fp32 scales [M, K/32], fp32 block sums [M, K/32]); `bufs` are
    preallocated flat buffers (int8, fp32, fp32) to view into (CUDA-graph friendly)."""
    M, K = x.shape
    if bufs is None:
        q8 = torch.empty(M, K, dtype=torch.int8, device=x.device)
        xd = torch.empty(M, K // 32, dtype=torch.float32, device=x.device)
        xs = torch.empty(M, K // 32, dtype=torch.float32, device=x.device)
    else:
        q8 = bufs[0][:M * K].view(M, K)
        xd = bufs[1][:M * (K // 32)].view(M, K // 32)
        xs = bufs[2][:M * (K // 32)].view(M, K // 32)
    _ext().quant_q8_1(x, q8, xd, xs)
    _bump()
    return q8, xd, xs


def dequant_rows(qtype: int, w, out, *, n_src_rows: int, k: int, row_ids=None, scale: float = 1.0) -> None:
    _ext().dequant_rows(qtype, w, row_ids, out, n_src_rows, k, scale)
    _bump()


def sample(logits, out_tokens, *, temperature=None, top_k=None, top_p=None, min_p=None, seeds=None,
           counters=None, allow_mask=None, out_logit=None) -> None:
    _ext().sample(logits, temperature, top_k, top_p, min_p, seeds, counters, allow_mask, out_tokens,
                  out_logit)
    _bump()


def argmax(logits, out, out_val=None) -> None:
    _ext().argmax(logits, out, out_val)
    _bump()


def argmax_combine(vals, idxs, out) -> None:
    _ext().argmax_combine(vals, idxs, out)
    _bump()


def argmax_exchange(logits, out, *, vocab_start: int, tab_ptrs: Sequence[int], max_rows: int, my_rank: int,
                    slot: int) -> None:
    """Vocab-parallel greedy sampling without a library collective: every rank stores (value, index) of
    its shard's argmax as one 64-bit word per row into every rank's table over peer memory (the word is
    its own arrival flag) and then combines the words of all ranks. `slot` alternates 0 / 1 per call."""
    _ext().argmax_exchange(logits, vocab_start, list(tab_ptrs), max_rows, my_rank, slot, out, status_word(logits.device),
                           SPIN_LIMIT)
    _bump(2)
