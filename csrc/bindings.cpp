// Python bindings of the sm_100a kernels (torch extension `oxb_cuda`).
// Every function launches on torch's current CUDA stream and allocates nothing unless noted.
#include <ATen/cuda/CUDAContext.h>
#include <c10/cuda/CUDAGuard.h>
#include <cuda.h>
#include <cuda_runtime.h>
#include <pybind11/stl.h>
#include <torch/extension.h>

#include <string>
#include <cstring>
#include <vector>

#include "common/device_info.h"
#include "common/tma_host.h"
#include "kernels/attn.cuh"
#include "kernels/fused_ops.cuh"
#include "kernels/gemm_bf16.cuh"
#include "kernels/gemm_fp8_block.cuh"
#include "kernels/gemv_bf16.cuh"
#include "kernels/quant_ops.cuh"
#include "kernels/sampler.cuh"

namespace py = pybind11;
using torch::Tensor;

namespace {

cudaStream_t cur_stream() { return at::cuda::getCurrentCUDAStream().stream(); }

void check_launch(const char* what) {
  cudaError_t e = cudaGetLastError();
  TORCH_CHECK(e == cudaSuccess, "oxb: launch of ", what, " failed: ", cudaGetErrorString(e));
}

const __nv_bfloat16* bf16_ptr(const c10::optional<Tensor>& t) {
  if (!t.has_value() || !t->defined()) return nullptr;
  TORCH_CHECK(t->scalar_type() == torch::kBFloat16 && t->is_cuda(), "expected a CUDA bf16 tensor");
  return reinterpret_cast<const __nv_bfloat16*>(t->data_ptr());
}
template <typename T>
T* opt_ptr(const c10::optional<Tensor>& t) {
  if (!t.has_value() || !t->defined()) return nullptr;
  return reinterpret_cast<T*>(t->data_ptr());
}

// ---------------------------------------------------------------------------------------------
// GEMM
// ---------------------------------------------------------------------------------------------
// a: [M, K] or [G, cap, K] bf16 (K contiguous);  w: [N, K] or [G, N, K] bf16.
void gemm_bf16(const Tensor& a, const Tensor& w, int64_t epi, const c10::optional<Tensor>& out,
               const c10::optional<Tensor>& bias, const std::vector<int64_t>& dst_ptrs,
               const std::vector<int64_t>& arrive_ptrs, const c10::optional<Tensor>& done_ticket,
               const c10::optional<Tensor>& reset_on_done, int64_t rows_per_owner,
               const c10::optional<Tensor>& group_counts, const c10::optional<Tensor>& row_meta,
               const c10::optional<Tensor>& ag_flags, int64_t ag_expected, int64_t ag_rows_per_src,
               const c10::optional<Tensor>& ag_ticket, const Tensor& status, int64_t bn,
               int64_t splits, int64_t act, int64_t m_tiles_override, int64_t dst_ld,
               int64_t my_rank, int64_t b_tiled, int64_t mt, const c10::optional<Tensor>& ws,
               const c10::optional<Tensor>& ws_tickets, int64_t spin_limit,
               const c10::optional<Tensor>& trace, int64_t wide_boxes, const c10::optional<Tensor>& sfa,
               const c10::optional<Tensor>& sfb, const c10::optional<Tensor>& a_gscale,
               const c10::optional<Tensor>& w_gscale) {
  TORCH_CHECK(a.is_cuda() && w.is_cuda(), "gemm_bf16: CUDA tensors required");
  // NVFP4: a and w hold e2m1 values packed two per byte ([.., K / 2] uint8) with block scales sfa / sfb
  const bool fp4 = sfa.has_value() && sfa->defined();
  if (fp4) {
    TORCH_CHECK(a.scalar_type() == torch::kUInt8 && w.scalar_type() == torch::kUInt8 && sfb.has_value() &&
                    sfb->defined() && sfa->scalar_type() == torch::kUInt8 && sfb->scalar_type() == torch::kUInt8,
                "gemm (nvfp4): packed uint8 operands and uint8 scale atoms required");
  } else {
    TORCH_CHECK(a.scalar_type() == torch::kBFloat16 && w.scalar_type() == torch::kBFloat16,
                "gemm_bf16: bf16 operands required");
  }
  TORCH_CHECK(a.stride(-1) == 1 && w.stride(-1) == 1, "gemm_bf16: K must be contiguous");
  TORCH_CHECK(b_tiled == 0 || !(group_counts.has_value() && group_counts->defined()),
              "gemm_bf16: grouped GEMMs take row-major weights");
  const bool grouped3d = a.dim() == 3;
  const bool tiled = b_tiled != 0;
  if (tiled) {
    TORCH_CHECK(a.dim() == 2 && w.dim() == 4 && w.size(2) == 128 && w.size(3) == 64 && w.is_contiguous(),
                "gemm_bf16: tile-major weights are [N/128, K/64, 128, 64] contiguous, 2-D activations");
  } else {
    TORCH_CHECK(w.dim() == a.dim(), "gemm_bf16: a and w must have the same rank");
  }
  const int64_t G = grouped3d ? a.size(0) : 1;
  const int64_t M = grouped3d ? a.size(1) : a.size(0);
  // K in operand elements of 2 bytes for the tile arithmetic below: a row of the packed fp4 operands
  // has K / 2 bytes = K / 4 such units, and one 128-byte k block covers 256 fp4 values
  const int64_t K = fp4 ? a.size(-1) / 2 : a.size(-1);
  const int64_t N = tiled ? w.size(0) * 128 : (grouped3d ? w.size(1) : w.size(0));
  TORCH_CHECK(tiled ? w.size(1) * 64 == K : w.size(-1) == a.size(-1), "gemm_bf16: K mismatch");
  TORCH_CHECK(K % 8 == 0, "gemm_bf16: K must be a multiple of 8 (16-byte TMA rows)");
  if (fp4) {
    TORCH_CHECK(!tiled && a.size(-1) % 128 == 0, "gemm (nvfp4): K must be a multiple of 256, row-major weights");
  }
  if (grouped3d) {
    TORCH_CHECK(w.size(0) == G, "gemm_bf16: group mismatch");
  }

  const uint64_t eb = fp4 ? 1 : 2;  // bytes per tensor element
  const uint64_t a_row = static_cast<uint64_t>(a.stride(-2)) * eb;
  const uint64_t w_row = tiled ? 128 : static_cast<uint64_t>(w.stride(-2)) * eb;
  const uint64_t a_grp = grouped3d ? static_cast<uint64_t>(a.stride(0)) * eb : a_row * M;
  const uint64_t w_grp = tiled ? 16384 : (grouped3d ? static_cast<uint64_t>(w.stride(0)) * eb : w_row * N);
  const int bn_i = bn == 64 ? 64 : (bn == 256 ? 256 : 128);
  // decode tiles (mt = 2): one copy per operand and stage instead of two 16 KB boxes each
  const bool wide = mt == 2 && !grouped3d && wide_boxes != 0;
  const CUtensorMapDataType dt = fp4 ? CU_TENSOR_MAP_DATA_TYPE_UINT8 : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16;
  const uint64_t k_inner = fp4 ? static_cast<uint64_t>(a.size(-1)) : static_cast<uint64_t>(K);  // elements of the map's type
  const uint32_t box_inner = fp4 ? 128 : 64;
  CUtensorMap tmA = oxb::make_tma_map(a.data_ptr(), dt, static_cast<int>(eb), 3, k_inner, M, G,
                                      a_row, a_grp, box_inner, wide ? 256 : 128, 1, CU_TENSOR_MAP_SWIZZLE_128B);
  const uint64_t total_kb_u = static_cast<uint64_t>((K + 63) / 64);
  CUtensorMap tmB =
      (tiled && wide && bn_i == 256)
          ? oxb::make_tma_map(w.data_ptr(), CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, 4, 64, 128, total_kb_u, 128,
                              16384, 64, 128, 1, CU_TENSOR_MAP_SWIZZLE_128B, static_cast<uint64_t>(w.size(0)),
                              16384 * total_kb_u, 2)
      : tiled ? oxb::make_tma_map(w.data_ptr(), CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, 3, 64, 128,
                                static_cast<uint64_t>(w.size(0) * w.size(1)), 128, 16384, 64,
                                bn_i < 128 ? bn_i : 128, 1, CU_TENSOR_MAP_SWIZZLE_128B)
            : oxb::make_tma_map(w.data_ptr(), dt, static_cast<int>(eb), 3, k_inner, N, G, w_row,
                                w_grp, box_inner, bn_i, 1, CU_TENSOR_MAP_SWIZZLE_128B);

  oxb::GemmParams p{};
  p.M = static_cast<int>(M);
  p.N = static_cast<int>(N);
  p.K = static_cast<int>(K);
  const int total_kb = static_cast<int>((K + 63) / 64);
  int s = static_cast<int>(splits < 1 ? 1 : splits);
  if (s > total_kb) s = total_kb;
  p.kb_per_split = (total_kb + s - 1) / s;
  s = (total_kb + p.kb_per_split - 1) / p.kb_per_split;
  p.epi = static_cast<int>(epi);
  p.act = static_cast<int>(act);
  p.b_tiled = static_cast<int>(b_tiled);
  p.wide_boxes = wide ? 1 : 0;
  p.spin_limit = static_cast<uint32_t>(spin_limit > 0 ? spin_limit : 0);
  if (fp4) {
    TORCH_CHECK(bn == 128 && mt != 2, "gemm (nvfp4): 128 x 128 tiles");
    p.kind = 1;
    p.kb_total = static_cast<int>(a.size(-1) / 128);
    const int64_t row_tiles = ((grouped3d ? a.size(1) : M) + 127) / 128;
    TORCH_CHECK(!grouped3d || a.size(1) % 128 == 0, "gemm (nvfp4): grouped slabs need a multiple of 128 rows per group");
    TORCH_CHECK(sfa->numel() >= G * row_tiles * p.kb_total * 2048 && sfa->is_contiguous(), "gemm (nvfp4): sfa too small");
    TORCH_CHECK(sfb->numel() >= G * ((N + 127) / 128) * p.kb_total * 2048 && sfb->is_contiguous(), "gemm (nvfp4): sfb too small");
    p.sfa = sfa->data_ptr<uint8_t>();
    p.sfb = sfb->data_ptr<uint8_t>();
    p.sfa_group_tiles = row_tiles;
    if (a_gscale.has_value() && a_gscale->defined()) {
      TORCH_CHECK(a_gscale->scalar_type() == torch::kFloat32 && a_gscale->numel() >= G * M, "gemm (nvfp4): a_gscale");
      p.a_gscale = a_gscale->data_ptr<float>();
      p.a_gs_stride = M;
    }
    if (w_gscale.has_value() && w_gscale->defined()) {
      TORCH_CHECK(w_gscale->scalar_type() == torch::kFloat32 && w_gscale->numel() >= G, "gemm (nvfp4): w_gscale");
      p.w_gscale = w_gscale->data_ptr<float>();
    }
  }
  if (trace.has_value() && trace->defined()) {
    TORCH_CHECK(trace->scalar_type() == torch::kInt64 && trace->numel() >= 8 * oxb::sm_count(),
                "gemm_bf16: trace must hold 8 int64 per SM");
    p.trace = reinterpret_cast<unsigned long long*>(trace->data_ptr());
  }
  const int mt_i = mt == 2 ? 2 : 1;
  const bool fixup = s > 1 && ws.has_value() && ws->defined() && epi != oxb::kEpiRedF32;
  const bool routed = epi == oxb::kEpiRedF32 || epi == oxb::kEpiSlabBf16;
  p.my_rank = static_cast<int>(my_rank);
  if (!routed) {
    TORCH_CHECK(out.has_value(), "gemm_bf16: out required for store epilogues");
    TORCH_CHECK(s == 1 || fixup, "gemm_bf16: split-K needs the fp32 reduction epilogue or a workspace");
    TORCH_CHECK(out->stride(-1) == 1, "gemm_bf16: out must be row-major");
    if (epi == oxb::kEpiStoreF32) {
      TORCH_CHECK(out->scalar_type() == torch::kFloat32, "gemm_bf16: fp32 out expected");
    } else {
      TORCH_CHECK(out->scalar_type() == torch::kBFloat16, "gemm_bf16: bf16 out expected");
    }
    p.C = out->data_ptr();
    p.ldc = out->stride(-2);
    p.c_group_stride = out->dim() == 3 ? out->stride(0) : 0;
  } else {
    TORCH_CHECK(epi == oxb::kEpiRedF32 || s == 1 || fixup,
                "gemm_bf16: the slab epilogue splits K only with a workspace");
    TORCH_CHECK(!dst_ptrs.empty() && dst_ptrs.size() <= oxb::kMaxRanks, "gemm_bf16: 1..8 owners");
    for (size_t i = 0; i < dst_ptrs.size(); ++i) p.dst[i] = reinterpret_cast<float*>(dst_ptrs[i]);
    for (size_t i = 0; i < arrive_ptrs.size() && i < oxb::kMaxRanks; ++i)
      p.arrive[i] = reinterpret_cast<uint32_t*>(arrive_ptrs[i]);
    p.n_owners = static_cast<int>(dst_ptrs.size());
    p.rows_per_owner = static_cast<int>(rows_per_owner > 0 ? rows_per_owner : M);
    p.dst_ld = dst_ld > 0 ? dst_ld : N;
  }
  if (epi == oxb::kEpiSwigluBf16) {
    TORCH_CHECK(N % bn_i == 0, "swiglu epilogue: N % BN must be 0");
  }
  p.bias = bf16_ptr(bias);
  p.done_ticket = opt_ptr<uint32_t>(done_ticket);
  if (reset_on_done.has_value() && reset_on_done->defined()) {
    p.reset_on_done = reinterpret_cast<uint32_t*>(reset_on_done->data_ptr());
    p.n_reset = static_cast<int>(reset_on_done->numel());
  }
  int m_tiles = static_cast<int>((M + 128 * mt_i - 1) / (128 * mt_i));
  if (group_counts.has_value() && group_counts->defined()) {
    TORCH_CHECK(mt_i == 1 && !fixup, "gemm_bf16: grouped GEMMs use 128-row tiles without the split-K fix-up");
    p.group_counts = reinterpret_cast<const uint32_t*>(group_counts->data_ptr());
    p.n_groups = static_cast<int>(G);
    TORCH_CHECK(m_tiles_override > 0, "gemm_bf16: grouped mode needs the m-tile bound");
    m_tiles = static_cast<int>(m_tiles_override);
    if (row_meta.has_value() && row_meta->defined()) {
      p.row_meta = reinterpret_cast<const oxb::RowMeta*>(row_meta->data_ptr());
      p.meta_group_stride = M;
    }
  } else {
    TORCH_CHECK(G == 1, "gemm_bf16: 3-D operands need group_counts");
  }
  if (ag_flags.has_value() && ag_flags->defined()) {
    TORCH_CHECK(ag_ticket.has_value(), "gemm_bf16: ag_ticket required with ag_flags");
    p.ag_flags = reinterpret_cast<const uint32_t*>(ag_flags->data_ptr());
    p.ag_n_src = static_cast<int>(ag_flags->numel());
    p.ag_expected = static_cast<uint32_t>(ag_expected);
    p.ag_rows_per_src = static_cast<int>(ag_rows_per_src);
    p.ag_ticket = reinterpret_cast<uint32_t*>(ag_ticket->data_ptr());
  }
  p.status = reinterpret_cast<int*>(status.data_ptr());
  p.m_tiles = m_tiles;
  p.splits = s;
  if (fixup) {
    TORCH_CHECK(ws_tickets.has_value() && ws_tickets->defined(), "gemm_bf16: ws_tickets required with ws");
    const int n_work = static_cast<int>((N + bn_i - 1) / bn_i) * m_tiles * s;
    TORCH_CHECK(n_work <= oxb::sm_count(),
                "gemm_bf16: split-K with the in-kernel fix-up needs one work item per SM at most (", n_work, ")");
    TORCH_CHECK(s <= oxb::gemm_max_fixup_splits(bn_i, mt_i, epi == oxb::kEpiSwigluBf16),
                "gemm_bf16: too many splits for the in-kernel fix-up of this tile shape (", s, ")");
    TORCH_CHECK(ws->is_cuda() && ws->is_contiguous() &&
                    static_cast<size_t>(ws->numel() * ws->element_size()) >=
                        oxb::gemm_ws_bytes(static_cast<int>(M), static_cast<int>(N), bn_i, mt_i, s),
                "gemm_bf16: split-K workspace too small");
    TORCH_CHECK(ws_tickets->numel() >= oxb::gemm_ws_tickets(static_cast<int>(M), static_cast<int>(N), bn_i, mt_i),
                "gemm_bf16: too few split-K tickets");
    p.ws = reinterpret_cast<__nv_bfloat16*>(ws->data_ptr());
    p.ws_tickets = reinterpret_cast<uint32_t*>(ws_tickets->data_ptr());
  }
  oxb::launch_gemm_bf16(tmA, tmB, p, bn_i, mt_i, cur_stream());
  check_launch("gemm_bf16");
}

// out[M, N] (+)= a[M, K] (bf16) x W^T with W kept as GGUF blocks: [N rows] of packed bytes of block type
// `qtype`, unpacked tile by tile inside the GEMM (no bf16 copy of the weights, no scratch pass).
// epi: store bf16 / store fp32 (splits == 1) or fp32 reduction into `out` (any splits; zero it first).
void gemm_packed(const Tensor& a, const Tensor& qw, int64_t qtype, int64_t N, const Tensor& out, int64_t epi,
                 int64_t mt, int64_t splits, const c10::optional<Tensor>& bias, const Tensor& status,
                 int64_t spin_limit) {
  TORCH_CHECK(a.is_cuda() && a.scalar_type() == torch::kBFloat16 && a.dim() == 2 && a.stride(1) == 1,
              "gemm_packed: bf16 [M, K] activations");
  TORCH_CHECK(qw.is_cuda() && qw.scalar_type() == torch::kUInt8 && qw.is_contiguous(), "gemm_packed: packed uint8 weights");
  TORCH_CHECK(oxb::mmvq_has_int8_path(static_cast<int>(qtype)), "gemm_packed: no in-kernel expansion for GGUF type ", qtype);
  const int64_t M = a.size(0), K = a.size(1);
  TORCH_CHECK(K % 256 == 0, "gemm_packed: K must be a multiple of 256");
  const long long row_bytes = oxb::quant_row_bytes(static_cast<int>(qtype), K);
  TORCH_CHECK(row_bytes > 0 && qw.numel() >= row_bytes * N, "gemm_packed: weight buffer too small");
  const bool k16 = qtype == 12 || qtype == 13;  // Q4_K / Q5_K rows are read with 16-byte loads
  TORCH_CHECK(reinterpret_cast<uintptr_t>(qw.data_ptr()) % 16 == 0 && (!k16 || row_bytes % 16 == 0),
              "gemm_packed: weight alignment");
  TORCH_CHECK(epi == oxb::kEpiStoreBf16 || epi == oxb::kEpiStoreF32 || epi == oxb::kEpiRedF32, "gemm_packed: epilogue");
  TORCH_CHECK(out.is_cuda() && out.dim() == 2 && out.stride(1) == 1 && out.size(0) >= M && out.size(1) >= N,
              "gemm_packed: out [M, N] row-major");
  const int mt_i = mt == 2 ? 2 : 1;
  const uint64_t a_row = static_cast<uint64_t>(a.stride(0)) * 2;
  CUtensorMap tmA = oxb::make_tma_map(a.data_ptr(), CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, 3, static_cast<uint64_t>(K),
                                      static_cast<uint64_t>(M), 1, a_row, a_row * M, 64, 128, 1,
                                      CU_TENSOR_MAP_SWIZZLE_128B);
  oxb::GemmParams p{};
  p.M = static_cast<int>(M);
  p.N = static_cast<int>(N);
  p.K = static_cast<int>(K);
  p.kind = 2;
  p.qw = qw.data_ptr<uint8_t>();
  p.q_row_bytes = row_bytes;
  p.q_type = static_cast<int>(qtype);
  const int total_kb = static_cast<int>(K / 64);
  int s = static_cast<int>(splits < 1 ? 1 : splits);
  if (s > total_kb) s = total_kb;
  p.kb_per_split = (total_kb + s - 1) / s;
  s = (total_kb + p.kb_per_split - 1) / p.kb_per_split;
  p.splits = s;
  p.epi = static_cast<int>(epi);
  p.spin_limit = static_cast<uint32_t>(spin_limit > 0 ? spin_limit : 0);
  p.bias = bf16_ptr(bias);
  p.m_tiles = static_cast<int>((M + 128 * mt_i - 1) / (128 * mt_i));
  p.status = reinterpret_cast<int*>(status.data_ptr());
  if (epi == oxb::kEpiRedF32) {
    TORCH_CHECK(out.scalar_type() == torch::kFloat32, "gemm_packed: fp32 out for the reduction epilogue");
    p.dst[0] = out.data_ptr<float>();
    p.n_owners = 1;
    p.rows_per_owner = static_cast<int>(M);
    p.dst_ld = out.stride(0);
  } else {
    TORCH_CHECK(s == 1, "gemm_packed: split-K needs the fp32 reduction epilogue");
    TORCH_CHECK(out.scalar_type() == (epi == oxb::kEpiStoreF32 ? torch::kFloat32 : torch::kBFloat16),
                "gemm_packed: out dtype does not match the epilogue");
    p.C = out.data_ptr();
    p.ldc = out.stride(0);
  }
  oxb::launch_gemm_bf16(tmA, tmA, p, 128, mt_i, cur_stream());
  check_launch("gemm_packed");
}

// a8: [M, K] e4m3 bytes; sa_t: [ceil(K/128), >= M] fp32; w8: [N, K] e4m3 bytes; sw: [ceil(N/128), ceil(K/128)].
// x: [rows, K] or [G, cap, K] bf16 -> q [.., K/2] uint8, sf (scale atoms), gscale [rows] fp32
void quant_act_nvfp4(const Tensor& x, const Tensor& q, const Tensor& sf, const Tensor& gscale,
                     const c10::optional<Tensor>& group_counts, const c10::optional<Tensor>& ag_flags,
                     int64_t ag_expected, const c10::optional<Tensor>& ag_ticket, const Tensor& status,
                     int64_t spin_limit) {
  TORCH_CHECK(x.is_cuda() && x.scalar_type() == torch::kBFloat16 && x.stride(-1) == 1, "quant_act_nvfp4: bf16 rows");
  const int64_t K = x.size(-1);
  TORCH_CHECK(K % 64 == 0, "quant_act_nvfp4: K must be a multiple of 64");
  const int64_t G = x.dim() == 3 ? x.size(0) : 1;
  const int64_t R = x.size(-2);
  TORCH_CHECK(x.dim() == 2 || x.stride(0) == R * x.stride(1), "quant_act_nvfp4: groups must be dense");
  TORCH_CHECK(G == 1 || R % 128 == 0, "quant_act_nvfp4: grouped rows must be a multiple of 128 per group");
  const int64_t tiles = (G * R + 127) / 128;
  TORCH_CHECK(q.scalar_type() == torch::kUInt8 && q.is_contiguous() && q.numel() >= G * R * K / 2, "quant_act_nvfp4: q");
  TORCH_CHECK(sf.scalar_type() == torch::kUInt8 && sf.is_contiguous() && sf.numel() >= tiles * (K / 64) * 512,
              "quant_act_nvfp4: sf too small");
  TORCH_CHECK(gscale.scalar_type() == torch::kFloat32 && gscale.numel() >= G * R, "quant_act_nvfp4: gscale");
  oxb::QuantActWait wait{};
  if (ag_flags.has_value() && ag_flags->defined()) {
    TORCH_CHECK(ag_ticket.has_value() && ag_ticket->defined(), "quant_act_nvfp4: ag_ticket required with ag_flags");
    wait.flags = reinterpret_cast<const uint32_t*>(ag_flags->data_ptr());
    wait.n_src = static_cast<int>(ag_flags->numel());
    wait.expected = static_cast<uint32_t>(ag_expected);
    wait.ticket = reinterpret_cast<uint32_t*>(ag_ticket->data_ptr());
    wait.status = reinterpret_cast<int*>(status.data_ptr());
  }
  oxb::launch_quant_act_nvfp4(reinterpret_cast<const __nv_bfloat16*>(x.data_ptr()), x.stride(-2), q.data_ptr<uint8_t>(),
                              sf.data_ptr<uint8_t>(), gscale.data_ptr<float>(), static_cast<int>(G),
                              static_cast<int>(R), static_cast<int>(K), opt_ptr<uint32_t>(group_counts), wait,
                              static_cast<uint32_t>(spin_limit > 0 ? spin_limit : 0), cur_stream());
  check_launch("quant_act_nvfp4");
}

void gemm_fp8_block(const Tensor& a8, const Tensor& sa_t, const Tensor& w8, const Tensor& sw,
                    const c10::optional<Tensor>& out_opt, const c10::optional<Tensor>& bias,
                    const Tensor& status, const std::vector<int64_t>& slab_ptrs,
                    const std::vector<int64_t>& arrive_ptrs, const c10::optional<Tensor>& done_ticket,
                    int64_t rows_per_owner, int64_t my_rank, int64_t slab_ld) {
  TORCH_CHECK(a8.is_cuda() && w8.is_cuda() && a8.element_size() == 1 && w8.element_size() == 1,
              "gemm_fp8_block: CUDA fp8 operands required");
  TORCH_CHECK(a8.dim() == 2 && w8.dim() == 2 && a8.stride(1) == 1 && w8.stride(1) == 1,
              "gemm_fp8_block: row-major 2-D operands required");
  const int64_t M = a8.size(0), K = a8.size(1), N = w8.size(0);
  TORCH_CHECK(w8.size(1) == K && K % 16 == 0, "gemm_fp8_block: K mismatch or K % 16 != 0");
  const int64_t n_kb = (K + 127) / 128;
  TORCH_CHECK(sa_t.scalar_type() == torch::kFloat32 && sa_t.dim() == 2 && sa_t.size(0) == n_kb &&
                  sa_t.size(1) >= M && sa_t.stride(1) == 1,
              "gemm_fp8_block: sa_t must be [K/128, >=M] fp32");
  TORCH_CHECK(sw.scalar_type() == torch::kFloat32 && sw.is_contiguous() &&
                  sw.size(0) == (N + 127) / 128 && sw.size(1) == n_kb,
              "gemm_fp8_block: sw must be [N/128, K/128] fp32");
  const bool routed = !slab_ptrs.empty();
  if (!routed) {
    TORCH_CHECK(out_opt.has_value(), "gemm_fp8_block: out required");
    const Tensor& out = *out_opt;
    TORCH_CHECK(out.scalar_type() == torch::kBFloat16 && out.size(0) == M && out.size(1) == N &&
                    out.stride(1) == 1,
                "gemm_fp8_block: out must be [M, N] bf16");
  } else {
    TORCH_CHECK(slab_ptrs.size() <= 8 && rows_per_owner > 0 && slab_ld >= N,
                "gemm_fp8_block: 1..8 owners, rows_per_owner > 0, slab_ld >= N");
  }
  CUtensorMap tmA = oxb::make_tma_map(a8.data_ptr(), CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, 2, K, M, 1,
                                      static_cast<uint64_t>(a8.stride(0)), 0, 128, 128, 1,
                                      CU_TENSOR_MAP_SWIZZLE_128B);
  CUtensorMap tmB = oxb::make_tma_map(w8.data_ptr(), CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, 2, K, N, 1,
                                      static_cast<uint64_t>(w8.stride(0)), 0, 128, 128, 1,
                                      CU_TENSOR_MAP_SWIZZLE_128B);
  oxb::Fp8GemmParams p{};
  p.M = static_cast<int>(M);
  p.N = static_cast<int>(N);
  p.K = static_cast<int>(K);
  p.sa_t = sa_t.data_ptr<float>();
  p.sa_ld = static_cast<int>(sa_t.stride(0));
  p.sw = sw.data_ptr<float>();
  if (!routed) {
    p.C = reinterpret_cast<__nv_bfloat16*>(out_opt->data_ptr());
    p.ldc = out_opt->stride(0);
  } else {
    for (size_t i = 0; i < slab_ptrs.size(); ++i) p.slab[i] = reinterpret_cast<__nv_bfloat16*>(slab_ptrs[i]);
    for (size_t i = 0; i < arrive_ptrs.size() && i < 8; ++i)
      p.arrive[i] = reinterpret_cast<uint32_t*>(arrive_ptrs[i]);
    p.n_owners = static_cast<int>(slab_ptrs.size());
    p.rows_per_owner = static_cast<int>(rows_per_owner);
    p.my_rank = static_cast<int>(my_rank);
    p.slab_ld = slab_ld;
    p.done_ticket = opt_ptr<uint32_t>(done_ticket);
  }
  p.bias = bf16_ptr(bias);
  p.status = reinterpret_cast<int*>(status.data_ptr());
  oxb::launch_gemm_fp8_block(tmA, tmB, p, cur_stream());
  check_launch("gemm_fp8_block");
}

void quant_act_fp8(const Tensor& x, const Tensor& q, const Tensor& sa_t,
                   const c10::optional<Tensor>& ag_flags, int64_t ag_expected, int64_t ag_rows_per_src,
                   const c10::optional<Tensor>& ag_ticket, const Tensor& status) {
  TORCH_CHECK(x.is_cuda() && x.scalar_type() == torch::kBFloat16 && x.dim() == 2 && x.stride(1) == 1,
              "quant_act_fp8: [M, K] bf16 input required");
  TORCH_CHECK(q.element_size() == 1 && q.size(0) == x.size(0) && q.size(1) == x.size(1) &&
                  q.stride(1) == 1,
              "quant_act_fp8: q must be [M, K] bytes");
  TORCH_CHECK(sa_t.scalar_type() == torch::kFloat32 && sa_t.size(0) == (x.size(1) + 127) / 128 &&
                  sa_t.size(1) >= x.size(0) && sa_t.stride(1) == 1,
              "quant_act_fp8: sa_t must be [K/128, >=M] fp32");
  oxb::QuantActWait wait{};
  if (ag_flags.has_value() && ag_flags->defined()) {
    TORCH_CHECK(ag_ticket.has_value(), "quant_act_fp8: ag_ticket required with ag_flags");
    wait.flags = reinterpret_cast<const uint32_t*>(ag_flags->data_ptr());
    wait.n_src = static_cast<int>(ag_flags->numel());
    wait.expected = static_cast<uint32_t>(ag_expected);
    wait.rows_per_src = static_cast<int>(ag_rows_per_src);
    wait.ticket = reinterpret_cast<uint32_t*>(ag_ticket->data_ptr());
    wait.status = reinterpret_cast<int*>(status.data_ptr());
  }
  oxb::launch_quant_act_fp8(reinterpret_cast<const __nv_bfloat16*>(x.data_ptr()), x.stride(0),
                            reinterpret_cast<uint8_t*>(q.data_ptr()), q.stride(0),
                            sa_t.data_ptr<float>(), static_cast<int>(sa_t.stride(0)),
                            static_cast<int>(x.size(0)), static_cast<int>(x.size(1)), wait, cur_stream());
  check_launch("quant_act_fp8");
}

// ---------------------------------------------------------------------------------------------
// attention
// ---------------------------------------------------------------------------------------------
void paged_decode(const Tensor& q, const Tensor& k_cache, const Tensor& v_cache,
                  const Tensor& block_tables, const Tensor& seq_lens, const Tensor& pages_per_split,
                  const Tensor& part_o, const Tensor& part_ml, const Tensor& out, int64_t batch,
                  int64_t max_splits, int64_t window, double scale,
                  const c10::optional<Tensor>& status, const c10::optional<Tensor>& page_ml,
                  const c10::optional<Tensor>& block_mass, const c10::optional<Tensor>& q8,
                  const c10::optional<Tensor>& q8_d, const c10::optional<Tensor>& q8_s) {
  TORCH_CHECK(q.dim() == 3 && k_cache.dim() == 4, "paged_decode: q [B,Hq,D], cache [blk,Hkv,16,D]");
  TORCH_CHECK(k_cache.size(2) == 16, "paged_decode: 16-token pages");
  oxb::DecodeAttnParams p{};
  const int D = static_cast<int>(q.size(2));
  TORCH_CHECK(D == 64 || D == 128, "paged_decode: head_dim 64 or 128");
  p.q = reinterpret_cast<const __nv_bfloat16*>(q.data_ptr());
  p.q_stride = q.stride(0);
  TORCH_CHECK(q.stride(1) == D && q.stride(2) == 1, "paged_decode: q heads must be packed");
  p.k_cache = reinterpret_cast<const __nv_bfloat16*>(k_cache.data_ptr());
  p.v_cache = reinterpret_cast<const __nv_bfloat16*>(v_cache.data_ptr());
  p.block_tables = block_tables.data_ptr<int>();
  p.seq_lens = seq_lens.data_ptr<int>();
  p.pages_per_split = pages_per_split.data_ptr<int>();
  p.part_o = part_o.data_ptr<float>();
  p.part_ml = part_ml.data_ptr<float>();
  p.out = reinterpret_cast<__nv_bfloat16*>(out.data_ptr());
  p.out_stride = out.stride(0);
  p.max_blocks = static_cast<int>(block_tables.size(1));
  p.Hq = static_cast<int>(q.size(1));
  p.Hkv = static_cast<int>(k_cache.size(1));
  TORCH_CHECK(p.Hq % p.Hkv == 0 && p.Hq / p.Hkv <= 16, "paged_decode: group size must be <= 16");
  p.max_splits = static_cast<int>(max_splits);
  TORCH_CHECK(part_o.numel() >= batch * p.Hq * max_splits * D, "paged_decode: part_o too small");
  TORCH_CHECK(part_ml.numel() >= batch * p.Hq * max_splits * 2, "paged_decode: part_ml too small");
  p.window = static_cast<int>(window);
  p.scale_log2 = static_cast<float>(scale * 1.4426950408889634);
  p.status = opt_ptr<int>(status);  // given only when bounds checking is on
  p.num_blocks = p.status != nullptr ? static_cast<int>(k_cache.size(0)) : 0;
  TORCH_CHECK(page_ml.has_value() == block_mass.has_value(), "paged_decode: page_ml and block_mass go together");
  if (page_ml.has_value()) {
    TORCH_CHECK(p.Hq <= 128, "paged_decode: block mass supports up to 128 query heads per rank");
    TORCH_CHECK(page_ml->scalar_type() == at::kFloat && block_mass->scalar_type() == at::kFloat &&
                    page_ml->is_contiguous() && block_mass->is_contiguous(),
                "paged_decode: page_ml / block_mass must be contiguous fp32");
    TORCH_CHECK(page_ml->numel() >= batch * p.max_blocks * p.Hq * 2, "paged_decode: page_ml too small");
    TORCH_CHECK(block_mass->numel() >= batch * p.max_blocks, "paged_decode: block_mass too small");
    p.page_ml = page_ml->data_ptr<float>();
    p.block_mass = block_mass->data_ptr<float>();
  }
  if (q8.has_value() && q8->defined()) {
    const int64_t kq = static_cast<int64_t>(p.Hq) * D;
    TORCH_CHECK(q8_d.has_value() && q8_s.has_value() && q8->element_size() == 1 && q8->numel() >= batch * kq &&
                    q8_d->numel() >= batch * (kq / 32) && q8_s->numel() >= batch * (kq / 32) &&
                    q8_d->scalar_type() == at::kFloat && q8_s->scalar_type() == at::kFloat,
                "paged_decode: q8 [B, Hq*D] int8 with q8_d / q8_s [B, Hq*D / 32] fp32 expected");
    p.q8 = reinterpret_cast<signed char*>(q8->data_ptr());
    p.q8_d = q8_d->data_ptr<float>();
    p.q8_s = q8_s->data_ptr<float>();
  }
  (void)oxb::launch_paged_decode(p, static_cast<int>(batch), D, cur_stream());
  check_launch("paged_decode");
}

void paged_prefill_tc(const Tensor& q, const Tensor& k_cache, const Tensor& v_cache,
                      const Tensor& block_tables, const Tensor& tile_seq, const Tensor& tile_q0,
                      const Tensor& q_start, const Tensor& q_lens, const Tensor& ctx_lens,
                      const Tensor& out, int64_t n_tiles, int64_t window, double scale,
                      const Tensor& status) {
  TORCH_CHECK(q.dim() == 3 && k_cache.dim() == 4, "paged_prefill_tc: q [T,Hq,D], cache [blk,Hkv,16,D]");
  TORCH_CHECK(k_cache.is_contiguous() && v_cache.is_contiguous(), "paged_prefill_tc: contiguous caches");
  oxb::PrefillAttnParams p{};
  const int D = static_cast<int>(q.size(2));
  TORCH_CHECK(D == 64 || D == 128, "paged_prefill_tc: head_dim 64 or 128");
  TORCH_CHECK(q.stride(1) == D && q.stride(2) == 1, "paged_prefill_tc: q heads must be packed");
  p.q = reinterpret_cast<const __nv_bfloat16*>(q.data_ptr());
  p.q_stride = q.stride(0);
  p.k_cache = reinterpret_cast<const __nv_bfloat16*>(k_cache.data_ptr());
  p.v_cache = reinterpret_cast<const __nv_bfloat16*>(v_cache.data_ptr());
  p.block_tables = block_tables.data_ptr<int>();
  p.tile_seq = tile_seq.data_ptr<int>();
  p.tile_q0 = tile_q0.data_ptr<int>();
  p.q_start = q_start.data_ptr<int>();
  p.q_lens = q_lens.data_ptr<int>();
  p.ctx_lens = ctx_lens.data_ptr<int>();
  p.out = reinterpret_cast<__nv_bfloat16*>(out.data_ptr());
  p.out_stride = out.stride(0);
  p.max_blocks = static_cast<int>(block_tables.size(1));
  p.Hq = static_cast<int>(q.size(1));
  p.Hkv = static_cast<int>(k_cache.size(1));
  p.window = static_cast<int>(window);
  p.scale_log2 = static_cast<float>(scale * 1.4426950408889634);
  const uint64_t T = q.size(0);
  const uint64_t kv_rows = static_cast<uint64_t>(k_cache.size(0)) * p.Hkv * 16;
  CUtensorMap tmQ = oxb::make_tma_map(q.data_ptr(), CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, 2,
                                      static_cast<uint64_t>(p.Hq) * D, T, 1,
                                      static_cast<uint64_t>(q.stride(0)) * 2, 0, 64, 128, 1,
                                      CU_TENSOR_MAP_SWIZZLE_128B);
  CUtensorMap tmK = oxb::make_tma_map(k_cache.data_ptr(), CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, 2, D,
                                      kv_rows, 1, static_cast<uint64_t>(D) * 2, 0, 64, 16, 1,
                                      CU_TENSOR_MAP_SWIZZLE_128B);
  CUtensorMap tmV = oxb::make_tma_map(v_cache.data_ptr(), CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, 2, D,
                                      kv_rows, 1, static_cast<uint64_t>(D) * 2, 0, 64, 16, 1,
                                      CU_TENSOR_MAP_SWIZZLE_128B);
  p.num_blocks = static_cast<int>(k_cache.size(0));
  oxb::launch_paged_prefill_tc(tmQ, tmK, tmV, p, static_cast<int>(n_tiles), D,
                               reinterpret_cast<int*>(status.data_ptr()), cur_stream());
  check_launch("paged_prefill_tc");
}

// ---------------------------------------------------------------------------------------------
// fused finalize kernels
// ---------------------------------------------------------------------------------------------
void finalize_norm(const c10::optional<Tensor>& acc, const c10::optional<Tensor>& rs_slab,
                   int64_t n_slabs, int64_t slab_stride, const c10::optional<Tensor>& arrive,
                   int64_t expected, const c10::optional<Tensor>& ticket,
                   const c10::optional<Tensor>& residual_in,
                   const c10::optional<Tensor>& residual_out, const c10::optional<Tensor>& bias,
                   const c10::optional<Tensor>& norm_w, double eps, double w_offset,
                   const std::vector<int64_t>& out_ptrs, const std::vector<int64_t>& out_flag_ptrs,
                   int64_t out_row_off, const c10::optional<Tensor>& out_row_map, int64_t rows,
                   int64_t N, const Tensor& status,
                   const c10::optional<Tensor>& router_w, int64_t top_k, int64_t experts_per_rank,
                   double routed_scale, const std::vector<int64_t>& slab_ptrs,
                   const std::vector<int64_t>& meta_ptrs, const std::vector<int64_t>& cnt_ptrs,
                   int64_t cap, int64_t my_rank, int64_t spin_limit, const c10::optional<Tensor>& q8,
                   const c10::optional<Tensor>& q8_d, const c10::optional<Tensor>& q8_s) {
  TORCH_CHECK(N % 8 == 0 && N <= 1024 * 8 * 4, "finalize_norm: N must be a multiple of 8 and <= 32768");
  oxb::FinalizeNormParams p{};
  p.acc = opt_ptr<float>(acc);
  p.rs_slab = bf16_ptr(rs_slab);
  p.n_slabs = static_cast<int>(n_slabs);
  p.slab_stride = slab_stride;
  p.arrive = opt_ptr<uint32_t>(arrive);
  p.expected = static_cast<uint32_t>(expected);
  p.ticket = opt_ptr<uint32_t>(ticket);
  if (p.arrive != nullptr) {
    TORCH_CHECK(p.ticket != nullptr, "finalize_norm: ticket required");
  }
  p.residual_in = bf16_ptr(residual_in);
  p.residual_out = const_cast<__nv_bfloat16*>(bf16_ptr(residual_out));
  p.bias = bf16_ptr(bias);
  p.norm_w = bf16_ptr(norm_w);
  p.eps = static_cast<float>(eps);
  p.w_offset = static_cast<float>(w_offset);
  TORCH_CHECK(out_ptrs.size() <= oxb::kMaxPeers, "finalize_norm: at most 8 destinations");
  for (size_t i = 0; i < out_ptrs.size(); ++i)
    p.out[i] = reinterpret_cast<__nv_bfloat16*>(out_ptrs[i]);
  for (size_t i = 0; i < out_flag_ptrs.size() && i < oxb::kMaxPeers; ++i)
    p.out_flag[i] = reinterpret_cast<uint32_t*>(out_flag_ptrs[i]);
  p.n_dst = static_cast<int>(out_ptrs.size() > 0 ? out_ptrs.size() : out_flag_ptrs.size());
  p.out_row_off = out_row_off;
  p.out_row_map = opt_ptr<int>(out_row_map);
  p.rows = static_cast<int>(rows);
  p.N = static_cast<int>(N);
  p.status = reinterpret_cast<int*>(status.data_ptr());
  p.spin_limit = static_cast<uint32_t>(spin_limit > 0 ? spin_limit : 0);
  if (router_w.has_value() && router_w->defined()) {
    p.router_w = bf16_ptr(router_w);
    p.n_experts = static_cast<int>(router_w->size(0));
    TORCH_CHECK(p.n_experts <= 64 && top_k <= 8, "finalize_norm: <= 64 experts, top_k <= 8");
    p.top_k = static_cast<int>(top_k);
    p.experts_per_rank = static_cast<int>(experts_per_rank);
    p.routed_scale = static_cast<float>(routed_scale);
    TORCH_CHECK(slab_ptrs.size() == meta_ptrs.size() && slab_ptrs.size() == cnt_ptrs.size() &&
                    slab_ptrs.size() <= oxb::kMaxPeers,
                "finalize_norm: slab/meta/cnt tables must match");
    for (size_t i = 0; i < slab_ptrs.size(); ++i) {
      p.slab[i] = reinterpret_cast<__nv_bfloat16*>(slab_ptrs[i]);
      p.meta[i] = reinterpret_cast<oxb::MoeRowMeta*>(meta_ptrs[i]);
      p.slab_cnt[i] = reinterpret_cast<uint32_t*>(cnt_ptrs[i]);
    }
    p.n_dst = static_cast<int>(slab_ptrs.size());
    p.cap = static_cast<int>(cap);
    p.my_rank = static_cast<int>(my_rank);
  }
  if (q8.has_value() && q8->defined()) {
    TORCH_CHECK(q8_d.has_value() && q8_s.has_value() && N % 32 == 0 && q8->element_size() == 1 &&
                    q8->numel() >= rows * N && q8_d->numel() >= rows * (N / 32) && q8_s->numel() >= rows * (N / 32) &&
                    q8_d->scalar_type() == at::kFloat && q8_s->scalar_type() == at::kFloat &&
                    reinterpret_cast<uintptr_t>(q8->data_ptr()) % 8 == 0,
                "finalize_norm: q8 [rows, N] int8 with q8_d / q8_s [rows, N / 32] fp32 expected");
    p.q8 = reinterpret_cast<int8_t*>(q8->data_ptr());
    p.q8_d = q8_d->data_ptr<float>();
    p.q8_s = q8_s->data_ptr<float>();
  }
  oxb::launch_finalize_norm(p, cur_stream());
  check_launch("finalize_norm");
}

void qkv_rope_append(const c10::optional<Tensor>& acc_f32, const c10::optional<Tensor>& qkv_bf16,
                     const c10::optional<Tensor>& bias, const c10::optional<Tensor>& q_norm_w,
                     const c10::optional<Tensor>& k_norm_w, double norm_eps, double norm_w_offset,
                     const Tensor& positions, const Tensor& slot_mapping, const Tensor& inv_freq,
                     double rope_mscale, const Tensor& q_out, const Tensor& k_cache,
                     const Tensor& v_cache, int64_t M, int64_t Hq, int64_t Hkv, int64_t D,
                     const Tensor& status) {
  oxb::QkvRopeParams p{};
  p.acc_f32 = opt_ptr<float>(acc_f32);
  p.qkv_bf16 = bf16_ptr(qkv_bf16);
  TORCH_CHECK((p.acc_f32 != nullptr) != (p.qkv_bf16 != nullptr), "qkv_rope_append: one input");
  TORCH_CHECK(D >= 2 && D <= 256 && D % 2 == 0, "qkv_rope_append: head_dim must be even and <= 256");
  p.bias = bf16_ptr(bias);
  p.q_norm_w = bf16_ptr(q_norm_w);
  p.k_norm_w = bf16_ptr(k_norm_w);
  p.norm_eps = static_cast<float>(norm_eps);
  p.norm_w_offset = static_cast<float>(norm_w_offset);
  TORCH_CHECK(positions.scalar_type() == torch::kInt32 && slot_mapping.scalar_type() == torch::kInt64,
              "qkv_rope_append: positions int32, slot_mapping int64");
  p.positions = positions.data_ptr<int>();
  p.slot_mapping = reinterpret_cast<const long long*>(slot_mapping.data_ptr<int64_t>());
  p.inv_freq = inv_freq.data_ptr<float>();
  TORCH_CHECK(inv_freq.numel() == D / 2, "qkv_rope_append: inv_freq must have D/2 entries");
  p.rope_mscale = static_cast<float>(rope_mscale);
  p.q_out = reinterpret_cast<__nv_bfloat16*>(q_out.data_ptr());
  p.k_cache = reinterpret_cast<__nv_bfloat16*>(k_cache.data_ptr());
  p.v_cache = reinterpret_cast<__nv_bfloat16*>(v_cache.data_ptr());
  p.M = static_cast<int>(M);
  p.Hq = static_cast<int>(Hq);
  p.Hkv = static_cast<int>(Hkv);
  p.D = static_cast<int>(D);
  TORCH_CHECK(Hq + Hkv <= 160 && (D % 8) == 0, "qkv_rope_append: unsupported head layout");
  p.num_slots = k_cache.size(0) * 16;
  p.status = reinterpret_cast<int*>(status.data_ptr());
  oxb::launch_qkv_rope_append(p, cur_stream());
  check_launch("qkv_rope_append");
}

void swiglu(const c10::optional<Tensor>& acc_f32, const c10::optional<Tensor>& gu_bf16,
            const Tensor& out, int64_t M, int64_t I, int64_t act, const c10::optional<Tensor>& q8,
            const c10::optional<Tensor>& q8_d, const c10::optional<Tensor>& q8_s) {
  oxb::SwigluParams p{};
  p.acc_f32 = opt_ptr<float>(acc_f32);
  p.gu_bf16 = bf16_ptr(gu_bf16);
  TORCH_CHECK(I % 4 == 0, "swiglu: I must be a multiple of 4");
  p.out = reinterpret_cast<__nv_bfloat16*>(out.data_ptr());
  p.M = static_cast<int>(M);
  p.I = static_cast<int>(I);
  p.act = static_cast<int>(act);
  if (q8.has_value() && q8->defined()) {
    TORCH_CHECK(q8_d.has_value() && q8_s.has_value() && I % 32 == 0 && q8->element_size() == 1 &&
                    q8->numel() >= M * I && q8_d->numel() >= M * (I / 32) && q8_s->numel() >= M * (I / 32) &&
                    q8_d->scalar_type() == at::kFloat && q8_s->scalar_type() == at::kFloat &&
                    reinterpret_cast<uintptr_t>(q8->data_ptr()) % 4 == 0,
                "swiglu: q8 [M, I] int8 with q8_d / q8_s [M, I / 32] fp32 expected");
    p.q8 = reinterpret_cast<int8_t*>(q8->data_ptr());
    p.q8_d = q8_d->data_ptr<float>();
    p.q8_s = q8_s->data_ptr<float>();
  }
  oxb::launch_swiglu(p, cur_stream());
  check_launch("swiglu");
}

void embed_gather(const Tensor& tokens, const Tensor& table, const Tensor& out, double scale,
                  int64_t vocab_start) {
  TORCH_CHECK(tokens.scalar_type() == torch::kInt32, "embed_gather: int32 tokens");
  TORCH_CHECK(table.size(1) % 8 == 0, "embed_gather: hidden must be a multiple of 8");
  oxb::launch_embed_gather(tokens.data_ptr<int>(), bf16_ptr(table),
                           reinterpret_cast<__nv_bfloat16*>(out.data_ptr()),
                           static_cast<int>(tokens.numel()), static_cast<int>(table.size(1)),
                           static_cast<int>(table.size(0)), static_cast<float>(scale),
                           static_cast<int>(vocab_start), cur_stream());
  check_launch("embed_gather");
}

void cast_acc_bf16(const Tensor& acc, const c10::optional<Tensor>& bias, const Tensor& out,
                   int64_t M, int64_t N) {
  TORCH_CHECK(N % 4 == 0, "cast_acc_bf16: N must be a multiple of 4");
  oxb::launch_cast_acc_bf16(acc.data_ptr<float>(), bf16_ptr(bias),
                            reinterpret_cast<__nv_bfloat16*>(out.data_ptr()), static_cast<int>(M),
                            static_cast<int>(N), out.stride(0), cur_stream());
  check_launch("cast_acc_bf16");
}

void fwht128(const Tensor& x) {
  TORCH_CHECK(x.scalar_type() == torch::kFloat32 && x.numel() % 128 == 0, "fwht128: fp32, 128 | n");
  oxb::launch_fwht128(x.data_ptr<float>(), x.numel() / 128, cur_stream());
  check_launch("fwht128");
}

void kv_block_copy(const Tensor& k_cache, const Tensor& v_cache, const Tensor& src,
                   const Tensor& dst) {
  const long long block_elems = k_cache.stride(0);
  oxb::launch_kv_block_copy(reinterpret_cast<__nv_bfloat16*>(k_cache.data_ptr()),
                            reinterpret_cast<__nv_bfloat16*>(v_cache.data_ptr()),
                            src.data_ptr<int>(), dst.data_ptr<int>(),
                            static_cast<int>(src.numel()), block_elems, cur_stream());
  check_launch("kv_block_copy");
}

void softcap(const Tensor& logits, double cap) {
  oxb::launch_softcap(logits.data_ptr<float>(), logits.numel(), static_cast<float>(cap),
                      cur_stream());
  check_launch("softcap");
}

// Page-locked host memory that the device can write directly: returns the host view (int64 words)
// and the device address of the same bytes. Freed with the tensor.
std::tuple<Tensor, int64_t> alloc_mapped_host(int64_t n_words) {
  TORCH_CHECK(n_words > 0, "alloc_mapped_host: size");
  void* host = nullptr;
  cudaError_t e = cudaHostAlloc(&host, static_cast<size_t>(n_words) * 8, cudaHostAllocMapped);
  TORCH_CHECK(e == cudaSuccess, "cudaHostAlloc(mapped): ", cudaGetErrorString(e));
  void* dev = nullptr;
  e = cudaHostGetDevicePointer(&dev, host, 0);
  if (e != cudaSuccess) {
    cudaFreeHost(host);
    TORCH_CHECK(false, "cudaHostGetDevicePointer: ", cudaGetErrorString(e));
  }
  std::memset(host, 0, static_cast<size_t>(n_words) * 8);
  Tensor t = torch::from_blob(host, {n_words}, [](void* p) { cudaFreeHost(p); },
                              torch::TensorOptions().dtype(torch::kInt64).device(torch::kCPU));
  return {t, static_cast<int64_t>(reinterpret_cast<uintptr_t>(dev))};
}

void advance_decode_step(const Tensor& token_ids, const Tensor& positions, const Tensor& slot_mapping,
                         const Tensor& seq_lens, const Tensor& block_tables, const Tensor& sampled,
                         int64_t mailbox_dev, const Tensor& step_counter, int64_t rows, int64_t ring,
                         const c10::optional<Tensor>& status) {
  TORCH_CHECK(token_ids.is_cuda() && token_ids.scalar_type() == at::kInt && positions.scalar_type() == at::kInt &&
                  slot_mapping.scalar_type() == at::kLong && seq_lens.scalar_type() == at::kInt &&
                  block_tables.scalar_type() == at::kInt && sampled.scalar_type() == at::kInt &&
                  step_counter.scalar_type() == at::kInt,
              "advance_decode_step: dtypes");
  TORCH_CHECK(block_tables.dim() == 2 && block_tables.stride(1) == 1 && block_tables.stride(0) == block_tables.size(1),
              "advance_decode_step: block_tables [rows, max_blocks] contiguous");
  TORCH_CHECK(rows > 0 && token_ids.numel() >= rows && positions.numel() >= rows && slot_mapping.numel() >= rows &&
                  seq_lens.numel() >= rows && sampled.numel() >= rows && block_tables.size(0) >= rows,
              "advance_decode_step: rows");
  TORCH_CHECK(mailbox_dev != 0 && ring > 0, "advance_decode_step: mailbox");
  oxb::AdvanceStepParams p{};
  p.token_ids = token_ids.data_ptr<int>();
  p.positions = positions.data_ptr<int>();
  p.slot_mapping = reinterpret_cast<long long*>(slot_mapping.data_ptr<int64_t>());
  p.seq_lens = seq_lens.data_ptr<int>();
  p.block_tables = block_tables.data_ptr<int>();
  p.sampled = sampled.data_ptr<int>();
  p.mailbox = reinterpret_cast<unsigned long long*>(static_cast<uintptr_t>(mailbox_dev));
  p.step_counter = reinterpret_cast<unsigned int*>(step_counter.data_ptr<int>());
  p.rows = static_cast<int>(rows);
  p.max_blocks = static_cast<int>(block_tables.size(1));
  p.ring = static_cast<int>(ring);
  p.status = opt_ptr<int>(status);
  oxb::launch_advance_decode_step(p, cur_stream());
  check_launch("advance_decode_step");
}

// ---------------------------------------------------------------------------------------------
// quantized weights
// ---------------------------------------------------------------------------------------------
void mmvq(int64_t qtype, const Tensor& w, const Tensor& x, const c10::optional<Tensor>& bias,
          const Tensor& out, int64_t N, int64_t K, bool add, const c10::optional<Tensor>& xq,
          const c10::optional<Tensor>& xd, const c10::optional<Tensor>& xs) {
  TORCH_CHECK(w.scalar_type() == torch::kUInt8 && w.is_cuda(), "mmvq: packed uint8 weights");
  TORCH_CHECK(K % 32 == 0, "mmvq: K must be a multiple of 32");
  oxb::MmvqParams p{};
  p.w = w.data_ptr<uint8_t>();
  p.row_bytes = oxb::quant_row_bytes(static_cast<int>(qtype), K);
  TORCH_CHECK(p.row_bytes > 0 && w.numel() >= p.row_bytes * N, "mmvq: weight buffer too small");
  p.x = bf16_ptr(x);
  p.ldx = x.stride(0);
  p.bias = bf16_ptr(bias);
  if (out.scalar_type() == torch::kFloat32)
    p.out_f32 = out.data_ptr<float>();
  else
    p.out_bf16 = reinterpret_cast<__nv_bfloat16*>(out.data_ptr());
  p.ldo = out.stride(0);
  p.M = static_cast<int>(x.size(0));
  p.N = static_cast<int>(N);
  p.K = static_cast<int>(K);
  p.add = add ? 1 : 0;
  if (xq.has_value() && xq->defined()) {
    TORCH_CHECK(xd.has_value() && xs.has_value() && xq->element_size() == 1 && xq->is_contiguous() &&
                    xq->size(0) >= x.size(0) && xq->size(1) == K && xd->is_contiguous() &&
                    xs->is_contiguous() && xd->size(1) == K / 32 && xs->size(1) == K / 32,
                "mmvq: xq [M, K] int8 with xd / xs [M, K/32] fp32 expected");
    p.xq = reinterpret_cast<const int8_t*>(xq->data_ptr());
    p.xd = xd->data_ptr<float>();
    p.xs = xs->data_ptr<float>();
  }
  TORCH_CHECK(oxb::launch_mmvq(static_cast<int>(qtype), p, cur_stream()),
              "mmvq: no device decoder for GGUF type ", qtype);
  check_launch("mmvq");
}

// Stacked packed matrices of different block types sharing K (one launch): out[:, sum of n_i].
void mmvq_mixed(const std::vector<int64_t>& qtypes, const std::vector<Tensor>& ws, const std::vector<int64_t>& ns,
                const Tensor& x, const Tensor& out, int64_t K, const Tensor& xq, const Tensor& xd,
                const Tensor& xs) {
  const size_t n_seg = qtypes.size();
  TORCH_CHECK(n_seg >= 1 && n_seg <= 4 && ws.size() == n_seg && ns.size() == n_seg, "mmvq_mixed: 1..4 segments");
  TORCH_CHECK(K % 32 == 0, "mmvq_mixed: K must be a multiple of 32");
  oxb::MmvqParams p{};
  int64_t rows = 0;
  for (size_t i = 0; i < n_seg; ++i) {
    TORCH_CHECK(ws[i].scalar_type() == torch::kUInt8 && ws[i].is_cuda(), "mmvq_mixed: packed uint8 weights");
    p.seg_type[i] = static_cast<int>(qtypes[i]);
    p.seg_w[i] = ws[i].data_ptr<uint8_t>();
    p.seg_row_bytes[i] = oxb::quant_row_bytes(p.seg_type[i], K);
    TORCH_CHECK(p.seg_row_bytes[i] > 0 && ws[i].numel() >= p.seg_row_bytes[i] * ns[i],
                "mmvq_mixed: weight buffer ", i, " too small");
    rows += ns[i];
    p.seg_row_end[i] = static_cast<int>(rows);
  }
  p.n_seg = static_cast<int>(n_seg);
  p.x = bf16_ptr(x);
  p.ldx = x.stride(0);
  if (out.scalar_type() == torch::kFloat32)
    p.out_f32 = out.data_ptr<float>();
  else
    p.out_bf16 = reinterpret_cast<__nv_bfloat16*>(out.data_ptr());
  TORCH_CHECK(out.size(1) >= rows && out.size(0) >= x.size(0), "mmvq_mixed: out too small");
  p.ldo = out.stride(0);
  p.M = static_cast<int>(x.size(0));
  p.N = static_cast<int>(rows);
  p.K = static_cast<int>(K);
  TORCH_CHECK(xq.element_size() == 1 && xq.is_contiguous() && xq.size(0) >= x.size(0) && xq.size(1) == K &&
                  xd.is_contiguous() && xs.is_contiguous() && xd.size(1) == K / 32 && xs.size(1) == K / 32,
              "mmvq_mixed: xq [M, K] int8 with xd / xs [M, K/32] fp32 expected");
  p.xq = reinterpret_cast<const int8_t*>(xq.data_ptr());
  p.xd = xd.data_ptr<float>();
  p.xs = xs.data_ptr<float>();
  TORCH_CHECK(oxb::launch_mmvq_mixed(p, cur_stream()),
              "mmvq_mixed: a segment's block type has no integer path or an operand is misaligned");
  check_launch("mmvq_mixed");
}

// x: [M <= 8, K] bf16; w: [N, K] bf16 or tile-major [N/128, K/64, 128, 64]; out: [M, N] (or [M, N/2] with swiglu).
void gemv_bf16(const Tensor& x, const Tensor& w, const Tensor& out, const c10::optional<Tensor>& bias,
               bool swiglu, int64_t act) {
  TORCH_CHECK(x.is_cuda() && w.is_cuda() && x.scalar_type() == torch::kBFloat16 &&
                  w.scalar_type() == torch::kBFloat16 && x.dim() == 2 && x.stride(1) == 1 && w.is_contiguous(),
              "gemv_bf16: bf16 CUDA operands, contiguous weights");
  const bool tiled = w.dim() == 4;
  const int64_t M = x.size(0), K = x.size(1);
  const int64_t N = tiled ? w.size(0) * 128 : w.size(0);
  TORCH_CHECK(M >= 1 && M <= 8, "gemv_bf16: 1..8 rows");
  TORCH_CHECK((tiled ? w.size(1) * 64 : w.size(1)) == K && K % 64 == 0 && N % 2 == 0,
              "gemv_bf16: K mismatch, K % 64 != 0 or odd N");
  TORCH_CHECK(x.stride(0) % 8 == 0 && (reinterpret_cast<uintptr_t>(x.data_ptr()) & 15) == 0,
              "gemv_bf16: activation rows must be 16-byte aligned");
  TORCH_CHECK(!swiglu || N % 64 == 0, "gemv_bf16: the SwiGLU form needs N % 64 == 0");
  const int64_t n_out = swiglu ? N / 2 : N;
  TORCH_CHECK(out.dim() == 2 && out.size(0) >= M && out.size(1) >= n_out && out.stride(1) == 1,
              "gemv_bf16: out too small");
  oxb::GemvParams p{};
  p.w = reinterpret_cast<const __nv_bfloat16*>(w.data_ptr());
  p.x = reinterpret_cast<const __nv_bfloat16*>(x.data_ptr());
  p.ldx = x.stride(0);
  p.bias = bf16_ptr(bias);
  if (out.scalar_type() == torch::kFloat32)
    p.out_f32 = out.data_ptr<float>();
  else
    p.out_bf16 = reinterpret_cast<__nv_bfloat16*>(out.data_ptr());
  p.ldo = out.stride(0);
  p.M = static_cast<int>(M);
  p.N = static_cast<int>(N);
  p.K = static_cast<int>(K);
  p.tiled = tiled ? 1 : 0;
  p.swiglu = swiglu ? 1 : 0;
  p.act = static_cast<int>(act);
  oxb::launch_gemv_bf16(p, cur_stream());
  check_launch("gemv_bf16");
}

void quant_q8_1(const Tensor& x, const Tensor& xq, const Tensor& xd, const Tensor& xs) {
  TORCH_CHECK(x.is_cuda() && x.scalar_type() == torch::kBFloat16 && x.dim() == 2 && x.stride(1) == 1 &&
                  x.size(1) % 32 == 0,
              "quant_q8_1: [M, K] bf16 input with K % 32 == 0");
  const int64_t M = x.size(0), K = x.size(1);
  TORCH_CHECK(xq.element_size() == 1 && xq.is_contiguous() && xq.size(0) >= M && xq.size(1) == K &&
                  xd.scalar_type() == torch::kFloat32 && xd.is_contiguous() && xd.size(0) >= M &&
                  xd.size(1) == K / 32 && xs.scalar_type() == torch::kFloat32 && xs.is_contiguous() &&
                  xs.size(0) >= M && xs.size(1) == K / 32,
              "quant_q8_1: xq [M, K] int8, xd / xs [M, K/32] fp32");
  oxb::launch_quant_q8_1(reinterpret_cast<const __nv_bfloat16*>(x.data_ptr()), x.stride(0),
                         reinterpret_cast<int8_t*>(xq.data_ptr()), xd.data_ptr<float>(),
                         xs.data_ptr<float>(), static_cast<int>(M), static_cast<int>(K), cur_stream());
  check_launch("quant_q8_1");
}

void dequant_rows(int64_t qtype, const Tensor& w, const c10::optional<Tensor>& row_ids,
                  const Tensor& out, int64_t n_src_rows, int64_t K, double scale) {
  TORCH_CHECK(w.scalar_type() == torch::kUInt8 && w.is_cuda(), "dequant_rows: packed weights");
  TORCH_CHECK(K % 32 == 0, "dequant_rows: K must be a multiple of 32");
  const long long rb = oxb::quant_row_bytes(static_cast<int>(qtype), K);
  const int* ids = nullptr;
  if (row_ids.has_value() && row_ids->defined()) ids = row_ids->data_ptr<int>();
  TORCH_CHECK(oxb::launch_dequant_rows(static_cast<int>(qtype), w.data_ptr<uint8_t>(), rb, ids,
                                       static_cast<int>(out.size(0)), static_cast<int>(K),
                                       reinterpret_cast<__nv_bfloat16*>(out.data_ptr()),
                                       out.stride(0), static_cast<float>(scale),
                                       static_cast<int>(n_src_rows), cur_stream()),
              "dequant_rows: no device decoder for GGUF type ", qtype);
  check_launch("dequant_rows");
}

int64_t quant_row_bytes(int64_t qtype, int64_t K) {
  return oxb::quant_row_bytes(static_cast<int>(qtype), K);
}

// ---------------------------------------------------------------------------------------------
// sampler
// ---------------------------------------------------------------------------------------------
void sample(const Tensor& logits, const c10::optional<Tensor>& temperature,
            const c10::optional<Tensor>& top_k, const c10::optional<Tensor>& top_p,
            const c10::optional<Tensor>& min_p, const c10::optional<Tensor>& seeds,
            const c10::optional<Tensor>& counters, const c10::optional<Tensor>& allow_mask,
            const Tensor& out_tokens, const c10::optional<Tensor>& out_logit) {
  TORCH_CHECK(logits.scalar_type() == torch::kFloat32 && logits.dim() == 2, "sample: fp32 [B,V]");
  oxb::SampleParams p{};
  p.logits = logits.data_ptr<float>();
  p.ld = logits.stride(0);
  p.V = static_cast<int>(logits.size(1));
  p.temperature = opt_ptr<float>(temperature);
  p.top_k = opt_ptr<int>(top_k);
  p.top_p = opt_ptr<float>(top_p);
  p.min_p = opt_ptr<float>(min_p);
  p.seeds = opt_ptr<uint64_t>(seeds);
  p.counters = opt_ptr<uint64_t>(counters);
  p.allow_mask = opt_ptr<uint32_t>(allow_mask);
  p.mask_words = allow_mask.has_value() && allow_mask->defined()
                     ? static_cast<int>(allow_mask->size(1))
                     : 0;
  p.out_tokens = out_tokens.data_ptr<int>();
  p.out_logit = opt_ptr<float>(out_logit);
  oxb::launch_sample(p, static_cast<int>(logits.size(0)), cur_stream());
  check_launch("sample");
}

void argmax(const Tensor& logits, const Tensor& out, const c10::optional<Tensor>& out_val) {
  TORCH_CHECK(logits.scalar_type() == torch::kFloat32 && logits.dim() == 2, "argmax: fp32 [B,V]");
  oxb::launch_argmax(logits.data_ptr<float>(), logits.stride(0), static_cast<int>(logits.size(1)),
                     static_cast<int>(logits.size(0)), out.data_ptr<int>(), opt_ptr<float>(out_val),
                     cur_stream());
  check_launch("argmax");
}

void argmax_combine(const Tensor& vals, const Tensor& idxs, const Tensor& out) {
  oxb::launch_argmax_combine(vals.data_ptr<float>(), idxs.data_ptr<int>(),
                             static_cast<int>(vals.size(0)), static_cast<int>(vals.size(1)),
                             out.data_ptr<int>(), cur_stream());
  check_launch("argmax_combine");
}

// Vocab-parallel greedy sampling through peer memory (see ArgmaxExchangeParams): `tab_ptrs[o]` is the
// table of rank o ([2, ranks, max_rows] 64-bit words, zero-initialised), one call per step on every rank.
void argmax_exchange(const Tensor& logits, int64_t vocab_start, const std::vector<int64_t>& tab_ptrs,
                     int64_t max_rows, int64_t my_rank, int64_t slot, const Tensor& out, const Tensor& status,
                     int64_t spin_limit) {
  TORCH_CHECK(logits.is_cuda() && logits.scalar_type() == at::kFloat && logits.dim() == 2 && logits.stride(1) == 1,
              "argmax_exchange: fp32 [rows, V_local] logits");
  TORCH_CHECK(tab_ptrs.size() >= 1 && tab_ptrs.size() <= 8 && my_rank >= 0 &&
                  my_rank < static_cast<int64_t>(tab_ptrs.size()) && (slot == 0 || slot == 1),
              "argmax_exchange: 1..8 ranks, slot 0 or 1");
  TORCH_CHECK(logits.size(0) <= max_rows && out.scalar_type() == at::kInt && out.numel() >= logits.size(0),
              "argmax_exchange: rows");
  oxb::ArgmaxExchangeParams p{};
  p.logits = logits.data_ptr<float>();
  p.ld = logits.stride(0);
  p.V_local = static_cast<int>(logits.size(1));
  p.vocab_start = static_cast<int>(vocab_start);
  p.rows = static_cast<int>(logits.size(0));
  p.max_rows = static_cast<int>(max_rows);
  p.ranks = static_cast<int>(tab_ptrs.size());
  p.my_rank = static_cast<int>(my_rank);
  p.slot = static_cast<int>(slot);
  for (size_t i = 0; i < tab_ptrs.size(); ++i) {
    TORCH_CHECK(tab_ptrs[i] % 8 == 0, "argmax_exchange: table alignment");
    p.tab[i] = reinterpret_cast<unsigned long long*>(tab_ptrs[i]);
  }
  p.out_tokens = out.data_ptr<int>();
  p.status = reinterpret_cast<int*>(status.data_ptr());
  p.spin_limit = static_cast<uint32_t>(spin_limit > 0 ? spin_limit : 0);
  oxb::launch_argmax_exchange(p, cur_stream());
  check_launch("argmax_exchange");
}

// ---------------------------------------------------------------------------------------------
// peer memory (CUDA IPC): symmetric buffers that kernels address directly over NVLink
// ---------------------------------------------------------------------------------------------
int64_t ipc_alloc(int64_t bytes) {  // allocates: raw cudaMalloc so that the handle is exportable
  void* p = nullptr;
  cudaError_t e = cudaMalloc(&p, static_cast<size_t>(bytes));
  TORCH_CHECK(e == cudaSuccess, "ipc_alloc: ", cudaGetErrorString(e));
  e = cudaMemset(p, 0, static_cast<size_t>(bytes));
  TORCH_CHECK(e == cudaSuccess, "ipc_alloc memset: ", cudaGetErrorString(e));
  return reinterpret_cast<int64_t>(p);
}
void ipc_free(int64_t ptr) { cudaFree(reinterpret_cast<void*>(ptr)); }
py::bytes ipc_get_handle(int64_t ptr) {
  cudaIpcMemHandle_t h;
  cudaError_t e = cudaIpcGetMemHandle(&h, reinterpret_cast<void*>(ptr));
  TORCH_CHECK(e == cudaSuccess, "ipc_get_handle: ", cudaGetErrorString(e));
  return py::bytes(reinterpret_cast<const char*>(&h), sizeof(h));
}
int64_t ipc_open_handle(const std::string& handle) {
  TORCH_CHECK(handle.size() == sizeof(cudaIpcMemHandle_t), "ipc_open_handle: bad handle size");
  cudaIpcMemHandle_t h;
  memcpy(&h, handle.data(), sizeof(h));
  void* p = nullptr;
  cudaError_t e = cudaIpcOpenMemHandle(&p, h, cudaIpcMemLazyEnablePeerAccess);
  TORCH_CHECK(e == cudaSuccess, "ipc_open_handle: ", cudaGetErrorString(e));
  return reinterpret_cast<int64_t>(p);
}
void ipc_close_handle(int64_t ptr) { cudaIpcCloseMemHandle(reinterpret_cast<void*>(ptr)); }

Tensor tensor_from_ptr(int64_t ptr, const std::vector<int64_t>& shape, const std::string& dtype,
                       int64_t device) {
  auto dt = torch::kUInt8;
  if (dtype == "bf16") dt = torch::kBFloat16;
  else if (dtype == "f32") dt = torch::kFloat32;
  else if (dtype == "i32") dt = torch::kInt32;
  else if (dtype == "u8") dt = torch::kUInt8;
  else TORCH_CHECK(false, "tensor_from_ptr: unknown dtype ", dtype);
  auto opts = torch::TensorOptions().dtype(dt).device(torch::kCUDA, static_cast<int>(device));
  return torch::from_blob(reinterpret_cast<void*>(ptr), shape, [](void*) {}, opts);
}

}  // namespace

PYBIND11_MODULE(TORCH_EXTENSION_NAME, m) {
  m.doc() = "sm_100a kernels of the B200-native Oxide engine";
  m.def("gemm_bf16", &gemm_bf16);
  m.def("quant_act_nvfp4", &quant_act_nvfp4);
  m.def("gemm_max_fixup_splits", &oxb::gemm_max_fixup_splits);
  m.def("set_pdl", [](bool on) { oxb::pdl_enabled() = on; },
        "programmatic dependent launch of the GEMM / finalize / RoPE / decode-attention kernels");
  m.def("pdl_enabled", []() { return oxb::pdl_enabled(); });
  m.def("gemm_fp8_block", &gemm_fp8_block);
  m.def("quant_act_fp8", &quant_act_fp8);
  m.def("paged_decode", &paged_decode);
  m.def("paged_prefill_tc", &paged_prefill_tc);
  m.def("finalize_norm", &finalize_norm);
  m.def("qkv_rope_append", &qkv_rope_append);
  m.def("swiglu", &swiglu);
  m.def("embed_gather", &embed_gather);
  m.def("cast_acc_bf16", &cast_acc_bf16);
  m.def("fwht128", &fwht128);
  m.def("kv_block_copy", &kv_block_copy);
  m.def("softcap", &softcap);
  m.def("alloc_mapped_host", &alloc_mapped_host);
  m.def("advance_decode_step", &advance_decode_step);
  m.def("gemm_packed", &gemm_packed);
  m.def("mmvq_mixed", &mmvq_mixed);
  m.def("mmvq_has_int8_path", [](int64_t t) { return oxb::mmvq_has_int8_path(static_cast<int>(t)); });
  m.def("mmvq", &mmvq);
  m.def("gemv_bf16", &gemv_bf16);
  m.def("quant_q8_1", &quant_q8_1);
  m.def("dequant_rows", &dequant_rows);
  m.def("quant_row_bytes", &quant_row_bytes);
  m.def("sample", &sample);
  m.def("argmax", &argmax);
  m.def("argmax_combine", &argmax_combine);
  m.def("argmax_exchange", &argmax_exchange);
  m.def("ipc_alloc", &ipc_alloc);
  m.def("ipc_free", &ipc_free);
  m.def("ipc_get_handle", &ipc_get_handle);
  m.def("ipc_open_handle", &ipc_open_handle);
  m.def("ipc_close_handle", &ipc_close_handle);
  m.def("tensor_from_ptr", &tensor_from_ptr);
}
