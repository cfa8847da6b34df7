// Parameters of the tcgen05 bf16 GEMM  C[g][M,N] (+)= A[g][M,K] * B[g][N,K]^T  (g = group /
// expert index, 1 for a plain GEMM) and of the routed-reduction epilogue that turns it into a
// fused GEMM -> reduce-scatter (dense TP) or grouped-GEMM -> combine (MoE EP).
#pragma once
#include <cuda.h>
#include <cuda_bf16.h>
#include <stdint.h>

namespace oxb {

constexpr int kMaxRanks = 8;

enum GemmEpilogue : int {
  kEpiStoreBf16 = 0,   // C[row, col] = bf16(acc + bias[col])
  kEpiRedF32 = 1,      // dst[owner][row', col] += w * acc   (fp32 red; local or peer memory)
  kEpiStoreF32 = 2,    // C[row, col] = acc + bias[col]      (fp32)
  kEpiSwigluBf16 = 3,  // C[row, n/2] = act(gate) * up; weight rows interleaved [32 gate | 32 up]
  kEpiSlabBf16 = 4,    // dst[owner][my_rank, row', col] = bf16(acc): partial tiles stored into the
                       // row owner's receive slab (peer stores); the owner sums the slabs
};

// Per-row routing record of the MoE combine: which rank / row / weight a slab row goes back to.
struct RowMeta {
  int rank;
  int row;
  float weight;
  int pad;
};

struct GemmParams {
  int M, N, K;        // M = rows per group when group_counts == nullptr
  int kb_per_split;   // 64-wide k blocks per split
  int splits;         // number of K slices
  int m_tiles;        // M tiles of 128 * mt rows (grouped mode: upper bound over all groups, mt = 1)
  int epi;
  int act;            // kEpiSwigluBf16: 0 = SiLU, 1 = tanh-GELU
  int wide_boxes;     // 1: one TMA copy per operand and stage (A box of 256 rows; tile-major B through a
                      //    4-D map that spans both 128-row weight tiles of a 256-wide tile)
  int b_tiled;        // 1: B is stored tile-major [N/128][K/64][128][64]: every TMA box is one contiguous 16 KB
  void* C;            // kEpiStoreBf16 / kEpiStoreF32 / kEpiSwigluBf16
  long long ldc;
  long long c_group_stride;   // elements between groups of C
  const __nv_bfloat16* bias;  // optional, length N (per group: bias + g * N)
  // --- grouped (MoE) mode ---
  const uint32_t* group_counts;  // [n_groups] rows used in each group (device); nullptr = dense
  int n_groups;
  const RowMeta* row_meta;       // [n_groups, meta_group_stride] routing of each slab row
  long long meta_group_stride;
  // --- routed fp32 reduction (split-K on one GPU; reduce-scatter / combine across GPUs) ---
  float* dst[kMaxRanks];        // accumulator of owner o (a peer mapping when o != this rank)
  long long dst_ld;             // row stride of the accumulators (elements)
  uint32_t* arrive[kMaxRanks];  // counter on owner o, bumped once when this whole GEMM has landed
  uint32_t* done_ticket;        // local ticket that finds the last CTA (nullptr = no signalling)
  uint32_t* reset_on_done;      // optional local words zeroed by the last CTA before signalling
  int n_reset;
  int my_rank;                  // kEpiSlabBf16: slab index this rank writes into
  int rows_per_owner;           // dense: row r belongs to owner r / rows_per_owner
  int n_owners;
  // --- wait on the A operand (rows written into local memory by peers) ---
  const uint32_t* ag_flags;  // local counters, one per source rank; nullptr = A is ready
  uint32_t ag_expected;      // value each needed counter must reach
  int ag_rows_per_src;       // rows [s*n, (s+1)*n) come from source s; <= 0: wait for every source
  int ag_n_src;
  uint32_t* ag_ticket;       // local ticket used to re-arm the counters after the last CTA passed
  int* status;               // error word (0 = ok)
  uint32_t spin_limit;       // iterations of every bounded wait (0 = OXB_SPIN_LIMIT)
  // --- split-K with an in-kernel fix-up (store / SwiGLU / slab epilogues with splits > 1) ---
  // Every split stores its partial tile as bf16 into its own slab of `ws`, the splits of a tile
  // meet at a ticket (bounded wait; the launch is cooperative so they are co-resident), and each
  // of them then sums a share of the tile's columns over all slabs and runs the epilogue on it.
  __nv_bfloat16* ws;         // [tiles * splits][mt][BN / 8][128][8] partial tiles; nullptr = off
  uint32_t* ws_tickets;      // [2 * tiles] arrival / departure counters, zero between launches
  // --- block-scaled fp4 operands (kind = 1, NVFP4): a and w are e2m1 values packed two per byte
  // (row-major, K / 2 bytes per row), one ue4m3 scale per 16 values of K in 512-byte atoms
  // [row tile of 128][K / 64][(row % 32) * 16 + (row / 32 % 4) * 4 + (k / 16 % 4)], and the
  // accumulator of row r is multiplied by a_gscale[g * a_gs_stride + r] * w_gscale[g] ---
  int kind;                   // 0 = bf16 operands, 1 = NVFP4, 2 = bf16 A x GGUF-packed B unpacked in the kernel
  int kb_total;               // k blocks of 128 operand bytes (kind 1: K / 256; kind 0: ceil(K / 64))
  const uint8_t* sfa;         // scales of A
  const uint8_t* sfb;         // scales of B
  long long sfa_group_tiles;  // 128-row tiles per group in sfa
  const float* a_gscale;      // per-row second-level scale of A (nullable: 1)
  long long a_gs_stride;
  const float* w_gscale;      // per-group second-level scale of B (nullable: 1)
  // --- GGUF-packed weights (kind = 2): B is [N rows] of packed blocks, q_row_bytes apart, of block
  // type q_type (one with an integer expansion: Q4_0 Q4_1 Q5_0 Q5_1 Q8_0 Q4_K Q5_K Q6_K). Four extra
  // warps (one k block each, round robin) unpack the 128 x 64 weight tiles into the bf16, 128-byte-swizzled
  // operand stage that TMA would have filled; K must be a multiple of 256, 128-column tiles, not grouped. ---
  const uint8_t* qw;
  long long q_row_bytes;
  int q_type;
  // Optional timeline of every CTA (bench_gemm --trace): 8 x uint64 nanosecond stamps per CTA
  // [entry, first accumulator ready, partial stored, splits met, epilogue done, exit, 0, 0].
  unsigned long long* trace;
};

// Bytes of partial-tile workspace and number of ticket words a split-K launch with fix-up needs.
size_t gemm_ws_bytes(int M, int N, int bn, int mt, int splits);
int gemm_ws_tickets(int M, int N, int bn, int mt);
// Largest split-K factor the in-kernel fix-up takes for a tile shape (the partial slabs of one
// output unit are landed in the operand ring together).
int gemm_max_fixup_splits(int bn, int mt, bool swiglu);

// bn: 64 / 128 / 256 output columns per tile; mt: 1 or 2 row halves of 128 per tile (mt = 2 keeps
// all 256 rows of a decode batch with the CTA that streams a weight tile).
void launch_gemm_bf16(const CUtensorMap& tmA, const CUtensorMap& tmB, const GemmParams& p, int bn,
                      int mt, cudaStream_t stream);

// Activation quantiser of the NVFP4 GEMM: bf16 rows -> packed e2m1 + ue4m3 block scales (atom layout
// above) + one fp32 scale per row (row amax / (448 * 6)). Rows are [groups, rows_per_group, K];
// with group_counts only the first group_counts[g] rows of a group are converted. With wait.flags the
// kernel is the consumer of an MoE dispatch: it waits (bounded) until every source has signalled.
struct QuantActWait;  // bounded wait on arrival flags before the rows are read (gemm_fp8_block.cuh)
void launch_quant_act_nvfp4(const __nv_bfloat16* x, long long x_ld, uint8_t* q, uint8_t* sf, float* gscale,
                            int groups, int rows_per_group, int K, const uint32_t* group_counts,
                            const QuantActWait& wait, uint32_t spin_limit, cudaStream_t stream);

}  // namespace oxb
