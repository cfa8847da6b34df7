// Parameter blocks of the fused "finalize" kernels that sit between GEMMs:
// reduce-scatter tail + residual + RMSNorm + all-gather push, QKV bias/QK-norm/RoPE/KV-append,
// SwiGLU, embedding gather.
#pragma once
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace oxb {

constexpr int kMaxPeers = 8;

// Same layout as RowMeta of the GEMM: home rank, home row and routing weight of a slab row.
struct MoeRowMeta {
  int rank;
  int row;
  float weight;
  int pad;
};

struct FinalizeNormParams {
  float* acc;               // [rows, N] fp32 accumulator owned by this rank (nullable); zeroed here
  const __nv_bfloat16* rs_slab; // [n_slabs, slab rows, N] bf16 partials, one slab per source rank (nullable)
  int n_slabs;
  long long slab_stride;    // elements between slabs
  const uint32_t* arrive;   // local arrival counter the accumulator's writers bump (nullable)
  uint32_t expected;        // arrivals to wait for
  uint32_t* ticket;         // local ticket; the last CTA re-arms `arrive`
  const __nv_bfloat16* residual_in;  // [rows, N] (nullable)
  __nv_bfloat16* residual_out;       // [rows, N] (nullable)
  const __nv_bfloat16* bias;         // [N] (nullable)
  const __nv_bfloat16* norm_w;       // [N] (nullable: no normalisation, out = h)
  float eps;
  float w_offset;           // added to the norm weight (Gemma: 1.0)
  __nv_bfloat16* out[kMaxPeers];   // destination buffers ([*, N]); rows land at out_row_off + r
  uint32_t* out_flag[kMaxPeers];   // counter to bump on each destination (nullable entries)
  int n_dst;
  long long out_row_off;
  const int* out_row_map;   // optional [rows]: destination row (replaces out_row_off + r); < 0 = skip
  int rows, N;
  int* status;
  uint32_t spin_limit;      // iterations of the bounded arrival wait (0 = OXB_SPIN_LIMIT)
  // Optional int8 view of the output rows for the integer GEMV that consumes them (the same numbers
  // as launch_quant_q8_1 on the bf16 output): q8 [*, N] int8, q8_d / q8_s [*, N / 32] block scale and
  // scale * sum, indexed by the destination row. N must be a multiple of 32.
  int8_t* q8;
  float* q8_d;
  float* q8_s;
  // --- MoE dispatch mode (router_w != nullptr): the normed row goes only to the ranks that own
  //     its top-k experts, into that expert's receive slab, instead of to out[] ---
  const __nv_bfloat16* router_w;  // [n_experts, N]
  int n_experts, top_k, experts_per_rank;
  float routed_scale;             // multiplies the routing weights (1.0 for Mixtral)
  __nv_bfloat16* slab[kMaxPeers];  // on rank o: [experts_per_rank, cap, N]
  MoeRowMeta* meta[kMaxPeers];     // on rank o: [experts_per_rank, cap]
  uint32_t* slab_cnt[kMaxPeers];   // on rank o: [experts_per_rank] rows used so far
  int cap;                         // rows per expert slab
  int my_rank;
};
void launch_finalize_norm(const FinalizeNormParams& p, cudaStream_t stream);

struct QkvRopeParams {
  const float* acc_f32;          // [M, (Hq+2Hkv)*D] fp32 (zeroed after the read) or nullptr
  const __nv_bfloat16* qkv_bf16; // same shape in bf16 when acc_f32 is nullptr
  const __nv_bfloat16* bias;     // [(Hq+2Hkv)*D] nullable
  const __nv_bfloat16* q_norm_w; // [D] nullable (per-head RMSNorm before RoPE)
  const __nv_bfloat16* k_norm_w; // [D] nullable
  float norm_eps, norm_w_offset;
  const int* positions;          // [M]
  const long long* slot_mapping; // [M], slot = block * 16 + offset; < 0 = do not store
  const float* inv_freq;         // [D/2]
  float rope_mscale;             // attention scaling of YaRN-style tables (1.0 otherwise)
  __nv_bfloat16* q_out;          // [M, Hq*D]
  __nv_bfloat16* k_cache;        // [blocks, Hkv, 16, D]
  __nv_bfloat16* v_cache;
  int M, Hq, Hkv, D;
  long long num_slots;           // bound for slot indices
  int* status;
};
void launch_qkv_rope_append(const QkvRopeParams& p, cudaStream_t stream);

struct SwigluParams {
  const float* acc_f32;            // [M, 2I] gate | up (zeroed after the read) or nullptr
  const __nv_bfloat16* gu_bf16;    // same in bf16 when acc_f32 is nullptr
  __nv_bfloat16* out;              // [M, I]
  int M, I;
  int act;                         // 0 = SiLU (SwiGLU), 1 = tanh-GELU (GeGLU)
  // optional int8 view of `out` (see FinalizeNormParams::q8); I must be a multiple of 32
  int8_t* q8;
  float* q8_d;
  float* q8_s;
};
void launch_swiglu(const SwigluParams& p, cudaStream_t stream);

void launch_embed_gather(const int* tokens, const __nv_bfloat16* table, __nv_bfloat16* out, int M,
                         int N, int vocab, float scale, int vocab_start, cudaStream_t stream);
void launch_cast_acc_bf16(float* acc, const __nv_bfloat16* bias, __nv_bfloat16* out, int M, int N,
                          long long ldo, cudaStream_t stream);
void launch_fwht128(float* x, long long n_blocks, cudaStream_t stream);
void launch_kv_block_copy(__nv_bfloat16* k_cache, __nv_bfloat16* v_cache, const int* src_blocks,
                          const int* dst_blocks, int n_pairs, long long block_elems,
                          cudaStream_t stream);
void launch_softcap(float* logits, long long n, float cap, cudaStream_t stream);

// In-graph step advance of a decode burst: after the step's argmax, row r of the step descriptor is
// rewritten for the next step (token = the sampled id, position and length + 1, KV slot of the new
// position from the row's block table), and the sampled ids are posted to a ring in mapped pinned
// host memory that the host polls, so that several replays of the decode graph run back to back
// without a host round trip. Mailbox word = (step number << 32) | token; the step counter lives on
// the device and counts from 1.
struct AdvanceStepParams {
  int* token_ids;            // [rows]
  int* positions;            // [rows]
  long long* slot_mapping;   // [rows]
  int* seq_lens;             // [rows]
  const int* block_tables;   // [rows, max_blocks]
  const int* sampled;        // [rows] this step's argmax
  unsigned long long* mailbox;  // device address of mapped host memory, [ring][rows]
  unsigned int* step_counter;   // device, [1]
  int rows, max_blocks, ring;
  int* status;               // a position past the block-table row is recorded (kStatusBadIndex), the row stops advancing
};
void launch_advance_decode_step(const AdvanceStepParams& p, cudaStream_t stream);

}  // namespace oxb
