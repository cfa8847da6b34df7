/* Paged flash-decode for callers that cannot allocate device memory.
 *
 * This entry point has no counterpart in the reference engine; it exists for host programs that
 * embed the decode-attention kernel but must not call cudaMalloc themselves or through a
 * library: code running inside a region where the allocator is frozen (a pre-sized serving
 * process whose memory budget was fixed at start-up, a plugin loaded into another runtime that
 * owns the whole device heap, a real-time loop that may not take the allocator's locks).
 *
 * The regular entry point (the `paged_decode` binding) needs two scratch buffers for the
 * split-KV partial results, which its caller allocates. Here the scratch is a file-scope
 * `__device__` array inside this library: every GPU that loads the library holds
 * OXB_NOALLOC_SCRATCH_BYTES (32 MiB) until the process exits, and the call itself performs no
 * cudaMalloc / cudaFree and uses no allocating library routine.
 *
 * Set-up: the first call on a device resolves the array's device address (one
 * cudaGetSymbolAddress, with that device current) and caches it. Make that first call outside
 * any stream capture.
 *
 * Limits: batch * hq * max_splits * (head_dim + 2) + 64 floats must fit into the scratch; a larger
 * request is rejected with OXB_NOALLOC_TOO_LARGE before anything is launched. hkv and max_splits
 * are grid dimensions and may not exceed 65535.
 *
 * What is checked on the host, before any launch: null pointers, the shape rules below, 16-byte
 * alignment of q, k_cache, v_cache and out (the kernels use 16-byte loads and stores), q_stride and
 * out_stride a multiple of 8 elements and at least hq * head_dim, the size limit above (computed
 * without overflow). What is checked on the device: every block id read from a block table is
 * compared with num_blocks and a sequence length is cut at max_blocks * 16 tokens; a violation
 * reads block 0 / stops at the end of the table row instead of touching memory outside the pool,
 * and is reported through `status` when that pointer is given (the word is set to 5 once and is
 * otherwise left alone; the caller zeroes it).
 *
 * Coverage: split z of a sequence attends pages [first + z * pages_per_split, + pages_per_split),
 * so pages_per_split * max_splits * 16 must be at least the longest attended window (the longest
 * sequence, or `window` + 15 tokens with a sliding window). Tokens beyond that are left out of the
 * result without any error: the lengths live in device memory and are not known to this call.
 *
 * Sharing: all calls on a device use the same scratch, which keeps the previous call's
 * contents. The kernels overwrite every entry they later read, so nothing has to be cleared
 * between calls, but two calls that overlap on the GPU (different streams, or a graph replay
 * next to a live call) race on it. Issue calls for one device on one stream, or serialise them.
 */
#ifndef OXB_NOALLOC_H_
#define OXB_NOALLOC_H_

#ifdef __cplusplus
extern "C" {
#endif

#define OXB_NOALLOC_SCRATCH_BYTES (32u * 1024u * 1024u)

#define OXB_NOALLOC_OK 0
#define OXB_NOALLOC_BAD_ARGUMENT (-1)
#define OXB_NOALLOC_TOO_LARGE (-2)
#define OXB_NOALLOC_CUDA_ERROR (-3)

/* q           [batch, hq, head_dim] bf16, rows q_stride elements apart
 * k_cache,
 * v_cache     [num_blocks, hkv, 16, head_dim] bf16
 * block_tables[batch, max_blocks] int32, seq_lens [batch] int32 (device memory)
 * out         [batch, hq * head_dim] bf16, rows out_stride elements apart
 * num_blocks  blocks in the cache pool: bound for the ids in block_tables
 * pages_per_split >= 1 pages of 16 tokens per KV split, max_splits = grid depth (see Coverage)
 * scale       softmax scale (1/sqrt(head_dim)); window = sliding window in tokens, 0 = none
 * stream      a cudaStream_t (NULL = default stream)
 * status      optional device int32 that receives 5 when a block id or a length was out of range
 * err/err_len optional buffer that receives a message when the return value is not OXB_NOALLOC_OK
 */
int oxb_paged_decode_noalloc(const void* q, long long q_stride, const void* k_cache,
                             const void* v_cache, const int* block_tables, const int* seq_lens,
                             void* out, long long out_stride, int batch, int hq, int hkv,
                             int head_dim, int num_blocks, int max_blocks, int pages_per_split,
                             int max_splits, int window, float scale, void* stream, int* status,
                             char* err, int err_len);

#ifdef __cplusplus
}
#endif
#endif /* OXB_NOALLOC_H_ */
