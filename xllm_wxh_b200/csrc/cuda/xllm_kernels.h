/* C interface of libxllm_kernels.so that is meant to be called from outside the Python package.
 *
 * Every function takes raw device pointers and a CUDA stream (0 = default stream) and returns 0 on success or a
 * negative code (-1 CUDA error, -2 bad argument, -3 unsupported shape, -4 descriptor error, -5 size limit).
 */
#pragma once
#ifdef __cplusplus
extern "C" {
#endif

/* Split-KV paged GQA decode attention that allocates nothing.
 *
 * This entry point has no counterpart in the reference engine.  It exists for callers that cannot call cudaMalloc
 * (or any allocating library routine) at the point where they need attention: code that runs inside another
 * framework's memory plan, a host thread that must not touch the allocator while a CUDA graph is being captured
 * elsewhere in the process, or an embedding application that hands this library a fixed set of buffers and
 * forbids it to create more.  The regular path (`xl_decode_attention_tma` + `xl_decode_split_merge`) expects the
 * caller to provide the split-KV workspace and uses a library-allocated status word and a heap-backed descriptor
 * cache; this variant keeps the workspace and the status word in device arrays that are part of the library image
 * and builds its TMA descriptors on the stack.  It calls no cudaMalloc, cudaFree, or other allocating routine.
 *
 * Inputs / outputs (all caller-owned, device memory, bf16 unless noted):
 *   q            [rows, n_q * head_dim] with row pitch `q_stride` elements; sequence i owns rows q_cu[i]..q_cu[i+1]
 *   k_cache/v_cache [num_blocks_total, block_size, n_kv, head_dim]
 *   out          [rows, n_q * head_dim]
 *   q_cu         int32 [n_seqs + 1], kv_lens int32 [n_seqs], block_tables int32 [n_seqs, max_blocks]
 *   max_rows     upper bound of q_cu[n_seqs] (rows in this call); (n_q / n_kv) * rows-per-sequence must be <= 16.  Both
 *                are checked again on the device against the real q_cu: a sequence beyond either limit is skipped (its
 *                output rows are left untouched) and XL_ERR_BOUNDS (6) is recorded in the status word below
 *   num_splits   KV splits per (sequence, kv head); 1 needs no workspace at all
 *   err/err_len  optional buffer that receives a message when the call is rejected
 *
 * Limits and rules:
 *   - the built-in workspace is 16 MiB: max_rows * n_q * num_splits * (head_dim + 1) * 4 bytes must fit, otherwise
 *     the call returns -5 and launches nothing; every GPU that loads the library holds these 16 MiB until exit;
 *   - the first call on each device looks up the arrays' device addresses (cudaGetSymbolAddress, with that device
 *     current); make that first call before any stream capture begins;
 *   - all calls on one device share the workspace, which simply keeps the previous call's partial results: nothing
 *     in it has to start at zero (each call overwrites every slot it later reads; slots of skipped sequences are not
 *     read), but two calls whose kernels overlap on the GPU (different streams, no dependency) race on it; serialise
 *     them.
 */
int xl_decode_attention_noalloc(const void* q, const void* k_cache, const void* v_cache, void* out, const void* q_cu,
                                const void* kv_lens, const void* block_tables, int n_seqs, int max_rows, int max_blocks,
                                int block_size, int num_blocks_total, int n_q, int n_kv, int head_dim, int q_stride, float scale,
                                int num_splits, void* stream, char* err, int err_len);

/* Status word of the allocation-free entry point on the current device (also without a counterpart in the reference):
 * 0 when every kernel it launched so far ran to the end, otherwise the code recorded last (1..4 a bounded wait expired,
 * 6 a sequence was skipped for its size).  Synchronises `stream`, clears the word, allocates nothing.  -1: the entry
 * point has not run on this device yet, or a CUDA call failed. */
int xl_decode_attention_noalloc_status(void* stream);

#ifdef __cplusplus
}
#endif
