// Decode attention for callers that cannot allocate device memory.
//
// This entry point has no counterpart in luozoupi/Qwen-Triton.  It exists for host programs that
// drive the decode-attention kernel directly through the C ABI but are not in a position to call
// cudaMalloc: a plug-in running inside someone else's CUDA context under a fixed memory budget, a
// replay loop whose allocator is frozen once its buffers are laid out, or code between the begin and
// end of a stream capture, where allocation calls are not allowed at all.  Such a caller can still
// hand over its inputs and its output buffer, but it has nowhere to put the split-KV partial results
// that qt_attention_decode_mma expects as `part_acc` / `part_ml`.  Here that scratch lives inside the
// library instead, in a file-scope device array of fixed size.
//
// What to know before using it:
//  * The scratch array holds QT_STATIC_SCRATCH_FLOATS floats (8 MiB).  Every GPU that loads this
//    library reserves that much until the process exits, whether or not the function is ever called.
//  * A call needs n_seqs * nq * n_splits * (d + 2) floats of it.  Larger requests are refused with
//    QT_ERR_ARG and a message that names both numbers; nothing is launched.
//  * The first call on a device looks up the array's device address (cudaGetSymbolAddress, with that
//    device current) and raises the kernels' shared-memory limit.  Make that first call outside any
//    stream capture; later calls on the same device only launch kernels.
//  * No call allocates or frees: no cudaMalloc, cudaFree, or library routine that allocates.
//  * All calls share the one array, and it keeps whatever the previous call left.  That is harmless
//    here: every partial-result slot that the merge kernel reads is written by the split kernel of the
//    same call first (empty key ranges write an explicit "nothing" record), so nothing needs clearing.
//    But two calls whose kernels overlap on the GPU (different streams, no ordering between them)
//    race on the array and corrupt each other's results.  Serialise them.
//
// Arguments and result are those of qt_attention_decode_mma without the two scratch pointers:
// bfloat16 q [n_seqs, nq, d], paged bfloat16 caches [pages, nkv, 64, d], int32 block_table
// [n_seqs, max_blocks], int32 seq_len [n_seqs] (every entry at least 1: the query's own key is among
// those it sees; a sequence with no keys has no softmax and its output row would be 0/0), bfloat16 out
// [n_seqs, nq, d]; head_dim a multiple of 16 up to 128; nkv * ceil((nq / nkv) / 16) at most 65,535.  Returns 0, or a negative code with the text available from
// qt_last_error_attention_decode_static().
#pragma once

#ifdef __cplusplus
extern "C" {
#endif

#define QT_STATIC_SCRATCH_FLOATS (2 * 1024 * 1024)

int qt_attention_decode_static(const void* q, const void* k_cache, const void* v_cache, void* out,
                               const int* block_table, int max_blocks, const int* seq_len, int n_seqs, int nq,
                               int nkv, int d, int page_tokens, int ring_tokens, int window, float scale,
                               int n_splits, void* stream);

const char* qt_last_error_attention_decode_static(void);

#ifdef __cplusplus
}
#endif
