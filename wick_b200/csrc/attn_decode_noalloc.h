/* Decode attention without any device allocation.
 *
 * This entry point has no counterpart in pMag11-alt/wick.  It exists for hosts
 * that must not, or cannot, allocate GPU memory themselves: code that runs
 * inside someone else's memory pool, a latency-critical loop where cudaMalloc's
 * implicit synchronisation is unacceptable, or a deployment whose device memory
 * is handed out once at start-up.  Such a host still owns the inputs (q, the
 * cache, the length and page tables) and the output; the only thing the
 * ordinary entry point (wick_attn_decode_bf16) would ask of it in addition, a
 * scratch buffer for partial results, lives inside the library instead.
 *
 * Limits and rules (details beside the definition in attn_decode.cu):
 *   - scratch capacity: wick_attn_decode_noalloc_capacity() floats (8 MiB),
 *     resident on every GPU that loads the library; larger problems are refused;
 *   - the first call on a device looks up the array's device address; make it
 *     outside stream capture;
 *   - calls share the array: do not let two of them overlap on the GPU.
 *
 * The library is built for one head size (WICK_HD) per shared object.
 * Returns 0, or non-zero with the text available from wick_last_error().
 */
#pragma once

#ifdef __cplusplus
extern "C" {
#endif

long long wick_attn_decode_noalloc_capacity(void);

/* q, out: bfloat16 [n_seqs, n_heads, head_dim]; kv: one layer's cache, bfloat16
 * [pages, 2, n_kv, 64, head_dim]; kv_len: int32 [n_seqs], tokens cached per
 * sequence (the new token included); page_table: int32 [n_seqs, table_width];
 * max_kv_len: an upper bound of kv_len; status: device int32 that receives a
 * non-zero code if a block gave up a bounded wait (may be null); stream: a
 * cudaStream_t. */
int wick_attn_decode_noalloc_bf16(const void* q, const void* kv, void* out, const int* kv_len, int n_seqs,
                                  int max_kv_len, const int* page_table, int table_width, int n_heads, int n_kv,
                                  float scale, int* status, void* stream);

const char* wick_last_error(void);

#ifdef __cplusplus
}
#endif
