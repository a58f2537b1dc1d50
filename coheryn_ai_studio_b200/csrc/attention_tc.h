// The tcgen05 attention kernel for prompt portions (attention_tc.cu), as the dispatcher in
// attention_bf16.cu sees it.  Both live in the per-head-size attention library.
#pragma once
#include <cuda_runtime.h>

// Whether the kernel handles this head grouping and page size at the compiled head size.
bool coheryn_attention_tc_takes(int nh, int nkv, int page_size);

// CTAs per row tile that split its key tiles (1, 2, 4 or 8; 0: chosen by shape).  For tests.
void coheryn_attention_tc_set_cluster(int cluster);

// Whether a CTA takes two consecutive row tiles and fetches every key tile once for both (head
// sizes up to 128, unsplit row tiles): 0 never, 1 always, 2 when the pairs still fill the GPU (the
// default).  For tests.
void coheryn_attention_tc_set_two_tiles(int mode);

// Attention of every request of the batch with more than 16 rows per kv head (all requests
// when skip_small is 0).  q: [total_tokens, >= nh * HD] bfloat16 rows of stride q_stride;
// caches: [num_pages][nkv][page_size][HD]; max_rows and max_kv_len bound the batch's rows per kv head and
// lengths.  Returns 0, or -1 with the library's error set.
int coheryn_attention_tc_launch(const void* q, long q_stride, int total_tokens, void* out, long out_stride,
                                const void* k_cache, const void* v_cache, int num_pages, const int* block_tables,
                                int max_blocks, const int* cu_q, const int* kv_lens, int B, int nh, int nkv,
                                int page_size, int window, float scale_log2, int max_rows, int max_kv_len, int skip_small,
                                int* status, cudaStream_t stream);
