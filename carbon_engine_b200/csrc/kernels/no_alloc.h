// An entry point for callers that cannot allocate device memory.
//
// This has no counterpart in the reference.  It exists for hosts that drive the engine's kernels
// from a place where cudaMalloc is off limits: a plug-in inside another process's memory pool, a
// real-time loop that must not take the allocator's lock, a runtime that has handed all device
// memory to its own arena.  Such a caller still owns its inputs and outputs, but has nowhere to put
// the scratch memory that the split-KV decode attention needs between its two kernels.
//
// ce_attention_decode_bf16_static() is ce_attention_decode_bf16() with that scratch taken from a
// fixed array inside the library instead of from the caller.  See attention_decode_static.cu.
#pragma once
#include <cuda_runtime.h>

#ifdef __cplusplus
extern "C" {
#endif

// Floats of scratch the library holds per GPU for this entry point (8 MiB), and its counter slots.
#define CE_STATIC_SCRATCH_FLOATS (2 * 1024 * 1024)
#define CE_STATIC_COUNTERS 4096

// Same arguments and result as ce_attention_decode_bf16, without `scratch`, `counters`, `n_counters`.
// Returns CE_ERR_SIZE (-1) if n_seqs * nh * max_splits * (d + 2) exceeds CE_STATIC_SCRATCH_FLOATS.
int ce_attention_decode_bf16_static(const void* q, const void* k_pool, const void* v_pool, void* out,
                                    const int* positions, const int* seq_slot, const int* q_start, const int* ctx_len,
                                    const int* block_table, int* status, int n_seqs, int nh, int nkv, int d,
                                    int q_stride, int page_size, int max_pages, int num_pages, int window, float scale,
                                    int max_splits, cudaStream_t stream);

#ifdef __cplusplus
}
#endif
