// Split-KV decode attention for callers that may not allocate: the scratch memory between the
// split kernel and the merge kernel lives in a fixed array of this library.
//
// What a caller has to know:
//  * The array is CE_STATIC_SCRATCH_FLOATS floats (8 MiB) plus CE_STATIC_COUNTERS ints.  Every GPU
//    that loads this library holds them from load until the process exits, used or not.
//  * A call whose partial results do not fit (n_seqs * nh * max_splits * (head_dim + 2) floats) is
//    refused with an error; nothing is launched.
//  * The first call on each device looks up the array's device address (cudaGetSymbolAddress, with
//    that device current).  That is a set-up step, not a stream operation: make the first call on a
//    device before you start capturing a stream.
//  * No call allocates or frees: no cudaMalloc, no cudaFree, no library routine that allocates.
//  * All calls on a device share the one array.  The partial results of a call are dead once its
//    merge kernel has run, so calls that follow each other in one stream are fine; two calls that can
//    run on the GPU at the same time (different streams, no dependency between them) would write
//    over each other's partials.  Do not overlap them.
//  * The counters must be zero when the split kernel starts; they are cleared on the stream before
//    every launch, since the array keeps whatever the last call left.
#include "common.cuh"
#include "no_alloc.h"
#include <mutex>

extern "C" long long ce_attention_decode_scratch(int n_seqs, int nh, int d, int max_splits);
extern "C" int ce_attention_decode_bf16(const void* q, const void* k_pool, const void* v_pool, void* out, float* scratch,
                                        int* counters, int n_counters, const int* positions, const int* seq_slot,
                                        const int* q_start, const int* ctx_len, const int* block_table, int* status,
                                        int n_seqs, int nh, int nkv, int d, int q_stride, int page_size, int max_pages,
                                        int num_pages, int window, float scale, int max_splits, cudaStream_t stream);

// In host code these names are host-side stand-ins for the device arrays, not device addresses:
// a kernel must be given what cudaGetSymbolAddress returns for them.
static __device__ __align__(256) float g_static_scratch[CE_STATIC_SCRATCH_FLOATS];
static __device__ __align__(256) int g_static_counters[CE_STATIC_COUNTERS];

namespace {
constexpr int MAX_DEVICES = 64;
struct DeviceArrays { float* scratch; int* counters; bool ready; };
DeviceArrays g_arrays[MAX_DEVICES];
std::mutex g_setup;

// The device addresses of the arrays on the current device; looked up once per device.
int arrays_of_current_device(DeviceArrays* out) {
    int dev = -1;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return ce_fail(CE_ERR_CUDA, "ce_attention_decode_bf16_static: cudaGetDevice: %s", cudaGetErrorString(e));
    if (dev < 0 || dev >= MAX_DEVICES) return ce_fail(CE_ERR_SIZE, "ce_attention_decode_bf16_static: device %d", dev);
    std::lock_guard<std::mutex> lock(g_setup);
    if (!g_arrays[dev].ready) {
        float* s = nullptr;
        int* c = nullptr;
        e = cudaGetSymbolAddress((void**)&s, g_static_scratch);
        if (e != cudaSuccess) return ce_fail(CE_ERR_CUDA, "ce_attention_decode_bf16_static: scratch address: %s", cudaGetErrorString(e));
        e = cudaGetSymbolAddress((void**)&c, g_static_counters);
        if (e != cudaSuccess) return ce_fail(CE_ERR_CUDA, "ce_attention_decode_bf16_static: counter address: %s", cudaGetErrorString(e));
        g_arrays[dev] = DeviceArrays{s, c, true};
    }
    *out = g_arrays[dev];
    return CE_OK;
}
}  // namespace

extern "C" int ce_attention_decode_bf16_static(const void* q, const void* k_pool, const void* v_pool, void* out,
                                               const int* positions, const int* seq_slot, const int* q_start,
                                               const int* ctx_len, const int* block_table, int* status, int n_seqs,
                                               int nh, int nkv, int d, int q_stride, int page_size, int max_pages,
                                               int num_pages, int window, float scale, int max_splits,
                                               cudaStream_t stream) {
    if (n_seqs == 0) return CE_OK;
    if (n_seqs < 0 || nh <= 0 || nkv <= 0 || d <= 0 || max_splits <= 0)
        return ce_fail(CE_ERR_SIZE, "ce_attention_decode_bf16_static: bad sizes");
    long long need = ce_attention_decode_scratch(n_seqs, nh, d, max_splits);
    if (need > CE_STATIC_SCRATCH_FLOATS)
        return ce_fail(CE_ERR_SIZE, "ce_attention_decode_bf16_static: %lld floats of scratch needed, the library holds %d "
                       "(n_seqs * heads * max_splits * (head_dim + 2) must not exceed it)", need, CE_STATIC_SCRATCH_FLOATS);
    long long counters = (long long)n_seqs * nkv * ((nh / nkv + 15) / 16);
    if (counters > CE_STATIC_COUNTERS)
        return ce_fail(CE_ERR_SIZE, "ce_attention_decode_bf16_static: %lld counters needed, the library holds %d", counters,
                       CE_STATIC_COUNTERS);
    DeviceArrays arr;
    int rc = arrays_of_current_device(&arr);
    if (rc) return rc;
    cudaError_t e = cudaMemsetAsync(arr.counters, 0, (size_t)counters * sizeof(int), stream);
    if (e != cudaSuccess) return ce_fail(CE_ERR_CUDA, "ce_attention_decode_bf16_static: clearing counters: %s", cudaGetErrorString(e));
    return ce_attention_decode_bf16(q, k_pool, v_pool, out, arr.scratch, arr.counters, CE_STATIC_COUNTERS, positions, seq_slot,
                                    q_start, ctx_len, block_table, status, n_seqs, nh, nkv, d, q_stride, page_size, max_pages,
                                    num_pages, window, scale, max_splits, stream);
}
