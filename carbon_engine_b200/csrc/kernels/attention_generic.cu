// Causal grouped-query attention over the paged cache, for any number of new tokens per sequence,
// in plain float32 arithmetic.  It is the attention of the float32 path and the plain twin of the
// tensor-core kernels.
//
// One block per (token, query head).  The query at absolute position p sees keys lo..p, where
// lo = max(0, p - window + 1) for a windowed layer and 0 otherwise; query head h reads KV head
// h / (nh / nkv).  Keys are taken in chunks of 128 positions that start at multiples of 128, with
// an online softmax across chunks, so the order of every sum depends on p only: not on how the
// tokens were cut into steps, not on the batch, not on the pages.
//
// Semantics follow the reference's float32 kernels: scale applied to the dot product, running
// maximum and sum in float32, one rounding at the store (src/kernels/attention.cu:51-110 decode,
// :126-219 prefill; causal offset kv_len - q_len + i, src/model/attention.rs:1038-1063).
#include "common.cuh"

#define ATT_THREADS 128
#define ATT_MAX_ACC 8            // head_dim <= ATT_THREADS * ATT_MAX_ACC

struct AttnArgs {
    const void* q;               // [T, q_stride] ; head h at column h*d
    const void* k_pool;          // [num_pages, nkv, page_size, d]
    const void* v_pool;
    void* out;                   // [T, nh*d]
    const int* positions;        // [T]
    const int* seq_of_token;     // [T]
    const int* seq_slot;         // [B]
    const int* block_table;      // [slots, max_pages]
    int* status;
    int T, nh, nkv, d, q_stride, page_size, max_pages, num_pages, window;
    float scale;
};

template <typename T>
__global__ void attention_generic_kernel(AttnArgs a) {
    ce_pdl_begin();
    extern __shared__ __align__(16) unsigned char smem_raw[];
    long long* vrow = (long long*)smem_raw;           // ATT_THREADS
    float* probs = (float*)(vrow + ATT_THREADS);      // ATT_THREADS
    float* scratch = probs + ATT_THREADS;             // 32
    float* qs = scratch + 32;                         // d

    int t = blockIdx.x, h = blockIdx.y, tid = threadIdx.x, d = a.d;
    int kvh = h / (a.nh / a.nkv);
    int p = a.positions[t];
    int slot = a.seq_slot[a.seq_of_token[t]];
    const int* table = a.block_table + (size_t)slot * a.max_pages;
    const T* qrow = (const T*)a.q + (size_t)t * a.q_stride + (size_t)h * d;
    for (int j = tid; j < d; j += ATT_THREADS) qs[j] = CeType<T>::load(qrow + j);
    __syncthreads();

    int lo = a.window > 0 ? max(0, p - a.window + 1) : 0;
    float m_run = -INFINITY, l_run = 0.f;
    float acc[ATT_MAX_ACC];
#pragma unroll
    for (int i = 0; i < ATT_MAX_ACC; ++i) acc[i] = 0.f;

    for (int k0 = lo / ATT_THREADS * ATT_THREADS; k0 <= p; k0 += ATT_THREADS) {
        int key = k0 + tid;
        bool valid = key >= lo && key <= p;
        float s = -INFINITY;
        long long row = -1;
        if (valid) {
            int page = table[key / a.page_size];
            if (page < 0 || page >= a.num_pages) {
                atomicExch(a.status, 4);
                valid = false;
            } else {
                row = (((long long)page * a.nkv + kvh) * a.page_size + key % a.page_size) * d;
                const T* kr = (const T*)a.k_pool + row;
                float dot = 0.f;
                for (int j = 0; j < d; ++j) dot = fmaf(qs[j], CeType<T>::load(kr + j), dot);
                s = dot * a.scale;
            }
        }
        float m_chunk = ce_block_max(s, scratch);
        float m_new = fmaxf(m_run, m_chunk);
        float pr = valid ? expf(s - m_new) : 0.f;
        __syncthreads();                 // everyone has read scratch before it is reused
        probs[tid] = pr;
        vrow[tid] = row;
        float l_chunk = ce_block_sum(pr, scratch);   // syncs: probs/vrow visible afterwards
        float alpha = m_run == -INFINITY ? 0.f : expf(m_run - m_new);
        l_run = l_run * alpha + l_chunk;
        m_run = m_new;
        int n = min(ATT_THREADS, p - k0 + 1);
#pragma unroll
        for (int i = 0; i < ATT_MAX_ACC; ++i) {
            int j = tid + i * ATT_THREADS;
            if (j < d) {
                float o = acc[i] * alpha;
                for (int kk = 0; kk < n; ++kk) {
                    long long r = vrow[kk];
                    if (r >= 0) o = fmaf(probs[kk], CeType<T>::load((const T*)a.v_pool + r + j), o);
                }
                acc[i] = o;
            }
        }
        __syncthreads();
    }
    T* orow = (T*)a.out + ((size_t)t * a.nh + h) * d;
    float inv = l_run > 0.f ? 1.0f / l_run : 0.f;
#pragma unroll
    for (int i = 0; i < ATT_MAX_ACC; ++i) {
        int j = tid + i * ATT_THREADS;
        if (j < d) CeType<T>::store(orow + j, acc[i] * inv);
    }
}

extern "C" int ce_attention_generic(const void* q, const void* k_pool, const void* v_pool, void* out, int dtype,
                                    const int* positions, const int* seq_of_token, const int* seq_slot,
                                    const int* block_table, int* status, int T, int nh, int nkv, int d, int q_stride,
                                    int page_size, int max_pages, int num_pages, int window, float scale,
                                    cudaStream_t stream) {
    if (T == 0) return CE_OK;
    if (!q || !k_pool || !v_pool || !out || !positions || !seq_of_token || !seq_slot || !block_table || !status)
        return ce_fail(CE_ERR_ARG, "ce_attention_generic: null pointer");
    if (d <= 0 || d > ATT_THREADS * ATT_MAX_ACC)
        return ce_fail(CE_ERR_SIZE, "ce_attention_generic: head_dim %d not in 1..%d", d, ATT_THREADS * ATT_MAX_ACC);
    if (nkv <= 0 || nh % nkv != 0)
        return ce_fail(CE_ERR_SIZE, "ce_attention_generic: %d heads are not a multiple of %d kv heads", nh, nkv);
    AttnArgs a{q, k_pool, v_pool, out, positions, seq_of_token, seq_slot, block_table, status,
               T, nh, nkv, d, q_stride, page_size, max_pages, num_pages, window, scale};
    size_t smem = (d + ATT_THREADS + 32) * sizeof(float) + ATT_THREADS * sizeof(long long);
    dim3 grid(T, nh);
    if (dtype == CE_F32)
        { ce_note("attention_generic_kernel"); ce_launch(attention_generic_kernel<float>, grid, ATT_THREADS, smem, stream, a); }
    else if (dtype == CE_BF16)
        { ce_note("attention_generic_kernel"); ce_launch(attention_generic_kernel<__nv_bfloat16>, grid, ATT_THREADS, smem, stream, a); }
    else
        return ce_fail(CE_ERR_ARG, "ce_attention_generic: unknown dtype %d", dtype);
    return ce_check_launch("ce_attention_generic");
}
