// Token selection on the device: greedy pick, and temperature / top-k / top-p / min-p sampling.
//
// One block per logits row (float32, [rows, V]).  The meaning of the options is the reference's
// host sampler's (src/sampling.rs:137-181): logits are scaled by 1/max(T, 1e-5); top-k keeps the
// k largest; the softmax is taken over what top-k kept; top-p keeps the shortest prefix of the
// descending order whose mass reaches p; min-p drops tokens below min_p times the largest
// probability; one token is drawn from what is left.  Greedy (temperature <= 0 or top_k == 1,
// src/sampling.rs:48-50) returns the first maximum, the lowest index on ties
// (src/sampling.rs:96-106).
//
// The draw is an exact Gumbel-max over the kept set, as in the reference's device sampler when no
// nucleus is asked for (src/kernels/sampling.cu:161-182), with its counter-based uniform numbers
// (splitmix64 finaliser of seed and index, src/kernels/sampling.cu:30-42).  Unlike the reference,
// top-p is exact for any distribution: the cut is found by bisection on the logit value with
// block-wide sums in a fixed order, so no row ever goes back to the host.  Tokens that tie with
// the cut value are all kept.
#include "common.cuh"

#define SMP_THREADS 1024

__device__ __forceinline__ unsigned int smp_key(float f) {   // order-preserving float -> uint
    unsigned int u = (unsigned int)__float_as_int(f);
    return (u & 0x80000000u) ? ~u : (u | 0x80000000u);
}
__device__ __forceinline__ float smp_unkey(unsigned int k) {
    unsigned int u = (k & 0x80000000u) ? (k & 0x7fffffffu) : ~k;
    return __int_as_float((int)u);
}
__device__ __forceinline__ unsigned long long smp_mix(unsigned long long x) {
    x += 0x9e3779b97f4a7c15ull;
    x = (x ^ (x >> 30)) * 0xbf58476d1ce4e5b9ull;
    x = (x ^ (x >> 27)) * 0x94d049bb133111ebull;
    return x ^ (x >> 31);
}
__device__ __forceinline__ float smp_uniform(unsigned long long seed, unsigned long long i) {
    unsigned long long h = smp_mix(seed ^ smp_mix(i + 0x632be59bd9b4e019ull));
    return ((float)(h >> 40) + 0.5f) * (1.0f / 16777216.0f);
}

// (largest value, lowest index) over the block, fixed order
__device__ void smp_argmax(float& v, int& i, float* sv, int* si) {
    for (int o = 16; o > 0; o >>= 1) {
        float ov = __shfl_down_sync(0xffffffffu, v, o);
        int oi = __shfl_down_sync(0xffffffffu, i, o);
        if (ov > v || (ov == v && oi < i)) { v = ov; i = oi; }
    }
    int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    __syncthreads();
    if (lane == 0) { sv[warp] = v; si[warp] = i; }
    __syncthreads();
    float bv = sv[0];
    int bi = si[0];
    for (int w = 1; w < SMP_THREADS / 32; ++w)
        if (sv[w] > bv || (sv[w] == bv && si[w] < bi)) { bv = sv[w]; bi = si[w]; }
    v = bv;
    i = bi;
}

__device__ unsigned int smp_count_ge(const float* l, int V, float inv_t, unsigned int key, float* scratch) {
    int c = 0;
    for (int i = threadIdx.x; i < V; i += SMP_THREADS) c += smp_key(l[i] * inv_t) >= key;
    // counts are exact in float up to 2^24; V is far below that
    return (unsigned int)(ce_block_sum((float)c, scratch) + 0.5f);
}

__device__ float smp_mass_ge(const float* l, int V, float inv_t, unsigned int key, unsigned int floor_key, float zmax,
                             float* scratch) {
    float s = 0.f;
    for (int i = threadIdx.x; i < V; i += SMP_THREADS) {
        float z = l[i] * inv_t;
        unsigned int k = smp_key(z);
        if (k >= key && k >= floor_key) s += expf(z - zmax);
    }
    return ce_block_sum(s, scratch);
}

// params per row: temperature, top_p, min_p (float), top_k (int), seed (u64)
struct SampleRow {
    float temperature, top_p, min_p;
    int top_k;
    unsigned long long seed;
};

__global__ void __launch_bounds__(SMP_THREADS) sample_kernel(const float* __restrict__ logits, int V,
                                                            const SampleRow* __restrict__ params,
                                                            int* __restrict__ out) {
    ce_pdl_begin();
    __shared__ float sv[32];
    __shared__ int si[32];
    __shared__ float scratch[32];
    int r = blockIdx.x;
    const float* l = logits + (size_t)r * V;
    SampleRow p = params[r];
    bool greedy = p.temperature <= 0.f || p.top_k == 1;
    float inv_t = greedy ? 1.f : 1.0f / fmaxf(p.temperature, 1e-5f);

    float bv = -INFINITY;
    int bi = 0x7fffffff;
    for (int i = threadIdx.x; i < V; i += SMP_THREADS) {
        float z = l[i] * inv_t;
        if (z > bv) { bv = z; bi = i; }
    }
    smp_argmax(bv, bi, sv, si);
    if (greedy) {
        if (threadIdx.x == 0) out[r] = bi == 0x7fffffff ? 0 : bi;
        return;
    }
    float zmax = bv;
    unsigned int floor_key = 0;       // tokens with key < floor_key are dropped

    if (p.top_k > 0 && p.top_k < V) {
        // largest key with count(key' >= key) >= k : bisection over the 32-bit key space
        unsigned int lo = 0, hi = smp_key(zmax);
        while (lo < hi) {
            unsigned int mid = lo + (hi - lo + 1) / 2;
            if (smp_count_ge(l, V, inv_t, mid, scratch) >= (unsigned int)p.top_k) lo = mid; else hi = mid - 1;
        }
        floor_key = lo;
    }
    if (p.top_p < 1.0f) {
        float total = smp_mass_ge(l, V, inv_t, 0u, floor_key, zmax, scratch);
        float target = p.top_p * total;
        // largest key with mass(key' >= key) >= target
        unsigned int lo = floor_key, hi = smp_key(zmax);
        while (lo < hi) {
            unsigned int mid = lo + (hi - lo + 1) / 2;
            if (smp_mass_ge(l, V, inv_t, mid, floor_key, zmax, scratch) >= target) lo = mid; else hi = mid - 1;
        }
        floor_key = max(floor_key, lo);
    }
    if (p.min_p > 0.f) {
        // p_i >= min_p * p_max  <=>  exp(z_i - zmax) >= min_p
        float cut = zmax + logf(p.min_p);
        unsigned int k = smp_key(cut);
        // the maximum itself always stays
        floor_key = max(floor_key, min(k, smp_key(zmax)));
    }
    float gv = -INFINITY;
    int gi = 0x7fffffff;
    for (int i = threadIdx.x; i < V; i += SMP_THREADS) {
        float z = l[i] * inv_t;
        if (smp_key(z) < floor_key) continue;
        float u = smp_uniform(p.seed, (unsigned long long)i);
        float g = z - logf(-logf(u));
        if (g > gv) { gv = g; gi = i; }
    }
    smp_argmax(gv, gi, sv, si);
    if (threadIdx.x == 0) out[r] = gi == 0x7fffffff ? bi : gi;
}

extern "C" int ce_sample(const float* logits, int rows, int V, const void* params, int* out, cudaStream_t stream) {
    if (rows == 0) return CE_OK;
    if (!logits || !params || !out) return ce_fail(CE_ERR_ARG, "ce_sample: null pointer");
    if (V <= 0 || V >= (1 << 24)) return ce_fail(CE_ERR_SIZE, "ce_sample: vocabulary %d not in 1..2^24", V);
    ce_launch(sample_kernel, rows, SMP_THREADS, 0, stream, logits, V, (const SampleRow*)params, out);
    return ce_check_launch("ce_sample");
}

// Greedy pick for all rows: the first maximum of each row.
__global__ void __launch_bounds__(SMP_THREADS) argmax_kernel(const float* __restrict__ logits, int V, int* __restrict__ out) {
    ce_pdl_begin();
    __shared__ float sv[32];
    __shared__ int si[32];
    int r = blockIdx.x;
    const float* l = logits + (size_t)r * V;
    float bv = -INFINITY;
    int bi = 0x7fffffff;
    int i = threadIdx.x;
    // eight loads in flight per thread; indices rise within a thread, so "first maximum" holds
    for (; i + 7 * SMP_THREADS < V; i += 8 * SMP_THREADS) {
        float z[8];
#pragma unroll
        for (int k = 0; k < 8; ++k) z[k] = l[i + k * SMP_THREADS];
#pragma unroll
        for (int k = 0; k < 8; ++k)
            if (z[k] > bv) { bv = z[k]; bi = i + k * SMP_THREADS; }
    }
    for (; i < V; i += SMP_THREADS) {
        float z = l[i];
        if (z > bv) { bv = z; bi = i; }
    }
    smp_argmax(bv, bi, sv, si);
    if (threadIdx.x == 0) out[r] = bi == 0x7fffffff ? 0 : bi;
}

extern "C" int ce_argmax(const float* logits, int rows, int V, int* out, cudaStream_t stream) {
    if (rows == 0) return CE_OK;
    if (!logits || !out) return ce_fail(CE_ERR_ARG, "ce_argmax: null pointer");
    if (V <= 0) return ce_fail(CE_ERR_SIZE, "ce_argmax: vocabulary %d", V);
    ce_launch(argmax_kernel, rows, SMP_THREADS, 0, stream, logits, V, out);
    return ce_check_launch("ce_argmax");
}

// Penalties on the logits of one row (src/sampling.rs:108-134): for every token seen in the prompt
// or the output, divide a positive logit by the repetition penalty or multiply a negative one; for
// every token of the output, subtract presence + frequency * count.
// entries: [n, 4] int32 = (row, token, seen flag, count in the output)
__global__ void penalties_kernel(float* __restrict__ logits, int V, const int* __restrict__ entries, int n,
                                 const float* __restrict__ row_params /* [rows, 3] rep, presence, frequency */) {
    ce_pdl_begin();
    int e = blockIdx.x * blockDim.x + threadIdx.x;
    if (e >= n) return;
    int row = entries[4 * e], tok = entries[4 * e + 1], seen = entries[4 * e + 2], cnt = entries[4 * e + 3];
    if (tok < 0 || tok >= V) return;
    float rep = row_params[3 * row], pres = row_params[3 * row + 1], freq = row_params[3 * row + 2];
    float* l = logits + (size_t)row * V + tok;
    float v = *l;
    if (seen && rep != 1.0f) v = v > 0.f ? v / rep : v * rep;
    if (cnt > 0 && (pres != 0.f || freq != 0.f)) v -= pres + freq * (float)cnt;
    *l = v;
}

extern "C" int ce_apply_penalties(float* logits, int V, const int* entries, int n, const float* row_params,
                                  cudaStream_t stream) {
    if (n == 0) return CE_OK;
    if (!logits || !entries || !row_params) return ce_fail(CE_ERR_ARG, "ce_apply_penalties: null pointer");
    ce_launch(penalties_kernel, (n + 255) / 256, 256, 0, stream, logits, V, entries, n, row_params);
    return ce_check_launch("ce_apply_penalties");
}
