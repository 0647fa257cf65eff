// Token selection on the device: greedy pick, and temperature / top-k / top-p / min-p sampling.
//
// One block per logits row (float32, [rows, V]), or a cluster of eight for a large vocabulary.  The meaning of the options is the reference's
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
// top-p is exact for any distribution: the cut is found by a search on the logit value (four parts a
// pass) with sums over the row in a fixed order, so no row ever goes back to the host.  Tokens that tie with
// the cut value are all kept.
#include "common.cuh"

#define SMP_THREADS 1024
#define SMP_MAX_BLOCKS 8        // blocks that may share a row

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

// ---- a row is shared by the blocks of a cluster ------------------------------------------------
// Block `rank` of `nb` takes elements rank*SMP_THREADS + thread, then every nb*SMP_THREADS-th.  A reduction
// is taken over the block first (fixed order), written to a slot in the block's shared memory, and after a
// cluster barrier every block adds (or compares) the slots of all blocks in rank order: the same value in
// every block, the same from run to run.  Slots alternate between two sets, so one barrier a reduction
// is enough (a set is written again only after the barrier of the reduction in between).
struct SmpShared {
    float sv[32];
    int si[32];
    float scratch[32];
    float sw[32];
    float xf[2][4];
    int xi[2];
};
__device__ __forceinline__ uint32_t smp_smem(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ float smp_peer_f(const float* p, int rank) {
    uint32_t a;
    float v;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(a) : "r"(smp_smem(p)), "r"(rank));
    asm volatile("ld.shared::cluster.f32 %0, [%1];" : "=f"(v) : "r"(a));
    return v;
}
__device__ __forceinline__ int smp_peer_i(const int* p, int rank) {
    uint32_t a;
    int v;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(a) : "r"(smp_smem(p)), "r"(rank));
    asm volatile("ld.shared::cluster.s32 %0, [%1];" : "=r"(v) : "r"(a));
    return v;
}
__device__ __forceinline__ void smp_cluster_sync() {
    asm volatile("barrier.cluster.arrive.release.aligned;\nbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}

// (largest value, lowest index) over the row
__device__ void smp_row_argmax(float& v, int& i, SmpShared& sh, int nb, int& set) {
    smp_argmax(v, i, sh.sv, sh.si);
    if (nb > 1) {
        if (threadIdx.x == 0) { sh.xf[set][0] = v; sh.xi[set] = i; }
        smp_cluster_sync();
        float pv[SMP_MAX_BLOCKS];
        int pi[SMP_MAX_BLOCKS];
#pragma unroll
        for (int r = 0; r < SMP_MAX_BLOCKS; ++r) {         // all loads on their way before the first is used
            pv[r] = r < nb ? smp_peer_f(&sh.xf[set][0], r) : -INFINITY;
            pi[r] = r < nb ? smp_peer_i(&sh.xi[set], r) : 0x7fffffff;
        }
        float bv = pv[0];
        int bi = pi[0];
#pragma unroll
        for (int r = 1; r < SMP_MAX_BLOCKS; ++r)
            if (r < nb && (pv[r] > bv || (pv[r] == bv && pi[r] < bi))) { bv = pv[r]; bi = pi[r]; }
        v = bv; i = bi;
        set ^= 1;
    }
}
// sums of three values over the row: warps by shuffles, the block's warps in index order, the blocks in rank order
__device__ void smp_row_sum3(float (&v)[3], SmpShared& sh, int nb, int& set) {
#pragma unroll
    for (int j = 0; j < 3; ++j)
        for (int o = 16; o > 0; o >>= 1) v[j] += __shfl_down_sync(0xffffffffu, v[j], o);
    int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    __syncthreads();
    if (lane == 0) { sh.sv[warp] = v[0]; sh.scratch[warp] = v[1]; sh.sw[warp] = v[2]; }
    __syncthreads();
    float t[3] = {0.f, 0.f, 0.f};
    for (int w = 0; w < SMP_THREADS / 32; ++w) { t[0] += sh.sv[w]; t[1] += sh.scratch[w]; t[2] += sh.sw[w]; }
    if (nb > 1) {
        if (threadIdx.x == 0) { sh.xf[set][0] = t[0]; sh.xf[set][1] = t[1]; sh.xf[set][2] = t[2]; }
        smp_cluster_sync();
        float pv[3][SMP_MAX_BLOCKS];
#pragma unroll
        for (int j = 0; j < 3; ++j)
#pragma unroll
            for (int r = 0; r < SMP_MAX_BLOCKS; ++r) pv[j][r] = r < nb ? smp_peer_f(&sh.xf[set][j], r) : 0.f;
#pragma unroll
        for (int j = 0; j < 3; ++j) {
            t[j] = 0.f;
#pragma unroll
            for (int r = 0; r < SMP_MAX_BLOCKS; ++r) t[j] += pv[j][r];
        }
        set ^= 1;
    }
#pragma unroll
    for (int j = 0; j < 3; ++j) v[j] = t[j];
}

// how many elements of the row have a key >= each of three keys (exact in float: V < 2^24)
__device__ void smp_count_ge3(const float* l, int V, float inv_t, const unsigned int (&key)[3], unsigned int (&cnt)[3],
                              SmpShared& sh, int first, int stride, int nb, int& set) {
    int c[3] = {0, 0, 0};
    for (int i = first; i < V; i += stride) {
        unsigned int k = smp_key(l[i] * inv_t);
        c[0] += k >= key[0]; c[1] += k >= key[1]; c[2] += k >= key[2];
    }
    float f[3] = {(float)c[0], (float)c[1], (float)c[2]};
    smp_row_sum3(f, sh, nb, set);
#pragma unroll
    for (int j = 0; j < 3; ++j) cnt[j] = (unsigned int)(f[j] + 0.5f);
}
// mass exp(z - zmax) of the elements with key >= max(key[j], floor_key), for three keys
__device__ void smp_mass_ge3(const float* l, int V, float inv_t, const unsigned int (&key)[3], unsigned int floor_key,
                             float zmax, float (&mass)[3], SmpShared& sh, int first, int stride, int nb, int& set) {
    float s[3] = {0.f, 0.f, 0.f};
    for (int i = first; i < V; i += stride) {
        float z = l[i] * inv_t;
        unsigned int k = smp_key(z);
        if (k >= floor_key && k >= key[0]) {          // key[0] <= key[1] <= key[2]
            float e = expf(z - zmax);
            s[0] += e;
            if (k >= key[1]) s[1] += e;
            if (k >= key[2]) s[2] += e;
        }
    }
    smp_row_sum3(s, sh, nb, set);
#pragma unroll
    for (int j = 0; j < 3; ++j) mass[j] = s[j];
}
// The three keys that cut (lo, hi] into four parts: lo < m1 <= m2 <= m3 <= hi
__device__ __forceinline__ void smp_cuts(unsigned int lo, unsigned int hi, unsigned int (&m)[3]) {
    unsigned long long w = (unsigned long long)hi - lo;
#pragma unroll
    for (int j = 0; j < 3; ++j) m[j] = lo + (unsigned int)((w * (j + 1) + 3) / 4);
}

// params per row: temperature, top_p, min_p (float), top_k (int), seed (u64)
struct SampleRow {
    float temperature, top_p, min_p;
    int top_k;
    unsigned long long seed;
};

// grid: rows x nb blocks, the nb blocks of a row form a cluster
__global__ void __launch_bounds__(SMP_THREADS) sample_kernel(const float* __restrict__ logits, int V,
                                                            const SampleRow* __restrict__ params,
                                                            int* __restrict__ out, int nb) {
    ce_pdl_begin();
    __shared__ SmpShared sh;
    int r = blockIdx.x / nb, rank = blockIdx.x - r * nb;
    int first = rank * SMP_THREADS + threadIdx.x, stride = nb * SMP_THREADS;
    int set = 0;
    const float* l = logits + (size_t)r * V;
    SampleRow p = params[r];
    bool greedy = p.temperature <= 0.f || p.top_k == 1;
    float inv_t = greedy ? 1.f : 1.0f / fmaxf(p.temperature, 1e-5f);

    float bv = -INFINITY;
    int bi = 0x7fffffff;
    for (int i = first; i < V; i += stride) {
        float z = l[i] * inv_t;
        if (z > bv) { bv = z; bi = i; }
    }
    smp_row_argmax(bv, bi, sh, nb, set);
    if (greedy) {
        if (rank == 0 && threadIdx.x == 0) out[r] = bi == 0x7fffffff ? 0 : bi;
        if (nb > 1) smp_cluster_sync();     // nobody's slots go away while another block may still read them
        return;
    }
    float zmax = bv;
    unsigned int floor_key = 0;       // tokens with key < floor_key are dropped

    if (p.top_k > 0 && p.top_k < V) {
        // largest key with count(key' >= key) >= k: search over the 32-bit key space, four parts a pass
        unsigned int lo = 0, hi = smp_key(zmax);
        while (lo < hi) {
            unsigned int m[3], c[3];
            smp_cuts(lo, hi, m);
            smp_count_ge3(l, V, inv_t, m, c, sh, first, stride, nb, set);
            unsigned int k = (unsigned int)p.top_k;
            if (c[2] >= k) lo = m[2];
            else if (c[1] >= k) { lo = m[1]; hi = m[2] - 1; }
            else if (c[0] >= k) { lo = m[0]; hi = m[1] - 1; }
            else hi = m[0] - 1;
        }
        floor_key = lo;
    }
    if (p.top_p < 1.0f) {
        unsigned int zero[3] = {0u, 0u, 0u};
        float tot[3];
        smp_mass_ge3(l, V, inv_t, zero, floor_key, zmax, tot, sh, first, stride, nb, set);
        float target = p.top_p * tot[0];
        // largest key with mass(key' >= key) >= target
        unsigned int lo = floor_key, hi = smp_key(zmax);
        while (lo < hi) {
            unsigned int m[3];
            float ms[3];
            smp_cuts(lo, hi, m);
            smp_mass_ge3(l, V, inv_t, m, floor_key, zmax, ms, sh, first, stride, nb, set);
            if (ms[2] >= target) lo = m[2];
            else if (ms[1] >= target) { lo = m[1]; hi = m[2] - 1; }
            else if (ms[0] >= target) { lo = m[0]; hi = m[1] - 1; }
            else hi = m[0] - 1;
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
    for (int i = first; i < V; i += stride) {
        float z = l[i] * inv_t;
        if (smp_key(z) < floor_key) continue;
        float u = smp_uniform(p.seed, (unsigned long long)i);
        float g = z - logf(-logf(u));
        if (g > gv) { gv = g; gi = i; }
    }
    smp_row_argmax(gv, gi, sh, nb, set);
    if (rank == 0 && threadIdx.x == 0) out[r] = gi == 0x7fffffff ? bi : gi;
    if (nb > 1) smp_cluster_sync();
}

extern "C" int ce_sample(const float* logits, int rows, int V, const void* params, int* out, cudaStream_t stream) {
    if (rows == 0) return CE_OK;
    if (!logits || !params || !out) return ce_fail(CE_ERR_ARG, "ce_sample: null pointer");
    if (V <= 0 || V >= (1 << 24)) return ce_fail(CE_ERR_SIZE, "ce_sample: vocabulary %d not in 1..2^24", V);
    // a large vocabulary is shared by the 8 blocks of a cluster (8 SMs a row)
    // (as many blocks a row as leave every row a place on the 148 SMs at once)
    int nb = 1;
    if (V >= 16384)
        while (nb < SMP_MAX_BLOCKS && (long long)rows * nb * 2 <= ce_sm_count()) nb *= 2;
    if ((long long)rows * nb > 2147483647LL) return ce_fail(CE_ERR_SIZE, "ce_sample: %d rows", rows);
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)(rows * nb));
    cfg.blockDim = dim3(SMP_THREADS);
    cfg.stream = stream;
    cudaLaunchAttribute attr[2];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = nb; attr[0].val.clusterDim.y = 1; attr[0].val.clusterDim.z = 1;
    attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[1].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = ce_pdl_enabled() ? 2 : 1;
    ce_note("sample_kernel");
    cudaError_t e = cudaLaunchKernelEx(&cfg, sample_kernel, logits, V, (const SampleRow*)params, out, nb);
    if (e != cudaSuccess) return ce_fail(CE_ERR_CUDA, "ce_sample: %s", cudaGetErrorString(e));
    return ce_check_launch("ce_sample");
}

// Greedy pick for all rows: the first maximum of each row.  A large vocabulary is shared by the blocks of a
// cluster (block `rank` of nb takes elements rank*SMP_THREADS + thread, then every nb*SMP_THREADS-th), as in
// the sampling kernel: a decode step's few rows of 152 K logits then use 8 SMs a row instead of one (12 -> 8 us
// at batch 8).  Pairs (value, index) are compared, so the pick is the first maximum however the row is dealt.
__global__ void __launch_bounds__(SMP_THREADS) argmax_kernel(const float* __restrict__ logits, int V, int* __restrict__ out, int nb) {
    ce_pdl_begin();
    __shared__ SmpShared sh;
    int r = blockIdx.x / nb, rank = blockIdx.x % nb;
    const float* l = logits + (size_t)r * V;
    float bv = -INFINITY;
    int bi = 0x7fffffff;
    int stride = nb * SMP_THREADS;
    int i = rank * SMP_THREADS + threadIdx.x;
    // eight loads in flight per thread; indices rise within a thread, so "first maximum" holds
    for (; i + 7 * stride < V; i += 8 * stride) {
        float z[8];
#pragma unroll
        for (int k = 0; k < 8; ++k) z[k] = l[i + k * stride];
#pragma unroll
        for (int k = 0; k < 8; ++k)
            if (z[k] > bv) { bv = z[k]; bi = i + k * stride; }
    }
    for (; i < V; i += stride) {
        float z = l[i];
        if (z > bv) { bv = z; bi = i; }
    }
    int set = 0;
    smp_row_argmax(bv, bi, sh, nb, set);
    if (rank == 0 && threadIdx.x == 0) out[r] = bi == 0x7fffffff ? 0 : bi;
    if (nb > 1) smp_cluster_sync();     // nobody's slots go away while another block may still read them
}

extern "C" int ce_argmax(const float* logits, int rows, int V, int* out, cudaStream_t stream) {
    if (rows == 0) return CE_OK;
    if (!logits || !out) return ce_fail(CE_ERR_ARG, "ce_argmax: null pointer");
    if (V <= 0) return ce_fail(CE_ERR_SIZE, "ce_argmax: vocabulary %d", V);
    int nb = 1;         // (as many blocks a row as leave every row a place on the SMs at once)
    if (V >= 16384)
        while (nb < SMP_MAX_BLOCKS && (long long)rows * nb * 2 <= ce_sm_count()) nb *= 2;
    if ((long long)rows * nb > 2147483647LL) return ce_fail(CE_ERR_SIZE, "ce_argmax: %d rows", rows);
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)(rows * nb));
    cfg.blockDim = dim3(SMP_THREADS);
    cfg.stream = stream;
    cudaLaunchAttribute attr[2];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = nb; attr[0].val.clusterDim.y = 1; attr[0].val.clusterDim.z = 1;
    attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[1].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = ce_pdl_enabled() ? 2 : 1;
    ce_note("argmax_kernel");
    cudaError_t e = cudaLaunchKernelEx(&cfg, argmax_kernel, logits, V, out, nb);
    if (e != cudaSuccess) return ce_fail(CE_ERR_CUDA, "ce_argmax: %s", cudaGetErrorString(e));
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
    { ce_note("penalties_kernel"); ce_launch(penalties_kernel, (n + 255) / 256, 256, 0, stream, logits, V, entries, n, row_params); }
    return ce_check_launch("ce_apply_penalties");
}
