// Memory-bound kernels of a decoder step: embedding gather, RMSNorm, the fused per-head
// q/k norm + rotary embedding + paged K/V write, the residual add and SwiGLU.
//
// The residual stream is float32 in both precisions; norms, rotation and SiLU are computed in
// float32 and rounded once at the store.  The reference gets these ops from its tensor library
// one by one (src/model/layers.rs:140-146 rms_norm, :315-325 rope, :151 silu,
// src/model/mod.rs:781-784 embedding gather, src/kvcache/mod.rs:371-372 K/V scatter).
#include "common.cuh"

// ---------------------------------------------------------------------------------------------
// Embedding: x[t, :] = float(table[token[t], :])
// ---------------------------------------------------------------------------------------------
template <typename T>
__global__ void embed_kernel(const T* __restrict__ table, const int* __restrict__ tokens,
                             float* __restrict__ x, int H, int V, int* __restrict__ status) {
    ce_pdl_begin();
    int t = blockIdx.x;
    int tok = tokens[t];
    if (tok < 0 || tok >= V) {
        if (threadIdx.x == 0) atomicExch(status, 1);
        for (int j = threadIdx.x; j < H; j += blockDim.x) x[(size_t)t * H + j] = 0.f;
        return;
    }
    const T* row = table + (size_t)tok * H;
#pragma unroll 4
    for (int j = threadIdx.x; j < H; j += blockDim.x) x[(size_t)t * H + j] = CeType<T>::load(row + j);
}

extern "C" int ce_embed(const void* table, int dtype, const int* tokens, float* x, int T, int H, int V,
                        int* status, cudaStream_t stream) {
    if (T == 0) return CE_OK;
    if (!table || !tokens || !x || !status) return ce_fail(CE_ERR_ARG, "ce_embed: null pointer");
    if (dtype == CE_F32)
        { ce_note("embed_kernel"); ce_launch(embed_kernel<float>, T, H >= 1024 ? 1024 : 256, 0, stream, (const float*)table, tokens, x, H, V, status); }
    else if (dtype == CE_BF16)
        { ce_note("embed_kernel"); ce_launch(embed_kernel<__nv_bfloat16>, T, H >= 1024 ? 1024 : 256, 0, stream, (const __nv_bfloat16*)table, tokens, x, H, V, status); }
    else
        return ce_fail(CE_ERR_ARG, "ce_embed: unknown dtype %d", dtype);
    return ce_check_launch("ce_embed");
}

// ---------------------------------------------------------------------------------------------
// RMSNorm over the last dimension: out[r, :] = x[row(r), :] * (1/sqrt(mean(x^2) + eps)) * w
// One block of 256 threads per row, so the order of the sum depends on the width only.
// ---------------------------------------------------------------------------------------------
template <typename T>
__global__ void rmsnorm_kernel(const float* __restrict__ x, const float* __restrict__ w, T* __restrict__ out,
                               const int* __restrict__ rows, int H, float eps) {
    ce_pdl_begin();
    __shared__ float scratch[32];
    int r = blockIdx.x;
    const float* xr = x + (size_t)(rows ? rows[r] : r) * H;
    float ss = 0.f;
    for (int j = threadIdx.x; j < H; j += blockDim.x) {
        float v = xr[j];
        ss = fmaf(v, v, ss);
    }
    ss = ce_block_sum(ss, scratch);
    float inv = 1.0f / sqrtf(ss / (float)H + eps);
    T* o = out + (size_t)r * H;
    for (int j = threadIdx.x; j < H; j += blockDim.x) CeType<T>::store(o + j, xr[j] * inv * w[j]);
}

// The same for widths that are multiples of 4 and at most 4 * 4 * blockDim: every thread keeps its
// float4 elements in registers, so the row is read once and all loads are in flight together.
// four consecutive outputs as one store (the row starts on a 16-byte boundary: H is a multiple of 4)
__device__ __forceinline__ void store4(float* p, float a, float b, float c, float d) {
    *reinterpret_cast<float4*>(p) = make_float4(a, b, c, d);
}
__device__ __forceinline__ void store4(__nv_bfloat16* p, float a, float b, float c, float d) {
    __nv_bfloat162 lo = __floats2bfloat162_rn(a, b), hi = __floats2bfloat162_rn(c, d);
    uint2 r;
    r.x = *reinterpret_cast<uint32_t*>(&lo); r.y = *reinterpret_cast<uint32_t*>(&hi);
    *reinterpret_cast<uint2*>(p) = r;
}

template <typename T>
__global__ void __launch_bounds__(1024) rmsnorm_vec_kernel(const float* __restrict__ x, const float* __restrict__ w,
                                                          T* __restrict__ out, const int* __restrict__ rows, int H,
                                                          float eps) {
    ce_pdl_launch_dependents();          // the weights (and the row list) do not depend on the kernel before
    __shared__ float scratch[32];
    int r = blockIdx.x, n4 = H >> 2;
    const float4* wr = reinterpret_cast<const float4*>(w);
    float4 v[4], g[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        int j = threadIdx.x + i * blockDim.x;
        g[i] = j < n4 ? wr[j] : make_float4(0.f, 0.f, 0.f, 0.f);
    }
    const float4* xr = reinterpret_cast<const float4*>(x + (size_t)(rows ? rows[r] : r) * H);
    ce_pdl_wait();
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        int j = threadIdx.x + i * blockDim.x;
        v[i] = j < n4 ? xr[j] : make_float4(0.f, 0.f, 0.f, 0.f);
    }
    float ss = 0.f;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        ss = fmaf(v[i].x, v[i].x, ss); ss = fmaf(v[i].y, v[i].y, ss);
        ss = fmaf(v[i].z, v[i].z, ss); ss = fmaf(v[i].w, v[i].w, ss);
    }
    ss = ce_block_sum(ss, scratch);
    float inv = 1.0f / sqrtf(ss / (float)H + eps);
    T* o = out + (size_t)r * H;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        int j = threadIdx.x + i * blockDim.x;
        if (j < n4) store4(o + 4 * j, v[i].x * inv * g[i].x, v[i].y * inv * g[i].y, v[i].z * inv * g[i].z, v[i].w * inv * g[i].w);
    }
}

// Threads per row of the vector kernel: a function of the width only, so that the order of the sum
// never depends on the batch.  0: use the scalar kernel.
static int rmsnorm_vec_threads(int H, const void* x, const void* w, const void* out) {
    if (H % 4 || (((uintptr_t)x | (uintptr_t)w | (uintptr_t)out) & 15)) return 0;
    int n4 = H / 4;
    int threads = ((n4 + 3) / 4 + 31) / 32 * 32;       // four float4 per thread where possible
    if (threads < 128) threads = 128;
    if (threads > 1024) return 0;
    return threads;
}

extern "C" int ce_rmsnorm(const float* x, const float* w, void* out, int out_dtype, const int* rows, int R, int H,
                          float eps, cudaStream_t stream) {
    if (R == 0) return CE_OK;
    if (!x || !w || !out) return ce_fail(CE_ERR_ARG, "ce_rmsnorm: null pointer");
    if (H <= 0) return ce_fail(CE_ERR_SIZE, "ce_rmsnorm: width %d", H);
    int vt = rmsnorm_vec_threads(H, x, w, out);
    if (out_dtype == CE_F32) {
        if (vt) { ce_note("rmsnorm_vec_kernel"); ce_launch(rmsnorm_vec_kernel<float>, R, vt, 0, stream, x, w, (float*)out, rows, H, eps); }
        else { ce_note("rmsnorm_kernel"); ce_launch(rmsnorm_kernel<float>, R, 256, 0, stream, x, w, (float*)out, rows, H, eps); }
    } else if (out_dtype == CE_BF16) {
        if (vt) { ce_note("rmsnorm_vec_kernel"); ce_launch(rmsnorm_vec_kernel<__nv_bfloat16>, R, vt, 0, stream, x, w, (__nv_bfloat16*)out, rows, H, eps); }
        else { ce_note("rmsnorm_kernel"); ce_launch(rmsnorm_kernel<__nv_bfloat16>, R, 256, 0, stream, x, w, (__nv_bfloat16*)out, rows, H, eps); }
    } else
        return ce_fail(CE_ERR_ARG, "ce_rmsnorm: unknown dtype %d", out_dtype);
    return ce_check_launch("ce_rmsnorm");
}

// ---------------------------------------------------------------------------------------------
// Per-head q/k RMSNorm, rotary embedding, and the write of K and V into the paged cache.
//
// Input  qkv [T, (nh + 2*nkv) * d]: q heads, then k heads, then v heads (one GEMM output).
// q heads are normalised and rotated in place.  k heads are normalised, rotated and stored at
// the token's place in the K pool; v heads are copied to the V pool.  Pools are
// [num_pages, nkv, page_size, d].  A token's place is found from its sequence's block-table row:
// page = table[slot, pos / page_size], offset = pos % page_size.
//
// Order follows the reference: norm over the head (weight shared by all heads) BEFORE the
// rotation (src/model/attention.rs:884-889); rotate-half pairing (i, i + rd/2)
// (src/model/layers.rs:159, spelled out in src/kernels/qsa.cu:107-116), or, as a parameter for other
// position encodings, the interleaved pairing (2i, 2i + 1); K is stored after norm and
// rotation, V as projected (src/model/attention.rs:890).
// ---------------------------------------------------------------------------------------------
struct QkRopeArgs {
    void* qkv;
    void* k_pool;
    void* v_pool;
    const float* q_weight;   // [d] or null: no q norm
    const float* k_weight;   // [d] or null: no k norm
    const float* cos_table;  // [max_pos, rd/2] or null: no rotation
    const float* sin_table;
    const int* positions;    // [T]
    const int* seq_of_token; // [T]
    const int* seq_slot;     // [B]
    const int* block_table;  // [slots, max_pages]
    int* status;
    int T, nh, nkv, d, rd, page_size, max_pages, num_pages, max_pos, write_kv;
    float eps;
    int pairing;             // partners of a rotation: 0 = (i, i + rd/2) ("rotate-half"), 1 = (2i, 2i + 1) (interleaved)
};

template <typename T>
__global__ void qk_rope_kvwrite_kernel(QkRopeArgs a) {
    ce_pdl_begin();
    extern __shared__ float sh[];     // d floats + 32 scratch
    float* vals = sh;
    float* scratch = sh + a.d;
    int t = blockIdx.x, hh = blockIdx.y, j = threadIdx.x;
    int d = a.d;
    bool is_q = hh < a.nh, is_k = !is_q && hh < a.nh + a.nkv;
    if (!is_q && !a.write_kv) return;
    T* src = (T*)a.qkv + (size_t)t * (a.nh + 2 * a.nkv) * d + (size_t)hh * d;
    float v = j < d ? CeType<T>::load(src + j) : 0.f;
    int pos = a.positions[t];

    T* dst = nullptr;
    if (is_q) {
        dst = src;
    } else {
        int slot = a.seq_slot[a.seq_of_token[t]];
        int page = a.block_table[(size_t)slot * a.max_pages + pos / a.page_size];
        if (page < 0 || page >= a.num_pages) {
            if (j == 0) atomicExch(a.status, 2);
            return;
        }
        int kvh = is_k ? hh - a.nh : hh - a.nh - a.nkv;
        T* pool = (T*)(is_k ? a.k_pool : a.v_pool);
        dst = pool + (((size_t)page * a.nkv + kvh) * a.page_size + pos % a.page_size) * d;
    }
    if (!is_q && !is_k) {               // V: plain copy
        if (j < d) CeType<T>::store(dst + j, v);
        return;
    }
    const float* w = is_q ? a.q_weight : a.k_weight;
    if (w) {
        float ss = ce_block_sum(v * v, scratch);
        float inv = 1.0f / sqrtf(ss / (float)d + a.eps);
        if (j < d) v = v * inv * w[j];
    }
    if (a.cos_table) {
        if (pos >= a.max_pos) {
            if (j == 0) atomicExch(a.status, 3);
            return;
        }
        if (j < d) vals[j] = v;
        __syncthreads();
        int half = a.rd / 2;
        const float* c = a.cos_table + (size_t)pos * half;
        const float* s = a.sin_table + (size_t)pos * half;
        if (a.pairing == 1) {           // interleaved: elements 2f and 2f + 1 turn by angle f
            if (j < a.rd) {
                int f = j >> 1;
                v = (j & 1) ? vals[j] * c[f] + vals[j - 1] * s[f] : vals[j] * c[f] - vals[j + 1] * s[f];
            }
        } else if (j < half)
            v = vals[j] * c[j] - vals[j + half] * s[j];
        else if (j < a.rd)
            v = vals[j] * c[j - half] + vals[j - half] * s[j - half];
    }
    if (j < d) CeType<T>::store(dst + j, v);
}

// Vectors of VW consecutive elements to and from float (2 and 4 elements as one access)
template <typename T, int VW> struct RopeVec {
    static __device__ __forceinline__ void load(const T* p, float (&v)[VW]) {
#pragma unroll
        for (int i = 0; i < VW; ++i) v[i] = CeType<T>::load(p + i);
    }
    static __device__ __forceinline__ void store(T* p, const float (&v)[VW]) {
#pragma unroll
        for (int i = 0; i < VW; ++i) CeType<T>::store(p + i, v[i]);
    }
};
template <> struct RopeVec<float, 2> {
    static __device__ __forceinline__ void load(const float* p, float (&v)[2]) { float2 t = *reinterpret_cast<const float2*>(p); v[0] = t.x; v[1] = t.y; }
    static __device__ __forceinline__ void store(float* p, const float (&v)[2]) { *reinterpret_cast<float2*>(p) = make_float2(v[0], v[1]); }
};
template <> struct RopeVec<float, 4> {
    static __device__ __forceinline__ void load(const float* p, float (&v)[4]) { float4 t = *reinterpret_cast<const float4*>(p); v[0] = t.x; v[1] = t.y; v[2] = t.z; v[3] = t.w; }
    static __device__ __forceinline__ void store(float* p, const float (&v)[4]) { *reinterpret_cast<float4*>(p) = make_float4(v[0], v[1], v[2], v[3]); }
};
template <> struct RopeVec<__nv_bfloat16, 2> {
    static __device__ __forceinline__ void load(const __nv_bfloat16* p, float (&v)[2]) {
        float2 t = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(p)); v[0] = t.x; v[1] = t.y;
    }
    static __device__ __forceinline__ void store(__nv_bfloat16* p, const float (&v)[2]) {
        *reinterpret_cast<__nv_bfloat162*>(p) = __floats2bfloat162_rn(v[0], v[1]);
    }
};
template <> struct RopeVec<__nv_bfloat16, 4> {
    static __device__ __forceinline__ void load(const __nv_bfloat16* p, float (&v)[4]) {
        uint2 r = *reinterpret_cast<const uint2*>(p);
        float2 lo = __bfloat1622float2(*reinterpret_cast<__nv_bfloat162*>(&r.x)), hi = __bfloat1622float2(*reinterpret_cast<__nv_bfloat162*>(&r.y));
        v[0] = lo.x; v[1] = lo.y; v[2] = hi.x; v[3] = hi.y;
    }
    static __device__ __forceinline__ void store(__nv_bfloat16* p, const float (&v)[4]) {
        __nv_bfloat162 lo = __floats2bfloat162_rn(v[0], v[1]), hi = __floats2bfloat162_rn(v[2], v[3]);
        uint2 r;
        r.x = *reinterpret_cast<uint32_t*>(&lo); r.y = *reinterpret_cast<uint32_t*>(&hi);
        *reinterpret_cast<uint2*>(p) = r;
    }
};

// Head sizes that are multiples of 64 (up to 256) with a full rotation: one warp per group of `hpw`
// consecutive heads of one token.  A lane holds VW = d/64 consecutive elements of the first half of a
// head and the VW elements d/2 further on, their partners in the rotation, so nothing is exchanged
// between lanes but the sum of squares.  The token's position, page, cosines and sines are looked up
// once per warp, a head's address is the last one plus a stride, and the elements of four heads are in
// flight together; with one head per warp (few tokens: decoding) the grid is as large as it can be, with many (portions of
// prompts) a token's heads share the lookups.  A head's arithmetic does not depend on hpw.
// n heads, one after the other from src (stride d) to dst (stride dst_stride): RMS norm with weights w1/w2
// (NORM), rotation by cs/sn (ROT), or neither (values: a copy).  Four heads are in flight together.
template <typename T, int VW, bool NORM, bool ROT>
__device__ __forceinline__ void rope_heads(const T* src, T* dst, size_t dst_stride, int n, int d, int e0, float eps,
                                           const float (&w1)[VW], const float (&w2)[VW], const float (&cs)[VW],
                                           const float (&sn)[VW]) {
    constexpr int U = 4;
    int half = d >> 1;
    float inv_d = 1.0f / (float)d;
    for (int hb = 0; hb < n; hb += U) {
        float x1[U][VW], x2[U][VW];
#pragma unroll
        for (int u = 0; u < U; ++u) {
            if (hb + u < n) {
                RopeVec<T, VW>::load(src + (size_t)u * d + e0, x1[u]);
                RopeVec<T, VW>::load(src + (size_t)u * d + half + e0, x2[u]);
            }
        }
#pragma unroll
        for (int u = 0; u < U; ++u) {
            if (hb + u >= n) break;
            if (NORM) {
                float ss = 0.f;
#pragma unroll
                for (int i = 0; i < VW; ++i) ss = fmaf(x1[u][i], x1[u][i], ss);
#pragma unroll
                for (int i = 0; i < VW; ++i) ss = fmaf(x2[u][i], x2[u][i], ss);
#pragma unroll
                for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
                float inv = rsqrtf(fmaf(ss, inv_d, eps));
#pragma unroll
                for (int i = 0; i < VW; ++i) { x1[u][i] = x1[u][i] * inv * w1[i]; x2[u][i] = x2[u][i] * inv * w2[i]; }
            }
            if (ROT) {
#pragma unroll
                for (int i = 0; i < VW; ++i) {
                    float p = x1[u][i], q = x2[u][i];
                    x1[u][i] = p * cs[i] - q * sn[i];
                    x2[u][i] = q * cs[i] + p * sn[i];
                }
            }
            RopeVec<T, VW>::store(dst + u * dst_stride + e0, x1[u]);
            RopeVec<T, VW>::store(dst + u * dst_stride + half + e0, x2[u]);
        }
        src += (size_t)U * d;
        dst += U * dst_stride;
    }
}

template <typename T, int VW>
__device__ __forceinline__ void rope_heads_any(const T* src, T* dst, size_t dst_stride, int n, int d, int e0, float eps,
                                               const float* w, bool rot, const float (&cs)[VW], const float (&sn)[VW]) {
    float w1[VW], w2[VW];
#pragma unroll
    for (int i = 0; i < VW; ++i) w1[i] = w2[i] = 1.f;
    if (w) {
        RopeVec<float, VW>::load(w + e0, w1);
        RopeVec<float, VW>::load(w + (d >> 1) + e0, w2);
    }
    if (w && rot) rope_heads<T, VW, true, true>(src, dst, dst_stride, n, d, e0, eps, w1, w2, cs, sn);
    else if (w) rope_heads<T, VW, true, false>(src, dst, dst_stride, n, d, e0, eps, w1, w2, cs, sn);
    else if (rot) rope_heads<T, VW, false, true>(src, dst, dst_stride, n, d, e0, eps, w1, w2, cs, sn);
    else rope_heads<T, VW, false, false>(src, dst, dst_stride, n, d, e0, eps, w1, w2, cs, sn);
}

template <typename T, int VW>
__global__ void __launch_bounds__(128) qk_rope_kvwrite_warp_kernel(QkRopeArgs a, int hpw) {
    // positions, slots, block tables, cosines, sines and norm weights are inputs of the step or constants:
    // they are looked up while the kernel before this one (the QKV product) still runs; only its output waits
    ce_pdl_launch_dependents();
    int lane = threadIdx.x & 31;
    int heads_per_token = a.nh + 2 * a.nkv;
    int groups = (heads_per_token + hpw - 1) / hpw;
    long long wg = (long long)blockIdx.x * 4 + (threadIdx.x >> 5);
    if (wg >= (long long)a.T * groups) return;
    int t = (int)(wg / groups), g = (int)(wg - (long long)t * groups);
    int hh0 = g * hpw, hh1 = min(hh0 + hpw, heads_per_token);
    if (!a.write_kv) hh1 = min(hh1, a.nh);
    if (hh0 >= hh1) return;
    int d = a.d, half = d >> 1, e0 = VW * lane;
    int pos = a.positions[t];
    bool rotate = a.cos_table != nullptr;
    if (rotate && pos >= a.max_pos && hh0 < a.nh + a.nkv) {
        if (lane == 0) atomicExch(a.status, 3);
        return;
    }
    float cs[VW], sn[VW];
#pragma unroll
    for (int i = 0; i < VW; ++i) { cs[i] = 1.f; sn[i] = 0.f; }
    if (rotate && hh0 < a.nh + a.nkv) {
        RopeVec<float, VW>::load(a.cos_table + (size_t)pos * half + e0, cs);
        RopeVec<float, VW>::load(a.sin_table + (size_t)pos * half + e0, sn);
    }
    size_t page_row = 0;
    if (hh1 > a.nh) {                      // a K or V head in this group: where the token's row lies in the pools
        int slot = a.seq_slot[a.seq_of_token[t]];
        int page = a.block_table[(size_t)slot * a.max_pages + pos / a.page_size];
        if (page < 0 || page >= a.num_pages) {
            if (lane == 0) atomicExch(a.status, 2);
            return;
        }
        page_row = (size_t)page * a.nkv * a.page_size + pos % a.page_size;
    }
    T* row = (T*)a.qkv + (size_t)t * heads_per_token * d;
    ce_pdl_wait();
    // the group's query heads (in place), key heads and value heads (into the pools)
    int q1 = min(hh1, a.nh);
    if (hh0 < q1) rope_heads_any<T, VW>(row + (size_t)hh0 * d, row + (size_t)hh0 * d, (size_t)d, q1 - hh0, d, e0, a.eps, a.q_weight, rotate, cs, sn);
    int k0 = max(hh0, a.nh), k1 = min(hh1, a.nh + a.nkv);
    if (k0 < k1)
        rope_heads_any<T, VW>(row + (size_t)k0 * d, (T*)a.k_pool + (page_row + (size_t)(k0 - a.nh) * a.page_size) * d,
                              (size_t)a.page_size * d, k1 - k0, d, e0, a.eps, a.k_weight, rotate, cs, sn);
    int v0 = max(hh0, a.nh + a.nkv);
    if (v0 < hh1)
        rope_heads_any<T, VW>(row + (size_t)v0 * d, (T*)a.v_pool + (page_row + (size_t)(v0 - a.nh - a.nkv) * a.page_size) * d,
                              (size_t)a.page_size * d, hh1 - v0, d, e0, a.eps, nullptr, false, cs, sn);
}

template <typename T>
static bool launch_rope_warp(const QkRopeArgs& a, cudaStream_t stream) {
    int heads_per_token = a.nh + 2 * a.nkv;
    if (a.d % 64 || a.d > 256 || (a.cos_table && (a.rd != a.d || a.pairing != 0))) return false;
    // few tokens: a warp per head; many: four warps share a token's heads
    int hpw = a.T >= 256 ? (heads_per_token + 3) / 4 : 1;
    long long warps = (long long)a.T * ((heads_per_token + hpw - 1) / hpw);
    if ((warps + 3) / 4 > 2147483647LL) return false;
    unsigned blocks = (unsigned)((warps + 3) / 4);
    switch (a.d / 64) {
        case 1: { ce_note("qk_rope_kvwrite_warp_kernel"); ce_launch(qk_rope_kvwrite_warp_kernel<T, 1>, blocks, 128, 0, stream, a, hpw); } return true;
        case 2: { ce_note("qk_rope_kvwrite_warp_kernel"); ce_launch(qk_rope_kvwrite_warp_kernel<T, 2>, blocks, 128, 0, stream, a, hpw); } return true;
        case 3: { ce_note("qk_rope_kvwrite_warp_kernel"); ce_launch(qk_rope_kvwrite_warp_kernel<T, 3>, blocks, 128, 0, stream, a, hpw); } return true;
        case 4: { ce_note("qk_rope_kvwrite_warp_kernel"); ce_launch(qk_rope_kvwrite_warp_kernel<T, 4>, blocks, 128, 0, stream, a, hpw); } return true;
    }
    return false;
}

extern "C" int ce_qk_rope_kvwrite(void* qkv, void* k_pool, void* v_pool, int dtype, const float* q_weight,
                                  const float* k_weight, const float* cos_table, const float* sin_table,
                                  const int* positions, const int* seq_of_token, const int* seq_slot,
                                  const int* block_table, int* status, int T, int nh, int nkv, int d, int rd,
                                  int page_size, int max_pages, int num_pages, int max_pos, int write_kv, float eps,
                                  int pairing, cudaStream_t stream) {
    if (T == 0) return CE_OK;
    if (d <= 0 || d > 1024) return ce_fail(CE_ERR_SIZE, "ce_qk_rope_kvwrite: head_dim %d not in 1..1024", d);
    if (rd < 0 || rd > d || (rd & 1)) return ce_fail(CE_ERR_SIZE, "ce_qk_rope_kvwrite: rotary_dim %d must be even and <= head_dim %d", rd, d);
    if (pairing != 0 && pairing != 1) return ce_fail(CE_ERR_ARG, "ce_qk_rope_kvwrite: pairing %d (0: halves, 1: interleaved)", pairing);
    if (!qkv || !positions || !status) return ce_fail(CE_ERR_ARG, "ce_qk_rope_kvwrite: null pointer");
    if (write_kv && (!k_pool || !v_pool || !seq_of_token || !seq_slot || !block_table))
        return ce_fail(CE_ERR_ARG, "ce_qk_rope_kvwrite: cache pointers missing");
    QkRopeArgs a{qkv, k_pool, v_pool, q_weight, k_weight, cos_table, sin_table, positions, seq_of_token, seq_slot,
                 block_table, status, T, nh, nkv, d, rd, page_size, max_pages, num_pages, max_pos, write_kv, eps, pairing};
    int threads = (d + 31) / 32 * 32;
    dim3 grid(T, nh + 2 * nkv);
    size_t smem = (d + 32) * sizeof(float);
    if (dtype == CE_F32) {
        if (!launch_rope_warp<float>(a, stream)) { ce_note("qk_rope_kvwrite_kernel"); ce_launch(qk_rope_kvwrite_kernel<float>, grid, threads, smem, stream, a); }
    } else if (dtype == CE_BF16) {
        if (!launch_rope_warp<__nv_bfloat16>(a, stream))
            { ce_note("qk_rope_kvwrite_kernel"); ce_launch(qk_rope_kvwrite_kernel<__nv_bfloat16>, grid, threads, smem, stream, a); }
    } else
        return ce_fail(CE_ERR_ARG, "ce_qk_rope_kvwrite: unknown dtype %d", dtype);
    return ce_check_launch("ce_qk_rope_kvwrite");
}

// ---------------------------------------------------------------------------------------------
// x += delta (float32 residual, delta in the activation dtype)
// ---------------------------------------------------------------------------------------------
template <typename T>
__global__ void add_residual_kernel(float* __restrict__ x, const T* __restrict__ delta, size_t n) {
    ce_pdl_begin();
    size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    size_t stride = (size_t)gridDim.x * blockDim.x;
    for (; i < n; i += stride) x[i] += CeType<T>::load(delta + i);
}

extern "C" int ce_add_residual(float* x, const void* delta, int dtype, long long n, cudaStream_t stream) {
    if (n == 0) return CE_OK;
    if (!x || !delta) return ce_fail(CE_ERR_ARG, "ce_add_residual: null pointer");
    int blocks = (int)((n + 255) / 256 < 148 * 16 ? (n + 255) / 256 : 148 * 16);
    if (dtype == CE_F32)
        { ce_note("add_residual_kernel"); ce_launch(add_residual_kernel<float>, blocks, 256, 0, stream, x, (const float*)delta, (size_t)n); }
    else if (dtype == CE_BF16)
        { ce_note("add_residual_kernel"); ce_launch(add_residual_kernel<__nv_bfloat16>, blocks, 256, 0, stream, x, (const __nv_bfloat16*)delta, (size_t)n); }
    else
        return ce_fail(CE_ERR_ARG, "ce_add_residual: unknown dtype %d", dtype);
    return ce_check_launch("ce_add_residual");
}

// ---------------------------------------------------------------------------------------------
// SwiGLU: out[t, i] = silu(gu[t, i]) * gu[t, I + i], silu(z) = z / (1 + exp(-z))
// (src/model/layers.rs:568, 625-648)
// ---------------------------------------------------------------------------------------------
template <typename T>
__global__ void swiglu_kernel(const T* __restrict__ gu, T* __restrict__ out, int I, size_t total) {
    ce_pdl_begin();
    size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    size_t stride = (size_t)gridDim.x * blockDim.x;
    for (; i < total; i += stride) {
        size_t t = i / I, c = i - t * I;
        float g = CeType<T>::load(gu + t * 2 * I + c);
        float u = CeType<T>::load(gu + t * 2 * I + I + c);
        CeType<T>::store(out + i, g / (1.0f + expf(-g)) * u);
    }
}

extern "C" int ce_swiglu(const void* gu, void* out, int dtype, int T, int I, cudaStream_t stream) {
    size_t total = (size_t)T * I;
    if (total == 0) return CE_OK;
    if (!gu || !out) return ce_fail(CE_ERR_ARG, "ce_swiglu: null pointer");
    int blocks = (int)((total + 255) / 256 < 148 * 16 ? (total + 255) / 256 : 148 * 16);
    if (dtype == CE_F32)
        { ce_note("swiglu_kernel"); ce_launch(swiglu_kernel<float>, blocks, 256, 0, stream, (const float*)gu, (float*)out, I, total); }
    else if (dtype == CE_BF16)
        { ce_note("swiglu_kernel"); ce_launch(swiglu_kernel<__nv_bfloat16>, blocks, 256, 0, stream, (const __nv_bfloat16*)gu, (__nv_bfloat16*)out, I, total); }
    else
        return ce_fail(CE_ERR_ARG, "ce_swiglu: unknown dtype %d", dtype);
    return ce_check_launch("ce_swiglu");
}

// ---------------------------------------------------------------------------------------------
// dst[idx[i]] = val[i]: applies the block-table entries that changed since the last step.
// ---------------------------------------------------------------------------------------------
__global__ void scatter_i32_kernel(int* __restrict__ dst, const int* __restrict__ idx, const int* __restrict__ val,
                                   int n, long long dst_len) {
    // No early launch of dependents here: block tables are step inputs, and kernels further down the
    // stream read them BEFORE their own wait (the decode attention looks up pages while the kernels
    // before it still run).  Without the early launch the next kernel starts only when these writes are
    // complete, and so does everything after it.
    ce_pdl_wait();
    int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n && idx[i] >= 0 && idx[i] < dst_len) dst[idx[i]] = val[i];
}

extern "C" int ce_scatter_i32(int* dst, const int* idx, const int* val, int n, long long dst_len, cudaStream_t stream) {
    if (n == 0) return CE_OK;
    if (!dst || !idx || !val) return ce_fail(CE_ERR_ARG, "ce_scatter_i32: null pointer");
    { ce_note("scatter_i32_kernel"); ce_launch(scatter_i32_kernel, (n + 255) / 256, 256, 0, stream, dst, idx, val, n, dst_len); }
    return ce_check_launch("ce_scatter_i32");
}
