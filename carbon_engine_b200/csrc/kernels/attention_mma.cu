// bfloat16 attention over the paged cache on the tensor cores (mma.sync m16n8k16, float32
// accumulators): a split-KV kernel for sequences that bring one token, and a flash kernel for
// sequences that bring a portion of a prompt.  Both read keys and values through the block table.
//
// Decode: one block per (sequence, KV head, group of up to 16 query heads, split of the positions).
// The query heads that share the KV head are the 16 rows of the MMA tile, so K and V are read once
// per KV head (the reference's paged_decode_tc does the same for up to 8 heads,
// src/kernels/attention_tc.cu:682-807).  Each of the 4 warps takes 16 of every 64 staged keys and
// keeps a running (max, sum, output); the warps are combined in shared memory and the block writes
// one partial per split to scratch memory; a merge kernel combines the splits in split order
// (src/kernels/attention_tc.cu:810-830).  Splits are cut at fixed positions, so a sequence's result
// does not depend on the batch or on the longest sequence beside it.
//
// Prefill: one block per (tile of 64 new tokens of one sequence, query head); each warp owns 16
// queries, keys are staged 64 at a time, causal and window limits are applied per row
// (src/kernels/attention_tc.cu:180-565 is the reference's counterpart).
//
// Scores are scaled in float32, the softmax runs in float32 with exp2, probabilities are rounded to
// bfloat16 for the PV product (as in src/kernels/attention_tc.cu:505-515), outputs are rounded once.
#include "common.cuh"
#include "tensor_map.h"
#include <stdlib.h>

#define AM_THREADS 128
#define AM_TILE 64           // keys staged per iteration
#define AM_SPLIT 128         // decode splits are multiples of this many positions
#define AM_STAGES 3          // decode: staged tiles in flight: loads of tiles i+1, i+2 run while tile i is computed
#define AM_PF_STAGES 2       // prefill: two stages, so that three blocks fit one SM
#define AM_PAD 8             // padding of a staged row, in elements (keeps 32-bit and ldmatrix reads conflict-free)

typedef __nv_bfloat16 bf16;

__device__ __forceinline__ void mma16816(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ void ldmatrix_x4_trans(uint32_t (&r)[4], const bf16* p) {
    uint32_t addr = (uint32_t)__cvta_generic_to_shared(p);
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];\n"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
__device__ __forceinline__ void cp_async16(bf16* dst, const bf16* src, bool valid) {
    uint32_t addr = (uint32_t)__cvta_generic_to_shared(dst);
    int n = valid ? 16 : 0;      // 0 bytes read: the 16 bytes are filled with zeros
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;\n" ::"r"(addr), "l"(src), "r"(n));
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;\n" ::); }
template <int N> __device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;\n" ::"n"(N)); }
__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
    __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&v);
}

struct MmaAttnArgs {
    const bf16* q;              // [T, q_stride]; head h at column h*d
    const bf16* k_pool;         // [num_pages, nkv, page_size, d]
    const bf16* v_pool;
    bf16* out;                  // [T, nh*d]
    float* part_o;              // decode scratch [rows, nh, max_splits, d]
    float* part_ml;             // decode scratch [rows, nh, max_splits, 2]
    const int* positions;       // [T]
    const int* seq_slot;        // [B]
    const int* q_start;         // [B+1]
    const int* ctx_len;         // [B]  keys of the sequence after this step
    const int* block_table;     // [slots, max_pages]
    const int* tiles;           // prefill: [n_tiles, 2] = (sequence, first new token of the tile)
    int* counters;              // decode: one per (sequence, KV head, head group), zero between launches
    int* status;
    int nh, nkv, d, q_stride, page_size, max_pages, num_pages, window, max_splits, split, fused_merge;
    int cluster_merge;          // TMA decode kernel: the splits of a sequence form a cluster and merge through shared memory
    float scale_log2;           // scale * log2(e)
};

// Stage keys [k0, k0 + AM_TILE) of one KV head into shared memory rows of d + AM_PAD elements.
// Keys outside [lo, hi] are filled with zeros, so that a masked probability of 0 never meets a NaN.
__device__ __forceinline__ void stage_tile(bf16* Ks, bf16* Vs, const MmaAttnArgs& a, const int* table, int kvh, int k0,
                                           int lo, int hi) {
    // 16-byte chunks c = thread, thread + 128, ...: (key, part) advance by fixed steps, without divisions
    int d = a.d, ld = d + AM_PAD, chunks = d >> 3;
    int kl = threadIdx.x / chunks, part = threadIdx.x - kl * chunks;
    int dkl = AM_THREADS / chunks, dpart = AM_THREADS - dkl * chunks;
    bool pow2 = (a.page_size & (a.page_size - 1)) == 0;
    int shift = 31 - __clz(a.page_size);
    if (pow2 && a.page_size >= AM_TILE && (k0 & (AM_TILE - 1)) == 0 && dpart == 0) {
        // the whole tile lies in one page and every thread keeps its 16-byte column: one table lookup,
        // then source and destination advance by constant strides
        int page = (k0 <= hi && k0 + AM_TILE > lo) ? table[k0 >> shift] : 0;
        bool page_ok = page >= 0 && page < a.num_pages;
        if (!page_ok) { atomicExch(a.status, 4); page = 0; }
        size_t base = (((size_t)page * a.nkv + kvh) * a.page_size + (k0 & (a.page_size - 1)) + kl) * d + part * 8;
        const bf16* ksrc = a.k_pool + base;
        const bf16* vsrc = a.v_pool + base;
        bf16* kdst = Ks + kl * ld + part * 8;
        bf16* vdst = Vs + kl * ld + part * 8;
        bool all_valid = page_ok && k0 >= lo && k0 + AM_TILE - 1 <= hi;
        for (; kl < AM_TILE; kl += dkl) {
            bool valid = all_valid || (page_ok && k0 + kl >= lo && k0 + kl <= hi);
            cp_async16(kdst, ksrc, valid);
            cp_async16(vdst, vsrc, valid);
            ksrc += dkl * d; vsrc += dkl * d;
            kdst += dkl * ld; vdst += dkl * ld;
        }
        return;
    }
    while (kl < AM_TILE) {
        int key = k0 + kl;
        bool valid = key >= lo && key <= hi;
        size_t row = 0;
        if (valid) {
            int pi = pow2 ? key >> shift : key / a.page_size;
            int off = pow2 ? key & (a.page_size - 1) : key - pi * a.page_size;
            int page = table[pi];
            if (page < 0 || page >= a.num_pages) {
                atomicExch(a.status, 4);
                valid = false;
            } else {
                row = (((size_t)page * a.nkv + kvh) * a.page_size + off) * d + part * 8;
            }
        }
        cp_async16(Ks + kl * ld + part * 8, a.k_pool + row, valid);
        cp_async16(Vs + kl * ld + part * 8, a.v_pool + row, valid);
        kl += dkl;
        part += dpart;
        if (part >= chunks) { part -= chunks; ++kl; }
    }
}

// One warp: scores of its 16 rows against NK8*8 staged keys, online softmax, output update.
// lo/hi: first and last visible key of rows (lane/4) and (lane/4 + 8).
__device__ __forceinline__ void ldmatrix_x4(uint32_t (&r)[4], const bf16* p) {
    uint32_t addr = (uint32_t)__cvta_generic_to_shared(p);
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];\n"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}

// MASK false: every staged key of the tile is visible to every row of the warp (no compares).
template <int DMAX, int NK8, bool MASK>
__device__ __forceinline__ void warp_tile(const uint32_t (&qf)[DMAX / 16][4], float (&o)[DMAX / 8][4], float (&m)[2],
                                          float (&l)[2], const bf16* Ks, const bf16* Vs, int ld, int d, int key_base,
                                          const int (&lo)[2], const int (&hi)[2], float scale_log2) {
    int lane = threadIdx.x & 31, quad = lane & 3;
    int mi = lane >> 3, rr = lane & 7;
    float s[NK8][4];
#pragma unroll
    for (int j = 0; j < NK8; ++j) s[j][0] = s[j][1] = s[j][2] = s[j][3] = 0.f;
    // K fragments: one ldmatrix.x4 brings the B operands of two key tiles for one step of 16 along d
    const bf16* krow = Ks + ((mi >> 1) * 8 + rr) * ld + (mi & 1) * 8;
    if (NK8 == 2) {
        // few key tiles: odd steps along d go to a second pair of accumulators, which halves the
        // chain of MMAs that wait for one another
        float s2[2][4] = {{0.f, 0.f, 0.f, 0.f}, {0.f, 0.f, 0.f, 0.f}};
#pragma unroll
        for (int kk = 0; kk < DMAX / 16; ++kk) {
            if (kk * 16 < d) {
                uint32_t kb[4];
                ldmatrix_x4(kb, krow + kk * 16);
                if (kk & 1) { mma16816(s2[0], qf[kk], kb[0], kb[1]); mma16816(s2[1], qf[kk], kb[2], kb[3]); }
                else { mma16816(s[0], qf[kk], kb[0], kb[1]); mma16816(s[1], qf[kk], kb[2], kb[3]); }
            }
        }
#pragma unroll
        for (int e = 0; e < 4; ++e) { s[0][e] += s2[0][e]; s[1][e] += s2[1][e]; }
    } else {
#pragma unroll
        for (int kk = 0; kk < DMAX / 16; ++kk) {
            if (kk * 16 < d) {
#pragma unroll
                for (int j = 0; j < NK8; j += 2) {
                    uint32_t kb[4];
                    ldmatrix_x4(kb, krow + j * 8 * ld + kk * 16);
                    mma16816(s[j], qf[kk], kb[0], kb[1]);
                    mma16816(s[j + 1], qf[kk], kb[2], kb[3]);
                }
            }
        }
    }
    // raw maxima; the scale (positive) is applied inside the exponent: p = 2^(s * scale - m)
    float mx[2] = {-INFINITY, -INFINITY};
#pragma unroll
    for (int j = 0; j < NK8; ++j) {
#pragma unroll
        for (int e = 0; e < 4; ++e) {
            if (MASK) {
                int r = e >> 1;
                int key = key_base + j * 8 + 2 * quad + (e & 1);
                if (!(key >= lo[r] && key <= hi[r])) s[j][e] = -INFINITY;
            }
            mx[e >> 1] = fmaxf(mx[e >> 1], s[j][e]);
        }
    }
    float alpha[2], muse[2];
#pragma unroll
    for (int r = 0; r < 2; ++r) {
        mx[r] = fmaxf(mx[r], __shfl_xor_sync(0xffffffffu, mx[r], 1));
        mx[r] = fmaxf(mx[r], __shfl_xor_sync(0xffffffffu, mx[r], 2));
        float mn = fmaxf(m[r], mx[r] * scale_log2);
        muse[r] = mn == -INFINITY ? 0.f : mn;
        alpha[r] = ce_exp2_fast(m[r] - muse[r]);
        m[r] = mn;
        l[r] *= alpha[r];
    }
#pragma unroll
    for (int j = 0; j < NK8; ++j) {
#pragma unroll
        for (int e = 0; e < 4; ++e) {
            float p = ce_exp2_fast(fmaf(s[j][e], scale_log2, -muse[e >> 1]));
            s[j][e] = p;
            l[e >> 1] += p;
        }
    }
#pragma unroll
    for (int dn = 0; dn < DMAX / 8; ++dn) {
        o[dn][0] *= alpha[0]; o[dn][1] *= alpha[0]; o[dn][2] *= alpha[1]; o[dn][3] *= alpha[1];
    }
#pragma unroll
    for (int c = 0; c < NK8 / 2; ++c) {
        uint32_t pa[4] = {pack_bf16(s[2 * c][0], s[2 * c][1]), pack_bf16(s[2 * c][2], s[2 * c][3]),
                          pack_bf16(s[2 * c + 1][0], s[2 * c + 1][1]), pack_bf16(s[2 * c + 1][2], s[2 * c + 1][3])};
        const bf16* vrow = Vs + (c * 16 + (mi & 1) * 8 + rr) * ld + (mi >> 1) * 8;
#pragma unroll
        for (int dn = 0; dn < DMAX / 8; dn += 2) {
            if (dn * 8 < d) {
                uint32_t vb[4];
                ldmatrix_x4_trans(vb, vrow + dn * 8);
                mma16816(o[dn], pa, vb[0], vb[1]);
                mma16816(o[dn + 1], pa, vb[2], vb[3]);
            }
        }
    }
}

// ---------------------------------------------------------------------------------------------
// Decode: grid (n_seqs * max_splits, nkv, head groups of 16)
// ---------------------------------------------------------------------------------------------
template <int DMAX, int ST>
__global__ void __launch_bounds__(AM_THREADS) attention_decode_kernel(MmaAttnArgs a) {
    ce_pdl_begin();
    extern __shared__ __align__(16) unsigned char smem_raw[];
    int b = blockIdx.x / a.max_splits, split = blockIdx.x % a.max_splits;
    int kvh = blockIdx.y, hg = blockIdx.z;
    int G = a.nh / a.nkv;
    int t = b;                                    // one-token sequences come first: sequence b brings token b
    int pos = a.positions[t];
    int lo = a.window > 0 ? max(0, pos - a.window + 1) : 0;
    int k_begin = split * a.split, k_end = min(k_begin + a.split, pos + 1);
    if (k_begin > pos || k_end <= lo) return;     // the merge kernel skips these splits too
    const int* table = a.block_table + (size_t)a.seq_slot[b] * a.max_pages;
    int d = a.d, ld = d + AM_PAD;
    bf16* Ks = reinterpret_cast<bf16*>(smem_raw);
    bf16* Vs = Ks + ST * AM_TILE * ld;

    int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, quad = lane & 3, grp = lane >> 2;
    int heads_here = min(16, G - hg * 16);
    uint32_t qf[DMAX / 16][4];
    {
        int h0 = kvh * G + hg * 16;
        const bf16* q0 = a.q + (size_t)t * a.q_stride + (size_t)(h0 + grp) * d;
        const bf16* q1 = q0 + (size_t)8 * d;
        bool v0 = grp < heads_here, v1 = grp + 8 < heads_here;
#pragma unroll
        for (int kk = 0; kk < DMAX / 16; ++kk) {
            int col = kk * 16 + 2 * quad;
            bool in = kk * 16 < d;
            qf[kk][0] = (in && v0) ? *reinterpret_cast<const uint32_t*>(q0 + col) : 0u;
            qf[kk][1] = (in && v1) ? *reinterpret_cast<const uint32_t*>(q1 + col) : 0u;
            qf[kk][2] = (in && v0) ? *reinterpret_cast<const uint32_t*>(q0 + col + 8) : 0u;
            qf[kk][3] = (in && v1) ? *reinterpret_cast<const uint32_t*>(q1 + col + 8) : 0u;
        }
    }
    float o[DMAX / 8][4];
#pragma unroll
    for (int i = 0; i < DMAX / 8; ++i) o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f;
    float m[2] = {-INFINITY, -INFINITY}, l[2] = {0.f, 0.f};
    int los[2] = {lo, lo}, his[2] = {pos, pos};

    int n_tiles = (k_end - k_begin + AM_TILE - 1) / AM_TILE;
#pragma unroll
    for (int p = 0; p < ST - 1; ++p) {
        if (p < n_tiles) stage_tile(Ks + p * AM_TILE * ld, Vs + p * AM_TILE * ld, a, table, kvh, k_begin + p * AM_TILE, lo, pos);
        cp_async_commit();
    }
    for (int it = 0; it < n_tiles; ++it) {
        cp_async_wait<ST - 2>();       // tile `it` has landed
        __syncthreads();                      // ... for everyone, and everyone is done with tile it-1
        int nxt = it + ST - 1;
        if (nxt < n_tiles) {
            int st = nxt % ST;         // the stage tile it-1 was computed from
            stage_tile(Ks + st * AM_TILE * ld, Vs + st * AM_TILE * ld, a, table, kvh, k_begin + nxt * AM_TILE, lo, pos);
        }
        cp_async_commit();
        int cur = it % ST;
        int k0 = k_begin + it * AM_TILE + warp * 16;
        if (k0 <= pos) {
            const bf16* kt = Ks + (cur * AM_TILE + warp * 16) * ld;
            const bf16* vt = Vs + (cur * AM_TILE + warp * 16) * ld;
            if (k0 >= lo && k0 + 15 <= pos) warp_tile<DMAX, 2, false>(qf, o, m, l, kt, vt, ld, d, k0, los, his, a.scale_log2);
            else warp_tile<DMAX, 2, true>(qf, o, m, l, kt, vt, ld, d, k0, los, his, a.scale_log2);
        }
    }
    cp_async_wait<0>();
    __syncthreads();
#pragma unroll
    for (int r = 0; r < 2; ++r) {
        l[r] += __shfl_xor_sync(0xffffffffu, l[r], 1);
        l[r] += __shfl_xor_sync(0xffffffffu, l[r], 2);
    }
    // combine the 4 warps through shared memory (the staging buffers are free now)
    float* so = reinterpret_cast<float*>(smem_raw);          // [4][16][d]
    float* sm = so + 4 * 16 * d;                             // [4][16]
    float* sl = sm + 64;                                     // [4][16]
#pragma unroll
    for (int dn = 0; dn < DMAX / 8; ++dn) {
        if (dn * 8 < d) {
            int col = dn * 8 + 2 * quad;
            so[(warp * 16 + grp) * d + col] = o[dn][0];
            so[(warp * 16 + grp) * d + col + 1] = o[dn][1];
            so[(warp * 16 + grp + 8) * d + col] = o[dn][2];
            so[(warp * 16 + grp + 8) * d + col + 1] = o[dn][3];
        }
    }
    if (quad == 0) {
        sm[warp * 16 + grp] = m[0]; sm[warp * 16 + grp + 8] = m[1];
        sl[warp * 16 + grp] = l[0]; sl[warp * 16 + grp + 8] = l[1];
    }
    __syncthreads();
    for (int e = threadIdx.x; e < heads_here * d; e += AM_THREADS) {
        int r = e / d, col = e - r * d;
        float M = fmaxf(fmaxf(sm[r], sm[16 + r]), fmaxf(sm[32 + r], sm[48 + r]));
        float acc = 0.f, L = 0.f;
#pragma unroll
        for (int w = 0; w < 4; ++w) {
            float f = sm[w * 16 + r] == -INFINITY ? 0.f : ce_exp2_fast(sm[w * 16 + r] - M);
            acc += so[(w * 16 + r) * d + col] * f;
            L += sl[w * 16 + r] * f;
        }
        int h = kvh * G + hg * 16 + r;
        size_t base = ((size_t)b * a.nh + h) * a.max_splits + split;
        a.part_o[base * d + col] = acc;
        if (col == 0) {
            a.part_ml[base * 2] = M;
            a.part_ml[base * 2 + 1] = L;
        }
    }
    if (!a.fused_merge) return;
    // The block that arrives last for this (sequence, KV head, head group) merges the splits.  The
    // result does not depend on which block that is: weights and sums are taken in split order.
    __shared__ int s_ticket;
    __threadfence();
    __syncthreads();
    int s0 = lo / a.split, s1 = pos / a.split, ns = s1 - s0 + 1;       // the splits that hold visible keys
    int cidx = (b * a.nkv + kvh) * gridDim.z + hg;
    if (threadIdx.x == 0) s_ticket = atomicAdd(&a.counters[cidx], 1);
    __syncthreads();
    if (s_ticket != ns - 1) return;
    __threadfence();
    float* wts = reinterpret_cast<float*>(smem_raw);                  // [heads_here][ns]: the staging buffers are free
    for (int r = warp; r < heads_here; r += 4) {                       // one warp per head: lanes over splits
        size_t base = ((size_t)b * a.nh + kvh * G + hg * 16 + r) * a.max_splits + s0;
        float M = -INFINITY;
        for (int s = lane; s < ns; s += 32) M = fmaxf(M, __ldcg(&a.part_ml[(base + s) * 2]));
        for (int o2 = 16; o2 > 0; o2 >>= 1) M = fmaxf(M, __shfl_xor_sync(0xffffffffu, M, o2));
        float L = 0.f;
        for (int s = lane; s < ns; s += 32) {
            float ms = __ldcg(&a.part_ml[(base + s) * 2]);
            float f = ms == -INFINITY ? 0.f : ce_exp2_fast(ms - M);
            wts[r * ns + s] = f;
            L += __ldcg(&a.part_ml[(base + s) * 2 + 1]) * f;
        }
        for (int o2 = 16; o2 > 0; o2 >>= 1) L += __shfl_xor_sync(0xffffffffu, L, o2);
        float inv = L > 0.f ? 1.0f / L : 0.f;
        __syncwarp();
        for (int s = lane; s < ns; s += 32) wts[r * ns + s] *= inv;
    }
    __syncthreads();
    for (int e = threadIdx.x; e < heads_here * d; e += AM_THREADS) {
        int r = e / d, col = e - r * d;
        int h = kvh * G + hg * 16 + r;
        const float* po = a.part_o + (((size_t)b * a.nh + h) * a.max_splits + s0) * d + col;
        float acc = 0.f;
#pragma unroll 8
        for (int s = 0; s < ns; ++s) acc = fmaf(__ldcg(po + (size_t)s * d), wts[r * ns + s], acc);
        a.out[((size_t)t * a.nh + h) * d + col] = __float2bfloat16_rn(acc);
    }
    if (threadIdx.x == 0) a.counters[cidx] = 0;                        // ready for the next launch
}


// ---------------------------------------------------------------------------------------------
// Decode with TMA staging (head sizes that are multiples of 64, pages of a power of two >= 8 rows).
// Same work split and same arithmetic as attention_decode_kernel, but a fifth warp's first lane brings
// every tile of 64 keys with a few cp.async.bulk.tensor copies (one per page piece and 64 columns)
// into 128-byte-swizzled shared memory, counted on an mbarrier per stage; the four computing warps
// never stage anything, meet no block-wide barrier inside the loop (a warp frees a stage with one
// mbarrier arrival), and skip rescaling the output when no row's maximum moved.  A copy brings whole
// page pieces, whatever they hold: a warp zeroes the V rows of its keys that are not visible before it
// uses them, so that a probability of 0 never meets a NaN; scores of such keys are masked as before.
// ---------------------------------------------------------------------------------------------
#define AMT_THREADS 160
#define AMT_SPIN (1u << 22)

__device__ __forceinline__ uint32_t amt_smem(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ bool amt_wait(uint64_t* bar, uint32_t parity) {
    for (uint32_t i = 0; i < AMT_SPIN; ++i) {
        uint32_t ok;
        asm volatile("{\n.reg .pred p;\nmbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2;\nselp.u32 %0, 1, 0, p;\n}"
                     : "=r"(ok) : "r"(amt_smem(bar)), "r"(parity) : "memory");
        if (ok) return true;
        if (i > 256) __nanosleep(64);
    }
    return false;
}
__device__ __forceinline__ uint32_t amt_map(uint32_t local_addr, int rank) {
    uint32_t r;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(local_addr), "r"(rank));
    return r;
}
__device__ __forceinline__ float amt_ld_cluster(uint32_t cluster_addr) {
    float v;
    asm volatile("ld.shared::cluster.f32 %0, [%1];" : "=f"(v) : "r"(cluster_addr) : "memory");
    return v;
}
__device__ __forceinline__ void amt_cluster_sync() {
    asm volatile("barrier.cluster.arrive.release.aligned;\nbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
__device__ __forceinline__ void ldmatrix_x4_addr(uint32_t (&r)[4], uint32_t addr) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];\n"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
__device__ __forceinline__ void ldmatrix_x4_trans_addr(uint32_t (&r)[4], uint32_t addr) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];\n"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}

// One warp: its 16 keys (rows slab .. slab+15 of the staged tile) against up to 8 query heads, with the
// KEYS as the 16 rows of the MMA tile and the heads as its 8 columns: S^T = K Q^T and O^T = V^T P^T.  A
// group of 4 heads wastes half of a tile this way, not three quarters, and the products take half as
// many mma.sync instructions, which is what bounds this kernel.  A thread's score fragment holds keys
// lane/4 and lane/4 + 8 for heads 2*(lane%4) and 2*(lane%4) + 1; its running maxima, sums and output
// columns are for those two heads.
// ks, vs: shared addresses of the stage's K and V; each is d/64 panels of [64 keys][128 bytes], swizzled.
template <int DMAX, bool MASK>
__device__ __forceinline__ void warp_tile_swz(const uint32_t (&qf)[DMAX / 16][2], float (&o)[DMAX / 16][4], float (&m)[2],
                                              float (&l)[2], uint32_t ks, uint32_t vs, int slab, int d, int key_base,
                                              int lo, int hi, float scale_log2) {
    int lane = threadIdx.x & 31, quad = lane & 3, grp = lane >> 2;
    int mi = lane >> 3, rr = lane & 7;
    float s[4] = {0.f, 0.f, 0.f, 0.f}, s2[4] = {0.f, 0.f, 0.f, 0.f}, s3[4] = {0.f, 0.f, 0.f, 0.f}, s4[4] = {0.f, 0.f, 0.f, 0.f};
    // K as the A operand: matrices 0,1 = keys slab.., slab+8.. at columns +0; matrices 2,3 at columns +8
    uint32_t krow = ks + (uint32_t)(slab + (mi & 1) * 8 + rr) * 128u;
#pragma unroll
    for (int kk = 0; kk < DMAX / 16; ++kk) {
        if (kk * 16 < d) {
            uint32_t ka[4];
            uint32_t chunk = (uint32_t)((kk & 3) * 2 + (mi >> 1));
            ldmatrix_x4_addr(ka, krow + (uint32_t)(kk >> 2) * 8192u + ((chunk ^ (uint32_t)rr) << 4));
            // four chains of accumulators: an MMA waits for the one four steps before it, not for the last
            if ((kk & 3) == 0) mma16816(s, ka, qf[kk][0], qf[kk][1]);
            else if ((kk & 3) == 1) mma16816(s2, ka, qf[kk][0], qf[kk][1]);
            else if ((kk & 3) == 2) mma16816(s3, ka, qf[kk][0], qf[kk][1]);
            else mma16816(s4, ka, qf[kk][0], qf[kk][1]);
        }
    }
#pragma unroll
    for (int e = 0; e < 4; ++e) s[e] = (s[e] + s2[e]) + (s3[e] + s4[e]);
    if (MASK) {
        int k_a = key_base + grp, k_b = k_a + 8;
        if (!(k_a >= lo && k_a <= hi)) s[0] = s[1] = -INFINITY;
        if (!(k_b >= lo && k_b <= hi)) s[2] = s[3] = -INFINITY;
    }
    // maxima over the 16 keys: within the thread, then over the 8 threads that share lane % 4
    float mx[2] = {fmaxf(s[0], s[2]), fmaxf(s[1], s[3])};
    float alpha[2], muse[2];
#pragma unroll
    for (int r = 0; r < 2; ++r) {
        mx[r] = fmaxf(mx[r], __shfl_xor_sync(0xffffffffu, mx[r], 4));
        mx[r] = fmaxf(mx[r], __shfl_xor_sync(0xffffffffu, mx[r], 8));
        mx[r] = fmaxf(mx[r], __shfl_xor_sync(0xffffffffu, mx[r], 16));
        float mn = fmaxf(m[r], mx[r] * scale_log2);
        muse[r] = mn == -INFINITY ? 0.f : mn;
        alpha[r] = ce_exp2_fast(m[r] - muse[r]);
        m[r] = mn;
        l[r] *= alpha[r];
    }
    float p[4];
#pragma unroll
    for (int e = 0; e < 4; ++e) {
        p[e] = ce_exp2_fast(fmaf(s[e], scale_log2, -muse[e & 1]));
        l[e & 1] += p[e];                       // this thread's keys only: the 8 partial sums are added at the end
    }
    // most tiles move no head's maximum: then every alpha is exactly 1 and the output needs no rescaling
    if (__any_sync(0xffffffffu, alpha[0] != 1.0f || alpha[1] != 1.0f)) {
#pragma unroll
        for (int dn = 0; dn < DMAX / 16; ++dn) {
            o[dn][0] *= alpha[0]; o[dn][1] *= alpha[1]; o[dn][2] *= alpha[0]; o[dn][3] *= alpha[1];
        }
    }
    // P^T as the B operand: this thread needs head lane/4 at keys 2q, 2q+1 (b0) and 2q+8, 2q+9 (b1), q = lane%4.
    // Key 2q (+8) lies in the thread with lane/4 = 2q, key 2q+1 (+8) in the one with lane/4 = 2q+1; both
    // hold the head pair (lane/4)/2 when their lane%4 equals that; the head's parity picks the half.
    uint32_t p01 = pack_bf16(p[0], p[1]), p23 = pack_bf16(p[2], p[3]);
    int src_a = ((2 * quad) << 2) | (grp >> 1), src_b = ((2 * quad + 1) << 2) | (grp >> 1);
    uint32_t a01 = __shfl_sync(0xffffffffu, p01, src_a), a23 = __shfl_sync(0xffffffffu, p23, src_a);
    uint32_t b01 = __shfl_sync(0xffffffffu, p01, src_b), b23 = __shfl_sync(0xffffffffu, p23, src_b);
    uint32_t sel = (grp & 1) ? 0x7632u : 0x5410u;       // high halves or low halves of (x, y)
    uint32_t pb0 = __byte_perm(a01, b01, sel), pb1 = __byte_perm(a23, b23, sel);
    // V^T as the A operand (transposed on load): matrices 0,1 = keys slab..+7 at d columns +0, +8;
    // matrices 2,3 = keys slab+8..+15 at d columns +0, +8
    uint32_t vrow = vs + (uint32_t)(slab + (mi >> 1) * 8 + rr) * 128u;
#pragma unroll
    for (int dn = 0; dn < DMAX / 16; ++dn) {
        if (dn * 16 < d) {
            uint32_t va[4];
            uint32_t chunk = (uint32_t)(dn * 2 + (mi & 1));
            ldmatrix_x4_trans_addr(va, vrow + (chunk >> 3) * 8192u + (((chunk & 7u) ^ (uint32_t)rr) << 4));
            mma16816(o[dn], va, pb0, pb1);
        }
    }
}

template <int DMAX, int ST>
__global__ void __launch_bounds__(AMT_THREADS) attention_decode_tma_kernel(const __grid_constant__ CUtensorMap map_k,
                                                                          const __grid_constant__ CUtensorMap map_v,
                                                                          MmaAttnArgs a, int box_rows) {
    // Dependent launch: positions, sequence slots and block tables are inputs of the step (complete
    // before its first kernel may start), and every key but the newest was written by earlier steps.  So
    // the block looks up its pages and starts the copies of all tiles except the one that holds the
    // newest key while the kernels before it still run; only that tile, the query and everything the
    // block writes wait for them.
    ce_pdl_launch_dependents();
    extern __shared__ __align__(1024) unsigned char smem_raw[];
    __shared__ __align__(8) uint64_t full_bar[ST], empty_bar[ST];
    int b = blockIdx.x / a.max_splits, split = blockIdx.x % a.max_splits;
    int kvh = blockIdx.y, hg = blockIdx.z;
    int G = a.nh / a.nkv;
    int t = b;
    int pos = a.positions[t];
    int lo = a.window > 0 ? max(0, pos - a.window + 1) : 0;
    int k_begin = split * a.split, k_end = min(k_begin + a.split, pos + 1);
    bool idle = k_begin > pos || k_end <= lo;     // no visible key in this split: the merge skips it
    if (idle && !a.cluster_merge) return;
    const int* table = a.block_table + (size_t)a.seq_slot[b] * a.max_pages;
    int d = a.d, panels = d >> 6;
    uint32_t base = (amt_smem(smem_raw) + 1023u) & ~1023u;        // the swizzle is keyed on address bits
    unsigned char* tiles = smem_raw + (base - amt_smem(smem_raw));
    uint32_t kv_bytes = (uint32_t)panels * 8192u;                 // K (or V) of one stage
    uint32_t stage_bytes = 2u * kv_bytes;
    int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, quad = lane & 3, grp = lane >> 2;
    int n_tiles = idle ? 0 : (k_end - k_begin + AM_TILE - 1) / AM_TILE;

    if (threadIdx.x == 0) {
        for (int s = 0; s < ST; ++s) {
            asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(amt_smem(&full_bar[s])), "r"(1));
            asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(amt_smem(&empty_bar[s])), "r"(4));
        }
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncthreads();

    if (warp == 4) {
        // ---- producer
        // The page ids of this split's pieces, looked up by the whole warp at once: one trip to the block table
        // instead of one per piece in the copying thread's chain (the table is an input of the step).
        constexpr int PAGES_AHEAD = 512;
        __shared__ int s_pages[PAGES_AHEAD];
        {
            int shift = 31 - __clz(a.page_size);
            int pieces = n_tiles * (AM_TILE / box_rows);
            for (int e = lane; e < min(pieces, PAGES_AHEAD); e += 32) s_pages[e] = table[(k_begin + e * box_rows) >> shift];
            __syncwarp();
        }
        if (lane == 0) {
            int shift = 31 - __clz(a.page_size);
            int per_tile = AM_TILE / box_rows;
            int s = 0;
            uint32_t ph = 0;
            bool wrapped = false, ok = true, waited = false;
            for (int it = 0; it < n_tiles && ok; ++it) {
                if (wrapped) ok = amt_wait(&empty_bar[s], ph ^ 1);
                if (!ok) { atomicExch(a.status, 7); break; }
                int k0 = k_begin + it * AM_TILE;
                if (!waited && k0 + AM_TILE > pos) { ce_pdl_wait(); waited = true; }   // the newest key is written by the kernel before this one
                // the pieces of this tile that hold a visible key
                int first = 0, last = AM_TILE / box_rows - 1;
                while (first < last && k0 + (first + 1) * box_rows <= lo) ++first;
                while (last > first && k0 + last * box_rows > pos) --last;
                uint32_t bar = amt_smem(&full_bar[s]);
                uint32_t bytes = (uint32_t)(last - first + 1) * (uint32_t)box_rows * 128u * 2u * (uint32_t)panels;
                asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
                for (int j = first; j <= last; ++j) {
                    int key = k0 + j * box_rows;
                    int piece = it * per_tile + j;
                    int page = piece < PAGES_AHEAD ? s_pages[piece] : table[key >> shift];
                    if (page < 0 || page >= a.num_pages) { atomicExch(a.status, 4); page = 0; }
                    int row = (page * a.nkv + kvh) * a.page_size + (key & (a.page_size - 1));
                    uint32_t dst = base + (uint32_t)s * stage_bytes + (uint32_t)(j * box_rows) * 128u;
                    for (int pn = 0; pn < panels; ++pn) {
                        asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
                                     ::"r"(dst + (uint32_t)pn * 8192u), "l"(&map_k), "r"(bar), "r"(pn * 64), "r"(row) : "memory");
                        asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
                                     ::"r"(dst + kv_bytes + (uint32_t)pn * 8192u), "l"(&map_v), "r"(bar), "r"(pn * 64), "r"(row) : "memory");
                    }
                }
                if (++s == ST) { s = 0; ph ^= 1; wrapped = true; }
            }
        }
        if (!a.cluster_merge) return;       // the computing warps wait for every copy before they leave the loop
    }

    int heads_here = min(8, G - hg * 8);
    float* so = reinterpret_cast<float*>(tiles);             // [4][8][d]: the warps' outputs (the stages are free by then)
    float* sm = so + 4 * 8 * d;                              // [4][8] maxima
    float* sl = sm + 32;                                     // [4][8] sums
    float* fm = sl + 32;                                     // [8] the block's maximum per head
    float* fl = fm + 8;                                      // [8] the block's sum per head
    if (warp < 4) {
    ce_pdl_wait();
    // Q^T as the B operand: head lane/4, columns kk*16 + 2*(lane%4) (+1) and + 8 (+9)
    uint32_t qf[DMAX / 16][2];
    {
        const bf16* q0 = a.q + (size_t)t * a.q_stride + (size_t)(kvh * G + hg * 8 + grp) * d;
        bool v0 = grp < heads_here;
#pragma unroll
        for (int kk = 0; kk < DMAX / 16; ++kk) {
            int col = kk * 16 + 2 * quad;
            bool in = kk * 16 < d;
            qf[kk][0] = (in && v0) ? *reinterpret_cast<const uint32_t*>(q0 + col) : 0u;
            qf[kk][1] = (in && v0) ? *reinterpret_cast<const uint32_t*>(q0 + col + 8) : 0u;
        }
    }
    float o[DMAX / 16][4];      // O^T: rows d = dn*16 + lane/4 (+8), columns heads 2*(lane%4) (+1)
#pragma unroll
    for (int i = 0; i < DMAX / 16; ++i) o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f;
    float m[2] = {-INFINITY, -INFINITY}, l[2] = {0.f, 0.f};

    {
        int s = 0;
        uint32_t ph = 0;
        bool ok = true;
        for (int it = 0; it < n_tiles; ++it) {
            if (ok) ok = amt_wait(&full_bar[s], ph);
            if (!ok) { if (lane == 0) atomicExch(a.status, 7); break; }
            int k0 = k_begin + it * AM_TILE + warp * 16;
            if (k0 <= pos && k0 + 15 >= lo) {
                uint32_t ks = base + (uint32_t)s * stage_bytes, vs = ks + kv_bytes;
                if (k0 >= lo && k0 + 15 <= pos) {
                    warp_tile_swz<DMAX, false>(qf, o, m, l, ks, vs, warp * 16, d, k0, lo, pos, a.scale_log2);
                } else {
                    // zero the V rows of this warp's keys that are not visible (16 bytes a lane and step)
                    for (int c = lane; c < 16 * panels * 8; c += 32) {
                        int r = c / (panels * 8), rest = c - r * (panels * 8);
                        int key = k0 + r;
                        if (key < lo || key > pos)
                            *reinterpret_cast<uint4*>(tiles + (size_t)s * stage_bytes + kv_bytes + (size_t)(rest >> 3) * 8192 +
                                                      (size_t)(warp * 16 + r) * 128 + (size_t)(rest & 7) * 16) = make_uint4(0, 0, 0, 0);
                    }
                    __syncwarp();
                    warp_tile_swz<DMAX, true>(qf, o, m, l, ks, vs, warp * 16, d, k0, lo, pos, a.scale_log2);
                    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");   // before a later copy overwrites these rows
                }
            }
            __syncwarp();
            if (lane == 0) asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(amt_smem(&empty_bar[s])) : "memory");
            if (++s == ST) { s = 0; ph ^= 1; }
        }
    }
    asm volatile("bar.sync 1, 128;" ::: "memory");       // every warp is done with the staged tiles
#pragma unroll
    for (int r = 0; r < 2; ++r) {              // the sums of the 8 threads that share a head pair
        l[r] += __shfl_xor_sync(0xffffffffu, l[r], 4);
        l[r] += __shfl_xor_sync(0xffffffffu, l[r], 8);
        l[r] += __shfl_xor_sync(0xffffffffu, l[r], 16);
    }
    // combine the 4 warps through shared memory (the staging buffers are free now)
#pragma unroll
    for (int dn = 0; dn < DMAX / 16; ++dn) {
        if (dn * 16 < d) {
            int row = dn * 16 + grp;
            so[(warp * 8 + 2 * quad) * d + row] = o[dn][0];
            so[(warp * 8 + 2 * quad + 1) * d + row] = o[dn][1];
            so[(warp * 8 + 2 * quad) * d + row + 8] = o[dn][2];
            so[(warp * 8 + 2 * quad + 1) * d + row + 8] = o[dn][3];
        }
    }
    if (grp == 0) {
        sm[warp * 8 + 2 * quad] = m[0]; sm[warp * 8 + 2 * quad + 1] = m[1];
        sl[warp * 8 + 2 * quad] = l[0]; sl[warp * 8 + 2 * quad + 1] = l[1];
    }
    asm volatile("bar.sync 1, 128;" ::: "memory");
    for (int e = threadIdx.x; e < heads_here * d; e += 128) {
        int r = e / d, col = e - r * d;
        float M = fmaxf(fmaxf(sm[r], sm[8 + r]), fmaxf(sm[16 + r], sm[24 + r]));
        float acc = 0.f, L = 0.f;
#pragma unroll
        for (int w = 0; w < 4; ++w) {
            float f = sm[w * 8 + r] == -INFINITY ? 0.f : ce_exp2_fast(sm[w * 8 + r] - M);
            acc += so[(w * 8 + r) * d + col] * f;
            L += sl[w * 8 + r] * f;
        }
        if (a.cluster_merge) {
            // stays in this block's shared memory (in the slot of warp 0, which only this thread reads)
            so[r * d + col] = acc;
            if (col == 0) { fm[r] = idle ? -INFINITY : M; fl[r] = idle ? 0.f : L; }
            continue;
        }
        int h = kvh * G + hg * 8 + r;
        size_t pb = ((size_t)b * a.nh + h) * a.max_splits + split;
        a.part_o[pb * d + col] = acc;
        if (col == 0) {
            a.part_ml[pb * 2] = M;
            a.part_ml[pb * 2 + 1] = L;
        }
    }
    }   // warp < 4
    if (!a.cluster_merge) return;
    // Merge inside the cluster: the blocks of a cluster are the splits of one sequence and KV head.  Every
    // block has its (maximum, sum, output) per head in shared memory; block r of the cluster merges a
    // slice of the (head, column) elements of all blocks, in split order, and writes the result.  The
    // arithmetic is the merge kernel's: weights 2^(m_s - M) / sum_s l_s 2^(m_s - M).
    __syncwarp();
    amt_cluster_sync();
    if (warp < 4) {
        int ns = a.max_splits, rank = split;
        int total = heads_here * d, per = (total + ns - 1) / ns;
        int e_end = min(total, (rank + 1) * per);
        for (int e = rank * per + (int)threadIdx.x; e < e_end; e += 128) {
            int r = e / d, col = e - r * d;
            float ms[8], M = -INFINITY;
#pragma unroll
            for (int sp = 0; sp < 8; ++sp) {
                ms[sp] = sp < ns ? amt_ld_cluster(amt_map(amt_smem(fm + r), sp)) : -INFINITY;
                M = fmaxf(M, ms[sp]);
            }
            float L = 0.f, acc = 0.f, w[8];
#pragma unroll
            for (int sp = 0; sp < 8; ++sp) {
                w[sp] = (sp < ns && ms[sp] != -INFINITY) ? ce_exp2_fast(ms[sp] - M) : 0.f;
                if (w[sp] != 0.f) L += amt_ld_cluster(amt_map(amt_smem(fl + r), sp)) * w[sp];
            }
            float inv = L > 0.f ? 1.0f / L : 0.f;
#pragma unroll
            for (int sp = 0; sp < 8; ++sp)
                if (w[sp] != 0.f) acc = fmaf(amt_ld_cluster(amt_map(amt_smem(so + r * d + col), sp)), w[sp] * inv, acc);
            int h = kvh * G + hg * 8 + r;
            a.out[((size_t)t * a.nh + h) * d + col] = __float2bfloat16_rn(acc);
        }
    }
    __syncwarp();
    amt_cluster_sync();          // no block's shared memory goes away while another may still read it
}

// grid (n_seqs, nh), one warp per 32 output columns: out[t, h, :] = sum_s O_s w_s with
// w_s = 2^(m_s - M) / sum_s l_s 2^(m_s - M).  The weights are computed once per block by warp 0
// (lanes over splits, fixed shuffle order), then every thread adds its column in split order.
__global__ void attention_merge_kernel(MmaAttnArgs a) {
    ce_pdl_begin();
    extern __shared__ float wts[];                              // [s1 - s0 + 1]
    int b = blockIdx.x, h = blockIdx.y;
    int t = a.q_start[b];
    int pos = a.positions[t];
    int lo = a.window > 0 ? max(0, pos - a.window + 1) : 0;
    int s0 = lo / a.split, s1 = pos / a.split;                  // splits that hold visible keys
    int ns = s1 - s0 + 1;
    size_t base = ((size_t)b * a.nh + h) * a.max_splits + s0;
    if (threadIdx.x < 32) {
        int lane = threadIdx.x;
        float M = -INFINITY;
        for (int s = lane; s < ns; s += 32) M = fmaxf(M, a.part_ml[(base + s) * 2]);
        for (int o = 16; o > 0; o >>= 1) M = fmaxf(M, __shfl_xor_sync(0xffffffffu, M, o));
        float L = 0.f;
        for (int s = lane; s < ns; s += 32) {
            float ms = a.part_ml[(base + s) * 2];
            float f = ms == -INFINITY ? 0.f : ce_exp2_fast(ms - M);
            wts[s] = f;
            L += a.part_ml[(base + s) * 2 + 1] * f;
        }
        for (int o = 16; o > 0; o >>= 1) L += __shfl_xor_sync(0xffffffffu, L, o);
        float inv = L > 0.f ? 1.0f / L : 0.f;
        __syncwarp();
        for (int s = lane; s < ns; s += 32) wts[s] *= inv;
    }
    __syncthreads();
    for (int col = threadIdx.x; col < a.d; col += blockDim.x) {
        float acc = 0.f;
#pragma unroll 8
        for (int s = 0; s < ns; ++s) acc = fmaf(a.part_o[(base + s) * a.d + col], wts[s], acc);
        a.out[((size_t)t * a.nh + h) * a.d + col] = __float2bfloat16_rn(acc);
    }
}

// ---------------------------------------------------------------------------------------------
// Prefill: grid (n_tiles, nh)
// ---------------------------------------------------------------------------------------------
template <int DMAX>
__global__ void __launch_bounds__(AM_THREADS, DMAX <= 128 ? 3 : 1) attention_prefill_kernel(MmaAttnArgs a) {
    ce_pdl_begin();
    extern __shared__ __align__(16) unsigned char smem_raw[];
    int b = a.tiles[2 * blockIdx.x], q0 = a.tiles[2 * blockIdx.x + 1];
    int h = blockIdx.y, kvh = h / (a.nh / a.nkv);
    int t0 = a.q_start[b], q_len = a.q_start[b + 1] - t0;
    int ctx_before = a.ctx_len[b] - q_len;
    int nq = min(64, q_len - q0);
    int p_first = ctx_before + q0, p_last = p_first + nq - 1;
    int lo_tile = a.window > 0 ? max(0, p_first - a.window + 1) : 0;
    const int* table = a.block_table + (size_t)a.seq_slot[b] * a.max_pages;
    int d = a.d, ld = d + AM_PAD;
    bf16* Ks = reinterpret_cast<bf16*>(smem_raw);
    bf16* Vs = Ks + AM_PF_STAGES * AM_TILE * ld;

    int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, quad = lane & 3, grp = lane >> 2;
    int r0 = warp * 16 + grp, r1 = r0 + 8;                   // this thread's two query rows within the tile
    bool v0 = r0 < nq, v1 = r1 < nq;
    uint32_t qf[DMAX / 16][4];
    {
        const bf16* qa = a.q + (size_t)(t0 + q0 + r0) * a.q_stride + (size_t)h * d;
        const bf16* qb = a.q + (size_t)(t0 + q0 + r1) * a.q_stride + (size_t)h * d;
#pragma unroll
        for (int kk = 0; kk < DMAX / 16; ++kk) {
            int col = kk * 16 + 2 * quad;
            bool in = kk * 16 < d;
            qf[kk][0] = (in && v0) ? *reinterpret_cast<const uint32_t*>(qa + col) : 0u;
            qf[kk][1] = (in && v1) ? *reinterpret_cast<const uint32_t*>(qb + col) : 0u;
            qf[kk][2] = (in && v0) ? *reinterpret_cast<const uint32_t*>(qa + col + 8) : 0u;
            qf[kk][3] = (in && v1) ? *reinterpret_cast<const uint32_t*>(qb + col + 8) : 0u;
        }
    }
    float o[DMAX / 8][4];
#pragma unroll
    for (int i = 0; i < DMAX / 8; ++i) o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f;
    float m[2] = {-INFINITY, -INFINITY}, l[2] = {0.f, 0.f};
    int his[2] = {v0 ? p_first + r0 : -1, v1 ? p_first + r1 : -1};
    int los[2] = {a.window > 0 ? max(0, his[0] - a.window + 1) : 0, a.window > 0 ? max(0, his[1] - a.window + 1) : 0};
    int warp_hi = p_first + min(warp * 16 + 15, nq - 1);     // last key any row of this warp sees
    int warp_lo = a.window > 0 ? max(0, p_first + warp * 16 - a.window + 1) : 0;
    bool warp_rows_full = warp * 16 + 15 < nq;                // all 16 rows of the warp are real queries
    int warp_first_hi = p_first + warp * 16;                  // the warp's first row sees keys up to here
    int warp_last_lo = a.window > 0 ? max(0, p_first + warp * 16 + 15 - a.window + 1) : 0;

    int k_begin = lo_tile / AM_TILE * AM_TILE;
    int n_tiles = (p_last - k_begin) / AM_TILE + 1;
#pragma unroll
    for (int p = 0; p < AM_PF_STAGES - 1; ++p) {
        if (p < n_tiles)
            stage_tile(Ks + p * AM_TILE * ld, Vs + p * AM_TILE * ld, a, table, kvh, k_begin + p * AM_TILE, lo_tile, p_last);
        cp_async_commit();
    }
    for (int it = 0; it < n_tiles; ++it) {
        cp_async_wait<AM_PF_STAGES - 2>();
        __syncthreads();
        int nxt = it + AM_PF_STAGES - 1;
        if (nxt < n_tiles) {
            int st = nxt % AM_PF_STAGES;
            stage_tile(Ks + st * AM_TILE * ld, Vs + st * AM_TILE * ld, a, table, kvh, k_begin + nxt * AM_TILE, lo_tile, p_last);
        }
        cp_async_commit();
        int cur = it % AM_PF_STAGES;
        int k0 = k_begin + it * AM_TILE;
        if (warp * 16 < nq && k0 <= warp_hi && k0 + AM_TILE > warp_lo) {
            const bf16* kt = Ks + cur * AM_TILE * ld;
            const bf16* vt = Vs + cur * AM_TILE * ld;
            // all 64 keys visible to all 16 rows of the warp: at or below its first row, at or above its last row's window
            if (warp_rows_full && k0 + AM_TILE - 1 <= warp_first_hi && k0 >= warp_last_lo)
                warp_tile<DMAX, 8, false>(qf, o, m, l, kt, vt, ld, d, k0, los, his, a.scale_log2);
            else
                warp_tile<DMAX, 8, true>(qf, o, m, l, kt, vt, ld, d, k0, los, his, a.scale_log2);
        }
    }
    cp_async_wait<0>();
#pragma unroll
    for (int r = 0; r < 2; ++r) {
        l[r] += __shfl_xor_sync(0xffffffffu, l[r], 1);
        l[r] += __shfl_xor_sync(0xffffffffu, l[r], 2);
    }
    float inv0 = l[0] > 0.f ? 1.0f / l[0] : 0.f, inv1 = l[1] > 0.f ? 1.0f / l[1] : 0.f;
    bf16* oa = a.out + ((size_t)(t0 + q0 + r0) * a.nh + h) * d;
    bf16* ob = a.out + ((size_t)(t0 + q0 + r1) * a.nh + h) * d;
#pragma unroll
    for (int dn = 0; dn < DMAX / 8; ++dn) {
        if (dn * 8 < d) {
            int col = dn * 8 + 2 * quad;
            if (v0) *reinterpret_cast<uint32_t*>(oa + col) = pack_bf16(o[dn][0] * inv0, o[dn][1] * inv0);
            if (v1) *reinterpret_cast<uint32_t*>(ob + col) = pack_bf16(o[dn][2] * inv1, o[dn][3] * inv1);
        }
    }
}

static size_t stage_bytes(int d, int stages = AM_STAGES) { return (size_t)stages * 2 * AM_TILE * (d + AM_PAD) * sizeof(bf16); }

static int check_common(const char* who, int nh, int nkv, int d, int q_stride) {
    if (d < 16 || d > 256 || d % 16) return ce_fail(CE_ERR_SIZE, "%s: head_dim %d must be a multiple of 16 in 16..256", who, d);
    if (nkv <= 0 || nh % nkv) return ce_fail(CE_ERR_SIZE, "%s: %d heads are not a multiple of %d kv heads", who, nh, nkv);
    if (q_stride % 2) return ce_fail(CE_ERR_SIZE, "%s: the row stride of q must be even", who);
    return CE_OK;
}

template <typename F> static int set_smem(F kernel, size_t bytes, const char* who) {
    if (bytes > 48 * 1024) {
        cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)bytes);
        if (e != cudaSuccess) return ce_fail(CE_ERR_CUDA, "%s: %s", who, cudaGetErrorString(e));
    }
    return CE_OK;
}

// Scratch floats the decode kernel needs for n_seqs sequences.
extern "C" long long ce_attention_decode_scratch(int n_seqs, int nh, int d, int max_splits) {
    return (long long)n_seqs * nh * max_splits * (d + 2);
}

// The first n_seqs sequences of the step bring one token each (tokens 0 .. n_seqs-1).
// max_splits >= ceil(longest context / AM_SPLIT): the grid's upper bound; the split size is chosen from it
// and from the number of sequences (see below), so results differ in rounding between bounds, not more.
extern "C" int ce_attention_decode_split() { return AM_SPLIT; }
// Kernels one decode attention call launches: 1 when the last block merges the splits, else 2.
// (of the call before: the in-cluster merge needs one kernel, the merge kernel a second)
static int g_decode_launches = 2;
extern "C" int ce_attention_decode_kernels() { return g_decode_launches; }

// The TMA-staged decode kernel takes head sizes of 64, 128, 192, 256 and pages of a power of two >= 8.
extern "C" int ce_attention_decode_tma_supported(int d, int page_size) {
    return d >= 64 && d <= 256 && d % 64 == 0 && page_size >= 8 && (page_size & (page_size - 1)) == 0;
}

extern "C" int ce_attention_decode_bf16(const void* q, const void* k_pool, const void* v_pool, void* out, float* scratch,
                                        int* counters, int n_counters, const int* positions, const int* seq_slot, const int* q_start,
                                        const int* ctx_len, const int* block_table, int* status, int n_seqs, int nh,
                                        int nkv, int d, int q_stride, int page_size, int max_pages, int num_pages,
                                        int window, float scale, int max_splits, cudaStream_t stream) {
    if (n_seqs == 0) return CE_OK;
    if (!q || !k_pool || !v_pool || !out || !scratch || !counters || !positions || !seq_slot || !q_start || !ctx_len || !block_table || !status)
        return ce_fail(CE_ERR_ARG, "ce_attention_decode_bf16: null pointer");
    int rc = check_common("ce_attention_decode_bf16", nh, nkv, d, q_stride);
    if (rc) return rc;
    if (max_splits <= 0 || (long long)n_seqs * max_splits > 2147483647LL)
        return ce_fail(CE_ERR_SIZE, "ce_attention_decode_bf16: %d sequences x %d splits", n_seqs, max_splits);
    MmaAttnArgs a{};
    a.q = (const bf16*)q; a.k_pool = (const bf16*)k_pool; a.v_pool = (const bf16*)v_pool; a.out = (bf16*)out;
    a.part_o = scratch; a.part_ml = scratch + (size_t)n_seqs * nh * max_splits * d;
    a.positions = positions; a.seq_slot = seq_slot; a.q_start = q_start; a.ctx_len = ctx_len; a.block_table = block_table;
    a.status = status; a.nh = nh; a.nkv = nkv; a.d = d; a.q_stride = q_stride; a.page_size = page_size;
    a.max_pages = max_pages; a.num_pages = num_pages; a.window = window;
    a.scale_log2 = scale * 1.4426950408889634f;
    int G = nh / nkv;
    static int use_tma = getenv("CE_ATTN_NO_TMA") ? 0 : 1;
    static int fused = getenv("CE_ATTN_FUSED_MERGE") ? 1 : 0;
    bool tma = use_tma && !fused && ce_attention_decode_tma_supported(d, page_size);
    int hgroup = tma ? 8 : 16;           // query heads of one KV head that a block takes
    static int no_cluster = getenv("CE_ATTN_NO_CLUSTER") ? 1 : 0;
    bool cluster_ok = tma && !no_cluster;  // the splits of a sequence merge inside a cluster: no merge kernel
    // Split size: a multiple m of AM_SPLIT.  A block has a fixed cost (launch, the chain of loads that
    // leads to its first tile, combining its warps, writing a partial) counted as fourteen tiles of work, and
    // blocks run in waves of `slots`; m minimises waves x (tiles of a block + 14).  Few sequences get many
    // short splits that fill one wave; many sequences get one block each.  The splits of a sequence merge
    // inside a cluster (at most 8 of them) or, where that leaves most of the GPU idle (one sequence with a
    // long context: 8 KV heads x 8 splits are 64 blocks), through scratch memory and a merge kernel, whose
    // launch is worth about six tiles more.  The choice depends on the number of one-token sequences and on
    // max_splits, not on their contents.
    bool use_cluster = false;
    {
        long long pairs = (long long)n_seqs * nkv * ((G + hgroup - 1) / hgroup);
        long long slots = 2LL * ce_sm_count();           // two blocks share an SM (shared memory of three stages each)
        long long best = -1;
        int best_m = 1;
        for (int m = 1; m <= max_splits; ++m) {
            int splits = (max_splits + m - 1) / m;
            long long blocks = pairs * splits;
            // a block's fixed cost in tiles' worth of time.  The bound the splits are cut from is rounded up to a bucket
            // (one captured graph per bucket), so a sequence's last split is part empty; with a small fixed cost the
            // model cut many sequences in two unequal splits where one block a sequence is faster.  Measured with 6 /
            // 10 / 14 units, ms a step: batch 128 at 2,048 tokens 12.34 / 11.66 / 11.65, batch 64 at 8,192 17.54 /
            // 15.97 / 15.98, batch 8 at 32,768 9.57 / 9.57 / 9.03; batch 1 to 64 at 2,048 and batch 1 at 32,768 the same.
            const int fixed_units = 14;
            long long work = ((blocks + slots - 1) / slots) * ((long long)m * (AM_SPLIT / AM_TILE) + fixed_units);
            if (cluster_ok && splits <= 8 && (best < 0 || work < best)) { best = work; best_m = m; use_cluster = true; }
            long long with_merge = work + (splits > 1 ? 6 : 0);
            if ((!cluster_ok || splits > 8) && (best < 0 || with_merge < best)) { best = with_merge; best_m = m; use_cluster = false; }
        }
        a.split = best_m * AM_SPLIT;
        a.max_splits = (max_splits + best_m - 1) / best_m;
    }
    max_splits = a.max_splits;
    // A merge kernel combines the splits.  CE_ATTN_FUSED_MERGE=1 lets the last block of a (sequence,
    // KV head) do it instead; measured slower (4.9 -> 5.0 ms a step at batch 8, 8B sizes), so it is off.
    a.fused_merge = fused && (size_t)16 * max_splits * sizeof(float) <= 16 * 1024;
    dim3 grid(n_seqs * max_splits, nkv, (G + hgroup - 1) / hgroup);
    if (!tma && (long long)n_seqs * nkv * grid.z > n_counters)
        return ce_fail(CE_ERR_ARG, "ce_attention_decode_bf16: %lld counters needed, %d given", (long long)n_seqs * nkv * grid.z, n_counters);
    a.counters = counters;
    size_t comb = (size_t)(4 * 16 * d + 128) * sizeof(float);
    if (tma) {
        // staged by TMA: pieces of min(page, 64) rows x 64 columns
        int box_rows = page_size < AM_TILE ? page_size : AM_TILE;
        long long pool_rows = (long long)num_pages * nkv * page_size;
        CUtensorMap mk, mv;
        if ((rc = ce_tensor_map_bf16(k_pool, pool_rows, d, d, box_rows, &mk, "ce_attention_decode_bf16"))) return rc;
        if ((rc = ce_tensor_map_bf16(v_pool, pool_rows, d, d, box_rows, &mv, "ce_attention_decode_bf16"))) return rc;
        // three stages: with two (and three blocks an SM) the computing warps wait for data (measured:
        // 30 against 22 microseconds at batch 8)
        bool deep3 = d <= 128;
        size_t stage = (size_t)2 * (d / 64) * 8192;
        size_t tsmem = (deep3 ? 3 : 2) * stage;
        if (comb > tsmem) tsmem = comb;
        tsmem += 1024;
        a.cluster_merge = use_cluster;
        cudaLaunchConfig_t cfg = {};
        cfg.gridDim = grid;
        cfg.blockDim = dim3(AMT_THREADS);
        cfg.dynamicSmemBytes = tsmem;
        cfg.stream = stream;
        cudaLaunchAttribute attr[2];
        int n_attr = 0;
        if (ce_pdl_enabled()) {
            attr[n_attr].id = cudaLaunchAttributeProgrammaticStreamSerialization;
            attr[n_attr].val.programmaticStreamSerializationAllowed = 1;
            ++n_attr;
        }
        if (a.cluster_merge) {
            attr[n_attr].id = cudaLaunchAttributeClusterDimension;
            attr[n_attr].val.clusterDim.x = max_splits; attr[n_attr].val.clusterDim.y = 1; attr[n_attr].val.clusterDim.z = 1;
            ++n_attr;
        }
        cfg.attrs = attr;
        cfg.numAttrs = n_attr;
        cudaError_t le = cudaSuccess;
        ce_note(a.cluster_merge ? "attention_decode_tma_kernel (merge in the cluster)" : "attention_decode_tma_kernel");
#define AMT_CASE(DM)                                                                                                   \
        if (deep3) {                                                                                                   \
            if ((rc = set_smem(attention_decode_tma_kernel<DM, 3>, tsmem, "ce_attention_decode_bf16"))) return rc;     \
            le = cudaLaunchKernelEx(&cfg, attention_decode_tma_kernel<DM, 3>, mk, mv, a, box_rows);                    \
        } else {                                                                                                       \
            if ((rc = set_smem(attention_decode_tma_kernel<DM, 2>, tsmem, "ce_attention_decode_bf16"))) return rc;     \
            le = cudaLaunchKernelEx(&cfg, attention_decode_tma_kernel<DM, 2>, mk, mv, a, box_rows);                    \
        }
        if (d == 64) { AMT_CASE(64) } else if (d == 128) { AMT_CASE(128) } else { AMT_CASE(256) }
#undef AMT_CASE
        if (le != cudaSuccess) return ce_fail(CE_ERR_CUDA, "ce_attention_decode_bf16: %s", cudaGetErrorString(le));
        if ((rc = ce_check_launch("ce_attention_decode_bf16"))) return rc;
        g_decode_launches = a.cluster_merge ? 1 : 2;
        if (a.cluster_merge) return CE_OK;
        { ce_note("attention_merge_kernel"); ce_launch(attention_merge_kernel, dim3(n_seqs, nh), d >= 128 ? 128 : (d + 31) / 32 * 32, max_splits * sizeof(float), stream, a); }
        return ce_check_launch("ce_attention_decode_bf16 (merge)");
    }
    size_t smem = stage_bytes(d);
    if (comb > smem) smem = comb;
    // Few blocks: three staging buffers each (loads run further ahead).  Many blocks: two, so that three
    // blocks share an SM (measured: 4.67 vs 4.83 ms a step at batch 8, 5990 vs 5630 tokens/s at batch 64).
    bool deep = (long long)grid.x * grid.y * grid.z <= 1200;
    if (!deep) {
        smem = stage_bytes(d, 2);
        if (comb > smem) smem = comb;
    }
#define AM_DECODE_CASE(DM)                                                                                        \
    if (deep) {                                                                                                   \
        if ((rc = set_smem(attention_decode_kernel<DM, 3>, smem, "ce_attention_decode_bf16"))) return rc;         \
        { ce_note("attention_decode_kernel"); ce_launch(attention_decode_kernel<DM, 3>, grid, AM_THREADS, smem, stream, a); }                             \
    } else {                                                                                                      \
        if ((rc = set_smem(attention_decode_kernel<DM, 2>, smem, "ce_attention_decode_bf16"))) return rc;         \
        { ce_note("attention_decode_kernel"); ce_launch(attention_decode_kernel<DM, 2>, grid, AM_THREADS, smem, stream, a); }                             \
    }
    if (d <= 64) { AM_DECODE_CASE(64) } else if (d <= 128) { AM_DECODE_CASE(128) } else { AM_DECODE_CASE(256) }
#undef AM_DECODE_CASE
    if ((rc = ce_check_launch("ce_attention_decode_bf16"))) return rc;
    g_decode_launches = a.fused_merge ? 1 : 2;
    if (a.fused_merge) return CE_OK;
    { ce_note("attention_merge_kernel"); ce_launch(attention_merge_kernel, dim3(n_seqs, nh), d >= 128 ? 128 : (d + 31) / 32 * 32, max_splits * sizeof(float), stream, a); }
    return ce_check_launch("ce_attention_decode_bf16 (merge)");
}

// tiles: [n_tiles, 2] = (sequence, first new token of the tile); tiles cover the sequences that
// bring more than one token, 64 tokens at a time.
extern "C" int ce_attention_prefill_bf16(const void* q, const void* k_pool, const void* v_pool, void* out,
                                         const int* positions, const int* seq_slot, const int* q_start,
                                         const int* ctx_len, const int* block_table, const int* tiles, int* status,
                                         int n_tiles, int nh, int nkv, int d, int q_stride, int page_size,
                                         int max_pages, int num_pages, int window, float scale, cudaStream_t stream) {
    if (n_tiles == 0) return CE_OK;
    if (!q || !k_pool || !v_pool || !out || !positions || !seq_slot || !q_start || !ctx_len || !block_table || !tiles || !status)
        return ce_fail(CE_ERR_ARG, "ce_attention_prefill_bf16: null pointer");
    int rc = check_common("ce_attention_prefill_bf16", nh, nkv, d, q_stride);
    if (rc) return rc;
    if (nh > 65535) return ce_fail(CE_ERR_SIZE, "ce_attention_prefill_bf16: %d heads", nh);
    MmaAttnArgs a{};
    a.q = (const bf16*)q; a.k_pool = (const bf16*)k_pool; a.v_pool = (const bf16*)v_pool; a.out = (bf16*)out;
    a.positions = positions; a.seq_slot = seq_slot; a.q_start = q_start; a.ctx_len = ctx_len; a.block_table = block_table;
    a.tiles = tiles; a.status = status; a.nh = nh; a.nkv = nkv; a.d = d; a.q_stride = q_stride; a.page_size = page_size;
    a.max_pages = max_pages; a.num_pages = num_pages; a.window = window;
    a.scale_log2 = scale * 1.4426950408889634f;
    dim3 grid(n_tiles, nh);
    size_t smem = stage_bytes(d, AM_PF_STAGES);
    if (d <= 64) {
        if ((rc = set_smem(attention_prefill_kernel<64>, smem, "ce_attention_prefill_bf16"))) return rc;
        { ce_note("attention_prefill_kernel"); ce_launch(attention_prefill_kernel<64>, grid, AM_THREADS, smem, stream, a); }
    } else if (d <= 128) {
        if ((rc = set_smem(attention_prefill_kernel<128>, smem, "ce_attention_prefill_bf16"))) return rc;
        { ce_note("attention_prefill_kernel"); ce_launch(attention_prefill_kernel<128>, grid, AM_THREADS, smem, stream, a); }
    } else {
        if ((rc = set_smem(attention_prefill_kernel<256>, smem, "ce_attention_prefill_bf16"))) return rc;
        { ce_note("attention_prefill_kernel"); ce_launch(attention_prefill_kernel<256>, grid, AM_THREADS, smem, stream, a); }
    }
    return ce_check_launch("ce_attention_prefill_bf16");
}
