// y = x * W^T in bfloat16 on the 5th-generation tensor cores (tcgen05.mma, accumulators in tensor
// memory, operands brought into shared memory by TMA), with the epilogue fused: store in bfloat16,
// store float32 (logits), add into the float32 residual stream, or SwiGLU.
//
// The product is computed "swapped": a tile of 128 weight rows (output features) is the M operand of
// the MMA, the tokens are its N operand (16 to 256 of them), so that decode steps with a handful of
// tokens still fill the tensor core's M dimension and stream each weight exactly once.  Both operands
// are K-major as stored (W is [out, in], x is [tokens, in]), in 128-byte-swizzled tiles of 64 k.
//
// Up to 256 tokens (128 where a product has tiles enough for the CTA pairs): one CTA computes one 128 x BN
// output tile, optionally over a slice of K (split-K, used
// when there are fewer tiles than SMs).  For SwiGLU the 128 rows of a tile are 64 gate rows and the 64 up
// rows of the same features (two TMA boxes), so it is one product with one accumulator like the others,
// and it is never split.  More tokens: persistent kernels further down (CTA pairs with cta_group::2).
// Warp 0 issues the TMA loads, warp 1 owns tensor memory and issues the MMAs, warps 2-5 read the
// accumulators back (tcgen05.ld) and run the epilogue.  With split-K every CTA writes its partial
// sums to scratch memory; the CTA that arrives last for a tile adds the partials in split order
// (a fixed order, so the result does not depend on which CTA came last) and runs the epilogue.  With
// more than 8 tokens every CTA of the tile does that for its share of the tokens, once all partials
// are there (the CTAs of such a launch are resident together; the wait is bounded like the others).
// No load uses cluster multicast.  Every wait on an mbarrier is bounded: on a timeout the kernel sets
// status 5, waits (bounded) for its own copies in flight, frees its tensor memory and returns.
//
// The reference calls a library (cuBLAS through candle) for these products and runs the residual
// add, SiLU and multiply as separate kernels (src/model/layers.rs:441, 625-648).
#include "common.cuh"
#include "tensor_map.h"
#include <mutex>
#include <stdio.h>
#include <stdlib.h>
#include <unordered_map>

namespace {

constexpr int BM = 128;          // weight rows per tile = UMMA M
constexpr int BK = 64;           // k per stage: 64 bf16 = 128 bytes = one swizzle row
constexpr int UMMA_K = 16;
constexpr int THREADS = 192;
constexpr uint32_t SPIN_LIMIT = 1u << 20;     // with the back-off below: about a second at most

enum { TC_STORE = 0, TC_STORE_F32 = 1, TC_ACCUM_F32 = 2, TC_SWIGLU = 3 };

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count));
}
__device__ __forceinline__ void mbar_expect_tx(uint64_t* bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint64_t* bar, uint32_t parity) {
    uint32_t ok;
    asm volatile("{\n.reg .pred p;\nmbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2;\nselp.u32 %0, 1, 0, p;\n}"
                 : "=r"(ok) : "r"(smem_u32(bar)), "r"(parity) : "memory");
    return ok != 0;
}
// Bounded wait.  Returns false if the phase did not complete within the limit.
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity) {
    for (uint32_t i = 0; i < SPIN_LIMIT; ++i) {
        if (mbar_try_wait(bar, parity)) return true;
        if (i > 64) __nanosleep(i > 4096 ? 1024 : 128);       // test_wait never blocks: the bound is in this loop alone
    }
    return false;
}
__device__ __forceinline__ void tma_load_2d(void* dst, const CUtensorMap* map, uint64_t* bar, int x, int y) {
    asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
                 ::"r"(smem_u32(dst)), "l"(map), "r"(smem_u32(bar)), "r"(x), "r"(y) : "memory");
}
__device__ __forceinline__ uint64_t umma_desc(uint32_t smem_addr) {
    // K-major, 128-byte swizzle: rows of 128 bytes, 8-row groups 1024 bytes apart
    uint64_t d = 0;
    d |= (uint64_t)((smem_addr & 0x3FFFF) >> 4);          // start address
    d |= (uint64_t)1 << 16;                                // leading byte offset (unused for this layout)
    d |= (uint64_t)(1024 >> 4) << 32;                      // stride byte offset
    d |= (uint64_t)1 << 46;                                // descriptor version of sm_100
    d |= (uint64_t)2 << 61;                                // SWIZZLE_128B
    return d;
}
__device__ __forceinline__ void umma_bf16(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc, uint32_t accumulate) {
    asm volatile("{\n.reg .pred p;\nsetp.ne.b32 p, %4, 0;\ntcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n}"
                 ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate) : "memory");
}
__device__ __forceinline__ void umma_commit(uint64_t* bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void tmem_ld16(uint32_t taddr, float (&v)[16]) {
    uint32_t r[16];
    asm volatile("tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
                   "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
                 : "r"(taddr));
    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
    for (int i = 0; i < 16; ++i) v[i] = __uint_as_float(r[i]);
}

// Optional timing trace (CE_GEMM_TRACE=1): block (0,0,0) of every launch stamps %globaltimer at a few
// places into a ring of 256 records; ce_gemm_tc_trace() copies the ring out.  Off by default.
__device__ unsigned long long g_trace[256 * 8];
__device__ unsigned int g_trace_n;
__device__ unsigned long long g_trace_all[256 * 4];      // per launch (sequence number & 255): latest mainloop end, partials written, block end
__device__ __forceinline__ unsigned long long gtime() {
    unsigned long long t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    return t;
}


// ---- clusters: rank of this CTA, addresses in another CTA's shared memory, cluster-wide barrier
__device__ __forceinline__ uint32_t cluster_rank() {
    uint32_t r;
    asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
    return r;
}
__device__ __forceinline__ uint32_t map_to_cta(uint32_t local_addr, uint32_t rank) {
    uint32_t r;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(local_addr), "r"(rank));
    return r;
}
__device__ __forceinline__ float ld_cluster_f32(uint32_t cluster_addr) {
    float v;
    asm volatile("ld.shared::cluster.f32 %0, [%1];" : "=f"(v) : "r"(cluster_addr) : "memory");
    return v;
}
__device__ __forceinline__ void cluster_sync_all() {
    asm volatile("barrier.cluster.arrive.release.aligned;\nbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}

struct TcArgs {
    void* out;               // [M, ldo] bf16 or float32
    float* scratch;          // split-K partials: [splits][tiles][BN][128]
    int* counters;           // one per output tile, zero between launches
    int* status;
    int M, N, K, ldo, mode, splits, kblocks_per_split, kblocks, trace;
    int cluster;             // 1: the splits of a tile form a cluster and add their partial sums through shared memory
    int coop;                // 1: every split of a tile adds the partial sums for a share of the tile's tokens (more than 8 tokens)
};

__device__ __forceinline__ float silu_mul(float g, float u) { return g / (1.0f + __expf(-g)) * u; }
// the same with the approximate reciprocal (the result is rounded to bfloat16 right after)
__device__ __forceinline__ float silu_mul_fast(float g, float u) { return __fdividef(g, 1.0f + __expf(-g)) * u; }

__device__ __forceinline__ void epilogue_store(const TcArgs& a, int m, int n, float v, float up) {
    size_t o = (size_t)m * a.ldo + n;
    if (a.mode == TC_STORE) ((__nv_bfloat16*)a.out)[o] = __float2bfloat16_rn(v);
    else if (a.mode == TC_STORE_F32) ((float*)a.out)[o] = v;
    else if (a.mode == TC_ACCUM_F32) ((float*)a.out)[o] += v;
    else ((__nv_bfloat16*)a.out)[o] = __float2bfloat16_rn(silu_mul(v, up));
}

template <int BN, int NACC, bool COOP>
__global__ void __launch_bounds__(THREADS, 2) gemm_tc_kernel(const __grid_constant__ CUtensorMap map_w,
                                                         const __grid_constant__ CUtensorMap map_x, TcArgs a, int stages) {
    extern __shared__ __align__(1024) unsigned char smem_raw[];
    __shared__ __align__(8) uint64_t full_bar[8], empty_bar[8], acc_bar;
    __shared__ uint32_t tmem_slot;
    __shared__ int s_ticket, s_abort, s_acc_ok;
    // NACC == 2 stands for SwiGLU: the block's 128 weight rows are 64 gate rows and the 64 up rows of the
    // same features (two TMA boxes into one tile), the product has ONE accumulator like any other, and
    // the two threads of a feature meet in the epilogue through this buffer.  K is never split then.
    constexpr bool GU = NACC == 2;
    __shared__ float xbuf[GU ? 2 * 2 * 64 * 9 : 1];

    constexpr uint32_t W_BYTES = BM * BK * 2, X_BYTES = BN * BK * 2;
    constexpr uint32_t STAGE_BYTES = W_BYTES + X_BYTES;
    constexpr uint32_t TMEM_COLS = BN < 32 ? 32 : BN;
    // the dynamic buffer is aligned to 1024 bytes by hand: the swizzle pattern is keyed on address bits
    uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    unsigned char* tiles = smem_raw + (base - smem_u32(smem_raw));

    int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    int n0 = blockIdx.x * (GU ? BM / 2 : BM), m0 = blockIdx.y * BN, split = blockIdx.z;
    int kb0 = split * a.kblocks_per_split;
    int kb1 = min(kb0 + a.kblocks_per_split, a.kblocks);
    int nkb = kb1 - kb0;
    __shared__ unsigned long long* s_rec;
    bool tracing = a.trace && blockIdx.x == 0 && blockIdx.y == 0 && blockIdx.z == 0;
    if (tracing && threadIdx.x == 0) {
        unsigned int idx = atomicAdd(&g_trace_n, 1u) & 255u;
        s_rec = g_trace + idx * 8;
        s_rec[0] = gtime();
        s_rec[7] = ((unsigned long long)a.N << 32) | (unsigned)a.K;
    }

    // Dependent launch: this grid may start while the kernel before it still runs.  Weights are
    // written by no kernel, so their loads start at once; the tokens (and everything the epilogue
    // reads or writes) wait until the grids before this one are complete.
    ce_pdl_launch_dependents();
    if (threadIdx.x == 0) {
        for (int s = 0; s < stages; ++s) { mbar_init(&full_bar[s], 1); mbar_init(&empty_bar[s], 1); }
        mbar_init(&acc_bar, 1);
        s_abort = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&tmem_slot)), "r"(TMEM_COLS));
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;");
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    uint32_t tmem = tmem_slot;

    if (warp == 0) {
        if (lane == 0) {
            // ---- producer: TMA loads of the weight tile(s) and the token tile, stage after stage
            int issued = 0;
            bool ok = true;
            int first = min(nkb, stages);
            for (int i = 0; i < first; ++i) {            // weights of the first stages: before the wait
                unsigned char* st = tiles + (size_t)i * STAGE_BYTES;
                mbar_expect_tx(&full_bar[i], STAGE_BYTES);
                int k = (kb0 + i) * BK;
                tma_load_2d(st, &map_w, &full_bar[i], k, n0);
                if (GU) tma_load_2d(st + W_BYTES / 2, &map_w, &full_bar[i], k, a.N + n0);
            }
            ce_pdl_wait();
            if (tracing) s_rec[1] = gtime();
            for (int i = 0; i < first; ++i) {            // their tokens: after it
                tma_load_2d(tiles + (size_t)i * STAGE_BYTES + W_BYTES, &map_x, &full_bar[i], (kb0 + i) * BK, m0);
                issued = i + 1;
            }
            int s = first == stages ? 0 : first;         // stage and parity walk along without divisions
            uint32_t eph = 0;                            // parity of the phase that frees stage s for its next use
            for (int i = first; i < nkb && ok; ++i) {
                ok = mbar_wait(&empty_bar[s], eph);
                if (!ok) break;
                unsigned char* st = tiles + (size_t)s * STAGE_BYTES;
                mbar_expect_tx(&full_bar[s], STAGE_BYTES);
                int k = (kb0 + i) * BK;
                tma_load_2d(st, &map_w, &full_bar[s], k, n0);
                if (GU) tma_load_2d(st + W_BYTES / 2, &map_w, &full_bar[s], k, a.N + n0);
                tma_load_2d(st + W_BYTES, &map_x, &full_bar[s], k, m0);
                issued = i + 1;
                if (++s == stages) { s = 0; eph ^= 1; }
            }
            if (!ok) {
                atomicExch(a.status, 5);
                atomicExch(&s_abort, 1);
                // our own copies may still be in flight: wait for them (bounded) before the block ends
                for (int i = max(0, issued - stages); i < issued; ++i) mbar_wait(&full_bar[i % stages], (i / stages) & 1);
            }
        }
    } else if (warp == 1) {
        if (lane == 0) {
            // ---- MMA issuer
            uint32_t idesc = (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(BN >> 3) << 17) | ((uint32_t)(BM >> 4) << 24);
            bool ok = true, ready = false;
            int s = 0;
            uint32_t ph = 0;
            const uint64_t desc_hi = umma_desc(0);
            for (int i = 0; i < nkb; ++i) {
                // this thread's instruction stream bounds a block's rate when few blocks share the weights:
                // no divisions, and the next stage's barrier is tested before this stage's MMAs are issued
                if (!ready) ok = mbar_wait(&full_bar[s], ph);
                if (!ok) break;
                if (tracing && i == 0) s_rec[2] = gtime();
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                int sn = s + 1 == stages ? 0 : s + 1;
                uint32_t phn = sn == 0 ? ph ^ 1 : ph;
                ready = i + 1 < nkb && mbar_try_wait(&full_bar[sn], phn);
                uint32_t st = (base + s * STAGE_BYTES) >> 4;
#pragma unroll
                for (int kk = 0; kk < BK / UMMA_K; ++kk) {
                    uint64_t bdesc = desc_hi | (uint64_t)((st + ((W_BYTES + kk * UMMA_K * 2) >> 4)) & 0x3FFF);
                    uint32_t acc = (i > 0 || kk > 0) ? 1u : 0u;
                    umma_bf16(tmem, desc_hi | (uint64_t)((st + ((kk * UMMA_K * 2) >> 4)) & 0x3FFF), bdesc, idesc, acc);
                }
                umma_commit(&empty_bar[s]);          // the stage is free once these MMAs have read it
                s = sn; ph = phn;
            }
            if (ok) umma_commit(&acc_bar);           // the accumulators are complete
            else { atomicExch(a.status, 5); atomicExch(&s_abort, 1); }
            if (tracing) s_rec[3] = gtime();
            if (a.trace) atomicMax(&g_trace_all[(a.trace & 255) * 4 + 0], gtime());
        }
    } else {
        // ---- epilogue: 4 warps, each reads the 32 accumulator lanes of its quadrant
        int quad = warp & 3;
        int row = quad * 32 + lane;                  // feature within the tile
        int n = n0 + (GU ? (row & 63) : row);
        int m_valid = min(BN, a.M - m0);
        ce_pdl_wait();
        // one thread waits for the accumulators and the others take its verdict: threads that each polled for
        // themselves could disagree at the limit and then miss one another at the barriers below
        if (threadIdx.x == 64) {
            bool there = nkb > 0 ? mbar_wait(&acc_bar, 0) : true;
            if (!there) { atomicExch(a.status, 5); atomicExch(&s_abort, 1); }
            s_acc_ok = there ? 1 : 0;
        }
        asm volatile("bar.sync 1, 128;" ::: "memory");
        bool ok = s_acc_ok != 0;
        if (tracing && threadIdx.x == 64) s_rec[4] = gtime();
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        uint32_t taddr = tmem + ((uint32_t)(quad * 32) << 16);
        if (GU) {
            // Rows 64..127 of the tile hold the up values of the features whose gate values rows 0..63 hold.  The
            // two threads of a feature share each chunk of 16 tokens: the gate thread takes tokens 0..7 (and
            // needs their up values), the up thread tokens 8..15 (and needs their gate values).
            bool up_row = row >= 64;
#pragma unroll 1
            for (int c = 0; c < BN; c += 16) {
                if (c >= m_valid) break;
                float g[16];
                if (ok && nkb > 0) tmem_ld16(taddr + c, g);
                else {
#pragma unroll
                    for (int j = 0; j < 16; ++j) g[j] = 0.f;
                }
                float* xg = xbuf + ((c >> 4) & 1) * (2 * 64 * 9) + (row & 63) * 9;     // gate values of tokens 8..15
                float* xu = xg + 64 * 9;                                              // up values of tokens 0..7
#pragma unroll
                for (int j = 0; j < 8; ++j) {
                    if (up_row) xu[j] = g[j];
                    else xg[j] = g[8 + j];
                }
                asm volatile("bar.sync 2, 128;" ::: "memory");     // (the buffer used two chunks ago has been read by then)
                if (ok && n < a.N) {
                    int t0 = up_row ? 8 : 0;
                    __nv_bfloat16* op = (__nv_bfloat16*)a.out + (size_t)(m0 + c + t0) * a.ldo + n;
#pragma unroll
                    for (int j = 0; j < 8; ++j) {
                        float gate = up_row ? xg[j] : g[j];
                        float upv = up_row ? g[8 + j] : xu[j];
                        if (c + t0 + j < m_valid) op[(size_t)j * a.ldo] = __float2bfloat16_rn(silu_mul_fast(gate, upv));
                    }
                }
            }
        } else if (a.splits == 1) {
            if (ok) {
#pragma unroll 1
                for (int c = 0; c < BN; c += 16) {
                    if (c >= m_valid) break;
                    float g[16];
                    tmem_ld16(taddr + c, g);
                    if (n < a.N) {
                        if (a.mode == TC_ACCUM_F32) {
                            float* xp = (float*)a.out + (size_t)(m0 + c) * a.ldo + n;
                            float xv[16];
#pragma unroll
                            for (int j = 0; j < 16; ++j) xv[j] = (c + j < m_valid) ? xp[(size_t)j * a.ldo] : 0.f;
#pragma unroll
                            for (int j = 0; j < 16; ++j)
                                if (c + j < m_valid) xp[(size_t)j * a.ldo] = xv[j] + g[j];
                        } else {
#pragma unroll
                            for (int j = 0; j < 16; ++j)
                                if (c + j < m_valid) epilogue_store(a, m0 + c + j, n, g[j], 0.f);
                        }
                    }
                }
            }
        } else if (a.cluster) {
            // partial sums to this block's shared memory (the stages are free: every load has been
            // consumed by an MMA that has completed): [acc][m][128]; they are added after the role branches
            float* part = reinterpret_cast<float*>(tiles);
#pragma unroll 1
            for (int c = 0; c < BN; c += 16) {
                if (c >= m_valid) break;
                float g[16];
                if (nkb > 0 && ok) {
                    tmem_ld16(taddr + c, g);
                } else {
#pragma unroll
                    for (int j = 0; j < 16; ++j) g[j] = 0.f;
                }
#pragma unroll
                for (int j = 0; j < 16; ++j) {
                    if (c + j < m_valid) {
                        part[(size_t)(c + j) * BM + row] = g[j];
                    }
                }
            }
        } else {
            // partial sums to scratch: [split][tile][m][128]
            int tile = blockIdx.y * gridDim.x + blockIdx.x;
            int n_tiles = gridDim.x * gridDim.y;
            float* mine = a.scratch + ((size_t)split * n_tiles + tile) * BN * BM;
            if (ok) {
#pragma unroll 1
                for (int c = 0; c < BN; c += 16) {
                    if (c >= m_valid) break;
                    float g[16];
                    if (nkb > 0) {
                        tmem_ld16(taddr + c, g);
                        } else {
#pragma unroll
                        for (int j = 0; j < 16; ++j) g[j] = 0.f;
                    }
#pragma unroll
                    for (int j = 0; j < 16; ++j) {
                        if (c + j < m_valid) {
                            mine[(size_t)(c + j) * BM + row] = g[j];
                        }
                    }
                }
            }
            __threadfence();
            asm volatile("bar.sync 1, 128;" ::: "memory");
            if (tracing && threadIdx.x == 64) s_rec[5] = gtime();
            if (a.trace && threadIdx.x == 64) atomicMax(&g_trace_all[(a.trace & 255) * 4 + 1], gtime());
            // Who adds the partial sums.  Few tokens: the block of a tile that arrives last, all of them in one trip
            // to L2.  More tokens (coop): a single block would make a trip per 8 tokens, one after the other (11 us
            // for 64 tokens), so EVERY split of the tile waits until all partial sums are there (all splits of a
            // launch are resident at once: the grid is sized for that) and then adds them for its own share of the
            // tokens.  Either way each result is one sum in split order.
            int m_lo = 0, m_hi = m_valid;
            bool adds = false;
            if (COOP) {
                if (threadIdx.x == 64) {
                    atomicAdd(&a.counters[tile], 1);
                    bool there = false;
                    for (uint32_t i = 0; i < SPIN_LIMIT && !there; ++i) {
                        int v;
                        asm volatile("ld.acquire.gpu.global.s32 %0, [%1];" : "=r"(v) : "l"(a.counters + tile) : "memory");
                        there = v >= a.splits;
                        if (!there && i > 32) __nanosleep(i > 4096 ? 1024 : 64);
                    }
                    if (!there) { atomicExch(a.status, 5); atomicExch(&s_abort, 1); }
                    s_ticket = there ? 1 : 0;
                }
                asm volatile("bar.sync 1, 128;" ::: "memory");
                int per = ((m_valid + a.splits - 1) / a.splits + 7) & ~7;      // whole batches of 8 tokens
                m_lo = min(m_valid, split * per);
                m_hi = min(m_valid, m_lo + per);
                adds = s_ticket != 0;
            } else {
                if (threadIdx.x == 64) s_ticket = atomicAdd(&a.counters[tile], 1);
                asm volatile("bar.sync 1, 128;" ::: "memory");
                adds = s_ticket == a.splits - 1;
            }
            if (adds) {
                __threadfence();
                if (n < a.N && s_abort == 0) {
                    // A batch of tokens at a time, with the loads of up to eight splits (and of the residual
                    // values the tile adds into) all in flight together: one trip to L2 for up to eight
                    // splits.  Sums are taken in split order.
                    constexpr int TB = 8;
                    size_t split_stride = (size_t)n_tiles * BN * BM;
                    const float* p0 = a.scratch + (size_t)tile * BN * BM + row;
                    for (int mb = m_lo; mb < m_hi; mb += TB) {
                        float g[TB], xv[TB];
#pragma unroll
                        for (int j = 0; j < TB; ++j) {
                            g[j] = 0.f;
                            xv[j] = (a.mode == TC_ACCUM_F32 && mb + j < m_hi)
                                        ? __ldcg((const float*)a.out + (size_t)(m0 + mb + j) * a.ldo + n) : 0.f;
                        }
                        for (int s0 = 0; s0 < a.splits; s0 += 8) {
                            float tg[8][TB];
#pragma unroll
                            for (int s = 0; s < 8; ++s) {
                                const float* p = p0 + (size_t)(s0 + s) * split_stride;
#pragma unroll
                                for (int j = 0; j < TB; ++j) {
                                    bool in = s0 + s < a.splits && mb + j < m_hi;
                                    tg[s][j] = in ? __ldcg(p + (size_t)(mb + j) * BM) : 0.f;
                                }
                            }
#pragma unroll
                            for (int s = 0; s < 8; ++s) {
#pragma unroll
                                for (int j = 0; j < TB; ++j) g[j] += tg[s][j];
                            }
                        }
#pragma unroll
                        for (int j = 0; j < TB; ++j) {
                            if (mb + j >= m_hi) continue;
                            if (a.mode == TC_ACCUM_F32) ((float*)a.out)[(size_t)(m0 + mb + j) * a.ldo + n] = xv[j] + g[j];
                            else epilogue_store(a, m0 + mb + j, n, g[j], 0.f);
                        }
                    }
                }
            }
            if (COOP) {
                // the split that finishes last puts both counters back for the next launch (everyone has passed its wait by then)
                asm volatile("bar.sync 1, 128;" ::: "memory");
                if (threadIdx.x == 64 && atomicAdd(&a.counters[n_tiles + tile], 1) == a.splits - 1) {
                    a.counters[tile] = 0;
                    a.counters[n_tiles + tile] = 0;
                }
            } else if (adds) {
                if (threadIdx.x == 64) a.counters[tile] = 0;      // ready for the next launch
            }
        }
        asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    }
    __syncthreads();
    if (a.cluster && a.splits > 1) {
        // Split-K inside the cluster: every block has its partial tile in shared memory; block r adds rows
        // [r * rows_per, ...) of all blocks, in split order (the same order for every token, whatever else
        // is in the batch), and runs the epilogue for them.  No scratch memory, no ticket, no second pass
        // through L2.
        cluster_sync_all();
        if (warp >= 2) {
            int rank = (int)cluster_rank();
            int rows_per = (BM + a.splits - 1) / a.splits;
            int r0 = rank * rows_per, nrows = min(BM, r0 + rows_per) - r0;
            int m_valid = min(BN, a.M - m0);
            uint32_t part0 = smem_u32(tiles);
            int tid = threadIdx.x - 64;
            if (nrows > 0 && s_abort == 0) {
                for (int item = tid; item < nrows * m_valid; item += 128) {
                    int m = item / nrows, row = r0 + (item - m * nrows);
                    int n = n0 + row;
                    if (n >= a.N) continue;
                    uint32_t off = (uint32_t)(m * BM + row) * 4u;
                    float g = 0.f;
                    for (int sp = 0; sp < a.splits; ++sp) {
                        uint32_t remote = map_to_cta(part0 + off, (uint32_t)sp);
                        g += ld_cluster_f32(remote);
                    }
                    if (a.mode == TC_ACCUM_F32) {
                        float* xp = (float*)a.out + (size_t)(m0 + m) * a.ldo + n;
                        *xp = *xp + g;
                    } else {
                        epilogue_store(a, m0 + m, n, g, 0.f);
                    }
                }
            }
        }
        __syncwarp();
        cluster_sync_all();          // nobody's shared memory goes away while another block may still read it
    }
    if (a.trace && threadIdx.x == 0) {
        atomicMax(&g_trace_all[(a.trace & 255) * 4 + 2], gtime());
        if (tracing) { s_rec[6] = (unsigned long long)(a.trace & 255); }
    }
    if (warp == 1) {
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(TMEM_COLS));
    }
}


// ---------------------------------------------------------------------------------------------
// Many tokens (prefill): a persistent kernel.  One CTA per SM walks over output tiles (tokens
// fastest, so the CTAs that run together share weight tiles in L2); tensor memory holds two sets of
// accumulators, so the epilogue of one tile runs while the MMAs of the next fill the other set.
// ---------------------------------------------------------------------------------------------
__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void tmem_ld32(uint32_t taddr, float (&v)[32]) {
    uint32_t r[32];
    asm volatile("tcgen05.ld.sync.aligned.32x32b.x32.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,"
                 "%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31}, [%32];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
                   "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]),
                   "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]),
                   "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
                 : "r"(taddr));
    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
    for (int i = 0; i < 32; ++i) v[i] = __uint_as_float(r[i]);
}

template <int BN, int NACC>
__global__ void __launch_bounds__(THREADS) gemm_tc_persistent_kernel(const __grid_constant__ CUtensorMap map_w,
                                                                    const __grid_constant__ CUtensorMap map_x, TcArgs a,
                                                                    int stages, int tiles_n, int tiles_m) {
    extern __shared__ __align__(1024) unsigned char smem_raw[];
    __shared__ __align__(8) uint64_t full_bar[8], empty_bar[8], acc_full[2], acc_empty[2];
    __shared__ uint32_t tmem_slot;

    constexpr uint32_t W_BYTES = BM * BK * 2, X_BYTES = BN * BK * 2;
    constexpr uint32_t STAGE_BYTES = NACC * W_BYTES + X_BYTES;
    constexpr uint32_t ACC_COLS = NACC * BN;
    constexpr uint32_t TMEM_COLS = 2 * ACC_COLS;
    static_assert(TMEM_COLS <= 512 && (TMEM_COLS & (TMEM_COLS - 1)) == 0, "two accumulator sets must fit tensor memory");
    uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    unsigned char* tiles = smem_raw + (base - smem_u32(smem_raw));
    int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    int total = tiles_n * tiles_m;

    ce_pdl_launch_dependents();
    if (threadIdx.x == 0) {
        for (int s = 0; s < stages; ++s) { mbar_init(&full_bar[s], 1); mbar_init(&empty_bar[s], 1); }
        for (int b = 0; b < 2; ++b) { mbar_init(&acc_full[b], 1); mbar_init(&acc_empty[b], 1); }
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&tmem_slot)), "r"(TMEM_COLS));
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;");
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    uint32_t tmem = tmem_slot;

    if (warp == 0) {
        if (lane == 0) {
            ce_pdl_wait();
            int it = 0, first_in_flight = 0;
            bool ok = true;
            for (int tile = blockIdx.x; tile < total && ok; tile += gridDim.x) {
                int n0 = (tile / tiles_m) * BM, m0 = (tile % tiles_m) * BN;
                for (int kb = 0; kb < a.kblocks; ++kb, ++it) {
                    int s = it % stages;
                    if (it >= stages) ok = mbar_wait(&empty_bar[s], ((it / stages) - 1) & 1);
                    if (!ok) break;
                    unsigned char* st = tiles + (size_t)s * STAGE_BYTES;
                    mbar_expect_tx(&full_bar[s], STAGE_BYTES);
                    tma_load_2d(st, &map_w, &full_bar[s], kb * BK, n0);
                    if (NACC == 2) tma_load_2d(st + W_BYTES, &map_w, &full_bar[s], kb * BK, a.N + n0);
                    tma_load_2d(st + NACC * W_BYTES, &map_x, &full_bar[s], kb * BK, m0);
                }
            }
            if (!ok) {
                atomicExch(a.status, 5);
                first_in_flight = max(0, it - stages);
                for (int i = first_in_flight; i < it; ++i) mbar_wait(&full_bar[i % stages], (i / stages) & 1);
            }
        }
    } else if (warp == 1) {
        if (lane == 0) {
            uint32_t idesc = (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(BN >> 3) << 17) | ((uint32_t)(BM >> 4) << 24);
            int it = 0, lt = 0;
            bool ok = true;
            for (int tile = blockIdx.x; tile < total && ok; tile += gridDim.x, ++lt) {
                int buf = lt & 1;
                if (lt >= 2) ok = mbar_wait(&acc_empty[buf], ((lt >> 1) - 1) & 1);     // the epilogue has drained this set
                if (!ok) break;
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                uint32_t d_tmem = tmem + buf * ACC_COLS;
                for (int kb = 0; kb < a.kblocks; ++kb, ++it) {
                    int s = it % stages;
                    ok = mbar_wait(&full_bar[s], (it / stages) & 1);
                    if (!ok) break;
                    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                    uint32_t st = base + s * STAGE_BYTES;
#pragma unroll
                    for (int kk = 0; kk < BK / UMMA_K; ++kk) {
                        uint64_t bdesc = umma_desc(st + NACC * W_BYTES + kk * UMMA_K * 2);
                        uint32_t acc = (kb > 0 || kk > 0) ? 1u : 0u;
                        umma_bf16(d_tmem, umma_desc(st + kk * UMMA_K * 2), bdesc, idesc, acc);
                        if (NACC == 2) umma_bf16(d_tmem + BN, umma_desc(st + W_BYTES + kk * UMMA_K * 2), bdesc, idesc, acc);
                    }
                    umma_commit(&empty_bar[s]);
                }
                if (ok) umma_commit(&acc_full[buf]);
            }
            if (!ok) atomicExch(a.status, 5);
        }
    } else {
        int quad = warp & 3;
        int row = quad * 32 + lane;
        ce_pdl_wait();
        int lt = 0;
        bool ok = true;
        for (int tile = blockIdx.x; tile < total && ok; tile += gridDim.x, ++lt) {
            int buf = lt & 1;
            int n0 = (tile / tiles_m) * BM, m0 = (tile % tiles_m) * BN;
            int n = n0 + row;
            int m_valid = min(BN, a.M - m0);
            ok = mbar_wait(&acc_full[buf], (lt >> 1) & 1);
            if (!ok) { atomicExch(a.status, 5); break; }
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            uint32_t taddr = tmem + buf * ACC_COLS + ((uint32_t)(quad * 32) << 16);
#pragma unroll 1
            for (int c = 0; c < BN; c += 32) {
                if (c >= m_valid) break;
                float g[32], u[32];
                tmem_ld32(taddr + c, g);
                if (NACC == 2) tmem_ld32(taddr + BN + c, u);
                if (n < a.N) {
                    if (a.mode == TC_ACCUM_F32) {
                        float* xp = (float*)a.out + (size_t)(m0 + c) * a.ldo + n;
                        float xv[32];
#pragma unroll
                        for (int j = 0; j < 32; ++j) xv[j] = (c + j < m_valid) ? xp[(size_t)j * a.ldo] : 0.f;   // all loads first
#pragma unroll
                        for (int j = 0; j < 32; ++j)
                            if (c + j < m_valid) xp[(size_t)j * a.ldo] = xv[j] + g[j];
                    } else {
#pragma unroll
                        for (int j = 0; j < 32; ++j)
                            if (c + j < m_valid) epilogue_store(a, m0 + c + j, n, g[j], NACC == 2 ? u[j] : 0.f);
                    }
                }
            }
            asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
            asm volatile("bar.sync 1, 128;" ::: "memory");
            if (threadIdx.x == 64) mbar_arrive(&acc_empty[buf]);
        }
        asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    }
    __syncthreads();
    if (warp == 1) {
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(TMEM_COLS));
    }
}


// ---------------------------------------------------------------------------------------------
// Many tokens, CTA pairs: two CTAs of a cluster work on one tile of 256 weight rows x BN tokens with
// tcgen05.mma.cta_group::2.  Each CTA loads its own 128 weight rows and only HALF of the token tile;
// the tensor cores of both SMs read both halves, so a pair moves a third less operand data through
// L2 and shared memory per flop than two single CTAs (the single-CTA kernel is bound by exactly that).
// The leader CTA's MMA thread issues the MMAs for both; it learns that the peer's stage has landed
// from an mbarrier that the peer arrives on across the cluster; its tcgen05.commit frees the stage
// and publishes the accumulators in BOTH CTAs (commit with multicast::cluster; loads use none).
// Each CTA runs the epilogue for its own 128 rows out of its own tensor memory.
// ---------------------------------------------------------------------------------------------
// Arrival on a barrier of another CTA of the cluster.  Relaxed: it only says that tensor memory has been
// read (tcgen05.wait::ld has returned); a release here would also wait for the epilogue's global stores.
__device__ __forceinline__ void mbar_arrive_remote(uint32_t cluster_addr) {
    asm volatile("mbarrier.arrive.relaxed.cluster.shared::cluster.b64 _, [%0];" ::"r"(cluster_addr) : "memory");
}
__device__ __forceinline__ bool mbar_test_cluster(uint64_t* bar, uint32_t parity) {
    uint32_t ok;
    asm volatile("{\n.reg .pred p;\nmbarrier.test_wait.parity.acquire.cluster.shared::cta.b64 p, [%1], %2;\nselp.u32 %0, 1, 0, p;\n}"
                 : "=r"(ok) : "r"(smem_u32(bar)), "r"(parity) : "memory");
    return ok != 0;
}
__device__ __forceinline__ bool mbar_wait_cluster(uint64_t* bar, uint32_t parity) {
    for (uint32_t i = 0; i < SPIN_LIMIT; ++i) {
        uint32_t ok;
        asm volatile("{\n.reg .pred p;\nmbarrier.test_wait.parity.acquire.cluster.shared::cta.b64 p, [%1], %2;\nselp.u32 %0, 1, 0, p;\n}"
                     : "=r"(ok) : "r"(smem_u32(bar)), "r"(parity) : "memory");
        if (ok) return true;
        if (i > 64) __nanosleep(i > 4096 ? 1024 : 128);
    }
    return false;
}
// A TMA load of a CTA pair: the data goes to the executing CTA's shared memory, the bytes are counted on
// a barrier that may lie in the other CTA of the pair (a shared::cluster address).  No multicast.
__device__ __forceinline__ void tma_load_2d_pair(void* dst, const CUtensorMap* map, uint32_t cluster_bar, int x, int y) {
    asm volatile("cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
                 ::"r"(smem_u32(dst)), "l"(map), "r"(cluster_bar), "r"(x), "r"(y) : "memory");
}
__device__ __forceinline__ void umma2_bf16(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc, uint32_t accumulate) {
    asm volatile("{\n.reg .pred p;\nsetp.ne.b32 p, %4, 0;\ntcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n}"
                 ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate) : "memory");
}
__device__ __forceinline__ void umma2_commit_both(uint64_t* bar) {
    unsigned short mask = 3;          // the barrier at this offset in both CTAs of the pair
    asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;"
                 ::"r"(smem_u32(bar)), "h"(mask) : "memory");
}

// BN: tokens per pair tile (each CTA loads BN/2 of them).  KSUB: k-blocks of 64 per stage (per barrier
// round of the MMA thread).  GU (SwiGLU): a CTA's 128 rows are 64 gate rows and the 64 up rows of the same
// features, brought by two TMA boxes into ONE tile, so the product is the same single-accumulator product
// as any other and a pair tile covers 128 features; in the epilogue the warps that hold the up rows (lanes
// 64..127 of tensor memory) hand their values to the warps that hold the gate rows through shared memory.
template <int BN, bool GU, int KSUB>
__global__ void __launch_bounds__(THREADS) gemm_tc_pair_kernel(const __grid_constant__ CUtensorMap map_w,
                                                              const __grid_constant__ CUtensorMap map_x, TcArgs a,
                                                              int stages, int tiles_n, int tiles_m) {
    extern __shared__ __align__(1024) unsigned char smem_raw[];
    __shared__ __align__(8) uint64_t full_bar[8], empty_bar[8], acc_full[2], acc_empty[2];
    __shared__ uint32_t tmem_slot;
    __shared__ int s_acc_ok;                         // the epilogue's verdict on a wait, taken by one thread for all 128
    __shared__ float xbuf[GU ? 2 * 2 * 64 * 17 : 1]; // GU: per buffer, 16 gate and 16 up values of 64 features (padded rows)

    constexpr int HALF_N = BN / 2;
    constexpr int ROWS_N = GU ? BM / 2 : BM;         // output features of one CTA's tile
    constexpr uint32_t W_BYTES = BM * BK * 2, X_BYTES = HALF_N * BK * 2;
    constexpr uint32_t SUB_BYTES = W_BYTES + X_BYTES;                 // one k-block: weight rows, then tokens
    constexpr uint32_t STAGE_BYTES = KSUB * SUB_BYTES;
    constexpr uint32_t ACC_COLS = BN;
    constexpr uint32_t TMEM_COLS = 2 * ACC_COLS;
    static_assert(TMEM_COLS <= 512 && (TMEM_COLS & (TMEM_COLS - 1)) == 0, "two accumulator sets must fit tensor memory");
    const int rounds = (a.kblocks + KSUB - 1) / KSUB;                 // a k-block beyond K reads zeros
    uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    unsigned char* tiles = smem_raw + (base - smem_u32(smem_raw));
    int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    uint32_t rank = cluster_rank();                  // 0: leader
    int pair = blockIdx.x >> 1, n_pairs = gridDim.x >> 1;
    int total = tiles_n * tiles_m;                   // pair tiles: tiles_n of 2 * ROWS_N features, tiles_m of BN tokens

    ce_pdl_launch_dependents();
    if (threadIdx.x == 0) {
        for (int s = 0; s < stages; ++s) { mbar_init(&full_bar[s], 1); mbar_init(&empty_bar[s], 1); }
        for (int b = 0; b < 2; ++b) { mbar_init(&acc_full[b], 1); mbar_init(&acc_empty[b], 2); }
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&tmem_slot)), "r"(TMEM_COLS));
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;");
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    cluster_sync_all();                              // both CTAs' barriers exist before anything arrives on them
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    uint32_t tmem = tmem_slot;

    if (warp == 0) {
        if (lane == 0) {
            // ---- producer (in each CTA): its 128 weight rows (and the up rows for SwiGLU), its half of the
            // tokens, into its own shared memory; the bytes of BOTH CTAs are counted on the leader's barrier
            ce_pdl_wait();
            int s = 0, issued = 0;
            uint32_t ph = 0;                 // parity of the phase of empty_bar[s] that frees the stage's previous use
            bool ok = true, wrapped = false;
            for (int tile = pair; tile < total && ok; tile += n_pairs) {
                int n0 = (tile / tiles_m) * (2 * ROWS_N) + rank * ROWS_N, m0 = (tile % tiles_m) * BN + rank * HALF_N;
                for (int r = 0; r < rounds; ++r) {
                    if (wrapped) ok = mbar_wait_cluster(&empty_bar[s], ph ^ 1);
                    if (!ok) break;
                    uint32_t bar = map_to_cta(smem_u32(&full_bar[s]), 0);
                    if (rank == 0) mbar_expect_tx(&full_bar[s], 2 * STAGE_BYTES);
#pragma unroll
                    for (int j = 0; j < KSUB; ++j) {
                        unsigned char* st = tiles + (size_t)s * STAGE_BYTES + j * SUB_BYTES;
                        int kx = (r * KSUB + j) * BK;
                        tma_load_2d_pair(st, &map_w, bar, kx, n0);          // GU: a box of 64 gate rows ...
                        if (GU) tma_load_2d_pair(st + W_BYTES / 2, &map_w, bar, kx, a.N + n0);   // ... and the 64 up rows below them
                        tma_load_2d_pair(st + W_BYTES, &map_x, bar, kx, m0);
                    }
                    ++issued;
                    if (++s == stages) { s = 0; ph ^= 1; wrapped = true; }
                }
            }
            if (!ok) {
                // give the copies in flight time to land before the block may leave (the leader's barriers
                // count the bytes of both blocks; the peer cannot wait on them, so it waits by the clock)
                atomicExch(a.status, 51);
                if (rank == 0) for (int i = max(0, issued - stages); i < issued; ++i) mbar_wait_cluster(&full_bar[i % stages], (i / stages) & 1);
                else for (int i = 0; i < 64; ++i) __nanosleep(1000);
            }
        }
    } else if (warp == 1) {
        if (lane == 0 && rank == 0) {
            // ---- leader: MMAs for both CTAs.  This one thread's instruction stream is the critical path
            // (a barrier test alone takes about a hundred cycles), so the next stage's barrier is tested
            // BEFORE this stage's MMAs are issued: the test's latency passes while they are queued.
            int lt = 0, s = 0;
            uint32_t ph = 0;
            bool ok = true;
            uint32_t idesc = (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(BN >> 3) << 17) | ((uint32_t)((2 * BM) >> 4) << 24);
            const uint64_t desc_hi = umma_desc(0);
            bool ready = false;
            for (int tile = pair; tile < total && ok; tile += n_pairs, ++lt) {
                int buf = lt & 1;
                if (lt >= 2) ok = mbar_wait_cluster(&acc_empty[buf], ((lt >> 1) - 1) & 1);   // both epilogues have drained this set
                if (!ok) { atomicExch(a.status, 52); break; }
                uint32_t d_tmem = tmem + buf * ACC_COLS;
                for (int r = 0; r < rounds; ++r) {
                    if (!ready) ok = mbar_wait_cluster(&full_bar[s], ph);
                    if (!ok) { atomicExch(a.status, 53); break; }
                    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                    int sn = s + 1 == stages ? 0 : s + 1;
                    uint32_t phn = sn == 0 ? ph ^ 1 : ph;
                    ready = mbar_test_cluster(&full_bar[sn], phn);
#pragma unroll
                    for (int j = 0; j < KSUB; ++j) {
                        uint32_t st = (base + s * STAGE_BYTES + j * SUB_BYTES) >> 4;
#pragma unroll
                        for (int kk = 0; kk < BK / UMMA_K; ++kk) {
                            uint64_t bdesc = desc_hi | (uint64_t)((st + ((W_BYTES + kk * UMMA_K * 2) >> 4)) & 0x3FFF);
                            uint32_t acc = (r > 0 || j > 0 || kk > 0) ? 1u : 0u;
                            umma2_bf16(d_tmem, desc_hi | (uint64_t)((st + ((kk * UMMA_K * 2) >> 4)) & 0x3FFF), bdesc, idesc, acc);
                        }
                    }
                    umma2_commit_both(&empty_bar[s]);     // the stage is free in both CTAs
                    s = sn; ph = phn;
                }
                if (ok) umma2_commit_both(&acc_full[buf]);
            }
        }
    } else {
        // ---- epilogue (in each CTA): its own 128 rows
        int quad = warp & 3;
        int row = quad * 32 + lane;
        ce_pdl_wait();
        int lt = 0;
        bool ok = true;
        uint32_t leader_empty[2] = {map_to_cta(smem_u32(&acc_empty[0]), 0), map_to_cta(smem_u32(&acc_empty[1]), 0)};
        for (int tile = pair; tile < total && ok; tile += n_pairs, ++lt) {
            int buf = lt & 1;
            int n = (tile / tiles_m) * (2 * ROWS_N) + rank * ROWS_N + (GU ? (row & 63) : row);
            bool up_row = GU && row >= 64;
            int m0 = (tile % tiles_m) * BN;
            int m_valid = min(BN, a.M - m0);
            const bool accum = !GU && a.mode == TC_ACCUM_F32 && n < a.N;
            float xv[32];
            if (accum) {       // the residual values of the first 32 tokens are on their way before the accumulators are ready
                const float* xp = (const float*)a.out + (size_t)m0 * a.ldo + n;
#pragma unroll
                for (int j = 0; j < 32; ++j) xv[j] = j < m_valid ? xp[(size_t)j * a.ldo] : 0.f;
            }
            // One thread waits (bounded) and all 128 take its verdict: if each polled for itself, a wait that ran
            // out for some threads and not for others would leave them at different barriers for good.
            if (threadIdx.x == 64) s_acc_ok = mbar_wait_cluster(&acc_full[buf], (lt >> 1) & 1) ? 1 : 0;
            asm volatile("bar.sync 1, 128;" ::: "memory");
            ok = s_acc_ok != 0;
            if (!ok) { if (threadIdx.x == 64) atomicExch(a.status, 54); break; }
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            uint32_t taddr = tmem + buf * ACC_COLS + ((uint32_t)(quad * 32) << 16);
            if (!GU && a.mode == TC_ACCUM_F32) {
                // x += product, 32 tokens a chunk; the next chunk's residual values are loaded while this one is stored
#pragma unroll 1
                for (int c = 0; c < BN; c += 32) {
                    if (c >= m_valid) break;
                    float g[32], xn[32];
                    tmem_ld32(taddr + c, g);
                    if (accum) {
                        float* xp = (float*)a.out + (size_t)(m0 + c) * a.ldo + n;
#pragma unroll
                        for (int j = 0; j < 32; ++j) xn[j] = (c + 32 + j < m_valid) ? xp[(size_t)(32 + j) * a.ldo] : 0.f;
#pragma unroll
                        for (int j = 0; j < 32; ++j)
                            if (c + j < m_valid) xp[(size_t)j * a.ldo] = xv[j] + g[j];
#pragma unroll
                        for (int j = 0; j < 32; ++j) xv[j] = xn[j];
                    }
                }
            } else
#pragma unroll 1
            for (int c = 0; c < BN; c += 32) {
                if (c >= m_valid) break;
                float g[32];
                tmem_ld32(taddr + c, g);
                if (GU) {
                    // Rows 64..127 hold the up values of the features whose gate values rows 0..63 hold.  The two
                    // threads of a feature share its 32 tokens: the gate thread takes tokens 0..15 (and needs their
                    // up values), the up thread tokens 16..31 (and needs their gate values); both then work.
                    float* xg = xbuf + ((c >> 5) & 1) * (2 * 64 * 17) + (row & 63) * 17;     // gate values of tokens 16..31
                    float* xu = xg + 64 * 17;                                               // up values of tokens 0..15
#pragma unroll
                    for (int j = 0; j < 16; ++j) {
                        if (up_row) xu[j] = g[j];
                        else xg[j] = g[16 + j];
                    }
                    asm volatile("bar.sync 2, 128;" ::: "memory");     // (the buffer used two chunks ago has been read by then)
                    if (n < a.N) {
                        int t0 = up_row ? 16 : 0;
                        __nv_bfloat16* op = (__nv_bfloat16*)a.out + (size_t)(m0 + c + t0) * a.ldo + n;
#pragma unroll
                        for (int j = 0; j < 16; ++j) {
                            float gate = up_row ? xg[j] : g[j];
                            float upv = up_row ? g[16 + j] : xu[j];
                            if (c + t0 + j < m_valid) op[(size_t)j * a.ldo] = __float2bfloat16_rn(silu_mul_fast(gate, upv));
                        }
                    }
                    continue;
                }
                if (n < a.N) {
#pragma unroll
                    for (int j = 0; j < 32; ++j)
                        if (c + j < m_valid) epilogue_store(a, m0 + c + j, n, g[j], 0.f);
                }
            }
            asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
            asm volatile("bar.sync 1, 128;" ::: "memory");
            if (threadIdx.x == 64) mbar_arrive_remote(leader_empty[buf]);     // (two arrivals: one per CTA)
        }
        asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    }
    __syncthreads();
    cluster_sync_all();                              // nobody leaves while the other may still signal it
    if (warp == 1) {
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(TMEM_COLS));
    }
}

// ---- host side ------------------------------------------------------------------------------------
// bf16 matrix [rows, cols], row stride ld elements, boxes of box_rows x 64 columns, 128-byte swizzle
int get_map(const void* ptr, long long rows, long long cols, long long ld, int box_rows, CUtensorMap* out) {
    return ce_tensor_map_bf16(ptr, rows, cols, ld, box_rows, out, "ce_gemm_tc");
}

template <int BN, int NACC, bool COOP>
int launch(const CUtensorMap& mw, const CUtensorMap& mx, const TcArgs& a, dim3 grid, cudaStream_t stream) {
    constexpr size_t stage = BM * BK * 2 + BN * BK * 2;
    // small tiles: at most half an SM's shared memory, so that the blocks of the next kernel (launched
    // as a programmatic dependent) fit beside these and stream their weights while these finish
    // (measured: best for up to 16 tokens; from 32 tokens on one block per SM with a deeper pipeline wins)
    static int small_kb = getenv("CE_GEMM_SMEM_KB") ? atoi(getenv("CE_GEMM_SMEM_KB")) : 0;
    // (the SwiGLU product has twice the tiles and never splits K: two of its blocks share an SM at every tile size)
    size_t budget = small_kb ? (size_t)small_kb * 1024 : ((BN <= 16 || NACC == 2) ? 100 * 1024 : 200 * 1024);
    int stages = (int)(budget / stage);
    if (stages > 8) stages = 8;
    if (stages < 2) stages = 2;
    size_t smem = stages * stage + 1024;
    static bool attr_set = false;
    if (!attr_set) {
        cudaError_t e = cudaFuncSetAttribute(gemm_tc_kernel<BN, NACC, COOP>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return ce_fail(CE_ERR_CUDA, "ce_gemm_tc: %s", cudaGetErrorString(e));
        attr_set = true;
    }
    if (a.cluster) {
        if ((size_t)BN * BM * 4 > (size_t)stages * stage)
            return ce_fail(CE_ERR_SIZE, "ce_gemm_tc: the partial tile does not fit the stages");
        cudaLaunchConfig_t cfg = {};
        cfg.gridDim = grid;
        cfg.blockDim = dim3(THREADS);
        cfg.dynamicSmemBytes = smem;
        cfg.stream = stream;
        cudaLaunchAttribute attr[2];
        attr[0].id = cudaLaunchAttributeClusterDimension;
        attr[0].val.clusterDim.x = 1; attr[0].val.clusterDim.y = 1; attr[0].val.clusterDim.z = grid.z;
        attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attr[1].val.programmaticStreamSerializationAllowed = 1;
        cfg.attrs = attr;
        cfg.numAttrs = ce_pdl_enabled() ? 2 : 1;
        ce_note("gemm_tc_kernel (split-K in a cluster)");
        cudaError_t e = cudaLaunchKernelEx(&cfg, gemm_tc_kernel<BN, NACC, COOP>, mw, mx, a, stages);
        if (e != cudaSuccess) return ce_fail(CE_ERR_CUDA, "ce_gemm_tc (cluster of %d): %s", (int)grid.z, cudaGetErrorString(e));
        return ce_check_launch("ce_gemm_tc");
    }
    { ce_note(COOP ? "gemm_tc_kernel (split-K, splits add together)" : a.splits > 1 ? "gemm_tc_kernel (split-K)" : "gemm_tc_kernel"); ce_launch(gemm_tc_kernel<BN, NACC, COOP>, grid, THREADS, smem, stream, mw, mx, a, stages); }
    return ce_check_launch("ce_gemm_tc");
}

template <int BN, int NACC>
int launch_persistent(const CUtensorMap& mw, const CUtensorMap& mx, const TcArgs& a, int tiles_n, int tiles_m, cudaStream_t stream) {
    constexpr size_t stage = NACC * BM * BK * 2 + BN * BK * 2;
    int stages = (int)((200 * 1024) / stage);
    if (stages > 8) stages = 8;
    size_t smem = stages * stage + 1024;
    static bool attr_set = false;
    if (!attr_set) {
        cudaError_t e = cudaFuncSetAttribute(gemm_tc_persistent_kernel<BN, NACC>, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024 - 2048);
        if (e != cudaSuccess) return ce_fail(CE_ERR_CUDA, "ce_gemm_tc: %s", cudaGetErrorString(e));
        attr_set = true;
    }
    long long total = (long long)tiles_n * tiles_m;
    int grid = (int)(total < ce_sm_count() ? total : ce_sm_count());
    { ce_note("gemm_tc_persistent_kernel"); ce_launch(gemm_tc_persistent_kernel<BN, NACC>, grid, THREADS, smem, stream, mw, mx, a, stages, tiles_n, tiles_m); }
    return ce_check_launch("ce_gemm_tc (persistent)");
}

template <int BN, bool GU, int KSUB>
int launch_pair(const CUtensorMap& mw, const CUtensorMap& mx, const TcArgs& a, int tiles_n, int tiles_m, cudaStream_t stream) {
    constexpr size_t stage = KSUB * (BM * BK * 2 + (BN / 2) * BK * 2);
    int stages = (int)((200 * 1024) / stage);
    if (stages > 8) stages = 8;
    size_t smem = stages * stage + 1024;
    static bool attr_set = false;
    if (!attr_set) {
        cudaError_t e = cudaFuncSetAttribute(gemm_tc_pair_kernel<BN, GU, KSUB>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return ce_fail(CE_ERR_CUDA, "ce_gemm_tc: %s", cudaGetErrorString(e));
        attr_set = true;
    }
    long long total = (long long)tiles_n * tiles_m;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(2 * (ce_sm_count() / 2));
    cfg.blockDim = dim3(THREADS);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[2];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = 2; attr[0].val.clusterDim.y = 1; attr[0].val.clusterDim.z = 1;
    // Tiles are dealt to pairs in a fixed stride, so every pair has to be resident at once: not every
    // SM can be paired (a cluster lies within one GPC), so ask how many pairs fit.
    static int max_pairs = 0;
    if (max_pairs == 0) {
        cfg.attrs = attr;
        cfg.numAttrs = 1;
        int n = 0;
        cudaError_t e = cudaOccupancyMaxActiveClusters(&n, gemm_tc_pair_kernel<BN, GU, KSUB>, &cfg);
        if (e != cudaSuccess || n < 1) return ce_fail(CE_ERR_CUDA, "ce_gemm_tc (pairs): no resident cluster: %s", cudaGetErrorString(e));
        max_pairs = n;
        if (getenv("CE_GEMM_TRACE")) fprintf(stderr, "[carbon_engine_b200] gemm pairs<%d,%d>: %d resident\n", BN, (int)GU, n);
    }
    int pairs = max_pairs;
    if (total < pairs) pairs = (int)total;
    cfg.gridDim = dim3(2 * pairs);
    attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[1].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = ce_pdl_enabled() ? 2 : 1;
    ce_note("gemm_tc_pair_kernel");
    cudaError_t e = cudaLaunchKernelEx(&cfg, gemm_tc_pair_kernel<BN, GU, KSUB>, mw, mx, a, stages, tiles_n, tiles_m);
    if (e != cudaSuccess) return ce_fail(CE_ERR_CUDA, "ce_gemm_tc (pairs): %s", cudaGetErrorString(e));
    return ce_check_launch("ce_gemm_tc (pairs)");
}

}  // namespace

// Split-K partial sums go through scratch memory and are added by the block of a tile that finishes
// last.  CE_GEMM_CLUSTER=1 adds them inside a cluster, through shared memory, instead: its tail is
// shorter, but a cluster of 6 to 8 blocks is not always resident at once and smaller clusters leave too
// few blocks to keep the memory busy (measured at batch 8, 8B sizes: 4.64 to 4.73 ms a step against 4.56).
static bool cluster_split_k() {
    static int on = getenv("CE_GEMM_CLUSTER") ? 1 : 0;
    return on != 0;
}

// 129 to 256 tokens: a one-block tile of 128 weight rows x 256 tokens needs 48 KB of operands per 64 k, more
// than an SM takes in while it multiplies them; a pair's tile of 256 rows x 256 tokens needs 32 KB a block.  So
// products with at least a dozen pair tiles go to the CTA pairs from 129 tokens on (measured at 8B sizes: a
// 256-token step 8.26 -> 7.95 ms, a decode step at batch 256 20.9 -> 20.0 ms); fewer tiles would leave most
// pairs idle, and the one-block kernel splits K instead; for 65 to 128 tokens the pairs were slower (batch 128:
// 13.9 against 12.9 ms a step).  (CE_GEMM_PAIR_MIN_TOKENS / _TILES move the bounds.)
static bool pairs_from_129(int M, int N, int nacc) {
    static int pair_min_tokens = getenv("CE_GEMM_PAIR_MIN_TOKENS") ? atoi(getenv("CE_GEMM_PAIR_MIN_TOKENS")) : 129;
    static int pair_min_tiles = getenv("CE_GEMM_PAIR_MIN_TILES") ? atoi(getenv("CE_GEMM_PAIR_MIN_TILES")) : 12;
    static int no_pairs = getenv("CE_GEMM_NO_PAIRS") ? 1 : 0;
    long long pair_tiles = nacc == 2 ? (N + BM - 1) / BM : (N + 2 * BM - 1) / (2 * BM);
    return M <= 256 && M >= pair_min_tokens && N >= 2 * BM && pair_tiles >= pair_min_tiles && !no_pairs;
}

// How many splits of K a product of these sizes uses (it depends on N and K only while the tokens
// fit one tile, so a token's sums are taken in the same order whatever else is in the batch).
extern "C" int ce_gemm_tc_tile_tokens(int M);
extern "C" int ce_gemm_tc_splits(int M, int N, int K) {
    int kblocks = (K + BK - 1) / BK;
    if (M > 256 || pairs_from_129(M, N, 1)) return 1;
    int bn = ce_gemm_tc_tile_tokens(M);
    int tiles = ((N + BM - 1) / BM) * ((M + bn - 1) / bn);
    static int target = getenv("CE_GEMM_TARGET_CTAS") ? atoi(getenv("CE_GEMM_TARGET_CTAS")) : 0;
    // up to 16 tokens: about two CTAs per SM, each with half an SM of shared memory; more tokens: one per SM
    int s = (target ? target : (bn <= 16 ? 296 : 148)) / tiles;
    if (s > kblocks / 4) s = kblocks / 4;      // at least four k-blocks per split
    // partial sums cost S * bn * 4 / K of the weight bytes (through L2): at most 60 % (30 % left the O product of 128
    // tokens with 64 blocks: 12.84 against 12.36 ms a step at batch 128; smaller tiles are bound by the other limits)
    int by_traffic = (int)(0.6 * K / (4.0 * bn));
    if (s > by_traffic) s = by_traffic;
    if (s > 8 && bn <= 16) s = 8;              // the last block of a tile then adds all partial sums in one trip to L2
    if (s > 16) s = 16;
    static int max_cluster = getenv("CE_GEMM_MAX_CLUSTER") ? atoi(getenv("CE_GEMM_MAX_CLUSTER")) : 8;
    if (cluster_split_k() && s > max_cluster) s = max_cluster;     // the splits of a tile form one cluster (8 is the portable limit)
    return s < 1 ? 1 : s;
}

// Copies out the timing ring (256 records of 8 values) and the number of records written so far.
extern "C" int ce_gemm_tc_trace(unsigned long long* out, unsigned int* count, unsigned long long* all) {
    if (cudaMemcpyFromSymbol(out, g_trace, sizeof(unsigned long long) * 256 * 8) != cudaSuccess) return CE_ERR_CUDA;
    if (cudaMemcpyFromSymbol(count, g_trace_n, sizeof(unsigned int)) != cudaSuccess) return CE_ERR_CUDA;
    if (all && cudaMemcpyFromSymbol(all, g_trace_all, sizeof(unsigned long long) * 256 * 4) != cudaSuccess) return CE_ERR_CUDA;
    return CE_OK;
}

extern "C" int ce_gemm_tc_tile_tokens(int M) {
    return M <= 16 ? 16 : M <= 32 ? 32 : M <= 64 ? 64 : M <= 128 ? 128 : 256;
}

// Scratch floats a product needs (0 without split-K).
extern "C" long long ce_gemm_tc_scratch(int M, int N, int K, int mode) {
    int s = ce_gemm_tc_splits(M, N, K);
    if (s == 1 || mode == TC_SWIGLU) return 0;         // (the SwiGLU product never splits K)
    int bn = ce_gemm_tc_tile_tokens(M);
    long long tiles = (long long)((N + BM - 1) / BM) * ((M + bn - 1) / bn);
    return (long long)s * tiles * bn * BM;
}

extern "C" int ce_gemm_tc_supported(int M, int N, int K, int lda) {
    return M > 0 && N > 0 && K > 0 && K % 8 == 0 && lda % 8 == 0 && (long long)((N + BM - 1) / BM) <= 65535 * 32;
}

// A [M, K] bf16 (row stride lda), W [N or 2N, K] bf16, C [M, ldc].  N counts output columns
// (for SwiGLU the intermediate width).  counters: at least ceil(N/128) * ceil(M/BN) zeroed ints.
extern "C" int ce_gemm_tc(const void* A, const void* W, void* C, int M, int N, int K, int lda, int ldc, int mode,
                          float* scratch, long long scratch_floats, int* counters, int n_counters, int* status,
                          cudaStream_t stream) {
    if (M == 0 || N == 0) return CE_OK;
    if (!A || !W || !C || !status) return ce_fail(CE_ERR_ARG, "ce_gemm_tc: null pointer");
    if (!ce_gemm_tc_supported(M, N, K, lda))
        return ce_fail(CE_ERR_SIZE, "ce_gemm_tc: K=%d and the row stride %d must be multiples of 8", K, lda);
    if (((uintptr_t)A | (uintptr_t)W) & 15) return ce_fail(CE_ERR_SIZE, "ce_gemm_tc: operands must be 16-byte aligned");
    if (mode < 0 || mode > 3) return ce_fail(CE_ERR_ARG, "ce_gemm_tc: unknown epilogue %d", mode);
    int nacc = mode == TC_SWIGLU ? 2 : 1;
    int kblocks = (K + BK - 1) / BK;
    bool early_pairs = pairs_from_129(M, N, nacc);
    if (M > 256 || early_pairs) {       // many tokens: the persistent kernels, no split-K
        int pbn = nacc == 2 ? 128 : 256;
        long long tiles_m = (M + pbn - 1) / pbn, tiles_n = (N + BM - 1) / BM;
        if (tiles_m * tiles_n > 2147483647LL) return ce_fail(CE_ERR_SIZE, "ce_gemm_tc: too many tiles");
        CUtensorMap pw, px;
        int prc = get_map(W, (long long)N * nacc, K, K, BM, &pw);
        if (prc) return prc;
        if ((prc = get_map(A, M, K, lda, pbn, &px))) return prc;
        static int ptrace = getenv("CE_GEMM_TRACE") ? 1 : 0;
        TcArgs pa{C, scratch, counters, status, M, N, K, ldc, mode, 1, kblocks, kblocks, ptrace, 0};
        static int use_pairs = getenv("CE_GEMM_NO_PAIRS") ? 0 : 1;
        if (use_pairs && N >= 2 * BM) {     // CTA pairs: 256 weight rows a tile, each CTA loads half of the tokens
            // SwiGLU: 128 gate rows and their 128 up rows a pair tile (boxes of 64 rows), 256 tokens as well
            // 256 tokens a tile, or 128 where that needs clearly fewer waves of pairs (a few hundred tokens):
            // waves x time of a tile decides; a tile of 128 tokens takes 0.75 of the time of one of 256 (measured)
            long long rows_t = nacc == 2 ? (N + BM - 1) / BM : (N + 2 * BM - 1) / (2 * BM);
            long long n_pairs = ce_sm_count() / 2;
            long long t256 = rows_t * ((M + 255) / 256), t128 = rows_t * ((M + 127) / 128);
            double c256 = (double)((t256 + n_pairs - 1) / n_pairs), c128 = (double)((t128 + n_pairs - 1) / n_pairs) * 0.75;
            int ptok = c128 < c256 ? 128 : 256;
            CUtensorMap px2, pw2;
            if ((prc = get_map(A, M, K, lda, ptok / 2, &px2))) return prc;
            long long ptiles_m = (M + ptok - 1) / ptok;
            if (nacc == 2) {
                if ((prc = get_map(W, (long long)N * 2, K, K, BM / 2, &pw2))) return prc;
                return ptok == 128 ? launch_pair<128, true, 2>(pw2, px2, pa, (int)rows_t, (int)ptiles_m, stream)
                                   : launch_pair<256, true, 2>(pw2, px2, pa, (int)rows_t, (int)ptiles_m, stream);
            }
            return ptok == 128 ? launch_pair<128, false, 2>(pw, px2, pa, (int)rows_t, (int)ptiles_m, stream)
                               : launch_pair<256, false, 2>(pw, px2, pa, (int)rows_t, (int)ptiles_m, stream);
        }
        return nacc == 2 ? launch_persistent<128, 2>(pw, px, pa, (int)tiles_n, (int)tiles_m, stream)
                         : launch_persistent<256, 1>(pw, px, pa, (int)tiles_n, (int)tiles_m, stream);
    }
    int bn = ce_gemm_tc_tile_tokens(M);
    // SwiGLU: a block takes 64 features (64 gate rows and their 64 up rows in one tile) and all of K
    int rows_n = nacc == 2 ? BM / 2 : BM;
    int splits = nacc == 2 ? 1 : ce_gemm_tc_splits(M, N, K);
    dim3 grid((N + rows_n - 1) / rows_n, (M + bn - 1) / bn, splits);
    if (grid.y > 65535) return ce_fail(CE_ERR_SIZE, "ce_gemm_tc: M=%d is too large", M);
    if (splits > 1) {
        if (!scratch || !counters || scratch_floats < ce_gemm_tc_scratch(M, N, K, mode) || n_counters < (int)(grid.x * grid.y))
            return ce_fail(CE_ERR_ARG, "ce_gemm_tc: split-K needs %lld scratch floats and %d counters",
                           ce_gemm_tc_scratch(M, N, K, mode), grid.x * grid.y);
    }
    CUtensorMap mw, mx;
    int rc = get_map(W, (long long)N * nacc, K, K, rows_n, &mw);
    if (rc) return rc;
    if ((rc = get_map(A, M, K, lda, bn, &mx))) return rc;
    static int trace_on = getenv("CE_GEMM_TRACE") ? 1 : 0;
    static int trace_seq = 0;
    int trace = trace_on ? (++trace_seq | 256) : 0;
    // the partial tile of a block must fit its stages (launch<> sizes them the same way)
    size_t stage_b = (size_t)BM * BK * 2 + (size_t)bn * BK * 2;
    size_t budget_b = (bn <= 16 || nacc == 2) ? 100 * 1024 : 200 * 1024;
    size_t n_st = budget_b / stage_b > 8 ? 8 : (budget_b / stage_b < 2 ? 2 : budget_b / stage_b);
    int cluster = cluster_split_k() && splits > 1 && splits <= 8 && (size_t)bn * BM * 4 <= n_st * stage_b;
    // every split adds a share of the tokens only if all blocks of the launch are resident at once (they wait for one another)
    long long resident = (long long)ce_sm_count() * ((bn <= 16 || nacc == 2) ? 2 : 1);
    static int coop_off = getenv("CE_GEMM_NO_COOP") ? 1 : 0;
    int coop = !coop_off && splits > 1 && !cluster && M > 8 && (long long)grid.x * grid.y * grid.z <= resident &&
               n_counters >= 2 * (int)(grid.x * grid.y);
    TcArgs a{C, scratch, counters, status, M, N, K, ldc, mode, splits, (kblocks + splits - 1) / splits, kblocks, trace, cluster, coop};
#define TC_CASE(BN_)                                                                  \
    case BN_:                                                                         \
        return nacc == 2 ? launch<BN_, 2, false>(mw, mx, a, grid, stream)                  \
                         : a.coop ? launch<BN_, 1, true>(mw, mx, a, grid, stream) : launch<BN_, 1, false>(mw, mx, a, grid, stream);
    switch (bn) {
        TC_CASE(16)
        TC_CASE(32)
        TC_CASE(64)
        TC_CASE(128)
        TC_CASE(256)
    }
#undef TC_CASE
    return ce_fail(CE_ERR_SIZE, "ce_gemm_tc: no tile for M=%d", M);
}
