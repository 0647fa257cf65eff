// Causal flash attention for portions of prompts on the 5th-generation tensor cores: S = Q K^T and
// O += P V are tcgen05.mma instructions with accumulators in tensor memory; Q, K and V tiles come
// into shared memory by TMA straight out of the paged cache (no cluster multicast); the softmax runs
// in float32 with one thread per query row.
//
// One block per (tile of 128 new tokens of one sequence, query head).  Warp 0 issues the TMA loads
// (two stages of 64 keys), warp 1 owns tensor memory and issues the MMAs, warps 2-5 hold one query
// row each: they read the row's 64 scores from tensor memory, apply the causal and window limits,
// keep the running maximum and sum, write the probabilities as bfloat16 into a swizzled shared tile
// (the A operand of the PV product) and rescale the output accumulator when a row's maximum moved.
// V is used as stored, [keys, head_dim]: the B operand of the PV product is MN-major.
// Rows of V past the sequence's last key are zeroed in shared memory before they are multiplied,
// so a probability of zero never meets whatever lies in the unused part of a page.
//
// Every wait on an mbarrier is bounded; on a timeout the block sets a status of 61 to 68 (which wait
// gave up), waits (bounded) for
// its own copies in flight, frees its tensor memory and returns.
//
// Takes head sizes 64 and 128 and power-of-two page sizes; everything else goes to the mma.sync
// kernel of attention_mma.cu.  (The reference's counterpart is flash_prefill_tc,
// src/kernels/attention_tc.cu:180-565, on mma.sync m16n8k16.)
#include "common.cuh"
#include "tensor_map.h"
#include <mutex>
#include <unordered_map>

namespace {

constexpr int BM = 128;            // queries per block = UMMA M
constexpr int BN = 64;             // keys per iteration
constexpr int THREADS = 192;
constexpr int STAGES = 2;
constexpr uint32_t SPIN_LIMIT = 1u << 16;    // a tile takes microseconds; this is tens of milliseconds

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count));
}
__device__ __forceinline__ void mbar_expect_tx(uint64_t* bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint64_t* bar, uint32_t parity) {
    uint32_t ok;
    asm volatile("{\n.reg .pred p;\nmbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2;\nselp.u32 %0, 1, 0, p;\n}"
                 : "=r"(ok) : "r"(smem_u32(bar)), "r"(parity) : "memory");
    return ok != 0;
}
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
// Shared-memory operand descriptors, 128-byte swizzle.  K-major: rows of 128 bytes along K, 8-row
// groups 1024 bytes apart.  MN-major: rows of 128 bytes along MN (64 elements), one row per k,
// 8-row groups `sbo` apart, the next 64 MN elements `lbo` apart.
__device__ __forceinline__ uint64_t desc_kmajor(uint32_t addr) {
    return (uint64_t)((addr & 0x3FFFF) >> 4) | ((uint64_t)1 << 16) | ((uint64_t)(1024 >> 4) << 32) | ((uint64_t)1 << 46) |
           ((uint64_t)2 << 61);
}
__device__ __forceinline__ uint64_t desc_mnmajor(uint32_t addr, uint32_t lbo, uint32_t sbo) {
    return (uint64_t)((addr & 0x3FFFF) >> 4) | ((uint64_t)(lbo >> 4) << 16) | ((uint64_t)(sbo >> 4) << 32) | ((uint64_t)1 << 46) |
           ((uint64_t)2 << 61);
}
__device__ __forceinline__ void umma(uint32_t d_tmem, uint64_t a, uint64_t b, uint32_t idesc, uint32_t acc) {
    asm volatile("{\n.reg .pred p;\nsetp.ne.b32 p, %4, 0;\ntcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n}"
                 ::"r"(d_tmem), "l"(a), "l"(b), "r"(idesc), "r"(acc) : "memory");
}
__device__ __forceinline__ void umma_commit(uint64_t* bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar)) : "memory");
}
// 64 columns of this thread's lane: two loads in flight, one wait
__device__ __forceinline__ void tmem_ld64(uint32_t taddr, float (&v)[64]) {
    uint32_t r[64];
#pragma unroll
    for (int h = 0; h < 2; ++h) {
        uint32_t* q = r + 32 * h;
        asm volatile("tcgen05.ld.sync.aligned.32x32b.x32.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,"
                     "%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31}, [%32];"
                     : "=r"(q[0]), "=r"(q[1]), "=r"(q[2]), "=r"(q[3]), "=r"(q[4]), "=r"(q[5]), "=r"(q[6]), "=r"(q[7]),
                       "=r"(q[8]), "=r"(q[9]), "=r"(q[10]), "=r"(q[11]), "=r"(q[12]), "=r"(q[13]), "=r"(q[14]), "=r"(q[15]),
                       "=r"(q[16]), "=r"(q[17]), "=r"(q[18]), "=r"(q[19]), "=r"(q[20]), "=r"(q[21]), "=r"(q[22]), "=r"(q[23]),
                       "=r"(q[24]), "=r"(q[25]), "=r"(q[26]), "=r"(q[27]), "=r"(q[28]), "=r"(q[29]), "=r"(q[30]), "=r"(q[31])
                     : "r"(taddr + 32 * h));
    }
    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
    for (int i = 0; i < 64; ++i) v[i] = __uint_as_float(r[i]);
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
__device__ __forceinline__ void tmem_st32(uint32_t taddr, const float (&v)[32]) {
    asm volatile("tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,"
                 "%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31,%32};"
                 ::"r"(taddr), "r"(__float_as_uint(v[0])), "r"(__float_as_uint(v[1])), "r"(__float_as_uint(v[2])),
                   "r"(__float_as_uint(v[3])), "r"(__float_as_uint(v[4])), "r"(__float_as_uint(v[5])), "r"(__float_as_uint(v[6])),
                   "r"(__float_as_uint(v[7])), "r"(__float_as_uint(v[8])), "r"(__float_as_uint(v[9])), "r"(__float_as_uint(v[10])),
                   "r"(__float_as_uint(v[11])), "r"(__float_as_uint(v[12])), "r"(__float_as_uint(v[13])), "r"(__float_as_uint(v[14])),
                   "r"(__float_as_uint(v[15])), "r"(__float_as_uint(v[16])), "r"(__float_as_uint(v[17])), "r"(__float_as_uint(v[18])),
                   "r"(__float_as_uint(v[19])), "r"(__float_as_uint(v[20])), "r"(__float_as_uint(v[21])), "r"(__float_as_uint(v[22])),
                   "r"(__float_as_uint(v[23])), "r"(__float_as_uint(v[24])), "r"(__float_as_uint(v[25])), "r"(__float_as_uint(v[26])),
                   "r"(__float_as_uint(v[27])), "r"(__float_as_uint(v[28])), "r"(__float_as_uint(v[29])), "r"(__float_as_uint(v[30])),
                   "r"(__float_as_uint(v[31]))
                 : "memory");
}
// A softmax warp's wait: lane 0 polls (bounded), the warp takes its verdict.  The four warps are not lined
// up with one another here (a block-wide vote at every wait cost about a third of a tile's time): each
// arrives on s_free and p_full by itself.  If one warp gives up, it stops arriving, the MMA thread's next
// wait runs out, and so do the other warps' waits; every loop ends, only later.
__device__ __forceinline__ bool warp_wait(uint64_t* bar, uint32_t parity) {
    int lane = threadIdx.x & 31;
    uint32_t ok = lane == 0 ? (mbar_wait(bar, parity) ? 1u : 0u) : 1u;
    return __shfl_sync(0xffffffffu, ok, 0) != 0;
}
__device__ __forceinline__ uint32_t pack2(float lo, float hi) {
    __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&v);
}

struct TcAttnArgs {
    __nv_bfloat16* out;         // [T, nh*d]
    const int* seq_slot;        // [B]
    const int* q_start;         // [B+1]
    const int* ctx_len;         // [B]
    const int* block_table;     // [slots, max_pages]
    const int* tiles;           // [n_tiles, 2] = (sequence, first new token of the tile), 128 tokens a tile
    int* status;
    int nh, nkv, page_size, page_shift, max_pages, num_pages, window;
    float scale_log2;
};

template <int D>
__global__ void __launch_bounds__(THREADS) attention_prefill_tc_kernel(const __grid_constant__ CUtensorMap map_q,
                                                                      const __grid_constant__ CUtensorMap map_k,
                                                                      const __grid_constant__ CUtensorMap map_v, TcAttnArgs a) {
    extern __shared__ __align__(1024) unsigned char smem_raw[];

    constexpr int HALVES = D / 64;                        // 64-column boxes per row of D
    constexpr uint32_t Q_BYTES = BM * D * 2, K_BYTES = BN * D * 2, P_BYTES = BM * BN * 2;
    constexpr uint32_t Q_HALF = BM * 128, K_HALF = BN * 128;
    constexpr uint32_t STAGE_BYTES = 2 * K_BYTES;          // K then V
    constexpr uint32_t TMEM_COLS = 256;                    // S: 64 columns at 0; O: D columns at 64
    // No static shared memory and no alignment slack: the tiles start at the block's first shared byte
    // (checked below to be 1024-aligned, as the swizzle needs), the barriers follow the tiles; two
    // blocks then fit one SM.
    uint32_t base = smem_u32(smem_raw);
    unsigned char* sm = smem_raw;
    uint32_t q_addr = base, kv_addr = base + Q_BYTES, p_addr = kv_addr + STAGES * STAGE_BYTES;
    uint64_t* bars = reinterpret_cast<uint64_t*>(sm + Q_BYTES + STAGES * STAGE_BYTES + P_BYTES);
    // K and V have rings of their own: K(j) is free again as soon as S(j) is complete, long before V(j),
    // so the copy of K(j+2) starts two softmax periods before S(j+2) needs it
    uint64_t& q_full = bars[0];
    uint64_t* k_full = bars + 1;
    uint64_t* k_empty = bars + 1 + STAGES;
    uint64_t* v_full = bars + 1 + 2 * STAGES;
    uint64_t* v_empty = bars + 1 + 3 * STAGES;
    uint64_t& s_full = bars[1 + 4 * STAGES];
    uint64_t& s_free = bars[2 + 4 * STAGES];
    uint64_t& p_full = bars[3 + 4 * STAGES];
    uint64_t& pv_done = bars[4 + 4 * STAGES];
    uint32_t& tmem_slot = *reinterpret_cast<uint32_t*>(bars + 5 + 4 * STAGES);
    int& s_abort = *reinterpret_cast<int*>(bars + 6 + 4 * STAGES);
    if (base & 1023u) {                       // cannot happen with dynamic shared memory alone; refuse rather than mis-swizzle
        if (threadIdx.x == 0) atomicCAS(a.status, 0, 69);
        return;
    }

    int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    // grid (heads, tiles), tiles taken from the last: under a causal mask a sequence's later tiles have more
    // keys to visit, so the long blocks start first and the short ones fill the end of the launch
    int tile_idx = (int)(gridDim.y - 1 - blockIdx.y);
    int b = a.tiles[2 * tile_idx], q0 = a.tiles[2 * tile_idx + 1];
    int h = blockIdx.x, kvh = h / (a.nh / a.nkv);
    int t0 = a.q_start[b], q_len = a.q_start[b + 1] - t0;
    int ctx_before = a.ctx_len[b] - q_len;
    int nq = min(BM, q_len - q0);
    int p_first = ctx_before + q0, p_last = p_first + nq - 1;
    int lo_tile = a.window > 0 ? max(0, p_first - a.window + 1) : 0;
    int k_begin = lo_tile / BN * BN;
    int n_kv = (p_last - k_begin) / BN + 1;
    const int* table = a.block_table + (size_t)a.seq_slot[b] * a.max_pages;

    ce_pdl_launch_dependents();
    if (threadIdx.x == 0) {
        mbar_init(&q_full, 1);
        for (int s = 0; s < STAGES; ++s) { mbar_init(&k_full[s], 1); mbar_init(&k_empty[s], 1); mbar_init(&v_full[s], 1); mbar_init(&v_empty[s], 1); }
        mbar_init(&s_full, 1); mbar_init(&s_free, 4); mbar_init(&p_full, 4); mbar_init(&pv_done, 1);   // 4: one arrival per softmax warp
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
    uint32_t tmem_s = tmem, tmem_o = tmem + BN;
    ce_pdl_wait();

    if (warp == 0) {
        if (lane == 0) {
            // ---- producer: Q once, then K and V tiles of 64 keys, page by page
            bool ok = true;
            mbar_expect_tx(&q_full, Q_BYTES);
#pragma unroll
            for (int hf = 0; hf < HALVES; ++hf) tma_load_2d(sm + hf * Q_HALF, &map_q, &q_full, h * D + hf * 64, t0 + q0);
            int box_rows = min(a.page_size, BN);
            // one tile of K or V: pieces of a page, 64 columns a copy
            auto load_tile = [&](const CUtensorMap* map, unsigned char* dst, uint64_t* bar, int j) {
                mbar_expect_tx(bar, K_BYTES);
                int k0 = k_begin + j * BN;
                for (int r = 0; r < BN; r += box_rows) {
                    int key = k0 + r;
                    int page = key <= p_last ? table[key >> a.page_shift] : -1;
                    if (page < 0 || page >= a.num_pages) {        // past the context (or a bad table): any held page will do,
                        if (key <= p_last) atomicExch(a.status, 4);  // its keys are masked and its values zeroed
                        page = 0;
                    }
                    int row = (page * a.nkv + kvh) * a.page_size + (key & (a.page_size - 1));
#pragma unroll
                    for (int hf = 0; hf < HALVES; ++hf) tma_load_2d(dst + hf * K_HALF + r * 128, map, bar, hf * 64, row);
                }
            };
            // order K(0), then for every j: K(j+1), V(j): the keys run one tile ahead of the values
            int k_issued = 0, v_issued = 0;
            for (int j = -1; j < n_kv && ok; ++j) {
                int jk = j + 1;
                if (jk < n_kv) {
                    int s = jk % STAGES;
                    if (jk >= STAGES) ok = mbar_wait(&k_empty[s], ((jk / STAGES) - 1) & 1);
                    if (!ok) break;
                    load_tile(&map_k, sm + Q_BYTES + (size_t)s * STAGE_BYTES, &k_full[s], jk);
                    k_issued = jk + 1;
                }
                if (j >= 0) {
                    int s = j % STAGES;
                    if (j >= STAGES) ok = mbar_wait(&v_empty[s], ((j / STAGES) - 1) & 1);
                    if (!ok) break;
                    load_tile(&map_v, sm + Q_BYTES + (size_t)s * STAGE_BYTES + K_BYTES, &v_full[s], j);
                    v_issued = j + 1;
                }
            }
            if (!ok) {
                atomicCAS(a.status, 0, 61);                    // 61: the producer gave up waiting for a free stage
                atomicExch(&s_abort, 1);
                for (int j = max(0, k_issued - STAGES); j < k_issued; ++j) mbar_wait(&k_full[j % STAGES], (j / STAGES) & 1);
                for (int j = max(0, v_issued - STAGES); j < v_issued; ++j) mbar_wait(&v_full[j % STAGES], (j / STAGES) & 1);
            }
        }
    } else if (warp == 1) {
        if (lane == 0) {
            // ---- MMA issuer: S(j) = Q K(j)^T as soon as S is free; O += P(j-1) V(j-1) as soon as P is there
            uint32_t idesc_s = (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(BN >> 3) << 17) | ((uint32_t)(BM >> 4) << 24);
            uint32_t idesc_pv = (1u << 4) | (1u << 7) | (1u << 10) | (1u << 16) | ((uint32_t)(D >> 3) << 17) | ((uint32_t)(BM >> 4) << 24);
            int where = 62;                                    // 62..65: which wait of the MMA warp gave up
            bool ok = mbar_wait(&q_full, 0);
            for (int j = 0; j <= n_kv && ok; ++j) {
                if (j < n_kv) {
                    int s = j % STAGES;
                    where = 63;
                    ok = mbar_wait(&k_full[s], (j / STAGES) & 1);
                    if (ok && j > 0) { where = 64; ok = mbar_wait(&s_free, (j - 1) & 1); }
                    if (!ok) break;
                    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                    uint32_t k_addr = kv_addr + s * STAGE_BYTES;
#pragma unroll
                    for (int kk = 0; kk < D / 16; ++kk) {
                        uint32_t off = (kk / 4) * Q_HALF + (kk % 4) * 32;
                        uint32_t koff = (kk / 4) * K_HALF + (kk % 4) * 32;
                        umma(tmem_s, desc_kmajor(q_addr + off), desc_kmajor(k_addr + koff), idesc_s, kk > 0 ? 1u : 0u);
                    }
                    umma_commit(&k_empty[s]);           // the stage's K is free once these have read it
                    umma_commit(&s_full);
                }
                if (j > 0) {
                    int jp = j - 1, s = jp % STAGES;
                    where = 65;
                    ok = mbar_wait(&p_full, jp & 1) && mbar_wait(&v_full[s], (jp / STAGES) & 1);
                    if (!ok) break;
                    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                    uint32_t v_addr = kv_addr + s * STAGE_BYTES + K_BYTES;
#pragma unroll
                    for (int kk = 0; kk < BN / 16; ++kk)
                        umma(tmem_o, desc_kmajor(p_addr + kk * 32), desc_mnmajor(v_addr + kk * 16 * 128, K_HALF, 1024), idesc_pv,
                             (jp > 0 || kk > 0) ? 1u : 0u);
                    umma_commit(&v_empty[s]);           // the stage's V is free once these have read it
                    umma_commit(&pv_done);
                }
            }
            if (!ok) { atomicCAS(a.status, 0, where); atomicExch(&s_abort, 1); }
        }
    } else {
        // ---- softmax: one query row per thread
        int quad = warp & 3;
        int row = quad * 32 + lane;
        bool row_valid = row < nq;
        int pos = p_first + row;
        int lo = a.window > 0 ? max(0, pos - a.window + 1) : 0;
        uint32_t lane_base = (uint32_t)(quad * 32) << 16;
        float m_run = -INFINITY, l_run = 0.f;
        bool ok = true;
        int where = 66;                                        // 66..68: which wait of the softmax warps gave up
        for (int j = 0; j < n_kv; ++j) {
            int k0 = k_begin + j * BN;
            where = 66;
            if (!warp_wait(&s_full, j & 1)) { ok = false; break; }
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            float sv[BN];
            tmem_ld64(tmem_s + lane_base, sv);
            asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
            __syncwarp();
            if (lane == 0) mbar_arrive(&s_free);  // (one arrival per warp) S may be overwritten by the next product
            bool full = row_valid && k0 >= lo && k0 + BN - 1 <= pos;
            if (!full) {                          // only tiles on the diagonal, at the window's edge or past the rows
#pragma unroll
                for (int i = 0; i < BN; ++i) {
                    int key = k0 + i;
                    if (!(row_valid && key >= lo && key <= pos)) sv[i] = -INFINITY;
                }
            }
            float mx4[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
#pragma unroll
            for (int i = 0; i < BN; i += 4) {
                mx4[0] = fmaxf(mx4[0], sv[i]); mx4[1] = fmaxf(mx4[1], sv[i + 1]);
                mx4[2] = fmaxf(mx4[2], sv[i + 2]); mx4[3] = fmaxf(mx4[3], sv[i + 3]);
            }
            float mx = fmaxf(fmaxf(mx4[0], mx4[1]), fmaxf(mx4[2], mx4[3]));
            // The running maximum is only a scale: it is raised (and the sums rescaled) when a tile's maximum
            // exceeds it by more than 2^8; below that the probabilities stay within bfloat16's range and the
            // output accumulator is left alone.
            float m_tile = mx * a.scale_log2;
            bool raise = m_tile > m_run + 8.0f || (m_run == -INFINITY && m_tile != -INFINITY);
            float m_new = raise ? m_tile : m_run;
            float m_use = m_new == -INFINITY ? 0.f : m_new;
            float alpha = raise ? ce_exp2_fast(m_run - m_use) : 1.0f;
            float sum = 0.f, sum1 = 0.f;
            uint32_t packed[BN / 2];
#pragma unroll
            for (int i = 0; i < BN; i += 2) {
                float p0 = ce_exp2_fast(fmaf(sv[i], a.scale_log2, -m_use));
                float p1 = ce_exp2_fast(fmaf(sv[i + 1], a.scale_log2, -m_use));
                sum += p0; sum1 += p1;
                packed[i / 2] = pack2(p0, p1);
            }
            sum += sum1;
            l_run = l_run * alpha + sum;
            m_run = m_new;
            // P and (if a scale was raised) O may be touched only after the previous PV product is complete
            if (j > 0) {
                where = 67;
                if (!warp_wait(&pv_done, (j - 1) & 1)) { ok = false; break; }
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                if (__any_sync(0xffffffffu, alpha != 1.0f)) {
#pragma unroll 1
                    for (int c = 0; c < D; c += 32) {
                        float o[32];
                        tmem_ld32(tmem_o + lane_base + c, o);
#pragma unroll
                        for (int i = 0; i < 32; ++i) o[i] *= alpha;
                        tmem_st32(tmem_o + lane_base + c, o);
                    }
                    asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
                }
            }
            // probabilities: row `row` of a [128, 64] K-major tile, 16-byte chunks swizzled by the row
            {
                unsigned char* prow = sm + (p_addr - base) + row * 128;
#pragma unroll
                for (int c = 0; c < 8; ++c) {
                    uint4 v = make_uint4(packed[4 * c], packed[4 * c + 1], packed[4 * c + 2], packed[4 * c + 3]);
                    *reinterpret_cast<uint4*>(prow + ((c ^ (row & 7)) << 4)) = v;
                }
            }
            // the last tile may hold rows of V past the sequence's last key: zero them
            if (k0 + BN - 1 > p_last) {
                int s = j % STAGES;
                mbar_wait(&v_full[s], (j / STAGES) & 1);
                unsigned char* vst = sm + Q_BYTES + (size_t)s * STAGE_BYTES + K_BYTES;
                int first_bad = p_last + 1 - k0;
                for (int e = threadIdx.x - 64; e < (BN - first_bad) * HALVES * 8; e += 128) {
                    int chunk = e & 7, rest = e >> 3;
                    int hf = rest % HALVES, r = first_bad + rest / HALVES;
                    *reinterpret_cast<uint4*>(vst + hf * K_HALF + r * 128 + chunk * 16) = make_uint4(0, 0, 0, 0);
                }
            }
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
            asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
            __syncwarp();
            if (lane == 0) mbar_arrive(&p_full);  // (one arrival per warp) P, and the zeroed rows of V, are in shared memory
        }
        if (ok) {                       // (uniform within a warp: a warp leaves the loop above as one)
            where = 68;
            if (!warp_wait(&pv_done, (n_kv - 1) & 1)) ok = false;
        }
        if (!ok) { atomicCAS(a.status, 0, where); atomicExch(&s_abort, 1); }
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        if (ok) {
            // tensor-memory loads are warp-wide: every lane takes part, only real query rows store
            float inv = l_run > 0.f ? 1.0f / l_run : 0.f;
            __nv_bfloat16* orow = a.out + ((size_t)(t0 + q0 + row) * a.nh + h) * D;
#pragma unroll 1
            for (int c = 0; c < D; c += 32) {
                float o[32];
                tmem_ld32(tmem_o + lane_base + c, o);
                if (row_valid) {
#pragma unroll
                    for (int i = 0; i < 32; i += 8) {
                        uint4 v = make_uint4(pack2(o[i] * inv, o[i + 1] * inv), pack2(o[i + 2] * inv, o[i + 3] * inv),
                                             pack2(o[i + 4] * inv, o[i + 5] * inv), pack2(o[i + 6] * inv, o[i + 7] * inv));
                        *reinterpret_cast<uint4*>(orow + c + i) = v;
                    }
                }
            }
        }
        asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    }
    __syncthreads();
    if (warp == 1) {
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(TMEM_COLS));
    }
}

// ---- host side ------------------------------------------------------------------------------------
// bf16 matrix [rows, cols], row stride ld elements, boxes of box_rows x 64 columns, 128-byte swizzle
int get_map(const void* ptr, long long rows, long long cols, long long ld, int box_rows, CUtensorMap* out) {
    return ce_tensor_map_bf16(ptr, rows, cols, ld, box_rows, out, "ce_attention_prefill_tc");
}

template <int D>
int launch(const CUtensorMap& mq, const CUtensorMap& mk, const CUtensorMap& mv, const TcAttnArgs& a, dim3 grid, cudaStream_t stream) {
    size_t smem = (size_t)BM * D * 2 + STAGES * 2 * BN * D * 2 + BM * BN * 2 + 192;    // tiles + barriers
    static bool attr_set = false;
    if (!attr_set) {
        cudaError_t e = cudaFuncSetAttribute(attention_prefill_tc_kernel<D>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return ce_fail(CE_ERR_CUDA, "ce_attention_prefill_tc: %s", cudaGetErrorString(e));
        attr_set = true;
    }
    { ce_note("attention_prefill_tc_kernel"); ce_launch(attention_prefill_tc_kernel<D>, grid, THREADS, smem, stream, mq, mk, mv, a); }
    return ce_check_launch("ce_attention_prefill_tc");
}

}  // namespace

extern "C" int ce_attention_prefill_tc_supported(int d, int page_size, int q_stride) {
    return (d == 64 || d == 128) && page_size >= 8 && (page_size & (page_size - 1)) == 0 && q_stride % 8 == 0;
}

// tiles: [n_tiles, 2] = (sequence, first new token of the tile), 128 tokens a tile, over the
// sequences that bring more than one token.  total_tokens: rows of q.
extern "C" int ce_attention_prefill_tc(const void* q, const void* k_pool, const void* v_pool, void* out, const int* seq_slot,
                                       const int* q_start, const int* ctx_len, const int* block_table, const int* tiles,
                                       int* status, int n_tiles, int total_tokens, int nh, int nkv, int d, int q_stride,
                                       int page_size, int max_pages, int num_pages, int window, float scale,
                                       cudaStream_t stream) {
    if (n_tiles == 0) return CE_OK;
    if (!q || !k_pool || !v_pool || !out || !seq_slot || !q_start || !ctx_len || !block_table || !tiles || !status)
        return ce_fail(CE_ERR_ARG, "ce_attention_prefill_tc: null pointer");
    if (!ce_attention_prefill_tc_supported(d, page_size, q_stride))
        return ce_fail(CE_ERR_SIZE, "ce_attention_prefill_tc: head_dim %d (64 or 128), page size %d (a power of two >= 8)", d, page_size);
    if (nkv <= 0 || nh % nkv) return ce_fail(CE_ERR_SIZE, "ce_attention_prefill_tc: %d heads, %d kv heads", nh, nkv);
    if (((uintptr_t)q | (uintptr_t)k_pool | (uintptr_t)v_pool | (uintptr_t)out) & 15)
        return ce_fail(CE_ERR_SIZE, "ce_attention_prefill_tc: operands must be 16-byte aligned");
    CUtensorMap mq, mk, mv;
    int rc = get_map(q, total_tokens, (long long)nh * d, q_stride, BM, &mq);
    if (rc) return rc;
    long long pool_rows = (long long)num_pages * nkv * page_size;
    int box_rows = page_size < BN ? page_size : BN;
    if ((rc = get_map(k_pool, pool_rows, d, d, box_rows, &mk))) return rc;
    if ((rc = get_map(v_pool, pool_rows, d, d, box_rows, &mv))) return rc;
    int shift = 0;
    while ((1 << shift) < page_size) ++shift;
    TcAttnArgs a{(__nv_bfloat16*)out, seq_slot, q_start, ctx_len, block_table, tiles, status, nh, nkv, page_size, shift,
                 max_pages, num_pages, window, scale * 1.4426950408889634f};
    if (n_tiles > 65535) return ce_fail(CE_ERR_SIZE, "ce_attention_prefill_tc: %d tiles of 128 tokens in one step", n_tiles);
    dim3 grid(nh, n_tiles);
    return d == 64 ? launch<64>(mq, mk, mv, a, grid, stream) : launch<128>(mq, mk, mv, a, grid, stream);
}
