// Runs CUDA kernel sources of pedrosoares/carbon-engine on the CPU, so that their output can anchor the plain
// implementation of tests/plain_qwen3.py.  The reference's model code is Rust on a tensor library and
// cannot be built where these tests run; four of its kernel files are plain CUDA C and can, once the
// CUDA keywords are defined away and every lane of a block is run as a host thread:
//
//   src/kernels/attention.cu   paged_decode_f32, flash_prefill_f32   (attention semantics: slot tables,
//                              the causal offset kv_len - q_len, grouped heads, the scale)
//   src/kernels/sampling.cu    carbon_uniform                        (the sampler's counter-based uniforms)
//   src/kernels/qsa.cu         qsa_select_f32                        (its scratch scores expose an RMSNorm
//                              with a weight, followed by the rotate-half rotation over the first 2*HALF
//                              dimensions: src/kernels/qsa.cu:98-116)
//
// Build (tests/golden/make_reference_vectors.py does it):
//   g++ -std=c++20 -O2 -pthread -I <reference>/src/kernels reference_kernels_host.cpp -o ref_host
// Use:  ref_host decode|prefill|uniform|qsa IN OUT     (IN/OUT: records of int32 count + 4-byte values)
#include <algorithm>
#include <atomic>
#include <barrier>
#include <cmath>
#include <cstdint>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <functional>
#include <memory>
#include <string>
#include <thread>
#include <vector>

// ---- what the kernel sources expect of CUDA ---------------------------------------------------------
struct Index3 { unsigned x = 0, y = 0, z = 0; };
static thread_local Index3 threadIdx, blockIdx;
static Index3 blockDim, gridDim;

namespace lanes {
// one barrier per block, one per warp, and a 32-slot exchange buffer per warp for the shuffles
static std::barrier<>* block_barrier = nullptr;
static thread_local std::barrier<>* warp_barrier = nullptr;
static thread_local float* warp_exchange = nullptr;
}  // namespace lanes

#define CARBON_HOST_TEST
#define __device__
#define __global__
#define __forceinline__ inline
#define __restrict__
#define __shared__ static          // blocks run one after another, so one static copy is the block's shared memory
#define __expf(x) expf(x)
#ifndef INFINITY
#define INFINITY (__builtin_inff())
#endif
using std::min;
using std::max;

static inline float __int_as_float(int i) { float f; std::memcpy(&f, &i, sizeof f); return f; }
static inline int __float_as_int(float f) { int i; std::memcpy(&i, &f, sizeof i); return i; }
static inline float rsqrtf(float x) { return 1.0f / std::sqrt(x); }
static inline void __syncthreads() { lanes::block_barrier->arrive_and_wait(); }
static inline void __syncwarp() { lanes::warp_barrier->arrive_and_wait(); }
static inline unsigned atomicAdd(unsigned* p, unsigned v) { return std::atomic_ref<unsigned>(*p).fetch_add(v); }
static inline int atomicAdd(int* p, int v) { return std::atomic_ref<int>(*p).fetch_add(v); }
static inline unsigned atomicOr(unsigned* p, unsigned v) { return std::atomic_ref<unsigned>(*p).fetch_or(v); }

// a shuffle: every lane of the warp posts its value, waits, reads another lane's, waits again
static inline float exchange(float v, unsigned from) {
    lanes::warp_exchange[threadIdx.x & 31u] = v;
    lanes::warp_barrier->arrive_and_wait();
    float got = lanes::warp_exchange[from & 31u];
    lanes::warp_barrier->arrive_and_wait();
    return got;
}
static inline float __shfl_xor_sync(unsigned, float v, int lane_mask) { return exchange(v, (threadIdx.x & 31u) ^ (unsigned)lane_mask); }
static inline float __shfl_sync(unsigned, float v, int src) { return exchange(v, (unsigned)src); }

#include "attention.cu"
#include "sampling.cu"
// qsa.cu takes its element types from another file of the reference; attention.cu's have the same interface
typedef AF32 F32;
typedef ABF16 BF16;
typedef AF16 F16;
#include "qsa.cu"

// ---- running a grid: blocks in turn, a host thread per CUDA thread --------------------------------------
static void run_grid(unsigned grid, unsigned block, const std::function<void()>& body) {
    blockDim.x = block;
    gridDim.x = grid;
    const unsigned warps = (block + 31) / 32;
    for (unsigned b = 0; b < grid; ++b) {
        std::barrier<> whole(block);
        lanes::block_barrier = &whole;
        std::vector<std::unique_ptr<std::barrier<>>> per_warp;
        std::vector<std::vector<float>> slots(warps, std::vector<float>(32, 0.0f));
        for (unsigned w = 0; w < warps; ++w) {
            unsigned members = std::min(32u, block - 32 * w);
            per_warp.push_back(std::make_unique<std::barrier<>>(members));
        }
        std::vector<std::thread> threads;
        threads.reserve(block);
        for (unsigned t = 0; t < block; ++t)
            threads.emplace_back([&, t, b] {
                threadIdx.x = t;
                blockIdx.x = b;
                lanes::warp_barrier = per_warp[t / 32].get();
                lanes::warp_exchange = slots[t / 32].data();
                body();
            });
        for (auto& th : threads) th.join();
    }
}

// ---- records: int32 count, then that many 4-byte values -----------------------------------------------
struct Reader {
    FILE* f;
    explicit Reader(const char* path) : f(fopen(path, "rb")) { if (!f) { perror(path); exit(2); } }
    template <class T> std::vector<T> next() {
        static_assert(sizeof(T) == 4);
        int32_t n = 0;
        if (fread(&n, 4, 1, f) != 1 || n < 0) { fprintf(stderr, "short input\n"); exit(2); }
        std::vector<T> v((size_t)n);
        if (n && fread(v.data(), 4, (size_t)n, f) != (size_t)n) { fprintf(stderr, "short input\n"); exit(2); }
        return v;
    }
    int scalar() { return next<int32_t>().at(0); }
    float real() { return next<float>().at(0); }
};
template <class T> static void put(FILE* f, const std::vector<T>& v) {
    int32_t n = (int32_t)v.size();
    fwrite(&n, 4, 1, f);
    if (n) fwrite(v.data(), 4, v.size(), f);
}

int main(int argc, char** argv) {
    if (argc != 4) { fprintf(stderr, "use: %s decode|prefill|uniform|qsa IN OUT\n", argv[0]); return 2; }
    std::string what = argv[1];
    Reader in(argv[2]);
    FILE* out = fopen(argv[3], "wb");
    if (!out) { perror(argv[3]); return 2; }
    if (what == "decode") {
        // B, H, KVH, D, scale, q [B,H,D], k and v [S,KVH,D], slots, starts [B+1]
        int B = in.scalar(), H = in.scalar(), KVH = in.scalar(), D = in.scalar();
        float scale = in.real();
        auto q = in.next<float>(), k = in.next<float>(), v = in.next<float>();
        auto slots = in.next<unsigned>(), starts = in.next<unsigned>();
        std::vector<float> o((size_t)B * H * D, NAN);
        run_grid((unsigned)(B * H), 32 * ATT_WARPS, [&] {
            paged_decode_f32(q.data(), k.data(), v.data(), slots.data(), starts.data(), o.data(), H, KVH, D, scale);
        });
        put(out, o);
    } else if (what == "prefill") {
        // T, H, KVH, D, scale, q [T,H,D], k and v [S,KVH,D], slots, seqinfo [B,4], tiles [n,2]
        int T = in.scalar(), H = in.scalar(), KVH = in.scalar(), D = in.scalar();
        float scale = in.real();
        auto q = in.next<float>(), k = in.next<float>(), v = in.next<float>();
        auto slots = in.next<unsigned>(), seqinfo = in.next<unsigned>(), tiles = in.next<unsigned>();
        std::vector<float> o((size_t)T * H * D, NAN);
        unsigned n_tiles = (unsigned)(tiles.size() / 2);
        run_grid(n_tiles * (unsigned)H * FP_SUB, 32 * ATT_WARPS, [&] {
            flash_prefill_f32(q.data(), k.data(), v.data(), slots.data(), seqinfo.data(), tiles.data(), o.data(), H, KVH, D, scale);
        });
        put(out, o);
    } else if (what == "uniform") {
        // pairs (seed lo, seed hi), then indices lo/hi the same way
        auto seeds = in.next<unsigned>(), idx = in.next<unsigned>();
        std::vector<float> u;
        for (size_t s = 0; s + 1 < seeds.size(); s += 2)
            for (size_t i = 0; i + 1 < idx.size(); i += 2)
                u.push_back(carbon_uniform(((unsigned long long)seeds[s + 1] << 32) | seeds[s],
                                           ((unsigned long long)idx[i + 1] << 32) | idx[i]));
        put(out, u);
    } else if (what == "qsa") {
        // B, NH, Dm, HALF, K, R, MAXNB, eps, q [B,NH,Dm], pool [slots,Dm], knorm [Dm], cos and sin [P,HALF], slots, starts
        int B = in.scalar(), NH = in.scalar(), Dm = in.scalar(), HALF = in.scalar(), K = in.scalar(), R = in.scalar(),
            MAXNB = in.scalar();
        float eps = in.real();
        auto q = in.next<float>(), pool = in.next<float>(), knorm = in.next<float>(), c = in.next<float>(), s = in.next<float>();
        auto slots = in.next<unsigned>(), starts = in.next<unsigned>();
        std::vector<float> scores((size_t)B * MAXNB, NAN);
        std::vector<unsigned> out_slots((size_t)B * (K + 1) * R + 16, 0u), out_starts((size_t)B + 1, 0u);
        run_grid((unsigned)B, QSA_THREADS, [&] {
            qsa_select_f32(q.data(), pool.data(), knorm.data(), c.data(), s.data(), slots.data(), starts.data(), scores.data(),
                           out_slots.data(), out_starts.data(), NH, Dm, HALF, K, R, MAXNB, eps);
        });
        put(out, scores);
        put(out, out_slots);
        put(out, out_starts);
    } else {
        fprintf(stderr, "unknown mode %s\n", what.c_str());
        return 2;
    }
    fclose(out);
    return 0;
}
