// Shared declarations of the engine's CUDA kernels (sm_100a).
//
// Every launcher is an extern "C" function that takes raw device pointers and a stream, checks
// the sizes it is given, and returns 0 or a negative code after storing a message that
// ce_last_error() returns.  A launcher never allocates memory and never synchronises.
#pragma once
#include <cuda_runtime.h>
#include <cuda_bf16.h>
#include <stdint.h>

#define CE_OK 0
#define CE_ERR_SIZE -1      // a size this kernel refuses
#define CE_ERR_CUDA -2      // the launch itself failed
#define CE_ERR_ARG -3       // a null pointer or an unknown dtype

// dtype codes shared with the Python side
#define CE_F32 0
#define CE_BF16 1

#include <utility>

extern "C" const char* ce_last_error();
// Programmatic dependent launch: a kernel launched through ce_launch() may be scheduled while the
// kernel before it in the stream still runs.  Every kernel therefore begins with ce_pdl_begin():
// it lets its own dependents be scheduled early, and then waits until all grids before it are
// complete and their memory is visible, before it touches anything they wrote or still read.
// (Both instructions do nothing in a kernel launched the ordinary way.)
bool ce_pdl_enabled();
__device__ __forceinline__ void ce_pdl_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }
__device__ __forceinline__ void ce_pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void ce_pdl_begin() { ce_pdl_launch_dependents(); ce_pdl_wait(); }

template <typename... KArgs, typename... Args>
inline cudaError_t ce_launch(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream, Args&&... args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = ce_pdl_enabled() ? 1 : 0;
    return cudaLaunchKernelEx(&cfg, kernel, std::forward<Args>(args)...);
}
int ce_fail(int code, const char* fmt, ...);
// Counts a launch under the kernel's name (ce_kernel_counts() lists them), so that a test or a
// measurement can see WHICH kernel took a shape.  Called by the launchers once per launch.
void ce_note(const char* kernel_name);
int ce_check_launch(const char* what);
int ce_sm_count();

// 2^x in one MUFU instruction (relative error about 2^-22; -inf gives 0).  exp2f() costs several
// instructions around the same MUFU; the bfloat16 attention kernels, whose probabilities are rounded to
// 8 bits of mantissa anyway, are bound by exactly those instructions.
__device__ __forceinline__ float ce_exp2_fast(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}

template <typename T> struct CeType;
template <> struct CeType<float> {
    static __device__ __forceinline__ float load(const float* p) { return *p; }
    static __device__ __forceinline__ void store(float* p, float v) { *p = v; }
};
template <> struct CeType<__nv_bfloat16> {
    static __device__ __forceinline__ float load(const __nv_bfloat16* p) { return __bfloat162float(*p); }
    static __device__ __forceinline__ void store(__nv_bfloat16* p, float v) { *p = __float2bfloat16_rn(v); }
};

// Sum over a block in a fixed order: warp shuffles down, then warp 0 adds the warp sums in index
// order.  The result depends on blockDim only, never on the grid or on other rows.
__device__ __forceinline__ float ce_block_sum(float v, float* scratch /* >= 32 floats */) {
    for (int o = 16; o > 0; o >>= 1) v += __shfl_down_sync(0xffffffffu, v, o);
    int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarp = (blockDim.x + 31) >> 5;
    __syncthreads();
    if (lane == 0) scratch[warp] = v;
    __syncthreads();
    float total = 0.f;
    for (int w = 0; w < nwarp; ++w) total += scratch[w];
    return total;
}

__device__ __forceinline__ float ce_block_max(float v, float* scratch) {
    for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_down_sync(0xffffffffu, v, o));
    int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarp = (blockDim.x + 31) >> 5;
    __syncthreads();
    if (lane == 0) scratch[warp] = v;
    __syncthreads();
    float m = scratch[0];
    for (int w = 1; w < nwarp; ++w) m = fmaxf(m, scratch[w]);
    return m;
}
