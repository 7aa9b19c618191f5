// Shared helpers of the sm_100a kernel library. Every exported function is
// extern "C", takes raw device pointers and a CUDA stream, launches on that
// stream and returns a cudaError_t as int (0 = launched). Arguments are
// validated on the host before a launch: a size the kernel cannot take is
// refused with LUMEN_ERR_UNSUPPORTED, never computed wrongly.
#pragma once
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#define LUMEN_API extern "C" __attribute__((visibility("default")))

// Error codes above the CUDA range, understood by the Python loader.
#define LUMEN_ERR_UNSUPPORTED 100001
#define LUMEN_ERR_BAD_ARGUMENT 100002

// Tokens per page of the paged key/value cache. A page holds, for one cache
// entry (one run of a layer), [n_kv][LUMEN_PAGE][head_dim] keys (and the same
// for values), so one (page, kv head) tile is contiguous.
#define LUMEN_PAGE 64

// Layouts of a (page, kv head) tile of the cache, LUMEN_PAGE keys x d values.
//   LUMEN_LAYOUT_LINEAR: [key][d].
//   LUMEN_LAYOUT_SW128 (2-byte elements, d a multiple of 64): [d/64][key][64], every
//     row 128 bytes, and the 16-byte chunk c of row `key` stored at chunk c ^ (key & 7).
//     This is the 128-byte-swizzled K-major tile that ldmatrix reads without bank
//     conflicts and that a tensor-core descriptor (SWIZZLE_128B) addresses directly, so
//     a plain bulk copy of the tile is all a kernel needs to stage it.
#define LUMEN_LAYOUT_LINEAR 0
#define LUMEN_LAYOUT_SW128 1

// Offset, in elements, of value e of key r inside its tile.
__host__ __device__ __forceinline__ int tile_offset(int layout, int r, int e, int d) {
    if (layout == LUMEN_LAYOUT_SW128) {
        const int cb = e >> 6, ce = e & 63;
        return cb * (LUMEN_PAGE * 64) + r * 64 + ((((ce >> 3) ^ (r & 7)) << 3) | (ce & 7));
    }
    return r * d + e;
}

// Programmatic dependent launch. Every kernel of this library calls pdl_wait() before it reads
// or writes global memory that another kernel may touch (only set-up that depends on nothing,
// and reads of weights and of cache pages written by earlier steps, may come first), and lets
// the next kernel in the stream start with pdl_trigger(): the short kernels (norms, rotary,
// SiLU, embedding) at their very top, the attention kernels after their wait, the
// weight-streaming product when its last loads are about to be asked for (csrc/gemm_tc.cu,
// TC_TRIGGER_AHEAD). A kernel that was started early still waits for the kernel before it,
// which waited for the one before that, so the order of the stream holds for everything behind
// the waits. Launched through lumen_launch with the attribute set, a kernel's set-up and first
// weight loads run under the tail of the kernels before; launched without it, both
// instructions do nothing. It is on (3.30 ms a decode step at batch 8 of the 8B shape against
// 3.55 with every trigger right behind the wait, and 3.8 without); lumen_set_pdl(0) turns it off
// for the module it is called in, which the kernel micro-benchmarks do on request.
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void pdl_trigger() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

#ifdef __CUDACC__
#include <utility>
static int g_lumen_pdl = 1;
static inline bool lumen_pdl_enabled() { return g_lumen_pdl != 0; }
// Measurement switch of this module (every module is one translation unit and has its own).
LUMEN_API void lumen_set_pdl(int on) { g_lumen_pdl = on ? 1 : 0; }
template <typename... KArgs, typename... Args>
static inline cudaError_t lumen_launch(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem,
                                       cudaStream_t stream, Args&&... args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = lumen_pdl_enabled() ? 1 : 0;
    return cudaLaunchKernelEx(&cfg, kernel, std::forward<Args>(args)...);
}
#endif

#define LUMEN_LAUNCH_CHECK()                         \
    do {                                             \
        cudaError_t e__ = cudaGetLastError();        \
        if (e__ != cudaSuccess) return (int)e__;     \
    } while (0)

__device__ __forceinline__ float to_f32(float x) { return x; }
__device__ __forceinline__ float to_f32(__nv_bfloat16 x) { return __bfloat162float(x); }

template <typename T> __device__ __forceinline__ T from_f32(float x);
template <> __device__ __forceinline__ float from_f32<float>(float x) { return x; }
template <> __device__ __forceinline__ __nv_bfloat16 from_f32<__nv_bfloat16>(float x) {
    return __float2bfloat16_rn(x);
}

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
    return v;
}

// Block-wide sum with a fixed order (warp butterflies, then warp 0 over the
// per-warp partials), so the result depends only on the block size.
// `red` must hold 32 floats. All threads get the result.
__device__ __forceinline__ float block_sum(float v, float* red) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int nwarp = (blockDim.x + 31) >> 5;
    v = warp_sum(v);
    __syncthreads();
    if (lane == 0) red[warp] = v;
    __syncthreads();
    float t = (lane < nwarp) ? red[lane] : 0.0f;
    t = warp_sum(t);
    return t;
}
__device__ __forceinline__ float block_max(float v, float* red) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int nwarp = (blockDim.x + 31) >> 5;
    v = warp_max(v);
    __syncthreads();
    if (lane == 0) red[warp] = v;
    __syncthreads();
    float t = (lane < nwarp) ? red[lane] : -INFINITY;
    t = warp_max(t);
    return t;
}
