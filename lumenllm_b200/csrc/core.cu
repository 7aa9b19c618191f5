// Memory-bound parts of a decoder step: embedding gather, residual add + RMSNorm,
// SiLU(gate)*up, the table of rotation angles, and the fused per-head RMSNorm + rotary
// encoding + cache write. All arithmetic is float32; the output type T is float (32-bit
// path) or __nv_bfloat16. Compiled without fast-math: sqrtf, expf and sincosf are the
// precise forms. Rows whose length is a multiple of 4 move as 16-byte vectors.
//
// Inputs that come from a split matrix product arrive as S partial results [S, rows, width];
// they are added in rising order of S while they are read.
#include <cooperative_groups.h>
#include "common.cuh"
#include "qk_head.cuh"

template <typename T> struct Pack4;
template <> struct Pack4<float> {
    static __device__ __forceinline__ void store(float* p, float a, float b, float c, float d) {
        *reinterpret_cast<float4*>(p) = make_float4(a, b, c, d);
    }
};
template <> struct Pack4<__nv_bfloat16> {
    static __device__ __forceinline__ void store(__nv_bfloat16* p, float a, float b, float c, float d) {
        __nv_bfloat162 lo = __floats2bfloat162_rn(a, b), hi = __floats2bfloat162_rn(c, d);
        uint2 v;
        v.x = *reinterpret_cast<uint32_t*>(&lo);
        v.y = *reinterpret_cast<uint32_t*>(&hi);
        *reinterpret_cast<uint2*>(p) = v;
    }
};
__device__ __forceinline__ float4 load4(const float* p) { return *reinterpret_cast<const float4*>(p); }
__device__ __forceinline__ float4 load4(const __nv_bfloat16* p) {
    const uint2 v = *reinterpret_cast<const uint2*>(p);
    const __nv_bfloat162 lo = *reinterpret_cast<const __nv_bfloat162*>(&v.x);
    const __nv_bfloat162 hi = *reinterpret_cast<const __nv_bfloat162*>(&v.y);
    return make_float4(__low2float(lo), __high2float(lo), __low2float(hi), __high2float(hi));
}

// ---------------------------------------------------------------- embedding
// h[t, :] = float(E[token[t], :]); a token outside the table writes zeros (the host has
// refused it before; this is the second guard).
template <typename TW>
__global__ void embed_kernel(const int* __restrict__ tokens, const TW* __restrict__ table,
                             float* __restrict__ h, int H, int V) {
    pdl_trigger();
    pdl_wait();      // nothing of this kernel touches global memory before this
    const int t = blockIdx.x;
    const int tok = tokens[t];
    float* out = h + (size_t)t * H;
    const bool ok = tok >= 0 && tok < V;
    const TW* row = table + (size_t)(ok ? tok : 0) * H;
    if ((H & 3) == 0) {
        for (int i = threadIdx.x * 4; i < H; i += blockDim.x * 4) {
            const float4 v = ok ? load4(row + i) : make_float4(0.f, 0.f, 0.f, 0.f);
            *reinterpret_cast<float4*>(out + i) = v;
        }
    } else {
        for (int i = threadIdx.x; i < H; i += blockDim.x) out[i] = ok ? to_f32(row[i]) : 0.0f;
    }
}

LUMEN_API int lumen_embed(const int* tokens, const void* table, int table_is_bf16, float* h,
                          int N, int H, int V, cudaStream_t stream) {
    if (N <= 0) return 0;
    if (H <= 0 || V <= 0) return LUMEN_ERR_BAD_ARGUMENT;
    if (table_is_bf16)
        lumen_launch(embed_kernel<__nv_bfloat16>, dim3(N), dim3(256), 0, stream, tokens, (const __nv_bfloat16*)table, h, H, V);
    else
        lumen_launch(embed_kernel<float>, dim3(N), dim3(256), 0, stream, tokens, (const float*)table, h, H, V);
    LUMEN_LAUNCH_CHECK();
    return 0;
}

// The same from a table kept in the tiled form of the tensor-core products (the head of
// csrc/gemm_tc.cu describes it): when the output head shares the embedding's matrix there is
// one copy of it, in the form the product reads. Piece c (8 values) of row r lies in k block
// c / 8 at row kb * w_rows + r, place (c & 7) ^ (r & 7).
__global__ void embed_tiled_kernel(const int* __restrict__ tokens, const uint4* __restrict__ table,
                                   float* __restrict__ h, int H, int V, int w_rows) {
    pdl_trigger();
    pdl_wait();      // nothing of this kernel touches global memory before this
    const int t = blockIdx.x;
    const int tok = tokens[t];
    float* out = h + (size_t)t * H;
    const bool ok = tok >= 0 && tok < V;
    for (int c = threadIdx.x; c < H / 8; c += blockDim.x) {
        float4 lo = make_float4(0.f, 0.f, 0.f, 0.f), hi = lo;
        if (ok) {
            const uint4 v = table[((size_t)(c >> 3) * w_rows + tok) * 8 + ((c & 7) ^ (tok & 7))];
            const __nv_bfloat162* b = reinterpret_cast<const __nv_bfloat162*>(&v);
            const float2 f0 = __bfloat1622float2(b[0]), f1 = __bfloat1622float2(b[1]);
            const float2 f2 = __bfloat1622float2(b[2]), f3 = __bfloat1622float2(b[3]);
            lo = make_float4(f0.x, f0.y, f1.x, f1.y);
            hi = make_float4(f2.x, f2.y, f3.x, f3.y);
        }
        *reinterpret_cast<float4*>(out + 8 * c) = lo;
        *reinterpret_cast<float4*>(out + 8 * c + 4) = hi;
    }
}

LUMEN_API int lumen_embed_tiled(const int* tokens, const void* table, float* h, int N, int H, int V, int w_rows,
                                cudaStream_t stream) {
    if (N <= 0) return 0;
    if (H <= 0 || V <= 0 || (H & 7) || w_rows < V || (w_rows & 7) || ((uintptr_t)table & 15) || ((uintptr_t)h & 15))
        return LUMEN_ERR_BAD_ARGUMENT;
    lumen_launch(embed_tiled_kernel, dim3(N), dim3(256), 0, stream, tokens, (const uint4*)table, h, H, V, w_rows);
    LUMEN_LAUNCH_CHECK();
    return 0;
}

// ---------------------------------------------------------------- add + RMSNorm
// x = h[r] + delta[0][r] + ... + delta[S-1][r] (summed in that order, float32); if write_h the
// sum is stored back to h[r]; y = x * 1/sqrt(mean(x^2)+eps) * w. With `rows`, block b reads
// row rows[b] and writes y row b (gather of the wanted rows); without, row b.
template <typename TOut>
__global__ void __launch_bounds__(1024)
add_rmsnorm_kernel(float* __restrict__ h, const float* __restrict__ delta, int S, size_t delta_stride,
                   const float* __restrict__ w, float eps, TOut* __restrict__ y,
                   const int* __restrict__ rows, int H, int write_h) {
    extern __shared__ __align__(16) float xs[];  // H floats
    __shared__ float red[32];
    const int b = blockIdx.x;
    // The norm's weight never changes: a thread whose share of the row is one group of four
    // values (the few-row launch: one thread a group) has it in registers before the kernel
    // ahead has finished, and the row's own chain is loads -> sum -> scale -> store.
    const bool one_group = (H & 3) == 0 && (int)blockDim.x * 4 >= H;
    float4 g_early = make_float4(0.f, 0.f, 0.f, 0.f);
    if (one_group && (int)threadIdx.x * 4 < H) g_early = load4(w + threadIdx.x * 4);
    pdl_trigger();
    pdl_wait();      // nothing else of this kernel touches global memory before this
    const int r = rows ? rows[b] : b;
    float* hr = h + (size_t)r * H;
    const float* dr = delta + (size_t)r * H;
    float ss = 0.0f;
    float4 x_mine = make_float4(0.f, 0.f, 0.f, 0.f);      // one_group: the thread's values stay in registers
    if ((H & 3) == 0) {
        for (int i = threadIdx.x * 4; i < H; i += blockDim.x * 4) {
            float4 x = load4(hr + i);
            // the partial sums are added in rising order; their loads go out eight at a time
            for (int s0 = 0; s0 < S; s0 += 8) {
                float4 d[8];
#pragma unroll
                for (int j = 0; j < 8; ++j)
                    if (s0 + j < S) d[j] = load4(dr + (size_t)(s0 + j) * delta_stride + i);
#pragma unroll
                for (int j = 0; j < 8; ++j)
                    if (s0 + j < S) { x.x += d[j].x; x.y += d[j].y; x.z += d[j].z; x.w += d[j].w; }
            }
            if (one_group) x_mine = x;
            else *reinterpret_cast<float4*>(xs + i) = x;
            if (write_h && S > 0) *reinterpret_cast<float4*>(hr + i) = x;
            ss += x.x * x.x;
            ss += x.y * x.y;
            ss += x.z * x.z;
            ss += x.w * x.w;
        }
    } else {
        for (int i = threadIdx.x; i < H; i += blockDim.x) {
            float x = hr[i];
            for (int s = 0; s < S; ++s) x += dr[(size_t)s * delta_stride + i];
            xs[i] = x;
            if (write_h && S > 0) hr[i] = x;
            ss += x * x;
        }
    }
    ss = block_sum(ss, red);
    const float scale = 1.0f / sqrtf(ss / (float)H + eps);
    TOut* yr = y + (size_t)b * H;
    if ((H & 3) == 0) {
        for (int i = threadIdx.x * 4; i < H; i += blockDim.x * 4) {
            const float4 x = one_group ? x_mine : *reinterpret_cast<const float4*>(xs + i);
            const float4 g = one_group ? g_early : load4(w + i);
            Pack4<TOut>::store(yr + i, x.x * scale * g.x, x.y * scale * g.y, x.z * scale * g.z,
                               x.w * scale * g.w);
        }
    } else {
        for (int i = threadIdx.x; i < H; i += blockDim.x) yr[i] = from_f32<TOut>(xs[i] * scale * w[i]);
    }
}

// The same for a single row (decode at batch 1), spread over a cluster of blocks. In a decode step the
// norm stands between two weight-streaming products whose blocks fill every SM with 181 KB of
// shared memory and some 46 K registers; a block of 1,024 threads finds no room beside them
// and starts only when one of them has left, while blocks of 256 threads fit, sit waiting at
// the dependency before the product ahead has finished, and have their weights loaded by
// then. So a row is taken by ARN_CLUSTER-or-fewer blocks of at most 256 threads, one group of
// four values a thread; each block sums its squares, writes that sum into every block's shared
// memory, and after ONE cluster barrier every block adds the sums in rank order (the same
// total in all of them). Blocks only write to their peers before the barrier and read their
// own memory after it, so a block may leave as soon as it is done.
#define ARN_CLUSTER 8
template <typename TOut>
__global__ void __launch_bounds__(256, 4)
add_rmsnorm_cluster_kernel(float* __restrict__ h, const float* __restrict__ delta, int S, size_t delta_stride,
                           const float* __restrict__ w, float eps, TOut* __restrict__ y,
                           const int* __restrict__ rows, int H, int write_h) {
    namespace cg = cooperative_groups;
    __shared__ float red[32];
    __shared__ float sums[ARN_CLUSTER];
    cg::cluster_group cluster = cg::this_cluster();
    const int rank = (int)cluster.block_rank(), nb = (int)cluster.num_blocks();
    const int b = blockIdx.x / nb;
    const int i = (rank * (int)blockDim.x + (int)threadIdx.x) * 4;
    const bool mine = i < H;
    const float4 g = mine ? load4(w + i) : make_float4(0.f, 0.f, 0.f, 0.f);
    pdl_trigger();
    pdl_wait();      // nothing else of this kernel touches global memory before this
    const int r = rows ? rows[b] : b;
    float* hr = h + (size_t)r * H;
    const float* dr = delta + (size_t)r * H;
    float4 x = mine ? load4(hr + i) : make_float4(0.f, 0.f, 0.f, 0.f);
    // the partial sums are added in rising order; their loads go out eight at a time
    for (int s0 = 0; s0 < S && mine; s0 += 8) {
        float4 d[8];
#pragma unroll
        for (int j = 0; j < 8; ++j)
            if (s0 + j < S) d[j] = load4(dr + (size_t)(s0 + j) * delta_stride + i);
#pragma unroll
        for (int j = 0; j < 8; ++j)
            if (s0 + j < S) { x.x += d[j].x; x.y += d[j].y; x.z += d[j].z; x.w += d[j].w; }
    }
    if (write_h && S > 0 && mine) *reinterpret_cast<float4*>(hr + i) = x;
    float ss = x.x * x.x;
    ss += x.y * x.y;
    ss += x.z * x.z;
    ss += x.w * x.w;
    ss = block_sum(ss, red);
    if ((int)threadIdx.x < nb) *cluster.map_shared_rank(&sums[rank], threadIdx.x) = ss;
    cluster.sync();
    float total = 0.0f;
    for (int k = 0; k < nb; ++k) total += sums[k];
    const float scale = 1.0f / sqrtf(total / (float)H + eps);
    if (mine)
        Pack4<TOut>::store(y + (size_t)b * H + i, x.x * scale * g.x, x.y * scale * g.y, x.z * scale * g.z,
                           x.w * scale * g.w);
}

template <typename TOut>
static cudaError_t add_rmsnorm_cluster_launch(int n_rows, int nb, int threads, cudaStream_t stream, float* h,
                                              const float* delta, int S, size_t delta_stride, const float* w,
                                              float eps, TOut* y, const int* rows, int H, int write_h) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(n_rows * nb);
    cfg.blockDim = dim3(threads);
    cfg.dynamicSmemBytes = 0;
    cfg.stream = stream;
    cudaLaunchAttribute attr[2];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = nb;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[1].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = lumen_pdl_enabled() ? 2 : 1;
    return cudaLaunchKernelEx(&cfg, add_rmsnorm_cluster_kernel<TOut>, h, delta, S, delta_stride, w, eps, y, rows, H,
                              write_h);
}

// The same for many rows (prompts) of at most 16 x 512 values: a thread keeps its four groups
// of four values in registers, so all loads of a row are in flight at once and nothing goes
// through shared memory; few registers, so that six blocks of 256 threads share an SM.
#define ARN_GROUPS 4
template <typename TOut>
__global__ void __launch_bounds__(512, 3)
add_rmsnorm_rows_kernel(float* __restrict__ h, const float* __restrict__ delta, int S, size_t delta_stride,
                        const float* __restrict__ w, float eps, TOut* __restrict__ y,
                        const int* __restrict__ rows, int H, int write_h) {
    __shared__ float red[32];
    const int b = blockIdx.x;
    float4 x[ARN_GROUPS];
    pdl_trigger();
    pdl_wait();      // nothing of this kernel touches global memory before this
    const int r = rows ? rows[b] : b;
    float* hr = h + (size_t)r * H;
    const float* dr = delta + (size_t)r * H;
#pragma unroll
    for (int j = 0; j < ARN_GROUPS; ++j) {
        const int i = (j * blockDim.x + threadIdx.x) * 4;
        x[j] = i < H ? load4(hr + i) : make_float4(0.f, 0.f, 0.f, 0.f);
    }
    for (int s = 0; s < S; ++s) {             // the partial sums are added in rising order
        float4 d[ARN_GROUPS];
#pragma unroll
        for (int j = 0; j < ARN_GROUPS; ++j) {
            const int i = (j * blockDim.x + threadIdx.x) * 4;
            d[j] = i < H ? load4(dr + (size_t)s * delta_stride + i) : make_float4(0.f, 0.f, 0.f, 0.f);
        }
#pragma unroll
        for (int j = 0; j < ARN_GROUPS; ++j) { x[j].x += d[j].x; x[j].y += d[j].y; x[j].z += d[j].z; x[j].w += d[j].w; }
    }
    float ss = 0.0f;
#pragma unroll
    for (int j = 0; j < ARN_GROUPS; ++j) {
        const int i = (j * blockDim.x + threadIdx.x) * 4;
        if (write_h && S > 0 && i < H) *reinterpret_cast<float4*>(hr + i) = x[j];
        ss += x[j].x * x[j].x;
        ss += x[j].y * x[j].y;
        ss += x[j].z * x[j].z;
        ss += x[j].w * x[j].w;
    }
    ss = block_sum(ss, red);
    const float scale = 1.0f / sqrtf(ss / (float)H + eps);
    TOut* yr = y + (size_t)b * H;
#pragma unroll
    for (int j = 0; j < ARN_GROUPS; ++j) {
        const int i = (j * blockDim.x + threadIdx.x) * 4;
        if (i < H) {
            const float4 g = load4(w + i);    // the same 16 KB for every row: it stays in L1
            Pack4<TOut>::store(yr + i, x[j].x * scale * g.x, x[j].y * scale * g.y, x[j].z * scale * g.z,
                               x[j].w * scale * g.w);
        }
    }
}

LUMEN_API int lumen_add_rmsnorm(float* h, const float* delta, int n_delta, long long delta_stride,
                                const float* w, float eps, void* y, int y_is_bf16,
                                const int* rows, int n_rows, int H, int write_h,
                                cudaStream_t stream) {
    if (n_rows <= 0) return 0;
    if (H <= 0 || n_delta < 0) return LUMEN_ERR_BAD_ARGUMENT;
    if (n_rows >= 2 * 148 && (H & 3) == 0 && H <= 512 * 4 * ARN_GROUPS) {
        int t = ((H / (4 * ARN_GROUPS) + 31) / 32) * 32;
        if (t < 64) t = 64;
        if (y_is_bf16)
            lumen_launch(add_rmsnorm_rows_kernel<__nv_bfloat16>, dim3(n_rows), dim3(t), 0, stream, h, delta, n_delta,
                         (size_t)delta_stride, w, eps, (__nv_bfloat16*)y, rows, H, write_h);
        else
            lumen_launch(add_rmsnorm_rows_kernel<float>, dim3(n_rows), dim3(t), 0, stream, h, delta, n_delta,
                         (size_t)delta_stride, w, eps, (float*)y, rows, H, write_h);
        LUMEN_LAUNCH_CHECK();
        return 0;
    }
    // One row only: measured inside a decode step, the cluster gains 0.7 % of the step at batch 1
    // (1.255 against 1.265 ms for 12 layers of the 8B shape) and loses 0.6 to 2 % at batch 2 to 16,
    // where several clusters meet at their barriers at once.
    if (n_rows == 1 && (H & 3) == 0 && H <= ARN_CLUSTER * 256 * 4) {
        const int nb = (H / 4 + 255) / 256;                       // blocks a row
        const int threads = (((H / 4 + nb - 1) / nb + 31) / 32) * 32;
        cudaError_t e = y_is_bf16
            ? add_rmsnorm_cluster_launch<__nv_bfloat16>(n_rows, nb, threads, stream, h, delta, n_delta,
                                                        (size_t)delta_stride, w, eps, (__nv_bfloat16*)y, rows, H, write_h)
            : add_rmsnorm_cluster_launch<float>(n_rows, nb, threads, stream, h, delta, n_delta, (size_t)delta_stride,
                                                w, eps, (float*)y, rows, H, write_h);
        if (e != cudaSuccess) return (int)e;
        LUMEN_LAUNCH_CHECK();
        return 0;
    }
    const size_t smem = (size_t)H * sizeof(float);
    if (smem > 200 * 1024) return LUMEN_ERR_UNSUPPORTED;
    // Few rows (decode): one row per block cannot fill the GPU, so each block is made wide and
    // every thread has all its loads in flight at once. Many rows: 256 threads a row.
    int threads = 256;
    if (n_rows < 2 * 148) {
        threads = ((H / 4 + 31) / 32) * 32;
        if (threads > 1024) threads = 1024;
        if (threads < 128) threads = 128;
    }
    if (y_is_bf16) {
        auto k = add_rmsnorm_kernel<__nv_bfloat16>;
        if (smem > 48 * 1024) cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        lumen_launch(k, dim3(n_rows), dim3(threads), smem, stream, h, delta, n_delta, (size_t)delta_stride, w, eps,
                                             (__nv_bfloat16*)y, rows, H, write_h);
    } else {
        auto k = add_rmsnorm_kernel<float>;
        if (smem > 48 * 1024) cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        lumen_launch(k, dim3(n_rows), dim3(threads), smem, stream, h, delta, n_delta, (size_t)delta_stride, w, eps, (float*)y,
                                             rows, H, write_h);
    }
    LUMEN_LAUNCH_CHECK();
    return 0;
}

// ---------------------------------------------------------------- SiLU(gate) * up
// gu: [S, N, 2*I] float32 partials with the gate in columns [0, I) and up in [I, 2I); or,
// interleaved, gate_i in column 2i and up_i in column 2i + 1.
template <typename TOut>
__global__ void silu_mul_kernel(const float* __restrict__ gu, int S, size_t split_stride,
                                TOut* __restrict__ z, long long total, int I, int interleaved) {
    pdl_trigger();
    pdl_wait();      // nothing of this kernel touches global memory before this
    long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    const long long step = (long long)gridDim.x * blockDim.x;
    if (interleaved && (I & 3) == 0) {
        // four (gate, up) pairs a thread: 32 bytes in, 8 out; the partial sums' loads go out
        // together and are added in rising order
        const long long total4 = total >> 2;
        const int I4 = I >> 2;
        for (; idx < total4; idx += step) {
            const long long n = idx / I4;
            const int i = (int)(idx - n * I4) * 4;
            const float* gp = gu + n * 2 * I + 2 * i;
            float4 a = load4(gp), b = load4(gp + 4);
            for (int s0 = 1; s0 < S; s0 += 4) {
                float4 a2[4], b2[4];
#pragma unroll
                for (int j = 0; j < 4; ++j)
                    if (s0 + j < S) { a2[j] = load4(gp + (s0 + j) * split_stride); b2[j] = load4(gp + (s0 + j) * split_stride + 4); }
#pragma unroll
                for (int j = 0; j < 4; ++j)
                    if (s0 + j < S) {
                        a.x += a2[j].x; a.y += a2[j].y; a.z += a2[j].z; a.w += a2[j].w;
                        b.x += b2[j].x; b.y += b2[j].y; b.z += b2[j].z; b.w += b2[j].w;
                    }
            }
            Pack4<TOut>::store(z + n * I + i, a.x / (1.0f + expf(-a.x)) * a.y, a.z / (1.0f + expf(-a.z)) * a.w,
                               b.x / (1.0f + expf(-b.x)) * b.y, b.z / (1.0f + expf(-b.z)) * b.w);
        }
    } else if (interleaved) {
        for (; idx < total; idx += step) {
            const long long n = idx / I;
            const int i = (int)(idx - n * I);
            const float* gp = gu + n * 2 * I + 2 * i;
            float2 v = *reinterpret_cast<const float2*>(gp);
            for (int s = 1; s < S; ++s) {
                const float2 v2 = *reinterpret_cast<const float2*>(gp + s * split_stride);
                v.x += v2.x; v.y += v2.y;
            }
            z[idx] = from_f32<TOut>(v.x / (1.0f + expf(-v.x)) * v.y);
        }
    } else if ((I & 3) == 0) {
        const long long total4 = total >> 2;
        const int I4 = I >> 2;
        for (; idx < total4; idx += step) {
            const long long n = idx / I4;
            const int i = (int)(idx - n * I4) * 4;
            const float* gp = gu + n * 2 * I + i;
            float4 g = load4(gp), u = load4(gp + I);
            for (int s = 1; s < S; ++s) {
                const float4 g2 = load4(gp + s * split_stride), u2 = load4(gp + s * split_stride + I);
                g.x += g2.x; g.y += g2.y; g.z += g2.z; g.w += g2.w;
                u.x += u2.x; u.y += u2.y; u.z += u2.z; u.w += u2.w;
            }
            Pack4<TOut>::store(z + n * I + i, g.x / (1.0f + expf(-g.x)) * u.x, g.y / (1.0f + expf(-g.y)) * u.y,
                               g.z / (1.0f + expf(-g.z)) * u.z, g.w / (1.0f + expf(-g.w)) * u.w);
        }
    } else {
        for (; idx < total; idx += step) {
            const long long n = idx / I;
            const int i = (int)(idx - n * I);
            float g = gu[n * 2 * I + i], u = gu[n * 2 * I + I + i];
            for (int s = 1; s < S; ++s) {
                g += gu[s * split_stride + n * 2 * I + i];
                u += gu[s * split_stride + n * 2 * I + I + i];
            }
            z[idx] = from_f32<TOut>(g / (1.0f + expf(-g)) * u);
        }
    }
}

LUMEN_API int lumen_silu_mul(const float* gu, int n_splits, void* z, int z_is_bf16, int N, int I,
                             int interleaved, cudaStream_t stream) {
    if (N <= 0) return 0;
    if (I <= 0 || n_splits < 1) return LUMEN_ERR_BAD_ARGUMENT;
    const long long total = (long long)N * I;
    const size_t stride = (size_t)N * 2 * I;
    long long blocks = (((I & 3) ? total : total / 4) + 255) / 256;
    if (blocks > 148 * 16) blocks = 148 * 16;
    if (blocks < 1) blocks = 1;
    if (z_is_bf16)
        lumen_launch(silu_mul_kernel<__nv_bfloat16>, dim3((int)blocks), dim3(256), 0, stream, gu, n_splits, stride,
                                                                       (__nv_bfloat16*)z, total, I, interleaved);
    else
        lumen_launch(silu_mul_kernel<float>, dim3((int)blocks), dim3(256), 0, stream, gu, n_splits, stride, (float*)z, total, I,
                                                                interleaved);
    LUMEN_LAUNCH_CHECK();
    return 0;
}

// ---------------------------------------------------------------- rotation angles
// cs[n, i] = (cos, sin) of angle = float(pos[n]) * inv_freq[i], i < half. Made once per step
// and read by every layer that shares the position encoding.
__global__ void rope_table_kernel(const int* __restrict__ pos, const float* __restrict__ inv_freq,
                                  float2* __restrict__ cs, int N, int half) {
    pdl_trigger();
    pdl_wait();      // nothing of this kernel touches global memory before this
    const long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= (long long)N * half) return;
    const int n = (int)(idx / half), i = (int)(idx - (long long)n * half);
    const float ang = (float)pos[n] * inv_freq[i];
    float s, c;
    sincosf(ang, &s, &c);
    cs[idx] = make_float2(c, s);
}

LUMEN_API int lumen_rope_table(const int* pos, const float* inv_freq, float* cs, int N, int half,
                               cudaStream_t stream) {
    if (N <= 0 || half <= 0) return 0;
    const long long total = (long long)N * half;
    lumen_launch(rope_table_kernel, dim3((int)((total + 255) / 256)), dim3(256), 0, stream, pos, inv_freq, (float2*)cs, N, half);
    LUMEN_LAUNCH_CHECK();
    return 0;
}

// ---------------------------------------------------------------- q/k norm + rotary + cache write
// Input row n of `qkv` (the sum of S partials) holds nq query heads, then nkv key heads, then
// nkv value heads, d floats each. One warp per (token, head):
//   q, k: optional RMSNorm over the head's d values with a weight of length d, then rotation
//         of pairs (i, i + rot/2), i < rot/2, by the angles of cs[n];
//   q goes to q_out[n, head, :]; k and v go to the paged cache at
//   page = block_table[tok_seq[n], cache_pos[n] / PAGE], row cache_pos[n] % PAGE.
#define QKR_MAX_D 512
template <typename T>
__global__ void qk_norm_rope_store_kernel(const float* __restrict__ qkv, int S, size_t split_stride,
                                          const float* __restrict__ qw, const float* __restrict__ kw,
                                          float eps, const float2* __restrict__ cs, int rot,
                                          const int* __restrict__ cache_pos,
                                          const int* __restrict__ tok_seq,
                                          const int* __restrict__ block_table, int bt_stride,
                                          T* __restrict__ q_out, T* __restrict__ kcache,
                                          T* __restrict__ vcache, int nq, int nkv, int d, int layout) {
    pdl_trigger();
    pdl_wait();      // nothing of this kernel touches global memory before this
    extern __shared__ __align__(16) float rowbuf[];  // [warps][d]
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int n = blockIdx.x;
    const int head = blockIdx.y * (blockDim.x >> 5) + warp;
    const int nheads = nq + 2 * nkv;
    if (head >= nheads) return;
    float* x = rowbuf + warp * d;
    const float* src = qkv + ((size_t)n * nheads + head) * d;
    for (int e = lane * 4; e < d; e += 128) {
        float4 v = load4(src + e);
        for (int s = 1; s < S; ++s) {
            const float4 v2 = load4(src + s * split_stride + e);
            v.x += v2.x; v.y += v2.y; v.z += v2.z; v.w += v2.w;
        }
        *reinterpret_cast<float4*>(x + e) = v;
    }
    __syncwarp();
    const bool is_q = head < nq;
    const bool is_k = !is_q && head < nq + nkv;
    const float* nw = is_q ? qw : (is_k ? kw : nullptr);
    if (nw) {
        float ss = 0.0f;
        for (int e = lane; e < d; e += 32) ss += x[e] * x[e];
        ss = warp_sum(ss);
        const float scale = 1.0f / sqrtf(ss / (float)d + eps);
        for (int e = lane; e < d; e += 32) x[e] = x[e] * scale * nw[e];
        __syncwarp();
    }
    if ((is_q || is_k) && rot > 0) {
        const int half = rot >> 1;
        const float2* csn = cs + (size_t)n * half;
        for (int i = lane; i < half; i += 32) {
            const float2 c_s = csn[i];
            const float a = x[i], b = x[i + half];
            x[i] = a * c_s.x - b * c_s.y;
            x[i + half] = a * c_s.y + b * c_s.x;
        }
        __syncwarp();
    }
    if (is_q) {
        T* dst = q_out + ((size_t)n * nq + head) * d;
        for (int e = lane * 4; e < d; e += 128) Pack4<T>::store(dst + e, x[e], x[e + 1], x[e + 2], x[e + 3]);
    } else {
        const int kvh = is_k ? head - nq : head - nq - nkv;
        const int cp = cache_pos[n];
        const int page = block_table[(size_t)tok_seq[n] * bt_stride + cp / LUMEN_PAGE];
        T* tile = (is_k ? kcache : vcache) + ((size_t)page * nkv + kvh) * LUMEN_PAGE * d;
        const int r = cp % LUMEN_PAGE;
        // groups of 4 values never straddle a 16-byte chunk, so they stay together in both layouts
        for (int e = lane * 4; e < d; e += 128)
            Pack4<T>::store(tile + tile_offset(layout, r, e, d), x[e], x[e + 1], x[e + 2], x[e + 3]);
    }
}

// The same for head size 128 rotated over all 128 values: a lane keeps 4 consecutive values
// in registers, the partner of value e in the rotation (e +- 64) lives 16 lanes away, and
// nothing goes through shared memory.
template <typename T>
__global__ void __launch_bounds__(256)
qk_norm_rope_store_d128_kernel(const float* __restrict__ qkv, int S, size_t split_stride,
                               const float* __restrict__ qw, const float* __restrict__ kw, float eps,
                               const float2* __restrict__ cs, int rot, const int* __restrict__ cache_pos,
                               const int* __restrict__ tok_seq, const int* __restrict__ block_table,
                               int bt_stride, T* __restrict__ q_out, T* __restrict__ kcache,
                               T* __restrict__ vcache, int nq, int nkv, int layout) {
    pdl_trigger();
    pdl_wait();      // nothing of this kernel touches global memory before this
    constexpr int d = 128;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int n = blockIdx.x;
    const int head = blockIdx.y * 8 + warp;
    const int nheads = nq + 2 * nkv;
    if (head >= nheads) return;
    const bool is_q = head < nq;
    const bool is_k = !is_q && head < nq + nkv;
    const float4 v = qk_head_d128(qkv + ((size_t)n * nheads + head) * d, S, split_stride,
                                  is_q ? qw : (is_k ? kw : nullptr), eps, cs + (size_t)n * 64,
                                  (is_q || is_k) && rot == d, lane);
    if (is_q) {
        Pack4<T>::store(q_out + ((size_t)n * nq + head) * d + 4 * lane, v.x, v.y, v.z, v.w);
    } else {
        const int kvh = is_k ? head - nq : head - nq - nkv;
        const int cp = cache_pos[n];
        const int page = block_table[(size_t)tok_seq[n] * bt_stride + cp / LUMEN_PAGE];
        T* tile = (is_k ? kcache : vcache) + ((size_t)page * nkv + kvh) * LUMEN_PAGE * d;
        Pack4<T>::store(tile + tile_offset(layout, cp % LUMEN_PAGE, 4 * lane, d), v.x, v.y, v.z, v.w);
    }
}

// The same for many tokens (prompts), laid out so that the rotation needs no exchange between
// lanes: a warp takes QKR_HPW consecutive heads of its token two at a time, the lower 16 lanes
// one head and the upper 16 the next; a lane holds values 4l..4l+3 and their partners
// 64+4l..64+4l+3, and a head's sum of squares runs over 16 lanes. The rotation table and the
// token's page are looked up once a warp, the norms' weights before the kernel ahead has
// finished. Which of q, k or v a lane's head is decides by selects, not branches.
#define QKR_HPW 4
template <typename T>
__global__ void __launch_bounds__(128, 8)
qk_norm_rope_store_d128_rows_kernel(const float* __restrict__ qkv, int S, size_t split_stride,
                                    const float* __restrict__ qw, const float* __restrict__ kw, float eps,
                                    const float2* __restrict__ cs, int rot, const int* __restrict__ cache_pos,
                                    const int* __restrict__ tok_seq, const int* __restrict__ block_table,
                                    int bt_stride, T* __restrict__ q_out, T* __restrict__ kcache,
                                    T* __restrict__ vcache, int nq, int nkv, int layout) {
    constexpr int d = 128;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int li = lane & 15, up = lane >> 4;
    const int n = blockIdx.x;
    const int head0 = (blockIdx.y * 4 + warp) * QKR_HPW;
    const int nheads = nq + 2 * nkv;
    const float4 one = make_float4(1.f, 1.f, 1.f, 1.f);
    const float4 gq_lo = qw ? load4(qw + 4 * li) : one, gq_hi = qw ? load4(qw + 64 + 4 * li) : one;
    const float4 gk_lo = kw ? load4(kw + 4 * li) : one, gk_hi = kw ? load4(kw + 64 + 4 * li) : one;
    pdl_trigger();
    pdl_wait();      // nothing else of this kernel touches global memory before this
    if (head0 >= nheads) return;
    float4 lo[QKR_HPW / 2], hi[QKR_HPW / 2];
    const float* src = qkv + ((size_t)n * nheads + head0 + up) * d + 4 * li;
#pragma unroll
    for (int j = 0; j < QKR_HPW / 2; ++j) {
        const bool have = head0 + 2 * j + up < nheads;
        lo[j] = have ? load4(src + 2 * j * d) : make_float4(0.f, 0.f, 0.f, 0.f);
        hi[j] = have ? load4(src + 2 * j * d + 64) : make_float4(0.f, 0.f, 0.f, 0.f);
    }
    float4 c01 = make_float4(1.f, 0.f, 1.f, 0.f), c23 = c01;
    if (rot == d) {
        const float4* csn = reinterpret_cast<const float4*>(cs + (size_t)n * 64 + 4 * li);
        c01 = csn[0];        // (cos, sin) of 4 consecutive pairs
        c23 = csn[1];
    }
    const int cp = cache_pos[n];
    const int page = head0 + QKR_HPW > nq ? block_table[(size_t)tok_seq[n] * bt_stride + cp / LUMEN_PAGE] : 0;
    const int off_lo = tile_offset(layout, cp % LUMEN_PAGE, 4 * li, d);
    const int off_hi = tile_offset(layout, cp % LUMEN_PAGE, 64 + 4 * li, d);
    for (int s = 1; s < S; ++s) {             // the partial sums are added in rising order
        float4 lo2[QKR_HPW / 2], hi2[QKR_HPW / 2];
#pragma unroll
        for (int j = 0; j < QKR_HPW / 2; ++j) {
            const bool have = head0 + 2 * j + up < nheads;
            lo2[j] = have ? load4(src + 2 * j * d + (size_t)s * split_stride) : make_float4(0.f, 0.f, 0.f, 0.f);
            hi2[j] = have ? load4(src + 2 * j * d + 64 + (size_t)s * split_stride) : make_float4(0.f, 0.f, 0.f, 0.f);
        }
#pragma unroll
        for (int j = 0; j < QKR_HPW / 2; ++j) {
            lo[j].x += lo2[j].x; lo[j].y += lo2[j].y; lo[j].z += lo2[j].z; lo[j].w += lo2[j].w;
            hi[j].x += hi2[j].x; hi[j].y += hi2[j].y; hi[j].z += hi2[j].z; hi[j].w += hi2[j].w;
        }
    }
#pragma unroll
    for (int j = 0; j < QKR_HPW / 2; ++j) {
        const int head = head0 + 2 * j + up;
        const bool is_q = head < nq;
        const bool is_k = !is_q && head < nq + nkv;
        float4 a = lo[j], b = hi[j];
        float ss = a.x * a.x;
        ss += a.y * a.y;
        ss += a.z * a.z;
        ss += a.w * a.w;
        ss += b.x * b.x;
        ss += b.y * b.y;
        ss += b.z * b.z;
        ss += b.w * b.w;
#pragma unroll
        for (int m = 8; m >= 1; m >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, m);   // over the head's 16 lanes
        if ((is_q && qw) || (is_k && kw)) {
            const float scale = 1.0f / sqrtf(ss / (float)d + eps);
            const float4 g_lo = is_q ? gq_lo : gk_lo, g_hi = is_q ? gq_hi : gk_hi;
            a.x = a.x * scale * g_lo.x; a.y = a.y * scale * g_lo.y; a.z = a.z * scale * g_lo.z; a.w = a.w * scale * g_lo.w;
            b.x = b.x * scale * g_hi.x; b.y = b.y * scale * g_hi.y; b.z = b.z * scale * g_hi.z; b.w = b.w * scale * g_hi.w;
        }
        if (is_q || is_k) {      // x'_i = x_i cos - x_{i+64} sin, x'_{i+64} = x_i sin + x_{i+64} cos
            const float4 a0 = a;
            a.x = a0.x * c01.x - b.x * c01.y; a.y = a0.y * c01.z - b.y * c01.w;
            a.z = a0.z * c23.x - b.z * c23.y; a.w = a0.w * c23.z - b.w * c23.w;
            b.x = a0.x * c01.y + b.x * c01.x; b.y = a0.y * c01.w + b.y * c01.z;
            b.z = a0.z * c23.y + b.z * c23.x; b.w = a0.w * c23.w + b.w * c23.z;
        }
        if (head < nheads) {
            T* p_lo;
            T* p_hi;
            if (is_q) {
                p_lo = q_out + ((size_t)n * nq + head) * d + 4 * li;
                p_hi = p_lo + 64;
            } else {
                const int kvh = is_k ? head - nq : head - nq - nkv;
                T* tile = (is_k ? kcache : vcache) + ((size_t)page * nkv + kvh) * LUMEN_PAGE * d;
                p_lo = tile + off_lo;
                p_hi = tile + off_hi;
            }
            Pack4<T>::store(p_lo, a.x, a.y, a.z, a.w);
            Pack4<T>::store(p_hi, b.x, b.y, b.z, b.w);
        }
    }
}

LUMEN_API int lumen_qk_norm_rope_store(const float* qkv, int n_splits, const float* qw, const float* kw,
                                       float eps, const float* cs, int rot, const int* cache_pos,
                                       const int* tok_seq, const int* block_table, int bt_stride,
                                       void* q_out, void* kcache, void* vcache, int is_bf16, int N,
                                       int nq, int nkv, int d, int layout, cudaStream_t stream) {
    if (N <= 0) return 0;
    if (d <= 0 || d > QKR_MAX_D || (d & 3) || rot < 0 || rot > d || (rot & 1) || nq < 0 || nkv < 0 ||
        n_splits < 1)
        return LUMEN_ERR_UNSUPPORTED;
    if (layout == LUMEN_LAYOUT_SW128 && (!is_bf16 || d % 64 != 0)) return LUMEN_ERR_UNSUPPORTED;
    if (layout != LUMEN_LAYOUT_SW128 && layout != LUMEN_LAYOUT_LINEAR) return LUMEN_ERR_BAD_ARGUMENT;
    const int warps = 4;
    const int nheads = nq + 2 * nkv;
    if (nheads == 0) return 0;
    if ((nheads + warps - 1) / warps > 65535) return LUMEN_ERR_UNSUPPORTED;
    if (d == 128 && (rot == 128 || rot == 0) && N >= 2 * 148) {
        dim3 g(N, (nheads + 4 * QKR_HPW - 1) / (4 * QKR_HPW));
        const size_t st = (size_t)N * nheads * d;
        if (is_bf16)
            lumen_launch(qk_norm_rope_store_d128_rows_kernel<__nv_bfloat16>, dim3(g), dim3(128), 0, stream,
                qkv, n_splits, st, qw, kw, eps, (const float2*)cs, rot, cache_pos, tok_seq, block_table,
                bt_stride, (__nv_bfloat16*)q_out, (__nv_bfloat16*)kcache, (__nv_bfloat16*)vcache, nq, nkv,
                layout);
        else
            lumen_launch(qk_norm_rope_store_d128_rows_kernel<float>, dim3(g), dim3(128), 0, stream,
                qkv, n_splits, st, qw, kw, eps, (const float2*)cs, rot, cache_pos, tok_seq, block_table,
                bt_stride, (float*)q_out, (float*)kcache, (float*)vcache, nq, nkv, layout);
        LUMEN_LAUNCH_CHECK();
        return 0;
    }
    if (d == 128 && (rot == 128 || rot == 0)) {
        dim3 g8(N, (nheads + 7) / 8);
        const size_t st = (size_t)N * nheads * d;
        if (is_bf16)
            lumen_launch(qk_norm_rope_store_d128_kernel<__nv_bfloat16>, dim3(g8), dim3(256), 0, stream, 
                qkv, n_splits, st, qw, kw, eps, (const float2*)cs, rot, cache_pos, tok_seq, block_table,
                bt_stride, (__nv_bfloat16*)q_out, (__nv_bfloat16*)kcache, (__nv_bfloat16*)vcache, nq, nkv,
                layout);
        else
            lumen_launch(qk_norm_rope_store_d128_kernel<float>, dim3(g8), dim3(256), 0, stream, 
                qkv, n_splits, st, qw, kw, eps, (const float2*)cs, rot, cache_pos, tok_seq, block_table,
                bt_stride, (float*)q_out, (float*)kcache, (float*)vcache, nq, nkv, layout);
        LUMEN_LAUNCH_CHECK();
        return 0;
    }
    dim3 grid(N, (nheads + warps - 1) / warps);
    const size_t smem = (size_t)warps * d * sizeof(float);
    const size_t stride = (size_t)N * nheads * d;
    if (is_bf16)
        lumen_launch(qk_norm_rope_store_kernel<__nv_bfloat16>, dim3(grid), dim3(warps * 32), smem, stream, 
            qkv, n_splits, stride, qw, kw, eps, (const float2*)cs, rot, cache_pos, tok_seq, block_table,
            bt_stride, (__nv_bfloat16*)q_out, (__nv_bfloat16*)kcache, (__nv_bfloat16*)vcache, nq, nkv, d,
            layout);
    else
        lumen_launch(qk_norm_rope_store_kernel<float>, dim3(grid), dim3(warps * 32), smem, stream, 
            qkv, n_splits, stride, qw, kw, eps, (const float2*)cs, rot, cache_pos, tok_seq, block_table,
            bt_stride, (float*)q_out, (float*)kcache, (float*)vcache, nq, nkv, d, layout);
    LUMEN_LAUNCH_CHECK();
    return 0;
}
