// Memory-bound parts of a decoder step: embedding gather, residual add + RMSNorm,
// SiLU(gate)*up, and the fused per-head RMSNorm + rotary encoding + cache write.
// All arithmetic is float32; the output type T is float (32-bit path) or
// __nv_bfloat16. Compiled without fast-math: sqrtf, expf and sincosf are the
// precise forms.
#include "common.cuh"

// ---------------------------------------------------------------- embedding
// h[t, :] = float(E[token[t], :]); a token outside the table writes zeros (the
// host has refused it before; this is the second guard).
template <typename TW>
__global__ void embed_kernel(const int* __restrict__ tokens, const TW* __restrict__ table,
                             float* __restrict__ h, int H, int V) {
    const int t = blockIdx.x;
    const int tok = tokens[t];
    float* out = h + (size_t)t * H;
    if (tok < 0 || tok >= V) {
        for (int i = threadIdx.x; i < H; i += blockDim.x) out[i] = 0.0f;
        return;
    }
    const TW* row = table + (size_t)tok * H;
    for (int i = threadIdx.x; i < H; i += blockDim.x) out[i] = to_f32(row[i]);
}

LUMEN_API int lumen_embed(const int* tokens, const void* table, int table_is_bf16, float* h,
                          int N, int H, int V, cudaStream_t stream) {
    if (N <= 0) return 0;
    if (H <= 0 || V <= 0) return LUMEN_ERR_BAD_ARGUMENT;
    if (table_is_bf16)
        embed_kernel<__nv_bfloat16><<<N, 256, 0, stream>>>(tokens, (const __nv_bfloat16*)table, h, H, V);
    else
        embed_kernel<float><<<N, 256, 0, stream>>>(tokens, (const float*)table, h, H, V);
    LUMEN_LAUNCH_CHECK();
    return 0;
}

// ---------------------------------------------------------------- add + RMSNorm
// x = h[r] + delta[0][r] + ... + delta[S-1][r] (summed in that order, float32);
// if write_h the sum is stored back to h[r]; y = x * 1/sqrt(mean(x^2)+eps) * w.
// With `rows`, block b reads row rows[b] and writes y row b (gather of the
// wanted rows); without, row b.
template <typename TOut>
__global__ void add_rmsnorm_kernel(float* __restrict__ h, const float* __restrict__ delta, int S,
                                   size_t delta_stride, const float* __restrict__ w, float eps,
                                   TOut* __restrict__ y, const int* __restrict__ rows, int H,
                                   int write_h) {
    extern __shared__ float xs[];  // H floats
    __shared__ float red[32];
    const int b = blockIdx.x;
    const int r = rows ? rows[b] : b;
    float* hr = h + (size_t)r * H;
    float ss = 0.0f;
    for (int i = threadIdx.x; i < H; i += blockDim.x) {
        float x = hr[i];
        for (int s = 0; s < S; ++s) x += delta[(size_t)s * delta_stride + (size_t)r * H + i];
        xs[i] = x;
        if (write_h && S > 0) hr[i] = x;
        ss += x * x;
    }
    ss = block_sum(ss, red);
    const float scale = 1.0f / sqrtf(ss / (float)H + eps);
    TOut* yr = y + (size_t)b * H;
    for (int i = threadIdx.x; i < H; i += blockDim.x) yr[i] = from_f32<TOut>(xs[i] * scale * w[i]);
}

LUMEN_API int lumen_add_rmsnorm(float* h, const float* delta, int n_delta, long long delta_stride,
                                const float* w, float eps, void* y, int y_is_bf16,
                                const int* rows, int n_rows, int H, int write_h,
                                cudaStream_t stream) {
    if (n_rows <= 0) return 0;
    if (H <= 0 || n_delta < 0) return LUMEN_ERR_BAD_ARGUMENT;
    const size_t smem = (size_t)H * sizeof(float);
    if (smem > 200 * 1024) return LUMEN_ERR_UNSUPPORTED;
    if (y_is_bf16) {
        auto k = add_rmsnorm_kernel<__nv_bfloat16>;
        if (smem > 48 * 1024) cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        k<<<n_rows, 256, smem, stream>>>(h, delta, n_delta, (size_t)delta_stride, w, eps,
                                         (__nv_bfloat16*)y, rows, H, write_h);
    } else {
        auto k = add_rmsnorm_kernel<float>;
        if (smem > 48 * 1024) cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        k<<<n_rows, 256, smem, stream>>>(h, delta, n_delta, (size_t)delta_stride, w, eps, (float*)y,
                                         rows, H, write_h);
    }
    LUMEN_LAUNCH_CHECK();
    return 0;
}

// ---------------------------------------------------------------- SiLU(gate) * up
// gu: [N, 2*I] float32 with the gate in columns [0, I) and up in [I, 2I).
template <typename TOut>
__global__ void silu_mul_kernel(const float* __restrict__ gu, TOut* __restrict__ z, long long total,
                                int I) {
    long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    const long long step = (long long)gridDim.x * blockDim.x;
    for (; idx < total; idx += step) {
        const long long n = idx / I;
        const int i = (int)(idx - n * I);
        const float g = gu[n * 2 * I + i];
        const float u = gu[n * 2 * I + I + i];
        z[idx] = from_f32<TOut>(g / (1.0f + expf(-g)) * u);
    }
}

LUMEN_API int lumen_silu_mul(const float* gu, void* z, int z_is_bf16, int N, int I,
                             cudaStream_t stream) {
    if (N <= 0) return 0;
    if (I <= 0) return LUMEN_ERR_BAD_ARGUMENT;
    const long long total = (long long)N * I;
    long long blocks = (total + 255) / 256;
    if (blocks > 148 * 16) blocks = 148 * 16;
    if (z_is_bf16)
        silu_mul_kernel<__nv_bfloat16><<<(int)blocks, 256, 0, stream>>>(gu, (__nv_bfloat16*)z, total, I);
    else
        silu_mul_kernel<float><<<(int)blocks, 256, 0, stream>>>(gu, (float*)z, total, I);
    LUMEN_LAUNCH_CHECK();
    return 0;
}

// ---------------------------------------------------------------- q/k norm + rotary + cache write
// Input row n of `qkv` holds nq query heads, then nkv key heads, then nkv value
// heads, d floats each. One warp per (token, head):
//   q, k: optional RMSNorm over the head's d values with a weight of length d,
//         then rotation of pairs (i, i + rot/2), i < rot/2, by
//         angle = float(pos) * inv_freq[i];
//   q goes to q_out[n, head, :]; k and v go to the paged cache at
//   page = block_table[tok_seq[n], cache_pos[n] / PAGE], row cache_pos[n] % PAGE.
#define QKR_MAX_D 512
template <typename T>
__global__ void qk_norm_rope_store_kernel(const float* __restrict__ qkv, const float* __restrict__ qw,
                                          const float* __restrict__ kw, float eps,
                                          const float* __restrict__ inv_freq, int rot,
                                          const int* __restrict__ rope_pos,
                                          const int* __restrict__ cache_pos,
                                          const int* __restrict__ tok_seq,
                                          const int* __restrict__ block_table, int bt_stride,
                                          T* __restrict__ q_out, T* __restrict__ kcache,
                                          T* __restrict__ vcache, int nq, int nkv, int d, int layout) {
    extern __shared__ float rowbuf[];  // [warps][d]
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int n = blockIdx.x;
    const int head = blockIdx.y * (blockDim.x >> 5) + warp;
    const int nheads = nq + 2 * nkv;
    if (head >= nheads) return;
    float* x = rowbuf + warp * d;
    const float* src = qkv + ((size_t)n * nheads + head) * d;
    for (int e = lane; e < d; e += 32) x[e] = src[e];
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
        const float pos = (float)rope_pos[n];
        for (int i = lane; i < half; i += 32) {
            const float ang = pos * inv_freq[i];
            float s, c;
            sincosf(ang, &s, &c);
            const float a = x[i], b = x[i + half];
            x[i] = a * c - b * s;
            x[i + half] = a * s + b * c;
        }
        __syncwarp();
    }
    if (is_q) {
        T* dst = q_out + ((size_t)n * nq + head) * d;
        for (int e = lane; e < d; e += 32) dst[e] = from_f32<T>(x[e]);
    } else {
        const int kvh = is_k ? head - nq : head - nq - nkv;
        const int cp = cache_pos[n];
        const int page = block_table[(size_t)tok_seq[n] * bt_stride + cp / LUMEN_PAGE];
        T* tile = (is_k ? kcache : vcache) + ((size_t)page * nkv + kvh) * LUMEN_PAGE * d;
        const int r = cp % LUMEN_PAGE;
        for (int e = lane; e < d; e += 32) tile[tile_offset(layout, r, e, d)] = from_f32<T>(x[e]);
    }
}

LUMEN_API int lumen_qk_norm_rope_store(const float* qkv, const float* qw, const float* kw, float eps,
                                       const float* inv_freq, int rot, const int* rope_pos,
                                       const int* cache_pos, const int* tok_seq,
                                       const int* block_table, int bt_stride, void* q_out,
                                       void* kcache, void* vcache, int is_bf16, int N, int nq,
                                       int nkv, int d, int layout, cudaStream_t stream) {
    if (N <= 0) return 0;
    if (d <= 0 || d > QKR_MAX_D || (d & 1) || rot < 0 || rot > d || (rot & 1) || nq < 0 || nkv < 0)
        return LUMEN_ERR_UNSUPPORTED;
    if (layout == LUMEN_LAYOUT_SW128 && (!is_bf16 || d % 64 != 0)) return LUMEN_ERR_UNSUPPORTED;
    if (layout != LUMEN_LAYOUT_SW128 && layout != LUMEN_LAYOUT_LINEAR) return LUMEN_ERR_BAD_ARGUMENT;
    const int warps = 4;
    const int nheads = nq + 2 * nkv;
    if (nheads == 0) return 0;
    dim3 grid(N, (nheads + warps - 1) / warps);
    const size_t smem = (size_t)warps * d * sizeof(float);
    if (is_bf16)
        qk_norm_rope_store_kernel<__nv_bfloat16><<<grid, warps * 32, smem, stream>>>(
            qkv, qw, kw, eps, inv_freq, rot, rope_pos, cache_pos, tok_seq, block_table, bt_stride,
            (__nv_bfloat16*)q_out, (__nv_bfloat16*)kcache, (__nv_bfloat16*)vcache, nq, nkv, d, layout);
    else
        qk_norm_rope_store_kernel<float><<<grid, warps * 32, smem, stream>>>(
            qkv, qw, kw, eps, inv_freq, rot, rope_pos, cache_pos, tok_seq, block_table, bt_stride,
            (float*)q_out, (float*)kcache, (float*)vcache, nq, nkv, d, layout);
    LUMEN_LAUNCH_CHECK();
    return 0;
}
