// General causal attention over the paged cache, for any number of new tokens
// per sequence (whole prompts and single decoded tokens alike), any head size
// that is a multiple of 16 up to 256, any number of heads and groups, with an
// optional window. All arithmetic is float32 with the precise expf. It is the
// attention of the 32-bit path and the plain device reference of the faster
// bfloat16 kernels.
//
// One block per (query token, query head). Keys are walked in chunks of 128
// whose boundaries are multiples of 128 in absolute position, so the order of
// every sum depends only on the query's own position: the result for a token
// is the same bit for bit whether it came in a prompt, alone, or in any batch.
#include "common.cuh"

#define AG_THREADS 128
#define AG_MAX_D 256

template <typename T>
__global__ void __launch_bounds__(AG_THREADS)
attn_generic_kernel(const T* __restrict__ q, const T* __restrict__ kcache, const T* __restrict__ vcache,
                    const int* __restrict__ block_table, int bt_stride,
                    const int* __restrict__ tok_seq, const int* __restrict__ tok_pos,
                    T* __restrict__ out, int nq, int nkv, int d, int window, float scale,
                    int layout) {
    pdl_wait();      // nothing of this kernel touches global memory before this
    pdl_trigger();
    __shared__ float qs[AG_MAX_D];
    __shared__ float ps[AG_THREADS];
    __shared__ float red[32];
    const int head = blockIdx.y, n = blockIdx.x, tid = threadIdx.x;
    const int kvh = head / (nq / nkv);
    const int p = tok_pos[n];
    const int* bt = block_table + (size_t)tok_seq[n] * bt_stride;
    const T* qrow = q + ((size_t)n * nq + head) * d;
    for (int e = tid; e < d; e += AG_THREADS) qs[e] = to_f32(qrow[e]);
    __syncthreads();

    int lo = 0;
    if (window > 0 && p - window + 1 > 0) lo = p - window + 1;
    float m = -INFINITY, l = 0.0f;
    float acc0 = 0.0f, acc1 = 0.0f;  // dims tid and tid + 128

    for (int c = lo / AG_THREADS; c <= p / AG_THREADS; ++c) {
        const int j = c * AG_THREADS + tid;
        const bool valid = (j >= lo) && (j <= p);
        float s = -INFINITY;
        if (valid) {
            const int page = bt[j / LUMEN_PAGE];
            const T* ktile = kcache + ((size_t)page * nkv + kvh) * LUMEN_PAGE * d;
            const int r = j % LUMEN_PAGE;
            float dot = 0.0f;
            for (int e = 0; e < d; ++e) dot = fmaf(qs[e], to_f32(ktile[tile_offset(layout, r, e, d)]), dot);
            s = dot * scale;
        }
        const float cm = block_max(s, red);
        const float m_new = fmaxf(m, cm);
        const float pj = valid ? expf(s - m_new) : 0.0f;
        const float corr = (m == -INFINITY) ? 0.0f : expf(m - m_new);
        __syncthreads();
        ps[tid] = pj;
        const float csum = block_sum(pj, red);  // has a __syncthreads before reading ps below
        l = l * corr + csum;
        acc0 *= corr;
        acc1 *= corr;
        __syncthreads();
        const int jbeg = max(c * AG_THREADS, lo), jend = min(c * AG_THREADS + AG_THREADS - 1, p);
        for (int jj = jbeg; jj <= jend; ++jj) {
            const int page = bt[jj / LUMEN_PAGE];
            const T* vtile = vcache + ((size_t)page * nkv + kvh) * LUMEN_PAGE * d;
            const int r = jj % LUMEN_PAGE;
            const float w = ps[jj - c * AG_THREADS];
            if (tid < d) acc0 = fmaf(w, to_f32(vtile[tile_offset(layout, r, tid, d)]), acc0);
            if (tid + AG_THREADS < d)
                acc1 = fmaf(w, to_f32(vtile[tile_offset(layout, r, tid + AG_THREADS, d)]), acc1);
        }
        m = m_new;
        __syncthreads();
    }
    T* orow = out + ((size_t)n * nq + head) * d;
    const float inv = 1.0f / l;
    if (tid < d) orow[tid] = from_f32<T>(acc0 * inv);
    if (tid + AG_THREADS < d) orow[tid + AG_THREADS] = from_f32<T>(acc1 * inv);
}

LUMEN_API int lumen_attn_generic(const void* q, const void* kcache, const void* vcache,
                                 const int* block_table, int bt_stride, const int* tok_seq,
                                 const int* tok_pos, void* out, int is_bf16, int N, int nq, int nkv,
                                 int d, int window, float scale, int layout, cudaStream_t stream) {
    if (N <= 0) return 0;
    if (d <= 0 || d > AG_MAX_D || nq <= 0 || nkv <= 0 || nq % nkv != 0 || window < 0)
        return LUMEN_ERR_UNSUPPORTED;
    if (nq > 65535) return LUMEN_ERR_UNSUPPORTED;
    if (layout == LUMEN_LAYOUT_SW128 && (!is_bf16 || d % 64 != 0)) return LUMEN_ERR_UNSUPPORTED;
    dim3 grid(N, nq);
    if (is_bf16)
        lumen_launch(attn_generic_kernel<__nv_bfloat16>, dim3(grid), dim3(AG_THREADS), 0, stream, 
            (const __nv_bfloat16*)q, (const __nv_bfloat16*)kcache, (const __nv_bfloat16*)vcache,
            block_table, bt_stride, tok_seq, tok_pos, (__nv_bfloat16*)out, nq, nkv, d, window, scale,
            layout);
    else
        lumen_launch(attn_generic_kernel<float>, dim3(grid), dim3(AG_THREADS), 0, stream, 
            (const float*)q, (const float*)kcache, (const float*)vcache, block_table, bt_stride,
            tok_seq, tok_pos, (float*)out, nq, nkv, d, window, scale, layout);
    LUMEN_LAUNCH_CHECK();
    return 0;
}
