// Token choice on the device: greedy argmax (equal maxima resolve to the lowest
// index) and the sampler temperature -> top-k -> top-p -> min-p -> draw over the
// WHOLE vocabulary, with the uniform number u supplied by the host.
//
// The sampler never sorts. In the order "larger logit first, equal logits by
// rising index" every filter keeps a prefix, so the kept set is described by a
// pair (threshold key, number of threshold ties kept), and both "the k-th
// element" and "the element at which the running weight reaches x" are found
// by a 4-level radix descent over the 32-bit ordered keys. Weights are summed
// as 2^-40 fixed-point integers, so every sum is exact and independent of the
// order in which threads add: the same logits, options and u give the same
// token in any batch.
#include "common.cuh"

#define SM_THREADS 1024
#define FX_ONE 1099511627776.0  // 2^40

typedef unsigned long long u64;

__device__ __forceinline__ bool finite_f(float x) { return fabsf(x) <= 3.402823466e38f; }

// Monotone map float -> unsigned: a < b  <=>  key(a) < key(b); -0 and +0 coincide.
__device__ __forceinline__ unsigned okey(float x) {
    unsigned b = __float_as_uint(x);
    if ((b << 1) == 0u) b = 0u;
    return (b & 0x80000000u) ? ~b : (b | 0x80000000u);
}
__device__ __forceinline__ float key_to_float(unsigned k) {
    unsigned b = (k & 0x80000000u) ? (k & 0x7fffffffu) : ~k;
    return __uint_as_float(b);
}
__device__ __forceinline__ float weight_f(float logit, float mx, float temp) {
    return expf((logit - mx) / temp);
}
__device__ __forceinline__ u64 weight_fx(float logit, float mx, float temp) {
    const float w = weight_f(logit, mx, temp);
    if (!(w > 0.0f) || !finite_f(w)) return 0ull;
    return (u64)((double)w * FX_ONE);
}

struct Prefix {       // kept set: keys > thr, plus the first `ties` (by index) of key == thr
    unsigned thr;
    unsigned ties;
    int all;          // 1: every finite element
};

struct Shared {
    u64 hist[256];
    float redf[32];
    int redi[32];
    unsigned redu[32];
    u64 red64[32];
    unsigned sel_key;
    u64 sel_before;
    u64 sel_bin;
    u64 total;
    int scan[SM_THREADS / 32];
    int found;
};

__device__ u64 block_sum_u64(u64 v, Shared& sh) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    __syncthreads();
    if (lane == 0) sh.red64[warp] = v;
    __syncthreads();
    u64 t = (lane < (int)(blockDim.x >> 5)) ? sh.red64[lane] : 0ull;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) t += __shfl_xor_sync(0xffffffffu, t, o);
    return t;
}

// amount(P): sum of weights (MASS) or count of the kept set.
template <bool MASS>
__device__ u64 prefix_amount(const float* lg, int V, float mx, float temp, Prefix P, Shared& sh) {
    u64 a = 0;
    for (int i = threadIdx.x; i < V; i += blockDim.x) {
        const float x = lg[i];
        if (!finite_f(x)) continue;
        if (!P.all && okey(x) <= P.thr) continue;
        a += MASS ? weight_fx(x, mx, temp) : 1ull;
    }
    a = block_sum_u64(a, sh);
    if (!P.all) a += (u64)P.ties * (MASS ? weight_fx(key_to_float(P.thr), mx, temp) : 1ull);
    return a;
}

// Within the kept set P, walking in rank order, finds the key K at which the
// running amount first reaches `target` (1 <= target <= amount(P)). Returns K,
// and through `ties_needed` how many elements of key K (by rising index) the
// prefix ending there holds.
template <bool MASS>
__device__ unsigned radix_select(const float* lg, int V, float mx, float temp, Prefix P, u64 target,
                                 unsigned* ties_needed, Shared& sh) {
    unsigned cur = 0;
    u64 before = 0;
    for (int level = 0; level < 4; ++level) {
        const int shift = 24 - 8 * level;
        const unsigned above = (level == 0) ? 0u : (0xffffffffu << (shift + 8));
        for (int b = threadIdx.x; b < 256; b += blockDim.x) sh.hist[b] = 0ull;
        __syncthreads();
        for (int i = threadIdx.x; i < V; i += blockDim.x) {
            const float x = lg[i];
            if (!finite_f(x)) continue;
            const unsigned k = okey(x);
            if ((k ^ cur) & above) continue;
            if (!P.all && k <= P.thr) continue;
            const u64 amt = MASS ? weight_fx(x, mx, temp) : 1ull;
            if (amt) atomicAdd(&sh.hist[(k >> shift) & 255u], amt);
        }
        __syncthreads();
        if (threadIdx.x == 0) {
            if (!P.all && !((P.thr ^ cur) & above)) {
                const u64 unit = MASS ? weight_fx(key_to_float(P.thr), mx, temp) : 1ull;
                sh.hist[(P.thr >> shift) & 255u] += (u64)P.ties * unit;
            }
            u64 acc = before;
            int digit = -1, lowest = 0;
            for (int b = 255; b >= 0; --b) {
                const u64 hb = sh.hist[b];
                if (hb) lowest = b;
                if (acc + hb >= target && hb) { digit = b; break; }
                acc += hb;
            }
            if (digit < 0) {  // target beyond the total: end at the last element
                digit = lowest;
                acc = acc - sh.hist[lowest];
            }
            sh.sel_key = cur | ((unsigned)digit << shift);
            sh.sel_before = acc;
            sh.sel_bin = sh.hist[digit];
        }
        __syncthreads();
        cur = sh.sel_key;
        before = sh.sel_before;
        __syncthreads();
    }
    const u64 bin = sh.sel_bin;
    const u64 unit = MASS ? weight_fx(key_to_float(cur), mx, temp) : 1ull;
    u64 have = unit ? bin / unit : 1ull;
    if (have < 1) have = 1;
    u64 need = (target > before) ? (target - before) : 1ull;
    need = unit ? (need + unit - 1) / unit : 1ull;
    if (need < 1) need = 1;
    if (need > have) need = have;
    *ties_needed = (unsigned)need;
    return cur;
}

// Index of the n-th (1-based, rising index) element whose key equals `key`.
__device__ int nth_equal(const float* lg, int V, unsigned key, unsigned n, Shared& sh) {
    const int chunk = (V + blockDim.x - 1) / blockDim.x;
    const int beg = threadIdx.x * chunk, end = min(beg + chunk, V);
    int cnt = 0;
    for (int i = beg; i < end; ++i) {
        const float x = lg[i];
        if (finite_f(x) && okey(x) == key) ++cnt;
    }
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    int inc = cnt;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
        const int t = __shfl_up_sync(0xffffffffu, inc, o);
        if (lane >= o) inc += t;
    }
    if (threadIdx.x == 0) sh.found = -1;
    __syncthreads();
    if (lane == 31) sh.scan[warp] = inc;
    __syncthreads();
    int offset = 0;
    for (int w = 0; w < warp; ++w) offset += sh.scan[w];
    const int excl = offset + inc - cnt;
    if ((unsigned)excl < n && n <= (unsigned)(excl + cnt)) {
        int seen = excl;
        for (int i = beg; i < end; ++i) {
            const float x = lg[i];
            if (finite_f(x) && okey(x) == key) {
                if ((unsigned)++seen == n) { sh.found = i; break; }
            }
        }
    }
    __syncthreads();
    return sh.found;
}

// Largest value and its lowest index. NaN never wins; if nothing compares, 0.
__device__ void block_argmax(const float* lg, int V, float* out_v, int* out_i, Shared& sh) {
    float bv = -INFINITY;
    int bi = 0x7fffffff;
    for (int i = threadIdx.x; i < V; i += blockDim.x) {
        const float x = lg[i];
        if (x > bv || (x == bv && i < bi)) { bv = x; bi = i; }
    }
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        const float ov = __shfl_xor_sync(0xffffffffu, bv, o);
        const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
        if (ov > bv || (ov == bv && oi < bi)) { bv = ov; bi = oi; }
    }
    __syncthreads();
    if (lane == 0) { sh.redf[warp] = bv; sh.redi[warp] = bi; }
    __syncthreads();
    bv = (lane < (int)(blockDim.x >> 5)) ? sh.redf[lane] : -INFINITY;
    bi = (lane < (int)(blockDim.x >> 5)) ? sh.redi[lane] : 0x7fffffff;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        const float ov = __shfl_xor_sync(0xffffffffu, bv, o);
        const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
        if (ov > bv || (ov == bv && oi < bi)) { bv = ov; bi = oi; }
    }
    if (bi == 0x7fffffff) bi = 0;
    *out_v = bv;
    *out_i = bi;
}

__global__ void __launch_bounds__(SM_THREADS)
argmax_kernel(const float* __restrict__ logits, long long row_stride, int V, int* __restrict__ out) {
    pdl_wait();      // nothing of this kernel touches global memory before this
    pdl_trigger();
    __shared__ Shared sh;
    float v;
    int i;
    block_argmax(logits + (size_t)blockIdx.x * row_stride, V, &v, &i, sh);
    if (threadIdx.x == 0) out[blockIdx.x] = i;
}

// Two-stage argmax for long rows: AM_SLICES blocks per row each reduce a slice, a small
// second kernel reduces the slices in rising order (so equal maxima still resolve to the
// lowest index).
#define AM_SLICES 64
__global__ void __launch_bounds__(256)
argmax_slices_kernel(const float* __restrict__ logits, long long row_stride, int V,
                     float* __restrict__ part_v, int* __restrict__ part_i) {
    pdl_wait();      // nothing of this kernel touches global memory before this
    pdl_trigger();
    __shared__ float sv[8];
    __shared__ int si[8];
    const int row = blockIdx.y, slice = blockIdx.x;
    const float* lg = logits + (size_t)row * row_stride;
    const int per = (V + AM_SLICES - 1) / AM_SLICES;
    const int beg = slice * per, end = min(beg + per, V);
    float bv = -INFINITY;
    int bi = 0x7fffffff;
    for (int i = beg + threadIdx.x; i < end; i += blockDim.x) {
        const float x = lg[i];
        if (x > bv || (x == bv && i < bi)) { bv = x; bi = i; }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        const float ov = __shfl_xor_sync(0xffffffffu, bv, o);
        const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
        if (ov > bv || (ov == bv && oi < bi)) { bv = ov; bi = oi; }
    }
    if ((threadIdx.x & 31) == 0) { sv[threadIdx.x >> 5] = bv; si[threadIdx.x >> 5] = bi; }
    __syncthreads();
    if (threadIdx.x == 0) {
        for (int w = 1; w < 8; ++w)
            if (sv[w] > bv || (sv[w] == bv && si[w] < bi)) { bv = sv[w]; bi = si[w]; }
        part_v[row * AM_SLICES + slice] = bv;
        part_i[row * AM_SLICES + slice] = bi;
    }
}
__global__ void argmax_final_kernel(const float* __restrict__ part_v, const int* __restrict__ part_i,
                                    int* __restrict__ out) {
    pdl_wait();      // nothing of this kernel touches global memory before this
    pdl_trigger();
    const int row = blockIdx.x, lane = threadIdx.x;   // 32 threads
    float bv = -INFINITY;
    int bi = 0x7fffffff;
    for (int s = lane; s < AM_SLICES; s += 32) {
        const float v = part_v[row * AM_SLICES + s];
        const int i = part_i[row * AM_SLICES + s];
        if (v > bv || (v == bv && i < bi)) { bv = v; bi = i; }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        const float ov = __shfl_xor_sync(0xffffffffu, bv, o);
        const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
        if (ov > bv || (ov == bv && oi < bi)) { bv = ov; bi = oi; }
    }
    if (lane == 0) out[row] = (bi == 0x7fffffff) ? 0 : bi;
}

// opts: per row (temperature, top_p, min_p, u); top_k: per row.
__global__ void __launch_bounds__(SM_THREADS)
sample_kernel(const float* __restrict__ logits, long long row_stride, int V,
              const float* __restrict__ opts, const int* __restrict__ top_k_arr,
              int* __restrict__ out) {
    pdl_wait();      // nothing of this kernel touches global memory before this
    pdl_trigger();
    __shared__ Shared sh;
    const float* lg = logits + (size_t)blockIdx.x * row_stride;
    const float temperature = opts[blockIdx.x * 4 + 0];
    const float top_p = opts[blockIdx.x * 4 + 1];
    const float min_p = opts[blockIdx.x * 4 + 2];
    const float u = opts[blockIdx.x * 4 + 3];
    const int top_k = top_k_arr[blockIdx.x];

    float amax_v;
    int amax_i;
    block_argmax(lg, V, &amax_v, &amax_i, sh);
    int result = amax_i;
    if (temperature <= 0.0f || top_k == 1) {
        if (threadIdx.x == 0) out[blockIdx.x] = result;
        return;
    }
    const float temp = fmaxf(temperature, 1e-6f);

    // Largest finite logit (the argmax may be +inf, which the sampler leaves out).
    float mx = -INFINITY;
    for (int i = threadIdx.x; i < V; i += blockDim.x) {
        const float x = lg[i];
        if (finite_f(x)) mx = fmaxf(mx, x);
    }
    mx = block_max(mx, sh.redf);
    __syncthreads();
    if (mx == -INFINITY) {  // nothing finite
        if (threadIdx.x == 0) out[blockIdx.x] = result;
        return;
    }

    Prefix P;
    P.all = 1; P.thr = 0; P.ties = 0;
    if (top_k > 0) {
        const u64 n_valid = prefix_amount<false>(lg, V, mx, temp, P, sh);
        if ((u64)top_k < n_valid) {
            unsigned ties;
            const unsigned k = radix_select<false>(lg, V, mx, temp, P, (u64)top_k, &ties, sh);
            P.all = 0; P.thr = k; P.ties = ties;
        }
    }
    u64 total = prefix_amount<true>(lg, V, mx, temp, P, sh);
    if (total == 0ull) {
        if (threadIdx.x == 0) out[blockIdx.x] = result;
        return;
    }
    if (top_p > 0.0f && top_p < 1.0f) {
        u64 cutoff = (u64)ceil((double)total * (double)top_p);
        if (cutoff < 1) cutoff = 1;
        if (cutoff > total) cutoff = total;
        unsigned ties;
        const unsigned k = radix_select<true>(lg, V, mx, temp, P, cutoff, &ties, sh);
        P.all = 0; P.thr = k; P.ties = ties;
    }
    if (min_p > 0.0f) {
        // The largest weight is exp(0) = 1, so the rule is w >= min_p.
        unsigned lowest = 0xffffffffu;
        for (int i = threadIdx.x; i < V; i += blockDim.x) {
            const float x = lg[i];
            if (!finite_f(x)) continue;
            const unsigned k = okey(x);
            if (!P.all && k < P.thr) continue;
            if (weight_f(x, mx, temp) >= 1.0f * min_p) lowest = min(lowest, k);
        }
        // block min over unsigned
        const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) lowest = min(lowest, __shfl_xor_sync(0xffffffffu, lowest, o));
        __syncthreads();
        if (lane == 0) sh.redu[warp] = lowest;
        __syncthreads();
        lowest = (lane < (int)(blockDim.x >> 5)) ? sh.redu[lane] : 0xffffffffu;
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) lowest = min(lowest, __shfl_xor_sync(0xffffffffu, lowest, o));
        if (lowest == 0xffffffffu) {  // min_p > 1 keeps nothing
            if (threadIdx.x == 0) out[blockIdx.x] = result;
            return;
        }
        if (P.all || lowest > P.thr) {
            // keep every element of key >= lowest: count the ties of `lowest`
            u64 c = 0;
            for (int i = threadIdx.x; i < V; i += blockDim.x) {
                const float x = lg[i];
                if (finite_f(x) && okey(x) == lowest) ++c;
            }
            c = block_sum_u64(c, sh);
            P.all = 0; P.thr = lowest; P.ties = (unsigned)c;
        }
    }
    total = prefix_amount<true>(lg, V, mx, temp, P, sh);
    if (total == 0ull) {
        if (threadIdx.x == 0) out[blockIdx.x] = result;
        return;
    }
    u64 target = (u64)ceil((double)u * (double)total);
    if (target < 1) target = 1;
    if (target > total) target = total;
    unsigned nth;
    const unsigned key = radix_select<true>(lg, V, mx, temp, P, target, &nth, sh);
    const int idx = nth_equal(lg, V, key, nth, sh);
    if (idx >= 0) result = idx;
    if (threadIdx.x == 0) out[blockIdx.x] = result;
}

// scratch: optional, 2 * 64 * B 4-byte words; with it long rows are reduced by many blocks.
LUMEN_API int lumen_argmax(const float* logits, long long row_stride, int B, int V, int* out,
                           void* scratch, cudaStream_t stream) {
    if (B <= 0) return 0;
    if (V <= 0) return LUMEN_ERR_BAD_ARGUMENT;
    if (scratch && V >= 16384 && B <= 65535) {
        float* pv = (float*)scratch;
        int* pi = (int*)scratch + (size_t)B * AM_SLICES;
        lumen_launch(argmax_slices_kernel, dim3(dim3(AM_SLICES, B)), dim3(256), 0, stream, logits, row_stride, V, pv, pi);
        LUMEN_LAUNCH_CHECK();
        lumen_launch(argmax_final_kernel, dim3(B), dim3(32), 0, stream, pv, pi, out);
    } else {
        lumen_launch(argmax_kernel, dim3(B), dim3(SM_THREADS), 0, stream, logits, row_stride, V, out);
    }
    LUMEN_LAUNCH_CHECK();
    return 0;
}

LUMEN_API int lumen_sample(const float* logits, long long row_stride, int B, int V,
                           const float* opts, const int* top_k, int* out, cudaStream_t stream) {
    if (B <= 0) return 0;
    if (V <= 0) return LUMEN_ERR_BAD_ARGUMENT;
    lumen_launch(sample_kernel, dim3(B), dim3(SM_THREADS), 0, stream, logits, row_stride, V, opts, top_k, out);
    LUMEN_LAUNCH_CHECK();
    return 0;
}
