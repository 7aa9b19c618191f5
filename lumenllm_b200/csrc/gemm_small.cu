// Matrix product for a handful of rows (decode): out[m, n] = sum_k x[m, k] W[n, k], M <= 16,
// W bfloat16 [N, K] row-major, float32 accumulation and output.
//
// With so few rows the product is a stream over the weights, and the kernel is shaped for
// HBM: every weight is read exactly once, with 16-byte loads that cover whole 128-byte
// lines, straight into the registers that feed the tensor cores, several loads in flight per
// lane. A warp owns 16 rows of W; the weights are the A operand of mma.sync m16n8k16 and the
// (transposed) activations the B operand, so the 8 columns of an mma are 8 batch rows. A lane
// loads 8 consecutive k of its two rows at once; which of the 16 k-slots of an mma an element
// lands in does not matter as long as the activations use the same assignment, which they do
// (see the loop). Activations are staged once per block in shared memory as bfloat16; the
// staging can apply SiLU(gate) * up on the fly, which removes a kernel and its traffic from
// the feed-forward.
//
// The k range is split over blockIdx.y (N alone seldom gives enough blocks to fill 148 SMs);
// each split writes its own partial [S, M, N], and the consumer adds the S partials in rising
// order. S depends on (N, K) only, never on M, so a row's result is the same in any batch.
#include <type_traits>
#include "common.cuh"
#include "mma_utils.cuh"

#define GS_WARPS 8
#define GS_THREADS (GS_WARPS * 32)
#define GS_ROWS (GS_WARPS * 16)   // rows of W per block
#define GS_UNROLL 4               // 64-wide k chunks in flight per warp
#define GS_SLOTS 296              // blocks that run at a time: two on each of 148 SMs
#define GS_UNIT 32                // k slices are cut in units of 32 values (64 bytes)

// First k of slice s of S: the units of K dealt out evenly, so slices differ by one unit at most.
__host__ __device__ __forceinline__ int gs_slice_begin(int s, int S, int K) {
    const int units = (K + GS_UNIT - 1) / GS_UNIT;
    const int k = (int)(((long long)s * units) / S) * GS_UNIT;
    return k < K ? k : K;
}

__device__ __forceinline__ uint4 ldg_stream(const void* p) {
    uint4 v;
    asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
                 : "l"(p));
    return v;
}
__device__ __forceinline__ uint32_t u4_get(const uint4& v, int j) {
    return j == 0 ? v.x : (j == 1 ? v.y : (j == 2 ? v.z : v.w));
}

// How the activations of a block's k-slice reach shared memory.
//   MODE 0: x is bfloat16 [M, K].
//   MODE 1: x is float32 [XS, M, 2K], XS partial sums of gate | up (added in rising order);
//           the staged value is silu(gate) * up.
//   MODE 2: as MODE 1, but gate_i and up_i alternate: columns 2i and 2i + 1.
template <int MODE>
__device__ __forceinline__ void stage_x(const void* x, int XS, __nv_bfloat16* xs, int M, int MP, int K,
                                        int k0, int klen, int xstride) {
    const int n8 = klen >> 3;   // 8-value groups per row
    for (int idx = threadIdx.x; idx < MP * n8; idx += GS_THREADS) {
        const int m = idx / n8, c = idx - m * n8;
        uint4 v = make_uint4(0u, 0u, 0u, 0u);
        if (m < M) {
            if (MODE == 0) {
                v = *reinterpret_cast<const uint4*>((const __nv_bfloat16*)x + (size_t)m * K + k0 + 8 * c);
            } else if (MODE == 2) {
                const float* src = (const float*)x + (size_t)m * 2 * K + 2 * (k0 + 8 * c);
                float4 q[4];
#pragma unroll
                for (int i = 0; i < 4; ++i) q[i] = *reinterpret_cast<const float4*>(src + 4 * i);
                for (int s = 1; s < XS; ++s) {
                    const size_t o = (size_t)s * M * 2 * K;
#pragma unroll
                    for (int i = 0; i < 4; ++i) {
                        const float4 a = *reinterpret_cast<const float4*>(src + o + 4 * i);
                        q[i].x += a.x; q[i].y += a.y; q[i].z += a.z; q[i].w += a.w;
                    }
                }
                auto f = [](float a, float b) { return a / (1.0f + expf(-a)) * b; };
                v.x = pack_bf16(f(q[0].x, q[0].y), f(q[0].z, q[0].w));
                v.y = pack_bf16(f(q[1].x, q[1].y), f(q[1].z, q[1].w));
                v.z = pack_bf16(f(q[2].x, q[2].y), f(q[2].z, q[2].w));
                v.w = pack_bf16(f(q[3].x, q[3].y), f(q[3].z, q[3].w));
            } else {
                const float* g = (const float*)x + (size_t)m * 2 * K + k0 + 8 * c;
                const float* u = g + K;
                float4 g0 = *reinterpret_cast<const float4*>(g), g1 = *reinterpret_cast<const float4*>(g + 4);
                float4 u0 = *reinterpret_cast<const float4*>(u), u1 = *reinterpret_cast<const float4*>(u + 4);
                for (int s = 1; s < XS; ++s) {
                    const size_t o = (size_t)s * M * 2 * K;
                    const float4 a0 = *reinterpret_cast<const float4*>(g + o), a1 = *reinterpret_cast<const float4*>(g + o + 4);
                    const float4 b0 = *reinterpret_cast<const float4*>(u + o), b1 = *reinterpret_cast<const float4*>(u + o + 4);
                    g0.x += a0.x; g0.y += a0.y; g0.z += a0.z; g0.w += a0.w;
                    g1.x += a1.x; g1.y += a1.y; g1.z += a1.z; g1.w += a1.w;
                    u0.x += b0.x; u0.y += b0.y; u0.z += b0.z; u0.w += b0.w;
                    u1.x += b1.x; u1.y += b1.y; u1.z += b1.z; u1.w += b1.w;
                }
                auto f = [](float a, float b) { return a / (1.0f + expf(-a)) * b; };
                v.x = pack_bf16(f(g0.x, u0.x), f(g0.y, u0.y));
                v.y = pack_bf16(f(g0.z, u0.z), f(g0.w, u0.w));
                v.z = pack_bf16(f(g1.x, u1.x), f(g1.y, u1.y));
                v.w = pack_bf16(f(g1.z, u1.z), f(g1.w, u1.w));
            }
        }
        *reinterpret_cast<uint4*>(xs + (size_t)m * xstride + 8 * c) = v;
    }
}

template <int NT, int MODE>   // NT: n-tiles of 8 batch rows (M <= 8 NT)
__global__ void __launch_bounds__(GS_THREADS)
gemm_small_kernel(const void* __restrict__ x, const __nv_bfloat16* __restrict__ W,
                  float* __restrict__ out, int M, int N, int K, int S, int XS) {
    extern __shared__ __align__(16) unsigned char smem_raw[];
    __nv_bfloat16* xs = reinterpret_cast<__nv_bfloat16*>(smem_raw);
    const int k0 = gs_slice_begin(blockIdx.y, S, K);
    const int klen = gs_slice_begin(blockIdx.y + 1, S, K) - k0;   // a multiple of 32 except at the end of K
    const int kpad = (klen + 63) & ~63;
    const int xstride = kpad + 32;                 // +64 bytes: rows 16 banks apart, no conflicts
    constexpr int MP = 8 * NT;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int g = lane >> 2, t = lane & 3;
    const int n0 = blockIdx.x * GS_ROWS + warp * 16;
    const int r0 = n0 + g, r1 = n0 + g + 8;
    const bool ok0 = r0 < N, ok1 = r1 < N;
    const __nv_bfloat16* w0 = W + (size_t)(ok0 ? r0 : 0) * K + k0 + 8 * t;
    const __nv_bfloat16* w1 = W + (size_t)(ok1 ? r1 : 0) * K + k0 + 8 * t;
    const int nchunks = kpad >> 6;
    const uint4 zero = make_uint4(0u, 0u, 0u, 0u);
    // The loads in flight are held in two halves that take turns: while one half's values feed
    // the tensor cores, the other half's loads are still on their way, and a half is requested
    // again as soon as it has been used, so the stream over the weights never pauses.
    constexpr int HALF = GS_UNROLL / 2;
    uint4 a[2][HALF][4];
    // a chunk's two halves: k in [kc + 8t, +8) and [kc + 32 + 8t, +8)
    auto load_half = [&](auto hsel, int cb) {
        constexpr int h = decltype(hsel)::value;
#pragma unroll
        for (int u = 0; u < HALF; ++u) {
            const int kc = (cb + u) << 6;
            const bool in_lo = (cb + u) < nchunks && kc + 8 * t + 8 <= klen;
            const bool in_hi = (cb + u) < nchunks && kc + 32 + 8 * t + 8 <= klen;
            a[h][u][0] = (ok0 && in_lo) ? ldg_stream(w0 + kc) : zero;
            a[h][u][1] = (ok1 && in_lo) ? ldg_stream(w1 + kc) : zero;
            a[h][u][2] = (ok0 && in_hi) ? ldg_stream(w0 + kc + 32) : zero;
            a[h][u][3] = (ok1 && in_hi) ? ldg_stream(w1 + kc + 32) : zero;
        }
    };
    using H0 = std::integral_constant<int, 0>;
    using H1 = std::integral_constant<int, 1>;
    // Weights never change: the first loads are on their way before the kernel ahead of this
    // one in the stream has finished. Activations and outputs come after the wait.
    load_half(H0{}, 0);
    load_half(H1{}, HALF);
    pdl_wait();
    pdl_trigger();

    // zero the padding of the last chunk, then stage
    if (kpad != klen)
        for (int idx = threadIdx.x; idx < MP * (kpad - klen); idx += GS_THREADS) {
            const int m = idx / (kpad - klen), c = idx - m * (kpad - klen);
            xs[(size_t)m * xstride + klen + c] = __float2bfloat16_rn(0.0f);
        }
    stage_x<MODE>(x, XS, xs, M, MP, K, k0, klen, xstride);
    __syncthreads();
    if (n0 >= N) return;

    float c[NT][4];
#pragma unroll
    for (int nt = 0; nt < NT; ++nt) c[nt][0] = c[nt][1] = c[nt][2] = c[nt][3] = 0.0f;
    auto use_half = [&](auto hsel, int cb) {
        constexpr int h = decltype(hsel)::value;
#pragma unroll
        for (int u = 0; u < HALF; ++u) {
            if (cb + u >= nchunks) break;
            const int kc = (cb + u) << 6;
#pragma unroll
            for (int nt = 0; nt < NT; ++nt) {
                // activations of batch row 8 nt + g, the same 8 + 8 values of k as the weights
                const __nv_bfloat16* xr = xs + (size_t)(8 * nt + g) * xstride + kc + 8 * t;
                const uint4 xlo = *reinterpret_cast<const uint4*>(xr);
                const uint4 xhi = *reinterpret_cast<const uint4*>(xr + 32);
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    // mma k-slots (2t, 2t+1) carry k = kc + 8t + 2j (+1); slots (2t+8, 2t+9)
                    // carry k = kc + 32 + 8t + 2j (+1), for A and B alike
                    const uint32_t af[4] = {u4_get(a[h][u][0], j), u4_get(a[h][u][1], j), u4_get(a[h][u][2], j),
                                            u4_get(a[h][u][3], j)};
                    mma_bf16(c[nt], af, u4_get(xlo, j), u4_get(xhi, j));
                }
            }
        }
    };
    for (int cb = 0; cb < nchunks; cb += GS_UNROLL) {
        use_half(H0{}, cb);
        if (cb + GS_UNROLL < nchunks) load_half(H0{}, cb + GS_UNROLL);
        use_half(H1{}, cb + HALF);
        if (cb + GS_UNROLL + HALF < nchunks) load_half(H1{}, cb + GS_UNROLL + HALF);
    }
    // c[nt][0..1]: W row r0, batch rows 8nt + 2t, +1; c[nt][2..3]: W row r1.
    float* o = out + (size_t)blockIdx.y * M * N;
#pragma unroll
    for (int nt = 0; nt < NT; ++nt) {
#pragma unroll
        for (int i = 0; i < 2; ++i) {
            const int m = 8 * nt + 2 * t + i;
            if (m < M) {
                if (ok0) o[(size_t)m * N + r0] = c[nt][i];
                if (ok1) o[(size_t)m * N + r1] = c[nt][2 + i];
            }
        }
    }
}

// Number of k splits for a weight of shape [N, K]. Two blocks of this kernel fit on an SM, so
// 296 run at a time; S is chosen so that the row blocks times S fill whole waves of 296 as
// nearly as possible (the smaller S on a tie), with slices no shorter than 256 and at most 8 of
// them: the kernel that adds the partial sums has eight loads in flight at a time, and a ninth
// costs it a second round trip (measured: 1.45 against 1.47 ms for 12 layers at batch 8). A
// function of (N, K) only. Slices are cut in units of 32 values (64 bytes) and differ by one unit at most.
LUMEN_API int lumen_gemm_small_splits(int N, int K) {
    const int row_blocks = (N + GS_ROWS - 1) / GS_ROWS;
    const int units = (K + GS_UNIT - 1) / GS_UNIT;
    int max_s = K / 256;
    if (max_s > 8) max_s = 8;
    if (max_s < 1) max_s = 1;
    int best = 1;
    double best_fill = 0.0;
    for (int s = 1; s <= max_s; ++s) {
        const int blocks = row_blocks * s;
        const int waves = (blocks + GS_SLOTS - 1) / GS_SLOTS;
        // the longest slice against the mean one: uneven cuts cost as empty slots do
        const int longest = (units + s - 1) / s;
        const double fill = (double)blocks / (waves * GS_SLOTS) * ((double)units / s) / longest;
        if (fill > best_fill + 0.02) { best_fill = fill; best = s; }
    }
    return best;
}
// x: mode 0 bfloat16 [M, K]; mode 1 float32 [x_splits, M, 2K] (partials of gate | up;
// SiLU(gate)*up is applied to their sum); mode 2 the same with gate_i, up_i in columns
// 2i, 2i + 1. out: float32 [S, M, N] with
// S = lumen_gemm_small_splits(N, K).
LUMEN_API int lumen_gemm_small(const void* x, int mode, int x_splits, const void* W, float* out, int M,
                               int N, int K, cudaStream_t stream) {
    if (M <= 0 || N <= 0) return 0;
    if (M > 16 || K <= 0 || (K & 7) || mode < 0 || mode > 2 || x_splits < 1) return LUMEN_ERR_UNSUPPORTED;
    const int S = lumen_gemm_small_splits(N, K);
    const int slice = (((K + GS_UNIT - 1) / GS_UNIT + S - 1) / S * GS_UNIT + 63) & ~63;   // the longest, padded
    const int NT = (M + 7) / 8;
    const size_t smem = (size_t)(8 * NT) * (slice + 32) * 2;
    if (smem > 200 * 1024) return LUMEN_ERR_UNSUPPORTED;
    dim3 grid((N + GS_ROWS - 1) / GS_ROWS, S);
    const __nv_bfloat16* Wp = (const __nv_bfloat16*)W;
#define GS_LAUNCH(NT_, MODE_)                                                                      \
    do {                                                                                           \
        auto k = gemm_small_kernel<NT_, MODE_>;                                                    \
        if (smem > 48 * 1024)                                                                      \
            cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);       \
        lumen_launch(k, dim3(grid), dim3(GS_THREADS), smem, stream, x, Wp, out, M, N, K, S, x_splits);               \
    } while (0)
    if (NT == 1 && mode == 0) GS_LAUNCH(1, 0);
    else if (NT == 1 && mode == 1) GS_LAUNCH(1, 1);
    else if (NT == 1) GS_LAUNCH(1, 2);
    else if (mode == 0) GS_LAUNCH(2, 0);
    else if (mode == 1) GS_LAUNCH(2, 1);
    else GS_LAUNCH(2, 2);
#undef GS_LAUNCH
    LUMEN_LAUNCH_CHECK();
    return 0;
}
