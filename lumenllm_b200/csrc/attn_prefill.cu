// Causal grouped-query flash attention for prompts (and any step in which sequences bring
// several tokens), bfloat16, over the paged cache in its 128-byte-swizzled layout.
//
// A block takes a tile of query tokens of one sequence and ONE kv head, and serves the G
// query heads of that kv head together: its 64 rows are (token, head) pairs, so every K/V
// tile staged in shared memory is used by G heads. Keys are walked page by page (64 keys);
// the K and V tile of a page are each one contiguous block of the cache, brought in by one
// bulk asynchronous copy each (cp.async.bulk + mbarrier) into a two-stage ring, while the
// tensor cores (mma.sync m16n8k16, bf16 in, float32 accumulate) work on the page before.
// Softmax is online, in float32, with exp2 of log2(e)-scaled scores; P is rounded to
// bfloat16 for the P V product, the row sum is taken before rounding.
//
// Sequences of a step have unequal numbers of new tokens; a block finds its sequence from
// seq_qlen. Page tiles always start at multiples of 64 in absolute position, so what a row
// computes depends only on its own position, never on the batch or on how the prompt was cut.
#include "common.cuh"
#include "mma_utils.cuh"

#define AP_THREADS 128
#define AP_ROWS 64

template <int D>
__global__ void __launch_bounds__(AP_THREADS)
attn_prefill_kernel(const __nv_bfloat16* __restrict__ q, const __nv_bfloat16* __restrict__ kcache,
                    const __nv_bfloat16* __restrict__ vcache, const int* __restrict__ block_table,
                    int bt_stride, const int* __restrict__ cu_q, const int* __restrict__ seq_start,
                    int B, __nv_bfloat16* __restrict__ out, int nq, int nkv, int window,
                    float scale_log2, int* __restrict__ err) {
    pdl_wait();      // nothing of this kernel touches global memory before this
    pdl_trigger();
    constexpr int TILE_BYTES = LUMEN_PAGE * D * 2;
    extern __shared__ __align__(1024) unsigned char smem[];   // [2 stages][K tile, V tile]
    __shared__ uint64_t full[2];

    const int G = nq / nkv;
    const int TQ = AP_ROWS / G;            // query tokens per block
    const int kvh = blockIdx.y;
    // which sequence, which tile of it
    int tile = blockIdx.x, b = 0, qlen = 0;
    for (; b < B; ++b) {
        qlen = cu_q[b + 1] - cu_q[b];
        const int nt = (qlen + TQ - 1) / TQ;
        if (tile < nt) break;
        tile -= nt;
    }
    if (b >= B) return;
    const int i0 = tile * TQ;                       // first token of the tile, within the step
    const int ntok = min(TQ, qlen - i0);
    const int n0 = cu_q[b] + i0;                    // row of that token in q / out
    const int pos0 = seq_start[b] + i0;             // its absolute position
    const int pos_last = pos0 + ntok - 1;
    int j_lo = 0;
    if (window > 0 && pos0 - window + 1 > 0) j_lo = pos0 - window + 1;
    const int pg_lo = j_lo / LUMEN_PAGE, pg_hi = pos_last / LUMEN_PAGE;
    const int* bt = block_table + (size_t)b * bt_stride;

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int g = lane >> 2, t = lane & 3;

    if (tid == 0) {
        mbar_init(&full[0], 1);
        mbar_init(&full[1], 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncthreads();
    auto issue = [&](int stage, int pg) {
        const size_t off = ((size_t)bt[pg] * nkv + kvh) * (size_t)(LUMEN_PAGE * D);
        unsigned char* dst = smem + stage * 2 * TILE_BYTES;
        mbar_expect_tx(&full[stage], 2 * TILE_BYTES);
        bulk_load(dst, kcache + off, TILE_BYTES, &full[stage]);
        bulk_load(dst + TILE_BYTES, vcache + off, TILE_BYTES, &full[stage]);
    };
    if (tid == 0) issue(0, pg_lo);

    // This thread's two rows: r0 = 16 warp + g and r1 = r0 + 8; row -> (token, head).
    const int r0 = 16 * warp + g, r1 = r0 + 8;
    const bool ok0 = r0 < ntok * G && r0 < TQ * G, ok1 = r1 < ntok * G && r1 < TQ * G;
    const int tok0 = r0 / G, tok1 = r1 / G;
    const int h0 = kvh * G + r0 % G, h1 = kvh * G + r1 % G;
    const int p0 = pos0 + tok0, p1 = pos0 + tok1;       // absolute positions of the rows
    const int lo0 = (window > 0) ? p0 - window + 1 : 0, lo1 = (window > 0) ? p1 - window + 1 : 0;

    uint32_t qa[D / 16][4];
    {
        const __nv_bfloat16* q0 = q + ((size_t)(n0 + tok0) * nq + h0) * D;
        const __nv_bfloat16* q1 = q + ((size_t)(n0 + tok1) * nq + h1) * D;
#pragma unroll
        for (int ks = 0; ks < D / 16; ++ks) {
            const int col = 16 * ks + 2 * t;
            qa[ks][0] = ok0 ? *reinterpret_cast<const uint32_t*>(q0 + col) : 0u;
            qa[ks][1] = ok1 ? *reinterpret_cast<const uint32_t*>(q1 + col) : 0u;
            qa[ks][2] = ok0 ? *reinterpret_cast<const uint32_t*>(q0 + col + 8) : 0u;
            qa[ks][3] = ok1 ? *reinterpret_cast<const uint32_t*>(q1 + col + 8) : 0u;
        }
    }

    float o[D / 8][4];
#pragma unroll
    for (int dt = 0; dt < D / 8; ++dt) o[dt][0] = o[dt][1] = o[dt][2] = o[dt][3] = 0.0f;
    float m0 = -INFINITY, m1 = -INFINITY, l0 = 0.0f, l1 = 0.0f;
    bool failed = false;

    for (int pg = pg_lo, it = 0; pg <= pg_hi; ++pg, ++it) {
        const int stage = it & 1;
        if (tid == 0 && pg + 1 <= pg_hi) issue(stage ^ 1, pg + 1);
        if (!mbar_wait(&full[stage], (it >> 1) & 1)) failed = true;
        const uint32_t ktile = smem_u32(smem + stage * 2 * TILE_BYTES);
        const uint32_t vtile = ktile + TILE_BYTES;

        float s[8][4];
#pragma unroll
        for (int nt = 0; nt < 8; ++nt) {
            s[nt][0] = s[nt][1] = s[nt][2] = s[nt][3] = 0.0f;
#pragma unroll
            for (int kp = 0; kp < D / 32; ++kp) {
                uint32_t r[4];
                ldsm_x4(r, ktile + sw_off(8 * nt + (lane & 7), 4 * kp + (lane >> 3)));
                mma_bf16(s[nt], qa[2 * kp], r[0], r[1]);
                mma_bf16(s[nt], qa[2 * kp + 1], r[2], r[3]);
            }
        }
        // scale into log2 units and mask
        const int jb = pg * LUMEN_PAGE;
        float mx0 = -INFINITY, mx1 = -INFINITY;
#pragma unroll
        for (int nt = 0; nt < 8; ++nt) {
#pragma unroll
            for (int i = 0; i < 2; ++i) {
                const int j = jb + 8 * nt + 2 * t + i;
                const bool v0 = (j <= p0) && (j >= lo0), v1 = (j <= p1) && (j >= lo1);
                s[nt][i] = v0 ? s[nt][i] * scale_log2 : -INFINITY;
                s[nt][2 + i] = v1 ? s[nt][2 + i] * scale_log2 : -INFINITY;
                mx0 = fmaxf(mx0, s[nt][i]);
                mx1 = fmaxf(mx1, s[nt][2 + i]);
            }
        }
        mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 1));
        mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 2));
        mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 1));
        mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 2));
        const float mn0 = fmaxf(m0, mx0), mn1 = fmaxf(m1, mx1);
        const float ms0 = (mn0 == -INFINITY) ? 0.0f : mn0, ms1 = (mn1 == -INFINITY) ? 0.0f : mn1;
        const float c0 = (m0 == -INFINITY) ? 0.0f : exp2f(m0 - ms0);
        const float c1 = (m1 == -INFINITY) ? 0.0f : exp2f(m1 - ms1);
        float rs0 = 0.0f, rs1 = 0.0f;
#pragma unroll
        for (int nt = 0; nt < 8; ++nt) {
#pragma unroll
            for (int i = 0; i < 2; ++i) {
                s[nt][i] = exp2f(s[nt][i] - ms0);
                s[nt][2 + i] = exp2f(s[nt][2 + i] - ms1);
                rs0 += s[nt][i];
                rs1 += s[nt][2 + i];
            }
        }
        rs0 += __shfl_xor_sync(0xffffffffu, rs0, 1);
        rs0 += __shfl_xor_sync(0xffffffffu, rs0, 2);
        rs1 += __shfl_xor_sync(0xffffffffu, rs1, 1);
        rs1 += __shfl_xor_sync(0xffffffffu, rs1, 2);
        l0 = l0 * c0 + rs0;
        l1 = l1 * c1 + rs1;
        m0 = mn0;
        m1 = mn1;
#pragma unroll
        for (int dt = 0; dt < D / 8; ++dt) {
            o[dt][0] *= c0; o[dt][1] *= c0;
            o[dt][2] *= c1; o[dt][3] *= c1;
        }
        uint32_t pa[4][4];
#pragma unroll
        for (int kk = 0; kk < 4; ++kk) {
            pa[kk][0] = pack_bf16(s[2 * kk][0], s[2 * kk][1]);
            pa[kk][1] = pack_bf16(s[2 * kk][2], s[2 * kk][3]);
            pa[kk][2] = pack_bf16(s[2 * kk + 1][0], s[2 * kk + 1][1]);
            pa[kk][3] = pack_bf16(s[2 * kk + 1][2], s[2 * kk + 1][3]);
        }
#pragma unroll
        for (int dtp = 0; dtp < D / 16; ++dtp) {
#pragma unroll
            for (int kk = 0; kk < 4; ++kk) {
                uint32_t r[4];
                const int mi = lane >> 3;
                ldsm_x4_t(r, vtile + sw_off(16 * kk + (mi & 1) * 8 + (lane & 7), 2 * dtp + (mi >> 1)));
                mma_bf16(o[2 * dtp], pa[kk], r[0], r[1]);
                mma_bf16(o[2 * dtp + 1], pa[kk], r[2], r[3]);
            }
        }
        // every warp is done with this stage before it is refilled
        if (__syncthreads_or(failed)) {
            if (tid == 0) atomicExch(err, 1);
            return;
        }
    }

    const float inv0 = (l0 > 0.0f) ? 1.0f / l0 : 0.0f, inv1 = (l1 > 0.0f) ? 1.0f / l1 : 0.0f;
    __nv_bfloat16* o0 = out + ((size_t)(n0 + tok0) * nq + h0) * D;
    __nv_bfloat16* o1 = out + ((size_t)(n0 + tok1) * nq + h1) * D;
#pragma unroll
    for (int dt = 0; dt < D / 8; ++dt) {
        const int col = 8 * dt + 2 * t;
        if (ok0) *reinterpret_cast<uint32_t*>(o0 + col) = pack_bf16(o[dt][0] * inv0, o[dt][1] * inv0);
        if (ok1) *reinterpret_cast<uint32_t*>(o1 + col) = pack_bf16(o[dt][2] * inv1, o[dt][3] * inv1);
    }
}

// q, out: bfloat16 [N, nq, d]; cu_q int32 [B+1]; seq_start int32 [B] (cached length of each
// sequence before this step); n_tiles = sum over sequences of ceil(q_len / (64 / (nq/nkv))).
LUMEN_API int lumen_attn_prefill(const void* q, const void* kcache, const void* vcache,
                                 const int* block_table, int bt_stride, const int* cu_q,
                                 const int* seq_start, int B, int n_tiles, void* out, int nq,
                                 int nkv, int d, int window, float scale, int* err,
                                 cudaStream_t stream) {
    if (B <= 0 || n_tiles <= 0) return 0;
    if (nq <= 0 || nkv <= 0 || nq % nkv != 0 || nq / nkv > 16 || window < 0) return LUMEN_ERR_UNSUPPORTED;
    if (nkv > 65535) return LUMEN_ERR_UNSUPPORTED;
    dim3 grid(n_tiles, nkv);
    const float scale_log2 = scale * 1.4426950408889634f;
    const __nv_bfloat16* qp = (const __nv_bfloat16*)q;
    const __nv_bfloat16* kp = (const __nv_bfloat16*)kcache;
    const __nv_bfloat16* vp = (const __nv_bfloat16*)vcache;
    if (d == 128) {
        const int smem = 4 * LUMEN_PAGE * 128 * 2;
        auto k = attn_prefill_kernel<128>;
        cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
        lumen_launch(k, dim3(grid), dim3(AP_THREADS), smem, stream, qp, kp, vp, block_table, bt_stride, cu_q, seq_start, B,
                                              (__nv_bfloat16*)out, nq, nkv, window, scale_log2, err);
    } else if (d == 64) {
        const int smem = 4 * LUMEN_PAGE * 64 * 2;
        auto k = attn_prefill_kernel<64>;
        lumen_launch(k, dim3(grid), dim3(AP_THREADS), smem, stream, qp, kp, vp, block_table, bt_stride, cu_q, seq_start, B,
                                              (__nv_bfloat16*)out, nq, nkv, window, scale_log2, err);
    } else {
        return LUMEN_ERR_UNSUPPORTED;
    }
    LUMEN_LAUNCH_CHECK();
    return 0;
}
