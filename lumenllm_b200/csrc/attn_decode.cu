// Decode attention over the paged cache for bfloat16, split over the keys.
//
// One query token per sequence. A block takes one SEGMENT of a sequence (a run of at most
// seg_pages pages; a sequence's pages are dealt out evenly over its segments) for one kv head and serves all query heads of that kv head at once, so every key and value
// is read from HBM exactly once per step. The block walks its pages through a ring of two or
// three stages (three while all blocks of the launch fit the SMs at once and a deeper ring is
// what hides latency; two, so that three blocks instead of two share an SM, when there are
// more blocks than that; the depth changes no result): the K tile and the V tile of a page are each one contiguous, already swizzled block
// of the cache and are brought in by one bulk asynchronous copy each (cp.async.bulk,
// completion on an mbarrier), while the tensor cores work on the page before: no tensor
// map, no address arithmetic per element. Each of the four warps owns 16 keys of a page:
// S = Q K^T and O = P V run as mma.sync m16n8k16 with the query heads of the group padded to
// 16 rows (the kernel is bound by HBM; the padding costs nothing), softmax online in
// float32 per warp across the pages, with scores and running maxima in units of log 2 so that
// every exponential is one ex2 instruction, and a row's sum kept per lane until the last page. At the end the block merges its four warps. A sequence
// that fits one segment is finished there; otherwise the block writes one partial
// (unnormalised O, running max m, sum l) per (sequence, head, segment) and the segments are
// merged in rising order, either by the block of the group that finishes last (it learns
// that from a counter; nobody waits) or by a second kernel. How a sequence is cut depends on
// its own length, the window and seg_pages only, and a key's place inside its page never
// changes, so neighbours in the batch do not change a token's result.
//
// The positions, the page table and every page but the one that holds the newest token were
// written before the kernel ahead of this one started, so the block requests its first pages
// before it waits for that kernel (programmatic dependent launch); the newest page and the
// query come after the wait.
//
// The kernel can also do the work of the rotary kernel that otherwise stands before it
// (lumen_attn_decode_qkv, head size 128): then it is given the QKV projection as the product
// left it, float32 partial sums, and every block makes the query heads of its group itself
// (sum of the parts, head norm, rotation; qk_head.cuh, the rotary kernel's own arithmetic) into
// shared memory; the block of a sequence's last segment also makes the new token's key and
// value, stores them in the cache for the steps to come, and puts them into its own copy of the
// page once that has arrived. One kernel, and one wait for a kernel ahead, fewer on the step's
// path; the first pages are requested before the wait as ever.
//
// Scratch: part_o [B, nq, max_segs, D] and part_ml [B, nq, max_segs, 2] float32.
#include "common.cuh"
#include "mma_utils.cuh"
#include "qk_head.cuh"

#define AD_THREADS 128
#define AD_SEG_PAGES 8            // the largest seg_pages a caller may ask for
#define AD_MAX_SEGS 32            // a sequence is never cut into more segments than this
#define AD_PAGE_IDS 16             // page numbers of a segment kept in shared memory
#define AD_MAX_STAGES 3           // ring depth: 3 when every block is resident at once, else 2

// The pages [pg_lo, pg_hi] that the query at position p sees, cut into nseg segments of
// per or per + 1 pages (the first rem have one more): segments of seg_pages pages at most,
// unless that would make more than AD_MAX_SEGS of them. Nothing here depends on the width of
// the page table.
struct SegPlan {
    int lo, pg_lo, pg_hi, nseg, per, rem;
    __device__ __forceinline__ int first(int seg) const { return pg_lo + seg * per + min(seg, rem); }
    __device__ __forceinline__ int count(int seg) const { return per + (seg < rem ? 1 : 0); }
};
__device__ __forceinline__ SegPlan seg_plan(int p, int window, int seg_pages) {
    SegPlan s;
    s.lo = 0;
    if (window > 0 && p - window + 1 > 0) s.lo = p - window + 1;
    s.pg_lo = s.lo / LUMEN_PAGE;
    s.pg_hi = p / LUMEN_PAGE;
    const int np = s.pg_hi - s.pg_lo + 1;
    s.nseg = min((np + seg_pages - 1) / seg_pages, AD_MAX_SEGS);
    s.per = np / s.nseg;
    s.rem = np - s.per * s.nseg;
    return s;
}

// 2^x on the special-function unit (2 ulp); scores and running maxima are kept in units of
// log 2, so every exponential of the softmax and of the merges is one instruction
__device__ __forceinline__ float ad_ex2(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}

// What the kernel needs to make q (and the newest k, v) itself; qkv == nullptr: q is given.
struct AdQkv {
    const float* qkv;          // [S][B][(nq + 2 nkv) * 128] partial sums of the projection
    int S;
    size_t split_stride;
    const float* qw;           // head norms' weights [128] or null
    const float* kw;
    float eps;
    const float2* cs;          // (cos, sin) [B][64]
    int rotate;                // whether q and k are rotated
    int store_kv;              // whether this run owns its cache: make and store the new k, v
    __nv_bfloat16* kcache;     // the same caches, to write
    __nv_bfloat16* vcache;
};

template <int D, int AD_STAGES>
__global__ void __launch_bounds__(AD_THREADS)
attn_decode_kernel(const __nv_bfloat16* __restrict__ q, const __nv_bfloat16* __restrict__ kcache,
                   const __nv_bfloat16* __restrict__ vcache, const int* __restrict__ block_table,
                   int bt_stride, const int* __restrict__ seq_pos, float* __restrict__ part_o,
                   float* __restrict__ part_ml, int nq, int nkv, int window, float scale,
                   int max_segs, int seg_pages, int* __restrict__ err, int* __restrict__ counters,
                   __nv_bfloat16* __restrict__ out, const AdQkv f) {
    constexpr int TILE_BYTES = LUMEN_PAGE * D * 2;
    __shared__ __align__(16) __nv_bfloat16 s_q[16 * D];     // the group's query heads, when made here
    extern __shared__ __align__(1024) unsigned char smem[];   // [stages][K tile, V tile]
    __shared__ uint64_t full[AD_STAGES];
    __shared__ float s_m[4][16], s_l[4][16];
    __shared__ int s_last;
    __shared__ int s_page[AD_PAGE_IDS];       // the segment's first page numbers, read once

    const int seg = blockIdx.x, kvh = blockIdx.y, b = blockIdx.z;
    const int p = seq_pos[b];                   // written before the step's first kernel
    const SegPlan plan = seg_plan(p, window, seg_pages);
    if (seg >= plan.nseg) return;
    const int lo = plan.lo, pg_a = plan.first(seg), npages = plan.count(seg), pg_hi = plan.pg_hi;

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int g = lane >> 2, t = lane & 3;
    const int G = nq / nkv;
    const int* bt = block_table + (size_t)b * bt_stride;

    if (tid == 0) {
        for (int i = 0; i < AD_STAGES; ++i) mbar_init(&full[i], 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    // The page table was written before the step's first kernel: the segment's page numbers
    // are fetched once, all at the same time, instead of one dependent load from global
    // memory in front of every copy (which held the whole block some 700 cycles a page).
    if (tid < AD_PAGE_IDS && tid < npages) s_page[tid] = bt[pg_a + tid];
    __syncthreads();
    auto issue = [&](int stage, int pg) {
        const int idx = pg - pg_a;
        const int page = idx < AD_PAGE_IDS ? s_page[idx] : bt[pg];
        const size_t off = ((size_t)page * nkv + kvh) * (size_t)(LUMEN_PAGE * D);
        unsigned char* dst = smem + stage * 2 * TILE_BYTES;
        mbar_expect_tx(&full[stage], 2 * TILE_BYTES);
        bulk_load(dst, kcache + off, TILE_BYTES, &full[stage]);
        bulk_load(dst + TILE_BYTES, vcache + off, TILE_BYTES, &full[stage]);
    };
    // The first pages of the ring, as far as they are older than this step; then wait for the
    // kernel ahead (it writes the newest token's key and value, and the query), then the rest.
    // (When this kernel itself makes the new key and value, nobody else writes the newest page
    // in this step, and it may come early too.)
    const bool makes_q = D == 128 && f.qkv != nullptr;
    const bool makes_kv = makes_q && f.store_kv != 0 && seg == plan.nseg - 1;
    int issued = 0;
    if (tid == 0)
        while (issued < AD_STAGES && issued < npages &&
               (pg_a + issued != pg_hi || (makes_q && f.store_kv != 0))) {
            issue(issued, pg_a + issued);
            ++issued;
        }
    pdl_wait();
    pdl_trigger();
    if (tid == 0)
        while (issued < AD_STAGES && issued < npages) {
            issue(issued, pg_a + issued);
            ++issued;
        }

    // The group's query heads, a warp a head, into shared memory; warps 2 and 3 of the last
    // segment's block then make the new token's key and value (4 values a lane, kept for the
    // block's copy of the page) and store them in the cache.
    uint2 kv_new = make_uint2(0u, 0u);
    if (makes_q) {
        const int nheads = nq + 2 * nkv;
        const float* tok = f.qkv + (size_t)b * nheads * 128;
        const float2* cs_b = f.cs + (size_t)b * 64;
        for (int hh = warp; hh < G; hh += 4) {
            const float4 v = qk_head_d128(tok + (size_t)(kvh * G + hh) * 128, f.S, f.split_stride, f.qw, f.eps, cs_b,
                                          f.rotate != 0, lane);
            uint2 w;
            w.x = pack_bf16(v.x, v.y);
            w.y = pack_bf16(v.z, v.w);
            *reinterpret_cast<uint2*>(s_q + hh * 128 + 4 * lane) = w;
        }
        if (makes_kv && warp >= 2) {
            const bool is_k = warp == 2;
            const float4 v = qk_head_d128(tok + (size_t)(nq + (is_k ? 0 : nkv) + kvh) * 128, f.S, f.split_stride,
                                          is_k ? f.kw : nullptr, f.eps, cs_b, is_k && f.rotate != 0, lane);
            kv_new.x = pack_bf16(v.x, v.y);
            kv_new.y = pack_bf16(v.z, v.w);
            const int idx = pg_hi - pg_a;
            const int page = idx < AD_PAGE_IDS ? s_page[idx] : bt[pg_hi];
            __nv_bfloat16* tile = (is_k ? f.kcache : f.vcache) + ((size_t)page * nkv + kvh) * (size_t)(LUMEN_PAGE * 128);
            *reinterpret_cast<uint2*>(tile + tile_offset(LUMEN_LAYOUT_SW128, p % LUMEN_PAGE, 4 * lane, 128)) = kv_new;
        }
        __syncthreads();
    }

    // Query fragments: rows = the G heads of this kv head (zero beyond G).
    uint32_t qa[D / 16][4];
    {
        const __nv_bfloat16* q0 = makes_q ? s_q + g * D : q + ((size_t)b * nq + (size_t)kvh * G + g) * D;
        const __nv_bfloat16* q1 = q0 + (size_t)8 * D;
        const bool r0 = g < G, r1 = g + 8 < G;
#pragma unroll
        for (int ks = 0; ks < D / 16; ++ks) {
            const int col = 16 * ks + 2 * t;
            qa[ks][0] = r0 ? *reinterpret_cast<const uint32_t*>(q0 + col) : 0u;
            qa[ks][1] = r1 ? *reinterpret_cast<const uint32_t*>(q1 + col) : 0u;
            qa[ks][2] = r0 ? *reinterpret_cast<const uint32_t*>(q0 + col + 8) : 0u;
            qa[ks][3] = r1 ? *reinterpret_cast<const uint32_t*>(q1 + col + 8) : 0u;
        }
    }

    float o[D / 8][4];
#pragma unroll
    for (int dt = 0; dt < D / 8; ++dt) o[dt][0] = o[dt][1] = o[dt][2] = o[dt][3] = 0.0f;
    float m0 = -INFINITY, m1 = -INFINITY, l0 = 0.0f, l1 = 0.0f;   // rows g and g + 8 of this warp's keys
    bool failed = false;
    const int rb = warp * 16;                                     // this warp's keys within a page

    for (int it = 0; it < npages; ++it) {
        const int stage = it % AD_STAGES;
        if (!mbar_wait(&full[stage], (it / AD_STAGES) & 1)) failed = true;
        if (makes_kv && it == npages - 1) {
            // the newest page as it arrived lacks this step's row: put it in
            if (warp >= 2)
                *reinterpret_cast<uint2*>(smem + stage * 2 * TILE_BYTES + (warp == 2 ? 0 : TILE_BYTES) +
                                          2 * tile_offset(LUMEN_LAYOUT_SW128, p % LUMEN_PAGE, 4 * lane, D)) = kv_new;
            __syncthreads();
        }
        const uint32_t ktile = smem_u32(smem + stage * 2 * TILE_BYTES);
        const uint32_t vtile = ktile + TILE_BYTES;

        float s[2][4];
#pragma unroll
        for (int nt = 0; nt < 2; ++nt) {
            s[nt][0] = s[nt][1] = s[nt][2] = s[nt][3] = 0.0f;
#pragma unroll
            for (int kp = 0; kp < D / 32; ++kp) {
                uint32_t r[4];
                ldsm_x4(r, ktile + sw_off(rb + 8 * nt + (lane & 7), 4 * kp + (lane >> 3)));
                mma_bf16(s[nt], qa[2 * kp], r[0], r[1]);
                mma_bf16(s[nt], qa[2 * kp + 1], r[2], r[3]);
            }
        }
        const int jbase = (pg_a + it) * LUMEN_PAGE + rb;
        float mx0 = -INFINITY, mx1 = -INFINITY;
#pragma unroll
        for (int nt = 0; nt < 2; ++nt) {
#pragma unroll
            for (int i = 0; i < 2; ++i) {
                const int j = jbase + 8 * nt + 2 * t + i;
                const bool valid = (j >= lo) && (j <= p);
                s[nt][i] = valid ? s[nt][i] * scale : -INFINITY;
                s[nt][2 + i] = valid ? s[nt][2 + i] * scale : -INFINITY;
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
        const float c0 = (m0 == -INFINITY) ? 0.0f : ad_ex2(m0 - ms0);
        const float c1 = (m1 == -INFINITY) ? 0.0f : ad_ex2(m1 - ms1);
        float rs0 = 0.0f, rs1 = 0.0f;
#pragma unroll
        for (int nt = 0; nt < 2; ++nt) {
#pragma unroll
            for (int i = 0; i < 2; ++i) {
                s[nt][i] = ad_ex2(s[nt][i] - ms0);
                s[nt][2 + i] = ad_ex2(s[nt][2 + i] - ms1);
                rs0 += s[nt][i];
                rs1 += s[nt][2 + i];
            }
        }
        // the sums stay per lane (four lanes share a row); they are put together once, after
        // the last page
        l0 = l0 * c0 + rs0;
        l1 = l1 * c1 + rs1;
        m0 = mn0;
        m1 = mn1;
        uint32_t pa[4];
        pa[0] = pack_bf16(s[0][0], s[0][1]);
        pa[1] = pack_bf16(s[0][2], s[0][3]);
        pa[2] = pack_bf16(s[1][0], s[1][1]);
        pa[3] = pack_bf16(s[1][2], s[1][3]);
#pragma unroll
        for (int dtp = 0; dtp < D / 16; ++dtp) {
            uint32_t r[4];
            const int mi = lane >> 3;
            ldsm_x4_t(r, vtile + sw_off(rb + (mi & 1) * 8 + (lane & 7), 2 * dtp + (mi >> 1)));
            o[2 * dtp][0] *= c0; o[2 * dtp][1] *= c0; o[2 * dtp][2] *= c1; o[2 * dtp][3] *= c1;
            o[2 * dtp + 1][0] *= c0; o[2 * dtp + 1][1] *= c0; o[2 * dtp + 1][2] *= c1; o[2 * dtp + 1][3] *= c1;
            mma_bf16(o[2 * dtp], pa, r[0], r[1]);
            mma_bf16(o[2 * dtp + 1], pa, r[2], r[3]);
        }
        // every warp is done with this stage before it is refilled
        if (__syncthreads_or(failed)) {
            if (tid == 0) atomicExch(err, 1);
            return;
        }
        // the refill is issued by two warps, the K copy by one and the V copy by another: a bulk
        // copy holds its issuing thread some 150 cycles, and the block waits for its slowest warp
        if (lane == 0 && warp < 2 && it + AD_STAGES < npages) {
            const int idx = it + AD_STAGES;
            const int page = idx < AD_PAGE_IDS ? s_page[idx] : bt[pg_a + idx];
            const size_t off = ((size_t)page * nkv + kvh) * (size_t)(LUMEN_PAGE * D);
            unsigned char* dst = smem + stage * 2 * TILE_BYTES;
            if (warp == 0) {
                mbar_expect_tx(&full[stage], 2 * TILE_BYTES);
                bulk_load(dst, kcache + off, TILE_BYTES, &full[stage]);
            } else {
                bulk_load(dst + TILE_BYTES, vcache + off, TILE_BYTES, &full[stage]);
            }
        }
    }

    l0 += __shfl_xor_sync(0xffffffffu, l0, 1);
    l0 += __shfl_xor_sync(0xffffffffu, l0, 2);
    l1 += __shfl_xor_sync(0xffffffffu, l1, 1);
    l1 += __shfl_xor_sync(0xffffffffu, l1, 2);
    // Merge the four warps through shared memory (all stages have been consumed).
    float* so = reinterpret_cast<float*>(smem);   // [4][G][D]
    if (t == 0) {
        if (g < G) { s_m[warp][g] = m0; s_l[warp][g] = l0; }
        if (g + 8 < G) { s_m[warp][g + 8] = m1; s_l[warp][g + 8] = l1; }
    }
#pragma unroll
    for (int dt = 0; dt < D / 8; ++dt) {
        if (g < G) {
            float* dst = so + ((size_t)(warp * G + g)) * D + 8 * dt + 2 * t;
            dst[0] = o[dt][0];
            dst[1] = o[dt][1];
        }
        if (g + 8 < G) {
            float* dst = so + ((size_t)(warp * G + g + 8)) * D + 8 * dt + 2 * t;
            dst[0] = o[dt][2];
            dst[1] = o[dt][3];
        }
    }
    __syncthreads();
    const bool single = (plan.nseg == 1);   // the whole sequence was this block's
    constexpr int D4 = D / 4;
    for (int idx = tid; idx < G * D4; idx += AD_THREADS) {
        const int row = idx / D4, e = (idx - row * D4) * 4;
        const float M = fmaxf(fmaxf(s_m[0][row], s_m[1][row]), fmaxf(s_m[2][row], s_m[3][row]));
        float4 acc = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
        float l = 0.0f;
#pragma unroll
        for (int w = 0; w < 4; ++w) {
            const float mw = s_m[w][row];
            const float f = (mw == -INFINITY) ? 0.0f : ad_ex2(mw - M);
            const float4 v = *reinterpret_cast<const float4*>(so + ((size_t)(w * G + row)) * D + e);
            acc.x += v.x * f; acc.y += v.y * f; acc.z += v.z * f; acc.w += v.w * f;
            l += s_l[w][row] * f;
        }
        const size_t head = (size_t)b * nq + (size_t)kvh * G + row;
        if (single) {
            const float inv = 1.0f / l;
            uint2 w2;
            w2.x = pack_bf16(acc.x * inv, acc.y * inv);
            w2.y = pack_bf16(acc.z * inv, acc.w * inv);
            *reinterpret_cast<uint2*>(out + head * D + e) = w2;
        } else {
            const size_t pi = head * max_segs + seg;
            *reinterpret_cast<float4*>(part_o + pi * D + e) = acc;
            if (e == 0) *reinterpret_cast<float2*>(part_ml + pi * 2) = make_float2(M, l);
        }
    }
    if (single || counters == nullptr) return;   // done, or a second kernel merges the segments

    // Merge without a second kernel and without waiting: every block of this (sequence, kv
    // head) counts itself in after its partials are visible; the one that counts last merges
    // all segments, in rising order whoever it is, and puts the counter back to zero.
    // (the barrier orders every thread's partials before thread 0's release, which is
    // cumulative; the last block's acquire and its barrier order them before the reads below)
    __syncthreads();
    if (tid == 0) {
        int ticket;
        asm volatile("atom.acq_rel.gpu.global.add.s32 %0, [%1], 1;"
                     : "=r"(ticket)
                     : "l"(counters + b * nkv + kvh)
                     : "memory");
        s_last = (ticket == plan.nseg - 1);
        if (s_last) counters[b * nkv + kvh] = 0;
    }
    __syncthreads();
    if (!s_last) return;
    // One pass with a running maximum, so that every load of a thread is in flight at once:
    // a thread owns four values of one head and reads each segment's (m, l) itself.
    const int nch = plan.nseg;
    for (int idx = tid; idx < G * D4; idx += AD_THREADS) {
        const int row = idx / D4, e = (idx - row * D4) * 4;
        const size_t head = (size_t)b * nq + (size_t)kvh * G + row;
        const size_t base = head * max_segs;
        float M = -INFINITY, L = 0.0f;
        float4 acc = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
#pragma unroll 8
        for (int cc = 0; cc < nch; ++cc) {
            const float2 ml = __ldcg(reinterpret_cast<const float2*>(part_ml + (base + cc) * 2));
            const float4 v = __ldcg(reinterpret_cast<const float4*>(part_o + (base + cc) * D + e));
            const float mn = fmaxf(M, ml.x);
            const float a = ad_ex2(M - mn), f = ad_ex2(ml.x - mn);   // a = 0 at the first segment
            acc.x = acc.x * a + v.x * f; acc.y = acc.y * a + v.y * f;
            acc.z = acc.z * a + v.z * f; acc.w = acc.w * a + v.w * f;
            L = L * a + ml.y * f;
            M = mn;
        }
        const float inv = 1.0f / L;
        uint2 w2;
        w2.x = pack_bf16(acc.x * inv, acc.y * inv);
        w2.y = pack_bf16(acc.z * inv, acc.w * inv);
        *reinterpret_cast<uint2*>(out + head * D + e) = w2;
    }
}

// Merges the segments of one (sequence, head) in rising order (used when no counters are given).
template <typename TOut>
__global__ void attn_decode_combine_kernel(const float* __restrict__ part_o,
                                           const float* __restrict__ part_ml,
                                           const int* __restrict__ seq_pos, TOut* __restrict__ out,
                                           int nq, int D, int window, int max_segs, int seg_pages) {
    pdl_wait();      // nothing of this kernel touches global memory before this
    pdl_trigger();
    const int head = blockIdx.x, b = blockIdx.y;
    const SegPlan plan = seg_plan(seq_pos[b], window, seg_pages);
    if (plan.nseg == 1) return; // a single segment: the first kernel has written the result
    const int c0 = 0, c1 = plan.nseg - 1;
    const size_t base = ((size_t)b * nq + head) * max_segs;
    float M = -INFINITY;
    for (int c = c0; c <= c1; ++c) M = fmaxf(M, part_ml[(base + c) * 2]);
    float L = 0.0f;
    for (int c = c0; c <= c1; ++c) L += part_ml[(base + c) * 2 + 1] * ad_ex2(part_ml[(base + c) * 2] - M);
    const float inv = 1.0f / L;
    for (int e = threadIdx.x; e < D; e += blockDim.x) {
        float acc = 0.0f;
        for (int c = c0; c <= c1; ++c)
            acc += part_o[(base + c) * D + e] * ad_ex2(part_ml[(base + c) * 2] - M);
        out[((size_t)b * nq + head) * D + e] = from_f32<TOut>(acc * inv);
    }
}

// Checks and launch of both entry points below.
static int attn_decode_launch(const void* q, const void* kcache, const void* vcache,
                              const int* block_table, int bt_stride, const int* seq_pos,
                              void* out, float* part_o, float* part_ml, int B, int nq, int nkv,
                              int d, int window, float scale, int max_segs, int seg_pages,
                              int* err, int* counters, cudaStream_t stream, const AdQkv& f) {
    if (B <= 0) return 0;
    if (nq <= 0 || nkv <= 0 || nq % nkv != 0 || nq / nkv > 16 || window < 0 || max_segs <= 0)
        return LUMEN_ERR_UNSUPPORTED;
    if (B > 65535 || nkv > 65535) return LUMEN_ERR_UNSUPPORTED;
    if (seg_pages < 1 || seg_pages > AD_SEG_PAGES) return LUMEN_ERR_BAD_ARGUMENT;
    if (max_segs < AD_MAX_SEGS && (long long)seg_pages * max_segs < bt_stride) return LUMEN_ERR_BAD_ARGUMENT;
    dim3 grid(max_segs, nkv, B);
    const __nv_bfloat16* qp = (const __nv_bfloat16*)q;
    const __nv_bfloat16* kp = (const __nv_bfloat16*)kcache;
    const __nv_bfloat16* vp = (const __nv_bfloat16*)vcache;
    cudaError_t e;
    static int sms = 0;
    if (!sms) {
        int dev = 0;
        cudaGetDevice(&dev);
        if (cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || sms <= 0) sms = 148;
    }
    const bool deep = (long long)max_segs * nkv * B <= 2LL * sms;
    scale *= 1.4426950408889634f;       // scores in units of log 2 (see ad_ex2)
    auto go = [&](auto kernel, int stages, int dd) -> cudaError_t {
        const int smem = stages * 2 * LUMEN_PAGE * dd * 2;
        cudaError_t err_ = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
        if (err_ != cudaSuccess) return err_;
        return lumen_launch(kernel, grid, dim3(AD_THREADS), smem, stream, qp, kp, vp, block_table, bt_stride,
                            seq_pos, part_o, part_ml, nq, nkv, window, scale, max_segs, seg_pages, err, counters,
                            (__nv_bfloat16*)out, f);
    };
    if (d == 128) {
        e = deep ? go(attn_decode_kernel<128, 3>, 3, 128) : go(attn_decode_kernel<128, 2>, 2, 128);
    } else if (d == 64) {
        e = deep ? go(attn_decode_kernel<64, 3>, 3, 64) : go(attn_decode_kernel<64, 2>, 2, 64);
    } else {
        return LUMEN_ERR_UNSUPPORTED;
    }
    if (e != cudaSuccess) return (int)e;
    LUMEN_LAUNCH_CHECK();
    if (counters != nullptr) return 0;
    dim3 cgrid(nq, B);
    e = lumen_launch(attn_decode_combine_kernel<__nv_bfloat16>, cgrid, dim3(128), 0, stream,
                     (const float*)part_o, (const float*)part_ml, seq_pos, (__nv_bfloat16*)out, nq, d, window,
                     max_segs, seg_pages);
    if (e != cudaSuccess) return (int)e;
    LUMEN_LAUNCH_CHECK();
    return 0;
}

// Entry point. q, out: bfloat16 [B, nq, D]; caches in the swizzled layout; seq_pos[b] is the
// position of sequence b's query (its cached length before this token). seg_pages: the most
// pages a segment has, 1 to 8 (callers that want a sequence's result to be the same in every
// batch pass the same number for every batch; the library's own decode step passes 4).
// max_segs: segments the scratch has room for per (sequence, head): at least
// min(ceil(bt_stride / seg_pages), 32), the most a sequence is cut into. part_o and part_ml
// are the caller's scratch (sizes above); err is a device int set to 1 if a copy never arrived.
// counters: null (a second kernel merges the segments), or B * nkv ints that are zero before
// the call and zero again after it (the last block of each group merges).
LUMEN_API int lumen_attn_decode(const void* q, const void* kcache, const void* vcache,
                                const int* block_table, int bt_stride, const int* seq_pos,
                                void* out, float* part_o, float* part_ml, int B, int nq, int nkv,
                                int d, int window, float scale, int max_segs, int seg_pages,
                                int* err, int* counters, cudaStream_t stream) {
    AdQkv f = {};
    return attn_decode_launch(q, kcache, vcache, block_table, bt_stride, seq_pos, out, part_o, part_ml, B, nq, nkv,
                              d, window, scale, max_segs, seg_pages, err, counters, stream, f);
}

// The same with the rotary kernel's work done by the attention blocks (head size 128). qkv:
// float32 [S][B][(nq + 2 nkv) * 128], the projection's partial sums, split_stride values
// apart; qw, kw: the head norms' weights [128] or null; cs: (cos, sin) [B][64] for rotate != 0;
// store_kv != 0: the new token's key and value are made and written to kcache / vcache (a run
// that reads another run's cache passes 0 and finds them there). The other arguments as above.
LUMEN_API int lumen_attn_decode_qkv(const float* qkv, int S, long long split_stride, const float* qw,
                                    const float* kw, float eps, const float* cs, int rotate, int store_kv,
                                    void* kcache, void* vcache, const int* block_table, int bt_stride,
                                    const int* seq_pos, void* out, float* part_o, float* part_ml, int B,
                                    int nq, int nkv, int d, int window, float scale, int max_segs,
                                    int seg_pages, int* err, int* counters, cudaStream_t stream) {
    if (d != 128) return LUMEN_ERR_UNSUPPORTED;
    if (!qkv || S < 1 || (S > 1 && split_stride <= 0) || ((uintptr_t)qkv & 15) || ((split_stride * 4) & 15) ||
        ((uintptr_t)qw & 15) || ((uintptr_t)kw & 15) || (rotate && (!cs || ((uintptr_t)cs & 15))))
        return LUMEN_ERR_BAD_ARGUMENT;
    AdQkv f;
    f.qkv = qkv;
    f.S = S;
    f.split_stride = (size_t)split_stride;
    f.qw = qw;
    f.kw = kw;
    f.eps = eps;
    f.cs = (const float2*)cs;
    f.rotate = rotate;
    f.store_kv = store_kv;
    f.kcache = (__nv_bfloat16*)kcache;
    f.vcache = (__nv_bfloat16*)vcache;
    return attn_decode_launch(nullptr, kcache, vcache, block_table, bt_stride, seq_pos, out, part_o, part_ml, B, nq,
                              nkv, d, window, scale, max_segs, seg_pages, err, counters, stream, f);
}

// ---------------------------------------------------------------------------------------
// The same decode attention for callers that must not allocate (declared and described in
// attn_decode_noalloc.h; the reference has no counterpart). The partial results live in one
// fixed array that is part of this library's device image.
// ---------------------------------------------------------------------------------------
#include <cstdio>
#include <mutex>

#include "attn_decode_noalloc.h"

static __device__ __align__(256) float lumen_decode_scratch[LUMEN_DECODE_NOALLOC_MAX_FLOATS];

#define LUMEN_NOALLOC_MAX_DEVICES 64
// Device address of lumen_decode_scratch on each device, looked up once per device. In host
// code the array's NAME is only a handle of the runtime, not memory a kernel may touch; the
// address a kernel needs comes from cudaGetSymbolAddress with that device current.
static float* s_scratch_on_device[LUMEN_NOALLOC_MAX_DEVICES];
static std::mutex s_scratch_lock;

LUMEN_API int lumen_attn_decode_noalloc(const void* q, const void* kcache, const void* vcache,
                                        const int* block_table, int bt_stride, const int* seq_pos,
                                        void* out, int B, int nq, int nkv, int d, int window,
                                        float scale, int max_segs, int* err, cudaStream_t stream) {
    if (B <= 0) return 0;
    if (nq <= 0 || max_segs <= 0 || d <= 0) return LUMEN_ERR_UNSUPPORTED;
    const unsigned long long rows = (unsigned long long)B * (unsigned long long)nq *
                                    (unsigned long long)max_segs;
    const unsigned long long need = rows * (unsigned long long)(d + 2);
    if (need > (unsigned long long)LUMEN_DECODE_NOALLOC_MAX_FLOATS) {
        std::fprintf(stderr,
                     "lumen_attn_decode_noalloc: batch %d x heads %d x segments %d x (head size %d + 2) = "
                     "%llu floats of scratch, the built-in array holds %llu; use a smaller batch or "
                     "page table, or the allocating entry point lumen_attn_decode\n",
                     B, nq, max_segs, d, need, (unsigned long long)LUMEN_DECODE_NOALLOC_MAX_FLOATS);
        return LUMEN_ERR_SCRATCH_TOO_SMALL;
    }
    int dev = -1;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return (int)e;
    if (dev < 0 || dev >= LUMEN_NOALLOC_MAX_DEVICES) return LUMEN_ERR_UNSUPPORTED;
    float* scratch;
    {
        std::lock_guard<std::mutex> guard(s_scratch_lock);
        if (s_scratch_on_device[dev] == nullptr) {
            float* p = nullptr;
            e = cudaGetSymbolAddress((void**)&p, lumen_decode_scratch);
            if (e != cudaSuccess) return (int)e;
            if (p == nullptr) return LUMEN_ERR_BAD_ARGUMENT;
            s_scratch_on_device[dev] = p;
        }
        scratch = s_scratch_on_device[dev];
    }
    // Nothing in the scratch has to start at zero: every (sequence, head, segment) entry that
    // the merge kernel reads is written in full by this call's first kernel; entries of
    // segments outside a sequence's range keep older contents and are never read.
    float* part_o = scratch;
    float* part_ml = scratch + rows * (unsigned long long)d;
    return lumen_attn_decode(q, kcache, vcache, block_table, bt_stride, seq_pos, out, part_o, part_ml,
                             B, nq, nkv, d, window, scale, max_segs, AD_SEG_PAGES, err, nullptr, stream);
}
