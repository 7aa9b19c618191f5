// Causal grouped-query flash attention for prompts on the 5th-generation tensor cores.
//
// A block takes 128 rows, each a (query token, query head) pair of ONE kv head (the G heads
// of the group times 128/G consecutive tokens of one sequence), and walks the keys page by
// page (64 keys). Per page:
//   S = Q K^T   tcgen05.mma 128 x 64 x D, Q and K from shared memory (K-major, 128-byte
//               swizzle), S into tensor memory (two S buffers, so the product for the next page
//               runs while this page's softmax does);
//   softmax     four warps, one thread per row: tcgen05.ld of the row, scale, mask, running
//               maximum and sum in float32, P = exp2(.) rounded to bfloat16 and written back
//               into tensor memory, over the columns its own scores came from (tcgen05.st);
//   O += P V    tcgen05.mma 128 x D x 64 with P as the A operand FROM TENSOR MEMORY and V
//               straight from its page tile in shared memory (N-major, 128-byte swizzle: the
//               cache layout is made for this), O accumulated in tensor memory.
// What bounds this kernel at long prompts is the time the tensor pipe takes over products of
// these shapes, read off clock stamps taken inside the kernel: the thread that issues them is
// held 75 cycles by each 128 x 64 x 16 product of S (32 cycles of arithmetic; 6 KB of operands
// from shared memory) and 92 by each 128 x 128 x 16 product of O (64 of arithmetic), with one
// block on the SM as with two, so a page costs 970 cycles of the pipe and two blocks an SM fill
// it (1,860 cycles a page and block). The softmax of a page takes a warp 875 cycles alone and
// about 1,000 beside its neighbour's, so it is not far behind: without any exponentials the
// kernel is 7 % faster, with half of the S products 7 %, with half of the O products 6 %.
// What was gained here: P in tensor memory instead of a 16 KB buffer in shared memory (no
// write and read of P through shared memory, and no wait for the product of the page before
// unless O is rescaled) 5 % at 8,192 tokens and 4 % at 2,048; one exponential in four on the
// FMA pipe 10 % at 2,048. Making the operand descriptors once instead of per product changed
// nothing. Products with more columns were tried as a kernel of its own: one block an SM
// with two Q tiles that share their K and V tiles, keys 128 at a time, S and O of both tiles
// in all 512 columns of tensor memory, the tiles taken in turn by the tensor pipe. Right
// results, and the S products did cost 66 cycles for 128 columns where they cost 75 for 64;
// but the O products, whose P operand comes from tensor memory, rose from 92 to 116 cycles
// under the tensor-memory traffic of eight softmax warps, a tile's chain (softmax of 128
// scores 2,270 cycles, then its O product, then its next S product) leaves the one issuing
// thread either held by the pipe or waiting, and a step of four page tiles took 4,100 to
// 4,300 cycles: 650 us at 8,192 tokens against 544 us for this kernel. Taken out again.
// So was the smaller step of this kernel with the S product taken over pairs of pages (one
// 128-column product into both S buffers, K tiles interleaved by 64-value block): the same
// bits, 634 against 544 us, because the next pair's S product cannot be issued before both O
// products of this pair, and the softmax, never idle here, then waits for it once a pair.
// O is rescaled only when a row's maximum has grown by more than 2^8 since the reference it
// was accumulated against (P and the row sum use the same reference, so the result is exact);
// the rescale is a read-modify-write of the row in tensor memory and is rare after the first
// pages. K and V tiles arrive through two two-stage rings of bulk asynchronous copies
// (cp.async.bulk + mbarrier; a page tile is one contiguous block of the cache). The rings are
// separate because their slots come free at different times: a K slot as soon as the S
// product that read it is done, which is a page ahead of the V slot that the O product of the
// same page frees; K for page i+2 is therefore on its way two pages early and V more than one,
// and the latency of the copies stays hidden with two slots each. Warp 0
// produces, warp 1 allocates tensor memory and issues all MMAs, warps 2..5 are the softmax.
// A block needs half of an SM's shared memory and half of its tensor memory, so two blocks
// share an SM and one's softmax runs under the other's products.
//
// Page tiles start at multiples of 64 in absolute position, so what a row computes depends
// only on its own position. Every wait is bounded; when one runs out the block raises the
// error flag, lets the other roles run out, frees its tensor memory and returns.
#include "common.cuh"
#include "mma_utils.cuh"

#define PT_THREADS 192
#define PT_ROWS 128
#define PT_STAGES 2
#define PT_RESCALE 8.0f
#define PT_FMA_EX2_OF_4 1         // of every four exponentials, this many go to the FMA pipe

__device__ __forceinline__ void pt_mbar_arrive(uint64_t* bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void pt_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void pt_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void pt_commit(uint64_t* bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar))
                 : "memory");
}
__device__ __forceinline__ void pt_mma(uint32_t d_tmem, uint64_t adesc, uint64_t bdesc, uint32_t idesc,
                                       uint32_t accumulate) {
    asm volatile(
        "{\n .reg .pred p;\n setp.ne.b32 p, %4, 0;\n"
        " tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n}" ::"r"(d_tmem),
        "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
        : "memory");
}
// The same product with the A operand in tensor memory: lane = row, two bfloat16 a column.
__device__ __forceinline__ void pt_mma_ts(uint32_t d_tmem, uint32_t a_tmem, uint64_t bdesc, uint32_t idesc,
                                          uint32_t accumulate) {
    asm volatile(
        "{\n .reg .pred p;\n setp.ne.b32 p, %4, 0;\n"
        " tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n}" ::"r"(d_tmem),
        "r"(a_tmem), "l"(bdesc), "r"(idesc), "r"(accumulate)
        : "memory");
}
__device__ __forceinline__ void pt_st32u(uint32_t taddr, const uint32_t (&v)[32]) {
    asm volatile(
        "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
        "{%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,"
        "%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31,%32};" ::"r"(taddr),
        "r"(v[0]), "r"(v[1]), "r"(v[2]), "r"(v[3]), "r"(v[4]), "r"(v[5]), "r"(v[6]), "r"(v[7]), "r"(v[8]),
        "r"(v[9]), "r"(v[10]), "r"(v[11]), "r"(v[12]), "r"(v[13]), "r"(v[14]), "r"(v[15]), "r"(v[16]),
        "r"(v[17]), "r"(v[18]), "r"(v[19]), "r"(v[20]), "r"(v[21]), "r"(v[22]), "r"(v[23]), "r"(v[24]),
        "r"(v[25]), "r"(v[26]), "r"(v[27]), "r"(v[28]), "r"(v[29]), "r"(v[30]), "r"(v[31])
        : "memory");
}
__device__ __forceinline__ void pt_ld32(uint32_t taddr, float (&v)[32]) {
    uint32_t r[32];
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
        "{%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,"
        "%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31}, [%32];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
          "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]),
          "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]),
          "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
        : "r"(taddr));
    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
    for (int i = 0; i < 32; ++i) v[i] = __uint_as_float(r[i]);
}
// 64 consecutive columns of this thread's row with one wait.
__device__ __forceinline__ void pt_ld64(uint32_t taddr, float (&v)[64]) {
    uint32_t r[64];
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x64.b32 "
        "{%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,"
        "%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31,"
        "%32,%33,%34,%35,%36,%37,%38,%39,%40,%41,%42,%43,%44,%45,%46,%47,"
        "%48,%49,%50,%51,%52,%53,%54,%55,%56,%57,%58,%59,%60,%61,%62,%63}, [%64];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
          "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]),
          "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]),
          "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31]),
          "=r"(r[32]), "=r"(r[33]), "=r"(r[34]), "=r"(r[35]), "=r"(r[36]), "=r"(r[37]), "=r"(r[38]), "=r"(r[39]),
          "=r"(r[40]), "=r"(r[41]), "=r"(r[42]), "=r"(r[43]), "=r"(r[44]), "=r"(r[45]), "=r"(r[46]), "=r"(r[47]),
          "=r"(r[48]), "=r"(r[49]), "=r"(r[50]), "=r"(r[51]), "=r"(r[52]), "=r"(r[53]), "=r"(r[54]), "=r"(r[55]),
          "=r"(r[56]), "=r"(r[57]), "=r"(r[58]), "=r"(r[59]), "=r"(r[60]), "=r"(r[61]), "=r"(r[62]), "=r"(r[63])
        : "r"(taddr));
    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
    for (int i = 0; i < 64; ++i) v[i] = __uint_as_float(r[i]);
}
// 2^x on the special-function unit (2 ulp; the result is rounded to bfloat16 or summed in
// float32 next to values up to 2^8 times larger).
__device__ __forceinline__ float pt_ex2(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}
// 2^x without the special-function unit: x = n + f with n the nearest integer (the magic-number
// add leaves n in the low mantissa bits), 2^f on [-0.5, 0.5] by a cubic (relative error 1e-4,
// a twentieth of the rounding to bfloat16 that follows), and n added into the exponent bits.
// The softmax does a part of its exponentials this way: the special-function unit makes 16 a
// cycle and SM, and at head size 128 that is as long a job as the page's two products.
__device__ __forceinline__ float pt_ex2_fma(float x) {
    x = fmaxf(x, -125.0f);                       // also what a masked (-inf) score becomes: 2^-125, nothing
    const float t = x + 12582912.0f;             // 1.5 * 2^23
    const float f = x - (t - 12582912.0f);
    float p = fmaf(0.05583828315138817f, f, 0.2426394820213318f);
    p = fmaf(p, f, 0.6931367516517639f);
    p = fmaf(p, f, 0.9999245405197144f);
    return __int_as_float(__float_as_int(p) + (__float_as_int(t) << 23));
}
__device__ __forceinline__ void pt_st32(uint32_t taddr, const float (&v)[32]) {
    asm volatile(
        "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
        "{%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,"
        "%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31,%32};" ::"r"(taddr),
        "r"(__float_as_uint(v[0])), "r"(__float_as_uint(v[1])), "r"(__float_as_uint(v[2])),
        "r"(__float_as_uint(v[3])), "r"(__float_as_uint(v[4])), "r"(__float_as_uint(v[5])),
        "r"(__float_as_uint(v[6])), "r"(__float_as_uint(v[7])), "r"(__float_as_uint(v[8])),
        "r"(__float_as_uint(v[9])), "r"(__float_as_uint(v[10])), "r"(__float_as_uint(v[11])),
        "r"(__float_as_uint(v[12])), "r"(__float_as_uint(v[13])), "r"(__float_as_uint(v[14])),
        "r"(__float_as_uint(v[15])), "r"(__float_as_uint(v[16])), "r"(__float_as_uint(v[17])),
        "r"(__float_as_uint(v[18])), "r"(__float_as_uint(v[19])), "r"(__float_as_uint(v[20])),
        "r"(__float_as_uint(v[21])), "r"(__float_as_uint(v[22])), "r"(__float_as_uint(v[23])),
        "r"(__float_as_uint(v[24])), "r"(__float_as_uint(v[25])), "r"(__float_as_uint(v[26])),
        "r"(__float_as_uint(v[27])), "r"(__float_as_uint(v[28])), "r"(__float_as_uint(v[29])),
        "r"(__float_as_uint(v[30])), "r"(__float_as_uint(v[31]))
        : "memory");
}
// Descriptor of a 128-byte-swizzled operand tile: rows of 128 bytes, groups of 8 rows 1024
// bytes apart (stride byte offset); `lbo` is the distance between 64-value blocks along the
// contiguous dimension (used by N-major operands wider than 64 values).
__device__ __forceinline__ uint64_t pt_desc(uint32_t smem_addr, uint32_t lbo_bytes) {
    uint64_t d = 0;
    d |= (uint64_t)((smem_addr >> 4) & 0x3FFF);
    d |= (uint64_t)((lbo_bytes >> 4) & 0x3FFF) << 16;
    d |= (uint64_t)(1024 >> 4) << 32;
    d |= (uint64_t)1 << 46;
    d |= (uint64_t)2 << 61;
    return d;
}
// D float32, A and B bfloat16, M = 128; b_mn: B is N-major (its contiguous dimension is N).
__host__ __device__ constexpr uint32_t pt_idesc(int n, int b_mn) {
    return (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)b_mn << 16) | ((uint32_t)(n >> 3) << 17) |
           ((uint32_t)(PT_ROWS >> 4) << 24);
}

template <int D>
__global__ void __launch_bounds__(PT_THREADS, 2)
attn_prefill_tc_kernel(const __nv_bfloat16* __restrict__ q, const __nv_bfloat16* __restrict__ kcache,
                       const __nv_bfloat16* __restrict__ vcache, const int* __restrict__ block_table,
                       int bt_stride, const int* __restrict__ cu_q, const int* __restrict__ seq_start,
                       int B, __nv_bfloat16* __restrict__ out, int nq, int nkv, int window,
                       float scale_log2, int* __restrict__ err) {
    pdl_wait();      // nothing of this kernel touches global memory before this
    pdl_trigger();
    constexpr int TILE_BYTES = LUMEN_PAGE * D * 2;      // one K or V page tile
    constexpr int Q_BYTES = PT_ROWS * D * 2;
    constexpr int NCOLS = 256;                          // S0 | S1 | O
    constexpr uint32_t O_COL = 128;
    // Operand tiles must start on 1024-byte boundaries (the swizzle pattern repeats there).
    // This kernel has no static shared memory, so its dynamic part starts the block's window;
    // there is no room for slack when two blocks share an SM, so the start is checked instead.
    extern __shared__ __align__(1024) unsigned char smem[];
    if (smem_u32(smem) & 1023u) {
        if (threadIdx.x == 0) atomicExch(err, 1);
        return;
    }
    unsigned char* sQ = smem;
    unsigned char* sKV = sQ + Q_BYTES;                  // [stage][K tile, V tile]
    uint64_t* bars = reinterpret_cast<uint64_t*>(sKV + PT_STAGES * 2 * TILE_BYTES);
    uint64_t* k_full = bars;                   // [stages] the K tile has landed
    uint64_t* k_empty = bars + PT_STAGES;      // [stages] the S product has read it
    uint64_t* v_full = bars + 2 * PT_STAGES;   // [stages] the V tile has landed
    uint64_t* v_empty = bars + 3 * PT_STAGES;  // [stages] the O product has read it
    uint64_t* s_full = bars + 4 * PT_STAGES;   // [2] S is in tensor memory
    uint64_t* p_ready = s_full + 2;            // [2] P is in tensor memory, O corrected
    uint64_t* pv_done = p_ready + 2;           // [2] the PV product of that page has finished
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(pv_done + 2);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

    const int G = nq / nkv;
    const int TQ = PT_ROWS / G;
    // blocks start in the order of blockIdx.x: tile-major, so that the longest tiles of ALL kv
    // heads start first and the short ones fill the tail
    const int kvh = blockIdx.x % nkv;
    int tile = blockIdx.x / nkv, b = 0, qlen = 0;
    for (; b < B; ++b) {
        qlen = cu_q[b + 1] - cu_q[b];
        const int nt = (qlen + TQ - 1) / TQ;
        if (tile < nt) break;
        tile -= nt;
    }
    if (b >= B) return;
    tile = (qlen + TQ - 1) / TQ - 1 - tile;    // the last tiles of a sequence see the most keys: start them first
    const int i0 = tile * TQ;
    const int ntok = min(TQ, qlen - i0);
    const int n0 = cu_q[b] + i0;
    const int pos0 = seq_start[b] + i0;
    const int pos_last = pos0 + ntok - 1;
    int j_lo = 0;
    if (window > 0 && pos0 - window + 1 > 0) j_lo = pos0 - window + 1;
    const int pg_lo = j_lo / LUMEN_PAGE, pg_hi = pos_last / LUMEN_PAGE;
    const int npages = pg_hi - pg_lo + 1;
    const int* bt = block_table + (size_t)b * bt_stride;

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

    if (threadIdx.x == 0) {
        for (int i = 0; i < PT_STAGES; ++i) {
            mbar_init(&k_full[i], 1); mbar_init(&k_empty[i], 1);
            mbar_init(&v_full[i], 1); mbar_init(&v_empty[i], 1);
        }
        for (int i = 0; i < 2; ++i) { mbar_init(&s_full[i], 1); mbar_init(&p_ready[i], 4); mbar_init(&pv_done[i], 1); }
        *abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        // the first tiles are on their way while the block gathers Q: K of pages 0 and 1, V of page 0
        for (int s = 0; s < 2 && s < npages; ++s) {
            const size_t off = ((size_t)bt[pg_lo + s] * nkv + kvh) * (size_t)(LUMEN_PAGE * D);
            mbar_expect_tx(&k_full[s], TILE_BYTES);
            bulk_load(sKV + s * 2 * TILE_BYTES, kcache + off, TILE_BYTES, &k_full[s]);
            if (s == 0) {
                mbar_expect_tx(&v_full[0], TILE_BYTES);
                bulk_load(sKV + TILE_BYTES, vcache + off, TILE_BYTES, &v_full[0]);
            }
        }
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)),
                     "r"(NCOLS)
                     : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    // Q: 128 rows of D values into [D/64][row][64], 16-byte chunk c of a row at c ^ (row & 7).
    for (int idx = threadIdx.x; idx < PT_ROWS * (D / 8); idx += PT_THREADS) {
        const int r = idx / (D / 8), c = idx - r * (D / 8);
        const int tok = r / G, h = r - tok * G;
        uint4 v = make_uint4(0u, 0u, 0u, 0u);
        if (tok < ntok && r < TQ * G)
            v = *reinterpret_cast<const uint4*>(q + ((size_t)(n0 + tok) * nq + kvh * G + h) * D + 8 * c);
        *reinterpret_cast<uint4*>(sQ + (c >> 3) * (PT_ROWS * 128) + r * 128 + (((c & 7) ^ (r & 7)) << 4)) = v;
    }
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");   // Q is read by the tensor cores
    pt_fence_before();
    __syncthreads();
    pt_fence_after();
    const uint32_t tmem_base = *tmem_slot;

    if (warp == 0) {
        if (lane == 0) {
            // K runs one page ahead of V: its slot comes free earlier (see above), and this way
            // no K waits behind a V whose slot is still being read
            // (steps 0 and 1, but for V of page 1, were taken before the Q gather)
            if (npages > 1) {
                const size_t off = ((size_t)bt[pg_lo + 1] * nkv + kvh) * (size_t)(LUMEN_PAGE * D);
                mbar_expect_tx(&v_full[1], TILE_BYTES);
                bulk_load(sKV + 2 * TILE_BYTES + TILE_BYTES, vcache + off, TILE_BYTES, &v_full[1]);
            }
            for (int s = 2; s <= npages && !*abort_flag; ++s) {
                if (s < npages) {
                    const int st = s % PT_STAGES, ph = (s / PT_STAGES) & 1;
                    const size_t off = ((size_t)bt[pg_lo + s] * nkv + kvh) * (size_t)(LUMEN_PAGE * D);
                    if (!mbar_wait(&k_empty[st], ph ^ 1)) { *abort_flag = 1; atomicExch(err, 1); break; }
                    mbar_expect_tx(&k_full[st], TILE_BYTES);
                    bulk_load(sKV + st * 2 * TILE_BYTES, kcache + off, TILE_BYTES, &k_full[st]);
                }
                if (s >= 3) {
                    const int it = s - 1, st = it % PT_STAGES, ph = (it / PT_STAGES) & 1;
                    const size_t off = ((size_t)bt[pg_lo + it] * nkv + kvh) * (size_t)(LUMEN_PAGE * D);
                    if (!mbar_wait(&v_empty[st], ph ^ 1)) { *abort_flag = 1; atomicExch(err, 1); break; }
                    mbar_expect_tx(&v_full[st], TILE_BYTES);
                    bulk_load(sKV + st * 2 * TILE_BYTES + TILE_BYTES, vcache + off, TILE_BYTES, &v_full[st]);
                }
            }
        }
    } else if (warp == 1) {
        if (lane == 0) {
            constexpr uint32_t idesc_qk = pt_idesc(LUMEN_PAGE, 0);
            constexpr uint32_t idesc_pv = pt_idesc(D, 1);
            auto issue_qk = [&](int it) {       // S[it & 1] = Q K(it)^T
                const int st = it % PT_STAGES;
                const uint32_t kt = smem_u32(sKV + st * 2 * TILE_BYTES);
#pragma unroll
                for (int ks = 0; ks < D / 16; ++ks) {
                    const uint32_t aoff = (ks >> 2) * (PT_ROWS * 128) + (ks & 3) * 32;
                    const uint32_t boff = (ks >> 2) * (LUMEN_PAGE * 128) + (ks & 3) * 32;
                    pt_mma(tmem_base + (it & 1) * LUMEN_PAGE, pt_desc(smem_u32(sQ) + aoff, 16),
                           pt_desc(kt + boff, 16), idesc_qk, ks > 0 ? 1u : 0u);
                }
                pt_commit(&k_empty[st]);        // the K slot is free once these MMAs have read it
                pt_commit(&s_full[it & 1]);
            };
            bool ok = mbar_wait(&k_full[0], 0);
            if (ok) {
                pt_fence_after();
                issue_qk(0);
            }
            for (int it = 0; ok && it < npages && !*abort_flag; ++it) {
                if (it + 1 < npages) {
                    const int st1 = (it + 1) % PT_STAGES;
                    if (!mbar_wait(&k_full[st1], ((it + 1) / PT_STAGES) & 1)) { ok = false; break; }
                    pt_fence_after();
                    issue_qk(it + 1);
                }
                const int st = it % PT_STAGES;
                if (!mbar_wait(&v_full[st], (it / PT_STAGES) & 1)) { ok = false; break; }
                if (!mbar_wait(&p_ready[it & 1], (it >> 1) & 1)) { ok = false; break; }
                pt_fence_after();
                const uint32_t vt = smem_u32(sKV + st * 2 * TILE_BYTES + TILE_BYTES);
                // P of this page lies over the first 32 columns of the S buffer it was made from
                const uint32_t pt = tmem_base + (it & 1) * LUMEN_PAGE;
#pragma unroll
                for (int kk = 0; kk < LUMEN_PAGE / 16; ++kk)     // 16 keys a step: 8 columns of P
                    pt_mma_ts(tmem_base + O_COL, pt + kk * 8,
                              pt_desc(vt + kk * (16 * 128), LUMEN_PAGE * 128), idesc_pv, (it > 0 || kk > 0) ? 1u : 0u);
                pt_commit(&v_empty[st]);
                pt_commit(&pv_done[it & 1]);
            }
            if (!ok) { *abort_flag = 1; atomicExch(err, 1); }
        }
    } else {
        const int qd = warp & 3;
        const int r = qd * 32 + lane;                      // this thread's row
        const int tok = r / G, h = r - tok * G;
        const bool row_ok = tok < ntok && r < TQ * G;
        const int prow = pos0 + tok;                       // absolute position of the row's query
        const int lorow = (window > 0) ? prow - window + 1 : 0;
        const uint32_t lane_addr = tmem_base + ((uint32_t)(qd * 32) << 16);
        float m_ref = -INFINITY, l = 0.0f;
        bool ok = true;
        for (int it = 0; it < npages; ++it) {
            if (__any_sync(0xffffffffu, *abort_flag != 0)) { ok = false; break; }
            bool w = mbar_wait(&s_full[it & 1], (it >> 1) & 1);
            if (!__all_sync(0xffffffffu, w)) { ok = false; break; }
            pt_fence_after();
            float s[64];
            pt_ld64(lane_addr + (it & 1) * LUMEN_PAGE, s);
            const int jb = (pg_lo + it) * LUMEN_PAGE;
            const bool full_page = (jb + LUMEN_PAGE - 1 <= prow) && (jb >= lorow);
            if (!__all_sync(0xffffffffu, full_page)) {       // only pages on the diagonal or the window's edge
#pragma unroll
                for (int j = 0; j < 64; ++j) {
                    const bool vis = (jb + j <= prow) && (jb + j >= lorow);
                    s[j] = vis ? s[j] : -INFINITY;
                }
            }
            // row maximum of the raw scores, four independent chains (the scale is positive)
            float mx4[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
#pragma unroll
            for (int j = 0; j < 64; j += 4) {
                mx4[0] = fmaxf(mx4[0], s[j]);
                mx4[1] = fmaxf(mx4[1], s[j + 1]);
                mx4[2] = fmaxf(mx4[2], s[j + 2]);
                mx4[3] = fmaxf(mx4[3], s[j + 3]);
            }
            const float mx = fmaxf(fmaxf(mx4[0], mx4[1]), fmaxf(mx4[2], mx4[3])) * scale_log2;
            // reference for the exponentials: moved only when the maximum has grown a lot
            float corr = 1.0f;
            if (mx > m_ref + PT_RESCALE || m_ref == -INFINITY) {
                const float nref = fmaxf(mx, m_ref);
                if (nref != -INFINITY) {
                    corr = (m_ref == -INFINITY) ? 0.0f : pt_ex2(m_ref - nref);
                    m_ref = nref;
                }
            }
            const float nbase = (m_ref == -INFINITY) ? 0.0f : -m_ref;
            float rs4[4] = {0.0f, 0.0f, 0.0f, 0.0f};
#pragma unroll
            for (int j = 0; j < 64; j += 4) {
                s[j] = pt_ex2(fmaf(s[j], scale_log2, nbase));
                s[j + 1] = (PT_FMA_EX2_OF_4 >= 2) ? pt_ex2_fma(fmaf(s[j + 1], scale_log2, nbase))
                                                  : pt_ex2(fmaf(s[j + 1], scale_log2, nbase));
                s[j + 2] = pt_ex2(fmaf(s[j + 2], scale_log2, nbase));
                s[j + 3] = (PT_FMA_EX2_OF_4 >= 1) ? pt_ex2_fma(fmaf(s[j + 3], scale_log2, nbase))
                                                  : pt_ex2(fmaf(s[j + 3], scale_log2, nbase));
                rs4[0] += s[j];
                rs4[1] += s[j + 1];
                rs4[2] += s[j + 2];
                rs4[3] += s[j + 3];
            }
            l = l * corr + ((rs4[0] + rs4[1]) + (rs4[2] + rs4[3]));
            // O is rescaled rarely; only then must the PV product of the page before be done (it
            // is accumulating into O). P needs no such wait: it goes where this page's scores
            // were, and the product that read the P of two pages ago finished before these
            // scores were made (the tensor pipe runs its products in the order of issue).
            if (it > 0 && __any_sync(0xffffffffu, corr != 1.0f)) {
                w = mbar_wait(&pv_done[(it - 1) & 1], ((it - 1) >> 1) & 1);
                if (!__all_sync(0xffffffffu, w)) { ok = false; break; }
                pt_fence_after();
#pragma unroll 1
                for (int c0 = 0; c0 < D; c0 += 32) {
                    float ov[32];
                    pt_ld32(lane_addr + O_COL + c0, ov);
#pragma unroll
                    for (int j = 0; j < 32; ++j) ov[j] *= corr;
                    pt_st32(lane_addr + O_COL + c0, ov);
                }
            }
            // P row: 64 bfloat16, two a column, keys in rising order
            uint32_t pk[32];
#pragma unroll
            for (int c = 0; c < 32; ++c) pk[c] = pack_bf16(s[2 * c], s[2 * c + 1]);
            pt_st32u(lane_addr + (it & 1) * LUMEN_PAGE, pk);
            asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
            pt_fence_before();
            __syncwarp();
            if (lane == 0) pt_mbar_arrive(&p_ready[it & 1]);
        }
        if (ok) {
            bool w = mbar_wait(&pv_done[(npages - 1) & 1], ((npages - 1) >> 1) & 1);
            ok = __all_sync(0xffffffffu, w);
        }
        if (!ok) {
            *abort_flag = 1;
            if (lane == 0) atomicExch(err, 1);
        } else {
            pt_fence_after();
            const float inv = (l > 0.0f) ? 1.0f / l : 0.0f;
            __nv_bfloat16* dst = out + ((size_t)(n0 + tok) * nq + kvh * G + h) * D;
#pragma unroll 1
            for (int c0 = 0; c0 < D; c0 += 32) {
                float ov[32];
                pt_ld32(lane_addr + O_COL + c0, ov);
                if (row_ok) {
#pragma unroll
                    for (int j = 0; j < 32; j += 8) {
                        uint4 v;
                        v.x = pack_bf16(ov[j] * inv, ov[j + 1] * inv);
                        v.y = pack_bf16(ov[j + 2] * inv, ov[j + 3] * inv);
                        v.z = pack_bf16(ov[j + 4] * inv, ov[j + 5] * inv);
                        v.w = pack_bf16(ov[j + 6] * inv, ov[j + 7] * inv);
                        *reinterpret_cast<uint4*>(dst + c0 + j) = v;
                    }
                }
            }
        }
    }

    pt_fence_before();
    __syncthreads();
    if (warp == 1) {
        pt_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(NCOLS) : "memory");
    }
}

// q, out: bfloat16 [N, nq, d]; cu_q int32 [B+1]; seq_start int32 [B] (cached length of each
// sequence before this step); n_tiles = sum over sequences of ceil(q_len / (128 / (nq/nkv))).
LUMEN_API int lumen_attn_prefill_tc(const void* q, const void* kcache, const void* vcache,
                                    const int* block_table, int bt_stride, const int* cu_q,
                                    const int* seq_start, int B, int n_tiles, void* out, int nq,
                                    int nkv, int d, int window, float scale, int* err,
                                    cudaStream_t stream) {
    if (B <= 0 || n_tiles <= 0) return 0;
    if (nq <= 0 || nkv <= 0 || nq % nkv != 0 || nq / nkv > 16 || window < 0) return LUMEN_ERR_UNSUPPORTED;
    if ((long long)n_tiles * nkv > 2147483647LL) return LUMEN_ERR_UNSUPPORTED;
    dim3 grid(n_tiles * nkv);
    const float scale_log2 = scale * 1.4426950408889634f;
    const __nv_bfloat16* qp = (const __nv_bfloat16*)q;
    const __nv_bfloat16* kp = (const __nv_bfloat16*)kcache;
    const __nv_bfloat16* vp = (const __nv_bfloat16*)vcache;
    cudaError_t e;
    if (d == 128) {
        const int smem = PT_ROWS * 128 * 2 + PT_STAGES * 2 * LUMEN_PAGE * 128 * 2 + 256;
        auto k = attn_prefill_tc_kernel<128>;
        e = cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
        if (e != cudaSuccess) return (int)e;
        e = lumen_launch(k, grid, dim3(PT_THREADS), smem, stream, qp, kp, vp, block_table, bt_stride, cu_q,
                         seq_start, B, (__nv_bfloat16*)out, nq, nkv, window, scale_log2, err);
    } else if (d == 64) {
        const int smem = PT_ROWS * 64 * 2 + PT_STAGES * 2 * LUMEN_PAGE * 64 * 2 + 256;
        auto k = attn_prefill_tc_kernel<64>;
        e = cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
        if (e != cudaSuccess) return (int)e;
        e = lumen_launch(k, grid, dim3(PT_THREADS), smem, stream, qp, kp, vp, block_table, bt_stride, cu_q,
                         seq_start, B, (__nv_bfloat16*)out, nq, nkv, window, scale_log2, err);
    } else {
        return LUMEN_ERR_UNSUPPORTED;
    }
    if (e != cudaSuccess) return (int)e;
    LUMEN_LAUNCH_CHECK();
    return 0;
}
