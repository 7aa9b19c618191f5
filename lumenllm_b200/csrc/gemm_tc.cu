// bfloat16 matrix product on the 5th-generation tensor cores: D[a, b] = sum_k A[a, k] B[b, k],
// both operands row-major with k contiguous ("K-major"), float32 accumulation in tensor memory.
//
//   * Operands reach shared memory by TMA (cp.async.bulk.tensor, 128-byte swizzle, one
//     64-wide k block per stage, no multicast), complete on mbarriers, and are consumed in
//     place by tcgen05.mma through shared-memory descriptors; one thread issues the MMAs.
//   * The accumulator of a 128 x BN tile lives in tensor memory; there are two of them, so
//     the epilogue of one tile (tcgen05.ld -> registers -> global) overlaps the next tile's
//     main loop.
//   * One persistent block per SM walks the list of tiles (static round robin). Warp 0
//     produces (TMA), warp 1 allocates tensor memory and issues the MMAs, warps 2..5 are the
//     epilogue (their index mod 4 selects the 32 lanes of tensor memory each may read).
//
// Two orientations share the code. With many rows of activations (prompts) A = activations and
// B = weights, BN up to 256 (prompt-sized products go to the two-SM kernel further down).
// With few rows (decode, short prompts) the roles are swapped: A = weights, so that the
// 128-row side of the MMA is filled by weight rows, and B = the activations padded to
// 16/32/64/128/256 rows; the product is then a stream over the weights through a TMA ring of five to eight stages (see TC_TRIGGER_AHEAD), and k may be split
// over several tiles so that all SMs pull from HBM. A split writes partial sums [S, M, N] that
// the consumer adds in rising order; S depends on the weight's shape only.
//
// Epilogues: float32 out; or, for a weight whose rows alternate gate_i, up_i, SiLU(gate)*up
// written as bfloat16 (no split then).
//
// Weights are not read row by row. A weight [N, K] is rewritten once, when it is loaded, into
// the image its tiles have in shared memory (lumen_tile_weight): k block after k block (64
// values of k each), within a k block all rows in groups of eight, a group being 8 rows x 128
// bytes = 1,024 contiguous bytes with the 16-byte pieces of row r at the places (piece ^ (r & 7))
// of the 128-byte swizzle; rows padded with zeros to a multiple of 256, k to a multiple of 64.
// Any run of rows that starts at a multiple of 8 is then ONE contiguous piece of memory for a
// given k block, and the copy engine fetches a 128-row tile as 16 KB in a row instead of 128
// pieces of 128 bytes that lie a whole matrix row apart (measured on 148 blocks that each
// stream 1 MB in 16 KB stages: 28.3 against 29.5 us; 3 MB each: 71.8 against 73.3 us). Its map
// describes that memory as a matrix of 128-byte rows without swizzle: row kb * rows_padded + r.
//
// Every wait is bounded: when one runs out the block raises an error flag, stops issuing work,
// lets the other roles run out likewise, frees its tensor memory and returns.
#include <cuda.h>

#include <cstdlib>
#include <mutex>
#include "common.cuh"
#include "mma_utils.cuh"

#define TC_BM 128
#define TC_BK 64
#define TC_THREADS 192
// The swapped (weight-streaming) product lets what follows it in the stream start when this
// many stages of a block's loads are still to be asked for (some 4 us before its stream ends).
// The short kernel behind it (norm, rotary, SiLU) lets ITS dependents go at its very top, so the
// next product's blocks come to rest beside this one's (a ring of six stages is 108 KB: two
// fit an SM) and ask for their first weights just as this product's last loads have been asked
// for: the stream from HBM does not stop between two products of a decode step. Measured at the
// 8B shape, batch 8 (ms a step): 3.40 with 0 stages ahead, 3.34 with 9, 3.30 with 11 to 15, 3.35
// with 18, 3.42 from 24 on and with the trigger at the kernel's top; 3.55 with the trigger right
// after the wait and a ring of ten stages, where the next product starts when this one has left.
#define TC_TRIGGER_AHEAD 12
#define TC_EPI_F32 0
#define TC_EPI_SILU 1
#define TC_EPI_ADD 2          // float32, added to what the output holds (two-SM kernel only)
#define TC_EPI_QKV 3          // heads of 128: q/k RMSNorm, rotation, q out in bfloat16, k and v into the paged cache (two-SM kernel only)

__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void tma_load_2d(void* dst, const CUtensorMap* map, int c0, int c1, uint64_t* bar) {
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];" ::"r"(
            smem_u32(dst)),
        "l"(reinterpret_cast<uint64_t>(map)), "r"(smem_u32(bar)), "r"(c0), "r"(c1)
        : "memory");
}
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_commit(uint64_t* bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar))
                 : "memory");
}
__device__ __forceinline__ void tc_mma(uint32_t d_tmem, uint64_t adesc, uint64_t bdesc, uint32_t idesc,
                                       uint32_t accumulate) {
    asm volatile(
        "{\n .reg .pred p;\n setp.ne.b32 p, %4, 0;\n"
        " tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n}" ::"r"(d_tmem),
        "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
        : "memory");
}
__device__ __forceinline__ void tc_ld16(uint32_t taddr, float (&v)[16]) {
    uint32_t r[16];
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
          "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
        : "r"(taddr));
    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
    for (int i = 0; i < 16; ++i) v[i] = __uint_as_float(r[i]);
}

// Shared-memory descriptor of a K-major tile in the 128-byte swizzle: rows of 128 bytes,
// groups of 8 rows 1024 bytes apart (stride byte offset), version 1, layout type 2.
__device__ __forceinline__ uint64_t tc_smem_desc(uint32_t smem_addr) {
    uint64_t d = 0;
    d |= (uint64_t)((smem_addr >> 4) & 0x3FFF);
    d |= (uint64_t)1 << 16;                 // leading byte offset (unused with swizzle): 1
    d |= (uint64_t)(1024 >> 4) << 32;       // stride byte offset
    d |= (uint64_t)1 << 46;                 // descriptor version
    d |= (uint64_t)2 << 61;                 // SWIZZLE_128B
    return d;
}
// Instruction descriptor: D float32, A and B bfloat16, both K-major, M = 128, N = BN.
__host__ __device__ constexpr uint32_t tc_idesc(int bn) {
    return (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(bn >> 3) << 17) | ((uint32_t)(TC_BM >> 4) << 24);
}

#define TC_TILE_FIXED 200   // fixed part of a tile's time, in columns of tile width (measured: a
                            // 128-wide tile takes 0.75 of the time of a 256-wide one)

struct TcParams {
    float* out_f32;           // EPI_F32: [S, M, N]
    __nv_bfloat16* out_bf16;  // EPI_SILU: [M, N / 2]
    int M, N;                 // rows of activations, rows of the weight
    int rowsA, rowsB;         // rows of the A and of the B operand
    int num_kb;               // 64-wide k blocks in K
    int splits, kb_per_split;
    int w_rows;               // rows of the tiled weight with padding: its k blocks lie this many 128-byte rows apart
    int tma_out;              // two-SM kernel: the output goes through shared memory and the copy engine
    int bn;                   // rows of a B tile: BN, or narrower (a multiple of 16) when that fills the SMs better
    int* err;
    // EPI_QKV: what the rotary kernel would be given
    const float* qw;          // norm weights of q and k heads [128], or null
    const float* kw;
    const float2* cs;         // (cos, sin) [M, 64], or null without rotation
    const int* cache_pos;     // [M] place of a row's token in its sequence
    const int* tok_seq;       // [M] which sequence
    const int* block_table;   // [B, bt_stride] pages
    __nv_bfloat16* kcache;    // [pages, nkv, 64, 128], 128-byte swizzled tiles
    __nv_bfloat16* vcache;
    float eps;
    int bt_stride, nq, nkv, rot;
};

template <int BN, int STAGES, bool SWAP, int EPI>
__global__ void __launch_bounds__(TC_THREADS, 1)
gemm_tc_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
               const TcParams p) {
    constexpr int A_BYTES = TC_BM * 128, B_BYTES = BN * 128;
    constexpr int NCOLS = (2 * BN < 32) ? 32 : 2 * BN;
    extern __shared__ __align__(1024) unsigned char smem_raw[];
    // operand tiles must start on 1024-byte boundaries (the swizzle pattern repeats there)
    unsigned char* smem = smem_raw + ((1024u - (smem_u32(smem_raw) & 1023u)) & 1023u);
    unsigned char* sA = smem;
    unsigned char* sB = smem + STAGES * A_BYTES;
    uint64_t* bars = reinterpret_cast<uint64_t*>(sB + STAGES * B_BYTES);
    uint64_t* full = bars;
    uint64_t* empty = bars + STAGES;
    uint64_t* tfull = bars + 2 * STAGES;
    uint64_t* tempty = bars + 2 * STAGES + 2;
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 2 * STAGES + 4);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int bn = SWAP ? BN : p.bn;            // the slot in shared memory and the accumulator keep BN
    const int tilesA = (p.rowsA + TC_BM - 1) / TC_BM, tilesB = (p.rowsB + bn - 1) / bn;
    const int n_items = tilesA * tilesB * p.splits;
    const uint32_t stage_bytes = A_BYTES + bn * 128;

    if (threadIdx.x == 0) {
        for (int i = 0; i < STAGES; ++i) { mbar_init(&full[i], 1); mbar_init(&empty[i], 1); }
        for (int i = 0; i < 2; ++i) { mbar_init(&tfull[i], 1); mbar_init(&tempty[i], 4); }
        *abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(&tmA)) : "memory");
        asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(&tmB)) : "memory");
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)),
                     "r"(NCOLS)
                     : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;
    // Set-up above depends on nothing. From here on every role waits for the kernels ahead
    // of this one before it touches activations or outputs; the producer first requests
    // weights (below).
    if (warp != 0) pdl_wait();

    // item -> (tile of A, tile of B, split); tiles of A vary fastest so that blocks working at
    // the same time share their B tile through L2
    auto decode = [&](int item, int& ta, int& tb, int& s) {
        s = item % p.splits;
        const int t = item / p.splits;
        ta = t % tilesA;
        tb = t / tilesA;
    };

    if (warp == 0) {
        if (lane == 0) {
            // the sequence of (tile of A, tile of B, k block) this block works through
            int item = blockIdx.x, ta = 0, tb = 0, s = 0, kb = 0, kb1 = 0;
            bool have = item < n_items;
            auto enter = [&]() {
                decode(item, ta, tb, s);
                kb = s * p.kb_per_split;
                kb1 = min(kb + p.kb_per_split, p.num_kb);
            };
            auto advance = [&]() {
                if (++kb >= kb1) {
                    item += gridDim.x;
                    have = item < n_items;
                    if (have) enter();
                }
            };
            if (have) enter();
            // Weights never change, so the first ring of weight tiles is requested before the
            // kernel ahead of this one in the stream has finished; activations only after.
            int npre = 0, pt[STAGES], pk[STAGES];
            while (have && npre < STAGES) {
                pt[npre] = SWAP ? tb : ta;
                pk[npre] = kb;
                mbar_expect_tx(&full[npre], stage_bytes);
                if (SWAP) tma_load_2d(sA + npre * A_BYTES, &tmA, 0, kb * p.w_rows + ta * TC_BM, &full[npre]);
                else      tma_load_2d(sB + npre * B_BYTES, &tmB, 0, kb * p.w_rows + tb * bn, &full[npre]);
                ++npre;
                advance();
            }
            pdl_wait();
            for (int i = 0; i < npre; ++i) {
                if (SWAP) tma_load_2d(sB + i * B_BYTES, &tmB, pk[i] * TC_BK, pt[i] * bn, &full[i]);
                else      tma_load_2d(sA + i * A_BYTES, &tmA, pk[i] * TC_BK, pt[i] * TC_BM, &full[i]);
            }
            const int my_items = blockIdx.x < n_items ? (n_items - 1 - (int)blockIdx.x) / (int)gridDim.x + 1 : 0;
            const int trigger_at = my_items * p.kb_per_split - TC_TRIGGER_AHEAD;
            bool triggered = false;
            for (int it = npre; have && !*abort_flag; ++it, advance()) {
                if (!triggered && it >= trigger_at) { pdl_trigger(); triggered = true; }
                const int st = it % STAGES, ph = (it / STAGES) & 1;
                if (!mbar_wait(&empty[st], ph ^ 1)) { *abort_flag = 1; atomicExch(p.err, 1); break; }
                mbar_expect_tx(&full[st], stage_bytes);
                if (SWAP) {
                    tma_load_2d(sA + st * A_BYTES, &tmA, 0, kb * p.w_rows + ta * TC_BM, &full[st]);
                    tma_load_2d(sB + st * B_BYTES, &tmB, kb * TC_BK, tb * bn, &full[st]);
                } else {
                    tma_load_2d(sA + st * A_BYTES, &tmA, kb * TC_BK, ta * TC_BM, &full[st]);
                    tma_load_2d(sB + st * B_BYTES, &tmB, 0, kb * p.w_rows + tb * bn, &full[st]);
                }
            }
            // every load of this block is asked for: what follows in the stream may start
            pdl_trigger();
        } else {
            pdl_wait();
        }
    } else if (warp == 1) {
        if (lane == 0) {
            const uint32_t idesc = tc_idesc(bn);
            int it = 0, acc_it = 0;
            for (int item = blockIdx.x; item < n_items && !*abort_flag; item += gridDim.x, ++acc_it) {
                int ta, tb, s;
                decode(item, ta, tb, s);
                const int kb0 = s * p.kb_per_split, kb1 = min(kb0 + p.kb_per_split, p.num_kb);
                const int acc = acc_it & 1, aph = (acc_it >> 1) & 1;
                if (!mbar_wait(&tempty[acc], aph ^ 1)) { *abort_flag = 1; atomicExch(p.err, 1); break; }
                tc_fence_after();
                const uint32_t d_tmem = tmem_base + acc * BN;
                bool ok = true;
                for (int kb = kb0; kb < kb1; ++kb, ++it) {
                    const int st = it % STAGES, ph = (it / STAGES) & 1;
                    if (!mbar_wait(&full[st], ph)) { ok = false; break; }
                    tc_fence_after();
                    const uint64_t ad = tc_smem_desc(smem_u32(sA + st * A_BYTES));
                    const uint64_t bd = tc_smem_desc(smem_u32(sB + st * B_BYTES));
#pragma unroll
                    for (int k = 0; k < TC_BK / 16; ++k)   // 16 values of k = 32 bytes = 2 units of 16 bytes
                        tc_mma(d_tmem, ad + 2 * k, bd + 2 * k, idesc, (kb > kb0 || k > 0) ? 1u : 0u);
                    tc_commit(&empty[st]);     // the stage is free once these MMAs have read it
                }
                if (!ok) { *abort_flag = 1; atomicExch(p.err, 1); break; }
                tc_commit(&tfull[acc]);        // the accumulator is complete once all MMAs are done
            }
        }
    } else {
        const int q = warp & 3;                // lanes of tensor memory this warp may read
        const int row_in_tile = q * 32 + lane;
        int acc_it = 0;
        for (int item = blockIdx.x; item < n_items; item += gridDim.x, ++acc_it) {
            // one decision per warp: the loads below are warp-wide instructions
            if (__any_sync(0xffffffffu, *abort_flag != 0)) break;
            int ta, tb, s;
            decode(item, ta, tb, s);
            const int acc = acc_it & 1, aph = (acc_it >> 1) & 1;
            bool ok = mbar_wait(&tfull[acc], aph);
            ok = __all_sync(0xffffffffu, ok);
            if (!ok) { *abort_flag = 1; if (lane == 0) atomicExch(p.err, 1); break; }
            tc_fence_after();
            const int a = ta * TC_BM + row_in_tile;                 // row of the A operand
            const uint32_t taddr0 = tmem_base + ((uint32_t)(q * 32) << 16) + acc * BN;
#pragma unroll 1
            for (int c0 = 0; c0 < bn; c0 += 16) {
                float v[16];
                tc_ld16(taddr0 + c0, v);
                const int b0 = tb * bn + c0;                        // first row of the B operand
                if (EPI == TC_EPI_F32) {
                    float* o = p.out_f32 + (size_t)s * p.M * p.N;
                    if (!SWAP) {            // a = activation row m, b = weight row n
                        if (a < p.M) {
                            float* dst = o + (size_t)a * p.N + b0;
                            if ((p.N & 3) == 0 && b0 + 16 <= p.N) {
#pragma unroll
                                for (int j = 0; j < 16; j += 4)
                                    *reinterpret_cast<float4*>(dst + j) = make_float4(v[j], v[j + 1], v[j + 2], v[j + 3]);
                            } else {
#pragma unroll
                                for (int j = 0; j < 16; ++j)
                                    if (b0 + j < p.N) dst[j] = v[j];
                            }
                        }
                    } else {                // a = weight row n, b = activation row m
#pragma unroll
                        for (int j = 0; j < 16; ++j)
                            if (a < p.N && b0 + j < p.M) o[(size_t)(b0 + j) * p.N + a] = v[j];
                    }
                } else {
                    const int half = p.N >> 1;
                    if (!SWAP) {            // columns 2i, 2i+1 of this thread are gate_i, up_i
                        if (a < p.M) {
                            __nv_bfloat16* dst = p.out_bf16 + (size_t)a * half + (b0 >> 1);
                            float z[8];
#pragma unroll
                            for (int j = 0; j < 8; ++j) z[j] = v[2 * j] / (1.0f + expf(-v[2 * j])) * v[2 * j + 1];
                            if ((half & 7) == 0 && b0 + 16 <= p.N) {
                                uint4 w;
                                w.x = pack_bf16(z[0], z[1]); w.y = pack_bf16(z[2], z[3]);
                                w.z = pack_bf16(z[4], z[5]); w.w = pack_bf16(z[6], z[7]);
                                *reinterpret_cast<uint4*>(dst) = w;
                            } else {
#pragma unroll
                                for (int j = 0; j < 8; ++j)
                                    if (b0 + 2 * j + 1 < p.N) dst[j] = __float2bfloat16_rn(z[j]);
                            }
                        }
                    } else {                // lanes 2i, 2i+1 hold gate_i, up_i of every column
#pragma unroll
                        for (int j = 0; j < 16; ++j) {
                            const float up = __shfl_xor_sync(0xffffffffu, v[j], 1);
                            if ((lane & 1) == 0 && a + 1 < p.N && b0 + j < p.M)
                                p.out_bf16[(size_t)(b0 + j) * half + (a >> 1)] =
                                    __float2bfloat16_rn(v[j] / (1.0f + expf(-v[j])) * up);
                        }
                    }
                }
            }
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(&tempty[acc]);
        }
    }

    tc_fence_before();
    __syncthreads();
    if (warp == 1) {
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(NCOLS) : "memory");
    }
}

// ------------------------------------------------------------------- two SMs on one tile
// For prompts the single-SM kernel above is held back by what it must pull from L2: 48 KB of
// operands for every 128 x 256 x 64 block of products. Here two CTAs on neighbouring SMs (a
// cluster of two) share a 256 x 256 tile: each loads its own 128 rows of activations and its own
// 128 rows of the weight tile (32 KB), and one thread of the even CTA issues
// tcgen05.mma.cta_group::2, which reads both halves of both operands from the two shared
// memories and accumulates each CTA's 128 rows in that CTA's own tensor memory. The same
// products need a third less operand traffic.
//
// Protocol (the barriers of both CTAs sit at the same offsets):
//   full[s]   in the even CTA only: its producer announces 64 KB, and all four TMA loads of a
//             stage, its own two and the odd CTA's two, complete on it.
//   empty[s]  in both: tcgen05.commit multicasts the "MMAs have read stage s" signal.
//   tfull[a]  in both: the same multicast commit once a tile's last MMA is issued.
//   tempty[a] in the even CTA only: the eight epilogue warps of both CTAs arrive on it.
// Every wait is bounded in time; when one runs out the CTA raises the error flag and all
// roles of both CTAs run out in turn and meet at the closing cluster barrier.
#define TC2_STAGES 5
#define TC2_OUT_BYTES (TC_BM * 128)       // one staged block of output: 128 rows of 128 bytes
#define TC2_TILE_BYTES (TC_BM * 128)      // one 128 x 64 operand tile

__device__ __forceinline__ uint32_t cluster_ctarank() {
    uint32_t r;
    asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
    return r;
}
__device__ __forceinline__ uint32_t map_to_cta(uint32_t smem_addr, uint32_t rank) {
    uint32_t r;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(smem_addr), "r"(rank));
    return r;
}
__device__ __forceinline__ void cluster_sync_all() {
    asm volatile("barrier.cluster.arrive.release.aligned;\n barrier.cluster.wait.acquire.aligned;" ::: "memory");
}
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t cluster_addr) {
    asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(cluster_addr) : "memory");
}
__device__ __forceinline__ uint64_t global_ns() {
    uint64_t t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    return t;
}
// Wait with cluster-scope acquire, given up after a quarter of a second.
__device__ __forceinline__ bool mbar_wait_timed(uint64_t* bar, uint32_t parity) {
    uint64_t t0 = 0;
    for (uint32_t it = 0;; ++it) {
        uint32_t ok;
        asm volatile(
            "{\n .reg .pred p;\n mbarrier.try_wait.parity.acquire.cluster.shared::cta.b64 p, [%1], %2;\n"
            " selp.u32 %0, 1, 0, p;\n}"
            : "=r"(ok)
            : "r"(smem_u32(bar)), "r"(parity)
            : "memory");
        if (ok) return true;
        if ((it & 255u) == 255u) {
            const uint64_t now = global_ns();
            if (t0 == 0) t0 = now;
            else if (now - t0 > 250000000ull) return false;
        }
    }
}
// TMA load into this CTA's shared memory that completes on a barrier of either CTA of the pair.
__device__ __forceinline__ void tma_load_2d_pair(void* dst, const CUtensorMap* map, int c0, int c1,
                                                 uint32_t bar_cluster_addr) {
    asm volatile(
        "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes"
        " [%0], [%1, {%3, %4}], [%2];" ::"r"(smem_u32(dst)),
        "l"(reinterpret_cast<uint64_t>(map)), "r"(bar_cluster_addr), "r"(c0), "r"(c1)
        : "memory");
}
__device__ __forceinline__ void tc2_commit_both(uint64_t* bar) {
    asm volatile(
        "tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;" ::"r"(
            smem_u32(bar)),
        "h"((uint16_t)3)
        : "memory");
}
__device__ __forceinline__ void tc2_mma(uint32_t d_tmem, uint64_t adesc, uint64_t bdesc, uint32_t idesc,
                                        uint32_t accumulate) {
    asm volatile(
        "{\n .reg .pred p;\n setp.ne.b32 p, %4, 0;\n"
        " tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n}" ::"r"(d_tmem),
        "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
        : "memory");
}
__device__ __forceinline__ void tc_ld32(uint32_t taddr, float (&v)[32]) {
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
// Store of a staged [128 rows][128 bytes] block (128-byte swizzle) to the output matrix; rows
// and columns beyond the matrix are left out by the copy engine.
__device__ __forceinline__ void tma_store_2d(const CUtensorMap* map, int c0, int c1, const void* src) {
    asm volatile("cp.async.bulk.tensor.2d.global.shared::cta.bulk_group [%0, {%2, %3}], [%1];" ::"l"(
                     reinterpret_cast<uint64_t>(map)),
                 "r"(smem_u32(src)), "r"(c0), "r"(c1)
                 : "memory");
}
// The same, added to the output's float32 values by the copy engine (one add an element).
__device__ __forceinline__ void tma_reduce_add_2d(const CUtensorMap* map, int c0, int c1, const void* src) {
    asm volatile("cp.reduce.async.bulk.tensor.2d.global.shared::cta.add.tile.bulk_group [%0, {%2, %3}], [%1];" ::"l"(
                     reinterpret_cast<uint64_t>(map)),
                 "r"(smem_u32(src)), "r"(c0), "r"(c1)
                 : "memory");
}
__device__ __forceinline__ void epi_bar() { asm volatile("bar.sync 1, 128;" ::: "memory"); }
// True in all 128 epilogue threads if it is true in any of them.
__device__ __forceinline__ bool epi_any(bool pred) {
    uint32_t r;
    asm volatile(
        "{\n .reg .pred p, q;\n setp.ne.u32 q, %1, 0;\n bar.red.or.pred p, 1, 128, q;\n selp.u32 %0, 1, 0, p;\n}"
        : "=r"(r)
        : "r"((uint32_t)pred)
        : "memory");
    return r != 0;
}

// D float32, A and B bfloat16, K-major, M = 256 over the pair, N = 256.
__host__ __device__ constexpr uint32_t tc2_idesc() {
    return (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(256 >> 3) << 17) | ((uint32_t)(256 >> 4) << 24);
}

template <int EPI>
__global__ void __launch_bounds__(TC_THREADS, 1)
gemm_tc2_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
                const __grid_constant__ CUtensorMap tmC, const TcParams p) {
    constexpr int STAGES = TC2_STAGES;
    extern __shared__ __align__(1024) unsigned char smem_raw[];
    unsigned char* smem = smem_raw + ((1024u - (smem_u32(smem_raw) & 1023u)) & 1023u);
    unsigned char* sA = smem;
    unsigned char* sB = smem + STAGES * TC2_TILE_BYTES;
    constexpr int NOUT = (EPI == TC_EPI_QKV) ? 4 : 2;               // staged output blocks
    unsigned char* sOut = sB + STAGES * TC2_TILE_BYTES;
    uint64_t* bars = reinterpret_cast<uint64_t*>(sOut + NOUT * TC2_OUT_BYTES);
    float* sG = reinterpret_cast<float*>(reinterpret_cast<unsigned char*>(bars) + 256);   // EPI_QKV: the norms' weights, q then k
    uint64_t* full = bars;
    uint64_t* empty = bars + STAGES;
    uint64_t* tfull = bars + 2 * STAGES;
    uint64_t* tempty = bars + 2 * STAGES + 2;
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 2 * STAGES + 4);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t rank = cluster_ctarank();          // 0: issues the MMAs; 1: its peer
    const int pair = blockIdx.x >> 1, n_pairs = gridDim.x >> 1;
    const int tilesA = (p.rowsA + 255) / 256, tilesB = (p.rowsB + 255) / 256;
    const int n_items = tilesA * tilesB;

    if (threadIdx.x == 0) {
        for (int i = 0; i < STAGES; ++i) { mbar_init(&full[i], 1); mbar_init(&empty[i], 1); }
        for (int i = 0; i < 2; ++i) { mbar_init(&tfull[i], 1); mbar_init(&tempty[i], 8); }
        *abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(&tmA)) : "memory");
        asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(&tmB)) : "memory");
        asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(&tmC)) : "memory");
    }
    if (warp == 1) {
        // each CTA takes all 512 columns of its own tensor memory, so both get the same address
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)),
                     "r"(512)
                     : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    cluster_sync_all();                   // the peer's barriers exist before anything signals them
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;
    if (tmem_base != 0 && threadIdx.x == 0) atomicExch(p.err, 1);   // the pair needs equal addresses

    auto decode = [&](int item, int& ta, int& tb) {
        ta = item % tilesA;
        tb = item / tilesA;
    };

    if (warp == 0) {
        if (lane == 0) {
            const uint32_t full0 = map_to_cta(smem_u32(full), 0);     // the even CTA's full[0]
            int item = pair, ta = 0, tb = 0, kb = 0;
            bool have = item < n_items;
            if (have) decode(item, ta, tb);
            auto advance = [&]() {
                if (++kb >= p.num_kb) {
                    kb = 0;
                    item += n_pairs;
                    have = item < n_items;
                    if (have) decode(item, ta, tb);
                }
            };
            // Weights never change: the first ring of weight tiles is requested before the
            // kernel ahead of this one has finished; activations only after.
            int npre = 0, pa[STAGES], pk[STAGES];
            while (have && npre < STAGES) {
                pa[npre] = ta;
                pk[npre] = kb;
                if (rank == 0) mbar_expect_tx(&full[npre], 4 * TC2_TILE_BYTES);
                tma_load_2d_pair(sB + npre * TC2_TILE_BYTES, &tmB, 0, kb * p.w_rows + tb * 256 + (int)rank * 128,
                                 full0 + npre * 8);
                ++npre;
                advance();
            }
            pdl_wait();
            pdl_trigger();
            for (int i = 0; i < npre; ++i)
                tma_load_2d_pair(sA + i * TC2_TILE_BYTES, &tmA, pk[i] * TC_BK, pa[i] * 256 + (int)rank * 128,
                                 full0 + i * 8);
            for (int it = npre; have && !*abort_flag; ++it, advance()) {
                const int st = it % STAGES, ph = (it / STAGES) & 1;
                if (!mbar_wait_timed(&empty[st], ph ^ 1)) { *abort_flag = 1; atomicExch(p.err, 1); break; }
                if (rank == 0) mbar_expect_tx(&full[st], 4 * TC2_TILE_BYTES);
                tma_load_2d_pair(sA + st * TC2_TILE_BYTES, &tmA, kb * TC_BK, ta * 256 + (int)rank * 128, full0 + st * 8);
                tma_load_2d_pair(sB + st * TC2_TILE_BYTES, &tmB, 0, kb * p.w_rows + tb * 256 + (int)rank * 128, full0 + st * 8);
            }
        } else {
            pdl_wait();
        }
    } else if (warp == 1) {
        pdl_wait();
        if (lane == 0 && rank == 0) {
            constexpr uint32_t idesc = tc2_idesc();
            int it = 0, acc_it = 0;
            for (int item = pair; item < n_items && !*abort_flag; item += n_pairs, ++acc_it) {
                const int acc = acc_it & 1, aph = (acc_it >> 1) & 1;
                if (!mbar_wait_timed(&tempty[acc], aph ^ 1)) { *abort_flag = 1; atomicExch(p.err, 1); break; }
                tc_fence_after();
                const uint32_t d_tmem = tmem_base + acc * 256;
                bool ok = true;
                for (int kb = 0; kb < p.num_kb; ++kb, ++it) {
                    const int st = it % STAGES, ph = (it / STAGES) & 1;
                    if (!mbar_wait_timed(&full[st], ph)) { ok = false; break; }
                    tc_fence_after();
                    const uint64_t ad = tc_smem_desc(smem_u32(sA + st * TC2_TILE_BYTES));
                    const uint64_t bd = tc_smem_desc(smem_u32(sB + st * TC2_TILE_BYTES));
#pragma unroll
                    for (int k = 0; k < TC_BK / 16; ++k)
                        tc2_mma(d_tmem, ad + 2 * k, bd + 2 * k, idesc, (kb > 0 || k > 0) ? 1u : 0u);
                    tc2_commit_both(&empty[st]);
                }
                if (!ok) { *abort_flag = 1; atomicExch(p.err, 1); break; }
                tc2_commit_both(&tfull[acc]);
            }
        }
    } else {
        pdl_wait();
        const int q = warp & 3;
        const int row_in_tile = q * 32 + lane;
        if (EPI == TC_EPI_QKV) {
            sG[row_in_tile] = p.qw ? p.qw[row_in_tile] : 1.0f;
            sG[128 + row_in_tile] = p.kw ? p.kw[row_in_tile] : 1.0f;
            epi_bar();
        }
        const uint32_t tempty0 = map_to_cta(smem_u32(tempty), 0);
        const bool issuer = (warp == 2 && lane == 0);    // hands staged blocks to the copy engine
        int acc_it = 0, out_it = 0;
        for (int item = pair; item < n_items; item += n_pairs, ++acc_it) {
            int ta, tb;
            decode(item, ta, tb);
            const int acc = acc_it & 1, aph = (acc_it >> 1) & 1;
            // EPI_QKV: what a row needs besides the products is fetched while the tensor cores
            // still work on the tile: its 64 (cos, sin) pairs and, for key and value heads, its page
            float4 csr[EPI == TC_EPI_QKV ? 32 : 1];
            int cpos = 0, page = 0;
            const int a = ta * 256 + (int)rank * 128 + row_in_tile;
            const bool row_ok = a < p.M;
            if (EPI == TC_EPI_QKV) {
                if (p.rot == 128 && row_ok && tb * 2 < p.nq + p.nkv) {
                    const float4* src = reinterpret_cast<const float4*>(p.cs + (size_t)a * 64);
#pragma unroll
                    for (int j = 0; j < 32; ++j) csr[j] = __ldg(src + j);
                } else {
#pragma unroll
                    for (int j = 0; j < 32; ++j) csr[j] = make_float4(1.f, 0.f, 1.f, 0.f);
                }
                if (row_ok && tb * 2 + 1 >= p.nq) {
                    cpos = p.cache_pos[a];
                    page = p.block_table[(size_t)p.tok_seq[a] * p.bt_stride + cpos / LUMEN_PAGE];
                }
            }
            const bool ok = mbar_wait_timed(&tfull[acc], aph);
            // one decision for all four warps: they meet at barriers further down
            if (epi_any(!ok || *abort_flag != 0)) { *abort_flag = 1; if (lane == 0) atomicExch(p.err, 1); break; }
            tc_fence_after();
            const uint32_t taddr0 = tmem_base + ((uint32_t)(q * 32) << 16) + acc * 256;
            const int row0 = ta * 256 + (int)rank * 128;                // first activation row of this CTA
            if (EPI == TC_EPI_QKV) {
                // A tile is two heads of 128 columns, and a thread holds a whole row of each: the
                // head's RMSNorm and the rotation of the pairs (i, i + 64) stay inside the thread.
                // A head is staged as two blocks of [128 rows][64 bfloat16] (columns 0-63 and
                // 64-127); the two heads of a tile have a pair of blocks each, so the second is
                // staged while the first is being copied out. A query head leaves through two TMA
                // stores; a key or value head goes row by row, 128 bytes a block, to the row's
                // place in its page, whose tiles have the same 128-byte swizzle (the row's chunks
                // are staged in the order of the destination row, so the copy is plain).
                const int nheads = p.nq + 2 * p.nkv;
#pragma unroll 1
                for (int hh = 0; hh < 2; ++hh) {
                    const int head = tb * 2 + hh;
                    if (head >= nheads) {     // a last tile of one head: an empty group keeps the count of two a tile
                        asm volatile("cp.async.bulk.commit_group;" ::: "memory");
                        break;
                    }
                    const bool is_q = head < p.nq, is_k = !is_q && head < p.nq + p.nkv;
                    const uint32_t tcol = taddr0 + hh * 128;
                    const float* gw = (is_q && p.qw) ? sG : ((is_k && p.kw) ? sG + 128 : nullptr);
                    unsigned char* blk0 = sOut + (2 * hh) * TC2_OUT_BYTES;
                    unsigned char* blk1 = blk0 + TC2_OUT_BYTES;
                    float scale = 1.0f;
                    if (gw) {
                        float ss = 0.0f;
#pragma unroll 1
                        for (int c = 0; c < 4; ++c) {
                            float v[32];
                            tc_ld32(tcol + 32 * c, v);
#pragma unroll
                            for (int j = 0; j < 32; ++j) ss += v[j] * v[j];
                        }
                        scale = 1.0f / sqrtf(ss / 128.0f + p.eps);
                    }
                    // this head's blocks are free once the copies of the tile before have read them:
                    // at most the other head's group may still be in flight
                    asm volatile("cp.async.bulk.wait_group.read 1;" ::: "memory");
                    epi_bar();
                    int r_dst = row_in_tile;
                    __nv_bfloat16* dst = nullptr;
                    if (!is_q && row_ok) {
                        const int kvh = is_k ? head - p.nq : head - p.nq - p.nkv;
                        r_dst = cpos % LUMEN_PAGE;
                        dst = (is_k ? p.kcache : p.vcache) + ((size_t)page * p.nkv + kvh) * (LUMEN_PAGE * 128) +
                              (size_t)r_dst * 64;
                    }
                    const uint32_t swz = (uint32_t)(r_dst & 7);
                    const bool rotate = (is_q || is_k) && p.rot == 128;
#pragma unroll
                    for (int hf = 0; hf < 2; ++hf) {
                        float lo[32], hi[32];
                        tc_ld32(tcol + 32 * hf, lo);
                        tc_ld32(tcol + 64 + 32 * hf, hi);
                        if (gw) {
#pragma unroll
                            for (int j = 0; j < 32; j += 4) {
                                const float4 g0 = *reinterpret_cast<const float4*>(gw + 32 * hf + j);
                                const float4 g1 = *reinterpret_cast<const float4*>(gw + 64 + 32 * hf + j);
                                lo[j] = lo[j] * scale * g0.x; lo[j + 1] = lo[j + 1] * scale * g0.y;
                                lo[j + 2] = lo[j + 2] * scale * g0.z; lo[j + 3] = lo[j + 3] * scale * g0.w;
                                hi[j] = hi[j] * scale * g1.x; hi[j + 1] = hi[j + 1] * scale * g1.y;
                                hi[j + 2] = hi[j + 2] * scale * g1.z; hi[j + 3] = hi[j + 3] * scale * g1.w;
                            }
                        }
                        if (rotate) {       // x'_i = x_i cos - x_{i+64} sin, x'_{i+64} = x_i sin + x_{i+64} cos
#pragma unroll
                            for (int j = 0; j < 32; j += 2) {
                                const float4 c = csr[16 * hf + (j >> 1)];   // (cos, sin) of pairs j and j + 1
                                const float l0 = lo[j], h0 = hi[j], l1 = lo[j + 1], h1 = hi[j + 1];
                                lo[j] = l0 * c.x - h0 * c.y; hi[j] = l0 * c.y + h0 * c.x;
                                lo[j + 1] = l1 * c.z - h1 * c.w; hi[j + 1] = l1 * c.w + h1 * c.z;
                            }
                        }
#pragma unroll
                        for (int ch = 0; ch < 4; ++ch) {
                            const uint32_t at = (uint32_t)row_in_tile * 128 + ((((uint32_t)(4 * hf + ch)) ^ swz) << 4);
                            uint4 w;
                            w.x = pack_bf16(lo[8 * ch], lo[8 * ch + 1]); w.y = pack_bf16(lo[8 * ch + 2], lo[8 * ch + 3]);
                            w.z = pack_bf16(lo[8 * ch + 4], lo[8 * ch + 5]); w.w = pack_bf16(lo[8 * ch + 6], lo[8 * ch + 7]);
                            *reinterpret_cast<uint4*>(blk0 + at) = w;
                            w.x = pack_bf16(hi[8 * ch], hi[8 * ch + 1]); w.y = pack_bf16(hi[8 * ch + 2], hi[8 * ch + 3]);
                            w.z = pack_bf16(hi[8 * ch + 4], hi[8 * ch + 5]); w.w = pack_bf16(hi[8 * ch + 6], hi[8 * ch + 7]);
                            *reinterpret_cast<uint4*>(blk1 + at) = w;
                        }
                    }
                    if (hh == 1 || head + 1 >= nheads) {                // the accumulator has been read out
                        tc_fence_before();
                        __syncwarp();
                        if (lane == 0) mbar_arrive_cluster(tempty0 + acc * 8);
                    }
                    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
                    epi_bar();
                    if (is_q) {
                        if (issuer && row0 < p.M) {
                            tma_store_2d(&tmC, head * 128, row0, blk0);
                            tma_store_2d(&tmC, head * 128 + 64, row0, blk1);
                        }
                    } else {
                        // a warp writes its own 32 rows, four rows an instruction: eight lanes
                        // take the eight 16-byte chunks of a row's 128 bytes in a block
                        const unsigned long long dptr = reinterpret_cast<unsigned long long>(dst);
#pragma unroll 1
                        for (int i = 0; i < 8; ++i) {
                            const int src_lane = 4 * i + (lane >> 3);
                            const unsigned long long d = __shfl_sync(0xffffffffu, dptr, src_lane);
                            if (d != 0ull) {
                                const uint32_t at = (uint32_t)(q * 32 + src_lane) * 128 + (uint32_t)(lane & 7) * 16;
                                __nv_bfloat16* drow = reinterpret_cast<__nv_bfloat16*>(d);
                                *reinterpret_cast<uint4*>(drow + (lane & 7) * 8) = *reinterpret_cast<const uint4*>(blk0 + at);
                                *reinterpret_cast<uint4*>(drow + LUMEN_PAGE * 64 + (lane & 7) * 8) =
                                    *reinterpret_cast<const uint4*>(blk1 + at);
                            }
                        }
                    }
                    asm volatile("cp.async.bulk.commit_group;" ::: "memory");
                }
                continue;
            }
            if (p.tma_out) {
                // Through shared memory: each thread puts 32 columns of its row into a staged
                // block (128 rows of 128 bytes, 16-byte chunk c of row r at c ^ (r & 7), which
                // keeps the stores free of bank conflicts); when a block is full one thread hands
                // it to the copy engine, which writes whole lines and clips at the matrix's edge.
                // Two blocks alternate, so the next is filled while the last is being read.
                constexpr int SUBS = (EPI != TC_EPI_SILU) ? 1 : 4;       // 32-column loads per staged block
                unsigned char* myrow0 = sOut + row_in_tile * 128;
                const uint32_t sw = (uint32_t)(row_in_tile & 7);
#pragma unroll 1
                for (int cb = 0; cb < 256 / (32 * SUBS); ++cb, ++out_it) {
                    unsigned char* blk = sOut + (out_it & 1) * TC2_OUT_BYTES;
                    unsigned char* myrow = myrow0 + (out_it & 1) * TC2_OUT_BYTES;
                    if (issuer) asm volatile("cp.async.bulk.wait_group.read 1;" ::: "memory");
                    epi_bar();                                          // the block's last store has read it
#pragma unroll
                    for (int sub = 0; sub < SUBS; ++sub) {
                        float v[32];
                        tc_ld32(taddr0 + (cb * SUBS + sub) * 32, v);
                        if (EPI != TC_EPI_SILU) {
#pragma unroll
                            for (int j = 0; j < 8; ++j)
                                *reinterpret_cast<float4*>(myrow + (((uint32_t)j ^ sw) << 4)) =
                                    make_float4(v[4 * j], v[4 * j + 1], v[4 * j + 2], v[4 * j + 3]);
                        } else {        // columns 2i, 2i+1 of this thread are gate_i, up_i
                            float z[16];
#pragma unroll
                            for (int j = 0; j < 16; ++j) z[j] = v[2 * j] / (1.0f + expf(-v[2 * j])) * v[2 * j + 1];
#pragma unroll
                            for (int h = 0; h < 2; ++h) {
                                uint4 w;
                                w.x = pack_bf16(z[8 * h], z[8 * h + 1]); w.y = pack_bf16(z[8 * h + 2], z[8 * h + 3]);
                                w.z = pack_bf16(z[8 * h + 4], z[8 * h + 5]); w.w = pack_bf16(z[8 * h + 6], z[8 * h + 7]);
                                *reinterpret_cast<uint4*>(myrow + (((uint32_t)(2 * sub + h) ^ sw) << 4)) = w;
                            }
                        }
                    }
                    if (cb == 256 / (32 * SUBS) - 1) {                  // the accumulator has been read out
                        tc_fence_before();
                        __syncwarp();
                        if (lane == 0) mbar_arrive_cluster(tempty0 + acc * 8);
                    }
                    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
                    epi_bar();
                    if (issuer) {
                        const int col0 = (EPI != TC_EPI_SILU) ? tb * 256 + cb * 32 : tb * 128 + cb * 64;
                        const int ncols = (EPI != TC_EPI_SILU) ? p.N : (p.N >> 1);
                        if (row0 < p.M && col0 < ncols) {
                            if (EPI == TC_EPI_ADD) tma_reduce_add_2d(&tmC, col0, row0, blk);
                            else tma_store_2d(&tmC, col0, row0, blk);
                        }
                        // a group a block, stored or not: the wait above counts groups
                        asm volatile("cp.async.bulk.commit_group;" ::: "memory");
                    }
                }
                continue;
            }
#pragma unroll 1
            for (int c0 = 0; c0 < 256; c0 += 16) {
                float v[16];
                tc_ld16(taddr0 + c0, v);
                const int b0 = tb * 256 + c0;                           // weight row n
                if (a >= p.M || b0 >= p.N) continue;
                if (EPI == TC_EPI_F32) {
                    float* dst = p.out_f32 + (size_t)a * p.N + b0;
                    if ((p.N & 3) == 0 && b0 + 16 <= p.N) {
#pragma unroll
                        for (int j = 0; j < 16; j += 4)
                            *reinterpret_cast<float4*>(dst + j) = make_float4(v[j], v[j + 1], v[j + 2], v[j + 3]);
                    } else {
#pragma unroll
                        for (int j = 0; j < 16; ++j)
                            if (b0 + j < p.N) dst[j] = v[j];
                    }
                } else {            // columns 2i, 2i+1 of this thread are gate_i, up_i
                    const int half = p.N >> 1;
                    __nv_bfloat16* dst = p.out_bf16 + (size_t)a * half + (b0 >> 1);
                    float z[8];
#pragma unroll
                    for (int j = 0; j < 8; ++j) z[j] = v[2 * j] / (1.0f + expf(-v[2 * j])) * v[2 * j + 1];
                    if ((half & 7) == 0 && b0 + 16 <= p.N) {
                        uint4 w;
                        w.x = pack_bf16(z[0], z[1]); w.y = pack_bf16(z[2], z[3]);
                        w.z = pack_bf16(z[4], z[5]); w.w = pack_bf16(z[6], z[7]);
                        *reinterpret_cast<uint4*>(dst) = w;
                    } else {
#pragma unroll
                        for (int j = 0; j < 8; ++j)
                            if (b0 + 2 * j + 1 < p.N) dst[j] = __float2bfloat16_rn(z[j]);
                    }
                }
            }
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive_cluster(tempty0 + acc * 8);
        }
        if (issuer || EPI == TC_EPI_QKV) asm volatile("cp.async.bulk.wait_group 0;" ::: "memory");   // all stores have landed
    }

    tc_fence_before();
    __syncthreads();
    cluster_sync_all();       // neither CTA leaves while the other may still signal it or read its tiles
    if (warp == 1) {
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(512) : "memory");
    }
}

// ------------------------------------------------------------------------------------ host
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*,
                                  CUtensorMapInterleave, CUtensorMapSwizzle, CUtensorMapL2promotion,
                                  CUtensorMapFloatOOBfill);

static EncodeTiledFn encode_fn() {
    static EncodeTiledFn fn = nullptr;
    if (!fn) {
        void* ptr = nullptr;
        cudaDriverEntryPointQueryResult res;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &res) == cudaSuccess &&
            res == cudaDriverEntryPointSuccess)
            fn = (EncodeTiledFn)ptr;
    }
    return fn;
}

// Map of a row-major bfloat16 matrix [rows, K] with boxes of box_rows x 64 values, 128-byte
// swizzle, zeros outside the matrix.
// A tensor map is a pure function of (address, rows, K, box rows); encoding one costs the host
// a microsecond or two, and a step makes some hundreds, nearly all of them for the same weights
// and the same activation buffers as the step before. A small direct-mapped table keeps them.
struct MapSlot {
    const void* base;
    int rows, K, box_rows, w_rows;
    bool full;
    CUtensorMap map;
};
static MapSlot g_maps[1024];
static std::mutex g_maps_lock;

// w_rows == 0: a row-major matrix [rows, K] (activations). w_rows > 0: a tiled weight of that
// many padded rows, seen as a matrix of 128-byte rows, ceil(K / 64) * w_rows of them, no swizzle
// (the pieces already lie where the swizzle would put them).
static int make_map(CUtensorMap* map, const void* base, int rows, int K, int box_rows, int w_rows = 0) {
    uint64_t h = (uint64_t)(uintptr_t)base * 0x9E3779B97F4A7C15ull;
    h ^= ((uint64_t)(uint32_t)rows << 32 | (uint32_t)K) * 0xC2B2AE3D27D4EB4Full + (uint64_t)box_rows +
         (uint64_t)w_rows * 0x165667B19E3779F9ull;
    MapSlot& slot = g_maps[(h >> 40) & 1023];
    std::lock_guard<std::mutex> guard(g_maps_lock);
    if (slot.full && slot.base == base && slot.rows == rows && slot.K == K && slot.box_rows == box_rows &&
        slot.w_rows == w_rows) {
        *map = slot.map;
        return 0;
    }
    EncodeTiledFn fn = encode_fn();
    if (!fn) return LUMEN_ERR_UNSUPPORTED;
    const cuuint64_t num_kb = (cuuint64_t)((K + TC_BK - 1) / TC_BK);
    cuuint64_t dims[2] = {(cuuint64_t)K, (cuuint64_t)rows};
    cuuint64_t strides[1] = {(cuuint64_t)K * 2};
    if (w_rows > 0) {
        dims[0] = TC_BK;
        dims[1] = num_kb * (cuuint64_t)w_rows;
        strides[0] = 128;
    }
    cuuint32_t box[2] = {TC_BK, (cuuint32_t)box_rows};
    cuuint32_t estr[2] = {1, 1};
    CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides, box, estr,
                    CU_TENSOR_MAP_INTERLEAVE_NONE, w_rows > 0 ? CU_TENSOR_MAP_SWIZZLE_NONE : CU_TENSOR_MAP_SWIZZLE_128B,
                    CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return LUMEN_ERR_BAD_ARGUMENT;
    slot.base = base; slot.rows = rows; slot.K = K; slot.box_rows = box_rows; slot.w_rows = w_rows;
    slot.map = *map;
    slot.full = true;
    return 0;
}

// ---------------------------------------------------------------------------- tiled weights
#define TC_W_ROW_PAD 256
LUMEN_API int lumen_tiled_weight_rows(int N) { return (N + TC_W_ROW_PAD - 1) / TC_W_ROW_PAD * TC_W_ROW_PAD; }
// bfloat16 values the tiled form of a weight [N, K] takes
LUMEN_API long long lumen_tiled_weight_elems(int N, int K) {
    return (long long)((K + TC_BK - 1) / TC_BK) * lumen_tiled_weight_rows(N) * TC_BK;
}
// One thread a 16-byte piece of the tiled form: piece j of row r in k block kb holds the values
// W[r, kb * 64 + (j ^ (r & 7)) * 8 ..+8], zeros outside the matrix.
__global__ void tile_weight_kernel(const uint4* __restrict__ W, uint4* __restrict__ Wt, int N, int K8, int w_rows,
                                   long long pieces) {
    pdl_wait();
    pdl_trigger();
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < pieces;
         i += (long long)gridDim.x * blockDim.x) {
        const int j = (int)(i & 7);
        const long long row_all = i >> 3;
        const int r = (int)(row_all % w_rows), kb = (int)(row_all / w_rows);
        const int c8 = kb * 8 + (j ^ (r & 7));
        uint4 v = make_uint4(0u, 0u, 0u, 0u);
        if (r < N && c8 < K8) v = W[(size_t)r * K8 + c8];
        Wt[i] = v;
    }
}
// W bfloat16 [N, K] row-major, K a multiple of 8 -> Wt, lumen_tiled_weight_elems(N, K) values.
LUMEN_API int lumen_tile_weight(const void* W, void* Wt, int N, int K, cudaStream_t stream) {
    if (N <= 0 || K <= 0 || (K & 7)) return LUMEN_ERR_UNSUPPORTED;
    if (((uintptr_t)W & 15) || ((uintptr_t)Wt & 127)) return LUMEN_ERR_BAD_ARGUMENT;
    const long long pieces = lumen_tiled_weight_elems(N, K) / 8;
    const long long want = (pieces + 255) / 256;
    const int grid = (int)(want < 148 * 16 ? want : 148 * 16);
    lumen_launch(tile_weight_kernel, dim3(grid), dim3(256), 0, stream, (const uint4*)W, (uint4*)Wt, N, K / 8,
                 lumen_tiled_weight_rows(N), pieces);
    LUMEN_LAUNCH_CHECK();
    return 0;
}

static int sm_count() {
    static int n = 0;
    if (!n) {
        int dev = 0;
        cudaGetDevice(&dev);
        cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev);
        if (n <= 0) n = 148;
    }
    return n;
}

// With up to 128 rows (256 for the plain float32 output) the product is still a stream over
// the weights: measured at 128 rows, 14 against 20 us for a 4,096 x 4,096 weight and 24 against
// 56 us for 4,096 x 12,288. Beyond that the activations fill 128-row tiles of their own.
static bool tc_swapped(int M, int epi) { return M <= 128 || (M <= 256 && epi == TC_EPI_F32); }

// Measurement switches (the kernel micro-benchmarks set them on request; the defaults are the
// product): prompt-sized products on the single-SM kernel only, and a fixed tile width for it.
static int g_tc_two_sm = 1, g_tc_forced_bn = 0;
LUMEN_API int lumen_gemm_tc_tune(int two_sm, int bn) {
    if (bn != 0 && (bn < 16 || bn > 256 || bn % 16)) return LUMEN_ERR_BAD_ARGUMENT;
    g_tc_two_sm = two_sm ? 1 : 0;
    g_tc_forced_bn = bn;
    return 0;
}

static bool tc_two_sm(int M, int N);
static void tc_plain_plan(int M, int N, int K, int epi, int* bn, int* splits);

// Number of k splits: a function of the weight's shape (and of the orientation) only. For the
// swapped orientation the split that fills the SMs most evenly is chosen, small splits first.
LUMEN_API int lumen_gemm_tc_splits(int M, int N, int K, int epi) {
    if (epi == TC_EPI_SILU) return 1;
    if (!tc_swapped(M, epi)) {
        if (tc_two_sm(M, N)) return 1;
        int bn, splits;
        tc_plain_plan(M, N, K, epi, &bn, &splits);
        return splits;
    }
    const int num_kb = (K + TC_BK - 1) / TC_BK;
    const int tiles = (N + TC_BM - 1) / TC_BM;
    const int sms = 148;   // fixed, so that the split never depends on the device at hand
    if (tiles >= 4 * sms) return 1;             // enough tiles: a split would only add traffic
    int best = 1;
    double best_eff = 0.0;
    // at most 8 parts: the kernel that adds the partial sums has eight loads in flight at a
    // time, and fewer, longer parts leave it less to add (measured inside a decode step: 1.37
    // against 1.41 ms for 12 layers at batch 8 when the 4,096-row weights are cut in 4, not 9)
    for (int s = 1; s <= 8 && s <= num_kb; ++s) {
        if (num_kb / s < 4) break;              // keep at least 4 k blocks per tile
        const int items = tiles * s;
        const double eff = (double)items / (double)(((items + sms - 1) / sms) * sms);
        if (eff > best_eff + 0.03) { best_eff = eff; best = s; }
    }
    const int per = (num_kb + best - 1) / best;
    return (num_kb + per - 1) / per;
}

// Width of the weight tiles for the single-SM kernel in the plain orientation (products too
// small for the two-SM kernel). Tiles are dealt out to 148 persistent blocks in waves; the
// cost of a shape is its number of waves times the time of a tile, which is a fixed part (the
// activation tile every k block needs whatever the width) plus a part that grows with the
// width. The width with the least cost wins, the wider on a tie: 256 rows x 4,096 run as 128
// tiles of 64 instead of 32 tiles of 256 (21.7 against 28.6 us). A function of the shape only;
// every width sums k in the same ascending order.
static int tc_pick_bn(int M, int N, long* cost_out) {
    const int tilesA = (M + TC_BM - 1) / TC_BM;
    int best = 256;
    long best_cost = -1;
    for (int bn = 256; bn >= 32; bn -= 16) {
        const long tiles = (long)tilesA * ((N + bn - 1) / bn);
        const long waves = (tiles + 147) / 148;
        const long cost = waves * (bn + TC_TILE_FIXED);
        if (best_cost < 0 || cost < best_cost) { best_cost = cost; best = bn; }
    }
    *cost_out = best_cost;
    return best;
}

// Tile width and k split of the single-SM kernel in the plain orientation. Besides narrow
// tiles there is a second way to give every SM work when the tiles are few: full-width tiles
// with k split in up to four parts (partial sums [S, M, N], float32 output only). In the cost
// model above a part of a tile costs its share of the tile plus a tenth for the partial sums.
static void tc_plain_plan(int M, int N, int K, int epi, int* bn, int* splits) {
    long narrow_cost;
    *bn = tc_pick_bn(M, N, &narrow_cost);
    *splits = 1;
    if (g_tc_forced_bn) {
        *bn = g_tc_forced_bn;
        return;
    }
    if (epi != TC_EPI_F32) return;
    const int num_kb = (K + TC_BK - 1) / TC_BK;
    const long tiles = (long)((M + TC_BM - 1) / TC_BM) * ((N + 255) / 256);
    int s = (int)(148 / tiles);
    if (s > 4) s = 4;
    if (s > num_kb / 8) s = num_kb / 8;
    if (s < 2) return;
    const long split_cost = (256 + TC_TILE_FIXED) * 11 / (10 * s);
    if (split_cost < narrow_cost) {
        *bn = 256;
        const int per = (num_kb + s - 1) / s;
        *splits = (num_kb + per - 1) / per;
    }
}

template <int BN, int STAGES, bool SWAP, int EPI>
static int tc_launch(const CUtensorMap& ma, const CUtensorMap& mb, const TcParams& p, cudaStream_t stream) {
    constexpr size_t smem = (size_t)STAGES * (TC_BM * 128 + BN * 128) + (2 * STAGES + 4) * 8 + 16 + 1024;
    auto k = gemm_tc_kernel<BN, STAGES, SWAP, EPI>;
    static bool attr_done = false;
    if (!attr_done) {
        cudaError_t e = cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return (int)e;
        attr_done = true;
    }
    const int tilesA = (p.rowsA + TC_BM - 1) / TC_BM, tilesB = (p.rowsB + p.bn - 1) / p.bn;
    const int items = tilesA * tilesB * p.splits;
    const int grid = items < sm_count() ? items : sm_count();
    lumen_launch(k, dim3(grid), dim3(TC_THREADS), smem, stream, ma, mb, p);
    LUMEN_LAUNCH_CHECK();
    return 0;
}

// Map of the output for the staged store: row-major [rows, cols] of float32 or bfloat16, blocks
// of 128 rows x 128 bytes, 128-byte swizzle.
static int make_out_map(CUtensorMap* map, void* base, int rows, int cols, bool f32) {
    EncodeTiledFn fn = encode_fn();
    if (!fn) return LUMEN_ERR_UNSUPPORTED;
    const int esz = f32 ? 4 : 2;
    cuuint64_t dims[2] = {(cuuint64_t)cols, (cuuint64_t)rows};
    cuuint64_t strides[1] = {(cuuint64_t)cols * esz};
    cuuint32_t box[2] = {(cuuint32_t)(128 / esz), TC_BM};
    cuuint32_t estr[2] = {1, 1};
    CUresult r = fn(map, f32 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT32 : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, base, dims,
                    strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                    CU_TENSOR_MAP_L2_PROMOTION_NONE, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    return r == CUDA_SUCCESS ? 0 : LUMEN_ERR_BAD_ARGUMENT;
}

// The two-SM kernel: clusters of two CTAs, one pair per two SMs, persistent over the tiles.
template <int EPI>
static int tc2_launch(const CUtensorMap& ma, const CUtensorMap& mb, const CUtensorMap& mc, const TcParams& p,
                      cudaStream_t stream) {
    constexpr size_t smem = (size_t)TC2_STAGES * 2 * TC2_TILE_BYTES + (EPI == TC_EPI_QKV ? 4 : 2) * TC2_OUT_BYTES +
                            256 + (EPI == TC_EPI_QKV ? 1024 : 0) + 1024;
    auto k = gemm_tc2_kernel<EPI>;
    static bool attr_done = false;
    if (!attr_done) {
        cudaError_t e = cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return (int)e;
        attr_done = true;
    }
    const int items = ((p.rowsA + 255) / 256) * ((p.rowsB + 255) / 256);
    const int pairs = items < sm_count() / 2 ? items : sm_count() / 2;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(2 * pairs);
    cfg.blockDim = dim3(TC_THREADS);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[2];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = 2;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[1].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = lumen_pdl_enabled() ? 2 : 1;
    cudaError_t e = cudaLaunchKernelEx(&cfg, k, ma, mb, mc, p);
    if (e != cudaSuccess) return (int)e;
    LUMEN_LAUNCH_CHECK();
    return 0;
}

// Whether the two-SM kernel takes a prompt-sized product: at least one full wave of 256 x 256
// tiles for the 74 pairs (fewer tiles are spread better by the single-SM kernel's narrow tiles).
static bool tc_two_sm(int M, int N) {
    if (!g_tc_two_sm) return false;
    const long items = (long)((M + 255) / 256) * ((N + 255) / 256);
    return items >= 74;
}

// Whether a product of this shape can be added to its output in place (epi 2): the shapes of
// the two-SM kernel with output rows that are multiples of 16 bytes.
LUMEN_API int lumen_gemm_tc_adds(int M, int N) { return (!tc_swapped(M, TC_EPI_F32) && tc_two_sm(M, N) && (N & 3) == 0) ? 1 : 0; }

// x bfloat16 [M, K]; W the tiled form (lumen_tile_weight) of a bfloat16 weight of w_rows padded
// rows, of which the first N are used; K a multiple of 8; x 16-byte, W 128-byte aligned.
// epi 2: out float32 [M, N] += x W^T (only where lumen_gemm_tc_adds says so).
// epi 0: out float32 [S, M, N], S = lumen_gemm_tc_splits(M, N, K, 0).
// epi 1: W's rows alternate gate_i, up_i; out bfloat16 [M, N / 2] = SiLU(gate) * up.
LUMEN_API int lumen_gemm_tc(const void* x, const void* W, void* out, int M, int N, int K, int w_rows, int epi,
                            int* err, cudaStream_t stream) {
    if (M <= 0 || N <= 0) return 0;
    if (K <= 0 || (K & 7) || (epi != TC_EPI_F32 && epi != TC_EPI_SILU && epi != TC_EPI_ADD)) return LUMEN_ERR_UNSUPPORTED;
    if (epi == TC_EPI_ADD && !lumen_gemm_tc_adds(M, N)) return LUMEN_ERR_UNSUPPORTED;
    if (epi == TC_EPI_SILU && (N & 1)) return LUMEN_ERR_UNSUPPORTED;
    if (((uintptr_t)x & 15) || ((uintptr_t)W & 127) || w_rows < N || w_rows % TC_W_ROW_PAD) return LUMEN_ERR_BAD_ARGUMENT;
    TcParams p;
    p.w_rows = w_rows;
    p.out_f32 = (float*)out;
    p.out_bf16 = (__nv_bfloat16*)out;
    p.M = M;
    p.N = N;
    p.num_kb = (K + TC_BK - 1) / TC_BK;
    p.splits = lumen_gemm_tc_splits(M, N, K, epi);
    p.kb_per_split = (p.num_kb + p.splits - 1) / p.splits;
    p.err = err;
    p.tma_out = 0;
    CUtensorMap ma, mb;
    int rc;
    if (tc_swapped(M, epi)) {
        const int bn = M <= 16 ? 16 : (M <= 32 ? 32 : (M <= 64 ? 64 : (M <= 128 ? 128 : 256)));
        p.rowsA = N;
        p.rowsB = M;
        p.bn = bn;
        if ((rc = make_map(&ma, W, N, K, TC_BM, w_rows))) return rc;
        if ((rc = make_map(&mb, x, M, K, bn))) return rc;
        if (epi == TC_EPI_F32) {
            if (bn == 16) return tc_launch<16, 6, true, TC_EPI_F32>(ma, mb, p, stream);
            if (bn == 32) return tc_launch<32, 5, true, TC_EPI_F32>(ma, mb, p, stream);
            if (bn == 64) return tc_launch<64, 8, true, TC_EPI_F32>(ma, mb, p, stream);
            if (bn == 128) return tc_launch<128, 6, true, TC_EPI_F32>(ma, mb, p, stream);
            return tc_launch<256, 4, true, TC_EPI_F32>(ma, mb, p, stream);
        }
        if (bn == 16) return tc_launch<16, 10, true, TC_EPI_SILU>(ma, mb, p, stream);
        if (bn == 32) return tc_launch<32, 9, true, TC_EPI_SILU>(ma, mb, p, stream);
        if (bn == 64) return tc_launch<64, 8, true, TC_EPI_SILU>(ma, mb, p, stream);
        if (bn == 128) return tc_launch<128, 6, true, TC_EPI_SILU>(ma, mb, p, stream);
        return tc_launch<256, 4, true, TC_EPI_SILU>(ma, mb, p, stream);
    }
    p.rowsA = M;
    p.rowsB = N;
    if (tc_two_sm(M, N)) {
        p.bn = 256;
        if ((rc = make_map(&ma, x, M, K, TC_BM))) return rc;
        if ((rc = make_map(&mb, W, N, K, TC_BM, w_rows))) return rc;
        // the staged store needs output rows that are multiples of 16 bytes
        const int out_cols = epi != TC_EPI_SILU ? N : N / 2;
        const int out_esz = epi != TC_EPI_SILU ? 4 : 2;
        CUtensorMap mc = ma;
        p.tma_out = ((out_cols * out_esz) % 16 == 0 && ((uintptr_t)out & 15) == 0) ? 1 : 0;
        if (p.tma_out && (rc = make_out_map(&mc, out, M, out_cols, epi != TC_EPI_SILU))) return rc;
        if (epi == TC_EPI_ADD) return p.tma_out ? tc2_launch<TC_EPI_ADD>(ma, mb, mc, p, stream) : LUMEN_ERR_BAD_ARGUMENT;
        if (epi == TC_EPI_F32) return tc2_launch<TC_EPI_F32>(ma, mb, mc, p, stream);
        return tc2_launch<TC_EPI_SILU>(ma, mb, mc, p, stream);
    }
    tc_plain_plan(M, N, K, epi, &p.bn, &p.splits);
    p.kb_per_split = (p.num_kb + p.splits - 1) / p.splits;
    if ((rc = make_map(&ma, x, M, K, TC_BM))) return rc;
    if ((rc = make_map(&mb, W, N, K, p.bn, w_rows))) return rc;
    if (epi == TC_EPI_F32) return tc_launch<256, 4, false, TC_EPI_F32>(ma, mb, p, stream);
    return tc_launch<256, 4, false, TC_EPI_SILU>(ma, mb, p, stream);
}

// The QKV product of a prompt with what follows it folded into the epilogue: per-head RMSNorm of
// q and k (weights qw, kw of 128 values, or null), rotation of the pairs (i, i + 64) by the
// (cos, sin) table cs [M, 64] (rot 128; rot 0: none), q out as bfloat16 [M, nq, 128], and k and
// v written to their rows' places in the paged cache (128-byte swizzled tiles of 64 keys x 128).
// W: bfloat16 [(nq + 2 nkv) * 128, K], rows in the order q heads, k heads, v heads.
LUMEN_API int lumen_gemm_tc_qkv_ok(int M, int N, int K, int nq, int nkv, int d, int rot) {
    return (d == 128 && (rot == 0 || rot == 128) && nq > 0 && nkv > 0 && N == (nq + 2 * nkv) * 128 && K > 0 &&
            (K & 7) == 0 && !tc_swapped(M, TC_EPI_F32) && tc_two_sm(M, N)) ? 1 : 0;
}

LUMEN_API int lumen_gemm_tc_qkv(const void* x, const void* W, int M, int N, int K, int w_rows, void* q_out, void* kcache,
                                void* vcache, const float* qw, const float* kw, float eps, const float* cs, int rot,
                                const int* cache_pos, const int* tok_seq, const int* block_table, int bt_stride,
                                int nq, int nkv, int* err, cudaStream_t stream) {
    if (!lumen_gemm_tc_qkv_ok(M, N, K, nq, nkv, 128, rot)) return LUMEN_ERR_UNSUPPORTED;
    if (w_rows < N || w_rows % TC_W_ROW_PAD) return LUMEN_ERR_BAD_ARGUMENT;
    if (((uintptr_t)x & 15) || ((uintptr_t)W & 127) || ((uintptr_t)q_out & 15) || ((uintptr_t)kcache & 127) ||
        ((uintptr_t)vcache & 127) || (rot == 128 && (!cs || ((uintptr_t)cs & 15))) || ((uintptr_t)qw & 15) ||
        ((uintptr_t)kw & 15) || !cache_pos || !tok_seq || !block_table)
        return LUMEN_ERR_BAD_ARGUMENT;
    TcParams p = {};
    p.out_f32 = nullptr;
    p.out_bf16 = (__nv_bfloat16*)q_out;
    p.M = M;
    p.N = N;
    p.rowsA = M;
    p.rowsB = N;
    p.num_kb = (K + TC_BK - 1) / TC_BK;
    p.splits = 1;
    p.kb_per_split = p.num_kb;
    p.tma_out = 1;
    p.bn = 256;
    p.w_rows = w_rows;
    p.err = err;
    p.qw = qw;
    p.kw = kw;
    p.cs = (const float2*)cs;
    p.cache_pos = cache_pos;
    p.tok_seq = tok_seq;
    p.block_table = block_table;
    p.kcache = (__nv_bfloat16*)kcache;
    p.vcache = (__nv_bfloat16*)vcache;
    p.eps = eps;
    p.bt_stride = bt_stride;
    p.nq = nq;
    p.nkv = nkv;
    p.rot = rot;
    CUtensorMap ma, mb, mc;
    int rc;
    if ((rc = make_map(&ma, x, M, K, TC_BM))) return rc;
    if ((rc = make_map(&mb, W, N, K, TC_BM, w_rows))) return rc;
    if ((rc = make_out_map(&mc, q_out, M, nq * 128, false))) return rc;
    return tc2_launch<TC_EPI_QKV>(ma, mb, mc, p, stream);
}
