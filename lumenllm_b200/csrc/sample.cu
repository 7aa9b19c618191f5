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
//
// Two routes give the same answer. The quick one bins the row ONCE, linearly in
// (max - logit) / temperature (2,048 bins over 32 units, monotone in the logit, so a bin is a
// run of the rank order), with the count and the exact weight of every bin; each selection
// then scans the bins, gathers the few hundred elements of the bin in which the target falls,
// orders them by (logit down, index up) and walks them. The radix descent over the keys is
// the route for everything the quick one declines: min-p, a bin too full to gather (long runs
// of equal or nearly equal logits), a target in the last, open-ended bin.
#include <cooperative_groups.h>
#include <cstdint>
#include "common.cuh"

#define SM_THREADS 1024
#define FX_ONE 1099511627776.0  // 2^40

typedef unsigned long long u64;

// Calls f(value, index) for every element of a row, each thread taking a strided share.
// Rows that start on a 16-byte boundary are read four values a load, four loads in flight a
// thread: one block reads a row of 150 thousand logits in a few microseconds instead of
// waiting out one L2 round trip per value. Every use is a sum, a maximum or a set of atomic
// adds, none of which depends on the order of the calls.
template <typename F>
__device__ __forceinline__ void row_each(const float* lg, int V, F f) {
    const int bd = blockDim.x;
    if ((reinterpret_cast<uintptr_t>(lg) & 15) == 0) {
        const int n4 = V >> 2;
        const float4* p4 = reinterpret_cast<const float4*>(lg);
        int i = threadIdx.x;
        for (; i + 3 * bd < n4; i += 4 * bd) {
            const float4 a = p4[i], b = p4[i + bd], c = p4[i + 2 * bd], d = p4[i + 3 * bd];
            f(a.x, 4 * i); f(a.y, 4 * i + 1); f(a.z, 4 * i + 2); f(a.w, 4 * i + 3);
            f(b.x, 4 * (i + bd)); f(b.y, 4 * (i + bd) + 1); f(b.z, 4 * (i + bd) + 2); f(b.w, 4 * (i + bd) + 3);
            f(c.x, 4 * (i + 2 * bd)); f(c.y, 4 * (i + 2 * bd) + 1); f(c.z, 4 * (i + 2 * bd) + 2); f(c.w, 4 * (i + 2 * bd) + 3);
            f(d.x, 4 * (i + 3 * bd)); f(d.y, 4 * (i + 3 * bd) + 1); f(d.z, 4 * (i + 3 * bd) + 2); f(d.w, 4 * (i + 3 * bd) + 3);
        }
        for (; i < n4; i += bd) {
            const float4 a = p4[i];
            f(a.x, 4 * i); f(a.y, 4 * i + 1); f(a.z, 4 * i + 2); f(a.w, 4 * i + 3);
        }
        for (int j = 4 * n4 + threadIdx.x; j < V; j += bd) f(lg[j], j);
    } else {
        for (int j = threadIdx.x; j < V; j += bd) f(lg[j], j);
    }
}

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
    return __float2ull_rz(w * 1099511627776.0f);      // w <= 1; scaling by 2^40 is exact
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
    row_each(lg, V, [&](float x, int i) {
        if (!finite_f(x)) return;
        if (!P.all && okey(x) <= P.thr) return;
        a += MASS ? weight_fx(x, mx, temp) : 1ull;
    });
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
        row_each(lg, V, [&](float x, int i) {
            if (!finite_f(x)) return;
            const unsigned k = okey(x);
            if ((k ^ cur) & above) return;
            if (!P.all && k <= P.thr) return;
            const u64 amt = MASS ? weight_fx(x, mx, temp) : 1ull;
            if (amt) atomicAdd(&sh.hist[(k >> shift) & 255u], amt);
        });
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
__device__ void block_argmax(const float* lg, int V, float* out_v, int* out_i, Shared& sh,
                             float* finite_max = nullptr) {
    float bv = -INFINITY, fm = -INFINITY;
    int bi = 0x7fffffff;
    row_each(lg, V, [&](float x, int i) {
        if (x > bv || (x == bv && i < bi)) { bv = x; bi = i; }
        if (finite_f(x)) fm = fmaxf(fm, x);
    });
    if (finite_max) {                 // the largest finite value, for the sampler
        fm = block_max(fm, sh.redf);
        __syncthreads();
        *finite_max = fm;
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

// ----------------------------------------------------------------------- the quick route
// A row is worked on by a cluster of up to QC blocks; each reads its own share of the row. Block 0
// decides: it adds up the blocks' bin tables, finds the bin a target falls in, tells the
// others (through their shared memory) which bin to gather, collects their lists and orders
// them. Commands and results cross at cluster barriers; nobody spins.
#define QC 8               // blocks a row at most (1, 2, 4 or 8: the fewer the more rows there are)
#define QB 2048            // bins
#define QSPAN 32.0f        // units of (max - logit) / temperature they cover; the last bin is open
#define QCAP 1024          // elements of one bin that can be gathered
#define QCMD_DONE 0
#define QCMD_GATHER 1
#define QCMD_MINKEY 2

struct Quick {
    u64 mass[QB];          // this block's share; in block 0, after the merge, the row's
    unsigned cnt[QB];
    unsigned lkey[QCAP];   // gathered, in arrival order (block 0: all blocks' lists)
    int lidx[QCAP];
    unsigned skey[QCAP];   // block 0: the same in rank order
    int sidx[QCAP];
    u64 wsum[SM_THREADS / 32];
    int n_list;
    int sel_bin;
    u64 sel_before;
    int sel_pos;
    float part_v[QC];      // every block's (largest value, its index, largest finite value)
    int part_i[QC];
    float part_fm[QC];
    unsigned part_key[QC]; // block 0: every block's answer to MINKEY
    int cmd, cmd_bin, cmd_all, cmd_pbin;
    unsigned cmd_thr;
    float cmd_minp;
};

// Kept set in bin terms: bins below `bin` whole, of bin `bin` the first cnt_in_bin elements of
// its rank order (weight mass_in_bin); thr / ties as in Prefix.
struct QPrefix {
    int all;
    unsigned thr, ties;
    int bin;
    unsigned cnt_in_bin;
    u64 mass_in_bin;
};

__device__ __forceinline__ int bin_of(float x, float mx, float temp) {
    const float fb = (mx - x) / temp * ((float)QB / QSPAN);
    return fb >= (float)(QB - 1) ? QB - 1 : (int)fb;
}

// Exclusive block scan of two values a thread (bins 2t and 2t+1 of a 2,048-bin table).
__device__ u64 block_scan_pair(u64 a, u64 b, u64* excl_a, Quick& q) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const u64 mine = a + b;
    u64 inc = mine;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
        const u64 t = __shfl_up_sync(0xffffffffu, inc, o);
        if (lane >= o) inc += t;
    }
    __syncthreads();
    if (lane == 31) q.wsum[warp] = inc;
    __syncthreads();
    u64 off = 0, total = 0;
    for (int w = 0; w < SM_THREADS / 32; ++w) {
        const u64 v = q.wsum[w];
        if (w < warp) off += v;
        total += v;
    }
    *excl_a = off + inc - mine;
    return total;
}

template <bool MASS>
__device__ __forceinline__ u64 kept_of_bin(const QPrefix& P, const Quick& q, int b) {
    if (P.all || b < P.bin) return MASS ? q.mass[b] : (u64)q.cnt[b];
    if (b == P.bin) return MASS ? P.mass_in_bin : (u64)P.cnt_in_bin;
    return 0ull;
}

// Amount (count or weight) of the kept set. Block 0.
template <bool MASS>
__device__ u64 quick_amount(const QPrefix& P, Quick& q) {
    u64 ex;
    return block_scan_pair(kept_of_bin<MASS>(P, q, 2 * threadIdx.x), kept_of_bin<MASS>(P, q, 2 * threadIdx.x + 1),
                           &ex, q);
}

// This block's share of the row: [beg, end), beg a multiple of 4.
__device__ __forceinline__ void row_share(int V, int rank, int qc, int* beg, int* end) {
    const int per = (((V + 3) / 4 + qc - 1) / qc) * 4;
    *beg = min(V, rank * per);
    *end = min(V, *beg + per);
}

// What every block does on GATHER: its elements of bin sb that the kept set may hold.
__device__ void quick_gather(const float* lg, int V, int rank, int qc, float mx, float temp, Quick& q) {
    if (threadIdx.x == 0) q.n_list = 0;
    __syncthreads();
    const int sb = q.cmd_bin, all = q.cmd_all, pbin = q.cmd_pbin;
    const unsigned thr = q.cmd_thr;
    int beg, end;
    row_share(V, rank, qc, &beg, &end);
    row_each(lg + beg, end - beg, [&](float x, int i) {
        if (!finite_f(x) || bin_of(x, mx, temp) != sb) return;
        const unsigned k = okey(x);
        if (!all && sb == pbin && k < thr) return;
        const int pos = atomicAdd(&q.n_list, 1);
        if (pos < QCAP) { q.lkey[pos] = k; q.lidx[pos] = beg + i; }
    });
    __syncthreads();
}

// What every block does on MINKEY: its lowest kept key whose weight is at least min_p.
__device__ unsigned quick_minkey(const float* lg, int V, int rank, int qc, float mx, float temp, Quick& q, Shared& sh) {
    const int all = q.cmd_all;
    const unsigned thr = q.cmd_thr;
    const float min_p = q.cmd_minp;
    int beg, end;
    row_share(V, rank, qc, &beg, &end);
    unsigned lowest = 0xffffffffu;
    row_each(lg + beg, end - beg, [&](float x, int i) {
        if (!finite_f(x)) return;
        const unsigned k = okey(x);
        if (!all && k < thr) return;
        if (weight_f(x, mx, temp) >= 1.0f * min_p) lowest = min(lowest, k);
    });
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) lowest = min(lowest, __shfl_xor_sync(0xffffffffu, lowest, o));
    __syncthreads();
    if (lane == 0) sh.redu[warp] = lowest;
    __syncthreads();
    lowest = (lane < (int)(blockDim.x >> 5)) ? sh.redu[lane] : 0xffffffffu;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) lowest = min(lowest, __shfl_xor_sync(0xffffffffu, lowest, o));
    return lowest;
}

// Block 0 publishes a command in every block's shared memory; the cluster barrier after it
// (the caller's) makes it visible.
template <typename Cluster>
__device__ void quick_publish(Cluster& cluster, Quick& q, int cmd, int bin, const QPrefix& P, float min_p) {
    if (threadIdx.x < cluster.num_blocks()) {
        Quick* r = cluster.map_shared_rank(&q, threadIdx.x);
        r->cmd = cmd;
        r->cmd_bin = bin;
        r->cmd_all = P.all;
        r->cmd_pbin = P.bin;
        r->cmd_thr = P.thr;
        r->cmd_minp = min_p;
    }
}

// Block 0: orders the gathered bin sb (all blocks' lists) and walks it. With take_all the
// whole list is the answer (its count and weight); otherwise the element at which the
// running amount, starting from `before`, first reaches target. Narrows P. False = decline.
template <bool MASS, typename Cluster>
__device__ bool quick_resolve(Cluster& cluster, float mx, float temp, QPrefix& P, int sb, u64 before,
                              u64 target, bool take_all, int* token, Quick& q) {
    const int t = threadIdx.x;
    // collect the other blocks' lists behind this block's own
    int n = q.n_list;
    bool fits = n <= QCAP;
    const int qc = (int)cluster.num_blocks();
    for (int r = 1; r < qc; ++r) {
        const Quick* rq = cluster.map_shared_rank(&q, r);
        const int nr = rq->n_list;
        fits = fits && nr <= QCAP && n + nr <= QCAP;
        if (fits && t < nr) { q.lkey[n + t] = rq->lkey[t]; q.lidx[n + t] = rq->lidx[t]; }
        n += nr;
    }
    __syncthreads();
    if (!fits || n == 0) return false;
    if (t == 0) q.sel_pos = -1;
    // rank order: larger key first, equal keys by rising index
    if (t < n) {
        const unsigned k = q.lkey[t];
        const int ix = q.lidx[t];
        int r = 0;
        for (int j = 0; j < n; ++j) {
            const unsigned kj = q.lkey[j];
            r += (kj > k || (kj == k && q.lidx[j] < ix)) ? 1 : 0;
        }
        q.skey[r] = k;
        q.sidx[r] = ix;
    }
    __syncthreads();
    if (!P.all && sb == P.bin) n = min(n, (int)P.cnt_in_bin);   // ties of thr beyond the kept ones
    const u64 amt_w = (t < n) ? weight_fx(key_to_float(q.skey[t]), mx, temp) : 0ull;
    const u64 amt = MASS ? amt_w : ((t < n) ? 1ull : 0ull);
    u64 ex_sel, ex_w;
    block_scan_pair(amt, 0ull, &ex_sel, q);
    if (take_all) {
        if (t == n - 1) q.sel_pos = t;
    } else if (t < n && amt && before + ex_sel < target && target <= before + ex_sel + amt) {
        q.sel_pos = t;
    }
    __syncthreads();
    const int pos = q.sel_pos;
    if (pos < 0) return false;
    block_scan_pair(amt_w, 0ull, &ex_w, q);
    if (t == pos) q.sel_before = ex_w + amt_w;       // weight of the list up to and including pos
    const unsigned kp = q.skey[pos];
    int tie = (t <= pos && t < n && q.skey[t] == kp) ? 1 : 0;
    tie = __syncthreads_count(tie);
    const u64 mass_to_pos = q.sel_before;
    *token = q.sidx[pos];
    P.all = 0;
    P.thr = kp;
    P.ties = (unsigned)tie;
    P.bin = sb;
    P.cnt_in_bin = (unsigned)(pos + 1);
    P.mass_in_bin = mass_to_pos;
    __syncthreads();
    return true;
}

// Block 0: the element of the kept set at which the running amount first reaches target.
// Two cluster barriers (command out, lists in) that the other blocks meet in their loop.
template <bool MASS, typename Cluster>
__device__ bool quick_select(Cluster& cluster, const float* lg, int V, float mx, float temp, QPrefix& P,
                             u64 target, int* token, Quick& q) {
    const int t = threadIdx.x;
    const u64 a = kept_of_bin<MASS>(P, q, 2 * t), b = kept_of_bin<MASS>(P, q, 2 * t + 1);
    if (t == 0) q.sel_bin = -1;
    u64 ex;
    block_scan_pair(a, b, &ex, q);            // has the barriers that order the line above
    if (a && ex < target && target <= ex + a) { q.sel_bin = 2 * t; q.sel_before = ex; }
    if (b && ex + a < target && target <= ex + a + b) { q.sel_bin = 2 * t + 1; q.sel_before = ex + a; }
    __syncthreads();
    const int sb = q.sel_bin;
    if (sb < 0 || sb == QB - 1) return false;
    const u64 before = q.sel_before;
    quick_publish(cluster, q, QCMD_GATHER, sb, P, 0.0f);
    cluster.sync();
    quick_gather(lg, V, 0, (int)cluster.num_blocks(), mx, temp, q);
    cluster.sync();
    return quick_resolve<MASS>(cluster, mx, temp, P, sb, before, target, false, token, q);
}

// Block 0, after the merge of the bin tables. temperature > 0, top_k != 1, mx finite.
// Returns the token, or -1 to decline (the caller then takes the radix route).
template <typename Cluster>
__device__ int sample_quick(Cluster& cluster, const float* lg, int V, float mx, float temp, int top_k,
                            float top_p, float min_p, float u, Quick& q, Shared& sh) {
    QPrefix P;
    P.all = 1; P.thr = 0; P.ties = 0; P.bin = QB; P.cnt_in_bin = 0; P.mass_in_bin = 0;
    int token = -1;
    // what falls into the open last bin must weigh nothing
    if (weight_fx(mx - QSPAN * temp * (1.0f - 1.0f / QB), mx, temp) != 0ull) return -1;
    if (top_k > 0) {
        const u64 n_valid = quick_amount<false>(P, q);
        if ((u64)top_k < n_valid && !quick_select<false>(cluster, lg, V, mx, temp, P, (u64)top_k, &token, q))
            return -1;
    }
    u64 total = quick_amount<true>(P, q);
    if (total == 0ull) return -1;
    if (top_p > 0.0f && top_p < 1.0f) {
        u64 cutoff = (u64)ceil((double)total * (double)top_p);
        if (cutoff < 1) cutoff = 1;
        if (cutoff > total) cutoff = total;
        if (!quick_select<true>(cluster, lg, V, mx, temp, P, cutoff, &token, q)) return -1;
    }
    if (min_p > 0.0f) {
        // the largest weight is exp(0) = 1, so the rule is w >= min_p: find the lowest kept key
        // that passes, then gather its bin down to that key; the whole list is kept
        quick_publish(cluster, q, QCMD_MINKEY, 0, P, min_p);
        cluster.sync();
        const int qc = (int)cluster.num_blocks();
        unsigned lowest = quick_minkey(lg, V, 0, qc, mx, temp, q, sh);
        cluster.sync();
        for (int r = 1; r < qc; ++r) lowest = min(lowest, q.part_key[r]);
        if (lowest == 0xffffffffu) return -1;
        if (P.all || lowest > P.thr) {
            const int sb = bin_of(key_to_float(lowest), mx, temp);
            if (sb == QB - 1) return -1;
            QPrefix cut = P;
            cut.all = 0; cut.thr = lowest; cut.bin = sb;      // gather: keys >= lowest of bin sb
            quick_publish(cluster, q, QCMD_GATHER, sb, cut, 0.0f);
            cluster.sync();
            quick_gather(lg, V, 0, qc, mx, temp, q);
            cluster.sync();
            // every gathered element counts: if the old threshold lies in the same bin, the
            // gathered keys (>= lowest > thr) are all inside the old kept set
            QPrefix open_ = P;
            open_.all = 1;
            if (!quick_resolve<true>(cluster, mx, temp, open_, sb, 0ull, 0ull, true, &token, q)) return -1;
            P = open_;
        }
    }
    total = quick_amount<true>(P, q);
    if (total == 0ull) return -1;
    u64 target = (u64)ceil((double)u * (double)total);
    if (target < 1) target = 1;
    if (target > total) target = total;
    if (!quick_select<true>(cluster, lg, V, mx, temp, P, target, &token, q)) return -1;
    return token;
}

// opts: per row (temperature, top_p, min_p, u); top_k: per row. A cluster of 1 to QC blocks a row
// (the launch says how many); the token does not depend on how many.
__global__ void __launch_bounds__(SM_THREADS)
sample_kernel(const float* __restrict__ logits, long long row_stride, int V,
              const float* __restrict__ opts, const int* __restrict__ top_k_arr,
              int* __restrict__ out) {
    pdl_wait();      // nothing of this kernel touches global memory before this
    pdl_trigger();
    namespace cg = cooperative_groups;
    cg::cluster_group cluster = cg::this_cluster();
    const int rank = (int)cluster.block_rank(), qc = (int)cluster.num_blocks();
    const int row = blockIdx.x / qc;
    __shared__ Shared sh;
    __shared__ Quick quick;
    const float* lg = logits + (size_t)row * row_stride;
    const float temperature = opts[row * 4 + 0];
    const float top_p = opts[row * 4 + 1];
    const float min_p = opts[row * 4 + 2];
    const float u = opts[row * 4 + 3];
    const int top_k = top_k_arr[row];

    // Every block: largest value (lowest index) and largest finite value of its share, told to all.
    {
        int beg, end;
        row_share(V, rank, qc, &beg, &end);
        float v, fm;
        int i;
        block_argmax(lg + beg, end - beg, &v, &i, sh, &fm);
        if (threadIdx.x < qc) {
            Quick* r = cluster.map_shared_rank(&quick, threadIdx.x);
            r->part_v[rank] = v;
            r->part_i[rank] = (end > beg) ? beg + i : 0x7fffffff;
            r->part_fm[rank] = fm;
        }
    }
    cluster.sync();
    float amax_v = -INFINITY, mx = -INFINITY;   // mx: largest finite logit (+inf is left out of sampling)
    int amax_i = 0x7fffffff;
    for (int r = 0; r < qc; ++r) {
        const float v = quick.part_v[r];
        const int i = quick.part_i[r];
        // an empty share reports no index; a share in which nothing compares (all NaN) reports
        // its first index with -inf, as a whole row would
        if (i != 0x7fffffff && (amax_i == 0x7fffffff || v > amax_v || (v == amax_v && i < amax_i))) {
            amax_v = v;
            amax_i = i;
        }
        mx = fmaxf(mx, quick.part_fm[r]);
    }
    if (amax_i == 0x7fffffff) amax_i = 0;
    int result = amax_i;
    if (temperature <= 0.0f || top_k == 1 || mx == -INFINITY) {   // greedy, or nothing finite
        if (rank == 0 && threadIdx.x == 0) out[row] = result;
        return;
    }
    const float temp = fmaxf(temperature, 1e-6f);

    // Every block: bin table of its share.
    for (int b = threadIdx.x; b < QB; b += blockDim.x) { quick.mass[b] = 0ull; quick.cnt[b] = 0u; }
    __syncthreads();
    {
        int beg, end;
        row_share(V, rank, qc, &beg, &end);
        unsigned far = 0;                     // the open last bin is counted in a register
        row_each(lg + beg, end - beg, [&](float x, int i) {
            if (!finite_f(x)) return;
            const int b = bin_of(x, mx, temp);
            if (b == QB - 1) { ++far; return; }
            if (top_k > 0) atomicAdd(&quick.cnt[b], 1u);      // counts serve top-k alone
            const u64 w = weight_fx(x, mx, temp);
            if (w) atomicAdd(&quick.mass[b], w);
        });
        if (far) atomicAdd(&quick.cnt[QB - 1], far);
    }
    cluster.sync();

    if (rank != 0) {
        // do as block 0 says until it says done
        for (;;) {
            cluster.sync();
            const int cmd = quick.cmd;
            if (cmd == QCMD_DONE) return;
            if (cmd == QCMD_GATHER) {
                quick_gather(lg, V, rank, qc, mx, temp, quick);
            } else {
                const unsigned lowest = quick_minkey(lg, V, rank, qc, mx, temp, quick, sh);
                if (threadIdx.x == 0) cluster.map_shared_rank(&quick, 0)->part_key[rank] = lowest;
            }
            cluster.sync();
        }
    }

    // Block 0: the row's bin table is the sum of the blocks' tables.
    for (int b = threadIdx.x; b < QB; b += blockDim.x) {
        u64 m = quick.mass[b];
        unsigned c = quick.cnt[b];
        for (int r = 1; r < qc; ++r) {
            const Quick* rq = cluster.map_shared_rank(&quick, r);
            m += rq->mass[b];
            c += rq->cnt[b];
        }
        quick.mass[b] = m;
        quick.cnt[b] = c;
    }
    __syncthreads();
    const int tok = sample_quick(cluster, lg, V, mx, temp, top_k, top_p, min_p, u, quick, sh);
    {
        QPrefix none;
        none.all = 1; none.thr = 0; none.ties = 0; none.bin = QB; none.cnt_in_bin = 0; none.mass_in_bin = 0;
        quick_publish(cluster, quick, QCMD_DONE, 0, none, 0.0f);
    }
    cluster.sync();                           // the others leave; from here on this block is alone
    if (tok >= 0) {
        if (threadIdx.x == 0) out[row] = tok;
        return;
    }
    __syncthreads();

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
        if (threadIdx.x == 0) out[row] = result;
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
        row_each(lg, V, [&](float x, int i) {
            if (!finite_f(x)) return;
            const unsigned k = okey(x);
            if (!P.all && k < P.thr) return;
            if (weight_f(x, mx, temp) >= 1.0f * min_p) lowest = min(lowest, k);
        });
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
            if (threadIdx.x == 0) out[row] = result;
            return;
        }
        if (P.all || lowest > P.thr) {
            // keep every element of key >= lowest: count the ties of `lowest`
            u64 c = 0;
            row_each(lg, V, [&](float x, int i) {
                if (finite_f(x) && okey(x) == lowest) ++c;
            });
            c = block_sum_u64(c, sh);
            P.all = 0; P.thr = lowest; P.ties = (unsigned)c;
        }
    }
    total = prefix_amount<true>(lg, V, mx, temp, P, sh);
    if (total == 0ull) {
        if (threadIdx.x == 0) out[row] = result;
        return;
    }
    u64 target = (u64)ceil((double)u * (double)total);
    if (target < 1) target = 1;
    if (target > total) target = total;
    unsigned nth;
    const unsigned key = radix_select<true>(lg, V, mx, temp, P, target, &nth, sh);
    const int idx = nth_equal(lg, V, key, nth, sh);
    if (idx >= 0) result = idx;
    if (threadIdx.x == 0) out[row] = result;
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
    // blocks a row: as many as keep about 148 SMs busy, so a few rows are spread wide and many
    // rows are not slowed down by blocks that mostly wait for their cluster's first
    const int qc = B <= 16 ? 8 : (B <= 32 ? 4 : (B <= 64 ? 2 : 1));
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(B * qc);
    cfg.blockDim = dim3(SM_THREADS);
    cfg.dynamicSmemBytes = 0;
    cfg.stream = stream;
    cudaLaunchAttribute attr[2];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = qc;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[1].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = lumen_pdl_enabled() ? 2 : 1;
    cudaError_t e = cudaLaunchKernelEx(&cfg, sample_kernel, logits, row_stride, V, opts, top_k, out);
    if (e != cudaSuccess) return (int)e;
    LUMEN_LAUNCH_CHECK();
    return 0;
}
