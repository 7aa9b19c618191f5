// A measurement, not a part of the model: how fast G blocks, one an SM, stream a matrix of
// bfloat16 weights into rings of shared memory, 16 KB (128 rows x 64 values of k) a stage, when
// nothing is done with the data. It answers two questions the matrix products' design rests on:
// what one SM can take in (55-65 GB/s, however deep the ring), and what the form of the weights
// in memory is worth (tiles that lie in one piece stream 3-6 % faster than boxes cut out of a
// row-major matrix). `python -m lumenllm_b200.kbench stream` runs it.
//
// mode 0: the matrix is row-major [G * 128, nkb * 64]; a stage is a tensor copy of a box of 128
//         rows x 128 bytes (128-byte swizzle), its rows a whole matrix row apart.
// mode 1: the matrix is in the tiled form of csrc/gemm_tc.cu (k block after k block, 128-byte
//         rows in a row); a stage is a tensor copy of 128 such rows, 16 KB in one piece.
// mode 2: tiled form as in mode 1, but the matrix has `rounds` times as many tiles as there are
//         blocks, and a block streams all k blocks of tile b, then of tile b + G, ... as the
//         weight-streaming product does with a tall weight (the k blocks of a tile lie a whole
//         matrix of tiles apart).
// mode 3: the same work on a matrix stored tile after tile (a tile's k blocks in a row).
// One thread asks for the copies, one waits for them, reads a word and gives the stage back.
// Every wait is bounded; a wait that runs out sets *err.
#include <cuda.h>

#include "common.cuh"
#include "mma_utils.cuh"

__device__ __forceinline__ void sp_arrive(uint64_t* bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void sp_tma_2d(void* dst, const CUtensorMap* map, int c0, int c1, uint64_t* bar) {
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];" ::"r"(
            smem_u32(dst)),
        "l"(reinterpret_cast<uint64_t>(map)), "r"(smem_u32(bar)), "r"(c0), "r"(c1)
        : "memory");
}

#define SP_MAX_STAGES 12
#define SP_STAGE_BYTES 16384

__global__ void __launch_bounds__(64, 1)
stream_probe_kernel(const __grid_constant__ CUtensorMap tm, int nkb, int stages, int mode, int rounds, int* err,
                    unsigned* sink) {
    extern __shared__ __align__(1024) unsigned char sp_smem_raw[];
    unsigned char* smem = sp_smem_raw + ((1024u - (smem_u32(sp_smem_raw) & 1023u)) & 1023u);
    __shared__ uint64_t full[SP_MAX_STAGES], empty[SP_MAX_STAGES];
    if (threadIdx.x == 0) {
        for (int i = 0; i < stages; ++i) { mbar_init(&full[i], 1); mbar_init(&empty[i], 1); }
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncthreads();
    if (threadIdx.x == 0) {
        const int tiles = gridDim.x * rounds;
        for (int it = 0; it < nkb * rounds; ++it) {
            const int st = it % stages, ph = (it / stages) & 1;
            if (it >= stages && !mbar_wait(&empty[st], ph ^ 1)) { atomicExch(err, 1); break; }
            mbar_expect_tx(&full[st], SP_STAGE_BYTES);
            const int kb = it % nkb, tile = blockIdx.x + (it / nkb) * gridDim.x;
            if (mode == 0)      sp_tma_2d(smem + st * SP_STAGE_BYTES, &tm, it * 64, blockIdx.x * 128, &full[st]);
            else if (mode == 3) sp_tma_2d(smem + st * SP_STAGE_BYTES, &tm, 0, (tile * nkb + kb) * 128, &full[st]);
            else                sp_tma_2d(smem + st * SP_STAGE_BYTES, &tm, 0, (kb * tiles + tile) * 128, &full[st]);
        }
    } else if (threadIdx.x == 32) {
        unsigned acc = 0;
        for (int it = 0; it < nkb * rounds; ++it) {
            const int st = it % stages, ph = (it / stages) & 1;
            if (!mbar_wait(&full[st], ph)) { atomicExch(err, 1); break; }
            acc += *reinterpret_cast<volatile unsigned*>(smem + st * SP_STAGE_BYTES + 4 * (it & 1023));
            sp_arrive(&empty[st]);
        }
        if (acc == 0x12345678u) *sink = acc;      // keeps the reads alive
    }
}

typedef CUresult (*SpEncodeFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                               const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                               CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

// base: G * rounds * nkb * 16 KB of device memory, 1,024-byte aligned (rounds = 1 for modes 0 and 1);
// scratch: two ints (error flag, sink).
LUMEN_API int lumen_stream_probe(void* base, int G, int nkb, int stages, int mode, int rounds, int* scratch,
                                 cudaStream_t stream) {
    if (mode < 2) rounds = 1;
    if (G < 1 || nkb < 1 || rounds < 1 || stages < 1 || stages > SP_MAX_STAGES || mode < 0 || mode > 3 || !base || !scratch ||
        ((uintptr_t)base & 1023))
        return LUMEN_ERR_BAD_ARGUMENT;
    static SpEncodeFn fn = nullptr;
    if (!fn) {
        void* ptr = nullptr;
        cudaDriverEntryPointQueryResult res;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &res) != cudaSuccess ||
            res != cudaDriverEntryPointSuccess)
            return LUMEN_ERR_UNSUPPORTED;
        fn = (SpEncodeFn)ptr;
    }
    CUtensorMap map;
    cuuint64_t dims[2] = {(cuuint64_t)nkb * 64, (cuuint64_t)G * 128};
    cuuint64_t strides[1] = {(cuuint64_t)nkb * 128};
    if (mode >= 1) {
        dims[0] = 64;
        dims[1] = (cuuint64_t)nkb * G * rounds * 128;
        strides[0] = 128;
    }
    cuuint32_t box[2] = {64, 128};
    cuuint32_t estr[2] = {1, 1};
    if (fn(&map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, base, dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
           mode == 0 ? CU_TENSOR_MAP_SWIZZLE_128B : CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
           CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS)
        return LUMEN_ERR_BAD_ARGUMENT;
    const int smem = stages * SP_STAGE_BYTES + 1024;
    static int attr_set = 0;
    if (attr_set < smem) {
        cudaError_t e = cudaFuncSetAttribute(stream_probe_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
        if (e != cudaSuccess) return (int)e;
        attr_set = smem;
    }
    stream_probe_kernel<<<G, 64, smem, stream>>>(map, nkb, stages, mode, rounds, scratch, (unsigned*)(scratch + 1));
    LUMEN_LAUNCH_CHECK();
    return 0;
}
