// One head of 128 values of the QKV projection, by one warp: the projection's partial sums
// added in rising order, the head's RMSNorm (weight nw, or none), the rotation of the pairs
// (i, i + 64) by the token's (cos, sin) table (or none). A lane holds values 4 lane .. 4 lane + 3;
// the partner of a value in the rotation lives 16 lanes away, so nothing goes through shared
// memory. The decode step's rotary kernel (core.cu) and the decode attention that does this
// work itself (attn_decode.cu) both call it, and so give the same bits.
// Formulas: crates/aegisllm-cuda/src/cuda/kernels/blackwell/norm_rope_kv.cu:36-62 (norm),
// :437-447, 465-492 (rotation).
#pragma once
#include "common.cuh"

__device__ __forceinline__ float4 qk_head_d128(const float* __restrict__ src, int S, size_t split_stride,
                                               const float* __restrict__ nw, float eps,
                                               const float2* __restrict__ cs_token, bool rotate, int lane) {
    src += 4 * lane;
    float4 v = *reinterpret_cast<const float4*>(src);
    for (int s0 = 1; s0 < S; s0 += 8) {       // the partial sums' loads go out together, added in rising order
        float4 v2[8];
#pragma unroll
        for (int j = 0; j < 8; ++j)
            if (s0 + j < S) v2[j] = *reinterpret_cast<const float4*>(src + (size_t)(s0 + j) * split_stride);
#pragma unroll
        for (int j = 0; j < 8; ++j)
            if (s0 + j < S) { v.x += v2[j].x; v.y += v2[j].y; v.z += v2[j].z; v.w += v2[j].w; }
    }
    if (nw) {
        float ss = v.x * v.x;
        ss += v.y * v.y;
        ss += v.z * v.z;
        ss += v.w * v.w;
        ss = warp_sum(ss);
        const float scale = 1.0f / sqrtf(ss / 128.0f + eps);
        const float4 g = *reinterpret_cast<const float4*>(nw + 4 * lane);
        v.x = v.x * scale * g.x; v.y = v.y * scale * g.y; v.z = v.z * scale * g.z; v.w = v.w * scale * g.w;
    }
    if (rotate) {
        const float4 o = make_float4(__shfl_xor_sync(0xffffffffu, v.x, 16), __shfl_xor_sync(0xffffffffu, v.y, 16),
                                     __shfl_xor_sync(0xffffffffu, v.z, 16), __shfl_xor_sync(0xffffffffu, v.w, 16));
        const float4* csn = reinterpret_cast<const float4*>(cs_token + 4 * (lane & 15));
        const float4 c01 = csn[0], c23 = csn[1];     // (cos, sin) of 4 consecutive pairs
        if (lane < 16) {     // x'_i = x_i cos - x_{i+64} sin
            v.x = v.x * c01.x - o.x * c01.y; v.y = v.y * c01.z - o.y * c01.w;
            v.z = v.z * c23.x - o.z * c23.y; v.w = v.w * c23.z - o.w * c23.w;
        } else {             // x'_{i+64} = x_i sin + x_{i+64} cos
            v.x = o.x * c01.y + v.x * c01.x; v.y = o.y * c01.w + v.y * c01.z;
            v.z = o.z * c23.y + v.z * c23.x; v.w = o.w * c23.w + v.w * c23.z;
        }
    }
    return v;
}
