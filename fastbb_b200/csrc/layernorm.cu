// LayerNorm over the last dimension fused with the cast to fp16 (input fp16, bf16 or fp32; output fp16).
// Replaces the aten native_layer_norm launches at the reference's call sites fastbb/vit.py:114,126,130,139,159,166,
// 170,184,241. One warp owns one row: the row is read from HBM once (16-byte vectors, kept in registers), mean and
// variance are computed in fp32 in two register passes (sum, then sum of squared deviations: no E[x^2]-E[x]^2
// cancellation), and the normalised row is written once. Algorithmic traffic: M*C*(in_bytes + 2) bytes.
#include "common.cuh"
#include "internal.h"

#include <cuda_bf16.h>

namespace fbb {

__device__ __forceinline__ void load8(const void* base, int64_t elem_off, int dtype, float* f) {
    if (dtype == FBB_DTYPE_F16) {
        uint4 u = __ldg(reinterpret_cast<const uint4*>(reinterpret_cast<const __half*>(base) + elem_off));
        const __half2* h = reinterpret_cast<const __half2*>(&u);
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            float2 t = __half22float2(h[i]);
            f[2 * i] = t.x;
            f[2 * i + 1] = t.y;
        }
    } else if (dtype == FBB_DTYPE_BF16) {
        uint4 u = __ldg(reinterpret_cast<const uint4*>(reinterpret_cast<const __nv_bfloat16*>(base) + elem_off));
        const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&u);
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            float2 t = __bfloat1622float2(h[i]);
            f[2 * i] = t.x;
            f[2 * i + 1] = t.y;
        }
    } else {
        const float4* p = reinterpret_cast<const float4*>(reinterpret_cast<const float*>(base) + elem_off);
        float4 a = __ldg(p), b = __ldg(p + 1);
        f[0] = a.x; f[1] = a.y; f[2] = a.z; f[3] = a.w;
        f[4] = b.x; f[5] = b.y; f[6] = b.z; f[7] = b.w;
    }
}

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}

// NV = 16-byte-output vectors per lane held in registers (row length C <= 256 * NV); C % 8 == 0.
template <int NV>
__global__ void __launch_bounds__(256) layernorm_rows_kernel(const void* __restrict__ x, __half* __restrict__ y,
                                                            const void* __restrict__ w, const void* __restrict__ b,
                                                            int64_t M, int C, int64_t ldx, int64_t ldy, float eps,
                                                            int in_dtype, int param_dtype) {
    const int lane = threadIdx.x & 31;
    const int64_t row = (int64_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    grid_dependency_wait();
    if (row >= M) return;
    const int nvec = C >> 3;
    float v[NV][8];
    float s = 0.f;
#pragma unroll
    for (int i = 0; i < NV; ++i) {
        const int vi = lane + 32 * i;
        if (vi < nvec) {
            load8(x, row * ldx + (int64_t)vi * 8, in_dtype, v[i]);
#pragma unroll
            for (int j = 0; j < 8; ++j) s += v[i][j];
        } else {
#pragma unroll
            for (int j = 0; j < 8; ++j) v[i][j] = 0.f;
        }
    }
    const float mean = warp_sum(s) / (float)C;
    float q = 0.f;
#pragma unroll
    for (int i = 0; i < NV; ++i) {
        if (lane + 32 * i < nvec) {
#pragma unroll
            for (int j = 0; j < 8; ++j) {
                const float d = v[i][j] - mean;
                q += d * d;
            }
        }
    }
    const float rstd = rsqrtf(warp_sum(q) / (float)C + eps);
#pragma unroll
    for (int i = 0; i < NV; ++i) {
        const int vi = lane + 32 * i;
        if (vi < nvec) {
            float g[8], be[8];
            if (w != nullptr) load8(w, (int64_t)vi * 8, param_dtype, g);
            if (b != nullptr) load8(b, (int64_t)vi * 8, param_dtype, be);
            uint4 out;
            uint32_t* o = reinterpret_cast<uint32_t*>(&out);
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                float a0 = (v[i][2 * j] - mean) * rstd, a1 = (v[i][2 * j + 1] - mean) * rstd;
                if (w != nullptr) { a0 *= g[2 * j]; a1 *= g[2 * j + 1]; }
                if (b != nullptr) { a0 += be[2 * j]; a1 += be[2 * j + 1]; }
                o[j] = pack_h2(a0, a1);
            }
            *reinterpret_cast<uint4*>(y + row * ldy + (int64_t)vi * 8) = out;
        }
    }
}

// Any C % 8 == 0 (rows longer than 2048): three passes over the row, the second and third served by L1/L2.
__global__ void __launch_bounds__(256) layernorm_long_rows_kernel(const void* __restrict__ x, __half* __restrict__ y,
                                                                 const void* __restrict__ w, const void* __restrict__ b,
                                                                 int64_t M, int C, int64_t ldx, int64_t ldy, float eps,
                                                                 int in_dtype, int param_dtype) {
    const int lane = threadIdx.x & 31;
    const int64_t row = (int64_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    grid_dependency_wait();
    if (row >= M) return;
    const int nvec = C >> 3;
    float f[8];
    float s = 0.f;
    for (int vi = lane; vi < nvec; vi += 32) {
        load8(x, row * ldx + (int64_t)vi * 8, in_dtype, f);
#pragma unroll
        for (int j = 0; j < 8; ++j) s += f[j];
    }
    const float mean = warp_sum(s) / (float)C;
    float q = 0.f;
    for (int vi = lane; vi < nvec; vi += 32) {
        load8(x, row * ldx + (int64_t)vi * 8, in_dtype, f);
#pragma unroll
        for (int j = 0; j < 8; ++j) q += (f[j] - mean) * (f[j] - mean);
    }
    const float rstd = rsqrtf(warp_sum(q) / (float)C + eps);
    for (int vi = lane; vi < nvec; vi += 32) {
        float g[8], be[8];
        load8(x, row * ldx + (int64_t)vi * 8, in_dtype, f);
        if (w != nullptr) load8(w, (int64_t)vi * 8, param_dtype, g);
        if (b != nullptr) load8(b, (int64_t)vi * 8, param_dtype, be);
        uint4 out;
        uint32_t* o = reinterpret_cast<uint32_t*>(&out);
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            float a0 = (f[2 * j] - mean) * rstd, a1 = (f[2 * j + 1] - mean) * rstd;
            if (w != nullptr) { a0 *= g[2 * j]; a1 *= g[2 * j + 1]; }
            if (b != nullptr) { a0 += be[2 * j]; a1 += be[2 * j + 1]; }
            o[j] = pack_h2(a0, a1);
        }
        *reinterpret_cast<uint4*>(y + row * ldy + (int64_t)vi * 8) = out;
    }
}

int launch_layernorm(const void* x, void* y, const void* w, const void* b, int64_t M, int C, int64_t ldx, int64_t ldy,
                     float eps, int in_dtype, int param_dtype, cudaStream_t stream) {
    if (M == 0) return FBB_OK;
    const int warps = 8;
    const unsigned grid = (unsigned)((M + warps - 1) / warps);
    const int nv = (C / 8 + 31) / 32;
    __half* yh = reinterpret_cast<__half*>(y);
    cudaError_t err = cudaSuccess;
#define FBB_LN_CASE(N)                                                                                              \
    case N:                                                                                                         \
        err = launch_pdl(layernorm_rows_kernel<N>, dim3(grid), dim3(warps * 32), 0, stream, x, yh, w, b, M, C, ldx, ldy, eps, in_dtype, param_dtype); \
        break;
    switch (nv) {
        FBB_LN_CASE(1)
        FBB_LN_CASE(2)
        FBB_LN_CASE(3)
        FBB_LN_CASE(4)
        FBB_LN_CASE(5)
        FBB_LN_CASE(6)
        FBB_LN_CASE(7)
        FBB_LN_CASE(8)
        default:
            err = launch_pdl(layernorm_long_rows_kernel, dim3(grid), dim3(warps * 32), 0, stream, x, yh, w, b, M, C, ldx, ldy, eps, in_dtype, param_dtype);
    }
#undef FBB_LN_CASE
    return cuda_status(err);
}

}  // namespace fbb
