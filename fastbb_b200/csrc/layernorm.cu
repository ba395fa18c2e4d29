// LayerNorm over the last dimension fused with the cast to fp16 (input fp16, bf16 or fp32; output fp16).
// Replaces the aten native_layer_norm launches at the reference's call sites fastbb/vit.py:114,126,130,139,159,166,
// 170,184,241. One warp owns one row: the row is read from HBM once (16-byte vectors, kept in registers), mean and
// variance are computed in fp32 in two register passes (sum, then sum of squared deviations: no E[x^2]-E[x]^2
// cancellation), and the normalised row is written once. Algorithmic traffic: M*C*(in_bytes + 2) bytes.
#include "common.cuh"
#include "internal.h"

#include <cuda_bf16.h>

namespace fbb {

// 16 bytes from global memory. RO = true goes through the non-coherent (read-only) path and is only for data that no
// kernel ever writes while this one may be resident: the affine parameters. The rows of x are written by the previous
// kernel of the stream, and under programmatic dependent launch this kernel can be resident before that one has
// finished, so x is read with ordinary coherent loads (after griddepcontrol.wait).
template <bool RO>
__device__ __forceinline__ uint4 ld16(const void* p) {
    if constexpr (RO) return __ldg(reinterpret_cast<const uint4*>(p));
    else return *reinterpret_cast<const uint4*>(p);
}

template <bool RO>
__device__ __forceinline__ void load8(const void* base, int64_t elem_off, int dtype, float* f) {
    if (dtype == FBB_DTYPE_F16) {
        uint4 u = ld16<RO>(reinterpret_cast<const __half*>(base) + elem_off);
        const __half2* h = reinterpret_cast<const __half2*>(&u);
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            float2 t = __half22float2(h[i]);
            f[2 * i] = t.x;
            f[2 * i + 1] = t.y;
        }
    } else if (dtype == FBB_DTYPE_BF16) {
        uint4 u = ld16<RO>(reinterpret_cast<const __nv_bfloat16*>(base) + elem_off);
        const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&u);
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            float2 t = __bfloat1622float2(h[i]);
            f[2 * i] = t.x;
            f[2 * i + 1] = t.y;
        }
    } else {
        const float* p = reinterpret_cast<const float*>(base) + elem_off;
        const uint4 a = ld16<RO>(p), b = ld16<RO>(p + 4);
        f[0] = __uint_as_float(a.x); f[1] = __uint_as_float(a.y); f[2] = __uint_as_float(a.z); f[3] = __uint_as_float(a.w);
        f[4] = __uint_as_float(b.x); f[5] = __uint_as_float(b.y); f[6] = __uint_as_float(b.z); f[7] = __uint_as_float(b.w);
    }
}

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}

// NV = 16-byte-output vectors per lane held in registers (row length C <= 256 * NV); C % 8 == 0.
template <int NV>
__global__ void __launch_bounds__(256) layernorm_rows_kernel(const void* x, __half* __restrict__ y,
                                                            const void* __restrict__ w, const void* __restrict__ b,
                                                            int64_t M, int C, int64_t ldx, int64_t ldy, float eps,
                                                            int in_dtype, int param_dtype) {
    const int lane = threadIdx.x & 31;
    const int64_t row = (int64_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    grid_dependency_wait();
    grid_launch_dependents();
    if (row >= M) return;
    const int nvec = C >> 3;
    float v[NV][8];
    float s = 0.f;
#pragma unroll
    for (int i = 0; i < NV; ++i) {
        const int vi = lane + 32 * i;
        if (vi < nvec) {
            load8<false>(x, row * ldx + (int64_t)vi * 8, in_dtype, v[i]);
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
            if (w != nullptr) load8<true>(w, (int64_t)vi * 8, param_dtype, g);
            if (b != nullptr) load8<true>(b, (int64_t)vi * 8, param_dtype, be);
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


// Fast path for fp16 input and fp16 affine parameters: one warp normalises TWO rows at a time, and every global load of
// the iteration (both rows and the parameter vectors) is issued before the first reduction, so a warp has 3*NV 16-byte
// loads in flight instead of NV and the parameter fetch no longer waits behind the statistics. Rows are kept as raw
// fp16 vectors (16 registers for C = 1024) and converted in each of the three register passes.
template <int NV>
__global__ void __launch_bounds__(128) layernorm_rows2_f16_kernel(const __half* x, __half* __restrict__ y,
                                                                 const __half* __restrict__ w, const __half* __restrict__ b,
                                                                 int64_t M, int C, int64_t ldx, int64_t ldy, float eps) {
    const int lane = threadIdx.x & 31;
    const int64_t row0 = 2 * ((int64_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5));
    grid_dependency_wait();
    grid_launch_dependents();
    if (row0 >= M) return;
    const bool two = row0 + 1 < M;
    const int nvec = C >> 3;
    uint4 xa[NV], xb[NV], gw[NV], gb[NV];
#pragma unroll
    for (int i = 0; i < NV; ++i) {
        const int vi = lane + 32 * i;
        const bool in = vi < nvec;
        xa[i] = in ? *(reinterpret_cast<const uint4*>(x + row0 * ldx) + vi) : make_uint4(0, 0, 0, 0);
        xb[i] = (in && two) ? *(reinterpret_cast<const uint4*>(x + (row0 + 1) * ldx) + vi) : make_uint4(0, 0, 0, 0);
        gw[i] = (in && w != nullptr) ? __ldg(reinterpret_cast<const uint4*>(w) + vi) : make_uint4(0x3C003C00u, 0x3C003C00u, 0x3C003C00u, 0x3C003C00u);
        gb[i] = (in && b != nullptr) ? __ldg(reinterpret_cast<const uint4*>(b) + vi) : make_uint4(0, 0, 0, 0);
    }
    float sa = 0.f, sb = 0.f;
#pragma unroll
    for (int i = 0; i < NV; ++i) {
        const __half2* ha = reinterpret_cast<const __half2*>(&xa[i]);
        const __half2* hb = reinterpret_cast<const __half2*>(&xb[i]);
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const float2 fa = __half22float2(ha[j]), fb = __half22float2(hb[j]);
            sa += fa.x + fa.y;
            sb += fb.x + fb.y;
        }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        sa += __shfl_xor_sync(0xffffffffu, sa, o);
        sb += __shfl_xor_sync(0xffffffffu, sb, o);
    }
    const float inv_c = 1.f / (float)C;
    const float ma = sa * inv_c, mb = sb * inv_c;
    float qa = 0.f, qb = 0.f;
#pragma unroll
    for (int i = 0; i < NV; ++i) {
        if (lane + 32 * i < nvec) {
            const __half2* ha = reinterpret_cast<const __half2*>(&xa[i]);
            const __half2* hb = reinterpret_cast<const __half2*>(&xb[i]);
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                const float2 fa = __half22float2(ha[j]), fb = __half22float2(hb[j]);
                qa += (fa.x - ma) * (fa.x - ma) + (fa.y - ma) * (fa.y - ma);
                qb += (fb.x - mb) * (fb.x - mb) + (fb.y - mb) * (fb.y - mb);
            }
        }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        qa += __shfl_xor_sync(0xffffffffu, qa, o);
        qb += __shfl_xor_sync(0xffffffffu, qb, o);
    }
    const float ra = rsqrtf(qa * inv_c + eps), rb = rsqrtf(qb * inv_c + eps);
#pragma unroll
    for (int i = 0; i < NV; ++i) {
        const int vi = lane + 32 * i;
        if (vi < nvec) {
            const __half2* ha = reinterpret_cast<const __half2*>(&xa[i]);
            const __half2* hb = reinterpret_cast<const __half2*>(&xb[i]);
            const __half2* hw = reinterpret_cast<const __half2*>(&gw[i]);
            const __half2* hbias = reinterpret_cast<const __half2*>(&gb[i]);
            uint4 oa, ob;
            uint32_t* pa = reinterpret_cast<uint32_t*>(&oa);
            uint32_t* pb = reinterpret_cast<uint32_t*>(&ob);
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                const float2 fa = __half22float2(ha[j]), fb = __half22float2(hb[j]);
                const float2 g = __half22float2(hw[j]), be = __half22float2(hbias[j]);
                pa[j] = pack_h2(fmaf((fa.x - ma) * ra, g.x, be.x), fmaf((fa.y - ma) * ra, g.y, be.y));
                pb[j] = pack_h2(fmaf((fb.x - mb) * rb, g.x, be.x), fmaf((fb.y - mb) * rb, g.y, be.y));
            }
            *(reinterpret_cast<uint4*>(y + row0 * ldy) + vi) = oa;
            if (two) *(reinterpret_cast<uint4*>(y + (row0 + 1) * ldy) + vi) = ob;
        }
    }
}

// Any C % 8 == 0 (rows longer than 2048): three passes over the row, the second and third served by L1/L2.
__global__ void __launch_bounds__(256) layernorm_long_rows_kernel(const void* x, __half* __restrict__ y,
                                                                 const void* __restrict__ w, const void* __restrict__ b,
                                                                 int64_t M, int C, int64_t ldx, int64_t ldy, float eps,
                                                                 int in_dtype, int param_dtype) {
    const int lane = threadIdx.x & 31;
    const int64_t row = (int64_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    grid_dependency_wait();
    grid_launch_dependents();
    if (row >= M) return;
    const int nvec = C >> 3;
    float f[8];
    float s = 0.f;
    for (int vi = lane; vi < nvec; vi += 32) {
        load8<false>(x, row * ldx + (int64_t)vi * 8, in_dtype, f);
#pragma unroll
        for (int j = 0; j < 8; ++j) s += f[j];
    }
    const float mean = warp_sum(s) / (float)C;
    float q = 0.f;
    for (int vi = lane; vi < nvec; vi += 32) {
        load8<false>(x, row * ldx + (int64_t)vi * 8, in_dtype, f);
#pragma unroll
        for (int j = 0; j < 8; ++j) q += (f[j] - mean) * (f[j] - mean);
    }
    const float rstd = rsqrtf(warp_sum(q) / (float)C + eps);
    for (int vi = lane; vi < nvec; vi += 32) {
        float g[8], be[8];
        load8<false>(x, row * ldx + (int64_t)vi * 8, in_dtype, f);
        if (w != nullptr) load8<true>(w, (int64_t)vi * 8, param_dtype, g);
        if (b != nullptr) load8<true>(b, (int64_t)vi * 8, param_dtype, be);
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

// Final norm of a ViT with its outputs split the way get_intermediate_layers hands them out (fastbb/vit.py:184,225-232):
// the rows of x [B, N, C] (fp16) are normalised (or just copied, apply_norm = 0) and written to three destinations in one
// launch: the cls row of each image to cls_out [B, C], the register rows to regs_out [B, n_prefix - 1, C], and the patch
// rows to patches_out either token-major [B, HW, C] or channel-major [B, C, HW] (= [B, C, h, w], what reshape=True
// returns after its permute + contiguous copy). A CTA takes 32 consecutive patch tokens of one image (or the prefix rows
// of one image): each warp normalises four rows in registers, two-pass statistics as in the kernels above; for the
// channel-major layout the fp16 rows go through a padded shared-memory tile so that the global stores run along the
// token axis (32 tokens = 64 contiguous bytes per channel) instead of scattering 2-byte elements C*HW apart.
constexpr int kSplitTokens = 32;

template <int NV>
__global__ void __launch_bounds__(256) layernorm_split_f16_kernel(const __half* x, const __half* __restrict__ w, const __half* __restrict__ b,
                                                                 __half* __restrict__ patches_out, __half* __restrict__ cls_out,
                                                                 __half* __restrict__ regs_out, int N, int C, int n_prefix, float eps,
                                                                 int apply_norm, int channel_major) {
    extern __shared__ __align__(16) uint8_t split_smem[];
    __half* tile = reinterpret_cast<__half*>(split_smem);  // [kSplitTokens][C + 2], channel-major output only
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int HW = N - n_prefix;
    const int tiles = (HW + kSplitTokens - 1) / kSplitTokens;  // patch tiles per image; tile index `tiles` = the prefix rows
    const int img = blockIdx.x / (tiles + 1);
    const int t = blockIdx.x - img * (tiles + 1);
    const bool prefix = t == tiles;
    const int row_begin = prefix ? 0 : n_prefix + t * kSplitTokens;
    const int row_end = prefix ? n_prefix : min(N, row_begin + kSplitTokens);
    const int nvec = C >> 3;
    const int ldt = C + 2;
    grid_dependency_wait();
    grid_launch_dependents();
    for (int r = row_begin + warp; r < row_end; r += 8) {
        const __half* xr = x + ((int64_t)img * N + r) * C;
        uint4 xv[NV];
#pragma unroll
        for (int i = 0; i < NV; ++i) {
            const int vi = lane + 32 * i;
            xv[i] = vi < nvec ? *(reinterpret_cast<const uint4*>(xr) + vi) : make_uint4(0, 0, 0, 0);
        }
        float mean = 0.f, rstd = 1.f;
        if (apply_norm) {
            float sum = 0.f;
#pragma unroll
            for (int i = 0; i < NV; ++i) {
                const __half2* h = reinterpret_cast<const __half2*>(&xv[i]);
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    const float2 f = __half22float2(h[j]);
                    sum += f.x + f.y;
                }
            }
            const float inv_c = 1.f / (float)C;  // same arithmetic as layernorm_rows2_f16_kernel: the two give identical bits
            mean = warp_sum(sum) * inv_c;
            float q = 0.f;
#pragma unroll
            for (int i = 0; i < NV; ++i) {
                if (lane + 32 * i < nvec) {
                    const __half2* h = reinterpret_cast<const __half2*>(&xv[i]);
#pragma unroll
                    for (int j = 0; j < 4; ++j) {
                        const float2 f = __half22float2(h[j]);
                        q += (f.x - mean) * (f.x - mean) + (f.y - mean) * (f.y - mean);
                    }
                }
            }
            rstd = rsqrtf(warp_sum(q) * inv_c + eps);
        }
        __half* dst;  // token-major destination row, or the shared tile row
        if (prefix) dst = r == 0 ? (cls_out != nullptr ? cls_out + (int64_t)img * C : nullptr)
                                 : (regs_out != nullptr ? regs_out + ((int64_t)img * (n_prefix - 1) + (r - 1)) * C : nullptr);
        else dst = channel_major ? tile + (r - row_begin) * ldt : patches_out + ((int64_t)img * HW + (r - n_prefix)) * C;
        if (dst == nullptr) continue;
#pragma unroll
        for (int i = 0; i < NV; ++i) {
            const int vi = lane + 32 * i;
            if (vi < nvec) {
                uint4 out = xv[i];
                if (apply_norm) {
                    const uint4 gw = w != nullptr ? __ldg(reinterpret_cast<const uint4*>(w) + vi) : make_uint4(0x3C003C00u, 0x3C003C00u, 0x3C003C00u, 0x3C003C00u);
                    const uint4 gb = b != nullptr ? __ldg(reinterpret_cast<const uint4*>(b) + vi) : make_uint4(0, 0, 0, 0);
                    const __half2* h = reinterpret_cast<const __half2*>(&xv[i]);
                    const __half2* hw = reinterpret_cast<const __half2*>(&gw);
                    const __half2* hb = reinterpret_cast<const __half2*>(&gb);
                    uint32_t* o = reinterpret_cast<uint32_t*>(&out);
#pragma unroll
                    for (int j = 0; j < 4; ++j) {
                        const float2 f = __half22float2(h[j]), g = __half22float2(hw[j]), be = __half22float2(hb[j]);
                        o[j] = pack_h2(fmaf((f.x - mean) * rstd, g.x, be.x), fmaf((f.y - mean) * rstd, g.y, be.y));
                    }
                }
                if (!prefix && channel_major) {  // tile rows are only 4-byte aligned (C + 2 halves): four 4-byte stores
                    uint32_t* d32 = reinterpret_cast<uint32_t*>(dst + vi * 8);
                    const uint32_t* o = reinterpret_cast<const uint32_t*>(&out);
                    d32[0] = o[0]; d32[1] = o[1]; d32[2] = o[2]; d32[3] = o[3];
                } else {
                    *(reinterpret_cast<uint4*>(dst) + vi) = out;
                }
            }
        }
    }
    if (prefix || !channel_major) return;
    __syncthreads();
    // transposed store: lane = token of the tile, a warp covers channel pairs c, c+1 (one 4-byte shared-memory read per
    // lane, bank (C/2 + 1) * lane + c/2: conflict-free because C/2 + 1 is odd) and writes two 64-byte runs along the tokens
    const int tok = row_begin - n_prefix + lane;
    const bool tok_ok = row_begin + lane < row_end;
    __half* base = patches_out + (int64_t)img * C * HW + tok;
    for (int c = 2 * warp; c < C; c += 16) {
        const __half2 v = *reinterpret_cast<const __half2*>(tile + lane * ldt + c);
        if (tok_ok) {
            base[(int64_t)c * HW] = __low2half(v);
            base[(int64_t)(c + 1) * HW] = __high2half(v);
        }
    }
}

int launch_layernorm_split(const void* x, const void* w, const void* b, void* patches_out, void* cls_out, void* regs_out, int B, int N, int C,
                           int n_prefix, float eps, int apply_norm, int channel_major, cudaStream_t stream) {
    if (B == 0 || N == 0) return FBB_OK;
    const int HW = N - n_prefix;
    const int tiles = (HW + kSplitTokens - 1) / kSplitTokens;
    const unsigned grid = (unsigned)B * (unsigned)(tiles + 1);
    const size_t smem = channel_major ? (size_t)kSplitTokens * (C + 2) * sizeof(__half) : 0;
    const int nv = (C / 8 + 31) / 32;
    const __half* xh = reinterpret_cast<const __half*>(x);
    const __half* wh = reinterpret_cast<const __half*>(w);
    const __half* bh = reinterpret_cast<const __half*>(b);
    __half *po = reinterpret_cast<__half*>(patches_out), *co = reinterpret_cast<__half*>(cls_out), *ro = reinterpret_cast<__half*>(regs_out);
    cudaError_t err = cudaSuccess;
#define FBB_LNS_CASE(NVV)                                                                                                       \
    case NVV: {                                                                                                                 \
        auto kern = layernorm_split_f16_kernel<NVV>;                                                                            \
        if (smem > 48 * 1024) {                                                                                                 \
            err = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);                           \
            if (err != cudaSuccess) break;                                                                                      \
        }                                                                                                                       \
        err = launch_pdl(kern, dim3(grid), dim3(256), smem, stream, xh, wh, bh, po, co, ro, N, C, n_prefix, eps, apply_norm, channel_major); \
        break;                                                                                                                  \
    }
    switch (nv) {
        FBB_LNS_CASE(1)
        FBB_LNS_CASE(2)
        FBB_LNS_CASE(3)
        FBB_LNS_CASE(4)
        FBB_LNS_CASE(5)
        FBB_LNS_CASE(6)
        FBB_LNS_CASE(7)
        FBB_LNS_CASE(8)
        default:
            return fail(FBB_ERR_SHAPE, "layernorm_split: rows longer than 2048 elements are not covered (C=%d)", C);
    }
#undef FBB_LNS_CASE
    return cuda_status(err);
}

int launch_layernorm(const void* x, void* y, const void* w, const void* b, int64_t M, int C, int64_t ldx, int64_t ldy,
                     float eps, int in_dtype, int param_dtype, cudaStream_t stream) {
    if (M == 0) return FBB_OK;
    const int warps = 8;
    const unsigned grid = (unsigned)((M + warps - 1) / warps);
    const int nv = (C / 8 + 31) / 32;
    __half* yh = reinterpret_cast<__half*>(y);
    cudaError_t err = cudaSuccess;
    if (in_dtype == FBB_DTYPE_F16 && param_dtype == FBB_DTYPE_F16 && nv >= 1 && nv <= 6) {
        const __half* xh = reinterpret_cast<const __half*>(x);
        const __half* wh = reinterpret_cast<const __half*>(w);
        const __half* bh = reinterpret_cast<const __half*>(b);
        const unsigned grid2 = (unsigned)((M + 7) / 8);  // 4 warps x 2 rows per block
#define FBB_LN2_CASE(N)                                                                                              \
    case N:                                                                                                          \
        err = launch_pdl(layernorm_rows2_f16_kernel<N>, dim3(grid2), dim3(128), 0, stream, xh, yh, wh, bh, M, C, ldx, ldy, eps); \
        break;
        switch (nv) {
            FBB_LN2_CASE(1)
            FBB_LN2_CASE(2)
            FBB_LN2_CASE(3)
            FBB_LN2_CASE(4)
            FBB_LN2_CASE(5)
            FBB_LN2_CASE(6)
        }
#undef FBB_LN2_CASE
        return cuda_status(err);
    }
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
