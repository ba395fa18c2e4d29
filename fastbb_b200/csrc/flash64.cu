// O = softmax(scale . Q K^T) V for head dimension 64, no mask, any N: tcgen05 UMMA for both products, softmax in
// registers, K/V tiles streamed by TMA. Replaces flash64_r{1,2}_{hh,fh,ff} (fastbb/fastbb_kernels.cu:58-312) and the
// SDPA fallback for small inputs (fastbb/vit.py:146-150). Q, K, V are read in place from the strided [b, n, h, 64]
// views of the packed qkv GEMM output; O is written as [b, n, h*64].
//
// One CTA owns NQ (1 or 2) tiles of 128 queries of one (batch, head) and walks the keys in blocks of 128:
//   warp 0          TMA producer: Q tiles once, then K_j and V_j into a ring of stages (128-byte swizzle, zero fill)
//   warp 1          UMMA issuer: S_t = Q_t K_j^T (both K-major, 4 x K16) into tensor memory; after the softmax group
//                   has written P_t (fp16) back into tensor memory, PV_t = P_t V_j (A from tensor memory, V as the
//                   MN-major B operand, 8 x K16) into a second tensor-memory region, from zero for every key block
//   warps 2..5/6..9 softmax group t: one thread per query row (tcgen05.ld 32x32b gives a thread its whole row, so the
//                   row maximum and row sum need no shuffles); running max / sum / O in fp32 registers, base-2
//                   exponentials; O = O * exp2(m_old - m_new) + PV_t is applied one key block late so the P.V product
//                   of block j overlaps the exponentials of block j+1. With NQ = 2 the two groups alternate on the
//                   tensor core (S of one tile is computed while the other tile is in its softmax).
// Variants (fastbb/attention.py:5-7): ff = fp32 accumulate for S and PV; fh = fp32 S, fp16-accumulated PV per key
// block added into the fp32 O; hh = fp16 accumulate for both, exponentials on half2 pairs.
#include "common.cuh"
#include "internal.h"

namespace fbb {

constexpr int FQ = 128;       // queries per tile
constexpr int FK = 128;       // keys per block
constexpr int kKVStages = 4;
constexpr int kTileBytes = 128 * 64 * 2;  // one [128 x 64] fp16 tile

// tensor-memory columns
constexpr uint32_t kColS = 0;      // S_t at kColS + t*128 (128 columns each)
constexpr uint32_t kColP = 256;    // P_t at kColP + t*64 (fp16 pairs: 64 columns each)
constexpr uint32_t kColPV = 384;   // PV_t at kColPV + t*64 (64 columns each)

struct FlashSmem {
    static constexpr int kQOff = 0;                                  // NQ x 16 KB
    static constexpr int kKOff = 2 * kTileBytes;                     // stages x 16 KB
    static constexpr int kVOff = kKOff + kKVStages * kTileBytes;     // stages x 16 KB
    static constexpr int kBarOff = kVOff + kKVStages * kTileBytes;
    // barriers: q_full, k_full[S], v_full[S], k_empty[S], v_empty[S], s_full[2], p_ready[2], pv_full[2], pv_empty[2]
    static constexpr int kNumBars = 1 + 4 * kKVStages + 8;
    static constexpr int kBytes = kBarOff + kNumBars * 8 + 16;
    static constexpr int kDynamic = kBytes + 1024;
};

struct FlashArgs {
    __half* o;
    int N, H;
    int64_t o_sb, o_sn, o_sh;
    float scale_log2;
};

template <int NQ, bool S16, bool PV16>
__global__ void __launch_bounds__(64 + 128 * NQ, 1)
flash64_umma_kernel(const __grid_constant__ CUtensorMap tmap_q, const __grid_constant__ CUtensorMap tmap_k,
                    const __grid_constant__ CUtensorMap tmap_v, const FlashArgs a) {
    using S = FlashSmem;
    extern __shared__ uint8_t smem_raw[];
    const uint32_t raw = smem_u32(smem_raw);
    const uint32_t base = (raw + 1023u) & ~1023u;
    uint8_t* gen = smem_raw + (base - raw);
    const uint32_t bar0 = base + S::kBarOff;
    const uint32_t q_full = bar0;
    auto k_full = [&](int s) { return bar0 + 8u * (1 + s); };
    auto v_full = [&](int s) { return bar0 + 8u * (1 + kKVStages + s); };
    auto k_empty = [&](int s) { return bar0 + 8u * (1 + 2 * kKVStages + s); };
    auto v_empty = [&](int s) { return bar0 + 8u * (1 + 3 * kKVStages + s); };
    auto s_full = [&](int t) { return bar0 + 8u * (1 + 4 * kKVStages + t); };
    auto p_ready = [&](int t) { return bar0 + 8u * (1 + 4 * kKVStages + 2 + t); };
    auto pv_full = [&](int t) { return bar0 + 8u * (1 + 4 * kKVStages + 4 + t); };
    auto pv_empty = [&](int t) { return bar0 + 8u * (1 + 4 * kKVStages + 6 + t); };
    volatile uint32_t* s_tmem = reinterpret_cast<volatile uint32_t*>(gen + S::kBarOff + S::kNumBars * 8);
    volatile int* s_abort = reinterpret_cast<volatile int*>(gen + S::kBarOff + S::kNumBars * 8 + 4);

    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;
    const int bh = blockIdx.y;
    const int b = bh / a.H, h = bh % a.H;
    const int q0 = blockIdx.x * (FQ * NQ);
    const int nkb = (a.N + FK - 1) / FK;

    if (threadIdx.x == 0) {
        mbar_init(q_full, 1);
        for (int s = 0; s < kKVStages; ++s) {
            mbar_init(k_full(s), 1);
            mbar_init(v_full(s), 1);
            mbar_init(k_empty(s), 1);
            mbar_init(v_empty(s), 1);
        }
        for (int t = 0; t < 2; ++t) {
            mbar_init(s_full(t), 1);
            mbar_init(p_ready(t), 4);
            mbar_init(pv_full(t), 1);
            mbar_init(pv_empty(t), 4);
        }
        *s_abort = 0;
        fence_barrier_init();
        tma_prefetch_desc(&tmap_q);
        tma_prefetch_desc(&tmap_k);
        tma_prefetch_desc(&tmap_v);
    }
    if (warp == 1) {
        __syncwarp();
        tmem_alloc<512>(smem_u32(const_cast<uint32_t*>(s_tmem)));
        tmem_relinquish();
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *s_tmem;

    if (warp == 0) {
        // ------------------------------------------------------------------ TMA producer
        if (lane == 0) {
            mbar_arrive_expect_tx(q_full, NQ * kTileBytes);
            for (int t = 0; t < NQ; ++t) tma_load_4d(base + S::kQOff + t * kTileBytes, &tmap_q, q_full, 0, h, q0 + t * FQ, b);
            int s = 0;
            uint32_t ph = 0;
            bool ok = true;
            for (int j = 0; j < nkb; ++j) {
                if (!mbar_wait(k_empty(s), ph ^ 1u, s_abort, DEV_TIMEOUT_SMEM_EMPTY, s)) { ok = false; break; }
                mbar_arrive_expect_tx(k_full(s), kTileBytes);
                tma_load_4d(base + S::kKOff + s * kTileBytes, &tmap_k, k_full(s), 0, h, j * FK, b);
                if (!mbar_wait(v_empty(s), ph ^ 1u, s_abort, DEV_TIMEOUT_SMEM_EMPTY, 16 + s)) { ok = false; break; }
                mbar_arrive_expect_tx(v_full(s), kTileBytes);
                tma_load_4d(base + S::kVOff + s * kTileBytes, &tmap_v, v_full(s), 0, h, j * FK, b);
                if (++s == kKVStages) { s = 0; ph ^= 1u; }
            }
            if (!ok) __nanosleep(20000);
        }
    } else if (warp == 1) {
        // ------------------------------------------------------------------ UMMA issuer
        if (lane == 0) {
            const uint32_t idesc_qk = make_idesc_f16(FQ, FK, !S16, false, false);
            const uint32_t idesc_pv = make_idesc_f16(FQ, 64, !PV16, false, true);
            constexpr uint64_t desc_hi = make_smem_desc_hi(16, 1024);
            auto issue_qk = [&](int t, int s) {
                const uint64_t qd = smem_desc(base + S::kQOff + t * kTileBytes, desc_hi);
                const uint64_t kd = smem_desc(base + S::kKOff + s * kTileBytes, desc_hi);
#pragma unroll
                for (int k = 0; k < 4; ++k) umma_ss(tmem_base + kColS + t * 128, qd + 2u * k, kd + 2u * k, idesc_qk, k != 0);
                umma_commit(s_full(t));
            };
            bool ok = mbar_wait(q_full, 0, s_abort, DEV_TIMEOUT_TMA_FULL, 100);
            if (ok) ok = mbar_wait(k_full(0), 0, s_abort, DEV_TIMEOUT_TMA_FULL, 0);
            if (ok) {
                tc_fence_after();
                for (int t = 0; t < NQ; ++t) issue_qk(t, 0);
                umma_commit(k_empty(0));
            }
            int s = 0;
            uint32_t ph = 0;
            for (int j = 0; j < nkb && ok; ++j) {
                const int sn = (s + 1 == kKVStages) ? 0 : s + 1;
                const uint32_t phn = (s + 1 == kKVStages) ? ph ^ 1u : ph;
                for (int t = 0; t < NQ && ok; ++t) {
                    // PV_t(j) = P_t(j) . V_j
                    if (!mbar_wait(p_ready(t), j & 1, s_abort, DEV_TIMEOUT_OTHER, 200 + t)) { ok = false; break; }
                    if (j > 0 && !mbar_wait(pv_empty(t), (j - 1) & 1, s_abort, DEV_TIMEOUT_TMEM_EMPTY, t)) { ok = false; break; }
                    if (t == 0 && !mbar_wait(v_full(s), ph, s_abort, DEV_TIMEOUT_TMA_FULL, 16 + s)) { ok = false; break; }
                    tc_fence_after();
                    const uint64_t vd = smem_desc(base + S::kVOff + s * kTileBytes, desc_hi);
#pragma unroll
                    for (int k = 0; k < 8; ++k)
                        umma_ts(tmem_base + kColPV + t * 64, tmem_base + kColP + t * 64 + 8u * k, vd + 128u * k, idesc_pv, k != 0);
                    umma_commit(pv_full(t));
                    if (t == NQ - 1) umma_commit(v_empty(s));
                    // S_t(j+1) = Q_t . K_{j+1}^T
                    if (j + 1 < nkb) {
                        if (t == 0 && !mbar_wait(k_full(sn), phn, s_abort, DEV_TIMEOUT_TMA_FULL, sn)) { ok = false; break; }
                        tc_fence_after();
                        issue_qk(t, sn);
                        if (t == NQ - 1) umma_commit(k_empty(sn));
                    }
                }
                s = sn;
                ph = phn;
            }
        }
    } else {
        // ------------------------------------------------------------------ softmax groups: one thread per query row
        const int t = (warp - 2) >> 2;
        const int quad = warp & 3;
        const int row_in_tile = quad * 32 + lane;
        const int row = q0 + t * FQ + row_in_tile;
        const uint32_t lane_addr = tmem_base + ((uint32_t)(quad * 32) << 16);
        const uint32_t tS = lane_addr + kColS + t * 128;
        const uint32_t tP = lane_addr + kColP + t * 64;
        const uint32_t tPV = lane_addr + kColPV + t * 64;
        const float sl = a.scale_log2;
        float o[64];
#pragma unroll
        for (int i = 0; i < 64; ++i) o[i] = 0.f;
        float m_run = -INFINITY, l_run = 0.f, c_prev = 0.f;
        bool ok = true;

        auto accumulate_pv = [&](float c) {
            // o = o * c + PV_t
            if constexpr (PV16) {
                uint32_t r[32];
                tmem_ld32_pack16(tPV, r);  // 64 fp16 columns as 32 half2 pairs
                tmem_wait_ld();
#pragma unroll
                for (int i = 0; i < 32; ++i) {
                    const float2 f = __half22float2(*reinterpret_cast<const __half2*>(&r[i]));
                    o[2 * i] = fmaf(o[2 * i], c, f.x);
                    o[2 * i + 1] = fmaf(o[2 * i + 1], c, f.y);
                }
            } else {
#pragma unroll
                for (int half = 0; half < 2; ++half) {
                    uint32_t r[32];
                    tmem_ld32(tPV + 32u * half, r);
                    tmem_wait_ld();
#pragma unroll
                    for (int i = 0; i < 32; ++i) o[32 * half + i] = fmaf(o[32 * half + i], c, __uint_as_float(r[i]));
                }
            }
        };

        for (int j = 0; j < nkb; ++j) {
            if (!mbar_wait(s_full(t), j & 1, s_abort, DEV_TIMEOUT_TMEM_FULL, t)) { ok = false; break; }
            tc_fence_after();
            if (j > 0) {
                // S_t(j) was committed after PV_t(j-1) was issued, so PV_t(j-1) is complete; this wait returns at once.
                if (!mbar_wait(pv_full(t), (j - 1) & 1, s_abort, DEV_TIMEOUT_TMEM_FULL, 8 + t)) { ok = false; break; }
                tc_fence_after();
                accumulate_pv(c_prev);
                tc_fence_before();
                __syncwarp();
                if (lane == 0) mbar_arrive(pv_empty(t));
            }
            const int key0 = j * FK;
            const bool tail = key0 + FK > a.N;
            float sum = 0.f;
            float m_new;
            if (!S16) {
                // ---- pass 1: row maximum
                float mx = -INFINITY;
#pragma unroll 1
                for (int c = 0; c < 4; ++c) {
                    uint32_t r[32];
                    tmem_ld32(tS + 32u * c, r);
                    tmem_wait_ld();
                    if (tail) {
#pragma unroll
                        for (int i = 0; i < 32; ++i)
                            if (key0 + c * 32 + i < a.N) mx = fmaxf(mx, __uint_as_float(r[i]));
                    } else {
#pragma unroll
                        for (int i = 0; i < 32; ++i) mx = fmaxf(mx, __uint_as_float(r[i]));
                    }
                }
                m_new = fmaxf(m_run, mx * sl);
                // ---- pass 2: p = 2^(s*sl - m), row sum in fp32, P as fp16 pairs back to tensor memory
#pragma unroll 1
                for (int c = 0; c < 4; ++c) {
                    uint32_t r[32];
                    uint32_t pk[16];
                    tmem_ld32(tS + 32u * c, r);
                    tmem_wait_ld();
#pragma unroll
                    for (int i = 0; i < 16; ++i) {
                        float p0 = ex2_approx(fmaf(__uint_as_float(r[2 * i]), sl, -m_new));
                        float p1 = ex2_approx(fmaf(__uint_as_float(r[2 * i + 1]), sl, -m_new));
                        if (tail) {
                            if (key0 + c * 32 + 2 * i >= a.N) p0 = 0.f;
                            if (key0 + c * 32 + 2 * i + 1 >= a.N) p1 = 0.f;
                        }
                        sum += p0 + p1;
                        pk[i] = pack_h2(p0, p1);
                    }
                    tmem_st16(tP + 16u * c, pk);
                }
            } else {
                // ---- fp16 S: values arrive as half2 pairs (two neighbouring keys per register)
                __half2 mx2 = __float2half2_rn(-INFINITY);
#pragma unroll 1
                for (int c = 0; c < 2; ++c) {
                    uint32_t r[32];
                    tmem_ld32_pack16(tS + 64u * c, r);
                    tmem_wait_ld();
#pragma unroll
                    for (int i = 0; i < 32; ++i) {
                        __half2 v = *reinterpret_cast<const __half2*>(&r[i]);
                        if (tail) {
                            const int key = key0 + c * 64 + 2 * i;
                            if (key >= a.N) v = __halves2half2(__float2half(-INFINITY), __high2half(v));
                            if (key + 1 >= a.N) v = __halves2half2(__low2half(v), __float2half(-INFINITY));
                        }
                        mx2 = __hmax2(mx2, v);
                    }
                }
                const float mx = fmaxf(__low2float(mx2), __high2float(mx2));
                // keep the running maximum representable in fp16 so the half2 fma below subtracts exactly this value
                m_new = fmaxf(m_run, __half2float(__float2half_rn(mx * sl)));
                const __half2 sl2 = __float2half2_rn(sl);
                const __half2 nm2 = __float2half2_rn(-m_new);
#pragma unroll 1
                for (int c = 0; c < 2; ++c) {
                    uint32_t r[32];
                    tmem_ld32_pack16(tS + 64u * c, r);
                    tmem_wait_ld();
#pragma unroll
                    for (int i = 0; i < 32; ++i) {
                        const __half2 x = __hfma2(*reinterpret_cast<const __half2*>(&r[i]), sl2, nm2);
                        uint32_t p = ex2_approx_h2(*reinterpret_cast<const uint32_t*>(&x));
                        if (tail) {
                            const int key = key0 + c * 64 + 2 * i;
                            if (key >= a.N) p &= 0xFFFF0000u;
                            if (key + 1 >= a.N) p &= 0x0000FFFFu;
                        }
                        const float2 f = __half22float2(*reinterpret_cast<const __half2*>(&p));
                        sum += f.x + f.y;
                        r[i] = p;
                    }
                    tmem_st32(tP + 32u * c, r);
                }
            }
            tmem_wait_st();
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(p_ready(t));
            c_prev = ex2_approx(m_run - m_new);
            l_run = fmaf(l_run, c_prev, sum);
            m_run = m_new;
        }
        if (ok && mbar_wait(pv_full(t), (nkb - 1) & 1, s_abort, DEV_TIMEOUT_TMEM_FULL, 8 + t)) {
            tc_fence_after();
            accumulate_pv(c_prev);
            if (row < a.N) {
                const float inv = 1.f / l_run;
                __half* dst = a.o + (int64_t)b * a.o_sb + (int64_t)row * a.o_sn + (int64_t)h * a.o_sh;
#pragma unroll
                for (int v = 0; v < 8; ++v) {
                    uint4 u;
                    u.x = pack_h2(o[8 * v + 0] * inv, o[8 * v + 1] * inv);
                    u.y = pack_h2(o[8 * v + 2] * inv, o[8 * v + 3] * inv);
                    u.z = pack_h2(o[8 * v + 4] * inv, o[8 * v + 5] * inv);
                    u.w = pack_h2(o[8 * v + 6] * inv, o[8 * v + 7] * inv);
                    *reinterpret_cast<uint4*>(dst + 8 * v) = u;
                }
            }
        }
    }

    tc_fence_before();
    __syncthreads();
    if (warp == 1) {
        __syncwarp();
        tc_fence_after();
        tmem_dealloc<512>(tmem_base);
    }
}

template <int NQ, bool S16, bool PV16>
static int launch_flash_variant(const CUtensorMap& tq, const CUtensorMap& tk, const CUtensorMap& tv, const FlashArgs& a, int B,
                                cudaStream_t stream) {
    static bool configured[64] = {};
    int dev = 0;
    cudaGetDevice(&dev);
    auto kern = flash64_umma_kernel<NQ, S16, PV16>;
    if (dev >= 0 && dev < 64 && !configured[dev]) {
        cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, FlashSmem::kDynamic);
        if (e != cudaSuccess) return fail((int)e, "cudaFuncSetAttribute(flash64_umma_kernel): %s", cudaGetErrorString(e));
        configured[dev] = true;
    }
    dim3 grid((unsigned)((a.N + FQ * NQ - 1) / (FQ * NQ)), (unsigned)(B * a.H), 1);
    kern<<<grid, 64 + 128 * NQ, FlashSmem::kDynamic, stream>>>(tq, tk, tv, a);
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) return fail((int)e, "flash64_umma_kernel launch: %s", cudaGetErrorString(e));
    return FBB_OK;
}

int launch_flash64(const void* q, const void* k, const void* v, void* o, int B, int N, int H, const int64_t* qs,
                   const int64_t* ks, const int64_t* vs, const int64_t* os, float scale, int variant, cudaStream_t stream) {
    CUtensorMap tq, tk, tv;
    const uint64_t dims[4] = {64, (uint64_t)H, (uint64_t)N, (uint64_t)B};
    const uint32_t box[4] = {64, 1, 128, 1};
    const void* ptrs[3] = {q, k, v};
    const int64_t* strides[3] = {qs, ks, vs};
    CUtensorMap* maps[3] = {&tq, &tk, &tv};
    for (int i = 0; i < 3; ++i) {
        // innermost first: d (contiguous), head, token, batch; a size-1 dimension may carry any stride, use a valid one
        int64_t st[4] = {1, strides[i][2], strides[i][1], strides[i][0]};
        if (H == 1 && st[1] == 0) st[1] = 64;
        if (B == 1 && st[3] == 0) st[3] = st[2] * (int64_t)N;
        int rc = make_tmap_f16(maps[i], ptrs[i], 4, dims, st, box);
        if (rc != FBB_OK) return rc;
    }
    FlashArgs a;
    a.o = reinterpret_cast<__half*>(o);
    a.N = N;
    a.H = H;
    a.o_sb = os[0];
    a.o_sn = os[1];
    a.o_sh = os[2];
    a.scale_log2 = scale * 1.4426950408889634f;
    // Small inputs: one 128-query tile per CTA so that more SMs get work (the small-token path).
    const int64_t ctas2 = (int64_t)((N + 2 * FQ - 1) / (2 * FQ)) * B * H;
    const bool two = ctas2 >= num_sms();
#define FBB_FLASH_DISPATCH(S16, PV16)                                                         \
    (two ? launch_flash_variant<2, S16, PV16>(tq, tk, tv, a, B, stream)                       \
         : launch_flash_variant<1, S16, PV16>(tq, tk, tv, a, B, stream))
    switch (variant) {
        case FBB_FLASH_FF: return FBB_FLASH_DISPATCH(false, false);
        case FBB_FLASH_FH: return FBB_FLASH_DISPATCH(false, true);
        default: return FBB_FLASH_DISPATCH(true, true);
    }
#undef FBB_FLASH_DISPATCH
}

}  // namespace fbb
