// C[M, Nout] = epilogue(A[M, K] . W[N, K]^T): fp16 operands, tcgen05 UMMA with the accumulator in tensor memory.
// Replaces F.linear + the separate bias / GELU / SwiGLU / LayerScale-residual passes of fastbb/vit.py:114-143 and the
// gemm_tn_* kernels of fastbb/fastbb_kernels.cu:323-446 (epilogue order bias -> act -> res + gamma*v, :418-427).
//
// K is consumed in 64-element (128-byte) blocks; both operands are K-major, so neither is transposed: nn.Linear's [N, K]
// weight is exactly the B operand. Three forms, picked per shape by launch_linear's cost model:
//   linear_umma_kernel<BN, SWIGLU, false>  persistent, one CTA per SM, 128 x BN output tiles (cta_group::1)
//   linear_umma_kernel<BN, SWIGLU, true>   persistent, a pair of CTAs (cluster of two, cta_group::2) on a 256 x BN tile: each
//                                          CTA stages its 128 rows of A and BN/2 of the W rows, the leader issues UMMAs that
//                                          read both CTAs' shared memory
//   linear_wide_pair_kernel                one pair per work item of 256 rows x w columns (w <= 512 in two accumulators), not
//                                          persistent: for shapes with few tiles, where fixed tiles quantise badly; optionally
//                                          with the LayerNorm of the output rows fused (clusters of up to four pairs)
// No load is multicast: every CTA fetches its own operands with plain TMA loads; only barrier signals cross a pair.
//   warp 0      TMA producer: A box [64 x 128] and the W boxes per stage (128-byte swizzle, zero fill outside)
//   warp 1      UMMA issuer: 4 x tcgen05.mma (K = 16 each) per stage and accumulator
//   warps 2..9  epilogue: tcgen05.ld -> bias -> GELU | SwiGLU -> gamma*v + res -> fp16 -> shared staging tile -> TMA store;
//               before that, the few rows beyond the last full row tile as dot products (remainder_rows_by_gemv)
// In the persistent forms two accumulators (2 x BN columns) let the epilogue of tile i overlap the main loop of tile i+1;
// the plain 256-column form cuts the tiles of a partly filled second wave into 128- or 64-column slices (narrow_tail).
#include "common.cuh"
#include <cstdlib>

#include "internal.h"

namespace fbb {

constexpr int BM = 128;
constexpr int BK = 64;
constexpr int kGemmThreads = 320;
constexpr int kEpiThreads = 256;

// CTA2: the CTA is one half of a pair (cta_group::2) that computes a 256-row tile; it stages its 128 rows of A and only
// BN/2 of the BN rows of W per k-block, which is what brings the operand traffic per FLOP down.
template <int BN, bool CTA2>
struct GemmSmem {
    static constexpr int kABytes = BM * BK * 2;
    static constexpr int kBBytes = (CTA2 ? BN / 2 : BN) * BK * 2;
    static constexpr int kStages = (kABytes + kBBytes) == 49152 ? 4 : ((kABytes + kBBytes) == 32768 ? 6 : 8);
    static constexpr int kStageBytes = kABytes + kBBytes;
    static constexpr int kParamFloats = 2 * 2 * BN;  // double-buffered bias + gamma
    static constexpr int kStoreBytes = 8 * 32 * 32 * 2;  // one [32 rows x 32 columns] fp16 staging tile per epilogue warp
    static constexpr int kStoreOffset = kStages * kStageBytes + kParamFloats * 4;
    static constexpr int kBarOffset = kStoreOffset + kStoreBytes;
    static constexpr int kNumBars = 2 * kStages + 4;
    static constexpr int kBytes = kBarOffset + kNumBars * 8 + 16;
    static constexpr int kDynamic = kBytes + 1024;  // slack to align the tile base to 1024 bytes
};

struct GemmArgs {
    __half* C;
    const __half* bias;
    const __half* res;
    const __half* gamma;
    int M, N, K;       // N = rows of W
    int n_out;         // output columns (N, or N/2 for SwiGLU)
    int64_t ldc, ldr;
    int act;           // 0 none, 1 gelu
    int acc_f16;       // 1: fp16 accumulator
    int tiles_m, tiles_n;
    // rows [gemv_row0, gemv_row0 + gemv_rows) have no tile: the epilogue warps compute them (see remainder_rows_by_gemv)
    const __half* A;
    const __half* W;
    int64_t lda, ldw;
    int gemv_row0, gemv_rows;
    // The last, partly filled wave of tiles may be cut into narrower items so that every CTA gets one (see narrow_tail):
    // items [0, wide_tiles) are whole tiles, the next narrow_tiles items are narrow_w-column slices of the tiles after them.
    int wide_tiles, narrow_w, narrow_tiles;
};

// The few rows beyond the last full row tile (every ViT token count is a multiple of the tile height plus the cls token:
// 257, 4097, 6145, 16385; batched, a handful of rows) do not get a tile of their own, which would cost a whole tile's
// main loop for one row (M = 6145 with 256-row pair tiles: 300 tiles on 74 pairs = 5 waves, 288 = 4 waves without them).
// The epilogue warps, idle until the first accumulator completes, compute them as dot products on the CUDA cores: one
// output element per warp at a time, fp32 accumulation, the same epilogue (bias -> GELU | SwiGLU -> res + gamma * v).
constexpr int kGemvMaxRows = 8;

__device__ __forceinline__ float warp_dot_f16(const __half* a, const __half* w, int nvec, int lane) {
    const uint4* ap = reinterpret_cast<const uint4*>(a);
    const uint4* wp = reinterpret_cast<const uint4*>(w);
    float acc = 0.f;
    for (int v = lane; v < nvec; v += 32) {
        const uint4 av = ap[v];  // A was written by the previous kernel: ordinary loads
        const uint4 wv = __ldg(wp + v);
        const __half2* ah = reinterpret_cast<const __half2*>(&av);
        const __half2* wh = reinterpret_cast<const __half2*>(&wv);
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const float2 af = __half22float2(ah[j]), wf = __half22float2(wh[j]);
            acc = fmaf(af.x, wf.x, acc);
            acc = fmaf(af.y, wf.y, acc);
        }
    }
#pragma unroll
    for (int sft = 16; sft > 0; sft >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, sft);
    return acc;
}

// warp_global / total_warps: this warp's index among all epilogue warps of the grid. swiglu: W holds [x1 rows | x2 rows].
__device__ __forceinline__ void remainder_rows_by_gemv(const GemmArgs& g, bool swiglu, int warp_global, int total_warps, int lane) {
    const int nvec = g.K >> 3;
    for (int o = warp_global; o < g.gemv_rows * g.n_out; o += total_warps) {
        const int mi = o / g.n_out, n = o - mi * g.n_out;
        const int64_t m = g.gemv_row0 + mi;
        const __half* a = g.A + m * g.lda;
        float v = warp_dot_f16(a, g.W + (int64_t)n * g.ldw, nvec, lane) + (g.bias != nullptr ? __half2float(g.bias[n]) : 0.f);
        if (swiglu) {
            const int n2 = g.N / 2 + n;
            const float x2 = warp_dot_f16(a, g.W + (int64_t)n2 * g.ldw, nvec, lane) + (g.bias != nullptr ? __half2float(g.bias[n2]) : 0.f);
            v = silu(v) * x2;
        } else if (g.act == 1) {
            v = gelu_erf(v);
        }
        if (lane == 0) {
            if (g.res != nullptr) v = fmaf(g.gamma != nullptr ? __half2float(g.gamma[n]) : 1.f, v, __half2float(g.res[m * g.ldr + n]));
            g.C[m * g.ldc + n] = __float2half_rn(v);
        }
    }
}

template <int BN, bool SWIGLU, bool CTA2, bool SLICES = false>
__global__ void __launch_bounds__(kGemmThreads, 1)
linear_umma_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_w,
                   const __grid_constant__ CUtensorMap tmap_wn, const __grid_constant__ CUtensorMap tmap_c, const GemmArgs g) {
    using S = GemmSmem<BN, CTA2>;
    // pair geometry: rank 0 (the leader) issues the UMMAs; work items are 256-row tiles shared by the pair
    const uint32_t rank = CTA2 ? cluster_ctarank() : 0u;
    const int worker = CTA2 ? (int)(blockIdx.x >> 1) : (int)blockIdx.x;
    const int num_workers = CTA2 ? (int)(gridDim.x >> 1) : (int)gridDim.x;
    constexpr int kTileRows = CTA2 ? 2 * BM : BM;
    constexpr int kStages = S::kStages;
    constexpr int kOutCols = SWIGLU ? BN / 2 : BN;  // output columns per tile
    extern __shared__ uint8_t smem_raw[];
    const uint32_t raw = smem_u32(smem_raw);
    const uint32_t base = (raw + 1023u) & ~1023u;
    uint8_t* gen = smem_raw + (base - raw);
    float* s_params = reinterpret_cast<float*>(gen + kStages * S::kStageBytes);
    const uint32_t bar0 = base + S::kBarOffset;
    auto full_bar = [&](int s) { return bar0 + 8u * s; };
    auto empty_bar = [&](int s) { return bar0 + 8u * (kStages + s); };
    auto tfull_bar = [&](int a) { return bar0 + 8u * (2 * kStages + a); };
    auto tempty_bar = [&](int a) { return bar0 + 8u * (2 * kStages + 2 + a); };
    volatile uint32_t* s_tmem = reinterpret_cast<volatile uint32_t*>(gen + S::kBarOffset + S::kNumBars * 8);
    volatile int* s_abort = reinterpret_cast<volatile int*>(gen + S::kBarOffset + S::kNumBars * 8 + 4);

    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;
    const int num_kb = (g.K + BK - 1) / BK;
    // Work items: whole tiles, then (plain single-CTA 256-column form only) the slices of the last wave's tiles. Every role
    // walks the same list: m0 = first row (of this CTA), n0 = first output column, w = W rows (= columns) of the item.
    static_assert(!SLICES || (!SWIGLU && !CTA2 && BN == 256), "slices: plain single-CTA 256-column form only");
    constexpr bool kNarrowOk = SLICES;  // without slices every width below is a compile-time constant
    const int num_items = g.wide_tiles + (kNarrowOk ? g.narrow_tiles : 0);
    auto item_at = [&](int idx, int& m0, int& n0, int& w) {
        int tile = idx, sub = 0;
        w = BN;
        if (kNarrowOk && idx >= g.wide_tiles) {
            const int per = BN / g.narrow_w, j = idx - g.wide_tiles;
            tile = g.wide_tiles + j / per;
            sub = j - (j / per) * per;
            w = g.narrow_w;
        }
        m0 = (tile / g.tiles_n) * kTileRows + (int)rank * BM;
        n0 = (tile % g.tiles_n) * kOutCols + sub * g.narrow_w;
    };

    if (threadIdx.x == 0) {
        for (int s = 0; s < kStages; ++s) {
            mbar_init(full_bar(s), 1);
            mbar_init(empty_bar(s), 1);
        }
        for (int a = 0; a < 2; ++a) {
            mbar_init(tfull_bar(a), 1);
            mbar_init(tempty_bar(a), (CTA2 ? 2 : 1) * kEpiThreads / 32);  // the leader's barrier also counts the peer's warps
        }
        *s_abort = 0;
        fence_barrier_init();
        tma_prefetch_desc(&tmap_a);
        tma_prefetch_desc(&tmap_w);
        tma_prefetch_desc(&tmap_c);
    }
    if (warp == 1) {
        __syncwarp();
        if constexpr (CTA2) {
            tmem_alloc_pair<2 * BN>(smem_u32(const_cast<uint32_t*>(s_tmem)));
            tmem_relinquish_pair();
        } else {
            tmem_alloc<2 * BN>(smem_u32(const_cast<uint32_t*>(s_tmem)));
            tmem_relinquish();
        }
    }
    tc_fence_before();
    __syncthreads();
    if constexpr (CTA2) cluster_sync_all();  // both CTAs' barriers exist before either signals the other
    tc_fence_after();
    const uint32_t tmem_base = *s_tmem;
    grid_dependency_wait();  // the set-up above may overlap the previous kernel's tail; its outputs are visible from here
    grid_launch_dependents();

    if (warp == 0) {
        // ------------------------------------------------------------------ TMA producer
        if (lane == 0) {
            int s = 0;
            uint32_t ph = 0;
            bool ok = true;
            for (int item = worker; item < num_items && ok; item += num_workers) {
                int m0, n0, w;
                item_at(item, m0, n0, w);
                const int nt = n0 / kOutCols;
                for (int kb = 0; kb < num_kb; ++kb) {
                    if (!mbar_wait(empty_bar(s), ph ^ 1u, s_abort, DEV_TIMEOUT_SMEM_EMPTY, s)) { ok = false; break; }
                    const uint32_t sa = base + s * S::kStageBytes;
                    const uint32_t sb = sa + S::kABytes;
                    if constexpr (CTA2) {
                        // the leader's barrier collects the bytes of both CTAs; each CTA loads its own A rows and its half of
                        // the W rows (SwiGLU: the leader the x1 rows, the peer the matching x2 rows)
                        if (rank == 0) mbar_arrive_expect_tx(full_bar(s), 2 * S::kStageBytes);
                        tma_load_2d_pair(sa, &tmap_a, full_bar(s), kb * BK, m0);
                        const int wrow = SWIGLU ? (rank == 0 ? nt * (BN / 2) : g.N / 2 + nt * (BN / 2)) : nt * BN + (int)rank * (BN / 2);
                        tma_load_2d_pair(sb, &tmap_w, full_bar(s), kb * BK, wrow);
                    } else if (kNarrowOk && w != BN) {
                        // a slice: its W rows in 64-row boxes, laid out like the first rows of a whole tile's box
                        mbar_arrive_expect_tx(full_bar(s), (uint32_t)(S::kABytes + w * BK * 2));
                        tma_load_2d(sa, &tmap_a, full_bar(s), kb * BK, m0);
                        for (int r = 0; r < w; r += 64) tma_load_2d(sb + (uint32_t)(r * BK * 2), &tmap_wn, full_bar(s), kb * BK, n0 + r);
                    } else {
                        mbar_arrive_expect_tx(full_bar(s), S::kStageBytes);
                        tma_load_2d(sa, &tmap_a, full_bar(s), kb * BK, m0);
                        if (SWIGLU) {
                            // x1 rows [nt*BN/2, +BN/2) and the matching x2 rows, offset by N/2
                            tma_load_2d(sb, &tmap_w, full_bar(s), kb * BK, nt * (BN / 2));
                            tma_load_2d(sb + S::kBBytes / 2, &tmap_w, full_bar(s), kb * BK, g.N / 2 + nt * (BN / 2));
                        } else {
                            tma_load_2d(sb, &tmap_w, full_bar(s), kb * BK, nt * BN);
                        }
                    }
                    if (++s == kStages) { s = 0; ph ^= 1u; }
                }
            }
            if (!ok) __nanosleep(20000);  // let copies already in flight land before the CTA leaves
        }
    } else if (warp == 1 && rank == 0) {
        // ------------------------------------------------------------------ UMMA issuer (the leader CTA of a pair only)
        // The whole warp runs this loop and one elected lane issues each instruction, so that descriptors and
        // addresses are warp-uniform values (uniform registers) rather than per-thread arithmetic in a divergent branch.
        const uint32_t idesc_tile = make_idesc_f16(kTileRows, BN, !g.acc_f16, false, false);
        const uint32_t idesc_slice = make_idesc_f16(kTileRows, (kNarrowOk && g.narrow_w > 0) ? g.narrow_w : BN, !g.acc_f16, false, false);
        constexpr uint64_t desc_hi = make_smem_desc_hi(16, 1024);
        const uint64_t adesc0 = smem_desc(base, desc_hi);
        auto all_ok = [&](bool mine) { return __all_sync(0xffffffffu, mine) != 0; };
        int s = 0;
        uint32_t ph = 0;
        int acc = 0;
        uint32_t acc_ph = 0;
        bool ok = true;
        for (int item = worker; item < num_items && ok; item += num_workers) {
            const uint32_t idesc = (kNarrowOk && item >= g.wide_tiles) ? idesc_slice : idesc_tile;
            if (!all_ok(mbar_wait(tempty_bar(acc), acc_ph ^ 1u, s_abort, DEV_TIMEOUT_TMEM_EMPTY, acc))) break;
            tc_fence_after();
            const uint32_t d_tmem = tmem_base + (uint32_t)(acc * BN);
            for (int kb = 0; kb < num_kb; ++kb) {
                if (!all_ok(mbar_wait(full_bar(s), ph, s_abort, DEV_TIMEOUT_TMA_FULL, s))) { ok = false; break; }
                tc_fence_after();
                const uint64_t adesc = adesc0 + (uint64_t)(s * (S::kStageBytes >> 4));
                const uint64_t bdesc = adesc + (uint64_t)(S::kABytes >> 4);
                if constexpr (CTA2) {
                    umma_ss_pair_warp(d_tmem, adesc, bdesc, idesc, kb != 0 ? 1u : 0u);
#pragma unroll
                    for (int k = 1; k < BK / 16; ++k) umma_ss_pair_warp(d_tmem, adesc + 2u * k, bdesc + 2u * k, idesc, 1u);
                    umma_commit_pair_warp(empty_bar(s));  // frees the stage in both CTAs
                } else {
                    umma_ss_warp(d_tmem, adesc, bdesc, idesc, kb != 0 ? 1u : 0u);
#pragma unroll
                    for (int k = 1; k < BK / 16; ++k) umma_ss_warp(d_tmem, adesc + 2u * k, bdesc + 2u * k, idesc, 1u);
                    umma_commit_warp(empty_bar(s));  // stage reusable once these UMMAs have read it
                }
                if (++s == kStages) { s = 0; ph ^= 1u; }
            }
            if (!ok) break;
            if constexpr (CTA2) umma_commit_pair_warp(tfull_bar(acc));  // both CTAs' accumulators complete
            else umma_commit_warp(tfull_bar(acc));
            if (++acc == 2) { acc = 0; acc_ph ^= 1u; }
        }
    } else if (warp >= 2) {
        // ------------------------------------------------------------------ epilogue (8 warps)
        const int ew = warp - 2;
        const int quad = warp & 3;        // tensor-memory lane quadrant this warp may read
        const int chalf = ew >> 2;        // which half of the output columns
        const int et = threadIdx.x - 64;  // 0..255
        uint8_t* stage_gen = gen + S::kStoreOffset + ew * 2048;
        const uint32_t stage_addr = base + S::kStoreOffset + ew * 2048;
        if (g.gemv_rows > 0) remainder_rows_by_gemv(g, SWIGLU, (int)blockIdx.x * 8 + ew, (int)gridDim.x * 8, lane);
        int acc = 0;
        uint32_t acc_ph = 0;
        for (int item = worker; item < num_items; item += num_workers) {
            int m0, n0, w;  // n0: first output column of the item
            item_at(item, m0, n0, w);
            const int half_cols = SWIGLU ? kOutCols / 2 : w / 2;  // output columns per half of the epilogue warps
            const int chunks = half_cols / 32;
            // stage bias (W-row indexed) and gamma (output-column indexed) for this item
            float* s_bias = s_params + acc * 2 * BN;
            float* s_gamma = s_bias + BN;
            for (int i = et; i < w; i += kEpiThreads) {
                int wrow;
                if (SWIGLU) wrow = i < BN / 2 ? n0 + i : g.N / 2 + n0 + (i - BN / 2);
                else wrow = n0 + i;
                const bool in = SWIGLU ? (n0 + (i % (BN / 2)) < g.n_out) : (wrow < g.N);
                s_bias[i] = (g.bias != nullptr && in) ? __half2float(g.bias[wrow]) : 0.f;
                if (!SWIGLU) s_gamma[i] = (g.gamma != nullptr && in) ? __half2float(g.gamma[wrow]) : 1.f;
            }
            named_bar_sync(1, kEpiThreads);
            const int row = m0 + quad * 32 + lane;
            const bool row_ok = row < g.M;
            const __half* r_row = g.res != nullptr ? g.res + (int64_t)row * g.ldr : nullptr;
            // The residual of this thread's row for all of its columns goes into registers BEFORE the wait for the accumulator:
            // the loads (one 64-byte piece per thread and chunk, L2 latency each) then run under the tile's main loop instead
            // of sitting, chunk after chunk, in the epilogue's critical path (measured: 4.7 us of an 18 us proj launch).
            constexpr int kChunks = kOutCols / 2 / 32;
            uint4 rr[SWIGLU ? 1 : kChunks][4];
            if constexpr (!SWIGLU) {
#pragma unroll
                for (int ci = 0; ci < kChunks; ++ci) {
                    if (ci >= chunks) break;
#pragma unroll
                    for (int q = 0; q < 4; ++q) {
                        const int col = n0 + chalf * half_cols + ci * 32 + q * 8;
                        rr[ci][q] = (r_row != nullptr && row_ok && col < g.n_out) ? *reinterpret_cast<const uint4*>(r_row + col) : make_uint4(0u, 0u, 0u, 0u);
                    }
                }
            }
            if (!mbar_wait(tfull_bar(acc), acc_ph, s_abort, DEV_TIMEOUT_TMEM_FULL, acc)) break;
            tc_fence_after();
            const uint32_t t_row = tmem_base + ((uint32_t)(quad * 32) << 16) + (uint32_t)(acc * BN);
#pragma unroll
            for (int ci = 0; ci < kChunks; ++ci) {
                if (ci >= chunks) break;
                const int c0 = chalf * half_cols + ci * 32;
                uint32_t r[32];
                float v[32];
                tmem_ld32(t_row + (uint32_t)c0, r);
                tmem_wait_ld();
                if (g.acc_f16) {
#pragma unroll
                    for (int j = 0; j < 32; ++j) v[j] = __half2float(__ushort_as_half((unsigned short)(r[j] & 0xFFFFu)));
                } else {
#pragma unroll
                    for (int j = 0; j < 32; ++j) v[j] = __uint_as_float(r[j]);
                }
                if (SWIGLU) {
                    uint32_t r2[32];
                    tmem_ld32(t_row + (uint32_t)(BN / 2 + c0), r2);
                    tmem_wait_ld();
#pragma unroll
                    for (int j = 0; j < 32; ++j) {
                        const float x2 = (g.acc_f16 ? __half2float(__ushort_as_half((unsigned short)(r2[j] & 0xFFFFu)))
                                                    : __uint_as_float(r2[j])) + s_bias[BN / 2 + c0 + j];
                        v[j] = silu(v[j] + s_bias[c0 + j]) * x2;
                    }
                } else {
#pragma unroll
                    for (int j = 0; j < 32; ++j) v[j] += s_bias[c0 + j];
                    if (g.act == 1) {
#pragma unroll
                        for (int j = 0; j < 32; j += 2) {
                            const float2 y = gelu_erf2(make_float2(v[j], v[j + 1]));
                            v[j] = y.x;
                            v[j + 1] = y.y;
                        }
                    }
                }
                // residual + LayerScale (columns beyond n_out and rows beyond M hold zeros and are clipped by the store)
                if constexpr (!SWIGLU) {
                    if (r_row != nullptr) {
#pragma unroll
                        for (int q = 0; q < 4; ++q) {
                            const __half2* rh = reinterpret_cast<const __half2*>(&rr[ci][q]);
#pragma unroll
                            for (int j = 0; j < 4; ++j) {
                                const float2 rf = __half22float2(rh[j]);
                                v[q * 8 + 2 * j] = fmaf(s_gamma[c0 + q * 8 + 2 * j], v[q * 8 + 2 * j], rf.x);
                                v[q * 8 + 2 * j + 1] = fmaf(s_gamma[c0 + q * 8 + 2 * j + 1], v[q * 8 + 2 * j + 1], rf.y);
                            }
                        }
                    }
                }
                // fp16 -> this warp's staging tile (64-byte rows, 16-byte chunks XOR-swizzled as the tensor map's 64-byte
                // mode expects: conflict-free) -> one TMA store of [32 rows x 32 columns]; rows >= M and columns >= n_out
                // are clipped by the hardware. The previous store must have finished reading the tile first.
                if (lane == 0) bulk_wait_read_all();
                __syncwarp();
#pragma unroll
                for (int q = 0; q < 4; ++q) {
                    uint4 o;
                    o.x = pack_h2(v[q * 8 + 0], v[q * 8 + 1]);
                    o.y = pack_h2(v[q * 8 + 2], v[q * 8 + 3]);
                    o.z = pack_h2(v[q * 8 + 4], v[q * 8 + 5]);
                    o.w = pack_h2(v[q * 8 + 6], v[q * 8 + 7]);
                    *reinterpret_cast<uint4*>(stage_gen + lane * 64 + ((q ^ ((lane >> 1) & 3)) << 4)) = o;
                }
                fence_proxy_async_smem();
                __syncwarp();
                if (lane == 0 && n0 + c0 < g.n_out && m0 + quad * 32 < g.M) {
                    tma_store_2d(&tmap_c, stage_addr, n0 + c0, m0 + quad * 32);
                    bulk_commit();
                }
            }
            tc_fence_before();
            __syncwarp();
            if (lane == 0) {
                if constexpr (CTA2) mbar_arrive_remote(tempty_bar(acc), 0u);  // the leader issues the next tile for both CTAs
                else mbar_arrive(tempty_bar(acc));
            }
            if (++acc == 2) { acc = 0; acc_ph ^= 1u; }
        }
        if (lane == 0) bulk_wait_all();  // this warp's output stores are complete before the CTA gives up its shared memory
    }

    tc_fence_before();
    __syncthreads();
    if constexpr (CTA2) cluster_sync_all();  // the peer may still be signalling this CTA's barriers / reading its operands
    if (warp == 1) {
        __syncwarp();
        tc_fence_after();
        if constexpr (CTA2) tmem_dealloc_pair<2 * BN>(tmem_base);
        else tmem_dealloc<2 * BN>(tmem_base);
    }
}

// ---------------------------------------------------------------------------------------------------------------------
// Wide pair form: one CTA pair per work item, an item = 256 rows x `w` output columns (w a multiple of 32, up to 512),
// held in two tensor-memory accumulators of wa and wb columns (wa + wb = w, each a multiple of 32 and at most 256) that
// share the A operand. Not persistent: the grid is one cluster per item. It exists for shapes whose tile count is small
// against the SM count, where fixed 256-column tiles quantise badly: M = 6145, N = 1024 is 25 x 4 pair tiles on 74 pairs
// (two waves, the second a third full); as 24 x 3 items of 352 columns it is one wave, and per k-block a CTA stages
// 16 KB of A and w x 64 bytes of W for w / 256 x 512 tensor clocks (55 bytes per clock at w = 352, against 96 for the
// one-CTA 256-column tile and 64 for the pair tile).
// The few rows beyond the last full 256-row tile are left to the epilogue warps (remainder_rows_by_gemv), as in the
// persistent forms.
constexpr int kWideMaxCols = 512;

struct WideArgs {
    const __half* A;
    const __half* W;
    __half* C;
    const __half* bias;
    const __half* res;
    const __half* gamma;
    int M, N, K;
    int64_t lda, ldw, ldc, ldr;
    int act, acc_f16;
    int w, wa, wb;             // item width and its two accumulators
    int chunks;                // items per 256-row tile: ceil(N / w)
    int gemv_row0, gemv_rows;  // rows [gemv_row0, gemv_row0 + gemv_rows) are left to the epilogue warps
    int stages, stage_bytes;   // operand ring: stage = A tile (16 KB) | this CTA's wa/2 rows of W | its wb/2 rows of W
    // Fused LayerNorm of the output rows (ln_y != null): y[m, :] = LN(C[m, :]) * ln_w + ln_b, fp16. The cluster then holds
    // all `chunks` items of a 256-row tile (2 * chunks CTAs), which exchange per-row statistics through shared memory.
    __half* ln_y;
    const __half* ln_w;
    const __half* ln_b;
    float ln_eps;
    int64_t ldy;
    unsigned* ln_counter;      // zero between launches: counts finished remainder-row elements (see the GEMV part)
};

struct WideSmem {
    // bias + gamma of the item's columns, LayerNorm weight + bias of them (fp32), then per-row statistics: the two
    // epilogue warp groups' partial (mean, M2), the CTA's partial, and the final (mean, rstd), 128 rows each
    static constexpr int kParamBytes = 4 * kWideMaxCols * 4 + 4 * 128 * 8;
    static constexpr int kStoreBytes = 8 * 32 * 32 * 2;       // one [32 x 32] fp16 staging tile per epilogue warp
    static constexpr int kMaxStages = 8;
    static constexpr int kNumBars = 2 * kMaxStages + 1;
    static constexpr int kTailBytes = kParamBytes + kStoreBytes + kNumBars * 8 + 16;
    static constexpr int kMaxDynamic = 227 * 1024;
    static int stages_for(int stage_bytes) {
        const int n = (kMaxDynamic - 1024 - kTailBytes) / stage_bytes;
        return n > kMaxStages ? kMaxStages : n;
    }
    static int dynamic_bytes(int stages, int stage_bytes) { return 1024 + stages * stage_bytes + kTailBytes; }
};

__global__ void __launch_bounds__(kGemmThreads, 1)
linear_wide_pair_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_wa,
                        const __grid_constant__ CUtensorMap tmap_wb, const __grid_constant__ CUtensorMap tmap_c,
                        const __grid_constant__ CUtensorMap tmap_y, const WideArgs g) {
    using S = WideSmem;
    const uint32_t crank = cluster_ctarank();  // a pair is two CTAs of adjacent ranks; with LayerNorm the cluster holds `chunks` pairs
    const uint32_t rank = crank & 1u;
    const bool fuse_ln = g.ln_y != nullptr;
    const int item = (int)(blockIdx.x >> 1);
    const int mt = item / g.chunks;
    const int n0 = (item - mt * g.chunks) * g.w;
    const int m0 = mt * 2 * BM + (int)rank * BM;
    extern __shared__ uint8_t smem_raw[];
    const uint32_t raw = smem_u32(smem_raw);
    const uint32_t base = (raw + 1023u) & ~1023u;
    uint8_t* gen = smem_raw + (base - raw);
    const int ring = g.stages * g.stage_bytes;
    float* s_bias = reinterpret_cast<float*>(gen + ring);
    float* s_gamma = s_bias + kWideMaxCols;
    float* s_lnw = s_gamma + kWideMaxCols;
    float* s_lnb = s_lnw + kWideMaxCols;
    float2* s_part_wg = reinterpret_cast<float2*>(s_lnb + kWideMaxCols);  // [2][128]: (mean, M2) of each warp group's columns
    float2* s_part_cta = s_part_wg + 256;                                 // [128]: (mean, M2) of this CTA's columns
    float2* s_row_stat = s_part_cta + 128;                                // [128]: (mean, rstd) of the whole row
    const int store_off = ring + S::kParamBytes;
    const uint32_t bar0 = base + store_off + S::kStoreBytes;
    auto full_bar = [&](int s) { return bar0 + 8u * s; };
    auto empty_bar = [&](int s) { return bar0 + 8u * (S::kMaxStages + s); };
    const uint32_t tfull_bar = bar0 + 8u * (2 * S::kMaxStages);
    volatile uint32_t* s_tmem = reinterpret_cast<volatile uint32_t*>(gen + store_off + S::kStoreBytes + S::kNumBars * 8);
    volatile int* s_abort = reinterpret_cast<volatile int*>(gen + store_off + S::kStoreBytes + S::kNumBars * 8 + 4);

    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;
    const int num_kb = (g.K + BK - 1) / BK;

    if (threadIdx.x == 0) {
        for (int s = 0; s < g.stages; ++s) {
            mbar_init(full_bar(s), 1);
            mbar_init(empty_bar(s), 1);
        }
        mbar_init(tfull_bar, 1);
        *s_abort = 0;
        fence_barrier_init();
        tma_prefetch_desc(&tmap_a);
        tma_prefetch_desc(&tmap_wa);
        tma_prefetch_desc(&tmap_wb);
        tma_prefetch_desc(&tmap_c);
        if (fuse_ln) tma_prefetch_desc(&tmap_y);
    }
    if (warp == 1) {
        __syncwarp();
        tmem_alloc_pair<512>(smem_u32(const_cast<uint32_t*>(s_tmem)));
        tmem_relinquish_pair();
    }
    tc_fence_before();
    __syncthreads();
    cluster_sync_all();  // both CTAs' barriers exist before either signals the other
    tc_fence_after();
    const uint32_t tmem_base = *s_tmem;
    grid_dependency_wait();
    grid_launch_dependents();

    if (warp == 0) {
        // ------------------------------------------------------------------ TMA producer (one lane in each CTA)
        if (lane == 0) {
            int s = 0;
            uint32_t ph = 0;
            bool ok = true;
            const int wrow_a = n0 + (int)rank * (g.wa / 2);
            const int wrow_b = n0 + g.wa + (int)rank * (g.wb / 2);
            for (int kb = 0; kb < num_kb; ++kb) {
                if (!mbar_wait(empty_bar(s), ph ^ 1u, s_abort, DEV_TIMEOUT_SMEM_EMPTY, s)) { ok = false; break; }
                const uint32_t sa = base + s * g.stage_bytes;
                if (rank == 0) mbar_arrive_expect_tx(full_bar(s), 2 * g.stage_bytes);  // the leader's barrier counts both CTAs' bytes
                tma_load_2d_pair(sa, &tmap_a, full_bar(s), kb * BK, m0);
                tma_load_2d_pair(sa + BM * BK * 2, &tmap_wa, full_bar(s), kb * BK, wrow_a);
                if (g.wb > 0) tma_load_2d_pair(sa + BM * BK * 2 + g.wa * BK, &tmap_wb, full_bar(s), kb * BK, wrow_b);
                if (++s == g.stages) { s = 0; ph ^= 1u; }
            }
            if (!ok) __nanosleep(20000);  // let copies already in flight land before the CTA leaves
        }
    } else if (warp == 1 && rank == 0) {
        // ------------------------------------------------------------------ UMMA issuer (leader CTA, warp-uniform)
        const uint32_t idesc_a = make_idesc_f16(2 * BM, g.wa, !g.acc_f16, false, false);
        const uint32_t idesc_b = make_idesc_f16(2 * BM, g.wb > 0 ? g.wb : 32, !g.acc_f16, false, false);
        constexpr uint64_t desc_hi = make_smem_desc_hi(16, 1024);
        const uint64_t adesc0 = smem_desc(base, desc_hi);
        const uint32_t d_a = tmem_base, d_b = tmem_base + 256u;
        auto all_ok = [&](bool mine) { return __all_sync(0xffffffffu, mine) != 0; };
        int s = 0;
        uint32_t ph = 0;
        bool ok = true;
        for (int kb = 0; kb < num_kb; ++kb) {
            if (!all_ok(mbar_wait(full_bar(s), ph, s_abort, DEV_TIMEOUT_TMA_FULL, s))) { ok = false; break; }
            tc_fence_after();
            const uint64_t adesc = adesc0 + (uint64_t)((s * g.stage_bytes) >> 4);
            const uint64_t bdesc_a = adesc + (uint64_t)((BM * BK * 2) >> 4);
            const uint64_t bdesc_b = bdesc_a + (uint64_t)((g.wa * BK) >> 4);
#pragma unroll
            for (int k = 0; k < BK / 16; ++k) {
                const uint32_t accumulate = (kb != 0 || k != 0) ? 1u : 0u;
                umma_ss_pair_warp(d_a, adesc + 2u * k, bdesc_a + 2u * k, idesc_a, accumulate);
                if (g.wb > 0) umma_ss_pair_warp(d_b, adesc + 2u * k, bdesc_b + 2u * k, idesc_b, accumulate);
            }
            umma_commit_pair_mask_warp(empty_bar(s), 3u << crank);  // frees the stage in both CTAs (the leader's rank is even)
            if (++s == g.stages) { s = 0; ph ^= 1u; }
        }
        if (ok) umma_commit_pair_mask_warp(tfull_bar, 3u << crank);  // both CTAs' accumulators complete
    } else if (warp >= 2) {
        // ------------------------------------------------------------------ epilogue warps
        const int ew = warp - 2;
        const int quad = warp & 3;  // tensor-memory lane quadrant this warp may read
        const int et = threadIdx.x - 64;
        // (1) while the main loop runs: the rows that have no tile (remainder_rows_by_gemv)
        if (g.gemv_rows > 0) {
            GemmArgs r;
            r.C = g.C; r.bias = g.bias; r.res = g.res; r.gamma = g.gamma;
            r.M = g.M; r.N = g.N; r.K = g.K; r.n_out = g.N;
            r.ldc = g.ldc; r.ldr = g.ldr; r.act = g.act; r.acc_f16 = g.acc_f16; r.tiles_m = r.tiles_n = 0;
            r.A = g.A; r.W = g.W; r.lda = g.lda; r.ldw = g.ldw; r.gemv_row0 = g.gemv_row0; r.gemv_rows = g.gemv_rows;
            const int gw = (int)blockIdx.x * 8 + ew, total_warps = (int)gridDim.x * 8, total = g.gemv_rows * g.N;
            remainder_rows_by_gemv(r, false, gw, total_warps, lane);
            if (fuse_ln && gw < total) {
                // LayerNorm of those rows: their elements are spread over the warps of the whole grid, so each warp adds the
                // number it has written to a counter, and the warp whose addition completes the count normalises the rows
                // (nobody waits for anybody). It leaves the counter at zero for the next launch on the stream.
                const int mine = (total - gw + total_warps - 1) / total_warps;
                int last = 0;
                if (lane == 0) {
                    __threadfence();
                    last = atomicAdd(g.ln_counter, (unsigned)mine) + (unsigned)mine == (unsigned)total;
                }
                last = __shfl_sync(0xffffffffu, last, 0);
                if (last) {
                    __threadfence();
                    const int nvec = g.N >> 3;
                    for (int mi = 0; mi < g.gemv_rows; ++mi) {
                        const int64_t m = g.gemv_row0 + mi;
                        const uint4* xr = reinterpret_cast<const uint4*>(g.C + m * g.ldc);
                        float sum = 0.f;
                        for (int v = lane; v < nvec; v += 32) {
                            const uint4 xv = __ldcg(xr + v);
                            const __half2* h = reinterpret_cast<const __half2*>(&xv);
#pragma unroll
                            for (int j = 0; j < 4; ++j) {
                                const float2 f = __half22float2(h[j]);
                                sum += f.x + f.y;
                            }
                        }
#pragma unroll
                        for (int sft = 16; sft > 0; sft >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, sft);
                        const float mean = sum / (float)g.N;
                        float q = 0.f;
                        for (int v = lane; v < nvec; v += 32) {
                            const uint4 xv = __ldcg(xr + v);
                            const __half2* h = reinterpret_cast<const __half2*>(&xv);
#pragma unroll
                            for (int j = 0; j < 4; ++j) {
                                const float2 f = __half22float2(h[j]);
                                q += (f.x - mean) * (f.x - mean) + (f.y - mean) * (f.y - mean);
                            }
                        }
#pragma unroll
                        for (int sft = 16; sft > 0; sft >>= 1) q += __shfl_xor_sync(0xffffffffu, q, sft);
                        const float rstd = rsqrtf(q / (float)g.N + g.ln_eps);
                        uint4* yr = reinterpret_cast<uint4*>(g.ln_y + m * g.ldy);
                        for (int v = lane; v < nvec; v += 32) {
                            const uint4 xv = __ldcg(xr + v);
                            const __half2* h = reinterpret_cast<const __half2*>(&xv);
                            uint4 out;
                            uint32_t* o = reinterpret_cast<uint32_t*>(&out);
#pragma unroll
                            for (int j = 0; j < 4; ++j) {
                                const float2 f = __half22float2(h[j]);
                                const int c = v * 8 + 2 * j;
                                const float w0 = g.ln_w != nullptr ? __half2float(g.ln_w[c]) : 1.f, w1 = g.ln_w != nullptr ? __half2float(g.ln_w[c + 1]) : 1.f;
                                const float b0 = g.ln_b != nullptr ? __half2float(g.ln_b[c]) : 0.f, b1 = g.ln_b != nullptr ? __half2float(g.ln_b[c + 1]) : 0.f;
                                o[j] = pack_h2(fmaf((f.x - mean) * rstd, w0, b0), fmaf((f.y - mean) * rstd, w1, b1));
                            }
                            yr[v] = out;
                        }
                    }
                    if (lane == 0) *g.ln_counter = 0u;
                }
            }
        }
        // (2) bias and gamma of the item's columns
        for (int i = et; i < g.w; i += kEpiThreads) {
            const int col = n0 + i;
            const bool in = col < g.N;
            s_bias[i] = (g.bias != nullptr && in) ? __half2float(g.bias[col]) : 0.f;
            s_gamma[i] = (g.gamma != nullptr && in) ? __half2float(g.gamma[col]) : 1.f;
            if (fuse_ln) {
                s_lnw[i] = (g.ln_w != nullptr && in) ? __half2float(g.ln_w[col]) : 1.f;
                s_lnb[i] = (g.ln_b != nullptr && in) ? __half2float(g.ln_b[col]) : 0.f;
            }
        }
        named_bar_sync(1, kEpiThreads);
        // (3) the accumulators: 32-column chunks, even chunks to warps 0-3, odd chunks to warps 4-7
        uint8_t* stage_gen = gen + store_off + ew * 2048;
        const uint32_t stage_addr = base + store_off + ew * 2048;
        // The residual of this thread's row goes into registers ahead of its use: the first kResRing chunks before the wait for
        // the accumulators (their L2 latency then runs under the main loop), chunk i + kResRing as soon as chunk i is done.
        const int row = m0 + quad * 32 + lane;
        const bool row_ok = row < g.M;
        const __half* r_row = (g.res != nullptr && row_ok) ? g.res + (int64_t)row * g.ldr : nullptr;
        constexpr int kResRing = 4, kMaxChunks = kWideMaxCols / 64;
        uint4 rr[kResRing][4];
        auto load_res = [&](int ci, uint4* dst) {
            const int c0 = (ew >> 2) * 32 + ci * 64;
#pragma unroll
            for (int q = 0; q < 4; ++q) {
                const int col = n0 + c0 + q * 8;
                dst[q] = (r_row != nullptr && c0 < g.w && col < g.N) ? *reinterpret_cast<const uint4*>(r_row + col) : make_uint4(0u, 0u, 0u, 0u);
            }
        };
#pragma unroll
        for (int ci = 0; ci < kResRing; ++ci) load_res(ci, rr[ci]);
        // With LayerNorm: running (count, mean, M2) of the fp16-rounded output values of this thread's row over its chunks
        // (Chan's merge of per-chunk two-pass statistics: no E[x^2] - E[x]^2 cancellation), and the rounded values
        // themselves parked in the operand ring, which is free once the accumulators are complete.
        float ln_cnt = 0.f, ln_mean = 0.f, ln_m2 = 0.f;
        const int stash_stride = g.w * 2 + 16;  // bytes; (stride / 16) is odd: conflict-free 16-byte accesses down a column
        uint8_t* stash_row = gen + (quad * 32 + lane) * stash_stride;
        if (mbar_wait(tfull_bar, 0u, s_abort, DEV_TIMEOUT_TMEM_FULL, 0)) {
            tc_fence_after();
            const uint32_t t_row = tmem_base + ((uint32_t)(quad * 32) << 16);
#pragma unroll
            for (int ci = 0; ci < kMaxChunks; ++ci) {
                const int c0 = (ew >> 2) * 32 + ci * 64;
                if (c0 >= g.w || n0 + c0 >= g.N) break;
                uint32_t r[32];
                float v[32];
                tmem_ld32(t_row + (uint32_t)(c0 < g.wa ? c0 : 256 + c0 - g.wa), r);
                tmem_wait_ld();
                if (g.acc_f16) {
#pragma unroll
                    for (int j = 0; j < 32; ++j) v[j] = __half2float(__ushort_as_half((unsigned short)(r[j] & 0xFFFFu)));
                } else {
#pragma unroll
                    for (int j = 0; j < 32; ++j) v[j] = __uint_as_float(r[j]);
                }
#pragma unroll
                for (int j = 0; j < 32; ++j) v[j] += s_bias[c0 + j];
                if (g.act == 1) {
#pragma unroll
                    for (int j = 0; j < 32; j += 2) {
                        const float2 y = gelu_erf2(make_float2(v[j], v[j + 1]));
                        v[j] = y.x;
                        v[j + 1] = y.y;
                    }
                }
                if (g.res != nullptr) {
#pragma unroll
                    for (int q = 0; q < 4; ++q) {
                        const __half2* rh = reinterpret_cast<const __half2*>(&rr[ci % kResRing][q]);
#pragma unroll
                        for (int j = 0; j < 4; ++j) {
                            const float2 rf = __half22float2(rh[j]);
                            v[q * 8 + 2 * j] = fmaf(s_gamma[c0 + q * 8 + 2 * j], v[q * 8 + 2 * j], rf.x);
                            v[q * 8 + 2 * j + 1] = fmaf(s_gamma[c0 + q * 8 + 2 * j + 1], v[q * 8 + 2 * j + 1], rf.y);
                        }
                    }
                    if (ci + kResRing < kMaxChunks) load_res(ci + kResRing, rr[ci % kResRing]);
                }
                if (lane == 0) bulk_wait_read_all();
                __syncwarp();
                uint4 ov[4];
#pragma unroll
                for (int q = 0; q < 4; ++q) {
                    ov[q].x = pack_h2(v[q * 8 + 0], v[q * 8 + 1]);
                    ov[q].y = pack_h2(v[q * 8 + 2], v[q * 8 + 3]);
                    ov[q].z = pack_h2(v[q * 8 + 4], v[q * 8 + 5]);
                    ov[q].w = pack_h2(v[q * 8 + 6], v[q * 8 + 7]);
                    *reinterpret_cast<uint4*>(stage_gen + lane * 64 + ((q ^ ((lane >> 1) & 3)) << 4)) = ov[q];
                }
                fence_proxy_async_smem();
                __syncwarp();
                if (lane == 0 && m0 + quad * 32 < g.M) {
                    tma_store_2d(&tmap_c, stage_addr, n0 + c0, m0 + quad * 32);
                    bulk_commit();
                }
                if (fuse_ln) {
                    float csum = 0.f;
#pragma unroll
                    for (int q = 0; q < 4; ++q) {
                        *reinterpret_cast<uint4*>(stash_row + c0 * 2 + q * 16) = ov[q];
                        const __half2* h = reinterpret_cast<const __half2*>(&ov[q]);
#pragma unroll
                        for (int j = 0; j < 4; ++j) {
                            const float2 f = __half22float2(h[j]);
                            v[q * 8 + 2 * j] = f.x;
                            v[q * 8 + 2 * j + 1] = f.y;
                            csum += f.x + f.y;
                        }
                    }
                    const float cmean = csum * (1.f / 32.f);
                    float cm2 = 0.f;
#pragma unroll
                    for (int j = 0; j < 32; ++j) cm2 = fmaf(v[j] - cmean, v[j] - cmean, cm2);
                    const float d = cmean - ln_mean, tot = ln_cnt + 32.f;
                    ln_mean += d * (32.f / tot);
                    ln_m2 += cm2 + d * d * (ln_cnt * 32.f / tot);
                    ln_cnt = tot;
                }
            }
        }
        if (fuse_ln) {
            // the two warp groups hold the even / odd chunks of the same rows: merge them into the CTA's partial per row
            const int rloc = quad * 32 + lane;
            s_part_wg[(ew >> 2) * 128 + rloc] = make_float2(ln_mean, ln_m2);
            named_bar_sync(1, kEpiThreads);
            if ((ew >> 2) == 0) {
                const int cols = min(g.w, g.N - n0);                    // valid columns of this item (multiples of 32)
                const float cnt1 = (float)(32 * (cols / 64)), cnt0 = (float)cols - cnt1;  // odd chunks / even chunks
                const float2 p1 = s_part_wg[128 + rloc];
                float mean = ln_mean, m2 = ln_m2;
                if (cnt1 > 0.f) {
                    const float d = p1.x - mean, tot = cnt0 + cnt1;
                    mean += d * (cnt1 / tot);
                    m2 += p1.y + d * d * (cnt0 * cnt1 / tot);
                }
                s_part_cta[rloc] = make_float2(mean, m2);
            }
        }
        if (lane == 0) bulk_wait_all();
    }

    if (fuse_ln) {
        // Every CTA of the cluster has its per-row partials in shared memory; the CTAs that hold the other column ranges of
        // the same rows (same parity of rank) are read through distributed shared memory. All threads take the barrier.
        __syncthreads();
        cluster_sync_all();
        if (warp >= 2) {
            const int ew = warp - 2, quad = warp & 3, rloc = quad * 32 + lane;
            if ((ew >> 2) == 0) {
                const int my_chunk = (int)(crank >> 1);
                const float2 mine = s_part_cta[rloc];
                float cnt = (float)min(g.w, g.N - n0), mean = mine.x, m2 = mine.y;
                for (int k = 0; k < g.chunks; ++k) {
                    if (k == my_chunk) continue;
                    const float2 p = ld_cluster_f32x2(smem_u32(&s_part_cta[rloc]), (uint32_t)(2 * k) | rank);
                    const float cntk = (float)min(g.w, g.N - k * g.w);
                    const float d = p.x - mean, tot = cnt + cntk;
                    mean += d * (cntk / tot);
                    m2 += p.y + d * d * (cnt * cntk / tot);
                    cnt = tot;
                }
                s_row_stat[rloc] = make_float2(mean, rsqrtf(m2 / cnt + g.ln_eps));
            }
            named_bar_sync(1, kEpiThreads);
            // second pass: the parked fp16 values, normalised, out through the staging tile to y
            const float2 st = s_row_stat[rloc];
            uint8_t* stage_gen = gen + store_off + ew * 2048;
            const uint32_t stage_addr = base + store_off + ew * 2048;
            const uint8_t* stash_row = gen + rloc * (g.w * 2 + 16);
#pragma unroll 1
            for (int c0 = (ew >> 2) * 32; c0 < g.w && n0 + c0 < g.N; c0 += 64) {
                if (lane == 0) bulk_wait_read_all();
                __syncwarp();
#pragma unroll
                for (int q = 0; q < 4; ++q) {
                    const uint4 xv = *reinterpret_cast<const uint4*>(stash_row + c0 * 2 + q * 16);
                    const __half2* h = reinterpret_cast<const __half2*>(&xv);
                    uint4 o;
                    uint32_t* op = reinterpret_cast<uint32_t*>(&o);
#pragma unroll
                    for (int j = 0; j < 4; ++j) {
                        const float2 f = __half22float2(h[j]);
                        const int c = c0 + q * 8 + 2 * j;
                        op[j] = pack_h2(fmaf((f.x - st.x) * st.y, s_lnw[c], s_lnb[c]), fmaf((f.y - st.x) * st.y, s_lnw[c + 1], s_lnb[c + 1]));
                    }
                    *reinterpret_cast<uint4*>(stage_gen + lane * 64 + ((q ^ ((lane >> 1) & 3)) << 4)) = o;
                }
                fence_proxy_async_smem();
                __syncwarp();
                if (lane == 0 && m0 + quad * 32 < g.M) {
                    tma_store_2d(&tmap_y, stage_addr, n0 + c0, m0 + quad * 32);
                    bulk_commit();
                }
            }
            if (lane == 0) bulk_wait_all();
        }
    }

    tc_fence_before();
    __syncthreads();
    cluster_sync_all();  // the peers may still be signalling this CTA's barriers / reading its operands or statistics
    if (warp == 1) {
        __syncwarp();
        tc_fence_after();
        tmem_dealloc_pair<512>(tmem_base);
    }
}

// Clusters of two that can be resident at once for this kernel on the current device (0: pairs cannot be launched).
template <int BN, bool SWIGLU>
static int max_pairs() {
    static int cached[64] = {};
    int dev = 0;
    cudaGetDevice(&dev);
    if (dev < 0 || dev >= 64) return 0;
    if (cached[dev] == 0) {
        using S = GemmSmem<BN, true>;
        auto kern = linear_umma_kernel<BN, SWIGLU, true>;
        int n = 0;
        if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, S::kDynamic) == cudaSuccess) {
            cudaLaunchConfig_t cfg = {};
            cfg.gridDim = dim3(2 * num_sms());
            cfg.blockDim = dim3(kGemmThreads);
            cfg.dynamicSmemBytes = S::kDynamic;
            cudaLaunchAttribute attr[1];
            attr[0].id = cudaLaunchAttributeClusterDimension;
            attr[0].val.clusterDim.x = 2;
            attr[0].val.clusterDim.y = 1;
            attr[0].val.clusterDim.z = 1;
            cfg.attrs = attr;
            cfg.numAttrs = 1;
            if (cudaOccupancyMaxActiveClusters(&n, kern, &cfg) != cudaSuccess) n = 0;
            cudaGetLastError();
        }
        cached[dev] = n > 0 ? n : -1;
    }
    return cached[dev] > 0 ? cached[dev] : 0;
}

// Rows left to the epilogue warps when M is a few rows more than a multiple of the tile height, and the row tiles then.
static int remainder_rows(int64_t M, int tile_rows) {
    const int r = (int)(M % tile_rows);
    return (M >= tile_rows && r > 0 && r <= kGemvMaxRows) ? r : 0;
}
static int64_t row_tiles(int64_t M, int tile_rows) { return remainder_rows(M, tile_rows) > 0 ? M / tile_rows : (M + tile_rows - 1) / tile_rows; }

// Whether a persistent form leaves the remainder rows to its epilogue warps instead of giving them a row of tiles of their
// own. Only when that saves a wave of tiles, and only when the dot products end well inside the grid's first tiles: each
// warp takes ceil(dots / warps) of them at about 0.3 us + 0.45 us per 256 elements of K (a chain of L2 round trips), a
// 256-column tile's main loop takes 0.37 us per k-block + 1 us. A small problem (M = 257: six CTAs, 48 warps, a spare SM
// for every extra tile) keeps the extra tiles: there the dot products measured 5 - 9 us per launch slower.
static bool remainder_by_gemv(int64_t M, int tile_rows, int64_t tiles_n, int workers, int64_t dots_per_row, int K, int bn) {
    const int r = remainder_rows(M, tile_rows);
    if (r == 0 || workers <= 0) return false;
    const int64_t full = (M / tile_rows) * tiles_n, with_tiles = full + tiles_n;
    if ((full + workers - 1) / workers == (with_tiles + workers - 1) / workers) return false;
    const int64_t warps = (full < workers ? full : workers) * (tile_rows / BM) * 8;
    const int64_t per_warp = (r * dots_per_row + warps - 1) / warps;
    const double gemv_us = (double)per_warp * (0.3 + 0.45 * (double)((K + 255) / 256));
    const double tile_us = (0.37 * (double)((K + BK - 1) / BK) + 1.0) * (double)bn / 256.0;
    return gemv_us <= 2.0 * tile_us;
}

// A launch of between one and two waves of tiles leaves most SMs idle for half of its time (M = 1370, N = 4096: 176 tiles =
// 148 + 28). The plain single-CTA 256-column form then cuts the tiles of the second wave into slices of 128 or 64 columns,
// as narrow as it takes for every slice to run at once: a slice costs more per column (the A tile is loaded for fewer
// columns: charged 0.85 / 0.45 of a whole tile's time, fitted so that M = 6145, N = 1024, K = 1024 keeps the wide pair
// form, 15.4 us against 16.1 us with 128-column slices) but the launch ends that much earlier (measured 21.4 -> 15 - 16 us
// for that shape). With two or more full waves before it the partial wave is cheap as it is - its few tiles run faster
// than tiles of a full wave, which share the L2-to-SM bandwidth - and slices measured slower (M = 6145, N = 4096: 46.4
// against 45.7 us; M = 16385: 127 against 118), so they are not used there.
// Returns the slice width (0: none) and its cost in tile times.
static int narrow_tail(int64_t tiles, int workers, double* cost) {
    if (cost != nullptr) *cost = 0.0;
    const char* f = getenv("FBB_GEMM_NARROW");  // 0 | 64 | 128: tuning and test override, read per call
    const int forced = f != nullptr ? atoi(f) : -1;
    if (workers <= 0 || tiles <= workers || forced == 0) return 0;
    const int64_t rest = tiles % workers;
    if (rest == 0) return 0;
    int w = 0;
    if (tiles / workers == 1) {
        if (rest * 4 <= workers) w = 64;
        else if (rest * 2 <= workers) w = 128;
    }
    if (forced == 64 || forced == 128) w = rest * (256 / forced) <= workers ? forced : 0;
    if (cost != nullptr) *cost = w == 64 ? 0.45 : (w == 128 ? 0.85 : 1.0);
    return w;
}

template <int BN, bool SWIGLU, bool CTA2>
static int launch_variant(const CUtensorMap& ta, const CUtensorMap& tw, const CUtensorMap& twn, const CUtensorMap& tc, GemmArgs g,
                          cudaStream_t stream) {
    using S = GemmSmem<BN, CTA2>;
    static bool configured[64] = {};
    int dev = 0;
    cudaGetDevice(&dev);
    auto kern = linear_umma_kernel<BN, SWIGLU, CTA2>;
    if (dev >= 0 && dev < 64 && !configured[dev]) {
        cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, S::kDynamic);
        if constexpr (!SWIGLU && !CTA2 && BN == 256) {
            if (e == cudaSuccess)
                e = cudaFuncSetAttribute(linear_umma_kernel<BN, false, false, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, S::kDynamic);
        }
        if (e != cudaSuccess) return fail((int)e, "cudaFuncSetAttribute(linear_umma_kernel): %s", cudaGetErrorString(e));
        configured[dev] = true;
    }
    constexpr int kOutCols = SWIGLU ? BN / 2 : BN;
    constexpr int kTileRows = CTA2 ? 2 * BM : BM;
    g.tiles_n = (g.n_out + kOutCols - 1) / kOutCols;
    const int workers_max = CTA2 ? max_pairs<BN, SWIGLU>() : num_sms();
    const bool gemv = remainder_by_gemv(g.M, kTileRows, g.tiles_n, workers_max, SWIGLU ? 2 * g.n_out : g.n_out, g.K, BN);
    g.gemv_rows = gemv ? remainder_rows(g.M, kTileRows) : 0;
    g.tiles_m = (int)(gemv ? g.M / kTileRows : (g.M + kTileRows - 1) / kTileRows);
    g.gemv_row0 = gemv ? g.tiles_m * kTileRows : g.M;
    const int tiles = g.tiles_m * g.tiles_n;
    const int workers = tiles < workers_max ? tiles : workers_max;
    const int grid = CTA2 ? 2 * workers : workers;
    g.wide_tiles = tiles;
    g.narrow_w = g.narrow_tiles = 0;
    if constexpr (!SWIGLU && !CTA2 && BN == 256) {
        g.narrow_w = narrow_tail(tiles, workers_max, nullptr);
        if (g.narrow_w > 0) {
            g.wide_tiles = tiles - tiles % workers_max;
            g.narrow_tiles = (tiles - g.wide_tiles) * (BN / g.narrow_w);
            // the instantiation whose item widths are run-time values (measured 2 - 7 % slower on whole tiles, which is
            // why launches without slices do not use it)
            cudaError_t e = launch_pdl_cluster(linear_umma_kernel<BN, false, false, true>, dim3(grid), dim3(kGemmThreads), S::kDynamic, stream,
                                               1u, ta, tw, twn, tc, g);
            if (e != cudaSuccess) return fail((int)e, "linear_umma_kernel (slices) launch: %s", cudaGetErrorString(e));
            return FBB_OK;
        }
    }
    cudaError_t e = launch_pdl_cluster(kern, dim3(grid), dim3(kGemmThreads), S::kDynamic, stream, CTA2 ? 2u : 1u, ta, tw, twn, tc, g);
    if (e != cudaSuccess) return fail((int)e, "linear_umma_kernel launch: %s", cudaGetErrorString(e));
    return FBB_OK;
}

// Clusters of `cluster_ctas` CTAs (2: a pair; 4, 6, 8: the pairs of a row tile that exchange LayerNorm statistics) of the
// wide kernel that can be resident at once on the current device (0: cannot be launched).
static int wide_max_clusters(int cluster_ctas) {
    static int cached[64][5] = {};
    int dev = 0;
    cudaGetDevice(&dev);
    const int slot = cluster_ctas / 2;
    if (dev < 0 || dev >= 64 || slot < 1 || slot > 4) return 0;
    if (cached[dev][slot] == 0) {
        int n = 0;
        bool ok = cudaFuncSetAttribute(linear_wide_pair_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, WideSmem::kMaxDynamic) == cudaSuccess;
        if (ok) {
            cudaLaunchConfig_t cfg = {};
            cfg.gridDim = dim3((unsigned)(cluster_ctas * num_sms()));
            cfg.blockDim = dim3(kGemmThreads);
            cfg.dynamicSmemBytes = WideSmem::kMaxDynamic;
            cudaLaunchAttribute attr[1];
            attr[0].id = cudaLaunchAttributeClusterDimension;
            attr[0].val.clusterDim.x = (unsigned)cluster_ctas;
            attr[0].val.clusterDim.y = 1;
            attr[0].val.clusterDim.z = 1;
            cfg.attrs = attr;
            cfg.numAttrs = 1;
            if (cudaOccupancyMaxActiveClusters(&n, linear_wide_pair_kernel, &cfg) != cudaSuccess) n = 0;
            cudaGetLastError();
        }
        cached[dev][slot] = n > 0 ? n : -1;
    }
    return cached[dev][slot] > 0 ? cached[dev][slot] : 0;
}
static int wide_max_pairs() { return wide_max_clusters(2); }

// Rows the wide form leaves to its epilogue warps: the remainder beyond the last full 256-row tile when it is small.
static int wide_gemv_rows(int64_t M) { return remainder_rows(M, 2 * BM); }
static int64_t wide_row_tiles(int64_t M) { return row_tiles(M, 2 * BM); }

// LayerNorm fused into the launch (see WideArgs); y == null: none.
struct WideLn {
    void* y = nullptr;
    const void* w = nullptr;
    const void* b = nullptr;
    float eps = 0.f;
    int64_t ldy = 0;
    unsigned* counter = nullptr;
};

static int launch_wide(const void* A, const void* W, void* C, const GemmArgs& base, int64_t lda, int64_t ldw, int w, cudaStream_t stream,
                       const WideLn& ln = WideLn()) {
    if (wide_max_pairs() == 0) return fail(FBB_ERR_SHAPE, "linear: this device cannot co-schedule CTA pairs");
    WideArgs g;
    g.ln_y = reinterpret_cast<__half*>(ln.y);
    g.ln_w = reinterpret_cast<const __half*>(ln.w);
    g.ln_b = reinterpret_cast<const __half*>(ln.b);
    g.ln_eps = ln.eps;
    g.ldy = ln.ldy;
    g.ln_counter = ln.counter;
    g.A = reinterpret_cast<const __half*>(A);
    g.W = reinterpret_cast<const __half*>(W);
    g.C = base.C;
    g.bias = base.bias;
    g.res = base.res;
    g.gamma = base.gamma;
    g.M = base.M;
    g.N = base.N;
    g.K = base.K;
    g.lda = lda;
    g.ldw = ldw;
    g.ldc = base.ldc;
    g.ldr = base.ldr;
    g.act = base.act;
    g.acc_f16 = base.acc_f16;
    g.w = w;
    g.wa = w <= 256 ? w : 32 * ((w + 63) / 64);
    g.wb = w - g.wa;
    g.chunks = (g.N + w - 1) / w;
    g.gemv_rows = wide_gemv_rows(g.M);
    g.gemv_row0 = g.gemv_rows > 0 ? (g.M / (2 * BM)) * (2 * BM) : g.M;
    g.stage_bytes = BM * BK * 2 + w * BK;
    g.stages = WideSmem::stages_for(g.stage_bytes);
    const int64_t items = wide_row_tiles(g.M) * g.chunks;
    if (items > 0x3FFFFFFFll) return fail(FBB_ERR_SHAPE, "linear: too many work items (%lld)", (long long)items);

    CUtensorMap ta, twa, twb, tc;
    uint64_t dims_a[2] = {(uint64_t)g.K, (uint64_t)g.M};
    int64_t str_a[2] = {1, lda};
    uint32_t box_a[2] = {BK, BM};
    int st = make_tmap_f16(&ta, A, 2, dims_a, str_a, box_a);
    if (st != FBB_OK) return st;
    uint64_t dims_w[2] = {(uint64_t)g.K, (uint64_t)g.N};
    int64_t str_w[2] = {1, ldw};
    uint32_t box_wa[2] = {BK, (uint32_t)(g.wa / 2)};
    st = make_tmap_f16(&twa, W, 2, dims_w, str_w, box_wa);
    if (st != FBB_OK) return st;
    uint32_t box_wb[2] = {BK, (uint32_t)(g.wb > 0 ? g.wb / 2 : g.wa / 2)};
    st = make_tmap_f16(&twb, W, 2, dims_w, str_w, box_wb);
    if (st != FBB_OK) return st;
    uint64_t dims_c[2] = {(uint64_t)g.N, (uint64_t)g.M};
    int64_t str_c[2] = {1, g.ldc};
    uint32_t box_c[2] = {32, 32};
    st = make_tmap_f16(&tc, C, 2, dims_c, str_c, box_c, CU_TENSOR_MAP_SWIZZLE_64B);
    if (st != FBB_OK) return st;
    CUtensorMap ty = tc;
    if (ln.y != nullptr) {
        int64_t str_y[2] = {1, ln.ldy};
        st = make_tmap_f16(&ty, ln.y, 2, dims_c, str_y, box_c, CU_TENSOR_MAP_SWIZZLE_64B);
        if (st != FBB_OK) return st;
    }

    const unsigned cluster = ln.y != nullptr ? 2u * (unsigned)g.chunks : 2u;
    cudaError_t e = launch_pdl_cluster(linear_wide_pair_kernel, dim3((unsigned)(2 * items)), dim3(kGemmThreads),
                                       (size_t)WideSmem::dynamic_bytes(g.stages, g.stage_bytes), stream, cluster, ta, twa, twb, tc, ty, g);
    if (e != cudaSuccess) return fail((int)e, "linear_wide_pair_kernel launch: %s", cudaGetErrorString(e));
    return FBB_OK;
}

static bool gemm_pairs_enabled();

// Item width of the fused GEMM + LayerNorm launch for this shape, 0 when it runs as two launches: the most column chunks
// (narrowest items, at most four pairs = eight CTAs per cluster) for which every row tile's cluster is resident at once.
// The fused form is OFF unless FBB_LN_FUSION=1: measured on B200 it is slower than the GEMM followed by the LayerNorm
// kernel on every shape of the ViT configurations (us, fused / two launches): M = 6145, N = 1024: K = 1024 33.5 / 23.3,
// K = 4096 71.8 / 48.7; M = 4097, N = 768: 19.4 / 14.0 and 26.2 / 21.2; M = 5480, N = 1536: 37.7 / 31.2 and 75.5 / 59.2;
// ViT-L/14 at 6145 tokens 10.4 instead of 9.3 ms per image. Its second epilogue pass and the cluster exchange overlap
// nothing, clusters of six or eight CTAs place worse than pairs, and the separate LayerNorm (5.4 us, most of it hidden
// behind its neighbours by programmatic dependent launch) was never the 0.3 ms it looks like in isolation.
static int fused_layernorm_width(int64_t M, int N, int epilogue, bool has_counter) {
    const char* on = getenv("FBB_LN_FUSION");
    if (on == nullptr || on[0] != '1') return 0;
    if (M <= 0 || epilogue == FBB_EPI_SWIGLU || (N % 32) != 0 || N > 4 * kWideMaxCols || !gemm_pairs_enabled() ||
        getenv("FBB_GEMM_FORCE") != nullptr || wide_max_pairs() == 0 || (wide_gemv_rows(M) > 0 && !has_counter))
        return 0;
    const int64_t tmw = wide_row_tiles(M);
    for (int chunks = 4; chunks >= 1; --chunks) {
        const int w = ((N + chunks - 1) / chunks + 31) / 32 * 32;
        if (w > kWideMaxCols || w < 64 || (N + w - 1) / w != chunks) continue;
        if (wide_max_clusters(2 * chunks) < tmw) continue;
        return w;
    }
    return 0;
}
int linear_layernorm_launches(int64_t M, int N, int epilogue, bool has_counter) {
    return M <= 0 ? 0 : (fused_layernorm_width(M, N, epilogue, has_counter) > 0 ? 1 : 2);
}

// out = epilogue(A . W^T) as launch_linear, and y = LayerNorm(out) * ln_w + ln_b. One launch (the wide pair form with the
// pairs of a row tile in one cluster) when the shape allows it, otherwise the GEMM followed by the LayerNorm kernel.
int launch_linear_layernorm(const void* A, const void* W, void* C, const void* bias, const void* res, const void* gamma, int64_t M, int N,
                            int K, int64_t lda, int64_t ldw, int64_t ldc, int64_t ldr, int epilogue, int accumulate, const void* ln_w,
                            const void* ln_b, float ln_eps, void* y, int64_t ldy, void* counter, cudaStream_t stream) {
    if (M == 0) return FBB_OK;
    {
        const int w = fused_layernorm_width(M, N, epilogue, counter != nullptr);
        if (w > 0) {
            GemmArgs g;
            g.C = reinterpret_cast<__half*>(C);
            g.bias = reinterpret_cast<const __half*>(bias);
            g.res = reinterpret_cast<const __half*>(res);
            g.gamma = res != nullptr ? reinterpret_cast<const __half*>(gamma) : nullptr;
            g.M = (int)M;
            g.N = N;
            g.K = K;
            g.n_out = N;
            g.ldc = ldc;
            g.ldr = ldr;
            g.act = epilogue == FBB_EPI_GELU ? 1 : 0;
            g.acc_f16 = accumulate == FBB_ACC_F16 ? 1 : 0;
            g.tiles_m = g.tiles_n = 0;
            g.A = reinterpret_cast<const __half*>(A);
            g.W = reinterpret_cast<const __half*>(W);
            g.lda = lda;
            g.ldw = ldw;
            g.gemv_row0 = (int)M;
            g.gemv_rows = 0;
            WideLn ln;
            ln.y = y;
            ln.w = ln_w;
            ln.b = ln_b;
            ln.eps = ln_eps;
            ln.ldy = ldy;
            ln.counter = reinterpret_cast<unsigned*>(counter);
            return launch_wide(A, W, C, g, lda, ldw, w, stream, ln);
        }
    }
    const int rc = launch_linear(A, W, C, bias, res, gamma, M, N, K, lda, ldw, ldc, ldr, epilogue, accumulate, stream);
    if (rc != FBB_OK) return rc;
    return launch_layernorm(C, y, ln_w, ln_b, M, N, ldc, ldy, ln_eps, FBB_DTYPE_F16, FBB_DTYPE_F16, stream);
}

static bool gemm_pairs_enabled() {
    static const bool on = []() {
        const char* e = getenv("FBB_GEMM_1CTA");
        return !(e != nullptr && e[0] == '1');
    }();
    return on;
}

int linear_max_pairs(int bn) { return bn == 128 ? max_pairs<128, false>() : max_pairs<256, false>(); }

int launch_linear(const void* A, const void* W, void* C, const void* bias, const void* res, const void* gamma, int64_t M,
                  int N, int K, int64_t lda, int64_t ldw, int64_t ldc, int64_t ldr, int epilogue, int accumulate,
                  cudaStream_t stream) {
    if (M == 0) return FBB_OK;
    const bool swiglu = epilogue == FBB_EPI_SWIGLU;
    GemmArgs g;
    g.C = reinterpret_cast<__half*>(C);
    g.bias = reinterpret_cast<const __half*>(bias);
    g.res = reinterpret_cast<const __half*>(res);
    g.gamma = res != nullptr ? reinterpret_cast<const __half*>(gamma) : nullptr;
    g.M = (int)M;
    g.N = N;
    g.K = K;
    g.n_out = swiglu ? N / 2 : N;
    g.ldc = ldc;
    g.ldr = ldr;
    g.act = epilogue == FBB_EPI_GELU ? 1 : 0;
    g.acc_f16 = accumulate == FBB_ACC_F16 ? 1 : 0;
    g.tiles_m = g.tiles_n = 0;
    g.A = reinterpret_cast<const __half*>(A);
    g.W = reinterpret_cast<const __half*>(W);
    g.lda = lda;
    g.ldw = ldw;
    g.gemv_row0 = (int)M;
    g.gemv_rows = 0;

    // Shape of the work item: one CTA with a 128x256 or 128x128 tile, or a CTA pair with a 256x256 tile (each CTA stages
    // its 128 rows of A and half of the W rows, which cuts the operand traffic from L2 per FLOP by a third).
    // Picked by a small cost model in units of one 128x256 one-CTA tile: waves of tiles over the workers (148 CTAs or 74
    // pairs) times the relative tile time, fitted to measurements on B200: 128-column tiles 0.60 (they move 1.3x the
    // operand bytes per FLOP), a pair's tile 0.895 per CTA plus a start-up term for the cluster launch that matters when
    // the per-tile K loop is short (M = 32768, N = 4096, K = 1024: 219 us one-CTA, 196 us pairs; M = 6145: 48 vs 50 us).
    // Pairs with 128-column tiles measured no better than single CTAs and are only reachable through the override.
    // FBB_GEMM_FORCE = s256 | s128 | p256 | p128 | w<columns> | wa (the wide form's own width) overrides the choice (tuning aid).
    const int sms = num_sms();
    const bool pairs_ok = gemm_pairs_enabled();
    const int pairs256 = pairs_ok ? (swiglu ? max_pairs<256, true>() : max_pairs<256, false>()) : 0;
    auto waves = [](int64_t tiles, int workers) { return (double)((tiles + workers - 1) / workers); };
    const int64_t tn256 = (g.n_out + 255) / 256, tn128 = (g.n_out + 127) / 128;
    const int64_t dots = swiglu ? 2 * g.n_out : g.n_out;
    // row tiles of a form: a remainder of a few rows gets none where launch_variant will leave it to the epilogue warps
    // (a SwiGLU tile of 256 weight rows yields 128 output columns)
    auto row_tiles_of = [&](int tile_rows, int64_t tiles_n, int workers, int bn) {
        const int64_t tn = swiglu ? tn128 : tiles_n;
        return remainder_by_gemv(M, tile_rows, tn, workers, dots, (int)K, bn) ? M / tile_rows : (M + tile_rows - 1) / tile_rows;
    };
    double best;
    {
        const int64_t t256 = row_tiles_of(BM, tn256, sms, 256) * tn256;
        double tail = 0.0;
        best = (!swiglu && narrow_tail(t256, sms, &tail) > 0) ? (double)(t256 / sms) + tail : waves(t256, sms) * 1.0;
    }
    bool use_pairs = false, use128 = false;
    if (!swiglu) {
        const double c = waves(row_tiles_of(BM, tn128, sms, 128) * tn128, sms) * 0.60;
        if (g.n_out <= 128 || c < best) { best = c; use128 = true; }
    }
    if (pairs256 > 0) {
        const double c = waves(row_tiles_of(2 * BM, tn256, pairs256, 256) * tn256, pairs256) * 0.895 + (K < 1536 ? 0.7 : 0.2);
        if (c < best) { best = c; use_pairs = true; use128 = false; }
    }
    // The wide pair form (items of w <= 512 columns, one wave): a candidate when every item fits on the device at once with
    // the narrowest such w and at least half of the pairs get an item. Its cost in the same units: 1.08 per 256 columns
    // (its epilogue overlaps nothing) plus about 1.8 us of start-up, a unit being one 256-column tile's main loop
    // (0.37 us per k-block + 1 us). Measured on B200 (us, wide against the best tiled form): M = 6145, N = 1024: K = 4096
    // 39.6 / 46.0, K = 1024 15.4 / 17.5 (w = 352); M = 4097, N = 768, K = 3072 17.5 / 21.0 (w = 192); not taken where it
    // measured slower: M = 5480, N = 1536 (w = 512: 25.6 / 22.8), M = 257 (a handful of items), and every shape with
    // more than one wave of items (N = 4096: 68 / 48).
    int wide_w = 0;  // > 0: the wide pair form with items of this many columns
    const int wide_pairs = (pairs_ok && !swiglu) ? wide_max_pairs() : 0;
    int wide_rule_w = 0;
    if (wide_pairs > 0) {
        const int64_t tmw = wide_row_tiles(M);
        const int64_t max_chunks = tmw > 0 ? wide_pairs / tmw : 0;
        if (max_chunks >= 1) {
            int w = (int)(((g.n_out + max_chunks - 1) / max_chunks + 31) / 32 * 32);
            if (w < 64) w = 64;
            if (w <= kWideMaxCols && tmw * ((g.n_out + w - 1) / w) <= wide_pairs) wide_rule_w = w;
        }
        if (wide_rule_w > 0) {
            const int64_t items = tmw * ((g.n_out + wide_rule_w - 1) / wide_rule_w);
            const double unit_us = 0.37 * (double)((K + BK - 1) / BK) + 1.0;
            const double c = (double)wide_rule_w / 256.0 * 1.08 + 1.8 / unit_us;
            if (2 * items >= wide_pairs && c < best) wide_w = wide_rule_w;
        }
    }
    if (const char* f = getenv("FBB_GEMM_FORCE")) {
        wide_w = 0;
        if (f[0] == 'w' && !swiglu && wide_max_pairs() > 0) {
            const int w = f[1] == 'a' ? wide_rule_w : atoi(f + 1);  // "wa": the rule's own width, whatever the cost model says
            if (w >= 32 && w <= kWideMaxCols && (w & 31) == 0) wide_w = w;
        }
        const bool want128 = f[0] != '\0' && f[1] == '1' && !swiglu;  // SwiGLU always uses 256-column tiles (x1 | x2 halves)
        if (f[0] == 's' || (f[0] == 'p' && pairs256 > 0 && (!want128 || max_pairs<128, false>() > 0))) {
            use_pairs = f[0] == 'p';
            use128 = want128;
        }
    }

    if (wide_w > 0) return launch_wide(A, W, C, g, lda, ldw, wide_w, stream);

    CUtensorMap ta, tw;
    uint64_t dims_a[2] = {(uint64_t)K, (uint64_t)M};
    int64_t str_a[2] = {1, lda};
    uint32_t box_a[2] = {BK, BM};
    int st = make_tmap_f16(&ta, A, 2, dims_a, str_a, box_a);
    if (st != FBB_OK) return st;
    uint64_t dims_w[2] = {(uint64_t)K, (uint64_t)N};
    int64_t str_w[2] = {1, ldw};
    // W box: the rows one CTA loads per k-block (a pair member loads half of the tile's rows; SwiGLU loads 128-row boxes)
    const uint32_t w_rows = swiglu ? 128u : (use128 ? 128u : 256u);
    uint32_t box_w[2] = {BK, use_pairs && !swiglu ? w_rows / 2 : w_rows};
    st = make_tmap_f16(&tw, W, 2, dims_w, str_w, box_w);
    if (st != FBB_OK) return st;
    CUtensorMap twn = tw;  // 64-row boxes of W for the slices of the last wave (plain 256-column form only)
    if (!swiglu && !use_pairs && !use128) {
        uint32_t box_wn[2] = {BK, 64};
        st = make_tmap_f16(&twn, W, 2, dims_w, str_w, box_wn);
        if (st != FBB_OK) return st;
    }

    CUtensorMap tc;
    uint64_t dims_c[2] = {(uint64_t)g.n_out, (uint64_t)M};
    int64_t str_c[2] = {1, ldc};
    uint32_t box_c[2] = {32, 32};
    st = make_tmap_f16(&tc, C, 2, dims_c, str_c, box_c, CU_TENSOR_MAP_SWIZZLE_64B);
    if (st != FBB_OK) return st;

    if (use_pairs) {
        if (swiglu) return launch_variant<256, true, true>(ta, tw, twn, tc, g, stream);
        if (use128) return launch_variant<128, false, true>(ta, tw, twn, tc, g, stream);
        return launch_variant<256, false, true>(ta, tw, twn, tc, g, stream);
    }
    if (swiglu) return launch_variant<256, true, false>(ta, tw, twn, tc, g, stream);
    if (use128) return launch_variant<128, false, false>(ta, tw, twn, tc, g, stream);
    return launch_variant<256, false, false>(ta, tw, twn, tc, g, stream);
}

}  // namespace fbb
