// O = softmax(scale . Q K^T) V for head dimension 64, no mask, any N: tcgen05 UMMA for both products, softmax in
// registers, K/V tiles streamed by TMA. Replaces flash64_r{1,2}_{hh,fh,ff} (fastbb/fastbb_kernels.cu:58-312) and the
// SDPA fallback for small inputs (fastbb/vit.py:146-150). Q, K, V are read in place from the strided [b, n, h, 64]
// views of the packed qkv GEMM output; O is written as [b, n, h*64].
//
// One CTA owns NQ (1 or 2) tiles of 128 queries of one (batch, head) and walks the keys in blocks of 128:
//   warp 0          TMA producer: Q tiles once, then K_j and V_j into a ring of stages (128-byte swizzle, zero fill)
//   warps 1, 2      UMMA issuers, one per tile: S_t = Q_t K_j^T (both K-major, 4 x K16) into tensor memory, issued as
//                   soon as the softmax group holds the previous S_t in registers; once the group has written P_t
//                   (fp16) back into tensor memory, O_t += P_t V_j (A from tensor memory, V as the MN-major B operand,
//                   8 x K16); O_t stays in tensor memory (fp32) over all key blocks
//   warps 4..11/12..19 softmax group t, 16 query rows per warp: tcgen05.ld 16x256b hands thread i the key pairs
//                   8k + 2(i%4), +1 of rows i/4 and i/4 + 8 (the m16n8 accumulator fragment), so a row's maximum and sum
//                   take two shuffles among the four threads that share it, and P (fp16 pairs) goes back with the
//                   matching 16x128b store. The 128-key block is loaded at once and S is released immediately; the
//                   maximum is taken with 3-input max, p = 2^(s*scale*log2e - m) with packed f32x2 FMAs.
//                   The running maximum m is only raised when a block exceeds it by more than 2^8 (then O_t and the
//                   running sum are rescaled in place, a rare event after the first blocks); otherwise P is taken
//                   relative to the older maximum, which keeps it <= 256 and exactly as accurate in fp16.
//                   Four softmax warps share each SM sub-partition and cover one another's waits (measured against
//                   one-thread-per-row groups of four warps: 740 -> 849 TFLOP/s at N = 16385).
// With NQ = 2 the two groups alternate on the tensor core (S of one tile is computed while the other tile is in its
// softmax). Variants (fastbb/attention.py:5-7) select the accumulate type of S: ff / fh -> fp32 S, hh -> fp16 S (an f16
// tensor-memory accumulator, read back as half2 pairs); the softmax arithmetic is fp32 in both, as in the reference.
// P.V accumulates in fp32 for every variant, because O lives in tensor memory across all key blocks: an fp16 accumulator
// there would add N terms in fp16, where the reference's fh / hh only ever add 64 (one key block) before going to fp32.
// The kernel is bound by the exponentials, not the tensor core: 128 x 128 of them per S tile against 16 results per
// clock per SM from the transcendental unit is twice the time of the tile's two matrix products (1024 vs 2 x 256 clocks).
#include "common.cuh"
#include "internal.h"

namespace fbb {

constexpr int FQ = 128;       // queries per tile
constexpr int FK = 128;       // keys per block
constexpr int kKVStages = 4;
constexpr int kTileBytes = 128 * 64 * 2;  // one [128 x 64] fp16 tile
constexpr float kLazyMax = 8.0f;          // raise the running maximum only beyond 2^8
// Which of every 8 consecutive key pairs get their exponentials from the polynomial on the FMA pipes (bit i = pair i).
// Measured on B200 (N = 16385, 16 heads): mask 0 -> 849, 0x88 -> 841, 0xAA -> 700 TFLOP/s: the extra FMA / ALU
// instructions cost what the transcendental unit saves, so the shipped default is 0 (the code path stays for tuning).
#ifndef FBB_EMU_MASK
#define FBB_EMU_MASK 0x00u
#endif
constexpr unsigned kEmuMask = FBB_EMU_MASK;  // e.g. 0x88: pairs 3 and 7 of 8 (25 %); 0: all on the transcendental unit
// Register split of the 640-thread (NQ = 2) kernel. It is launched with 96 registers per thread (the most 20 warps can
// get); setmaxnreg.inc WAITS until the CTA's own pool has the registers, so the split must fit in that pool or the
// kernel never starts its softmax: 128 * kRegsCtl + 512 * kRegsSoftmax <= 640 * 96.
constexpr int kRegsCtl = 40, kRegsSoftmax = 104;
static_assert(128 * kRegsCtl + 512 * kRegsSoftmax <= 640 * 96, "setmaxnreg split exceeds the CTA's register pool");

// tensor-memory columns
constexpr uint32_t kColS = 0;      // S_t at kColS + t*128 (128 columns each)
constexpr uint32_t kColO = 256;    // O_t at kColO + t*64 (fp32, 64 columns each)
constexpr uint32_t kColP = 384;    // P_t at kColP + t*64 (fp16 pairs: 64 columns each)

struct FlashSmem {
    static constexpr int kQOff = 0;                                  // NQ x 16 KB
    static constexpr int kKOff = 2 * kTileBytes;                     // stages x 16 KB
    static constexpr int kVOff = kKOff + kKVStages * kTileBytes;     // stages x 16 KB
    static constexpr int kBarOff = kVOff + kKVStages * kTileBytes;
    // barriers: q_full, k_full[S], v_full[S], k_empty[S], v_empty[S], s_full[2], p_ready[2], pv_done[2], s_free[2]
    static constexpr int kNumBars = 1 + 4 * kKVStages + 8;
    static constexpr int kBytes = kBarOff + kNumBars * 8 + 16;
    static constexpr int kDynamic = kBytes + 1024;
};

#ifdef FBB_FLASH_TRACE
// Development aid: per-iteration clock stamps of one softmax warp (CTA 0, lane 0 of warps 4 and 8) and of the UMMA
// issuer, written to a global buffer set through fbb_flash_trace_buffer(). Not compiled into the shipped library.
__device__ long long* g_flash_trace = nullptr;
#define FBB_TRACE(slot, j, k)                                                                                         \
    do {                                                                                                              \
        if (g_flash_trace != nullptr && blockIdx.x == 0 && blockIdx.y == 0 && lane == 0 && (j) < 64)                   \
            g_flash_trace[((slot) * 64 + (j)) * 8 + (k)] = clock64();                                                   \
    } while (0)
#else
#define FBB_TRACE(slot, j, k) do { } while (0)
#endif

struct FlashArgs {
    __half* o;
    int N, H;
    int64_t o_sb, o_sn, o_sh;
    float scale_log2;
};

template <int NQ, bool S16>
__global__ void __launch_bounds__(128 + 256 * NQ, 1)
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
    auto pv_done = [&](int t) { return bar0 + 8u * (1 + 4 * kKVStages + 4 + t); };
    auto s_free = [&](int t) { return bar0 + 8u * (1 + 4 * kKVStages + 6 + t); };
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
            mbar_init(k_empty(s), NQ);  // one commit per tile issuer
            mbar_init(v_empty(s), NQ);
        }
        for (int t = 0; t < 2; ++t) {
            mbar_init(s_full(t), 1);
            mbar_init(p_ready(t), 8);
            mbar_init(pv_done(t), 1);
            mbar_init(s_free(t), 8);
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
    grid_dependency_wait();  // the set-up above may overlap the previous kernel's tail; its outputs are visible from here

    // Warpgroup 0 holds the two single-thread roles (and two idle warps) and gives registers away; the softmax
    // warpgroups take them: a softmax thread keeps a whole 128-key row of S in registers.
    if (warp < 4) {
    if constexpr (NQ == 2) setmaxnreg_dec<kRegsCtl>();
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
    } else if (warp - 1 < NQ) {
        // ------------------------------------------------------------------ UMMA issuers: warp 1 for tile 0, warp 2 for tile 1
        // Each tile has its own issuer so that neither tile ever waits for the other one's turn. The whole warp runs the
        // code and one elected lane issues each instruction (descriptors and addresses stay warp-uniform).
        // Per key block j the order follows the order in which the softmax group produces its events:
        //   S_t free (the group has block j in registers)  ->  S_t(j+1) = Q_t K_{j+1}^T, issued while the group works on j
        //   P_t(j) written                                  ->  O_t += P_t(j) V_j
        const int t = warp - 1;
        const uint32_t idesc_qk = make_idesc_f16(FQ, FK, !S16, false, false);
        const uint32_t idesc_pv = make_idesc_f16(FQ, 64, true, false, true);
        constexpr uint64_t desc_hi = make_smem_desc_hi(16, 1024);
        const uint64_t qd = smem_desc(base + S::kQOff + t * kTileBytes, desc_hi);
        const uint64_t kd0 = smem_desc(base + S::kKOff, desc_hi);
        const uint64_t vd0 = smem_desc(base + S::kVOff, desc_hi);
        const uint32_t dS = tmem_base + kColS + t * 128, dO = tmem_base + kColO + t * 64, aP = tmem_base + kColP + t * 64;
        auto all_ok = [&](bool mine) { return __all_sync(0xffffffffu, mine) != 0; };
        auto issue_qk = [&](int s) {
            const uint64_t kd = kd0 + (uint64_t)(s * (kTileBytes >> 4));
            umma_ss_warp(dS, qd, kd, idesc_qk, 0u);
            umma_ss_warp(dS, qd + 2u, kd + 2u, idesc_qk, 1u);
            umma_ss_warp(dS, qd + 4u, kd + 4u, idesc_qk, 1u);
            umma_ss_warp(dS, qd + 6u, kd + 6u, idesc_qk, 1u);
            umma_commit_warp(s_full(t));
            umma_commit_warp(k_empty(s));
        };
        bool ok = all_ok(mbar_wait(q_full, 0, s_abort, DEV_TIMEOUT_TMA_FULL, 100));
        if (ok) ok = all_ok(mbar_wait(k_full(0), 0, s_abort, DEV_TIMEOUT_TMA_FULL, 0));
        // Tile 1 starts once tile 0's group has its first block in registers: the two groups then run slightly out of
        // step, so that one group's load / maximum / store phases overlap the other group's exponentials (measured at
        // N = 6145: 668 -> 695 TFLOP/s for ff, 600 -> 667 for hh; longer offsets change nothing).
        if (ok && t == 1 && nkb > 2) ok = all_ok(mbar_wait(s_free(0), 0, s_abort, DEV_TIMEOUT_TMEM_EMPTY, 50));
        if (ok) {
            tc_fence_after();
            issue_qk(0);
        }
        int s = 0;
        uint32_t ph = 0;
        for (int j = 0; j < nkb && ok; ++j) {
            const int sn = (s + 1 == kKVStages) ? 0 : s + 1;
            const uint32_t phn = (s + 1 == kKVStages) ? ph ^ 1u : ph;
            if (j + 1 < nkb) {
                if (!all_ok(mbar_wait(s_free(t), (uint32_t)j & 1u, s_abort, DEV_TIMEOUT_TMEM_EMPTY, t))) { ok = false; break; }
                if (!all_ok(mbar_wait(k_full(sn), phn, s_abort, DEV_TIMEOUT_TMA_FULL, sn))) { ok = false; break; }
                tc_fence_after();
                issue_qk(sn);
                FBB_TRACE(2 + t, j + 1, 3);
            }
            if (!all_ok(mbar_wait(p_ready(t), (uint32_t)j & 1u, s_abort, DEV_TIMEOUT_OTHER, 200 + t))) { ok = false; break; }
            if (!all_ok(mbar_wait(v_full(s), ph, s_abort, DEV_TIMEOUT_TMA_FULL, 16 + s))) { ok = false; break; }
            tc_fence_after();
            FBB_TRACE(2 + t, j, 1);
            const uint64_t vd = vd0 + (uint64_t)(s * (kTileBytes >> 4));
            umma_ts_warp(dO, aP, vd, idesc_pv, j != 0 ? 1u : 0u);
#pragma unroll
            for (int k = 1; k < 8; ++k) umma_ts_warp(dO, aP + 8u * k, vd + 128u * k, idesc_pv, 1u);
            umma_commit_warp(pv_done(t));
            umma_commit_warp(v_empty(s));
            FBB_TRACE(2 + t, j, 2);
            s = sn;
            ph = phn;
        }
    }
    } else {
        // ------------------------------------------------------------------ softmax groups
        // Eight warps per tile, 16 query rows per warp (tensor-memory lanes 32*(u%4) + 16*(u/4) ..+15), read with the
        // 16x256b shape: thread i holds, for rows i/4 and i/4 + 8, the key pairs 8k + 2*(i%4), +1 (k = 0..15) - the
        // m16n8 accumulator fragment. Row maxima and sums are finished with two shuffles inside the four threads that
        // share a row; P goes back with the 16x128b shape, whose layout is exactly those key pairs as fp16x2.
        // Four softmax warps per SM sub-partition keep the transcendental unit busy across one another's waits.
        if constexpr (NQ == 2) setmaxnreg_inc<kRegsSoftmax>();
        const int u = (warp - 4) & 7;
        const int t = (warp - 4) >> 3;
        const int lane_base = (u & 3) * 32 + (u >> 2) * 16;      // first tensor-memory lane (= row in the tile) of this warp
        const int cq = lane & 3;
        const int rowA = q0 + t * FQ + lane_base + (lane >> 2);  // this thread's rows: rowA and rowA + 8
        const uint32_t lane_addr = tmem_base + ((uint32_t)lane_base << 16);
        const uint32_t tS = lane_addr + kColS + t * 128;
        const uint32_t tO = lane_addr + kColO + t * 64;
        const uint32_t tP = lane_addr + kColP + t * 64;
        const float sl = a.scale_log2;
        float mA = -INFINITY, mB = -INFINITY, lA = 0.f, lB = 0.f;  // running maximum and (this thread's share of the) sum
        bool ok = true;
        // A warp whose 16 rows all lie beyond N (the padding of the last tile) only keeps the barriers moving.
        const bool warp_has_rows = q0 + t * FQ + lane_base < a.N;

        for (int j = 0; j < nkb; ++j) {
            if (u == 0) FBB_TRACE(t, j, 0);
            if (!mbar_wait(s_full(t), j & 1, s_abort, DEV_TIMEOUT_TMEM_FULL, t)) { ok = false; break; }
            tc_fence_after();
            if (u == 0) FBB_TRACE(t, j, 1);
            if (!warp_has_rows) {
                // S_t(j+1) can be ready long before the other warps have written P_t(j): this warp's arrival for block
                // j must not land in the phase of block j-1, so it watches that phase complete first.
                if (j > 0 && !mbar_wait(p_ready(t), (uint32_t)(j - 1) & 1u, s_abort, DEV_TIMEOUT_OTHER, 210 + t)) { ok = false; break; }
                tc_fence_before();
                __syncwarp();
                if (lane == 0) {
                    mbar_arrive(s_free(t));
                    mbar_arrive(p_ready(t));
                }
                continue;
            }
            const int key0 = j * FK + 2 * cq;
            const bool tail = j * FK + FK > a.N;
            uint32_t r[64];
            tmem_ld_16x256b_x16(tS, r);
            tmem_wait_ld();
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(s_free(t));  // S_t is in registers: the next Q K^T may overwrite it
            float va[64];
            if constexpr (!S16) {
#pragma unroll
                for (int i = 0; i < 64; ++i) va[i] = __uint_as_float(r[i]);
            } else {
#pragma unroll
                for (int i = 0; i < 64; ++i) va[i] = __half2float(__ushort_as_half((unsigned short)(r[i] & 0xFFFFu)));
            }
            if (tail) {
#pragma unroll
                for (int k = 0; k < 16; ++k) {
                    if (key0 + 8 * k >= a.N) va[4 * k] = va[4 * k + 2] = -INFINITY;
                    if (key0 + 8 * k + 1 >= a.N) va[4 * k + 1] = va[4 * k + 3] = -INFINITY;
                }
            }
            float mxA = fmaxf(va[0], va[1]), mxB = fmaxf(va[2], va[3]);
#pragma unroll
            for (int k = 1; k < 16; ++k) {
                mxA = fmax3(mxA, va[4 * k], va[4 * k + 1]);
                mxB = fmax3(mxB, va[4 * k + 2], va[4 * k + 3]);
            }
            mxA = fmaxf(mxA, __shfl_xor_sync(0xffffffffu, mxA, 1));
            mxB = fmaxf(mxB, __shfl_xor_sync(0xffffffffu, mxB, 1));
            mxA = fmaxf(mxA, __shfl_xor_sync(0xffffffffu, mxA, 2)) * sl;
            mxB = fmaxf(mxB, __shfl_xor_sync(0xffffffffu, mxB, 2)) * sl;
            if (u == 0) FBB_TRACE(t, j, 2);
            // O_t and P_t are still being read by P_t(j-1) . V until that product has completed (normally long ago)
            if (j > 0) {
                if (!mbar_wait(pv_done(t), (uint32_t)(j - 1) & 1u, s_abort, DEV_TIMEOUT_TMEM_FULL, 8 + t)) { ok = false; break; }
                tc_fence_after();
            }
            // ---- running maxima: raised only when this block exceeds them by more than 2^kLazyMax
            if (j == 0) {
                mA = mxA;
                mB = mxB;
            } else if (__any_sync(0xffffffffu, mxA > mA + kLazyMax || mxB > mB + kLazyMax)) {
                const float nA = fmaxf(mA, mxA), nB = fmaxf(mB, mxB);
                const float cA = ex2_approx(mA - nA), cB = ex2_approx(mB - nB);
                uint32_t o[32];
                tmem_ld_16x256b_x8(tO, o);
                tmem_wait_ld();
#pragma unroll
                for (int k = 0; k < 8; ++k) {
                    o[4 * k] = __float_as_uint(__uint_as_float(o[4 * k]) * cA);
                    o[4 * k + 1] = __float_as_uint(__uint_as_float(o[4 * k + 1]) * cA);
                    o[4 * k + 2] = __float_as_uint(__uint_as_float(o[4 * k + 2]) * cB);
                    o[4 * k + 3] = __float_as_uint(__uint_as_float(o[4 * k + 3]) * cB);
                }
                tmem_st_16x256b_x8(tO, o);
                lA *= cA;
                lB *= cB;
                mA = nA;
                mB = nB;
            }
            // ---- p = 2^(s*sl - m) in fp32; row sums in fp32; P as fp16 pairs back to tensor memory
            const float2 sl2 = make_float2(sl, sl), nmA = make_float2(-mA, -mA), nmB = make_float2(-mB, -mB);
            float2 accA = make_float2(0.f, 0.f), accB = make_float2(0.f, 0.f);
            uint32_t pk[32];
#pragma unroll
            for (int k = 0; k < 16; ++k) {
                const float2 xA = ffma2(make_float2(va[4 * k], va[4 * k + 1]), sl2, nmA);
                const float2 xB = ffma2(make_float2(va[4 * k + 2], va[4 * k + 3]), sl2, nmB);
                float2 pA, pB;
                if ((kEmuMask >> (k & 7)) & 1) {  // this key pair on the FMA pipes instead of the transcendental unit
                    pA = exp2_emulated(xA);
                    pB = exp2_emulated(xB);
                } else {
                    pA = make_float2(ex2_approx(xA.x), ex2_approx(xA.y));
                    pB = make_float2(ex2_approx(xB.x), ex2_approx(xB.y));
                }
                accA = fadd2(accA, pA);
                accB = fadd2(accB, pB);
                pk[2 * k] = pack_h2(pA.x, pA.y);
                pk[2 * k + 1] = pack_h2(pB.x, pB.y);
            }
            tmem_st_16x128b_x16(tP, pk);
            if (u == 0) FBB_TRACE(t, j, 3);
            tmem_wait_st();
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(p_ready(t));
            if (u == 0) FBB_TRACE(t, j, 4);
            lA += accA.x + accA.y;
            lB += accB.x + accB.y;
        }
        if (ok && warp_has_rows && mbar_wait(pv_done(t), (uint32_t)(nkb - 1) & 1u, s_abort, DEV_TIMEOUT_TMEM_FULL, 8 + t)) {
            tc_fence_after();
            // a row's sum is spread over the four threads that share it
            lA += __shfl_xor_sync(0xffffffffu, lA, 1);
            lB += __shfl_xor_sync(0xffffffffu, lB, 1);
            lA += __shfl_xor_sync(0xffffffffu, lA, 2);
            lB += __shfl_xor_sync(0xffffffffu, lB, 2);
            const float invA = 1.f / lA, invB = 1.f / lB;
            uint32_t o[32];
            tmem_ld_16x256b_x8(tO, o);
            tmem_wait_ld();
            __half* dstA = a.o + (int64_t)b * a.o_sb + (int64_t)rowA * a.o_sn + (int64_t)h * a.o_sh + 2 * cq;
            __half* dstB = dstA + 8 * a.o_sn;
#pragma unroll
            for (int k = 0; k < 8; ++k) {
                if (rowA < a.N)
                    *reinterpret_cast<uint32_t*>(dstA + 8 * k) = pack_h2(__uint_as_float(o[4 * k]) * invA, __uint_as_float(o[4 * k + 1]) * invA);
                if (rowA + 8 < a.N)
                    *reinterpret_cast<uint32_t*>(dstB + 8 * k) = pack_h2(__uint_as_float(o[4 * k + 2]) * invB, __uint_as_float(o[4 * k + 3]) * invB);
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

template <int NQ, bool S16>
static int launch_flash_variant(const CUtensorMap& tq, const CUtensorMap& tk, const CUtensorMap& tv, const FlashArgs& a, int B,
                                cudaStream_t stream) {
    static bool configured[64] = {};
    int dev = 0;
    cudaGetDevice(&dev);
    auto kern = flash64_umma_kernel<NQ, S16>;
    if (dev >= 0 && dev < 64 && !configured[dev]) {
        cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, FlashSmem::kDynamic);
        if (e != cudaSuccess) return fail((int)e, "cudaFuncSetAttribute(flash64_umma_kernel): %s", cudaGetErrorString(e));
        configured[dev] = true;
    }
    dim3 grid((unsigned)((a.N + FQ * NQ - 1) / (FQ * NQ)), (unsigned)(B * a.H), 1);
    cudaError_t e = launch_pdl(kern, grid, dim3(128 + 256 * NQ), FlashSmem::kDynamic, stream, tq, tk, tv, a);
    if (e != cudaSuccess) return fail((int)e, "flash64_umma_kernel launch: %s", cudaGetErrorString(e));
    return FBB_OK;
}

#ifdef FBB_FLASH_TRACE
extern "C" int fbb_flash_trace_buffer(void* buf) {
    long long* p = reinterpret_cast<long long*>(buf);
    return (int)cudaMemcpyToSymbol(g_flash_trace, &p, sizeof(p));
}
#endif

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
    const bool s16 = variant == FBB_FLASH_HH;
    if (two) return s16 ? launch_flash_variant<2, true>(tq, tk, tv, a, B, stream) : launch_flash_variant<2, false>(tq, tk, tv, a, B, stream);
    return s16 ? launch_flash_variant<1, true>(tq, tk, tv, a, B, stream) : launch_flash_variant<1, false>(tq, tk, tv, a, B, stream);
}

}  // namespace fbb
