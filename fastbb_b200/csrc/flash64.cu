// O = softmax(scale . Q K^T) V for head dimension 64, no mask, any N: tcgen05 UMMA for both products, softmax in
// registers, K/V tiles streamed by TMA. Replaces flash64_r{1,2}_{hh,fh,ff} (fastbb/fastbb_kernels.cu:58-312) and the
// SDPA fallback for small inputs (fastbb/vit.py:146-150). Q, K, V are read in place from the strided [b, n, h, 64]
// views of the packed qkv GEMM output; O is written as [b, n, h*64].
//
// Work: a "tile group" is NQ (1 or 2) tiles of 128 queries of one (batch, head); it walks the keys in blocks of 128, so
// the whole problem is groups x key blocks "units". Without a workspace every CTA takes exactly one group. With a
// workspace, and when the groups do not fill the SMs evenly, the grid is persistent (one CTA per SM): every CTA first
// takes whole groups round-robin (group = round * G + cta, so CTAs running together share heads, i.e. K/V tiles in L2)
// for all but the last full wave, then an equal share of the units of what is left (between one and two waves' worth,
// so a share is at least one group long and a group is split over at most two CTAs):
//   - the CTA whose share starts in the middle of a group (always the first item of its share) leaves the unnormalised
//     O (fp32), the running maxima and sums in its workspace slot and raises the slot's per-warp flags;
//   - the CTA that began that group (always the last item of its share, so it needs the slot late) merges the slot into
//     its own accumulators, clears the flags and writes the rows.
// With 400 groups on 148 SMs (ViT-L/14 at 896x1344) this replaces 3 waves by 2.7; part of the gain is lost because the
// two tiles of a long-lived CTA drift into step (see below): 2.5 % on whole-model time.
//
//   warp 0          TMA producer: the Q tiles of each item, then K_j and V_j into a ring of stages (128-byte swizzle, zero fill)
//   warps 1, 2      UMMA issuers, one per tile: S_t = Q_t K_j^T (both K-major, 4 x K16) into tensor memory, issued as
//                   soon as the softmax group holds the previous S_t in registers - also across items, so the first
//                   product of the next group overlaps the last softmax and the write-out of this one; once the group
//                   has written P_t (fp16) back into tensor memory, O_t += P_t V_j (A from tensor memory, V as the
//                   MN-major B operand, 8 x K16); O_t stays in tensor memory (fp32) over the key blocks of an item
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
// softmax). Variants (fastbb/attention.py:5-7) name the accumulate types of the two products in the reference's
// mma.sync kernels, where fp16 accumulation doubles the GeForce tensor rate. On tcgen05 an f16 accumulator runs at the
// same rate as an fp32 one, and reading it back costs a conversion per element (measured: 215 vs 201 us per launch at
// N = 6145), so ff, fh and hh all run with fp32 S here; the softmax arithmetic is fp32 as in the reference. P.V
// accumulates in fp32 as well, because O lives in tensor memory across all key blocks: an fp16 accumulator there would
// add N terms in fp16, where the reference's fh / hh only ever add 64 (one key block) before going to fp32. Every
// variant is therefore at least as accurate as the reference's.
// The kernel is bound by the exponentials, not the tensor core: 128 x 128 of them per S tile against 16 results per
// clock per SM from the transcendental unit is twice the time of the tile's two matrix products (1024 vs 2 x 256 clocks).
// Measured dynamics worth knowing before changing the pipeline: a softmax warp alone cannot saturate the transcendental
// unit, so the two tiles run fastest half a period apart (2800 clocks per unit); in step, every phase collides with its
// twin (3800 clocks). The half-period offset set at start-up is not stable: over some tens of units the later tile
// catches up. CTAs that live for one group (<= ~130 units) mostly keep it; the persistent form loses part of what it
// gains from the removed wave this way. Every way of forcing the offset that was built measured slower than letting the
// tiles run free (N = 6145, 16 heads, 198-200 us free): strict turns around a whole unit (3100 clocks per unit); turns
// around the exponential loop only, per SM sub-partition, so that one tile's load / maximum / store phases fall under the
// other's exponentials (218 us: the two warps a tile has on a sub-partition do not saturate its transcendental unit on
// their own, four contending warps use it better); a one-sided lock that only holds a tile back until the other is
// 4/16 .. 14/16 of the way through its exponentials (201-212 us). Batching the exponentials in the source (arguments,
// then exponentials, then sums) compiles to the same schedule; writing P back in two halves costs a second wait (212 us).
#include "common.cuh"
#include <cstdlib>

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
// kernel never starts its softmax: 128 * kRegsCtl + 512 * kRegsSoftmax <= 640 * 96. 32 / 112 measured 2 % faster than
// 40 / 104 (197 vs 201 us at N = 6145): a softmax thread holds 64 scores and up to 32 packed probabilities.
#ifndef FBB_REGS_CTL
#define FBB_REGS_CTL 32
#define FBB_REGS_SOFTMAX 112
#endif
constexpr int kRegsCtl = FBB_REGS_CTL, kRegsSoftmax = FBB_REGS_SOFTMAX;
static_assert(128 * kRegsCtl + 512 * kRegsSoftmax <= 640 * 96, "setmaxnreg split exceeds the CTA's register pool");

// tensor-memory columns of tile t: S_t (128 columns) at t * kColTileS, O_t (fp32, 64 columns) at kColO + t * kColTileOP,
// P_t (fp16 pairs, 64 columns) kColP after O_t
constexpr uint32_t kColTileS = 128, kColO = 256, kColTileOP = 64, kColP = 128;

struct FlashSmem {
    static constexpr int kQOff = 0;                                  // NQ (<= 2) tiles x 16 KB
    static constexpr int kKOff = 2 * kTileBytes;                     // stages x 16 KB
    static constexpr int kVOff = kKOff + kKVStages * kTileBytes;     // stages x 16 KB
    static constexpr int kBarOff = kVOff + kKVStages * kTileBytes;
    // barriers: q_full, q_empty, k_full[S], v_full[S], k_empty[S], v_empty[S], s_full[2], p_ready[2], pv_done[2], s_free[2], t1_go
    static constexpr int kNumBars = 2 + 4 * kKVStages + 8 + 1;
    static constexpr int kTailOff = kBarOff + kNumBars * 8 + 16;    // TailItems (40 bytes)
    static constexpr int kBytes = kTailOff + 48;
    // No slack for aligning by hand (the array is declared 1024-byte aligned): 160.4 KB keeps the CTA inside the 164 KB
    // shared-memory configuration, which leaves the rest of the SM's 256 KB to L1 (the softmax warps spill a few registers).
    static constexpr int kDynamic = kBytes;
};

// Workspace of the split form: per CTA one slot for the group it starts in the middle. A slot holds, for each of the 16
// softmax warps, 36 values per lane stored [value][lane] (32 accumulator registers of the 16x256b fragment, then the two
// running maxima and the lane's shares of the two running sums), preceded by one flag word per warp.
constexpr int kSlotWarps = 16;
constexpr int kSlotValues = 36;
constexpr size_t kSlotFloats = (size_t)kSlotWarps * kSlotValues * 32;
constexpr size_t kFlagBytesPerCta = kSlotWarps * sizeof(unsigned);
// Leftover query rows: every ViT token count is a multiple of the 256-row tile group plus the cls token (and a few
// registers), and a 25th group per head for ONE row costs the N = 6145 launch 3.5 % (N = 6144: 189 us, 6145: 200 us).
// Up to kSideMaxRows rows beyond the last full group are therefore not tiled: a second, small launch
// (flash64_side_rows_kernel) computes them on the CUDA cores. It is the tiled launch's programmatic dependent, so its
// CTAs (128 threads, 32 registers, no shared memory: what the tiled kernel leaves free on an SM) run beside the tiled
// kernel's, and it waits for that kernel only at its very end, so that whatever depends on it depends on both.
constexpr int kSideMaxRows = 8;
constexpr int kSideMaxChunks = 64;
constexpr int kSideValues = 66;  // per (row, key chunk): 64 outputs, maximum, sum
constexpr int kSideMaxTasks = 1024;
// flag words of the split form, then one counter per leftover row
constexpr size_t flag_region_bytes(int ctas) { return ((size_t)ctas * (kFlagBytesPerCta + sizeof(unsigned)) + 255) & ~(size_t)255; }
constexpr size_t side_region_bytes() { return ((size_t)kSideMaxTasks * kSideValues * sizeof(float) + 255) & ~(size_t)255; }
int64_t flash64_workspace_bytes();
static bool split_pays(int64_t groups, int sms);

// Built-in workspace of fbb_flash64_f16_static: room for the split form on a device of up to kStaticMaxSms SMs
// (11.5 MiB; zero-initialised when the module is loaded, as the flag words must be).
constexpr int kStaticMaxSms = 160;
constexpr size_t kStaticWsBytes = flag_region_bytes(kStaticMaxSms) + (size_t)kStaticMaxSms * kSlotFloats * sizeof(float) + side_region_bytes();
static __device__ __align__(256) unsigned char g_flash_static_ws[kStaticWsBytes];

#ifdef FBB_FLASH_TRACE
// Development aid: per-iteration clock stamps of one softmax warp (CTA 0, lane 0 of warps 4 and 8) and of the UMMA
// issuer, written to a global buffer set through fbb_flash_trace_buffer(). Not compiled into the shipped library.
__device__ long long* g_flash_trace = nullptr;
#define FBB_TRACE(slot, j, k)                                                                                         \
    do {                                                                                                              \
        if (g_flash_trace != nullptr && blockIdx.x == 0 && lane == 0 && (j) < 64)                                      \
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
    int groups_per_head;     // ceil(N / (128 * NQ))
    int nkb;                 // key blocks per group
    int rounds;              // whole groups every CTA takes round-robin before the tail region
    long long tail_units;    // (groups - rounds * gridDim.x) * nkb, dealt out in equal contiguous shares
    unsigned* ws_flags;      // [gridDim.x][16], all zero between launches; null when no group is ever split
    float* ws_data;          // [gridDim.x][kSlotFloats]
    int Nq;                  // query rows covered by tiles; rows [Nq, N) are left to flash64_side_rows_kernel
};

struct SideArgs {
    const __half *q, *k, *v;
    __half* o;
    int64_t q_sb, q_sn, q_sh, k_sb, k_sn, k_sh, v_sb, v_sn, v_sh, o_sb, o_sn, o_sh;
    int N, H, row0, rows, chunks, tasks;  // rows [row0, row0 + rows) of every (batch, head); tasks = B * H * rows * chunks
    float scale_log2;
    unsigned* count;         // [B * H * rows], all zero between launches
    float* part;             // [tasks][kSideValues]
};

// A CTA's work is a list of items (group w, key blocks [kb0, kb1)): first `rounds` whole groups taken round-robin
// (group = round * G + cta, so that the CTAs running at the same time share heads, i.e. K/V tiles in L2), then its share
// of the tail region, whose (group, key block) units are dealt out in contiguous runs of at least one group's length:
// at most three items (the end of a group another CTA began, a whole group, the beginning of one the next CTA ends).
// Thread 0 writes the tail items to shared memory once; every role walks the list by item index.
struct TailItems {
    int n;
    int w[3], kb0[3], kb1[3];
};

__device__ __forceinline__ unsigned ld_acquire_gpu(const unsigned* p) {
    unsigned v;
    asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ void st_release_gpu(unsigned* p, unsigned v) {
    asm volatile("st.release.gpu.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}

// Lane 0 polls a workspace flag until it is raised (bounded like every other wait); the result is warp-uniform.
__device__ __forceinline__ bool wait_slot_flag(const unsigned* flag, int lane, volatile int* abort_flag, unsigned detail) {
    bool ok = true;
    if (lane == 0 && ld_acquire_gpu(flag) == 0u) {
        const uint64_t t0 = globaltimer_ns();
        for (;;) {
            __nanosleep(200);
            if (ld_acquire_gpu(flag) != 0u) break;
            if (*abort_flag) { ok = false; break; }
            if (globaltimer_ns() - t0 > kWaitLimitNs) {
                report_error(DEV_TIMEOUT_OTHER, detail);
                *abort_flag = 1;
                __threadfence_block();
                ok = false;
                break;
            }
        }
    }
    ok = __all_sync(0xffffffffu, ok) != 0;
    __syncwarp();
    if (ok) (void)ld_acquire_gpu(flag);  // every lane orders its own reads of the slot after the flag
    return ok;
}

// One warp per (leftover query row, chunk of the keys). Scores: lane j takes key j of each 32-key step (fp32 dot product
// over the 64 dimensions); then the lanes switch to two output dimensions each and add p_j * v_j for the step's keys, p_j
// broadcast by shuffle: an online softmax in the scaled log2 domain of the tiled path (x = s * scale_log2). The partial
// (64 outputs, maximum, sum) goes to the workspace; the warp whose counter update completes a row merges its chunks and
// stores the row. No warp waits for another. 32 registers (16 CTAs of 128 threads would fit an SM): the point is to fit
// beside a resident CTA of the tiled kernel, which leaves 4096 registers and no shared memory to spare.
__global__ void __launch_bounds__(128, 16) flash64_side_rows_kernel(const SideArgs a) {
    grid_launch_dependents();
    const int lane = threadIdx.x & 31;
    const int task = (int)blockIdx.x * 4 + (int)(threadIdx.x >> 5);
    if (task < a.tasks) {
        const int chunk = task % a.chunks, rid = task / a.chunks;
        const int bh = rid / a.rows;
        const int row = a.row0 + (rid - bh * a.rows);
        const int b = bh / a.H, h = bh - b * a.H;
        const int per = (a.N + a.chunks - 1) / a.chunks;
        const int k0 = chunk * per, k1 = min(a.N, k0 + per);
        const uint4* qv = reinterpret_cast<const uint4*>(a.q + b * a.q_sb + (int64_t)row * a.q_sn + h * a.q_sh);
        const __half* kb = a.k + b * a.k_sb + h * a.k_sh;
        const __half* vb = a.v + b * a.v_sb + h * a.v_sh + 2 * lane;
        float m = -INFINITY, l = 0.f, o0 = 0.f, o1 = 0.f;
#pragma unroll 1
        for (int j0 = k0; j0 < k1; j0 += 32) {
            const int j = j0 + lane;
            float sc = -INFINITY;
            if (j < k1) {
                const uint4* kv = reinterpret_cast<const uint4*>(kb + (int64_t)j * a.k_sn);
                float acc = 0.f;
#pragma unroll 2
                for (int d = 0; d < 8; ++d) {
                    const uint4 kk = __ldcg(kv + d), qq = __ldg(qv + d);  // K and V stream past L1, which holds the tiled kernel's spills
                    const __half2* kh = reinterpret_cast<const __half2*>(&kk);
                    const __half2* qh = reinterpret_cast<const __half2*>(&qq);
#pragma unroll
                    for (int e = 0; e < 4; ++e) {
                        const float2 kf = __half22float2(kh[e]), qf = __half22float2(qh[e]);
                        acc = fmaf(kf.x, qf.x, acc);
                        acc = fmaf(kf.y, qf.y, acc);
                    }
                }
                sc = acc * a.scale_log2;
            }
            float mx = sc;
#pragma unroll
            for (int sft = 16; sft > 0; sft >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, sft));
            const float mn = fmaxf(m, mx);       // finite: the step holds at least one key
            const float c = ex2_approx(m - mn);   // 0 on the first step (m = -inf)
            const float p = ex2_approx(sc - mn);  // 0 for lanes beyond the chunk
            float ps = p;
#pragma unroll
            for (int sft = 16; sft > 0; sft >>= 1) ps += __shfl_xor_sync(0xffffffffu, ps, sft);
            l = l * c + ps;
            o0 *= c;
            o1 *= c;
            m = mn;
            const int cnt = min(32, k1 - j0);
#pragma unroll 4
            for (int jj = 0; jj < cnt; ++jj) {
                const float pj = __shfl_sync(0xffffffffu, p, jj);
                const unsigned vw = __ldcg(reinterpret_cast<const unsigned*>(vb + (int64_t)(j0 + jj) * a.v_sn));
                const float2 vf = __half22float2(*reinterpret_cast<const __half2*>(&vw));
                o0 = fmaf(pj, vf.x, o0);
                o1 = fmaf(pj, vf.y, o1);
            }
        }
        float* part = a.part + (size_t)task * kSideValues;
        *reinterpret_cast<float2*>(part + 2 * lane) = make_float2(o0, o1);
        if (lane == 0) {
            part[64] = m;
            part[65] = l;
        }
        __threadfence();
        __syncwarp();
        unsigned prev = 0u;
        if (lane == 0) prev = atomicAdd(a.count + rid, 1u);
        prev = __shfl_sync(0xffffffffu, prev, 0);
        if (prev + 1u == (unsigned)a.chunks) {
            // this warp completed the row: merge the chunks (an empty chunk has m = -inf and contributes nothing)
            __threadfence();
            const float* parts = a.part + (size_t)rid * a.chunks * kSideValues;
            float M = -INFINITY;
            for (int ci = 0; ci < a.chunks; ++ci) M = fmaxf(M, __ldcg(parts + ci * kSideValues + 64));
            float L = 0.f, O0 = 0.f, O1 = 0.f;
            for (int ci = 0; ci < a.chunks; ++ci) {
                const float* pc = parts + ci * kSideValues;
                const float w = ex2_approx(__ldcg(pc + 64) - M);
                const float2 oc = __ldcg(reinterpret_cast<const float2*>(pc + 2 * lane));
                L = fmaf(__ldcg(pc + 65), w, L);
                O0 = fmaf(oc.x, w, O0);
                O1 = fmaf(oc.y, w, O1);
            }
            const float inv = 1.f / L;
            __half* dst = a.o + b * a.o_sb + (int64_t)row * a.o_sn + h * a.o_sh + 2 * lane;
            *reinterpret_cast<__half2*>(dst) = __floats2half2_rn(O0 * inv, O1 * inv);
            if (lane == 0) a.count[rid] = 0u;  // free for the next launch
        }
    }
    // The tiled launch before this one in the stream is still running. Nothing above depends on it (q, k and v were complete
    // before it started, and the rows written here are not its rows), but whoever waits for THIS grid must find that one
    // complete as well.
    grid_dependency_wait();
}

template <int NQ>
__global__ void __launch_bounds__(128 + 256 * NQ, 1)
flash64_umma_kernel(const __grid_constant__ CUtensorMap tmap_q, const __grid_constant__ CUtensorMap tmap_k,
                    const __grid_constant__ CUtensorMap tmap_v, const FlashArgs a) {
    using S = FlashSmem;
    extern __shared__ __align__(1024) uint8_t smem_raw[];
    const uint32_t base = smem_u32(smem_raw);
    uint8_t* gen = smem_raw;
    const uint32_t bar0 = base + S::kBarOff;
    const uint32_t q_full = bar0, q_empty = bar0 + 8u;
    auto k_full = [&](int s) { return bar0 + 8u * (2 + s); };
    auto v_full = [&](int s) { return bar0 + 8u * (2 + kKVStages + s); };
    auto k_empty = [&](int s) { return bar0 + 8u * (2 + 2 * kKVStages + s); };
    auto v_empty = [&](int s) { return bar0 + 8u * (2 + 3 * kKVStages + s); };
    auto s_full = [&](int t) { return bar0 + 8u * (2 + 4 * kKVStages + t); };
    auto p_ready = [&](int t) { return bar0 + 8u * (2 + 4 * kKVStages + 2 + t); };
    auto pv_done = [&](int t) { return bar0 + 8u * (2 + 4 * kKVStages + 4 + t); };
    auto s_free = [&](int t) { return bar0 + 8u * (2 + 4 * kKVStages + 6 + t); };
    const uint32_t t1_go = bar0 + 8u * (2 + 4 * kKVStages + 8);  // completes once: tile 0's issuer has seen its group take the first block
    volatile uint32_t* s_tmem = reinterpret_cast<volatile uint32_t*>(gen + S::kBarOff + S::kNumBars * 8);
    volatile int* s_abort = reinterpret_cast<volatile int*>(gen + S::kBarOff + S::kNumBars * 8 + 4);
    TailItems* s_tail = reinterpret_cast<TailItems*>(gen + S::kTailOff);

    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;
    const int nkb = a.nkb;

    if (threadIdx.x == 0) {
        mbar_init(q_full, 1);
        mbar_init(q_empty, NQ);  // one commit per tile issuer, after the item's last Q K^T
        for (int s = 0; s < kKVStages; ++s) {
            mbar_init(k_full(s), 1);
            mbar_init(v_full(s), 1);
            mbar_init(k_empty(s), NQ);
            mbar_init(v_empty(s), NQ);
        }
        for (int t = 0; t < 2; ++t) {
            mbar_init(s_full(t), 1);
            mbar_init(p_ready(t), 8);
            mbar_init(pv_done(t), 1);
            mbar_init(s_free(t), 8);
        }
        mbar_init(t1_go, 1);
        *s_abort = 0;
        // this CTA's share [tb, te) of the tail region's units, cut into items at group boundaries
        long long tb = 0, te = 0;
        if (a.tail_units > 0) {
            tb = (long long)(((unsigned long long)a.tail_units * blockIdx.x) / gridDim.x);
            te = (long long)(((unsigned long long)a.tail_units * (blockIdx.x + 1u)) / gridDim.x);
        }
        int n = 0;
        for (long long uu = tb; uu < te && n < 3; ++n) {  // (no iterations without a tail region)
            const int wt = (int)(uu / nkb);
            const int kb0 = (int)(uu - (long long)wt * nkb);
            const int kb1 = (int)((te - uu < (long long)(nkb - kb0)) ? kb0 + (te - uu) : nkb);
            s_tail->w[n] = a.rounds * (int)gridDim.x + wt;
            s_tail->kb0[n] = kb0;
            s_tail->kb1[n] = kb1;
            uu += kb1 - kb0;
        }
        s_tail->n = n;
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
    grid_launch_dependents();

    // Item list of this CTA (see TailItems): items [0, rounds) are whole groups, the rest come from the table.
    const int n_items = a.rounds + s_tail->n;
    auto item_at = [&](int it, int& w, int& kb0, int& kb1) {
        if (it < a.rounds) {
            w = it * (int)gridDim.x + (int)blockIdx.x;
            kb0 = 0;
            kb1 = nkb;
        } else {
            w = s_tail->w[it - a.rounds];
            kb0 = s_tail->kb0[it - a.rounds];
            kb1 = s_tail->kb1[it - a.rounds];
        }
    };

    // Warpgroup 0 holds the two single-thread roles (and two idle warps) and gives registers away; the softmax
    // warpgroups take them: a softmax thread keeps a whole 128-key row of S in registers.
    if (warp < 4) {
    if constexpr (NQ == 2) setmaxnreg_dec<kRegsCtl>();
    if (warp == 0) {
        // ------------------------------------------------------------------ TMA producer
        if (lane == 0) {
            int s = 0;
            uint32_t ph = 0;
            bool ok = true;
#pragma unroll 1
            for (int it = 0; it < n_items && ok; ++it) {
                int w, kb0, kb1;
                item_at(it, w, kb0, kb1);
                const int bh = w / a.groups_per_head;
                const int q0 = (w - bh * a.groups_per_head) * (FQ * NQ);
                const int b = bh / a.H, h = bh - b * a.H;
                // Q is single-buffered: the previous item's last Q K^T must have read it (that product is issued one unit
                // early, so the reload overlaps the previous item's last softmax and write-out)
                if (!mbar_wait(q_empty, ((uint32_t)it & 1u) ^ 1u, s_abort, DEV_TIMEOUT_SMEM_EMPTY, 32)) { ok = false; break; }
                mbar_arrive_expect_tx(q_full, NQ * kTileBytes);
                for (int t = 0; t < NQ; ++t) tma_load_4d(base + S::kQOff + t * kTileBytes, &tmap_q, q_full, 0, h, q0 + t * FQ, b);
#pragma unroll 1
                for (int kb = kb0; kb < kb1; ++kb) {
                    if (!mbar_wait(k_empty(s), ph ^ 1u, s_abort, DEV_TIMEOUT_SMEM_EMPTY, s)) { ok = false; break; }
                    mbar_arrive_expect_tx(k_full(s), kTileBytes);
                    tma_load_4d(base + S::kKOff + s * kTileBytes, &tmap_k, k_full(s), 0, h, kb * FK, b);
                    if (!mbar_wait(v_empty(s), ph ^ 1u, s_abort, DEV_TIMEOUT_SMEM_EMPTY, 16 + s)) { ok = false; break; }
                    mbar_arrive_expect_tx(v_full(s), kTileBytes);
                    tma_load_4d(base + S::kVOff + s * kTileBytes, &tmap_v, v_full(s), 0, h, kb * FK, b);
                    if (++s == kKVStages) { s = 0; ph ^= 1u; }
                }
            }
            if (!ok) __nanosleep(20000);
        }
    } else if (warp - 1 < NQ) {
        // ------------------------------------------------------------------ UMMA issuers: warp 1 for tile 0, warp 2 for tile 1
        // Each tile has its own issuer so that neither tile ever waits for the other one's turn. The whole warp runs the
        // code and one elected lane issues each instruction (descriptors and addresses stay warp-uniform).
        // Per unit g (one key block of the current item) the order follows the softmax group's events:
        //   S_t free (the group has unit g in registers)  ->  S_t(g+1) = Q_t K^T of the next unit, which may belong to
        //                                                      the next item (other Q buffer), issued while the group works on g
        //   P_t(g) written                                 ->  O_t (+)= P_t(g) V
        const int t = warp - 1;
        const uint32_t idesc_qk = make_idesc_f16(FQ, FK, true, false, false);
        const uint32_t idesc_pv = make_idesc_f16(FQ, 64, true, false, true);
        constexpr uint64_t desc_hi = make_smem_desc_hi(16, 1024);
        const uint64_t qd0 = smem_desc(base + S::kQOff + t * kTileBytes, desc_hi);
        const uint64_t kd0 = smem_desc(base + S::kKOff, desc_hi);
        const uint64_t vd0 = smem_desc(base + S::kVOff, desc_hi);
        const uint32_t dS = tmem_base + t * kColTileS, dO = tmem_base + kColO + t * kColTileOP, aP = dO + kColP;
        auto all_ok = [&](bool mine) { return __all_sync(0xffffffffu, mine) != 0; };
        // S_t = Q_t K^T for one unit: Q buffer of item `it`, K in stage s; `last` = the item's last unit
        auto issue_qk = [&](int s, bool last) {
            const uint64_t qd = qd0;
            const uint64_t kd = kd0 + (uint64_t)(s * (kTileBytes >> 4));
            umma_ss_warp(dS, qd, kd, idesc_qk, 0u);
            umma_ss_warp(dS, qd + 2u, kd + 2u, idesc_qk, 1u);
            umma_ss_warp(dS, qd + 4u, kd + 4u, idesc_qk, 1u);
            umma_ss_warp(dS, qd + 6u, kd + 6u, idesc_qk, 1u);
            umma_commit_warp(s_full(t));
            umma_commit_warp(k_empty(s));
            if (last) umma_commit_warp(q_empty);  // the producer may load the next item's Q
        };
        int it = 0, kb = 0, kb1 = 0;
        bool ok = n_items > 0;
        if (ok) {
            int w;
            item_at(0, w, kb, kb1);
        }
        if (ok) ok = all_ok(mbar_wait(q_full, 0, s_abort, DEV_TIMEOUT_TMA_FULL, 100));
        if (ok) ok = all_ok(mbar_wait(k_full(0), 0, s_abort, DEV_TIMEOUT_TMA_FULL, 0));
        // Tile 1 starts once tile 0's group has its first block in registers: the two groups then run slightly out of
        // step, so that one group's load / maximum / store phases overlap the other group's exponentials (measured at
        // N = 6145: 668 -> 695 TFLOP/s for ff, 600 -> 667 for hh; longer offsets change nothing).
        // (a barrier of its own that completes exactly once: waiting on s_free(0) by parity could be overtaken by tile 0's
        // second block and then never return)
        if (ok && t == 1 && (n_items > 1 || kb1 - kb > 2)) ok = all_ok(mbar_wait(t1_go, 0, s_abort, DEV_TIMEOUT_TMEM_EMPTY, 50));
        if (ok) {
            tc_fence_after();
            issue_qk(0, kb + 1 == kb1);
        }
        int s = 0;
        uint32_t ph = 0, g = 0;
        bool first = true;  // this unit starts an item: O_t is overwritten, not accumulated
#pragma unroll 1
        while (ok) {
            const int sn = (s + 1 == kKVStages) ? 0 : s + 1;
            const uint32_t phn = (s + 1 == kKVStages) ? ph ^ 1u : ph;
            // the unit after this one
            int nit = it, nkb_ = kb + 1, nkb1 = kb1;
            bool nfirst = false, have_next = true;
            if (nkb_ == kb1) {
                nit = it + 1;
                nfirst = true;
                have_next = nit < n_items;
                if (have_next) {
                    int w;
                    item_at(nit, w, nkb_, nkb1);
                }
            }
            if (have_next) {
                if (!all_ok(mbar_wait(s_free(t), g & 1u, s_abort, DEV_TIMEOUT_TMEM_EMPTY, t))) { ok = false; break; }
                if (NQ == 2 && t == 0 && g == 0 && lane == 0) mbar_arrive(t1_go);  // tile 1 may start (see the gate above)
                if (nfirst && !all_ok(mbar_wait(q_full, (uint32_t)nit & 1u, s_abort, DEV_TIMEOUT_TMA_FULL, 101))) { ok = false; break; }
                if (!all_ok(mbar_wait(k_full(sn), phn, s_abort, DEV_TIMEOUT_TMA_FULL, sn))) { ok = false; break; }
                tc_fence_after();
                issue_qk(sn, nkb_ + 1 == nkb1);
                FBB_TRACE(2 + t, g + 1, 3);
            }
            if (!all_ok(mbar_wait(p_ready(t), g & 1u, s_abort, DEV_TIMEOUT_OTHER, 200 + t))) { ok = false; break; }
            if (!all_ok(mbar_wait(v_full(s), ph, s_abort, DEV_TIMEOUT_TMA_FULL, 16 + s))) { ok = false; break; }
            tc_fence_after();
            FBB_TRACE(2 + t, g, 1);
            const uint64_t vd = vd0 + (uint64_t)(s * (kTileBytes >> 4));
            umma_ts_warp(dO, aP, vd, idesc_pv, first ? 0u : 1u);
#pragma unroll
            for (int k = 1; k < 8; ++k) umma_ts_warp(dO, aP + 8u * k, vd + 128u * k, idesc_pv, 1u);
            umma_commit_warp(pv_done(t));
            umma_commit_warp(v_empty(s));
            FBB_TRACE(2 + t, g, 2);
            if (!have_next) break;
            it = nit;
            kb = nkb_;
            kb1 = nkb1;
            first = nfirst;
            s = sn;
            ph = phn;
            ++g;
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
        const uint32_t tS = tmem_base + ((uint32_t)lane_base << 16) + t * kColTileS;  // this warp's lanes of S_t
        const uint32_t tO = tmem_base + ((uint32_t)lane_base << 16) + kColO + t * kColTileOP;  // ... of O_t; P_t is kColP further
        const float sl = a.scale_log2;
        float mA = -INFINITY, mB = -INFINITY, lA = 0.f, lB = 0.f;  // running maximum and (this thread's share of the) sum
        bool ok = true;
        uint32_t g = 0;  // units done: the phase of the per-tile barriers

#pragma unroll 1
        for (int it = 0; ok && it < n_items; ++it) {
            int n;               // key blocks of this item still to do
            bool to_end;         // the item runs to the group's last key block
            bool warp_has_rows;  // a warp whose 16 rows all lie beyond N (padding of the last tile) only keeps the barriers moving
            {
                int w, kb0, kb1;
                item_at(it, w, kb0, kb1);
                n = kb1 - kb0;
                to_end = kb1 == nkb;
                warp_has_rows = (w % a.groups_per_head) * (FQ * NQ) + t * FQ + lane_base < a.Nq;
            }
            lA = lB = 0.f;
            bool first = true;
#pragma unroll 1
            for (; n > 0; --n, ++g, first = false) {
                if (u == 0) FBB_TRACE(t, g, 0);
                if (!mbar_wait(s_full(t), g & 1u, s_abort, DEV_TIMEOUT_TMEM_FULL, t)) { ok = false; break; }
                tc_fence_after();
                if (u == 0) FBB_TRACE(t, g, 1);
                if (!warp_has_rows) {
                    // This warp only keeps the barriers moving. Its arrival for unit g must wait until the issuer has taken
                    // p_ready of unit g-1 (it commits pv_done right after issuing that unit's P.V): a tile whose warps are
                    // all padding would otherwise complete p_ready for g-1 and for g back to back, and the issuer, which
                    // waits by phase parity, would see the barrier back at the parity it started from and never wake up.
                    // (Working warps are held the same way by their own wait for pv_done before they overwrite P.)
                    // S_t is released at once (the next Q K^T needs no more from this warp; its arrival for unit g + 1 can
                    // only follow S_t(g+1), which the issuer computes after it has seen this unit's release).
                    tc_fence_before();
                    __syncwarp();
                    if (lane == 0) mbar_arrive(s_free(t));
                    if (g > 0 && !mbar_wait(pv_done(t), (g - 1u) & 1u, s_abort, DEV_TIMEOUT_OTHER, 210 + t)) { ok = false; break; }
                    if (lane == 0) mbar_arrive(p_ready(t));
                    continue;
                }
                uint32_t r[64];
                tmem_ld_16x256b_x16(tS, r);
                tmem_wait_ld();
                tc_fence_before();
                __syncwarp();
                if (lane == 0) mbar_arrive(s_free(t));  // S_t is in registers: the next Q K^T may overwrite it
                float va[64];
#pragma unroll
                for (int i = 0; i < 64; ++i) va[i] = __uint_as_float(r[i]);
                if (to_end && n == 1 && (a.N & (FK - 1)) != 0) {  // the group's last key block is ragged: mask keys >= N
                    const int key0 = (nkb - 1) * FK + 2 * cq;
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
                if (u == 0) FBB_TRACE(t, g, 2);
                // ---- running maxima: raised only when this block exceeds them by more than 2^kLazyMax
                if (first) {
                    mA = mxA;
                    mB = mxB;
                } else if (__any_sync(0xffffffffu, mxA > mA + kLazyMax || mxB > mB + kLazyMax)) {
                    // O_t is still being accumulated by the previous unit's P.V
                    if (!mbar_wait(pv_done(t), (g - 1u) & 1u, s_abort, DEV_TIMEOUT_TMEM_FULL, 8 + t)) { ok = false; break; }
                    tc_fence_after();
                    const float nA = fmaxf(mA, mxA), nB = fmaxf(mB, mxB);
                    const float cA = ex2_approx(mA - nA), cB = ex2_approx(mB - nB);
                    // in place, 16 columns at a time: this path is rare, and a whole O tile in registers on top of the
                    // 64 scores held here would make the compiler spill in the hot loop around it
#pragma unroll 1
                    for (int c = 0; c < 4; ++c) {
                        uint32_t o[8];
                        tmem_ld_16x256b_x2(tO + 16u * c, o);
                        tmem_wait_ld();
#pragma unroll
                        for (int k = 0; k < 2; ++k) {
                            o[4 * k] = __float_as_uint(__uint_as_float(o[4 * k]) * cA);
                            o[4 * k + 1] = __float_as_uint(__uint_as_float(o[4 * k + 1]) * cA);
                            o[4 * k + 2] = __float_as_uint(__uint_as_float(o[4 * k + 2]) * cB);
                            o[4 * k + 3] = __float_as_uint(__uint_as_float(o[4 * k + 3]) * cB);
                        }
                        tmem_st_16x256b_x2(tO + 16u * c, o);
                    }
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
                // P_t is read by the previous unit's P.V until that product has completed: waiting here, not before the
                // exponentials, keeps the issue and run time of that product (~900 clocks) off the softmax warps' path
                if (g > 0) {
                    if (!mbar_wait(pv_done(t), (g - 1u) & 1u, s_abort, DEV_TIMEOUT_TMEM_FULL, 8 + t)) { ok = false; break; }
                    tc_fence_after();
                }
                tmem_st_16x128b_x16(tO + kColP, pk);
                if (u == 0) FBB_TRACE(t, g, 3);
                tmem_wait_st();
                tc_fence_before();
                __syncwarp();
                if (lane == 0) mbar_arrive(p_ready(t));
                if (u == 0) FBB_TRACE(t, g, 4);
                lA += accA.x + accA.y;
                lB += accB.x + accB.y;
            }
            if (!ok || !warp_has_rows) continue;

            // ---- end of an item: wait for its last P.V, then write the rows, or hand over / merge a split group
            if (!mbar_wait(pv_done(t), (g - 1u) & 1u, s_abort, DEV_TIMEOUT_TMEM_FULL, 8 + t)) { ok = false; break; }
            tc_fence_after();
            int w, kb0, kb1;
            item_at(it, w, kb0, kb1);
            uint32_t o[32];
            tmem_ld_16x256b_x8(tO, o);
            tmem_wait_ld();
            const int wslot = t * 8 + u;
            if (kb0 > 0) {
                // Another CTA began this group: leave the partial result for it.
                float* dst = a.ws_data + ((size_t)blockIdx.x * kSlotWarps + wslot) * (kSlotValues * 32) + lane;
#pragma unroll
                for (int i = 0; i < 32; ++i) dst[i * 32] = __uint_as_float(o[i]);
                dst[32 * 32] = mA;
                dst[33 * 32] = mB;
                dst[34 * 32] = lA;
                dst[35 * 32] = lB;
                __threadfence();
                __syncwarp();
                if (lane == 0) st_release_gpu(a.ws_flags + (size_t)blockIdx.x * kSlotWarps + wslot, 1u);
                continue;
            }
            if (kb1 != nkb) {
                // The next CTA holds the rest of this group's keys (the first thing it did in its tail share).
                unsigned* flag = a.ws_flags + (size_t)(blockIdx.x + 1u) * kSlotWarps + wslot;
                if (!wait_slot_flag(flag, lane, s_abort, 300 + wslot)) { ok = false; break; }
                const float* src = a.ws_data + ((size_t)(blockIdx.x + 1u) * kSlotWarps + wslot) * (kSlotValues * 32) + lane;
                const float pmA = __ldcg(src + 32 * 32), pmB = __ldcg(src + 33 * 32);
                const float nA = fmaxf(mA, pmA), nB = fmaxf(mB, pmB);
                const float cA = ex2_approx(mA - nA), cB = ex2_approx(mB - nB);
                const float dA = ex2_approx(pmA - nA), dB = ex2_approx(pmB - nB);
#pragma unroll
                for (int k = 0; k < 8; ++k) {
                    o[4 * k] = __float_as_uint(__uint_as_float(o[4 * k]) * cA + __ldcg(src + (4 * k) * 32) * dA);
                    o[4 * k + 1] = __float_as_uint(__uint_as_float(o[4 * k + 1]) * cA + __ldcg(src + (4 * k + 1) * 32) * dA);
                    o[4 * k + 2] = __float_as_uint(__uint_as_float(o[4 * k + 2]) * cB + __ldcg(src + (4 * k + 2) * 32) * dB);
                    o[4 * k + 3] = __float_as_uint(__uint_as_float(o[4 * k + 3]) * cB + __ldcg(src + (4 * k + 3) * 32) * dB);
                }
                lA = lA * cA + __ldcg(src + 34 * 32) * dA;
                lB = lB * cB + __ldcg(src + 35 * 32) * dB;
                __syncwarp();
                if (lane == 0) *flag = 0u;  // the slot is free for the next launch
            }
            // a row's sum is spread over the four threads that share it
            lA += __shfl_xor_sync(0xffffffffu, lA, 1);
            lB += __shfl_xor_sync(0xffffffffu, lB, 1);
            lA += __shfl_xor_sync(0xffffffffu, lA, 2);
            lB += __shfl_xor_sync(0xffffffffu, lB, 2);
            const float invA = 1.f / lA, invB = 1.f / lB;
            const int bh = w / a.groups_per_head;
            const int b = bh / a.H, h = bh - b * a.H;
            const int rowA = (w - bh * a.groups_per_head) * (FQ * NQ) + t * FQ + lane_base + (lane >> 2);  // this thread's rows: rowA, rowA + 8
            __half* dstA = a.o + (int64_t)b * a.o_sb + (int64_t)rowA * a.o_sn + (int64_t)h * a.o_sh + 2 * cq;
            __half* dstB = dstA + 8 * a.o_sn;
#pragma unroll
            for (int k = 0; k < 8; ++k) {
                if (rowA < a.Nq)
                    *reinterpret_cast<uint32_t*>(dstA + 8 * k) = pack_h2(__uint_as_float(o[4 * k]) * invA, __uint_as_float(o[4 * k + 1]) * invA);
                if (rowA + 8 < a.Nq)
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

template <int NQ>
static int launch_flash_variant(const CUtensorMap& tq, const CUtensorMap& tk, const CUtensorMap& tv, FlashArgs a, int B, void* ws,
                                int64_t ws_bytes, cudaStream_t stream) {
    static bool configured[64] = {};
    int dev = 0;
    cudaGetDevice(&dev);
    auto kern = flash64_umma_kernel<NQ>;
    if (dev >= 0 && dev < 64 && !configured[dev]) {
        cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, FlashSmem::kDynamic);
        if (e != cudaSuccess) return fail((int)e, "cudaFuncSetAttribute(flash64_umma_kernel): %s", cudaGetErrorString(e));
        configured[dev] = true;
    }
    a.groups_per_head = (a.Nq + FQ * NQ - 1) / (FQ * NQ);
    a.nkb = (a.N + FK - 1) / FK;
    const int64_t groups = (int64_t)a.groups_per_head * B * a.H;
    if (groups > 0x7FFFFFFFll) return fail(FBB_ERR_SHAPE, "flash64: too many query tiles (%lld)", (long long)groups);
    a.ws_flags = nullptr;
    a.ws_data = nullptr;
    // One CTA per tile group, unless the groups do not fill the SMs evenly and the caller lent a workspace: then one
    // persistent CTA per SM takes whole groups round-robin for all but the last full wave, and an equal share of the
    // (group, key block) units of what is left (between one and two waves' worth, so every share is at least one group
    // long and a group is split over at most two CTAs, which merge through the workspace).
    const int sms = num_sms();
    int64_t ctas = groups;
    a.rounds = 1;
    a.tail_units = 0;
    const bool plain_only = getenv("FBB_FLASH_NO_SPLIT") != nullptr;  // tuning aid: always one CTA per group
    if (groups > sms && groups % sms == 0 && !plain_only) {
        ctas = sms;
        a.rounds = (int)(groups / sms);
    } else if (ws != nullptr && !plain_only && split_pays(groups, sms)) {
        if (ws_bytes < flash64_workspace_bytes()) return fail(FBB_ERR_SHAPE, "flash64: workspace of %lld bytes, %lld needed", (long long)ws_bytes, (long long)flash64_workspace_bytes());
        ctas = sms;
        a.rounds = (int)(groups / sms) - 1;
        a.tail_units = (groups - (int64_t)a.rounds * sms) * a.nkb;
        a.ws_flags = reinterpret_cast<unsigned*>(ws);
        a.ws_data = reinterpret_cast<float*>(reinterpret_cast<uint8_t*>(ws) + flag_region_bytes(sms));
    }
    if ((int64_t)a.rounds * a.nkb + 2 * (int64_t)a.nkb * 2 > 0x7FFFFFFFll) return fail(FBB_ERR_SHAPE, "flash64: too many key blocks per CTA");
    cudaError_t e = launch_pdl(kern, dim3((unsigned)ctas), dim3(128 + 256 * NQ), FlashSmem::kDynamic, stream, tq, tk, tv, a);
    if (e != cudaSuccess) return fail((int)e, "flash64_umma_kernel launch: %s", cudaGetErrorString(e));
    return FBB_OK;
}

#ifdef FBB_FLASH_TRACE
extern "C" int fbb_flash_trace_buffer(void* buf) {
    long long* p = reinterpret_cast<long long*>(buf);
    return (int)cudaMemcpyToSymbol(g_flash_trace, &p, sizeof(p));
}
#endif

// Whether the persistent split form is worth it: the groups do not fill the SMs evenly and the partly filled last wave
// wastes at least 9 % of the whole-wave schedule. Measured, about a third of that waste is recovered (long-lived CTAs
// lose some speed to the two tiles drifting into step), so smaller savings do not pay: 8 % -> -0.6 %, 10 % -> +2.5 %,
// 31 % -> +11 % on whole-model time.
static bool split_pays(int64_t groups, int sms) {
    if (groups <= sms || groups % sms == 0) return false;
    const int64_t whole = (groups + sms - 1) / sms;
    const char* f = getenv("FBB_FLASH_SPLIT_WASTE");  // tuning aid: the least wasted share of the whole-wave schedule that splits
    const double least = f != nullptr ? atof(f) : 0.09;
    return (double)(whole * sms - groups) >= least * (double)(whole * sms);
}

// Two query tiles per CTA once that still gives every SM a CTA; small inputs take one tile per CTA (the small-token path).
static bool two_tiles_per_cta(int B, int N, int H) { return (int64_t)((N + 2 * FQ - 1) / (2 * FQ)) * B * H >= num_sms(); }

int64_t flash64_workspace_bytes() {
    return (int64_t)(flag_region_bytes(num_sms()) + (size_t)num_sms() * kSlotFloats * sizeof(float) + side_region_bytes());
}

// Query rows beyond the last full two-tile group that the side launch takes instead of a tile group of their own
// (0: none): a few rows (cls token, registers), few enough in all and a sequence long enough for the side launch to
// hide behind the tiled one, and the rest still worth two tiles per CTA. FBB_FLASH_NO_SIDE switches it off (tuning and test aid).
static int side_rows_for(int B, int N, int H) {
    const int r = N % (2 * FQ);
    if (r < 1 || r > kSideMaxRows || N <= 2 * FQ || getenv("FBB_FLASH_NO_SIDE") != nullptr || getenv("FBB_FLASH_NO_SPLIT") != nullptr) return 0;
    const int sms = num_sms();
    // The side launch gets four warps per SM (what fits beside the tiled kernel) and each of them is bound by the latency
    // of its loads, so it only hides behind the tiled launch when that is long and the rows are few. Measured on B200
    // (side / tiled only, us): N = 6145, 16 rows 194 / 200; 4097, 12 rows 76.1 / 77.5; 3073, 16 rows 61.5 / 62.6; 2561
    // 47.8 / 47.4; but 6149 (5 rows per head: 80 rows) 308 / 200 and 1281 with 64 rows 63.6 / 55.5.
    if ((int64_t)B * H * r > sms / 8 || N < 3072 || !two_tiles_per_cta(B, N - r, H)) return 0;
    // Only where the tiled launch stays in a persistent form (split, or whole groups in equal rounds). One CTA per group
    // measured 3 % slower per group than the persistent forms at N = 16385, where dropping the 65th group per head would
    // have moved the launch from the split form (1040 groups) to one CTA per group (1024): 1453 against 1430 us.
    const int64_t groups = (int64_t)((N - r) / (2 * FQ)) * B * H;
    if (!(split_pays(groups, sms) || (groups > sms && groups % sms == 0))) return 0;
    return r;
}

int64_t flash64_workspace_bytes_for(int B, int N, int H) {
    if (B <= 0 || N <= 0 || H <= 0 || getenv("FBB_FLASH_NO_SPLIT") != nullptr) return 0;
    const int r = side_rows_for(B, N, H);
    const int nq = two_tiles_per_cta(B, N - r, H) ? 2 : 1;
    const int64_t groups = (int64_t)((N - r + FQ * nq - 1) / (FQ * nq)) * B * H;
    const int sms = num_sms();
    return (r > 0 || split_pays(groups, sms)) ? flash64_workspace_bytes() : 0;
}

int flash64_launches(int B, int N, int H, bool has_workspace) { return (B > 0 && N > 0 && H > 0 && has_workspace && side_rows_for(B, N, H) > 0) ? 2 : 1; }

// The leftover rows [N - rows, N): enqueued right after the tiled launch (see kSideMaxRows).
static int launch_side_rows(const FlashArgs& f, const void* q, const void* k, const void* v, int B, const int64_t* qs, const int64_t* ks,
                            const int64_t* vs, int rows, void* ws, cudaStream_t stream) {
    SideArgs a = {};
    a.q = reinterpret_cast<const __half*>(q);
    a.k = reinterpret_cast<const __half*>(k);
    a.v = reinterpret_cast<const __half*>(v);
    a.o = f.o;
    a.q_sb = qs[0]; a.q_sn = qs[1]; a.q_sh = qs[2];
    a.k_sb = ks[0]; a.k_sn = ks[1]; a.k_sh = ks[2];
    a.v_sb = vs[0]; a.v_sn = vs[1]; a.v_sh = vs[2];
    a.o_sb = f.o_sb; a.o_sn = f.o_sn; a.o_sh = f.o_sh;
    a.N = f.N;
    a.H = f.H;
    a.row0 = f.N - rows;
    a.rows = rows;
    a.scale_log2 = f.scale_log2;
    const int sms = num_sms();
    const int64_t nrows = (int64_t)B * f.H * rows;  // <= sms
    int64_t chunks = (4 * (int64_t)sms) / nrows;     // about four warps per SM
    const int64_t most = (f.N + 63) / 64;            // at least two 32-key steps per chunk
    chunks = chunks > most ? most : chunks;
    chunks = chunks > kSideMaxChunks ? kSideMaxChunks : (chunks < 1 ? 1 : chunks);
    while (nrows * chunks > kSideMaxTasks) --chunks;
    a.chunks = (int)chunks;
    a.tasks = (int)(nrows * chunks);
    uint8_t* w8 = reinterpret_cast<uint8_t*>(ws);
    a.count = reinterpret_cast<unsigned*>(w8 + (size_t)sms * kFlagBytesPerCta);
    a.part = reinterpret_cast<float*>(w8 + flag_region_bytes(sms) + (size_t)sms * kSlotFloats * sizeof(float));
    cudaError_t e = launch_pdl(flash64_side_rows_kernel, dim3((unsigned)((a.tasks + 3) / 4)), dim3(128), 0, stream, a);
    if (e != cudaSuccess) return fail((int)e, "flash64_side_rows_kernel launch: %s", cudaGetErrorString(e));
    return FBB_OK;
}

// Address and size of the built-in workspace on the current device; the address is looked up once per device. Enqueues
// the clearing of its flag words on `stream` (calls share the array, and a launch that gave up a wait may have left some
// raised). No memory is allocated.
int flash64_static_workspace(void** ptr, int64_t* bytes, cudaStream_t stream) {
    static void* addr[64] = {};
    int dev = -1;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return fail((int)e, "cudaGetDevice: %s", cudaGetErrorString(e));
    if (dev < 0 || dev >= 64) return fail(FBB_ERR_SHAPE, "flash64 static workspace: device ordinal %d not supported", dev);
    if (addr[dev] == nullptr) {
        void* p = nullptr;
        e = cudaGetSymbolAddress(&p, g_flash_static_ws);
        if (e != cudaSuccess || p == nullptr) return fail(e != cudaSuccess ? (int)e : FBB_ERR_DRIVER, "cudaGetSymbolAddress(static workspace): %s", cudaGetErrorString(e));
        addr[dev] = p;
    }
    if (flash64_workspace_bytes() > (int64_t)kStaticWsBytes)
        return fail(FBB_ERR_SHAPE, "flash64 static workspace holds %lld bytes (%d SMs), this device needs %lld", (long long)kStaticWsBytes,
                    kStaticMaxSms, (long long)flash64_workspace_bytes());
    e = cudaMemsetAsync(addr[dev], 0, flag_region_bytes(num_sms()), stream);
    if (e != cudaSuccess) return fail((int)e, "cudaMemsetAsync(static workspace flags): %s", cudaGetErrorString(e));
    *ptr = addr[dev];
    *bytes = (int64_t)kStaticWsBytes;
    return FBB_OK;
}

int launch_flash64(const void* q, const void* k, const void* v, void* o, int B, int N, int H, const int64_t* qs,
                   const int64_t* ks, const int64_t* vs, const int64_t* os, float scale, int variant, void* ws, int64_t ws_bytes,
                   cudaStream_t stream) {
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
    FlashArgs a = {};
    a.o = reinterpret_cast<__half*>(o);
    a.N = N;
    a.H = H;
    a.o_sb = os[0];
    a.o_sn = os[1];
    a.o_sh = os[2];
    a.scale_log2 = scale * 1.4426950408889634f;
    (void)variant;  // ff, fh and hh run the same kernel on this part (see the note on variants at the top of the file)
    // leftover rows go to the side launch only when the caller lent a workspace (their partial results live there)
    const int side = ws != nullptr ? side_rows_for(B, N, H) : 0;
    if (side > 0 && ws_bytes < flash64_workspace_bytes())
        return fail(FBB_ERR_SHAPE, "flash64: workspace of %lld bytes, %lld needed", (long long)ws_bytes, (long long)flash64_workspace_bytes());
    a.Nq = N - side;
    int rc;
    if (two_tiles_per_cta(B, a.Nq, H)) rc = launch_flash_variant<2>(tq, tk, tv, a, B, ws, ws_bytes, stream);
    else rc = launch_flash_variant<1>(tq, tk, tv, a, B, ws, ws_bytes, stream);  // (never with side rows: see side_rows_for)
    if (rc != FBB_OK || side == 0) return rc;
    return launch_side_rows(a, q, k, v, B, qs, ks, vs, side, ws, stream);
}

}  // namespace fbb
