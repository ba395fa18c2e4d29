// Shared device helpers for the sm_100a kernels: mbarrier, TMA, tcgen05 (UMMA + tensor memory) wrappers.
// Every wait in here is bounded: a wait that runs out records a code in g_fbb_status and returns false so the
// calling kernel can wind down (free its tensor memory, return) instead of spinning on a shared GPU.
#pragma once
#include <cuda.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace fbb {

// ---------------------------------------------------------------------------------------------- device status word
// [0] first error code (0 = none), [1] detail (barrier id / stage), [2] block index, [3] count of errors.
// Read and cleared by fbb_device_status(); kernels only ever write to it when a bounded wait gives up.
__device__ unsigned int g_fbb_status[4] = {0u, 0u, 0u, 0u};

enum DeviceError : unsigned int {
    DEV_OK = 0,
    DEV_TIMEOUT_TMA_FULL = 1,    // consumer never saw a TMA stage arrive
    DEV_TIMEOUT_SMEM_EMPTY = 2,  // producer never got a stage back
    DEV_TIMEOUT_TMEM_FULL = 3,   // epilogue / softmax never saw the MMA commit
    DEV_TIMEOUT_TMEM_EMPTY = 4,  // MMA issuer never got an accumulator back
    DEV_TIMEOUT_OTHER = 5,
};

#ifdef FBB_DEBUG_WAITS
// Development aid: every wait that gives up or is cut short by the abort flag logs (code, detail, block, warp, parity).
__device__ unsigned int g_fbb_debug_n = 0;
__device__ unsigned int g_fbb_debug[256][5];
__device__ __forceinline__ void debug_log_wait(unsigned int code, unsigned int detail, unsigned int parity) {
    if ((threadIdx.x & 31) != 0) return;
    const unsigned int i = atomicAdd(&g_fbb_debug_n, 1u);
    if (i < 256) {
        g_fbb_debug[i][0] = code; g_fbb_debug[i][1] = detail; g_fbb_debug[i][2] = blockIdx.x; g_fbb_debug[i][3] = threadIdx.x >> 5; g_fbb_debug[i][4] = parity;
    }
}
#endif
__device__ __forceinline__ void report_error(unsigned int code, unsigned int detail) {
    if (atomicCAS(&g_fbb_status[0], 0u, code) == 0u) {
        g_fbb_status[1] = detail;
        g_fbb_status[2] = blockIdx.x + blockIdx.y * gridDim.x;
    }
    atomicAdd(&g_fbb_status[3], 1u);
}

// ---------------------------------------------------------------------------------------------- misc
__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ uint64_t globaltimer_ns() {
    uint64_t t;
    asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
    return t;
}


// Warpgroup-wide register reallocation (all four warps of an aligned warpgroup execute the same one).
template <int N>
__device__ __forceinline__ void setmaxnreg_inc() { asm volatile("setmaxnreg.inc.sync.aligned.u32 %0;" ::"n"(N)); }
template <int N>
__device__ __forceinline__ void setmaxnreg_dec() { asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;" ::"n"(N)); }

// Programmatic dependent launch: a kernel launched with the programmatic-serialization attribute may start while the
// previous kernel of the stream is still draining; everything before this wait (barrier set-up, tensor-memory
// allocation, descriptor prefetch) overlaps that tail, everything after it sees the previous kernel's memory.
// Without the attribute the instruction does nothing.
__device__ __forceinline__ void grid_dependency_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
// Lets the NEXT kernel of the stream (launched with the same attribute) be scheduled as soon as every CTA of this grid
// has executed this or exited, instead of at the end of the grid: its CTAs then start on each SM as this grid's CTAs
// leave it, and their set-up runs under this grid's tail. The next kernel still sees this grid's memory only after its
// own griddepcontrol.wait, which returns when this grid has completed. Every kernel here issues it right after its own
// wait: nothing a kernel does before its wait touches global memory.
__device__ __forceinline__ void grid_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

// ---------------------------------------------------------------------------------------------- mbarrier
__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void fence_barrier_init() {
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void mbar_arrive_expect_tx(uint32_t bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t"
        ".reg .pred P1;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 P1, [%1], %2;\n\t"
        "selp.b32 %0, 1, 0, P1;\n\t"
        "}\n"
        : "=r"(ok)
        : "r"(bar), "r"(parity)
        : "memory");
    return ok != 0;
}


// Wait limit: 2 s of wall time (checked every 256 polls). A healthy pipeline never comes near it.
#ifdef FBB_DEBUG_WAITS
constexpr uint64_t kWaitLimitNs = 20000000ull;
#else
constexpr uint64_t kWaitLimitNs = 2000000000ull;
#endif

// Returns true when the phase with `parity` completed; false after `limit_ns` (error recorded, *abort set).
__device__ __forceinline__ bool mbar_wait_limit(uint32_t bar, uint32_t parity, volatile int* abort_flag, unsigned int code,
                                                unsigned int detail, uint64_t limit_ns) {
    if (mbar_try_wait(bar, parity)) return true;
    uint64_t t0 = globaltimer_ns();
    for (;;) {
#pragma unroll 1
        for (int i = 0; i < 256; ++i)
            if (mbar_try_wait(bar, parity)) return true;
#ifdef FBB_DEBUG_WAITS
        if (*abort_flag) { debug_log_wait(code, detail, parity); return false; }
#else
        if (*abort_flag) return false;
#endif
        if (globaltimer_ns() - t0 > limit_ns) {
#ifdef FBB_DEBUG_WAITS
            debug_log_wait(code + 100u, detail, parity);
#endif
            report_error(code, detail);
            *abort_flag = 1;
            __threadfence_block();
            return false;
        }
    }
}
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, volatile int* abort_flag, unsigned int code,
                                          unsigned int detail) {
    return mbar_wait_limit(bar, parity, abort_flag, code, detail, kWaitLimitNs);
}

// ---------------------------------------------------------------------------------------------- proxies / fences
__device__ __forceinline__ void fence_proxy_async_smem() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void named_bar_sync(int id, int nthreads) {
    asm volatile("bar.sync %0, %1;" ::"r"(id), "r"(nthreads) : "memory");
}

// ---------------------------------------------------------------------------------------------- TMA (no multicast)
__device__ __forceinline__ void tma_prefetch_desc(const void* map) {
    asm volatile("prefetch.tensormap [%0];" ::"l"(map) : "memory");
}
__device__ __forceinline__ void tma_load_2d(uint32_t dst, const void* map, uint32_t bar, int c0, int c1) {
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
        ::"r"(dst), "l"(map), "r"(bar), "r"(c0), "r"(c1)
        : "memory");
}
__device__ __forceinline__ void tma_load_4d(uint32_t dst, const void* map, uint32_t bar, int c0, int c1, int c2, int c3) {
    asm volatile(
        "cp.async.bulk.tensor.4d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5, %6}], [%2];"
        ::"r"(dst), "l"(map), "r"(bar), "r"(c0), "r"(c1), "r"(c2), "r"(c3)
        : "memory");
}

// Tile store shared -> global through a tensor map (rows / columns outside the tensor are clipped by the hardware).
__device__ __forceinline__ void tma_store_2d(const void* map, uint32_t src, int c0, int c1) {
    asm volatile("cp.async.bulk.tensor.2d.global.shared::cta.bulk_group [%0, {%2, %3}], [%1];" ::"l"(map), "r"(src), "r"(c0), "r"(c1)
                 : "memory");
}
__device__ __forceinline__ void bulk_commit() { asm volatile("cp.async.bulk.commit_group;" ::: "memory"); }
// Until the bulk stores committed by this thread have finished READING shared memory (the buffer may be rewritten).
__device__ __forceinline__ void bulk_wait_read_all() { asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory"); }
// Until the bulk stores committed by this thread have completed.
__device__ __forceinline__ void bulk_wait_all() { asm volatile("cp.async.bulk.wait_group 0;" ::: "memory"); }

// ---------------------------------------------------------------------------------------------- tensor memory
template <int NCOLS>
__device__ __forceinline__ void tmem_alloc(uint32_t smem_dst) {  // one full warp
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_dst), "n"(NCOLS) : "memory");
}
__device__ __forceinline__ void tmem_relinquish() {
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
template <int NCOLS>
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr) {  // one full warp
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "n"(NCOLS) : "memory");
}

// 32 lanes x 32 columns of 32-bit: thread t of the warp gets lane (warp%4)*32+t, registers = consecutive columns.
__device__ __forceinline__ void tmem_ld32(uint32_t taddr, uint32_t* r) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
        "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
          "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]),
          "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]),
          "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
        : "r"(taddr)
        : "memory");
}
// 16-lane shapes: the warp touches 16 tensor-memory lanes starting at the lane in the address. Register layout (checked on
// hardware): 16x256b.xN -> thread t holds r[4k+j]: lane t/4 + 8*(j/2), column 8k + 2*(t%4) + j%2 (the mma m16n8 accumulator
// fragment); 16x128b.xN -> r[2k+j]: lane t/4 + 8*j, column 4k + t%4.
__device__ __forceinline__ void tmem_ld_16x256b_x16(uint32_t taddr, uint32_t* r) {
    asm volatile("tcgen05.ld.sync.aligned.16x256b.x16.b32 {%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31, %32, %33, %34, %35, %36, %37, %38, %39, %40, %41, %42, %43, %44, %45, %46, %47, %48, %49, %50, %51, %52, %53, %54, %55, %56, %57, %58, %59, %60, %61, %62, %63}, [%64];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31]), "=r"(r[32]), "=r"(r[33]), "=r"(r[34]), "=r"(r[35]), "=r"(r[36]), "=r"(r[37]), "=r"(r[38]), "=r"(r[39]), "=r"(r[40]), "=r"(r[41]), "=r"(r[42]), "=r"(r[43]), "=r"(r[44]), "=r"(r[45]), "=r"(r[46]), "=r"(r[47]), "=r"(r[48]), "=r"(r[49]), "=r"(r[50]), "=r"(r[51]), "=r"(r[52]), "=r"(r[53]), "=r"(r[54]), "=r"(r[55]), "=r"(r[56]), "=r"(r[57]), "=r"(r[58]), "=r"(r[59]), "=r"(r[60]), "=r"(r[61]), "=r"(r[62]), "=r"(r[63])
        : "r"(taddr)
        : "memory");
}
__device__ __forceinline__ void tmem_ld_16x256b_x8(uint32_t taddr, uint32_t* r) {
    asm volatile("tcgen05.ld.sync.aligned.16x256b.x8.b32 {%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
        : "r"(taddr)
        : "memory");
}
__device__ __forceinline__ void tmem_st_16x256b_x8(uint32_t taddr, const uint32_t* r) {
    asm volatile("tcgen05.st.sync.aligned.16x256b.x8.b32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31, %32};"
        ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]), "r"(r[8]), "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]), "r"(r[16]), "r"(r[17]), "r"(r[18]), "r"(r[19]), "r"(r[20]), "r"(r[21]), "r"(r[22]), "r"(r[23]), "r"(r[24]), "r"(r[25]), "r"(r[26]), "r"(r[27]), "r"(r[28]), "r"(r[29]), "r"(r[30]), "r"(r[31])
        : "memory");
}
// 16 columns at a time (8 registers): for the rare in-place rescale of O, which must not hold a whole tile in registers
__device__ __forceinline__ void tmem_ld_16x256b_x2(uint32_t taddr, uint32_t* r) {
    asm volatile("tcgen05.ld.sync.aligned.16x256b.x2.b32 {%0, %1, %2, %3, %4, %5, %6, %7}, [%8];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7])
        : "r"(taddr)
        : "memory");
}
__device__ __forceinline__ void tmem_st_16x256b_x2(uint32_t taddr, const uint32_t* r) {
    asm volatile("tcgen05.st.sync.aligned.16x256b.x2.b32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8};"
        ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7])
        : "memory");
}
__device__ __forceinline__ void tmem_st_16x128b_x16(uint32_t taddr, const uint32_t* r) {
    asm volatile("tcgen05.st.sync.aligned.16x128b.x16.b32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31, %32};"
        ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]), "r"(r[8]), "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]), "r"(r[16]), "r"(r[17]), "r"(r[18]), "r"(r[19]), "r"(r[20]), "r"(r[21]), "r"(r[22]), "r"(r[23]), "r"(r[24]), "r"(r[25]), "r"(r[26]), "r"(r[27]), "r"(r[28]), "r"(r[29]), "r"(r[30]), "r"(r[31])
        : "memory");
}
__device__ __forceinline__ void tmem_wait_ld() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }
__device__ __forceinline__ void tmem_wait_st() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }

// ---------------------------------------------------------------------------------------------- UMMA descriptors
// Shared-memory operand descriptor (64 bit): start address >> 4 in [0,14), leading byte offset >> 4 in [16,30),
// stride byte offset >> 4 in [32,46), descriptor version 1 in [46,48), swizzle mode in [61,64) (2 = 128-byte swizzle).
// 128-byte-swizzled tiles made of 128-byte rows (what a TMA box with a 128-byte inner extent and SWIZZLE_128B
// writes): 8 consecutive rows form one 1024-byte swizzle atom, so the offset between 8-row groups is 1024 bytes.
//  * K-major operand (rows = M or N index, the 128 bytes of a row = 64 fp16 along K): SBO = 1024, LBO unused.
//    One UMMA consumes 16 elements of K = 32 bytes, so the k-th UMMA inside the tile starts 32*k bytes further.
//  * MN-major operand (rows = K index, the 128 bytes of a row = 64 fp16 along M or N): SBO = 1024 is the offset
//    between groups of 8 K-rows, LBO is the offset between 64-element groups along MN (unused when MN extent = 64).
//    One UMMA consumes 16 K-rows = 2048 bytes.
constexpr uint64_t kSwizzle128 = 2ull;
__host__ __device__ constexpr uint64_t make_smem_desc_hi(uint32_t lbo_bytes, uint32_t sbo_bytes) {
    return ((uint64_t)((lbo_bytes >> 4) & 0x3FFF) << 16) | ((uint64_t)((sbo_bytes >> 4) & 0x3FFF) << 32) | (1ull << 46) |
           (kSwizzle128 << 61);
}
__device__ __forceinline__ uint64_t smem_desc(uint32_t saddr, uint64_t hi_bits) {
    return hi_bits | (uint64_t)((saddr >> 4) & 0x3FFF);
}

// Instruction descriptor for kind::f16 (fp16 A and B): accumulator format in [4,6) (0 = f16, 1 = f32), A/B formats
// in [7,10)/[10,13) (0 = fp16), A/B major in bit 15/16 (0 = K-major, 1 = MN-major), N>>3 in [17,23), M>>4 in [24,29).
__host__ __device__ constexpr uint32_t make_idesc_f16(int M, int N, bool acc_f32, bool a_mn_major, bool b_mn_major) {
    return ((acc_f32 ? 1u : 0u) << 4) | ((a_mn_major ? 1u : 0u) << 15) | ((b_mn_major ? 1u : 0u) << 16) |
           ((uint32_t)(N >> 3) << 17) | ((uint32_t)(M >> 4) << 24);
}


// Warp-collective forms: every lane of a converged warp executes the call, one elected lane issues the instruction.
// Keeping the issuing code warp-uniform lets the compiler hold descriptors and addresses in uniform registers, which is
// what keeps the per-instruction issue cost of a long UMMA sequence low.
__device__ __forceinline__ void umma_ss_warp(uint32_t d_tmem, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t"
        ".reg .pred p, q;\n\t"
        "elect.sync _|q, 0xFFFFFFFF;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "@q tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t"
        "}\n"
        ::"r"(d_tmem), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
        : "memory");
}
__device__ __forceinline__ void umma_ts_warp(uint32_t d_tmem, uint32_t a_tmem, uint64_t bdesc, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t"
        ".reg .pred p, q;\n\t"
        "elect.sync _|q, 0xFFFFFFFF;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "@q tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n\t"
        "}\n"
        ::"r"(d_tmem), "r"(a_tmem), "l"(bdesc), "r"(idesc), "r"(accumulate)
        : "memory");
}
__device__ __forceinline__ void umma_commit_warp(uint32_t bar) {
    asm volatile(
        "{\n\t"
        ".reg .pred q;\n\t"
        "elect.sync _|q, 0xFFFFFFFF;\n\t"
        "@q tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];\n\t"
        "}\n"
        ::"r"(bar)
        : "memory");
}

// ---------------------------------------------------------------------------------------------- CTA pairs (cta_group::2)
// Two CTAs of a cluster work on one 256-row UMMA: each holds its 128 rows of A and its half of the B rows in its own
// shared memory, the leader (cluster rank 0) issues the instruction, each CTA's tensor memory receives its 128 rows
// of D. No load is multicast: every CTA fetches its own operands; only barrier signals cross the pair.
__device__ __forceinline__ uint32_t cluster_ctarank() {
    uint32_t r;
    asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
    return r;
}
__device__ __forceinline__ void cluster_sync_all() {
    asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
    asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
}
// Arrive (count 1) on the barrier at the same shared-memory offset in CTA `rank` of the cluster.
__device__ __forceinline__ void mbar_arrive_remote(uint32_t bar, uint32_t rank) {
    asm volatile(
        "{\n\t"
        ".reg .b32 ra;\n\t"
        "mapa.shared::cluster.u32 ra, %0, %1;\n\t"
        "mbarrier.arrive.release.cluster.shared::cluster.b64 _, [ra];\n\t"
        "}\n"
        ::"r"(bar), "r"(rank)
        : "memory");
}
// TMA tile load of a CTA pair member: data lands in this CTA's shared memory, the byte count is credited to the LEADER's
// barrier (same offset, cluster rank 0: the CTA-rank bit of the shared::cluster address cleared).
__device__ __forceinline__ void tma_load_2d_pair(uint32_t dst, const void* map, uint32_t bar, int c0, int c1) {
    asm volatile(
        "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
        ::"r"(dst), "l"(map), "r"(bar & 0xFEFFFFFFu), "r"(c0), "r"(c1)
        : "memory");
}
template <int NCOLS>
__device__ __forceinline__ void tmem_alloc_pair(uint32_t smem_dst) {  // one full warp in EACH CTA of the pair
    asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_dst), "n"(NCOLS) : "memory");
}
__device__ __forceinline__ void tmem_relinquish_pair() {
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
}
template <int NCOLS>
__device__ __forceinline__ void tmem_dealloc_pair(uint32_t taddr) {
    asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(taddr), "n"(NCOLS) : "memory");
}
__device__ __forceinline__ void umma_ss_pair_warp(uint32_t d_tmem, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t"
        ".reg .pred p, q;\n\t"
        "elect.sync _|q, 0xFFFFFFFF;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "@q tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n\t"
        "}\n"
        ::"r"(d_tmem), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
        : "memory");
}
// Arrive on the barrier at this offset in BOTH CTAs of the pair once the UMMAs issued so far have completed.
__device__ __forceinline__ void umma_commit_pair_warp(uint32_t bar) {
    asm volatile(
        "{\n\t"
        ".reg .pred q;\n\t"
        ".reg .b16 m;\n\t"
        "mov.b16 m, 3;\n\t"
        "elect.sync _|q, 0xFFFFFFFF;\n\t"
        "@q tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], m;\n\t"
        "}\n"
        ::"r"(bar)
        : "memory");
}

// The same for a pair inside a larger cluster: `mask` has the bits of the two CTAs' ranks in the cluster.
__device__ __forceinline__ void umma_commit_pair_mask_warp(uint32_t bar, uint32_t mask) {
    asm volatile(
        "{\n\t"
        ".reg .pred q;\n\t"
        ".reg .b16 m;\n\t"
        "cvt.u16.u32 m, %1;\n\t"
        "elect.sync _|q, 0xFFFFFFFF;\n\t"
        "@q tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], m;\n\t"
        "}\n"
        ::"r"(bar), "r"(mask)
        : "memory");
}
// Two floats from the shared memory of CTA `rank` of this cluster, at the offset `addr` has in this CTA (distributed
// shared memory; the data must have been published by a cluster barrier).
__device__ __forceinline__ float2 ld_cluster_f32x2(uint32_t addr, uint32_t rank) {
    float2 v;
    asm volatile(
        "{\n\t"
        ".reg .b32 ra;\n\t"
        "mapa.shared::cluster.u32 ra, %2, %3;\n\t"
        "ld.shared::cluster.v2.f32 {%0, %1}, [ra];\n\t"
        "}\n"
        : "=f"(v.x), "=f"(v.y)
        : "r"(addr), "r"(rank)
        : "memory");
    return v;
}

// ---------------------------------------------------------------------------------------------- math
__device__ __forceinline__ float ex2_approx(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}
// Two fp32 FMAs in one instruction (packed f32x2 pipe of sm_100): d = a * b + c element-wise.
__device__ __forceinline__ float2 ffma2(float2 a, float2 b, float2 c) {
    float2 d;
    asm("{\n\t"
        ".reg .b64 ra, rb, rc, rd;\n\t"
        "mov.b64 ra, {%2, %3};\n\t"
        "mov.b64 rb, {%4, %5};\n\t"
        "mov.b64 rc, {%6, %7};\n\t"
        "fma.rn.f32x2 rd, ra, rb, rc;\n\t"
        "mov.b64 {%0, %1}, rd;\n\t"
        "}\n"
        : "=f"(d.x), "=f"(d.y)
        : "f"(a.x), "f"(a.y), "f"(b.x), "f"(b.y), "f"(c.x), "f"(c.y));
    return d;
}
__device__ __forceinline__ float2 fadd2(float2 a, float2 b) {
    float2 d;
    asm("{\n\t"
        ".reg .b64 ra, rb, rd;\n\t"
        "mov.b64 ra, {%2, %3};\n\t"
        "mov.b64 rb, {%4, %5};\n\t"
        "add.rn.f32x2 rd, ra, rb;\n\t"
        "mov.b64 {%0, %1}, rd;\n\t"
        "}\n"
        : "=f"(d.x), "=f"(d.y)
        : "f"(a.x), "f"(a.y), "f"(b.x), "f"(b.y));
    return d;
}
__device__ __forceinline__ float fmax3(float a, float b, float c) {
    float d;
    asm("max.f32 %0, %1, %2, %3;" : "=f"(d) : "f"(a), "f"(b), "f"(c));
    return d;
}
// 2^x for a pair of values on the FMA / ALU pipes instead of the 16-lane-per-SM transcendental unit: round-to-nearest
// range reduction with the 1.5 * 2^23 trick (the low mantissa bits of x + magic hold round(x)), a degree-3 polynomial for
// 2^f on [-0.5, 0.5] (max relative error 7.5e-5, a quarter of one fp16 rounding), and the integer part added into the
// exponent field. Inputs below -126 are clamped (the result is then ~1e-38, i.e. zero for the softmax).
__device__ __forceinline__ float2 exp2_emulated(float2 x) {
    const float kMagic = 12582912.0f;
    x.x = fmaxf(x.x, -126.0f);
    x.y = fmaxf(x.y, -126.0f);
    const float2 xm = fadd2(x, make_float2(kMagic, kMagic));
    const float2 n = fadd2(xm, make_float2(-kMagic, -kMagic));
    const float2 f = ffma2(n, make_float2(-1.0f, -1.0f), x);
    float2 p = ffma2(f, make_float2(0.05517163872718811f, 0.05517163872718811f), make_float2(0.2426111251115799f, 0.2426111251115799f));
    p = ffma2(p, f, make_float2(0.6932609677314758f, 0.6932609677314758f));
    p = ffma2(p, f, make_float2(0.9999280571937561f, 0.9999280571937561f));
    p.x = __int_as_float(__float_as_int(p.x) + (__float_as_int(xm.x) << 23));
    p.y = __int_as_float(__float_as_int(p.y) + (__float_as_int(xm.y) << 23));
    return p;
}
__device__ __forceinline__ uint32_t pack_h2(float lo, float hi) {
    __half2 h = __floats2half2_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&h);
}
__device__ __forceinline__ float2 fmul2(float2 a, float2 b) {
    float2 d;
    asm("{\n\t"
        ".reg .b64 ra, rb, rd;\n\t"
        "mov.b64 ra, {%2, %3};\n\t"
        "mov.b64 rb, {%4, %5};\n\t"
        "mul.rn.f32x2 rd, ra, rb;\n\t"
        "mov.b64 {%0, %1}, rd;\n\t"
        "}\n"
        : "=f"(d.x), "=f"(d.y)
        : "f"(a.x), "f"(a.y), "f"(b.x), "f"(b.y));
    return d;
}
// Exact (erf) GELU, branch-free, for a pair of values: x * Phi(x) with Phi from the complementary error function of
// z = |x| / sqrt(2) in the form erfc(z) = (1 + a1 z + ... + a6 z^6)^-16 (Abramowitz & Stegun 7.1.28, |error| <= 3e-7).
// With the coefficients scaled by 2^(1/16) the sixteenth power is 2 / erfc(z), so one reciprocal gives q = erfc(z) / 2 and
// x > 0 -> x - x q, x <= 0 -> x q, i.e. max(x, 0) - |x q| (no 1 - erf cancellation in the negative tail; a power that
// overflows gives q = 0, the right limit). Against float64 erf-GELU: max abs error 7.1e-7 over [-12, 12], below 1e-2 of an
// fp16 rounding of the result except around x = -4 (results ~1e-4, up to 8 fp16 steps). Six packed FMAs, five packed
// multiplies and ONE transcendental (the reciprocal) per value: the form with exp(-z^2) needed two, and the 16-lane
// transcendental unit is what the GELU epilogue of a 128 x 256 tile waits for.
__device__ __forceinline__ float2 gelu_erf2(float2 x) {
    const float2 z = make_float2(fabsf(x.x) * 0.70710678118654752440f, fabsf(x.y) * 0.70710678118654752440f);
    float2 p = ffma2(z, make_float2(4.49703984e-05f, 4.49703984e-05f), make_float2(0.000288811862f, 0.000288811862f));
    p = ffma2(p, z, make_float2(0.000158744544f, 0.000158744544f));
    p = ffma2(p, z, make_float2(0.00968096871f, 0.00968096871f));
    p = ffma2(p, z, make_float2(0.0441539958f, 0.0441539958f));
    p = ffma2(p, z, make_float2(0.0736454055f, 0.0736454055f));
    p = ffma2(p, z, make_float2(1.04427373f, 1.04427373f));
    p = fmul2(p, p);
    p = fmul2(p, p);
    p = fmul2(p, p);
    p = fmul2(p, p);
    float2 q;
    asm("rcp.approx.ftz.f32 %0, %1;" : "=f"(q.x) : "f"(p.x));
    asm("rcp.approx.ftz.f32 %0, %1;" : "=f"(q.y) : "f"(p.y));
    const float2 h = fmul2(x, q);
    return make_float2(fmaxf(x.x, 0.f) - fabsf(h.x), fmaxf(x.y, 0.f) - fabsf(h.y));
}
__device__ __forceinline__ float gelu_erf(float x) { return gelu_erf2(make_float2(x, x)).x; }
// v * sigmoid(v) with two transcendentals (ex2, reciprocal) and two FMAs; an IEEE division here costs ten instructions per
// value in the SwiGLU epilogue. exp(-v) overflowing to inf gives 1 / inf = 0, the right limit.
__device__ __forceinline__ float silu(float v) {
    float r;
    asm("rcp.approx.ftz.f32 %0, %1;" : "=f"(r) : "f"(1.0f + ex2_approx(v * -1.4426950408889634f)));
    return v * r;
}

}  // namespace fbb
