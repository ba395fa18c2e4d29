// The extern "C" surface of libfastbb_b200.so: argument validation on the host, then one launch per call.
#include <cstdarg>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <mutex>

#include "common.cuh"
#include "internal.h"

namespace fbb {

static thread_local char t_last_error[512] = "";

int fail(int status, const char* fmt, ...) {
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(t_last_error, sizeof(t_last_error), fmt, ap);
    va_end(ap);
    return status;
}

EncodeTiledFn encode_tiled_fn() {
    static EncodeTiledFn fn = []() -> EncodeTiledFn {
        void* p = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) != cudaSuccess) return nullptr;
        if (q != cudaDriverEntryPointSuccess) return nullptr;
        return reinterpret_cast<EncodeTiledFn>(p);
    }();
    return fn;
}

// Encoded tensor maps are kept in a small direct-mapped table: a map is a pure function of (base, rank, dims, strides,
// box, swizzle), so a hit can never be stale, and a block stack asks for the same few dozen maps on every call (the
// driver call costs microseconds, which is what an eager small-model forward is made of). The table is the one piece of
// mutable state shared between calls; a mutex guards it.
namespace {
struct TmapKey {
    const void* base;
    uint64_t dims[4];
    int64_t strides[4];
    uint32_t box[4];
    int rank, swizzle;
    bool operator==(const TmapKey& o) const { return memcmp(this, &o, sizeof(TmapKey)) == 0; }
};
struct TmapEntry {
    TmapKey key;
    CUtensorMap map;
    bool used;
};
constexpr int kTmapSlots = 2048;
TmapEntry g_tmap_cache[kTmapSlots];
std::mutex g_tmap_mutex;
uint64_t tmap_hash(const TmapKey& k) {
    uint64_t h = 1469598103934665603ull;
    const unsigned char* p = reinterpret_cast<const unsigned char*>(&k);
    for (size_t i = 0; i < sizeof(TmapKey); ++i) h = (h ^ p[i]) * 1099511628211ull;
    return h;
}
}  // namespace

int make_tmap_f16(CUtensorMap* map, const void* base, int rank, const uint64_t* dims, const int64_t* strides_elems,
                  const uint32_t* box, CUtensorMapSwizzle swizzle) {
    EncodeTiledFn enc = encode_tiled_fn();
    if (enc == nullptr) return fail(FBB_ERR_DRIVER, "cuTensorMapEncodeTiled is not available from this driver");
    if (rank < 1 || rank > 4) return fail(FBB_ERR_SHAPE, "tensor map rank %d not supported", rank);
    TmapKey key;
    memset(&key, 0, sizeof(key));  // padding bytes too: the key is compared and hashed as raw bytes
    key.base = base;
    key.rank = rank;
    key.swizzle = (int)swizzle;
    for (int i = 0; i < rank; ++i) {
        key.dims[i] = dims[i];
        key.strides[i] = i > 0 ? strides_elems[i] : 1;
        key.box[i] = box[i];
    }
    TmapEntry& slot = g_tmap_cache[tmap_hash(key) % kTmapSlots];
    {
        std::lock_guard<std::mutex> lock(g_tmap_mutex);
        if (slot.used && slot.key == key) {
            *map = slot.map;
            return FBB_OK;
        }
    }
    cuuint64_t gdim[5];
    cuuint64_t gstr[4];
    cuuint32_t bx[5];
    cuuint32_t es[5];
    for (int i = 0; i < rank; ++i) {
        gdim[i] = dims[i];
        bx[i] = box[i];
        es[i] = 1;
        if (i > 0) gstr[i - 1] = (cuuint64_t)strides_elems[i] * 2u;
    }
    CUresult r = enc(map, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, (cuuint32_t)rank, const_cast<void*>(base), gdim, gstr, bx, es,
                     CU_TENSOR_MAP_INTERLEAVE_NONE, swizzle, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                     CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return fail(FBB_ERR_DRIVER, "cuTensorMapEncodeTiled failed with CUresult %d", (int)r);
    std::lock_guard<std::mutex> lock(g_tmap_mutex);
    slot.key = key;
    slot.map = *map;
    slot.used = true;
    return FBB_OK;
}

int num_sms() {
    static int cached[64] = {};
    int dev = 0;
    cudaGetDevice(&dev);
    if (dev < 0 || dev >= 64) dev = 0;
    if (cached[dev] == 0) {
        int n = 0;
        cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev);
        cached[dev] = n > 0 ? n : 148;
    }
    return cached[dev];
}

bool pdl_enabled() {
    static const bool on = []() {
        const char* e = getenv("FBB_NO_PDL");
        return !(e != nullptr && e[0] == '1');
    }();
    return on;
}

static bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

// Diagnostics. wait_timeout_probe_kernel: one warp initialises an mbarrier that nothing ever arrives on and waits for it
// with the library's bounded wait and a caller-given limit; the wait gives up, records DEV_TIMEOUT_OTHER with `detail`
// in the status word and the kernel returns normally. This is the path every pipeline wait takes when it runs out.
__global__ void wait_timeout_probe_kernel(unsigned long long limit_ns, unsigned int detail, unsigned int* gave_up) {
    __shared__ __align__(8) uint64_t bar;
    __shared__ int abort_flag;
    if (threadIdx.x == 0) {
        mbar_init(smem_u32(&bar), 1);
        abort_flag = 0;
        fence_barrier_init();
    }
    __syncwarp();
    if (threadIdx.x == 0) {
        const bool done = mbar_wait_limit(smem_u32(&bar), 0u, &abort_flag, DEV_TIMEOUT_OTHER, detail, limit_ns);
        if (gave_up != nullptr) *gave_up = done ? 0u : 1u;
    }
}

// sm_clock_probe_kernel: one thread counts `spin_clocks` SM clocks against the nanosecond timer and stores the ratio in
// MHz: the SM clock the kernels around it on the stream actually ran at (the driver's sampled clock reading is too
// coarse to tell a power-capped stretch of a few milliseconds from an uncapped one).
__global__ void sm_clock_probe_kernel(float* out_mhz, long long spin_clocks) {
    const uint64_t t0 = globaltimer_ns();
    const long long c0 = clock64();
    long long c1 = c0;
    while (c1 - c0 < spin_clocks) c1 = clock64();  // ends after spin_clocks clocks: the counter always advances
    const uint64_t t1 = globaltimer_ns();
    *out_mhz = t1 > t0 ? (float)((double)(c1 - c0) * 1000.0 / (double)(t1 - t0)) : 0.f;
}

}  // namespace fbb

using namespace fbb;

extern "C" {

int fbb_version(void) { return FBB_VERSION; }

const char* fbb_status_string(int status) {
    switch (status) {
        case FBB_OK: return "ok";
        case FBB_ERR_NULL: return "a required pointer is null";
        case FBB_ERR_SHAPE: return "unsupported size or leading dimension";
        case FBB_ERR_ALIGN: return "pointer or stride is not 16-byte aligned";
        case FBB_ERR_ENUM: return "unknown enum value";
        case FBB_ERR_DRIVER: return "CUDA driver tensor-map entry point failed";
        case FBB_ERR_DEVICE_WAIT: return "a kernel gave up a bounded wait";
        default: return status > 0 ? cudaGetErrorString((cudaError_t)status) : "unknown status";
    }
}

const char* fbb_last_error(void) { return t_last_error; }

int fbb_device_status(unsigned int out[4]) {
    if (out == nullptr) return fail(FBB_ERR_NULL, "fbb_device_status: out is null");
    cudaError_t e = cudaDeviceSynchronize();
    if (e != cudaSuccess) return fail((int)e, "fbb_device_status: %s", cudaGetErrorString(e));
    e = cudaMemcpyFromSymbol(out, g_fbb_status, sizeof(unsigned int) * 4);
    if (e != cudaSuccess) return fail((int)e, "fbb_device_status: %s", cudaGetErrorString(e));
    if (out[0] != 0u || out[3] != 0u) {
        const unsigned int zero[4] = {0u, 0u, 0u, 0u};
        cudaMemcpyToSymbol(g_fbb_status, zero, sizeof(zero));
        return fail(FBB_ERR_DEVICE_WAIT, "device wait ran out: code %u detail %u block %u (%u reports)", out[0], out[1],
                    out[2], out[3]);
    }
    return FBB_OK;
}

#ifndef FBB_FLASH_ONLY  // the attention-only build leaves out the linear, LayerNorm and block entry points
int fbb_linear_max_cta_pairs(int tile_columns) {
    if (tile_columns != 128 && tile_columns != 256) return fail(FBB_ERR_ENUM, "tile_columns must be 128 or 256");
    return linear_max_pairs(tile_columns);
}

int fbb_layernorm_f16(const void* x, void* y, const void* w, const void* b, int64_t M, int C, int64_t ldx, int64_t ldy,
                      float eps, int in_dtype, int param_dtype, void* stream) {
    if (x == nullptr || y == nullptr) return fail(FBB_ERR_NULL, "layernorm: x or y is null");
    if (in_dtype < FBB_DTYPE_F16 || in_dtype > FBB_DTYPE_F32 || param_dtype < FBB_DTYPE_F16 || param_dtype > FBB_DTYPE_F32)
        return fail(FBB_ERR_ENUM, "layernorm: unknown dtype code (in %d, param %d)", in_dtype, param_dtype);
    if (M < 0 || C <= 0 || (C & 7) != 0) return fail(FBB_ERR_SHAPE, "layernorm: need M >= 0 and C %% 8 == 0 (M=%lld C=%d)", (long long)M, C);
    if (ldx < C || ldy < C) return fail(FBB_ERR_SHAPE, "layernorm: row stride smaller than C");
    const int in_vec = in_dtype == FBB_DTYPE_F32 ? 4 : 8;
    if ((ldx % in_vec) != 0 || (ldy & 7) != 0 || !aligned16(x) || !aligned16(y) || !aligned16(w) || !aligned16(b))
        return fail(FBB_ERR_ALIGN, "layernorm: pointers must be 16-byte aligned and row strides multiples of 16 bytes");
    if (!(eps >= 0.f)) return fail(FBB_ERR_SHAPE, "layernorm: eps must be >= 0");
    return launch_layernorm(x, y, w, b, M, C, ldx, ldy, eps, in_dtype, param_dtype, (cudaStream_t)stream);
}

int fbb_layernorm_split_f16(const void* x, const void* w, const void* b, void* patches_out, void* cls_out, void* regs_out, int B, int N,
                            int C, int n_prefix, float eps, int apply_norm, int channel_major, void* stream) {
    if (x == nullptr || patches_out == nullptr) return fail(FBB_ERR_NULL, "layernorm_split: x or patches_out is null");
    if (B < 0 || N < 0 || C <= 0 || (C & 7) != 0 || C > 2048) return fail(FBB_ERR_SHAPE, "layernorm_split: need B, N >= 0 and C %% 8 == 0, C <= 2048 (B=%d N=%d C=%d)", B, N, C);
    if (n_prefix < 1 || n_prefix > 32 || (N > 0 && n_prefix > N)) return fail(FBB_ERR_SHAPE, "layernorm_split: n_prefix (cls + registers) must be in [1, min(32, N)], got %d", n_prefix);
    if (!aligned16(x) || !aligned16(w) || !aligned16(b) || !aligned16(cls_out) || !aligned16(regs_out)) return fail(FBB_ERR_ALIGN, "layernorm_split: pointers must be 16-byte aligned");
    if (channel_major ? (reinterpret_cast<uintptr_t>(patches_out) & 1u) != 0 : !aligned16(patches_out)) return fail(FBB_ERR_ALIGN, "layernorm_split: patches_out is misaligned");
    if (!(eps >= 0.f)) return fail(FBB_ERR_SHAPE, "layernorm_split: eps must be >= 0");
    return launch_layernorm_split(x, w, b, patches_out, cls_out, regs_out, B, N, C, n_prefix, eps, apply_norm != 0, channel_major != 0, (cudaStream_t)stream);
}

int fbb_linear_f16(const void* A, const void* W, void* C, const void* bias, const void* res, const void* gamma, int64_t M,
                   int N, int K, int64_t lda, int64_t ldw, int64_t ldc, int64_t ldr, int epilogue, int accumulate,
                   void* stream) {
    if (A == nullptr || W == nullptr || C == nullptr) return fail(FBB_ERR_NULL, "linear: A, W or C is null");
    if (epilogue < FBB_EPI_NONE || epilogue > FBB_EPI_SWIGLU) return fail(FBB_ERR_ENUM, "linear: unknown epilogue %d", epilogue);
    if (accumulate != FBB_ACC_F32 && accumulate != FBB_ACC_F16) return fail(FBB_ERR_ENUM, "linear: unknown accumulate %d", accumulate);
    if (M < 0 || M > 0x7FFFFF00ll || N <= 0 || K <= 0) return fail(FBB_ERR_SHAPE, "linear: bad M/N/K (%lld, %d, %d)", (long long)M, N, K);
    if ((K & 7) != 0 || (N & 7) != 0) return fail(FBB_ERR_SHAPE, "linear: need K %% 8 == 0 and N %% 8 == 0 (N=%d K=%d)", N, K);
    const bool swiglu = epilogue == FBB_EPI_SWIGLU;
    if (swiglu && ((N & 15) != 0 || res != nullptr || gamma != nullptr))
        return fail(FBB_ERR_SHAPE, "linear: SwiGLU needs N %% 16 == 0 and no res / gamma");
    const int n_out = swiglu ? N / 2 : N;
    if (lda < K || ldw < K || ldc < n_out || (res != nullptr && ldr < n_out))
        return fail(FBB_ERR_SHAPE, "linear: a leading dimension is smaller than its row length");
    if ((lda & 7) || (ldw & 7) || (ldc & 7) || (res != nullptr && (ldr & 7)) || !aligned16(A) || !aligned16(W) || !aligned16(C) ||
        !aligned16(res))
        return fail(FBB_ERR_ALIGN, "linear: A, W, C, res must be 16-byte aligned with leading dimensions %% 8 == 0");
    return launch_linear(A, W, C, bias, res, gamma, M, N, K, lda, ldw, ldc, ldr, epilogue, accumulate, (cudaStream_t)stream);
}

int fbb_linear_layernorm_launches(int64_t M, int N, int epilogue, int has_counter) {
    return linear_layernorm_launches(M, N, epilogue, has_counter != 0);
}

int fbb_linear_layernorm_f16(const void* A, const void* W, void* C, const void* bias, const void* res, const void* gamma, int64_t M, int N,
                             int K, int64_t lda, int64_t ldw, int64_t ldc, int64_t ldr, int epilogue, int accumulate, const void* ln_w,
                             const void* ln_b, float ln_eps, void* y, int64_t ldy, void* counter, void* stream) {
    if (A == nullptr || W == nullptr || C == nullptr || y == nullptr) return fail(FBB_ERR_NULL, "linear_layernorm: A, W, C or y is null");
    if (epilogue != FBB_EPI_NONE && epilogue != FBB_EPI_GELU) return fail(FBB_ERR_ENUM, "linear_layernorm: epilogue must be none or gelu (got %d)", epilogue);
    if (accumulate != FBB_ACC_F32 && accumulate != FBB_ACC_F16) return fail(FBB_ERR_ENUM, "linear_layernorm: unknown accumulate %d", accumulate);
    if (M < 0 || M > 0x7FFFFF00ll || N <= 0 || K <= 0) return fail(FBB_ERR_SHAPE, "linear_layernorm: bad M/N/K (%lld, %d, %d)", (long long)M, N, K);
    if ((K & 7) != 0 || (N & 7) != 0) return fail(FBB_ERR_SHAPE, "linear_layernorm: need K %% 8 == 0 and N %% 8 == 0 (N=%d K=%d)", N, K);
    if (lda < K || ldw < K || ldc < N || ldy < N || (res != nullptr && ldr < N))
        return fail(FBB_ERR_SHAPE, "linear_layernorm: a leading dimension is smaller than its row length");
    if ((lda & 7) || (ldw & 7) || (ldc & 7) || (ldy & 7) || (res != nullptr && (ldr & 7)) || !aligned16(A) || !aligned16(W) || !aligned16(C) ||
        !aligned16(res) || !aligned16(y) || !aligned16(ln_w) || !aligned16(ln_b))
        return fail(FBB_ERR_ALIGN, "linear_layernorm: pointers must be 16-byte aligned with leading dimensions %% 8 == 0");
    if (counter != nullptr && (reinterpret_cast<uintptr_t>(counter) & 3u)) return fail(FBB_ERR_ALIGN, "linear_layernorm: counter must be 4-byte aligned");
    if (!(ln_eps >= 0.f)) return fail(FBB_ERR_SHAPE, "linear_layernorm: eps must be >= 0");
    if (y == C) return fail(FBB_ERR_SHAPE, "linear_layernorm: y must not alias C");
    return launch_linear_layernorm(A, W, C, bias, res, gamma, M, N, K, lda, ldw, ldc, ldr, epilogue, accumulate, ln_w, ln_b, ln_eps, y, ldy,
                                   counter, (cudaStream_t)stream);
}

#endif  // FBB_FLASH_ONLY

int64_t fbb_flash64_workspace_bytes(int B, int N, int H) { return flash64_workspace_bytes_for(B, N, H); }
int fbb_flash64_launches(int B, int N, int H, int has_workspace) { return flash64_launches(B, N, H, has_workspace != 0); }

// Host-side checks shared by the three attention entry points; FBB_OK means the launch may go ahead.
static int check_flash_args(const void* q, const void* k, const void* v, void* o, int B, int N, int H, const int64_t* qs, const int64_t* ks,
                            const int64_t* vs, const int64_t* os, float scale, int variant) {
    if (q == nullptr || k == nullptr || v == nullptr || o == nullptr) return fail(FBB_ERR_NULL, "flash64: q, k, v or o is null");
    if (variant < FBB_FLASH_FF || variant > FBB_FLASH_HH) return fail(FBB_ERR_ENUM, "flash64: unknown variant %d", variant);
    if (B < 0 || N < 0 || H <= 0 || (int64_t)B * H > 0x7FFFFFFFll) return fail(FBB_ERR_SHAPE, "flash64: bad B/N/H (%d, %d, %d)", B, N, H);
    if (!(scale > 0.f)) return fail(FBB_ERR_SHAPE, "flash64: scale must be > 0");
    for (int i = 0; i < 3; ++i)
        if ((qs[i] & 7) || (ks[i] & 7) || (vs[i] & 7) || (os[i] & 7) || qs[i] < 0 || ks[i] < 0 || vs[i] < 0 || os[i] < 0)
            return fail(FBB_ERR_ALIGN, "flash64: strides must be non-negative multiples of 8 elements");
    if (!aligned16(q) || !aligned16(k) || !aligned16(v) || !aligned16(o)) return fail(FBB_ERR_ALIGN, "flash64: pointers must be 16-byte aligned");
    if (qs[1] < 64 || ks[1] < 64 || vs[1] < 64 || os[1] < 64) return fail(FBB_ERR_SHAPE, "flash64: token stride smaller than the head dimension");
    return FBB_OK;
}

int fbb_flash64_f16_ws(const void* q, const void* k, const void* v, void* o, int B, int N, int H, int64_t q_sb, int64_t q_sn,
                       int64_t q_sh, int64_t k_sb, int64_t k_sn, int64_t k_sh, int64_t v_sb, int64_t v_sn, int64_t v_sh,
                       int64_t o_sb, int64_t o_sn, int64_t o_sh, float scale, int variant, void* workspace, int64_t workspace_bytes,
                       void* stream) {
    const int64_t qs[3] = {q_sb, q_sn, q_sh}, ks[3] = {k_sb, k_sn, k_sh}, vs[3] = {v_sb, v_sn, v_sh}, os[3] = {o_sb, o_sn, o_sh};
    const int rc = check_flash_args(q, k, v, o, B, N, H, qs, ks, vs, os, scale, variant);
    if (rc != FBB_OK) return rc;
    if (workspace != nullptr && (!aligned16(workspace) || workspace_bytes < 0)) return fail(FBB_ERR_ALIGN, "flash64: workspace must be 16-byte aligned");
    if (B == 0 || N == 0) return FBB_OK;
    return launch_flash64(q, k, v, o, B, N, H, qs, ks, vs, os, scale, variant, workspace, workspace_bytes, (cudaStream_t)stream);
}

int fbb_flash64_f16(const void* q, const void* k, const void* v, void* o, int B, int N, int H, int64_t q_sb, int64_t q_sn,
                    int64_t q_sh, int64_t k_sb, int64_t k_sn, int64_t k_sh, int64_t v_sb, int64_t v_sn, int64_t v_sh,
                    int64_t o_sb, int64_t o_sn, int64_t o_sh, float scale, int variant, void* stream) {
    return fbb_flash64_f16_ws(q, k, v, o, B, N, H, q_sb, q_sn, q_sh, k_sb, k_sn, k_sh, v_sb, v_sn, v_sh, o_sb, o_sn, o_sh, scale, variant,
                              nullptr, 0, stream);
}

int fbb_flash64_f16_static(const void* q, const void* k, const void* v, void* o, int B, int N, int H, int64_t q_sb, int64_t q_sn,
                           int64_t q_sh, int64_t k_sb, int64_t k_sn, int64_t k_sh, int64_t v_sb, int64_t v_sn, int64_t v_sh,
                           int64_t o_sb, int64_t o_sn, int64_t o_sh, float scale, int variant, void* stream) {
    // every argument is checked before the array is looked up or anything is enqueued: a rejected call leaves no trace
    const int64_t qs[3] = {q_sb, q_sn, q_sh}, ks[3] = {k_sb, k_sn, k_sh}, vs[3] = {v_sb, v_sn, v_sh}, os[3] = {o_sb, o_sn, o_sh};
    const int rc0 = check_flash_args(q, k, v, o, B, N, H, qs, ks, vs, os, scale, variant);
    if (rc0 != FBB_OK) return rc0;
    if (B == 0 || N == 0) return FBB_OK;
    void* ws = nullptr;
    int64_t ws_bytes = 0;
    if (flash64_workspace_bytes_for(B, N, H) > 0) {  // only shapes that are split touch the array
        const int rc = flash64_static_workspace(&ws, &ws_bytes, (cudaStream_t)stream);
        if (rc != FBB_OK) return rc;
    }
    return launch_flash64(q, k, v, o, B, N, H, qs, ks, vs, os, scale, variant, ws, ws_bytes, (cudaStream_t)stream);
}

#ifdef FBB_DEBUG_WAITS
int fbb_debug_waits(unsigned int* out, int max_entries) {
    unsigned int n = 0;
    cudaDeviceSynchronize();
    cudaMemcpyFromSymbol(&n, g_fbb_debug_n, sizeof(n));
    if (n > 256u) n = 256u;
    if ((int)n > max_entries) n = (unsigned)max_entries;
    cudaMemcpyFromSymbol(out, g_fbb_debug, sizeof(unsigned int) * 5 * n);
    const unsigned int zero = 0;
    cudaMemcpyToSymbol(g_fbb_debug_n, &zero, sizeof(zero));
    return (int)n;
}
#endif

int fbb_diag_wait_timeout(uint64_t limit_ns, unsigned int detail, void* stream) {
    if (limit_ns == 0 || limit_ns > 100000000ull) return fail(FBB_ERR_SHAPE, "diag: limit must be in (0, 100 ms]");
    wait_timeout_probe_kernel<<<1, 32, 0, (cudaStream_t)stream>>>((unsigned long long)limit_ns, detail, nullptr);
    return cuda_status(cudaGetLastError());
}

int fbb_diag_sm_clock_mhz(float* out_mhz, int64_t spin_clocks, void* stream) {
    if (out_mhz == nullptr) return fail(FBB_ERR_NULL, "diag: out_mhz is null");
    if (spin_clocks < 1024 || spin_clocks > (1ll << 24)) return fail(FBB_ERR_SHAPE, "diag: spin_clocks must be in [1024, 2^24]");
    sm_clock_probe_kernel<<<1, 1, 0, (cudaStream_t)stream>>>(out_mhz, (long long)spin_clocks);
    return cuda_status(cudaGetLastError());
}

#ifndef FBB_FLASH_ONLY
int64_t fbb_stack_scratch_bytes(const fbb_block_desc* blocks, int n_blocks, int64_t tokens) {
    if (blocks == nullptr || n_blocks <= 0 || tokens <= 0) return 0;
    return stack_scratch_bytes(blocks, n_blocks, tokens);
}

int fbb_stack_launches(const fbb_block_desc* blocks, int n_blocks, int64_t tokens) {
    if (blocks == nullptr || n_blocks <= 0 || tokens <= 0) return 0;
    return stack_launches(blocks, n_blocks, tokens);
}

int fbb_stack_forward_f16(const fbb_block_desc* blocks, int n_blocks, void* x, int B, int N, void* scratch, int64_t scratch_bytes,
                          void* workspace, int64_t workspace_bytes, void* stream) {
    if (workspace != nullptr && (!aligned16(workspace) || workspace_bytes < 0)) return fail(FBB_ERR_ALIGN, "block: workspace must be 16-byte aligned");
    return stack_forward(blocks, n_blocks, x, B, N, scratch, scratch_bytes, workspace, workspace_bytes, (cudaStream_t)stream);
}

int fbb_block_forward_f16(const fbb_block_desc* block, void* x, int B, int N, void* scratch, int64_t scratch_bytes, void* workspace,
                          int64_t workspace_bytes, void* stream) {
    return fbb_stack_forward_f16(block, 1, x, B, N, scratch, scratch_bytes, workspace, workspace_bytes, stream);
}

#endif  // FBB_FLASH_ONLY

}  // extern "C"
