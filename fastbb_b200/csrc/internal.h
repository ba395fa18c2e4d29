// Host-side declarations shared by the translation units of libfastbb_b200.so (not part of the public ABI).
#pragma once
#include <cuda.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "../../include/fastbb_b200.h"

namespace fbb {

inline int cuda_status(cudaError_t e) { return e == cudaSuccess ? FBB_OK : (int)e; }

// Records a thread-local message for fbb_last_error() and returns `status` unchanged.
int fail(int status, const char* fmt, ...);

// cuTensorMapEncodeTiled resolved through the runtime (no link-time dependency on libcuda); nullptr if unavailable.
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                  const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
EncodeTiledFn encode_tiled_fn();

// fp16 tensor map with 128-byte swizzle, zero fill outside the tensor. dims/strides innermost first; strides in
// elements for dims 1..rank-1 (dim 0 is contiguous); box innermost first (box[0] * 2 bytes = the swizzle span: 64
// elements for the 128-byte mode, 32 for the 64-byte mode).
int make_tmap_f16(CUtensorMap* map, const void* base, int rank, const uint64_t* dims, const int64_t* strides_elems,
                  const uint32_t* box, CUtensorMapSwizzle swizzle = CU_TENSOR_MAP_SWIZZLE_128B);

int num_sms();  // SM count of the current device

// Launch with programmatic stream serialization (see grid_dependency_wait in common.cuh). FBB_NO_PDL=1 in the environment
// turns the attribute off (plain stream order).
bool pdl_enabled();
// cluster_x > 1 launches thread-block clusters of that many CTAs along x (the grid must be a multiple of it).
template <typename... KArgs, typename... Args>
inline cudaError_t launch_pdl_cluster(void (*kern)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream, unsigned cluster_x,
                                      Args&&... args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[2];
    unsigned n = 0;
    if (cluster_x > 1) {
        attr[n].id = cudaLaunchAttributeClusterDimension;
        attr[n].val.clusterDim.x = cluster_x;
        attr[n].val.clusterDim.y = 1;
        attr[n].val.clusterDim.z = 1;
        ++n;
    }
    if (pdl_enabled()) {
        attr[n].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attr[n].val.programmaticStreamSerializationAllowed = 1;
        ++n;
    }
    cfg.attrs = attr;
    cfg.numAttrs = n;
    return cudaLaunchKernelEx(&cfg, kern, static_cast<KArgs>(args)...);
}
template <typename... KArgs, typename... Args>
inline cudaError_t launch_pdl(void (*kern)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream, Args&&... args) {
    return launch_pdl_cluster(kern, grid, block, smem, stream, 1u, static_cast<Args&&>(args)...);
}

int launch_layernorm(const void* x, void* y, const void* w, const void* b, int64_t M, int C, int64_t ldx, int64_t ldy,
                     float eps, int in_dtype, int param_dtype, cudaStream_t stream);

// Final norm with split outputs (layernorm.cu): x [B, N, C] fp16 contiguous -> cls / register / patch destinations.
int launch_layernorm_split(const void* x, const void* w, const void* b, void* patches_out, void* cls_out, void* regs_out, int B, int N, int C,
                           int n_prefix, float eps, int apply_norm, int channel_major, cudaStream_t stream);

int launch_linear(const void* A, const void* W, void* C, const void* bias, const void* res, const void* gamma, int64_t M,
                  int N, int K, int64_t lda, int64_t ldw, int64_t ldc, int64_t ldr, int epilogue, int accumulate,
                  cudaStream_t stream);

// The same followed by y = LayerNorm(C) * ln_w + ln_b (rows of N elements), fused into the GEMM launch when the shape
// allows. `counter`: 4 bytes of zeroed device memory that every launch leaves zero (needed when M has remainder rows).
int launch_linear_layernorm(const void* A, const void* W, void* C, const void* bias, const void* res, const void* gamma, int64_t M, int N,
                            int K, int64_t lda, int64_t ldw, int64_t ldc, int64_t ldr, int epilogue, int accumulate, const void* ln_w,
                            const void* ln_b, float ln_eps, void* y, int64_t ldy, void* counter, cudaStream_t stream);

int linear_layernorm_launches(int64_t M, int N, int epilogue, bool has_counter);  // 1: one fused launch, 2: GEMM then LayerNorm

// How many CTA pairs (clusters of two) of the linear kernel with `bn`-column tiles fit on the current device at once.
int linear_max_pairs(int bn);

// ws / ws_bytes: optional workspace (see fbb_flash64_f16_ws); null = one tile group per CTA, never split.
int launch_flash64(const void* q, const void* k, const void* v, void* o, int B, int N, int H, const int64_t* qs,
                   const int64_t* ks, const int64_t* vs, const int64_t* os, float scale, int variant, void* ws, int64_t ws_bytes,
                   cudaStream_t stream);
// The library's own (static device array) workspace for fbb_flash64_f16_static; clears its flag words on `stream`.
int flash64_static_workspace(void** ptr, int64_t* bytes, cudaStream_t stream);
// Workspace the split form needs on the current device for this shape; 0 when the shape is never split.
int64_t flash64_workspace_bytes_for(int B, int N, int H);
int flash64_launches(int B, int N, int H, bool has_workspace);

// One FFI crossing per block / stack (block.cu): scratch needed for `tokens` tokens, and the launches themselves.
int64_t stack_scratch_bytes(const fbb_block_desc* d, int n_blocks, int64_t tokens);
int stack_launches(const fbb_block_desc* d, int n_blocks, int64_t tokens);  // kernels stack_forward enqueues for this run
int stack_forward(const fbb_block_desc* d, int n_blocks, void* x, int B, int N, void* scratch, int64_t scratch_bytes, void* ws,
                  int64_t ws_bytes, cudaStream_t stream);

}  // namespace fbb
