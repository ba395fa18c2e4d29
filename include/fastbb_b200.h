/* fastbb_b200 — C ABI of the B200 (sm_100a) ViT block kernels.
 *
 * This is the boundary the host side (Python, ctypes.CDLL) crosses. In the reference the same boundary is
 * ctypes -> libcuda with a kernel-name + signature-string table (fastbb/kernels.py:19-41 SIGNATURES,
 * fastbb/kernels.py:118-133 Kernels.launch); here it is a plain shared library with one entry point per operator.
 *
 * Conventions
 *  - every pointer is a device pointer in the caller's current CUDA context/device; nothing is allocated or freed by
 *    the library on any of these calls (the one kernel that wants scratch memory takes it from the caller, see
 *    fbb_flash64_f16_ws, or from a device array built into the library, see fbb_flash64_f16_static), and no call
 *    synchronises except fbb_device_status();
 *  - `stream` is a cudaStream_t passed as void* (0 = legacy default stream); work is only enqueued;
 *  - all leading dimensions and strides are in ELEMENTS, not bytes;
 *  - return value: 0 = success, < 0 = argument rejected on the host before any launch (FBB_ERR_*), > 0 = cudaError_t;
 *    fbb_last_error() gives a thread-local message for the last non-zero status of the calling thread;
 *  - thread-compatible: the mutable state shared between calls is (a) a workspace the caller passes to both, (b) the
 *    built-in device array of fbb_flash64_f16_static, shared by every call of that entry point on a device (calls that
 *    overlap on the GPU race on it), and (c) a mutex-guarded host table of encoded tensor maps (a pure cache).
 */
#ifndef FASTBB_B200_H_
#define FASTBB_B200_H_

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define FBB_VERSION 100 /* major*10000 + minor*100 + patch */

enum fbb_status {
    FBB_OK = 0,
    FBB_ERR_NULL = -1,        /* a required pointer is null */
    FBB_ERR_SHAPE = -2,       /* a size / leading dimension is not supported (see each function) */
    FBB_ERR_ALIGN = -3,       /* a pointer or stride breaks the 16-byte rule */
    FBB_ERR_ENUM = -4,        /* unknown dtype / epilogue / accumulate / variant code */
    FBB_ERR_DRIVER = -5,      /* the CUDA driver entry point for tensor maps could not be resolved or failed */
    FBB_ERR_DEVICE_WAIT = -6  /* fbb_device_status(): a kernel gave up a bounded wait (details in out[]) */
};

enum fbb_dtype { FBB_DTYPE_F16 = 0, FBB_DTYPE_BF16 = 1, FBB_DTYPE_F32 = 2 };

/* epilogue of fbb_linear_f16 (applied in fp32 on the accumulator, in this order):
 *   v = acc + bias[n]; v = act(v); out = res[m,n] + gamma[n] * v   (gamma null -> res + v; res null -> v)       */
enum fbb_epilogue {
    FBB_EPI_NONE = 0,  /* act = identity                                        (gemm.py act None / "none")     */
    FBB_EPI_GELU = 1,  /* act = exact erf GELU                                  (gemm.py act "gelu")            */
    FBB_EPI_SWIGLU = 2 /* W holds w12 = [x1 rows | x2 rows]; out[m,j] = silu(x1_j) * x2_j, j < N/2 (vit.py:139-141) */
};

enum fbb_accumulate {
    FBB_ACC_F32 = 0, /* fp32 tensor-memory accumulator   (reference g0 and g3; gemm variants f32, c1, c2, c4) */
    FBB_ACC_F16 = 1  /* fp16 tensor-memory accumulator   (reference g1, g2 except fc2; gemm variant h)        */
};

/* The reference's names for the accumulate types of Q.K^T and P.V in its mma.sync kernels (attention.py variants). All
 * three are accepted; on tcgen05 an f16 accumulator is no faster than an fp32 one and costs a conversion when it is read
 * back, so every variant computes both products with fp32 accumulators (at least the reference's accuracy). */
enum fbb_flash_variant {
    FBB_FLASH_FF = 0, /* reference: fp32 accumulate for Q.K^T and for P.V */
    FBB_FLASH_FH = 1, /* reference: fp32 Q.K^T, fp16-accumulated P.V per key block */
    FBB_FLASH_HH = 2  /* reference: fp16 accumulate for both */
};

/* Library version (FBB_VERSION of the build). */
int fbb_version(void);

/* Static text for a status code returned by any function below. */
const char* fbb_status_string(int status);

/* Message for the last non-zero status returned to the calling thread ("" if none). */
const char* fbb_last_error(void);

/* Synchronises the current device, copies the device status word into out[4] = {code, detail, block, count} and
 * clears it. Returns FBB_OK when no kernel recorded an error, FBB_ERR_DEVICE_WAIT when one ran out of a bounded
 * wait (its output is then undefined), or a cudaError_t. Meant for tests and debugging, never for the hot path. */
int fbb_device_status(unsigned int out[4]);

/* Diagnostics: launches one warp that waits, with the library's bounded wait and the given limit (nanoseconds, at most
 * 100 ms), on a barrier nothing ever arrives on. The wait gives up and the kernel returns normally, after recording
 * {code 5 (other wait), detail, block 0} in the device status word: the next fbb_device_status() returns
 * FBB_ERR_DEVICE_WAIT with those values and clears them. Exercises the path every pipeline wait of the kernels takes
 * when it runs out; nothing faults or hangs. No counterpart in the reference. */
int fbb_diag_wait_timeout(uint64_t limit_ns, unsigned int detail, void* stream);

/* Diagnostics: enqueues a one-thread kernel that counts spin_clocks (1024 .. 2^24) SM clocks against the nanosecond
 * timer and writes the ratio in MHz to *out_mhz (device memory): the SM clock at that point of the stream, as the
 * kernels around it see it. No counterpart in the reference. */
int fbb_diag_sm_clock_mhz(float* out_mhz, int64_t spin_clocks, void* stream);

/* Diagnostics: how many two-CTA clusters of the linear kernel (tile_columns = 128 or 256) the current device can hold at
 * once; 0 means the kernel runs in its one-CTA form. No counterpart in the reference (its GEMMs are cuBLAS calls). */
int fbb_linear_max_cta_pairs(int tile_columns);

/* y[m, :] = LayerNorm(x[m, :]) * w + b, statistics in fp32, output fp16.
 * Replaces: the nn.LayerNorm calls of fastbb/vit.py:114,126,130,139,159,166,170 (norm1 / norm2) and :184,241 (vit.norm).
 * x: [M, C] of in_dtype with row stride ldx; y: [M, C] fp16 with row stride ldy; w, b: [C] of param_dtype or null.
 * Requires C % 8 == 0, ldx % 8 == 0 (fp16/bf16) or % 4 (fp32), ldy % 8 == 0, 16-byte aligned pointers. */
int fbb_layernorm_f16(const void* x, void* y, const void* w, const void* b, int64_t M, int C, int64_t ldx, int64_t ldy,
                      float eps, int in_dtype, int param_dtype, void* stream);

/* The final norm of a ViT with the outputs split as get_intermediate_layers returns them, in one launch.
 * Replaces: vit.norm followed by the cls split, the register drop and, for reshape=True, the permute + contiguous copy
 * into [B, C, h, w] (fastbb/vit.py:184,225-232).
 * x: [B, N, C] fp16 contiguous; row 0 of an image is its cls token, rows 1 .. n_prefix-1 its register tokens, the other
 * HW = N - n_prefix rows its patch tokens. w, b: [C] fp16 or null. apply_norm = 0 copies the rows unnormalised (norm=False).
 *   cls_out  [B, C] or null;  regs_out [B, n_prefix-1, C] or null;
 *   patches_out: channel_major = 0: [B, HW, C] (token-major);  channel_major = 1: [B, C, HW], i.e. [B, C, h, w].
 * Requires C % 8 == 0, C <= 2048, 1 <= n_prefix <= 32, 16-byte aligned pointers. */
int fbb_layernorm_split_f16(const void* x, const void* w, const void* b, void* patches_out, void* cls_out, void* regs_out, int B, int N,
                            int C, int n_prefix, float eps, int apply_norm, int channel_major, void* stream);

/* C[M, Nout] = epilogue(A[M, K] . W[N, K]^T), fp16 operands, tcgen05 tensor cores.
 * Replaces: F.linear / torch._addmm_activation / F.gelu / F.silu.mul_ / addcmul of fastbb/vit.py:114-143, and
 * gemm.linear + gemm_tn_{f32,c1,c2,c4,h}_{128,256} of fastbb/gemm.py:30-63 and fastbb/fastbb_kernels.cu:323-446.
 * A: row stride lda; W: nn.Linear layout [N, K] with row stride ldw; C: row stride ldc; res: [M, Nout] fp16 with row
 * stride ldr or null; bias: [N] fp16 or null; gamma: [Nout] fp16 or null (only read when res is given).
 * Nout = N, or N/2 for FBB_EPI_SWIGLU (res and gamma must then be null). C may alias res (same pointer and stride).
 * Requires K % 8 == 0, N % 8 == 0 (N % 16 for SwiGLU), lda/ldw/ldc/ldr % 8 == 0, 16-byte aligned A, W, C, res. */
int fbb_linear_f16(const void* A, const void* W, void* C, const void* bias, const void* res, const void* gamma, int64_t M,
                   int N, int K, int64_t lda, int64_t ldw, int64_t ldc, int64_t ldr, int epilogue, int accumulate,
                   void* stream);

/* fbb_linear_f16 (epilogue none or GELU) followed by the LayerNorm of the output rows: C as above, and
 * y[m, :] = LayerNorm(C[m, :]) * ln_w + ln_b (fp16, row stride ldy; ln_w, ln_b: [N] fp16 or null). In one launch when the
 * shape allows it (the CTA pairs that hold a row tile's columns form one thread-block cluster and exchange per-row
 * statistics through distributed shared memory), otherwise as the GEMM followed by the LayerNorm kernel: the results are
 * the same up to fp32 rounding of the statistics.
 * Replaces: proj / fc2 with LayerScale + residual followed by norm2 of the same block / norm1 of the next block,
 * fastbb/vit.py:116-118 + 126|130|139 and :137-143 + :114.
 * counter: 4 bytes of device memory, zero when the call starts; every launch leaves it zero again, so one counter
 * serves all calls on a stream (calls that may overlap on the GPU need different ones). It may be null when M is a
 * multiple of 256 or has more than 8 rows beyond one; otherwise a null counter selects the two-launch form.
 * y must not alias C; C may alias res. Requirements as for fbb_linear_f16, and ldy % 8 == 0. */
int fbb_linear_layernorm_f16(const void* A, const void* W, void* C, const void* bias, const void* res, const void* gamma, int64_t M, int N,
                             int K, int64_t lda, int64_t ldw, int64_t ldc, int64_t ldr, int epilogue, int accumulate, const void* ln_w,
                             const void* ln_b, float ln_eps, void* y, int64_t ldy, void* counter, void* stream);

/* Diagnostics: how many kernels fbb_linear_layernorm_f16 enqueues for this shape on the current device (1: fused, 2: the
 * GEMM and the LayerNorm kernel, 0: nothing to do). No counterpart in the reference. */
int fbb_linear_layernorm_launches(int64_t M, int N, int epilogue, int has_counter);

/* O = softmax(scale . Q K^T) V for head dimension 64, no mask, any sequence length N >= 1.
 * Replaces: attention.attention + flash64_r{1,2}_{hh,fh,ff} (fastbb/attention.py:31-60,
 * fastbb/fastbb_kernels.cu:58-312) and the F.scaled_dot_product_attention fallback of fastbb/vit.py:149-150.
 * q, k, v, o: fp16, element (b, n, h, d) at ptr[b*sb + n*sn + h*sh + d] (d contiguous): e.g. the three unbound views
 * of the packed [B, N, 3, H, 64] qkv GEMM output, and o as [B, N, H*64]. Strides must be multiples of 8 elements,
 * pointers 16-byte aligned, scale > 0. */
int fbb_flash64_f16(const void* q, const void* k, const void* v, void* o, int B, int N, int H, int64_t q_sb, int64_t q_sn,
                    int64_t q_sh, int64_t k_sb, int64_t k_sn, int64_t k_sh, int64_t v_sb, int64_t v_sn, int64_t v_sh,
                    int64_t o_sb, int64_t o_sn, int64_t o_sh, float scale, int variant, void* stream);

/* The same operator with a caller-owned workspace, which lets it balance the last, partly filled wave of query tiles:
 * one persistent CTA per SM takes an equal share of the (query tile, key block) steps, and a tile whose keys end up
 * split over two CTAs is merged through the workspace (unnormalised fp32 partial results + running maxima / sums).
 * No counterpart in the reference (its kernels run one CTA per query tile); results are the same up to fp32 rounding
 * of the merge.
 * With a workspace the few query rows beyond the last full 256-row tile group (the cls token and registers of a ViT: at
 * most 8 rows per head and 18 over all batch x head pairs, sequences of 3072 tokens and more) are not tiled either: a second, small launch computes
 * them on the CUDA cores beside the tiled one (partial results per key chunk in the workspace, merged by the warp that
 * completes a row), so that one row does not cost every head a tile group.
 *   fbb_flash64_workspace_bytes(B, N, H): bytes needed on the current device for this shape, 0 if it uses none.
 *   fbb_flash64_launches(B, N, H, has_workspace): kernel launches the call enqueues (1, or 2 with leftover rows).
 *   workspace: device memory of at least that size, 16-byte aligned, ZEROED once by the caller before its first use;
 *     it starts with one flag word per softmax warp and SM and one counter per SM (68 bytes per SM), which every launch
 *     leaves zero again, so it can be reused by any later call of any shape; the rest is overwritten freely. null (or a shape that needs
 *     none) gives exactly fbb_flash64_f16. Calls that may overlap in time (different streams) need different workspaces.
 *     If fbb_device_status() ever reports a failed wait, zero the workspace again before reusing it. */
int64_t fbb_flash64_workspace_bytes(int B, int N, int H);
int fbb_flash64_launches(int B, int N, int H, int has_workspace);
int fbb_flash64_f16_ws(const void* q, const void* k, const void* v, void* o, int B, int N, int H, int64_t q_sb, int64_t q_sn,
                       int64_t q_sh, int64_t k_sb, int64_t k_sn, int64_t k_sh, int64_t v_sb, int64_t v_sn, int64_t v_sh,
                       int64_t o_sb, int64_t o_sn, int64_t o_sh, float scale, int variant, void* workspace,
                       int64_t workspace_bytes, void* stream);

/* fbb_flash64_f16_ws with the workspace built into the library: a file-scope device array of 11.5 MiB, enough for the
 * split form on devices of up to 160 SMs (a device that needs more is rejected with FBB_ERR_SHAPE; shapes that are never
 * split do not touch it). No counterpart in the reference. The call allocates and frees nothing: the array's address
 * is looked up once per device (cudaGetSymbolAddress, with that device current) and kept.
 *  - All calls on a device share the one array: two calls that may overlap in time (different streams) race on it and
 *    give wrong results; use fbb_flash64_f16_ws with separate workspaces for that.
 *  - The flag words at the start of the array must be zero when the kernel starts. They are when the library is loaded,
 *    every completed launch leaves them so, and each call also enqueues a clear of them on `stream` ahead of the kernel,
 *    so a launch that gave up a wait (see fbb_device_status) does not poison later calls.
 *  - Make the first call on a device outside any stream capture: it is the one that resolves the array's address. */
int fbb_flash64_f16_static(const void* q, const void* k, const void* v, void* o, int B, int N, int H, int64_t q_sb, int64_t q_sn,
                           int64_t q_sh, int64_t k_sb, int64_t k_sn, int64_t k_sh, int64_t v_sb, int64_t v_sn, int64_t v_sh,
                           int64_t o_sb, int64_t o_sn, int64_t o_sh, float scale, int variant, void* stream);

/* ---- one FFI crossing per transformer block or per run of blocks -------------------------------------------------------
 * Replaces FastViT.block / block_chunked and the loop over blocks in FastViT.run (fastbb/vit.py:108-172, 175-187), which
 * cross from Python into torch / ctypes ten to eleven times per block. The same seven kernels are enqueued in the same
 * order as through the per-operator entry points, so the results are bit-identical to those.
 * All weights fp16 in nn.Linear layout, contiguous (leading dimension = row length); null bias / LayerNorm affine /
 * LayerScale pointers mean "absent". */
enum fbb_mlp_kind {
    FBB_MLP_GELU = 0,   /* fc1 [hidden, C] + erf-GELU, fc2 [C, hidden]            (fastbb/vit.py:121-131) */
    FBB_MLP_SWIGLU = 1  /* fc1 = w12 [2*hidden, C], silu(x1)*x2, fc2 = w3 [C, hidden] (fastbb/vit.py:139-143) */
};

typedef struct fbb_block_desc {
    const void *ln1_w, *ln1_b;     /* [C] */
    const void *qkv_w, *qkv_b;     /* [3C, C], [3C] */
    const void *proj_w, *proj_b;   /* [C, C], [C] */
    const void *gamma1;            /* LayerScale of the attention branch [C] */
    const void *ln2_w, *ln2_b;     /* [C] */
    const void *fc1_w, *fc1_b;     /* see fbb_mlp_kind */
    const void *fc2_w, *fc2_b;
    const void *gamma2;            /* LayerScale of the MLP branch [C] */
    int C, heads, hidden;          /* C = heads * 64; hidden = columns of the MLP's hidden activation */
    int mlp;                       /* fbb_mlp_kind */
    int acc_main, acc_fc2;         /* fbb_accumulate of qkv / proj / fc1, and of fc2 (the reference's g2 keeps fc2 in fp32) */
    int flash_variant;             /* fbb_flash_variant */
    float eps1, eps2;              /* LayerNorm epsilons */
    float scale;                   /* attention scale, > 0 */
} fbb_block_desc;

/* Bytes of scratch (LayerNorm output, packed qkv, attention output, MLP hidden, a counter) the blocks need for `tokens` = B*N tokens. */
int64_t fbb_stack_scratch_bytes(const fbb_block_desc* blocks, int n_blocks, int64_t tokens);

/* How many kernels fbb_stack_forward_f16 enqueues for this run on the current device (5 to 7 per block: each residual
 * GEMM and the LayerNorm that follows it are one launch where fbb_linear_layernorm_f16 can fuse them). */
int fbb_stack_launches(const fbb_block_desc* blocks, int n_blocks, int64_t tokens);

/* x [B, N, C] fp16 contiguous is updated IN PLACE by n_blocks blocks (the residual epilogues write over their residual
 * input). scratch: 256-byte aligned device memory of at least fbb_stack_scratch_bytes(); workspace: optional, as for
 * fbb_flash64_f16_ws. Nothing is allocated; fbb_stack_launches() kernels and one 256-byte memset are enqueued on `stream`. */
int fbb_stack_forward_f16(const fbb_block_desc* blocks, int n_blocks, void* x, int B, int N, void* scratch, int64_t scratch_bytes,
                          void* workspace, int64_t workspace_bytes, void* stream);
int fbb_block_forward_f16(const fbb_block_desc* block, void* x, int B, int N, void* scratch, int64_t scratch_bytes, void* workspace,
                          int64_t workspace_bytes, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* FASTBB_B200_H_ */
