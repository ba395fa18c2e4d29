// One transformer block, or a run of them, per FFI crossing: the launches of a pre-LN ViT block (LayerNorm, qkv, flash
// attention, proj + LayerScale + residual, LayerNorm, fc1 + GELU | w12 + SwiGLU, fc2 + LayerScale + residual) are
// enqueued by one C call from a table of weight pointers. Replaces FastViT.block / block_chunked (fastbb/vit.py:108-172),
// which cross from Python into torch / ctypes ten to eleven times per block. The kernels and their order are exactly the
// ones the per-operator entry points launch, so the results are bit-identical to calling those one by one.
// Each residual GEMM is followed by a LayerNorm of its output (proj by norm2 of the same block, fc2 by norm1 of the next
// block of the run): those pairs go through launch_linear_layernorm, which fuses them into one launch where the shape
// allows, so a block of the run costs five to seven launches (one more where the attention adds its side launch for leftover rows). Only the first block of a run normalises its own input.
#include "internal.h"

namespace fbb {

static int64_t align256(int64_t v) { return (v + 255) & ~(int64_t)255; }

struct BlockScratch {
    // byte offsets: LayerNorm output [T, C], qkv [T, 3C], attention output [T, C], MLP hidden [T, hidden], then 256 bytes
    // whose first word is the counter of launch_linear_layernorm (zeroed at the start of every stack call)
    int64_t y, qkv, o, h, counter, total;
};

static BlockScratch block_scratch(const fbb_block_desc& d, int64_t tokens) {
    BlockScratch s;
    s.y = 0;
    s.qkv = s.y + align256(tokens * d.C * 2);
    s.o = s.qkv + align256(tokens * 3 * d.C * 2);
    s.h = s.o + align256(tokens * d.C * 2);
    s.counter = s.h + align256(tokens * (int64_t)d.hidden * 2);
    s.total = s.counter + 256;
    return s;
}

static int check_desc(const fbb_block_desc& d) {
    if (d.C <= 0 || d.heads <= 0 || d.C != d.heads * 64) return fail(FBB_ERR_SHAPE, "block: C (%d) must be heads (%d) x 64", d.C, d.heads);
    if (d.hidden <= 0 || (d.hidden & 7)) return fail(FBB_ERR_SHAPE, "block: hidden (%d) must be a positive multiple of 8", d.hidden);
    if (d.mlp != FBB_MLP_GELU && d.mlp != FBB_MLP_SWIGLU) return fail(FBB_ERR_ENUM, "block: unknown mlp kind %d", d.mlp);
    if (d.qkv_w == nullptr || d.proj_w == nullptr || d.fc1_w == nullptr || d.fc2_w == nullptr) return fail(FBB_ERR_NULL, "block: a weight matrix is null");
    if (!(d.scale > 0.f)) return fail(FBB_ERR_SHAPE, "block: attention scale must be > 0");
    return FBB_OK;
}

// y_ready: the LayerNorm-1 output of this block is already in the scratch (written by the previous block's fc2 launch).
// next: the following block of the run (its norm1 is applied to this block's output), or null for the last one.
static int run_block(const fbb_block_desc& d, const fbb_block_desc* next, bool y_ready, void* x, int B, int N, uint8_t* scratch,
                     const BlockScratch& s, void* counter, void* ws, int64_t ws_bytes, cudaStream_t stream) {
    const int64_t T = (int64_t)B * N;
    const int C = d.C;
    void* y = scratch + s.y;
    void* qkv = scratch + s.qkv;
    void* o = scratch + s.o;
    void* h = scratch + s.h;
    int rc = FBB_OK;
    if (!y_ready) rc = launch_layernorm(x, y, d.ln1_w, d.ln1_b, T, C, C, C, d.eps1, FBB_DTYPE_F16, FBB_DTYPE_F16, stream);
    if (rc != FBB_OK) return rc;
    rc = launch_linear(y, d.qkv_w, qkv, d.qkv_b, nullptr, nullptr, T, 3 * C, C, C, C, 3 * C, 0, FBB_EPI_NONE, d.acc_main, stream);
    if (rc != FBB_OK) return rc;
    // q, k, v: the three [B, N, H, 64] views of the packed [B, N, 3, H, 64] buffer
    const int64_t qs[3] = {(int64_t)N * 3 * C, 3 * C, 64}, os[3] = {(int64_t)N * C, C, 64};
    const __half* q = reinterpret_cast<const __half*>(qkv);
    rc = launch_flash64(q, q + C, q + 2 * C, o, B, N, d.heads, qs, qs, qs, os, d.scale, d.flash_variant, ws, ws_bytes, stream);
    if (rc != FBB_OK) return rc;
    rc = launch_linear_layernorm(o, d.proj_w, x, d.proj_b, x, d.gamma1, T, C, C, C, C, C, C, FBB_EPI_NONE, d.acc_main, d.ln2_w, d.ln2_b, d.eps2, y, C,
                                 counter, stream);
    if (rc != FBB_OK) return rc;
    if (d.mlp == FBB_MLP_SWIGLU)
        rc = launch_linear(y, d.fc1_w, h, d.fc1_b, nullptr, nullptr, T, 2 * d.hidden, C, C, C, d.hidden, 0, FBB_EPI_SWIGLU, d.acc_main, stream);
    else
        rc = launch_linear(y, d.fc1_w, h, d.fc1_b, nullptr, nullptr, T, d.hidden, C, C, C, d.hidden, 0, FBB_EPI_GELU, d.acc_main, stream);
    if (rc != FBB_OK) return rc;
    if (next != nullptr)
        return launch_linear_layernorm(h, d.fc2_w, x, d.fc2_b, x, d.gamma2, T, C, d.hidden, d.hidden, d.hidden, C, C, FBB_EPI_NONE, d.acc_fc2, next->ln1_w,
                                       next->ln1_b, next->eps1, y, C, counter, stream);
    return launch_linear(h, d.fc2_w, x, d.fc2_b, x, d.gamma2, T, C, d.hidden, d.hidden, d.hidden, C, C, FBB_EPI_NONE, d.acc_fc2, stream);
}

int stack_launches(const fbb_block_desc* d, int n_blocks, int64_t tokens) {
    int n = 0;
    for (int i = 0; i < n_blocks; ++i) {
        const bool chain = i + 1 < n_blocks && d[i + 1].C == d[i].C;
        const bool y_ready = i > 0 && d[i - 1].C == d[i].C;
        n += (y_ready ? 0 : 1) + 3 + linear_layernorm_launches(tokens, d[i].C, FBB_EPI_NONE, true) +
             (chain ? linear_layernorm_launches(tokens, d[i].C, FBB_EPI_NONE, true) : 1);
    }
    return n;
}

int64_t stack_scratch_bytes(const fbb_block_desc* d, int n_blocks, int64_t tokens) {
    int64_t need = 0;
    for (int i = 0; i < n_blocks; ++i) {
        const int64_t t = block_scratch(d[i], tokens).total;
        if (t > need) need = t;
    }
    return need;
}

int stack_forward(const fbb_block_desc* d, int n_blocks, void* x, int B, int N, void* scratch, int64_t scratch_bytes, void* ws,
                  int64_t ws_bytes, cudaStream_t stream) {
    if (d == nullptr || x == nullptr) return fail(FBB_ERR_NULL, "block: descriptor table or x is null");
    if (n_blocks < 0 || B < 0 || N < 0) return fail(FBB_ERR_SHAPE, "block: bad n_blocks / B / N (%d, %d, %d)", n_blocks, B, N);
    if (n_blocks == 0 || B == 0 || N == 0) return FBB_OK;
    const int64_t T = (int64_t)B * N;
    for (int i = 0; i < n_blocks; ++i) {
        const int rc = check_desc(d[i]);
        if (rc != FBB_OK) return rc;
    }
    if (scratch == nullptr || (reinterpret_cast<uintptr_t>(scratch) & 255) || scratch_bytes < stack_scratch_bytes(d, n_blocks, T))
        return fail(FBB_ERR_SHAPE, "block: scratch must be 256-byte aligned and hold %lld bytes (got %lld)",
                    (long long)stack_scratch_bytes(d, n_blocks, T), (long long)scratch_bytes);
    if (reinterpret_cast<uintptr_t>(x) & 15) return fail(FBB_ERR_ALIGN, "block: x must be 16-byte aligned");
    // one counter for the whole run, at the end of the largest block's scratch layout; zero when the first launch reads it
    uint8_t* sc = reinterpret_cast<uint8_t*>(scratch);
    void* counter = sc + stack_scratch_bytes(d, n_blocks, T) - 256;
    cudaError_t e = cudaMemsetAsync(counter, 0, 256, stream);
    if (e != cudaSuccess) return fail((int)e, "block: cudaMemsetAsync(counter): %s", cudaGetErrorString(e));
    for (int i = 0; i < n_blocks; ++i) {
        const bool chain = i + 1 < n_blocks && d[i + 1].C == d[i].C;  // the next block normalises rows of the same width
        const bool y_ready = i > 0 && d[i - 1].C == d[i].C;
        const int rc = run_block(d[i], chain ? &d[i + 1] : nullptr, y_ready, x, B, N, sc, block_scratch(d[i], T), counter, ws, ws_bytes, stream);
        if (rc != FBB_OK) return rc;
    }
    return FBB_OK;
}

}  // namespace fbb
