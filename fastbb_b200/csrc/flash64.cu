#include "common.cuh"
#include "internal.h"
namespace fbb {
int launch_flash64(const void*, const void*, const void*, void*, int, int, int, const int64_t*, const int64_t*, const int64_t*,
                   const int64_t*, float, int, cudaStream_t) {
    return fail(FBB_ERR_ENUM, "flash64: not built yet");
}
}  // namespace fbb
