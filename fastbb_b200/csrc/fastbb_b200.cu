// Single translation unit of libfastbb_b200.so: the kernels share one device status word and one set of inline PTX
// helpers, so they are compiled together (no relocatable device code, no device link step).
#include "layernorm.cu"
#include "gemm.cu"
#include "flash64.cu"
#include "block.cu"
#include "api.cu"
