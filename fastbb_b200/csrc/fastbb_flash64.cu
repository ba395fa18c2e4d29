// Translation unit of libfastbb_flash64.so: the attention kernel and its entry points only (fbb_flash64_f16,
// fbb_flash64_f16_ws, fbb_flash64_f16_static, fbb_flash64_workspace_bytes and the version / status calls). This is the
// part of the library that projects which vendor only the reference's attention.py + kernels.py consume.
#define FBB_FLASH_ONLY 1
#include "flash64.cu"
#include "api.cu"
