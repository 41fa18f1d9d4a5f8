// Library-level entry points of the C ABI (version, last CUDA error).
#include "common.cuh"

namespace b200 {
int g_last_cuda_error = 0;
}

extern "C" {

int b200_version(void) { return 1; }

int b200_last_cuda_error(void) { return b200::g_last_cuda_error; }

}  // extern "C"
