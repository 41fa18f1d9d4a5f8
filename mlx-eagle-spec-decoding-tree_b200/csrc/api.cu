// Library-level entry points of the C ABI (version, last CUDA error, launch options).
#include "common.cuh"

namespace b200 {
int g_last_cuda_error = 0;
int g_use_pdl = 1;
unsigned g_wait_limit = 0;
}

extern "C" {

int b200_version(void) { return 1; }

int b200_last_cuda_error(void) { return b200::g_last_cuda_error; }

void b200_set_pdl(int enabled) { b200::g_use_pdl = enabled ? 1 : 0; }

void b200_set_wait_limit(unsigned int polls) { b200::g_wait_limit = polls; }

}  // extern "C"
