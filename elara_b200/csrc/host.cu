// Host-side entry points: library identification, status text, Adam scalars.
#include <cmath>
#include <cstring>

#include "common.cuh"

namespace srm2 {

static thread_local char g_cuda_err[256] = "";

int note_cuda(cudaError_t e) {
  if (e == cudaSuccess) return SRM2_OK;
  std::strncpy(g_cuda_err, cudaGetErrorString(e), sizeof(g_cuda_err) - 1);
  g_cuda_err[sizeof(g_cuda_err) - 1] = '\0';
  return SRM2_ERR_CUDA;
}

}  // namespace srm2

extern "C" int srm2_version(void) { return 100; }

extern "C" const char* srm2_status_string(int status) {
  switch (status) {
    case SRM2_OK: return "ok";
    case SRM2_ERR_ARG: return "invalid argument";
    case SRM2_ERR_UNSUPPORTED: return "size not supported";
    case SRM2_ERR_SCRATCH: return "scratch buffer too small";
    case SRM2_ERR_CUDA: return "CUDA runtime error";
    default: return "unknown status";
  }
}

extern "C" const char* srm2_last_cuda_error(void) { return srm2::g_cuda_err; }

// Double-precision evaluation, one rounding to float per value (srm2/csrc/srm2_cpu.cpp:15-20).
extern "C" int srm2_adam_scalars(double lr, double b1, double b2, double eps, int64_t step, float out[8]) {
  if (out == nullptr) return SRM2_ERR_ARG;
  out[0] = (float)lr;
  out[1] = (float)b1;
  out[2] = (float)(1.0 - b1);
  out[3] = (float)b2;
  out[4] = (float)(1.0 - b2);
  out[5] = (float)(1.0 - std::pow(b1, (double)step));
  out[6] = (float)(1.0 - std::pow(b2, (double)step));
  out[7] = (float)eps;
  return SRM2_OK;
}
