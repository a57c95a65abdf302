// Host-side entry points: library identification, status text, Adam scalars.
#include <atomic>
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

static std::atomic<int64_t> g_launches{0};
void add_launches(int k) { g_launches.fetch_add(k, std::memory_order_relaxed); }

static thread_local cudaEvent_t g_ev_begin = nullptr, g_ev_end = nullptr;
void stage_begin(cudaStream_t st) { if (g_ev_begin) note_cuda(cudaEventRecord(g_ev_begin, st)); }
void stage_end(cudaStream_t st) { if (g_ev_end) note_cuda(cudaEventRecord(g_ev_end, st)); }

}  // namespace srm2

extern "C" int srm2_version(void) { return 100; }

extern "C" int64_t srm2_launch_count(void) { return srm2::g_launches.load(std::memory_order_relaxed); }

extern "C" int srm2_stage_events(void* begin, void* end) {
  srm2::g_ev_begin = static_cast<cudaEvent_t>(begin);
  srm2::g_ev_end = static_cast<cudaEvent_t>(end);
  return SRM2_OK;
}

extern "C" const char* srm2_status_string(int status) {
  switch (status) {
    case SRM2_OK: return "ok";
    case SRM2_ERR_ARG: return "invalid argument";
    case SRM2_ERR_UNSUPPORTED: return "size not supported";
    case SRM2_ERR_SCRATCH: return "scratch buffer too small";
    case SRM2_ERR_CUDA: return "CUDA runtime error";
    case SRM2_ERR_LIMIT: return "size exceeds the built-in scratch of the no-allocation entry point";
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
