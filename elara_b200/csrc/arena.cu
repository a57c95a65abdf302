// Capacity-tier record arenas held in HBM: gather and scatter of records by physical id.
//
// The reference keeps its capacity tier in host memory as two payload arenas addressed by physical ids — MAT records
// [Mcap+1, 3, D] and log entries [Lcap+1, 1, D] (srm2/elara.py:40-48) — and moves records with multi-threaded memcpy loops
// (srm2/csrc/srm2_cpu.cpp:58-81: cpu_gather copies the first `ncomp` D-vectors of record rows[i] into out[i]; cpu_scatter
// writes src[i] over the first Wc D-vectors of record rows[i]).  On a B200 box the tier fits device memory (the 33.8 M-row
// store is 52 GB of MAT records at most); these two kernels are the same two copies on arenas that live there.
// One thread per 16-byte lane of one record; a record's lanes are consecutive threads, so every record moves as fully
// used runs of ncomp*D*4 bytes.  Bound by HBM bandwidth: ncomp*D*4 bytes read and written per record, plus 8 for the id.
#include "common.cuh"

namespace srm2 {

__global__ void __launch_bounds__(256)
srm2_arena_gather_kernel(float* __restrict__ out, const float* __restrict__ arena, const int64_t* __restrict__ ids, int64_t items,
                         int lanes, int64_t rec_floats, int64_t n_rec, uint32_t* __restrict__ bad) {
  const int64_t t = (int64_t)blockIdx.x * 256 + threadIdx.x;
  if (t >= items) return;
  const int64_t i = t / lanes; const int j = (int)(t - i * lanes) * 4;
  const int64_t r = ids[i];
  if (r < 0 || r >= n_rec) { if (bad) atomicOr(bad, 1u); return; }          // reported, never dereferenced
  st_stream4(out + i * (int64_t)lanes * 4 + j, *reinterpret_cast<const float4*>(arena + r * rec_floats + j));
}

__global__ void __launch_bounds__(256)
srm2_arena_scatter_kernel(float* __restrict__ arena, const float* __restrict__ src, const int64_t* __restrict__ ids, int64_t items,
                          int lanes, int64_t rec_floats, int64_t n_rec, uint32_t* __restrict__ bad) {
  const int64_t t = (int64_t)blockIdx.x * 256 + threadIdx.x;
  if (t >= items) return;
  const int64_t i = t / lanes; const int j = (int)(t - i * lanes) * 4;
  const int64_t r = ids[i];
  if (r < 0 || r >= n_rec) { if (bad) atomicOr(bad, 1u); return; }
  *reinterpret_cast<float4*>(arena + r * rec_floats + j) = ld_stream4(src + i * (int64_t)lanes * 4 + j);
}

static int arena_args(const void* a, const void* b, const int64_t* ids, int64_t n, int64_t n_rec, int64_t W, int64_t comp, int64_t D) {
  if (n < 0 || n_rec < 0 || W < 1 || comp < 1 || comp > W || D <= 0) return SRM2_ERR_ARG;
  if (n == 0) return SRM2_OK;
  if (a == nullptr || b == nullptr || ids == nullptr) return SRM2_ERR_ARG;
  if ((D & 3) != 0 || !aligned16(a) || !aligned16(b) || comp * D > ((int64_t)1 << 28)) return SRM2_ERR_UNSUPPORTED;
  return 1;
}

}  // namespace srm2

extern "C" int srm2_arena_gather_f32(float* out, const float* arena, const int64_t* ids, int64_t n, int64_t n_rec, int64_t W, int64_t ncomp,
                                     int64_t D, uint32_t* bad, srm2_stream_t stream) {
  using namespace srm2;
  const int rc = arena_args(out, arena, ids, n, n_rec, W, ncomp, D);
  if (rc <= 0) return rc;
  const int lanes = (int)(ncomp * D / 4);
  const int64_t items = n * lanes, blocks = (items + 255) / 256;
  if (blocks > 0x7fffffffLL) return SRM2_ERR_UNSUPPORTED;
  srm2_arena_gather_kernel<<<(unsigned)blocks, 256, 0, static_cast<cudaStream_t>(stream)>>>(out, arena, ids, items, lanes, W * D, n_rec, bad);
  return launch_status();
}

extern "C" int srm2_arena_scatter_f32(float* arena, const float* src, const int64_t* ids, int64_t n, int64_t n_rec, int64_t W, int64_t Wc,
                                      int64_t D, uint32_t* bad, srm2_stream_t stream) {
  using namespace srm2;
  const int rc = arena_args(arena, src, ids, n, n_rec, W, Wc, D);
  if (rc <= 0) return rc;
  const int lanes = (int)(Wc * D / 4);
  const int64_t items = n * lanes, blocks = (items + 255) / 256;
  if (blocks > 0x7fffffffLL) return SRM2_ERR_UNSUPPORTED;
  srm2_arena_scatter_kernel<<<(unsigned)blocks, 256, 0, static_cast<cudaStream_t>(stream)>>>(arena, src, ids, items, lanes, W * D, n_rec, bad);
  return launch_status();
}
