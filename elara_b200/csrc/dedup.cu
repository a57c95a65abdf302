// Deterministic dedup of row ids from a bounded universe [0, n_rows): sorted unique ids and, per lookup,
// the index of its id in that list — what torch.unique(ids, return_inverse=True) returns.
//
// No sort is needed.  A bitmap with one bit per row (n_rows/8 bytes: 4.2 MB for 33.8 M rows, 25 MB for
// 200 M rows — resident in the 126 MB L2) is marked with the ids; the rank of an id among the distinct ids
// is the number of set bits below it, i.e. an exclusive prefix sum of per-word popcounts plus a popcount
// inside its word.  Kernels: mark -> per-block popcount sums (+ scan of the block sums by the last block
// to finish) -> per-word prefixes and emission of the unique ids -> inverse.  Integer work on an
// L2-resident table: latency-bound, a few microseconds each.
#include <atomic>

#include "common.cuh"
#include "scan.cuh"

namespace srm2 {

constexpr int kDT = 256;                    // threads per block
constexpr int kWordsPerThread = 4;
constexpr int kWordsPerBlock = kDT * kWordsPerThread;   // 1024 words = 32768 rows per block

struct DedupScratch {
  uint32_t* bitmap;     // [words]
  uint32_t* wprefix;    // [words]    number of distinct ids below word w
  uint32_t* bsum;       // [nblocks]  distinct ids per block of words, then its exclusive scan
  uint32_t* counter;    // [1]        blocks finished (returns to 0 at the end of every call)
  uint32_t* flag;       // [1]        an id outside [0, n_rows) was seen
  int64_t words, nblocks;
};

static size_t align_up(size_t x, size_t a) { return (x + a - 1) / a * a; }

static size_t dedup_layout(int64_t n_rows, char* base, DedupScratch* s) {
  const int64_t words = (n_rows + 31) / 32;
  const int64_t nblocks = (words + kWordsPerBlock - 1) / kWordsPerBlock;
  size_t off = 0;
  auto take = [&](size_t bytes) { size_t o = off; off = align_up(off + bytes, 256); return o; };
  const size_t o_bm = take((size_t)(nblocks * kWordsPerBlock) * 4 + 256);   // padded to whole blocks; counter and flag behind it
  const size_t o_wp = take((size_t)(nblocks * kWordsPerBlock) * 4);
  const size_t o_bs = take((size_t)(nblocks + 1) * 4);
  if (s) {
    s->bitmap = reinterpret_cast<uint32_t*>(base + o_bm); s->wprefix = reinterpret_cast<uint32_t*>(base + o_wp);
    s->bsum = reinterpret_cast<uint32_t*>(base + o_bs); s->counter = s->bitmap + nblocks * kWordsPerBlock; s->flag = s->counter + 1;
    s->words = words; s->nblocks = nblocks;
  }
  return off;
}

// Marks the ids of one chunk of lookups.  Hot rows are looked up thousands of times per batch and the hottest ids of a
// table share a bitmap word, so naive atomics serialise on a few words in L2.  Each CTA therefore first ORs its bits
// into a direct-mapped shared-memory cache keyed by word index (collisions fall through to a global atomic) and then
// flushes every cached word with a single global atomicOr.
// *flag = 1 if an id outside [0, n_rows) was seen (it is ignored; its inverse is -1); the count kernel reports it.
constexpr int kMarkPerThread = 8;
constexpr int kMarkSlots = 2048;
__global__ void __launch_bounds__(kDT)
srm2_unique_mark_kernel(const int64_t* __restrict__ ids, int64_t n_host, const int64_t* __restrict__ n_dev, int64_t n_rows,
                        uint32_t* __restrict__ bitmap, uint32_t* __restrict__ flag) {
  const int64_t n = eff_count(n_host, n_dev);
  __shared__ uint32_t tag[kMarkSlots];
  __shared__ uint32_t val[kMarkSlots];
  for (int i = threadIdx.x; i < kMarkSlots; i += kDT) { tag[i] = 0xffffffffu; val[i] = 0u; }
  __syncthreads();
  const int64_t base = (int64_t)blockIdx.x * (kDT * kMarkPerThread);
  int64_t id[kMarkPerThread];
#pragma unroll
  for (int k = 0; k < kMarkPerThread; ++k) {
    const int64_t p = base + k * kDT + threadIdx.x;
    id[k] = p < n ? ids[p] : -2;
  }
#pragma unroll
  for (int k = 0; k < kMarkPerThread; ++k) {
    if (id[k] == -2) continue;
    if (id[k] < 0 || id[k] >= n_rows) { *flag = 1u; continue; }
    const uint32_t w = (uint32_t)(id[k] >> 5), bit = 1u << (id[k] & 31);
    const uint32_t slot = (w * 2654435761u) >> (32 - 11);
    const uint32_t prev = atomicCAS(&tag[slot], 0xffffffffu, w);
    if (prev == 0xffffffffu || prev == w) atomicOr(&val[slot], bit);
    else atomicOr(bitmap + w, bit);
  }
  __syncthreads();
  for (int i = threadIdx.x; i < kMarkSlots; i += kDT)
    if (tag[i] != 0xffffffffu) atomicOr(bitmap + tag[i], val[i]);
}

// Per block of 1024 words: number of set bits (a CTA takes every gridDim.x-th block).  The last CTA to finish turns bsum
// into its exclusive scan and writes the total (= number of unique ids).
__global__ void __launch_bounds__(kDT)
srm2_unique_count_kernel(const uint32_t* __restrict__ bitmap, uint32_t* __restrict__ bsum, uint32_t* __restrict__ counter,
                         const uint32_t* __restrict__ flag, int64_t nblocks, int64_t* __restrict__ out_count) {
  __shared__ uint32_t ws[33];
  __shared__ bool last;
  for (int64_t blk = blockIdx.x; blk < nblocks; blk += gridDim.x) {
    const uint4* src = reinterpret_cast<const uint4*>(bitmap + blk * kWordsPerBlock) + threadIdx.x * (kWordsPerThread / 4);
    uint32_t c = 0;
#pragma unroll
    for (int k = 0; k < kWordsPerThread / 4; ++k) { const uint4 v = src[k]; c += __popc(v.x) + __popc(v.y) + __popc(v.z) + __popc(v.w); }
    uint32_t total;
    block_exclusive_scan<kDT>(c, ws, &total);
    if (threadIdx.x == 0) bsum[blk] = total;
    __syncthreads();                                   // ws is reused by the next block of words
  }
  if (threadIdx.x == 0) {
    __threadfence();
    last = atomicAdd(counter, 1u) == gridDim.x - 1u;
  }
  __syncthreads();
  if (!last) return;
  __threadfence();
  // exclusive scan of bsum[0..nblocks) by this block, in rounds of 4 * kDT entries (thread t: entries 4t .. 4t+3)
  uint32_t carry = 0;
  for (int64_t base = 0; base < nblocks; base += 4 * kDT) {
    const int64_t i0 = base + 4 * (int64_t)threadIdx.x;
    uint32_t v[4];
#pragma unroll
    for (int e = 0; e < 4; ++e) v[e] = i0 + e < nblocks ? reinterpret_cast<volatile uint32_t*>(bsum)[i0 + e] : 0u;
    uint32_t tot;
    uint32_t run = carry + block_exclusive_scan<kDT>(v[0] + v[1] + v[2] + v[3], ws, &tot);
#pragma unroll
    for (int e = 0; e < 4; ++e) { if (i0 + e < nblocks) bsum[i0 + e] = run; run += v[e]; }
    carry += tot;
  }
  if (threadIdx.x == 0) { out_count[0] = (int64_t)carry; out_count[1] = (int64_t)*flag; *counter = 0u; }
}

// Per word: exclusive prefix of distinct ids; every set bit writes its id at its rank.
// The prefixes are computed with each thread owning 4 consecutive words (one 16-byte load).
__global__ void __launch_bounds__(kDT)
srm2_unique_emit_kernel(const uint32_t* __restrict__ bitmap, const uint32_t* __restrict__ bsum, uint32_t* __restrict__ wprefix,
                        int64_t* __restrict__ uniq, int64_t uniq_cap, int64_t nblocks) {
  __shared__ uint32_t ws[33];
  __shared__ uint32_t s_w[kWordsPerBlock];
  __shared__ uint32_t s_p[kWordsPerBlock];
  for (int64_t blk = blockIdx.x; blk < nblocks; blk += gridDim.x) {
    const int64_t wb = blk * kWordsPerBlock;
    const int t0 = threadIdx.x * kWordsPerThread;
    uint32_t wv[kWordsPerThread];
    const uint4* src = reinterpret_cast<const uint4*>(bitmap + wb + t0);
    const uint32_t bbase = bsum[blk];
    uint32_t c = 0;
#pragma unroll
    for (int k = 0; k < kWordsPerThread / 4; ++k) {
      const uint4 v = src[k];
      wv[4 * k] = v.x; wv[4 * k + 1] = v.y; wv[4 * k + 2] = v.z; wv[4 * k + 3] = v.w;
      c += __popc(v.x) + __popc(v.y) + __popc(v.z) + __popc(v.w);
    }
    uint32_t total;
    uint32_t run = bbase + block_exclusive_scan<kDT>(c, ws, &total);
    uint32_t pf[kWordsPerThread];
#pragma unroll
    for (int k = 0; k < kWordsPerThread; ++k) { pf[k] = run; run += __popc(wv[k]); s_w[t0 + k] = wv[k]; s_p[t0 + k] = pf[k]; }
    uint4* dst = reinterpret_cast<uint4*>(wprefix + wb + t0);
#pragma unroll
    for (int k = 0; k < kWordsPerThread / 4; ++k) dst[k] = make_uint4(pf[4 * k], pf[4 * k + 1], pf[4 * k + 2], pf[4 * k + 3]);
    __syncthreads();
    // ids: the words are dealt round-robin to the threads (word i -> thread i mod 256), so a run of dense words (the
    // frequent ids of a table are its smallest) is spread over many threads instead of piling up in one
    if (total != 0) {                                  // uniform: anything to emit in this block of words?
      for (int i = threadIdx.x; i < kWordsPerBlock; i += kDT) {
        uint32_t bits = s_w[i]; uint32_t r = s_p[i];
        while (bits) {
          const int b = __ffs(bits) - 1; bits &= bits - 1;
          if ((int64_t)r < uniq_cap) uniq[r] = ((wb + i) << 5) + b;
          ++r;
        }
      }
    }
    __syncthreads();                                   // s_w, s_p and ws are reused by the next block of words
  }
}

__global__ void __launch_bounds__(kDT)
srm2_unique_inverse_kernel(const int64_t* __restrict__ ids, int64_t n_host, const int64_t* __restrict__ n_dev, int64_t n_rows,
                           const uint32_t* __restrict__ bitmap, const uint32_t* __restrict__ wprefix, int64_t* __restrict__ inv) {
  const int64_t n = eff_count(n_host, n_dev);
  for (int64_t p = (int64_t)blockIdx.x * kDT + threadIdx.x; p < n; p += (int64_t)gridDim.x * kDT) {
    const int64_t id = ids[p];
    if (id < 0 || id >= n_rows) { inv[p] = -1; continue; }
    const uint32_t w = bitmap[id >> 5];
    inv[p] = (int64_t)(wprefix[id >> 5] + __popc(w & ((1u << (id & 31)) - 1u)));
  }
}

}  // namespace srm2

extern "C" size_t srm2_unique_scratch_bytes(int64_t n_rows) {
  if (n_rows <= 0) return 256;
  return srm2::dedup_layout(n_rows, nullptr, nullptr);
}

extern "C" int srm2_unique_inverse_i64(const int64_t* ids, int64_t n, int64_t n_rows, int64_t* uniq, int64_t uniq_cap,
                                       int64_t* inv, int64_t* out_count, void* scratch, size_t scratch_bytes,
                                       srm2_stream_t stream) {
  return srm2_unique_inverse_nd_i64(ids, n, nullptr, n_rows, uniq, uniq_cap, inv, out_count, scratch, scratch_bytes, stream);
}

extern "C" int srm2_unique_inverse_nd_i64(const int64_t* ids, int64_t n, const int64_t* n_dev, int64_t n_rows, int64_t* uniq,
                                          int64_t uniq_cap, int64_t* inv, int64_t* out_count, void* scratch,
                                          size_t scratch_bytes, srm2_stream_t stream) {
  using namespace srm2;
  if (n < 0 || n_rows <= 0 || uniq_cap < 0 || out_count == nullptr) return SRM2_ERR_ARG;
  if (n > 0 && (ids == nullptr || inv == nullptr)) return SRM2_ERR_ARG;
  if (uniq_cap > 0 && uniq == nullptr) return SRM2_ERR_ARG;
  if (n_rows > (int64_t)1 << 36 || n >= (int64_t)1 << 31) return SRM2_ERR_UNSUPPORTED;
  if (scratch == nullptr || !aligned16(scratch) || scratch_bytes < dedup_layout(n_rows, nullptr, nullptr)) return SRM2_ERR_SCRATCH;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  DedupScratch s;
  dedup_layout(n_rows, static_cast<char*>(scratch), &s);
  // bitmap (padded to whole blocks), block sums and the finished-blocks counter start at zero
  if (note_cuda(cudaMemsetAsync(s.bitmap, 0, (size_t)(s.nblocks * kWordsPerBlock) * 4 + 8, st))) return SRM2_ERR_CUDA;   // + counter, flag
  const unsigned grid_n = index_grid((n + kDT - 1) / kDT);
  const int64_t mark_blocks = (n + kDT * kMarkPerThread - 1) / (kDT * kMarkPerThread);
  if (n > 0) srm2_unique_mark_kernel<<<(unsigned)mark_blocks, kDT, 0, st>>>(ids, n, n_dev, n_rows, s.bitmap, s.flag);
  srm2_unique_count_kernel<<<index_grid(s.nblocks), kDT, 0, st>>>(s.bitmap, s.bsum, s.counter, s.flag, s.nblocks, out_count);
  srm2_unique_emit_kernel<<<index_grid(s.nblocks), kDT, 0, st>>>(s.bitmap, s.bsum, s.wprefix, uniq, uniq_cap, s.nblocks);
  if (n > 0) srm2_unique_inverse_kernel<<<grid_n, kDT, 0, st>>>(ids, n, n_dev, n_rows, s.bitmap, s.wprefix, inv);
  return launch_status(n > 0 ? 4 : 2);
}

// ---------------------------------------------------------------------------------------------------------
// Dedup without caller-supplied scratch.
//
// Some hosts of this library are not in a position to hand over a scratch buffer, because they must not allocate
// device memory at the point where they need a dedup: a process whose device memory is capped and already fully
// committed to its tables (the reference driver can cap itself that way), a latency-critical loop that cannot afford
// the implicit device synchronisation an allocation or a free may bring, or an embedding host in which another
// component owns every byte of device memory.  For them the same kernels run on a fixed scratch area that is part of
// the library image: a file-scope __device__ array.  Each GPU that loads the library carries it (about 1 MiB) until
// the process exits.  Its size bounds the universe: at most kNoAllocMaxRows row ids.
//
// The array's name is only a host-side handle; the kernels need its device address, which the runtime reports per
// device.  The first call on a device looks the address up (cudaGetSymbolAddress, with that device current) and keeps
// it; later calls on that device reuse it.
namespace srm2 {

constexpr int64_t kNoAllocMaxRows = 4194304;                                   // 2^22 rows
constexpr size_t kNoAllocScratchBytes = 2 * (size_t)(kNoAllocMaxRows / 32) * 4 + 4096;   // bitmap + word prefixes + counters

static __device__ __align__(256) unsigned char g_noalloc_scratch[kNoAllocScratchBytes];

constexpr int kNoAllocMaxDevices = 64;
static std::atomic<void*> g_noalloc_addr[kNoAllocMaxDevices];                  // device address of the array, per device

// Device address of g_noalloc_scratch on the current device (looked up once per device), or nullptr with *rc set.
static void* noalloc_scratch_address(int* rc) {
  int dev = -1;
  if ((*rc = note_cuda(cudaGetDevice(&dev))) != SRM2_OK) return nullptr;
  if (dev < 0 || dev >= kNoAllocMaxDevices) { *rc = SRM2_ERR_UNSUPPORTED; return nullptr; }
  void* p = g_noalloc_addr[dev].load(std::memory_order_acquire);
  if (p == nullptr) {
    if ((*rc = note_cuda(cudaGetSymbolAddress(&p, g_noalloc_scratch))) != SRM2_OK) return nullptr;
    g_noalloc_addr[dev].store(p, std::memory_order_release);                   // every thread finds the same address
  }
  return p;
}

}  // namespace srm2

extern "C" int64_t srm2_unique_noalloc_max_rows(void) { return srm2::kNoAllocMaxRows; }

extern "C" int srm2_unique_inverse_noalloc_i64(const int64_t* ids, int64_t n, int64_t n_rows, int64_t* uniq, int64_t uniq_cap,
                                               int64_t* inv, int64_t* out_count, srm2_stream_t stream) {
  using namespace srm2;
  if (n_rows <= 0) return SRM2_ERR_ARG;
  if (n_rows > kNoAllocMaxRows || dedup_layout(n_rows, nullptr, nullptr) > kNoAllocScratchBytes) return SRM2_ERR_LIMIT;
  int rc = SRM2_OK;
  void* scratch = noalloc_scratch_address(&rc);
  if (scratch == nullptr) return rc;
  // The shared array still holds whatever the previous call left there.  The dedup entry point clears everything that
  // has to start at zero (bitmap, block counter, result counts) on the caller's stream before its kernels run.
  return srm2_unique_inverse_i64(ids, n, n_rows, uniq, uniq_cap, inv, out_count, scratch, kNoAllocScratchBytes, stream);
}
