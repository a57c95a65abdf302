// Self-verification of the short correctly-rounded division and square-root sequences of exact.cuh against the
// compiler's IEEE operations, on the GPU that will run them (the approximations they start from come out of that GPU's
// own function unit).  Nothing here is on a product path; the tests call it through the C ABI.
//
//   SRM2_VERIFY_SQRT       every float bit pattern in [lo, hi) that lies in the guarded range: sqrt sequence vs sqrtf
//   SRM2_VERIFY_DIV_HARD   for every divisor significand B in [lo, hi) (B = 2^23 + index): all dividends whose quotient
//                          lies within `param` odd steps of a midpoint between two floats (the only quotients a sequence
//                          with a tiny final error can misround), both for A >= B and A < B; also checks |B*y - 1|
//   SRM2_VERIFY_DIV_ALL    every dividend significand against the divisor significands 2^23 + (i << param), i in [lo, hi)
//                          (param = 9 with i in [0, 2^14): exactly the divisors SRM2_VERIFY_DIV_HARD leaves out)
//   SRM2_VERIFY_DIV_RANDOM `hi - lo` pseudo-random pairs (seed lo) with exponents spread over the guarded range
//   SRM2_VERIFY_ADAM       `hi - lo` pseudo-random Adam steps on four elements (seed lo): the packed step against the plain
//                          IEEE one; param 0: operands as in training, 1: arbitrary bit patterns
#include "common.cuh"
#include "exact.cuh"

namespace srm2 {

struct VerifyOut { unsigned long long tested, mismatches, first_a, first_b, aux; };

__device__ __forceinline__ void report(VerifyOut* o, float a, float b) {
  if (atomicAdd(&o->mismatches, 1ull) == 0ull) { o->first_a = __float_as_uint(a); o->first_b = __float_as_uint(b); }
}

template <int VARIANT>
__global__ void __launch_bounds__(256) srm2_verify_sqrt_kernel(uint64_t lo, uint64_t hi, VerifyOut* o) {
  unsigned long long tested = 0;
  for (uint64_t u = lo + (uint64_t)blockIdx.x * 256 + threadIdx.x; u < hi; u += (uint64_t)gridDim.x * 256) {
    const float x = __uint_as_float((uint32_t)u);
    if (!(x >= 1.0842021724855044e-19f * 0.25f && x <= 1.1529215046068469e+18f * 4.0f)) continue;     // [2^-66, 2^62]
    const pf2 s = sqrt2_t<VARIANT>(pk1(x), exact_const());
    const float t = __fsqrt_rn(x);
    ++tested;
    if (__float_as_uint(lo_of(s)) != __float_as_uint(t) || __float_as_uint(hi_of(s)) != __float_as_uint(t)) report(o, x, 0.f);
  }
  atomicAdd(&o->tested, tested);
}

template <int CORR>
__device__ __forceinline__ bool div_matches(float a, float b) {
  const pf2 nb = pk1(-b);
  const pf2 q = div2_y_t<CORR>(pk1(a), nb, rcp2(pk1(b), nb, exact_const()));
  const float t = __fdiv_rn(a, b);
  return __float_as_uint(lo_of(q)) == __float_as_uint(t) && __float_as_uint(hi_of(q)) == __float_as_uint(t);
}

__device__ __forceinline__ uint32_t inverse_mod_2_32(uint32_t b) {       // b odd
  uint32_t x = b;                                                       // correct to 3 bits
#pragma unroll
  for (int i = 0; i < 5; ++i) x *= 2u - b * x;
  return x;
}

// one thread per (divisor significand, odd offset rho' = +-(2j+1)); ea / eb: biased exponents given to a and b
template <int CORR>
__global__ void __launch_bounds__(256)
srm2_verify_div_hard_kernel(uint32_t lo, uint32_t hi, int nrho, int max_s, uint32_t ea, uint32_t eb, VerifyOut* o) {
  const uint64_t t = (uint64_t)blockIdx.x * 256 + threadIdx.x;
  const uint64_t per = 2ull * nrho;
  if (t >= (uint64_t)(hi - lo) * per) return;
  const uint32_t B = (1u << 23) + lo + (uint32_t)(t / per);
  const int ri = (int)(t % per);
  const int64_t rho = (ri & 1) ? -(int64_t)(2 * (ri >> 1) + 1) : (int64_t)(2 * (ri >> 1) + 1);
  const int s = __ffs(B) - 1;
  if (s > max_s) return;                                   // those divisors are covered by SRM2_VERIFY_DIV_ALL
  const uint32_t Bo = B >> s;
  const uint32_t inv = inverse_mod_2_32(Bo);
  const float b = __uint_as_float((eb << 23) | (B & 0x7fffffu));
  unsigned long long tested = 0;
  if (ri == 0) {                                           // accuracy of the refined reciprocal of this divisor
    const float y = rcp1(b);
    const double err = fabs((double)b * (double)y - 1.0);
    if (err > 2.384185791015625e-07) atomicAdd(&o->aux, 1ull);       // 2^-22
  }
  for (int scale = 24; scale <= 25; ++scale) {             // 24: A >= B, quotient in [1,2); 25: A < B, quotient in [1/2,1)
    const int mbits = scale - s;                           // N is fixed modulo 2^mbits
    const uint32_t mask = (mbits >= 32) ? 0xffffffffu : ((1u << mbits) - 1u);
    const uint32_t n0 = ((uint32_t)(-rho) * inv) & mask;   // N = -rho' * Bo^-1 (mod 2^mbits)
    for (uint32_t k = 0; k < (1u << s); ++k) {
      uint64_t N = (uint64_t)n0 + ((uint64_t)k << mbits);
      if (scale == 24) N += 1ull << 24;
      if (N < (1ull << 24) || N >= (1ull << 25) || !(N & 1ull)) continue;
      const int64_t num = (int64_t)((uint64_t)B * N) + rho * ((int64_t)1 << s);
      if (num & (((int64_t)1 << scale) - 1)) continue;     // cannot happen by construction
      const int64_t A = num >> scale;
      if (A < (1 << 23) || A >= (1 << 24)) continue;
      const float a = __uint_as_float((ea << 23) | ((uint32_t)A & 0x7fffffu));
      ++tested;
      if (!div_matches<CORR>(a, b)) report(o, a, b);
    }
  }
  atomicAdd(&o->tested, tested);
}

template <int CORR>
__global__ void __launch_bounds__(256)
srm2_verify_div_all_kernel(uint32_t lo, uint32_t ea, uint32_t eb, int stride_log2, VerifyOut* o) {
  const uint32_t B = (1u << 23) + ((lo + blockIdx.y) << stride_log2);
  const float b = __uint_as_float((eb << 23) | (B & 0x7fffffu));
  unsigned long long tested = 0;
  for (uint32_t A = blockIdx.x * 256 + threadIdx.x; A < (1u << 23); A += gridDim.x * 256) {
    const float a = __uint_as_float((ea << 23) | A);
    ++tested;
    if (!div_matches<CORR>(a, b)) report(o, a, b);
  }
  atomicAdd(&o->tested, tested);
}

__device__ __forceinline__ uint64_t splitmix(uint64_t x) {
  x += 0x9E3779B97F4A7C15ull; x = (x ^ (x >> 30)) * 0xBF58476D1CE4E5B9ull; x = (x ^ (x >> 27)) * 0x94D049BB133111EBull;
  return x ^ (x >> 31);
}

template <int CORR>
__global__ void __launch_bounds__(256) srm2_verify_div_random_kernel(uint64_t seed, uint64_t count, VerifyOut* o) {
  unsigned long long tested = 0;
  for (uint64_t i = (uint64_t)blockIdx.x * 256 + threadIdx.x; i < count; i += (uint64_t)gridDim.x * 256) {
    const uint64_t r = splitmix(seed * 0x100000001B3ull + i), r2 = splitmix(r);
    // dividend in [2^-90, 2^64), divisor in [2^-36, 2^31), either sign for the dividend
    const uint32_t ea = 127 - 90 + (uint32_t)(r2 % 154u), eb = 127 - 36 + (uint32_t)((r2 >> 20) % 67u);
    const float a = __uint_as_float(((uint32_t)(r2 >> 63) << 31) | (ea << 23) | ((uint32_t)r & 0x7fffffu));
    const float b = __uint_as_float((eb << 23) | ((uint32_t)(r >> 32) & 0x7fffffu));
    const float q = __fdiv_rn(a, b);
    if (!(fabsf(q) >= 1.1754943508222875e-38f)) continue;            // quotient below the normal range: not in the guarded range
    ++tested;
    if (!div_matches<CORR>(a, b)) report(o, a, b);
  }
  atomicAdd(&o->tested, tested);
}

// The whole step: adam_vec4_fast against the plain IEEE step (adam_vec4), bit for bit, on pseudo-random operands.
// mode 0: operands as they occur in training (|w| ~ 1e-2, |g| ~ 1e-3 down to 1e-9, m and v their running averages, steps
// 1..4000 of the default hyper-parameters); mode 1: arbitrary bit patterns for everything, scalars included (zeros,
// subnormals, infinities and NaNs among them: the range check must route those to the IEEE path).
__global__ void __launch_bounds__(256) srm2_verify_adam_kernel(uint64_t seed, uint64_t count, int mode, VerifyOut* o) {
  unsigned long long tested = 0;
  for (uint64_t i = (uint64_t)blockIdx.x * 256 + threadIdx.x; i < count; i += (uint64_t)gridDim.x * 256) {
    uint64_t r = splitmix(seed * 0x100000001B3ull + i);
    auto next = [&]() { r = splitmix(r); return (uint32_t)(r >> 16); };
    auto any = [&]() { return __uint_as_float(next()); };
    auto scaled = [&](int e_lo, int e_hi) {       // random sign and significand, exponent uniform in [e_lo, e_hi]
      const uint32_t u = next(), e = (uint32_t)(127 + e_lo) + next() % (uint32_t)(e_hi - e_lo + 1);
      return __uint_as_float((u & 0x807fffffu) | (e << 23));
    };
    AdamSc s; float4 w, m, v, g;
    float* wp = &w.x; float* mp = &m.x; float* vp = &v.x; float* gp = &g.x;
    if (mode == 0) {
      const int step = 1 + (int)(next() % 4000u);
      s.lr = 1e-3f; s.b1 = 0.9f; s.omb1 = (float)(1.0 - 0.9); s.b2 = 0.999f; s.omb2 = (float)(1.0 - 0.999); s.eps = 1e-8f;
      s.bc1 = (float)(1.0 - pow(0.9, (double)step)); s.bc2 = (float)(1.0 - pow(0.999, (double)step));
      for (int e = 0; e < 4; ++e) {
        wp[e] = scaled(-12, -4); gp[e] = scaled(-30, -8); mp[e] = (next() & 7u) ? scaled(-30, -8) : 0.f;
        vp[e] = (next() & 7u) ? fabsf(scaled(-60, -16)) : 0.f;
      }
    } else {
      s.lr = any(); s.b1 = any(); s.omb1 = any(); s.b2 = any(); s.omb2 = any(); s.bc1 = any(); s.bc2 = any(); s.eps = any();
      if (next() & 1u) { s.lr = fabsf(scaled(-26, 5)); s.bc1 = fabsf(scaled(-22, 2)); s.bc2 = fabsf(scaled(-22, 2)); s.eps = fabsf(scaled(-40, 5)); }
      for (int e = 0; e < 4; ++e) { wp[e] = any(); gp[e] = any(); mp[e] = any(); vp[e] = any(); }
      if (next() & 1u) for (int e = 0; e < 4; ++e) { gp[e] = scaled(-70, 30); mp[e] = scaled(-70, 30); vp[e] = fabsf(scaled(-70, 42)); }
    }
    float4 w1 = w, m1 = m, v1 = v, w2 = w, m2 = m, v2 = v;
    adam_vec4(w1, m1, v1, g, s);
    adam_vec4_fast(w2, m2, v2, g, adam_fast_prepare(s));
    ++tested;
    const float* a = &w1.x; const float* b = &w2.x; const float* c = &m1.x; const float* d = &m2.x; const float* e1 = &v1.x; const float* f1 = &v2.x;
    bool same = true;
    for (int e = 0; e < 4; ++e)
      same = same && __float_as_uint(a[e]) == __float_as_uint(b[e]) && __float_as_uint(c[e]) == __float_as_uint(d[e]) &&
             __float_as_uint(e1[e]) == __float_as_uint(f1[e]);
    if (!same) report(o, g.x, m.x);
  }
  atomicAdd(&o->tested, tested);
}

}  // namespace srm2

extern "C" int srm2_verify_exact(int what, uint64_t lo, uint64_t hi, int variant, int param, uint64_t* out5, srm2_stream_t stream) {
  using namespace srm2;
  if (out5 == nullptr || hi < lo) return SRM2_ERR_ARG;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  VerifyOut* o = reinterpret_cast<VerifyOut*>(out5);
  const uint32_t e = 127;
  switch (what) {
    case SRM2_VERIFY_SQRT: {
      if (hi > (1ull << 32)) return SRM2_ERR_ARG;
      const int grid = kSMs * 16;
      if (variant == 1) srm2_verify_sqrt_kernel<1><<<grid, 256, 0, st>>>(lo, hi, o);
      else if (variant == 2) srm2_verify_sqrt_kernel<2><<<grid, 256, 0, st>>>(lo, hi, o);
      else if (variant == 3) srm2_verify_sqrt_kernel<3><<<grid, 256, 0, st>>>(lo, hi, o);
      else return SRM2_ERR_ARG;
      break;
    }
    case SRM2_VERIFY_DIV_HARD: {
      if (hi > (1ull << 23) || param < 1 || param > 4096) return SRM2_ERR_ARG;
      const uint64_t threads = (hi - lo) * 2ull * (uint64_t)param;
      const uint64_t blocks = (threads + 255) / 256;
      if (blocks == 0) return SRM2_OK;
      if (blocks > 0x7fffffffull) return SRM2_ERR_UNSUPPORTED;
      if (variant == 1) srm2_verify_div_hard_kernel<1><<<(unsigned)blocks, 256, 0, st>>>((uint32_t)lo, (uint32_t)hi, param, 8, e, e, o);
      else if (variant == 2) srm2_verify_div_hard_kernel<2><<<(unsigned)blocks, 256, 0, st>>>((uint32_t)lo, (uint32_t)hi, param, 8, e, e, o);
      else return SRM2_ERR_ARG;
      break;
    }
    case SRM2_VERIFY_DIV_ALL: {
      if (param < 0 || param > 22 || hi > (1ull << (23 - param)) || hi - lo > 65535) return SRM2_ERR_ARG;
      if (hi == lo) return SRM2_OK;
      const dim3 grid(kSMs * 4, (unsigned)(hi - lo));
      if (variant == 1) srm2_verify_div_all_kernel<1><<<grid, 256, 0, st>>>((uint32_t)lo, e, e, param, o);
      else if (variant == 2) srm2_verify_div_all_kernel<2><<<grid, 256, 0, st>>>((uint32_t)lo, e, e, param, o);
      else return SRM2_ERR_ARG;
      break;
    }
    case SRM2_VERIFY_DIV_RANDOM: {
      const int grid = kSMs * 16;
      if (variant == 1) srm2_verify_div_random_kernel<1><<<grid, 256, 0, st>>>(lo, hi - lo, o);
      else if (variant == 2) srm2_verify_div_random_kernel<2><<<grid, 256, 0, st>>>(lo, hi - lo, o);
      else return SRM2_ERR_ARG;
      break;
    }
    case SRM2_VERIFY_ADAM: {
      if (param < 0 || param > 1) return SRM2_ERR_ARG;
      srm2_verify_adam_kernel<<<kSMs * 16, 256, 0, st>>>(lo, hi - lo, param, o);
      break;
    }
    default: return SRM2_ERR_ARG;
  }
  return launch_status();
}
