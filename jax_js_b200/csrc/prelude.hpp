// Device-side prelude prepended to every NVRTC-compiled kernel.
//
// Scalar semantics follow the reference's Wasm emitter (src/backend/wasm/translation.ts)
// and its software transcendentals (src/backend/wasm/builtins.ts), so that results agree
// with the Wasm backend far inside the 1e-5 bar instead of differing wherever that
// backend's own approximations are loose (its log is ~1.7e-5 off near mantissa 2, its
// sin/cos reduce the argument in f32).  Only the algorithm is shared: the functions are
// written for CUDA (fused multiply-adds allowed, so results may differ by an ulp).
#pragma once

namespace jaxcuda {

static const char* const kPrelude = R"PRELUDE(
typedef unsigned int u32;
typedef unsigned short u16;
typedef long long i64;
typedef unsigned long long u64;

struct __align__(2) jx_half { u16 x; };

#ifdef JX_CHECKED
// Checked build: an index outside its buffer is counted at JX_OOB_ADDR, word 0 for a load that the
// Kernel allows to fall outside (it reads element 0), word 1 for a load whose range had been proven.
__device__ __forceinline__ int jx_ix(i64 ix, u32 len, int proven) {
  if (ix >= 0 && ix < (i64)len) return (int)ix;
  atomicAdd((u32*)JX_OOB_ADDR + proven, 1u);
  return 0;
}
#endif

#define JX_INF __int_as_float(0x7f800000)
#define JX_NAN __int_as_float(0x7fc00000)

__device__ __forceinline__ float jx_h2f(jx_half h) {
  float f; asm("cvt.f32.f16 %0, %1;" : "=f"(f) : "h"(h.x)); return f;
}
__device__ __forceinline__ jx_half jx_f2h(float f) {
  jx_half h; asm("cvt.rn.f16.f32 %0, %1;" : "=h"(h.x) : "f"(f)); return h;
}
__device__ __forceinline__ float jx_round_h(float f) { return jx_h2f(jx_f2h(f)); }
__device__ __forceinline__ float jx_h2f_bits(u32 bits16) {
  float f; asm("cvt.f32.f16 %0, %1;" : "=f"(f) : "h"((u16)bits16)); return f;
}

// f32.min / f32.max: NaN-propagating, -0 < +0 (translation.ts:72-74).
__device__ __forceinline__ float jx_fmin(float a, float b) {
  float r; asm("min.NaN.f32 %0, %1, %2;" : "=f"(r) : "f"(a), "f"(b)); return r;
}
__device__ __forceinline__ float jx_fmax(float a, float b) {
  float r; asm("max.NaN.f32 %0, %1, %2;" : "=f"(r) : "f"(a), "f"(b)); return r;
}
__device__ __forceinline__ double jx_dmin(double a, double b) {
  if (a != a || b != b) return __longlong_as_double(0x7ff8000000000000LL);
  if (a == b) return (__double_as_longlong(a) < 0) ? a : b;
  return a < b ? a : b;
}
__device__ __forceinline__ double jx_dmax(double a, double b) {
  if (a != a || b != b) return __longlong_as_double(0x7ff8000000000000LL);
  if (a == b) return (__double_as_longlong(a) < 0) ? b : a;
  return a > b ? a : b;
}
__device__ __forceinline__ int jx_imin(int a, int b) { return a < b ? a : b; }
__device__ __forceinline__ int jx_imax(int a, int b) { return a > b ? a : b; }
__device__ __forceinline__ u32 jx_umin(u32 a, u32 b) { return a < b ? a : b; }
__device__ __forceinline__ u32 jx_umax(u32 a, u32 b) { return a > b ? a : b; }

// i32.div_s / rem_s trap on a zero divisor (and INT_MIN / -1); a trap is not an
// option on a GPU, so those lanes yield 0 (INT_MIN for the overflowing quotient).
__device__ __forceinline__ int jx_idiv(int a, int b) {
  if (b == 0) return 0;
  if (b == -1) return (int)(0u - (u32)a);
  return a / b;
}
__device__ __forceinline__ int jx_imod(int a, int b) { return (b == 0 || b == -1) ? 0 : a % b; }
__device__ __forceinline__ u32 jx_udiv(u32 a, u32 b) { return b ? a / b : 0u; }
__device__ __forceinline__ u32 jx_umod(u32 a, u32 b) { return b ? a % b : 0u; }
__device__ __forceinline__ float jx_fidiv(float a, float b) { return truncf(a / b); }
__device__ __forceinline__ float jx_fmod(float a, float b) { return a - truncf(a / b) * b; }
__device__ __forceinline__ double jx_didiv(double a, double b) { return trunc(a / b); }
__device__ __forceinline__ double jx_dmod(double a, double b) { return a - trunc(a / b) * b; }

// e^x, two versions.  The reference computes k = nearest(x / ln2), r = x - k ln2, a degree-6
// Taylor polynomial in r (Horner, every step rounded) and a scale by 2^k, with +Inf for k > 127
// and 0 for k < -126 (builtins.ts:25-90).
//
// jx_exp_exact repeats those operations one by one with no fused multiply-add, so it returns the
// reference's bits.  It matters where a result is fed to a cancellation -- Adam's 1 - b^t turns a
// single ulp of exp into 1e-4 of the bias correction.
__device__ __forceinline__ float jx_exp_exact(float x) {
  const float kf = rintf(__fmul_rn(x, 1.4426950408889634f));
  const int k = __float2int_rz(kf);
  const float r = __fsub_rn(x, __fmul_rn(kf, 0.6931471805599453f));
  float p = 1.0f / 720.0f;
  p = __fadd_rn(__fmul_rn(p, r), 1.0f / 120.0f);
  p = __fadd_rn(__fmul_rn(p, r), 1.0f / 24.0f);
  p = __fadd_rn(__fmul_rn(p, r), 1.0f / 6.0f);
  p = __fadd_rn(__fmul_rn(p, r), 0.5f);
  p = __fadd_rn(__fmul_rn(p, r), 1.0f);
  p = __fadd_rn(__fmul_rn(p, r), 1.0f);
  float res = __fmul_rn(p, __int_as_float((k + 127) << 23));
  res = (k > 127) ? JX_INF : res;
  return (k < -126) ? 0.0f : res;   // NaN: k = 0 and r = NaN, so res is NaN
}
// jx_exp_fast is the same function as 2^(x log2 e) on the special-function unit: t = rn(x log2 e),
// the rounding residual of that product recovered exactly with two FMAs, ex2.approx(t) and the
// first-order correction 2^e = 1 + e ln2, with the reference's overflow and underflow thresholds
// (t > 127.5, t < -126.5).  Within 5e-7 relative of the exact version in ten issue slots instead
// of about twenty-five, which is what keeps exp-fused streaming kernels memory-bound.
__device__ __forceinline__ float jx_exp_fast(float x) {
  const float t = x * 1.4426950408889634f;
  float e = fmaf(x, 1.4426950408889634f, -t);
  e = fmaf(x, 1.925963033500978e-8f, e);        // log2 e - float(log2 e)
  float p;
  // .ftz: results below 2^-126 become 0, which is what the reference returns there (k < -126)
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(p) : "f"(t));
  float res = fmaf(p, e * 0.6931471805599453f, p);
  res = (t > 127.5f) ? JX_INF : res;
  return (t < -126.5f) ? 0.0f : res;
}
#ifdef JX_EXACT_TRANSCENDENTALS
#define jx_exp jx_exp_exact
#else
#define jx_exp jx_exp_fast
#endif

// ln x: exponent extraction plus the atanh series in t = (m-1)/(m+1) (builtins.ts:99-193).
__device__ __forceinline__ float jx_log(float x) {
  if (x < 0.0f) return JX_NAN;
  int bits = __float_as_int(x);
  int e = ((bits >> 23) & 255) - 127;
  if (e == -127) return -JX_INF;
  if (e == 128) return x;
  float m = __int_as_float((bits & 0x7fffff) | 0x3f800000);
  float t = (m - 1.0f) / (m + 1.0f);
  float t2 = t * t;
  float p = 2.0f / 7.0f;
  p = p * t2 + 2.0f / 5.0f;
  p = p * t2 + 2.0f / 3.0f;
  p = p * t2 + 2.0f;
  return p * t + (float)e * 0.69314718055994531f;
}

// sin / cos: reduce by the nearest multiple of 2pi, then of pi/2 (builtins.ts:203-310).
__device__ __forceinline__ void jx_sincos(float x, int& q, float& sz, float& cz) {
  float y = x - __fmul_rn(rintf(x * 0.15915494309189535f), 6.283185307179586f);  // unfused: the
  // reduction's rounding error is part of the reference's result for large arguments
  float qf = rintf(y * 0.63661977236758138f);
  q = __float2int_rz(qf);
  float z = y - __fmul_rn(qf, 1.5707963267948966f);
  float z2 = z * z;
  float s = -1.0f / 5040.0f;
  s = s * z2 + 1.0f / 120.0f;
  s = s * z2 - 1.0f / 6.0f;
  s = s * z2 + 1.0f;
  sz = s * z;
  float c = 1.0f / 40320.0f;
  c = c * z2 - 1.0f / 720.0f;
  c = c * z2 + 1.0f / 24.0f;
  c = c * z2 - 0.5f;
  cz = c * z2 + 1.0f;
}
__device__ __forceinline__ float jx_sin(float x) {
  int q; float sz, cz; jx_sincos(x, q, sz, cz);
  float mag = (q & 1) ? cz : sz;
  return (q & 2) ? -mag : mag;
}
__device__ __forceinline__ float jx_cos(float x) {
  int q; float sz, cz; jx_sincos(x, q, sz, cz);
  float mag = (q & 1) ? sz : cz;
  return ((q + 1) & 2) ? -mag : mag;
}
// atan: rational P/Q on [0,1], reciprocal fold above 1 (builtins.ts:313-392).
__device__ __forceinline__ float jx_atan(float x) {
  float ax = fabsf(x);
  float z = (ax >= 1.0f) ? 1.0f / ax : ax;
  float z2 = z * z;
  float P = (0.0415796528637f * z2 + 0.661705427875f) * z2 + 0.999998614341f;
  float Q = (0.173698870181f * z2 + 0.994987933645f) * z2 + 1.0f;
  float p = (P / Q) * z;
  float r = (ax >= 1.0f) ? 1.5707963267948966f - p : p;
  return copysignf(r, x);
}
__device__ __forceinline__ float jx_asin(float x) {  // builtins.ts:399-415
  return jx_atan(x / (sqrtf(1.0f - x * x) + 1.0f)) * 2.0f;
}
// erf / erfc: Abramowitz-Stegun 7.1.26 (builtins.ts:422-494, constants of alu.ts:1766-1777).
__device__ __forceinline__ float jx_erfapprox(float x) {
  float t = 1.0f / (1.0f + 0.3275911f * x);
  float p = 1.061405429f;
  p = p * t - 1.453152027f;
  p = p * t + 1.421413741f;
  p = p * t - 0.284496736f;
  p = p * t + 0.254829592f;
  p = p * t;
  return p * jx_exp((-x) * x);
}
__device__ __forceinline__ float jx_erf(float x) { return copysignf(1.0f - jx_erfapprox(fabsf(x)), x); }
__device__ __forceinline__ float jx_erfc(float x) {
  float e = jx_erfapprox(fabsf(x));
  return (x < 0.0f) ? 2.0f - e : e;
}

// Threefry-2x32, 20 rounds (alu.ts:1699-1745, builtins.ts:502-584). mode 0: x0^x1, 1: x0, 2: x1.
__device__ __forceinline__ u32 jx_rotl(u32 x, int r) { return __funnelshift_l(x, x, r); }
__device__ __forceinline__ u32 jx_threefry(u32 k0, u32 k1, u32 c0, u32 c1, int mode) {
  u32 ks0 = k0, ks1 = k1, ks2 = k0 ^ k1 ^ 0x1bd11bdau;
  u32 x0 = c0 + ks0, x1 = c1 + ks1;
#define JX_R4(a, b, c, d) \
  x0 += x1; x1 = jx_rotl(x1, a) ^ x0; x0 += x1; x1 = jx_rotl(x1, b) ^ x0; \
  x0 += x1; x1 = jx_rotl(x1, c) ^ x0; x0 += x1; x1 = jx_rotl(x1, d) ^ x0;
  JX_R4(13, 15, 26, 6)  x0 += ks1; x1 += ks2 + 1u;
  JX_R4(17, 29, 16, 24) x0 += ks2; x1 += ks0 + 2u;
  JX_R4(13, 15, 26, 6)  x0 += ks0; x1 += ks1 + 3u;
  JX_R4(17, 29, 16, 24) x0 += ks1; x1 += ks2 + 4u;
  JX_R4(13, 15, 26, 6)  x0 += ks2; x1 += ks0 + 5u;
#undef JX_R4
  return mode == 0 ? (x0 ^ x1) : mode == 1 ? x0 : x1;
}

// Vector carriers for 128-bit (and narrower) global accesses.
template <int BYTES> struct jx_vec;
template <> struct __align__(2)  jx_vec<2>  { u16 v; };
template <> struct __align__(4)  jx_vec<4>  { u32 v; };
template <> struct __align__(8)  jx_vec<8>  { u32 v[2]; };
template <> struct __align__(16) jx_vec<16> { u32 v[4]; };
template <> struct __align__(16) jx_vec<32> { u32 v[8]; };
template <> struct __align__(16) jx_vec<64> { u32 v[16]; };

template <class T, int N> struct jx_pack {
  union { jx_vec<sizeof(T) * N> raw; T e[N]; };
  __device__ __forceinline__ jx_pack() {}
};
template <class T, int N>
__device__ __forceinline__ void jx_load(jx_pack<T, N>& p, const T* src) {
#if defined(JX_LD_HINT) && JX_LD_HINT > 0
  // Streaming reads: 128-bit non-coherent loads that do not allocate in L1 and ask L2 to fetch
  // 256-byte lines, which keeps DRAM bursts long when a warp only touches 512 bytes of a row.
  if constexpr (sizeof(T) * N == 16) {
    u32 w0, w1, w2, w3;
    asm volatile("ld.global.nc.L1::no_allocate.L2::256B.v4.u32 {%0, %1, %2, %3}, [%4];"
                 : "=r"(w0), "=r"(w1), "=r"(w2), "=r"(w3) : "l"(src));
    u32* w = reinterpret_cast<u32*>(&p.raw);
    w[0] = w0; w[1] = w1; w[2] = w2; w[3] = w3;
    return;
  }
#endif
  p.raw = *reinterpret_cast<const jx_vec<sizeof(T) * N>*>(src);
}
template <class T, int N>
__device__ __forceinline__ void jx_store(T* dst, const jx_pack<T, N>& p) {
  *reinterpret_cast<jx_vec<sizeof(T) * N>*>(dst) = p.raw;
}

template <class T> __device__ __forceinline__ T jx_shfl_down(T v, int o, int w) {
  return __shfl_down_sync(0xffffffffu, v, o, w);
}
)PRELUDE";

}  // namespace jaxcuda
