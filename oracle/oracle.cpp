// CPU oracle for the jax-js Kernel / Routine hot path.  TEST INFRASTRUCTURE ONLY:
// nothing in the product (the package, libjaxcuda.so) links, imports or runs this
// file; only tests/, the smoke check and the bench's CPU-baseline legs do.
//
// It restates, for one lowered Kernel image (include/jaxcuda_ir.h), the arithmetic of
// the reference's two CPU backends:
//
//   mode WASM  the Wasm backend: f32 arithmetic, non-fused, op rules of
//              src/backend/wasm/translation.ts:36-236, software transcendentals of
//              src/backend/wasm/builtins.ts:25-494, sequential-k accumulation per
//              output (src/backend/wasm/codegen.ts:560-694), out-of-range loads read
//              element 0 (translation.ts:221-234).
//   mode CPU   the `cpu` debug backend (src/backend/cpu.ts:83-134): every float is
//              a JS double evaluated by AluExp.evaluate (src/alu.ts:1059-1213) and
//              rounded once, on the store to the typed output array.  This is the
//              only reference semantics that exists for float16
//              (translation.ts:558-586 rejects it).
//
// Routines follow src/routine.ts: Sort / Argsort :185-214, Scatter :226-296, TriangularSolve
// :298-338, Cholesky :340-366, LU :368-432, JacobiEigh :434-541, Fft :543-624 (double
// intermediates, one rounding per store, as JavaScript numbers over typed arrays behave).
//
// Parity pins: the known-answer vectors of the reference's own tests
// (src/backend/backend.test.ts, src/alu.test.ts, src/backend/wasm/builtins.test.ts,
// test/numpy.test.ts sort/argsort/matmul, test/nn.test.ts, test/argreduce.test.ts,
// test/lax-linalg.test.ts, test/numpy-fft.test.ts) are replayed against this file by
// tests/test_oracle_golden.py and the CPU halves of tests/test_scatter.py and
// tests/test_linalg.py.  The reference itself cannot be executed in the build
// container (no JavaScript or WebAssembly runtime), so the pins are those vectors.
#include <algorithm>
#include <cmath>
#include <cstdint>
#include <cstdio>
#include <cstring>
#include <limits>
#include <string>
#include <vector>

#include "../include/jaxcuda_ir.h"

namespace {

thread_local std::string g_error;

constexpr int B = 128;  // outputs interpreted together (lanes)

enum Mode { MODE_AUTO = 0, MODE_WASM = 1, MODE_CPU = 2 };
enum Rep { REP_F, REP_D, REP_I, REP_U };  // float, double, int32 (and Bool), uint32

struct Node {
  uint32_t op, dtype, nsrc, src[4];
  uint64_t arg0;
  uint32_t arg1;
  Rep rep;
  bool dep_r;  // value changes with ridx
};

struct Program {
  uint32_t nargs;
  uint64_t size;
  bool has_red;
  uint32_t red_dtype, red_op, red_size;
  std::vector<Node> exp, epi;
};

union alignas(64) Lanes {
  float f[B];
  double d[B];
  int32_t i[B];
  uint32_t u[B];
};

bool is_float_dtype(uint32_t dt) { return dt == JAXCUDA_F32 || dt == JAXCUDA_F16 || dt == JAXCUDA_F64; }

Rep rep_of(uint32_t dtype, Mode mode) {
  switch (dtype) {
    case JAXCUDA_F32: return mode == MODE_CPU ? REP_D : REP_F;
    case JAXCUDA_F16:
    case JAXCUDA_F64: return REP_D;
    case JAXCUDA_U32: return REP_U;
    default: return REP_I;
  }
}

bool parse(const uint8_t* ir, size_t len, Program& p) {
  if (len < JAXCUDA_IR_HEADER_WORDS * 4 || len % 4) { g_error = "truncated kernel image"; return false; }
  std::vector<uint32_t> w(len / 4);
  memcpy(w.data(), ir, len);
  if (w[0] != JAXCUDA_IR_MAGIC) { g_error = "bad magic"; return false; }
  p.nargs = w[1];
  p.size = (uint64_t)w[2] | ((uint64_t)w[3] << 32);
  p.has_red = w[4] != 0;
  p.red_dtype = w[5]; p.red_op = w[6]; p.red_size = w[7];
  size_t n_exp = w[8], n_epi = w[9];
  if (w.size() != JAXCUDA_IR_HEADER_WORDS + (n_exp + n_epi) * JAXCUDA_IR_NODE_WORDS) {
    g_error = "kernel image length does not match node counts"; return false;
  }
  auto read_nodes = [&](size_t base, size_t n, std::vector<Node>& out) {
    out.resize(n);
    for (size_t k = 0; k < n; k++) {
      const uint32_t* q = &w[base + k * JAXCUDA_IR_NODE_WORDS];
      Node& nd = out[k];
      nd.op = q[0]; nd.dtype = q[1]; nd.nsrc = q[2];
      for (int s = 0; s < 4; s++) nd.src[s] = q[3 + s];
      nd.arg0 = (uint64_t)q[7] | ((uint64_t)q[8] << 32);
      nd.arg1 = q[9];
      if (nd.op >= JAXCUDA_OP_COUNT || nd.dtype > JAXCUDA_F64 || nd.nsrc > 4) return false;
      for (uint32_t s = 0; s < nd.nsrc; s++) if (nd.src[s] >= k) return false;
    }
    return true;
  };
  if (!read_nodes(JAXCUDA_IR_HEADER_WORDS, n_exp, p.exp) ||
      !read_nodes(JAXCUDA_IR_HEADER_WORDS + n_exp * JAXCUDA_IR_NODE_WORDS, n_epi, p.epi)) {
    g_error = "malformed node"; return false;
  }
  if (n_exp == 0 || (p.has_red && n_epi == 0)) { g_error = "empty expression"; return false; }
  return true;
}

// ---- float16 <-> double (IEEE binary16, round to nearest even) ---------------------
double half_to_double(uint16_t h) {
  uint32_t sign = h >> 15, e = (h >> 10) & 31, m = h & 1023;
  double v;
  if (e == 0) v = std::ldexp((double)m, -24);
  else if (e == 31) v = m ? std::numeric_limits<double>::quiet_NaN() : std::numeric_limits<double>::infinity();
  else v = std::ldexp((double)(m | 1024), (int)e - 25);
  return sign ? -v : v;
}

uint16_t double_to_half(double x) {
  uint16_t sign = std::signbit(x) ? 0x8000 : 0;
  if (std::isnan(x)) return sign | 0x7e00;
  double a = std::fabs(x);
  if (a >= 65520.0) return sign | 0x7c00;  // rounds to infinity
  if (a < std::ldexp(1.0, -25)) return sign;  // below half of the least subnormal (ties to even = 0)
  int e;
  std::frexp(a, &e);  // a = f * 2^e, f in [0.5, 1)
  int shift = (e - 1 < -14) ? -24 : (e - 1) - 10;  // exponent of one ulp
  double q = std::nearbyint(std::ldexp(a, -shift));  // default rounding mode: ties to even
  if (e - 1 < -14) return sign | (uint16_t)q;  // subnormal (q may reach 1024 = least normal)
  uint32_t m = (uint32_t)q;  // in [1024, 2048]
  int be = e - 1 + 15;
  if (m == 2048) { m = 1024; be++; }
  if (be >= 31) return sign | 0x7c00;
  return sign | (uint16_t)(be << 10) | (uint16_t)(m & 1023);
}

// ---- Wasm software transcendentals (src/backend/wasm/builtins.ts) -------------------
// Every operation is a separate f32 operation, as Wasm executes it (this file is built
// with -ffp-contract=off).  `nearest` is round-half-to-even (f32.nearest).
inline float poly(float x, const float* a, int n) {  // builtins.ts:6-17 (skips +0 terms)
  float acc = a[n - 1];
  for (int k = n - 2; k >= 0; k--) { acc = acc * x; if (a[k] != 0.0f) acc = acc + a[k]; }
  return acc;
}
inline int32_t trunc_sat_s(float x) {  // i32.trunc_sat_f32_s
  if (x != x) return 0;
  if (x >= 2147483648.0f) return INT32_MAX;
  if (x <= -2147483648.0f) return INT32_MIN;
  return (int32_t)x;
}
inline int32_t trunc_sat_s(double x) {
  if (x != x) return 0;
  if (x >= 2147483647.0) return INT32_MAX;
  if (x <= -2147483648.0) return INT32_MIN;
  return (int32_t)x;
}
inline uint32_t trunc_sat_u(float x) {
  if (!(x > 0.0f)) return 0;
  if (x >= 4294967296.0f) return UINT32_MAX;
  return (uint32_t)x;
}
inline uint32_t trunc_sat_u(double x) {
  if (!(x > 0.0)) return 0;
  if (x >= 4294967295.0) return UINT32_MAX;
  return (uint32_t)x;
}
inline float bits_f(uint32_t b) { float f; memcpy(&f, &b, 4); return f; }
inline uint32_t f_bits(float f) { uint32_t b; memcpy(&b, &f, 4); return b; }

float wasm_exp(float x) {  // builtins.ts:25-90
  const float inv_ln2 = (float)(1.0 / 0.6931471805599453), ln2 = (float)0.6931471805599453;
  float kf = std::nearbyintf(x * inv_ln2);
  int32_t k = trunc_sat_s(kf);
  if (k > 127) return std::numeric_limits<float>::infinity();
  if (k < -126) return 0.0f;
  float r = x - kf * ln2;
  static const float c[7] = {1.0f, 1.0f, (float)(1.0 / 2), (float)(1.0 / 6), (float)(1.0 / 24),
                             (float)(1.0 / 120), (float)(1.0 / 720)};
  float p = poly(r, c, 7);
  float scale = bits_f((uint32_t)(k + 127) << 23);
  return p * scale;
}

float wasm_log(float x) {  // builtins.ts:99-193
  if (x < 0.0f) return std::numeric_limits<float>::quiet_NaN();
  uint32_t bits = f_bits(x);
  int32_t e = (int32_t)((bits >> 23) & 255) - 127;
  if (e == -127) return -std::numeric_limits<float>::infinity();  // zero and subnormals
  if (e == 128) return x;  // Infinity, NaN
  float m = bits_f((bits & 0x7fffff) | 0x3f800000);
  float t = (m - 1.0f) / (m + 1.0f);
  float t2 = t * t;
  static const float c[4] = {2.0f, (float)(2.0 / 3), (float)(2.0 / 5), (float)(2.0 / 7)};
  float lnm = poly(t2, c, 4) * t;
  float el2 = (float)e * (float)0.6931471805599453;
  return lnm + el2;
}

void wasm_sincos(float x, int32_t& q, float& sz, float& cz) {  // builtins.ts:203-256
  const double PI = 3.141592653589793;
  float y = x - std::nearbyintf(x * (float)(1.0 / (2 * PI))) * (float)(2 * PI);
  float qf = std::nearbyintf(y * (float)(2 / PI));
  q = trunc_sat_s(qf);
  float z = y - qf * (float)(PI / 2);
  float z2 = z * z;
  static const float s[4] = {1.0f, (float)(-1.0 / 6), (float)(1.0 / 120), (float)(-1.0 / 5040)};
  static const float c[5] = {1.0f, (float)(-1.0 / 2), (float)(1.0 / 24), (float)(-1.0 / 720), (float)(1.0 / 40320)};
  sz = poly(z2, s, 4) * z;
  cz = poly(z2, c, 5);
}
float wasm_sin(float x) {  // builtins.ts:263-281
  int32_t q; float sz, cz;
  wasm_sincos(x, q, sz, cz);
  float mag = (q & 1) ? cz : sz;
  return (q & 2) ? -mag : mag;
}
float wasm_cos(float x) {  // builtins.ts:288-309
  int32_t q; float sz, cz;
  wasm_sincos(x, q, sz, cz);
  float mag = (q & 1) ? sz : cz;
  return ((q + 1) & 2) ? -mag : mag;
}
float wasm_atan(float x) {  // builtins.ts:313-392
  float ax = std::fabs(x);
  float z = (ax >= 1.0f) ? 1.0f / ax : ax;
  float z2 = z * z;
  static const float P[3] = {(float)0.999998614341, (float)0.661705427875, (float)0.0415796528637};
  static const float Q[3] = {1.0f, (float)0.994987933645, (float)0.173698870181};
  float p = (poly(z2, P, 3) / poly(z2, Q, 3)) * z;
  float r = (ax >= 1.0f) ? (float)(3.141592653589793 / 2) - p : p;
  return std::copysign(r, x);
}
float wasm_asin(float x) {  // builtins.ts:399-415
  return wasm_atan(x / (std::sqrt(1.0f - x * x) + 1.0f)) * 2.0f;
}
float wasm_erfapprox(float x) {  // builtins.ts:422-455, constants of src/alu.ts:1766-1777
  float t = 1.0f / (1.0f + (float)0.3275911 * x);
  static const float a[6] = {0.0f, (float)0.254829592, (float)-0.284496736, (float)1.421413741,
                             (float)-1.453152027, (float)1.061405429};
  return poly(t, a, 6) * wasm_exp((-x) * x);
}
float wasm_erf(float x) { return std::copysign(1.0f - wasm_erfapprox(std::fabs(x)), x); }  // :458-471
float wasm_erfc(float x) {  // builtins.ts:474-494
  float e = wasm_erfapprox(std::fabs(x));
  return (x < 0.0f) ? 2.0f - e : e;
}

// `cpu` backend transcendentals: JS Math.* on doubles; erf/erfc of src/alu.ts:1766-1793.
double js_erfapprox(double x) {
  const double p = 0.3275911, a1 = 0.254829592, a2 = -0.284496736, a3 = 1.421413741,
               a4 = -1.453152027, a5 = 1.061405429;
  double t = 1 / (1 + p * x);
  return ((((a5 * t + a4) * t + a3) * t + a2) * t + a1) * t * std::exp(-x * x);
}
double js_erf(double x) { return x >= 0 ? 1 - js_erfapprox(x) : js_erfapprox(-x) - 1; }
double js_erfc(double x) { return x >= 0 ? js_erfapprox(x) : 2 - js_erfapprox(-x); }

// Threefry-2x32, 20 rounds (src/alu.ts:1699-1745 == builtins.ts:502-584).
inline uint32_t rotl(uint32_t x, int r) { return (x << r) | (x >> (32 - r)); }
void threefry2x32(uint32_t k0, uint32_t k1, uint32_t c0, uint32_t c1, uint32_t& o0, uint32_t& o1) {
  static const int R[2][4] = {{13, 15, 26, 6}, {17, 29, 16, 24}};
  uint32_t ks[3] = {k0, k1, k0 ^ k1 ^ 0x1bd11bdau};
  uint32_t x0 = c0 + ks[0], x1 = c1 + ks[1];
  for (int g = 0; g < 5; g++) {
    for (int j = 0; j < 4; j++) { x0 += x1; x1 = rotl(x1, R[g & 1][j]) ^ x0; }
    x0 += ks[(g + 1) % 3];
    x1 += ks[(g + 2) % 3] + (uint32_t)(g + 1);
  }
  o0 = x0; o1 = x1;
}

// ---- min/max with Wasm f32.min/max rules: NaN-propagating, -0 < +0 -----------------
template <class T> inline T fmin_wasm(T a, T b) {
  if (a != a || b != b) return std::numeric_limits<T>::quiet_NaN();
  if (a == b) return std::signbit(a) ? a : b;
  return a < b ? a : b;
}
template <class T> inline T fmax_wasm(T a, T b) {
  if (a != a || b != b) return std::numeric_limits<T>::quiet_NaN();
  if (a == b) return std::signbit(a) ? b : a;
  return a > b ? a : b;
}

struct Ctx {
  Mode mode;
  const void* const* args;
  int fma;
};

#define LOOP for (int l = 0; l < n; l++)

// Evaluate one node for n lanes.  g0 = first output index of the block, r = ridx.
void eval_node(const Ctx& cx, const std::vector<Node>& nodes, size_t k, std::vector<Lanes>& v,
               uint64_t g0, uint32_t r, int n, const Lanes* acc) {
  const Node& nd = nodes[k];
  Lanes& o = v[k];
  const Lanes* a = nd.nsrc > 0 ? &v[nd.src[0]] : nullptr;
  const Lanes* b = nd.nsrc > 1 ? &v[nd.src[1]] : nullptr;
  const Lanes* c = nd.nsrc > 2 ? &v[nd.src[2]] : nullptr;
  const Rep rep = nd.rep;
  const bool is_bool = nd.dtype == JAXCUDA_BOOL;
  const bool wasm = cx.mode == MODE_WASM;
  switch (nd.op) {
    case JAXCUDA_OP_ADD:
      if (is_bool) LOOP o.i[l] = a->i[l] | b->i[l];
      else if (rep == REP_F) LOOP o.f[l] = a->f[l] + b->f[l];
      else if (rep == REP_D) LOOP o.d[l] = a->d[l] + b->d[l];
      else LOOP o.u[l] = a->u[l] + b->u[l];
      break;
    case JAXCUDA_OP_SUB:
      if (rep == REP_F) LOOP o.f[l] = a->f[l] - b->f[l];
      else if (rep == REP_D) LOOP o.d[l] = a->d[l] - b->d[l];
      else LOOP o.u[l] = a->u[l] - b->u[l];
      break;
    case JAXCUDA_OP_MUL:
      if (is_bool) LOOP o.i[l] = a->i[l] & b->i[l];
      else if (rep == REP_F) LOOP o.f[l] = a->f[l] * b->f[l];
      else if (rep == REP_D) LOOP o.d[l] = a->d[l] * b->d[l];
      else LOOP o.u[l] = a->u[l] * b->u[l];
      break;
    case JAXCUDA_OP_IDIV:  // translation.ts:46-52; integer division by zero traps in Wasm: yield 0
      if (rep == REP_F) LOOP o.f[l] = std::trunc(a->f[l] / b->f[l]);
      else if (rep == REP_D) LOOP o.d[l] = std::trunc(a->d[l] / b->d[l]);
      else if (rep == REP_U) LOOP o.u[l] = b->u[l] ? a->u[l] / b->u[l] : 0;
      else LOOP {
        int32_t x = a->i[l], y = b->i[l];
        o.i[l] = y == 0 ? 0 : (x == INT32_MIN && y == -1) ? INT32_MIN : x / y;
      }
      break;
    case JAXCUDA_OP_MOD:  // translation.ts:53-70; JS `%` (fmod) in the cpu backend
      if (rep == REP_F) LOOP { float x = a->f[l], y = b->f[l]; o.f[l] = x - std::trunc(x / y) * y; }
      else if (rep == REP_D) LOOP {
        double x = a->d[l], y = b->d[l];
        o.d[l] = wasm ? x - std::trunc(x / y) * y : std::fmod(x, y);
      }
      else if (rep == REP_U) LOOP o.u[l] = b->u[l] ? a->u[l] % b->u[l] : 0;
      else LOOP { int32_t x = a->i[l], y = b->i[l]; o.i[l] = (y == 0 || y == -1) ? 0 : x % y; }
      break;
    case JAXCUDA_OP_MIN:
      if (is_bool) LOOP o.i[l] = a->i[l] & b->i[l];
      else if (rep == REP_F) LOOP o.f[l] = fmin_wasm(a->f[l], b->f[l]);
      else if (rep == REP_D) LOOP o.d[l] = fmin_wasm(a->d[l], b->d[l]);
      else if (rep == REP_U) LOOP o.u[l] = std::min(a->u[l], b->u[l]);
      else LOOP o.i[l] = std::min(a->i[l], b->i[l]);
      break;
    case JAXCUDA_OP_MAX:
      if (is_bool) LOOP o.i[l] = a->i[l] | b->i[l];
      else if (rep == REP_F) LOOP o.f[l] = fmax_wasm(a->f[l], b->f[l]);
      else if (rep == REP_D) LOOP o.d[l] = fmax_wasm(a->d[l], b->d[l]);
      else if (rep == REP_U) LOOP o.u[l] = std::max(a->u[l], b->u[l]);
      else LOOP o.i[l] = std::max(a->i[l], b->i[l]);
      break;
#define UNARY_F(WASMFN, JSFN)                                                         \
      if (rep == REP_F) LOOP o.f[l] = WASMFN(a->f[l]);                                \
      else if (wasm) LOOP o.d[l] = (double)WASMFN((float)a->d[l]); /* f64 demoted, translation.ts:115-122 */ \
      else LOOP o.d[l] = JSFN(a->d[l]);                                               \
      break;
    case JAXCUDA_OP_SIN: UNARY_F(wasm_sin, std::sin)
    case JAXCUDA_OP_COS: UNARY_F(wasm_cos, std::cos)
    case JAXCUDA_OP_ASIN: UNARY_F(wasm_asin, std::asin)
    case JAXCUDA_OP_ATAN: UNARY_F(wasm_atan, std::atan)
    case JAXCUDA_OP_EXP: UNARY_F(wasm_exp, std::exp)
    case JAXCUDA_OP_LOG: UNARY_F(wasm_log, std::log)
    case JAXCUDA_OP_ERF: UNARY_F(wasm_erf, js_erf)
    case JAXCUDA_OP_ERFC: UNARY_F(wasm_erfc, js_erfc)
#undef UNARY_F
    case JAXCUDA_OP_SQRT:
      if (rep == REP_F) LOOP o.f[l] = std::sqrt(a->f[l]); else LOOP o.d[l] = std::sqrt(a->d[l]);
      break;
    case JAXCUDA_OP_FLOOR:
      if (rep == REP_F) LOOP o.f[l] = std::floor(a->f[l]); else LOOP o.d[l] = std::floor(a->d[l]);
      break;
    case JAXCUDA_OP_CEIL:
      if (rep == REP_F) LOOP o.f[l] = std::ceil(a->f[l]); else LOOP o.d[l] = std::ceil(a->d[l]);
      break;
    case JAXCUDA_OP_RECIPROCAL:
      if (rep == REP_F) LOOP o.f[l] = 1.0f / a->f[l]; else LOOP o.d[l] = 1.0 / a->d[l];
      break;
    case JAXCUDA_OP_CAST: {  // translation.ts:139-173; alu.ts:1130-1139
      const Node& s = nodes[nd.src[0]];
      const Rep sr = s.rep;
      if (nd.dtype == JAXCUDA_BOOL) {
        if (sr == REP_F) LOOP o.i[l] = a->f[l] != 0.0f;
        else if (sr == REP_D) LOOP o.i[l] = a->d[l] != 0.0;
        else LOOP o.i[l] = a->u[l] != 0;
      } else if (nd.dtype == JAXCUDA_I32) {
        if (sr == REP_F) LOOP o.i[l] = trunc_sat_s(a->f[l]);
        else if (sr == REP_D) LOOP o.i[l] = trunc_sat_s(a->d[l]);
        else LOOP o.i[l] = a->i[l];
      } else if (nd.dtype == JAXCUDA_U32) {
        if (sr == REP_F) LOOP o.u[l] = trunc_sat_u(a->f[l]);
        else if (sr == REP_D) LOOP o.u[l] = trunc_sat_u(a->d[l]);
        else LOOP o.u[l] = a->u[l];
      } else if (rep == REP_F) {
        if (sr == REP_F) LOOP o.f[l] = a->f[l];
        else if (sr == REP_D) LOOP o.f[l] = (float)a->d[l];
        else if (sr == REP_U) LOOP o.f[l] = (float)a->u[l];
        else LOOP o.f[l] = (float)a->i[l];
      } else {  // to a double-held float (f64, f16, or any float in cpu mode): no rounding, alu.ts:1136
        if (sr == REP_F) LOOP o.d[l] = (double)a->f[l];
        else if (sr == REP_D) LOOP o.d[l] = a->d[l];
        else if (sr == REP_U) LOOP o.d[l] = (double)a->u[l];
        else LOOP o.d[l] = (double)a->i[l];
      }
      break;
    }
    case JAXCUDA_OP_BITCAST: {  // among f32/i32/u32 (translation.ts:175-189)
      const Rep sr = nodes[nd.src[0]].rep;
      LOOP {
        uint32_t bits = sr == REP_F ? f_bits(a->f[l]) : sr == REP_D ? f_bits((float)a->d[l]) : a->u[l];
        if (rep == REP_F) o.f[l] = bits_f(bits);
        else if (rep == REP_D) o.d[l] = (double)bits_f(bits);
        else o.u[l] = bits;
      }
      break;
    }
    case JAXCUDA_OP_BITCOMBINE:
      if (nd.arg0 == 0) LOOP o.u[l] = a->u[l] & b->u[l];
      else if (nd.arg0 == 1) LOOP o.u[l] = a->u[l] | b->u[l];
      else LOOP o.u[l] = a->u[l] ^ b->u[l];
      break;
    case JAXCUDA_OP_BITINVERT:
      if (is_bool) LOOP o.i[l] = !a->i[l]; else LOOP o.u[l] = ~a->u[l];
      break;
    case JAXCUDA_OP_BITSHIFT:  // count masked to 5 bits; shr is logical (translation.ts:101-103)
      if (nd.arg0 == 0) LOOP o.u[l] = a->u[l] << (b->u[l] & 31);
      else LOOP o.u[l] = a->u[l] >> (b->u[l] & 31);
      break;
    case JAXCUDA_OP_CMPLT: {
      const Node& s = nodes[nd.src[0]];
      if (s.rep == REP_F) LOOP o.i[l] = a->f[l] < b->f[l];
      else if (s.rep == REP_D) LOOP o.i[l] = a->d[l] < b->d[l];
      else if (s.rep == REP_U) LOOP o.i[l] = a->u[l] < b->u[l];
      else LOOP o.i[l] = a->i[l] < b->i[l];
      break;
    }
    case JAXCUDA_OP_CMPNE: {
      const Node& s = nodes[nd.src[0]];
      if (s.rep == REP_F) LOOP o.i[l] = a->f[l] != b->f[l];
      else if (s.rep == REP_D) LOOP o.i[l] = a->d[l] != b->d[l];
      else LOOP o.i[l] = a->u[l] != b->u[l];
      break;
    }
    case JAXCUDA_OP_WHERE:
      if (rep == REP_D) LOOP o.d[l] = a->i[l] ? b->d[l] : c->d[l];
      else LOOP o.u[l] = a->i[l] ? b->u[l] : c->u[l];
      break;
    case JAXCUDA_OP_THREEFRY2X32: {
      const Lanes* d = &v[nd.src[3]];
      LOOP {
        uint32_t x0, x1;
        threefry2x32(a->u[l], b->u[l], c->u[l], d->u[l], x0, x1);
        o.u[l] = nd.arg0 == 0 ? (x0 ^ x1) : nd.arg0 == 1 ? x0 : x1;
      }
      break;
    }
    case JAXCUDA_OP_CONST:
      if (rep == REP_F) { double dv; memcpy(&dv, &nd.arg0, 8); LOOP o.f[l] = (float)dv; }
      else if (rep == REP_D) { double dv; memcpy(&dv, &nd.arg0, 8); LOOP o.d[l] = dv; }
      else LOOP o.u[l] = (uint32_t)nd.arg0;
      break;
    case JAXCUDA_OP_SPECIAL:
      if (nd.arg0 == 0) LOOP o.i[l] = (int32_t)(g0 + l); else LOOP o.i[l] = (int32_t)r;
      break;
    case JAXCUDA_OP_VARIABLE:
      o = *acc;
      break;
    case JAXCUDA_OP_GLOBALINDEX: {  // out-of-range index reads element 0 (translation.ts:221-228)
      const uint32_t len = nd.arg1;
      const void* base = cx.args[nd.arg0];
      if (nd.dtype == JAXCUDA_F16) {
        const uint16_t* p = (const uint16_t*)base;
        LOOP { uint32_t ix = a->u[l] < len ? a->u[l] : 0; o.d[l] = len ? half_to_double(p[ix]) : 0.0; }
      } else if (nd.dtype == JAXCUDA_F64) {
        const double* p = (const double*)base;
        LOOP { uint32_t ix = a->u[l] < len ? a->u[l] : 0; o.d[l] = len ? p[ix] : 0.0; }
      } else if (nd.dtype == JAXCUDA_F32) {
        const float* p = (const float*)base;
        if (rep == REP_F) LOOP { uint32_t ix = a->u[l] < len ? a->u[l] : 0; o.f[l] = len ? p[ix] : 0.0f; }
        else LOOP { uint32_t ix = a->u[l] < len ? a->u[l] : 0; o.d[l] = len ? (double)p[ix] : 0.0; }
      } else {
        const uint32_t* p = (const uint32_t*)base;
        LOOP { uint32_t ix = a->u[l] < len ? a->u[l] : 0; o.u[l] = len ? p[ix] : 0; }
      }
      break;
    }
  }
}

void mark(std::vector<Node>& nodes, Mode mode) {
  for (auto& nd : nodes) {
    nd.rep = rep_of(nd.dtype, mode);
    nd.dep_r = nd.op == JAXCUDA_OP_SPECIAL && nd.arg0 == 1;
    for (uint32_t s = 0; s < nd.nsrc; s++) nd.dep_r = nd.dep_r || nodes[nd.src[s]].dep_r;
  }
}

void store(uint32_t dtype, Rep rep, const Lanes& v, void* out, uint64_t at, int n) {
  switch (dtype) {
    case JAXCUDA_F32: {
      float* p = (float*)out + at;
      if (rep == REP_F) LOOP p[l] = v.f[l]; else LOOP p[l] = (float)v.d[l];
      break;
    }
    case JAXCUDA_F16: { uint16_t* p = (uint16_t*)out + at; LOOP p[l] = double_to_half(v.d[l]); break; }
    case JAXCUDA_F64: { double* p = (double*)out + at; LOOP p[l] = v.d[l]; break; }
    default: { uint32_t* p = (uint32_t*)out + at; LOOP p[l] = v.u[l]; break; }
  }
}

void reduce_step(uint32_t op, uint32_t dtype, Rep rep, Lanes& acc, const Lanes& x, int n) {
  const bool is_bool = dtype == JAXCUDA_BOOL;
  switch (op) {  // src/alu.ts:1606-1660
    case JAXCUDA_OP_ADD:
      if (is_bool) LOOP acc.i[l] |= x.i[l];
      else if (rep == REP_F) LOOP acc.f[l] = acc.f[l] + x.f[l];
      else if (rep == REP_D) LOOP acc.d[l] = acc.d[l] + x.d[l];
      else LOOP acc.u[l] += x.u[l];
      break;
    case JAXCUDA_OP_MUL:
      if (is_bool) LOOP acc.i[l] &= x.i[l];
      else if (rep == REP_F) LOOP acc.f[l] = acc.f[l] * x.f[l];
      else if (rep == REP_D) LOOP acc.d[l] = acc.d[l] * x.d[l];
      else LOOP acc.u[l] *= x.u[l];
      break;
    case JAXCUDA_OP_MIN:
      if (is_bool) LOOP acc.i[l] &= x.i[l];
      else if (rep == REP_F) LOOP acc.f[l] = fmin_wasm(acc.f[l], x.f[l]);
      else if (rep == REP_D) LOOP acc.d[l] = fmin_wasm(acc.d[l], x.d[l]);
      else if (rep == REP_U) LOOP acc.u[l] = std::min(acc.u[l], x.u[l]);
      else LOOP acc.i[l] = std::min(acc.i[l], x.i[l]);
      break;
    case JAXCUDA_OP_MAX:
      if (is_bool) LOOP acc.i[l] |= x.i[l];
      else if (rep == REP_F) LOOP acc.f[l] = fmax_wasm(acc.f[l], x.f[l]);
      else if (rep == REP_D) LOOP acc.d[l] = fmax_wasm(acc.d[l], x.d[l]);
      else if (rep == REP_U) LOOP acc.u[l] = std::max(acc.u[l], x.u[l]);
      else LOOP acc.i[l] = std::max(acc.i[l], x.i[l]);
      break;
  }
}

void identity(uint32_t op, uint32_t dtype, Rep rep, Lanes& acc) {  // src/alu.ts:1584-1604
  const int n = B;
  if (dtype == JAXCUDA_BOOL) { int32_t v = (op == JAXCUDA_OP_ADD || op == JAXCUDA_OP_MAX) ? 0 : 1; LOOP acc.i[l] = v; return; }
  if (rep == REP_I) {
    int32_t v = op == JAXCUDA_OP_ADD ? 0 : op == JAXCUDA_OP_MUL ? 1 : op == JAXCUDA_OP_MIN ? INT32_MAX : INT32_MIN;
    LOOP acc.i[l] = v;
  } else if (rep == REP_U) {
    uint32_t v = op == JAXCUDA_OP_ADD ? 0 : op == JAXCUDA_OP_MUL ? 1 : op == JAXCUDA_OP_MIN ? UINT32_MAX : 0;
    LOOP acc.u[l] = v;
  } else {
    double v = op == JAXCUDA_OP_ADD ? 0 : op == JAXCUDA_OP_MUL ? 1
               : op == JAXCUDA_OP_MIN ? std::numeric_limits<double>::infinity()
                                      : -std::numeric_limits<double>::infinity();
    if (rep == REP_F) LOOP acc.f[l] = (float)v; else LOOP acc.d[l] = v;
  }
}

#undef LOOP

}  // namespace

extern "C" {

const char* oracle_last_error() { return g_error.c_str(); }

// Evaluate out[g] for g in [begin, end) of the kernel image `ir` (the range form the
// Wasm module exports: kernel(...ptrs, begin, end), src/backend/wasm.ts:258-262).
// `out` is the full output buffer; only [begin, end) is written.
// mode: 0 auto (CPU when any node is float16, else WASM), 1 WASM, 2 CPU.
// fma: accumulate a*b+acc of an f32 Mul root under an Add reduction with one rounding,
//      as the optional f32x4.relaxed_madd path does (codegen.ts:318-322).
// threads: OpenMP threads over blocks of outputs (the browser worker pool splits the
//      output range the same way, parallel.ts:205-243); 1 mirrors Node.
int oracle_kernel(const uint8_t* ir, size_t len, const void* const* args, void* out,
                  uint64_t begin, uint64_t end, int mode, int fma, int threads) {
  Program p;
  if (!parse(ir, len, p)) return 1;
  if (end > p.size || begin > end) { g_error = "range outside kernel size"; return 1; }
  Mode m = (Mode)mode;
  if (m == MODE_AUTO) {
    m = MODE_WASM;
    for (auto* list : {&p.exp, &p.epi})
      for (auto& nd : *list) if (nd.dtype == JAXCUDA_F16) m = MODE_CPU;
  }
  mark(p.exp, m);
  mark(p.epi, m);
  Ctx cx{m, args, fma};
  const Node& root = p.exp.back();
  const uint32_t out_dtype = p.has_red ? p.epi.back().dtype : root.dtype;
  const Rep acc_rep = rep_of(p.red_dtype, m);
  if (p.has_red && root.rep != acc_rep) { g_error = "body dtype differs from accumulator dtype"; return 1; }
  const bool use_fma = fma && p.has_red && p.red_op == JAXCUDA_OP_ADD && root.op == JAXCUDA_OP_MUL && root.rep == REP_F;
  const int64_t nblocks = (int64_t)((end - begin + B - 1) / B);
  if (threads < 1) threads = 1;
#pragma omp parallel for schedule(dynamic, 16) num_threads(threads)
  for (int64_t blk = 0; blk < nblocks; blk++) {
    const uint64_t g0 = begin + (uint64_t)blk * B;
    const int n = (int)std::min<uint64_t>(B, end - g0);
    std::vector<Lanes> v(p.exp.size());
    if (!p.has_red) {
      for (size_t k = 0; k < p.exp.size(); k++) eval_node(cx, p.exp, k, v, g0, 0, n, nullptr);
      store(out_dtype, root.rep, v.back(), out, g0, n);
      continue;
    }
    Lanes acc;
    identity(p.red_op, p.red_dtype, acc_rep, acc);
    for (size_t k = 0; k < p.exp.size(); k++)
      if (!p.exp[k].dep_r) eval_node(cx, p.exp, k, v, g0, 0, n, nullptr);
    for (uint32_t r = 0; r < p.red_size; r++) {
      const size_t last = p.exp.size() - (use_fma ? 1 : 0);
      for (size_t k = 0; k < last; k++)
        if (p.exp[k].dep_r) eval_node(cx, p.exp, k, v, g0, r, n, nullptr);
      if (use_fma) {
        const Lanes& a = v[root.src[0]];
        const Lanes& b = v[root.src[1]];
        for (int l = 0; l < n; l++) acc.f[l] = std::fmaf(a.f[l], b.f[l], acc.f[l]);
      } else {
        reduce_step(p.red_op, p.red_dtype, acc_rep, acc, v.back(), n);
      }
    }
    std::vector<Lanes> e(p.epi.size());
    for (size_t k = 0; k < p.epi.size(); k++) eval_node(cx, p.epi, k, e, g0, 0, n, &acc);
    store(out_dtype, p.epi.back().rep, e.back(), out, g0, n);
  }
  return 0;
}

// Sort along the last axis: TypedArray.prototype.sort() per row (src/routine.ts:185-193):
// numeric order, -0 before +0, NaN last.  dtype is the element type (Bool as int32).
int oracle_sort(int dtype, const void* x, void* y, uint64_t batch, uint64_t n) {
  auto run = [&](auto* xp, auto* yp, auto less) {
    std::copy(xp, xp + batch * n, yp);
    for (uint64_t b = 0; b < batch; b++) std::sort(yp + b * n, yp + (b + 1) * n, less);
  };
  auto fless = [](auto a, auto b) {
    if (a != a) return false;
    if (b != b) return true;
    if (a == b) return std::signbit(a) && !std::signbit(b);
    return a < b;
  };
  switch (dtype) {
    case JAXCUDA_F32: run((const float*)x, (float*)y, fless); break;
    case JAXCUDA_F64: run((const double*)x, (double*)y, fless); break;
    case JAXCUDA_U32: run((const uint32_t*)x, (uint32_t*)y, std::less<uint32_t>()); break;
    case JAXCUDA_I32:
    case JAXCUDA_BOOL: run((const int32_t*)x, (int32_t*)y, std::less<int32_t>()); break;
    case JAXCUDA_F16: {
      const uint16_t* xp = (const uint16_t*)x; uint16_t* yp = (uint16_t*)y;
      std::copy(xp, xp + batch * n, yp);
      for (uint64_t b = 0; b < batch; b++)
        std::sort(yp + b * n, yp + (b + 1) * n,
                  [&](uint16_t p, uint16_t q) { return fless(half_to_double(p), half_to_double(q)); });
      break;
    }
    default: g_error = "sort: unsupported dtype"; return 1;
  }
  return 0;
}

// Stable argsort along the last axis (src/routine.ts:195-214): NaNs compare equal to each
// other and after everything else, -0 == +0, ties keep index order.  Writes the gathered
// values to y and the int32 indices to yi.
int oracle_argsort(int dtype, const void* x, void* y, int32_t* yi, uint64_t batch, uint64_t n) {
  auto run = [&](auto* xp, auto* yp, auto to_num) {
    for (uint64_t b = 0; b < batch; b++) {
      auto* row = xp + b * n;
      int32_t* idx = yi + b * n;
      for (uint64_t k = 0; k < n; k++) idx[k] = (int32_t)k;
      std::stable_sort(idx, idx + n, [&](int32_t p, int32_t q) {
        auto a = to_num(row[p]); auto c = to_num(row[q]);
        if (a != a) return false;
        if (c != c) return true;
        return a < c;
      });
      for (uint64_t k = 0; k < n; k++) yp[b * n + k] = row[idx[k]];
    }
  };
  auto same = [](auto v) { return v; };
  switch (dtype) {
    case JAXCUDA_F32: run((const float*)x, (float*)y, same); break;
    case JAXCUDA_F64: run((const double*)x, (double*)y, same); break;
    case JAXCUDA_U32: run((const uint32_t*)x, (uint32_t*)y, same); break;
    case JAXCUDA_I32:
    case JAXCUDA_BOOL: run((const int32_t*)x, (int32_t*)y, same); break;
    case JAXCUDA_F16: run((const uint16_t*)x, (uint16_t*)y, [](uint16_t h) { return half_to_double(h); }); break;
    default: g_error = "argsort: unsupported dtype"; return 1;
  }
  return 0;
}

// Scatter (src/routine.ts:226-296): zero-fill, then for every update element translate its
// coordinate to a destination and store / add / or.  Shapes are passed flat; `axis[k]` is the output
// axis that index input k addresses.  Elements are 4 bytes (f32 / i32 / u32 / Bool) or f64 / f16.
int oracle_scatter(int dtype, int add, int unique, int out_dim, int out_rank, const int64_t* out_shape,
                   int upd_rank, const int64_t* upd_shape, int n_index, const int32_t* axis,
                   const int32_t* idx_ranks, const int64_t* idx_shapes, const void* updates,
                   const int32_t* const* indices, void* output) {
  int64_t out_stride[16], upd_stride[16], out_size = 1, n_upd = 1;
  for (int i = out_rank - 1; i >= 0; i--) { out_stride[i] = out_size; out_size *= out_shape[i]; }
  for (int i = upd_rank - 1; i >= 0; i--) { upd_stride[i] = n_upd; n_upd *= upd_shape[i]; }
  const int eb = dtype == JAXCUDA_F16 ? 2 : dtype == JAXCUDA_F64 ? 8 : 4;
  memset(output, 0, (size_t)out_size * eb);
  const bool accumulate = add && !unique;
  int index_rank = 0;
  std::vector<std::vector<int64_t>> ishape(n_index), istride(n_index);
  const int64_t* sh = idx_shapes;
  for (int k = 0; k < n_index; k++) {
    ishape[k].assign(sh, sh + idx_ranks[k]);
    istride[k].assign(idx_ranks[k], 1);
    for (int j = idx_ranks[k] - 2; j >= 0; j--) istride[k][j] = istride[k][j + 1] * ishape[k][j + 1];
    sh += idx_ranks[k];
    index_rank = std::max(index_rank, idx_ranks[k]);
  }
  std::vector<int> free_dims;
  for (int i = 0; i < upd_rank; i++) if (i < out_dim || i >= out_dim + index_rank) free_dims.push_back(i);
  for (int64_t i = 0; i < n_upd; i++) {
    int64_t at = 0;
    bool valid = true;
    size_t fd = 0;
    for (int ax = 0; ax < out_rank && valid; ax++) {
      int which = -1;
      for (int k = 0; k < n_index; k++) if (axis[k] == ax) which = k;
      int64_t coord;
      if (which < 0) {
        const int ud = free_dims[fd++];
        coord = (i / upd_stride[ud]) % upd_shape[ud];
      } else {
        const int first = out_dim + index_rank - idx_ranks[which];
        int64_t off = 0;
        for (int j = 0; j < idx_ranks[which]; j++) {
          if (ishape[which][j] == 1) continue;
          const int ud = first + j;
          off += ((i / upd_stride[ud]) % upd_shape[ud]) * istride[which][j];
        }
        coord = indices[which][off];
      }
      if (coord < 0 || coord >= out_shape[ax]) valid = false;
      else at += coord * out_stride[ax];
    }
    if (!valid) continue;
    if (dtype == JAXCUDA_F32) { float* o = (float*)output; const float v = ((const float*)updates)[i]; if (accumulate) o[at] += v; else o[at] = v; }
    else if (dtype == JAXCUDA_F64) { double* o = (double*)output; const double v = ((const double*)updates)[i]; if (accumulate) o[at] += v; else o[at] = v; }
    else if (dtype == JAXCUDA_F16) {
      uint16_t* o = (uint16_t*)output; const uint16_t v = ((const uint16_t*)updates)[i];
      o[at] = accumulate ? double_to_half(half_to_double(o[at]) + half_to_double(v)) : v;
    } else {
      uint32_t* o = (uint32_t*)output; const uint32_t v = ((const uint32_t*)updates)[i];
      if (accumulate && dtype == JAXCUDA_BOOL) o[at] |= v; else if (accumulate) o[at] += v; else o[at] = v;
    }
  }
  return 0;
}

// Scalar entry points for the known-answer tests of the software transcendentals.
float oracle_wasm_unary(int op, float x) {
  switch (op) {
    case JAXCUDA_OP_SIN: return wasm_sin(x);
    case JAXCUDA_OP_COS: return wasm_cos(x);
    case JAXCUDA_OP_ASIN: return wasm_asin(x);
    case JAXCUDA_OP_ATAN: return wasm_atan(x);
    case JAXCUDA_OP_EXP: return wasm_exp(x);
    case JAXCUDA_OP_LOG: return wasm_log(x);
    case JAXCUDA_OP_ERF: return wasm_erf(x);
    case JAXCUDA_OP_ERFC: return wasm_erfc(x);
    default: return std::numeric_limits<float>::quiet_NaN();
  }
}
void oracle_threefry2x32(uint32_t k0, uint32_t k1, uint32_t c0, uint32_t c1, uint32_t* out) {
  threefry2x32(k0, k1, c0, c1, out[0], out[1]);
}
uint16_t oracle_double_to_half(double x) { return double_to_half(x); }
double oracle_half_to_double(uint16_t h) { return half_to_double(h); }

}  // extern "C"

// ---- dense linear-algebra routines (src/routine.ts:298-432) --------------------------------------
// The reference runs on typed arrays with JavaScript numbers: every intermediate is a double, a
// value is rounded to the element type when it is stored and read back rounded.  T is float or
// double; `volatile`-free plain code with -ffp-contract=off keeps multiply and subtract separate.
namespace {

template <class T>
void triangular_solve_ref(const T* a, const T* b, T* x, int64_t mats, int64_t rows, int64_t n, bool unit) {  // :298-338
  for (int64_t c = 0; c < mats; c++) {
    const T* a1 = a + c * n * n;
    for (int64_t t = 0; t < rows; t++) {
      const T* b1 = b + (c * rows + t) * n;
      T* x1 = x + (c * rows + t) * n;
      for (int64_t i = n - 1; i >= 0; i--) {
        double sum = b1[i];
        for (int64_t j = i + 1; j < n; j++) sum -= (double)a1[i * n + j] * (double)x1[j];
        x1[i] = (T)(unit ? sum : sum / (double)a1[i * n + i]);
      }
    }
  }
}

template <class T>
void cholesky_ref(const T* x, T* y, int64_t batch, int64_t n) {  // :340-366
  for (int64_t i = 0; i < batch * n * n; i++) y[i] = 0;
  for (int64_t m = 0; m < batch; m++) {
    const T* ar = x + m * n * n;
    T* out = y + m * n * n;
    for (int64_t i = 0; i < n; i++)
      for (int64_t j = 0; j <= i; j++) {
        double sum = ar[i * n + j];
        for (int64_t k = 0; k < j; k++) sum -= (double)out[i * n + k] * (double)out[j * n + k];
        out[i * n + j] = (T)(i == j ? std::sqrt(sum) : sum / (double)out[j * n + j]);
      }
  }
}

template <class T>
void lu_ref(const T* a, T* lu, int32_t* pivots, int32_t* perm, int64_t batch, int64_t m, int64_t n) {  // :368-432
  const int64_t r = std::min(m, n);
  for (int64_t bi = 0; bi < batch; bi++) {
    const T* ar = a + bi * m * n;
    T* out = lu + bi * m * n;
    int32_t* piv = pivots + bi * r;
    int32_t* p = perm + bi * m;
    for (int64_t i = 0; i < m * n; i++) out[i] = ar[i];
    for (int64_t i = 0; i < m; i++) p[i] = (int32_t)i;
    for (int64_t j = 0; j < r; j++) {
      double maxVal = std::fabs((double)out[j * n + j]);
      int64_t maxRow = j;
      for (int64_t i = j + 1; i < m; i++) {
        const double val = std::fabs((double)out[i * n + j]);
        if (val > maxVal) { maxVal = val; maxRow = i; }
      }
      piv[j] = (int32_t)maxRow;
      if (maxRow != j) {
        for (int64_t col = 0; col < n; col++) std::swap(out[j * n + col], out[maxRow * n + col]);
        std::swap(p[j], p[maxRow]);
      }
      const double diag = out[j * n + j];
      if (diag != 0) {
        for (int64_t i = j + 1; i < m; i++) {
          const double factor = (double)out[i * n + j] / diag;
          out[i * n + j] = (T)factor;
          for (int64_t col = j + 1; col < n; col++)
            out[i * n + col] = (T)((double)out[i * n + col] - factor * (double)out[j * n + col]);
        }
      }
    }
  }
}

}  // namespace

extern "C" {

// dtype: JAXCUDA_F32 or JAXCUDA_F64; returns 0, or 1 for another dtype.
int oracle_triangular_solve(int dtype, const void* a, const void* b, void* x, int64_t mats, int64_t rows, int64_t n, int unit) {
  if (dtype == JAXCUDA_F32) triangular_solve_ref((const float*)a, (const float*)b, (float*)x, mats, rows, n, unit != 0);
  else if (dtype == JAXCUDA_F64) triangular_solve_ref((const double*)a, (const double*)b, (double*)x, mats, rows, n, unit != 0);
  else return 1;
  return 0;
}
int oracle_cholesky(int dtype, const void* x, void* y, int64_t batch, int64_t n) {
  if (dtype == JAXCUDA_F32) cholesky_ref((const float*)x, (float*)y, batch, n);
  else if (dtype == JAXCUDA_F64) cholesky_ref((const double*)x, (double*)y, batch, n);
  else return 1;
  return 0;
}
int oracle_lu(int dtype, const void* a, void* lu, int32_t* pivots, int32_t* perm, int64_t batch, int64_t m, int64_t n) {
  if (dtype == JAXCUDA_F32) lu_ref((const float*)a, (float*)lu, pivots, perm, batch, m, n);
  else if (dtype == JAXCUDA_F64) lu_ref((const double*)a, (double*)lu, pivots, perm, batch, m, n);
  else return 1;
  return 0;
}

}  // extern "C"

// ---- JacobiEigh (src/routine.ts:434-541) and Fft (:543-624) ----------------------------------------
namespace {

template <class T>
void jacobi_eigh_ref(const T* input, T* diagonalized, T* vectors, int64_t batch, int64_t n, int max_sweeps, double tolerance) {
  auto sym = [n](int64_t i, int64_t j) { return i >= j ? i * n + j : j * n + i; };
  for (int64_t m = 0; m < batch; m++) {
    const T* x = input + m * n * n;
    T* a = diagonalized + m * n * n;
    T* v = vectors + m * n * n;
    for (int64_t i = 0; i < n * n; i++) { a[i] = 0; v[i] = 0; }
    for (int64_t i = 0; i < n; i++) {
      for (int64_t j = 0; j <= i; j++) a[i * n + j] = x[i * n + j];
      v[i * n + i] = 1;
    }
    double max_abs = 1;
    for (int64_t i = 0; i < n; i++)
      for (int64_t j = 0; j <= i; j++) max_abs = std::max(max_abs, std::fabs((double)a[i * n + j]));
    auto off_diagonal = [&]() {
      double mx = 0;
      for (int64_t i = 0; i < n; i++)
        for (int64_t j = 0; j < i; j++) mx = std::max(mx, std::fabs((double)a[i * n + j]));
      return mx;
    };
    const double threshold = tolerance * max_abs;
    double off = off_diagonal();
    for (int sweep = 0; sweep < max_sweeps && off > threshold; sweep++) {
      for (int64_t p = 0; p < n - 1; p++)
        for (int64_t q = p + 1; q < n; q++) {
          const int64_t pp = p * n + p, qq = q * n + q, pq = sym(p, q);
          const double app = a[pp], aqq = a[qq], apq = a[pq];
          if (apq == 0) continue;
          const double tau = (aqq - app) / (2 * apq);
          const double tau_sign = tau >= 0 ? 1 : -1;
          const double t = tau_sign / (std::fabs(tau) + std::sqrt(tau * tau + 1));
          const double c = 1 / std::sqrt(t * t + 1);
          const double s = t * c;
          for (int64_t k = 0; k < n; k++) {
            if (k == p || k == q) continue;
            const int64_t kp = sym(k, p), kq = sym(k, q);
            const double akp = a[kp], akq = a[kq];
            a[kp] = (T)(c * akp - s * akq);
            a[kq] = (T)(s * akp + c * akq);
          }
          a[pp] = (T)(c * c * app - 2 * s * c * apq + s * s * aqq);
          a[qq] = (T)(s * s * app + 2 * s * c * apq + c * c * aqq);
          a[pq] = 0;
          for (int64_t k = 0; k < n; k++) {
            const double vkp = v[k * n + p], vkq = v[k * n + q];
            v[k * n + p] = (T)(c * vkp - s * vkq);
            v[k * n + q] = (T)(s * vkp + c * vkq);
          }
        }
      off = off_diagonal();
    }
  }
}

template <class T>
void fft_ref(const T* real, const T* imag, T* out_real, T* out_imag, int64_t batch, int64_t n, const int* factors, int nf,
             bool inverse) {
  const double angle_scale = (inverse ? 2 : -2) * 3.141592653589793;
  std::vector<int64_t> permutation(n);
  int max_factor = 1;
  for (int f = 0; f < nf; f++) max_factor = std::max(max_factor, factors[f]);
  for (int64_t index = 0; index < n; index++) {
    int64_t remaining = index, stride = 1, reversed = 0;
    for (int f = 0; f < nf; f++) {
      const int64_t digit = remaining % factors[f];
      remaining /= factors[f];
      stride *= factors[f];
      reversed += digit * (n / stride);
    }
    permutation[index] = reversed;
  }
  std::vector<double> sr(max_factor), si(max_factor);
  for (int64_t row = 0; row < batch; row++) {
    const int64_t offset = row * n;
    for (int64_t index = 0; index < n; index++) {
      out_real[offset + index] = real[offset + permutation[index]];
      out_imag[offset + index] = imag[offset + permutation[index]];
    }
    int64_t prev = 1;
    for (int stage = 0; stage < nf; stage++) {
      const int64_t radix = factors[stage], span = prev * radix;
      const double stage_scale = (inverse && stage == nf - 1) ? 1.0 / (double)n : 1.0;
      for (int64_t group = 0; group < n; group += span)
        for (int64_t j = 0; j < prev; j++) {
          for (int64_t q = 0; q < radix; q++) {
            const int64_t idx = offset + group + j + q * prev;
            const double angle = (angle_scale * (double)q * (double)j) / (double)span;
            const double c = std::cos(angle), s = std::sin(angle);
            const double xr = out_real[idx], xi = out_imag[idx];
            sr[q] = xr * c - xi * s;
            si[q] = xr * s + xi * c;
          }
          for (int64_t p = 0; p < radix; p++) {
            double sum_real = 0, sum_imag = 0;
            for (int64_t q = 0; q < radix; q++) {
              const double angle = (angle_scale * (double)q * (double)p) / (double)radix;
              const double c = std::cos(angle), s = std::sin(angle);
              sum_real += sr[q] * c - si[q] * s;
              sum_imag += sr[q] * s + si[q] * c;
            }
            const int64_t idx = offset + group + j + p * prev;
            out_real[idx] = (T)(sum_real * stage_scale);
            out_imag[idx] = (T)(sum_imag * stage_scale);
          }
        }
      prev = span;
    }
  }
}

}  // namespace

extern "C" {

int oracle_jacobi_eigh(int dtype, const void* x, void* diagonalized, void* vectors, int64_t batch, int64_t n, int max_sweeps,
                       double tolerance) {
  if (dtype == JAXCUDA_F32) jacobi_eigh_ref((const float*)x, (float*)diagonalized, (float*)vectors, batch, n, max_sweeps, tolerance);
  else if (dtype == JAXCUDA_F64) jacobi_eigh_ref((const double*)x, (double*)diagonalized, (double*)vectors, batch, n, max_sweeps, tolerance);
  else return 1;
  return 0;
}
int oracle_fft(int dtype, const void* real, const void* imag, void* out_real, void* out_imag, int64_t batch, int64_t n,
               const int* factors, int n_factors, int inverse) {
  if (dtype == JAXCUDA_F32) fft_ref((const float*)real, (const float*)imag, (float*)out_real, (float*)out_imag, batch, n, factors, n_factors, inverse != 0);
  else if (dtype == JAXCUDA_F64) fft_ref((const double*)real, (const double*)imag, (double*)out_real, (double*)out_imag, batch, n, factors, n_factors, inverse != 0);
  else return 1;
  return 0;
}

}  // extern "C"
