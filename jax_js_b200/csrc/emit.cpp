#include "emit.hpp"

#include <algorithm>
#include <cstdlib>
#include <cstring>
#include <map>
#include <sstream>
#include <stdexcept>

#include "prelude.hpp"

namespace jaxcuda {

namespace {

// ---- small helpers ------------------------------------------------------------------

std::string S(int64_t v) { return std::to_string(v); }

const char* ctype(uint32_t dt) {  // type a value of this dtype has in registers
  switch (dt) {
    case JAXCUDA_F32: case JAXCUDA_F16: return "float";  // f16 values are carried as f32, rounded on Cast/store
    case JAXCUDA_F64: return "double";
    case JAXCUDA_U32: return "u32";
    default: return "int";
  }
}
const char* ptype(uint32_t dt) {  // element type in memory
  switch (dt) {
    case JAXCUDA_F32: return "float";
    case JAXCUDA_F16: return "jx_half";
    case JAXCUDA_F64: return "double";
    case JAXCUDA_U32: return "u32";
    default: return "int";
  }
}

[[noreturn]] void unsupported(uint32_t op, uint32_t dtype, const std::string& extra = "") {
  // wording of UnsupportedOpError, src/backend.ts:228-234
  throw std::runtime_error(std::string(op_name(op)) + "<" + dtype_name(dtype) + "> not supported in cuda backend" +
                           (extra.empty() ? "" : " with arg " + extra));
}

std::string hex32(uint32_t v) { char b[16]; snprintf(b, sizeof b, "0x%08xu", v); return b; }

std::string literal(const Node& nd) {
  if (nd.dtype == JAXCUDA_F32 || nd.dtype == JAXCUDA_F16) {
    double d; memcpy(&d, &nd.arg0, 8);
    float f = (float)d; uint32_t bits; memcpy(&bits, &f, 4);
    return "__uint_as_float(" + hex32(bits) + ")";
  }
  if (nd.dtype == JAXCUDA_F64) {
    char b[48]; snprintf(b, sizeof b, "__longlong_as_double(0x%016llxLL)", (unsigned long long)nd.arg0);
    return b;
  }
  if (nd.dtype == JAXCUDA_U32) return hex32((uint32_t)nd.arg0);
  if (nd.dtype == JAXCUDA_BOOL) return (nd.arg0 & 0xffffffffu) ? "1" : "0";
  return "((int)" + hex32((uint32_t)nd.arg0) + ")";
}

struct Env {
  std::string prefix = "t";
  std::string gidx = "gidx", ridx = "ridx", acc = "acc";
  const std::map<size_t, std::string>* load_override = nullptr;  // node -> expression of the loaded value
};

bool in_range(const std::optional<Affine>& a, uint32_t len) { return a && a->lo >= 0 && a->hi < (int64_t)len; }

std::string load_value(const Node& nd, const std::string& ix, bool proven) {
  const uint32_t len = nd.arg1;
  if (len == 0) return nd.dtype == JAXCUDA_F64 ? "0.0" : (nd.dtype == JAXCUDA_F32 || nd.dtype == JAXCUDA_F16) ? "0.0f" : "0";
  // An index outside the buffer reads element 0, as the Wasm emitter does (translation.ts:221-228).
  std::string at = proven ? ix : "((u32)(" + ix + ") < " + S(len) + "u ? (" + ix + ") : 0)";
  // Checked build: every scalar load tests its index, also those whose range the affine analysis
  // has proven, and counts the misses by kind.
  if (emit_checked()) at = "jx_ix((i64)(" + ix + "), " + S(len) + "u, " + (proven ? "1" : "0") + ")";
  std::string p = std::string("((const ") + ptype(nd.dtype) + "*)p" + S((int64_t)nd.arg0) + ")[" + at + "]";
  return nd.dtype == JAXCUDA_F16 ? "jx_h2f(" + p + ")" : p;
}

std::string binary_expr(uint32_t op, uint32_t dt, const std::string& a, const std::string& b, uint64_t arg0,
                        const Node* bnode) {
  const bool f = dt == JAXCUDA_F32 || dt == JAXCUDA_F16, d = dt == JAXCUDA_F64, bo = dt == JAXCUDA_BOOL,
             i = dt == JAXCUDA_I32, u = dt == JAXCUDA_U32;
  auto wrap = [&](const char* sym) {  // integer arithmetic wraps modulo 2^32 (translation.ts:38-45)
    if (i) return "(int)((u32)" + a + " " + sym + " (u32)" + b + ")";
    return "(" + a + " " + sym + " " + b + ")";
  };
  switch (op) {
    case JAXCUDA_OP_ADD: return bo ? "(" + a + " | " + b + ")" : wrap("+");
    case JAXCUDA_OP_SUB: if (bo) unsupported(op, dt); return wrap("-");
    case JAXCUDA_OP_MUL: return bo ? "(" + a + " & " + b + ")" : wrap("*");
    case JAXCUDA_OP_IDIV: {
      if (f) return "jx_fidiv(" + a + ", " + b + ")";
      if (d) return "jx_didiv(" + a + ", " + b + ")";
      const bool safe_const = bnode && bnode->op == JAXCUDA_OP_CONST && (uint32_t)bnode->arg0 != 0 &&
                              (uint32_t)bnode->arg0 != 0xffffffffu;
      if (i) return safe_const ? "(" + a + " / " + b + ")" : "jx_idiv(" + a + ", " + b + ")";
      if (u) return safe_const ? "(" + a + " / " + b + ")" : "jx_udiv(" + a + ", " + b + ")";
      unsupported(op, dt);
    }
    case JAXCUDA_OP_MOD: {
      if (f) return "jx_fmod(" + a + ", " + b + ")";
      if (d) return "jx_dmod(" + a + ", " + b + ")";
      const bool safe_const = bnode && bnode->op == JAXCUDA_OP_CONST && (uint32_t)bnode->arg0 != 0 &&
                              (uint32_t)bnode->arg0 != 0xffffffffu;
      if (i) return safe_const ? "(" + a + " % " + b + ")" : "jx_imod(" + a + ", " + b + ")";
      if (u) return safe_const ? "(" + a + " % " + b + ")" : "jx_umod(" + a + ", " + b + ")";
      unsupported(op, dt);
    }
    case JAXCUDA_OP_MIN:
      if (bo) return "(" + a + " & " + b + ")";
      return std::string(f ? "jx_fmin(" : d ? "jx_dmin(" : i ? "jx_imin(" : "jx_umin(") + a + ", " + b + ")";
    case JAXCUDA_OP_MAX:
      if (bo) return "(" + a + " | " + b + ")";
      return std::string(f ? "jx_fmax(" : d ? "jx_dmax(" : i ? "jx_imax(" : "jx_umax(") + a + ", " + b + ")";
    case JAXCUDA_OP_BITCOMBINE: {
      if (f || d) unsupported(op, dt);
      const char* sym = arg0 == 0 ? "&" : arg0 == 1 ? "|" : "^";
      return "(" + a + " " + sym + " " + b + ")";
    }
    case JAXCUDA_OP_BITSHIFT: {  // count masked to 5 bits; shr is logical for every dtype (translation.ts:101-103)
      if (f || d || bo) unsupported(op, dt);
      const char* sym = arg0 == 0 ? "<<" : ">>";
      return std::string("(") + ctype(dt) + ")((u32)" + a + " " + sym + " ((u32)" + b + " & 31u))";
    }
    default: unsupported(op, dt);
  }
}

std::string unary_math(uint32_t op, uint32_t dt, const std::string& a) {
  const char* fn = nullptr;
  switch (op) {
    case JAXCUDA_OP_SIN: fn = "jx_sin"; break;
    case JAXCUDA_OP_COS: fn = "jx_cos"; break;
    case JAXCUDA_OP_ASIN: fn = "jx_asin"; break;
    case JAXCUDA_OP_ATAN: fn = "jx_atan"; break;
    case JAXCUDA_OP_EXP: fn = "jx_exp"; break;
    case JAXCUDA_OP_LOG: fn = "jx_log"; break;
    case JAXCUDA_OP_ERF: fn = "jx_erf"; break;
    case JAXCUDA_OP_ERFC: fn = "jx_erfc"; break;
    default: break;
  }
  if (!dtype_is_float(dt)) unsupported(op, dt);
  if (fn) {  // f32 routines; f64 is demoted and promoted as in translation.ts:115-122
    if (dt == JAXCUDA_F64) return std::string("(double)") + fn + "((float)" + a + ")";
    return std::string(fn) + "(" + a + ")";
  }
  const bool d = dt == JAXCUDA_F64;
  switch (op) {
    case JAXCUDA_OP_SQRT: return (d ? "sqrt(" : "sqrtf(") + a + ")";
    case JAXCUDA_OP_FLOOR: return (d ? "floor(" : "floorf(") + a + ")";
    case JAXCUDA_OP_CEIL: return (d ? "ceil(" : "ceilf(") + a + ")";
    case JAXCUDA_OP_RECIPROCAL: return (d ? "(1.0 / " : "(1.0f / ") + a + ")";  // true division (translation.ts:132-134)
    default: unsupported(op, dt);
  }
}

std::string cast_expr(uint32_t to, uint32_t from, const std::string& a) {  // translation.ts:139-173
  const bool from_f = from == JAXCUDA_F32 || from == JAXCUDA_F16, from_d = from == JAXCUDA_F64;
  switch (to) {
    case JAXCUDA_BOOL:
      return from == JAXCUDA_BOOL ? a : "(int)(" + a + (from_f ? " != 0.0f)" : from_d ? " != 0.0)" : " != 0)");
    case JAXCUDA_I32:
      if (from_f) return "__float2int_rz(" + a + ")";      // trunc_sat: saturates, NaN -> 0
      if (from_d) return "__double2int_rz(" + a + ")";
      return "(int)" + a;
    case JAXCUDA_U32:
      if (from_f) return "__float2uint_rz(" + a + ")";
      if (from_d) return "__double2uint_rz(" + a + ")";
      return "(u32)" + a;
    case JAXCUDA_F32:
      if (from == JAXCUDA_F32 || from == JAXCUDA_F16) return a;
      return "(float)" + a;  // signed convert for int32 and Bool, unsigned for uint32
    case JAXCUDA_F16:
      if (from == JAXCUDA_F16) return a;
      if (from_f) return "jx_round_h(" + a + ")";
      return "jx_round_h((float)" + a + ")";
    case JAXCUDA_F64:
      return from_d ? a : "(double)" + a;
    default: unsupported(JAXCUDA_OP_CAST, to);
  }
}

std::string bitcast_expr(uint32_t to, uint32_t from, const std::string& a) {  // translation.ts:175-189
  auto is_i = [](uint32_t t) { return t == JAXCUDA_I32 || t == JAXCUDA_U32; };
  if (to == from) return a;
  if (is_i(to) && from == JAXCUDA_F32) return to == JAXCUDA_I32 ? "__float_as_int(" + a + ")" : "__float_as_uint(" + a + ")";
  if (is_i(to) && is_i(from)) return std::string("(") + ctype(to) + ")" + a;
  if (to == JAXCUDA_F32 && from == JAXCUDA_I32) return "__int_as_float(" + a + ")";
  if (to == JAXCUDA_F32 && from == JAXCUDA_U32) return "__uint_as_float(" + a + ")";
  unsupported(JAXCUDA_OP_BITCAST, to, dtype_name(from));
}

// Emit `const T name = expr;` for every wanted node that has no name yet.
void emit_nodes(std::ostream& os, const std::vector<Node>& nodes, const Analysis& an,
                std::vector<std::string>& names, const std::vector<char>& want, const Env& env,
                const std::string& indent) {
  for (size_t i = 0; i < nodes.size(); i++) {
    if (!want[i] || !names[i].empty()) continue;
    const Node& nd = nodes[i];
    auto a = [&](int s) -> const std::string& { return names[nd.src[s]]; };
    std::string expr;
    switch (nd.op) {
      case JAXCUDA_OP_CONST: names[i] = literal(nd); continue;
      case JAXCUDA_OP_SPECIAL: names[i] = nd.arg0 == 0 ? env.gidx : env.ridx; continue;
      case JAXCUDA_OP_VARIABLE: names[i] = env.acc; continue;
      case JAXCUDA_OP_GLOBALINDEX: {
        if (env.load_override) {
          auto it = env.load_override->find(i);
          if (it != env.load_override->end()) { expr = it->second; break; }
        }
        expr = load_value(nd, a(0), in_range(an.affine[nd.src[0]], nd.arg1));
        break;
      }
      case JAXCUDA_OP_CAST: expr = cast_expr(nd.dtype, nodes[nd.src[0]].dtype, a(0)); break;
      case JAXCUDA_OP_BITCAST: expr = bitcast_expr(nd.dtype, nodes[nd.src[0]].dtype, a(0)); break;
      case JAXCUDA_OP_BITINVERT:
        if (dtype_is_float(nd.dtype)) unsupported(nd.op, nd.dtype);
        expr = nd.dtype == JAXCUDA_BOOL ? "(" + a(0) + " ^ 1)" : "(~" + a(0) + ")";
        break;
      case JAXCUDA_OP_CMPLT: expr = "(int)(" + a(0) + " < " + a(1) + ")"; break;
      case JAXCUDA_OP_CMPNE: expr = "(int)(" + a(0) + " != " + a(1) + ")"; break;
      case JAXCUDA_OP_WHERE: expr = "(" + a(0) + " ? " + a(1) + " : " + a(2) + ")"; break;
      case JAXCUDA_OP_THREEFRY2X32:
        if (nd.arg0 > 2) unsupported(nd.op, nd.dtype, S((int64_t)nd.arg0));
        expr = "jx_threefry(" + a(0) + ", " + a(1) + ", " + a(2) + ", " + a(3) + ", " + S((int64_t)nd.arg0) + ")";
        break;
      default:
        if (nd.nsrc == 2) expr = binary_expr(nd.op, nd.dtype, a(0), a(1), nd.arg0, &nodes[nd.src[1]]);
        else expr = unary_math(nd.op, nd.dtype, a(0));
    }
    names[i] = env.prefix + S((int64_t)i);
    os << indent << "const " << ctype(nd.dtype) << " " << names[i] << " = " << expr << ";\n";
  }
}

std::vector<char> closure(const std::vector<Node>& nodes, size_t root) {
  std::vector<char> m(nodes.size(), 0);
  m[root] = 1;
  for (size_t i = root + 1; i-- > 0;)
    if (m[i]) for (uint32_t s = 0; s < nodes[i].nsrc; s++) m[nodes[i].src[s]] = 1;
  return m;
}

std::string to_storage(uint32_t dt, const std::string& v) { return dt == JAXCUDA_F16 ? "jx_f2h(" + v + ")" : v; }
std::string from_storage(uint32_t dt, const std::string& v) { return dt == JAXCUDA_F16 ? "jx_h2f(" + v + ")" : v; }

std::string identity_literal(uint32_t op, uint32_t dt) {  // src/alu.ts:1584-1604
  if (dt == JAXCUDA_BOOL) return (op == JAXCUDA_OP_ADD || op == JAXCUDA_OP_MAX) ? "0" : "1";
  if (dt == JAXCUDA_I32) return op == JAXCUDA_OP_ADD ? "0" : op == JAXCUDA_OP_MUL ? "1" : op == JAXCUDA_OP_MIN ? "2147483647" : "(-2147483647 - 1)";
  if (dt == JAXCUDA_U32) return op == JAXCUDA_OP_ADD ? "0u" : op == JAXCUDA_OP_MUL ? "1u" : op == JAXCUDA_OP_MIN ? "0xffffffffu" : "0u";
  if (dt == JAXCUDA_F64) return op == JAXCUDA_OP_ADD ? "0.0" : op == JAXCUDA_OP_MUL ? "1.0" : op == JAXCUDA_OP_MIN ? "(double)JX_INF" : "(double)(-JX_INF)";
  return op == JAXCUDA_OP_ADD ? "0.0f" : op == JAXCUDA_OP_MUL ? "1.0f" : op == JAXCUDA_OP_MIN ? "JX_INF" : "(-JX_INF)";
}

// How a load behaves over an aligned run of V consecutive values of `var`.
enum LoadKind { LK_GATHER, LK_BROADCAST, LK_VECTOR };

LoadKind classify_load(const Node& nd, const std::optional<Affine>& ix, int var, int V) {
  if (!ix || !in_range(ix, nd.arg1)) return LK_GATHER;
  int64_t cv = 0;
  for (const Term& t : ix->terms) {
    if (t.var != var) continue;
    if (t.div == 1) {
      if (t.mod && t.mod % V) return LK_GATHER;
      cv = t.coef;
    } else if (t.div % V) {
      return LK_GATHER;
    }
  }
  if (cv == 0) return LK_BROADCAST;
  if (cv != 1 || ix->c0 % V) return LK_GATHER;
  for (const Term& t : ix->terms)
    if (!(t.var == var && t.div == 1) && t.coef % V) return LK_GATHER;
  return LK_VECTOR;
}

struct Builder {
  const KernelIR& k;
  const Options& opt;

  // Source header: the prelude, with the bit-faithful transcendentals selected for kernels small
  // enough to be latency-bound (and for all kernels when asked).
  std::string header(int hint_default = 0) const {
    const double work = (double)k.size * (k.has_red ? (double)k.red_size : 1.0);
    const bool exact = opt.exact_math == 1 || (opt.exact_math < 0 && work < opt.exact_math_work);
    return std::string(exact ? "#define JX_EXACT_TRANSCENDENTALS 1\n" : "") + "#define JX_LD_HINT " + S(opt.ld_hint >= 0 ? opt.ld_hint : hint_default) + "\n" + kPrelude;
  }

  Analysis an_exp, an_epi;
  uint32_t out_dt;

  Builder(const KernelIR& k_, const Options& o) : k(k_), opt(o) {
    an_exp = analyze(k.exp, k.size, k.has_red ? k.red_size : 0);
    if (k.has_red) an_epi = analyze(k.epi, k.size, 0);
    out_dt = k.out_dtype();
  }

  std::string params() const {
    std::ostringstream os;
    for (uint32_t i = 0; i < k.nargs; i++) os << "const void* __restrict__ p" << i << ", ";
    os << ptype(out_dt) << "* __restrict__ out, void* __restrict__ scratch";
    return os.str();
  }

  std::string params_rev() const { return params() + ", int jx_rev"; }
  static const char* rev_block() { return "  const unsigned jx_bx = jx_rev ? gridDim.x - 1 - blockIdx.x : blockIdx.x;\n"; }

  std::string red(const std::string& a, const std::string& b) const {
    return binary_expr(k.red_op, k.red_dtype, a, b, 0, nullptr);
  }

  void account(Plan& p) const {
    std::map<uint32_t, double> bytes;
    auto scan = [&](const std::vector<Node>& nodes) {
      for (const Node& nd : nodes)
        if (nd.op == JAXCUDA_OP_GLOBALINDEX)
          bytes[(uint32_t)nd.arg0] = std::max(bytes[(uint32_t)nd.arg0], (double)nd.arg1 * dtype_bytes(nd.dtype));
    };
    scan(k.exp);
    scan(k.epi);
    p.algo_bytes = (double)k.size * dtype_bytes(out_dt);
    for (auto& kv : bytes) p.algo_bytes += kv.second;
    p.algo_flops = (double)k.size * (k.has_red ? 2.0 * k.red_size : 1.0);
  }

  // Loads of `nodes` that can be fetched once per run of V values of `var` starting at an
  // aligned position: emits the index closure at the run start (prefix b) and the fetch,
  // and records the per-lane expression (pack element or broadcast scalar) as an override.
  // `slot` is an optional array suffix for ILP copies, e.g. "[j]".
  void preload(std::ostream& decl, std::ostream& fetch, const std::vector<Node>& nodes, const Analysis& an,
               const std::vector<char>& live, int var, int V, const Env& base_env, const std::string& run_start,
               const std::string& slot_decl, const std::string& slot_use, const std::string& lane,
               std::map<size_t, std::string>& override_, std::vector<std::string>& bnames,
               const std::string& indent) const {
    Env env = base_env;
    env.prefix = "b";
    if (var == 0) env.gidx = run_start; else env.ridx = run_start;
    for (size_t i = 0; i < nodes.size(); i++) {
      const Node& nd = nodes[i];
      if (!live[i] || nd.op != JAXCUDA_OP_GLOBALINDEX || nd.arg1 == 0) continue;
      LoadKind lk = classify_load(nd, an.affine[nd.src[0]], var, V);
      if (lk == LK_GATHER) continue;
      if (lk == LK_BROADCAST && !(var == 0 ? an.dep_g[i] : an.dep_r[i])) continue;  // invariant anyway
      std::vector<char> need = closure(nodes, nd.src[0]);
      emit_nodes(fetch, nodes, an, bnames, need, env, indent);
      const std::string ix = bnames[nd.src[0]];
      const std::string ptr = std::string("((const ") + ptype(nd.dtype) + "*)p" + S((int64_t)nd.arg0) + ")";
      if (lk == LK_VECTOR) {
        decl << indent << "jx_pack<" << ptype(nd.dtype) << ", " << V << "> pk" << i << slot_decl << ";\n";
        fetch << indent << "jx_load(pk" << i << slot_use << ", " << ptr << " + " << ix << ");\n";
        override_[i] = from_storage(nd.dtype, "pk" + S((int64_t)i) + slot_use + ".e[" + lane + "]");
      } else {
        decl << indent << ptype(nd.dtype) << " bc" << i << slot_decl << ";\n";
        fetch << indent << "bc" << i << slot_use << " = " << ptr << "[" << ix << "];\n";
        override_[i] = from_storage(nd.dtype, "bc" + S((int64_t)i) + slot_use);
      }
    }
  }

  // ---- elementwise -----------------------------------------------------------------
  // An elementwise Kernel whose largest load walks memory along another digit of gidx than the
  // output does (a materialised transpose: `jit` emits them for the weight gradients that
  // `transposeDot` produces in [out, in] order and for the batch axis that `vmap` moves to the
  // front).  Read directly, a warp's 32 loads hit 32 different 128-byte lines.  Here a CTA takes
  // a 32 x 32 tile over the output's unit digit A and the load's unit digit B: the load is read
  // with B across the lanes into shared memory, then the Kernel's body runs with A across the lanes.
  bool elementwise_transposed(Plan& p) const {
    if (k.size < (1u << 18) || dtype_bytes(out_dt) != 4) return false;
    size_t best = 0;
    int64_t dB = 0, mB = 0, mA = 0;
    uint64_t best_len = 0;
    for (size_t i = 0; i < k.exp.size(); i++) {
      const Node& nd = k.exp[i];
      if (nd.op != JAXCUDA_OP_GLOBALINDEX || dtype_bytes(nd.dtype) != 4) continue;
      const std::optional<Affine>& ix = an_exp.affine[nd.src[0]];
      if (!ix || !in_range(ix, nd.arg1)) continue;
      const Term* ta = nullptr;
      const Term* tb = nullptr;
      for (const Term& t : ix->terms) {
        if (t.var != 0) continue;
        if (t.div == 1) ta = &t;
        else if (t.coef == 1) tb = &t;
      }
      if (!tb) continue;
      const int64_t a_mod = ta ? (ta->mod ? ta->mod : (int64_t)k.size) : 0;
      if (!ta || std::llabs(ta->coef) < 32 || a_mod < 16) continue;       // the output's unit digit must stride the load
      if (tb->div % a_mod) continue;
      const int64_t b_mod = tb->mod ? tb->mod : (int64_t)k.size / tb->div;
      if (b_mod < 16 || nd.arg1 < best_len) continue;
      best = i; best_len = nd.arg1; dB = tb->div; mB = b_mod; mA = a_mod;
    }
    if (!best_len || (int64_t)k.size % (dB * mB)) return false;
    // (a small strided array is staged as well: read directly, each of a warp's loads touches 32
    // lines whatever the array's size, and that is what bounds such a Kernel, not the bytes)
    const int64_t tilesA = (mA + 31) / 32, tilesB = (mB + 31) / 32, mids = dB / mA, his = (int64_t)k.size / (dB * mB);
    const int64_t blocks = tilesA * tilesB * mids * his;
    if (blocks > 0x7fffffffLL) return false;
    const Node& ld = k.exp[best];
    std::ostringstream os;
    os << header();
    os << "extern \"C\" __global__ void __launch_bounds__(256) jx_transpose(" << params() << ") {\n";
    os << "  __shared__ " << ctype(ld.dtype) << " tile[32][33];\n";
    os << "  const int tx = threadIdx.x & 31, ty = threadIdx.x >> 5;\n";
    os << "  long long blk = blockIdx.x;\n";
    os << "  const int ta = (int)(blk % " << tilesA << "LL); blk /= " << tilesA << "LL;\n";
    os << "  const int tb = (int)(blk % " << tilesB << "LL); blk /= " << tilesB << "LL;\n";
    os << "  const long long mid = blk % " << mids << "LL, hi = blk / " << mids << "LL;\n";
    os << "  const long long base = hi * " << dB * mB << "LL + mid * " << mA << "LL;\n";
    // phase 1: lanes along B
    os << "  {\n    const int b = tb * 32 + tx;\n    #pragma unroll\n    for (int i = ty; i < 32; i += 8) {\n";
    os << "      const int a = ta * 32 + i;\n      if (a < " << mA << " && b < " << mB << ") {\n";
    os << "        const int gidx = (int)(base + (long long)b * " << dB << "LL + a);\n";
    {
      std::vector<std::string> names(k.exp.size());
      Env env;
      env.prefix = "l";
      emit_nodes(os, k.exp, an_exp, names, closure(k.exp, best), env, "        ");
      os << "        tile[i][tx] = " << names[best] << ";\n";
    }
    os << "      }\n    }\n  }\n  __syncthreads();\n";
    // phase 2: lanes along A
    os << "  {\n    const int a = ta * 32 + tx;\n    #pragma unroll\n    for (int i = ty; i < 32; i += 8) {\n";
    os << "      const int b = tb * 32 + i;\n      if (a < " << mA << " && b < " << mB << ") {\n";
    os << "        const int gidx = (int)(base + (long long)b * " << dB << "LL + a);\n";
    {
      std::map<size_t, std::string> ov;
      ov[best] = "tile[tx][i]";
      // every node except the staged load's own index arithmetic (unless something else uses it)
      std::vector<char> want(k.exp.size(), 0);
      want.back() = 1;
      for (size_t i = k.exp.size(); i-- > 0;)
        if (want[i] && i != best) for (uint32_t sidx = 0; sidx < k.exp[i].nsrc; sidx++) want[k.exp[i].src[sidx]] = 1;
      std::vector<std::string> names(k.exp.size());
      Env env;
      env.load_override = &ov;
      emit_nodes(os, k.exp, an_exp, names, want, env, "        ");
      os << "        out[gidx] = " << to_storage(out_dt, names.back()) << ";\n";
    }
    os << "      }\n    }\n  }\n}\n";
    p.source = os.str();
    Stage st;
    st.entry = "jx_transpose";
    st.grid[0] = (unsigned)blocks;
    st.block[0] = 256;
    p.stages.push_back(st);
    p.describe = "elementwise transposed tile 32x32 A=" + S(mA) + " B=" + S(mB) + "@" + S(dB) + " grid=" + S(blocks);
    return true;
  }

  Plan elementwise() const {
    Plan p;
    p.skeleton = SK_ELEMENTWISE;
    account(p);
    if (opt.force_skeleton < 0 && elementwise_transposed(p)) return p;
    const int T = 256;
    int V = std::max(1, 16 / dtype_bytes(out_dt));
    if (k.size < (uint64_t)V * 64) V = 1;
    const int64_t nvec = (int64_t)(k.size / V);
    const int64_t tail = (int64_t)(k.size - nvec * V);
    int ILP = V > 1 ? std::max(1, opt.ew_ilp) : 1;
    while (ILP > 1 && nvec < (int64_t)T * ILP * opt.sm_count) ILP >>= 1;
    const bool exact = nvec % ((int64_t)T * ILP) == 0;
    std::vector<char> all(k.exp.size(), 1);
    const size_t root = k.exp.size() - 1;

    std::ostringstream os;
    os << header();
    os << "extern \"C\" __global__ void __launch_bounds__(" << T << ") jx_elementwise(" << params_rev() << ") {\n";
    p.takes_rev = true;
    os << rev_block();
    if (nvec > 0) {
      std::map<size_t, std::string> ov;
      std::ostringstream decl, fetch;
      std::vector<std::string> bnames(k.exp.size());
      Env env;
      if (V > 1)
        preload(decl, fetch, k.exp, an_exp, all, 0, V, env, "g0", "[" + S(ILP) + "]", "[j]", "u", ov, bnames, "        ");
      os << "  for (int base = jx_bx * " << T * ILP << "; base < " << nvec << "; base += gridDim.x * " << T * ILP << ") {\n";
      os << decl.str();
      os << "    #pragma unroll\n    for (int j = 0; j < " << ILP << "; j++) {\n";
      os << "      const int vi = base + j * " << T << " + threadIdx.x;\n";
      os << (exact ? "      {\n" : "      if (vi < " + S(nvec) + ") {\n");
      os << "        const int g0 = vi * " << V << ";\n";
      os << fetch.str();
      os << "      }\n    }\n";
      os << "    #pragma unroll\n    for (int j = 0; j < " << ILP << "; j++) {\n";
      os << "      const int vi = base + j * " << T << " + threadIdx.x;\n";
      os << (exact ? "      {\n" : "      if (vi < " + S(nvec) + ") {\n");
      os << "        const int g0 = vi * " << V << ";\n";
      os << "        jx_pack<" << ptype(out_dt) << ", " << V << "> res;\n";
      os << "        #pragma unroll\n        for (int u = 0; u < " << V << "; u++) {\n";
      os << "          const int gidx = g0 + u;\n";
      std::vector<std::string> names(k.exp.size());
      env.load_override = &ov;
      emit_nodes(os, k.exp, an_exp, names, all, env, "          ");
      os << "          res.e[u] = " << to_storage(out_dt, names[root]) << ";\n";
      os << "        }\n";
      os << "        jx_store(out + g0, res);\n";
      os << "      }\n    }\n  }\n";
    }
    if (tail > 0) {
      os << "  if (blockIdx.x == 0) {\n";
      os << "    for (int gidx = " << nvec * V << " + threadIdx.x; gidx < " << k.size << "; gidx += " << T << ") {\n";
      std::vector<std::string> names(k.exp.size());
      Env env;
      emit_nodes(os, k.exp, an_exp, names, all, env, "      ");
      os << "      out[gidx] = " << to_storage(out_dt, names[root]) << ";\n";
      os << "    }\n  }\n";
    }
    os << "}\n";
    p.source = os.str();
    Stage st;
    st.entry = "jx_elementwise";
    int64_t blocks = nvec > 0 ? (nvec + (int64_t)T * ILP - 1) / ((int64_t)T * ILP) : 1;
    blocks = std::min<int64_t>(blocks, (int64_t)opt.sm_count * opt.ew_blocks_per_sm);
    st.grid[0] = (unsigned)std::max<int64_t>(1, blocks);
    st.block[0] = T;
    p.stages.push_back(st);
    p.describe = "elementwise V=" + S(V) + " ILP=" + S(ILP) + " grid=" + S(st.grid[0]) + "x" + S(T);
    return p;
  }

  // ---- reductions --------------------------------------------------------------------
  void emit_epilogue_store(std::ostream& os, const std::string& indent, const std::string& dst) const {
    std::vector<std::string> names(k.epi.size());
    std::vector<char> all(k.epi.size(), 1);
    Env env;
    env.prefix = "e";
    emit_nodes(os, k.epi, an_epi, names, all, env, indent);
    os << indent << dst << " = " << to_storage(out_dt, names.back()) << ";\n";
  }

  // The whole Kernel as a loop nest of one CTA of `threads` threads (a stage of a small batch): expects
  // the arguments as p0 .. and `out` in scope.
  void emit_serial(std::ostream& os, int threads, const std::string& indent) const {
    std::vector<char> all(k.exp.size(), 1);
    std::vector<std::string> names(k.exp.size());
    Env env;
    os << indent << "for (int gidx = threadIdx.x; gidx < " << k.size << "; gidx += " << threads << ") {\n";
    if (!k.has_red) {
      emit_nodes(os, k.exp, an_exp, names, all, env, indent + "  ");
      os << indent << "  out[gidx] = " << to_storage(out_dt, names.back()) << ";\n";
    } else {
      const char* AT = ctype(k.red_dtype);
      os << indent << "  " << AT << " acc = " << identity_literal(k.red_op, k.red_dtype) << ";\n";
      os << indent << "  for (int ridx = 0; ridx < " << k.red_size << "; ridx++) {\n";
      emit_nodes(os, k.exp, an_exp, names, all, env, indent + "    ");
      os << indent << "    acc = " << red("acc", names.back()) << ";\n" << indent << "  }\n";
      emit_epilogue(os, indent + "  ", "acc", "out[gidx]");
    }
    os << indent << "}\n";
  }

  // The Kernel's epilogue for one output: expects `gidx` and the accumulator `acc_name` in scope.
  void emit_epilogue(std::ostream& os, const std::string& indent, const std::string& acc_name, const std::string& dst) const {
    std::vector<std::string> en(k.epi.size());
    std::vector<char> eall(k.epi.size(), 1);
    Env ee;
    ee.prefix = "e";
    ee.acc = acc_name;
    emit_nodes(os, k.epi, an_epi, en, eall, ee, indent);
    os << indent << dst << " = " << to_storage(out_dt, en.back()) << ";\n";
  }

  void emit_finish_kernel(std::ostream& os, int splits) const {
    const char* AT = ctype(k.red_dtype);
    os << "extern \"C\" __global__ void __launch_bounds__(256) jx_finish(" << params() << ") {\n";
    os << "  const int gidx = blockIdx.x * 256 + threadIdx.x;\n  if (gidx >= " << k.size << ") return;\n";
    os << "  const " << AT << "* part = (const " << AT << "*)scratch;\n";
    os << "  " << AT << " acc = " << identity_literal(k.red_op, k.red_dtype) << ";\n";
    os << "  for (int s = 0; s < " << splits << "; s++) { const " << AT << " v = part[(size_t)s * " << k.size
       << " + gidx]; acc = " << red("acc", "v") << "; }\n";
    emit_epilogue_store(os, "  ", "out[gidx]");
    os << "}\n";
  }

  bool has_load(int var_contig) const {  // some in-range load whose index moves by 1 with var (div 1)
    for (size_t i = 0; i < k.exp.size(); i++) {
      const Node& nd = k.exp[i];
      if (nd.op != JAXCUDA_OP_GLOBALINDEX || !an_exp.dep_r[i]) continue;  // loads hoisted out of the loop do not count
      const auto& ix = an_exp.affine[nd.src[0]];
      if (ix && ix->coef_of(var_contig, 1) == 1) return true;
    }
    return false;
  }

  int min_load_bytes(int var, int Vmax) const {  // narrowest element among loads that vectorise over var
    int b = 0;
    for (size_t i = 0; i < k.exp.size(); i++) {
      const Node& nd = k.exp[i];
      if (nd.op != JAXCUDA_OP_GLOBALINDEX) continue;
      if (classify_load(nd, an_exp.affine[nd.src[0]], var, Vmax) == LK_VECTOR)
        b = b ? std::min(b, dtype_bytes(nd.dtype)) : dtype_bytes(nd.dtype);
    }
    return b;
  }

  Plan reduce_row() const {
    Plan p;
    p.skeleton = SK_REDUCE_ROW;
    account(p);
    const int64_t K = k.red_size;
    const int T = 256;
    // A body with transcendentals does more work per load: half-size row groups keep more rows
    // (and their loads) in flight per SM while the special-function unit is busy.
    bool heavy = false;
    for (const Node& nd : k.exp) heavy = heavy || (nd.op >= JAXCUDA_OP_SIN && nd.op <= JAXCUDA_OP_ERFC);
    // vector width over ridx
    int V = 1;
    for (int cand : {8, 4, 2}) {
      if (K % cand) continue;
      int eb = min_load_bytes(1, cand);
      if (eb && eb * cand <= 16) { V = cand; break; }
    }
    // Rows of at least 1024 elements: 256 threads per row once every thread still has four 128-bit
    // loads of its own, else 128 (f16 matvec over 4096 columns: 0.81 of the copy rate against 0.75).
    int TPR = K >= 1024 ? (heavy || K < 256 * 4 * V ? 128 : 256) : K >= 128 ? 32 : 8;
    if (opt.row_tpr == 8 || opt.row_tpr == 32 || opt.row_tpr == 64 || opt.row_tpr == 128 || opt.row_tpr == 256)
      TPR = opt.row_tpr;
    const int RPC = T / TPR;
    int64_t row_blocks = ((int64_t)k.size + RPC - 1) / RPC;
    // few outputs and a long axis: split ridx across CTAs, finish in a second pass
    int splits = 1;
    if (row_blocks < opt.sm_count && K >= 16384) {
      int64_t want = (2 * opt.sm_count + row_blocks - 1) / row_blocks;
      int64_t max_splits = K / ((int64_t)TPR * V * 4);
      splits = (int)std::max<int64_t>(1, std::min(want, max_splits));
    }
    int64_t rchunk = (K + splits - 1) / splits;
    rchunk = (rchunk + V - 1) / V * V;
    splits = (int)((K + rchunk - 1) / rchunk);
    const char* AT = ctype(k.red_dtype);
    const size_t root = k.exp.size() - 1;

    std::vector<char> hoist(k.exp.size(), 0), inner(k.exp.size(), 0);
    for (size_t i = 0; i < k.exp.size(); i++) (an_exp.dep_r[i] ? inner : hoist)[i] = 1;

    std::ostringstream os;
    os << header();
    os << "extern \"C\" __global__ void __launch_bounds__(" << T << ") jx_reduce_row(" << params_rev() << ") {\n";
    p.takes_rev = true;
    os << rev_block();
    os << "  const int lane = threadIdx.x % " << TPR << ", rowc = threadIdx.x / " << TPR << ";\n";
    os << "  const long long gl = (long long)jx_bx * " << RPC << " + rowc;\n";
    os << "  const bool active = gl < " << k.size << "LL;\n";
    os << "  const int gidx = active ? (int)gl : 0;\n";
    if (splits > 1) {
      os << "  const int rbeg = blockIdx.y * " << rchunk << ";\n";
      os << "  const int rend = min(" << K << ", rbeg + " << rchunk << ");\n";
    } else {
      os << "  const int rbeg = 0, rend = " << K << ";\n";
    }
    std::vector<std::string> names(k.exp.size());
    Env env;
    emit_nodes(os, k.exp, an_exp, names, hoist, env, "  ");
    os << "  " << AT << " acc = " << identity_literal(k.red_op, k.red_dtype) << ";\n";
    std::map<size_t, std::string> ov;
    std::ostringstream decl, fetch;
    std::vector<std::string> bnames = names;  // hoisted values stay visible to the index closures
    if (V > 1) preload(decl, fetch, k.exp, an_exp, inner, 1, V, env, "r0", "", "", "u", ov, bnames, "    ");
    const int64_t iters = std::max<int64_t>(1, (rchunk + (int64_t)TPR * V - 1) / ((int64_t)TPR * V));
    os << "  #pragma unroll " << (opt.row_unroll > 0 ? opt.row_unroll : (int)std::min<int64_t>(iters, 4)) << "\n";
    os << "  for (int r0 = rbeg + lane * " << V << "; r0 < rend; r0 += " << TPR * V << ") {\n";
    os << decl.str() << fetch.str();
    os << "    #pragma unroll\n    for (int u = 0; u < " << V << "; u++) {\n";
    os << "      const int ridx = r0 + u;\n";
    env.load_override = &ov;
    std::vector<std::string> inames = names;
    emit_nodes(os, k.exp, an_exp, inames, inner, env, "      ");
    os << "      acc = " << red("acc", inames[root]) << ";\n";
    os << "    }\n  }\n";
    const int W = std::min(TPR, 32);
    os << "  #pragma unroll\n  for (int o = " << W / 2 << "; o > 0; o >>= 1) { const " << AT
       << " v = jx_shfl_down(acc, o, " << W << "); acc = " << red("acc", "v") << "; }\n";
    if (TPR > 32) {
      // one partial per warp; the first warp of each row folds its row's TPR/32 partials
      const int WPR = TPR / 32;
      os << "  __shared__ " << AT << " sm[" << T / 32 << "];\n";
      os << "  if ((threadIdx.x & 31) == 0) sm[threadIdx.x >> 5] = acc;\n  __syncthreads();\n";
      os << "  if (lane < 32) {\n";
      os << "    acc = lane < " << WPR << " ? sm[rowc * " << WPR << " + lane] : " << identity_literal(k.red_op, k.red_dtype) << ";\n";
      os << "    #pragma unroll\n    for (int o = " << WPR / 2 << "; o > 0; o >>= 1) { const " << AT
         << " v = jx_shfl_down(acc, o, 32); acc = " << red("acc", "v") << "; }\n  }\n";
    }
    os << "  if (lane == 0 && active) {\n";
    if (splits > 1) {
      os << "    ((" << AT << "*)scratch)[(size_t)blockIdx.y * " << k.size << " + gidx] = acc;\n";
    } else {
      emit_epilogue_store(os, "    ", "out[gidx]");
    }
    os << "  }\n}\n";
    if (splits > 1) emit_finish_kernel(os, splits);
    p.source = os.str();
    Stage st;
    st.entry = "jx_reduce_row";
    st.grid[0] = (unsigned)row_blocks;
    st.grid[1] = (unsigned)splits;
    st.block[0] = T;
    p.stages.push_back(st);
    if (splits > 1) {
      Stage fin;
      fin.entry = "jx_finish";
      fin.grid[0] = (unsigned)((k.size + 255) / 256);
      fin.block[0] = 256;
      p.stages.push_back(fin);
      p.scratch_bytes = (size_t)splits * k.size * dtype_bytes(k.red_dtype == JAXCUDA_F16 ? JAXCUDA_F32 : k.red_dtype);
    }
    p.describe = "reduce-row TPR=" + S(TPR) + " V=" + S(V) + " splits=" + S(splits) + " grid=" + S(row_blocks);
    return p;
  }

  // One thread per vector of V adjacent outputs walks ridx; TY such threads share a vector and
  // take interleaved ridx values (folded through shared memory in a fixed order), and `splits`
  // CTAs along grid.y take contiguous ridx chunks whose partials a second kernel folds.
  // group > 0: every thread owns `group` adjacent outputs (a run of gidx that shares its other
  // operand, e.g. the N = 10 columns of one row of a skinny dot) instead of a 128-bit vector.
  Plan reduce_col(int group = 0) const {
    Plan p;
    p.skeleton = SK_REDUCE_COL;
    account(p);
    const int64_t K = k.red_size;
    int V = 1;
    for (int cand : {8, 4, 2}) {
      if (k.size % cand) continue;
      int eb = min_load_bytes(0, cand);
      if (eb && eb * cand <= 16 && (int64_t)k.size / cand >= 256) { V = cand; break; }
    }
    const bool grouped = group > 1 && k.size % group == 0;
    if (grouped) V = group;
    const int64_t nvec = ((int64_t)k.size + V - 1) / V;
    // r-parallelism wanted so that the grid fills the machine: col_ctas_per_sm CTAs of 256 threads per SM
    const int64_t target_threads = (int64_t)opt.sm_count * opt.col_ctas_per_sm * 256;
    int64_t par = std::max<int64_t>(1, std::min<int64_t>((target_threads + nvec - 1) / nvec, K / 8));
    int TY = 1;
    while (TY < 8 && TY < par) TY <<= 1;
    if (opt.col_ty > 0) TY = opt.col_ty;
    const int T = TY == 1 ? std::max(32, opt.col_threads) : 256;
    const int TX = T / TY;
    const int64_t gblocks = (nvec + TX - 1) / TX;
    int splits = (int)std::max<int64_t>(1, (par + TY - 1) / TY);
    int64_t rchunk = (K + splits - 1) / splits;
    rchunk = (rchunk + TY - 1) / TY * TY;
    splits = (int)((K + rchunk - 1) / std::max<int64_t>(1, rchunk));
    if (K == 0) { splits = 1; rchunk = 0; }
    if (splits > 1) {
      // All CTAs of such a grid are resident at once, so the kernel lasts as long as the SM with the
      // most CTAs: 602 CTAs on 148 SMs leave some SMs five chunks and most of them four.  Among the
      // split counts near the wanted one take that with the smallest (CTAs on the fullest SM) x
      // (rows per chunk), at most six CTAs per SM.
      int64_t best_cost = 0;
      int best_s = splits;
      for (int s = std::max(2, splits * 2 / 3); s <= splits * 3 / 2 + 1; s++) {
        int64_t rc = ((K + s - 1) / s + TY - 1) / TY * TY;
        int64_t se = (K + rc - 1) / rc;
        int64_t per_sm = (gblocks * se + opt.sm_count - 1) / opt.sm_count;
        if (per_sm > 6 || rc < (int64_t)TY * opt.col_unroll) continue;
        int64_t cost = per_sm * rc;
        if (!best_cost || cost < best_cost || (cost == best_cost && std::abs(s - splits) < std::abs(best_s - splits))) {
          best_cost = cost;
          best_s = s;
        }
      }
      if (best_cost) {
        rchunk = ((K + best_s - 1) / best_s + TY - 1) / TY * TY;
        splits = (int)((K + rchunk - 1) / rchunk);
      }
    }
    const char* AT = ctype(k.red_dtype);
    const size_t root = k.exp.size() - 1;
    std::vector<char> all(k.exp.size(), 1);

    std::ostringstream os;
    os << header(1);  // streamed once, column by column: the no-allocate hint measured 3 % faster here, slower in the row skeleton
    os << "extern \"C\" __global__ void __launch_bounds__(" << T << ") jx_reduce_col(" << params() << ") {\n";
    os << "  const int tx = threadIdx.x % " << TX << ", ty = threadIdx.x / " << TX << ";\n";
    os << "  const int gv = blockIdx.x * " << TX << " + tx;\n  const bool active = gv < " << nvec << ";\n";
    os << "  const int g0 = active ? gv * " << V << " : 0;\n";
    if (splits > 1) {
      os << "  const int rbeg = blockIdx.y * " << rchunk << ";\n  const int rend = min(" << K << ", rbeg + " << rchunk << ");\n";
    } else {
      os << "  const int rbeg = 0, rend = " << K << ";\n";
    }
    os << "  " << AT << " acc[" << V << "];\n  #pragma unroll\n  for (int u = 0; u < " << V << "; u++) acc[u] = "
       << identity_literal(k.red_op, k.red_dtype) << ";\n";
    std::map<size_t, std::string> ov;
    std::ostringstream decl, fetch;
    std::vector<std::string> bnames(k.exp.size());
    Env env;
    // The ridx loop runs in batches of U steps: first every 128-bit load of the batch is issued,
    // then the batch is consumed, so that U loads per thread are in flight whatever the compiler
    // makes of the accumulator dependences.
    const int U = (V > 1 && !grouped) ? std::max(1, opt.col_unroll) : 1;
    if (V > 1 && !grouped) preload(decl, fetch, k.exp, an_exp, all, 0, V, env, "g0", "[" + S(U) + "]", "[j]", "u", ov, bnames, "        ");
    if (U > 1) {
      os << "  for (int rb = rbeg + ty; rb < rend; rb += " << TY * U << ") {\n";
      os << decl.str();
      os << "    #pragma unroll\n    for (int j = 0; j < " << U << "; j++) {\n      const int ridx = rb + j * " << TY << ";\n";
      os << "      if (ridx < rend) {\n" << fetch.str() << "      }\n    }\n";
      os << "    #pragma unroll\n    for (int j = 0; j < " << U << "; j++) {\n      const int ridx = rb + j * " << TY << ";\n";
      os << "      if (ridx < rend) {\n";
      os << "        #pragma unroll\n        for (int u = 0; u < " << V << "; u++) {\n          const int gidx = g0 + u;\n";
      env.load_override = &ov;
      std::vector<std::string> names(k.exp.size());
      emit_nodes(os, k.exp, an_exp, names, all, env, "          ");
      os << "          acc[u] = " << red("acc[u]", names[root]) << ";\n        }\n      }\n    }\n  }\n";
    } else {
      os << "  #pragma unroll 4\n  for (int ridx = rbeg + ty; ridx < rend; ridx += " << TY << ") {\n";
      os << "    #pragma unroll\n    for (int u = 0; u < " << V << "; u++) {\n      const int gidx = g0 + u;\n";
      std::vector<std::string> names(k.exp.size());
      emit_nodes(os, k.exp, an_exp, names, all, env, "      ");
      os << "      acc[u] = " << red("acc[u]", names[root]) << ";\n    }\n  }\n";
    }
    if (TY > 1) {
      os << "  __shared__ " << AT << " sm[" << TY * V * TX << "];\n";
      os << "  #pragma unroll\n  for (int u = 0; u < " << V << "; u++) sm[(ty * " << V << " + u) * " << TX << " + tx] = acc[u];\n";
      os << "  __syncthreads();\n";
      os << "  if (ty == 0) {\n    #pragma unroll\n    for (int u = 0; u < " << V << "; u++)\n      for (int y = 1; y < " << TY
         << "; y++) { const " << AT << " v = sm[(y * " << V << " + u) * " << TX << " + tx]; acc[u] = " << red("acc[u]", "v") << "; }\n  }\n";
    }
    const int64_t counter_bytes = 1024 + gblocks * 4;  // per-column-block arrival counters ahead of the partials
    const int64_t counter_pad = (counter_bytes + 255) / 256 * 256;
    if (splits > 1) {
      // Every CTA stores its partial; the CTA that arrives last at its column block's counter folds
      // all partials in split order (so the result does not depend on arrival order), applies the
      // epilogue and re-arms the counter.  The counters live at the head of a scratch area that is
      // zeroed once when the executable is prepared.
      os << "  " << AT << "* parts = (" << AT << "*)((char*)scratch + " << counter_pad << ");\n";
      os << "  if (ty == 0 && active) {\n    " << AT << "* part = parts + (size_t)blockIdx.y * " << k.size << " + g0;\n";
      os << "    #pragma unroll\n    for (int u = 0; u < " << V << "; u++) part[u] = acc[u];\n  }\n";
      emit_split_tail(os, splits, (int64_t)TX * V, T);
    } else {
      os << "  if (ty != 0 || !active) return;\n";
      os << "  #pragma unroll\n  for (int u = 0; u < " << V << "; u++) {\n    const int gidx = g0 + u;\n    const " << AT << " acc_u = acc[u];\n";
      emit_epilogue(os, "    ", "acc_u", "out[gidx]");
      os << "  }\n";
    }
    os << "}\n";
    p.source = os.str();
    Stage st;
    st.entry = "jx_reduce_col";
    st.grid[0] = (unsigned)std::max<int64_t>(1, gblocks);
    st.grid[1] = (unsigned)splits;
    st.block[0] = T;
    p.stages.push_back(st);
    if (splits > 1) {
      p.scratch_bytes = (size_t)counter_pad + (size_t)splits * k.size * (k.red_dtype == JAXCUDA_F64 ? 8 : 4);
      p.scratch_persistent = true;
    }
    p.describe = "reduce-col V=" + S(V) + " TY=" + S(TY) + " splits=" + S(splits) + " grid=" + S(gblocks) + "x" + S(T);
    return p;
  }

  // ---- GEMM recognition ----------------------------------------------------------------
  // Body = [Cast<f32>] Mul(load, load) under an f32 Add reduction, both indices affine with
  // ridx plain: the form `jitRules[Dot]` builds (src/frontend/jit.ts:639-648).
  GemmDesc match_gemm() const {
    GemmDesc g;
    if (!k.has_red || k.red_op != JAXCUDA_OP_ADD || k.red_dtype != JAXCUDA_F32 || k.red_size < 1) return g;
    size_t r = k.exp.size() - 1;
    const Node* mul = &k.exp[r];
    if (mul->op == JAXCUDA_OP_CAST && mul->dtype == JAXCUDA_F32 && k.exp[mul->src[0]].dtype == JAXCUDA_F16) {
      mul = &k.exp[mul->src[0]];
      g.round_product_f16 = true;
    }
    if (mul->op != JAXCUDA_OP_MUL) return g;
    auto operand = [&](uint32_t idx) -> const Node* {
      const Node* nd = &k.exp[idx];
      if (nd->op == JAXCUDA_OP_CAST && nd->dtype == JAXCUDA_F32) nd = &k.exp[nd->src[0]];
      if (nd->op != JAXCUDA_OP_GLOBALINDEX) return nullptr;
      if (nd->dtype != JAXCUDA_F32 && nd->dtype != JAXCUDA_F16) return nullptr;
      return nd;
    };
    const Node* L[2] = {operand(mul->src[0]), operand(mul->src[1])};
    if (!L[0] || !L[1]) return g;
    const std::optional<Affine>* ix[2] = {&an_exp.affine[L[0]->src[0]], &an_exp.affine[L[1]->src[0]]};
    for (int s = 0; s < 2; s++) {
      if (!*ix[s] || !in_range(*ix[s], L[s]->arg1)) return g;
      if (!(*ix[s])->only_plain(1) || (*ix[s])->coef_of(1, 1) == 0) return g;
    }
    for (int swap = 0; swap < 2; swap++) {
      const Affine& A = **ix[swap];
      const Affine& Bx = **ix[1 - swap];
      // N: modulus of B's unit digit of gidx
      int64_t N = 0, sBn = 0;
      for (const Term& t : Bx.terms) if (t.var == 0 && t.div == 1) { N = t.mod; sBn = t.coef; }
      if (N <= 1 || (int64_t)k.size % N) continue;
      int64_t M = 0, sAm = 0;
      for (const Term& t : A.terms) if (t.var == 0 && t.div == N) { M = t.mod ? t.mod : (int64_t)k.size / N; sAm = t.coef; }
      if (M <= 0 || ((int64_t)k.size / N) % M) continue;
      const int64_t batch = (int64_t)k.size / (M * N);
      bool ok = true;
      int64_t sAb = 0, sBb = 0;
      for (const Term& t : A.terms) {
        if (t.var != 0) continue;
        if (t.div == N && (t.mod == 0 || t.mod == M)) continue;
        if (t.div == M * N && t.mod == 0 && batch > 1) { sAb = t.coef; continue; }
        ok = false;
      }
      for (const Term& t : Bx.terms) {
        if (t.var != 0) continue;
        if (t.div == 1 && t.mod == N) continue;
        if (t.div == M * N && t.mod == 0 && batch > 1) { sBb = t.coef; continue; }
        ok = false;
      }
      if (!ok) continue;
      g.valid = true;
      g.gidA = (uint32_t)L[swap]->arg0; g.gidB = (uint32_t)L[1 - swap]->arg0;
      g.dtA = L[swap]->dtype; g.dtB = L[1 - swap]->dtype;
      g.lenA = L[swap]->arg1; g.lenB = L[1 - swap]->arg1;
      g.M = M; g.N = N; g.K = k.red_size; g.batch = batch;
      g.offA = A.c0; g.sAm = sAm; g.sAk = A.coef_of(1, 1); g.sAb = sAb;
      g.offB = Bx.c0; g.sBn = sBn; g.sBk = Bx.coef_of(1, 1); g.sBb = sBb;
      return g;
    }
    return g;
  }

  // ---- convolution recognition ------------------------------------------------------------
  // `jitRules[Conv]` (src/frontend/jit.ts:649-660) builds a convolution as a Dot over pooled views:
  // body = Mul(patch, weight) under an f32 Add reduction, where the weight is a plain load indexed by
  // one digit of gidx (the output channel) and ridx, and the patch is any expression (guarded,
  // div/mod-indexed loads of the input, src/frontend/convolution.ts) of the other digits of gidx
  // and ridx.  With gidx = (b * M + m) * N + n, m the weight's digit, this is, per b,
  // C[m, n] = sum_k W[m, k] * P[k, n]: a GEMM whose B operand is gathered by evaluating the patch.
  // Returns the GEMM description (b_gathered) and the node of the patch.
  GemmDesc match_conv(size_t& patch_node) const {
    GemmDesc g;
    if (!k.has_red || k.red_op != JAXCUDA_OP_ADD || k.red_dtype != JAXCUDA_F32 || k.red_size < 1) return g;
    const Node* mul = &k.exp.back();
    if (mul->op == JAXCUDA_OP_CAST && mul->dtype == JAXCUDA_F32 && k.exp[mul->src[0]].dtype == JAXCUDA_F16) {
      mul = &k.exp[mul->src[0]];
      g.round_product_f16 = true;
    }
    if (mul->op != JAXCUDA_OP_MUL) return g;
    for (int wside = 0; wside < 2; wside++) {
      const Node* w = &k.exp[mul->src[wside]];
      if (w->op == JAXCUDA_OP_CAST && w->dtype == JAXCUDA_F32) w = &k.exp[w->src[0]];
      if (w->op != JAXCUDA_OP_GLOBALINDEX || (w->dtype != JAXCUDA_F32 && w->dtype != JAXCUDA_F16)) continue;
      const std::optional<Affine>& wi = an_exp.affine[w->src[0]];
      if (!wi || !in_range(wi, w->arg1) || !wi->only_plain(1) || wi->coef_of(1, 1) == 0) continue;
      // exactly one digit of gidx
      const Term* digit = nullptr;
      int gterms = 0;
      for (const Term& t : wi->terms) if (t.var == 0) { digit = &t; gterms++; }
      if (gterms != 1 || digit->div < 2) continue;
      const int64_t N = digit->div;
      if ((int64_t)k.size % N) continue;
      const int64_t M = digit->mod ? digit->mod : (int64_t)k.size / N;
      if (M < 1 || ((int64_t)k.size / N) % M) continue;
      const int64_t batch = (int64_t)k.size / (M * N);
      // The patch must not look at the weight's digit.  An index expression in affine form is judged
      // by its digits of gidx (only digits under the channel digit or the batch digits above it);
      // any other node is clean when all its sources are.  Wide forms such as gidx itself may only
      // feed further index arithmetic.
      const size_t proot = mul->src[1 - wside];
      const std::vector<char> in_patch = closure(k.exp, proot);
      std::vector<char> wide(k.exp.size(), 0);
      bool ok = true;
      for (size_t i = 0; i <= proot && ok; i++) {
        if (!in_patch[i]) continue;
        const Node& nd = k.exp[i];
        if (an_exp.affine[i]) {
          for (const Term& t : an_exp.affine[i]->terms) {
            if (t.var != 0) continue;
            const bool below = t.mod != 0 && t.div * t.mod <= N;
            const bool above = t.div >= M * N;
            if (!below && !above) wide[i] = 1;
          }
        } else if (nd.op == JAXCUDA_OP_SPECIAL) {
          wide[i] = nd.arg0 == 0;
        } else {
          for (uint32_t sidx = 0; sidx < nd.nsrc; sidx++)
            if (wide[nd.src[sidx]]) ok = false;
        }
      }
      if (wide[proot]) ok = false;
      if (!ok) continue;
      const int eb = dtype_bytes(w->dtype);
      g.valid = true;
      g.b_gathered = true;
      g.b_pitch = (N + 63) / 64 * 64;
      g.gidA = (uint32_t)w->arg0; g.gidB = 0;
      g.dtA = w->dtype; g.dtB = w->dtype;
      g.lenA = w->arg1;
      g.M = M; g.N = N; g.K = k.red_size; g.batch = batch;
      g.offA = wi->c0; g.sAm = digit->coef; g.sAk = wi->coef_of(1, 1); g.sAb = 0;
      g.offB = 0; g.sBn = 1; g.sBk = g.b_pitch; g.sBb = g.K * g.b_pitch;
      g.lenB = (uint64_t)(batch * g.K * g.b_pitch);
      (void)eb;
      patch_node = proot;
      if (k.exp[proot].dtype != w->dtype && !(k.exp[proot].dtype == JAXCUDA_F32 && w->dtype == JAXCUDA_F32)) { g.valid = false; continue; }
      return g;
    }
    return g;
  }

  // ---- evaluating a convolution's patch expression for a run of consecutive pixels ------------------
  // Both gather variants give a thread `per` consecutive n (gidx0 .. gidx0 + per - 1) and many k.  The
  // nodes of the patch are emitted in three groups: what depends on gidx alone (once per thread),
  // what depends on ridx alone (once per k) and the mixed rest (per element).  When N is a multiple
  // of `per` a run never leaves its row of pixels, and most of the mixed part is the same for the
  // whole run or moves by a constant per pixel: a digit (gidx / d) % m with d a multiple of `per` is
  // constant over the run, the lowest digit gidx % m (m a multiple of `per`) grows by one, and any
  // node all of whose sources are constant over the run is constant too.  Those nodes are computed
  // for the first pixel only (for a 3 x 3 window over [N, C, H, W]: the row test of the window, the
  // row part of the address; per pixel remain the column test, one add for the address, the load).
  struct PatchRun {
    const Builder& bd;
    size_t root;
    int per;
    bool aligned;
    std::vector<char> patch, only_g, not_g, uniform, sloped;
    std::vector<int64_t> slope;
    std::vector<std::vector<std::string>> names;

    PatchRun(const Builder& b, size_t patch_node, int per_, bool aligned_)
        : bd(b), root(patch_node), per(per_), aligned(aligned_), patch(closure(b.k.exp, patch_node)) {
      const auto& exp = bd.k.exp;
      const size_t n = exp.size();
      only_g.assign(n, 0); not_g.assign(n, 0); uniform.assign(n, 0); sloped.assign(n, 0); slope.assign(n, 0);
      names.assign(per, std::vector<std::string>(n));
      for (size_t i = 0; i < n; i++) {
        if (!patch[i]) continue;
        const Node& nd = exp[i];
        only_g[i] = !bd.an_exp.dep_r[i];
        not_g[i] = !bd.an_exp.dep_g[i];
        if (!aligned) continue;
        if (!bd.an_exp.dep_g[i]) { uniform[i] = 1; continue; }
        if (nd.op == JAXCUDA_OP_SPECIAL) { sloped[i] = 1; slope[i] = 1; continue; }   // gidx itself
        if (bd.an_exp.affine[i] && nd.dtype == JAXCUDA_I32) {
          bool ok = true;
          int64_t sl = 0;
          for (const Term& t : bd.an_exp.affine[i]->terms) {
            if (t.var != 0 || t.div % per == 0) continue;
            if (t.div == 1 && (t.mod == 0 || t.mod % per == 0)) sl += t.coef;
            else ok = false;
          }
          if (ok) {
            if (sl == 0) uniform[i] = 1; else { sloped[i] = 1; slope[i] = sl; }
            continue;
          }
        }
        bool all = nd.nsrc > 0;
        for (uint32_t sidx = 0; sidx < nd.nsrc; sidx++) all = all && uniform[nd.src[sidx]];
        uniform[i] = all;
      }
    }
    // pixels after the first take over what the first one computed
    void share(int j, const std::vector<char>& mask) {
      if (j == 0 || !aligned) return;
      for (size_t i = 0; i < names[j].size(); i++) {
        if (!mask[i] || !names[j][i].empty() || names[0][i].empty()) continue;
        if (uniform[i]) names[j][i] = names[0][i];
        else if (sloped[i]) names[j][i] = "(" + names[0][i] + " + " + S((int64_t)j * slope[i]) + ")";
      }
    }
    // once per thread; expects `gidx0 .. gidx<per-1>` in scope
    void hoisted(std::ostream& os, const std::string& indent) {
      for (int j = 0; j < per; j++) {
        Env env;
        env.prefix = "h" + S(j) + "_";
        env.gidx = "gidx" + S(j);
        share(j, only_g);
        emit_nodes(os, bd.k.exp, bd.an_exp, names[j], only_g, env, indent);
      }
    }
    // once per k; expects `ridx` in scope and returns the value expressions of the run
    std::vector<std::string> row(std::ostream& os, const std::string& indent) {
      std::vector<std::vector<std::string>> local = names;   // names of this k only
      {
        std::vector<std::string> shared(bd.k.exp.size());
        Env env;
        env.prefix = "r";
        emit_nodes(os, bd.k.exp, bd.an_exp, shared, not_g, env, indent);
        for (int j = 0; j < per; j++)
          for (size_t i = 0; i < shared.size(); i++)
            if (local[j][i].empty() && !shared[i].empty()) local[j][i] = shared[i];
      }
      std::vector<std::string> out;
      names.swap(local);
      for (int j = 0; j < per; j++) {
        Env env;
        env.prefix = "q" + S(j) + "_";
        env.gidx = "gidx" + S(j);
        share(j, patch);
        emit_nodes(os, bd.k.exp, bd.an_exp, names[j], patch, env, indent);
        out.push_back(names[j][root]);
      }
      names.swap(local);
      return out;
    }
  };

  // CUDA C of the stage that evaluates a convolution's patch expression into the B operand
  // [batch][K][pitch] (n contiguous, zero beyond N) at the start of the scratch, followed for f32 by
  // the 3xTF32 remainder plane.  A thread owns four consecutive n of one batch entry and walks a
  // chunk of k (grid.y).
  static constexpr int kGatherKChunk = 32;
  std::string gather_source(const GemmDesc& g, size_t patch_node) const {
    const bool f16 = g.dtB == JAXCUDA_F16;
    const bool aligned = g.N % 4 == 0;
    PatchRun run(*this, patch_node, 4, aligned);
    std::ostringstream os;
    os << "extern \"C\" __global__ void __launch_bounds__(256) jx_gather_b(" << params() << ") {\n";
    os << "  const i64 quads = " << g.b_pitch / 4 << "LL, total = quads * " << g.batch << "LL;\n";
    os << "  const i64 t = (i64)blockIdx.x * 256 + threadIdx.x;\n  if (t >= total) return;\n";
    os << "  const int n0 = (int)(t % quads) * 4, b = (int)(t / quads);\n";
    os << "  const int k0 = blockIdx.y * " << kGatherKChunk << ", k1 = min(" << g.K << ", k0 + " << kGatherKChunk << ");\n";
    os << "  const bool n_in = n0 < " << g.N << ";   // the padding between N and the pitch is written as zeros\n";
    for (int j = 0; j < 4; j++) {
      if (aligned) os << "  const int gidx" << j << " = b * " << g.M * g.N << " + (n_in ? n0 : 0) + " << j << ";\n";
      else os << "  const int gidx" << j << " = b * " << g.M * g.N << " + min(n0 + " << j << ", " << g.N - 1 << ");\n";
    }
    run.hoisted(os, "  ");
    os << "  #pragma unroll 2\n  for (int ridx = k0; ridx < k1; ridx++) {\n";
    const std::vector<std::string> val = run.row(os, "    ");
    os << "    float v[4];\n";
    for (int j = 0; j < 4; j++)
      os << "    v[" << j << "] = n0 + " << j << " < " << g.N << " ? (float)" << val[j] << " : 0.0f;\n";
    os << "    const i64 row = (i64)b * " << g.K << "LL + ridx;\n";
    if (f16) {
      os << "    jx_pack<jx_half, 4> h;\n    #pragma unroll\n    for (int j = 0; j < 4; j++) h.e[j] = jx_f2h(v[j]);\n";
      os << "    jx_store((jx_half*)scratch + row * " << g.b_pitch << "LL + n0, h);\n";
    } else {
      os << "    jx_pack<float, 4> hi, lo;\n    #pragma unroll\n    for (int j = 0; j < 4; j++) {\n";
      os << "      hi.e[j] = v[j];\n      lo.e[j] = v[j] - __uint_as_float(__float_as_uint(v[j]) & 0xffffe000u);\n    }\n";
      os << "    jx_store((float*)scratch + row * " << g.b_pitch << "LL + n0, hi);\n";
      os << "    jx_store((float*)scratch + LEN_B_PAD + row * " << g.b_pitch << "LL + n0, lo);\n";
    }
    os << "  }\n}\n";
    return os.str();
  }

  // The same evaluation as a device function of the GEMM kernel (implicit GEMM): the gather threads
  // of a CTA fill rows k0 .. k0 + BK of one [BK x BN] tile of the patch operand in shared memory, in
  // the layout a TMA load of an MN-major operand produces (boxes of BK rows x 128 bytes, swizzled).
  // A thread owns one 16-byte piece of the tile's n-extent (4 or 8 consecutive pixels, the same for
  // the whole tile, so what depends on the pixels alone stays in registers over the K loop) and
  // every rgs-th row of k.  Rows beyond K and pixels beyond N are written as zeros.
  std::string gather_tile_source(const GemmDesc& g, size_t patch_node) const {
    const bool f16 = g.dtB == JAXCUDA_F16;
    const int per = f16 ? 8 : 4;
    const bool aligned = g.N % per == 0;
    PatchRun run(*this, patch_node, per, aligned);
    std::ostringstream os;
    os << "#if B_GATHER\n";
    os << "__device__ __forceinline__ void jx_gather_tile(JX_PARAMS, u32 sb, int b, int n_tile, int k0, int gt) {\n";
    os << "  const int piece = gt % (BN / " << per << "), rg = gt / (BN / " << per << ");\n";
    os << "  const int rgs = GROUP_WARPS * 32 / (BN / " << per << ");\n";
    os << "  const int n_first = n_tile + piece * " << per << ";\n";
    os << "  const bool n_in = n_first < " << g.N << ";\n";
    os << "  const u32 box = sb + (u32)(piece * " << per << " / BK) * BOX_BYTES, in_row = (u32)(piece * " << per << " % BK) * ELEM;\n";
    for (int j = 0; j < per; j++) {
      if (aligned) os << "  const int gidx" << j << " = b * " << g.M * g.N << " + (n_in ? n_first : 0) + " << j << ";\n";
      else os << "  const int gidx" << j << " = b * " << g.M * g.N << " + min(n_first + " << j << ", " << g.N - 1 << ");\n";
    }
    run.hoisted(os, "  ");
    os << "  #pragma unroll " << (f16 ? 4 : 8) << "\n  for (int ri = 0; ri < (BK + rgs - 1) / rgs; ri++) {\n    const int r = rg + ri * rgs;\n";
    os << "    if (r >= BK) break;\n";
    os << "    const bool k_in = k0 + r < " << g.K << ";\n    const int ridx = k_in ? k0 + r : " << g.K - 1 << ";\n";
    const std::vector<std::string> val = run.row(os, "    ");
    os << "    float v[" << per << "];\n";
    for (int j = 0; j < per; j++)
      os << "    v[" << j << "] = (k_in && n_first + " << j << " < " << g.N << ") ? (float)" << val[j] << " : 0.0f;\n";
    os << "    const u32 at = box + box_swizzle((u32)r * 128u + in_row);\n";
    if (f16) {
      os << "    __align__(16) jx_half h[8];\n    #pragma unroll\n    for (int j = 0; j < 8; j++) h[j] = jx_f2h(v[j]);\n";
      os << "    st_shared_16(at, *reinterpret_cast<const uint4*>(h));\n";
    } else {
      os << "    uint4 hi, lo;\n";
      os << "    hi.x = __float_as_uint(v[0]); hi.y = __float_as_uint(v[1]); hi.z = __float_as_uint(v[2]); hi.w = __float_as_uint(v[3]);\n";
      os << "    lo.x = __float_as_uint(v[0] - __uint_as_float(hi.x & 0xffffe000u)); lo.y = __float_as_uint(v[1] - __uint_as_float(hi.y & 0xffffe000u));\n";
      os << "    lo.z = __float_as_uint(v[2] - __uint_as_float(hi.z & 0xffffe000u)); lo.w = __float_as_uint(v[3] - __uint_as_float(hi.w & 0xffffe000u));\n";
      os << "    st_shared_16(at, hi);\n    st_shared_16(at + B_BYTES, lo);\n";
    }
    os << "  }\n}\n#endif\n";
    return os.str();
  }

  // Epilogue statements for one output: expects `acc` (float) and `gidx` (int) in scope and
  // assigns the storage-typed result to `dst`.
  std::string epilogue_body(const std::string& indent, const std::string& dst) const {
    std::ostringstream os;
    emit_epilogue_store(os, indent, dst);
    return os.str();
  }

  Plan gemm_ffma(const GemmDesc& g) const {
    Plan p;
    p.skeleton = SK_GEMM_FFMA;
    p.gemm = g;
    account(p);
    p.algo_flops = 2.0 * g.M * g.N * g.K * g.batch;
    const int BM = 128, BN = 128, BK = 16, T = 256;
    std::ostringstream os;
    os << header();
    os << "#define BM " << BM << "\n#define BN " << BN << "\n#define BK " << BK << "\n";
    os << "#define GM " << g.M << "\n#define GN " << g.N << "\n#define GK " << g.K << "\n";
    os << "#define OFFA " << g.offA << "LL\n#define SAM " << g.sAm << "LL\n#define SAK " << g.sAk << "LL\n#define SAB " << g.sAb << "LL\n";
    os << "#define OFFB " << g.offB << "LL\n#define SBN " << g.sBn << "LL\n#define SBK " << g.sBk << "LL\n#define SBB " << g.sBb << "LL\n";
    os << "typedef " << ptype(g.dtA) << " TA;\ntypedef " << ptype(g.dtB) << " TB;\n";
    os << "__device__ __forceinline__ float jx_ldA(const TA* p) { return " << from_storage(g.dtA, "*p") << "; }\n";
    os << "__device__ __forceinline__ float jx_ldB(const TB* p) { return " << from_storage(g.dtB, "*p") << "; }\n";
    // thread -> tile element mapping for the global loads: adjacent threads walk the contiguous axis
    const bool a_kcontig = std::llabs(g.sAk) <= std::llabs(g.sAm);
    const bool b_kcontig = std::llabs(g.sBk) <= std::llabs(g.sBn);
    os << "extern \"C\" __global__ void __launch_bounds__(" << T << ") jx_gemm_ffma(" << params() << ") {\n";
    os << R"(  __shared__ __align__(16) float As[2][BK][BM + 4];
  __shared__ __align__(16) float Bs[2][BK][BN + 4];
  const int t = threadIdx.x;
  const int bz = blockIdx.z, bm = blockIdx.y * BM, bn = blockIdx.x * BN;
)";
    os << "  const TA* A = (const TA*)p" << g.gidA << " + OFFA + (i64)bz * SAB;\n";
    os << "  const TB* B = (const TB*)p" << g.gidB << " + OFFB + (i64)bz * SBB;\n";
    os << "  const int tx = t % 16, ty = t / 16;\n";
    os << "  float c[8][8];\n  #pragma unroll\n  for (int i = 0; i < 8; i++)\n    #pragma unroll\n    for (int j = 0; j < 8; j++) c[i][j] = 0.0f;\n";
    os << "  float ra[8], rb[8];\n";
    // element e (0..7) of this thread within the A tile: (m, k)
    if (a_kcontig) os << "  #define A_K(e) (t % BK)\n  #define A_M(e) (t / BK + (e) * " << T / BK << ")\n";
    else os << "  #define A_M(e) (t % BM)\n  #define A_K(e) (t / BM + (e) * " << T / BM << ")\n";
    if (b_kcontig) os << "  #define B_K(e) (t % BK)\n  #define B_N(e) (t / BK + (e) * " << T / BK << ")\n";
    else os << "  #define B_N(e) (t % BN)\n  #define B_K(e) (t / BN + (e) * " << T / BN << ")\n";
    os << R"(  auto fetch = [&](int k0) {
    #pragma unroll
    for (int e = 0; e < 8; e++) {
      const int m = bm + A_M(e), ka = k0 + A_K(e);
      ra[e] = (m < GM && ka < GK) ? jx_ldA(A + (i64)m * SAM + (i64)ka * SAK) : 0.0f;
      const int n = bn + B_N(e), kb = k0 + B_K(e);
      rb[e] = (n < GN && kb < GK) ? jx_ldB(B + (i64)n * SBN + (i64)kb * SBK) : 0.0f;
    }
  };
  auto stash = [&](int buf) {
    #pragma unroll
    for (int e = 0; e < 8; e++) {
      As[buf][A_K(e)][A_M(e)] = ra[e];
      Bs[buf][B_K(e)][B_N(e)] = rb[e];
    }
  };
  fetch(0);
  stash(0);
  __syncthreads();
  int buf = 0;
  for (int k0 = 0; k0 < GK; k0 += BK) {
    const bool more = k0 + BK < GK;
    if (more) fetch(k0 + BK);
    #pragma unroll
    for (int kk = 0; kk < BK; kk++) {
      float a[8], b[8];
      *(float4*)&a[0] = *(const float4*)&As[buf][kk][ty * 4];
      *(float4*)&a[4] = *(const float4*)&As[buf][kk][ty * 4 + 64];
      *(float4*)&b[0] = *(const float4*)&Bs[buf][kk][tx * 4];
      *(float4*)&b[4] = *(const float4*)&Bs[buf][kk][tx * 4 + 64];
      #pragma unroll
      for (int i = 0; i < 8; i++)
        #pragma unroll
        for (int j = 0; j < 8; j++) c[i][j] = fmaf(a[i], b[j], c[i][j]);
    }
    if (more) { stash(buf ^ 1); __syncthreads(); buf ^= 1; }
  }
  #pragma unroll
  for (int i = 0; i < 8; i++) {
    const int m = bm + ty * 4 + (i & 3) + (i >> 2) * 64;
    if (m >= GM) continue;
    #pragma unroll
    for (int j = 0; j < 8; j++) {
      const int n = bn + tx * 4 + (j & 3) + (j >> 2) * 64;
      if (n >= GN) continue;
      const int gidx = (int)(((i64)bz * GM + m) * GN + n);
      const float acc = c[i][j];
)";
    os << epilogue_body("      ", "out[gidx]");
    os << "    }\n  }\n}\n";
    p.source = os.str();
    Stage st;
    st.entry = "jx_gemm_ffma";
    st.grid[0] = (unsigned)((g.N + BN - 1) / BN);
    st.grid[1] = (unsigned)((g.M + BM - 1) / BM);
    st.grid[2] = (unsigned)g.batch;
    st.block[0] = T;
    p.stages.push_back(st);
    p.describe = "gemm-ffma " + S(g.batch) + "x" + S(g.M) + "x" + S(g.N) + "x" + S(g.K) + " tile 128x128x16";
    return p;
  }

  // Skinny dot with a k-contiguous big operand: C[m, n] = sum_k A[m, k] B[n, k], N <= 16.
  // A warp owns four rows of A and walks k with 128-bit loads; B is staged once per CTA in shared
  // memory as [n][k] (f32), so that a lane's four (or eight) k values of every column are one
  // conflict-free 128-bit shared load shared by its four rows; the N x 4 partial sums per lane are
  // folded with warp shuffles.  CTAs are persistent over blocks of 32 rows, so A is read from HBM
  // exactly once and B from L2 once per CTA.
  bool dot_skinny(const GemmDesc& g, Plan& p) const {
    const int e = dtype_bytes(g.dtA);
    const int VX = 16 / e;                                   // k elements per 128-bit load
    if (g.K % VX || (g.sAm * e) % 16 || (g.offA * e) % 16 || g.sAm <= 0) return false;
    const int64_t pitch = g.K;
    const int64_t smem = g.N * pitch * 4;
    if (smem > 160 * 1024) return false;
    p.skeleton = SK_REDUCE_ROW;
    p.gemm = g;
    account(p);
    p.algo_flops = 2.0 * g.M * g.N * g.K;
    const int R = 4, T = 256, ROWS = (T / 32) * R;
    const int64_t blocks = (g.M + ROWS - 1) / ROWS;
    std::ostringstream os;
    os << header();
    os << "#define GM " << g.M << "\n#define GN " << g.N << "\n#define GK " << g.K << "\n#define VX " << VX << "\n#define BP " << pitch << "\n";
    os << "#define OFFA " << g.offA << "LL\n#define SAM " << g.sAm << "LL\n";
    os << "#define OFFB " << g.offB << "LL\n#define SBN " << g.sBn << "LL\n#define SBK " << g.sBk << "LL\n";
    os << "typedef " << ptype(g.dtA) << " TA;\ntypedef " << ptype(g.dtB) << " TB;\n";
    os << "extern \"C\" __global__ void __launch_bounds__(" << T << ") jx_dot_skinny(" << params() << ") {\n";
    os << "  extern __shared__ __align__(16) float Bs[];   // [GN][BP]\n";
    os << "  const TA* A = (const TA*)p" << g.gidA << " + OFFA;\n  const TB* B = (const TB*)p" << g.gidB << " + OFFB;\n";
    // linear, conflict-free stores; the loads of a [K, N] operand are N elements apart (reading it in
    // memory order and transposing through padded rows measured slower: 35 us against 29 at 8192 rows)
    os << "  for (int i = threadIdx.x; i < GN * GK; i += " << T << ") {\n    const int n = i / GK, kk = i - n * GK;\n";
    os << "    Bs[n * BP + kk] = " << from_storage(g.dtB, "B[(i64)n * SBN + (i64)kk * SBK]") << ";\n  }\n  __syncthreads();\n";
    os << "  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;\n";
    os << "  for (int blk = blockIdx.x; blk < " << blocks << "; blk += gridDim.x) {\n";
    os << "    const int m0 = blk * " << ROWS << " + warp * " << R << ";\n";
    os << "    float acc[" << R << "][GN];\n    #pragma unroll\n    for (int r = 0; r < " << R << "; r++)\n      #pragma unroll\n      for (int n = 0; n < GN; n++) acc[r][n] = 0.0f;\n";
    os << "    #pragma unroll 2\n    for (int k0 = lane * VX; k0 < GK; k0 += 32 * VX) {\n";
    os << "      jx_pack<TA, VX> x[" << R << "];\n      #pragma unroll\n      for (int r = 0; r < " << R << "; r++) {\n";
    os << "        const int m = (m0 + r < GM) ? m0 + r : GM - 1;\n        jx_load(x[r], A + (i64)m * SAM + k0);\n      }\n";
    os << "      #pragma unroll\n      for (int n = 0; n < GN; n++) {\n        #pragma unroll\n        for (int v = 0; v < VX; v += 4) {\n";
    os << "          const float4 y = *reinterpret_cast<const float4*>(&Bs[n * BP + k0 + v]);\n";
    os << "          #pragma unroll\n          for (int r = 0; r < " << R << "; r++) {\n";
    os << "            acc[r][n] = fmaf(" << from_storage(g.dtA, "x[r].e[v]") << ", y.x, acc[r][n]);\n";
    os << "            acc[r][n] = fmaf(" << from_storage(g.dtA, "x[r].e[v + 1]") << ", y.y, acc[r][n]);\n";
    os << "            acc[r][n] = fmaf(" << from_storage(g.dtA, "x[r].e[v + 2]") << ", y.z, acc[r][n]);\n";
    os << "            acc[r][n] = fmaf(" << from_storage(g.dtA, "x[r].e[v + 3]") << ", y.w, acc[r][n]);\n";
    os << "          }\n        }\n      }\n    }\n";
    os << "    #pragma unroll\n    for (int r = 0; r < " << R << "; r++)\n      #pragma unroll\n      for (int n = 0; n < GN; n++)\n";
    os << "        #pragma unroll\n        for (int o = 16; o > 0; o >>= 1) acc[r][n] += __shfl_xor_sync(0xffffffffu, acc[r][n], o);\n";
    os << "    // every lane now holds all sums; lane j finishes output j of the warp's R x GN block\n";
    os << "    #pragma unroll\n    for (int r = 0; r < " << R << "; r++) {\n      #pragma unroll\n      for (int n = 0; n < GN; n++) {\n";
    os << "        if (lane == ((r * GN + n) & 31) && m0 + r < GM) {\n";
    os << "          const int gidx = (m0 + r) * GN + n;\n          const float acc_v = acc[r][n];\n";
    emit_epilogue(os, "          ", "acc_v", "out[gidx]");
    os << "        }\n      }\n    }\n  }\n}\n";
    p.source = os.str();
    Stage st;
    st.entry = "jx_dot_skinny";
    st.grid[0] = (unsigned)std::min<int64_t>(blocks, (int64_t)opt.sm_count * (smem > 100 * 1024 ? 1 : 2));
    st.block[0] = T;
    st.smem = (unsigned)smem;
    p.stages.push_back(st);
    p.describe = "dot-skinny " + S(g.M) + "x" + S(g.N) + "x" + S(g.K) + " rows/warp=4 grid=" + S(st.grid[0]) + "x" + S(T);
    return true;
  }

  // Split-reduction tail shared by the skeletons that keep `[counters | splits x size partials]`
  // in a persistent scratch area: the CTA that arrives last at its column block's counter folds the
  // partials in split order (so the result does not depend on arrival order), applies the epilogue
  // and re-arms the counter.  `outs` = outputs per column block, T = threads per CTA.
  // `gidx_of_gl`: the Kernel's output index of the skeleton's linear output position `gl`, where
  // the two differ (empty: they are the same).
  void emit_split_tail(std::ostream& os, int splits, int64_t outs, int T, const std::string& gidx_of_gl = "") const {
    const char* AT = ctype(k.red_dtype);
    os << "  __shared__ int last;\n  __threadfence();\n  __syncthreads();\n";
    os << "  if (threadIdx.x == 0) last = atomicAdd((int*)scratch + blockIdx.x, 1) == " << splits - 1 << ";\n";
    os << "  __syncthreads();\n  if (!last) return;\n  __threadfence();\n";
    os << "  for (int o = threadIdx.x; o < " << outs << "; o += " << T << ") {\n";
    os << "    const long long gl = (long long)blockIdx.x * " << outs << " + o;\n    if (gl >= " << k.size << "LL) break;\n";
    os << "    const int gidx = " << (gidx_of_gl.empty() ? "(int)gl" : gidx_of_gl) << ";\n    " << AT << " acc_u = " << identity_literal(k.red_op, k.red_dtype) << ";\n";
    os << "    for (int s = 0; s < " << splits << "; s++) { const " << AT << " v = __ldcg(parts + (size_t)s * " << k.size
       << " + gl); acc_u = " << red("acc_u", "v") << "; }\n";
    emit_epilogue(os, "    ", "acc_u", "out[gidx]");
    os << "  }\n";
    os << "  if (threadIdx.x == 0) ((int*)scratch)[blockIdx.x] = 0;\n";
  }

  // Skinny dot with an m-contiguous big operand: C[m, n] = sum_k A[k, m] B[k, n], N <= 16 (the
  // weight gradient of a class-count sized layer: K is the batch).  A thread owns four consecutive
  // m (one 128-bit load of A per k) and all N columns, 4N accumulators; TY thread rows interleave k
  // and keep four loads in flight each; the CTA's slice of B sits in shared memory, rows padded to
  // a multiple of four floats, so that a warp reads it with broadcast 128-bit loads.  K is split
  // over grid.y; partials are folded by the last CTA to arrive (deterministic order).
  // `transposed`: the description has its operands swapped (the big, m-contiguous operand is the
  // Kernel's right factor), so the output element (m, n) of this skeleton is the Kernel's
  // gidx = n * GM + m.
  bool dot_skinny_t(const GemmDesc& g, Plan& p, bool transposed = false) const {
    const int e = dtype_bytes(g.dtA);
    if (g.sAm != 1 || g.M % 4 || (g.offA * e) % (4 * e) || (g.sAk * e) % (4 * e) || g.N > 16) return false;
    const int T = 256, U = 4;
    const int TX = 32, TY = T / TX;   // 128 rows of m per CTA: more column blocks, fewer splits for the last CTA to fold
    const int NP = (int)((g.N + 3) / 4 * 4);
    const int64_t gx = (g.M / 4 + TX - 1) / TX;
    int64_t splits = std::max<int64_t>(1, ((int64_t)opt.sm_count * 2 + gx - 1) / gx);
    splits = std::min<int64_t>(splits, std::max<int64_t>(1, g.K / (TY * U)));
    splits = std::max<int64_t>(splits, (g.K * NP * 4 + 48 * 1024 - 1) / (48 * 1024));
    int64_t rchunk = (g.K + splits - 1) / splits;
    rchunk = (rchunk + TY - 1) / TY * TY;
    splits = (g.K + rchunk - 1) / rchunk;
    const int64_t outs = (int64_t)TX * 4 * g.N;
    const int64_t counter_pad = (1024 + gx * 4 + 255) / 256 * 256;
    p.skeleton = SK_REDUCE_COL;
    p.gemm = g;
    account(p);
    p.algo_flops = 2.0 * g.M * g.N * g.K;
    std::ostringstream os;
    os << header();
    os << "#define GM " << g.M << "\n#define GN " << g.N << "\n#define GK " << g.K << "\n#define NP " << NP << "\n";
    os << "#define TX " << TX << "\n#define TY " << TY << "\n#define RCHUNK " << rchunk << "\n";
    os << "#define OFFA " << g.offA << "LL\n#define SAK " << g.sAk << "LL\n";
    os << "#define OFFB " << g.offB << "LL\n#define SBN " << g.sBn << "LL\n#define SBK " << g.sBk << "LL\n";
    os << "typedef " << ptype(g.dtA) << " TA;\ntypedef " << ptype(g.dtB) << " TB;\n";
    os << "extern \"C\" __global__ void __launch_bounds__(" << T << ") jx_dot_skinny_t(" << params() << ") {\n";
    os << "  extern __shared__ __align__(16) float smem[];\n  float* Bs = smem;                  // [RCHUNK][NP]\n";
    os << "  float* fold = smem + RCHUNK * NP;   // [4 * GN][TX]\n";
    os << "  const TA* A = (const TA*)p" << g.gidA << " + OFFA;\n  const TB* B = (const TB*)p" << g.gidB << " + OFFB;\n";
    os << "  const int tx = threadIdx.x % TX, ty = threadIdx.x / TX;\n";
    os << "  const int m0 = (blockIdx.x * TX + tx) * 4;\n  const bool active = m0 < GM;\n";
    os << "  const int k0 = blockIdx.y * RCHUNK;\n  const int kn = min(GK - k0, RCHUNK);\n";
    os << "  for (int i = threadIdx.x; i < kn * NP; i += " << T << ") {\n    const int kk = i / NP, n = i - kk * NP;\n";
    os << "    Bs[i] = n < GN ? " << from_storage(g.dtB, "B[(i64)n * SBN + (i64)(k0 + kk) * SBK]") << " : 0.0f;\n  }\n  __syncthreads();\n";
    os << "  float acc[4 * GN];\n  #pragma unroll\n  for (int q = 0; q < 4 * GN; q++) acc[q] = 0.0f;\n";
    os << "  const TA* Ap = A + (i64)k0 * SAK + (active ? m0 : 0);\n";
    os << "  for (int kb = ty; kb < kn; kb += TY * " << U << ") {\n    jx_pack<TA, 4> x[" << U << "];\n";
    os << "    #pragma unroll\n    for (int j = 0; j < " << U << "; j++) {\n      const int kk = kb + j * TY;\n";
    os << "      if (kk < kn) jx_load(x[j], Ap + (i64)kk * SAK);\n    }\n";
    os << "    #pragma unroll\n    for (int j = 0; j < " << U << "; j++) {\n      const int kk = kb + j * TY;\n      if (kk < kn) {\n";
    os << "        float bv[NP];\n        #pragma unroll\n        for (int q = 0; q < NP; q += 4) *reinterpret_cast<float4*>(&bv[q]) = *reinterpret_cast<const float4*>(&Bs[kk * NP + q]);\n";
    os << "        #pragma unroll\n        for (int v = 0; v < 4; v++) {\n          const float a = " << from_storage(g.dtA, "x[j].e[v]") << ";\n";
    os << "          #pragma unroll\n          for (int n = 0; n < GN; n++) acc[v * GN + n] = fmaf(a, bv[n], acc[v * GN + n]);\n        }\n      }\n    }\n  }\n";
    os << "  for (int y = 1; y < TY; y++) {\n    if (ty == y) {\n      #pragma unroll\n      for (int q = 0; q < 4 * GN; q++) fold[q * TX + tx] = acc[q];\n    }\n    __syncthreads();\n";
    os << "    if (ty == 0) {\n      #pragma unroll\n      for (int q = 0; q < 4 * GN; q++) acc[q] += fold[q * TX + tx];\n    }\n    __syncthreads();\n  }\n";
    if (splits > 1) {
      os << "  float* parts = (float*)((char*)scratch + " << counter_pad << ");\n";
      os << "  if (ty == 0 && active) {\n    float* part = parts + (size_t)blockIdx.y * " << k.size << " + (size_t)m0 * GN;\n";
      os << "    #pragma unroll\n    for (int q = 0; q < 4 * GN; q += 4) *reinterpret_cast<float4*>(part + q) = make_float4(acc[q], acc[q + 1], acc[q + 2], acc[q + 3]);\n  }\n";
      emit_split_tail(os, (int)splits, outs, T, transposed ? "(int)(gl % GN) * GM + (int)(gl / GN)" : "");
    } else {
      os << "  if (ty != 0 || !active) return;\n  #pragma unroll\n  for (int q = 0; q < 4 * GN; q++) {\n";
      os << "    const int gidx = " << (transposed ? "(q % GN) * GM + m0 + q / GN" : "m0 * GN + q") << ";\n    const float acc_u = acc[q];\n";
      emit_epilogue(os, "    ", "acc_u", "out[gidx]");
      os << "  }\n";
    }
    os << "}\n";
    p.source = os.str();
    Stage st;
    st.entry = "jx_dot_skinny_t";
    st.grid[0] = (unsigned)gx;
    st.grid[1] = (unsigned)splits;
    st.block[0] = T;
    st.smem = (unsigned)((rchunk * NP + outs) * 4);
    p.stages.push_back(st);
    if (splits > 1) {
      p.scratch_bytes = (size_t)counter_pad + (size_t)splits * k.size * 4;
      p.scratch_persistent = true;
    }
    p.describe = std::string("dot-skinny-t ") + (transposed ? "(operands swapped) " : "") + S(g.M) + "x" + S(g.N) + "x" + S(g.K) + " TY=" + S(TY) + " splits=" + S(splits) + " grid=" + S(gx) + "x" + S(T);
    return true;
  }

  // Dot with a tiny contraction (K <= 16, e.g. back-propagation through a class-count sized layer):
  // C[m, n] = epilogue(sum_k A[m, k] B[n, k]).  The kernel is bound by writing C (and by whatever the
  // epilogue reads per element), so it is laid out like the elementwise skeleton: a thread owns four
  // consecutive n, keeps its 4 x K slice of B in registers for its whole life, and walks the CTA's
  // rows two at a time; the rows of A sit in shared memory and are read with broadcast loads; loads
  // of the epilogue that are contiguous in gidx are fetched as 128-bit vectors ahead of the math.
  bool dot_small_k(const GemmDesc& g, Plan& p) const {
    if (g.K > 16 || g.N % 4 || g.N < 128 || g.M < 64) return false;
    const int T = 256, NB = T * 4, NBP = NB + 4, ILP = 2;
    const int KA = (int)((g.K + 3) / 4 * 4);
    const int64_t gx = (g.N + NB - 1) / NB;
    const int64_t want_y = std::max<int64_t>(1, (int64_t)opt.sm_count * 4 / gx);
    int64_t rc = std::min<int64_t>(256, std::max<int64_t>(ILP, (g.M + want_y - 1) / want_y));
    rc = (rc + ILP - 1) / ILP * ILP;
    const int64_t gy = (g.M + rc - 1) / rc;
    if (gy > 65535) return false;
    p.skeleton = SK_GEMM_FFMA;
    p.gemm = g;
    account(p);
    p.algo_flops = 2.0 * g.M * g.N * g.K;
    const bool b_kcontig = std::llabs(g.sBk) <= std::llabs(g.sBn);
    std::ostringstream os;
    os << header();
    os << "#define GM " << g.M << "\n#define GN " << g.N << "\n#define GK " << g.K << "\n#define KA " << KA << "\n";
    os << "#define NB " << NB << "\n#define NBP " << NBP << "\n#define RC " << rc << "\n";
    os << "#define OFFA " << g.offA << "LL\n#define SAM " << g.sAm << "LL\n#define SAK " << g.sAk << "LL\n";
    os << "#define OFFB " << g.offB << "LL\n#define SBN " << g.sBn << "LL\n#define SBK " << g.sBk << "LL\n";
    os << "typedef " << ptype(g.dtA) << " TA;\ntypedef " << ptype(g.dtB) << " TB;\n";
    os << "extern \"C\" __global__ void __launch_bounds__(" << T << ") jx_dot_small_k(" << params() << ") {\n";
    os << "  extern __shared__ __align__(16) float smem[];\n  float* Bs = smem;              // [GK][NBP]\n  float* As = smem + GK * NBP;   // [RC][KA]\n";
    os << "  const TA* A = (const TA*)p" << g.gidA << " + OFFA;\n  const TB* B = (const TB*)p" << g.gidB << " + OFFB;\n";
    os << "  const int nb = blockIdx.x * NB, n0 = nb + threadIdx.x * 4;\n  const bool active = n0 < GN;\n";
    os << "  const int r0 = blockIdx.y * RC;\n  const int rn = min(GM - r0, RC);\n";
    os << "  for (int i = threadIdx.x; i < NB * GK; i += " << T << ") {\n";
    if (b_kcontig) os << "    const int n = i / GK, kk = i - n * GK;\n";
    else os << "    const int kk = i / NB, n = i - kk * NB;\n";
    os << "    Bs[kk * NBP + n] = nb + n < GN ? " << from_storage(g.dtB, "B[(i64)(nb + n) * SBN + (i64)kk * SBK]") << " : 0.0f;\n  }\n";
    os << "  for (int i = threadIdx.x; i < RC * KA; i += " << T << ") {\n    const int r = i / KA, kk = i - r * KA;\n";
    os << "    As[i] = (r < rn && kk < GK) ? " << from_storage(g.dtA, "A[(i64)(r0 + r) * SAM + (i64)kk * SAK]") << " : 0.0f;\n  }\n  __syncthreads();\n";
    os << "  if (!active) return;\n";
    os << "  float w[4][GK];\n  #pragma unroll\n  for (int kk = 0; kk < GK; kk++) {\n    const float4 t = *reinterpret_cast<const float4*>(&Bs[kk * NBP + threadIdx.x * 4]);\n";
    os << "    w[0][kk] = t.x; w[1][kk] = t.y; w[2][kk] = t.z; w[3][kk] = t.w;\n  }\n";
    std::map<size_t, std::string> ov;
    std::ostringstream decl, fetch;
    std::vector<std::string> bnames(k.epi.size());
    std::vector<char> eall(k.epi.size(), 1);
    Env env;
    env.prefix = "e";
    preload(decl, fetch, k.epi, an_epi, eall, 0, 4, env, "g0", "[" + S(ILP) + "]", "[j]", "u", ov, bnames, "        ");
    os << "  for (int rb = 0; rb < rn; rb += " << ILP << ") {\n";
    os << decl.str();
    os << "    #pragma unroll\n    for (int j = 0; j < " << ILP << "; j++) {\n      if (rb + j < rn) {\n";
    os << "        const int g0 = (r0 + rb + j) * GN + n0;\n";
    os << fetch.str();
    os << "      }\n    }\n";
    os << "    #pragma unroll\n    for (int j = 0; j < " << ILP << "; j++) {\n      if (rb + j < rn) {\n";
    os << "        const int g0 = (r0 + rb + j) * GN + n0;\n";
    os << "        float a[KA];\n        #pragma unroll\n        for (int q = 0; q < KA; q += 4) *reinterpret_cast<float4*>(&a[q]) = *reinterpret_cast<const float4*>(&As[(rb + j) * KA + q]);\n";
    os << "        jx_pack<" << ptype(out_dt) << ", 4> res;\n";
    os << "        #pragma unroll\n        for (int u = 0; u < 4; u++) {\n          const int gidx = g0 + u;\n";
    os << "          float acc_u = 0.0f;\n          #pragma unroll\n          for (int kk = 0; kk < GK; kk++) acc_u = fmaf(a[kk], w[u][kk], acc_u);\n";
    {
      std::vector<std::string> en(k.epi.size());
      Env ee;
      ee.prefix = "e";
      ee.acc = "acc_u";
      ee.load_override = &ov;
      emit_nodes(os, k.epi, an_epi, en, eall, ee, "          ");
      os << "          res.e[u] = " << to_storage(out_dt, en.back()) << ";\n";
    }
    os << "        }\n        jx_store(out + g0, res);\n      }\n    }\n  }\n}\n";
    p.source = os.str();
    Stage st;
    st.entry = "jx_dot_small_k";
    st.grid[0] = (unsigned)gx;
    st.grid[1] = (unsigned)gy;
    st.block[0] = T;
    st.smem = (unsigned)((g.K * NBP + rc * KA) * 4);
    p.stages.push_back(st);
    p.describe = "dot-small-k " + S(g.M) + "x" + S(g.N) + "x" + S(g.K) + " rows/cta=" + S(rc) + " grid=" + S(gx) + "x" + S(gy) + "x" + S(T);
    return true;
  }

  Plan build() const {
    if (!k.has_red) return elementwise();
    if (opt.force_skeleton == SK_REDUCE_ROW) return reduce_row();
    if (opt.force_skeleton == SK_REDUCE_COL) return reduce_col();
    GemmDesc g = match_gemm();
    if (g.valid && g.batch == 1 && opt.force_skeleton < 0) {
      // Skinny dots (a class-count sized N): the big operand is streamed once and every thread or
      // warp keeps all N partial sums of its rows.
      if (g.N <= 16 && g.M >= 256 && g.K >= 64) {
        if (g.sAk == 1) { Plan p; if (dot_skinny(g, p)) return p; }
        if (g.sAm == 1 && g.K >= 256) {
          Plan p;
          if (dot_skinny_t(g, p)) return p;
          return reduce_col((int)g.N);
        }
      }
      if (g.K <= 16) { Plan p; if (dot_small_k(g, p)) return p; }
      // few output rows, many columns, a long contraction (the weight gradient of a class-count sized
      // layer written [classes, hidden]): the same skinny skeleton with the operands' roles swapped
      if (g.M <= 16 && g.N >= 256 && g.K >= 256 && g.sBn == 1) {
        GemmDesc t = g;
        t.gidA = g.gidB; t.gidB = g.gidA; t.dtA = g.dtB; t.dtB = g.dtA; t.lenA = g.lenB; t.lenB = g.lenA;
        t.M = g.N; t.N = g.M;
        t.offA = g.offB; t.sAm = g.sBn; t.sAk = g.sBk; t.offB = g.offA; t.sBn = g.sAm; t.sBk = g.sAk;
        Plan p;
        if (dot_skinny_t(t, p, true)) return p;
      }
    }
    if (g.valid && g.batch <= 65535 &&
        ((g.M >= opt.gemm_min_dim && g.N >= opt.gemm_min_dim && g.K >= 8) || opt.force_skeleton == SK_GEMM_FFMA)) {
      if (opt.allow_tc && opt.force_skeleton != SK_GEMM_FFMA) {
        Plan p;
        p.gemm = g;
        account(p);
        p.algo_flops = 2.0 * g.M * g.N * g.K * g.batch;
        // the tensor-core epilogue hands a thread 16 consecutive outputs of one row
        std::string body, pre;
        if (g.N % 16 == 0) {
          std::map<size_t, std::string> ov;
          std::ostringstream decl, fetch, bos;
          std::vector<std::string> bnames(k.epi.size()), en(k.epi.size());
          std::vector<char> eall(k.epi.size(), 1);
          Env env;
          env.prefix = "e";
          preload(decl, fetch, k.epi, an_epi, eall, 0, 16, env, "g0", "", "", "j", ov, bnames, "          ");
          pre = decl.str() + fetch.str();
          env.load_override = &ov;
          emit_nodes(bos, k.epi, an_epi, en, eall, env, "      ");
          bos << "      JX_DST = " << to_storage(out_dt, en.back()) << ";\n";
          body = bos.str();
        } else {
          body = epilogue_body("      ", "JX_DST");
        }
        if (plan_gemm_tc(k, g, opt, p, body, params(), pre)) return p;
      }
      return gemm_ffma(g);
    }
    if (!g.valid && opt.allow_tc && opt.force_skeleton < 0) {
      size_t patch = 0;
      GemmDesc c = match_conv(patch);
      // worth the gather pass once the GEMM is large enough to fill the machine
      if (c.valid && c.M >= 64 && c.N >= 64 && c.K >= 32 && c.K <= 32 * 65535 && c.batch <= 65535 &&
          2.0 * c.M * c.N * c.K * c.batch >= 2e8) {
        Plan p;
        p.gemm = c;
        account(p);
        p.algo_flops = 2.0 * c.M * c.N * c.K * c.batch;
        c.b_implicit = opt.conv_implicit != 0;
        p.gemm = c;
        if (plan_gemm_tc(k, c, opt, p, epilogue_body("      ", "JX_DST"), params(), std::string(),
                         c.b_implicit ? gather_tile_source(c, patch) : gather_source(c, patch))) {
          p.describe = "conv as " + p.describe + (c.b_implicit ? " patches gathered in the kernel" : " patches gathered first");
          return p;
        }
      }
    }
    const int64_t K = k.red_size;
    const bool r_contig = has_load(1), g_contig = has_load(0);
    bool row;
    if (r_contig && !g_contig) row = K >= 16;
    else if (g_contig && !r_contig) row = false;
    else if (r_contig && g_contig) row = k.size < 4096 && K >= 128;
    else row = k.size < 2048 && K >= 128;
    return row ? reduce_row() : reduce_col();
  }
};

}  // namespace

namespace {

// A reduction over a single element is no reduction: out = epilogue(exp at ridx 0).  The batching
// rules produce such Kernels (a Dot or Reduce over an axis of size 1 under vmap); as elementwise
// Kernels they get the vectorised streaming skeleton instead of a reduce loop that runs once.
KernelIR fold_unit_reduction(const KernelIR& k) {
  KernelIR f;
  f.nargs = k.nargs;
  f.size = k.size;
  f.has_red = false;
  f.exp = k.exp;
  for (Node& nd : f.exp)
    if (nd.op == JAXCUDA_OP_SPECIAL && nd.arg0 == 1) { nd.op = JAXCUDA_OP_CONST; nd.dtype = JAXCUDA_I32; nd.nsrc = 0; nd.arg0 = 0; nd.arg1 = 0; }
  uint32_t root = (uint32_t)f.exp.size() - 1;
  if (f.exp[root].dtype != k.red_dtype) {   // the accumulator's type (an f16 product accumulates in f32)
    Node c;
    c.op = JAXCUDA_OP_CAST; c.dtype = k.red_dtype; c.nsrc = 1; c.src[0] = root;
    f.exp.push_back(c);
    root++;
  }
  std::vector<uint32_t> at(k.epi.size());
  for (size_t i = 0; i < k.epi.size(); i++) {
    const Node& nd = k.epi[i];
    if (nd.op == JAXCUDA_OP_VARIABLE) { at[i] = root; continue; }
    Node c = nd;
    for (uint32_t s = 0; s < c.nsrc; s++) c.src[s] = at[nd.src[s]];
    f.exp.push_back(c);
    at[i] = (uint32_t)f.exp.size() - 1;
  }
  if (at.back() != f.exp.size() - 1) {   // the epilogue is the accumulator itself: the root must come last
    Node c = f.exp[at.back()];
    f.exp.push_back(c);
  }
  return f;
}

}  // namespace

bool compose_elementwise(const KernelIR& a_in, const KernelIR& b, uint32_t b_arg, KernelIR& out, std::string& why) {
  if (b.has_red) { why = "the consumer reduces"; return false; }
  if (a_in.has_red && (a_in.red_size != 1 || a_in.exp.empty() || a_in.epi.empty())) { why = "the producer reduces"; return false; }
  const KernelIR a = a_in.has_red ? fold_unit_reduction(a_in) : a_in;
  if (a.exp.empty() || b.exp.empty() || b_arg >= b.nargs) { why = "empty kernel"; return false; }
  const uint32_t a_dt = a.exp.back().dtype;
  if (dtype_bytes(a_dt) != 4) { why = "the producer's output is not a 4-byte type"; return false; }   // f16 rounds on its store
  if (b.nargs - 1 + a.nargs > 64) { why = "too many arguments"; return false; }
  int loads = 0;
  size_t load_at = 0;
  for (size_t i = 0; i < b.exp.size(); i++)
    if (b.exp[i].op == JAXCUDA_OP_GLOBALINDEX && b.exp[i].arg0 == b_arg) { loads++; load_at = i; }
  if (loads != 1) { why = "the consumer loads the array more than once"; return false; }
  const Node& ld = b.exp[load_at];
  if (ld.dtype != a_dt || ld.arg1 != a.size) { why = "the load does not see the whole output in its own type"; return false; }
  const Analysis an = analyze(b.exp, b.size, 1);
  if (!in_range(an.affine[ld.src[0]], ld.arg1)) { why = "the load's index is not proven in range"; return false; }
  for (const Node& nd : a.exp)
    if (nd.op == JAXCUDA_OP_SPECIAL && nd.arg0 != 0) { why = "the producer reads ridx"; return false; }
  out = KernelIR();
  out.nargs = b.nargs - 1 + a.nargs;
  out.size = b.size;
  out.has_red = false;
  std::vector<uint32_t> bmap(b.exp.size(), 0);
  auto b_argno = [&](uint64_t g) { return g < b_arg ? g : g - 1; };
  for (size_t i = 0; i < b.exp.size(); i++) {
    if (i == load_at) {
      const uint32_t index_node = bmap[ld.src[0]];
      std::vector<uint32_t> amap(a.exp.size(), 0);
      for (size_t j = 0; j < a.exp.size(); j++) {
        const Node& nd = a.exp[j];
        if (nd.op == JAXCUDA_OP_SPECIAL) { amap[j] = index_node; continue; }   // A's gidx is B's load index
        Node c = nd;
        for (uint32_t sidx = 0; sidx < c.nsrc; sidx++) c.src[sidx] = amap[nd.src[sidx]];
        if (c.op == JAXCUDA_OP_GLOBALINDEX) c.arg0 = (b.nargs - 1) + nd.arg0;
        out.exp.push_back(c);
        amap[j] = (uint32_t)out.exp.size() - 1;
      }
      bmap[i] = amap.back();
      continue;
    }
    Node c = b.exp[i];
    for (uint32_t sidx = 0; sidx < c.nsrc; sidx++) c.src[sidx] = bmap[b.exp[i].src[sidx]];
    if (c.op == JAXCUDA_OP_GLOBALINDEX) c.arg0 = b_argno(c.arg0);
    out.exp.push_back(c);
    bmap[i] = (uint32_t)out.exp.size() - 1;
  }
  if (bmap.back() != out.exp.size() - 1) out.exp.push_back(out.exp[bmap.back()]);   // the root comes last
  return true;
}

bool compose_epilogue(const KernelIR& a, const KernelIR& b, uint32_t b_arg, KernelIR& out, std::string& why) {
  if (!a.has_red || a.epi.empty() || a.red_size < 2) { why = "the producer does not reduce"; return false; }
  if (b.has_red || b.exp.empty() || b.size != a.size || b_arg >= b.nargs) { why = "the consumer is no elementwise Kernel over the same outputs"; return false; }
  const uint32_t a_dt = a.epi.back().dtype;
  if (dtype_bytes(a_dt) != 4) { why = "the producer's output is not a 4-byte type"; return false; }
  if (a.nargs + b.nargs - 1 > 64) { why = "too many arguments"; return false; }
  int loads = 0;
  size_t load_at = 0;
  for (size_t i = 0; i < b.exp.size(); i++)
    if (b.exp[i].op == JAXCUDA_OP_GLOBALINDEX && b.exp[i].arg0 == b_arg) { loads++; load_at = i; }
  if (loads != 1) { why = "the consumer loads the array more than once"; return false; }
  const Node& ld = b.exp[load_at];
  if (ld.dtype != a_dt || ld.arg1 != a.size) { why = "the load does not see the whole output in its own type"; return false; }
  const Analysis an = analyze(b.exp, b.size, 1);
  const std::optional<Affine>& ix = an.affine[ld.src[0]];
  if (!ix || ix->c0 != 0 || ix->terms.size() != 1 || ix->terms[0].var != 0 || ix->terms[0].div != 1 || ix->terms[0].mod != 0 ||
      ix->terms[0].coef != 1) { why = "the consumer does not read the output at gidx"; return false; }
  for (const Node& nd : b.exp)
    if (nd.op == JAXCUDA_OP_SPECIAL && nd.arg0 != 0) { why = "the consumer reads ridx"; return false; }
  out = a;
  out.nargs = a.nargs + b.nargs - 1;
  const uint32_t a_root = (uint32_t)out.epi.size() - 1;
  std::vector<uint32_t> bmap(b.exp.size(), 0);
  for (size_t i = 0; i < b.exp.size(); i++) {
    if (i == load_at) { bmap[i] = a_root; continue; }
    Node c = b.exp[i];
    for (uint32_t sidx = 0; sidx < c.nsrc; sidx++) c.src[sidx] = bmap[b.exp[i].src[sidx]];
    if (c.op == JAXCUDA_OP_GLOBALINDEX) c.arg0 = a.nargs + (c.arg0 < b_arg ? c.arg0 : c.arg0 - 1);
    out.epi.push_back(c);
    bmap[i] = (uint32_t)out.epi.size() - 1;
  }
  if (bmap.back() != out.epi.size() - 1) out.epi.push_back(out.epi[bmap.back()]);   // the root comes last
  return true;
}

bool plan_small_batch(const std::vector<BatchStage>& stages, int n_params, const Options& opt, Plan& plan, std::string& why) {
  if (stages.size() < 2) { why = "nothing to batch"; return false; }
  const int T = 512;
  std::ostringstream os;
  os << "#define JX_EXACT_TRANSCENDENTALS 1\n#define JX_LD_HINT 0\n" << kPrelude;
  // plain pointers, no __restrict__ and no read-only path: a later stage reads what an earlier one wrote
  os << "extern \"C\" __global__ void __launch_bounds__(" << T << ") jx_batch(";
  for (int i = 0; i < n_params; i++) os << (i ? ", " : "") << "void* q" << i;
  os << ") {\n";
  plan = Plan();
  plan.skeleton = SK_ELEMENTWISE;
  for (size_t s = 0; s < stages.size(); s++) {
    const KernelIR& k = *stages[s].ir;
    KernelIR folded;
    const KernelIR* use = &k;
    if (k.has_red && k.red_size == 1 && !k.exp.empty() && !k.epi.empty()) { folded = fold_unit_reduction(k); use = &folded; }
    Builder b(*use, opt);
    Plan acc;
    b.account(acc);
    plan.algo_bytes += acc.algo_bytes;
    plan.algo_flops += acc.algo_flops;
    if (s) os << "  __threadfence_block();\n  __syncthreads();\n";
    os << "  {  // Kernel " << s << "\n";
    for (uint32_t a = 0; a < use->nargs; a++) os << "    const void* p" << a << " = q" << stages[s].in_param[a] << ";\n";
    os << "    " << ptype(b.out_dt) << "* out = (" << ptype(b.out_dt) << "*)q" << stages[s].out_param << ";\n";
    b.emit_serial(os, T, "    ");
    os << "  }\n";
  }
  os << "}\n";
  plan.source = os.str();
  Stage st;
  st.entry = "jx_batch";
  st.block[0] = T;
  plan.stages.push_back(st);
  plan.describe = "batch of " + S((int64_t)stages.size()) + " small kernels, one CTA of " + S(T);
  return true;
}

Plan make_plan(const KernelIR& k, const Options& opt) {
  if (k.has_red && k.red_size == 1 && opt.force_skeleton < 0 && !k.exp.empty() && !k.epi.empty()) {
    const KernelIR folded = fold_unit_reduction(k);
    Builder b(folded, opt);
    Plan p = b.build();
    p.describe += " (unit reduction folded)";
    return p;
  }
  Builder b(k, opt);
  return b.build();
}

// ---- row programs: several Kernels over the rows of one array as one kernel -------------------

namespace {

enum RowLoad { RL_BAD = 0, RL_BIG, RL_VEC, RL_COL, RL_SCALAR };

// How a load addresses its argument in terms of (row, column).  `row_index` is true where gidx is
// the row itself: in a per-row Kernel and in the epilogue of a row reduction.
RowLoad classify_row_load(RowStageType type, bool row_index, const Node& nd, const std::optional<Affine>& ix, int64_t R,
                          int64_t C) {
  if (!ix || dtype_bytes(nd.dtype) != 4) return RL_BAD;
  const int64_t len = nd.arg1;
  if (ix->terms.empty()) return (ix->c0 >= 0 && ix->c0 < len) ? RL_SCALAR : RL_BAD;
  if (ix->c0 != 0) return RL_BAD;
  auto is = [&](size_t i, int var, int64_t div, int64_t mod, int64_t coef) {
    const Term& t = ix->terms[i];
    return t.var == var && t.div == div && t.mod == mod && t.coef == coef;
  };
  const size_t n = ix->terms.size();
  if (row_index || type == RS_PER_ROW) return (n == 1 && is(0, 0, 1, 0, 1) && len >= R) ? RL_VEC : RL_BAD;
  if (type == RS_REDUCE) {
    if (n == 2 && ((is(0, 0, 1, 0, C) && is(1, 1, 1, 0, 1)) || (is(1, 0, 1, 0, C) && is(0, 1, 1, 0, 1))))
      return len == R * C ? RL_BIG : RL_BAD;
    if (n == 1 && is(0, 0, 1, 0, 1)) return len >= R ? RL_VEC : RL_BAD;
    if (n == 1 && is(0, 1, 1, 0, 1)) return len >= C ? RL_COL : RL_BAD;
    return RL_BAD;
  }
  if (n != 1) return RL_BAD;
  if (is(0, 0, 1, 0, 1)) return len == R * C ? RL_BIG : RL_BAD;   // gidx
  if (is(0, 0, C, 0, 1)) return len >= R ? RL_VEC : RL_BAD;       // gidx / cols
  if (is(0, 0, 1, C, 1)) return len >= C ? RL_COL : RL_BAD;       // gidx % cols
  return RL_BAD;
}

bool four_byte_nodes(const std::vector<Node>& nodes) {
  for (const Node& nd : nodes)
    if (dtype_bytes(nd.dtype) != 4) return false;
  return true;
}

// The nodes a root needs, not descending into the index of a load (every load of a row program is
// replaced by a register or by a (row, column) access).
std::vector<char> closure_above_loads(const std::vector<Node>& nodes, size_t root) {
  std::vector<char> m(nodes.size(), 0);
  m[root] = 1;
  for (size_t i = root + 1; i-- > 0;)
    if (m[i] && nodes[i].op != JAXCUDA_OP_GLOBALINDEX)
      for (uint32_t s = 0; s < nodes[i].nsrc; s++) m[nodes[i].src[s]] = 1;
  return m;
}

}  // namespace

RowStageType row_stage_type(const KernelIR& k, int64_t R, int64_t C) {
  if (R < 2 || C < 2 || R * C >= (int64_t)1 << 31) return RS_NONE;
  if (!four_byte_nodes(k.exp) || (k.has_red && !four_byte_nodes(k.epi))) return RS_NONE;
  RowStageType type;
  if (k.has_red) {
    if ((int64_t)k.size != R || (int64_t)k.red_size != C || dtype_bytes(k.red_dtype) != 4) return RS_NONE;
    type = RS_REDUCE;
  } else if ((int64_t)k.size == R * C) {
    type = RS_ELEMENTWISE;
  } else if ((int64_t)k.size == R) {
    type = RS_PER_ROW;
  } else {
    return RS_NONE;
  }
  const Analysis an = analyze(k.exp, k.size, k.has_red ? k.red_size : 0);
  for (size_t i = 0; i < k.exp.size(); i++)
    if (k.exp[i].op == JAXCUDA_OP_GLOBALINDEX &&
        classify_row_load(type, false, k.exp[i], an.affine[k.exp[i].src[0]], R, C) == RL_BAD)
      return RS_NONE;
  if (k.has_red) {
    const Analysis ae = analyze(k.epi, k.size, 0);
    for (size_t i = 0; i < k.epi.size(); i++)
      if (k.epi[i].op == JAXCUDA_OP_GLOBALINDEX &&
          classify_row_load(type, true, k.epi[i], ae.affine[k.epi[i].src[0]], R, C) == RL_BAD)
        return RS_NONE;
  }
  return type;
}

bool plan_row_fusion(const std::vector<FuseStage>& stages, const std::vector<FuseBuffer>& bufs, int64_t R, int64_t C,
                     const Options& opt, Plan& plan, std::vector<int>& params, std::string& why) {
  auto no = [&](const std::string& m) { why = m; return false; };
  if (C % 4) return no("cols is not a multiple of 4");
  const int64_t chunks = C / 4;   // 128-bit pieces of a row
  const int per_thread = (opt.fuse_chunks == 1 || opt.fuse_chunks == 2 || opt.fuse_chunks == 4) ? opt.fuse_chunks : 4;
  int T = 32;
  while (T < 1024 && (int64_t)T * per_thread < chunks) T *= 2;
  const int E = (int)((chunks + T - 1) / T);
  if (E > 4) return no("row too long for one CTA's registers");
  const int NW = T / 32;

  // what every buffer is inside the program
  const int nb = (int)bufs.size();
  std::vector<int> kind(nb, 0);         // 1: rows x cols, 2: one value per row (produced inside)
  std::vector<uint32_t> dtype(nb, JAXCUDA_F32);
  std::vector<char> produced(nb, 0), read_later(nb, 0), preload(nb, 0), used(nb, 0);
  std::vector<double> ext_bytes(nb, 0.0);   // what the program reads of every outside array
  std::vector<RowStageType> types(stages.size());
  for (size_t s = 0; s < stages.size(); s++) {
    const KernelIR& k = *stages[s].ir;
    types[s] = row_stage_type(k, R, C);
    if (types[s] == RS_NONE) return no("stage " + S((int64_t)s) + " is not a row stage");
  }
  struct LoadRef { RowLoad how; int buf; };
  std::vector<std::map<size_t, LoadRef>> exp_loads(stages.size()), epi_loads(stages.size());
  for (size_t s = 0; s < stages.size(); s++) {
    const KernelIR& k = *stages[s].ir;
    auto scan = [&](const std::vector<Node>& nodes, bool epi, std::map<size_t, LoadRef>& out) -> bool {
      const Analysis an = analyze(nodes, k.size, (!epi && k.has_red) ? k.red_size : 0);
      for (size_t i = 0; i < nodes.size(); i++) {
        const Node& nd = nodes[i];
        if (nd.op != JAXCUDA_OP_GLOBALINDEX) continue;
        const RowLoad how = classify_row_load(types[s], epi, nd, an.affine[nd.src[0]], R, C);
        const int b = stages[s].in_buf[nd.arg0];
        used[b] = 1;
        if (produced[b]) {
          if ((kind[b] == 1 && how != RL_BIG) || (kind[b] == 2 && how != RL_VEC)) return false;
          if (dtype[b] != nd.dtype) return false;
          read_later[b] = 1;
        } else {
          if (!bufs[b].external) return false;
          ext_bytes[b] = std::max(ext_bytes[b], how == RL_BIG ? (double)R * C * 4 : how == RL_VEC ? (double)R * 4
                                                : how == RL_COL ? (double)C * 4 : 4.0);
          if (how == RL_BIG) {
            if (preload[b] && dtype[b] != nd.dtype) return false;
            preload[b] = 1;
            dtype[b] = nd.dtype;
          }
        }
        out[i] = LoadRef{how, b};
      }
      return true;
    };
    if (!scan(k.exp, false, exp_loads[s])) return no("a load of stage " + S((int64_t)s) + " does not match its producer");
    if (k.has_red && !scan(k.epi, true, epi_loads[s])) return no("an epilogue load of stage " + S((int64_t)s) + " does not match its producer");
    const int ob = stages[s].out_buf;
    if (bufs[ob].external && used[ob]) return no("a stage overwrites an array the program reads");
    produced[ob] = 1;
    kind[ob] = types[s] == RS_ELEMENTWISE ? 1 : 2;
    dtype[ob] = k.out_dtype();
  }
  int arrays = 0;
  for (int b = 0; b < nb; b++) arrays += preload[b] || (produced[b] && kind[b] == 1 && read_later[b]);
  if (arrays * E > 16) return no("too many rows x cols arrays live at once");

  params.clear();
  for (int b = 0; b < nb; b++)
    if ((bufs[b].external && used[b]) || (produced[b] && bufs[b].store)) params.push_back(b);

  const double work = (double)R * (double)C;
  const bool exact = opt.exact_math == 1 || (opt.exact_math < 0 && work < opt.exact_math_work);
  std::ostringstream os;
  os << (exact ? "#define JX_EXACT_TRANSCENDENTALS 1\n" : "") << "#define JX_LD_HINT " << std::max(0, opt.ld_hint) << "\n" << kPrelude;
  os << "extern \"C\" __global__ void __launch_bounds__(" << T;
  // 1536 resident threads per SM hold the allocation at 42 registers: measured best for 4096-column rows (44 us against 47 at 1024)
  const int min_ctas = opt.fuse_min_ctas > 0 ? std::min(opt.fuse_min_ctas, 2048 / T) : opt.fuse_min_ctas < 0 ? 0 : std::max(1, 1536 / T);
  if (min_ctas > 0) os << ", " << std::min(min_ctas, 32);
  os << ") jx_rowfuse(";
  for (size_t i = 0; i < params.size(); i++) {
    const int b = params[i];
    const bool written = produced[b] && bufs[b].store;
    os << (i ? ", " : "") << (written ? "" : "const ") << "void* __restrict__ b" << b;
  }
  os << ") {\n";
  os << "  const int row = blockIdx.x, tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;\n";
  os << "  (void)lane; (void)warp;\n";
  const std::string row_off = "(size_t)row * " + S(C);
  auto loop_open = [&](const std::string& ind) {
    os << ind << "#pragma unroll\n" << ind << "for (int e = 0; e < " << E << "; e++) {\n";
    os << ind << "  const int c0 = (e * " << T << " + tid) * 4;\n";
    os << ind << "  if (c0 < " << C << ") {\n";
  };
  auto loop_close = [&](const std::string& ind) { os << ind << "  }\n" << ind << "}\n"; };
  // register arrays and per-row values
  for (int b = 0; b < nb; b++) {
    if (preload[b] || (produced[b] && kind[b] == 1 && read_later[b])) os << "  " << ctype(dtype[b]) << " B" << b << "[" << E * 4 << "];\n";
    if (produced[b] && kind[b] == 2) os << "  " << ctype(dtype[b]) << " v" << b << ";\n";
  }
  for (int b = 0; b < nb; b++) {
    if (!preload[b]) continue;
    loop_open("  ");
    os << "      jx_pack<" << ptype(dtype[b]) << ", 4> t;\n";
    os << "      jx_load(t, (const " << ptype(dtype[b]) << "*)b" << b << " + " << row_off << " + c0);\n";
    os << "      #pragma unroll\n      for (int j = 0; j < 4; j++) B" << b << "[e * 4 + j] = t.e[j];\n";
    loop_close("  ");
  }
  auto overrides = [&](const std::map<size_t, LoadRef>& loads, const std::vector<Node>& nodes, const std::string& col,
                       std::map<size_t, std::string>& ov, std::map<int, uint32_t>* col_packs = nullptr) {
    for (const auto& kv : loads) {
      const Node& nd = nodes[kv.first];
      const int b = kv.second.buf;
      const std::string ptr = std::string("((const ") + ptype(nd.dtype) + "*)b" + S(b) + ")";
      switch (kv.second.how) {
        case RL_BIG: ov[kv.first] = "B" + S(b) + "[e * 4 + j]"; break;
        case RL_VEC: ov[kv.first] = produced[b] ? "v" + S(b) : ptr + "[row]"; break;
        case RL_COL:
          // fetched as one 128-bit load per run of four columns (see `col_fetch`)
          if (col_packs) { (*col_packs)[b] = nd.dtype; ov[kv.first] = "cp" + S(b) + ".e[j]"; }
          else ov[kv.first] = ptr + "[" + col + "]";
          break;
        default: {
          const Analysis an = analyze(nodes, 1, 0);
          ov[kv.first] = ptr + "[" + S(an.affine[nd.src[0]] ? an.affine[nd.src[0]]->c0 : 0) + "]";
        }
      }
    }
  };
  auto col_fetch = [&](const std::map<int, uint32_t>& packs) {
    for (const auto& kv : packs) {
      os << "        jx_pack<" << ptype(kv.second) << ", 4> cp" << kv.first << ";\n";
      os << "        jx_load(cp" << kv.first << ", (const " << ptype(kv.second) << "*)b" << kv.first << " + c0);\n";
    }
  };
  double bytes = 0;
  for (int b = 0; b < nb; b++) bytes += ext_bytes[b];

  // Emission order.  A row reduction costs a CTA-wide barrier, so reductions whose inputs are ready
  // are accumulated together and folded behind one barrier; per-row and elementwise stages that can
  // run first do, because they may make further reductions ready.  Dependences are by buffer.
  const size_t ns = stages.size();
  std::vector<int> producer(nb, -1);
  for (size_t s = 0; s < ns; s++) producer[stages[s].out_buf] = (int)s;
  std::vector<char> done(ns, 0), accumulated(ns, 0);
  auto ready = [&](size_t s) {
    for (int b : stages[s].in_buf)
      if (producer[b] >= 0 && !done[producer[b]]) return false;
    return true;
  };
  auto stage_env = [&](size_t s, std::map<size_t, std::string>& ov) {
    Env env;
    env.prefix = "s" + S((int64_t)s) + "_";
    env.load_override = &ov;
    return env;
  };
  auto store_row_value = [&](size_t s) {
    const int ob = stages[s].out_buf;
    if (bufs[ob].store)
      os << "    if (tid == 0) ((" << ptype(stages[s].ir->out_dtype()) << "*)b" << ob << ")[row] = v" << ob << ";\n";
  };
  auto red_of = [&](size_t s, const std::string& x, const std::string& y) {
    return binary_expr(stages[s].ir->red_op, stages[s].ir->red_dtype, x, y, 0, nullptr);
  };
  auto emit_per_row = [&](size_t s) {
    const KernelIR& k = *stages[s].ir;
    const Analysis an = analyze(k.exp, k.size, 0);
    std::map<size_t, std::string> ov;
    overrides(exp_loads[s], k.exp, "0", ov);
    Env env = stage_env(s, ov);
    env.gidx = "row";
    os << "  {  // stage " << s << ": per row\n";
    std::vector<std::string> names(k.exp.size());
    emit_nodes(os, k.exp, an, names, closure_above_loads(k.exp, k.exp.size() - 1), env, "    ");
    os << "    v" << stages[s].out_buf << " = " << names.back() << ";\n";
    store_row_value(s);
    os << "  }\n";
  };
  auto emit_elementwise = [&](size_t s) {
    const KernelIR& k = *stages[s].ir;
    const int ob = stages[s].out_buf;
    const uint32_t odt = k.out_dtype();
    const Analysis an = analyze(k.exp, k.size, 0);
    std::map<size_t, std::string> ov;
    std::map<int, uint32_t> col_packs;
    overrides(exp_loads[s], k.exp, "cidx", ov, &col_packs);
    Env env = stage_env(s, ov);
    os << "  {  // stage " << s << ": elementwise\n";
    loop_open("    ");
    col_fetch(col_packs);
    os << "        jx_pack<" << ptype(odt) << ", 4> o;\n";
    os << "        #pragma unroll\n        for (int j = 0; j < 4; j++) {\n";
    os << "          const int cidx = c0 + j;\n          const int gidx = row * " << C << " + cidx;\n          (void)gidx;\n";
    std::vector<std::string> names(k.exp.size());
    emit_nodes(os, k.exp, an, names, closure_above_loads(k.exp, k.exp.size() - 1), env, "          ");
    os << "          o.e[j] = " << names.back() << ";\n";
    if (read_later[ob]) os << "          B" << ob << "[e * 4 + j] = " << names.back() << ";\n";
    os << "        }\n";
    if (bufs[ob].store) os << "        jx_store((" << ptype(odt) << "*)b" << ob << " + " << row_off << " + c0, o);\n";
    loop_close("    ");
    os << "  }\n";
  };
  auto emit_accumulate = [&](size_t s) {   // this thread's share and the warp's: leaves the warp's value in acc<s>
    const KernelIR& k = *stages[s].ir;
    const Analysis an = analyze(k.exp, k.size, k.red_size);
    const char* AT = ctype(k.red_dtype);
    std::map<size_t, std::string> ov;
    std::map<int, uint32_t> col_packs;
    overrides(exp_loads[s], k.exp, "ridx", ov, &col_packs);
    Env env = stage_env(s, ov);
    env.gidx = "row";
    const std::string acc = "acc" + S((int64_t)s);
    os << "  " << AT << " " << acc << " = " << identity_literal(k.red_op, k.red_dtype) << ";  // stage " << s << ": row reduction\n";
    if (NW > 1) os << "  __shared__ " << AT << " sm" << s << "[" << NW << "];\n";
    os << "  {\n";
    loop_open("    ");
    col_fetch(col_packs);
    os << "        #pragma unroll\n        for (int j = 0; j < 4; j++) {\n          const int ridx = c0 + j;\n          (void)ridx;\n";
    std::vector<std::string> names(k.exp.size());
    emit_nodes(os, k.exp, an, names, closure_above_loads(k.exp, k.exp.size() - 1), env, "          ");
    os << "          " << acc << " = " << red_of(s, acc, names.back()) << ";\n        }\n";
    loop_close("    ");
    os << "    #pragma unroll\n    for (int o = 16; o > 0; o >>= 1) { const " << AT << " v = __shfl_xor_sync(0xffffffffu, " << acc
       << ", o); " << acc << " = " << red_of(s, acc, "v") << "; }\n";
    if (NW > 1) os << "    if (lane == 0) sm" << s << "[warp] = " << acc << ";\n";
    os << "  }\n";
  };
  auto emit_finish = [&](const std::vector<size_t>& group) {   // one barrier for all of them, then fold and epilogue
    if (NW > 1) os << "  __syncthreads();\n";
    for (size_t s : group) {
      const KernelIR& k = *stages[s].ir;
      const std::string acc = "acc" + S((int64_t)s);
      os << "  {  // stage " << s << ": fold and epilogue\n";
      if (NW > 1) {
        os << "    " << acc << " = sm" << s << "[0];\n";
        os << "    #pragma unroll\n    for (int w = 1; w < " << NW << "; w++) " << acc << " = " << red_of(s, acc, "sm" + S((int64_t)s) + "[w]") << ";\n";
      }
      const Analysis ae = analyze(k.epi, k.size, 0);
      std::map<size_t, std::string> eov;
      overrides(epi_loads[s], k.epi, "0", eov);
      Env ee;
      ee.prefix = "s" + S((int64_t)s) + "e_";
      ee.gidx = "row";
      ee.acc = acc;
      ee.load_override = &eov;
      std::vector<std::string> en(k.epi.size());
      emit_nodes(os, k.epi, ae, en, closure_above_loads(k.epi, k.epi.size() - 1), ee, "    ");
      os << "    v" << stages[s].out_buf << " = " << en.back() << ";\n";
      store_row_value(s);
      os << "  }\n";
    }
  };
  size_t left = ns;
  while (left) {
    bool progress = false;
    for (size_t s = 0; s < ns; s++)   // cheap stages first: they can only make more work ready
      if (!done[s] && types[s] == RS_PER_ROW && ready(s)) { emit_per_row(s); done[s] = 1; left--; progress = true; }
    if (progress) continue;
    // an elementwise stage that feeds a reduction goes before the reductions; the others wait
    for (size_t s = 0; s < ns; s++) {
      if (done[s] || types[s] != RS_ELEMENTWISE || !ready(s) || !read_later[stages[s].out_buf]) continue;
      emit_elementwise(s); done[s] = 1; left--; progress = true;
    }
    if (progress) continue;
    std::vector<size_t> group;
    for (size_t s = 0; s < ns; s++)
      if (!done[s] && types[s] == RS_REDUCE && ready(s)) { emit_accumulate(s); group.push_back(s); }
    if (!group.empty()) {
      emit_finish(group);
      for (size_t s : group) { done[s] = 1; left--; }
      continue;
    }
    for (size_t s = 0; s < ns; s++)
      if (!done[s] && types[s] == RS_ELEMENTWISE && ready(s)) { emit_elementwise(s); done[s] = 1; left--; progress = true; }
    if (!progress) return no("the stages depend on each other in a cycle");
  }
  for (size_t s = 0; s < ns; s++)
    if (bufs[stages[s].out_buf].store) bytes += types[s] == RS_ELEMENTWISE ? (double)R * C * 4 : (double)R * 4;
  os << "}\n";

  plan = Plan();
  plan.skeleton = SK_ELEMENTWISE;
  plan.source = os.str();
  Stage st;
  st.entry = "jx_rowfuse";
  st.grid[0] = (unsigned)R;
  st.block[0] = (unsigned)T;
  plan.stages.push_back(st);
  plan.algo_bytes = bytes;
  plan.algo_flops = 0;
  plan.describe = "row-fused " + S((int64_t)stages.size()) + " kernels rows=" + S(R) + " cols=" + S(C) + " T=" + S(T) + " E=" + S(E);
  return true;
}

}  // namespace jaxcuda
