#include "ir.hpp"

#include <algorithm>
#include <cstring>

namespace jaxcuda {

const char* dtype_name(uint32_t dt) {
  static const char* names[] = {"float32", "int32", "uint32", "bool", "float16", "float64"};
  return dt <= JAXCUDA_F64 ? names[dt] : "?";
}

const char* op_name(uint32_t op) {
  static const char* names[] = {
      "Add", "Sub", "Mul", "Idiv", "Mod", "Min", "Max", "Sin", "Cos", "Asin", "Atan", "Exp", "Log",
      "Erf", "Erfc", "Sqrt", "Floor", "Ceil", "Reciprocal", "Cast", "Bitcast", "BitCombine",
      "BitInvert", "BitShift", "Cmplt", "Cmpne", "Where", "Threefry2x32", "Const", "Special",
      "Variable", "GlobalIndex"};
  return op < JAXCUDA_OP_COUNT ? names[op] : "?";
}

static int expected_nsrc(uint32_t op) {
  switch (op) {
    case JAXCUDA_OP_CONST: case JAXCUDA_OP_SPECIAL: case JAXCUDA_OP_VARIABLE: return 0;
    case JAXCUDA_OP_WHERE: return 3;
    case JAXCUDA_OP_THREEFRY2X32: return 4;
    case JAXCUDA_OP_GLOBALINDEX: case JAXCUDA_OP_BITINVERT: return 1;
    default: break;
  }
  if (op >= JAXCUDA_OP_SIN && op <= JAXCUDA_OP_BITCAST) return 1;
  return 2;
}

std::string parse_kernel(const uint8_t* ir, size_t len, KernelIR& k) {
  if (!ir || len < JAXCUDA_IR_HEADER_WORDS * 4 || len % 4) return "kernel image is truncated";
  std::vector<uint32_t> w(len / 4);
  memcpy(w.data(), ir, len);
  if (w[0] != JAXCUDA_IR_MAGIC) return "kernel image has a bad magic word";
  k.nargs = w[1];
  k.size = (uint64_t)w[2] | ((uint64_t)w[3] << 32);
  k.has_red = w[4] != 0;
  k.red_dtype = w[5];
  k.red_op = w[6];
  k.red_size = w[7];
  const size_t n_exp = w[8], n_epi = w[9];
  if (w.size() != JAXCUDA_IR_HEADER_WORDS + (n_exp + n_epi) * JAXCUDA_IR_NODE_WORDS)
    return "kernel image length does not match its node counts";
  if (k.size >= (1ull << 31)) return "kernel size exceeds int32 indexing";
  if (n_exp == 0) return "kernel has no expression";
  if (k.has_red) {
    if (n_epi == 0) return "reduction kernel has no epilogue";
    if (k.red_dtype > JAXCUDA_F64) return "bad reduction dtype";
    if (k.red_op != JAXCUDA_OP_ADD && k.red_op != JAXCUDA_OP_MUL && k.red_op != JAXCUDA_OP_MIN &&
        k.red_op != JAXCUDA_OP_MAX)
      return "unsupported reduction op";
  } else if (n_epi != 0) {
    return "epilogue without a reduction";
  }
  auto read_nodes = [&](size_t base, size_t n, std::vector<Node>& out, bool epilogue) -> std::string {
    out.resize(n);
    for (size_t i = 0; i < n; i++) {
      const uint32_t* q = &w[base + i * JAXCUDA_IR_NODE_WORDS];
      Node& nd = out[i];
      nd.op = q[0]; nd.dtype = q[1]; nd.nsrc = q[2];
      for (int s = 0; s < 4; s++) nd.src[s] = q[3 + s];
      nd.arg0 = (uint64_t)q[7] | ((uint64_t)q[8] << 32);
      nd.arg1 = q[9];
      if (nd.op >= JAXCUDA_OP_COUNT) return "unknown op";
      if (nd.dtype > JAXCUDA_F64) return "unknown dtype";
      if ((int)nd.nsrc != expected_nsrc(nd.op)) return std::string("wrong operand count for ") + op_name(nd.op);
      for (uint32_t s = 0; s < nd.nsrc; s++)
        if (nd.src[s] >= i) return "node operands are not topologically ordered";
      if (nd.op == JAXCUDA_OP_GLOBALINDEX && nd.arg0 >= k.nargs) return "GlobalIndex names a missing argument";
      if (nd.op == JAXCUDA_OP_SPECIAL) {
        if (nd.arg0 > 1) return "unknown Special";
        if (nd.arg0 == 1 && (epilogue || !k.has_red)) return "ridx used outside a reduction body";
      }
      if (nd.op == JAXCUDA_OP_VARIABLE && !epilogue) return "acc used outside an epilogue";
      if (nd.op == JAXCUDA_OP_VARIABLE && nd.dtype != k.red_dtype) return "acc dtype differs from the reduction dtype";
    }
    return "";
  };
  std::string err = read_nodes(JAXCUDA_IR_HEADER_WORDS, n_exp, k.exp, false);
  if (!err.empty()) return err;
  err = read_nodes(JAXCUDA_IR_HEADER_WORDS + n_exp * JAXCUDA_IR_NODE_WORDS, n_epi, k.epi, true);
  if (!err.empty()) return err;
  if (k.has_red && k.exp.back().dtype != k.red_dtype) return "body dtype differs from the reduction dtype";
  return "";
}

// ---- affine forms -------------------------------------------------------------------

int64_t Affine::coef_of(int var, int64_t div) const {
  for (const Term& t : terms)
    if (t.var == var && t.div == div) return t.coef;
  return 0;
}
bool Affine::depends_on(int var) const {
  for (const Term& t : terms)
    if (t.var == var) return true;
  return false;
}
bool Affine::only_plain(int var) const {
  for (const Term& t : terms)
    if (t.var == var && !(t.div == 1 && t.mod == 0)) return false;
  return true;
}

namespace {

struct Space { int64_t n[2]; };  // index ranges of gidx and ridx

int64_t digit_max(const Term& t, const Space& sp) {
  int64_t n = sp.n[t.var];
  if (n <= 0) return 0;
  int64_t top = (n - 1) / t.div;
  return (t.mod && t.mod - 1 < top) ? t.mod - 1 : top;
}

void normalize(Affine& a, const Space& sp) {
  std::vector<Term> out;
  for (Term t : a.terms) {
    if (t.coef == 0) continue;
    int64_t n = sp.n[t.var];
    if (n <= 0 || t.div > n - 1) continue;           // the digit is always zero
    if (t.mod == 1) continue;
    if (t.mod && (n - 1) / t.div < t.mod) t.mod = 0;  // the modulus never bites
    bool merged = false;
    for (Term& o : out)
      if (o.var == t.var && o.div == t.div && o.mod == t.mod) { o.coef += t.coef; merged = true; break; }
    if (!merged) out.push_back(t);
  }
  out.erase(std::remove_if(out.begin(), out.end(), [](const Term& t) { return t.coef == 0; }), out.end());
  a.terms = out;
  a.lo = a.hi = a.c0;
  for (const Term& t : a.terms) {
    int64_t m = digit_max(t, sp) * t.coef;
    if (m > 0) a.hi += m; else a.lo += m;
  }
}

std::optional<Affine> combine(const Affine& x, const Affine& y, int64_t sy, const Space& sp) {
  Affine r;
  r.c0 = x.c0 + sy * y.c0;
  r.terms = x.terms;
  for (Term t : y.terms) { t.coef *= sy; r.terms.push_back(t); }
  normalize(r, sp);
  return r;
}

std::optional<Affine> scale(const Affine& x, int64_t s, const Space& sp) {
  Affine r = x;
  r.c0 *= s;
  for (Term& t : r.terms) t.coef *= s;
  normalize(r, sp);
  return r;
}

bool is_const(const Affine& a) { return a.terms.empty(); }
bool single_digit(const Affine& a) { return a.c0 == 0 && a.terms.size() == 1 && a.terms[0].coef == 1; }

// A non-negative mixed-radix form splits at c into the digits whose weights are multiples of c and
// the rest, when the rest never reaches c: x = c * high + low with 0 <= low < c.  This is what
// recovers the digits of an index that an earlier Kernel's view had flattened
// ((a * 64 + b * 65536 + d) / 65536 = b when a * 64 + d stays below 65536).
bool split_at(const Affine& x, int64_t c, const Space& sp, Affine& high, Affine& low) {
  if (x.lo < 0 || x.c0 < 0) return false;
  high = Affine();
  low = Affine();
  high.c0 = x.c0 / c;
  low.c0 = x.c0 % c;
  for (Term t : x.terms) {
    if (t.coef < 0) return false;
    if (t.coef % c == 0) { t.coef /= c; high.terms.push_back(t); }
    else low.terms.push_back(t);
  }
  normalize(low, sp);
  if (low.hi >= c) return false;
  normalize(high, sp);
  return true;
}

std::optional<Affine> idiv(const Affine& x, int64_t c, const Space& sp) {
  if (c <= 0) return std::nullopt;
  if (x.lo >= 0 && x.hi < c) { Affine z; normalize(z, sp); return z; }
  if (single_digit(x)) {
    Term t = x.terms[0];
    if (t.mod && t.mod % c != 0) return std::nullopt;
    t.div *= c;
    if (t.mod) t.mod /= c;
    Affine r; r.terms = {t}; normalize(r, sp); return r;
  }
  bool divisible = x.lo >= 0 && x.c0 % c == 0;
  for (const Term& t : x.terms) divisible = divisible && t.coef % c == 0 && t.coef >= 0;
  if (divisible) {  // every part divisible: exact
    Affine r = x;
    r.c0 /= c;
    for (Term& t : r.terms) t.coef /= c;
    normalize(r, sp);
    return r;
  }
  Affine high, low;
  if (split_at(x, c, sp, high, low)) return high;
  return std::nullopt;
}

std::optional<Affine> mod(const Affine& x, int64_t c, const Space& sp) {
  if (c <= 0) return std::nullopt;
  if (x.lo >= 0 && x.hi < c) return x;
  if (single_digit(x)) {
    Term t = x.terms[0];
    if (t.mod && t.mod % c != 0) return std::nullopt;
    t.mod = c;
    Affine r; r.terms = {t}; normalize(r, sp); return r;
  }
  Affine high, low;
  if (split_at(x, c, sp, high, low)) return low;
  return std::nullopt;
}

}  // namespace

Analysis analyze(const std::vector<Node>& nodes, uint64_t gsize, uint64_t rsize) {
  Analysis an;
  const size_t n = nodes.size();
  an.affine.resize(n);
  an.dep_g.assign(n, false);
  an.dep_r.assign(n, false);
  Space sp{{(int64_t)gsize, (int64_t)rsize}};
  for (size_t i = 0; i < n; i++) {
    const Node& nd = nodes[i];
    for (uint32_t s = 0; s < nd.nsrc; s++) {
      an.dep_g[i] = an.dep_g[i] || an.dep_g[nd.src[s]];
      an.dep_r[i] = an.dep_r[i] || an.dep_r[nd.src[s]];
    }
    if (nd.op == JAXCUDA_OP_SPECIAL) (nd.arg0 == 0 ? an.dep_g : an.dep_r)[i] = true;
    if (nd.dtype != JAXCUDA_I32 && nd.dtype != JAXCUDA_U32) continue;
    auto src = [&](int s) -> const std::optional<Affine>& { return an.affine[nd.src[s]]; };
    switch (nd.op) {
      case JAXCUDA_OP_CONST: {
        Affine a;
        a.c0 = nd.dtype == JAXCUDA_I32 ? (int64_t)(int32_t)(uint32_t)nd.arg0 : (int64_t)(uint32_t)nd.arg0;
        normalize(a, sp);
        an.affine[i] = a;
        break;
      }
      case JAXCUDA_OP_SPECIAL: {
        Affine a;
        a.terms.push_back(Term{(int)nd.arg0, 1, 0, 1});
        normalize(a, sp);
        an.affine[i] = a;
        break;
      }
      case JAXCUDA_OP_ADD:
        if (src(0) && src(1)) an.affine[i] = combine(*src(0), *src(1), 1, sp);
        break;
      case JAXCUDA_OP_SUB:
        if (src(0) && src(1)) an.affine[i] = combine(*src(0), *src(1), -1, sp);
        break;
      case JAXCUDA_OP_MUL:
        if (src(0) && src(1)) {
          if (is_const(*src(1))) an.affine[i] = scale(*src(0), src(1)->c0, sp);
          else if (is_const(*src(0))) an.affine[i] = scale(*src(1), src(0)->c0, sp);
        }
        break;
      case JAXCUDA_OP_IDIV:
        if (src(0) && src(1) && is_const(*src(1))) an.affine[i] = idiv(*src(0), src(1)->c0, sp);
        break;
      case JAXCUDA_OP_MOD:
        if (src(0) && src(1) && is_const(*src(1))) an.affine[i] = mod(*src(0), src(1)->c0, sp);
        break;
      case JAXCUDA_OP_CAST:
        if (src(0) && src(0)->lo >= 0 &&
            (nodes[nd.src[0]].dtype == JAXCUDA_I32 || nodes[nd.src[0]].dtype == JAXCUDA_U32))
          an.affine[i] = *src(0);
        break;
      default: break;
    }
    // An index that could wrap int32 is not treated as affine.
    if (an.affine[i] && (an.affine[i]->hi > INT32_MAX || an.affine[i]->lo < INT32_MIN)) an.affine[i].reset();
  }
  return an;
}

}  // namespace jaxcuda
