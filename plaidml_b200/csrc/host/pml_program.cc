// Lowering of the expression tree to the flat program, including contraction bounds.
#include "pml_program.h"

#include <cuda_fp16.h>

#include <algorithm>
#include <cmath>
#include <cstring>
#include <limits>
#include <functional>
#include <map>
#include <numeric>
#include <sstream>

namespace pml {

// ------------------------------------------------------------------ rationals

Rational::Rational(int64_t n, int64_t d) {
  if (d == 0) throw std::runtime_error("Division by zero in index expression");
  if (d < 0) {
    n = -n;
    d = -d;
  }
  const int64_t g = std::gcd(n < 0 ? -n : n, d);
  num = g ? n / g : n;
  den = g ? d / g : d;
}
Rational operator+(Rational a, Rational b) { return Rational(a.num * b.den + b.num * a.den, a.den * b.den); }
Rational operator-(Rational a, Rational b) { return Rational(a.num * b.den - b.num * a.den, a.den * b.den); }
Rational operator*(Rational a, Rational b) { return Rational(a.num * b.num, a.den * b.den); }
Rational operator/(Rational a, Rational b) { return Rational(a.num * b.den, a.den * b.num); }

static int64_t floorDiv(int64_t a, int64_t b) {
  int64_t q = a / b;
  if ((a % b != 0) && ((a < 0) != (b < 0))) --q;
  return q;
}
static int64_t ceilR(Rational r) { return -floorDiv(-r.num, r.den); }
static int64_t floorR(Rational r) { return floorDiv(r.num, r.den); }

// ------------------------------------------------------------------ index polynomials

size_t IndexNumbering::indexOf(const PolyNode* node) {
  auto it = ids_.find(node);
  if (it != ids_.end()) return it->second;
  const size_t id = names_.size();
  ids_[node] = id;
  names_.push_back(node->name.empty() ? "x" + std::to_string(id) : node->name);
  return id;
}

static bool isConstant(const Affine& a) {
  for (const Rational& c : a.coef) {
    if (!c.isZero()) return false;
  }
  return true;
}

Affine evalPoly(const PolyPtr& poly, IndexNumbering* idxs, Evaluator* ev) {
  Affine out;
  switch (poly->kind) {
    case PolyNode::Dim:
      out.constant = Rational(ev->evaluate(poly->dim));
      return out;
    case PolyNode::Literal:
      out.constant = Rational(poly->value);
      return out;
    case PolyNode::Index: {
      const size_t id = idxs->indexOf(poly.get());
      out.resize(id + 1);
      out.coef[id] = Rational(1);
      return out;
    }
    case PolyNode::Op: {
      if (poly->op == AffineOp::Neg) {
        if (poly->operands.size() != 1) throw std::runtime_error("Negation takes one operand");
        Affine a = evalPoly(poly->operands[0], idxs, ev);
        for (auto& c : a.coef) c = Rational(0) - c;
        a.constant = Rational(0) - a.constant;
        return a;
      }
      if (poly->operands.size() != 2) throw std::runtime_error("Binary index operation takes two operands");
      Affine a = evalPoly(poly->operands[0], idxs, ev);
      Affine b = evalPoly(poly->operands[1], idxs, ev);
      const size_t n = std::max(a.coef.size(), b.coef.size());
      a.resize(n);
      b.resize(n);
      switch (poly->op) {
        case AffineOp::Add:
          for (size_t i = 0; i < n; ++i) a.coef[i] = a.coef[i] + b.coef[i];
          a.constant = a.constant + b.constant;
          return a;
        case AffineOp::Sub:
          for (size_t i = 0; i < n; ++i) a.coef[i] = a.coef[i] - b.coef[i];
          a.constant = a.constant - b.constant;
          return a;
        case AffineOp::Mul:
          if (isConstant(b)) {
            for (size_t i = 0; i < n; ++i) a.coef[i] = a.coef[i] * b.constant;
            a.constant = a.constant * b.constant;
            return a;
          }
          if (isConstant(a)) {
            for (size_t i = 0; i < n; ++i) b.coef[i] = b.coef[i] * a.constant;
            b.constant = b.constant * a.constant;
            return b;
          }
          throw std::runtime_error("Non-linear polynomial: index expressions may only be multiplied by constants");
        case AffineOp::Div:
          if (!isConstant(b)) throw std::runtime_error("Index expressions may only be divided by constants");
          if (b.constant.isZero()) throw std::runtime_error("Division by zero in index expression");
          for (size_t i = 0; i < n; ++i) a.coef[i] = a.coef[i] / b.constant;
          a.constant = a.constant / b.constant;
          return a;
        case AffineOp::Max:
        case AffineOp::Min: {
          if (!isConstant(a) || !isConstant(b)) throw std::runtime_error("max / min of index variables is not affine");
          const bool aLess = a.constant.num * b.constant.den < b.constant.num * a.constant.den;
          return (poly->op == AffineOp::Max) == aLess ? b : a;
        }
        default: break;
      }
      throw std::runtime_error("Invalid index operation");
    }
  }
  throw std::runtime_error("Invalid index polynomial");
}

// ------------------------------------------------------------------ bounds

void computeBounds(BoundedContraction* c, const TensorShape& out, const std::vector<TensorShape>& srcShapes) {
  const size_t n = c->nIdx();
  struct Cond {
    Affine f;
    int64_t bound;
  };
  std::vector<Cond> conds;
  auto add = [&](Affine f, int64_t bound) {
    f.resize(n);
    conds.push_back({std::move(f), bound});
  };
  for (size_t d = 0; d < c->sink.size(); ++d) add(c->sink[d], out.sizes[d]);
  for (size_t s = 0; s < c->srcs.size(); ++s) {
    if (c->srcs[s].size() != srcShapes[s].rank()) {
      throw std::runtime_error("Contraction operand is indexed with " + std::to_string(c->srcs[s].size()) +
                               " indices but has rank " + std::to_string(srcShapes[s].rank()));
    }
    for (size_t d = 0; d < c->srcs[s].size(); ++d) add(c->srcs[s][d], srcShapes[s].sizes[d]);
  }
  for (const auto& con : c->cons) add(con.first, con.second);

  constexpr int64_t kInf = std::numeric_limits<int64_t>::max() / 4;
  std::vector<int64_t> lo(n, -kInf), hi(n, kInf);
  bool changed = true;
  for (int iter = 0; iter < 64 && changed; ++iter) {
    changed = false;
    for (const Cond& cd : conds) {
      for (size_t j = 0; j < n; ++j) {
        const Rational aj = cd.f.coef[j];
        if (aj.isZero()) continue;
        // range of the rest of the form
        bool minFinite = true, maxFinite = true;
        Rational rmin = cd.f.constant, rmax = cd.f.constant;
        for (size_t i = 0; i < n; ++i) {
          if (i == j || cd.f.coef[i].isZero()) continue;
          const Rational ai = cd.f.coef[i];
          const bool pos = ai.num > 0;
          const int64_t l = pos ? lo[i] : hi[i];  // bound giving the smaller product
          const int64_t h = pos ? hi[i] : lo[i];
          if (l <= -kInf || l >= kInf) minFinite = false; else rmin = rmin + ai * Rational(l);
          if (h <= -kInf || h >= kInf) maxFinite = false; else rmax = rmax + ai * Rational(h);
        }
        // 0 <= aj * xj + rest <= bound - 1
        // => aj * xj >= -rmax   and   aj * xj <= bound - 1 - rmin
        if (maxFinite) {
          const Rational v = (Rational(0) - rmax) / aj;
          if (aj.num > 0) {
            const int64_t nl = ceilR(v);
            if (nl > lo[j]) { lo[j] = nl; changed = true; }
          } else {
            const int64_t nh = floorR(v);
            if (nh < hi[j]) { hi[j] = nh; changed = true; }
          }
        }
        if (minFinite) {
          const Rational v = (Rational(cd.bound - 1) - rmin) / aj;
          if (aj.num > 0) {
            const int64_t nh = floorR(v);
            if (nh < hi[j]) { hi[j] = nh; changed = true; }
          } else {
            const int64_t nl = ceilR(v);
            if (nl > lo[j]) { lo[j] = nl; changed = true; }
          }
        }
      }
    }
  }
  // Indices that only constraints on sums or differences limit (0 <= i + j < 5 together with
  // 0 <= i - j < 5 bounds both, but neither condition alone bounds either): the propagation above needs a
  // finite range of the other variable to start from.  For those the bounding box of the rational polytope
  // is computed by Fourier-Motzkin elimination and rounded inwards.  The reference solves an integer
  // program per index instead (pmlc/dialect/tile/transforms/contraction.cc:576-655,
  // pmlc/util/bilp/ilp_solver.h:26-100); a box that is a little larger costs only idle iterations here,
  // because the kernels test every condition at every point.
  auto unbounded = [&](size_t i) { return lo[i] <= -kInf || hi[i] >= kInf; };
  bool anyUnbounded = false;
  for (size_t i = 0; i < n; ++i) anyUnbounded = anyUnbounded || unbounded(i);
  if (anyUnbounded) {
    struct Ineq {   // constant + sum coef * x >= 0
      std::vector<Rational> coef;
      Rational constant;
    };
    std::vector<Ineq> base;
    for (const Cond& cd : conds) {
      Ineq ge{cd.f.coef, cd.f.constant};                       // f >= 0
      Ineq le{std::vector<Rational>(n), Rational(cd.bound - 1) - cd.f.constant};   // bound - 1 - f >= 0
      for (size_t i = 0; i < n; ++i) le.coef[i] = Rational(0) - cd.f.coef[i];
      base.push_back(std::move(ge));
      base.push_back(std::move(le));
    }
    for (size_t i = 0; i < n; ++i) {   // what the propagation already knows
      if (lo[i] > -kInf) {
        Ineq q{std::vector<Rational>(n), Rational(-lo[i])};
        q.coef[i] = Rational(1);
        base.push_back(std::move(q));
      }
      if (hi[i] < kInf) {
        Ineq q{std::vector<Rational>(n), Rational(hi[i])};
        q.coef[i] = Rational(-1);
        base.push_back(std::move(q));
      }
    }
    constexpr size_t kMaxIneq = 4000;
    for (size_t target = 0; target < n; ++target) {
      if (!unbounded(target)) continue;
      std::vector<Ineq> sys = base;
      bool gaveUp = false;
      for (size_t v = 0; v < n && !gaveUp; ++v) {
        if (v == target) continue;
        std::vector<Ineq> pos, neg, rest;
        for (Ineq& q : sys) {
          if (q.coef[v].isZero()) rest.push_back(std::move(q));
          else if (q.coef[v].num > 0) pos.push_back(std::move(q));
          else neg.push_back(std::move(q));
        }
        if (rest.size() + pos.size() * neg.size() > kMaxIneq) {
          gaveUp = true;
          break;
        }
        for (const Ineq& a : pos) {
          for (const Ineq& b : neg) {
            // a / a_v + b / (-b_v) has no x_v
            const Rational fa = Rational(1) / a.coef[v], fb = Rational(1) / (Rational(0) - b.coef[v]);
            Ineq q{std::vector<Rational>(n), a.constant * fa + b.constant * fb};
            bool trivial = true;
            for (size_t i = 0; i < n; ++i) {
              if (i == v) continue;
              q.coef[i] = a.coef[i] * fa + b.coef[i] * fb;
              if (!q.coef[i].isZero()) trivial = false;
            }
            if (!trivial) rest.push_back(std::move(q));
          }
        }
        sys = std::move(rest);
      }
      if (gaveUp) continue;
      for (const Ineq& q : sys) {
        const Rational a = q.coef[target];
        if (a.isZero()) continue;
        const Rational v = (Rational(0) - q.constant) / a;   // a x + c >= 0
        if (a.num > 0) lo[target] = std::max(lo[target], ceilR(v));
        else hi[target] = std::min(hi[target], floorR(v));
      }
    }
  }
  c->lower.assign(n, 0);
  c->extent.assign(n, 0);
  for (size_t i = 0; i < n; ++i) {
    if (lo[i] <= -kInf || hi[i] >= kInf) {
      throw std::runtime_error("Unbounded index '" + c->idxNames[i] + "' in contraction: no tensor dimension or constraint limits it");
    }
    c->lower[i] = lo[i];
    c->extent[i] = hi[i] >= lo[i] ? hi[i] - lo[i] + 1 : 0;
  }
}

// ------------------------------------------------------------------ scalar constants

static uint16_t f32ToBf16(float f) {
  uint32_t u;
  std::memcpy(&u, &f, 4);
  if ((u & 0x7fffffffu) > 0x7f800000u) return static_cast<uint16_t>((u >> 16) | 0x40);
  u += 0x7fffu + ((u >> 16) & 1u);
  return static_cast<uint16_t>(u >> 16);
}

static uint16_t f32ToF16(float f) {
  const __half h = __float2half_rn(f);
  uint16_t u;
  std::memcpy(&u, &h, 2);
  return u;
}

static float bf16ToF32(uint16_t h) {
  const uint32_t u = static_cast<uint32_t>(h) << 16;
  float f;
  std::memcpy(&f, &u, 4);
  return f;
}

static float f16ToF32(uint16_t u) {
  __half h;
  std::memcpy(&h, &u, 2);
  return __half2float(h);
}

BufferPtr makeScalarConstant(DType dtype, const Literal& lit) {
  DType dt = dtype;
  if (dt == DType::six) dt = DType::si32;
  if (dt == DType::uix) dt = DType::ui32;
  if (dt == DType::fx) dt = DType::f32;
  BufferPtr buf = Buffer::allocate(TensorShape(dt));
  const double asF = lit.kind == Literal::Float ? lit.f : (lit.kind == Literal::Signed ? static_cast<double>(lit.i) : static_cast<double>(lit.u));
  const int64_t asI = lit.kind == Literal::Float ? static_cast<int64_t>(lit.f) : (lit.kind == Literal::Signed ? lit.i : static_cast<int64_t>(lit.u));
  char* p = buf->data();
  switch (dt) {
    case DType::i1: { uint8_t v = asF != 0; std::memcpy(p, &v, 1); break; }
    case DType::si8: case DType::ui8: { int8_t v = static_cast<int8_t>(asI); std::memcpy(p, &v, 1); break; }
    case DType::si16: case DType::ui16: { int16_t v = static_cast<int16_t>(asI); std::memcpy(p, &v, 2); break; }
    case DType::si32: case DType::ui32: { int32_t v = static_cast<int32_t>(asI); std::memcpy(p, &v, 4); break; }
    case DType::si64: case DType::ui64: { std::memcpy(p, &asI, 8); break; }
    case DType::f16: { uint16_t v = f32ToF16(static_cast<float>(asF)); std::memcpy(p, &v, 2); break; }
    case DType::bf16: { uint16_t v = f32ToBf16(static_cast<float>(asF)); std::memcpy(p, &v, 2); break; }
    case DType::f32: { float v = static_cast<float>(asF); std::memcpy(p, &v, 4); break; }
    case DType::f64: { std::memcpy(p, &asF, 8); break; }
    default: throw std::runtime_error("Cannot materialise a literal of this type");
  }
  return buf;
}

// ------------------------------------------------------------------ printing

static std::string affineStr(const Affine& a, const std::vector<std::string>& names) {
  std::ostringstream os;
  bool any = false;
  for (size_t i = 0; i < a.coef.size(); ++i) {
    if (a.coef[i].isZero()) continue;
    if (any) os << " + ";
    if (!(a.coef[i].num == 1 && a.coef[i].den == 1)) {
      os << a.coef[i].num;
      if (a.coef[i].den != 1) os << "/" << a.coef[i].den;
      os << "*";
    }
    os << names[i];
    any = true;
  }
  if (!a.constant.isZero() || !any) {
    if (any) os << " + ";
    os << a.constant.num;
    if (a.constant.den != 1) os << "/" << a.constant.den;
  }
  return os.str();
}

std::string Program::str() const {
  static const char* aggNames[] = {"assign", "add", "max", "min", "mul"};
  static const char* comboNames[] = {"none", "add", "cond", "eq", "mul"};
  std::ostringstream os;
  os << "program @" << name << "(";
  bool first = true;
  for (int id : inputs) {
    os << (first ? "" : ", ") << "%" << id << ": " << values[id].shape.str();
    first = false;
  }
  for (int id : constants) {
    os << (first ? "" : ", ") << "%" << id << ": " << values[id].shape.str() << " {const}";
    first = false;
  }
  os << ") {\n";
  for (const POp& op : ops) {
    os << "  %" << op.result << " = ";
    if (op.kind == POp::Contraction) {
      const BoundedContraction& c = *op.c;
      os << "tile.contract " << aggNames[static_cast<int>(c.agg)] << ", " << comboNames[static_cast<int>(c.combo)];
      os << " sink (";
      for (size_t d = 0; d < c.sink.size(); ++d) os << (d ? ", " : "") << affineStr(c.sink[d], c.idxNames);
      os << ")";
      for (size_t s = 0; s < c.srcs.size(); ++s) {
        os << " %" << op.operands[s] << "(";
        for (size_t d = 0; d < c.srcs[s].size(); ++d) os << (d ? ", " : "") << affineStr(c.srcs[s][d], c.idxNames);
        os << ")";
      }
      if (c.hasInit) os << " init %" << op.operands.back();
      os << " {";
      for (size_t i = 0; i < c.nIdx(); ++i) {
        os << (i ? ", " : "") << c.idxNames[i] << " in [" << c.lower[i] << ", " << c.lower[i] + c.extent[i] << ")";
      }
      os << "}";
      for (const auto& con : c.cons) os << " where 0 <= " << affineStr(con.first, c.idxNames) << " < " << con.second;
      if (!op.label.empty()) os << " name=\"" << op.label << "\"";
    } else {
      os << "tile." << op.mnemonic;
      for (size_t i = 0; i < op.operands.size(); ++i) os << (i ? ", %" : " %") << op.operands[i];
    }
    os << " : " << values[op.result].shape.str() << "\n";
  }
  os << "  return";
  for (size_t i = 0; i < outputs.size(); ++i) os << (i ? ", %" : " %") << outputs[i];
  os << "\n}\n";
  return os.str();
}

// ------------------------------------------------------------------ tile-dialect spelling
//
// The text plaidml_program_repr returns in the reference is the printed MLIR module of the `tile`
// dialect (plaidml/core/ffi.cc: program repr -> module print); its tests match that text with
// FileCheck patterns (plaidml/edsl/tests/edsl_test.cc).  This printer spells the bounded program
// the same way: module / func @main, one `tile.constant` per distinct scalar literal, eltwise ops as
// `tile.<op> %a, %b : (types) -> type`, contractions with their initial value as first operand and
// the accesses as affine maps (constraints as an affine set).

namespace {

std::string mlirFloat(double v) {
  if (std::isinf(v)) return v < 0 ? "0xFFF0000000000000" : "0x7FF0000000000000";
  if (std::isnan(v)) return "0x7FF8000000000000";
  // MLIR's spelling: six decimals when the value has at most six significant digits, else the shortest
  // digits that read back exactly (scientific, capital E, for small and large exponents)
  char buf[64];
  std::snprintf(buf, sizeof buf, "%.5e", v);
  if (std::strtod(buf, nullptr) == v) {
    std::snprintf(buf, sizeof buf, "%e", v);
    return buf;
  }
  for (int prec = 6; prec <= 17; ++prec) {
    std::snprintf(buf, sizeof buf, "%.*E", prec, v);
    if (std::strtod(buf, nullptr) == v) break;
  }
  std::string t(buf);
  const size_t e = t.find('E');
  const std::string mant = t.substr(0, e);
  const int exponent = std::atoi(t.substr(e + 1).c_str());
  if (exponent >= -3 && exponent <= 15) {
    std::snprintf(buf, sizeof buf, "%.*f", std::max(0, static_cast<int>(mant.size()) - 2 - (mant[0] == '-' ? 1 : 0) - exponent), v);
    if (std::strtod(buf, nullptr) == v) return buf;
  }
  return mant + "E" + (exponent >= 0 ? "+" : "") + std::to_string(exponent);
}

std::string mlirAffine(const Affine& a) {
  // common denominator d: (sum of integer terms) floordiv d
  int64_t den = a.constant.den;
  auto lcm = [](int64_t x, int64_t y) {
    int64_t g = x, h = y;
    while (h) { const int64_t t = g % h; g = h; h = t; }
    return x / g * y;
  };
  for (const Rational& c : a.coef) if (!c.isZero()) den = lcm(den, c.den);
  std::ostringstream os;
  bool any = false;
  for (size_t i = 0; i < a.coef.size(); ++i) {
    if (a.coef[i].isZero()) continue;
    int64_t k = a.coef[i].num * (den / a.coef[i].den);
    if (any) os << (k < 0 ? " - " : " + ");
    else if (k < 0) os << "-";
    const int64_t mag = k < 0 ? -k : k;
    os << "d" << i;
    if (mag != 1) os << " * " << mag;
    any = true;
  }
  const int64_t k0 = a.constant.num * (den / a.constant.den);
  if (k0 != 0 || !any) {
    if (any) os << (k0 < 0 ? " - " : " + ") << (k0 < 0 ? -k0 : k0);
    else os << k0;
  }
  if (den == 1) return os.str();
  return "(" + os.str() + ") floordiv " + std::to_string(den);
}

std::string mlirDims(size_t n) {
  std::string out = "(";
  for (size_t i = 0; i < n; ++i) out += (i ? ", d" : "d") + std::to_string(i);
  return out + ")";
}

std::string mlirMap(const std::vector<Affine>& exprs, size_t n) {
  std::string out = "affine_map<" + mlirDims(n) + " -> (";
  for (size_t d = 0; d < exprs.size(); ++d) out += (d ? ", " : "") + mlirAffine(exprs[d]);
  return out + ")>";
}

// value of a rank-0 constant buffer / literal as (is float, f, i)
struct Scalar {
  bool isFloat = false;
  double f = 0;
  int64_t i = 0;
};

Scalar scalarOf(const PValue& v) {
  Scalar out;
  if (v.kind == PValue::LiteralValue) {
    out.isFloat = v.literal.kind == Literal::Float;
    out.f = v.literal.f;
    out.i = v.literal.kind == Literal::Unsigned ? static_cast<int64_t>(v.literal.u) : v.literal.i;
    return out;
  }
  const char* p = v.constant->data();
  switch (v.shape.dtype) {
    case DType::f16: { uint16_t h; std::memcpy(&h, p, 2); out.isFloat = true; out.f = f16ToF32(h); break; }
    case DType::bf16: { uint16_t h; std::memcpy(&h, p, 2); out.isFloat = true; out.f = bf16ToF32(h); break; }
    case DType::f32: { float f; std::memcpy(&f, p, 4); out.isFloat = true; out.f = f; break; }
    case DType::f64: { std::memcpy(&out.f, p, 8); out.isFloat = true; break; }
    case DType::i1: case DType::ui8: { uint8_t x; std::memcpy(&x, p, 1); out.i = x; break; }
    case DType::si8: { int8_t x; std::memcpy(&x, p, 1); out.i = x; break; }
    case DType::si16: { int16_t x; std::memcpy(&x, p, 2); out.i = x; break; }
    case DType::ui16: { uint16_t x; std::memcpy(&x, p, 2); out.i = x; break; }
    case DType::si32: { int32_t x; std::memcpy(&x, p, 4); out.i = x; break; }
    case DType::ui32: { uint32_t x; std::memcpy(&x, p, 4); out.i = x; break; }
    default: { std::memcpy(&out.i, p, 8); break; }
  }
  return out;
}

}  // namespace

std::string Program::mlir() const {
  static const char* aggNames[] = {"assign", "add", "max", "min", "mul"};
  static const char* comboNames[] = {"none", "add", "cond", "eq", "mul"};
  std::ostringstream head;
  size_t nargs = 0, nres = 0, ncst = 0, nprng = 0;

  // One region of the printed program: the function body or the body of a layer.  Names are per region
  // (a layer's body sees only its block arguments and what it defines itself).
  struct Region {
    std::map<int, std::string> local;              // value id -> SSA name inside this region
    std::map<std::string, std::string> cstByText;  // scalar constants defined at the top of this region
    std::ostringstream csts, body;
    std::string indent;
  };

  Region top;
  top.indent = "    ";
  head << "module @" << name << " {\n  func @main(";
  for (int id : inputs) {
    top.local[id] = "%arg" + std::to_string(nargs);
    head << (nargs ? ", " : "") << top.local[id] << ": " << values[id].shape.str();
    ++nargs;
  }
  for (int id : constants) {
    const PValue& v = values[id];
    if (v.kind == PValue::InternalConstant && v.shape.sizes.empty()) continue;   // a literal: tile.constant below
    top.local[id] = "%arg" + std::to_string(nargs);
    head << (nargs ? ", " : "") << top.local[id] << ": " << v.shape.str() << " {stdx.const}";
    ++nargs;
  }
  head << ") -> ";
  if (outputs.size() != 1) head << "(";
  for (size_t i = 0; i < outputs.size(); ++i) head << (i ? ", " : "") << values[outputs[i]].shape.str();
  if (outputs.size() != 1) head << ")";
  head << " {\n";

  // scalar constants: one per distinct (value, type) and region, all defined before the region's first op
  auto constantName = [&](Region& rg, const std::string& text) {
    auto it = rg.cstByText.find(text);
    if (it != rg.cstByText.end()) return it->second;
    const std::string nm = ncst == 0 ? "%cst" : "%cst_" + std::to_string(ncst - 1);
    ++ncst;
    rg.cstByText.emplace(text, nm);
    rg.csts << rg.indent << nm << " = " << text << "\n";
    return nm;
  };
  auto scalarText = [&](const Scalar& sc, DType dt) {
    std::string t = "tile.constant(";
    if (sc.isFloat || isFloat(dt)) t += mlirFloat(sc.isFloat ? sc.f : static_cast<double>(sc.i)) + " : f64";
    else t += std::to_string(sc.i) + " : i64";
    return t + ") : " + TensorShape(dt).str();
  };
  auto use = [&](Region& rg, int id) -> std::string {
    auto it = rg.local.find(id);
    if (it != rg.local.end()) return it->second;
    const PValue& v = values[id];
    std::string nm;
    if (v.kind == PValue::LiteralValue || (v.kind == PValue::InternalConstant && v.shape.sizes.empty())) {
      nm = constantName(rg, scalarText(scalarOf(v), v.shape.dtype));
    } else if (v.kind == PValue::InternalConstant) {
      // a tensor the builder computed from shapes alone (index, shape): a dense constant
      std::string t = "tile.constant(dense<" + std::string(v.name.empty() ? "..." : v.name) + "> : " + v.shape.str() + ") : " +
                      v.shape.str();
      nm = constantName(rg, t);
    } else {
      nm = "%<undefined " + std::to_string(id) + ">";   // (the builder rejects programs that would get here)
    }
    rg.local[id] = nm;
    return nm;
  };
  auto identity = [&](Region& rg, AggKind agg, DType dt) {
    Scalar sc;
    sc.isFloat = isFloat(dt);
    const size_t bits = dtypeBytes(dt) * 8;
    const bool sgn = isSignedInt(dt);
    switch (agg) {
      case AggKind::mul: sc.f = 1.0; sc.i = 1; break;
      case AggKind::max:
        sc.f = -std::numeric_limits<double>::infinity();
        sc.i = sgn ? (bits >= 64 ? std::numeric_limits<int64_t>::min() : -(int64_t{1} << (bits - 1))) : 0;
        break;
      case AggKind::min:
        sc.f = std::numeric_limits<double>::infinity();
        sc.i = bits >= 64 ? std::numeric_limits<int64_t>::max()
                          : (sgn ? (int64_t{1} << (bits - 1)) - 1 : (int64_t{1} << bits) - 1);
        break;
      default: break;
    }
    return constantName(rg, scalarText(sc, dt));
  };

  auto printOp = [&](Region& rg, const POp& op) {
    std::ostringstream& body = rg.body;
    std::vector<std::string> args;
    if (op.kind == POp::Contraction) {
      const BoundedContraction& c = *op.c;
      const size_t nsrc = op.operands.size() - (c.hasInit ? 1 : 0);
      const std::string init = c.hasInit ? use(rg, op.operands.back()) : identity(rg, c.agg, values[op.result].shape.dtype);
      for (size_t i = 0; i < nsrc; ++i) args.push_back(use(rg, op.operands[i]));
      rg.local[op.result] = "%" + std::to_string(nres++);
      body << rg.indent << rg.local[op.result] << " = tile.contract " << aggNames[static_cast<int>(c.agg)] << ", "
           << comboNames[static_cast<int>(c.combo)] << ", " << init;
      for (const std::string& a : args) body << ", " << a;
      body << " {";
      if (!c.cons.empty()) {
        body << "cons = affine_set<" << mlirDims(c.nIdx()) << " : (";
        for (size_t k = 0; k < c.cons.size(); ++k) {
          Affine hi = c.cons[k].first;
          for (Rational& r : hi.coef) r = Rational(0) - r;
          hi.constant = Rational(c.cons[k].second - 1) - hi.constant;
          body << (k ? ", " : "") << mlirAffine(c.cons[k].first) << " >= 0, " << mlirAffine(hi) << " >= 0";
        }
        body << ")>, ";
      }
      if (!op.label.empty()) body << "name = \"" << op.label << "\", ";
      body << "sink = " << mlirMap(c.sink, c.nIdx()) << ", srcs = [";
      for (size_t i = 0; i < nsrc; ++i) body << (i ? ", " : "") << mlirMap(c.srcs[i], c.nIdx());
      body << "]} : " << (c.hasInit ? values[op.operands.back()].shape.str() : TensorShape(values[op.result].shape.dtype).str());
      for (size_t i = 0; i < nsrc; ++i) body << ", " << values[op.operands[i]].shape.str();
      body << " -> " << values[op.result].shape.str() << "\n";
      return;
    }
    for (int id : op.operands) args.push_back(use(rg, id));
    if (op.kind == POp::Special) {
      const PSpecial& sp = *op.s;
      if (sp.op == PSpecial::PrngState) return;  // printed with the operation that gives the numbers
      auto types = [&]() {
        body << " : (";
        for (size_t i = 0; i < op.operands.size(); ++i) body << (i ? ", " : "") << values[op.operands[i]].shape.str();
        body << ") -> ";
      };
      if (sp.op == PSpecial::Prng) {
        const POp& tail = ops[sp.pair];
        const std::string suffix = nprng == 0 ? "" : "_" + std::to_string(nprng - 1);
        ++nprng;
        rg.local[op.result] = "%result" + suffix;
        rg.local[tail.result] = "%new_state" + suffix;
        body << rg.indent << rg.local[op.result] << ", " << rg.local[tail.result] << " = tile.prng " << args[0];
        types();
        body << "(" << values[op.result].shape.str() << ", " << values[tail.result].shape.str() << ")\n";
        return;
      }
      rg.local[op.result] = "%" + std::to_string(nres++);
      body << rg.indent << rg.local[op.result] << " = tile." << op.mnemonic << " ";
      if (sp.op == PSpecial::ArgSort) {
        body << (sp.mode ? "desc " : "asc ") << args[0] << "[" << sp.axis << "]";
      } else if (sp.op == PSpecial::Gather) {
        body << args[0] << " " << args[1] << " {OutOfBoundsMode = " << sp.outOfBounds << " : i64, axis = " << sp.axis
             << " : index, batchDims = " << sp.batchDims << " : index, cubeCoeff = " << mlirFloat(sp.cubeCoeff)
             << " : f64, interpolationMode = " << sp.interpolation << " : i64, mode = " << sp.mode
             << " : i64, nearestMode = " << sp.nearest << " : i64}";
      } else {
        body << args[0] << " " << args[1] << " " << args[2] << " {axis = " << sp.axis << " : index, mode = " << sp.mode
             << " : i64}";
      }
      types();
      body << values[op.result].shape.str() << "\n";
      return;
    }
    rg.local[op.result] = "%" + std::to_string(nres++);
    if (op.mnemonic == "pragma") {
      body << rg.indent << rg.local[op.result] << " = tile.pragma " << args[0] << " \"" << op.label << "\" {" << op.attrs
           << "} : " << values[op.result].shape.str() << "\n";
      return;
    }
    body << rg.indent << rg.local[op.result] << " = tile." << op.mnemonic;
    for (size_t i = 0; i < args.size(); ++i) body << (i ? ", " : " ") << args[i];
    body << " : (";
    for (size_t i = 0; i < op.operands.size(); ++i) body << (i ? ", " : "") << values[op.operands[i]].shape.str();
    body << ") -> " << values[op.result].shape.str() << "\n";
  };

  // first operation (in list order) inside a layer or anything nested in it; ops.size() if it has none
  std::vector<size_t> firstOp(layers.size(), ops.size());
  for (size_t i = ops.size(); i-- > 0;) {
    for (int l = ops[i].layer; l >= 0; l = layers[l].parent) firstOp[l] = i;
  }

  // Prints the operations and child layers of region `level` (-1: the function body) in an order in which every
  // value is defined before its use: list order, except that a layer (one item, placed at its first operation)
  // waits for all of its operands.
  std::function<void(Region&, int)> printRegion = [&](Region& rg, int level) {
    struct Item {
      size_t key;
      int op = -1, layer = -1;
      std::vector<int> needs;
      bool done = false;
    };
    std::vector<Item> items;
    std::map<int, size_t> producer;   // value id -> item
    for (size_t i = 0; i < ops.size(); ++i) {
      if (ops[i].layer != level) continue;
      Item it;
      it.key = i;
      it.op = static_cast<int>(i);
      it.needs = ops[i].operands;
      producer[ops[i].result] = items.size();
      items.push_back(std::move(it));
    }
    for (size_t l = 0; l < layers.size(); ++l) {
      if (layers[l].parent != level) continue;
      Item it;
      it.key = firstOp[l];
      it.layer = static_cast<int>(l);
      it.needs = layers[l].operands;
      for (int r : layers[l].results) producer[r] = items.size();
      items.push_back(std::move(it));
    }
    for (size_t printed = 0; printed < items.size(); ++printed) {
      size_t best = items.size();
      for (size_t k = 0; k < items.size(); ++k) {
        if (items[k].done) continue;
        bool ready = true;
        for (int v : items[k].needs) {
          auto pr = producer.find(v);
          if (pr != producer.end() && pr->second != k && !items[pr->second].done) ready = false;
        }
        if (ready && (best == items.size() || items[k].key < items[best].key)) best = k;
      }
      if (best == items.size()) break;   // (a cycle cannot happen in a program the builder made)
      Item& it = items[best];
      it.done = true;
      if (it.op >= 0) {
        printOp(rg, ops[it.op]);
        continue;
      }
      const PLayer& ly = layers[it.layer];
      std::vector<std::string> args;
      for (int v : ly.operands) args.push_back(use(rg, v));
      const std::string box = "%" + std::to_string(nres++);
      Region inner;
      inner.indent = rg.indent + "  ";
      std::ostringstream blockArgs;
      for (size_t k = 0; k < ly.operands.size(); ++k) {
        const std::string an = "%arg" + std::to_string(nargs++);
        if (!inner.local.count(ly.operands[k])) inner.local[ly.operands[k]] = an;
        blockArgs << (k ? ", " : "") << an << ": " << values[ly.operands[k]].shape.str();
      }
      printRegion(inner, it.layer);
      rg.body << rg.indent << box;
      if (ly.results.size() != 1) rg.body << ":" << ly.results.size();
      rg.body << " = layer.box \"" << ly.name << "\"(";
      for (size_t k = 0; k < args.size(); ++k) rg.body << (k ? ", " : "") << args[k];
      rg.body << ") {attrs = {" << ly.attrs << "}} : ";
      for (size_t k = 0; k < ly.operands.size(); ++k) rg.body << (k ? ", " : "") << values[ly.operands[k]].shape.str();
      rg.body << " -> ";
      for (size_t k = 0; k < ly.results.size(); ++k) rg.body << (k ? ", " : "") << values[ly.results[k]].shape.str();
      rg.body << " {\n" << rg.indent << "^bb0(" << blockArgs.str() << "):\n";
      std::ostringstream ret;
      ret << inner.indent << "layer.return";
      for (size_t k = 0; k < ly.results.size(); ++k) ret << (k ? ", " : " ") << use(inner, ly.results[k]);
      if (!ly.results.empty()) ret << " : ";
      for (size_t k = 0; k < ly.results.size(); ++k) ret << (k ? ", " : "") << values[ly.results[k]].shape.str();
      rg.body << inner.csts.str() << inner.body.str() << ret.str() << "\n" << rg.indent << "}\n";
      for (size_t k = 0; k < ly.results.size(); ++k) {
        rg.local[ly.results[k]] = ly.results.size() == 1 ? box : box + "#" + std::to_string(k);
      }
    }
  };
  printRegion(top, -1);

  std::ostringstream tail;
  tail << "    return";
  for (size_t i = 0; i < outputs.size(); ++i) tail << (i ? ", " : " ") << use(top, outputs[i]);
  if (!outputs.empty()) tail << " : ";
  for (size_t i = 0; i < outputs.size(); ++i) tail << (i ? ", " : "") << values[outputs[i]].shape.str();
  tail << "\n  }\n}\n";
  return head.str() + top.csts.str() + top.body.str() + tail.str();
}

// ------------------------------------------------------------------ builder

namespace {

class Builder {
 public:
  explicit Builder(Program* p) : prog_(p) {}

  int addValue(PValue v) {
    prog_->values.push_back(std::move(v));
    return static_cast<int>(prog_->values.size()) - 1;
  }

  int lower(const ExprPtr& e) {
    auto it = memo_.find(e.get());
    if (it != memo_.end()) return it->second;
    // operations emitted for this node belong to the layer that was open when the node was made
    const int saved = layer_;
    layer_ = e->parent ? layerOf(e->parent) : -1;
    const int id = lowerNode(e);
    layer_ = saved;
    memo_[e.get()] = id;
    return id;
  }

  // Index of the layer record of a Layer node (made on first use, enclosing layers first).
  int layerOf(const ExprPtr& node) {
    auto it = layerIds_.find(node.get());
    if (it != layerIds_.end()) return it->second;
    const int parent = node->parent ? layerOf(node->parent) : -1;
    const int id = static_cast<int>(prog_->layers.size());
    layerIds_[node.get()] = id;
    layerNodes_.push_back(node);
    PLayer rec;
    rec.name = node->op;
    rec.parent = parent;
    bool first = true;
    for (const auto& kv : node->attrs) {
      rec.attrs += (first ? "" : ", ") + kv.first + " = ";
      const VarPtr& v = kv.second;
      if (v && v->kind == VarNode::Str) rec.attrs += "\"" + v->s + "\"";
      else if (v && v->kind == VarNode::Int) rec.attrs += std::to_string(v->i) + " : i64";
      else if (v && v->kind == VarNode::Float) rec.attrs += std::to_string(v->f) + " : f64";
      else rec.attrs += v ? v->str() : "unit";
      first = false;
    }
    prog_->layers.push_back(std::move(rec));
    // operands are values of the enclosing region (lowered there), literals become tensors of their own
    std::vector<int> operands;
    for (const ExprPtr& o : node->operands) {
      int v = lower(o);
      if (prog_->values[v].kind == PValue::LiteralValue) v = materialise(v, prog_->values[v].shape.dtype);
      operands.push_back(v);
    }
    prog_->layers[id].operands = std::move(operands);
    return id;
  }

  // After all outputs are lowered: the layers' result values, and the check that a layer's body reads nothing
  // of the regions around it except through its operands (the reference's layer.box is isolated from above;
  // a body that uses a tensor not listed as an operand is rejected when the program is built).
  void finishLayers() {
    for (size_t l = 0; l < layerNodes_.size(); ++l) {
      std::vector<int> results;
      for (const ExprPtr& r : layerNodes_[l]->results) results.push_back(lower(r));
      prog_->layers[l].results = std::move(results);
    }
    auto inside = [&](int inner, int outer) {   // is region `inner` the region `outer` or nested in it
      for (int l = inner; l >= 0; l = prog_->layers[l].parent) {
        if (l == outer) return true;
      }
      return outer == -1;
    };
    auto visible = [&](int v, int level) {
      const PValue& pv = prog_->values[v];
      if (pv.kind == PValue::LiteralValue || (pv.kind == PValue::InternalConstant)) return true;
      if (level < 0) return true;
      const PLayer& ly = prog_->layers[level];
      if (std::find(ly.operands.begin(), ly.operands.end(), v) != ly.operands.end()) return true;
      if (pv.def < 0) return false;                       // a program argument that is not an operand
      const int defLevel = prog_->ops[pv.def].layer;
      if (defLevel == level) return true;
      // the result of a layer nested directly or deeper: visible only as a result of a child of `level`
      for (int l = defLevel; l >= 0; l = prog_->layers[l].parent) {
        if (prog_->layers[l].parent == level) {
          const std::vector<int>& rs = prog_->layers[l].results;
          return std::find(rs.begin(), rs.end(), v) != rs.end();
        }
      }
      return false;
    };
    (void)inside;
    for (const POp& op : prog_->ops) {
      if (op.layer < 0) continue;
      for (int v : op.operands) {
        if (!visible(v, op.layer)) {
          throw std::runtime_error("Layer '" + prog_->layers[op.layer].name + "' uses a tensor that is not among its operands" +
                                   (prog_->values[v].name.empty() ? "" : " ('" + prog_->values[v].name + "')"));
        }
      }
    }
    for (size_t l = 0; l < prog_->layers.size(); ++l) {
      for (int v : prog_->layers[l].results) {
        if (!visible(v, static_cast<int>(l))) {
          throw std::runtime_error("Layer '" + prog_->layers[l].name + "' returns a tensor that is not among its operands");
        }
      }
    }
  }

  void bindInput(const ExprPtr& e, const TensorShape* shape) {
    if (e->kind == ExprNode::ConstTensor && shape == nullptr) {
      // A constant tensor listed among the inputs (networks/oplib/resnet50.cc:317-319 of the reference passes
      // its weight constants that way): it takes an argument slot of its shape, which plaidml_executable_run
      // expects a buffer for, but the program computes with the constant's own data -- in the reference the
      // constant's second registration as a constant argument replaces the first (pmlc/ast/builder.cc:495-542).
      PValue v;
      v.kind = PValue::Input;
      v.shape = e->buffer->shape();
      v.name = e->name;
      prog_->inputs.push_back(addValue(v));
      return;
    }
    if (e->kind != ExprNode::Input) throw std::runtime_error("Program inputs must be input placeholders");
    if (shape && *shape != e->shape) e->shape = *shape;
    PValue v;
    v.kind = PValue::Input;
    v.shape = e->shape;
    v.name = e->name;
    const int id = addValue(v);
    memo_[e.get()] = id;
    prog_->inputs.push_back(id);
  }

  int emit(POp op, const TensorShape& shape) {
    PValue v;
    v.kind = PValue::Temp;
    v.shape = shape;
    v.shape.strides.clear();
    v.name = op.label;
    v.def = static_cast<int>(prog_->ops.size());
    op.layer = layer_;
    op.result = addValue(v);
    prog_->ops.push_back(std::move(op));
    return prog_->ops.back().result;
  }

  // A literal operand becomes a rank-0 internal constant of `dtype`.
  int materialise(int id, DType dtype) {
    const PValue& v = prog_->values[id];
    if (v.kind != PValue::LiteralValue) return id;
    PValue c;
    c.kind = PValue::InternalConstant;
    c.constant = makeScalarConstant(dtype, v.literal);
    c.shape = c.constant->shape();
    c.name = "literal";
    return addValue(c);
  }

  Evaluator ev;

 private:
  int layer_ = -1;                                          // layer of the node being lowered
  std::unordered_map<const ExprNode*, int> layerIds_;
  std::vector<ExprPtr> layerNodes_;

  int literal(const ExprPtr& e, Literal lit, DType dt) {
    (void)e;
    PValue v;
    v.kind = PValue::LiteralValue;
    v.shape = TensorShape(dt);
    v.literal = lit;
    return addValue(v);
  }

  int lowerNode(const ExprPtr& e) {
    switch (e->kind) {
      case ExprNode::Input:
        throw std::runtime_error("Input '" + e->name + "' is used by the program but was not listed among its inputs");
      case ExprNode::ConstTensor: {
        PValue v;
        v.kind = PValue::Constant;
        v.constant = e->buffer;
        v.shape = e->buffer->shape();
        v.name = e->name;
        const int id = addValue(v);
        prog_->constants.push_back(id);
        return id;
      }
      case ExprNode::ConstSigned: {
        Literal l;
        l.kind = Literal::Signed;
        l.i = e->ivalue;
        return literal(e, l, DType::six);
      }
      case ExprNode::ConstUnsigned: {
        Literal l;
        l.kind = Literal::Unsigned;
        l.u = e->uvalue;
        return literal(e, l, DType::uix);
      }
      case ExprNode::ConstFloat: {
        Literal l;
        l.kind = Literal::Float;
        l.f = e->fvalue;
        return literal(e, l, DType::fx);
      }
      case ExprNode::Dim: {
        Literal l;
        l.kind = Literal::Signed;
        l.i = ev.evaluate(e->dim);
        return literal(e, l, DType::six);
      }
      case ExprNode::Pragma: {
        // kept as an operation (tile.pragma), run as a copy of its operand (pmlc/ast/builder.cc:768-780)
        const int src = lower(e->expr);
        POp op;
        op.kind = POp::Eltwise;
        op.mnemonic = "pragma";
        op.label = e->op;
        bool first = true;
        for (const auto& kv : e->attrs) {
          op.attrs += (first ? "" : ", ") + kv.first + " = ";
          const VarPtr& v = kv.second;
          if (v && v->kind == VarNode::Str) op.attrs += "\"" + v->s + "\"";
          else if (v && v->kind == VarNode::Int) op.attrs += std::to_string(v->i) + " : i64";
          else if (v && v->kind == VarNode::Float) op.attrs += std::to_string(v->f) + " : f64";
          else op.attrs += v ? v->str() : "unit";
          first = false;
        }
        op.operands = {materialise(src, prog_->values[src].shape.dtype)};
        return emit(op, prog_->values[op.operands[0]].shape);
      }
      case ExprNode::Element: {
        const ExprPtr& src = e->expr;
        if (src->kind == ExprNode::Layer) {
          if (e->ordinal >= src->results.size()) throw std::runtime_error("Out of bounds element ordinal");
          return lower(src->results[e->ordinal]);
        }
        if (src->kind == ExprNode::Intrinsic && src->op == "prng") {
          if (e->ordinal > 1) throw std::runtime_error("Out of bounds element ordinal");
          const int numbers = lower(src);
          if (e->ordinal == 0) return numbers;
          return prog_->ops[prog_->ops[prog_->values[numbers].def].s->pair].result;
        }
        if (e->ordinal == 0) return lower(src);
        throw std::runtime_error("Out of bounds element ordinal");
      }
      case ExprNode::Layer:
        if (e->results.size() == 1) return lower(e->results[0]);
        throw std::runtime_error("Missing element needed to resolve multiple results.");
      case ExprNode::Cast: {
        const int src = lower(e->expr);
        const TensorShape shape = ev.getShape(e);
        if (prog_->values[src].kind == PValue::LiteralValue) return materialise(src, e->dtype);
        if (prog_->values[src].shape.dtype == e->dtype) return src;
        POp op;
        op.kind = POp::Cast;
        op.mnemonic = "cast";
        op.operands = {src};
        return emit(op, shape);
      }
      case ExprNode::Contraction: return lowerContraction(e);
      case ExprNode::Intrinsic: return lowerIntrinsic(e);
    }
    throw std::runtime_error("Invalid expression node");
  }

  int lowerContraction(const ExprPtr& e) {
    const TensorShape outShape = ev.getShape(e);
    auto c = std::make_shared<BoundedContraction>();
    c->agg = e->agg;
    c->combo = e->combo;
    const size_t need = e->combo == ComboKind::none ? 1 : (e->combo == ComboKind::cond ? 3 : 2);
    if (e->srcs.size() != need) {
      throw std::runtime_error("Contraction '" + e->name + "' has " + std::to_string(e->srcs.size()) +
                               " operands but its combination takes " + std::to_string(need));
    }
    IndexNumbering idxs;
    for (const PolyPtr& p : e->sinkIdxs) c->sink.push_back(evalPoly(p, &idxs, &ev));
    std::vector<TensorShape> srcShapes;
    POp op;
    op.kind = POp::Contraction;
    op.mnemonic = "contract";
    op.label = e->name;
    for (const PolyMap& src : e->srcs) {
      std::vector<Affine> forms;
      for (const PolyPtr& p : src.idxs) forms.push_back(evalPoly(p, &idxs, &ev));
      c->srcs.push_back(std::move(forms));
      const int id = lower(src.ref);
      if (prog_->values[id].kind == PValue::LiteralValue) {
        throw std::runtime_error("'contraction' operand data type is ambiguous, use a cast");
      }
      srcShapes.push_back(prog_->values[id].shape);
      op.operands.push_back(id);
    }
    for (const Constraint& con : e->constraints) {
      c->cons.emplace_back(evalPoly(con.lhs, &idxs, &ev), ev.evaluate(con.rhs));
    }
    c->idxNames = idxs.names();
    const size_t n = c->nIdx();
    for (Affine& a : c->sink) a.resize(n);
    for (auto& forms : c->srcs) {
      for (Affine& a : forms) a.resize(n);
    }
    for (auto& con : c->cons) con.first.resize(n);
    computeBounds(c.get(), outShape, srcShapes);
    if (e->init) {
      int init = lower(e->init);
      init = materialise(init, outShape.dtype);
      const TensorShape& is = prog_->values[init].shape;
      // the initial value must broadcast to the output shape
      std::vector<TensorShape> both = {outShape, is};
      if (inferShape(both).sizes != outShape.sizes) throw std::runtime_error("Contraction initial value does not broadcast to the result shape");
      c->hasInit = true;
      op.operands.push_back(init);
    }
    op.c = c;
    return emit(op, outShape);
  }

  int lowerIntrinsic(const ExprPtr& e) {
    const std::string& name = e->op;
    if (name == "prng") return lowerSpecial(e, TensorShape());  // (two results: it reads both shapes itself)
    const TensorShape shape = ev.getShape(e);
    if (name == "index") {
      int64_t axis = 0;
      if (!getIntegerValue(&ev, e->operands[0], &axis) || axis < 0) {
        throw std::runtime_error("'index' requires a valid axis");
      }
      // depends on the shape only: computed here, uploaded once with the executable
      BufferPtr buf = Buffer::allocate(shape);
      int32_t* p = reinterpret_cast<int32_t*>(buf->data());
      const std::vector<int64_t> st = shape.denseStrides();
      // (an axis past the last dimension is accepted when the program is built, as by the reference --
      // plaidml/edsl/tests/edsl_test.cc IndexOp builds index({X0}, 1); there is one position along it: 0)
      const bool inside = static_cast<size_t>(axis) < shape.rank();
      for (int64_t i = 0; i < shape.elements(); ++i) {
        p[i] = inside ? static_cast<int32_t>((i / st[axis]) % shape.sizes[axis]) : 0;
      }
      PValue v;
      v.kind = PValue::InternalConstant;
      v.constant = buf;
      v.shape = shape;
      v.name = "index";
      return addValue(v);
    }
    if (name == "shape") {
      const TensorShape src = ev.getShape(e->operands[0]);
      BufferPtr buf = Buffer::allocate(shape);
      int32_t* p = reinterpret_cast<int32_t*>(buf->data());
      for (size_t i = 0; i < src.rank(); ++i) p[i] = static_cast<int32_t>(src.sizes[i]);
      PValue v;
      v.kind = PValue::InternalConstant;
      v.constant = buf;
      v.shape = shape;
      v.name = "shape";
      const int id = addValue(v);
      // kept as an operation of the printed program (tile.shape); its value is known here, so nothing runs for it
      POp op;
      op.kind = POp::Eltwise;
      op.mnemonic = "shape";
      op.operands = {lower(e->operands[0])};
      op.result = id;
      prog_->values[id].def = static_cast<int>(prog_->ops.size());
      prog_->ops.push_back(op);
      return id;
    }
    if (name == "reshape") {
      const int src = lower(e->operands[0]);
      if (prog_->values[src].shape.elements() != shape.elements()) {
        throw std::runtime_error("'reshape' changes the number of elements");
      }
      // reshape(x, x.shape) is x (pmlc/dialect/tile/ir/ops.cc:88-94)
      if (prog_->values[src].shape.sizes == shape.sizes && prog_->values[src].shape.dtype == shape.dtype) return src;
      POp op;
      op.kind = POp::Reshape;
      op.mnemonic = "reshape";
      op.label = e->name;
      op.operands = {src};
      return emit(op, shape);
    }
    if (name == "argsort" || name == "gather" || name == "scatter") return lowerSpecial(e, shape);
    // element-wise
    std::vector<int> ids;
    DType promoted = DType::invalid;
    for (const ExprPtr& o : e->operands) {
      const int id = lower(o);
      ids.push_back(id);
      promoted = promote(promoted, prog_->values[id].shape.dtype);
    }
    if (name == "select" && ids.size() == 3) {
      // the condition keeps its type; the branches are promoted together
      promoted = promote(prog_->values[ids[1]].shape.dtype, prog_->values[ids[2]].shape.dtype);
      ids[0] = materialise(ids[0], DType::i1);
      ids[1] = materialise(ids[1], promoted);
      ids[2] = materialise(ids[2], promoted);
    } else {
      for (int& id : ids) id = materialise(id, promoted);
    }
    // commutative operations keep a scalar constant on the right, as MLIR's folder leaves them in the
    // reference (pmlc/dialect/tile/ir/eltwise.td: the ops marked Commutative)
    static const char* const kCommutative[] = {"add", "mul", "max", "min", "cmp_eq", "cmp_ne", "bit_and", "bit_or",
                                               "bit_xor", "logical_and", "logical_or", "logical_xor"};
    if (ids.size() == 2 && std::find(std::begin(kCommutative), std::end(kCommutative), name) != std::end(kCommutative)) {
      auto scalarConstant = [&](int id) {
        const PValue& v = prog_->values[id];
        return v.kind == PValue::LiteralValue || (v.kind == PValue::InternalConstant && v.shape.sizes.empty());
      };
      if (scalarConstant(ids[0]) && !scalarConstant(ids[1])) std::swap(ids[0], ids[1]);
    }
    POp op;
    op.kind = POp::Eltwise;
    op.mnemonic = name;
    op.label = e->name;
    op.operands = ids;
    TensorShape result = shape;
    if (isAmbiguous(result.dtype)) {
      result.dtype = result.dtype == DType::fx ? DType::f32 : (result.dtype == DType::six ? DType::si32 : DType::ui32);
    }
    return emit(op, result);
  }

  int tensorOperand(const ExprPtr& e, const std::string& op) {
    const int id = lower(e);
    if (prog_->values[id].kind == PValue::LiteralValue) {
      throw std::runtime_error("'" + op + "' needs tensors, not scalar constants, as its data operands");
    }
    return id;
  }

  // argsort / gather / scatter / prng; the operands after the tensors are compile-time constants
  // (pmlc/ast/builder.cc:685-690 and the make*Op functions they name).
  int lowerSpecial(const ExprPtr& e, const TensorShape& shape) {
    const std::string& name = e->op;
    auto constant = [&](size_t i) {
      int64_t v = 0;
      getIntegerValue(&ev, e->operands[i], &v);
      return v;
    };
    POp op;
    op.kind = POp::Special;
    op.mnemonic = name;
    op.label = e->name;
    op.s = std::make_shared<PSpecial>();
    if (name == "argsort") {
      op.s->op = PSpecial::ArgSort;
      op.s->axis = constant(1);
      op.s->mode = constant(2);
      const int64_t rank = static_cast<int64_t>(shape.rank());
      if (op.s->axis < -rank || op.s->axis >= rank) throw std::runtime_error("'argsort' axis is outside the tensor's dimensions");
      if (op.s->mode != 0 && op.s->mode != 1) throw std::runtime_error("'argsort' direction must be 0 (asc) or 1 (desc)");
      op.operands = {tensorOperand(e->operands[0], name)};
      return emit(op, shape);
    }
    if (name == "gather") {
      op.s->op = PSpecial::Gather;
      op.s->axis = constant(2);
      op.s->interpolation = constant(3);
      op.s->nearest = constant(4);
      op.s->cubeCoeff = e->operands[5]->fvalue;
      op.s->mode = constant(6);
      op.s->batchDims = constant(7);
      op.s->outOfBounds = constant(8);
      op.operands = {tensorOperand(e->operands[0], name), tensorOperand(e->operands[1], name)};
      return emit(op, shape);
    }
    if (name == "scatter") {
      op.s->op = PSpecial::Scatter;
      op.s->axis = constant(3);
      op.s->mode = constant(4);
      op.operands = {tensorOperand(e->operands[0], name), tensorOperand(e->operands[1], name),
                     tensorOperand(e->operands[2], name)};
      const DType dt = prog_->values[op.operands[0]].shape.dtype;
      if (prog_->values[op.operands[2]].shape.dtype != dt) {
        throw std::runtime_error("'scatter' needs data and updates of one element type, use a cast");
      }
      return emit(op, shape);
    }
    // prng: two operations over the same state
    const std::vector<TensorShape> both = ev.getShapes(e.get());
    const int state = tensorOperand(e->operands[0], name);
    const TensorShape st = prog_->values[state].shape;
    if (st.dtype != DType::ui32 && st.dtype != DType::si32) throw std::runtime_error("'prng' needs a state of 32-bit integers");
    if (st.elements() < 3) throw std::runtime_error("'prng' needs a state of at least three words");
    op.s->op = PSpecial::Prng;
    op.operands = {state};
    const int numbers = emit(op, both[0]);
    const int first = prog_->values[numbers].def;
    POp tail;
    tail.kind = POp::Special;
    tail.mnemonic = "prng_state";
    tail.s = std::make_shared<PSpecial>();
    tail.s->op = PSpecial::PrngState;
    tail.s->pair = first;
    tail.s->dims = both[0].sizes;
    tail.operands = {state};
    const int after = emit(tail, both[1]);
    prog_->ops[first].s->pair = prog_->values[after].def;
    return numbers;
  }

  Program* prog_;
  std::unordered_map<const ExprNode*, int> memo_;
};

}  // namespace

std::shared_ptr<Program> buildProgram(const std::string& name, const std::vector<ExprPtr>& inputs,
                                      const std::vector<const TensorShape*>& shapes,
                                      const std::vector<ExprPtr>& outputs) {
  auto prog = std::make_shared<Program>();
  prog->name = name;
  Builder b(prog.get());
  for (size_t i = 0; i < inputs.size(); ++i) b.bindInput(inputs[i], i < shapes.size() ? shapes[i] : nullptr);
  std::vector<int> seen;
  for (const ExprPtr& out : outputs) {
    int id = b.lower(out);
    const PValue::Kind kind = prog->values[id].kind;
    if (kind == PValue::LiteralValue) id = b.materialise(id, prog->values[id].shape.dtype);
    const bool dup = std::find(seen.begin(), seen.end(), id) != seen.end();
    const int def = prog->values[id].def;
    const bool view = def >= 0 && prog->ops[def].kind == POp::Reshape;
    if (prog->values[id].kind != PValue::Temp || dup || view) {
      // outputs are distinct buffers written by the program: an argument, a reshaped view or a value returned
      // twice is copied by an ident (pmlc/ast/builder.cc:580-593)
      POp op;
      op.kind = POp::Eltwise;
      op.mnemonic = "ident";
      op.operands = {id};
      id = b.emit(op, prog->values[id].shape);
    }
    seen.push_back(id);
    prog->outputs.push_back(id);
  }
  b.finishLayers();
  return prog;
}

}  // namespace pml
