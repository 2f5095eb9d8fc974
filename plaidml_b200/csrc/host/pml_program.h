// The flat program `plaidml_build` produces from an expression tree, and its builder.
//
// It plays the role of the reference's `tile` dialect module (pmlc/ast/builder.cc:303-624,
// pmlc/dialect/tile/ir/ops.td:20-83) without MLIR: a list of values and operations in
// definition order.  Contractions are stored already bounded (the job of the reference's
// tile-compute-bounds pass, pmlc/dialect/tile/transforms/contraction.cc:657-681): every
// index variable has a range and every access is an affine form over the variables.
#pragma once

#include <memory>
#include <string>
#include <unordered_map>
#include <vector>

#include "pml_ast.h"

namespace pml {

struct Rational {
  int64_t num = 0;
  int64_t den = 1;
  Rational() = default;
  Rational(int64_t n) : num(n) {}  // NOLINT
  Rational(int64_t n, int64_t d);
  bool isZero() const { return num == 0; }
  bool isInt() const { return den == 1; }
};
Rational operator+(Rational a, Rational b);
Rational operator-(Rational a, Rational b);
Rational operator*(Rational a, Rational b);
Rational operator/(Rational a, Rational b);

// constant + sum_i coef[i] * x_i
struct Affine {
  std::vector<Rational> coef;
  Rational constant;
  explicit Affine(size_t n = 0) : coef(n) {}
  void resize(size_t n) { if (coef.size() < n) coef.resize(n); }
};

struct BoundedContraction {
  AggKind agg = AggKind::assign;
  ComboKind combo = ComboKind::none;
  std::vector<std::string> idxNames;
  std::vector<int64_t> lower;   // first value of each index variable
  std::vector<int64_t> extent;  // number of values
  std::vector<Affine> sink;                      // one per output dim, in terms of x (not shifted)
  std::vector<std::vector<Affine>> srcs;         // [operand][dim]
  std::vector<std::pair<Affine, int64_t>> cons;  // 0 <= form < bound
  bool hasInit = false;
  size_t nIdx() const { return idxNames.size(); }
};

struct Literal {
  enum Kind { Signed, Unsigned, Float } kind = Signed;
  int64_t i = 0;
  uint64_t u = 0;
  double f = 0;
};

struct PValue {
  enum Kind { Input, Constant, InternalConstant, Temp, LiteralValue } kind = Temp;
  TensorShape shape;
  std::string name;
  BufferPtr constant;   // Constant / InternalConstant
  Literal literal;      // LiteralValue (never materialised; consumers fold it)
  int def = -1;         // defining op, -1 for arguments
};

// gather / scatter / argsort / prng: the tile operations that are not contractions
// (pmlc/dialect/tile/ir/ops.td:97-191).  prng, the one operation with two results, is kept as two operations that
// read the same state: Prng gives the numbers, PrngState the state after them; they print as one `tile.prng`.
struct PSpecial {
  enum Op { Gather, Scatter, ArgSort, Prng, PrngState } op = Gather;
  int64_t axis = 0;           // argsort: as written (negative counts from the end)
  int64_t mode = 0;           // gather: 0 along an axis, 1 nd; scatter: ScatterMode; argsort: 0 ascending, 1 descending
  int64_t batchDims = 0, interpolation = 3, nearest = 0, outOfBounds = 0;
  double cubeCoeff = -0.75;
  int pair = -1;              // Prng: the PrngState operation; PrngState: the Prng operation
  std::vector<int64_t> dims;  // PrngState: shape of the numbers generated
};

struct POp {
  enum Kind { Contraction, Eltwise, Cast, Reshape, Special } kind = Eltwise;
  std::shared_ptr<PSpecial> s;  // Special
  std::string mnemonic;  // eltwise op name ("add", "relu", ...), "cast", "reshape", "contract", "gather", ...
  std::string label;     // user-given name (contraction / layer name); the pragma's name for "pragma"
  std::string attrs;     // "pragma": its attributes as printed, e.g. msg = "text"
  std::vector<int> operands;  // value ids; for contractions: sources then the init (if any)
  int result = -1;
  int layer = -1;        // innermost enclosing layer (index into Program::layers), -1 at function level
  std::shared_ptr<BoundedContraction> c;
};

// A named region of the program (edsl `layer(...)`, pmlc/ast/builder.cc:704-762): the operations built while the
// layer was open, isolated from the values around them except for its operands.  Execution ignores layers (the
// operation list is flat); the printed program shows them as `layer.box` regions.
struct PLayer {
  std::string name;
  std::string attrs;          // as printed inside {attrs = {...}}
  int parent = -1;            // enclosing layer
  std::vector<int> operands;  // values of the enclosing region, in the order given (block arguments)
  std::vector<int> results;   // values of the body returned by the layer
};

struct Program {
  std::string name;
  std::vector<PValue> values;
  std::vector<POp> ops;
  std::vector<PLayer> layers;
  std::vector<int> inputs;     // value ids, user order
  std::vector<int> constants;  // value ids, discovery order (appended program arguments)
  std::vector<int> outputs;    // value ids
  std::string target;          // set by plaidml_program_compile
  bool compiled = false;
  std::string str() const;    // the bounded form the planner consumes: index ranges, rational accesses
  std::string mlir() const;   // the same program spelled like the reference's printed `tile` module
};

std::shared_ptr<Program> buildProgram(const std::string& name, const std::vector<ExprPtr>& inputs,
                                      const std::vector<const TensorShape*>& shapes,
                                      const std::vector<ExprPtr>& outputs);

// Evaluates an index polynomial into an affine form over the contraction's variables,
// numbering variables in first-seen order (pmlc/ast/builder.cc:311-323,434-438).
class IndexNumbering {
 public:
  size_t indexOf(const PolyNode* node);
  const std::vector<std::string>& names() const { return names_; }
  size_t size() const { return names_.size(); }

 private:
  std::unordered_map<const PolyNode*, size_t> ids_;
  std::vector<std::string> names_;
};

Affine evalPoly(const PolyPtr& poly, IndexNumbering* idxs, Evaluator* ev);

// Fills lower / extent of every index variable from the in-range conditions of all
// accesses plus the explicit constraints, by interval propagation.  Throws when a variable
// has no finite range.
void computeBounds(BoundedContraction* c, const TensorShape& out, const std::vector<TensorShape>& srcShapes);

BufferPtr makeScalarConstant(DType dtype, const Literal& lit);

}  // namespace pml

struct plaidml_program {
  std::shared_ptr<pml::Program> program;
};
