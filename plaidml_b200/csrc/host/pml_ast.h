// Expression tree built through the EDSL entry points, plus the shape / type evaluator.
//
// Node kinds follow pmlc/ast/ast.h:95-371 of the reference (dims, index polynomials, tensor
// expressions, the op-library value variant); typing rules follow pmlc/ast/eval.cc:22-298 and
// the intrinsic table of pmlc/ast/ast_ops.cc:54-316.  No MLIR is emitted: `plaidml_build`
// lowers this tree to the flat program of pml_program.h.
#pragma once

#include <map>
#include <memory>
#include <string>
#include <unordered_map>
#include <vector>

#include "pml_core.h"

namespace pml {

enum class AffineOp { Neg, Add, Sub, Mul, Div, Max, Min };
enum class AggKind { assign, add, max, min, mul };
enum class ComboKind { none, add, cond, eq, mul };

struct ExprNode;
using ExprPtr = std::shared_ptr<ExprNode>;

// ---------------------------------------------------------------- dims
struct DimNode {
  enum Kind { None, Literal, Op, Ref } kind = None;
  int64_t value = 0;                                // Literal
  AffineOp op = AffineOp::Add;                      // Op
  std::vector<std::shared_ptr<DimNode>> operands;   // Op
  ExprPtr ref;                                      // Ref: dimension `dim` of tensor `ref`
  size_t dim = 0;
  std::string str() const;
};
using DimPtr = std::shared_ptr<DimNode>;
DimPtr makeDimLiteral(int64_t v);

// ---------------------------------------------------------------- index polynomials
struct PolyNode {
  enum Kind { Dim, Index, Literal, Op } kind = Literal;
  DimPtr dim;          // Dim
  std::string name;    // Index (identity of an index is the node, not the name)
  int64_t value = 0;   // Literal
  AffineOp op = AffineOp::Add;
  std::vector<std::shared_ptr<PolyNode>> operands;
  std::string str() const;
};
using PolyPtr = std::shared_ptr<PolyNode>;

struct PolyMap {
  ExprPtr ref;
  std::vector<PolyPtr> idxs;
};

struct Constraint {
  PolyPtr lhs;
  DimPtr rhs;
};

// ---------------------------------------------------------------- op-library values
struct VarNode {
  enum Kind { None, Dim, Expr, Float, Int, Str, Tuple } kind = None;
  DimPtr dim;
  ExprPtr expr;
  double f = 0;
  int64_t i = 0;
  std::string s;
  std::vector<std::shared_ptr<VarNode>> tuple;
  std::string str() const;
};
using VarPtr = std::shared_ptr<VarNode>;

// ---------------------------------------------------------------- tensor expressions
struct ExprNode {
  enum Kind {
    Cast, ConstSigned, ConstUnsigned, ConstFloat, ConstTensor, Contraction, Dim, Element, Input,
    Intrinsic, Layer, Pragma
  } kind;
  std::string name;
  ExprPtr parent;  // enclosing layer, if any

  // Cast
  DType dtype = DType::invalid;
  ExprPtr expr;  // Cast / Element / Pragma operand
  // literals
  int64_t ivalue = 0;
  uint64_t uvalue = 0;
  double fvalue = 0;
  // ConstTensor
  BufferPtr buffer;
  // Contraction
  AggKind agg = AggKind::assign;
  ComboKind combo = ComboKind::none;
  std::vector<DimPtr> sinkDims;
  std::vector<PolyPtr> sinkIdxs;
  std::vector<PolyMap> srcs;
  std::vector<Constraint> constraints;
  ExprPtr init;
  // Dim
  DimPtr dim;
  // Element
  size_t ordinal = 0;
  // Input
  TensorShape shape;
  // Intrinsic / Layer / Pragma
  std::string op;
  std::vector<ExprPtr> operands;
  std::vector<ExprPtr> results;                 // Layer
  std::map<std::string, VarPtr> attrs;          // Layer / Pragma

  // A node made while a layer is open on this thread belongs to it (plaidml/edsl/ffi.cc:95-113), whichever
  // entry point made it (the EDSL calls or the operation library).
  explicit ExprNode(Kind k) : kind(k), parent(openLayer()) {}
  std::string str() const;

  // Innermost layer open on this thread (null outside layers); set by plaidml_expr_layer_begin / _end.
  static ExprPtr& openLayer();
};

// ---------------------------------------------------------------- evaluator
class Evaluator {
 public:
  void verify(const ExprPtr& node) { (void)getShapes(node.get()); }
  int64_t evaluate(const DimPtr& dim);
  TensorShape getShape(const ExprPtr& node) { return getShape(node.get()); }
  TensorShape getShape(const ExprNode* node);
  TensorShape getShape(const ExprNode* node, size_t ordinal);
  const std::vector<TensorShape>& getShapes(const ExprNode* node);
  // plaidml_expr_bind_dims: may replace the nodes the handles point to.
  void bindDims(const ExprPtr& expr, const std::vector<DimPtr*>& into);

 private:
  std::vector<TensorShape> computeShapes(const ExprNode* node);
  std::unordered_map<const ExprNode*, std::vector<TensorShape>> cache_;
};

// Broadcast result of element-wise operands (pmlc/ast/eval.cc:46-136); `override` != invalid
// forces the element type.
TensorShape inferShape(const std::vector<TensorShape>& operands, DType override = DType::invalid);

// Integer value of a literal / dim expression used as an intrinsic parameter; false if the
// expression is not a compile-time integer.
bool getIntegerValue(Evaluator* ev, const ExprPtr& e, int64_t* out);

}  // namespace pml

struct plaidml_expr {
  pml::ExprPtr node;
};
struct plaidml_poly_expr {
  pml::PolyPtr node;
};
struct plaidml_dim_expr {
  pml::DimPtr node;
};
struct plaidml_value {
  pml::VarPtr node;
};
