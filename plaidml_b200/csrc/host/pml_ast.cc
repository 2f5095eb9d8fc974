// Printing and shape / type evaluation of the expression tree.
#include "pml_ast.h"

#include <algorithm>
#include <sstream>

namespace pml {

static const char* affineOpStr(AffineOp op) {
  switch (op) {
    case AffineOp::Neg: return "neg";
    case AffineOp::Add: return "add";
    case AffineOp::Sub: return "sub";
    case AffineOp::Mul: return "mul";
    case AffineOp::Div: return "div";
    case AffineOp::Max: return "max";
    case AffineOp::Min: return "min";
  }
  return "?";
}

DimPtr makeDimLiteral(int64_t v) {
  auto d = std::make_shared<DimNode>();
  d->kind = DimNode::Literal;
  d->value = v;
  return d;
}

std::string DimNode::str() const {
  switch (kind) {
    case None: return "?";
    case Literal: return std::to_string(value);
    case Ref: return "dim(" + (ref ? ref->str() : std::string("?")) + "[" + std::to_string(dim) + "])";
    case Op: {
      std::ostringstream os;
      os << affineOpStr(op) << "(";
      for (size_t i = 0; i < operands.size(); ++i) os << (i ? ", " : "") << operands[i]->str();
      os << ")";
      return os.str();
    }
  }
  return "?";
}

std::string PolyNode::str() const {
  switch (kind) {
    case Dim: return dim->str();
    case Index: return "%" + (name.empty() ? std::string("x") : name);
    case Literal: return std::to_string(value);
    case Op: {
      std::ostringstream os;
      os << affineOpStr(op) << "(";
      for (size_t i = 0; i < operands.size(); ++i) os << (i ? ", " : "") << operands[i]->str();
      os << ")";
      return os.str();
    }
  }
  return "?";
}

std::string VarNode::str() const {
  switch (kind) {
    case None: return "none";
    case Dim: return dim->str();
    case Expr: return expr->str();
    case Float: return std::to_string(f);
    case Int: return std::to_string(i);
    case Str: return "\"" + s + "\"";
    case Tuple: {
      std::ostringstream os;
      os << "(";
      for (size_t k = 0; k < tuple.size(); ++k) os << (k ? ", " : "") << tuple[k]->str();
      os << ")";
      return os.str();
    }
  }
  return "?";
}

ExprPtr& ExprNode::openLayer() {
  thread_local ExprPtr layer;
  return layer;
}

std::string ExprNode::str() const {
  switch (kind) {
    case Cast: return std::string("cast(") + dtypeName(dtype) + ")";
    case ConstSigned: return std::to_string(ivalue) + ":six";
    case ConstUnsigned: return std::to_string(uvalue) + ":uix";
    case ConstFloat: return std::to_string(fvalue) + ":fx";
    case ConstTensor: return "constant_tensor(" + name + ")";
    case Contraction: return "contraction(" + name + ")";
    case Dim: return dim->str();
    case Element: return "element(" + (expr ? expr->str() : std::string("?")) + "[" + std::to_string(ordinal) + "])";
    case Input: return "input(" + name + ", " + shape.str() + ")";
    case Intrinsic: return op + "()";
    case Layer: return "layer(" + op + ")";
    case Pragma: return "pragma(" + op + ")";
  }
  return "?";
}

// ------------------------------------------------------------------ broadcasting

static bool mergeShapes(TensorShape* into, const TensorShape& from, DType override) {
  const std::vector<int64_t>& a = into->sizes;
  const std::vector<int64_t>& b = from.sizes;
  std::vector<int64_t> result = a.size() > b.size() ? a : b;
  auto ia = a.rbegin(), ib = b.rbegin();
  auto ir = result.rbegin();
  for (; ia != a.rend() && ib != b.rend(); ++ia, ++ib, ++ir) {
    if (*ia == 0 || *ib == 0) {
      // unknown extents: the larger known one wins, as in the reference
      if (*ia > 1) *ir = *ia;
      else if (*ib > 1) *ir = *ib;
      else if (*ia == 1) *ir = *ib;
      else if (*ib == 1) *ir = *ia;
      else *ir = 0;
    } else if (*ia == *ib || *ib == 1) {
      *ir = *ia;
    } else if (*ia == 1) {
      *ir = *ib;
    } else {
      return false;
    }
  }
  DType dt = override != DType::invalid ? override : promote(into->dtype, from.dtype);
  *into = TensorShape(dt, result);
  return true;
}

TensorShape inferShape(const std::vector<TensorShape>& operands, DType override) {
  if (operands.empty()) throw std::runtime_error("operation without operands");
  TensorShape ret = operands.front();
  ret.strides.clear();
  if (override != DType::invalid) ret.dtype = override;
  for (size_t i = 1; i < operands.size(); ++i) {
    if (!mergeShapes(&ret, operands[i], override)) {
      std::ostringstream os;
      os << "Incompatible types: (";
      for (size_t k = 0; k < operands.size(); ++k) os << (k ? ", " : "") << operands[k].str();
      os << ")";
      throw std::runtime_error(os.str());
    }
  }
  return ret;
}

bool getIntegerValue(Evaluator* ev, const ExprPtr& e, int64_t* out) {
  switch (e->kind) {
    case ExprNode::ConstSigned: *out = e->ivalue; return true;
    case ExprNode::ConstUnsigned: *out = static_cast<int64_t>(e->uvalue); return true;
    case ExprNode::Dim: *out = ev->evaluate(e->dim); return true;
    default: return false;
  }
}

// ------------------------------------------------------------------ evaluator

int64_t Evaluator::evaluate(const DimPtr& node) {
  switch (node->kind) {
    case DimNode::Literal: return node->value;
    case DimNode::None: throw std::runtime_error("DimNodeNone cannot be evaluated");
    case DimNode::Ref: {
      TensorShape shape = getShape(node->ref);
      if (shape.rank() <= node->dim) throw std::runtime_error("DimNodeRef out of bounds");
      return shape.sizes[node->dim];
    }
    case DimNode::Op: {
      if (node->op == AffineOp::Neg) {
        if (node->operands.size() != 1) throw std::runtime_error("AffineOp::Neg expected single operand");
        return -evaluate(node->operands[0]);
      }
      if (node->operands.size() != 2) throw std::runtime_error("Binary DimNodeOp expected 2 operands");
      const int64_t l = evaluate(node->operands[0]), r = evaluate(node->operands[1]);
      switch (node->op) {
        case AffineOp::Add: return l + r;
        case AffineOp::Sub: return l - r;
        case AffineOp::Mul: return l * r;
        case AffineOp::Div:
          if (r == 0) throw std::runtime_error("Division by zero in dimension expression");
          return l / r;
        case AffineOp::Max: return std::max(l, r);
        case AffineOp::Min: return std::min(l, r);
        default: throw std::runtime_error("Invalid AffineOp");
      }
    }
  }
  throw std::runtime_error("Invalid DimNode");
}

TensorShape Evaluator::getShape(const ExprNode* node) {
  const auto& shapes = getShapes(node);
  if (shapes.size() != 1) throw std::runtime_error("Missing element needed to resolve multiple results.");
  return shapes[0];
}

TensorShape Evaluator::getShape(const ExprNode* node, size_t ordinal) {
  const auto& shapes = getShapes(node);
  if (shapes.size() <= ordinal) throw std::runtime_error("Out of bounds element ordinal");
  return shapes[ordinal];
}

const std::vector<TensorShape>& Evaluator::getShapes(const ExprNode* node) {
  auto it = cache_.find(node);
  if (it == cache_.end()) it = cache_.emplace(node, computeShapes(node)).first;
  return it->second;
}

static bool isBooleanOp(const std::string& op) {
  return op == "cmp_eq" || op == "cmp_ge" || op == "cmp_gt" || op == "cmp_le" || op == "cmp_lt" ||
         op == "cmp_ne" || op == "logical_and" || op == "logical_not" || op == "logical_or" ||
         op == "logical_xor";
}

std::vector<TensorShape> Evaluator::computeShapes(const ExprNode* node) {
  switch (node->kind) {
    case ExprNode::Cast: {
      TensorShape s = getShape(node->expr);
      s.dtype = node->dtype;
      s.strides.clear();
      return {s};
    }
    case ExprNode::ConstSigned: return {TensorShape(DType::six)};
    case ExprNode::ConstUnsigned: return {TensorShape(DType::uix)};
    case ExprNode::ConstFloat: return {TensorShape(DType::fx)};
    case ExprNode::ConstTensor: return {node->buffer->shape()};
    case ExprNode::Contraction: {
      DType dt;
      if (node->combo == ComboKind::eq) {
        dt = DType::i1;
      } else if (node->combo == ComboKind::cond) {
        if (node->srcs.size() != 3) throw std::runtime_error("'cond' combination needs three operands");
        dt = getShape(node->srcs[2].ref).dtype;
      } else {
        dt = DType::invalid;
        for (const PolyMap& src : node->srcs) dt = promote(dt, getShape(src.ref).dtype);
      }
      if (isAmbiguous(dt)) throw std::runtime_error("'contraction' operand data type is ambiguous, use a cast");
      TensorShape s(dt);
      for (const DimPtr& d : node->sinkDims) s.sizes.push_back(evaluate(d));
      return {s};
    }
    case ExprNode::Dim: return {TensorShape(DType::six)};
    case ExprNode::Element: return {getShape(node->expr.get(), node->ordinal)};
    case ExprNode::Layer: {
      std::vector<TensorShape> ret;
      for (const ExprPtr& r : node->results) ret.push_back(getShape(r));
      return ret;
    }
    case ExprNode::Input: return {node->shape};
    case ExprNode::Pragma: return getShapes(node->expr.get());
    case ExprNode::Intrinsic: {
      std::vector<TensorShape> shapes;
      for (const ExprPtr& o : node->operands) shapes.push_back(getShape(o));
      const std::string& op = node->op;
      if (isBooleanOp(op)) return {inferShape(shapes, DType::i1)};
      if (op == "index") {
        if (node->operands.size() < 2) {
          throw std::runtime_error("'index' requires an axis operand and at least 1 dimension");
        }
        TensorShape ret(DType::si32);
        for (size_t i = 1; i < node->operands.size(); ++i) {
          int64_t v;
          if (!getIntegerValue(this, node->operands[i], &v)) {
            throw std::runtime_error("Additional parameters to 'index' must be integers or TensorDims.");
          }
          ret.sizes.push_back(v);
        }
        return {ret};
      }
      if (op == "reshape") {
        if (node->operands.empty()) throw std::runtime_error("'reshape' requires at least one argument.");
        TensorShape ret(shapes[0].dtype);
        for (size_t i = 1; i < node->operands.size(); ++i) {
          int64_t v;
          if (!getIntegerValue(this, node->operands[i], &v)) {
            throw std::runtime_error("Additional parameters to 'reshape' must be integers or TensorDims.");
          }
          ret.sizes.push_back(v);
        }
        return {ret};
      }
      if (op == "shape") {
        if (node->operands.size() != 1) throw std::runtime_error("'shape' requires exactly one argument.");
        return {TensorShape(DType::si32, {static_cast<int64_t>(shapes[0].rank())})};
      }
      if (op == "select") {
        if (shapes.size() != 3) throw std::runtime_error("'select' requires three arguments.");
        TensorShape s = inferShape(shapes);
        const DType dt = promote(shapes[1].dtype, shapes[2].dtype);
        if (isAmbiguous(dt)) throw std::runtime_error("'select' has ambiguous operand types, use a cast");
        for (size_t i = 1; i < 3; ++i) {
          if (shapes[i].dtype != dt && !isAmbiguous(shapes[i].dtype)) {
            throw std::runtime_error("'select' has unmatched operand types, use a cast");
          }
        }
        return {TensorShape(dt, s.sizes)};
      }
      // the four operations that are not contractions (pmlc/ast/ast_ops.cc:54-72,101-264)
      auto integerOperand = [&](size_t i, int64_t* v) { return getIntegerValue(this, node->operands[i], v); };
      if (op == "argsort") {
        int64_t v;
        if (node->operands.size() != 3) throw std::runtime_error("'argsort' requires 3 arguments.");
        if (!integerOperand(1, &v)) throw std::runtime_error("'argsort' requires operand #2 to be an integer.");
        if (!integerOperand(2, &v)) throw std::runtime_error("'argsort' requires operand #3 to be an integer.");
        return {TensorShape(DType::si32, shapes[0].sizes)};
      }
      if (op == "gather") {
        if (node->operands.size() != 9) throw std::runtime_error("'gather' requires nine arguments.");
        const TensorShape& tensor = shapes[0];
        const TensorShape& idxs = shapes[1];
        const int64_t rank = static_cast<int64_t>(tensor.rank());
        if (!rank) throw std::runtime_error("'gather' requires first operand to have at least one dimension.");
        int64_t axis, interpolation, nearest, mode, batchDims, outOfBounds;
        if (!integerOperand(2, &axis) || axis >= rank || axis < 0) {
          throw std::runtime_error(
              "'gather' primitive expects the 'axis' argument to be a positive integer that is less than the tensor rank.");
        }
        if (!integerOperand(3, &interpolation)) {
          throw std::runtime_error("'gather' primitive expects the 'interpolationMode' argument to be a constant integer");
        }
        if (!integerOperand(4, &nearest)) {
          throw std::runtime_error("'gather' primitive expects the 'nearestMode' argument to be a constant integer");
        }
        if (node->operands[5]->kind != ExprNode::ConstFloat) {
          throw std::runtime_error("'gather' primitive expects the 'cubeCoeff' argument to be a constant float");
        }
        if (!integerOperand(6, &mode)) {
          throw std::runtime_error("'gather' primitive expects the 'mode' argument to be a constant integer");
        }
        if (mode == 1 && (isFloat(idxs.dtype) || idxs.dtype == DType::i1 || idxs.dtype == DType::invalid)) {
          throw std::runtime_error("'gather' ND mode requires indices elements to be integers.");
        }
        if (!integerOperand(7, &batchDims)) {
          throw std::runtime_error("'gather' primitive expects the 'batchDims' argument to be a constant integer");
        }
        if (!integerOperand(8, &outOfBounds)) {
          throw std::runtime_error("'gather' primitive expects the 'outOfBoundsMode' argument to be a constant integer");
        }
        TensorShape ret(tensor.dtype);
        if (mode == 0) {
          for (int64_t i = 0; i < axis; ++i) ret.sizes.push_back(tensor.sizes[i]);
          ret.sizes.insert(ret.sizes.end(), idxs.sizes.begin(), idxs.sizes.end());
          for (int64_t i = axis + 1; i < rank; ++i) ret.sizes.push_back(tensor.sizes[i]);
        } else {
          if (idxs.rank() < 1) throw std::runtime_error("'gather' ND mode requires indices of at least one dimension.");
          for (size_t i = 0; i + 1 < idxs.rank(); ++i) ret.sizes.push_back(idxs.sizes[i]);
          for (int64_t i = idxs.sizes.back() + batchDims; i < rank; ++i) ret.sizes.push_back(tensor.sizes[i]);
        }
        return {ret};
      }
      if (op == "prng") {
        if (node->operands.empty()) throw std::runtime_error("'prng' requires at least one argument.");
        TensorShape ret(DType::f32);
        for (size_t i = 1; i < node->operands.size(); ++i) {
          int64_t v;
          if (!integerOperand(i, &v)) throw std::runtime_error("'prng' has invalid operands, dims must be tensor dimensions");
          ret.sizes.push_back(v);
        }
        return {ret, shapes[0]};
      }
      if (op == "scatter") {
        if (node->operands.size() != 5) throw std::runtime_error("'scatter' requires 5 operands.");
        const int64_t rank = static_cast<int64_t>(shapes[0].rank());
        if (!rank) throw std::runtime_error("'scatter' requires operand #1 to have at least one dimension.");
        if (shapes[1].dtype != DType::si32 && shapes[1].dtype != DType::ui32) {
          throw std::runtime_error("'scatter' requires operand #2 to be an integer.");
        }
        int64_t axis, mode;
        if (!integerOperand(3, &axis) || axis >= rank) {
          throw std::runtime_error(
              "'scatter' primitive expects the 'axis' argument to be a positive integer that is less than the updates "
              "tensor rank.");
        }
        if (!integerOperand(4, &mode)) {
          throw std::runtime_error("'scatter' primitive expects the 'mode' argument to be a constant integer.");
        }
        return {TensorShape(shapes[0].dtype, shapes[0].sizes)};
      }
      return {inferShape(shapes)};
    }
  }
  throw std::runtime_error("Invalid expression node");
}

void Evaluator::bindDims(const ExprPtr& expr, const std::vector<DimPtr*>& into) {
  TensorShape shape = getShape(expr);
  if (into.size() != shape.rank()) throw std::runtime_error("Rank mismatch in bind_dims");
  bool failed = false;
  for (size_t i = 0; i < into.size(); ++i) {
    DimPtr* ptr = into[i];
    const int64_t dim = shape.sizes[i];
    switch ((*ptr)->kind) {
      case DimNode::None:
        if (dim) {
          *ptr = makeDimLiteral(dim);
        } else {
          auto ref = std::make_shared<DimNode>();
          ref->kind = DimNode::Ref;
          ref->ref = expr;
          ref->dim = i;
          *ptr = ref;
        }
        break;
      case DimNode::Ref:
        if (dim) *ptr = makeDimLiteral(dim);
        break;
      case DimNode::Literal:
        if (dim && dim != (*ptr)->value) failed = true;
        break;
      default:
        throw std::runtime_error("Can only bind dims to an unbound or previously bound TensorDim.");
    }
  }
  if (failed) {
    std::ostringstream s1, s2;
    for (size_t i = 0; i < shape.sizes.size(); ++i) {
      s1 << (i ? ", " : "");
      if (shape.sizes[i]) s1 << shape.sizes[i]; else s1 << '?';
    }
    for (size_t i = 0; i < into.size(); ++i) {
      s2 << (i ? ", " : "");
      const int64_t v = evaluate(*into[i]);
      if (v) s2 << v; else s2 << '?';
    }
    throw std::runtime_error("bind dims mismatch: shape=[" + s1.str() + "] != dims=[" + s2.str() + "]");
  }
}

}  // namespace pml
