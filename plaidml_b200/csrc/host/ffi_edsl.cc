// C ABI: the EDSL expression builder.  Reference counterparts: plaidml/edsl/ffi.cc:95-870.
#include <deque>
#include <mutex>

#include "pml_ast.h"
#include "pml_exec.h"
#include "pml_program.h"

using pml::ffiWrap;
using pml::ffiWrapVoid;
using pml::ExprNode;
using pml::ExprPtr;

namespace {

pml::AggKind aggOf(plaidml_agg_op op) {
  switch (op) {
    case PLAIDML_AGG_OP_ASSIGN: return pml::AggKind::assign;
    case PLAIDML_AGG_OP_MAX: return pml::AggKind::max;
    case PLAIDML_AGG_OP_MIN: return pml::AggKind::min;
    case PLAIDML_AGG_OP_PROD: return pml::AggKind::mul;
    case PLAIDML_AGG_OP_SUM: return pml::AggKind::add;
    default: break;
  }
  throw std::runtime_error("Unsupported agg_op");
}

pml::ComboKind comboOf(plaidml_combo_op op) {
  switch (op) {
    case PLAIDML_COMBO_OP_ADD: return pml::ComboKind::add;
    case PLAIDML_COMBO_OP_COND: return pml::ComboKind::cond;
    case PLAIDML_COMBO_OP_EQ: return pml::ComboKind::eq;
    case PLAIDML_COMBO_OP_MUL: return pml::ComboKind::mul;
    case PLAIDML_COMBO_OP_NONE: return pml::ComboKind::none;
    default: break;
  }
  throw std::runtime_error("Unsupported combo_op");
}

pml::AffineOp affineOf(plaidml_int_op op) {
  switch (op) {
    case PLAIDML_INT_OP_ADD: return pml::AffineOp::Add;
    case PLAIDML_INT_OP_DIV: return pml::AffineOp::Div;
    case PLAIDML_INT_OP_MUL: return pml::AffineOp::Mul;
    case PLAIDML_INT_OP_NEG: return pml::AffineOp::Neg;
    case PLAIDML_INT_OP_SUB: return pml::AffineOp::Sub;
    case PLAIDML_INT_OP_MAX: return pml::AffineOp::Max;
    case PLAIDML_INT_OP_MIN: return pml::AffineOp::Min;
  }
  throw std::runtime_error("Unknown polynomial op");
}

// Nesting of open layers on this thread (plaidml/edsl/ffi.cc:95-113).
struct LayerContext {
  static LayerContext* get() {
    thread_local LayerContext ctx;
    return &ctx;
  }
  void addNode(const ExprPtr& node) {
    if (!stack.empty()) node->parent = stack.front();
  }
  std::deque<ExprPtr> stack;
};

ExprPtr makeExpr(ExprNode::Kind kind) {
  auto node = std::make_shared<ExprNode>(kind);
  return node;
}

plaidml_expr* wrap(const ExprPtr& node) {
  LayerContext::get()->addNode(node);
  return new plaidml_expr{node};
}

pml::VarPtr makeVar(pml::VarNode::Kind kind) {
  auto v = std::make_shared<pml::VarNode>();
  v->kind = kind;
  return v;
}

}  // namespace

extern "C" {

void plaidml_edsl_init(plaidml_error* err) {
  ffiWrapVoid(err, [&] {});
}

// ------------------------------------------------------------------ tensor expressions

void plaidml_expr_free(plaidml_error* err, plaidml_expr* expr) {
  ffiWrapVoid(err, [&] { delete expr; });
}

void* plaidml_expr_ptr(plaidml_error* err, plaidml_expr* expr) {
  return ffiWrap<void*>(err, nullptr, [&] { return static_cast<void*>(expr->node.get()); });
}

plaidml_datatype plaidml_expr_get_dtype(plaidml_error* err, plaidml_expr* expr) {
  return ffiWrap<plaidml_datatype>(err, PLAIDML_DATA_INVALID, [&] {
    pml::Evaluator ev;
    return pml::toFfi(ev.getShape(expr->node).dtype);
  });
}

size_t plaidml_expr_get_rank(plaidml_error* err, plaidml_expr* expr) {
  return ffiWrap<size_t>(err, 0, [&] {
    pml::Evaluator ev;
    return ev.getShape(expr->node).rank();
  });
}

plaidml_shape* plaidml_expr_get_shape(plaidml_error* err, plaidml_expr* expr) {
  return ffiWrap<plaidml_shape*>(err, nullptr, [&] {
    pml::Evaluator ev;
    return new plaidml_shape{ev.getShape(expr->node)};
  });
}

void plaidml_expr_bind_dims(plaidml_error* err, plaidml_expr* expr, size_t rank, plaidml_dim_expr** dims) {
  ffiWrapVoid(err, [&] {
    std::vector<pml::DimPtr*> into;
    for (size_t i = 0; i < rank; ++i) into.push_back(&dims[i]->node);
    pml::Evaluator ev;
    ev.bindDims(expr->node, into);
  });
}

plaidml_string* plaidml_expr_repr(plaidml_error* err, plaidml_expr* expr) {
  return ffiWrap<plaidml_string*>(err, nullptr, [&] { return new plaidml_string{expr->node->str()}; });
}

plaidml_expr* plaidml_expr_clone(plaidml_error* err, plaidml_expr* expr) {
  return ffiWrap<plaidml_expr*>(err, nullptr, [&] { return new plaidml_expr{expr->node}; });
}

plaidml_dim_expr* plaidml_expr_get_dim(plaidml_error* err, plaidml_expr* expr) {
  return ffiWrap<plaidml_dim_expr*>(err, nullptr, [&] {
    if (expr->node->kind != ExprNode::Dim) throw std::bad_cast();
    return new plaidml_dim_expr{expr->node->dim};
  });
}

plaidml_expr* plaidml_expr_dim(plaidml_error* err, plaidml_dim_expr* expr) {
  return ffiWrap<plaidml_expr*>(err, nullptr, [&] {
    ExprPtr node = makeExpr(ExprNode::Dim);
    node->dim = expr->node;
    return wrap(node);
  });
}

plaidml_expr* plaidml_expr_input(plaidml_error* err, plaidml_shape* shape, const char* name) {
  return ffiWrap<plaidml_expr*>(err, nullptr, [&] {
    if (shape->shape.dtype == pml::DType::invalid) throw std::runtime_error("Placeholder with an invalid data type");
    ExprPtr node = makeExpr(ExprNode::Input);
    node->shape = shape->shape;
    node->name = name ? name : "";
    return wrap(node);
  });
}

plaidml_expr* plaidml_expr_constant(plaidml_error* err, plaidml_buffer* buffer, const char* name) {
  return ffiWrap<plaidml_expr*>(err, nullptr, [&] {
    ExprPtr node = makeExpr(ExprNode::ConstTensor);
    node->buffer = buffer->buffer;
    node->name = name ? name : "";
    // constants live in the global scope (they become program arguments); every open layer
    // lists them as an operand
    for (const ExprPtr& layer : LayerContext::get()->stack) layer->operands.push_back(node);
    return new plaidml_expr{node};
  });
}

plaidml_expr* plaidml_expr_uint(plaidml_error* err, uint64_t value) {
  return ffiWrap<plaidml_expr*>(err, nullptr, [&] {
    ExprPtr node = makeExpr(ExprNode::ConstUnsigned);
    node->uvalue = value;
    return wrap(node);
  });
}

plaidml_expr* plaidml_expr_int(plaidml_error* err, int64_t value) {
  return ffiWrap<plaidml_expr*>(err, nullptr, [&] {
    ExprPtr node = makeExpr(ExprNode::ConstSigned);
    node->ivalue = value;
    return wrap(node);
  });
}

plaidml_expr* plaidml_expr_float(plaidml_error* err, double value) {
  return ffiWrap<plaidml_expr*>(err, nullptr, [&] {
    ExprPtr node = makeExpr(ExprNode::ConstFloat);
    node->fvalue = value;
    return wrap(node);
  });
}

plaidml_expr* plaidml_expr_cast(plaidml_error* err, plaidml_expr* tensor, plaidml_datatype dtype) {
  return ffiWrap<plaidml_expr*>(err, nullptr, [&] {
    ExprPtr node = makeExpr(ExprNode::Cast);
    node->dtype = pml::fromFfi(dtype);
    node->expr = tensor->node;
    return wrap(node);
  });
}

plaidml_expr* plaidml_expr_element(plaidml_error* err, plaidml_expr* expr, size_t ordinal) {
  return ffiWrap<plaidml_expr*>(err, nullptr, [&] {
    ExprPtr node = makeExpr(ExprNode::Element);
    node->expr = expr->node;
    node->ordinal = ordinal;
    return wrap(node);
  });
}

plaidml_expr* plaidml_expr_pragma(plaidml_error* err, plaidml_expr* tensor, const char* op, size_t nattrs,
                                  plaidml_attr** attrs) {
  return ffiWrap<plaidml_expr*>(err, nullptr, [&] {
    ExprPtr node = makeExpr(ExprNode::Pragma);
    node->expr = tensor->node;
    node->op = op ? op : "";
    for (size_t i = 0; i < nattrs; ++i) node->attrs[attrs[i]->key] = attrs[i]->value->node;
    return wrap(node);
  });
}

plaidml_expr* plaidml_expr_intrinsic(plaidml_error* err, const char* fn, size_t nargs, plaidml_expr** args,
                                     const char* name) {
  return ffiWrap<plaidml_expr*>(err, nullptr, [&] {
    ExprPtr node = makeExpr(ExprNode::Intrinsic);
    node->op = fn;
    node->name = name ? name : "";
    for (size_t i = 0; i < nargs; ++i) node->operands.push_back(args[i]->node);
    pml::Evaluator ev;
    ev.verify(node);
    return wrap(node);
  });
}

plaidml_expr* plaidml_expr_contraction(plaidml_error* err, plaidml_agg_op agg_op, plaidml_combo_op combo_op, size_t rank,
                                       plaidml_poly_expr** idxs, plaidml_dim_expr** dims, plaidml_expr* init,
                                       const char* name) {
  return ffiWrap<plaidml_expr*>(err, nullptr, [&] {
    ExprPtr node = makeExpr(ExprNode::Contraction);
    node->name = name ? name : "";
    node->agg = aggOf(agg_op);
    node->combo = comboOf(combo_op);
    for (size_t i = 0; i < rank; ++i) {
      node->sinkDims.push_back(dims[i]->node);
      node->sinkIdxs.push_back(idxs[i]->node);
    }
    if (init) node->init = init->node;
    return wrap(node);
  });
}

void plaidml_contraction_add_operand(plaidml_error* err, plaidml_expr* expr, plaidml_expr* tensor, size_t rank,
                                     plaidml_poly_expr** idxs) {
  ffiWrapVoid(err, [&] {
    if (expr->node->kind != ExprNode::Contraction) throw std::bad_cast();
    pml::PolyMap map;
    map.ref = tensor->node;
    for (size_t i = 0; i < rank; ++i) map.idxs.push_back(idxs[i]->node);
    expr->node->srcs.push_back(std::move(map));
  });
}

void plaidml_contraction_add_constraint(plaidml_error* err, plaidml_expr* expr, plaidml_poly_expr* lhs,
                                        plaidml_dim_expr* rhs) {
  ffiWrapVoid(err, [&] {
    if (expr->node->kind != ExprNode::Contraction) throw std::bad_cast();
    expr->node->constraints.push_back({lhs->node, rhs->node});
  });
}

void plaidml_contraction_build(plaidml_error* err, plaidml_expr* expr) {
  ffiWrapVoid(err, [&] {
    pml::Evaluator ev;
    ev.verify(expr->node);
  });
}

void plaidml_exprs_free(plaidml_error* err, plaidml_exprs* exprs) {
  ffiWrapVoid(err, [&] {
    delete[] exprs->elts;
    delete exprs;
  });
}

plaidml_expr* plaidml_expr_layer_begin(plaidml_error* err, const char* op, size_t ninputs, plaidml_expr** inputs,
                                       size_t nattrs, plaidml_attr** attrs) {
  return ffiWrap<plaidml_expr*>(err, nullptr, [&] {
    ExprPtr node = makeExpr(ExprNode::Layer);
    node->op = op ? op : "";
    for (size_t i = 0; i < ninputs; ++i) node->operands.push_back(inputs[i]->node);
    for (size_t i = 0; i < nattrs; ++i) node->attrs[attrs[i]->key] = attrs[i]->value->node;
    LayerContext::get()->addNode(node);
    LayerContext::get()->stack.push_front(node);
    ExprNode::openLayer() = node;
    return new plaidml_expr{node};
  });
}

plaidml_exprs* plaidml_expr_layer_end(plaidml_error* err, plaidml_expr* expr, size_t noutputs, plaidml_expr** outputs) {
  return ffiWrap<plaidml_exprs*>(err, nullptr, [&] {
    if (expr->node->kind != ExprNode::Layer) throw std::bad_cast();
    auto& stack = LayerContext::get()->stack;
    if (!stack.empty()) stack.pop_front();
    ExprNode::openLayer() = stack.empty() ? ExprPtr() : stack.front();
    expr->node->results.clear();
    std::vector<plaidml_expr*> outer;
    for (size_t i = 0; i < noutputs; ++i) {
      expr->node->results.push_back(outputs[i]->node);
      ExprPtr elt = makeExpr(ExprNode::Element);
      elt->expr = expr->node;
      elt->ordinal = i;
      outer.push_back(new plaidml_expr{elt});
    }
    return pml::makeList<plaidml_exprs, plaidml_expr*>(outer);
  });
}

// ------------------------------------------------------------------ index polynomials

void plaidml_poly_expr_free(plaidml_error* err, plaidml_poly_expr* expr) {
  ffiWrapVoid(err, [&] { delete expr; });
}

plaidml_string* plaidml_poly_expr_repr(plaidml_error* err, plaidml_poly_expr* expr) {
  return ffiWrap<plaidml_string*>(err, nullptr, [&] { return new plaidml_string{expr->node->str()}; });
}

plaidml_poly_expr* plaidml_poly_expr_dim(plaidml_error* err, plaidml_dim_expr* expr) {
  return ffiWrap<plaidml_poly_expr*>(err, nullptr, [&] {
    auto node = std::make_shared<pml::PolyNode>();
    node->kind = pml::PolyNode::Dim;
    node->dim = expr->node;
    return new plaidml_poly_expr{node};
  });
}

plaidml_poly_expr* plaidml_poly_expr_index(plaidml_error* err, const char* name) {
  return ffiWrap<plaidml_poly_expr*>(err, nullptr, [&] {
    auto node = std::make_shared<pml::PolyNode>();
    node->kind = pml::PolyNode::Index;
    node->name = name ? name : "";
    return new plaidml_poly_expr{node};
  });
}

plaidml_poly_expr* plaidml_poly_expr_literal(plaidml_error* err, int64_t value) {
  return ffiWrap<plaidml_poly_expr*>(err, nullptr, [&] {
    auto node = std::make_shared<pml::PolyNode>();
    node->kind = pml::PolyNode::Literal;
    node->value = value;
    return new plaidml_poly_expr{node};
  });
}

plaidml_poly_expr* plaidml_poly_expr_op(plaidml_error* err, plaidml_int_op op, size_t nargs, plaidml_poly_expr** args) {
  return ffiWrap<plaidml_poly_expr*>(err, nullptr, [&] {
    auto node = std::make_shared<pml::PolyNode>();
    node->kind = pml::PolyNode::Op;
    node->op = affineOf(op);
    for (size_t i = 0; i < nargs; ++i) node->operands.push_back(args[i]->node);
    return new plaidml_poly_expr{node};
  });
}

// ------------------------------------------------------------------ dimension expressions

void plaidml_dim_expr_free(plaidml_error* err, plaidml_dim_expr* expr) {
  ffiWrapVoid(err, [&] { delete expr; });
}

plaidml_string* plaidml_dim_expr_repr(plaidml_error* err, plaidml_dim_expr* expr) {
  return ffiWrap<plaidml_string*>(err, nullptr, [&] { return new plaidml_string{expr->node->str()}; });
}

plaidml_dim_expr* plaidml_dim_expr_none(plaidml_error* err) {
  return ffiWrap<plaidml_dim_expr*>(err, nullptr, [&] { return new plaidml_dim_expr{std::make_shared<pml::DimNode>()}; });
}

plaidml_dim_expr* plaidml_dim_expr_int(plaidml_error* err, int64_t value) {
  return ffiWrap<plaidml_dim_expr*>(err, nullptr, [&] { return new plaidml_dim_expr{pml::makeDimLiteral(value)}; });
}

plaidml_dim_expr* plaidml_dim_expr_op(plaidml_error* err, plaidml_int_op op, size_t nargs, plaidml_dim_expr** args) {
  return ffiWrap<plaidml_dim_expr*>(err, nullptr, [&] {
    auto node = std::make_shared<pml::DimNode>();
    node->kind = pml::DimNode::Op;
    node->op = affineOf(op);
    for (size_t i = 0; i < nargs; ++i) node->operands.push_back(args[i]->node);
    return new plaidml_dim_expr{node};
  });
}

// ------------------------------------------------------------------ values

void plaidml_tuple_free(plaidml_error* err, plaidml_tuple* tuple) {
  ffiWrapVoid(err, [&] {
    for (size_t i = 0; i < tuple->size; ++i) delete tuple->elts[i];
    delete[] tuple->elts;
    delete tuple;
  });
}

void plaidml_value_free(plaidml_error* err, plaidml_value* value) {
  ffiWrapVoid(err, [&] { delete value; });
}

plaidml_value* plaidml_value_clone(plaidml_error* err, plaidml_value* value) {
  return ffiWrap<plaidml_value*>(err, nullptr, [&] { return new plaidml_value{value->node}; });
}

plaidml_value_kind plaidml_value_get_kind(plaidml_error* err, plaidml_value* value) {
  return ffiWrap<plaidml_value_kind>(err, PLAIDML_VALUE_NONE, [&] {
    switch (value->node->kind) {
      case pml::VarNode::Dim: return PLAIDML_VALUE_DIM;
      case pml::VarNode::Expr: return PLAIDML_VALUE_EXPR;
      case pml::VarNode::Float: return PLAIDML_VALUE_FLOAT;
      case pml::VarNode::Int: return PLAIDML_VALUE_INT;
      case pml::VarNode::Str: return PLAIDML_VALUE_STR;
      case pml::VarNode::Tuple: return PLAIDML_VALUE_TUPLE;
      default: return PLAIDML_VALUE_NONE;
    }
  });
}

plaidml_value* plaidml_value_none(plaidml_error* err) {
  return ffiWrap<plaidml_value*>(err, nullptr, [&] { return new plaidml_value{makeVar(pml::VarNode::None)}; });
}

plaidml_value* plaidml_value_dim(plaidml_error* err, plaidml_dim_expr* expr) {
  return ffiWrap<plaidml_value*>(err, nullptr, [&] {
    if (!expr) throw std::runtime_error("plaidml_value_dim requires non-null expr");
    auto v = makeVar(pml::VarNode::Dim);
    v->dim = expr->node;
    return new plaidml_value{v};
  });
}

plaidml_value* plaidml_value_expr(plaidml_error* err, plaidml_expr* expr) {
  return ffiWrap<plaidml_value*>(err, nullptr, [&] {
    if (!expr) throw std::runtime_error("plaidml_value_expr requires non-null expr");
    auto v = makeVar(pml::VarNode::Expr);
    v->expr = expr->node;
    return new plaidml_value{v};
  });
}

plaidml_value* plaidml_value_float(plaidml_error* err, double value) {
  return ffiWrap<plaidml_value*>(err, nullptr, [&] {
    auto v = makeVar(pml::VarNode::Float);
    v->f = value;
    return new plaidml_value{v};
  });
}

plaidml_value* plaidml_value_int(plaidml_error* err, int64_t value) {
  return ffiWrap<plaidml_value*>(err, nullptr, [&] {
    auto v = makeVar(pml::VarNode::Int);
    v->i = value;
    return new plaidml_value{v};
  });
}

plaidml_value* plaidml_value_str(plaidml_error* err, const char* value) {
  return ffiWrap<plaidml_value*>(err, nullptr, [&] {
    auto v = makeVar(pml::VarNode::Str);
    v->s = value ? value : "";
    return new plaidml_value{v};
  });
}

plaidml_value* plaidml_value_tuple(plaidml_error* err, size_t nelts, plaidml_value** elts) {
  return ffiWrap<plaidml_value*>(err, nullptr, [&] {
    auto v = makeVar(pml::VarNode::Tuple);
    for (size_t i = 0; i < nelts; ++i) v->tuple.push_back(elts[i]->node);
    return new plaidml_value{v};
  });
}

plaidml_dim_expr* plaidml_value_dim_get(plaidml_error* err, plaidml_value* value) {
  return ffiWrap<plaidml_dim_expr*>(err, nullptr, [&] {
    if (value->node->kind != pml::VarNode::Dim) throw std::bad_cast();
    return new plaidml_dim_expr{value->node->dim};
  });
}

plaidml_expr* plaidml_value_expr_get(plaidml_error* err, plaidml_value* value) {
  return ffiWrap<plaidml_expr*>(err, nullptr, [&] {
    if (value->node->kind != pml::VarNode::Expr) throw std::bad_cast();
    return new plaidml_expr{value->node->expr};
  });
}

double plaidml_value_float_get(plaidml_error* err, plaidml_value* value) {
  return ffiWrap<double>(err, 0, [&] {
    if (value->node->kind != pml::VarNode::Float) throw std::bad_cast();
    return value->node->f;
  });
}

int64_t plaidml_value_int_get(plaidml_error* err, plaidml_value* value) {
  return ffiWrap<int64_t>(err, 0, [&] {
    if (value->node->kind != pml::VarNode::Int) throw std::bad_cast();
    return value->node->i;
  });
}

plaidml_string* plaidml_value_str_get(plaidml_error* err, plaidml_value* value) {
  return ffiWrap<plaidml_string*>(err, nullptr, [&] {
    if (value->node->kind != pml::VarNode::Str) throw std::bad_cast();
    return new plaidml_string{value->node->s};
  });
}

plaidml_tuple* plaidml_value_tuple_get(plaidml_error* err, plaidml_value* value) {
  return ffiWrap<plaidml_tuple*>(err, nullptr, [&] {
    if (value->node->kind != pml::VarNode::Tuple) throw std::bad_cast();
    std::vector<plaidml_value*> elts;
    for (const pml::VarPtr& v : value->node->tuple) elts.push_back(new plaidml_value{v});
    return pml::makeList<plaidml_tuple, plaidml_value*>(elts);
  });
}

plaidml_string* plaidml_value_repr(plaidml_error* err, plaidml_value* value) {
  return ffiWrap<plaidml_string*>(err, nullptr, [&] { return new plaidml_string{value->node->str()}; });
}

// ------------------------------------------------------------------ targets / build

plaidml_strings* plaidml_targets_get(plaidml_error* err) {
  return ffiWrap<plaidml_strings*>(err, nullptr, [&] {
    std::vector<plaidml_string*> out;
    for (const std::string& t : pml::listTargets()) out.push_back(new plaidml_string{t});
    return pml::makeList<plaidml_strings, plaidml_string*>(out);
  });
}

plaidml_program* plaidml_build(plaidml_error* err, const char* name, size_t ninputs, plaidml_expr** inputs,
                               plaidml_shape** shapes, size_t noutputs, plaidml_expr** outputs) {
  return ffiWrap<plaidml_program*>(err, nullptr, [&] {
    std::vector<ExprPtr> ins, outs;
    std::vector<const pml::TensorShape*> shp;
    for (size_t i = 0; i < ninputs; ++i) {
      ins.push_back(inputs[i]->node);
      shp.push_back(shapes && shapes[i] ? &shapes[i]->shape : nullptr);
    }
    for (size_t i = 0; i < noutputs; ++i) outs.push_back(outputs[i]->node);
    return new plaidml_program{pml::buildProgram(name ? name : "", ins, shp, outs)};
  });
}

}  // extern "C"
