// The operation library: plaidml_op_make(name, args) builds EDSL expressions for named
// tensor operations.  Reference counterpart: plaidml/op/lib/ops.cc (argument conventions per
// operation are cited below); the registry there is plaidml/op/lib/ops.cc:3632-3680.
//
// Scope: the operations that build the contraction path's networks and tests -- convolution
// (forward, ungrouped), pool, dot, relu, mean / sum / max / min / prod, softmax -- plus the
// thin element-wise and layout ones that cost a few lines each.
#include <array>
#include <functional>
#include <map>
#include <set>

#include "pml_ast.h"

using pml::ExprNode;
using pml::ExprPtr;
using pml::PolyPtr;
using pml::VarNode;
using pml::VarPtr;

namespace {

// ------------------------------------------------------------------ small builder layer

pml::TensorShape shapeOf(const ExprPtr& e) {
  pml::Evaluator local;
  return local.getShape(e);
}

// Manual padding lists all "before" values, then all "after" values.  Missing "before" values are 0 and
// a missing "after" value repeats the "before" value of its dimension (plaidml/op/lib/ops.cc:420-436).
void splitManualPadding(std::vector<int64_t> pads, size_t rank, std::vector<int64_t>* lo, std::vector<int64_t>* hi) {
  if (pads.size() > 2 * rank) {
    throw std::runtime_error("Inconsistent spatial rank: operation with " + std::to_string(rank) + " spatial dimensions had " +
                             std::to_string(pads.size()) + " manual padding values given");
  }
  while (pads.size() < rank) pads.push_back(0);
  while (pads.size() < 2 * rank) pads.push_back(pads[pads.size() - rank]);
  lo->assign(pads.begin(), pads.begin() + rank);
  hi->assign(pads.begin() + rank, pads.end());
}

PolyPtr newIndex(const std::string& name = "") {
  auto p = std::make_shared<pml::PolyNode>();
  p->kind = pml::PolyNode::Index;
  p->name = name;
  return p;
}

PolyPtr polyLit(int64_t v) {
  auto p = std::make_shared<pml::PolyNode>();
  p->kind = pml::PolyNode::Literal;
  p->value = v;
  return p;
}

PolyPtr polyOp(pml::AffineOp op, PolyPtr a, PolyPtr b) {
  auto p = std::make_shared<pml::PolyNode>();
  p->kind = pml::PolyNode::Op;
  p->op = op;
  p->operands = {std::move(a), std::move(b)};
  return p;
}
PolyPtr operator+(PolyPtr a, PolyPtr b) { return polyOp(pml::AffineOp::Add, std::move(a), std::move(b)); }
PolyPtr operator-(PolyPtr a, PolyPtr b) { return polyOp(pml::AffineOp::Sub, std::move(a), std::move(b)); }
PolyPtr operator*(int64_t a, PolyPtr b) { return polyOp(pml::AffineOp::Mul, polyLit(a), std::move(b)); }
PolyPtr operator+(PolyPtr a, int64_t b) { return std::move(a) + polyLit(b); }
PolyPtr operator-(PolyPtr a, int64_t b) { return std::move(a) - polyLit(b); }

struct Operand {
  ExprPtr tensor;
  std::vector<PolyPtr> idxs;
};

struct Cons {
  PolyPtr lhs;
  int64_t rhs;
};

ExprPtr contraction(pml::AggKind agg, pml::ComboKind combo, const std::vector<int64_t>& dims,
                    const std::vector<PolyPtr>& idxs, const std::vector<Operand>& srcs,
                    const std::vector<Cons>& cons = {}, const std::string& name = "") {
  auto node = std::make_shared<ExprNode>(ExprNode::Contraction);
  node->name = name;
  node->agg = agg;
  node->combo = combo;
  for (size_t i = 0; i < dims.size(); ++i) {
    node->sinkDims.push_back(pml::makeDimLiteral(dims[i]));
    node->sinkIdxs.push_back(idxs[i]);
  }
  for (const Operand& o : srcs) node->srcs.push_back({o.tensor, o.idxs});
  for (const Cons& c : cons) node->constraints.push_back({c.lhs, pml::makeDimLiteral(c.rhs)});
  pml::Evaluator local;
  local.verify(node);
  return node;
}

ExprPtr intrinsic(const std::string& fn, const std::vector<ExprPtr>& args, const std::string& name = "") {
  auto node = std::make_shared<ExprNode>(ExprNode::Intrinsic);
  node->op = fn;
  node->name = name;
  node->operands = args;
  pml::Evaluator local;
  local.verify(node);
  return node;
}

ExprPtr litInt(int64_t v) {
  auto node = std::make_shared<ExprNode>(ExprNode::ConstSigned);
  node->ivalue = v;
  return node;
}

ExprPtr litFloat(double v) {
  auto node = std::make_shared<ExprNode>(ExprNode::ConstFloat);
  node->fvalue = v;
  return node;
}

ExprPtr castTo(const ExprPtr& e, pml::DType dt) {
  auto node = std::make_shared<ExprNode>(ExprNode::Cast);
  node->dtype = dt;
  node->expr = e;
  return node;
}

ExprPtr reshapeTo(const ExprPtr& e, const std::vector<int64_t>& dims) {
  std::vector<ExprPtr> args = {e};
  for (int64_t d : dims) args.push_back(litInt(d));
  return intrinsic("reshape", args);
}

// ------------------------------------------------------------------ argument access

VarPtr exprValue(const ExprPtr& e) {
  auto v = std::make_shared<VarNode>();
  v->kind = VarNode::Expr;
  v->expr = e;
  return v;
}

const std::vector<VarPtr>& asTuple(const VarPtr& v, const char* what) {
  if (v->kind != VarNode::Tuple) throw std::runtime_error(std::string(what) + ": expected a tuple");
  return v->tuple;
}

ExprPtr asTensor(const VarPtr& v) {
  switch (v->kind) {
    case VarNode::Expr: return v->expr;
    case VarNode::Int: return litInt(v->i);
    case VarNode::Float: return litFloat(v->f);
    case VarNode::Dim: {
      auto node = std::make_shared<ExprNode>(ExprNode::Dim);
      node->dim = v->dim;
      return node;
    }
    default: throw std::runtime_error("Expected a tensor argument");
  }
}

int64_t asInt(const VarPtr& v) {
  if (v->kind == VarNode::Int) return v->i;
  if (v->kind == VarNode::Dim) {
    pml::Evaluator local;
    return local.evaluate(v->dim);
  }
  throw std::runtime_error("Expected an integer argument");
}

bool asBool(const VarPtr& v) { return asInt(v) != 0; }

std::string asStr(const VarPtr& v) {
  if (v->kind == VarNode::Str) return v->s;
  if (v->kind == VarNode::None) return "";
  throw std::runtime_error("Expected a string argument");
}

std::vector<int64_t> asIntTuple(const VarPtr& v) {
  std::vector<int64_t> out;
  if (v->kind == VarNode::None) return out;
  for (const VarPtr& e : asTuple(v, "integer tuple")) out.push_back(asInt(e));
  return out;
}

int64_t normalizeAxis(int64_t axis, size_t ndims, const char* op) {
  const int64_t a = axis < 0 ? axis + static_cast<int64_t>(ndims) : axis;
  if (a < 0 || a >= static_cast<int64_t>(ndims)) {
    throw std::runtime_error(std::string("Axis out of range for ") + op + " op (axis " + std::to_string(axis) +
                             " requested for tensors with " + std::to_string(ndims) + " dimensions)");
  }
  return a;
}

enum AutoPad { kPadExplicit = 0, kPadSameLower = 1, kPadSameUpper = 2, kPadValid = 3 };
enum Layout { kNXC = 0, kNCX = 1, kKCX = 2, kXCK = 3 };
enum PoolMode { kPoolAvg = 0, kPoolMax = 1, kPoolMin = 2, kPoolSum = 3 };

// plaidml/op/lib/ops.cc:347-382
void paddingAndOutput(int64_t in, int64_t filter, int64_t stride, int autopad, int64_t padLo, int64_t padHi,
                      int64_t dilation, int64_t dataDilation, bool ceilMode, int64_t* padBefore, int64_t* out) {
  const int64_t iEff = dataDilation * (in - 1) + 1;
  const int64_t fEff = dilation * (filter - 1) + 1;
  const int64_t ceilTerm = ceilMode ? stride - 1 : 0;
  switch (autopad) {
    case kPadExplicit:
      *padBefore = padLo;
      *out = (iEff + padLo + padHi - fEff + stride + ceilTerm) / stride;
      return;
    case kPadValid:
      *padBefore = 0;
      *out = (iEff - fEff + stride + ceilTerm) / stride;
      return;
    case kPadSameLower:
    case kPadSameUpper: {
      *out = (iEff + stride - 1) / stride;
      const int64_t lowerTerm = autopad == kPadSameLower ? 1 : 0;
      *padBefore = (std::max<int64_t>(0, (*out - 1) * stride + fEff - iEff) + lowerTerm) / 2;
      return;
    }
    default: throw std::runtime_error("Unexpected autopadding mode");
  }
}

// ------------------------------------------------------------------ reductions (AggregationAxes, ops.cc:71-127)

struct AggAxes {
  std::vector<PolyPtr> srcIdxs, dstIdxs;
  std::vector<int64_t> dstDims;
  std::set<size_t> axes;
  AggAxes(const pml::TensorShape& shape, const VarPtr& inAxes, bool keepdims) {
    const size_t n = shape.rank();
    for (size_t i = 0; i < n; ++i) srcIdxs.push_back(newIndex());
    if (inAxes->kind == VarNode::None) {
      for (size_t i = 0; i < n; ++i) axes.insert(i);
    } else if (inAxes->kind == VarNode::Tuple) {
      for (const VarPtr& a : inAxes->tuple) axes.insert(static_cast<size_t>(normalizeAxis(asInt(a), n, "aggregation")));
    } else {
      axes.insert(static_cast<size_t>(normalizeAxis(asInt(inAxes), n, "aggregation")));
    }
    for (size_t i = 0; i < n; ++i) {
      if (axes.count(i)) {
        if (keepdims) {
          dstIdxs.push_back(newIndex());
          dstDims.push_back(1);
        }
      } else {
        dstIdxs.push_back(srcIdxs[i]);
        dstDims.push_back(shape.sizes[i]);
      }
    }
  }
};

VarPtr reduceOp(const VarPtr& value, pml::AggKind agg, const char* name) {
  const auto& args = asTuple(value, name);
  if (args.size() != 3) throw std::runtime_error(std::string(name) + " expects 3 arguments");
  ExprPtr I = asTensor(args[0]);
  const pml::TensorShape shape = shapeOf(I);
  if (args[1]->kind == VarNode::Tuple && args[1]->tuple.empty()) return exprValue(I);
  AggAxes ax(shape, args[1], asBool(args[2]));
  return exprValue(contraction(agg, pml::ComboKind::none, ax.dstDims, ax.dstIdxs, {{I, ax.srcIdxs}}, {}, name));
}

// ------------------------------------------------------------------ operations

// plaidml/op/lib/ops.cc:1512-1561
VarPtr opDot(const VarPtr& value) {
  const auto& args = asTuple(value, "dot");
  if (args.size() != 3) throw std::runtime_error("dot expects 3 arguments");
  ExprPtr X = asTensor(args[0]), Y = asTensor(args[1]);
  std::string name = asStr(args[2]);
  if (name.empty()) name = "dot";
  const pml::TensorShape xs = shapeOf(X), ys = shapeOf(Y);
  if (xs.dtype != ys.dtype) {
    throw std::runtime_error(std::string("Invalid dtype in dot: X.dtype = '") + pml::dtypeName(xs.dtype) +
                             "', Y.dtype = '" + pml::dtypeName(ys.dtype) + "'");
  }
  if (xs.rank() == 1 && ys.rank() == 1) {
    if (xs.sizes[0] != ys.sizes[0]) throw std::runtime_error("bind dims mismatch in dot");
    PolyPtr i = newIndex();
    return exprValue(contraction(pml::AggKind::add, pml::ComboKind::mul, {}, {}, {{X, {i}}, {Y, {i}}}, {}, name));
  }
  if (xs.rank() >= 1 && ys.rank() >= 2) {
    std::vector<PolyPtr> xi, yi;
    for (size_t i = 0; i < xs.rank(); ++i) xi.push_back(newIndex());
    for (size_t i = 0; i < ys.rank(); ++i) yi.push_back(newIndex());
    PolyPtr z = newIndex();
    xi[xs.rank() - 1] = z;
    yi[ys.rank() - 2] = z;
    // (the two contracted dimensions are bound to separate dims in the reference: unequal sizes are not an error,
    // the shared index simply ranges over the smaller one -- plaidml/op/op_test.cc Dot multiplies 7x7x3x64 by 7x7x3x64)
    std::vector<int64_t> od;
    std::vector<PolyPtr> oi;
    for (size_t i = 0; i + 1 < xs.rank(); ++i) {
      od.push_back(xs.sizes[i]);
      oi.push_back(xi[i]);
    }
    for (size_t i = 0; i + 2 < ys.rank(); ++i) {
      od.push_back(ys.sizes[i]);
      oi.push_back(yi[i]);
    }
    od.push_back(ys.sizes.back());
    oi.push_back(yi.back());
    return exprValue(contraction(pml::AggKind::add, pml::ComboKind::mul, od, oi, {{X, xi}, {Y, yi}}, {}, name));
  }
  throw std::runtime_error("Unsupported dims for dot operation");
}

// plaidml/op/lib/ops.cc:879-1467, forward pass, ungrouped, layouts NXC/XCK or NCX/KCX
VarPtr opConvolution(const VarPtr& value) {
  const auto& args = asTuple(value, "convolution");
  if (args.size() != 18) throw std::runtime_error("Convolution op expects 18 arguments");
  ExprPtr I = asTensor(args[0]), F = asTensor(args[1]);
  std::vector<int64_t> strides = asIntTuple(args[2]);
  std::vector<int64_t> dilations = asIntTuple(args[3]);
  std::vector<int64_t> dataDilations = asIntTuple(args[4]);
  const std::vector<int64_t> filterShape = asIntTuple(args[5]);
  const int64_t groups = asInt(args[6]);
  const int autopad = static_cast<int>(asInt(args[7]));
  std::vector<int64_t> manualPadding = asIntTuple(args[8]);
  const int inputLayout = static_cast<int>(asInt(args[9]));
  const int filterLayout = static_cast<int>(asInt(args[10]));
  std::string name = asStr(args[13]);
  const int64_t derivMode = asInt(args[15]);
  if (name.empty()) name = "conv";
  const int groupLayout = static_cast<int>(asInt(args[11]));     // 0 none, 1 separate, 2 in C, 3 in K
  const int autogroup = static_cast<int>(asInt(args[14]));       // 0 ungrouped, 1 explicit, 2 auto, 3 depthwise
  if (derivMode != 0) throw std::runtime_error("Only the forward convolution is offered by the cuda target's op library");
  enum { kGKCX = 4, kXGCK = 5 };
  const bool nxc = inputLayout == kNXC;
  if (inputLayout != kNXC && inputLayout != kNCX) throw std::runtime_error("Invalid input_layout");
  if (filterLayout != kKCX && filterLayout != kXCK && filterLayout != kGKCX && filterLayout != kXGCK) {
    throw std::runtime_error("Invalid filter_layout");
  }
  const bool filterHasG = filterLayout == kGKCX || filterLayout == kXGCK;
  const bool filterSpatialFirst = filterLayout == kXCK || filterLayout == kXGCK;
  if (filterHasG != (groupLayout == 1)) {
    throw std::runtime_error("Filter layouts with a group dimension go with the SEPARATE group layout, and only with it");
  }
  const pml::TensorShape is = shapeOf(I), fs = shapeOf(F);
  if (is.rank() < 3 || fs.rank() != is.rank() + (filterHasG ? 1 : 0)) {
    throw std::runtime_error("Convolution input and filter ranks are inconsistent");
  }
  const size_t sr = is.rank() - 2;  // spatial rank
  if (strides.empty()) strides.assign(sr, 1);
  if (dilations.empty()) dilations.assign(sr, 1);
  if (dataDilations.empty()) dataDilations.assign(sr, 1);
  if (strides.size() != sr || dilations.size() != sr || dataDilations.size() != sr) {
    throw std::runtime_error("Convolution strides / dilations do not match the spatial rank");
  }
  for (size_t i = 0; i < sr; ++i) {
    if (strides[i] <= 0 || dilations[i] <= 0 || dataDilations[i] <= 0) {
      throw std::runtime_error("Convolution strides and dilations must be positive");
    }
  }
  if (!manualPadding.empty() && autopad != kPadExplicit) {
    throw std::runtime_error("Autopadding and manual padding both requested for single conv operation");
  }
  std::vector<int64_t> padLo, padHi;
  splitManualPadding(manualPadding, sr, &padLo, &padHi);
  const int64_t N = is.sizes[0];
  const int64_t CI = nxc ? is.sizes.back() : is.sizes[1];
  // filter dims: [G] K C x...   or   x... [G] C K
  std::vector<int64_t> X(sr), K(sr);
  int64_t FG = 1, FCI, FCO;
  if (filterSpatialFirst) {
    for (size_t i = 0; i < sr; ++i) K[i] = fs.sizes[i];
    size_t at = sr;
    if (filterHasG) FG = fs.sizes[at++];
    FCI = fs.sizes[at];
    FCO = fs.sizes[at + 1];
  } else {
    size_t at = 0;
    if (filterHasG) FG = fs.sizes[at++];
    FCO = fs.sizes[at];
    FCI = fs.sizes[at + 1];
    for (size_t i = 0; i < sr; ++i) K[i] = fs.sizes[at + 2 + i];
  }
  for (size_t i = 0; i < sr; ++i) X[i] = nxc ? is.sizes[1 + i] : is.sizes[2 + i];
  // group count (plaidml/op/lib/ops.cc:1029-1056)
  int64_t G = groups;
  switch (autogroup) {
    case 0:
    case 1: break;
    case 3:
      G = CI;
      if ((groupLayout == 3 || groupLayout == 1) && FCI != 1) {
        throw std::runtime_error("Depthwise convolutions take filters with one input channel per group");
      }
      if (groupLayout == 0) throw std::runtime_error("Unsupported group layout 'GroupLayout::NONE' used with autogroup mode DEPTHWISE");
      break;
    case 2:
      if (groupLayout == 1) {
        G = FG;
      } else if (groupLayout == 3) {
        if (FCI <= 0 || CI % FCI != 0) throw std::runtime_error("Cannot infer the group count: input channels are not a multiple of the filter's");
        G = CI / FCI;
      } else {
        throw std::runtime_error("Unsupported group layout used with autogroup mode AUTO");
      }
      break;
    default: throw std::runtime_error("Unrecognized AutoGroupMode");
  }
  if (G < 1) throw std::runtime_error("Convolution group count must be positive");
  int64_t CO = FCO;
  switch (groupLayout) {
    case 0:
      if (G != 1) throw std::runtime_error("Grouped convolutions need a group layout");
      if (FCI != CI) throw std::runtime_error("Convolution input channels do not match the filter");
      break;
    case 2:  // groups inside the filter's input-channel dimension
      if (FCI != CI) throw std::runtime_error("Convolution input channels do not match the filter");
      CO = FCO * G;
      break;
    case 3:  // groups inside the filter's output-channel dimension
      if (FCI * G != CI) throw std::runtime_error("Convolution input channels do not match the filter");
      break;
    case 1:
      if (FG != G) throw std::runtime_error("Convolution group count does not match the filter");
      if (FCI * G != CI) throw std::runtime_error("Convolution input channels do not match the filter");
      CO = FCO * G;
      break;
    default: throw std::runtime_error("Invalid group_layout");
  }
  if (CI % G != 0 || CO % G != 0) throw std::runtime_error("Channel counts must be multiples of the group count");
  if (!filterShape.empty()) {
    if (filterShape.size() != sr) throw std::runtime_error("Filter shape does not match the spatial rank");
    for (size_t i = 0; i < sr; ++i) {
      if (filterShape[i] != K[i]) throw std::runtime_error("Filter shape does not match the filter tensor");
    }
  }
  PolyPtr n = newIndex("n"), ci = newIndex("ci"), co = newIndex("co"), g = newIndex("g");
  std::vector<PolyPtr> x, k, inSpatial;
  std::vector<int64_t> outSpatial;
  for (size_t i = 0; i < sr; ++i) {
    x.push_back(newIndex("x" + std::to_string(i)));
    k.push_back(newIndex("k" + std::to_string(i)));
    int64_t padBefore = 0, outSize = 0;
    paddingAndOutput(X[i], K[i], strides[i], autopad, padLo[i], padHi[i], dilations[i], dataDilations[i], false, &padBefore,
                     &outSize);
    outSpatial.push_back(outSize);
    PolyPtr pos = strides[i] * x[i] + dilations[i] * k[i] - padBefore;
    // data dilation: only positions that fall on an input element (an integral quotient) contribute
    if (dataDilations[i] != 1) pos = polyOp(pml::AffineOp::Div, pos, polyLit(dataDilations[i]));
    inSpatial.push_back(pos);
  }
  const bool grouped = groupLayout != 0;
  PolyPtr iChan = grouped ? (CI / G) * g + ci : ci;
  PolyPtr oChan = grouped ? (CO / G) * g + co : co;
  PolyPtr fCo = co, fCi = ci;
  std::vector<Cons> cons;
  if (groupLayout == 2) {
    fCi = (CI / G) * g + ci;
    cons.push_back({ci, CI / G});
  } else if (groupLayout == 3) {
    fCo = (CO / G) * g + co;
    cons.push_back({co, CO / G});
  }
  std::vector<PolyPtr> iIdx, fIdx, oIdx;
  std::vector<int64_t> oDims;
  iIdx.push_back(n);
  oIdx.push_back(n);
  oDims.push_back(N);
  if (nxc) {
    for (auto& p : inSpatial) iIdx.push_back(p);
    iIdx.push_back(iChan);
    for (size_t i = 0; i < sr; ++i) {
      oIdx.push_back(x[i]);
      oDims.push_back(outSpatial[i]);
    }
    oIdx.push_back(oChan);
    oDims.push_back(CO);
  } else {
    iIdx.push_back(iChan);
    for (auto& p : inSpatial) iIdx.push_back(p);
    oIdx.push_back(oChan);
    oDims.push_back(CO);
    for (size_t i = 0; i < sr; ++i) {
      oIdx.push_back(x[i]);
      oDims.push_back(outSpatial[i]);
    }
  }
  if (filterSpatialFirst) {
    for (auto& p : k) fIdx.push_back(p);
    if (filterHasG) fIdx.push_back(g);
    fIdx.push_back(fCi);
    fIdx.push_back(fCo);
  } else {
    if (filterHasG) fIdx.push_back(g);
    fIdx.push_back(fCo);
    fIdx.push_back(fCi);
    for (auto& p : k) fIdx.push_back(p);
  }
  return exprValue(contraction(pml::AggKind::add, pml::ComboKind::mul, oDims, oIdx, {{I, iIdx}, {F, fIdx}}, cons, name));
}

// plaidml/op/lib/ops.cc:2562-2703
VarPtr opPool(const VarPtr& value) {
  const auto& args = asTuple(value, "pool");
  if (args.size() != 10) throw std::runtime_error("PlaidML pool op expects 10 arguments");
  ExprPtr I = asTensor(args[0]);
  const int mode = static_cast<int>(asInt(args[1]));
  const std::vector<int64_t> poolSize = asIntTuple(args[2]);
  const std::vector<int64_t> strides = asIntTuple(args[3]);
  const int autopad = static_cast<int>(asInt(args[4]));
  std::vector<int64_t> manualPadding = asIntTuple(args[5]);
  const int layout = static_cast<int>(asInt(args[6]));
  const bool includePadding = asBool(args[7]);
  const bool ceilMode = asBool(args[8]);
  std::string name = asStr(args[9]);
  if (name.empty()) name = "pool";
  const pml::TensorShape is = shapeOf(I);
  const size_t sr = poolSize.size();
  if (!manualPadding.empty() && autopad != kPadExplicit) {
    throw std::runtime_error("Autopadding and manual padding both requested for single pool operation");
  }
  if (strides.size() != sr) throw std::runtime_error("Inconsistent spatial rank in pool op");
  if (is.rank() != sr + 2) throw std::runtime_error("Inconsistent spatial rank in pool op");
  if (layout != kNXC && layout != kNCX) throw std::runtime_error("Tensor layout requested in pool op does not apply to pooling");
  std::vector<int64_t> padLo, padHi;
  splitManualPadding(manualPadding, sr, &padLo, &padHi);
  const bool nxc = layout == kNXC;
  PolyPtr n = newIndex("n"), c = newIndex("c");
  std::vector<PolyPtr> x, k, inSpatial;
  std::vector<int64_t> outSpatial;
  std::vector<Cons> cons;
  for (size_t i = 0; i < sr; ++i) {
    const int64_t X = nxc ? is.sizes[1 + i] : is.sizes[2 + i];
    x.push_back(newIndex("x" + std::to_string(i)));
    k.push_back(newIndex("k" + std::to_string(i)));
    int64_t padBefore = 0, outSize = 0;
    paddingAndOutput(X, poolSize[i], strides[i], autopad, padLo[i], padHi[i], 1, 1, ceilMode, &padBefore, &outSize);
    outSpatial.push_back(outSize);
    inSpatial.push_back(strides[i] * x[i] + k[i] - padBefore);
    cons.push_back({k[i], poolSize[i]});
  }
  const int64_t N = is.sizes[0], C = nxc ? is.sizes.back() : is.sizes[1];
  std::vector<PolyPtr> iIdx = {n}, oIdx = {n};
  std::vector<int64_t> oDims = {N};
  if (!nxc) {
    iIdx.push_back(c);
    oIdx.push_back(c);
    oDims.push_back(C);
  }
  for (size_t i = 0; i < sr; ++i) {
    iIdx.push_back(inSpatial[i]);
    oIdx.push_back(x[i]);
    oDims.push_back(outSpatial[i]);
  }
  if (nxc) {
    iIdx.push_back(c);
    oIdx.push_back(c);
    oDims.push_back(C);
  }
  const pml::AggKind agg = mode == kPoolMax ? pml::AggKind::max : (mode == kPoolMin ? pml::AggKind::min : pml::AggKind::add);
  ExprPtr O = contraction(agg, pml::ComboKind::none, oDims, oIdx, {{I, iIdx}}, cons, name);
  if (mode != kPoolAvg) return exprValue(O);
  if (includePadding) {
    int64_t total = 1;
    for (int64_t s : poolSize) total *= s;
    return exprValue(intrinsic("div", {O, litInt(total)}));
  }
  // average over the taps that fall inside the input: count them with a second contraction
  ExprPtr one = castTo(litInt(1), is.dtype);
  ExprPtr ones = contraction(pml::AggKind::assign, pml::ComboKind::none, is.sizes, oIdx, {{one, {}}}, {}, name);
  ExprPtr count = contraction(pml::AggKind::add, pml::ComboKind::none, oDims, oIdx, {{ones, iIdx}}, cons, name);
  return exprValue(intrinsic("div", {O, count}));
}

// plaidml/op/lib/ops.cc:2705-2728
VarPtr opRelu(const VarPtr& value) {
  const auto& args = asTuple(value, "relu");
  if (args.size() != 5) throw std::runtime_error("relu expects 5 arguments");
  ExprPtr I = asTensor(args[0]);
  const VarPtr& alpha = args[1];
  const VarPtr& maxValue = args[2];
  const VarPtr& threshold = args[3];
  const double T = threshold->kind == VarNode::None ? 0.0 : (threshold->kind == VarNode::Float ? threshold->f : static_cast<double>(asInt(threshold)));
  const bool alphaZero = alpha->kind == VarNode::None || (alpha->kind == VarNode::Float && alpha->f == 0.0);
  if (alphaZero && maxValue->kind == VarNode::None && T == 0.0) return exprValue(intrinsic("relu", {I}));
  const pml::DType dt = shapeOf(I).dtype;
  ExprPtr A = alpha->kind == VarNode::None ? litFloat(0.0) : asTensor(alpha);
  ExprPtr shifted = intrinsic("sub", {I, litFloat(T)});
  ExprPtr O = intrinsic("select", {intrinsic("cmp_lt", {I, litFloat(T)}), castTo(intrinsic("mul", {A, shifted}), dt), I});
  if (maxValue->kind != VarNode::None) {
    ExprPtr M = castTo(asTensor(maxValue), dt);
    O = intrinsic("select", {intrinsic("cmp_lt", {O, M}), O, M});
  }
  return exprValue(O);
}

// plaidml/op/lib/ops.cc:1970-2003
VarPtr opMean(const VarPtr& value) {
  const auto& args = asTuple(value, "mean");
  if (args.size() != 3) throw std::runtime_error("mean expects 3 arguments");
  ExprPtr I = asTensor(args[0]);
  const pml::TensorShape shape = shapeOf(I);
  if (shape.rank() == 0) return exprValue(I);
  if (args[1]->kind == VarNode::Tuple && args[1]->tuple.empty()) return exprValue(I);
  AggAxes ax(shape, args[1], asBool(args[2]));
  ExprPtr SO = contraction(pml::AggKind::add, pml::ComboKind::none, ax.dstDims, ax.dstIdxs, {{I, ax.srcIdxs}}, {}, "mean");
  int64_t denom = 1;
  for (size_t a : ax.axes) denom *= shape.sizes[a];
  return exprValue(intrinsic("div", {SO, litInt(denom)}));
}

// plaidml/op/lib/ops.cc:3049-3099 (the soft-max axis must be the last one here)
VarPtr opSoftmax(const VarPtr& value) {
  const auto& args = asTuple(value, "softmax");
  if (args.size() != 3) throw std::runtime_error("softmax expects 3 arguments");
  ExprPtr I = asTensor(args[0]);
  std::string name = asStr(args[2]);
  if (name.empty()) name = "softmax";
  const pml::TensorShape shape = shapeOf(I);
  const int64_t axis = normalizeAxis(asInt(args[1]), shape.rank(), "softmax");
  if (axis != static_cast<int64_t>(shape.rank()) - 1) {
    throw std::runtime_error("softmax over an inner axis: transpose it to the last axis first");
  }
  std::vector<PolyPtr> idxs, ridxs;
  std::vector<int64_t> rdims = shape.sizes;
  for (size_t i = 0; i < shape.rank(); ++i) idxs.push_back(newIndex());
  ridxs = idxs;
  rdims[axis] = 1;
  ridxs[axis] = polyLit(0);
  ExprPtr M = contraction(pml::AggKind::max, pml::ComboKind::none, rdims, ridxs, {{I, idxs}}, {}, name);
  ExprPtr E = intrinsic("exp", {intrinsic("sub", {I, M})});
  ExprPtr Nrm = contraction(pml::AggKind::add, pml::ComboKind::none, rdims, ridxs, {{E, idxs}}, {}, name);
  return exprValue(intrinsic("div", {E, Nrm}));
}

VarPtr unary(const VarPtr& value, const char* fn) {
  ExprPtr I = value->kind == VarNode::Tuple ? asTensor(value->tuple.at(0)) : asTensor(value);
  return exprValue(intrinsic(fn, {I}));
}

VarPtr opSquare(const VarPtr& value) {
  ExprPtr I = value->kind == VarNode::Tuple ? asTensor(value->tuple.at(0)) : asTensor(value);
  return exprValue(intrinsic("mul", {I, I}));
}

VarPtr opMaximum(const VarPtr& value) {
  const auto& args = asTuple(value, "maximum");
  if (args.size() != 2) throw std::runtime_error("maximum expects 2 arguments");
  ExprPtr X = asTensor(args[0]), Y = asTensor(args[1]);
  return exprValue(intrinsic("select", {intrinsic("cmp_lt", {X, Y}), Y, X}));
}

VarPtr opMinimum(const VarPtr& value) {
  const auto& args = asTuple(value, "minimum");
  if (args.size() != 2) throw std::runtime_error("minimum expects 2 arguments");
  ExprPtr X = asTensor(args[0]), Y = asTensor(args[1]);
  return exprValue(intrinsic("select", {intrinsic("cmp_lt", {X, Y}), X, Y}));
}

VarPtr opClip(const VarPtr& value) {
  const auto& args = asTuple(value, "clip");
  if (args.size() != 3) throw std::runtime_error("clip expects 3 arguments");
  ExprPtr O = asTensor(args[0]);
  if (args[1]->kind != VarNode::None) {
    ExprPtr lo = asTensor(args[1]);
    O = intrinsic("select", {intrinsic("cmp_gt", {O, lo}), O, lo});
  }
  if (args[2]->kind != VarNode::None) {
    ExprPtr hi = asTensor(args[2]);
    O = intrinsic("select", {intrinsic("cmp_lt", {O, hi}), O, hi});
  }
  return exprValue(O);
}

VarPtr opReshape(const VarPtr& value) {
  const auto& args = asTuple(value, "reshape");
  if (args.size() != 2) throw std::runtime_error("reshape expects 2 arguments");
  ExprPtr I = asTensor(args[0]);
  const pml::TensorShape shape = shapeOf(I);
  std::vector<int64_t> dims;
  int64_t known = 1;
  int fill = -1;
  const auto& want = asTuple(args[1], "reshape dims");
  for (size_t i = 0; i < want.size(); ++i) {
    int64_t d = asInt(want[i]);
    if (d == 0) d = i < shape.rank() ? shape.sizes[i] : 0;  // 0 copies the input extent
    if (d == -1) {
      if (fill >= 0) throw std::runtime_error("reshape: at most one dimension may be -1");
      fill = static_cast<int>(i);
      d = 1;
    } else {
      known *= d;
    }
    dims.push_back(d);
  }
  if (fill >= 0) dims[fill] = known ? shape.elements() / known : 0;
  return exprValue(reshapeTo(I, dims));
}

VarPtr opTranspose(const VarPtr& value) {
  const auto& args = asTuple(value, "transpose");
  if (args.size() != 2) throw std::runtime_error("transpose expects 2 arguments");
  ExprPtr I = asTensor(args[0]);
  const pml::TensorShape shape = shapeOf(I);
  std::vector<int64_t> pattern;
  if (args[1]->kind == VarNode::None) {
    for (size_t i = 0; i < shape.rank(); ++i) pattern.push_back(static_cast<int64_t>(shape.rank() - 1 - i));
  } else {
    pattern = asIntTuple(args[1]);
  }
  if (pattern.size() != shape.rank()) throw std::runtime_error("transpose pattern does not match the tensor rank");
  std::vector<PolyPtr> iIdx, oIdx;
  std::vector<int64_t> oDims;
  for (size_t i = 0; i < shape.rank(); ++i) iIdx.push_back(newIndex());
  for (int64_t a : pattern) {
    const int64_t ax = normalizeAxis(a, shape.rank(), "transpose");
    oIdx.push_back(iIdx[ax]);
    oDims.push_back(shape.sizes[ax]);
  }
  return exprValue(contraction(pml::AggKind::assign, pml::ComboKind::none, oDims, oIdx, {{I, iIdx}}, {}, "transpose"));
}

VarPtr opSqueeze(const VarPtr& value) {
  const auto& args = asTuple(value, "squeeze");
  ExprPtr I = asTensor(args.at(0));
  const pml::TensorShape shape = shapeOf(I);
  std::set<int64_t> axes;
  for (int64_t a : asIntTuple(args.at(1))) axes.insert(normalizeAxis(a, shape.rank(), "squeeze"));
  std::vector<int64_t> dims;
  for (size_t i = 0; i < shape.rank(); ++i) {
    if (axes.count(static_cast<int64_t>(i))) {
      if (shape.sizes[i] != 1) throw std::runtime_error("squeeze: axis extent is not 1");
    } else {
      dims.push_back(shape.sizes[i]);
    }
  }
  return exprValue(reshapeTo(I, dims));
}

VarPtr opUnsqueeze(const VarPtr& value) {
  const auto& args = asTuple(value, "unsqueeze");
  ExprPtr I = asTensor(args.at(0));
  const pml::TensorShape shape = shapeOf(I);
  std::vector<int64_t> axes = asIntTuple(args.at(1));
  const size_t newRank = shape.rank() + axes.size();
  std::set<int64_t> at;
  for (int64_t a : axes) at.insert(normalizeAxis(a, newRank, "unsqueeze"));
  std::vector<int64_t> dims;
  size_t src = 0;
  for (size_t i = 0; i < newRank; ++i) {
    if (at.count(static_cast<int64_t>(i))) dims.push_back(1);
    else dims.push_back(shape.sizes[src++]);
  }
  return exprValue(reshapeTo(I, dims));
}

VarPtr opFlip(const VarPtr& value) {
  const auto& args = asTuple(value, "flip");
  ExprPtr I = asTensor(args.at(0));
  const pml::TensorShape shape = shapeOf(I);
  const int64_t axis = normalizeAxis(asInt(args.at(1)), shape.rank(), "flip");
  std::vector<PolyPtr> iIdx, oIdx;
  for (size_t i = 0; i < shape.rank(); ++i) iIdx.push_back(newIndex());
  oIdx = iIdx;
  oIdx[axis] = polyLit(shape.sizes[axis] - 1) - iIdx[axis];
  return exprValue(contraction(pml::AggKind::assign, pml::ComboKind::none, shape.sizes, oIdx, {{I, iIdx}}, {}, "flip"));
}

// plaidml/op/lib/ops.cc cumsum: O[.., i, ..] += I[.., i - k, ..] with k < N
VarPtr opCumsum(const VarPtr& value) {
  const auto& args = asTuple(value, "cumsum");
  ExprPtr I = asTensor(args.at(0));
  const pml::TensorShape shape = shapeOf(I);
  const int64_t axis = normalizeAxis(asInt(args.at(1)), shape.rank(), "cumsum");
  std::vector<PolyPtr> oIdx, iIdx;
  for (size_t i = 0; i < shape.rank(); ++i) oIdx.push_back(newIndex());
  iIdx = oIdx;
  PolyPtr k = newIndex("k");
  // plaidml/op/lib/ops.cc:1490-1511: the exclusive form leaves the element itself out (O[i] = sum of I[j], j < i)
  const bool exclusive = args.size() > 2 && asBool(args[2]);
  iIdx[axis] = exclusive ? oIdx[axis] - k - 1 : oIdx[axis] - k;
  return exprValue(contraction(pml::AggKind::add, pml::ComboKind::none, shape.sizes, oIdx, {{I, iIdx}},
                               {{k, shape.sizes[axis]}}, "cumsum"));
}

VarPtr opVariance(const VarPtr& value) {
  const auto& args = asTuple(value, "variance");
  if (args.size() != 3) throw std::runtime_error("variance expects 3 arguments");
  ExprPtr I = asTensor(args[0]);
  auto keep = std::make_shared<VarNode>();
  keep->kind = VarNode::Int;
  keep->i = 1;
  auto meanArgs = std::make_shared<VarNode>();
  meanArgs->kind = VarNode::Tuple;
  meanArgs->tuple = {args[0], args[1], keep};
  ExprPtr mean = opMean(meanArgs)->expr;
  ExprPtr diff = intrinsic("sub", {I, mean});
  auto sqArgs = std::make_shared<VarNode>();
  sqArgs->kind = VarNode::Tuple;
  sqArgs->tuple = {exprValue(intrinsic("mul", {diff, diff})), args[1], args[2]};
  return opMean(sqArgs);
}

VarPtr opSpatialPadding(const VarPtr& value) {
  const auto& args = asTuple(value, "spatial_padding");
  if (args.size() != 4) throw std::runtime_error("spatial_padding expects 4 arguments");
  ExprPtr I = asTensor(args[0]);
  const std::vector<int64_t> lo = asIntTuple(args[1]), hi = asIntTuple(args[2]);
  const int layout = static_cast<int>(asInt(args[3]));
  const pml::TensorShape shape = shapeOf(I);
  const size_t sr = shape.rank() - 2;
  if (lo.size() != sr || hi.size() != sr) throw std::runtime_error("spatial_padding: pads do not match the spatial rank");
  const size_t first = layout == kNXC ? 1 : 2;
  std::vector<PolyPtr> iIdx, oIdx;
  std::vector<int64_t> oDims = shape.sizes;
  for (size_t i = 0; i < shape.rank(); ++i) iIdx.push_back(newIndex());
  oIdx = iIdx;
  for (size_t i = 0; i < sr; ++i) {
    oDims[first + i] += lo[i] + hi[i];
    oIdx[first + i] = iIdx[first + i] + lo[i];
  }
  return exprValue(contraction(pml::AggKind::assign, pml::ComboKind::none, oDims, oIdx, {{I, iIdx}}, {}, "spatial_padding"));
}

VarPtr opElu(const VarPtr& value) {
  const auto& args = asTuple(value, "elu");
  ExprPtr I = asTensor(args.at(0));
  ExprPtr alpha = asTensor(args.at(1));
  ExprPtr neg = intrinsic("mul", {alpha, intrinsic("sub", {intrinsic("exp", {I}), litFloat(1.0)})});
  return exprValue(intrinsic("select", {intrinsic("cmp_lt", {I, litFloat(0.0)}), castTo(neg, shapeOf(I).dtype), I}));
}

// ------------------------------------------------------------------ small value builders

VarPtr intVar(int64_t v) {
  auto n = std::make_shared<VarNode>();
  n->kind = VarNode::Int;
  n->i = v;
  return n;
}

VarPtr noneVar() { return std::make_shared<VarNode>(); }

VarPtr tupleVar(std::vector<VarPtr> elts) {
  auto n = std::make_shared<VarNode>();
  n->kind = VarNode::Tuple;
  n->tuple = std::move(elts);
  return n;
}

VarPtr intTupleVar(const std::vector<int64_t>& v) {
  std::vector<VarPtr> e;
  for (int64_t x : v) e.push_back(intVar(x));
  return tupleVar(std::move(e));
}

ExprPtr binary(const char* fn, const ExprPtr& a, const ExprPtr& b) { return intrinsic(fn, {a, b}); }

// 0 / 1 in the tensor's own type: select(I == 0, 0, 1) (plaidml/op/lib/ops.cc:459-461)
ExprPtr asZeroOne(const ExprPtr& I, pml::DType dt) {
  return intrinsic("select", {binary("cmp_eq", I, litInt(0)), castTo(litInt(0), dt), castTo(litInt(1), dt)});
}

// plaidml/op/lib/ops.cc:450-503: all = product of the 0/1 image, any = its sum compared with 0; u8 results
VarPtr opAllAny(const VarPtr& value, bool all) {
  const char* name = all ? "all" : "any";
  const auto& args = asTuple(value, name);
  if (args.size() != 3) throw std::runtime_error(std::string(name) + " expects 3 arguments");
  ExprPtr I = asTensor(args[0]);
  const pml::TensorShape shape = shapeOf(I);
  ExprPtr B = asZeroOne(I, shape.dtype);
  if (shape.rank() == 0 || (args[1]->kind == VarNode::Tuple && args[1]->tuple.empty())) {
    return exprValue(castTo(B, pml::DType::ui8));
  }
  AggAxes ax(shape, args[1], asBool(args[2]));
  ExprPtr R = contraction(all ? pml::AggKind::mul : pml::AggKind::add, pml::ComboKind::none, ax.dstDims, ax.dstIdxs,
                          {{B, ax.srcIdxs}}, {}, name);
  if (!all) R = asZeroOne(R, shape.dtype);
  return exprValue(castTo(R, pml::DType::ui8));
}

// plaidml/op/lib/ops.cc:505-521: the maximum, then the largest flattened index whose element equals it
VarPtr opArgmax(const VarPtr& value) {
  const auto& args = asTuple(value, "argmax");
  if (args.size() != 2) throw std::runtime_error("argmax expects 2 arguments");
  ExprPtr I = asTensor(args[0]);
  const pml::TensorShape shape = shapeOf(I);
  AggAxes ax(shape, args[1], false);
  ExprPtr M = contraction(pml::AggKind::max, pml::ComboKind::none, ax.dstDims, ax.dstIdxs, {{I, ax.srcIdxs}}, {}, "argmax");
  std::vector<ExprPtr> ixArgs;
  std::vector<PolyPtr> redIdxs;
  std::vector<int64_t> redDims;
  for (size_t a : ax.axes) {
    redIdxs.push_back(ax.srcIdxs[a]);
    redDims.push_back(shape.sizes[a]);
  }
  // index(dims, 0): a tensor of shape `reduce dims` whose elements are their own coordinate along axis 0
  ixArgs.push_back(litInt(0));
  for (int64_t d : redDims) ixArgs.push_back(litInt(d));
  ExprPtr IX = intrinsic("index", ixArgs);
  ExprPtr AM = contraction(pml::AggKind::max, pml::ComboKind::cond, ax.dstDims, ax.dstIdxs,
                           {{I, ax.srcIdxs}, {M, ax.dstIdxs}, {IX, redIdxs}}, {}, "argmax");
  return exprValue(castTo(AM, pml::DType::ui32));
}

// plaidml/op/lib/ops.cc:523-544
VarPtr opBinaryCrossentropy(const VarPtr& value) {
  const auto& args = asTuple(value, "binary_crossentropy");
  if (args.size() != 3) throw std::runtime_error("binary_crossentropy expects 3 arguments");
  ExprPtr T = asTensor(args[0]);
  if (args[2]->kind != VarNode::Float && args[2]->kind != VarNode::Int) throw std::runtime_error("Expected a float argument");
  const double eps = args[2]->kind == VarNode::Float ? args[2]->f : static_cast<double>(args[2]->i);
  if (eps < 0. || eps >= 0.5) {
    throw std::runtime_error("The epsilon used in binary_crossentropy must be between 0 and 0.5, received " + std::to_string(eps));
  }
  auto lo = std::make_shared<VarNode>();
  lo->kind = VarNode::Float;
  lo->f = eps;
  auto hi = std::make_shared<VarNode>();
  hi->kind = VarNode::Float;
  hi->f = 1. - eps;
  ExprPtr P = opClip(tupleVar({args[1], lo, hi}))->expr;
  // -T * log(P) - (1 - T) * log(1 - P)
  ExprPtr a = binary("mul", intrinsic("neg", {T}), intrinsic("log", {P}));
  ExprPtr b = binary("mul", binary("sub", litInt(1), T), intrinsic("log", {binary("sub", litInt(1), P)}));
  return exprValue(binary("sub", a, b));
}

// plaidml/op/lib/ops.cc:546-584: input dim i feeds output dim axes[i]; size-1 input dims repeat
VarPtr opBroadcast(const VarPtr& value) {
  const auto& args = asTuple(value, "broadcast");
  if (args.size() != 3) throw std::runtime_error("PlaidML broadcast op expects 3 arguments (received " + std::to_string(args.size()) + ")");
  ExprPtr I = asTensor(args[0]);
  const pml::TensorShape shape = shapeOf(I);
  const std::vector<int64_t> target = asIntTuple(args[1]);
  const std::vector<int64_t> axes = asIntTuple(args[2]);
  if (shape.rank() != axes.size()) {
    throw std::runtime_error("Mismatched broadcast axes (received " + std::to_string(axes.size()) +
                             " broadcast axes for input tensor of rank " + std::to_string(shape.rank()) + ")");
  }
  std::vector<PolyPtr> oIdx, iIdx;
  for (size_t i = 0; i < target.size(); ++i) oIdx.push_back(newIndex());
  for (size_t i = 0; i < axes.size(); ++i) {
    if (shape.sizes[i] == 1) {
      iIdx.push_back(polyLit(0));
    } else {
      if (axes[i] < 0 || axes[i] >= static_cast<int64_t>(target.size())) throw std::runtime_error("broadcast axis out of range");
      iIdx.push_back(oIdx[axes[i]]);
    }
  }
  return exprValue(contraction(pml::AggKind::assign, pml::ComboKind::none, target, oIdx, {{I, iIdx}}, {}, "broadcast"));
}

// plaidml/op/lib/ops.cc:608-668: each input assigned into its span of a zero-filled result, results added
ExprPtr concatExprs(const std::vector<ExprPtr>& tensors, int64_t rawAxis) {
  if (tensors.empty()) throw std::runtime_error("The concatenate op requires at least one input tensor");
  const pml::TensorShape first = shapeOf(tensors[0]);
  const size_t nd = first.rank();
  const size_t axis = static_cast<size_t>(normalizeAxis(rawAxis, nd, "concatenate"));
  std::vector<int64_t> dims = first.sizes;
  std::vector<int64_t> offsets;
  int64_t total = 0;
  for (const ExprPtr& t : tensors) {
    const pml::TensorShape ts = shapeOf(t);
    if (ts.rank() != nd) throw std::runtime_error("concatenate: ranks differ");
    for (size_t d = 0; d < nd; ++d) {
      if (d != axis && ts.sizes[d] != first.sizes[d]) throw std::runtime_error("concatenate: bind dims mismatch off the axis");
    }
    offsets.push_back(total);
    total += ts.sizes[axis];
  }
  dims[axis] = total;
  ExprPtr result;
  for (size_t t = 0; t < tensors.size(); ++t) {
    std::vector<PolyPtr> iIdx, oIdx;
    for (size_t d = 0; d < nd; ++d) iIdx.push_back(newIndex(d == axis ? "a" : "n" + std::to_string(d)));
    oIdx = iIdx;
    oIdx[axis] = iIdx[axis] + offsets[t];
    ExprPtr R = contraction(pml::AggKind::assign, pml::ComboKind::none, dims, oIdx, {{tensors[t], iIdx}}, {}, "concatenate");
    result = result ? binary("add", result, R) : R;
  }
  return result;
}

VarPtr opConcatenate(const VarPtr& value) {
  const auto& args = asTuple(value, "concatenate");
  if (args.size() != 2) throw std::runtime_error("concatenate expects 2 arguments");
  std::vector<ExprPtr> tensors;
  for (const VarPtr& v : asTuple(args[0], "concatenate tensors")) tensors.push_back(asTensor(v));
  return exprValue(concatExprs(tensors, asInt(args[1])));
}

// ------------------------------------------------------------------ gather / sort family

VarPtr intValue(int64_t i) {
  auto v = std::make_shared<VarNode>();
  v->kind = VarNode::Int;
  v->i = i;
  return v;
}

VarPtr tupleValue(std::vector<VarPtr> items) {
  auto v = std::make_shared<VarNode>();
  v->kind = VarNode::Tuple;
  v->tuple = std::move(items);
  return v;
}

VarPtr intTupleValue(const std::vector<int64_t>& items) {
  std::vector<VarPtr> vs;
  for (int64_t i : items) vs.push_back(intValue(i));
  return tupleValue(std::move(vs));
}

// index(dims, axis): a tensor of shape `dims` whose elements are their own coordinate along `axis`
ExprPtr indexExpr(const std::vector<int64_t>& dims, int64_t axis) {
  std::vector<ExprPtr> args = {litInt(axis)};
  for (int64_t d : dims) args.push_back(litInt(d));
  return intrinsic("index", args);
}

// The gather intrinsic with its nine operands (plaidml/edsl/edsl.h:1645-1690); interpolation 3 = none.
ExprPtr gatherExpr(const ExprPtr& x, const ExprPtr& y, int64_t axis, int64_t interpolation = 3, int64_t nearest = 0,
                   double cubeCoeff = -0.75, int64_t mode = 0, int64_t batchDims = 0, int64_t outOfBounds = 0) {
  return intrinsic("gather", {x, y, litInt(axis), litInt(interpolation), litInt(nearest), litFloat(cubeCoeff), litInt(mode),
                              litInt(batchDims), litInt(outOfBounds)});
}

VarPtr opUnsqueeze(const VarPtr& value);
VarPtr opSqueeze(const VarPtr& value);
VarPtr opExplicitPadding(const VarPtr& value);
VarPtr opBroadcast(const VarPtr& value);

ExprPtr unsqueezeExpr(const ExprPtr& I, const std::vector<int64_t>& axes) {
  return opUnsqueeze(tupleValue({exprValue(I), intTupleValue(axes)}))->expr;
}

ExprPtr squeezeExpr(const ExprPtr& I, const std::vector<int64_t>& axes) {
  return opSqueeze(tupleValue({exprValue(I), intTupleValue(axes)}))->expr;
}

// plaidml/op/lib/ops.cc:1728-1801.  Without interpolation: the gather intrinsic in nd mode.  LINEAR: the data is
// zero-padded by two along every addressed dim, and the 2^K corners around each (float) index row are gathered
// and blended.
ExprPtr gatherNDExpr(const ExprPtr& I, const ExprPtr& idx, int64_t batchDims, int64_t interpolation) {
  const pml::TensorShape iShape = shapeOf(I);
  const pml::TensorShape idxShape = shapeOf(idx);
  if (idxShape.rank() == 0) throw std::runtime_error("gatherND: indices need at least one dimension");
  const int64_t rank = static_cast<int64_t>(iShape.rank());
  const int64_t k = idxShape.sizes.back();
  if (k + batchDims > rank) {
    throw std::runtime_error("Invalid Indices: Data(shape: '" + iShape.str() + "'), Indices(shape: '" + idxShape.str() +
                             "'), BatchDims('" + std::to_string(batchDims) + "')");
  }
  if (interpolation == 3) return gatherExpr(I, idx, 0, interpolation, 0, -0.75, 1, batchDims, 0);
  if (interpolation != 1) throw std::runtime_error("Unsupported InterpolationMode in gatherND");
  const int64_t padLength = 2;
  std::vector<int64_t> pads(rank, 0);
  for (int64_t i = 0; i < k; ++i) pads[i + batchDims] = padLength;
  ExprPtr X = opExplicitPadding(tupleValue({exprValue(I), intTupleValue(pads), intTupleValue(pads), intValue(0),
                                            exprValue(litInt(0))}))->expr;
  ExprPtr Y = binary("add", idx, litInt(padLength));
  if (static_cast<int64_t>(idxShape.rank()) - batchDims != 2) {
    throw std::runtime_error(
        " Indices dimension should be batch_dims plus two in interpolated gatherND, please reshape indices to satisfy this "
        "requirement.");
  }
  ExprPtr Yf = castTo(Y, pml::DType::f32);
  const int64_t lastAxis = static_cast<int64_t>(idxShape.rank()) - 1;
  std::vector<ExprPtr> dims;
  std::vector<std::array<ExprPtr, 2>> bounds;
  for (int64_t i = 0; i < k; ++i) {
    ExprPtr at = binary("add", castTo(indexExpr({1}, 0), pml::DType::si32), litInt(i));
    ExprPtr dim = gatherExpr(Yf, at, lastAxis);
    dims.push_back(dim);
    ExprPtr lo = intrinsic("floor", {dim});
    bounds.push_back({lo, binary("add", intrinsic("floor", {dim}), litFloat(1.0))});
  }
  ExprPtr zero = castTo(indexExpr({1}, 0), pml::DType::f32);
  ExprPtr result = zero;
  const int64_t corners = int64_t{1} << k;
  for (int64_t i = 0; i < corners; ++i) {
    std::vector<ExprPtr> corner;
    ExprPtr coeff = binary("add", zero, litInt(1));
    int64_t j = i;
    for (int64_t d = 0; d < k; ++d, j /= 2) {
      const int side = static_cast<int>(j % 2);
      corner.push_back(bounds[d][side]);
      coeff = side == 0 ? binary("mul", coeff, squeezeExpr(binary("sub", bounds[d][1], dims[d]), {-1}))
                        : binary("mul", coeff, squeezeExpr(binary("sub", dims[d], bounds[d][0]), {-1}));
    }
    ExprPtr cornerIdx = castTo(concatExprs(corner, -1), pml::DType::si32);
    ExprPtr vertex = gatherNDExpr(X, cornerIdx, batchDims, 3);
    const pml::TensorShape vShape = shapeOf(vertex);
    std::vector<int64_t> axes;
    for (size_t a = 0; a < shapeOf(coeff).rank(); ++a) axes.push_back(static_cast<int64_t>(a));
    ExprPtr wide = opBroadcast(tupleValue({exprValue(coeff), intTupleValue(vShape.sizes), intTupleValue(axes)}))->expr;
    result = binary("add", result, binary("mul", vertex, wide));
  }
  return result;
}

VarPtr opGatherND(const VarPtr& value) {
  const auto& args = asTuple(value, "gatherND");
  if (args.size() != 4) throw std::runtime_error("gatherND expects 4 arguments");
  return exprValue(gatherNDExpr(asTensor(args[0]), asTensor(args[1]), asInt(args[2]), asInt(args[3])));
}

// plaidml/op/lib/ops.cc:3100-3127: the sorted positions along the axis, the element's own coordinates elsewhere,
// joined into index rows for gatherND
ExprPtr sortExpr(const ExprPtr& I, int64_t rawAxis, int64_t direction) {
  if (direction != 0 && direction != 1) throw std::runtime_error("Invalid sort direction");
  const pml::TensorShape shape = shapeOf(I);
  const int64_t nd = static_cast<int64_t>(shape.rank());
  const int64_t axis = normalizeAxis(rawAxis, shape.rank(), "sort");
  std::vector<ExprPtr> parts;
  for (int64_t i = 0; i < nd; ++i) {
    if (i == axis) parts.push_back(unsqueezeExpr(intrinsic("argsort", {I, litInt(axis), litInt(direction)}), {nd}));
    else parts.push_back(unsqueezeExpr(indexExpr(shape.sizes, i), {nd}));
  }
  return gatherNDExpr(I, concatExprs(parts, -1), 0, 3);
}

VarPtr opSort(const VarPtr& value) {
  const auto& args = asTuple(value, "sort");
  if (args.size() != 3) throw std::runtime_error("sort expects 3 arguments");
  return exprValue(sortExpr(asTensor(args[0]), asInt(args[1]), asInt(args[2])));
}

// plaidml/op/lib/ops.cc:2420-2467: the first k sorted values and their positions; with sort type INDEX (1) the
// positions are put in ascending order and the values follow them
VarPtr opTopk(const VarPtr& value) {
  const auto& args = asTuple(value, "topk");
  if (args.size() != 6) throw std::runtime_error("topk expects 6 arguments");
  ExprPtr I = asTensor(args[0]);
  const int64_t k = asInt(args[1]);
  const int64_t rawAxis = asInt(args[2]);
  const int64_t direction = asInt(args[3]);
  const int64_t sortType = asInt(args[4]);
  if (direction != 0 && direction != 1) throw std::runtime_error("Invalid sort direction");
  const pml::TensorShape shape = shapeOf(I);
  const int64_t nd = static_cast<int64_t>(shape.rank());
  const int64_t axis = normalizeAxis(rawAxis, shape.rank(), "topk");
  ExprPtr values = sortExpr(I, axis, direction);
  ExprPtr positions = intrinsic("argsort", {I, litInt(axis), litInt(direction)});
  ExprPtr firstK = indexExpr({k}, 0);
  ExprPtr topPositions = gatherExpr(positions, firstK, axis);
  if (sortType == 0) return tupleValue({exprValue(gatherExpr(values, firstK, axis)), exprValue(topPositions)});
  if (sortType != 1) throw std::runtime_error("invalid topk sort type");
  ExprPtr ordered = sortExpr(topPositions, axis, 0);
  const pml::TensorShape topShape = shapeOf(topPositions);
  std::vector<ExprPtr> parts;
  for (int64_t i = 0; i < nd; ++i) {
    if (i == axis) parts.push_back(unsqueezeExpr(ordered, {nd}));
    else parts.push_back(unsqueezeExpr(indexExpr(topShape.sizes, i), {nd}));
  }
  ExprPtr topValues = gatherNDExpr(I, concatExprs(parts, -1), 0, 3);
  return tupleValue({exprValue(topValues), exprValue(ordered)});
}

// plaidml/op/lib/ops.cc:1469-1488
VarPtr opCumprod(const VarPtr& value) {
  const auto& args = asTuple(value, "cumprod");
  if (args.size() != 2) throw std::runtime_error("cumprod expects 2 arguments");
  ExprPtr I = asTensor(args[0]);
  const pml::TensorShape shape = shapeOf(I);
  const int64_t axis = normalizeAxis(asInt(args[1]), shape.rank(), "cumprod");
  std::vector<PolyPtr> oIdx, iIdx;
  for (size_t i = 0; i < shape.rank(); ++i) oIdx.push_back(newIndex());
  iIdx = oIdx;
  PolyPtr k = newIndex("k");
  iIdx[axis] = oIdx[axis] - k;
  return exprValue(contraction(pml::AggKind::mul, pml::ComboKind::none, shape.sizes, oIdx, {{I, iIdx}},
                               {{k, shape.sizes[axis]}}, "cumprod"));
}

double asFloat(const VarPtr& v) {
  if (v->kind == VarNode::Float) return v->f;
  if (v->kind == VarNode::Int) return static_cast<double>(v->i);
  throw std::runtime_error("Expected a float argument");
}

// ------------------------------------------------------------------ non-maximum suppression
//
// plaidml/op/lib/ops.cc:2034-2419 (decode_boxes, compute_iou, nms).  Boxes [batch, boxes, 4], scores
// [batch, classes, boxes]; per (batch, class) the best-scoring box is taken `max_output_boxes_per_class` times, every
// box whose overlap with it reaches the threshold loses its score (or, with a soft-NMS sigma, part of it).  Results:
// [rows, 3] (batch, class, box) and [rows, 3] (batch, class, score) with -1 rows for picks that found nothing, and the
// number of valid picks.  Built from the same operations as the reference builds it from, so the printed program and
// the arithmetic are its own: comparisons and selects, reshapes, argsort / gather / scatter / topk / gatherND.
// BoxesDecodeMode::SSD (prior boxes with variances and location offsets) is not offered.

struct Ex {
  ExprPtr e;
};
Ex operator+(const Ex& a, const Ex& b) { return {binary("add", a.e, b.e)}; }
Ex operator-(const Ex& a, const Ex& b) { return {binary("sub", a.e, b.e)}; }
Ex operator*(const Ex& a, const Ex& b) { return {binary("mul", a.e, b.e)}; }
Ex operator/(const Ex& a, const Ex& b) { return {binary("div", a.e, b.e)}; }
Ex flt(double v) { return {litFloat(v)}; }
Ex cmp(const char* fn, const Ex& a, const Ex& b) { return {binary(fn, a.e, b.e)}; }
Ex sel(const Ex& c, const Ex& a, const Ex& b) { return {intrinsic("select", {c.e, a.e, b.e})}; }
Ex maxOf(const Ex& a, const Ex& b) { return sel(cmp("cmp_lt", a, b), b, a); }
Ex minOf(const Ex& a, const Ex& b) { return sel(cmp("cmp_lt", a, b), a, b); }
Ex shaped(const Ex& a, const std::vector<int64_t>& dims) { return {reshapeTo(a.e, dims)}; }
Ex typed(const Ex& a, pml::DType dt) { return {castTo(a.e, dt)}; }
// position `i` along `axis`, keeping the axis with extent 1 (edsl::gather(x, i).axis(axis))
Ex pick(const Ex& a, int64_t i, int64_t axis) {
  ExprPtr at = binary("add", castTo(indexExpr({1}, 0), pml::DType::si32), litInt(i));
  return {gatherExpr(a.e, at, normalizeAxis(axis, shapeOf(a.e).rank(), "nms"))};
}
Ex clip01(const Ex& a) {
  return minOf(maxOf(a, typed(flt(0.0), pml::DType::f32)), typed(flt(1.0), pml::DType::f32));
}

VarPtr opNms(const VarPtr& value) {
  const auto& args = asTuple(value, "nms");
  if (args.size() != 21) throw std::runtime_error("nms expects 21 arguments");
  Ex boxes{asTensor(args[0])}, scores{asTensor(args[1])}, iouThreshold{asTensor(args[2])}, scoreThreshold{asTensor(args[3])};
  const int64_t maxPerClass = asInt(args[4]);
  const double softSigma = asFloat(args[5]);
  const bool centerPoint = asBool(args[6]), sortDescending = asBool(args[7]);
  const pml::DType boxOutType = static_cast<pml::DType>(asInt(args[8]));
  if (asInt(args[9]) != 0) throw std::runtime_error("nms: the SSD box decoding is not in the cuda target's op library");
  const bool clipBefore = asBool(args[10]);
  if (asBool(args[16])) throw std::runtime_error("nms: the SSD box decoding is not in the cuda target's op library");
  const int64_t style = asInt(args[18]);
  if (style < 0 || style > 2) throw std::runtime_error("Invalid nms style");
  const bool shareLocation = asBool(args[19]), hardSuppression = asBool(args[20]);

  const pml::DType boxType = shapeOf(boxes.e).dtype;
  pml::DType thresType = shapeOf(iouThreshold.e).dtype;
  if (pml::isAmbiguous(thresType)) thresType = pml::DType::f32;
  const pml::TensorShape scoreShape = shapeOf(scores.e);
  if (scoreShape.rank() != 3 || shapeOf(boxes.e).rank() != 3) throw std::runtime_error("nms expects boxes and scores of rank 3");
  const int64_t nb = scoreShape.sizes[0], nc = scoreShape.sizes[1], nx = scoreShape.sizes[2];
  const int64_t locClasses = shareLocation ? 1 : nc;

  const Ex zero = typed(Ex{indexExpr({1}, 0)}, boxType);
  const Ex zeroInt = typed(zero, pml::DType::si32);
  const Ex one = zero + Ex{litInt(1)};
  const Ex neg1{intrinsic("neg", {one.e})};
  const Ex neg1Out = typed(neg1, boxOutType);

  // corners (y1, x1, y2, x2) of every box: [batch, 1, boxes, 1]
  const Ex b4 = shaped(boxes, {nb, 1, shapeOf(boxes.e).sizes[1], shapeOf(boxes.e).sizes[2]});
  Ex y1, x1, y2, x2;
  if (centerPoint) {
    const Ex xc = pick(b4, 0, 3), yc = pick(b4, 1, 3), hw = pick(b4, 2, 3) / flt(2.0), hh = pick(b4, 3, 3) / flt(2.0);
    x1 = xc - hw;
    x2 = xc + hw;
    y1 = yc - hh;
    y2 = yc + hh;
  } else {
    const Ex ya = pick(b4, 0, 3), xa = pick(b4, 1, 3), yb = pick(b4, 2, 3), xb = pick(b4, 3, 3);
    y1 = minOf(ya, yb);
    x1 = minOf(xa, xb);
    y2 = maxOf(ya, yb);
    x2 = maxOf(xa, xb);
  }
  if (clipBefore) {
    y1 = clip01(y1);
    x1 = clip01(x1);
    y2 = clip01(y2);
    x2 = clip01(x2);
  }
  // overlap of every pair of boxes: [batch, location classes, boxes, boxes]
  y1 = shaped(y1, {nb, locClasses, nx});
  x1 = shaped(x1, {nb, locClasses, nx});
  y2 = shaped(y2, {nb, locClasses, nx});
  x2 = shaped(x2, {nb, locClasses, nx});
  const std::vector<int64_t> asRows{nb, locClasses, nx, 1}, asCols{nb, locClasses, 1, nx};
  const Ex area = (y2 - y1) * (x2 - x1);
  const Ex ygap = minOf(shaped(y2, asRows), shaped(y2, asCols)) - maxOf(shaped(y1, asRows), shaped(y1, asCols));
  const Ex xgap = minOf(shaped(x2, asRows), shaped(x2, asCols)) - maxOf(shaped(x1, asRows), shaped(x1, asCols));
  const Ex inter = sel(cmp("cmp_gt", ygap, flt(0.0)), ygap, zero) * sel(cmp("cmp_gt", xgap, flt(0.0)), xgap, zero);
  const Ex denom = shaped(area, asRows) + shaped(area, asCols) - inter;
  const Ex iou = inter * sel(cmp("cmp_le", denom, flt(0.0)), zero, flt(1.0) / denom);

  const double weight = softSigma != 0 ? -0.5 / softSigma : 0.0;
  pml::TensorShape nodeShape(pml::DType::f32, {1, 1, 2});
  pml::BufferPtr nodeBuffer = pml::Buffer::allocate(nodeShape);
  reinterpret_cast<float*>(nodeBuffer->data())[0] = -1.0f;
  reinterpret_cast<float*>(nodeBuffer->data())[1] = -1.0f;
  auto nodeConstant = std::make_shared<ExprNode>(ExprNode::ConstTensor);
  nodeConstant->buffer = nodeBuffer;
  nodeConstant->name = "invalid_node";
  const Ex invalidNode = typed(Ex{nodeConstant}, boxOutType);

  const int64_t perClass = maxPerClass != 0 ? std::min(nx, maxPerClass) : nx;
  const Ex indexBC = typed(Ex{concatExprs({indexExpr({nb, nc, 1}, 0), indexExpr({nb, nc, 1}, 1)}, 2)}, boxOutType);
  const Ex scoreThr = typed(scoreThreshold, boxType), iouThr = typed(iouThreshold, boxType);
  Ex live = sel(cmp("cmp_gt", scores, scoreThr), scores, zero);

  auto zeros = [&](const std::vector<int64_t>& dims) {
    std::vector<PolyPtr> idx;
    for (size_t i = 0; i < dims.size(); ++i) idx.push_back(newIndex());
    return Ex{contraction(pml::AggKind::assign, pml::ComboKind::none, dims, idx, {{zero.e, {polyLit(0)}}}, {}, "nms")};
  };
  auto topk = [&](const Ex& x, int64_t k, int64_t axis, int64_t sortType) {
    VarPtr r = opTopk(tupleValue({exprValue(x.e), intValue(k), intValue(axis), intValue(1), intValue(sortType),
                                  intValue(static_cast<int64_t>(pml::DType::si32))}));
    return std::make_pair(Ex{r->tuple[0]->expr}, Ex{r->tuple[1]->expr});
  };
  if (style == 0) {            // CAFFE: only the best `perClass` boxes of a class compete
    auto [vals, pos] = topk(live, perClass, 2, 0);
    live = Ex{intrinsic("scatter", {zeros({nb, nc, nx}).e, pos.e, vals.e, litInt(2), litInt(2)})};
  } else if (style == 1) {     // MXNET: every box keeps its best class only, then the best `perClass` boxes
    const Ex classOf = shaped(pick(Ex{intrinsic("argsort", {live.e, litInt(1), litInt(1)})}, 0, 1), {nb, nx});
    const Ex bestScore = shaped(pick(Ex{sortExpr(live.e, 1, 1)}, 0, 1), {nb, nx});
    auto [vals, boxPos] = topk(bestScore, perClass, 1, 1);
    const Ex classes{gatherNDExpr(classOf.e, unsqueezeExpr(boxPos.e, {-1}), 1, 3)};
    const pml::TensorShape cs = shapeOf(classes.e);
    const Ex where{concatExprs({unsqueezeExpr(indexExpr(cs.sizes, 0), {-1}), unsqueezeExpr(classes.e, {-1}),
                                unsqueezeExpr(boxPos.e, {-1})}, -1)};
    live = Ex{intrinsic("scatter", {zeros({nb, nc, nx}).e, where.e, vals.e, litInt(0), litInt(3)})};
  }
  const Ex zeroColumn = zeros({nb, nc, 1});

  std::vector<ExprPtr> boxParts, scoreParts;
  Ex valid = zero;
  for (int64_t k = 0; k < perClass; ++k) {
    const Ex candidate = pick(Ex{intrinsic("argsort", {live.e, litInt(2), litInt(1)})}, 0, 2);   // [batch, classes, 1]
    const VarPtr none = std::make_shared<VarNode>();
    Ex score = shaped(Ex{reduceOp(tupleValue({exprValue(live.e), intValue(2), intValue(0)}), pml::AggKind::max, "max")->expr},
                      {nb, nc, 1});
    const Ex node = sel(cmp("cmp_gt", score, flt(0.0)), indexBC, invalidNode);
    valid = valid + Ex{reduceOp(tupleValue({exprValue(sel(cmp("cmp_ne", score, flt(0.0)), one, zero).e), none, intValue(0)}),
                                pml::AggKind::add, "sum")->expr};
    scoreParts.push_back(typed(node, thresType).e);
    score = sel(cmp("cmp_gt", score, flt(0.0)), score, neg1);
    scoreParts.push_back(typed(score, thresType).e);
    // the pick leaves the competition ...
    live = shaped(Ex{intrinsic("scatter", {live.e, candidate.e, zeroColumn.e, litInt(2), litInt(2)})}, {nb, nc, nx});
    // ... and so does every box that overlaps it too much
    const Ex classIdx = shareLocation ? Ex{opBroadcast(tupleValue({exprValue(zeroInt.e), intTupleValue({nb, nc, 1}),
                                                                   intTupleValue({1})}))->expr}
                                      : Ex{indexExpr({nb, nc, 1}, 1)};
    const Ex overlap{gatherNDExpr(iou.e, concatExprs({classIdx.e, candidate.e}, 2), 1, 3)};   // [batch, classes, boxes]
    live = sel(cmp(hardSuppression ? "cmp_ge" : "cmp_gt", overlap, iouThr), zero, live);
    boxParts.push_back(node.e);
    boxParts.push_back(shaped(sel(cmp("cmp_gt", score, flt(0.0)), typed(candidate, boxOutType), neg1Out), {nb, nc, 1}).e);
    if (softSigma != 0) {
      live = live * Ex{intrinsic("exp", {(overlap * overlap * flt(weight)).e})};
      live = sel(cmp("cmp_gt", live, scoreThr), live, zero);
    }
  }
  const int64_t rows = nb * nc * perClass;
  Ex scoreRows = shaped(Ex{concatExprs(scoreParts, 2)}, {rows, 3});
  Ex boxRows = shaped(Ex{concatExprs(boxParts, 2)}, {rows, 3});
  if (sortDescending) {
    const Ex order{intrinsic("argsort", {shaped(pick(scoreRows, 2, 1), {rows}).e, litInt(0), litInt(1)})};
    scoreRows = Ex{gatherExpr(scoreRows.e, order.e, 0)};
    boxRows = Ex{gatherExpr(boxRows.e, order.e, 0)};
  } else {
    // valid entries first, in their order: every -1 entry is sent behind them
    const int64_t flat = rows * 3;
    const Ex flatScores = shaped(scoreRows, {flat}), flatBoxes = shaped(boxRows, {flat});
    const Ex key = sel(cmp("cmp_ne", flatScores, typed(Ex{litInt(-1)}, thresType)), Ex{indexExpr({flat}, 0)},
                       typed(Ex{litInt(flat)}, pml::DType::si32));
    const Ex order{intrinsic("argsort", {typed(key, pml::DType::f32).e, litInt(0), litInt(0)})};
    scoreRows = shaped(Ex{gatherExpr(flatScores.e, order.e, 0)}, {rows, 3});
    boxRows = shaped(Ex{gatherExpr(flatBoxes.e, order.e, 0)}, {rows, 3});
  }
  return tupleValue({exprValue(boxRows.e), exprValue(scoreRows.e), exprValue(typed(valid, boxOutType).e)});
}

// plaidml/op/lib/ops.cc:1586-1685: CONSTANT (0) pads with a value through the contraction's
// initial tensor, EDGE (1) repeats the border by concatenating slices; SYMMETRIC / REFLECT are
// unimplemented there too
VarPtr opExplicitPadding(const VarPtr& value) {
  const auto& args = asTuple(value, "explicit_padding");
  if (args.size() < 5) throw std::runtime_error("explicit_padding expects 5 arguments");
  ExprPtr I = asTensor(args[0]);
  const pml::TensorShape shape = shapeOf(I);
  const std::vector<int64_t> lo = asIntTuple(args[1]), hi = asIntTuple(args[2]);
  const int64_t mode = asInt(args[3]);
  const size_t nd = shape.rank();
  if (lo.size() != nd) {
    throw std::runtime_error("Inconsistent shapes in explicit_padding op (received an input tensor with " + std::to_string(nd) +
                             " dims, but received lower padding for " + std::to_string(lo.size()) + " dims.)");
  }
  if (hi.size() != nd) {
    throw std::runtime_error("Inconsistent shapes in explicit_padding op (received an input tensor with " + std::to_string(nd) +
                             " dims, but received higher padding for " + std::to_string(hi.size()) + " dims.)");
  }
  if (mode == 0) {
    std::vector<PolyPtr> iIdx, oIdx;
    std::vector<int64_t> oDims;
    for (size_t d = 0; d < nd; ++d) {
      iIdx.push_back(newIndex("x" + std::to_string(d)));
      oIdx.push_back(iIdx[d] + lo[d]);
      oDims.push_back(shape.sizes[d] + lo[d] + hi[d]);
    }
    ExprPtr O = contraction(pml::AggKind::assign, pml::ComboKind::none, oDims, oIdx, {{I, iIdx}}, {}, "explicit_padding");
    O->init = asTensor(args[4]);
    pml::Evaluator local;
    local.verify(O);
    return exprValue(O);
  }
  if (mode == 1) {
    ExprPtr O = I;
    for (size_t d = 0; d < nd; ++d) {
      const pml::TensorShape cur = shapeOf(O);
      std::vector<ExprPtr> parts;
      for (int side = 0; side < 2; ++side) {
        const int64_t width = side == 0 ? lo[d] : hi[d];
        if (side == 1) parts.push_back(O);
        if (width <= 0) continue;
        std::vector<PolyPtr> dst, src;
        std::vector<int64_t> dims = cur.sizes;
        for (size_t e = 0; e < nd; ++e) dst.push_back(newIndex());
        src = dst;
        src[d] = polyLit(side == 0 ? 0 : cur.sizes[d] - 1);
        dims[d] = width;
        parts.push_back(contraction(pml::AggKind::assign, pml::ComboKind::none, dims, dst, {{O, src}}, {}, "explicit_padding"));
      }
      O = parts.size() == 1 ? parts[0] : concatExprs(parts, static_cast<int64_t>(d));
    }
    return exprValue(O);
  }
  if (mode == 2 || mode == 3) throw std::runtime_error("Unimplemented padding mode: " + std::string(mode == 2 ? "REFLECT" : "SYMMETRIC"));
  throw std::runtime_error("Unrecognized padding mode");
}

// plaidml/op/lib/ops.cc:1803-1820
VarPtr opHardSigmoid(const VarPtr& value) {
  const auto& args = asTuple(value, "hard_sigmoid");
  if (args.size() != 2) throw std::runtime_error("hard_sigmoid expects 2 arguments");
  ExprPtr I = asTensor(args[0]);
  const double slope = asFloat(args[1]);
  if (slope <= 0) throw std::runtime_error("hard_sigmoid expects positive slope, received " + std::to_string(slope));
  const double hiCusp = 1. / (2. * slope);
  const pml::DType dt = shapeOf(I).dtype;
  ExprPtr mid = binary("add", binary("mul", litFloat(slope), I), litFloat(0.5));
  ExprPtr upper = intrinsic("select", {binary("cmp_gt", I, litFloat(hiCusp)), castTo(litFloat(1.), dt), mid});
  return exprValue(intrinsic("select", {binary("cmp_lt", I, litFloat(-hiCusp)), castTo(litFloat(0.), dt), upper}));
}

// plaidml/op/lib/ops.cc:129-160,1920-1940: I / (alpha * windowed sum of squares + epsilon) ^ beta
VarPtr opLrn(const VarPtr& value) {
  const auto& args = asTuple(value, "lrn");
  if (args.size() != 6) throw std::runtime_error("lrn expects 6 arguments");
  ExprPtr I = asTensor(args[0]);
  const pml::TensorShape shape = shapeOf(I);
  const std::vector<int64_t> widths = asIntTuple(args[1]);
  std::set<int64_t> axes;
  for (int64_t a : asIntTuple(args[2])) axes.insert(normalizeAxis(a, shape.rank(), "lrn"));
  if (axes.size() != widths.size()) {
    throw std::runtime_error("Inconsistent axis count and window width count in LRN (" + std::to_string(axes.size()) + " vs " +
                             std::to_string(widths.size()) + ")");
  }
  const double alpha = asFloat(args[3]), beta = asFloat(args[4]), eps = asFloat(args[5]);
  std::vector<PolyPtr> dst, src;
  for (size_t d = 0; d < shape.rank(); ++d) dst.push_back(newIndex());
  src = dst;
  std::vector<Cons> cons;
  size_t w = 0;
  for (int64_t a : axes) {
    PolyPtr win = newIndex();
    cons.push_back({win, widths[w]});
    src[a] = dst[a] + win - (widths[w] / 2);
    ++w;
  }
  ExprPtr sq = binary("mul", I, I);
  ExprPtr sum = contraction(pml::AggKind::add, pml::ComboKind::none, shape.sizes, dst, {{sq, src}}, cons, "lrn");
  ExprPtr denom = binary("pow", binary("add", binary("mul", litFloat(alpha), sum), litFloat(eps)), litFloat(beta));
  return exprValue(binary("div", I, denom));
}

// plaidml/op/lib/ops.cc:2469-2503
VarPtr opMvn(const VarPtr& value) {
  const auto& args = asTuple(value, "mvn");
  if (args.size() != 6) throw std::runtime_error("mvn expects 6 arguments");
  ExprPtr I = asTensor(args[0]);
  VarPtr axes = args[1];
  const bool normVar = asBool(args[2]);
  const double eps = asFloat(args[3]);
  const bool acrossChannels = asBool(args[4]);
  const std::string layout = asStr(args[5]);
  if (axes->kind == VarNode::None) {
    if (layout.empty()) throw std::runtime_error("Either axes or layout must be specified for MVN");
    std::vector<int64_t> raw;
    for (size_t i = 0; i < layout.size(); ++i) {
      if (layout[i] == 'N') continue;
      if (layout[i] == 'C' && !acrossChannels) continue;
      raw.push_back(static_cast<int64_t>(i));
    }
    axes = intTupleVar(raw);
  }
  ExprPtr R = binary("sub", I, opMean(tupleVar({args[0], axes, intVar(1)}))->expr);
  if (normVar) {
    ExprPtr stdev = intrinsic("sqrt", {opVariance(tupleVar({args[0], axes, intVar(1)}))->expr});
    ExprPtr floor = castTo(litFloat(eps), shapeOf(I).dtype);
    R = binary("div", R, intrinsic("select", {binary("cmp_lt", stdev, floor), floor, stdev}));
  }
  return exprValue(R);
}

// plaidml/op/lib/ops.cc:2505-2530: sqrt(sum(I^2, axes, keepdims) (+ | max) epsilon); eps_mode 0 = ADD, 1 = MAX
VarPtr opL2norm(const VarPtr& value) {
  const auto& args = asTuple(value, "l2norm");
  if (args.size() != 4) throw std::runtime_error("norm expects 4 arguments");
  ExprPtr I = asTensor(args[0]);
  const double eps = asFloat(args[2]);
  const int64_t mode = asInt(args[3]);
  ExprPtr X = reduceOp(tupleVar({exprValue(binary("mul", I, I)), intTupleVar(asIntTuple(args[1])), intVar(1)}),
                       pml::AggKind::add, "sum")->expr;
  if (mode == 0) {
    X = binary("add", X, litFloat(eps));
  } else if (mode == 1) {
    ExprPtr e = castTo(litFloat(eps), shapeOf(X).dtype);
    X = intrinsic("select", {binary("cmp_lt", X, e), e, X});
  } else {
    throw std::runtime_error("Unrecognized eps_mode in l2norm op");
  }
  return exprValue(intrinsic("sqrt", {X}));
}

// plaidml/op/lib/ops.cc:2782-2816: numpy-style repeat of every element along one axis
VarPtr opRepeat(const VarPtr& value) {
  const auto& args = asTuple(value, "repeat");
  if (args.size() != 3) throw std::runtime_error("PlaidML repeat op expects 3 arguments (received " + std::to_string(args.size()) + ")");
  ExprPtr I = asTensor(args[0]);
  if (args[1]->kind != VarNode::Int && args[1]->kind != VarNode::Dim) {
    throw std::runtime_error("Repeat only accepts int or TensorDim for repeats parameter");
  }
  const int64_t reps = asInt(args[1]);
  const pml::TensorShape shape = shapeOf(I);
  const size_t axis = static_cast<size_t>(normalizeAxis(asInt(args[2]), shape.rank(), "repeat"));
  std::vector<PolyPtr> iIdx, oIdx;
  for (size_t d = 0; d < shape.rank(); ++d) iIdx.push_back(newIndex());
  oIdx = iIdx;
  PolyPtr inner = newIndex();
  oIdx[axis] = reps * iIdx[axis] + inner;
  std::vector<int64_t> dims = shape.sizes;
  dims[axis] *= reps;
  return exprValue(contraction(pml::AggKind::assign, pml::ComboKind::none, dims, oIdx, {{I, iIdx}}, {{inner, reps}}, "repeat"));
}

// plaidml/op/lib/ops.cc:3454-3487: numpy-style tile
// Resize the two spatial dimensions of an image tensor by positive integer factors: nearest (two repeats) or
// bilinear with corners aligned to 0 and factor * (dim - 1) over zero padding, as a contraction with a
// (2 fh - 1) x (2 fw - 1) triangular kernel built by contractions (plaidml/op/lib/ops.cc:1822-1917).
VarPtr opImageResize(const VarPtr& value) {
  const auto& args = asTuple(value, "image_resize");
  if (args.size() != 4) throw std::runtime_error("image_resize expects 4 arguments");
  ExprPtr I = asTensor(args[0]);
  const std::vector<int64_t> factors = asIntTuple(args[1]);
  const int64_t interp = asInt(args[2]);
  const int64_t layout = asInt(args[3]);
  if (interp < 0 || interp > 1) throw std::runtime_error("Invalid enumeration value: " + std::to_string(interp));
  for (int64_t f : factors) {
    if (f <= 0) {
      throw std::runtime_error("All scaling factors in image_resize must be positive (received " + std::to_string(f) + ")");
    }
  }
  const pml::TensorShape shape = shapeOf(I);
  const size_t nd = shape.rank();
  size_t pre;
  if (layout == 1) pre = 2;        // NCX
  else if (layout == 0) pre = 1;   // NXC
  else throw std::runtime_error("Unable to apply image_resize to a tensor with layout '" + std::to_string(layout) + "'");
  if (nd < 2 || nd - 2 != 2) {
    throw std::runtime_error("Expected 2 spatial dims for resize_images, received " + std::to_string(static_cast<int64_t>(nd) - 2));
  }
  if (factors.size() != 2) {
    throw std::runtime_error("Cannot resize a 2D image using " + std::to_string(factors.size()) + " spatial scaling factors");
  }
  if (interp == 0) {
    VarPtr rows = opRepeat(tupleVar({args[0], intVar(factors[0]), intVar(static_cast<int64_t>(pre))}));
    return opRepeat(tupleVar({rows, intVar(factors[1]), intVar(static_cast<int64_t>(pre) + 1)}));
  }
  // one axis of the kernel: ramp[y] = sum over j < f of (1/f)[j + y - f + 1], a triangle of height 1 at y = f - 1
  auto ramp = [](int64_t f) {
    ExprPtr coeff = castTo(litFloat(1.0 / static_cast<double>(f)), pml::DType::f32);
    PolyPtr y = newIndex("y");
    ExprPtr vec = contraction(pml::AggKind::assign, pml::ComboKind::none, {f}, {y}, {{coeff, {}}}, {}, "image_resize");
    PolyPtr j = newIndex("j"), y2 = newIndex("y");
    return contraction(pml::AggKind::add, pml::ComboKind::none, {2 * f - 1}, {y2}, {{vec, {j + y2 - f + 1}}}, {{j, f}},
                       "image_resize");
  };
  const int64_t fh = factors[0], fw = factors[1];
  ExprPtr hk = ramp(fh), wk = ramp(fw);
  PolyPtr ky = newIndex("y"), kx = newIndex("x");
  ExprPtr kernel = contraction(pml::AggKind::assign, pml::ComboKind::mul, {2 * fh - 1, 2 * fw - 1}, {ky, kx},
                               {{hk, {ky}}, {wk, {kx}}}, {}, "image_resize");
  std::vector<PolyPtr> iIdx, oIdx;
  for (size_t d = 0; d < nd; ++d) iIdx.push_back(newIndex());
  oIdx = iIdx;
  PolyPtr j = newIndex("j"), i = newIndex("i");
  std::vector<int64_t> oDims = shape.sizes;
  oDims[pre] *= fh;
  oDims[pre + 1] *= fw;
  oIdx[pre] = fh * iIdx[pre] + j - fh + 1;
  oIdx[pre + 1] = fw * iIdx[pre + 1] + i - fw + 1;
  return exprValue(contraction(pml::AggKind::add, pml::ComboKind::mul, oDims, oIdx, {{I, iIdx}, {kernel, {j, i}}}, {},
                               "image_resize"));
}

VarPtr opTile(const VarPtr& value) {
  const auto& args = asTuple(value, "tile");
  if (args.size() != 2) throw std::runtime_error("Tile expects 2 arguments");
  ExprPtr I = asTensor(args[0]);
  std::vector<int64_t> reps = asIntTuple(args[1]);
  const pml::TensorShape shape = shapeOf(I);
  if (reps.empty()) throw std::runtime_error("No tiling factors provided to tile operation");
  while (reps.size() < shape.rank()) reps.push_back(1);
  if (reps.size() > shape.rank()) throw std::runtime_error("More tiling factors provided to tile operation than tensor dimensions");
  std::vector<PolyPtr> iIdx, oIdx;
  std::vector<int64_t> dims;
  for (size_t d = 0; d < shape.rank(); ++d) {
    iIdx.push_back(newIndex());
    oIdx.push_back(shape.sizes[d] * newIndex() + iIdx[d]);
    dims.push_back(shape.sizes[d] * reps[d]);
  }
  return exprValue(contraction(pml::AggKind::assign, pml::ComboKind::none, dims, oIdx, {{I, iIdx}}, {}, "tile"));
}

// plaidml/op/lib/ops.cc:2888-2903: the forward pass is the identity
VarPtr opScaleGradient(const VarPtr& value) {
  const auto& args = asTuple(value, "scale_gradient");
  if (args.size() != 2) throw std::runtime_error("scale_gradient expects 2 arguments");
  return exprValue(asTensor(args[0]));
}

// plaidml/op/lib/ops.cc:2917-3042: per axis an integer (the axis disappears) or (start, stop, step)
// with None defaults and negative values counted from the end
VarPtr opSlice(const VarPtr& value) {
  const auto& args = asTuple(value, "slice");
  if (args.size() != 2) throw std::runtime_error("slice expects 2 arguments");
  ExprPtr I = asTensor(args[0]);
  const pml::TensorShape shape = shapeOf(I);
  const size_t nd = shape.rank();
  if (nd == 0) return exprValue(I);
  const auto& slices = asTuple(args[1], "slices");
  if (slices.size() != nd) {
    throw std::runtime_error(std::to_string(slices.size()) + " slice axes provided to slice " + std::to_string(nd) + "-dimensional tensor");
  }
  std::vector<PolyPtr> oIdx, iIdx;
  std::vector<int64_t> oDims;
  for (size_t d = 0; d < nd; ++d) {
    const VarPtr& sl = slices[d];
    const int64_t size = shape.sizes[d];
    if (sl->kind == VarNode::Int) {
      iIdx.push_back(polyLit(sl->i < 0 ? sl->i + size : sl->i));
      continue;
    }
    if (sl->kind != VarNode::Tuple) throw std::runtime_error("Attempted to define slice with invalid type");
    if (sl->tuple.size() != 3) {
      throw std::runtime_error("Attempted to slice with " + std::to_string(sl->tuple.size()) + " entries, 3 required");
    }
    const int64_t step = sl->tuple[2]->kind == VarNode::None ? 1 : asInt(sl->tuple[2]);
    if (step == 0) throw std::runtime_error("Cannot slice with step size 0");
    int64_t start, stop;
    if (sl->tuple[0]->kind == VarNode::None) {
      start = step > 0 ? 0 : size - 1;
    } else {
      start = asInt(sl->tuple[0]);
      if (start < 0) start += size;
    }
    if (sl->tuple[1]->kind == VarNode::None) {
      stop = step > 0 ? size : -1;
    } else {
      stop = asInt(sl->tuple[1]);
      if (stop < 0) stop += size;
    }
    const int64_t toCeil = step > 0 ? step - 1 : step + 1;
    const int64_t count = (stop - start + toCeil) / step;    // truncating division, as the dimension arithmetic does
    PolyPtr o = newIndex();
    oIdx.push_back(o);
    oDims.push_back(count);
    iIdx.push_back(step * o + start);
  }
  return exprValue(contraction(pml::AggKind::assign, pml::ComboKind::none, oDims, oIdx, {{I, iIdx}}, {}, "slice"));
}

// plaidml/op/lib/ops.cc:2730-2780: YOLO's space-to-depth shuffle (and its inverse) on a 4-d tensor given in
// `layout` (a permutation of NCHW)
VarPtr opReorgYolo(const VarPtr& value) {
  const auto& args = asTuple(value, "reorg_yolo");
  if (args.size() != 4) throw std::runtime_error("PlaidML reorg_yolo op expects 4 arguments (received " + std::to_string(args.size()) + ")");
  ExprPtr I = asTensor(args[0]);
  const int64_t stride = asInt(args[1]);
  const bool decrease = asBool(args[2]);
  const std::string layout = asStr(args[3]);
  const pml::TensorShape shape = shapeOf(I);
  if (shape.rank() != 4) throw std::runtime_error("PlaidML reorg_yolo op expects I to have 4 dimensions (received " + std::to_string(shape.rank()) + ")");
  if (layout.size() != 4) throw std::runtime_error("source and target rank mismatch");
  // position of each of N, C, H, W in the given layout
  size_t pos[4];
  const std::string canon = "NCHW";
  for (size_t i = 0; i < 4; ++i) {
    const size_t at = layout.find(canon[i]);
    if (at == std::string::npos) throw std::runtime_error("source and target dims mismatch");
    pos[i] = at;
  }
  const int64_t N = shape.sizes[pos[0]], C = shape.sizes[pos[1]], H = shape.sizes[pos[2]], W = shape.sizes[pos[3]];
  if (stride <= 0) throw std::runtime_error("reorg_yolo expects a positive stride");
  PolyPtr b = newIndex("b"), i = newIndex("i"), j = newIndex("j"), k = newIndex("k"), x = newIndex("x"), y = newIndex("y");
  PolyPtr h = stride * j + y, w = stride * i + x;
  auto place = [&](PolyPtr n_, PolyPtr c_, PolyPtr h_, PolyPtr w_) {
    std::vector<PolyPtr> v(4);
    v[pos[0]] = n_; v[pos[1]] = c_; v[pos[2]] = h_; v[pos[3]] = w_;
    return v;
  };
  auto placeDims = [&](int64_t n_, int64_t c_, int64_t h_, int64_t w_) {
    std::vector<int64_t> v(4);
    v[pos[0]] = n_; v[pos[1]] = c_; v[pos[2]] = h_; v[pos[3]] = w_;
    return v;
  };
  const std::vector<Cons> cons = {{y, stride}, {x, stride}};
  if (decrease) {
    const int64_t cOut = C / (stride * stride);
    PolyPtr c = k + cOut * (x + stride * y);
    return exprValue(contraction(pml::AggKind::assign, pml::ComboKind::none, placeDims(N, cOut, H * stride, W * stride),
                                 place(b, k, h, w), {{I, place(b, c, j, i)}}, cons, "reorg_yolo"));
  }
  const int64_t cOut = C * stride * stride;
  PolyPtr c = k + C * (x + stride * y);
  return exprValue(contraction(pml::AggKind::assign, pml::ComboKind::none, placeDims(N, cOut, H / stride, W / stride),
                               place(b, c, j, i), {{I, place(b, k, h, w)}}, cons, "reorg_yolo"));
}

const std::map<std::string, std::function<VarPtr(const VarPtr&)>>& registry() {
  static const std::map<std::string, std::function<VarPtr(const VarPtr&)>> ops = {
      {"abs", [](const VarPtr& v) { return unary(v, "abs"); }},
      {"all", [](const VarPtr& v) { return opAllAny(v, true); }},
      {"any", [](const VarPtr& v) { return opAllAny(v, false); }},
      {"argmax", opArgmax},
      {"binary_crossentropy", opBinaryCrossentropy},
      {"broadcast", opBroadcast},
      {"concatenate", opConcatenate},
      {"cumprod", opCumprod},
      {"explicit_padding", opExplicitPadding},
      {"hard_sigmoid", opHardSigmoid},
      {"image_resize", opImageResize},
      {"l2norm", opL2norm},
      {"lrn", opLrn},
      {"mvn", opMvn},
      {"reorg_yolo", opReorgYolo},
      {"repeat", opRepeat},
      {"scale_gradient", opScaleGradient},
      {"slice", opSlice},
      {"tile", opTile},
      {"clip", opClip},
      {"convolution", opConvolution},
      {"cumsum", opCumsum},
      {"dot", opDot},
      {"elu", opElu},
      {"flip", opFlip},
      {"max", [](const VarPtr& v) { return reduceOp(v, pml::AggKind::max, "max"); }},
      {"maximum", opMaximum},
      {"gatherND", opGatherND},
      {"nms", opNms},
      {"sort", opSort},
      {"topk", opTopk},
      {"mean", opMean},
      {"min", [](const VarPtr& v) { return reduceOp(v, pml::AggKind::min, "min"); }},
      {"minimum", opMinimum},
      {"pool", opPool},
      {"prod", [](const VarPtr& v) { return reduceOp(v, pml::AggKind::mul, "prod"); }},
      {"relu", opRelu},
      {"reshape", opReshape},
      {"sigmoid", [](const VarPtr& v) { return unary(v, "sigmoid"); }},
      {"softmax", opSoftmax},
      {"spatial_padding", opSpatialPadding},
      {"square", opSquare},
      {"squeeze", opSqueeze},
      {"sum", [](const VarPtr& v) { return reduceOp(v, pml::AggKind::add, "sum"); }},
      {"transpose", opTranspose},
      {"unsqueeze", opUnsqueeze},
      {"variance", opVariance},
  };
  return ops;
}

}  // namespace

extern "C" {

plaidml_value* plaidml_op_make(plaidml_error* err, const char* op_name, plaidml_value* value) {
  return pml::ffiWrap<plaidml_value*>(err, nullptr, [&] {
    const auto& ops = registry();
    auto it = ops.find(op_name ? op_name : "");
    if (it == ops.end()) {
      throw std::runtime_error(std::string("Operation '") + (op_name ? op_name : "") +
                               "' is not in the cuda target's op library");
    }
    return new plaidml_value{it->second(value->node)};
  });
}

}  // extern "C"
