// Planner and executor of the `cuda` device.
#include "pml_exec.h"

#include "pml_shard.h"

#include "../kernels/conv_route.h"

#include <algorithm>
#include <chrono>
#include <cstring>
#include <map>
#include <regex>
#include <set>
#include <sstream>

extern "C" pmlb_status pmlb_plan_share_status(pmlb_plan* plan, int* device_word);

namespace pml {

namespace {

void cudaCheck(cudaError_t e, const char* what) {
  if (e != cudaSuccess) throw std::runtime_error(std::string(what) + ": " + cudaGetErrorString(e));
}

void pmlbCheck(pmlb_status s, const std::string& what) {
  if (s != PMLB_OK) throw std::runtime_error(what + ": " + pmlb_last_error());
}

int pmlbAgg(AggKind a) {
  switch (a) {
    case AggKind::add: return PMLB_AGG_SUM;
    case AggKind::max: return PMLB_AGG_MAX;
    case AggKind::min: return PMLB_AGG_MIN;
    case AggKind::mul: return PMLB_AGG_PROD;
    default: return PMLB_AGG_ASSIGN;
  }
}

int pmlbCombo(ComboKind c) {
  switch (c) {
    case ComboKind::mul: return PMLB_COMBO_MUL;
    case ComboKind::add: return PMLB_COMBO_ADD;
    case ComboKind::eq: return PMLB_COMBO_EQ;
    case ComboKind::cond: return PMLB_COMBO_COND;
    default: return PMLB_COMBO_NONE;
  }
}

std::string shapeStr(const std::vector<int64_t>& v) {
  std::ostringstream os;
  for (size_t i = 0; i < v.size(); ++i) os << (i ? "x" : "") << v[i];
  return os.str();
}

// One index variable's use inside one tensor access.
struct VarUse {
  bool present = false;
  int64_t stride = 0;  // elements, in the dense layout of the tensor
};

// A contraction with extent-1 variables folded away and integer coefficients checked.
struct Simplified {
  bool ok = false;
  size_t n = 0;
  std::vector<int64_t> extent;
  // per tensor (0 = out, 1.. = sources), per dim: integer coefficients and constant
  std::vector<std::vector<std::vector<int64_t>>> coef;
  std::vector<std::vector<int64_t>> cst;
};

Simplified simplify(const BoundedContraction& c) {
  Simplified s;
  s.n = c.nIdx();
  s.extent = c.extent;
  auto addTensor = [&](const std::vector<Affine>& forms) -> bool {
    std::vector<std::vector<int64_t>> cf;
    std::vector<int64_t> cs;
    for (const Affine& a : forms) {
      std::vector<int64_t> row(s.n, 0);
      Rational k = a.constant;
      for (size_t i = 0; i < s.n; ++i) {
        const Rational ci = i < a.coef.size() ? a.coef[i] : Rational(0);
        k = k + ci * Rational(c.lower[i]);           // shift variables to start at 0
        if (c.extent[i] <= 1 || ci.isZero()) continue;  // a single-valued variable is a constant
        if (!ci.isInt()) return false;
        row[i] = ci.num;
      }
      if (!k.isInt()) return false;
      cf.push_back(row);
      cs.push_back(k.num);
    }
    s.coef.push_back(cf);
    s.cst.push_back(cs);
    return true;
  };
  if (!addTensor(c.sink)) return s;
  for (const auto& src : c.srcs) {
    if (!addTensor(src)) return s;
  }
  // constraints must be implied by the ranges: single variable, unit coefficient
  for (const auto& con : c.cons) {
    int var = -1;
    Rational k = con.first.constant;
    for (size_t i = 0; i < s.n; ++i) {
      const Rational ci = i < con.first.coef.size() ? con.first.coef[i] : Rational(0);
      k = k + ci * Rational(c.lower[i]);
      if (ci.isZero() || c.extent[i] <= 1) continue;
      if (var >= 0 || !(ci.num == 1 && ci.den == 1)) return s;
      var = static_cast<int>(i);
    }
    if (!k.isInt() || k.num < 0) return s;
    const int64_t ext = var >= 0 ? c.extent[var] : 1;
    if (k.num + ext > con.second) return s;
  }
  for (size_t i = 0; i < s.n; ++i) {
    if (c.extent[i] <= 0) return s;
  }
  s.ok = true;
  return s;
}

// Is dim `d` of tensor `t` exactly one variable (coefficient 1, constant 0)?  Returns the
// variable or -1; -2 when the dim is a constant 0 (all its variables single-valued).
int pureVar(const Simplified& s, size_t t, size_t d) {
  int var = -1;
  for (size_t i = 0; i < s.n; ++i) {
    if (s.coef[t][d][i] == 0) continue;
    if (var >= 0 || s.coef[t][d][i] != 1) return -1;
    var = static_cast<int>(i);
  }
  if (s.cst[t][d] != 0) return -1;
  return var >= 0 ? var : -2;
}

}  // namespace

// ==================================================================== planner

class Planner {
 public:
  Planner(Executable* exe) : exe_(exe), prog_(*exe->prog_) {}

  void run() {
    const size_t nv = prog_.values.size();
    uses_.assign(nv, 0);
    isOutput_.assign(nv, false);
    for (const POp& op : prog_.ops) {
      for (int o : op.operands) ++uses_[o];
    }
    for (int o : prog_.outputs) {
      ++uses_[o];
      isOutput_[o] = true;
    }
    users_.assign(nv, {});
    for (size_t i = 0; i < prog_.ops.size(); ++i) {
      for (int o : prog_.ops[i].operands) users_[o].push_back(static_cast<int>(i));
    }
    absorbed_.assign(prog_.ops.size(), false);
    alias_.assign(nv, -1);

    // ---- phase A: choose a kernel for every operation, fusing neighbours into it
    for (size_t i = 0; i < prog_.ops.size(); ++i) {
      if (absorbed_[i]) continue;
      const POp& op = prog_.ops[i];
      // an operation whose value the builder already computed from shapes alone (tile.shape): nothing to run
      if (prog_.values[op.result].kind == PValue::InternalConstant) continue;
      Pending pd;
      pd.op = static_cast<int>(i);
      pd.position = static_cast<int>(i);
      pd.result = op.result;
      switch (op.kind) {
        case POp::Reshape:
          alias_[op.result] = op.operands[0];
          continue;
        case POp::Contraction:
          planContraction(&pd);
          break;
        case POp::Cast:
        case POp::Eltwise:
          pd.kind = Pending::Eltwise;
          pd.inputs = op.operands;
          break;
        case POp::Special:
          pd.kind = Pending::Special;
          pd.inputs = op.operands;
          break;
      }
      pending_.push_back(std::move(pd));
    }

    // A step with fused consumers runs where its last consumer stood, so that operands
    // joined late (a residual computed by a sibling branch) are ready.
    std::stable_sort(pending_.begin(), pending_.end(),
                     [](const Pending& x, const Pending& y) { return x.position < y.position; });

    fuseRowMaxima();
    fuseConvMaxPool();
    fuseShortcutProjections();

    // ---- phase B: which steps are needed for the outputs
    std::vector<bool> needed(nv, false);
    for (int o : prog_.outputs) needed[root(o)] = true;
    std::vector<bool> keep(pending_.size(), false);
    for (size_t k = pending_.size(); k-- > 0;) {
      Pending& pd = pending_[k];
      if (pd.dropped) continue;
      const bool mainNeeded = needed[root(pd.result)];
      const bool sideNeeded = pd.rowmax >= 0 && needed[root(pd.rowmax)];
      if (!mainNeeded && !sideNeeded) continue;
      if (pd.rowmax >= 0) {
        pd.storeMain = mainNeeded;
        if (!sideNeeded) {
          pd.rowmax = -1;
          pd.gemm.epilogue &= ~PMLB_EPI_ROWMAX;
        }
      }
      keep[k] = true;
      for (int in : pd.inputs) needed[root(in)] = true;
    }

    // an input that no kept step reads and that is not returned stays on the host (a network builder may list its
    // weights as inputs although the operations use constants: networks/oplib/resnet50.cc does)
    exe_->inputUsed_.assign(prog_.inputs.size(), true);
    for (size_t i = 0; i < prog_.inputs.size(); ++i) exe_->inputUsed_[i] = needed[root(prog_.inputs[i])];

    // ---- phase C: device memory, then kernel plans
    allocate(needed);
    for (size_t k = 0; k < pending_.size(); ++k) {
      if (!keep[k]) continue;
      const size_t before = exe_->steps_.size();
      emit(pending_[k]);
      for (size_t s = before; s < exe_->steps_.size(); ++s) exe_->steps_[s].position = pending_[k].position;
    }
  }

 private:
  struct Pending {
    enum Kind { Gemm, Conv, Reduce, Pool, Generic, Eltwise, Special } kind = Generic;
    int op = -1;
    int position = -1;          // program position the step runs at: its last fused operation
    int result = -1;            // value the step writes (after fused consumers)
    std::vector<int> inputs;    // values the step reads
    std::string fused;          // description of fused neighbours
    pmlb_gemm_desc gemm;
    pmlb_conv_desc conv;
    pmlb_reduce_desc reduce;
    pmlb_pool_desc pool;
    int a = -1, b = -1, bias = -1, residual = -1;  // value ids
    bool swapped = false;
    int a2 = -1;                // GEMM with A in two parts (a fused shortcut projection): the second part's value
    const void* bDerived = nullptr;     // ... its stacked weights and summed bias on the device (planner-owned)
    const void* biasDerived = nullptr;
    int rowmax = -1;            // GEMM: value that receives the row maxima of the product (fused max-reduction)
    bool storeMain = true;      // GEMM with fused row maxima: false if nothing else reads the product
    bool dropped = false;       // folded into another step
  };

  int root(int v) const {
    while (alias_[v] >= 0) v = alias_[v];
    return v;
  }

  // R[b, i] = max_j S[b, i, j] right after the GEMM that produces S: the GEMM's epilogue folds
  // each accumulator row into R (one atomic max per row and tile) and the separate pass over S
  // goes away; S itself is still written if anything else reads it.  (The Q.K^T-then-row-max
  // pattern of attention scores.)
  void fuseRowMaxima() {
    for (size_t r = 0; r < pending_.size(); ++r) {
      Pending& red = pending_[r];
      if (red.dropped || red.kind != Pending::Reduce) continue;
      const pmlb_reduce_desc& rd = red.reduce;
      if (rd.agg != PMLB_AGG_MAX || rd.dtype != PMLB_F32 || rd.out_dtype != PMLB_F32 || rd.inner != 1) continue;
      for (size_t g = 0; g < r; ++g) {
        Pending& gm = pending_[g];
        if (gm.dropped || gm.kind != Pending::Gemm || gm.rowmax >= 0) continue;
        if (root(gm.result) != root(red.a)) continue;
        const pmlb_gemm_desc& gd = gm.gemm;
        if (gd.out_dtype != PMLB_F32 || rd.reduce != gd.n || rd.outer != static_cast<int64_t>(gd.batch) * gd.m) continue;
        if (gd.ldc != gd.n || (gd.batch > 1 && gd.stride_c != static_cast<int64_t>(gd.m) * gd.n)) continue;
        // The kernel folds row maxima only into a product with no other epilogue term (a bias, residual or
        // ReLU already fused into this GEMM keeps the reduction a separate step), and the fusion is kept only
        // if the library accepts the combined descriptor: a refusal after this point could not be undone,
        // since the reduction step is gone and the product may not even be stored.
        if (gd.epilogue != 0) continue;
        {
          pmlb_gemm_desc trial = gd;
          trial.epilogue |= PMLB_EPI_ROWMAX;
          pmlb_plan* probe = nullptr;
          const pmlb_status rc = pmlb_gemm_dispatch(&trial, &probe);
          if (probe) pmlb_plan_free(probe);
          if (rc != PMLB_OK) continue;
        }
        gm.gemm.epilogue |= PMLB_EPI_ROWMAX;
        gm.rowmax = red.result;
        gm.fused += "+rowmax";
        red.dropped = true;
        break;
      }
    }
  }

  // relu(A2 * W2 + b2 + (A1 * W1 + b1)): the last 1x1 convolution of a residual block whose residual is the block's
  // shortcut projection, both GEMMs over the same rows.  One GEMM over [A2 | A1] and the stacked weights computes
  // the sum in one accumulator; the projection's output (four times its input at ResNet's first stage) is neither
  // written nor read back, and its launch goes away.  Needs both weights as constants stored [k][n] and both biases
  // constant; kept only if the library accepts the descriptor.  (The sum is rounded once instead of the
  // projection being rounded to 16 bits first: the fused form is the more accurate one.)
  void fuseShortcutProjections() {
    if (getenvFlag("PLAIDML_CUDA_NO_SHORTCUT_FUSION")) return;
    auto hostConstant = [&](int v) -> const Buffer* {
      if (v < 0) return nullptr;
      const PValue& pv = val(root(v));
      if (pv.kind != PValue::Constant && pv.kind != PValue::InternalConstant) return nullptr;
      return pv.constant.get();
    };
    for (size_t m2 = 0; m2 < pending_.size(); ++m2) {
      Pending& main = pending_[m2];
      if (main.dropped || main.kind != Pending::Gemm || main.residual < 0 || main.a2 >= 0 || main.rowmax >= 0) continue;
      const int mid = root(main.residual);
      for (size_t m1 = 0; m1 < m2; ++m1) {
        Pending& proj = pending_[m1];
        if (proj.dropped || root(proj.result) != mid) continue;
        if (proj.kind != Pending::Gemm && proj.kind != Pending::Conv) break;
        const pmlb_gemm_desc& g2 = main.gemm;
        if (proj.residual >= 0 || proj.rowmax >= 0 || proj.a2 >= 0) break;
        // the projection as "rows x k1 times k1 x n": a GEMM over the same rows, or a 1x1 convolution (possibly
        // strided: a block that halves the resolution) whose output pixels are those rows
        int k1 = 0, a2Stride = 0, a2n = 0, a2h = 0, a2w = 0;
        int64_t lda2 = 0;
        if (proj.kind == Pending::Gemm) {
          const pmlb_gemm_desc& g1 = proj.gemm;
          if ((g1.epilogue & ~PMLB_EPI_BIAS) != 0 || g1.batch != 1 || g1.m != g2.m || g1.n != g2.n ||
              g1.in_dtype != g2.in_dtype || g1.b_is_nk || g1.ldb != g1.n || g1.lda != g1.k) {
            break;
          }
          k1 = g1.k;
          lda2 = g1.lda;
        } else {
          const pmlb_conv_desc& c1 = proj.conv;
          if ((c1.epilogue & ~PMLB_EPI_BIAS) != 0 || c1.r != 1 || c1.s != 1 || c1.pad_h != 0 || c1.pad_w != 0 ||
              c1.stride_h != c1.stride_w || c1.dil_h != 1 || c1.dil_w != 1 || c1.k != g2.n || c1.in_dtype != g2.in_dtype ||
              static_cast<int64_t>(c1.n) * c1.p * c1.q != g2.m || c1.p != (c1.h + c1.stride_h - 1) / c1.stride_h ||
              c1.q != (c1.w + c1.stride_w - 1) / c1.stride_w) {
            break;
          }
          k1 = c1.c;
          a2Stride = c1.stride_h;
          a2n = c1.n, a2h = c1.h, a2w = c1.w;
        }
        if (g2.batch != 1 || g2.in_dtype == PMLB_F32 || g2.b_is_nk || g2.ldb != g2.n || g2.lda != g2.k || g2.ldr != g2.n) break;
        // the projection's output feeds this residual and nothing else
        if (isOutput_[mid] || uses_[mid] != 1) break;
        {
          const POp& u = prog_.ops[users_[mid][0]];
          if (u.kind == POp::Cast) {
            if (isOutput_[u.result] || uses_[u.result] != 1 || !absorbed_[users_[u.result][0]]) break;
          } else if (!absorbed_[users_[mid][0]]) {
            break;
          }
        }
        const Buffer* w1 = hostConstant(proj.b);
        const Buffer* w2 = hostConstant(main.b);
        const Buffer* b1 = hostConstant(proj.bias);
        const Buffer* b2 = hostConstant(main.bias);
        if (!w1 || !w2 || (proj.bias >= 0 && !b1) || (main.bias >= 0 && !b2)) break;
        const size_t eb = g2.in_dtype == PMLB_I8 ? 1 : 2;
        const bool intPath = g2.in_dtype == PMLB_I8;
        if (w1->size() != static_cast<size_t>(k1) * g2.n * eb || w2->size() != static_cast<size_t>(g2.k) * g2.n * eb) break;
        pmlb_gemm_desc trial = g2;
        trial.k = g2.k + k1;
        trial.k_first = g2.k;
        trial.lda2 = lda2;
        trial.a2_stride = a2Stride;
        trial.a2_n = a2n, trial.a2_h = a2h, trial.a2_w = a2w;
        trial.epilogue = (g2.epilogue & ~PMLB_EPI_RESIDUAL) | ((b1 || b2) ? PMLB_EPI_BIAS : 0);
        pmlb_plan* probe = nullptr;
        const pmlb_status rc = pmlb_gemm_dispatch(&trial, &probe);
        if (probe) pmlb_plan_free(probe);
        if (rc != PMLB_OK) break;
        // stacked weights [W2 ; W1] and the summed bias, on the device
        void* wDev = nullptr;
        cudaCheck(cudaMalloc(&wDev, w1->size() + w2->size()), "cudaMalloc(stacked weights)");
        exe_->derived_.push_back(wDev);
        cudaCheck(cudaMemcpy(wDev, w2->data(), w2->size(), cudaMemcpyHostToDevice), "upload of stacked weights");
        cudaCheck(cudaMemcpy(static_cast<char*>(wDev) + w2->size(), w1->data(), w1->size(), cudaMemcpyHostToDevice),
                  "upload of stacked weights");
        void* bDev = nullptr;
        if (b1 || b2) {
          std::vector<char> sum(static_cast<size_t>(g2.n) * 4, 0);
          for (const Buffer* b : {b2, b1}) {
            if (!b) continue;
            for (int j = 0; j < g2.n; ++j) {
              if (intPath) {
                reinterpret_cast<int32_t*>(sum.data())[j] += reinterpret_cast<const int32_t*>(b->data())[j];
              } else {
                reinterpret_cast<float*>(sum.data())[j] += reinterpret_cast<const float*>(b->data())[j];
              }
            }
          }
          cudaCheck(cudaMalloc(&bDev, sum.size()), "cudaMalloc(summed bias)");
          exe_->derived_.push_back(bDev);
          cudaCheck(cudaMemcpy(bDev, sum.data(), sum.size(), cudaMemcpyHostToDevice), "upload of the summed bias");
        }
        main.gemm = trial;
        main.a2 = proj.a;
        main.bDerived = wDev;
        main.biasDerived = bDev;
        main.residual = -1;
        main.inputs.erase(std::remove_if(main.inputs.begin(), main.inputs.end(), [&](int v) { return root(v) == mid; }),
                          main.inputs.end());
        main.inputs.push_back(proj.a);
        {
          const size_t at = main.fused.find("+residual");
          const std::string tag = "+shortcut(k" + std::to_string(k1) + (a2Stride > 1 ? "/" + std::to_string(a2Stride) : "") + ")";
          if (at != std::string::npos) main.fused.replace(at, 9, tag);
          else main.fused += tag;
        }
        proj.dropped = true;
        break;
      }
    }
  }

  // A 3 x 3 / 2 max pool (one pixel of padding) right behind a convolution that nothing else reads, where
  // the library has a kernel for the pair (the first layer of image networks: the convolution's output, four
  // times the pooled tensor, is then never written).  Kept only if the library accepts the combined descriptor.
  void fuseConvMaxPool() {
    if (getenvFlag("PLAIDML_CUDA_NO_POOL_FUSION")) return;
    for (size_t r = 0; r < pending_.size(); ++r) {
      Pending& pl = pending_[r];
      if (pl.dropped || pl.kind != Pending::Pool) continue;
      const pmlb_pool_desc& pd = pl.pool;
      if (pd.agg != PMLB_AGG_MAX || pd.r != 3 || pd.s != 3 || pd.stride_h != 2 || pd.stride_w != 2 || pd.pad_h != 1 ||
          pd.pad_w != 1) {
        continue;
      }
      const int mid = root(pl.a);
      for (size_t g = 0; g < r; ++g) {
        Pending& cv = pending_[g];
        if (cv.dropped || cv.kind != Pending::Conv || root(cv.result) != mid) continue;
        const pmlb_conv_desc& cd = cv.conv;
        if (cd.n != pd.n || cd.p != pd.h || cd.q != pd.w || cd.k != pd.c || cd.out_dtype != pd.dtype ||
            pd.p * 2 != cd.p || pd.q * 2 != cd.q || cv.residual >= 0) {
          break;
        }
        // the convolution's output has no other reader and is not a program output
        bool shared = false;
        for (int o : prog_.outputs) shared = shared || root(o) == mid;
        for (size_t k = 0; k < pending_.size() && !shared; ++k) {
          if (k == r || pending_[k].dropped) continue;
          for (int in : pending_[k].inputs) shared = shared || root(in) == mid;
        }
        if (shared) break;
        pmlb_conv_desc trial = cd;
        trial.flags |= PMLB_CONV_MAX_POOL_3X3_S2;
        pmlb_plan* probe = nullptr;
        const pmlb_status rc = pmlb_conv_dispatch(&trial, &probe);
        if (probe) pmlb_plan_free(probe);
        if (rc != PMLB_OK) break;
        cv.conv = trial;
        cv.result = pl.result;
        cv.position = pl.position;
        cv.fused += "+maxpool3x3/2 -> " + std::to_string(pd.p) + "x" + std::to_string(pd.q);
        pl.dropped = true;
        break;
      }
    }
  }

  const PValue& val(int v) const { return prog_.values[v]; }

  // Looks through a widening cast feeding a contraction: returns the cast's source if
  // `v` is cast(bf16|f16 -> f32) or cast(si8 -> si32), else v itself.
  int throughCast(int v) const {
    const PValue& pv = val(v);
    if (pv.def < 0) return v;
    const POp& op = prog_.ops[pv.def];
    if (op.kind != POp::Cast) return v;
    const DType from = val(op.operands[0]).shape.dtype, to = pv.shape.dtype;
    const bool ok = (to == DType::f32 && (from == DType::bf16 || from == DType::f16)) ||
                    (to == DType::si32 && from == DType::si8);
    return ok ? op.operands[0] : v;
  }

  bool denseValue(int v) const { return val(root(v)).shape.isDense(); }

  // ------------------------------------------------------------ contraction planning
  void planContraction(Pending* pd) {
    const POp& op = prog_.ops[pd->op];
    const BoundedContraction& c = *op.c;
    pd->kind = Pending::Generic;
    pd->inputs = op.operands;
    for (int o : op.operands) {
      if (!denseValue(o)) throw std::runtime_error("The cuda target takes dense row-major tensors");
    }
    const Simplified s = simplify(c);
    if (s.ok && !c.hasInit && !getenvFlag("PLAIDML_CUDA_GENERIC_ONLY")) {
      if (c.agg == AggKind::add && c.combo == ComboKind::mul) {
        if (tryConv(pd, s) || tryGemm(pd, s)) return;
      }
      if (c.combo == ComboKind::none && (c.agg == AggKind::add || c.agg == AggKind::max || c.agg == AggKind::min)) {
        if (tryPool(pd, s) || tryReduce(pd, s)) return;
      }
    }
  }

  static bool getenvFlag(const char* name) {
    const char* v = std::getenv(name);
    return v && v[0] && v[0] != '0';
  }

  // Element type triple of a tensor-core contraction; false if the operand types do not
  // form one of the supported combinations.
  bool tcTypes(int opA, int opB, DType resultType, int* a, int* b, int* inDtype, int* outDtype) const {
    const int ca = throughCast(opA), cb = throughCast(opB);
    const DType ta = val(ca).shape.dtype, tb = val(cb).shape.dtype;
    if (ta != tb) {
      // mixed: fall back to the un-cast operands
      const DType ua = val(opA).shape.dtype, ub = val(opB).shape.dtype;
      if (ua != ub) return false;
      *a = opA;
      *b = opB;
      return tcTypesPlain(ua, resultType, inDtype, outDtype);
    }
    if ((ca != opA) != (cb != opB)) {
      // only one side is a cast: e.g. f32 x cast(bf16): use both as written
      const DType ua = val(opA).shape.dtype, ub = val(opB).shape.dtype;
      if (ua != ub) return false;
      *a = opA;
      *b = opB;
      return tcTypesPlain(ua, resultType, inDtype, outDtype);
    }
    *a = ca;
    *b = cb;
    if (ca != opA) {
      // both operands widened by casts: narrow inputs, wide accumulate
      if (ta == DType::si8 && resultType == DType::si32) {
        *inDtype = PMLB_I8;
        *outDtype = PMLB_I32;
        return true;
      }
      if ((ta == DType::bf16 || ta == DType::f16) && resultType == DType::f32) {
        *inDtype = ta == DType::bf16 ? PMLB_BF16 : PMLB_F16;
        *outDtype = PMLB_F32;
        return true;
      }
      return false;
    }
    return tcTypesPlain(ta, resultType, inDtype, outDtype);
  }

  static bool tcTypesPlain(DType t, DType resultType, int* inDtype, int* outDtype) {
    if (t != resultType) return false;
    switch (t) {
      case DType::f32: *inDtype = PMLB_F32; *outDtype = PMLB_F32; return true;
      case DType::bf16: *inDtype = PMLB_BF16; *outDtype = PMLB_BF16; return true;
      case DType::f16: *inDtype = PMLB_F16; *outDtype = PMLB_F16; return true;
      case DType::si8: *inDtype = PMLB_I8; *outDtype = PMLB_I8; return true;
      default: return false;
    }
  }

  // Walks the single-use consumer chain of a tensor-core contraction and folds
  // bias add -> residual add -> relu -> cast into its epilogue.
  void fuseEpilogue(Pending* pd, int inDtype, int* outDtype, int64_t nCols, int* epilogue) {
    const bool intPath = inDtype == PMLB_I8;
    struct Link {
      int op;
      int flag;        // PMLB_EPI_* this link adds, 0 for the cast
      int value;       // value the link produces
    };
    std::vector<Link> chain;
    int cur = pd->result;
    int stage = 0;  // 0 nothing yet, 1 bias, 2 residual, 3 relu, 4 cast
    int bias = -1, resWritten = -1, resSource = -1;
    int castDtype = -1;
    while (stage < 4) {
      if (uses_[cur] != 1 || isOutput_[cur] || users_[cur].size() != 1) break;
      const int ui = users_[cur][0];
      // (an add of two contractions' results is the epilogue of one of them only: the one planned first)
      if (absorbed_[ui]) break;
      const POp& u = prog_.ops[ui];
      const TensorShape& rs = val(u.result).shape;
      if (rs.sizes != val(cur).shape.sizes) break;
      int flag = -1;
      if (u.kind == POp::Eltwise && u.mnemonic == "add" && u.operands.size() == 2 && stage < 3 &&
          rs.dtype == val(cur).shape.dtype) {
        const int other = u.operands[0] == cur ? u.operands[1] : u.operands[0];
        const TensorShape& os = val(other).shape;
        const bool isBias = stage < 1 && os.rank() >= 1 && os.sizes.back() == nCols && os.elements() == nCols &&
                            denseValue(other) && os.dtype == (intPath ? DType::si32 : DType::f32);
        if (isBias) {
          bias = other;
          flag = PMLB_EPI_BIAS;
          stage = 1;
        } else if (stage < 2 && os.sizes == rs.sizes && denseValue(other)) {
          resWritten = other;
          resSource = throughCast(other);
          flag = PMLB_EPI_RESIDUAL;
          stage = 2;
        }
      } else if (u.kind == POp::Eltwise && u.mnemonic == "relu" && stage < 3 && rs.dtype == val(cur).shape.dtype) {
        flag = PMLB_EPI_RELU;
        stage = 3;
      } else if (u.kind == POp::Cast && !intPath && *outDtype == PMLB_F32 &&
                 (rs.dtype == DType::bf16 || rs.dtype == DType::f16)) {
        castDtype = rs.dtype == DType::bf16 ? PMLB_BF16 : PMLB_F16;
        flag = 0;
        stage = 4;
      }
      if (flag < 0) break;
      chain.push_back({ui, flag, u.result});
      cur = u.result;
    }
    // The kernel reads the residual in the element type it stores: keep the residual (and
    // what follows it) only if one of its two forms has that type.
    int finalDtype = castDtype >= 0 ? castDtype : *outDtype;
    int residual = -1;
    if (resWritten >= 0) {
      if (static_cast<int>(val(resSource).shape.dtype) == finalDtype) {
        residual = resSource;
      } else if (static_cast<int>(val(resWritten).shape.dtype) == finalDtype) {
        residual = resWritten;
      } else {
        size_t cut = 0;
        while (cut < chain.size() && chain[cut].flag != PMLB_EPI_RESIDUAL) ++cut;
        chain.resize(cut);
        finalDtype = *outDtype;
      }
    }
    int flags = 0;
    for (const Link& l : chain) {
      flags |= l.flag;
      absorbed_[l.op] = true;
      pd->position = std::max(pd->position, l.op);
    }
    if (!chain.empty()) pd->result = chain.back().value;
    pd->bias = (flags & PMLB_EPI_BIAS) ? bias : -1;
    pd->residual = residual;
    if (pd->bias >= 0) pd->inputs.push_back(pd->bias);
    if (residual >= 0) pd->inputs.push_back(residual);
    *outDtype = finalDtype;
    *epilogue = flags;
    std::ostringstream os;
    if (flags & PMLB_EPI_BIAS) os << "+bias";
    if (flags & PMLB_EPI_RESIDUAL) os << "+residual";
    if (flags & PMLB_EPI_RELU) os << "+relu";
    if (!chain.empty() && chain.back().flag == 0) os << "+cast";
    pd->fused = os.str();
  }

  // Per-variable strides of every tensor if all its dims are pure variables.
  bool pureStrides(const Simplified& s, size_t t, const TensorShape& shape, std::vector<VarUse>* out) const {
    out->assign(s.n, VarUse());
    const std::vector<int64_t> st = shape.denseStrides();
    for (size_t d = 0; d < shape.rank(); ++d) {
      const int v = pureVar(s, t, d);
      if (v == -1) return false;
      if (v == -2) continue;
      if ((*out)[v].present) return false;  // diagonal access
      (*out)[v].present = true;
      (*out)[v].stride = st[d];
    }
    return true;
  }

  struct Merged {
    bool any = false;
    int64_t extent = 1;
    int64_t strideOut = 0, strideA = 0, strideB = 0;
  };

  // Merges the variables of one class (ordered outer to inner by `key` stride) into a
  // single dimension; false if they are not contiguous in every tensor holding them.
  static bool mergeClass(const std::vector<int>& vars, const Simplified& s, const std::vector<VarUse>& o,
                         const std::vector<VarUse>& a, const std::vector<VarUse>& b, int keyTensor, Merged* m) {
    std::vector<int> order = vars;
    auto key = [&](int v) {
      return keyTensor == 0 ? o[v].stride : (keyTensor == 1 ? a[v].stride : b[v].stride);
    };
    std::sort(order.begin(), order.end(), [&](int x, int y) { return key(x) > key(y); });
    m->any = !order.empty();
    m->extent = 1;
    for (size_t i = 0; i < order.size(); ++i) {
      const int v = order[i];
      m->extent *= s.extent[v];
      if (i + 1 < order.size()) {
        const int w = order[i + 1];
        if (o[v].present && o[v].stride != o[w].stride * s.extent[w]) return false;
        if (a[v].present && a[v].stride != a[w].stride * s.extent[w]) return false;
        if (b[v].present && b[v].stride != b[w].stride * s.extent[w]) return false;
      }
    }
    if (!order.empty()) {
      const int inner = order.back();
      m->strideOut = o[inner].stride;
      m->strideA = a[inner].stride;
      m->strideB = b[inner].stride;
    }
    return true;
  }

  bool tryGemm(Pending* pd, const Simplified& s) {
    const POp& op = prog_.ops[pd->op];
    if (op.operands.size() != 2) return false;
    const TensorShape& outShape = val(op.result).shape;
    for (int order = 0; order < 2; ++order) {
      const int opA = op.operands[order], opB = op.operands[1 - order];
      const size_t tA = 1 + order, tB = 2 - order;
      int a, b, inDtype, outDtype;
      if (!tcTypes(opA, opB, outShape.dtype, &a, &b, &inDtype, &outDtype)) return false;
      std::vector<VarUse> uo, ua, ub;
      if (!pureStrides(s, 0, outShape, &uo) || !pureStrides(s, tA, val(opA).shape, &ua) ||
          !pureStrides(s, tB, val(opB).shape, &ub)) {
        return false;
      }
      // The index ranges must cover the whole output: a dim the contraction writes only partly (a range
      // shorter than the dim, or index 0 of a longer dim) keeps the aggregation's identity elsewhere, which
      // the general kernel initialises and this one would leave unwritten.
      bool covers = true;
      for (size_t d = 0; d < outShape.rank(); ++d) {
        const int v = pureVar(s, 0, d);
        const int64_t span = v >= 0 ? s.extent[v] : 1;
        if (span != outShape.sizes[d]) covers = false;
      }
      if (!covers) return false;
      std::vector<int> mv, nv, kv, bv;
      bool bad = false;
      for (size_t i = 0; i < s.n; ++i) {
        if (s.extent[i] <= 1) continue;
        const bool io = uo[i].present, ia = ua[i].present, ib = ub[i].present;
        if (io && ia && ib) bv.push_back(static_cast<int>(i));
        else if (io && ia) mv.push_back(static_cast<int>(i));
        else if (io && ib) nv.push_back(static_cast<int>(i));
        else if (ia && ib) kv.push_back(static_cast<int>(i));
        else bad = true;
      }
      if (bad || kv.empty()) continue;
      Merged M, N, K, B;
      if (!mergeClass(mv, s, uo, ua, ub, 0, &M) || !mergeClass(nv, s, uo, ua, ub, 0, &N) ||
          !mergeClass(kv, s, uo, ua, ub, 1, &K) || !mergeClass(bv, s, uo, ua, ub, 0, &B)) {
        continue;
      }
      // layout the kernel takes: out [batch][m][n] with n contiguous, A with k contiguous
      if (N.any && N.strideOut != 1) continue;
      if (K.strideA != 1) continue;
      const bool bIsNk = K.strideB == 1 && (!N.any || N.strideB >= K.extent);
      const bool bIsKn = N.any ? (N.strideB == 1 && K.strideB >= N.extent) : false;
      if (!bIsNk && !bIsKn) continue;
      if (M.extent > INT32_MAX || N.extent > INT32_MAX || K.extent > INT32_MAX || B.extent > INT32_MAX) continue;
      // batch must be outermost in the output
      if (B.any && M.any && B.strideOut < M.strideOut * M.extent) continue;
      // A tiny fp32 product gains nothing from the tensor cores (the launch dominates) and would lose the
      // last bits to the three-TF32-product form; the general kernel computes it in plain f32, which is what
      // the reference's exact small-matrix expectations (plaidml/edsl/examples/gemm.cc:79-90) were written for.
      if (inDtype == PMLB_F32 && M.extent * N.extent * K.extent * B.extent <= 32768) return false;
      pmlb_gemm_desc d;
      std::memset(&d, 0, sizeof(d));
      d.in_dtype = inDtype;
      d.m = static_cast<int32_t>(M.extent);
      d.n = static_cast<int32_t>(N.extent);
      d.k = static_cast<int32_t>(K.extent);
      d.batch = static_cast<int32_t>(B.extent);
      d.lda = M.any ? M.strideA : K.extent;
      d.ldc = M.any ? M.strideOut : N.extent;
      d.b_is_nk = bIsNk ? 1 : 0;
      d.ldb = bIsNk ? (N.any ? N.strideB : K.extent) : K.strideB;
      d.stride_a = B.any ? B.strideA : 0;
      d.stride_b = B.any ? B.strideB : 0;
      d.stride_c = B.any ? B.strideOut : 0;
      if (d.lda < d.k || d.ldc < d.n) continue;
      if (inDtype != PMLB_F32) {
        // rows of A (and of a [n][k] B) must start on 16-byte boundaries for TMA
        const int64_t eb = inDtype == PMLB_I8 ? 1 : 2;
        if ((d.lda * eb) % 16 != 0 || (d.stride_a * eb) % 16 != 0) continue;
        if (bIsNk && ((d.ldb * eb) % 16 != 0 || (d.stride_b * eb) % 16 != 0)) continue;
      }
      pd->kind = Pending::Gemm;
      pd->a = a;
      pd->b = b;
      pd->inputs = {a, b};
      int epi = 0;
      fuseEpilogue(pd, inDtype, &outDtype, N.extent, &epi);
      d.out_dtype = outDtype;
      d.epilogue = epi;
      d.ldr = d.ldc;
      d.stride_r = d.stride_c;
      pd->gemm = d;
      return true;
    }
    return false;
  }

  // out[n, x0, x1, co] += I[n, s0*x0 + d0*k0 - p0, s1*x1 + d1*k1 - p1, ci] * F[k0, k1, ci, co]
  bool tryConv(Pending* pd, const Simplified& s) {
    const POp& op = prog_.ops[pd->op];
    if (op.operands.size() != 2) return false;
    const TensorShape& outShape = val(op.result).shape;
    if (outShape.rank() != 4) return false;
    for (int order = 0; order < 2; ++order) {
      const int opI = op.operands[order], opF = op.operands[1 - order];
      const size_t tI = 1 + order, tF = 2 - order;
      const TensorShape& is = val(opI).shape;
      const TensorShape& fs = val(opF).shape;
      if (is.rank() != 4 || fs.rank() != 4) continue;
      const int vn = pureVar(s, 0, 0), vx0 = pureVar(s, 0, 1), vx1 = pureVar(s, 0, 2), vco = pureVar(s, 0, 3);
      const int vk0 = pureVar(s, tF, 0), vk1 = pureVar(s, tF, 1), vci = pureVar(s, tF, 2), vco2 = pureVar(s, tF, 3);
      if (vn == -1 || vx0 == -1 || vx1 == -1 || vco < 0 || vk0 == -1 || vk1 == -1 || vci < 0 || vco2 != vco) continue;
      if (pureVar(s, tI, 0) != vn || pureVar(s, tI, 3) != vci) continue;
      // spatial dims of the input: stride * x + dilation * k - pad
      int64_t stride[2] = {1, 1}, dil[2] = {1, 1}, pad[2] = {0, 0};
      const int vx[2] = {vx0, vx1}, vk[2] = {vk0, vk1};
      bool okSpatial = true;
      for (int d = 0; d < 2 && okSpatial; ++d) {
        const auto& row = s.coef[tI][1 + d];
        for (size_t i = 0; i < s.n; ++i) {
          if (row[i] == 0) continue;
          if (static_cast<int>(i) == vx[d]) stride[d] = row[i];
          else if (static_cast<int>(i) == vk[d]) dil[d] = row[i];
          else okSpatial = false;
        }
        if (vx[d] >= 0 && row[vx[d]] <= 0) okSpatial = false;
        if (vk[d] >= 0 && row[vk[d]] <= 0) okSpatial = false;
        pad[d] = -s.cst[tI][1 + d];
        if (pad[d] < 0) okSpatial = false;
      }
      if (!okSpatial) continue;
      // every variable must be one of the seven
      std::set<int> known = {vn, vx0, vx1, vco, vk0, vk1, vci};
      bool extra = false;
      for (size_t i = 0; i < s.n; ++i) {
        if (s.extent[i] > 1 && !known.count(static_cast<int>(i))) extra = true;
      }
      if (extra) continue;
      auto ext = [&](int v) { return v >= 0 ? s.extent[v] : 1; };
      // the recognised variables must span the tensors completely
      if (ext(vn) != outShape.sizes[0] || ext(vx0) != outShape.sizes[1] || ext(vx1) != outShape.sizes[2] ||
          ext(vco) != outShape.sizes[3] || ext(vk0) != fs.sizes[0] || ext(vk1) != fs.sizes[1] ||
          ext(vci) != fs.sizes[2] || ext(vci) != is.sizes[3] || ext(vn) != is.sizes[0]) {
        continue;
      }
      int a, b, inDtype, outDtype;
      if (!tcTypes(opI, opF, outShape.dtype, &a, &b, &inDtype, &outDtype)) continue;
      if (inDtype != PMLB_BF16 && inDtype != PMLB_F16 && inDtype != PMLB_F32) continue;
      // plain 1x1 stride-1 convolutions are GEMMs; let that path take them
      if (fs.sizes[0] == 1 && fs.sizes[1] == 1 && stride[0] == 1 && stride[1] == 1 && pad[0] == 0 && pad[1] == 0) {
        return false;
      }
      pmlb_conv_desc d;
      std::memset(&d, 0, sizeof(d));
      d.in_dtype = inDtype;
      d.n = static_cast<int32_t>(is.sizes[0]);
      d.h = static_cast<int32_t>(is.sizes[1]);
      d.w = static_cast<int32_t>(is.sizes[2]);
      d.c = static_cast<int32_t>(is.sizes[3]);
      d.r = static_cast<int32_t>(fs.sizes[0]);
      d.s = static_cast<int32_t>(fs.sizes[1]);
      d.k = static_cast<int32_t>(fs.sizes[3]);
      d.p = static_cast<int32_t>(outShape.sizes[1]);
      d.q = static_cast<int32_t>(outShape.sizes[2]);
      d.stride_h = static_cast<int32_t>(stride[0]);
      d.stride_w = static_cast<int32_t>(stride[1]);
      d.pad_h = static_cast<int32_t>(pad[0]);
      d.pad_w = static_cast<int32_t>(pad[1]);
      d.dil_h = static_cast<int32_t>(dil[0]);
      d.dil_w = static_cast<int32_t>(dil[1]);
      if (d.pad_h > 127 || d.pad_w > 127 || d.stride_h > 8 || d.stride_w > 8) continue;
      // the im2col route needs whole 16-byte channel groups; thin inputs take the packed-row route
      // (fp32: any channel count, the split pre-pass pads it)
      if (inDtype != PMLB_F32 && d.c % 8 != 0 && !pmlb::conv_takes_packed_rows(d) && !pmlb::conv_takes_s2d(d)) continue;
      pd->kind = Pending::Conv;
      pd->a = a;
      pd->b = b;
      pd->inputs = {a, b};
      int epi = 0;
      fuseEpilogue(pd, inDtype, &outDtype, outShape.sizes[3], &epi);
      d.out_dtype = outDtype;
      d.epilogue = epi;
      pd->conv = d;
      return true;
    }
    return false;
  }

  // out[outer..., inner...] = agg over reduce... of in[outer..., reduce..., inner...]
  bool tryReduce(Pending* pd, const Simplified& s) {
    const POp& op = prog_.ops[pd->op];
    const BoundedContraction& c = *op.c;
    if (op.operands.size() != 1) return false;
    const int src = throughCastForReduce(op.operands[0], val(op.result).shape.dtype, c.agg);
    const TensorShape& outShape = val(op.result).shape;
    const TensorShape& inShape = val(op.operands[0]).shape;
    std::vector<VarUse> uo, ui;
    if (!pureStrides(s, 0, outShape, &uo) || !pureStrides(s, 1, inShape, &ui)) return false;
    // walk the input dims outer -> inner: kept dims, then reduced dims, then kept dims
    int phase = 0;  // 0 outer, 1 reduce, 2 inner
    int64_t outer = 1, red = 1, inner = 1;
    std::vector<int> keptOrder;
    for (size_t d = 0; d < inShape.rank(); ++d) {
      const int v = pureVar(s, 1, d);
      if (v == -1) return false;
      if (v == -2) {
        if (inShape.sizes[d] != 1) return false;  // a fixed slice of a larger dim
        continue;
      }
      if (s.extent[v] != inShape.sizes[d]) return false;
      const bool kept = uo[v].present;
      if (kept) {
        if (phase == 1) phase = 2;
        (phase == 0 ? outer : inner) *= s.extent[v];
        keptOrder.push_back(v);
      } else {
        if (phase == 2) return false;
        phase = 1;
        red *= s.extent[v];
      }
    }
    // kept variables must appear in the output in the same order, densely
    std::vector<int> outOrder;
    for (size_t d = 0; d < outShape.rank(); ++d) {
      const int v = pureVar(s, 0, d);
      if (v == -1) return false;
      if (v == -2) {
        if (outShape.sizes[d] != 1) return false;
        continue;
      }
      if (s.extent[v] != outShape.sizes[d]) return false;
      outOrder.push_back(v);
    }
    if (outOrder != keptOrder) return false;
    const DType inDt = val(src).shape.dtype, outDt = outShape.dtype;
    pmlb_reduce_desc d;
    std::memset(&d, 0, sizeof(d));
    d.agg = pmlbAgg(c.agg);
    d.dtype = static_cast<int>(inDt);
    d.out_dtype = static_cast<int>(outDt);
    d.outer = outer;
    d.reduce = red;
    d.inner = inner;
    d.scale = 1.0;
    const bool typesOk = (inDt == outDt && (inDt == DType::f32 || inDt == DType::bf16 || inDt == DType::f16 ||
                                            inDt == DType::si32 || inDt == DType::si8)) ||
                         (outDt == DType::f32 && (inDt == DType::bf16 || inDt == DType::f16));
    if (!typesOk) return false;
    pd->kind = Pending::Reduce;
    pd->reduce = d;
    pd->a = src;
    pd->inputs = {src};
    fuseMeanTail(pd);
    return true;
  }

  // sum -> div by a literal -> (cast back to the 16-bit input type): the tail of `mean`
  // (plaidml/op/lib/ops.cc:1970-2003) folds into the reduction kernel, which divides its f32
  // sum by the count and rounds once.
  void fuseMeanTail(Pending* pd) {
    pmlb_reduce_desc& d = pd->reduce;
    if (d.agg != PMLB_AGG_SUM || d.out_dtype != PMLB_F32) return;
    int cur = pd->result;
    auto soleUser = [&](int v) -> int {
      if (uses_[v] != 1 || isOutput_[v] || users_[v].size() != 1) return -1;
      return users_[v][0];
    };
    const int di = soleUser(cur);
    if (di < 0) return;
    const POp& dv = prog_.ops[di];
    if (dv.kind != POp::Eltwise || dv.mnemonic != "div" || dv.operands.size() != 2 || dv.operands[0] != cur) return;
    // (a literal operand of an element-wise operation is a rank-0 internal constant of the other operand's type)
    const PValue& lit = val(dv.operands[1]);
    if (lit.kind != PValue::InternalConstant || !lit.constant || lit.shape.elements() != 1 ||
        lit.shape.dtype != DType::f32) {
      return;
    }
    const double count = static_cast<double>(*reinterpret_cast<const float*>(lit.constant->data()));
    const TensorShape& rs = val(dv.result).shape;
    if (!(count > 0) || rs.sizes != val(cur).shape.sizes || rs.dtype != DType::f32) return;
    d.scale = count;
    d.divide = 1;
    absorbed_[di] = true;
    pd->position = std::max(pd->position, di);
    pd->result = dv.result;
    pd->fused = "+div";
    // ... -> cast to the type the input has: the kernel's same-type form (f32 sum, one rounding)
    const int ci = soleUser(dv.result);
    if (ci < 0) return;
    const POp& cs = prog_.ops[ci];
    const DType ct = val(cs.result).shape.dtype;
    if (cs.kind != POp::Cast || static_cast<int>(ct) != d.dtype || !(ct == DType::bf16 || ct == DType::f16)) return;
    d.out_dtype = d.dtype;
    absorbed_[ci] = true;
    pd->position = std::max(pd->position, ci);
    pd->result = cs.result;
    pd->fused += "+cast";
  }

  // sum(cast(x: 16-bit float -> f32)) can read x directly (the widening is exact); for
  // max / min only when nothing else is gained, so keep the cast there.
  int throughCastForReduce(int v, DType resultType, AggKind agg) const {
    if (agg != AggKind::add || resultType != DType::f32) return v;
    const int c = throughCast(v);
    const DType t = val(c).shape.dtype;
    return (t == DType::bf16 || t == DType::f16) ? c : v;
  }

  // out[n, x0, x1, c] = agg I[n, s0*x0 + k0 - p0, s1*x1 + k1 - p1, c]
  bool tryPool(Pending* pd, const Simplified& s) {
    const POp& op = prog_.ops[pd->op];
    const BoundedContraction& c = *op.c;
    if (op.operands.size() != 1) return false;
    const TensorShape& outShape = val(op.result).shape;
    const TensorShape& is = val(op.operands[0]).shape;
    if (outShape.rank() != 4 || is.rank() != 4 || is.dtype != outShape.dtype) return false;
    const int vn = pureVar(s, 0, 0), vx0 = pureVar(s, 0, 1), vx1 = pureVar(s, 0, 2), vc = pureVar(s, 0, 3);
    if (vn == -1 || vx0 == -1 || vx1 == -1 || vc == -1) return false;
    if (pureVar(s, 1, 0) != vn || pureVar(s, 1, 3) != vc) return false;
    int64_t stride[2] = {1, 1}, pad[2] = {0, 0}, win[2] = {1, 1};
    const int vx[2] = {vx0, vx1};
    int vk[2] = {-1, -1};
    for (int d = 0; d < 2; ++d) {
      const auto& row = s.coef[1][1 + d];
      for (size_t i = 0; i < s.n; ++i) {
        if (row[i] == 0) continue;
        if (static_cast<int>(i) == vx[d]) {
          stride[d] = row[i];
        } else if (vk[d] < 0 && row[i] == 1) {
          vk[d] = static_cast<int>(i);
          win[d] = s.extent[i];
        } else {
          return false;
        }
      }
      if (vx[d] >= 0 && stride[d] <= 0) return false;
      pad[d] = -s.cst[1][1 + d];
      if (pad[d] < 0) return false;
    }
    if (vk[0] >= 0 && vk[0] == vk[1]) return false;
    std::set<int> known = {vn, vx0, vx1, vc, vk[0], vk[1]};
    for (size_t i = 0; i < s.n; ++i) {
      if (s.extent[i] > 1 && !known.count(static_cast<int>(i))) return false;
    }
    // window variables must not appear in the output
    for (int d = 0; d < 2; ++d) {
      if (vk[d] >= 0) {
        for (size_t od = 0; od < 4; ++od) {
          if (s.coef[0][od][vk[d]] != 0) return false;
        }
      }
    }
    auto ext = [&](int v) { return v >= 0 ? s.extent[v] : 1; };
    if (ext(vn) != outShape.sizes[0] || ext(vx0) != outShape.sizes[1] || ext(vx1) != outShape.sizes[2] ||
        ext(vc) != outShape.sizes[3] || ext(vn) != is.sizes[0] || ext(vc) != is.sizes[3]) {
      return false;
    }
    if (win[0] == 1 && win[1] == 1 && stride[0] == 1 && stride[1] == 1) return false;  // a copy, not a pool
    const DType dt = is.dtype;
    if (!(dt == DType::f32 || dt == DType::bf16 || dt == DType::f16 || dt == DType::si32 || dt == DType::si8)) return false;
    pmlb_pool_desc d;
    std::memset(&d, 0, sizeof(d));
    d.agg = pmlbAgg(c.agg);
    d.dtype = static_cast<int>(dt);
    d.n = static_cast<int32_t>(is.sizes[0]);
    d.h = static_cast<int32_t>(is.sizes[1]);
    d.w = static_cast<int32_t>(is.sizes[2]);
    d.c = static_cast<int32_t>(is.sizes[3]);
    d.r = static_cast<int32_t>(win[0]);
    d.s = static_cast<int32_t>(win[1]);
    d.p = static_cast<int32_t>(outShape.sizes[1]);
    d.q = static_cast<int32_t>(outShape.sizes[2]);
    d.stride_h = static_cast<int32_t>(stride[0]);
    d.stride_w = static_cast<int32_t>(stride[1]);
    d.pad_h = static_cast<int32_t>(pad[0]);
    d.pad_w = static_cast<int32_t>(pad[1]);
    pd->kind = Pending::Pool;
    pd->pool = d;
    pd->a = op.operands[0];
    pd->inputs = {op.operands[0]};
    return true;
  }

  // ------------------------------------------------------------ memory
  void allocate(const std::vector<bool>& needed) {
    const size_t nv = prog_.values.size();
    exe_->dev_.assign(nv, nullptr);
    std::vector<size_t> offset(nv, 0);
    size_t total = 0;
    for (size_t v = 0; v < nv; ++v) {
      const PValue& pv = prog_.values[v];
      if (pv.kind == PValue::LiteralValue) continue;
      if (alias_[v] >= 0) continue;
      const bool arg = pv.kind == PValue::Input;
      if (!needed[v] && !arg) continue;
      size_t bytes = pv.shape.byteSize();
      if (bytes == 0) bytes = 16;
      offset[v] = total;
      total += (bytes + 255) / 256 * 256;
    }
    exe_->arenaBytes_ = total ? total : 256;
    cudaCheck(cudaMalloc(reinterpret_cast<void**>(&exe_->arena_), exe_->arenaBytes_), "cudaMalloc(program arena)");
    for (size_t v = 0; v < nv; ++v) {
      const PValue& pv = prog_.values[v];
      if (pv.kind == PValue::LiteralValue || alias_[v] >= 0) continue;
      if (!needed[v] && pv.kind != PValue::Input) continue;
      exe_->dev_[v] = exe_->arena_ + offset[v];
    }
    for (size_t v = 0; v < nv; ++v) {
      if (alias_[v] >= 0) exe_->dev_[v] = exe_->dev_[root(static_cast<int>(v))];
    }
    // constants are uploaded once, like the reference packs them in its `init` closure
    for (size_t v = 0; v < nv; ++v) {
      const PValue& pv = prog_.values[v];
      if ((pv.kind == PValue::Constant || pv.kind == PValue::InternalConstant) && exe_->dev_[v]) {
        cudaCheck(cudaMemcpyAsync(exe_->dev_[v], pv.constant->data(), pv.shape.byteSize(), cudaMemcpyHostToDevice,
                                  exe_->stream_),
                  "upload of a constant");
      }
    }
    cudaCheck(cudaStreamSynchronize(exe_->stream_), "constant upload");
  }

  char* dev(int v) const {
    char* p = exe_->dev_[v];
    if (!p) throw std::runtime_error("internal: value %" + std::to_string(v) + " was never materialised");
    return p;
  }

  // ------------------------------------------------------------ kernel plans
  void emit(const Pending& pd) {
    const POp& op = prog_.ops[pd.op];
    Step st;
    const std::string label = op.label.empty() ? op.mnemonic : op.label;
    switch (pd.kind) {
      case Pending::Gemm: {
        pmlb_plan* plan = nullptr;
        pmlb_status rc = pmlb_gemm_dispatch(&pd.gemm, &plan);
        if (rc == PMLB_ERR_UNSUPPORTED) {
          emitGenericFallback(pd, std::string("tensor-core GEMM not applicable: ") + pmlb_last_error());
          return;
        }
        pmlbCheck(rc, "gemm dispatch for '" + label + "'");
        pmlbCheck(pmlb_plan_share_status(plan, exe_->status_), "status word");
        st.plan = plan;
        st.kernel = "tc_gemm";
        std::ostringstream os;
        os << label << " b" << pd.gemm.batch << " m" << pd.gemm.m << " n" << pd.gemm.n << " k" << pd.gemm.k
           << " in=" << dtypeName(static_cast<DType>(pd.gemm.in_dtype)) << " out=" << dtypeName(static_cast<DType>(pd.gemm.out_dtype))
           << (pd.gemm.b_is_nk ? " B[n][k]" : " B[k][n]") << pd.fused;
        if (pmlb_plan_split_k(plan) > 1) os << " splitk=" << pmlb_plan_split_k(plan);
        st.detail = os.str();
        // (+ the TF32 split of both operands, + the row-max fill, + the combining pass of a split K range)
        st.launches = 1 + (pd.gemm.in_dtype == PMLB_F32 ? 1 : 0) + (pd.rowmax >= 0 ? 1 : 0) + (pmlb_plan_split_k(plan) > 1 ? 1 : 0);
        const void* a = dev(pd.a);
        const void* a2 = pd.a2 >= 0 ? dev(pd.a2) : nullptr;
        const void* b = pd.bDerived ? pd.bDerived : dev(pd.b);
        void* c = pd.storeMain ? dev(pd.result) : nullptr;
        const void* bias = pd.biasDerived ? pd.biasDerived : (pd.bias >= 0 && !pd.bDerived ? dev(pd.bias) : nullptr);
        const void* res = pd.residual >= 0 ? dev(pd.residual) : nullptr;
        float* rowmax = pd.rowmax >= 0 ? reinterpret_cast<float*>(dev(pd.rowmax)) : nullptr;
        st.launch = [plan, a, a2, b, c, bias, res, rowmax](cudaStream_t s) {
          return pmlb_gemm_invoke_two(plan, s, a, a2, b, c, bias, res, rowmax);
        };
        // row-sliceable: plain 8/16-bit GEMM from a program input to a program output
        if (pd.gemm.batch == 1 && pd.gemm.in_dtype != PMLB_F32 && pd.rowmax < 0 && pd.residual < 0 && pd.storeMain &&
            pd.gemm.lda == pd.gemm.k && pd.gemm.ldc == pd.gemm.n) {
          const int aRoot = root(pd.a), cRoot = root(pd.result);
          for (size_t i = 0; i < prog_.inputs.size(); ++i) {
            if (prog_.inputs[i] == aRoot) st.aInput = static_cast<int>(i);
          }
          for (size_t i = 0; i < prog_.outputs.size(); ++i) {
            if (root(prog_.outputs[i]) == cRoot) st.cOutput = static_cast<int>(i);
          }
          if (st.aInput >= 0 && st.cOutput >= 0 && aRoot != root(pd.b)) {
            st.rowSliceable = true;
            st.gemm = pd.gemm;
            st.bPtr = b;
            st.biasPtr = bias;
          }
        }
        break;
      }
      case Pending::Conv: {
        pmlb_plan* plan = nullptr;
        pmlb_status rc = pmlb_conv_dispatch(&pd.conv, &plan);
        if (rc == PMLB_ERR_UNSUPPORTED) {
          emitGenericFallback(pd, std::string("implicit-GEMM convolution not applicable: ") + pmlb_last_error());
          return;
        }
        pmlbCheck(rc, "conv dispatch for '" + label + "'");
        pmlbCheck(pmlb_plan_share_status(plan, exe_->status_), "status word");
        st.plan = plan;
        st.kernel = pmlb_plan_kind(plan);          // "tc_conv", "tc_conv_halo", "tc_conv_rows", "tc_conv_s2d" or "tc_conv_s2d_pool"
        const std::string route = st.kernel;
        const int extra = (route == "tc_conv_rows" || route == "tc_conv_s2d" || route == "tc_conv_s2d_pool") ? 1 : 0;   // their activation packing pass
        st.launches = 1 + extra;
        std::ostringstream os;
        const pmlb_conv_desc& d = pd.conv;
        os << label << " n" << d.n << " " << d.h << "x" << d.w << "x" << d.c << " (*) " << d.r << "x" << d.s << "/"
           << d.stride_h << " pad" << d.pad_h << " -> " << d.p << "x" << d.q << "x" << d.k
           << " out=" << dtypeName(static_cast<DType>(d.out_dtype)) << pd.fused;
        st.detail = os.str();
        const void* x = dev(pd.a);
        const void* f = dev(pd.b);
        void* out = dev(pd.result);
        const void* bias = pd.bias >= 0 ? dev(pd.bias) : nullptr;
        const void* res = pd.residual >= 0 ? dev(pd.residual) : nullptr;
        const int fdt = static_cast<int>(val(pd.b).shape.dtype);
        const PValue::Kind fk = val(root(pd.b)).kind;
        if (fk == PValue::Constant || fk == PValue::InternalConstant) {
          // weights known now: lay them out once
          pmlbCheck(pmlb_conv_set_filter(plan, exe_->stream_, f, fdt), "filter layout");
          st.launch = [plan, x, out, bias, res](cudaStream_t s) { return pmlb_conv_invoke(plan, s, x, out, bias, res); };
        } else {
          st.launches = 2 + extra;
          st.launch = [plan, x, f, fdt, out, bias, res](cudaStream_t s) {
            pmlb_status r = pmlb_conv_set_filter(plan, s, f, fdt);
            if (r != PMLB_OK) return r;
            return pmlb_conv_invoke(plan, s, x, out, bias, res);
          };
        }
        break;
      }
      case Pending::Reduce: {
        pmlb_plan* plan = nullptr;
        pmlb_status rc = pmlb_reduce_dispatch(&pd.reduce, &plan);
        if (rc == PMLB_ERR_UNSUPPORTED) {
          emitGenericFallback(pd, "reduction kernel not applicable");
          return;
        }
        pmlbCheck(rc, "reduce dispatch for '" + label + "'");
        st.plan = plan;
        st.kernel = pmlb_plan_kind(plan);
        std::ostringstream os;
        os << label << " outer" << pd.reduce.outer << " reduce" << pd.reduce.reduce << " inner" << pd.reduce.inner << pd.fused;
        st.detail = os.str();
        const void* in = dev(pd.a);
        void* out = dev(pd.result);
        st.launch = [plan, in, out](cudaStream_t s) { return pmlb_reduce_invoke(plan, s, in, out); };
        break;
      }
      case Pending::Pool: {
        pmlb_plan* plan = nullptr;
        pmlb_status rc = pmlb_pool_dispatch(&pd.pool, &plan);
        if (rc == PMLB_ERR_UNSUPPORTED) {
          emitGenericFallback(pd, "pooling kernel not applicable");
          return;
        }
        pmlbCheck(rc, "pool dispatch for '" + label + "'");
        st.plan = plan;
        st.kernel = "nhwc_pool";
        std::ostringstream os;
        os << label << " " << pd.pool.r << "x" << pd.pool.s << "/" << pd.pool.stride_h;
        st.detail = os.str();
        const void* in = dev(pd.a);
        void* out = dev(pd.result);
        st.launch = [plan, in, out](cudaStream_t s) { return pmlb_pool_invoke(plan, s, in, out); };
        break;
      }
      case Pending::Generic:
        emitGeneric(pd, "");
        return;
      case Pending::Eltwise:
        emitEltwise(pd);
        return;
      case Pending::Special:
        emitSpecial(pd);
        return;
    }
    exe_->steps_.push_back(std::move(st));
  }

  // A specialised plan was refused at dispatch: undo its fusions and run the contraction,
  // then the fused element-wise operations, on the general kernels.
  void emitGenericFallback(const Pending& pd, const std::string& why) {
    const POp& op = prog_.ops[pd.op];
    if (pd.rowmax >= 0) {
      // (fuseRowMaxima dispatches the combined descriptor before it drops the reduction step)
      throw std::runtime_error("Contraction '" + op.label + "': " + why + " (after a row maximum was folded into it)");
    }
    if (pd.result != op.result) {
      throw std::runtime_error("Contraction '" + op.label + "': " + why +
                               " (after its consumers were fused; re-run with PLAIDML_CUDA_GENERIC_ONLY=1)");
    }
    // operands that were reached through casts are read with their own types
    Pending g = pd;
    g.kind = Pending::Generic;
    std::vector<int> ins;
    if (pd.kind == Pending::Gemm || pd.kind == Pending::Conv) {
      // keep the looked-through sources in the original operand order
      ins = pd.swapped ? std::vector<int>{pd.b, pd.a} : std::vector<int>{pd.a, pd.b};
      // operand order of the contraction is that of op.operands; match by looking through casts
      std::vector<int> ordered;
      for (int o : op.operands) {
        const int t = throughCast(o);
        ordered.push_back((t == pd.a || t == pd.b) ? t : o);
      }
      ins = ordered;
    } else {
      ins = {pd.a};
    }
    g.inputs = ins;
    emitGeneric(g, why);
  }

  void emitGeneric(const Pending& pd, const std::string& why) {
    const POp& op = prog_.ops[pd.op];
    const BoundedContraction& c = *op.c;
    const TensorShape& outShape = val(op.result).shape;
    if (c.nIdx() > PMLB_MAX_IDX) throw std::runtime_error("Contraction uses more than 10 index variables");
    if (c.cons.size() > PMLB_MAX_CONS) throw std::runtime_error("Contraction has more than 8 constraints");
    pmlb_contract_desc d;
    std::memset(&d, 0, sizeof(d));
    d.agg = pmlbAgg(c.agg);
    d.combo = pmlbCombo(c.combo);
    d.n_idx = static_cast<int32_t>(c.nIdx());
    d.n_src = static_cast<int32_t>(c.srcs.size());
    for (size_t i = 0; i < c.nIdx(); ++i) d.range[i] = c.extent[i];
    auto fill = [&](pmlb_access* acc, const std::vector<Affine>& forms, const TensorShape& shape, DType dt) {
      if (shape.rank() > PMLB_MAX_RANK) throw std::runtime_error("Tensors of rank above 8 are not supported");
      acc->dtype = static_cast<int32_t>(dt);
      acc->rank = static_cast<int32_t>(shape.rank());
      const std::vector<int64_t> st = shape.denseStrides();
      for (size_t dd = 0; dd < shape.rank(); ++dd) {
        acc->sizes[dd] = shape.sizes[dd];
        acc->strides[dd] = st[dd];
        const Affine& a = forms[dd];
        int64_t den = a.constant.den;
        for (size_t i = 0; i < c.nIdx(); ++i) {
          const int64_t di = i < a.coef.size() ? a.coef[i].den : 1;
          den = den / std::__gcd(den, di) * di;
        }
        Rational k = a.constant;
        for (size_t i = 0; i < c.nIdx(); ++i) {
          const Rational ci = i < a.coef.size() ? a.coef[i] : Rational(0);
          k = k + ci * Rational(c.lower[i]);
          acc->coef[dd][i] = static_cast<int32_t>(ci.num * (den / ci.den));
        }
        acc->off[dd] = k.num * (den / k.den);
        acc->den[dd] = static_cast<int32_t>(den);
      }
    };
    fill(&d.out, c.sink, outShape, outShape.dtype);
    std::vector<const void*> srcPtrs;
    for (size_t s2 = 0; s2 < c.srcs.size(); ++s2) {
      const int v = pd.inputs.size() > s2 ? pd.inputs[s2] : op.operands[s2];
      fill(&d.src[s2], c.srcs[s2], val(op.operands[s2]).shape, val(v).shape.dtype);
      srcPtrs.push_back(dev(v));
    }
    while (srcPtrs.size() < 3) srcPtrs.push_back(nullptr);
    d.n_cons = static_cast<int32_t>(c.cons.size());
    for (size_t q = 0; q < c.cons.size(); ++q) {
      const Affine& a = c.cons[q].first;
      int64_t den = a.constant.den;
      for (size_t i = 0; i < c.nIdx(); ++i) {
        const int64_t di = i < a.coef.size() ? a.coef[i].den : 1;
        den = den / std::__gcd(den, di) * di;
      }
      Rational k = a.constant;
      for (size_t i = 0; i < c.nIdx(); ++i) {
        const Rational ci = i < a.coef.size() ? a.coef[i] : Rational(0);
        k = k + ci * Rational(c.lower[i]);
        d.cons_coef[q][i] = static_cast<int32_t>(ci.num * (den / ci.den));
      }
      // 0 <= form < bound, scaled by the common denominator
      d.cons_off[q] = k.num * (den / k.den);
      d.cons_range[q] = c.cons[q].second * den;
    }
    const void* initPtr = nullptr;
    if (c.hasInit) {
      const int iv = op.operands.back();
      const TensorShape& is = val(iv).shape;
      d.has_init = 1;
      d.init.dtype = static_cast<int32_t>(is.dtype);
      d.init.rank = static_cast<int32_t>(outShape.rank());
      const std::vector<int64_t> st = is.denseStrides();
      const size_t shift = outShape.rank() - is.rank();
      for (size_t dd = 0; dd < outShape.rank(); ++dd) {
        d.init.sizes[dd] = outShape.sizes[dd];
        d.init.den[dd] = 1;
        if (dd < shift) {
          d.init.strides[dd] = 0;
        } else {
          const size_t sd = dd - shift;
          d.init.strides[dd] = (is.sizes[sd] == 1 && outShape.sizes[dd] != 1) ? 0 : st[sd];
        }
      }
      initPtr = dev(iv);
    }
    pmlb_plan* plan = nullptr;
    pmlbCheck(pmlb_contract_dispatch(&d, &plan), "general contraction dispatch for '" + op.label + "'");
    Step st;
    st.plan = plan;
    st.kernel = "generic_contract";
    st.detail = (op.label.empty() ? std::string("contract") : op.label) + " -> " + outShape.str() +
                (why.empty() ? "" : " [" + why + "]");
    void* out = dev(op.result);
    const void* s0 = srcPtrs[0];
    const void* s1 = srcPtrs[1];
    const void* s2p = srcPtrs[2];
    st.launch = [plan, s0, s1, s2p, initPtr, out](cudaStream_t s) {
      return pmlb_contract_invoke(plan, s, s0, s1, s2p, initPtr, out);
    };
    exe_->steps_.push_back(std::move(st));
  }

  void emitEltwise(const Pending& pd) {
    const POp& op = prog_.ops[pd.op];
    const TensorShape& outShape = val(op.result).shape;
    if (outShape.rank() > PMLB_MAX_RANK) throw std::runtime_error("Tensors of rank above 8 are not supported");
    if (op.operands.size() > 3) throw std::runtime_error("Element-wise '" + op.mnemonic + "' takes more than three operands");
    pmlb_eltwise_desc d;
    std::memset(&d, 0, sizeof(d));
    std::strncpy(d.op, op.mnemonic == "pragma" ? "ident" : op.mnemonic.c_str(), sizeof(d.op) - 1);   // a pragma copies its operand
    d.n_in = static_cast<int32_t>(op.operands.size());
    d.rank = static_cast<int32_t>(outShape.rank());
    d.out_dtype = static_cast<int32_t>(outShape.dtype);
    for (size_t i = 0; i < outShape.rank(); ++i) d.sizes[i] = outShape.sizes[i];
    const void* ins[3] = {nullptr, nullptr, nullptr};
    for (size_t k = 0; k < op.operands.size(); ++k) {
      const TensorShape& is = val(op.operands[k]).shape;
      d.in_dtype[k] = static_cast<int32_t>(is.dtype);
      const std::vector<int64_t> st = is.denseStrides();
      if (is.rank() > outShape.rank()) throw std::runtime_error("Element-wise operand has higher rank than the result");
      const size_t shift = outShape.rank() - is.rank();
      for (size_t dd = shift; dd < outShape.rank(); ++dd) {
        const size_t sd = dd - shift;
        d.in_strides[k][dd] = (is.sizes[sd] == 1 && outShape.sizes[dd] != 1) ? 0 : st[sd];
      }
      ins[k] = dev(op.operands[k]);
    }
    pmlb_plan* plan = nullptr;
    pmlbCheck(pmlb_eltwise_dispatch(&d, &plan), "element-wise dispatch for '" + op.mnemonic + "'");
    Step st;
    st.plan = plan;
    st.kernel = "eltwise";
    st.detail = op.mnemonic + " -> " + outShape.str();
    void* out = dev(op.result);
    const void* i0 = ins[0];
    const void* i1 = ins[1];
    const void* i2 = ins[2];
    st.launch = [plan, i0, i1, i2, out](cudaStream_t s) { return pmlb_eltwise_invoke(plan, s, i0, i1, i2, out); };
    exe_->steps_.push_back(std::move(st));
  }

  // gather / scatter / argsort / prng: one descriptor each, no fusion with their neighbours.
  void emitSpecial(const Pending& pd) {
    const POp& op = prog_.ops[pd.op];
    const PSpecial& sp = *op.s;
    const TensorShape& outShape = val(op.result).shape;
    pmlb_special_desc d;
    std::memset(&d, 0, sizeof(d));
    auto sizes = [&](const TensorShape& shape, int32_t* rank, int64_t* into) {
      if (shape.rank() > PMLB_MAX_RANK) throw std::runtime_error("Tensors of rank above 8 are not supported");
      *rank = static_cast<int32_t>(shape.rank());
      for (size_t i = 0; i < shape.rank(); ++i) into[i] = shape.sizes[i];
    };
    const TensorShape& first = val(op.operands[0]).shape;
    const void* in0 = dev(op.operands[0]);
    const void* in1 = op.operands.size() > 1 ? dev(op.operands[1]) : nullptr;
    const void* in2 = op.operands.size() > 2 ? dev(op.operands[2]) : nullptr;
    void* out0 = dev(op.result);
    void* out1 = nullptr;
    switch (sp.op) {
      case PSpecial::Gather:
        d.op = PMLB_SPECIAL_GATHER;
        d.dtype = static_cast<int32_t>(first.dtype);
        d.idx_dtype = static_cast<int32_t>(val(op.operands[1]).shape.dtype);
        sizes(first, &d.rank, d.sizes);
        sizes(val(op.operands[1]).shape, &d.idx_rank, d.idx_sizes);
        d.axis = static_cast<int32_t>(sp.axis);
        d.mode = static_cast<int32_t>(sp.mode);
        d.batch_dims = static_cast<int32_t>(sp.batchDims);
        d.interpolation = static_cast<int32_t>(sp.interpolation);
        d.nearest = static_cast<int32_t>(sp.nearest);
        d.out_of_bounds = static_cast<int32_t>(sp.outOfBounds);
        d.cube_coeff = sp.cubeCoeff;
        break;
      case PSpecial::Scatter:
        d.op = PMLB_SPECIAL_SCATTER;
        d.dtype = static_cast<int32_t>(first.dtype);
        d.idx_dtype = static_cast<int32_t>(val(op.operands[1]).shape.dtype);
        sizes(first, &d.rank, d.sizes);
        sizes(val(op.operands[1]).shape, &d.idx_rank, d.idx_sizes);
        sizes(val(op.operands[2]).shape, &d.upd_rank, d.upd_sizes);
        d.axis = static_cast<int32_t>(sp.axis);
        d.mode = static_cast<int32_t>(sp.mode);
        break;
      case PSpecial::ArgSort:
        d.op = PMLB_SPECIAL_ARGSORT;
        d.dtype = static_cast<int32_t>(first.dtype);
        sizes(first, &d.rank, d.sizes);
        d.axis = static_cast<int32_t>(sp.axis < 0 ? sp.axis + static_cast<int64_t>(first.rank()) : sp.axis);
        d.mode = static_cast<int32_t>(sp.mode);
        break;
      case PSpecial::Prng:
        d.op = PMLB_SPECIAL_PRNG;
        sizes(outShape, &d.rank, d.sizes);
        d.state_elems = first.elements();
        break;
      case PSpecial::PrngState: {
        // the state after the numbers of the paired operation: the same generator, nothing written but the state
        d.op = PMLB_SPECIAL_PRNG;
        TensorShape numbers(DType::f32, sp.dims);
        sizes(numbers, &d.rank, d.sizes);
        d.state_elems = first.elements();
        out1 = out0;
        out0 = nullptr;
        break;
      }
    }
    pmlb_plan* plan = nullptr;
    pmlbCheck(pmlb_special_dispatch(&d, &plan), "dispatch of '" + op.mnemonic + "'");
    if (sp.op != PSpecial::PrngState && pmlb_special_out_elems(&d) != outShape.elements()) {
      pmlb_plan_free(plan);
      throw std::runtime_error("'" + op.mnemonic + "': result shape " + outShape.str() + " does not follow from its operands");
    }
    Step st;
    st.plan = plan;
    st.kernel = op.mnemonic;
    st.detail = op.mnemonic + " -> " + outShape.str();
    if (sp.op == PSpecial::ArgSort) {
      // one block sort of runs of up to 4096 positions, then a merge pass per doubling beyond that
      int passes = 0;
      while ((int64_t{1} << passes) < first.sizes[d.axis]) ++passes;
      st.launches = 1 + (passes > 12 ? passes - 12 : 0);
    }
    st.launch = [plan, in0, in1, in2, out0, out1](cudaStream_t s) {
      return pmlb_special_invoke(plan, s, in0, in1, in2, out0, out1);
    };
    exe_->steps_.push_back(std::move(st));
  }

  Executable* exe_;
  const Program& prog_;
  std::vector<int> uses_;
  std::vector<bool> isOutput_;
  std::vector<std::vector<int>> users_;
  std::vector<bool> absorbed_;
  std::vector<int> alias_;
  std::vector<Pending> pending_;
};

// ==================================================================== executable

Executable::Executable(std::shared_ptr<Program> program, int device) : prog_(std::move(program)), device_(device) {
  int count = 0;
  if (cudaGetDeviceCount(&count) != cudaSuccess || count == 0) {
    cudaGetLastError();
    throw std::runtime_error("No CUDA device is available; the cuda target has no CPU execution path");
  }
  if (device < 0 || device >= count) throw std::runtime_error("No such device: cuda." + std::to_string(device));
  cudaCheck(cudaSetDevice(device_), "cudaSetDevice");
  int major = 0;
  cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, device_);
  if (major != 10) throw std::runtime_error("cuda." + std::to_string(device) + " is not an sm_100 device");
  for (int id : prog_->inputs) {
    if (!prog_->values[id].shape.isDense()) throw std::runtime_error("The cuda target takes dense row-major inputs");
  }
  cudaCheck(cudaStreamCreateWithFlags(&stream_, cudaStreamNonBlocking), "cudaStreamCreate");
  cudaCheck(cudaEventCreate(&evStart_), "cudaEventCreate");
  cudaCheck(cudaEventCreate(&evStop_), "cudaEventCreate");
  cudaCheck(cudaMalloc(reinterpret_cast<void**>(&status_), sizeof(int)), "cudaMalloc(status)");
  cudaCheck(cudaMemset(status_, 0, sizeof(int)), "cudaMemset(status)");
  try {
    Planner planner(this);
    planner.run();
    cudaCheck(cudaStreamSynchronize(stream_), "executable set-up");
  } catch (...) {
    for (Step& s : steps_) pmlb_plan_free(s.plan);
    steps_.clear();
    for (void* q : derived_) cudaFree(q);
    derived_.clear();
    if (arena_) cudaFree(arena_);
    cudaFree(status_);
    cudaEventDestroy(evStart_);
    cudaEventDestroy(evStop_);
    cudaStreamDestroy(stream_);
    throw;
  }
}

Executable::~Executable() {
  cudaSetDevice(device_);
  if (stream_) cudaStreamSynchronize(stream_);
  for (pmlb_plan* q : slicePlans_) pmlb_plan_free(q);
  for (pmlb_plan* q : blockPlans_) pmlb_plan_free(q);
  for (cudaEvent_t ev : sliceDone_) cudaEventDestroy(ev);
  if (copyStream_) cudaStreamDestroy(copyStream_);
  for (cudaGraphExec_t g : graphs_) cudaGraphExecDestroy(g);
  for (cudaEvent_t ev : groupReady_) cudaEventDestroy(ev);
  if (uploadStream_) cudaStreamDestroy(uploadStream_);
  for (Step& s : steps_) pmlb_plan_free(s.plan);
  for (void* q : derived_) cudaFree(q);
  if (arena_) cudaFree(arena_);
  if (flush_) cudaFree(flush_);
  if (gathered_) cudaFree(gathered_);
  if (status_) cudaFree(status_);
  if (evStart_) cudaEventDestroy(evStart_);
  if (evStop_) cudaEventDestroy(evStop_);
  for (cudaEvent_t ev : timingEvents_) cudaEventDestroy(ev);
  if (stream_) cudaStreamDestroy(stream_);
}

void Executable::launchStepsDirect(size_t first, size_t last) {
  for (size_t i = first; i < last; ++i) {
    Step& s = steps_[i];
    const pmlb_status rc = s.launch(stream_);
    if (rc != PMLB_OK) throw std::runtime_error("Kernel step '" + s.kernel + " " + s.detail + "' failed: " + pmlb_last_error());
  }
}

// Records the kernel sequence once (one graph per segment); the same launches, replayed by the driver without the
// per-launch host work (tensor-map encoding, attribute calls, argument marshalling).  Any
// failure leaves the executable on direct launches.
void Executable::captureGraph() {
  graphState_ = 2;
  std::vector<cudaGraphExec_t> made;
  for (size_t k = 0; k < segStart_.size(); ++k) {
    const size_t first = segStart_[k], last = k + 1 < segStart_.size() ? segStart_[k + 1] : steps_.size();
    bool ok = cudaStreamBeginCapture(stream_, cudaStreamCaptureModeThreadLocal) == cudaSuccess;
    cudaGraph_t g = nullptr;
    if (ok) {
      for (size_t i = first; i < last && ok; ++i) ok = steps_[i].launch(stream_) == PMLB_OK;
      ok = (cudaStreamEndCapture(stream_, &g) == cudaSuccess) && ok && g != nullptr;
    }
    cudaGraphExec_t exec = nullptr;
    if (ok) ok = cudaGraphInstantiate(&exec, g, 0) == cudaSuccess && exec != nullptr;
    if (g) cudaGraphDestroy(g);
    if (!ok) {
      for (cudaGraphExec_t e : made) cudaGraphExecDestroy(e);
      cudaGetLastError();
      return;
    }
    made.push_back(exec);
  }
  graphs_ = std::move(made);
  graphState_ = 1;
}

void Executable::enqueueSteps(const std::vector<cudaEvent_t>* waits) {
  ++passes_;
  if (graphState_ == 0 && passes_ >= 2) {
    const bool wanted = steps_.size() >= 2 && Settings::instance().getOr("PLAIDML_CUDA_GRAPH", "1") != "0";
    if (wanted) {
      captureGraph();
    } else {
      graphState_ = 2;
    }
  }
  for (size_t k = 0; k < segStart_.size(); ++k) {
    if (waits) cudaCheck(cudaStreamWaitEvent(stream_, (*waits)[k], 0), "cudaStreamWaitEvent");
    if (graphState_ == 1) {
      cudaCheck(cudaGraphLaunch(graphs_[k], stream_), "cudaGraphLaunch");
    } else {
      launchStepsDirect(segStart_[k], k + 1 < segStart_.size() ? segStart_[k + 1] : steps_.size());
    }
  }
}

// Decides once whether a run's uploads overlap its kernels.  An input is needed by the first step whose program
// position is not before the first operation that uses it (looking through reshapes): a step reads an input only
// through an operation fused into it, and a step's position is that of its last fused operation, so in the
// position-ordered step list no step before that one can read it.  Inputs are grouped in order of need until a
// group holds a few megabytes; a group's first step starts a segment.
void Executable::planUploadOverlap() {
  overlapState_ = 2;
  if (Settings::instance().getOr("PLAIDML_CUDA_UPLOAD_OVERLAP", "1") == "0") return;
  if (ShardComm::instance().world() > 1 || prog_->inputs.size() < 2 || steps_.size() < 2) return;
  const size_t nv = prog_->values.size();
  std::vector<int> root(nv);
  for (size_t v = 0; v < nv; ++v) root[v] = static_cast<int>(v);
  for (const POp& op : prog_->ops) {     // (operations are in definition order: an operand's root is final here)
    if (op.kind == POp::Reshape && op.result >= 0) root[op.result] = root[op.operands[0]];
  }
  std::vector<int> firstOp(nv, -1);
  for (size_t j = 0; j < prog_->ops.size(); ++j) {
    const POp& op = prog_->ops[j];
    if (op.kind == POp::Reshape) continue;
    for (int o : op.operands) {
      if (firstOp[root[o]] < 0) firstOp[root[o]] = static_cast<int>(j);
    }
  }
  struct Need {
    size_t step, input, bytes;
  };
  std::vector<Need> needs;
  size_t total = 0;
  for (size_t i = 0; i < prog_->inputs.size(); ++i) {
    const int id = prog_->inputs[i];
    size_t step = 0;   // an input no operation uses (or that is itself an output) travels with the first group
    const bool isOutput = std::find(prog_->outputs.begin(), prog_->outputs.end(), id) != prog_->outputs.end();
    if (firstOp[id] >= 0 && !isOutput) {
      while (step < steps_.size() && steps_[step].position < firstOp[id]) ++step;
      if (step == steps_.size()) step = 0;
    }
    const size_t bytes = inputUsed_[i] ? prog_->values[id].shape.byteSize() : 0;
    needs.push_back({step, i, bytes});
    total += bytes;
  }
  for (size_t i = 0; i < steps_.size(); ++i) {
    // (a step without a position, or a list that is not in position order: stay on the plain path)
    if (steps_[i].position < 0 || (i > 0 && steps_[i].position < steps_[i - 1].position)) return;
  }
  std::stable_sort(needs.begin(), needs.end(), [](const Need& a, const Need& b) { return a.step < b.step; });
  const size_t quantum = std::max<size_t>(size_t{4} << 20, total / 12);
  std::vector<size_t> starts{0};
  std::vector<std::vector<size_t>> groups(1);
  size_t inGroup = 0;
  for (const Need& n : needs) {
    if (inGroup >= quantum && n.step > starts.back()) {
      starts.push_back(n.step);
      groups.emplace_back();
      inGroup = 0;
    }
    groups.back().push_back(n.input);
    inGroup += n.bytes;
  }
  if (groups.size() < 2) return;
  if (cudaStreamCreateWithFlags(&uploadStream_, cudaStreamNonBlocking) != cudaSuccess) {
    cudaGetLastError();
    uploadStream_ = nullptr;
    return;
  }
  for (size_t k = 0; k < groups.size(); ++k) {
    cudaEvent_t ev = nullptr;
    if (cudaEventCreateWithFlags(&ev, cudaEventDisableTiming) != cudaSuccess) {
      cudaGetLastError();
      return;
    }
    groupReady_.push_back(ev);
  }
  segStart_ = std::move(starts);
  inputGroup_ = std::move(groups);
  overlapState_ = 1;
}

void Executable::checkStatus() {
  int code = 0;
  cudaCheck(cudaMemcpyAsync(&code, status_, sizeof(int), cudaMemcpyDeviceToHost, stream_), "status readback");
  cudaCheck(cudaStreamSynchronize(stream_), "run");
  if (code != 0) {
    cudaMemset(status_, 0, sizeof(int));
    throw std::runtime_error("A device-side pipeline wait gave up (role code " + std::to_string(code) + ")");
  }
}

double Executable::run(const std::vector<BufferPtr>& inputs, const std::vector<BufferPtr>& outputs) {
  // argument checks of plaidml_executable_run (plaidml/exec/ffi.cc:92-120)
  if (inputs.size() != prog_->inputs.size()) {
    throw std::runtime_error("Program expects " + std::to_string(prog_->inputs.size()) + " inputs, but " +
                             std::to_string(inputs.size()) + " were specified");
  }
  if (outputs.size() != prog_->outputs.size()) {
    throw std::runtime_error("Program expects " + std::to_string(prog_->outputs.size()) + " outputs, but " +
                             std::to_string(outputs.size()) + " were specified");
  }
  for (size_t i = 0; i < inputs.size(); ++i) {
    const TensorShape& want = prog_->values[prog_->inputs[i]].shape;
    if (inputs[i]->shape() != want) {
      throw std::runtime_error("Shape mismatch for input buffer " + std::to_string(i) + ", expected '" + want.str() +
                               "' but '" + inputs[i]->shape().str() + "' was specified");
    }
  }
  for (size_t i = 0; i < outputs.size(); ++i) {
    const TensorShape& want = prog_->values[prog_->outputs[i]].shape;
    if (outputs[i]->shape() != want) {
      throw std::runtime_error("Shape mismatch for output buffer " + std::to_string(i) + ", expected '" + want.str() +
                               "' but '" + outputs[i]->shape().str() + "' was specified");
    }
  }
  cudaCheck(cudaSetDevice(device_), "cudaSetDevice");
  if (slicedState_ == 0) slicedState_ = prepareSlicedRun() ? 1 : 2;
  if (slicedState_ == 1) return runSliced(inputs, outputs);
  const auto t0 = std::chrono::steady_clock::now();
  if (overlapState_ == 0) planUploadOverlap();   // (before the graph is captured: it fixes the segments)
  if (overlapState_ == 1) {
    for (size_t k = 0; k < inputGroup_.size(); ++k) {
      for (size_t i : inputGroup_[k]) {
        const int id = prog_->inputs[i];
        const size_t bytes = prog_->values[id].shape.byteSize();
        if (bytes && inputUsed_[i]) {
          cudaCheck(cudaMemcpyAsync(dev_[id], inputs[i]->data(), bytes, cudaMemcpyHostToDevice, uploadStream_), "input upload");
        }
      }
      cudaCheck(cudaEventRecord(groupReady_[k], uploadStream_), "cudaEventRecord");
    }
    inputsResident_ = true;
    enqueueSteps(&groupReady_);
  } else {
    for (size_t i = 0; i < inputs.size(); ++i) {
      if (inputUsed_[i]) uploadInput(i, inputs[i]);
    }
    inputsResident_ = true;
    enqueueSteps();
  }
  for (size_t i = 0; i < outputs.size(); ++i) {
    const int id = prog_->outputs[i];
    const size_t bytes = prog_->values[id].shape.byteSize();
    if (bytes) {
      cudaCheck(cudaMemcpyAsync(outputs[i]->data(), dev_[id], bytes, cudaMemcpyDeviceToHost, stream_), "output download");
    }
  }
  checkStatus();
  const auto t1 = std::chrono::steady_clock::now();
  return std::chrono::duration<double, std::milli>(t1 - t0).count();
}

// Host -> device copy of one program input on the executable's stream.  In the sharded mode a
// replicated input travels as this rank's slice only; the all-gather behind it fills in the rest.
void Executable::uploadInput(size_t i, const BufferPtr& buf) {
  const int id = prog_->inputs[i];
  const size_t bytes = prog_->values[id].shape.byteSize();
  if (!bytes) return;
  ShardComm& comm = ShardComm::instance();
  const size_t world = static_cast<size_t>(comm.world());
  // (slices of whole 16-byte units keep every rank's part aligned for the collective)
  if (world > 1 && i < replicated_.size() && replicated_[i] && bytes % (16 * world) == 0) {
    const size_t part = bytes / world;
    const size_t off = part * static_cast<size_t>(comm.rank());
    cudaCheck(cudaMemcpyAsync(dev_[id] + off, static_cast<const char*>(buf->data()) + off, part, cudaMemcpyHostToDevice,
                              stream_), "input upload");
    comm.allGatherBytes(dev_[id] + off, dev_[id], part, stream_);
    return;
  }
  cudaCheck(cudaMemcpyAsync(dev_[id], buf->data(), bytes, cudaMemcpyHostToDevice, stream_), "input upload");
}

void Executable::setInputReplicated(size_t index, bool on) {
  if (index >= prog_->inputs.size()) throw std::runtime_error("No such input");
  if (replicated_.size() < prog_->inputs.size()) replicated_.assign(prog_->inputs.size(), false);
  replicated_[index] = on;
}

void* Executable::gatherOutput(size_t index, size_t* nbytes, size_t iters, double* meanMs) {
  if (index >= prog_->outputs.size()) throw std::runtime_error("No such output");
  cudaCheck(cudaSetDevice(device_), "cudaSetDevice");
  ShardComm& comm = ShardComm::instance();
  const int id = prog_->outputs[index];
  const size_t bytes = prog_->values[id].shape.byteSize();
  const size_t total = bytes * static_cast<size_t>(comm.world());
  if (gatheredBytes_ < total) {
    cudaCheck(cudaStreamSynchronize(stream_), "gather");
    if (gathered_) cudaFree(gathered_);
    gathered_ = nullptr;
    gatheredBytes_ = 0;
    cudaCheck(cudaMalloc(reinterpret_cast<void**>(&gathered_), total ? total : 256), "cudaMalloc(gathered output)");
    gatheredBytes_ = total;
  }
  if (iters == 0) iters = 1;
  cudaCheck(cudaEventRecord(evStart_, stream_), "cudaEventRecord");
  for (size_t i = 0; i < iters; ++i) comm.allGatherBytes(dev_[id], gathered_, bytes, stream_);
  cudaCheck(cudaEventRecord(evStop_, stream_), "cudaEventRecord");
  cudaCheck(cudaStreamSynchronize(stream_), "gather");
  if (meanMs) {
    float ms = 0.f;
    cudaCheck(cudaEventElapsedTime(&ms, evStart_, evStop_), "cudaEventElapsedTime");
    *meanMs = static_cast<double>(ms) / static_cast<double>(iters);
  }
  if (nbytes) *nbytes = total;
  return gathered_;
}

// A program that is one large GEMM from a host input to a host output is bound by the host link,
// not by the kernel.  Its rows are then processed in four slices: while slice i's rows of C travel
// device -> host on a second stream, slice i + 1's rows of A travel host -> device, so the two
// directions of the link overlap instead of taking turns.  When B comes from the host as well, the
// first row slice is further cut into four column blocks, each computed as soon as its quarter of
// B has arrived: the download (the longer direction) then starts after a quarter of A and a quarter
// of B instead of after a quarter of A and all of B.  Same kernels, same results.
bool Executable::prepareSlicedRun() {
  constexpr int kSlices = 4;
  if (steps_.size() != 1 || !steps_[0].rowSliceable || prog_->outputs.size() != 1) return false;
  if (Settings::instance().getOr("PLAIDML_CUDA_SLICED_RUN", "1") == "0") return false;
  const Step& st = steps_[0];
  const pmlb_gemm_desc& d = st.gemm;
  const size_t outBytes = prog_->values[prog_->outputs[0]].shape.byteSize();
  if (d.m % (kSlices * 256) != 0 || outBytes < (16u << 20)) return false;
  for (int i = 0; i < kSlices; ++i) {
    pmlb_gemm_desc sd = d;
    sd.m = d.m / kSlices;
    pmlb_plan* plan = nullptr;
    if (pmlb_gemm_dispatch(&sd, &plan) != PMLB_OK || pmlb_plan_share_status(plan, status_) != PMLB_OK) {
      if (plan) pmlb_plan_free(plan);
      for (pmlb_plan* q : slicePlans_) pmlb_plan_free(q);
      slicePlans_.clear();
      return false;
    }
    slicePlans_.push_back(plan);
  }
  // column blocks of the first slice, if B is a program input
  for (size_t i = 0; i < prog_->inputs.size(); ++i) {
    if (static_cast<int>(i) != st.aInput && dev_[prog_->inputs[i]] == st.bPtr) bInput_ = static_cast<int>(i);
  }
  if (bInput_ >= 0 && d.n % (kSlices * 256) == 0 && d.ldc == d.n && d.ldb == (d.b_is_nk ? d.k : d.n)) {
    for (int j = 0; j < kSlices; ++j) {
      pmlb_gemm_desc bd = d;
      bd.m = d.m / kSlices;
      bd.n = d.n / kSlices;
      pmlb_plan* plan = nullptr;
      if (pmlb_gemm_dispatch(&bd, &plan) != PMLB_OK || pmlb_plan_share_status(plan, status_) != PMLB_OK) {
        if (plan) pmlb_plan_free(plan);
        for (pmlb_plan* q : blockPlans_) pmlb_plan_free(q);
        blockPlans_.clear();
        break;
      }
      blockPlans_.push_back(plan);
    }
  }
  if (blockPlans_.empty()) bInput_ = -1;
  if (cudaStreamCreateWithFlags(&copyStream_, cudaStreamNonBlocking) != cudaSuccess) return false;
  for (int i = 0; i < 2 * kSlices; ++i) {
    cudaEvent_t ev = nullptr;
    if (cudaEventCreateWithFlags(&ev, cudaEventDisableTiming) != cudaSuccess) return false;
    sliceDone_.push_back(ev);
  }
  return true;
}

double Executable::runSliced(const std::vector<BufferPtr>& inputs, const std::vector<BufferPtr>& outputs) {
  const Step& st = steps_[0];
  const pmlb_gemm_desc& d = st.gemm;
  const int slices = static_cast<int>(slicePlans_.size());
  const auto t0 = std::chrono::steady_clock::now();
  // (a replicated B arrives by slice upload + all-gather, as a whole, before the first block)
  const bool bGathered = bInput_ >= 0 && ShardComm::instance().world() > 1 &&
                         static_cast<size_t>(bInput_) < replicated_.size() && replicated_[bInput_];
  const int bInput = bGathered ? -1 : bInput_;
  for (size_t i = 0; i < inputs.size(); ++i) {
    if (static_cast<int>(i) == st.aInput || static_cast<int>(i) == bInput) continue;
    uploadInput(i, inputs[i]);
  }
  const int aId = prog_->inputs[st.aInput], cId = prog_->outputs[st.cOutput];
  const size_t aBytes = prog_->values[aId].shape.byteSize() / slices;
  const size_t cBytes = prog_->values[cId].shape.byteSize() / slices;
  int first = 0;
  if (bInput >= 0) {
    // first row slice by column blocks: A's rows, then a quarter of B at a time
    const int blocks = static_cast<int>(blockPlans_.size());
    const int bId = prog_->inputs[bInput];
    const size_t eb = prog_->values[bId].shape.byteSize() / (static_cast<size_t>(d.n) * d.k);
    const size_t ob = prog_->values[cId].shape.byteSize() / (static_cast<size_t>(d.m) * d.n);
    const size_t nb = static_cast<size_t>(d.n) / blocks;          // columns per block
    const char* bHost = static_cast<const char*>(inputs[bInput]->data());
    char* cHost = static_cast<char*>(outputs[st.cOutput]->data());
    cudaCheck(cudaMemcpyAsync(dev_[aId], inputs[st.aInput]->data(), aBytes, cudaMemcpyHostToDevice, stream_), "input upload");
    for (int j = 0; j < blocks; ++j) {
      size_t bOff;
      if (d.b_is_nk) {   // B stored [n][k]: a block of columns is a run of whole rows
        bOff = nb * j * d.k * eb;
        cudaCheck(cudaMemcpyAsync(dev_[bId] + bOff, bHost + bOff, nb * d.k * eb, cudaMemcpyHostToDevice, stream_), "input upload");
      } else {           // B stored [k][n]: a block of columns is a pitched rectangle
        bOff = nb * j * eb;
        cudaCheck(cudaMemcpy2DAsync(dev_[bId] + bOff, d.n * eb, bHost + bOff, d.n * eb, nb * eb, d.k,
                                    cudaMemcpyHostToDevice, stream_), "input upload");
      }
      char* cDev = dev_[cId] + nb * j * ob;
      const void* bias = st.biasPtr ? static_cast<const char*>(st.biasPtr) + nb * j * 4 : nullptr;
      const pmlb_status rc = pmlb_gemm_invoke(blockPlans_[j], stream_, dev_[aId], dev_[bId] + bOff, cDev, bias, nullptr, nullptr);
      if (rc != PMLB_OK) throw std::runtime_error("Kernel step '" + st.kernel + " " + st.detail + "' failed: " + pmlb_last_error());
      cudaEvent_t ev = sliceDone_[slices + j];
      cudaCheck(cudaEventRecord(ev, stream_), "cudaEventRecord");
      cudaCheck(cudaStreamWaitEvent(copyStream_, ev, 0), "cudaStreamWaitEvent");
      cudaCheck(cudaMemcpy2DAsync(cHost + nb * j * ob, d.n * ob, cDev, d.n * ob, nb * ob, d.m / slices,
                                  cudaMemcpyDeviceToHost, copyStream_), "output download");
    }
    first = 1;
  }
  for (int i = first; i < slices; ++i) {
    char* aDev = dev_[aId] + aBytes * i;
    char* cDev = dev_[cId] + cBytes * i;
    cudaCheck(cudaMemcpyAsync(aDev, static_cast<const char*>(inputs[st.aInput]->data()) + aBytes * i, aBytes,
                              cudaMemcpyHostToDevice, stream_), "input upload");
    const pmlb_status rc = pmlb_gemm_invoke(slicePlans_[i], stream_, aDev, st.bPtr, cDev, st.biasPtr, nullptr, nullptr);
    if (rc != PMLB_OK) throw std::runtime_error("Kernel step '" + st.kernel + " " + st.detail + "' failed: " + pmlb_last_error());
    cudaCheck(cudaEventRecord(sliceDone_[i], stream_), "cudaEventRecord");
    cudaCheck(cudaStreamWaitEvent(copyStream_, sliceDone_[i], 0), "cudaStreamWaitEvent");
    cudaCheck(cudaMemcpyAsync(static_cast<char*>(outputs[st.cOutput]->data()) + cBytes * i, cDev, cBytes,
                              cudaMemcpyDeviceToHost, copyStream_), "output download");
  }
  inputsResident_ = true;
  cudaCheck(cudaStreamSynchronize(copyStream_), "run");
  checkStatus();
  const auto t1 = std::chrono::steady_clock::now();
  return std::chrono::duration<double, std::milli>(t1 - t0).count();
}

double Executable::runResident(size_t iters) {
  if (!inputsResident_) throw std::runtime_error("run the executable once before re-running it on resident inputs");
  if (iters == 0) return 0.0;
  cudaCheck(cudaSetDevice(device_), "cudaSetDevice");
  cudaCheck(cudaEventRecord(evStart_, stream_), "cudaEventRecord");
  for (size_t i = 0; i < iters; ++i) enqueueSteps();
  cudaCheck(cudaEventRecord(evStop_, stream_), "cudaEventRecord");
  checkStatus();
  float ms = 0.f;
  cudaCheck(cudaEventElapsedTime(&ms, evStart_, evStop_), "cudaEventElapsedTime");
  return static_cast<double>(ms) / static_cast<double>(iters);
}

double Executable::timeSteps(size_t iters, bool flushL2, double* perPassMs) {
  if (!inputsResident_) throw std::runtime_error("run the executable once before timing it on resident inputs");
  if (iters == 0) return 0.0;
  cudaCheck(cudaSetDevice(device_), "cudaSetDevice");
  constexpr size_t kFlushBytes = 256u << 20;  // twice the 126 MB L2
  if (flushL2 && !flush_) cudaCheck(cudaMalloc(reinterpret_cast<void**>(&flush_), kFlushBytes), "cudaMalloc(L2 flush)");
  // Up to 64 passes are enqueued before the host waits, each between its own event pair: the stream then
  // always holds work ahead of the device, so a pass's interval never includes time the host took to
  // submit it (a descheduled host thread would otherwise show up as a slow pass).
  constexpr size_t kBatch = 64;
  const size_t pairs = std::min(iters, kBatch);
  while (timingEvents_.size() < 2 * pairs) {
    cudaEvent_t ev = nullptr;
    cudaCheck(cudaEventCreate(&ev), "cudaEventCreate");
    timingEvents_.push_back(ev);
  }
  double total = 0.0;
  for (size_t done = 0; done < iters; done += kBatch) {
    const size_t n = std::min(kBatch, iters - done);
    for (size_t i = 0; i < n; ++i) {
      if (flushL2) {
        cudaCheck(cudaMemsetAsync(flush_, static_cast<int>((done + i) & 0xff), kFlushBytes, stream_), "L2 flush");
      }
      cudaCheck(cudaEventRecord(timingEvents_[2 * i], stream_), "cudaEventRecord");
      enqueueSteps();
      cudaCheck(cudaEventRecord(timingEvents_[2 * i + 1], stream_), "cudaEventRecord");
    }
    cudaCheck(cudaEventSynchronize(timingEvents_[2 * n - 1]), "cudaEventSynchronize");
    for (size_t i = 0; i < n; ++i) {
      float ms = 0.f;
      cudaCheck(cudaEventElapsedTime(&ms, timingEvents_[2 * i], timingEvents_[2 * i + 1]), "cudaEventElapsedTime");
      total += ms;
      if (perPassMs) perPassMs[done + i] = ms;
    }
  }
  checkStatus();
  return total / static_cast<double>(iters);
}

void Executable::timeEachStep(size_t iters, bool flushL2, double* out) {
  if (!inputsResident_) throw std::runtime_error("run the executable once before timing it on resident inputs");
  if (iters == 0) iters = 1;
  cudaCheck(cudaSetDevice(device_), "cudaSetDevice");
  constexpr size_t kFlushBytes = 256u << 20;
  if (flushL2 && !flush_) cudaCheck(cudaMalloc(reinterpret_cast<void**>(&flush_), kFlushBytes), "cudaMalloc(L2 flush)");
  // Each step is captured `iters` times back to back into a CUDA graph of its own, which is launched once
  // untimed and once between an event pair: the host cost of a launch (tensor-map encoding, attribute
  // calls), which exceeds the run time of a small kernel, stays out of the measurement, as it does when
  // the whole program replays as a graph.
  for (size_t k = 0; k < steps_.size(); ++k) {
    cudaCheck(cudaStreamBeginCapture(stream_, cudaStreamCaptureModeThreadLocal), "cudaStreamBeginCapture");
    pmlb_status rc = PMLB_OK;
    for (size_t it = 0; it < iters && rc == PMLB_OK; ++it) rc = steps_[k].launch(stream_);
    cudaGraph_t g = nullptr;
    const cudaError_t endErr = cudaStreamEndCapture(stream_, &g);
    if (rc != PMLB_OK || endErr != cudaSuccess || g == nullptr) {
      if (g) cudaGraphDestroy(g);
      cudaGetLastError();
      throw std::runtime_error("Kernel step '" + steps_[k].kernel + "' could not be captured: " + pmlb_last_error());
    }
    cudaGraphExec_t exec = nullptr;
    if (cudaGraphInstantiate(&exec, g, 0) != cudaSuccess || exec == nullptr) {
      cudaGraphDestroy(g);
      cudaGetLastError();
      throw std::runtime_error("cudaGraphInstantiate failed for a kernel step");
    }
    cudaCheck(cudaGraphLaunch(exec, stream_), "cudaGraphLaunch");
    if (flushL2) cudaCheck(cudaMemsetAsync(flush_, static_cast<int>(k & 0xff), kFlushBytes, stream_), "L2 flush");
    cudaCheck(cudaEventRecord(evStart_, stream_), "cudaEventRecord");
    cudaCheck(cudaGraphLaunch(exec, stream_), "cudaGraphLaunch");
    cudaCheck(cudaEventRecord(evStop_, stream_), "cudaEventRecord");
    cudaCheck(cudaEventSynchronize(evStop_), "cudaEventSynchronize");
    float ms = 0.f;
    cudaCheck(cudaEventElapsedTime(&ms, evStart_, evStop_), "cudaEventElapsedTime");
    out[k] = ms;
    cudaGraphExecDestroy(exec);
    cudaGraphDestroy(g);
  }
  for (size_t k = 0; k < steps_.size(); ++k) out[k] /= static_cast<double>(iters);
  checkStatus();
}

std::string Executable::describe() const {
  std::ostringstream os;
  for (const Step& s : steps_) os << s.kernel << " " << s.detail << "\n";
  return os.str();
}

size_t Executable::launchCount() const {
  size_t n = 0;
  for (const Step& s : steps_) n += static_cast<size_t>(s.launches);
  return n;
}

void* Executable::outputDevicePtr(size_t index, size_t* nbytes) const {
  if (index >= prog_->outputs.size()) throw std::runtime_error("No such output");
  const int id = prog_->outputs[index];
  if (nbytes) *nbytes = prog_->values[id].shape.byteSize();
  return dev_[id];
}

// ==================================================================== devices / targets

std::vector<std::string> listDevices() {
  std::vector<std::string> out;
  int count = 0;
  if (cudaGetDeviceCount(&count) != cudaSuccess) {
    cudaGetLastError();
    return out;
  }
  for (int d = 0; d < count; ++d) {
    int major = 0;
    cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, d);
    if (major == 10) out.push_back("cuda." + std::to_string(d));
  }
  return out;
}

int parseDeviceId(const std::string& id) {
  static const std::regex re("([a-zA-Z0-9_]+(?:-[a-zA-Z0-9_]+)*)\\.([0-9]+)");
  std::smatch m;
  if (!std::regex_match(id, m, re)) throw std::runtime_error("Invalid device id: '" + id + "'");
  if (m[1].str() != "cuda") throw std::runtime_error("Unknown runtime '" + m[1].str() + "': the only device family is 'cuda'");
  return std::stoi(m[2].str());
}

std::vector<std::string> listTargets() { return {"cuda"}; }

}  // namespace pml
