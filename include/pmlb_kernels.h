/*
 * pmlb_kernels.h -- C ABI of the sm_100a kernel library behind the PlaidML `cuda` device.
 *
 * This is the layer the reference fills with libxsmm: JIT-compiled x86 code calls
 * `plaidml_rt_xsmm_*_dispatch_f32` once per tile shape and `*_invoke_f32` per tile
 * (pmlc/rt/xsmm.cc:17-56, 235-342, 457-856).  Here a *dispatch* builds a plan for a whole
 * contraction (tile shape, instruction descriptor, scratch size) and an *invoke* enqueues
 * the kernels of that plan on a CUDA stream.  Plain pointers and sizes only; every
 * pointer passed to an invoke is a device pointer unless stated otherwise.
 *
 * Conventions
 *   - every function returns a pmlb_status; pmlb_last_error() gives the message of the
 *     last failure on the calling thread;
 *   - no entry point falls back to the CPU: without a usable sm_100 device the dispatch
 *     functions fail with PMLB_ERR_UNSUPPORTED;
 *   - dispatch functions may allocate device scratch (released by pmlb_plan_free);
 *     invoke functions never allocate and never synchronise.
 */
#ifndef PMLB_KERNELS_H_
#define PMLB_KERNELS_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef enum {
  PMLB_OK = 0,
  PMLB_ERR_INVALID = 1,     /* bad argument */
  PMLB_ERR_CUDA = 2,        /* a CUDA call failed */
  PMLB_ERR_UNSUPPORTED = 3, /* shape / type outside what the kernel covers */
  PMLB_ERR_TIMEOUT = 4      /* a device-side wait gave up; see pmlb_plan_check */
} pmlb_status;

/* Element types.  Values equal plaidml_datatype (plaidml/core/ffi.h:139-156) so that a
 * TensorShape's dtype can be passed through unchanged; BFLOAT16 is appended. */
typedef enum {
  PMLB_BOOL = 4,
  PMLB_I8 = 5,
  PMLB_U8 = 6,
  PMLB_I16 = 7,
  PMLB_U16 = 8,
  PMLB_I32 = 9,
  PMLB_U32 = 10,
  PMLB_I64 = 11,
  PMLB_U64 = 12,
  PMLB_F16 = 13,
  PMLB_F32 = 14,
  PMLB_F64 = 15,
  PMLB_BF16 = 16
} pmlb_dtype;

/* Aggregations and combinations of a Tile contraction; values equal plaidml_agg_op /
 * plaidml_combo_op (plaidml/edsl/ffi.h:218-233). */
typedef enum { PMLB_AGG_NONE = 0, PMLB_AGG_SUM, PMLB_AGG_MAX, PMLB_AGG_MIN, PMLB_AGG_PROD, PMLB_AGG_ASSIGN } pmlb_agg;
typedef enum { PMLB_COMBO_NONE = 0, PMLB_COMBO_MUL, PMLB_COMBO_ADD, PMLB_COMBO_EQ, PMLB_COMBO_COND } pmlb_combo;

/* Epilogue steps fused into the GEMM / convolution kernels; the role of the reference's
 * `_bias`, `_relu` and `_relu_beta1` microkernel variants (pmlc/rt/xsmm.cc:58-233). */
enum {
  PMLB_EPI_BIAS = 1,     /* out[.., j] += bias[j]; bias is f32 (float paths) or i32 (int8 path) */
  PMLB_EPI_RESIDUAL = 2, /* out += residual (same shape and element type as out) */
  PMLB_EPI_RELU = 4,     /* x < 0 ? 0 : x, as pmlc/conversion/pxa_to_affine/pxa_to_affine.cc:312-332 */
  PMLB_EPI_ROWMAX = 8    /* additionally reduce each output row with max into `rowmax` (f32);
                            not combinable with the other steps */
};

const char* pmlb_last_error(void);
const char* pmlb_version(void);

/* Number of CUDA devices with compute capability 10.x; 0 when there is none. */
int pmlb_device_count(void);

/* Debugging aid: while `device_buffer` (4 * 2048 * 3 int64, zero-filled by the caller) is
 * set, CTA 0 of every tensor-core launch logs {tile, event, clock64} records of its producer,
 * MMA and epilogue warps to it.  NULL (the default) turns logging off.  The records exist only
 * in a library built with -DPMLB_TC_TRACE (they slow the kernel's roles by several per cent even
 * when unused); otherwise the call is accepted and nothing is logged. */
void pmlb_debug_set_trace(void* device_buffer);

typedef struct pmlb_plan pmlb_plan;

void pmlb_plan_free(pmlb_plan* plan);

/* Device scratch the plan holds, in bytes (0 when its kernels need none). */
size_t pmlb_plan_scratch_bytes(const pmlb_plan* plan);

/* Synchronises `stream` and reports whether any kernel of the plan recorded a device-side
 * error since the last check (a bounded wait that expired): PMLB_OK or PMLB_ERR_TIMEOUT. */
pmlb_status pmlb_plan_check(pmlb_plan* plan, void* stream);

/* Makes the plan record device-side errors in `device_word` (an int in device memory owned by
 * the caller, zero-initialised) instead of its own word, so that one readback covers many
 * plans.  pmlb_plan_check then reads that word. */
pmlb_status pmlb_plan_share_status(pmlb_plan* plan, int* device_word);

/* Name of the kernel family a plan resolved to ("tc_gemm", "tc_conv", "row_reduce", ...). */
const char* pmlb_plan_kind(const pmlb_plan* plan);
/* Parts the K range of a GEMM plan is split into (1 = a single pass). */
int pmlb_plan_split_k(const pmlb_plan* plan);
/* Test hook for the bounded waits of the tensor-core kernel (no counterpart in the reference).  Every
 * device-side wait (on an operand stage, an accumulator, a residual row) gives up after a wall-clock limit,
 * normally two seconds; the CTA then raises an abort flag, all its roles leave their loops, it waits a
 * bounded time for copies still in flight, frees its TMEM, writes a role code to the plan's status word and
 * returns -- the launch ends, the context stays usable, and pmlb_plan_check reports PMLB_ERR_TIMEOUT.
 * This call arms the NEXT pmlb_gemm_invoke of a single-pass 8/16-bit GEMM plan so that exactly this
 * happens: the first CTA's producer never issues its first operand load (nothing is in flight for that
 * stage, nothing faults) and waits give up after `wait_limit_ms` (1..100).  The launch after it is normal. */
pmlb_status pmlb_plan_arm_timeout_test(pmlb_plan* plan, int wait_limit_ms);

/* ---------------------------------------------------------------- GEMM
 * C[b, i, j] = sum_k A[b, i, k] * B[b, k, j]   (b_is_nk == 0, B stored [k][n])
 * C[b, i, j] = sum_k A[b, i, k] * B[b, j, k]   (b_is_nk == 1, B stored [n][k])
 * Replaces plaidml_rt_xsmm_gemm/brgemm_{dispatch,invoke}_f32 (pmlc/rt/xsmm.cc:17-56,235-287)
 * and, for int8 / 16-bit inputs, the plain LLVM loops the x86 target emits for
 * non-f32 contractions (pmlc/target/x86/pipeline.cc:185-202).
 *
 * in_dtype / out_dtype:  F32 -> F32 (three TF32 products per term, f32 accumulate)
 *                        BF16 or F16 -> F32, BF16 or F16 (f32 accumulate)
 *                        I8 -> I32, or I8 (two's-complement wrap of the 32-bit sum)
 * A batch stride of 0 shares one matrix between all batch entries.
 */
typedef struct {
  int32_t in_dtype;
  int32_t out_dtype;
  int32_t m, n, k, batch;
  int64_t lda, ldb, ldc;             /* elements between rows */
  int64_t stride_a, stride_b, stride_c; /* elements between batch entries */
  int32_t b_is_nk;
  int32_t epilogue;                  /* PMLB_EPI_* */
  int64_t ldr, stride_r;             /* residual row / batch strides (elements) */
  int32_t tile_n;                    /* 0 = choose; 64, 128 or 256 forces the tile width */
  int32_t flags;                     /* PMLB_GEMM_* */
  /* A in two parts (0 = off): columns [0, k_first) of A come from `a`, columns [k_first, k) from a second
   * matrix `a2` (its own column 0 first, rows lda2 elements apart), both with m rows; B and k describe the
   * whole product.  C = [A1 | A2] * B is the sum of two GEMMs in one accumulator, which is how a residual
   * block's shortcut projection joins its last convolution (C = A1 * W1 + A2 * W2 + (b1 + b2)) without the
   * projection's output ever being written or read back.  8/16-bit inputs, batch 1, k_first a multiple of
   * the 128-byte k-block; run with pmlb_gemm_invoke_two.  No counterpart in the reference. */
  int32_t k_first;
  int32_t a2_stride;                 /* 0: the second part is a matrix (rows lda2 apart); s >= 1: it is an NHWC
                                      * activation [a2_n][a2_h][a2_w][k - k_first] and row i of the product is its
                                      * pixel (i / (P Q), s * (i / Q % P), s * (i % Q)), P = ceil(a2_h / s),
                                      * Q = ceil(a2_w / s), m = a2_n * P * Q: a strided 1x1 convolution's view of it
                                      * (the shortcut projection of a block that halves the resolution) */
  int64_t lda2;
  int32_t a2_n, a2_h, a2_w, reserved0;
} pmlb_gemm_desc;

/* With b_is_nk == 0 the 16-bit and 8-bit kernels read B tiles straight from the [k][n]
 * matrix (an "MN-major" tensor-core operand).  This flag makes the plan transpose B into
 * [n][k] scratch first and run the K-major kernel instead. */
#define PMLB_GEMM_TRANSPOSE_B 1
/* Take the epilogue that serves outputs whose rows are not 16-byte aligned even when the
 * staged TMA-store epilogue would apply (for testing that path). */
#define PMLB_GEMM_PLAIN_STORES 2
/* Keep the staged epilogue but read the residual with ordinary loads instead of fetching its
 * rows by TMA ahead of each chunk (for testing that both routes round identically). */
#define PMLB_GEMM_PLAIN_RESIDUAL 4
/* Large 8/16-bit GEMMs run two CTAs per 256 x 256 tile (a cluster of two with paired MMAs) when
 * that fills the device; these flags force the choice for 256-wide tiles (for testing). */
#define PMLB_GEMM_CTA_PAIRS 8
#define PMLB_GEMM_NO_CTA_PAIRS 16
/* When the tiles left over after the last full wave occupy at most half of the SMs, 256-wide
 * tiles of that tail are computed as two 128-wide halves; this flag keeps them whole (testing). */
#define PMLB_GEMM_NO_TAIL_SPLIT 32
/* Few output tiles and a long K (fewer tiles than half the SMs, eight k-blocks or more, batch 1): the K
 * range is split over 2..8 CTAs per tile as a batch of partial products into plan scratch (f32 / i32),
 * and a second small kernel sums the parts in order and applies bias / residual / ReLU / cast.  The
 * result does not depend on timing (no atomics), but the order of the f32 additions differs from the
 * single pass, so a problem that is split at one size and not at another (the tile count decides) can
 * differ in the last bits between the two.  NO_SPLIT_K keeps one pass; SPLIT_K splits whenever the
 * k-blocks divide evenly, whatever the tile count (for testing); PMLB_SPLIT_K=0 in the environment turns
 * the library's own choice off for a whole process. */
#define PMLB_GEMM_NO_SPLIT_K 64
#define PMLB_GEMM_SPLIT_K 128

pmlb_status pmlb_gemm_dispatch(const pmlb_gemm_desc* desc, pmlb_plan** plan);

/* `rowmax` (f32[batch * m]) is written only with PMLB_EPI_ROWMAX; `c` may then be NULL to
 * skip materialising the product. */
/* The same for a plan whose descriptor has k_first > 0: `a2` is the second part of A. */
pmlb_status pmlb_gemm_invoke_two(pmlb_plan* plan, void* stream, const void* a, const void* a2, const void* b, void* c,
                                 const void* bias, const void* residual, float* rowmax);
pmlb_status pmlb_gemm_invoke(pmlb_plan* plan, void* stream, const void* a, const void* b, void* c,
                             const void* bias, const void* residual, float* rowmax);

/* ---------------------------------------------------------------- fp32 GEMM without allocation
 * (no counterpart in the reference)
 *
 * For hosts that own all device memory themselves and must not see this library allocate: a
 * server whose arena was sized to the card, a plug-in inside another framework's allocator, a
 * loop that cannot take the stall of a driver allocation.  Computes what pmlb_gemm_dispatch /
 * pmlb_gemm_invoke compute for in_dtype = out_dtype = F32, batch = 1, no epilogue:
 *     C[i, j] = sum_k A[i, k] * B[k, j]   (b_is_nk == 0)   or   A[i, k] * B[j, k]   (b_is_nk != 0)
 * but keeps its scratch (the TF32 hi / lo copies of A and B) in a fixed device array inside the
 * library image of PMLB_NOALLOC_SCRATCH_BYTES, which every GPU that loads the library holds
 * until the process ends.  It calls no cudaMalloc / cudaFree and no allocating routine.
 *   - Limit: 8 * (m + n) * round_up(k, 4) + 256 bytes must fit in the array (1024^3 needs
 *     16 MiB); larger problems return PMLB_ERR_UNSUPPORTED with the sizes in the message.
 *   - The first call on each device looks the array's address up (with that device current);
 *     make that first call before starting any stream capture.  With CUDA's default lazy module
 *     loading the array comes into being at that first call, not when the library is loaded: a
 *     host that sizes its own pool to what the card has left must make the first call (any small
 *     problem) on every device BEFORE it measures free memory and builds the pool; afterwards a
 *     call leaves the amount of free device memory unchanged.
 *   - All calls share the one array per device and each call overwrites it: two calls whose
 *     kernels can overlap on the GPU (different streams, no dependency) race.  Serialise them.
 *   - `wait` != 0 synchronises the stream before returning and reports a device-side pipeline
 *     time-out as PMLB_ERR_TIMEOUT; with `wait` == 0 the call only enqueues, and a time-out of that
 *     launch stays in the array's status word until pmlb_gemm_f32_noalloc_status is asked or the
 *     next call clears the word: a caller that enqueues must ask before it trusts the results.
 * a, b, c are device pointers; lda / ldb / ldc count elements between rows. */
#define PMLB_NOALLOC_SCRATCH_BYTES (32u << 20)
pmlb_status pmlb_gemm_f32_noalloc(void* stream, const float* a, const float* b, float* c, int32_t m, int32_t n,
                                  int32_t k, int64_t lda, int64_t ldb, int64_t ldc, int32_t b_is_nk, int32_t wait);
/* (no counterpart in the reference)  Synchronises `stream` and reports what the launches enqueued by
 * pmlb_gemm_f32_noalloc(..., wait = 0) on the current device left in the status word: PMLB_OK, or
 * PMLB_ERR_TIMEOUT (and clears the word).  Allocates nothing. */
pmlb_status pmlb_gemm_f32_noalloc_status(void* stream);

/* ---------------------------------------------------------------- convolution
 * NHWC activation [n, h, w, c] (*) filter [r, s, c, k] -> [n, p, q, k]:
 *   O[n, y, x, ko] = sum_{fr, fs, ci} I[n, stride_h*y + dil_h*fr - pad_h, stride_w*x + dil_w*fs - pad_w, ci]
 *                                      * F[fr, fs, ci, ko]
 * with out-of-range taps skipped, i.e. the contraction op::convolution builds for
 * NXC / XCK layouts (plaidml/op/lib/ops.cc:1351-1357,1405-1446).  Replaces
 * plaidml_rt_xsmm_brgemm_offs_* (pmlc/rt/xsmm.cc:289-342,650-856).
 * in_dtype BF16 or F16; out_dtype F32, BF16 or F16; f32 accumulate.
 */
typedef struct {
  int32_t in_dtype;
  int32_t out_dtype;
  int32_t n, h, w, c;
  int32_t r, s, k;
  int32_t p, q;
  int32_t stride_h, stride_w;
  int32_t pad_h, pad_w;
  int32_t dil_h, dil_w;
  int32_t epilogue;
  int32_t tile_n;
  int32_t flags;                     /* PMLB_CONV_* */
} pmlb_conv_desc;

/* Thin inputs (c padded to a multiple of 8 is at most 32, s * that <= 64 elements, k <= 64,
 * no dilation: the first layer of image networks) take the packed-row route: the activation
 * is first copied into plan scratch with its rows zero-padded and its channels padded to a
 * multiple of 8, and each filter row then costs one 64-element k-block instead of s of them.
 * Such inputs may have any channel count; all others need c % 8 == 0.  This flag keeps an
 * eligible convolution on the general im2col route (for testing one against the other). */
#define PMLB_CONV_NO_PACKED_ROWS 1
/* Stride-1, undilated convolutions on whole 64-channel blocks into exactly 64 output channels
 * take the halo route (weights resident in shared memory, each tile's padded pixels fetched
 * once and every tap read as a shifted window).  This flag keeps them on the im2col route. */
#define PMLB_CONV_NO_HALO 2
/* Stride-2 convolutions of inputs with at most 4 channels into at most 64 output channels take
 * the space-to-depth route (a pre-pass packs the 2 x 2 pixel phases as channels; the kernel then
 * runs the stride-1 form with resident weights).  This flag sends them down the next route that
 * accepts them (packed rows, else im2col). */
#define PMLB_CONV_NO_S2D 4
/* im2col route: CTA pairs (two CTAs on one 256-pixel tile, each fetching half of the tile's
 * weights) always where the shape allows / never; without either flag the library chooses. */
#define PMLB_CONV_CTA_PAIRS 8
#define PMLB_CONV_NO_CTA_PAIRS 16
/* Halo route with three filter columns on 64 input channels: normally one 128 x 128 MMA per filter row
 * computes two columns' products side by side, one 128 x 64 MMA the third, and the epilogue adds the second
 * block one position late (the pixels are read from shared memory twice per filter row instead of once
 * per tap).  This flag keeps one MMA per tap (the form every other halo shape takes). */
#define PMLB_CONV_NO_COLUMN_MERGE 32
/* The convolution is followed by a 3 x 3 max pool of stride 2 with one pixel of padding on each side, and
 * the plan computes both: `output` of pmlb_conv_invoke is then [n][p / 2][q / 2][k] and the convolution's
 * own output is never written.  Accepted (else pmlb_conv_dispatch returns PMLB_ERR_UNSUPPORTED and the
 * caller plans the two steps separately) for the space-to-depth route with a 7-wide filter, k = 64, a
 * 16-bit output, p a multiple of 4 and q at most 124, bias and ReLU as the only epilogue terms: the first
 * layer of image networks.  No counterpart in the reference, whose stencil pass fuses no pooling. */
#define PMLB_CONV_MAX_POOL_3X3_S2 64

pmlb_status pmlb_conv_dispatch(const pmlb_conv_desc* desc, pmlb_plan** plan);

/* One-time re-layout of the filter from [r][s][c][k] (filter_dtype F32, BF16 or F16) into the
 * plan's K-major scratch copy; the analogue of the reference's `init` closure that packs
 * constants once per executable (pmlc/rt/jit_executable.cc:404-420). */
pmlb_status pmlb_conv_set_filter(pmlb_plan* plan, void* stream, const void* filter_rsck,
                                 int32_t filter_dtype);

pmlb_status pmlb_conv_invoke(pmlb_plan* plan, void* stream, const void* input, void* output,
                             const void* bias, const void* residual);

/* ---------------------------------------------------------------- reductions
 * out[o, i] = agg_{r} in[o, r, i] for agg in {SUM, MAX, MIN}; in is dense
 * [outer][reduce][inner].  inner == 1 is the row reduction (row max of cfg "Q.K^T then
 * max"), inner > 1 the strided one (global average pooling sums).  These are the
 * contractions the x86 target leaves as plain loops (pmlc/dialect/pxa/transforms/
 * stencil_gemm.cc:60-75 matches add-of-mul only).  out_dtype == dtype, or F32 for a
 * BF16/F16 input summed in f32.  `scale` (0 = none) multiplies a float sum, or with `divide`
 * != 0 divides it (the count of a mean: sum / count is what the reference's `mean` computes,
 * plaidml/op/lib/ops.cc:1970-2003; a positive divisor).
 */
typedef struct {
  int32_t agg;
  int32_t dtype;
  int32_t out_dtype;
  int32_t divide;
  int64_t outer, reduce, inner;
  double scale;
} pmlb_reduce_desc;

pmlb_status pmlb_reduce_dispatch(const pmlb_reduce_desc* desc, pmlb_plan** plan);
pmlb_status pmlb_reduce_invoke(pmlb_plan* plan, void* stream, const void* in, void* out);

/* NHWC window pooling: out[n, y, x, c] = agg over the r x s window, out-of-range taps
 * skipped (plaidml/op/lib/ops.cc:2562-2703).  agg MAX, MIN or SUM; with `average` the sum is
 * divided by the number of in-range taps (include_padding == 0) or by r*s. */
typedef struct {
  int32_t agg;
  int32_t dtype;
  int32_t n, h, w, c;
  int32_t r, s;
  int32_t p, q;
  int32_t stride_h, stride_w;
  int32_t pad_h, pad_w;
  int32_t average;
  int32_t include_padding;
} pmlb_pool_desc;

pmlb_status pmlb_pool_dispatch(const pmlb_pool_desc* desc, pmlb_plan** plan);
pmlb_status pmlb_pool_invoke(pmlb_plan* plan, void* stream, const void* in, void* out);

/* ---------------------------------------------------------------- general contraction
 * Any bounded Tile contraction (pmlc/dialect/tile/ir/ops.td:20-83 after
 * tile-compute-bounds, pmlc/dialect/tile/transforms/contraction.cc:657-681):
 *   for x in box:  if every access is in range, every constraint holds and every index
 *                  expression is integral:  O[s(x)] = agg(O[s(x)], combo(T1[a1(x)], ..))
 * Index expressions are affine with rational coefficients: coordinate of tensor dim d is
 * (off[d] + sum_i coef[d][i] * x_i) / den[d].  Slow but complete; the planner only sends
 * here what no specialised kernel covers.
 */
#define PMLB_MAX_IDX 10
#define PMLB_MAX_RANK 8
#define PMLB_MAX_CONS 8

typedef struct {
  int32_t dtype;
  int32_t rank;
  int64_t sizes[PMLB_MAX_RANK];
  int64_t strides[PMLB_MAX_RANK]; /* elements */
  int32_t coef[PMLB_MAX_RANK][PMLB_MAX_IDX];
  int64_t off[PMLB_MAX_RANK];
  int32_t den[PMLB_MAX_RANK];     /* >= 1 */
} pmlb_access;

typedef struct {
  int32_t agg;
  int32_t combo;
  int32_t n_idx;
  int32_t n_src;                  /* 1..3 */
  int64_t range[PMLB_MAX_IDX];    /* x_i in [0, range[i]) */
  pmlb_access out;
  pmlb_access src[3];
  int32_t n_cons;
  int32_t has_init;               /* 1: `init` holds a tensor broadcast-compatible with out */
  int32_t cons_coef[PMLB_MAX_CONS][PMLB_MAX_IDX];
  int64_t cons_off[PMLB_MAX_CONS];
  int64_t cons_range[PMLB_MAX_CONS]; /* 0 <= off + coef . x < range */
  pmlb_access init;               /* indexed by the output coordinates (coef unused):
                                     strides 0 on broadcast dims */
} pmlb_contract_desc;

pmlb_status pmlb_contract_dispatch(const pmlb_contract_desc* desc, pmlb_plan** plan);
pmlb_status pmlb_contract_invoke(pmlb_plan* plan, void* stream, const void* src0, const void* src1,
                                 const void* src2, const void* init, void* out);

/* ---------------------------------------------------------------- element-wise
 * out = op(in0, in1, in2) with numpy-style broadcasting (pmlc/ast/eval.cc:46-105); the
 * operations are the tile dialect's eltwise set (pmlc/dialect/tile/ir/eltwise.td:121-170),
 * named by the same mnemonics ("add", "cmp_lt", "select", "cast", ...).
 */
typedef struct {
  char op[24];
  int32_t n_in;                        /* 1..3 */
  int32_t rank;
  int32_t out_dtype;
  int32_t in_dtype[3];
  int64_t sizes[PMLB_MAX_RANK];        /* output shape (dense row-major) */
  int64_t in_strides[3][PMLB_MAX_RANK];/* elements; 0 on broadcast dims */
} pmlb_eltwise_desc;

pmlb_status pmlb_eltwise_dispatch(const pmlb_eltwise_desc* desc, pmlb_plan** plan);
pmlb_status pmlb_eltwise_invoke(pmlb_plan* plan, void* stream, const void* in0, const void* in1,
                                const void* in2, void* out);

/* ---------------------------------------------------------------- gather, scatter, argsort, prng
 * The four operations of the tile dialect that are not contractions (pmlc/dialect/tile/ir/ops.td: GatherOp,
 * ScatterOp, ArgSortOp, PrngOp), with the meaning their lowering gives them
 * (pmlc/conversion/linalg_to_pxa/tile_to_pxa_special_patterns.cc, pmlc/rt/prng.cc).  Tensors are dense row-major.
 *
 * gather   normal: out[o.., j.., i..] = tensor[o.., indices[j..], i..] along `axis` (out = tensor dims before the
 *          axis, the dims of indices, tensor dims after the axis).  Integer indices select; float indices
 *          interpolate (nearest with a rounding rule, linear, cubic with `cube_coeff`) in the tensor's float type,
 *          rounding after every operation, between neighbours clamped to the axis; out_of_bounds = 1 returns 0 for
 *          an index outside [0, len - 1].  A float index into an integer tensor is truncated.
 *          nd: the last dim of indices (K entries) addresses dims [batch_dims, batch_dims + K) of the tensor; the
 *          first batch_dims dims of indices and tensor run together.
 *          An integer index outside the axis selects the nearest edge (the reference reads out of bounds there).
 * scatter  out = data, then for every element of updates: out[dst] += u (mode 0) or out[dst] = u (modes 1..3), dst
 *          built from the element's coordinates with the `axis` coordinate (or, mode 3, the first K coordinates)
 *          replaced by entries of indices: mode 0 / 2 index with the first idx_rank coordinates of the element,
 *          mode 1 with the idx_rank coordinates from `axis` on (which collapse into one), mode 3 with the first
 *          idx_rank - 1 coordinates and the K = last-dim entries of indices.  An update that lands outside data is
 *          dropped.  Equal destinations: sums accumulate atomically (in any order); with an assigning mode one of
 *          the updates stays.
 * argsort  int32 positions that sort the tensor along `axis`, ties in their original order (mode 0 ascending,
 *          1 descending).
 * prng     `state` holds three uint32 words of a combined Tausworthe generator; out0[i] = (s0 ^ s1 ^ s2) / 2^32 as
 *          f32 for i in element order, the words stepping once per element; out1 = state with its first three
 *          words replaced by the generator's words after the last element.  Computed in parallel by jumping each
 *          thread's generator ahead with precomputed powers of the step matrices.
 */
#define PMLB_SPECIAL_GATHER 0
#define PMLB_SPECIAL_SCATTER 1
#define PMLB_SPECIAL_ARGSORT 2
#define PMLB_SPECIAL_PRNG 3

typedef struct {
  int32_t op;                        /* PMLB_SPECIAL_* */
  int32_t dtype;                     /* gather / argsort: the tensor; scatter: data, updates and result */
  int32_t idx_dtype;                 /* gather / scatter: the indices */
  int32_t rank, idx_rank, upd_rank;
  int64_t sizes[PMLB_MAX_RANK];      /* gather / argsort: the tensor; scatter: data; prng: the result */
  int64_t idx_sizes[PMLB_MAX_RANK];
  int64_t upd_sizes[PMLB_MAX_RANK];  /* scatter: updates */
  int32_t axis;
  int32_t mode;                      /* gather: 0 normal, 1 nd; scatter: 0 add, 1 slice, 2 element, 3 nd;
                                        argsort: 0 ascending, 1 descending */
  int32_t batch_dims;                /* gather nd */
  int32_t interpolation;             /* gather: 0 nearest, 1 linear, 2 cubic, 3 none */
  int32_t nearest;                   /* 0 round (half down), 1 round (half up), 2 floor, 3 ceil, 4 truncate */
  int32_t out_of_bounds;             /* 0 clamp to the edge, 1 return zero */
  double cube_coeff;
  int64_t state_elems;               /* prng: elements of the state tensor (>= 3) */
} pmlb_special_desc;

/* Elements of the result the descriptor implies (0 if the descriptor is inconsistent). */
int64_t pmlb_special_out_elems(const pmlb_special_desc* desc);
pmlb_status pmlb_special_dispatch(const pmlb_special_desc* desc, pmlb_plan** plan);
/* gather: in0 tensor, in1 indices -> out0.  scatter: in0 data, in1 indices, in2 updates -> out0.
 * argsort: in0 tensor -> out0 (int32).  prng: in0 state -> out0 (f32), out1 (new state, uint32); one of the two
 * may be null, and then only the other is computed. */
pmlb_status pmlb_special_invoke(pmlb_plan* plan, void* stream, const void* in0, const void* in1, const void* in2,
                                void* out0, void* out1);

#ifdef __cplusplus
}
#endif
#endif /* PMLB_KERNELS_H_ */
