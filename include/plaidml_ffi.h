/*
 * plaidml_ffi.h -- the C ABI of libplaidml.so as rebuilt for the B200 `cuda` target.
 *
 * These are the entry points the reference exports from its four FFI headers
 * (plaidml/core/ffi.h:72-267, plaidml/edsl/ffi.h:31-362, plaidml/op/ffi.h:11-14,
 * plaidml/exec/ffi.h:11-40; export list plaidml/symbols.cmake:1-105), with identical names,
 * argument order and ownership rules, so that the reference's C++ wrappers (core.h, edsl.h,
 * op.h, exec.h) and its cffi loader (plaidml/ffi.py) bind against this library unchanged.
 * One header instead of four; the declarations are grouped the way the reference groups them.
 *
 * Conventions (plaidml/core/internal.h:40-70, plaidml/core/core.h:55-109):
 *   - every function except plaidml_string_ptr / plaidml_string_free takes `plaidml_error* err`
 *     first; it is cleared on entry and on failure set to {code = 1, msg = owned string} while
 *     the function returns NULL / 0;
 *   - every returned handle or list is owned by the caller and released with its *_free;
 *     plaidml_strings_free, plaidml_shapes_free and plaidml_exprs_free release the list but not
 *     its elements (the caller takes each one), plaidml_tuple_free releases its elements too;
 *   - nothing throws across this boundary.
 *
 * Additions over the reference: PLAIDML_DATA_BFLOAT16, the `cuda` target / `cuda.N` devices,
 * and the pmlb_exec_* inspection calls at the end of this file.
 */
#ifndef PLAIDML_FFI_H_
#define PLAIDML_FFI_H_

#include <stdbool.h>
#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* ------------------------------------------------------------------ handles and lists
 * plaidml/core/ffi.h:14-66 */
typedef struct plaidml_string plaidml_string;
typedef struct plaidml_shape plaidml_shape;
typedef struct plaidml_buffer plaidml_buffer;
typedef struct plaidml_executable plaidml_executable;
typedef struct plaidml_program plaidml_program;
typedef struct plaidml_dim_expr plaidml_dim_expr;
typedef struct plaidml_expr plaidml_expr;
typedef struct plaidml_poly_expr plaidml_poly_expr;
typedef struct plaidml_value plaidml_value;

typedef struct { size_t size; plaidml_string** elts; } plaidml_strings;
typedef struct { size_t size; int64_t* elts; } plaidml_integers;
typedef struct { plaidml_string* key; plaidml_string* value; } plaidml_kvp;
typedef struct { size_t size; plaidml_kvp* elts; } plaidml_kvps;
typedef struct { size_t size; plaidml_shape** elts; } plaidml_shapes;
typedef struct { size_t code; plaidml_string* msg; } plaidml_error;

/* ------------------------------------------------------------------ strings, library, settings
 * plaidml/core/ffi.h:72-131; implementation notes plaidml/core/ffi.cc:45-62 (init),
 * plaidml/core/settings.cc:19-88 (settings file + environment override). */
const char* plaidml_string_ptr(plaidml_string* str);
void plaidml_string_free(plaidml_string* str);

void plaidml_init(plaidml_error* err);
void plaidml_shutdown(plaidml_error* err);
const char* plaidml_version(plaidml_error* err);

void plaidml_integers_free(plaidml_error* err, plaidml_integers* ints);
void plaidml_strings_free(plaidml_error* err, plaidml_strings* strs);
void plaidml_kvps_free(plaidml_error* err, plaidml_kvps* kvps);
void plaidml_shapes_free(plaidml_error* err, plaidml_shapes* shapes);

plaidml_kvps* plaidml_settings_list(plaidml_error* err);
plaidml_string* plaidml_settings_get(plaidml_error* err, const char* key);
void plaidml_settings_set(plaidml_error* err, const char* key, const char* value);
void plaidml_settings_load(plaidml_error* err);
void plaidml_settings_save(plaidml_error* err);

/* ------------------------------------------------------------------ shapes
 * plaidml/core/ffi.h:137-206.  Enum values are ABI; BFLOAT16 is appended (the reference has
 * no bf16 element type).  In type promotion bf16 ranks between FLOAT16 and FLOAT32. */
typedef enum {
  PLAIDML_DATA_INVALID = 0,
  PLAIDML_DATA_INTX = 1,
  PLAIDML_DATA_UINTX = 2,
  PLAIDML_DATA_FLOATX = 3,
  PLAIDML_DATA_BOOLEAN = 4,
  PLAIDML_DATA_INT8 = 5,
  PLAIDML_DATA_UINT8 = 6,
  PLAIDML_DATA_INT16 = 7,
  PLAIDML_DATA_UINT16 = 8,
  PLAIDML_DATA_INT32 = 9,
  PLAIDML_DATA_UINT32 = 10,
  PLAIDML_DATA_INT64 = 11,
  PLAIDML_DATA_UINT64 = 12,
  PLAIDML_DATA_FLOAT16 = 13,
  PLAIDML_DATA_FLOAT32 = 14,
  PLAIDML_DATA_FLOAT64 = 15,
  PLAIDML_DATA_BFLOAT16 = 16
} plaidml_datatype;

void plaidml_shape_free(plaidml_error* err, plaidml_shape* shape);
/* `strides` may be NULL for a dense row-major tensor (plaidml/core/ffi.cc:184-198). */
plaidml_shape* plaidml_shape_alloc(plaidml_error* err, plaidml_datatype dtype, size_t rank,
                                   const int64_t* sizes, const int64_t* strides);
plaidml_shape* plaidml_shape_clone(plaidml_error* err, plaidml_shape* shape);
plaidml_string* plaidml_shape_repr(plaidml_error* err, plaidml_shape* shape);
size_t plaidml_shape_get_rank(plaidml_error* err, plaidml_shape* shape);
plaidml_datatype plaidml_shape_get_dtype(plaidml_error* err, plaidml_shape* shape);
plaidml_integers* plaidml_shape_get_sizes(plaidml_error* err, plaidml_shape* shape);
plaidml_integers* plaidml_shape_get_strides(plaidml_error* err, plaidml_shape* shape);
uint64_t plaidml_shape_get_nbytes(plaidml_error* err, plaidml_shape* shape);

/* ------------------------------------------------------------------ buffers
 * plaidml/core/ffi.h:212-243.  plaidml_buffer_data returns a HOST pointer valid for direct
 * reads and writes at any time outside plaidml_executable_run (the reference's wrappers
 * memcpy through it, plaidml/core/core.h:363-365).  plaidml_buffer_alloc returns zero-filled
 * page-locked memory that the cuda device uses directly as its staging area;
 * plaidml_buffer_adopt borrows caller memory for the buffer's lifetime. */
plaidml_buffer* plaidml_buffer_alloc(plaidml_error* err, plaidml_shape* shape);
plaidml_buffer* plaidml_buffer_adopt(plaidml_error* err, plaidml_shape* shape, char* data, size_t size);
void plaidml_buffer_free(plaidml_error* err, plaidml_buffer* buffer);
plaidml_buffer* plaidml_buffer_clone(plaidml_error* err, plaidml_buffer* buffer);
plaidml_shape* plaidml_buffer_shape(plaidml_error* err, plaidml_buffer* buffer);
char* plaidml_buffer_data(plaidml_error* err, plaidml_buffer* buffer);
size_t plaidml_buffer_size(plaidml_error* err, plaidml_buffer* buffer);

/* ------------------------------------------------------------------ programs
 * plaidml/core/ffi.h:249-284.  plaidml_program_compile("" target) resolves PLAIDML_TARGET
 * (plaidml/core/ffi.cc:376-389); the only target is "cuda" (options in braces are accepted
 * and ignored, as in pmlc/compiler/program.cc:176-188).  plaidml_program_save reports that
 * the target has no save support, like the x86 target (pmlc/target/x86/register.cc:26-33).
 * plaidml_program_repr returns the program spelled like the reference's printed `tile` module
 * (module @name { func @main(...) { tile.constant / tile.<eltwise> / tile.contract ... } }), the text
 * the FileCheck lines of plaidml/edsl/tests/edsl_test.cc match.  plaidml_program_get_passes returns
 * two entries: "tile" (that text) and "bounds" (every contraction with its index ranges and
 * rational access forms, the form the planner consumes). */
void plaidml_program_free(plaidml_error* err, plaidml_program* program);
plaidml_string* plaidml_program_repr(plaidml_error* err, plaidml_program* program);
plaidml_shapes* plaidml_program_get_inputs(plaidml_error* err, plaidml_program* program);
plaidml_shapes* plaidml_program_get_outputs(plaidml_error* err, plaidml_program* program);
plaidml_kvps* plaidml_program_get_passes(plaidml_error* err, plaidml_program* program);
void plaidml_program_compile(plaidml_error* err, plaidml_program* program, bool debug, const char* target);
plaidml_buffer* plaidml_program_save(plaidml_error* err, plaidml_program* program, size_t nkvps,
                                     const char** keys, const char** values);

/* ------------------------------------------------------------------ EDSL
 * plaidml/edsl/ffi.h:11-362. */
typedef enum {
  PLAIDML_INT_OP_NEG, PLAIDML_INT_OP_ADD, PLAIDML_INT_OP_SUB, PLAIDML_INT_OP_MUL,
  PLAIDML_INT_OP_DIV, PLAIDML_INT_OP_MAX, PLAIDML_INT_OP_MIN
} plaidml_int_op;

typedef enum {
  PLAIDML_VALUE_NONE, PLAIDML_VALUE_DIM, PLAIDML_VALUE_EXPR, PLAIDML_VALUE_FLOAT,
  PLAIDML_VALUE_INT, PLAIDML_VALUE_STR, PLAIDML_VALUE_TUPLE
} plaidml_value_kind;

typedef enum {
  PLAIDML_AGG_OP_NONE, PLAIDML_AGG_OP_SUM, PLAIDML_AGG_OP_MAX, PLAIDML_AGG_OP_MIN,
  PLAIDML_AGG_OP_PROD, PLAIDML_AGG_OP_ASSIGN
} plaidml_agg_op;

typedef enum {
  PLAIDML_COMBO_OP_NONE, PLAIDML_COMBO_OP_MUL, PLAIDML_COMBO_OP_ADD, PLAIDML_COMBO_OP_EQ,
  PLAIDML_COMBO_OP_COND
} plaidml_combo_op;

typedef struct { const char* key; plaidml_value* value; } plaidml_attr;
typedef struct { size_t size; plaidml_expr** elts; } plaidml_exprs;
typedef struct { size_t size; plaidml_value** elts; } plaidml_tuple;

void plaidml_edsl_init(plaidml_error* err);

/* index polynomials (plaidml/edsl/ffi.cc:437-520) */
void plaidml_poly_expr_free(plaidml_error* err, plaidml_poly_expr* expr);
plaidml_string* plaidml_poly_expr_repr(plaidml_error* err, plaidml_poly_expr* expr);
plaidml_poly_expr* plaidml_poly_expr_dim(plaidml_error* err, plaidml_dim_expr* expr);
plaidml_poly_expr* plaidml_poly_expr_index(plaidml_error* err, const char* name);
plaidml_poly_expr* plaidml_poly_expr_literal(plaidml_error* err, int64_t value);
plaidml_poly_expr* plaidml_poly_expr_op(plaidml_error* err, plaidml_int_op op, size_t nargs,
                                        plaidml_poly_expr** args);

/* dimension expressions */
void plaidml_dim_expr_free(plaidml_error* err, plaidml_dim_expr* expr);
plaidml_string* plaidml_dim_expr_repr(plaidml_error* err, plaidml_dim_expr* expr);
plaidml_dim_expr* plaidml_dim_expr_none(plaidml_error* err);
plaidml_dim_expr* plaidml_dim_expr_int(plaidml_error* err, int64_t value);
plaidml_dim_expr* plaidml_dim_expr_op(plaidml_error* err, plaidml_int_op op, size_t nargs,
                                      plaidml_dim_expr** args);

/* tensor expressions (plaidml/edsl/ffi.cc:132-363) */
void plaidml_expr_free(plaidml_error* err, plaidml_expr* expr);
void* plaidml_expr_ptr(plaidml_error* err, plaidml_expr* expr);
plaidml_datatype plaidml_expr_get_dtype(plaidml_error* err, plaidml_expr* expr);
size_t plaidml_expr_get_rank(plaidml_error* err, plaidml_expr* expr);
plaidml_shape* plaidml_expr_get_shape(plaidml_error* err, plaidml_expr* expr);
/* Binds each unbound dim to the tensor's size (replacing dims[i]'s content in place) and
 * checks already-bound ones (pmlc/ast/eval.cc:300-362). */
void plaidml_expr_bind_dims(plaidml_error* err, plaidml_expr* expr, size_t rank, plaidml_dim_expr** dims);
plaidml_string* plaidml_expr_repr(plaidml_error* err, plaidml_expr* expr);
plaidml_expr* plaidml_expr_clone(plaidml_error* err, plaidml_expr* expr);
plaidml_dim_expr* plaidml_expr_get_dim(plaidml_error* err, plaidml_expr* expr);
plaidml_expr* plaidml_expr_dim(plaidml_error* err, plaidml_dim_expr* expr);
plaidml_expr* plaidml_expr_input(plaidml_error* err, plaidml_shape* shape, const char* name);
plaidml_expr* plaidml_expr_constant(plaidml_error* err, plaidml_buffer* buffer, const char* name);
plaidml_expr* plaidml_expr_uint(plaidml_error* err, uint64_t value);
plaidml_expr* plaidml_expr_int(plaidml_error* err, int64_t value);
plaidml_expr* plaidml_expr_float(plaidml_error* err, double value);
plaidml_expr* plaidml_expr_element(plaidml_error* err, plaidml_expr* expr, size_t ordinal);
plaidml_expr* plaidml_expr_intrinsic(plaidml_error* err, const char* fn, size_t nargs,
                                     plaidml_expr** args, const char* name);
plaidml_expr* plaidml_expr_cast(plaidml_error* err, plaidml_expr* tensor, plaidml_datatype dtype);
plaidml_expr* plaidml_expr_pragma(plaidml_error* err, plaidml_expr* tensor, const char* op,
                                  size_t nattrs, plaidml_attr** attrs);
void plaidml_exprs_free(plaidml_error* err, plaidml_exprs* exprs);
plaidml_expr* plaidml_expr_layer_begin(plaidml_error* err, const char* op, size_t ninputs,
                                       plaidml_expr** inputs, size_t nattrs, plaidml_attr** attrs);
plaidml_exprs* plaidml_expr_layer_end(plaidml_error* err, plaidml_expr* expr, size_t noutputs,
                                      plaidml_expr** outputs);

/* contractions (plaidml/edsl/ffi.cc:365-435): O[idxs : dims] = agg(combo(operands...)), each
 * constraint meaning 0 <= lhs < rhs; `init` may be NULL. */
plaidml_expr* plaidml_expr_contraction(plaidml_error* err, plaidml_agg_op agg_op, plaidml_combo_op combo_op,
                                       size_t rank, plaidml_poly_expr** idxs, plaidml_dim_expr** dims,
                                       plaidml_expr* init, const char* name);
void plaidml_contraction_add_operand(plaidml_error* err, plaidml_expr* expr, plaidml_expr* tensor,
                                     size_t rank, plaidml_poly_expr** idxs);
void plaidml_contraction_add_constraint(plaidml_error* err, plaidml_expr* expr, plaidml_poly_expr* lhs,
                                        plaidml_dim_expr* rhs);
void plaidml_contraction_build(plaidml_error* err, plaidml_expr* expr);

/* values: the variant used for op-library arguments (plaidml/edsl/ffi.cc:522-770) */
void plaidml_tuple_free(plaidml_error* err, plaidml_tuple* tuple);
void plaidml_value_free(plaidml_error* err, plaidml_value* value);
plaidml_value* plaidml_value_clone(plaidml_error* err, plaidml_value* value);
plaidml_value_kind plaidml_value_get_kind(plaidml_error* err, plaidml_value* value);
plaidml_value* plaidml_value_none(plaidml_error* err);
plaidml_value* plaidml_value_dim(plaidml_error* err, plaidml_dim_expr* expr);
plaidml_value* plaidml_value_expr(plaidml_error* err, plaidml_expr* expr);
plaidml_value* plaidml_value_float(plaidml_error* err, double value);
plaidml_value* plaidml_value_int(plaidml_error* err, int64_t value);
plaidml_value* plaidml_value_str(plaidml_error* err, const char* value);
plaidml_value* plaidml_value_tuple(plaidml_error* err, size_t nelts, plaidml_value** elts);
plaidml_dim_expr* plaidml_value_dim_get(plaidml_error* err, plaidml_value* value);
plaidml_expr* plaidml_value_expr_get(plaidml_error* err, plaidml_value* value);
double plaidml_value_float_get(plaidml_error* err, plaidml_value* value);
int64_t plaidml_value_int_get(plaidml_error* err, plaidml_value* value);
plaidml_string* plaidml_value_str_get(plaidml_error* err, plaidml_value* value);
plaidml_tuple* plaidml_value_tuple_get(plaidml_error* err, plaidml_value* value);
plaidml_string* plaidml_value_repr(plaidml_error* err, plaidml_value* value);

plaidml_strings* plaidml_targets_get(plaidml_error* err);

/* Builds a program from output expressions (plaidml/edsl/ffi.cc:772-793,
 * pmlc/ast/builder.cc:492-624): arguments are `inputs` in the given order (each optionally
 * re-shaped by shapes[i], which may be NULL), then every constant tensor in discovery order. */
plaidml_program* plaidml_build(plaidml_error* err, const char* name, size_t ninputs, plaidml_expr** inputs,
                               plaidml_shape** shapes, size_t noutputs, plaidml_expr** outputs);

/* ------------------------------------------------------------------ op library
 * plaidml/op/ffi.h:11-14, registry plaidml/op/lib/ops.cc:3632-3680.  Implemented here: the
 * operations that build the contraction path's networks -- convolution (forward, NXC / XCK,
 * ungrouped), pool, dot, relu, mean, sum, max, min, softmax, plus thin element-wise ones. */
plaidml_value* plaidml_op_make(plaidml_error* err, const char* op_name, plaidml_value* value);

/* ------------------------------------------------------------------ execution
 * plaidml/exec/ffi.h:11-40.  Devices are "cuda.0" .. "cuda.N-1", one per visible GPU of
 * compute capability 10.x; plaidml_jit("" device) resolves PLAIDML_DEVICE
 * (plaidml/exec/ffi.cc:61-73).  plaidml_executable_run checks argument counts and exact
 * shape equality (plaidml/exec/ffi.cc:92-120), copies inputs to the device, runs the kernel
 * sequence, copies outputs back into the output buffers and returns the elapsed
 * milliseconds, complete on return. */
void plaidml_exec_init(plaidml_error* err);
plaidml_strings* plaidml_devices_get(plaidml_error* err);
plaidml_executable* plaidml_jit(plaidml_error* err, plaidml_program* program, const char* device);
void plaidml_executable_free(plaidml_error* err, plaidml_executable* exec);
double plaidml_executable_run(plaidml_error* err, plaidml_executable* exec, size_t ninputs,
                              plaidml_buffer** inputs, size_t noutputs, plaidml_buffer** outputs);

/* ------------------------------------------------------------------ additions (no reference counterpart)
 * Inspection of a compiled executable, used by tests and benchmarks. */

/* One line per kernel step: "<kernel family> <contraction or op name> ..." */
plaidml_string* pmlb_exec_describe(plaidml_error* err, plaidml_executable* exec);
/* Number of kernel launches one run enqueues. */
size_t pmlb_exec_launch_count(plaidml_error* err, plaidml_executable* exec);
/* 1 once the kernel sequence has been captured into a CUDA graph and passes replay it (from the
 * second pass on, for programs of two or more steps, unless PLAIDML_CUDA_GRAPH=0), else 0. */
int pmlb_exec_uses_graph(plaidml_error* err, plaidml_executable* exec);
/* Number of groups plaidml_executable_run uploads the inputs in (known after the first run).  1: all inputs, then the
 * kernels.  More: the program has several inputs first used at different depths (weights passed as inputs), so the
 * step list is cut where a group of a few megabytes is first needed and each part starts when its group has arrived,
 * the later groups still crossing the host link (PLAIDML_CUDA_UPLOAD_OVERLAP=0 turns it off). */
size_t pmlb_exec_upload_groups(plaidml_error* err, plaidml_executable* exec);
/* Re-runs the kernel sequence `iters` times on the inputs already resident on the device from
 * the last plaidml_executable_run (no host copies) and returns the mean milliseconds per
 * iteration measured with CUDA events on the executable's stream. */
double pmlb_exec_run_resident(plaidml_error* err, plaidml_executable* exec, size_t iters);
/* Like pmlb_exec_run_resident, but every pass is bracketed by its own CUDA event pair and,
 * with `flush_l2`, preceded by an untimed overwrite of a 256 MiB device buffer so that no
 * pass finds its operands in the 126 MB L2.  Passes are enqueued up to 64 ahead of the host's
 * wait, so an interval holds device time only; returns the mean interval in milliseconds. */
double pmlb_exec_time_steps(plaidml_error* err, plaidml_executable* exec, size_t iters, bool flush_l2);
/* The same, with every pass's interval written to ms_out[0 .. iters) (milliseconds). */
void pmlb_exec_time_passes(plaidml_error* err, plaidml_executable* exec, size_t iters, bool flush_l2, double* ms_out);
/* Every kernel step on its own: ms_out[i] (i < the returned step count, line i of pmlb_exec_describe) receives the
 * mean milliseconds of step i over `iters` launches back to back, replayed from a CUDA graph between one event pair
 * (so the host cost of launching is not in the figure, as in a replayed program).  Nothing is run when
 * ms_out is NULL or `capacity` is below the step count; the count is returned either way. */
size_t pmlb_exec_time_each_step(plaidml_error* err, plaidml_executable* exec, size_t iters, bool flush_l2, double* ms_out,
                                size_t capacity);
/* Device address and byte size of output `index` (valid until the executable is freed). */
void* pmlb_exec_output_device_ptr(plaidml_error* err, plaidml_executable* exec, size_t index, size_t* nbytes);
/* CUDA stream (cudaStream_t) the executable enqueues on. */
void* pmlb_exec_stream(plaidml_error* err, plaidml_executable* exec);


/* ------------------------------------------------------------------ sharded mode (no reference counterpart)
 * One process per GPU, each compiling the same program for its slice of the independent dimension
 * (rows of M, images of a batch); the reference splits one fixed problem over threads that share one
 * memory instead (pmlc/dialect/pxa/transforms/cpu_thread.cc:49-92).  The data path has no exchange
 * step.  Two collectives exist around it, each one NCCL all-gather over NVLink on buffers the
 * executable owns; NCCL (libnccl.so.2) is bound with dlopen at the first of these calls.
 *
 * pmlb_shard_unique_id: called on rank 0; the caller carries the 128 bytes to the other ranks.
 * pmlb_shard_init: collective; makes `device` ("cuda.N", or PLAIDML_DEVICE when empty) current and
 *   joins the process to the communicator.  world == 1 needs no id and loads nothing.
 * pmlb_exec_set_input_replicated: marks a program input as holding the same data on every rank (the
 *   B matrix of a row-sharded GEMM).  plaidml_executable_run then uploads only bytes / world of it
 *   from this rank's host buffer and completes it with an all-gather, so that the operand crosses the
 *   host link once per box, not once per rank.  Every rank must mark the same inputs.
 * pmlb_exec_gather_output: all ranks' copies of output `index` concatenated in rank order, in device
 *   memory the executable owns (valid until the next gather or until it is freed); *nbytes receives
 *   world x the output's size.  Complete on return.  iters > 1 repeats the collective and *mean_ms
 *   (may be NULL) receives the mean device time of one, by CUDA events on the executable's stream. */
#define PMLB_SHARD_ID_BYTES 128
void pmlb_shard_unique_id(plaidml_error* err, char* id);
void pmlb_shard_init(plaidml_error* err, int rank, int world, const char* id, const char* device);
void pmlb_shard_shutdown(plaidml_error* err);
int pmlb_shard_rank(plaidml_error* err);
int pmlb_shard_world(plaidml_error* err);
void pmlb_exec_set_input_replicated(plaidml_error* err, plaidml_executable* exec, size_t index, int replicated);
void* pmlb_exec_gather_output(plaidml_error* err, plaidml_executable* exec, size_t index, size_t* nbytes, size_t iters,
                              double* mean_ms);

#ifdef __cplusplus
}
#endif
#endif /* PLAIDML_FFI_H_ */
