// fp32 GEMM for hosts that must not allocate device memory after start-up.
//
// Some programs that load this library hand every byte of a GPU to a pool of their own when
// they start -- an inference server that sized its arena to the card, a plug-in living inside
// another framework's caching allocator, a control loop that cannot afford the device-wide
// stall a driver allocation may cause.  For them a cudaMalloc (or any library routine that
// allocates) made later, from inside this library, either fails, fragments the card or
// blocks at the wrong moment.  The regular fp32 path needs scratch memory (the TF32 hi / lo
// copies of both operands, made by a preparation kernel) and takes it from a plan that
// allocates at dispatch time; this file offers the same computation with the scratch in a
// fixed array that is part of the library image instead.
//
// The price: every GPU that loads the library carries kStaticScratchBytes of device memory
// until the process exits, used or not, and problems whose scratch does not fit are refused.
#include <cuda_runtime.h>

#include <mutex>
#include <string>

#include "pmlb_kernels.h"
#include "prepass.h"
#include "tc_gemm.cuh"
#include "tc_launch.h"

namespace {

constexpr size_t kStaticScratchBytes = PMLB_NOALLOC_SCRATCH_BYTES;
constexpr size_t kStatusBytes = 256;  // first slot: the device word pipeline waits report into
constexpr int kMaxDevices = 64;

// Lives in every device's copy of the module.  In host code this name is only a handle for
// cudaGetSymbolAddress -- it is not a device address and must never be passed to a kernel.
static __device__ __align__(256) unsigned char g_static_scratch[kStaticScratchBytes];

std::mutex g_setup_mutex;
unsigned char* g_scratch_addr[kMaxDevices] = {nullptr};

thread_local std::string g_error;

// Resolves the array's address on the current device, once per device.
unsigned char* scratch_for_current_device(std::string* err) {
  int dev = -1;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess || dev < 0 || dev >= kMaxDevices) {
    *err = std::string("cudaGetDevice: ") + cudaGetErrorString(e);
    return nullptr;
  }
  std::lock_guard<std::mutex> lock(g_setup_mutex);
  if (g_scratch_addr[dev] == nullptr) {
    void* ptr = nullptr;
    e = cudaGetSymbolAddress(&ptr, g_static_scratch);
    if (e != cudaSuccess || ptr == nullptr) {
      *err = std::string("cudaGetSymbolAddress(static scratch): ") + cudaGetErrorString(e);
      return nullptr;
    }
    g_scratch_addr[dev] = static_cast<unsigned char*>(ptr);
  }
  return g_scratch_addr[dev];
}

}  // namespace

// Declared in tc-path code; reports through the same thread-local message as the other entry points.
extern "C" const char* pmlb_last_error(void);
void pmlb_set_last_error_message(const std::string& msg);

extern "C" pmlb_status pmlb_gemm_f32_noalloc(void* stream_v, const float* a, const float* b, float* c, int32_t m,
                                             int32_t n, int32_t k, int64_t lda, int64_t ldb, int64_t ldc,
                                             int32_t b_is_nk, int32_t wait) {
  auto fail = [](pmlb_status code, const std::string& msg) {
    pmlb_set_last_error_message(msg);
    return code;
  };
  if (!a || !b || !c) return fail(PMLB_ERR_INVALID, "gemm_f32_noalloc: null operand");
  if (m <= 0 || n <= 0 || k <= 0) return fail(PMLB_ERR_INVALID, "gemm_f32_noalloc: m, n and k must be positive");
  const int64_t min_ldb = b_is_nk ? k : n;
  if (lda < k || ldb < min_ldb || ldc < n) {
    return fail(PMLB_ERR_INVALID, "gemm_f32_noalloc: leading dimension smaller than the row length");
  }
  // scratch layout: [status word | A hi | A lo | B hi | B lo], the four copies K-major with
  // K padded to a multiple of 4 floats so that every row starts on a 16-byte boundary
  const int64_t kp = (static_cast<int64_t>(k) + 3) / 4 * 4;
  const size_t a_elems = static_cast<size_t>(m) * kp;
  const size_t b_elems = static_cast<size_t>(n) * kp;
  const size_t need = kStatusBytes + 2 * sizeof(float) * (a_elems + b_elems);
  if (need > kStaticScratchBytes) {
    return fail(PMLB_ERR_UNSUPPORTED,
                "gemm_f32_noalloc: this problem needs " + std::to_string(need) +
                    " bytes of scratch (8 * (m + n) * round_up(k, 4) + 256) but the static area holds " +
                    std::to_string(kStaticScratchBytes) + "; use pmlb_gemm_dispatch / pmlb_gemm_invoke instead");
  }
  std::string err;
  unsigned char* base = scratch_for_current_device(&err);
  if (!base) return fail(PMLB_ERR_CUDA, "gemm_f32_noalloc: " + err);
  cudaStream_t stream = static_cast<cudaStream_t>(stream_v);
  int* status = reinterpret_cast<int*>(base);
  float* a_hi = reinterpret_cast<float*>(base + kStatusBytes);
  float* a_lo = a_hi + a_elems;
  float* b_hi = a_lo + a_elems;
  float* b_lo = b_hi + b_elems;
  // The array keeps whatever the previous call left.  The status word must start at zero; the
  // operand copies are rewritten in full (padding included) by the two preparation launches.
  cudaError_t e = cudaMemsetAsync(status, 0, sizeof(int), stream);
  if (e != cudaSuccess) return fail(PMLB_ERR_CUDA, std::string("gemm_f32_noalloc: clearing the status word: ") + cudaGetErrorString(e));
  e = pmlb::launch_split_tf32(a, lda, 0, a_hi, a_lo, kp, 0, m, k, 1, false, stream);
  if (e != cudaSuccess) return fail(PMLB_ERR_CUDA, std::string("gemm_f32_noalloc: split(A): ") + cudaGetErrorString(e));
  if (b_is_nk) {
    e = pmlb::launch_split_tf32(b, ldb, 0, b_hi, b_lo, kp, 0, n, k, 1, false, stream);
  } else {
    e = pmlb::launch_split_tf32(b, ldb, 0, b_hi, b_lo, kp, 0, k, n, 1, true, stream);
  }
  if (e != cudaSuccess) return fail(PMLB_ERR_CUDA, std::string("gemm_f32_noalloc: split(B): ") + cudaGetErrorString(e));
  pmlb::TcLaunch L;
  L.elem_bytes = 4;
  L.nsplit = 2;
  L.m = m;
  L.n = n;
  L.k = k;
  L.batch = 1;
  L.a0 = a_hi;
  L.a1 = a_lo;
  L.lda = kp;
  L.b0 = b_hi;
  L.b1 = b_lo;
  L.ldb = kp;
  L.b_mn = false;
  L.out = c;
  L.ldc = ldc;
  L.out_dtype = PMLB_F32;
  L.status = status;
  const int rc = pmlb::tc_launch(L, stream, &err);
  if (rc != 0) return fail(static_cast<pmlb_status>(rc), "gemm_f32_noalloc: " + err);
  if (wait) {
    e = cudaStreamSynchronize(stream);
    if (e != cudaSuccess) return fail(PMLB_ERR_CUDA, std::string("gemm_f32_noalloc: ") + cudaGetErrorString(e));
    int code = 0;
    e = cudaMemcpy(&code, status, sizeof(int), cudaMemcpyDeviceToHost);
    if (e != cudaSuccess) return fail(PMLB_ERR_CUDA, std::string("gemm_f32_noalloc: ") + cudaGetErrorString(e));
    if (code != 0) {
      return fail(PMLB_ERR_TIMEOUT, "gemm_f32_noalloc: a device-side pipeline wait gave up (role code " + std::to_string(code) + ")");
    }
  }
  return PMLB_OK;
}

extern "C" pmlb_status pmlb_gemm_f32_noalloc_status(void* stream_v) {
  auto fail = [](pmlb_status code, const std::string& msg) {
    pmlb_set_last_error_message(msg);
    return code;
  };
  int dev = -1;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess || dev < 0 || dev >= kMaxDevices) {
    return fail(PMLB_ERR_CUDA, std::string("gemm_f32_noalloc_status: cudaGetDevice: ") + cudaGetErrorString(e));
  }
  unsigned char* base = nullptr;
  {
    std::lock_guard<std::mutex> lock(g_setup_mutex);
    base = g_scratch_addr[dev];
  }
  e = cudaStreamSynchronize(static_cast<cudaStream_t>(stream_v));
  if (e != cudaSuccess) return fail(PMLB_ERR_CUDA, std::string("gemm_f32_noalloc_status: ") + cudaGetErrorString(e));
  if (base == nullptr) return PMLB_OK;   // no call has run on this device yet
  int code = 0;
  e = cudaMemcpy(&code, base, sizeof(int), cudaMemcpyDeviceToHost);
  if (e != cudaSuccess) return fail(PMLB_ERR_CUDA, std::string("gemm_f32_noalloc_status: ") + cudaGetErrorString(e));
  if (code != 0) {
    cudaMemset(base, 0, sizeof(int));
    return fail(PMLB_ERR_TIMEOUT,
                "gemm_f32_noalloc: a device-side pipeline wait gave up (role code " + std::to_string(code) + ")");
  }
  return PMLB_OK;
}
