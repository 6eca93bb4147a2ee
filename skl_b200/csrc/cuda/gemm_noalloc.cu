// gemm_noalloc.cu -- the bf16 x fp8-E4M3 GEMM for callers that cannot allocate device memory.
//
// The regular entry point (skl_gemm_ex_sm100a with a bf16 A and an fp8 B) widens B to bf16 in a
// workspace it obtains with cudaMalloc and keeps cached.  Two kinds of caller cannot live with that:
//   * a serving loop with a latency budget -- cudaMalloc and cudaFree stall the whole device, so a first
//     call (or a call with a larger shape than any before) would produce a latency spike;
//   * a process whose free device memory already belongs to someone else's pool (an inference
//     framework's caching allocator usually takes nearly all of it at start-up) -- a cudaMalloc issued
//     from inside this library would simply fail there.
// This file gives them one entry point that never allocates: the widened copy of B goes into a
// fixed array that is part of the library image.  Every GPU that loads the library therefore
// carries that array (SKL_B200_NOALLOC_SCRATCH_BYTES, 32 MiB) until the process exits, whether the
// entry point is used or not, and problems whose widened B does not fit are refused.
//
// Rules for users, all consequences of the single shared array:
//   * The first call on each device looks up the array's device address (cudaGetSymbolAddress) and
//     caches it; that first call should come before any stream capture begins.  Every call, the first
//     included, waits for its own work on the stream it was given before it returns, so that stream
//     must not be in capture mode during a call.
//   * The array keeps whatever the previous call left in it.  Nothing in it has to start at zero --
//     each call rewrites every element it later reads -- but the four status words next to it do, and
//     the entry point clears them itself at the start of every call.
//   * Two calls whose GPU work overlaps in time (different streams, different host threads) both
//     write the same array and corrupt each other.  Issue them one after the other.  The entry point
//     waits for its own work before it returns, so back-to-back calls from one thread are safe.
//   * Inputs and outputs are the caller's and must be device memory; host pointers are refused,
//     because staging them would need an allocation.
#include <cstdarg>
#include <cstdio>
#include <mutex>

#include "numerics.cuh"

#define SKL_B200_NOALLOC_SCRATCH_BYTES (32u << 20)

namespace {

constexpr size_t kScratchElems = SKL_B200_NOALLOC_SCRATCH_BYTES / sizeof(uint16_t);
constexpr int kMaxDevices = 64;

// Widened B lives here.  In host code these names are host-side stand-ins for the device arrays, not
// device addresses: they are only ever handed to cudaGetSymbolAddress, never to a kernel.
static __device__ __align__(256) uint16_t g_noalloc_scratch[kScratchElems];
static __device__ __align__(256) uint32_t g_noalloc_status[SKL_B200_DEVSTATUS_WORDS];

struct DeviceSlots {
  void *scratch;
  uint32_t *status;
  bool ready;
};
DeviceSlots g_slots[kMaxDevices];
std::mutex g_slots_mutex;
// Error text goes to the caller's buffer (may be null).
struct Message {
  char *buf;
  size_t len;
  void set(const char *fmt, ...) const {
    if (!buf || len == 0) return;
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(buf, len, fmt, ap);
    va_end(ap);
  }
};

int fail(const Message &msg, int code, const char *text) {
  msg.set("%s", text);
  return code;
}

// Device (or managed) memory of the current device `dev`?
bool is_device_pointer(const void *p, int dev) {
  cudaPointerAttributes at;
  if (cudaPointerGetAttributes(&at, p) != cudaSuccess) {
    (void)cudaGetLastError();
    return false;
  }
  if (at.type == cudaMemoryTypeManaged) return true;
  return at.type == cudaMemoryTypeDevice && at.device == dev;
}

// Once per device, with that device current: resolve the device addresses of the two arrays.
int resolve_slots(DeviceSlots **out, const Message &msg) {
  int dev = -1;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) {
    (void)cudaGetLastError();
    return fail(msg, 2, "no current CUDA device");
  }
  std::lock_guard<std::mutex> lock(g_slots_mutex);
  DeviceSlots &s = g_slots[dev];
  if (!s.ready) {
    void *scratch = nullptr, *status = nullptr;
    cudaError_t e = cudaGetSymbolAddress(&scratch, g_noalloc_scratch);
    if (e == cudaSuccess) e = cudaGetSymbolAddress(&status, g_noalloc_status);
    if (e != cudaSuccess) {
      (void)cudaGetLastError();
      msg.set("cudaGetSymbolAddress failed: %s", cudaGetErrorString(e));
      return 2;
    }
    s.scratch = scratch;
    s.status = static_cast<uint32_t *>(status);
    s.ready = true;
  }
  *out = &s;
  return 0;
}

}  // namespace

// C[m x n] (bf16) = narrow( (alpha * sum_k A[i,k]*widen(B[k,j])) * col_scale[j] ), A bf16, B fp8 E4M3.
// Same arithmetic, kernels and results as skl_gemm_ex_sm100a(BF16, F8E4M3 -> BF16, beta = 0) whenever that
// call takes the tensor-core kernel (it sends problems under 32768 multiply-adds, and layouts the tensor-core
// kernel declines, to the any-stride kernel; this entry point always uses the tensor-core kernel and refuses
// those layouts with code 5); the only other difference is where the widened B is kept.
// Returns 0, or a skl_b200_status_t value:
//   1 bad argument (null or host pointer, B with no unit stride, widened B larger than the fixed array),
//   2 CUDA error, 4 a bounded wait inside the kernel expired, 5 layout the tensor-core kernel declines.
// On a non-zero return a sentence saying why is written to error_text (error_text_len bytes, may be
// null / 0).  The call returns after the work finished on `cuda_stream`.
extern "C" int skl_gemm_bf16_f8e4m3_bf16_noalloc_sm100a(size_t m, size_t n, size_t k, float alpha,
                                                        const void *a, size_t rsa, size_t csa,
                                                        const void *b, size_t rsb, size_t csb,
                                                        const float *col_scale, void *c, size_t rsc,
                                                        size_t csc, void *cuda_stream, char *error_text,
                                                        size_t error_text_len) {
  const Message msg{error_text, error_text_len};
  msg.set("%s", "");
  if (m == 0 || n == 0) return 0;
  if (k == 0)
    return fail(msg, 1, "k == 0 is not served by this entry point (nothing to widen); use skl_gemm_ex_sm100a");
  if (!a || !b || !c) return fail(msg, 1, "null matrix pointer");
  if (m >= (size_t(1) << 31) || n >= (size_t(1) << 31) || k >= (size_t(1) << 31))
    return fail(msg, 1, "m, n and k must each be below 2^31");
  int dev = -1;
  if (cudaGetDevice(&dev) != cudaSuccess) {
    (void)cudaGetLastError();
    return fail(msg, 2, "no current CUDA device");
  }
  if (!is_device_pointer(a, dev) || !is_device_pointer(b, dev) || !is_device_pointer(c, dev) ||
      (col_scale && !is_device_pointer(col_scale, dev)))
    return fail(msg, 1, "all pointers must be device memory of the current device: staging host memory would need "
                        "an allocation");

  // Orientation of B decides the shape of its widened copy: rows x cols with cols contiguous.
  size_t rows, cols, ld_src;
  bool k_major;
  if (rsb == 1 && (n == 1 || csb >= k)) {
    rows = n; cols = k; ld_src = csb; k_major = true;
  } else if (csb == 1 && (k == 1 || rsb >= n)) {
    rows = k; cols = n; ld_src = rsb; k_major = false;
  } else {
    return fail(msg, 1, "B needs a unit stride along k or along n");
  }
  // Like the regular entry point, an n-contiguous B of a problem with at least 512 rows is written into the
  // array k-contiguous (the tensor-core kernel is faster on that orientation; the results are the same bits).
  const bool transpose = !k_major && m >= 512 && (reinterpret_cast<uintptr_t>(b) & 3u) == 0 && ld_src % 4 == 0;
  const size_t out_rows = transpose ? cols : rows, out_cols = transpose ? rows : cols;
  const size_t ld_dst = (out_cols + 7) & ~size_t(7);  // 16-byte aligned rows for TMA
  if (out_rows > kScratchElems / ld_dst) {  // dimensions are below 2^31: no product here can wrap
    msg.set("widened B needs %zu bytes, the fixed scratch array holds %u: split the problem along n or use "
            "skl_gemm_ex_sm100a",
            out_rows * ld_dst * sizeof(uint16_t), (unsigned)SKL_B200_NOALLOC_SCRATCH_BYTES);
    return 1;
  }
  if (transpose) k_major = true;  // rows of the copy are B's columns

  DeviceSlots *slots = nullptr;
  if (int rc = resolve_slots(&slots, msg)) return rc;
  cudaStream_t stream = static_cast<cudaStream_t>(cuda_stream);

  skl_b200_gemm_args g{};
  g.m0 = m; g.n0 = n; g.k0 = k;
  g.m1 = g.n1 = g.k1 = 1;
  g.ta = SKL_DT_BF16; g.tb = SKL_DT_BF16; g.tc = SKL_DT_BF16;
  g.epilogue = SKL_EPI_FLOAT;
  g.a = a; g.b = slots->scratch; g.c = c;
  g.rsa0 = (int64_t)rsa; g.csa0 = (int64_t)csa;
  g.rsb0 = k_major ? 1 : (int64_t)ld_dst;
  g.csb0 = k_major ? (int64_t)ld_dst : 1;
  g.rsc0 = (int64_t)rsc; g.csc0 = (int64_t)csc;
  g.alpha_f = alpha; g.beta_f = 0.0f;
  g.col_scale = col_scale;
  if (!skl_b200_gemm_tc_supported(&g))
    return fail(msg, 5, "A must have a unit stride, a 16-byte aligned base and a leading stride that is a multiple of 8");

  cudaError_t e = cudaMemsetAsync(slots->status, 0, SKL_B200_DEVSTATUS_WORDS * sizeof(uint32_t), stream);
  if (e == cudaSuccess)
    e = (cudaError_t)(transpose ? skl_b200_launch_cvt_f8_to_bf16_2d_transposed(slots->scratch, ld_dst, b, ld_src,
                                                                               SKL_DT_F8E4M3, rows, cols, stream)
                                : skl_b200_launch_cvt_f8_to_bf16_2d(slots->scratch, ld_dst, b, ld_src, SKL_DT_F8E4M3,
                                                                    rows, cols, stream));
  if (e == cudaSuccess) e = (cudaError_t)skl_b200_launch_gemm_tc(&g, slots->status, stream);
  // The status word comes back on the caller's stream too, so the only wait is for that stream (a copy on the
  // default stream would wait for every other stream of the process).
  uint32_t word = 0;
  if (e == cudaSuccess) e = cudaMemcpyAsync(&word, slots->status, sizeof word, cudaMemcpyDeviceToHost, stream);
  if (e == cudaSuccess) e = cudaStreamSynchronize(stream);
  if (e != cudaSuccess) {
    (void)cudaGetLastError();
    msg.set("%s: %s", cudaGetErrorName(e), cudaGetErrorString(e));
    return 2;
  }
  if (word != 0) {
    msg.set("bounded device wait expired, stage code 0x%x", word);
    return 4;
  }
  return 0;
}
