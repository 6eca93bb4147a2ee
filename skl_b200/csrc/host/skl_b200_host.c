/*
 * skl_b200_host.c -- the C99 host layer of libskl_b200.
 *
 * Implements every entry point declared in include/skl-b200.h on top of the launch ABI in ../abi.h:
 * argument checks, host/device pointer classification, staging of host operands through cached
 * device workspaces, kernel-family dispatch, and the per-thread status side channel that SKL's
 * void signatures have no room for.  No arithmetic on matrix data happens on the CPU: when the
 * device path cannot run, the call records an error and returns.
 *
 * Plain C (gnu99); the CUDA runtime is used only through its C API.
 */
#include "../../../include/skl-b200.h"
#include "../abi.h"

#include <cuda_runtime_api.h>
#include <pthread.h>
#include <stdio.h>
#include <stdlib.h>
#include <string.h>

/* ------------------------------------------------------------------ per-thread context */

enum { WS_A = 0, WS_B, WS_C, WS_ROW, WS_COL, WS_WIDEN, WS_BIAS, WS_GMAX, WS_PLAIN_A, WS_PLAIN_B, WS_PLAIN_C, WS_COUNT };

#define PIPE_MAX_CHUNKS 16

/* largest m the dp4a skinny kernel serves; above it the transposed tensor-core route is faster */
#ifndef SKINNY_DP4A_MAX
#define SKINNY_DP4A_MAX 2
#endif

typedef struct {
  void *ptr;
  size_t cap;
} workspace_t;

typedef struct {
  void *stream;
  int async;
  int static_weights; /* skl_b200_set_static_weights */
  /* widened copy of a static fp8 B kept from the previous call: source, geometry, format, where it lives */
  const void *wide_src;
  size_t wide_rows, wide_cols, wide_ld;
  int wide_fmt, wide_transposed;
  void *wide_ptr; /* 0 = nothing cached */
  skl_b200_status_t status;
  char cuda_err[192];
  skl_b200_path_t last_path;
  int last_launches;
  int force_path;
  int device;           /* device the cached resources belong to, -1 = none */
  uint32_t *dev_status; /* mapped pinned host words written by kernels on a bounded-wait expiry */
  workspace_t ws[WS_COUNT];
  /* optional timing of the main GEMM kernel of each call: pairs of events on the launch stream */
  cudaEvent_t *prof_ev;
  int prof_cap, prof_used;
  /* row-chunk pipeline for host operands */
  int exit_registered; /* this thread's exit hook (thread_exit_release) is in place */
  unsigned wait_limit_ms; /* skl_b200_set_wait_limit: bound of the kernels' device-side waits, 0 = default */
  int debug_skip_loads;   /* skl_b200_debug_skip_loads */
  int pipe_ready;
  cudaStream_t s_in, s_out;
  cudaEvent_t ev_in[PIPE_MAX_CHUNKS], ev_done[PIPE_MAX_CHUNKS], ev_ready;
} ctx_t;

static __thread ctx_t g_ctx = {.status = SKL_B200_OK, .last_path = SKL_B200_PATH_NONE, .device = -1};

static void set_err(skl_b200_status_t s) {
  if (g_ctx.status == SKL_B200_OK) g_ctx.status = s;
}

static int cuda_ok(cudaError_t e) {
  if (e == cudaSuccess) return 1;
  if (g_ctx.status == SKL_B200_OK) {
    g_ctx.status = SKL_B200_ERR_CUDA;
    snprintf(g_ctx.cuda_err, sizeof g_ctx.cuda_err, "%s: %s", cudaGetErrorName(e), cudaGetErrorString(e));
  }
  (void)cudaGetLastError();
  return 0;
}

static void release_resources(void) {
  for (int i = 0; i < WS_COUNT; ++i) {
    if (g_ctx.ws[i].ptr) (void)cudaFree(g_ctx.ws[i].ptr);
    g_ctx.ws[i].ptr = 0;
    g_ctx.ws[i].cap = 0;
    g_ctx.wide_ptr = 0;
  }
  if (g_ctx.dev_status) (void)cudaFreeHost(g_ctx.dev_status);
  g_ctx.dev_status = 0;
  if (g_ctx.pipe_ready) {
    (void)cudaStreamDestroy(g_ctx.s_in);
    (void)cudaStreamDestroy(g_ctx.s_out);
    for (int i = 0; i < PIPE_MAX_CHUNKS; ++i) {
      (void)cudaEventDestroy(g_ctx.ev_in[i]);
      (void)cudaEventDestroy(g_ctx.ev_done[i]);
    }
    (void)cudaEventDestroy(g_ctx.ev_ready);
    g_ctx.pipe_ready = 0;
  }
  g_ctx.device = -1;
}

/* A thread that used the library owns device workspaces, pinned status words, streams and events.  They are
 * released when the thread ends: a pthread key whose destructor runs at thread exit (registered by the
 * thread's first call) makes the owning device current and frees them.  The main thread's resources go with
 * the process.  skl_b200_release_workspace() does the same on request. */
static pthread_key_t g_exit_key;
static pthread_once_t g_exit_once = PTHREAD_ONCE_INIT;

static void thread_exit_release(void *arg) {
  (void)arg;
  if (g_ctx.device < 0) return;
  int cur = -1;
  if (cudaGetDevice(&cur) != cudaSuccess) {
    (void)cudaGetLastError();
    return; /* the runtime is already gone (process teardown): nothing left to free */
  }
  if (cur != g_ctx.device && cudaSetDevice(g_ctx.device) != cudaSuccess) {
    (void)cudaGetLastError();
    return;
  }
  (void)cudaStreamSynchronize((cudaStream_t)g_ctx.stream);
  release_resources();
  if (g_ctx.prof_ev) {
    for (int i = 0; i < 2 * g_ctx.prof_cap; ++i) (void)cudaEventDestroy(g_ctx.prof_ev[i]);
    free(g_ctx.prof_ev);
    g_ctx.prof_ev = 0;
  }
  (void)cudaGetLastError();
}

static void make_exit_key(void) { (void)pthread_key_create(&g_exit_key, thread_exit_release); }

static void register_thread_exit(void) {
  (void)pthread_once(&g_exit_once, make_exit_key);
  if (!g_ctx.exit_registered) {
    /* any non-null value makes the destructor run for this thread */
    if (pthread_setspecific(g_exit_key, &g_ctx) == 0) g_ctx.exit_registered = 1;
  }
}

/* Start of every public call: clears the status, binds the cached resources to the current device. */
static int begin_call(void) {
  g_ctx.status = SKL_B200_OK;
  g_ctx.cuda_err[0] = 0;
  g_ctx.last_launches = 0;
  (void)skl_b200_launch_counter(1);
  register_thread_exit();
  int dev = -1;
  if (!cuda_ok(cudaGetDevice(&dev))) return 0;
  if (dev != g_ctx.device) {
    if (g_ctx.device >= 0) {
      int cur = dev;
      (void)cudaSetDevice(g_ctx.device);
      release_resources();
      (void)cudaSetDevice(cur);
    }
    int major = 0;
    if (!cuda_ok(cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, dev))) return 0;
    if (major != 10) {
      g_ctx.status = SKL_B200_ERR_CUDA;
      snprintf(g_ctx.cuda_err, sizeof g_ctx.cuda_err, "device %d is not compute capability 10.x", dev);
      return 0;
    }
    g_ctx.device = dev;
  }
  return 1;
}

static void end_call(void) { g_ctx.last_launches = skl_b200_launch_counter(0); }

/* End of every public call that got past begin_call().  A call that failed half way may have queued copies to or
 * from the caller's host buffers (staging, the row-chunk pipeline): they are waited for before the call returns,
 * so that the caller, who sees the error status, may free or reuse those buffers at once. */
static void leave_call(void) {
  if (g_ctx.status != SKL_B200_OK) {
    (void)cudaStreamSynchronize((cudaStream_t)g_ctx.stream);
    if (g_ctx.pipe_ready) {
      (void)cudaStreamSynchronize(g_ctx.s_in);
      (void)cudaStreamSynchronize(g_ctx.s_out);
    }
    (void)cudaGetLastError();
  }
  end_call();
}

static uint32_t *device_status_words(void) {
  if (!g_ctx.dev_status) {
    void *p = 0;
    if (!cuda_ok(cudaHostAlloc(&p, SKL_B200_DEVSTATUS_WORDS * sizeof(uint32_t), cudaHostAllocMapped))) return 0;
    memset(p, 0, SKL_B200_DEVSTATUS_WORDS * sizeof(uint32_t));
    g_ctx.dev_status = (uint32_t *)p;
  }
  return g_ctx.dev_status;
}

static void *workspace(int slot, size_t bytes) {
  workspace_t *w = &g_ctx.ws[slot];
  if (bytes == 0) bytes = 16;
  if (w->cap < bytes) {
    if (w->ptr) {
      /* the previous call's work on this buffer has completed or is ordered before the free */
      (void)cudaStreamSynchronize((cudaStream_t)g_ctx.stream);
      (void)cudaFree(w->ptr);
      w->ptr = 0;
      w->cap = 0;
      if (slot == WS_WIDEN) g_ctx.wide_ptr = 0;
    }
    size_t want = bytes + bytes / 8 + 256;
    void *p = 0;
    cudaError_t e = cudaMalloc(&p, want);
    if (e != cudaSuccess) {
      (void)cudaGetLastError();
      set_err(SKL_B200_ERR_ALLOC);
      return 0;
    }
    w->ptr = p;
    w->cap = want;
  }
  return w->ptr;
}

static int on_device(const void *p) {
  struct cudaPointerAttributes at;
  if (p == 0) return 1;
  if (cudaPointerGetAttributes(&at, p) != cudaSuccess) {
    (void)cudaGetLastError();
    return 0;
  }
  return at.type == cudaMemoryTypeDevice || at.type == cudaMemoryTypeManaged;
}

static void finish(int had_host_operand) {
  if (g_ctx.status != SKL_B200_OK) {
    (void)cudaStreamSynchronize((cudaStream_t)g_ctx.stream);
    return;
  }
  if (had_host_operand || !g_ctx.async) {
    cuda_ok(cudaStreamSynchronize((cudaStream_t)g_ctx.stream));
    if (g_ctx.dev_status && g_ctx.dev_status[0] != 0) {
      g_ctx.status = SKL_B200_ERR_DEVICE_TIMEOUT;
      snprintf(g_ctx.cuda_err, sizeof g_ctx.cuda_err, "bounded device wait expired, stage code 0x%x",
               g_ctx.dev_status[0]);
      g_ctx.dev_status[0] = 0;
    }
  }
}

/* ------------------------------------------------------------------ side channel */

skl_b200_status_t skl_b200_last_status(void) { return g_ctx.status; }

const char *skl_b200_status_string(skl_b200_status_t s) {
  switch (s) {
  case SKL_B200_OK: return "ok";
  case SKL_B200_ERR_INVALID_ARGUMENT: return "invalid argument";
  case SKL_B200_ERR_CUDA: return "CUDA error";
  case SKL_B200_ERR_ALLOC: return "device workspace allocation failed";
  case SKL_B200_ERR_DEVICE_TIMEOUT: return "bounded device wait expired";
  case SKL_B200_ERR_UNSUPPORTED: return "unsupported type combination";
  default: return "unknown status";
  }
}

const char *skl_b200_last_cuda_error(void) { return g_ctx.cuda_err; }
void skl_b200_set_stream(void *cuda_stream) {
  if (cuda_stream != g_ctx.stream) g_ctx.wide_ptr = 0; /* the cached widened B was produced in the old stream's order */
  g_ctx.stream = cuda_stream;
}
void *skl_b200_get_stream(void) { return g_ctx.stream; }
void skl_b200_set_async(int enabled) { g_ctx.async = enabled != 0; }
void skl_b200_set_static_weights(int enabled) { g_ctx.static_weights = enabled != 0; }
skl_b200_path_t skl_b200_last_path(void) { return g_ctx.last_path; }
int skl_b200_last_launch_count(void) { return g_ctx.last_launches; }
void skl_b200_force_path(int path) { g_ctx.force_path = path; }
void skl_b200_set_wait_limit(unsigned milliseconds) { g_ctx.wait_limit_ms = milliseconds; }
void skl_b200_debug_skip_loads(int enabled) { g_ctx.debug_skip_loads = enabled != 0; }

void skl_b200_profile_begin(int max_calls) {
  if (g_ctx.prof_ev) {
    for (int i = 0; i < 2 * g_ctx.prof_cap; ++i) (void)cudaEventDestroy(g_ctx.prof_ev[i]);
    free(g_ctx.prof_ev);
    g_ctx.prof_ev = 0;
  }
  g_ctx.prof_cap = 0;
  g_ctx.prof_used = 0;
  if (max_calls <= 0) return;
  g_ctx.prof_ev = (cudaEvent_t *)calloc((size_t)(2 * max_calls), sizeof(cudaEvent_t));
  if (!g_ctx.prof_ev) return;
  for (int i = 0; i < 2 * max_calls; ++i) {
    if (cudaEventCreate(&g_ctx.prof_ev[i]) != cudaSuccess) {
      (void)cudaGetLastError();
      for (int j = 0; j < i; ++j) (void)cudaEventDestroy(g_ctx.prof_ev[j]);
      free(g_ctx.prof_ev);
      g_ctx.prof_ev = 0;
      return;
    }
  }
  g_ctx.prof_cap = max_calls;
}

int skl_b200_profile_end(double *total_ms) {
  double sum = 0.0;
  int n = g_ctx.prof_used;
  (void)cudaStreamSynchronize((cudaStream_t)g_ctx.stream);
  for (int i = 0; i < n; ++i) {
    float ms = 0.0f;
    if (cudaEventElapsedTime(&ms, g_ctx.prof_ev[2 * i], g_ctx.prof_ev[2 * i + 1]) == cudaSuccess) sum += ms;
    else (void)cudaGetLastError();
  }
  if (total_ms) *total_ms = sum;
  skl_b200_profile_begin(0);
  return n;
}

void skl_b200_synchronize(void) {
  g_ctx.status = SKL_B200_OK;
  g_ctx.cuda_err[0] = 0;
  cuda_ok(cudaStreamSynchronize((cudaStream_t)g_ctx.stream));
  if (g_ctx.dev_status && g_ctx.dev_status[0] != 0) {
    set_err(SKL_B200_ERR_DEVICE_TIMEOUT);
    g_ctx.dev_status[0] = 0;
  }
}

void skl_b200_release_workspace(void) {
  (void)cudaStreamSynchronize((cudaStream_t)g_ctx.stream);
  release_resources();
}

void skl_b200_shard_columns(size_t n, size_t parts, size_t index, size_t align, size_t *start,
                            size_t *count) {
  size_t s = 0, c = 0;
  if (parts != 0 && index < parts) {
    if (align == 0) align = 1;
    size_t units = (n + align - 1) / align; /* whole `align`-column units, the last may be short */
    size_t base = units / parts, extra = units % parts;
    size_t u0 = index * base + (index < extra ? index : extra);
    size_t u1 = u0 + base + (index < extra ? 1 : 0);
    s = u0 * align;
    size_t e = u1 * align;
    if (s > n) s = n;
    if (e > n) e = n;
    c = e - s;
  }
  if (start) *start = s;
  if (count) *count = c;
}

/* ------------------------------------------------------------------ staging helpers */

static size_t dt_size(int dt) {
  if (dt == SKL_DT_F64) return 8;
  return (dt == SKL_DT_F32 || dt == SKL_DT_I32) ? 4 : ((dt == SKL_DT_BF16 || dt == SKL_DT_F16) ? 2 : 1);
}

/* Elements spanned by a blocked matrix: last addressed offset + 1 (0 when empty). */
static size_t span4(uint64_t r0, uint64_t c0, uint64_t r1, uint64_t c1, int64_t rs0, int64_t cs0,
                    int64_t rs1, int64_t cs1) {
  if (r0 == 0 || c0 == 0 || r1 == 0 || c1 == 0) return 0;
  return (size_t)((r0 - 1) * (uint64_t)rs0 + (c0 - 1) * (uint64_t)cs0 + (r1 - 1) * (uint64_t)rs1 +
                  (c1 - 1) * (uint64_t)cs1 + 1);
}

static const void *stage_in(int slot, const void *host, size_t bytes) {
  void *d = workspace(slot, bytes);
  if (!d) return 0;
  if (bytes && !cuda_ok(cudaMemcpyAsync(d, host, bytes, cudaMemcpyHostToDevice, (cudaStream_t)g_ctx.stream)))
    return 0;
  return d;
}

/* A host-resident output matrix staged on the device with the caller's own strides. */
typedef struct {
  void *host;
  void *dev;
  size_t span_bytes;
  /* 2-D form: `height` runs of `width` bytes every `pitch` bytes; width == 0 means "whole span" */
  size_t width, height, pitch;
} out_stage_t;

static int stage_out_begin(out_stage_t *o, void *host, size_t span_bytes, size_t width, size_t height,
                           size_t pitch, int need_old) {
  o->host = host;
  o->span_bytes = span_bytes;
  o->width = width;
  o->height = height;
  o->pitch = pitch;
  o->dev = workspace(WS_C, span_bytes);
  if (!o->dev) return 0;
  cudaStream_t s = (cudaStream_t)g_ctx.stream;
  if (width == 0) {
    /* irregular addressing: bring the whole span over so untouched bytes survive the round trip */
    return cuda_ok(cudaMemcpyAsync(o->dev, host, span_bytes, cudaMemcpyHostToDevice, s));
  }
  if (need_old)
    return cuda_ok(cudaMemcpy2DAsync(o->dev, pitch, host, pitch, width, height, cudaMemcpyHostToDevice, s));
  return 1;
}

static int stage_out_end(const out_stage_t *o) {
  cudaStream_t s = (cudaStream_t)g_ctx.stream;
  if (o->width == 0) return cuda_ok(cudaMemcpyAsync(o->host, o->dev, o->span_bytes, cudaMemcpyDeviceToHost, s));
  return cuda_ok(
      cudaMemcpy2DAsync(o->host, o->pitch, o->dev, o->pitch, o->width, o->height, cudaMemcpyDeviceToHost, s));
}

/* ------------------------------------------------------------------ GEMM driver */

/* bf16 x fp8: widen the fp8 operand exactly to bf16 when that makes the tensor-core path usable.
 * Rewrites g->b / tb / strides to the widened copy.  Returns 0 on failure. */
static int widen_fp8_operand(skl_b200_gemm_args *g) {
  const uint64_t K = g->k0 * g->k1;
  if (!(g->ta == SKL_DT_BF16 && (g->tb == SKL_DT_F8E4M3 || g->tb == SKL_DT_F8E5M2) && g->k1 == 1 && g->n1 == 1 &&
        g->m1 == 1 && K != 0 && g_ctx.force_path != SKL_B200_PATH_GENERIC))
    return 1;
  size_t rows = 0, cols = 0, ld_src = 0;
  int k_major = 0;
  if (g->rsb0 == 1 && (g->n0 == 1 || (uint64_t)g->csb0 >= g->k0)) {
    rows = (size_t)g->n0; cols = (size_t)g->k0; ld_src = (size_t)g->csb0; k_major = 1;
  } else if (g->csb0 == 1 && (g->k0 == 1 || (uint64_t)g->rsb0 >= g->n0)) {
    rows = (size_t)g->k0; cols = (size_t)g->n0; ld_src = (size_t)g->rsb0;
  }
  if (rows == 0) return 1;
  /* An n-contiguous B (K x N row-major) is widened into the k-contiguous orientation when the GEMM is large
   * enough to repay the slightly slower transposing pass: the tensor-core kernel runs 6-7 % faster on a
   * k-contiguous B (measured on the c5 shape and on 8192^3). */
  const int transpose = !k_major && g->m0 >= 512 && ((uintptr_t)g->b & 3u) == 0 && ld_src % 4 == 0 &&
                        !getenv("SKL_B200_WIDEN_KEEP_LAYOUT");
  size_t ld_dst = ((transpose ? rows : cols) + 7) & ~(size_t)7; /* 16-byte aligned rows */
  void *wide = workspace(WS_WIDEN, (transpose ? cols : rows) * ld_dst * 2);
  if (!wide) return 0;
  /* Weights declared static (skl_b200_set_static_weights) are widened once: the copy made by the previous call is
   * reused while the same matrix keeps arriving.  Anything else is widened afresh, which also drops the cached copy. */
  const int cached = g->b_static && g_ctx.wide_ptr == wide && g_ctx.wide_src == g->b && g_ctx.wide_rows == rows &&
                     g_ctx.wide_cols == cols && g_ctx.wide_ld == ld_src && g_ctx.wide_fmt == g->tb &&
                     g_ctx.wide_transposed == transpose;
  if (!cached) {
    g_ctx.wide_ptr = 0;
    const int rc = transpose ? skl_b200_launch_cvt_f8_to_bf16_2d_transposed(wide, ld_dst, g->b, ld_src, g->tb, rows, cols,
                                                                            g_ctx.stream)
                             : skl_b200_launch_cvt_f8_to_bf16_2d(wide, ld_dst, g->b, ld_src, g->tb, rows, cols, g_ctx.stream);
    if (!cuda_ok((cudaError_t)rc)) return 0;
    if (g->b_static) {
      g_ctx.wide_ptr = wide;
      g_ctx.wide_src = g->b;
      g_ctx.wide_rows = rows;
      g_ctx.wide_cols = cols;
      g_ctx.wide_ld = ld_src;
      g_ctx.wide_fmt = g->tb;
      g_ctx.wide_transposed = transpose;
    }
  }
  if (transpose) k_major = 1; /* rows of the copy are B's columns: k runs along the unit stride */
  g->b = wide;
  g->tb = SKL_DT_BF16;
  if (k_major) {
    g->rsb0 = 1;
    g->csb0 = (int64_t)ld_dst;
  } else {
    g->rsb0 = (int64_t)ld_dst;
    g->csb0 = 1;
  }
  return 1;
}

/* Chooses the kernel family for a device-resident problem and enqueues it on the library stream. */
/* Does the epilogue read C's previous contents (so that a host C has to be copied in first)? */
static int reads_old_c(const skl_b200_gemm_args *g) {
  if (g->epilogue == SKL_EPI_INT) return g->beta_i != 0;
  if (g->epilogue == SKL_EPI_F64) return g->beta_d != 0.0;
  if (g->epilogue == SKL_EPI_F16ACC) return g->beta_f != 0.0f;
  return g->beta_f != 0.0f || g->activation == SKL_ACT_SWIGLU;
}

static int dispatch_launch(const skl_b200_gemm_args *gin) {
  skl_b200_gemm_args local = *gin, *g = &local;
  local.wait_limit_ms = g_ctx.wait_limit_ms;
  local.debug_skip_loads = g_ctx.debug_skip_loads;
  const uint64_t M = g->m0 * g->m1, N = g->n0 * g->n1, K = g->k0 * g->k1;
  int path = SKL_B200_PATH_GENERIC;
  const int gemv_ok = K != 0 && skl_b200_gemv_i8_supported(g);
  const int tc_ok = K != 0 && skl_b200_gemm_tc_supported(g);
  if (g_ctx.force_path == SKL_B200_PATH_GEMV && gemv_ok) {
    path = SKL_B200_PATH_GEMV;
  } else if (g_ctx.force_path == SKL_B200_PATH_TCGEN05 && tc_ok) {
    path = SKL_B200_PATH_TCGEN05;
  } else if (g_ctx.force_path == 0) {
    if (gemv_ok)
      path = SKL_B200_PATH_GEMV;
    else if (tc_ok && (double)M * (double)N * (double)K >= 32768.0)
      path = SKL_B200_PATH_TCGEN05;
  }
  /* Skinny int8 with more than SKINNY_DP4A_MAX activation rows: dp4a on the CUDA cores cannot keep up
   * with HBM there (two warp instructions per clock per SM against 4*m dp4a per 16 weight bytes), so
   * the problem is handed to the tensor-core kernel transposed -- the weights become the 128-row
   * operand, the activations the (at most 16-column) narrow one, C is written through swapped strides. */
  skl_b200_gemm_args swapped;
  int dp4a_max = SKINNY_DP4A_MAX;
  {
    const char *e = getenv("SKL_B200_SKINNY_DP4A_MAX"); /* tuning override */
    if (e) dp4a_max = atoi(e);
  }
  if (path == SKL_B200_PATH_GEMV && (int)g->m0 > dp4a_max && g_ctx.force_path != SKL_B200_PATH_GEMV) {
    swapped = *g;
    swapped.m0 = g->n0; swapped.n0 = g->m0;
    swapped.a = g->b; swapped.rsa0 = g->csb0; swapped.csa0 = g->rsb0;
    swapped.b = g->a; swapped.rsb0 = g->csa0; swapped.csb0 = g->rsa0;
    swapped.rsc0 = g->csc0; swapped.csc0 = g->rsc0;
    swapped.row_scale = g->col_scale; swapped.col_scale = g->row_scale;
    swapped.col_scale_first = 1; /* keep (acc * row_scale[m]) * col_scale[n] */
    swapped.bias_per_row = 1;    /* the bias is indexed by the original column = the transposed row */
    if (skl_b200_gemm_tc_supported(&swapped)) {
      g = &swapped;
      path = SKL_B200_PATH_TCGEN05;
    }
  }
  int rc = 0;
  const int prof = g_ctx.prof_ev && g_ctx.prof_used < g_ctx.prof_cap;
  if (prof) (void)cudaEventRecord(g_ctx.prof_ev[2 * g_ctx.prof_used], (cudaStream_t)g_ctx.stream);
  if (path == SKL_B200_PATH_GEMV) {
    uint32_t *st = device_status_words();
    if (!st) return 0;
    rc = skl_b200_launch_gemv_i8(g, st, g_ctx.stream);
  } else if (path == SKL_B200_PATH_TCGEN05) {
    uint32_t *st = device_status_words();
    if (!st) return 0;
    rc = skl_b200_launch_gemm_tc(g, st, g_ctx.stream);
  } else {
    rc = skl_b200_launch_gemm_generic(g, g_ctx.stream);
  }
  if (prof) {
    (void)cudaEventRecord(g_ctx.prof_ev[2 * g_ctx.prof_used + 1], (cudaStream_t)g_ctx.stream);
    g_ctx.prof_used++;
  }
  g_ctx.last_path = (skl_b200_path_t)path;
  return cuda_ok((cudaError_t)rc);
}

/* Side streams and events for the row-chunk pipeline (created on first use, kept per thread). */
static int pipe_resources(void) {
  if (g_ctx.pipe_ready) return 1;
  if (!cuda_ok(cudaStreamCreateWithFlags(&g_ctx.s_in, cudaStreamNonBlocking))) return 0;
  if (!cuda_ok(cudaStreamCreateWithFlags(&g_ctx.s_out, cudaStreamNonBlocking))) return 0;
  for (int i = 0; i < PIPE_MAX_CHUNKS; ++i) {
    if (!cuda_ok(cudaEventCreateWithFlags(&g_ctx.ev_in[i], cudaEventDisableTiming))) return 0;
    if (!cuda_ok(cudaEventCreateWithFlags(&g_ctx.ev_done[i], cudaEventDisableTiming))) return 0;
  }
  if (!cuda_ok(cudaEventCreateWithFlags(&g_ctx.ev_ready, cudaEventDisableTiming))) return 0;
  g_ctx.pipe_ready = 1;
  return 1;
}

/* Large row-major problems with A and/or C in host memory: instead of "copy everything in, compute,
 * copy everything out" the rows are cut into chunks and the three phases overlap -- chunk i+1's rows
 * of A travel host-to-device while chunk i is computed and chunk i-1's rows of C travel back, the two
 * copy directions on their own streams so the link runs full duplex.  B, the scale vectors and the
 * fp8 widening are done once, before the first chunk.  Returns 1 if the pipeline ran (successfully or
 * not), 0 if the problem does not qualify and the caller should take the plain route. */
static int run_gemm_pipelined(skl_b200_gemm_args *g, int a_host, int c_host, int *host_any) {
  const uint64_t M = g->m0, N = g->n0, K = g->k0;
  if (g->m1 != 1 || g->n1 != 1 || g->k1 != 1 || K == 0 || M < 4096) return 0;
  if (!a_host && !c_host) return 0;
  const size_t ea = dt_size(g->ta), ec = dt_size(g->tc);
  if (a_host && !(g->csa0 == 1 && (uint64_t)g->rsa0 >= K)) return 0;
  if (!(g->csc0 == 1 && (uint64_t)g->rsc0 >= N)) return 0;
  if ((a_host ? M * K * ea : 0) + (c_host ? M * N * ec : 0) < ((size_t)32 << 20)) return 0;
  {
    const char *e = getenv("SKL_B200_HOST_PIPELINE"); /* 0 disables */
    if (e && atoi(e) == 0) return 0;
  }
  if (!pipe_resources()) return 1;
  *host_any = 1;
  cudaStream_t main_s = (cudaStream_t)g_ctx.stream;

  const void *host_a = g->a;
  void *host_c = g->c;
  uint8_t *dev_a = (uint8_t *)g->a, *dev_c = (uint8_t *)g->c;
  if (a_host) {
    dev_a = (uint8_t *)workspace(WS_A, (size_t)((M - 1) * (uint64_t)g->rsa0 + K) * ea);
    if (!dev_a) return 1;
  }
  if (c_host) {
    dev_c = (uint8_t *)workspace(WS_C, (size_t)((M - 1) * (uint64_t)g->rsc0 + N) * ec);
    if (!dev_c) return 1;
  }
  if (!widen_fp8_operand(g)) return 1;
  /* the copy streams start after everything already queued on the library stream (B, scales, widening) */
  if (!cuda_ok(cudaEventRecord(g_ctx.ev_ready, main_s))) return 1;
  if (!cuda_ok(cudaStreamWaitEvent(g_ctx.s_out, g_ctx.ev_ready, 0))) return 1;

  /* Chunk schedule (whole 256-row tiles): 256, 512, 1024 rows first, so that the device->host direction -- the
   * longer one -- starts as early as possible and then never waits for a chunk, then equal chunks of about
   * 2048 rows. */
  uint64_t sizes[PIPE_MAX_CHUNKS];
  int n_chunks = 0;
  {
    uint64_t left = M;
    for (uint64_t ramp = 256; ramp <= 1024 && left > 4096; ramp *= 2) {
      sizes[n_chunks++] = ramp;
      left -= ramp;
    }
    int rest = (int)((left + 2047) / 2048);
    if (rest > PIPE_MAX_CHUNKS - n_chunks) rest = PIPE_MAX_CHUNKS - n_chunks;
    if (rest < 1) rest = 1;
    const uint64_t rows_per = ((left + rest - 1) / rest + 255) / 256 * 256;
    while (left > 0) {
      const uint64_t r = left < rows_per ? left : rows_per;
      sizes[n_chunks++] = r;
      left -= r;
    }
  }
  const int need_old = reads_old_c(g);
  uint64_t i0 = 0;
  for (int c_idx = 0; c_idx < n_chunks; i0 += sizes[c_idx], ++c_idx) {
    const uint64_t rows = sizes[c_idx];
    const size_t a_off = (size_t)(i0 * (uint64_t)g->rsa0) * ea, c_off = (size_t)(i0 * (uint64_t)g->rsc0) * ec;
    if (a_host) {
      if (!cuda_ok(cudaMemcpy2DAsync(dev_a + a_off, (size_t)g->rsa0 * ea, (const uint8_t *)host_a + a_off,
                                     (size_t)g->rsa0 * ea, (size_t)K * ea, (size_t)rows, cudaMemcpyHostToDevice,
                                     g_ctx.s_in)))
        return 1;
    }
    if (c_host && need_old) {
      if (!cuda_ok(cudaMemcpy2DAsync(dev_c + c_off, (size_t)g->rsc0 * ec, (const uint8_t *)host_c + c_off,
                                     (size_t)g->rsc0 * ec, (size_t)N * ec, (size_t)rows, cudaMemcpyHostToDevice,
                                     g_ctx.s_in)))
        return 1;
    }
    if (a_host || (c_host && need_old)) {
      if (!cuda_ok(cudaEventRecord(g_ctx.ev_in[c_idx], g_ctx.s_in))) return 1;
      if (!cuda_ok(cudaStreamWaitEvent(main_s, g_ctx.ev_in[c_idx], 0))) return 1;
    }
    skl_b200_gemm_args part = *g;
    part.m0 = rows;
    part.a = dev_a + a_off;
    part.c = dev_c + c_off;
    if (part.row_scale) part.row_scale += i0;
    if (!dispatch_launch(&part)) return 1;
    if (c_host) {
      if (!cuda_ok(cudaEventRecord(g_ctx.ev_done[c_idx], main_s))) return 1;
      if (!cuda_ok(cudaStreamWaitEvent(g_ctx.s_out, g_ctx.ev_done[c_idx], 0))) return 1;
      if (!cuda_ok(cudaMemcpy2DAsync((uint8_t *)host_c + c_off, (size_t)g->rsc0 * ec, dev_c + c_off,
                                     (size_t)g->rsc0 * ec, (size_t)N * ec, (size_t)rows, cudaMemcpyDeviceToHost,
                                     g_ctx.s_out)))
        return 1;
    }
  }
  (void)cuda_ok(cudaStreamSynchronize(g_ctx.s_in));
  (void)cuda_ok(cudaStreamSynchronize(g_ctx.s_out));
  return 1;
}

/* Blocked (packed) operands on the tensor cores.  The any-stride kernel serves every blocked description, but
 * for a large problem one pass of the re-layout kernel over each operand (O(MK + KN + MN) bytes at HBM speed) is
 * far cheaper than running O(MNK) work on the CUDA cores: A and B are unblocked into k-major plain workspaces,
 * C (when it is read) into a row-major one, the problem runs as a plain GEMM, and C is blocked back.  The
 * packed GEMM's matrices are exactly m0*m1 x n0*n1 (ref/gemm/gemm_i8rcprc_i8rcprc_i32rcprc.c:10-37), so the
 * way back writes every element of C's blocks and nothing else.  Device pointers only (staged by the caller). */
typedef struct {
  int active;
  skl_b200_gemm_args packed; /* the caller's description, for the way back */
  size_t ldc;
} unblock_t;

static int unblock_operands(skl_b200_gemm_args *g, unblock_t *u) {
  memset(u, 0, sizeof *u);
  if (g->m1 == 1 && g->n1 == 1 && g->k1 == 1) return 1;
  /* panels the tensor-core kernel reads in place (the matrix-engine packed layout with 128-byte rows) */
  if (g_ctx.force_path != SKL_B200_PATH_GENERIC && g->k0 * g->k1 != 0 && skl_b200_gemm_tc_supported(g)) return 1;
  const uint64_t M = g->m0 * g->m1, N = g->n0 * g->n1, K = g->k0 * g->k1;
  double threshold = 16777216.0; /* 2^24 multiply-adds */
  {
    const char *e = getenv("SKL_B200_UNBLOCK_MIN_MNK"); /* tuning / test override */
    if (e) threshold = atof(e);
  }
  if (K == 0 || (double)M * (double)N * (double)K < threshold) return 1;
  if (g_ctx.force_path == SKL_B200_PATH_GENERIC) return 1;
  if (K > 65536 && g->ta == SKL_DT_I8) return 1; /* the tensor path's int8 limit */
  if (g->ta == SKL_DT_F32 || g->ta == SKL_DT_F64) return 1; /* no tensor-core kernel for these */
  if (g->epilogue == SKL_EPI_F16ACC) return 1;               /* nor for an fp16 accumulator */
  const size_t ea = dt_size(g->ta), eb = dt_size(g->tb), ec = dt_size(g->tc);
  const size_t ldk_a = (size_t)((K * ea + 15) / 16 * 16) / ea, ldk_b = (size_t)((K * eb + 15) / 16 * 16) / eb;
  const size_t ldc = (size_t)((N * ec + 15) / 16 * 16) / ec;
  void *pa = workspace(WS_PLAIN_A, (size_t)M * ldk_a * ea);
  void *pb = pa ? workspace(WS_PLAIN_B, (size_t)N * ldk_b * eb) : 0;
  void *pc = pb ? workspace(WS_PLAIN_C, (size_t)M * ldc * ec) : 0;
  if (!pc) return 0;
  /* A: blocks m0 x k0 -> [M][ldk]; B: blocks k0 x n0 -> [N][ldk] (k contiguous) */
  if (!cuda_ok((cudaError_t)skl_b200_launch_unpack(ea, g->m0, g->k0, g->a, (size_t)g->rsa0, (size_t)g->csa0,
                                                   (size_t)g->rsa1, (size_t)g->csa1, M, K, pa, ldk_a, 1, g_ctx.stream)))
    return 0;
  if (!cuda_ok((cudaError_t)skl_b200_launch_unpack(eb, g->k0, g->n0, g->b, (size_t)g->rsb0, (size_t)g->csb0,
                                                   (size_t)g->rsb1, (size_t)g->csb1, K, N, pb, 1, ldk_b, g_ctx.stream)))
    return 0;
  if (reads_old_c(g) &&
      !cuda_ok((cudaError_t)skl_b200_launch_unpack(ec, g->m0, g->n0, g->c, (size_t)g->rsc0, (size_t)g->csc0,
                                                   (size_t)g->rsc1, (size_t)g->csc1, M, N, pc, ldc, 1, g_ctx.stream)))
    return 0;
  u->active = 1;
  u->packed = *g;
  u->ldc = ldc;
  g->m0 = M; g->n0 = N; g->k0 = K;
  g->m1 = g->n1 = g->k1 = 1;
  g->a = pa; g->rsa0 = (int64_t)ldk_a; g->csa0 = 1; g->rsa1 = g->csa1 = 0;
  g->b = pb; g->rsb0 = 1; g->csb0 = (int64_t)ldk_b; g->rsb1 = g->csb1 = 0;
  g->c = pc; g->rsc0 = (int64_t)ldc; g->csc0 = 1; g->rsc1 = g->csc1 = 0;
  g->b_static = 0; /* B was just written on this stream */
  return 1;
}

static int reblock_result(const skl_b200_gemm_args *plain, const unblock_t *u) {
  if (!u->active) return 1;
  const skl_b200_gemm_args *q = &u->packed;
  return cuda_ok((cudaError_t)skl_b200_launch_pack(dt_size(q->tc), (size_t)plain->m0, (size_t)plain->n0, plain->c, u->ldc,
                                                   1, q->m0, q->n0, q->c, (size_t)q->rsc0, (size_t)q->csc0,
                                                   (size_t)q->rsc1, (size_t)q->csc1, 0, g_ctx.stream));
}

static void run_gemm_body(skl_b200_gemm_args *g) {
  g_ctx.last_path = SKL_B200_PATH_NONE;
  const uint64_t M = g->m0 * g->m1, N = g->n0 * g->n1, K = g->k0 * g->k1;
  if (M == 0 || N == 0) {
    return;
  }
  if (!g->c || (K != 0 && (!g->a || !g->b))) {
    set_err(SKL_B200_ERR_INVALID_ARGUMENT);
    return;
  }
  const size_t ea = dt_size(g->ta), eb = dt_size(g->tb), ec = dt_size(g->tc);
  int host_any = 0;
  const int a_host = K != 0 && !on_device(g->a);
  const int c_host = !on_device(g->c);

  /* a B that this call stages itself is written on the stream just before the kernel: never "static" */
  g->b_static = (g_ctx.static_weights && K != 0 && on_device(g->b)) ? 1 : 0;

  /* B and the scale vectors are staged whole in either route */
  if (K != 0 && !on_device(g->b)) {
    host_any = 1;
    size_t bytes = span4(g->k0, g->n0, g->k1, g->n1, g->rsb0, g->csb0, g->rsb1, g->csb1) * eb;
    g->b = stage_in(WS_B, g->b, bytes);
    if (!g->b) return;
  }
  if (g->row_scale && !on_device(g->row_scale)) {
    host_any = 1;
    g->row_scale = (const float *)stage_in(WS_ROW, g->row_scale, (size_t)M * sizeof(float));
    if (!g->row_scale) return;
  }
  if (g->col_scale && !on_device(g->col_scale)) {
    host_any = 1;
    g->col_scale = (const float *)stage_in(WS_COL, g->col_scale, (size_t)N * sizeof(float));
    if (!g->col_scale) return;
  }

  if (g->bias && !on_device(g->bias)) {
    host_any = 1;
    g->bias = (const float *)stage_in(WS_BIAS, g->bias, (size_t)N * sizeof(float));
    if (!g->bias) return;
  }
  float *host_gmax = 0;
  if (g->global_max && !on_device(g->global_max)) {
    host_any = 1;
    host_gmax = g->global_max;
    g->global_max = (float *)stage_in(WS_GMAX, host_gmax, sizeof(float));
    if (!g->global_max) return;
  }

  if (run_gemm_pipelined(g, a_host, c_host, &host_any)) {
    if (host_gmax && g_ctx.status == SKL_B200_OK)
      cuda_ok(cudaMemcpyAsync(host_gmax, g->global_max, sizeof(float), cudaMemcpyDeviceToHost, (cudaStream_t)g_ctx.stream));
    finish(host_any);
    return;
  }

  if (a_host) {
    host_any = 1;
    size_t bytes = span4(g->m0, g->k0, g->m1, g->k1, g->rsa0, g->csa0, g->rsa1, g->csa1) * ea;
    g->a = stage_in(WS_A, g->a, bytes);
    if (!g->a) return;
  }

  /* output */
  out_stage_t out;
  if (c_host) {
    host_any = 1;
    size_t span = span4(g->m0, g->n0, g->m1, g->n1, g->rsc0, g->csc0, g->rsc1, g->csc1) * ec;
    int need_old = reads_old_c(g);
    size_t width = 0, height = 0, pitch = 0;
    if (g->m1 == 1 && g->n1 == 1) {
      if (g->csc0 == 1 && (uint64_t)g->rsc0 >= g->n0) {
        width = (size_t)g->n0 * ec;
        height = (size_t)g->m0;
        pitch = (size_t)g->rsc0 * ec;
      } else if (g->rsc0 == 1 && (uint64_t)g->csc0 >= g->m0) {
        width = (size_t)g->m0 * ec;
        height = (size_t)g->n0;
        pitch = (size_t)g->csc0 * ec;
      }
      if (height == 1) pitch = width; /* a single run: any pitch >= width is legal for the 2-D copy */
    }
    if (!stage_out_begin(&out, g->c, span, width, height, pitch, need_old)) return;
    g->c = out.dev;
  }

  unblock_t unblocked;
  if (!unblock_operands(g, &unblocked)) return;
  if (!widen_fp8_operand(g)) return;
  if (!dispatch_launch(g)) return;
  if (!reblock_result(g, &unblocked)) return;

  if (c_host && !stage_out_end(&out)) return;
  if (host_gmax &&
      !cuda_ok(cudaMemcpyAsync(host_gmax, g->global_max, sizeof(float), cudaMemcpyDeviceToHost, (cudaStream_t)g_ctx.stream)))
    return;
  finish(host_any);
}

static void run_gemm(skl_b200_gemm_args *g) {
  if (!begin_call()) return;
  run_gemm_body(g);
  leave_call();
}

static void gemm_plain(int ta, int tb, int tc, int epi, size_t m, size_t n, size_t k, const void *a,
                       size_t rsa, size_t csa, const void *b, size_t rsb, size_t csb, void *c,
                       size_t rsc, size_t csc, int32_t alpha_i, int32_t beta_i, float alpha_f,
                       float beta_f, const float *row_scale, const float *col_scale, const float *bias,
                       float *global_max, int activation, float act_param) {
  skl_b200_gemm_args g;
  memset(&g, 0, sizeof g);
  g.m0 = m; g.n0 = n; g.k0 = k;
  g.m1 = 1; g.n1 = 1; g.k1 = 1;
  g.ta = ta; g.tb = tb; g.tc = tc;
  g.epilogue = epi;
  g.a = a; g.b = b; g.c = c;
  g.rsa0 = (int64_t)rsa; g.csa0 = (int64_t)csa;
  g.rsb0 = (int64_t)rsb; g.csb0 = (int64_t)csb;
  g.rsc0 = (int64_t)rsc; g.csc0 = (int64_t)csc;
  g.alpha_i = alpha_i; g.beta_i = beta_i;
  g.alpha_f = alpha_f; g.beta_f = beta_f;
  g.row_scale = row_scale; g.col_scale = col_scale;
  g.bias = bias; g.global_max = global_max;
  g.activation = activation; g.act_param = act_param;
  run_gemm(&g);
}

static void gemm_packed(int t, int tc, int epi, size_t m0, size_t n0, size_t k0, size_t m1, size_t n1,
                        size_t k1, const void *a, size_t rsa0, size_t csa0, size_t rsa1, size_t csa1,
                        const void *b, size_t rsb0, size_t csb0, size_t rsb1, size_t csb1, void *c,
                        size_t rsc0, size_t csc0, size_t rsc1, size_t csc1, int32_t alpha_i,
                        int32_t beta_i, float alpha_f, float beta_f) {
  skl_b200_gemm_args g;
  memset(&g, 0, sizeof g);
  g.m0 = m0; g.n0 = n0; g.k0 = k0;
  g.m1 = m1; g.n1 = n1; g.k1 = k1;
  g.ta = t; g.tb = t; g.tc = tc;
  g.epilogue = epi;
  g.a = a; g.b = b; g.c = c;
  g.rsa0 = (int64_t)rsa0; g.csa0 = (int64_t)csa0; g.rsa1 = (int64_t)rsa1; g.csa1 = (int64_t)csa1;
  g.rsb0 = (int64_t)rsb0; g.csb0 = (int64_t)csb0; g.rsb1 = (int64_t)rsb1; g.csb1 = (int64_t)csb1;
  g.rsc0 = (int64_t)rsc0; g.csc0 = (int64_t)csc0; g.rsc1 = (int64_t)rsc1; g.csc1 = (int64_t)csc1;
  g.alpha_i = alpha_i; g.beta_i = beta_i;
  g.alpha_f = alpha_f; g.beta_f = beta_f;
  /* a blocked description with a single block per dimension is a plain matrix */
  run_gemm(&g);
}

/* ------------------------------------------------------------------ GEMM entry points */

void skl_gemm_i8rc_i8rc_i32rc_sm100a(size_t m, size_t n, size_t k, int32_t alpha, const int8_t *a,
                                     size_t rsa, size_t csa, const int8_t *b, size_t rsb, size_t csb,
                                     int32_t beta, int32_t *c, size_t rsc, size_t csc) {
  gemm_plain(SKL_DT_I8, SKL_DT_I8, SKL_DT_I32, SKL_EPI_INT, m, n, k, a, rsa, csa, b, rsb, csb, c, rsc, csc,
             alpha, beta, 0.0f, 0.0f, 0, 0, 0, 0, SKL_ACT_NONE, 0.0f);
}

#define SKL_B200_DEF_GEMM_RC_F32(NAME, TYPE, DT)                                                      \
  void NAME(size_t m, size_t n, size_t k, float alpha, const TYPE *a, size_t rsa, size_t csa,         \
            const TYPE *b, size_t rsb, size_t csb, float beta, float *c, size_t rsc, size_t csc) {    \
    gemm_plain(DT, DT, SKL_DT_F32, SKL_EPI_FLOAT, m, n, k, a, rsa, csa, b, rsb, csb, c, rsc, csc, 0, 0, \
               alpha, beta, 0, 0, 0, 0, SKL_ACT_NONE, 0.0f);                                          \
  }
SKL_B200_DEF_GEMM_RC_F32(skl_gemm_bf16rc_bf16rc_f32rc_sm100a, skl_bf16_t, SKL_DT_BF16)
SKL_B200_DEF_GEMM_RC_F32(skl_gemm_f16rc_f16rc_f32rc_sm100a, skl_f16_t, SKL_DT_F16)
SKL_B200_DEF_GEMM_RC_F32(skl_gemm_f8e4m3rc_f8e4m3rc_f32rc_sm100a, uint8_t, SKL_DT_F8E4M3)
SKL_B200_DEF_GEMM_RC_F32(skl_gemm_f8e5m2rc_f8e5m2rc_f32rc_sm100a, uint8_t, SKL_DT_F8E5M2)

/* row-major A, B, C: column strides are 1 */
void skl_gemm_i8_i8_i32_sm100a(size_t m, size_t n, size_t k, int32_t alpha, const int8_t *a, size_t rsa,
                               const int8_t *b, size_t rsb, int32_t beta, int32_t *c, size_t rsc) {
  skl_gemm_i8rc_i8rc_i32rc_sm100a(m, n, k, alpha, a, rsa, 1, b, rsb, 1, beta, c, rsc, 1);
}
void skl_gemm_bf16_bf16_f32_sm100a(size_t m, size_t n, size_t k, float alpha, const skl_bf16_t *a,
                                   size_t rsa, const skl_bf16_t *b, size_t rsb, float beta, float *c,
                                   size_t rsc) {
  skl_gemm_bf16rc_bf16rc_f32rc_sm100a(m, n, k, alpha, a, rsa, 1, b, rsb, 1, beta, c, rsc, 1);
}
void skl_gemm_f16_f16_f32_sm100a(size_t m, size_t n, size_t k, float alpha, const skl_f16_t *a,
                                 size_t rsa, const skl_f16_t *b, size_t rsb, float beta, float *c,
                                 size_t rsc) {
  skl_gemm_f16rc_f16rc_f32rc_sm100a(m, n, k, alpha, a, rsa, 1, b, rsb, 1, beta, c, rsc, 1);
}

/* column-major A (row stride 1), row-major B and C */
void skl_gemm_i8c_i8_i32_sm100a(size_t m, size_t n, size_t k, int32_t alpha, const int8_t *a, size_t csa,
                                const int8_t *b, size_t rsb, int32_t beta, int32_t *c, size_t rsc) {
  skl_gemm_i8rc_i8rc_i32rc_sm100a(m, n, k, alpha, a, 1, csa, b, rsb, 1, beta, c, rsc, 1);
}
#define SKL_B200_DEF_GEMM_C_F32(NAME, GENERAL, TYPE)                                                  \
  void NAME(size_t m, size_t n, size_t k, float alpha, const TYPE *a, size_t csa, const TYPE *b,      \
            size_t rsb, float beta, float *c, size_t rsc) {                                           \
    GENERAL(m, n, k, alpha, a, 1, csa, b, rsb, 1, beta, c, rsc, 1);                                   \
  }
SKL_B200_DEF_GEMM_C_F32(skl_gemm_bf16c_bf16_f32_sm100a, skl_gemm_bf16rc_bf16rc_f32rc_sm100a, skl_bf16_t)
SKL_B200_DEF_GEMM_C_F32(skl_gemm_f16c_f16_f32_sm100a, skl_gemm_f16rc_f16rc_f32rc_sm100a, skl_f16_t)
SKL_B200_DEF_GEMM_C_F32(skl_gemm_f8e4m3c_f8e4m3_f32_sm100a, skl_gemm_f8e4m3rc_f8e4m3rc_f32rc_sm100a, uint8_t)
SKL_B200_DEF_GEMM_C_F32(skl_gemm_f8e5m2c_f8e5m2_f32_sm100a, skl_gemm_f8e5m2rc_f8e5m2rc_f32rc_sm100a, uint8_t)

/* packed operands */
void skl_gemm_i8rcprc_i8rcprc_i32rcprc_sm100a(size_t m0, size_t n0, size_t k0, size_t m1, size_t n1,
                                              size_t k1, int32_t alpha, const int8_t *a, size_t rsa0,
                                              size_t csa0, size_t rsa1, size_t csa1, const int8_t *b,
                                              size_t rsb0, size_t csb0, size_t rsb1, size_t csb1,
                                              int32_t beta, int32_t *c, size_t rsc0, size_t csc0,
                                              size_t rsc1, size_t csc1) {
  gemm_packed(SKL_DT_I8, SKL_DT_I32, SKL_EPI_INT, m0, n0, k0, m1, n1, k1, a, rsa0, csa0, rsa1, csa1, b, rsb0,
              csb0, rsb1, csb1, c, rsc0, csc0, rsc1, csc1, alpha, beta, 0.0f, 0.0f);
}
#define SKL_B200_DEF_GEMM_PACKED_F32(NAME, TYPE, DT)                                                  \
  void NAME(size_t m0, size_t n0, size_t k0, size_t m1, size_t n1, size_t k1, float alpha,            \
            const TYPE *a, size_t rsa0, size_t csa0, size_t rsa1, size_t csa1, const TYPE *b,         \
            size_t rsb0, size_t csb0, size_t rsb1, size_t csb1, float beta, float *c, size_t rsc0,    \
            size_t csc0, size_t rsc1, size_t csc1) {                                                  \
    gemm_packed(DT, SKL_DT_F32, SKL_EPI_FLOAT, m0, n0, k0, m1, n1, k1, a, rsa0, csa0, rsa1, csa1, b,  \
                rsb0, csb0, rsb1, csb1, c, rsc0, csc0, rsc1, csc1, 0, 0, alpha, beta);                \
  }
SKL_B200_DEF_GEMM_PACKED_F32(skl_gemm_bf16rcprc_bf16rcprc_f32rcprc_sm100a, skl_bf16_t, SKL_DT_BF16)
SKL_B200_DEF_GEMM_PACKED_F32(skl_gemm_f16rcprc_f16rcprc_f32rcprc_sm100a, skl_f16_t, SKL_DT_F16)
SKL_B200_DEF_GEMM_PACKED_F32(skl_gemm_f8e4m3rcprc_f8e4m3rcprc_f32rcprc_sm100a, uint8_t, SKL_DT_F8E4M3)
SKL_B200_DEF_GEMM_PACKED_F32(skl_gemm_f8e5m2rcprc_f8e5m2rcprc_f32rcprc_sm100a, uint8_t, SKL_DT_F8E5M2)

/* Operands packed for the matrix engine (src/gemm/gemm_i8c_i8_i32_xsfmm32a8i.h:62-100 and siblings): the general
 * packed GEMM with m0 = n0 = TE, k0 = 1, (rsa0, csa0) = (1, 0), (rsb0, csb0) = (0, 1).  With TE = 128 the tensor-core
 * kernel reads these panels directly (see skl_b200_gemm_tc_supported): no unblocking pass. */
size_t skl_b200_te(void) { return SKL_B200_TE; }

void skl_gemm_i8rcptex1c_i8rcp1xte_i32rcptexterc_sm100a(size_t m1, size_t n1, size_t k, int32_t alpha, const int8_t *a,
                                                        size_t rsa1, size_t csa1, const int8_t *b, size_t rsb1,
                                                        size_t csb1, int32_t beta, int32_t *c, size_t rsc0, size_t csc0,
                                                        size_t rsc1, size_t csc1) {
  gemm_packed(SKL_DT_I8, SKL_DT_I32, SKL_EPI_INT, SKL_B200_TE, SKL_B200_TE, 1, m1, n1, k, a, 1, 0, rsa1, csa1, b, 0, 1,
              rsb1, csb1, c, rsc0, csc0, rsc1, csc1, alpha, beta, 0.0f, 0.0f);
}
#define SKL_B200_DEF_GEMM_TE_F32(NAME, TYPE, DT)                                                                  \
  void NAME(size_t m1, size_t n1, size_t k, float alpha, const TYPE *a, size_t rsa1, size_t csa1, const TYPE *b,   \
            size_t rsb1, size_t csb1, float beta, float *c, size_t rsc0, size_t csc0, size_t rsc1, size_t csc1) {  \
    gemm_packed(DT, SKL_DT_F32, SKL_EPI_FLOAT, SKL_B200_TE, SKL_B200_TE, 1, m1, n1, k, a, 1, 0, rsa1, csa1, b, 0, 1, \
                rsb1, csb1, c, rsc0, csc0, rsc1, csc1, 0, 0, alpha, beta);                                         \
  }
SKL_B200_DEF_GEMM_TE_F32(skl_gemm_bf16rcptex1c_bf16rcp1xte_f32rcptexterc_sm100a, skl_bf16_t, SKL_DT_BF16)
SKL_B200_DEF_GEMM_TE_F32(skl_gemm_f16rcptex1c_f16rcp1xte_f32rcptexterc_sm100a, skl_f16_t, SKL_DT_F16)
SKL_B200_DEF_GEMM_TE_F32(skl_gemm_f8e4m3rcptex1c_f8e4m3rcp1xte_f32rcptexterc_sm100a, uint8_t, SKL_DT_F8E4M3)
SKL_B200_DEF_GEMM_TE_F32(skl_gemm_f8e5m2rcptex1c_f8e5m2rcp1xte_f32rcptexterc_sm100a, uint8_t, SKL_DT_F8E5M2)
SKL_B200_DEF_GEMM_TE_F32(skl_gemm_f32rcptex1c_f32rcp1xte_f32rcptexterc_sm100a, float, SKL_DT_F32)

/* src/gemm/gemm_i8rcp1x4_i8p4x1c_i32_xsfvqdotq.h:43-52: the general packed GEMM with m0 = n0 = 1, k0 = 4 */
void skl_gemm_i8rcp1x4_i8p4x1c_i32_sm100a(size_t m, size_t n, size_t k1, int32_t alpha, const int8_t *a, size_t rsa1,
                                          size_t csa1, const int8_t *b, size_t rsb1, int32_t beta, int32_t *c,
                                          size_t rsc) {
  skl_gemm_i8rcprc_i8rcprc_i32rcprc_sm100a(1, 1, 4, m, n, k1, alpha, a, 0, 1, rsa1, csa1, b, 1, 0, rsb1, 4, beta, c, 0, 0,
                                           rsc, 1);
}

/* fp32 and fp64 GEMMs (ref/gemm/gemm_f32rc_f32rc_f32rc.c:9-22, gemm_f64rc_f64rc_f64rc.c:9-22 and the packed forms):
 * on the any-stride kernel, one accumulator per output, k ascending, product and sum rounded separately. */
void skl_gemm_f32rc_f32rc_f32rc_sm100a(size_t m, size_t n, size_t k, float alpha, const float *a, size_t rsa,
                                       size_t csa, const float *b, size_t rsb, size_t csb, float beta, float *c,
                                       size_t rsc, size_t csc) {
  gemm_plain(SKL_DT_F32, SKL_DT_F32, SKL_DT_F32, SKL_EPI_FLOAT, m, n, k, a, rsa, csa, b, rsb, csb, c, rsc, csc, 0, 0,
             alpha, beta, 0, 0, 0, 0, SKL_ACT_NONE, 0.0f);
}
void skl_gemm_f32rcprc_f32rcprc_f32rcprc_sm100a(size_t m0, size_t n0, size_t k0, size_t m1, size_t n1, size_t k1,
                                                float alpha, const float *a, size_t rsa0, size_t csa0, size_t rsa1,
                                                size_t csa1, const float *b, size_t rsb0, size_t csb0, size_t rsb1,
                                                size_t csb1, float beta, float *c, size_t rsc0, size_t csc0,
                                                size_t rsc1, size_t csc1) {
  gemm_packed(SKL_DT_F32, SKL_DT_F32, SKL_EPI_FLOAT, m0, n0, k0, m1, n1, k1, a, rsa0, csa0, rsa1, csa1, b, rsb0, csb0,
              rsb1, csb1, c, rsc0, csc0, rsc1, csc1, 0, 0, alpha, beta);
}
void skl_gemm_f64rcprc_f64rcprc_f64rcprc_sm100a(size_t m0, size_t n0, size_t k0, size_t m1, size_t n1, size_t k1,
                                                double alpha, const double *a, size_t rsa0, size_t csa0,
                                                size_t rsa1, size_t csa1, const double *b, size_t rsb0,
                                                size_t csb0, size_t rsb1, size_t csb1, double beta, double *c,
                                                size_t rsc0, size_t csc0, size_t rsc1, size_t csc1) {
  skl_b200_gemm_args g;
  memset(&g, 0, sizeof g);
  g.m0 = m0; g.n0 = n0; g.k0 = k0;
  g.m1 = m1; g.n1 = n1; g.k1 = k1;
  g.ta = SKL_DT_F64; g.tb = SKL_DT_F64; g.tc = SKL_DT_F64;
  g.epilogue = SKL_EPI_F64;
  g.a = a; g.b = b; g.c = c;
  g.rsa0 = (int64_t)rsa0; g.csa0 = (int64_t)csa0; g.rsa1 = (int64_t)rsa1; g.csa1 = (int64_t)csa1;
  g.rsb0 = (int64_t)rsb0; g.csb0 = (int64_t)csb0; g.rsb1 = (int64_t)rsb1; g.csb1 = (int64_t)csb1;
  g.rsc0 = (int64_t)rsc0; g.csc0 = (int64_t)csc0; g.rsc1 = (int64_t)rsc1; g.csc1 = (int64_t)csc1;
  g.alpha_d = alpha; g.beta_d = beta;
  run_gemm(&g);
}
void skl_gemm_f64rc_f64rc_f64rc_sm100a(size_t m, size_t n, size_t k, double alpha, const double *a, size_t rsa,
                                       size_t csa, const double *b, size_t rsb, size_t csb, double beta, double *c,
                                       size_t rsc, size_t csc) {
  skl_gemm_f64rcprc_f64rcprc_f64rcprc_sm100a(m, n, k, 1, 1, 1, alpha, a, rsa, csa, 0, 0, b, rsb, csb, 0, 0, beta, c, rsc,
                                             csc, 0, 0);
}

/* fp16 operands with an fp16 accumulator and fp16 C (ref/gemm/gemm_f16rc_f16rc_f16rc.c:9-22 and
 * gemm_f16rcprc_f16rcprc_f16rcprc.c): on the any-stride kernel, every statement of the reference evaluated in fp32
 * and rounded to fp16 once.  The *_f32scalars forms take alpha and beta as floats (rounded to fp16 first) for
 * callers whose language binding cannot pass a 16-bit float by value. */
static float as_f16_value(float x) { return (float)(skl_f16_t)x; }

void skl_gemm_f16rcprc_f16rcprc_f16rcprc_f32scalars_sm100a(size_t m0, size_t n0, size_t k0, size_t m1, size_t n1,
                                                           size_t k1, float alpha, const skl_f16_t *a, size_t rsa0,
                                                           size_t csa0, size_t rsa1, size_t csa1, const skl_f16_t *b,
                                                           size_t rsb0, size_t csb0, size_t rsb1, size_t csb1,
                                                           float beta, skl_f16_t *c, size_t rsc0, size_t csc0,
                                                           size_t rsc1, size_t csc1) {
  gemm_packed(SKL_DT_F16, SKL_DT_F16, SKL_EPI_F16ACC, m0, n0, k0, m1, n1, k1, a, rsa0, csa0, rsa1, csa1, b, rsb0, csb0,
              rsb1, csb1, c, rsc0, csc0, rsc1, csc1, 0, 0, as_f16_value(alpha), as_f16_value(beta));
}
void skl_gemm_f16rcprc_f16rcprc_f16rcprc_sm100a(size_t m0, size_t n0, size_t k0, size_t m1, size_t n1, size_t k1,
                                                skl_f16_t alpha, const skl_f16_t *a, size_t rsa0, size_t csa0,
                                                size_t rsa1, size_t csa1, const skl_f16_t *b, size_t rsb0, size_t csb0,
                                                size_t rsb1, size_t csb1, skl_f16_t beta, skl_f16_t *c, size_t rsc0,
                                                size_t csc0, size_t rsc1, size_t csc1) {
  skl_gemm_f16rcprc_f16rcprc_f16rcprc_f32scalars_sm100a(m0, n0, k0, m1, n1, k1, (float)alpha, a, rsa0, csa0, rsa1, csa1,
                                                        b, rsb0, csb0, rsb1, csb1, (float)beta, c, rsc0, csc0, rsc1,
                                                        csc1);
}
void skl_gemm_f16rc_f16rc_f16rc_f32scalars_sm100a(size_t m, size_t n, size_t k, float alpha, const skl_f16_t *a,
                                                  size_t rsa, size_t csa, const skl_f16_t *b, size_t rsb, size_t csb,
                                                  float beta, skl_f16_t *c, size_t rsc, size_t csc) {
  skl_gemm_f16rcprc_f16rcprc_f16rcprc_f32scalars_sm100a(m, n, k, 1, 1, 1, alpha, a, rsa, csa, 0, 0, b, rsb, csb, 0, 0,
                                                        beta, c, rsc, csc, 0, 0);
}
void skl_gemm_f16rc_f16rc_f16rc_sm100a(size_t m, size_t n, size_t k, skl_f16_t alpha, const skl_f16_t *a, size_t rsa,
                                       size_t csa, const skl_f16_t *b, size_t rsb, size_t csb, skl_f16_t beta,
                                       skl_f16_t *c, size_t rsc, size_t csc) {
  skl_gemm_f16rc_f16rc_f16rc_f32scalars_sm100a(m, n, k, (float)alpha, a, rsa, csa, b, rsb, csb, (float)beta, c, rsc,
                                               csc);
}

/* extended epilogue */
static int is_f8(int t) { return t == SKL_DT_F8E4M3 || t == SKL_DT_F8E5M2; }

void skl_gemm_fused_sm100a(size_t m, size_t n, size_t k, skl_b200_dtype_t ta, const void *a, size_t rsa,
                           size_t csa, skl_b200_dtype_t tb, const void *b, size_t rsb, size_t csb,
                           const skl_b200_fused_t *f, skl_b200_dtype_t tc, void *c, size_t rsc, size_t csc) {
  if (!f) {
    g_ctx.status = SKL_B200_ERR_INVALID_ARGUMENT;
    g_ctx.cuda_err[0] = 0;
    return;
  }
  int pair_ok = (ta == SKL_B200_I8 && tb == SKL_B200_I8) || (is_f8(ta) && is_f8(tb)) ||
                (ta == SKL_B200_BF16 && tb == SKL_B200_BF16) || (ta == SKL_B200_F16 && tb == SKL_B200_F16) ||
                (ta == SKL_B200_BF16 && is_f8(tb));
  int out_ok = tc == SKL_B200_F32 || tc == SKL_B200_BF16 || tc == SKL_B200_F16 || tc == SKL_B200_F8E4M3 ||
               tc == SKL_B200_I8;
  if (!pair_ok || !out_ok) {
    g_ctx.status = SKL_B200_ERR_UNSUPPORTED;
    g_ctx.cuda_err[0] = 0;
    return;
  }
  if (f->activation < SKL_ACT_NONE || f->activation > SKL_ACT_SWIGLU ||
      (f->activation == SKL_ACT_SWIGLU && f->beta != 0.0f)) {
    g_ctx.status = SKL_B200_ERR_INVALID_ARGUMENT;
    g_ctx.cuda_err[0] = 0;
    return;
  }
  gemm_plain((int)ta, (int)tb, (int)tc, SKL_EPI_FLOAT, m, n, k, a, rsa, csa, b, rsb, csb, c, rsc, csc, 0, 0,
             f->alpha, f->beta, f->row_scale, f->col_scale, f->bias, f->global_max, f->activation, f->act_param);
}

void skl_gemm_ex_sm100a(size_t m, size_t n, size_t k, skl_b200_dtype_t ta, const void *a, size_t rsa,
                        size_t csa, skl_b200_dtype_t tb, const void *b, size_t rsb, size_t csb,
                        float alpha, const float *row_scale, const float *col_scale, float beta,
                        skl_b200_dtype_t tc, void *c, size_t rsc, size_t csc) {
  skl_b200_fused_t f;
  f.alpha = alpha;
  f.beta = beta;
  f.row_scale = row_scale;
  f.col_scale = col_scale;
  f.bias = 0;
  f.global_max = 0;
  f.activation = SKL_B200_ACT_NONE;
  f.act_param = 0.0f;
  skl_gemm_fused_sm100a(m, n, k, ta, a, rsa, csa, tb, b, rsb, csb, &f, tc, c, rsc, csc);
}

/* ------------------------------------------------------------------ cvt */

static void run_cvt_to_f8_body(void *dst, const void *src, int src_type, int fmt, int sat, float scale, size_t n) {
  if (n == 0) return;
  if (!dst || !src) { set_err(SKL_B200_ERR_INVALID_ARGUMENT); return; }
  int host_any = 0;
  const void *dsrc = src;
  void *ddst = dst;
  if (!on_device(src)) {
    host_any = 1;
    dsrc = stage_in(WS_A, src, n * dt_size(src_type));
    if (!dsrc) return;
  }
  int dst_host = !on_device(dst);
  if (dst_host) {
    host_any = 1;
    ddst = workspace(WS_C, n);
    if (!ddst) return;
  }
  if (!cuda_ok((cudaError_t)skl_b200_launch_cvt_to_f8(ddst, dsrc, src_type, fmt, sat, scale, n, g_ctx.stream)))
    return;
  if (dst_host &&
      !cuda_ok(cudaMemcpyAsync(dst, ddst, n, cudaMemcpyDeviceToHost, (cudaStream_t)g_ctx.stream)))
    return;
  finish(host_any);
}

static void run_cvt_to_f8(void *dst, const void *src, int src_type, int fmt, int sat, float scale, size_t n) {
  if (!begin_call()) return;
  run_cvt_to_f8_body(dst, src, src_type, fmt, sat, scale, n);
  leave_call();
}

#define SKL_B200_DEF_CVT_TO_F8(NAME, SRC_T, SRC_DT, FMT, SAT)                           \
  void NAME(uint8_t *pDst, const SRC_T *pSrc, float scaling_factor, size_t n) {         \
    run_cvt_to_f8(pDst, pSrc, SRC_DT, FMT, SAT, scaling_factor, n);                     \
  }
SKL_B200_DEF_CVT_TO_F8(skl_cvt_f32_f8e4m3_sm100a, float, SKL_DT_F32, SKL_DT_F8E4M3, 0)
SKL_B200_DEF_CVT_TO_F8(skl_cvt_sat_f32_f8e4m3_sm100a, float, SKL_DT_F32, SKL_DT_F8E4M3, 1)
SKL_B200_DEF_CVT_TO_F8(skl_cvt_f32_f8e5m2_sm100a, float, SKL_DT_F32, SKL_DT_F8E5M2, 0)
SKL_B200_DEF_CVT_TO_F8(skl_cvt_sat_f32_f8e5m2_sm100a, float, SKL_DT_F32, SKL_DT_F8E5M2, 1)
SKL_B200_DEF_CVT_TO_F8(skl_cvt_bf16_f8e4m3_sm100a, skl_bf16_t, SKL_DT_BF16, SKL_DT_F8E4M3, 0)
SKL_B200_DEF_CVT_TO_F8(skl_cvt_sat_bf16_f8e4m3_sm100a, skl_bf16_t, SKL_DT_BF16, SKL_DT_F8E4M3, 1)
SKL_B200_DEF_CVT_TO_F8(skl_cvt_bf16_f8e5m2_sm100a, skl_bf16_t, SKL_DT_BF16, SKL_DT_F8E5M2, 0)
SKL_B200_DEF_CVT_TO_F8(skl_cvt_sat_bf16_f8e5m2_sm100a, skl_bf16_t, SKL_DT_BF16, SKL_DT_F8E5M2, 1)

/* widening directions: mode 0 = fp8 -> bf16 (out 2 bytes/elt, in 1), mode 1 = fp4 -> fp8 (out 1, in 1/2) */
static void run_cvt_widen_body(void *dst, const void *src, int mode, int fmt, size_t n) {
  if (n == 0) return;
  if (!dst || !src) { set_err(SKL_B200_ERR_INVALID_ARGUMENT); return; }
  const size_t in_bytes = mode == 0 ? n : (n + 1) / 2, out_bytes = mode == 0 ? 2 * n : n;
  int host_any = 0;
  const void *dsrc = src;
  void *ddst = dst;
  if (!on_device(src)) {
    host_any = 1;
    dsrc = stage_in(WS_A, src, in_bytes);
    if (!dsrc) return;
  }
  int dst_host = !on_device(dst);
  if (dst_host) {
    host_any = 1;
    ddst = workspace(WS_C, out_bytes);
    if (!ddst) return;
  }
  int rc = mode == 0 ? skl_b200_launch_cvt_f8_to_bf16(ddst, dsrc, fmt, n, g_ctx.stream)
                     : skl_b200_launch_cvt_f4_to_f8e4m3(ddst, dsrc, n, g_ctx.stream);
  if (!cuda_ok((cudaError_t)rc)) return;
  if (dst_host &&
      !cuda_ok(cudaMemcpyAsync(dst, ddst, out_bytes, cudaMemcpyDeviceToHost, (cudaStream_t)g_ctx.stream)))
    return;
  finish(host_any);
}

static void run_cvt_widen(void *dst, const void *src, int mode, int fmt, size_t n) {
  if (!begin_call()) return;
  run_cvt_widen_body(dst, src, mode, fmt, n);
  leave_call();
}

void skl_cvt_f8e4m3_bf16_sm100a(skl_bf16_t *pDst, const uint8_t *pSrc, size_t n) {
  run_cvt_widen(pDst, pSrc, 0, SKL_DT_F8E4M3, n);
}
void skl_cvt_f8e5m2_bf16_sm100a(skl_bf16_t *pDst, const uint8_t *pSrc, size_t n) {
  run_cvt_widen(pDst, pSrc, 0, SKL_DT_F8E5M2, n);
}
void skl_cvt_f4e2m1_f8e4m3_sm100a(uint8_t *pDst, const uint8_t *pSrc, size_t n) {
  run_cvt_widen(pDst, pSrc, 1, 0, n);
}

/* ------------------------------------------------------------------ MX-FP4 GEMM (block-scaled E2M1) */

/* Device operands with TMA-compatible packed rows run on the block-scaled tensor-core kernel; otherwise both operands
 * are widened exactly to bf16 (element x 2^(scale - 127)) into workspaces and multiplied by the bf16 tensor-core path
 * with fp32 accumulation. */
void skl_gemm_mxf4e2m1_mxf4e2m1_f32_sm100a(size_t m, size_t n, size_t k, float alpha, const uint8_t *a, size_t rsa,
                                           const uint8_t *sa, size_t rssa, const uint8_t *b, size_t csb,
                                           const uint8_t *sb, size_t cssb, float beta, float *c, size_t rsc) {
  if (!begin_call()) return;
  do {
    if ((k & 31u) != 0 || rsa < k / 2 || csb < k / 2 || rssa < k / 32 || cssb < k / 32 || m >= (1ull << 31) ||
        n >= (1ull << 31) || k >= (1ull << 31)) {
      set_err(SKL_B200_ERR_INVALID_ARGUMENT);
      break;
    }
    if (m == 0 || n == 0) break;
    const size_t kb = k / 32;
    void *wa = 0, *wb = 0;
    if (k > 0) {
      const void *da = a, *dsa = sa, *db = b, *dsb = sb;
      if (!on_device(a)) da = stage_in(WS_A, a, (m - 1) * rsa + k / 2);
      if (!on_device(sa)) dsa = stage_in(WS_ROW, sa, (m - 1) * rssa + kb);
      if (!on_device(b)) db = stage_in(WS_B, b, (n - 1) * csb + k / 2);
      if (!on_device(sb)) dsb = stage_in(WS_COL, sb, (n - 1) * cssb + kb);
      if (!da || !dsa || !db || !dsb) break;
      /* the block-scaled tensor-core instruction, when the packed rows are TMA-compatible and C is on the device */
      {
        const char *e = getenv("SKL_B200_MXF4_NATIVE"); /* 0: always widen to bf16 */
        const int native = !(e && atoi(e) == 0) && g_ctx.force_path != SKL_B200_PATH_GENERIC && on_device(c) &&
                           skl_b200_gemm_mxf4_supported(da, (int64_t)rsa, db, (int64_t)csb, (int64_t)m, (int64_t)n, (int64_t)k);
        if (native) {
          uint32_t *st = device_status_words();
          if (!st) break;
          void *psa = workspace(WS_PLAIN_A, skl_b200_gemm_mxf4_scale_bytes((int64_t)m, (int64_t)k));
          void *psb = psa ? workspace(WS_PLAIN_B, skl_b200_gemm_mxf4_scale_bytes((int64_t)n, (int64_t)k)) : 0;
          if (!psb) break;
          if (cuda_ok((cudaError_t)skl_b200_launch_gemm_mxf4(da, (int64_t)rsa, dsa, (int64_t)rssa, db, (int64_t)csb, dsb,
                                                              (int64_t)cssb, c, (int64_t)rsc, (int64_t)m, (int64_t)n,
                                                              (int64_t)k, alpha, beta, psa, psb, g_ctx.wait_limit_ms, st,
                                                              g_ctx.stream))) {
            g_ctx.last_path = SKL_B200_PATH_TCGEN05;
            finish(!on_device(a) || !on_device(b) || !on_device(sa) || !on_device(sb));
          }
          break;
        }
      }
      wa = workspace(WS_PLAIN_A, m * k * 2);
      wb = wa ? workspace(WS_PLAIN_B, n * k * 2) : 0;
      if (!wb) break;
      if (!cuda_ok((cudaError_t)skl_b200_launch_cvt_mxf4_to_bf16(wa, k, da, rsa, dsa, rssa, m, kb, g_ctx.stream))) break;
      if (!cuda_ok((cudaError_t)skl_b200_launch_cvt_mxf4_to_bf16(wb, k, db, csb, dsb, cssb, n, kb, g_ctx.stream))) break;
    }
    skl_b200_gemm_args g;
    memset(&g, 0, sizeof g);
    g.m0 = m; g.n0 = n; g.k0 = k;
    g.m1 = 1; g.n1 = 1; g.k1 = 1;
    g.ta = SKL_DT_BF16; g.tb = SKL_DT_BF16; g.tc = SKL_DT_F32;
    g.epilogue = SKL_EPI_FLOAT;
    g.a = wa; g.b = wb; g.c = c;
    g.rsa0 = (int64_t)k; g.csa0 = 1;
    g.rsb0 = 1; g.csb0 = (int64_t)k;
    g.rsc0 = (int64_t)rsc; g.csc0 = 1;
    g.alpha_f = alpha; g.beta_f = beta;
    run_gemm_body(&g);
  } while (0);
  leave_call();
}

/* ------------------------------------------------------------------ pack / unpack / transpose */

/* op: 0 pack, 1 unpack, 2 transpose.  `plain` is the 2-D side, `blk` the blocked side. */
static void run_relayout_body(int op, size_t esize, size_t m, size_t n, const void *src, void *dst, size_t rs,
                         size_t cs, size_t m0, size_t n0, size_t rs0, size_t cs0, size_t rs1, size_t cs1,
                         uint32_t pad) {
  if (op != 2 && (m0 == 0 || n0 == 0)) return; /* ref/pack/unpack_e8rcprc_e8rc.c:16-18 */
  if (m == 0 || n == 0) return;
  if (!src || !dst) { set_err(SKL_B200_ERR_INVALID_ARGUMENT); return; }
  size_t src_span, dst_span;
  if (op == 0) {
    size_t m1 = (m + m0 - 1) / m0, n1 = (n + n0 - 1) / n0;
    src_span = span4(m, n, 1, 1, (int64_t)rs, (int64_t)cs, 0, 0);
    dst_span = span4(m0, n0, m1, n1, (int64_t)rs0, (int64_t)cs0, (int64_t)rs1, (int64_t)cs1);
  } else if (op == 1) {
    size_t m1 = (m + m0 - 1) / m0, n1 = (n + n0 - 1) / n0;
    src_span = span4(m0, n0, m1, n1, (int64_t)rs0, (int64_t)cs0, (int64_t)rs1, (int64_t)cs1);
    dst_span = span4(m, n, 1, 1, (int64_t)rs, (int64_t)cs, 0, 0);
  } else {
    src_span = span4(m, n, 1, 1, (int64_t)rs, 1, 0, 0);
    dst_span = span4(n, m, 1, 1, (int64_t)rs0, 1, 0, 0); /* rs0 carries rsat */
  }
  int host_any = 0;
  const void *dsrc = src;
  void *ddst = dst;
  if (!on_device(src)) {
    host_any = 1;
    dsrc = stage_in(WS_A, src, src_span * esize);
    if (!dsrc) return;
  }
  out_stage_t out;
  int dst_host = !on_device(dst);
  if (dst_host) {
    host_any = 1;
    /* destinations may have gaps the operation must not disturb: round-trip the whole span */
    if (!stage_out_begin(&out, dst, dst_span * esize, 0, 0, 0, 1)) return;
    ddst = out.dev;
  }
  int rc;
  if (op == 0)
    rc = skl_b200_launch_pack(esize, m, n, dsrc, rs, cs, m0, n0, ddst, rs0, cs0, rs1, cs1, pad, g_ctx.stream);
  else if (op == 1)
    rc = skl_b200_launch_unpack(esize, m0, n0, dsrc, rs0, cs0, rs1, cs1, m, n, ddst, rs, cs, g_ctx.stream);
  else
    rc = skl_b200_launch_transpose(esize, m, n, dsrc, rs, ddst, rs0, g_ctx.stream);
  if (!cuda_ok((cudaError_t)rc)) return;
  if (dst_host && !stage_out_end(&out)) return;
  finish(host_any);
}

static void run_relayout(int op, size_t esize, size_t m, size_t n, const void *src, void *dst, size_t rs,
                         size_t cs, size_t m0, size_t n0, size_t rs0, size_t cs0, size_t rs1, size_t cs1,
                         uint32_t pad) {
  if (!begin_call()) return;
  run_relayout_body(op, esize, m, n, src, dst, rs, cs, m0, n0, rs0, cs0, rs1, cs1, pad);
  leave_call();
}

#define SKL_B200_DEF_PACK(BITS, TYPE)                                                                  \
  void skl_pack_e##BITS##rc_e##BITS##rcprc_sm100a(size_t m, size_t n, const TYPE *SKL_RESTRICT src,    \
                                                  size_t rs, size_t cs, size_t m0, size_t n0,          \
                                                  TYPE *SKL_RESTRICT dst, size_t rs0, size_t cs0,      \
                                                  size_t rs1, size_t cs1, TYPE pad) {                  \
    run_relayout(0, sizeof(TYPE), m, n, src, dst, rs, cs, m0, n0, rs0, cs0, rs1, cs1, (uint32_t)pad);  \
  }                                                                                                    \
  void skl_transpose_e##BITS##_sm100a(size_t m, size_t n, const TYPE *SKL_RESTRICT a, size_t rsa,      \
                                      TYPE *SKL_RESTRICT at, size_t rsat) {                            \
    run_relayout(2, sizeof(TYPE), m, n, a, at, rsa, 1, 1, 1, rsat, 1, 0, 0, 0);                        \
  }
SKL_B200_DEF_PACK(8, uint8_t)
SKL_B200_DEF_PACK(16, uint16_t)
SKL_B200_DEF_PACK(32, uint32_t)

/* Gathered column shards -> row-major matrix (see the header).  Equal shards: the buffer is a packed matrix of
 * 1 x parts blocks of m x n/parts, unpacked in one launch; otherwise each shard is a 1 x 1 "packed" matrix. */
void skl_b200_unshard_columns_sm100a(size_t esize, size_t m, size_t n, size_t parts, size_t align,
                                     const void *gathered, size_t part_stride, void *dst, size_t rsd) {
  if ((esize != 1 && esize != 2 && esize != 4) || parts == 0 || rsd < n) {
    g_ctx.status = SKL_B200_ERR_INVALID_ARGUMENT;
    g_ctx.cuda_err[0] = 0;
    return;
  }
  size_t start0 = 0, count0 = 0;
  int equal = 1;
  skl_b200_shard_columns(n, parts, 0, align, &start0, &count0);
  for (size_t g = 1; g < parts && equal; ++g) {
    size_t s_g = 0, c_g = 0;
    skl_b200_shard_columns(n, parts, g, align, &s_g, &c_g);
    if (c_g != count0 || s_g != g * count0) equal = 0;
  }
  if (equal) {
    run_relayout(1, esize, m, n, gathered, dst, rsd, 1, m, count0, count0, 1, 0, part_stride, 0);
    return;
  }
  for (size_t g = 0; g < parts; ++g) {
    size_t s_g = 0, c_g = 0;
    skl_b200_shard_columns(n, parts, g, align, &s_g, &c_g);
    if (c_g == 0) continue;
    run_relayout(1, esize, m, c_g, (const uint8_t *)gathered + g * part_stride * esize, (uint8_t *)dst + s_g * esize, rsd,
                 1, m, c_g, c_g, 1, 0, 0, 0);
    if (g_ctx.status != SKL_B200_OK) return;
  }
}

/* src/pack/pack_e16_xsfmmbase.h:20-51: the general pack with (m0, n0) = (TE, 1), (rs0, cs0) = (1, 0), row-major src */
#define SKL_B200_DEF_PACK_TE(BITS, TYPE)                                                                       \
  void skl_pack_e##BITS##_e##BITS##rcptex1c_sm100a(size_t m, size_t n, const TYPE *src, size_t rs, TYPE *dst,  \
                                                   size_t rs1, size_t cs1, TYPE pad) {                         \
    run_relayout(0, sizeof(TYPE), m, n, src, dst, rs, 1, SKL_B200_TE, 1, 1, 0, rs1, cs1, (uint32_t)pad);       \
  }
SKL_B200_DEF_PACK_TE(8, uint8_t)
SKL_B200_DEF_PACK_TE(16, uint16_t)
SKL_B200_DEF_PACK_TE(32, uint32_t)

void skl_unpack_e8rcprc_e8rc_sm100a(size_t m0, size_t n0, const uint8_t *SKL_RESTRICT src, size_t rs0,
                                    size_t cs0, size_t rs1, size_t cs1, size_t m, size_t n,
                                    uint8_t *SKL_RESTRICT dst, size_t rs, size_t cs) {
  run_relayout(1, 1, m, n, src, dst, rs, cs, m0, n0, rs0, cs0, rs1, cs1, 0);
}
