// cvt.cu -- OCP fp8 / fp4 conversion kernels.
//
// dst[i] = narrow(src[i] * scale), with the product rounded to fp32 first, exactly as
// ref/cvt/cvt_ofp8.c:174-242 defines it; the widening directions are exact.  All kernels are
// HBM-bound streaming kernels: 16 elements per thread per step, 16-byte loads and stores whenever the
// pointers allow, a grid-stride loop over a grid sized from the SM count.
// Algorithmic bytes per element: fp32->fp8 5, bf16->fp8 3, fp8->bf16 3, fp4->fp8 1.5.
#include "numerics.cuh"

namespace sklb {
namespace {

constexpr int CVT_THREADS = 256;

inline int cvt_grid(size_t n, int per_thread) {
  static int sms = 0;
  if (sms == 0) {
    int dev = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    if (sms <= 0) sms = 148;
  }
  size_t blocks = (n + (size_t)CVT_THREADS * per_thread - 1) / ((size_t)CVT_THREADS * per_thread);
  size_t cap = (size_t)sms * 8;
  if (blocks > cap) blocks = cap;
  if (blocks == 0) blocks = 1;
  return (int)blocks;
}

template <int FMT>
__device__ __forceinline__ uint32_t enc_pair(float lo, float hi, bool sat) {
  return FMT == SKL_DT_F8E4M3 ? enc_e4m3x2(lo, hi, sat) : enc_e5m2x2(lo, hi, sat);
}
template <int FMT>
__device__ __forceinline__ uint32_t enc_one(float x, bool sat) {
  return enc_pair<FMT>(x, 0.0f, sat) & 0xFFu;
}

// fp32 / bf16 -> fp8.  SRC_BF16 selects the 16-bit source.
template <int FMT, bool SRC_BF16>
__global__ void __launch_bounds__(CVT_THREADS)
    cvt_to_f8_kernel(uint8_t *__restrict__ dst, const void *__restrict__ src, float scale, size_t n,
                     bool sat, bool vec_ok) {
  const size_t stride = (size_t)gridDim.x * blockDim.x;
  const size_t tid = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  const size_t nvec = vec_ok ? n / 16 : 0;
  for (size_t v = tid; v < nvec; v += stride) {
    float x[16];
    if (SRC_BF16) {
      const uint4 *s = reinterpret_cast<const uint4 *>(src) + v * 2;
      uint4 q0 = __ldg(s), q1 = __ldg(s + 1);
      uint32_t w[8] = {q0.x, q0.y, q0.z, q0.w, q1.x, q1.y, q1.z, q1.w};
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        x[2 * i] = u2f(w[i] << 16);
        x[2 * i + 1] = u2f(w[i] & 0xFFFF0000u);
      }
    } else {
      const float4 *s = reinterpret_cast<const float4 *>(src) + v * 4;
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        float4 f = __ldg(s + i);
        x[4 * i] = f.x;
        x[4 * i + 1] = f.y;
        x[4 * i + 2] = f.z;
        x[4 * i + 3] = f.w;
      }
    }
    uint32_t o[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      uint32_t p0 = enc_pair<FMT>(__fmul_rn(x[4 * i], scale), __fmul_rn(x[4 * i + 1], scale), sat);
      uint32_t p1 = enc_pair<FMT>(__fmul_rn(x[4 * i + 2], scale), __fmul_rn(x[4 * i + 3], scale), sat);
      o[i] = p0 | (p1 << 16);
    }
    reinterpret_cast<uint4 *>(dst)[v] = make_uint4(o[0], o[1], o[2], o[3]);
  }
  for (size_t i = nvec * 16 + tid; i < n; i += stride) {
    float x = SRC_BF16 ? dec_bf16(((const uint16_t *)src)[i]) : ((const float *)src)[i];
    dst[i] = (uint8_t)enc_one<FMT>(__fmul_rn(x, scale), sat);
  }
}

template <int FMT>
__device__ __forceinline__ uint32_t f8_to_bf16_bits(uint32_t code) {
  // exact: every finite fp8 value fits bf16; the NaN codes become +qNaN 0x7FC0 as the reference's
  // decode-then-cast does (ref/cvt/cvt_ofp8.c:230-242).
  float f = FMT == SKL_DT_F8E4M3 ? dec_e4m3(code) : dec_e5m2(code);
  return f2u(f) >> 16;
}

// Two fp8 codes (low 16 bits of `two`, lower byte first) -> two bf16 patterns, without a branch: the hardware
// decoder to f16x2 (exact for every code, subnormals included), f16 -> f32 -> bf16x2 (exact: at most 4
// significant bits), then the one place where the converters and the reference differ: they produce the NaN
// pattern 0x7FFF (sign kept), the reference's decode-then-cast produces +qNaN 0x7FC0 for every NaN code
// (ref/cvt/cvt_ofp8.c:18-52, 230-242).  No finite or infinite value has the low 15 bits 0x7FFF.
template <int FMT>
__device__ __forceinline__ uint32_t f8x2_to_bf16x2(uint32_t two) {
  const uint16_t in = (uint16_t)two;
  uint32_t h2;
  if (FMT == SKL_DT_F8E4M3)
    asm("cvt.rn.f16x2.e4m3x2 %0, %1;" : "=r"(h2) : "h"(in));
  else
    asm("cvt.rn.f16x2.e5m2x2 %0, %1;" : "=r"(h2) : "h"(in));
  float f0, f1;
  asm("{\n\t.reg .f16 a, b;\n\tmov.b32 {a, b}, %2;\n\tcvt.f32.f16 %0, a;\n\tcvt.f32.f16 %1, b;\n\t}"
      : "=f"(f0), "=f"(f1)
      : "r"(h2));
  uint32_t r;
  asm("cvt.rn.bf16x2.f32 %0, %1, %2;" : "=r"(r) : "f"(f1), "f"(f0));
  const uint32_t t = r & 0x7FFF7FFFu;
  const uint32_t nan1 = ((t + 0x00010001u) >> 15) & 0x00010001u;  // 1 in each half that holds 0x7FFF
  const uint32_t mask = nan1 * 0xFFFFu;
  return (r & ~mask) | (0x7FC07FC0u & mask);
}

// Four fp8 codes (one 32-bit word, lowest byte first) -> four bf16 patterns in two words.
template <int FMT>
__device__ __forceinline__ void f8x4_to_bf16x4(uint32_t w, uint32_t &lo, uint32_t &hi) {
  lo = f8x2_to_bf16x2<FMT>(w);
  hi = f8x2_to_bf16x2<FMT>(w >> 16);
}

// Widening: the unit of work is 8 codes = one 8-byte load and one 16-byte store, consecutive lanes taking
// consecutive units, so that every warp-level load covers 256 contiguous bytes and every store 512 (a thread
// that converted 16 codes would write its 32 bytes as two 16-byte halves, and each warp-level store would
// then touch 32 sectors half-way).  Eight units per thread are in flight to cover the HBM latency.
template <int FMT>
__global__ void __launch_bounds__(CVT_THREADS)
    cvt_f8_to_bf16_kernel(uint16_t *__restrict__ dst, const uint8_t *__restrict__ src, size_t n,
                          bool vec_ok) {
  constexpr int U = 8;
  const size_t stride = (size_t)gridDim.x * blockDim.x;
  const size_t tid = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  const size_t nvec = vec_ok ? n / 8 : 0;
  for (size_t v0 = tid; v0 < nvec; v0 += U * stride) {
    uint2 q[U];
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const size_t v = v0 + u * stride;
      q[u] = v < nvec ? __ldg(reinterpret_cast<const uint2 *>(src) + v) : make_uint2(0, 0);
    }
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const size_t v = v0 + u * stride;
      if (v >= nvec) break;
      uint32_t o[4];
      f8x4_to_bf16x4<FMT>(q[u].x, o[0], o[1]);
      f8x4_to_bf16x4<FMT>(q[u].y, o[2], o[3]);
      reinterpret_cast<uint4 *>(dst)[v] = make_uint4(o[0], o[1], o[2], o[3]);
    }
  }
  for (size_t i = nvec * 8 + tid; i < n; i += stride) dst[i] = (uint16_t)f8_to_bf16_bits<FMT>(src[i]);
}

// rows x cols matrix, unit stride along cols, separate leading dimensions; cols % 8 == 0 and rows aligned
// to 8 (source) / 16 (destination) bytes take the vector path.
template <int FMT>
__global__ void __launch_bounds__(CVT_THREADS)
    cvt_f8_to_bf16_2d_kernel(uint16_t *__restrict__ dst, size_t ld_dst, const uint8_t *__restrict__ src,
                             size_t ld_src, size_t rows, size_t cols, bool vec_ok) {
  constexpr int U = 8;
  const size_t stride = (size_t)gridDim.x * blockDim.x;
  const size_t tid = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (vec_ok) {
    const size_t cvec = cols / 8;
    const size_t total = rows * cvec;
    // (row, unit-in-row) of this thread's next unit, advanced by one grid stride at a time without dividing
    const size_t dr = stride / cvec, dc = stride - dr * cvec;
    size_t r = tid / cvec, c = tid - r * cvec;
    for (size_t v0 = tid; v0 < total; v0 += U * stride) {
      uint2 q[U];
      size_t doff[U];  // destination offset in 16-byte units
#pragma unroll
      for (int u = 0; u < U; ++u) {
        const size_t v = v0 + u * stride;
        doff[u] = r * (ld_dst / 8) + c;
        q[u] = v < total ? __ldg(reinterpret_cast<const uint2 *>(src + r * ld_src) + c) : make_uint2(0, 0);
        r += dr;
        c += dc;
        if (c >= cvec) {
          c -= cvec;
          ++r;
        }
      }
#pragma unroll
      for (int u = 0; u < U; ++u) {
        if (v0 + u * stride >= total) break;
        uint32_t o[4];
        f8x4_to_bf16x4<FMT>(q[u].x, o[0], o[1]);
        f8x4_to_bf16x4<FMT>(q[u].y, o[2], o[3]);
        reinterpret_cast<uint4 *>(dst)[doff[u]] = make_uint4(o[0], o[1], o[2], o[3]);
      }
    }
  } else {
    const size_t total = rows * cols;
    for (size_t e = tid; e < total; e += stride) {
      size_t r = e / cols, c = e - r * cols;
      dst[r * ld_dst + c] = (uint16_t)f8_to_bf16_bits<FMT>(src[r * ld_src + c]);
    }
  }
}

// E2M1 nibble -> E4M3 byte: all eight magnitudes are exact in E4M3 (ref/cvt/cvt_ofp4.c:18-60).
__device__ __forceinline__ uint32_t f4_to_e4m3(uint32_t nib) {
  // magnitudes 0, .5, 1, 1.5, 2, 3, 4, 6 -> 0x00 0x30 0x38 0x3C 0x40 0x44 0x48 0x4C
  const uint64_t lut = 0x4C4844403C383000ull;
  uint32_t mag = (uint32_t)(lut >> ((nib & 7u) * 8)) & 0xFFu;
  return mag | ((nib & 8u) << 4);
}

__global__ void __launch_bounds__(CVT_THREADS)
    cvt_f4_to_f8_kernel(uint8_t *__restrict__ dst, const uint8_t *__restrict__ src, size_t n) {
  const size_t stride = (size_t)gridDim.x * blockDim.x;
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride) {
    uint32_t byte = src[i >> 1];
    dst[i] = (uint8_t)f4_to_e4m3((i & 1) ? (byte >> 4) : (byte & 0xFu));
  }
}

template <int FMT>
__global__ void __launch_bounds__(CVT_THREADS)
    cvt_selfcheck_kernel(bool sat, uint64_t first, uint64_t count, unsigned long long *mismatches) {
  const uint64_t stride = (uint64_t)gridDim.x * blockDim.x;
  unsigned long long bad = 0;
  for (uint64_t i = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x; i < count; i += stride) {
    float x = u2f((uint32_t)(first + i));
    uint32_t fast = enc_one<FMT>(x, sat);
    uint32_t soft = FMT == SKL_DT_F8E4M3 ? enc_e4m3_soft(x, sat) : enc_e5m2_soft(x, sat);
    bad += (fast != soft);
  }
  if (bad) atomicAdd(mismatches, bad);
}

inline bool aligned16(const void *p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

}  // namespace
}  // namespace sklb

using namespace sklb;

extern "C" int skl_b200_launch_cvt_to_f8(void *dst, const void *src, int src_type, int dst_fmt,
                                         int saturate, float scale, size_t n, void *stream) {
  if (n == 0) return 0;
  cudaStream_t s = (cudaStream_t)stream;
  const bool vec = aligned16(dst) && aligned16(src);
  const int grid = cvt_grid(n, 16);
  const bool sat = saturate != 0;
  uint8_t *d = (uint8_t *)dst;
  if (src_type == SKL_DT_F32) {
    if (dst_fmt == SKL_DT_F8E4M3)
      cvt_to_f8_kernel<SKL_DT_F8E4M3, false><<<grid, CVT_THREADS, 0, s>>>(d, src, scale, n, sat, vec);
    else
      cvt_to_f8_kernel<SKL_DT_F8E5M2, false><<<grid, CVT_THREADS, 0, s>>>(d, src, scale, n, sat, vec);
  } else {
    if (dst_fmt == SKL_DT_F8E4M3)
      cvt_to_f8_kernel<SKL_DT_F8E4M3, true><<<grid, CVT_THREADS, 0, s>>>(d, src, scale, n, sat, vec);
    else
      cvt_to_f8_kernel<SKL_DT_F8E5M2, true><<<grid, CVT_THREADS, 0, s>>>(d, src, scale, n, sat, vec);
  }
  SKLB_COUNT_LAUNCH();
  return (int)cudaGetLastError();
}

extern "C" int skl_b200_launch_cvt_f8_to_bf16(void *dst, const void *src, int src_fmt, size_t n,
                                              void *stream) {
  if (n == 0) return 0;
  cudaStream_t s = (cudaStream_t)stream;
  const bool vec = aligned16(dst) && aligned16(src);
  const int grid = cvt_grid(n, 8 * 8);
  if (src_fmt == SKL_DT_F8E4M3)
    cvt_f8_to_bf16_kernel<SKL_DT_F8E4M3>
        <<<grid, CVT_THREADS, 0, s>>>((uint16_t *)dst, (const uint8_t *)src, n, vec);
  else
    cvt_f8_to_bf16_kernel<SKL_DT_F8E5M2>
        <<<grid, CVT_THREADS, 0, s>>>((uint16_t *)dst, (const uint8_t *)src, n, vec);
  SKLB_COUNT_LAUNCH();
  return (int)cudaGetLastError();
}

extern "C" int skl_b200_launch_cvt_f8_to_bf16_2d(void *dst, size_t ld_dst, const void *src,
                                                 size_t ld_src, int src_fmt, size_t rows,
                                                 size_t cols, void *stream) {
  if (rows == 0 || cols == 0) return 0;
  cudaStream_t s = (cudaStream_t)stream;
  const bool vec = aligned16(dst) && aligned16(src) && (cols % 8 == 0) && (ld_src % 8 == 0) && (ld_dst % 8 == 0);
  const int grid = cvt_grid(rows * cols, 8 * 8);
  if (src_fmt == SKL_DT_F8E4M3)
    cvt_f8_to_bf16_2d_kernel<SKL_DT_F8E4M3><<<grid, CVT_THREADS, 0, s>>>(
        (uint16_t *)dst, ld_dst, (const uint8_t *)src, ld_src, rows, cols, vec);
  else
    cvt_f8_to_bf16_2d_kernel<SKL_DT_F8E5M2><<<grid, CVT_THREADS, 0, s>>>(
        (uint16_t *)dst, ld_dst, (const uint8_t *)src, ld_src, rows, cols, vec);
  SKLB_COUNT_LAUNCH();
  return (int)cudaGetLastError();
}

extern "C" int skl_b200_launch_cvt_f4_to_f8e4m3(void *dst, const void *src, size_t n, void *stream) {
  if (n == 0) return 0;
  cvt_f4_to_f8_kernel<<<cvt_grid(n, 1), CVT_THREADS, 0, (cudaStream_t)stream>>>(
      (uint8_t *)dst, (const uint8_t *)src, n);
  SKLB_COUNT_LAUNCH();
  return (int)cudaGetLastError();
}

extern "C" int skl_b200_launch_cvt_selfcheck(int dst_fmt, int saturate, uint64_t first,
                                             uint64_t count, unsigned long long *mismatches,
                                             void *stream) {
  if (count == 0) return 0;
  cudaStream_t s = (cudaStream_t)stream;
  const int grid = cvt_grid(count, 64);
  if (dst_fmt == SKL_DT_F8E4M3)
    cvt_selfcheck_kernel<SKL_DT_F8E4M3><<<grid, CVT_THREADS, 0, s>>>(saturate != 0, first, count, mismatches);
  else
    cvt_selfcheck_kernel<SKL_DT_F8E5M2><<<grid, CVT_THREADS, 0, s>>>(saturate != 0, first, count, mismatches);
  SKLB_COUNT_LAUNCH();
  return (int)cudaGetLastError();
}
