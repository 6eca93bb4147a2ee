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

__device__ __forceinline__ bool has_zero_byte(uint32_t v) {
  return ((v - 0x01010101u) & ~v & 0x80808080u) != 0u;
}

// Four fp8 codes (one 32-bit word, lowest byte first) -> four bf16 patterns in two words.
// Normal codes are widened with packed integer arithmetic, two per word:
//     E4M3: bf16 = sign<<8 | ((code & 0x7F) << 4) + (120 << 7)      E5M2: ... << 5) + (112 << 7)
// A word that holds any code with a zero exponent field (zero, subnormal) or an all-ones one
// (E4M3 NaN, E5M2 Inf / NaN) takes the per-element decoder instead.
template <int FMT>
__device__ __forceinline__ void f8x4_to_bf16x4(uint32_t w, uint32_t &lo, uint32_t &hi) {
  constexpr uint32_t EXPF = FMT == SKL_DT_F8E4M3 ? 0x78787878u : 0x7C7C7C7Cu;
  const uint32_t e = w & EXPF;
  // E4M3's only non-finite code is exponent and mantissa all ones; E5M2's are every all-ones exponent
  const uint32_t top = FMT == SKL_DT_F8E4M3 ? ((w & 0x7F7F7F7Fu) ^ 0x7F7F7F7Fu) : (e ^ EXPF);
  if (has_zero_byte(e) || has_zero_byte(top)) {
    lo = f8_to_bf16_bits<FMT>(w & 0xFFu) | (f8_to_bf16_bits<FMT>((w >> 8) & 0xFFu) << 16);
    hi = f8_to_bf16_bits<FMT>((w >> 16) & 0xFFu) | (f8_to_bf16_bits<FMT>(w >> 24) << 16);
    return;
  }
  constexpr int SH = FMT == SKL_DT_F8E4M3 ? 4 : 5;
  constexpr uint32_t BIAS = FMT == SKL_DT_F8E4M3 ? 0x3C003C00u : 0x38003800u;
  const uint32_t x0 = __byte_perm(w, 0u, 0x4140);  // 0x00b1_00b0
  const uint32_t x1 = __byte_perm(w, 0u, 0x4342);  // 0x00b3_00b2
  lo = (((x0 & 0x007F007Fu) << SH) + BIAS) | ((x0 & 0x00800080u) << 8);
  hi = (((x1 & 0x007F007Fu) << SH) + BIAS) | ((x1 & 0x00800080u) << 8);
}

template <int FMT>
__global__ void __launch_bounds__(CVT_THREADS)
    cvt_f8_to_bf16_kernel(uint16_t *__restrict__ dst, const uint8_t *__restrict__ src, size_t n,
                          bool vec_ok) {
  const size_t stride = (size_t)gridDim.x * blockDim.x;
  const size_t tid = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  const size_t nvec = vec_ok ? n / 16 : 0;
  // four independent 16-byte loads per thread per step: enough bytes in flight to cover HBM latency
  for (size_t v0 = tid; v0 < nvec; v0 += 4 * stride) {
    uint4 q[4];
#pragma unroll
    for (int u = 0; u < 4; ++u) {
      const size_t v = v0 + u * stride;
      q[u] = v < nvec ? __ldg(reinterpret_cast<const uint4 *>(src) + v) : make_uint4(0, 0, 0, 0);
    }
#pragma unroll
    for (int u = 0; u < 4; ++u) {
      const size_t v = v0 + u * stride;
      if (v >= nvec) break;
      uint32_t w[4] = {q[u].x, q[u].y, q[u].z, q[u].w};
      uint32_t o[8];
#pragma unroll
      for (int i = 0; i < 4; ++i) f8x4_to_bf16x4<FMT>(w[i], o[2 * i], o[2 * i + 1]);
      uint4 *d = reinterpret_cast<uint4 *>(dst) + v * 2;
      d[0] = make_uint4(o[0], o[1], o[2], o[3]);
      d[1] = make_uint4(o[4], o[5], o[6], o[7]);
    }
  }
  for (size_t i = nvec * 16 + tid; i < n; i += stride) dst[i] = (uint16_t)f8_to_bf16_bits<FMT>(src[i]);
}

// rows x cols matrix, unit stride along cols, separate leading dimensions; cols % 16 == 0 and
// 16-byte aligned rows take the vector path.
template <int FMT>
__global__ void __launch_bounds__(CVT_THREADS)
    cvt_f8_to_bf16_2d_kernel(uint16_t *__restrict__ dst, size_t ld_dst, const uint8_t *__restrict__ src,
                             size_t ld_src, size_t rows, size_t cols, bool vec_ok) {
  const size_t stride = (size_t)gridDim.x * blockDim.x;
  const size_t tid = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (vec_ok) {
    const size_t cvec = cols / 16;
    const size_t total = rows * cvec;
    for (size_t v0 = tid; v0 < total; v0 += 4 * stride) {
      uint4 q[4];
      size_t rr[4], cc[4];
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        const size_t v = v0 + u * stride;
        rr[u] = v / cvec;
        cc[u] = v - rr[u] * cvec;
        q[u] = v < total ? __ldg(reinterpret_cast<const uint4 *>(src + rr[u] * ld_src) + cc[u]) : make_uint4(0, 0, 0, 0);
      }
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        if (v0 + u * stride >= total) break;
        uint32_t w[4] = {q[u].x, q[u].y, q[u].z, q[u].w};
        uint32_t o[8];
#pragma unroll
        for (int i = 0; i < 4; ++i) f8x4_to_bf16x4<FMT>(w[i], o[2 * i], o[2 * i + 1]);
        uint4 *d = reinterpret_cast<uint4 *>(dst + rr[u] * ld_dst) + cc[u] * 2;
        d[0] = make_uint4(o[0], o[1], o[2], o[3]);
        d[1] = make_uint4(o[4], o[5], o[6], o[7]);
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
  const int grid = cvt_grid(n, 16);
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
  const bool vec = aligned16(dst) && aligned16(src) && (cols % 16 == 0) && (ld_src % 16 == 0) &&
                   (ld_dst % 8 == 0);
  const int grid = cvt_grid(rows * cols, 16);
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
