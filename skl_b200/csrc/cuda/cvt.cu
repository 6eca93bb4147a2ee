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
  // Launched as a programmatic dependent of the kernel before it on the stream (its CTAs are resident and past their
  // index set-up when that kernel ends) and itself lets the GEMM that follows start its own set-up early.
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  const size_t stride = (size_t)gridDim.x * blockDim.x;
  const size_t tid = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  asm volatile("griddepcontrol.wait;" ::: "memory");  // nothing is read before the preceding kernel has finished
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

// Widening with a transpose: src is rows x cols fp8 with unit stride along cols, dst is cols x rows bf16 with unit
// stride along rows (dst[c][r] = widen(src[r][c])).  Used for the fp8 operand of a bf16 x fp8 GEMM whose B arrives
// n-contiguous: the tensor-core kernel runs several percent faster on a k-contiguous B, and since the widened copy
// has to be written anyway it is written in that orientation.
// Tile: 128 rows x 64 cols.  A thread takes 4 rows x 4 cols as four 4-byte loads, transposes the 4 x 4 bytes in
// registers, widens each column's 4 codes (consecutive along dst's unit stride) to 8 bytes and puts them into a
// shared-memory tile laid out like dst; the tile then leaves as 16-byte stores, 256 contiguous bytes per dst row.
constexpr int WT_R = 128, WT_C = 64, WT_PITCH = 2 * WT_R + 8;  // pitch in bytes, 8-byte aligned, odd in 8-byte units
template <int FMT>
__global__ void __launch_bounds__(256)
    cvt_f8_to_bf16_transpose_kernel(uint16_t *__restrict__ dst, size_t ld_dst, const uint8_t *__restrict__ src,
                                    size_t ld_src, uint32_t rows, uint32_t cols, uint32_t tiles_r, uint32_t tiles_c) {
  __shared__ __align__(16) uint8_t tile[WT_C * WT_PITCH];
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");  // see cvt_f8_to_bf16_2d_kernel
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const uint32_t num_tiles = tiles_r * tiles_c;
  asm volatile("griddepcontrol.wait;" ::: "memory");
  for (uint32_t t = blockIdx.x; t < num_tiles; t += gridDim.x) {
    const uint32_t r0 = (t / tiles_c) * WT_R, c0 = (t % tiles_c) * WT_C;
    const bool full = r0 + WT_R <= rows && c0 + WT_C <= cols;
    if (full) {
      // 32 x 16 micro-tiles of 4 rows x 4 cols; a warp step covers 4 (rows) x 8 (cols) of them
#pragma unroll
      for (int w = warp; w < 16; w += 8) {
        const int cx = (w & 1) * 8 + (lane & 7);   // micro-tile column 0..15
        const int ry = (w >> 1) * 4 + (lane >> 3);  // micro-tile row 0..31
        uint32_t r[4];
#pragma unroll
        for (int q = 0; q < 4; ++q)
          r[q] = __ldg(reinterpret_cast<const uint32_t *>(src + (size_t)(r0 + 4 * ry + q) * ld_src + c0 + 4 * cx));
        const uint32_t a0 = __byte_perm(r[0], r[1], 0x5140), a1 = __byte_perm(r[0], r[1], 0x7362);
        const uint32_t b0 = __byte_perm(r[2], r[3], 0x5140), b1 = __byte_perm(r[2], r[3], 0x7362);
        const uint32_t col[4] = {__byte_perm(a0, b0, 0x5410), __byte_perm(a0, b0, 0x7632), __byte_perm(a1, b1, 0x5410),
                                 __byte_perm(a1, b1, 0x7632)};  // col[b] = codes of rows 4ry..4ry+3 in column 4cx+b
#pragma unroll
        for (int b = 0; b < 4; ++b) {
          uint32_t lo, hi;
          f8x4_to_bf16x4<FMT>(col[b], lo, hi);
          *reinterpret_cast<uint2 *>(tile + (4 * cx + b) * WT_PITCH + 8 * ry) = make_uint2(lo, hi);
        }
      }
      __syncthreads();
      // 64 dst rows of 256 bytes = 16 pieces of 16 bytes each
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const int e = threadIdx.x + 256 * i, row = e >> 4, piece = e & 15;
        const uint2 x = *reinterpret_cast<const uint2 *>(tile + row * WT_PITCH + 16 * piece);
        const uint2 y = *reinterpret_cast<const uint2 *>(tile + row * WT_PITCH + 16 * piece + 8);
        *reinterpret_cast<uint4 *>(dst + (size_t)(c0 + row) * ld_dst + r0 + 8 * piece) = make_uint4(x.x, x.y, y.x, y.y);
      }
      __syncthreads();
    } else {
      // ragged edge tile: one element at a time
      for (int e = threadIdx.x; e < WT_R * WT_C; e += 256) {
        const uint32_t rr = r0 + e / WT_C, cc = c0 + e % WT_C;
        if (rr < rows && cc < cols) dst[(size_t)cc * ld_dst + rr] = (uint16_t)f8_to_bf16_bits<FMT>(src[(size_t)rr * ld_src + cc]);
      }
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

// Launch configuration of a kernel that may start as a programmatic dependent of its predecessor on the stream
// (the widening kernels of the bf16 x fp8 GEMM: they sit between two GEMM launches of a decode or training loop).
static cudaLaunchConfig_t dependent_launch(int grid, int threads, cudaStream_t s, cudaLaunchAttribute *attr) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3((unsigned)grid);
  cfg.blockDim = dim3((unsigned)threads);
  cfg.dynamicSmemBytes = 0;
  cfg.stream = s;
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  return cfg;
}

extern "C" int skl_b200_launch_cvt_f8_to_bf16_2d(void *dst, size_t ld_dst, const void *src,
                                                 size_t ld_src, int src_fmt, size_t rows,
                                                 size_t cols, void *stream) {
  if (rows == 0 || cols == 0) return 0;
  cudaStream_t s = (cudaStream_t)stream;
  const bool vec = aligned16(dst) && aligned16(src) && (cols % 8 == 0) && (ld_src % 8 == 0) && (ld_dst % 8 == 0);
  const int grid = cvt_grid(rows * cols, 8 * 8);
  cudaLaunchAttribute attr[1];
  const cudaLaunchConfig_t cfg = dependent_launch(grid, CVT_THREADS, s, attr);
  cudaError_t e;
  if (src_fmt == SKL_DT_F8E4M3)
    e = cudaLaunchKernelEx(&cfg, cvt_f8_to_bf16_2d_kernel<SKL_DT_F8E4M3>, (uint16_t *)dst, ld_dst, (const uint8_t *)src,
                           ld_src, rows, cols, vec);
  else
    e = cudaLaunchKernelEx(&cfg, cvt_f8_to_bf16_2d_kernel<SKL_DT_F8E5M2>, (uint16_t *)dst, ld_dst, (const uint8_t *)src,
                           ld_src, rows, cols, vec);
  SKLB_COUNT_LAUNCH();
  if (e != cudaSuccess) return (int)e;
  return (int)cudaGetLastError();
}

extern "C" int skl_b200_launch_cvt_f8_to_bf16_2d_transposed(void *dst, size_t ld_dst, const void *src,
                                                            size_t ld_src, int src_fmt, size_t rows,
                                                            size_t cols, void *stream) {
  if (rows == 0 || cols == 0) return 0;
  // word loads along src rows, 16-byte stores along dst rows
  if (!aligned16(dst) || (reinterpret_cast<uintptr_t>(src) & 3u) != 0 || ld_src % 4 != 0 || ld_dst % 8 != 0 ||
      rows >= (1ull << 31) || cols >= (1ull << 31))
    return (int)cudaErrorInvalidValue;
  const uint32_t tr = (uint32_t)((rows + WT_R - 1) / WT_R), tc = (uint32_t)((cols + WT_C - 1) / WT_C);
  const uint64_t tiles = (uint64_t)tr * tc;
  const uint64_t cap = (uint64_t)cvt_grid(~(size_t)0 >> 8, 1);  // 8 CTAs per SM
  const int grid = (int)(tiles < cap ? tiles : cap);
  cudaStream_t s = (cudaStream_t)stream;
  cudaLaunchAttribute attr[1];
  const cudaLaunchConfig_t cfg = dependent_launch(grid, 256, s, attr);
  cudaError_t e;
  if (src_fmt == SKL_DT_F8E4M3)
    e = cudaLaunchKernelEx(&cfg, cvt_f8_to_bf16_transpose_kernel<SKL_DT_F8E4M3>, (uint16_t *)dst, ld_dst,
                           (const uint8_t *)src, ld_src, (uint32_t)rows, (uint32_t)cols, tr, tc);
  else
    e = cudaLaunchKernelEx(&cfg, cvt_f8_to_bf16_transpose_kernel<SKL_DT_F8E5M2>, (uint16_t *)dst, ld_dst,
                           (const uint8_t *)src, ld_src, (uint32_t)rows, (uint32_t)cols, tr, tc);
  SKLB_COUNT_LAUNCH();
  if (e != cudaSuccess) return (int)e;
  return (int)cudaGetLastError();
}

// OCP MX-FP4 -> bf16: element = E2M1 value (ref/cvt/cvt_ofp4.c:18-60) x 2^(scale - 127), one E8M0 scale byte per 32
// consecutive k (scale 255 = NaN).  The result has at most 2 significant bits and bf16 has fp32's exponent range, so
// the widening is exact wherever the fp32 product is.  One thread per block of 32 elements: 16 bytes in, 64 out.
__global__ void __launch_bounds__(CVT_THREADS)
    cvt_mxf4_to_bf16_kernel(uint16_t *__restrict__ dst, size_t ld_dst, const uint8_t *__restrict__ src, size_t ld_src,
                            const uint8_t *__restrict__ scales, size_t ld_scales, uint32_t rows, uint32_t kblocks) {
  const uint64_t total = (uint64_t)rows * kblocks, stride = (uint64_t)gridDim.x * blockDim.x;
  for (uint64_t i = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += stride) {
    const uint32_t r = (uint32_t)(i / kblocks), kb = (uint32_t)(i - (uint64_t)r * kblocks);
    const uint8_t *sp = src + (size_t)r * ld_src + (size_t)kb * 16;
    const uint32_t sc = scales[(size_t)r * ld_scales + kb];
    // 2^(sc - 127) as fp32 bits: sc = 0 is the subnormal 2^-127, sc = 255 NaN
    const float f = sc == 255u ? __uint_as_float(0x7FC00000u) : (sc == 0u ? __uint_as_float(0x00400000u) : __uint_as_float(sc << 23));
    uint32_t w[4];
    if ((reinterpret_cast<uintptr_t>(sp) & 15u) == 0) {
      const uint4 v = *reinterpret_cast<const uint4 *>(sp);
      w[0] = v.x; w[1] = v.y; w[2] = v.z; w[3] = v.w;
    } else {
#pragma unroll
      for (int q = 0; q < 4; ++q) w[q] = sp[4 * q] | (sp[4 * q + 1] << 8) | (sp[4 * q + 2] << 16) | ((uint32_t)sp[4 * q + 3] << 24);
    }
    uint16_t *dp = dst + (size_t)r * ld_dst + (size_t)kb * 32;
#pragma unroll
    for (int q = 0; q < 4; ++q) {
#pragma unroll
      for (int e = 0; e < 8; e += 2) {  // nibbles low first
        const uint32_t n0 = (w[q] >> (4 * e)) & 0xFu, n1 = (w[q] >> (4 * e + 4)) & 0xFu;
        // magnitudes 0, .5, 1, 1.5, 2, 3, 4, 6 as bf16 bit patterns of the fp32 value's upper half
        const uint64_t lut_lo = 0x3FC03F803F000000ull, lut_hi = 0x40C0408040404000ull;
        auto val = [&](uint32_t nib) {
          const uint32_t m = nib & 7u;
          const uint32_t hi16 = (uint32_t)((m < 4 ? lut_lo >> (16 * m) : lut_hi >> (16 * (m - 4))) & 0xFFFFu);
          const float x = __uint_as_float((hi16 << 16) | ((nib & 8u) << 28));
          return __float_as_uint(__fmul_rn(x, f)) >> 16;  // exact: the low 16 bits of the product are zero
        };
        const uint32_t pair = val(n0) | (val(n1) << 16);
        *reinterpret_cast<uint32_t *>(dp + 8 * q + e) = pair;
      }
    }
  }
}

extern "C" int skl_b200_launch_cvt_mxf4_to_bf16(void *dst, size_t ld_dst, const void *src, size_t ld_src, const void *scales,
                                                size_t ld_scales, size_t rows, size_t kblocks, void *stream) {
  if (rows == 0 || kblocks == 0) return 0;
  cvt_mxf4_to_bf16_kernel<<<cvt_grid(rows * kblocks, 1), CVT_THREADS, 0, (cudaStream_t)stream>>>(
      (uint16_t *)dst, ld_dst, (const uint8_t *)src, ld_src, (const uint8_t *)scales, ld_scales, (uint32_t)rows,
      (uint32_t)kblocks);
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
