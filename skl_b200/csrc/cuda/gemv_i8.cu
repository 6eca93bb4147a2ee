// gemv_i8.cu -- skinny int8 GEMM (m <= 16): the decode-shape case.
//
// C[i, j] = sum_k A[i, k] * B[k, j] with A = activations (m rows, k contiguous) and B = weights stored
// one output column per contiguous k-run ("[N][K]": rsb == 1, csb == row pitch).  With m this small
// the arithmetic intensity is at most 2*m ops per weight byte, far below the tensor-core ridge, so
// the kernel is a weight-streaming kernel bounded by HBM bandwidth: every weight byte is read once
// with 16-byte no-allocate loads, activations sit in shared memory, products use dp4a on the
// integer pipe, and the k-split across the 32 lanes of a warp is folded with warp shuffles.  No tensor
// cores.  SKL's counterpart is the m == 1 branch of its int8 kernel
// (src/gemm/gemm_i8rcp1x4_i8p4x1c_i32_xsfvqdotq.c:543-632, dispatch :645-658).
//
// Work split: one persistent CTA per SM owns a contiguous slab of weight rows; each warp takes
// groups of R = 4 rows; each lane walks 16-byte chunks lane, lane+32, ... of those rows.
// Algorithmic bytes per launch: N*K (weights) + m*K (activations) + output and scale vectors.
#include "numerics.cuh"

namespace sklb {
namespace {

constexpr int GV_THREADS = 512;
constexpr int GV_R = 4;

struct GemvParams {
  const int8_t *x;  // activations, row i at x + i*ldx
  const int8_t *w;  // weights, output column j at w + j*ldw
  void *c;
  int64_t ldx, ldw, rsc, csc;
  int m, n, k;
  int epilogue, tc;
  int32_t alpha_i, beta_i;
  float alpha_f, beta_f;
  const float *row_scale, *col_scale;
};

__device__ __forceinline__ uint4 ld_stream16(const void *p) {
  uint4 v;
  asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
               : "l"(p));
  return v;
}

// Folds V partial sums held by every lane across the warp.  Each halving step exchanges half of the
// values a lane still holds, so the total is V-1+... shuffles instead of 5*V.  On return v[0..W)
// (W = max(V/32, 1)) are complete sums; lane L holds value indices (L >> s) * W + w where
// s = max(0, 5 - log2 V).
template <int V>
__device__ __forceinline__ void warp_fold(int32_t (&v)[V], int lane) {
  int cur = V;
#pragma unroll
  for (int off = 16; off >= 1; off >>= 1) {
    if (cur > 1) {
      const int half = cur / 2;
      const bool upper = (lane & off) != 0;
#pragma unroll
      for (int i = 0; i < V / 2; ++i) {
        if (i < half) {
          int32_t send = upper ? v[i] : v[i + half];
          int32_t keep = upper ? v[i + half] : v[i];
          v[i] = keep + __shfl_xor_sync(0xFFFFFFFFu, send, off);
        }
      }
      cur = half;
    } else {
      v[0] += __shfl_xor_sync(0xFFFFFFFFu, v[0], off);
    }
  }
}

template <int MP>
__global__ void __launch_bounds__(GV_THREADS, 1) gemv_i8_kernel(const GemvParams p) {
  extern __shared__ uint4 xs[];  // [MP][k/16]
  const int kc = p.k >> 4;
  for (int e = threadIdx.x; e < MP * kc; e += GV_THREADS) {
    int mi = e / kc, ch = e - mi * kc;
    uint4 v = make_uint4(0, 0, 0, 0);
    if (mi < p.m) v = *reinterpret_cast<const uint4 *>(p.x + (int64_t)mi * p.ldx + (int64_t)ch * 16);
    xs[e] = v;
  }
  __syncthreads();

  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  constexpr int NW = GV_THREADS / 32;
  const int groups = (p.n + GV_R - 1) / GV_R;
  const int g_begin = (int)(((int64_t)groups * blockIdx.x) / gridDim.x);
  const int g_end = (int)(((int64_t)groups * (blockIdx.x + 1)) / gridDim.x);

  for (int g = g_begin + warp; g < g_end; g += NW) {
    const int n0 = g * GV_R;
    const int8_t *wrow[GV_R];
#pragma unroll
    for (int r = 0; r < GV_R; ++r) {
      int nr = n0 + r < p.n ? n0 + r : p.n - 1;  // clamp: rows past the end are loaded twice, never stored
      wrow[r] = p.w + (int64_t)nr * p.ldw;
    }
    int32_t acc[GV_R * MP];
#pragma unroll
    for (int i = 0; i < GV_R * MP; ++i) acc[i] = 0;

#pragma unroll 2
    for (int ch = lane; ch < kc; ch += 32) {
      uint4 wv[GV_R];
#pragma unroll
      for (int r = 0; r < GV_R; ++r) wv[r] = ld_stream16(wrow[r] + (int64_t)ch * 16);
#pragma unroll
      for (int mi = 0; mi < MP; ++mi) {
        const uint4 xv = xs[mi * kc + ch];
#pragma unroll
        for (int r = 0; r < GV_R; ++r) {
          int32_t a = acc[r * MP + mi];
          a = __dp4a((int)wv[r].x, (int)xv.x, a);
          a = __dp4a((int)wv[r].y, (int)xv.y, a);
          a = __dp4a((int)wv[r].z, (int)xv.z, a);
          a = __dp4a((int)wv[r].w, (int)xv.w, a);
          acc[r * MP + mi] = a;
        }
      }
    }

    warp_fold<GV_R * MP>(acc, lane);

    constexpr int V = GV_R * MP;
    constexpr int W = V >= 32 ? V / 32 : 1;
    constexpr int LOGV = V >= 32 ? 5 : (V == 16 ? 4 : (V == 8 ? 3 : 2));
    const int share = 5 - LOGV;                   // lanes sharing one value: 2^share
    if ((lane & ((1 << share) - 1)) == 0) {       // one writer per value
#pragma unroll
      for (int w = 0; w < W; ++w) {
        const int idx = (lane >> share) * W + w;  // = r*MP + mi
        const int r = idx / MP, mi = idx - r * MP;
        const int j = n0 + r;
        if (j < p.n && mi < p.m) {
          const int64_t o = (int64_t)mi * p.rsc + (int64_t)j * p.csc;
          const int32_t a = acc[w];
          if (p.epilogue == SKL_EPI_INT) {
            int32_t *cp = (int32_t *)p.c + o;
            uint32_t old = p.beta_i != 0 ? (uint32_t)p.beta_i * (uint32_t)*cp : 0u;
            *cp = (int32_t)(old + (uint32_t)p.alpha_i * (uint32_t)a);
          } else {
            float v = epilogue_value((float)a, p.alpha_f, p.row_scale, p.col_scale, mi, j);
            if (p.beta_f != 0.0f) v = __fadd_rn(__fmul_rn(p.beta_f, load_c_f32(p.tc, p.c, o)), v);
            store_c_f32(p.tc, p.c, o, v);
          }
        }
      }
    }
  }
}

constexpr size_t GV_MAX_SMEM = 160 * 1024;

inline bool al16(const void *p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

int num_sms() {
  static int sms = 0;
  if (sms == 0) {
    int dev = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    if (sms <= 0) sms = 148;
  }
  return sms;
}

}  // namespace
}  // namespace sklb

using namespace sklb;

extern "C" int skl_b200_gemv_i8_supported(const skl_b200_gemm_args *g) {
  if (g->ta != SKL_DT_I8 || g->tb != SKL_DT_I8) return 0;
  if (g->m1 != 1 || g->n1 != 1 || g->k1 != 1) return 0;
  if (g->m0 == 0 || g->m0 > 16 || g->n0 == 0 || g->k0 == 0) return 0;
  if (g->csa0 != 1 || g->rsb0 != 1) return 0;
  if ((g->k0 & 15) != 0 || g->k0 > (1u << 20) || g->n0 > (1u << 30)) return 0;
  if (!al16(g->a) || !al16(g->b)) return 0;
  if ((g->m0 > 1 && (g->rsa0 & 15) != 0) || (g->n0 > 1 && (g->csb0 & 15) != 0)) return 0;
  int mp = 1;
  while (mp < (int)g->m0) mp <<= 1;
  if ((size_t)mp * g->k0 > GV_MAX_SMEM) return 0;
  if (g->epilogue == SKL_EPI_INT && g->tc != SKL_DT_I32) return 0;
  if (g->epilogue == SKL_EPI_FLOAT && g->tc == SKL_DT_I32) return 0;
  return 1;
}

extern "C" int skl_b200_launch_gemv_i8(const skl_b200_gemm_args *g, void *stream) {
  GemvParams p;
  p.x = (const int8_t *)g->a;
  p.w = (const int8_t *)g->b;
  p.c = g->c;
  p.ldx = g->rsa0;
  p.ldw = g->csb0;
  p.rsc = g->rsc0;
  p.csc = g->csc0;
  p.m = (int)g->m0;
  p.n = (int)g->n0;
  p.k = (int)g->k0;
  p.epilogue = g->epilogue;
  p.tc = g->tc;
  p.alpha_i = g->alpha_i;
  p.beta_i = g->beta_i;
  p.alpha_f = g->alpha_f;
  p.beta_f = g->beta_f;
  p.row_scale = g->row_scale;
  p.col_scale = g->col_scale;
  int mp = 1;
  while (mp < p.m) mp <<= 1;
  const size_t smem = (size_t)mp * p.k;
  const int groups = (p.n + GV_R - 1) / GV_R;
  int grid = num_sms();
  if (grid > groups) grid = groups;
  cudaStream_t s = (cudaStream_t)stream;
  cudaError_t e = cudaSuccess;
#define GV_LAUNCH(MPV)                                                                            \
  do {                                                                                            \
    if (smem > 48 * 1024)                                                                         \
      e = cudaFuncSetAttribute(gemv_i8_kernel<MPV>, cudaFuncAttributeMaxDynamicSharedMemorySize,  \
                               (int)smem);                                                        \
    if (e == cudaSuccess) gemv_i8_kernel<MPV><<<grid, GV_THREADS, smem, s>>>(p);                  \
  } while (0)
  switch (mp) {
    case 1: GV_LAUNCH(1); break;
    case 2: GV_LAUNCH(2); break;
    case 4: GV_LAUNCH(4); break;
    case 8: GV_LAUNCH(8); break;
    default: GV_LAUNCH(16); break;
  }
#undef GV_LAUNCH
  if (e != cudaSuccess) return (int)e;
  SKLB_COUNT_LAUNCH();
  return (int)cudaGetLastError();
}
