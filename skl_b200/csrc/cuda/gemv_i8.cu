// gemv_i8.cu -- skinny int8 GEMM (m <= 16): the decode-shape case.
//
// C[i, j] = sum_k A[i, k] * B[k, j] with A = activations (m rows, k contiguous) and B = weights stored
// one output column per contiguous k-run ("[N][K]": rsb == 1, csb == row pitch).  With m this small
// the arithmetic intensity is at most 2*m ops per weight byte, far below the tensor-core ridge, so
// the kernel is a weight-streaming kernel bounded by HBM bandwidth.  No tensor cores.  SKL's
// counterpart is the m == 1 branch of its int8 kernel
// (src/gemm/gemm_i8rcp1x4_i8p4x1c_i32_xsfvqdotq.c:543-632, dispatch :645-658).
//
// Design: one CTA of 8 warps per SM.  Every warp of the grid owns a contiguous, near-equal range of
// weight rows and is its own producer and consumer: lane 0 streams row segments (up to 2 KiB each)
// into a private ring in shared memory with cp.async.bulk, completion signalled on one mbarrier per
// ring slot; the warp then consumes four rows at a time -- 16-byte shared-memory loads of the weights
// and of the activations (copied to shared memory once per CTA), dp4a, a butterfly warp-shuffle fold
// of the k-split, fused alpha/beta or dequantising epilogue -- and refills the slots it just drained.
// The rings hold 130-190 KiB per SM in flight, independent of register pressure, which is what a
// 6.5 TB/s stream needs to cover HBM latency.  Every mbarrier wait is bounded; on expiry the warp
// records a code in the status words and stops.
// Algorithmic bytes per launch: N*K (weights) + m*K (activations) + output and scale vectors.
#include "numerics.cuh"

namespace sklb {
namespace {

constexpr int GV_THREADS = 256;
constexpr int GV_WARPS = GV_THREADS / 32;
constexpr int GV_R = 4;
constexpr uint32_t GV_ERR_WAIT = 0x201;

struct GemvParams {
  const int8_t *x;  // activations, row i at x + i*ldx
  const int8_t *w;  // weights, output column j at w + j*ldw
  void *c;
  int64_t ldx, ldw, rsc, csc;
  int m, n, k;
  int seg_bytes, nseg, stages;  // ring geometry: slot size, segments per row, slots per warp
  int epilogue, tc;
  int32_t alpha_i, beta_i;
  float alpha_f, beta_f;
  const float *row_scale, *col_scale, *bias;
  float *global_max;
  int activation;
  float act_param;
  int overlap;  // launched as a programmatic dependent: see the kernel's first lines
  uint32_t *status;
};

__device__ __forceinline__ uint32_t gv_smem_u32(const void *p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ bool gv_try(uint32_t bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(bar), "r"(parity)
      : "memory");
  return ok != 0;
}

// Bounded wait (about two seconds).  false = gave up; the status word then holds GV_ERR_WAIT.
__device__ __forceinline__ bool gv_wait(uint32_t bar, uint32_t parity, uint32_t *status) {
  if (gv_try(bar, parity)) return true;
  uint64_t t0 = 0;
  for (uint32_t spins = 1;; ++spins) {
    if (gv_try(bar, parity)) return true;
    if ((spins & 63u) == 0u) {
      uint64_t now;
      asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(now));
      if (t0 == 0) t0 = now;
      if (now - t0 > 2000000000ull) {
        atomicCAS(status, 0u, GV_ERR_WAIT);
        return false;
      }
    }
  }
}

__device__ __forceinline__ void gv_bulk_load(uint32_t dst, const void *src, uint32_t bytes, uint32_t bar) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
  asm volatile(
      "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(dst),
      "l"(src), "r"(bytes), "r"(bar)
      : "memory");
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
      for (int i = 0; i < (V > 1 ? V / 2 : 1); ++i) {
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

// rs / cs: the row and column scale of this element, fetched ahead of time (1.0f when absent; the
// multiplication is skipped then, so the result is the same as without a scale vector).
// Returns the stored value (float epilogue) for the optional global maximum, else -INFINITY.
__device__ __forceinline__ float gemv_store(const GemvParams &p, int mi, int j, int32_t a, float rs, float cs,
                                            float bias) {
  const int64_t o = (int64_t)mi * p.rsc + (int64_t)j * p.csc;
  if (p.epilogue == SKL_EPI_INT) {
    int32_t *cp = (int32_t *)p.c + o;
    uint32_t old = p.beta_i != 0 ? (uint32_t)p.beta_i * (uint32_t)*cp : 0u;
    *cp = (int32_t)(old + (uint32_t)p.alpha_i * (uint32_t)a);
    return -INFINITY;
  }
  float v = __fmul_rn(p.alpha_f, (float)a);
  if (p.row_scale) v = __fmul_rn(v, rs);
  if (p.col_scale) v = __fmul_rn(v, cs);
  if (p.bias) v = __fadd_rn(v, bias);
  if (p.beta_f != 0.0f) v = __fadd_rn(__fmul_rn(p.beta_f, load_c_f32(p.tc, p.c, o)), v);
  if (p.activation)
    v = activation_value(p.activation, p.act_param, v, p.activation == SKL_ACT_SWIGLU ? load_c_f32(p.tc, p.c, o) : 0.0f);
  store_c_f32(p.tc, p.c, o, v);
  return (v == v) ? v : -INFINITY;
}

template <int MP>
__global__ void __launch_bounds__(GV_THREADS, 1) gemv_i8_kernel(const GemvParams p) {
  extern __shared__ __align__(128) uint8_t gv_smem[];
  // layout: activations [MP][k] | rings [warps][stages][seg_bytes] | barriers [warps][stages]
  const int kc = p.k >> 4;
  uint4 *xs = reinterpret_cast<uint4 *>(gv_smem);
  const uint32_t x_bytes = ((uint32_t)MP * (uint32_t)p.k + 127u) & ~127u;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int S = p.stages, SEG = p.seg_bytes, NSEG = p.nseg;
  uint8_t *ring = gv_smem + x_bytes + (size_t)warp * S * SEG;
  const uint32_t ring_s = gv_smem_u32(ring);
  const uint32_t bars = gv_smem_u32(gv_smem + x_bytes + (size_t)GV_WARPS * S * SEG) + warp * S * 8;

  // this warp's rows
  const int64_t gw = (int64_t)blockIdx.x * GV_WARPS + warp;
  const int64_t nw = (int64_t)gridDim.x * GV_WARPS;
  const int row_begin = (int)(((int64_t)p.n * gw) / nw);
  const int row_end = (int)(((int64_t)p.n * (gw + 1)) / nw);
  const int nrows = row_end - row_begin;
  const int full_groups = nrows / GV_R, tail_rows = nrows - full_groups * GV_R;
  const int items_full = full_groups * GV_R * NSEG;
  const int n_items = nrows * NSEG;

  // Producer side.  Items (row segments) are issued in the order they are consumed: group, segment,
  // row in group.  `pq` counts issued items and is uniform across the warp; lane l issues item pq + l,
  // so a refill of up to 4 slots, and the initial fill of the whole ring, cost one item's worth of
  // address arithmetic instead of a serial loop on one lane.
  int pq = 0;
  const int group_items = GV_R * NSEG;
  auto issue = [&](int count) {  // issue items pq .. pq+count-1, count <= 32, uniform
    const int q = pq + lane;
    if (lane < count && q < n_items) {
      int row, seg;
      if (q < items_full) {
        const int g = q / group_items, w = q - g * group_items;
        seg = w / GV_R;
        row = row_begin + g * GV_R + (w - seg * GV_R);
      } else {
        const int w = q - items_full;
        seg = w / tail_rows;
        row = row_begin + full_groups * GV_R + (w - seg * tail_rows);
      }
      const int off = seg * SEG;
      const uint32_t bytes = (uint32_t)((p.k - off) < SEG ? (p.k - off) : SEG);
      const int slot = q % S;
      gv_bulk_load(ring_s + slot * SEG, p.w + (int64_t)row * p.ldw + off, bytes, bars + slot * 8);
    }
    pq += count;
  };

  // Overlapped launch (the caller declared the weights static): let the next launch on the stream start on
  // each SM as soon as this one's CTA there has left, and -- being such a dependent launch itself -- start
  // the weight stream at once but wait for the previous kernel to finish before touching anything that
  // kernel may have written (activations, scales, bias, C).
  if (p.overlap) asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  if (lane < S) asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"(bars + lane * 8));
  asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
  __syncwarp();
  issue(S);  // weights start streaming before the activations are staged
  if (p.overlap) asm volatile("griddepcontrol.wait;" ::: "memory");
  for (int e = threadIdx.x; e < MP * kc; e += GV_THREADS) {
    int mi = e / kc, ch = e - mi * kc;
    uint4 v = make_uint4(0, 0, 0, 0);
    if (mi < p.m) v = *reinterpret_cast<const uint4 *>(p.x + (int64_t)mi * p.ldx + (int64_t)ch * 16);
    xs[e] = v;
  }
  __syncthreads();

  int q0 = 0, c_slot = 0;
  uint32_t c_par = 0;  // parity of the ring pass the consumer is in
  bool ok = true;
  float warp_max = -INFINITY;  // this lane's largest result so far (optional global maximum)
  for (int g = 0; ok && q0 < n_items; ++g) {
    const int rc = g < full_groups ? GV_R : tail_rows;  // rows in this group
    const int row0 = row_begin + g * GV_R;
    int32_t acc[GV_R * MP];
#pragma unroll
    for (int i = 0; i < GV_R * MP; ++i) acc[i] = 0;
    // scales this lane will need after the fold, requested now so their latency hides behind the stream
    constexpr int V = GV_R * MP;
    constexpr int W = V >= 32 ? V / 32 : 1;
    constexpr int LOGV = V >= 32 ? 5 : (V == 16 ? 4 : (V == 8 ? 3 : 2));
    const int share = 5 - LOGV;  // 2^share lanes hold the same finished value
    float rs_pre[W], cs_pre[W], bias_pre[W];
#pragma unroll
    for (int w = 0; w < W; ++w) {
      const int idx = (lane >> share) * W + w;  // = r*MP + mi
      const int r = idx / MP, mi = idx - r * MP;
      rs_pre[w] = (p.row_scale && mi < p.m) ? __ldg(p.row_scale + mi) : 1.0f;
      cs_pre[w] = (p.col_scale && r < rc) ? __ldg(p.col_scale + row0 + r) : 1.0f;
      bias_pre[w] = (p.bias && r < rc) ? __ldg(p.bias + row0 + r) : 0.0f;
    }

    for (int seg = 0; seg < NSEG && ok; ++seg) {
      const int off = seg * SEG;
      const int nch = ((p.k - off) < SEG ? (p.k - off) : SEG) >> 4;
      uint32_t slot_addr[GV_R];
      {
        int sl = c_slot;
        uint32_t par = c_par;
        const int sl0 = c_slot;
#pragma unroll
        for (int r = 0; r < GV_R; ++r) {
          if (r < rc) {
            slot_addr[r] = ring_s + sl * SEG;
            if (ok) ok = gv_wait(bars + sl * 8, par, p.status);
            if (++sl == S) {
              sl = 0;
              par ^= 1u;
            }
          } else {
            slot_addr[r] = ring_s + sl0 * SEG;  // placeholder: a valid slot whose result is discarded
          }
        }
        c_slot = sl;
        c_par = par;
      }
      ok = __all_sync(0xFFFFFFFFu, ok);
      if (!ok) break;
      const uint4 *xseg = xs + (off >> 4);
#pragma unroll 2
      for (int ch = lane; ch < nch; ch += 32) {
        uint4 wv[GV_R];
#pragma unroll
        for (int r = 0; r < GV_R; ++r) {
          asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];"
                       : "=r"(wv[r].x), "=r"(wv[r].y), "=r"(wv[r].z), "=r"(wv[r].w)
                       : "r"(slot_addr[r] + ch * 16));
        }
#pragma unroll
        for (int mi = 0; mi < MP; ++mi) {
          const uint4 xv = xseg[mi * kc + ch];
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
      __syncwarp();  // every lane is done reading these slots before they are refilled
      issue(rc);
      q0 += rc;
    }
    if (!ok) break;

    warp_fold<GV_R * MP>(acc, lane);
    if ((lane & ((1 << share) - 1)) == 0) {  // one writer per value
#pragma unroll
      for (int w = 0; w < W; ++w) {
        const int idx = (lane >> share) * W + w;  // = r*MP + mi
        const int r = idx / MP, mi = idx - r * MP;
        if (r < rc && mi < p.m)
          warp_max = fmaxf(warp_max, gemv_store(p, mi, row0 + r, acc[w], rs_pre[w], cs_pre[w], bias_pre[w]));
      }
    }
  }
  if (p.global_max) {
    warp_max = warp_max_f32(warp_max);
    if (lane == 0 && warp_max != -INFINITY) atomic_max_f32(p.global_max, warp_max);
  }
}

constexpr size_t GV_MAX_X = 96 * 1024;        // activations in shared memory
constexpr size_t GV_SMEM_BUDGET = 224 * 1024;  // per CTA, of the 227 KiB an SM offers

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
  if ((size_t)mp * g->k0 > GV_MAX_X) return 0;
  if (g->epilogue == SKL_EPI_INT && g->tc != SKL_DT_I32) return 0;
  if (g->epilogue == SKL_EPI_FLOAT && g->tc == SKL_DT_I32) return 0;
  return 1;
}

extern "C" int skl_b200_launch_gemv_i8(const skl_b200_gemm_args *g, uint32_t *dev_status, void *stream) {
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
  p.bias = g->bias;
  p.global_max = g->global_max;
  p.activation = g->activation;
  p.act_param = g->act_param;
  p.overlap = g->b_static ? 1 : 0;
  p.status = dev_status;
  int mp = 1;
  while (mp < p.m) mp <<= 1;
  // ring geometry: slots of up to 2 KiB, at least 2*R slots per warp, as many as shared memory allows
  const size_t x_bytes = ((size_t)mp * p.k + 127) & ~(size_t)127;
  int seg = p.k < 2048 ? p.k : 2048;
  size_t room = GV_SMEM_BUDGET - x_bytes - 1024;
  int stages = (int)(room / ((size_t)GV_WARPS * seg));
  while (stages < 2 * GV_R && seg > 256) {
    seg >>= 1;
    seg &= ~15;
    stages = (int)(room / ((size_t)GV_WARPS * seg));
  }
  // Two groups of rows per warp are enough to keep HBM busy (128 KiB in flight per SM); deeper rings
  // measured slower at every size tried (the first burst of requests grows, the steady state does not).
  if (stages > 2 * GV_R) stages = 2 * GV_R;
  if (stages < GV_R) return (int)cudaErrorInvalidValue;
  p.seg_bytes = seg;
  p.nseg = (p.k + seg - 1) / seg;
  p.stages = stages;
  const size_t smem = x_bytes + (size_t)GV_WARPS * stages * seg + (size_t)GV_WARPS * stages * 8;
  int grid = num_sms();
  const int want = (p.n + GV_WARPS - 1) / GV_WARPS;  // at least one row per warp
  if (grid > want) grid = want;
  cudaStream_t s = (cudaStream_t)stream;
  cudaError_t e = cudaSuccess;
#define GV_LAUNCH(MPV)                                                                             \
  do {                                                                                             \
    static bool attr_set[64] = {}; /* per device */                                                \
    int dev = 0;                                                                                   \
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) dev = 0;                       \
    if (!attr_set[dev]) {                                                                          \
      e = cudaFuncSetAttribute(gemv_i8_kernel<MPV>, cudaFuncAttributeMaxDynamicSharedMemorySize,   \
                               (int)GV_SMEM_BUDGET);                                               \
      attr_set[dev] = (e == cudaSuccess);                                                          \
    }                                                                                              \
    if (e == cudaSuccess) {                                                                        \
      cudaLaunchConfig_t cfg = {};                                                                 \
      cfg.gridDim = dim3((unsigned)grid);                                                          \
      cfg.blockDim = dim3(GV_THREADS);                                                             \
      cfg.dynamicSmemBytes = smem;                                                                 \
      cfg.stream = s;                                                                              \
      cudaLaunchAttribute attr[1];                                                                 \
      attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;                             \
      attr[0].val.programmaticStreamSerializationAllowed = 1;                                      \
      cfg.attrs = attr;                                                                            \
      cfg.numAttrs = p.overlap ? 1 : 0;                                                            \
      e = cudaLaunchKernelEx(&cfg, gemv_i8_kernel<MPV>, p);                                        \
    }                                                                                              \
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
