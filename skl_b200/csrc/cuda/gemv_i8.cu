// gemv_i8.cu -- skinny int8 GEMM (m <= 16): the decode-shape case.
//
// C[i, j] = sum_k A[i, k] * B[k, j] with A = activations (m rows, k contiguous) and B = weights stored
// one output column per contiguous k-run ("[N][K]": rsb == 1, csb == row pitch).  With m this small
// the arithmetic intensity is at most 2*m ops per weight byte, far below the tensor-core ridge, so
// the kernel is a weight-streaming kernel bounded by HBM bandwidth.  SKL's counterpart is the m == 1
// branch of its int8 kernel (src/gemm/gemm_i8rcp1x4_i8p4x1c_i32_xsfvqdotq.c:543-632, dispatch :645-658).
//
// Design.  A plain 16-byte-per-thread read of the weight matrix with 128 KiB of loads in flight per SM runs
// at 0.96 of the device's copy bandwidth at this size; staging the rows through shared memory with bulk
// copies measured 20-50 % slower.  So the kernel IS that read, with the arithmetic hung on it:
//   * One CTA of 16 warps per SM; every thread keeps 16 independent 16-byte loads (ld.global.nc, no L1
//     allocation) in flight in registers.
//   * The weight rows are dealt to the CTAs in layers: layer l is a run of consecutive rows cut into one
//     piece per CTA, so at any moment all CTAs read neighbouring rows and every CTA gets the same number
//     of bytes to within one row.  A piece is up to 8 rows (more when k is short).
//   * Inside a CTA the k range is split over the warps in 128-byte blocks, so the warps are balanced
//     whatever the row count.  One warp-wide load fetches 64 bytes of each of 8 rows: lane (g, t) holds
//     bytes [16t, 16t+16) of row g -- the operand layout of mma.m16n8k32 with the 8 weight rows as its
//     8-column operand (the k order inside a fragment is a fixed permutation applied to both operands).
//       m <= 2   dp4a on that chunk against the same chunk of the activations, two shuffles fold the
//                four lanes of a row.  No tensor cores.
//       m >= 3   mma.sync.m16n8k32.s8 with the activations as the 16-row operand: dp4a cannot keep up
//                with HBM here (4*m dp4a per 16 weight bytes on a two-per-clock pipe).
//     The activations sit in shared memory, rows 64 bytes off the 128-byte grid so that the fragment loads
//     of neighbouring rows hit different banks.
//   * A warp's partial sums go to its own slice of shared memory without any synchronisation; after the
//     CTA's last piece (or every `round` pieces when there are many) one barrier, then one thread per
//     output adds the partial sums and runs the fused alpha/beta or dequantising epilogue.  int32 sums wrap
//     around like the reference's, in any order, so the result is exact.
// The kernel has no waits on barriers that another agent completes, hence nothing that could time out.
//
// Launch overlap.  The kernel lets its successor on the stream start early (griddepcontrol) and is itself
// launched as such a dependent; it waits for its predecessor before its first global read.  When the caller
// declared the weights static the first loads of the weight stream are issued before that wait.
// Algorithmic bytes per launch: N*K (weights) + m*K (activations) + output and scale vectors.
#include <cstdlib>

#include "numerics.cuh"

namespace sklb {
namespace {

constexpr int GV_WARPS = 16;
constexpr int GV_THREADS = GV_WARPS * 32;
constexpr int GV_G = 8;            // weight rows per warp-wide load (the 8-column operand of one mma)
constexpr int GV_INFLIGHT = 16;    // 16-byte loads a thread keeps in flight
constexpr int GV_OUT_PER_THREAD = 4;  // outputs one thread finishes per round, at most
constexpr int GV_MATH_DP4A = 0, GV_MATH_MMA = 1;

struct GemvParams {
  const int8_t *x;  // activations, row i at x + i*ldx
  const int8_t *w;  // weights, output column j at w + j*ldw
  void *c;
  int64_t ldx, ldw, rsc, csc;
  int m, n, k;
  int ksplit_log2;    // warps sharing one group of 8 rows: KS = 1 << ksplit_log2 (they split k in 128-byte blocks)
  int piece_rows;     // rows of one piece = 8 * (GV_WARPS / KS)
  int xpitch;         // bytes between activation rows in shared memory (64 mod 128)
  int layers;         // pieces per CTA
  int round;          // pieces between two reductions
  // layer l covers rows [l*lq + min(l, lr), +lq + (l < lr)); a layer of length len is cut into gridDim.x pieces,
  // piece b = [b*pq + min(b, pr), +pq + (b < pr)) with (pq, pr) = (len / grid, len % grid), given for both lengths
  int lq, lr, pq0, pr0, pq1, pr1;
  int epilogue, tc;
  int32_t alpha_i, beta_i;
  float alpha_f, beta_f;
  const float *row_scale, *col_scale, *bias;
  float *global_max;
  int activation;
  float act_param;
  int overlap;  // the weights were declared static: the first loads are issued before waiting for the predecessor
};

__device__ __forceinline__ uint32_t gv_smem_u32(const void *p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ uint4 gv_ldg(const void *p) {
  uint4 v;
  asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
               : "l"(p));
  return v;
}
__device__ __forceinline__ uint4 gv_lds128(uint32_t addr) {
  uint4 v;
  asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(addr));
  return v;
}
// D (16 x 8, int32) += A (16 x 32, int8, row) * B (32 x 8, int8, col); sums wrap around.
__device__ __forceinline__ void gv_mma(int32_t (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                       uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k32.row.col.s32.s8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
      : "+r"(d[0]), "+r"(d[1]), "+r"(d[2]), "+r"(d[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
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

// First row and row count of the piece CTA `b` takes from layer `l` (no divisions: see GemvParams).
__device__ __forceinline__ void gv_piece(const GemvParams &p, int l, int b, int &r0, int &nr) {
  const bool longer = l < p.lr;
  const int lo = l * p.lq + (l < p.lr ? l : p.lr);
  const int pq = longer ? p.pq1 : p.pq0, pr = longer ? p.pr1 : p.pr0;
  r0 = lo + b * pq + (b < pr ? b : pr);
  nr = pq + (b < pr ? 1 : 0);
}

// MATH: GV_MATH_DP4A with MP in {1, 2} (activation rows, padded), or GV_MATH_MMA with MP in {8, 16}.
// NBW: 128-byte k blocks per warp and group (1, 2, 4 or 8: k up to 2048 * NBW bytes at a 16-way split).
template <int MATH, int MP, int NBW>
__global__ void __launch_bounds__(GV_THREADS, 1) gemv_i8_kernel(const GemvParams p) {
  constexpr int L = 2 * NBW;           // 16-byte loads per lane and piece: two 64-byte halves of every block
  constexpr int U = GV_INFLIGHT / L;   // pieces in flight
  constexpr int NOUT = GV_G * MP;      // outputs per group of 8 rows
  extern __shared__ __align__(128) uint8_t gv_smem[];
  // layout: activations [MP][xpitch] | partial sums [round][GV_WARPS][NOUT]
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int g = lane >> 2, t = lane & 3;
  const int KS = 1 << p.ksplit_log2;
  const int ks = warp & (KS - 1), rs = warp >> p.ksplit_log2;  // this warp's share of k and its group inside a piece
  const uint32_t x_s = gv_smem_u32(gv_smem);
  int32_t *red = reinterpret_cast<int32_t *>(gv_smem + (size_t)MP * p.xpitch);
  const int b = (int)blockIdx.x;

  // The next kernel on the stream may be scheduled from now on (it waits for this one where it must).
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  if (!p.overlap) asm volatile("griddepcontrol.wait;" ::: "memory");

  uint4 wv[U][L];
  // Requests the loads of piece `l` into one register set.  Lane (g, t) fetches, for every 128-byte block this warp
  // owns, bytes [16t, 16t+16) of both 64-byte halves of row g of the warp's group; rows and k past the end read as 0.
  auto issue = [&](uint4 (&dst)[L], int l) {
    int r0, nr;
    gv_piece(p, l, b, r0, nr);
    const int row = rs * GV_G + g;
    const bool row_ok = row < nr;
    const int8_t *src = p.w + (int64_t)(r0 + row) * p.ldw + t * 16;
#pragma unroll
    for (int j = 0; j < NBW; ++j) {
#pragma unroll
      for (int h = 0; h < 2; ++h) {
        const int off = ((ks + (j << p.ksplit_log2)) << 7) + h * 64;
        dst[2 * j + h] = (row_ok && off + t * 16 < p.k) ? gv_ldg(src + off) : make_uint4(0, 0, 0, 0);
      }
    }
  };

#pragma unroll
  for (int u = 0; u < U; ++u)
    if (u < p.layers) issue(wv[u], u);
  if (p.overlap) asm volatile("griddepcontrol.wait;" ::: "memory");

  // Activations -> shared memory (rows past m are zero), while the first weights are on their way.
  {
    const int chunks = p.k >> 4;
    for (int e = tid; e < MP * chunks; e += GV_THREADS) {
      const int mi = e / chunks, ch = e - mi * chunks;
      uint4 v = make_uint4(0, 0, 0, 0);
      if (mi < p.m) v = *reinterpret_cast<const uint4 *>(p.x + (int64_t)mi * p.ldx + (int64_t)ch * 16);
      *reinterpret_cast<uint4 *>(gv_smem + (size_t)mi * p.xpitch + (size_t)ch * 16) = v;
    }
  }
  __syncthreads();

  float my_max = -INFINITY;
  const int groups_per_piece = GV_WARPS >> p.ksplit_log2;
  for (int base = 0; base < p.layers; base += p.round) {
    const int count = (p.layers - base) < p.round ? (p.layers - base) : p.round;
    // Scales and bias of the outputs this thread will finish after this round, requested now so that their latency
    // hides behind the stream.  Output o of the round: piece o / (groups * NOUT), then group, then mi*8 + row.
    float cs_pre[GV_OUT_PER_THREAD], bias_pre[GV_OUT_PER_THREAD];
    const int per_piece = groups_per_piece * NOUT, total = count * per_piece;
#pragma unroll
    for (int q = 0; q < GV_OUT_PER_THREAD; ++q) {
      cs_pre[q] = 1.0f;
      bias_pre[q] = 0.0f;
      const int o = tid + q * GV_THREADS;
      if (o < total && (p.col_scale || p.bias)) {
        const int pc = o / per_piece, rem = o - pc * per_piece;
        const int grp = rem / NOUT, wr = (rem - grp * NOUT) & 7;
        int r0, nr;
        gv_piece(p, base + pc, b, r0, nr);
        const int row = grp * GV_G + wr;
        if (row < nr) {
          if (p.col_scale) cs_pre[q] = __ldg(p.col_scale + r0 + row);
          if (p.bias) bias_pre[q] = __ldg(p.bias + r0 + row);
        }
      }
    }

    for (int l0 = 0; l0 < count; l0 += U) {
#pragma unroll
      for (int u = 0; u < U; ++u) {
        const int l = l0 + u;  // piece inside the round; (base + l) % U == u because round is a multiple of U
        if (l < count) {
          int32_t acc[MATH == GV_MATH_MMA ? 4 : MP];
#pragma unroll
          for (int i = 0; i < (MATH == GV_MATH_MMA ? 4 : MP); ++i) acc[i] = 0;
#pragma unroll
          for (int j = 0; j < NBW; ++j) {
#pragma unroll
            for (int h = 0; h < 2; ++h) {
              const int off = ((ks + (j << p.ksplit_log2)) << 7) + h * 64;
              if (off < p.k) {  // uniform across the warp
                const uint4 wq = wv[u][2 * j + h];
                const uint32_t xa_addr = x_s + (uint32_t)off + (uint32_t)t * 16;
                if constexpr (MATH == GV_MATH_DP4A) {
#pragma unroll
                  for (int mi = 0; mi < MP; ++mi) {
                    const uint4 xq = gv_lds128(xa_addr + mi * p.xpitch);
                    int32_t a = acc[mi];
                    a = __dp4a((int)wq.x, (int)xq.x, a);
                    a = __dp4a((int)wq.y, (int)xq.y, a);
                    a = __dp4a((int)wq.z, (int)xq.z, a);
                    a = __dp4a((int)wq.w, (int)xq.w, a);
                    acc[mi] = a;
                  }
                } else {
                  const uint4 xa = gv_lds128(xa_addr + g * p.xpitch);
                  if constexpr (MP == 16) {
                    const uint4 xb = gv_lds128(xa_addr + (g + 8) * p.xpitch);
                    gv_mma(acc, xa.x, xb.x, xa.y, xb.y, wq.x, wq.y);
                    gv_mma(acc, xa.z, xb.z, xa.w, xb.w, wq.z, wq.w);
                  } else {
                    gv_mma(acc, xa.x, 0u, xa.y, 0u, wq.x, wq.y);
                    gv_mma(acc, xa.z, 0u, xa.w, 0u, wq.z, wq.w);
                  }
                }
              }
            }
          }
          // the registers are free again: request the piece U further on (possibly of the next round)
          if (base + l + U < p.layers) issue(wv[u], base + l + U);
          // this warp's partial sums for its group of the piece, index mi*8 + row
          int32_t *mine = red + ((size_t)l * GV_WARPS + warp) * NOUT;
          if constexpr (MATH == GV_MATH_DP4A) {
#pragma unroll
            for (int mi = 0; mi < MP; ++mi) {
              int32_t a = acc[mi];
              a += __shfl_xor_sync(0xFFFFFFFFu, a, 1);
              a += __shfl_xor_sync(0xFFFFFFFFu, a, 2);
              if (t == 0) mine[mi * 8 + g] = a;
            }
          } else {
            // lane (g, t) holds D[g][2t], D[g][2t+1], D[g+8][2t], D[g+8][2t+1]: activation row x weight row
            *reinterpret_cast<int2 *>(mine + g * 8 + 2 * t) = make_int2(acc[0], acc[1]);
            if constexpr (MP == 16) *reinterpret_cast<int2 *>(mine + (g + 8) * 8 + 2 * t) = make_int2(acc[2], acc[3]);
          }
        }
      }
    }
    __syncthreads();
    // one thread per output: add the KS partial sums, run the epilogue
#pragma unroll
    for (int q = 0; q < GV_OUT_PER_THREAD; ++q) {
      const int o = tid + q * GV_THREADS;
      if (o < total) {
        const int pc = o / per_piece, rem = o - pc * per_piece;
        const int grp = rem / NOUT, idx = rem - grp * NOUT;
        const int mi = idx >> 3, wr = idx & 7;
        int r0, nr;
        gv_piece(p, base + pc, b, r0, nr);
        const int row = grp * GV_G + wr;
        if (row < nr && mi < p.m) {
          const int32_t *src = red + ((size_t)pc * GV_WARPS + (grp << p.ksplit_log2)) * NOUT + idx;
          int32_t sum = 0;
          for (int s = 0; s < KS; ++s) sum += src[s * NOUT];
          const float rsc = p.row_scale ? __ldg(p.row_scale + mi) : 1.0f;
          my_max = fmaxf(my_max, gemv_store(p, mi, r0 + row, sum, rsc, cs_pre[q], bias_pre[q]));
        }
      }
    }
    if (base + p.round < p.layers) __syncthreads();  // the partial sums are rewritten by the next round
  }
  if (p.global_max) {
    my_max = warp_max_f32(my_max);
    if (lane == 0 && my_max != -INFINITY) atomic_max_f32(p.global_max, my_max);
  }
}

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

constexpr size_t GV_SMEM_MAX = 200 * 1024;

// Activation rows the kernel variant for m carries (dp4a: m itself; mma: 8 or 16).
inline int padded_m(int m) { return m <= 2 ? m : (m <= 8 ? 8 : 16); }
inline int x_pitch(int k) { return ((k + 63) / 128) * 128 + 64; }

}  // namespace
}  // namespace sklb

using namespace sklb;

extern "C" int skl_b200_gemv_i8_supported(const skl_b200_gemm_args *g) {
  if (g->ta != SKL_DT_I8 || g->tb != SKL_DT_I8) return 0;
  if (g->m1 != 1 || g->n1 != 1 || g->k1 != 1) return 0;
  if (g->m0 == 0 || g->m0 > 16 || g->n0 == 0 || g->k0 == 0) return 0;
  if (g->csa0 != 1 || g->rsb0 != 1) return 0;
  if ((g->k0 & 15) != 0 || g->k0 > 16384 || g->n0 > (1u << 30)) return 0;  // 8 blocks of 128 bytes per warp
  if (!al16(g->a) || !al16(g->b)) return 0;
  if ((g->m0 > 1 && (g->rsa0 & 15) != 0) || (g->n0 > 1 && (g->csb0 & 15) != 0)) return 0;
  // the activations and the partial sums of eight pieces (as many as can be in flight) must fit in shared memory
  const int mp = padded_m((int)g->m0);
  if ((size_t)mp * x_pitch((int)g->k0) + 8 * (size_t)GV_WARPS * GV_G * mp * 4 > GV_SMEM_MAX) return 0;
  if (g->epilogue == SKL_EPI_INT && g->tc != SKL_DT_I32) return 0;
  if (g->epilogue == SKL_EPI_FLOAT && g->tc == SKL_DT_I32) return 0;
  return 1;
}

extern "C" int skl_b200_launch_gemv_i8(const skl_b200_gemm_args *g, uint32_t *dev_status, void *stream) {
  (void)dev_status;  // no device-side waits in this kernel
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

  // k split: the 128-byte blocks of a row go round the KS warps that share a group of 8 rows; KS is the largest
  // power of two (at most 16) not above the block count, the other warps take further groups of the same piece.
  const int blocks = (p.k + 127) / 128;
  int ks_log2 = 0;
  while (ks_log2 < 4 && (2 << ks_log2) <= blocks) ++ks_log2;
  const int KS = 1 << ks_log2;
  const int nbw_need = (blocks + KS - 1) / KS;  // 1..8 since k <= 16384
  int nbw = 1;
  while (nbw < nbw_need) nbw <<= 1;
  p.ksplit_log2 = ks_log2;
  p.piece_rows = GV_G * (GV_WARPS / KS);
  p.xpitch = x_pitch(p.k);
  const int mp = padded_m(p.m);
  const int nout = GV_G * mp;

  int grid = num_sms();
  {
    const int want = (p.n + GV_G - 1) / GV_G;  // at least one group of rows per CTA
    if (grid > want) grid = want;
  }
  p.layers = (int)(((int64_t)p.n + (int64_t)p.piece_rows * grid - 1) / ((int64_t)p.piece_rows * grid));
  p.lq = p.n / p.layers;
  p.lr = p.n % p.layers;
  p.pq0 = p.lq / grid;
  p.pr0 = p.lq % grid;
  p.pq1 = (p.lq + 1) / grid;
  p.pr1 = (p.lq + 1) % grid;

  // pieces per round: bounded by the outputs a thread can finish (its scale registers) and by shared memory;
  // a multiple of the pieces in flight so that a piece always lands in the same register set
  const int u = GV_INFLIGHT / (2 * nbw);
  const size_t x_bytes = (size_t)mp * p.xpitch;
  const size_t piece_red = (size_t)GV_WARPS * nout * 4;
  int round = (GV_OUT_PER_THREAD * GV_THREADS) / ((GV_WARPS / KS) * nout);
  const int by_smem = (int)((GV_SMEM_MAX - x_bytes) / piece_red);
  if (round > by_smem) round = by_smem;
  round = round / u * u;
  if (round < u) return (int)cudaErrorInvalidValue;
  if (round > ((p.layers + u - 1) / u) * u) round = ((p.layers + u - 1) / u) * u;
  p.round = round;
  const size_t smem = x_bytes + (size_t)round * piece_red;

  cudaStream_t s = (cudaStream_t)stream;
  cudaError_t e = cudaSuccess;
#define GV_LAUNCH(MATHV, MPV, NBWV)                                                                          \
  do {                                                                                                       \
    static bool attr_set[64] = {}; /* per device */                                                          \
    int dev = 0;                                                                                             \
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) dev = 0;                                 \
    if (!attr_set[dev]) {                                                                                    \
      e = cudaFuncSetAttribute(gemv_i8_kernel<MATHV, MPV, NBWV>, cudaFuncAttributeMaxDynamicSharedMemorySize, \
                               (int)GV_SMEM_MAX);                                                            \
      attr_set[dev] = (e == cudaSuccess);                                                                    \
    }                                                                                                        \
    if (e == cudaSuccess) {                                                                                  \
      cudaLaunchConfig_t cfg = {};                                                                           \
      cfg.gridDim = dim3((unsigned)grid);                                                                    \
      cfg.blockDim = dim3(GV_THREADS);                                                                       \
      cfg.dynamicSmemBytes = smem;                                                                           \
      cfg.stream = s;                                                                                        \
      cudaLaunchAttribute attr[1];                                                                           \
      attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;                                       \
      attr[0].val.programmaticStreamSerializationAllowed = 1;                                                \
      cfg.attrs = attr;                                                                                      \
      cfg.numAttrs = 1;                                                                                      \
      e = cudaLaunchKernelEx(&cfg, gemv_i8_kernel<MATHV, MPV, NBWV>, p);                                     \
    }                                                                                                        \
  } while (0)
#define GV_LAUNCH_NBW(MATHV, MPV)              \
  do {                                         \
    if (nbw == 1)                              \
      GV_LAUNCH(MATHV, MPV, 1);                \
    else if (nbw == 2)                         \
      GV_LAUNCH(MATHV, MPV, 2);                \
    else if (nbw == 4)                         \
      GV_LAUNCH(MATHV, MPV, 4);                \
    else                                       \
      GV_LAUNCH(MATHV, MPV, 8);                \
  } while (0)
  if (p.m == 1)
    GV_LAUNCH_NBW(GV_MATH_DP4A, 1);
  else if (p.m == 2)
    GV_LAUNCH_NBW(GV_MATH_DP4A, 2);
  else if (p.m <= 8)
    GV_LAUNCH_NBW(GV_MATH_MMA, 8);
  else
    GV_LAUNCH_NBW(GV_MATH_MMA, 16);
#undef GV_LAUNCH_NBW
#undef GV_LAUNCH
  if (e != cudaSuccess) return (int)e;
  SKLB_COUNT_LAUNCH();
  return (int)cudaGetLastError();
}
