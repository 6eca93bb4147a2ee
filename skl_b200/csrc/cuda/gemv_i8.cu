// gemv_i8.cu -- skinny int8 GEMM (m <= 16): the decode-shape case.
//
// C[i, j] = sum_k A[i, k] * B[k, j] with A = activations (m rows, k contiguous) and B = weights stored
// one output column per contiguous k-run ("[N][K]": rsb == 1, csb == row pitch).  With m this small
// the arithmetic intensity is at most 2*m ops per weight byte, far below the tensor-core ridge, so
// the kernel is a weight-streaming kernel bounded by HBM bandwidth.  SKL's counterpart is the m == 1
// branch of its int8 kernel (src/gemm/gemm_i8rcp1x4_i8p4x1c_i32_xsfvqdotq.c:543-632, dispatch :645-658).
//
// Design.  A plain 16-byte-per-thread read of the weight matrix, 1024 threads per SM with 8 loads each in flight
// (128 KiB per SM), runs at 0.96 of the device's copy bandwidth at this size; staging the rows through shared memory
// with bulk copies measured 20-50 % slower, and so did fewer threads with more loads each or warp-wide loads that
// gather 64-byte pieces of 8 rows.  So one warp-wide access is always 512 contiguous bytes of one weight row, and:
//   * One CTA of 32 warps per SM.  The weight rows are dealt to the CTAs in layers: layer l is a run of consecutive
//     rows cut into one piece per CTA, so at any moment all CTAs read neighbouring rows and every CTA gets the same
//     number of bytes to within one row.  (Measured against per-CTA contiguous ranges and a grid-stride over 8-row
//     units: 9.9 vs 10.6 / 10.3 us.)
//   * m <= 2: the kernel IS that read, with the arithmetic hung on it.  A warp owns 512 bytes of k (KS = k / 512
//     warps share a group of 8 rows; the other warps of the CTA take further groups), a step of the CTA reads up to 32
//     consecutive rows of 4 KiB, every thread holding 8 independent 16-byte loads (ld.global.nc, no L1 allocation);
//     dp4a straight from the load registers against the same chunk of the activations, a butterfly warp-shuffle fold
//     of the 8 rows' partial sums.  The KS partial sums of an output meet in shared memory through integer atomic adds
//     (int32 sums wrap around like the reference's, in any order, so the result is exact); after the CTA's last piece
//     (or every `round` pieces when there are many) one barrier, then one thread per output runs the fused alpha/beta
//     or dequantising epilogue.  No tensor cores, no waits on barriers that another agent completes.
//   * 3 <= m <= 16: dp4a cannot keep up with HBM (4*m dp4a per 16 weight bytes on a two-per-clock pipe), so the sums
//     are formed by mma.sync.m16n8k32.s8 straight from the same load registers after a transposition across the warp
//     (see the kernel's comment).  The library's dispatcher prefers the tcgen05 GEMM kernel with swapped operands for
//     these m (15.3 us against 17.4 us on 14336 x 4096 at m = 4); this variant serves callers that force the skinny
//     path.  Other designs measured on that size and dropped: tcgen05.mma on 128-row tiles filled by plain loads and
//     st.shared (20-25 us), the same filled by cp.async in three 72 KiB stages (16.7 us: the tensor core's reads of a
//     tile and the fills of the next did not overlap), fragments re-read from a warp-private shared-memory tile (22-30 us),
//     the activations as the 64-row operand of tcgen05.mma against 97-row TMA boxes of weights (0.375 us per 128 bytes of k
//     on every SM, i.e. slower than the 128-row form's 0.28 us, plus a 16-lane epilogue: 25 us).
//
// Launch overlap.  The kernels let their successor on the stream start early (griddepcontrol) and are themselves
// launched as such dependents; they wait for their predecessor before their first global read, having asked the L2
// for the first lines.  When the caller declared the weights static the first reads of the weight stream are issued
// before that wait.
// Algorithmic bytes per launch: N*K (weights) + m*K (activations) + output and scale vectors.
#include <cstdlib>

#include "numerics.cuh"

namespace sklb {
namespace {

constexpr int GV_WARPS = 32;
constexpr int GV_THREADS = GV_WARPS * 32;
constexpr int GV_G = 8;               // weight rows per warp and step
constexpr int GV_KW = 512;            // bytes of k per warp
constexpr int GV_KSEG = 8 * GV_KW;    // most bytes of k per step

struct GemvParams {
  const int8_t *x;  // activations, row i at x + i*ldx
  const int8_t *w;  // weights, output column j at w + j*ldw
  void *c;
  int64_t ldx, ldw, rsc, csc;
  int m, n, k;
  int ksplit_log2;    // warps sharing one group of 8 rows: KS = 1 << ksplit_log2, each takes 512 bytes of a k segment
  int nseg;           // k segments of KS * 512 bytes
  int piece_rows;     // rows of one piece = 8 * (GV_WARPS / KS)
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

__device__ __forceinline__ uint4 gv_lds128(uint32_t addr) {
  uint4 v;
  asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(addr));
  return v;
}
__device__ __forceinline__ uint2 gv_lds64(uint32_t addr) {
  uint2 v;
  asm volatile("ld.shared.v2.u32 {%0,%1}, [%2];" : "=r"(v.x), "=r"(v.y) : "r"(addr));
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

// First row and row count of the piece CTA `b` takes from layer `l` (no divisions: see GemvParams).
__device__ __forceinline__ void gv_piece(const GemvParams &p, int l, int b, int &r0, int &nr) {
  const bool longer = l < p.lr;
  const int lo = l * p.lq + (l < p.lr ? l : p.lr);
  const int pq = longer ? p.pq1 : p.pq0, pr = longer ? p.pr1 : p.pr0;
  r0 = lo + b * pq + (b < pr ? b : pr);
  nr = pq + (b < pr ? 1 : 0);
}

// 16-byte global load that bypasses L1 allocation.
__device__ __forceinline__ uint4 gv_ldg(const void *p) {
  uint4 v;
  asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
               : "l"(p));
  return v;
}

// Shared-memory carve-up of the dp4a kernel: sums | column scale and bias | row scales.
struct GvSmem {
  int32_t *red;    // sums [round * piece_rows][MP]
  float2 *scl;     // (column scale, bias) of every row slot of the round
  float *rowsc;    // 16 row scales (1.0 when absent), after scl
  int red_ints;
};

// Start of a round: clears the sums and brings the round's column scales and biases into shared memory, so that their
// latency hides behind the stream.  Row slot = piece of the round, then row of the piece.
__device__ __forceinline__ void gv_round_begin(const GemvParams &p, const GvSmem &sm, int base, int count, int b, int tid) {
  for (int e = tid; e < sm.red_ints; e += GV_THREADS) sm.red[e] = 0;
  if (tid < 16) sm.rowsc[tid] = (p.row_scale && tid < p.m) ? __ldg(p.row_scale + tid) : 1.0f;
  if (p.col_scale || p.bias) {
    const int slots = count * p.piece_rows;
    for (int slot = tid; slot < slots; slot += GV_THREADS) {
      const int pc = slot / p.piece_rows, row = slot - pc * p.piece_rows;
      int r0, nr;
      gv_piece(p, base + pc, b, r0, nr);
      float2 v = make_float2(1.0f, 0.0f);
      if (row < nr) {
        if (p.col_scale) v.x = __ldg(p.col_scale + r0 + row);
        if (p.bias) v.y = __ldg(p.bias + r0 + row);
      }
      sm.scl[slot] = v;
    }
  }
}

// End of a round (after a barrier): one thread per output runs the epilogue.  Returns the largest value stored.
template <int MP>
__device__ __forceinline__ float gv_round_end(const GemvParams &p, const GvSmem &sm, int base, int count, int b, int tid) {
  float mx = -INFINITY;
  const int total = count * p.piece_rows * MP;
  for (int o = tid; o < total; o += GV_THREADS) {
    const int slot = o / MP, mi = o - slot * MP, pc = slot / p.piece_rows, row = slot - pc * p.piece_rows;
    int r0, nr;
    gv_piece(p, base + pc, b, r0, nr);
    if (row < nr && mi < p.m) {
      const float rsc = sm.rowsc[mi];
      const float2 cb = (p.col_scale || p.bias) ? sm.scl[slot] : make_float2(1.0f, 0.0f);
      mx = fmaxf(mx, gemv_store(p, mi, r0 + row, sm.red[o], rsc, cb.x, cb.y));
    }
  }
  return mx;
}

// ---- m <= 2: dp4a straight from the load registers, the thread's chunk of the activations in registers as well.
// The 8 loads of a step are two half batches of 4 rows that are consumed and re-requested separately, which keeps the
// memory pipe fuller across step boundaries (measured: 10.25 vs 11.1 us with the arithmetic below on the configured size).
template <int MP>
__global__ void __launch_bounds__(GV_THREADS, 1) gemv_i8_dp4a_kernel(const GemvParams p) {
  extern __shared__ __align__(128) uint8_t gv_smem[];
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5, b = (int)blockIdx.x;
  const int KS = 1 << p.ksplit_log2;
  const int ks = warp & (KS - 1), grp = warp >> p.ksplit_log2;  // this warp's share of k and its group inside a piece
  GvSmem sm;
  sm.red = reinterpret_cast<int32_t *>(gv_smem);
  sm.red_ints = p.round * p.piece_rows * MP;
  sm.scl = reinterpret_cast<float2 *>(sm.red + sm.red_ints);
  sm.rowsc = reinterpret_cast<float *>(sm.scl + p.round * p.piece_rows);
  const int kw0 = ks * GV_KW + lane * 16;  // this lane's byte of k inside a segment
  const int seg_bytes = KS * GV_KW;

  // The next kernel on the stream may be scheduled from now on (it waits for this one where it must).
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  if (!p.overlap) {
    // While the preceding kernel drains, ask the L2 for the lines of the first step: a prefetch changes no
    // architectural state, so it is safe even if that kernel is still writing the weights (its writes go through
    // the same L2), and the first loads after the wait then find their data on chip.
    if (p.layers > 0 && (lane & 7) == 0 && kw0 < p.k) {
      int r0, nr;
      gv_piece(p, 0, b, r0, nr);
      const int rows = nr - grp * GV_G;
      const int8_t *src = p.w + (int64_t)(r0 + grp * GV_G) * p.ldw + kw0;
      for (int u = 0; u < GV_G && u < rows; ++u) asm volatile("prefetch.global.L2 [%0];" ::"l"(src + (int64_t)u * p.ldw));
    }
    asm volatile("griddepcontrol.wait;" ::: "memory");
  }

  // Step = (piece l, k segment seg).  A half batch h (rows 4h .. 4h+3 of the warp's group) is requested for a step;
  // rows past the end of the piece and k past the end of the row read as 0.
  uint4 va[4], vb[4];
  auto request = [&](uint4 (&dst)[4], int h, int l, int seg) {
    int r0, nr;
    gv_piece(p, l, b, r0, nr);
    const int koff = seg * seg_bytes + kw0;
    const int first = grp * GV_G + 4 * h;
    const int rows = koff < p.k ? nr - first : 0;
    const int8_t *src = p.w + (int64_t)(r0 + first) * p.ldw + koff;
#pragma unroll
    for (int u = 0; u < 4; ++u) dst[u] = u < rows ? gv_ldg(src + (int64_t)u * p.ldw) : make_uint4(0, 0, 0, 0);
  };
  const int steps = p.layers * p.nseg;
  if (steps > 0) {
    request(va, 0, 0, 0);
    request(vb, 1, 0, 0);
  }
  if (p.overlap) asm volatile("griddepcontrol.wait;" ::: "memory");

  // this lane's 16 bytes of every activation row for the current k segment
  uint4 xq[MP];
  auto load_x = [&](int seg) {
    const int koff = seg * seg_bytes + kw0;
#pragma unroll
    for (int mi = 0; mi < MP; ++mi)
      xq[mi] = (mi < p.m && koff < p.k) ? *reinterpret_cast<const uint4 *>(p.x + (int64_t)mi * p.ldx + koff)
                                        : make_uint4(0, 0, 0, 0);
  };
  load_x(0);

  float my_max = -INFINITY;
  int l_next = 0, seg_next = 0;  // the step after the one being consumed
  auto advance = [&]() {
    if (++seg_next == p.nseg) {
      seg_next = 0;
      ++l_next;
    }
  };
  advance();
  for (int base = 0; base < p.layers; base += p.round) {
    const int count = (p.layers - base) < p.round ? (p.layers - base) : p.round;
    gv_round_begin(p, sm, base, count, b, tid);
    __syncthreads();
    for (int l = 0; l < count; ++l) {
      int32_t *sums = sm.red + (size_t)(l * p.piece_rows + grp * GV_G) * MP;  // this warp's 8 rows of the piece
      for (int seg = 0; seg < p.nseg; ++seg) {
        const bool more = l_next < p.layers;
        int32_t acc[GV_G * MP];
#pragma unroll
        for (int u = 0; u < 4; ++u) {
#pragma unroll
          for (int mi = 0; mi < MP; ++mi) {
            int32_t a = __dp4a((int)va[u].x, (int)xq[mi].x, 0);
            a = __dp4a((int)va[u].y, (int)xq[mi].y, a);
            a = __dp4a((int)va[u].z, (int)xq[mi].z, a);
            acc[u * MP + mi] = __dp4a((int)va[u].w, (int)xq[mi].w, a);
          }
        }
        if (more) request(va, 0, l_next, seg_next);
#pragma unroll
        for (int u = 0; u < 4; ++u) {
#pragma unroll
          for (int mi = 0; mi < MP; ++mi) {
            int32_t a = __dp4a((int)vb[u].x, (int)xq[mi].x, 0);
            a = __dp4a((int)vb[u].y, (int)xq[mi].y, a);
            a = __dp4a((int)vb[u].z, (int)xq[mi].z, a);
            acc[(4 + u) * MP + mi] = __dp4a((int)vb[u].w, (int)xq[mi].w, a);
          }
        }
        if (more) request(vb, 1, l_next, seg_next);
        if (p.nseg > 1 && more) load_x(seg_next);  // the activations of the next step's k segment
        advance();
        constexpr int V = GV_G * MP;
        constexpr int share = V == 16 ? 1 : 2;  // 2^share lanes hold the same finished value
        warp_fold<V>(acc, lane);
        if ((lane & ((1 << share) - 1)) == 0) atomicAdd(sums + (lane >> share), acc[0]);  // index row*MP + mi
      }
    }
    __syncthreads();
    my_max = fmaxf(my_max, gv_round_end<MP>(p, sm, base, count, b, tid));
    if (base + p.round < p.layers) __syncthreads();  // the sums are cleared for the next round
  }
  if (p.global_max) {
    my_max = warp_max_f32(my_max);
    if (lane == 0 && my_max != -INFINITY) atomic_max_f32(p.global_max, my_max);
  }
}

// ---- 3 <= m <= 16: mma.sync.m16n8k32.s8 straight from the load registers, after a transposition across the warp.
// The loads leave lane L with chunk L (16 bytes) of each of the 8 rows; the instruction wants lane (g, t) = (L / 4,
// L % 4) to supply bytes of row g.  Three rounds of exchanges (lanes 4, 8, 16 apart swap half of their registers) turn
// "register u = row u, lane = chunk" into "register j = chunk 4 j + t of row g": 48 shuffles for 4 KiB.  The order of k
// inside a fragment is then a fixed permutation, which the activations' fragments -- built once per CTA in shared
// memory, one 16-byte (MP = 16) or 8-byte (MP = 8) entry per lane and instruction, so that a warp reads 512 or 256
// contiguous bytes -- follow.  The activations are the 16-row operand (rows past m are zero), the 8 weight rows the
// 8-column one.  Everything else is the dp4a kernel: same loads, pieces, sums in shared memory, epilogue.
template <int MP>
__global__ void __launch_bounds__(GV_THREADS, 1) gemv_i8_mma_kernel(const GemvParams p) {
  extern __shared__ __align__(128) uint8_t gv_smem[];
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5, b = (int)blockIdx.x;
  const int KS = 1 << p.ksplit_log2;
  const int ks = warp & (KS - 1), grp = warp >> p.ksplit_log2;
  const int g = lane >> 2, t = lane & 3;
  // layout: activation fragments [windows of 512 bytes][16 instructions][32 lanes] | sums | column scale and bias | row scales
  constexpr int ENTRY = MP == 16 ? 16 : 8;
  const int windows = p.nseg * KS;
  GvSmem sm;
  sm.red = reinterpret_cast<int32_t *>(gv_smem + (size_t)windows * 512 * ENTRY);
  sm.red_ints = p.round * p.piece_rows * MP;
  sm.scl = reinterpret_cast<float2 *>(sm.red + sm.red_ints);
  sm.rowsc = reinterpret_cast<float *>(sm.scl + p.round * p.piece_rows);
  const uint32_t xfrag = gv_smem_u32(gv_smem);
  const int kw0 = ks * GV_KW + lane * 16;
  const int seg_bytes = KS * GV_KW;

  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  if (!p.overlap) {
    if (p.layers > 0 && (lane & 7) == 0 && kw0 < p.k) {
      int r0, nr;
      gv_piece(p, 0, b, r0, nr);
      const int rows = nr - grp * GV_G;
      const int8_t *src = p.w + (int64_t)(r0 + grp * GV_G) * p.ldw + kw0;
      for (int u = 0; u < GV_G && u < rows; ++u) asm volatile("prefetch.global.L2 [%0];" ::"l"(src + (int64_t)u * p.ldw));
    }
    asm volatile("griddepcontrol.wait;" ::: "memory");
  }

  uint4 va[4], vb[4];
  auto request = [&](uint4 (&dst)[4], int h, int l, int seg) {
    int r0, nr;
    gv_piece(p, l, b, r0, nr);
    const int koff = seg * seg_bytes + kw0;
    const int first = grp * GV_G + 4 * h;
    const int rows = koff < p.k ? nr - first : 0;
    const int8_t *src = p.w + (int64_t)(r0 + first) * p.ldw + koff;
#pragma unroll
    for (int u = 0; u < 4; ++u) dst[u] = u < rows ? gv_ldg(src + (int64_t)u * p.ldw) : make_uint4(0, 0, 0, 0);
  };
  const int steps = p.layers * p.nseg;
  if (steps > 0) {
    request(va, 0, 0, 0);
    request(vb, 1, 0, 0);
  }
  if (p.overlap) asm volatile("griddepcontrol.wait;" ::: "memory");

  // Activation fragments.  A thread takes one 16-byte chunk of one row (lanes: 8 rows x 4 chunks, 64 contiguous bytes
  // per row) and scatters its 4 words: word w of chunk 4 j + t of row i belongs to instruction 2 j + w / 2 of the
  // window, lane (i % 8, t), operand register (w % 2) * 2 + i / 8.
  {
    const int items = windows * 8 * (MP / 8) * 32;  // (window, j, upper half of the rows) x lane
    for (int e = tid; e < items; e += GV_THREADS) {
      const int ln = e & 31, rest = e >> 5;
      const int hi = MP == 16 ? (rest & 1) : 0, r2 = MP == 16 ? (rest >> 1) : rest;
      const int j = r2 & 7, win = r2 >> 3;
      const int row = (ln >> 2) + 8 * hi, tt = ln & 3;
      const int koff = win * GV_KW + 16 * (4 * j + tt);
      uint4 v = make_uint4(0, 0, 0, 0);
      if (row < p.m && koff < p.k) v = *reinterpret_cast<const uint4 *>(p.x + (int64_t)row * p.ldx + koff);
      const uint32_t e0 = xfrag + (uint32_t)(((win * 16 + 2 * j) * 32 + ln) * ENTRY) + (uint32_t)(hi * 4);
      const uint32_t step2 = MP == 16 ? 8u : 4u;  // distance between the operand registers of the two halves of k
      asm volatile("st.shared.u32 [%0], %1;" ::"r"(e0), "r"(v.x) : "memory");
      asm volatile("st.shared.u32 [%0], %1;" ::"r"(e0 + step2), "r"(v.y) : "memory");
      asm volatile("st.shared.u32 [%0], %1;" ::"r"(e0 + 32u * ENTRY), "r"(v.z) : "memory");
      asm volatile("st.shared.u32 [%0], %1;" ::"r"(e0 + 32u * ENTRY + step2), "r"(v.w) : "memory");
    }
  }

  float my_max = -INFINITY;
  int l_next = 0, seg_next = 0;
  auto advance = [&]() {
    if (++seg_next == p.nseg) {
      seg_next = 0;
      ++l_next;
    }
  };
  advance();
  // one exchange: lanes `dist` apart swap, the lower one giving `hi` for the partner's `lo`
  auto swap_words = [&](uint4 &lo, uint4 &hi, bool upper, int dist) {
    uint32_t s, r;
    s = upper ? lo.x : hi.x; r = __shfl_xor_sync(0xFFFFFFFFu, s, dist); if (upper) lo.x = r; else hi.x = r;
    s = upper ? lo.y : hi.y; r = __shfl_xor_sync(0xFFFFFFFFu, s, dist); if (upper) lo.y = r; else hi.y = r;
    s = upper ? lo.z : hi.z; r = __shfl_xor_sync(0xFFFFFFFFu, s, dist); if (upper) lo.z = r; else hi.z = r;
    s = upper ? lo.w : hi.w; r = __shfl_xor_sync(0xFFFFFFFFu, s, dist); if (upper) lo.w = r; else hi.w = r;
  };
  const bool up4 = (lane & 4) != 0, up8 = (lane & 8) != 0, up16 = (lane & 16) != 0;
  for (int base = 0; base < p.layers; base += p.round) {
    const int count = (p.layers - base) < p.round ? (p.layers - base) : p.round;
    gv_round_begin(p, sm, base, count, b, tid);
    __syncthreads();  // also: the activation fragments are complete
    for (int l = 0; l < count; ++l) {
      int32_t *sums = sm.red + (size_t)(l * p.piece_rows + grp * GV_G) * MP;
      for (int seg = 0; seg < p.nseg; ++seg) {
        const bool more = l_next < p.layers;
        const uint32_t xw = xfrag + (uint32_t)(((seg * KS + ks) * 16 * 32 + lane) * ENTRY);
        // rows <-> chunks: register j ends up holding chunk 4 j + t of row g
        swap_words(va[0], va[1], up4, 4);
        swap_words(va[2], va[3], up4, 4);
        swap_words(va[0], va[2], up8, 8);
        swap_words(va[1], va[3], up8, 8);
        swap_words(vb[0], vb[1], up4, 4);
        swap_words(vb[2], vb[3], up4, 4);
        swap_words(vb[0], vb[2], up8, 8);
        swap_words(vb[1], vb[3], up8, 8);
#pragma unroll
        for (int u = 0; u < 4; ++u) swap_words(va[u], vb[u], up16, 16);
        int32_t d[4] = {0, 0, 0, 0};
        auto fma_slot = [&](const uint4 &w, int j) {
          if constexpr (MP == 16) {
            const uint4 a = gv_lds128(xw + (uint32_t)((2 * j) * 32 * ENTRY));
            const uint4 c = gv_lds128(xw + (uint32_t)((2 * j + 1) * 32 * ENTRY));
            gv_mma(d, a.x, a.y, a.z, a.w, w.x, w.y);
            gv_mma(d, c.x, c.y, c.z, c.w, w.z, w.w);
          } else {
            const uint2 a = gv_lds64(xw + (uint32_t)((2 * j) * 32 * ENTRY));
            const uint2 c = gv_lds64(xw + (uint32_t)((2 * j + 1) * 32 * ENTRY));
            gv_mma(d, a.x, 0u, a.y, 0u, w.x, w.y);
            gv_mma(d, c.x, 0u, c.y, 0u, w.z, w.w);
          }
        };
#pragma unroll
        for (int u = 0; u < 4; ++u) fma_slot(va[u], u);
        if (more) request(va, 0, l_next, seg_next);
#pragma unroll
        for (int u = 0; u < 4; ++u) fma_slot(vb[u], 4 + u);
        if (more) request(vb, 1, l_next, seg_next);
        advance();
        // lane (g, t) holds the sums of activation rows g, g + 8 with weight rows 2 t, 2 t + 1 of the group
        atomicAdd(sums + (2 * t) * MP + g, d[0]);
        atomicAdd(sums + (2 * t + 1) * MP + g, d[1]);
        if constexpr (MP == 16) {
          atomicAdd(sums + (2 * t) * MP + g + 8, d[2]);
          atomicAdd(sums + (2 * t + 1) * MP + g + 8, d[3]);
        }
      }
    }
    __syncthreads();
    my_max = fmaxf(my_max, gv_round_end<MP>(p, sm, base, count, b, tid));
    if (base + p.round < p.layers) __syncthreads();
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

constexpr size_t GV_SMEM_MAX = 227 * 1024;
constexpr size_t GV_RED_MAX = 8 * 1024;  // shared memory for one round's sums; their rows' scale and bias take at most as much again

// Activation rows the kernel variant for m carries (dp4a: m itself; mma: 8 or 16).
inline int padded_m(int m) { return m <= 2 ? m : (m <= 8 ? 8 : 16); }
// k split: a warp takes 512 bytes of k; KS = 2^result warps (at most 8) share a group of 8 rows and cover a segment
// of KS * 512 bytes, longer k is walked segment by segment; the other warps take further groups of the piece.
inline int k_split_log2(int k) {
  const int kseg = k < GV_KSEG ? k : GV_KSEG;
  int s = 0;
  while ((GV_KW << s) < kseg) ++s;  // 0..3
  return s;
}
// Shared memory of the activation fragments (mma variant): k rounded up to whole segments, times the rows carried.
inline size_t xfrag_bytes(int m, int k) {
  if (m <= 2) return 0;
  const int seg = GV_KW << k_split_log2(k);
  return (size_t)((k + seg - 1) / seg) * seg * padded_m(m);
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
  // the activation fragments (m >= 3) and one round of sums must fit in shared memory
  if (xfrag_bytes((int)g->m0, (int)g->k0) + 2 * GV_RED_MAX + 64 > GV_SMEM_MAX) return 0;
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

  const int ks_log2 = k_split_log2(p.k);
  const int KS = 1 << ks_log2;
  p.ksplit_log2 = ks_log2;
  p.nseg = (p.k + KS * GV_KW - 1) / (KS * GV_KW);
  p.piece_rows = GV_G * (GV_WARPS / KS);
  const int mp = padded_m(p.m);

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

  // pieces per round: as many as one round's sums (and the threads' scale registers) allow
  int round = (int)(GV_RED_MAX / 4) / (p.piece_rows * mp);
  if (round < 1) round = 1;  // 256 rows x 16 activations: one piece fills 16 KiB
  if (round > p.layers) round = p.layers;
  p.round = round;
  const size_t smem = xfrag_bytes(p.m, p.k) + (size_t)round * p.piece_rows * (mp * 4 + 8) + 64;
  if (smem > GV_SMEM_MAX) return (int)cudaErrorInvalidValue;

  cudaStream_t s = (cudaStream_t)stream;
  cudaError_t e = cudaSuccess;
#define GV_LAUNCH(KERNEL)                                                                              \
  do {                                                                                                 \
    static bool attr_set[64] = {}; /* per device */                                                    \
    int dev = 0;                                                                                       \
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) dev = 0;                           \
    if (!attr_set[dev]) {                                                                              \
      e = cudaFuncSetAttribute(KERNEL, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)GV_SMEM_MAX);  \
      attr_set[dev] = (e == cudaSuccess);                                                              \
    }                                                                                                  \
    if (e == cudaSuccess) {                                                                            \
      cudaLaunchConfig_t cfg = {};                                                                     \
      cfg.gridDim = dim3((unsigned)grid);                                                              \
      cfg.blockDim = dim3(GV_THREADS);                                                                 \
      cfg.dynamicSmemBytes = smem;                                                                     \
      cfg.stream = s;                                                                                  \
      cudaLaunchAttribute attr[1];                                                                     \
      attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;                                 \
      attr[0].val.programmaticStreamSerializationAllowed = 1;                                          \
      cfg.attrs = attr;                                                                                \
      cfg.numAttrs = 1;                                                                                \
      e = cudaLaunchKernelEx(&cfg, KERNEL, p);                                                         \
    }                                                                                                  \
  } while (0)
  if (p.m == 1)
    GV_LAUNCH(gemv_i8_dp4a_kernel<1>);
  else if (p.m == 2)
    GV_LAUNCH(gemv_i8_dp4a_kernel<2>);
  else if (p.m <= 8)
    GV_LAUNCH(gemv_i8_mma_kernel<8>);
  else
    GV_LAUNCH(gemv_i8_mma_kernel<16>);
#undef GV_LAUNCH
  if (e != cudaSuccess) return (int)e;
  SKLB_COUNT_LAUNCH();
  return (int)cudaGetLastError();
}
