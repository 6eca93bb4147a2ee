// gemm_tc.cu -- the tensor-core GEMM for sm_100a: TMA-staged operands, tcgen05.mma, TMEM accumulators.
//
// Stands in for SKL's matrix-engine kernels (src/gemm/gemm_i8c_i8_i32_xsfmm32a8i.c:2466-2555 and the
// bf16 / f16 / fp8 siblings): there the accumulator tile lives in matrix-tile registers for the whole
// K loop and a fused alpha/beta kernel runs on it before the store (:603-641); here it lives in TMEM
// and the epilogue warps apply alpha/beta, scale vectors and the output narrowing on the way out.
//
// One CTA = one 128 x BN output tile at a time, persistent over a static tile schedule
// (unit = blockIdx.x + i*gridDim.x; tiles are visited in L2-sized groups of m-tiles, and the tiles left
// after the last full round are cut into column strips, one per CTA).  192 threads in three roles:
//   warp 0      TMA producer: one lane issues cp.async.bulk.tensor loads of the A and B k-slabs
//               (128 bytes of K per slab, 128-byte swizzle) into a ring of shared-memory stages;
//   warp 1      MMA issuer: allocates TMEM, and one lane issues 4 tcgen05.mma (K = 32 bytes each) per
//               stage, then tcgen05.commit to hand the stage back / to publish the finished tile;
//   warps 2..5  epilogue: each warp first copies the tile's column scales / bias into its own
//               shared-memory slice, then reads the finished accumulator with tcgen05.ld 32 columns at
//               a time (two accumulators in TMEM, so tile i+1's MMAs overlap tile i's epilogue),
//               applies alpha/beta, scales, bias, activation and narrowing, and writes the 32 x 32
//               chunk through swizzled shared-memory staging and a TMA store (16-byte or element
//               stores when C is not a row-major matrix with 16-byte rows).
// The kernel is launched as a programmatic dependent of the kernel before it on the stream and waits
// for that kernel (griddepcontrol.wait) only after its own set-up.
// Operands may be K-major (k contiguous) or MN-major (m or n contiguous) in global memory; the
// shared-memory matrix descriptors and the instruction descriptor carry the difference, no
// transposing pre-pass is needed.  Edges in M, N and K rely on TMA zero fill.
//
// Every mbarrier wait is bounded (two seconds of wall time unless the caller set another limit); on expiry the thread records a
// code in the status words, raises a CTA-wide abort flag and all roles fall through to the common
// exit, which frees TMEM.  The kernel never spins unboundedly.
//
// Roofline: tensor pipe.  Work per launch = 2*M*N*K operations.  HBM traffic is at least
// (M*K + K*N)*esize + M*N*csize; operand re-reads between tiles are served by the 126 MB L2.
#include <cuda.h>

#include <cstdio>
#include <cstdlib>
#include <type_traits>

#include "numerics.cuh"

namespace sklb {
namespace {

constexpr int BM = 128;
constexpr int SLAB_BYTES = 128;  // bytes of K per stage row = one swizzle atom
constexpr int NUM_THREADS = 192;
#ifndef TC_SKINNY_ISSUERS
#define TC_SKINNY_ISSUERS 2
#endif
constexpr int KIND_F16 = 0, KIND_F8 = 1, KIND_I8 = 2;
constexpr int PLAIN_PANEL = 0x7fffffff;  // TcParams::a_panel / b_panel of a plain (unpanelled) MN-major matrix

constexpr uint32_t ERR_WAIT_EMPTY = 0x101, ERR_WAIT_FULL = 0x102, ERR_WAIT_TMEM_EMPTY = 0x103,
                   ERR_WAIT_TMEM_FULL = 0x104;

struct TcParams {
  int M, N, K;
  int tiles_m, tiles_n, num_kb;
  int raster_gm;   // m-tiles per rasterisation group (tiles of one group are visited n-major)
  // Tail splitting (one-CTA kernel): the tiles left over after the last full round of the grid are cut
  // into `tail_split` column strips each, one strip per CTA, so the last round is short instead of idle.
  int main_tiles, tail_round, tail_units, tail_split;
  // Width of a full tile: the kernel's BN, or less (a multiple of 32 columns) when narrower tiles fill the rounds
  // of the grid better; the shared-memory stage and the accumulator keep BN columns of room either way.
  int bn_main;
  int main_b_atoms;        // MN-major B: boxes a full tile loads per k-slab
  uint32_t main_b_bytes;   // bytes of B a full tile loads per k-slab
  uint32_t idesc_tail;  // instruction descriptor with N = bn_main / tail_split
  int tail_b_atoms;     // MN-major B: boxes one strip loads per k-slab
  uint32_t tail_b_bytes;  // bytes of B one strip loads per k-slab
  int a_mn, b_mn;  // 1: operand is MN-major in global/shared memory
  // MN-major operands are described to TMA as panels: `panel` consecutive m (n) elements, then k, then the panel
  // index.  A plain column-major A / row-major B is a single panel as wide as the matrix; SKL's matrix-engine
  // packed operands (TE x 1 blocks of A, 1 x TE blocks of B) are panels of TE.
  int a_panel, b_panel;
  uint32_t idesc;
  void *c;
  int64_t rsc, csc;
  // Blocked C (SKL's packed C): blocks of c_block_m x c_block_n elements, rsc / csc inside a block, rsc1 / csc1
  // between blocks.  c_block_m == 0: a plain matrix.
  int c_block_m, c_block_n;
  int64_t rsc1, csc1;
  int tc, epilogue;
  int c_vec_ok;  // csc == 1 and rows 16-byte aligned
  int c_tma;     // C has a tensor map: results leave through shared memory and TMA stores
  int32_t alpha_i, beta_i;
  float alpha_f, beta_f;
  const float *row_scale, *col_scale;
  int col_scale_first;
  const float *bias;
  int bias_per_row;
  float *global_max;
  int activation;
  float act_param;
  uint32_t *status;
  uint64_t wait_ns;  // bound of every mbarrier wait
  int skip_loads;    // testing aid: the producer announces its loads but never issues them
  // One-CTA kernel, k-major A: rows of A per tile (<= 128).  Fewer than 128 when that makes the number of tiles a
  // whole number of rounds of the grid (a tall-skinny problem is a stream of A, so every SM must have a tile): the
  // TMA box holds bm_rows rows, the MMA still reads 128 (the accumulator lanes past bm_rows hold garbage that the
  // epilogue never stores).
  int bm_rows;
  uint32_t a_tx;     // bytes of A per stage = bm_rows * 128
};

// ------------------------------------------------------------------ PTX wrappers
__device__ __forceinline__ uint32_t smem_u32(const void *p) {
  return (uint32_t)__cvta_generic_to_shared(p);
}
__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count));
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ bool mbar_try(uint32_t bar, uint32_t parity) {
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
__device__ __forceinline__ uint64_t globaltimer_ns() {
  uint64_t t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}

// Bounded wait.  Returns false when the wait expired or another thread of the CTA already gave up.
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, volatile uint32_t *abort_flag,
                                          uint32_t *status, uint32_t code, uint64_t limit_ns) {
  if (mbar_try(bar, parity)) return true;
  uint64_t t0 = 0;
  for (uint32_t spins = 1;; ++spins) {
    if (mbar_try(bar, parity)) return true;
    if ((spins & 63u) == 0u) {
      if (*abort_flag) return false;
      uint64_t now = globaltimer_ns();
      if (t0 == 0) t0 = now;
      if (now - t0 > limit_ns) {
        *abort_flag = 1u;
        atomicCAS(status, 0u, code);
        return false;
      }
    }
  }
}

__device__ __forceinline__ void tma_load_2d(uint32_t dst, const CUtensorMap *tm, uint32_t bar, int x, int y) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
      ::"r"(dst), "l"(tm), "r"(bar), "r"(x), "r"(y)
      : "memory");
}

// MN-major operands: x = element inside the panel, y = k, z = panel.
__device__ __forceinline__ void tma_load_3d(uint32_t dst, const CUtensorMap *tm, uint32_t bar, int x, int y, int z) {
  asm volatile(
      "cp.async.bulk.tensor.3d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5}], [%2];"
      ::"r"(dst), "l"(tm), "r"(bar), "r"(x), "r"(y), "r"(z)
      : "memory");
}
// Box coordinates of the MN-major boxes of one tile, worked out once per tile (the division stays out of the k loop):
// box i starts at element mn0 + i*step of the operand, i.e. at (x[i], z[i]) = (element in panel, panel).
template <int NB>
struct MnBoxes {
  int x[NB], z[NB];
  __device__ __forceinline__ void set(int mn0, int step, int panel) {
    int zz = mn0 / panel, xx = mn0 - zz * panel;
#pragma unroll
    for (int i = 0; i < NB; ++i) {
      x[i] = xx;
      z[i] = zz;
      xx += step;
      if (xx >= panel) {  // panels are whole numbers of boxes; a plain matrix (one unbounded panel) never wraps
        xx -= panel;
        ++zz;
      }
    }
  }
};

// Offset of element (row, col) of C: plain strides, or SKL's blocked description.
__device__ __forceinline__ int64_t c_offset(const TcParams &p, int row, int col) {
  if (p.c_block_m == 0) return (int64_t)row * p.rsc + (int64_t)col * p.csc;
  const int bi = row / p.c_block_m, bj = col / p.c_block_n;
  return (int64_t)bi * p.rsc1 + (int64_t)bj * p.csc1 + (int64_t)(row - bi * p.c_block_m) * p.rsc +
         (int64_t)(col - bj * p.c_block_n) * p.csc;
}

template <int KIND>
__device__ __forceinline__ void umma(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t idesc,
                                     uint32_t accumulate) {
  if (KIND == KIND_F16) {
    asm volatile(
        "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}" ::"r"(tmem_d),
        "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
        : "memory");
  } else if (KIND == KIND_F8) {
    asm volatile(
        "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f8f6f4 [%0], %1, %2, %3, p;\n\t}" ::"r"(tmem_d),
        "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
        : "memory");
  } else {
    asm volatile(
        "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::i8 [%0], %1, %2, %3, p;\n\t}" ::"r"(tmem_d),
        "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
        : "memory");
  }
}
__device__ __forceinline__ void umma_commit(uint32_t bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar)
               : "memory");
}
__device__ __forceinline__ void tc_fence_before() {
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
}
__device__ __forceinline__ void tc_fence_after() {
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
}
__device__ __forceinline__ void tmem_ld32(uint32_t taddr, uint32_t (&r)[32]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
      "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
        "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]),
        "=r"(r[15]), "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]),
        "=r"(r[22]), "=r"(r[23]), "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]),
        "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
      : "r"(taddr));
  asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}

// 16 columns (the narrow-tile kernel); the upper half of r is cleared.
__device__ __forceinline__ void tmem_ld16(uint32_t taddr, uint32_t (&r)[32]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x16.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
        "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]),
        "=r"(r[15])
      : "r"(taddr));
  asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
  for (int i = 16; i < 32; ++i) r[i] = 0u;
}

// Shared-memory matrix descriptor (tcgen05): start address, leading / stride byte offsets in 16-byte
// units, descriptor version 1 at bit 46, 128-byte swizzle (value 2) at bits 61..63.
__device__ __forceinline__ uint64_t make_smem_desc(uint32_t saddr, uint32_t lbo_bytes, uint32_t sbo_bytes) {
  uint64_t d = 0;
  d |= (uint64_t)((saddr >> 4) & 0x3FFFu);
  d |= (uint64_t)((lbo_bytes >> 4) & 0x3FFFu) << 16;
  d |= (uint64_t)((sbo_bytes >> 4) & 0x3FFFu) << 32;
  d |= 1ull << 46;
  d |= 2ull << 61;
  return d;
}

// Tile order.  Tiles are visited in groups of `gm` consecutive m-tiles; inside a group the n index
// moves slowest, so the CTAs running at the same time share a few B tiles and a bounded set of A
// rows (gm * tile_rows * K * esize bytes, chosen on the host to sit well inside the L2), instead of
// streaming all of A once per B tile.
__device__ __forceinline__ void tile_coords(int t, int tiles_m, int tiles_n, int gm, int &mi, int &ni) {
  const int group = gm * tiles_n;
  const int g = t / group, r = t - g * group;
  const int first = g * gm;
  const int cur = (tiles_m - first) < gm ? (tiles_m - first) : gm;
  ni = r / cur;
  mi = first + (r - ni * cur);
}

// Work unit `it` of this CTA in the one-CTA kernel: a full tile, or one strip of a split tail tile.
struct TileUnit {
  int m0, n0, ncols;
  uint32_t idesc;
};
template <int BN>
__device__ __forceinline__ bool get_unit(const TcParams &p, int it, TileUnit &u) {
  const int t = (int)blockIdx.x + it * (int)gridDim.x;
  int mi, ni;
  if (t < p.main_tiles) {
    tile_coords(t, p.tiles_m, p.tiles_n, p.raster_gm, mi, ni);
    u.m0 = mi * p.bm_rows;
    u.n0 = ni * p.bn_main;
    u.ncols = p.bn_main;
    u.idesc = p.idesc;
    return true;
  }
  if (it == p.tail_round && (int)blockIdx.x < p.tail_units) {
    const int tt = p.main_tiles + (int)blockIdx.x / p.tail_split, sub = (int)blockIdx.x % p.tail_split;
    tile_coords(tt, p.tiles_m, p.tiles_n, p.raster_gm, mi, ni);
    u.ncols = p.bn_main / p.tail_split;
    u.m0 = mi * p.bm_rows;
    u.n0 = ni * p.bn_main + sub * u.ncols;
    u.idesc = p.idesc_tail;
    return true;
  }
  return false;
}

// ---- two-CTA (cta_group::2) helpers
__device__ __forceinline__ uint32_t cluster_ctarank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
__device__ __forceinline__ uint32_t mapa(uint32_t saddr, uint32_t rank) {
  uint32_t r;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(saddr), "r"(rank));
  return r;
}
__device__ __forceinline__ void cluster_sync_all() {
  asm volatile("barrier.cluster.arrive.release;" ::: "memory");
  asm volatile("barrier.cluster.wait.acquire;" ::: "memory");
}
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t cluster_bar) {
  asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(cluster_bar) : "memory");
}
// TMA load issued by either CTA of a pair into its own shared memory; the bytes are credited to the
// barrier at `cluster_bar`, which may live in the partner CTA.  No multicast: each CTA fetches its own data.
__device__ __forceinline__ void tma_load_2d_pair(uint32_t dst, const CUtensorMap *tm, uint32_t cluster_bar, int x,
                                                 int y) {
  asm volatile(
      "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
      ::"r"(dst), "l"(tm), "r"(cluster_bar), "r"(x), "r"(y)
      : "memory");
}
__device__ __forceinline__ void tma_load_3d_pair(uint32_t dst, const CUtensorMap *tm, uint32_t cluster_bar, int x, int y,
                                                 int z) {
  asm volatile(
      "cp.async.bulk.tensor.3d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5}], [%2];"
      ::"r"(dst), "l"(tm), "r"(cluster_bar), "r"(x), "r"(y), "r"(z)
      : "memory");
}
template <int KIND>
__device__ __forceinline__ void umma_pair(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t idesc,
                                          uint32_t accumulate) {
  if (KIND == KIND_F16) {
    asm volatile(
        "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n\t}" ::"r"(tmem_d),
        "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
        : "memory");
  } else if (KIND == KIND_F8) {
    asm volatile(
        "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::2.kind::f8f6f4 [%0], %1, %2, %3, p;\n\t}" ::"r"(tmem_d),
        "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
        : "memory");
  } else {
    asm volatile(
        "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::2.kind::i8 [%0], %1, %2, %3, p;\n\t}" ::"r"(tmem_d),
        "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
        : "memory");
  }
}
// One commit that arrives on the barrier at the same shared-memory offset in both CTAs of the pair
// (a commit signal, not a data load: nothing is copied).
__device__ __forceinline__ void umma_commit_pair_both(uint32_t bar) {
  const uint16_t mask = 3;
  asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;" ::"r"(bar),
               "h"(mask)
               : "memory");
}

// ---- results through shared memory and TMA stores
// Each epilogue warp owns EPI_STAGE_BYTES of staging.  A 32-row x 32-column chunk is written there one row per
// lane in the tensor map's swizzled order (the 16-byte piece index XORed with address bits 7 and up, so the 32
// lanes' pieces spread over all banks), then one lane hands the box to the TMA engine, which writes whole rows
// of the box to global memory and clips at the matrix edge.  A box is 2 KiB (1 KiB for 1-byte elements), so 2 or
// 4 boxes rotate through the staging area and a store only waits for the one issued that many boxes earlier.
constexpr int EPI_STAGE_BYTES = 4096;
__device__ __forceinline__ void tma_store_2d(const CUtensorMap *tm, uint32_t src, int x, int y) {
  asm volatile("cp.async.bulk.tensor.2d.global.shared::cta.bulk_group [%0, {%2, %3}], [%1];" ::"l"(tm), "r"(src),
               "r"(x), "r"(y)
               : "memory");
}
__device__ __forceinline__ void bulk_commit() { asm volatile("cp.async.bulk.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void bulk_wait_read() {
  asm volatile("cp.async.bulk.wait_group.read %0;" ::"n"(N) : "memory");
}
__device__ __forceinline__ void bulk_wait_all() { asm volatile("cp.async.bulk.wait_group 0;" ::: "memory"); }

struct EpiStage {
  const CUtensorMap *tm;  // nullptr: direct stores
  uint32_t base;          // this warp's staging area (shared-memory address, 1024-byte aligned)
  uint32_t count;         // chunks stored so far
};

// One box: PITCH bytes per row (64 or 32 = the map's swizzle span), 32 rows, NBUF boxes rotating through the
// staging area.  w: the lane's row of the box, PITCH / 4 words.
template <int PITCH, int NBUF>
__device__ __forceinline__ void tma_store_box(EpiStage &st, int lane, const uint32_t *w, int x, int y) {
  constexpr int PIECES = PITCH / 16;  // 16-byte pieces per row
  static_assert(NBUF * 32 * PITCH <= EPI_STAGE_BYTES, "boxes exceed the staging area");
  const uint32_t buf = st.base + (st.count % NBUF) * (32 * PITCH);
  if (lane == 0) bulk_wait_read<NBUF - 1>();
  __syncwarp();
  const uint32_t rowoff = (uint32_t)lane * PITCH;
  const uint32_t sw = (rowoff >> 7) & (PIECES - 1);
#pragma unroll
  for (int q = 0; q < PIECES; ++q)
    asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(buf + rowoff + 16u * ((uint32_t)q ^ sw)),
                 "r"(w[4 * q]), "r"(w[4 * q + 1]), "r"(w[4 * q + 2]), "r"(w[4 * q + 3])
                 : "memory");
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
  __syncwarp();
  if (lane == 0) {
    tma_store_2d(st.tm, buf, x, y);
    bulk_commit();
  }
  ++st.count;
}

// w: the lane's row of a 32-column chunk, 32 elements of ES bytes packed into 8 * ES words.  4-byte elements go
// out as two boxes of 16 columns so that, like the narrower types, one store is always in flight while the
// next box is being filled.
template <int ES>
__device__ __forceinline__ void tma_store_chunk(EpiStage &st, int lane, const uint32_t *w, int x, int y) {
  if (ES == 4) {
    tma_store_box<64, 2>(st, lane, w, x, y);
    tma_store_box<64, 2>(st, lane, w + 16, x + 16, y);
  } else if (ES == 2) {
    tma_store_box<64, 2>(st, lane, w, x, y);
  } else {
    tma_store_box<32, 4>(st, lane, w, x, y);
  }
}

// Per-warp shared-memory copies of the tile's column scales and column bias.  Each epilogue warp fills
// its own copy before it waits for the accumulator, so the global loads hide behind the main loop and
// the per-element reads are shared-memory broadcasts; only __syncwarp orders them.  Columns past N (and,
// for tiles narrower than one 32-column chunk, past the tile) read as 1 and 0.
template <int BN>
struct EpiVectors {
  static constexpr int COLS = BN < 32 ? 32 : BN;
  static constexpr int BYTES = 4 /*warps*/ * 2 /*scale, bias*/ * COLS * 4;
  __device__ static __forceinline__ float *scale(uint8_t *base, int quad) {
    return reinterpret_cast<float *>(base) + quad * 2 * COLS;
  }
  __device__ static __forceinline__ float *bias(uint8_t *base, int quad) { return scale(base, quad) + COLS; }
  __device__ static __forceinline__ void fill(const TcParams &p, float *cs, float *bs, int n0, int ncols, int lane) {
    const bool col_bias = p.bias && !p.bias_per_row;
    if (!p.col_scale && !col_bias) return;
    const int lim = ncols < 32 ? 32 : ncols;
    __syncwarp();  // this warp's reads of the previous tile's values are done
    for (int i = lane; i < lim; i += 32) {
      const bool in = i < ncols && n0 + i < p.N;
      if (p.col_scale) cs[i] = in ? __ldg(p.col_scale + n0 + i) : 1.0f;
      if (col_bias) bs[i] = in ? __ldg(p.bias + n0 + i) : 0.0f;
    }
    __syncwarp();
  }
};

template <int BN>
struct TcConfig {
  static constexpr int A_BYTES = BM * SLAB_BYTES;
  static constexpr int B_BYTES = BN * SLAB_BYTES;
  static constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
  static constexpr int STAGES_RAW = (220 * 1024) / STAGE_BYTES;
  static constexpr int STAGES = STAGES_RAW > 8 ? 8 : STAGES_RAW;
  // The 16-column tile (tall-skinny problems) has ISSUERS threads issuing MMAs, each for every ISSUERS-th k block
  // and into its own accumulator, which the epilogue adds up (see the MMA issuer's comment).
  static constexpr int ISSUERS = BN == 16 ? TC_SKINNY_ISSUERS : 1;
  static constexpr int THREADS = NUM_THREADS + 32 * (ISSUERS - 1);
  static constexpr int ACC_COLS = BN * ISSUERS;
  static constexpr int TMEM_COLS = 2 * ACC_COLS < 32 ? 32 : 2 * ACC_COLS;
  static constexpr int SMEM_BYTES =
      STAGES * STAGE_BYTES + 1024 /*align*/ + 4 * EPI_STAGE_BYTES + 256 /*barriers*/ + EpiVectors<BN>::BYTES;
  static_assert(SMEM_BYTES <= 227 * 1024, "exceeds the shared memory one CTA can have");
};

// ------------------------------------------------------------------ epilogue for 32 accumulator columns
// Called by every lane of an epilogue warp (lane = row of the 32-row box; `row_ok` says whether that row exists).
// Returns the largest value written (for the optional global maximum); -INFINITY for the int epilogue.
template <bool ACC_INT, bool ACT>
__device__ __forceinline__ float epilogue_chunk(const TcParams &p, const uint32_t (&r)[32], int row, bool row_ok,
                                                int col0, const float *cs, const float *bs, float rs,
                                                float row_bias, EpiStage &st, int lane) {
  const int ncols = (p.N - col0) < 32 ? (p.N - col0) : 32;
  // a 32-column chunk never crosses a block of a blocked C (block widths are multiples of 32)
  const int64_t base = c_offset(p, row, col0);
  if (p.epilogue == SKL_EPI_INT) {
    uint32_t o[32];
    if (p.beta_i != 0 && row_ok) {
      const int32_t *crow = (const int32_t *)p.c + base;
      if (p.c_vec_ok && ncols == 32) {
        const uint4 *src = reinterpret_cast<const uint4 *>(crow);
#pragma unroll
        for (int q = 0; q < 8; ++q) {
          const uint4 old = src[q];
          o[4 * q] = (uint32_t)p.beta_i * old.x + (uint32_t)p.alpha_i * r[4 * q];
          o[4 * q + 1] = (uint32_t)p.beta_i * old.y + (uint32_t)p.alpha_i * r[4 * q + 1];
          o[4 * q + 2] = (uint32_t)p.beta_i * old.z + (uint32_t)p.alpha_i * r[4 * q + 2];
          o[4 * q + 3] = (uint32_t)p.beta_i * old.w + (uint32_t)p.alpha_i * r[4 * q + 3];
        }
      } else {
#pragma unroll
        for (int e = 0; e < 32; ++e)
          o[e] = (e < ncols ? (uint32_t)p.beta_i * (uint32_t)crow[(int64_t)e * p.csc] : 0u) + (uint32_t)p.alpha_i * r[e];
      }
    } else {
#pragma unroll
      for (int e = 0; e < 32; ++e) o[e] = (uint32_t)p.alpha_i * r[e];
    }
    if (st.tm) {
      tma_store_chunk<4>(st, lane, o, col0, row - lane);
    } else if (row_ok) {
      int32_t *crow = (int32_t *)p.c + base;
      if (p.c_vec_ok && ncols == 32) {
        uint4 *dst = reinterpret_cast<uint4 *>(crow);
#pragma unroll
        for (int q = 0; q < 8; ++q) dst[q] = make_uint4(o[4 * q], o[4 * q + 1], o[4 * q + 2], o[4 * q + 3]);
      } else {
#pragma unroll
        for (int e = 0; e < 32; ++e)
          if (e < ncols) crow[(int64_t)e * p.csc] = (int32_t)o[e];
      }
    }
    return -INFINITY;
  }
  // float epilogue
  // cs / bs: this warp's shared-memory copies for these 32 columns (nullptr when the vector is absent);
  // rs / row_bias: this row's scale and bias, loaded once per tile.
  float v[32];
#pragma unroll
  for (int e = 0; e < 32; ++e) {
    float acc = ACC_INT ? (float)(int32_t)r[e] : __uint_as_float(r[e]);
    v[e] = __fmul_rn(p.alpha_f, acc);
  }
  if (p.row_scale && !p.col_scale_first) {
#pragma unroll
    for (int e = 0; e < 32; ++e) v[e] = __fmul_rn(v[e], rs);
  }
  if (cs) {
    const float4 *cs4 = reinterpret_cast<const float4 *>(cs);
#pragma unroll
    for (int q = 0; q < 8; ++q) {
      const float4 c4 = cs4[q];
      v[4 * q] = __fmul_rn(v[4 * q], c4.x);
      v[4 * q + 1] = __fmul_rn(v[4 * q + 1], c4.y);
      v[4 * q + 2] = __fmul_rn(v[4 * q + 2], c4.z);
      v[4 * q + 3] = __fmul_rn(v[4 * q + 3], c4.w);
    }
  }
  if (p.row_scale && p.col_scale_first) {
#pragma unroll
    for (int e = 0; e < 32; ++e) v[e] = __fmul_rn(v[e], rs);
  }
  if (bs) {
    const float4 *bs4 = reinterpret_cast<const float4 *>(bs);
#pragma unroll
    for (int q = 0; q < 8; ++q) {
      const float4 b4 = bs4[q];
      v[4 * q] = __fadd_rn(v[4 * q], b4.x);
      v[4 * q + 1] = __fadd_rn(v[4 * q + 1], b4.y);
      v[4 * q + 2] = __fadd_rn(v[4 * q + 2], b4.z);
      v[4 * q + 3] = __fadd_rn(v[4 * q + 3], b4.w);
    }
  } else if (p.bias) {
#pragma unroll
    for (int e = 0; e < 32; ++e) v[e] = __fadd_rn(v[e], row_bias);
  }
  if (p.beta_f != 0.0f && row_ok) {
#pragma unroll
    for (int e = 0; e < 32; ++e)
      if (e < ncols)
        v[e] = __fadd_rn(__fmul_rn(p.beta_f, load_c_f32(p.tc, p.c, base + (int64_t)e * p.csc)), v[e]);
  }
  if (ACT && p.activation) {
    if (p.activation == SKL_ACT_SWIGLU) {
      if (row_ok) {
#pragma unroll
        for (int e = 0; e < 32; ++e)
          if (e < ncols)
            v[e] =
                activation_value(SKL_ACT_SWIGLU, p.act_param, v[e], load_c_f32(p.tc, p.c, base + (int64_t)e * p.csc));
      }
    } else if (p.activation == SKL_ACT_GELU) {
#pragma unroll
      for (int e = 0; e < 32; ++e) v[e] = gelu_f32(v[e]);
    } else {
      const bool times_v = p.activation == SKL_ACT_SWISH;
#pragma unroll
      for (int e = 0; e < 32; ++e) {
        const float o = logistic_f32(p.act_param, v[e]);
        v[e] = times_v ? __fmul_rn(o, v[e]) : o;
      }
    }
  }
  float vmax = -INFINITY;
  if (p.global_max && row_ok) {
#pragma unroll
    for (int e = 0; e < 32; ++e)
      if (e < ncols && v[e] == v[e]) vmax = fmaxf(vmax, v[e]);
  }
  const bool vec = st.tm != nullptr || (p.c_vec_ok && ncols == 32);
  if (vec) {
    // narrow and pack the row, then either hand it to the TMA store or write it as 16-byte pieces
    uint32_t w[32];
    int words;
    if (p.tc == SKL_DT_F32) {
      words = 32;
#pragma unroll
      for (int e = 0; e < 32; ++e) w[e] = __float_as_uint(v[e]);
    } else if (p.tc == SKL_DT_BF16 || p.tc == SKL_DT_F16) {
      words = 16;
      // A NaN anywhere in the row makes the sum NaN (so does inf - inf, which only costs the slow path): the
      // hardware converter handles everything else, the bit-exact NaN encoding is kept for the rare row.
      float t[8];
#pragma unroll
      for (int q = 0; q < 8; ++q) t[q] = (v[4 * q] + v[4 * q + 1]) + (v[4 * q + 2] + v[4 * q + 3]);
      const float total = ((t[0] + t[1]) + (t[2] + t[3])) + ((t[4] + t[5]) + (t[6] + t[7]));
      if (total == total) {
        if (p.tc == SKL_DT_BF16) {
#pragma unroll
          for (int q = 0; q < 16; ++q) w[q] = pack_bf16x2_no_nan(v[2 * q], v[2 * q + 1]);
        } else {
#pragma unroll
          for (int q = 0; q < 16; ++q) w[q] = pack_f16x2_no_nan(v[2 * q], v[2 * q + 1]);
        }
      } else {
#pragma unroll
        for (int q = 0; q < 16; ++q) {
          uint32_t lo = p.tc == SKL_DT_BF16 ? enc_bf16(v[2 * q]) : enc_f16(v[2 * q]);
          uint32_t hi = p.tc == SKL_DT_BF16 ? enc_bf16(v[2 * q + 1]) : enc_f16(v[2 * q + 1]);
          w[q] = lo | (hi << 16);
        }
      }
    } else if (p.tc == SKL_DT_I8) {  // requantised: round to nearest even, saturating
      words = 8;
#pragma unroll
      for (int q = 0; q < 8; ++q)
        w[q] = enc_i8_sat(v[4 * q]) | (enc_i8_sat(v[4 * q + 1]) << 8) | (enc_i8_sat(v[4 * q + 2]) << 16) |
               (enc_i8_sat(v[4 * q + 3]) << 24);
    } else {  // F8E4M3, saturating
      words = 8;
#pragma unroll
      for (int q = 0; q < 8; ++q)
        w[q] = enc_e4m3x2(v[4 * q], v[4 * q + 1], true) | (enc_e4m3x2(v[4 * q + 2], v[4 * q + 3], true) << 16);
    }
    if (st.tm) {
      if (words == 32)
        tma_store_chunk<4>(st, lane, w, col0, row - lane);
      else if (words == 16)
        tma_store_chunk<2>(st, lane, w, col0, row - lane);
      else
        tma_store_chunk<1>(st, lane, w, col0, row - lane);
    } else if (row_ok) {
      uint4 *dst = reinterpret_cast<uint4 *>((uint8_t *)p.c + base * (words / 8));
#pragma unroll
      for (int q = 0; q < 8; ++q)
        if (4 * q < words) dst[q] = make_uint4(w[4 * q], w[4 * q + 1], w[4 * q + 2], w[4 * q + 3]);
    }
  } else if (row_ok) {
#pragma unroll
    for (int e = 0; e < 32; ++e)
      if (e < ncols) store_c_f32(p.tc, p.c, base + (int64_t)e * p.csc, v[e]);
  }
  return vmax;
}

// ------------------------------------------------------------------ the kernel
template <int BN, int KIND, bool ACT>
__global__ void __launch_bounds__(TcConfig<BN>::THREADS, 1)
    gemm_tc_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
                   const __grid_constant__ CUtensorMap tmBs, const __grid_constant__ CUtensorMap tmC,
                   const TcParams p) {
  using Cfg = TcConfig<BN>;
  constexpr int ES = (KIND == KIND_F16) ? 2 : 1;   // operand element size
  constexpr int BKE = SLAB_BYTES / ES;             // k elements per stage
  constexpr int UMMA_KE = 32 / ES;                 // k elements per tcgen05.mma
  constexpr int MN_PER_ATOM = SLAB_BYTES / ES;     // MN elements across one 128-byte swizzle row
  constexpr int ATOM_BYTES = BKE * SLAB_BYTES;     // one MN-major box: BKE rows of 128 bytes
  constexpr int A_ATOMS = BM / MN_PER_ATOM;        // MN-major boxes per A stage
  constexpr int B_ATOMS = (BN / MN_PER_ATOM) > 0 ? (BN / MN_PER_ATOM) : 1;
  static_assert(BN % MN_PER_ATOM == 0 || BN < MN_PER_ATOM, "BN must cover whole swizzle atoms");

  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw = smem_u32(smem_raw);
  const uint32_t tiles = (raw + 1023u) & ~1023u;   // stage ring, 1024-byte aligned
  const uint32_t epi_stage = tiles + Cfg::STAGES * Cfg::STAGE_BYTES;  // 4 warps x EPI_STAGE_BYTES
  const uint32_t bars = epi_stage + 4 * EPI_STAGE_BYTES;
  // barrier block: full[STAGES], empty[STAGES], tmem_full[2], tmem_empty[2], then tmem base + abort flag
  const uint32_t full_bar = bars, empty_bar = bars + 8 * Cfg::STAGES;
  const uint32_t tfull_bar = bars + 16 * Cfg::STAGES, tempty_bar = tfull_bar + 16;
  uint8_t *bar_gen = smem_raw + (bars - raw);
  volatile uint32_t *tmem_slot = reinterpret_cast<volatile uint32_t *>(bar_gen + 16 * Cfg::STAGES + 32);
  volatile uint32_t *abort_flag = tmem_slot + 1;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

  if (threadIdx.x == 0) {
    for (int s = 0; s < Cfg::STAGES; ++s) {
      mbar_init(full_bar + 8 * s, 1);
      mbar_init(empty_bar + 8 * s, 1);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(tfull_bar + 8 * b, Cfg::ISSUERS);
      mbar_init(tempty_bar + 8 * b, 128);
    }
    *abort_flag = 0u;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(
                     smem_u32((const void *)tmem_slot)),
                 "r"((uint32_t)Cfg::TMEM_COLS)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  // Launched as a programmatic dependent of the kernel before it on the stream: the set-up above ran while
  // that kernel was still draining; nothing it may have written is read before this point.  The next such
  // launch may likewise begin its own set-up as this kernel's CTAs leave.
  asm volatile("griddepcontrol.wait;" ::: "memory");
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");

  if (warp == 0) {
    // ---------------------------------------------------------------- TMA producer
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      const bool panelled = p.a_panel != PLAIN_PANEL;  // the packed matrix-engine form: both operands in panels
      TileUnit u;
      for (int it = 0; ok && get_unit<BN>(p, it, u); ++it) {
        const int m0 = u.m0, n0 = u.n0;
        // a tail strip loads only its own columns of B: a narrower box (k-major, through tmBs) or fewer boxes
        const bool strip = u.ncols != p.bn_main;
        const uint32_t stage_tx = p.a_tx + (strip ? p.tail_b_bytes : p.main_b_bytes);
        const int b_boxes = strip ? p.tail_b_atoms : p.main_b_atoms;
        // The k loop exists twice: plain operands (2-D maps, box coordinates known without arithmetic) and panelled ones
        // (3-D maps).  The producer thread issues up to five loads per stage and is close to being the bottleneck for
        // an MN-major B, so the choice is made once per tile, not once per box.
        if (!panelled) {
          for (int kb = 0; kb < p.num_kb; ++kb) {
            if (!mbar_wait(empty_bar + 8 * stage, phase ^ 1u, abort_flag, p.status, ERR_WAIT_EMPTY, p.wait_ns)) {
              ok = false;
              break;
            }
            const uint32_t fb = full_bar + 8 * stage;
            const uint32_t sa = tiles + stage * Cfg::STAGE_BYTES, sb = sa + Cfg::A_BYTES;
            mbar_expect_tx(fb, stage_tx);
            if (p.skip_loads) {  // testing aid: the bytes never arrive, the waits on this stage run out
              ok = false;
              break;
            }
            const int k0 = kb * BKE;
            if (!p.a_mn) {
              tma_load_2d(sa, &tmA, fb, k0, m0);
            } else {
#pragma unroll
              for (int i = 0; i < A_ATOMS; ++i) tma_load_2d(sa + i * ATOM_BYTES, &tmA, fb, m0 + i * MN_PER_ATOM, k0);
            }
            if (!p.b_mn) {
              tma_load_2d(sb, strip ? &tmBs : &tmB, fb, k0, n0);
            } else {
#pragma unroll
              for (int i = 0; i < B_ATOMS; ++i)
                if (i < b_boxes) tma_load_2d(sb + i * ATOM_BYTES, &tmB, fb, n0 + i * MN_PER_ATOM, k0);
            }
            if (++stage == Cfg::STAGES) {
              stage = 0;
              phase ^= 1u;
            }
          }
        } else {
          MnBoxes<A_ATOMS> abox;
          MnBoxes<B_ATOMS> bbox;
          abox.set(m0, MN_PER_ATOM, p.a_panel);
          bbox.set(n0, MN_PER_ATOM, p.b_panel);
          for (int kb = 0; kb < p.num_kb; ++kb) {
            if (!mbar_wait(empty_bar + 8 * stage, phase ^ 1u, abort_flag, p.status, ERR_WAIT_EMPTY, p.wait_ns)) {
              ok = false;
              break;
            }
            const uint32_t fb = full_bar + 8 * stage;
            const uint32_t sa = tiles + stage * Cfg::STAGE_BYTES, sb = sa + Cfg::A_BYTES;
            mbar_expect_tx(fb, stage_tx);
            if (p.skip_loads) {
              ok = false;
              break;
            }
            const int k0 = kb * BKE;
#pragma unroll
            for (int i = 0; i < A_ATOMS; ++i) tma_load_3d(sa + i * ATOM_BYTES, &tmA, fb, abox.x[i], k0, abox.z[i]);
#pragma unroll
            for (int i = 0; i < B_ATOMS; ++i)
              if (i < b_boxes) tma_load_3d(sb + i * ATOM_BYTES, &tmB, fb, bbox.x[i], k0, bbox.z[i]);
            if (++stage == Cfg::STAGES) {
              stage = 0;
              phase ^= 1u;
            }
          }
        }
      }
    }
  } else if (warp == 1 || warp >= 6) {
    // ---------------------------------------------------------------- MMA issuer(s)
    // One thread issues all MMAs, except for the 16-column tile: there a k block's 4 MMAs take the issuing thread
    // about 0.28 us whatever the width, which bounds a tall-skinny problem (a stream of A) well below the memory
    // rate.  So warps 6.. each hold one more issuing thread; issuer i takes the k blocks with kb % ISSUERS == i and
    // accumulates into its own columns.  A stage is read by exactly one issuer, whose commit hands it back.
    if (lane == 0) {
      const int me = warp == 1 ? 0 : warp - 5;
      int stage = 0;
      uint32_t phase = 0, acc = 0, acc_phase = 0;
      bool ok = true;
      // descriptor geometry per operand
      const uint32_t a_lbo = p.a_mn ? ATOM_BYTES : 16, b_lbo = p.b_mn ? ATOM_BYTES : 16;
      const uint32_t a_adv = p.a_mn ? (UMMA_KE * SLAB_BYTES) >> 4 : 32 >> 4;
      const uint32_t b_adv = p.b_mn ? (UMMA_KE * SLAB_BYTES) >> 4 : 32 >> 4;
      TileUnit u;
      for (int it = 0; ok && get_unit<BN>(p, it, u); ++it) {
        if (!mbar_wait(tempty_bar + 8 * acc, acc_phase ^ 1u, abort_flag, p.status, ERR_WAIT_TMEM_EMPTY, p.wait_ns))
          break;
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + acc * Cfg::ACC_COLS + (uint32_t)(me * BN);
        for (int kb = 0; kb < p.num_kb; ++kb) {
          if (Cfg::ISSUERS == 1 || kb % Cfg::ISSUERS == me) {
            if (!mbar_wait(full_bar + 8 * stage, phase, abort_flag, p.status, ERR_WAIT_FULL, p.wait_ns)) {
              ok = false;
              break;
            }
            tc_fence_after();
            const uint32_t sa = tiles + stage * Cfg::STAGE_BYTES, sb = sa + Cfg::A_BYTES;
            const uint64_t da = make_smem_desc(sa, a_lbo, 1024), db = make_smem_desc(sb, b_lbo, 1024);
#pragma unroll
            for (int k = 0; k < SLAB_BYTES / 32; ++k)
              umma<KIND>(d_tmem, da + (uint64_t)(k * a_adv), db + (uint64_t)(k * b_adv), u.idesc,
                         (uint32_t)((kb >= Cfg::ISSUERS) || k != 0));
            umma_commit(empty_bar + 8 * stage);
          }
          if (++stage == Cfg::STAGES) {
            stage = 0;
            phase ^= 1u;
          }
        }
        if (!ok) break;
        umma_commit(tfull_bar + 8 * acc);
        acc ^= 1u;
        if (acc == 0) acc_phase ^= 1u;
      }
    }
  } else {
    // ---------------------------------------------------------------- epilogue warps
    const int quad = warp & 3;
    uint32_t acc = 0, acc_phase = 0;
    float tile_max = -INFINITY;  // running maximum of this thread's results (optional global maximum)
    float *cs = EpiVectors<BN>::scale(bar_gen + 256, quad), *bs = EpiVectors<BN>::bias(bar_gen + 256, quad);
    const bool has_cs = p.col_scale != nullptr, has_bs = p.bias != nullptr && !p.bias_per_row;
    EpiStage st = {p.c_tma ? &tmC : nullptr, epi_stage + (uint32_t)quad * EPI_STAGE_BYTES, 0u};
    TileUnit u;
    for (int it = 0; get_unit<BN>(p, it, u); ++it) {
      const int m0 = u.m0, n0 = u.n0;
      const int row = m0 + quad * 32 + lane;
      const bool row_ok = quad * 32 + lane < p.bm_rows && row < p.M;
      EpiVectors<BN>::fill(p, cs, bs, n0, u.ncols, lane);
      const float rs = (p.row_scale && row_ok) ? __ldg(p.row_scale + row) : 1.0f;
      const float row_bias = (p.bias && p.bias_per_row && row_ok) ? __ldg(p.bias + row) : 0.0f;
      if (!mbar_wait(tfull_bar + 8 * acc, acc_phase, abort_flag, p.status, ERR_WAIT_TMEM_FULL, p.wait_ns)) break;
      tc_fence_after();
      const uint32_t taddr = tmem_base + acc * Cfg::ACC_COLS + ((uint32_t)(quad * 32) << 16);
#pragma unroll 1
      for (int c0 = 0; c0 < u.ncols; c0 += 32) {
        if (n0 + c0 >= p.N) break;  // uniform across the warp
        uint32_t r[32];
        if (BN >= 32) {
          tmem_ld32(taddr + c0, r);
        } else {
          tmem_ld16(taddr + c0, r);
          // add the other issuers' partial sums (exact for int32); an issuer that had no k block left its columns unwritten
#pragma unroll 1
          for (int a = 1; a < Cfg::ISSUERS && a < p.num_kb; ++a) {
            uint32_t r2[32];
            tmem_ld16(taddr + (uint32_t)(a * BN) + c0, r2);
#pragma unroll
            for (int i = 0; i < 16; ++i)
              r[i] = KIND == KIND_I8 ? r[i] + r2[i]
                                     : __float_as_uint(__fadd_rn(__uint_as_float(r[i]), __uint_as_float(r2[i])));
          }
        }
        tile_max = fmaxf(tile_max, epilogue_chunk<KIND == KIND_I8, ACT>(p, r, row, row_ok, n0 + c0,
                                                                        has_cs ? cs + c0 : nullptr,
                                                                        has_bs ? bs + c0 : nullptr, rs, row_bias, st, lane));
      }
      tc_fence_before();
      mbar_arrive(tempty_bar + 8 * acc);
      acc ^= 1u;
      if (acc == 0) acc_phase ^= 1u;
    }
    if (p.global_max) {
      tile_max = warp_max_f32(tile_max);
      if (lane == 0 && tile_max != -INFINITY) atomic_max_f32(p.global_max, tile_max);
    }
    if (st.tm && lane == 0) bulk_wait_all();  // the staging memory must outlive the stores that read it
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base),
                 "r"((uint32_t)Cfg::TMEM_COLS)
                 : "memory");
  }
}


// ------------------------------------------------------------------ the two-CTA kernel
// A pair of CTAs on neighbouring SMs (cluster of 2) computes one 256 x BN tile with
// tcgen05.mma.cta_group::2: CTA r of the pair stages its own 128 rows of A and its own BN/2 columns of
// B; one thread of CTA 0 issues the MMAs for both; each CTA's TMEM receives the accumulator for its
// 128 rows and all BN columns, and each CTA's epilogue warps store those rows.  Per SM this halves the
// shared-memory traffic for B (both the TMA writes and the tensor-core reads), which is what bounds
// the one-CTA kernel.  Synchronisation, all through mbarriers:
//   full[s]    lives in CTA 0; both CTAs' TMA loads credit their bytes to it (cta_group::2 loads);
//   empty[s]   one per CTA; one tcgen05.commit signals the barrier at the same offset in both CTAs
//              (two separate commits, local and remote, cost 5-10 % on every shape);
//   tfull[a]   one per CTA; signalled in both the same way when a tile's MMAs are issued;
//   tempty[a]  lives in CTA 0, 256 arrivals: the epilogue threads of both CTAs (remote arrive from CTA 1).
// No operand data is ever multicast: each CTA fetches its own bytes.
// The pair is held together by a cluster barrier after set-up and before TMEM is released.
template <int BN>
struct Tc2Config {
  static constexpr int A_BYTES = BM * SLAB_BYTES;
  static constexpr int B_BYTES = (BN / 2) * SLAB_BYTES;
  static constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
  static constexpr int STAGES_RAW = (220 * 1024) / STAGE_BYTES;
  static constexpr int STAGES = STAGES_RAW > 8 ? 8 : STAGES_RAW;
  static constexpr int TMEM_COLS = 2 * BN;
  static constexpr int SMEM_BYTES = STAGES * STAGE_BYTES + 1024 + 4 * EPI_STAGE_BYTES + 256 + EpiVectors<BN>::BYTES;
  static_assert(SMEM_BYTES <= 227 * 1024, "exceeds the shared memory one CTA can have");
};

template <int BN, int KIND, bool ACT>
__global__ void __launch_bounds__(NUM_THREADS, 1)
    gemm_tc2_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
                    const __grid_constant__ CUtensorMap tmC, const TcParams p) {
  using Cfg = Tc2Config<BN>;
  constexpr int ES = (KIND == KIND_F16) ? 2 : 1;
  constexpr int BKE = SLAB_BYTES / ES;
  constexpr int UMMA_KE = 32 / ES;
  constexpr int MN_PER_ATOM = SLAB_BYTES / ES;
  constexpr int ATOM_BYTES = BKE * SLAB_BYTES;
  constexpr int A_ATOMS = BM / MN_PER_ATOM;
  constexpr int BH = BN / 2;  // columns of B staged by each CTA
  constexpr int B_ATOMS = (BH / MN_PER_ATOM) > 0 ? (BH / MN_PER_ATOM) : 1;

  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw = smem_u32(smem_raw);
  const uint32_t tiles = (raw + 1023u) & ~1023u;
  const uint32_t epi_stage = tiles + Cfg::STAGES * Cfg::STAGE_BYTES;  // 4 warps x EPI_STAGE_BYTES
  const uint32_t bars = epi_stage + 4 * EPI_STAGE_BYTES;
  const uint32_t full_bar = bars, empty_bar = bars + 8 * Cfg::STAGES;
  const uint32_t tfull_bar = bars + 16 * Cfg::STAGES, tempty_bar = tfull_bar + 16;
  uint8_t *bar_gen = smem_raw + (bars - raw);
  volatile uint32_t *tmem_slot = reinterpret_cast<volatile uint32_t *>(bar_gen + 16 * Cfg::STAGES + 32);
  volatile uint32_t *abort_flag = tmem_slot + 1;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t rank = cluster_ctarank();  // 0 = leader (issues the MMAs)
  const int pair = blockIdx.x >> 1, num_pairs = gridDim.x >> 1;

  if (threadIdx.x == 0) {
    for (int s = 0; s < Cfg::STAGES; ++s) {
      mbar_init(full_bar + 8 * s, 1);
      mbar_init(empty_bar + 8 * s, 1);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(tfull_bar + 8 * b, 1);
      mbar_init(tempty_bar + 8 * b, 256);
    }
    *abort_flag = 0u;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(
                     smem_u32((const void *)tmem_slot)),
                 "r"((uint32_t)Cfg::TMEM_COLS)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
  }
  tc_fence_before();
  __syncthreads();
  cluster_sync_all();  // both CTAs' barriers are initialised before either touches the other's
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  asm volatile("griddepcontrol.wait;" ::: "memory");  // see gemm_tc_kernel
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");

  const int num_tiles = p.tiles_m * p.tiles_n;  // tiles of 256 rows

  if (warp == 0) {
    // ---------------------------------------------------------------- TMA producer (both CTAs)
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      const uint32_t leader_full = mapa(full_bar, 0);
      for (int t = pair; ok && t < num_tiles; t += num_pairs) {
        int mi, ni;
        tile_coords(t, p.tiles_m, p.tiles_n, p.raster_gm, mi, ni);
        const int m0 = mi * (2 * BM) + (int)rank * BM, n0 = ni * BN + (int)rank * BH;
        MnBoxes<A_ATOMS> abox;
        MnBoxes<B_ATOMS> bbox;
        if (p.a_panel != PLAIN_PANEL) abox.set(m0, MN_PER_ATOM, p.a_panel);
        if (p.b_panel != PLAIN_PANEL) bbox.set(n0, MN_PER_ATOM, p.b_panel);
        for (int kb = 0; kb < p.num_kb; ++kb) {
          if (!mbar_wait(empty_bar + 8 * stage, phase ^ 1u, abort_flag, p.status, ERR_WAIT_EMPTY, p.wait_ns)) {
            ok = false;
            break;
          }
          const uint32_t fb = leader_full + 8 * stage;
          const uint32_t sa = tiles + stage * Cfg::STAGE_BYTES, sb = sa + Cfg::A_BYTES;
          if (rank == 0) mbar_expect_tx(full_bar + 8 * stage, 2 * Cfg::STAGE_BYTES);
          if (p.skip_loads) {  // testing aid, as in gemm_tc_kernel
            ok = false;
            break;
          }
          const int k0 = kb * BKE;
          if (!p.a_mn) {
            tma_load_2d_pair(sa, &tmA, fb, k0, m0);
          } else {
#pragma unroll
            for (int i = 0; i < A_ATOMS; ++i) {
              if (p.a_panel == PLAIN_PANEL)
                tma_load_2d_pair(sa + i * ATOM_BYTES, &tmA, fb, m0 + i * MN_PER_ATOM, k0);
              else
                tma_load_3d_pair(sa + i * ATOM_BYTES, &tmA, fb, abox.x[i], k0, abox.z[i]);
            }
          }
          if (!p.b_mn) {
            tma_load_2d_pair(sb, &tmB, fb, k0, n0);
          } else {
#pragma unroll
            for (int i = 0; i < B_ATOMS; ++i) {
              if (p.b_panel == PLAIN_PANEL)
                tma_load_2d_pair(sb + i * ATOM_BYTES, &tmB, fb, n0 + i * MN_PER_ATOM, k0);
              else
                tma_load_3d_pair(sb + i * ATOM_BYTES, &tmB, fb, bbox.x[i], k0, bbox.z[i]);
            }
          }
          if (++stage == Cfg::STAGES) {
            stage = 0;
            phase ^= 1u;
          }
        }
      }
    }
  } else if (warp == 1) {
    // ---------------------------------------------------------------- MMA issuer (leader CTA only)
    if (lane == 0 && rank == 0) {
      int stage = 0;
      uint32_t phase = 0, acc = 0, acc_phase = 0;
      bool ok = true;
      const uint32_t a_lbo = p.a_mn ? ATOM_BYTES : 16, b_lbo = p.b_mn ? ATOM_BYTES : 16;
      const uint32_t a_adv = p.a_mn ? (UMMA_KE * SLAB_BYTES) >> 4 : 32 >> 4;
      const uint32_t b_adv = p.b_mn ? (UMMA_KE * SLAB_BYTES) >> 4 : 32 >> 4;
      for (int t = pair; ok && t < num_tiles; t += num_pairs) {
        if (!mbar_wait(tempty_bar + 8 * acc, acc_phase ^ 1u, abort_flag, p.status, ERR_WAIT_TMEM_EMPTY, p.wait_ns))
          break;
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + acc * BN;
        for (int kb = 0; kb < p.num_kb; ++kb) {
          if (!mbar_wait(full_bar + 8 * stage, phase, abort_flag, p.status, ERR_WAIT_FULL, p.wait_ns)) {
            ok = false;
            break;
          }
          tc_fence_after();
          const uint32_t sa = tiles + stage * Cfg::STAGE_BYTES, sb = sa + Cfg::A_BYTES;
          const uint64_t da = make_smem_desc(sa, a_lbo, 1024), db = make_smem_desc(sb, b_lbo, 1024);
#pragma unroll
          for (int k = 0; k < SLAB_BYTES / 32; ++k)
            umma_pair<KIND>(d_tmem, da + (uint64_t)(k * a_adv), db + (uint64_t)(k * b_adv), p.idesc,
                            (uint32_t)((kb | k) != 0));
          umma_commit_pair_both(empty_bar + 8 * stage);
          if (++stage == Cfg::STAGES) {
            stage = 0;
            phase ^= 1u;
          }
        }
        if (!ok) break;
        umma_commit_pair_both(tfull_bar + 8 * acc);
        acc ^= 1u;
        if (acc == 0) acc_phase ^= 1u;
      }
    }
  } else {
    // ---------------------------------------------------------------- epilogue warps (both CTAs)
    const int quad = warp & 3;
    uint32_t acc = 0, acc_phase = 0;
    float tile_max = -INFINITY;
    const uint32_t leader_tempty = mapa(tempty_bar, 0);
    float *cs = EpiVectors<BN>::scale(bar_gen + 256, quad), *bs = EpiVectors<BN>::bias(bar_gen + 256, quad);
    const bool has_cs = p.col_scale != nullptr, has_bs = p.bias != nullptr && !p.bias_per_row;
    EpiStage st = {p.c_tma ? &tmC : nullptr, epi_stage + (uint32_t)quad * EPI_STAGE_BYTES, 0u};
    for (int t = pair; t < num_tiles; t += num_pairs) {
      int mi, ni;
      tile_coords(t, p.tiles_m, p.tiles_n, p.raster_gm, mi, ni);
      const int m0 = mi * (2 * BM) + (int)rank * BM, n0 = ni * BN;
      const int row = m0 + quad * 32 + lane;
      EpiVectors<BN>::fill(p, cs, bs, n0, BN, lane);
      const float rs = (p.row_scale && row < p.M) ? __ldg(p.row_scale + row) : 1.0f;
      const float row_bias = (p.bias && p.bias_per_row && row < p.M) ? __ldg(p.bias + row) : 0.0f;
      if (!mbar_wait(tfull_bar + 8 * acc, acc_phase, abort_flag, p.status, ERR_WAIT_TMEM_FULL, p.wait_ns)) break;
      tc_fence_after();
      const uint32_t taddr = tmem_base + acc * BN + ((uint32_t)(quad * 32) << 16);
#pragma unroll 1
      for (int c0 = 0; c0 < BN; c0 += 32) {
        if (n0 + c0 >= p.N) break;
        uint32_t r[32];
        tmem_ld32(taddr + c0, r);
        tile_max = fmaxf(tile_max, epilogue_chunk<KIND == KIND_I8, ACT>(p, r, row, row < p.M, n0 + c0,
                                                                        has_cs ? cs + c0 : nullptr,
                                                                        has_bs ? bs + c0 : nullptr, rs, row_bias, st, lane));
      }
      tc_fence_before();
      mbar_arrive_cluster(leader_tempty + 8 * acc);
      acc ^= 1u;
      if (acc == 0) acc_phase ^= 1u;
    }
    if (p.global_max) {
      tile_max = warp_max_f32(tile_max);
      if (lane == 0 && tile_max != -INFINITY) atomic_max_f32(p.global_max, tile_max);
    }
    if (st.tm && lane == 0) bulk_wait_all();  // the staging memory must outlive the stores that read it
  }

  tc_fence_before();
  __syncthreads();
  cluster_sync_all();  // neither CTA's barriers or TMEM are touched by the partner after this point
  if (warp == 1) {
    tc_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(tmem_base),
                 "r"((uint32_t)Cfg::TMEM_COLS)
                 : "memory");
  }
}

// ====================================================================== MX-FP4 (block-scaled E2M1) GEMM
// C[m, n] (fp32, row-major) = beta * C + alpha * sum_k A[m, k] * B[n, k], A and B packed E2M1 (two per byte, k
// contiguous) with one E8M0 scale per 32 consecutive k, on tcgen05.mma.kind::mxf4.block_scale (K = 64 per instruction,
// two scales per row and instruction; the scale bytes of an instruction are picked by the scale-factor id in the
// instruction descriptor: 0 or 2 inside the 4-byte column).
//
// Scales.  The smem -> TMEM scale copy (tcgen05.cp 32x128b.warpx4) wants, per 128 rows and 4 k blocks, a 512-byte
// chunk with row r at (r % 32) * 16 + (r / 32) * 4.  mx_pack_scales_kernel re-lays the caller's row-major scale
// matrices into [row tile][chunk][512 bytes] once per call (one launch for both operands) (rows and k blocks that do not exist get 127 = 1.0), after
// which a stage's scales of A and of B are one 1024-byte bulk copy each.
//
// Kernel.  Persistent, one CTA per SM, 128 x 256 tiles (n fastest): the tensor core spends 128 clocks on an MMA of 128
// rows whatever its width, so only 256-column instructions reach its rate (128 x 128 tiles measured 2.6 PFLOP/s with
// the pipe 30 % busy).  4 stages of 256 elements of k: a 128 x 128-byte box of A, a 256 x 128-byte box of B (TMA,
// 128-byte swizzle) and three 1 KiB scale pieces.  Warp 0 issues the copies, warp 1 the scale copies into TMEM and the
// MMAs (the scale copies come from warp 10), warps 2..9 run the epilogue.  The accumulator takes 256 of the 512 TMEM columns and the scales need columns
// too, so there is one accumulator: the epilogue warps copy it into registers at once (128 columns per thread) and
// hand it back, so that only those loads, not the stores, keep the tensor core waiting.  Every wait is bounded like the main kernel's.
namespace mx {
constexpr int BM = 128, BN = 256, STAGE_K_BYTES = 128, STAGES = 4;
constexpr int A_BYTES = BM * STAGE_K_BYTES, B_BYTES = BN * STAGE_K_BYTES, SF_BYTES = 2 * 512;  // SF_BYTES: 128 rows, one stage
constexpr int STAGE_BYTES = A_BYTES + B_BYTES + 3 * SF_BYTES;  // scales: 128 rows of A, 2 x 128 columns of B
constexpr int SMEM_BYTES = 1024 + STAGES * STAGE_BYTES + 256;
constexpr int THREADS = 352;  // producer, MMA issuer, 8 epilogue warps, scale copier
constexpr uint32_t ERR_EMPTY = 0x301, ERR_FULL = 0x302, ERR_TFULL = 0x303, ERR_TEMPTY = 0x304, ERR_SF = 0x305;

struct Params {
  const uint8_t *psa, *psb;  // packed scales: [row tile][stage][1024 bytes]
  float *c;
  int64_t rsc;
  int M, N, kblocks;         // kblocks = K / 32
  int tiles_m, tiles_n;
  float alpha, beta;
  uint64_t wait_ns;
  uint32_t *status;
  int c_vec;                 // the rows of C are 16-byte aligned
};

// dst[(tile * chunks + chunk) * 512 + (r % 32) * 16 + (r / 32) * 4 + e] = src[(tile * 128 + r) * ld + chunk * 4 + e],
// for the scales of A (the first total_a words) and of B (the rest) in one launch
__global__ void __launch_bounds__(256)
    mx_pack_scales_kernel(uint32_t *__restrict__ dst_a, const uint8_t *__restrict__ src_a, int64_t ld_a, int rows_a,
                          int64_t total_a, uint32_t *__restrict__ dst_b, const uint8_t *__restrict__ src_b, int64_t ld_b,
                          int rows_b, int64_t total_b, int kblocks, int chunks) {
  const int64_t stride = (int64_t)gridDim.x * blockDim.x;
  for (int64_t j = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; j < total_a + total_b; j += stride) {
    const bool second = j >= total_a;
    const int64_t i = second ? j - total_a : j;
    const uint8_t *src = second ? src_b : src_a;
    const int64_t ld = second ? ld_b : ld_a;
    const int rows = second ? rows_b : rows_a;
    // i = (tile * chunks + chunk) * 128 + slot, slot = (r % 32) * 4 + r / 32  (one 4-byte word each)
    const int slot = (int)(i & 127);
    const int64_t tc = i >> 7;
    const int chunk = (int)(tc % chunks);
    const int64_t tile = tc / chunks;
    const int r = (slot >> 2) + 32 * (slot & 3);
    const int64_t row = tile * 128 + r;
    uint32_t w = 0x7F7F7F7Fu;
    if (row < rows) {
      const uint8_t *sp = src + row * ld + chunk * 4;
#pragma unroll
      for (int e = 0; e < 4; ++e)
        if (chunk * 4 + e < kblocks) w = (w & ~(0xFFu << (8 * e))) | ((uint32_t)__ldg(sp + e) << (8 * e));
    }
    (second ? dst_b : dst_a)[i] = w;
  }
}

// no-swizzle k-major descriptor of a 32-row x 16-byte scale chunk: 8-row groups 128 bytes apart
__device__ __forceinline__ uint64_t sf_desc(uint32_t saddr) {
  uint64_t d = 0;
  d |= (uint64_t)((saddr >> 4) & 0x3FFFu);
  d |= (uint64_t)(128u >> 4) << 32;
  d |= 1ull << 46;
  return d;
}
__device__ __forceinline__ void bulk_load(uint32_t dst, const void *src, uint32_t bytes, uint32_t bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(dst), "l"(src),
               "r"(bytes), "r"(bar)
               : "memory");
}

// 32 accumulator columns of this thread's lane, without waiting for the load
__device__ __forceinline__ void tmem_ld32_async(uint32_t taddr, uint32_t (&r)[32]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
      "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
        "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]),
        "=r"(r[15]), "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]),
        "=r"(r[22]), "=r"(r[23]), "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]),
        "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
      : "r"(taddr));
}

__global__ void __launch_bounds__(THREADS, 1)
    gemm_mxf4_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB, const Params p) {
  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw = smem_u32(smem_raw);
  const uint32_t tiles = (raw + 1023u) & ~1023u;
  const uint32_t bars = tiles + STAGES * STAGE_BYTES;
  const uint32_t full_bar = bars, empty_bar = bars + 8 * STAGES, tfull_bar = bars + 16 * STAGES, tempty_bar = tfull_bar + 16;
  const uint32_t sf_bar = tfull_bar + 32;  // [2]: the scales of a stage are in their TMEM region
  uint8_t *gen = smem_raw + (bars - raw);
  volatile uint32_t *tmem_slot = reinterpret_cast<volatile uint32_t *>(gen + 16 * STAGES + 64);
  volatile uint32_t *abort_flag = tmem_slot + 1;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int num_kb = (p.kblocks + 7) / 8;  // stages of 256 elements per tile
  const int total_tiles = p.tiles_m * p.tiles_n;

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(full_bar + 8 * s, 1);
      mbar_init(empty_bar + 8 * s, 1);
    }
    mbar_init(tfull_bar, 1);
    mbar_init(tempty_bar, 256);
    mbar_init(sf_bar, 1);
    mbar_init(sf_bar + 8, 1);
    *abort_flag = 0u;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], 512;" ::"r"(
                     smem_u32((const void *)tmem_slot))
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0) {
    if (lane == 0) {
      int g = 0;  // stages issued so far, over all tiles
      bool ok = true;
      for (int t = (int)blockIdx.x; ok && t < total_tiles; t += (int)gridDim.x) {
        const int mi = t / p.tiles_n, ni = t - mi * p.tiles_n;
        const uint8_t *sfa_src = p.psa + (int64_t)mi * num_kb * SF_BYTES, *sfb_src = p.psb + (int64_t)(2 * ni) * num_kb * SF_BYTES;
        for (int kb = 0; kb < num_kb; ++kb, ++g) {
          const int stage = g % STAGES;
          if (g >= STAGES &&
              !mbar_wait(empty_bar + 8 * stage, (uint32_t)(g / STAGES - 1) & 1u, abort_flag, p.status, ERR_EMPTY, p.wait_ns)) {
            ok = false;
            break;
          }
          const uint32_t sa = tiles + stage * STAGE_BYTES, sb = sa + A_BYTES, sfa = sb + B_BYTES, sfb = sfa + SF_BYTES;
          const uint32_t fb = full_bar + 8 * stage;
          mbar_expect_tx(fb, STAGE_BYTES);
          tma_load_2d(sa, &tmA, fb, kb * STAGE_K_BYTES, mi * BM);
          tma_load_2d(sb, &tmB, fb, kb * STAGE_K_BYTES, ni * BN);
          bulk_load(sfa, sfa_src + (int64_t)kb * SF_BYTES, SF_BYTES, fb);
          bulk_load(sfb, sfb_src + (int64_t)kb * SF_BYTES, SF_BYTES, fb);                               // columns 0..127
          bulk_load(sfb + SF_BYTES, sfb_src + (int64_t)(num_kb + kb) * SF_BYTES, SF_BYTES, fb);  // columns 128..255
        }
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      int g = 0;
      uint32_t acc_phase = 0;
      bool ok = true;
      for (int t = (int)blockIdx.x; ok && t < total_tiles; t += (int)gridDim.x) {
        // one accumulator (256 of the 512 columns; the scales need columns too): the epilogue of the previous tile
        // must have read it, while the copies of this tile's first stages are already under way
        if (!mbar_wait(tempty_bar, acc_phase ^ 1u, abort_flag, p.status, ERR_TEMPTY, p.wait_ns)) break;
        tc_fence_after();
        const uint32_t d_tmem = tmem_base;
        for (int kb = 0; kb < num_kb; ++kb, ++g) {
          const int stage = g % STAGES;
          if (!mbar_wait(full_bar + 8 * stage, (uint32_t)(g / STAGES) & 1u, abort_flag, p.status, ERR_FULL, p.wait_ns)) {
            ok = false;
            break;
          }
          tc_fence_after();
          const uint32_t sa = tiles + stage * STAGE_BYTES, sb = sa + A_BYTES;
          // the scale copier (warp 10) has put this stage's scales into TMEM region g % 2 (columns 256 + 32 (g % 2)):
          // A chunks at +0, +4; B chunk c at +8 + 8 c (columns 0..127 of the tile) and +12 + 8 c (columns 128..255)
          const uint32_t tsf = tmem_base + 256u + (uint32_t)(g & 1) * 32u;
          if (!mbar_wait(sf_bar + 8 * (g & 1), (uint32_t)(g >> 1) & 1u, abort_flag, p.status, ERR_SF, p.wait_ns)) {
            ok = false;
            break;
          }
          tc_fence_after();
          const uint64_t da = make_smem_desc(sa, 16, 1024), db = make_smem_desc(sb, 16, 1024);
          const int left = p.kblocks - kb * 8;               // scale blocks left from this stage on
          const int mmas = left >= 8 ? 4 : (left + 1) / 2;   // 64 elements = 2 scale blocks per instruction
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            if (j < mmas) {
              const uint32_t sf_id = (uint32_t)(j & 1) * 2u;
              // E2M1 x E2M1, E8M0 scales, N = 256, M = 128, K = 64
              const uint32_t idesc = (sf_id << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(BN >> 3) << 17) | (1u << 23) |
                                     ((uint32_t)(BM >> 4) << 24) | (sf_id << 29);
              const uint32_t accum = (uint32_t)((kb | j) != 0);
              asm volatile(
                  "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
                  "tcgen05.mma.cta_group::1.kind::mxf4.block_scale.scale_vec::2X [%0], %1, %2, %3, [%5], [%6], p;\n\t}" ::"r"(
                      d_tmem),
                  "l"(da + (uint64_t)(2 * j)), "l"(db + (uint64_t)(2 * j)), "r"(idesc), "r"(accum),
                  "r"(tsf + 4u * (uint32_t)(j >> 1)), "r"(tsf + 8u + 8u * (uint32_t)(j >> 1))
                  : "memory");
            }
          }
          umma_commit(empty_bar + 8 * stage);
        }
        if (!ok) break;
        umma_commit(tfull_bar);
        acc_phase ^= 1u;
      }
    }
  } else if (warp == 10) {
    // ---- scale copier: smem -> TMEM copies of a stage's scales, issued from a thread of its own so that they do not
    // queue between the MMAs of the issuing thread.  Stage g's copies may overwrite region g % 2 once the MMAs of stage
    // g - 2 are done, which is when that stage's buffer was handed back.
    if (lane == 0) {
      int g = 0;
      bool ok = true;
      for (int t = (int)blockIdx.x; ok && t < total_tiles; t += (int)gridDim.x) {
        for (int kb = 0; kb < num_kb; ++kb, ++g) {
          const int stage = g % STAGES;
          if (!mbar_wait(full_bar + 8 * stage, (uint32_t)(g / STAGES) & 1u, abort_flag, p.status, ERR_FULL, p.wait_ns)) {
            ok = false;
            break;
          }
          if (g >= 2) {
            const int g2 = g - 2;
            if (!mbar_wait(empty_bar + 8 * (g2 % STAGES), (uint32_t)(g2 / STAGES) & 1u, abort_flag, p.status, ERR_EMPTY, p.wait_ns)) {
              ok = false;
              break;
            }
          }
          tc_fence_after();
          const uint32_t sfa = tiles + stage * STAGE_BYTES + A_BYTES + B_BYTES, sfb = sfa + SF_BYTES;
          const uint32_t tsf = tmem_base + 256u + (uint32_t)(g & 1) * 32u;
#pragma unroll
          for (int c = 0; c < 2; ++c) {
            asm volatile("tcgen05.cp.cta_group::1.32x128b.warpx4 [%0], %1;" ::"r"(tsf + 4u * c), "l"(sf_desc(sfa + 512u * c)) : "memory");
            asm volatile("tcgen05.cp.cta_group::1.32x128b.warpx4 [%0], %1;" ::"r"(tsf + 8u + 8u * c), "l"(sf_desc(sfb + 512u * c)) : "memory");
            asm volatile("tcgen05.cp.cta_group::1.32x128b.warpx4 [%0], %1;" ::"r"(tsf + 12u + 8u * c), "l"(sf_desc(sfb + SF_BYTES + 512u * c)) : "memory");
          }
          umma_commit(sf_bar + 8 * (g & 1));
        }
      }
    }
  } else {
    // ---- epilogue.  There is one accumulator, so the tensor core waits while it is read: 8 warps (quarter q = warp % 4
    // reads lanes 32 q .., lane = row; warps 2..5 take columns 0..127, warps 6..9 columns 128..255) pull their 128
    // columns into registers at once and hand the accumulator back before they scale and store.
    const int quad = warp & 3, half = warp >= 6 ? 1 : 0;
    uint32_t acc_phase = 0;
    for (int t = (int)blockIdx.x; t < total_tiles; t += (int)gridDim.x) {
      const int mi = t / p.tiles_n, ni = t - mi * p.tiles_n;
      const int row = mi * BM + quad * 32 + lane, n0 = ni * BN + half * (BN / 2);
      if (!mbar_wait(tfull_bar, acc_phase, abort_flag, p.status, ERR_TFULL, p.wait_ns)) break;
      tc_fence_after();
      const uint32_t taddr = tmem_base + (uint32_t)(half * (BN / 2)) + ((uint32_t)(quad * 32) << 16);
      uint32_t r[4][32];
#pragma unroll
      for (int ch = 0; ch < 4; ++ch) tmem_ld32_async(taddr + 32 * ch, r[ch]);
      asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
      tc_fence_before();
      mbar_arrive(tempty_bar);
      acc_phase ^= 1u;
      if (row < p.M) {
#pragma unroll
        for (int ch = 0; ch < 4; ++ch) {
          const int c0 = 32 * ch;
          if (n0 + c0 >= p.N) break;
          float *cp = p.c + (int64_t)row * p.rsc + n0 + c0;
          if (p.c_vec && n0 + c0 + 32 <= p.N) {  // 16-byte stores: eight per lane cover the chunk's 128 bytes of the row
#pragma unroll
            for (int q = 0; q < 8; ++q) {
              float4 v = make_float4(__fmul_rn(p.alpha, __uint_as_float(r[ch][4 * q])), __fmul_rn(p.alpha, __uint_as_float(r[ch][4 * q + 1])),
                                     __fmul_rn(p.alpha, __uint_as_float(r[ch][4 * q + 2])), __fmul_rn(p.alpha, __uint_as_float(r[ch][4 * q + 3])));
              if (p.beta != 0.0f) {
                const float4 o = *reinterpret_cast<const float4 *>(cp + 4 * q);
                v.x = __fadd_rn(__fmul_rn(p.beta, o.x), v.x);
                v.y = __fadd_rn(__fmul_rn(p.beta, o.y), v.y);
                v.z = __fadd_rn(__fmul_rn(p.beta, o.z), v.z);
                v.w = __fadd_rn(__fmul_rn(p.beta, o.w), v.w);
              }
              *reinterpret_cast<float4 *>(cp + 4 * q) = v;
            }
          } else {
#pragma unroll
            for (int e = 0; e < 32; ++e) {
              if (n0 + c0 + e < p.N) {
                float v = __fmul_rn(p.alpha, __uint_as_float(r[ch][e]));
                if (p.beta != 0.0f) v = __fadd_rn(__fmul_rn(p.beta, cp[e]), v);
                cp[e] = v;
              }
            }
          }
        }
      }
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, 512;" ::"r"(tmem_base) : "memory");
  }
}
}  // namespace mx


// ------------------------------------------------------------------ host side
typedef CUresult (*EncodeTiledFn)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *, const cuuint64_t *,
                                  const cuuint64_t *, const cuuint32_t *, const cuuint32_t *,
                                  CUtensorMapInterleave, CUtensorMapSwizzle, CUtensorMapL2promotion,
                                  CUtensorMapFloatOOBfill);

EncodeTiledFn encode_fn() {
  static EncodeTiledFn fn = nullptr;
  static bool tried = false;
  if (!tried) {
    tried = true;
    void *sym = nullptr;
    cudaDriverEntryPointQueryResult qres;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &sym, cudaEnableDefault, &qres) == cudaSuccess &&
        qres == cudaDriverEntryPointSuccess)
      fn = (EncodeTiledFn)sym;
  }
  return fn;
}

struct OperandView {
  int mn_major;     // 1: unit stride runs along m (A) / n (B)
  int64_t ld;       // leading stride in elements (MN-major: the stride between consecutive k)
  bool ok;
  // MN-major only: the operand as `panels` panels of `panel` consecutive m (n) elements, `panel_ld` elements apart
  int64_t panel, panels, panel_ld;
  bool panel_form;  // SKL's packed matrix-engine operand (3-D tensor map) rather than a plain matrix
};

// extent_mn x K operand with strides (s_mn, s_k) in elements.
OperandView classify(const void *base, int64_t extent_mn, int64_t K, int64_t s_mn, int64_t s_k, int es) {
  OperandView v{0, 0, false, extent_mn, 1, 0, false};
  if ((reinterpret_cast<uintptr_t>(base) & 15u) != 0) return v;
  auto ld_ok = [&](int64_t ld, int64_t inner, int64_t outer) {
    if (outer <= 1) return true;
    return ld >= inner && ((ld * es) & 15) == 0;
  };
  if (s_k == 1 && ld_ok(s_mn, K, extent_mn)) {  // K-major
    v.mn_major = 0;
    v.ld = s_mn;
    v.ok = true;
  } else if (s_mn == 1 && ld_ok(s_k, extent_mn, K)) {  // MN-major
    v.mn_major = 1;
    v.ld = s_k;
    v.ok = true;
  }
  return v;
}

// SKL's matrix-engine packed operand (src/gemm/gemm_i8c_i8_i32_xsfmm32a8i.h:86-100): blocks of `panel` x 1 (A) or
// 1 x `panel` (B) elements with unit stride inside a block, `k_stride` between consecutive k and `panel_stride`
// between block rows (A) / block columns (B).  TMA reads it as an MN-major operand when a panel is a whole number
// of 128-byte rows.
OperandView classify_panels(const void *base, int64_t panel, int64_t panels, int64_t K, int64_t k_stride,
                            int64_t panel_stride, int es) {
  OperandView v{1, k_stride, false, panel, panels, panel_stride, true};
  if ((reinterpret_cast<uintptr_t>(base) & 15u) != 0) return v;
  if (panel <= 0 || (panel * es) % SLAB_BYTES != 0) return v;
  if (K > 1 && (k_stride < panel || ((k_stride * es) & 15) != 0)) return v;
  if (panels > 1 && (panel_stride < panel || ((panel_stride * es) & 15) != 0)) return v;
  v.ok = true;
  return v;
}

// The two operand views of a problem: plain matrices (one block per dimension) or the panel form above
// (k0 == 1: every k is its own block row / column).
bool operand_views(const skl_b200_gemm_args *g, int es, OperandView &va, OperandView &vb) {
  const int64_t K = (int64_t)(g->k0 * g->k1);
  if (g->m1 == 1 && g->n1 == 1 && g->k1 == 1) {
    va = classify(g->a, (int64_t)g->m0, K, g->rsa0, g->csa0, es);
    vb = classify(g->b, (int64_t)g->n0, K, g->csb0, g->rsb0, es);
    return va.ok && vb.ok;
  }
  if (g->k0 != 1 || g->rsa0 != 1 || g->csb0 != 1) return false;
  va = classify_panels(g->a, (int64_t)g->m0, (int64_t)g->m1, K, g->csa1, g->rsa1, es);
  vb = classify_panels(g->b, (int64_t)g->n0, (int64_t)g->n1, K, g->rsb1, g->csb1, es);
  return va.ok && vb.ok;
}

int kind_of(int ta, int tb) {
  if (ta == SKL_DT_I8 && tb == SKL_DT_I8) return KIND_I8;
  if ((ta == SKL_DT_BF16 && tb == SKL_DT_BF16) || (ta == SKL_DT_F16 && tb == SKL_DT_F16)) return KIND_F16;
  const bool fa = (ta == SKL_DT_F8E4M3 || ta == SKL_DT_F8E5M2), fb = (tb == SKL_DT_F8E4M3 || tb == SKL_DT_F8E5M2);
  if (fa && fb) return KIND_F8;
  return -1;
}

bool make_map(CUtensorMap *tm, int kind, int dt, const void *base, const OperandView &v, int64_t extent_mn,
              int64_t K, int box_mn) {
  EncodeTiledFn enc = encode_fn();
  if (!enc) return false;
  const int es = kind == KIND_F16 ? 2 : 1;
  CUtensorMapDataType cdt = kind == KIND_F16 ? (dt == SKL_DT_BF16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16
                                                                  : CU_TENSOR_MAP_DATA_TYPE_FLOAT16)
                                             : CU_TENSOR_MAP_DATA_TYPE_UINT8;
  cuuint64_t dims[3], strides[2];
  cuuint32_t box[3], estr[3] = {1, 1, 1};
  const int per_row = SLAB_BYTES / es;  // elements across 128 bytes
  cuuint32_t rank = 2;
  if (!v.mn_major) {
    dims[0] = (cuuint64_t)K;
    dims[1] = (cuuint64_t)extent_mn;
    box[0] = (cuuint32_t)per_row;
    box[1] = (cuuint32_t)box_mn;
    int64_t ld = v.ld;
    if (dims[1] <= 1) ld = (int64_t)((dims[0] * es + 15) / 16 * 16) / es;  // stride unused; keep it legal
    strides[0] = (cuuint64_t)ld * es;
  } else if (!v.panel_form) {
    dims[0] = (cuuint64_t)extent_mn;
    dims[1] = (cuuint64_t)K;
    box[0] = (cuuint32_t)per_row;
    box[1] = (cuuint32_t)per_row;  // BKE rows
    int64_t ld = v.ld;
    if (dims[1] <= 1) ld = (int64_t)((dims[0] * es + 15) / 16 * 16) / es;  // stride unused; keep it legal
    strides[0] = (cuuint64_t)ld * es;
  } else {
    // (element in panel, k, panel)
    rank = 3;
    dims[0] = (cuuint64_t)v.panel;
    dims[1] = (cuuint64_t)K;
    dims[2] = (cuuint64_t)v.panels;
    box[0] = (cuuint32_t)per_row;
    box[1] = (cuuint32_t)per_row;  // BKE rows
    box[2] = 1;
    int64_t ld = v.ld;
    if (dims[1] <= 1) ld = (int64_t)((dims[0] * es + 15) / 16 * 16) / es;  // stride unused; keep it legal
    strides[0] = (cuuint64_t)ld * es;
    int64_t pld = v.panels > 1 ? v.panel_ld : ld;  // unused for a single panel; keep it legal
    strides[1] = (cuuint64_t)pld * es;
  }
  CUresult r = enc(tm, cdt, rank, const_cast<void *>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                   CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                   CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS;
}

// Tensor map of C for the epilogue's stores: boxes of 32 rows x 32 columns (16 columns for 4-byte elements),
// swizzled over the box's row bytes (64 / 64 / 32 for 4- / 2- / 1-byte elements) to match tma_store_box.
bool make_c_map(CUtensorMap *tm, void *base, int64_t M, int64_t N, int64_t ld, int es) {
  EncodeTiledFn enc = encode_fn();
  if (!enc) return false;
  cuuint64_t dims[2] = {(cuuint64_t)N, (cuuint64_t)M}, strides[1];
  cuuint32_t box[2] = {es == 4 ? 16u : 32u, 32}, estr[2] = {1, 1};
  if (M <= 1) ld = (int64_t)((N * es + 15) / 16 * 16) / es;  // stride unused; keep it legal
  strides[0] = (cuuint64_t)ld * es;
  const CUtensorMapDataType cdt = es == 4   ? CU_TENSOR_MAP_DATA_TYPE_UINT32
                                  : es == 2 ? CU_TENSOR_MAP_DATA_TYPE_UINT16
                                            : CU_TENSOR_MAP_DATA_TYPE_UINT8;
  const CUtensorMapSwizzle sw = es == 1 ? CU_TENSOR_MAP_SWIZZLE_32B : CU_TENSOR_MAP_SWIZZLE_64B;
  CUresult r = enc(tm, cdt, 2, base, dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, sw,
                   CU_TENSOR_MAP_L2_PROMOTION_NONE, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS;
}

uint32_t fmt_code(int kind, int dt) {
  if (kind == KIND_F16) return dt == SKL_DT_BF16 ? 1u : 0u;
  if (kind == KIND_I8) return 1u;  // signed 8-bit
  return dt == SKL_DT_F8E5M2 ? 1u : 0u;
}

int current_device() {
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess) (void)cudaGetLastError();
  return (dev < 0 || dev >= 64) ? 0 : dev;
}

int sm_count() {
  static int sms = 0;
  if (sms == 0) {
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, current_device());
    if (sms <= 0) sms = 148;
  }
  return sms;
}

int pick_bn(int64_t M, int64_t N, int kind, bool b_mn_major) {
  // A k-major B with at most 16 columns: the skinny case.  A 128 x 16 tile streams the tall operand
  // through 8 stages of 18 KiB per SM, which keeps HBM busy; the MMA work is negligible.
  if (N <= 16 && !b_mn_major) return 16;
  const int64_t tm = (M + BM - 1) / BM;
  const int sms = sm_count();
  const int cand[3] = {256, 128, 64};
  const double eff[3] = {1.0, 0.8, 0.55};
  int best = 256;
  double best_cost = 1e300;
  for (int i = 0; i < 3; ++i) {
    const int bn = cand[i];
    if (kind != KIND_F16 && bn < 128) continue;  // 8-bit MN-major boxes span 128 columns
    const int64_t tiles = tm * ((N + bn - 1) / bn);
    const int64_t waves = (tiles + sms - 1) / sms;
    const double cost = (double)waves * (bn / eff[i] + 24.0);
    if (cost < best_cost) {
      best_cost = cost;
      best = bn;
    }
  }
  return best;
}

// Launch as a programmatic dependent of the preceding kernel (its set-up overlaps that kernel's tail; see the
// griddepcontrol.wait in the kernels).  SKL_B200_TC_OVERLAP=0 turns it off.
bool overlap_launch() {
  static int on = -1;
  if (on < 0) {
    const char *e = getenv("SKL_B200_TC_OVERLAP");
    on = (e && atoi(e) == 0) ? 0 : 1;
  }
  return on != 0;
}

template <int BN, int KIND, bool ACT>
int launch_cfg_act(const CUtensorMap &ta, const CUtensorMap &tb, const CUtensorMap &tbs, const CUtensorMap &tc,
                   const TcParams &p, cudaStream_t s) {
  using Cfg = TcConfig<BN>;
  static bool attr_set[64] = {};  // per device: function attributes do not carry over between devices
  const int dev = current_device();
  if (!attr_set[dev]) {
    cudaError_t e = cudaFuncSetAttribute(gemm_tc_kernel<BN, KIND, ACT>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         Cfg::SMEM_BYTES);
    if (e != cudaSuccess) return (int)e;
    attr_set[dev] = true;
  }
  int grid = p.tiles_m * p.tiles_n;
  if (grid > sm_count()) grid = sm_count();
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3((unsigned)grid);
  cfg.blockDim = dim3(Cfg::THREADS);
  cfg.dynamicSmemBytes = Cfg::SMEM_BYTES;
  cfg.stream = s;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = overlap_launch() ? 1 : 0;
  cudaError_t e = cudaLaunchKernelEx(&cfg, gemm_tc_kernel<BN, KIND, ACT>, ta, tb, tbs, tc, p);
  SKLB_COUNT_LAUNCH();
  if (e != cudaSuccess) return (int)e;
  return (int)cudaGetLastError();
}

// The activation code lives in instantiations of its own so that the plain epilogue carries none of it.
template <int BN, int KIND>
int launch_cfg(const CUtensorMap &ta, const CUtensorMap &tb, const CUtensorMap &tbs, const CUtensorMap &tc,
               const TcParams &p, cudaStream_t s) {
  return p.activation ? launch_cfg_act<BN, KIND, true>(ta, tb, tbs, tc, p, s)
                      : launch_cfg_act<BN, KIND, false>(ta, tb, tbs, tc, p, s);
}

template <int BN, int KIND, bool ACT>
int launch_cfg2_act(const CUtensorMap &ta, const CUtensorMap &tb, const CUtensorMap &tc, const TcParams &p,
                    cudaStream_t s) {
  using Cfg = Tc2Config<BN>;
  static int max_pairs_dev[64];
  static bool pairs_known[64] = {};
  const int dev = current_device();
  int &max_pairs = max_pairs_dev[dev];
  if (!pairs_known[dev]) {
    pairs_known[dev] = true;
    max_pairs = -1;
    cudaError_t e = cudaFuncSetAttribute(gemm_tc2_kernel<BN, KIND, ACT>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         Cfg::SMEM_BYTES);
    if (e != cudaSuccess) return (int)e;
    // how many 2-CTA clusters the device can hold at once (some SMs may have no free neighbour)
    cudaLaunchConfig_t q = {};
    q.gridDim = dim3(2 * sm_count());
    q.blockDim = dim3(NUM_THREADS);
    q.dynamicSmemBytes = Cfg::SMEM_BYTES;
    cudaLaunchAttribute qa[1];
    qa[0].id = cudaLaunchAttributeClusterDimension;
    qa[0].val.clusterDim.x = 2;
    qa[0].val.clusterDim.y = 1;
    qa[0].val.clusterDim.z = 1;
    q.attrs = qa;
    q.numAttrs = 1;
    int n = 0;
    e = cudaOccupancyMaxActiveClusters(&n, gemm_tc2_kernel<BN, KIND, ACT>, &q);
    if (e != cudaSuccess || n <= 0) {
      (void)cudaGetLastError();
      n = sm_count() / 2;
    }
    max_pairs = n;
  }
  int pairs = p.tiles_m * p.tiles_n;
  if (pairs > max_pairs) pairs = max_pairs;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(2 * pairs);
  cfg.blockDim = dim3(NUM_THREADS);
  cfg.dynamicSmemBytes = Cfg::SMEM_BYTES;
  cfg.stream = s;
  cudaLaunchAttribute attr[2];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = 2;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[1].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = overlap_launch() ? 2 : 1;
  cudaError_t e = cudaLaunchKernelEx(&cfg, gemm_tc2_kernel<BN, KIND, ACT>, ta, tb, tc, p);
  SKLB_COUNT_LAUNCH();
  if (e != cudaSuccess) return (int)e;
  return (int)cudaGetLastError();
}

template <int BN, int KIND>
int launch_cfg2(const CUtensorMap &ta, const CUtensorMap &tb, const CUtensorMap &tc, const TcParams &p,
                cudaStream_t s) {
  return p.activation ? launch_cfg2_act<BN, KIND, true>(ta, tb, tc, p, s)
                      : launch_cfg2_act<BN, KIND, false>(ta, tb, tc, p, s);
}

// 0 = never, 1 = when the heuristic says so (default), 2 = whenever the layout allows it
int pair_mode() {
  const char *e = getenv("SKL_B200_TC_PAIR");
  if (!e) return 1;
  return atoi(e);
}

// Is the two-CTA kernel usable / worthwhile for this problem?  Measured on B200 against the one-CTA kernel at
// equal data: it moves a third less data from L2 to the SMs and runs at a higher clock under the power cap;
// the net effect is +2-7 % for int8, +2 % for fp8 and +2-4 % for bf16 on large problems.  It has no tail strips, so it is
// chosen for the 8-bit kinds only and only when its last round of 256 x 256 tiles is nearly full.
bool use_pair_kernel(int kind, int64_t M, int64_t N, const OperandView &vb) {
  const int mode = pair_mode();
  if (mode == 0) return false;
  (void)vb;
  if (mode == 2) return N > 16;
  if (M <= 128) return false;
  const int64_t tiles = ((M + 255) / 256) * ((N + 255) / 256), pairs = sm_count() / 2;
  if (tiles < pairs) return false;
  const int64_t rounds = (tiles + pairs - 1) / pairs;
  // 16-bit operands: the pair wins from about five rounds of tiles on (measured on bf16: +2.3 ... +3.6 % on
  // 16384 x 4096 x {14336, 7168, 3584, 1792}, -1.7 % on 4096^3 with its 3.5 rounds).  The one-CTA kernel's column strips
  // for a short last round do not decide this: a 128-row MMA takes 128 clocks at any width, so strips shorten only
  // the loads and the epilogue (the 1792-column problem measures the same with and without them).
  if (kind == KIND_F16) return rounds >= 5;
  const double fill = (double)tiles / (double)(rounds * pairs);
  return kind == KIND_I8 ? fill >= 0.85 : fill >= 0.95;
}

}  // namespace
}  // namespace sklb

using namespace sklb;

extern "C" int skl_b200_gemm_tc_supported(const skl_b200_gemm_args *g) {
  const int kind = kind_of(g->ta, g->tb);
  if (kind < 0) return 0;
  if (g->epilogue != SKL_EPI_INT && g->epilogue != SKL_EPI_FLOAT) return 0;  // fp16 / fp64 accumulators: CUDA cores
  if (g->m0 >= (1ull << 31) || g->m1 >= (1ull << 31) || g->n0 >= (1ull << 31) || g->n1 >= (1ull << 31) ||
      g->k0 >= (1ull << 31) || g->k1 >= (1ull << 31))
    return 0;
  const int64_t M = (int64_t)(g->m0 * g->m1), N = (int64_t)(g->n0 * g->n1), K = (int64_t)(g->k0 * g->k1);
  if (M < 1 || N < 1 || K < 1) return 0;
  if (M >= (1ll << 31) - 256 || N >= (1ll << 31) - 256 || K >= (1ll << 31) - 256) return 0;
  if (kind == KIND_I8 && K > 65536) return 0;  // keeps |acc| < 2^31 so no wrap-around question arises
  const int es = kind == KIND_F16 ? 2 : 1;
  OperandView va, vb;
  if (!operand_views(g, es, va, vb)) return 0;
  if (g->m1 != 1 || g->n1 != 1) {
    // blocked C: a 32-column chunk of the epilogue must stay inside one block
    if (g->n0 % 32 != 0) return 0;
  }
  if (g->epilogue == SKL_EPI_INT) {
    if (kind != KIND_I8 || g->tc != SKL_DT_I32) return 0;
  } else {
    if (!(g->tc == SKL_DT_F32 || g->tc == SKL_DT_BF16 || g->tc == SKL_DT_F16 || g->tc == SKL_DT_F8E4M3 ||
          g->tc == SKL_DT_I8))
      return 0;
  }
  if (encode_fn() == nullptr) return 0;
  return 1;
}

extern "C" int skl_b200_launch_gemm_tc(const skl_b200_gemm_args *g, uint32_t *dev_status, void *stream) {
  const int kind = kind_of(g->ta, g->tb);
  const int64_t M = (int64_t)(g->m0 * g->m1), N = (int64_t)(g->n0 * g->n1), K = (int64_t)(g->k0 * g->k1);
  const int es = kind == KIND_F16 ? 2 : 1;
  OperandView va, vb;
  if (kind < 0 || !operand_views(g, es, va, vb)) return (int)cudaErrorInvalidValue;
  const bool blocked_c = g->m1 != 1 || g->n1 != 1;
  const bool pair = use_pair_kernel(kind, M, N, vb);
  const int bn = pair ? 256 : pick_bn(M, N, kind, vb.mn_major != 0);
  const int tile_rows = pair ? 2 * BM : BM;

  // Full tiles may be narrower than the kernel's 256 columns when that fills the rounds of the grid better
  // (one-CTA kernel only).  Candidates keep whole 32-column epilogue chunks and, for an MN-major B, whole boxes.
  int bn_main = bn;
  if (!pair && bn == 256) {
    const int step = vb.mn_major ? SLAB_BYTES / es : 32;
    const int64_t tm = (M + BM - 1) / BM;
    const int sms = sm_count();
    static const int forced = [] {
      const char *e = getenv("SKL_B200_TC_BN");  // tuning override
      return e ? atoi(e) : 0;
    }();
    double best = 1e300;
    for (int w = 256; w >= 160; w -= 32) {
      if (w % step != 0) continue;
      const int64_t T = tm * ((N + w - 1) / w);
      const int64_t full = T / sms, rem = T % sms;
      // cost of one tile ~ its width plus a fixed part (pipeline fill, epilogue tail, narrower MMAs being a little
      // less efficient); a short last round is cut into strips (see below), so it costs about a strip
      double cost = (double)full * (w + 28.0);
      if (rem > 0) {
        int split = 1;
        if (T > sms && rem * 2 <= sms && (w / 2) % 32 == 0 && (w / 2) % step == 0) split = 2;
        if (T > sms && rem * 4 <= sms && (w / 4) % 32 == 0 && (w / 4) % step == 0) split = 4;
        cost += (double)w / split + 28.0;
      }
      if (forced ? w == forced : cost < best) {
        best = cost;
        bn_main = w;
        if (forced) break;
      }
    }
  }

  // Tall-skinny problems (the 16-column tile) are a stream of A: when the 128-row tiles make more than one round of
  // the grid, shorten them so that their number fills whole rounds, e.g. 57344 rows = 448 tiles = 3.03 rounds of 148 SMs
  // become 592 tiles of 97 rows = 4 rounds (measured 48.6 -> 42.6 us at 16 columns; 28672 rows 27.1 -> 24.6 us).  A
  // single round gains nothing from it (14336 rows: 15.5 us with 112 tiles of 128 rows, 15.9 us with 148 of 97): there
  // the time is the chain of a tile's 4 K / 128 k blocks, about 0.28 us each on the MMA thread, not the bandwidth.
  int bm_rows = BM;
  if (!pair && bn == 16 && !va.mn_major && !va.panel_form && !blocked_c) {
    static const bool off = [] {
      const char *e = getenv("SKL_B200_TC_SHORT_TILES");  // tuning override
      return e && atoi(e) == 0;
    }();
    const int64_t tm = (M + BM - 1) / BM, tn = (N + bn_main - 1) / bn_main, sms = sm_count();
    const int64_t rounds = (tm * tn + sms - 1) / sms, want_m = rounds * sms / tn;
    if (!off && want_m > tm && tm * tn > sms) {
      const int64_t r = (M + want_m - 1) / want_m;
      if (r >= 32 && r < BM) bm_rows = (int)r;
    }
  }
  CUtensorMap tmA, tmB;
  if (!make_map(&tmA, kind, g->ta, g->a, va, M, K, bm_rows)) return (int)cudaErrorInvalidValue;
  if (!make_map(&tmB, kind, g->tb, g->b, vb, N, K, pair ? bn / 2 : bn_main)) return (int)cudaErrorInvalidValue;

  TcParams p;
  p.M = (int)M;
  p.N = (int)N;
  p.K = (int)K;
  p.tiles_m = (int)((M + (pair ? tile_rows : bm_rows) - 1) / (pair ? tile_rows : bm_rows));
  p.bm_rows = bm_rows;
  p.a_tx = (uint32_t)bm_rows * SLAB_BYTES;
  p.tiles_n = (int)((N + bn_main - 1) / bn_main);
  p.bn_main = bn_main;
  const int bke = SLAB_BYTES / es;
  p.num_kb = (int)((K + bke - 1) / bke);
  p.a_mn = va.mn_major;
  p.b_mn = vb.mn_major;
  // A plain MN-major matrix keeps its 2-D tensor map and box-aligned x (TMA needs x * element size to be a multiple
  // of 16 bytes; a tile that reaches past the last row / column reads the zero fill).  Panelled operands get a 3-D
  // map; panels are whole numbers of boxes (classify_panels), so x stays aligned there too.
  p.a_panel = va.panel_form ? (int)va.panel : PLAIN_PANEL;
  p.b_panel = vb.panel_form ? (int)vb.panel : PLAIN_PANEL;
  p.c_block_m = blocked_c ? (int)g->m0 : 0;
  p.c_block_n = blocked_c ? (int)g->n0 : 0;
  p.rsc1 = g->rsc1;
  p.csc1 = g->csc1;
  const uint32_t cfmt = kind == KIND_I8 ? 2u : 1u;  // S32 : F32 accumulator
  p.idesc = (cfmt << 4) | (fmt_code(kind, g->ta) << 7) | (fmt_code(kind, g->tb) << 10) |
            ((uint32_t)va.mn_major << 15) | ((uint32_t)vb.mn_major << 16) | ((uint32_t)(bn_main >> 3) << 17) |
            ((uint32_t)(tile_rows >> 4) << 24);
  {
    // rasterisation group: keep the A rows of one group near 32 MiB (a quarter of the L2)
    const char *e = getenv("SKL_B200_RASTER_GM");
    int64_t gm = e ? atoi(e) : (32ll << 20) / ((int64_t)tile_rows * K * es);
    if (gm < 1) gm = 1;
    if (gm > p.tiles_m) gm = p.tiles_m;
    p.raster_gm = (int)gm;
  }
  {
    // tail splitting: only the one-CTA kernel with 256-wide tiles; strips must keep whole swizzle atoms
    const int T = p.tiles_m * p.tiles_n, G = T < sm_count() ? T : sm_count();
    p.main_tiles = T;
    p.tail_round = 0;
    p.tail_units = 0;
    p.tail_split = 1;
    const int rem = T % G;
    const char *e = getenv("SKL_B200_TC_TAIL_SPLIT");
    const bool enabled = !(e && atoi(e) == 0);
    if (enabled && !pair && bn == 256 && T > G && rem > 0 && rem * 2 <= G) {
      const int atom_cols = vb.mn_major ? SLAB_BYTES / es : 32;  // columns per MN-major box; else the epilogue chunk
      int split = 1;
      if ((bn_main / 2) % 32 == 0 && (bn_main / 2) % atom_cols == 0) split = 2;
      if (rem * 4 <= G && (bn_main / 4) % 32 == 0 && (bn_main / 4) % atom_cols == 0) split = 4;
      if (split > 1) {
        p.main_tiles = T - rem;
        p.tail_round = p.main_tiles / G;
        p.tail_split = split;
        p.tail_units = rem * split;
      }
    }
    p.idesc_tail = (p.idesc & ~(0x3Fu << 17)) | ((uint32_t)((bn_main / p.tail_split) >> 3) << 17);
    const int strip_cols = bn_main / p.tail_split, per_atom = SLAB_BYTES / es;
    p.tail_b_atoms = (strip_cols + per_atom - 1) / per_atom;
    p.tail_b_bytes = vb.mn_major ? (uint32_t)p.tail_b_atoms * (uint32_t)(per_atom * SLAB_BYTES)
                                 : (uint32_t)strip_cols * SLAB_BYTES;
    p.main_b_atoms = (bn_main + per_atom - 1) / per_atom;
    p.main_b_bytes = vb.mn_major ? (uint32_t)p.main_b_atoms * (uint32_t)(per_atom * SLAB_BYTES)
                                 : (uint32_t)bn_main * SLAB_BYTES;
  }
  CUtensorMap tmBs = tmB;  // the strips' own box of B (k-major B only; MN-major strips load fewer boxes of tmB)
  if (p.tail_split > 1 && !vb.mn_major && !make_map(&tmBs, kind, g->tb, g->b, vb, N, K, bn_main / p.tail_split))
    return (int)cudaErrorInvalidValue;
  p.c = g->c;
  p.rsc = g->rsc0;
  p.csc = g->csc0;
  p.tc = g->tc;
  p.epilogue = g->epilogue;
  const int cs = dtype_size(g->tc);
  p.c_vec_ok = (g->csc0 == 1 && (reinterpret_cast<uintptr_t>(g->c) & 15u) == 0 &&
                (M <= 1 || ((g->rsc0 * cs) & 15) == 0) &&
                (!blocked_c || (((g->rsc1 * cs) & 15) == 0 && ((g->csc1 * cs) & 15) == 0)))
                   ? 1
                   : 0;
  // Results leave through TMA stores when C is a plain row-major matrix with 16-byte-aligned rows; any other C
  // (column-major, strided columns, unaligned) is written with direct stores.  SKL_B200_TC_TMA_STORE=0 disables.
  CUtensorMap tmC = tmA;  // a valid map in either case; unused unless c_tma
  p.c_tma = 0;
  {
    const char *e = getenv("SKL_B200_TC_TMA_STORE");
    // The row length must be a whole number of 16-byte units: a store box that crosses the matrix edge inside
    // such a unit was observed to write the unit's remaining bytes.
    if (!blocked_c && bm_rows == BM && p.c_vec_ok && (N * cs) % 16 == 0 && !(e && atoi(e) == 0) &&
        make_c_map(&tmC, g->c, M, N, g->rsc0, cs))
      p.c_tma = 1;
  }
  p.alpha_i = g->alpha_i;
  p.beta_i = g->beta_i;
  p.alpha_f = g->alpha_f;
  p.beta_f = g->beta_f;
  p.row_scale = g->row_scale;
  p.col_scale = g->col_scale;
  p.col_scale_first = g->col_scale_first;
  p.bias = g->bias;
  p.bias_per_row = g->bias_per_row;
  p.global_max = g->global_max;
  p.activation = g->activation;
  p.act_param = g->act_param;
  p.status = dev_status;
  p.wait_ns = (uint64_t)(g->wait_limit_ms ? g->wait_limit_ms : 2000u) * 1000000ull;
  p.skip_loads = g->debug_skip_loads;
  cudaStream_t s = (cudaStream_t)stream;

  if (pair) {
    switch (kind) {
      case KIND_F16: return launch_cfg2<256, KIND_F16>(tmA, tmB, tmC, p, s);
      case KIND_F8: return launch_cfg2<256, KIND_F8>(tmA, tmB, tmC, p, s);
      default: return launch_cfg2<256, KIND_I8>(tmA, tmB, tmC, p, s);
    }
  }
#define TC_DISPATCH(BNV)                                                      \
  switch (kind) {                                                             \
    case KIND_F16: return launch_cfg<BNV, KIND_F16>(tmA, tmB, tmBs, tmC, p, s);          \
    case KIND_F8: return launch_cfg<BNV, KIND_F8>(tmA, tmB, tmBs, tmC, p, s);            \
    default: return launch_cfg<BNV, KIND_I8>(tmA, tmB, tmBs, tmC, p, s);                 \
  }
  if (bn == 256) {
    TC_DISPATCH(256)
  } else if (bn == 128) {
    TC_DISPATCH(128)
  } else if (bn == 16) {
    TC_DISPATCH(16)
  } else {
    return launch_cfg<64, KIND_F16>(tmA, tmB, tmBs, tmC, p, s);
  }
#undef TC_DISPATCH
}

// ---- MX-FP4 on the block-scaled MMA: 16-byte aligned packed rows, k a positive multiple of 32
extern "C" int skl_b200_gemm_mxf4_supported(const void *a, int64_t rsa, const void *b, int64_t csb, int64_t m, int64_t n,
                                            int64_t k) {
  if (m < 1 || n < 1 || k < 32 || (k & 31) != 0) return 0;
  if (m >= (1ll << 31) - 256 || n >= (1ll << 31) - 256 || k >= (1ll << 31)) return 0;
  if ((reinterpret_cast<uintptr_t>(a) & 15u) || (reinterpret_cast<uintptr_t>(b) & 15u)) return 0;
  if ((m > 1 && (rsa & 15)) || (n > 1 && (csb & 15))) return 0;
  return encode_fn() != nullptr;
}

extern "C" size_t skl_b200_gemm_mxf4_scale_bytes(int64_t rows, int64_t k) {
  return (size_t)(2 * ((rows + 255) / 256)) * (size_t)((k + 255) / 256) * mx::SF_BYTES;  // row tiles of 128, an even number
}

// ws_sa / ws_sb: device buffers of skl_b200_gemm_mxf4_scale_bytes(m, k) / (n, k) bytes for the re-laid scales
extern "C" int skl_b200_launch_gemm_mxf4(const void *a, int64_t rsa, const void *sa, int64_t rssa, const void *b,
                                         int64_t csb, const void *sb, int64_t cssb, float *c, int64_t rsc, int64_t m,
                                         int64_t n, int64_t k, float alpha, float beta, void *ws_sa, void *ws_sb,
                                         uint32_t wait_limit_ms, uint32_t *dev_status, void *stream) {
  EncodeTiledFn enc = encode_fn();
  if (!enc) return (int)cudaErrorNotSupported;
  CUtensorMap tmA, tmB;
  cuuint32_t box[2] = {(cuuint32_t)mx::STAGE_K_BYTES, 0}, estr[2] = {1, 1};
  for (int which = 0; which < 2; ++which) {
    const cuuint64_t rows = (cuuint64_t)(which ? n : m);
    box[1] = (cuuint32_t)(which ? mx::BN : mx::BM);
    cuuint64_t dims[2] = {(cuuint64_t)(k / 2), rows}, strides[1];
    int64_t ld = which ? csb : rsa;
    if (rows <= 1) ld = (k / 2 + 15) / 16 * 16;  // stride unused; keep it legal
    strides[0] = (cuuint64_t)ld;
    if (enc(which ? &tmB : &tmA, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<void *>(which ? b : a), dims, strides, box,
            estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
            CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS)
      return (int)cudaErrorInvalidValue;
  }
  const int kblocks = (int)(k / 32), chunks = 2 * ((kblocks + 7) / 8);
  {
    const int64_t total_a = ((m + mx::BM - 1) / mx::BM) * chunks * 128, total_b = 2 * ((n + mx::BN - 1) / mx::BN) * chunks * 128;
    int64_t grid = (total_a + total_b + 255) / 256;
    if (grid > 8 * sm_count()) grid = 8 * sm_count();
    mx::mx_pack_scales_kernel<<<(unsigned)grid, 256, 0, (cudaStream_t)stream>>>(
        (uint32_t *)ws_sa, (const uint8_t *)sa, rssa, (int)m, total_a, (uint32_t *)ws_sb, (const uint8_t *)sb, cssb, (int)n,
        total_b, kblocks, chunks);
    SKLB_COUNT_LAUNCH();
  }
  mx::Params p;
  p.psa = (const uint8_t *)ws_sa;
  p.psb = (const uint8_t *)ws_sb;
  p.c = c;
  p.rsc = rsc;
  p.M = (int)m;
  p.N = (int)n;
  p.kblocks = kblocks;
  p.tiles_m = (int)((m + mx::BM - 1) / mx::BM);
  p.tiles_n = (int)((n + mx::BN - 1) / mx::BN);
  p.alpha = alpha;
  p.beta = beta;
  p.wait_ns = (uint64_t)(wait_limit_ms ? wait_limit_ms : 2000u) * 1000000ull;
  p.status = dev_status;
  p.c_vec = ((reinterpret_cast<uintptr_t>(c) & 15u) == 0 && (m <= 1 || (rsc & 3) == 0)) ? 1 : 0;
  static bool attr_set[64] = {};
  const int dev = current_device();
  if (!attr_set[dev]) {
    cudaError_t e = cudaFuncSetAttribute(mx::gemm_mxf4_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, mx::SMEM_BYTES);
    if (e != cudaSuccess) return (int)e;
    attr_set[dev] = true;
  }
  int64_t grid = (int64_t)p.tiles_m * p.tiles_n;
  if (grid > sm_count()) grid = sm_count();
  mx::gemm_mxf4_kernel<<<(unsigned)grid, mx::THREADS, mx::SMEM_BYTES, (cudaStream_t)stream>>>(tmA, tmB, p);
  SKLB_COUNT_LAUNCH();
  return (int)cudaGetLastError();
}
