// pack.cu -- pack / unpack / transpose as one tiled re-layout kernel.
//
// All three SKL operations are "copy element (i, j) of a strided source to a strided destination"
// where either side may be a blocked 4-D layout (ref/pack/pack_e8rc_e8rcprc.c:10-35,
// unpack_e8rcprc_e8rc.c:10-37, transpose_e8.c:11-19):
//     pack       plain source  -> blocked destination, positions outside m x n receive `pad`
//     unpack     blocked source -> plain destination, only the m x n real elements are written
//     transpose  plain source  -> plain destination with row/column strides exchanged
// The kernel walks 64 x 64 tiles of the logical (i, j) index space.  Each tile is read with the
// thread index running along the source's unit-stride direction, parked in shared memory, and
// written with the thread index running along the destination's unit-stride direction, so both
// sides are coalesced even when the two directions differ (the transposing cases).  Along the
// unit-stride direction a thread moves 4 bytes at a time (4 / 2 / 1 elements) whenever the layout
// keeps such a group contiguous and aligned; otherwise it falls back to single elements.  Only
// addressed destination elements are written.  Algorithmic bytes: 2 x elements x element size
// (+ padding written by pack).
#include "numerics.cuh"

namespace sklb {
namespace {

constexpr int RT = 64;  // tile edge

struct Side {
  int64_t rs0, cs0, rs1, cs1;
  uint32_t b0r, b0c;  // block extents (rows, cols); unused when plain
  int plain;          // 1: offset = i*rs0 + j*cs0
  int fast_j;         // 1: the unit stride runs along j
  int vec_ok;         // groups of 4 bytes along the unit-stride direction are contiguous and aligned
};

__device__ __forceinline__ int64_t side_off(const Side &s, uint32_t i, uint32_t j) {
  if (s.plain) return (int64_t)i * s.rs0 + (int64_t)j * s.cs0;
  const uint32_t bi = i / s.b0r, bj = j / s.b0c;
  return (int64_t)bi * s.rs1 + (int64_t)(i - bi * s.b0r) * s.rs0 + (int64_t)bj * s.cs1 +
         (int64_t)(j - bj * s.b0c) * s.cs0;
}

struct RelayoutParams {
  uint32_t MI, NJ;  // logical extent walked (padded extent for pack, real extent otherwise)
  uint32_t m, n;    // extent for which the source holds data
  Side src, dst;
  uint32_t pad;
  uint32_t tiles_i, tiles_j;
};

template <typename T>
__global__ void __launch_bounds__(256) relayout_kernel(const T *__restrict__ src, T *__restrict__ dst,
                                                       const RelayoutParams p) {
  constexpr int VEC = 4 / sizeof(T);   // elements per 4-byte group
  constexpr int GROUPS = RT / VEC;     // groups along the fast direction of a tile
  __shared__ T tile[RT][RT + 4 / sizeof(T)];
  const uint32_t num_tiles = p.tiles_i * p.tiles_j;
  for (uint32_t t = blockIdx.x; t < num_tiles; t += gridDim.x) {
    const uint32_t i0 = (t / p.tiles_j) * RT, j0 = (t % p.tiles_j) * RT;

    // ---- read phase: thread index along the source's unit stride
    for (int e = threadIdx.x; e < RT * GROUPS; e += 256) {
      const int grp = e % GROUPS, slow = e / GROUPS;
      const int f0 = grp * VEC;
      const int ti = p.src.fast_j ? slow : f0, tj = p.src.fast_j ? f0 : slow;
      const uint32_t i = i0 + ti, j = j0 + tj;
      const uint32_t lim_fast = p.src.fast_j ? p.n : p.m;
      const uint32_t pos_fast = p.src.fast_j ? j : i;
      const bool slow_in = p.src.fast_j ? (i < p.m) : (j < p.n);
      T v[VEC];
      if (VEC > 1 && p.src.vec_ok && slow_in && pos_fast + VEC <= lim_fast) {
        const uint32_t w = *reinterpret_cast<const uint32_t *>(src + side_off(p.src, i, j));
#pragma unroll
        for (int q = 0; q < VEC; ++q) v[q] = (T)(w >> (8 * sizeof(T) * q));
      } else {
#pragma unroll
        for (int q = 0; q < VEC; ++q) {
          const uint32_t ii = p.src.fast_j ? i : i + q, jj = p.src.fast_j ? j + q : j;
          v[q] = (ii < p.m && jj < p.n) ? src[side_off(p.src, ii, jj)] : (T)p.pad;
        }
      }
#pragma unroll
      for (int q = 0; q < VEC; ++q) {
        if (p.src.fast_j)
          tile[ti][tj + q] = v[q];
        else
          tile[ti + q][tj] = v[q];
      }
    }
    __syncthreads();

    // ---- write phase: thread index along the destination's unit stride
    for (int e = threadIdx.x; e < RT * GROUPS; e += 256) {
      const int grp = e % GROUPS, slow = e / GROUPS;
      const int f0 = grp * VEC;
      const int ti = p.dst.fast_j ? slow : f0, tj = p.dst.fast_j ? f0 : slow;
      const uint32_t i = i0 + ti, j = j0 + tj;
      const uint32_t lim_fast = p.dst.fast_j ? p.NJ : p.MI;
      const uint32_t pos_fast = p.dst.fast_j ? j : i;
      const bool slow_in = p.dst.fast_j ? (i < p.MI) : (j < p.NJ);
      if (!slow_in || pos_fast >= lim_fast) continue;
      T v[VEC];
#pragma unroll
      for (int q = 0; q < VEC; ++q) v[q] = p.dst.fast_j ? tile[ti][tj + q] : tile[ti + q][tj];
      if (VEC > 1 && p.dst.vec_ok && pos_fast + VEC <= lim_fast) {
        uint32_t w = 0;
#pragma unroll
        for (int q = 0; q < VEC; ++q) w |= (uint32_t)v[q] << (8 * sizeof(T) * q);
        *reinterpret_cast<uint32_t *>(dst + side_off(p.dst, i, j)) = w;
      } else {
#pragma unroll
        for (int q = 0; q < VEC; ++q) {
          const uint32_t ii = p.dst.fast_j ? i : i + q, jj = p.dst.fast_j ? j + q : j;
          if (ii < p.MI && jj < p.NJ) dst[side_off(p.dst, ii, jj)] = v[q];
        }
      }
    }
    __syncthreads();
  }
}

// ---- fast path 1: no change of direction (source and destination share the unit-stride direction).
// No shared memory: each thread moves one 16-byte group along the unit-stride direction, so a warp
// reads and writes 512 contiguous bytes per row.  Requires 16-byte aligned groups on both sides (base,
// other strides, block extents along the unit-stride direction all multiples of the group).
template <typename T>
__global__ void __launch_bounds__(256) copy_groups_kernel(const T *__restrict__ src, T *__restrict__ dst,
                                                          const RelayoutParams p) {
  constexpr uint32_t G = 16 / sizeof(T);  // elements per group
  const bool fj = p.src.fast_j != 0;
  const uint32_t fast_ext = fj ? p.NJ : p.MI, slow_ext = fj ? p.MI : p.NJ;
  const uint32_t fast_src = fj ? p.n : p.m, slow_src = fj ? p.m : p.n;
  const uint32_t groups = (fast_ext + G - 1) / G;
  const uint64_t total = (uint64_t)groups * slow_ext;
  for (uint64_t e = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x; e < total; e += (uint64_t)gridDim.x * blockDim.x) {
    const uint32_t slow = (uint32_t)(e / groups), f0 = (uint32_t)(e - (uint64_t)slow * groups) * G;
    const uint32_t i = fj ? slow : f0, j = fj ? f0 : slow;
    T *d = dst + side_off(p.dst, i, j);
    if (slow < slow_src && f0 + G <= fast_src && f0 + G <= fast_ext) {
      *reinterpret_cast<uint4 *>(d) = __ldg(reinterpret_cast<const uint4 *>(src + side_off(p.src, i, j)));
    } else {
      // group touches the padding region or the ragged edge: element by element
      for (uint32_t q = 0; q < G && f0 + q < fast_ext; ++q) {
        const uint32_t ii = fj ? i : i + q, jj = fj ? j + q : j;
        const T v = (ii < p.m && jj < p.n) ? src[side_off(p.src, ii, jj)] : (T)p.pad;
        dst[side_off(p.dst, ii, jj)] = v;
      }
    }
  }
}

// ---- fast path 2: plain 2-D transpose (source unit stride along j, destination along i).
// Each thread owns V x V micro-tiles with V = 4 / sizeof(T) (4 x 4 bytes, 2 x 2 halfwords, 1 word):
// V loads of 4 bytes along the source rows, an in-register V x V transpose with byte permutes, V
// stores of 4 bytes into a transposed shared-memory tile; then every thread writes 16-byte runs of the
// destination rows.  Both global sides move whole 32-byte sectors.  The tile is TD x TD elements
// (16 KB for bytes and words, 32 KB for halfwords) so that a resident CTA keeps enough bytes in flight
// to cover the memory latency; a warp covers (32 / V) x V micro-tiles on the way in and 4 rows x 8 runs
// on the way out, which with the odd row pitch touches 32 distinct banks both times.
template <typename T, int TD>
__global__ void __launch_bounds__(256) transpose_fast_kernel(const T *__restrict__ src, T *__restrict__ dst,
                                                             const RelayoutParams p) {
  constexpr int V = 4 / sizeof(T);
  constexpr int WPR = TD / V;                  // 4-byte words per tile row
  constexpr int PITCHW = WPR + 1;              // odd pitch in words
  constexpr int TXW = 32 / V, TYW = V;         // micro-tiles one warp covers along j and along i
  constexpr int WX = WPR / TXW;                // warp steps across a tile
  constexpr int RUNS = TD * (int)sizeof(T) / 16;  // 16-byte runs per destination row
  __shared__ uint32_t tileT[TD * PITCHW];      // [j][i / V]
  const uint32_t tiles_i = (p.m + TD - 1) / TD, tiles_j = (p.n + TD - 1) / TD;
  const uint32_t num_tiles = tiles_i * tiles_j;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  for (uint32_t t = blockIdx.x; t < num_tiles; t += gridDim.x) {
    const uint32_t i0 = (t / tiles_j) * TD, j0 = (t % tiles_j) * TD;
    const bool full = i0 + TD <= p.m && j0 + TD <= p.n;
    if (full) {
#pragma unroll 4
      for (int w = warp; w < WX * (WPR / TYW); w += 8) {
        const int tx = (w % WX) * TXW + lane % TXW;  // micro-tile column (along j)
        const int ty = (w / WX) * TYW + lane / TXW;  // micro-tile row (along i)
        uint32_t r[4];
#pragma unroll
        for (int q = 0; q < V; ++q)
          r[q] = __ldg(reinterpret_cast<const uint32_t *>(src + (int64_t)(i0 + V * ty + q) * p.src.rs0 + j0 + V * tx));
        uint32_t *col = &tileT[(V * tx) * PITCHW + ty];
        if (V == 4) {
          // r[q] byte b = element (row q, col b); the word stored for column b holds byte q = the same element
          const uint32_t a0 = __byte_perm(r[0], r[1], 0x5140), a1 = __byte_perm(r[0], r[1], 0x7362);
          const uint32_t b0 = __byte_perm(r[2], r[3], 0x5140), b1 = __byte_perm(r[2], r[3], 0x7362);
          col[0] = __byte_perm(a0, b0, 0x5410);
          col[(V > 1) * PITCHW] = __byte_perm(a0, b0, 0x7632);
          col[(V > 2) * 2 * PITCHW] = __byte_perm(a1, b1, 0x5410);
          col[(V > 2) * 3 * PITCHW] = __byte_perm(a1, b1, 0x7632);
        } else if (V == 2) {
          col[0] = __byte_perm(r[0], r[1], 0x5410);  // (row 0, col 0), (row 1, col 0)
          col[(V > 1) * PITCHW] = __byte_perm(r[0], r[1], 0x7632);
        } else {
          col[0] = r[0];
        }
      }
      __syncthreads();
      for (int w = warp; w < (RUNS / 8) * (TD / 4); w += 8) {
        const int run = (w % (RUNS / 8)) * 8 + lane % 8;
        const int row = (w / (RUNS / 8)) * 4 + lane / 8;
        const uint32_t *rp = &tileT[row * PITCHW + 4 * run];
        const uint4 v = make_uint4(rp[0], rp[1], rp[2], rp[3]);
        *reinterpret_cast<uint4 *>(reinterpret_cast<uint8_t *>(dst + (int64_t)(j0 + row) * p.dst.cs0 + i0) + 16 * run) = v;
      }
      __syncthreads();
    } else {
      // ragged edge tile: element by element, still coalesced along each side's unit stride
      T *tb = reinterpret_cast<T *>(tileT);  // viewed as [j][i] elements
      constexpr int PITCH = PITCHW * V;
      for (int e = threadIdx.x; e < TD * TD; e += 256) {
        const int tj = e % TD, ti = e / TD;
        const uint32_t i = i0 + ti, j = j0 + tj;
        if (i < p.m && j < p.n) tb[tj * PITCH + ti] = src[(int64_t)i * p.src.rs0 + j];
      }
      __syncthreads();
      for (int e = threadIdx.x; e < TD * TD; e += 256) {
        const int ti = e % TD, tj = e / TD;
        const uint32_t i = i0 + ti, j = j0 + tj;
        if (i < p.m && j < p.n) dst[(int64_t)j * p.dst.cs0 + i] = tb[tj * PITCH + ti];
      }
      __syncthreads();
    }
  }
}

int relayout_grid(uint64_t tiles) {
  static int sms = 0;
  if (sms == 0) {
    int dev = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    if (sms <= 0) sms = 148;
  }
  const uint64_t cap = (uint64_t)sms * 8;  // 8 resident CTAs of 256 threads per SM
  return (int)(tiles < cap ? tiles : cap);
}

// Can 4-byte groups along the unit-stride direction be moved as one word?  Needs a true unit stride,
// every other stride and the base a multiple of the group, and blocks that do not split a group.
void finish_side(Side &s, const void *base, size_t esize) {
  const int64_t vec = 4 / (int64_t)esize;
  const int64_t unit = s.fast_j ? s.cs0 : s.rs0;
  const int64_t other0 = s.fast_j ? s.rs0 : s.cs0;
  bool ok = vec > 1 && unit == 1 && (reinterpret_cast<uintptr_t>(base) & 3u) == 0 && other0 % vec == 0;
  if (ok && !s.plain) {
    const uint32_t bfast = s.fast_j ? s.b0c : s.b0r;
    ok = bfast % vec == 0 && s.rs1 % vec == 0 && s.cs1 % vec == 0;
  }
  s.vec_ok = ok ? 1 : 0;
}

// 16-byte groups along the unit-stride direction: contiguous, aligned, never split by a block edge.
bool groups16_ok(const Side &s, const void *base, size_t esize) {
  const int64_t vec = 16 / (int64_t)esize;
  const int64_t unit = s.fast_j ? s.cs0 : s.rs0;
  const int64_t other0 = s.fast_j ? s.rs0 : s.cs0;
  if (unit != 1 || (reinterpret_cast<uintptr_t>(base) & 15u) != 0 || other0 % vec != 0) return false;
  if (!s.plain) {
    const uint32_t bfast = s.fast_j ? s.b0c : s.b0r;
    if (bfast % vec != 0 || s.rs1 % vec != 0 || s.cs1 % vec != 0) return false;
  }
  return true;
}

int launch_relayout(size_t esize, const void *src, void *dst, RelayoutParams p, cudaStream_t s) {
  if (p.MI == 0 || p.NJ == 0) return 0;
  finish_side(p.src, src, esize);
  finish_side(p.dst, dst, esize);
  p.tiles_i = (p.MI + RT - 1) / RT;
  p.tiles_j = (p.NJ + RT - 1) / RT;
  const int grid = relayout_grid((uint64_t)p.tiles_i * p.tiles_j);
  if (p.src.fast_j == p.dst.fast_j && groups16_ok(p.src, src, esize) && groups16_ok(p.dst, dst, esize)) {
    const uint64_t fast_ext = p.src.fast_j ? p.NJ : p.MI, slow_ext = p.src.fast_j ? p.MI : p.NJ;
    const uint64_t total = ((fast_ext * esize + 15) / 16) * slow_ext;
    const int g = relayout_grid((total + 255) / 256);
    switch (esize) {
      case 1:
        copy_groups_kernel<uint8_t><<<g, 256, 0, s>>>((const uint8_t *)src, (uint8_t *)dst, p);
        break;
      case 2:
        copy_groups_kernel<uint16_t><<<g, 256, 0, s>>>((const uint16_t *)src, (uint16_t *)dst, p);
        break;
      default:
        copy_groups_kernel<uint32_t><<<g, 256, 0, s>>>((const uint32_t *)src, (uint32_t *)dst, p);
        break;
    }
    SKLB_COUNT_LAUNCH();
    return (int)cudaGetLastError();
  }
  const int64_t v4 = 4 / (int64_t)esize, v16 = 16 / (int64_t)esize;
  if (p.src.plain && p.dst.plain && p.src.fast_j && !p.dst.fast_j && p.src.cs0 == 1 && p.dst.rs0 == 1 &&
      p.MI == p.m && p.NJ == p.n && (reinterpret_cast<uintptr_t>(src) & 3u) == 0 && p.src.rs0 % v4 == 0 &&
      (reinterpret_cast<uintptr_t>(dst) & 15u) == 0 && p.dst.cs0 % v16 == 0) {
    // One wave of resident CTAs: the halfword kernel's 32 KB tile fits fewer than 8 per SM, and CTAs left
    // for a second wave would run it at a fraction of the occupancy.
    static int resident[3] = {0, 0, 0};
    const int which = esize == 1 ? 0 : esize == 2 ? 1 : 2;
    if (resident[which] == 0) {
      int per_sm = 0;
      cudaError_t qe =
          which == 0   ? cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, transpose_fast_kernel<uint8_t, 128>, 256, 0)
          : which == 1 ? cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, transpose_fast_kernel<uint16_t, 128>, 256, 0)
                       : cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, transpose_fast_kernel<uint32_t, 64>, 256, 0);
      if (qe != cudaSuccess) (void)cudaGetLastError();
      resident[which] = (qe == cudaSuccess && per_sm > 0) ? (per_sm < 8 ? per_sm : 8) : 4;
    }
    const uint64_t td = esize == 4 ? 64 : 128;
    const uint64_t tiles = ((p.m + td - 1) / td) * ((p.n + td - 1) / td);
    const uint64_t cap = (uint64_t)relayout_grid(~0ull) / 8 * (uint64_t)resident[which];
    const int tg = (int)(tiles < cap ? tiles : cap);
    switch (esize) {
      case 1:
        transpose_fast_kernel<uint8_t, 128><<<tg, 256, 0, s>>>((const uint8_t *)src, (uint8_t *)dst, p);
        break;
      case 2:
        transpose_fast_kernel<uint16_t, 128><<<tg, 256, 0, s>>>((const uint16_t *)src, (uint16_t *)dst, p);
        break;
      default:
        transpose_fast_kernel<uint32_t, 64><<<tg, 256, 0, s>>>((const uint32_t *)src, (uint32_t *)dst, p);
        break;
    }
    SKLB_COUNT_LAUNCH();
    return (int)cudaGetLastError();
  }
  switch (esize) {
    case 1:
      relayout_kernel<uint8_t><<<grid, 256, 0, s>>>((const uint8_t *)src, (uint8_t *)dst, p);
      break;
    case 2:
      relayout_kernel<uint16_t><<<grid, 256, 0, s>>>((const uint16_t *)src, (uint16_t *)dst, p);
      break;
    default:
      relayout_kernel<uint32_t><<<grid, 256, 0, s>>>((const uint32_t *)src, (uint32_t *)dst, p);
      break;
  }
  SKLB_COUNT_LAUNCH();
  return (int)cudaGetLastError();
}

Side plain_side(size_t rs, size_t cs) {
  Side s{};
  s.rs0 = (int64_t)rs;
  s.cs0 = (int64_t)cs;
  s.plain = 1;
  s.fast_j = (cs == 1 || rs != 1) ? 1 : 0;
  return s;
}

Side blocked_side(size_t m0, size_t n0, size_t rs0, size_t cs0, size_t rs1, size_t cs1) {
  Side s{};
  s.rs0 = (int64_t)rs0;
  s.cs0 = (int64_t)cs0;
  s.rs1 = (int64_t)rs1;
  s.cs1 = (int64_t)cs1;
  s.b0r = (uint32_t)m0;
  s.b0c = (uint32_t)n0;
  s.plain = 0;
  s.fast_j = (cs0 == 1 || rs0 != 1) ? 1 : 0;
  return s;
}

// extents are walked with 32-bit indices
bool fits(size_t a, size_t b) { return a < (1ull << 31) && b < (1ull << 31); }

}  // namespace
}  // namespace sklb

using namespace sklb;

extern "C" int skl_b200_launch_pack(size_t esize, size_t m, size_t n, const void *src, size_t rs,
                                    size_t cs, size_t m0, size_t n0, void *dst, size_t rs0,
                                    size_t cs0, size_t rs1, size_t cs1, uint32_t pad, void *stream) {
  if (m0 == 0 || n0 == 0) return 0;
  const size_t m1 = (m + m0 - 1) / m0, n1 = (n + n0 - 1) / n0;
  if (!fits(m1 * m0, n1 * n0) || !fits(m0, n0)) return (int)cudaErrorInvalidValue;
  RelayoutParams p{};
  p.MI = (uint32_t)(m1 * m0);
  p.NJ = (uint32_t)(n1 * n0);
  p.m = (uint32_t)m;
  p.n = (uint32_t)n;
  p.src = plain_side(rs, cs);
  p.dst = blocked_side(m0, n0, rs0, cs0, rs1, cs1);
  p.pad = pad;
  return launch_relayout(esize, src, dst, p, (cudaStream_t)stream);
}

extern "C" int skl_b200_launch_unpack(size_t esize, size_t m0, size_t n0, const void *src, size_t rs0,
                                      size_t cs0, size_t rs1, size_t cs1, size_t m, size_t n,
                                      void *dst, size_t rs, size_t cs, void *stream) {
  if (m0 == 0 || n0 == 0) return 0;
  if (!fits(m, n) || !fits(m0, n0)) return (int)cudaErrorInvalidValue;
  RelayoutParams p{};
  p.MI = (uint32_t)m;
  p.NJ = (uint32_t)n;
  p.m = (uint32_t)m;
  p.n = (uint32_t)n;
  p.src = blocked_side(m0, n0, rs0, cs0, rs1, cs1);
  p.dst = plain_side(rs, cs);
  p.pad = 0;
  return launch_relayout(esize, src, dst, p, (cudaStream_t)stream);
}

extern "C" int skl_b200_launch_transpose(size_t esize, size_t m, size_t n, const void *a, size_t rsa,
                                         void *at, size_t rsat, void *stream) {
  if (!fits(m, n)) return (int)cudaErrorInvalidValue;
  RelayoutParams p{};
  p.MI = (uint32_t)m;
  p.NJ = (uint32_t)n;
  p.m = (uint32_t)m;
  p.n = (uint32_t)n;
  p.src = plain_side(rsa, 1);
  p.src.fast_j = 1;
  p.dst = plain_side(1, rsat);  // at[j*rsat + i]
  p.dst.fast_j = 0;
  p.pad = 0;
  return launch_relayout(esize, a, at, p, (cudaStream_t)stream);
}
