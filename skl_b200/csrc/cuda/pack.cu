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
// sides are coalesced even when the two directions differ (the transposing cases).  Only addressed
// destination elements are written.  Algorithmic bytes: 2 x elements x element size (+ padding).
#include "numerics.cuh"

namespace sklb {
namespace {

constexpr int RT = 64;  // tile edge

struct Side {
  int64_t b0r, b0c;  // block extents (rows, cols); plain layout: the whole extent (>= 1)
  int64_t rs0, cs0, rs1, cs1;
};

__device__ __forceinline__ int64_t side_off(const Side &s, int64_t i, int64_t j) {
  return (i / s.b0r) * s.rs1 + (i % s.b0r) * s.rs0 + (j / s.b0c) * s.cs1 + (j % s.b0c) * s.cs0;
}

struct RelayoutParams {
  int64_t MI, NJ;  // logical extent walked (padded extent for pack, real extent otherwise)
  int64_t m, n;    // extent for which the source holds data
  Side src, dst;
  uint32_t pad;
  int src_fast_j;  // 1: source unit stride runs along j
  int dst_fast_j;
  int64_t tiles_j;
};

template <typename T>
__global__ void __launch_bounds__(256) relayout_kernel(const T *__restrict__ src, T *__restrict__ dst,
                                                       const RelayoutParams p) {
  __shared__ T tile[RT][RT + 4 / sizeof(T)];
  for (int64_t t = blockIdx.x; t < p.tiles_j * ((p.MI + RT - 1) / RT); t += gridDim.x) {
    const int64_t i0 = (t / p.tiles_j) * RT, j0 = (t % p.tiles_j) * RT;
    for (int e = threadIdx.x; e < RT * RT; e += 256) {
      int fast = e & (RT - 1), slow = e >> 6;
      int ti = p.src_fast_j ? slow : fast, tj = p.src_fast_j ? fast : slow;
      int64_t i = i0 + ti, j = j0 + tj;
      T v = (T)p.pad;
      if (i < p.m && j < p.n) v = src[side_off(p.src, i, j)];
      tile[ti][tj] = v;
    }
    __syncthreads();
    for (int e = threadIdx.x; e < RT * RT; e += 256) {
      int fast = e & (RT - 1), slow = e >> 6;
      int ti = p.dst_fast_j ? slow : fast, tj = p.dst_fast_j ? fast : slow;
      int64_t i = i0 + ti, j = j0 + tj;
      if (i < p.MI && j < p.NJ) dst[side_off(p.dst, i, j)] = tile[ti][tj];
    }
    __syncthreads();
  }
}

int launch_relayout(size_t esize, const void *src, void *dst, RelayoutParams p, cudaStream_t s) {
  if (p.MI <= 0 || p.NJ <= 0) return 0;
  p.tiles_j = (p.NJ + RT - 1) / RT;
  int64_t tiles = p.tiles_j * ((p.MI + RT - 1) / RT);
  int64_t grid = tiles < (int64_t)148 * 16 ? tiles : (int64_t)148 * 16;
  switch (esize) {
    case 1:
      relayout_kernel<uint8_t><<<(unsigned)grid, 256, 0, s>>>((const uint8_t *)src, (uint8_t *)dst, p);
      break;
    case 2:
      relayout_kernel<uint16_t><<<(unsigned)grid, 256, 0, s>>>((const uint16_t *)src, (uint16_t *)dst, p);
      break;
    default:
      relayout_kernel<uint32_t><<<(unsigned)grid, 256, 0, s>>>((const uint32_t *)src, (uint32_t *)dst, p);
      break;
  }
  SKLB_COUNT_LAUNCH();
  return (int)cudaGetLastError();
}

inline int64_t nz(int64_t v) { return v > 0 ? v : 1; }

}  // namespace
}  // namespace sklb

using namespace sklb;

extern "C" int skl_b200_launch_pack(size_t esize, size_t m, size_t n, const void *src, size_t rs,
                                    size_t cs, size_t m0, size_t n0, void *dst, size_t rs0,
                                    size_t cs0, size_t rs1, size_t cs1, uint32_t pad, void *stream) {
  if (m0 == 0 || n0 == 0) return 0;
  RelayoutParams p;
  const int64_t m1 = (int64_t)((m + m0 - 1) / m0), n1 = (int64_t)((n + n0 - 1) / n0);
  p.MI = m1 * (int64_t)m0;
  p.NJ = n1 * (int64_t)n0;
  p.m = (int64_t)m;
  p.n = (int64_t)n;
  p.src = Side{nz(p.MI), nz(p.NJ), (int64_t)rs, (int64_t)cs, 0, 0};
  p.dst = Side{(int64_t)m0, (int64_t)n0, (int64_t)rs0, (int64_t)cs0, (int64_t)rs1, (int64_t)cs1};
  p.pad = pad;
  p.src_fast_j = (cs == 1 || rs != 1) ? 1 : 0;
  p.dst_fast_j = (cs0 == 1 || rs0 != 1) ? 1 : 0;
  return launch_relayout(esize, src, dst, p, (cudaStream_t)stream);
}

extern "C" int skl_b200_launch_unpack(size_t esize, size_t m0, size_t n0, const void *src, size_t rs0,
                                      size_t cs0, size_t rs1, size_t cs1, size_t m, size_t n,
                                      void *dst, size_t rs, size_t cs, void *stream) {
  if (m0 == 0 || n0 == 0) return 0;
  RelayoutParams p;
  p.MI = (int64_t)m;
  p.NJ = (int64_t)n;
  p.m = (int64_t)m;
  p.n = (int64_t)n;
  p.src = Side{(int64_t)m0, (int64_t)n0, (int64_t)rs0, (int64_t)cs0, (int64_t)rs1, (int64_t)cs1};
  p.dst = Side{nz(p.MI), nz(p.NJ), (int64_t)rs, (int64_t)cs, 0, 0};
  p.pad = 0;
  p.src_fast_j = (cs0 == 1 || rs0 != 1) ? 1 : 0;
  p.dst_fast_j = (cs == 1 || rs != 1) ? 1 : 0;
  return launch_relayout(esize, src, dst, p, (cudaStream_t)stream);
}

extern "C" int skl_b200_launch_transpose(size_t esize, size_t m, size_t n, const void *a, size_t rsa,
                                         void *at, size_t rsat, void *stream) {
  RelayoutParams p;
  p.MI = (int64_t)m;
  p.NJ = (int64_t)n;
  p.m = (int64_t)m;
  p.n = (int64_t)n;
  p.src = Side{nz(p.MI), nz(p.NJ), (int64_t)rsa, 1, 0, 0};
  p.dst = Side{nz(p.MI), nz(p.NJ), 1, (int64_t)rsat, 0, 0};  // at[j*rsat + i]
  p.pad = 0;
  p.src_fast_j = 1;
  p.dst_fast_j = 0;
  return launch_relayout(esize, a, at, p, (cudaStream_t)stream);
}
