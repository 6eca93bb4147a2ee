// gemm_generic.cu -- any-stride SIMT GEMM.
//
// Serves every problem the tensor-core and skinny kernels decline: arbitrary element strides on all
// three matrices, blocked (packed) operands with their twelve strides, k == 0, tiny shapes,
// unaligned bases.  Semantics are those of the scalar definitions in
// ref/gemm/gemm_i8rc_i8rc_i32rc.c:10-26 / gemm_i8rcprc_i8rcprc_i32rcprc.c:10-37 and the float
// siblings: one accumulator per output element, k ascending, products and sums each rounded once
// to fp32 -- so for float operands this kernel reproduces the reference's summation order exactly.
//
// Layout: 64 x 64 output tile per CTA, 16 x 16 threads, 4 x 4 outputs per thread spaced 16 apart,
// K staged 16 at a time through shared memory as already-decoded 32-bit values.  HBM traffic is
// operand bytes x (number of tiles sharing them) -- this is the compatibility path, not the fast one.
#include "numerics.cuh"

namespace sklb {

int &launch_counter_ref() {
  static thread_local int counter = 0;
  return counter;
}

namespace {

constexpr int TM = 64, TN = 64, TK = 16;

struct GenericParams {
  skl_b200_gemm_args g;
  int64_t M, N, K;
};

template <bool BLOCKED>
__device__ __forceinline__ int64_t offs(int64_t r, int64_t c, int64_t r0, int64_t c0, int64_t rs0,
                                        int64_t cs0, int64_t rs1, int64_t cs1) {
  if (!BLOCKED) return r * rs0 + c * cs0;
  return (r / r0) * rs1 + (r % r0) * rs0 + (c / c0) * cs1 + (c % c0) * cs0;
}

// fp32 value rounded to fp16 and back: the rounding the fp16-accumulate GEMM applies after every statement.
__device__ __forceinline__ float round_to_f16(float x) { return dec_f16(enc_f16(x)); }

// ACC: 0 = int32 (int8 operands), 1 = fp32 (bf16 / f16 / fp8 / f32 operands), 2 = fp64 (f64 operands),
//      3 = fp16 accumulator held as an fp32 value (fp16 operands, SKL_EPI_F16ACC)
template <int ACC, bool BLOCKED>
__global__ void __launch_bounds__(256) gemm_generic_kernel(const GenericParams p) {
  constexpr bool IS_INT = ACC == 0;
  using acc_t = typename std::conditional<ACC == 0, int32_t, typename std::conditional<ACC == 2, double, float>::type>::type;
  __shared__ acc_t As[TK][TM + 1];
  __shared__ acc_t Bs[TK][TN + 1];

  const skl_b200_gemm_args &g = p.g;
  const int tid = threadIdx.x;
  const int tx = tid & 15, ty = tid >> 4;
  const int64_t row0 = (int64_t)blockIdx.y * TM;
  const int64_t col0 = (int64_t)blockIdx.x * TN;

  acc_t acc[4][4];
#pragma unroll
  for (int r = 0; r < 4; ++r)
#pragma unroll
    for (int c = 0; c < 4; ++c) acc[r][c] = 0;

  // Pick the staging order whose fastest-moving thread index follows the operand's unit stride.
  const bool a_k_fast = (g.csa0 == 1);
  const bool b_k_fast = (g.rsb0 == 1);

  for (int64_t kt = 0; kt < p.K; kt += TK) {
#pragma unroll
    for (int q = 0; q < 4; ++q) {
      int e = tid + q * 256;
      int kk, rr;
      if (a_k_fast) {
        kk = e & 15;
        rr = e >> 4;
      } else {
        rr = e & 63;
        kk = e >> 6;
      }
      int64_t i = row0 + rr, kidx = kt + kk;
      acc_t v = 0;
      if (i < p.M && kidx < p.K) {
        int64_t o = offs<BLOCKED>(i, kidx, g.m0, g.k0, g.rsa0, g.csa0, g.rsa1, g.csa1);
        if (IS_INT)
          v = (acc_t)((const int8_t *)g.a)[o];
        else if (ACC == 2)
          v = (acc_t)((const double *)g.a)[o];
        else
          v = (acc_t)load_as_f32(g.ta, g.a, o);
      }
      As[kk][rr] = v;
    }
#pragma unroll
    for (int q = 0; q < 4; ++q) {
      int e = tid + q * 256;
      int kk, cc;
      if (b_k_fast) {
        kk = e & 15;
        cc = e >> 4;
      } else {
        cc = e & 63;
        kk = e >> 6;
      }
      int64_t j = col0 + cc, kidx = kt + kk;
      acc_t v = 0;
      if (j < p.N && kidx < p.K) {
        int64_t o = offs<BLOCKED>(kidx, j, g.k0, g.n0, g.rsb0, g.csb0, g.rsb1, g.csb1);
        if (IS_INT)
          v = (acc_t)((const int8_t *)g.b)[o];
        else if (ACC == 2)
          v = (acc_t)((const double *)g.b)[o];
        else
          v = (acc_t)load_as_f32(g.tb, g.b, o);
      }
      Bs[kk][cc] = v;
    }
    __syncthreads();
    const int klim = (int)((p.K - kt) < TK ? (p.K - kt) : TK);  // no padded terms enter the sum
    for (int kk = 0; kk < klim; ++kk) {
      acc_t av[4], bv[4];
#pragma unroll
      for (int r = 0; r < 4; ++r) av[r] = As[kk][ty + 16 * r];
#pragma unroll
      for (int c = 0; c < 4; ++c) bv[c] = Bs[kk][tx + 16 * c];
#pragma unroll
      for (int r = 0; r < 4; ++r)
#pragma unroll
        for (int c = 0; c < 4; ++c) {
          if (IS_INT)
            acc[r][c] = (acc_t)((uint32_t)acc[r][c] + (uint32_t)((int32_t)av[r] * (int32_t)bv[c]));
          else if (ACC == 2)
            acc[r][c] = (acc_t)__dadd_rn((double)acc[r][c], __dmul_rn((double)av[r], (double)bv[c]));
          else if (ACC == 3)
            acc[r][c] = (acc_t)round_to_f16(__fadd_rn((float)acc[r][c], __fmul_rn((float)av[r], (float)bv[c])));
          else
            acc[r][c] = (acc_t)__fadd_rn((float)acc[r][c], __fmul_rn((float)av[r], (float)bv[c]));
        }
    }
    __syncthreads();
  }

  float local_max = -INFINITY;
#pragma unroll
  for (int r = 0; r < 4; ++r) {
    int64_t i = row0 + ty + 16 * r;
    if (i >= p.M) continue;
#pragma unroll
    for (int c = 0; c < 4; ++c) {
      int64_t j = col0 + tx + 16 * c;
      if (j >= p.N) continue;
      int64_t o = offs<BLOCKED>(i, j, g.m0, g.n0, g.rsc0, g.csc0, g.rsc1, g.csc1);
      if (g.epilogue == SKL_EPI_INT) {
        int32_t *cp = (int32_t *)g.c + o;
        uint32_t prod = (uint32_t)g.alpha_i * (uint32_t)(int32_t)acc[r][c];
        uint32_t old = (g.beta_i != 0) ? (uint32_t)g.beta_i * (uint32_t)*cp : 0u;
        *cp = (int32_t)(old + prod);
      } else if (g.epilogue == SKL_EPI_F16ACC) {
        uint16_t *cp = (uint16_t *)g.c + o;
        const float prod = __fmul_rn(g.alpha_f, (float)acc[r][c]);  // exact: two fp16 values
        const float v = (g.beta_f != 0.0f) ? __fadd_rn(__fmul_rn(g.beta_f, dec_f16(*cp)), prod) : prod;
        *cp = (uint16_t)enc_f16(v);
      } else if (g.epilogue == SKL_EPI_F64) {
        double *cp = (double *)g.c + o;
        const double prod = __dmul_rn(g.alpha_d, (double)acc[r][c]);
        *cp = (g.beta_d != 0.0) ? __dadd_rn(__dmul_rn(g.beta_d, *cp), prod) : prod;
      } else {
        float v = epilogue_value((float)acc[r][c], g.alpha_f, g.row_scale, g.col_scale, i, j);
        if (g.bias) v = __fadd_rn(v, g.bias[g.bias_per_row ? i : j]);
        if (g.beta_f != 0.0f) v = __fadd_rn(__fmul_rn(g.beta_f, load_c_f32(g.tc, g.c, o)), v);
        if (g.activation)
          v = activation_value(g.activation, g.act_param, v,
                               g.activation == SKL_ACT_SWIGLU ? load_c_f32(g.tc, g.c, o) : 0.0f);
        if (v == v) local_max = fmaxf(local_max, v);
        store_c_f32(g.tc, g.c, o, v);
      }
    }
  }
  if (g.epilogue == SKL_EPI_FLOAT && g.global_max) {
    local_max = warp_max_f32(local_max);
    if ((tid & 31) == 0 && local_max != -INFINITY) atomic_max_f32(g.global_max, local_max);
  }
}

}  // namespace
}  // namespace sklb

extern "C" int skl_b200_launch_counter(int reset) {
  int &c = sklb::launch_counter_ref();
  int v = c;
  if (reset) c = 0;
  return v;
}

extern "C" int skl_b200_launch_gemm_generic(const skl_b200_gemm_args *args, void *stream) {
  using namespace sklb;
  GenericParams p;
  p.g = *args;
  p.M = (int64_t)(args->m0 * args->m1);
  p.N = (int64_t)(args->n0 * args->n1);
  p.K = (int64_t)(args->k0 * args->k1);
  if (p.M == 0 || p.N == 0) return 0;
  const bool blocked = !(args->m1 == 1 && args->n1 == 1 && args->k1 == 1);
  const bool is_int = (args->ta == SKL_DT_I8);
  const bool is_f64 = (args->ta == SKL_DT_F64);
  const bool is_f16acc = (args->epilogue == SKL_EPI_F16ACC);
  dim3 grid((unsigned)((p.N + TN - 1) / TN), (unsigned)((p.M + TM - 1) / TM));
  if (grid.y > 65535u) return (int)cudaErrorInvalidConfiguration;
  cudaStream_t s = (cudaStream_t)stream;
  if (is_int) {
    if (blocked)
      gemm_generic_kernel<0, true><<<grid, 256, 0, s>>>(p);
    else
      gemm_generic_kernel<0, false><<<grid, 256, 0, s>>>(p);
  } else if (is_f64) {
    if (blocked)
      gemm_generic_kernel<2, true><<<grid, 256, 0, s>>>(p);
    else
      gemm_generic_kernel<2, false><<<grid, 256, 0, s>>>(p);
  } else if (is_f16acc) {
    if (blocked)
      gemm_generic_kernel<3, true><<<grid, 256, 0, s>>>(p);
    else
      gemm_generic_kernel<3, false><<<grid, 256, 0, s>>>(p);
  } else {
    if (blocked)
      gemm_generic_kernel<1, true><<<grid, 256, 0, s>>>(p);
    else
      gemm_generic_kernel<1, false><<<grid, 256, 0, s>>>(p);
  }
  SKLB_COUNT_LAUNCH();
  return (int)cudaGetLastError();
}
