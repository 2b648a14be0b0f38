// CUDA-core fp32 GEMM used for shapes the tensor-core kernel does not take (feature counts
// that break the TMA alignment rules, tiny contractions) and as the bring-up comparison for it.
// Y[M,N] = A[M,Kc] W[Kc,N] (+ bias on the first `bias_rows` rows), all row-major fp32.
#include "gemm.cuh"

namespace fl {
namespace {

constexpr int BM = 64, BN = 64, BK = 16;

__global__ void __launch_bounds__(256)
gemm_ffma_kernel(const float* __restrict__ A, const float* __restrict__ W,
                 const float* __restrict__ bias, float* __restrict__ Y, int64_t M, int Kc, int N,
                 int64_t bias_rows) {
  __shared__ float As[BK][BM + 4];
  __shared__ float Ws[BK][BN + 4];
  const int tx = threadIdx.x & 15, ty = threadIdx.x >> 4;
  const int64_t m0 = (int64_t)blockIdx.x * BM;
  const int n0 = blockIdx.y * BN;
  float acc[4][4] = {};
  for (int k0 = 0; k0 < Kc; k0 += BK) {
    // A tile: 64 rows x 16 k, each thread loads 4 elements
    for (int e = threadIdx.x; e < BM * BK; e += 256) {
      int r = e / BK, c = e % BK;
      int64_t gm = m0 + r;
      int gk = k0 + c;
      As[c][r] = (gm < M && gk < Kc) ? A[gm * Kc + gk] : 0.f;
    }
    for (int e = threadIdx.x; e < BK * BN; e += 256) {
      int r = e / BN, c = e % BN;
      int gk = k0 + r, gn = n0 + c;
      Ws[r][c] = (gk < Kc && gn < N) ? W[(int64_t)gk * N + gn] : 0.f;
    }
    __syncthreads();
#pragma unroll
    for (int k = 0; k < BK; ++k) {
      float a[4], b[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) a[i] = As[k][ty * 4 + i];
#pragma unroll
      for (int j = 0; j < 4; ++j) b[j] = Ws[k][tx * 4 + j];
#pragma unroll
      for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(a[i], b[j], acc[i][j]);
    }
    __syncthreads();
  }
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    int64_t gm = m0 + ty * 4 + i;
    if (gm >= M) continue;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      int gn = n0 + tx * 4 + j;
      if (gn >= N) continue;
      float v = acc[i][j];
      if (bias && gm < bias_rows) v += bias[gn];
      Y[gm * N + gn] = v;
    }
  }
}

// Short contracted axis (first layers: 4 or 16 input features): the product is a stream -- read
// Kc floats per row, write N -- so one thread owns four output columns, keeps its Kc x 4 block of W
// in registers and walks down the rows; a warp writes whole 128-byte lines.  HBM-bound:
// 4 M (Kc + N) bytes.
template <int KC>
__global__ void __launch_bounds__(256)
gemm_smallk_kernel(const float* __restrict__ A, const float* __restrict__ W,
                   const float* __restrict__ bias, float* __restrict__ Y, int64_t M, int N,
                   int64_t bias_rows) {
  const int cg_count = N / 4;              // column groups of 4 (N % 4 == 0, N <= 1024)
  const int rows_per_pass = 256 / cg_count;
  const int cg = threadIdx.x % cg_count, r_off = threadIdx.x / cg_count;
  if (r_off >= rows_per_pass) return;
  float4 w[KC];
#pragma unroll
  for (int k = 0; k < KC; ++k) w[k] = __ldg(reinterpret_cast<const float4*>(W + (int64_t)k * N) + cg);
  const float4 bv = bias ? __ldg(reinterpret_cast<const float4*>(bias) + cg) : make_float4(0.f, 0.f, 0.f, 0.f);
  const int64_t stride = (int64_t)gridDim.x * rows_per_pass;
  for (int64_t row = (int64_t)blockIdx.x * rows_per_pass + r_off; row < M; row += stride) {
    float a[KC];
    if constexpr (KC % 4 == 0) {
#pragma unroll
      for (int k4 = 0; k4 < KC / 4; ++k4) {
        const float4 v = __ldg(reinterpret_cast<const float4*>(A + row * KC) + k4);
        a[4 * k4] = v.x; a[4 * k4 + 1] = v.y; a[4 * k4 + 2] = v.z; a[4 * k4 + 3] = v.w;
      }
    } else {
#pragma unroll
      for (int k = 0; k < KC; ++k) a[k] = __ldg(A + row * KC + k);
    }
    float4 acc = row < bias_rows ? bv : make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
    for (int k = 0; k < KC; ++k) {
      acc.x = fmaf(a[k], w[k].x, acc.x); acc.y = fmaf(a[k], w[k].y, acc.y);
      acc.z = fmaf(a[k], w[k].z, acc.z); acc.w = fmaf(a[k], w[k].w, acc.w);
    }
    __stcs(reinterpret_cast<float4*>(Y + row * N) + cg, acc);
  }
}

// Few output columns (a final Dense(1), N <= 8): every row is N dot products of length Kc.  One
// warp per row, lanes stride over k (coalesced reads of A, W comes from the cache), partial sums
// meet in a shuffle reduction.  HBM-bound: 4 M Kc bytes.
template <int NC>
__global__ void __launch_bounds__(256)
gemm_smalln_kernel(const float* __restrict__ A, const float* __restrict__ W,
                   const float* __restrict__ bias, float* __restrict__ Y, int64_t M, int Kc,
                   int64_t bias_rows) {
  const int lane = threadIdx.x & 31;
  const int64_t warps = (int64_t)gridDim.x * 8;
  for (int64_t row = (int64_t)blockIdx.x * 8 + (threadIdx.x >> 5); row < M; row += warps) {
    float acc[NC];
#pragma unroll
    for (int j = 0; j < NC; ++j) acc[j] = 0.f;
    const float* a = A + row * Kc;
    for (int k = lane; k < Kc; k += 32) {
      const float av = __ldg(a + k);
#pragma unroll
      for (int j = 0; j < NC; ++j) acc[j] = fmaf(av, __ldg(W + (int64_t)k * NC + j), acc[j]);
    }
#pragma unroll
    for (int j = 0; j < NC; ++j)
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) acc[j] += __shfl_xor_sync(0xffffffffu, acc[j], o);
    if (lane < NC) {
      float v = 0.f;
#pragma unroll
      for (int j = 0; j < NC; ++j) v = lane == j ? acc[j] : v;
      if (bias && row < bias_rows) v += bias[lane];
      Y[row * NC + lane] = v;
    }
  }
}

template <int NC>
int32_t launch_smalln(const float* A, int64_t M, int64_t Kc, const float* W, const float* bias,
                      int64_t bias_rows, float* Y, cudaStream_t st) {
  int64_t blocks = (M + 7) / 8;
  const int64_t cap = (int64_t)sm_count() * 16;
  if (blocks > cap) blocks = cap;
  gemm_smalln_kernel<NC><<<(unsigned)blocks, 256, 0, st>>>(A, W, bias, Y, M, (int)Kc, bias_rows);
  FL_CHECK_LAUNCH("gemm_smalln launch");
  return FL_OK;
}

template <int KC>
int32_t launch_smallk(const float* A, int64_t M, int64_t N, const float* W, const float* bias,
                      int64_t bias_rows, float* Y, cudaStream_t st) {
  const int rows_per_pass = 256 / (int)(N / 4);
  int64_t blocks = (M + rows_per_pass - 1) / rows_per_pass;
  const int64_t cap = (int64_t)sm_count() * 16;  // a few passes per block amortise the W registers
  if (blocks > cap) blocks = cap;
  gemm_smallk_kernel<KC><<<(unsigned)blocks, 256, 0, st>>>(A, W, bias, Y, M, (int)N, bias_rows);
  FL_CHECK_LAUNCH("gemm_smallk launch");
  return FL_OK;
}

}  // namespace

int32_t gemm_ffma(const float* A, int64_t M, int64_t Kc, int64_t N, const float* W,
                  const float* bias, int64_t bias_rows, float* Y, cudaStream_t st) {
  if (M == 0 || N == 0) return FL_OK;
  // streaming kernel for a short contracted axis
  if (Kc <= 16 && N % 4 == 0 && N <= 1024 && aligned16(W) && aligned16(Y) &&
      (bias == nullptr || aligned16(bias)) && (Kc % 4 != 0 || aligned16(A))) {
    switch ((int)Kc) {
#define FL_SK(K) case K: return launch_smallk<K>(A, M, N, W, bias, bias_rows, Y, st);
      FL_SK(1) FL_SK(2) FL_SK(3) FL_SK(4) FL_SK(5) FL_SK(6) FL_SK(7) FL_SK(8) FL_SK(12) FL_SK(16)
#undef FL_SK
      default: break;
    }
  }
  // a handful of output columns over a long contracted axis: one warp per row
  if (N <= 8 && Kc >= 32 && Kc < (1 << 30)) {
    switch ((int)N) {
#define FL_SN(C) case C: return launch_smalln<C>(A, M, Kc, W, bias, bias_rows, Y, st);
      FL_SN(1) FL_SN(2) FL_SN(3) FL_SN(4) FL_SN(5) FL_SN(6) FL_SN(7) FL_SN(8)
#undef FL_SN
      default: break;
    }
  }
  int64_t gx = (M + BM - 1) / BM;
  int64_t gy = (N + BN - 1) / BN;
  FL_REQUIRE(gx < (1ll << 31) && gy < 65536, FL_EBADSHAPE, "gemm: grid too large");
  gemm_ffma_kernel<<<dim3((unsigned)gx, (unsigned)gy), 256, 0, st>>>(A, W, bias, Y, M, (int)Kc,
                                                                     (int)N, bias_rows);
  FL_CHECK_LAUNCH("gemm_ffma launch");
  return FL_OK;
}

}  // namespace fl
