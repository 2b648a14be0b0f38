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

}  // namespace

int32_t gemm_ffma(const float* A, int64_t M, int64_t Kc, int64_t N, const float* W,
                  const float* bias, int64_t bias_rows, float* Y, cudaStream_t st) {
  if (M == 0 || N == 0) return FL_OK;
  int64_t gx = (M + BM - 1) / BM;
  int64_t gy = (N + BN - 1) / BN;
  FL_REQUIRE(gx < (1ll << 31) && gy < 65536, FL_EBADSHAPE, "gemm: grid too large");
  gemm_ffma_kernel<<<dim3((unsigned)gx, (unsigned)gy), 256, 0, st>>>(A, W, bias, Y, M, (int)Kc,
                                                                     (int)N, bias_rows);
  FL_CHECK_LAUNCH("gemm_ffma launch");
  return FL_OK;
}

}  // namespace fl
