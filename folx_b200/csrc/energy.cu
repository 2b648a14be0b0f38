// Local energy of every walker and its block-reduced statistics.
//
//   E_L = -1/2 (lap + sum_k J_k^2) + V        (kinetic energy of log|psi| plus the potential)
//   sums = [ sum_w E_L, sum_w E_L^2, number of walkers ]   in fp64
//
// The reference has no such step (it stops at (laplacian, jacobian), folx/operators.py:34-36);
// it is the one place where walkers are combined, and the three fp64 sums are what a multi-GPU
// run all-reduces.  Two launches keep the result deterministic without floating-point atomics:
// blocks write their partial sums to caller-provided scratch, then a single block adds them in a
// fixed order.
#include "common.cuh"

namespace fl {
namespace {

constexpr int kThreads = 256;

__global__ void __launch_bounds__(kThreads)
energy_kernel(const float* __restrict__ lap, const float* __restrict__ jac, int64_t js,
              const float* __restrict__ pot, int64_t B, int K, float* __restrict__ E,
              double* __restrict__ partials) {
  __shared__ double s1[kThreads / 32], s2[kThreads / 32];
  const int64_t w = (int64_t)blockIdx.x * kThreads + threadIdx.x;
  double e = 0.0, e2 = 0.0;
  if (w < B) {
    float g2 = 0.f;
    for (int k = 0; k < K; ++k) {
      float v = jac[(int64_t)k * js + w];
      g2 = fmaf(v, v, g2);
    }
    float el = -0.5f * (lap[w] + g2) + (pot ? pot[w] : 0.f);
    E[w] = el;
    e = (double)el;
    e2 = e * e;
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    e += __shfl_xor_sync(0xffffffffu, e, o);
    e2 += __shfl_xor_sync(0xffffffffu, e2, o);
  }
  if ((threadIdx.x & 31) == 0) {
    s1[threadIdx.x >> 5] = e;
    s2[threadIdx.x >> 5] = e2;
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    double a = 0.0, b = 0.0;
    for (int i = 0; i < kThreads / 32; ++i) { a += s1[i]; b += s2[i]; }
    partials[2 * (int64_t)blockIdx.x] = a;
    partials[2 * (int64_t)blockIdx.x + 1] = b;
  }
}

__global__ void energy_finish_kernel(const double* __restrict__ partials, int64_t n_blocks, int64_t B,
                                     double* __restrict__ sums) {
  // one thread, fixed order: n_blocks is B / 256, a few dozen entries at most per launch
  if (threadIdx.x == 0 && blockIdx.x == 0) {
    double a = 0.0, b = 0.0;
    for (int64_t i = 0; i < n_blocks; ++i) { a += partials[2 * i]; b += partials[2 * i + 1]; }
    sums[0] = a;
    sums[1] = b;
    sums[2] = (double)B;
  }
}

}  // namespace

int64_t energy_blocks(int64_t B) { return (B + kThreads - 1) / kThreads; }

int32_t energy_launch(const float* lap, const float* jac, int64_t js, const float* pot, int64_t B,
                      int64_t K, float* E, double* partials, double* sums, cudaStream_t st) {
  const int64_t nb = energy_blocks(B);
  energy_kernel<<<(unsigned)nb, kThreads, 0, st>>>(lap, jac, js, pot, B, (int)K, E, partials);
  FL_CHECK_LAUNCH("fl_local_energy launch");
  energy_finish_kernel<<<1, 32, 0, st>>>(partials, nb, B, sums);
  FL_CHECK_LAUNCH("fl_local_energy finish launch");
  return FL_OK;
}

}  // namespace fl

extern "C" int64_t fl_local_energy_workspace_bytes(int64_t B) {
  return B <= 0 ? 16 : fl::energy_blocks(B) * 2 * (int64_t)sizeof(double);
}

extern "C" int32_t fl_local_energy(const float* lap, const float* jac, int64_t jac_stride,
                                   const float* pot, int64_t B, int64_t K, float* energy,
                                   void* workspace, int64_t workspace_bytes, double* sums,
                                   void* stream) {
  using namespace fl;
  FL_REQUIRE(B >= 0 && K >= 0 && K < (1ll << 31), FL_EBADSHAPE, "fl_local_energy: bad sizes");
  FL_REQUIRE(sums != nullptr, FL_EBADSHAPE, "fl_local_energy: sums is NULL");
  FL_REQUIRE(energy_blocks(B) < (1ll << 31), FL_EBADSHAPE, "fl_local_energy: too many walkers");
  if (B == 0) {
    FL_CUDA(cudaMemsetAsync(sums, 0, 3 * sizeof(double), (cudaStream_t)stream));
    return FL_OK;
  }
  FL_REQUIRE(lap && energy && (K == 0 || jac) && workspace, FL_EBADSHAPE,
             "fl_local_energy: null pointer");
  FL_REQUIRE(K <= 1 || jac_stride >= B, FL_EBADSHAPE, "fl_local_energy: Jacobian row stride < B");
  FL_REQUIRE(workspace_bytes >= fl_local_energy_workspace_bytes(B), FL_EBADSHAPE,
             "fl_local_energy: workspace too small");
  FL_REQUIRE((reinterpret_cast<uintptr_t>(workspace) & 7) == 0, FL_EBADSHAPE,
             "fl_local_energy: workspace must be 8-byte aligned");
  return energy_launch(lap, jac, jac_stride, pot, B, K, energy, (double*)workspace, sums,
                       (cudaStream_t)stream);
}

// ---------------------------------------------------------------------------------------------
// Allocation-free variant.
//
// Some callers cannot hand over scratch memory and must not trigger an allocation themselves:
// an XLA/JAX custom call whose buffers were all planned by the compiler before the step runs, a
// Monte-Carlo driver whose framework has already claimed the whole device for its own pool (a
// cudaMalloc from a plug-in then fails or fragments that pool), code running between the steps of
// a latency-critical loop where an allocation would stall the stream.  For them the per-block
// partial sums live in a fixed array inside the library image instead of a workspace argument.
//
// The array exists once per GPU that loads the library (FL_LOCAL_ENERGY_STATIC_MAX_WALKERS / 256
// blocks x 2 doubles = 64 KiB, held until the process exits).  Host code cannot use the array's
// name as a device address -- it has to ask the runtime for it -- so the first call on each
// device looks the address up (cudaGetSymbolAddress, with that device current) and remembers it.
// All calls on a device share the array and it keeps whatever the previous call left there; that
// is harmless here because every entry the finishing launch reads was written by the same
// call's first launch, so nothing needs clearing -- but two calls that are in flight at the same
// time on one GPU (different streams) would overwrite each other's partial sums.
// ---------------------------------------------------------------------------------------------
namespace fl {
namespace {

constexpr int64_t kStaticMaxBlocks = FL_LOCAL_ENERGY_STATIC_MAX_WALKERS / kThreads;
static __device__ __align__(256) double g_static_partials[2 * kStaticMaxBlocks];

constexpr int kMaxDevices = 64;
static double* g_static_ptr[kMaxDevices] = {nullptr};

// Device address of the static scratch on the current device (looked up once per device).
int32_t static_scratch(double** out) {
  int dev = -1;
  FL_CUDA(cudaGetDevice(&dev));
  FL_REQUIRE(dev >= 0 && dev < kMaxDevices, FL_EUNSUPPORTED,
             "fl_local_energy_static: device ordinal %d out of range", dev);
  if (g_static_ptr[dev] == nullptr) {
    double* p = nullptr;
    cudaError_t e = cudaGetSymbolAddress((void**)&p, g_static_partials);
    if (e != cudaSuccess) return cuda_fail(e, "cudaGetSymbolAddress(static energy scratch)");
    FL_REQUIRE(p != nullptr, FL_ECUDA, "fl_local_energy_static: no address for the static scratch");
    g_static_ptr[dev] = p;
  }
  *out = g_static_ptr[dev];
  return FL_OK;
}

}  // namespace
}  // namespace fl

extern "C" int32_t fl_local_energy_static(const float* lap, const float* jac, int64_t jac_stride,
                                          const float* pot, int64_t B, int64_t K, float* energy,
                                          double* sums, void* stream) {
  using namespace fl;
  FL_REQUIRE(B >= 0 && K >= 0 && K < (1ll << 31), FL_EBADSHAPE, "fl_local_energy_static: bad sizes");
  FL_REQUIRE(B <= FL_LOCAL_ENERGY_STATIC_MAX_WALKERS, FL_EBADSHAPE,
             "fl_local_energy_static: %lld walkers exceed the built-in scratch (max %lld); use "
             "fl_local_energy with a caller-provided workspace",
             (long long)B, (long long)FL_LOCAL_ENERGY_STATIC_MAX_WALKERS);
  FL_REQUIRE(sums != nullptr, FL_EBADSHAPE, "fl_local_energy_static: sums is NULL");
  if (B == 0) {
    FL_CUDA(cudaMemsetAsync(sums, 0, 3 * sizeof(double), (cudaStream_t)stream));
    return FL_OK;
  }
  FL_REQUIRE(lap && energy && (K == 0 || jac), FL_EBADSHAPE, "fl_local_energy_static: null pointer");
  FL_REQUIRE(K <= 1 || jac_stride >= B, FL_EBADSHAPE,
             "fl_local_energy_static: Jacobian row stride < B");
  double* scratch = nullptr;
  int32_t rc = static_scratch(&scratch);
  if (rc != FL_OK) return rc;
  return energy_launch(lap, jac, jac_stride, pot, B, K, energy, scratch, sums, (cudaStream_t)stream);
}
