// Binary elementwise forward-Laplacian rules (add, sub, mul, div) on two triplets whose
// Jacobian rows are aligned (row k of both operands refers to the same input coordinate).
//
//   mul: y = a b,  J = Ja b + a Jb,  lap = la b + a lb + 2 sum_k Ja_k Jb_k
//        (reference: folx/wrapped_functions.py:375-377, folx/hessian.py:177-188)
//   div: y = a / b, J = Ja / b - a Jb / b^2,
//        lap = la / b - a lb / b^2 - (2 / b^2) sum_k Ja_k Jb_k + (2 a / b^3) sum_k Jb_k^2
//        (reference: folx/wrapped_functions.py:378-383, folx/custom_hessian.py:35-59)
//   add/sub: linear in both operands, no Hessian term (folx/wrapped_functions.py:364-369).
//
// Either operand may be a constant array (its lap pointer, and jac pointer, are NULL): then its Jacobian
// and Laplacian are zero.  Operand b may be periodic along the position axis (broadcast).
// HBM-bound, one pass; algorithmic traffic 4 (K + 2) (N_a + N_b + N) bytes.
#include "common.cuh"

namespace fl {
namespace {

template <int OP>
__device__ __forceinline__ void coeffs(float a, float b, float& y, float& ca, float& cb,
                                       float& hab, float& hbb) {
  // y, dy/da, dy/db, and the Hessian weights multiplying sum Ja Jb and sum Jb Jb.
  if constexpr (OP == FL_BIN_ADD) {
    y = a + b; ca = 1.f; cb = 1.f; hab = 0.f; hbb = 0.f;
  } else if constexpr (OP == FL_BIN_SUB) {
    y = a - b; ca = 1.f; cb = -1.f; hab = 0.f; hbb = 0.f;
  } else if constexpr (OP == FL_BIN_MUL) {
    y = a * b; ca = b; cb = a; hab = 2.f; hbb = 0.f;
  } else {
    float inv = 1.0f / b;
    y = a * inv;
    ca = inv;
    cb = -a * inv * inv;
    hab = -2.0f * inv * inv;
    hbb = 2.0f * a * inv * inv * inv;
  }
}

template <int OP, bool A_TRIPLET, bool B_TRIPLET>
__global__ void __launch_bounds__(256)
binary_kernel(const float* __restrict__ a, const float* __restrict__ ja,
              const float* __restrict__ la, int64_t jas, const float* __restrict__ b,
              const float* __restrict__ jb, const float* __restrict__ lb, int64_t jbs,
              float* __restrict__ y, float* __restrict__ jy, float* __restrict__ ly, int64_t jys,
              int K, int64_t N, int64_t b_period) {
  int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= N) return;
  int64_t ib = (b_period == N) ? i : (i % b_period);
  float av = a[i], bv = b[ib];
  float yv, ca, cb, hab, hbb;
  coeffs<OP>(av, bv, yv, ca, cb, hab, hbb);
  y[i] = yv;
  float sab = 0.f, sbb = 0.f;
#pragma unroll 4
  for (int k = 0; k < K; ++k) {
    float va = A_TRIPLET ? __ldcs(ja + (int64_t)k * jas + i) : 0.f;
    float vb = B_TRIPLET ? __ldg(jb + (int64_t)k * jbs + ib) : 0.f;
    if constexpr (OP == FL_BIN_MUL || OP == FL_BIN_DIV) {
      sab = fmaf(va, vb, sab);
      if constexpr (OP == FL_BIN_DIV) sbb = fmaf(vb, vb, sbb);
    }
    __stcs(jy + (int64_t)k * jys + i, fmaf(ca, va, cb * vb));
  }
  float lav = A_TRIPLET ? la[i] : 0.f;
  float lbv = B_TRIPLET ? lb[ib] : 0.f;
  ly[i] = fmaf(ca, lav, cb * lbv) + hab * sab + hbb * sbb;
}

template <int OP>
int32_t dispatch(const float* a, const float* ja, const float* la, int64_t jas, const float* b,
                 const float* jb, const float* lb, int64_t jbs, float* y, float* jy, float* ly,
                 int64_t jys, int64_t K, int64_t N, int64_t b_period, cudaStream_t st) {
  unsigned blocks = (unsigned)((N + 255) / 256);
  bool at = la != nullptr, bt = lb != nullptr;
#define FL_LAUNCH(AT, BT)                                                                     \
  binary_kernel<OP, AT, BT><<<blocks, 256, 0, st>>>(a, ja, la, jas, b, jb, lb, jbs, y, jy, ly, \
                                                    jys, (int)K, N, b_period)
  if (at && bt) FL_LAUNCH(true, true);
  else if (at) FL_LAUNCH(true, false);
  else if (bt) FL_LAUNCH(false, true);
  else FL_LAUNCH(false, false);
#undef FL_LAUNCH
  FL_CHECK_LAUNCH("fl_binary launch");
  return FL_OK;
}

}  // namespace
}  // namespace fl

extern "C" int32_t fl_binary(int32_t op, const float* a, const float* jac_a, const float* lap_a,
                             int64_t jac_a_stride, const float* b, const float* jac_b,
                             const float* lap_b, int64_t jac_b_stride, float* y, float* jac_y,
                             float* lap_y, int64_t jac_y_stride, int64_t K, int64_t N,
                             int64_t b_period, void* stream) {
  using namespace fl;
  FL_REQUIRE(op >= FL_BIN_ADD && op <= FL_BIN_DIV, FL_EUNSUPPORTED, "fl_binary: unknown op %d", op);
  FL_REQUIRE(K >= 0 && N >= 0 && K < (1ll << 31) && (N + 255) / 256 < (1ll << 31), FL_EBADSHAPE,
             "fl_binary: bad sizes K=%lld N=%lld", (long long)K, (long long)N);
  if (N == 0) return FL_OK;
  FL_REQUIRE(b_period > 0 && b_period <= N && N % b_period == 0, FL_EBADSHAPE,
             "fl_binary: b_period %lld does not divide N %lld", (long long)b_period, (long long)N);
  FL_REQUIRE(a && b && y && lap_y && (K == 0 || jac_y), FL_EBADSHAPE, "fl_binary: null pointer");
  // an operand is a triplet iff its lap pointer is given; its jac may be NULL only when K == 0
  FL_REQUIRE((lap_a != nullptr || jac_a == nullptr) && (lap_b != nullptr || jac_b == nullptr) &&
                 (K == 0 || ((lap_a == nullptr) == (jac_a == nullptr) &&
                             (lap_b == nullptr) == (jac_b == nullptr))),
             FL_EBADSHAPE, "fl_binary: jac and lap of an operand must both be given or both NULL");
  cudaStream_t st = (cudaStream_t)stream;
  switch (op) {
    case FL_BIN_ADD:
      return dispatch<FL_BIN_ADD>(a, jac_a, lap_a, jac_a_stride, b, jac_b, lap_b, jac_b_stride, y,
                                  jac_y, lap_y, jac_y_stride, K, N, b_period, st);
    case FL_BIN_SUB:
      return dispatch<FL_BIN_SUB>(a, jac_a, lap_a, jac_a_stride, b, jac_b, lap_b, jac_b_stride, y,
                                  jac_y, lap_y, jac_y_stride, K, N, b_period, st);
    case FL_BIN_MUL:
      return dispatch<FL_BIN_MUL>(a, jac_a, lap_a, jac_a_stride, b, jac_b, lap_b, jac_b_stride, y,
                                  jac_y, lap_y, jac_y_stride, K, N, b_period, st);
    default:
      return dispatch<FL_BIN_DIV>(a, jac_a, lap_a, jac_a_stride, b, jac_b, lap_b, jac_b_stride, y,
                                  jac_y, lap_y, jac_y_stride, K, N, b_period, st);
  }
}
