// Split-fp32 products on the warp-level tensor-core instruction (mma.sync m16n8k8, TF32 operands,
// fp32 accumulation): v = hi + lo with hi = v truncated to TF32 and lo = v - hi, every product
// taken as lo*hi + hi*lo + hi*hi, so the result keeps fp32 accuracy.  Fragments are read straight
// from row-major shared-memory tiles; g = lane / 4 and t = lane % 4 throughout.
#pragma once

#include "common.cuh"

namespace fl {

struct FragA { uint32_t hi[4], lo[4]; };
struct FragB { uint32_t hi[2], lo[2]; };

__device__ __forceinline__ void split_tf32(float v, uint32_t& hi, uint32_t& lo) {
  hi = __float_as_uint(v) & 0xffffe000u;  // a valid TF32 number: the tensor core uses it as is
  lo = __float_as_uint(v - __uint_as_float(hi));
}

__device__ __forceinline__ void mma_tf32(float (&c)[4], const uint32_t (&a)[4], const uint32_t (&b)[2]) {
  asm volatile(
      "mma.sync.aligned.m16n8k8.row.col.f32.tf32.tf32.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, "
      "{%8, %9}, {%0, %1, %2, %3};"
      : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b[0]), "r"(b[1]));
}

__device__ __forceinline__ void mma3(float (&c)[4], const FragA& a, const FragB& b) {
  mma_tf32(c, a.lo, b.hi);
  mma_tf32(c, a.hi, b.lo);
  mma_tf32(c, a.hi, b.hi);
}

// A fragment (16 x 8) of the row-major tile X (pitch P): rows m0 .., columns k0 ..
template <int P>
__device__ __forceinline__ void load_a(FragA& f, const float* X, int m0, int k0, int g, int t) {
  const float* p = X + (m0 + g) * P + k0 + t;
  split_tf32(p[0], f.hi[0], f.lo[0]);
  split_tf32(p[8 * P], f.hi[1], f.lo[1]);
  split_tf32(p[4], f.hi[2], f.lo[2]);
  split_tf32(p[8 * P + 4], f.hi[3], f.lo[3]);
}
// B fragment (8 x 8) of the operand B[k][n] = X[n][k]: X row-major with pitch P
template <int P>
__device__ __forceinline__ void load_bt(FragB& f, const float* X, int n0, int k0, int g, int t) {
  const float* p = X + (n0 + g) * P + k0 + t;
  split_tf32(p[0], f.hi[0], f.lo[0]);
  split_tf32(p[4], f.hi[1], f.lo[1]);
}
// B fragment (8 x 8) of the operand B[k][n] = X[k][n]
template <int P>
__device__ __forceinline__ void load_b(FragB& f, const float* X, int k0, int n0, int g, int t) {
  const float* p = X + (k0 + t) * P + n0 + g;
  split_tf32(p[0], f.hi[0], f.lo[0]);
  split_tf32(p[4 * P], f.hi[1], f.lo[1]);
}

}  // namespace fl
