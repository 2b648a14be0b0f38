// One-pass LayerNorm forward-Laplacian rule over the feature axis.
//
// The reference evaluates LayerNorm as a chain of registry rules (reduce_sum, sub, square, add,
// rsqrt, mul, div: folx/wrapped_functions.py:364-391, 409 with folx/custom_hessian.py:35-59 for
// the division), each a full pass over the Jacobian.  Their composition has the closed form
//   c = x - mean(x), r = (mean(c^2) + eps)^-1/2, z = c r,
//   u_k = r (J_k - mean(J_k)), b_k = mean(z u_k), lc = lap - mean(lap),
//   Jz_k  = u_k - z b_k,
//   lap_z = r (lc - z mean(z lc)) + sum_k [ -2 b_k u_k + z (3 b_k^2 - mean(u_k^2)) ],
//   y = gamma z + beta, J_y = gamma Jz, lap_y = gamma lap_z,
// with all means taken over the F features of one position.  One warp owns one position: the
// feature reductions are warp shuffles, the K Jacobian rows stream through registers once.
// HBM-bound; algorithmic traffic 8 (K + 2) P F bytes.
#include "common.cuh"

namespace fl {
namespace {

constexpr int kWarpsPerBlock = 8;
constexpr int kRowUnroll = 4;

__device__ __forceinline__ float hsum(float4 v) { return (v.x + v.y) + (v.z + v.w); }
__device__ __forceinline__ float hdot(float4 a, float4 b) {
  return fmaf(a.x, b.x, fmaf(a.y, b.y, fmaf(a.z, b.z, a.w * b.w)));
}

// F == 128 * VPL: lane l holds float4 number l + 32 j of the row, j < VPL.
// TWO: the input is the sum a + c2 * b of two triplets (a residual connection feeding the
// normalisation), added while loading: x2 / jac2 / lap2 with K2 <= K rows, row stride js2_4.
__device__ __forceinline__ float4 axpy4(float4 a, float c, float4 b) {
  return make_float4(fmaf(c, b.x, a.x), fmaf(c, b.y, a.y), fmaf(c, b.z, a.z), fmaf(c, b.w, a.w));
}

// SPLIT > 1: SPLIT consecutive warps of a block share one position and take K / SPLIT Jacobian
// rows each (every one of them recomputes the statistics of x); their partial sums meet in shared
// memory before the Laplacian row is written.  Used when there are too few positions to fill the
// machine with one warp each.
template <int VPL, bool TWO, int SPLIT>
__global__ void __launch_bounds__(kWarpsPerBlock * 32)
layernorm_rows(const float4* __restrict__ x, const float4* __restrict__ jac,
               const float4* __restrict__ lap, const float4* __restrict__ gamma,
               const float4* __restrict__ beta, float eps, float4* __restrict__ y,
               float4* __restrict__ jy, float4* __restrict__ ly, int64_t P, int K, int64_t js4,
               int64_t jys4, const float4* __restrict__ x2, const float4* __restrict__ jac2,
               const float4* __restrict__ lap2, int K2, int64_t js2_4, float c2) {
  const int lane = threadIdx.x & 31;
  const int wib = threadIdx.x >> 5;
  const int part = wib % SPLIT;
  const int64_t p_raw = (int64_t)blockIdx.x * (kWarpsPerBlock / SPLIT) + wib / SPLIT;
  if (SPLIT == 1 && p_raw >= P) return;
  // with SPLIT > 1 every warp reaches the block barrier: out-of-range warps redo the last position
  // and write nothing
  const bool live = p_raw < P;
  const int64_t p = live ? p_raw : P - 1;
  constexpr int F4 = 32 * VPL;
  const float invF = 1.0f / (float)(F4 * 4);
  const int64_t row = p * F4;

  float4 z[VPL], g[VPL];
  float s = 0.f;
#pragma unroll
  for (int j = 0; j < VPL; ++j) {
    z[j] = ld_stream(x + row + lane + 32 * j);
    if constexpr (TWO) z[j] = axpy4(z[j], c2, ld_stream(x2 + row + lane + 32 * j));
    s += hsum(z[j]);
    g[j] = gamma ? __ldg(gamma + lane + 32 * j) : make_float4(1.f, 1.f, 1.f, 1.f);
  }
  const float mean = warp_sum(s) * invF;
  float q = 0.f;
#pragma unroll
  for (int j = 0; j < VPL; ++j) {
    z[j].x -= mean; z[j].y -= mean; z[j].z -= mean; z[j].w -= mean;
    q += hdot(z[j], z[j]);
  }
  const float r = rsqrtf(warp_sum(q) * invF + eps);
#pragma unroll
  for (int j = 0; j < VPL; ++j) {
    z[j].x *= r; z[j].y *= r; z[j].z *= r; z[j].w *= r;
    if (part == 0 && live) {
      float4 bt = beta ? __ldg(beta + lane + 32 * j) : make_float4(0.f, 0.f, 0.f, 0.f);
      st_stream(y + row + lane + 32 * j,
                make_float4(fmaf(g[j].x, z[j].x, bt.x), fmaf(g[j].y, z[j].y, bt.y),
                            fmaf(g[j].z, z[j].z, bt.z), fmaf(g[j].w, z[j].w, bt.w)));
    }
  }

  float4 s1[VPL];  // sum_k b_k u_k
#pragma unroll
  for (int j = 0; j < VPL; ++j) s1[j] = make_float4(0.f, 0.f, 0.f, 0.f);
  float s2 = 0.f;  // sum_k (3 b_k^2 - mean(u_k^2))

  auto process = [&](float4 (&v)[VPL], int64_t k) {
    float t = 0.f;
#pragma unroll
    for (int j = 0; j < VPL; ++j) t += hsum(v[j]);
    const float m = warp_sum(t) * invF;
    float tb = 0.f, tq = 0.f;
#pragma unroll
    for (int j = 0; j < VPL; ++j) {
      v[j].x = r * (v[j].x - m); v[j].y = r * (v[j].y - m);
      v[j].z = r * (v[j].z - m); v[j].w = r * (v[j].w - m);
      tb += hdot(z[j], v[j]);
      tq += hdot(v[j], v[j]);
    }
    const float b = warp_sum(tb) * invF;
    const float uu = warp_sum(tq) * invF;
    s2 += 3.0f * b * b - uu;
    float4* out = jy + k * jys4 + row + lane;
#pragma unroll
    for (int j = 0; j < VPL; ++j) {
      s1[j].x = fmaf(b, v[j].x, s1[j].x); s1[j].y = fmaf(b, v[j].y, s1[j].y);
      s1[j].z = fmaf(b, v[j].z, s1[j].z); s1[j].w = fmaf(b, v[j].w, s1[j].w);
      if (SPLIT == 1 || live)
        st_stream(out + 32 * j, make_float4(g[j].x * (v[j].x - z[j].x * b), g[j].y * (v[j].y - z[j].y * b),
                                          g[j].z * (v[j].z - z[j].z * b), g[j].w * (v[j].w - z[j].w * b)));
    }
  };

  // rows [k, k_end) of this warp's share
  const int per = (K + SPLIT - 1) / SPLIT;
  int k = part * per;
  const int k_end = min(K, k + per);
  for (; k + kRowUnroll <= k_end; k += kRowUnroll) {
    float4 v[kRowUnroll][VPL];
#pragma unroll
    for (int u = 0; u < kRowUnroll; ++u)
#pragma unroll
      for (int j = 0; j < VPL; ++j) {
        v[u][j] = ld_stream(jac + (int64_t)(k + u) * js4 + row + lane + 32 * j);
        if constexpr (TWO)
          if (k + u < K2)
            v[u][j] = axpy4(v[u][j], c2, ld_stream(jac2 + (int64_t)(k + u) * js2_4 + row + lane + 32 * j));
      }
#pragma unroll
    for (int u = 0; u < kRowUnroll; ++u) process(v[u], k + u);
  }
  for (; k < k_end; ++k) {
    float4 v[VPL];
#pragma unroll
    for (int j = 0; j < VPL; ++j) {
      v[j] = ld_stream(jac + (int64_t)k * js4 + row + lane + 32 * j);
      if constexpr (TWO)
        if (k < K2) v[j] = axpy4(v[j], c2, ld_stream(jac2 + (int64_t)k * js2_4 + row + lane + 32 * j));
    }
    process(v, k);
  }

  if constexpr (SPLIT > 1) {
    __shared__ float4 sh1[kWarpsPerBlock][VPL * 32];
    __shared__ float sh2[kWarpsPerBlock];
    if (part != 0) {
#pragma unroll
      for (int j = 0; j < VPL; ++j) sh1[wib][lane + 32 * j] = s1[j];
      if (lane == 0) sh2[wib] = s2;
    }
    __syncthreads();
    if (part != 0 || !live) return;
#pragma unroll
    for (int o = 1; o < SPLIT; ++o) {
#pragma unroll
      for (int j = 0; j < VPL; ++j) {
        const float4 a = sh1[wib + o][lane + 32 * j];
        s1[j].x += a.x; s1[j].y += a.y; s1[j].z += a.z; s1[j].w += a.w;
      }
      s2 += sh2[wib + o];
    }
  }

  float4 l[VPL];
  float t = 0.f;
#pragma unroll
  for (int j = 0; j < VPL; ++j) {
    l[j] = ld_stream(lap + row + lane + 32 * j);
    if constexpr (TWO) l[j] = axpy4(l[j], c2, ld_stream(lap2 + row + lane + 32 * j));
    t += hsum(l[j]);
  }
  const float lm = warp_sum(t) * invF;
  float tz = 0.f;
#pragma unroll
  for (int j = 0; j < VPL; ++j) {
    l[j].x -= lm; l[j].y -= lm; l[j].z -= lm; l[j].w -= lm;
    tz += hdot(z[j], l[j]);
  }
  const float zl = warp_sum(tz) * invF;
#pragma unroll
  for (int j = 0; j < VPL; ++j) {
    float4 o;
    o.x = g[j].x * (r * (l[j].x - z[j].x * zl) - 2.0f * s1[j].x + z[j].x * s2);
    o.y = g[j].y * (r * (l[j].y - z[j].y * zl) - 2.0f * s1[j].y + z[j].y * s2);
    o.z = g[j].z * (r * (l[j].z - z[j].z * zl) - 2.0f * s1[j].z + z[j].z * s2);
    o.w = g[j].w * (r * (l[j].w - z[j].w * zl) - 2.0f * s1[j].w + z[j].w * s2);
    st_stream(ly + row + lane + 32 * j, o);
  }
}

// Any F: lanes stride over the features; z and the running sums live in shared memory.
__global__ void __launch_bounds__(kWarpsPerBlock * 32)
layernorm_rows_generic(const float* __restrict__ x, const float* __restrict__ jac,
                       const float* __restrict__ lap, const float* __restrict__ gamma,
                       const float* __restrict__ beta, float eps, float* __restrict__ y,
                       float* __restrict__ jy, float* __restrict__ ly, int64_t P, int F, int K,
                       int64_t js, int64_t jys) {
  extern __shared__ float smem[];
  const int lane = threadIdx.x & 31;
  const int w = threadIdx.x >> 5;
  const int64_t p = (int64_t)blockIdx.x * kWarpsPerBlock + w;
  if (p >= P) return;
  float* z = smem + (size_t)w * 2 * F;
  float* s1 = z + F;
  const float invF = 1.0f / (float)F;
  const int64_t row = p * F;
  float s = 0.f;
  for (int f = lane; f < F; f += 32) s += x[row + f];
  const float mean = warp_sum(s) * invF;
  float q = 0.f;
  for (int f = lane; f < F; f += 32) {
    float c = x[row + f] - mean;
    q = fmaf(c, c, q);
  }
  const float r = rsqrtf(warp_sum(q) * invF + eps);
  for (int f = lane; f < F; f += 32) {
    float zz = (x[row + f] - mean) * r;
    z[f] = zz;
    s1[f] = 0.f;
    y[row + f] = fmaf(gamma ? gamma[f] : 1.f, zz, beta ? beta[f] : 0.f);
  }
  float s2 = 0.f;
  for (int k = 0; k < K; ++k) {
    const float* jr = jac + (int64_t)k * js + row;
    float t = 0.f;
    for (int f = lane; f < F; f += 32) t += jr[f];
    const float m = warp_sum(t) * invF;
    float tb = 0.f, tq = 0.f;
    for (int f = lane; f < F; f += 32) {
      float u = r * (jr[f] - m);
      tb = fmaf(z[f], u, tb);
      tq = fmaf(u, u, tq);
    }
    const float b = warp_sum(tb) * invF;
    const float uu = warp_sum(tq) * invF;
    s2 += 3.0f * b * b - uu;
    float* out = jy + (int64_t)k * jys + row;
    for (int f = lane; f < F; f += 32) {
      float u = r * (jr[f] - m);
      s1[f] = fmaf(b, u, s1[f]);
      out[f] = (gamma ? gamma[f] : 1.f) * (u - z[f] * b);
    }
  }
  float t = 0.f;
  for (int f = lane; f < F; f += 32) t += lap[row + f];
  const float lm = warp_sum(t) * invF;
  float tz = 0.f;
  for (int f = lane; f < F; f += 32) tz = fmaf(z[f], lap[row + f] - lm, tz);
  const float zl = warp_sum(tz) * invF;
  for (int f = lane; f < F; f += 32) {
    float lc = lap[row + f] - lm;
    ly[row + f] = (gamma ? gamma[f] : 1.f) * (r * (lc - z[f] * zl) - 2.0f * s1[f] + z[f] * s2);
  }
}

// Warps per position: 1 when the positions alone give every SM ~40 warps, else 2, and 4 only when
// there are very few positions (measured on B200 at K = 96: P = 4096 x 256 features 0.160 -> 0.144
// ms with 2; P = 512 x 1024 features 0.105 -> 0.076 ms with 4).
int pick_split(int64_t P, int64_t K) {
  const int64_t want = (int64_t)sm_count() * 40;
  if (P >= want || K < 8) return 1;
  if (4 * P >= want || K < 16) return 2;
  return 4;
}

template <int VPL, bool TWO>
void launch_rows(int split, int64_t P, cudaStream_t st, const float* x, const float* jac,
                 const float* lap, const float* gamma, const float* beta, float eps, float* y,
                 float* jac_y, float* lap_y, int K, int64_t js4, int64_t jys4, const float* x2,
                 const float* jac2, const float* lap2, int K2, int64_t js2_4, float c2) {
#define FL_LN_GO(S)                                                                               \
  layernorm_rows<VPL, TWO, S>                                                                     \
      <<<(unsigned)((P + kWarpsPerBlock / S - 1) / (kWarpsPerBlock / S)), kWarpsPerBlock * 32, 0, \
         st>>>((const float4*)x, (const float4*)jac, (const float4*)lap, (const float4*)gamma,    \
               (const float4*)beta, eps, (float4*)y, (float4*)jac_y, (float4*)lap_y, P, K, js4,   \
               jys4, (const float4*)x2, (const float4*)jac2, (const float4*)lap2, K2, js2_4, c2)
  if (split == 4) FL_LN_GO(4);
  else if (split == 2) FL_LN_GO(2);
  else FL_LN_GO(1);
#undef FL_LN_GO
}

}  // namespace
}  // namespace fl

extern "C" int32_t fl_layernorm(const float* x, const float* jac, const float* lap,
                                const float* gamma, const float* beta, float eps, float* y,
                                float* jac_y, float* lap_y, int64_t P, int64_t F, int64_t K,
                                int64_t jac_stride, int64_t jac_y_stride, void* stream) {
  using namespace fl;
  FL_REQUIRE(P >= 0 && F > 0 && K >= 0 && K < (1ll << 31) && F < (1ll << 20), FL_EBADSHAPE,
             "fl_layernorm: bad sizes P=%lld F=%lld K=%lld", (long long)P, (long long)F, (long long)K);
  FL_REQUIRE(K == 0 || (jac_stride >= P * F && jac_y_stride >= P * F), FL_EBADSHAPE,
             "fl_layernorm: Jacobian row stride smaller than P*F");
  if (P == 0) return FL_OK;
  FL_REQUIRE(x && lap && y && lap_y && (K == 0 || (jac && jac_y)), FL_EBADSHAPE,
             "fl_layernorm: null pointer");
  cudaStream_t st = (cudaStream_t)stream;
  int64_t blocks = (P + kWarpsPerBlock - 1) / kWarpsPerBlock;
  FL_REQUIRE(blocks < (1ll << 31), FL_EBADSHAPE, "fl_layernorm: P too large");
  bool vec = (F % 128 == 0) && F <= 1024 && (K <= 1 || (jac_stride % 4 == 0 && jac_y_stride % 4 == 0)) &&
             aligned16(x) && aligned16(lap) && aligned16(y) && aligned16(lap_y) &&
             (K == 0 || (aligned16(jac) && aligned16(jac_y))) && (!gamma || aligned16(gamma)) &&
             (!beta || aligned16(beta));
  if (vec) {
    const int split = pick_split(P, K);
#define FL_LN(V)                                                                                  \
  case V:                                                                                         \
    launch_rows<V, false>(split, P, st, x, jac, lap, gamma, beta, eps, y, jac_y, lap_y, (int)K,   \
                          jac_stride / 4, jac_y_stride / 4, nullptr, nullptr, nullptr, 0, 0, 0.f); \
    break;
    switch ((int)(F / 128)) {
      FL_LN(1) FL_LN(2) FL_LN(3) FL_LN(4) FL_LN(5) FL_LN(6) FL_LN(7) FL_LN(8)
    }
#undef FL_LN
  } else {
    size_t smem = (size_t)kWarpsPerBlock * 2 * F * sizeof(float);
    FL_REQUIRE(smem <= 200 * 1024, FL_EUNSUPPORTED, "fl_layernorm: F=%lld too wide", (long long)F);
    if (smem > 48 * 1024)
      FL_CUDA(cudaFuncSetAttribute(layernorm_rows_generic,
                                   cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    layernorm_rows_generic<<<(unsigned)blocks, kWarpsPerBlock * 32, smem, st>>>(
        x, jac, lap, gamma, beta, eps, y, jac_y, lap_y, P, (int)F, (int)K, jac_stride,
        jac_y_stride);
  }
  FL_CHECK_LAUNCH("fl_layernorm launch");
  return FL_OK;
}

extern "C" int32_t fl_add_layernorm(const float* x, const float* jac, const float* lap,
                                    const float* x2, const float* jac2, const float* lap2,
                                    int64_t K2, int64_t jac2_stride, float scale2,
                                    const float* gamma, const float* beta, float eps, float* y,
                                    float* jac_y, float* lap_y, int64_t P, int64_t F, int64_t K,
                                    int64_t jac_stride, int64_t jac_y_stride, void* stream) {
  using namespace fl;
  FL_REQUIRE(P >= 0 && F > 0 && K >= 0 && K2 >= 0 && K2 <= K && K < (1ll << 31), FL_EBADSHAPE,
             "fl_add_layernorm: bad sizes P=%lld F=%lld K=%lld K2=%lld", (long long)P, (long long)F,
             (long long)K, (long long)K2);
  if (P == 0) return FL_OK;
  FL_REQUIRE(x && lap && x2 && lap2 && y && lap_y && (K == 0 || (jac && jac_y)) && (K2 == 0 || jac2),
             FL_EBADSHAPE, "fl_add_layernorm: null pointer");
  FL_REQUIRE(K == 0 || (jac_stride >= P * F && jac_y_stride >= P * F), FL_EBADSHAPE,
             "fl_add_layernorm: Jacobian row stride smaller than P*F");
  FL_REQUIRE(K2 <= 1 || jac2_stride >= P * F, FL_EBADSHAPE,
             "fl_add_layernorm: second Jacobian row stride smaller than P*F");
  bool vec = (F % 128 == 0) && F <= 1024 && (K <= 1 || (jac_stride % 4 == 0 && jac_y_stride % 4 == 0)) &&
             (K2 <= 1 || jac2_stride % 4 == 0) && aligned16(x) && aligned16(lap) && aligned16(x2) &&
             aligned16(lap2) && aligned16(y) && aligned16(lap_y) &&
             (K == 0 || (aligned16(jac) && aligned16(jac_y))) && (K2 == 0 || aligned16(jac2)) &&
             (!gamma || aligned16(gamma)) && (!beta || aligned16(beta));
  FL_REQUIRE(vec, FL_EUNSUPPORTED,
             "fl_add_layernorm: needs F a multiple of 128 (<= 1024) and 16-byte aligned buffers");
  cudaStream_t st = (cudaStream_t)stream;
  int64_t blocks = (P + kWarpsPerBlock - 1) / kWarpsPerBlock;
  FL_REQUIRE(blocks < (1ll << 31), FL_EBADSHAPE, "fl_add_layernorm: P too large");
  const int split = pick_split(P, K);
#define FL_LN2(V)                                                                                 \
  case V:                                                                                         \
    launch_rows<V, true>(split, P, st, x, jac, lap, gamma, beta, eps, y, jac_y, lap_y, (int)K,    \
                         jac_stride / 4, jac_y_stride / 4, x2, jac2, lap2, (int)K2,               \
                         jac2_stride / 4, scale2);                                                \
    break;
  switch ((int)(F / 128)) {
    FL_LN2(1) FL_LN2(2) FL_LN2(3) FL_LN2(4) FL_LN2(5) FL_LN2(6) FL_LN2(7) FL_LN2(8)
  }
#undef FL_LN2
  FL_CHECK_LAUNCH("fl_add_layernorm launch");
  return FL_OK;
}
