// Sum of up to five triplets followed by an elementwise function, in one pass:
//     s = sum_t c_t a_t            (c_t = +1 / -1; a term may be broadcast or a constant)
//     y = f(s_x),  J_y[k] = f'(s_x) s_J[k],  lap_y = f'(s_x) s_lap + f''(s_x) sum_k s_J[k]^2
// The reference evaluates such an expression as a chain of `add` rules and one elementwise rule
// (folx/wrapped_functions.py:364-369, 384-431), each a full pass over the Jacobian that XLA may
// or may not fuse; here the chain `tanh(x W + pair + pooled)` of a FermiNet layer reads every
// operand once and writes the result once.  Terms with fewer Jacobian rows than the output are
// zero beyond their last row (dense Jacobians truncated at the highest referenced input,
// folx/api.py:182-196, folx/utils.py:432-450).  HBM-bound.
#include "common.cuh"

namespace fl {
namespace {

constexpr int kMaxTerms = FL_ADDN_MAX_TERMS;

struct Terms {
  int n;
  const float* x[kMaxTerms];
  const float* jac[kMaxTerms];
  const float* lap[kMaxTerms];
  int64_t js[kMaxTerms];     // Jacobian row stride (elements, or float4 units in the vector kernel)
  int K[kMaxTerms];          // Jacobian rows of the term (0 for a constant)
  int64_t inner[kMaxTerms];  // broadcast: term position = (i / (inner * mid)) * inner + i % inner
  int64_t mid[kMaxTerms];
  float scale[kMaxTerms];
};

struct D3 { float y, d1, d2; };

// identity plus the nonlinearities that follow sums in the benchmark networks; everything else
// goes through fl_elementwise after a plain sum
__device__ __forceinline__ D3 act(int op, float x) {
  D3 r;
  if (op == FL_ADDN_TANH) {
    r.y = tanhf(x);
    r.d1 = 1.0f - r.y * r.y;
    r.d2 = -2.0f * r.y * r.d1;
  } else if (op == FL_ADDN_SILU) {
    float s = 1.0f / (1.0f + expf(-x));
    r.y = x * s;
    r.d1 = s * (1.0f + x * (1.0f - s));
    r.d2 = s * (1.0f - s) * (2.0f + x * (1.0f - 2.0f * s));
  } else if (op == FL_ADDN_EXP) {
    r.y = expf(x); r.d1 = r.y; r.d2 = r.y;
  } else {
    r.y = x; r.d1 = 1.0f; r.d2 = 0.0f;
  }
  return r;
}

template <bool RES>
__global__ void __launch_bounds__(256)
addn_vec4(int fop, Terms t, float4* __restrict__ y, float4* __restrict__ jy, float4* __restrict__ ly,
          int64_t jys, int K, int64_t n4) {
  const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n4) return;
  // RES: the last term stays outside the function, y = f(sum of the others) + last
  const int nf = RES ? t.n - 1 : t.n;
  int64_t pos[kMaxTerms];
  const float4 zero = make_float4(0.f, 0.f, 0.f, 0.f);
  float4 sx = zero, sl = zero, rx = zero, rl = zero;
#pragma unroll
  for (int q = 0; q < kMaxTerms; ++q) {
    if (q < t.n) {
      pos[q] = (t.mid[q] == 1) ? i : (i / (t.inner[q] * t.mid[q])) * t.inner[q] + i % t.inner[q];
      const float c = t.scale[q];
      float4 v = __ldg(reinterpret_cast<const float4*>(t.x[q]) + pos[q]);
      float4 w = t.lap[q] ? __ldg(reinterpret_cast<const float4*>(t.lap[q]) + pos[q]) : zero;
      if (!RES || q < nf) {
        sx.x = fmaf(c, v.x, sx.x); sx.y = fmaf(c, v.y, sx.y); sx.z = fmaf(c, v.z, sx.z); sx.w = fmaf(c, v.w, sx.w);
        sl.x = fmaf(c, w.x, sl.x); sl.y = fmaf(c, w.y, sl.y); sl.z = fmaf(c, w.z, sl.z); sl.w = fmaf(c, w.w, sl.w);
      } else {
        rx = make_float4(c * v.x, c * v.y, c * v.z, c * v.w);
        rl = make_float4(c * w.x, c * w.y, c * w.z, c * w.w);
      }
    }
  }
  const D3 a = act(fop, sx.x), b = act(fop, sx.y), c = act(fop, sx.z), d = act(fop, sx.w);
  st_stream(y + i, make_float4(a.y + rx.x, b.y + rx.y, c.y + rx.z, d.y + rx.w));
  float4 acc = zero;
  // two Jacobian rows per trip: all their loads are issued before the first use
  for (int k = 0; k < K; k += 2) {
    float4 v[2][kMaxTerms];
#pragma unroll
    for (int u = 0; u < 2; ++u)
#pragma unroll
      for (int q = 0; q < kMaxTerms; ++q)
        v[u][q] = (q < t.n && k + u < t.K[q])
                      ? __ldcs(reinterpret_cast<const float4*>(t.jac[q]) + (int64_t)(k + u) * t.js[q] + pos[q])
                      : zero;
#pragma unroll
    for (int u = 0; u < 2; ++u) {
      if (k + u < K) {
        float4 s = zero, r = zero;
#pragma unroll
        for (int q = 0; q < kMaxTerms; ++q) {
          const float cq = t.scale[q];  // 0 for the unused slots
          const float4 w = v[u][q];
          if (!RES || q < nf) {
            s.x = fmaf(cq, w.x, s.x); s.y = fmaf(cq, w.y, s.y); s.z = fmaf(cq, w.z, s.z); s.w = fmaf(cq, w.w, s.w);
          } else if (q < t.n) {
            r = make_float4(cq * w.x, cq * w.y, cq * w.z, cq * w.w);
          }
        }
        acc.x = fmaf(s.x, s.x, acc.x); acc.y = fmaf(s.y, s.y, acc.y);
        acc.z = fmaf(s.z, s.z, acc.z); acc.w = fmaf(s.w, s.w, acc.w);
        st_stream(jy + (int64_t)(k + u) * jys + i, make_float4(fmaf(a.d1, s.x, r.x), fmaf(b.d1, s.y, r.y),
                                                               fmaf(c.d1, s.z, r.z), fmaf(d.d1, s.w, r.w)));
      }
    }
  }
  st_stream(ly + i, make_float4(fmaf(a.d2, acc.x, fmaf(a.d1, sl.x, rl.x)), fmaf(b.d2, acc.y, fmaf(b.d1, sl.y, rl.y)),
                                fmaf(c.d2, acc.z, fmaf(c.d1, sl.z, rl.z)), fmaf(d.d2, acc.w, fmaf(d.d1, sl.w, rl.w))));
}

template <bool RES>
__global__ void __launch_bounds__(256)
addn_scalar(int fop, Terms t, float* __restrict__ y, float* __restrict__ jy, float* __restrict__ ly,
            int64_t jys, int K, int64_t n) {
  const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n) return;
  const int nf = RES ? t.n - 1 : t.n;
  int64_t pos[kMaxTerms];
  float sx = 0.f, sl = 0.f, rx = 0.f, rl = 0.f;
#pragma unroll
  for (int q = 0; q < kMaxTerms; ++q) {
    if (q < t.n) {
      pos[q] = (t.mid[q] == 1) ? i : (i / (t.inner[q] * t.mid[q])) * t.inner[q] + i % t.inner[q];
      const float v = t.scale[q] * t.x[q][pos[q]];
      const float w = t.lap[q] ? t.scale[q] * t.lap[q][pos[q]] : 0.f;
      if (q < nf) { sx += v; sl += w; } else { rx = v; rl = w; }
    }
  }
  const D3 a = act(fop, sx);
  y[i] = a.y + rx;
  float acc = 0.f;
  for (int k = 0; k < K; ++k) {
    float s = 0.f, r = 0.f;
#pragma unroll
    for (int q = 0; q < kMaxTerms; ++q)
      if (q < t.n && k < t.K[q]) {
        const float v = t.scale[q] * t.jac[q][(int64_t)k * t.js[q] + pos[q]];
        if (q < nf) s += v; else r = v;
      }
    acc = fmaf(s, s, acc);
    jy[(int64_t)k * jys + i] = fmaf(a.d1, s, r);
  }
  ly[i] = fmaf(a.d2, acc, fmaf(a.d1, sl, rl));
}

}  // namespace
}  // namespace fl

extern "C" int32_t fl_addn_elementwise(int32_t op, int32_t n_terms, const FlAddnTerm* terms, float* y,
                                       float* jac_y, float* lap_y, int64_t K, int64_t N,
                                       int64_t jac_y_stride, void* stream) {
  using namespace fl;
  FL_REQUIRE(op >= FL_ADDN_IDENTITY && op <= FL_ADDN_EXP_RESIDUAL, FL_EUNSUPPORTED,
             "fl_addn_elementwise: unknown op %d", op);
  FL_REQUIRE(n_terms >= 1 && n_terms <= kMaxTerms && terms, FL_EBADSHAPE,
             "fl_addn_elementwise: between 1 and %d terms", kMaxTerms);
  FL_REQUIRE(op <= FL_ADDN_EXP || n_terms >= 2, FL_EBADSHAPE,
             "fl_addn_elementwise: a residual form needs at least two terms");
  FL_REQUIRE(K >= 0 && N >= 0 && K < (1ll << 31) && (N + 255) / 256 < (1ll << 31), FL_EBADSHAPE,
             "fl_addn_elementwise: bad sizes");
  if (N == 0) return FL_OK;
  FL_REQUIRE(y && lap_y && (K == 0 || jac_y), FL_EBADSHAPE, "fl_addn_elementwise: null output");
  Terms t;
  t.n = n_terms;
  bool vec = N % 4 == 0 && jac_y_stride % 4 == 0 && aligned16(y) && aligned16(lap_y) &&
             (K == 0 || aligned16(jac_y));
  for (int q = 0; q < n_terms; ++q) {
    const FlAddnTerm& s = terms[q];
    FL_REQUIRE(s.x != nullptr && s.K >= 0 && s.K <= K && (s.K == 0 || s.jac != nullptr), FL_EBADSHAPE,
               "fl_addn_elementwise: term %d is malformed", q);
    FL_REQUIRE(s.inner > 0 && s.mid > 0 && N % (s.inner * s.mid) == 0, FL_EBADSHAPE,
               "fl_addn_elementwise: broadcast of term %d does not tile N", q);
    t.x[q] = s.x; t.jac[q] = s.jac; t.lap[q] = s.lap; t.js[q] = s.jac_stride; t.K[q] = (int)s.K;
    t.inner[q] = s.inner; t.mid[q] = s.mid; t.scale[q] = s.scale;
    vec = vec && s.inner % 4 == 0 && s.jac_stride % 4 == 0 && aligned16(s.x) &&
          (!s.jac || aligned16(s.jac)) && (!s.lap || aligned16(s.lap));
  }
  for (int q = n_terms; q < kMaxTerms; ++q) {
    t.x[q] = nullptr; t.jac[q] = nullptr; t.lap[q] = nullptr; t.js[q] = 0; t.K[q] = 0;
    t.inner[q] = 1; t.mid[q] = 1; t.scale[q] = 0.f;
  }
  cudaStream_t st = (cudaStream_t)stream;
  const bool res = op > FL_ADDN_EXP;
  const int fop = res ? op - FL_ADDN_EXP : op;
  if (vec) {
    for (int q = 0; q < n_terms; ++q) { t.js[q] /= 4; t.inner[q] /= 4; }
    const int64_t n4 = N / 4;
    const unsigned blocks = (unsigned)((n4 + 255) / 256);
    if (res)
      addn_vec4<true><<<blocks, 256, 0, st>>>(fop, t, (float4*)y, (float4*)jac_y, (float4*)lap_y,
                                              jac_y_stride / 4, (int)K, n4);
    else
      addn_vec4<false><<<blocks, 256, 0, st>>>(fop, t, (float4*)y, (float4*)jac_y, (float4*)lap_y,
                                               jac_y_stride / 4, (int)K, n4);
  } else {
    const unsigned blocks = (unsigned)((N + 255) / 256);
    if (res) addn_scalar<true><<<blocks, 256, 0, st>>>(fop, t, y, jac_y, lap_y, jac_y_stride, (int)K, N);
    else addn_scalar<false><<<blocks, 256, 0, st>>>(fop, t, y, jac_y, lap_y, jac_y_stride, (int)K, N);
  }
  FL_CHECK_LAUNCH("fl_addn_elementwise launch");
  return FL_OK;
}
