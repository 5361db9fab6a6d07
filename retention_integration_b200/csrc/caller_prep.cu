// What the reference's callers do between their projection GEMM and the operator, in one pass:
//
//   deploy/nanoGPT/model.py:66-84        qkvg = c_attn(x); split into q, k, v and the gate column;
//                                        log_g = logsigmoid(6.906768 + gate.float()); rotary on q and k
//                                        (interleaved pairs, :153-164); .contiguous() copies
//   deploy/models/powercoder/modeling_powercoder.py:152-159
//                                        the same with separate projections, logsigmoid without a bias
//                                        and the half-split rotary of :43-74
//
// Unfused that is six elementwise kernels and two copies over tensors the size of the
// activations.  Here one kernel reads the projection output once and writes Q [b,t,hq,d],
// K, V [b,t,h,d] (16 bit) and log_g [b,t,h] (fp32) in the layout the operator takes; a second one
// is its gradient.  HBM bound: every thread moves 16-byte vectors, a token's row of the input is
// read by consecutive threads, cos / sin come from a small fp32 table [t, d/2] that stays in L2.
//
// Arithmetic as deploy/nanoGPT/model.py:159-164: x * cos and rotate(x) * sin are rounded fp32
// products, their sum is rounded once more, then cast to the input's dtype (no fused multiply-add,
// so that the 16-bit results are the reference's bit for bit).
#include <algorithm>

#include "host.cuh"
#include "sm100.cuh"

namespace pr {
namespace {

constexpr int kCpThreads = 256;

// numerically safe log(sigmoid(x)) = min(x, 0) - log1p(exp(-|x|))
__device__ __forceinline__ float log_sigmoid(float x) { return fminf(x, 0.f) - log1pf(__expf(-fabsf(x))); }

template <typename T>
__device__ __forceinline__ void unpack8(const uint4& v, float (&x)[8]) {
  const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
  for (int k = 0; k < 4; ++k) {
    const float2 p = Pack2<T>::to_f32(w[k]);
    x[2 * k] = p.x;
    x[2 * k + 1] = p.y;
  }
}
template <typename T>
__device__ __forceinline__ uint4 pack8(const float (&x)[8]) {
  return make_uint4(Pack2<T>::from_f32(x[0], x[1]), Pack2<T>::from_f32(x[2], x[3]), Pack2<T>::from_f32(x[4], x[5]),
                    Pack2<T>::from_f32(x[6], x[7]));
}

// y = x cos + rot(x) sin with rot(x)[2i] = -x[2i+1], rot(x)[2i+1] = x[2i]; sign = -1 gives the
// transpose (the gradient).  Each product and the sum rounded separately.
__device__ __forceinline__ void rotate_pair(float x0, float x1, float c, float s, float sign, float* y0, float* y1) {
  *y0 = __fadd_rn(__fmul_rn(x0, c), __fmul_rn(-sign * x1, s));
  *y1 = __fadd_rn(__fmul_rn(x1, c), __fmul_rn(sign * x0, s));
}

struct CallerPrepParams {
  int t, h, hq, d;
  long long in_stride;    // elements between consecutive tokens of the projection output
  long long cs_bstride;   // floats between batch entries of cos / sin (0: one table for all)
  int half_split;         // 0: pairs (2i, 2i+1); 1: pairs (i, i + d/2)
  int gated;
  float gate_bias;
  size_t tokens;          // b * t
};

// One work item = one 16-byte vector of q or k (a pair of vectors when the rotary pairs are
// half-split) or of v; consecutive threads take consecutive items, so a warp reads 512 contiguous
// bytes of a token's row and writes 512 contiguous bytes of Q, K or V.  The item number is split
// into (token, vector) with 32-bit arithmetic whenever the problem allows (IDX = unsigned): the
// 64-bit divisions of the general case cost as many issue slots as the rest of the item.
// GRAD: inputs are dQ, dK, dV, dlog_g and the saved projection output (for the gate's derivative);
// the output is the gradient with respect to the projection output.
template <typename T, bool GRAD, bool HALF, typename IDX>
__global__ void __launch_bounds__(kCpThreads, HALF ? 4 : 8)
caller_prep_kernel(const CallerPrepParams p, const T* __restrict__ in, const float* __restrict__ cosT,
                   const float* __restrict__ sinT, T* __restrict__ Q, T* __restrict__ K, T* __restrict__ V,
                   float* __restrict__ log_g, T* __restrict__ grad_in) {
  const int d = p.d, vpr = d / 8;                 // vectors per head row
  const int units_rot = HALF ? vpr / 2 : vpr;     // work items per rotated head row
  const int n_rot = (p.hq + p.h) * units_rot;     // q heads, then k heads: one contiguous span of the row
  const IDX per_tok = (IDX)(n_rot + p.h * vpr);
  const long long off_v = (long long)(p.hq + p.h) * d, off_g = off_v + (long long)p.h * d;
  const IDX total = (IDX)p.tokens * per_tok;
  const IDX step = (IDX)gridDim.x * kCpThreads;
  const float sign = GRAD ? -1.f : 1.f;
  for (IDX idx = (IDX)blockIdx.x * kCpThreads + threadIdx.x; idx < total; idx += step) {
    const IDX tok_i = idx / per_tok;
    const int u = (int)(idx - tok_i * per_tok);
    const size_t tok = tok_i;
    const T* row_in = in + tok * p.in_stride;
    T* row_g = GRAD ? grad_in + tok * p.in_stride : nullptr;
    if (u < n_rot) {
      const int head = u / units_rot, j = u - head * units_rot;
      const bool is_q = head < p.hq;
      const long long col = (long long)head * d + j * 8;
      T* dense = (is_q ? Q + (tok * p.hq + head) * d : K + (tok * p.h + (head - p.hq)) * d) + j * 8;
      const IDX batch = tok_i / (IDX)p.t;
      const size_t trow = (size_t)batch * p.cs_bstride + (size_t)(tok_i - batch * (IDX)p.t) * (d / 2) + (HALF ? j * 8 : j * 4);
      const T* src = GRAD ? dense : row_in + col;
      T* dst = GRAD ? row_g + col : dense;
      if (!HALF) {
        const uint4 v = *reinterpret_cast<const uint4*>(src);
        const float4 c4 = *reinterpret_cast<const float4*>(cosT + trow), s4 = *reinterpret_cast<const float4*>(sinT + trow);
        float x[8], y[8];
        unpack8<T>(v, x);
        const float c[4] = {c4.x, c4.y, c4.z, c4.w}, s[4] = {s4.x, s4.y, s4.z, s4.w};
#pragma unroll
        for (int e = 0; e < 4; ++e) rotate_pair(x[2 * e], x[2 * e + 1], c[e], s[e], sign, &y[2 * e], &y[2 * e + 1]);
        *reinterpret_cast<uint4*>(dst) = pack8<T>(y);
      } else {
        // elements 8j..8j+7 pair with 8j + d/2 .. 8j + d/2 + 7
        const uint4 va = *reinterpret_cast<const uint4*>(src), vb = *reinterpret_cast<const uint4*>(src + d / 2);
        float c[8], s[8], x0[8], x1[8], y0[8], y1[8];
        *reinterpret_cast<float4*>(c) = *reinterpret_cast<const float4*>(cosT + trow);
        *reinterpret_cast<float4*>(c + 4) = *reinterpret_cast<const float4*>(cosT + trow + 4);
        *reinterpret_cast<float4*>(s) = *reinterpret_cast<const float4*>(sinT + trow);
        *reinterpret_cast<float4*>(s + 4) = *reinterpret_cast<const float4*>(sinT + trow + 4);
        unpack8<T>(va, x0);
        unpack8<T>(vb, x1);
#pragma unroll
        for (int e = 0; e < 8; ++e) rotate_pair(x0[e], x1[e], c[e], s[e], sign, &y0[e], &y1[e]);
        *reinterpret_cast<uint4*>(dst) = pack8<T>(y0);
        *reinterpret_cast<uint4*>(dst + d / 2) = pack8<T>(y1);
      }
    } else {
      const int w = u - n_rot;            // vector of the token's value span
      const int head = w / vpr;
      T* dense = V + tok * ((size_t)p.h * d) + (size_t)w * 8;
      if (GRAD)
        *reinterpret_cast<uint4*>(row_g + off_v + (long long)w * 8) = *reinterpret_cast<const uint4*>(dense);
      else
        *reinterpret_cast<uint4*>(dense) = *reinterpret_cast<const uint4*>(row_in + off_v + (long long)w * 8);
      // the token's gate columns ride with the first vector of each value head: one gate per thread
      if (p.gated && w - head * vpr == 0) {
        const float pre = float(row_in[off_g + head]) + p.gate_bias;
        if (GRAD) {
          // d/dx log sigmoid(x) = sigmoid(-x)
          const float sg = 1.f / (1.f + __expf(pre));
          row_g[off_g + head] = T(log_g[tok * p.h + head] * sg);
        } else {
          log_g[tok * p.h + head] = log_sigmoid(pre);
        }
      }
    }
  }
}

template <typename T>
int launch_caller_prep(bool grad, const CallerPrepParams& p, const void* in, const float* cosT, const float* sinT, void* Q,
                       void* K, void* V, float* log_g, void* grad_in, cudaStream_t s) {
  const int vpr = p.d / 8, ur = p.half_split ? vpr / 2 : vpr;
  const size_t per_tok = (size_t)(p.hq + p.h) * ur + (size_t)p.h * vpr;
  const size_t total = p.tokens * per_tok;
  // every thread takes a few items; the grid is a multiple of the SM count (eight CTAs resident per SM)
  int sms = 148, dev = 0;
  PR_CUDA(cudaGetDevice(&dev));
  PR_CUDA(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev));
  const size_t want = (total + kCpThreads - 1) / kCpThreads;
  const unsigned grid = (unsigned)std::min<size_t>(want, (size_t)sms * 32);
  const bool small = total + (size_t)grid * kCpThreads < ((size_t)1 << 32);  // the item counter may not wrap
#define PR_LAUNCH_CP(G, H)                                                                                         \
  do {                                                                                                             \
    if (small)                                                                                                     \
      caller_prep_kernel<T, G, H, unsigned><<<grid, kCpThreads, 0, s>>>(                                           \
          p, static_cast<const T*>(in), cosT, sinT, static_cast<T*>(Q), static_cast<T*>(K), static_cast<T*>(V),    \
          log_g, static_cast<T*>(grad_in));                                                                        \
    else                                                                                                           \
      caller_prep_kernel<T, G, H, unsigned long long><<<grid, kCpThreads, 0, s>>>(                                 \
          p, static_cast<const T*>(in), cosT, sinT, static_cast<T*>(Q), static_cast<T*>(K), static_cast<T*>(V),    \
          log_g, static_cast<T*>(grad_in));                                                                        \
  } while (0)
  if (grad) {
    if (p.half_split) PR_LAUNCH_CP(true, true); else PR_LAUNCH_CP(true, false);
  } else {
    if (p.half_split) PR_LAUNCH_CP(false, true); else PR_LAUNCH_CP(false, false);
  }
#undef PR_LAUNCH_CP
  PR_CUDA(cudaGetLastError());
  return PR_OK;
}

int check_caller_prep(int dtype, int b, int t, int h, int hq, int d, long long in_stride, int gated, int half_split) {
  PR_REQUIRE(dtype == PR_BF16 || dtype == PR_FP16, PR_ERR_BAD_ARG, "dtype %d", dtype);
  PR_REQUIRE(b > 0 && t > 0 && h > 0 && hq > 0 && hq % h == 0, PR_ERR_BAD_ARG, "bad sizes b=%d t=%d h=%d hq=%d", b, t, h, hq);
  PR_REQUIRE(d % 8 == 0 && d >= 8 && (!half_split || d % 16 == 0), PR_ERR_BAD_ARG, "head dim %d", d);
  const long long need = (long long)(hq + 2 * h) * d + (gated ? h : 0);
  PR_REQUIRE(in_stride >= need && in_stride % 8 == 0, PR_ERR_BAD_ARG,
             "row stride %lld: at least %lld elements and a multiple of 8", in_stride, need);
  return PR_OK;
}

}  // namespace
}  // namespace pr

extern "C" int pr_caller_prep_fwd(int dtype, int b, int t, int h, int hq, int d, const void* qkvg, long long row_stride,
                                  const float* cos_table, const float* sin_table, long long table_bstride,
                                  int half_split, int gated, float gate_bias, void* Q, void* K, void* V, float* log_g,
                                  int device, void* stream) {
  using namespace pr;
  int rc = check_caller_prep(dtype, b, t, h, hq, d, row_stride, gated, half_split);
  if (rc) return rc;
  PR_REQUIRE(qkvg && cos_table && sin_table && Q && K && V && (!gated || log_g), PR_ERR_BAD_ARG, "null pointer");
  PR_REQUIRE(aligned16(qkvg) && aligned16(cos_table) && aligned16(sin_table) && aligned16(Q) && aligned16(K) &&
                 aligned16(V) && table_bstride % 4 == 0,
             PR_ERR_BAD_ARG, "misaligned pointer");
  PR_CUDA(cudaSetDevice(device));
  CallerPrepParams p{t, h, hq, d, row_stride, table_bstride, half_split, gated, gate_bias, (size_t)b * t};
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  return dtype == PR_BF16
             ? launch_caller_prep<__nv_bfloat16>(false, p, qkvg, cos_table, sin_table, Q, K, V, log_g, nullptr, s)
             : launch_caller_prep<__half>(false, p, qkvg, cos_table, sin_table, Q, K, V, log_g, nullptr, s);
}

extern "C" int pr_caller_prep_bwd(int dtype, int b, int t, int h, int hq, int d, const void* qkvg, long long row_stride,
                                  const float* cos_table, const float* sin_table, long long table_bstride,
                                  int half_split, int gated, float gate_bias, const void* dQ, const void* dK,
                                  const void* dV, const float* dlog_g, void* dqkvg, int device, void* stream) {
  using namespace pr;
  int rc = check_caller_prep(dtype, b, t, h, hq, d, row_stride, gated, half_split);
  if (rc) return rc;
  PR_REQUIRE(qkvg && cos_table && sin_table && dQ && dK && dV && dqkvg && (!gated || dlog_g), PR_ERR_BAD_ARG,
             "null pointer");
  PR_REQUIRE(aligned16(qkvg) && aligned16(cos_table) && aligned16(sin_table) && aligned16(dQ) && aligned16(dK) &&
                 aligned16(dV) && aligned16(dqkvg) && table_bstride % 4 == 0,
             PR_ERR_BAD_ARG, "misaligned pointer");
  PR_CUDA(cudaSetDevice(device));
  CallerPrepParams p{t, h, hq, d, row_stride, table_bstride, half_split, gated, gate_bias, (size_t)b * t};
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  // the kernel's Q, K, V, log_g arguments carry the incoming gradients in this direction
  void* q = const_cast<void*>(dQ);
  void* k = const_cast<void*>(dK);
  void* v = const_cast<void*>(dV);
  float* g = const_cast<float*>(dlog_g);
  return dtype == PR_BF16 ? launch_caller_prep<__nv_bfloat16>(true, p, qkvg, cos_table, sin_table, q, k, v, g, dqkvg, s)
                          : launch_caller_prep<__half>(true, p, qkvg, cos_table, sin_table, q, k, v, g, dqkvg, s);
}
