// Gated prefix scan of chunk states over the chunk axis and its reverse-mode
// counterpart (the reference's discumsum, retention/_discumsum/reference.py:3-15,
// and the backward recurrence of retention/_discumsum/triton.py:104-204 with the gate
// index autograd actually yields).  Bandwidth-bound: each thread owns 8 consecutive
// 16-bit elements (one 128-bit access per chunk), keeps the running state in fp32
// registers and walks the chunk axis with the next loads already in flight.
//
//   forward :  Y[0] = carry_in (0 if absent);  Y[m+1] = Y[m]*exp(A[m]) + X[m]
//              writes Y[0..n_out-1]  (n_out = n: states entering each chunk, may alias X;
//              n_out = n+1: the reference's output with the trailing total)
//   backward:  G[n] = carry_in;  G[m] = dY[m] + exp(A[m]) * G[m+1]
//              dX[m] = w (.) G[m+1]  (may alias dY),  dA[m] += exp(A[m]) * <Y[m], G[m+1]>
#include "host.cuh"
#include "layout.cuh"
#include "sm100.cuh"

namespace pr {

constexpr int kScanThreads = 256;
// Chunks in flight per thread and CTAs per SM the kernels are compiled for: measured on the benchmark's shape,
// 4 chunks at three CTAs per SM (register cap 85) beat deeper unrolling at lower occupancy (forward 0.073 ms
// against 0.080, backward 0.101 against 0.119).
#ifndef PR_SCAN_UNROLL
#define PR_SCAN_UNROLL 4
#endif
constexpr int kScanUnroll = PR_SCAN_UNROLL;

// fewer CTAs than two per SM: the launch cannot fill the GPU with resident CTAs
inline bool few_ctas(long long ctas, int device) {
  int sms = 148;
  cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, device);
  return ctas < 2ll * sms;
}
#ifndef PR_SCAN_MINB
#define PR_SCAN_MINB 3
#endif

template <typename T>
__device__ __forceinline__ void unpack8(const uint4& v, float (&f)[8]) {
  const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
  for (int k = 0; k < 4; ++k) {
    const float2 p = Pack2<T>::to_f32(w[k]);
    f[2 * k] = p.x;
    f[2 * k + 1] = p.y;
  }
}
template <typename T>
__device__ __forceinline__ uint4 pack8(const float (&f)[8]) {
  uint4 v;
  v.x = Pack2<T>::from_f32(f[0], f[1]);
  v.y = Pack2<T>::from_f32(f[2], f[3]);
  v.z = Pack2<T>::from_f32(f[4], f[5]);
  v.w = Pack2<T>::from_f32(f[6], f[7]);
  return v;
}

// ---- Gram matrices (d x d fp32 per chunk): tiny, one thread per element.
// forward: Zg[m] (entering chunk m) as hi + lo 16-bit halves for the tensor cores,
// and optionally in fp32 for the backward dot product.
// Arguments of a Gram scan riding along with a state scan (extra CTAs of the same launch).
struct GramScanArgs {
  const float* in;      // G (forward) or dZg (backward); null: no Gram scan in this launch
  const float* zg;      // backward: Zg
  void* hi;
  void* lo;
  float* full;          // forward: optional fp32 copy
  const float* carry_in;
  float* carry_out;
  float* dA_part;       // backward
  int d;
};

template <typename T>
__device__ __forceinline__ void scan_gram_fwd_body(const float* __restrict__ G, T* __restrict__ hi, T* __restrict__ lo,
                                                   float* __restrict__ full, const float* __restrict__ A,
                                                   const float* __restrict__ carry_in, float* __restrict__ carry_out,
                                                   int n, int h, int E, int blk, int head, int batch) {
  const int e = blk * kScanThreads + threadIdx.x;
  if (e >= E) return;
  float run = carry_in ? carry_in[((size_t)batch * h + head) * E + e] : 0.f;
  for (int m = 0; m < n; ++m) {
    const size_t idx = (((size_t)batch * n + m) * h + head) * E + e;
    const float x = G[idx];
    const float g = __expf(A[((size_t)batch * n + m) * h + head]);
    const T hv = Pack2<T>::is_bf16 ? T(__float2bfloat16_rn(run)) : T(__float2half_rn(run));
    hi[idx] = hv;
    lo[idx] = T(run - float(hv));
    if (full) full[idx] = run;
    run = fmaf(run, g, x);
  }
  if (carry_out) carry_out[((size_t)batch * h + head) * E + e] = run;
}
template <typename T>
__global__ void __launch_bounds__(kScanThreads)
scan_gram_fwd_kernel(const float* __restrict__ G, T* __restrict__ hi, T* __restrict__ lo, float* __restrict__ full,
                     const float* __restrict__ A, const float* __restrict__ carry_in, float* __restrict__ carry_out,
                     int n, int h, int E) {
  scan_gram_fwd_body<T>(G, hi, lo, full, A, carry_in, carry_out, n, h, E, blockIdx.x, blockIdx.y, blockIdx.z);
}

// backward: dG[m] = Gamma[m+1] (+ its transpose: the consumer needs the symmetrised
// matrix) as hi + lo halves, and the gate-gradient partial sums.  One thread per matrix
// element; it carries the running gradient of its own element and of the mirrored one.
template <typename T>
__device__ __forceinline__ void scan_gram_bwd_body(const float* __restrict__ dZg, const float* __restrict__ Zg,
                                                   T* __restrict__ hi, T* __restrict__ lo, const float* __restrict__ A,
                                                   const float* __restrict__ carry_in, float* __restrict__ carry_out,
                                                   float* __restrict__ dA_part, int n, int h, int d, int blk, int nblk,
                                                   int head, int batch) {
  const int E = d * d;
  const int e = blk * 256 + threadIdx.x;
  const bool active = e < E;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int et = active ? (e % d) * d + e / d : 0;  // mirrored element
  const size_t cbase = ((size_t)batch * h + head) * E;
  float run = (active && carry_in) ? carry_in[cbase + e] : 0.f;
  float run_t = (active && carry_in) ? carry_in[cbase + et] : 0.f;
  float* part = dA_part + (((size_t)batch * h + head) * nblk * 8 + blk * 8 + warp) * n;
  // The loads of a chunk do not depend on the running gradient: four chunks' worth are issued
  // before the dependent chain of FMAs walks through them.
  constexpr int UN = 4;
  for (int m0 = n - 1; m0 >= 0; m0 -= UN) {
    float dz[UN], dzt[UN], zg[UN], gg[UN];
#pragma unroll
    for (int u = 0; u < UN; ++u) {
      const int m = m0 - u;
      dz[u] = dzt[u] = zg[u] = 0.f;
      gg[u] = 1.f;
      if (m >= 0) {
        const size_t base = (((size_t)batch * n + m) * h + head) * E;
        gg[u] = A[((size_t)batch * n + m) * h + head];
        if (active) {
          dz[u] = dZg[base + e];
          dzt[u] = dZg[base + et];
          zg[u] = Zg[base + e];
        }
      }
    }
#pragma unroll
    for (int u = 0; u < UN; ++u) {
      const int m = m0 - u;
      if (m < 0) break;
      const size_t base = (((size_t)batch * n + m) * h + head) * E;
      const float g = __expf(gg[u]);
      float dot = 0.f;
      if (active) {
        const float sym = run + run_t;
        const T hv = Pack2<T>::is_bf16 ? T(__float2bfloat16_rn(sym)) : T(__float2half_rn(sym));
        hi[base + e] = hv;
        lo[base + e] = T(sym - float(hv));
        dot = zg[u] * run * g;
        run = fmaf(run, g, dz[u]);
        run_t = fmaf(run_t, g, dzt[u]);
      }
#pragma unroll
      for (int off = 16; off > 0; off >>= 1) dot += __shfl_xor_sync(0xffffffffu, dot, off);
      if (lane == 0) part[m] = dot;
    }
  }
  if (active && carry_out) carry_out[cbase + e] = run;
}
template <typename T>
__global__ void __launch_bounds__(256)
scan_gram_bwd_kernel(const float* __restrict__ dZg, const float* __restrict__ Zg, T* __restrict__ hi,
                     T* __restrict__ lo, const float* __restrict__ A, const float* __restrict__ carry_in,
                     float* __restrict__ carry_out, float* __restrict__ dA_part, int n, int h, int d) {
  scan_gram_bwd_body<T>(dZg, Zg, hi, lo, A, carry_in, carry_out, dA_part, n, h, d, blockIdx.x, gridDim.x, blockIdx.y,
                        blockIdx.z);
}

// X, Y: [b, n(_out), h, E]; A: [b, n, h]; carries: [b, h, E] fp32
template <typename T, int UN>
__global__ void __launch_bounds__(kScanThreads, UN <= kScanUnroll ? PR_SCAN_MINB : 2)
scan_fwd_kernel(const T* X, T* Y, const float* __restrict__ A,  // X and Y may be the same buffer: no __restrict__
                const float* __restrict__ carry_in, float* __restrict__ carry_out, int n, int n_out, int h,
                size_t E, int state_blocks, GramScanArgs gram) {
  const int head = blockIdx.y, batch = blockIdx.z;
  if ((int)blockIdx.x >= state_blocks) {
    // the Gram matrices' scan rides along in the last CTAs of the grid: its 4096 serial chains per head would
    // otherwise be a launch of their own that does nothing but wait for memory
    scan_gram_fwd_body<T>(gram.in, static_cast<T*>(gram.hi), static_cast<T*>(gram.lo), gram.full, A, gram.carry_in,
                          gram.carry_out, n, h, gram.d * gram.d, (int)blockIdx.x - state_blocks, head, batch);
    return;
  }
  const size_t e0 = ((size_t)blockIdx.x * kScanThreads + threadIdx.x) * 8;
  if (e0 >= E) return;
  float run[8];
  if (carry_in != nullptr) {
    const float4* ci = reinterpret_cast<const float4*>(carry_in + ((size_t)batch * h + head) * E + e0);
    const float4 c0 = ci[0], c1 = ci[1];
    run[0] = c0.x; run[1] = c0.y; run[2] = c0.z; run[3] = c0.w;
    run[4] = c1.x; run[5] = c1.y; run[6] = c1.z; run[7] = c1.w;
  } else {
#pragma unroll
    for (int k = 0; k < 8; ++k) run[k] = 0.f;
  }
  const size_t in_stride = (size_t)h * E;
  const T* xin = X + ((size_t)batch * n * h + head) * E + e0;
  T* yout = Y ? Y + ((size_t)batch * n_out * h + head) * E + e0 : nullptr;
  const float* Ap = A + (size_t)batch * n * h + head;
  for (int m0 = 0; m0 < n; m0 += UN) {
    uint4 xv[UN];
    float g[UN];
#pragma unroll
    for (int u = 0; u < UN; ++u) {
      if (m0 + u < n) {
        xv[u] = *reinterpret_cast<const uint4*>(xin + (size_t)(m0 + u) * in_stride);
        g[u] = __expf(Ap[(size_t)(m0 + u) * h]);
      }
    }
#pragma unroll
    for (int u = 0; u < UN; ++u) {
      if (m0 + u < n) {
        if (yout) *reinterpret_cast<uint4*>(yout + (size_t)(m0 + u) * in_stride) = pack8<T>(run);
        float x[8];
        unpack8<T>(xv[u], x);
#pragma unroll
        for (int k = 0; k < 8; ++k) run[k] = fmaf(run[k], g[u], x[k]);
      }
    }
  }
  if (yout && n_out > n) *reinterpret_cast<uint4*>(yout + (size_t)n * in_stride) = pack8<T>(run);
  if (carry_out != nullptr) {
    float4* co = reinterpret_cast<float4*>(carry_out + ((size_t)batch * h + head) * E + e0);
    co[0] = make_float4(run[0], run[1], run[2], run[3]);
    co[1] = make_float4(run[4], run[5], run[6], run[7]);
  }
}

// dY, dX: [b, n, h, E] (may alias); Y: [b, n, h, E] states entering each chunk;
// dA_part: [b, h, 8 * gridDim.x, n] per-warp partial sums of exp(A[m]) * <Y[m], G[m+1]>.
// row_weights: apply the key-side weight (1 or 2) of expanded row (e / row_len) to dX.
template <typename T, int UN>
__global__ void __launch_bounds__(kScanThreads, UN <= kScanUnroll ? PR_SCAN_MINB : 2)
scan_bwd_kernel(const T* dY, const T* __restrict__ Y, T* dX, const float* __restrict__ A,  // dY may alias dX
                const float* __restrict__ carry_in, float* __restrict__ carry_out, float* __restrict__ dA_part, int n,
                int h, size_t E, int row_len, int row_weights, int state_blocks, GramScanArgs gram) {
  const int head = blockIdx.y, batch = blockIdx.z;
  if ((int)blockIdx.x >= state_blocks) {
    scan_gram_bwd_body<T>(gram.in, gram.zg, static_cast<T*>(gram.hi), static_cast<T*>(gram.lo), A, gram.carry_in,
                          gram.carry_out, gram.dA_part, n, h, gram.d, (int)blockIdx.x - state_blocks,
                          (int)gridDim.x - state_blocks, head, batch);
    return;
  }
  const size_t e0 = ((size_t)blockIdx.x * kScanThreads + threadIdx.x) * 8;
  const bool active = e0 < E;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  float run[8];
#pragma unroll
  for (int k = 0; k < 8; ++k) run[k] = 0.f;
  if (active && carry_in != nullptr) {
    const float4* ci = reinterpret_cast<const float4*>(carry_in + ((size_t)batch * h + head) * E + e0);
    const float4 c0 = ci[0], c1 = ci[1];
    run[0] = c0.x; run[1] = c0.y; run[2] = c0.z; run[3] = c0.w;
    run[4] = c1.x; run[5] = c1.y; run[6] = c1.z; run[7] = c1.w;
  }
  float wgt = 1.f;
  if (active && row_weights) {
    int a, b;
    ref_decode((int)(e0 / row_len), &a, &b);
    wgt = ref_key_weight(a, b);
  }
  const size_t stride = (size_t)h * E;
  const size_t base = ((size_t)batch * n * h + head) * E + e0;
  const float* Ap = A + (size_t)batch * n * h + head;
  const bool reduce_only = (dX == nullptr);
  // one partial per warp and chunk: no block-wide barrier inside the chunk loop
  float* part = reduce_only ? nullptr
                            : dA_part + (((size_t)batch * h + head) * state_blocks * (kScanThreads / 32) +
                                         blockIdx.x * (kScanThreads / 32) + warp) * n;
  for (int m0 = n - 1; m0 >= 0; m0 -= UN) {
    uint4 gv[UN], yv[UN];
    float g[UN];
#pragma unroll
    for (int u = 0; u < UN; ++u) {
      const int m = m0 - u;
      if (m >= 0 && active) {
        gv[u] = *reinterpret_cast<const uint4*>(dY + base + (size_t)m * stride);
        if (!reduce_only) yv[u] = *reinterpret_cast<const uint4*>(Y + base + (size_t)m * stride);
      }
      if (m >= 0) g[u] = __expf(Ap[(size_t)m * h]);
    }
#pragma unroll
    for (int u = 0; u < UN; ++u) {
      const int m = m0 - u;
      if (m < 0) continue;
      if (reduce_only) {
        // only the carry leaving this block of chunks is wanted
        if (active) {
          float dy[8];
          unpack8<T>(gv[u], dy);
#pragma unroll
          for (int k = 0; k < 8; ++k) run[k] = fmaf(run[k], g[u], dy[k]);
        }
        continue;
      }
      float dot = 0.f;
      if (active) {
        float o[8], y[8], dy[8];
#pragma unroll
        for (int k = 0; k < 8; ++k) o[k] = wgt * run[k];
        *reinterpret_cast<uint4*>(dX + base + (size_t)m * stride) = pack8<T>(o);
        unpack8<T>(yv[u], y);
        unpack8<T>(gv[u], dy);
#pragma unroll
        for (int k = 0; k < 8; ++k) {
          dot = fmaf(y[k], run[k], dot);
          run[k] = fmaf(run[k], g[u], dy[k]);
        }
      }
      dot *= g[u];
#pragma unroll
      for (int off = 16; off > 0; off >>= 1) dot += __shfl_xor_sync(0xffffffffu, dot, off);
      if (lane == 0) part[m] = dot;
    }
  }
  if (active && carry_out != nullptr) {
    float4* co = reinterpret_cast<float4*>(carry_out + ((size_t)batch * h + head) * E + e0);
    co[0] = make_float4(run[0], run[1], run[2], run[3]);
    co[1] = make_float4(run[4], run[5], run[6], run[7]);
  }
}

}  // namespace pr

namespace pr {
static int launch_scan_fwd(int dtype, int b, int n, int n_out, int h, long long E, const void* X, void* Y, const float* A,
                           const float* carry_in, float* carry_out, const GramScanArgs& gram, int device,
                           void* stream) {
  PR_REQUIRE(b > 0 && n > 0 && h > 0 && E > 0 && E % 8 == 0, PR_ERR_BAD_ARG, "bad sizes b=%d n=%d h=%d E=%lld", b, n,
             h, E);
  PR_REQUIRE(n_out == n || n_out == n + 1, PR_ERR_BAD_ARG, "n_out=%d must be n or n+1", n_out);
  PR_REQUIRE(n_out == n || X != Y, PR_ERR_BAD_ARG, "in-place scan needs n_out == n");
  PR_REQUIRE(X && A && aligned16(X) && aligned16(Y), PR_ERR_BAD_ARG, "null or misaligned pointer");
  PR_REQUIRE(Y != nullptr || carry_out != nullptr, PR_ERR_BAD_ARG, "neither an output nor a carry was requested");
  PR_REQUIRE(h <= 65535 && b <= 65535, PR_ERR_BAD_ARG, "h and b must be <= 65535");
  PR_REQUIRE(gram.in == nullptr || (gram.hi && gram.lo && gram.d > 0), PR_ERR_BAD_ARG, "Gram scan without outputs");
  PR_CUDA(cudaSetDevice(device));
  const int state_blocks = (int)((E / 8 + kScanThreads - 1) / kScanThreads);
  const int gram_blocks = gram.in ? (gram.d * gram.d + kScanThreads - 1) / kScanThreads : 0;
  dim3 grid((unsigned)(state_blocks + gram_blocks), h, b);
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  // Few CTAs (one or two heads per GPU: 80-160 CTAs of serial 64-chunk chains) cannot hide the memory latency
  // with four chunks of loads in flight per thread; they get eight (two CTAs per SM).
  const bool deep = few_ctas((long long)state_blocks * h * b, device);
#define PR_LAUNCH_SCAN_F(TT, UNV)                                                                              \
  scan_fwd_kernel<TT, UNV><<<grid, kScanThreads, 0, s>>>(static_cast<const TT*>(X), static_cast<TT*>(Y), A,     \
                                                         carry_in, carry_out, n, n_out, h, (size_t)E,          \
                                                         state_blocks, gram)
  if (dtype == PR_BF16) {
    if (deep) PR_LAUNCH_SCAN_F(__nv_bfloat16, 8); else PR_LAUNCH_SCAN_F(__nv_bfloat16, kScanUnroll);
  } else if (dtype == PR_FP16) {
    if (deep) PR_LAUNCH_SCAN_F(__half, 8); else PR_LAUNCH_SCAN_F(__half, kScanUnroll);
  } else {
    return fail(PR_ERR_BAD_ARG, "dtype %d", dtype);
  }
#undef PR_LAUNCH_SCAN_F
  PR_CUDA(cudaGetLastError());
  return PR_OK;
}
}  // namespace pr

extern "C" int pr_discumsum_fwd(int dtype, int b, int n, int n_out, int h, long long E, const void* X, void* Y,
                                const float* A, const float* carry_in, float* carry_out, int device, void* stream) {
  pr::GramScanArgs none = {};
  return pr::launch_scan_fwd(dtype, b, n, n_out, h, E, X, Y, A, carry_in, carry_out, none, device, stream);
}

// pr_discumsum_fwd (in place: n_out = n) and pr_gram_scan_fwd in ONE launch: the Gram scan takes the last CTAs.
extern "C" int pr_state_scan_fwd(int dtype, int b, int n, int h, int d, long long E, void* Z, const float* A,
                                 const float* carry_in, float* carry_out, const float* G, void* g_hi, void* g_lo,
                                 float* g_full, const float* g_carry_in, float* g_carry_out, int device, void* stream) {
  PR_REQUIRE(G && g_hi && g_lo && d > 0, PR_ERR_BAD_ARG, "null Gram pointers");
  pr::GramScanArgs g = {};
  g.in = G;
  g.hi = g_hi;
  g.lo = g_lo;
  g.full = g_full;
  g.carry_in = g_carry_in;
  g.carry_out = g_carry_out;
  g.d = d;
  return pr::launch_scan_fwd(dtype, b, n, n, h, E, Z, Z, A, carry_in, carry_out, g, device, stream);
}

extern "C" int pr_discumsum_bwd_blocks(long long E) {
  return (int)((E / 8 + pr::kScanThreads - 1) / pr::kScanThreads) * (pr::kScanThreads / 32);
}

namespace pr {
static int launch_scan_bwd(int dtype, int b, int n, int h, long long E, const void* dY, const void* Y, void* dX,
                           const float* A, const float* carry_in, float* carry_out, float* dA_part, int row_len,
                           int row_weights, const GramScanArgs& gram, int device, void* stream) {
  PR_REQUIRE(b > 0 && n > 0 && h > 0 && E > 0 && E % 8 == 0, PR_ERR_BAD_ARG, "bad sizes b=%d n=%d h=%d E=%lld", b, n,
             h, E);
  PR_REQUIRE(dY && A && aligned16(dY) && aligned16(Y) && aligned16(dX), PR_ERR_BAD_ARG,
             "null or misaligned pointer");
  PR_REQUIRE((dX == nullptr && carry_out != nullptr) || (dX != nullptr && Y != nullptr && dA_part != nullptr),
             PR_ERR_BAD_ARG, "give dX, Y and dA_part together, or none of them and a carry_out");
  PR_REQUIRE(!row_weights || (row_len > 0 && row_len % 8 == 0), PR_ERR_BAD_ARG, "row_len %d", row_len);
  PR_REQUIRE(gram.in == nullptr || (gram.zg && gram.hi && gram.lo && gram.dA_part && gram.d > 0 && gram.d <= 128),
             PR_ERR_BAD_ARG, "Gram scan without its tensors");
  PR_CUDA(cudaSetDevice(device));
  const int state_blocks = (int)((E / 8 + kScanThreads - 1) / kScanThreads);
  const int gram_blocks = gram.in ? (gram.d * gram.d + 255) / 256 : 0;
  dim3 grid((unsigned)(state_blocks + gram_blocks), h, b);
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const bool deep = few_ctas((long long)state_blocks * h * b, device);  // as in the forward scan
#define PR_LAUNCH_SCAN_B(TT, UNV)                                                                              \
  scan_bwd_kernel<TT, UNV><<<grid, kScanThreads, 0, s>>>(static_cast<const TT*>(dY), static_cast<const TT*>(Y), \
                                                         static_cast<TT*>(dX), A, carry_in, carry_out, dA_part, \
                                                         n, h, (size_t)E, row_len, row_weights, state_blocks,  \
                                                         gram)
  if (dtype == PR_BF16) {
    if (deep) PR_LAUNCH_SCAN_B(__nv_bfloat16, 8); else PR_LAUNCH_SCAN_B(__nv_bfloat16, kScanUnroll);
  } else if (dtype == PR_FP16) {
    if (deep) PR_LAUNCH_SCAN_B(__half, 8); else PR_LAUNCH_SCAN_B(__half, kScanUnroll);
  } else {
    return fail(PR_ERR_BAD_ARG, "dtype %d", dtype);
  }
#undef PR_LAUNCH_SCAN_B
  PR_CUDA(cudaGetLastError());
  return PR_OK;
}
}  // namespace pr

extern "C" int pr_discumsum_bwd(int dtype, int b, int n, int h, long long E, const void* dY, const void* Y, void* dX,
                                const float* A, const float* carry_in, float* carry_out, float* dA_part, int row_len,
                                int row_weights, int device, void* stream) {
  pr::GramScanArgs none = {};
  return pr::launch_scan_bwd(dtype, b, n, h, E, dY, Y, dX, A, carry_in, carry_out, dA_part, row_len, row_weights, none,
                             device, stream);
}

// pr_discumsum_bwd (in place, with key weights) and pr_gram_scan_bwd in ONE launch.
extern "C" int pr_state_scan_bwd(int dtype, int b, int n, int h, int d, long long E, void* dZ, const void* Z,
                                 const float* A, const float* carry_in, float* carry_out, float* dA_part,
                                 const float* dZg, const float* Zg, void* g_hi, void* g_lo, const float* g_carry_in,
                                 float* g_carry_out, float* g_dA_part, int device, void* stream) {
  PR_REQUIRE(dZg && Zg && g_hi && g_lo && g_dA_part && d > 0, PR_ERR_BAD_ARG, "null Gram pointers");
  pr::GramScanArgs g = {};
  g.in = dZg;
  g.zg = Zg;
  g.hi = g_hi;
  g.lo = g_lo;
  g.carry_in = g_carry_in;
  g.carry_out = g_carry_out;
  g.dA_part = g_dA_part;
  g.d = d;
  return pr::launch_scan_bwd(dtype, b, n, h, E, dZ, Z, dZ, A, carry_in, carry_out, dA_part, d, 1, g, device, stream);
}

extern "C" int pr_gram_scan_fwd(int dtype, int b, int n, int h, int d, const float* G, void* hi, void* lo,
                                float* full, const float* A, const float* carry_in, float* carry_out, int device,
                                void* stream) {
  using namespace pr;
  PR_REQUIRE(b > 0 && n > 0 && h > 0 && d > 0, PR_ERR_BAD_ARG, "bad sizes");
  PR_REQUIRE(G && hi && lo && A, PR_ERR_BAD_ARG, "null pointer");
  PR_CUDA(cudaSetDevice(device));
  const int E = d * d;
  dim3 grid((E + 255) / 256, h, b);
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  if (dtype == PR_BF16)
    scan_gram_fwd_kernel<__nv_bfloat16><<<grid, 256, 0, s>>>(G, static_cast<__nv_bfloat16*>(hi),
                                                            static_cast<__nv_bfloat16*>(lo), full, A, carry_in,
                                                            carry_out, n, h, E);
  else if (dtype == PR_FP16)
    scan_gram_fwd_kernel<__half><<<grid, 256, 0, s>>>(G, static_cast<__half*>(hi), static_cast<__half*>(lo), full, A,
                                                     carry_in, carry_out, n, h, E);
  else
    return fail(PR_ERR_BAD_ARG, "dtype %d", dtype);
  PR_CUDA(cudaGetLastError());
  return PR_OK;
}

extern "C" int pr_gram_scan_bwd_blocks(int d) { return (d * d + 255) / 256 * 8; }

extern "C" int pr_gram_scan_bwd(int dtype, int b, int n, int h, int d, const float* dZg, const float* Zg, void* hi,
                                void* lo, const float* A, const float* carry_in, float* carry_out, float* dA_part,
                                int device, void* stream) {
  using namespace pr;
  PR_REQUIRE(b > 0 && n > 0 && h > 0 && d > 0 && d <= 128, PR_ERR_BAD_ARG, "bad sizes");
  PR_REQUIRE(dZg && Zg && hi && lo && A && dA_part, PR_ERR_BAD_ARG, "null pointer");
  PR_CUDA(cudaSetDevice(device));
  dim3 grid((d * d + 255) / 256, h, b);
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  if (dtype == PR_BF16)
    scan_gram_bwd_kernel<__nv_bfloat16><<<grid, 256, 0, s>>>(dZg, Zg, static_cast<__nv_bfloat16*>(hi),
                                                            static_cast<__nv_bfloat16*>(lo), A, carry_in, carry_out,
                                                            dA_part, n, h, d);
  else if (dtype == PR_FP16)
    scan_gram_bwd_kernel<__half><<<grid, 256, 0, s>>>(dZg, Zg, static_cast<__half*>(hi), static_cast<__half*>(lo), A,
                                                     carry_in, carry_out, dA_part, n, h, d);
  else
    return fail(PR_ERR_BAD_ARG, "dtype %d", dtype);
  PR_CUDA(cudaGetLastError());
  return PR_OK;
}
