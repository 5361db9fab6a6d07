// Gate preparation: per (batch, chunk, head) the inclusive cumulative log-gate
// a_i inside the chunk, the chunk total A, and the gated, transposed copy of the
// keys (or queries) that the token-contracting kernels read:
//     keys   : XT[d][i] = round(k_i[d] * exp((A - a_i)/2))
//     queries: XT[d][i] = round(q_i[d] * mult * exp(a_i/2))
// Restates the eager glue of the reference's wrapper
// (retention/power_retention_maker.py:143-155,183-186) as one pass over HBM.
#include "host.cuh"
#include "sm100.cuh"

namespace pr {

constexpr int kPrepThreads = 256;

template <typename T>
__global__ void __launch_bounds__(kPrepThreads)
gate_prep_kernel(const float* __restrict__ log_g, const T* __restrict__ x, float* __restrict__ a_out,
                 float* __restrict__ A_out, T* __restrict__ xt, int t, int h, int hx, int d, int c, int cp,
                 int query_side, float mult, int write_a) {
  extern __shared__ float sm_f[];
  float* sm_a = sm_f;                                    // [c] cumulative gates
  T* tile = reinterpret_cast<T*>(sm_f + ((c + 3) & ~3)); // [64][d + 2]
  __shared__ float warp_tot[kPrepThreads / 32];
  __shared__ float carry_s;

  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int n = t / c;
  const int head = blockIdx.x % hx;
  const int chunk = (blockIdx.x / hx) % n;
  const int batch = blockIdx.x / (hx * n);
  const int gh = head / (hx / h);  // gate / kv head of this head
  const size_t tok0 = (size_t)batch * t + (size_t)chunk * c;

  // ---- block-wide inclusive scan of the chunk's log gates
  if (log_g != nullptr) {
    if (tid == 0) carry_s = 0.f;
    __syncthreads();
    for (int base = 0; base < c; base += kPrepThreads) {
      const int i = base + tid;
      float v = (i < c) ? log_g[(tok0 + i) * h + gh] : 0.f;
#pragma unroll
      for (int off = 1; off < 32; off <<= 1) {
        const float o = __shfl_up_sync(0xffffffffu, v, off);
        if (lane >= off) v += o;
      }
      if (lane == 31) warp_tot[warp] = v;
      __syncthreads();
      float pre = carry_s;
      for (int w = 0; w < warp; ++w) pre += warp_tot[w];
      v += pre;
      if (i < c) sm_a[i] = v;
      __syncthreads();
      if (tid == kPrepThreads - 1) carry_s = v;
      __syncthreads();
    }
  } else {
    for (int i = tid; i < c; i += kPrepThreads) sm_a[i] = 0.f;
    __syncthreads();
  }
  const float A = sm_a[c - 1];
  if (write_a) {
    if (a_out != nullptr)
      for (int i = tid; i < c; i += kPrepThreads) a_out[(tok0 + i) * h + gh] = sm_a[i];
    if (tid == 0 && A_out != nullptr) A_out[((size_t)batch * n + chunk) * h + gh] = A;
  }
  if (xt == nullptr) return;

  // ---- gated transpose, 64 tokens at a time
  const int ld = d + 2;
  const int vec_per_row = d / 8;
  T* out_base = xt + ((size_t)(batch * n + chunk) * hx + head) * (size_t)d * cp;
  for (int tb = 0; tb < cp; tb += 64) {
    __syncthreads();
    for (int idx = tid; idx < 64 * vec_per_row; idx += kPrepThreads) {
      const int r = idx / vec_per_row, v = idx % vec_per_row;
      const int i = tb + r;
      uint4 raw = make_uint4(0, 0, 0, 0);
      float f = 0.f;
      if (i < c) {
        raw = *reinterpret_cast<const uint4*>(x + ((tok0 + i) * hx + head) * (size_t)d + v * 8);
        f = query_side ? mult * __expf(0.5f * sm_a[i]) : mult * __expf(0.5f * (A - sm_a[i]));
      }
      uint32_t w[4] = {raw.x, raw.y, raw.z, raw.w};
#pragma unroll
      for (int k = 0; k < 4; ++k) {
        float2 p = Pack2<T>::to_f32(w[k]);
        w[k] = Pack2<T>::from_f32(p.x * f, p.y * f);
      }
      uint32_t* dst = reinterpret_cast<uint32_t*>(tile + r * ld + v * 8);
      dst[0] = w[0]; dst[1] = w[1]; dst[2] = w[2]; dst[3] = w[3];
    }
    __syncthreads();
    // each thread writes 8 consecutive tokens of one feature row
    for (int idx = tid; idx < d * 8; idx += kPrepThreads) {
      const int row = idx >> 3, tv = idx & 7;
      T vals[8];
#pragma unroll
      for (int k = 0; k < 8; ++k) vals[k] = tile[(tv * 8 + k) * ld + row];
      *reinterpret_cast<uint4*>(out_base + (size_t)row * cp + tb + tv * 8) = *reinterpret_cast<uint4*>(vals);
    }
  }
}

}  // namespace pr

extern "C" int pr_gate_prep(int dtype, int b, int t, int h, int hx, int d, int c, const float* log_g, const void* x,
                            float* a_out, float* A_out, void* xt, int query_side, float mult, int write_a, int device,
                            void* stream) {
  using namespace pr;
  PR_REQUIRE(b > 0 && t > 0 && h > 0 && hx > 0 && hx % h == 0, PR_ERR_BAD_ARG, "bad sizes b=%d t=%d h=%d hx=%d", b, t,
             h, hx);
  PR_REQUIRE(c > 0 && t % c == 0, PR_ERR_BAD_ARG, "t=%d is not a multiple of the chunk size %d", t, c);
  PR_REQUIRE(d % 8 == 0 && d >= 16 && d <= 128, PR_ERR_BAD_ARG, "head dim %d unsupported", d);
  PR_REQUIRE(c <= 16384, PR_ERR_BAD_ARG, "chunk size %d exceeds 16384", c);
  PR_REQUIRE(dtype == PR_BF16 || dtype == PR_FP16, PR_ERR_BAD_ARG, "dtype %d", dtype);
  PR_REQUIRE(xt == nullptr || (x != nullptr && aligned16(x) && aligned16(xt)), PR_ERR_BAD_ARG,
             "x / xt null or misaligned");
  PR_CUDA(cudaSetDevice(device));
  const int cp = (c + 63) / 64 * 64;
  const size_t smem = (size_t)((c + 3) & ~3) * 4 + (size_t)64 * (d + 2) * 2;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const int grid = b * (t / c) * hx;
  if (dtype == PR_BF16) {
    PR_CUDA(cudaFuncSetAttribute(gate_prep_kernel<__nv_bfloat16>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                 (int)smem));
    gate_prep_kernel<__nv_bfloat16><<<grid, kPrepThreads, smem, s>>>(
        log_g, static_cast<const __nv_bfloat16*>(x), a_out, A_out, static_cast<__nv_bfloat16*>(xt), t, h, hx, d, c, cp,
        query_side, mult, write_a);
  } else {
    PR_CUDA(cudaFuncSetAttribute(gate_prep_kernel<__half>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    gate_prep_kernel<__half><<<grid, kPrepThreads, smem, s>>>(log_g, static_cast<const __half*>(x), a_out, A_out,
                                                              static_cast<__half*>(xt), t, h, hx, d, c, cp, query_side,
                                                              mult, write_a);
  }
  PR_CUDA(cudaGetLastError());
  return PR_OK;
}
