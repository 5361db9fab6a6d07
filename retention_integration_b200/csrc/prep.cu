// Gate preparation: per (batch, chunk, head) the inclusive cumulative log-gate
// a_i inside the chunk, the chunk total A, and the gated, transposed copy of the
// keys (or queries) that the token-contracting kernels read:
//     keys   : XT[d][i] = round(k_i[d] * exp((A - a_i)/2))
//     queries: XT[d][i] = round(q_i[d] * mult * exp(a_i/2))
// Restates the eager glue of the reference's wrapper
// (retention/power_retention_maker.py:143-155,183-186) as one pass over HBM.
#include <algorithm>

#include "host.cuh"
#include "sm100.cuh"

namespace pr {

constexpr int kPrepThreads = 256;   // gate_grad
constexpr int kGpThreads = 128;     // gate_prep: small CTAs, eight per SM, four 16-byte loads in flight per thread

template <typename T, int NV, bool PAIRED>
__global__ void __launch_bounds__(kGpThreads, NV == 4 ? 8 : 4)
gate_prep_kernel(const float* __restrict__ log_g, const float* __restrict__ a_in, const T* __restrict__ x,
                 float* __restrict__ a_out, float* __restrict__ A_out, T* __restrict__ xt,
                 const float* __restrict__ row_scale, T* __restrict__ xts, int t, int h, int hx, int d, int c, int cp,
                 int query_side, float mult, int write_a) {
  extern __shared__ float sm_f[];
  float* sm_a = sm_f;                                    // [c] cumulative gates (given, or scanned here)
  // transposed tiles [d features][64 tokens], 128-byte rows; the 16-byte chunk holding tokens 8j..8j+7 of
  // feature f sits at chunk j ^ ((f >> 3) & 7), which keeps both the scattered 16-bit writes and the 128-bit
  // row reads free of bank conflicts
  T* tile = reinterpret_cast<T*>(sm_f + ((c + 3) & ~3));
  T* tile2 = tile + 64 * d;                               // same, times row_scale
  __shared__ float warp_tot[kGpThreads / 32];
  __shared__ float carry_s;

  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int n = t / c;
  const int head = blockIdx.x % hx;
  const int chunk = (blockIdx.x / hx) % n;
  const int batch = blockIdx.x / (hx * n);
  const int gh = head / (hx / h);  // gate / kv head of this head
  const size_t tok0 = (size_t)batch * t + (size_t)chunk * c;

  // ---- the chunk's cumulative log gates: read if a pass before this one has made them, else a
  // block-wide inclusive scan of the log gates
  if (a_in != nullptr) {
    for (int i = tid; i < c; i += kGpThreads) sm_a[i] = a_in[(tok0 + i) * h + gh];
    __syncthreads();
  } else if (log_g != nullptr) {
    if (tid == 0) carry_s = 0.f;
    __syncthreads();
    // four consecutive gates per thread and round (their loads are independent), then one
    // block-wide scan of the per-thread totals: a 1024-token chunk is one round
    for (int base = 0; base < c; base += 4 * kGpThreads) {
      const int i0 = base + 4 * tid;
      float p[4];
#pragma unroll
      for (int k = 0; k < 4; ++k) p[k] = (i0 + k < c) ? log_g[(tok0 + i0 + k) * h + gh] : 0.f;
      p[1] += p[0];
      p[2] += p[1];
      p[3] += p[2];
      float v = p[3];
#pragma unroll
      for (int off = 1; off < 32; off <<= 1) {
        const float o = __shfl_up_sync(0xffffffffu, v, off);
        if (lane >= off) v += o;
      }
      if (lane == 31) warp_tot[warp] = v;
      __syncthreads();
      float pre = carry_s + (v - p[3]);  // everything before this thread's four gates
      for (int w = 0; w < warp; ++w) pre += warp_tot[w];
#pragma unroll
      for (int k = 0; k < 4; ++k)
        if (i0 + k < c) sm_a[i0 + k] = p[k] + pre;
      __syncthreads();
      if (tid == kGpThreads - 1) carry_s = p[3] + pre;
      __syncthreads();
    }
  } else {
    for (int i = tid; i < c; i += kGpThreads) sm_a[i] = 0.f;
    __syncthreads();
  }
  const float A = sm_a[c - 1];
  if (write_a && blockIdx.y == 0) {
    if (a_out != nullptr)
      for (int i = tid; i < c; i += kGpThreads) a_out[(tok0 + i) * h + gh] = sm_a[i];
    if (tid == 0 && A_out != nullptr) A_out[((size_t)batch * n + chunk) * h + gh] = A;
  }
  if (xt == nullptr) return;

  // ---- gated transpose, 64 tokens at a time
  const int vec_per_row = d / 8;
  T* out_base = xt + ((size_t)(batch * n + chunk) * hx + head) * (size_t)d * cp;
  T* out2_base = xts ? xts + ((size_t)(batch * n + chunk) * hx + head) * (size_t)d * cp : nullptr;
  // the chunk's 64-token tiles are split over gridDim.y blocks (each recomputes the cheap scan)
  const int tiles = cp / 64, tiles_per = (tiles + gridDim.y - 1) / gridDim.y;
  const int tb_end = min(cp, (int)(blockIdx.y + 1) * tiles_per * 64);
  // The loads of tile k+1 are issued before tile k is transposed and written out, so a CTA always has
  // a tile's worth of reads in flight (64 tokens x d features: up to four 16-byte vectors per thread).
  constexpr int kMaxVec = NV;  // 4 covers d <= 64, 8 covers d <= 128
  const int nvec = (64 * vec_per_row + kGpThreads - 1) / kGpThreads;  // <= kMaxVec for d <= 128
  uint4 raw[kMaxVec];
  float fac[kMaxVec], rsc[kMaxVec];
  // d = 64: a thread's vectors 2p and 2p + 1 hold the same eight features of tokens r and r + 1, so the
  // transposing stores below write two tokens of a feature as one 32-bit word (half as many stores; the
  // kernel is bound by instruction issue, not by bandwidth)
  constexpr bool paired = PAIRED;  // d = 64
  auto where = [&](int q, int* r, int* v) {
    if (paired) {
      *r = 2 * (tid >> 3) + (q & 1) + 32 * (q >> 1);
      *v = tid & 7;
    } else {
      const int idx = tid + q * kGpThreads;
      *r = idx / vec_per_row;
      *v = idx % vec_per_row;
    }
  };
  auto load_tile = [&](int tb) {
#pragma unroll
    for (int q = 0; q < kMaxVec; ++q) {
      const int idx = tid + q * kGpThreads;
      raw[q] = make_uint4(0, 0, 0, 0);
      fac[q] = rsc[q] = 0.f;
      if (q < nvec && idx < 64 * vec_per_row) {
        int r, v;
        where(q, &r, &v);
        const int i = tb + r;
        if (i < c) {
          raw[q] = *reinterpret_cast<const uint4*>(x + ((tok0 + i) * hx + head) * (size_t)d + v * 8);
          fac[q] = query_side ? mult * __expf(0.5f * sm_a[i]) : mult * __expf(0.5f * (A - sm_a[i]));
          if (xts != nullptr) rsc[q] = row_scale[(tok0 + i) * hx + head];
        }
      }
    }
  };
  const int tb_begin = blockIdx.y * tiles_per * 64;
  if (tb_begin < tb_end) load_tile(tb_begin);
  for (int tb = tb_begin; tb < tb_end; tb += 64) {
    __syncthreads();
    uint32_t wa[4] = {0, 0, 0, 0}, wa2[4] = {0, 0, 0, 0};  // the even token of a pair, kept for the odd one
#pragma unroll
    for (int q = 0; q < kMaxVec; ++q) {
      const int idx = tid + q * kGpThreads;
      if (q >= nvec || idx >= 64 * vec_per_row) continue;
      int r, v;
      where(q, &r, &v);
      const float f = fac[q], rs = rsc[q];
      uint32_t w[4] = {raw[q].x, raw[q].y, raw[q].z, raw[q].w};
      uint32_t w2[4];
#pragma unroll
      for (int k = 0; k < 4; ++k) {
        float2 p = Pack2<T>::to_f32(w[k]);
        w[k] = Pack2<T>::from_f32(p.x * f, p.y * f);
        // the scaled copy multiplies the ROUNDED gated value, so that both copies describe the same x~
        float2 pr_ = Pack2<T>::to_f32(w[k]);
        w2[k] = Pack2<T>::from_f32(pr_.x * rs, pr_.y * rs);
      }
      if (paired) {
        if ((q & 1) == 0) {
#pragma unroll
          for (int k = 0; k < 4; ++k) {
            wa[k] = w[k];
            wa2[k] = w2[k];
          }
          continue;
        }
        // tokens r - 1 (wa) and r (w): features v*8 .. v*8+7, one 32-bit store per feature
        const int pos = ((((r >> 3) ^ v) & 7) << 3) + ((r - 1) & 7);
        uint32_t* dst = reinterpret_cast<uint32_t*>(reinterpret_cast<uint16_t*>(tile) + (v * 8) * 64 + pos);
#pragma unroll
        for (int k = 0; k < 4; ++k) {
          dst[(2 * k) * 32] = __byte_perm(wa[k], w[k], 0x5410);
          dst[(2 * k + 1) * 32] = __byte_perm(wa[k], w[k], 0x7632);
        }
        if (xts != nullptr) {
          uint32_t* dst2 = reinterpret_cast<uint32_t*>(reinterpret_cast<uint16_t*>(tile2) + (v * 8) * 64 + pos);
#pragma unroll
          for (int k = 0; k < 4; ++k) {
            dst2[(2 * k) * 32] = __byte_perm(wa2[k], w2[k], 0x5410);
            dst2[(2 * k + 1) * 32] = __byte_perm(wa2[k], w2[k], 0x7632);
          }
        }
        continue;
      }
      // features v*8 .. v*8+7 of token r: one 16-bit store each, into the row of its feature
      const int pos = ((((r >> 3) ^ v) & 7) << 3) + (r & 7);
      uint16_t* dst = reinterpret_cast<uint16_t*>(tile) + (v * 8) * 64 + pos;
#pragma unroll
      for (int k = 0; k < 4; ++k) {
        dst[(2 * k) * 64] = (uint16_t)(w[k] & 0xffffu);
        dst[(2 * k + 1) * 64] = (uint16_t)(w[k] >> 16);
      }
      if (xts != nullptr) {
        uint16_t* dst2 = reinterpret_cast<uint16_t*>(tile2) + (v * 8) * 64 + pos;
#pragma unroll
        for (int k = 0; k < 4; ++k) {
          dst2[(2 * k) * 64] = (uint16_t)(w2[k] & 0xffffu);
          dst2[(2 * k + 1) * 64] = (uint16_t)(w2[k] >> 16);
        }
      }
    }
    if (tb + 64 < tb_end) load_tile(tb + 64);  // in flight while this tile is written out
    __syncthreads();
    // each thread writes 8 consecutive tokens of one feature row
    for (int idx = tid; idx < d * 8; idx += kGpThreads) {
      const int row = idx >> 3, tv = idx & 7;
      const int chunk8 = ((tv ^ (row >> 3)) & 7) << 3;
      *reinterpret_cast<uint4*>(out_base + (size_t)row * cp + tb + tv * 8) =
          *reinterpret_cast<const uint4*>(tile + row * 64 + chunk8);
      if (xts != nullptr)
        *reinterpret_cast<uint4*>(out2_base + (size_t)row * cp + tb + tv * 8) =
            *reinterpret_cast<const uint4*>(tile2 + row * 64 + chunk8);
    }
  }
}

// Backward prologue per output row: delta = <O, dO>, dy = dO / l (16-bit), dl = -delta / l.
// (O = y / l, so dL/dy = dO / l and dL/dl = -<dO, y> / l^2 = -delta / l.)
template <typename T>
__global__ void dout_prep_kernel(const T* __restrict__ O, const T* __restrict__ dO, const float* __restrict__ l,
                                 T* __restrict__ dy, float* __restrict__ dl, size_t rows, int d) {
  const int lanes_per_row = d / 8;  // 4, 8 or 16 threads share a row
  const size_t gid = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  const size_t row = gid / lanes_per_row;
  const int sub = (int)(gid % lanes_per_row);
  const bool active = row < rows;
  float part = 0.f, inv = 0.f;
  uint4 g = make_uint4(0, 0, 0, 0);
  if (active) {
    const uint4 o = *reinterpret_cast<const uint4*>(O + row * d + sub * 8);
    g = *reinterpret_cast<const uint4*>(dO + row * d + sub * 8);
    inv = safe_recip(l[row]);
    const uint32_t ow[4] = {o.x, o.y, o.z, o.w}, gw[4] = {g.x, g.y, g.z, g.w};
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      const float2 a = Pack2<T>::to_f32(ow[k]), b = Pack2<T>::to_f32(gw[k]);
      part = fmaf(a.x, b.x, fmaf(a.y, b.y, part));
    }
  }
  for (int off = lanes_per_row >> 1; off > 0; off >>= 1) part += __shfl_xor_sync(0xffffffffu, part, off);
  if (active) {
    uint32_t gw[4] = {g.x, g.y, g.z, g.w};
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      const float2 b = Pack2<T>::to_f32(gw[k]);
      gw[k] = Pack2<T>::from_f32(b.x * inv, b.y * inv);
    }
    *reinterpret_cast<uint4*>(dy + row * d + sub * 8) = make_uint4(gw[0], gw[1], gw[2], gw[3]);
    if (sub == 0) dl[row] = -part * inv;
  }
}


// Gate gradient assembly.  With a_i the inclusive cumulative log-gate inside a chunk and
// A the chunk total, dlog_G[u] = sum_{i >= u in chunk} da_i + dA, where
//   da_i = sum over the group's query heads of (attention term + state read-out term)
//          + key-side attention term - key discount term,
//   dA   = scan terms (state and Gram) + sum_i key discount term.
__global__ void __launch_bounds__(kPrepThreads)
gate_grad_kernel(const float* __restrict__ da_q, const float* __restrict__ gq, const float* __restrict__ da_k,
                 const float* __restrict__ wk, const float* __restrict__ dA_scan, int scan_blocks,
                 const float* __restrict__ dA_gram, int gram_blocks, float* __restrict__ dlog_g, int t, int h, int hq,
                 int c) {
  __shared__ float warp_tot[kPrepThreads / 32];
  __shared__ float carry_s, wk_sum_s;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int n = t / c, ratio = hq / h;
  const int head = blockIdx.x % h;
  const int chunk = (blockIdx.x / h) % n;
  const int batch = blockIdx.x / (h * n);
  const size_t tok0 = (size_t)batch * t + (size_t)chunk * c;

  // chunk-gate gradient: key discount terms of the chunk + the reverse scans' partial sums
  // ([b, h, scan_blocks, n] and [b, h, gram_blocks, n]), all reduced by the whole block
  float part = 0.f;
  if (wk != nullptr)
    for (int i = tid; i < c; i += kPrepThreads) part += wk[(tok0 + i) * h + head];
  if (dA_scan != nullptr) {
    const float* ps = dA_scan + ((size_t)batch * h + head) * scan_blocks * n + chunk;
    for (int k = tid; k < scan_blocks; k += kPrepThreads) part += ps[(size_t)k * n];
  }
  if (dA_gram != nullptr) {
    const float* pg = dA_gram + ((size_t)batch * h + head) * gram_blocks * n + chunk;
    for (int k = tid; k < gram_blocks; k += kPrepThreads) part += pg[(size_t)k * n];
  }
#pragma unroll
  for (int off = 16; off > 0; off >>= 1) part += __shfl_xor_sync(0xffffffffu, part, off);
  if (lane == 0) warp_tot[warp] = part;
  __syncthreads();
  if (tid == 0) {
    float s = 0.f;
    for (int w = 0; w < kPrepThreads / 32; ++w) s += warp_tot[w];
    wk_sum_s = s;
    carry_s = 0.f;
  }
  __syncthreads();
  const float dA = wk_sum_s;

  // reverse inclusive scan: walk the chunk from its end
  for (int base = 0; base < c; base += kPrepThreads) {
    const int ri = base + tid;     // distance from the end
    const int i = c - 1 - ri;
    float v = 0.f;
    if (ri < c) {
      const size_t tk = (tok0 + i) * h + head;
      v = da_k[tk] - (wk ? wk[tk] : 0.f);
      for (int r = 0; r < ratio; ++r) {
        const size_t tq = (tok0 + i) * hq + head * ratio + r;
        v += da_q[tq] + (gq ? gq[tq] : 0.f);
      }
    }
#pragma unroll
    for (int off = 1; off < 32; off <<= 1) {
      const float o = __shfl_up_sync(0xffffffffu, v, off);
      if (lane >= off) v += o;
    }
    __syncthreads();
    if (lane == 31) warp_tot[warp] = v;
    __syncthreads();
    float pre = carry_s;
    for (int w = 0; w < warp; ++w) pre += warp_tot[w];
    v += pre;
    if (ri < c) dlog_g[(tok0 + i) * h + head] = v + dA;
    __syncthreads();
    if (tid == kPrepThreads - 1) carry_s = v;
    __syncthreads();
  }
}

}  // namespace pr

extern "C" int pr_dout_prep(int dtype, long long rows, int d, const void* O, const void* dO, const float* l, void* dy,
                            float* dl, int device, void* stream) {
  using namespace pr;
  PR_REQUIRE(rows > 0 && (d == 32 || d == 64 || d == 128), PR_ERR_BAD_ARG, "rows=%lld d=%d", rows, d);
  PR_REQUIRE(O && dO && l && dy && dl && aligned16(O) && aligned16(dO) && aligned16(dy), PR_ERR_BAD_ARG,
             "null or misaligned pointer");
  PR_CUDA(cudaSetDevice(device));
  const size_t threads = (size_t)rows * (d / 8);
  const unsigned grid = (unsigned)((threads + 255) / 256);
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  if (dtype == PR_BF16)
    dout_prep_kernel<__nv_bfloat16><<<grid, 256, 0, s>>>(static_cast<const __nv_bfloat16*>(O),
                                                        static_cast<const __nv_bfloat16*>(dO), l,
                                                        static_cast<__nv_bfloat16*>(dy), dl, (size_t)rows, d);
  else if (dtype == PR_FP16)
    dout_prep_kernel<__half><<<grid, 256, 0, s>>>(static_cast<const __half*>(O), static_cast<const __half*>(dO), l,
                                                 static_cast<__half*>(dy), dl, (size_t)rows, d);
  else
    return fail(PR_ERR_BAD_ARG, "dtype %d", dtype);
  PR_CUDA(cudaGetLastError());
  return PR_OK;
}

extern "C" int pr_gate_prep(int dtype, int b, int t, int h, int hx, int d, int c, const float* log_g, const void* x,
                            float* a_out, float* A_out, void* xt, const float* row_scale, void* xts, int query_side,
                            float mult, int write_a, int device, void* stream) {
  using namespace pr;
  PR_REQUIRE(b > 0 && t > 0 && h > 0 && hx > 0 && hx % h == 0, PR_ERR_BAD_ARG, "bad sizes b=%d t=%d h=%d hx=%d", b, t,
             h, hx);
  PR_REQUIRE(c > 0 && t % c == 0, PR_ERR_BAD_ARG, "t=%d is not a multiple of the chunk size %d", t, c);
  PR_REQUIRE(d % 8 == 0 && d >= 16 && d <= 128, PR_ERR_BAD_ARG, "head dim %d unsupported", d);
  PR_REQUIRE(c <= 16384, PR_ERR_BAD_ARG, "chunk size %d exceeds 16384", c);
  PR_REQUIRE(dtype == PR_BF16 || dtype == PR_FP16, PR_ERR_BAD_ARG, "dtype %d", dtype);
  PR_REQUIRE(xt == nullptr || (x != nullptr && aligned16(x) && aligned16(xt)), PR_ERR_BAD_ARG,
             "x / xt null or misaligned");
  PR_REQUIRE(xts == nullptr || (xt != nullptr && row_scale != nullptr && aligned16(xts)), PR_ERR_BAD_ARG,
             "scaled copy requested without xt or row_scale");
  PR_CUDA(cudaSetDevice(device));
  const int cp = (c + 63) / 64 * 64;
  const size_t smem = (size_t)((c + 3) & ~3) * 4 + (size_t)2 * 64 * d * 2;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const int tiles = cp / 64;
  // The chunk's 64-token tiles are split over grid.y: four ways (two for short chunks), and further - down to one
  // tile per CTA - while that leaves fewer CTAs than fill the GPU (one head per GPU: 64 chunks x 4 = 256 CTAs, each
  // walking four tiles one after the other, took 28 us against 12 with one tile each).
  int ysplit = tiles >= 8 ? 4 : (tiles >= 2 ? 2 : 1);
  {
    int sms = 148;
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, device);
    const long long base = (long long)b * (t / c) * hx;
    const long long want = ((long long)sms * 8 + base - 1) / base;  // eight 128-thread CTAs per SM are resident
    ysplit = (int)std::min<long long>(tiles, std::max<long long>(ysplit, want));
  }
  const dim3 grid(b * (t / c) * hx, xt ? ysplit : 1);
  // The cumulative gates are scanned once per (batch, chunk, gate head), not once per CTA of the transposing
  // pass: either they are handed in (write_a = 0 with a_out given: the backward reuses the forward's), or a
  // first small launch makes them and the transposing launch reads them.
  const float* a_in = (write_a == 0 && a_out != nullptr && log_g != nullptr) ? a_out : nullptr;
  const bool two_pass = write_a && xt != nullptr && log_g != nullptr && a_out != nullptr && !query_side && hx == h;
#define PR_LAUNCH_PREP_K(KERNEL, TT, GRID, LG, AIN, XT, XTS, WRITE)                                            \
  do {                                                                                                         \
    PR_SMEM_ATTR(KERNEL, smem, device, false);                                                                 \
    KERNEL<<<GRID, kGpThreads, smem, s>>>(LG, AIN, static_cast<const TT*>(x), a_out, A_out, static_cast<TT*>(XT), \
                                          row_scale, static_cast<TT*>(XTS), t, h, hx, d, c, cp, query_side, mult, \
                                          WRITE);                                                              \
    PR_CUDA(cudaGetLastError());                                                                               \
  } while (0)
#define PR_LAUNCH_PREP(TT, GRID, LG, AIN, XT, XTS, WRITE)                                                       \
  do {                                                                                                         \
    if (d == 64)                                                                                               \
      PR_LAUNCH_PREP_K((gate_prep_kernel<TT, 4, true>), TT, GRID, LG, AIN, XT, XTS, WRITE);                    \
    else if (d < 64)                                                                                           \
      PR_LAUNCH_PREP_K((gate_prep_kernel<TT, 4, false>), TT, GRID, LG, AIN, XT, XTS, WRITE);                   \
    else                                                                                                       \
      PR_LAUNCH_PREP_K((gate_prep_kernel<TT, 8, false>), TT, GRID, LG, AIN, XT, XTS, WRITE);                   \
  } while (0)
  if (dtype == PR_BF16) {
    if (two_pass) {
      PR_LAUNCH_PREP(__nv_bfloat16, dim3(b * (t / c) * h, 1), log_g, nullptr, nullptr, nullptr, 1);
      PR_LAUNCH_PREP(__nv_bfloat16, grid, log_g, a_out, xt, xts, 0);
    } else {
      PR_LAUNCH_PREP(__nv_bfloat16, grid, log_g, a_in, xt, xts, write_a);
    }
  } else {
    if (two_pass) {
      PR_LAUNCH_PREP(__half, dim3(b * (t / c) * h, 1), log_g, nullptr, nullptr, nullptr, 1);
      PR_LAUNCH_PREP(__half, grid, log_g, a_out, xt, xts, 0);
    } else {
      PR_LAUNCH_PREP(__half, grid, log_g, a_in, xt, xts, write_a);
    }
  }
#undef PR_LAUNCH_PREP
#undef PR_LAUNCH_PREP_K
  return PR_OK;
}

extern "C" int pr_gate_grad(int b, int t, int h, int hq, int c, const float* da_q, const float* gq, const float* da_k,
                            const float* wk, const float* dA_scan, int scan_blocks, const float* dA_gram,
                            int gram_blocks, float* dlog_g, int device, void* stream) {
  using namespace pr;
  PR_REQUIRE(b > 0 && t > 0 && h > 0 && hq > 0 && hq % h == 0 && c > 0 && t % c == 0, PR_ERR_BAD_ARG,
             "bad sizes b=%d t=%d h=%d hq=%d c=%d", b, t, h, hq, c);
  PR_REQUIRE(da_q && da_k && dlog_g, PR_ERR_BAD_ARG, "null pointer");
  PR_CUDA(cudaSetDevice(device));
  gate_grad_kernel<<<b * (t / c) * h, kPrepThreads, 0, static_cast<cudaStream_t>(stream)>>>(
      da_q, gq, da_k, wk, dA_scan, scan_blocks, dA_gram, gram_blocks, dlog_g, t, h, hq, c);
  PR_CUDA(cudaGetLastError());
  return PR_OK;
}
