// Self-test of the tensor-core building blocks every contraction kernel of this
// library is made of: swizzled shared-memory operands written by threads or by
// TMA, K-major and MN-major B, A read from tensor memory, accumulators read back
// with tcgen05.ld.  One CTA, one 128 x N x K product.
#include "host.cuh"
#include "sm100.cuh"

namespace pr {

template <typename T>
__global__ void __launch_bounds__(128)
selftest_kernel(int variant, int n, int k, const T* __restrict__ a, const T* __restrict__ b,
                float* __restrict__ out, int* status, const __grid_constant__ CUtensorMap tm_a,
                const __grid_constant__ CUtensorMap tm_b) {
  extern __shared__ uint8_t smem_raw[];
  __shared__ uint64_t bar_tma, bar_mma;
  __shared__ uint32_t tmem_base_s;
  __shared__ int abort_flag;

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t* sm = smem_raw + (base - smem_u32(smem_raw));
  const int kblocks = k / 64;
  uint8_t* smA = sm;                       // kblocks x [128 rows x 128 B]
  uint8_t* smB = sm + kblocks * 16384;     // K-major: kblocks x [n x 128 B]; MN-major: [k x 128 B]
  const bool b_mn = (variant == 1 || variant == 2 || variant == 3);
  const bool a_tmem = (variant == 2 || variant == 3);
  const bool tma_b = (variant == 3 || variant == 4);
  const bool tma_a = (variant == 4);

  if (tid == 0) {
    abort_flag = 0;
    mbar_init(&bar_tma, 1);
    mbar_init(&bar_mma, 1);
    fence_mbar_init();
  }
  if (warp == 0) {
    tmem_alloc(&tmem_base_s, 512);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_d = tmem_base_s;
  const uint32_t tmem_a = tmem_base_s + 256;

  // ---- stage operands
  if (!tma_a && !a_tmem) {
    const int cpr = k / 8;  // 16-byte chunks per row
    for (int idx = tid; idx < 128 * cpr; idx += 128) {
      const int m = idx / cpr, cc = idx % cpr, kb = cc >> 3, c = cc & 7;
      const uint4 v = *reinterpret_cast<const uint4*>(a + (size_t)m * k + cc * 8);
      *reinterpret_cast<uint4*>(smA + kb * 16384 + swz128(m, c)) = v;
    }
  }
  if (a_tmem) {
    // thread = row; two consecutive K elements per 32-bit column, low half first
    const uint32_t* arow = reinterpret_cast<const uint32_t*>(a + (size_t)tid * k);
    for (int c0 = 0; c0 < k / 2; c0 += 8) {
      uint32_t r[8];
#pragma unroll
      for (int j = 0; j < 8; ++j) r[j] = arow[c0 + j];
      tmem_st8(tmem_a + ((uint32_t)(warp * 32) << 16) + c0, r);
    }
    tmem_wait_st();
  }
  if (!tma_b) {
    if (!b_mn) {
      const int cpr = k / 8;
      for (int idx = tid; idx < n * cpr; idx += 128) {
        const int r = idx / cpr, cc = idx % cpr, kb = cc >> 3, c = cc & 7;
        const uint4 v = *reinterpret_cast<const uint4*>(b + (size_t)r * k + cc * 8);
        *reinterpret_cast<uint4*>(smB + kb * (n * 128) + swz128(r, c)) = v;
      }
    } else {
      for (int idx = tid; idx < k * 8; idx += 128) {
        const int kk = idx >> 3, c = idx & 7;
        const uint4 v = *reinterpret_cast<const uint4*>(b + (size_t)kk * 64 + c * 8);
        *reinterpret_cast<uint4*>(smB + swz128(kk, c)) = v;
      }
    }
  }
  fence_async_smem();
  tc_fence_before();
  __syncthreads();

  bool ok = true;
  if (tid == 0) {
    if (tma_a || tma_b) {
      uint32_t bytes = 0;
      if (tma_a) bytes += 128 * k * 2;
      if (tma_b) bytes += n * k * 2;
      mbar_expect_tx(&bar_tma, bytes);
      for (int kb = 0; kb < kblocks; ++kb) {
        if (tma_a) tma_load_2d(smA + kb * 16384, &tm_a, &bar_tma, 64 * kb, 0);
        if (tma_b) {
          if (b_mn)
            tma_load_2d(smB + kb * 8192, &tm_b, &bar_tma, 0, 64 * kb);
          else
            tma_load_2d(smB + kb * (n * 128), &tm_b, &bar_tma, 64 * kb, 0);
        }
      }
      ok = mbar_wait(&bar_tma, 0, &abort_flag);
    }
    if (ok) {
      tc_fence_after();
      const uint32_t idesc = umma_idesc(128, n, Pack2<T>::is_bf16, false, b_mn);
      const uint32_t a_addr = smem_u32(smA), b_addr = smem_u32(smB);
      for (int ks = 0; ks < k / 16; ++ks) {
        const uint64_t bd = b_mn ? umma_desc_sw128(b_addr + ks * 2048, 8192, 1024)
                                 : umma_desc_sw128(b_addr + (ks >> 2) * (n * 128) + (ks & 3) * 32, 16, 1024);
        if (a_tmem) {
          umma_ts(tmem_d, tmem_a + ks * 8, bd, idesc, ks > 0);
        } else {
          const uint64_t ad = umma_desc_sw128(a_addr + (ks >> 2) * 16384 + (ks & 3) * 32, 16, 1024);
          umma_ss(tmem_d, ad, bd, idesc, ks > 0);
        }
      }
      umma_commit(&bar_mma);
    }
  }
  __syncwarp();
  ok = mbar_wait(&bar_mma, 0, &abort_flag);
  tc_fence_after();
  if (ok) {
    for (int c0 = 0; c0 < n; c0 += 32) {
      uint32_t r[32];
      tmem_ld32(tmem_d + ((uint32_t)(warp * 32) << 16) + c0, r);
      tmem_wait_ld();
      float* orow = out + (size_t)(warp * 32 + lane) * n + c0;
#pragma unroll
      for (int j = 0; j < 32; ++j) orow[j] = __uint_as_float(r[j]);
    }
  } else if (tid == 0) {
    *status = ST_TIMEOUT;
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 0) tmem_dealloc(tmem_base_s, 512);
}

template <typename T>
static int launch_selftest(int variant, int n, int k, const void* a, const void* b, float* out, int* status,
                           cudaStream_t stream) {
  CUtensorMap tm_a, tm_b;
  memset(&tm_a, 0, sizeof(tm_a));
  memset(&tm_b, 0, sizeof(tm_b));
  const bool b_mn = (variant >= 1 && variant <= 3);
  if (variant == 4) {
    uint64_t dims[2] = {(uint64_t)k, 128}, strides[2] = {0, (uint64_t)k * 2};
    uint32_t box[2] = {64, 128};
    int rc = make_tmap(&tm_a, a, 2, 2, dims, strides, box, true);
    if (rc) return rc;
  }
  if (variant >= 3) {
    if (b_mn) {
      uint64_t dims[2] = {64, (uint64_t)k}, strides[2] = {0, 128};
      uint32_t box[2] = {64, 64};
      int rc = make_tmap(&tm_b, b, 2, 2, dims, strides, box, true);
      if (rc) return rc;
    } else {
      uint64_t dims[2] = {(uint64_t)k, (uint64_t)n}, strides[2] = {0, (uint64_t)k * 2};
      uint32_t box[2] = {64, (uint32_t)n};
      int rc = make_tmap(&tm_b, b, 2, 2, dims, strides, box, true);
      if (rc) return rc;
    }
  }
  const size_t smem = 1024 + (size_t)(k / 64) * 16384 + (size_t)n * k * 2;
  PR_CUDA(cudaFuncSetAttribute(selftest_kernel<T>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
  selftest_kernel<T><<<1, 128, smem, stream>>>(variant, n, k, static_cast<const T*>(a), static_cast<const T*>(b), out,
                                               status, tm_a, tm_b);
  PR_CUDA(cudaGetLastError());
  return PR_OK;
}

}  // namespace pr

extern "C" int pr_selftest_umma(int variant, int dtype, int n, int k, const void* a, const void* b, float* out,
                                int device, void* stream) {
  using namespace pr;
  PR_REQUIRE(variant >= 0 && variant <= 4, PR_ERR_BAD_ARG, "variant %d not in 0..4", variant);
  PR_REQUIRE(k >= 64 && k <= 256 && k % 64 == 0, PR_ERR_BAD_ARG, "k=%d must be 64, 128, 192 or 256", k);
  PR_REQUIRE(n == 64 || n == 128 || n == 256, PR_ERR_BAD_ARG, "n=%d must be 64, 128 or 256", n);
  PR_REQUIRE(!(variant >= 1 && variant <= 3) || n == 64, PR_ERR_BAD_ARG, "MN-major variants need n=64");
  PR_REQUIRE(a && b && out && aligned16(a) && aligned16(b) && aligned16(out), PR_ERR_BAD_ARG,
             "null or misaligned pointer");
  PR_REQUIRE(dtype == PR_BF16 || dtype == PR_FP16, PR_ERR_BAD_ARG, "dtype %d", dtype);
  PR_CUDA(cudaSetDevice(device));
  int* status = nullptr;
  int rc = status_word(device, &status, nullptr);
  if (rc) return rc;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  return dtype == PR_BF16 ? launch_selftest<__nv_bfloat16>(variant, n, k, a, b, out, status, s)
                          : launch_selftest<__half>(variant, n, k, a, b, out, status, s);
}

// Micro-benchmark: tensor-memory read bandwidth.  `nwarps` warps (4, 8 or 16) each issue
// `iters` loads of 32 lanes x 32 columns from an allocated region; returns SM clock cycles.
namespace pr {
// mode 0: x32 load then wait; 1: two x32 loads then one wait; 2: x16 loads; 3: x8 loads
__global__ void tmem_bw_kernel(int iters, int mode, long long* cycles, float* sink) {
  __shared__ uint32_t tmem_base_s;
  const int warp = threadIdx.x >> 5;
  if (warp == 0) {
    tmem_alloc(&tmem_base_s, 512);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = tmem_base_s + ((uint32_t)((warp & 3) * 32) << 16);
  uint32_t v[64];
  float acc = 0.f;
  __syncthreads();
  const long long t0 = clock64();
  if (mode == 0) {
    for (int it = 0; it < iters; ++it) {
      tmem_ld32(tmem + ((it * 32) & 511), v);
      tmem_wait_ld();
      acc += __uint_as_float(v[it & 31]);
    }
  } else if (mode == 1) {
    for (int it = 0; it < iters; it += 2) {
      tmem_ld32(tmem + ((it * 32) & 511), v);
      tmem_ld32(tmem + ((it * 32 + 32) & 511), v + 32);
      tmem_wait_ld();
      acc += __uint_as_float(v[it & 63]);
    }
  } else if (mode == 2) {
    for (int it = 0; it < iters; ++it) {
      tmem_ld16(tmem + ((it * 32) & 511), v);
      tmem_ld16(tmem + ((it * 32 + 16) & 511), v + 16);
      tmem_wait_ld();
      acc += __uint_as_float(v[it & 31]);
    }
  } else {
    for (int it = 0; it < iters; ++it) {
      uint32_t w[8];
#pragma unroll
      for (int k = 0; k < 4; ++k) {
        tmem_ld8(tmem + ((it * 32 + 8 * k) & 511), w);
        v[8 * k] = w[0] ^ w[7];
      }
      tmem_wait_ld();
      acc += __uint_as_float(v[(it & 3) * 8]);
    }
  }
  __syncthreads();
  const long long t1 = clock64();
  if (threadIdx.x == 0) cycles[blockIdx.x] = t1 - t0;
  if (acc == 123.456f) sink[0] = acc;
  tc_fence_before();
  __syncthreads();
  if (warp == 0) tmem_dealloc(tmem_base_s, 512);
}
}  // namespace pr

namespace pr {
// Micro-benchmark: issue rate of tcgen05.mma for the operand shapes the kernels use.
// mode 0: A,B in smem, N=128 (K-major); 1: A,B in smem, N=64; 2: A in TMEM, B MN-major smem, N=64;
// 3: A in TMEM, B MN-major, N=128 (two 64-wide blocks).  `reps` groups of four K=16 steps.
__global__ void mma_rate_kernel(int reps, int mode, long long* cycles) {
  extern __shared__ uint8_t smem_raw[];
  __shared__ uint64_t bar;
  __shared__ uint32_t tmem_base_s;
  __shared__ int abort_flag;
  const int tid = threadIdx.x, warp = tid >> 5;
  const uint32_t sbase = (smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t* sm = smem_raw + (sbase - smem_u32(smem_raw));
  for (int i = tid; i < 49152 / 4; i += blockDim.x) reinterpret_cast<uint32_t*>(sm)[i] = 0;
  if (tid == 0) {
    abort_flag = 0;
    mbar_init(&bar, 1);
    fence_mbar_init();
  }
  if (warp == 0) {
    tmem_alloc(&tmem_base_s, 512);
    tmem_relinquish();
  }
  fence_async_smem();
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  if (tid == 0) {
    const uint32_t a_addr = smem_u32(sm), b_addr = smem_u32(sm + 16384), tmem = tmem_base_s;
    // modes 4-7 repeat 0-3 with two accumulators used alternately; mode 8: smem x smem, N=256
    const int alt = (mode >= 4 && mode <= 7) ? 1 : 0;
    const int m4 = mode & 3;
    const int n = mode == 8 ? 256 : ((m4 == 0 || m4 == 3) ? 128 : 64);
    const bool ts = mode != 8 && m4 >= 2;
    const uint32_t idesc = umma_idesc(128, n, true, false, ts);
    const long long t0 = clock64();
    for (int r = 0; r < reps; ++r) {
#pragma unroll
      for (int ks = 0; ks < 4; ++ks) {
        const uint32_t dcol = tmem + (alt ? (ks & 1) * 128 : 0);
        if (ts)
          umma_ts(dcol, tmem + 256 + ks * 8, umma_desc_sw128(b_addr + ks * 2048, 8192, 1024), idesc, 1u);
        else
          umma_ss(dcol, umma_desc_sw128(a_addr + ks * 32, 16, 1024), umma_desc_sw128(b_addr + ks * 32, 16, 1024),
                  idesc, 1u);
      }
    }
    umma_commit(&bar);
    mbar_wait(&bar, 0, &abort_flag);
    cycles[0] = clock64() - t0;
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 0) tmem_dealloc(tmem_base_s, 512);
}
}  // namespace pr

extern "C" int pr_selftest_mma_rate(int reps, int mode, long long* cycles, int device, void* stream) {
  using namespace pr;
  PR_REQUIRE(reps > 0 && mode >= 0 && mode <= 8 && cycles, PR_ERR_BAD_ARG, "bad arguments");
  PR_CUDA(cudaSetDevice(device));
  PR_CUDA(cudaFuncSetAttribute(mma_rate_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 51200));
  mma_rate_kernel<<<1, 128, 51200, static_cast<cudaStream_t>(stream)>>>(reps, mode, cycles);
  PR_CUDA(cudaGetLastError());
  return PR_OK;
}

namespace pr {
// Micro-benchmark: round trip of tcgen05.ld (32 lanes x 32 columns, then wait) as seen by
// `nwarps` reader warps, alone or while one more thread keeps the tensor core busy with
// smem x smem products (M = 128, N = mma_n, K = 16) into other columns.  cycles[0] = SM clocks
// the slowest reader took for `iters` loads, cycles[1] = clocks for the products.  With burst > 0 the
// products come as mma_reps bursts of `burst` groups, each waited for, `gap` idle clocks apart:
// cycles[1] = clocks inside bursts, [2] / [3] = first / last burst, [4] = clocks spent issuing (products and commit), [5] = products only.
__global__ void tmem_ld_contention_kernel(int iters, int mma_reps, int mma_n, int burst, int gap, long long* cycles,
                                          float* sink) {
  extern __shared__ uint8_t smem_raw[];
  __shared__ uint64_t bar;
  __shared__ uint32_t tmem_base_s;
  __shared__ int abort_flag;
  __shared__ unsigned long long worst;
  const int tid = threadIdx.x, warp = tid >> 5;
  const int readers = (blockDim.x >> 5) - 1;
  const uint32_t sbase = (smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t* sm = smem_raw + (sbase - smem_u32(smem_raw));
  for (int i = tid; i < 49152 / 4; i += blockDim.x) reinterpret_cast<uint32_t*>(sm)[i] = 0;
  if (tid == 0) {
    abort_flag = 0;
    worst = 0;
    mbar_init(&bar, 1);
    fence_mbar_init();
  }
  if (warp == 0) {
    tmem_alloc(&tmem_base_s, 512);
    tmem_relinquish();
  }
  fence_async_smem();
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = tmem_base_s;
  if (warp < readers) {
    const uint32_t base = tmem + ((uint32_t)((warp & 3) * 32) << 16);
    uint32_t acc = 0;
    const long long t0 = clock64();
    for (int it = 0; it < iters; ++it) {
      uint32_t v[32];
      tmem_ld32(base + ((it * 32) & 255), v);
      tmem_wait_ld();
#pragma unroll
      for (int j = 0; j < 32; ++j) acc ^= v[j];
    }
    const long long t1 = clock64();
    atomicMax(&worst, (unsigned long long)(t1 - t0));
    if (acc == 0x12345u) sink[0] = 1.f;
  } else if (tid == readers * 32 && mma_reps > 0) {
    const uint32_t a_addr = smem_u32(sm), b_addr = smem_u32(sm + 16384);
    const uint32_t idesc = umma_idesc(128, mma_n, true, false, false);
    if (burst <= 0) {
      const long long t0 = clock64();
      for (int r = 0; r < mma_reps; ++r) {
#pragma unroll
        for (int ks = 0; ks < 4; ++ks)
          umma_ss(tmem + 256, umma_desc_sw128(a_addr + ks * 32, 16, 1024),
                  umma_desc_sw128(b_addr + ks * 32, 16, 1024), idesc, 1u);
      }
      umma_commit(&bar);
      mbar_wait(&bar, 0, &abort_flag);
      cycles[1] = clock64() - t0;
    } else {
      // bursts of `burst` groups of four products, each burst waited for, `gap` idle clocks between bursts
      long long in_burst = 0, issue = 0, mma_issue = 0;
      for (int r = 0; r < mma_reps; ++r) {
        const long long t0 = clock64();
        for (int g = 0; g < burst; ++g) {
#pragma unroll
          for (int ks = 0; ks < 4; ++ks)
            umma_ss(tmem + 256, umma_desc_sw128(a_addr + ks * 32, 16, 1024),
                    umma_desc_sw128(b_addr + ks * 32, 16, 1024), idesc, 1u);
        }
        const long long tm = clock64();
        umma_commit(&bar);
        const long long t1 = clock64();
        mbar_wait(&bar, r & 1, &abort_flag);
        const long long t2 = clock64();
        issue += t1 - t0;
        mma_issue += tm - t0;
        in_burst += t2 - t0;
        if (r == 0) cycles[2] = t2 - t0;
        if (r == mma_reps - 1) cycles[3] = t2 - t0;
        while (clock64() - t2 < gap) {
        }
      }
      cycles[1] = in_burst;
      cycles[4] = issue;
      cycles[5] = mma_issue;
    }
  }
  tc_fence_before();
  __syncthreads();
  if (tid == 0) cycles[0] = (long long)worst;
  if (warp == 0) tmem_dealloc(tmem_base_s, 512);
}
}  // namespace pr

extern "C" int pr_selftest_tmem_ld_contention(int nwarps, int iters, int mma_reps, int mma_n, int burst, int gap,
                                              long long* cycles, float* sink, int device, void* stream) {
  using namespace pr;
  PR_REQUIRE((nwarps == 4 || nwarps == 8 || nwarps == 16) && iters > 0 && mma_reps >= 0 &&
                 (mma_n == 64 || mma_n == 128 || mma_n == 256) && cycles && sink,
             PR_ERR_BAD_ARG, "bad arguments");
  PR_CUDA(cudaSetDevice(device));
  PR_CUDA(cudaFuncSetAttribute(tmem_ld_contention_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 51200));
  tmem_ld_contention_kernel<<<1, (nwarps + 1) * 32, 51200, static_cast<cudaStream_t>(stream)>>>(
      iters, mma_reps, mma_n, burst, gap, cycles, sink);
  PR_CUDA(cudaGetLastError());
  return PR_OK;
}

namespace pr {
// Micro-benchmark: how fast the SMs can stream 16 KB tiles (128 rows x 128 B, swizzled) out of
// L2 with TMA.  Every CTA walks `tiles` consecutive tiles of its region `reps` times through a
// ring of `depth` stages; CTAs with the same blockIdx.x / share walk the same region.
__global__ void __launch_bounds__(64)
tma_stream_kernel(int tiles, int reps, int depth, int share, long long* cycles,
                  const __grid_constant__ CUtensorMap tm) {
  extern __shared__ uint8_t smem_raw[];
  __shared__ uint64_t full[12], empty[12];
  __shared__ int abort_flag;
  const int tid = threadIdx.x;
  const uint32_t sbase = (smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t* sm = smem_raw + (sbase - smem_u32(smem_raw));
  if (tid == 0) {
    abort_flag = 0;
    for (int s = 0; s < depth; ++s) {
      mbar_init(&full[s], 1);
      mbar_init(&empty[s], 1);
    }
    fence_mbar_init();
  }
  __syncthreads();
  const int region = blockIdx.x / share;
  const int total = tiles * reps;
  const long long t0 = clock64();
  if (tid == 0) {
    for (int i = 0; i < total; ++i) {
      const int s = i % depth, ph = (i / depth) & 1;
      if (!mbar_wait(&empty[s], ph ^ 1, &abort_flag)) break;
      mbar_expect_tx(&full[s], 16384);
      tma_load_2d(sm + s * 16384, &tm, &full[s], 0, (region * tiles + i % tiles) * 128);
    }
  } else if (tid == 32) {
    for (int i = 0; i < total; ++i) {
      const int s = i % depth, ph = (i / depth) & 1;
      if (!mbar_wait(&full[s], ph, &abort_flag)) break;
      mbar_arrive(&empty[s]);
    }
    cycles[blockIdx.x] = clock64() - t0;
  }
}
}  // namespace pr

// buf_bytes must cover ceil(grid / share) * tiles * 16384 bytes.  cycles: one entry per CTA.
extern "C" int pr_selftest_tma_stream(const void* buf, long long buf_bytes, int grid, int tiles, int reps, int depth,
                                      int share, int min_smem, long long* cycles, int device, void* stream) {
  using namespace pr;
  PR_REQUIRE(buf && cycles && grid > 0 && tiles > 0 && reps > 0 && depth >= 1 && depth <= 12 && share >= 1,
             PR_ERR_BAD_ARG, "bad arguments");
  PR_REQUIRE((long long)((grid + share - 1) / share) * tiles * 16384 <= buf_bytes, PR_ERR_BAD_ARG,
             "buffer of %lld bytes is smaller than the %d regions of %d tiles", buf_bytes, (grid + share - 1) / share,
             tiles);
  PR_CUDA(cudaSetDevice(device));
  CUtensorMap tm;
  uint64_t dims[2] = {64, (uint64_t)((grid + share - 1) / share) * tiles * 128};
  uint64_t strides[2] = {0, 128};
  uint32_t box[2] = {64, 128};
  int rc = make_tmap(&tm, buf, 2, 2, dims, strides, box, true);
  if (rc) return rc;
  const int smem = max(1024 + depth * 16384, min(min_smem, 227 * 1024));  // min_smem limits the CTAs per SM
  PR_CUDA(cudaFuncSetAttribute(tma_stream_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem));
  tma_stream_kernel<<<grid, 64, smem, static_cast<cudaStream_t>(stream)>>>(tiles, reps, depth, share, cycles, tm);
  PR_CUDA(cudaGetLastError());
  return PR_OK;
}

extern "C" int pr_selftest_tmem_bw(int nwarps, int iters, long long* cycles, float* sink, int device, void* stream) {
  using namespace pr;
  PR_REQUIRE(nwarps == 4 || nwarps == 8 || nwarps == 16, PR_ERR_BAD_ARG, "nwarps must be 4, 8 or 16");
  PR_REQUIRE(cycles && sink && iters > 0, PR_ERR_BAD_ARG, "bad arguments");
  PR_CUDA(cudaSetDevice(device));
  tmem_bw_kernel<<<1, nwarps * 32, 0, static_cast<cudaStream_t>(stream)>>>(iters & 0xffffff, iters >> 24, cycles, sink);
  PR_CUDA(cudaGetLastError());
  return PR_OK;
}
