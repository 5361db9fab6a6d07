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

// Self-test of the give-up path of the bounded waits.  One CTA allocates tensor memory and
// waits on an mbarrier that nothing ever arrives at; the wait budget is `budget_us`
// microseconds instead of the library's two seconds.  Every warp gives up on its own, the
// CTA meets at its teardown barrier, writes ST_TIMEOUT to the status word, releases its
// tensor memory and returns: no trap, no unbounded spin, and the context stays usable.
namespace pr {
__global__ void __launch_bounds__(128) selftest_timeout_kernel(unsigned long long budget_ns, int* status, int* gave_up) {
  __shared__ uint64_t never;
  __shared__ uint32_t tmem_base_s;
  __shared__ int abort_flag;
  const int tid = threadIdx.x, warp = tid >> 5;
  if (tid == 0) {
    abort_flag = 0;
    mbar_init(&never, 1);
    fence_mbar_init();
  }
  if (warp == 0) {
    tmem_alloc(&tmem_base_s, 32);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const bool ok = mbar_wait_for(&never, 0, &abort_flag, budget_ns);
  if (!ok) atomicAdd(gave_up, 1);
  tc_fence_before();
  __syncthreads();
  if (tid == 0 && abort_flag) *status = ST_TIMEOUT;
  if (warp == 0) tmem_dealloc(tmem_base_s, 32);
}
}  // namespace pr

extern "C" int pr_selftest_timeout(int budget_us, int* gave_up, int device, void* stream) {
  using namespace pr;
  PR_REQUIRE(budget_us > 0 && budget_us <= 100000, PR_ERR_BAD_ARG, "budget of %d us not in (0, 100000]", budget_us);
  PR_REQUIRE(gave_up != nullptr, PR_ERR_BAD_ARG, "gave_up is null");
  PR_CUDA(cudaSetDevice(device));
  int* status = nullptr;
  int rc = status_word(device, &status, nullptr);
  if (rc) return rc;
  selftest_timeout_kernel<<<1, 128, 0, static_cast<cudaStream_t>(stream)>>>((unsigned long long)budget_us * 1000ull,
                                                                            status, gave_up);
  PR_CUDA(cudaGetLastError());
  return PR_OK;
}
