// Inference kernels (the reference's _power_retention_inference,
// retention/power_retention_maker.py:287-390, for a single query token per sequence):
//
//   pr_decode_state : reads the recurrent state once.  For every (batch, kv head) the
//                     state S [D, 64] and sum_of_keys s [D] (exact layout, D = C(d+1,2)) are
//                     contracted with phi(q~) of the group's query heads, q~ = s*q*exp(a_last/2):
//                     y = sum_D phi(q~)[D] S[D,:],  l = sum_D phi(q~)[D] s[D].
//                     HBM bound: 128-bit loads, each 128-byte state row read by 8 threads,
//                     D split over several CTAs; partial sums go to a small workspace.
//   pr_decode_step  : the whole step in one kernel; the state is streamed by TMA and contracted on
//                     the tensor cores (decode_tc_kernel below).  pr_decode_state / pr_decode_finish
//                     are the same step in two CUDA-core kernels, kept for callers that want the
//                     partial sums.
//   pr_decode_finish: adds the attention over the tokens cached since the last
//                     switch-over, sums the partials, normalises and writes the output.
//   pr_state_merge  : prefill-to-state switch-over: new_state = state*exp(a_last) + S_chunk,
//                     converting the chunk state from the kernels' internal layout to the
//                     exact layout on the fly; same for sum_of_keys from the Gram matrix.
#include <mutex>

#include "host.cuh"
#include "layout.cuh"
#include "sm100.cuh"

namespace pr {

namespace dec {
constexpr int HD = 64;
constexpr int DEX = HD * (HD + 1) / 2;  // 2080
constexpr int THREADS = 256;
constexpr int ROWS_PER_ITER = THREADS / 8;  // 32 state rows per iteration
constexpr int RG_MAX = 4;                   // query heads handled per CTA (template: 1 or 4)
}  // namespace dec

// exact-layout row -> (a, b), a <= b.  Row a starts at off(a) = a d - a (a - 1) / 2; the closed form
// a = floor(((2d + 1) - sqrt((2d + 1)^2 - 8 D)) / 2) is evaluated in fp32 and corrected by at most a
// step either way (a walk over the rows from 0 costs up to d iterations per call, which made the
// layout-converting kernels issue-bound).
__device__ __forceinline__ void exact_decode(int D, int* a, int* b) {
  constexpr int d = dec::HD;
  auto off = [](int r) { return r * d - r * (r - 1) / 2; };
  int aa = (int)(((float)(2 * d + 1) - sqrtf((float)((2 * d + 1) * (2 * d + 1)) - 8.f * (float)D)) * 0.5f);
  aa = max(0, min(aa, d - 1));
  while (aa + 1 <= d - 1 && off(aa + 1) <= D) ++aa;
  while (aa > 0 && off(aa) > D) --aa;
  *a = aa;
  *b = aa + (D - off(aa));
}

template <typename T, int RG>
__global__ void __launch_bounds__(dec::THREADS)
decode_state_kernel(const T* __restrict__ Q, const T* __restrict__ state, const float* __restrict__ sok,
                    const float* __restrict__ a_last, long long a_batch_stride, long long q_bs, float scale, int h,
                    int hq, int nsplit, float* __restrict__ part_y, float* __restrict__ part_l) {
  pdl_launch_dependents();
  pdl_wait();
  using namespace dec;
  __shared__ float sq[RG][HD];
  __shared__ float red_y[THREADS / 32][RG][HD];
  __shared__ float red_l[THREADS / 32][RG];
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int bh = blockIdx.x, split = blockIdx.y, grp = blockIdx.z;
  const int batch = bh / h, head = bh % h;
  const int ratio = hq / h;
  const int r0 = grp * RG, nr = min(RG, ratio - r0);

  // gated, scaled, rounded queries of this group (as the reference rounds Q*exp(.) to Q's dtype)
  float f = scale;
  if (a_last != nullptr) f *= __expf(0.5f * a_last[(size_t)batch * a_batch_stride + head]);
  for (int i = tid; i < nr * HD; i += THREADS) {
    const int r = i / HD, e = i % HD;
    const float q = float(Q[(size_t)batch * q_bs + (size_t)(head * ratio + r0 + r) * HD + e]);
    sq[r][e] = float(T(q * f));
  }
  __syncthreads();

  const int rows_per_split = (DEX + nsplit - 1) / nsplit;
  const int d_begin = split * rows_per_split, d_end = min(DEX, d_begin + rows_per_split);
  const int sub = tid & 7;
  int D = d_begin + (tid >> 3);
  int a = 0, b = 0;
  if (D < DEX) exact_decode(D, &a, &b);

  float acc[RG][8];
  float accl[RG];
#pragma unroll
  for (int r = 0; r < RG; ++r) {
    accl[r] = 0.f;
#pragma unroll
    for (int k = 0; k < 8; ++k) acc[r][k] = 0.f;
  }
  const T* sbase = state + (size_t)bh * DEX * HD;
  const float* kbase = sok + (size_t)bh * DEX;
  // four rows per thread in flight: the loads are issued before any of them is used
#ifndef PR_DEC_UN
#define PR_DEC_UN 4
#endif
  constexpr int UN = PR_DEC_UN;
  for (; D < d_end; D += UN * ROWS_PER_ITER) {
    uint4 v[UN];
    float sk[UN];
    int ra[UN], rb[UN];
#pragma unroll
    for (int u = 0; u < UN; ++u) {
      const int Du = D + u * ROWS_PER_ITER;
      ra[u] = a;
      rb[u] = b;
      if (Du < d_end) {
        v[u] = __ldg(reinterpret_cast<const uint4*>(sbase + (size_t)Du * HD + sub * 8));
        sk[u] = __ldg(kbase + Du);
      }
      // advance (a, b) by ROWS_PER_ITER rows of the triangle
      b += ROWS_PER_ITER;
      while (b >= HD && a < HD) {
        b = b - HD + a + 1;
        ++a;
      }
    }
#pragma unroll
    for (int u = 0; u < UN; ++u) {
      if (D + u * ROWS_PER_ITER >= d_end) break;
      float x[8];
      const uint32_t w[4] = {v[u].x, v[u].y, v[u].z, v[u].w};
#pragma unroll
      for (int k = 0; k < 4; ++k) {
        const float2 p2 = Pack2<T>::to_f32(w[k]);
        x[2 * k] = p2.x;
        x[2 * k + 1] = p2.y;
      }
#pragma unroll
      for (int r = 0; r < RG; ++r) {
        if (r < nr) {
          const float phi = float(T(sq[r][min(ra[u], HD - 1)] * sq[r][min(rb[u], HD - 1)]));  // rounded like the inputs
#pragma unroll
          for (int k = 0; k < 8; ++k) acc[r][k] = fmaf(phi, x[k], acc[r][k]);
          accl[r] = fmaf(phi, sk[u], accl[r]);
        }
      }
    }
  }
  // reduce the 4 rows a warp covers (lanes with equal sub), then the 8 warps
#pragma unroll
  for (int r = 0; r < RG; ++r) {
#pragma unroll
    for (int k = 0; k < 8; ++k) {
      float t = acc[r][k];
      t += __shfl_xor_sync(0xffffffffu, t, 8);
      t += __shfl_xor_sync(0xffffffffu, t, 16);
      acc[r][k] = t;
    }
    float t = accl[r];  // every lane of a row holds the same l term: count it once (sub == 0)
    t = (sub == 0) ? t : 0.f;
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) t += __shfl_xor_sync(0xffffffffu, t, off);
    accl[r] = t;
  }
  if (lane < 8) {
#pragma unroll
    for (int r = 0; r < RG; ++r)
#pragma unroll
      for (int k = 0; k < 8; ++k) red_y[warp][r][lane * 8 + k] = acc[r][k];
  }
  if (lane == 0) {
#pragma unroll
    for (int r = 0; r < RG; ++r) red_l[warp][r] = accl[r];
  }
  __syncthreads();
  for (int i = tid; i < nr * HD; i += THREADS) {
    const int r = i / HD, e = i % HD;
    float t = 0.f;
#pragma unroll
    for (int w = 0; w < THREADS / 32; ++w) t += red_y[w][r][e];
    part_y[(((size_t)batch * hq + head * ratio + r0 + r) * nsplit + split) * HD + e] = t;
  }
  if (tid < nr) {
    float t = 0.f;
#pragma unroll
    for (int w = 0; w < THREADS / 32; ++w) t += red_l[w][tid];
    part_l[((size_t)batch * hq + head * ratio + r0 + tid) * nsplit + split] = t;
  }
}

// One CTA per (batch, query head): attention over the tk cached tokens + merge + normalise.
// Eight lanes share a token (16 bytes of its key and value row each), so a warp streams four
// tokens per iteration with fully used 128-byte rows; two iterations are in flight per lane.
template <typename T>
__global__ void __launch_bounds__(128)
decode_finish_kernel(const T* __restrict__ Q, const T* __restrict__ K, const T* __restrict__ V,
                     const float* __restrict__ a, long long q_bs, long long kv_bs, float scale, int tk, int h, int hq,
                     int nsplit, const float* __restrict__ part_y, const float* __restrict__ part_l,
                     T* __restrict__ O) {
  pdl_launch_dependents();
  pdl_wait();
  constexpr int HD = dec::HD;
  __shared__ float red[4][HD + 1];
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int sub = lane & 7, slot = lane >> 3;
  const int batch = blockIdx.x / hq, qh = blockIdx.x % hq;
  const int kvh = qh / (hq / h);
  // this lane's eight query features
  float q[8];
  {
    const uint4 qv = *reinterpret_cast<const uint4*>(Q + (size_t)batch * q_bs + (size_t)qh * HD + sub * 8);
    const uint32_t w[4] = {qv.x, qv.y, qv.z, qv.w};
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      const float2 p2 = Pack2<T>::to_f32(w[k]);
      q[2 * k] = p2.x;
      q[2 * k + 1] = p2.y;
    }
  }
  float y[8];
#pragma unroll
  for (int e = 0; e < 8; ++e) y[e] = 0.f;
  float l = 0.f;
  if (K != nullptr && tk > 0) {
    const float a_q = a ? a[((size_t)batch * tk + tk - 1) * h + kvh] : 0.f;
    const float s2 = scale * scale;
    const T* kb = K + (size_t)batch * kv_bs + (size_t)kvh * HD + sub * 8;
    const T* vb = V + (size_t)batch * kv_bs + (size_t)kvh * HD + sub * 8;
    constexpr int UN = 2;
    // the trip count depends on the warp only: every lane takes part in the shuffles below, lanes
    // whose token lies past the cache contribute zero weight
    for (int base = warp * 4; base < tk; base += 16 * UN) {
      const int j0 = base + slot;
      uint4 kv[UN], vv[UN];
      float aj[UN];
#pragma unroll
      for (int u = 0; u < UN; ++u) {
        const int j = j0 + 16 * u;
        kv[u] = vv[u] = make_uint4(0, 0, 0, 0);
        aj[u] = 0.f;
        if (j < tk) {
          kv[u] = *reinterpret_cast<const uint4*>(kb + (size_t)j * h * HD);
          vv[u] = *reinterpret_cast<const uint4*>(vb + (size_t)j * h * HD);
          if (a) aj[u] = a[((size_t)batch * tk + j) * h + kvh];
        }
      }
#pragma unroll
      for (int u = 0; u < UN; ++u) {
        const int j = j0 + 16 * u;
        const uint32_t kw[4] = {kv[u].x, kv[u].y, kv[u].z, kv[u].w};
        float sdot = 0.f;
#pragma unroll
        for (int k = 0; k < 4; ++k) {
          const float2 p2 = Pack2<T>::to_f32(kw[k]);
          sdot = fmaf(p2.x, q[2 * k], sdot);
          sdot = fmaf(p2.y, q[2 * k + 1], sdot);
        }
        sdot += __shfl_xor_sync(0xffffffffu, sdot, 1);
        sdot += __shfl_xor_sync(0xffffffffu, sdot, 2);
        sdot += __shfl_xor_sync(0xffffffffu, sdot, 4);
        float wgt = (j < tk) ? s2 * sdot * sdot : 0.f;
        if (a && j < tk) wgt *= __expf(a_q - aj[u]);
        if (sub == 0) l += wgt;
        const uint32_t vw[4] = {vv[u].x, vv[u].y, vv[u].z, vv[u].w};
#pragma unroll
        for (int k = 0; k < 4; ++k) {
          const float2 p2 = Pack2<T>::to_f32(vw[k]);
          y[2 * k] = fmaf(wgt, p2.x, y[2 * k]);
          y[2 * k + 1] = fmaf(wgt, p2.y, y[2 * k + 1]);
        }
      }
    }
  }
  // sum over the four token slots of the warp, then over the warps
#pragma unroll
  for (int e = 0; e < 8; ++e) {
    y[e] += __shfl_xor_sync(0xffffffffu, y[e], 8);
    y[e] += __shfl_xor_sync(0xffffffffu, y[e], 16);
  }
#pragma unroll
  for (int off = 16; off > 0; off >>= 1) l += __shfl_xor_sync(0xffffffffu, l, off);
  if (lane < 8) {
#pragma unroll
    for (int e = 0; e < 8; ++e) red[warp][lane * 8 + e] = y[e];
  }
  if (lane == 0) red[warp][HD] = l;
  __syncthreads();
  if (tid < HD) {
    float yt = red[0][tid] + red[1][tid] + red[2][tid] + red[3][tid];
    float lt = red[0][HD] + red[1][HD] + red[2][HD] + red[3][HD];
    if (part_y != nullptr) {
      const size_t base = ((size_t)batch * hq + qh) * nsplit;
      for (int sp = 0; sp < nsplit; ++sp) {
        yt += part_y[(base + sp) * HD + tid];
        lt += part_l[base + sp];
      }
    }
    O[((size_t)batch * hq + qh) * HD + tid] = T(yt * safe_recip(lt));
  }
}

// The whole decode step for one (batch, kv head, group of up to RG query heads) in one CTA, with
// the state read-out on the tensor cores.  Split `blockIdx.y` takes the 64-row state stages
// [st_begin, st_begin + n_st) and the cached tokens [t_begin, t_end).  The gate sums the step needs
// are formed here from log_g itself: the total a_last (the state's decay, folded into the query as
// exp(a_last / 2)) and, per cached token j, the suffix sum of the gates after j, so no
// cumulative-gate scratch is written or read.  With one split the CTA normalises and writes the
// output itself; otherwise it writes partial sums and decode_merge_kernel finishes.
//
// y = phi(q~)^T S is a [1 x 2080] x [2080 x 64] product per query head.  On the CUDA cores it costs
// some 80 issued instructions per 512 bytes of state, which left the step bound by instruction issue
// and by the bytes a 64-register thread can keep in flight, not by HBM.  Here the state never
// passes through registers: one thread streams it with TMA, 64 rows (8 KB) per stage and NSB stages
// in flight per CTA, into 128-byte-swizzled shared memory, where it is the N-major B operand of
// tcgen05.mma; the A operand is one 8-row swizzle atom per stage holding phi(q~) of the group's
// query heads in rows 0..nr-1 and zeros below (the descriptor's 8-row-group stride is 0, so all
// sixteen row groups of the M = 128 product read that one atom and accumulator lanes r, r + 8, ...
// are copies); the fp32 accumulator lives in 64 columns of tensor memory.  The streaming starts
// before the gate sums and the queries are ready, so that serial prologue is hidden.
//
// Roles: warps 0-4 compute the attention over the cached tokens on the CUDA cores, as before
// (gate suffix sums in blocks of 4 * CT tokens, synchronised among themselves with a named barrier),
// at the same time as warp 5 builds the A atoms and the normaliser phi(q~) . sum_of_keys, one
// thread of warp 6 issues the products and one thread of warp 7 drives the TMA ring.  Every wait
// is bounded; a wait that runs out sets the CTA's abort flag and the device status word.
namespace dec {
constexpr int CT = 160;                                    // threads of the cache-attention warps
constexpr int NSB = 5;                                     // state stages in flight per CTA
constexpr int ST_ROWS = 64;                                // state rows per stage
constexpr int B_BYTES = ST_ROWS * HD * 2;                  // 8 KB
constexpr int A_BYTES = 1024;                              // one swizzle atom: 8 rows x 64 K
constexpr int N_STAGES = (DEX + ST_ROWS - 1) / ST_ROWS;    // 33, the last one half full
constexpr int TC_TMEM_COLS = 64;
constexpr int MAX_DEVICES = 64;                               // device ordinals the entry points accept
constexpr int K_BYTES = ST_ROWS * 4;                       // the stage's slice of sum_of_keys
constexpr size_t TC_SMEM = 1024 + (size_t)NSB * (B_BYTES + A_BYTES + K_BYTES);
}  // namespace dec

__device__ __forceinline__ void bar_sync_named(int id, int count) {
  asm volatile("bar.sync %0, %1;" ::"r"(id), "r"(count) : "memory");
}

template <typename T, int RG>
__global__ void __launch_bounds__(dec::THREADS, RG == 1 ? 4 : 2)
decode_tc_kernel(const __grid_constant__ CUtensorMap tm_state, const T* __restrict__ Q, long long q_bs,
                 const T* __restrict__ K, const T* __restrict__ V, long long kv_bs, const float* __restrict__ log_g,
                 long long g_bs, int has_state, const float* __restrict__ sok, float scale, int tk, int h, int hq,
                 int nsplit, float* __restrict__ part_y, float* __restrict__ part_l, T* __restrict__ O,
                 int* __restrict__ status) {
  using namespace dec;
  constexpr int BLK = 4 * CT;  // cached tokens per gate block
  constexpr int CW = CT / 32;  // cache-attention warps
  extern __shared__ uint8_t smem_raw[];
  __shared__ uint64_t b_full[NSB], a_full[NSB], done[NSB], acc_done;
  __shared__ uint32_t tmem_base_s;
  __shared__ int abort_flag;
  __shared__ float sq[RG][HD];                 // gated, scaled, rounded queries (state phase)
  __shared__ __align__(16) float sqr[RG][HD];  // raw queries (attention phase)
  __shared__ float red_y[CW + 1][RG][HD];      // per cache warp, then the state's
  __shared__ float red_l[CW + 1][RG];
  __shared__ float sfx[BLK];
  __shared__ float wsum[THREADS / 32][2];
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  pdl_launch_dependents();
  const int bh = blockIdx.x, split = blockIdx.y, grp = blockIdx.z;
  const int batch = bh / h, head = bh % h;
  const int ratio = hq / h;
  const int r0 = grp * RG, nr = min(RG, ratio - r0);
  const bool gated = (log_g != nullptr) && tk > 0;
  const int t_per = (tk + nsplit - 1) / nsplit;
  const int t_begin = min(tk, split * t_per), t_end = min(tk, t_begin + t_per);
  const int st_per = (N_STAGES + nsplit - 1) / nsplit;
  const int st_begin = min(N_STAGES, split * st_per);
  const int n_st = has_state ? min(N_STAGES, st_begin + st_per) - st_begin : 0;

  const uint32_t sbase = (smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t* smB = smem_raw + (sbase - smem_u32(smem_raw));  // NSB x B_BYTES
  uint8_t* smA = smB + NSB * B_BYTES;                      // NSB x A_BYTES
  uint8_t* smK = smA + NSB * A_BYTES;                      // NSB x K_BYTES
  const float* kbase = sok + (size_t)bh * DEX;

  if (tid == 0) {
    abort_flag = 0;
    for (int s = 0; s < NSB; ++s) {
      mbar_init(&b_full[s], 1);
      mbar_init(&a_full[s], 1);
      mbar_init(&done[s], 1);
    }
    mbar_init(&acc_done, 1);
    fence_mbar_init();
  }
  // rows nr..7 of every A atom stay zero for the whole kernel
  for (int i = tid; i < NSB * A_BYTES / 16; i += THREADS) reinterpret_cast<uint4*>(smA)[i] = make_uint4(0, 0, 0, 0);
  fence_async_smem();
  if (warp == 0 && n_st > 0) {
    tmem_alloc(&tmem_base_s, TC_TMEM_COLS);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = n_st > 0 ? tmem_base_s : 0u;
  pdl_wait();  // everything above overlaps the tail of the kernel before this one

  // the first stages are requested before anything else is known
  if (warp == 7 && lane == 0) {
    for (int it = 0; it < min(n_st, NSB); ++it) {
      const int D0 = (st_begin + it) * ST_ROWS;
      const uint32_t kb = (uint32_t)min(ST_ROWS, DEX - D0) * 4u;
      mbar_expect_tx(&b_full[it], B_BYTES + kb);
      tma_load_3d(smB + it * B_BYTES, &tm_state, &b_full[it], 0, D0, bh);
      bulk_load_1d(smK + it * K_BYTES, kbase + D0, kb, &b_full[it]);
    }
  }

  // ---- gate sums: the total, and the part after this split's last token
  float a_last = 0.f, tail = 0.f;
  if (gated) {
    const float* gp = log_g + (size_t)batch * g_bs + head;
    float tot = 0.f, tl = 0.f;
    for (int u = tid; u < tk; u += THREADS) {
      const float g = gp[(size_t)u * h];
      tot += g;
      if (u >= t_end) tl += g;
    }
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) {
      tot += __shfl_xor_sync(0xffffffffu, tot, off);
      tl += __shfl_xor_sync(0xffffffffu, tl, off);
    }
    if (lane == 0) {
      wsum[warp][0] = tot;
      wsum[warp][1] = tl;
    }
    __syncthreads();
#pragma unroll
    for (int w = 0; w < THREADS / 32; ++w) {
      a_last += wsum[w][0];
      tail += wsum[w][1];
    }
    __syncthreads();
  }
  const float f = scale * (gated ? __expf(0.5f * a_last) : 1.f);
  for (int i = tid; i < RG * HD; i += THREADS) {
    const int r = i / HD, e = i % HD;
    float q = 0.f;
    if (r < nr) q = float(Q[(size_t)batch * q_bs + (size_t)(head * ratio + r0 + r) * HD + e]);
    sqr[r][e] = q;
    sq[r][e] = float(T(q * f));  // rounded like the reference rounds Q * exp(.) to Q's dtype
  }
  __syncthreads();

  const int sub = tid & 7;
  if (warp < CW) {
    // ------------------------------------------------ cached tokens, newest block first
    float acc[RG][8];
    float accl[RG];
#pragma unroll
    for (int r = 0; r < RG; ++r) {
      accl[r] = 0.f;
#pragma unroll
      for (int k = 0; k < 8; ++k) acc[r][k] = 0.f;
    }
    if (K != nullptr && t_end > t_begin) {
      const float s2 = scale * scale;
      const int slot = lane >> 3;
      const T* kb = K + (size_t)batch * kv_bs + (size_t)head * HD + sub * 8;
      const T* vb = V + (size_t)batch * kv_bs + (size_t)head * HD + sub * 8;
      float q[RG][8];
#pragma unroll
      for (int r = 0; r < RG; ++r) {
        const float4 q0 = *reinterpret_cast<const float4*>(&sqr[r][sub * 8]);
        const float4 q1 = *reinterpret_cast<const float4*>(&sqr[r][sub * 8 + 4]);
        q[r][0] = q0.x; q[r][1] = q0.y; q[r][2] = q0.z; q[r][3] = q0.w;
        q[r][4] = q1.x; q[r][5] = q1.y; q[r][6] = q1.z; q[r][7] = q1.w;
      }
      for (int blk_end = t_end; blk_end > t_begin; blk_end -= BLK) {
        const int blk_lo = max(t_begin, blk_end - BLK);
        const int n_blk = blk_end - blk_lo;
        if (gated) {
          // sfx[i] = sum of the gates after token blk_lo + i (up to the newest token of the cache)
          const float* gp = log_g + (size_t)batch * g_bs + head;
          float g4[4];
#pragma unroll
          for (int k = 0; k < 4; ++k) {
            const int i = 4 * tid + k;
            g4[k] = i < n_blk ? gp[(size_t)(blk_lo + i) * h] : 0.f;
          }
          const float mine = g4[0] + g4[1] + g4[2] + g4[3];
          // inclusive reverse scan of the per-thread totals over the block
          float inc = mine;
#pragma unroll
          for (int off = 1; off < 32; off <<= 1) {
            const float o = __shfl_down_sync(0xffffffffu, inc, off);
            if (lane + off < 32) inc += o;
          }
          if (lane == 0) wsum[warp][0] = inc;
          bar_sync_named(1, CT);
          float after = tail;  // everything after this thread's four tokens
#pragma unroll
          for (int w = 0; w < CW; ++w) {
            if (w > warp) after += wsum[w][0];
          }
          after += inc - mine;
          float blk_total = 0.f;
#pragma unroll
          for (int w = 0; w < CW; ++w) blk_total += wsum[w][0];
          sfx[4 * tid + 3] = after;
          sfx[4 * tid + 2] = after + g4[3];
          sfx[4 * tid + 1] = after + g4[3] + g4[2];
          sfx[4 * tid + 0] = after + g4[3] + g4[2] + g4[1];
          tail += blk_total;
          bar_sync_named(1, CT);
        }
        constexpr int UNT = 2;
        // the trip count depends on the warp only: every lane takes part in the shuffles, lanes whose
        // token lies outside the block contribute zero weight
        for (int base = warp * 4; base < n_blk; base += CW * 4 * UNT) {
          uint4 kv[UNT], vv[UNT];
          float sf[UNT];
#pragma unroll
          for (int u = 0; u < UNT; ++u) {
            const int i = base + slot + CW * 4 * u;
            kv[u] = vv[u] = make_uint4(0, 0, 0, 0);
            sf[u] = 0.f;
            if (i < n_blk) {
              const size_t j = (size_t)(blk_lo + i);
              kv[u] = *reinterpret_cast<const uint4*>(kb + j * h * HD);
              vv[u] = *reinterpret_cast<const uint4*>(vb + j * h * HD);
              if (gated) sf[u] = sfx[i];
            }
          }
#pragma unroll
          for (int u = 0; u < UNT; ++u) {
            const int i = base + slot + CW * 4 * u;
            const uint32_t kw[4] = {kv[u].x, kv[u].y, kv[u].z, kv[u].w};
            const uint32_t vw[4] = {vv[u].x, vv[u].y, vv[u].z, vv[u].w};
            float kf[8], vf[8];
#pragma unroll
            for (int k = 0; k < 4; ++k) {
              const float2 p2 = Pack2<T>::to_f32(kw[k]);
              kf[2 * k] = p2.x;
              kf[2 * k + 1] = p2.y;
              const float2 v2 = Pack2<T>::to_f32(vw[k]);
              vf[2 * k] = v2.x;
              vf[2 * k + 1] = v2.y;
            }
            const float gf = (i < n_blk) ? (gated ? s2 * __expf(sf[u]) : s2) : 0.f;
#pragma unroll
            for (int r = 0; r < RG; ++r) {
              float sdot = 0.f;
#pragma unroll
              for (int k = 0; k < 8; ++k) sdot = fmaf(kf[k], q[r][k], sdot);
              sdot += __shfl_xor_sync(0xffffffffu, sdot, 1);
              sdot += __shfl_xor_sync(0xffffffffu, sdot, 2);
              sdot += __shfl_xor_sync(0xffffffffu, sdot, 4);
              const float wgt = gf * sdot * sdot;
              if (sub == 0) accl[r] += wgt;
#pragma unroll
              for (int k = 0; k < 8; ++k) acc[r][k] = fmaf(wgt, vf[k], acc[r][k]);
            }
          }
        }
        if (gated) bar_sync_named(1, CT);  // sfx is rewritten by the next block
      }
    }
    // the four tokens a warp covers per pass (lanes with equal sub)
#pragma unroll
    for (int r = 0; r < RG; ++r) {
#pragma unroll
      for (int k = 0; k < 8; ++k) {
        float t = acc[r][k];
        t += __shfl_xor_sync(0xffffffffu, t, 8);
        t += __shfl_xor_sync(0xffffffffu, t, 16);
        acc[r][k] = t;
      }
      float t = accl[r];
#pragma unroll
      for (int off = 16; off > 0; off >>= 1) t += __shfl_xor_sync(0xffffffffu, t, off);
      accl[r] = t;
    }
    if (lane < 8) {
#pragma unroll
      for (int r = 0; r < RG; ++r)
#pragma unroll
        for (int k = 0; k < 8; ++k) red_y[warp][r][lane * 8 + k] = acc[r][k];
    }
    if (lane == 0) {
#pragma unroll
      for (int r = 0; r < RG; ++r) red_l[warp][r] = accl[r];
    }
    if (warp == CW - 1) {
      // this warp owns tensor-memory lanes 0-31: fetch the state's share of the output
      bool have = n_st > 0 && mbar_wait(&acc_done, 0, &abort_flag);
      if (have) tc_fence_after();
#pragma unroll
      for (int j = 0; j < HD / 16; ++j) {
        uint32_t v[16];
        if (have) {
          tmem_ld16(tmem + j * 16, v);
          tmem_wait_ld();
        }
        if (lane < RG) {
#pragma unroll
          for (int k = 0; k < 16; ++k) red_y[CW][lane][j * 16 + k] = have ? __uint_as_float(v[k]) : 0.f;
        }
      }
    }
  } else if (warp == 5) {
    // ------------------------------------------------ A atoms and the normaliser
    float l_acc[RG];
#pragma unroll
    for (int r = 0; r < RG; ++r) l_acc[r] = 0.f;
    if (n_st > 0) {
      int D = st_begin * ST_ROWS + 2 * lane;  // this lane's rows D and D + 1 of every stage
      int a = 0, b = 0;
      exact_decode(min(D, DEX - 1), &a, &b);
      const uint32_t a_off = swz128(0, lane >> 2) + (lane & 3) * 4;
      for (int it = 0; it < n_st; ++it) {
        const int s = it % NSB;
        if (it >= NSB && !mbar_wait(&done[s], ((it / NSB) - 1) & 1, &abort_flag)) break;
        if (!mbar_wait(&b_full[s], (it / NSB) & 1, &abort_flag)) break;  // the stage's sum_of_keys slice
        const bool in = D < DEX;  // D is even and so is DEX: D + 1 is inside whenever D is
        int a1 = a, b1 = b + 1;
        if (b1 >= HD) {
          a1 = min(a + 1, HD - 1);
          b1 = a1;
        }
        float2 sk = make_float2(0.f, 0.f);
        if (in) sk = *reinterpret_cast<const float2*>(smK + s * K_BYTES + 8 * lane);
#pragma unroll
        for (int r = 0; r < RG; ++r) {
          if (r < nr) {
            const uint32_t w = in ? Pack2<T>::from_f32(sq[r][a] * sq[r][b], sq[r][a1] * sq[r][b1]) : 0u;
            // row r of the atom: swz128(r, c) = r * 128 + ((c ^ r) << 4) for r < 8
            *reinterpret_cast<uint32_t*>(smA + s * A_BYTES + r * 128 + ((a_off ^ (r << 4)))) = w;
            const float2 ph = Pack2<T>::to_f32(w);
            l_acc[r] = fmaf(ph.x, sk.x, fmaf(ph.y, sk.y, l_acc[r]));
          }
        }
        fence_async_smem();
        __syncwarp();
        if (lane == 0) mbar_arrive(&a_full[s]);
        D += ST_ROWS;
        b += ST_ROWS;
        while (b >= HD && a < HD - 1) {
          b = b - HD + a + 1;
          ++a;
        }
        b = min(b, HD - 1);
      }
    }
#pragma unroll
    for (int r = 0; r < RG; ++r) {
      float t = l_acc[r];
#pragma unroll
      for (int off = 16; off > 0; off >>= 1) t += __shfl_xor_sync(0xffffffffu, t, off);
      if (lane == 0) red_l[CW][r] = t;
    }
  } else if (warp == 6) {
    // ------------------------------------------------ MMA issuer
    if (lane == 0 && n_st > 0) {
      const uint32_t idesc = umma_idesc(128, HD, Pack2<T>::is_bf16, false, true);
      bool ok = true;
      for (int it = 0; it < n_st; ++it) {
        const int s = it % NSB, ph = (it / NSB) & 1;
        ok = mbar_wait(&b_full[s], ph, &abort_flag) && mbar_wait(&a_full[s], ph, &abort_flag);
        if (!ok) break;
        tc_fence_after();
        const uint32_t a_addr = smem_u32(smA + s * A_BYTES), b_addr = smem_u32(smB + s * B_BYTES);
#pragma unroll
        for (int ks = 0; ks < ST_ROWS / 16; ++ks)
          umma_ss(tmem, umma_desc_sw128(a_addr + ks * 32, 16, 0), umma_desc_sw128(b_addr + ks * 2048, 8192, 1024), idesc,
                  (it > 0 || ks > 0) ? 1u : 0u);
        umma_commit(&done[s]);
      }
      if (ok) umma_commit(&acc_done);
    }
  } else {
    // ------------------------------------------------ TMA producer, stages NSB and up
    if (lane == 0) {
      for (int it = NSB; it < n_st; ++it) {
        const int s = it % NSB;
        if (!mbar_wait(&done[s], ((it / NSB) - 1) & 1, &abort_flag)) break;
        const int D0 = (st_begin + it) * ST_ROWS;
        const uint32_t kb = (uint32_t)min(ST_ROWS, DEX - D0) * 4u;
        mbar_expect_tx(&b_full[s], B_BYTES + kb);
        tma_load_3d(smB + s * B_BYTES, &tm_state, &b_full[s], 0, D0, bh);
        bulk_load_1d(smK + s * K_BYTES, kbase + D0, kb, &b_full[s]);
      }
    }
  }

  tc_fence_before();
  __syncthreads();
  if (tid == 0 && abort_flag) *status = ST_TIMEOUT;
  for (int i = tid; i < nr * HD; i += THREADS) {
    const int r = i / HD, e = i % HD;
    float yt = 0.f, lt = 0.f;
#pragma unroll
    for (int w = 0; w <= CW; ++w) {
      yt += red_y[w][r][e];
      lt += red_l[w][r];
    }
    const size_t row = (size_t)batch * hq + head * ratio + r0 + r;
    if (nsplit == 1) {
      O[row * HD + e] = T(yt * safe_recip(lt));
    } else {
      part_y[(row * nsplit + split) * HD + e] = yt;
      if (e == 0) part_l[row * nsplit + split] = lt;
    }
  }
  if (warp == 0 && n_st > 0) tmem_dealloc(tmem, TC_TMEM_COLS);
}


// Sums the partial results of a split decode step, normalises and writes the output.
template <typename T>
__global__ void __launch_bounds__(dec::HD)
decode_merge_kernel(const float* __restrict__ part_y, const float* __restrict__ part_l, int nsplit, T* __restrict__ O) {
  pdl_launch_dependents();
  pdl_wait();
  const size_t row = blockIdx.x;
  const int e = threadIdx.x;
  float yt = 0.f, lt = 0.f;
  for (int sp = 0; sp < nsplit; ++sp) {
    yt += part_y[(row * nsplit + sp) * dec::HD + e];
    lt += part_l[row * nsplit + sp];
  }
  O[row * dec::HD + e] = T(yt * safe_recip(lt));
}

// Cumulative log gates of the cached tokens, a[b, tk, h] (dense) from log_g whose batch entries are
// g_bs floats apart (a cache kept as a slice of a longer preallocated tensor).  One CTA per
// (batch, head); tk is small (below the switch-over length), so one block-wide scan per 256 tokens.
__global__ void __launch_bounds__(256)
decode_gate_cumsum_kernel(const float* __restrict__ log_g, long long g_bs, float* __restrict__ a, int tk, int h) {
  pdl_launch_dependents();
  pdl_wait();
  __shared__ float warp_tot[8];
  __shared__ float carry_s;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int batch = blockIdx.x / h, head = blockIdx.x % h;
  if (tid == 0) carry_s = 0.f;
  __syncthreads();
  for (int base = 0; base < tk; base += 256) {
    const int i = base + tid;
    float v = (i < tk) ? log_g[(size_t)batch * g_bs + (size_t)i * h + head] : 0.f;
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
    if (i < tk) a[((size_t)batch * tk + i) * h + head] = v;
    __syncthreads();
    if (tid == 255) carry_s = v;
    __syncthreads();
  }
}

// new_state (exact layout) = decay * state + S (chunk-state layout); new_sok = decay * sok + w * gram.
template <typename T>
__global__ void state_merge_kernel(const T* __restrict__ state, const float* __restrict__ sok,
                                   const T* __restrict__ S, const float* __restrict__ gram,
                                   const float* __restrict__ a_last, T* __restrict__ new_state,
                                   float* __restrict__ new_sok, int bh_total) {
  pdl_launch_dependents();
  pdl_wait();
  constexpr int HD = dec::HD, DEX = dec::DEX, DR = ref_dim(HD);
  const size_t gid = (size_t)blockIdx.x * blockDim.x + threadIdx.x;  // one thread per 8 elements
  const size_t total = (size_t)bh_total * DEX * 8;
  if (gid >= total) return;
  const int sub = (int)(gid & 7);
  const size_t rowg = gid >> 3;
  const int D = (int)(rowg % DEX);
  const int bh = (int)(rowg / DEX);
  int a, b;
  exact_decode(D, &a, &b);
  // chunk-state rows of the pair: (a, b) always exists (a <= b); inside a 16-block the mirrored
  // entry (b, a) holds the other half of the pair's weight
  const int yb = b >> 4;
  const int row1 = ref_block_base(yb) + 16 * a + (b & 15);
  const bool mirrored = (a != b) && ((a >> 4) == yb);
  const int row2 = ref_block_base(yb) + 16 * b + (a & 15);
  const float decay = (state != nullptr) ? (a_last ? __expf(a_last[bh]) : 1.f) : 0.f;
  const uint4 sv = *reinterpret_cast<const uint4*>(S + ((size_t)bh * DR + row1) * HD + sub * 8);
  uint4 sv2 = make_uint4(0, 0, 0, 0);
  if (mirrored) sv2 = *reinterpret_cast<const uint4*>(S + ((size_t)bh * DR + row2) * HD + sub * 8);
  uint4 ov = make_uint4(0, 0, 0, 0);
  if (state != nullptr) ov = *reinterpret_cast<const uint4*>(state + ((size_t)bh * DEX + D) * HD + sub * 8);
  const uint32_t sw[4] = {sv.x, sv.y, sv.z, sv.w}, sw2[4] = {sv2.x, sv2.y, sv2.z, sv2.w},
                 ow[4] = {ov.x, ov.y, ov.z, ov.w};
  uint32_t rw[4];
#pragma unroll
  for (int k = 0; k < 4; ++k) {
    const float2 s2 = Pack2<T>::to_f32(sw[k]), s3 = Pack2<T>::to_f32(sw2[k]), o2 = Pack2<T>::to_f32(ow[k]);
    // the reference rounds state*decay to the state dtype before adding (:374-382)
    const float2 od = Pack2<T>::to_f32(Pack2<T>::from_f32(o2.x * decay, o2.y * decay));
    rw[k] = Pack2<T>::from_f32(od.x + s2.x + s3.x, od.y + s2.y + s3.y);
  }
  *reinterpret_cast<uint4*>(new_state + ((size_t)bh * DEX + D) * HD + sub * 8) = make_uint4(rw[0], rw[1], rw[2], rw[3]);
  if (sub == 0) {
    const float g = gram[((size_t)bh * HD + a) * HD + b] * (a == b ? 1.f : 2.f);
    new_sok[(size_t)bh * DEX + D] = (sok != nullptr ? sok[(size_t)bh * DEX + D] * decay : 0.f) + g;
  }
}

// Inverse of the switch-over conversion: a state in the exact layout (as inference keeps it) into
// the chunk-state layout the training kernels read, as 16-bit rows (a state for pr_chunk_out) and /
// or as an fp32 carry for the scans; sum_of_keys into the Gram matrix (fp32 and / or hi + lo
// 16-bit halves).  Pairs stored twice in the chunk layout (both indices in one 16-block) get half
// of the exact entry each.
template <typename T>
__global__ void state_to_chunk_kernel(const T* __restrict__ state, const float* __restrict__ sok,
                                      T* __restrict__ out16, float* __restrict__ out32, float* __restrict__ gram,
                                      T* __restrict__ ghi, T* __restrict__ glo, int bh_total) {
  pdl_launch_dependents();
  pdl_wait();
  constexpr int HD = dec::HD, DEX = dec::DEX, DR = ref_dim(HD);
  const size_t gid = (size_t)blockIdx.x * blockDim.x + threadIdx.x;  // one thread per 8 elements
  if (gid < (size_t)bh_total * HD * HD && (gram || ghi)) {
    const int bh = (int)(gid / (HD * HD)), a = (int)(gid / HD) % HD, b = (int)(gid % HD);
    const int lo = min(a, b), hi = max(a, b);
    const float v = sok[(size_t)bh * DEX + lo * HD - lo * (lo - 1) / 2 + (hi - lo)] * (a == b ? 1.f : 0.5f);
    if (gram) gram[gid] = v;
    if (ghi) {
      const T hv = T(v);
      ghi[gid] = hv;
      glo[gid] = T(v - float(hv));
    }
  }
  if (gid >= (size_t)bh_total * DR * 8) return;
  const int sub = (int)(gid & 7);
  const size_t rowg = gid >> 3;
  const int r = (int)(rowg % DR);
  const int bh = (int)(rowg / DR);
  int a, b;
  ref_decode(r, &a, &b);
  const int lo = min(a, b), hi = max(a, b);
  const float coef = (a != b && (a >> 4) == (b >> 4)) ? 0.5f : 1.f;
  const uint4 sv =
      *reinterpret_cast<const uint4*>(state + ((size_t)bh * DEX + lo * HD - lo * (lo - 1) / 2 + (hi - lo)) * HD + sub * 8);
  const uint32_t sw[4] = {sv.x, sv.y, sv.z, sv.w};
  float x[8];
#pragma unroll
  for (int k = 0; k < 4; ++k) {
    const float2 p2 = Pack2<T>::to_f32(sw[k]);
    x[2 * k] = p2.x * coef;
    x[2 * k + 1] = p2.y * coef;
  }
  const size_t o = ((size_t)bh * DR + r) * HD + sub * 8;
  if (out16)
    *reinterpret_cast<uint4*>(out16 + o) = make_uint4(Pack2<T>::from_f32(x[0], x[1]), Pack2<T>::from_f32(x[2], x[3]),
                                                      Pack2<T>::from_f32(x[4], x[5]), Pack2<T>::from_f32(x[6], x[7]));
  if (out32) {
    *reinterpret_cast<float4*>(out32 + o) = make_float4(x[0], x[1], x[2], x[3]);
    *reinterpret_cast<float4*>(out32 + o + 4) = make_float4(x[4], x[5], x[6], x[7]);
  }
}

}  // namespace pr

#ifndef PR_DEC_NSPLIT
#define PR_DEC_NSPLIT 5
#endif
extern "C" int pr_decode_nsplit(void) { return PR_DEC_NSPLIT; }

namespace pr {
// Splits of the expanded dimension actually used for a problem (<= pr_decode_nsplit(), which sizes
// the partial-sum workspace).  A CTA that walks all 2080 rows of its (batch, head) state amortises
// its prologue and reduction best - 71 % of the measured copy bandwidth at 512 CTAs against 57 %
// with five splits - so the read is only split when there are too few (batch, head) pairs to fill
// the GPU.  Both kernels of a step derive the count from the same sizes.
static int decode_split(int b, int h, int hq) {
  const int ratio = hq / h;
  const int rg = ratio == 1 ? 1 : dec::RG_MAX;
  const long long ctas = (long long)b * h * ((ratio + rg - 1) / rg);
  return ctas >= 384 ? 1 : (ctas >= 160 ? 2 : PR_DEC_NSPLIT);
}
}  // namespace pr

// Parts a decode step of this shape is split into (1: no partial-sum workspace is needed).
extern "C" int pr_decode_split(int b, int h, int hq) {
  if (b <= 0 || h <= 0 || hq <= 0 || hq % h != 0) return pr::fail(PR_ERR_BAD_ARG, "bad sizes b=%d h=%d hq=%d", b, h, hq);
  return pr::decode_split(b, h, hq);
}

extern "C" int pr_decode_state(int dtype, int b, int h, int hq, int d, const void* Q, const void* state,
                               const float* sum_of_keys, const float* a_last, float scale, float* part_y,
                               float* part_l, int device, void* stream) {
  return pr_decode_state_strided(dtype, b, h, hq, d, Q, state, sum_of_keys, a_last, h, scale, part_y, part_l, device,
                                 stream);
}

namespace pr {
static int launch_decode_state(int dtype, int b, int h, int hq, int d, const void* Q, long long q_bs, const void* state,
                               const float* sum_of_keys, const float* a_last, long long a_batch_stride, float scale,
                               float* part_y, float* part_l, int device, void* stream);
static int launch_decode_finish(int dtype, int b, int tk, int h, int hq, int d, const void* Q, long long q_bs,
                                const void* K, const void* V, long long kv_bs, const float* a, float scale,
                                const float* part_y, const float* part_l, void* O, int device, void* stream);
}  // namespace pr

extern "C" int pr_decode_state_strided(int dtype, int b, int h, int hq, int d, const void* Q, const void* state,
                                       const float* sum_of_keys, const float* a_last, long long a_batch_stride,
                                       float scale, float* part_y, float* part_l, int device, void* stream) {
  return pr::launch_decode_state(dtype, b, h, hq, d, Q, (long long)hq * d, state, sum_of_keys, a_last, a_batch_stride,
                                 scale, part_y, part_l, device, stream);
}

static int pr::launch_decode_state(int dtype, int b, int h, int hq, int d, const void* Q, long long q_bs,
                                   const void* state, const float* sum_of_keys, const float* a_last,
                                   long long a_batch_stride, float scale, float* part_y, float* part_l, int device,
                                   void* stream) {
  using namespace pr;
  PR_REQUIRE(d == dec::HD, PR_ERR_BAD_ARG, "head dim %d: this build handles d = 64", d);
  PR_REQUIRE(b > 0 && h > 0 && hq > 0 && hq % h == 0, PR_ERR_BAD_ARG, "bad sizes b=%d h=%d hq=%d", b, h, hq);
  PR_REQUIRE(Q && state && sum_of_keys && part_y && part_l && aligned16(state) && aligned16(Q), PR_ERR_BAD_ARG,
             "null or misaligned pointer");
  PR_CUDA(cudaSetDevice(device));
  const int nsplit = decode_split(b, h, hq);
  const int ratio = hq / h;
  const int rg = ratio == 1 ? 1 : dec::RG_MAX;
  dim3 grid(b * h, nsplit, (ratio + rg - 1) / rg);
  cudaStream_t s = static_cast<cudaStream_t>(stream);
#define PR_LAUNCH_DECODE(TT, RGV)                                                                              \
  PR_CUDA(launch(decode_state_kernel<TT, RGV>, dim3(grid), dim3(dec::THREADS), 0, s, static_cast<const TT*>(Q), static_cast<const TT*>(state), \
                                                             sum_of_keys, a_last, a_batch_stride, q_bs, scale, h,    \
                                                             hq, nsplit, part_y, part_l))
  if (dtype == PR_BF16) {
    if (rg == 1) PR_LAUNCH_DECODE(__nv_bfloat16, 1); else PR_LAUNCH_DECODE(__nv_bfloat16, 4);
  } else if (dtype == PR_FP16) {
    if (rg == 1) PR_LAUNCH_DECODE(__half, 1); else PR_LAUNCH_DECODE(__half, 4);
  } else {
    return fail(PR_ERR_BAD_ARG, "dtype %d", dtype);
  }
#undef PR_LAUNCH_DECODE
  PR_CUDA(cudaGetLastError());
  return PR_OK;
}

extern "C" int pr_decode_finish(int dtype, int b, int tk, int h, int hq, int d, const void* Q, const void* K,
                                const void* V, const float* a, float scale, const float* part_y, const float* part_l,
                                void* O, int device, void* stream) {
  return pr::launch_decode_finish(dtype, b, tk, h, hq, d, Q, (long long)hq * d, K, V, (long long)tk * h * d, a, scale,
                                  part_y, part_l, O, device, stream);
}

static int pr::launch_decode_finish(int dtype, int b, int tk, int h, int hq, int d, const void* Q, long long q_bs,
                                    const void* K, const void* V, long long kv_bs, const float* a, float scale,
                                    const float* part_y, const float* part_l, void* O, int device, void* stream) {
  using namespace pr;
  PR_REQUIRE(kv_bs % 8 == 0 && q_bs % 8 == 0 && aligned16(Q), PR_ERR_BAD_ARG,
             "Q must be 16-byte aligned and the batch strides of Q, K, V multiples of 8 elements");
  PR_REQUIRE(d == dec::HD, PR_ERR_BAD_ARG, "head dim %d: this build handles d = 64", d);
  PR_REQUIRE(b > 0 && h > 0 && hq > 0 && hq % h == 0 && tk >= 0, PR_ERR_BAD_ARG, "bad sizes");
  PR_REQUIRE(Q && O && aligned16(K) && aligned16(V), PR_ERR_BAD_ARG, "null or misaligned pointer");
  PR_REQUIRE((part_y == nullptr) == (part_l == nullptr), PR_ERR_BAD_ARG, "partials must come together");
  PR_REQUIRE(part_y != nullptr || (K != nullptr && tk > 0), PR_ERR_BAD_ARG, "neither a state nor cached tokens");
  PR_CUDA(cudaSetDevice(device));
  const int nsplit = decode_split(b, h, hq);
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  if (dtype == PR_BF16)
    PR_CUDA(launch(decode_finish_kernel<__nv_bfloat16>, dim3(b * hq), dim3(128), 0, s, 
        static_cast<const __nv_bfloat16*>(Q), static_cast<const __nv_bfloat16*>(K),
        static_cast<const __nv_bfloat16*>(V), a, q_bs, kv_bs, scale, tk, h, hq, nsplit, part_y, part_l,
        static_cast<__nv_bfloat16*>(O)));
  else if (dtype == PR_FP16)
    PR_CUDA(launch(decode_finish_kernel<__half>, dim3(b * hq), dim3(128), 0, s, static_cast<const __half*>(Q), static_cast<const __half*>(K),
                                                        static_cast<const __half*>(V), a, q_bs, kv_bs, scale, tk, h, hq,
                                                        nsplit,
                                                        part_y, part_l, static_cast<__half*>(O)));
  else
    return fail(PR_ERR_BAD_ARG, "dtype %d", dtype);
  PR_CUDA(cudaGetLastError());
  return PR_OK;
}

extern "C" int pr_state_merge(int dtype, int b, int h, int d, const void* state, const float* sum_of_keys,
                              const void* S, const float* gram, const float* a_last, void* new_state,
                              float* new_sum_of_keys, int device, void* stream) {
  using namespace pr;
  PR_REQUIRE(d == dec::HD, PR_ERR_BAD_ARG, "head dim %d: this build handles d = 64", d);
  PR_REQUIRE(b > 0 && h > 0, PR_ERR_BAD_ARG, "bad sizes");
  PR_REQUIRE(S && gram && new_state && new_sum_of_keys && aligned16(S) && aligned16(new_state) && aligned16(state),
             PR_ERR_BAD_ARG, "null or misaligned pointer");
  PR_REQUIRE((state == nullptr) == (sum_of_keys == nullptr), PR_ERR_BAD_ARG, "state and sum_of_keys come together");
  PR_CUDA(cudaSetDevice(device));
  const size_t threads = (size_t)b * h * dec::DEX * 8;
  const unsigned grid = (unsigned)((threads + 255) / 256);
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  if (dtype == PR_BF16)
    PR_CUDA(launch(state_merge_kernel<__nv_bfloat16>, dim3(grid), dim3(256), 0, s, 
        static_cast<const __nv_bfloat16*>(state), sum_of_keys, static_cast<const __nv_bfloat16*>(S), gram, a_last,
        static_cast<__nv_bfloat16*>(new_state), new_sum_of_keys, b * h));
  else if (dtype == PR_FP16)
    PR_CUDA(launch(state_merge_kernel<__half>, dim3(grid), dim3(256), 0, s, static_cast<const __half*>(state), sum_of_keys,
                                                    static_cast<const __half*>(S), gram, a_last,
                                                    static_cast<__half*>(new_state), new_sum_of_keys, b * h));
  else
    return fail(PR_ERR_BAD_ARG, "dtype %d", dtype);
  PR_CUDA(cudaGetLastError());
  return PR_OK;
}

// Exact-layout state [b,h,2080,d] and sum_of_keys [b,h,2080] -> chunk-state layout: out16 [b,h,D2,d]
// (16-bit, a state pr_chunk_out can read), out32 (the same in fp32: a carry for pr_discumsum_fwd), gram
// [b,h,d,d] fp32 (carry for pr_gram_scan_fwd), gram_hi / gram_lo (16-bit halves for pr_chunk_out).  Any output
// may be NULL.  The layout change of layout.exact_to_reference as one kernel.
extern "C" int pr_state_to_chunk_layout(int dtype, int b, int h, int d, const void* state, const float* sum_of_keys,
                                        void* out16, float* out32, float* gram, void* gram_hi, void* gram_lo,
                                        int device, void* stream) {
  using namespace pr;
  PR_REQUIRE(d == dec::HD, PR_ERR_BAD_ARG, "head dim %d: this build handles d = 64", d);
  PR_REQUIRE(b > 0 && h > 0 && state && sum_of_keys, PR_ERR_BAD_ARG, "bad sizes or null inputs");
  PR_REQUIRE(aligned16(state) && aligned16(out16) && aligned16(out32), PR_ERR_BAD_ARG, "misaligned pointer");
  PR_REQUIRE((gram_hi == nullptr) == (gram_lo == nullptr), PR_ERR_BAD_ARG, "gram_hi and gram_lo come together");
  PR_CUDA(cudaSetDevice(device));
  const size_t threads = (size_t)b * h * ref_dim(d) * 8;
  const unsigned grid = (unsigned)((threads + 255) / 256);
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  if (dtype == PR_BF16)
    PR_CUDA(launch(state_to_chunk_kernel<__nv_bfloat16>, dim3(grid), dim3(256), 0, s, 
        static_cast<const __nv_bfloat16*>(state), sum_of_keys, static_cast<__nv_bfloat16*>(out16), out32, gram,
        static_cast<__nv_bfloat16*>(gram_hi), static_cast<__nv_bfloat16*>(gram_lo), b * h));
  else if (dtype == PR_FP16)
    PR_CUDA(launch(state_to_chunk_kernel<__half>, dim3(grid), dim3(256), 0, s, static_cast<const __half*>(state), sum_of_keys,
                                                      static_cast<__half*>(out16), out32, gram,
                                                      static_cast<__half*>(gram_hi), static_cast<__half*>(gram_lo), b * h));
  else
    return fail(PR_ERR_BAD_ARG, "dtype %d", dtype);
  PR_CUDA(cudaGetLastError());
  return PR_OK;
}

// Cumulative log gates of whole sequences, a[b, t, h] = cumsum_t log_g (the reference's
// log_G.cumsum(1), retention/power_retention_maker.py:129,347), for any t: one CTA per (batch, head)
// walks the sequence in blocks of 256 tokens.  Serves the state-free quadratic branch and long caches,
// where the chunk-local gate pass (pr_gate_prep) would not fit a chunk in shared memory.
extern "C" int pr_gate_cumsum(int b, int t, int h, const float* log_g, long long g_bstride, float* a_out, int device,
                              void* stream) {
  using namespace pr;
  PR_REQUIRE(b > 0 && t > 0 && h > 0 && g_bstride >= (long long)t * h, PR_ERR_BAD_ARG, "bad sizes b=%d t=%d h=%d", b,
             t, h);
  PR_REQUIRE(log_g && a_out, PR_ERR_BAD_ARG, "null pointer");
  PR_CUDA(cudaSetDevice(device));
  PR_CUDA(launch(decode_gate_cumsum_kernel, dim3(b * h), dim3(256), 0, static_cast<cudaStream_t>(stream), log_g, g_bstride, a_out, t, h));
  PR_CUDA(cudaGetLastError());
  return PR_OK;
}

// One decode step in a single call (one kernel; a second, tiny one when the work of a (batch, head)
// pair is split over several CTAs because there are too few pairs to fill the GPU): gate sums of the
// cached tokens, state read-out, attention over the cache, merge, normalisation.
// part_y / part_l as for pr_decode_state; they are touched only when the step is split
// (b * h * ceil(ratio / 4) < 384 CTAs).  a_scratch is not used any more (the gate sums are formed
// inside the kernel) and may be NULL; the argument stays so that existing callers keep working.
extern "C" int pr_decode_step(int dtype, int b, int tk, int h, int hq, int d, const void* Q, const void* K,
                              const void* V, const float* log_g, const void* state, const float* sum_of_keys,
                              float scale, float* a_scratch, float* part_y, float* part_l, void* O, int device,
                              void* stream) {
  return pr_decode_step_strided(dtype, b, tk, h, hq, d, Q, (long long)hq * d, K, V, (long long)tk * h * d, log_g,
                                (long long)tk * h, state, sum_of_keys, scale, a_scratch, part_y, part_l, O, device,
                                stream);
}

// The same step for a query and a cache that are slices of longer preallocated tensors: batch
// entry i of Q starts q_bstride elements after entry i-1, of K and V kv_bstride elements, of
// log_g g_bstride floats; inside a batch entry the tensors are dense ([1,hq,d], [tk,h,d], [tk,h]).
extern "C" int pr_decode_step_strided(int dtype, int b, int tk, int h, int hq, int d, const void* Q,
                                      long long q_bstride, const void* K, const void* V, long long kv_bstride,
                                      const float* log_g, long long g_bstride, const void* state,
                                      const float* sum_of_keys, float scale, float* a_scratch, float* part_y,
                                      float* part_l, void* O, int device, void* stream) {
  using namespace pr;
  (void)a_scratch;
  const bool has_cache = (K != nullptr && V != nullptr && tk > 0);
  const bool gated = has_cache && log_g != nullptr;
  PR_REQUIRE(d == dec::HD, PR_ERR_BAD_ARG, "head dim %d: this build handles d = 64", d);
  PR_REQUIRE(b > 0 && h > 0 && hq > 0 && hq % h == 0 && tk >= 0, PR_ERR_BAD_ARG, "bad sizes");
  PR_REQUIRE(dtype == PR_BF16 || dtype == PR_FP16, PR_ERR_BAD_ARG, "dtype %d", dtype);
  PR_REQUIRE(state != nullptr || has_cache, PR_ERR_BAD_ARG, "neither a state nor cached tokens");
  PR_REQUIRE(state == nullptr || sum_of_keys != nullptr, PR_ERR_BAD_ARG, "a state needs its sum_of_keys");
  PR_REQUIRE(Q && O && aligned16(Q) && aligned16(K) && aligned16(V) && aligned16(state) && aligned16(sum_of_keys),
             PR_ERR_BAD_ARG, "null or misaligned pointer");
  PR_REQUIRE(q_bstride >= (long long)hq * d && (!has_cache || kv_bstride >= (long long)tk * h * d) &&
                 (!gated || g_bstride >= (long long)tk * h),
             PR_ERR_BAD_ARG, "a batch stride is smaller than one batch entry");
  PR_REQUIRE(q_bstride % 8 == 0 && (!has_cache || kv_bstride % 8 == 0), PR_ERR_BAD_ARG,
             "the batch strides of Q, K, V must be multiples of 8 elements");
  PR_REQUIRE(device >= 0 && device < dec::MAX_DEVICES, PR_ERR_BAD_ARG, "device ordinal %d out of range", device);
  const int nsplit = decode_split(b, h, hq);
  PR_REQUIRE(nsplit == 1 || (part_y != nullptr && part_l != nullptr), PR_ERR_BAD_ARG,
             "this problem is split %d ways and needs the partial-sum workspace", nsplit);
  PR_CUDA(cudaSetDevice(device));
  const int ratio = hq / h;
  const int rg = ratio == 1 ? 1 : dec::RG_MAX;
  dim3 grid(b * h, nsplit, (ratio + rg - 1) / rg);
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  int* status = nullptr;
  int rc = status_word(device, &status, nullptr);
  if (rc) return rc;
  CUtensorMap tm_state;
  {
    // without a state the map is never used; it still has to be a valid one
    const void* base = state ? state : Q;
    uint64_t dims[3] = {(uint64_t)dec::HD, (uint64_t)(state ? dec::DEX : 1), (uint64_t)(state ? b * h : 1)};
    uint64_t strides[3] = {0, (uint64_t)dec::HD * 2, (uint64_t)dec::DEX * dec::HD * 2};
    uint32_t box[3] = {(uint32_t)dec::HD, (uint32_t)(state ? dec::ST_ROWS : 1), 1};
    rc = make_tmap(&tm_state, base, 2, 3, dims, strides, box, true);
    if (rc) return rc;
  }
#define PR_LAUNCH_FUSED(TT, RGV)                                                                                      \
  do {                                                                                                                \
    static bool configured[dec::MAX_DEVICES] = {false}; /* per instantiation and device */                           \
    if (!configured[device]) {                                                                                        \
      PR_CUDA(cudaFuncSetAttribute(decode_tc_kernel<TT, RGV>, cudaFuncAttributeMaxDynamicSharedMemorySize,            \
                                   (int)dec::TC_SMEM));                                                               \
      PR_CUDA(cudaFuncSetAttribute(decode_tc_kernel<TT, RGV>, cudaFuncAttributePreferredSharedMemoryCarveout, 100));  \
      configured[device] = true;                                                                                      \
    }                                                                                                                 \
    PR_CUDA(launch(decode_tc_kernel<TT, RGV>, dim3(grid), dim3(dec::THREADS), dec::TC_SMEM, s,                                                \
        tm_state, static_cast<const TT*>(Q), q_bstride, static_cast<const TT*>(has_cache ? K : nullptr),              \
        static_cast<const TT*>(has_cache ? V : nullptr), kv_bstride, gated ? log_g : nullptr, g_bstride,              \
        state != nullptr ? 1 : 0, sum_of_keys, scale, has_cache ? tk : 0, h, hq, nsplit, part_y, part_l,              \
        static_cast<TT*>(O), status));                                                                                 \
  } while (0)
  if (dtype == PR_BF16) {
    if (rg == 1) PR_LAUNCH_FUSED(__nv_bfloat16, 1); else PR_LAUNCH_FUSED(__nv_bfloat16, 4);
  } else {
    if (rg == 1) PR_LAUNCH_FUSED(__half, 1); else PR_LAUNCH_FUSED(__half, 4);
  }
#undef PR_LAUNCH_FUSED
  PR_CUDA(cudaGetLastError());
  if (nsplit > 1) {
    if (dtype == PR_BF16)
      PR_CUDA(launch(decode_merge_kernel<__nv_bfloat16>, dim3(b * hq), dim3(dec::HD), 0, s, part_y, part_l, nsplit, static_cast<__nv_bfloat16*>(O)));
    else
      PR_CUDA(launch(decode_merge_kernel<__half>, dim3(b * hq), dim3(dec::HD), 0, s, part_y, part_l, nsplit, static_cast<__half*>(O)));
    PR_CUDA(cudaGetLastError());
  }
  return PR_OK;
}

namespace pr {
// Pure-recurrent decode step: the state is advanced by one token and read in the same pass,
//     S' = e^g S + phi_K(k) v^T,   z' = e^g z + phi_K(k),   y = phi(s q)^T S' / phi(s q) . z'
// which is the reference's inference step with switch_over_seq_len = 1 (one cached token, then
// compression, retention/power_retention_maker.py:354-382) without the cache round trip.  Every
// state row is read once and written once.
//
// The state is streamed by TMA in both directions (same roles and rings as
// decode_tc_kernel).  A 64-row stage lands in swizzled shared memory and the tensor core contracts it,
// as stored, with phi(s q); once those products have completed, warps 0-3 advance the stage in place,
//     S' = round(round(e^g S) + phi_K(k) v^T),
// and one thread of warp 4 hands it to a TMA store into new_state.  The output is
//     y = e^g (phi(s q)^T S) + (phi(s q) . phi_K(k)) v,
// i.e. the stored state is read as the reference's query_state reads it and the new token enters
// exactly, as it does through the reference's attention over the one cached token
// (power_retention_maker.py:354-363) - not through the 16-bit rounding of the advanced state.
// Warp 5 advances the stage's slice of sum_of_keys, writes it, and forms the normaliser, the token's
// weight phi(s q) . phi_K(k) and the A atoms.  A ring slot is refilled once its store has read it.
// In place (new_state == state) every stage is loaded before it is stored and no other CTA touches
// it; with several groups of query heads per kv head only group 0 stores, and the buffers must differ.
template <typename T, int RG>
__global__ void __launch_bounds__(dec::THREADS, RG == 1 ? 4 : 2)
decode_recurrent_tc_kernel(const __grid_constant__ CUtensorMap tm_state, const __grid_constant__ CUtensorMap tm_new,
                           const T* __restrict__ Q, long long q_bs, const T* __restrict__ Kt,
                           const T* __restrict__ Vt, long long kv_bs, const float* __restrict__ log_g, long long g_bs,
                           const float* sok, float* new_sok, float scale, int h, int hq, int nsplit,
                           float* __restrict__ part_y, float* __restrict__ part_l, T* __restrict__ O,
                           int* __restrict__ status) {
  using namespace dec;
  constexpr int UW = 4;  // warps advancing the state
  extern __shared__ uint8_t smem_raw[];
  __shared__ uint64_t b_full[NSB], u_full[NSB], a_full[NSB], done[NSB], st_done[NSB], acc_done;
  __shared__ uint32_t tmem_base_s;
  __shared__ int abort_flag;
  __shared__ float sq[RG][HD];
  __shared__ float skv[2][HD];  // the token's key and value
  __shared__ float red_y[RG][HD];
  __shared__ float red_l[RG], red_c[RG];
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  pdl_launch_dependents();
  const int bh = blockIdx.x, split = blockIdx.y, grp = blockIdx.z;
  const int batch = bh / h, head = bh % h;
  const int ratio = hq / h;
  const int r0 = grp * RG, nr = min(RG, ratio - r0);
  const bool writer = (grp == 0);  // one group of query heads writes the new state
  const int st_per = (N_STAGES + nsplit - 1) / nsplit;
  const int st_begin = min(N_STAGES, split * st_per);
  const int n_st = min(N_STAGES, st_begin + st_per) - st_begin;

  const uint32_t sbase = (smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t* smB = smem_raw + (sbase - smem_u32(smem_raw));  // NSB x B_BYTES
  uint8_t* smA = smB + NSB * B_BYTES;                      // NSB x A_BYTES
  uint8_t* smK = smA + NSB * A_BYTES;                      // NSB x K_BYTES
  const float* kbase = sok + (size_t)bh * DEX;

  if (tid == 0) {
    abort_flag = 0;
    for (int s = 0; s < NSB; ++s) {
      mbar_init(&b_full[s], 1);
      mbar_init(&u_full[s], UW);
      mbar_init(&a_full[s], 1);
      mbar_init(&done[s], 1);
      mbar_init(&st_done[s], 1);
    }
    mbar_init(&acc_done, 1);
    fence_mbar_init();
  }
  for (int i = tid; i < NSB * A_BYTES / 16; i += THREADS) reinterpret_cast<uint4*>(smA)[i] = make_uint4(0, 0, 0, 0);
  fence_async_smem();
  if (warp == 0 && n_st > 0) {
    tmem_alloc(&tmem_base_s, TC_TMEM_COLS);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = n_st > 0 ? tmem_base_s : 0u;
  pdl_wait();  // everything above overlaps the tail of the kernel before this one

  if (warp == 7 && lane == 0) {
    for (int it = 0; it < min(n_st, NSB); ++it) {
      const int D0 = (st_begin + it) * ST_ROWS;
      const uint32_t kb = (uint32_t)min(ST_ROWS, DEX - D0) * 4u;
      mbar_expect_tx(&b_full[it], B_BYTES + kb);
      tma_load_3d(smB + it * B_BYTES, &tm_state, &b_full[it], 0, D0, bh);
      bulk_load_1d(smK + it * K_BYTES, kbase + D0, kb, &b_full[it]);
    }
  }

  const float decay = log_g ? __expf(log_g[(size_t)batch * g_bs + head]) : 1.f;
  for (int i = tid; i < RG * HD; i += THREADS) {
    const int r = i / HD, e = i % HD;
    float q = 0.f;
    if (r < nr) q = float(Q[(size_t)batch * q_bs + (size_t)(head * ratio + r0 + r) * HD + e]);
    sq[r][e] = float(T(q * scale));
  }
  if (tid < 2 * HD) {
    const T* src = (tid < HD ? Kt : Vt) + (size_t)batch * kv_bs + (size_t)head * HD + (tid & (HD - 1));
    skv[tid / HD][tid & (HD - 1)] = float(*src);
  }
  __syncthreads();

  if (warp < UW) {
    // ------------------------------------------------ the state, advanced in place in shared memory
    const int sub = tid & 7, row16 = tid >> 3;  // this thread's 16-byte column group and row within a pass
    float vt[8];
#pragma unroll
    for (int k = 0; k < 8; ++k) vt[k] = skv[1][sub * 8 + k];
    int D = st_begin * ST_ROWS + row16;
    int a = 0, b = 0;
    exact_decode(min(D, DEX - 1), &a, &b);
    for (int it = 0; it < n_st; ++it) {
      const int s = it % NSB;
      if (!mbar_wait(&done[s], (it / NSB) & 1, &abort_flag)) break;  // the stage has been read as stored
      uint8_t* tile = smB + s * B_BYTES;
#pragma unroll
      for (int ps = 0; ps < ST_ROWS / 16; ++ps) {
        const int r = row16 + 16 * ps;
        if (writer && D < DEX) {
          uint4* cell = reinterpret_cast<uint4*>(tile + swz128(r, sub));
          const uint4 v = *cell;
          // key-side expansion entry of the new token, rounded like the inputs, with the pair weight
          const float phik = float(T(skv[0][a] * skv[0][b])) * (a == b ? 1.f : 2.f);
          const uint32_t w[4] = {v.x, v.y, v.z, v.w};
          uint32_t ow[4];
#pragma unroll
          for (int k = 0; k < 4; ++k) {
            const float2 p2 = Pack2<T>::to_f32(w[k]);
            // the reference rounds state * decay to the state's dtype before adding the update (:374-382)
            const float2 od = Pack2<T>::to_f32(Pack2<T>::from_f32(p2.x * decay, p2.y * decay));
            ow[k] = Pack2<T>::from_f32(fmaf(phik, vt[2 * k], od.x), fmaf(phik, vt[2 * k + 1], od.y));
          }
          *cell = make_uint4(ow[0], ow[1], ow[2], ow[3]);
        }
        D += 16;
        b += 16;
        while (b >= HD && a < HD - 1) {
          b = b - HD + a + 1;
          ++a;
        }
        b = min(b, HD - 1);
      }
      fence_async_smem();
      __syncwarp();
      if (lane == 0) mbar_arrive(&u_full[s]);
    }
  } else if (warp == 4) {
    // ------------------------------------------------ stores of the advanced stages, then the output
    if (lane == 0 && n_st > 0) {
      bool ok = true;
      for (int it = 0; it < n_st; ++it) {
        const int s = it % NSB;
        ok = mbar_wait(&u_full[s], (it / NSB) & 1, &abort_flag);
        if (!ok) break;
        if (writer) {
          tma_store_3d(&tm_new, smB + s * B_BYTES, 0, (st_begin + it) * ST_ROWS, bh);
          bulk_commit_group();
          bulk_wait_group_read<1>();  // the store before this one has read its stage
        }
        if (it > 0) mbar_arrive(&st_done[(it - 1) % NSB]);
      }
      bulk_wait_group_read<0>();
      if (ok) mbar_arrive(&st_done[(n_st - 1) % NSB]);
      bulk_wait_group<0>();  // the stores are performed before this CTA is done
    }
    __syncwarp();
    // this warp owns tensor-memory lanes 0-31: fetch the output
    const bool have = n_st > 0 && mbar_wait(&acc_done, 0, &abort_flag);
    if (have) tc_fence_after();
#pragma unroll
    for (int j = 0; j < HD / 16; ++j) {
      uint32_t v[16];
      if (have) {
        tmem_ld16(tmem + j * 16, v);
        tmem_wait_ld();
      }
      if (lane < RG) {
#pragma unroll
        for (int k = 0; k < 16; ++k) red_y[lane][j * 16 + k] = have ? __uint_as_float(v[k]) : 0.f;
      }
    }
  } else if (warp == 5) {
    // ------------------------------------------------ sum_of_keys, the normaliser and the A atoms
    float l_acc[RG], c_acc[RG];
#pragma unroll
    for (int r = 0; r < RG; ++r) l_acc[r] = c_acc[r] = 0.f;
    if (n_st > 0) {
      int D = st_begin * ST_ROWS + 2 * lane;  // this lane's rows D and D + 1 of every stage
      int a = 0, b = 0;
      exact_decode(min(D, DEX - 1), &a, &b);
      float* okbase = new_sok + (size_t)bh * DEX;
      const uint32_t a_off = swz128(0, lane >> 2) + (lane & 3) * 4;
      for (int it = 0; it < n_st; ++it) {
        const int s = it % NSB;
        if (it >= NSB && !mbar_wait(&done[s], ((it / NSB) - 1) & 1, &abort_flag)) break;
        if (!mbar_wait(&b_full[s], (it / NSB) & 1, &abort_flag)) break;  // the stage's sum_of_keys slice
        const bool in = D < DEX;  // D is even and so is DEX: D + 1 is inside whenever D is
        int a1 = a, b1 = b + 1;
        if (b1 >= HD) {
          a1 = min(a + 1, HD - 1);
          b1 = a1;
        }
        float2 sk = make_float2(0.f, 0.f), pk = make_float2(0.f, 0.f);
        if (in) {
          sk = *reinterpret_cast<const float2*>(smK + s * K_BYTES + 8 * lane);
          pk.x = float(T(skv[0][a] * skv[0][b])) * (a == b ? 1.f : 2.f);
          pk.y = float(T(skv[0][a1] * skv[0][b1])) * (a1 == b1 ? 1.f : 2.f);
          sk.x = fmaf(sk.x, decay, pk.x);
          sk.y = fmaf(sk.y, decay, pk.y);
          if (writer) *reinterpret_cast<float2*>(okbase + D) = sk;
        }
#pragma unroll
        for (int r = 0; r < RG; ++r) {
          if (r < nr) {
            const uint32_t w = in ? Pack2<T>::from_f32(sq[r][a] * sq[r][b], sq[r][a1] * sq[r][b1]) : 0u;
            *reinterpret_cast<uint32_t*>(smA + s * A_BYTES + r * 128 + ((a_off ^ (r << 4)))) = w;
            const float2 ph = Pack2<T>::to_f32(w);
            l_acc[r] = fmaf(ph.x, sk.x, fmaf(ph.y, sk.y, l_acc[r]));
            c_acc[r] = fmaf(ph.x, pk.x, fmaf(ph.y, pk.y, c_acc[r]));
          }
        }
        fence_async_smem();
        __syncwarp();
        if (lane == 0) mbar_arrive(&a_full[s]);
        D += ST_ROWS;
        b += ST_ROWS;
        while (b >= HD && a < HD - 1) {
          b = b - HD + a + 1;
          ++a;
        }
        b = min(b, HD - 1);
      }
    }
#pragma unroll
    for (int r = 0; r < RG; ++r) {
      float t = l_acc[r], u = c_acc[r];
#pragma unroll
      for (int off = 16; off > 0; off >>= 1) {
        t += __shfl_xor_sync(0xffffffffu, t, off);
        u += __shfl_xor_sync(0xffffffffu, u, off);
      }
      if (lane == 0) {
        red_l[r] = t;
        red_c[r] = u;
      }
    }
  } else if (warp == 6) {
    // ------------------------------------------------ MMA issuer: products on the stages as stored
    if (lane == 0 && n_st > 0) {
      const uint32_t idesc = umma_idesc(128, HD, Pack2<T>::is_bf16, false, true);
      bool ok = true;
      for (int it = 0; it < n_st; ++it) {
        const int s = it % NSB, ph = (it / NSB) & 1;
        ok = mbar_wait(&b_full[s], ph, &abort_flag) && mbar_wait(&a_full[s], ph, &abort_flag);
        if (!ok) break;
        tc_fence_after();
        const uint32_t a_addr = smem_u32(smA + s * A_BYTES), b_addr = smem_u32(smB + s * B_BYTES);
#pragma unroll
        for (int ks = 0; ks < ST_ROWS / 16; ++ks)
          umma_ss(tmem, umma_desc_sw128(a_addr + ks * 32, 16, 0), umma_desc_sw128(b_addr + ks * 2048, 8192, 1024), idesc,
                  (it > 0 || ks > 0) ? 1u : 0u);
        umma_commit(&done[s]);
      }
      if (ok) umma_commit(&acc_done);
    }
  } else {
    // ------------------------------------------------ TMA loads, stages NSB and up
    if (lane == 0) {
      for (int it = NSB; it < n_st; ++it) {
        const int s = it % NSB;
        if (!mbar_wait(&st_done[s], ((it / NSB) - 1) & 1, &abort_flag)) break;  // stored, hence read and advanced
        const int D0 = (st_begin + it) * ST_ROWS;
        const uint32_t kb = (uint32_t)min(ST_ROWS, DEX - D0) * 4u;
        mbar_expect_tx(&b_full[s], B_BYTES + kb);
        tma_load_3d(smB + s * B_BYTES, &tm_state, &b_full[s], 0, D0, bh);
        bulk_load_1d(smK + s * K_BYTES, kbase + D0, kb, &b_full[s]);
      }
    }
  }

  tc_fence_before();
  __syncthreads();
  if (tid == 0 && abort_flag) *status = ST_TIMEOUT;
  for (int i = tid; i < nr * HD; i += THREADS) {
    const int r = i / HD, e = i % HD;
    const float yt = fmaf(decay, red_y[r][e], red_c[r] * skv[1][e]), lt = red_l[r];
    const size_t row = (size_t)batch * hq + head * ratio + r0 + r;
    if (nsplit == 1) {
      O[row * HD + e] = T(yt * safe_recip(lt));
    } else {
      part_y[(row * nsplit + split) * HD + e] = yt;
      if (e == 0) part_l[row * nsplit + split] = lt;
    }
  }
  if (warp == 0 && n_st > 0) tmem_dealloc(tmem, TC_TMEM_COLS);
}

}  // namespace pr

// Pure-recurrent decode step (see decode_recurrent_tc_kernel): q [b,1,hq,d], k, v [b,1,h,d] (batch
// entries q_bstride / kv_bstride elements apart), log_g [b,1,h] (g_bstride floats apart) or NULL.
// new_state / new_sum_of_keys may alias state / sum_of_keys when hq / h <= 4 (each state row is then
// read and written by one thread only); with more query heads per kv head they must be other buffers.
extern "C" int pr_decode_recurrent(int dtype, int b, int h, int hq, int d, const void* Q, long long q_bstride,
                                   const void* K, const void* V, long long kv_bstride, const float* log_g,
                                   long long g_bstride, const void* state, const float* sum_of_keys, void* new_state,
                                   float* new_sum_of_keys, float scale, float* part_y, float* part_l, void* O,
                                   int device, void* stream) {
  using namespace pr;
  PR_REQUIRE(d == dec::HD, PR_ERR_BAD_ARG, "head dim %d: this build handles d = 64", d);
  PR_REQUIRE(b > 0 && h > 0 && hq > 0 && hq % h == 0, PR_ERR_BAD_ARG, "bad sizes b=%d h=%d hq=%d", b, h, hq);
  PR_REQUIRE(dtype == PR_BF16 || dtype == PR_FP16, PR_ERR_BAD_ARG, "dtype %d", dtype);
  PR_REQUIRE(Q && K && V && state && sum_of_keys && new_state && new_sum_of_keys && O, PR_ERR_BAD_ARG, "null pointer");
  PR_REQUIRE(aligned16(Q) && aligned16(state) && aligned16(new_state) && aligned16(sum_of_keys) &&
                 aligned16(new_sum_of_keys),
             PR_ERR_BAD_ARG, "misaligned pointer");
  PR_REQUIRE(device >= 0 && device < dec::MAX_DEVICES, PR_ERR_BAD_ARG, "device ordinal %d out of range", device);
  PR_REQUIRE(q_bstride >= (long long)hq * d && kv_bstride >= (long long)h * d && (!log_g || g_bstride >= h),
             PR_ERR_BAD_ARG, "a batch stride is smaller than one batch entry");
  const int ratio = hq / h;
  const int rg = ratio == 1 ? 1 : dec::RG_MAX;
  const int groups = (ratio + rg - 1) / rg;
  PR_REQUIRE(groups == 1 || (new_state != state && new_sum_of_keys != sum_of_keys), PR_ERR_BAD_ARG,
             "in-place update needs hq / h <= %d", dec::RG_MAX);
  const int nsplit = decode_split(b, h, hq);
  PR_REQUIRE(nsplit == 1 || (part_y != nullptr && part_l != nullptr), PR_ERR_BAD_ARG,
             "this problem is split %d ways and needs the partial-sum workspace", nsplit);
  PR_CUDA(cudaSetDevice(device));
  dim3 grid(b * h, nsplit, groups);
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  int* status = nullptr;
  int rc = status_word(device, &status, nullptr);
  if (rc) return rc;
  CUtensorMap tm_state, tm_new;
  {
    uint64_t dims[3] = {(uint64_t)dec::HD, (uint64_t)dec::DEX, (uint64_t)b * h};
    uint64_t strides[3] = {0, (uint64_t)dec::HD * 2, (uint64_t)dec::DEX * dec::HD * 2};
    uint32_t box[3] = {(uint32_t)dec::HD, (uint32_t)dec::ST_ROWS, 1};
    if ((rc = make_tmap(&tm_state, state, 2, 3, dims, strides, box, true))) return rc;
    if ((rc = make_tmap(&tm_new, new_state, 2, 3, dims, strides, box, true))) return rc;
  }
#define PR_LAUNCH_REC(TT, RGV)                                                                                        \
  do {                                                                                                                \
    static bool configured[dec::MAX_DEVICES] = {false}; /* per instantiation and device */                           \
    if (!configured[device]) {                                                                                        \
      PR_CUDA(cudaFuncSetAttribute(decode_recurrent_tc_kernel<TT, RGV>, cudaFuncAttributeMaxDynamicSharedMemorySize,  \
                                   (int)dec::TC_SMEM));                                                               \
      PR_CUDA(cudaFuncSetAttribute(decode_recurrent_tc_kernel<TT, RGV>,                                               \
                                   cudaFuncAttributePreferredSharedMemoryCarveout, 100));                             \
      configured[device] = true;                                                                                      \
    }                                                                                                                 \
    PR_CUDA(launch(decode_recurrent_tc_kernel<TT, RGV>, grid, dim3(dec::THREADS), dec::TC_SMEM, s, tm_state, tm_new,  \
                   static_cast<const TT*>(Q), q_bstride, static_cast<const TT*>(K), static_cast<const TT*>(V),        \
                   kv_bstride, log_g, g_bstride, sum_of_keys, new_sum_of_keys, scale, h, hq, nsplit, part_y, part_l,  \
                   static_cast<TT*>(O), status));                                                                     \
  } while (0)
  if (dtype == PR_BF16) {
    if (rg == 1) PR_LAUNCH_REC(__nv_bfloat16, 1); else PR_LAUNCH_REC(__nv_bfloat16, 4);
  } else {
    if (rg == 1) PR_LAUNCH_REC(__half, 1); else PR_LAUNCH_REC(__half, 4);
  }
#undef PR_LAUNCH_REC
  PR_CUDA(cudaGetLastError());
  if (nsplit > 1) {
    if (dtype == PR_BF16)
      PR_CUDA(launch(decode_merge_kernel<__nv_bfloat16>, dim3(b * hq), dim3(dec::HD), 0, s, part_y, part_l, nsplit, static_cast<__nv_bfloat16*>(O)));
    else
      PR_CUDA(launch(decode_merge_kernel<__half>, dim3(b * hq), dim3(dec::HD), 0, s, part_y, part_l, nsplit, static_cast<__half*>(O)));
    PR_CUDA(cudaGetLastError());
  }
  return PR_OK;
}

// ---------------------------------------------------------------------------------------
// Decode step for callers that must not allocate.
//
// pr_decode_step needs scratch memory from its caller whenever the step is split over several
// CTAs per (batch, head) pair: the partial sums of the parts.  Some hosts of this library
// cannot provide it: a serving loop that froze its memory pool after start-up, or a process
// whose device allocator belongs to a different component and hands out nothing at request
// time.  (The entry point still makes CUDA runtime calls - set device, launches, a one-time
// symbol lookup - so it is not for host callbacks enqueued on a stream, which may make none.)
// For them the same step is offered with its scratch in the fixed device array below, which
// every GPU that loads this library carries until the process exits (kStaticScratchBytes,
// about 1.3 MB).
//
// Limit: batch * query_heads <= kStaticMaxRows; larger problems are refused with
// PR_ERR_BAD_ARG.  All calls on a device share the one array: two calls whose kernels overlap
// on the GPU (different streams, or different threads) race on it, so keep such calls on one
// stream.  Nothing in the array has to start at zero - each call overwrites every word it later
// reads - so stale contents of the previous call are harmless.  The device address of the array
// is looked up the first time the entry point runs on a device; make that first call outside
// any stream capture.
namespace pr {
namespace {
constexpr int kStaticMaxRows = 1024;                                              // batch * query heads
constexpr int kStaticSplit = PR_DEC_NSPLIT;                                       // == pr_decode_nsplit()
constexpr size_t kStaticPartY = (size_t)kStaticMaxRows * kStaticSplit * dec::HD;  // floats
constexpr size_t kStaticPartL = (size_t)kStaticMaxRows * kStaticSplit;
constexpr size_t kStaticFloats = kStaticPartY + kStaticPartL;
constexpr size_t kStaticScratchBytes = kStaticFloats * sizeof(float);

static __device__ __align__(256) float g_decode_scratch[kStaticFloats];

constexpr int kStaticMaxDevices = 64;
float* g_scratch_addr[kStaticMaxDevices] = {nullptr};  // device address of the array, per device
std::mutex g_scratch_mu;

// In host code `g_decode_scratch` names a host-side shadow, not device memory; the address a
// kernel may use has to be asked for, with the target device current.
int static_scratch(int device, float** out) {
  PR_REQUIRE(device >= 0 && device < kStaticMaxDevices, PR_ERR_BAD_ARG, "device ordinal %d out of range", device);
  std::lock_guard<std::mutex> lock(g_scratch_mu);
  if (g_scratch_addr[device] == nullptr) {
    void* p = nullptr;
    PR_CUDA(cudaGetSymbolAddress(&p, g_decode_scratch));
    PR_REQUIRE(p != nullptr, PR_ERR_CUDA, "cudaGetSymbolAddress returned a null address");
    g_scratch_addr[device] = static_cast<float*>(p);
  }
  *out = g_scratch_addr[device];
  return PR_OK;
}
}  // namespace
}  // namespace pr

extern "C" int pr_decode_step_static(int dtype, int b, int tk, int h, int hq, int d, const void* Q, const void* K,
                                     const void* V, const float* log_g, const void* state, const float* sum_of_keys,
                                     float scale, void* O, int device, void* stream) {
  using namespace pr;
  PR_REQUIRE(b > 0 && h > 0 && hq > 0 && tk >= 0, PR_ERR_BAD_ARG, "bad sizes b=%d h=%d hq=%d tk=%d", b, h, hq, tk);
  PR_REQUIRE(pr_decode_nsplit() == kStaticSplit, PR_ERR_BAD_ARG, "static scratch was sized for another split count");
  PR_REQUIRE((long long)b * hq <= kStaticMaxRows, PR_ERR_BAD_ARG,
             "batch * query heads = %lld exceeds the static scratch limit of %d rows", (long long)b * hq,
             kStaticMaxRows);
  PR_REQUIRE(device >= 0 && device < kStaticMaxDevices, PR_ERR_BAD_ARG, "device ordinal %d out of range", device);
  PR_CUDA(cudaSetDevice(device));
  float* scratch = nullptr;
  int rc = static_scratch(device, &scratch);
  if (rc) return rc;
  float* part_y = scratch;
  float* part_l = scratch + kStaticPartY;
  return pr_decode_step(dtype, b, tk, h, hq, d, Q, K, V, log_g, state, sum_of_keys, scale, nullptr, part_y, part_l, O,
                        device, stream);
}
