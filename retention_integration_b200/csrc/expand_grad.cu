// Gradient of the symmetric-power expansion with respect to its argument:
//     dphi_i[(a,b)] = sum_e W[i,e] * State[(a,b), e]         (tensor cores, K = 64)
//     dx~_i[a] += dphi_i[(a,b)] * x~_i[b],  dx~_i[b] += dphi_i[(a,b)] * x~_i[a]   (CUDA cores)
//     dx~_i    += g_i * mult * Gs x~_i                        (Gram part: tensor cores)
// and the chain rule through the gate factor f_i (x~ = round(x f_i)):
//     dX_i = dx~_i * f_i,     gdot_i = <x~_i, dx~_i> / 2      (the gate-gradient term).
//
// Query side (gradient of the state read-out, retention/_query_state/triton.py:181-325):
//   W = dO / l, State = Z_m (state entering the chunk), Gs = Zg_m, g_i = dl_i, mult = 2,
//   f_i = s * exp(a_i / 2).
// Key side (gradient of the chunk state, retention/_update_state/reference.py:55-83):
//   W = V, State = w (.) dS_m, Gs = dG_m + dG_m^T, g_i = 1, mult = 1, f_i = exp((A_m - a_i)/2).
//
// One CTA owns one row tile of 128 tokens of one (batch, chunk, head) and two CTAs share an SM
// (Cfg<1>; Cfg<2> is the earlier shape, two row tiles in one CTA per SM, 7 % slower: measured
// 0.302 vs 0.282 ms per launch at b1 t65536 h8).  The expansion gradient dphi is never written to
// memory: tiles of 128 expanded rows are produced in tensor memory, two buffers per row tile, and
// drained by the row tile's four warps while the tensor core fills the other buffer.  Each thread owns one token row and keeps x~ and dx~ in registers; the
// triangle's (a, b) pattern is resolved at compile time, so the drain is two FMAs per entry.
#include <type_traits>

#include "host.cuh"
#include "layout.cuh"
#include "sm100.cuh"

namespace pr {

namespace eg {
constexpr int HD = 64;
constexpr int D2 = ref_dim(HD);          // 2560 expanded rows (block layout, see layout.cuh)
constexpr int NT = D2 / 128;             // 20 tiles of 128 rows = 8 first factors x 16
constexpr int TILE_BYTES = 128 * 128;
constexpr int G_BYTES = 64 * 128;
// NRT row tiles of 128 tokens per CTA.  Warps: 4 NRT drain warps (one group of four per row tile), one
// TMA warp, 2 NRT issuing warps (two threads per row tile).
//   NRT = 2: one CTA per SM; each state tile fetched from L2 feeds two products.
//   NRT = 1: two CTAs per SM, so that one CTA's prologue (operand loads, gating, Gram part) and epilogue
//            (write-out) - a quarter of a CTA's life, all of it on the drain warps - run while the other
//            CTA drains; the state tiles are fetched once per row tile, and the Gram operand borrows
//            the last slot of the state ring until the Gram products have completed.
template <int NRT>
struct Cfg {
  static constexpr int THREADS = 32 * (6 * NRT + 1);
  static constexpr int ROWS = 128 * NRT;
  static constexpr int NSS = NRT == 2 ? 4 : 2;  // state tiles in flight per CTA (64 KB per SM either way)
  static constexpr bool G_IN_RING = NRT == 1;
  static constexpr uint32_t TMEM_COLS = 256 * NRT;
  static constexpr size_t SMEM =
      1024 + (size_t)(2 * NRT + NSS) * TILE_BYTES + (G_IN_RING ? 0 : 2 * G_BYTES) + (size_t)NRT * 64 * 128 * 4;
};
#ifndef PR_EG_NRT
#define PR_EG_NRT 1
#endif
// Tensor memory: two 128-column buffers per row tile, buffer b of row tile rt at (2 rt + b) * 128.
// Before the first use of buffer 1 its columns hold the Gram part: the gated row as A operand
// (32 columns at +0) and u = x~ Gs (64 columns at +64), read into the accumulators' initial value.
__device__ __forceinline__ constexpr uint32_t col_d(int rt, int b) { return (uint32_t)((2 * rt + b) * 128); }
constexpr uint32_t OFF_XA = 0, OFF_U = 64;

}  // namespace eg

struct ExpandGradParams {
  int h, hx;             // gate/state heads, operand heads (hx = h * ratio)
  int n_chunks, c;
  int tiles_per_chunk;
  int chunk_lo, chunk_hi;  // chunks in [lo, hi] have a state term; the others get zeros
  int query_side;
  float scale;           // s (query side only)
  float gram_mult;
  const float* a;        // [b, t, h] or null
  const float* A;        // [b, n, h] or null
  const float* row_g;    // [b, t, hx] (query side: dl) or null (= 1)
  float* dX;             // [b, t, hx, 64] fp32
  float* gdot;           // [b, t, hx]
  int* status;
};

template <typename T, int NRT>
__global__ void __launch_bounds__(eg::Cfg<NRT>::THREADS, NRT == 1 ? 2 : 1)
expand_grad_kernel(const ExpandGradParams p, const __grid_constant__ CUtensorMap tm_w,
                   const __grid_constant__ CUtensorMap tm_x, const __grid_constant__ CUtensorMap tm_s,
                   const __grid_constant__ CUtensorMap tm_ghi, const __grid_constant__ CUtensorMap tm_glo) {
  using namespace eg;
  constexpr int THREADS = Cfg<NRT>::THREADS, ROWS = Cfg<NRT>::ROWS, NSS = Cfg<NRT>::NSS;
  constexpr uint32_t TMEM_COLS = Cfg<NRT>::TMEM_COLS;
  constexpr int W_TMA = 4 * NRT;  // the TMA warp; issuing warps follow
  extern __shared__ uint8_t smem_raw[];
  __shared__ uint64_t w_full, g_full, xa_full[2], u_full[2], s_full[NSS], s_empty[NSS], d_full[2][2], d_empty[2][2];
  __shared__ uint32_t tmem_base_s;
  __shared__ int abort_flag;

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int tile_i = blockIdx.x % p.tiles_per_chunk;
  const int chunk = blockIdx.x / p.tiles_per_chunk;
  const int head = blockIdx.y, batch = blockIdx.z;
  const int gh = head / (p.hx / p.h);
  const int row0 = tile_i * ROWS;
  const size_t tok0 = (size_t)batch * p.n_chunks * p.c + (size_t)chunk * p.c;

  if (chunk < p.chunk_lo || chunk > p.chunk_hi) {
    // no state term for this chunk: zero gradient
    if (tid < ROWS) {
      const int row = row0 + tid;
      if (row < p.c) {
        float4* dst = reinterpret_cast<float4*>(p.dX + ((tok0 + row) * p.hx + head) * HD);
#pragma unroll
        for (int j = 0; j < 16; ++j) dst[j] = make_float4(0.f, 0.f, 0.f, 0.f);
        p.gdot[(tok0 + row) * p.hx + head] = 0.f;
      }
    }
    return;
  }

  const uint32_t sbase = (smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t* sm = smem_raw + (sbase - smem_u32(smem_raw));
  uint8_t* smW = sm;                            // NRT x TILE_BYTES (one per row tile)
  uint8_t* smX = smW + NRT * TILE_BYTES;        // NRT x TILE_BYTES
  uint8_t* smS = smX + NRT * TILE_BYTES;        // NSS x TILE_BYTES (ring of state tiles)
  // Gram operand (hi, lo): its own 16 KB, or the ring's last slot until the Gram products are done
  uint8_t* smG = Cfg<NRT>::G_IN_RING ? smS + (NSS - 1) * TILE_BYTES : smS + NSS * TILE_BYTES;
  // NRT x [64][128] fp32: dx~ terms indexed at run time
  float* smR = reinterpret_cast<float*>(smS + NSS * TILE_BYTES + (Cfg<NRT>::G_IN_RING ? 0 : 2 * G_BYTES));

  if (tid == 0) {
    abort_flag = 0;
    mbar_init(&w_full, 1);
    mbar_init(&g_full, 1);
    for (int s = 0; s < 2; ++s) {
      mbar_init(&xa_full[s], 4);
      mbar_init(&u_full[s], 1);
      for (int b = 0; b < 2; ++b) {
        mbar_init(&d_full[s][b], 1);
        mbar_init(&d_empty[s][b], 4);
      }
    }
    for (int s = 0; s < NSS; ++s) {
      mbar_init(&s_full[s], 1);
      mbar_init(&s_empty[s], NRT);  // one issuing thread per row tile releases a state tile
    }
    fence_mbar_init();
  }
  if (warp == 0) {
    tmem_alloc(&tmem_base_s, TMEM_COLS);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = tmem_base_s;
  const int ch = (batch * p.n_chunks + chunk) * p.h + gh;

  if (warp == W_TMA) {
    if (lane == 0) {
      mbar_expect_tx(&w_full, 2 * NRT * TILE_BYTES);
      for (int rt = 0; rt < NRT; ++rt) {
        tma_load_4d(smW + rt * TILE_BYTES, &tm_w, &w_full, 0, head, chunk * p.c + row0 + rt * 128, batch);
        tma_load_4d(smX + rt * TILE_BYTES, &tm_x, &w_full, 0, head, chunk * p.c + row0 + rt * 128, batch);
      }
      mbar_expect_tx(&g_full, 2 * G_BYTES);
      tma_load_2d(smG, &tm_ghi, &g_full, 0, ch * HD);
      tma_load_2d(smG + G_BYTES, &tm_glo, &g_full, 0, ch * HD);
      for (int nt = 0; nt < NT; ++nt) {
        const int s = nt % NSS, ph = (nt / NSS) & 1;
        if (!mbar_wait(&s_empty[s], ph ^ 1, &abort_flag)) break;
        // the slot lent to the Gram operand is free once the Gram products have completed
        if (Cfg<NRT>::G_IN_RING && nt == NSS - 1 && !mbar_wait(&u_full[0], 0, &abort_flag)) break;
        mbar_expect_tx(&s_full[s], TILE_BYTES);
        tma_load_2d(smS + s * TILE_BYTES, &tm_s, &s_full[s], 0, ch * D2 + nt * 128);
      }
    }
  } else if (warp > W_TMA) {
    // Two issuing threads per row tile, one per tensor-memory buffer (even / odd state tiles): a thread
    // needs ~108 clocks per tcgen05.mma it issues and more per commit, whatever the shape (measured), and
    // traced timelines showed one thread per row tile setting the kernel's pace at ~1300 clocks per tile
    // against ~900 for the drain.
    if (lane == 0) {
      const int rt = (warp - (W_TMA + 1)) >> 1, par = (warp - (W_TMA + 1)) & 1;
      bool ok = mbar_wait(&w_full, 0, &abort_flag);
      const uint32_t w_addr = smem_u32(smW) + rt * TILE_BYTES;
      const uint32_t idesc = umma_idesc(128, 128, Pack2<T>::is_bf16, false, false);
      for (int nt = par; nt < NT && ok; nt += 2) {
        const int s = nt % NSS, ph = (nt / NSS) & 1;
        const int b = par;
        // buffer 0 has been drained nt/2 times before tile nt; buffer 1 once more (the Gram part)
        ok = mbar_wait(&d_empty[rt][b], ((nt >> 1) & 1) ^ (b ^ 1), &abort_flag) &&
             mbar_wait(&s_full[s], ph, &abort_flag);
        if (!ok) break;
        tc_fence_after();
        const uint32_t s_addr = smem_u32(smS + s * TILE_BYTES);
#pragma unroll
        for (int ks = 0; ks < 4; ++ks)
          umma_ss(tmem + col_d(rt, b), umma_desc_sw128(w_addr + ks * 32, 16, 1024),
                  umma_desc_sw128(s_addr + ks * 32, 16, 1024), idesc, ks > 0 ? 1u : 0u);
        umma_commit(&d_full[rt][b]);
        umma_commit(&s_empty[s]);
        if (nt == 0) {
          // Gram part: u = x~ (Gs_hi + Gs_lo), once per row tile, in the columns of buffer 1 (whose own
          // issuing thread waits until the rows have taken u out)
          ok = mbar_wait(&g_full, 0, &abort_flag) && mbar_wait(&xa_full[rt], 0, &abort_flag);
          if (!ok) break;
          tc_fence_after();
          const uint32_t idesc_g = umma_idesc(128, HD, Pack2<T>::is_bf16, false, false);
          const uint32_t g_addr = smem_u32(smG);
#pragma unroll
          for (int half = 0; half < 2; ++half)
#pragma unroll
            for (int ks = 0; ks < 4; ++ks)
              umma_ts(tmem + col_d(rt, 1) + OFF_U, tmem + col_d(rt, 1) + OFF_XA + ks * 8,
                      umma_desc_sw128(g_addr + half * G_BYTES + ks * 32, 16, 1024), idesc_g,
                      (half > 0 || ks > 0) ? 1u : 0u);
          umma_commit(&u_full[rt]);
        }
      }
    }
  } else {
    // ------------------------------------------------------------ drain warps
    const int rt = warp >> 2;                  // row tile owned by this warp group
    const int r = (warp & 3) * 32 + lane;      // token row inside the tile = TMEM lane
    const int row = row0 + rt * 128 + r;
    const bool row_valid = row < p.c;
    const uint32_t lane_addr = (uint32_t)((warp & 3) * 32) << 16;

    float f = p.query_side ? p.scale : 1.f;
    if (p.a != nullptr) {
      const float a_i = row_valid ? p.a[(tok0 + row) * p.h + gh] : 0.f;
      f *= p.query_side ? __expf(0.5f * a_i) : __expf(0.5f * (p.A[ch] - a_i));
    }
    bool ok = mbar_wait(&w_full, 0, &abort_flag);
    {
      uint32_t xp[32];
      uint8_t* xs = smX + rt * TILE_BYTES;
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        const uint4 v = *reinterpret_cast<const uint4*>(xs + swz128(r, j));
        const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
        for (int k = 0; k < 4; ++k) {
          const float2 raw = Pack2<T>::to_f32(w[k]);
          xp[4 * j + k] = Pack2<T>::from_f32(raw.x * f, raw.y * f);
        }
      }
      // the gated row replaces the raw one in this thread's slot of the tile (fetched by a
      // run-time index in the drain)
#pragma unroll
      for (int j = 0; j < 8; ++j)
        *reinterpret_cast<uint4*>(smX + rt * TILE_BYTES + swz128(r, j)) =
            make_uint4(xp[4 * j], xp[4 * j + 1], xp[4 * j + 2], xp[4 * j + 3]);
      if (ok) {
        tmem_st32(tmem + lane_addr + col_d(rt, 1) + OFF_XA, xp);
        tmem_wait_st();
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(&xa_full[rt]);
      }
    }
    // Gram part first: dx~ starts at g_i * mult * (Gs x~)_i, which also frees buffer 1
    {
      float g = p.gram_mult;
      if (p.row_g != nullptr) g *= row_valid ? p.row_g[(tok0 + row) * p.hx + head] : 0.f;
      if (ok) ok = mbar_wait(&u_full[rt], 0, &abort_flag);
      tc_fence_after();
      uint32_t u[64];
      if (ok) {
        tmem_ld32(tmem + lane_addr + col_d(rt, 1) + OFF_U, u);
        tmem_ld32(tmem + lane_addr + col_d(rt, 1) + OFF_U + 32, u + 32);
        tmem_wait_ld();
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(&d_empty[rt][1]);
      }
      // dx~ lives in this thread's private column of shared memory (64 floats, stride 128): the
      // first-factor terms are added at a run-time index, and the second-factor terms of a
      // 16-block are kept in registers only while that block is being drained.  Keeping all 64
      // accumulators and the row itself in registers left the compiler no room to overlap the
      // FMAs of neighbouring entries.
      float* sdx0 = smR + rt * 64 * 128 + r;
#pragma unroll
      for (int e = 0; e < HD; ++e) sdx0[e * 128] = ok ? g * __uint_as_float(u[e]) : 0.f;
    }
    float* sdx = smR + rt * 64 * 128 + r;
    const uint8_t* xrow = smX + rt * TILE_BYTES;  // holds the gated row again (written above)

    int nt = 0;
    static_for<0, HD / 16>([&](auto yc) {
      constexpr int Y = decltype(yc)::value;
      // second factors x~[16Y .. 16Y+15] of this block and their gradient accumulators, as pairs:
      // the drain runs on packed fp32 FMAs (two entries per instruction)
      float2 x[8], dx[8];
#pragma unroll
      for (int j = 0; j < 2; ++j) {
        const uint4 v4 = *reinterpret_cast<const uint4*>(xrow + swz128(r, 2 * Y + j));
        const uint32_t w[4] = {v4.x, v4.y, v4.z, v4.w};
#pragma unroll
        for (int k = 0; k < 4; ++k) {
          x[4 * j + k] = Pack2<T>::to_f32(w[k]);
          dx[4 * j + k] = make_float2(0.f, 0.f);
        }
      }
#pragma unroll 1
      for (int tt = 0; tt < 2 * (Y + 1); ++tt, ++nt) {
        const int b = nt & 1;
        if (ok) ok = mbar_wait(&d_full[rt][b], (nt >> 1) & 1, &abort_flag);
        tc_fence_after();
        if (!ok) continue;
        const uint32_t cd = tmem + lane_addr + col_d(rt, b);
        // the tile's eight first factors x~[8 tt .. 8 tt + 7] in one 16-byte load, and their gradient
        // terms collected in registers: the shared-memory column is touched once per tile, after the
        // loop, so no load of the loop has to wait behind a store to the same memory space
        float xa8[8], rsum[8];
        {
          const uint4 w4 = *reinterpret_cast<const uint4*>(xrow + swz128(r, tt));
          const uint32_t w[4] = {w4.x, w4.y, w4.z, w4.w};
#pragma unroll
          for (int k = 0; k < 4; ++k) {
            const float2 f2 = Pack2<T>::to_f32(w[k]);
            xa8[2 * k] = f2.x;
            xa8[2 * k + 1] = f2.y;
          }
        }
        // two register buffers: the load of the next 32 columns is in flight while these are used
        uint32_t v[2][32];
        tmem_ld32(cd, v[0]);
#pragma unroll
        for (int q = 0; q < 4; ++q) {
          tmem_wait_ld();
          if (q < 3) {
            tmem_ld32(cd + (q + 1) * 32, v[(q + 1) & 1]);
          } else {
            // all of this thread's reads of the buffer are done
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(&d_empty[rt][b]);
          }
#pragma unroll
          for (int aa = 0; aa < 2; ++aa) {
            const float xs = xa8[2 * q + aa];  // first factor a = 8 tt + 2 q + aa
            const float2 xa = make_float2(xs, xs);
            float2 ra0 = make_float2(0.f, 0.f), ra1 = ra0;
#pragma unroll
            for (int i = 0; i < 8; ++i) {
              const float2 val = make_float2(__uint_as_float(v[q & 1][16 * aa + 2 * i]),
                                             __uint_as_float(v[q & 1][16 * aa + 2 * i + 1]));
              dx[i] = __ffma2_rn(val, xa, dx[i]);
              if (i & 1)
                ra1 = __ffma2_rn(val, x[i], ra1);
              else
                ra0 = __ffma2_rn(val, x[i], ra0);
            }
            rsum[2 * q + aa] = (ra0.x + ra0.y) + (ra1.x + ra1.y);
          }
        }
#pragma unroll
        for (int j = 0; j < 8; ++j) sdx[(8 * tt + j) * 128] += rsum[j];
      }
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        sdx[(16 * Y + 2 * i) * 128] += dx[i].x;
        sdx[(16 * Y + 2 * i + 1) * 128] += dx[i].y;
      }
    });

    if (ok && row_valid) {
      float dot = 0.f;
      float4* dst = reinterpret_cast<float4*>(p.dX + ((tok0 + row) * p.hx + head) * HD);
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        const uint4 v4 = *reinterpret_cast<const uint4*>(xrow + swz128(r, j));
        const uint32_t w[4] = {v4.x, v4.y, v4.z, v4.w};
        float d8[8];
#pragma unroll
        for (int k = 0; k < 4; ++k) {
          const float2 f2 = Pack2<T>::to_f32(w[k]);
          d8[2 * k] = sdx[(8 * j + 2 * k) * 128];
          d8[2 * k + 1] = sdx[(8 * j + 2 * k + 1) * 128];
          dot = fmaf(f2.x, d8[2 * k], dot);
          dot = fmaf(f2.y, d8[2 * k + 1], dot);
        }
        // one 32-byte store: a full sector per thread and instruction
        asm volatile("st.global.v8.f32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8};" ::"l"(dst + 2 * j), "f"(d8[0] * f),
                     "f"(d8[1] * f), "f"(d8[2] * f), "f"(d8[3] * f), "f"(d8[4] * f), "f"(d8[5] * f), "f"(d8[6] * f),
                     "f"(d8[7] * f)
                     : "memory");
      }
      p.gdot[(tok0 + row) * p.hx + head] = 0.5f * dot;
    }
  }
  tc_fence_before();
  __syncthreads();
  if (tid == 0 && abort_flag) *p.status = ST_TIMEOUT;
  if (warp == 0) tmem_dealloc(tmem, TMEM_COLS);
}

}  // namespace pr

extern "C" int pr_expand_grad(int dtype, int b, int t, int h, int hx, int d, int c, const void* W, const void* X,
                              const void* State, const void* g_hi, const void* g_lo, const float* a, const float* A,
                              const float* row_g, int query_side, float scale, float gram_mult, int chunk_lo,
                              int chunk_hi, float* dX, float* gdot, int device, void* stream) {
  using namespace pr;
  using namespace pr::eg;
  PR_REQUIRE(d == HD, PR_ERR_BAD_ARG, "head dim %d: this build handles d = 64", d);
  PR_REQUIRE(b > 0 && t > 0 && h > 0 && hx > 0 && hx % h == 0 && c > 0 && t % c == 0, PR_ERR_BAD_ARG,
             "bad sizes b=%d t=%d h=%d hx=%d c=%d", b, t, h, hx, c);
  PR_REQUIRE(dtype == PR_BF16 || dtype == PR_FP16, PR_ERR_BAD_ARG, "dtype %d", dtype);
  PR_REQUIRE(W && X && State && g_hi && g_lo && dX && gdot, PR_ERR_BAD_ARG, "null pointer");
  PR_REQUIRE(aligned16(W) && aligned16(X) && aligned16(State) && aligned16(g_hi) && aligned16(g_lo) && aligned16(dX),
             PR_ERR_BAD_ARG, "misaligned pointer");
  PR_REQUIRE((a == nullptr) == (A == nullptr), PR_ERR_BAD_ARG, "a and A must be given together");
  PR_REQUIRE(hx <= 65535 && b <= 65535, PR_ERR_BAD_ARG, "hx and b must be <= 65535");
  PR_CUDA(cudaSetDevice(device));
  const int n = t / c;
  ExpandGradParams p;
  p.h = h;
  p.hx = hx;
  p.n_chunks = n;
  p.c = c;
  using C = Cfg<PR_EG_NRT>;
  p.tiles_per_chunk = (c + C::ROWS - 1) / C::ROWS;
  p.chunk_lo = chunk_lo;
  p.chunk_hi = chunk_hi;
  p.query_side = query_side;
  p.scale = scale;
  p.gram_mult = gram_mult;
  p.a = a;
  p.A = A;
  p.row_g = row_g;
  p.dX = dX;
  p.gdot = gdot;
  int rc = status_word(device, &p.status, nullptr);
  if (rc) return rc;
  CUtensorMap tm_w, tm_x, tm_s, tm_ghi, tm_glo;
  {
    uint64_t dims[4] = {(uint64_t)d, (uint64_t)hx, (uint64_t)t, (uint64_t)b};
    uint64_t str[4] = {0, (uint64_t)d * 2, (uint64_t)hx * d * 2, (uint64_t)t * hx * d * 2};
    uint32_t box[4] = {64, 1, 128, 1};
    if ((rc = make_tmap(&tm_w, W, 2, 4, dims, str, box, true))) return rc;
    if ((rc = make_tmap(&tm_x, X, 2, 4, dims, str, box, true))) return rc;
  }
  {
    uint64_t ds[2] = {64, (uint64_t)b * n * h * D2};
    uint64_t dg[2] = {64, (uint64_t)b * n * h * d};
    uint64_t st[2] = {0, 128};
    uint32_t box_s[2] = {64, 128}, box_g[2] = {64, 64};
    if ((rc = make_tmap(&tm_s, State, 2, 2, ds, st, box_s, true))) return rc;
    if ((rc = make_tmap(&tm_ghi, g_hi, 2, 2, dg, st, box_g, true))) return rc;
    if ((rc = make_tmap(&tm_glo, g_lo, 2, 2, dg, st, box_g, true))) return rc;
  }
  const size_t smem = C::SMEM;
  dim3 grid(p.tiles_per_chunk * n, hx, b);
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  if (dtype == PR_BF16) {
    PR_SMEM_ATTR((expand_grad_kernel<__nv_bfloat16, PR_EG_NRT>), smem, device, true);
    expand_grad_kernel<__nv_bfloat16, PR_EG_NRT><<<grid, C::THREADS, smem, s>>>(p, tm_w, tm_x, tm_s, tm_ghi, tm_glo);
  } else {
    PR_SMEM_ATTR((expand_grad_kernel<__half, PR_EG_NRT>), smem, device, true);
    expand_grad_kernel<__half, PR_EG_NRT><<<grid, C::THREADS, smem, s>>>(p, tm_w, tm_x, tm_s, tm_ghi, tm_glo);
  }
  PR_CUDA(cudaGetLastError());
  return PR_OK;
}
