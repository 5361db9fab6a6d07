// Backward of the intra-chunk attention with respect to the queries, merged with the
// state-path query gradient (the reference's attn_bwd_dq, retention/_attention/triton.py:496-603,
// for deg = 2 without the division by the score).
//
// One CTA owns 128 query rows of one (batch, chunk, query head); thread = row.  For every
// tile of 64 keys up to the diagonal (tiles double-buffered in shared memory; 256 tensor
// memory columns, so two CTAs share an SM and hide each other's waits):
//     S  = Q K_J^T,  dP = dO V_J^T                      (tensor cores, fp32 in tensor memory)
//     p  = (s S)^2 e^{a_i-a_j},  dp = dP / l_i + dl_i,  e = p dp,  dS = 2 s^2 S e^{a_i-a_j} dp
//     dQ += dS K_J                                      (A = dS from tensor memory)
//     da_i += sum_j e_ij                                (gate gradient, query side)
// with dl = -<O, dO> / l from the backward prologue.  dO enters the tensor cores unscaled and
// 1/l_i is applied in fp32, so the cancellation between dP / l and dl (exact for a row with a
// single key) is not spoiled by a 16-bit rounding of dO / l.  The epilogue adds the
// state-path gradient (fp32, from the expansion-gradient kernel) and writes dQ.
#include "host.cuh"
#include "sm100.cuh"

namespace pr {

namespace dq {
constexpr int HD = 64;
constexpr int THREADS = 224;             // warps 0-3 rows, 4 TMA, 5 and 6 issue tcgen05.mma
constexpr int TILE_BYTES = 128 * 128;   // 128 query rows x 64 features
constexpr int TW = 64;                  // keys per step
constexpr int KV_BYTES = TW * 128;      // one key or value tile
constexpr int NKV = 4;                  // key/value tiles in flight
constexpr uint32_t TMEM_COLS = 256;     // two CTAs per SM
constexpr uint32_t COL_S = 0, COL_DP = 128, COL_ACC = 192;  // S double-buffered (2 x 64); dS overwrites its S
}  // namespace dq

struct ChunkDqParams {
  int hq, h, n_chunks, c, tiles_per_chunk;
  float scale;
  const float* a;         // [b, t, h] or null
  const float* dl;        // [b, t, hq]
  const float* l;         // [b, t, hq] row sums saved by the forward
  const float* dq_state;  // [b, t, hq, 64] fp32 or null
  void* dQ;               // [b, t, hq, 64]
  float* da_q;            // [b, t, hq]
  int* status;
};

// One 32-column half of a step for one row: dS = 2 s^2 S g dp into `pk`, row sum of dS * S into da2.
// SEP: the gate factor is c_i * fk[col] (c_i carries 2 s^2); otherwise 2 s^2 e^{a_i - ak[col]} per pair.
// MASK: columns beyond `lim` (the row's own position, relative to the step) are dropped.
template <typename T, int DEG, bool SEP, bool MASK>
__device__ __forceinline__ void dq_half(const uint32_t (&sv)[32], const uint32_t (&pv)[32], const float* __restrict__ fk,
                                        float c_i, float a_i, float inv_l, float dl_i, int lim, uint32_t (&pk)[16],
                                        float& da2) {
  // two columns per instruction: packed fp32 multiplies and FMAs
  const float4* f4 = reinterpret_cast<const float4*>(fk);
  const float2 c2 = make_float2(c_i, c_i), il2 = make_float2(inv_l, inv_l), dl2 = make_float2(dl_i, dl_i);
  float2 acc = make_float2(0.f, 0.f);
#pragma unroll
  for (int j = 0; j < 32; j += 4) {
    const float4 f = f4[j >> 2];
    const float2 fv[2] = {make_float2(f.x, f.y), make_float2(f.z, f.w)};
#pragma unroll
    for (int u = 0; u < 2; ++u) {
      const int col = j + 2 * u;
      const float2 s = make_float2(__uint_as_float(sv[col]), __uint_as_float(sv[col + 1]));
      const float2 p = make_float2(__uint_as_float(pv[col]), __uint_as_float(pv[col + 1]));
      const float2 dp = __ffma2_rn(p, il2, dl2);
      float2 g;
      if (SEP) {
        g = __fmul2_rn(c2, fv[u]);
      } else {
        g = make_float2(c_i * __expf(a_i - fv[u].x), c_i * __expf(a_i - fv[u].y));
      }
      if (MASK) {
        g.x = (col <= lim) ? g.x : 0.f;
        g.y = (col + 1 <= lim) ? g.y : 0.f;
      }
      const float2 sp = DEG == 4 ? __fmul2_rn(s, __fmul2_rn(s, s)) : s;  // S^(deg-1)
      const float2 ds = __fmul2_rn(__fmul2_rn(sp, g), dp);  // deg s^deg S^(deg-1) e^{a_i-a_j} dp
      acc = __ffma2_rn(ds, s, acc);
      pk[col >> 1] = Pack2<T>::from_f32(ds.x, ds.y);
    }
  }
  da2 += acc.x + acc.y;
}

template <typename T, int DEG>
__global__ void __launch_bounds__(dq::THREADS, 2)
chunk_dq_kernel(const ChunkDqParams p, const __grid_constant__ CUtensorMap tm_q,
                const __grid_constant__ CUtensorMap tm_dy, const __grid_constant__ CUtensorMap tm_k,
                const __grid_constant__ CUtensorMap tm_v, const __grid_constant__ CUtensorMap tm_st) {
  using namespace dq;
  extern __shared__ uint8_t smem_raw[];
  __shared__ uint64_t q_full, kv_full[NKV], kv_empty[NKV], sp_full, ds_full, acc_done, qdy_free, st_full, dq_done[2];
  __shared__ uint32_t tmem_base_s;
  __shared__ int abort_flag;
  __shared__ __align__(16) float sm_ak[2][TW];  // gate sums a_j of the step's keys
  __shared__ __align__(16) float sm_fk[2][TW];  // e^{r - a_j}, r = gate sum at the step's last key
  __shared__ float sm_r[2];
  __shared__ int sm_wide[2][2];                 // a loader warp saw r - a_j > 80 (overflow guard)

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const uint32_t sbase = (smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t* sm = smem_raw + (sbase - smem_u32(smem_raw));
  uint8_t* smQ = sm;
  uint8_t* smDY = smQ + TILE_BYTES;
  uint8_t* smK = smDY + TILE_BYTES;      // NKV stages x KV_BYTES
  uint8_t* smV = smK + NKV * KV_BYTES;   // NKV stages x KV_BYTES

  const int tile_i = blockIdx.x % p.tiles_per_chunk;
  const int chunk = blockIdx.x / p.tiles_per_chunk;
  const int qhead = blockIdx.y, batch = blockIdx.z;
  const int kvhead = qhead / (p.hq / p.h);
  const int row0 = tile_i * 128;
  const int nJ = min(p.c - 1, row0 + 127) / TW + 1;
  const int tok_chunk = chunk * p.c;
  const bool has_st = p.dq_state != nullptr;

  if (tid == 0) {
    abort_flag = 0;
    mbar_init(&q_full, 1);
    for (int s = 0; s < NKV; ++s) {
      mbar_init(&kv_full[s], 1);
      mbar_init(&kv_empty[s], 1);
    }
    mbar_init(&sp_full, 1);
    mbar_init(&ds_full, 4);
    mbar_init(&acc_done, 1);
    mbar_init(&qdy_free, 1);
    mbar_init(&st_full, 1);
    mbar_init(&dq_done[0], 1);
    mbar_init(&dq_done[1], 1);
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

  if (warp == 4) {
    if (lane == 0) {
      mbar_expect_tx(&q_full, 2 * TILE_BYTES);
      tma_load_4d(smQ, &tm_q, &q_full, 0, qhead, tok_chunk + row0, batch);
      tma_load_4d(smDY, &tm_dy, &q_full, 0, qhead, tok_chunk + row0, batch);
      bool ok = true;
      for (int J = 0; J < nJ; ++J) {
        const int s = J % NKV, ph = (J / NKV) & 1;
        if (!(ok = mbar_wait(&kv_empty[s], ph ^ 1, &abort_flag))) break;
        mbar_expect_tx(&kv_full[s], 2 * KV_BYTES);
        tma_load_4d(smK + s * KV_BYTES, &tm_k, &kv_full[s], 0, kvhead, tok_chunk + J * TW, batch);
        tma_load_4d(smV + s * KV_BYTES, &tm_v, &kv_full[s], 0, kvhead, tok_chunk + J * TW, batch);
      }
      // The query and dO tiles are dead once the last S and dP are computed: the fp32
      // state-path gradient of these rows (two 32-column halves) takes their place.
      if (ok && has_st && mbar_wait(&qdy_free, 0, &abort_flag)) {
        mbar_expect_tx(&st_full, 2 * TILE_BYTES);
        tma_load_4d(smQ, &tm_st, &st_full, 0, qhead, tok_chunk + row0, batch);
        tma_load_4d(smDY, &tm_st, &st_full, 32, qhead, tok_chunk + row0, batch);
      }
    }
  } else if (warp == 5) {
    // Issuing thread A: S and dP.  One thread issues a product only every ~108 clocks whatever its
    // shape (measured), so the three products of a step are shared between two threads: this one runs
    // ahead with S(J+1) and dP(J+1), thread B follows with dQ(J).
    if (lane == 0) {
      bool ok = mbar_wait(&q_full, 0, &abort_flag);
      const uint32_t idesc_s = umma_idesc(128, TW, Pack2<T>::is_bf16, false, false);
      const uint32_t q_addr = smem_u32(smQ), dy_addr = smem_u32(smDY);
      auto issue_s = [&](int J) {
        const uint32_t k_addr = smem_u32(smK + (J % NKV) * KV_BYTES);
#pragma unroll
        for (int ks = 0; ks < 4; ++ks)
          umma_ss(tmem + COL_S + (J & 1) * TW, umma_desc_sw128(q_addr + ks * 32, 16, 1024),
                  umma_desc_sw128(k_addr + ks * 32, 16, 1024), idesc_s, ks > 0 ? 1u : 0u);
      };
      auto issue_dp = [&](int J) {
        const uint32_t v_addr = smem_u32(smV + (J % NKV) * KV_BYTES);
#pragma unroll
        for (int ks = 0; ks < 4; ++ks)
          umma_ss(tmem + COL_DP, umma_desc_sw128(dy_addr + ks * 32, 16, 1024),
                  umma_desc_sw128(v_addr + ks * 32, 16, 1024), idesc_s, ks > 0 ? 1u : 0u);
        umma_commit(&sp_full);
        if (J == nJ - 1) umma_commit(&qdy_free);
      };
      if (ok) ok = mbar_wait(&kv_full[0], 0, &abort_flag);
      if (ok) {
        tc_fence_after();
        issue_s(0);
        issue_dp(0);
      }
      for (int J = 0; J + 1 < nJ && ok; ++J) {
        ok = mbar_wait(&kv_full[(J + 1) % NKV], ((J + 1) / NKV) & 1, &abort_flag);
        // S(J+1) overwrites the buffer whose dS fed dQ(J-1): that product must have completed
        if (ok && J >= 1) ok = mbar_wait(&dq_done[(J + 1) & 1], ((J - 1) >> 1) & 1, &abort_flag);
        if (!ok) break;
        tc_fence_after();
        issue_s(J + 1);
        // dP(J+1) overwrites dP(J), which the rows have read once dS(J) is in tensor memory
        ok = mbar_wait(&ds_full, J & 1, &abort_flag);
        if (!ok) break;
        tc_fence_after();
        issue_dp(J + 1);
      }
    }
  } else if (warp == 6) {
    // Issuing thread B: dQ += dS(J) K_J, releases the key/value stage
    if (lane == 0) {
      bool ok = true;
      const uint32_t idesc_q = umma_idesc(128, HD, Pack2<T>::is_bf16, false, true);
      for (int J = 0; J < nJ && ok; ++J) {
        ok = mbar_wait(&ds_full, J & 1, &abort_flag);
        if (!ok) break;
        tc_fence_after();
        const uint32_t k_addr = smem_u32(smK + (J % NKV) * KV_BYTES);
#pragma unroll
        for (int ks = 0; ks < TW / 16; ++ks)
          umma_ts(tmem + COL_ACC, tmem + COL_S + (J & 1) * TW + ks * 8,
                  umma_desc_sw128(k_addr + ks * 2048, 8192, 1024), idesc_q, (J > 0 || ks > 0) ? 1u : 0u);
        umma_commit(&kv_empty[J % NKV]);
        umma_commit(&dq_done[J & 1]);
      }
      if (ok) umma_commit(&acc_done);
    }
  } else {
    const int row = row0 + tid;
    const bool row_valid = row < p.c;
    const uint32_t lane_addr = (uint32_t)(warp * 32) << 16;
    const bool gated = p.a != nullptr;
    const size_t tok = (size_t)batch * p.n_chunks * p.c + tok_chunk + row;
    const float* a_chunk = gated ? p.a + ((size_t)batch * p.n_chunks * p.c + tok_chunk) * p.h + kvhead : nullptr;
    const float a_i = (gated && row_valid) ? a_chunk[(size_t)row * p.h] : 0.f;
    const float dl_i = row_valid ? p.dl[tok * p.hq + qhead] : 0.f;
    const float inv_l = row_valid ? safe_recip(p.l[tok * p.hq + qhead]) : 0.f;
    const float s2x2 = DEG == 4 ? 4.f * (p.scale * p.scale) * (p.scale * p.scale) : 2.f * p.scale * p.scale;  // deg s^deg
    const int wrow0 = row0 + (warp << 5);  // first row of this warp
    float da2 = 0.f;                       // twice the row sum of p * dp
    bool ok = true;
    // gate sums of the next step's keys, loaded one step ahead by the first TW threads
    float av_n = 0.f, r_n = 0.f;
    auto load_gates = [&](int J) {
      if (tid < TW && gated) {
        const int kp = J * TW + tid;
        av_n = kp < p.c ? a_chunk[(size_t)kp * p.h] : 0.f;
        r_n = a_chunk[(size_t)min(J * TW + TW - 1, p.c - 1) * p.h];
      }
    };
    load_gates(0);
    for (int J = 0; J < nJ; ++J) {
      const int kp0 = J * TW;
      const int sb = J & 1;
      const uint32_t col_s = COL_S + sb * TW;
      if (tid < TW) {
        sm_ak[sb][tid] = av_n;
        sm_fk[sb][tid] = __expf(r_n - av_n);
        const bool wide = __any_sync(0xffffffffu, (r_n - av_n) > 80.f);
        if (lane == 0) sm_wide[sb][warp] = wide;
        if (tid == 0) sm_r[sb] = r_n;
      }
      asm volatile("bar.sync 1, 128;" ::: "memory");
      if (J + 1 < nJ) load_gates(J + 1);  // in flight while this step is computed
      ok = mbar_wait(&sp_full, J & 1, &abort_flag);
      if (!ok) break;
      tc_fence_after();
      // The gate factor separates, e^{a_i - a_j} = e^{a_i - r} * e^{r - a_j}: one exponential
      // per row and per key instead of one per pair.  Both exponents are <= 0 below the
      // diagonal for gates <= 0; if one exceeds 80 (growing gates) the warp takes the per-pair
      // form.  Steps wholly below the diagonal need no mask; a warp whose rows all precede the
      // step's keys writes zeros without reading the scores.
      const int lim = min(row, p.c - 1) - kp0;  // last column this row keeps
      if (kp0 > min(wrow0 + 31, p.c - 1)) {
        uint32_t z[16];
#pragma unroll
        for (int j = 0; j < 16; ++j) z[j] = 0u;
        tmem_st16(tmem + lane_addr + col_s, z);
        tmem_st16(tmem + lane_addr + col_s + 16, z);
      } else {
        const float r = sm_r[sb];
        const bool mask = (kp0 + TW - 1 > wrow0) || (kp0 + TW - 1 >= p.c);
        const bool sep = !(sm_wide[sb][0] | sm_wide[sb][1]) && !__any_sync(0xffffffffu, (a_i - r) > 80.f);
        const float c_i = sep ? s2x2 * __expf(a_i - r) : s2x2;
#pragma unroll 1
        for (int q4 = 0; q4 < TW / 32; ++q4) {
          uint32_t sv[32], pv[32], pk[16];
          tmem_ld32(tmem + lane_addr + col_s + q4 * 32, sv);
          tmem_ld32(tmem + lane_addr + COL_DP + q4 * 32, pv);
          tmem_wait_ld();
          const int lm = lim - q4 * 32;
          if (sep) {
            if (mask) dq_half<T, DEG, true, true>(sv, pv, sm_fk[sb] + q4 * 32, c_i, a_i, inv_l, dl_i, lm, pk, da2);
            else dq_half<T, DEG, true, false>(sv, pv, sm_fk[sb] + q4 * 32, c_i, a_i, inv_l, dl_i, lm, pk, da2);
          } else {
            dq_half<T, DEG, false, true>(sv, pv, sm_ak[sb] + q4 * 32, c_i, a_i, inv_l, dl_i, lm, pk, da2);
          }
          tmem_st16(tmem + lane_addr + col_s + q4 * 16, pk);
        }
      }
      tmem_wait_st();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&ds_full);
    }
    if (ok) ok = mbar_wait(&acc_done, 0, &abort_flag);
    if (ok && has_st) ok = mbar_wait(&st_full, 0, &abort_flag);
    tc_fence_after();
    if (ok) {
      uint32_t acc[64];
      tmem_ld32(tmem + lane_addr + COL_ACC, acc);
      tmem_ld32(tmem + lane_addr + COL_ACC + 32, acc + 32);
      tmem_wait_ld();
      if (row_valid) {
        uint4* dst = reinterpret_cast<uint4*>(static_cast<T*>(p.dQ) + (tok * p.hq + qhead) * HD);
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          float4 s0 = make_float4(0.f, 0.f, 0.f, 0.f), s1 = s0;
          if (has_st) {
            // columns 8j..8j+7: 16-byte chunks 2j, 2j+1 of the row in its 32-column half
            const uint8_t* half = (j < 4) ? smQ : smDY;
            s0 = *reinterpret_cast<const float4*>(half + swz128(tid, (2 * j) & 7));
            s1 = *reinterpret_cast<const float4*>(half + swz128(tid, (2 * j + 1) & 7));
          }
          uint4 v;
          v.x = Pack2<T>::from_f32(__uint_as_float(acc[8 * j + 0]) + s0.x, __uint_as_float(acc[8 * j + 1]) + s0.y);
          v.y = Pack2<T>::from_f32(__uint_as_float(acc[8 * j + 2]) + s0.z, __uint_as_float(acc[8 * j + 3]) + s0.w);
          v.z = Pack2<T>::from_f32(__uint_as_float(acc[8 * j + 4]) + s1.x, __uint_as_float(acc[8 * j + 5]) + s1.y);
          v.w = Pack2<T>::from_f32(__uint_as_float(acc[8 * j + 6]) + s1.z, __uint_as_float(acc[8 * j + 7]) + s1.w);
          dst[j] = v;
        }
        p.da_q[tok * p.hq + qhead] = (1.f / DEG) * da2;
      }
    }
  }
  tc_fence_before();
  __syncthreads();
  if (tid == 0 && abort_flag) *p.status = ST_TIMEOUT;
  if (warp == 0) tmem_dealloc(tmem, dq::TMEM_COLS);
}

}  // namespace pr

extern "C" int pr_chunk_dq(int dtype, int b, int t, int hq, int h, int d, int c, const void* Q, const void* dO,
                           const void* K, const void* V, const float* a, const float* dl, const float* l,
                           const float* dq_state, float scale, int deg, void* dQ, float* da_q, int device,
                           void* stream) {
  using namespace pr;
  using namespace pr::dq;
  PR_REQUIRE(deg == 2 || (deg == 4 && dq_state == nullptr), PR_ERR_BAD_ARG,
             "deg=%d: states exist for deg 2; deg 4 runs state-free (attention only)", deg);
  PR_REQUIRE(d == HD, PR_ERR_BAD_ARG, "head dim %d: this build handles d = 64", d);
  PR_REQUIRE(b > 0 && t > 0 && hq > 0 && h > 0 && hq % h == 0 && c > 0 && t % c == 0, PR_ERR_BAD_ARG,
             "bad sizes b=%d t=%d hq=%d h=%d c=%d", b, t, hq, h, c);
  PR_REQUIRE(dtype == PR_BF16 || dtype == PR_FP16, PR_ERR_BAD_ARG, "dtype %d", dtype);
  PR_REQUIRE(Q && dO && K && V && dl && l && dQ && da_q, PR_ERR_BAD_ARG, "null pointer");
  PR_REQUIRE(aligned16(Q) && aligned16(dO) && aligned16(K) && aligned16(V) && aligned16(dQ) && aligned16(dq_state),
             PR_ERR_BAD_ARG, "misaligned pointer");
  PR_REQUIRE(hq <= 65535 && b <= 65535, PR_ERR_BAD_ARG, "hq and b must be <= 65535");
  PR_CUDA(cudaSetDevice(device));
  ChunkDqParams p;
  p.hq = hq;
  p.h = h;
  p.n_chunks = t / c;
  p.c = c;
  p.tiles_per_chunk = (c + 127) / 128;
  p.scale = scale;
  p.a = a;
  p.dl = dl;
  p.l = l;
  p.dq_state = dq_state;
  p.dQ = dQ;
  p.da_q = da_q;
  int rc = status_word(device, &p.status, nullptr);
  if (rc) return rc;
  CUtensorMap tm_q, tm_dy, tm_k, tm_v, tm_st;
  uint64_t dq_[4] = {(uint64_t)d, (uint64_t)hq, (uint64_t)t, (uint64_t)b};
  uint64_t sq[4] = {0, (uint64_t)d * 2, (uint64_t)hq * d * 2, (uint64_t)t * hq * d * 2};
  uint64_t dk[4] = {(uint64_t)d, (uint64_t)h, (uint64_t)t, (uint64_t)b};
  uint64_t sk[4] = {0, (uint64_t)d * 2, (uint64_t)h * d * 2, (uint64_t)t * h * d * 2};
  uint32_t box[4] = {64, 1, 128, 1};
  if ((rc = make_tmap(&tm_q, Q, 2, 4, dq_, sq, box, true))) return rc;
  if ((rc = make_tmap(&tm_dy, dO, 2, 4, dq_, sq, box, true))) return rc;
  uint32_t box_kv[4] = {64, 1, (uint32_t)TW, 1};
  if ((rc = make_tmap(&tm_k, K, 2, 4, dk, sk, box_kv, true))) return rc;
  if ((rc = make_tmap(&tm_v, V, 2, 4, dk, sk, box_kv, true))) return rc;
  tm_st = tm_q;  // unused without a state-path gradient
  if (dq_state) {
    uint64_t ss[4] = {0, (uint64_t)d * 4, (uint64_t)hq * d * 4, (uint64_t)t * hq * d * 4};
    uint32_t box_st[4] = {32, 1, 128, 1};
    if ((rc = make_tmap(&tm_st, dq_state, 4, 4, dq_, ss, box_st, true))) return rc;
  }
  const size_t smem = 1024 + 2 * TILE_BYTES + 2 * NKV * KV_BYTES;
  dim3 grid(p.tiles_per_chunk * p.n_chunks, hq, b);
  cudaStream_t s = static_cast<cudaStream_t>(stream);
#define PR_LAUNCH_DQ(TT, DG)                                                                                      \
  do {                                                                                                           \
    PR_SMEM_ATTR((chunk_dq_kernel<TT, DG>), smem, device, true);                                                   \
    chunk_dq_kernel<TT, DG><<<grid, THREADS, smem, s>>>(p, tm_q, tm_dy, tm_k, tm_v, tm_st);                         \
  } while (0)
  if (dtype == PR_BF16) {
    if (deg == 4) PR_LAUNCH_DQ(__nv_bfloat16, 4); else PR_LAUNCH_DQ(__nv_bfloat16, 2);
  } else {
    if (deg == 4) PR_LAUNCH_DQ(__half, 4); else PR_LAUNCH_DQ(__half, 2);
  }
#undef PR_LAUNCH_DQ
  PR_CUDA(cudaGetLastError());
  return PR_OK;
}
