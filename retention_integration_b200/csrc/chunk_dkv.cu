// Backward of the intra-chunk attention with respect to keys and values, merged with the
// state-path gradients (the reference's attn_bwd_dkdv, retention/_attention/triton.py:390-493,
// and the dV part of retention/_update_state/reference.py:55-60).
//
// One CTA owns 128 key rows (tile J) of one (batch, chunk, kv head); thread = key row.  For
// every tile of 64 queries at or after the key tile, of every query head of the group (tiles
// double-buffered in shared memory; 256 tensor memory columns, two CTAs per SM):
//     S^T = K_J Q_I^T,  dP^T = V_J dO_I^T                (tensor cores)
//     p = (s S)^2 e^{a_i-a_j},  dp = dP / l_i + dl_i,  dS = 2 s^2 S e^{a_i-a_j} dp
//     dV += (P / l)^T dO_I,   dK += dS^T Q_I             (A operands from tensor memory)
//     da_j -= sum_i p dp                                 (gate gradient, key side)
// then the state path of the values, dV += phi(k~_j)^T (w (.) dS_m) with k~ the discounted
// key (same expansion pipeline as the forward read-out).  The epilogue adds the state-path
// key gradient (fp32, from the expansion-gradient kernel) and writes dK, dV.
#include "host.cuh"
#include "layout.cuh"
#include "sm100.cuh"

namespace pr {

namespace dkv {
constexpr int HD = 64;
constexpr int NS = 2;                    // expanded-operand ring in tensor memory: 2 stages of 128 entries (64 columns)
constexpr int NR = 4;                    // shared-memory ring: stages of 16 KB (a query and a dO tile, or two state blocks)
constexpr int THREADS = 192;
constexpr int TILE_BYTES = 128 * 128;   // 128 key rows x 64 features
constexpr int TW = 64;                  // queries per step
constexpr int QD_BYTES = TW * 128;      // one query or dO tile
constexpr int Z_BYTES = 64 * 128;
constexpr int R_BYTES = 2 * QD_BYTES;   // one ring stage
constexpr int DR = ref_dim(HD);
constexpr int NBLK = DR / 64;           // 40 stages of 64 expanded rows
constexpr uint32_t TMEM_COLS = 256;     // two CTAs per SM
constexpr uint32_t COL_S = 0, COL_P = 0, COL_DP = 64, COL_DS = 64, COL_DV = 128, COL_DK = 192, COL_A = 0;
}  // namespace dkv

struct ChunkDkvParams {
  int hq, h, n_chunks, c, tiles_per_chunk;
  int state_chunk_hi;     // chunks <= this have a state-path dV term
  float scale;
  const float* a;         // [b, t, h] or null
  const float* A;         // [b, n, h] or null
  const float* dl;        // [b, t, hq]
  const float* l;         // [b, t, hq] row sums saved by the forward
  const float* dk_state;  // [b, t, h, 64] fp32 or null
  void* dK;
  void* dV;
  float* da_k;            // [b, t, h]
  int* status;
};

// One 32-column half of a step for one key row: P / l into `pk`, dS into `dk`, twice the row sum of
// p * dp into da2.  SEP: the gate factor is c_j * fq[col] (c_j carries 2 s^2); otherwise
// 2 s^2 e^{aq[col] - a_j} per pair, with columns beyond `hi` (past the chunk) dropped as well.
// MASK: columns before `lo` (queries that precede this key) are dropped.
template <typename T, int DEG, bool SEP, bool MASK>
__device__ __forceinline__ void dkv_half(const uint32_t (&sv)[32], const uint32_t (&pv)[32], const float* __restrict__ fq,
                                         const float* __restrict__ il, const float* __restrict__ hl,
                                         const float* __restrict__ dl, float c_j, float a_j, int lo, int hi,
                                         uint32_t (&pk)[16], uint32_t (&dk)[16], float& da2) {
  // two columns per instruction: packed fp32 multiplies and FMAs
  const float4* f4 = reinterpret_cast<const float4*>(fq);
  const float4* i4 = reinterpret_cast<const float4*>(il);
  const float4* h4 = reinterpret_cast<const float4*>(hl);
  const float4* d4 = reinterpret_cast<const float4*>(dl);
  const float2 c2 = make_float2(c_j, c_j);
  float2 acc = make_float2(0.f, 0.f);
#pragma unroll
  for (int j = 0; j < 32; j += 4) {
    const float4 f = f4[j >> 2], iq = i4[j >> 2], hq = h4[j >> 2], dq = d4[j >> 2];
    const float2 fv[2] = {make_float2(f.x, f.y), make_float2(f.z, f.w)};
    const float2 iv[2] = {make_float2(iq.x, iq.y), make_float2(iq.z, iq.w)};
    const float2 hv[2] = {make_float2(hq.x, hq.y), make_float2(hq.z, hq.w)};
    const float2 dv[2] = {make_float2(dq.x, dq.y), make_float2(dq.z, dq.w)};
#pragma unroll
    for (int u = 0; u < 2; ++u) {
      const int col = j + 2 * u;
      const float2 s = make_float2(__uint_as_float(sv[col]), __uint_as_float(sv[col + 1]));
      const float2 p = make_float2(__uint_as_float(pv[col]), __uint_as_float(pv[col + 1]));
      float2 g;
      if (SEP) {
        g = __fmul2_rn(c2, fv[u]);
      } else {
        g = make_float2(c_j * __expf(fv[u].x - a_j), c_j * __expf(fv[u].y - a_j));
        g.x = (col <= hi) ? g.x : 0.f;
        g.y = (col + 1 <= hi) ? g.y : 0.f;
      }
      if (MASK) {
        g.x = (col >= lo) ? g.x : 0.f;
        g.y = (col + 1 >= lo) ? g.y : 0.f;
      }
      const float2 sp = DEG == 4 ? __fmul2_rn(s, __fmul2_rn(s, s)) : s;  // S^(deg-1)
      const float2 sg2 = __fmul2_rn(sp, g);  // deg s^deg S^(deg-1) e^{a_i-a_j}
      const float2 dp = __ffma2_rn(p, iv[u], dv[u]);
      const float2 ds = __fmul2_rn(sg2, dp);
      acc = __ffma2_rn(ds, s, acc);
      const float2 pw = __fmul2_rn(__fmul2_rn(sg2, s), hv[u]);
      pk[col >> 1] = Pack2<T>::from_f32(pw.x, pw.y);
      dk[col >> 1] = Pack2<T>::from_f32(ds.x, ds.y);
    }
  }
  da2 += acc.x + acc.y;
}

template <typename T, int DEG>
__global__ void __launch_bounds__(dkv::THREADS, 2)
chunk_dkv_kernel(const ChunkDkvParams p, const __grid_constant__ CUtensorMap tm_k,
                 const __grid_constant__ CUtensorMap tm_v, const __grid_constant__ CUtensorMap tm_q,
                 const __grid_constant__ CUtensorMap tm_dy, const __grid_constant__ CUtensorMap tm_ds) {
  using namespace dkv;
  extern __shared__ uint8_t smem_raw[];
  __shared__ uint64_t kv_full, r_full[NR], r_empty[NR], sp_full, pd_full, attn_done, acc_done;
  __shared__ uint64_t a_full[NS];
  __shared__ uint32_t tmem_base_s;
  __shared__ int abort_flag;
  __shared__ __align__(16) float sm_aq[2][TW], sm_dl[2][TW], sm_il[2][TW];
  __shared__ __align__(16) float sm_fq[2][TW];  // e^{a_i - r}, r = gate sum at the step's first query
  __shared__ __align__(16) float sm_hl[2][TW];  // 1 / (2 l_i)
  __shared__ float sm_r[2];
  __shared__ int sm_wide[2][2];                 // a loader warp saw a_i - r > 80 (overflow guard)

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const uint32_t sbase = (smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t* sm = smem_raw + (sbase - smem_u32(smem_raw));
  uint8_t* smK = sm;
  uint8_t* smV = smK + TILE_BYTES;
  // One ring serves both phases: attention step st takes stage st % NR (query tile, then dO tile);
  // the state phase goes on with the same stage counter, two 64-row state blocks per stage, so
  // state blocks stream in while the last attention steps are still being computed.
  uint8_t* smR = smV + TILE_BYTES;       // NR x R_BYTES

  const int tile_j = blockIdx.x % p.tiles_per_chunk;
  const int chunk = blockIdx.x / p.tiles_per_chunk;
  const int kvhead = blockIdx.y, batch = blockIdx.z;
  const int ratio = p.hq / p.h;
  const int row0 = tile_j * 128;
  const int tok_chunk = chunk * p.c;
  const int q_tiles = (p.c + TW - 1) / TW;      // query tiles of TW rows in the chunk
  const int qt0 = row0 / TW;                    // first query tile that can see this key tile
  const int nI = q_tiles - qt0;
  const int n_steps = nI * ratio;
  const bool has_state = chunk <= p.state_chunk_hi;

  if (tid == 0) {
    abort_flag = 0;
    mbar_init(&kv_full, 1);
    for (int s = 0; s < NR; ++s) {
      mbar_init(&r_full[s], 1);
      mbar_init(&r_empty[s], 1);
    }
    mbar_init(&sp_full, 1);
    mbar_init(&pd_full, 4);
    mbar_init(&attn_done, 1);
    mbar_init(&acc_done, 1);
    for (int s = 0; s < NS; ++s) {
      mbar_init(&a_full[s], 4);
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

  if (warp == 4) {
    if (lane == 0) {
      bool ok = true;
      mbar_expect_tx(&kv_full, 2 * TILE_BYTES);
      tma_load_4d(smK, &tm_k, &kv_full, 0, kvhead, tok_chunk + row0, batch);
      tma_load_4d(smV, &tm_v, &kv_full, 0, kvhead, tok_chunk + row0, batch);
      const int ch = (batch * p.n_chunks + chunk) * p.h + kvhead;
      const int n_ring = n_steps + (has_state ? NBLK / 2 : 0);
      for (int g = 0; g < n_ring && ok; ++g) {
        const int s = g % NR, ph = (g / NR) & 1;
        ok = mbar_wait(&r_empty[s], ph ^ 1, &abort_flag);
        if (!ok) break;
        mbar_expect_tx(&r_full[s], R_BYTES);
        uint8_t* dst = smR + s * R_BYTES;
        if (g < n_steps) {
          const int I = qt0 + g / ratio, qh = kvhead * ratio + g % ratio;
          tma_load_4d(dst, &tm_q, &r_full[s], 0, qh, tok_chunk + I * TW, batch);
          tma_load_4d(dst + QD_BYTES, &tm_dy, &r_full[s], 0, qh, tok_chunk + I * TW, batch);
        } else {
          const int blk = 2 * (g - n_steps);
          tma_load_2d(dst, &tm_ds, &r_full[s], 0, ch * DR + blk * 64);
          tma_load_2d(dst + Z_BYTES, &tm_ds, &r_full[s], 0, ch * DR + (blk + 1) * 64);
        }
      }
    }
  } else if (warp == 5) {
    if (lane == 0) {
      bool ok = mbar_wait(&kv_full, 0, &abort_flag);
      const uint32_t idesc_s = umma_idesc(128, TW, Pack2<T>::is_bf16, false, false);
      const uint32_t idesc_o = umma_idesc(128, HD, Pack2<T>::is_bf16, false, true);
      const uint32_t k_addr = smem_u32(smK), v_addr = smem_u32(smV);
      for (int st = 0; st < n_steps && ok; ++st) {
        const int sg = st % NR;
        ok = mbar_wait(&r_full[sg], (st / NR) & 1, &abort_flag);
        if (!ok) break;
        tc_fence_after();
        const uint32_t q_addr = smem_u32(smR + sg * R_BYTES), dy_addr = q_addr + QD_BYTES;
#pragma unroll
        for (int ks = 0; ks < 4; ++ks)
          umma_ss(tmem + COL_S, umma_desc_sw128(k_addr + ks * 32, 16, 1024),
                  umma_desc_sw128(q_addr + ks * 32, 16, 1024), idesc_s, ks > 0 ? 1u : 0u);
#pragma unroll
        for (int ks = 0; ks < 4; ++ks)
          umma_ss(tmem + COL_DP, umma_desc_sw128(v_addr + ks * 32, 16, 1024),
                  umma_desc_sw128(dy_addr + ks * 32, 16, 1024), idesc_s, ks > 0 ? 1u : 0u);
        umma_commit(&sp_full);
        ok = mbar_wait(&pd_full, st & 1, &abort_flag);
        if (!ok) break;
        tc_fence_after();
#pragma unroll
        for (int ks = 0; ks < TW / 16; ++ks)
          umma_ts(tmem + COL_DV, tmem + COL_P + ks * 8, umma_desc_sw128(dy_addr + ks * 2048, 8192, 1024), idesc_o,
                  (st > 0 || ks > 0) ? 1u : 0u);
#pragma unroll
        for (int ks = 0; ks < TW / 16; ++ks)
          umma_ts(tmem + COL_DK, tmem + COL_DS + ks * 8, umma_desc_sw128(q_addr + ks * 2048, 8192, 1024), idesc_o,
                  (st > 0 || ks > 0) ? 1u : 0u);
        umma_commit(&r_empty[sg]);
        if (st == n_steps - 1) umma_commit(&attn_done);
      }
      if (ok && has_state) {
        // 128 expanded entries against two state blocks (one ring stage) per item: eight products
        // per pair of waits and commits keep this thread off the critical path
        for (int k = 0; k < NBLK / 2 && ok; ++k) {
          const int s = k % NS, ph = (k / NS) & 1;
          const int g = n_steps + k, rs = g % NR;
          ok = mbar_wait(&a_full[s], ph, &abort_flag) && mbar_wait(&r_full[rs], (g / NR) & 1, &abort_flag);
          if (!ok) break;
          tc_fence_after();
          const uint32_t z_addr = smem_u32(smR + rs * R_BYTES);
#pragma unroll
          for (int ks = 0; ks < 8; ++ks)
            umma_ts(tmem + COL_DV, tmem + COL_A + s * 64 + ks * 8,
                    umma_desc_sw128(z_addr + (ks >> 2) * Z_BYTES + (ks & 3) * 2048, 8192, 1024), idesc_o, 1u);
          // one commit per item: it frees the ring stage for the TMA thread and, two items on, the
          // tensor-memory slot for the expansion warps
          umma_commit(&r_empty[rs]);
        }
      }
      if (ok) umma_commit(&acc_done);
    }
  } else {
    const int row = row0 + tid;  // key index inside the chunk
    const bool row_valid = row < p.c;
    const uint32_t lane_addr = (uint32_t)(warp * 32) << 16;
    const bool gated = p.a != nullptr;
    const size_t tok_base = (size_t)batch * p.n_chunks * p.c + tok_chunk;
    const float* a_chunk = gated ? p.a + tok_base * p.h + kvhead : nullptr;
    const float a_j = (gated && row_valid) ? a_chunk[(size_t)row * p.h] : 0.f;
    const float s2 = DEG == 4 ? (p.scale * p.scale) * (p.scale * p.scale) : p.scale * p.scale;  // s^deg
    float da2 = 0.f;  // twice the row sum of p * dp
    bool ok = true;
    // per-query values of the next step, loaded one step ahead by the first TW threads
    float av_n = 0.f, r_n = 0.f, dl_n = 0.f, l_n = 1.f;
    auto load_cols = [&](int st) {
      if (tid < TW) {
        const int qp0 = (qt0 + st / ratio) * TW, qh = kvhead * ratio + st % ratio;
        const int qp = qp0 + tid;
        const bool v = qp < p.c;
        av_n = (gated && v) ? a_chunk[(size_t)qp * p.h] : 0.f;
        r_n = gated ? a_chunk[(size_t)qp0 * p.h] : 0.f;
        dl_n = v ? p.dl[(tok_base + qp) * p.hq + qh] : 0.f;
        l_n = v ? p.l[(tok_base + qp) * p.hq + qh] : 1.f;
      }
    };
    if (n_steps > 0) load_cols(0);
    for (int st = 0; st < n_steps; ++st) {
      const int I = qt0 + st / ratio;
      const int qp0 = I * TW;
      const int sb = st & 1;
      if (tid < TW) {
        const bool v = qp0 + tid < p.c;
        const float il = v ? safe_recip(l_n) : 0.f;
        sm_aq[sb][tid] = av_n;
        sm_dl[sb][tid] = dl_n;
        sm_il[sb][tid] = il;
        sm_hl[sb][tid] = (1.f / DEG) * il;
        sm_fq[sb][tid] = v ? __expf(av_n - r_n) : 0.f;
        const bool wide = __any_sync(0xffffffffu, (av_n - r_n) > 80.f);
        if (lane == 0) sm_wide[sb][warp] = wide;
        if (tid == 0) sm_r[sb] = r_n;
      }
      asm volatile("bar.sync 1, 128;" ::: "memory");
      if (st + 1 < n_steps) load_cols(st + 1);  // in flight while this step is computed
      ok = mbar_wait(&sp_full, st & 1, &abort_flag);
      if (!ok) break;
      tc_fence_after();
      // The gate factor separates, e^{a_i - a_j} = e^{a_i - r} * e^{r - a_j}: one exponential per
      // key and per query instead of one per pair (both exponents <= 0 off the diagonal for gates
      // <= 0; a warp falls back to the per-pair form if one exceeds 80).  Steps whose queries all
      // come after this warp's keys need no mask; a warp whose keys all come after the step's
      // queries writes zeros without reading the scores.
      const int wrow0 = row0 + (warp << 5);
      if (qp0 + TW - 1 < wrow0 || wrow0 >= p.c) {
        uint32_t z[16];
#pragma unroll
        for (int j = 0; j < 16; ++j) z[j] = 0u;
        tmem_st16(tmem + lane_addr + COL_P, z);
        tmem_st16(tmem + lane_addr + COL_P + 16, z);
        tmem_st16(tmem + lane_addr + COL_DS, z);
        tmem_st16(tmem + lane_addr + COL_DS + 16, z);
      } else {
        const float r = sm_r[sb];
        const bool mask = (wrow0 + 31 > qp0) || (wrow0 + 31 >= p.c);
        const bool sep = (qp0 + TW - 1 < p.c) && !(sm_wide[sb][0] | sm_wide[sb][1]) &&
                         !__any_sync(0xffffffffu, (r - a_j) > 80.f);
        const float c_j = sep ? (float)DEG * s2 * __expf(r - a_j) : (float)DEG * s2;
        const int lo = row_valid ? row - qp0 : TW;  // first query column this key keeps
        const int hi = p.c - 1 - qp0;               // last column inside the chunk
#pragma unroll 1
        for (int q4 = 0; q4 < TW / 32; ++q4) {
          uint32_t sv[32], pv[32], pk[16], dk[16];
          tmem_ld32(tmem + lane_addr + COL_S + q4 * 32, sv);
          tmem_ld32(tmem + lane_addr + COL_DP + q4 * 32, pv);
          tmem_wait_ld();
          const float* il = sm_il[sb] + q4 * 32;
          const float* hl = sm_hl[sb] + q4 * 32;
          const float* dl = sm_dl[sb] + q4 * 32;
          const int lo4 = lo - q4 * 32, hi4 = hi - q4 * 32;
          if (sep) {
            if (mask) dkv_half<T, DEG, true, true>(sv, pv, sm_fq[sb] + q4 * 32, il, hl, dl, c_j, a_j, lo4, hi4, pk, dk, da2);
            else dkv_half<T, DEG, true, false>(sv, pv, sm_fq[sb] + q4 * 32, il, hl, dl, c_j, a_j, lo4, hi4, pk, dk, da2);
          } else {
            dkv_half<T, DEG, false, true>(sv, pv, sm_aq[sb] + q4 * 32, il, hl, dl, c_j, a_j, lo4, hi4, pk, dk, da2);
          }
          tmem_st16(tmem + lane_addr + COL_P + q4 * 16, pk);
          tmem_st16(tmem + lane_addr + COL_DS + q4 * 16, dk);
        }
      }
      tmem_wait_st();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&pd_full);
    }

    if (ok && has_state) {
      ok = mbar_wait(&kv_full, 0, &abort_flag);
      float f = 1.f;
      if (gated) {
        const float A = p.A[(batch * p.n_chunks + chunk) * p.h + kvhead];
        f = __expf(0.5f * (A - a_j));
      }
      uint32_t k2[32];
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        const uint4 v = *reinterpret_cast<const uint4*>(smK + swz128(tid, j));
        const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
        for (int k = 0; k < 4; ++k) {
          const float2 x = Pack2<T>::to_f32(w[k]);
          k2[4 * j + k] = Pack2<T>::from_f32(x.x * f, x.y * f);
        }
      }
      if (ok && n_steps > 0) ok = mbar_wait(&attn_done, 0, &abort_flag);
      tc_fence_after();
      // the discounted row goes back to its own slot of the key tile (first factors are fetched
      // by a runtime index); the attention products that read the tile have completed
      if (ok) {
#pragma unroll
        for (int j = 0; j < 8; ++j)
          *reinterpret_cast<uint4*>(smK + swz128(tid, j)) = make_uint4(k2[4 * j], k2[4 * j + 1], k2[4 * j + 2], k2[4 * j + 3]);
      }
      int k = 0;
      static_for<0, HD / 16>([&](auto yc) {
        constexpr int Y = decltype(yc)::value;
#pragma unroll 1
        for (int a0 = 0; a0 < 16 * (Y + 1); a0 += 8, ++k) {
          uint32_t r0[32], r1[32];
          expand_stage<T, Y>(smK, tid, a0, k2, r0);
          expand_stage<T, Y>(smK, tid, a0 + 4, k2, r1);
          const int s = k % NS;
          if (ok && k >= NS) {
            // the slot was last used by item k - NS, whose completion is reported on its ring stage's barrier
            const int g2 = n_steps + k - NS;
            ok = mbar_wait(&r_empty[g2 % NR], (g2 / NR) & 1, &abort_flag);
          }
          if (ok) {
            tc_fence_after();
            tmem_st32(tmem + lane_addr + COL_A + s * 64, r0);
            tmem_st32(tmem + lane_addr + COL_A + s * 64 + 32, r1);
            tmem_wait_st();
            tc_fence_before();
          }
          __syncwarp();
          if (ok && lane == 0) mbar_arrive(&a_full[s]);
        }
      });
    }

    if (ok) ok = mbar_wait(&acc_done, 0, &abort_flag);
    tc_fence_after();
    if (ok) {
      uint32_t acc[64];
      const size_t tok = tok_base + row;
      // dV
      tmem_ld32(tmem + lane_addr + COL_DV, acc);
      tmem_ld32(tmem + lane_addr + COL_DV + 32, acc + 32);
      tmem_wait_ld();
      if (row_valid) {
        uint4* dst = reinterpret_cast<uint4*>(static_cast<T*>(p.dV) + (tok * p.h + kvhead) * HD);
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          uint4 v;
          v.x = Pack2<T>::from_f32(__uint_as_float(acc[8 * j + 0]), __uint_as_float(acc[8 * j + 1]));
          v.y = Pack2<T>::from_f32(__uint_as_float(acc[8 * j + 2]), __uint_as_float(acc[8 * j + 3]));
          v.z = Pack2<T>::from_f32(__uint_as_float(acc[8 * j + 4]), __uint_as_float(acc[8 * j + 5]));
          v.w = Pack2<T>::from_f32(__uint_as_float(acc[8 * j + 6]), __uint_as_float(acc[8 * j + 7]));
          dst[j] = v;
        }
      }
      // dK
      tmem_ld32(tmem + lane_addr + COL_DK, acc);
      tmem_ld32(tmem + lane_addr + COL_DK + 32, acc + 32);
      tmem_wait_ld();
      if (row_valid) {
        const float4* st = p.dk_state ? reinterpret_cast<const float4*>(p.dk_state + (tok * p.h + kvhead) * HD)
                                      : nullptr;
        uint4* dst = reinterpret_cast<uint4*>(static_cast<T*>(p.dK) + (tok * p.h + kvhead) * HD);
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          float4 s0 = make_float4(0.f, 0.f, 0.f, 0.f), s1 = s0;
          if (st) {
            s0 = st[2 * j];
            s1 = st[2 * j + 1];
          }
          uint4 v;
          v.x = Pack2<T>::from_f32(__uint_as_float(acc[8 * j + 0]) + s0.x, __uint_as_float(acc[8 * j + 1]) + s0.y);
          v.y = Pack2<T>::from_f32(__uint_as_float(acc[8 * j + 2]) + s0.z, __uint_as_float(acc[8 * j + 3]) + s0.w);
          v.z = Pack2<T>::from_f32(__uint_as_float(acc[8 * j + 4]) + s1.x, __uint_as_float(acc[8 * j + 5]) + s1.y);
          v.w = Pack2<T>::from_f32(__uint_as_float(acc[8 * j + 6]) + s1.z, __uint_as_float(acc[8 * j + 7]) + s1.w);
          dst[j] = v;
        }
        p.da_k[tok * p.h + kvhead] = (-1.f / DEG) * da2;
      }
    }
  }
  tc_fence_before();
  __syncthreads();
  if (tid == 0 && abort_flag) *p.status = ST_TIMEOUT;
  if (warp == 0) tmem_dealloc(tmem, dkv::TMEM_COLS);
}

}  // namespace pr

extern "C" int pr_chunk_dkv(int dtype, int b, int t, int hq, int h, int d, int c, const void* Q, const void* dO,
                            const void* K, const void* V, const void* wdS, const float* a, const float* A,
                            const float* dl, const float* l, const float* dk_state, int state_chunk_hi, float scale,
                            int deg, void* dK, void* dV, float* da_k, int device, void* stream) {
  using namespace pr;
  using namespace pr::dkv;
  PR_REQUIRE(deg == 2 || (deg == 4 && wdS == nullptr && dk_state == nullptr), PR_ERR_BAD_ARG,
             "deg=%d: states exist for deg 2; deg 4 runs state-free (attention only)", deg);
  PR_REQUIRE(d == HD, PR_ERR_BAD_ARG, "head dim %d: this build handles d = 64", d);
  PR_REQUIRE(b > 0 && t > 0 && hq > 0 && h > 0 && hq % h == 0 && c > 0 && t % c == 0, PR_ERR_BAD_ARG,
             "bad sizes b=%d t=%d hq=%d h=%d c=%d", b, t, hq, h, c);
  PR_REQUIRE(dtype == PR_BF16 || dtype == PR_FP16, PR_ERR_BAD_ARG, "dtype %d", dtype);
  PR_REQUIRE(Q && dO && K && V && dl && l && dK && dV && da_k, PR_ERR_BAD_ARG, "null pointer");
  PR_REQUIRE(aligned16(Q) && aligned16(dO) && aligned16(K) && aligned16(V) && aligned16(dK) && aligned16(dV) &&
                 aligned16(wdS) && aligned16(dk_state),
             PR_ERR_BAD_ARG, "misaligned pointer");
  PR_REQUIRE(!(wdS != nullptr && a != nullptr) || A != nullptr, PR_ERR_BAD_ARG,
             "gated state path needs the chunk gate totals A");
  PR_REQUIRE(h <= 65535 && b <= 65535, PR_ERR_BAD_ARG, "h and b must be <= 65535");
  PR_CUDA(cudaSetDevice(device));
  ChunkDkvParams p;
  p.hq = hq;
  p.h = h;
  p.n_chunks = t / c;
  p.c = c;
  p.tiles_per_chunk = (c + 127) / 128;
  p.state_chunk_hi = wdS ? state_chunk_hi : -1;
  p.scale = scale;
  p.a = a;
  p.A = A;
  p.dl = dl;
  p.l = l;
  p.dk_state = dk_state;
  p.dK = dK;
  p.dV = dV;
  p.da_k = da_k;
  int rc = status_word(device, &p.status, nullptr);
  if (rc) return rc;
  CUtensorMap tm_q, tm_dy, tm_k, tm_v, tm_ds;
  uint64_t dq_[4] = {(uint64_t)d, (uint64_t)hq, (uint64_t)t, (uint64_t)b};
  uint64_t sq[4] = {0, (uint64_t)d * 2, (uint64_t)hq * d * 2, (uint64_t)t * hq * d * 2};
  uint64_t dk[4] = {(uint64_t)d, (uint64_t)h, (uint64_t)t, (uint64_t)b};
  uint64_t sk[4] = {0, (uint64_t)d * 2, (uint64_t)h * d * 2, (uint64_t)t * h * d * 2};
  uint32_t box[4] = {64, 1, 128, 1};
  uint32_t box_q[4] = {64, 1, (uint32_t)TW, 1};
  if ((rc = make_tmap(&tm_q, Q, 2, 4, dq_, sq, box_q, true))) return rc;
  if ((rc = make_tmap(&tm_dy, dO, 2, 4, dq_, sq, box_q, true))) return rc;
  if ((rc = make_tmap(&tm_k, K, 2, 4, dk, sk, box, true))) return rc;
  if ((rc = make_tmap(&tm_v, V, 2, 4, dk, sk, box, true))) return rc;
  if (wdS) {
    uint64_t dz[2] = {64, (uint64_t)b * p.n_chunks * h * ref_dim(d)};
    uint64_t st[2] = {0, 128};
    uint32_t bz[2] = {64, 64};
    if ((rc = make_tmap(&tm_ds, wdS, 2, 2, dz, st, bz, true))) return rc;
  } else {
    tm_ds = tm_q;
  }
  const size_t smem = 1024 + 2 * TILE_BYTES + NR * R_BYTES;
  dim3 grid(p.tiles_per_chunk * p.n_chunks, h, b);
  cudaStream_t s = static_cast<cudaStream_t>(stream);
#define PR_LAUNCH_DKV(TT, DG)                                                                                      \
  do {                                                                                                             \
    PR_SMEM_ATTR((chunk_dkv_kernel<TT, DG>), smem, device, true);                                                   \
    chunk_dkv_kernel<TT, DG><<<grid, THREADS, smem, s>>>(p, tm_k, tm_v, tm_q, tm_dy, tm_ds);                         \
  } while (0)
  if (dtype == PR_BF16) {
    if (deg == 4) PR_LAUNCH_DKV(__nv_bfloat16, 4); else PR_LAUNCH_DKV(__nv_bfloat16, 2);
  } else {
    if (deg == 4) PR_LAUNCH_DKV(__half, 4); else PR_LAUNCH_DKV(__half, 2);
  }
#undef PR_LAUNCH_DKV
  PR_CUDA(cudaGetLastError());
  return PR_OK;
}
