// Fused output kernel: intra-chunk causal power attention, state read-out, merge and
// normalisation in one pass (the reference's _attention followed by _query_state,
// retention/_attention/reference.py:10-69 and retention/_query_state/reference.py:36-96,
// with the gate glue of retention/power_retention_maker.py:180-190).
//
// One CTA owns 128 query rows of one (batch, chunk, query head).  For deg = 2
//     y_i = sum_{j<=i} (s q_i.k_j)^2 e^{a_i-a_j} v_j + phi(q~_i)^T Z_m
//     l_i = sum_{j<=i} (s q_i.k_j)^2 e^{a_i-a_j}     + q~_i^T Zg_m q~_i
//     O_i = y_i / l_i,           q~_i = s q_i e^{a_i/2}
// where Z_m is the state entering the chunk (pair-aligned triangle layout) and Zg_m the
// scanned Gram matrix of the discounted keys (equivalent to the reference's sum_of_keys).
// Because both terms share one fp32 accumulator in tensor memory, the reference's
// rowmax / sqrt(D) range management is not needed.
//
// Warp roles: warps 0-3 own one query row per thread (scores -> weights P, expansion
// phi(q~), epilogue), warp 4 issues TMA loads, warp 5 issues tcgen05.mma.
//   S = Q K_J^T        : A, B K-major in shared memory (TMA, 128-byte swizzle)
//   acc += P V_J       : A = P written to tensor memory by the row threads, B = V_J MN-major
//   acc += phi(q~) Z   : A = expansion written to tensor memory 64 rows at a time,
//                        B = 64-row blocks of Z by TMA
//   u = q~ Zg          : A = q~ in tensor memory, B = Zg (hi + lo halves)
#include "host.cuh"
#include "layout.cuh"
#include "sm100.cuh"

namespace pr {

namespace co {
constexpr int HD = 64;
constexpr int NS = 2;                 // expanded-operand ring in tensor memory: 2 stages of 128 entries (64 columns)
constexpr int NR = 4;                 // shared-memory ring: stages of 16 KB (a key and a value tile, or two state blocks)
constexpr int THREADS = 192;
constexpr int TILE_BYTES = 128 * 128;  // 128 rows x 64 16-bit features
constexpr int TW = 64;                 // keys per attention step
constexpr int KV_BYTES = TW * 128;     // one key or value tile
constexpr int Z_BYTES = 64 * 128;      // 64 expanded rows x 64 features
constexpr int R_BYTES = 2 * KV_BYTES;  // one ring stage
constexpr int DR = ref_dim(HD);        // 2560 expanded rows
constexpr int NBLK = DR / 64;          // 40 stages of 64 expanded rows (4 first factors x 16)
constexpr uint32_t TMEM_COLS = 256;
constexpr uint32_t COL_ACC = 0, COL_U = 64, COL_S = 128, COL_A = 128;  // S: 2 buffers x 64 columns, P aliased
}  // namespace co

struct ChunkOutParams {
  int hq, h;            // query heads, kv heads
  int n_chunks;         // chunks per batch element
  int cq, ck;           // queries / keys per chunk (query i sits at key position i + ck - cq)
  int tiles_per_chunk;  // ceil(cq / 128)
  int state_from_chunk; // chunks >= this read the state (n_chunks: never)
  int q_gate_last;      // 1: gate the state read-out with the gate at the last key (inference)
  int normalize;        // 1: O = y / l; 0: O = y (l is written either way when l_out != null)
  int has_attn;         // 0: no keys at all (state-only read-out)
  float scale;          // s
  const float* a;       // [b, n*ck, h] cumulative log gates inside each chunk, or null
  void* O;              // [b, n*cq, hq, 64]
  float* l_out;         // [b, n*cq, hq] or null
  int* status;
};

__device__ __forceinline__ void named_bar_sync(int id, int nthreads) {
  asm volatile("bar.sync %0, %1;" ::"r"(id), "r"(nthreads) : "memory");
}

// One 32-column half of an attention step for one query row: p = s^2 S^2 g into `pk`, row sum into
// l_acc.  SEP: the gate factor is c_i * fk[col] (c_i carries s^2); otherwise s^2 e^{a_i - ak[col]} per
// pair.  MASK: columns beyond `lim` (the row's own key position, relative to the step) are dropped.
template <typename T, int DEG, bool SEP, bool MASK>
__device__ __forceinline__ void out_half(const uint32_t (&sv)[32], const float* __restrict__ fk, float c_i, float a_i,
                                         int lim, uint32_t (&pk)[16], float& l_acc) {
  // two columns per instruction: packed fp32 multiplies and adds
  const float4* f4 = reinterpret_cast<const float4*>(fk);
  const float2 c2 = make_float2(c_i, c_i);
  float2 acc = make_float2(0.f, 0.f);
#pragma unroll
  for (int j = 0; j < 32; j += 4) {
    const float4 f = f4[j >> 2];
    const float2 fv[2] = {make_float2(f.x, f.y), make_float2(f.z, f.w)};
#pragma unroll
    for (int u = 0; u < 2; ++u) {
      const int col = j + 2 * u;
      const float2 s = make_float2(__uint_as_float(sv[col]), __uint_as_float(sv[col + 1]));
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
      float2 sq = __fmul2_rn(s, s);
      if (DEG == 4) sq = __fmul2_rn(sq, sq);
      const float2 pv = __fmul2_rn(sq, g);
      acc = __fadd2_rn(acc, pv);
      pk[col >> 1] = Pack2<T>::from_f32(pv.x, pv.y);
    }
  }
  l_acc += acc.x + acc.y;
}

template <typename T, int DEG>
__global__ void __launch_bounds__(co::THREADS, 2)
chunk_out_kernel(const ChunkOutParams p, const __grid_constant__ CUtensorMap tm_q,
                 const __grid_constant__ CUtensorMap tm_k, const __grid_constant__ CUtensorMap tm_v,
                 const __grid_constant__ CUtensorMap tm_z, const __grid_constant__ CUtensorMap tm_ghi,
                 const __grid_constant__ CUtensorMap tm_glo) {
  using namespace co;
  extern __shared__ uint8_t smem_raw[];
  __shared__ uint64_t q_full, r_full[NR], r_empty[NR], s_full[2], p_full[2], attn_done, g_full, acc_done;
  __shared__ uint64_t a_full[NS], a_empty[NS];
  __shared__ uint32_t tmem_base_s;
  __shared__ int abort_flag;
  __shared__ __align__(16) float sm_ak[2][TW];
  __shared__ __align__(16) float sm_fk[2][TW];  // e^{r - a_j}, r = gate sum at the step's last key
  __shared__ float sm_r[2];
  __shared__ int sm_wide[2][2];                 // a loader warp saw r - a_j > 80 (overflow guard)

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const uint32_t sbase = (smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t* sm = smem_raw + (sbase - smem_u32(smem_raw));
  uint8_t* smQ = sm;
  // One ring serves both phases: attention step J takes stage J % NR (key tile, then value tile);
  // the state read-out goes on with the same stage counter, two 64-row state blocks per stage,
  // so state blocks stream in while the last attention steps are still being computed.
  uint8_t* smR = smQ + TILE_BYTES;        // NR x R_BYTES
  uint8_t* smG = smR + NR * R_BYTES;      // hi, lo: 2 x Z_BYTES

  const int tile_i = blockIdx.x % p.tiles_per_chunk;
  const int chunk = blockIdx.x / p.tiles_per_chunk;
  const int qhead = blockIdx.y, batch = blockIdx.z;
  const int kvhead = qhead / (p.hq / p.h);
  const int q_off = p.ck - p.cq;
  const int row0 = tile_i * 128;
  const int last_key = min(p.ck - 1, row0 + 127 + q_off);
  const int nJ = p.has_attn ? last_key / TW + 1 : 0;
  const bool has_state = chunk >= p.state_from_chunk;

  if (tid == 0) {
    abort_flag = 0;
    mbar_init(&q_full, 1);
    for (int s = 0; s < 2; ++s) {
      mbar_init(&s_full[s], 1);
      mbar_init(&p_full[s], 4);
    }
    for (int s = 0; s < NR; ++s) {
      mbar_init(&r_full[s], 1);
      mbar_init(&r_empty[s], 1);
    }
    mbar_init(&attn_done, 1);
    mbar_init(&g_full, 1);
    mbar_init(&acc_done, 1);
    for (int s = 0; s < NS; ++s) {
      mbar_init(&a_full[s], 4);
      mbar_init(&a_empty[s], 1);
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
    // ------------------------------------------------------------ TMA producer
    if (lane == 0) {
      bool ok = true;
      mbar_expect_tx(&q_full, TILE_BYTES);
      tma_load_4d(smQ, &tm_q, &q_full, 0, qhead, chunk * p.cq + row0, batch);
      const int ch = (batch * p.n_chunks + chunk) * p.h + kvhead;
      if (has_state) {
        mbar_expect_tx(&g_full, 2 * Z_BYTES);
        tma_load_2d(smG, &tm_ghi, &g_full, 0, ch * HD);
        tma_load_2d(smG + Z_BYTES, &tm_glo, &g_full, 0, ch * HD);
      }
      const int n_ring = nJ + (has_state ? NBLK / 2 : 0);
      for (int g = 0; g < n_ring && ok; ++g) {
        const int s = g % NR, ph = (g / NR) & 1;
        ok = mbar_wait(&r_empty[s], ph ^ 1, &abort_flag);
        if (!ok) break;
        mbar_expect_tx(&r_full[s], R_BYTES);
        uint8_t* dst = smR + s * R_BYTES;
        if (g < nJ) {
          tma_load_4d(dst, &tm_k, &r_full[s], 0, kvhead, chunk * p.ck + g * TW, batch);
          tma_load_4d(dst + KV_BYTES, &tm_v, &r_full[s], 0, kvhead, chunk * p.ck + g * TW, batch);
        } else {
          const int blk = 2 * (g - nJ);
          tma_load_2d(dst, &tm_z, &r_full[s], 0, ch * DR + blk * 64);
          tma_load_2d(dst + Z_BYTES, &tm_z, &r_full[s], 0, ch * DR + (blk + 1) * 64);
        }
      }
    }
  } else if (warp == 5) {
    // -------------------------------------------------------------- MMA issuer
    if (lane == 0) {
      bool ok = mbar_wait(&q_full, 0, &abort_flag);
      const uint32_t idesc_s = umma_idesc(128, TW, Pack2<T>::is_bf16, false, false);
      const uint32_t idesc_v = umma_idesc(128, HD, Pack2<T>::is_bf16, false, true);
      const uint32_t idesc_g = umma_idesc(128, HD, Pack2<T>::is_bf16, false, false);
      const uint32_t q_addr = smem_u32(smQ);
      // scores of tile J+1 are issued before the P V product of tile J, so the row threads
      // always have the next tile waiting (two score buffers, two key/value stages)
      auto issue_scores = [&](int J) -> bool {
        const int s = J & 1;
        if (!mbar_wait(&r_full[J % NR], (J / NR) & 1, &abort_flag)) return false;
        tc_fence_after();
        const uint32_t k_addr = smem_u32(smR + (J % NR) * R_BYTES);
#pragma unroll
        for (int ks = 0; ks < 4; ++ks)
          umma_ss(tmem + COL_S + s * TW, umma_desc_sw128(q_addr + ks * 32, 16, 1024),
                  umma_desc_sw128(k_addr + ks * 32, 16, 1024), idesc_s, ks > 0 ? 1u : 0u);
        umma_commit(&s_full[s]);
        return true;
      };
      if (ok && nJ > 0) ok = issue_scores(0);
      for (int J = 0; J < nJ && ok; ++J) {
        const int s = J & 1;
        if (J + 1 < nJ) ok = issue_scores(J + 1);
        if (!ok) break;
        ok = mbar_wait(&p_full[s], (J >> 1) & 1, &abort_flag);
        if (!ok) break;
        tc_fence_after();
        const uint32_t v_addr = smem_u32(smR + (J % NR) * R_BYTES + KV_BYTES);
#pragma unroll
        for (int ks = 0; ks < TW / 16; ++ks)
          umma_ts(tmem + COL_ACC, tmem + COL_S + s * TW + ks * 8, umma_desc_sw128(v_addr + ks * 2048, 8192, 1024),
                  idesc_v, (J > 0 || ks > 0) ? 1u : 0u);
        umma_commit(&r_empty[J % NR]);
        if (J == nJ - 1) umma_commit(&attn_done);
      }
      if (ok && has_state) {
        // item 0: u = q~ Zg (hi then lo)
        ok = mbar_wait(&a_full[0], 0, &abort_flag) && mbar_wait(&g_full, 0, &abort_flag);
        if (ok) {
          tc_fence_after();
          const uint32_t g_addr = smem_u32(smG);
#pragma unroll
          for (int half = 0; half < 2; ++half)
#pragma unroll
            for (int ks = 0; ks < 4; ++ks)
              umma_ts(tmem + COL_U, tmem + COL_A + ks * 8,
                      umma_desc_sw128(g_addr + half * Z_BYTES + ks * 32, 16, 1024), idesc_g,
                      (half > 0 || ks > 0) ? 1u : 0u);
          umma_commit(&a_empty[0]);
        }
        // ring items 1 .. NBLK/2: 128 expanded entries against two state blocks (one ring stage);
        // eight products per pair of waits and commits keep this thread off the critical path
        for (int k = 1; k <= NBLK / 2 && ok; ++k) {
          const int s = k % NS, ph = (k / NS) & 1;
          const int g = nJ + k - 1, rs = g % NR;
          ok = mbar_wait(&a_full[s], ph, &abort_flag) && mbar_wait(&r_full[rs], (g / NR) & 1, &abort_flag);
          if (!ok) break;
          tc_fence_after();
          const uint32_t z_addr = smem_u32(smR + rs * R_BYTES);
#pragma unroll
          for (int ks = 0; ks < 8; ++ks)
            umma_ts(tmem + COL_ACC, tmem + COL_A + s * 64 + ks * 8,
                    umma_desc_sw128(z_addr + (ks >> 2) * Z_BYTES + (ks & 3) * 2048, 8192, 1024), idesc_v,
                    (nJ > 0 || k > 1 || ks > 0) ? 1u : 0u);
          // one commit per item: it frees the ring stage for the TMA thread and, two items on, the
          // tensor-memory slot for the expansion warps (a commit costs this thread ~150 clocks, a sixth of an item)
          umma_commit(&r_empty[rs]);
        }
      }
      if (ok) umma_commit(&acc_done);
    }
  } else {
    // --------------------------------------------------------- row-owning warps
    const int row = row0 + tid;                 // query index inside the chunk
    const bool row_valid = row < p.cq;
    const int qpos = row + q_off;               // key position of this query
    const uint32_t lane_addr = (uint32_t)(warp * 32) << 16;
    const bool gated = p.a != nullptr;
    const float* a_chunk = gated ? p.a + ((size_t)batch * p.n_chunks * p.ck + (size_t)chunk * p.ck) * p.h + kvhead
                                 : nullptr;
    const float a_i = (gated && row_valid) ? a_chunk[(size_t)qpos * p.h] : 0.f;
    const float s2 = DEG == 4 ? (p.scale * p.scale) * (p.scale * p.scale) : p.scale * p.scale;  // s^deg
    float l_acc = 0.f;
    bool ok = true;
    // gate sums of the next step's keys, loaded one step ahead by the first TW threads
    float av_n = 0.f, r_n = 0.f;
    auto load_gates = [&](int J) {
      if (tid < TW && gated) {
        const int kp = J * TW + tid;
        av_n = kp < p.ck ? a_chunk[(size_t)kp * p.h] : 0.f;
        r_n = a_chunk[(size_t)min(J * TW + TW - 1, p.ck - 1) * p.h];
      }
    };
    if (nJ > 0) load_gates(0);

    for (int J = 0; J < nJ; ++J) {
      const int kp0 = J * TW;
      const int sb = J & 1;
      if (tid < TW) {
        sm_ak[sb][tid] = av_n;
        sm_fk[sb][tid] = __expf(r_n - av_n);
        const bool wide = __any_sync(0xffffffffu, (r_n - av_n) > 80.f);
        if (lane == 0) sm_wide[sb][warp] = wide;
        if (tid == 0) sm_r[sb] = r_n;
      }
      named_bar_sync(1, 128);
      if (J + 1 < nJ) load_gates(J + 1);  // in flight while this step is computed
      ok = mbar_wait(&s_full[sb], (J >> 1) & 1, &abort_flag);
      if (!ok) break;
      tc_fence_after();
      const uint32_t col_s = COL_S + sb * TW;
      // The gate factor separates, e^{a_i - a_j} = e^{a_i - r} * e^{r - a_j}: one exponential per
      // row and per key instead of one per pair (both exponents <= 0 below the diagonal for gates
      // <= 0; a warp falls back to the per-pair form if one exceeds 80).  Steps wholly below the
      // diagonal need no mask; a warp whose rows all precede the step's keys writes zeros
      // without reading the scores.
      const int wq0 = row0 + (warp << 5) + q_off;  // key position of this warp's first query
      if (kp0 > min(wq0 + 31, p.ck - 1)) {
        uint32_t z[16];
#pragma unroll
        for (int j = 0; j < 16; ++j) z[j] = 0u;
        tmem_st16(tmem + lane_addr + col_s, z);
        tmem_st16(tmem + lane_addr + col_s + 16, z);
      } else {
        const float r = sm_r[sb];
        const bool mask = (kp0 + TW - 1 > wq0) || (kp0 + TW - 1 >= p.ck);
        const bool sep = !(sm_wide[sb][0] | sm_wide[sb][1]) && !__any_sync(0xffffffffu, (a_i - r) > 80.f);
        const float c_i = sep ? s2 * __expf(a_i - r) : s2;
        const int lim = min(qpos, p.ck - 1) - kp0;  // last column this row keeps
#pragma unroll 1
        for (int q4 = 0; q4 < TW / 32; ++q4) {
          uint32_t sv[32], pk[16];
          tmem_ld32(tmem + lane_addr + col_s + q4 * 32, sv);
          tmem_wait_ld();
          const int lm = lim - q4 * 32;
          if (sep) {
            if (mask) out_half<T, DEG, true, true>(sv, sm_fk[sb] + q4 * 32, c_i, a_i, lm, pk, l_acc);
            else out_half<T, DEG, true, false>(sv, sm_fk[sb] + q4 * 32, c_i, a_i, lm, pk, l_acc);
          } else {
            out_half<T, DEG, false, true>(sv, sm_ak[sb] + q4 * 32, c_i, a_i, lm, pk, l_acc);
          }
          tmem_st16(tmem + lane_addr + col_s + q4 * 16, pk);
        }
      }
      tmem_wait_st();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&p_full[sb]);
    }

    // gated, scaled query row as 32 packed pairs
    uint32_t q2[32];
    if (ok && has_state) {
      ok = mbar_wait(&q_full, 0, &abort_flag);
      float f = p.scale;
      if (gated) {
        const float a_g = p.q_gate_last ? a_chunk[(size_t)(p.ck - 1) * p.h] : a_i;
        f *= __expf(0.5f * a_g);
      }
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        const uint4 v = *reinterpret_cast<const uint4*>(smQ + swz128(tid, j));
        const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
        for (int k = 0; k < 4; ++k) {
          const float2 x = Pack2<T>::to_f32(w[k]);
          q2[4 * j + k] = Pack2<T>::from_f32(x.x * f, x.y * f);
        }
      }
      // the P columns alias the expansion ring: wait until the last P V product has read them
      if (ok && nJ > 0) ok = mbar_wait(&attn_done, 0, &abort_flag);
      tc_fence_after();
      if (ok) {
        // item 0: q~ itself (A operand of u = q~ Zg)
        tmem_st32(tmem + lane_addr + COL_A, q2);
        tmem_wait_st();
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(&a_full[0]);
      }
      // ring items 1..NBLK/2: 128 expanded entries (64 packed products) each.  The gated row goes
      // back to its own slot of the query tile so that the first factor can be fetched by a runtime
      // index; the loop over first factors then has a body of 64 multiplies per stage.
      if (ok) {
#pragma unroll
        for (int j = 0; j < 8; ++j)
          *reinterpret_cast<uint4*>(smQ + swz128(tid, j)) = make_uint4(q2[4 * j], q2[4 * j + 1], q2[4 * j + 2], q2[4 * j + 3]);
      }
      int k = 1;
      static_for<0, HD / 16>([&](auto yc) {
        constexpr int Y = decltype(yc)::value;
#pragma unroll 1
        for (int a0 = 0; a0 < 16 * (Y + 1); a0 += 8, ++k) {
          uint32_t r0[32], r1[32];
          expand_stage<T, Y>(smQ, tid, a0, q2, r0);
          expand_stage<T, Y>(smQ, tid, a0 + 4, q2, r1);
          const int s = k % NS;
          // the slot was last used by item k - 2: the Gram item (its own barrier) or a ring item, whose
          // completion the issuing thread reports on the ring stage's barrier
          if (ok && k == 2) ok = mbar_wait(&a_empty[0], 0, &abort_flag);
          if (ok && k >= 3) {
            const int g2 = nJ + k - 3;
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
      float l = l_acc;
      if (has_state) {
        // the state part of the row sum first, so that u and the accumulators are not live together
        uint32_t u[64];
        tmem_ld32(tmem + lane_addr + COL_U, u);
        tmem_ld32(tmem + lane_addr + COL_U + 32, u + 32);
        tmem_wait_ld();
        float ls0 = 0.f, ls1 = 0.f;
#pragma unroll
        for (int j = 0; j < 32; ++j) {
          const float2 qv = Pack2<T>::to_f32(q2[j]);
          ls0 = fmaf(__uint_as_float(u[2 * j]), qv.x, ls0);
          ls1 = fmaf(__uint_as_float(u[2 * j + 1]), qv.y, ls1);
        }
        l += ls0 + ls1;
      }
      uint32_t acc[64];
      tmem_ld32(tmem + lane_addr + COL_ACC, acc);
      tmem_ld32(tmem + lane_addr + COL_ACC + 32, acc + 32);
      tmem_wait_ld();
      if (row_valid) {
        const size_t tok = (size_t)batch * p.n_chunks * p.cq + (size_t)chunk * p.cq + row;
        const float inv = p.normalize ? safe_recip(l) : 1.f;
        uint4* dst = reinterpret_cast<uint4*>(static_cast<T*>(p.O) + (tok * p.hq + qhead) * HD);
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          uint4 v;
          v.x = Pack2<T>::from_f32(inv * __uint_as_float(acc[8 * j + 0]), inv * __uint_as_float(acc[8 * j + 1]));
          v.y = Pack2<T>::from_f32(inv * __uint_as_float(acc[8 * j + 2]), inv * __uint_as_float(acc[8 * j + 3]));
          v.z = Pack2<T>::from_f32(inv * __uint_as_float(acc[8 * j + 4]), inv * __uint_as_float(acc[8 * j + 5]));
          v.w = Pack2<T>::from_f32(inv * __uint_as_float(acc[8 * j + 6]), inv * __uint_as_float(acc[8 * j + 7]));
          dst[j] = v;
        }
        if (p.l_out != nullptr) p.l_out[tok * p.hq + qhead] = l;
      }
    }
  }
  tc_fence_before();
  __syncthreads();
  if (tid == 0 && abort_flag) *p.status = ST_TIMEOUT;
  if (warp == 0) tmem_dealloc(tmem, co::TMEM_COLS);
}

}  // namespace pr

extern "C" int pr_chunk_out(int dtype, int b, int n_chunks, int cq, int ck, int hq, int h, int d, const void* Q,
                            const void* K, const void* V, const float* a, const void* Z, const void* zg_hi,
                            const void* zg_lo, int state_from_chunk, int q_gate_last, int normalize, float scale,
                            int deg, void* O, float* l_out, int device, void* stream) {
  using namespace pr;
  using namespace pr::co;
  PR_REQUIRE(d == HD, PR_ERR_BAD_ARG, "head dim %d: this build handles d = 64", d);
  PR_REQUIRE(b > 0 && n_chunks > 0 && cq > 0 && ck >= cq && hq > 0 && h > 0 && hq % h == 0, PR_ERR_BAD_ARG,
             "bad sizes b=%d n=%d cq=%d ck=%d hq=%d h=%d", b, n_chunks, cq, ck, hq, h);
  PR_REQUIRE(dtype == PR_BF16 || dtype == PR_FP16, PR_ERR_BAD_ARG, "dtype %d", dtype);
  PR_REQUIRE(deg == 2 || (deg == 4 && Z == nullptr), PR_ERR_BAD_ARG,
             "deg=%d: states exist for deg 2; deg 4 runs state-free (attention only)", deg);
  const bool has_attn = (K != nullptr && V != nullptr);
  PR_REQUIRE(Q && O && aligned16(Q) && aligned16(O) && aligned16(K) && aligned16(V), PR_ERR_BAD_ARG,
             "null or misaligned pointer");
  PR_REQUIRE(has_attn || Z != nullptr, PR_ERR_BAD_ARG, "neither keys/values nor a state were given");
  const bool with_state = (Z != nullptr) && state_from_chunk < n_chunks;
  PR_REQUIRE(!with_state || (zg_hi && zg_lo && aligned16(Z) && aligned16(zg_hi) && aligned16(zg_lo)), PR_ERR_BAD_ARG,
             "state given without its Gram matrices");
  PR_REQUIRE(hq <= 65535 && b <= 65535, PR_ERR_BAD_ARG, "hq and b must be <= 65535");
  PR_CUDA(cudaSetDevice(device));
  ChunkOutParams p;
  p.hq = hq;
  p.h = h;
  p.n_chunks = n_chunks;
  p.cq = cq;
  p.ck = ck;
  p.tiles_per_chunk = (cq + 127) / 128;
  p.state_from_chunk = with_state ? state_from_chunk : n_chunks;
  p.q_gate_last = q_gate_last;
  p.normalize = normalize;
  p.has_attn = has_attn ? 1 : 0;
  p.scale = scale;
  p.a = a;
  p.O = O;
  p.l_out = l_out;
  int rc = status_word(device, &p.status, nullptr);
  if (rc) return rc;
  CUtensorMap tm_q, tm_k, tm_v, tm_z, tm_ghi, tm_glo;
  {
    const uint64_t tq = (uint64_t)n_chunks * cq, tk = (uint64_t)n_chunks * ck;
    uint64_t dq[4] = {(uint64_t)d, (uint64_t)hq, tq, (uint64_t)b};
    uint64_t sq[4] = {0, (uint64_t)d * 2, (uint64_t)hq * d * 2, tq * hq * d * 2};
    uint64_t dk[4] = {(uint64_t)d, (uint64_t)h, tk, (uint64_t)b};
    uint64_t sk[4] = {0, (uint64_t)d * 2, (uint64_t)h * d * 2, tk * h * d * 2};
    uint32_t box[4] = {64, 1, 128, 1};
    uint32_t box_kv[4] = {64, 1, (uint32_t)TW, 1};
    if ((rc = make_tmap(&tm_q, Q, 2, 4, dq, sq, box, true))) return rc;
    if (has_attn) {
      if ((rc = make_tmap(&tm_k, K, 2, 4, dk, sk, box_kv, true))) return rc;
      if ((rc = make_tmap(&tm_v, V, 2, 4, dk, sk, box_kv, true))) return rc;
    } else {
      tm_k = tm_q;
      tm_v = tm_q;
    }
  }
  if (with_state) {
    uint64_t dz[2] = {64, (uint64_t)b * n_chunks * h * ref_dim(d)};
    uint64_t dg[2] = {64, (uint64_t)b * n_chunks * h * d};
    uint64_t st[2] = {0, 128};
    uint32_t box[2] = {64, 64};
    if ((rc = make_tmap(&tm_z, Z, 2, 2, dz, st, box, true))) return rc;
    if ((rc = make_tmap(&tm_ghi, zg_hi, 2, 2, dg, st, box, true))) return rc;
    if ((rc = make_tmap(&tm_glo, zg_lo, 2, 2, dg, st, box, true))) return rc;
  } else {
    tm_z = tm_q;
    tm_ghi = tm_q;
    tm_glo = tm_q;
  }
  const size_t smem = 1024 + TILE_BYTES + NR * R_BYTES + 2 * Z_BYTES;
  dim3 grid(p.tiles_per_chunk * n_chunks, hq, b);
  cudaStream_t s = static_cast<cudaStream_t>(stream);
#define PR_LAUNCH_OUT(TT, DG)                                                                                      \
  do {                                                                                                             \
    PR_SMEM_ATTR((chunk_out_kernel<TT, DG>), smem, device, true);                                                   \
    chunk_out_kernel<TT, DG><<<grid, THREADS, smem, s>>>(p, tm_q, tm_k, tm_v, tm_z, tm_ghi, tm_glo);                 \
  } while (0)
  if (dtype == PR_BF16) {
    if (deg == 4) PR_LAUNCH_OUT(__nv_bfloat16, 4); else PR_LAUNCH_OUT(__nv_bfloat16, 2);
  } else {
    if (deg == 4) PR_LAUNCH_OUT(__half, 4); else PR_LAUNCH_OUT(__half, 2);
  }
#undef PR_LAUNCH_OUT
  PR_CUDA(cudaGetLastError());
  return PR_OK;
}
