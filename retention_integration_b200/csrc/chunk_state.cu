// Token-contracting expansion kernel:  out[D2, e] = w (.) sum_i phi(x_i) v_i^T  per
// (batch, chunk, head), and the d x d Gram matrix  gram = sum_i xs_i x_i^T.
//
// Forward use (the reference's update_state, retention/_update_state/reference.py:31-53):
//   x = discounted keys, v = values, key weights on -> chunk state S_m; the Gram matrix
//   of the discounted keys carries the same information as the reference's sum_of_keys
//   N_m (N[(a,b)] = w(a,b) * gram[a][b]).
// Backward use (gradient of the state read-out, retention/_query_state/triton.py:337-448):
//   x = gated queries, v = dO / l, weights off -> dZ_m; xs = x * dl -> gram = d(gram of Z).
//
// One CTA owns two tiles of 128 expanded rows, so every operand stage fetched from L2 feeds two
// products.  The expansion is never written to shared or global memory: each thread owns the
// expanded rows (a, b) and (a + 8, b) - the same row of both tiles, which share their second
// factor - for half of the tokens of a stage, multiplies rows a, a + 8 and b of the transposed
// operand (TMA-loaded, 128-byte swizzled) with packed 16-bit multiplies and stores the products
// straight into tensor memory as the A operands of tcgen05.mma.  The kernel is bound by the
// shared-memory reads that feed those multiplies (traced: ~1000 clocks per stage and SM against ~430
// for the tensor core), which is why the second factor is read once for two products; the values come in by TMA as the MN-major B operand; fp32 accumulation in
// tensor memory.  The last grid slot in x computes the Gram matrix with both operands
// in shared memory.
#include "host.cuh"
#include "layout.cuh"
#include "sm100.cuh"

namespace pr {

namespace cs {
constexpr int HD = 64;          // head dim handled by this build of the kernel
constexpr int NS = 4;           // shared-memory pipeline stages
constexpr int NSA = 2;          // tensor-memory stages of each group's expansion ring
constexpr int NG = 2;           // row tiles (groups of 4 warps) per CTA: each loaded stage feeds both
constexpr int TOK = 64;         // tokens per stage
constexpr int THREADS = 352;    // warps 0-3 / 4-7 expand + epilogue (one group per row tile), 8 TMA, 9 / 10 MMA of group 0 / 1
constexpr int XT_BYTES = HD * TOK * 2;   // 8 KB
constexpr int W_BYTES = TOK * HD * 2;    // 8 KB
constexpr int GA_BYTES = 128 * TOK * 2;  // Gram A operand padded to 128 rows
constexpr uint32_t TMEM_COLS = 256;
constexpr uint32_t COL_ACC = 0;    // NG x 64 columns
constexpr uint32_t COL_A = 128;    // NG rings of NSA x 32 columns
}  // namespace cs

struct ChunkStateParams {
  int n_tiles;      // tiles of 128 expanded rows; grid.x = ceil(n_tiles / 2) + (gram ? 1 : 0)
  int nh;           // kv heads of the output
  int group;        // operand heads summed into one output head (GQA ratio in backward)
  int c, cp;        // chunk length, padded to 64
  int n_chunks;     // chunks per batch element
  int key_weights;  // 1: weight 2 on pairs from different 16-blocks; 0: all weights 1
  void* out;        // [b, n, nh, D2, 64]
  float* gram;      // [b, n, nh, 64, 64] or null
  int* status;
};

template <typename T>
__global__ void __maxnreg__(80)
chunk_state_kernel(const ChunkStateParams p, const __grid_constant__ CUtensorMap tm_xt,
                   const __grid_constant__ CUtensorMap tm_xs, const __grid_constant__ CUtensorMap tm_w) {
  using namespace cs;
  extern __shared__ uint8_t smem_raw[];
  // done[g][s]: the products of group g on stage s have completed.  ONE commit per stage and issuing thread
  // serves both waiters - the expansion warps (their tensor-memory slot of two stages ago is free) and the TMA
  // thread (the value tile of four stages ago is free): a commit costs the issuing thread ~150 clocks, a third
  // of what the four products of a stage cost it.
  __shared__ uint64_t x_full[NS], x_empty[NS], w_full[NS], w_empty[NS], a_full[NG][NSA], done[NG][NS], acc_done;
  __shared__ uint32_t tmem_base_s;
  __shared__ int abort_flag;

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const uint32_t sbase = (smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t* sm = smem_raw + (sbase - smem_u32(smem_raw));
  uint8_t* smX = sm;                          // NS x XT_BYTES (rows = features, 64 tokens)
  uint8_t* smW = sm + NS * XT_BYTES;          // NS x W_BYTES  (rows = tokens, 64 features)
  uint8_t* smG = smW;                         // Gram CTA only: 2 x GA_BYTES over the (unused) value ring

  // grid.x = slots * (batch, chunk, head) triples, slot fastest: the CTAs of one triple run together and
  // share their operand tiles through L2, and the triple count is not bound by the 65535 limit of grid.y
  const int n_tile_ctas = (p.n_tiles + NG - 1) / NG;
  const int slots = n_tile_ctas + (p.gram ? 1 : 0);
  const int slot = (int)(blockIdx.x % (unsigned)slots);
  const bool gram_cta = (slot == n_tile_ctas);
  const int ch = (int)(blockIdx.x / (unsigned)slots);  // (batch * n + chunk) * nh + head
  const int head = ch % p.nh;
  const int chunk = (ch / p.nh) % p.n_chunks;
  const int batch = ch / (p.nh * p.n_chunks);
  const int kblocks = p.cp / TOK;
  const int total = kblocks * p.group;

  if (tid == 0) {
    abort_flag = 0;
    for (int s = 0; s < NS; ++s) {
      mbar_init(&x_full[s], 1);
      mbar_init(&x_empty[s], 4 * NG);  // every expansion warp
      mbar_init(&w_full[s], 1);
      mbar_init(&w_empty[s], 1);  // Gram CTA only
    }
    for (int g = 0; g < NG; ++g)
      for (int s = 0; s < NSA; ++s) {
        mbar_init(&a_full[g][s], 4 * NG);  // every expansion warp fills its half of each tile's stage
      }
    for (int g = 0; g < NG; ++g)
      for (int s = 0; s < NS; ++s) mbar_init(&done[g][s], 1);
    mbar_init(&acc_done, gram_cta ? 1 : NG);
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

  if (warp == 4 * NG) {
    // ------------------------------------------------------------ TMA producer
    if (lane == 0) {
      for (int it = 0; it < total; ++it) {
        const int s = it % NS, ph = (it / NS) & 1;
        const int g = it / kblocks, kb = it % kblocks;
        const int xhead = head * p.group + g;
        const int xrow = ((batch * p.n_chunks + chunk) * (p.nh * p.group) + xhead) * HD;
        if (!gram_cta && !mbar_wait(&x_empty[s], ph ^ 1, &abort_flag)) break;
        if (gram_cta) {
          // two stages only: the padded A operand is twice the size of a value stage
          const int gs = it & 1, gph = (it >> 1) & 1;
          if (!mbar_wait(&w_empty[gs], gph ^ 1, &abort_flag)) break;
          mbar_expect_tx(&w_full[gs], 2 * XT_BYTES);
          tma_load_2d(smX + gs * XT_BYTES, &tm_xt, &w_full[gs], kb * TOK, xrow);
          tma_load_2d(smG + gs * GA_BYTES, &tm_xs, &w_full[gs], kb * TOK, xrow);
        } else {
          mbar_expect_tx(&x_full[s], XT_BYTES);
          tma_load_2d(smX + s * XT_BYTES, &tm_xt, &x_full[s], kb * TOK, xrow);
          if (it >= NS && !(mbar_wait(&done[0][s], ph ^ 1, &abort_flag) && mbar_wait(&done[1][s], ph ^ 1, &abort_flag)))
            break;
          mbar_expect_tx(&w_full[s], W_BYTES);
          tma_load_4d(smW + s * W_BYTES, &tm_w, &w_full[s], 0, xhead, chunk * p.c + kb * TOK, batch);
        }
      }
    }
  } else if (warp >= 4 * NG + 1) {
    // ------------------------------------------------------------- MMA issuers
    // One issuing thread per group: a single thread needs some 60-80 clocks per tcgen05.mma it
    // issues and as many per commit or barrier wait, which made one thread serving both groups
    // the slowest stage of the pipeline.
    const int g = warp - (4 * NG + 1);
    if (lane == 0 && (!gram_cta || g == 0)) {
      bool ok = true;
      if (gram_cta) {
        const uint32_t idesc = umma_idesc(128, HD, Pack2<T>::is_bf16, false, false);
        for (int it = 0; it < total && ok; ++it) {
          const int gs = it & 1, gph = (it >> 1) & 1;
          ok = mbar_wait(&w_full[gs], gph, &abort_flag);
          if (!ok) break;
          tc_fence_after();
          const uint32_t a_addr = smem_u32(smG + gs * GA_BYTES), b_addr = smem_u32(smX + gs * XT_BYTES);
#pragma unroll
          for (int ks = 0; ks < TOK / 16; ++ks)
            umma_ss(tmem + COL_ACC, umma_desc_sw128(a_addr + ks * 32, 16, 1024),
                    umma_desc_sw128(b_addr + ks * 32, 16, 1024), idesc, (it > 0 || ks > 0) ? 1u : 0u);
          umma_commit(&w_empty[gs]);
        }
      } else {
        const uint32_t idesc = umma_idesc(128, HD, Pack2<T>::is_bf16, false, true);
        for (int it = 0; it < total && ok; ++it) {
          const int s = it % NS, ph = (it / NS) & 1;
          const int sa = it % NSA, pha = (it / NSA) & 1;
          ok = mbar_wait(&w_full[s], ph, &abort_flag) && mbar_wait(&a_full[g][sa], pha, &abort_flag);
          if (!ok) break;
          tc_fence_after();
          const uint32_t b_addr = smem_u32(smW + s * W_BYTES);
#pragma unroll
          for (int ks = 0; ks < TOK / 16; ++ks)
            umma_ts(tmem + COL_ACC + g * 64, tmem + COL_A + (g * NSA + sa) * 32 + ks * 8,
                    umma_desc_sw128(b_addr + ks * 2048, 8192, 1024), idesc, (it > 0 || ks > 0) ? 1u : 0u);
          umma_commit(&done[g][s]);
        }
      }
      if (ok) umma_commit(&acc_done);
    }
  } else {
    // ------------------------------------------------- expansion + epilogue warps
    const int grp = warp >> 2;
    const int row_in_tile = (warp & 3) * 32 + lane;
    const uint32_t lane_addr = (uint32_t)((warp & 3) * 32) << 16;
    const int D2 = ref_dim(HD);
    // expansion: this thread's row of both tiles (first factors a0 and a0 + 8, common second factor b),
    // tokens [32 grp, 32 grp + 32) of every stage; epilogue: its row of tile `grp`
    const int drow0 = slot * NG * 128 + row_in_tile;
    int a0 = 0, b = 0;
    if (!gram_cta && drow0 < D2) ref_decode(drow0, &a0, &b);
    const int a1 = min(a0 + 8, HD - 1);  // the second tile of a pair lies in the same block of second factors
    const int tile = slot * NG + grp;
    const int drow = tile * 128 + row_in_tile;
    const bool valid = !gram_cta && drow < D2;  // rows past the end still take part in the pipeline
    const int a = grp ? a1 : a0;
    bool ok = true;
    // swz128(row, j) = (row * 128 + ((row & 7) << 4)) ^ (j << 4): one XOR per address
    const uint32_t a0_base = a0 * 128 + ((a0 & 7) << 4), a1_base = a1 * 128 + ((a1 & 7) << 4),
                   b_base = b * 128 + ((b & 7) << 4);
    if (!gram_cta) {
      for (int it = 0; it < total; ++it) {
        const int s = it % NS, ph = (it / NS) & 1;
        ok = mbar_wait(&x_full[s], ph, &abort_flag);
        if (!ok) break;
        const uint8_t* xs = smX + s * XT_BYTES;
        uint32_t r0[16], r1[16];
#pragma unroll
        for (int jj = 0; jj < 4; ++jj) {
          const uint32_t off = (uint32_t)((4 * grp + jj) << 4);
          const uint4 vb = *reinterpret_cast<const uint4*>(xs + (b_base ^ off));
          const uint4 va = *reinterpret_cast<const uint4*>(xs + (a0_base ^ off));
          const uint4 vc = *reinterpret_cast<const uint4*>(xs + (a1_base ^ off));
          r0[4 * jj + 0] = Pack2<T>::mul(va.x, vb.x);
          r0[4 * jj + 1] = Pack2<T>::mul(va.y, vb.y);
          r0[4 * jj + 2] = Pack2<T>::mul(va.z, vb.z);
          r0[4 * jj + 3] = Pack2<T>::mul(va.w, vb.w);
          r1[4 * jj + 0] = Pack2<T>::mul(vc.x, vb.x);
          r1[4 * jj + 1] = Pack2<T>::mul(vc.y, vb.y);
          r1[4 * jj + 2] = Pack2<T>::mul(vc.z, vb.z);
          r1[4 * jj + 3] = Pack2<T>::mul(vc.w, vb.w);
        }
        const int sa = it % NSA;
        if (it >= NSA) {
          // both tiles' products of stage it - NSA have read this tensor-memory slot
          const int sp = (it - NSA) % NS, php = ((it - NSA) / NS) & 1;
          ok = mbar_wait(&done[0][sp], php, &abort_flag) && mbar_wait(&done[1][sp], php, &abort_flag);
          if (!ok) break;
        }
        tc_fence_after();
        tmem_st16(tmem + lane_addr + COL_A + (0 * NSA + sa) * 32 + 16 * grp, r0);
        tmem_st16(tmem + lane_addr + COL_A + (1 * NSA + sa) * 32 + 16 * grp, r1);
        // The shared-memory stage goes back to TMA only here: the stores above have consumed every
        // product, so every load of the stage has delivered its data.  Released right after the
        // loads were issued (a plain arrive), a refill could overtake loads still queued in this
        // LDS-heavy kernel, and single rows of the state came out built from the wrong 64 tokens
        // (seen only with two CTAs per SM at grids of thousands of CTAs).  The proxy fence orders
        // this thread's generic-proxy reads before the async-proxy write that follows the release.
        fence_async_smem();
        __syncwarp();
        if (lane == 0) mbar_arrive(&x_empty[s]);
        tmem_wait_st();
        tc_fence_before();
        __syncwarp();
        if (lane == 0) {
          mbar_arrive(&a_full[0][sa]);
          mbar_arrive(&a_full[1][sa]);
        }
      }
    }
    if (ok) ok = mbar_wait(&acc_done, 0, &abort_flag);
    tc_fence_after();
    if (ok) {
      uint32_t acc[64];
      tmem_ld32(tmem + lane_addr + COL_ACC + grp * 64, acc);
      tmem_ld32(tmem + lane_addr + COL_ACC + grp * 64 + 32, acc + 32);
      tmem_wait_ld();
      if (gram_cta) {
        if (grp == 0 && row_in_tile < HD && p.gram != nullptr) {
          float4* dst = reinterpret_cast<float4*>(p.gram + ((size_t)ch * HD + row_in_tile) * HD);
#pragma unroll
          for (int j = 0; j < 16; ++j)
            dst[j] = make_float4(__uint_as_float(acc[4 * j]), __uint_as_float(acc[4 * j + 1]),
                                 __uint_as_float(acc[4 * j + 2]), __uint_as_float(acc[4 * j + 3]));
        }
      } else if (valid) {
        const float wgt = p.key_weights ? ref_key_weight(a, b) : 1.f;
        T* dst = static_cast<T*>(p.out) + ((size_t)ch * D2 + drow) * HD;
        // four 32-byte stores: a full sector per thread and instruction
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          uint32_t v[8];
#pragma unroll
          for (int k = 0; k < 8; ++k)
            v[k] = Pack2<T>::from_f32(wgt * __uint_as_float(acc[16 * j + 2 * k]), wgt * __uint_as_float(acc[16 * j + 2 * k + 1]));
          asm volatile("st.global.v8.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8};" ::"l"(dst + 16 * j), "r"(v[0]), "r"(v[1]),
                       "r"(v[2]), "r"(v[3]), "r"(v[4]), "r"(v[5]), "r"(v[6]), "r"(v[7])
                       : "memory");
        }
      }
    }
  }
  if (tid == 0 && abort_flag) *p.status = ST_TIMEOUT;
  tc_fence_before();
  __syncthreads();
  if (tid == 0 && abort_flag) *p.status = ST_TIMEOUT;
  if (warp == 0) tmem_dealloc(tmem, cs::TMEM_COLS);
}

template <typename T>
static int launch_chunk_state(const ChunkStateParams& p, int b, const CUtensorMap& tm_xt, const CUtensorMap& tm_xs,
                              const CUtensorMap& tm_w, cudaStream_t stream) {
  using namespace cs;
  const size_t smem = 1024 + NS * (XT_BYTES + W_BYTES);
  static_assert(2 * GA_BYTES <= NS * W_BYTES, "Gram stages must fit in the value ring");
  int device = 0;
  PR_CUDA(cudaGetDevice(&device));  // the entry point has made the caller's device current
  PR_SMEM_ATTR(chunk_state_kernel<T>, smem, device, true);
  const long long ctas = (long long)((p.n_tiles + NG - 1) / NG + (p.gram ? 1 : 0)) * b * p.n_chunks * p.nh;
  PR_REQUIRE(ctas < (1ll << 31), PR_ERR_BAD_ARG, "%lld CTAs exceed the grid limit", ctas);
  dim3 grid((unsigned)ctas);
  chunk_state_kernel<T><<<grid, THREADS, smem, stream>>>(p, tm_xt, tm_xs, tm_w);
  PR_CUDA(cudaGetLastError());
  return PR_OK;
}

}  // namespace pr

extern "C" int pr_chunk_state(int dtype, int b, int t, int nh, int group, int d, int c, const void* xt, const void* xts,
                              const void* v, void* out, float* gram, int key_weights, int device, void* stream) {
  using namespace pr;
  PR_REQUIRE(d == cs::HD, PR_ERR_BAD_ARG, "head dim %d: this build handles d = 64", d);
  PR_REQUIRE(b > 0 && t > 0 && nh > 0 && group > 0 && c > 0 && t % c == 0, PR_ERR_BAD_ARG,
             "bad sizes b=%d t=%d heads=%d group=%d c=%d", b, t, nh, group, c);
  PR_REQUIRE(dtype == PR_BF16 || dtype == PR_FP16, PR_ERR_BAD_ARG, "dtype %d", dtype);
  PR_REQUIRE(xt && v && out && aligned16(xt) && aligned16(v) && aligned16(out), PR_ERR_BAD_ARG,
             "null or misaligned pointer");
  PR_REQUIRE(gram == nullptr || (xts != nullptr && aligned16(xts) && aligned16(gram)), PR_ERR_BAD_ARG,
             "gram requested without a scaled operand");
  PR_CUDA(cudaSetDevice(device));
  ChunkStateParams p;
  p.n_tiles = (ref_dim(d) + 127) / 128;
  p.nh = nh;
  p.group = group;
  p.c = c;
  p.cp = (c + 63) / 64 * 64;
  p.n_chunks = t / c;
  p.key_weights = key_weights;
  p.out = out;
  p.gram = gram;
  int rc = status_word(device, &p.status, nullptr);
  if (rc) return rc;
  const int hx = nh * group;
  CUtensorMap tm_xt, tm_xs, tm_w;
  {
    uint64_t dims[2] = {(uint64_t)p.cp, (uint64_t)b * p.n_chunks * hx * d};
    uint64_t strides[2] = {0, (uint64_t)p.cp * 2};
    uint32_t box[2] = {64, (uint32_t)d};
    rc = make_tmap(&tm_xt, xt, 2, 2, dims, strides, box, true);
    if (rc) return rc;
    rc = make_tmap(&tm_xs, gram ? xts : xt, 2, 2, dims, strides, box, true);
    if (rc) return rc;
  }
  {
    uint64_t dims[4] = {(uint64_t)d, (uint64_t)hx, (uint64_t)t, (uint64_t)b};
    uint64_t strides[4] = {0, (uint64_t)d * 2, (uint64_t)hx * d * 2, (uint64_t)t * hx * d * 2};
    uint32_t box[4] = {64, 1, 64, 1};
    rc = make_tmap(&tm_w, v, 2, 4, dims, strides, box, true);
    if (rc) return rc;
  }
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  return dtype == PR_BF16 ? launch_chunk_state<__nv_bfloat16>(p, b, tm_xt, tm_xs, tm_w, s)
                          : launch_chunk_state<__half>(p, b, tm_xt, tm_xs, tm_w, s);
}
