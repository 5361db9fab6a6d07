/* C ABI of libpr_b200.so: power retention (chunked forward/backward and
 * inference) as hand-written sm_100a kernels.
 *
 * The reference package has no FFI of its own for this path: its native module
 * (`retention_cuda`, imported by retention/_attention/cuda.py:5,
 * retention/_update_state/cuda.py:6, retention/_discumsum/cuda.py:12 and
 * retention/_query_state/cuda.py:10) is absent from its tree.  The entry points below
 * are what a binding for the reference's four-operator plugin interface
 * (retention/power_retention_maker.py:92-104) needs; each one names the reference
 * function it stands in for.
 *
 * Conventions for every entry point
 *   - returns PR_OK (0) or a negative PR_ERR_* code; pr_last_error() gives a
 *     thread-local message for the last failure on the calling thread;
 *   - never aborts, traps or allocates device memory: the caller passes every
 *     input, output and workspace as a raw device pointer (16-byte aligned);
 *   - work is enqueued on the given stream (a cudaStream_t passed as void*) of
 *     the given device ordinal; the call sets that device current itself, so it
 *     may be called from any thread (autograd's backward thread included);
 *   - `dtype` is PR_BF16 or PR_FP16 for Q/K/V-like tensors; gates, row sums and
 *     Gram matrices are fp32;
 *   - tensors are dense and row-major in the stated shape;
 *   - head dim d = 64 in this build; deg = 2.
 *
 * Shapes use b batch, t tokens, h kv heads, hq query heads (multiple of h), d head
 * dim, c chunk length, n = t / c chunks, cp = c rounded up to 64, and
 * D2 = 128*(d/16)*(d/16+1) rows (2560 at d = 64) of the expansion layout the kernels and chunk states
 * use: the reference's own block layout, retention/_update_state/reference.py:5-29 (see layout.cuh).
 * Inference states cross this ABI in the exact layout, d*(d+1)/2 = 2080 rows.
 */
#ifndef PR_B200_H_
#define PR_B200_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define PR_ABI_VERSION 1

enum { PR_BF16 = 0, PR_FP16 = 1 };

enum {
  PR_OK = 0,
  PR_ERR_BAD_ARG = -1,     /* unsupported shape, null or misaligned pointer */
  PR_ERR_CUDA = -2,        /* a CUDA runtime/driver call failed */
  PR_ERR_TIMEOUT = -3,     /* a bounded device-side wait ran out */
  PR_ERR_UNSUPPORTED = -4  /* the device is not sm_100 */
};

int pr_abi_version(void);
const char* pr_last_error(void);

/* Reads (and clears) the status word that kernels of this library write when a
 * bounded device-side wait gives up.  Call after synchronising the stream.
 * *status is 0 when nothing failed. */
int pr_device_status(int device, int* status);

/* The same read as an error code: PR_OK, or PR_ERR_TIMEOUT when a kernel gave up on a bounded
 * wait since the last read (the outputs of that launch are then undefined).  Clears the word. */
int pr_device_check(int device);

/* Strided copy of `rows` rows of `width_bytes` between pinned host memory and device memory
 * (to_device = 1: host -> device), e.g. one slice of heads of a [b,t,h,d] tensor; the host-buffer
 * variant of the public call pipelines such slices.  No counterpart in the reference, whose
 * operators take device tensors only. */
int pr_copy_2d(void* dst, long long dst_pitch, const void* src, long long src_pitch, long long width_bytes,
               long long rows, int to_device, int device, void* stream);

/* Self-test of the tensor-core building blocks on a 128 x N x K product:
 *   variant 0: A, B K-major in shared memory (manual swizzled stores)
 *   variant 1: A K-major, B MN-major in shared memory
 *   variant 2: A in tensor memory, B MN-major in shared memory
 *   variant 3: as 2, with B brought in by TMA
 *   variant 4: as 0, with A and B brought in by TMA
 * a: [128, k] row-major; b: [n, k] row-major for K-major variants, [k, n]
 * row-major for MN-major variants; out: [128, n] fp32.  k multiple of 64,
 * n in {64, 128, 256} (MN-major variants: n = 64). */
int pr_selftest_umma(int variant, int dtype, int n, int k, const void* a, const void* b, float* out,
                     int device, void* stream);

/* Self-test of the bounded device-side waits: one CTA waits on a barrier that nothing arrives at,
 * with a budget of budget_us microseconds (the kernels of the library use two seconds), gives up,
 * releases its tensor memory and returns.  *gave_up (device int, zeroed by the caller) counts the
 * threads whose wait ran out; afterwards pr_device_status reports 1 and pr_device_check returns
 * PR_ERR_TIMEOUT.  Nothing traps and the context stays usable.  No counterpart in the reference. */
int pr_selftest_timeout(int budget_us, int* gave_up, int device, void* stream);

/* Gate glue of retention/power_retention_maker.py:143-155,183-186 in one pass.
 * log_g [b,t,h] or NULL; x [b,t,hx,d].  Writes (when write_a) a [b,t,h] = inclusive
 * cumulative log gate inside each chunk and A [b,n,h] = chunk totals; xt [b,n,hx,d,cp] =
 * gated, transposed copy of x (keys: x*exp((A-a)/2); queries: x*mult*exp(a/2)), zero
 * padded to cp; xts = xt scaled per token by row_scale [b,t,hx] (or NULL).  With write_a = 0 and a_out given,
 * a_out is an INPUT: the cumulative gates an earlier call wrote, read instead of scanned again. */
int pr_gate_prep(int dtype, int b, int t, int h, int hx, int d, int c, const float* log_g, const void* x,
                 float* a_out, float* A_out, void* xt, const float* row_scale, void* xts, int query_side,
                 float mult, int write_a, int device, void* stream);

/* log_G.cumsum(1) of retention/power_retention_maker.py:129,347 for sequences of any length:
 * a_out [b,t,h] (dense) from log_g whose batch entries are g_bstride floats apart.  Used where one
 * "chunk" is the whole sequence (state-free quadratic branch, long inference caches) and the chunk
 * would not fit pr_gate_prep's shared memory (c > 16384). */
int pr_gate_cumsum(int b, int t, int h, const float* log_g, long long g_bstride, float* a_out, int device,
                   void* stream);

/* update_state (retention/_update_state/reference.py:31-53; the old binding
 * compute_update_states, retention/_update_state/cuda.py:30).
 * xt, xts [b,n,nh*group,d,cp] from pr_gate_prep; v [b,t,nh*group,d].
 * out [b,n,nh,D2,d] = w (.) sum_i phi(x_i) v_i^T summed over the group's heads, with key
 * weights {1,2,0} (key_weights=1) or {1,1,0}; gram [b,n,nh,d,d] fp32 = sum_i xs_i x_i^T
 * (NULL to skip).  The Gram matrix of the discounted keys replaces the reference's
 * sum_of_keys: N[(a,b)] = w(a,b) * gram[a][b]. */
int pr_chunk_state(int dtype, int b, int t, int nh, int group, int d, int c, const void* xt, const void* xts,
                   const void* v, void* out, float* gram, int key_weights, int device, void* stream);

/* discumsum (retention/_discumsum/reference.py:3-15; old binding discumsum,
 * retention/_discumsum/cuda.py:39-41).  X [b,n,h,E] 16-bit, A [b,n,h];
 * Y[0] = carry_in (or 0), Y[m+1] = Y[m]*exp(A[m]) + X[m]; writes Y[0..n_out-1], n_out = n
 * (may alias X) or n+1.  carry_in/out [b,h,E] fp32, optional (sequence-parallel hand-over). */
int pr_discumsum_fwd(int dtype, int b, int n, int n_out, int h, long long E, const void* X, void* Y,
                     const float* A, const float* carry_in, float* carry_out, int device, void* stream);

/* discumsum backward (old binding discumsum_bwd, retention/_discumsum/cuda.py:75; gate
 * index as autograd of the reference gives it).  dY, Y, dX [b,n,h,E]; dX may alias dY.
 * dA_part [b,h,pr_discumsum_bwd_blocks(E),n]: per-warp partial sums of the chunk-gate
 * gradient.  row_weights=1 multiplies dX rows (row_len elements each) by the key
 * weights of the expansion layout. */
int pr_discumsum_bwd_blocks(long long E);
int pr_discumsum_bwd(int dtype, int b, int n, int h, long long E, const void* dY, const void* Y, void* dX,
                     const float* A, const float* carry_in, float* carry_out, float* dA_part, int row_len,
                     int row_weights, int device, void* stream);

/* The same scans for the d x d Gram matrices (fp32 in; hi + lo 16-bit halves out for the
 * tensor cores; `full` fp32 copy optional).  Backward emits the symmetrised gradient. */
int pr_gram_scan_fwd(int dtype, int b, int n, int h, int d, const float* G, void* hi, void* lo, float* full,
                     const float* A, const float* carry_in, float* carry_out, int device, void* stream);
int pr_gram_scan_bwd_blocks(int d);
int pr_gram_scan_bwd(int dtype, int b, int n, int h, int d, const float* dZg, const float* Zg, void* hi, void* lo,
                     const float* A, const float* carry_in, float* carry_out, float* dA_part, int device,
                     void* stream);

/* The two forward scans of a pass (states in place, then Gram matrices) in ONE launch, and the two reverse scans
 * likewise: same arguments and results as pr_discumsum_fwd (n_out = n, Y = X = Z) + pr_gram_scan_fwd, and as
 * pr_discumsum_bwd (dX = dY = dZ, row_len = d, key weights on) + pr_gram_scan_bwd.  The reference scans the
 * states and the sum of keys with two discumsum calls (retention/power_retention_maker.py:167-170). */
int pr_state_scan_fwd(int dtype, int b, int n, int h, int d, long long E, void* Z, const float* A,
                      const float* carry_in, float* carry_out, const float* G, void* g_hi, void* g_lo, float* g_full,
                      const float* g_carry_in, float* g_carry_out, int device, void* stream);
int pr_state_scan_bwd(int dtype, int b, int n, int h, int d, long long E, void* dZ, const void* Z, const float* A,
                      const float* carry_in, float* carry_out, float* dA_part, const float* dZg, const float* Zg,
                      void* g_hi, void* g_lo, const float* g_carry_in, float* g_carry_out, float* g_dA_part, int device,
                      void* stream);

/* attention + query_state fused (retention/_attention/reference.py:10-69 and
 * retention/_query_state/reference.py:36-96; old bindings attention_fwd,
 * retention/_attention/cuda.py:34, and compute_query_states, retention/_query_state/cuda.py:42-44).
 * Q [b,n*cq,hq,d]; K,V [b,n*ck,h,d] or NULL (state only); a [b,n*ck,h] or NULL;
 * Z [b,n,h,D2,d], zg_hi/zg_lo [b,n,h,d,d] or NULL.  Query i of a chunk sits at key
 * position i + ck - cq.  Chunks >= state_from_chunk read the state.  O [b,n*cq,hq,d] =
 * y / l (normalize=1) or y; l_out [b,n*cq,hq] or NULL.  deg = 2, or 4 without a state (the
 * reference's attention takes any even degree, its state operators degree 2 only). */
int pr_chunk_out(int dtype, int b, int n_chunks, int cq, int ck, int hq, int h, int d, const void* Q,
                 const void* K, const void* V, const float* a, const void* Z, const void* zg_hi, const void* zg_lo,
                 int state_from_chunk, int q_gate_last, int normalize, float scale, int deg, void* O, float* l_out,
                 int device, void* stream);

/* Backward prologue: dy = dO / l, dl = -<O, dO> / l over `rows` rows of d elements. */
int pr_dout_prep(int dtype, long long rows, int d, const void* O, const void* dO, const float* l, void* dy,
                 float* dl, int device, void* stream);

/* Gradient through the expansion (query side: retention/_query_state/triton.py:181-325; key
 * side: retention/_update_state/reference.py:55-83; old bindings query_states_bwd,
 * retention/_query_state/cuda.py:86-87, and update_states_bwd, retention/_update_state/cuda.py:64).
 * W, X [b,t,hx,d]; State [b,n,h,D2,d]; g_hi/g_lo [b,n,h,d,d]; a [b,t,h], A [b,n,h] or both
 * NULL; row_g [b,t,hx] or NULL.  dX [b,t,hx,d] fp32 (gradient w.r.t. the ungated x),
 * gdot [b,t,hx] = <x~, dx~>/2.  Chunks outside [chunk_lo, chunk_hi] get zeros. */
int pr_expand_grad(int dtype, int b, int t, int h, int hx, int d, int c, const void* W, const void* X,
                   const void* State, const void* g_hi, const void* g_lo, const float* a, const float* A,
                   const float* row_g, int query_side, float scale, float gram_mult, int chunk_lo, int chunk_hi,
                   float* dX, float* gdot, int device, void* stream);

/* attention backward (retention/_attention/triton.py:390-603; old binding attention_bwd,
 * retention/_attention/cuda.py:75), split by output.  dO [b,t,hq,d] unscaled; l, dl [b,t,hq]
 * from the forward and from pr_dout_prep.
 * pr_chunk_dq : dQ [b,t,hq,d] (+ dq_state fp32 if given), da_q [b,t,hq].
 * pr_chunk_dkv: dK, dV [b,t,h,d] (+ dk_state; + the state path of dV from wdS
 *               [b,n,h,D2,d] for chunks <= state_chunk_hi), da_k [b,t,h].
 * deg = 2, or 4 without state-path terms. */
int pr_chunk_dq(int dtype, int b, int t, int hq, int h, int d, int c, const void* Q, const void* dO, const void* K,
                const void* V, const float* a, const float* dl, const float* l, const float* dq_state, float scale,
                int deg, void* dQ, float* da_q, int device, void* stream);
int pr_chunk_dkv(int dtype, int b, int t, int hq, int h, int d, int c, const void* Q, const void* dO, const void* K,
                 const void* V, const void* wdS, const float* a, const float* A, const float* dl, const float* l,
                 const float* dk_state, int state_chunk_hi, float scale, int deg, void* dK, void* dV, float* da_k,
                 int device, void* stream);

/* Assembles dlog_G [b,t,h] (the autograd of the cumsum / exp glue of
 * retention/power_retention_maker.py:143-186): reverse cumulative sum inside each chunk of
 * the per-token terms plus the chunk-gate gradient.  gq, wk, dA_scan, dA_gram may be NULL. */
int pr_gate_grad(int b, int t, int h, int hq, int c, const float* da_q, const float* gq, const float* da_k,
                 const float* wk, const float* dA_scan, int scan_blocks, const float* dA_gram, int gram_blocks,
                 float* dlog_g, int device, void* stream);

/* Inference (retention/power_retention_maker.py:287-390).  States use the exact layout:
 * state [b,h,D,d] 16-bit, sum_of_keys [b,h,D] fp32, D = d*(d+1)/2, pair (a<=b) at
 * a*d - a*(a-1)/2 + (b-a), weight 2 on a != b.
 *
 * pr_decode_state: one query token per sequence against the state (query_state of the
 * reference, retention/_query_state/reference.py:36-96, for tq = 1): Q [b,1,hq,d];
 * a_last [b,h] = cumulative log gate at the last cached key, or NULL.  Writes partial sums
 * part_y and part_l: workspaces of b*hq*pr_decode_nsplit()*d and b*hq*pr_decode_nsplit() floats.  How many
 * splits a call uses depends on b, h and hq only (one when there are enough (batch, head) pairs to fill the GPU);
 * the contents are a hand-over to pr_decode_finish with the same sizes, not an interface.
 * pr_decode_finish: attention over the tk cached tokens (K,V [b,tk,h,d], a [b,tk,h]; may be
 * absent) + the partials (may be absent) -> O [b,1,hq,d].
 * pr_state_merge: the switch-over of :366-382: new_state = state*exp(a_last) + S, with
 * S [b,1,h,D2,d] and gram [b,1,h,d,d] from pr_chunk_state over the cached tokens; state and
 * sum_of_keys may be NULL (first compression). */
int pr_decode_nsplit(void);
/* Parts the decode step of a given shape is split into, in [1, pr_decode_nsplit()]; 1 means that
 * pr_decode_step / pr_decode_recurrent need no part_y / part_l.  Negative on bad sizes. */
int pr_decode_split(int b, int h, int hq);
int pr_decode_state(int dtype, int b, int h, int hq, int d, const void* Q, const void* state,
                    const float* sum_of_keys, const float* a_last, float scale, float* part_y, float* part_l,
                    int device, void* stream);
/* As pr_decode_state with a_last element (batch, head) at a_last[batch*a_batch_stride + head]. */
int pr_decode_state_strided(int dtype, int b, int h, int hq, int d, const void* Q, const void* state,
                            const float* sum_of_keys, const float* a_last, long long a_batch_stride, float scale,
                            float* part_y, float* part_l, int device, void* stream);
/* One decode step (retention/power_retention_maker.py:287-363 for tq = 1) in one call and one kernel:
 * gate sums of the tk cached tokens, state read-out and attention over the cache, merged and
 * normalised into O [b,1,hq,d].  K/V/log_g and state/sum_of_keys may each be absent.  part_y
 * [b,hq,pr_decode_nsplit(),d] and part_l [b,hq,pr_decode_nsplit()] are needed (and a second, tiny
 * kernel runs) only when b*h*ceil(hq/h/4) < 384, where each (batch, head) pair is split over several
 * CTAs; a_scratch is unused (kept for callers of the earlier three-kernel step) and may be NULL.
 * The state is streamed by TMA into shared memory and contracted with phi(q) by tcgen05.mma (it never
 * passes through registers); state and sum_of_keys must be 16-byte aligned and dense.  The kernel's
 * waits are bounded: pr_device_check() reports PR_ERR_TIMEOUT if one ran out. */
int pr_decode_step(int dtype, int b, int tk, int h, int hq, int d, const void* Q, const void* K, const void* V,
                   const float* log_g, const void* state, const float* sum_of_keys, float scale, float* a_scratch,
                   float* part_y, float* part_l, void* O, int device, void* stream);
/* pr_decode_step for a query and a cache that are slices of longer preallocated tensors (a serving loop's KV and gate
 * cache [b, max_len, h, d] read as [:, :tk]): consecutive batch entries of Q are q_bstride elements apart, of K and V
 * kv_bstride elements (a multiple of 8), of log_g g_bstride floats; inside a batch entry the tensors are dense.  The
 * reference takes such slices as they are (torch indexing); here they need no copy either.  No counterpart of its
 * own in the reference: it is retention/power_retention_maker.py:287-390 for tq = 1 on strided inputs. */
int pr_decode_step_strided(int dtype, int b, int tk, int h, int hq, int d, const void* Q, long long q_bstride,
                           const void* K, const void* V, long long kv_bstride, const float* log_g, long long g_bstride,
                           const void* state, const float* sum_of_keys, float scale, float* a_scratch, float* part_y,
                           float* part_l, void* O, int device, void* stream);
/* ---- The whole operator in one call per pass -------------------------------------------------
 * power_retention's chunked branch (retention/power_retention_maker.py:143-193) and its backward
 * (what autograd runs: retention/_query_state/triton.py:544-621, _attention/triton.py:742-810,
 * _discumsum/triton.py:334-355, _update_state/triton.py:329-355 and the gradients of the glue),
 * sequenced in native code over the entry points above.  t must be a multiple of c (the caller
 * pads, as the reference's wrapper does, :71-90); deg = 2. */
typedef struct pr_problem {
  int dtype;   /* PR_BF16 / PR_FP16 */
  int b, t;    /* batch, tokens */
  int h, hq;   /* kv heads, query heads (multiple of h) */
  int d;       /* head dim (64) */
  int c;       /* chunk length */
  float scale; /* score scale (the reference's default is 1/sqrt(d)) */
} pr_problem;

enum { PR_WS_SAVED = 0, PR_WS_FWD_SCRATCH = 1, PR_WS_BWD_SCRATCH = 2 };

/* Bytes of the three caller-allocated workspaces of a problem: PR_WS_SAVED (written by the forward,
 * read by the backward: gate sums, row sums, scanned states), PR_WS_FWD_SCRATCH and
 * PR_WS_BWD_SCRATCH (dead once the call's work has run; reusable by later calls on the same stream). */
int pr_workspace_bytes(const pr_problem* problem, int what, size_t* out);

/* Forward.  Q [b,t,hq,d]; K, V [b,t,h,d]; log_G [b,t,h] fp32 or NULL; O [b,t,hq,d].
 * carry_state [b,h,D2*d] / carry_gram [b,h,d*d] fp32 or NULL: the state entering the first chunk
 * (initial_state, :158-160; from pr_state_to_chunk_layout).  final_state / final_gram (same
 * shapes) or NULL receive the state after the last chunk (return_final_state, :171-172). */
int pr_retention_fwd(const pr_problem* problem, const void* Q, const void* K, const void* V, const float* log_G,
                     const float* carry_state, const float* carry_gram, void* O, void* saved, void* scratch,
                     float* final_state, float* final_gram, int device, void* stream);

/* The chunk size to run a request with (0 = no chunking asked for): same results, fewer and longer chunks.
 * The chunk size blocks the computation of retention/power_retention_maker.py:143-193 without changing its
 * result; on this hardware 1024 is fastest (5.3 ms per step at chunk 128 against 2.6 at 1024 for b1 t65536 h8).
 * pr_retention_fwd / _bwd run whatever pr_problem.c says; a host that wants the fast blocking passes
 * c = pr_fast_chunk(t, its_chunk) and pads t to a multiple of it with zero tokens behind gates of 1. */
int pr_fast_chunk(long long t, int requested_chunk);

/* Backward.  dO [b,t,hq,d] -> dQ, dK, dV (shapes of Q, K, V) and dlog_G [b,t,h] fp32 (NULL when
 * ungated).  `saved` as the forward left it; had_carry = 1 when the forward was given carries.
 * The query-side branch (expand_grad on the saved states, chunk_dq) runs on a second stream that
 * the library owns (one per device, created at the first call - make that call outside any
 * stream capture), forked from and joined back into `stream` with events, so everything is
 * complete in `stream` order when the call's work is; PR_BWD_OVERLAP=0 in the environment keeps
 * the whole pass on `stream`. */
int pr_retention_bwd(const pr_problem* problem, const void* Q, const void* K, const void* V, const float* log_G,
                     const void* O, const void* dO, int had_carry, void* saved, void* scratch, void* dQ, void* dK,
                     void* dV, float* dlog_G, int device, void* stream);

/* Between the caller's projection GEMM and the operator (deploy/nanoGPT/model.py:66-84,
 * deploy/models/powercoder/modeling_powercoder.py:152-159): one pass over the projection output
 * qkvg [b,t,row_stride] 16-bit, a token's row holding hq*d query, h*d key, h*d value features and,
 * when gated, h gate pre-activations.  Writes Q [b,t,hq,d], K, V [b,t,h,d] (rotary applied to Q
 * and K) and log_g [b,t,h] = logsigmoid(gate_bias + gate) fp32 - the tensors pr_retention_fwd takes.
 * cos_table / sin_table [t, d/2] fp32 (batch entries table_bstride floats apart, 0 = one table);
 * half_split = 0: rotary pairs (2i, 2i+1) as deploy/nanoGPT/model.py:153-164, 1: pairs (i, i+d/2)
 * as modeling_powercoder.py:43-74.  Products and sum are rounded separately in fp32, then once to
 * 16 bits, which reproduces model.py:159-164 bit for bit.  Any d that is a multiple of 8 (16 when
 * half_split).  pr_caller_prep_bwd is its gradient: dQ, dK, dV, dlog_g -> dqkvg (same shape as
 * qkvg, which it reads for the gate's derivative; padding columns of a wider row are left as they are). */
int pr_caller_prep_fwd(int dtype, int b, int t, int h, int hq, int d, const void* qkvg, long long row_stride,
                       const float* cos_table, const float* sin_table, long long table_bstride, int half_split,
                       int gated, float gate_bias, void* Q, void* K, void* V, float* log_g, int device, void* stream);
int pr_caller_prep_bwd(int dtype, int b, int t, int h, int hq, int d, const void* qkvg, long long row_stride,
                       const float* cos_table, const float* sin_table, long long table_bstride, int half_split,
                       int gated, float gate_bias, const void* dQ, const void* dK, const void* dV, const float* dlog_g,
                       void* dqkvg, int device, void* stream);

/* A state in the exact layout (state [b,h,d(d+1)/2,d], sum_of_keys [b,h,d(d+1)/2]) converted to the
 * chunk-state layout of the training kernels: out16 [b,h,D2,d] 16-bit, out32 the same in fp32 (a carry_in
 * for pr_discumsum_fwd), gram [b,h,d,d] fp32 (carry_in for pr_gram_scan_fwd), gram_hi / gram_lo 16-bit
 * halves (for pr_chunk_out); any output may be NULL.  Serves initial_state of
 * retention/power_retention_maker.py:72-73,158-160 and several-token queries against a state (:354-363). */
int pr_state_to_chunk_layout(int dtype, int b, int h, int d, const void* state, const float* sum_of_keys, void* out16,
                             float* out32, float* gram, void* gram_hi, void* gram_lo, int device, void* stream);
/* Pure-recurrent decode step: the state is advanced by one token (k, v [b,1,h,d], log_g [b,1,h] or NULL)
 * and read by q [b,1,hq,d] in one pass over it: the reference's inference step with
 * switch_over_seq_len = 1 (retention/power_retention_maker.py:354-382: one cached token, then
 * compression) and what deploy/models/powercoder/kvgs_dynamic_cache.py:131-172 would hold as a cache
 * of length one.  Batch entries of q / k, v / log_g are q_bstride / kv_bstride / g_bstride elements
 * apart.  new_state, new_sum_of_keys may alias the inputs when hq / h <= 4.  part_y / part_l as for
 * pr_decode_step (needed only for small b*h).  The state moves by TMA in both directions (16-byte aligned,
 * dense); the output reads the stored state as the reference's query_state does and takes the new token
 * exactly, y = e^g (phi(q) . S) + (phi(q) . phi_K(k)) v, not through the 16-bit rounding of the advanced state. */
int pr_decode_recurrent(int dtype, int b, int h, int hq, int d, const void* Q, long long q_bstride, const void* K,
                        const void* V, long long kv_bstride, const float* log_g, long long g_bstride,
                        const void* state, const float* sum_of_keys, void* new_state, float* new_sum_of_keys,
                        float scale, float* part_y, float* part_l, void* O, int device, void* stream);
/* No counterpart in the reference.  pr_decode_step for hosts that cannot hand over scratch
 * memory (a memory pool frozen after start-up, an allocator owned by another component): the
 * partial-sum scratch of a split step sits in a fixed device array of about 1.3 MB that the library
 * carries on every GPU.  Limit: b*hq <= 1024, beyond which PR_ERR_BAD_ARG is returned.  The array is shared by all calls on a device, so calls that overlap on the GPU
 * race; nothing in it needs zeroing between calls.  The first call on a device looks up the
 * array's device address and should be made outside any stream capture. */
int pr_decode_step_static(int dtype, int b, int tk, int h, int hq, int d, const void* Q, const void* K,
                          const void* V, const float* log_g, const void* state, const float* sum_of_keys,
                          float scale, void* O, int device, void* stream);
int pr_decode_finish(int dtype, int b, int tk, int h, int hq, int d, const void* Q, const void* K, const void* V,
                     const float* a, float scale, const float* part_y, const float* part_l, void* O, int device,
                     void* stream);
int pr_state_merge(int dtype, int b, int h, int d, const void* state, const float* sum_of_keys, const void* S,
                   const float* gram, const float* a_last, void* new_state, float* new_sum_of_keys, int device,
                   void* stream);

#ifdef __cplusplus
}
#endif
#endif /* PR_B200_H_ */
