// Whole-operator entry points: the chunked forward and backward of power retention
// (retention/power_retention_maker.py:96-197 and what autograd executes for it) as ONE call
// each.  The launch sequence that the Python wrapper otherwise drives kernel by kernel lives
// here in native code, so a host in any language runs the operator through three symbols
// (pr_workspace_bytes, pr_retention_fwd, pr_retention_bwd) and a Python host pays one ctypes
// call per pass instead of six / eleven.
//
// Memory: the caller allocates everything.  `saved` is what the backward needs from the
// forward (gate sums, row sums, scanned states and Gram matrices); `scratch` is dead when the
// call returns its work to the stream and may be reused by the next call on the same stream.
#include <mutex>

#include "host.cuh"
#include "layout.cuh"

namespace pr {
namespace {

constexpr size_t kAlign = 256;
inline size_t up(size_t x) { return (x + kAlign - 1) / kAlign * kAlign; }

struct Sizes {
  int n, cp, DR, esz;
  size_t a, A, l, Z, zh, zfull;             // saved
  size_t KT, gram;                          // forward scratch
  size_t dy, dl, QT, dZ, dZg, partS, partG, gh, dqs, gq, dks, wk, daq, dak;  // backward scratch
  int blocksS, blocksG;
};

int sizes_of(const pr_problem* p, Sizes* s) {
  PR_REQUIRE(p != nullptr, PR_ERR_BAD_ARG, "problem is null");
  PR_REQUIRE(p->d == 64, PR_ERR_BAD_ARG, "head dim %d: this build handles d = 64", p->d);
  PR_REQUIRE(p->dtype == PR_BF16 || p->dtype == PR_FP16, PR_ERR_BAD_ARG, "dtype %d", p->dtype);
  PR_REQUIRE(p->b > 0 && p->t > 0 && p->h > 0 && p->hq > 0 && p->hq % p->h == 0 && p->c > 0 && p->t % p->c == 0,
             PR_ERR_BAD_ARG, "bad sizes b=%d t=%d h=%d hq=%d c=%d", p->b, p->t, p->h, p->hq, p->c);
  const size_t b = p->b, t = p->t, h = p->h, hq = p->hq, d = p->d;
  s->n = p->t / p->c;
  s->cp = (p->c + 63) / 64 * 64;
  s->DR = ref_dim(p->d);
  s->esz = 2;
  const size_t n = s->n, DR = s->DR, cp = s->cp;
  s->a = up(b * t * h * 4);
  s->A = up(b * n * h * 4);
  s->l = up(b * t * hq * 4);
  s->Z = up(b * n * h * DR * d * 2);
  s->zh = up(b * n * h * d * d * 2);
  s->zfull = up(b * n * h * d * d * 4);
  s->KT = up(b * n * h * d * cp * 2);
  s->gram = up(b * n * h * d * d * 4);
  s->dy = up(b * t * hq * d * 2);
  s->dl = up(b * t * hq * 4);
  s->QT = up(b * n * hq * d * cp * 2);
  s->dZ = s->Z;
  s->dZg = s->gram;
  s->blocksS = pr_discumsum_bwd_blocks((long long)DR * d);
  s->blocksG = pr_gram_scan_bwd_blocks(p->d);
  s->partS = up(b * h * s->blocksS * n * 4);
  s->partG = up(b * h * s->blocksG * n * 4);
  s->gh = s->zh;
  s->dqs = up(b * t * hq * d * 4);
  s->gq = up(b * t * hq * 4);
  s->dks = up(b * t * h * d * 4);
  s->wk = up(b * t * h * 4);
  s->daq = up(b * t * hq * 4);
  s->dak = up(b * t * h * 4);
  return PR_OK;
}

struct Carver {
  uint8_t* p;
  template <typename T>
  T* take(size_t bytes) {
    T* r = reinterpret_cast<T*>(p);
    p += bytes;
    return r;
  }
};

struct Saved {
  float *a, *A, *l, *zfull;
  void *Z, *zhi, *zlo;
};
Saved carve_saved(void* base, const Sizes& s) {
  Carver c{static_cast<uint8_t*>(base)};
  Saved v;
  v.a = c.take<float>(s.a);
  v.A = c.take<float>(s.A);
  v.l = c.take<float>(s.l);
  v.Z = c.take<void>(s.Z);
  v.zhi = c.take<void>(s.zh);
  v.zlo = c.take<void>(s.zh);
  v.zfull = c.take<float>(s.zfull);
  return v;
}

// The backward has two independent branches after dout_prep: the query side (expand_grad on the
// saved states, then chunk_dq) needs nothing from the reverse scan, which heads the key side
// (gate_prep, chunk_state, scan, expand_grad, chunk_dkv).  The query side is enqueued on a second
// stream, forked from and joined back into the caller's stream with events, so that its CTAs fill
// the partial last wave of each key-side launch (and vice versa).  One stream and event pair per
// device, created on first use (outside any stream capture: a capture of the caller's stream
// then records the fork and the join like any cross-stream dependency); `mu` is held while a
// backward is being enqueued, so concurrent callers take turns at using the pair.
struct SideStream {
  std::mutex mu;
  cudaStream_t stream = nullptr;
  cudaEvent_t fork = nullptr, join = nullptr;
};
constexpr int kMaxDevices = 64;
SideStream g_side[kMaxDevices];

bool overlap_enabled() {
  static const bool on = [] {
    const char* e = getenv("PR_BWD_OVERLAP");
    return !(e && e[0] == '0');
  }();
  return on;
}

// with s->mu held
int side_stream_ready(SideStream* s) {
  if (s->stream != nullptr) return PR_OK;
  PR_CUDA(cudaStreamCreateWithFlags(&s->stream, cudaStreamNonBlocking));
  PR_CUDA(cudaEventCreateWithFlags(&s->fork, cudaEventDisableTiming));
  PR_CUDA(cudaEventCreateWithFlags(&s->join, cudaEventDisableTiming));
  return PR_OK;
}

}  // namespace
}  // namespace pr

// The chunk size to run a request with.  The operator's result does not depend on the chunk size, its speed
// does: every chunk's state is written, scanned and read again (1.3 GB per pass at chunk 128 against 0.17 GB at
// 1024 for b1 t65536 h8), and above 1024 the intra-chunk attention grows.  Below 1024: the largest multiple of the
// request up to 1024 that pads the sequence by at most 1/16 more than the request would; above: the largest divisor
// of the request in [256, 1024]; 0 (no chunking) on more than 2048 tokens: 1024 or 512 if that pads by at most
// 1/16, else 0.  Mirrors retention.py: effective_chunk, for hosts that do not go through the Python API.
extern "C" int pr_fast_chunk(long long t, int requested) {
  const int fast = 1024;
  if (t <= 0 || requested < 0) return requested;
  auto padded_to = [t](long long c) { return (t + c - 1) / c * c; };
  if (requested == 0) {
    if (t <= 2 * fast) return 0;
    for (int ce : {fast, fast / 2})
      if (padded_to(ce) <= t + t / 16) return ce;
    return 0;
  }
  if (requested > fast) {
    for (int ce = fast; ce >= 256; --ce)
      if (requested % ce == 0) return ce;
    return requested;
  }
  if (requested == fast) return requested;
  const long long padded = padded_to(requested);
  for (int m = fast / requested; m > 1; --m) {
    const long long ce = (long long)m * requested;
    if (padded_to(ce) <= padded + padded / 16) return (int)ce;
  }
  return requested;
}

extern "C" int pr_workspace_bytes(const pr_problem* prob, int what, size_t* out) {
  using namespace pr;
  PR_REQUIRE(out != nullptr, PR_ERR_BAD_ARG, "out is null");
  Sizes s;
  int rc = sizes_of(prob, &s);
  if (rc) return rc;
  switch (what) {
    case PR_WS_SAVED:
      *out = s.a + s.A + s.l + s.Z + 2 * s.zh + s.zfull;
      break;
    case PR_WS_FWD_SCRATCH:
      *out = s.KT + s.gram;
      break;
    case PR_WS_BWD_SCRATCH:
      *out = s.dy + s.dl + 2 * s.QT + s.dZ + s.dZg + s.partS + s.partG + 2 * s.gh + s.dqs + s.gq + s.dks + s.wk +
             s.daq + s.dak;
      break;
    default:
      return fail(PR_ERR_BAD_ARG, "workspace kind %d", what);
  }
  return PR_OK;
}

extern "C" int pr_retention_fwd(const pr_problem* prob, const void* Q, const void* K, const void* V,
                                const float* log_G, const float* carry_state, const float* carry_gram, void* O,
                                void* saved, void* scratch, float* final_state, float* final_gram, int device,
                                void* stream) {
  using namespace pr;
  Sizes s;
  int rc = sizes_of(prob, &s);
  if (rc) return rc;
  PR_REQUIRE(Q && K && V && O && saved && scratch, PR_ERR_BAD_ARG, "null pointer");
  PR_REQUIRE(aligned16(saved) && aligned16(scratch), PR_ERR_BAD_ARG, "workspaces must be 16-byte aligned");
  PR_REQUIRE((carry_state == nullptr) == (carry_gram == nullptr), PR_ERR_BAD_ARG, "the two carries come together");
  PR_REQUIRE((final_state == nullptr) == (final_gram == nullptr), PR_ERR_BAD_ARG, "the two final carries come together");
  const pr_problem& p = *prob;
  const bool gated = log_G != nullptr;
  Saved sv = carve_saved(saved, s);
  Carver c{static_cast<uint8_t*>(scratch)};
  void* KT = c.take<void>(s.KT);
  float* gram = c.take<float>(s.gram);
  const long long E = (long long)s.DR * p.d;
  // gate sums, discounted transposed keys
  if ((rc = pr_gate_prep(p.dtype, p.b, p.t, p.h, p.h, p.d, p.c, log_G, K, gated ? sv.a : nullptr, sv.A, KT, nullptr,
                         nullptr, 0, 1.f, 1, device, stream)))
    return rc;
  // chunk states and Gram matrices, then their scans (in place: Z[m] = state entering chunk m)
  if ((rc = pr_chunk_state(p.dtype, p.b, p.t, p.h, 1, p.d, p.c, KT, KT, V, sv.Z, gram, 1, device, stream))) return rc;
  if ((rc = pr_state_scan_fwd(p.dtype, p.b, s.n, p.h, p.d, E, sv.Z, sv.A, carry_state, final_state, gram, sv.zhi,
                              sv.zlo, sv.zfull, carry_gram, final_gram, device, stream)))
    return rc;
  // attention + state read-out + normalisation
  return pr_chunk_out(p.dtype, p.b, s.n, p.c, p.c, p.hq, p.h, p.d, Q, K, V, gated ? sv.a : nullptr, sv.Z, sv.zhi,
                      sv.zlo, carry_state ? 0 : 1, 0, 1, p.scale, 2, O, sv.l, device, stream);
}

extern "C" int pr_retention_bwd(const pr_problem* prob, const void* Q, const void* K, const void* V,
                                const float* log_G, const void* O, const void* dO, int had_carry, void* saved,
                                void* scratch, void* dQ, void* dK, void* dV, float* dlog_G, int device, void* stream) {
  using namespace pr;
  Sizes s;
  int rc = sizes_of(prob, &s);
  if (rc) return rc;
  PR_REQUIRE(Q && K && V && O && dO && saved && scratch && dQ && dK && dV, PR_ERR_BAD_ARG, "null pointer");
  PR_REQUIRE(aligned16(saved) && aligned16(scratch), PR_ERR_BAD_ARG, "workspaces must be 16-byte aligned");
  const pr_problem& p = *prob;
  const bool gated = log_G != nullptr;
  PR_REQUIRE(!gated || dlog_G != nullptr, PR_ERR_BAD_ARG, "gated problem without a dlog_G output");
  Saved sv = carve_saved(saved, s);
  Carver c{static_cast<uint8_t*>(scratch)};
  void* dy = c.take<void>(s.dy);
  float* dl = c.take<float>(s.dl);
  void* QT = c.take<void>(s.QT);
  void* QTs = c.take<void>(s.QT);
  void* dZ = c.take<void>(s.dZ);
  float* dZg = c.take<float>(s.dZg);
  float* partS = c.take<float>(s.partS);
  float* partG = c.take<float>(s.partG);
  void* ghi = c.take<void>(s.gh);
  void* glo = c.take<void>(s.gh);
  float* dqs = c.take<float>(s.dqs);
  float* gq = c.take<float>(s.gq);
  float* dks = c.take<float>(s.dks);
  float* wk = c.take<float>(s.wk);
  float* daq = c.take<float>(s.daq);
  float* dak = c.take<float>(s.dak);
  const long long E = (long long)s.DR * p.d;
  const float* a = gated ? sv.a : nullptr;
  const float* A = gated ? sv.A : nullptr;
  const int group = p.hq / p.h;
  // dy = dO / l, dl = -<O, dO> / l
  if ((rc = pr_dout_prep(p.dtype, (long long)p.b * p.t * p.hq, p.d, O, dO, sv.l, dy, dl, device, stream))) return rc;

  // ---- query side, on the second stream when there is one: gradient through the read-out's expansion
  // (saved states), then the attention backward merged with it
  PR_REQUIRE(device >= 0 && device < kMaxDevices, PR_ERR_BAD_ARG, "device ordinal %d out of range", device);
  SideStream* side = overlap_enabled() ? &g_side[device] : nullptr;
  std::unique_lock<std::mutex> lock;
  void* qstream = stream;
  if (side != nullptr) {
    lock = std::unique_lock<std::mutex>(side->mu);
    PR_CUDA(cudaSetDevice(device));
    if ((rc = side_stream_ready(side))) return rc;
    PR_CUDA(cudaEventRecord(side->fork, static_cast<cudaStream_t>(stream)));
    PR_CUDA(cudaStreamWaitEvent(side->stream, side->fork, 0));
    qstream = side->stream;
  }
  rc = pr_expand_grad(p.dtype, p.b, p.t, p.h, p.hq, p.d, p.c, dy, Q, sv.Z, sv.zhi, sv.zlo, a, A, dl, 1, p.scale, 2.f,
                      had_carry ? 0 : 1, s.n - 1, dqs, gq, device, qstream);
  if (!rc)
    rc = pr_chunk_dq(p.dtype, p.b, p.t, p.hq, p.h, p.d, p.c, Q, dO, K, V, a, dl, sv.l, dqs, p.scale, 2, dQ, daq, device,
                     qstream);
  if (side != nullptr) {
    // joined even after an error, so that a capture of the caller's stream is left in a closable state
    cudaEventRecord(side->join, side->stream);
  }

  // ---- key side: gradient of the state read-out (dZ_m, dZg_m from the gated queries; the forward's
  // cumulative gates are read, not rescanned), reverse scans (in place: dZ becomes w (.) dS_m), gradient
  // through the chunk states' expansion, attention backward merged with it
  if (!rc)
    rc = pr_gate_prep(p.dtype, p.b, p.t, p.h, p.hq, p.d, p.c, log_G, Q, gated ? sv.a : nullptr, nullptr, QT, dl, QTs, 1,
                      p.scale, 0, device, stream);
  if (!rc) rc = pr_chunk_state(p.dtype, p.b, p.t, p.h, group, p.d, p.c, QT, QTs, dy, dZ, dZg, 0, device, stream);
  if (!rc)
    rc = pr_state_scan_bwd(p.dtype, p.b, s.n, p.h, p.d, E, dZ, sv.Z, sv.A, nullptr, nullptr, partS, dZg, sv.zfull, ghi,
                           glo, nullptr, nullptr, partG, device, stream);
  if (!rc)
    rc = pr_expand_grad(p.dtype, p.b, p.t, p.h, p.h, p.d, p.c, V, K, dZ, ghi, glo, a, A, nullptr, 0, 1.f, 1.f, 0,
                        s.n - 2, dks, wk, device, stream);
  if (!rc)
    rc = pr_chunk_dkv(p.dtype, p.b, p.t, p.hq, p.h, p.d, p.c, Q, dO, K, V, dZ, a, A, dl, sv.l, dks, s.n - 2, p.scale, 2,
                      dK, dV, dak, device, stream);
  if (side != nullptr) {
    cudaError_t e = cudaStreamWaitEvent(static_cast<cudaStream_t>(stream), side->join, 0);
    if (!rc && e != cudaSuccess) rc = fail(PR_ERR_CUDA, "joining the second stream failed: %s", cudaGetErrorString(e));
    lock.unlock();
  }
  if (rc) return rc;
  if (gated)
    return pr_gate_grad(p.b, p.t, p.h, p.hq, p.c, daq, gq, dak, wk, partS, s.blocksS, partG, s.blocksG, dlog_G, device,
                        stream);
  return PR_OK;
}
