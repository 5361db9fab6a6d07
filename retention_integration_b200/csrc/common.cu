// Host-side plumbing of the C ABI: version, error string, status word, tensor maps.
#include <map>
#include <mutex>
#include <utility>

#include "host.cuh"
#include "sm100.cuh"

namespace pr {

namespace {
constexpr int kMaxDevices = 64;
struct StatusSlot {
  int* host = nullptr;
  int* dev = nullptr;
};
StatusSlot g_status[kMaxDevices];
std::mutex g_status_mu;

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
EncodeTiledFn g_encode = nullptr;
std::once_flag g_encode_once;
}  // namespace

int status_word(int device, int** dev_ptr, volatile int** host_ptr) {
  PR_REQUIRE(device >= 0 && device < kMaxDevices, PR_ERR_BAD_ARG, "device ordinal %d out of range", device);
  std::lock_guard<std::mutex> lock(g_status_mu);
  StatusSlot& s = g_status[device];
  if (!s.host) {
    // Pinned, mapped host memory: 4 bytes per device, kept until the process exits.
    PR_CUDA(cudaSetDevice(device));
    void* h = nullptr;
    PR_CUDA(cudaHostAlloc(&h, 64, cudaHostAllocMapped | cudaHostAllocPortable));
    void* d = nullptr;
    PR_CUDA(cudaHostGetDevicePointer(&d, h, 0));
    *static_cast<volatile int*>(h) = 0;
    s.host = static_cast<int*>(h);
    s.dev = static_cast<int*>(d);
  }
  if (dev_ptr) *dev_ptr = s.dev;
  if (host_ptr) *host_ptr = s.host;
  return PR_OK;
}

int smem_attr(const void* kernel, size_t bytes, int device, bool carveout) {
  static std::mutex mu;
  static std::map<std::pair<const void*, int>, size_t> set_bytes;
  // never below the 48 KB every kernel may use without the attribute
  const size_t want = bytes < 49152 ? 49152 : bytes;
  std::lock_guard<std::mutex> lock(mu);
  size_t& have = set_bytes[{kernel, device}];
  if (have >= want) return PR_OK;
  PR_CUDA(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)want));
  if (carveout) PR_CUDA(cudaFuncSetAttribute(kernel, cudaFuncAttributePreferredSharedMemoryCarveout, 100));
  have = want;
  return PR_OK;
}

bool pdl_enabled() {
  static const bool on = [] {
    const char* e = getenv("PR_PDL");
    return !(e && e[0] == '0');
  }();
  return on;
}

int make_tmap(CUtensorMap* out, const void* base, int elem_bytes, int rank, const uint64_t* dims,
              const uint64_t* strides_bytes, const uint32_t* box, bool swizzle128) {
  std::call_once(g_encode_once, [] {
    void* fn = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &q) == cudaSuccess &&
        q == cudaDriverEntryPointSuccess)
      g_encode = reinterpret_cast<EncodeTiledFn>(fn);
  });
  PR_REQUIRE(g_encode != nullptr, PR_ERR_CUDA, "cuTensorMapEncodeTiled is not available from the driver");
  PR_REQUIRE(rank >= 2 && rank <= 5, PR_ERR_BAD_ARG, "tensor map rank %d", rank);
  PR_REQUIRE(aligned16(base), PR_ERR_BAD_ARG, "tensor map base %p is not 16-byte aligned", base);
  cuuint64_t gdim[5], gstr[4];
  cuuint32_t bdim[5], estr[5];
  for (int i = 0; i < rank; ++i) {
    gdim[i] = dims[i];
    bdim[i] = box[i];
    estr[i] = 1;
    if (i > 0) {
      PR_REQUIRE(strides_bytes[i] % 16 == 0, PR_ERR_BAD_ARG, "tensor map stride %d = %llu bytes, not a multiple of 16",
                 i, (unsigned long long)strides_bytes[i]);
      gstr[i - 1] = strides_bytes[i];
    }
  }
  PR_REQUIRE((uint64_t)box[0] * elem_bytes % 16 == 0, PR_ERR_BAD_ARG, "tensor map inner box is not 16-byte sized");
  if (swizzle128)
    PR_REQUIRE((uint64_t)box[0] * elem_bytes <= 128, PR_ERR_BAD_ARG, "swizzled inner box wider than 128 bytes");
  CUtensorMapDataType dt = elem_bytes == 2   ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16
                           : elem_bytes == 4 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT32
                                             : CU_TENSOR_MAP_DATA_TYPE_UINT8;
  CUresult r = g_encode(out, dt, (cuuint32_t)rank, const_cast<void*>(base), gdim, gstr, bdim, estr,
                        CU_TENSOR_MAP_INTERLEAVE_NONE,
                        swizzle128 ? CU_TENSOR_MAP_SWIZZLE_128B : CU_TENSOR_MAP_SWIZZLE_NONE,
                        CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  PR_REQUIRE(r == CUDA_SUCCESS, PR_ERR_CUDA, "cuTensorMapEncodeTiled failed with CUresult %d", (int)r);
  return PR_OK;
}

}  // namespace pr

extern "C" int pr_abi_version(void) { return PR_ABI_VERSION; }
extern "C" const char* pr_last_error(void) { return pr::err_buf(); }

extern "C" int pr_device_status(int device, int* status) {
  PR_REQUIRE(status != nullptr, PR_ERR_BAD_ARG, "status is null");
  volatile int* h = nullptr;
  int rc = pr::status_word(device, nullptr, &h);
  if (rc != PR_OK) return rc;
  *status = *h;
  *h = 0;
  return PR_OK;
}

// The status word turned into an error code: PR_ERR_TIMEOUT when a kernel gave up on a bounded
// wait since the last read, PR_ERR_BAD_ARG when a kernel refused its arguments.  Clears the word.
extern "C" int pr_device_check(int device) {
  int st = 0;
  int rc = pr_device_status(device, &st);
  if (rc != PR_OK) return rc;
  if (st == pr::ST_TIMEOUT)
    return pr::fail(PR_ERR_TIMEOUT, "a kernel on device %d gave up on a bounded device-side wait", device);
  if (st != pr::ST_OK) return pr::fail(PR_ERR_BAD_ARG, "a kernel on device %d reported status %d", device, st);
  return PR_OK;
}

// Strided host<->device copy of a [rows, width_bytes] window (cudaMemcpy2DAsync): used to move a
// slice of heads of a [b, t, h, d] tensor between pinned host memory and a dense device buffer.
extern "C" int pr_copy_2d(void* dst, long long dst_pitch, const void* src, long long src_pitch,
                          long long width_bytes, long long rows, int to_device, int device, void* stream) {
  using namespace pr;
  PR_REQUIRE(dst && src && width_bytes > 0 && rows > 0 && dst_pitch >= width_bytes && src_pitch >= width_bytes,
             PR_ERR_BAD_ARG, "bad 2-D copy arguments");
  PR_CUDA(cudaSetDevice(device));
  PR_CUDA(cudaMemcpy2DAsync(dst, (size_t)dst_pitch, src, (size_t)src_pitch, (size_t)width_bytes, (size_t)rows,
                            to_device ? cudaMemcpyHostToDevice : cudaMemcpyDeviceToHost,
                            static_cast<cudaStream_t>(stream)));
  return PR_OK;
}
