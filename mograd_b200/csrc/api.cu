// Library identity, thread-local error text and cached device attributes.
#include <atomic>
#include <mutex>

#include "common.cuh"
#include "sm100.cuh"

namespace mgb {

static thread_local char g_err[512] = "";

int fail(int code, const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(g_err, sizeof(g_err), fmt, ap);
  va_end(ap);
  return code;
}

static std::atomic<unsigned long long> g_launches{0};

int check_launch(const char* what) {
  g_launches.fetch_add(1, std::memory_order_relaxed);
  const cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return fail(MGB_ECUDA, "%s: %s", what, cudaGetErrorString(e));
  return MGB_OK;
}

namespace {
constexpr int kMaxDev = 64;
struct DevInfo {
  std::once_flag once;
  int sms = 0;
  int smem_optin = 0;
};
DevInfo g_dev[kMaxDev];

DevInfo& dev_info() {
  int d = 0;
  cudaGetDevice(&d);
  if (d < 0 || d >= kMaxDev) d = 0;
  DevInfo& di = g_dev[d];
  std::call_once(di.once, [&] {
    cudaDeviceGetAttribute(&di.sms, cudaDevAttrMultiProcessorCount, d);
    cudaDeviceGetAttribute(&di.smem_optin, cudaDevAttrMaxSharedMemoryPerBlockOptin, d);
    if (di.sms <= 0) di.sms = 148;
  });
  return di;
}
}  // namespace

int sm_count() { return dev_info().sms; }
int max_smem_optin() { return dev_info().smem_optin; }

// ---------------------------------------------------------------- TMA maps
namespace {
using EncodeTiledFn = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                   const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                   CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
std::once_flag g_encode_once;
EncodeTiledFn g_encode = nullptr;
}  // namespace

static bool encode_tmap(CUtensorMap* out, CUtensorMapDataType dt, const void* base, int rank, const uint64_t* dims,
                        const uint64_t* strides_bytes, const uint32_t* box);

bool encode_tmap_bf16(CUtensorMap* out, const void* base, int rank, const uint64_t* dims,
                      const uint64_t* strides_bytes, const uint32_t* box) {
  return encode_tmap(out, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, base, rank, dims, strides_bytes, box);
}
bool encode_tmap_f32(CUtensorMap* out, const void* base, int rank, const uint64_t* dims,
                     const uint64_t* strides_bytes, const uint32_t* box) {
  return encode_tmap(out, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, base, rank, dims, strides_bytes, box);
}

static bool encode_tmap(CUtensorMap* out, CUtensorMapDataType dt, const void* base, int rank, const uint64_t* dims,
                        const uint64_t* strides_bytes, const uint32_t* box) {
  std::call_once(g_encode_once, [] {
    void* fn = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &q) == cudaSuccess &&
        q == cudaDriverEntryPointSuccess)
      g_encode = reinterpret_cast<EncodeTiledFn>(fn);
  });
  if (!g_encode) {
    fail(MGB_ECUDA, "cuTensorMapEncodeTiled is not available from this driver");
    return false;
  }
  cuuint64_t gdim[5];
  cuuint64_t gstr[4];
  cuuint32_t bx[5], es[5];
  for (int i = 0; i < rank; ++i) {
    gdim[i] = dims[i];
    bx[i] = box[i];
    es[i] = 1;
  }
  for (int i = 0; i + 1 < rank; ++i) gstr[i] = strides_bytes[i];
  const CUresult r = g_encode(out, dt, static_cast<cuuint32_t>(rank),
                              const_cast<void*>(base), gdim, gstr, bx, es, CU_TENSOR_MAP_INTERLEAVE_NONE,
                              CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                              CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) {
    fail(MGB_ECUDA, "cuTensorMapEncodeTiled failed with CUresult %d (rank %d, dims %llu x %llu, box %u x %u)",
         static_cast<int>(r), rank, (unsigned long long)dims[0], (unsigned long long)(rank > 1 ? dims[1] : 1), box[0],
         rank > 1 ? box[1] : 1u);
    return false;
  }
  return true;
}

// ------------------------------------------------------ device status word
__device__ int g_device_status[4];

int* device_status_ptr() {
  struct Slot {
    std::once_flag once;
    int* ptr = nullptr;
  };
  static Slot slots[kMaxDev];
  int d = 0;
  cudaGetDevice(&d);
  if (d < 0 || d >= kMaxDev) d = 0;
  Slot& sl = slots[d];
  std::call_once(sl.once, [&] {  // once per device, with that device current
    void* p = nullptr;
    if (cudaGetSymbolAddress(&p, g_device_status) == cudaSuccess) sl.ptr = static_cast<int*>(p);
  });
  return sl.ptr;
}

// One warp waits, with the given limit, on an mbarrier phase that nothing ever completes; when the wait gives up
// it records code 901 and the elapsed microseconds in the status word and the kernel returns normally.
__global__ void __launch_bounds__(32) wait_expiry_kernel(unsigned long long limit_ns, int* status) {
  __shared__ __align__(8) unsigned long long bar_storage;
  const uint32_t bar = sm100::smem_u32(&bar_storage);
  if (threadIdx.x == 0) {
    sm100::mbar_init(bar, 1);
    sm100::mbar_fence_init();
  }
  __syncwarp();
  if (threadIdx.x == 0) {
    const unsigned long long t0 = sm100::global_ns();
    if (!sm100::mbar_wait_limit(bar, 0, limit_ns)) {
      status[1] = static_cast<int>((sm100::global_ns() - t0) / 1000ull);
      atomicExch(status, 901);
    }
  }
}

}  // namespace mgb

MGB_EXPORT int mograd_b200_device_status_async(int* host_words, void* stream) {
  MGB_REQUIRE(host_words, MGB_EINVAL, "device_status_async: host_words is NULL");
  int* p = mgb::device_status_ptr();
  if (!p) return mgb::fail(MGB_ECUDA, "device_status_async: status word not addressable on this device");
  const cudaError_t e =
      cudaMemcpyAsync(host_words, p, 4 * sizeof(int), cudaMemcpyDeviceToHost, static_cast<cudaStream_t>(stream));
  if (e != cudaSuccess) return mgb::fail(MGB_ECUDA, "device_status_async: %s", cudaGetErrorString(e));
  return MGB_OK;
}

MGB_EXPORT int mograd_b200_selftest_wait_expiry(unsigned int limit_us, void* stream) {
  MGB_REQUIRE(limit_us >= 1 && limit_us <= 100000, MGB_EINVAL, "selftest_wait_expiry: limit_us=%u outside 1..100000",
              limit_us);
  int* st = mgb::device_status_ptr();
  if (!st) return mgb::fail(MGB_ECUDA, "selftest_wait_expiry: status word not addressable on this device");
  mgb::wait_expiry_kernel<<<1, 32, 0, static_cast<cudaStream_t>(stream)>>>(1000ull * limit_us, st);
  return mgb::check_launch("wait_expiry_kernel");
}

MGB_EXPORT int mograd_b200_abi_version(void) { return MOGRAD_B200_ABI_VERSION; }
MGB_EXPORT unsigned long long mograd_b200_launch_count(void) { return mgb::g_launches.load(std::memory_order_relaxed); }
MGB_EXPORT const char* mograd_b200_last_error(void) { return mgb::g_err; }

MGB_EXPORT int mograd_b200_device_status(int* code, int* detail) {
  int* p = mgb::device_status_ptr();
  if (!p) return mgb::fail(MGB_ECUDA, "device_status: status word not addressable on this device");
  int host[4] = {0, 0, 0, 0};
  cudaError_t e = cudaMemcpy(host, p, sizeof(host), cudaMemcpyDeviceToHost);
  if (e != cudaSuccess) return mgb::fail(MGB_ECUDA, "device_status: %s", cudaGetErrorString(e));
  if (code) *code = host[0];
  if (detail) *detail = host[1];
  if (host[0] != 0) {
    e = cudaMemset(p, 0, sizeof(host));
    if (e != cudaSuccess) return mgb::fail(MGB_ECUDA, "device_status reset: %s", cudaGetErrorString(e));
  }
  return MGB_OK;
}
