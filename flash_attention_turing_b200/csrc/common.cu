// Host-side helpers: thread-local error text, TMA descriptor encoding through the driver entry
// point (no link-time dependency on libcuda), device capability check, device status word.
#include "common.h"
#define FA_WAIT_INLINE
#include "ptx.cuh"

#include <cudaTypedefs.h>

#include <mutex>

namespace fa {

namespace {
thread_local std::string g_last_error;

// One status word per device; kernels receive its address as a parameter.
__device__ int g_device_status;

__device__ int g_sched_slots[2 * kSchedSlots];

constexpr int kMaxDevices = 64;
int* g_status_ptr[kMaxDevices] = {};
int* g_sched_ptr[kMaxDevices] = {};
unsigned g_sched_next[kMaxDevices] = {};
int g_sm_count[kMaxDevices] = {};
int g_sm100_ok[kMaxDevices] = {};  // 0 unknown, 1 yes, -1 no
std::mutex g_mutex;

PFN_cuTensorMapEncodeTiled_v12000 get_encode_fn() {
  static PFN_cuTensorMapEncodeTiled_v12000 fn = []() -> PFN_cuTensorMapEncodeTiled_v12000 {
    void* ptr = nullptr;
    cudaDriverEntryPointQueryResult qres;
    cudaError_t err =
        cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &qres);
    if (err != cudaSuccess || qres != cudaDriverEntryPointSuccess) return nullptr;
    return reinterpret_cast<PFN_cuTensorMapEncodeTiled_v12000>(ptr);
  }();
  return fn;
}
}  // namespace

int set_error(int code, const std::string& msg) {
  g_last_error = msg;
  return code;
}

const std::string& last_error() { return g_last_error; }

int make_tensor_map_4d(CUtensorMap* map, const void* base, int d, int64_t heads, int64_t rows,
                       int64_t batch, int64_t head_stride, int64_t row_stride, int64_t batch_stride,
                       int box_rows, const char* what) {
  auto encode = get_encode_fn();
  if (!encode) return set_error(FA_ERR_CUDA, "cuTensorMapEncodeTiled entry point not available");
  if (!aligned16(base))
    return set_error(FA_ERR_INVALID_ARGUMENT, std::string(what) + ": base pointer must be 16-byte aligned");
  if (heads < 1 || rows < 1 || batch < 1)
    return set_error(FA_ERR_INVALID_ARGUMENT, std::string(what) + ": empty tensor");
  // A dimension of extent 1 never contributes to an address; give it any legal stride.
  if (heads == 1) head_stride = d;
  if (batch == 1) batch_stride = row_stride * rows > 0 ? row_stride * rows : d;
  if (rows == 1 && (row_stride % 8) != 0) row_stride = d;
  if ((head_stride % 8) || (row_stride % 8) || (batch_stride % 8))
    return set_error(FA_ERR_INVALID_ARGUMENT,
                     std::string(what) + ": strides must be multiples of 8 elements (16 bytes)");
  if (head_stride <= 0 || row_stride <= 0 || batch_stride <= 0)
    return set_error(FA_ERR_INVALID_ARGUMENT, std::string(what) + ": strides must be positive");
  cuuint64_t gdim[4] = {static_cast<cuuint64_t>(d), static_cast<cuuint64_t>(heads),
                        static_cast<cuuint64_t>(rows), static_cast<cuuint64_t>(batch)};
  cuuint64_t gstr[3] = {static_cast<cuuint64_t>(head_stride) * 2,
                        static_cast<cuuint64_t>(row_stride) * 2,
                        static_cast<cuuint64_t>(batch_stride) * 2};
  cuuint32_t box[4] = {64, 1, static_cast<cuuint32_t>(box_rows), 1};
  cuuint32_t estr[4] = {1, 1, 1, 1};
  CUresult res = encode(map, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 4, const_cast<void*>(base), gdim, gstr,
                        box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                        CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (res != CUDA_SUCCESS)
    return set_error(FA_ERR_CUDA, std::string(what) + ": cuTensorMapEncodeTiled failed with code " +
                                      std::to_string(static_cast<int>(res)));
  return FA_OK;
}

int check_device_sm100() {
  int dev = 0;
  FA_CHECK_CUDA(cudaGetDevice(&dev));
  if (dev < 0 || dev >= kMaxDevices) return set_error(FA_ERR_UNSUPPORTED, "device index out of range");
  std::lock_guard<std::mutex> lock(g_mutex);
  if (g_sm100_ok[dev] == 0) {
    int major = 0, minor = 0;
    FA_CHECK_CUDA(cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, dev));
    FA_CHECK_CUDA(cudaDeviceGetAttribute(&minor, cudaDevAttrComputeCapabilityMinor, dev));
    g_sm100_ok[dev] = (major == 10 && minor == 0) ? 1 : -1;
  }
  if (g_sm100_ok[dev] != 1)
    return set_error(FA_ERR_UNSUPPORTED, "this library contains sm_100a kernels only (B200 required)");
  return FA_OK;
}

int* device_status_ptr() {
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) return nullptr;
  std::lock_guard<std::mutex> lock(g_mutex);
  if (!g_status_ptr[dev]) {
    void* p = nullptr;
    if (cudaGetSymbolAddress(&p, g_device_status) != cudaSuccess) return nullptr;
    g_status_ptr[dev] = static_cast<int*>(p);
  }
  return g_status_ptr[dev];
}

int* next_sched_slot() {
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) return nullptr;
  std::lock_guard<std::mutex> lock(g_mutex);
  if (!g_sched_ptr[dev]) {
    void* p = nullptr;
    if (cudaGetSymbolAddress(&p, g_sched_slots) != cudaSuccess) return nullptr;
    g_sched_ptr[dev] = static_cast<int*>(p);
  }
  return g_sched_ptr[dev] + 2 * (g_sched_next[dev]++ % kSchedSlots);
}

int device_sm_count() {
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) return 0;
  std::lock_guard<std::mutex> lock(g_mutex);
  if (g_sm_count[dev] == 0) {
    int n = 0;
    if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess) return 0;
    g_sm_count[dev] = n;
  }
  return g_sm_count[dev];
}

}  // namespace fa

extern "C" {

const char* fa_last_error(void) { return fa::last_error().c_str(); }

int fa_abi_version(void) { return 2; }

int fa_device_status(int reset) {
  int* p = fa::device_status_ptr();
  if (!p) return fa::set_error(FA_ERR_CUDA, "status word not available");
  int value = 0;
  FA_CHECK_CUDA(cudaDeviceSynchronize());
  FA_CHECK_CUDA(cudaMemcpy(&value, p, sizeof(int), cudaMemcpyDeviceToHost));
  if (reset && value != 0) {
    int zero = 0;
    FA_CHECK_CUDA(cudaMemcpy(p, &zero, sizeof(int), cudaMemcpyHostToDevice));
    void* slots = nullptr;  // a launch that gave up leaves its work counters dirty
    FA_CHECK_CUDA(cudaGetSymbolAddress(&slots, fa::g_sched_slots));
    FA_CHECK_CUDA(cudaMemset(slots, 0, sizeof(int) * 2 * fa::kSchedSlots));
  }
  return value;
}

}  // extern "C"

// ---------------------------------------------------------------------------------------------------------
// Self-test of the bounded waits: one tiny CTA waits on a barrier that nobody ever arrives on, with a short
// limit instead of the kernels' 4 s.  The wait gives up, records the time-out in the status word and the
// kernel returns normally -- the same code path a real time-out takes, exercised without a hung launch.
// ---------------------------------------------------------------------------------------------------------
namespace fa {
namespace {
__global__ void wait_timeout_selftest_kernel(int* status, unsigned long long limit_ns) {
  __shared__ uint64_t bar;
  __shared__ int abort_flag;
  if (threadIdx.x == 0) {
    mbar_init(&bar, 1);
    abort_flag = 0;
    fence_mbar_init();
  }
  __syncthreads();
  WaitCtx ctx{&abort_flag, status};
  ctx.tag = 0x7f;  // marks the self-test in the diagnosis bits
  ctx.limit_ns = limit_ns;
  const bool ok = mbar_wait_warp(&bar, 0, ctx);  // never completes: every lane gives up after limit_ns
  if (ok && status) atomicOr(status, 0x40000000);  // cannot happen; would show as a different code
}
}  // namespace
}  // namespace fa

extern "C" int fa_selftest_wait_timeout(uint32_t limit_us, fa_stream_t stream) {
  using namespace fa;
  FA_CHECK_ARG(limit_us >= 1 && limit_us <= 1000000, "fa_selftest_wait_timeout: limit_us must be in [1, 1000000]");
  int rc = check_device_sm100();
  if (rc != FA_OK) return rc;
  int* status = device_status_ptr();
  if (!status) return set_error(FA_ERR_CUDA, "status word not available");
  wait_timeout_selftest_kernel<<<1, 32, 0, static_cast<cudaStream_t>(stream)>>>(status, 1000ull * limit_us);
  FA_CHECK_CUDA(cudaGetLastError());
  return FA_OK;
}
