// Library state: thread-local error message, the per-device kernel status word, device
// queries, TMA tensor-map encoding (through the driver entry point, so the library does not
// link libcuda directly).
#include "host.h"

#include <atomic>
#include <mutex>
#include <vector>

namespace cdl {

std::string& last_error() {
  static thread_local std::string msg;
  return msg;
}

int32_t fail(int32_t code, const char* fmt, ...) {
  char buf[1024];
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(buf, sizeof buf, fmt, ap);
  va_end(ap);
  last_error() = buf;
  return code;
}

// One word per device (each device that loads the module gets its own copy).
__device__ int g_kernel_status = 0;

static constexpr int kMaxDevices = 64;

int* device_status_ptr() {
  static int* ptrs[kMaxDevices] = {};
  static std::mutex mu;
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) return nullptr;
  std::lock_guard<std::mutex> lock(mu);
  if (!ptrs[dev]) {
    void* p = nullptr;
    if (cudaGetSymbolAddress(&p, g_kernel_status) != cudaSuccess) return nullptr;
    ptrs[dev] = static_cast<int*>(p);
  }
  return ptrs[dev];
}

int sm_count() {
  static int counts[kMaxDevices] = {};
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) return 148;
  if (!counts[dev]) {
    int n = 0;
    if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0)
      n = 148;
    counts[dev] = n;
  }
  return counts[dev];
}

// Work counters of the kernels that hand out their work at run time (the CTA-pair GEMM's units,
// kind 0; the persistent attention forward's items, kind 1; the persistent attention backward
// kernels' items, kinds 2 and 3): one per kind, device and stream, zero
// between launches (the kernel's last draw puts its counter back).  Launches on one stream run
// one after the other, so they can share a counter; launches on different streams may overlap and
// must not.  Inside the library's device image: nothing is allocated.  A launch that gets no
// counter (more than SCHED_STREAMS streams on a device) runs with its fixed assignment.
#ifndef CDL_DYNAMIC_WORK
#define CDL_DYNAMIC_WORK 1
#endif
constexpr int SCHED_KINDS = 4;
constexpr int SCHED_STREAMS = 256;
__device__ unsigned int g_sched_counters[SCHED_KINDS * SCHED_STREAMS];

unsigned int* sched_counter_for(int kind, int dev, cudaStream_t stream) {
#if CDL_DYNAMIC_WORK
  static std::mutex mu;
  static unsigned int* base[kMaxDevices] = {};
  static cudaStream_t owner[kMaxDevices][SCHED_STREAMS];
  static int used[kMaxDevices] = {};
  if (dev < 0 || dev >= kMaxDevices || kind < 0 || kind >= SCHED_KINDS) return nullptr;
  std::lock_guard<std::mutex> lock(mu);
  if (base[dev] == nullptr) {
    void* ptr = nullptr;
    if (cudaGetSymbolAddress(&ptr, g_sched_counters) != cudaSuccess) {
      (void)cudaGetLastError();
      return nullptr;
    }
    base[dev] = static_cast<unsigned int*>(ptr);
  }
  int slot = -1;
  for (int i = 0; i < used[dev]; ++i)
    if (owner[dev][i] == stream) slot = i;
  if (slot < 0) {
    if (used[dev] == SCHED_STREAMS) return nullptr;
    slot = used[dev]++;
    owner[dev][slot] = stream;
  }
  return base[dev] + kind * SCHED_STREAMS + slot;
#else
  (void)kind;
  (void)dev;
  (void)stream;
  return nullptr;
#endif
}

using EncodeTiledFn = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*,
                                   const cuuint64_t*, const cuuint64_t*, const cuuint32_t*,
                                   const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                   CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn encode_fn() {
  static EncodeTiledFn fn = [] {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) !=
            cudaSuccess ||
        q != cudaDriverEntryPointSuccess)
      p = nullptr;
    return reinterpret_cast<EncodeTiledFn>(p);
  }();
  return fn;
}

int32_t encode_tmap(CUtensorMap* out, const void* base, int32_t dtype, int rank,
                    const uint64_t* dims, const uint64_t* strides_bytes, const uint32_t* box,
                    bool swizzle128) {
  EncodeTiledFn fn = encode_fn();
  if (!fn) return fail(CDL_ERR_CUDA, "cuTensorMapEncodeTiled is not available from the driver");
  cuuint64_t gdim[5];
  cuuint64_t gstr[5];
  cuuint32_t bx[5];
  cuuint32_t estr[5];
  for (int i = 0; i < rank; ++i) {
    gdim[i] = dims[i];
    bx[i] = box[i];
    estr[i] = 1;
    if (i > 0) gstr[i - 1] = strides_bytes[i];
  }
  CUtensorMapDataType dt = dtype == CDL_BF16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16
                           : dtype == TMAP_U8  ? CU_TENSOR_MAP_DATA_TYPE_UINT8
                                               : CU_TENSOR_MAP_DATA_TYPE_FLOAT32;
  CUresult r = fn(out, dt, static_cast<cuuint32_t>(rank), const_cast<void*>(base), gdim, gstr, bx,
                  estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                  swizzle128 ? CU_TENSOR_MAP_SWIZZLE_128B : CU_TENSOR_MAP_SWIZZLE_NONE,
                  CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS)
    return fail(CDL_ERR_INVALID,
                "tensor map encode failed (CUresult %d): base %p rank %d dims [%llu,%llu,%llu,%llu] "
                "stride bytes [%llu,%llu,%llu] box [%u,%u,%u,%u]",
                static_cast<int>(r), base, rank, (unsigned long long)gdim[0],
                (unsigned long long)(rank > 1 ? gdim[1] : 0),
                (unsigned long long)(rank > 2 ? gdim[2] : 0),
                (unsigned long long)(rank > 3 ? gdim[3] : 0),
                (unsigned long long)(rank > 1 ? gstr[0] : 0),
                (unsigned long long)(rank > 2 ? gstr[1] : 0),
                (unsigned long long)(rank > 3 ? gstr[2] : 0), bx[0], rank > 1 ? bx[1] : 0,
                rank > 2 ? bx[2] : 0, rank > 3 ? bx[3] : 0);
  return CDL_OK;
}

// ---------------------------------------------------------------- per-launch profiler
struct ProfileState {
  std::mutex mu;
  std::vector<cudaEvent_t> start, stop;
  std::vector<int> kind;
  std::vector<double> work;
  std::atomic<int> next{0};
  std::atomic<bool> enabled{false};
};
static ProfileState& prof() {
  static ProfileState s;
  return s;
}

ProfileScope::ProfileScope(int kind, double work, cudaStream_t stream) : index_(-1), stream_(stream) {
  ProfileState& p = prof();
  if (!p.enabled.load(std::memory_order_relaxed)) return;
  const int i = p.next.fetch_add(1);
  if (i >= static_cast<int>(p.start.size())) return;
  index_ = i;
  p.kind[i] = kind;
  p.work[i] = work;
  cudaEventRecord(p.start[i], stream);
}
ProfileScope::~ProfileScope() {
  if (index_ >= 0) cudaEventRecord(prof().stop[index_], stream_);
}

}  // namespace cdl

extern "C" {

int32_t cdl_b200_profile_start(int32_t max_records) {
  cdl::ProfileState& p = cdl::prof();
  std::lock_guard<std::mutex> lock(p.mu);
  if (max_records <= 0) return cdl::fail(CDL_ERR_INVALID, "profile_start: max_records must be positive");
  p.enabled.store(false);
  while (static_cast<int>(p.start.size()) < max_records) {
    cudaEvent_t a, b;
    CDL_CUDA(cudaEventCreate(&a));
    CDL_CUDA(cudaEventCreate(&b));
    p.start.push_back(a);
    p.stop.push_back(b);
  }
  p.kind.assign(p.start.size(), 0);
  p.work.assign(p.start.size(), 0.0);
  p.next.store(0);
  p.enabled.store(true);
  return CDL_OK;
}

int32_t cdl_b200_profile_stop(cdl_profile_record* out, int32_t capacity, int32_t* count) {
  cdl::ProfileState& p = cdl::prof();
  std::lock_guard<std::mutex> lock(p.mu);
  p.enabled.store(false);
  CDL_CUDA(cudaDeviceSynchronize());
  int n = p.next.load();
  if (n > static_cast<int>(p.start.size())) n = static_cast<int>(p.start.size());
  int written = 0;
  for (int i = 0; i < n && written < capacity; ++i) {
    float ms = 0.f;
    if (cudaEventElapsedTime(&ms, p.start[i], p.stop[i]) != cudaSuccess) continue;
    if (out) {
      out[written].kind = p.kind[i];
      out[written].ms = ms;
      out[written].work = p.work[i];
    }
    ++written;
  }
  if (count) *count = written;
  return CDL_OK;
}

const char* cdl_b200_last_error(void) { return cdl::last_error().c_str(); }

int32_t cdl_b200_device_ok(int32_t device) {
  int major = 0, minor = 0;
  CDL_CUDA(cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, device));
  CDL_CUDA(cudaDeviceGetAttribute(&minor, cudaDevAttrComputeCapabilityMinor, device));
  if (major != 10)
    return cdl::fail(CDL_ERR_UNSUPPORTED,
                     "device %d has compute capability %d.%d; this library only holds sm_100a code",
                     device, major, minor);
  return CDL_OK;
}

int32_t cdl_b200_device_status(int32_t* status_out) {
  int* p = cdl::device_status_ptr();
  if (!p) return cdl::fail(CDL_ERR_CUDA, "cannot resolve the device status word");
  CDL_CUDA(cudaDeviceSynchronize());
  int v = 0;
  CDL_CUDA(cudaMemcpy(&v, p, sizeof v, cudaMemcpyDeviceToHost));
  if (v != 0) {
    int zero = 0;
    CDL_CUDA(cudaMemcpy(p, &zero, sizeof zero, cudaMemcpyHostToDevice));
  }
  if (status_out) *status_out = v;
  return CDL_OK;
}

}  // extern "C"
