// Host-side helpers shared by the operator implementations: error reporting, operand
// validation and TMA tensor-map encoding.
#pragma once
#include <cuda.h>
#include <cuda_runtime.h>
#include <stdarg.h>
#include <stdint.h>
#include <stdio.h>

#include <string>
#include <utility>

#include "../../include/cleandl_b200.h"

namespace cdl {

// Thread-local message of the last failure; returned by cdl_b200_last_error().
std::string& last_error();
// Records a formatted message and returns `code`.
int32_t fail(int32_t code, const char* fmt, ...) __attribute__((format(printf, 2, 3)));

#define CDL_CUDA(expr)                                                                     \
  do {                                                                                     \
    cudaError_t _e = (expr);                                                               \
    if (_e != cudaSuccess)                                                                 \
      return ::cdl::fail(CDL_ERR_CUDA, "%s failed: %s", #expr, cudaGetErrorString(_e));    \
  } while (0)

#define CDL_CHECK(expr)           \
  do {                            \
    int32_t _s = (expr);          \
    if (_s != CDL_OK) return _s;  \
  } while (0)

inline size_t dtype_size(int32_t dt) { return dt == CDL_BF16 ? 2 : 4; }
inline const char* dtype_name(int32_t dt) {
  return dt == CDL_BF16 ? "bf16" : dt == CDL_F32 ? "f32" : dt == CDL_I32 ? "i32" : "?";
}

// Device-global status word written by kernels whose bounded waits ran out (see ptx.cuh).
int* device_status_ptr();  // device address for the current device; nullptr on failure

// The number of SMs of the current device (cached per device).
int sm_count();

// Element type of a tensor map over bytes (block-scaled FP8 values); not a cdl_dtype.
constexpr int32_t TMAP_U8 = 100;

// Encodes a tiled tensor map over bf16 / f32 / byte data.  dims/strides are innermost-first; strides are
// in BYTES for dims 1.. (the innermost is contiguous).  box is innermost-first.
int32_t encode_tmap(CUtensorMap* out, const void* base, int32_t dtype, int rank,
                    const uint64_t* dims, const uint64_t* strides_bytes, const uint32_t* box,
                    bool swizzle128);

// Launches `kernel` with the programmatic-serialization attribute (see grid_dep_wait in ptx.cuh):
// the kernel may begin before the previous kernel of the stream has finished and MUST call
// grid_dep_wait() before its first access to global memory.  CDL_PDL=0 builds launch normally.
#ifndef CDL_PDL
#define CDL_PDL 1
#endif
template <typename... KArgs, typename... Args>
inline cudaError_t launch_pdl(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem,
                              cudaStream_t stream, Args&&... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = CDL_PDL ? 1 : 0;
  return cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...);
}

// Device counter for a kernel that hands out its work at run time (see host.cu); nullptr: none.
unsigned int* sched_counter_for(int kind, int dev, cudaStream_t stream);

// Opt-in per-launch timing (cdl_b200_profile_start / _stop).  When enabled, a launcher brackets
// its kernel with two pre-created CUDA events on the launching stream; when disabled the scope
// costs one relaxed atomic load.
enum ProfileKind { PROF_GEMM = 1, PROF_NORM_FWD = 2, PROF_NORM_BWD = 3, PROF_ATTN_FWD = 4,
                   PROF_ATTN_BWD = 5, PROF_ELEMENTWISE = 6 };
class ProfileScope {
 public:
  ProfileScope(int kind, double work, cudaStream_t stream);
  ~ProfileScope();
 private:
  int index_;
  cudaStream_t stream_;
};

}  // namespace cdl
