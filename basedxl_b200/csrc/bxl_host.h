// Host-side plumbing shared by the C-ABI entry points: error reporting, the
// device status word, and TMA descriptor encoding through the driver entry
// point (the library does not link against libcuda).
#pragma once
#include <cuda.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace bxl {

// status codes returned over the C ABI (0 = ok, negative = error)
enum : int {
  kOk = 0,
  kErrInvalidArg = -1,
  kErrCuda = -2,
  kErrUnsupported = -3,
  kErrDevice = -4,   // a kernel recorded a failure in the device status word
  kErrTooLarge = -5,
};

int fail(int code, const char* fmt, ...);          // records the message, returns code
int check_cuda(cudaError_t e, const char* what);   // kOk or kErrCuda (+ message)
int* device_status_ptr();                          // per-device status word (3 ints), nullptr on failure

// 16-bit (fp16) tiled tensor map with 128-byte swizzle and zero fill.
// dims/box: innermost first.  strides_bytes: rank-1 entries for dims 1..rank-1.
int encode_tmap_f16(CUtensorMap* out, const void* base, int rank, const uint64_t* dims, const uint64_t* strides_bytes,
                    const uint32_t* box);

int sm_count();

// Whether kernels are launched with programmatic stream serialisation (default on;
// BXL_PDL=0 in the environment or bxl_set_pdl(0) turns it off).
bool pdl_enabled();
// Whether weight operands (GEMM B, packed conv weights, LayerNorm scale/shift) may be fetched
// before a kernel waits for its predecessor (bxl_set_static_weights).
bool static_weights();
void set_static_weights(bool on);

// Launch through cudaLaunchKernelEx with the programmatic-serialisation attribute and
// an optional thread-block cluster width.
template <typename... KArgs, typename... Args>
int launch_kernel(const char* what, void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream,
                  int cluster_x, Args&&... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[2];
  int n = 0;
  if (cluster_x > 1) {
    attr[n].id = cudaLaunchAttributeClusterDimension;
    attr[n].val.clusterDim.x = cluster_x;
    attr[n].val.clusterDim.y = 1;
    attr[n].val.clusterDim.z = 1;
    ++n;
  }
  if (pdl_enabled()) {
    attr[n].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[n].val.programmaticStreamSerializationAllowed = 1;
    ++n;
  }
  cfg.attrs = attr;
  cfg.numAttrs = n;
  return check_cuda(cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...), what);
}

}  // namespace bxl
