#include "bxl_host.h"

#include <stdarg.h>
#include <stdio.h>
#include <stdlib.h>
#include <string.h>

#include "../../include/basedxl_b200.h"

namespace bxl {

static thread_local char g_err[512] = "";

int fail(int code, const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(g_err, sizeof(g_err), fmt, ap);
  va_end(ap);
  return code;
}

int check_cuda(cudaError_t e, const char* what) {
  if (e == cudaSuccess) return kOk;
  return fail(kErrCuda, "%s: %s", what, cudaGetErrorString(e));
}

// One status word per device, living in device memory for the life of the
// process.  Kernels only ever write it on failure.
__device__ int g_dev_status[4];

static int* g_status_ptr[64] = {};
static int g_sm_count[64] = {};

int* device_status_ptr() {
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return nullptr;
  if (!g_status_ptr[dev]) {
    void* p = nullptr;
    if (cudaGetSymbolAddress(&p, g_dev_status) != cudaSuccess) return nullptr;
    if (cudaMemset(p, 0, sizeof(int) * 4) != cudaSuccess) return nullptr;
    g_status_ptr[dev] = static_cast<int*>(p);
  }
  return g_status_ptr[dev];
}

int sm_count() {
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return 148;
  if (!g_sm_count[dev]) {
    int n = 0;
    if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) n = 148;
    g_sm_count[dev] = n;
  }
  return g_sm_count[dev];
}

static int g_pdl = -1;
static int g_static_weights = 0;
bool static_weights() { return g_static_weights != 0; }
void set_static_weights(bool on) { g_static_weights = on ? 1 : 0; }
bool pdl_enabled() {
  if (g_pdl < 0) {
    const char* e = getenv("BXL_PDL");
    g_pdl = (e && e[0] == '0') ? 0 : 1;
  }
  return g_pdl != 0;
}

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
static EncodeTiledFn g_encode = nullptr;

static int load_encode() {
  if (g_encode) return kOk;
  void* fn = nullptr;
  cudaDriverEntryPointQueryResult q;
  cudaError_t e = cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &q);
  if (e != cudaSuccess || q != cudaDriverEntryPointSuccess || !fn)
    return fail(kErrCuda, "cuTensorMapEncodeTiled entry point unavailable (%s)", cudaGetErrorString(e));
  g_encode = reinterpret_cast<EncodeTiledFn>(fn);
  return kOk;
}

int encode_tmap_f16(CUtensorMap* out, const void* base, int rank, const uint64_t* dims, const uint64_t* strides_bytes,
                    const uint32_t* box) {
  if (int rc = load_encode()) return rc;
  if ((reinterpret_cast<uintptr_t>(base) & 15u) != 0) return fail(kErrInvalidArg, "tensor base %p not 16-byte aligned", base);
  cuuint64_t gdim[5];
  cuuint64_t gstr[4];
  cuuint32_t bdim[5];
  cuuint32_t estr[5];
  for (int i = 0; i < rank; ++i) {
    gdim[i] = dims[i];
    bdim[i] = box[i];
    estr[i] = 1;
    if (i > 0) {
      gstr[i - 1] = strides_bytes[i - 1];
      if (gstr[i - 1] % 16 != 0) return fail(kErrInvalidArg, "tensor stride %llu not a multiple of 16 bytes", (unsigned long long)gstr[i - 1]);
    }
  }
  CUresult r = g_encode(out, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, (cuuint32_t)rank, const_cast<void*>(base), gdim, gstr, bdim,
                        estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                        CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return fail(kErrCuda, "cuTensorMapEncodeTiled failed with CUresult %d (rank %d)", (int)r, rank);
  return kOk;
}

}  // namespace bxl

extern "C" {

const char* bxl_last_error(void) { return bxl::g_err; }

int bxl_init(void) {
  if (!bxl::device_status_ptr()) return bxl::fail(bxl::kErrCuda, "cannot set up the device status word (no CUDA device?)");
  if (int rc = bxl::load_encode()) return rc;
  int dev = 0, major = 0;
  cudaGetDevice(&dev);
  cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, dev);
  if (major != 10) return bxl::fail(bxl::kErrUnsupported, "device compute capability %d.x: this library is sm_100a only", major);
  return bxl::kOk;
}

int bxl_device_status(int* code, int* site, int* block) {
  int* p = bxl::device_status_ptr();
  if (!p) return bxl::fail(bxl::kErrCuda, "no device status word");
  int h[4] = {0, 0, 0, 0};
  if (int rc = bxl::check_cuda(cudaMemcpy(h, p, sizeof(h), cudaMemcpyDeviceToHost), "read device status")) return rc;
  if (code) *code = h[0];
  if (site) *site = h[1];
  if (block) *block = h[2];
  if (h[0] != 0) {
    cudaMemset(p, 0, sizeof(h));
    return bxl::fail(bxl::kErrDevice, "kernel reported status %d at wait site %d (block %d)", h[0], h[1], h[2]);
  }
  return bxl::kOk;
}

int bxl_sm_count(void) { return bxl::sm_count(); }

int bxl_set_pdl(int enabled) {
  bxl::g_pdl = enabled ? 1 : 0;
  return bxl::kOk;
}

}  // extern "C"
