#include <cstdlib>
#include "host_common.h"

#include <mutex>

namespace fluxb {

static thread_local std::string g_last_error;

void set_last_error(const std::string& msg) { g_last_error = msg; }

int fail(int code, const std::string& msg) {
  g_last_error = msg;
  return code;
}

void* driver_entry(const char* name) {
  void* fn = nullptr;
  cudaDriverEntryPointQueryResult q;
  if (cudaGetDriverEntryPoint(name, &fn, cudaEnableDefault, &q) != cudaSuccess ||
      q != cudaDriverEntryPointSuccess) {
    (void)cudaGetLastError();
    return nullptr;
  }
  return fn;
}

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*,
                                  const cuuint64_t*, const cuuint64_t*, const cuuint32_t*,
                                  const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

int encode_tmap(CUtensorMap* out, CUtensorMapDataType dt, int nd, const void* base,
                const uint64_t* dims, const uint64_t* strides_bytes, const uint32_t* box,
                Swz swz) {
  static EncodeTiledFn fn = reinterpret_cast<EncodeTiledFn>(driver_entry("cuTensorMapEncodeTiled"));
  if (fn == nullptr) return fail(kErrCuda, "cuTensorMapEncodeTiled is not available (no driver?)");
  if ((reinterpret_cast<uintptr_t>(base) & 15u) != 0)
    return fail(kErrInvalid, "tensor base address must be 16-byte aligned for TMA");
  // L2 promotion of the tiled loads: 256 B unless FLUXB_TMAP_L2PROMO says 0 (none), 64 or 128
  static const CUtensorMapL2promotion l2promo = [] {
    const char* e = getenv("FLUXB_TMAP_L2PROMO");
    const int v = e ? atoi(e) : 256;
    if (v == 0) return CU_TENSOR_MAP_L2_PROMOTION_NONE;
    if (v == 64) return CU_TENSOR_MAP_L2_PROMOTION_L2_64B;
    if (v == 128) return CU_TENSOR_MAP_L2_PROMOTION_L2_128B;
    return CU_TENSOR_MAP_L2_PROMOTION_L2_256B;
  }();
  cuuint64_t gdim[5];
  cuuint64_t gstr[5];
  cuuint32_t bdim[5];
  cuuint32_t estr[5];
  for (int i = 0; i < nd; ++i) {
    gdim[i] = dims[i];
    bdim[i] = box[i];
    estr[i] = 1;
    if (i > 0) {
      if (strides_bytes[i - 1] % 16 != 0)
        return fail(kErrInvalid, "tensor row pitch must be a multiple of 16 bytes for TMA");
      gstr[i - 1] = strides_bytes[i - 1];
    }
  }
  CUresult r = fn(out, dt, static_cast<cuuint32_t>(nd), const_cast<void*>(base), gdim, gstr, bdim,
                  estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                  swz == Swz::B128 ? CU_TENSOR_MAP_SWIZZLE_128B : CU_TENSOR_MAP_SWIZZLE_NONE,
                  l2promo, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS)
    return fail(kErrCuda, "cuTensorMapEncodeTiled failed with CUresult " + std::to_string(int(r)));
  return kOk;
}

int device_sm_count(int* out) {
  static int cached[64] = {0};
  int dev = 0;
  FLUXB_CUDA_OK(cudaGetDevice(&dev));
  if (dev < 64 && cached[dev] > 0) {
    *out = cached[dev];
    return kOk;
  }
  int n = 0;
  FLUXB_CUDA_OK(cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev));
  if (dev < 64) cached[dev] = n;
  *out = n;
  return kOk;
}

}  // namespace fluxb

extern "C" const char* fluxb_last_error() { return fluxb::g_last_error.c_str(); }
