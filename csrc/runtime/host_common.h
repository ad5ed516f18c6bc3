// Host-side helpers shared by every translation unit of libfluxb: error strings returned
// through the C API, late-bound driver entry points (no link-time dependency on libcuda, the
// role of the reference's src/cuda/cuda_stub.cc), and tensor-map encoding.
#pragma once

#include <cuda.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include <string>

namespace fluxb {

// Error codes returned by every extern "C" entry point.
enum : int {
  kOk = 0,
  kErrInvalid = 1,     // bad argument (shape, alignment, dtype)
  kErrCuda = 2,        // a CUDA runtime / driver call failed
  kErrUnsupported = 3, // valid request this build does not cover
  kErrTimeout = 4,     // a bounded device wait gave up (see Status)
};

void set_last_error(const std::string& msg);
int fail(int code, const std::string& msg);

#define FLUXB_CUDA_OK(expr)                                                              \
  do {                                                                                   \
    cudaError_t _e = (expr);                                                             \
    if (_e != cudaSuccess)                                                               \
      return ::fluxb::fail(::fluxb::kErrCuda, std::string(#expr) + ": " + cudaGetErrorString(_e)); \
  } while (0)

#define FLUXB_REQUIRE(cond, msg)                                          \
  do {                                                                    \
    if (!(cond)) return ::fluxb::fail(::fluxb::kErrInvalid, std::string(msg) + " [" #cond "]"); \
  } while (0)

// Driver entry points resolved at first use through the runtime.
void* driver_entry(const char* name);

enum class Swz { None, B128 };

// rank-`nd` tiled tensor map over row-major memory. dims/box in elements (innermost first),
// strides in bytes for dims 1..nd-1. Returns kOk or an error code.
int encode_tmap(CUtensorMap* out, CUtensorMapDataType dt, int nd, const void* base,
                const uint64_t* dims, const uint64_t* strides_bytes, const uint32_t* box, Swz swz);

int device_sm_count(int* out);
// A zeroed device word from a small per-device pool, for launches that keep their CTAs in step wave
// by wave; the launch leaves it at zero again. One word per stream (csrc/ops/dense_gemm.cu); null
// when the pool has no word left for a new stream.
uint32_t* wave_counter_for(cudaStream_t stream);

}  // namespace fluxb
