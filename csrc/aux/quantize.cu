// Block-scaled FP8 quantisation: 1x128 (per row, per 128 columns) and 128x128 blocks, each with
// an optional second output for the transposed matrix, in one pass over the input.
//
//   scale     = 448 / max(amax, eps)       (e4m3; 57344 for e5m2), 1 if the block is all zero
//   q         = saturate_to_fp8(x * scale)
//   scale_inv = 1 / scale                  (what is stored)
//
// 1x128 layout: q [M,K], scale_inv [ceil(M/128), ceil(K/128), 128] (row inside the block last);
// the transposed output is a separate quantisation of x^T with its own 1x128 blocks, i.e. one
// scale per column of x per 128 rows: q_t [K,M], scale_inv_t [ceil(K/128), ceil(M/128), 128].
// 128x128 layout: scale_inv [ceil(M/128), ceil(K/128)], q_t = transpose(q),
// scale_inv_t [ceil(K/128), ceil(M/128)].
// Reference: src/quantization/quantization.cu (ComputeScale :306-362, kernels :428-1193) and
// src/quantization/ths_op/quantization.cc:75-172.
#include "../include/fluxb.h"
#include "../runtime/host_common.h"

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_fp8.h>

#include <atomic>

namespace fluxb {
extern std::atomic<uint64_t> g_launches;

namespace {

constexpr int kTile = 128;
constexpr int kThreads = 256;

template <typename T>
__device__ __forceinline__ float to_f32(T v);
template <>
__device__ __forceinline__ float to_f32<__nv_bfloat16>(__nv_bfloat16 v) { return __bfloat162float(v); }
template <>
__device__ __forceinline__ float to_f32<__half>(__half v) { return __half2float(v); }
template <>
__device__ __forceinline__ float to_f32<float>(float v) { return v; }

__device__ __forceinline__ float compute_scale(float amax, float eps, float fp8_max) {
  const float a = fmaxf(amax, eps);
  if (a == 0.f) return 1.f;
  const float s = fp8_max / a;
  if (isinf(s)) return 3.3895313892515355e38f;  // largest finite bf16: the clamp of the reference
  return s;
}

__device__ __forceinline__ uint8_t to_fp8(float v, bool e5m2) {
  return static_cast<uint8_t>(
      __nv_cvt_float_to_fp8(v, __NV_SATFINITE, e5m2 ? __NV_E5M2 : __NV_E4M3));
}

// One CTA per 128x128 tile. The tile is staged in shared memory in the input type with a
// padded pitch so that both row-wise and column-wise passes are bank-conflict free.
template <typename T, bool SQUARE>
__global__ void __launch_bounds__(kThreads) quant_block_kernel(
    const T* __restrict__ x, int64_t ldx, uint8_t* __restrict__ q, uint8_t* __restrict__ qt,
    float* __restrict__ sinv, float* __restrict__ sinv_t, int M, int K, float eps, int e5m2,
    int64_t batch_stride_x, int64_t batch_stride_q, int64_t batch_stride_s) {
  constexpr int kPitch = kTile + 16 / sizeof(T);  // elements
  extern __shared__ __align__(16) uint8_t smem_raw[];
  T* tile = reinterpret_cast<T*>(smem_raw);
  __shared__ float red[kThreads / 32];
  __shared__ float col_scale[kTile];

  const int kb = blockIdx.x, mb = blockIdx.y, bz = blockIdx.z;
  const int MB = gridDim.y, KB = gridDim.x;
  x += bz * batch_stride_x;
  q += bz * batch_stride_q;
  if (qt) qt += bz * batch_stride_q;
  sinv += bz * batch_stride_s;
  if (sinv_t) sinv_t += bz * batch_stride_s;
  const int row0 = mb * kTile, col0 = kb * kTile;
  const int rows = min(kTile, M - row0), cols = min(kTile, K - col0);
  const float fp8_max = e5m2 ? 57344.f : 448.f;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;

  // ---- load (vectorised when the row pitch allows 16-byte accesses)
  constexpr int VEC = 16 / sizeof(T);
  const bool vec_ok = (ldx % VEC == 0) && (cols == kTile) &&
                      ((reinterpret_cast<uintptr_t>(x) & 15) == 0);
  if (vec_ok) {
    for (int i = tid; i < kTile * (kTile / VEC); i += kThreads) {
      const int r = i / (kTile / VEC), c = (i % (kTile / VEC)) * VEC;
      uint4 v = make_uint4(0, 0, 0, 0);
      if (r < rows) v = *reinterpret_cast<const uint4*>(x + (row0 + r) * ldx + col0 + c);
      *reinterpret_cast<uint4*>(tile + r * kPitch + c) = v;
    }
  } else {
    for (int i = tid; i < kTile * kTile; i += kThreads) {
      const int r = i / kTile, c = i % kTile;
      T v = T(0.f);
      if (r < rows && c < cols) v = x[(row0 + r) * ldx + col0 + c];
      tile[r * kPitch + c] = v;
    }
  }
  __syncthreads();

  if constexpr (SQUARE) {
    // ---- one scale for the whole tile
    float amax = 0.f;
    for (int i = tid; i < kTile * kTile; i += kThreads)
      amax = fmaxf(amax, fabsf(to_f32(tile[(i / kTile) * kPitch + (i % kTile)])));
    for (int o = 16; o > 0; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
    if (lane == 0) red[warp] = amax;
    __syncthreads();
    amax = red[0];
    for (int w = 1; w < kThreads / 32; ++w) amax = fmaxf(amax, red[w]);
    const float scale = compute_scale(amax, eps, fp8_max);
    if (tid == 0) {
      sinv[mb * KB + kb] = 1.f / scale;
      if (sinv_t) sinv_t[kb * MB + mb] = 1.f / scale;
    }
    // rows of q: each lane packs 4 consecutive columns
    for (int r = warp; r < rows; r += kThreads / 32) {
      const int c = lane * 4;
      uint32_t pk = 0;
#pragma unroll
      for (int j = 0; j < 4; ++j)
        pk |= static_cast<uint32_t>(to_fp8(to_f32(tile[r * kPitch + c + j]) * scale, e5m2)) << (8 * j);
      uint8_t* dst = q + static_cast<int64_t>(row0 + r) * K + col0 + c;
      if (cols == kTile && (K & 3) == 0) {
        *reinterpret_cast<uint32_t*>(dst) = pk;
      } else {
        for (int j = 0; j < 4; ++j)
          if (c + j < cols) dst[j] = static_cast<uint8_t>(pk >> (8 * j));
      }
    }
    if (qt) {
      // rows of q_t are columns of the tile; lane l takes rows l, l+32, l+64, l+96 so that a
      // warp reads 32 different rows (few bank conflicts) and writes 32 consecutive bytes
      for (int c = warp; c < cols; c += kThreads / 32) {
        uint8_t* dst = qt + static_cast<int64_t>(col0 + c) * M + row0;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const int r = lane + 32 * j;
          if (r < rows) dst[r] = to_fp8(to_f32(tile[r * kPitch + c]) * scale, e5m2);
        }
      }
    }
  } else {
    // ---- q: one scale per row of the tile (a warp owns 16 rows)
    for (int r = warp; r < kTile; r += kThreads / 32) {
      const int c = lane * 4;
      float v[4];
      float amax = 0.f;
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        v[j] = to_f32(tile[r * kPitch + c + j]);
        amax = fmaxf(amax, fabsf(v[j]));
      }
      for (int o = 16; o > 0; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
      const float scale = compute_scale(amax, eps, fp8_max);
      if (lane == 0) sinv[(static_cast<int64_t>(mb) * KB + kb) * kTile + r] = 1.f / scale;
      if (r < rows) {
        uint32_t pk = 0;
#pragma unroll
        for (int j = 0; j < 4; ++j) pk |= static_cast<uint32_t>(to_fp8(v[j] * scale, e5m2)) << (8 * j);
        uint8_t* dst = q + static_cast<int64_t>(row0 + r) * K + col0 + c;
        if (cols == kTile && (K & 3) == 0) {
          *reinterpret_cast<uint32_t*>(dst) = pk;
        } else {
          for (int j = 0; j < 4; ++j)
            if (c + j < cols) dst[j] = static_cast<uint8_t>(pk >> (8 * j));
        }
      }
    }
    if (qt) {
      // ---- q_t: one scale per column of the tile
      if (tid < kTile) {
        float amax = 0.f;
        for (int r = 0; r < kTile; ++r) amax = fmaxf(amax, fabsf(to_f32(tile[r * kPitch + tid])));
        const float scale = compute_scale(amax, eps, fp8_max);
        col_scale[tid] = scale;
        sinv_t[(static_cast<int64_t>(kb) * MB + mb) * kTile + tid] = 1.f / scale;
      }
      __syncthreads();
      for (int c = warp; c < cols; c += kThreads / 32) {
        const float scale = col_scale[c];
        uint8_t* dst = qt + static_cast<int64_t>(col0 + c) * M + row0;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const int r = lane + 32 * j;
          if (r < rows) dst[r] = to_fp8(to_f32(tile[r * kPitch + c]) * scale, e5m2);
        }
      }
    }
  }
}

template <typename T, bool SQUARE>
int launch_quant(const void* x, int64_t ldx, void* q, void* qt, float* sinv, float* sinv_t, int M,
                 int K, int batch, float eps, int e5m2, cudaStream_t stream) {
  constexpr int kPitch = kTile + 16 / sizeof(T);
  constexpr int smem = kTile * kPitch * sizeof(T);
  static bool configured[64] = {false};
  int dev = 0;
  FLUXB_CUDA_OK(cudaGetDevice(&dev));
  if (smem > 48 * 1024 && (dev >= 64 || !configured[dev])) {
    FLUXB_CUDA_OK(cudaFuncSetAttribute(quant_block_kernel<T, SQUARE>,
                                       cudaFuncAttributeMaxDynamicSharedMemorySize, smem));
    if (dev < 64) configured[dev] = true;
  }
  const int MB = (M + kTile - 1) / kTile, KB = (K + kTile - 1) / kTile;
  dim3 grid(KB, MB, batch);
  const int64_t sstride = SQUARE ? static_cast<int64_t>(MB) * KB : static_cast<int64_t>(MB) * KB * kTile;
  quant_block_kernel<T, SQUARE><<<grid, kThreads, smem, stream>>>(
      reinterpret_cast<const T*>(x), ldx, reinterpret_cast<uint8_t*>(q),
      reinterpret_cast<uint8_t*>(qt), sinv, sinv_t, M, K, eps, e5m2,
      static_cast<int64_t>(M) * ldx, static_cast<int64_t>(M) * K, sstride);
  FLUXB_CUDA_OK(cudaGetLastError());
  g_launches.fetch_add(1, std::memory_order_relaxed);
  return kOk;
}

}  // namespace
}  // namespace fluxb

using namespace fluxb;

extern "C" int fluxb_quantize_blockwise(const void* x, int64_t ldx, int in_dtype, void* q, void* qt,
                                        float* scale_inv, float* scale_inv_t, int M, int K,
                                        int batch, int square, float eps, int out_dtype,
                                        void* stream) {
  FLUXB_REQUIRE(x && q && scale_inv && M > 0 && K > 0 && batch > 0, "quantize arguments");
  FLUXB_REQUIRE((qt == nullptr) == (scale_inv_t == nullptr), "transposed output and scale go together");
  FLUXB_REQUIRE(out_dtype == FLUXB_FP8_E4M3 || out_dtype == FLUXB_FP8_E5M2, "fp8 output type");
  const int e5m2 = out_dtype == FLUXB_FP8_E5M2;
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
#define FLUXB_QUANT(T)                                                                           \
  return square ? launch_quant<T, true>(x, ldx, q, qt, scale_inv, scale_inv_t, M, K, batch, eps, \
                                        e5m2, s)                                                 \
                : launch_quant<T, false>(x, ldx, q, qt, scale_inv, scale_inv_t, M, K, batch, eps, \
                                         e5m2, s)
  switch (in_dtype) {
    case FLUXB_BF16: FLUXB_QUANT(__nv_bfloat16);
    case FLUXB_FP16: FLUXB_QUANT(__half);
    case FLUXB_FP32: FLUXB_QUANT(float);
    default: return fail(kErrUnsupported, "quantize input must be bf16, fp16 or fp32");
  }
#undef FLUXB_QUANT
}
