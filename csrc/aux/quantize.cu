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
#include <type_traits>

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

// ---------------------------------------------------------------------------------------------
// Fast path for 16-bit inputs and whole 128 x 128 tiles: the tile lives in registers. A thread owns
// 4 consecutive rows x 8 columns (16 bytes per row) in each of two passes over the 32 row groups,
// so that a half-warp reads one 256-byte row segment per instruction; row maxima are reduced by
// shuffles, column maxima through a small shared array; q leaves as 8-byte stores (128 contiguous
// bytes per row), q^T is transposed through a swizzled shared tile (a thread's 4 rows of one column
// are one 32-bit word) and leaves as 16-byte stores. About five instructions per element instead
// of forty: the kernel is memory bound.
// ---------------------------------------------------------------------------------------------
template <bool BF16>
__device__ __forceinline__ uint32_t habs2_bits(uint32_t v) {
  return v & 0x7FFF7FFFu;
}
template <bool BF16>
__device__ __forceinline__ uint32_t hmax2_bits(uint32_t a, uint32_t b) {
  // operands are non-negative 16-bit floats: their order is the order of their bit patterns
  uint32_t r;
  asm("max.u16x2 %0, %1, %2;" : "=r"(r) : "r"(a), "r"(b));
  return r;
}
template <bool BF16>
__device__ __forceinline__ float h_lo(uint32_t v) {
  if constexpr (BF16) return __uint_as_float(v << 16);
  else return __half2float(__ushort_as_half(static_cast<unsigned short>(v & 0xFFFFu)));
}
template <bool BF16>
__device__ __forceinline__ float h_hi(uint32_t v) {
  if constexpr (BF16) return __uint_as_float(v & 0xFFFF0000u);
  else return __half2float(__ushort_as_half(static_cast<unsigned short>(v >> 16)));
}
__device__ __forceinline__ uint32_t cvt_fp8x2(float lo, float hi, bool e5m2) {
  return static_cast<uint32_t>(
      __nv_cvt_float2_to_fp8x2(make_float2(lo, hi), __NV_SATFINITE, e5m2 ? __NV_E5M2 : __NV_E4M3));
}

template <bool BF16, bool SQUARE>
__global__ void __launch_bounds__(kThreads) quant_tile_kernel(
    const uint16_t* __restrict__ x, int64_t ldx, uint8_t* __restrict__ q, uint8_t* __restrict__ qt,
    float* __restrict__ sinv, float* __restrict__ sinv_t, int M, int K, float eps, int e5m2,
    int64_t batch_stride_x, int64_t batch_stride_q, int64_t batch_stride_s) {
  __shared__ uint32_t colred[kThreads / 32][64];         // packed column maxima per warp
  __shared__ float col_scale[kTile];
  __shared__ float red[kThreads / 32];
  __shared__ __align__(16) uint32_t tile_t[kTile * 32];   // q^T tile: 128 rows (columns of x) x 128 bytes, swizzled
  const int kb = blockIdx.x, mb = blockIdx.y, bz = blockIdx.z;
  const int MB = gridDim.y, KB = gridDim.x;
  x += bz * batch_stride_x;
  q += bz * batch_stride_q;
  if (qt) qt += bz * batch_stride_q;
  sinv += bz * batch_stride_s;
  if (sinv_t) sinv_t += bz * batch_stride_s;
  const int row0 = mb * kTile, col0 = kb * kTile;
  const float fp8_max = e5m2 ? 57344.f : 448.f;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int chunk = lane & 15;                  // 8-column chunk of the tile
  const bool e5 = e5m2 != 0;

  // ---- load: pass `it`, row group g = it * 16 + warp * 2 + lane / 16, rows 4g .. 4g + 3
  uint4 v[2][4];
#pragma unroll
  for (int it = 0; it < 2; ++it) {
    const int g = it * 16 + warp * 2 + (lane >> 4);
#pragma unroll
    for (int r = 0; r < 4; ++r)
      v[it][r] = *reinterpret_cast<const uint4*>(x + static_cast<int64_t>(row0 + 4 * g + r) * ldx + col0 + chunk * 8);
  }
  // ---- maxima: per row (over the 16 lanes that share it) and per column pair (over this thread's rows)
  float row_amax[2][4];
  uint32_t cm[4] = {0u, 0u, 0u, 0u};
#pragma unroll
  for (int it = 0; it < 2; ++it)
#pragma unroll
    for (int r = 0; r < 4; ++r) {
      const uint32_t a0 = habs2_bits<BF16>(v[it][r].x), a1 = habs2_bits<BF16>(v[it][r].y);
      const uint32_t a2 = habs2_bits<BF16>(v[it][r].z), a3 = habs2_bits<BF16>(v[it][r].w);
      cm[0] = hmax2_bits<BF16>(cm[0], a0);
      cm[1] = hmax2_bits<BF16>(cm[1], a1);
      cm[2] = hmax2_bits<BF16>(cm[2], a2);
      cm[3] = hmax2_bits<BF16>(cm[3], a3);
      uint32_t m = hmax2_bits<BF16>(hmax2_bits<BF16>(a0, a1), hmax2_bits<BF16>(a2, a3));
#pragma unroll
      for (int o = 8; o > 0; o >>= 1) m = hmax2_bits<BF16>(m, __shfl_xor_sync(0xffffffffu, m, o));
      row_amax[it][r] = fmaxf(h_lo<BF16>(m), h_hi<BF16>(m));
    }
  if (qt != nullptr || SQUARE) {
#pragma unroll
    for (int w = 0; w < 4; ++w) cm[w] = hmax2_bits<BF16>(cm[w], __shfl_xor_sync(0xffffffffu, cm[w], 16));
    if (lane < 16) {
#pragma unroll
      for (int w = 0; w < 4; ++w) colred[warp][chunk * 4 + w] = cm[w];
    }
  }
  float tile_scale = 1.f;
  if constexpr (SQUARE) {
    __syncthreads();
    // one scale for the tile: maximum over all packed column maxima
    uint32_t m = 0u;
    if (tid < 64) {
#pragma unroll
      for (int w = 0; w < kThreads / 32; ++w) m = hmax2_bits<BF16>(m, colred[w][tid]);
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) m = hmax2_bits<BF16>(m, __shfl_xor_sync(0xffffffffu, m, o));
    if (lane == 0) red[warp] = fmaxf(h_lo<BF16>(m), h_hi<BF16>(m));
    __syncthreads();
    const float amax = fmaxf(red[0], red[1]);
    tile_scale = compute_scale(amax, eps, fp8_max);
    if (tid == 0) {
      sinv[mb * KB + kb] = 1.f / tile_scale;
      if (sinv_t) sinv_t[kb * MB + mb] = 1.f / tile_scale;
    }
  }
  // ---- q: one scale per row (or the tile's), 8 bytes per thread and row
#pragma unroll
  for (int it = 0; it < 2; ++it) {
    const int g = it * 16 + warp * 2 + (lane >> 4);
#pragma unroll
    for (int r = 0; r < 4; ++r) {
      float scale = tile_scale;
      if constexpr (!SQUARE) {
        scale = compute_scale(row_amax[it][r], eps, fp8_max);
        if (chunk == 0) sinv[(static_cast<int64_t>(mb) * KB + kb) * kTile + 4 * g + r] = 1.f / scale;
      }
      const uint32_t w[4] = {v[it][r].x, v[it][r].y, v[it][r].z, v[it][r].w};
      uint2 o;
      o.x = cvt_fp8x2(h_lo<BF16>(w[0]) * scale, h_hi<BF16>(w[0]) * scale, e5) |
            (cvt_fp8x2(h_lo<BF16>(w[1]) * scale, h_hi<BF16>(w[1]) * scale, e5) << 16);
      o.y = cvt_fp8x2(h_lo<BF16>(w[2]) * scale, h_hi<BF16>(w[2]) * scale, e5) |
            (cvt_fp8x2(h_lo<BF16>(w[3]) * scale, h_hi<BF16>(w[3]) * scale, e5) << 16);
      *reinterpret_cast<uint2*>(q + static_cast<int64_t>(row0 + 4 * g + r) * K + col0 + chunk * 8) = o;
    }
  }
  if (qt == nullptr) return;
  // ---- q^T: one scale per column (or the tile's)
  if constexpr (!SQUARE) {
    __syncthreads();
    if (tid < 64) {
      uint32_t m = 0u;
#pragma unroll
      for (int w = 0; w < kThreads / 32; ++w) m = hmax2_bits<BF16>(m, colred[w][tid]);
      const float s0 = compute_scale(h_lo<BF16>(m), eps, fp8_max), s1 = compute_scale(h_hi<BF16>(m), eps, fp8_max);
      col_scale[2 * tid] = s0;
      col_scale[2 * tid + 1] = s1;
      float* st = sinv_t + (static_cast<int64_t>(kb) * MB + mb) * kTile + 2 * tid;
      st[0] = 1.f / s0;
      st[1] = 1.f / s1;
    }
    __syncthreads();
  }
  // a thread's 4 rows of one column are one word of row c of the transposed tile; word g of row c
  // sits at (g ^ swizzle(c)) so that the lanes of a warp hit different banks
#pragma unroll
  for (int it = 0; it < 2; ++it) {
    const int g = it * 16 + warp * 2 + (lane >> 4);
    uint32_t w[4][4];
#pragma unroll
    for (int r = 0; r < 4; ++r) {
      w[r][0] = v[it][r].x;
      w[r][1] = v[it][r].y;
      w[r][2] = v[it][r].z;
      w[r][3] = v[it][r].w;
    }
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const int c = chunk * 8 + j;
      const float scale = SQUARE ? tile_scale : col_scale[c];
      float f[4];
#pragma unroll
      for (int r = 0; r < 4; ++r) f[r] = ((j & 1) ? h_hi<BF16>(w[r][j >> 1]) : h_lo<BF16>(w[r][j >> 1])) * scale;
      const uint32_t word = cvt_fp8x2(f[0], f[1], e5) | (cvt_fp8x2(f[2], f[3], e5) << 16);
      tile_t[c * 32 + (g ^ ((chunk * 4) & 31))] = word;
    }
  }
  __syncthreads();
  // rows of q^T: 8 x 16 bytes each
#pragma unroll
  for (int k = 0; k < 4; ++k) {
    const int idx = tid + k * kThreads;          // 0 .. 1023
    const int c = idx >> 3, part = idx & 7;      // row of q^T, 16-byte piece
    const int phys = (part * 4) ^ (((c >> 3) * 4) & 31);
    const uint4 o = *reinterpret_cast<const uint4*>(&tile_t[c * 32 + phys]);
    *reinterpret_cast<uint4*>(qt + static_cast<int64_t>(col0 + c) * M + row0 + part * 16) = o;
  }
}

template <typename T, bool SQUARE>
int launch_quant(const void* x, int64_t ldx, void* q, void* qt, float* sinv, float* sinv_t, int M,
                 int K, int batch, float eps, int e5m2, cudaStream_t stream) {
  if constexpr (sizeof(T) == 2) {
    // whole tiles, 16-byte aligned rows everywhere: the register-tile kernel
    const bool aligned = M % kTile == 0 && K % kTile == 0 && ldx % 8 == 0 &&
                         ((reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(q) |
                           reinterpret_cast<uintptr_t>(qt)) & 15) == 0;
    if (aligned) {
      constexpr bool kBf16 = std::is_same<T, __nv_bfloat16>::value;
      dim3 grid(K / kTile, M / kTile, batch);
      const int64_t sstride = SQUARE ? static_cast<int64_t>(M / kTile) * (K / kTile)
                                     : static_cast<int64_t>(M / kTile) * (K / kTile) * kTile;
      quant_tile_kernel<kBf16, SQUARE><<<grid, kThreads, 0, stream>>>(
          reinterpret_cast<const uint16_t*>(x), ldx, reinterpret_cast<uint8_t*>(q), reinterpret_cast<uint8_t*>(qt),
          sinv, sinv_t, M, K, eps, e5m2, static_cast<int64_t>(M) * ldx, static_cast<int64_t>(M) * K, sstride);
      FLUXB_CUDA_OK(cudaGetLastError());
      g_launches.fetch_add(1, std::memory_order_relaxed);
      return kOk;
    }
  }
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
