// Small single-GPU kernels: in-place fp32->bf16 compaction, bitwise compare, uniform fill,
// vector copy, and the stable MoE routing-index build.
// Reference: src/inplace_cast/inplace_cast.cu, src/cuda/bitwise_check.cu,
// src/cuda/random_initialize.cu, src/cuda/cuda_common.cu, src/cuda/moe_utils.cu,
// src/moe_ag_scatter/sort_util.cu (calc_gather_index).
#include "../include/fluxb.h"
#include "../runtime/host_common.h"
#include "../sm100/ptx.cuh"

#include <atomic>

namespace fluxb {
extern std::atomic<uint64_t> g_launches;

namespace {

// ----------------------------------------------------------------------------------------
// In-place fp32 -> bf16: the bf16 results are packed at the front of the same buffer.
// Output chunk c (kChunk elements) lands on the bytes of input chunk c/2, so it may be written
// only after that chunk has been read into registers. CTAs claim chunks in increasing order
// from a counter; "chunk read" is published as flag[c] = epoch; the wait on flag[c/2] is bounded.
// ----------------------------------------------------------------------------------------
constexpr int kCastThreads = 256;
constexpr int kCastVec = 8;                               // floats per 32-byte piece
constexpr int kCastPieces = 8;                            // pieces per thread, 2048 elements apart
constexpr int kChunk = kCastThreads * kCastVec * kCastPieces;  // 16384 elements: 64 KiB in, 32 KiB out

// Every thread converts its pieces as soon as they are loaded and keeps only the packed results
// (32 registers for eight pieces): the conversion needs the data, so when the CTA's barrier is
// passed every load of the chunk has completed, and "chunk read" can be published with a gpu-scope
// release. The chunk whose bytes are about to be overwritten (c / 2) was claimed long before this
// one except at the very start, so the acquire load of its flag almost never waits.
__global__ void __launch_bounds__(kCastThreads) inplace_cast_kernel(
    float* data, int64_t n, uint32_t* flags, uint32_t* claim, uint32_t epoch, uint64_t timeout_ns,
    Status* status) {
  __shared__ uint32_t abort_word;
  __shared__ uint32_t chunk_slot;
  if (threadIdx.x == 0) abort_word = 0;
  const uint32_t chunks = static_cast<uint32_t>((n + kChunk - 1) / kChunk);
  WaitCtx wc{status, &abort_word, timeout_ns};
  __nv_bfloat16* out = reinterpret_cast<__nv_bfloat16*>(data);
  while (true) {
    __syncthreads();
    if (threadIdx.x == 0) {
      const uint32_t got = atomicAdd(claim, 1u);
      if (got == chunks + gridDim.x - 1u) atomicExch(claim, 0u);  // last claim of the launch
      chunk_slot = got;
    }
    __syncthreads();
    const uint32_t c = chunk_slot;
    if (c >= chunks) break;
    uint4 o[kCastPieces];
    float4 a[kCastPieces], b[kCastPieces];
    const int64_t cbase = static_cast<int64_t>(c) * kChunk;
    const bool whole = cbase + kChunk <= n;
    if (whole) {
#pragma unroll
      for (int p = 0; p < kCastPieces; ++p) {
        const int64_t base = cbase + (p * kCastThreads + threadIdx.x) * kCastVec;
        a[p] = *reinterpret_cast<const float4*>(data + base);
        b[p] = *reinterpret_cast<const float4*>(data + base + 4);
      }
    } else {
#pragma unroll
      for (int p = 0; p < kCastPieces; ++p) {
        const int64_t base = cbase + (p * kCastThreads + threadIdx.x) * kCastVec;
        float t[kCastVec];
#pragma unroll
        for (int j = 0; j < kCastVec; ++j) t[j] = base + j < n ? data[base + j] : 0.f;
        a[p] = make_float4(t[0], t[1], t[2], t[3]);
        b[p] = make_float4(t[4], t[5], t[6], t[7]);
      }
    }
#pragma unroll
    for (int p = 0; p < kCastPieces; ++p) {
      o[p].x = ptx::pack_bf16x2(a[p].x, a[p].y);
      o[p].y = ptx::pack_bf16x2(a[p].z, a[p].w);
      o[p].z = ptx::pack_bf16x2(b[p].x, b[p].y);
      o[p].w = ptx::pack_bf16x2(b[p].z, b[p].w);
    }
    __syncthreads();  // every thread of the CTA has consumed its part of chunk c
    if (threadIdx.x == 0) {
      asm volatile("st.release.gpu.global.u32 [%0], %1;" ::"l"(flags + c), "r"(epoch) : "memory");
      // bounded wait on the chunk whose bytes this one overwrites
      const uint32_t* f = flags + (c >> 1);
      const uint64_t t0 = ptx::globaltimer_ns();
      uint32_t spins = 0;
      while (static_cast<int32_t>(ptx::ld_acquire_gpu(f) - epoch) < 0) {
        if ((++spins & 31u) == 0u && ptx::globaltimer_ns() - t0 > timeout_ns) {
          wait_give_up(wc, kSiteInplaceCast, *f, epoch);
          break;
        }
      }
    }
    __syncthreads();
    if (abort_word) break;   // the wait gave up: write nothing more
    if (whole) {
#pragma unroll
      for (int p = 0; p < kCastPieces; ++p)
        *reinterpret_cast<uint4*>(out + cbase + (p * kCastThreads + threadIdx.x) * kCastVec) = o[p];
    } else {
#pragma unroll
      for (int p = 0; p < kCastPieces; ++p) {
        const int64_t base = cbase + (p * kCastThreads + threadIdx.x) * kCastVec;
        const uint32_t w[4] = {o[p].x, o[p].y, o[p].z, o[p].w};
#pragma unroll
        for (int j = 0; j < kCastVec; ++j)
          if (base + j < n)
            reinterpret_cast<uint16_t*>(out)[base + j] = static_cast<uint16_t>(w[j >> 1] >> (16 * (j & 1)));
      }
    }
  }
}

// ----------------------------------------------------------------------------------------
// Sum of `cnt` rows per output row in fp32, 16-bit rows: out[t] = sum_j in[row(t, j)] with
// row(t, j) = idx[t * cnt + j] (the top-k reduce of expert outputs) or j * slab_rows + t (the sum
// over the leading dimension of a [B, M, N] tensor). One warp per output row, 16 bytes per lane and
// trip, up to eight source rows in flight.
// Reference: topk_scatter_reduce (src/pybind/gemm_grouped_v3_gather_rs.cc:33), bsr_reduce
// (src/gemm_rs/bsr_reduce.cu:26-126).
// ----------------------------------------------------------------------------------------
__global__ void __launch_bounds__(256) rows_sum_kernel(const uint16_t* __restrict__ in, const int32_t* __restrict__ idx,
                                                       uint16_t* __restrict__ out, int64_t rows_out, int cols,
                                                       int cnt, int64_t slab_rows, int f16) {
  const int lane = threadIdx.x & 31;
  const int64_t gwarp = static_cast<int64_t>(blockIdx.x) * 8 + (threadIdx.x >> 5);
  const int64_t nwarps = static_cast<int64_t>(gridDim.x) * 8;
  const int chunks = cols / 8;
  const bool h = f16 != 0;
  for (int64_t t = gwarp; t < rows_out; t += nwarps) {
    for (int c = lane; c < chunks; c += 32) {
      float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
      for (int j0 = 0; j0 < cnt; j0 += 8) {
        uint4 v[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          if (j0 + j < cnt) {
            const int64_t r = idx != nullptr ? idx[t * cnt + j0 + j] : (j0 + j) * slab_rows + t;
            v[j] = ptx::ld_global_v4(in + r * cols + c * 8);
          }
        }
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          if (j0 + j < cnt) {
            const uint32_t w[4] = {v[j].x, v[j].y, v[j].z, v[j].w};
#pragma unroll
            for (int e = 0; e < 4; ++e) {
              acc[2 * e] += ptx::half_bits_to_float(static_cast<uint16_t>(w[e] & 0xFFFFu), h);
              acc[2 * e + 1] += ptx::half_bits_to_float(static_cast<uint16_t>(w[e] >> 16), h);
            }
          }
        }
      }
      uint4 o;
      o.x = ptx::pack_half2(h, acc[0], acc[1]);
      o.y = ptx::pack_half2(h, acc[2], acc[3]);
      o.z = ptx::pack_half2(h, acc[4], acc[5]);
      o.w = ptx::pack_half2(h, acc[6], acc[7]);
      *reinterpret_cast<uint4*>(out + t * cols + c * 8) = o;
    }
  }
}

// ----------------------------------------------------------------------------------------
// bitwise compare / uniform fill / copy
// ----------------------------------------------------------------------------------------
__global__ void bitwise_check_kernel(const uint8_t* a, const uint8_t* b, int64_t nbytes,
                                     unsigned long long* mismatches) {
  const int64_t stride = static_cast<int64_t>(gridDim.x) * blockDim.x;
  const int64_t tid = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  unsigned long long local = 0;
  const int64_t n16 = (((reinterpret_cast<uintptr_t>(a) | reinterpret_cast<uintptr_t>(b)) & 15) == 0)
                          ? nbytes / 16 : 0;
  const uint4* a4 = reinterpret_cast<const uint4*>(a);
  const uint4* b4 = reinterpret_cast<const uint4*>(b);
  for (int64_t i = tid; i < n16; i += stride) {
    const uint4 x = a4[i], y = b4[i];
    local += (x.x != y.x) + (x.y != y.y) + (x.z != y.z) + (x.w != y.w);
  }
  for (int64_t i = n16 * 16 + tid; i < nbytes; i += stride) local += a[i] != b[i];
  for (int o = 16; o > 0; o >>= 1) local += __shfl_xor_sync(0xffffffffu, local, o);
  if ((threadIdx.x & 31) == 0 && local) atomicAdd(mismatches, local);
}

__device__ __forceinline__ uint32_t hash32(uint64_t x) {
  x ^= x >> 33; x *= 0xff51afd7ed558ccdull; x ^= x >> 33; x *= 0xc4ceb9fe1a85ec53ull; x ^= x >> 33;
  return static_cast<uint32_t>(x);
}

template <typename T>
__device__ __forceinline__ T from_f32(float v);
template <> __device__ __forceinline__ float from_f32<float>(float v) { return v; }
template <> __device__ __forceinline__ __nv_bfloat16 from_f32<__nv_bfloat16>(float v) { return __float2bfloat16_rn(v); }
template <> __device__ __forceinline__ __half from_f32<__half>(float v) { return __float2half_rn(v); }

template <typename T>
__global__ void uniform_fill_kernel(T* out, int64_t n, uint64_t seed, float lo, float hi) {
  const int64_t stride = static_cast<int64_t>(gridDim.x) * blockDim.x;
  for (int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < n; i += stride) {
    const float u = (hash32(seed * 0x9E3779B97F4A7C15ull + i) >> 8) * (1.0f / 16777216.0f);
    out[i] = from_f32<T>(lo + (hi - lo) * u);
  }
}

__global__ void copy_bytes_kernel(uint8_t* dst, const uint8_t* src, int64_t nbytes) {
  const int64_t stride = static_cast<int64_t>(gridDim.x) * blockDim.x;
  const int64_t tid = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  const bool al = ((reinterpret_cast<uintptr_t>(dst) | reinterpret_cast<uintptr_t>(src)) & 15) == 0;
  const int64_t n16 = al ? nbytes / 16 : 0;
  for (int64_t i = tid; i < n16; i += stride)
    reinterpret_cast<uint4*>(dst)[i] = reinterpret_cast<const uint4*>(src)[i];
  for (int64_t i = n16 * 16 + tid; i < nbytes; i += stride) dst[i] = src[i];
}

// ----------------------------------------------------------------------------------------
// MoE routing index build: a stable counting sort of the flattened expert choices.
//   experts[n]        expert id of flattened (token, k) entry n, n = token * topk + k
//   splits[e]         number of entries routed to expert e
//   offsets[e]        exclusive prefix sum of splits (E + 1 entries)
//   scatter_index[n]  row of entry n in the expert-sorted order (stable inside an expert)
//   gather_index[r]   token of sorted row r          topk_index[r]   k of sorted row r
// Three passes: per-block histograms, one-block scan, stable placement.
// ----------------------------------------------------------------------------------------
constexpr int kIdxThreads = 256;
constexpr int kIdxPerBlock = 4096;
constexpr int kMaxExperts = 512;

__global__ void __launch_bounds__(kIdxThreads) moe_hist_kernel(const int32_t* experts, int64_t n,
                                                               int E, int32_t* block_hist) {
  extern __shared__ int32_t hist[];
  for (int e = threadIdx.x; e < E; e += kIdxThreads) hist[e] = 0;
  __syncthreads();
  const int64_t base = static_cast<int64_t>(blockIdx.x) * kIdxPerBlock;
  for (int i = threadIdx.x; i < kIdxPerBlock; i += kIdxThreads) {
    const int64_t idx = base + i;
    if (idx < n) {
      const int e = experts[idx];
      if (e >= 0 && e < E) atomicAdd(&hist[e], 1);
    }
  }
  __syncthreads();
  for (int e = threadIdx.x; e < E; e += kIdxThreads) block_hist[blockIdx.x * E + e] = hist[e];
}

// block_hist[b][e] -> exclusive start of (expert e, block b); splits; offsets
__global__ void __launch_bounds__(kMaxExperts) moe_scan_kernel(int32_t* block_hist, int nblocks, int E,
                                                               int32_t* splits, int32_t* offsets) {
  __shared__ int32_t totals[kMaxExperts];
  const int e = threadIdx.x;
  int32_t total = 0;
  if (e < E) {
    for (int b = 0; b < nblocks; ++b) {
      const int32_t c = block_hist[b * E + e];
      block_hist[b * E + e] = total;  // exclusive count of expert e in earlier blocks
      total += c;
    }
    totals[e] = total;
    if (splits) splits[e] = total;
  }
  __syncthreads();
  if (e == 0) {
    int32_t run = 0;
    for (int i = 0; i < E; ++i) {
      const int32_t c = totals[i];
      totals[i] = run;
      offsets[i] = run;
      run += c;
    }
    offsets[E] = run;
  }
  __syncthreads();
  if (e < E) {
    const int32_t start = totals[e];
    for (int b = 0; b < nblocks; ++b) block_hist[b * E + e] += start;
  }
}

__global__ void __launch_bounds__(kIdxThreads) moe_place_kernel(
    const int32_t* experts, int64_t n, int E, int topk, const int32_t* block_start,
    int32_t* scatter_index, int32_t* gather_index, int32_t* topk_index) {
  // running[e]: next free row of expert e for this block; warps are served in order and lanes in
  // order inside a warp, so equal experts keep their input order
  extern __shared__ int32_t running[];
  for (int e = threadIdx.x; e < E; e += kIdxThreads) running[e] = block_start[blockIdx.x * E + e];
  __syncthreads();
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int64_t base = static_cast<int64_t>(blockIdx.x) * kIdxPerBlock;
  for (int step = 0; step < kIdxPerBlock / kIdxThreads; ++step) {
    const int64_t idx = base + step * kIdxThreads + threadIdx.x;
    int e = -1;
    if (idx < n) {
      e = experts[idx];
      if (e < 0 || e >= E) e = -1;
    }
    const unsigned peers = __match_any_sync(0xffffffffu, e);
    const int rank_in_warp = __popc(peers & ((1u << lane) - 1u));
    const int leader = __ffs(peers) - 1;
    for (int w = 0; w < kIdxThreads / 32; ++w) {
      if (w == warp && e >= 0) {
        int start = 0;
        if (lane == leader) {
          start = running[e];
          running[e] = start + __popc(peers);
        }
        start = __shfl_sync(peers, start, leader);
        const int32_t row = start + rank_in_warp;
        scatter_index[idx] = row;
        if (gather_index) gather_index[row] = static_cast<int32_t>(idx / topk);
        if (topk_index) topk_index[row] = static_cast<int32_t>(idx % topk);
      }
      __syncthreads();
    }
  }
}

}  // namespace
}  // namespace fluxb

using namespace fluxb;

extern "C" int fluxb_inplace_cast_fp32_to_bf16(float* data, int64_t n, uint32_t* flags,
                                               uint32_t* claim, uint32_t epoch, uint64_t timeout_ns,
                                               fluxb_status_t* status, void* stream) {
  FLUXB_REQUIRE(data && flags && claim && n > 0, "inplace cast arguments");
  FLUXB_REQUIRE((reinterpret_cast<uintptr_t>(data) & 15) == 0, "buffer must be 16-byte aligned");
  int sms = 0, rc;
  if ((rc = device_sm_count(&sms))) return rc;
  const int64_t chunks = (n + kChunk - 1) / kChunk;
  // every chunk waits on a lower-numbered one, so all claiming CTAs must be resident at once
  const int grid = static_cast<int>(chunks < sms * 4 ? chunks : sms * 4);
  inplace_cast_kernel<<<grid, kCastThreads, 0, reinterpret_cast<cudaStream_t>(stream)>>>(
      data, n, flags, claim, epoch, timeout_ns ? timeout_ns : 2000000000ull,
      reinterpret_cast<Status*>(status));
  FLUXB_CUDA_OK(cudaGetLastError());
  g_launches.fetch_add(1, std::memory_order_relaxed);
  return kOk;
}

extern "C" int fluxb_rows_sum(const void* in, const int32_t* idx, void* out, int64_t rows_out, int cols, int cnt,
                              int64_t slab_rows, int dtype, void* stream) {
  FLUXB_REQUIRE(in && out && rows_out >= 0 && cnt >= 1, "rows_sum arguments");
  FLUXB_REQUIRE(cols > 0 && cols % 8 == 0, "rows must be multiples of 8 elements (16 bytes)");
  FLUXB_REQUIRE(dtype == FLUXB_BF16 || dtype == FLUXB_FP16, "rows_sum runs on bf16 / fp16");
  FLUXB_REQUIRE(((reinterpret_cast<uintptr_t>(in) | reinterpret_cast<uintptr_t>(out)) & 15) == 0,
                "buffers must be 16-byte aligned");
  if (rows_out == 0) return kOk;
  int sms = 0, rc;
  if ((rc = device_sm_count(&sms))) return rc;
  int64_t blocks = (rows_out + 7) / 8;
  if (blocks > sms * 8) blocks = sms * 8;
  rows_sum_kernel<<<static_cast<int>(blocks), 256, 0, reinterpret_cast<cudaStream_t>(stream)>>>(
      reinterpret_cast<const uint16_t*>(in), idx, reinterpret_cast<uint16_t*>(out), rows_out, cols, cnt, slab_rows,
      dtype == FLUXB_FP16);
  FLUXB_CUDA_OK(cudaGetLastError());
  g_launches.fetch_add(1, std::memory_order_relaxed);
  return kOk;
}

extern "C" int fluxb_bitwise_check(const void* a, const void* b, int64_t nbytes,
                                   unsigned long long* mismatches, void* stream) {
  FLUXB_REQUIRE(a && b && mismatches && nbytes >= 0, "bitwise check arguments");
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
  FLUXB_CUDA_OK(cudaMemsetAsync(mismatches, 0, sizeof(unsigned long long), s));
  if (nbytes == 0) return kOk;
  int sms = 0, rc;
  if ((rc = device_sm_count(&sms))) return rc;
  bitwise_check_kernel<<<sms * 8, 256, 0, s>>>(reinterpret_cast<const uint8_t*>(a),
                                               reinterpret_cast<const uint8_t*>(b), nbytes, mismatches);
  FLUXB_CUDA_OK(cudaGetLastError());
  g_launches.fetch_add(1, std::memory_order_relaxed);
  return kOk;
}

extern "C" int fluxb_uniform_fill(void* out, int64_t n, int dtype, uint64_t seed, float lo, float hi,
                                  void* stream) {
  FLUXB_REQUIRE(out && n >= 0, "uniform fill arguments");
  if (n == 0) return kOk;
  int sms = 0, rc;
  if ((rc = device_sm_count(&sms))) return rc;
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
  switch (dtype) {
    case FLUXB_FP32: uniform_fill_kernel<float><<<sms * 8, 256, 0, s>>>(static_cast<float*>(out), n, seed, lo, hi); break;
    case FLUXB_BF16:
      uniform_fill_kernel<__nv_bfloat16><<<sms * 8, 256, 0, s>>>(static_cast<__nv_bfloat16*>(out), n, seed, lo, hi);
      break;
    case FLUXB_FP16: uniform_fill_kernel<__half><<<sms * 8, 256, 0, s>>>(static_cast<__half*>(out), n, seed, lo, hi); break;
    default: return fail(kErrUnsupported, "uniform fill supports fp32, bf16, fp16");
  }
  FLUXB_CUDA_OK(cudaGetLastError());
  g_launches.fetch_add(1, std::memory_order_relaxed);
  return kOk;
}

extern "C" int fluxb_copy_bytes(void* dst, const void* src, int64_t nbytes, void* stream) {
  FLUXB_REQUIRE(dst && src && nbytes >= 0, "copy arguments");
  if (nbytes == 0) return kOk;
  int sms = 0, rc;
  if ((rc = device_sm_count(&sms))) return rc;
  copy_bytes_kernel<<<sms * 8, 256, 0, reinterpret_cast<cudaStream_t>(stream)>>>(
      static_cast<uint8_t*>(dst), static_cast<const uint8_t*>(src), nbytes);
  FLUXB_CUDA_OK(cudaGetLastError());
  g_launches.fetch_add(1, std::memory_order_relaxed);
  return kOk;
}

// scratch: int32 workspace of at least fluxb_moe_index_scratch_elems(n, E) elements
extern "C" int64_t fluxb_moe_index_scratch_elems(int64_t n, int E) {
  return ((n + kIdxPerBlock - 1) / kIdxPerBlock) * E;
}

extern "C" int fluxb_moe_index_build(const int32_t* experts, int64_t n, int E, int topk,
                                     int32_t* splits, int32_t* offsets, int32_t* scatter_index,
                                     int32_t* gather_index, int32_t* topk_index, int32_t* scratch,
                                     void* stream) {
  FLUXB_REQUIRE(experts && offsets && scatter_index && scratch, "moe index arguments");
  FLUXB_REQUIRE(E >= 1 && E <= kMaxExperts && topk >= 1 && n > 0, "moe index sizes");
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
  const int nblocks = static_cast<int>((n + kIdxPerBlock - 1) / kIdxPerBlock);
  moe_hist_kernel<<<nblocks, kIdxThreads, E * sizeof(int32_t), s>>>(experts, n, E, scratch);
  moe_scan_kernel<<<1, kMaxExperts, 0, s>>>(scratch, nblocks, E, splits, offsets);
  moe_place_kernel<<<nblocks, kIdxThreads, E * sizeof(int32_t), s>>>(
      experts, n, E, topk, scratch, scatter_index, gather_index, topk_index);
  FLUXB_CUDA_OK(cudaGetLastError());
  g_launches.fetch_add(3, std::memory_order_relaxed);
  return kOk;
}

// ----------------------------------------------------------------------------------------
// Routing-index build without any allocation (see moe_index_static.h). The per-block histogram
// scratch is this fixed array. In host code `g_moe_index_static` only names the symbol; the
// address a kernel can use comes from cudaGetSymbolAddress, looked up once per device.
// ----------------------------------------------------------------------------------------
#include "moe_index_static.h"

static __device__ __align__(256) int32_t g_moe_index_static[FLUXB_MOE_INDEX_STATIC_ELEMS];

extern "C" int fluxb_moe_index_build_static(const int32_t* experts, int64_t n, int E, int topk,
                                            int32_t* splits, int32_t* offsets,
                                            int32_t* scatter_index, int32_t* gather_index,
                                            int32_t* topk_index, void* stream) {
  FLUXB_REQUIRE(experts && offsets && scatter_index, "moe index arguments");
  FLUXB_REQUIRE(E >= 1 && E <= kMaxExperts && topk >= 1 && n > 0, "moe index sizes");
  const int64_t nblocks64 = (n + kIdxPerBlock - 1) / kIdxPerBlock;
  if (nblocks64 * E > FLUXB_MOE_INDEX_STATIC_ELEMS)
    return fail(kErrInvalid,
                "fluxb_moe_index_build_static: ceil(n/4096)*E = " + std::to_string(nblocks64 * E) +
                    " exceeds the built-in scratch of " + std::to_string(FLUXB_MOE_INDEX_STATIC_ELEMS) +
                    " int32; use fluxb_moe_index_build with a caller-provided scratch buffer");
  // set-up, once per device, with that device current. The cache is atomic: two host threads that
  // make their first call on a device at the same time both look the address up and store the same
  // value.
  static std::atomic<int32_t*> scratch_of_device[64];
  int dev = 0;
  FLUXB_CUDA_OK(cudaGetDevice(&dev));
  FLUXB_REQUIRE(dev >= 0 && dev < 64, "device ordinal out of range");
  int32_t* scratch = scratch_of_device[dev].load(std::memory_order_relaxed);
  if (scratch == nullptr) {
    void* addr = nullptr;
    cudaError_t e = cudaGetSymbolAddress(&addr, g_moe_index_static);
    if (e != cudaSuccess)
      return fail(kErrCuda, std::string("cudaGetSymbolAddress(g_moe_index_static): ") + cudaGetErrorString(e));
    scratch = static_cast<int32_t*>(addr);
    scratch_of_device[dev].store(scratch, std::memory_order_relaxed);
  }
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
  const int nblocks = static_cast<int>(nblocks64);
  moe_hist_kernel<<<nblocks, kIdxThreads, E * sizeof(int32_t), s>>>(experts, n, E, scratch);
  moe_scan_kernel<<<1, kMaxExperts, 0, s>>>(scratch, nblocks, E, splits, offsets);
  moe_place_kernel<<<nblocks, kIdxThreads, E * sizeof(int32_t), s>>>(
      experts, n, E, topk, scratch, scatter_index, gather_index, topk_index);
  FLUXB_CUDA_OK(cudaGetLastError());
  g_launches.fetch_add(3, std::memory_order_relaxed);
  return kOk;
}
