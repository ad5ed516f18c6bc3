// Row exchange between the ranks of a node over peer memory: variable-split all-to-all and
// all-gather in one kernel, plus the host-initiated signal helpers of the send/recv op.
// Split sizes stay on the device: every rank first publishes its split vector into every peer's
// table, then computes from the complete W x W table where its rows start in each destination.
// Reference: src/coll/all2all_impl.cu (NVSHMEM put + signal), src/coll/all2all_single_2d_impl.cu,
// src/coll/ths_op/all_gather_op.cc, src/coll/ths_op/isendrecv.cc.
#include "../include/fluxb.h"
#include "../runtime/host_common.h"
#include "../sm100/ptx.cuh"

#include <atomic>

namespace fluxb {
extern std::atomic<uint64_t> g_launches;
namespace {

constexpr int kR = FLUXB_MAX_RANKS;

struct A2AParams {
  const uint8_t* in;
  const int32_t* in_splits;      // [W] rows sent to each destination (null when broadcast)
  int32_t rows_in;               // broadcast: rows sent to every destination
  int32_t broadcast;
  int64_t row_bytes;             // multiple of 16
  int32_t rank, world;
  uint32_t epoch;
  uint64_t timeout_ns;
  Status* status;
  uint8_t* out[kR];              // destination buffer of every rank
  int32_t* table[kR];            // on every rank: [W src][W dst] row counts
  uint32_t* flags[kR];           // on every rank: [0..W) table row of src present, [W..2W) data of src landed
  uint32_t* local_cnt;           // [W]
  int32_t* out_splits;           // optional [W]: rows received from each source
  int32_t* out_offsets;          // optional [W + 1]: where each source's rows start in the output
  int64_t out_capacity_rows;
};

__global__ void __launch_bounds__(256) a2a_rows_kernel(const __grid_constant__ A2AParams p) {
  __shared__ uint32_t abort_word;
  __shared__ int32_t s_cnt[kR][kR];
  if (threadIdx.x == 0) abort_word = 0;
  __syncthreads();
  WaitCtx wc{p.status, &abort_word, p.timeout_ns};
  const int W = p.world, lane = threadIdx.x & 31;
  // ---- phase 0: publish this rank's split vector everywhere
  if (blockIdx.x == 0 && threadIdx.x < W) {
    const int d = threadIdx.x;
    for (int j = 0; j < W; ++j) p.table[d][p.rank * W + j] = p.broadcast ? p.rows_in : p.in_splits[j];
    __threadfence_system();
    ptx::st_release_sys(p.flags[d] + p.rank, p.epoch);
  }
  // ---- phase 1: read the complete table
  if (threadIdx.x < W) flag_wait_ge(wc, p.flags[p.rank] + threadIdx.x, p.epoch, kSiteA2AFlag);
  __syncthreads();
  if (threadIdx.x < W * W) s_cnt[threadIdx.x / W][threadIdx.x % W] = p.table[p.rank][threadIdx.x];
  __syncthreads();
  if (blockIdx.x == 0 && threadIdx.x == 0) {
    int run = 0;
    for (int s = 0; s < W; ++s) {
      if (p.out_splits) p.out_splits[s] = s_cnt[s][p.rank];
      if (p.out_offsets) p.out_offsets[s] = run;
      run += s_cnt[s][p.rank];
    }
    if (p.out_offsets) p.out_offsets[W] = run;
  }
  // ---- phase 2: copy my rows into each destination, nearest rank first
  const int64_t chunks_per_row = p.row_bytes >> 4;
  for (int step = 0; step < W; ++step) {
    int d = p.rank + step;
    if (d >= W) d -= W;
    int64_t src_row = 0;
    if (!p.broadcast)
      for (int j = 0; j < d; ++j) src_row += s_cnt[p.rank][j];
    int64_t dst_row = 0;
    for (int s = 0; s < p.rank; ++s) dst_row += s_cnt[s][d];
    int64_t rows = s_cnt[p.rank][d];
    if (dst_row + rows > p.out_capacity_rows) {
      rows = p.out_capacity_rows - dst_row;
      if (rows < 0) rows = 0;
    }
    const uint4* src = reinterpret_cast<const uint4*>(p.in + src_row * p.row_bytes);
    uint4* dst = reinterpret_cast<uint4*>(p.out[d] + dst_row * p.row_bytes);
    const int64_t n = rows * chunks_per_row;
    // eight 16-byte pieces per thread in flight, a warp's pieces of one round contiguous (512 B)
    constexpr int kU = 8;
    for (int64_t i = static_cast<int64_t>(blockIdx.x) * 256 * kU + threadIdx.x; i < n;
         i += static_cast<int64_t>(gridDim.x) * 256 * kU) {
      uint4 v[kU];
#pragma unroll
      for (int u = 0; u < kU; ++u)
        if (i + u * 256 < n) v[u] = ptx::ld_global_v4(src + i + u * 256);
#pragma unroll
      for (int u = 0; u < kU; ++u)
        if (i + u * 256 < n) ptx::st_global_v4(dst + i + u * 256, v[u]);
    }
    __syncthreads();
    if (threadIdx.x == 0) {
      uint32_t* cnt = p.local_cnt + step;
      if (ptx::atom_add_acq_rel_sys(cnt, 1u) == gridDim.x - 1u) {
        *cnt = 0;
        ptx::st_release_sys(p.flags[d] + W + p.rank, p.epoch);
      }
    }
  }
  // ---- phase 3: stay until everything addressed to this rank has landed
  if (threadIdx.x < W) flag_wait_ge(wc, p.flags[p.rank] + W + threadIdx.x, p.epoch, kSiteA2AFlag);
  __syncthreads();
  (void)lane;
}

// ---- strided exchange: the stand-alone all-to-all (+ transpose) of the Ulysses ops ------------
// For every destination rank up to kMaxCopies copy descriptors: a 3-D grid of items of `vec_bytes`
// contiguous bytes, each with its own byte strides on the source (local) and the destination (that
// rank's buffer) side. One kernel covers seq->heads, heads->seq, packed q/k/v with grouped heads
// and per-rank sequence lengths: only the descriptors differ.
// Reference: src/gemm_a2a_transpose/pre_attn_a2a_transpose_impls.cu,
// pre_attn_qkv_pack_a2a_impls.cu (pull kernels) and src/a2a_transpose_gemm/
// post_attn_a2a_transpose_impls.cu (push kernels, fixed and dynamic sequence lengths).
constexpr int kMaxCopies = 3;

struct StridedCopy {
  const uint8_t* src;
  uint8_t* dst;
  int32_t n0, n1, n2, vec_bytes;      // vec_bytes: multiple of 16
  int64_t ss0, ss1, ss2, ds0, ds1, ds2;
};

struct ExchangeParams {
  StridedCopy copy[kR][kMaxCopies];   // [destination][group]
  int32_t ncopies;
  int32_t rank, world;
  uint32_t epoch;
  uint64_t timeout_ns;
  Status* status;
  uint32_t* flags[kR];                // on every rank: [W src] last call whose data has landed
  uint32_t* start_ctr[kR];
  uint32_t* local_cnt;                // [W]
};

__global__ void __launch_bounds__(256) strided_exchange_kernel(const __grid_constant__ ExchangeParams p) {
  __shared__ uint32_t abort_word;
  if (threadIdx.x == 0) abort_word = 0;
  __syncthreads();
  WaitCtx wc{p.status, &abort_word, p.timeout_ns};
  const int W = p.world;
  // nobody writes into a peer before that peer has entered this call
  if (blockIdx.x == 0 && threadIdx.x < W) ptx::st_release_sys(p.start_ctr[threadIdx.x] + p.rank, p.epoch);
  if (threadIdx.x < W) flag_wait_ge(wc, p.start_ctr[p.rank] + threadIdx.x, p.epoch, kSiteStartBarrier);
  __syncthreads();
  for (int step = 1; step <= W; ++step) {     // nearest peer first, the own part last
    int d = p.rank + step;
    if (d >= W) d -= W;
    for (int g = 0; g < p.ncopies; ++g) {
      const StridedCopy& c = p.copy[d][g];
      const int64_t per_item = c.vec_bytes >> 4;
      const int64_t n = static_cast<int64_t>(c.n0) * c.n1 * c.n2 * per_item;
      constexpr int kU = 4;
      for (int64_t i = static_cast<int64_t>(blockIdx.x) * 256 * kU + threadIdx.x; i < n;
           i += static_cast<int64_t>(gridDim.x) * 256 * kU) {
        uint4 v[kU];
        int64_t doff[kU];
#pragma unroll
        for (int u = 0; u < kU; ++u) {
          const int64_t j = i + u * 256;
          if (j < n) {
            const int64_t item = j / per_item, piece = j - item * per_item;
            const int64_t i2 = item % c.n2, r = item / c.n2;
            const int64_t i1 = r % c.n1, i0 = r / c.n1;
            v[u] = ptx::ld_global_v4(c.src + i0 * c.ss0 + i1 * c.ss1 + i2 * c.ss2 + piece * 16);
            doff[u] = i0 * c.ds0 + i1 * c.ds1 + i2 * c.ds2 + piece * 16;
          }
        }
#pragma unroll
        for (int u = 0; u < kU; ++u)
          if (i + u * 256 < n) ptx::st_global_v4(c.dst + doff[u], v[u]);
      }
    }
    ptx::fence_acq_rel_sys();
    __syncthreads();
    if (threadIdx.x == 0) {
      uint32_t* cnt = p.local_cnt + (step % W);
      if (ptx::atom_add_acq_rel_sys(cnt, 1u) == gridDim.x - 1u) {
        *cnt = 0;
        ptx::st_release_sys(p.flags[d] + p.rank, p.epoch);
      }
    }
  }
  if (threadIdx.x < W) flag_wait_ge(wc, p.flags[p.rank] + threadIdx.x, p.epoch, kSiteA2AFlag);
  __syncthreads();
}

__global__ void set_flag_kernel(uint32_t* flag, uint32_t value) {
  __threadfence_system();
  ptx::st_release_sys(flag, value);
}

}  // namespace
}  // namespace fluxb

using namespace fluxb;

extern "C" int fluxb_a2a_rows(const fluxb_a2a_rows_args_t* a) {
  FLUXB_REQUIRE(a != nullptr && a->in != nullptr, "a2a arguments");
  FLUXB_REQUIRE(a->world >= 1 && a->world <= kR && a->rank >= 0 && a->rank < a->world, "ranks");
  FLUXB_REQUIRE(a->row_bytes > 0 && a->row_bytes % 16 == 0, "row size must be a multiple of 16 bytes");
  FLUXB_REQUIRE(a->broadcast || a->in_splits != nullptr, "split vector missing");
  A2AParams p;
  memset(&p, 0, sizeof(p));
  p.in = reinterpret_cast<const uint8_t*>(a->in);
  p.in_splits = a->in_splits;
  p.rows_in = a->rows_in;
  p.broadcast = a->broadcast;
  p.row_bytes = a->row_bytes;
  p.rank = a->rank;
  p.world = a->world;
  p.epoch = a->epoch;
  p.timeout_ns = a->timeout_ns ? a->timeout_ns : 5000000000ull;
  p.status = reinterpret_cast<Status*>(a->status);
  p.local_cnt = a->local_cnt;
  p.out_splits = a->out_splits;
  p.out_offsets = a->out_offsets;
  p.out_capacity_rows = a->out_capacity_rows;
  FLUXB_REQUIRE(a->local_cnt != nullptr, "local arrival scratch missing");
  for (int r = 0; r < a->world; ++r) {
    FLUXB_REQUIRE(a->out[r] && a->table[r] && a->flags[r], "peer pointers missing");
    p.out[r] = reinterpret_cast<uint8_t*>(a->out[r]);
    p.table[r] = a->table[r];
    p.flags[r] = a->flags[r];
  }
  int sms = 0, rc;
  if ((rc = device_sm_count(&sms))) return rc;
  int grid = a->num_ctas > 0 ? a->num_ctas : 128;
  if (grid > sms) grid = sms;  // all CTAs must be resident: they count arrivals together
  a2a_rows_kernel<<<grid, 256, 0, reinterpret_cast<cudaStream_t>(a->stream)>>>(p);
  FLUXB_CUDA_OK(cudaGetLastError());
  g_launches.fetch_add(1, std::memory_order_relaxed);
  return kOk;
}

extern "C" int fluxb_strided_exchange(const fluxb_strided_exchange_args_t* a) {
  FLUXB_REQUIRE(a != nullptr && a->local_cnt != nullptr, "exchange arguments");
  FLUXB_REQUIRE(a->world >= 1 && a->world <= kR && a->rank >= 0 && a->rank < a->world, "ranks");
  FLUXB_REQUIRE(a->ncopies >= 1 && a->ncopies <= kMaxCopies, "1..3 copies per destination");
  ExchangeParams p;
  memset(&p, 0, sizeof(p));
  p.ncopies = a->ncopies;
  p.rank = a->rank;
  p.world = a->world;
  p.epoch = a->epoch;
  p.timeout_ns = a->timeout_ns ? a->timeout_ns : 5000000000ull;
  p.status = reinterpret_cast<Status*>(a->status);
  p.local_cnt = a->local_cnt;
  for (int r = 0; r < a->world; ++r) {
    FLUXB_REQUIRE(a->flags[r] && a->start_ctr[r], "peer pointers missing");
    p.flags[r] = a->flags[r];
    p.start_ctr[r] = a->start_ctr[r];
    for (int g = 0; g < a->ncopies; ++g) {
      const fluxb_strided_copy_t& c = a->copy[r][g];
      const bool empty = c.n0 == 0 || c.n1 == 0 || c.n2 == 0;
      FLUXB_REQUIRE(empty || (c.src && c.dst), "copy pointers missing");
      FLUXB_REQUIRE(c.n0 >= 0 && c.n1 >= 0 && c.n2 >= 0 && c.vec_bytes > 0 && c.vec_bytes % 16 == 0,
                    "copy extents / item size (multiple of 16 bytes)");
      FLUXB_REQUIRE(((reinterpret_cast<uintptr_t>(c.src) | reinterpret_cast<uintptr_t>(c.dst) | c.ss0 | c.ss1 |
                      c.ss2 | c.ds0 | c.ds1 | c.ds2) & 15) == 0,
                    "copy addresses and strides must be multiples of 16 bytes");
      StridedCopy& o = p.copy[r][g];
      o.src = reinterpret_cast<const uint8_t*>(c.src);
      o.dst = reinterpret_cast<uint8_t*>(c.dst);
      o.n0 = c.n0; o.n1 = c.n1; o.n2 = c.n2; o.vec_bytes = c.vec_bytes;
      o.ss0 = c.ss0; o.ss1 = c.ss1; o.ss2 = c.ss2; o.ds0 = c.ds0; o.ds1 = c.ds1; o.ds2 = c.ds2;
    }
  }
  int sms = 0, rc;
  if ((rc = device_sm_count(&sms))) return rc;
  int grid = a->num_ctas > 0 ? a->num_ctas : 96;
  if (grid > sms) grid = sms;  // all CTAs must be resident: they count arrivals together
  strided_exchange_kernel<<<grid, 256, 0, reinterpret_cast<cudaStream_t>(a->stream)>>>(p);
  FLUXB_CUDA_OK(cudaGetLastError());
  g_launches.fetch_add(1, std::memory_order_relaxed);
  return kOk;
}

extern "C" int fluxb_set_flag(uint32_t* flag, uint32_t value, void* stream) {
  FLUXB_REQUIRE(flag != nullptr, "flag pointer");
  set_flag_kernel<<<1, 1, 0, reinterpret_cast<cudaStream_t>(stream)>>>(flag, value);
  FLUXB_CUDA_OK(cudaGetLastError());
  g_launches.fetch_add(1, std::memory_order_relaxed);
  return kOk;
}
