// Expert-parallel token dispatch over peer memory: every rank sends each of its token rows only
// to the ranks that own one of the token's top-k experts, straight into the row's place in the
// receiver's expert-sorted buffer. One warp per (token, k) entry copies the row with 16-byte
// loads and peer stores; the last CTA of a source tells every receiver, and every rank stays
// until all sources have told it, so when the kernel completes the local buffer holds all rows
// of this rank's experts.
// Reference: src/coll/dis_scatter_forward_impl.cu (dis_scatter_forward_*_kernel: NVSHMEM
// putmem_nbi_warp per routed row + signals, hierarchical across nodes). Here one NVSwitch domain:
// plain peer stores, call-number flags, bounded waits.
#include "../include/fluxb.h"
#include "../runtime/host_common.h"
#include "../sm100/ptx.cuh"

#include <atomic>

namespace fluxb {
extern std::atomic<uint64_t> g_launches;
namespace {

constexpr int kR = FLUXB_MAX_RANKS;
constexpr int kMaxE = 512;

struct DispatchParams {
  const uint8_t* x;              // [tokens_local, row_bytes] this rank's tokens
  const int32_t* scatter_index;  // [tokens_total * topk] sorted row of every (token, k), all ranks' tokens
  const int32_t* splits;         // [E] rows per expert
  int64_t token0;                // global index of this rank's first token
  int32_t tokens_local, topk, E, E_local, tp;   // tp: ranks that share one group of experts
  int64_t row_bytes;             // multiple of 16
  int64_t capacity_rows;         // rows each receive buffer can hold
  int32_t rank, world;
  uint32_t epoch;
  uint64_t timeout_ns;
  Status* status;
  uint8_t* out[kR];              // receive buffer of every rank: [capacity_rows][row_bytes]
  uint32_t* flags[kR];           // on every rank: [W src] last call whose rows have all landed
  uint32_t* start_ctr[kR];
  uint32_t* local_cnt;           // [1]
  int32_t* out_rows;             // optional [1]: rows this rank received (sum of its experts' splits)
};

__global__ void __launch_bounds__(256) ep_dispatch_kernel(const __grid_constant__ DispatchParams p) {
  __shared__ uint32_t abort_word;
  __shared__ int32_t s_base[kR + 1];   // first sorted row of every expert group
  if (threadIdx.x == 0) {
    abort_word = 0;
    const int groups = p.world / p.tp;
    int run = 0, g = 0;
    for (int e = 0; e < p.E; ++e) {
      if (e == g * p.E_local) s_base[g++] = run;
      run += p.splits[e];
    }
    while (g <= groups) s_base[g++] = run;
    if (blockIdx.x == 0 && p.out_rows != nullptr) {
      const int mine = p.rank / p.tp;
      *p.out_rows = s_base[mine + 1] - s_base[mine];
    }
  }
  __syncthreads();
  WaitCtx wc{p.status, &abort_word, p.timeout_ns};
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int groups = p.world / p.tp;
  // nobody writes into a receiver before that receiver has entered this call (its buffer of the
  // previous call is consumed by then)
  if (blockIdx.x == 0 && threadIdx.x < p.world) ptx::st_release_sys(p.start_ctr[threadIdx.x] + p.rank, p.epoch);
  if (lane < p.world) flag_wait_ge(wc, p.start_ctr[p.rank] + lane, p.epoch, kSiteStartBarrier);
  __syncwarp();

  const int64_t entries = static_cast<int64_t>(p.tokens_local) * p.topk;
  const int64_t chunks = p.row_bytes >> 4;
  const int64_t gwarp = static_cast<int64_t>(blockIdx.x) * 8 + warp, nwarps = static_cast<int64_t>(gridDim.x) * 8;
  for (int64_t i = gwarp; i < entries; i += nwarps) {
    const int64_t tl = i / p.topk;
    const int r = p.scatter_index[(p.token0 + tl) * p.topk + (i - tl * p.topk)];
    int g = 0;
    while (g + 1 < groups && r >= s_base[g + 1]) ++g;
    const int64_t drow = r - s_base[g];
    if (drow >= p.capacity_rows) {
      // more rows routed to one rank than its buffer holds: report, drop the row
      if (lane == 0) wait_give_up(wc, kSiteCapacity, static_cast<uint32_t>(drow), static_cast<uint32_t>(p.capacity_rows));
      continue;
    }
    const uint4* src = reinterpret_cast<const uint4*>(p.x + tl * p.row_bytes);
    // every rank of the expert group gets the row
    for (int j = 0; j < p.tp; ++j) {
      uint4* dst = reinterpret_cast<uint4*>(p.out[g * p.tp + j] + drow * p.row_bytes);
      for (int64_t c = lane; c < chunks; c += 128) {
        uint4 v[4];
#pragma unroll
        for (int u = 0; u < 4; ++u)
          if (c + 32 * u < chunks) v[u] = ptx::ld_global_v4(src + c + 32 * u);
#pragma unroll
        for (int u = 0; u < 4; ++u)
          if (c + 32 * u < chunks) ptx::st_global_v4(dst + c + 32 * u, v[u]);
      }
    }
  }
  // all rows of this CTA are written: the last CTA tells every receiver
  ptx::fence_acq_rel_sys();
  __syncthreads();
  if (threadIdx.x == 0) {
    if (ptx::atom_add_acq_rel_sys(p.local_cnt, 1u) == gridDim.x - 1u) {
      *p.local_cnt = 0;
      for (int d = 0; d < p.world; ++d) ptx::st_release_sys(p.flags[d] + p.rank, p.epoch);
    }
  }
  if (threadIdx.x < p.world) flag_wait_ge(wc, p.flags[p.rank] + threadIdx.x, p.epoch, kSiteMoeFlag);
  __syncthreads();
}

}  // namespace
}  // namespace fluxb

using namespace fluxb;

extern "C" int fluxb_ep_dispatch(const fluxb_ep_dispatch_args_t* a) {
  FLUXB_REQUIRE(a != nullptr && a->x && a->scatter_index && a->splits && a->local_cnt, "dispatch arguments");
  FLUXB_REQUIRE(a->world >= 1 && a->world <= kR && a->rank >= 0 && a->rank < a->world, "ranks");
  FLUXB_REQUIRE(a->tp >= 1 && a->world % a->tp == 0, "tp must divide the group");
  FLUXB_REQUIRE(a->E >= 1 && a->E <= kMaxE && a->E_local >= 1 && a->E_local * (a->world / a->tp) == a->E,
                "experts must divide over the expert groups");
  FLUXB_REQUIRE(a->row_bytes > 0 && a->row_bytes % 16 == 0, "row size must be a multiple of 16 bytes");
  FLUXB_REQUIRE(a->tokens_local >= 0 && a->topk >= 1 && a->capacity_rows > 0, "sizes");
  DispatchParams p;
  memset(&p, 0, sizeof(p));
  p.x = reinterpret_cast<const uint8_t*>(a->x);
  p.scatter_index = a->scatter_index;
  p.splits = a->splits;
  p.token0 = a->token0;
  p.tokens_local = a->tokens_local;
  p.topk = a->topk;
  p.E = a->E;
  p.E_local = a->E_local;
  p.tp = a->tp;
  p.row_bytes = a->row_bytes;
  p.capacity_rows = a->capacity_rows;
  p.rank = a->rank;
  p.world = a->world;
  p.epoch = a->epoch;
  p.timeout_ns = a->timeout_ns ? a->timeout_ns : 5000000000ull;
  p.status = reinterpret_cast<Status*>(a->status);
  p.local_cnt = a->local_cnt;
  p.out_rows = a->out_rows;
  for (int r = 0; r < a->world; ++r) {
    FLUXB_REQUIRE(a->out[r] && a->flags[r] && a->start_ctr[r], "peer pointers missing");
    p.out[r] = reinterpret_cast<uint8_t*>(a->out[r]);
    p.flags[r] = a->flags[r];
    p.start_ctr[r] = a->start_ctr[r];
  }
  int sms = 0, rc;
  if ((rc = device_sm_count(&sms))) return rc;
  // every CTA counts its arrival, so all of them must be resident: two per SM at most
  int grid = a->num_ctas > 0 ? a->num_ctas : 2 * sms;
  if (grid > 2 * sms) grid = 2 * sms;
  ep_dispatch_kernel<<<grid, 256, 0, reinterpret_cast<cudaStream_t>(a->stream)>>>(p);
  FLUXB_CUDA_OK(cudaGetLastError());
  g_launches.fetch_add(1, std::memory_order_relaxed);
  return kOk;
}
