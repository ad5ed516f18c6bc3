// MoE layers: routing-schedule kernels, the grouped GEMM launcher and the top-k combine +
// reduce-scatter kernel.
//   layer 0 (reference: flux.GemmGroupedV3AGScatter): all-gather of token shards + gather by
//           routing index + per-expert GEMM, in one kernel (gemm_grouped.cuh);
//   layer 1 (reference: flux.GemmGroupedV3GatherRS / TopkReduceScatterOp): per-expert GEMM with
//           the row's gate weight applied in the epilogue, then one kernel that sums each token's
//           local top-k rows, pushes the partial to the token's owner rank over NVLink and has
//           the owner add up the W partials.
#include "../include/fluxb.h"
#include "../runtime/host_common.h"
#include "../sm100/gemm_grouped.cuh"

#include <atomic>
#include <cstdlib>
#include <string>

namespace fluxb {
extern std::atomic<uint64_t> g_launches;

namespace {

constexpr int kMaxE = 512;

// ---- scatter_index -> gather_index, per-(expert, source rank) counts -------------------------
__global__ void moe_gather_index_kernel(const int32_t* scatter_index, const int32_t* splits, int64_t n,
                                        int E, int topk, int tokens_per_rank, int W,
                                        int32_t* gather_index, int32_t* cnt /* [E][W], zeroed */) {
  __shared__ int32_t offs[kMaxE + 1];
  if (threadIdx.x == 0) {
    int run = 0;
    for (int e = 0; e < E; ++e) {
      offs[e] = run;
      run += splits[e];
    }
    offs[E] = run;
  }
  __syncthreads();
  const int64_t stride = static_cast<int64_t>(gridDim.x) * blockDim.x;
  for (int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < n; i += stride) {
    const int r = scatter_index[i];
    const int tok = static_cast<int>(i / topk);
    gather_index[r] = tok;
    int lo = 0, hi = E;  // largest e with offs[e] <= r
    while (hi - lo > 1) {
      const int mid = (lo + hi) >> 1;
      if (offs[mid] <= r) lo = mid; else hi = mid;
    }
    atomicAdd(&cnt[lo * W + tok / tokens_per_rank], 1);
  }
}

// ---- schedule: sub-problems (expert, source) in the order this rank should run them ---------
// With routing_idx the launch has more than one block and all of them also fill row_entry: the
// index token * topk + k of every sorted row that lives on this rank.
__global__ void moe_schedule_kernel(const int32_t* splits, const int32_t* cnt /* [E][W] or null */,
                                    int E, int e0, int E_local, int rank, int W, int n_tiles, int BM,
                                    SubProblem* sp, int32_t* tile_begin, int32_t* hdr,
                                    const int32_t* routing_idx, int64_t n_entries, int32_t* row_entry) {
  __shared__ int32_t offs[kMaxE + 1];
  if (threadIdx.x == 0) {
    int run = 0;
    for (int e = 0; e < E; ++e) {
      offs[e] = run;
      run += splits[e];
    }
    offs[E] = run;
  }
  __syncthreads();
  if (routing_idx != nullptr) {
    const int base = offs[e0], rows = offs[e0 + E_local] - offs[e0];
    const int64_t stride = static_cast<int64_t>(gridDim.x) * blockDim.x;
    for (int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < n_entries; i += stride) {
      const int r = routing_idx[i] - base;
      if (r >= 0 && r < rows) row_entry[r] = static_cast<int32_t>(i);
    }
  }
  if (threadIdx.x == 0 && blockIdx.x == 0) {
    hdr[0] = offs[e0];
    hdr[1] = offs[e0 + E_local] - offs[e0];
    int tiles = 0, s = 0;
    if (cnt != nullptr) {
      for (int step = 0; step < W; ++step) {
        int src = rank + step;
        if (src >= W) src -= W;
        for (int el = 0; el < E_local; ++el, ++s) {
          const int e = e0 + el;
          int begin = offs[e];
          for (int r = 0; r < src; ++r) begin += cnt[e * W + r];
          const int rows = cnt[e * W + src];
          sp[s] = SubProblem{begin, begin + rows, el, src};
          tile_begin[s] = tiles;
          tiles += ((rows + BM - 1) / BM) * n_tiles;
        }
      }
    } else {
      for (int el = 0; el < E_local; ++el, ++s) {
        const int e = e0 + el;
        sp[s] = SubProblem{offs[e], offs[e + 1], el, -1};
        tile_begin[s] = tiles;
        tiles += ((offs[e + 1] - offs[e] + BM - 1) / BM) * n_tiles;
      }
    }
    tile_begin[s] = tiles;
  }
}

// ---- top-k combine + reduce-scatter -----------------------------------------------------------
struct CombineParams {
  const uint16_t* y;            // [rows_ep, H] gate-weighted expert outputs of this rank
  const int32_t* hdr;           // [0] row_base, [1] rows_ep
  const int32_t* routing_idx;   // [tokens * topk] sorted row of every (token, k)
  int32_t topk, tokens_per_rank, H, rank, world, out_f16;
  uint32_t epoch;
  uint64_t timeout_ns;
  Status* status;
  uint16_t* stage[kMaxRanks];   // on every rank: [W src][tokens_per_rank][H]
  uint32_t* flags[kMaxRanks];   // on every rank: [W src]
  uint32_t* start_ctr[kMaxRanks];
  uint32_t* local_cnt;          // [W]
  uint16_t* out;                // [tokens_per_rank, H]
};

__global__ void __launch_bounds__(256, 4) moe_combine_kernel(const __grid_constant__ CombineParams p) {
  __shared__ uint32_t abort_word;
  if (threadIdx.x == 0) abort_word = 0;
  __syncthreads();
  WaitCtx wc{p.status, &abort_word, p.timeout_ns};
  const int lane = threadIdx.x & 31;
  const int gwarp = blockIdx.x * 8 + (threadIdx.x >> 5), nwarps = gridDim.x * 8;
  const bool f16 = p.out_f16 != 0;
  const int row_base = p.hdr[0], rows_ep = p.hdr[1];
  const int chunks = p.H / 8;  // 16-byte chunks per row
  const bool multi = p.world > 1;
  if (multi) {
    if (blockIdx.x == 0 && threadIdx.x < p.world) ptx::st_release_sys(p.start_ctr[threadIdx.x] + p.rank, p.epoch);
    if (lane < p.world) flag_wait_ge(wc, p.start_ctr[p.rank] + lane, p.epoch, kSiteStartBarrier);
    __syncwarp();
  }
  // ---- phase 1: partial sums of every token, sent to the token's owner (own tokens last)
  for (int d = 1; d <= p.world; ++d) {
    int owner = p.rank + d;
    if (owner >= p.world) owner -= p.world;
    uint16_t* slab = p.stage[owner] + static_cast<int64_t>(p.rank) * p.tokens_per_rank * p.H;
    for (int tl = gwarp; tl < p.tokens_per_rank; tl += nwarps) {
      const int64_t t = static_cast<int64_t>(owner) * p.tokens_per_rank + tl;
      int rows[16];
      int nloc = 0;
      for (int k = 0; k < p.topk && k < 16; ++k) {
        const int r = p.routing_idx[t * p.topk + k] - row_base;
        if (r >= 0 && r < rows_ep) rows[nloc++] = r;
      }
      // four 16-byte chunks per lane per trip, all loads of a trip issued before the first add
      for (int c0 = lane; c0 < chunks; c0 += 128) {
        float acc[4][8];
#pragma unroll
        for (int u = 0; u < 4; ++u)
#pragma unroll
          for (int e = 0; e < 8; ++e) acc[u][e] = 0.f;
        for (int j = 0; j < nloc; ++j) {
          const uint16_t* yrow = p.y + static_cast<int64_t>(rows[j]) * p.H;
          uint4 v[4];
#pragma unroll
          for (int u = 0; u < 4; ++u)
            if (c0 + 32 * u < chunks) v[u] = *reinterpret_cast<const uint4*>(yrow + (c0 + 32 * u) * 8);
#pragma unroll
          for (int u = 0; u < 4; ++u) {
            if (c0 + 32 * u < chunks) {
              const uint32_t w[4] = {v[u].x, v[u].y, v[u].z, v[u].w};
#pragma unroll
              for (int e = 0; e < 4; ++e) {
                acc[u][2 * e] += ptx::half_bits_to_float(static_cast<uint16_t>(w[e] & 0xFFFFu), f16);
                acc[u][2 * e + 1] += ptx::half_bits_to_float(static_cast<uint16_t>(w[e] >> 16), f16);
              }
            }
          }
        }
#pragma unroll
        for (int u = 0; u < 4; ++u) {
          if (c0 + 32 * u < chunks) {
            uint4 o;
            o.x = ptx::pack_half2(f16, acc[u][0], acc[u][1]);
            o.y = ptx::pack_half2(f16, acc[u][2], acc[u][3]);
            o.z = ptx::pack_half2(f16, acc[u][4], acc[u][5]);
            o.w = ptx::pack_half2(f16, acc[u][6], acc[u][7]);
            ptx::st_global_v4(slab + static_cast<int64_t>(tl) * p.H + (c0 + 32 * u) * 8, o);
          }
        }
      }
    }
    // everything this CTA had for `owner` is written: the last CTA tells the owner
    __syncthreads();
    if (threadIdx.x == 0) {
      uint32_t* cnt = p.local_cnt + (d % p.world);
      if (ptx::atom_add_acq_rel_sys(cnt, 1u) == gridDim.x - 1u) {
        *cnt = 0;
        ptx::st_release_sys(p.flags[owner] + p.rank, p.epoch);
      }
    }
  }
  // ---- phase 2: the owner adds the W partials of each of its tokens, in rank order
  if (lane < p.world) flag_wait_ge(wc, p.flags[p.rank] + lane, p.epoch, kSiteMoeFlag);
  __syncwarp();
  const uint16_t* mine = p.stage[p.rank];
  const int64_t slab_elems = static_cast<int64_t>(p.tokens_per_rank) * p.H;
  for (int tl = gwarp; tl < p.tokens_per_rank; tl += nwarps) {
    for (int c = lane; c < chunks; c += 32) {
      float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
      uint4 v[kMaxRanks];
#pragma unroll
      for (int s = 0; s < kMaxRanks; ++s)
        if (s < p.world) v[s] = ptx::ld_global_cs_v4(mine + s * slab_elems + static_cast<int64_t>(tl) * p.H + c * 8);
#pragma unroll
      for (int s = 0; s < kMaxRanks; ++s) {
        if (s < p.world) {
          const uint32_t w[4] = {v[s].x, v[s].y, v[s].z, v[s].w};
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            acc[2 * e] += ptx::half_bits_to_float(static_cast<uint16_t>(w[e] & 0xFFFFu), f16);
            acc[2 * e + 1] += ptx::half_bits_to_float(static_cast<uint16_t>(w[e] >> 16), f16);
          }
        }
      }
      uint4 o;
      o.x = ptx::pack_half2(f16, acc[0], acc[1]);
      o.y = ptx::pack_half2(f16, acc[2], acc[3]);
      o.z = ptx::pack_half2(f16, acc[4], acc[5]);
      o.w = ptx::pack_half2(f16, acc[6], acc[7]);
      *reinterpret_cast<uint4*>(p.out + static_cast<int64_t>(tl) * p.H + c * 8) = o;
    }
  }
}

template <class Cfg>
int launch_grouped(const GroupedParams& p, int grid, cudaStream_t stream) {
  static bool configured[64] = {false};
  int dev = 0;
  FLUXB_CUDA_OK(cudaGetDevice(&dev));
  if (dev >= 64 || !configured[dev]) {
    FLUXB_CUDA_OK(cudaFuncSetAttribute(grouped_gemm_kernel<Cfg>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                       Cfg::SMEM_BYTES));
    if (dev < 64) configured[dev] = true;
  }
  grouped_gemm_kernel<Cfg><<<grid, Cfg::THREADS, Cfg::SMEM_BYTES, stream>>>(p);
  FLUXB_CUDA_OK(cudaGetLastError());
  g_launches.fetch_add(1, std::memory_order_relaxed);
  return kOk;
}

}  // namespace
}  // namespace fluxb

using namespace fluxb;

// Bytes of int32 scratch the schedule needs: sub-problems, tile prefix, header, counts.
extern "C" int64_t fluxb_moe_schedule_scratch_bytes(int E, int world) {
  const int64_t S = static_cast<int64_t>(E) * world;
  return S * sizeof(SubProblem) + (S + 1) * 4 + 16 + static_cast<int64_t>(E) * world * 4 + 256;
}

extern "C" int64_t fluxb_moe_hdr_offset(int E, int world) {
  const int64_t S = static_cast<int64_t>(E) * world;
  return S * sizeof(SubProblem) + (S + 1) * 4;
}

extern "C" int fluxb_moe_grouped_gemm(const fluxb_moe_gemm_args_t* a) {
  FLUXB_REQUIRE(a != nullptr, "null args");
  FLUXB_REQUIRE(a->E >= 1 && a->E <= kMaxE && a->e0 >= 0 && a->E_local >= 1 && a->e0 + a->E_local <= a->E,
                "expert range");
  FLUXB_REQUIRE(a->N > 0 && a->K > 0 && a->N % 8 == 0, "N, K");
  FLUXB_REQUIRE(a->in_dtype == FLUXB_BF16 || a->in_dtype == FLUXB_FP16 || a->in_dtype == FLUXB_FP8_E4M3 ||
                    a->in_dtype == FLUXB_FP8_E5M2,
                "grouped GEMM runs on bf16 / fp16 / fp8 (e4m3, e5m2; 16-bit output, scales in the epilogue)");
  FLUXB_REQUIRE(a->world >= 1 && a->world <= FLUXB_MAX_RANKS && a->rank >= 0 && a->rank < a->world, "ranks");
  FLUXB_REQUIRE(a->splits && a->scratch && a->weights && (a->d || a->scatter), "pointers");
  const bool in8 = a->in_dtype == FLUXB_FP8_E4M3 || a->in_dtype == FLUXB_FP8_E5M2;
  const int elt = in8 ? 1 : 2;
  const uint32_t bk = 128 / elt;   // elements of one 128-byte swizzle row
  const CUtensorMapDataType in_dt = in8 ? CU_TENSOR_MAP_DATA_TYPE_UINT8 : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16;
  FLUXB_REQUIRE((a->K * elt) % 16 == 0, "K row bytes must be a multiple of 16");
  cudaStream_t stream = reinterpret_cast<cudaStream_t>(a->stream);
  const int bn = (a->N % 256 == 0 || a->N > 1024) ? 256 : 128;
  const int n_tiles = (a->N + bn - 1) / bn;
  const bool by_src = a->gathered && a->world > 1 && a->do_allgather;
  const int64_t S = by_src ? static_cast<int64_t>(a->E_local) * a->world : a->E_local;

  // scratch layout
  uint8_t* sc = reinterpret_cast<uint8_t*>(a->scratch);
  SubProblem* sp = reinterpret_cast<SubProblem*>(sc);
  int32_t* tile_begin = reinterpret_cast<int32_t*>(sc + static_cast<int64_t>(a->E) * a->world * sizeof(SubProblem));
  int32_t* hdr = tile_begin + static_cast<int64_t>(a->E) * a->world + 1;
  int32_t* cnt = hdr + 4;

  if (a->gathered) {
    FLUXB_REQUIRE(a->scatter_index && a->gather_index && a->n_entries > 0 && a->topk > 0, "routing indices");
    FLUXB_CUDA_OK(cudaMemsetAsync(cnt, 0, static_cast<size_t>(a->E) * a->world * 4, stream));
    moe_gather_index_kernel<<<296, 256, 0, stream>>>(a->scatter_index, a->splits, a->n_entries, a->E, a->topk,
                                                     a->tokens_per_rank, a->world, a->gather_index, cnt);
    g_launches.fetch_add(1, std::memory_order_relaxed);
  }
  if (a->scatter) {
    FLUXB_REQUIRE(!a->gathered, "the fused combine takes contiguous rows");
    FLUXB_REQUIRE(a->routing_idx && a->row_entry && a->n_entries > 0 && a->topk >= 1 && a->tokens_per_rank > 0 &&
                      a->sc_out && a->local_cnt,
                  "fused combine: routing index / scratch / output missing");
    moe_schedule_kernel<<<148, 256, 0, stream>>>(a->splits, nullptr, a->E, a->e0, a->E_local, a->rank, a->world,
                                                 n_tiles, 128, sp, tile_begin, hdr, a->routing_idx, a->n_entries,
                                                 a->row_entry);
  } else {
    moe_schedule_kernel<<<1, 32, 0, stream>>>(a->splits, by_src ? cnt : nullptr, a->E, a->e0, a->E_local, a->rank,
                                              a->world, n_tiles, 128, sp, tile_begin, hdr, nullptr, 0, nullptr);
  }
  g_launches.fetch_add(1, std::memory_order_relaxed);
  FLUXB_CUDA_OK(cudaGetLastError());

  GroupedParams p;
  memset(&p, 0, sizeof(p));
  p.sp = sp;
  p.tile_begin = tile_begin;
  p.hdr = hdr;
  p.S = static_cast<int32_t>(S);
  p.N = a->N;
  p.K = a->K;
  p.gathered = a->gathered;
  p.tokens_per_rank = a->tokens_per_rank;
  p.gather_index = a->gather_index;
  p.d = a->d;
  p.ldd = a->ldd;
  p.expert_scale = a->expert_scale;
  p.scalar_scale = a->scalar_scale;
  p.row_scale = a->row_scale;
  p.out_f16 = a->in_dtype == FLUXB_FP16;   // 8-bit inputs give bf16 outputs
  p.ab_fmt = (a->in_dtype == FLUXB_BF16 || a->in_dtype == FLUXB_FP8_E5M2) ? 1 : 0;
  p.rank = a->rank;
  p.world = a->world;
  p.do_allgather = a->do_allgather;
  p.epoch = a->epoch;
  p.timeout_ns = a->timeout_ns ? a->timeout_ns : 5000000000ull;
  p.status = reinterpret_cast<Status*>(a->status);
  int rc;
  {
    uint64_t dims[3] = {static_cast<uint64_t>(a->K), static_cast<uint64_t>(a->N), static_cast<uint64_t>(a->E_local)};
    uint64_t str[2] = {static_cast<uint64_t>(a->K) * elt, static_cast<uint64_t>(a->K) * elt * a->N};
    uint32_t box[3] = {bk, static_cast<uint32_t>(bn), 1};
    if ((rc = encode_tmap(&p.tm_b, in_dt, 3, a->weights, dims, str, box, Swz::B128)))
      return rc;
  }
  // gathered rows: by default the communication warps copy them into a sorted buffer (when the
  // caller provides one); FLUXB_MOE_GATHER=cpasync | gather4 selects the in-loader variants
  static const int gather_mode = [] {
    const char* e = getenv("FLUXB_MOE_GATHER");
    if (e && std::string(e) == "cpasync") return 1;
    if (e && std::string(e) == "gather4") return 2;
    return 3;
  }();
  static const int wave_env = [] {
    const char* e = getenv("FLUXB_MOE_WAVE_SYNC");
    return e ? atoi(e) : 0;
  }();
  // (the sorted buffer's per-sub-problem flags have room for 512 sub-problems)
  const bool pregather = a->gathered && gather_mode == 3 && a->a_sorted != nullptr && S <= 512;
  const bool use_gather4 = a->gathered && gather_mode == 2;
  p.E_local = a->E_local;
  p.by_src = by_src ? 1 : 0;
  if (a->gathered) {
    FLUXB_REQUIRE(a->a_tokens != nullptr, "token matrix missing");
    p.a_tokens = a->a_tokens;
    if (pregather) {
      FLUXB_REQUIRE(a->a_sorted_rows > 0 && a->local_cnt != nullptr, "sorted buffer / local scratch");
      p.a_sorted = a->a_sorted;
      p.local_cnt = a->local_cnt;
      uint64_t dims[2] = {static_cast<uint64_t>(a->K), static_cast<uint64_t>(a->a_sorted_rows)};
      uint64_t str[1] = {static_cast<uint64_t>(a->K) * elt};
      uint32_t box[2] = {bk, 128};
      if ((rc = encode_tmap(&p.tm_a, in_dt, 2, a->a_sorted, dims, str, box, Swz::B128)))
        return rc;
    } else if (use_gather4) {
      uint64_t dims[2] = {static_cast<uint64_t>(a->K),
                          static_cast<uint64_t>(a->tokens_per_rank) * (a->do_allgather || a->world > 1 ? a->world : 1)};
      uint64_t str[1] = {static_cast<uint64_t>(a->K) * elt};
      uint32_t box[2] = {bk, 1};
      if ((rc = encode_tmap(&p.tm_a, in_dt, 2, a->a_tokens, dims, str, box, Swz::B128)))
        return rc;
    }
    if (a->do_allgather) {
      FLUXB_REQUIRE(a->ag_src && a->local_cnt, "all-gather source / scratch missing");
      p.ag_src = a->ag_src;
      p.local_cnt = a->local_cnt;
      for (int r = 0; r < a->world; ++r) {
        FLUXB_REQUIRE(a->ag_land[r] && a->ag_flags[r] && a->start_ctr[r], "all-gather peer pointers missing");
        p.ag_land[r] = a->ag_land[r];
        p.ag_flags[r] = a->ag_flags[r];
        p.start_ctr[r] = a->start_ctr[r];
      }
    }
  } else {
    if (a->scatter) {
      p.topk = a->topk;
      p.row_entry = a->row_entry;
      p.sc_out = reinterpret_cast<uint16_t*>(a->sc_out);
      p.local_cnt = a->local_cnt;
      for (int r = 0; r < a->world; ++r) {
        FLUXB_REQUIRE(a->sc_stage[r] && a->sc_flags[r] && a->start_ctr[r], "fused combine: peer pointers missing");
        p.sc_stage[r] = reinterpret_cast<uint16_t*>(a->sc_stage[r]);
        p.sc_flags[r] = a->sc_flags[r];
        p.start_ctr[r] = a->start_ctr[r];
      }
    }
    FLUXB_REQUIRE(a->a != nullptr && a->a_rows > 0, "contiguous A missing");
    uint64_t dims[2] = {static_cast<uint64_t>(a->K), static_cast<uint64_t>(a->a_rows)};
    uint64_t str[1] = {static_cast<uint64_t>(a->K) * elt};
    uint32_t box[2] = {bk, 128};
    if ((rc = encode_tmap(&p.tm_a, in_dt, 2, a->a, dims, str, box, Swz::B128)))
      return rc;
  }
  int sms = 0;
  if ((rc = device_sm_count(&sms))) return rc;
  {
    static const int inflight_env = [] {
      const char* e = getenv("FLUXB_MOE_INFLIGHT");
      return e ? atoi(e) : 0;
    }();
    p.ring_inflight = inflight_env;
    static const int split_env = [] {
      const char* e = getenv("FLUXB_MOE_COMM_SPLIT");
      return e ? atoi(e) : 0;   // measured slower at four ranks: 1.97 against 1.88 ms for layer 0
    }();
    p.comm_split = split_env;
  }
  // (the cp.async variant keeps its own producer warps per tile and is left alone)
  if (wave_env != 0 && !(a->gathered && gather_mode == 1)) p.wave_ctr = wave_counter_for(stream);
  if (in8) {
    // 8-bit operands (tcgen05 kind::f8f6f4): contiguous A, the sorted-buffer gather and the fused combine
    FLUXB_REQUIRE(!a->gathered || pregather, "fp8 grouped GEMM gathers rows through the sorted buffer only");
    if (pregather) {
      if (bn == 256) return launch_grouped<GroupedCfg<256, 1, 4, 3>>(p, sms, stream);
      return launch_grouped<GroupedCfg<128, 1, 5, 3>>(p, sms, stream);
    }
    if (a->scatter) {
      if (bn == 256) return launch_grouped<GroupedCfg<256, 1, 4, 0, true>>(p, sms, stream);
      return launch_grouped<GroupedCfg<128, 1, 6, 0, true>>(p, sms, stream);
    }
    if (bn == 256) return launch_grouped<GroupedCfg<256, 1, 4, 0>>(p, sms, stream);
    return launch_grouped<GroupedCfg<128, 1, 6, 0>>(p, sms, stream);
  }
  if (pregather) {
    if (bn == 256) return launch_grouped<GroupedCfg<256, 0, 4, 3>>(p, sms, stream);
    return launch_grouped<GroupedCfg<128, 0, 5, 3>>(p, sms, stream);
  }
  if (a->gathered && use_gather4) {
    if (bn == 256) return launch_grouped<GroupedCfg<256, 0, 4, 2>>(p, sms, stream);
    return launch_grouped<GroupedCfg<128, 0, 5, 2>>(p, sms, stream);
  }
  if (a->gathered) {
    if (bn == 256) return launch_grouped<GroupedCfg<256, 0, 4, 1>>(p, sms, stream);
    return launch_grouped<GroupedCfg<128, 0, 5, 1>>(p, sms, stream);
  }
  if (a->scatter) {
    // every CTA takes part in the arrival counting and in the tail: full grid
    if (bn == 256) return launch_grouped<GroupedCfg<256, 0, 4, 0, true>>(p, sms, stream);
    return launch_grouped<GroupedCfg<128, 0, 6, 0, true>>(p, sms, stream);
  }
  if (bn == 256) return launch_grouped<GroupedCfg<256, 0, 4, 0>>(p, sms, stream);
  return launch_grouped<GroupedCfg<128, 0, 6, 0>>(p, sms, stream);
}

extern "C" int fluxb_moe_combine(const fluxb_moe_combine_args_t* a) {
  FLUXB_REQUIRE(a != nullptr && a->y && a->hdr && a->routing_idx && a->out, "combine arguments");
  FLUXB_REQUIRE(a->H % 8 == 0 && a->topk >= 1 && a->topk <= 16, "H must be a multiple of 8, topk <= 16");
  FLUXB_REQUIRE(a->world >= 1 && a->world <= FLUXB_MAX_RANKS, "world");
  CombineParams p;
  memset(&p, 0, sizeof(p));
  p.y = reinterpret_cast<const uint16_t*>(a->y);
  p.hdr = a->hdr;
  p.routing_idx = a->routing_idx;
  p.topk = a->topk;
  p.tokens_per_rank = a->tokens_per_rank;
  p.H = a->H;
  p.rank = a->rank;
  p.world = a->world;
  p.out_f16 = a->dtype == FLUXB_FP16;
  p.epoch = a->epoch;
  p.timeout_ns = a->timeout_ns ? a->timeout_ns : 5000000000ull;
  p.status = reinterpret_cast<Status*>(a->status);
  p.local_cnt = a->local_cnt;
  p.out = reinterpret_cast<uint16_t*>(a->out);
  for (int r = 0; r < a->world; ++r) {
    FLUXB_REQUIRE(a->stage[r] && a->flags[r] && a->start_ctr[r], "combine peer pointers missing");
    p.stage[r] = reinterpret_cast<uint16_t*>(a->stage[r]);
    p.flags[r] = a->flags[r];
    p.start_ctr[r] = a->start_ctr[r];
  }
  FLUXB_REQUIRE(a->local_cnt != nullptr, "local arrival scratch missing");
  int sms = 0, rc;
  if ((rc = device_sm_count(&sms))) return rc;
  // every CTA takes part in the arrival counting, so all of them must be resident
  // latency-bound streaming kernel: four CTAs per SM (64 registers) keep more rows in flight
  static const int per_sm = [] {
    const char* e = getenv("FLUXB_COMBINE_CTAS_PER_SM");
    const int v = e ? atoi(e) : 4;
    return v >= 1 && v <= 4 ? v : 4;
  }();
  moe_combine_kernel<<<sms * per_sm, 256, 0, reinterpret_cast<cudaStream_t>(a->stream)>>>(p);
  FLUXB_CUDA_OK(cudaGetLastError());
  g_launches.fetch_add(1, std::memory_order_relaxed);
  return kOk;
}
