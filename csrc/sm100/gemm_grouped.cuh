// Grouped (per-expert) GEMM for MoE layers on sm_100a, same tcgen05/TMEM pipeline as the dense
// kernel, with two things the dense kernel does not have:
//   * a device-built schedule of sub-problems (expert, source rank, row range) walked by every
//     CTA, so neither per-expert row counts nor pointer arrays ever visit the host;
//   * optional gathered A: row r of the expert-sorted order is token gather_index[r] of the
//     all-gathered token matrix. Four producer warps fetch those rows with 16-byte cp.async
//     into the same 128-byte-swizzled layout TMA would produce; B (the expert's weight) comes
//     by TMA from a 3-D map [expert][N][K].
// In MoE layer 0 the kernel also performs the all-gather: warps 2-3 push this rank's token shard
// into every peer's landing buffer (bulk-copy ring) and sub-problems of source rank s start
// once s's shard has landed, own shard first.
// In MoE layer 1 (SCATTER_) the epilogue multiplies every row by its gate weight and stores it
// straight into the slot [token][k] of the staging buffer of the rank that owns the token, over
// NVLink; when the rows of all W ranks have landed, the tail of the same kernel adds the top-k
// rows of each of this rank's tokens in fp32 (k = 0, 1, ...) and writes the result. The
// expert-sorted product never exists in memory.
// Reference: src/moe_ag_scatter (GemmGroupedV3AGScatter, sort_util.cu, gather_tensor.hpp,
// sm90_ag_scatter_fetcher.hpp) and src/moe_gather_rs (compute CTAs + DMA CTAs of
// sm90_gemm_array_threadblock_specialized.hpp, topk_gather_rs.cu).
#pragma once

#include "gemm_dense.cuh"

namespace fluxb {

struct SubProblem {
  int32_t row_begin, row_end;  // rows of the expert-sorted order
  int32_t expert;              // local expert index (z coordinate of the weight map)
  int32_t src;                 // source rank whose tokens these rows are (-1: no gating)
};

struct GroupedParams {
  CUtensorMap tm_a;            // contiguous A [rows, K], box {BK, 128}; gather4: tokens [T, K], box {BK, 1}
  CUtensorMap tm_b;            // weights [E_local][N][K], box {BK, BN, 1}
  const SubProblem* sp;        // [S]
  const int32_t* tile_begin;   // [S + 1] prefix sums of (row tiles x column tiles)
  int32_t S, N, K;
  const int32_t* hdr;          // device: [0] row_base: sorted row r lives at row r - row_base of the
                               // contiguous A and of D; [1] number of rows of this rank
  int32_t gathered;            // 1: A rows are tokens picked by gather_index
  int32_t tokens_per_rank;
  const void* a_tokens;        // [W * tokens_per_rank, K] all-gathered tokens (landing buffer)
  void* a_sorted;              // pre-gather mode: [rows of this rank, K] expert-sorted copy of the rows
  int32_t E_local, by_src;     // schedule shape: S = E_local * (by_src ? world : 1)
  const int32_t* gather_index; // [total sorted rows] token of each sorted row
  void* d;                     // [rows_out, N], 16-bit
  int64_t ldd;
  const float* expert_scale;   // [E_local] or null
  const float* scalar_scale;   // [1] or null
  const float* row_scale;      // [rows_out] or null (top-k gate weight of the row)
  int32_t out_f16, ab_fmt;
  // all-gather of the token shards (layer 0)
  int32_t rank, world, do_allgather;
  uint32_t epoch;
  uint64_t timeout_ns;
  Status* status;
  const void* ag_src;          // this rank's shard [tokens_per_rank, K]
  void* ag_land[kMaxRanks];
  uint32_t* ag_flags[kMaxRanks];   // on every rank: [W src] last call whose shard landed
  uint32_t* start_ctr[kMaxRanks];
  uint32_t* local_cnt;             // [W]
  uint32_t* wave_ctr;              // optional: tiles whose loads are all issued (wave-synchronous starts)
  int32_t ring_inflight;           // loads in flight ahead of the stores in the push / gather rings (0 = all slots but one)
  int32_t comm_split;              // 1: with an all-gather and a pre-gather to do, warp 2 pushes and warp 3 gathers
  // ---- layer 1 with the combine fused in (SCATTER_)
  int32_t topk;
  const int32_t* row_entry;        // [rows of this rank] token * topk + k of every local sorted row
  uint16_t* sc_stage[kMaxRanks];   // on every rank: [tokens_per_rank][topk][N], 16-bit
  uint32_t* sc_flags[kMaxRanks];   // on every rank: [W src] last call whose rows have all landed
  uint16_t* sc_out;                // [tokens_per_rank, N]
};

// GATHER_: 0 = contiguous A by TMA; 1 = gathered A rows by cp.async from four producer warps;
// 2 = gathered A rows by TMA tile::gather4 (four indexed rows per instruction) from the producer lane;
// 3 = the communication warps copy the gathered rows, whole rows at a time, into an expert-sorted
//     buffer as soon as their source shard has landed, and the GEMM reads that buffer by TMA.
template <int BN_, int KIND_, int STAGES_, int GATHER_, bool SCATTER_ = false>
struct GroupedCfg {
  static constexpr bool SCATTER = SCATTER_;        // layer 1: rows go to the token owner's [token][k] slot
  static_assert(!SCATTER_ || GATHER_ == 0, "the scatter epilogue reads contiguous A");
  static constexpr int BM = 128, BN = BN_, KIND = KIND_, STAGES = STAGES_;
  static constexpr bool GATHER = GATHER_ == 1;     // cp.async producers
  static constexpr bool GATHER4 = GATHER_ == 2;    // TMA gather4
  static constexpr bool PREGATHER = GATHER_ == 3;  // rows copied into a sorted buffer by the comm warps
  static constexpr bool ANY_GATHER = GATHER_ != 0;
  static constexpr int ELT = KIND_ == 0 ? 2 : 1;
  static constexpr int BK = 128 / ELT;
  static constexpr int UMMA_K = 32 / ELT;
  static constexpr int A_BYTES = BM * 128, B_BYTES = BN * 128, STAGE_BYTES = A_BYTES + B_BYTES;
  // scatter epilogue: every epilogue warp stages 32 rows x 64 columns (128 bytes per row, 144-byte
  // pitch so that the lanes' 16-byte writes fall into different banks) before the rows leave as
  // one bulk copy each
  static constexpr int SC_PITCH = 144;
  static constexpr int SC_WARP_BYTES = 32 * SC_PITCH;
  static constexpr int COMM_BYTES = GATHER_ != 0 ? 32768 : (SCATTER_ ? 4 * SC_WARP_BYTES : 0);
  static constexpr int BAR_BYTES = 256 + 1024;     // barriers, then two 128-entry row-index buffers
  static constexpr int THREADS = GATHER_ == 1 ? 384 : 256;
  static constexpr int SMEM_BYTES = STAGES * STAGE_BYTES + COMM_BYTES + BAR_BYTES + 1024;
  static_assert(SMEM_BYTES <= 232448, "over the 227 KB shared memory limit");
};

// words of GroupedParams::local_cnt: [0, 16) arrival counters of the push steps, then one arrival
// counter and one "rows are in the sorted buffer" flag per sub-problem (at most 512)
constexpr int kGatherCountBase = 64;
constexpr int kGatherFlagBase = 64 + 512;

struct GroupedTile {
  int sp, row0, rows, n0, expert, src;
};

// Walks the schedule for increasing tile ids; `cursor` is the sub-problem of the previous tile.
__device__ __forceinline__ GroupedTile grouped_decode(const GroupedParams& p, int t, int& cursor,
                                                      int n_tiles, int BM, int BN) {
  while (cursor + 1 < p.S && t >= p.tile_begin[cursor + 1]) ++cursor;
  const SubProblem s = p.sp[cursor];
  const int local = t - p.tile_begin[cursor];
  const int m_tiles = (s.row_end - s.row_begin + BM - 1) / BM;
  const int mt = local % m_tiles, nt = local / m_tiles;   // row tiles innermost: B tile reused
  GroupedTile g;
  g.sp = cursor;
  g.row0 = s.row_begin + mt * BM;
  g.rows = min(BM, s.row_end - g.row0);
  g.n0 = nt * BN;
  g.expert = s.expert;
  g.src = s.src;
  (void)n_tiles;
  return g;
}

template <class Cfg>
__global__ void __launch_bounds__(Cfg::THREADS, 1) grouped_gemm_kernel(const __grid_constant__ GroupedParams p) {
  constexpr int BM = Cfg::BM, BN = Cfg::BN, BK = Cfg::BK, STAGES = Cfg::STAGES;
  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw_addr = ptx::smem_u32(smem_raw);
  const uint32_t pad = (1024u - (raw_addr & 1023u)) & 1023u;
  uint8_t* smem = smem_raw + pad;
  const uint32_t smem_base = raw_addr + pad;
  const uint32_t comm_base = smem_base + STAGES * Cfg::STAGE_BYTES;
  const uint32_t bar_base = comm_base + Cfg::COMM_BYTES;
  uint8_t* bar_ptr = smem + STAGES * Cfg::STAGE_BYTES + Cfg::COMM_BYTES;
  auto full_bar = [&](int s) { return bar_base + 8u * s; };
  auto empty_bar = [&](int s) { return bar_base + 8u * (STAGES + s); };
  auto tfull_bar = [&](int a) { return bar_base + 8u * (2 * STAGES + a); };
  auto tempty_bar = [&](int a) { return bar_base + 8u * (2 * STAGES + 2 + a); };
  volatile uint32_t* tmem_slot = reinterpret_cast<volatile uint32_t*>(bar_ptr + 8 * (2 * STAGES + 4));
  volatile uint32_t* abort_word = tmem_slot + 1;
  const uint32_t ring_bar_base = bar_base + 8u * (2 * STAGES + 4) + 16u;
  static_assert(8 * (2 * STAGES + 4) + 16 + 64 <= Cfg::BAR_BYTES, "barrier block too small");

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      // B arrives by TMA (one arrival + bytes); gathered A adds one arrival per producer thread
      ptx::mbar_init(full_bar(s), Cfg::GATHER ? 1 + 128 : 1);
      ptx::mbar_init(empty_bar(s), 1);
    }
    for (int a = 0; a < 2; ++a) {
      ptx::mbar_init(tfull_bar(a), 1);
      ptx::mbar_init(tempty_bar(a), 4);
    }
    for (int i = 0; i < 8; ++i) ptx::mbar_init(ring_bar_base + 8u * i, 1);
    *abort_word = 0;
    ptx::fence_mbar_init();
    ptx::prefetch_tmap(&p.tm_b);
  }
  if (warp == 1) {
    ptx::tmem_alloc<1>(ptx::smem_u32(const_cast<uint32_t*>(tmem_slot)), 512);
    ptx::tmem_relinquish<1>();
  }
  ptx::tc_fence_before();
  __syncthreads();
  ptx::tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  WaitCtx wc{p.status, abort_word, p.timeout_ns};

  const int n_tiles = (p.N + BN - 1) / BN;
  const int total_tiles = p.tile_begin[p.S];
  const int k_blocks = (p.K + BK - 1) / BK;
  const bool multi = p.world > 1 && p.do_allgather;
  const int row_base = p.hdr[0];

  if (warp == 0) {
    // ------------------------------------------------------------------ TMA producer (B, and A unless cp.async gathers it)
    int stage = 0, cursor = 0, ready_src = -1, nt = 0;
    uint32_t phase = 0;
    int32_t* idx_buf = reinterpret_cast<int32_t*>(bar_ptr + 256);
    for (int t = blockIdx.x; t < total_tiles; t += gridDim.x, ++nt) {
      if (*abort_word) break;   // a wait gave up: issue nothing more
      const GroupedTile g = grouped_decode(p, t, cursor, n_tiles, BM, BN);
      int32_t* idx = idx_buf + (nt & 1) * 128;
      if constexpr (Cfg::GATHER4) {
        if (g.src >= 0 && g.src != ready_src) {
          // tokens of this source must have landed (sub-problems are ordered by source, own first)
          if (lane == 0) {
            flag_wait_ge(wc, p.ag_flags[p.rank] + g.src, p.epoch, kSiteMoeFlag);
            ptx::fence_proxy_async_all();
          }
          ready_src = g.src;
        }
        // the 128 token ids of this tile (rows past the end of the sub-problem read token 0; their
        // results are never stored)
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const int r = lane * 4 + j;
          idx[r] = r < g.rows ? p.gather_index[g.row0 + r] : 0;
        }
        __syncwarp();
      }
      if constexpr (Cfg::PREGATHER) {
        // the rows of this sub-problem must be in the sorted buffer (one flag per sub-problem, so
        // the GEMM follows the gather expert by expert instead of source by source)
        if (g.sp != ready_src) {
          if (lane == 0) {
            flag_wait_ge(wc, p.local_cnt + kGatherFlagBase + g.sp, p.epoch, kSiteMoeFlag);
            ptx::fence_proxy_async_all();
          }
          ready_src = g.sp;
        }
      }
      if (lane == 0) {
        // wave-synchronous starts: tile nt of this CTA waits until every CTA has issued the loads
        // of its tile nt - 1, which keeps the CTAs on neighbouring tiles and k ranges (L2 reuse)
        if (p.wave_ctr != nullptr && nt > 0) {
          const uint32_t need = min(static_cast<uint32_t>(nt) * gridDim.x, static_cast<uint32_t>(total_tiles));
          flag_wait_ge(wc, p.wave_ctr, need, kSiteStartBarrier);
        }
        for (int kb = 0; kb < k_blocks; ++kb) {
          mbar_wait(wc, empty_bar(stage), phase ^ 1u, kSiteSmemEmpty);
          const uint32_t sa = smem_base + stage * Cfg::STAGE_BYTES;
          if constexpr (Cfg::GATHER) {
            ptx::mbar_arrive_expect_tx(full_bar(stage), Cfg::B_BYTES);
          } else if constexpr (Cfg::GATHER4) {
            ptx::mbar_arrive_expect_tx(full_bar(stage), Cfg::STAGE_BYTES);
#pragma unroll 4
            for (int i = 0; i < 32; ++i)
              ptx::tma_gather4_2d(sa + i * 512, &p.tm_a, full_bar(stage), kb * BK, idx[4 * i], idx[4 * i + 1],
                                  idx[4 * i + 2], idx[4 * i + 3]);
          } else {
            ptx::mbar_arrive_expect_tx(full_bar(stage), Cfg::STAGE_BYTES);
            ptx::tma_load_2d(sa, &p.tm_a, full_bar(stage), kb * BK, g.row0 - row_base);
          }
          ptx::tma_load_3d(sa + Cfg::A_BYTES, &p.tm_b, full_bar(stage), kb * BK, g.n0, g.expert);
          if (++stage == STAGES) {
            stage = 0;
            phase ^= 1u;
          }
        }
        if (p.wave_ctr != nullptr &&
            atomicAdd(p.wave_ctr, 1u) == static_cast<uint32_t>(total_tiles) - 1u)
          atomicExch(p.wave_ctr, 0u);   // last tile of the launch: every wait was for a smaller value
      }
      __syncwarp();
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------------ MMA issuer
    if (lane == 0) {
      const uint32_t idesc = ptx::umma_idesc(p.ab_fmt, p.ab_fmt, BM, BN);
      int stage = 0, it = 0;
      uint32_t phase = 0;
      for (int t = blockIdx.x; t < total_tiles; t += gridDim.x, ++it) {
        if (*abort_word) break;   // a wait gave up: issue nothing more
        const int acc = it & 1;
        mbar_wait(wc, tempty_bar(acc), (((it >> 1) & 1) ^ 1u), kSiteTmemEmpty);
        ptx::tc_fence_after();
        const uint32_t d_tmem = tmem_base + acc * BN;
        for (int kb = 0; kb < k_blocks; ++kb) {
          mbar_wait(wc, full_bar(stage), phase, kSiteSmemFull);
          // gathered A rows were written through the generic proxy (cp.async)
          if constexpr (Cfg::GATHER) ptx::fence_proxy_async_smem();
          ptx::tc_fence_after();
          const uint32_t sa = smem_base + stage * Cfg::STAGE_BYTES;
          const uint64_t adesc = ptx::umma_desc_k_sw128(sa);
          const uint64_t bdesc = ptx::umma_desc_k_sw128(sa + Cfg::A_BYTES);
#pragma unroll
          for (int k = 0; k < BK / Cfg::UMMA_K; ++k)
            ptx::umma_ss<1, Cfg::KIND>(d_tmem, adesc + 2u * k, bdesc + 2u * k, idesc, (kb | k) != 0 ? 1u : 0u);
          ptx::umma_commit(empty_bar(stage));
          if (++stage == STAGES) {
            stage = 0;
            phase ^= 1u;
          }
        }
        ptx::umma_commit(tfull_bar(acc));
      }
    }
  } else if (warp == 2 || warp == 3) {
    if constexpr (Cfg::SCATTER) {
      // "this rank has entered call `epoch`": its staging slots of the previous call are consumed
      if (warp == 3 && blockIdx.x == 0 && lane < p.world) ptx::st_release_sys(p.start_ctr[lane] + p.rank, p.epoch);
    }
    // ------------------------------------------------------------------ all-gather push of the token shard
    if constexpr (Cfg::ANY_GATHER) {
      if (multi && warp == 3 && blockIdx.x == 0 && lane < p.world)
        ptx::st_release_sys(p.start_ctr[lane] + p.rank, p.epoch);
      if (multi) {
        if (lane < p.world) flag_wait_ge(wc, p.start_ctr[p.rank] + lane, p.epoch, kSiteStartBarrier);
        __syncwarp();
      }
      if (lane == 0 && (p.do_allgather || Cfg::PREGATHER)) {
        // One lane per warp drives a ring of staging slots (bulk load -> bulk store). Per step d:
        // push this rank's shard to peer rank-d (d = 0: the own landing slot), then - in pre-gather
        // mode - copy the rows that come from source rank+d, which arrives during the same step
        // because every rank walks the same rotation, into the expert-sorted buffer.
        // Optional (comm_split): with both jobs to do (all-gather and pre-gather on several ranks) warp 2
        // pushes all steps and warp 3 gathers all steps, so that the NVLink transfer of step d + 1 does not
        // wait for the local copies of step d. Measured slower than both warps doing both in turn (layer 0
        // at four ranks: 1.97 against 1.88 ms), so it is off by default.
        const bool split = Cfg::PREGATHER && p.do_allgather && p.world > 1 && p.comm_split != 0;
        const bool do_push = p.do_allgather && (!split || warp == 2);
        const bool do_gather = Cfg::PREGATHER && (!split || warp == 3);
        const uint32_t ring = comm_base + (warp - 2) * (Cfg::COMM_BYTES / 2);
        const uint32_t rbar = ring_bar_base + (warp - 2) * 4 * 8u;
        const uint32_t cw = split ? blockIdx.x : blockIdx.x * 2 + (warp - 2);
        const uint32_t ncw = split ? gridDim.x : gridDim.x * 2;
        const int64_t row_bytes = static_cast<int64_t>(p.K) * Cfg::ELT;
        uint32_t used[4] = {0u, 0u, 0u, 0u};   // loads seen by each ring barrier (their phase)
        struct Item {
          const uint8_t* from;
          uint8_t* to;
          uint32_t sz;
        };
        // Copies the pieces that `gen` hands out through NS staging slots of SZ bytes (barrier of
        // slot i: i * bar_stride): NS - 1 loads are in flight ahead of the store that is being
        // issued, so neither the load latency nor the store latency is paid per piece. Every slot
        // is free when this starts (each step ends with a full bulk wait).
        auto pipe = [&](auto&& gen, const uint32_t NS, const uint32_t SZ, const uint32_t bar_stride) {
          Item q[4];
          uint32_t qph[4];
          uint32_t head = 0, tail = 0;
          auto issue = [&](const Item& it) {
            const uint32_t slot = tail % NS, bar = slot * bar_stride;
            qph[slot] = used[bar] & 1u;
            ++used[bar];
            q[slot] = it;
            ptx::mbar_arrive_expect_tx(rbar + 8u * bar, it.sz);
            ptx::bulk_load(ring + slot * SZ, it.from, it.sz, rbar + 8u * bar);
            ++tail;
          };
          Item it;
          const uint32_t depth = p.ring_inflight >= 1 && static_cast<uint32_t>(p.ring_inflight) < NS
                                     ? static_cast<uint32_t>(p.ring_inflight) : NS - 1;
          for (uint32_t k = 0; k < depth; ++k) {
            if (!gen(it)) break;
            issue(it);
          }
          while (head < tail) {
            const uint32_t slot = head % NS, bar = slot * bar_stride;
            mbar_wait(wc, rbar + 8u * bar, qph[slot], kSiteSmemFull);
            ptx::bulk_store(q[slot].to, ring + slot * SZ, q[slot].sz);
            ptx::bulk_commit();
            ++head;
            if (gen(it)) {
              // the slot's last store (NS - depth + 1 stores back) has read it
              if (NS - depth == 1) ptx::bulk_wait_read<1>();
              else if (NS - depth == 2) ptx::bulk_wait_read<2>();
              else ptx::bulk_wait_read<3>();
              issue(it);
            }
          }
        };
        const int steps = p.do_allgather ? p.world : 1;
        for (int d = 0; d < steps; ++d) {
          if (do_push) {
            constexpr uint32_t CH = Cfg::COMM_BYTES / 2 / 4;   // 4 slots of 4 KiB
            const uint8_t* src = reinterpret_cast<const uint8_t*>(p.ag_src);
            const int64_t bytes = static_cast<int64_t>(p.tokens_per_rank) * row_bytes;
            const uint32_t nch = static_cast<uint32_t>((bytes + CH - 1) / CH);
            int peer = p.rank - d;
            if (peer < 0) peer += p.world;
            uint8_t* land = reinterpret_cast<uint8_t*>(p.ag_land[peer]) + static_cast<int64_t>(p.rank) * bytes;
            uint32_t c = cw;
            pipe(
                [&](Item& it) -> bool {
                  if (c >= nch) return false;
                  const int64_t off = static_cast<int64_t>(c) * CH;
                  const int64_t left = bytes - off;
                  it.from = src + off;
                  it.to = land + off;
                  it.sz = left < static_cast<int64_t>(CH) ? static_cast<uint32_t>(left) : CH;
                  c += ncw;
                  return true;
                },
                4u, CH, 1u);
            ptx::bulk_wait<0>();
            ptx::fence_proxy_async_all();
            uint32_t* cnt = p.local_cnt + d;
            if (ptx::atom_add_acq_rel_sys(cnt, 1u) == ncw - 1u) {
              *cnt = 0;
              ptx::st_release_sys(p.ag_flags[peer] + p.rank, p.epoch);
            }
          }
          if (Cfg::PREGATHER && do_gather) {
            constexpr uint32_t SLOT = Cfg::COMM_BYTES / 2 / 2;  // 2 slots of 8 KiB (over ring slots {0,1}, {2,3})
            const uint8_t* tokens = reinterpret_cast<const uint8_t*>(p.a_tokens);
            uint8_t* sorted = reinterpret_cast<uint8_t*>(p.a_sorted);
            if (p.by_src) {
              int src = p.rank + d;
              if (src >= p.world) src -= p.world;
              flag_wait_ge(wc, p.ag_flags[p.rank] + src, p.epoch, kSiteMoeFlag);
              ptx::fence_proxy_async_all();
            }
            // rows of the sub-problems of this step, every ncw-th row, each in pieces of SLOT bytes;
            // each sub-problem is published on its own
            for (int el = 0; el < p.E_local; ++el) {
              const int spi = d * p.E_local + el;
              const SubProblem sp = p.sp[spi];
              int r = sp.row_begin + static_cast<int>(cw) - static_cast<int>(ncw);
              bool have_row = false;
              int64_t off = 0;
              const uint8_t* from_row = nullptr;
              uint8_t* to_row = nullptr;
              pipe(
                  [&](Item& it) -> bool {
                    for (;;) {
                      if (have_row && off < row_bytes) {
                        const int64_t left = row_bytes - off;
                        it.from = from_row + off;
                        it.to = to_row + off;
                        it.sz = left < static_cast<int64_t>(SLOT) ? static_cast<uint32_t>(left) : SLOT;
                        off += SLOT;
                        return true;
                      }
                      r += static_cast<int>(ncw);
                      if (r >= sp.row_end) return false;
                      const int tok = p.gather_index[r];
                      const int tok_limit = p.tokens_per_rank * (p.world > 1 ? p.world : 1);
                      if (!dcheck(wc, tok >= 0 && tok < tok_limit && r >= row_base, kCheckMoeGather,
                                  static_cast<uint32_t>(r), static_cast<uint32_t>(tok)))
                        return false;
                      from_row = tokens + static_cast<int64_t>(tok) * row_bytes;
                      to_row = sorted + static_cast<int64_t>(r - row_base) * row_bytes;
                      off = 0;
                      have_row = true;
                    }
                  },
                  2u, SLOT, 2u);
              ptx::bulk_wait<0>();
              ptx::fence_proxy_async_all();
              uint32_t* cnt = p.local_cnt + kGatherCountBase + spi;
              if (ptx::atom_add_acq_rel_sys(cnt, 1u) == ncw - 1u) {
                *cnt = 0;
                ptx::st_release_sys(p.local_cnt + kGatherFlagBase + spi, p.epoch);
              }
            }
          }
        }
      }
    }
  } else if (warp < 8) {
    // ------------------------------------------------------------------ epilogue
    const int q = warp & 3;
    const bool f16 = p.out_f16 != 0;
    const float sscale = p.scalar_scale ? *p.scalar_scale : 1.f;
    int it = 0, cursor = 0;
    uint16_t* dbase = reinterpret_cast<uint16_t*>(p.d);
    if constexpr (Cfg::SCATTER) {
      // nobody writes into an owner's slots before that owner has entered this call
      if (lane < p.world) flag_wait_ge(wc, p.start_ctr[p.rank] + lane, p.epoch, kSiteStartBarrier);
      __syncwarp();
    }
    for (int t = blockIdx.x; t < total_tiles; t += gridDim.x, ++it) {
      if (*abort_word) break;   // a wait gave up: issue nothing more
      const GroupedTile g = grouped_decode(p, t, cursor, n_tiles, BM, BN);
      const int acc = it & 1;
      const uint32_t par = (it >> 1) & 1;
      if (lane == 0) mbar_wait(wc, tfull_bar(acc), par, kSiteTmemFull);
      __syncwarp();
      mbar_wait(wc, tfull_bar(acc), par, kSiteTmemFull);
      ptx::tc_fence_after();
      const int r_in_tile = q * 32 + lane;
      const bool row_ok = r_in_tile < g.rows;
      const int64_t orow = static_cast<int64_t>(g.row0) - row_base + r_in_tile;
      float scale = sscale;
      if (p.expert_scale) scale *= p.expert_scale[g.expert];
      if (p.row_scale && row_ok) scale *= p.row_scale[orow];
      uint16_t* drow_base = dbase + orow * p.ldd;
      if constexpr (Cfg::SCATTER) {
        if (row_ok) {
          const int entry = p.row_entry[orow];
          const int token = entry / p.topk;
          const int owner = token / p.tokens_per_rank;
          const int64_t slot = static_cast<int64_t>(token - owner * p.tokens_per_rank) * p.topk + (entry - token * p.topk);
          drow_base = p.sc_stage[owner] + slot * p.N;
        }
      }
#pragma unroll 1
      for (int ch = 0; ch < BN / 64; ++ch) {
        uint32_t r0[32], r1[32];
        const uint32_t taddr = tmem_base + (static_cast<uint32_t>(q * 32) << 16) + acc * BN + ch * 64;
        ptx::tmem_ld_32x32b_x32(taddr, r0);
        ptx::tmem_ld_32x32b_x32(taddr + 32, r1);
        ptx::tmem_ld_wait();
        if (ch == BN / 64 - 1) {
          ptx::tc_fence_before();
          __syncwarp();
          if (lane == 0) ptx::mbar_arrive(tempty_bar(acc));
        }
        const int col0 = g.n0 + ch * 64;
        if constexpr (Cfg::SCATTER) {
          // this lane's 64 columns -> its row of the warp's staging block -> one bulk copy of the
          // row piece (up to 128 bytes) to the owner's slot: whole lines travel over NVLink instead
          // of 16-byte stores scattered over 32 rows
          const uint32_t my_row = comm_base + (warp - 4) * Cfg::SC_WARP_BYTES + lane * Cfg::SC_PITCH;
          ptx::bulk_wait_read<0>();      // this lane's previous copy has read the row
          __syncwarp();
          auto pk = [&](const uint32_t (&r)[32], int i) {
            return ptx::pack_half2(f16, __uint_as_float(r[i]) * scale, __uint_as_float(r[i + 1]) * scale);
          };
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(my_row + 16 * j), "r"(pk(r0, 8 * j)),
                         "r"(pk(r0, 8 * j + 2)), "r"(pk(r0, 8 * j + 4)), "r"(pk(r0, 8 * j + 6))
                         : "memory");
            asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(my_row + 64 + 16 * j), "r"(pk(r1, 8 * j)),
                         "r"(pk(r1, 8 * j + 2)), "r"(pk(r1, 8 * j + 4)), "r"(pk(r1, 8 * j + 6))
                         : "memory");
          }
          ptx::fence_proxy_async_smem();
          if (row_ok && col0 < p.N) {
            const int ncol = p.N - col0 < 64 ? p.N - col0 : 64;     // a multiple of 8
            ptx::bulk_store(drow_base + col0, my_row, static_cast<uint32_t>(ncol) * 2u);
          }
          ptx::bulk_commit();
          continue;
        }
        if (row_ok && col0 < p.N) {
          uint16_t* drow = drow_base + col0;
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            if (col0 + 8 * j < p.N) {
              uint4 v;
              v.x = ptx::pack_half2(f16, __uint_as_float(r0[8 * j + 0]) * scale, __uint_as_float(r0[8 * j + 1]) * scale);
              v.y = ptx::pack_half2(f16, __uint_as_float(r0[8 * j + 2]) * scale, __uint_as_float(r0[8 * j + 3]) * scale);
              v.z = ptx::pack_half2(f16, __uint_as_float(r0[8 * j + 4]) * scale, __uint_as_float(r0[8 * j + 5]) * scale);
              v.w = ptx::pack_half2(f16, __uint_as_float(r0[8 * j + 6]) * scale, __uint_as_float(r0[8 * j + 7]) * scale);
              *reinterpret_cast<uint4*>(drow + 8 * j) = v;
            }
            if (col0 + 32 + 8 * j < p.N) {
              uint4 v;
              v.x = ptx::pack_half2(f16, __uint_as_float(r1[8 * j + 0]) * scale, __uint_as_float(r1[8 * j + 1]) * scale);
              v.y = ptx::pack_half2(f16, __uint_as_float(r1[8 * j + 2]) * scale, __uint_as_float(r1[8 * j + 3]) * scale);
              v.z = ptx::pack_half2(f16, __uint_as_float(r1[8 * j + 4]) * scale, __uint_as_float(r1[8 * j + 5]) * scale);
              v.w = ptx::pack_half2(f16, __uint_as_float(r1[8 * j + 6]) * scale, __uint_as_float(r1[8 * j + 7]) * scale);
              *reinterpret_cast<uint4*>(drow + 32 + 8 * j) = v;
            }
          }
        }
      }
    }
    if constexpr (Cfg::SCATTER) {
      // every row this warp had is written (each lane waits for its own copies); the last warp of
      // the grid tells every owner
      ptx::bulk_wait<0>();
      ptx::fence_proxy_async_all();
      ptx::fence_acq_rel_sys();
      __syncwarp();
      if (lane == 0) {
        if (ptx::atom_add_acq_rel_sys(p.local_cnt, 1u) == gridDim.x * 4u - 1u) {
          *p.local_cnt = 0;
          for (int d = 0; d < p.world; ++d) ptx::st_release_sys(p.sc_flags[d] + p.rank, p.epoch);
        }
      }
    }
  } else {
    // ------------------------------------------------------------------ gathered-A producers (warps 8..11)
    if constexpr (Cfg::GATHER) {
      const int i = threadIdx.x - 256;            // row of the tile this thread fetches
      const uint8_t* tokens = reinterpret_cast<const uint8_t*>(p.a_tokens);
      const int64_t row_bytes = static_cast<int64_t>(p.K) * Cfg::ELT;
      int stage = 0, cursor = 0, ready_src = -1;
      uint32_t phase = 0;
      for (int t = blockIdx.x; t < total_tiles; t += gridDim.x) {
        if (*abort_word) break;   // a wait gave up: issue nothing more
        const GroupedTile g = grouped_decode(p, t, cursor, n_tiles, BM, BN);
        if (g.src >= 0 && g.src != ready_src) {
          // tokens of this source must have landed (sub-problems are ordered by source, own first)
          if (lane == 0) flag_wait_ge(wc, p.ag_flags[p.rank] + g.src, p.epoch, kSiteMoeFlag);
          __syncwarp();
          ready_src = g.src;
        }
        const bool valid = i < g.rows;
        const uint8_t* src_row = tokens;
        if (valid) src_row = tokens + static_cast<int64_t>(p.gather_index[g.row0 + i]) * row_bytes;
        for (int kb = 0; kb < k_blocks; ++kb) {
          mbar_wait(wc, empty_bar(stage), phase ^ 1u, kSiteSmemEmpty);
          const uint32_t dst = smem_base + stage * Cfg::STAGE_BYTES + i * 128;
          if (valid) {
            const uint8_t* s = src_row + static_cast<int64_t>(kb) * 128;
            const int64_t left = row_bytes - static_cast<int64_t>(kb) * 128;   // bytes of the row still in range
#pragma unroll
            for (int c = 0; c < 8; ++c) {
              const uint32_t n = left >= (c + 1) * 16 ? 16u : 0u;             // zero-fill past K
              ptx::cp_async_16(dst + ((c ^ (i & 7)) << 4), s + c * 16, n);
            }
          }
          ptx::cp_async_mbar_arrive_noinc(full_bar(stage));
          if (++stage == STAGES) {
            stage = 0;
            phase ^= 1u;
          }
        }
      }
    }
  }

  __syncwarp();
  if (*abort_word) {
    // a wait gave up and the roles left their loops early: let copies and MMAs in flight land
    // before this CTA's shared memory and TMEM go away
    const uint64_t t0 = ptx::globaltimer_ns();
    while (ptx::globaltimer_ns() - t0 < 200000ull) __nanosleep(2000);
  }
  ptx::tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    ptx::tc_fence_after();
    ptx::tmem_dealloc<1>(tmem_base, 512);
  }

  if constexpr (Cfg::SCATTER) {
    // ---------------------------------------------------------------- top-k sum of this rank's tokens
    // The slots of a token are topk consecutive rows of the staging buffer: one warp per token, 16
    // bytes per lane and trip, all k loads of a trip in flight before the first add.
    if (static_cast<int>(threadIdx.x) < p.world)
      flag_wait_ge(wc, p.sc_flags[p.rank] + threadIdx.x, p.epoch, kSiteMoeFlag);
    __syncthreads();
    const bool f16 = p.out_f16 != 0;
    const uint16_t* mine = p.sc_stage[p.rank];
    const int chunks = p.N / 8;
    const int gwarp = blockIdx.x * (Cfg::THREADS / 32) + warp, nwarps = gridDim.x * (Cfg::THREADS / 32);
    for (int tl = gwarp; tl < p.tokens_per_rank; tl += nwarps) {
      const uint16_t* trow = mine + static_cast<int64_t>(tl) * p.topk * p.N;
      for (int c = lane; c < chunks; c += 32) {
        float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
        for (int k0 = 0; k0 < p.topk; k0 += 8) {
          uint4 v[8];
#pragma unroll
          for (int j = 0; j < 8; ++j)
            if (k0 + j < p.topk) v[j] = ptx::ld_global_cs_v4(trow + static_cast<int64_t>(k0 + j) * p.N + c * 8);
#pragma unroll
          for (int j = 0; j < 8; ++j) {
            if (k0 + j < p.topk) {
              const uint32_t w[4] = {v[j].x, v[j].y, v[j].z, v[j].w};
#pragma unroll
              for (int e = 0; e < 4; ++e) {
                acc[2 * e] += ptx::half_bits_to_float(static_cast<uint16_t>(w[e] & 0xFFFFu), f16);
                acc[2 * e + 1] += ptx::half_bits_to_float(static_cast<uint16_t>(w[e] >> 16), f16);
              }
            }
          }
        }
        uint4 o;
        o.x = ptx::pack_half2(f16, acc[0], acc[1]);
        o.y = ptx::pack_half2(f16, acc[2], acc[3]);
        o.z = ptx::pack_half2(f16, acc[4], acc[5]);
        o.w = ptx::pack_half2(f16, acc[6], acc[7]);
        *reinterpret_cast<uint4*>(p.sc_out + static_cast<int64_t>(tl) * p.N + c * 8) = o;
      }
    }
  }
}

}  // namespace fluxb
