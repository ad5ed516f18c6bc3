// Host side of the dense GEMM family (GemmOnly, AG+GEMM, GEMM+RS): argument checks, tensor
// maps, tile-shape choice and the launch of dense_gemm_kernel.
#include "../include/fluxb.h"
#include "../runtime/host_common.h"
#include "../sm100/gemm_dense.cuh"

#include <atomic>
#include <cstdlib>
#include <mutex>

namespace fluxb {

std::atomic<uint64_t> g_launches{0};

// Wave counters for launches whose caller brings none: a small pool per device, zeroed once. A
// slot belongs to one stream (launches of a stream run one after the other, and each leaves its
// counter at zero), so launches that overlap on the GPU never share a word. A process that uses
// more streams than slots gets no counter for the extra ones (those launches run free).
namespace {
constexpr int kWaveSlots = 64;
std::mutex g_wave_mu;
uint32_t* g_wave_pool[64] = {nullptr};
cudaStream_t g_wave_owner[64][kWaveSlots];
int g_wave_used[64] = {0};
}  // namespace

uint32_t* wave_counter_for(cudaStream_t stream) {
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return nullptr;
  std::lock_guard<std::mutex> lock(g_wave_mu);
  if (g_wave_pool[dev] == nullptr) {
    uint32_t* p = nullptr;
    if (cudaMalloc(&p, kWaveSlots * 128) != cudaSuccess) return nullptr;
    cudaMemset(p, 0, kWaveSlots * 128);
    g_wave_pool[dev] = p;
  }
  for (int i = 0; i < g_wave_used[dev]; ++i)
    if (g_wave_owner[dev][i] == stream) return g_wave_pool[dev] + i * 32;
  if (g_wave_used[dev] == kWaveSlots) return nullptr;
  const int i = g_wave_used[dev]++;
  g_wave_owner[dev][i] = stream;
  return g_wave_pool[dev] + i * 32;
}

namespace {

// coop: the launch carries the cooperative attribute, so the grid only starts when all of its CTAs
// can be resident together (and the launch fails, instead of waiting forever inside the kernel, when
// they never can). Every launch whose CTAs wait for one another or for peers asks for it.
template <class Cfg>
int launch_dense(const DenseGemmParams& p, int grid, cudaStream_t stream, bool coop = false) {
  constexpr int kThreads = Cfg::THREADS;
  static bool configured[64] = {false};
  int dev = 0;
  FLUXB_CUDA_OK(cudaGetDevice(&dev));
  if (dev >= 64 || !configured[dev]) {
    FLUXB_CUDA_OK(cudaFuncSetAttribute(dense_gemm_kernel<Cfg>,
                                       cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg::SMEM_BYTES));
    if (dev < 64) configured[dev] = true;
  }
  {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(grid, 1, 1);
    cfg.blockDim = dim3(kThreads, 1, 1);
    cfg.dynamicSmemBytes = Cfg::SMEM_BYTES;
    cfg.stream = stream;
    cudaLaunchAttribute attr[2];
    int na = 0;
    if constexpr (Cfg::CG == 2) {
      attr[na].id = cudaLaunchAttributeClusterDimension;
      attr[na].val.clusterDim.x = 2;
      attr[na].val.clusterDim.y = 1;
      attr[na].val.clusterDim.z = 1;
      ++na;
    }
    if (coop) {
      attr[na].id = cudaLaunchAttributeCooperative;
      attr[na].val.cooperative = 1;
      ++na;
    }
    cfg.attrs = attr;
    cfg.numAttrs = na;
    FLUXB_CUDA_OK(cudaLaunchKernelEx(&cfg, dense_gemm_kernel<Cfg>, p));
  }
  FLUXB_CUDA_OK(cudaGetLastError());
  g_launches.fetch_add(1, std::memory_order_relaxed);
  return kOk;
}

}  // namespace
}  // namespace fluxb

using namespace fluxb;

extern "C" uint64_t fluxb_launch_count(void) { return g_launches.load(); }

// Zero the launcher's wave-counter pool of the current device (after a launch was cut short by a
// timed-out wait; a completed launch leaves its counter at zero by itself). Synchronises the device.
extern "C" int fluxb_reset_wave_counters(void) {
  int dev = 0;
  FLUXB_CUDA_OK(cudaGetDevice(&dev));
  FLUXB_CUDA_OK(cudaDeviceSynchronize());
  std::lock_guard<std::mutex> lock(g_wave_mu);
  if (dev >= 0 && dev < 64 && g_wave_pool[dev] != nullptr)
    FLUXB_CUDA_OK(cudaMemset(g_wave_pool[dev], 0, kWaveSlots * 128));
  return kOk;
}

static int dense_impl(const fluxb_dense_args_t* a, const fluxb_a2a_args_t* x);

extern "C" int fluxb_dense_gemm(const fluxb_dense_args_t* a) {
  FLUXB_REQUIRE(a != nullptr, "null args");
  FLUXB_REQUIRE(a->mode >= FLUXB_PLAIN && a->mode <= FLUXB_REDUCE_SCATTER, "mode");
  return dense_impl(a, nullptr);
}

// Reduce-scatter with bands that span two segments: whether the first visited segment is a group of
// its own, so that the last one (the own segment) is too: W even -> 1 | 2 2 ... 2 | 1, W odd -> 2 ... 2 | 1.
extern "C" int fluxb_rs_solo_first(int32_t num_seg) { return num_seg % 2 == 0 ? 1 : 0; }

// The last, partial wave: its tiles are cut into 2 or 4 column pieces when all the pieces still fit one
// wave of `slots` CTAs (or CTA pairs); a problem smaller than one wave is all "last wave". mode: 0 = never,
// 1 = halves or quarters, 2 = halves only. Returns the first tile that is cut and the shift (pieces = 1 << shift).
extern "C" int fluxb_tail_split(int64_t tiles, int64_t slots, int32_t mode, int32_t* split_from, int32_t* split_shift) {
  FLUXB_REQUIRE(tiles >= 0 && slots >= 1 && split_from != nullptr && split_shift != nullptr, "tail split arguments");
  *split_from = static_cast<int32_t>(tiles);
  *split_shift = 0;
  const int64_t rest = tiles % slots;
  if (mode == 0 || rest == 0) return kOk;
  int shift = 0;
  if (4 * rest <= slots) shift = 2;
  else if (2 * rest <= slots) shift = 1;
  if (mode == 2 && shift > 1) shift = 1;
  *split_from = static_cast<int32_t>(tiles - rest);
  *split_shift = shift;
  return kOk;
}

// The tile order of the dense kernel, evaluated on the host by the same function the kernel
// calls: out[3 * t .. 3 * t + 2] = (segment, tile row inside the segment, first column) of tile t.
extern "C" int fluxb_decode_tiles(int32_t num_seg, int32_t seg_first, int32_t m_tiles_seg, int32_t n_tiles,
                                  int32_t group_m, int32_t seg_span, int32_t seg_solo_first, int32_t bm,
                                  int32_t bn, int32_t* out, int32_t n) {
  FLUXB_REQUIRE(out != nullptr && num_seg >= 1 && m_tiles_seg >= 1 && n_tiles >= 1 && group_m >= 1, "tile grid");
  FLUXB_REQUIRE(n <= num_seg * m_tiles_seg * n_tiles, "more tiles asked for than the grid has");
  DenseGemmParams p;
  memset(&p, 0, sizeof(p));
  p.num_seg = num_seg;
  p.seg_first = seg_first;
  p.group_m = group_m;
  p.seg_span = seg_span;
  p.seg_solo_first = seg_solo_first;
  for (int t = 0; t < n; ++t) {
    const TileCoord c = decode_tile(p, t, m_tiles_seg, n_tiles, bm, bn);
    out[3 * t] = c.seg;
    out[3 * t + 1] = c.m_tile;
    out[3 * t + 2] = c.n0;
  }
  return kOk;
}

// The same for the work items of a launch whose last wave is cut into column pieces (split_from /
// split_shift as fluxb_tail_split returns them): out[4 * t .. 4 * t + 3] = (segment, tile row, first column,
// shift) of work item t; an item is bn >> shift columns wide.
extern "C" int fluxb_decode_work_items(int32_t num_seg, int32_t seg_first, int32_t m_tiles_seg, int32_t n_tiles,
                                       int32_t group_m, int32_t seg_span, int32_t seg_solo_first, int32_t bm,
                                       int32_t bn, int32_t split_from, int32_t split_shift, int32_t* out, int32_t n) {
  FLUXB_REQUIRE(out != nullptr && num_seg >= 1 && m_tiles_seg >= 1 && n_tiles >= 1 && group_m >= 1, "tile grid");
  const int64_t tiles = static_cast<int64_t>(num_seg) * m_tiles_seg * n_tiles;
  FLUXB_REQUIRE(split_from >= 0 && split_from <= tiles && split_shift >= 0 && split_shift <= 2, "split");
  FLUXB_REQUIRE(n <= split_from + ((tiles - split_from) << split_shift), "more work items asked for than there are");
  DenseGemmParams p;
  memset(&p, 0, sizeof(p));
  p.num_seg = num_seg;
  p.seg_first = seg_first;
  p.group_m = group_m;
  p.seg_span = seg_span;
  p.seg_solo_first = seg_solo_first;
  p.split_from = split_from;
  p.split_shift = split_shift;
  for (int t = 0; t < n; ++t) {
    const TileCoord c = decode_tile(p, t, m_tiles_seg, n_tiles, bm, bn);
    out[4 * t] = c.seg;
    out[4 * t + 1] = c.m_tile;
    out[4 * t + 2] = c.n0;
    out[4 * t + 3] = c.shift;
  }
  return kOk;
}

extern "C" int fluxb_ulysses_gemm(const fluxb_a2a_args_t* x) {
  FLUXB_REQUIRE(x != nullptr, "null args");
  FLUXB_REQUIRE(x->base.mode == FLUXB_GEMM_A2A || x->base.mode == FLUXB_A2A_GEMM, "mode");
  return dense_impl(&x->base, x);
}

// (hd, seq, head, batch)-ordered 4-D map over a head-sharded activation buffer
static int encode_heads_map(CUtensorMap* out, const void* base, int layout, int hd, int seq, int heads,
                            int bs, uint32_t box_inner, Swz swz) {
  const uint64_t e = 2;
  uint64_t dims[4] = {static_cast<uint64_t>(hd), static_cast<uint64_t>(seq),
                      static_cast<uint64_t>(heads), static_cast<uint64_t>(bs)};
  uint64_t str[3];
  if (layout == 0) {  // [bs, heads, seq, hd]
    str[0] = hd * e;
    str[1] = static_cast<uint64_t>(seq) * hd * e;
  } else {            // [bs, seq, heads, hd]
    str[0] = static_cast<uint64_t>(heads) * hd * e;
    str[1] = hd * e;
  }
  str[2] = static_cast<uint64_t>(heads) * seq * hd * e;
  uint32_t box[4] = {box_inner, 32, 1, 1};
  return encode_tmap(out, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 4, base, dims, str, box, swz);
}

static int dense_impl(const fluxb_dense_args_t* a, const fluxb_a2a_args_t* x) {
  FLUXB_REQUIRE(a != nullptr, "null args");
  FLUXB_REQUIRE(a->M > 0 && a->N > 0 && a->K > 0, "empty problem");
  FLUXB_REQUIRE(a->in_dtype == FLUXB_BF16 || a->in_dtype == FLUXB_FP8_E4M3 ||
                    a->in_dtype == FLUXB_FP16 || a->in_dtype == FLUXB_FP8_E5M2 || a->in_dtype == FLUXB_INT8,
                "input dtype");
  FLUXB_REQUIRE(a->out_dtype == FLUXB_BF16 || a->out_dtype == FLUXB_FP16, "output dtype");
  FLUXB_REQUIRE(a->world >= 1 && a->world <= FLUXB_MAX_RANKS, "world size 1..8");
  FLUXB_REQUIRE(a->rank >= 0 && a->rank < a->world, "rank");
  const bool in16 = a->in_dtype == FLUXB_BF16 || a->in_dtype == FLUXB_FP16;
  const int elt = in16 ? 2 : 1;
  const bool multi = a->world > 1 && a->mode != FLUXB_PLAIN;
  const bool a2a = a->mode == FLUXB_GEMM_A2A || a->mode == FLUXB_A2A_GEMM;
  const bool segmented = multi && !a2a;   // M is cut into one segment per rank
  FLUXB_REQUIRE((a->K * elt) % 16 == 0, "K row bytes must be a multiple of 16");
  FLUXB_REQUIRE(a->N % 8 == 0, "N must be a multiple of 8");
  if (segmented) FLUXB_REQUIRE(a->M % a->world == 0, "M must divide evenly over ranks");

  DenseGemmParams p;
  memset(&p, 0, sizeof(p));
  p.M = a->M;
  p.N = a->N;
  p.K = a->K;
  p.rank = a->rank;
  p.world = a->world;
  p.mode = (multi || a2a) ? a->mode : kModePlain;
  p.num_seg = segmented ? a->world : 1;
  p.seg_rows = a->M / p.num_seg;
  p.epoch = a->epoch;
  p.timeout_ns = a->timeout_ns ? a->timeout_ns : 2000000000ull;
  p.status = reinterpret_cast<Status*>(a->status);
  p.bias = a->bias;
  p.trace = a->trace;
  p.bias_row_stride = a->bias_row_stride;
  p.scale_a = a->scale_a;
  p.scale_b = a->scale_b;
  p.scale_flags = a->scale_flags & 3u;
  FLUXB_REQUIRE(!(a->scale_flags & 1u) || a->scale_a, "per-row scale vector missing");
  FLUXB_REQUIRE(!(a->scale_flags & 2u) || a->scale_b, "per-column scale vector missing");
  p.sa = a->sa;
  p.sb = a->sb;
  p.sb_groupwise = a->blockscale == 2 ? 1 : 0;
  p.b_kn = a->b_kn ? 1 : 0;
  FLUXB_REQUIRE(!a->b_kn || (in16 && !a->blockscale), "a [K, N] weight is read in place for 16-bit inputs only");
  FLUXB_REQUIRE(!a->b_kn || (a->ldb % 8 == 0 && a->N % 8 == 0), "[K, N] weight: N and its row pitch in multiples of 8");
  p.ab_fmt = (a->in_dtype == FLUXB_BF16 || a->in_dtype == FLUXB_FP8_E5M2 || a->in_dtype == FLUXB_INT8) ? 1 : 0;
  p.out_f16 = a->out_dtype == FLUXB_FP16 ? 1 : 0;
  p.act = a->act;

  int bn = a->tile_n;
  if (bn == 0) bn = (a->N % 256 == 0 || a->N > 2048) ? 256 : 128;
  FLUXB_REQUIRE(bn == 128 || bn == 192 || bn == 256, "tile_n must be 128, 192 or 256");
  int cg = a->cta_group;
  FLUXB_REQUIRE(cg >= 0 && cg <= 2, "cta_group must be 0 (auto), 1 or 2");
  if (cg == 0) cg = 1;
  if (a->blockscale) {
    FLUXB_REQUIRE(a->in_dtype == FLUXB_FP8_E4M3, "block-scaled GEMM takes e4m3 operands");
    FLUXB_REQUIRE(a->sa && a->sb, "block scales missing");
    FLUXB_REQUIRE(a->K % 128 == 0 && a->N % 128 == 0, "block-scaled GEMM needs K and N multiples of 128");
    // (one rank: the last row block may be partial - its scales exist, its rows are clipped)
    FLUXB_REQUIRE(!multi || (a->M / a->world) % 128 == 0,
                  "block-scaled fused ops need rows per rank in multiples of 128");
    // Single CTAs on 128 x 128 tiles. CTA pairs on 256 x 128 tiles (half of B per CTA) exist and are
    // chosen by cta_group = 2, but measured slower (977 against 1128 TFLOP/s at 16384 x 3584 x 8192): the
    // k-block hand-over then waits for the slowest of sixteen promotion warps on two SMs.
    cg = (a->cta_group == 2 && a->tile_n != 256 && a->M / (multi ? a->world : 1) >= 256) ? 2 : 1;
    // 128 x 256 tiles wherever N allows (tile_n = 128 pins the narrow ones): 1330 - 1350 against 1010 - 1060
    // TFLOP/s. Per-tensor fp8 GEMMs on 128 x 128 tiles stop at 1450 TFLOP/s here (the operand stream into the
    // SM is the bound), on 128 x 256 at 2600.
    bn = (cg == 1 && a->tile_n != 128 && (a->N % 256 == 0 || a->N >= 2048)) ? 256 : 128;
  } else if (a->mode == FLUXB_A2A_GEMM) {
    if (cg == 2 && a->M >= 256) bn = 256;
    else { cg = 1; bn = 128; }
  } else if (multi && a->mode == FLUXB_ALLGATHER) {
    // the all-gather variants exist for CTA pairs on 256-wide tiles and single CTAs on 128-wide
    if (cg == 2 && a->M / a->world >= 256) bn = 256;
    else { cg = 1; bn = 128; }
  }
  // int8 is built for 256-wide CTA-pair tiles and 128-wide tiles only
  if (a->in_dtype == FLUXB_INT8 && !a->blockscale && !(cg == 2 && bn == 256)) bn = 128;
  // 512-row tiles (two MMAs per k-step on one B tile): CTA pairs on 256 columns, 16-bit and fp8 inputs,
  // segments that 512 rows tile without much padding
  int mt = 1;
  {
    static const int tile_m_env = [] {
      const char* e = getenv("FLUXB_TILE_M");
      return e ? atoi(e) : 0;
    }();
    const int want = a->tile_m > 0 ? a->tile_m : tile_m_env;
    const int seg_rows = a->M / (segmented ? a->world : 1);
    const bool can = cg == 2 && bn == 256 && !a->blockscale && !a2a && a->in_dtype != FLUXB_INT8 && seg_rows >= 512;
    if (want > 0) {
      // (512 is honoured where the mode, the types and the rows allow it; elsewhere - the Ulysses projections,
      // short segments - it falls back to one MMA per k-step)
      FLUXB_REQUIRE(want == 128 * cg || want == 512,
                    "tile_m must be 128 * cta_group, or 512 for CTA pairs on 256-column tiles");
      mt = (want == 512 && can) ? 2 : 1;
    } else if (can && (seg_rows % 512 == 0 || seg_rows >= 4096)) {
      mt = 2;
    }
  }
  FLUXB_REQUIRE(!a->b_kn || (bn / cg) % 64 == 0,
                "[K, N] weight: 64-column operand boxes need tile_n / cta_group in multiples of 64");
  const int bm = 128 * cg * mt;
  const int bk = 128 / elt;
  const CUtensorMapDataType in_dt =
      in16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_UINT8;
  const CUtensorMapDataType out_dt = CU_TENSOR_MAP_DATA_TYPE_BFLOAT16;  // any 16-bit type moves alike

  int rc;
  // ---- A
  {
    const uint64_t rows = (p.mode == kModeAllGather) ? p.seg_rows : a->M;
    const void* a_base = a->a;
    int64_t lda = a->lda;
    if (p.mode == kModeA2AGemm) {
      a_base = x->land[a->rank];
      lda = a->K;
    }
    uint64_t dims[2] = {static_cast<uint64_t>(a->K), rows};
    uint64_t str[1] = {static_cast<uint64_t>(lda) * elt};
    uint32_t box[2] = {static_cast<uint32_t>(bk), static_cast<uint32_t>(128 * mt)};
    if ((rc = encode_tmap(&p.tm_a, in_dt, 2, a_base, dims, str, box, Swz::B128))) return rc;
  }
  if (a2a) {
    FLUXB_REQUIRE(in16, "the Ulysses projections run on bf16 / fp16");
    FLUXB_REQUIRE(x->hd == 64 || x->hd == 128, "head_dim must be 64 or 128");
    FLUXB_REQUIRE(x->local_seq % 32 == 0, "the local sequence length must be a multiple of 32");
    FLUXB_REQUIRE(a->M == x->bs * x->local_seq, "M must equal bs * local_seq");
    FLUXB_REQUIRE(a->local_cnt != nullptr, "local arrival scratch missing");
    p.local_cnt = a->local_cnt;
    p.a2a_hd = x->hd;
    p.a2a_local_seq = x->local_seq;
    p.a2a_bs = x->bs;
    const int seq = x->local_seq * a->world;
    for (int r = 0; r < a->world; ++r) {
      FLUXB_REQUIRE(x->a2a_flags[r] != nullptr, "all-to-all flags missing");
      p.a2a_flags[r] = x->a2a_flags[r];
    }
    if (p.mode == kModeGemmA2A) {
      FLUXB_REQUIRE(x->groups >= 1 && x->groups <= kMaxHeadGroups, "1..3 head groups");
      p.a2a_groups = x->groups;
      int start = 0;
      for (int g = 0; g < x->groups; ++g) {
        FLUXB_REQUIRE(x->group_heads[g] > 0 && x->group_heads[g] % a->world == 0,
                      "heads of every group must divide over the ranks");
        p.a2a_group_start[g] = start;
        start += x->group_heads[g];
        for (int r = 0; r < a->world; ++r) {
          FLUXB_REQUIRE(x->out[g][r] != nullptr, "output buffer missing");
          if ((rc = encode_heads_map(&p.tm_a2a[g * kMaxRanks + r], x->out[g][r], x->layout, x->hd, seq,
                                     x->group_heads[g] / a->world, x->bs, 64, Swz::B128)))
            return rc;
        }
      }
      p.a2a_group_start[x->groups] = start;
      FLUXB_REQUIRE(start * x->hd == a->N, "N must equal total heads * head_dim");
    } else {
      FLUXB_REQUIRE(a->K % (a->world * x->hd) == 0, "K must equal heads * head_dim with heads divisible by W");
      p.a2a_local_heads = a->K / x->hd / a->world;
      FLUXB_REQUIRE(x->attn != nullptr, "attention output missing");
      p.a2a_attn = x->attn;
      p.a2a_layout = x->layout;
      // the own slice is read in place when a 128-row tile never straddles two batches
      p.a2a_copy_local = (x->copy_local || !(x->bs == 1 || x->local_seq % 128 == 0)) ? 1 : 0;
      {
        const uint64_t e = 2;
        const uint64_t lh = static_cast<uint64_t>(p.a2a_local_heads);
        uint64_t dims[4] = {static_cast<uint64_t>(x->hd), static_cast<uint64_t>(seq), lh,
                            static_cast<uint64_t>(x->bs)};
        uint64_t str[3];
        if (x->layout == 0) {
          str[0] = x->hd * e;
          str[1] = static_cast<uint64_t>(seq) * x->hd * e;
        } else {
          str[0] = lh * x->hd * e;
          str[1] = x->hd * e;
        }
        str[2] = lh * seq * x->hd * e;
        uint32_t box[4] = {64, 128, 1, 1};
        if ((rc = encode_tmap(&p.tm_a_own, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 4, x->attn, dims, str, box,
                              Swz::B128)))
          return rc;
      }
      for (int r = 0; r < a->world; ++r) {
        FLUXB_REQUIRE(x->land[r] != nullptr, "landing buffer missing");
        p.a2a_land[r] = x->land[r];
      }
      {
        // own landing buffer, one slab per source: (hd, M, head, source)
        const uint64_t e = 2;
        const uint64_t lh = static_cast<uint64_t>(p.a2a_local_heads);
        const uint64_t Mr = static_cast<uint64_t>(a->M);
        uint64_t dims[4] = {static_cast<uint64_t>(x->hd), Mr, lh, static_cast<uint64_t>(a->world)};
        uint64_t str[3];
        if (x->layout == 0) {
          str[0] = x->hd * e;
          str[1] = Mr * x->hd * e;
        } else {
          str[0] = lh * x->hd * e;
          str[1] = x->hd * e;
        }
        str[2] = lh * Mr * x->hd * e;
        uint32_t box[4] = {64, 128, 1, 1};
        if ((rc = encode_tmap(&p.tm_a_land4, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 4, x->land[a->rank], dims, str,
                              box, Swz::B128)))
          return rc;
      }
    }
  }
  if (p.mode == kModeAllGather) {
    FLUXB_REQUIRE(a->ag_land[a->rank] != nullptr, "all-gather landing buffer missing");
    uint64_t dims[2] = {static_cast<uint64_t>(a->K), static_cast<uint64_t>(a->M)};
    uint64_t str[1] = {static_cast<uint64_t>(a->K) * elt};
    uint32_t box[2] = {static_cast<uint32_t>(bk), static_cast<uint32_t>(128 * mt)};
    if ((rc = encode_tmap(&p.tm_a_land, in_dt, 2, a->ag_land[a->rank], dims, str, box, Swz::B128)))
      return rc;
    FLUXB_REQUIRE(a->lda == a->K, "all-gather input shard must be contiguous");
    p.ag_src = a->a;
    for (int r = 0; r < a->world; ++r) {
      p.ag_land[r] = a->ag_land[r];
      p.ag_flags[r] = a->ag_flags[r];
      FLUXB_REQUIRE(p.ag_land[r] && p.ag_flags[r], "all-gather peer pointers missing");
      if (a->blockscale) {
        FLUXB_REQUIRE(a->ag_scale_land[r] != nullptr, "all-gather scale landing buffers missing");
        p.ag_scale_land[r] = a->ag_scale_land[r];
      }
    }
    p.ag_scale_src = a->sa;
    p.sa_land = a->ag_scale_land[a->rank];
  }
  // ---- D
  {
    uint32_t box[3] = {64, 32, 1};
    if (p.mode == kModeReduceScatter) {
      FLUXB_REQUIRE(a->rs_out != nullptr, "reduce-scatter output missing");
      {
        // Two ranks: the own tiles add the peer's slab in their epilogue. Three and more: the own tiles go to
        // the own staging slab and a tail of the same kernel sums the W slabs (FLUXB_RS_TAIL=0 / 1 overrides).
        static const int tail_env = [] {
          const char* e = getenv("FLUXB_RS_TAIL");
          return e ? atoi(e) : -1;
        }();
        // (in the block-scaled variants, whose warps 0-3 have given their registers away, the eight promotion
        // warps run the tail)
        p.rs_tail = (multi && (tail_env >= 0 ? tail_env != 0 : a->world >= 3)) ? 1 : 0;
        p.rs_claim = a->wave_ctr ? a->wave_ctr + 1 : nullptr;
      }
      for (int r = 0; r < a->world; ++r) {
        FLUXB_REQUIRE(a->rs_stage[r] && a->rs_ctr[r], "reduce-scatter peer pointers missing");
        // peers: their staging slabs [W][seg_rows][N]; own entry without the tail: the output, as a single
        // slab (the own segment's tiles add the peers' slabs in their epilogue and store the result)
        const bool own = r == a->rank && !p.rs_tail;
        uint64_t dims[3] = {static_cast<uint64_t>(a->N), static_cast<uint64_t>(p.seg_rows),
                            own ? 1ull : static_cast<uint64_t>(a->world)};
        uint64_t str[2] = {static_cast<uint64_t>(a->N) * 2,
                           static_cast<uint64_t>(a->N) * 2 * p.seg_rows};
        if ((rc = encode_tmap(&p.tm_d[r], out_dt, 3, own ? a->rs_out : a->rs_stage[r], dims,
                              str, box, Swz::B128)))
          return rc;
        p.rs_ctr[r] = a->rs_ctr[r];
      }
      p.rs_stage = a->rs_stage[a->rank];
      p.rs_out = a->rs_out;
    } else if (p.mode != kModeGemmA2A) {
      void* out = a->d ? a->d : a->rs_out;
      const int64_t ldd = a->d ? a->ldd : a->N;
      FLUXB_REQUIRE(out != nullptr, "output missing");
      uint64_t dims[3] = {static_cast<uint64_t>(a->N), static_cast<uint64_t>(p.seg_rows),
                          static_cast<uint64_t>(p.num_seg)};
      uint64_t str[2] = {static_cast<uint64_t>(ldd) * 2, static_cast<uint64_t>(ldd) * 2 * p.seg_rows};
      if ((rc = encode_tmap(&p.tm_d[0], out_dt, 3, out, dims, str, box,
                            Swz::B128)))
        return rc;
    }
  }
  if (multi) {
    FLUXB_REQUIRE(a->local_cnt != nullptr, "local arrival scratch missing");
    p.local_cnt = a->local_cnt;
    for (int r = 0; r < a->world; ++r) {
      FLUXB_REQUIRE(a->start_ctr[r] != nullptr, "start counters missing");
      p.start_ctr[r] = a->start_ctr[r];
    }
  }
  // segment visiting order: all-gather starts with the own shard, reduce-scatter ends with it
  p.seg_first = 0;
  if (p.mode == kModeAllGather) p.seg_first = a->rank;
  if (p.mode == kModeReduceScatter) p.seg_first = (a->rank + 1) % a->world;

  // arrival flags of the pushes cover about 32 MB of a shard each (one flag per shard when it is
  // smaller): few enough that counting the pushing warps stays cheap, fine enough for big shards
  {
    const int64_t row_b = p.mode == kModeA2AGemm ? static_cast<int64_t>(a->K / a->world) * elt
                                                 : static_cast<int64_t>(a->K) * elt;
    static const int unit_mb_env = [] {
      const char* e = getenv("FLUXB_AG_UNIT_MB");
      return e ? atoi(e) : 0;
    }();
    int64_t unit = (static_cast<int64_t>(unit_mb_env > 0 ? unit_mb_env : 32) << 20) / (row_b > 0 ? row_b : 1);
    unit = (unit + bm - 1) / bm * bm;
    const int64_t seg_round = (static_cast<int64_t>(p.seg_rows) + bm - 1) / bm * bm;
    if (unit > seg_round || unit * 3 / 2 > seg_round) unit = seg_round;
    // the post-attention exchange is short next to its GEMM: 1024-row units let the first wave of
    // tiles start on the first quarter of what arrives
    if (p.mode == kModeA2AGemm && seg_round >= 2048) unit = 1024;
    p.flag_unit_rows = static_cast<int32_t>(unit);
  }
  const int m_tiles_seg = (p.seg_rows + bm - 1) / bm;
  p.group_m = a->group_m > 0 ? a->group_m : 16 / cg;
  // post-attention: the first wave of tiles should need as few rows of the exchange as possible
  if (p.mode == kModeA2AGemm && a->world > 1 && p.group_m > 4) p.group_m = 4;
  {
    static const int inflight_env = [] {
      const char* e = getenv("FLUXB_AG_INFLIGHT");
      return e ? atoi(e) : 0;
    }();
    // Three loads ahead move the shards fastest, but tiles that run while 7/8 of A is arriving are
    // slowed by it; with many ranks a paced push (one load at a time, 176 MB in ~520 us instead
    // of ~300 us at 8 ranks) gave the shorter kernel (0.958 against 1.043 ms), with two ranks the
    // fast one did (3.94-4.02 against 4.10-4.12 ms).
    p.ag_inflight = inflight_env > 0 ? inflight_env : (a->world > 2 ? 1 : 3);
  }
  {
    static const int hints_env = [] {
      const char* e = getenv("FLUXB_L2_HINTS");
      return e ? atoi(e) : 0;
    }();
    p.l2_hints = hints_env;
  }
  // segmented modes: a raster band may span two consecutive segments when one segment has fewer
  // tile rows than the band (the own shard of the all-gather stays alone: it is all there is at first)
  p.seg_span = 1;
  {
    static const int pair_env = [] {
      const char* e = getenv("FLUXB_SEG_PAIR");
      return e ? atoi(e) : 1;
    }();
    if (segmented && pair_env != 0 && p.num_seg >= 3 && p.group_m > m_tiles_seg) {
      p.seg_span = 2;
      p.seg_solo_first = p.mode == kModeAllGather ? 1 : 0;
      // Reduce-scatter: the own segment (visited last) must stay a group of its own. Its tiles wait for
      // the peers' partial tiles; in a band shared with another segment such a wait would sit in front of
      // partial tiles that a peer's own tiles wait for in turn, and the ranks would wait in a circle.
      if (p.mode == kModeReduceScatter) p.seg_solo_first = fluxb_rs_solo_first(p.num_seg);
    }
  }
  if (p.group_m > p.seg_span * m_tiles_seg) p.group_m = p.seg_span * m_tiles_seg;

  int sms = 0;
  if ((rc = device_sm_count(&sms))) return rc;
  if (a->num_sms > 0 && a->num_sms < sms) sms = a->num_sms;
  const int64_t tiles = static_cast<int64_t>(p.num_seg) * m_tiles_seg * ((a->N + bn - 1) / bn);
  int grid = sms;
  // every CTA of a multi-rank launch takes part in the flag protocol, so the grid stays full
  // (a plain launch shrinks to its work items below)
  if (cg == 2) grid &= ~1;
  // ---- the last, partial wave: cut its tiles into 2 or 4 column pieces when all the pieces still
  // fit one wave (a problem smaller than one wave is all "last wave")
  p.split_from = static_cast<int32_t>(tiles);
  p.split_shift = 0;
  {
    static const int split_env = [] {
      const char* e = getenv("FLUXB_TAIL_SPLIT");
      return e ? atoi(e) : 1;
    }();
    if (bn == 256 && !a->blockscale && !a->b_kn)
      if ((rc = fluxb_tail_split(tiles, grid / cg, split_env, &p.split_from, &p.split_shift))) return rc;
  }
  p.total_vtiles = p.split_from + static_cast<int32_t>((tiles - p.split_from) << p.split_shift);
  if (!multi && !a2a && static_cast<int64_t>(p.total_vtiles) * cg < grid) grid = p.total_vtiles * cg;
  // ---- B (the pieces of split tiles load narrower boxes)
  {
    uint64_t dims[2] = {static_cast<uint64_t>(a->K), static_cast<uint64_t>(a->N)};
    uint64_t str[1] = {static_cast<uint64_t>(a->ldb) * elt};
    uint32_t box[2] = {static_cast<uint32_t>(bk), static_cast<uint32_t>(bn / cg)};
    if (a->b_kn) {
      // [K, N], N contiguous: boxes of 64 columns x bk k-rows (128-byte rows along N)
      dims[0] = static_cast<uint64_t>(a->N);
      dims[1] = static_cast<uint64_t>(a->K);
      box[0] = 64;
      box[1] = static_cast<uint32_t>(bk);
    }
    if ((rc = encode_tmap(&p.tm_b, in_dt, 2, a->b, dims, str, box, Swz::B128))) return rc;
    if (p.split_shift >= 1) {
      box[1] = static_cast<uint32_t>(bn / cg / 2);
      if ((rc = encode_tmap(&p.tm_b_half, in_dt, 2, a->b, dims, str, box, Swz::B128))) return rc;
    }
    if (p.split_shift >= 2) {
      box[1] = static_cast<uint32_t>(bn / cg / 4);
      if ((rc = encode_tmap(&p.tm_b_quarter, in_dt, 2, a->b, dims, str, box, Swz::B128))) return rc;
    }
  }

  cudaStream_t stream = reinterpret_cast<cudaStream_t>(a->stream);
  // CTAs that wait for one another (wave-synchronous starts) or for peers (every multi-rank mode) must
  // all be resident: those launches are cooperative unless FLUXB_COOPERATIVE=0
  // (a kernel profiler that replays launches could not replay a cooperative cluster launch here:
  // under an injected profiler the attribute is left off unless FLUXB_COOPERATIVE=1 asks for it)
  static const int coop_env = [] {
    const char* e = getenv("FLUXB_COOPERATIVE");
    if (e) return atoi(e);
    return (getenv("CUDA_INJECTION64_PATH") || getenv("NV_COMPUTE_PROFILER_PERFWORKS_DIR")) ? 0 : 1;
  }();
  bool coop = coop_env != 0 && (multi || a2a);
  {
    // wave-synchronous tile starts pay off when a wave's operands do not fit L2 together
    static const int wave_env = [] {
      const char* e = getenv("FLUXB_WAVE_SYNC");
      return e ? atoi(e) : -1;
    }();
    // (tiles long enough that the bubble at a wave boundary is noise, and more than two waves)
    const int kblocks = (a->K + bk - 1) / bk;
    const bool want = wave_env >= 0 ? wave_env != 0 : kblocks >= 48;
    if (want && p.total_vtiles > 2 * (grid / cg)) p.wave_ctr = a->wave_ctr ? a->wave_ctr : wave_counter_for(stream);
    if (p.wave_ctr != nullptr && coop_env != 0) coop = true;
  }
  if (a->blockscale) {
    if (cg == 2) {
      if (p.mode == kModeAllGather) return launch_dense<DenseCfg<128, 1, 5, 2, 32768, true>>(p, grid, stream, coop);
      return launch_dense<DenseCfg<128, 1, 6, 2, 0, true>>(p, grid, stream, coop);
    }
    if (bn == 256) {
      if (p.mode == kModeAllGather) return launch_dense<DenseCfg<256, 1, 3, 1, 32768, true>>(p, grid, stream, coop);
      return launch_dense<DenseCfg<256, 1, 4, 1, 0, true>>(p, grid, stream, coop);
    }
    if (p.mode == kModeAllGather) return launch_dense<DenseCfg<128, 1, 4, 1, 32768, true>>(p, grid, stream, coop);
    return launch_dense<DenseCfg<128, 1, 5, 1, 0, true>>(p, grid, stream, coop);
  }
  if (p.mode == kModeAllGather || p.mode == kModeA2AGemm) {
    // variants that carry the staging rings of the all-gather / all-to-all push
    if (mt == 2) {
      if (in16) return launch_dense<DenseCfg<256, 0, 4, 2, 16384, false, 2>>(p, grid, stream, coop);
      return launch_dense<DenseCfg<256, 1, 4, 2, 16384, false, 2>>(p, grid, stream, coop);
    }
    if (cg == 2 && bn == 256) {
      if (in16) return launch_dense<DenseCfg<256, 0, 6, 2, 16384>>(p, grid, stream, coop);
      if (a->in_dtype == FLUXB_INT8) return launch_dense<DenseCfg<256, 2, 6, 2, 16384>>(p, grid, stream, coop);
      return launch_dense<DenseCfg<256, 1, 6, 2, 16384>>(p, grid, stream, coop);
    }
    FLUXB_REQUIRE(cg == 1 && bn == 128, "all-gather GEMM runs as CTA pairs on 256-wide tiles or single CTAs on 128-wide tiles");
    if (in16) return launch_dense<DenseCfg<128, 0, 6, 1, 16384>>(p, grid, stream, coop);
    if (a->in_dtype == FLUXB_INT8) return launch_dense<DenseCfg<128, 2, 6, 1, 16384>>(p, grid, stream, coop);
    return launch_dense<DenseCfg<128, 1, 6, 1, 16384>>(p, grid, stream, coop);
  }
  if (a->in_dtype == FLUXB_INT8) {
    // signed 8-bit operands, s32 accumulation (tcgen05 kind::i8)
    if (cg == 2 && bn == 256) return launch_dense<DenseCfg<256, 2, 6, 2>>(p, grid, stream, coop);
    FLUXB_REQUIRE(bn == 128, "int8 runs on 256-wide CTA-pair tiles or 128-wide single-CTA tiles");
    if (cg == 2) return launch_dense<DenseCfg<128, 2, 8, 2>>(p, grid, stream, coop);
    return launch_dense<DenseCfg<128, 2, 6>>(p, grid, stream, coop);
  }
  if (mt == 2) {
    if (in16) return launch_dense<DenseCfg<256, 0, 4, 2, 0, false, 2>>(p, grid, stream, coop);
    return launch_dense<DenseCfg<256, 1, 4, 2, 0, false, 2>>(p, grid, stream, coop);
  }
  if (cg == 2) {
    if (in16) {
      if (bn == 256) return launch_dense<DenseCfg<256, 0, 6, 2>>(p, grid, stream, coop);
      if (bn == 192) return launch_dense<DenseCfg<192, 0, 6, 2>>(p, grid, stream, coop);
      return launch_dense<DenseCfg<128, 0, 8, 2>>(p, grid, stream, coop);
    }
    if (bn == 256) return launch_dense<DenseCfg<256, 1, 6, 2>>(p, grid, stream, coop);
    if (bn == 192) return launch_dense<DenseCfg<192, 1, 6, 2>>(p, grid, stream, coop);
    return launch_dense<DenseCfg<128, 1, 8, 2>>(p, grid, stream, coop);
  }
  if (in16) {
    if (bn == 256) return launch_dense<DenseCfg<256, 0, 4>>(p, grid, stream, coop);
    if (bn == 192) return launch_dense<DenseCfg<192, 0, 4>>(p, grid, stream, coop);
    return launch_dense<DenseCfg<128, 0, 6>>(p, grid, stream, coop);
  } else {
    if (bn == 256) return launch_dense<DenseCfg<256, 1, 4>>(p, grid, stream, coop);
    if (bn == 192) return launch_dense<DenseCfg<192, 1, 4>>(p, grid, stream, coop);
    return launch_dense<DenseCfg<128, 1, 6>>(p, grid, stream, coop);
  }
}
