// Dense GEMM core for sm_100a: D[M,N] = A[M,K] * B[N,K]^T (+bias), fp32 accumulation in TMEM.
//
// One persistent CTA per SM, 8 warps with fixed roles:
//   warp 0      TMA producer    (one lane): A/B k-blocks -> shared-memory ring
//   warp 1      MMA issuer      (one lane): tcgen05.mma from the ring into one of two TMEM
//                                accumulators; tcgen05.commit frees ring slots / publishes tiles
//   warps 2,3   communication   cross-rank "everyone entered this call" handshake; in all-gather
//                                mode they push this rank's A shard into every peer's landing
//                                buffer with 16-byte peer stores and bump arrival flags
//   warps 4..7  epilogue        tcgen05.ld -> (+bias) -> bf16 -> swizzled smem -> TMA store, to
//                                local memory or, in reduce-scatter mode, straight into the
//                                owner rank's staging buffer over NVLink
// In reduce-scatter mode the tiles of this rank's own segment come last; their epilogue adds the
// W-1 partial tiles that the peers have pushed into this rank's staging buffer to the fp32
// accumulator and stores the finished rows, so no separate reduction pass exists.
//
// The same kernel serves the three dense ops of the library; they differ only in how the M
// dimension is cut into per-rank segments and where tiles come from / go to:
//   GemmOnly        1 segment.                                   (reference: src/comm_none)
//   AllGather+GEMM  W segments, own first; A of a remote segment is read from the local
//                   landing buffer once its flags show that the owner's push has landed.
//                                                                (reference: src/ag_gemm, src/coll)
//   GEMM+ReduceScatter  W segments, own last; a tile of segment s is stored into rank s's
//                   staging slab [this rank]; the owner adds the slabs to its own tiles.
//                                                                (reference: src/gemm_rs)
//
// Tile shapes. CG_ = 2, MT_ = 2 is the large-problem shape: a CTA pair owns a 512 x 256 tile, each
// CTA stages 256 rows of A and 128 rows of B per k-block and the leader issues two 256 x 256
// MMAs that share the B tile, so 96 KB enter the pair's shared memory per k-block where two
// 256 x 256 tiles would take 128 KB. Its two accumulators fill TMEM, so the epilogue of a tile
// overlaps only the first STAGES k-blocks of the next one (issued into accumulator 0 while
// accumulator 1 is still being read).
// The last, partial wave of tiles may be cut into 2 or 4 column pieces each (split_shift), so that
// all CTAs share the remaining work instead of a few CTAs running whole tiles.
#pragma once

#include "ptx.cuh"

namespace fluxb {

constexpr int kMaxRanks = 8;

enum DenseMode : int32_t {
  kModePlain = 0,
  kModeAllGather = 1,
  kModeReduceScatter = 2,
  kModeGemmA2A = 3,   // Ulysses pre-attention: GEMM, then seq->heads all-to-all in the epilogue
  kModeA2AGemm = 4,   // Ulysses post-attention: heads->seq all-to-all feeding the GEMM's K loop
};

// slots of the optional per-CTA timeline (DenseGemmParams::trace)
enum TraceSlot : int {
  kTraceEntry = 0,        // roles start
  kTraceHandshake = 1,    // communication warp 2: every peer has entered the call
  kTracePushDone = 2,     // communication warp 2: its last push is published
  kTraceFirstLoads = 3,   // producer: all loads of the CTA's first tile issued
  kTraceLastLoads = 4,    // producer: all loads of its last tile issued
  kTraceFirstStore = 5,   // epilogue warp 4: first tile handed to the TMA store
  kTraceEnd = 6,          // epilogue warp 4: done
  kTraceFlagWait = 7,     // producer: total time spent waiting for arrival flags
  kTraceSlice0 = 8,       // producer, first tile: 8 + j = K slice j (post-attention) became readable;
                          // reduce-scatter: 8 = first tile of the own segment reached by epilogue warp 4
                          // (epilogue form), 9 / 10 = the tail that sums the slabs entered / left;
                          // block-scaled variants of the self-checking build: 8 / 9 = cycles promotion warp 4
                          // waited for MMAs / read TMEM, 10 = its cycles in all, 11 = its k-blocks,
                          // 12 / 13 = cycles the issuer waited for a free TMEM buffer / for operands
};
constexpr int kTraceWords = 16;  // words per CTA
constexpr int kMaxHeadGroups = 3;  // q, k, v

struct DenseGemmParams {
  CUtensorMap tm_a;              // A rows owned by this launch: [rows, K], box {BK, 128}
  CUtensorMap tm_a_land;         // all-gather landing buffer viewed as [W*seg_rows, K]
  CUtensorMap tm_b;              // B [N, K], box {BK, BN / CG}
  CUtensorMap tm_b_half;         // same, box {BK, BN / CG / 2}: column pieces of split tiles
  CUtensorMap tm_b_quarter;      // same, box {BK, BN / CG / 4}
  CUtensorMap tm_d[kMaxRanks];   // 3-D store maps [slab][seg_rows][N], box {64, 32, 1}; in reduce-scatter
                                 // mode entry `rank` covers rs_out ([1][seg_rows][N])
  int32_t M, N, K;
  int32_t num_seg, seg_rows, seg_first;
  int32_t rank, world;
  int32_t mode;
  int32_t group_m;
  int32_t seg_span, seg_solo_first;  // raster groups of visited segments, see decode_tile
  int32_t split_from, split_shift;   // tiles >= split_from are cut into 1 << split_shift column pieces
  int32_t total_vtiles;              // work items of the launch: split_from + ((tiles - split_from) << split_shift)
  int32_t reserved5;
  int32_t ag_inflight;           // all-gather push: loads in flight ahead of the stores (1..3)
  int32_t l2_hints;              // 1: A tiles are loaded evict_last (the band is reused by the next waves),
                                 // B tiles evict_first (streamed once per wave)
  uint32_t epoch;                // call number of the owning op object, starts at 1
  uint32_t scale_flags;          // bit 0: scale_a holds one float per row of the problem, bit 1: scale_b one per column
  uint64_t timeout_ns;
  Status* status;
  uint64_t* trace;               // optional [gridDim.x][kTraceWords] globaltimer stamps (ns), see kTrace*
  const void* bias;              // output dtype, may be null
  int64_t bias_row_stride;       // elements between bias rows; 0 = one row broadcast over M
  const float* scale_a;          // optional per-tensor scales (fp8): D = (A*B^T) * sa * sb
  const float* scale_b;
  int32_t ab_fmt;                // tcgen05 operand format: kind::f16 0 = f16, 1 = bf16;
                                 // kind::f8f6f4 0 = e4m3, 1 = e5m2
  int32_t out_f16;               // 1: D, bias and staging are fp16 instead of bf16
  int32_t act;                   // epilogue activation after bias: 0 none, 1 gelu(tanh), 2 relu, 3 silu
  int32_t reserved1;
  // block scales (fp8 block-scaled variant): inverse scales as the quantiser stores them
  const float* sa;               // for the rows of tm_a:      [rows/128, K/128, 128]
  const float* sa_land;          // for the rows of tm_a_land: [W*seg_rows/128, K/128, 128]
  const float* sb;               // [N/128, K/128], or with sb_groupwise [N/128, K/128, 128] (one per column)
  int32_t sb_groupwise;          // 1: the weight carries 1x128 scales too (the weight-gradient form)
  int32_t rs_tail;               // reduce-scatter: 1 = own tiles go to the own staging slab too and a tail sums the W slabs
  uint32_t* rs_claim;            // tail: work-claim counter (zero between calls); null = units dealt out round-robin
  int32_t b_kn;                  // 1: B is [K, N] with N contiguous (16-bit inputs): MN-major operand tiles
  int32_t reserved7;
  const float* ag_scale_src;     // all-gather: this rank's A scales (== sa), pushed with the shard
  float* ag_scale_land[kMaxRanks];
  // all-gather
  const void* ag_src;            // this rank's shard [seg_rows, K]
  void* ag_land[kMaxRanks];      // landing buffer of every rank, [W][seg_rows][K]
  uint32_t* ag_flags[kMaxRanks]; // on every rank: [W src][units] = last call whose rows landed
  int32_t flag_unit_rows;        // rows per arrival flag of the all-gather / all-to-all pushes
                                 // (a multiple of the tile height; units = ceil(rows / this))
  int32_t reserved4;
  // cross-rank start handshake
  uint32_t* start_ctr[kMaxRanks];  // on every rank: [W] last call number entered, by source
  // reduce-scatter
  uint32_t* rs_ctr[kMaxRanks];   // on every rank: [m_tiles_seg][8 src] = last call whose tiles landed
  uint32_t* local_cnt;           // local scratch [W][m_tiles_seg], zero between calls: counts the
                                 // warps of this GPU that finished their part of one (peer, tile row)
  const void* rs_stage;          // local staging [W][seg_rows][N] bf16
  void* rs_out;                  // [seg_rows, N] bf16
  uint32_t* wave_ctr;            // optional, zero between launches: number of tiles whose loads have been
                                 // issued. CTAs start wave i only after all of wave i-1 has been issued, so
                                 // the whole grid walks K together and shared tiles are read while in L2.
  // ---- Ulysses all-to-all modes. Activations are [bs, local_seq, heads, hd] on the sequence-
  // sharded side and [bs, heads/W, seq, hd] (or [bs, seq, heads/W, hd]) on the head-sharded side;
  // every 4-D tensor map below is ordered (hd, seq, head, batch) whatever the memory order is.
  CUtensorMap tm_a2a[kMaxHeadGroups * kMaxRanks];  // kModeGemmA2A: output of (group g, rank d),
                                                   //   box {64, 32, 1, 1}
  const void* a2a_attn;          // kModeA2AGemm: this rank's attention output
  void* a2a_land[kMaxRanks];     // kModeA2AGemm: rank d's landing buffer, one slab per source rank laid
                                 // out like the source: [W][heads/W][M][hd] (layout 0) or
                                 // [W][M][heads/W][hd] (layout 1), so every 32-row piece of a head is
                                 // one contiguous run on both sides of the copy
  CUtensorMap tm_a_land4;        // kModeA2AGemm: own landing buffer as (hd, M, head, source), box {64, 128, 1, 1}
  int32_t a2a_layout;
  int32_t a2a_hd, a2a_local_seq, a2a_bs, a2a_groups;
  int32_t a2a_group_start[kMaxHeadGroups + 1];  // first global head of each group (q | k | v)
  int32_t a2a_local_heads;       // kModeA2AGemm: heads per rank
  int32_t a2a_copy_local;        // kModeA2AGemm: 1 = the own slice is copied into the landing buffer too;
                                 // 0 = the K loop reads it in place through tm_a_own
  CUtensorMap tm_a_own;          // kModeA2AGemm: the attention output as (hd, seq, head, batch), box {64, 128, 1, 1}
  uint32_t* a2a_flags[kMaxRanks];  // kModeGemmA2A: [W src] "all my tiles for you have landed";
                                   // kModeA2AGemm: [W src][m_tiles] per tile row
};

// CG_ = 1: one CTA per 128 x BN tile. CG_ = 2: a pair of CTAs (one cluster) shares a (256 * MT_) x BN
// tile: each CTA stages its own 128 * MT_ rows of A and its own BN/2 rows of B, the pair leader issues
// tcgen05.mma.cta_group::2 (MT_ of them per k-step, one per 256-row half), and each CTA ends up with
// its 128 * MT_ x BN slice of D in its own TMEM.
// COMM_ > 0 reserves COMM_ bytes of shared memory as staging rings for the all-gather push.
// BS_ = true: block-scaled fp8 (1x128 A scales, 128x128 B scales): every 128-deep k-block is
// accumulated into a fresh TMEM buffer (512 / BN_ of them: the issuer runs that many k-blocks ahead)
// and promoted into fp32 registers, multiplied by its scales, by eight epilogue warps: two per
// TMEM lane quadrant, each owning half of the tile's columns for the whole tile. BN_ = 256 (one CTA,
// 128 x 256 tiles) is the faster shape: on 128 x 128 tiles even a kernel that promotes nothing stops at
// a third of the fp8 rate. With CG_ = 2 and BN_ = 128 a CTA pair shares a 256 x 128 tile (each CTA loads
// half of B; measured slower than single CTAs).
template <int BN_, int KIND_, int STAGES_, int CG_ = 1, int COMM_ = 0, bool BS_ = false, int MT_ = 1>
struct DenseCfg {
  static constexpr int COMM_BYTES = COMM_;
  static constexpr bool BS = BS_;
  static constexpr int MT = MT_;
  static constexpr int EPI_WARPS = BS_ ? 8 : 4;
  static constexpr int THREADS = 128 + 32 * EPI_WARPS;
  // MT_ == 1: two accumulators used alternately (the epilogue of a tile overlaps the next main loop);
  // MT_ == 2: the two row halves of one tile; block-scaled: one buffer per k-block in flight (4 or 2)
  static constexpr int ACC_BUFS = BS_ ? 512 / BN_ : 2;
  static_assert(!BS_ || (KIND_ == 1 && (BN_ == 128 || (BN_ == 256 && CG_ == 1))),
                "block-scaled variant: fp8; 128 columns (128 or 256 rows) or 128 x 256 tiles");
  static_assert(MT_ == 1 || (MT_ == 2 && CG_ == 2 && BN_ == 256 && !BS_), "512-row tiles: CTA pairs, 256 columns");
  static constexpr int CG = CG_;
  static constexpr int BM_CTA = 128 * MT_;                 // rows of A / D per CTA
  static constexpr int BM = BM_CTA * CG_;                  // rows per tile
  static constexpr int BN = BN_;
  static constexpr int KIND = KIND_;                       // 0 = bf16 / fp16, 1 = fp8, 2 = int8 (s32 accumulators)
  static constexpr int ELT = KIND_ == 0 ? 2 : 1;
  static constexpr int BK = 128 / ELT;                     // one 128-byte swizzle row
  static constexpr int UMMA_K = 32 / ELT;
  static constexpr int STAGES = STAGES_;
  static constexpr int A_HALF_BYTES = 128 * 128;           // one 128-row block of A
  static constexpr int A_BYTES = BM_CTA * 128;
  static constexpr int B_ROWS_CTA = BN / CG_;
  static constexpr int B_BYTES = B_ROWS_CTA * 128;
  static constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
  static constexpr int EPI_BUF_BYTES = 32 * 128;           // 32 rows x 64 bf16
  // staging buffers per epilogue warp: the variants with a communication ring give one of the two
  // to a sixth pipeline stage (the epilogue of a tile hides behind the next tile's main loop anyway);
  // block-scaled 256-column tiles give it to the fourth 48 KB stage
  static constexpr int EPI_BUFS = ((COMM_ > 0 && !BS_) || (BS_ && BN_ == 256)) ? 1 : 2;
  static constexpr int EPI_BYTES = EPI_WARPS * EPI_BUFS * EPI_BUF_BYTES;
  static constexpr int BAR_BYTES = 256;
  static constexpr int SMEM_BYTES = STAGES * STAGE_BYTES + EPI_BYTES + COMM_BYTES + BAR_BYTES + 1024;
  static_assert(SMEM_BYTES <= 232448, "over the 227 KB shared memory limit");
  static constexpr int TMEM_COLS = 512;
  static_assert(ACC_BUFS * BN <= TMEM_COLS, "accumulators must fit TMEM");
  // column pieces of a split tile are BN >> shift wide; the epilogue moves 64 columns at a time
  static constexpr int MAX_SPLIT_SHIFT = (BN_ == 256 && !BS_) ? 2 : 0;
};

struct TileCoord {
  int seg;       // segment (owner rank) of the tile
  int m_in_seg;  // first row inside the segment
  int m_tile;    // tile row index inside the segment
  int n0;        // first output column
  int shift;     // the work item is BN >> shift columns wide (a piece of a split tile)
};

__host__ __device__ __forceinline__ TileCoord decode_tile(const DenseGemmParams& p, int t, int m_tiles_seg,
                                                 int n_tiles, int BM, int BN) {
  // Work items past split_from are column pieces of the tiles at the end of the order
  int shift = 0, piece = 0;
  if (t >= p.split_from) {
    const int h = t - p.split_from;
    shift = p.split_shift;
    piece = h & ((1 << shift) - 1);
    t = p.split_from + (h >> shift);
  }
  // Segments are visited in the order seg_first, seg_first + 1, ... and rastered in groups of
  // seg_span consecutive segments (1 or 2; seg_solo_first: the first visited segment is a group
  // of its own), so that a band of group_m tile rows can span two segments.
  const int per_seg = m_tiles_seg * n_tiles;
  int v0, span, r;
  if (p.seg_span <= 1) {
    v0 = t / per_seg;
    span = 1;
    r = t - v0 * per_seg;
  } else if (p.seg_solo_first && t < per_seg) {
    v0 = 0;
    span = 1;
    r = t;
  } else {
    const int lead = p.seg_solo_first ? 1 : 0;
    const int tt = t - lead * per_seg;
    const int gi = tt / (2 * per_seg);
    v0 = lead + 2 * gi;
    span = min(2, p.num_seg - v0);
    r = tt - gi * 2 * per_seg;
  }
  const int m_tiles_g = span * m_tiles_seg;
  const int G = p.group_m;
  const int per_group = G * n_tiles;
  const int gid = r / per_group;
  const int first_m = gid * G;
  const int gsz = min(G, m_tiles_g - first_m);
  r -= gid * per_group;
  int mt = first_m + r % gsz;
  const int nt = r / gsz;
  int v = v0;
  if (mt >= m_tiles_seg) {
    mt -= m_tiles_seg;
    ++v;
  }
  int seg = p.seg_first + v;
  if (seg >= p.num_seg) seg -= p.num_seg;
  TileCoord c;
  c.seg = seg;
  c.m_tile = mt;
  c.m_in_seg = mt * BM;
  c.n0 = nt * BN + piece * (BN >> shift);
  c.shift = shift;
  return c;
}

template <class Cfg>
__global__ void __launch_bounds__(Cfg::THREADS, 1) dense_gemm_kernel(const __grid_constant__ DenseGemmParams p) {
  constexpr int BM = Cfg::BM, BN = Cfg::BN, BK = Cfg::BK, STAGES = Cfg::STAGES;
  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw_addr = ptx::smem_u32(smem_raw);
  const uint32_t pad = (1024u - (raw_addr & 1023u)) & 1023u;
  uint8_t* smem = smem_raw + pad;
  const uint32_t smem_base = raw_addr + pad;

  const uint32_t epi_base = smem_base + STAGES * Cfg::STAGE_BYTES;
  uint8_t* epi_ptr = smem + STAGES * Cfg::STAGE_BYTES;
  const uint32_t comm_base = epi_base + Cfg::EPI_BYTES;
  const uint32_t bar_base = comm_base + Cfg::COMM_BYTES;
  uint8_t* bar_ptr = epi_ptr + Cfg::EPI_BYTES + Cfg::COMM_BYTES;
  // barrier block: full[STAGES], empty[STAGES], tmem_full[2], tmem_empty[2], three words, then
  // the 8 barriers of the all-gather staging rings
  auto full_bar = [&](int s) { return bar_base + 8u * s; };
  auto empty_bar = [&](int s) { return bar_base + 8u * (STAGES + s); };
  constexpr int NACC = Cfg::ACC_BUFS;
  auto tfull_bar = [&](int a) { return bar_base + 8u * (2 * STAGES + a); };
  auto tempty_bar = [&](int a) { return bar_base + 8u * (2 * STAGES + NACC + a); };
  volatile uint32_t* tmem_slot =
      reinterpret_cast<volatile uint32_t*>(bar_ptr + 8 * (2 * STAGES + 2 * NACC));
  volatile uint32_t* abort_word = tmem_slot + 1;
  volatile uint32_t* claim_slot = tmem_slot + 2;   // reduce-scatter tail: the work unit this CTA claimed
  const uint32_t ring_bar_base = bar_base + 8u * (2 * STAGES + 2 * NACC) + 16u;
  static_assert(8 * (2 * STAGES + 2 * NACC) + 16 + 64 + 16 <= Cfg::BAR_BYTES, "barrier block too small");

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  constexpr int CG = Cfg::CG;
  // position inside the CTA pair (CG == 2): rank 0 leads (issues the MMAs, owns the barriers
  // that both CTAs' loads and epilogues report to)
  const uint32_t cta_rank = CG == 2 ? ptx::cluster_ctarank() : 0u;
  const bool leader = cta_rank == 0;
  const int tile_slot = blockIdx.x / CG;          // which tile stream this CTA (pair) walks
  const int tile_stride = gridDim.x / CG;

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      ptx::mbar_init(full_bar(s), 1);
      ptx::mbar_init(empty_bar(s), 1);
    }
    for (int a = 0; a < NACC; ++a) {
      ptx::mbar_init(tfull_bar(a), 1);
      // one epilogue warp per TMEM lane quadrant reads a buffer (block-scaled: two, 64 columns each)
      ptx::mbar_init(tempty_bar(a), Cfg::BS ? 8 * CG : 4 * CG);
    }
    for (int i = 0; i < 8; ++i) ptx::mbar_init(ring_bar_base + 8u * i, 1);
    *abort_word = 0;
    ptx::fence_mbar_init();
    ptx::prefetch_tmap(&p.tm_a);
    ptx::prefetch_tmap(&p.tm_b);
  }
  if (warp == 1) {
    ptx::tmem_alloc<CG>(ptx::smem_u32(const_cast<uint32_t*>(tmem_slot)), Cfg::TMEM_COLS);
    ptx::tmem_relinquish<CG>();
  }
  ptx::tc_fence_before();
  if constexpr (CG == 2) ptx::cluster_sync(); else __syncthreads();
  ptx::tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  WaitCtx wc{p.status, abort_word, p.timeout_ns};
  auto stamp = [&](int slot) {
    if (p.trace != nullptr) p.trace[blockIdx.x * kTraceWords + slot] = ptx::globaltimer_ns();
  };

  const int m_tiles_seg = (p.seg_rows + BM - 1) / BM;
  const int n_tiles = (p.N + BN - 1) / BN;
  const int total_tiles = p.total_vtiles;   // work items: whole tiles, then the column pieces of split ones
  const int k_blocks = (p.K + BK - 1) / BK;
  const bool multi = p.world > 1 && p.mode != kModePlain;

  // -------------------------------------------------------------------- reduce-scatter tail
  // Run by 256 threads of the CTA (tid 0..255; `sync` is a barrier among exactly those): all threads after
  // the teardown, or - block-scaled variants, whose leading warps have given their registers away - the
  // eight promotion warps at the end of their role.
  auto rs_tail = [&](const int tid, auto&& sync) {
    // Three ranks and more: the own tiles went to the own staging slab like everybody else's, and
    // all threads of the grid now sum the W slabs into rs_out (fp32 sums of 16-bit addends, slabs in
    // rank order). Adding W-1 slabs inside the epilogue of the own tiles, as two ranks do, costs
    // more here than this tail: those epilogues hold the accumulators that the next tile waits for.
    // A work unit is kUnit 16-byte pieces of the [seg_rows, N] output; units are claimed from a
    // counter (every CTA makes exactly one failing claim; whoever makes the very last claim of the
    // launch puts the counter back to zero), or dealt out round-robin when there is no counter.
    constexpr int kUnit = 256 * 16;
    const int64_t pieces_per_row = p.N >> 3;
    const int64_t total_pieces = static_cast<int64_t>(p.seg_rows) * pieces_per_row;
    const uint32_t units = static_cast<uint32_t>((total_pieces + kUnit - 1) / kUnit);
    const uint4* stage = reinterpret_cast<const uint4*>(p.rs_stage);
    uint4* out = reinterpret_cast<uint4*>(p.rs_out);
    const bool tail_f16 = p.out_f16 != 0;
    if (tid == 0) stamp(kTraceSlice0 + 1);      // reduce tail entered
    uint32_t next_static = blockIdx.x;
    uint32_t rows_seen = 0;   // (threads 0..W-1) tile rows whose slab of source tid was seen to have landed
    auto claim = [&]() -> uint32_t {
      if (*abort_word) return 0xFFFFFFFFu;
      uint32_t got;
      if (p.rs_claim != nullptr) {
        got = atomicAdd(p.rs_claim, 1u);
        if (got == units + gridDim.x - 1u) atomicExch(p.rs_claim, 0u);
      } else {
        got = next_static;
        next_static += gridDim.x;
      }
      return got;
    };
    int par = 0;
    sync();
    // (claims are made by a thread that does not also look at arrival flags)
    if (tid == 32) claim_slot[0] = claim();
    sync();
    while (true) {
      const uint32_t u = claim_slot[par];
      if (u >= units) break;
      // the next unit is claimed while this one is summed
      if (tid == 32) claim_slot[par ^ 1] = claim();
      {
        // every source's rows of this unit must have landed: one thread per source looks at the flags
        // of the tile rows that the unit touches (usually one); the block barrier passes it on
        const int64_t c0 = static_cast<int64_t>(u) * kUnit;
        const int64_t c1 = (c0 + kUnit < total_pieces ? c0 + kUnit : total_pieces) - 1;
        const int mt0 = static_cast<int>((c0 / pieces_per_row) / BM);
        const int mt1 = static_cast<int>((c1 / pieces_per_row) / BM);
        if (static_cast<int>(tid) < p.world)
          for (int mt = mt0; mt <= mt1; ++mt) {
            if (mt < 32 && ((rows_seen >> mt) & 1u)) continue;
            flag_wait_ge(wc, p.rs_ctr[p.rank] + mt * kMaxRanks + tid, p.epoch, kSiteTileCounter);
            if (mt < 32) rows_seen |= 1u << mt;
          }
        sync();
      }
      constexpr int PIECES = 4;          // 16-byte pieces per thread in flight per source
#pragma unroll 1
      for (int rep = 0; rep < kUnit / 256; rep += PIECES) {
        int64_t idx[PIECES];
        bool ok[PIECES];
#pragma unroll
        for (int h = 0; h < PIECES; ++h) {
          idx[h] = static_cast<int64_t>(u) * kUnit + (rep + h) * 256 + tid;
          ok[h] = idx[h] < total_pieces;
        }
        uint4 v[kMaxRanks][PIECES];
#pragma unroll
        for (int sr = 0; sr < kMaxRanks; ++sr)
#pragma unroll
          for (int h = 0; h < PIECES; ++h)
            if (sr < p.world && ok[h]) v[sr][h] = ptx::ld_global_cs_v4(stage + sr * total_pieces + idx[h]);
        float accv[PIECES][8];
#pragma unroll
        for (int h = 0; h < PIECES; ++h)
#pragma unroll
          for (int e = 0; e < 8; ++e) accv[h][e] = 0.f;
#pragma unroll
        for (int sr = 0; sr < kMaxRanks; ++sr)
#pragma unroll
          for (int h = 0; h < PIECES; ++h) {
            if (sr < p.world && ok[h]) {
              const uint32_t w[4] = {v[sr][h].x, v[sr][h].y, v[sr][h].z, v[sr][h].w};
#pragma unroll
              for (int e = 0; e < 4; ++e) {
                accv[h][2 * e] += ptx::half_bits_to_float(static_cast<uint16_t>(w[e] & 0xFFFFu), tail_f16);
                accv[h][2 * e + 1] += ptx::half_bits_to_float(static_cast<uint16_t>(w[e] >> 16), tail_f16);
              }
            }
          }
#pragma unroll
        for (int h = 0; h < PIECES; ++h) {
          if (!ok[h]) continue;
          uint4 o;
          o.x = ptx::pack_half2(tail_f16, accv[h][0], accv[h][1]);
          o.y = ptx::pack_half2(tail_f16, accv[h][2], accv[h][3]);
          o.z = ptx::pack_half2(tail_f16, accv[h][4], accv[h][5]);
          o.w = ptx::pack_half2(tail_f16, accv[h][6], accv[h][7]);
          out[idx[h]] = o;
        }
      }
      sync();
      par ^= 1;
    }
    if (tid == 0) stamp(kTraceSlice0 + 2);  // reduce tail left
  };

  if (warp < 4) {
  // (block-scaled variant) producer, issuer and communication warps give registers to the
  // promotion warps; all four warps of the group execute the same instruction here. With 256-column
  // tiles the promotion warps hold 128 accumulators and take all they can get: 40 / 232 measured
  // 1560 TFLOP/s where 56 / 224 gave 1376 and 24 / 240 the same 1560 (the compiler's spill report:
  // 168, 176 and 226 bytes per thread, the last mostly in the leading warps).
  if constexpr (Cfg::BS) ptx::setmaxnreg_dec<(BN == 256 ? 40 : 88)>();
  if (warp == 0) {
    // ------------------------------------------------------------------ TMA producer
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      const uint32_t full_owner0 = CG == 2 ? ptx::mapa_u32(full_bar(0), 0) : full_bar(0);
      int wave = 0;
      uint64_t flag_ns = 0;
      const uint64_t pol_a = ptx::l2_policy_evict_last(), pol_b = ptx::l2_policy_evict_first();
      uint64_t ag_seen = 0;               // all-gather: shard units seen to have arrived
      uint32_t a2a_seen[kMaxRanks] = {};  // post-attention: row units seen, per source
      stamp(kTraceEntry);
      for (int t = tile_slot; t < total_tiles; t += tile_stride, ++wave) {
        if (*abort_word) break;   // a wait gave up: issue nothing more
        const TileCoord c = decode_tile(p, t, m_tiles_seg, n_tiles, BM, BN);
        if (!dcheck(wc, c.seg >= 0 && c.seg < p.num_seg && c.m_in_seg >= 0 && c.m_in_seg < p.seg_rows &&
                            c.n0 >= 0 && c.n0 < n_tiles * BN,   // (a piece of a split edge tile may lie past N)
                    kCheckTileDecode, static_cast<uint32_t>(t), static_cast<uint32_t>(c.seg)))
          break;
        if (p.wave_ctr != nullptr && leader && wave > 0) {
          const uint32_t need = min(static_cast<uint32_t>(wave) * tile_stride, static_cast<uint32_t>(total_tiles));
          flag_wait_ge(wc, p.wave_ctr, need, kSiteStartBarrier);
        }
        const CUtensorMap* tma = &p.tm_a;
        const CUtensorMap* tmb = c.shift == 0 ? &p.tm_b : (c.shift == 1 ? &p.tm_b_half : &p.tm_b_quarter);
        const uint32_t stage_tx = Cfg::A_BYTES + (Cfg::B_BYTES >> c.shift);
        const int b_row = c.n0 + static_cast<int>(cta_rank) * (Cfg::B_ROWS_CTA >> c.shift);
        const int m_cta = c.m_in_seg + static_cast<int>(cta_rank) * Cfg::BM_CTA;
        int a_row = c.seg * p.seg_rows + m_cta;
        if (p.mode == kModeAllGather && multi) {
          if (c.seg == p.rank) {
            a_row = m_cta;  // own shard straight from the caller's tensor
          } else {
            tma = &p.tm_a_land;
            // a shard unit that this thread has seen arrive needs neither the acquire nor the
            // proxy fence again (a few microseconds per tile otherwise)
            const int ag_units = (p.seg_rows + p.flag_unit_rows - 1) / p.flag_unit_rows;
            const int fi = c.seg * ag_units + c.m_in_seg / p.flag_unit_rows;
            if (fi >= 64 || ((ag_seen >> fi) & 1ull) == 0ull) {
              const uint64_t w0 = p.trace != nullptr ? ptx::globaltimer_ns() : 0;
              flag_wait_ge(wc, p.ag_flags[p.rank] + fi, p.epoch, kSiteShardFlag);
              ptx::fence_proxy_async_all();
              if (fi < 64) ag_seen |= 1ull << fi;
              if (p.trace != nullptr) flag_ns += ptx::globaltimer_ns() - w0;
            }
          }
        }
        // post-attention mode: the K range is W slices, one per source rank, landing
        // independently; start with the own slice and gate each slice on its flag
        const int kb_per_src = p.mode == kModeA2AGemm ? (p.a2a_local_heads * p.a2a_hd) / BK : k_blocks;
        // (no division in the k loop: one thread issues every load of the CTA, and a few dozen
        // dependent integer instructions per k-block are enough to starve the tensor pipe)
        const bool a2a_in = p.mode == kModeA2AGemm;
        const bool own_in_place = a2a_in && p.a2a_copy_local == 0;
        const int hd_shift = p.a2a_hd == 128 ? 7 : 6;
        const int own_b = own_in_place ? m_cta / p.a2a_local_seq : 0;
        const int own_s = own_in_place ? p.rank * p.a2a_local_seq + m_cta % p.a2a_local_seq : 0;
        const int a2a_unit = a2a_in ? c.m_in_seg / p.flag_unit_rows : 0;
        const uint32_t* a2a_flag_row = a2a_in ? p.a2a_flags[p.rank] + a2a_unit : nullptr;
        const int a2a_units = a2a_in ? (p.seg_rows + p.flag_unit_rows - 1) / p.flag_unit_rows : 0;
        int src = p.rank, kin = 0;   // source rank of the current K slice, k-block within the slice
        for (int ki = 0; ki < k_blocks; ++ki) {
          int kb = ki;
          bool in_place = false;
          if (a2a_in) {
            // slice j of the K loop is the one that source rank-j pushed at its step j
            kb = src * kb_per_src + kin;
            in_place = own_in_place && src == p.rank;
            if (kin == 0 && !in_place && (a2a_unit >= 32 || ((a2a_seen[src] >> a2a_unit) & 1u) == 0u)) {
              const uint64_t w0 = p.trace != nullptr ? ptx::globaltimer_ns() : 0;
              flag_wait_ge(wc, a2a_flag_row + src * a2a_units, p.epoch, kSiteA2AFlag);
              ptx::fence_proxy_async_all();
              if (a2a_unit < 32) a2a_seen[src] |= 1u << a2a_unit;
              if (p.trace != nullptr) {
                flag_ns += ptx::globaltimer_ns() - w0;
                int j = p.rank - src;
                if (j < 0) j += p.world;
                if (wave == 0) stamp(kTraceSlice0 + j);
              }
            }
          }
          // (a wait that gave up, here or in another role: stop issuing at once, so that what is in flight
          // at the teardown is bounded by the depth of the pipeline)
          if (!mbar_wait(wc, empty_bar(stage), phase ^ 1u, kSiteSmemEmpty)) break;
          const uint32_t sa = smem_base + stage * Cfg::STAGE_BYTES;
          // post-attention input: (column in head, head of the slice, source); the own slice comes
          // straight from the attention output
          const int own_k = kin * BK;
          const int own_head = own_k >> hd_shift;
          const int own_col = own_k & (p.a2a_hd - 1);
          const int ld_src = src;
          if (a2a_in && ++kin == kb_per_src) {
            kin = 0;
            src = src == 0 ? p.world - 1 : src - 1;
          }
          if constexpr (CG == 1) {
            ptx::mbar_arrive_expect_tx(full_bar(stage), stage_tx);
            if (in_place) ptx::tma_load_4d(sa, &p.tm_a_own, full_bar(stage), own_col, own_s, own_head, own_b);
            else if (a2a_in) ptx::tma_load_4d(sa, &p.tm_a_land4, full_bar(stage), own_col, m_cta, own_head, ld_src);
            else if (p.l2_hints) ptx::tma_load_2d_hint(sa, tma, full_bar(stage), kb * BK, a_row, pol_a);
            else ptx::tma_load_2d(sa, tma, full_bar(stage), kb * BK, a_row);
            if (Cfg::KIND == 0 && p.b_kn) {
              // B as [K, N]: boxes of 64 columns x BK k-rows, one after the other
#pragma unroll
              for (int j = 0; j < Cfg::B_ROWS_CTA / 64; ++j)
                ptx::tma_load_2d(sa + Cfg::A_BYTES + j * (BK * 128), tmb, full_bar(stage), b_row + j * 64, kb * BK);
            } else if (p.l2_hints) ptx::tma_load_2d_hint(sa + Cfg::A_BYTES, tmb, full_bar(stage), kb * BK, b_row, pol_b);
            else ptx::tma_load_2d(sa + Cfg::A_BYTES, tmb, full_bar(stage), kb * BK, b_row);
          } else {
            // both CTAs' bytes are counted on the leader's barrier
            const uint32_t fb = full_owner0 + 8u * stage;
            if (leader) ptx::mbar_arrive_expect_tx(full_bar(stage), 2 * stage_tx);
            if (in_place) ptx::tma_load_4d_cg2(sa, &p.tm_a_own, fb, own_col, own_s, own_head, own_b);
            else if (a2a_in) ptx::tma_load_4d_cg2(sa, &p.tm_a_land4, fb, own_col, m_cta, own_head, ld_src);
            else if (p.l2_hints) ptx::tma_load_2d_cg2_hint(sa, tma, fb, kb * BK, a_row, pol_a);
            else ptx::tma_load_2d_cg2(sa, tma, fb, kb * BK, a_row);
            if (Cfg::KIND == 0 && p.b_kn) {
#pragma unroll
              for (int j = 0; j < Cfg::B_ROWS_CTA / 64; ++j)
                ptx::tma_load_2d_cg2(sa + Cfg::A_BYTES + j * (BK * 128), tmb, fb, b_row + j * 64, kb * BK);
            } else if (p.l2_hints) ptx::tma_load_2d_cg2_hint(sa + Cfg::A_BYTES, tmb, fb, kb * BK, b_row, pol_b);
            else ptx::tma_load_2d_cg2(sa + Cfg::A_BYTES, tmb, fb, kb * BK, b_row);
          }
          if (++stage == STAGES) {
            stage = 0;
            phase ^= 1u;
          }
        }
        if (p.wave_ctr != nullptr && leader) {
          // this tile's loads are all issued; whoever issues the last tile of the launch puts the
          // counter back to zero (every wait of the launch is for a smaller value)
          if (atomicAdd(p.wave_ctr, 1u) == static_cast<uint32_t>(total_tiles) - 1u) atomicExch(p.wave_ctr, 0u);
        }
        if (wave == 0) stamp(kTraceFirstLoads);
      }
      stamp(kTraceLastLoads);
      if (p.trace != nullptr) p.trace[blockIdx.x * kTraceWords + kTraceFlagWait] = flag_ns;
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------------ MMA issuer
    if (lane == 0 && leader) {
      // one instruction covers 128 rows per CTA of the group
      // B as [K, N] (16-bit inputs): MN-major operand tiles - 64-column groups BK * 128 bytes apart, 8-k-row
      // groups 1024 bytes apart, one UMMA_K step = 16 k-rows of 128 bytes
      const bool b_kn = Cfg::KIND == 0 && p.b_kn != 0;
      const uint32_t b_major = b_kn ? 1u : 0u;
      const uint32_t bstep = b_kn ? static_cast<uint32_t>(Cfg::UMMA_K * 128) >> 4 : 2u;
      auto make_bdesc = [&](uint32_t saddr) -> uint64_t {
        return b_kn ? ptx::umma_desc_mn_sw128(saddr, BK * 128, 1024) : ptx::umma_desc_k_sw128(saddr);
      };
      const uint32_t idesc_full =
          ptx::umma_idesc(p.ab_fmt, p.ab_fmt, 128 * CG, BN, 0, b_major, Cfg::KIND == 2 ? 2u : 1u);
      int stage = 0;
      uint32_t phase = 0;
      int it = 0;
#ifdef FLUXB_DEBUG_CHECKS
      uint64_t probe_tempty = 0, probe_full = 0;
#endif
      for (int t = tile_slot; t < total_tiles; t += tile_stride, ++it) {
        if (*abort_word) break;
        // a column piece of a split tile is a narrower instruction on the same operands
        const int shift = t >= p.split_from ? p.split_shift : 0;
        const uint32_t idesc = shift == 0 ? idesc_full
                                          : ptx::umma_idesc(p.ab_fmt, p.ab_fmt, 128 * CG, BN >> shift, 0, b_major,
                                                            Cfg::KIND == 2 ? 2u : 1u);
        if constexpr (Cfg::BS) {
          // every k-block goes to its own TMEM buffer; the epilogue warps promote it
          for (int kb = 0; kb < k_blocks; ++kb) {
            const uint32_t n = static_cast<uint32_t>(it) * k_blocks + kb;
            const int buf = n % NACC;
#ifdef FLUXB_DEBUG_CHECKS
            const long long pc0 = clock64();
#endif
            if (!mbar_wait(wc, tempty_bar(buf), ((n / NACC) & 1u) ^ 1u, kSiteTmemEmpty)) break;
#ifdef FLUXB_DEBUG_CHECKS
            const long long pc1 = clock64();
#endif
            if (!mbar_wait(wc, full_bar(stage), phase, kSiteSmemFull)) break;
#ifdef FLUXB_DEBUG_CHECKS
            // self-checking build: cycles the issuer waited for a free TMEM buffer / for operands
            probe_tempty += static_cast<uint64_t>(pc1 - pc0);
            probe_full += static_cast<uint64_t>(clock64() - pc1);
#endif
            ptx::tc_fence_after();
            const uint32_t sa = smem_base + stage * Cfg::STAGE_BYTES;
            const uint64_t adesc = ptx::umma_desc_k_sw128(sa);
            const uint64_t bdesc = ptx::umma_desc_k_sw128(sa + Cfg::A_BYTES);
#pragma unroll
            for (int k = 0; k < BK / Cfg::UMMA_K; ++k)
              ptx::umma_ss<CG, Cfg::KIND>(tmem_base + buf * BN, adesc + 2u * k, bdesc + 2u * k, idesc,
                                          k != 0 ? 1u : 0u);
            if constexpr (CG == 1) {
              ptx::umma_commit(empty_bar(stage));
              ptx::umma_commit(tfull_bar(buf));
            } else {
              ptx::umma_commit_cg2(empty_bar(stage), 3);
              ptx::umma_commit_cg2(tfull_bar(buf), 3);
            }
            if (++stage == STAGES) {
              stage = 0;
              phase ^= 1u;
            }
          }
          continue;
        }
        if constexpr (Cfg::MT == 2) {
          // Two accumulators = the two 256-row halves of the tile; both read the same B tile. The
          // epilogue of the previous tile drains accumulator 0 first: the first k-blocks of this
          // tile go into accumulator 0 while accumulator 1 is still being read, then the same
          // k-blocks into accumulator 1 (which releases their stages).
          const uint32_t par_e = (static_cast<uint32_t>(it) & 1u) ^ 1u;
          const int head = k_blocks < STAGES ? k_blocks : STAGES;
          auto issue_half = [&](int st, int half, bool first) {
            const uint32_t sa = smem_base + st * Cfg::STAGE_BYTES;
            const uint64_t adesc = ptx::umma_desc_k_sw128(sa + half * Cfg::A_HALF_BYTES);
            const uint64_t bdesc = make_bdesc(sa + Cfg::A_BYTES);
#pragma unroll
            for (int k = 0; k < BK / Cfg::UMMA_K; ++k)
              ptx::umma_ss<CG, Cfg::KIND>(tmem_base + half * BN, adesc + 2u * k, bdesc + bstep * k, idesc,
                                          (!first || k != 0) ? 1u : 0u);
          };
          if (!mbar_wait(wc, tempty_bar(0), par_e, kSiteTmemEmpty)) break;
          ptx::tc_fence_after();
          {
            int st = stage;
            uint32_t ph = phase;
            for (int kb = 0; kb < head; ++kb) {
              if (!mbar_wait(wc, full_bar(st), ph, kSiteSmemFull)) break;
              ptx::tc_fence_after();
              issue_half(st, 0, kb == 0);
              if (++st == STAGES) {
                st = 0;
                ph ^= 1u;
              }
            }
          }
          if (*abort_word || !mbar_wait(wc, tempty_bar(1), par_e, kSiteTmemEmpty)) break;
          ptx::tc_fence_after();
          for (int kb = 0; kb < head; ++kb) {
            issue_half(stage, 1, kb == 0);
            ptx::umma_commit_cg2(empty_bar(stage), 3);
            if (++stage == STAGES) {
              stage = 0;
              phase ^= 1u;
            }
          }
          for (int kb = head; kb < k_blocks; ++kb) {
            if (!mbar_wait(wc, full_bar(stage), phase, kSiteSmemFull)) break;
            ptx::tc_fence_after();
            issue_half(stage, 0, false);
            issue_half(stage, 1, false);
            ptx::umma_commit_cg2(empty_bar(stage), 3);
            if (++stage == STAGES) {
              stage = 0;
              phase ^= 1u;
            }
          }
          ptx::umma_commit_cg2(tfull_bar(0), 3);
          continue;
        }
        const int acc = it & 1;
        const uint32_t acc_phase = (it >> 1) & 1;
        if (!mbar_wait(wc, tempty_bar(acc), acc_phase ^ 1u, kSiteTmemEmpty)) break;
        ptx::tc_fence_after();
        const uint32_t d_tmem = tmem_base + acc * BN;
        for (int kb = 0; kb < k_blocks; ++kb) {
          if (!mbar_wait(wc, full_bar(stage), phase, kSiteSmemFull)) break;
          ptx::tc_fence_after();
          const uint32_t sa = smem_base + stage * Cfg::STAGE_BYTES;
          const uint64_t adesc = ptx::umma_desc_k_sw128(sa);
          const uint64_t bdesc = make_bdesc(sa + Cfg::A_BYTES);
#pragma unroll
          for (int k = 0; k < BK / Cfg::UMMA_K; ++k) {
            // 32 bytes per UMMA_K step inside the 128-byte swizzled row: +2 in 16-byte units
            ptx::umma_ss<CG, Cfg::KIND>(d_tmem, adesc + 2u * k, bdesc + bstep * k, idesc,
                                        (kb | k) != 0 ? 1u : 0u);
          }
          if constexpr (CG == 1) ptx::umma_commit(empty_bar(stage));
          else ptx::umma_commit_cg2(empty_bar(stage), 3);
          if (++stage == STAGES) {
            stage = 0;
            phase ^= 1u;
          }
        }
        if constexpr (CG == 1) ptx::umma_commit(tfull_bar(acc));
        else ptx::umma_commit_cg2(tfull_bar(acc), 3);
      }
#ifdef FLUXB_DEBUG_CHECKS
      if (Cfg::BS && p.trace != nullptr) {
        p.trace[blockIdx.x * kTraceWords + 12] = probe_tempty;
        p.trace[blockIdx.x * kTraceWords + 13] = probe_full;
      }
#endif
    }
  } else if (warp == 2 || warp == 3) {
    // ------------------------------------------------------------------ handshake + all-gather push
    if (multi && warp == 3 && blockIdx.x == 0 && lane < p.world) {
      // "this rank has entered call `epoch`": nobody writes into a peer before that peer is
      // done with the previous call's buffers. One word per source rank, so a fast rank's
      // next call can never be mistaken for a slow rank's current one.
      ptx::st_release_sys(p.start_ctr[lane] + p.rank, p.epoch);
    }
    if constexpr (Cfg::COMM_BYTES > 0) {
      if (p.mode == kModeAllGather && multi) {
        if (lane < p.world) flag_wait_ge(wc, p.start_ctr[p.rank] + lane, p.epoch, kSiteStartBarrier);
        __syncwarp();
        if (lane == 0 && warp == 2) stamp(kTraceHandshake);
        if (lane == 0) {
          // One lane per warp drives a ring of NSLOT staging slots: bulk-load a chunk of the local
          // shard into a slot, bulk-store it into the peer's landing slab, reuse the slot once
          // the store has read it. The peer that consumes this shard first (rank-1 starts with
          // segment `rank`) is served first; all ranks walk the same rotation, so every step is
          // a permutation on NVSwitch.
          constexpr int NSLOT = 4;
          constexpr uint32_t CH = Cfg::COMM_BYTES / 2 / NSLOT;
          constexpr int LAG = 4;  // chunk stores that may still be in flight when a step is published
          const uint32_t ring = comm_base + (warp - 2) * (Cfg::COMM_BYTES / 2);
          const uint32_t rbar = ring_bar_base + (warp - 2) * NSLOT * 8u;
          const uint8_t* src = reinterpret_cast<const uint8_t*>(p.ag_src);
          const int64_t row_bytes = static_cast<int64_t>(p.K) * Cfg::ELT;
          const int64_t slab_off = static_cast<int64_t>(p.rank) * p.seg_rows * row_bytes;
          const uint32_t cw = blockIdx.x * 2 + (warp - 2);
          const uint32_t ncw = gridDim.x * 2;
          const int UR = p.flag_unit_rows;
          const int units = (p.seg_rows + UR - 1) / UR;
          // scales of a block-scaled shard ride along as a second byte range per tile row:
          // [rows/128][K/128][128] floats
          const int64_t srow_bytes = Cfg::BS ? static_cast<int64_t>(k_blocks) * 512 : 0;  // per 128 rows
          const int64_t sslab_off = static_cast<int64_t>(p.rank) * (p.seg_rows / 128) * srow_bytes;
          const uint8_t* ssrc = reinterpret_cast<const uint8_t*>(p.ag_scale_src);
          auto payload_chunks = [&](int mt) -> uint32_t {
            const int rows = min(UR, p.seg_rows - mt * UR);
            return static_cast<uint32_t>((rows * row_bytes + CH - 1) / CH);
          };
          auto scale_bytes = [&](int mt) -> int64_t {
            const int rows = min(UR, p.seg_rows - mt * UR);
            return static_cast<int64_t>((rows + 127) / 128) * srow_bytes;
          };
          auto step_chunks = [&](int mt) -> uint32_t {  // chunks of tile row mt that this warp moves
            const uint32_t nch = payload_chunks(mt) + static_cast<uint32_t>((scale_bytes(mt) + CH - 1) / CH);
            return nch > cw ? (nch - cw - 1) / ncw + 1 : 0u;
          };
          auto publish = [&](int d, int mt) {
            int peer = p.rank - d;
            if (peer < 0) peer += p.world;
            ptx::fence_proxy_async_all();
            // the last of the 2*gridDim.x pushing warps publishes the tile row to the peer
            uint32_t* cnt = p.local_cnt + d * units + mt;
            if (ptx::atom_add_acq_rel_sys(cnt, 1u) == ncw - 1u) {
              *cnt = 0;
              ptx::st_release_sys(p.ag_flags[peer] + p.rank * units + mt, p.epoch);
            }
          };
          // this warp's chunks, step by step (destination, then row unit); chunk c of a step
          // belongs to warp c % ncw
          int g_d = 1, g_mt = 0;
          uint32_t g_c = cw;
          auto gen = [&](const uint8_t*& from, uint8_t*& to, uint32_t& sz) -> bool {
            for (;;) {
              if (g_d >= p.world) return false;
              const int rows = min(UR, p.seg_rows - g_mt * UR);
              const uint32_t nch_p = payload_chunks(g_mt);
              const int64_t sbytes = scale_bytes(g_mt);
              const uint32_t nch = nch_p + static_cast<uint32_t>((sbytes + CH - 1) / CH);
              if (g_c < nch) {
                int peer = p.rank - g_d;
                if (peer < 0) peer += p.world;
                int64_t left;
                if (g_c < nch_p) {
                  const int64_t off = static_cast<int64_t>(g_mt) * UR * row_bytes + static_cast<int64_t>(g_c) * CH;
                  from = src + off;
                  to = reinterpret_cast<uint8_t*>(p.ag_land[peer]) + slab_off + off;
                  left = rows * row_bytes - static_cast<int64_t>(g_c) * CH;
                } else {
                  const int64_t off = static_cast<int64_t>(g_mt) * (UR / 128) * srow_bytes +
                                      static_cast<int64_t>(g_c - nch_p) * CH;
                  from = ssrc + off;
                  to = reinterpret_cast<uint8_t*>(p.ag_scale_land[peer]) + sslab_off + off;
                  left = sbytes - static_cast<int64_t>(g_c - nch_p) * CH;
                }
                sz = left < static_cast<int64_t>(CH) ? static_cast<uint32_t>(left) : CH;
                g_c += ncw;
                if (!dcheck(wc, left > 0 && (sz & 15u) == 0u && (reinterpret_cast<uintptr_t>(from) & 15u) == 0u &&
                                    (reinterpret_cast<uintptr_t>(to) & 15u) == 0u,
                            kCheckAgPush, static_cast<uint32_t>(g_d * units + g_mt), sz))
                  return false;
                return true;
              }
              g_c = cw;
              if (++g_mt == units) {
                g_mt = 0;
                ++g_d;
              }
            }
          };
          // NSLOT - 1 loads are in flight ahead of the store being issued
          uint8_t* q_to[NSLOT];
          uint32_t q_sz[NSLOT];
          uint32_t head = 0, tail = 0;   // stores issued, loads issued
          auto issue = [&]() -> bool {
            const uint8_t* from;
            uint8_t* to;
            uint32_t sz;
            if (!gen(from, to, sz)) return false;
            const uint32_t slot = tail % NSLOT;
            q_to[slot] = to;
            q_sz[slot] = sz;
            ptx::mbar_arrive_expect_tx(rbar + 8u * slot, sz);
            ptx::bulk_load(ring + slot * CH, from, sz, rbar + 8u * slot);
            ++tail;
            return true;
          };
          int sig_d = 1, sig_mt = 0;           // next step to publish
          uint32_t sig_end = step_chunks(0);   // own chunks through that step
          const int inflight = p.ag_inflight >= 1 && p.ag_inflight <= NSLOT - 1 ? p.ag_inflight : NSLOT - 1;
          for (int k = 0; k < inflight; ++k)
            if (!issue()) break;
          while (head < tail) {
            const uint32_t slot = head % NSLOT;
            mbar_wait(wc, rbar + 8u * slot, (head / NSLOT) & 1u, kSiteSmemFull);
            ptx::bulk_store(q_to[slot], ring + slot * CH, q_sz[slot]);
            ptx::bulk_commit();
            ++head;
            // the slot of the next load was last read by the store NSLOT - inflight + 1 back
            if (inflight == 3) ptx::bulk_wait_read<1>();
            else if (inflight == 2) ptx::bulk_wait_read<2>();
            else ptx::bulk_wait_read<3>();
            issue();
            // everything but the LAG most recent chunk stores has landed: publish the steps
            // that lie entirely before that point
            ptx::bulk_wait<LAG>();
            const uint32_t done = head > LAG ? head - LAG : 0u;
            while (sig_d < p.world && sig_end <= done) {
              publish(sig_d, sig_mt);
              if (++sig_mt == units) { sig_mt = 0; ++sig_d; }
              if (sig_d < p.world) sig_end += step_chunks(sig_mt);
            }
          }
          ptx::bulk_wait<0>();
          while (sig_d < p.world) {
            publish(sig_d, sig_mt);
            if (++sig_mt == units) { sig_mt = 0; ++sig_d; }
          }
          if (warp == 2) stamp(kTracePushDone);
        }
      }
    }
    if constexpr (Cfg::COMM_BYTES > 0) {
      if (p.mode == kModeA2AGemm) {
        // heads->seq all-to-all: every rank sends, for each destination d, the rows of its
        // attention output that belong to d's sequence range, re-laid out so that they form
        // columns [rank*local_heads*hd, +local_heads*hd) of d's GEMM input.
        if (multi) {
          if (lane < p.world) flag_wait_ge(wc, p.start_ctr[p.rank] + lane, p.epoch, kSiteStartBarrier);
          __syncwarp();
        }
        if (lane == 0 && warp == 2) stamp(kTraceHandshake);
        if (lane == 0) {
          // One lane per warp: bulk-load a 4 KiB piece of the attention output (RG rows of one head,
          // one contiguous run) into one of two staging slots, one load ahead of the stores, and
          // bulk-store it into the peer's landing slab for this source. The pieces of the whole
          // exchange are numbered in the order (row unit, destination step, piece) and claimed in
          // that order, four at a time, by the pushing warps: warps on SMs that get more of the
          // link take more pieces, and every rank fills the first row unit of all its peers first -
          // the rows that the first wave of tiles reads. Small pieces keep the time between a piece
          // landing and its step being published short.
          constexpr int NSLOT = 2;
          constexpr int PF = NSLOT - 1;                            // loads in flight ahead of the store
          constexpr uint32_t SLOT = Cfg::COMM_BYTES / 2 / NSLOT;   // 4 KiB
          constexpr int LAG = 2;        // stores that may still be on their way when arrivals are counted
          constexpr uint32_t BATCH = 4; // pieces per claim
          const uint32_t ring = comm_base + (warp - 2) * (Cfg::COMM_BYTES / 2);
          const uint32_t rbar = ring_bar_base + (warp - 2) * 4 * 8u;
          const uint32_t ncw = gridDim.x * 2;
          const int hd = p.a2a_hd, lh = p.a2a_local_heads, ls = p.a2a_local_seq;
          const int RG = static_cast<int>(SLOT) / (hd * 2);         // rows per piece: 16 (hd 128) or 32 (hd 64)
          const uint32_t chunk_bytes = static_cast<uint32_t>(RG) * hd * 2u;
          const int UR = p.flag_unit_rows;
          const int rows_total = p.a2a_bs * ls;
          const int units = (rows_total + UR - 1) / UR;
          const int d0 = p.a2a_copy_local ? 0 : 1;             // step 0 is the local slice
          const int nd = p.world - d0;
          const int nsteps = units * nd;
          auto step_nch = [&](int s) -> uint32_t {             // pieces of step s
            const int mt = s / nd;
            const int rows = min(UR, rows_total - mt * UR);
            return static_cast<uint32_t>(((rows + RG - 1) / RG) * lh);
          };
          uint32_t total = 0;
          for (int s = 0; s < nsteps; ++s) total += step_nch(s);
          const uint32_t nbatch = (total + BATCH - 1) / BATCH;
          const uint8_t* attn = reinterpret_cast<const uint8_t*>(p.a2a_attn);
          const int64_t seq = static_cast<int64_t>(ls) * p.world;
          // walker over the steps (this warp's pieces come in increasing order)
          int w_s = 0, w_mt = 0, w_peer = 0;
          uint32_t w_first = 0, w_n = nsteps > 0 ? step_nch(0) : 0u;
          auto enter_step = [&]() {
            w_mt = w_s / nd;
            w_peer = p.rank + d0 + w_s % nd;
            if (w_peer >= p.world) w_peer -= p.world;
          };
          enter_step();
          // what is in each staging slot: destination, offset there, step
          int q_peer[NSLOT], q_step[NSLOT];
          int64_t q_doff[NSLOT];
          auto issue_load = [&](uint32_t g, uint32_t idx) {
            while (g >= w_first + w_n) {
              w_first += w_n;
              ++w_s;
              w_n = step_nch(w_s);
              enter_step();
            }
            const uint32_t c = g - w_first;
            const int i = static_cast<int>(c % lh);                      // head (layout 0) / part of the row group
            const int row0 = w_mt * UR + static_cast<int>(c / lh) * RG;  // row of the peer's GEMM input
            const int b = row0 / ls, s0 = row0 % ls;
            int64_t soff, doff;
            if (p.a2a_layout == 0) {
              soff = ((static_cast<int64_t>(b) * lh + i) * seq + static_cast<int64_t>(w_peer) * ls + s0) * hd * 2;
              doff = ((static_cast<int64_t>(p.rank) * lh + i) * rows_total + row0) * hd * 2;
            } else {
              // RG rows of all heads are one run of lh pieces
              soff = ((static_cast<int64_t>(b) * seq + static_cast<int64_t>(w_peer) * ls + s0) * lh + i * RG) * hd * 2;
              doff = ((static_cast<int64_t>(p.rank) * rows_total + row0) * lh + i * RG) * hd * 2;
            }
            const uint32_t slot = idx % NSLOT;
            {
              const int64_t src_bytes = static_cast<int64_t>(p.a2a_bs) * lh * seq * hd * 2;
              const int64_t land_bytes = static_cast<int64_t>(p.world) * lh * rows_total * hd * 2;
              dcheck(wc, soff >= 0 && soff + chunk_bytes <= src_bytes && doff >= 0 &&
                             doff + chunk_bytes <= land_bytes && ((soff | doff) & 15) == 0,
                     kCheckA2APush, g, static_cast<uint32_t>(w_s));
            }
            q_peer[slot] = w_peer;
            q_step[slot] = w_s;
            q_doff[slot] = doff;
            ptx::mbar_arrive_expect_tx(rbar + 8u * slot, chunk_bytes);
            ptx::bulk_load(ring + slot * SLOT, attn + soff, chunk_bytes, rbar + 8u * slot);
          };
          // Pieces of step s have landed (their bulk groups are complete: the bytes are visible to
          // this thread, and the release below carries them); whoever lands the last piece of the
          // step tells the peer. Arrivals of the same step are counted together, up to BATCH.
          int pend_s = -1;
          uint32_t pend_n = 0;
          auto flush = [&]() {
            if (pend_n == 0) return;
            const int mt = pend_s / nd;
            int peer = p.rank + d0 + pend_s % nd;
            if (peer >= p.world) peer -= p.world;
            uint32_t* cnt = p.local_cnt + pend_s;
            if (ptx::atom_add_acq_rel_gpu(cnt, pend_n) + pend_n == step_nch(pend_s)) {
              *cnt = 0;
              ptx::st_release_sys(p.a2a_flags[peer] + p.rank * units + mt, p.epoch);
            }
            pend_n = 0;
          };
          auto landed = [&](int s) {
            if (s != pend_s) {
              flush();
              pend_s = s;
            }
            if (++pend_n == BATCH) flush();
          };
          // claims: batch b is pieces [b * BATCH, (b + 1) * BATCH); every warp ends with one failed
          // claim, and the last of those puts the counter back to zero
          uint32_t* claim = p.local_cnt + 1024;
          bool exhausted = false;
          uint32_t cur = 0, cur_end = 0;
          constexpr uint32_t NONE = 0xffffffffu;
          auto next_piece = [&]() -> uint32_t {
            if (cur == cur_end) {
              if (exhausted) return NONE;
              const uint32_t b = atomicAdd(claim, 1u);
              if (b >= nbatch) {
                exhausted = true;
                if (b == nbatch + ncw - 1u) atomicExch(claim, 0u);
                return NONE;
              }
              cur = b * BATCH;
              cur_end = min(cur + BATCH, total);
            }
            return cur++;
          };
          int stepq[8];           // step of the last eight stored pieces
          uint32_t nload = 0, nstore = 0, counted = 0;
          for (int k = 0; k < PF; ++k) {
            const uint32_t g = next_piece();
            if (g == NONE) break;
            issue_load(g, nload);
            ++nload;
          }
          while (nstore < nload) {
            const uint32_t slot = nstore % NSLOT;
            mbar_wait(wc, rbar + 8u * slot, (nstore / NSLOT) & 1u, kSiteSmemFull);
            ptx::bulk_store(reinterpret_cast<uint8_t*>(p.a2a_land[q_peer[slot]]) + q_doff[slot], ring + slot * SLOT,
                            chunk_bytes);
            ptx::bulk_commit();
            stepq[nstore & 7u] = q_step[slot];
            ++nstore;
            const uint32_t gn = next_piece();
            if (gn != NONE) {
              ptx::bulk_wait_read<NSLOT - 1>();   // the store that last used the slot (piece nload - NSLOT) has read it
              issue_load(gn, nload);
              ++nload;
            }
            // all but the LAG most recent stores have landed
            ptx::bulk_wait<LAG>();
            while (counted + LAG < nstore) {
              landed(stepq[counted & 7u]);
              ++counted;
            }
          }
          ptx::bulk_wait<0>();
          while (counted < nstore) {
            landed(stepq[counted & 7u]);
            ++counted;
          }
          flush();
          if (warp == 2) stamp(kTracePushDone);
        }
      }
    }
  }
  } else {
      if constexpr (Cfg::BS) ptx::setmaxnreg_inc<(BN == 256 ? 232 : 208)>();
    // ------------------------------------------------------------------ epilogue
    const int q = warp & 3;              // TMEM lane quadrant this warp may read
    const int ew = warp - 4;             // epilogue warp index
    uint8_t* my_epi = epi_ptr + ew * Cfg::EPI_BUFS * Cfg::EPI_BUF_BYTES;
    const uint32_t my_epi_u32 = epi_base + ew * Cfg::EPI_BUFS * Cfg::EPI_BUF_BYTES;
    const uint16_t* bias = reinterpret_cast<const uint16_t*>(p.bias);
    const bool f16 = p.out_f16 != 0;
    const bool sa_vec = (p.scale_flags & 1u) != 0u, sb_vec = (p.scale_flags & 2u) != 0u;
    float alpha = 1.f;
    if (p.scale_a != nullptr && !sa_vec) alpha *= *p.scale_a;
    if (p.scale_b != nullptr && !sb_vec) alpha *= *p.scale_b;
    const bool scaled = p.scale_a != nullptr || p.scale_b != nullptr;
    int it = 0;
    uint32_t nstore = 0;
    bool started = !(multi && (p.mode == kModeReduceScatter || p.mode == kModeGemmA2A));

    // Reduce-scatter, tiles of the own segment: add the partial results that the W-1 peers stored
    // into this rank's staging slabs (64 columns of this thread's row per source, sources in the
    // order rank+1, rank+2, ...; the loads of the next source are in flight while one is added).
    const uint8_t* rs_stage_b = reinterpret_cast<const uint8_t*>(p.rs_stage);
    auto add_peers = [&](uint32_t (&r0)[32], uint32_t (&r1)[32], int col0, int row) {
      if (row >= p.seg_rows || col0 >= p.N) return;
      uint4 v[2][8];
      const int64_t row_bytes = static_cast<int64_t>(p.N) * 2;
      const int64_t slab_bytes = row_bytes * p.seg_rows;
      const int ncol = p.N - col0;   // valid columns from col0 on (a multiple of 8)
      auto load_src = [&](uint4 (&dst)[8], int d) {
        int src = p.rank + d;
        if (src >= p.world) src -= p.world;
        const uint8_t* base = rs_stage_b + src * slab_bytes + row * row_bytes + static_cast<int64_t>(col0) * 2;
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          if (8 * j < ncol) dst[j] = ptx::ld_global_cs_v4(base + 16 * j);
          else dst[j] = make_uint4(0u, 0u, 0u, 0u);
        }
      };
      auto add_src = [&](const uint4 (&src)[8]) {
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          const uint32_t w[4] = {src[j].x, src[j].y, src[j].z, src[j].w};
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            const int c = 8 * j + 2 * e;   // column inside the 64-column chunk
            const float lo = ptx::half_bits_to_float(static_cast<uint16_t>(w[e] & 0xFFFFu), f16);
            const float hi = ptx::half_bits_to_float(static_cast<uint16_t>(w[e] >> 16), f16);
            if (c < 32) {
              r0[c] = __float_as_uint(__uint_as_float(r0[c]) + lo);
              r0[c + 1] = __float_as_uint(__uint_as_float(r0[c + 1]) + hi);
            } else {
              r1[c - 32] = __float_as_uint(__uint_as_float(r1[c - 32]) + lo);
              r1[c - 31] = __float_as_uint(__uint_as_float(r1[c - 31]) + hi);
            }
          }
        }
      };
      load_src(v[1], 1);
#pragma unroll
      for (int d = 1; d < kMaxRanks; ++d) {
        if (d < p.world) {
          if (d + 1 < p.world) load_src(v[(d + 1) & 1], d + 1);
          add_src(v[d & 1]);
        }
      }
    };

    // 32 rows x 64 columns of fp32 results (r0: columns 0..31, r1: 32..63 of the chunk, this
    // thread's row) -> scale, bias, activation (-> + peers' partial results) -> 16-bit -> swizzled
    // staging -> TMA store
    auto emit_chunk = [&](uint32_t (&r0)[32], uint32_t (&r1)[32], int col0, int row, int64_t grow,
                          int store_row0, const CUtensorMap* tmd, int z, bool own_rs) {
      if constexpr (Cfg::KIND == 2) {   // s32 accumulators of the int8 kind
#pragma unroll
        for (int j = 0; j < 32; ++j) {
          r0[j] = __float_as_uint(__int2float_rn(static_cast<int32_t>(r0[j])));
          r1[j] = __float_as_uint(__int2float_rn(static_cast<int32_t>(r1[j])));
        }
      }
      if (scaled) {
        // per-tensor scales, or one scale per row (A) / per column (B)
        float ar = alpha;
        if (sa_vec) ar *= row < p.seg_rows ? p.scale_a[grow] : 0.f;
        if (sb_vec) {
#pragma unroll
          for (int j = 0; j < 32; ++j) {
            const float b0 = col0 + j < p.N ? p.scale_b[col0 + j] : 0.f;
            const float b1 = col0 + 32 + j < p.N ? p.scale_b[col0 + 32 + j] : 0.f;
            r0[j] = __float_as_uint(__uint_as_float(r0[j]) * (ar * b0));
            r1[j] = __float_as_uint(__uint_as_float(r1[j]) * (ar * b1));
          }
        } else {
#pragma unroll
          for (int j = 0; j < 32; ++j) {
            r0[j] = __float_as_uint(__uint_as_float(r0[j]) * ar);
            r1[j] = __float_as_uint(__uint_as_float(r1[j]) * ar);
          }
        }
      }
      if (bias != nullptr && col0 < p.N) {
        const uint16_t* brow = bias + (p.bias_row_stride ? grow * p.bias_row_stride : 0);
        const bool row_ok = row < p.seg_rows;
#pragma unroll
        for (int j = 0; j < 32; ++j) {
          if (row_ok && col0 + j < p.N)
            r0[j] = __float_as_uint(__uint_as_float(r0[j]) + ptx::half_bits_to_float(brow[col0 + j], f16));
          if (row_ok && col0 + 32 + j < p.N)
            r1[j] = __float_as_uint(__uint_as_float(r1[j]) +
                                    ptx::half_bits_to_float(brow[col0 + 32 + j], f16));
        }
      }
      if (p.act != 0) {
#pragma unroll
        for (int j = 0; j < 32; ++j) {
          r0[j] = __float_as_uint(ptx::activate(__uint_as_float(r0[j]), p.act));
          r1[j] = __float_as_uint(ptx::activate(__uint_as_float(r1[j]), p.act));
        }
      }
      if (own_rs) add_peers(r0, r1, col0, row);
      const uint32_t buf = Cfg::EPI_BUFS == 2 ? (nstore & 1u) : 0u;
      if (lane == 0) ptx::bulk_wait_read<Cfg::EPI_BUFS - 1>();
      __syncwarp();
      uint8_t* dst = my_epi + buf * Cfg::EPI_BUF_BYTES + lane * 128;
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        uint4 v;
        v.x = ptx::pack_half2(f16, __uint_as_float(r0[8 * j + 0]), __uint_as_float(r0[8 * j + 1]));
        v.y = ptx::pack_half2(f16, __uint_as_float(r0[8 * j + 2]), __uint_as_float(r0[8 * j + 3]));
        v.z = ptx::pack_half2(f16, __uint_as_float(r0[8 * j + 4]), __uint_as_float(r0[8 * j + 5]));
        v.w = ptx::pack_half2(f16, __uint_as_float(r0[8 * j + 6]), __uint_as_float(r0[8 * j + 7]));
        *reinterpret_cast<uint4*>(dst + ((j ^ (lane & 7)) << 4)) = v;
      }
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        uint4 v;
        v.x = ptx::pack_half2(f16, __uint_as_float(r1[8 * j + 0]), __uint_as_float(r1[8 * j + 1]));
        v.y = ptx::pack_half2(f16, __uint_as_float(r1[8 * j + 2]), __uint_as_float(r1[8 * j + 3]));
        v.z = ptx::pack_half2(f16, __uint_as_float(r1[8 * j + 4]), __uint_as_float(r1[8 * j + 5]));
        v.w = ptx::pack_half2(f16, __uint_as_float(r1[8 * j + 6]), __uint_as_float(r1[8 * j + 7]));
        *reinterpret_cast<uint4*>(dst + (((j + 4) ^ (lane & 7)) << 4)) = v;
      }
      ptx::fence_proxy_async_smem();
      __syncwarp();
      if (lane == 0 && col0 < p.N && store_row0 < p.seg_rows &&
          dcheck(wc, store_row0 >= 0 && col0 >= 0 && (col0 & 7) == 0 && z >= 0 && z < kMaxRanks, kCheckStore,
                 static_cast<uint32_t>(col0), static_cast<uint32_t>(store_row0))) {
        if (p.mode == kModeGemmA2A) {
          // 64 columns of one head, 32 consecutive sequence positions of one batch entry:
          // goes to the rank that owns the head, at this rank's place in the full sequence
          const int head = col0 / p.a2a_hd, e0 = col0 % p.a2a_hd;
          int g = 0;
          while (g + 1 < p.a2a_groups && head >= p.a2a_group_start[g + 1]) ++g;
          const int hh = head - p.a2a_group_start[g];
          const int lh = (p.a2a_group_start[g + 1] - p.a2a_group_start[g]) / p.world;
          const int b = store_row0 / p.a2a_local_seq, s0 = store_row0 % p.a2a_local_seq;
          ptx::tma_store_4d(&p.tm_a2a[g * kMaxRanks + hh / lh], my_epi_u32 + buf * Cfg::EPI_BUF_BYTES, e0,
                            p.rank * p.a2a_local_seq + s0, hh % lh, b);
        } else {
          ptx::tma_store_3d(tmd, my_epi_u32 + buf * Cfg::EPI_BUF_BYTES, col0, store_row0, z);
        }
      }
      if (lane == 0) ptx::bulk_commit();
      if (nstore == 0 && ew == 0 && lane == 0) stamp(kTraceFirstStore);
      ++nstore;
    };

    // the tile row's slab has fully landed at the owner: the last of the warps that store into
    // it tells the owner
    // (counted in 64-column chunk stores per warp, so that split tiles add up to the same total)
    const uint32_t rs_row_total = static_cast<uint32_t>(n_tiles) * (BN / 64) * Cfg::MT * 4u * CG;
    auto rs_arrive = [&](int seg, int mt, uint32_t chunks) {
      ptx::fence_proxy_async_all();
      uint32_t* cnt = p.local_cnt + seg * m_tiles_seg + mt;
      if (ptx::atom_add_acq_rel_sys(cnt, chunks) + chunks == rs_row_total) {
        *cnt = 0;
        ptx::st_release_sys(p.rs_ctr[seg] + mt * kMaxRanks + p.rank, p.epoch);
      }
    };
    int pend_seg = -1, pend_mt = 0;
    uint32_t pend_chunks = 0;
    uint32_t own_seen = 0;   // tile rows of the own segment whose W-1 slabs were seen to have landed
    uint64_t bs_acc[Cfg::BS ? BN / 4 : 1];   // block-scaled: this thread's row x BN / 2 columns, fp32 pairs
#ifdef FLUXB_DEBUG_CHECKS
    uint64_t probe_wait = 0, probe_ld = 0, probe_kb = 0, probe_total = 0;
    const long long probe_t0 = clock64();
#endif
    for (int t = tile_slot; t < total_tiles; t += tile_stride, ++it) {
      if (*abort_word) break;
      const TileCoord c = decode_tile(p, t, m_tiles_seg, n_tiles, BM, BN);
      const int m_cta = c.m_in_seg + static_cast<int>(cta_rank) * Cfg::BM_CTA;
      const CUtensorMap* tmd = &p.tm_d[0];
      int z = c.seg;
      if (p.mode == kModeGemmA2A && multi && !started) {
        if (lane < p.world) flag_wait_ge(wc, p.start_ctr[p.rank] + lane, p.epoch, kSiteStartBarrier);
        __syncwarp();
        started = true;
      }
      bool own_rs = false;
      if (p.mode == kModeReduceScatter && multi) {
        tmd = &p.tm_d[c.seg];
        z = p.rank;
        if (c.seg == p.rank && !p.rs_tail) {
          // own segment: every peer's partial rows of this tile row must have landed; the result
          // goes to rs_out (tm_d[rank] covers it as one slab)
          own_rs = true;
          z = 0;
          // The arrival of this warp's last tile for a peer is still pending (it is counted one
          // tile late). It must be counted before this warp waits for the peers, whose own tiles
          // wait for exactly such arrivals from this rank: otherwise the ranks wait for each other.
          if (pend_seg >= 0) {
            if (lane == 0) {
              ptx::bulk_wait<0>();
              rs_arrive(pend_seg, pend_mt, pend_chunks);
            }
            pend_seg = -1;
            __syncwarp();
          }
          if (c.m_tile >= 32 || ((own_seen >> c.m_tile) & 1u) == 0u) {
            if (own_seen == 0 && ew == 0 && lane == 0) stamp(kTraceSlice0);
            if (lane < p.world && lane != p.rank)
              flag_wait_ge(wc, p.rs_ctr[p.rank] + c.m_tile * kMaxRanks + lane, p.epoch, kSiteTileCounter);
            __syncwarp();
            if (c.m_tile < 32) own_seen |= 1u << c.m_tile;
          }
        }
        if (!started) {
          // peers may still be reducing the previous call's slabs until they enter this call
          if (lane < p.world) flag_wait_ge(wc, p.start_ctr[p.rank] + lane, p.epoch, kSiteStartBarrier);
          __syncwarp();
          started = true;
        }
      }
      int row = m_cta + q * 32 + lane;                         // row inside the segment
      int64_t grow = static_cast<int64_t>(c.seg) * p.seg_rows + row;  // global row

      if constexpr (Cfg::BS) {
        // ---- block-scaled: promote every k-block's partial product into fp32 registers.
        // Eight epilogue warps: warp (quadrant q, half) owns rows q*32.. of the tile and columns
        // half*64.. for every k-block, so its partial sums never leave its registers. Two warps share
        // a scheduler: while one waits for its TMEM read, the other multiplies.
        const int half = ew >> 2;
        const int kbs = k_blocks;                               // scale blocks along K (BK == 128)
        const float* sa_rows = p.sa;
        // rows of a pair tile past the end of the segment (their results are clipped by the store) have no
        // scales: they read those of the segment's first row
        const int row_s = row < ((p.seg_rows + 127) & ~127) ? row : 0;
        int64_t srow = static_cast<int64_t>(c.seg) * p.seg_rows + row_s;   // row in the scale tensor's frame
        if (p.mode == kModeAllGather && multi) {
          if (c.seg == p.rank) {
            srow = row_s;
          } else {
            sa_rows = p.sa_land;
            // the scales travelled with the shard: make this thread's reads follow the flag
            const uint32_t* f = p.ag_flags[p.rank] + c.seg * ((p.seg_rows + p.flag_unit_rows - 1) / p.flag_unit_rows) +
                                c.m_in_seg / p.flag_unit_rows;
            if (lane == 0) flag_wait_ge(wc, f, p.epoch, kSiteShardFlag);
            __syncwarp();
          }
        }
        const float* sa_ptr = sa_rows + (srow >> 7) * static_cast<int64_t>(kbs) * 128 + (srow & 127);
        // this warp's columns: half * CW .. + CW of the tile (CW = 64 of 128, or 128 of 256: then the two
        // halves lie in different 128-column scale blocks of the weight)
        constexpr int CW = BN / 2, NCH = CW / 64;
        int nblk = (c.n0 >> 7) + (BN == 256 ? half : 0);
        if (nblk >= (p.N >> 7)) nblk = (p.N >> 7) - 1;          // (the clipped half of the last tile)
        const float* sb_ptr = p.sb + static_cast<int64_t>(nblk) * kbs;
        const int sb_col = BN == 256 ? 0 : half * 64;           // first column of the warp inside its scale block
        const uint32_t lane_base = tmem_base + (static_cast<uint32_t>(q * 32) << 16) + half * CW;
#pragma unroll
        for (int j = 0; j < NCH * 32; ++j) bs_acc[j] = 0ull;
        const uint32_t n0 = static_cast<uint32_t>(it) * kbs;
        // Scales are fetched G k-blocks at a time, one group ahead: four with 128-column tiles; two with
        // 256-column tiles, whose 128 accumulator registers per thread leave little room (one k-block ahead
        // measured 1170 TFLOP/s, two 1350, four 1320 with more spills).
        constexpr int G = NCH == 2 ? 2 : 4;
        float csa[G], csb[G], nsa[G], nsb[G];
        auto load_scales = [&](int kb0, float* dsa, float* dsb) {
#pragma unroll
          for (int i = 0; i < G; ++i) {
            const int kk = kb0 + i < kbs ? kb0 + i : kbs - 1;   // past the end: a repeated, unused load
            dsa[i] = sa_ptr[static_cast<int64_t>(kk) * 128];
            dsb[i] = p.sb_groupwise ? 1.f : sb_ptr[kk];
          }
        };
        load_scales(0, csa, csb);
        for (int kb0 = 0; kb0 < kbs; kb0 += G) {
          load_scales(kb0 + G, nsa, nsb);
#pragma unroll
          for (int ki = 0; ki < G; ++ki) {
            const int kb = kb0 + ki;
            if (kb >= kbs) break;
            const uint32_t n = n0 + kb;
            const int buf = n % NACC;
            const uint32_t par = (n / NACC) & 1u;
            const float sc = csa[ki] * csb[ki];
            const uint64_t sc2 = ptx::pack_f32x2(sc, sc);
            // 32 columns of the k-block's partial product (in r), first accumulator a0, first column col
            // of the warp's range: acc += r * scale
            auto promote = [&](const uint32_t (&r)[32], int a0, int col) {
              if (p.sb_groupwise) {
                // per-column weight scales of this k-block (the same for every row)
                const float4* sbv = reinterpret_cast<const float4*>(
                    p.sb + (static_cast<int64_t>(nblk) * kbs + kb) * 128 + sb_col + col);
#pragma unroll
                for (int j = 0; j < 8; ++j) {
                  const float4 sv = sbv[j];
                  bs_acc[a0 + 2 * j] = ptx::ffma2(ptx::pack_b32x2(r[4 * j], r[4 * j + 1]),
                                                  ptx::pack_f32x2(sc * sv.x, sc * sv.y), bs_acc[a0 + 2 * j]);
                  bs_acc[a0 + 2 * j + 1] = ptx::ffma2(ptx::pack_b32x2(r[4 * j + 2], r[4 * j + 3]),
                                                      ptx::pack_f32x2(sc * sv.z, sc * sv.w), bs_acc[a0 + 2 * j + 1]);
                }
              } else {
#pragma unroll
                for (int j = 0; j < 16; ++j)
                  bs_acc[a0 + j] = ptx::ffma2(ptx::pack_b32x2(r[2 * j], r[2 * j + 1]), sc2, bs_acc[a0 + j]);
              }
            };
            auto hand_over = [&]() {
              ptx::tc_fence_before();
              __syncwarp();
              if (lane == 0) {
                // The buffer's contents are in registers (wait::ld), so the hand-over needs no release ordering.
                // A cluster-scope release arrive also waits for the warp's scale loads in flight, which
                // halved the throughput of CTA pairs.
                if (CG == 1 || cta_rank == 0) ptx::mbar_arrive_relaxed(tempty_bar(buf));
                else ptx::mbar_arrive_remote_relaxed(tempty_bar(buf), 0);
              }
            };
#ifdef FLUXB_DEBUG_CHECKS
            const long long pc0 = clock64();
#endif
            if (lane == 0) mbar_wait(wc, tfull_bar(buf), par, kSiteTmemFull);
            __syncwarp();
            mbar_wait(wc, tfull_bar(buf), par, kSiteTmemFull);
            ptx::tc_fence_after();
#ifdef FLUXB_DEBUG_CHECKS
            const long long pc1 = clock64();
#endif
            const uint32_t taddr = lane_base + buf * BN;
            if constexpr (NCH == 1) {
              uint32_t r0[32], r1[32];
              ptx::tmem_ld_32x32b_x32(taddr, r0);
              ptx::tmem_ld_32x32b_x32(taddr + 32, r1);
              ptx::tmem_ld_wait();
#ifdef FLUXB_DEBUG_CHECKS
              probe_ld += static_cast<uint64_t>(clock64() - pc1);
#endif
              hand_over();
              promote(r0, 0, 0);
              promote(r1, 16, 32);
            } else {
              // 128 columns, 32 at a time through one set of staging registers: the warp that shares the
              // scheduler multiplies while this one waits for its read
              uint32_t r0[32];
#pragma unroll
              for (int c4 = 0; c4 < 4; ++c4) {
                ptx::tmem_ld_32x32b_x32(taddr + 32 * c4, r0);
                ptx::tmem_ld_wait();
                if (c4 == 3) {
#ifdef FLUXB_DEBUG_CHECKS
                  probe_ld += static_cast<uint64_t>(clock64() - pc1);
#endif
                  hand_over();
                }
                promote(r0, 16 * c4, 32 * c4);
              }
            }
#ifdef FLUXB_DEBUG_CHECKS
            // self-checking build: cycles of this warp waiting for the k-block's MMAs (the multiply-adds of
            // k-block kb are charged to the wait of k-block kb + 1 where they are still in flight) and
            // reading TMEM (with 256-column tiles: including the first half's multiply-adds)
            probe_wait += static_cast<uint64_t>(pc1 - pc0);
            probe_kb += 1;
            probe_total = static_cast<uint64_t>(clock64() - probe_t0);   // whole promotion loop of this warp so far
#endif
          }
#pragma unroll
          for (int i = 0; i < G; ++i) {
            csa[i] = nsa[i];
            csb[i] = nsb[i];
          }
        }
        // ---- this warp's 32 rows x CW columns of the tile
#pragma unroll
        for (int ch = 0; ch < NCH; ++ch) {
          uint32_t r0[32], r1[32];
#pragma unroll
          for (int j = 0; j < 16; ++j) {
            r0[2 * j] = static_cast<uint32_t>(bs_acc[ch * 32 + j]);
            r0[2 * j + 1] = static_cast<uint32_t>(bs_acc[ch * 32 + j] >> 32);
            r1[2 * j] = static_cast<uint32_t>(bs_acc[ch * 32 + 16 + j]);
            r1[2 * j + 1] = static_cast<uint32_t>(bs_acc[ch * 32 + 16 + j] >> 32);
          }
          emit_chunk(r0, r1, c.n0 + half * CW + ch * 64, row, grow, m_cta + q * 32, tmd, z, own_rs);
        }
      } else if constexpr (Cfg::MT == 2) {
        // both row halves of the tile complete together; accumulator 0 is drained (and handed
        // back to the issuer) first
        const uint32_t par = static_cast<uint32_t>(it) & 1u;
        if (lane == 0) mbar_wait(wc, tfull_bar(0), par, kSiteTmemFull);
        __syncwarp();
        mbar_wait(wc, tfull_bar(0), par, kSiteTmemFull);
        ptx::tc_fence_after();
        const int nch = (BN >> c.shift) / 64;
#pragma unroll 1
        for (int h = 0; h < 2; ++h) {
          row = m_cta + h * 128 + q * 32 + lane;
          grow = static_cast<int64_t>(c.seg) * p.seg_rows + row;
#pragma unroll 1
          for (int ch = 0; ch < nch; ++ch) {
            uint32_t r0[32], r1[32];
            const uint32_t taddr = tmem_base + (static_cast<uint32_t>(q * 32) << 16) + h * BN + ch * 64;
            ptx::tmem_ld_32x32b_x32(taddr, r0);
            ptx::tmem_ld_32x32b_x32(taddr + 32, r1);
            ptx::tmem_ld_wait();
            if (ch == nch - 1) {
              ptx::tc_fence_before();
              __syncwarp();
              if (lane == 0) ptx::mbar_arrive_remote(tempty_bar(h), 0);
            }
            emit_chunk(r0, r1, c.n0 + ch * 64, row, grow, m_cta + h * 128 + q * 32, tmd, z, own_rs);
          }
        }
      } else {
        const int acc = it & 1;
        const uint32_t acc_phase = (it >> 1) & 1;
        // one lane polls; the others sleep at the warp barrier and then observe the completed
        // phase with a single try_wait of their own
        if (lane == 0) mbar_wait(wc, tfull_bar(acc), acc_phase, kSiteTmemFull);
        __syncwarp();
        mbar_wait(wc, tfull_bar(acc), acc_phase, kSiteTmemFull);
        ptx::tc_fence_after();
        const int nch = (BN >> c.shift) / 64;
#pragma unroll 1
        for (int ch = 0; ch < nch; ++ch) {
          uint32_t r0[32], r1[32];
          const uint32_t taddr = tmem_base + (static_cast<uint32_t>(q * 32) << 16) + acc * BN + ch * 64;
          ptx::tmem_ld_32x32b_x32(taddr, r0);
          ptx::tmem_ld_32x32b_x32(taddr + 32, r1);
          ptx::tmem_ld_wait();
          if (ch == nch - 1) {
            ptx::tc_fence_before();
            __syncwarp();
            if (lane == 0) {
              if constexpr (CG == 1) ptx::mbar_arrive(tempty_bar(acc));
              else ptx::mbar_arrive_remote(tempty_bar(acc), 0);
            }
          }
          emit_chunk(r0, r1, c.n0 + ch * 64, row, grow, m_cta + q * 32, tmd, z, own_rs);
        }
      }
      if (p.mode == kModeReduceScatter && multi) {
        // Arrival counting runs one tile behind: waiting for this tile's stores to land would
        // stall the warp for an NVLink round trip, so wait only for the previous tile's (all but
        // the store groups committed for this tile) and count that one.
        if (lane == 0) {
          // store groups this warp committed for a whole tile; a piece of a split tile commits
          // fewer, so there everything is waited for
          constexpr int kGroupsPerTile = Cfg::BS ? BN / 128 : Cfg::MT * BN / 64;
          if (c.shift == 0) ptx::bulk_wait<kGroupsPerTile>();
          else ptx::bulk_wait<0>();
          if (pend_seg >= 0) rs_arrive(pend_seg, pend_mt, pend_chunks);
        }
        // own tiles that were summed in the epilogue stay here: nobody is told
        pend_seg = own_rs ? -1 : c.seg;
        pend_mt = c.m_tile;
        pend_chunks = Cfg::BS ? static_cast<uint32_t>(BN / 128)
                              : static_cast<uint32_t>(Cfg::MT * ((BN >> c.shift) / 64));
        __syncwarp();
      }
    }
    if (lane == 0) ptx::bulk_wait<0>();
    if (p.mode == kModeReduceScatter && multi && lane == 0 && pend_seg >= 0) rs_arrive(pend_seg, pend_mt, pend_chunks);
    __syncwarp();
    if constexpr (Cfg::BS) {
      // (named barrier 1: the eight promotion warps)
      if (p.mode == kModeReduceScatter && multi && p.rs_tail)
        rs_tail(static_cast<int>(threadIdx.x) - 128, [] { asm volatile("bar.sync 1, 256;" ::: "memory"); });
    }
    if (p.mode == kModeGemmA2A && multi) {
      // all stores of this warp have landed; the last warp of the whole grid tells every rank,
      // and everybody stays until all W sources have said so: when this kernel completes, the
      // local head-sharded output is complete
      if (lane == 0) {
        ptx::fence_proxy_async_all();
        if (ptx::atom_add_acq_rel_sys(p.local_cnt, 1u) == gridDim.x * Cfg::EPI_WARPS - 1u) {
          *p.local_cnt = 0;
          for (int d = 0; d < p.world; ++d) ptx::st_release_sys(p.a2a_flags[d] + p.rank, p.epoch);
        }
      }
      __syncwarp();
      if (lane < p.world) flag_wait_ge(wc, p.a2a_flags[p.rank] + lane, p.epoch, kSiteA2AFlag);
      __syncwarp();
    }
    if (ew == 0 && lane == 0) stamp(kTraceEnd);
#ifdef FLUXB_DEBUG_CHECKS
    if (Cfg::BS && p.trace != nullptr && ew == 0 && lane == 0) {
      uint64_t* tr = p.trace + blockIdx.x * kTraceWords;
      tr[8] = probe_wait;
      tr[9] = probe_ld;
      tr[11] = probe_kb;
      tr[10] = probe_total;   // cycles from this warp's start to the end of its last promotion
    }
#endif
  }

  // -------------------------------------------------------------------- teardown of the GEMM
  __syncwarp();
  if (*abort_word) {
    // A wait gave up and the roles left their loops early: give the copies and MMAs that are
    // still in flight time to land before this CTA's shared memory and TMEM go away.
    const uint64_t t0 = ptx::globaltimer_ns();
    while (ptx::globaltimer_ns() - t0 < 200000ull) __nanosleep(2000);
  }
  ptx::tc_fence_before();
  // CG == 2: nobody leaves (or frees TMEM) while the partner may still read this CTA's shared
  // memory or signal its barriers
  if constexpr (CG == 2) ptx::cluster_sync(); else __syncthreads();
  if (warp == 1) {
    ptx::tc_fence_after();
    ptx::tmem_dealloc<CG>(tmem_base, Cfg::TMEM_COLS);
  }

  // -------------------------------------------------------------------- reduce-scatter tail
  if constexpr (!Cfg::BS)
    if (p.mode == kModeReduceScatter && multi && p.rs_tail) rs_tail(static_cast<int>(threadIdx.x), [] { __syncthreads(); });
}

}  // namespace fluxb
