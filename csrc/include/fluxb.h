/* C ABI of libfluxb. Every function returns 0 on success or a fluxb error code
 * (1 invalid argument, 2 CUDA error, 3 unsupported, 4 device wait timed out);
 * fluxb_last_error() gives the message of the calling thread's last failure.
 * Pointers are device pointers unless stated otherwise; `stream` is a cudaStream_t. */
#ifndef FLUXB_H_
#define FLUXB_H_

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define FLUXB_MAX_RANKS 8

const char* fluxb_last_error(void);

/* element types */
enum { FLUXB_BF16 = 0, FLUXB_FP8_E4M3 = 1, FLUXB_FP16 = 2, FLUXB_FP32 = 3, FLUXB_FP8_E5M2 = 4, FLUXB_INT8 = 5 };
/* dense modes */
enum { FLUXB_PLAIN = 0, FLUXB_ALLGATHER = 1, FLUXB_REDUCE_SCATTER = 2, FLUXB_GEMM_A2A = 3, FLUXB_A2A_GEMM = 4 };

/* Status record written by device code when a bounded wait gives up. 16 bytes. */
typedef struct {
  uint32_t code, block, detail0, detail1;
} fluxb_status_t;

/* D = A * B^T (+ bias). A [rows, K] and B [N, K] row-major with K contiguous, D row-major.
 *   FLUXB_PLAIN          D[M, N]
 *   FLUXB_ALLGATHER      a = this rank's shard [M/world, K]; D[M, N]; peers' shards arrive in
 *                        ag_land[rank] ([world][M/world][K]) pushed by the peers' kernels
 *   FLUXB_REDUCE_SCATTER a = [M, K]; partial tiles of the peers' segments go to rs_stage[owner]
 *                        ([world][M/world][N]); the tiles of the own segment, computed last, add the
 *                        peers' slabs and store the sum over ranks to rs_out [M/world, N]
 * With world == 1 every mode degenerates to FLUXB_PLAIN on (a, d / rs_out). */
typedef struct {
  const void* a;
  const void* b;
  void* d;
  const void* bias;
  int64_t lda, ldb, ldd;     /* elements */
  int64_t bias_row_stride;   /* 0: bias is one row of N */
  int32_t M, N, K;
  int32_t in_dtype;          /* FLUXB_BF16 | FLUXB_FP16 | FLUXB_FP8_E4M3 | FLUXB_FP8_E5M2 | FLUXB_INT8 (signed) */
  int32_t out_dtype;         /* FLUXB_BF16 | FLUXB_FP16 (also the dtype of bias and rs_stage) */
  const float* scale_a;      /* optional device scales: D = (A*B^T) * scale_a * scale_b; one float each, or - see
                                scale_flags - scale_a one float per row of the whole problem ([M], the int8
                                convention of the reference) and scale_b one float per column ([N]) */
  const float* scale_b;
  int32_t mode, rank, world;
  int32_t group_m;           /* 0 = default raster group */
  int32_t num_sms;           /* 0 = all */
  int32_t tile_n;            /* 0 = auto, else 128 | 256 */
  int32_t act;               /* epilogue activation after bias: 0 none, 1 gelu(tanh), 2 relu, 3 silu */
  int32_t cta_group;         /* 0 = auto, 1 = one CTA per 128-row tile, 2 = CTA pair per 256-row tile */
  uint32_t epoch;            /* call number of the owning op, starting at 1 */
  uint32_t scale_flags;      /* bit 0: scale_a is a vector [M]; bit 1: scale_b is a vector [N] */
  uint64_t timeout_ns;       /* 0 = default (2 s) */
  fluxb_status_t* status;    /* device memory, may be null */
  void* ag_land[FLUXB_MAX_RANKS];
  uint32_t* ag_flags[FLUXB_MAX_RANKS];
  uint32_t* start_ctr[FLUXB_MAX_RANKS];
  void* rs_stage[FLUXB_MAX_RANKS];
  uint32_t* rs_ctr[FLUXB_MAX_RANKS];
  void* rs_out;
  uint32_t* wave_ctr;        /* optional: two device words owned by the caller (per op object), zero between
                                launches: [0] counts wave-synchronous tile starts (null = a word of the
                                launcher's per-stream pool), [1] hands out the work units of the
                                reduce-scatter tail (null = units dealt out round-robin) */
  uint32_t* local_cnt;       /* local scratch of world * ceil(M/world/128) uint32, zero at first use */
  /* block-scaled fp8 (blockscale != 0): inverse scales as fluxb_quantize_blockwise stores them.
   * sa [rows/128, K/128, 128] for the rows of `a`; sb [N/128, K/128]. In all-gather mode the
   * scales of the peers' shards arrive in ag_scale_land[rank] ([M/128, K/128, 128]). Needs
   * in_dtype FLUXB_FP8_E4M3, K % 128 == 0, N % 128 == 0 and M/world % 128 == 0. */
  const float* sa;
  const float* sb;
  float* ag_scale_land[FLUXB_MAX_RANKS];
  int32_t blockscale;        /* 0 off, 1: sb is [N/128, K/128], 2: sb is [N/128, K/128, 128] (one scale per weight row
                                and k-block: both operands carry 1x128 scales, the weight-gradient form) */
  int32_t tile_m;            /* 0 = auto, else 128 * cta_group, or 512 (CTA pairs on 256-column tiles: two
                                256-row MMAs per k-step share one B tile) */
  void* stream;
  /* optional timeline: [CTAs][16] uint64 of device memory receiving %globaltimer stamps (ns):
   * 0 roles start, 1 start handshake done, 2 pushes of communication warp 2 published, 3 loads of
   * the CTA's first tile issued, 4 loads of its last tile issued, 5 first epilogue store, 6 epilogue
   * done, 7 total ns the producer spent waiting for arrival flags, 8 + j: K slice j of the first tile
   * became readable (post-attention mode); reduce-scatter: 8 first own tile reached (two ranks), 9 / 10
   * the tail that sums the slabs entered / left (three ranks and more). Null = off. */
  uint64_t* trace;
  int32_t b_kn;              /* 1: b is [K, N] with N contiguous and ldb elements between k-rows (a weight held
                                transposed, e.g. for the data gradient): read in place as an MN-major operand;
                                16-bit inputs, not block-scaled */
  int32_t reserved_tail;
} fluxb_dense_args_t;

int fluxb_dense_gemm(const fluxb_dense_args_t* args);
/* Tile order of the reduce-scatter mode when raster bands span two segments: 1 when the first visited
 * segment must be a group of its own so that the own segment, visited last, is one too. */
int fluxb_rs_solo_first(int32_t num_seg);
/* Host evaluation of the dense kernel's tile order (the function the kernel itself calls):
 * out[3t..3t+2] = (segment, tile row in the segment, first column) of tile t, t < n. No GPU needed. */
int fluxb_decode_tiles(int32_t num_seg, int32_t seg_first, int32_t m_tiles_seg, int32_t n_tiles,
                       int32_t group_m, int32_t seg_span, int32_t seg_solo_first, int32_t bm, int32_t bn,
                       int32_t* out, int32_t n);
/* The launcher's rule for cutting the tiles of the last, partial wave into column pieces (mode as
 * FLUXB_TAIL_SPLIT: 0 never, 1 halves or quarters, 2 halves only), and the kernel's order of the resulting
 * work items: out[4t..4t+3] = (segment, tile row, first column, shift); an item is bn >> shift columns wide. */
int fluxb_tail_split(int64_t tiles, int64_t slots, int32_t mode, int32_t* split_from, int32_t* split_shift);
int fluxb_decode_work_items(int32_t num_seg, int32_t seg_first, int32_t m_tiles_seg, int32_t n_tiles,
                            int32_t group_m, int32_t seg_span, int32_t seg_solo_first, int32_t bm, int32_t bn,
                            int32_t split_from, int32_t split_shift, int32_t* out, int32_t n);
/* number of kernels libfluxb launched from this process so far */
uint64_t fluxb_launch_count(void);
/* zero the launcher's per-stream wave counters of the current device (synchronises the device);
 * needed only after a launch was cut short by a timed-out wait */
int fluxb_reset_wave_counters(void);

/* ---- Ulysses sequence-parallel projections (base.mode = FLUXB_GEMM_A2A | FLUXB_A2A_GEMM) ----
 * FLUXB_GEMM_A2A  (pre-attention): base.a = x [bs*local_seq, K], base.b = W [N, K] with
 *   N = heads*hd laid out as `groups` head groups (1: plain heads; 3: q | k | v); each 64-column
 *   piece of the product is stored by the GEMM epilogue straight into out[g][d], the buffer of
 *   the rank d that owns the head: layout 0 = [bs, heads_g/W, seq, hd], 1 = [bs, seq, heads_g/W, hd].
 *   The kernel returns when this rank's own buffers have received every rank's part.
 * FLUXB_A2A_GEMM  (post-attention): attn = this rank's attention output, layout 0 =
 *   [bs, heads/W, seq, hd], 1 = [bs, seq, heads/W, hd]; its slice for rank d's sequence range is
 *   pushed into slab `rank` of land[d], which keeps the source's layout ([W][heads/W][M][hd] for
 *   layout 0, [W][M][heads/W][hd] for layout 1, M = bs*local_seq) so that every piece moves as one
 *   contiguous run; base.d [M, N] = (the W slabs side by side along K) * W^T with the K loop gated
 *   slab by slab. base.a is ignored.
 * a2a_flags[r]: W*ceil(M/128)+W uint32 per rank in symmetric memory, zero at first use. */
typedef struct {
  fluxb_dense_args_t base;
  int32_t bs, local_seq, hd, groups;
  int32_t group_heads[3];    /* global head count of each group */
  int32_t layout;
  void* out[3][FLUXB_MAX_RANKS];
  const void* attn;
  void* land[FLUXB_MAX_RANKS];
  uint32_t* a2a_flags[FLUXB_MAX_RANKS];
  int32_t copy_local;        /* FLUXB_A2A_GEMM: 1 = land[rank] also receives this rank's own slice (the
                                whole GEMM input is then readable there); 0 = the own slice is read in
                                place from attn */
} fluxb_a2a_args_t;

int fluxb_ulysses_gemm(const fluxb_a2a_args_t* args);

/* ---- MoE layers (csrc/ops/moe.cu) ---------------------------------------------------------
 * Grouped GEMM over this rank's experts [e0, e0 + E_local) of E: D[rows_ep, N] = A_e * W_e^T.
 * Rows live in the expert-sorted order defined by splits [E] (device, int32 counts).
 *   gathered = 1 (layer 0): row r of that order is token gather_index[r] of a_tokens
 *     ([world * tokens_per_rank, K]); gather_index is written by this call from scatter_index
 *     ([n_entries] = tokens * topk, destination row of every (token, k)). With do_allgather the
 *     kernel also gathers the token shards: ag_src = this rank's shard, ag_land[r] = rank r's
 *     token matrix (a_tokens == ag_land[rank]).
 *   gathered = 0 (layer 1): A = a [a_rows, K] holds this rank's rows contiguously.
 * Epilogue: D = acc * scalar_scale[0] * expert_scale[e] * row_scale[row], any of them optional.
 * scratch: fluxb_moe_schedule_scratch_bytes(E, world) bytes, kept by the caller between this call
 * and fluxb_moe_combine (its header is the combine's `hdr`: scratch + fluxb_moe_hdr_offset). */
typedef struct {
  const int32_t* splits;
  const int32_t* scatter_index;
  int32_t* gather_index;
  int64_t n_entries;
  int32_t E, e0, E_local, topk;
  int32_t tokens_per_rank, gathered, do_allgather, in_dtype;
  int32_t N, K;
  const void* a;
  int64_t a_rows;
  const void* a_tokens;
  void* a_sorted;             /* optional [a_sorted_rows, K] scratch for the expert-sorted copy of the
                                 gathered rows (a_sorted_rows >= rows of this rank) */
  int64_t a_sorted_rows;
  const void* weights;        /* [E_local, N, K] */
  void* d;
  int64_t ldd;
  const float* expert_scale;
  const float* scalar_scale;
  const float* row_scale;
  void* scratch;
  int32_t rank, world;
  uint32_t epoch, reserved;
  uint64_t timeout_ns;
  fluxb_status_t* status;
  const void* ag_src;
  void* ag_land[FLUXB_MAX_RANKS];
  uint32_t* ag_flags[FLUXB_MAX_RANKS];
  uint32_t* start_ctr[FLUXB_MAX_RANKS];
  uint32_t* local_cnt;       /* local scratch, 1152 uint32, zero at first use: push-step counters, then
                                one arrival counter and one flag per (expert, source) sub-problem */
  void* stream;
  /* Layer 1 with the top-k combine and the reduce-scatter fused in (scatter != 0, gathered == 0,
   * every expert whole on one rank): the epilogue stores row r, times its scales, into slot
   * [token][k] of sc_stage[owner of the token] ([tokens_per_rank][topk][N] on every rank), and the
   * tail of the kernel adds the topk slots of each local token into sc_out [tokens_per_rank, N].
   * routing_idx [world * tokens_per_rank * topk] = sorted row of every (token, k); row_entry: int32
   * scratch of at least (rows of this rank) words; sc_flags[r]: world uint32 on rank r, zero at first
   * use; start_ctr and local_cnt (1 word) as above. d is not written. */
  int32_t scatter, reserved2;
  const int32_t* routing_idx;
  int32_t* row_entry;
  void* sc_stage[FLUXB_MAX_RANKS];
  uint32_t* sc_flags[FLUXB_MAX_RANKS];
  void* sc_out;
} fluxb_moe_gemm_args_t;

int64_t fluxb_moe_schedule_scratch_bytes(int E, int world);
int64_t fluxb_moe_hdr_offset(int E, int world);
int fluxb_moe_grouped_gemm(const fluxb_moe_gemm_args_t* args);

/* Top-k combine + reduce-scatter: out[tokens_per_rank, H] = sum over ranks and over the top-k
 * entries of each of this rank's tokens of y[routing_idx[token, k] - row_base]; rows that are not
 * on a rank contribute nothing there. stage[r]: [world][tokens_per_rank][H] on rank r. */
typedef struct {
  const void* y;
  const int32_t* hdr;         /* device: [0] row_base, [1] rows on this rank */
  const int32_t* routing_idx; /* [world * tokens_per_rank * topk] */
  int32_t topk, tokens_per_rank, H, dtype;
  int32_t rank, world;
  uint32_t epoch, reserved;
  uint64_t timeout_ns;
  fluxb_status_t* status;
  void* stage[FLUXB_MAX_RANKS];
  uint32_t* flags[FLUXB_MAX_RANKS];
  uint32_t* start_ctr[FLUXB_MAX_RANKS];
  uint32_t* local_cnt;
  void* out;
  void* stream;
} fluxb_moe_combine_args_t;

int fluxb_moe_combine(const fluxb_moe_combine_args_t* args);

/* ---- row exchange over peer memory (csrc/ops/a2a.cu) ----
 * Variable-split all-to-all of rows (broadcast = 0: rows [sum(in_splits[:d]), +in_splits[d]) of
 * `in` go to rank d) or all-gather (broadcast = 1: all rows_in rows go to every rank). In the
 * destination, rows are ordered by source rank. out[r], table[r] (world*world int32) and
 * flags[r] (2*world uint32) live in symmetric memory, zero at first use; out_splits [world] and
 * out_offsets [world + 1] (optional, local) receive the row counts / start rows per source. */
typedef struct {
  const void* in;
  const int32_t* in_splits;
  int32_t rows_in, broadcast;
  int64_t row_bytes;
  int32_t rank, world;
  uint32_t epoch;
  int32_t num_ctas;
  uint64_t timeout_ns;
  fluxb_status_t* status;
  void* out[FLUXB_MAX_RANKS];
  int32_t* table[FLUXB_MAX_RANKS];
  uint32_t* flags[FLUXB_MAX_RANKS];
  uint32_t* local_cnt;
  int32_t* out_splits;
  int32_t* out_offsets;
  int64_t out_capacity_rows;
  void* stream;
} fluxb_a2a_rows_args_t;

int fluxb_a2a_rows(const fluxb_a2a_rows_args_t* args);

/* ---- expert-parallel dispatch (csrc/ops/ep_dispatch.cu) ----
 * Row (token, k) of this rank's tokens x [tokens_local, row_bytes] goes to every rank of the expert
 * group that owns sorted row r = scatter_index[(token0 + token) * topk + k], at row r - (first row of
 * that group) of its receive buffer out[rank] ([capacity_rows][row_bytes], symmetric memory). Expert
 * group g = ranks [g * tp, (g + 1) * tp) owns experts [g * E_local, (g + 1) * E_local). The kernel
 * returns when the rows of every source have landed here. flags[r]: world uint32 on rank r;
 * local_cnt: 1 uint32; both zero at first use. out_rows (optional, local) receives the number of
 * rows this rank got. A row beyond capacity_rows is dropped and reported through `status` (code 13). */
typedef struct {
  const void* x;
  const int32_t* scatter_index;
  const int32_t* splits;
  int64_t token0;
  int32_t tokens_local, topk, E, E_local, tp, num_ctas;
  int64_t row_bytes, capacity_rows;
  int32_t rank, world;
  uint32_t epoch, reserved;
  uint64_t timeout_ns;
  fluxb_status_t* status;
  void* out[FLUXB_MAX_RANKS];
  uint32_t* flags[FLUXB_MAX_RANKS];
  uint32_t* start_ctr[FLUXB_MAX_RANKS];
  uint32_t* local_cnt;
  int32_t* out_rows;
  void* stream;
} fluxb_ep_dispatch_args_t;

int fluxb_ep_dispatch(const fluxb_ep_dispatch_args_t* args);
/* ---- strided exchange: stand-alone all-to-all (+ transpose) over peer memory ----
 * copy[d][g], g < ncopies: n0 x n1 x n2 items of vec_bytes contiguous bytes; item (i0, i1, i2) is
 * read at src + i0*ss0 + i1*ss1 + i2*ss2 (local memory) and written at dst + i0*ds0 + i1*ds1 + i2*ds2
 * (rank d's buffer). All addresses, strides and vec_bytes are multiples of 16 bytes. The kernel
 * returns when the data of every source has landed in this rank's buffers. flags[r]: world uint32 on
 * rank r, local_cnt: world uint32, both zero at first use. */
typedef struct {
  const void* src;
  void* dst;
  int32_t n0, n1, n2, vec_bytes;
  int64_t ss0, ss1, ss2, ds0, ds1, ds2;
} fluxb_strided_copy_t;

typedef struct {
  fluxb_strided_copy_t copy[FLUXB_MAX_RANKS][3];
  int32_t ncopies, num_ctas;
  int32_t rank, world;
  uint32_t epoch, reserved;
  uint64_t timeout_ns;
  fluxb_status_t* status;
  uint32_t* flags[FLUXB_MAX_RANKS];
  uint32_t* start_ctr[FLUXB_MAX_RANKS];
  uint32_t* local_cnt;
  void* stream;
} fluxb_strided_exchange_args_t;

int fluxb_strided_exchange(const fluxb_strided_exchange_args_t* args);
/* *flag = value with system-scope release, stream ordered (flag may be peer memory) */
int fluxb_set_flag(uint32_t* flag, uint32_t value, void* stream);

/* ---- symmetric memory (CUDA IPC). `handle` is 64 bytes of host memory. ---- */
int fluxb_symm_alloc(uint64_t bytes, void** ptr, void* handle);
int fluxb_symm_open(const void* handle, void** ptr);
int fluxb_symm_close(void* ptr);
int fluxb_symm_free(void* ptr);
/* can `dev` read and write `peer`'s memory directly? */
int fluxb_can_access_peer(int dev, int peer, int* out);

/* ---- cross-rank barrier on a stream. flags[r] points at rank r's flag block of `world`
 * uint32 (one word per source rank). Every rank passes the same, ever-growing `epoch`. ---- */
int fluxb_barrier_all(uint32_t* const* flags, int rank, int world, uint32_t epoch,
                      uint64_t timeout_ns, fluxb_status_t* status, void* stream);
/* Wait-only probe used by failure-detection tests: waits until *flag >= expected or the time
 * limit passes, then returns; the outcome is in `status`. */
int fluxb_wait_flag(const uint32_t* flag, uint32_t expected, uint64_t timeout_ns,
                    fluxb_status_t* status, void* stream);
/* Same, but waits for *flag == expected exactly (signals of the send/recv op). */
int fluxb_wait_flag_eq(const uint32_t* flag, uint32_t expected, uint64_t timeout_ns,
                       fluxb_status_t* status, void* stream);

/* ---- block-scaled fp8 quantisation (see csrc/aux/quantize.cu for layouts) ---- */
int fluxb_quantize_blockwise(const void* x, int64_t ldx, int in_dtype, void* q, void* qt,
                             float* scale_inv, float* scale_inv_t, int M, int K, int batch,
                             int square, float eps, int out_dtype, void* stream);

/* ---- small utilities (csrc/aux/utils.cu) ---- */
/* In-place fp32 -> bf16 compaction of data[0..n): results are packed at the front of the buffer.
 * flags: ceil(n/8192) uint32 of scratch, claim: one uint32; both zero at first use and owned by
 * the caller across calls; epoch grows by one per call. */
int fluxb_inplace_cast_fp32_to_bf16(float* data, int64_t n, uint32_t* flags, uint32_t* claim,
                                    uint32_t epoch, uint64_t timeout_ns, fluxb_status_t* status,
                                    void* stream);
/* out[t, :] = sum over j < cnt of in[row(t, j), :] in fp32, bf16 / fp16 rows of `cols` elements
 * (a multiple of 8): row(t, j) = idx[t * cnt + j], or j * slab_rows + t when idx is null. */
int fluxb_rows_sum(const void* in, const int32_t* idx, void* out, int64_t rows_out, int cols, int cnt,
                   int64_t slab_rows, int dtype, void* stream);
int fluxb_bitwise_check(const void* a, const void* b, int64_t nbytes,
                        unsigned long long* mismatches, void* stream);
int fluxb_uniform_fill(void* out, int64_t n, int dtype, uint64_t seed, float lo, float hi,
                       void* stream);
int fluxb_copy_bytes(void* dst, const void* src, int64_t nbytes, void* stream);
/* Stable counting sort of flattened expert choices; see csrc/aux/utils.cu. */
int64_t fluxb_moe_index_scratch_elems(int64_t n, int E);
int fluxb_moe_index_build(const int32_t* experts, int64_t n, int E, int topk, int32_t* splits,
                          int32_t* offsets, int32_t* scatter_index, int32_t* gather_index,
                          int32_t* topk_index, int32_t* scratch, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* FLUXB_H_ */
