// Host side of the dense GEMM family (GemmOnly, AG+GEMM, GEMM+RS): argument checks, tensor
// maps, tile-shape choice and the launch of dense_gemm_kernel.
#include "../include/fluxb.h"
#include "../runtime/host_common.h"
#include "../sm100/gemm_dense.cuh"

#include <atomic>

namespace fluxb {

std::atomic<uint64_t> g_launches{0};

namespace {

template <class Cfg>
int launch_dense(const DenseGemmParams& p, int grid, cudaStream_t stream) {
  constexpr int kThreads = Cfg::THREADS;
  static bool configured[64] = {false};
  int dev = 0;
  FLUXB_CUDA_OK(cudaGetDevice(&dev));
  if (dev >= 64 || !configured[dev]) {
    FLUXB_CUDA_OK(cudaFuncSetAttribute(dense_gemm_kernel<Cfg>,
                                       cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg::SMEM_BYTES));
    if (dev < 64) configured[dev] = true;
  }
  if constexpr (Cfg::CG == 1) {
    dense_gemm_kernel<Cfg><<<grid, kThreads, Cfg::SMEM_BYTES, stream>>>(p);
  } else {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(grid, 1, 1);
    cfg.blockDim = dim3(kThreads, 1, 1);
    cfg.dynamicSmemBytes = Cfg::SMEM_BYTES;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = 2;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
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

extern "C" int fluxb_dense_gemm(const fluxb_dense_args_t* a) {
  FLUXB_REQUIRE(a != nullptr, "null args");
  FLUXB_REQUIRE(a->M > 0 && a->N > 0 && a->K > 0, "empty problem");
  FLUXB_REQUIRE(a->in_dtype == FLUXB_BF16 || a->in_dtype == FLUXB_FP8_E4M3 ||
                    a->in_dtype == FLUXB_FP16 || a->in_dtype == FLUXB_FP8_E5M2,
                "input dtype");
  FLUXB_REQUIRE(a->out_dtype == FLUXB_BF16 || a->out_dtype == FLUXB_FP16, "output dtype");
  FLUXB_REQUIRE(a->world >= 1 && a->world <= FLUXB_MAX_RANKS, "world size 1..8");
  FLUXB_REQUIRE(a->rank >= 0 && a->rank < a->world, "rank");
  const bool in16 = a->in_dtype == FLUXB_BF16 || a->in_dtype == FLUXB_FP16;
  const int elt = in16 ? 2 : 1;
  const bool multi = a->world > 1 && a->mode != FLUXB_PLAIN;
  FLUXB_REQUIRE((a->K * elt) % 16 == 0, "K row bytes must be a multiple of 16");
  FLUXB_REQUIRE(a->N % 8 == 0, "N must be a multiple of 8");
  if (multi) FLUXB_REQUIRE(a->M % a->world == 0, "M must divide evenly over ranks");

  DenseGemmParams p;
  memset(&p, 0, sizeof(p));
  p.M = a->M;
  p.N = a->N;
  p.K = a->K;
  p.rank = a->rank;
  p.world = a->world;
  p.mode = multi ? a->mode : kModePlain;
  p.num_seg = multi ? a->world : 1;
  p.seg_rows = a->M / p.num_seg;
  p.epoch = a->epoch;
  p.timeout_ns = a->timeout_ns ? a->timeout_ns : 2000000000ull;
  p.status = reinterpret_cast<Status*>(a->status);
  p.bias = a->bias;
  p.bias_row_stride = a->bias_row_stride;
  p.scale_a = a->scale_a;
  p.scale_b = a->scale_b;
  p.sa = a->sa;
  p.sb = a->sb;
  p.ab_fmt = (a->in_dtype == FLUXB_BF16 || a->in_dtype == FLUXB_FP8_E5M2) ? 1 : 0;
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
    FLUXB_REQUIRE((a->M / (multi ? a->world : 1)) % 128 == 0, "block-scaled GEMM needs rows per rank in multiples of 128");
    cg = 1;
    bn = 128;
  } else if (multi && a->mode == FLUXB_ALLGATHER) {
    // the all-gather variants exist for CTA pairs on 256-wide tiles and single CTAs on 128-wide
    if (cg == 2 && a->M / a->world >= 256) bn = 256;
    else { cg = 1; bn = 128; }
  }
  const int bm = 128 * cg;
  const int bk = 128 / elt;
  const CUtensorMapDataType in_dt =
      in16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_UINT8;
  const CUtensorMapDataType out_dt = CU_TENSOR_MAP_DATA_TYPE_BFLOAT16;  // any 16-bit type moves alike

  int rc;
  // ---- A
  {
    const uint64_t rows = (p.mode == kModeAllGather) ? p.seg_rows : a->M;
    uint64_t dims[2] = {static_cast<uint64_t>(a->K), rows};
    uint64_t str[1] = {static_cast<uint64_t>(a->lda) * elt};
    uint32_t box[2] = {static_cast<uint32_t>(bk), 128};
    if ((rc = encode_tmap(&p.tm_a, in_dt, 2, a->a, dims, str, box, Swz::B128))) return rc;
  }
  if (p.mode == kModeAllGather) {
    FLUXB_REQUIRE(a->ag_land[a->rank] != nullptr, "all-gather landing buffer missing");
    uint64_t dims[2] = {static_cast<uint64_t>(a->K), static_cast<uint64_t>(a->M)};
    uint64_t str[1] = {static_cast<uint64_t>(a->K) * elt};
    uint32_t box[2] = {static_cast<uint32_t>(bk), 128};
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
  // ---- B
  {
    uint64_t dims[2] = {static_cast<uint64_t>(a->K), static_cast<uint64_t>(a->N)};
    uint64_t str[1] = {static_cast<uint64_t>(a->ldb) * elt};
    uint32_t box[2] = {static_cast<uint32_t>(bk), static_cast<uint32_t>(bn / cg)};
    if ((rc = encode_tmap(&p.tm_b, in_dt, 2, a->b, dims, str, box, Swz::B128))) return rc;
  }
  // ---- D
  {
    uint32_t box[3] = {64, 32, 1};
    if (p.mode == kModeReduceScatter) {
      FLUXB_REQUIRE(a->rs_out && a->rs_work, "reduce-scatter output / work counter missing");
      for (int r = 0; r < a->world; ++r) {
        FLUXB_REQUIRE(a->rs_stage[r] && a->rs_ctr[r], "reduce-scatter peer pointers missing");
        uint64_t dims[3] = {static_cast<uint64_t>(a->N), static_cast<uint64_t>(p.seg_rows),
                            static_cast<uint64_t>(a->world)};
        uint64_t str[2] = {static_cast<uint64_t>(a->N) * 2,
                           static_cast<uint64_t>(a->N) * 2 * p.seg_rows};
        if ((rc = encode_tmap(&p.tm_d[r], out_dt, 3, a->rs_stage[r], dims,
                              str, box, Swz::B128)))
          return rc;
        p.rs_ctr[r] = a->rs_ctr[r];
      }
      p.rs_stage = a->rs_stage[a->rank];
      p.rs_out = a->rs_out;
      p.rs_work = a->rs_work;
    } else {
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

  const int m_tiles_seg = (p.seg_rows + bm - 1) / bm;
  p.group_m = a->group_m > 0 ? a->group_m : 16 / cg;
  if (p.group_m > m_tiles_seg) p.group_m = m_tiles_seg;

  int sms = 0;
  if ((rc = device_sm_count(&sms))) return rc;
  if (a->num_sms > 0 && a->num_sms < sms) sms = a->num_sms;
  const int64_t tiles = static_cast<int64_t>(p.num_seg) * m_tiles_seg * ((a->N + bn - 1) / bn);
  int grid = sms;
  // every CTA of a multi-rank launch takes part in the flag protocol, so the grid stays full
  if (!multi && tiles * cg < grid) grid = static_cast<int>(tiles) * cg;
  if (cg == 2) grid &= ~1;

  cudaStream_t stream = reinterpret_cast<cudaStream_t>(a->stream);
  if (a->blockscale) {
    if (p.mode == kModeAllGather) return launch_dense<DenseCfg<128, 1, 4, 1, 32768, true>>(p, grid, stream);
    return launch_dense<DenseCfg<128, 1, 4, 1, 0, true>>(p, grid, stream);
  }
  if (p.mode == kModeAllGather) {
    // variants that carry the staging rings of the all-gather push
    if (cg == 2 && bn == 256) {
      if (in16) return launch_dense<DenseCfg<256, 0, 5, 2, 32768>>(p, grid, stream);
      return launch_dense<DenseCfg<256, 1, 5, 2, 32768>>(p, grid, stream);
    }
    FLUXB_REQUIRE(cg == 1 && bn == 128, "all-gather GEMM runs as CTA pairs on 256-wide tiles or single CTAs on 128-wide tiles");
    if (in16) return launch_dense<DenseCfg<128, 0, 5, 1, 32768>>(p, grid, stream);
    return launch_dense<DenseCfg<128, 1, 5, 1, 32768>>(p, grid, stream);
  }
  if (cg == 2) {
    if (in16) {
      if (bn == 256) return launch_dense<DenseCfg<256, 0, 6, 2>>(p, grid, stream);
      if (bn == 192) return launch_dense<DenseCfg<192, 0, 6, 2>>(p, grid, stream);
      return launch_dense<DenseCfg<128, 0, 8, 2>>(p, grid, stream);
    }
    if (bn == 256) return launch_dense<DenseCfg<256, 1, 6, 2>>(p, grid, stream);
    if (bn == 192) return launch_dense<DenseCfg<192, 1, 6, 2>>(p, grid, stream);
    return launch_dense<DenseCfg<128, 1, 8, 2>>(p, grid, stream);
  }
  if (in16) {
    if (bn == 256) return launch_dense<DenseCfg<256, 0, 4>>(p, grid, stream);
    if (bn == 192) return launch_dense<DenseCfg<192, 0, 4>>(p, grid, stream);
    return launch_dense<DenseCfg<128, 0, 6>>(p, grid, stream);
  } else {
    if (bn == 256) return launch_dense<DenseCfg<256, 1, 4>>(p, grid, stream);
    if (bn == 192) return launch_dense<DenseCfg<192, 1, 4>>(p, grid, stream);
    return launch_dense<DenseCfg<128, 1, 6>>(p, grid, stream);
  }
}
