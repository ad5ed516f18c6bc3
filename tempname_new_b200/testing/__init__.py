"""Test-support library (reference: ``python/flux/testing``): distributed set-up, data
generation, MoE gating tensors, PyTorch statements of every fused op, and a B200 roofline model."""
from .utils import (DTYPE_TOLERANCE, NNODES, TP_GROUP, bitwise_eq, generate_data, init_seed,  # noqa: F401
                    initialize_distributed, run_perf, split_torch_process_group)
from .moe_utils import (calc_gather_index_stable, calc_scatter_index_stable, gate_func,  # noqa: F401
                        gen_moe_gating_args, is_gather_index_stable, moe_gating_args)
from .perf_model import (estimate_fused_sol_time_ms, estimate_gemm_sol_time_ms, get_dram_gbps,  # noqa: F401
                         get_nvlink_gbps, get_tflops, roofline_fraction)
from ..ops.ulysses import (post_attn_a2a_torch as torch_post_attn_all_to_all_transpose,  # noqa: F401
                           pre_attn_a2a_torch as torch_pre_attn_all_to_all_transpose,
                           pre_attn_qkv_pack_a2a_torch as torch_pre_attn_qkv_pack_a2a)
from ..ops.moe import moe_layer0_torch, moe_layer1_partial_torch  # noqa: F401
from ..ops.blockscale_gemm import blockscale_gemm_torch  # noqa: F401
from .perf_log import PerfResult, log_perf  # noqa: F401
