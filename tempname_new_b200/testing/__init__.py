"""Test-support library (reference: ``python/flux/testing``): distributed set-up, data
generation, MoE gating tensors, PyTorch statements of every fused op, and a B200 roofline model."""
from .utils import (DTYPE_TOLERANCE, NNODES, TP_GROUP, all_gather_into_tensor_with_fp8, bitwise_eq,  # noqa: F401
                    clone_with_fp8, empty_non_determinisitc, generate_data, get_global_args, init_local_groups,
                    init_seed, initialize_distributed, is_local_tp_group_initialized, matmul_int8,
                    nvshmem_split_team_2d, ones_with_fp8, rand_with_fp8, run_perf, set_global_args,
                    split_torch_process_group, zeros_with_fp8)
from .moe_utils import (calc_gather_index, calc_gather_index_stable, calc_scatter_index_stable,  # noqa: F401
                        calc_scatter_index_stable_sync, gate_func, gen_moe_gating_args, is_gather_index_stable,
                        moe_gather_rs_forward_torch, moe_gating_args)
from .moe_ag_scatter_utils import MoeAgScatterWithTorch, MoeMlp1Ctx  # noqa: F401
from .perf_model import (estimate_fused_sol_time_ms, estimate_gemm_sol_time_ms, get_clock_rate_in_khz,  # noqa: F401
                         get_device_multi_processor_count, get_device_property, get_device_shared_memory_size,
                         get_dram_gbps, get_dram_gbps_by_device_name, get_full_tflops_approx,
                         get_max_simd_tflops, get_max_tensorcore_tflops, get_nvlink_gbps, get_simd_tflops,
                         get_tensorcore_tflops, get_tflops, get_tflops_approx, is_fp8_dtype, nvsmi,
                         print_gemm_sol_time, print_grouped_gemm_sol_time_ms, roofline_fraction)
from ..ops.ulysses import (post_attn_a2a_torch as torch_post_attn_all_to_all_transpose,  # noqa: F401
                           pre_attn_a2a_torch as torch_pre_attn_all_to_all_transpose,
                           pre_attn_qkv_pack_a2a_torch as torch_pre_attn_qkv_pack_a2a)
from ..ops.moe import moe_layer0_torch, moe_layer1_partial_torch  # noqa: F401
from ..ops.blockscale_gemm import blockscale_gemm_torch  # noqa: F401
from .perf_log import (PerfResult, log_perf, log_perf_rds, log_perf_stdout, query,  # noqa: F401
                       should_log_to_rds, upload_to_rds)
