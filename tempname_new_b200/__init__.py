"""B200-native compute/communication overlap kernel library.

The public names follow the reference's ``flux`` package (``python/flux/cpp_mod.py``): code
written as ``import flux`` runs with ``import tempname_new_b200 as flux`` (or ``import fluxb as
flux``).
"""
__version__ = "0.1.0"

from . import _native  # noqa: F401
from .ops.options import (A2ARingMode, AGRingMode, AllGatherOption, AllToAllOption,  # noqa: F401
                          PreAttnAllToAllCommOp, ReduceScatterOption, RingMode,
                          get_default_a2a_ring_mode, get_default_ag_ring_mode,
                          get_default_rs_ring_mode)
from .parallel.symm import (FluxTimeoutError, GroupBarrier, SymmBuffer, create_tensor, create_tensor_list,  # noqa: F401
                            flux_create_shm_tensor_list,
                            init_flux_shm)
from .parallel.dist_env import DistEnvTP, DistEnvTPWithEP, MoeArguments  # noqa: F401
from .ops.gemm_only import GemmOnly  # noqa: F401
from .ops._dense import KernelTimeline  # noqa: F401
from .ops.gemm_rs import (GemmRS, SegmentInfo, calc_gemm_rs_threadblock_segments_info,  # noqa: F401
                          get_gemm_rs_threadblock_segments_info)
from .ops.ag_gemm import AGKernel  # noqa: F401
from .ops.quantization import Quantization  # noqa: F401
from .ops.misc import (InplaceCast, bitwise_check, calc_scatter_index, inplace_cast_fp32_to_bf16,  # noqa: F401
                       moe_index_build, uniform_initialize)
from .ops.blockscale_gemm import BlockScaleGemm, blockscale_gemm_torch  # noqa: F401
from .ops.ulysses import AllToAllTransposeGemm, GemmAllToAllTranspose  # noqa: F401
from .ops.moe import (GemmGroupedV2, GemmGroupedV2AGScatterOp, GemmGroupedV2GatherRSOp, GemmGroupedV3,  # noqa: F401
                      GemmGroupedV3AGScatter, GemmGroupedV3GatherRS, calc_moe_triton_blocked_gather_a,
                      prepare_moe_ag_scatter_args, topk_scatter_reduce)
from .utils.util import (bench_func, get_arch, get_torch_prof_ctx, group_profile, is_fp8_dtype,  # noqa: F401
                         torch_allclose, with_torch_deterministic)
from .utils import util  # noqa: F401
from .utils import dist_utils  # noqa: F401
from .utils.dist_utils import exec_in_rank_order, get_dist_env  # noqa: F401
from .tuning.profiling import ProfilingContext, TuningRecord  # noqa: F401
from .parallel.layers import ColumnParallelLinear, RowParallelLinear, patch_megatron_linears  # noqa: F401
from . import models, ops, parallel, testing, tuning, utils  # noqa: F401
from .ops.coll import All2AllOp, All2AllSingle, AllGatherOp, AsyncSendRecv  # noqa: F401
from .ops.ep_dispatch import (AGKernelInterNode, AGKernelXNode, All2AllInference, DisScatterBackward,  # noqa: F401
                              DisScatterForward, GemmRS_multinode, GemmRSInterNode, GemmRSTaco,
                              GemmRSTacoDoubleBuffered, TopkReduceScatterOp, TransportOp,
                              bsr_reduce,
                              load_tuning_record, pad_m_to_TPxTile)
from .parallel.teams import (TEAM_INVALID, TEAM_WORLD, TeamConfig, _nvshmem_team_destroy,  # noqa: F401,E402
                             _nvshmem_team_get_config, _nvshmem_team_my_pe, _nvshmem_team_npes,
                             _nvshmem_team_npes as _nvshmem_team_n_pes,
                             _nvshmem_team_split_2d, _nvshmem_team_split_strided, _nvshmem_team_translate_pe,
                             team_group)
from .utils.dist_utils import (DistEnv, get_inter_node_ag_group, get_inter_node_rs_group,  # noqa: F401,E402
                               get_intra_node_ag_group, get_intra_node_pg_group, initialize_inter_node_rs_group)

