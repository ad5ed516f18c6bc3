from .symm import (FluxTimeoutError, GroupBarrier, SymmBuffer, create_tensor_list,  # noqa: F401
                   init_flux_shm)
from .dist_env import DistEnvTP, DistEnvTPWithEP, MoeArguments  # noqa: F401
