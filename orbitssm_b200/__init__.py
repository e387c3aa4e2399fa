"""orbitssm_b200: the B200 (sm_100a) ``backend="cuda"`` of the SSD-MIMO and HybridMamba layer hot paths.

Host side mirrors the reference's config + execution interface (`SSDMimoConfig`, `HybridMambaConfig`, `Execution`,
`SSDMimoSSM`, `HybridMambaSSM`, `State`); the arithmetic between the two projection GEMMs runs in hand-written CUDA behind the C-ABI library
declared in ``include/orbit_b200.h``.
"""
from .config import Execution, HybridMambaConfig, SSDMimoConfig, mamba2_config
from .graphs import CaptureError, GraphedDecode, GraphedStep
from .hybrid_mamba import HybridMambaSSM
from .model import BlockStack, ResidualBlock
from .ops import check_device_status
from .ssd_mimo import SSDMimoSSM
from .state import State

__all__ = ["BlockStack", "ResidualBlock", "CaptureError", "Execution", "GraphedDecode", "GraphedStep", "HybridMambaConfig", "HybridMambaSSM", "SSDMimoConfig", "SSDMimoSSM",
           "State", "check_device_status", "mamba2_config"]
