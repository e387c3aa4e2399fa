"""orbitssm_b200: the B200 (sm_100a) ``backend="cuda"`` of the SSD-MIMO layer hot path.

Host side mirrors the reference's config + execution interface (`SSDMimoConfig`, `Execution`, `SSDMimoSSM`,
`State`); the arithmetic between the two projection GEMMs runs in hand-written CUDA behind the C-ABI library
declared in ``include/orbit_b200.h``.
"""
from .config import Execution, SSDMimoConfig, mamba2_config
from .model import BlockStack, ResidualBlock
from .ssd_mimo import SSDMimoSSM
from .state import State

__all__ = ["BlockStack", "ResidualBlock", "Execution", "SSDMimoConfig", "SSDMimoSSM", "State", "mamba2_config"]
