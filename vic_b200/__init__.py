"""vic_b200: the vib3 INT4 MoE decode hot path (paged INT4 expert GEMV, fused SwiGLU chain,
router top-k) as hand-written sm_100a CUDA behind the reference's launcher C ABI."""
from .core_types import KIMI, MIXTRAL, MoeShape, PageId  # noqa: F401
from .lib import Vib3Error  # noqa: F401
