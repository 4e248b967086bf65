"""Plan records (stand-in: the reference only uses ``EPPlanConfig`` as a type annotation)."""
from dataclasses import dataclass, field
from typing import List, Optional


@dataclass
class EPPlanConfig:
    apply_modules: List[str] = field(default_factory=list)
    use_npu_fused_ops: bool = False
    dispatcher: str = "alltoall"
    apply_efsdp_modules: List[str] = field(default_factory=list)
    _gradient_divide_factor: Optional[float] = None
