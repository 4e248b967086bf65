"""Dataset registry (``data_register`` of mindspeed_mm/fsdp/utils/register.py:61)."""
from ..models.registry import data_register  # noqa: F401
