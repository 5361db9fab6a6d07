"""Power retention on B200: the reference's `power_retention` / `power_retention_inference`
signatures on hand-written sm_100a kernels behind a C ABI (libpr_b200.so)."""
from .retention import power_retention, power_retention_inference  # noqa: F401
from .cache import RetentionCache  # noqa: F401
from .caller import prepare_qkvg, rotary_tables  # noqa: F401
from ._lib import PRError  # noqa: F401

__all__ = ["power_retention", "power_retention_inference", "RetentionCache", "prepare_qkvg", "rotary_tables", "PRError"]
