"""Process launch and NCCL communication for data-parallel training
(mytorch/distributed/launch.py and the cupyx NCCLBackend use in mytorch/accelerate.py)."""
from .comm import NCCLBackend, exchange_unique_id, plan_buckets

__all__ = ["NCCLBackend", "exchange_unique_id", "plan_buckets"]
