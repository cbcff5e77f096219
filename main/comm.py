"""Drop-in path of the reference's ``main.comm`` module."""
from fsdp_comm_opt_b200.parallel.hooks import QuantizedAllGather

__all__ = ["QuantizedAllGather"]
