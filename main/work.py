"""Drop-in path of the reference's ``main.work`` module."""
from fsdp_comm_opt_b200.parallel.work import AggregatedWork

__all__ = ["AggregatedWork"]
