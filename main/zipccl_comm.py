"""Drop-in path of the reference's ``main.zipccl_comm`` module (plus the reduce-scatter hook)."""
from fsdp_comm_opt_b200.parallel.hooks import ZipCCLAllGather, ZipCCLReduceScatter

__all__ = ["ZipCCLAllGather", "ZipCCLReduceScatter"]
