"""The reference's import paths and signatures keep working: ``main.{comm,zipccl_comm,work}``, the
ten functions of ``zipccl.hopper_fastzip2`` and their stub file."""
import ast
import inspect
import os

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))

TEN = ["compress_8", "decompress_8", "compress_8_padded", "decompress_8_padded", "decompress_8_unpad",
       "compress_split_store", "decompress_split_store", "decompress_split_store_unpad",
       "decompress_split_store_unpad_v", "compress_split_store_pad"]

def test_reference_module_paths_and_constructor_signatures():
    from main.comm import QuantizedAllGather
    from main.work import AggregatedWork
    from main.zipccl_comm import ZipCCLAllGather, ZipCCLReduceScatter

    # reference: main/zipccl_comm.py:11 (base_exponent=122, base_update_interval=16), main/comm.py:9
    sig = inspect.signature(ZipCCLAllGather.__init__)
    assert sig.parameters["base_exponent"].default == 122
    assert sig.parameters["base_update_interval"].default == 16
    assert inspect.signature(QuantizedAllGather.__init__).parameters["min_quantize_numel"].default == 0
    for hook in (ZipCCLAllGather(), QuantizedAllGather()):
        assert callable(hook) and callable(hook.allocate)
        assert list(inspect.signature(hook.__call__).parameters)[:3] == ["output_tensor", "input_tensor", "group"]
    rs = ZipCCLReduceScatter()
    assert list(inspect.signature(rs.__call__).parameters)[:4] == ["output_tensor", "input_tensor", "group", "op"]
    import torch.distributed as dist

    assert issubclass(AggregatedWork, dist.Work)


def test_extension_module_exports_match_the_stub():
    from zipccl import hopper_fastzip2 as hz

    with open(os.path.join(ROOT, "zipccl", "hopper_fastzip2.pyi")) as fp:
        stub = ast.parse(fp.read())
    stub_fns = {n.name: n for n in stub.body if isinstance(n, ast.FunctionDef)}
    assert len(stub_fns) == 10
    for name in TEN:
        assert name in stub_fns, name
    for name, node in stub_fns.items():
        fn = getattr(hz, name)
        assert callable(fn), name
        want = [a.arg for a in node.args.args]
        got = list(inspect.signature(fn).parameters)
        assert got[:len(want)] == want, (name, got, want)
