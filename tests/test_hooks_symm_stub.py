"""The hooks' fused-transport call path, run on CPU against a stand-in for the symmetric-memory
channel: which wire mode reaches the kernels for every ``wire`` setting, and that the per-call
attributes (urgent, exclusive, residual) are passed on.  The real channel needs NVLink peers; this
catches what would otherwise only fail on a multi-GPU box."""
import pytest
import torch
import torch.distributed as dist

import fsdp_comm_opt_b200.parallel.hooks as H
import fsdp_comm_opt_b200.parallel.symm_impl as S


class _FakeChannel:
    def __init__(self, log):
        self.log = log

    def all_gather(self, out, x, **kw):
        self.log.append(("ag", kw))

    def reduce_scatter(self, out, x, **kw):
        self.log.append(("rs", kw))


@pytest.fixture
def fused(monkeypatch):
    log = []
    monkeypatch.setattr(S, "channel_for", lambda group, device, kind: _FakeChannel(log))
    monkeypatch.setattr(H, "_resolve_transport", lambda transport, device, group: "symm")
    monkeypatch.setattr(dist, "get_world_size", lambda group=None: 2)
    return log


@pytest.mark.parametrize("wire,expected", [("auto", "nibble"), ("nibble", "nibble"), ("compressed", "compressed"),
                                           ("verbatim", "verbatim")])
def test_wire_mode_that_reaches_the_fused_kernels(fused, wire, expected):
    x, out = torch.zeros(8, dtype=torch.bfloat16), torch.zeros(16, dtype=torch.bfloat16)
    ag = H.ZipCCLAllGather(wire=wire)
    ag.urgent, ag.exclusive = False, True
    ag(out, x, None, async_op=True)
    rs = H.ZipCCLReduceScatter(wire=wire)
    rs(torch.zeros(4), torch.zeros(8), None, dist.ReduceOp.AVG)
    (k1, a), (k2, r) = fused
    assert (k1, k2) == ("ag", "rs")
    assert a["wire"] == r["wire"] == expected and S._WIRE_CODE[expected] in (0, 1, 2)
    assert a["urgent"] is False and a["exclusive"] is True and a["async_op"] is True and a["mode"] == "zip"
    assert r["scale"] == 0.5 and r["residual"] is not None and r["residual"].dtype == torch.bfloat16   # fp32 rows: error feedback
    assert ag.last_transport == rs.last_transport == "symm"


def test_unknown_wire_is_refused():
    with pytest.raises(ValueError):
        H.ZipCCLReduceScatter(wire="gzip")
