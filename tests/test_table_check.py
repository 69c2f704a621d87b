"""Debug mode of the persistent kernels (per-chunk validation of the segment table)."""
import os

import pytest
import torch
import torch.nn as nn

from apexw_b200 import ApexW, _native
from apexw_b200.utils import table_check as tc


def test_switch_and_error_text_on_cpu():
    assert not tc.enabled()
    with tc.table_checks():
        assert tc.enabled()
        with tc.table_checks(False):
            assert not tc.enabled()
        assert tc.enabled()
    assert not tc.enabled() and tc.ENV not in os.environ
    err = tc.TableFaultError({"state": dict(code=7, segment=3, chunk=41, skipped=2),
                              "zero": dict(code=0, segment=0, chunk=0, skipped=0)})
    assert "block size" in str(err) and "segment 3" in str(err) and "zero" not in str(err)
    assert err.report["state"]["chunk"] == 41
    if not torch.cuda.is_available():
        assert tc.report() is None
        tc.check()          # nothing to read: no error


@pytest.mark.gpu
def test_device_checker_classifies_hand_made_records():
    """The checker runs on 15 records that are wrong in exactly one way (or in none); no record is dereferenced."""
    assert _native.available(), _native.load_error()
    assert tc.selftest() == 0x7FFF


@pytest.mark.gpu
@pytest.mark.parametrize("prec,kw", [("compact", {}), ("8bit", {}), ("8bit", dict(int4_m=False)), ("compact", dict(cautious=True)),
                                     ("compact", dict(amsgrad=True))])
def test_checks_pass_on_real_plans_and_change_nothing(prec, kw):
    def run(on):
        torch.manual_seed(0)
        ps = [nn.Parameter(torch.randn(s, device="cuda").bfloat16() * 0.05)
              for s in [(256, 128), (70,), (3, 1000), (2048 * 3 + 8,), (16384 + 4,), (1,)]]
        opt = ApexW(ps, lr=1e-2, precision=prec, weight_decay=0.1, seed=3, **kw)
        with tc.table_checks(on):
            for s in range(2):
                g = torch.Generator(device="cuda").manual_seed(s)
                for p in ps:
                    p.grad = (torch.randn(p.shape, device="cuda", generator=g) * 1e-3).bfloat16()
                opt.step()              # raises TableFaultError if a kernel rejected a record
        assert opt._native_launches > 0
        return [p.detach().clone() for p in ps]

    tc.report(clear=True)
    plain, checked = run(False), run(True)
    for a, b in zip(plain, checked):
        assert torch.equal(a, b)
    r = tc.report()
    assert r is not None and all(m["code"] == 0 and m["skipped"] == 0 for m in r.values())


@pytest.mark.gpu
@pytest.mark.parametrize("prec", ["compact", "8bit"])
def test_checks_pass_in_the_peer_kernel_at_world_one(prec):
    from apexw_b200.parallel.zero import ApexWZeRO
    dev = torch.device("cuda")

    def run(on):
        g0 = torch.Generator().manual_seed(0)
        ps = [nn.Parameter((torch.randn(s, generator=g0) * 0.05).bfloat16().to(dev))
              for s in [(512, 256)] * 4 + [(256,), (1000, 40), (70,), (3, 5)]]
        opt = ApexWZeRO(ps, lr=1e-2, precision=prec, betas=(0.9, 0.99), seed=3)
        assert opt._fused
        with tc.table_checks(on):
            for s in range(2):
                g = torch.Generator().manual_seed(100 + s)
                for p in ps:
                    p.grad.copy_((torch.randn(p.shape, generator=g) * 1e-3).bfloat16().to(dev))
                opt.step()
        opt.check_status()
        return [p.detach().clone() for p in ps]

    tc.report(clear=True)
    plain, checked = run(False), run(True)
    for a, b in zip(plain, checked):
        assert torch.equal(a, b)
    r = tc.report()
    assert r["zero"]["code"] == 0 and r["zero"]["skipped"] == 0
