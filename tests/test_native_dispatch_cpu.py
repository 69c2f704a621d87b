"""Host-side dispatch of the fused kernels, exercised without a GPU.

``torch.Tensor.is_cuda`` is patched to True and the native module is replaced by a recorder, so ``ApexW.step`` takes
the path it takes on a GPU: eligibility, kernel class, which state tensors travel in which slot of the launch plan,
step flags, device-resident scalars, launch bookkeeping.  The arithmetic itself is covered by the GPU tests.
"""
from unittest import mock

import pytest
import torch
import torch.nn as nn

from apexw_b200 import ApexW, _native
from apexw_b200.optim import apexw as impl


class _Plan:
    made = []

    def __init__(self, kernel_class, params, m, v, m_scale, v_scale, flags, salts, block_sizes, offsets, device_index, decay_ranges):
        self.kernel_class = kernel_class
        self.args = dict(params=params, m=m, v=v, m_scale=m_scale, v_scale=v_scale, flags=flags, salts=salts,
                         block_sizes=block_sizes, decay_ranges=decay_ranges)
        self.steps, self.dyn, self.vlog4 = [], None, None
        _Plan.made.append(self)

    def step(self, grads, beta1, beta2, step_size, eps_scaled, eps, eps_quad, eps_quad_scaled, decay_factor, inv_scale,
             gain_hi, gain_lo, step_key, flags, found_inf, grad_scale, ctas_per_sm, beta3=0.0, slow_ratio=0.0, lr=0.0):
        assert len(grads) == len(self.args["params"])
        self.steps.append(dict(flags=flags, step_size=step_size, beta3=beta3, slow_ratio=slow_ratio, lr=lr, step_key=step_key,
                               decay_factor=decay_factor))

    def set_device_scalars(self, step_dev, lr_dev, step_host, lr_host, alpha, weight_decay, seed):
        self.dyn = dict(step_dev=step_dev, lr_dev=lr_dev, step_host=step_host, lr_host=lr_host, weight_decay=weight_decay)

    def clear_device_scalars(self):
        self.dyn = None

    def set_v_scale_log4(self, ks):
        self.vlog4 = list(ks)


class _FakeNative:
    StatePlan = _Plan


SHAPES = [(1024, 512)] + [(256, 256)] * 5 + [(128,), (64, 40), (70,)]     # eight or more tensors: shared variances are on


def _run(steps=2, dtype=torch.bfloat16, **kw):
    _Plan.made = []
    ps = [nn.Parameter(torch.randn(s).to(dtype)) for s in SHAPES]
    before = _native.launch_count()
    with mock.patch.object(torch.Tensor, "is_cuda", new_callable=mock.PropertyMock, return_value=True), \
            mock.patch.object(_native, "require", return_value=_FakeNative), \
            mock.patch.object(_native, "disabled_by_env", return_value=False):
        opt = ApexW(ps, weight_decay=0.1, seed=5, **kw)
        for s in range(steps):
            for p in ps:
                p.grad = torch.randn_like(p) * 1e-3
            opt.step()
    plan = opt._execution_plans[id(opt.param_groups[0])]
    return opt, plan, _native.launch_count() - before


def _classes(plan):
    return sorted(sp.kernel_class for sp, _ in plan.classes)


def test_default_layouts_pick_their_classes():
    opt, plan, n = _run(lr=1e-3, precision="compact")
    assert not plan.fallback and set(_classes(plan)) <= {impl._KC_DENSE, impl._KC_DENSE_QUAD}
    assert impl._KC_DENSE_QUAD in _classes(plan)
    assert n == 2 * len(plan.classes) and opt._native_launches == n         # one kernel per class and step
    opt, plan, _ = _run(lr=1e-3, precision="8bit")
    assert not plan.fallback and impl._KC_NF4_QUAD in _classes(plan)
    for sp, ps in plan.classes:
        if sp.kernel_class >= impl._KC_INT8:
            assert len(sp.args["m_scale"]) == len(ps) == len(sp.args["v_scale"])
    # one launch plan survives the steps: built once
    assert len(_Plan.made) == len(plan.classes)


def test_lion_amsgrad_ademamix_carry_their_extra_state_in_the_scale_slots():
    opt, plan, _ = _run(lr=1e-4, precision="compact", lion=True, betas=(0.9, 0.99))
    assert not plan.fallback and _classes(plan) == [impl._KC_DENSE]
    sp = plan.classes[0][0]
    assert all(a is b for a, b in zip(sp.args["m"], sp.args["v"]))          # no second moment: the slot repeats m
    assert sp.steps[-1]["flags"] & impl._STEP_LION and sp.steps[-1]["lr"] == pytest.approx(1e-4)

    opt, plan, _ = _run(lr=1e-3, precision="compact", amsgrad=True, betas=(0.9, 0.999, 0.9999), alpha=4.0)
    assert not plan.fallback and _classes(plan) == [impl._KC_DENSE]
    sp, ps = plan.classes[0]
    assert [t.data_ptr() for t in sp.args["m_scale"]] == [opt.state[p]["exp_avg_slow"].data_ptr() for p in ps]
    assert [t.data_ptr() for t in sp.args["v_scale"]] == [opt.state[p]["max_exp_avg_sq"].data_ptr() for p in ps]
    last = sp.steps[-1]
    assert last["flags"] & impl._STEP_SLOW and last["flags"] & impl._STEP_AMSGRAD and not last["flags"] & impl._STEP_LION
    assert last["beta3"] == pytest.approx(0.9999) and last["slow_ratio"] > 0


def test_dense_cautious_counts_two_kernels_per_launch():
    opt, plan, n = _run(lr=1e-3, precision="compact", cautious=True)
    assert not plan.fallback
    assert all(sp.steps[-1]["flags"] & impl._STEP_CAUTIOUS for sp, _ in plan.classes)
    assert n == 2 * 2 * len(plan.classes)              # counting pass + update, per class and step
    _, plan, _ = _run(lr=1e-3, precision="compact", cautious=True, nesterov=True)
    assert len(plan.fallback) == len(SHAPES)            # this pair stays with the torch engine


def test_ultra_factored_and_int8_lion_classes():
    opt, plan, _ = _run(lr=1e-3, precision="ultra")
    assert not plan.fallback and impl._KC_ULTRA in _classes(plan)
    for sp, ps in plan.classes:
        if sp.kernel_class == impl._KC_ULTRA:
            assert len(sp.args["m_scale"]) == len(ps) and sp.args["v_scale"] == []
            assert all(b in (256, 2048) for b in sp.args["block_sizes"])

    opt, plan, n = _run(lr=1e-3, precision="8bit", factored_v=True)
    assert not plan.fallback and impl._KC_FACTORED in _classes(plan)
    for sp, ps in plan.classes:
        if sp.kernel_class == impl._KC_FACTORED:
            assert [t.numel() for t in sp.args["v"]] == [p.shape[0] for p in ps]            # row statistics
            assert [t.numel() for t in sp.args["v_scale"]] == [p.numel() // p.shape[0] for p in ps]
            assert len(sp.args["m_scale"]) == len(ps)                                       # int8 first moment
    others = sum(1 for sp, _ in plan.classes if sp.kernel_class != impl._KC_FACTORED)
    assert n == 2 * (3 + others)                        # statistics + finish + update for the factored class

    opt, plan, _ = _run(lr=1e-4, precision="8bit", lion=True, betas=(0.9, 0.99))
    assert not plan.fallback and _classes(plan) == [impl._KC_LION8]
    assert opt.state[plan.classes[0][1][0]]["exp_avg"].dtype == torch.int8


def test_a_learning_rate_tensor_switches_the_plan_to_device_scalars_and_back():
    _Plan.made = []
    ps = [nn.Parameter(torch.randn(s).bfloat16()) for s in SHAPES]
    lr_t = torch.tensor(1e-3)
    with mock.patch.object(torch.Tensor, "is_cuda", new_callable=mock.PropertyMock, return_value=True), \
            mock.patch.object(_native, "require", return_value=_FakeNative), \
            mock.patch.object(_native, "disabled_by_env", return_value=False):
        opt = ApexW(ps, lr=lr_t, precision="compact", weight_decay=0.1)
        for p in ps:
            p.grad = torch.randn_like(p) * 1e-3
        opt.step()
        plan = opt._execution_plans[id(opt.param_groups[0])]
        assert not plan.fallback and plan.dynamic
        for sp, _ in plan.classes:
            # (under the patch the host-side step counter looks like a device tensor too; on a GPU only lr_dev is set)
            assert sp.dyn is not None and sp.dyn["lr_dev"] is not None and sp.dyn["lr_host"] == 0.0
            assert sp.dyn["step_host"] == 1.0 and sp.dyn["weight_decay"] == pytest.approx(0.1)
        opt.param_groups[0]["lr"] = 5e-4                # a plain number again: the plan is rebuilt without the mode
        for p in ps:
            p.grad = torch.randn_like(p) * 1e-3
        opt.step()
        plan2 = opt._execution_plans[id(opt.param_groups[0])]
        assert plan2 is not plan and all(sp.dyn is None for sp, _ in plan2.classes)


def test_plan_cache_keeps_sub_sets_and_evicts_the_least_recently_used(monkeypatch):
    monkeypatch.setattr(impl, "_MAX_CACHED_PLANS", 3)
    ps = [nn.Parameter(torch.randn(256, 256).bfloat16()) for _ in range(5)]
    with mock.patch.object(torch.Tensor, "is_cuda", new_callable=mock.PropertyMock, return_value=True), \
            mock.patch.object(_native, "require", return_value=_FakeNative), \
            mock.patch.object(_native, "disabled_by_env", return_value=False):
        opt = ApexW(ps, lr=1e-3, precision="compact")
        g = opt.param_groups[0]
        for p in ps:
            p.grad = torch.randn_like(p) * 1e-3
        ctx = opt._group_ctx()
        for p in ps:
            opt._init_state(p, g, ctx)
        keys = []
        for i in (0, 1, 2):
            opt._plan_for(g, [ps[i]])
            keys.append((id(g), (id(ps[i]),)))
        assert list(opt._execution_plans) == keys
        first = opt._execution_plans[keys[0]]
        assert opt._plan_for(g, [ps[0]]) is first                      # a hit: moved to the recent end
        opt._plan_for(g, [ps[3]])                                      # evicts the plan of ps[1], not of ps[0]
        assert keys[0] in opt._execution_plans and keys[1] not in opt._execution_plans
        assert len(opt._execution_plans) == 3


def test_capturable_groups_hand_their_step_tensor_to_the_plan(monkeypatch):
    from apexw_b200.optim import rules
    monkeypatch.setattr(rules, "CAPTURABLE_SUPPORTED_DEVICES", tuple(rules.CAPTURABLE_SUPPORTED_DEVICES) + ("cpu",))
    opt, plan, n = _run(lr=1e-3, precision="8bit", capturable=True, steps=3)
    assert not plan.fallback and plan.dynamic
    for sp, ps in plan.classes:
        assert sp.dyn["step_dev"] is opt.state[ps[0]]["step"] and sp.dyn["lr_dev"] is None
        assert sp.dyn["lr_host"] == pytest.approx(1e-3) and sp.dyn["step_host"] == 1.0
        assert float(opt.state[ps[0]]["step"]) == 3.0
    assert n == 3 * 2 * len(plan.classes)               # scalar kernel + update, per class and step
    assert len(_Plan.made) == len(plan.classes)         # the plans of the first step serve the later ones


@pytest.mark.parametrize("kw,expected", [
    (dict(precision="compact"), True), (dict(precision="8bit"), True), (dict(precision="8bit", cautious=True), True),
    (dict(precision="compact", cautious=True), False),       # the kept fraction of a tensor would span ranks
    (dict(precision="compact", lion=True, betas=(0.9, 0.99)), False), (dict(precision="compact", amsgrad=True), False),
    (dict(precision="compact", betas=(0.9, 0.999, 0.9999)), False), (dict(precision="ultra"), False),
    (dict(precision="8bit", factored_v=True), False), (dict(precision="compact", capturable=True), False),
    (dict(precision="compact", clip_grad_norm=1.0), True), (dict(precision="compact", grad_centralization=True), False),
])
def test_which_modes_the_peer_memory_step_accepts(kw, expected):
    """``ApexWZeRO`` takes its one-kernel step only for the modes that kernel implements; everything else goes through
    collectives and the local optimizer (which still uses the single-GPU kernels)."""
    from apexw_b200.parallel.zero import ApexWZeRO
    ps = [nn.Parameter(torch.randn(s).bfloat16()) for s in SHAPES]
    opt = ApexWZeRO(ps, lr=1e-3, weight_decay=0.1, **kw)
    with mock.patch.object(torch.Tensor, "is_cuda", new_callable=mock.PropertyMock, return_value=True):
        assert opt._fused_supported_locally() is expected


def test_deterministic_mode_keeps_the_factored_layout_off_the_atomics():
    torch.use_deterministic_algorithms(True)
    try:
        _, plan, _ = _run(lr=1e-3, precision="8bit", factored_v=True, steps=1)
    finally:
        torch.use_deterministic_algorithms(False)
    assert impl._KC_FACTORED not in _classes(plan) and len(plan.fallback) >= 1     # those tensors take the torch engine
    _, plan, _ = _run(lr=1e-3, precision="8bit", factored_v=True, steps=1)
    assert impl._KC_FACTORED in _classes(plan) and not plan.fallback
