"""Registration of the b200 tier behind the reference's planner (no GPU): the literals, the mode table, the planner
factory and the dispatch of ``build`` on the plan's tier."""
import dataclasses

import pytest

from reference_support import require_fastmace


@pytest.fixture()
def registered():
    require_fastmace()
    from fastmace_b200 import planner_hook
    planner_class = planner_hook.register()
    yield planner_hook, planner_class
    planner_hook.unregister()


def test_literals_and_mode_table(registered):
    hook, _ = registered
    import fastmace.config as config
    import fastmace.planner.minimal as minimal
    assert "b200" in config.MODES and "b200" in minimal.MODES
    assert minimal.MODE_TIERS["b200"].code == "mode-b200"
    engine = config.EngineConfig(backend="b200", compile_mode="none", pipelined="off")      # _check_choices accepts it
    assert engine.backend == "b200"
    with pytest.raises(ValueError):
        config.EngineConfig(backend="no-such-backend")
    mode, reason = minimal.MinimalPlanner._mode("b200", None, None)
    assert mode == "b200" and reason.code == "mode-b200"


def test_default_planner_is_replaced_and_restored(registered):
    hook, planner_class = registered
    import torch
    import fastmace.planner.minimal as minimal
    assert minimal.default_planner.original is not minimal.default_planner
    planner = minimal.default_planner(object())
    if torch.cuda.is_available():
        assert isinstance(planner, planner_class)
    else:
        assert type(planner) is minimal.MinimalPlanner          # no CPU path: FastMACE's own tiers serve the CPU
    assert issubclass(planner_class, minimal.MinimalPlanner)
    hook.unregister()
    assert not hasattr(minimal.default_planner, "original")
    hook.register()


def test_build_dispatches_on_the_tier(registered, monkeypatch):
    hook, planner_class = registered
    import fastmace.config as config
    from fastmace.planner.plan import Plan
    calls = []
    monkeypatch.setattr(hook, "build_b200", lambda planner, plan, ff, atoms, temperature_K=None:
                        calls.append((plan.tier, temperature_K)) or "engine")
    planner = planner_class(engine=config.EngineConfig(device="cpu", compile_mode="none"))
    plan = Plan(tier="b200", engine=config.EngineConfig(backend="b200", device="cpu", compile_mode="none",
                                                        pipelined="off"))
    assert planner.build(plan, object(), object(), temperature_K=300.0) == "engine"
    assert calls == [("b200", 300.0)]
    with pytest.raises(ValueError):
        planner.build(dataclasses.replace(plan, tier="no-such-tier"), object(), object())


def test_model_container_is_read_and_a_foreign_module_is_refused(registered):
    hook, _ = registered
    from types import SimpleNamespace
    from fastmace_b200.model import SMALL, init_weights
    container = SimpleNamespace(spec=SMALL, weights=init_weights(SMALL, 0))
    assert hook.spec_of(container) is SMALL and hook.weights_of(container) is container.weights
    with pytest.raises(NotImplementedError):
        hook.spec_of(object())
    with pytest.raises(ValueError):
        from fastmace.planner.plan import Plan
        hook.build_b200(None, Plan(tier="graph"), container, object())
