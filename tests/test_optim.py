"""Optimizers on CPU: loss-scaler schedule, the two fp16 optimizers against hand-computed values, Adam against
torch.optim.AdamW, learning-rate schedules, optimizer-state sharding."""
import copy
import math

import pytest
import torch

from metaseq_b200.dataclass.utils import Cfg
from metaseq_b200.optim.dynamic_loss_scaler import DynamicLossScaler
from metaseq_b200.optim.fp16_optimizer import FP16Optimizer, MemoryEfficientFP16Optimizer


def _to_cfg(d):
    return Cfg({k: _to_cfg(v) if isinstance(v, dict) else v for k, v in d.items()})


def _cfg(bf16=False):
    return _to_cfg({
        "optimization": {"lr": [0.1]},
        "optimizer": {"_name": "adam", "lr": [0.1], "adam_betas": "(0.9, 0.999)", "adam_eps": 1e-8, "weight_decay": 0.0},
        "common": {"bf16": bf16, "fp16": not bf16, "fp16_init_scale": 1, "fp16_scale_window": 1, "fp16_scale_tolerance": 1,
                   "threshold_loss_scale": 1, "min_loss_scale": 1e-4, "fp16_no_flatten_grads": False},
    })


def _problem(dtype):
    x = torch.tensor([2.0], dtype=dtype)
    model = torch.nn.Linear(1, 1)
    model.weight.data = torch.tensor([[3.0]])
    model.bias.data = torch.tensor([5.0])
    model = model.to(dtype)
    target = torch.tensor([2.0 * 3.0 + 5.0 + 1.0], dtype=dtype)
    return model, x, target


def _run_iter(model, x, target, optimizer):
    optimizer.zero_grad()
    loss = torch.nn.L1Loss()(model(x), target)
    optimizer.backward(loss)
    assert loss.item() == 1.0
    grad_norm = optimizer.clip_grad_norm(0)
    assert abs(float(grad_norm) - 2.2361) < 1e-4  # sqrt(2^2 + 1^2)
    optimizer.step()


@pytest.mark.parametrize("cls", [MemoryEfficientFP16Optimizer, FP16Optimizer])
def test_fp16_optimizer_exact_update_and_scale_growth(cls):
    model, x, target = _problem(torch.float16)
    opt = cls.build_optimizer(_cfg(), list(model.parameters()))
    _run_iter(model, x, target, opt)
    # first Adam step moves every weight by lr = 0.1; in fp16 that is 3.0996 / 5.1016
    assert model.weight.item() == pytest.approx(3.0996, abs=1e-4)
    assert model.bias.item() == pytest.approx(5.1016, abs=1e-4)
    assert opt.scaler.loss_scale == 2.0  # window of 1: the scale doubles after one clean update
    if cls is FP16Optimizer:
        flat = torch.cat([p.view(-1) for p in (opt.fp32_params.values() if isinstance(opt.fp32_params, dict) else opt.fp32_params)])
        assert torch.allclose(flat, torch.tensor([3.1, 5.1]), atol=1e-6)


@pytest.mark.parametrize("cls", [MemoryEfficientFP16Optimizer, FP16Optimizer])
def test_skip_gradient_update_on_clip_norm_rejects_the_batch(cls):
    """A norm above the threshold raises OverflowError (the trainer then skips the update); weights, moments and the
    loss scale stay as they were; a norm below the threshold goes through."""
    model, x, target = _problem(torch.float16)
    opt = cls.build_optimizer(_cfg(), list(model.parameters()))
    opt.zero_grad()
    opt.backward(torch.nn.L1Loss()(model(x), target))
    before = (model.weight.item(), model.bias.item(), opt.scaler.loss_scale)
    with pytest.raises(OverflowError, match="rejecting batch"):
        opt.clip_grad_norm(1.0, skip_gradient_update_on_clip_norm=True)  # the norm is 2.236
    assert (model.weight.item(), model.bias.item(), opt.scaler.loss_scale) == before
    opt.zero_grad()
    opt.backward(torch.nn.L1Loss()(model(x), target))
    gn = opt.clip_grad_norm(5.0, skip_gradient_update_on_clip_norm=True)
    assert abs(float(gn) - 2.2361) < 1e-4
    opt.step()
    assert model.weight.item() == pytest.approx(3.0996, abs=1e-4)


def test_bf16_has_no_loss_scaler():
    model, x, target = _problem(torch.bfloat16)
    opt = MemoryEfficientFP16Optimizer.build_optimizer(_cfg(bf16=True), list(model.parameters()))
    assert opt.scaler is None
    opt.zero_grad()
    opt.backward(torch.nn.L1Loss()(model(x), target))
    opt.clip_grad_norm(0)
    opt.step()
    assert model.weight.item() == pytest.approx(3.1, abs=2e-2)


def test_memory_efficient_state_stays_fp32_after_reload():
    model, x, target = _problem(torch.float16)
    opt = MemoryEfficientFP16Optimizer.build_optimizer(_cfg(), list(model.parameters()))
    _run_iter(model, x, target, opt)
    state = copy.deepcopy(opt.state_dict())
    model2, _, _ = _problem(torch.float16)
    opt2 = MemoryEfficientFP16Optimizer.build_optimizer(_cfg(), list(model2.parameters()))
    opt2.load_state_dict(state)
    assert opt2.scaler.loss_scale == 2.0
    for st in opt2.optimizer.state.values():
        for v in st.values():
            if torch.is_tensor(v) and v.is_floating_point():
                assert v.dtype == torch.float32


def test_memory_efficient_reload_keeps_values_that_fp16_cannot_hold():
    """The second moments of a trained model are far below the smallest fp16 number; a reload that passes them
    through the parameters' dtype turns them into zeros and the next update divides by eps alone."""
    model, x, target = _problem(torch.float16)
    opt = MemoryEfficientFP16Optimizer.build_optimizer(_cfg(), list(model.parameters()))
    _run_iter(model, x, target, opt)
    state = copy.deepcopy(opt.state_dict())
    tiny = 3.0e-10
    for st in state["state"].values():
        st["exp_avg_sq"] = torch.full_like(st["exp_avg_sq"], tiny, dtype=torch.float32)
        st["exp_avg"] = torch.full_like(st["exp_avg"], 1.2345678e-5, dtype=torch.float32)
    model2, _, _ = _problem(torch.float16)
    opt2 = MemoryEfficientFP16Optimizer.build_optimizer(_cfg(), list(model2.parameters()))
    opt2.load_state_dict(state)
    assert len(opt2.optimizer.state) == len(state["state"]) > 0
    for st in opt2.optimizer.state.values():
        assert st["exp_avg_sq"].dtype == torch.float32 and float(st["exp_avg_sq"].flatten()[0]) == pytest.approx(tiny, rel=1e-6)
        assert float(st["exp_avg"].flatten()[0]) == pytest.approx(1.2345678e-5, rel=1e-6)
        assert int(st["step"]) == 1


def test_overflow_skips_update_and_halves_scale():
    model, x, target = _problem(torch.float16)
    cfg = _cfg()
    cfg.common.fp16_init_scale = 4
    cfg.common.fp16_scale_tolerance = 0.0
    cfg.common.threshold_loss_scale = None
    opt = MemoryEfficientFP16Optimizer.build_optimizer(cfg, list(model.parameters()))
    opt.zero_grad()
    opt.backward(torch.nn.L1Loss()(model(x), target))
    model.weight.grad.fill_(float("inf"))
    w0 = model.weight.item()
    with pytest.raises(OverflowError):
        opt.clip_grad_norm(0)
    assert opt.scaler.loss_scale == 2.0 and model.weight.item() == w0


def test_dynamic_loss_scaler_window_grows_and_shrinks_with_scale():
    s = DynamicLossScaler(init_scale=4.0, scale_window=2, tolerance=0.0)
    for _ in range(2):
        s.update()
    assert s.loss_scale == 8.0 and s.scale_window == 4  # scale and window both doubled
    with pytest.raises(OverflowError):
        s.check_overflow(float("inf"))
    assert s.loss_scale == 4.0 and s.scale_window == 2
    with pytest.raises(OverflowError):
        s.check_overflow(float("nan"))
    assert s.loss_scale == 2.0 and s.scale_window == 1
    s.check_overflow(1.5)  # finite norm: nothing happens


def test_dynamic_loss_scaler_respects_floor_and_threshold():
    s = DynamicLossScaler(init_scale=2.0, scale_window=100, tolerance=0.0, threshold=1.5, min_loss_scale=1.0)
    with pytest.raises(OverflowError):
        s.check_overflow(float("inf"))
    assert s.loss_scale == 1.5  # threshold applied on the way down
    s2 = DynamicLossScaler(init_scale=1.0, scale_window=100, tolerance=0.0, min_loss_scale=1.0)
    with pytest.raises(OverflowError):
        s2.check_overflow(float("inf"))
    assert s2.loss_scale == 1.0  # never stored below the floor


def test_adam_matches_torch_adamw():
    from metaseq_b200.optim.adam import Adam

    torch.manual_seed(0)
    p_ref = torch.nn.Parameter(torch.randn(257))
    p_new = torch.nn.Parameter(p_ref.detach().clone())
    ref = torch.optim.AdamW([p_ref], lr=1e-2, betas=(0.9, 0.95), eps=1e-8, weight_decay=0.1)
    new = Adam([p_new], lr=1e-2, betas=(0.9, 0.95), eps=1e-8, weight_decay=0.1)
    for step in range(5):
        g = torch.randn(257, generator=torch.Generator().manual_seed(step))
        p_ref.grad = g.clone()
        p_new.grad = g.clone()
        ref.step()
        new.step()
    assert torch.allclose(p_ref, p_new, rtol=1e-5, atol=1e-6)


def test_adam_step_with_scale_divides_gradients():
    from metaseq_b200.optim.adam import Adam

    a = torch.nn.Parameter(torch.ones(16))
    b = torch.nn.Parameter(torch.ones(16))
    oa, ob = Adam([a], lr=0.1), Adam([b], lr=0.1)
    g = torch.linspace(-1, 1, 16)
    a.grad = g * 8.0
    b.grad = g.clone()
    oa.step(scale=8.0)
    ob.step()
    assert torch.allclose(a, b, atol=1e-6)


def test_polynomial_decay_schedule_values():
    from metaseq_b200.optim import build_optimizer
    from metaseq_b200.optim.lr_scheduler import build_lr_scheduler

    p = torch.nn.Parameter(torch.zeros(1))
    opt = build_optimizer(_to_cfg({"_name": "adam", "lr": [1.0], "adam_betas": "(0.9, 0.999)", "adam_eps": 1e-8,
                                   "weight_decay": 0.0}), [p])
    cfg = _to_cfg({"_name": "polynomial_decay", "warmup_updates": 4, "zero_lr_warmup_steps": 2, "force_anneal": None,
                   "end_learning_rate": 0.1, "power": 1.0, "total_num_update": 14, "lr": [1.0]})
    sched = build_lr_scheduler(cfg, opt)
    lrs = [sched.step_update(i) for i in range(0, 20)]
    assert lrs[0] == 0 and lrs[2] == 0  # zero-lr warm-up
    assert lrs[3] == pytest.approx(0.25) and lrs[6] == pytest.approx(1.0)  # linear warm-up over 4 updates
    assert lrs[10] == pytest.approx(1.0 - 0.9 * (10 - 6) / (14 - 6))  # linear decay to the end value
    assert lrs[14] == pytest.approx(0.1) and lrs[19] == pytest.approx(0.1)


def test_inverse_sqrt_and_cosine_schedules():
    from metaseq_b200.optim import build_optimizer
    from metaseq_b200.optim.lr_scheduler import build_lr_scheduler

    p = torch.nn.Parameter(torch.zeros(1))
    opt = build_optimizer(_to_cfg({"_name": "adam", "lr": [0.01], "adam_betas": "(0.9, 0.999)", "adam_eps": 1e-8,
                                   "weight_decay": 0.0}), [p])
    inv = build_lr_scheduler(_to_cfg({"_name": "inverse_sqrt", "warmup_updates": 100, "warmup_init_lr": 0.0, "lr": [0.01]}), opt)
    assert inv.step_update(50) == pytest.approx(0.005)
    assert inv.step_update(400) == pytest.approx(0.01 * math.sqrt(100 / 400))
    cos = build_lr_scheduler(_to_cfg({"_name": "cosine", "warmup_updates": 0, "warmup_init_lr": -1, "max_lr": 0.01,
                                      "min_lr": 0.0, "t_mult": 1.0, "lr_period_updates": 100, "lr_shrink": 1.0,
                                      "lr": [0.01], "max_update": 100}), opt)
    assert cos.step_update(50) == pytest.approx(0.005, rel=1e-3)


def test_optimizer_state_sharding_partitions_and_steps():
    from metaseq_b200.optim.shard import ShardedOptimizer, partition_parameters

    ps = [torch.nn.Parameter(torch.randn(n)) for n in (10, 3, 7, 5)]
    parts = partition_parameters([{"params": ps, "lr": 1}], 2)
    sizes = [sum(p.numel() for g in r for p in g["params"]) for r in parts]
    assert sorted(sizes) == [12, 13]
    opt = ShardedOptimizer([{"params": ps, "lr": 0.1}], torch.optim.SGD, lr=0.1)
    before = [p.detach().clone() for p in ps]
    for p in ps:
        p.grad = torch.ones_like(p)
    opt.step()
    for b, p in zip(before, ps):
        assert torch.allclose(b - 0.1, p)


def _adam_pair(fp16_stats_kw, n=513, steps=6, tiny_grads=False):
    from metaseq_b200.optim.adam import Adam

    torch.manual_seed(0)
    p_a = torch.nn.Parameter(torch.randn(n))
    p_b = torch.nn.Parameter(p_a.detach().clone())
    a = Adam([p_a], lr=1e-2, betas=(0.9, 0.95), eps=1e-8, weight_decay=0.1)
    b = Adam([p_b], lr=1e-2, betas=(0.9, 0.95), eps=1e-8, weight_decay=0.1, **fp16_stats_kw)
    for step in range(steps):
        g = torch.randn(n, generator=torch.Generator().manual_seed(step))
        if tiny_grads:
            g = g * 1e-6  # second moments near 1e-13: far below what unscaled fp16 can hold
        p_a.grad, p_b.grad = g.clone(), g.clone()
        a.step()
        b.step()
    return p_a, p_b, a, b


@pytest.mark.parametrize("tiny_grads", [False, True])
def test_fp16_adam_stats_track_the_fp32_moments(tiny_grads):
    p32, p16, _, opt = _adam_pair({"use_fp16_stats": True}, tiny_grads=tiny_grads)
    st = opt.state[p16]
    assert st["exp_avg"].dtype == torch.float16 and st["exp_avg_sq"].dtype == torch.float16
    assert float(st["exp_avg"].float().abs().max()) == pytest.approx(65504.0, rel=2e-3)  # the scale uses the full range
    # six steps of lr 1e-2: the scaled 11-bit moments move the parameters by well under a percent of a step
    assert (p32 - p16).abs().max().item() < 2e-4
    assert (p32 - p16).abs().max().item() > 0  # and they are really quantised


def test_fp16_adam_stats_flag_reaches_the_optimizer_and_survives_reload():
    cfg = _cfg()
    cfg.optimizer.fp16_adam_stats = True
    model, x, target = _problem(torch.float16)
    opt = MemoryEfficientFP16Optimizer.build_optimizer(cfg, list(model.parameters()))
    assert opt.optimizer.use_fp16_stats
    _run_iter(model, x, target, opt)
    saved = copy.deepcopy(opt.state_dict())
    for st in saved["state"].values():
        assert st["exp_avg"].dtype == torch.float16 and "exp_avg_scale" in st and "exp_avg_sq_scale" in st
    model2, _, _ = _problem(torch.float16)
    model2.load_state_dict(model.state_dict())
    opt2 = MemoryEfficientFP16Optimizer.build_optimizer(cfg, list(model2.parameters()))
    opt2.load_state_dict(saved)
    for st, st2 in zip(opt.optimizer.state.values(), opt2.optimizer.state.values()):
        assert st2["exp_avg"].dtype == torch.float16
        assert torch.equal(st["exp_avg"], st2["exp_avg"]) and torch.equal(st["exp_avg_sq"], st2["exp_avg_sq"])
        assert float(st2["exp_avg_sq_scale"]) == pytest.approx(float(st["exp_avg_sq_scale"]), rel=1e-6)
    # the next update is the same on both
    for m, o in ((model, opt), (model2, opt2)):
        o.zero_grad()
        loss = torch.nn.L1Loss()(m(x), target)
        o.backward(loss)
        o.clip_grad_norm(0)
        o.step()
    assert torch.equal(model.weight, model2.weight) and torch.equal(model.bias, model2.bias)


def test_fp16_adam_stats_survive_a_loader_that_casts_state_to_fp32():
    # torch.optim casts loaded state to the parameter's dtype: with fp32 parameters the stored fp16 values arrive as
    # fp32 and the scale still applies
    from metaseq_b200.optim.adam import Adam

    _, p16, _, opt = _adam_pair({"use_fp16_stats": True}, n=64, steps=3)
    saved = copy.deepcopy(opt.state_dict())
    q = torch.nn.Parameter(p16.detach().clone())
    opt2 = Adam([q], lr=1e-2, betas=(0.9, 0.95), eps=1e-8, weight_decay=0.1, use_fp16_stats=True)
    opt2.load_state_dict(saved)
    assert opt2.state[q]["exp_avg"].dtype == torch.float32  # torch's cast
    g = torch.randn(64, generator=torch.Generator().manual_seed(9))
    p16.grad, q.grad = g.clone(), g.clone()
    opt.step()
    opt2.step()
    assert torch.allclose(p16, q, rtol=0, atol=1e-7)
    assert opt2.state[q]["exp_avg"].dtype == torch.float16


def test_resharding_joins_scaled_fp16_moments_as_fp32():
    from metaseq_b200.checkpoint import flat_shards

    full_m = torch.linspace(-1.0, 1.0, 8)
    full_v = torch.linspace(1e-12, 3e-9, 8)

    def shard(i):
        m, v = full_m[4 * i: 4 * i + 4], full_v[4 * i: 4 * i + 4]
        ms, vs = m.abs().max() / 65504.0 + 1e-8, v.abs().max() / 65504.0 + 1e-8
        md = {"param_metadata": [{"fsdp_path": "", "params": {"flat_param_0": {
            "names": ["w"], "shapes": [[8]], "numels": [8], "padding": 0}},
            "no_broadcast_optim_state": False, "shared_param_info": []}], "buffer_names": []}
        return {"model": {"flat_param_0": torch.zeros(4)}, "shard_metadata": md,
                "last_optimizer_state": {"state": {0: {"step": 3, "exp_avg": (m / ms).half(), "exp_avg_scale": ms,
                                                       "exp_avg_sq": (v / vs).half(), "exp_avg_sq_scale": vs}},
                                         "param_groups": [{"params": [0]}]}}

    out = flat_shards.reshard_optimizer_state([shard(0), shard(1)], 0, 1)
    st = out["state"][0]
    assert "exp_avg_scale" not in st and "exp_avg_sq_scale" not in st and st["step"] == 3
    assert st["exp_avg"].dtype == torch.float32 and st["exp_avg"].numel() == 8
    assert torch.allclose(st["exp_avg"], full_m, rtol=2e-3, atol=1e-7)
    assert torch.allclose(st["exp_avg_sq"], full_v, rtol=2e-3, atol=1e-15)
