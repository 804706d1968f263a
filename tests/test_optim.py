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
