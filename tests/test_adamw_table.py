"""Chunk table of the flat AdamW: built from learning-rate RATIOS, so a schedule that scales every group alike
reuses it and only refreshes the one-element base learning-rate tensor."""
import torch


def _make():
    from maester_b200.optimizers.adamw import FusedAdamW
    master = torch.zeros(3000)
    grad = torch.zeros(3000)
    a = torch.nn.Parameter(master[:2000].view(40, 50))
    b = torch.nn.Parameter(master[2000:].view(1000))
    opt = FusedAdamW([{"params": [a], "lr": 1e-3, "weight_decay": 0.1}, {"params": [b], "lr": 5e-4, "weight_decay": 0.0}])
    opt.attach_flat(master, grad, None, {a: (0, 2000), b: (2000, 1000)})
    return opt


def test_table_is_reused_when_all_groups_scale_together():
    opt = _make()
    (chunks, tensors, n), lr_t = opt._table()
    assert n == 2 and torch.allclose(tensors, torch.tensor([[1.0, 0.1], [0.5, 0.0]]))
    assert lr_t.item() == torch.tensor(1e-3).item()
    for g in opt.param_groups:  # what a scheduler does
        g["lr"] *= 0.25
    (chunks2, tensors2, n2), lr_t2 = opt._table()
    assert chunks2 is chunks and tensors2 is tensors and lr_t2 is lr_t
    assert abs(lr_t.item() - 2.5e-4) < 1e-10


def test_table_is_rebuilt_when_ratios_or_decay_change():
    opt = _make()
    (chunks, tensors, _), _ = opt._table()
    opt.param_groups[1]["lr"] *= 2.0
    (chunks2, tensors2, _), lr_t = opt._table()
    assert chunks2 is not chunks and torch.allclose(tensors2[:, 0], torch.tensor([1.0, 1.0]))
    opt.param_groups[0]["weight_decay"] = 0.0
    (_, tensors3, _), _ = opt._table()
    assert tensors3[0, 1].item() == 0.0


def test_zero_learning_rate_step_keeps_effective_rate_zero():
    opt = _make()
    for g in opt.param_groups:
        g["lr"] = 0.0
    (_, tensors, _), lr_t = opt._table()
    assert (tensors[:, 0] * lr_t).abs().max().item() == 0.0
