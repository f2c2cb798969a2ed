"""Optimizer in the weight-gradient epilogue (``FusedAdam.fuse_into_backward``): host-side logic.

On CPU the fused GEMM front-end runs its PyTorch path, so this checks the plumbing: expert weights
are updated by their weight-gradient task, ``step`` skips them, ``w1`` is only queued after the last
GEMM that reads it, and two training steps end with the same parameters as the separate optimizer."""
import torch

import fluidmoe_b200 as fm
from fluidmoe_b200.ops import gemm
from fluidmoe_b200.ops.optim import FusedAdam
from fluidmoe_b200.parallel.scheduler import get_backward_scheduler


def _train(fuse: bool, calls: list):
    torch.manual_seed(0)
    model = fm.TransformerModel(2, 64, 4, 2, 128, 4, 2, None, None, activation_func="swiglu",
                                norm_type="rmsnorm", dtype=torch.bfloat16, device="cpu")
    sched = get_backward_scheduler()
    sched.enable()
    ddp = fm.FluidDDP(None, model, sched)
    opt = fm.FluidOptimizerWrapper(FusedAdam(model.parameters(), lr=1e-2, weight_decay=0.01,
                                             state_dtype=torch.bfloat16), sched)
    if fuse:
        assert opt.fuse_into_backward() == 4      # w1 and w2 of both layers
    before = [p.detach().float().clone() for p in model.parameters()]
    torch.manual_seed(1)
    for _ in range(2):
        x = torch.randn(32, 1, 64).bfloat16().requires_grad_(True)
        ddp.zero_grad_buffer()
        ddp(x).float().pow(2).mean().backward()
        ddp.finish_grad_sync()
        opt.step()
    return before, [p.detach().float().clone() for p in model.parameters()]


def test_fused_optimizer_matches_separate_step(monkeypatch):
    calls = []
    real = gemm.grouped_gemm_wgrad_adam

    def counted(*a, **k):
        calls.append(k.get("step"))
        return real(*a, **k)
    monkeypatch.setattr(gemm, "grouped_gemm_wgrad_adam", counted)
    before, separate = _train(False, calls)
    assert not calls
    _, fused = _train(True, calls)
    assert calls == [1] * 4 + [2] * 4            # four expert weights per step, bias-correction step t
    changed = 0
    for b, s, f in zip(before, separate, fused):
        upd = (s - b).norm().item()
        if upd == 0.0:
            assert torch.equal(s, f)
            continue
        changed += 1
        # the separate path rounds the stored gradient to the buffer dtype, the fused one does not
        assert (s - f).norm().item() <= 0.05 * upd, ((s - f).norm().item(), upd)
    assert changed >= 8


def test_fuse_into_backward_refuses_fp32_state():
    p = torch.nn.Parameter(torch.zeros(2, 8, 8, dtype=torch.bfloat16))
    p.allreduce = False
    assert FusedAdam([p], state_dtype=torch.float32).fuse_into_backward() == 0
    assert FusedAdam([p], state_dtype=torch.bfloat16, master_weights=True).fuse_into_backward() == 0
    assert FusedAdam([p], state_dtype=torch.bfloat16).fuse_into_backward() == 1


def test_stream_mode_is_the_plain_path_on_cpu():
    """``mode="stream"`` needs CUDA streams; on CPU the gradient is stored and ``step`` updates the
    parameter as usual, with the same result as the separate optimizer."""
    torch.manual_seed(0)
    model = fm.TransformerModel(1, 64, 4, 2, 128, 4, 2, None, None, activation_func="swiglu",
                                norm_type="rmsnorm", dtype=torch.bfloat16, device="cpu")
    sched = get_backward_scheduler()
    sched.enable()
    ddp = fm.FluidDDP(None, model, sched)
    opt = fm.FluidOptimizerWrapper(FusedAdam(model.parameters(), lr=1e-2, state_dtype=torch.bfloat16), sched)
    assert opt.fuse_into_backward(mode="stream") == 2
    before = [p.detach().float().clone() for p in model.parameters()]
    x = torch.randn(32, 1, 64).bfloat16().requires_grad_(True)
    ddp.zero_grad_buffer()
    ddp(x).float().pow(2).mean().backward()
    ddp.finish_grad_sync()
    opt.step()
    changed = sum(int(not torch.equal(b, p.detach().float())) for b, p in zip(before, model.parameters()))
    assert changed >= 4
