"""LM head + cross-entropy (fused path) and the embedding on a GPU against fp32 autograd."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def test_head_loss_matches_autograd_with_ignored_labels_and_a_scaled_loss():
    from fluidmoe_b200.models.gpt import _HeadLoss
    from fluidmoe_b200.parallel.scheduler import BackwardScheduler, get_backward_scheduler
    BackwardScheduler.reset()
    get_backward_scheduler().disable()
    dev = torch.device("cuda", 0)
    torch.manual_seed(0)
    T, H, V = 384, 256, 1024
    h = (torch.randn(T, H, device=dev) * 0.5).bfloat16().requires_grad_(True)
    w = (torch.randn(V, H, device=dev) * 0.05).bfloat16().requires_grad_(True)
    labels = torch.randint(0, V, (T,), device=dev)
    labels[::7] = -1                                   # ignored positions
    loss = _HeadLoss.apply(h, w, labels)
    (loss * 0.37).backward()                           # an upstream factor (gradient accumulation)

    hf, wf = h.detach().float().requires_grad_(True), w.detach().float().requires_grad_(True)
    ref = torch.nn.functional.cross_entropy(hf @ wf.t(), labels, ignore_index=-1)
    (ref * 0.37).backward()

    def rel(a, b):
        return ((a.float() - b).norm() / (b.norm() + 1e-12)).item()
    assert abs(loss.item() - ref.item()) < 2e-2 * abs(ref.item())
    assert rel(h.grad, hf.grad) < 2e-2, rel(h.grad, hf.grad)
    gw = w.main_grad if getattr(w, "main_grad", None) is not None and w.grad is None else w.grad
    assert rel(gw, wf.grad) < 2e-2, rel(gw, wf.grad)
    BackwardScheduler.reset()


def test_embedding_backward_on_gpu_adds_rows_into_main_grad():
    from fluidmoe_b200.models.gpt import _Embedding
    dev = torch.device("cuda", 0)
    torch.manual_seed(1)
    V, H = 1000, 128
    ids = torch.randint(0, V, (256, 2), device=dev)
    ids[:8] = 3                                        # many repeats of one row
    gy = torch.randn(256, 2, H, device=dev).bfloat16()
    w = torch.randn(V, H, device=dev).bfloat16().requires_grad_(True)
    w.main_grad = torch.zeros(V, H, device=dev)
    _Embedding.apply(ids, w).backward(gy)
    ref = torch.zeros(V, H, device=dev).index_add_(0, ids.reshape(-1), gy.reshape(-1, H).float())
    assert w.grad is None
    assert (w.main_grad - ref).abs().max().item() < 1e-3 * (ref.abs().max().item() + 1)
