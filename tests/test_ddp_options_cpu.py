"""Options of the fused data-parallel optimizer (AdamW / SGD with momentum / Lion, weight-decay
exemptions, clipping by the global gradient norm) on the host path of the engine, against the
framework's own optimizers and ``ClipGradNorm`` applied to an fp32 copy of the same model."""
import copy

import pytest
import torch


def _models():
    from gonn_b200 import nn
    torch.manual_seed(0)
    net = nn.Sequential(nn.Linear(12, 16), nn.Tanh(), nn.LayerNorm(16), nn.Linear(16, 4))
    return net, copy.deepcopy(net)


def _data():
    g = torch.Generator().manual_seed(1)
    return torch.randn(32, 12, generator=g), torch.randn(32, 4, generator=g)


@pytest.mark.parametrize("kind", ["adamw", "sgd", "lion"])
@pytest.mark.parametrize("clip", [None, 0.05])
@pytest.mark.parametrize("no_decay", [None, "1d"])
def test_fused_optimizer_options_match_reference_optimizers(kind, clip, no_decay):
    from gonn_b200 import optim
    from gonn_b200.distributed.ddp import DistributedDataParallel
    net, ref = _models()
    net = net.to(torch.bfloat16)
    # the engine keeps fp32 master weights: start the reference from the same (bf16-rounded) values
    ref.load_state_dict({k: v.float() for k, v in net.state_dict().items()})
    opt = dict(kind=kind, lr=1e-2, weight_decay=0.1, max_grad_norm=clip, no_decay=no_decay)
    if kind == "sgd":
        opt["momentum"] = 0.9
    ddp = DistributedDataParallel(net, optimizer=opt, bucket_mb=0.0005, rank=0, world=1)
    assert len(ddp.buckets) > 1
    decay = [p for p in ref.parameters() if p.dim() > 1 or no_decay is None]
    plain = [p for p in ref.parameters() if not (p.dim() > 1 or no_decay is None)]
    groups = [dict(params=decay, weight_decay=0.1)] + ([dict(params=plain, weight_decay=0.0)] if plain else [])
    if kind == "adamw":
        ropt = optim.AdamW(groups, lr=1e-2)
    elif kind == "sgd":
        ropt = optim.SGD(groups, lr=1e-2, momentum=0.9)
    else:
        ropt = optim.Lion(groups, lr=1e-2)
    x, y = _data()
    for step in range(4):
        ((net(x.to(torch.bfloat16)).float() - y) ** 2).mean().backward()
        # the reference takes the engine's (bf16) gradients, so that only the optimizer is compared
        for (n, p), q in zip(net.named_parameters(), ref.parameters()):
            q.grad = p.grad.detach().float().clone()
        ddp.step()
        if clip is not None:
            norm = optim.ClipGradNorm(list(ref.parameters()), clip)
            assert abs(float(ddp.grad_norm) - norm) < 1e-3 * (1 + norm)
        ropt.step()
        ropt.zero_grad()
    for (n, p), q in zip(net.named_parameters(), ref.parameters()):
        # the engine's parameters are the bf16 rounding of its fp32 master copy
        assert (p.detach().float() - q.detach()).abs().max().item() < 2 ** -7 * (1 + q.abs().max().item()), n
    assert ddp.state_bytes_per_rank() == (12 if kind == "adamw" else 8) * sum(b.length for b in ddp.buckets)
