"""A training step replayed as a CUDA graph must be the same computation as the eager step:
identical parameter bytes after several steps (all kernels are deterministic), with the
optimizer scalars and the collectives' epochs advancing from replay to replay."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def _run(graph: bool, steps: int = 5):
    from gonn_b200.distributed.ddp import DistributedDataParallel
    from gonn_b200.models import TransformerLM
    from gonn_b200.utils.graph import GraphedStep
    torch.manual_seed(3)
    dev = torch.device("cuda", 0)
    model = TransformerLM(vocab=512, d_model=128, n_layers=2, n_heads=2, d_ff=256, max_seq=128,
                          dtype=torch.bfloat16, device=dev)
    ddp = DistributedDataParallel(model, optimizer=dict(kind="adamw", lr=1e-2, weight_decay=0.1), bucket_mb=0.25)
    g = torch.Generator(device="cpu").manual_seed(5)
    batches = [torch.randint(0, 512, (4, 128), generator=g).to(dev) for _ in range(steps + 3)]

    def step(x, y):
        loss = model.loss(x, y)
        loss.backward()
        ddp.step()
        return loss

    losses = []
    if graph:
        # the three warm-up runs inside GraphedStep are real steps on the first batch
        gs = GraphedStep(step, ddp, (batches[0], torch.roll(batches[0], -1, 1)), warmup=3)
        for b in batches[3:]:
            losses.append(float(gs(b, torch.roll(b, -1, 1))))
        assert gs.launches_per_step > 20
    else:
        for _ in range(3):
            step(batches[0], torch.roll(batches[0], -1, 1))
        for b in batches[3:]:
            losses.append(float(step(b, torch.roll(b, -1, 1))))
    torch.cuda.synchronize()
    return losses, ddp.flat_params.clone(), ddp.t


def test_graphed_step_equals_eager_step(status_ok):
    le, pe, te = _run(False)
    lg, pg, tg = _run(True)
    assert te == tg == 8
    assert le == lg
    assert torch.equal(pe, pg)
    assert le[-1] < le[0]


def test_graphed_step_refuses_active_dropout():
    from gonn_b200 import nn
    from gonn_b200.distributed.ddp import DistributedDataParallel
    from gonn_b200.utils.graph import GraphedStep
    dev = torch.device("cuda", 0)
    net = nn.Sequential(nn.Linear(8, 8, dtype=torch.bfloat16, device=dev), nn.Dropout(0.5))
    ddp = DistributedDataParallel(net, optimizer=dict(kind="adamw", lr=1e-3))
    with pytest.raises(ValueError):
        GraphedStep(lambda x: net(x).float().sum(), ddp, (torch.zeros(2, 8, device=dev, dtype=torch.bfloat16),))
