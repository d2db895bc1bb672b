"""SyncBatchNorm over CPU ranks vs single-process BatchNorm (distributed/syncbn_test.go:109-211):
two ranks each see half of the batch; outputs, input gradients, summed parameter gradients and
running statistics must match the full-batch layer; evaluation needs no communication."""
import threading

import torch

from gonn_b200 import distributed as D
from gonn_b200.distributed.syncbn import NewSyncBatchNorm2d
from gonn_b200.nn.batchnorm import BatchNorm2d


def test_two_rank_halves_match_full_batch():
    torch.manual_seed(0)
    x = torch.randn(8, 3, 4, 5, dtype=torch.float64)
    gy = torch.randn(8, 3, 4, 5, dtype=torch.float64)
    w = torch.rand(3, dtype=torch.float64) + 0.5
    b = torch.randn(3, dtype=torch.float64)
    bn = BatchNorm2d(3, dtype=torch.float64)
    with torch.no_grad():
        bn.weight.copy_(w); bn.bias.copy_(b)
    xr = x.clone().requires_grad_(True)
    yr = bn(xr)
    yr.backward(gy)
    addr = D.free_addr()
    out = [None, None]

    def body(r):
        g = D.Init(r, 2, [addr], timeout=10)
        sb = NewSyncBatchNorm2d(g, 3, dtype=torch.float64)
        with torch.no_grad():
            sb.weight.copy_(w); sb.bias.copy_(b)
        xs = x[r * 4:(r + 1) * 4].clone().requires_grad_(True)
        y = sb(xs)
        y.backward(gy[r * 4:(r + 1) * 4])
        g.Close()
        sb.eval()
        ye = sb(xs.detach())          # evaluation after the group is closed: no collectives
        out[r] = (y.detach(), xs.grad, sb.weight.grad, sb.bias.grad, sb.running_mean.clone(),
                  sb.running_var.clone(), ye)

    ts = [threading.Thread(target=body, args=(r,)) for r in range(2)]
    [t.start() for t in ts]
    [t.join(30) for t in ts]
    assert out[0] is not None and out[1] is not None
    y = torch.cat([out[0][0], out[1][0]])
    dx = torch.cat([out[0][1], out[1][1]])
    assert (y - yr.detach()).abs().max().item() < 1e-12
    assert (dx - xr.grad).abs().max().item() < 1e-10
    assert (out[0][2] + out[1][2] - bn.weight.grad).abs().max().item() < 1e-10
    assert (out[0][3] + out[1][3] - bn.bias.grad).abs().max().item() < 1e-10
    assert torch.equal(out[0][4], out[1][4]) and torch.equal(out[0][5], out[1][5])
    assert (out[0][4] - bn.running_mean).abs().max().item() < 1e-12
    assert (out[0][5] - bn.running_var).abs().max().item() < 1e-12
    bn.eval()
    assert (torch.cat([out[0][6], out[1][6]]) - bn(x)).abs().max().item() < 1e-12


def test_state_dict_names_match_batchnorm():
    g = D.Init(0, 1, ["127.0.0.1:1"])
    sb = NewSyncBatchNorm2d(g, 4)
    assert sorted(sb.state_dict()) == sorted(BatchNorm2d(4).state_dict()) == ["bias", "running_mean", "running_var", "weight"]
