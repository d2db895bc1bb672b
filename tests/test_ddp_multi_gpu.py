"""Two real GPUs, one process each: the fused reduce-scatter + AdamW + all-gather step must
leave bit-identical parameters on both ranks and follow a single-process run on the combined
batch (pattern: distributed_test.go:205-277 of the reference).  Skipped with fewer than two
GPUs.  NVLS is off and a rank leaves only between steps."""
import os
import subprocess
import sys

import pytest
import torch

pytestmark = pytest.mark.gpu

CHILD = r'''
import os, sys, torch, torch.distributed as dist
sys.path.insert(0, os.environ["GB_ROOT"])
from gonn_b200.distributed.ddp import DistributedDataParallel
from gonn_b200.models import TransformerLM
from gonn_b200 import lib
rank = int(os.environ["RANK"]); world = int(os.environ["WORLD_SIZE"])
torch.cuda.set_device(rank)
dist.init_process_group("nccl", device_id=torch.device("cuda", rank))
torch.manual_seed(0)
kw = dict(vocab=512, d_model=128, n_layers=2, n_heads=2, d_ff=256, max_seq=64, dtype=torch.bfloat16, device="cuda")
model = TransformerLM(**kw)
if rank == 1:
    with torch.no_grad():
        for p in model.parameters():
            p.add_(1.0)          # rank 1 starts different: the wrapper must broadcast rank 0's values
ddp = DistributedDataParallel(model, optimizer=dict(kind="adamw", lr=1e-2, weight_decay=0.1), bucket_mb=0.25)
init = ddp.flat_params.clone()
g = torch.Generator().manual_seed(5)
ids = torch.randint(0, 512, (8, 64), generator=g).cuda()
tgt = torch.roll(ids, -1, 1)
lo = rank * 4
losses = []
def step(x, y):
    loss = model.loss(x, y)
    loss.backward()
    ddp.step()
    return loss
for _ in range(3):
    losses.append(step(ids[lo:lo + 4], tgt[lo:lo + 4]).item())
torch.cuda.synchronize()
ddp.check()
flat = ddp.flat_params.clone()
gathered = [torch.empty_like(flat) for _ in range(world)]
dist.all_gather(gathered, flat)
same = all(torch.equal(gathered[0], t) for t in gathered)
all_losses = [torch.zeros(3, device="cuda") for _ in range(world)]
dist.all_gather(all_losses, torch.tensor(losses, device="cuda"))
# the same step replayed as a CUDA graph: two more eager steps inside GraphedStep, then three
# replays; every replay must use fresh barrier epochs and the advancing Adam bias corrections
from gonn_b200.utils.graph import GraphedStep
gs = GraphedStep(step, ddp, (ids[lo:lo + 4].clone(), tgt[lo:lo + 4].clone()), warmup=2)
glosses = [gs(ids[lo:lo + 4], tgt[lo:lo + 4]).item() for _ in range(3)]
torch.cuda.synchronize()
ddp.check()
gflat = ddp.flat_params.clone()
ggathered = [torch.empty_like(gflat) for _ in range(world)]
dist.all_gather(ggathered, gflat)
gsame = all(torch.equal(ggathered[0], t) for t in ggathered)
if rank == 0:
    torch.save({"params": flat.cpu(), "init": init.cpu(), "same": same, "losses": torch.stack(all_losses).cpu(),
                "graph_same": gsame, "graph_params": gflat.cpu(), "graph_losses": glosses, "t": ddp.t},
               os.environ["GB_OUT"])
dist.barrier()
ddp.close()
dist.destroy_process_group()
'''


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_two_rank_fused_step_matches_single_process(tmp_path):
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    script = tmp_path / "child.py"
    script.write_text(CHILD)
    out = tmp_path / "out.pt"
    env = dict(os.environ, GB_ROOT=root, GB_OUT=str(out), NCCL_NVLS_ENABLE="0", MASTER_ADDR="127.0.0.1")
    r = subprocess.run([sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", "2",
                        "--master-addr", "127.0.0.1", "--master-port", "29533", str(script)],
                       env=env, capture_output=True, text=True, timeout=600)
    assert r.returncode == 0, r.stdout[-2000:] + r.stderr[-2000:]
    res = torch.load(out)
    assert res["same"], "ranks ended with different parameters"
    assert res["graph_same"], "ranks ended with different parameters after the graph replays"
    assert res["t"] == 8

    # single process, combined batch of 8 = mean of the two shard means
    from gonn_b200.distributed.ddp import DistributedDataParallel
    from gonn_b200.models import TransformerLM
    torch.manual_seed(0)
    kw = dict(vocab=512, d_model=128, n_layers=2, n_heads=2, d_ff=256, max_seq=64, dtype=torch.bfloat16,
              device="cuda")
    model = TransformerLM(**kw)
    ddp = DistributedDataParallel(model, optimizer=dict(kind="adamw", lr=1e-2, weight_decay=0.1),
                                  bucket_mb=0.25, world=1, rank=0)
    g = torch.Generator().manual_seed(5)
    ids = torch.randint(0, 512, (8, 64), generator=g).cuda()
    tgt = torch.roll(ids, -1, 1)
    start_values = {id(p): p.detach().clone() for p in model.parameters()}
    single_losses = []
    for _ in range(3):
        loss = model.loss(ids, tgt)
        loss.backward()
        ddp.step()
        single_losses.append(loss.item())
    # the loss on the whole batch is the mean of the two ranks' shard losses
    two = res["losses"].mean(0)
    for a, b in zip(single_losses, two.tolist()):
        assert abs(a - b) < 2e-2 * abs(a), (single_losses, two)
    # layouts differ in padding between world sizes: compare parameter by parameter
    got = res["params"].cuda()
    first = res["init"].cuda()
    moved = agree = far = count = 0
    # rebuild the 2-rank layout's offsets
    from gonn_b200.distributed.ddp import ordered_parameters
    off = 0
    align = 2 * 8
    limit = max(int(0.25 * (1 << 20) / 2), align)
    start = 0
    for p in ordered_parameters(model):
        n = p.numel()
        # compare the UPDATES (three AdamW steps at lr 1e-2 move a weight by up to 3e-2): the
        # direction of every sizeable update must agree, and its size to bf16 resolution
        d2 = (got[off:off + n].float() - first[off:off + n].float())
        d1 = (p.detach().reshape(-1).float() - start_values[id(p)].reshape(-1).float())
        assert (first[off:off + n].float() - start_values[id(p)].reshape(-1).float()).abs().max().item() == 0
        big = d1.abs() > 1e-2
        moved += int(big.sum())
        agree += int((torch.sign(d1[big]) == torch.sign(d2[big])).sum())
        # Adam's normalised update flips with the sign of a near-zero gradient, so single elements
        # may differ by a few learning rates; they must be rare
        far += int(((d1 - d2).abs() > 1.2e-2).sum())
        count += n
        off += (n + 7) // 8 * 8
        if off - start >= limit:
            off = start + (off - start + align - 1) // align * align
            start = off
    assert moved > 1000 and agree >= 0.98 * moved, (moved, agree)
    assert far <= 0.005 * count, (far, count)


CHILD_FP32_SYNCBN = r'''
import os, sys, torch, torch.distributed as dist
sys.path.insert(0, os.environ["GB_ROOT"])
from gonn_b200.distributed.ddp import DistributedDataParallel
from gonn_b200.models.mlp import MLP
from gonn_b200.models.cnn import SmallCNN
from gonn_b200.nn.loss import MSELoss
rank = int(os.environ["RANK"]); world = int(os.environ["WORLD_SIZE"])
torch.cuda.set_device(rank)
dist.init_process_group("nccl", device_id=torch.device("cuda", rank))
out = {}
# ---- fp32 parameters: gradients are all-reduced (mean), any optimizer may follow ----
torch.manual_seed(0)
mlp = MLP([16, 32, 8], dtype=torch.float32, device="cuda")
ddp = DistributedDataParallel(mlp, optimizer=None, bucket_mb=0.001)
g = torch.Generator().manual_seed(1)
x = torch.randn(8, 16, generator=g).cuda(); y = torch.randn(8, 8, generator=g).cuda()
lo = rank * 4
MSELoss(mlp(x[lo:lo + 4]), y[lo:lo + 4]).backward()
ddp.step()
torch.cuda.synchronize(); ddp.check()
out["fp32_grads"] = ddp.flat_grads.clone().cpu()
ddp.close()
# ---- SyncBatchNorm inside the CNN: halves of a batch on two ranks == the whole batch on one ----
torch.manual_seed(0)
cnn = SmallCNN(sync_bn=True, dtype=torch.bfloat16, device="cuda")
ddp2 = DistributedDataParallel(cnn, optimizer=None)
g = torch.Generator().manual_seed(2)
img = torch.randn(16, 3, 32, 32, generator=g).to(torch.bfloat16).cuda()
lab = torch.randint(0, 10, (16,), generator=g).cuda()
lo = rank * 8
logits = cnn(img[lo:lo + 8])
torch.nn.functional.cross_entropy(logits.float(), lab[lo:lo + 8]).backward()
ddp2.step()
torch.cuda.synchronize(); ddp2.check()
gathered = [torch.empty_like(logits) for _ in range(world)]
dist.all_gather(gathered, logits.detach().contiguous())
out["logits"] = torch.cat(gathered).float().cpu()
out["running_mean"] = cnn.bn1.running_mean.float().cpu()
out["running_var"] = cnn.bn1.running_var.float().cpu()
out["conv1_grad"] = cnn.conv1.weight.grad.float().cpu()
if rank == 0:
    torch.save(out, os.environ["GB_OUT"])
dist.barrier()
ddp2.close()
dist.destroy_process_group()
'''


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_two_rank_fp32_allreduce_and_syncbn_match_single_process(tmp_path):
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    script = tmp_path / "child2.py"
    script.write_text(CHILD_FP32_SYNCBN)
    out = tmp_path / "out2.pt"
    env = dict(os.environ, GB_ROOT=root, GB_OUT=str(out), NCCL_NVLS_ENABLE="0", MASTER_ADDR="127.0.0.1")
    r = subprocess.run([sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", "2",
                        "--master-addr", "127.0.0.1", "--master-port", "29534", str(script)],
                       env=env, capture_output=True, text=True, timeout=600)
    assert r.returncode == 0, r.stdout[-2000:] + r.stderr[-2000:]
    res = torch.load(out)

    from gonn_b200.models.cnn import SmallCNN
    from gonn_b200.models.mlp import MLP
    from gonn_b200.nn.loss import MSELoss
    torch.manual_seed(0)
    mlp = MLP([16, 32, 8], dtype=torch.float32, device="cuda")
    g = torch.Generator().manual_seed(1)
    x = torch.randn(8, 16, generator=g).cuda()
    y = torch.randn(8, 8, generator=g).cuda()
    MSELoss(mlp(x), y).backward()
    want = torch.cat([p.grad.reshape(-1) for p in mlp.parameters()]).cpu()
    got = res["fp32_grads"]
    # the flat buffer pads every parameter to a multiple of 8 elements: compare parameter by parameter
    off = 0
    for p in mlp.parameters():
        n = p.numel()
        assert torch.allclose(got[off:off + n], p.grad.reshape(-1).cpu(), rtol=1e-4, atol=1e-6)
        off += (n + 7) // 8 * 8
    assert want.numel() > 0

    torch.manual_seed(0)
    cnn = SmallCNN(sync_bn=False, dtype=torch.bfloat16, device="cuda")
    g = torch.Generator().manual_seed(2)
    img = torch.randn(16, 3, 32, 32, generator=g).to(torch.bfloat16).cuda()
    lab = torch.randint(0, 10, (16,), generator=g).cuda()
    logits = cnn(img)
    torch.nn.functional.cross_entropy(logits.float(), lab).backward()
    assert torch.allclose(res["logits"], logits.float().cpu(), rtol=5e-2, atol=5e-2)
    assert torch.allclose(res["running_mean"], cnn.bn1.running_mean.float().cpu(), rtol=2e-2, atol=2e-3)
    assert torch.allclose(res["running_var"], cnn.bn1.running_var.float().cpu(), rtol=2e-2, atol=2e-3)
    ref_g = cnn.conv1.weight.grad.float().cpu()
    err = (res["conv1_grad"] - ref_g).abs().max() / ref_g.abs().max().clamp_min(1e-6)
    assert err < 0.1, err


CHILD_MULTIMEM = r'''
import os, sys, torch, torch.distributed as dist
sys.path.insert(0, os.environ["GB_ROOT"])
from gonn_b200.distributed.nvlink import SymmetricMemory
rank = int(os.environ["RANK"]); world = int(os.environ["WORLD_SIZE"])
torch.cuda.set_device(rank)
dist.init_process_group("nccl", device_id=torch.device("cuda", rank))
n = world * 8 * 4096
sm = SymmetricMemory(8 * n + 4096, rank, world, device=torch.device("cuda", rank), multicast=True)
res = {"multicast": sm.multicast, "vmm_error": getattr(sm, "_vmm_error", None)}
for dtype, off in ((torch.bfloat16, 0), (torch.float32, 4 * n)):
    g = torch.Generator(device="cuda").manual_seed(7 + rank)
    mine = torch.randn(n, device="cuda", generator=g).to(dtype)
    sm.view(off, n, dtype).copy_(mine)
    every = [torch.empty_like(mine) for _ in range(world)]
    dist.all_gather(every, mine)
    torch.cuda.synchronize(); dist.barrier()
    sm.fused_step(0, dtype, off, off, n, None, None, None, [0, 0, 0, 0, 0, 1, 1, 1.0], 16)
    torch.cuda.synchronize(); sm.check()
    want = sum(t.float() for t in every) / world
    got = sm.view(off, n, dtype).float()
    res[str(dtype)] = float((got - want).abs().max())
    allg = [torch.empty_like(got) for _ in range(world)]
    dist.all_gather(allg, got.contiguous())
    res[str(dtype) + "_same"] = all(torch.equal(allg[0], t) for t in allg)
if rank == 0:
    torch.save(res, os.environ["GB_OUT"])
dist.barrier()
sm.close()
dist.destroy_process_group()
'''


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_two_rank_multimem_allreduce(tmp_path):
    """The NVSwitch multicast path (multimem.ld_reduce / multimem.st) of the fused step on two ranks:
    the mean of the ranks' vectors on every rank, identical bytes everywhere.  Where the fabric gives
    no multicast mapping the same call takes plain peer loads and the check still holds."""
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    script = tmp_path / "child_mm.py"
    script.write_text(CHILD_MULTIMEM)
    out = tmp_path / "out_mm.pt"
    env = dict(os.environ, GB_ROOT=root, GB_OUT=str(out), MASTER_ADDR="127.0.0.1")
    r = subprocess.run([sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", "2",
                        "--master-addr", "127.0.0.1", "--master-port", "29537", str(script)],
                       env=env, capture_output=True, text=True, timeout=600)
    assert r.returncode == 0, r.stdout[-2000:] + r.stderr[-2000:]
    res = torch.load(out)
    print("multicast mapping:", res["multicast"], res["vmm_error"])
    assert res["torch.bfloat16"] < 2e-2 and res["torch.float32"] < 1e-5, res
    assert res["torch.bfloat16_same"] and res["torch.float32_same"], res
