"""Data-parallel host logic on CPU with two gloo ranks: the flat gradient bucket is summed with one all-reduce
and the update equals the single-rank update on the averaged gradient. (The kernels themselves need no
exchange: samples are independent.) A GPU test runs the quaternion ResNet-18 harness for a few steps."""
import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, out):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    from phoenix_core_b200.qresnet import reduce_and_apply
    g = torch.Generator().manual_seed(5)
    w = torch.randn(1000, generator=g)
    mom = torch.zeros(1000)
    grad = (torch.randn(1000, generator=torch.Generator().manual_seed(10 + rank)) * 64).to(torch.float16)
    reduce_and_apply(w, mom, grad, world, lr=0.1, momentum=0.9, loss_scale=64.0)
    if rank == 0:
        torch.save(w, out)
    dist.barrier()
    dist.destroy_process_group()


def _worker_split(rank, world, port, out):
    """The two-part exchange: the tail of the bucket is reduced by an asynchronous all-reduce started earlier (as the
    backward pass of the harness does), the head inside reduce_and_apply."""
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    from phoenix_core_b200.qresnet import reduce_and_apply
    w = torch.randn(1000, generator=torch.Generator().manual_seed(5))
    mom = torch.zeros(1000)
    grad = (torch.randn(1000, generator=torch.Generator().manual_seed(10 + rank)) * 64).to(torch.float16)
    split = 384
    pending = dist.all_reduce(grad[split:], async_op=True)
    reduce_and_apply(w, mom, grad, world, lr=0.1, momentum=0.9, loss_scale=64.0, split=split, pending=pending)
    if rank == 0:
        torch.save(w, out)
    dist.barrier()
    dist.destroy_process_group()


def test_two_part_exchange_equals_one_part(tmp_path):
    a, b = str(tmp_path / "one.pt"), str(tmp_path / "two.pt")
    mp.spawn(_worker, args=(2, _free_port(), a), nprocs=2, join=True)
    mp.spawn(_worker_split, args=(2, _free_port(), b), nprocs=2, join=True)
    assert torch.equal(torch.load(a), torch.load(b))


def test_two_rank_bucket_update_equals_single_rank_on_mean_gradient(tmp_path):
    out = str(tmp_path / "w.pt")
    mp.spawn(_worker, args=(2, _free_port(), out), nprocs=2, join=True)
    got = torch.load(out)
    from phoenix_core_b200.qresnet import reduce_and_apply
    w = torch.randn(1000, generator=torch.Generator().manual_seed(5))
    mom = torch.zeros(1000)
    grads = [(torch.randn(1000, generator=torch.Generator().manual_seed(10 + r)) * 64).to(torch.float16) for r in range(2)]
    mean = ((grads[0].float() + grads[1].float()) / 2).to(torch.float16)        # what each rank would see on the whole batch
    reduce_and_apply(w, mom, mean, 1, lr=0.1, momentum=0.9, loss_scale=64.0)
    assert torch.allclose(got, w, atol=2e-3)


@pytest.mark.gpu
def test_qresnet18_harness_trains_on_a_fixed_batch():
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    from phoenix_core_b200.qresnet import QResNet18
    dev = torch.device("cuda", 0)
    model = QResNet18(dev, seed=1)
    assert model.num_parameters() == 2927784           # conv + fc weights + fc bias of the quaternion ResNet-18
    g = torch.Generator().manual_seed(3)
    images = torch.randn((8, 3, 64, 64), generator=g).to(torch.float16).to(dev)
    labels = torch.randint(0, 1000, (8,), generator=g).to(dev)
    losses = [float(model.train_step(images, labels, lr=0.01).detach()) for _ in range(12)]
    assert all(l == l for l in losses), losses          # finite
    assert losses[-1] < 1.0 < losses[0], losses         # the fixed batch is being fitted (7.97 -> ~0.02)
