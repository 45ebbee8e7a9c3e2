"""The QResNet-18 harness's training step replayed as a CUDA graph: the capture succeeds (every kernel of the library, its
side stream, its memsets and the framework glue are capturable) and a replayed step gives the gradients and the update of
an eager step from the same state, to within the run-to-run noise of the atomically summed batch-norm statistics."""
import pytest

pytestmark = pytest.mark.gpu


def test_graphed_training_step_matches_the_eager_step():
    import torch
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    from phoenix_core_b200 import qresnet
    torch.backends.cudnn.enabled = False
    dev = torch.device("cuda", 0)
    g = torch.Generator(device="cpu").manual_seed(5)
    images = torch.randn((8, 3, 64, 64), generator=g).to(torch.float16).to(dev)
    labels = torch.randint(0, 1000, (8,), generator=g).to(dev)
    model = qresnet.QResNet18(dev, seed=3)
    for _ in range(3):
        model.train_step(images, labels, 1, lr=0.01)
    torch.cuda.synchronize()
    assert model.capture(images, labels, lr=0.01)
    state = [t.clone() for t in (model.flat_w32, model.flat_mom, model.bn_w, model.bn_m)]

    def run(graphed):
        for t, v in zip((model.flat_w32, model.flat_mom, model.bn_w, model.bn_m), state):
            t.copy_(v)
        loss = model.step(images, labels, 1, lr=0.01) if graphed else model.train_step(images, labels, 1, lr=0.01)
        torch.cuda.synchronize()
        return float(loss.detach()), model.flat_g16.float().clone(), model.bn_g.clone(), model.flat_w32.clone()

    eager, graphed, again = run(False), run(True), run(True)

    def rel(a, b):
        return float((a - b).abs().max() / b.abs().max())

    for got in (graphed, again):
        assert abs(got[0] - eager[0]) <= 2e-2 * abs(eager[0])
        assert rel(got[1], eager[1]) <= 0.1          # filter gradients (fp16 bucket)
        assert rel(got[2], eager[2]) <= 0.1          # batch-norm parameter gradients
        assert rel(got[3], eager[3]) <= 1e-2         # updated master weights
    assert torch.isfinite(graphed[1]).all() and float(graphed[1].abs().max()) > 0
