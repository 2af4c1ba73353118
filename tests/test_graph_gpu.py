"""The whole inference forward recorded as one CUDA graph gives the bits of the eager forward, for the recorded batch
and for further batches of the same signature, and the library refuses to allocate scratch during a capture."""
import numpy as np
import pytest
import torch

from flash3dtransformer_b200 import synthetic

pytestmark = pytest.mark.gpu


def _batch(dev, sizes, seed):
    from flash3dtransformer_b200.psh import batching
    c32, seps = synthetic.batch(synthetic.lidar_scan, sizes, seed=seed)
    host = torch.from_numpy(seps.astype(np.uint32))
    return torch.from_numpy(c32.astype(np.float16)).to(dev), batching.attach_host_seps(host.to(dev), host)


def test_graphed_forward_equals_eager_forward(cuda_device):
    from flash3dtransformer_b200 import configs, graph
    from flash3dtransformer_b200.lib import pshattn
    torch.manual_seed(0)
    model = configs.flash3d_backbone(channels=(32, 64, 128, 256), depths=(1, 1, 2, 1)).to(cuda_device).eval()
    sizes = [21000, 17000, 30000]
    coords, seps = _batch(cuda_device, sizes, seed=3)
    with torch.no_grad():
        eager = model(coords, None, seps).clone()
    gf = graph.GraphedForward(model, coords, seps)
    launches = pshattn.launch_count()
    out = gf(coords)
    torch.cuda.synchronize()
    assert pshattn.launch_count() == launches          # a replay issues no launch through the library's entry points
    assert torch.equal(out, eager)
    for seed in (4, 5):                                # further batches of the same signature through the same graph
        c2, s2 = _batch(cuda_device, sizes, seed=seed)
        assert gf.matches(s2)
        with torch.no_grad():
            want = model(c2, None, s2).clone()
        got = gf(c2)
        torch.cuda.synchronize()
        assert torch.equal(got, want)
    _, other = _batch(cuda_device, [21000, 17001, 29999], seed=3)
    assert not gf.matches(other)
    with pytest.raises(RuntimeError, match="recorded for"):
        gf(coords[:-1])
    pshattn.device_status()


def test_scratch_is_not_allocated_during_capture(cuda_device):
    """A call whose scratch block does not exist yet on the capturing stream is refused with a message instead of
    allocating (which would break the capture); after one run on that stream the same capture works."""
    from flash3dtransformer_b200.psh import psh_main
    coords, seps = _batch(cuda_device, [9000, 7000], seed=9)
    stream = torch.cuda.Stream(cuda_device)
    g = torch.cuda.CUDAGraph()
    stream.wait_stream(torch.cuda.current_stream(cuda_device))
    with pytest.raises(RuntimeError, match="capturing"):
        with torch.cuda.graph(g, stream=stream):
            psh_main.batch_bucket_scatter(coords, seps, 256, coords.shape[0], 2)
    torch.cuda.synchronize()
    with torch.cuda.stream(stream):
        _, want = psh_main.batch_bucket_scatter(coords, seps, 256, coords.shape[0], 2)
    stream.synchronize()
    want_id = want.bucket_id.clone()
    g2 = torch.cuda.CUDAGraph()
    with torch.cuda.graph(g2, stream=stream):
        _, got = psh_main.batch_bucket_scatter(coords, seps, 256, coords.shape[0], 2)
    got.bucket_id.fill_(0)
    g2.replay()
    torch.cuda.synchronize()
    assert torch.equal(got.bucket_id, want_id)
