"""HostPipeline (pinned host tensors in, pinned host tensors out) against the direct device call."""
import pytest
import torch

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("dtype,d,chunk", [(torch.bfloat16, 64, 2), (torch.float32, 32, 1)])
def test_host_pipeline_matches_direct_call(dtype, d, chunk):
    from simplicial_attention_b200.attention import sa2_backward, sa2_forward
    from simplicial_attention_b200.host import HostPipeline

    torch.manual_seed(5)
    b, n, h, w1, w2 = 3, 300, 2, 160, 12
    host = [torch.randn(b, n, h, d).to(dtype).pin_memory() for _ in range(6)]
    outs = [torch.zeros(b, n, h, d, dtype=dtype).pin_memory() for _ in range(6)]
    pipe = HostPipeline("cuda:0", w1=w1, w2=w2, chunk=chunk)
    pipe.run(host, outs)
    pipe.run(host, outs)            # queued back to back: the second call reuses the staging slots
    pipe.synchronize()

    dev = [t.cuda() for t in host]
    out, lse = sa2_forward(*dev[:5], w1, w2)
    grads = sa2_backward(*dev[:5], out, lse, dev[5], w1, w2)
    torch.cuda.synchronize()
    for got, want in zip(outs, (out, *grads)):
        assert torch.equal(got, want.cpu())       # batch elements are independent: bitwise equal
