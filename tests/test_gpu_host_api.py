"""The host-buffer entry point (pinned host tensors in, pinned host tensors out, chunked and pipelined) gives the
bits of the device-resident call, for chunkings with short end chunks, a remainder, and a single chunk."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def _inputs(B, T=16, Hk=2, Hv=4, D=128, seed=7):
    dev = torch.device("cuda", 0)
    g = torch.Generator(device=dev).manual_seed(seed)
    rn = lambda *s: torch.randn(*s, device=dev, generator=g)  # noqa: E731
    norm = torch.nn.functional.normalize
    bf = torch.bfloat16
    return dict(q=norm(rn(B, T, Hk, D), dim=-1).to(bf), k=norm(rn(B, T, Hk, D), dim=-1).to(bf), v=rn(B, T, Hv, D).to(bf),
                g=torch.exp(-torch.nn.functional.softplus(rn(B, T, Hv))).to(bf), beta=torch.sigmoid(rn(B, T, Hv)).to(bf),
                state=0.05 * rn(B, Hv, D, D), n=torch.randint(0, T + 1, (B,), device=dev, generator=g).int())


@pytest.mark.parametrize("B,chunk", [(50, 8), (37, 16), (9, 64), (64, 16)])
def test_host_buffers_match_device_call(B, chunk):
    from swiftlm_b200 import host_api, kernels
    x = _inputs(B)
    y = torch.empty_like(x["v"])
    so = torch.empty_like(x["state"])
    kernels.gated_delta_into(x["q"], x["k"], x["v"], x["g"], x["beta"], x["state"], x["n"], y, so)
    hx = host_api.pin_replay_inputs(x)
    hout = host_api.alloc_replay_outputs(hx)
    h2d, d2h = host_api.gated_delta_from_host(hx, hout, chunk=chunk)
    torch.cuda.synchronize()
    kernels.device_status()
    assert torch.equal(hout["y"], y.cpu()) and torch.equal(hout["state"], so.cpu())
    assert h2d == sum(t.numel() * t.element_size() for t in hx.values())
    assert d2h == hout["y"].numel() * hout["y"].element_size() + hout["state"].numel() * 4

