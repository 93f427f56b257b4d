"""GPU: the allocation-free expert FFN entry point (b200moe_expert_ffn_noalloc).

Some callers may not allocate device memory at all: the engine's pools own the GPU, or a cudaMalloc
(which synchronises the whole device) would stall the step loop.  For them the library keeps a small
fixed scratch array of its own.  This file is collected last on purpose; it must pass alone in a
fresh process and after every other test.  Output is checked against the context-based entry point
(b200moe_expert_ffn) on two calls in a row, because the second call reuses the scratch the first left,
and against the CPU oracle's FFN; the status word of the scratch must read zero after every call."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def _case(n, H, I, dtype, seed):
    g = torch.Generator().manual_seed(seed)
    x = torch.randn(n, H, generator=g).to(dtype).cuda()
    gate = (torch.randn(I, H, generator=g) * 0.02).to(dtype).cuda()
    up = (torch.randn(I, H, generator=g) * 0.02).to(dtype).cuda()
    down = (torch.randn(H, I, generator=g) * 0.02).to(dtype).cuda()
    return x, gate, up, down


def _agree(a, b, dtype):
    a, b = a.double().cpu(), b.double().cpu()
    if dtype == torch.float32:
        assert float((a - b).abs().max()) <= 1e-5
        return
    ulp = 2.0 ** -6 if dtype == torch.bfloat16 else 2.0 ** -9
    assert float(((a - b).abs() - (2e-2 + ulp * b.abs())).max()) <= 0          # max-abs 2e-2 (+ two ulps)
    assert float((a - b).abs().mean() / b.abs().mean()) <= 1e-3                # mean-rel, same bar as the other FFN tests


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32, torch.float16])
def test_noalloc_matches_context_entry_point_twice_in_a_row(dtype):
    from on_device_sd_b200 import expert_forward_with_weights
    from on_device_sd_b200.noalloc import expert_forward_noalloc, noalloc_status
    from oracle import moe_oracle as O
    # two different calls back to back: the second runs over the leftovers of the first
    for seed, (n, H, I) in enumerate([(5, 256, 384), (3, 128, 64)]):
        x, gate, up, down = _case(n, H, I, dtype, seed)
        want = expert_forward_with_weights(x, gate, up, down)          # existing entry point (b200moe_expert_ffn)
        out = torch.full_like(x, float("nan"))
        got = expert_forward_noalloc(x, gate, up, down, out)
        assert noalloc_status(x.device) == 0                              # waits for the stream; no bounded wait gave up
        assert got.data_ptr() == out.data_ptr()
        _agree(got, want, dtype)
        _agree(got, O.expert_ffn(x.cpu(), gate.cpu(), up.cpu(), down.cpu()), dtype)   # and the oracle itself
    # and the very same call twice gives the very same bits
    again = expert_forward_noalloc(x, gate, up, down, torch.empty_like(x))
    assert torch.equal(again, got)


def test_noalloc_at_the_largest_supported_shape_matches_the_oracle():
    """64 rows at a Mixtral-sized intermediate (64 x 14336 bf16 = 1.75 MiB of the 2 MiB scratch); the
    oracle's FFN runs on the same CUDA tensors (torch eager = the reference's arithmetic on this device)."""
    from on_device_sd_b200.noalloc import expert_forward_noalloc, noalloc_status
    from oracle import moe_oracle as O
    g = torch.Generator(device="cuda").manual_seed(5)
    n, H, I = 64, 1024, 14336
    x = torch.randn(n, H, device="cuda", generator=g).bfloat16()
    gate = (torch.randn(I, H, device="cuda", generator=g) * 0.02).bfloat16()
    up = (torch.randn(I, H, device="cuda", generator=g) * 0.02).bfloat16()
    down = (torch.randn(H, I, device="cuda", generator=g) * 0.02).bfloat16()
    got = expert_forward_noalloc(x, gate, up, down, torch.empty_like(x))
    assert noalloc_status(x.device) == 0
    _agree(got, O.expert_ffn(x, gate, up, down), torch.bfloat16)


def test_noalloc_allocates_nothing_and_rejects_oversize():
    from on_device_sd_b200 import B200MoEError
    from on_device_sd_b200.noalloc import expert_forward_noalloc
    x, gate, up, down = _case(64, 256, 512, torch.bfloat16, 7)
    out = torch.empty_like(x)
    expert_forward_noalloc(x, gate, up, down, out)       # first call on the device: scratch address looked up
    torch.cuda.synchronize()
    free_before, _ = torch.cuda.mem_get_info()
    for _ in range(3):
        expert_forward_noalloc(x, gate, up, down, out)
    torch.cuda.synchronize()
    free_after, _ = torch.cuda.mem_get_info()
    assert free_after == free_before                      # no cudaMalloc behind the caller's back
    # more rows than the built-in scratch serves
    x2, g2, u2, d2 = _case(65, 256, 512, torch.bfloat16, 8)
    with pytest.raises(B200MoEError, match="exceeds the built-in scratch"):
        expert_forward_noalloc(x2, g2, u2, d2, torch.empty_like(x2))
    # too large an intermediate (64 x 32768 x 2 bytes = 4 MiB)
    x3 = torch.zeros(64, 64, dtype=torch.bfloat16, device="cuda")
    g3 = torch.zeros(32768, 64, dtype=torch.bfloat16, device="cuda")
    d3 = torch.zeros(64, 32768, dtype=torch.bfloat16, device="cuda")
    with pytest.raises(B200MoEError, match="exceeds the built-in scratch"):
        expert_forward_noalloc(x3, g3, g3.clone(), d3, torch.empty_like(x3))
    # empty input is a no-op
    e = torch.zeros(0, 256, dtype=torch.bfloat16, device="cuda")
    assert expert_forward_noalloc(e, gate, up, down, torch.empty_like(e)).shape == (0, 256)
