"""The mixture-of-experts layer built on the grouped GEMM and the quantiser kernel, against
the same computation done stage by stage with the harness's torch quantiser and GEMM
reference."""

import pytest
import torch

from harness import moe
from harness.workloads import quantization as q

pytestmark = pytest.mark.gpu


def quantised_weights(experts, rows, k, seed, device):
    g = torch.Generator().manual_seed(seed)
    w = torch.randn(experts, rows, k, generator=g) * 0.05
    packed, scales = q.quantize_nvfp4(w.permute(1, 2, 0))
    packed = packed.permute(2, 0, 1).contiguous().to(device)          # [E, rows, k/2]
    scales = scales.permute(2, 0, 1).contiguous().to(device)          # [E, rows, k/16] logical
    blocked = q.to_blocked_scales(scales.permute(1, 2, 0))            # [E, rb, cb, 32, 4, 4]
    return packed, scales, blocked


@pytest.mark.parametrize("tokens,hidden,inter,experts,choices", [(200, 256, 128, 6, 2), (33, 512, 256, 4, 1)])
def test_moe_layer_matches_stagewise_reference(tokens, hidden, inter, experts, choices):
    device = torch.device("cuda:0")
    g = torch.Generator().manual_seed(tokens)
    x = torch.randn(tokens, hidden, generator=g).to(device)
    scores = torch.rand(tokens, experts, generator=g)
    scores[:, experts - 1] = -1.0                      # one expert gets no token at all
    weights, ids = torch.topk(scores, choices, dim=1)
    weights = (weights / weights.sum(dim=1, keepdim=True)).to(device)
    ids = ids.to(device)
    w13, w13_logical, w13_blocked = quantised_weights(experts, 2 * inter, hidden, 1, device)
    w2, w2_logical, w2_blocked = quantised_weights(experts, hidden, inter, 2, device)

    out = moe.moe_forward(x, ids, weights, w13, w13_blocked, w2, w2_blocked)
    torch.cuda.synchronize()
    ref = moe.moe_reference(x, ids, weights, w13, w13_logical, w2, w2_logical)

    assert out.shape == ref.shape == (tokens, hidden) and torch.isfinite(out).all()
    scale = ref.abs().max().item()
    assert scale > 0
    # Each stage rounds the same FP32 values except for the summation order inside a GEMM;
    # an FP16 ulp there can move an intermediate across an E2M1 rounding boundary, which
    # changes single terms of a few outputs.
    assert (out - ref).norm().item() <= 2e-3 * ref.norm().item()
    assert (out - ref).abs().max().item() <= 2e-2 * scale


def test_route_rows_pads_every_expert_to_whole_scale_atoms():
    ids = torch.tensor([[0, 2], [2, 1], [2, 0], [0, 2]], device="cuda")
    source, counts, starts = moe.route_rows(ids, 4)
    assert counts == [3, 1, 4, 0] and starts == [0, 128, 256, 384]
    assert source.numel() == 384
    assert source[:3].tolist() == [0, 5, 6] and source[128].item() == 3
    assert source[256:260].tolist() == [1, 2, 4, 7] and (source[3:128] == -1).all()
