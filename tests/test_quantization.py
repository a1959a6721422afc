"""The harness's NVFP4 helpers: E2M1 decoding, input distributions, the blocked scale
layout (and each workload's view of it) and the chunked torch reference GEMM. Follows
the reference's own unit tests for this module (tests/test_quantization.py there), with
the numpy oracle and the golden fixtures as second opinions."""

from unittest import mock

import numpy as np
import pytest
import torch

from conftest import load_golden
from harness.workloads import nvfp4_dual_gemm, nvfp4_gemm, nvfp4_group_gemm
from harness.workloads import quantization as q
from oracle import nvfp4_oracle as o


class CpuDevice:
    device = torch.device("cpu")


def random_scales(rows, cols, batches, seed):
    g = torch.Generator().manual_seed(seed)
    data = torch.randint(1, 127, (batches, rows, cols), generator=g, dtype=torch.uint8)
    return data.view(torch.float8_e4m3fn).permute(1, 2, 0)


SHAPES = ((128, 8, 1), (200, 6, 2), (1, 2, 1), (260, 32, 3), (129, 16, 3))


def test_nibble_order_sign_and_scale_boundary():
    packed = torch.tensor([0x10, 0x32, 0x54, 0x76, 0x98, 0xBA, 0xDC, 0xFE] * 2,
                          dtype=torch.uint8).reshape(1, 16, 1)
    scales = torch.tensor([2.0, 0.5]).reshape(1, 2, 1)
    decoded = q.dequant_fp4(packed, scales).flatten()
    values = torch.tensor([0, 0.5, 1, 1.5, 2, 3, 4, 6, 0, -0.5, -1, -1.5, -2, -3, -4, -6])
    torch.testing.assert_close(decoded, torch.cat((2 * values, 0.5 * values)))
    golden = load_golden("dequant_known_answer.npz")
    assert np.array_equal(decoded.numpy().reshape(golden["decoded"].shape), golden["decoded"])


def test_distributions():
    g = torch.Generator().manual_seed(0)
    data, _ = q.make_fp4(CpuDevice, g, 64, 256, 2, values="restricted")
    assert sorted(torch.cat((data & 15, data >> 4)).unique().tolist()) == [0, 1, 2, 3, 8, 9, 10, 11]
    data, _ = q.make_fp4(CpuDevice, g, 64, 256, 2, values="full")
    assert torch.cat((data & 15, data >> 4)).unique().numel() == 16
    checks = {
        "int0_3": lambda s: set(s.unique().tolist()) == {0, 1, 2, 3},
        "int1_2": lambda s: set(s.unique().tolist()) == {1, 2},
        "unit": lambda s: bool((s == 0).any() and ((s > 0) & (s < 2**-6)).any() and s.max() <= 1),
        "uniform": lambda s: bool(s.min() >= 0.125 and s.max() <= 0.875),
    }
    for name, check in checks.items():
        _, s = q.make_fp4(CpuDevice, g, 512, 1024, 1, scales=name)
        assert check(s.float()), name
    with pytest.raises(ValueError):
        q.make_fp4(CpuDevice, g, 4, 32, 1, scales="normal")


def test_make_fp4_views_and_storage():
    g = torch.Generator().manual_seed(3)
    data, scales = q.make_fp4(CpuDevice, g, 40, 96, 3)
    assert tuple(data.shape) == (40, 48, 3) and data.permute(2, 0, 1).is_contiguous()
    assert tuple(scales.shape) == (40, 6, 3) and scales.permute(2, 0, 1).is_contiguous()
    assert scales.dtype == torch.float8_e4m3fn


def test_reference_is_exact_and_chunk_independent():
    g = torch.Generator().manual_seed(1)
    a, sa = q.make_fp4(CpuDevice, g, 37, 96, 2, scales="int0_3")
    b, sb = q.make_fp4(CpuDevice, g, 300, 96, 2, scales="int0_3")
    before = [t.clone() for t in (a, b, sa, sb)]
    lhs = q.dequant_fp4(a, sa).double().permute(2, 0, 1)
    rhs = q.dequant_fp4(b, sb).double().permute(2, 0, 1)
    exact = (0.375 * torch.bmm(lhs, rhs.transpose(1, 2))).permute(1, 2, 0)
    for chunk in (q.CHUNK, 1000, 1):
        with mock.patch.object(q, "CHUNK", chunk):
            out = q.fp4_matmul(a, b, sa, sb, alpha=0.375)
            half = q.fp4_matmul(a, b, sa, sb, alpha=0.375, out_dtype=torch.half)
        assert torch.equal(out.double(), exact)
        assert torch.equal(half, exact.half())
        assert out.permute(2, 0, 1).is_contiguous()
    for old, new in zip(before, (a, b, sa, sb)):
        assert torch.equal(old.view(torch.uint8), new.view(torch.uint8))
    # The numpy oracle agrees bit for bit (integer scales).
    mine = o.gemm(a.permute(2, 0, 1).numpy(), b.permute(2, 0, 1).numpy(),
                  sa.permute(2, 0, 1).contiguous().view(torch.uint8).numpy(),
                  sb.permute(2, 0, 1).contiguous().view(torch.uint8).numpy(), 0.375)
    assert np.array_equal(mine, out.permute(2, 0, 1).numpy())


@pytest.mark.parametrize("rows,cols,batches", SHAPES)
def test_blocked_layout(rows, cols, batches):
    scales = random_scales(rows, cols, batches, rows + cols)
    blocked = q.to_blocked_scales(scales)
    assert blocked.is_contiguous() and blocked.dtype == scales.dtype
    memory = blocked.view(torch.uint8).flatten()
    logical = scales.permute(2, 0, 1).contiguous().view(torch.uint8).numpy()
    assert np.array_equal(memory.numpy(), o.to_blocked(logical).reshape(-1))
    golden = load_golden("blocked_layout.npz")
    assert np.array_equal(logical, golden[f"r{rows}_c{cols}_l{batches}_logical"])
    assert np.array_equal(memory.numpy(), golden[f"r{rows}_c{cols}_l{batches}_blocked"].reshape(-1))
    kb, size = blocked.shape[2], blocked[0].numel()
    for r, c, b in ((0, 0, 0), (rows - 1, cols - 1, batches - 1)):
        offset = ((r % 32) * 16 + ((r // 32) % 4) * 4 + c % 4 + (c // 4) * 512
                  + (r // 128) * 512 * kb + b * size)
        assert memory[offset] == scales.view(torch.uint8)[r, c, b]
    back = q.from_blocked_scales(blocked, rows, cols)
    assert torch.equal(back.view(torch.uint8), scales.view(torch.uint8))


@pytest.mark.parametrize("rows,cols,batches", SHAPES)
def test_workload_views_address_the_same_bytes(rows, cols, batches):
    k = 16 * cols
    scales = random_scales(rows, cols, batches, 7 * rows)
    memory = q.to_blocked_scales(scales).view(torch.uint8).flatten()
    task = nvfp4_gemm.to_task_scales(scales)
    assert tuple(task.shape) == nvfp4_gemm.blocked_scale_shape(rows, k, batches)
    assert task.permute(*nvfp4_gemm.BLOCKED_ORDER).is_contiguous()
    ii, jj = torch.meshgrid(torch.arange(rows), torch.arange(cols), indexing="ij")
    for b in range(batches):
        # The NVIDIA task's index map into its permuted scale tensor.
        picked = task[ii % 32, (ii % 128) // 32, ii // 128, jj % 4, jj // 4, b]
        assert torch.equal(picked.view(torch.uint8), scales[:, :, b].view(torch.uint8))
    back = nvfp4_gemm.from_task_scales(task, rows, cols)
    assert torch.equal(back.view(torch.uint8), scales.view(torch.uint8))

    packed = nvfp4_dual_gemm.pack_scales_reference(scales)
    assert packed.shape[0] == batches
    assert torch.equal(packed.view(torch.uint8).flatten(), memory)
    back = nvfp4_dual_gemm.unpack_scales_reference(packed, rows, cols)
    assert torch.equal(back.view(torch.uint8), scales.view(torch.uint8))

    if batches == 1:
        group = nvfp4_group_gemm.to_blocked(scales[:, :, 0])
        assert tuple(group.shape) == nvfp4_group_gemm.blocked_shape(rows, k)
        assert torch.equal(group.view(torch.uint8).flatten(), memory)
        back = nvfp4_group_gemm.from_blocked(group, rows, cols)
        assert torch.equal(back.view(torch.uint8), scales[:, :, 0].view(torch.uint8))


def test_quantiser_matches_reference_convention():
    data = load_golden("quantiser.npz")
    packed, scales = q.quantize_nvfp4(torch.from_numpy(data["x"]))
    assert np.array_equal(scales.view(torch.uint8).numpy(), data["scale_bits"])
    assert np.array_equal(packed.numpy(), data["packed"])
    # Blocks whose largest magnitude is exactly 6 have scale 1, so their other elements
    # show the bare E2M1 rounding, ties included (the grid has every multiple of 1/256).
    grid = torch.from_numpy(data["grid"]).clamp(-6, 6)[:4096].reshape(-1, 16).clone()
    grid[:, 0] = 6.0
    p, s = q.quantize_nvfp4(grid.reshape(1, -1))
    assert (s.float() == 1.0).all()
    assert np.array_equal(o.unpack_nibbles(p.numpy()), o.encode_e2m1(grid.reshape(1, -1).numpy()))
    batched, batched_scales = q.quantize_nvfp4(torch.from_numpy(data["x"]).reshape(48, 256, 1))
    assert tuple(batched.shape) == (48, 128, 1) and tuple(batched_scales.shape) == (48, 16, 1)
    assert batched.permute(2, 0, 1).is_contiguous()


def test_oracle_quantised_gemm_is_the_torch_quantiser_of_the_torch_product():
    """The oracle of the GEMM with NVFP4 output composes two pinned pieces (the FP32 product
    and the quantiser); the harness's torch versions of both give the same bytes."""
    g = torch.Generator().manual_seed(5)

    class Host:
        device = torch.device("cpu")

    a, sa = q.make_fp4(Host, g, 64, 128, 2, scales="int0_3")
    b, sb = q.make_fp4(Host, g, 128, 128, 2, scales="int0_3")
    product = q.fp4_matmul(a, b, sa, sb, alpha=0.25, out_dtype=torch.float32)
    want_packed, want_scales = q.quantize_nvfp4(product)
    store = lambda t: np.ascontiguousarray(  # noqa: E731
        (t.view(torch.uint8) if t.dtype == torch.float8_e4m3fn else t).permute(2, 0, 1).numpy())
    packed, scales = o.gemm_quantized(store(a), store(b), store(sa), store(sb), alpha=0.25)
    assert np.array_equal(packed, store(want_packed))
    assert np.array_equal(scales, store(want_scales))


def test_oracle_bf16_rounding_matches_torch():
    rng = np.random.default_rng(3)
    x = (rng.standard_normal(200_000) * 10.0 ** rng.integers(-20, 20, 200_000)).astype(np.float32)
    x[:6] = [np.inf, -np.inf, 0.0, -0.0, 1.00390625, 1.01171875]  # the last two are ties
    want = torch.from_numpy(x).to(torch.bfloat16).view(torch.int16).numpy().view(np.uint16)
    assert np.array_equal(o.round_to_bf16_bits(x), want)
    assert np.array_equal(o.bf16_bits_to_float(want),
                          torch.from_numpy(x).to(torch.bfloat16).float().numpy())
