"""NVFP4 storage conventions, seeded input distributions, the blocked scale layout and
the torch reference GEMM the workloads validate against.

Conventions (those of ``harness/workloads/quantization.py:1-37`` in the reference):

* packed E2M1 is ``uint8``, two values per byte, low nibble = even K index; operands
  are ``(rows, k/2, l)`` views of contiguous ``(l, rows, k/2)`` storage;
* scales are UE4M3 (``float8_e4m3fn`` with the sign bit clear), one per 16 K elements;
  logical scales are ``(rows, k/16, l)`` views of ``(l, rows, k/16)`` storage;
* the blocked layout is contiguous ``(l, ceil(rows/128), ceil(cols/4), 32, 4, 4)``
  with logical ``(r, c)`` at ``[r // 128, c // 4, r % 32, (r // 32) % 4, c % 4]`` and
  zero padding: a 512-byte atom per 128 rows x 64 K elements, which is what one
  ``tcgen05.cp.32x128b.warpx4`` moves into tensor memory;
* D is an ``(m, n, l)`` view of contiguous ``(l, m, n)`` storage.

Input distributions are named as the reference names them: values ``full`` (every
byte) or ``restricted`` (bytes masked with 0xBB: magnitudes 0, 0.5, 1, 1.5); scales
``int0_3``, ``int1_2``, ``unit`` (U[0,1) rounded to E4M3: zeros and subnormals occur)
or ``uniform`` (U[0.125, 0.875)). Every E2M1 x UE4M3 product is exact in FP32, and
with integer scales the FP32 sums are exact in any order below 2**22, so a kernel and
``fp4_matmul`` then agree bit for bit.
"""

from __future__ import annotations

import torch

SF_VEC = 16  # K elements per scale factor
SF_ROWS = 128  # rows per scale atom
SF_COLS = 4  # scale columns per atom (64 K elements)

E2M1 = (0, 0.5, 1, 1.5, 2, 3, 4, 6, -0.0, -0.5, -1, -1.5, -2, -3, -4, -6)
VALUES = ("full", "restricted")
SCALES = ("int0_3", "int1_2", "unit", "uniform")
RESTRICTED_MASK = 0xBB

# FP32 elements a reference materializes at a time (a few hundred MiB of scratch).
CHUNK = 1 << 26


def ceil_div(a: int, b: int) -> int:
    return -(-a // b)


def make_fp4(workload, g, rows, k, batches, *, values="full", scales="uniform"):
    """Seeded packed E2M1 ``(rows, k/2, l)`` and logical UE4M3 scales
    ``(rows, k/16, l)`` on ``workload.device``, drawn with generator ``g`` in the
    order data, then scales (``quantization.py:61-84`` of the reference, so that a
    case's seed gives the same tensors as there)."""
    if values not in VALUES or scales not in SCALES:
        raise ValueError(f"unknown distribution {values!r}/{scales!r}")
    device = workload.device
    data = torch.randint(0, 256, (batches, rows, k // 2), device=device, dtype=torch.uint8,
                         generator=g)
    if values == "restricted":
        data &= RESTRICTED_MASK
    shape = (batches, rows, k // SF_VEC)
    if scales == "int0_3":
        raw = torch.randint(0, 4, shape, device=device, generator=g).float()
    elif scales == "int1_2":
        raw = torch.randint(1, 3, shape, device=device, generator=g).float()
    elif scales == "unit":
        raw = torch.rand(shape, device=device, generator=g)
    else:
        raw = torch.rand(shape, device=device, generator=g) * 0.75 + 0.125
    return data.permute(1, 2, 0), raw.to(torch.float8_e4m3fn).permute(1, 2, 0)


# -- blocked scale layout ---------------------------------------------------------------


def _blocked_offsets(rows: int, cols: int, device) -> torch.Tensor:
    """Byte offset inside one batch's blocked scales of every logical ``(r, c)``."""
    cb = ceil_div(cols, SF_COLS)
    r = torch.arange(rows, device=device)[:, None]
    c = torch.arange(cols, device=device)[None, :]
    atom = (r // SF_ROWS) * cb + c // SF_COLS
    inside = (r % 32) * 16 + ((r // 32) % 4) * 4 + c % SF_COLS
    return atom * 512 + inside


def to_blocked_scales(scales: torch.Tensor) -> torch.Tensor:
    """Logical ``(rows, cols, l)`` scales (any strides) -> a fresh contiguous
    ``(l, rb, cb, 32, 4, 4)`` tensor of the same dtype in the blocked layout, zero
    padded to whole atoms."""
    rows, cols, batches = scales.shape
    rb, cb = ceil_div(rows, SF_ROWS), ceil_div(cols, SF_COLS)
    source = scales.permute(2, 0, 1).contiguous().view(torch.uint8).reshape(batches, -1)
    flat = torch.zeros((batches, rb * cb * 512), dtype=torch.uint8, device=scales.device)
    flat[:, _blocked_offsets(rows, cols, scales.device).reshape(-1)] = source
    return flat.view(scales.dtype).view(batches, rb, cb, 32, 4, 4)


def from_blocked_scales(blocked: torch.Tensor, rows: int, cols: int) -> torch.Tensor:
    """Inverse of ``to_blocked_scales``: the logical ``(rows, cols, l)`` scales of a
    ``(l, rb, cb, 32, 4, 4)`` tensor (padding dropped)."""
    batches = blocked.shape[0]
    flat = blocked.contiguous().view(torch.uint8).reshape(batches, -1)
    picked = flat[:, _blocked_offsets(rows, cols, blocked.device).reshape(-1)]
    return picked.view(blocked.dtype).view(batches, rows, cols).permute(1, 2, 0)


# -- references -----------------------------------------------------------------------------


def dequant_fp4(packed: torch.Tensor, scales: torch.Tensor) -> torch.Tensor:
    """FP32 ``(rows, k, l)`` (a view of contiguous ``(l, rows, k)``): decoded E2M1
    times the logical scale of each 16-element block. Exact."""
    rows, half_k, batches = packed.shape
    k = 2 * half_k
    table = torch.tensor(E2M1, dtype=torch.float32, device=packed.device)
    codes = packed.permute(2, 0, 1).reshape(batches * rows, half_k)
    factors = scales.permute(2, 0, 1).reshape(batches * rows, k // SF_VEC)
    out = torch.empty((batches * rows, k), dtype=torch.float32, device=packed.device)
    step = max(1, CHUNK // max(k, 1))
    for begin in range(0, batches * rows, step):
        block = codes[begin:begin + step]
        even = table[(block & 0xF).long()]
        odd = table[(block >> 4).long()]
        values = torch.stack((even, odd), dim=-1).reshape(block.shape[0], k)
        scale = factors[begin:begin + step].float()
        out[begin:begin + step] = (
            values.view(block.shape[0], k // SF_VEC, SF_VEC) * scale[:, :, None]
        ).reshape(block.shape[0], k)
    return out.view(batches, rows, k).permute(1, 2, 0)


def fp4_matmul(a, b, sa, sb, *, alpha: float = 1.0, out_dtype: torch.dtype = torch.float32):
    """``alpha * (A * SA) @ (B * SB)^T`` per batch: FP32 accumulation, ``alpha``
    applied in FP32 when it is not 1, one rounding to ``out_dtype``; an ``(m, n, l)``
    view of contiguous ``(l, m, n)`` storage. ``a``/``b`` are packed ``(rows, k/2, l)``,
    ``sa``/``sb`` logical scales. B is decoded in row chunks; the result does not
    depend on the chunking."""
    m, half_k, batches = a.shape
    n, k = b.shape[0], 2 * half_k
    lhs = dequant_fp4(a, sa).permute(2, 0, 1)
    out = torch.empty((batches, m, n), dtype=out_dtype, device=a.device)
    step = max(1, CHUNK // max(k, m, 1))
    for begin in range(0, n, step):
        rhs = dequant_fp4(b[begin:begin + step], sb[begin:begin + step]).permute(2, 1, 0)
        product = torch.bmm(lhs, rhs)
        if alpha != 1.0:
            product *= alpha
        out[:, :, begin:begin + step] = product
    return out.permute(1, 2, 0)


def empty_fp4_output(a, b, dtype=torch.float16):
    """Uninitialized ``(m, n, l)`` output in batch-major storage."""
    batches, m, n = a.shape[2], a.shape[0], b.shape[0]
    return torch.empty((batches, m, n), dtype=dtype, device=a.device).permute(1, 2, 0)


# -- FP32 -> NVFP4 ----------------------------------------------------------------------------

# Decision thresholds between neighbouring E2M1 magnitudes (0, .5, 1, 1.5, 2, 3, 4, 6) and
# whether a value exactly on the threshold rounds up (to the code with an even mantissa).
_E2M1_THRESHOLDS = ((0.25, False), (0.75, True), (1.25, False), (1.75, True), (2.5, False),
                    (3.5, True), (5.0, False))


def quantize_nvfp4(x: torch.Tensor) -> tuple[torch.Tensor, torch.Tensor]:
    """FP32 ``(rows, k, l)`` (or ``(rows, k)``) -> packed E2M1 ``(rows, k/2[, l])`` and
    logical UE4M3 scales ``(rows, k/16[, l])``: per 16-element K block
    ``scale = e4m3(amax / 6)`` (round to nearest even, saturating at 448) and each
    element is the round-to-nearest-even E2M1 code of ``x / scale``, saturating at
    +-6; a zero scale gives zero codes. The NVFP4 convention of the reference's
    quantised-operand checks (``harness/workloads/batched_gemm/trtllm.py:530-547``,
    ``formats.py:57-82``). Used to make the benchmark's N(0,1) operands."""
    squeeze = x.dim() == 2
    if squeeze:
        x = x[..., None]
    rows, k, batches = x.shape
    if k % SF_VEC:
        raise ValueError("k must be a multiple of 16")
    blocks = x.permute(2, 0, 1).float().reshape(batches, rows, k // SF_VEC, SF_VEC)
    amax = blocks.abs().amax(dim=-1)
    scales = (amax / 6.0).clamp(max=448.0).to(torch.float8_e4m3fn)
    scale = scales.float()
    safe = torch.where(scale > 0, scale, torch.ones_like(scale))
    ratio = blocks / safe[..., None]
    magnitude = ratio.abs()
    code = torch.zeros_like(magnitude, dtype=torch.uint8)
    for threshold, ties_up in _E2M1_THRESHOLDS:
        code += (magnitude >= threshold if ties_up else magnitude > threshold).to(torch.uint8)
    code += ((ratio < 0) & (code > 0)).to(torch.uint8) * 8
    code = torch.where((scale > 0)[..., None], code, torch.zeros_like(code))
    code = code.reshape(batches, rows, k)
    packed = (code[..., 0::2] | (code[..., 1::2] << 4)).permute(1, 2, 0)
    scales = scales.permute(1, 2, 0)
    if squeeze:
        return packed[..., 0], scales[..., 0]
    return packed, scales


def shuffle_rows(rows: int, block: int) -> torch.Tensor:
    """Row order of weights prepared for FlashInfer's trtllm-gen ``mm_fp4`` kernels
    (``nvfp4_quantize(..., do_shuffle=True)``): physical row i of the packed data and of
    the logical scales holds logical row ``idx[i]``. Inside blocks of ``block`` rows (32,
    or 16 for kernels whose epilogue tile is not a multiple of 128 rows) logical row
    ``base + o`` sits at physical row ``base + (o % g) * 8 + o // g``, ``g = block / 8``
    (the reference's ``harness/workloads/batched_gemm/formats.py:143-161``)."""
    if block not in (16, 32) or rows % block:
        raise ValueError(f"rows must be a multiple of the shuffle block (16 or 32), got {rows}, {block}")
    g = block // 8
    old = torch.arange(rows)
    o = old % block
    physical = old - o + (o % g) * 8 + o // g
    idx = torch.empty(rows, dtype=torch.long)
    idx[physical] = old
    return idx


def quantize_nvfp4_native(x: torch.Tensor) -> tuple[torch.Tensor, torch.Tensor]:
    """``quantize_nvfp4`` on the GPU by the library's kernel (``nvfp4_quantize``): FP32 or
    BF16 ``(rows, k, l)`` (a view of contiguous ``(l, rows, k)``) on a CUDA device ->
    packed E2M1 ``(rows, k/2, l)`` and the scales already in the blocked layout, as a
    contiguous ``(l, rb, cb, 32, 4, 4)`` tensor. Same bytes as ``quantize_nvfp4`` followed
    by ``to_blocked_scales``, in one pass over ``x``."""
    from .. import native

    if x.dim() != 3 or not x.permute(2, 0, 1).is_contiguous() or x.device.type != "cuda":
        raise ValueError("expected a CUDA (rows, k, l) view of contiguous (l, rows, k) storage")
    if x.dtype not in (torch.float32, torch.bfloat16) or x.shape[1] % SF_VEC:
        raise ValueError("expected FP32 or BF16 with k a multiple of 16")
    rows, k, batches = x.shape
    packed = torch.empty((batches, rows, k // 2), dtype=torch.uint8, device=x.device)
    blocked = torch.empty((batches, ceil_div(rows, SF_ROWS), ceil_div(k // SF_VEC, SF_COLS), 32, 4, 4),
                          dtype=torch.float8_e4m3fn, device=x.device)
    with torch.cuda.device(x.device):
        native.quantize(x.data_ptr(), native.IN_F32 if x.dtype == torch.float32 else native.IN_BF16,
                        packed.data_ptr(), blocked.data_ptr(), rows, k, batches,
                        torch.cuda.current_stream(x.device).cuda_stream)
    return packed.permute(1, 2, 0), blocked


_FP4_OUT_PLANS: dict = {}


def fp4_matmul_quantized_native(a: torch.Tensor, b: torch.Tensor, sfa: torch.Tensor,
                                sfb: torch.Tensor, alpha: torch.Tensor
                                ) -> tuple[torch.Tensor, torch.Tensor]:
    """``alpha * A @ B^T`` quantised to NVFP4 in the GEMM's epilogue (``nvfp4_gemm_launch_fp4``):
    the same bytes as ``quantize_nvfp4_native`` applied to the FP32 product, without writing
    the product to memory. ``a`` ``(m, k/2, l)`` and ``b`` ``(n, k/2, l)`` are packed E2M1
    views of contiguous ``(l, rows, k/2)`` storage, ``sfa`` / ``sfb`` their scales in the
    blocked layout (any shape, contiguous), ``alpha`` a one-element FP32 CUDA tensor.
    Returns packed D ``(m, n/2, l)`` and D's blocked scales ``(l, ceil(m/128), n/64, 32, 4, 4)``;
    ``n`` must be a multiple of 64. Rows of the last scale atom row beyond ``m`` are zero."""
    from .. import native

    m, half_k, batches = a.shape
    n = b.shape[0]
    if a.device.type != "cuda" or n % 64 or b.shape[1] != half_k or b.shape[2] != batches:
        raise ValueError("expected CUDA operands with equal k and l, and n a multiple of 64")
    for t in (a, b):
        if t.dtype != torch.uint8 or not t.permute(2, 0, 1).is_contiguous():
            raise ValueError("expected packed uint8 (rows, k/2, l) views of (l, rows, k/2) storage")
    device = a.device
    index = device.index if device.index is not None else torch.cuda.current_device()
    key = (index, m, n, 2 * half_k, batches)
    with torch.cuda.device(device):
        stream = torch.cuda.current_stream(device).cuda_stream
        if key not in _FP4_OUT_PLANS:
            plan = native.Plan.dense(index, native.OUT_FP4, m, n, 2 * half_k, batches)
            workspace = torch.empty(max(plan.workspace_bytes(), 256), dtype=torch.uint8, device=device)
            plan.init_workspace(workspace.data_ptr(), stream)
            _FP4_OUT_PLANS[key] = (plan, workspace)
        plan, workspace = _FP4_OUT_PLANS[key]
        packed = torch.empty((batches, m, n // 2), dtype=torch.uint8, device=device)
        scales = torch.zeros((batches, ceil_div(m, SF_ROWS), n // 64, 32, 4, 4),
                             dtype=torch.uint8, device=device)
        plan.launch_dense_fp4(a.data_ptr(), b.data_ptr(), sfa.data_ptr(), sfb.data_ptr(),
                              alpha.data_ptr(), packed.data_ptr(), scales.data_ptr(),
                              workspace.data_ptr(), stream)
    return packed.permute(1, 2, 0), scales.view(torch.float8_e4m3fn)
