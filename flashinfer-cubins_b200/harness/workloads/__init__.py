"""Importing this package registers the NVFP4 workloads."""

from . import nvfp4_dual_gemm, nvfp4_gemm, nvfp4_group_gemm  # noqa: F401
