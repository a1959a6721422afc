"""Constructors for throughput cases that record where each shape comes from
(``CaseSpec.source``), and seeded ragged lengths. Mirrors the helpers the NVFP4 case
lists use from the reference's ``harness/throughput.py`` (lines 31-44, 87-113)."""

from __future__ import annotations

import json
import random
from functools import lru_cache

from .models import MODELS
from .workload import ROOT, CaseSpec

# The reference's downloaded trace inventories (none of them belongs to an NVFP4 GEMM
# workload; they are read only where ``REFERENCE_ROOT`` names a checkout that has them).
DATA = ROOT / "resources/benchmark_workloads"


@lru_cache(None)
def inventory(name):
    """(rows, manifest entry) of trace inventory ``name`` (``harness/throughput.py:47-55``
    in the reference)."""
    rows = [json.loads(line)["workload"]
            for line in (DATA / f"{name}.jsonl").read_text().splitlines()]
    return rows, json.loads((DATA / "manifest.json").read_text())[name]


def throughput_cases(package):
    """The throughput cases the kernels of ``harness.workloads.<package>`` must serve
    together (that module's ``throughput_cases()``)."""
    from importlib import import_module

    return import_module(f"{__package__}.workloads.{package}").throughput_cases()


def skewed_lengths(total, batch, seed=0, sigma=1.0, minimum=1):
    """``batch`` seeded log-normal lengths, each at least ``minimum``, summing to
    ``total``: a few long entries among many short ones. Uses Python's ``random`` with
    the draw order weights-first so that a seed gives the same lengths everywhere."""
    if batch * minimum > total:
        raise ValueError(f"{batch} lengths of at least {minimum} exceed {total}")
    rng = random.Random(seed)
    weights = [rng.lognormvariate(0.0, sigma) for _ in range(batch)]
    free = total - batch * minimum
    unit = free / sum(weights)
    lengths = [minimum + int(weight * unit) for weight in weights]
    # Hand the rounding remainder to the heaviest entries, one each.
    order = sorted(range(batch), key=lambda index: -weights[index])
    for index in order[: total - sum(lengths)]:
        lengths[index] += 1
    return lengths


def _label(label: str, suite: str) -> str:
    return ("throughput_" if suite == "throughput" else "") + label


def model_case(label, params, model, layer=None, *, suite="throughput", seed=1111):
    """A case whose shape is ``layer`` of ``model`` (a ``harness.models`` key)."""
    source = {"kind": "model_shape", "model": model, "hf": MODELS[model].hf}
    if layer is not None:
        source["layer"] = layer
    return CaseSpec(_label(label, suite), params, seed, suite, source)


def upstream_case(label, params, test, *, suite="smoke", seed=0, revision=None):
    """A case mirroring an upstream test parametrization ``test``."""
    source = {"kind": "upstream_test", "test": test}
    if revision is not None:
        source["revision"] = revision
    return CaseSpec(_label(label, suite), params, seed, suite, source)


def gemm_case(name, shape, source):
    """A throughput case for ``shape`` = (m, n, k[, l])."""
    params = dict(zip(("m", "n", "k", "l"), shape))
    label = "_".join(f"{key}{value}" for key, value in params.items())
    return CaseSpec("throughput_" + label, params, 1111, "throughput", source)
