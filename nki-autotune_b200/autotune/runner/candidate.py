"""Candidate descriptors: the text carried in ``KernelJob.source``.

Upstream, ``KernelJob.source`` is NKI kernel source produced by replaying schedule
transforms (``examples/tune_matmul_lhsT_rhs.py:147-186``).  Here the device code is a
fixed set of sm_100a kernels, and a candidate is a point in a flat meta-parameter grid
(tile M/N/K, pipeline depth, cluster shape, rasterisation swizzle).  The descriptor is a
small Python file of literal assignments so that the cache layout stays
``<cache>/<stem>/<stem>.py``.
"""

from __future__ import annotations

import ast
import itertools
from dataclasses import dataclass, field

from autotune.runner.types import KernelJob

FAMILIES = ("matmul_lhsT_rhs", "matmul_lhs_rhs", "rmsnorm_matmul")
CONFIG_KEYS = ("tile_m", "tile_n", "tile_k", "stages", "cluster_m", "cluster_n", "swizzle", "split_k", "norm_mode")


@dataclass(frozen=True)
class Candidate:
    """Kernel family + meta-parameters (+ scalar arguments such as ``eps``)."""

    family: str
    config: dict = field(default_factory=dict)
    scalars: dict = field(default_factory=dict)

    def to_source(self) -> str:
        cfg = {k: int(self.config.get(k, 0)) for k in CONFIG_KEYS}
        cfg["cluster_m"] = cfg["cluster_m"] or 1
        cfg["cluster_n"] = cfg["cluster_n"] or 1
        extra = {k: v for k, v in self.config.items() if k.startswith("_")}
        cfg.update(extra)
        return (
            "# b200 autotune candidate descriptor (literal assignments only)\n"
            f"FAMILY = {self.family!r}\n"
            f"CONFIG = {cfg!r}\n"
            f"SCALARS = {dict(self.scalars)!r}\n"
        )


def parse_source(source: str) -> Candidate:
    """Inverse of :meth:`Candidate.to_source`; raises ``ValueError`` on anything else."""
    try:
        tree = ast.parse(source)
    except SyntaxError as exc:
        raise ValueError(f"candidate descriptor is not valid Python: {exc}") from exc
    found: dict[str, object] = {}
    for node in tree.body:
        if isinstance(node, ast.Assign) and len(node.targets) == 1 and isinstance(node.targets[0], ast.Name):
            found[node.targets[0].id] = ast.literal_eval(node.value)
    family = found.get("FAMILY")
    if family not in FAMILIES:
        raise ValueError(f"candidate descriptor: FAMILY must be one of {FAMILIES}, got {family!r}")
    config = found.get("CONFIG", {})
    scalars = found.get("SCALARS", {})
    if not isinstance(config, dict) or not isinstance(scalars, dict):
        raise ValueError("candidate descriptor: CONFIG and SCALARS must be dict literals")
    return Candidate(family=family, config=dict(config), scalars=dict(scalars))


def make_job(
    candidate: Candidate,
    output_shape: tuple[int, ...],
    input_specs: dict[str, tuple],
) -> KernelJob:
    """Wrap a candidate as a ``KernelJob`` (cf. ``_make_job``, ``examples/tune_matmul_lhsT_rhs.py:175-186``)."""
    return KernelJob(
        source=candidate.to_source(),
        func_name=candidate.family,
        output_shape=tuple(output_shape),
        input_specs=input_specs,
    )


def enumerate_grid(
    family: str,
    tile_m=(128, 256),
    tile_n=(128, 256),
    tile_k=(64, 128),
    stages=(3, 4, 5, 6),
    cluster_m=(1, 2),
    swizzle=(0,),
    split_k=(0,),
    scalars: dict | None = None,
) -> list[Candidate]:
    """Cartesian grid of candidates in a fixed, documented order.

    The default is the 64-point sweep: tile M in {128,256} x tile N in {128,256} x tile K in
    {64,128} x stages 3..6 x cluster {1x1, 2x1}.  Nothing is filtered: points that do not fit
    shared or tensor memory are reported as failures by the validation step.  ``split_k`` adds
    the split of every tile's K range as a further dimension (plain GEMM families; worth
    sweeping when the problem has fewer tiles than SMs).
    """
    out = []
    for tm, tn, tk, st, cm, sw, sk in itertools.product(tile_m, tile_n, tile_k, stages, cluster_m, swizzle, split_k):
        cfg = {"tile_m": tm, "tile_n": tn, "tile_k": tk, "stages": st, "cluster_m": cm, "cluster_n": 1,
               "swizzle": sw, "split_k": sk}
        out.append(Candidate(family=family, config=cfg, scalars=dict(scalars or {})))
    return out


def extended_grid(family: str, scalars: dict | None = None) -> list[Candidate]:
    """The 64-point grid followed by 24 large-tile points that use all 512 tensor-memory columns
    for one accumulator: 512x256 and 512x128 (CTA pair, two UMMAs along M), 256x512 (CTA pair, two
    UMMAs along N) and 128x512 (single CTA), each with tile K in {64,128} and 2..4 stages; and by 6
    points that vary the rasterisation swizzle (1, 4, 8) on the 512x256 and 256x512 tiles."""
    out = enumerate_grid(family, scalars=scalars)
    for (tm, tn, cm), tk, st in itertools.product(
            [(512, 256, 2), (512, 128, 2), (256, 512, 2), (128, 512, 1)], (64, 128), (2, 3, 4)):
        cfg = {"tile_m": tm, "tile_n": tn, "tile_k": tk, "stages": st, "cluster_m": cm, "cluster_n": 1,
               "swizzle": 0, "split_k": 0}
        out.append(Candidate(family=family, config=cfg, scalars=dict(scalars or {})))
    # the rasterisation group width as a dimension, on the two fastest tile shapes
    for (tm, tn), sw in itertools.product([(512, 256), (256, 512)], (1, 4, 8)):
        cfg = {"tile_m": tm, "tile_n": tn, "tile_k": 64, "stages": 4, "cluster_m": 2, "cluster_n": 1,
               "swizzle": sw, "split_k": 0}
        out.append(Candidate(family=family, config=cfg, scalars=dict(scalars or {})))
    return out


def jobs_from_candidates(
    candidates: list[Candidate],
    output_shape: tuple[int, ...],
    input_specs: dict[str, tuple],
) -> dict[str, KernelJob]:
    """Name candidates ``<family>_<i>.py`` so that they sort numerically in ``results.json``."""
    return {
        f"{c.family}_{i}.py": make_job(c, output_shape, input_specs)
        for i, c in enumerate(candidates)
    }
