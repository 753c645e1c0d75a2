"""Every CUDA library the package can ask for, so that all of them can be built ahead of time."""

from __future__ import annotations

from tandem_b200.kernels.build import compile_many

# (source stem, defines)
LIBRARIES = [
    ("tokenwise", ()),
    ("gemm_f32", ()),
    ("attention_simt", ()),
    ("sampling", ()),
    ("gemm_skinny", ()), ("gemm_wide", ()), ("gemm_wide_pair", ()), ("gemv_bf16", ()),
] + [(stem, (f"TB_HD={hd}",)) for hd in (16, 32, 48, 64, 128) for stem in ("attention_decode", "attention_prefill")] \
    + [("attention_prefill_tc", (f"TB_HD={hd}",)) for hd in (64, 128)]


def build_all(verbose: bool = True, prune: bool = True) -> list:
    """Build every library; with ``prune``, libraries in the build folder that none of them is
    (older versions of the sources, head sizes built on demand) are removed."""
    import glob
    import os

    from tandem_b200.kernels.build import build_dir

    paths = compile_many(LIBRARIES, verbose)
    if prune:
        for stale in set(glob.glob(os.path.join(build_dir(), "tb_*.so"))) - set(paths):
            os.remove(stale)
    return paths
