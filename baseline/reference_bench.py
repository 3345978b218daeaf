"""Reference arm of bench.py: the reference's own CPU code on the same metric.

The reference is MPI C++ with no build system that pip understands and no MPI
exists on this image, so until the shim build below is in place this prints the
`unavailable` record.
"""
from __future__ import annotations


def run(args) -> dict:
    return {"impl": "reference", "unavailable": "reference is MPI C++ without a Python package; shim build not installed"}
