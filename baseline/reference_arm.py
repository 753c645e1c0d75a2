"""The reference arm of bench.py: 12vivi/tandem itself, unmodified, from ``baseline/_ref``.

``baseline/_ref`` is where ``pip install --target baseline/_ref <reference checkout>`` would put
the reference.  Its build backend (hatchling) is not in the offline wheelhouse, so the install fails
here and the arm reports itself unavailable."""

from __future__ import annotations

import os


def run_reference(args) -> dict:
    ref = os.path.join(os.path.dirname(os.path.abspath(__file__)), "_ref", "tandem")
    if not os.path.isdir(ref):
        return {"impl": "reference", "unavailable": "12vivi/tandem could not be installed offline: its build backend "
                "hatchling is not in the wheelhouse (pip install --no-index --no-build-isolation failed)"}
    return {"impl": "reference", "unavailable": "the installed reference has no random-weights mode or B200 path to time"}
