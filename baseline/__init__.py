"""Baselines: the unmodified reference library (built with dependency shims) and NCCL."""


def reference_source():
    """Directory of the unmodified reference sources, or None.

    ``PS_REFERENCE_SRC`` names it; without that variable the copy that ``build_ref.py`` made
    under ``baseline/_ref/ps-lite`` is used when present."""
    import os
    env = os.environ.get("PS_REFERENCE_SRC")
    if env:
        return env if os.path.isdir(env) else None
    here = os.path.join(os.path.dirname(os.path.abspath(__file__)), "_ref", "ps-lite")
    return here if os.path.isdir(here) else None
