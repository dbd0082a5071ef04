"""Ahead-of-time compiler slice for the sm_100a routed-MoE path: contracts, shape profiles,
tactic catalog, planner, static memory plan, engine-directory emitter and validator.

Mirrors the roles of the reference's ``compiler/netra_compiler`` package (``contracts.py``,
``profiles.py``, ``backends/gfx950/catalog.py``, ``planner.py``, ``memory.py``, ``engine.py``,
``validation.py``, ``cli.py``) for one target, ``sm_100a``.
"""
from .engine import compile_engine  # noqa: F401
from .validation import validate_engine_directory  # noqa: F401

__version__ = "0.1.0"
