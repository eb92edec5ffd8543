"""JAX plugin registration for the B200 backend (entry point group `jax_plugins`).

Mirrors the reference's shim (src/jax_plugins/mps/__init__.py:94-163): find the
PJRT library, register it with jax under the platform name "b200". It needs two
things this build machine lacks — jax itself and the PJRT adapter library
(`libpjrt_plugin_b200.so`, compiled from the C ABI in include/b200_core.h where
xla/pjrt/c/pjrt_c_api.h is available) — and says so instead of registering a
half-working backend."""
from __future__ import annotations

import os
from pathlib import Path

_LIB_NAME = "libpjrt_plugin_b200.so"


class B200PluginError(Exception):
    """Raised when the plugin cannot be initialised."""


def _find_library() -> str | None:
    env = os.environ.get("B200_PJRT_LIBRARY_PATH")
    if env:
        if Path(env).exists():
            return env
        raise B200PluginError(f"B200_PJRT_LIBRARY_PATH is set to '{env}', but the file does not exist.")
    here = Path(__file__).resolve().parent
    for p in (here / _LIB_NAME, here / "lib" / _LIB_NAME, here.parents[1] / "b200" / _LIB_NAME):
        if p.exists():
            return str(p)
    return None


def initialize() -> None:
    """Called by jax's plugin discovery."""
    try:
        from jax._src import xla_bridge as xb
    except ImportError as e:
        raise B200PluginError("jax is not installed; use the `b200.Client` API directly") from e
    lib = _find_library()
    if lib is None:
        raise B200PluginError(f"{_LIB_NAME} not found: compile the PJRT function-table adapter (one forwarding function per "
                              "entry of include/b200_core.h, built against xla/pjrt/c/pjrt_c_api.h) and place it beside this "
                              "file, or point B200_PJRT_LIBRARY_PATH at it")
    # The plugin executes per-shard programs itself; there is no SPMD partitioner behind it.
    xb.register_plugin("b200", priority=500, library_path=lib, options=None)
