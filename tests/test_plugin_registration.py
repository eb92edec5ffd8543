"""Registration of the plugin with jax, without a device (the reference's tests/test_plugin_registration.py:25-34 drives
`initialize()` on CPU-only CI): the entry point is declared in the `jax_plugins` group, `initialize()` hands jax the
platform name, the library path and a priority, and every way it can fail says what is missing instead of registering
a half-working backend. jax itself is not installed here, so its `xla_bridge` is a stand-in that records the call."""
import importlib
import sys
import types
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parent.parent


def _plugin():
    sys.path.insert(0, str(ROOT / "jax-mps_b200"))
    return importlib.import_module("jax_plugins.b200")


def test_entry_point_group_names_the_plugin_module():
    text = (ROOT / "jax-mps_b200" / "pyproject.toml").read_text()
    assert '[project.entry-points."jax_plugins"]' in text and 'b200 = "jax_plugins.b200"' in text
    assert hasattr(_plugin(), "initialize")


def test_initialize_registers_the_platform_with_jax(monkeypatch, tmp_path):
    calls = []
    xb = types.ModuleType("jax._src.xla_bridge")
    xb.register_plugin = lambda name, priority=0, library_path=None, options=None: calls.append((name, priority, library_path, options))
    jax = types.ModuleType("jax")
    src = types.ModuleType("jax._src")
    src.xla_bridge = xb
    jax._src = src
    monkeypatch.setitem(sys.modules, "jax", jax)
    monkeypatch.setitem(sys.modules, "jax._src", src)
    monkeypatch.setitem(sys.modules, "jax._src.xla_bridge", xb)
    lib = tmp_path / "libpjrt_plugin_b200.so"
    lib.write_bytes(b"\x7fELF")
    monkeypatch.setenv("B200_PJRT_LIBRARY_PATH", str(lib))
    _plugin().initialize()
    assert calls == [("b200", 500, str(lib), None)]


def test_initialize_says_what_is_missing(monkeypatch, tmp_path):
    plugin = _plugin()
    monkeypatch.setitem(sys.modules, "jax", None)               # importing jax fails
    with pytest.raises(plugin.B200PluginError, match="jax is not installed"):
        plugin.initialize()
    monkeypatch.setenv("B200_PJRT_LIBRARY_PATH", str(tmp_path / "nowhere.so"))
    with pytest.raises(plugin.B200PluginError, match="does not exist"):
        plugin._find_library()
    monkeypatch.delenv("B200_PJRT_LIBRARY_PATH")
    assert plugin._find_library() is None                       # the adapter library is not built on this machine
