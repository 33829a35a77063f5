"""Run programs written against `popxl` / `popxl_addons` without editing their imports.

    import popxl_addons_b200.compat          # installs the aliases (or: compat.install())
    import popxl                             # -> popxl_addons_b200.xl
    import popxl_addons as addons            # -> popxl_addons_b200
    from popxl_addons.layers import Linear   # any submodule path of either package
    import popdist                           # -> launcher queries answered from the torchrun environment

The aliases are import-system entries only: `popxl.X` is the module `popxl_addons_b200.xl.X`, `popxl_addons.X` is
`popxl_addons_b200.X`; nothing is copied or wrapped. A real `popxl` installation, if there is one, is left alone
unless `force=True`.
"""
import importlib
import importlib.abc
import importlib.util
import pkgutil
import sys

__all__ = ["install", "ALIASES"]

ALIASES = {"popxl_addons": "popxl_addons_b200", "popxl": "popxl_addons_b200.xl"}
_SKIP = (".csrc", ".lib", ".build", ".compat", ".utils.kernel_bench")


class _AliasFinder(importlib.abc.MetaPathFinder, importlib.abc.Loader):
    """Resolves `alias.sub.module` to the already importable `real.sub.module` (same module object)."""

    def find_spec(self, name, path, target=None):
        root = name.split(".")[0]
        if root in ALIASES:
            return importlib.util.spec_from_loader(name, self)
        return None

    def create_module(self, spec):
        root, _, rest = spec.name.partition(".")
        return importlib.import_module(ALIASES[root] + ("." + rest if rest else ""))

    def exec_module(self, module):
        pass


_FINDER = None


def _popdist_module():
    """The launcher queries programs make through `popdist`, answered from the `torchrun` environment: an "instance"
    is a process, and every process hosts `devices_per_replica` = 1 device of one replica unless the program's `Ir`
    says otherwise."""
    import os
    import types

    def _env(name, default):
        return int(os.environ.get(name, default))

    m = types.ModuleType("popdist")
    m.__doc__ = _popdist_module.__doc__
    m.isPopdistEnvSet = lambda: _env("WORLD_SIZE", 1) > 1
    m.getInstanceIndex = lambda: _env("RANK", 0)
    m.getNumInstances = lambda: _env("WORLD_SIZE", 1)
    m.getNumTotalReplicas = lambda: _env("WORLD_SIZE", 1)
    m.getNumLocalReplicas = lambda: 1
    m.getReplicaIndexOffset = lambda: _env("RANK", 0)
    m.getNumIpusPerReplica = lambda: 1
    m.getDeviceId = lambda: _env("LOCAL_RANK", 0)
    return m


def install(force: bool = False) -> None:
    """Make `import popxl` and `import popxl_addons` (and their submodules) resolve to this package. Submodules that
    are already imported are registered at once, so a later `from popxl.ops.call import ...` neither re-imports them
    nor rebinds a function of the same name on the parent package."""
    global _FINDER
    for alias, real in ALIASES.items():
        if not force and alias in sys.modules and not sys.modules[alias].__name__.startswith("popxl_addons_b200"):
            continue  # a genuine installation is loaded: keep it
        pkg = importlib.import_module(real)
        sys.modules[alias] = pkg
        for info in pkgutil.walk_packages(pkg.__path__, real + "."):
            if real == "popxl_addons_b200" and info.name.startswith("popxl_addons_b200.xl"):
                continue
            if any(part in info.name for part in _SKIP):
                continue
            try:
                mod = importlib.import_module(info.name)
            except Exception:  # optional pieces (native library on a machine without it, ...): resolved lazily
                continue
            sys.modules.setdefault(alias + info.name[len(real):], mod)
    if force or "popdist" not in sys.modules:
        try:
            if force:
                raise ImportError
            importlib.import_module("popdist")  # a genuine launcher library wins
        except ImportError:
            sys.modules["popdist"] = _popdist_module()
    if _FINDER is None:
        _FINDER = _AliasFinder()
        sys.meta_path.insert(0, _FINDER)


install()
