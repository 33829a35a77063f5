"""The reference ships every native op as a package whose code sits in an inner module (`ops.rotary_pos_embed.
rotary_pos_embed`, `ops.static_sparse_ops.dense_sparse_matmul`); programs import through either path. Here an op is one
module; `also_importable_as` makes the inner path resolve to it."""
import sys


def also_importable_as(module_name: str, *inner: str) -> None:
    mod = sys.modules[module_name]
    if not hasattr(mod, "__path__"):
        mod.__path__ = []  # lets the import system look for `module_name.<inner>`, which it finds in sys.modules
    for leaf in inner or (module_name.rsplit(".", 1)[1],):
        sys.modules.setdefault(f"{module_name}.{leaf}", mod)
