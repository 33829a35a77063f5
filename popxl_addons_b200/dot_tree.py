"""DotTree: an ordered tree addressed with dotted keys, the base of every named container in the package.

Parity: popxl_addons/dot_tree.py:35-281 (insert/get/update/pop/copy/filter_keys/to_dict/from_dict/pack/unpack/map/
to_mapping, numeric and negative numeric keys, identifier validation).
"""
import re
from typing import Callable, Dict, Generic, Iterable, List, Mapping, Tuple, TypeVar, Union

from .utils import OrderedDict

L = TypeVar("L")
V = TypeVar("V")

__all__ = ["DotTree", "sanitise", "to_mapping"]


def sanitise(name: str) -> str:
    """Replace every character that cannot appear in a python identifier by `_` (and guard a leading digit)."""
    return re.sub(r"\W|^(?=\d)", "_", name)


def to_mapping(key: "DotTree", value: "DotTree") -> Dict:
    """`{key_tree[k]: value_tree[k]}` over the flat keys both trees share."""
    kd, vd = key.to_dict(), value.to_dict()
    return {kd[k]: vd[k] for k in kd if k in vd}


def _is_numeric(key) -> bool:
    return isinstance(key, int) or (isinstance(key, str) and key.isnumeric())


class DotTree(Generic[L]):
    """Nested ordered container. `tree.a.b`, `tree["a.b"]`, `tree[0]` and `tree[-1]` (last numeric key) all work."""

    def __init__(self, **kwargs):
        object.__setattr__(self, "_map", OrderedDict())
        for k, v in kwargs.items():
            self.insert(k, v)

    # ---- access -----------------------------------------------------------------------------------------------
    def _available(self) -> str:
        return "    \n".join(self._map.keys())

    def _get_numeric(self, key: int):
        if key < 0:
            numeric = [int(k) for k in self._map if k.isnumeric()]
            if not numeric:
                raise KeyError(f"Negative numerical key does not exist: {key}. Available keys: {self._available()}")
            top = max(numeric)
            resolved = top + 1 + key
            if resolved < 0:
                raise KeyError(
                    f"Negative numerical key does not exist: {key}. Max numerical key: {top}. "
                    f"Available keys: {self._available()}"
                )
            if str(resolved) not in self._map:
                raise KeyError(
                    f"Negative numerical key does not exist: {key}. Equivalent positive key: {resolved}. "
                    f"Available keys: {self._available()}"
                )
            return self._map[str(resolved)]
        if str(key) not in self._map:
            raise KeyError(f"Numerical key does not exist: {key}. Available keys: {self._available()}")
        return self._map[str(key)]

    def get(self, key: Union[str, int]):
        """Look a (possibly dotted, possibly numeric) key up; KeyError names the available keys."""
        if isinstance(key, int):
            return self._get_numeric(key)
        if key.lstrip("-").isnumeric():
            return self._get_numeric(int(key))
        head, _, rest = key.partition(".")
        if head not in self._map:
            raise KeyError(f"Key does not exist: {head}. Available keys: {self._available()}")
        node = self._map[head]
        if not rest:
            return node
        if not isinstance(node, type(self)):
            raise KeyError(
                f"Key exists ({head}) but is not a sub-DotTree of type {type(self)} "
                f"and therefore you cannot access the sub-key: {rest.split('.')}."
            )
        return node.get(rest)

    __getitem__ = get

    def __getattr__(self, key: str):
        # only reached when normal attribute lookup failed
        if key == "_map" or (key.startswith("__") and key.endswith("__")):
            raise AttributeError(key)
        try:
            return self.get(key)
        except KeyError:
            raise AttributeError(f"No attribute '{key}'. Available Keys:\n{self._available()}") from None

    def __contains__(self, key) -> bool:
        try:
            self.get(key)
        except KeyError:
            return False
        return True

    # ---- mutation ---------------------------------------------------------------------------------------------
    def _validate_key(self, key: str, allow_existing: bool):
        if key in self._map and not allow_existing:
            raise ValueError(f"'{key}' already exists")
        if not (key.isnumeric() or key.isidentifier()):
            raise ValueError(f"'{key}' is not a valid python identifier")

    def insert(self, key: Union[str, int], value, overwrite: bool = False):
        """Add `value` under `key`. Dots descend/create sub-trees; duplicates raise unless `overwrite`
        (in which case sub-trees are merged and leaves replaced)."""
        if isinstance(key, int):
            if key < 0:
                raise ValueError(f"Numerical key cannot be negative: {key}")
            key = str(key)
        head, _, rest = key.partition(".")
        self._validate_key(head, overwrite)
        if not rest:
            self._map[head] = value
            return
        current = self._map.get(head)
        # work on a copy so a failing nested insert leaves this tree untouched
        child = current.copy() if isinstance(current, type(self)) else type(self)()
        child.insert(rest, value, overwrite)
        self._map[head] = child

    def update(self, values: "DotTree", overwrite: bool = False):
        for k, v in values.copy()._map.items():
            self.insert(k, v, overwrite)

    def pop(self, key: str):
        head, _, rest = str(key).partition(".")
        if rest:
            return self.get(head).pop(rest)
        return self._map.pop(head)

    def _clear(self):
        """Drop every leaf but keep the (now empty) nested trees, so references to sub-trees stay valid."""
        for k in list(self._map.keys()):
            v = self._map[k]
            if isinstance(v, DotTree):
                v._clear()
            else:
                del self._map[k]

    # ---- views / conversion -----------------------------------------------------------------------------------
    def copy(self):
        """Shallow copy: nested trees are copied, leaves are shared."""
        out = type(self)()
        for k, v in self._map.items():
            out._map[k] = v.copy() if isinstance(v, DotTree) else v
        return out

    def filter_keys(self, keys: Iterable[Union[str, int]]):
        keys = list(keys)
        if len(set(keys)) != len(keys):
            raise ValueError("`keys` cannot contain duplicate values.")
        out = type(self)()
        for k in keys:
            out.insert(k, self.get(k), overwrite=True)
        return out

    def keys(self) -> List[str]:
        return list(self._map.keys())

    def values(self) -> List:
        return list(self._map.values())

    def keys_flat(self) -> List[str]:
        return list(self.to_dict().keys())

    def values_flat(self) -> List:
        return list(self.to_dict().values())

    def len(self) -> int:
        return len(self._map)

    def len_flat(self) -> int:
        return len(self.to_dict())

    def to_mapping(self, values: "DotTree") -> Dict:
        return to_mapping(self, values)

    def to_dict(self) -> "OrderedDict":
        flat = OrderedDict()

        # depth-first, insertion order preserved
        def walk(prefix, node):
            for k, v in node._map.items():
                if isinstance(v, DotTree):
                    walk(f"{prefix}{k}.", v)
                else:
                    flat[f"{prefix}{k}"] = v

        walk("", self)
        return flat

    @classmethod
    def from_dict(cls, d: Mapping):
        tree = cls()
        for flat_key, value in d.items():
            parts = str(flat_key).split(".")
            node = tree
            for p in parts[:-1]:
                if p not in node._map:
                    node.insert(p, cls())
                node = node._map[p]
            node.insert(parts[-1], value)
        return tree

    def unpack(self) -> Tuple[List[str], List]:
        """(keys, values) of the flattened tree, sorted by key."""
        items = sorted(self.to_dict().items(), key=lambda kv: kv[0])
        if not items:
            return [], []
        ks, vs = zip(*items)
        return ks, vs

    @classmethod
    def pack(cls, keys: Iterable, values: Iterable):
        return cls.from_dict(dict(zip(keys, values)))

    def map(self, fn: Callable):
        return self.from_dict(OrderedDict((k, fn(v)) for k, v in self.to_dict().items()))

    def __repr__(self) -> str:
        try:
            return f"{type(self).__name__}({self.to_dict()})"
        except Exception:
            return object.__repr__(self)
