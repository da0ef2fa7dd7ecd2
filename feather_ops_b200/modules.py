"""Putting a kernel in front of the `forward` of modules that already exist, without replacing them.

A loaded model keeps its module objects (parameter identities, patchers and offload bookkeeping depend on
them), so the instance is given a cached subclass that lists a mixin before its current class. Names follow
the reference (`feather_ops/modules.py`).
"""

from collections.abc import Callable

from torch import nn

_RELABELLED: dict[tuple[type, type], type] = {}


def relabelled_class(cls: type, mixin: type) -> type:
    """The one subclass of `cls` with `mixin` first in its bases (created on first use, then reused, so
    `type(module)` is stable and every `isinstance` check still holds)."""
    try:
        return _RELABELLED[(cls, mixin)]
    except KeyError:
        made = type(f"Feather{cls.__name__}", (mixin, cls), {"__module__": __name__, "__qualname__": cls.__qualname__})
        _RELABELLED[(cls, mixin)] = made
        return made


def relabel_modules(root: nn.Module, mixin: type, accept: Callable[[nn.Module], bool]) -> int:
    """Relabel every module of `root` that `accept` approves and that does not carry `mixin` yet. Returns
    how many changed, so a second call returns 0."""
    changed = 0
    for module in root.modules():
        if not isinstance(module, mixin) and accept(module):
            module.__class__ = relabelled_class(type(module), mixin)
            changed += 1
    return changed
