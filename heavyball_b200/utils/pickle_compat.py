"""Two-way checkpoint compatibility for the pickled ``precond_schedule`` entry of the optimizer
``state_dict`` (``state_dict()["heavyball"]["precond_schedule"]``).

The reference stores ``pickle.dumps(self.precond_schedule)`` (``heavyball/utils.py:1527-1549``); for
the built-in schedules that pickle names globals of the module ``heavyball.utils``.  To interoperate
without importing that package:

* :func:`dumps` emits the built-in schedule functions under the module path ``heavyball.utils``, so a
  checkpoint written here loads in the reference;
* :func:`loads` resolves ``heavyball.utils.<name>`` (and this package's own path) to the functions
  defined here and refuses every other global except ``functools.partial``, so loading a checkpoint
  cannot execute arbitrary code.
"""

from __future__ import annotations

import functools
import io
import pickle
import types

_FOREIGN_MODULE = "heavyball.utils"
_LOCAL_MODULES = ("heavyball_b200.utils", "heavyball_b200.utils.psgd", "heavyball_b200.utils.soap")


def _exported():
    from . import psgd, soap

    return {
        "_inner_precond_update_prob_schedule": psgd._inner_precond_update_prob_schedule,
        "precond_schedule": soap.precond_schedule,
    }


class _CompatPickler(pickle._Pickler):  # the pure-Python pickler allows overriding ``save_global``
    def save_global(self, obj, name=None):
        for exported_name, fn in _exported().items():
            if obj is fn:
                self.write(pickle.GLOBAL + _FOREIGN_MODULE.encode() + b"\n" + exported_name.encode() + b"\n")
                self.memoize(obj)
                return
        super().save_global(obj, name)

    dispatch = dict(pickle._Pickler.dispatch)
    dispatch[types.FunctionType] = save_global


def dumps(schedule) -> bytes:
    buf = io.BytesIO()
    try:
        _CompatPickler(buf, protocol=2).dump(schedule)
    except Exception:  # user-supplied callables: fall back to the stock pickler
        return pickle.dumps(schedule)
    return buf.getvalue()


# Extra globals a user has declared loadable: {"module.qualname": object}.  Empty by default.
allowed_globals: dict = {}


def allow_global(obj, module: str = None, name: str = None):
    """Declares a user-defined schedule function loadable from checkpoints (by its module path and name, which is
    how pickle refers to it).  Returns ``obj`` so it can be used as a decorator."""
    module = obj.__module__ if module is None else module
    name = obj.__qualname__ if name is None else name
    allowed_globals[f"{module}.{name}"] = obj
    return obj


class _RestrictedUnpickler(pickle.Unpickler):
    def find_class(self, module, name):
        if module == "functools" and name == "partial":
            return functools.partial
        if module == _FOREIGN_MODULE or module in _LOCAL_MODULES:
            table = _exported()
            if name in table:
                return table[name]
        hit = allowed_globals.get(f"{module}.{name}")
        if hit is not None:
            return hit
        raise pickle.UnpicklingError(
            f"precond_schedule refers to global {module}.{name}, which is not on the allow-list; register it with "
            "heavyball_b200.utils.pickle_compat.allow_global(fn) before loading"
        )


def loads(data: bytes):
    return _RestrictedUnpickler(io.BytesIO(data)).load()
