"""Layer 1 of a conformance suite in the reference's style: a recorded inventory of the public
surface (classes and functions defined by each module) that must keep existing.  Regenerate
``tests/conformance/surface_inventory.json`` deliberately when the surface grows; a name that
disappears fails here."""
import importlib
import inspect
import json
import os

import pytest

INV = json.load(open(os.path.join(os.path.dirname(__file__), "conformance", "surface_inventory.json")))


@pytest.mark.parametrize("module", sorted(INV))
def test_public_surface_is_stable(module):
    mod = importlib.import_module(module)
    missing = [n for n in INV[module] if not hasattr(mod, n)]
    assert not missing, "%s lost %s" % (module, missing)
    for n in INV[module]:
        o = getattr(mod, n)
        assert inspect.isclass(o) or callable(o), (module, n)


def test_inventory_covers_every_module_with_public_names():
    import pkgutil

    import ferrotorch_b200

    have = set(INV)
    for m in pkgutil.walk_packages(ferrotorch_b200.__path__, "ferrotorch_b200."):
        if m.ispkg or m.name.endswith("._native") or m.name.endswith(".reference"):
            continue
        if m.name not in have and m.name.rsplit(".", 1)[0] not in have:
            mod = importlib.import_module(m.name)
            own = [n for n, o in vars(mod).items() if not n.startswith("_") and (inspect.isclass(o) or inspect.isfunction(o))
                   and getattr(o, "__module__", "") == m.name]
            assert not own, "module %s is not in the surface inventory" % m.name
