"""Import name of the package in the folder ``vt-transformer_b200`` (a hyphen cannot be
imported): ``import vt_transformer_b200`` loads that folder as this module, and
``python -m vt_transformer_b200`` runs its command line."""
import importlib.util
import os
import sys

_dir = os.path.join(os.path.dirname(os.path.abspath(__file__)), "vt-transformer_b200")


def _load(name):
    spec = importlib.util.spec_from_file_location(name, os.path.join(_dir, "__init__.py"),
                                                  submodule_search_locations=[_dir])
    mod = importlib.util.module_from_spec(spec)
    sys.modules[name] = mod
    spec.loader.exec_module(mod)
    return mod


if __name__ == "__main__":
    _load("vt_transformer_b200")
    from vt_transformer_b200.cli import main
    sys.exit(main())
else:
    _load(__name__)
