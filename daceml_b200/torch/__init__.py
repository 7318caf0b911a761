"""``from daceml_b200.torch import DaceModule, dace_module`` (``daceml/torch/__init__.py``)."""
from .module import DaceModule, dace_module  # noqa: F401
