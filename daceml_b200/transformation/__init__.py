from .fusion import fuse_subgraphs  # noqa: F401
from .constant_folding import fold_constants  # noqa: F401


def parameter_to_transient(dace_module, parameter_path: str):
    """Accepted for code written against the reference (``daceml/transformation/parameter_to_transient.py:15-106``), where
    it turns a module parameter that is passed on every call into a persistently allocated device array.  Here every
    parameter is bound as a device-resident constant when the SDFG is built, so there is nothing left to convert: the
    function only checks that ``parameter_path`` names a parameter or buffer of the wrapped module."""
    import operator
    operator.attrgetter(parameter_path)(dace_module.model)
