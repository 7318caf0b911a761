from .utils import op_implementation  # noqa: F401
from . import b200_implementations  # noqa: F401
from . import indexing_implementations  # noqa: F401
