from .fusion import fuse_subgraphs  # noqa: F401
