"""Cross-node fusion: rewrites sub-graphs of an exported model into the fused operators this
library has kernels for.  The analogue of the reference's ``ReplacementTransformation`` /
``HorizontalEinsumFusion`` / ``PadConvFusion`` (``daceml/transformation/replacement.py:67-181``,
``einsum_fusion.py:19-151``, ``pad_conv_fusion.py:14-97``)."""


def fuse_subgraphs(sdfg):
    """Applies every fusion pattern until none matches; returns the number of rewrites."""
    from . import patterns
    total = 0
    while True:
        n = sum(p(sdfg) for p in patterns.PATTERNS)
        if n == 0:
            return total
        total += n
